"""Packed-checkpoint save / restore / mode conversion for models that use this package's modules.

Same on-disk layout as the reference (qwen35_quant_io.py): ``model.safetensors`` holds the model's
``state_dict`` (MoE buffers ``<layer>.mlp.bit_weights.<bit>.{gate_up,down}_{indices_packed,codebook,norms}``,
packed Linear buffers ``packed_indices / norms / codebook [/ bias]``) plus one scalar int64 tensor per
rotation seed under ``qmeta/...``; ``meta.json`` holds everything that is not a tensor (shapes, seeds,
expert offsets, bit lists), keyed by the module's dotted path.  A checkpoint written by the reference
loads here unchanged and the other way round.

    collect_quant_metadata   qwen35_quant_io.py:103     save_quantized_model   :241
    restore_quant_metadata   :348                        load_quantized_state_dict :612
    convert_model_to_wxa8 / wxfp8 / wxfp4   :416 / :452 / :503

Only the parts that touch the quantized modules are here; building the skeleton model (a transformers
class on the meta device) stays with the caller.
"""
from __future__ import annotations

import json
import os
import warnings
from typing import Callable, Dict, Optional, Tuple, Union

import torch

from . import format as fmt
from .linear import WxA16Linear, WxA8Linear, WxFP8Linear
from .moe import (WxA16BitPartitionedGroupMoE, WxA8BitPartitionedGroupMoE, WxFP4BitPartitionedGroupMoE,
                  WxFP8BitPartitionedGroupMoE)

PrefixMap = Union[None, Tuple[str, str], Callable[[str], str]]
_SIDES = ("gate_up", "down")


# --------------------------------------------------------------------------- metadata (save side)

def _linear_entry(lin: WxA16Linear) -> dict:
    return {
        "type": "wxa16_linear", "in_features": lin.in_features, "out_features": lin.out_features,
        "bit_width": lin.bit_width, "group_size": lin.group_size, "seed": lin.seed, "rotation": lin.rotation,
        "orig_dtype": str(lin.orig_dtype), "has_bias": lin.bias is not None,
        "indices_packed_shape": list(lin.packed_indices.shape), "codebook_shape": list(lin.codebook.shape),
        "norms_shape": list(lin.norms.shape),
        "bias_shape": None if lin.bias is None else list(lin.bias.shape),
        "codebook_type": getattr(lin, "codebook_type", "lloydmax"),
    }


def _side_entry(packed: dict) -> dict:
    out = {k: packed.get(k) for k in ("seed", "group_size", "bit_width", "rotation", "orig_dtype")}
    out["shape"] = list(packed["shape"])
    for name in ("indices_packed", "codebook", "norms"):
        out[name + "_shape"] = list(packed[name].shape)
    return out


def _moe_entry(moe: WxA16BitPartitionedGroupMoE) -> dict:
    return {
        "type": "wxa16_moe", "num_experts": moe.num_experts, "hidden_size": moe.hidden_size,
        "intermediate_size": moe.intermediate_size, "top_k": moe.top_k, "bit_list": list(moe.bit_list),
        "inter_size_by_bit": {str(b): n for b, n in moe.inter_size_by_bit.items()},
        # the offsets are plain tensors outside the state dict: they travel as lists
        "expert_offsets": {b: (t.cpu().tolist() if torch.is_tensor(t) else list(t)) for b, t in moe.expert_offsets.items()},
        "bits": {b: {"gate_up": _side_entry(w.gate_up_packed), "down": _side_entry(w.down_packed)}
                 for b, w in moe.bit_weights.items()},
        "enable_timing": moe.enable_timing,
    }


def collect_quant_metadata(model, quant_args: Optional[dict] = None, model_id: Optional[str] = None,
                           base_model: Optional[str] = None) -> dict:
    """Everything about the quantized modules that ``state_dict`` does not carry, keyed by dotted path."""
    meta = {"base_model": base_model, "model_class": type(model).__name__, "quant_args": quant_args or {},
            "modules": {}, "layers": {}}
    if model_id:
        meta["model_id"] = model_id
    for path, mod in model.named_modules():
        if not path:
            continue
        if isinstance(mod, WxA16Linear):
            meta["modules"][path] = _linear_entry(mod)
        elif isinstance(mod, WxA16BitPartitionedGroupMoE):
            meta["layers"][path] = _moe_entry(mod)
    return meta


def _seed_items(meta: dict):
    """(qmeta key, seed) for every seed the metadata records."""
    for path, m in meta.get("modules", {}).items():
        if m.get("seed") is not None:
            yield f"qmeta/{path}/seed", int(m["seed"])
    for path, layer in meta.get("layers", {}).items():
        for bit, sides in layer["bits"].items():
            for side in _SIDES:
                if sides[side].get("seed") is not None:
                    yield f"qmeta/{path}/bits/{bit}/{side}/seed", int(sides[side]["seed"])
    qa = meta.get("quant_args", {}).get("seed")
    if qa is not None:
        yield "qmeta/quant_args/seed", int(qa)


def check_qmeta_seeds(meta: dict, qmeta_tensors: Dict[str, torch.Tensor]) -> Tuple[list, list]:
    """Cross-check the redundant seed tensors of the weight file against ``meta.json`` (guards against files
    from two different runs being combined).  Returns (mismatched, missing); warns on either."""
    if not qmeta_tensors:
        warnings.warn("weight file carries no qmeta seeds (old format)")
        return [], []
    bad, missing = [], []
    for key, want in _seed_items(meta):
        got = qmeta_tensors.get(key)
        if got is None:
            missing.append(key)
        elif int(got.item()) != want:
            bad.append((key, want, int(got.item())))
    if bad:
        warnings.warn(f"{len(bad)} qmeta seeds differ from meta.json, e.g. {bad[:3]}: the two files may not belong together")
    elif missing:
        warnings.warn(f"{len(missing)} qmeta seed keys missing, e.g. {missing[:3]}")
    return bad, missing


def save_quantized_model(model, save_dir: str, base_model_path: Optional[str] = None,
                         quant_args: Optional[dict] = None) -> dict:
    """Write ``meta.json`` + ``model.safetensors`` (CPU copies; the model itself is left where it is)."""
    from safetensors.torch import save_file
    os.makedirs(save_dir, exist_ok=True)
    meta = collect_quant_metadata(model, quant_args, getattr(model, "model_id", None), base_model_path)
    with open(os.path.join(save_dir, "meta.json"), "w", encoding="utf-8") as f:
        json.dump(meta, f, indent=1, ensure_ascii=False)
    tensors, seen = {}, set()
    for name, t in model.state_dict().items():
        if id(t) in seen:
            raise AssertionError(f"state_dict shares one tensor under two names ({name})")
        seen.add(id(t))
        tensors[name] = t.detach().cpu().contiguous()
    for key, seed in _seed_items(meta):
        tensors[key] = torch.tensor(seed, dtype=torch.int64)
    save_file(tensors, os.path.join(save_dir, "model.safetensors"))
    return meta


def load_quantized_state_dict(quant_dir: str) -> Tuple[dict, Dict[str, torch.Tensor]]:
    """(meta, tensors) of a checkpoint directory: one ``model.safetensors`` or the shards listed in
    ``model.safetensors.index.json``."""
    from safetensors.torch import load_file
    with open(os.path.join(quant_dir, "meta.json"), "r", encoding="utf-8") as f:
        meta = json.load(f)
    index = os.path.join(quant_dir, "model.safetensors.index.json")
    tensors: Dict[str, torch.Tensor] = {}
    if os.path.isfile(index):
        with open(index, "r", encoding="utf-8") as f:
            shards = sorted(set(json.load(f)["weight_map"].values()))
        for shard in shards:
            tensors.update(load_file(os.path.join(quant_dir, shard)))
    else:
        tensors = load_file(os.path.join(quant_dir, "model.safetensors"))
    return meta, tensors


# --------------------------------------------------------------------------- restore (load side)

def _mapper(key_prefix_map: PrefixMap) -> Callable[[str], str]:
    if key_prefix_map is None:
        return lambda p: p
    if callable(key_prefix_map):
        return key_prefix_map
    old, new = key_prefix_map
    return lambda p: new + p[len(old):] if p.startswith(old) else p


def _parent_of(root, path: str):
    parts = path.split(".")
    mod = root
    for name in parts[:-1]:
        mod = getattr(mod, name)
    return mod, parts[-1]


def restore_quant_metadata(model, meta: dict, state_dict: Optional[dict] = None, key_prefix_map: PrefixMap = None):
    """Swap the skeleton model's dense modules for packed ones described by ``meta`` and fill them.

    Order matters: packed Linears first (the shared expert's projections still sit in the original mlp), then each
    mlp is replaced by a ``WxA16BitPartitionedGroupMoE`` that takes over the old mlp's ``gate``, ``shared_expert``
    and ``shared_expert_gate``, then ``load_state_dict(strict=True, assign=True)``: every key must match.
    ``key_prefix_map`` renames paths and keys (a ``(old, new)`` prefix pair or a callable), for skeletons whose
    module tree is rooted differently from the checkpoint's.
    """
    rename = _mapper(key_prefix_map)
    for path, m in meta.get("modules", {}).items():
        if m.get("type") != "wxa16_linear":
            continue
        parent, attr = _parent_of(model, rename(path))
        setattr(parent, attr, WxA16Linear.from_metadata(m))
    for path, m in meta.get("layers", {}).items():
        parent, attr = _parent_of(model, rename(path))
        old = getattr(parent, attr)
        moe = WxA16BitPartitionedGroupMoE.from_metadata(
            m, gate=old.gate, shared_expert=getattr(old, "shared_expert", None),
            shared_expert_gate=getattr(old, "shared_expert_gate", None))
        setattr(parent, attr, moe)
    if state_dict is not None:
        seeds = {k: v for k, v in state_dict.items() if k.startswith("qmeta/")}
        weights = {rename(k): v for k, v in state_dict.items() if not k.startswith("qmeta/")}
        res = model.load_state_dict(weights, strict=True, assign=True)
        if res.missing_keys or res.unexpected_keys:
            raise AssertionError(f"state dict mismatch: missing {res.missing_keys[:5]}, unexpected {res.unexpected_keys[:5]}")
        left = [n for n, b in model.named_buffers() if b.is_meta]
        if left:
            warnings.warn(f"buffers still on the meta device after loading: {left[:5]}")
        check_qmeta_seeds(meta, seeds)
    return model


def load_quantized_layers(model, quant_dir: str, key_prefix_map: PrefixMap = None):
    """``restore_quant_metadata`` from a checkpoint directory."""
    meta, tensors = load_quantized_state_dict(quant_dir)
    return restore_quant_metadata(model, meta, tensors, key_prefix_map)


# --------------------------------------------------------------------------- activation-mode conversion

def _convert(model, moe_cls, linear_rule: Callable[[WxA16Linear], Optional[type]]) -> Dict[str, int]:
    """In-place class switch of every quantized module (zero copy: the packed storage is mode independent)."""
    count = {"moe": 0, "linear": 0, "kept": 0}
    for sub in list(model.modules()):
        if isinstance(sub, WxA16BitPartitionedGroupMoE):
            moe_cls.from_wxa16(sub)
            count["moe"] += 1
        elif isinstance(sub, WxA16Linear) and sub.bit_width == 8:
            cls = linear_rule(sub)
            if cls is None:
                count["kept"] += 1
            elif cls is not type(sub):
                cls.from_wxa16(sub)
                count["linear"] += 1
    return count


def _int8_if_uniform(lin: WxA16Linear):
    # a Lloyd-Max 8-bit codebook squeezed onto the int8 grid would lose about a quarter of its levels:
    # such layers keep fp16 activations
    return WxA8Linear if fmt.is_uniform_codebook(lin.codebook) else None


def convert_model_to_wxa8(model) -> Dict[str, int]:
    """MoE layers -> INT8 activations; 8-bit packed Linears with a uniform codebook -> WxA8Linear, others stay."""
    return _convert(model, WxA8BitPartitionedGroupMoE, _int8_if_uniform)


def convert_model_to_wxfp8(model, attn: str = "wxa8") -> Dict[str, int]:
    """MoE layers -> e4m3 activations.  ``attn`` picks the path of the 8-bit packed Linears: ``"wxa8"`` (int8 where
    the codebook is uniform), ``"wxfp8"`` (e4m3 LUT, any codebook) or ``"wxa16"`` (left alone)."""
    if attn not in ("wxa8", "wxfp8", "wxa16"):
        raise ValueError(f"unknown attn mode {attn!r}")
    rule = {"wxa8": _int8_if_uniform, "wxfp8": lambda lin: WxFP8Linear, "wxa16": lambda lin: type(lin)}[attn]
    return _convert(model, WxFP8BitPartitionedGroupMoE, rule)


def convert_model_to_wxfp4(model) -> Dict[str, int]:
    """MoE layers -> e2m1 activations for the 1- and 4-bit pools, INT8 for 2-bit; packed Linears as in WxA8."""
    return _convert(model, WxFP4BitPartitionedGroupMoE, _int8_if_uniform)
