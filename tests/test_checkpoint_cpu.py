"""Checkpoint format and module construction against files and tensors written by the reference itself
(tests/golden/make_golden.py, ``checkpoint`` step): pool layout of ``from_build_block``, and a
``meta.json`` + ``model.safetensors`` pair saved by the reference's ``save_quantized_model``."""
import json
import os

import numpy as np
import pytest
import torch
import torch.nn as nn

import dartmoq_b200 as D
from dartmoq_b200 import checkpoint as ckpt

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CKPT = os.path.join(ROOT, "tests", "golden", "ckpt_ref")
H, E = 128, 4
NEURONS = {0: {4: 128}, 1: {4: 128, 2: 128}, 2: {2: 256}, 3: {2: 128}}


def test_from_build_block_matches_reference(golden):
    """Staged fp16 sub-experts -> packed pools: gate rows then up rows per expert, down columns, offsets, seeds
    42+bit / 42+bit+1000, bit for bit what the reference's from_build_block produced from the same weights."""
    g = golden("build_block")

    class Sub(nn.Module):
        def __init__(self, e, bit, n):
            super().__init__()
            self._quant_bit = bit
            self.gate_proj, self.up_proj = nn.Linear(H, n, bias=False), nn.Linear(H, n, bias=False)
            self.down_proj = nn.Linear(n, H, bias=False)
            for name in ("gate_proj", "up_proj", "down_proj"):
                getattr(self, name).weight.data.copy_(torch.from_numpy(g[f"w_{e}_{bit}_{name}"]))

    class Wrapper(nn.Module):
        def __init__(self, e):
            super().__init__()
            self.sub_experts = nn.ModuleList([Sub(e, b, n) for b, n in NEURONS[e].items()])

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.gate = nn.Linear(H, E, bias=False)
            self.top_k = 2
            self.experts = nn.ModuleList([Wrapper(e) for e in range(E)])

    md = {"num_experts": E, "hidden_size": H, "intermediate_size": 256, "bit_list": [4, 2],
          "expert_bit_indices": [{b: list(range(n)) for b, n in NEURONS[e].items()} for e in range(E)]}
    moe = D.WxA16BitPartitionedGroupMoE.from_build_block(Block(), md, group_size=128)
    assert moe.top_k == 2 and moe.bit_list == [4, 2] and set(moe.bit_weights.keys()) == {"4", "2"}
    for bs, w in moe.bit_weights.items():
        assert moe.expert_offsets[bs].tolist() == g[f"offsets_{bs}"].tolist()
        for side, pk in (("gate_up", w.gate_up_packed), ("down", w.down_packed)):
            assert int(pk["seed"]) == int(g[f"{side}_seed_{bs}"]) == 42 + int(bs) + (1000 if side == "down" else 0)
            for k in ("indices_packed", "norms", "codebook"):
                assert np.array_equal(pk[k].cpu().numpy(), g[f"{side}_{k}_{bs}"]), (bs, side, k)


def _skeleton():
    """The dense model the loader starts from: an mlp with gate / shared expert / shared gate, one attention Linear."""
    mlp = nn.Module()
    mlp.gate = nn.Linear(H, E, bias=False)
    mlp.shared_expert = nn.Module()
    mlp.shared_expert.gate_proj, mlp.shared_expert.up_proj = nn.Linear(H, 128, bias=False), nn.Linear(H, 128, bias=False)
    mlp.shared_expert.down_proj = nn.Linear(128, H, bias=False)
    mlp.shared_expert_gate = nn.Linear(H, 1, bias=False)
    layer = nn.Module()
    layer.mlp = mlp
    layer.self_attn = nn.Module()
    layer.self_attn.q_proj = nn.Linear(H, 256, bias=True)
    model = nn.Module()
    model.model = nn.Module()
    model.model.layers = nn.ModuleList([layer])
    return model


def test_reference_checkpoint_loads_and_converts(tmp_path):
    from safetensors.torch import load_file
    meta, tensors = ckpt.load_quantized_state_dict(CKPT)
    assert set(meta["layers"]) == {"model.layers.0.mlp"} and len(meta["modules"]) == 4
    model = ckpt.restore_quant_metadata(_skeleton(), meta, tensors)
    layer = model.model.layers[0]
    moe = layer.mlp
    assert type(moe) is D.WxA16BitPartitionedGroupMoE and type(layer.self_attn.q_proj) is D.WxA16Linear
    assert type(moe.shared_expert.gate_proj) is D.WxA16Linear
    # every tensor of the file sits in the model, nothing else does (strict load), seeds come from meta.json
    sd = model.state_dict()
    weights = {k: v for k, v in tensors.items() if not k.startswith("qmeta/")}
    assert set(sd) == set(weights)
    for k, v in weights.items():
        assert torch.equal(sd[k], v), k
    lm = meta["layers"]["model.layers.0.mlp"]
    for bs, w in moe.bit_weights.items():
        assert moe._offsets_lists()[bs] == lm["expert_offsets"][bs]
        assert w.gate_up_packed["seed"] == lm["bits"][bs]["gate_up"]["seed"] == int(tensors[f"qmeta/model.layers.0.mlp/bits/{bs}/gate_up/seed"])
        assert tuple(w.down_packed["shape"]) == tuple(lm["bits"][bs]["down"]["shape"])
    assert layer.self_attn.q_proj.seed == 78 and layer.self_attn.q_proj.bias is not None
    assert moe._shared_packs() is not None            # the loaded shared expert runs as a pool of the layer
    bad, missing = ckpt.check_qmeta_seeds(meta, {k: v for k, v in tensors.items() if k.startswith("qmeta/")})
    assert not bad and not missing
    # a seed that disagrees with meta.json is reported
    wrong = dict(tensors)
    wrong["qmeta/model.layers.0.mlp/bits/2/down/seed"] = torch.tensor(7, dtype=torch.int64)
    with pytest.warns(UserWarning):
        bad, _ = ckpt.check_qmeta_seeds(meta, {k: v for k, v in wrong.items() if k.startswith("qmeta/")})
    assert len(bad) == 1
    # a missing tensor fails the strict load
    short = {k: v for k, v in tensors.items() if not k.endswith("down_norms")}
    with pytest.raises((AssertionError, RuntimeError)):
        ckpt.restore_quant_metadata(_skeleton(), meta, short)

    # ---- saving the loaded model gives the reference's files back
    out = tmp_path / "resaved"
    ckpt.save_quantized_model(model, str(out), quant_args={"seed": 0})
    meta2 = json.load(open(out / "meta.json"))
    assert meta2["layers"] == meta["layers"] and meta2["modules"] == meta["modules"]
    t2 = load_file(str(out / "model.safetensors"))
    assert set(t2) == set(tensors) and all(torch.equal(t2[k], tensors[k]) for k in tensors)

    # ---- activation-mode conversion: class switches only, no tensor moves
    ptrs = {k: v.data_ptr() for k, v in model.state_dict().items()}
    n = ckpt.convert_model_to_wxa8(model)
    assert n == {"moe": 1, "linear": 4, "kept": 0}
    assert type(moe) is D.WxA8BitPartitionedGroupMoE and type(layer.self_attn.q_proj) is D.WxA8Linear
    assert {k: v.data_ptr() for k, v in model.state_dict().items()} == ptrs
    model = ckpt.restore_quant_metadata(_skeleton(), meta, tensors)
    ckpt.convert_model_to_wxfp8(model, attn="wxfp8")
    assert type(model.model.layers[0].mlp) is D.WxFP8BitPartitionedGroupMoE
    assert type(model.model.layers[0].self_attn.q_proj) is D.WxFP8Linear
    model = ckpt.restore_quant_metadata(_skeleton(), meta, tensors)
    ckpt.convert_model_to_wxfp8(model, attn="wxa16")
    assert type(model.model.layers[0].self_attn.q_proj) is D.WxA16Linear
    model = ckpt.restore_quant_metadata(_skeleton(), meta, tensors)
    ckpt.convert_model_to_wxfp4(model)
    assert type(model.model.layers[0].mlp) is D.WxFP4BitPartitionedGroupMoE
    assert type(model.model.layers[0].mlp.shared_expert.down_proj) is D.WxA8Linear
    with pytest.raises(ValueError):
        ckpt.convert_model_to_wxfp8(model, attn="int4")


def test_prefix_map_renames_paths():
    meta, tensors = ckpt.load_quantized_state_dict(CKPT)
    inner = _skeleton()
    outer = nn.Module()
    outer.language_model = inner
    ckpt.restore_quant_metadata(outer, meta, tensors, key_prefix_map=("model.", "language_model.model."))
    assert type(outer.language_model.model.layers[0].mlp) is D.WxA16BitPartitionedGroupMoE
    outer2 = nn.Module()
    outer2.language_model = _skeleton()
    ckpt.restore_quant_metadata(outer2, meta, tensors, key_prefix_map=lambda k: "language_model." + k)
    assert torch.equal(outer2.state_dict()["language_model.model.layers.0.mlp.gate.weight"],
                       tensors["model.layers.0.mlp.gate.weight"])
