"""Packed dense Linear layers (the shared expert's projections use these).

Same storage and constructor as the reference classes
    WxA16Linear   quantization/wxa16/linear.py:25
    WxA8Linear    quantization/wxa8/linear.py:75   (8-bit uniform codebook, weight = index-128)
    WxFP8Linear   quantization/wxfp8/linear.py:33
state_dict keys: ``packed_indices`` (uint8), ``norms`` (fp16), ``codebook`` (fp16), optional ``bias``.
``forward`` = group rotation (+ activation quantisation) followed by the same
grouped LUT-dequant GEMM the MoE uses, run as a single "expert" over all rows.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Optional

import torch
import torch.nn as nn

from . import _lib
from . import format as fmt
from . import kernels as K
from ._lib import A16, A8, FP8, EPI_PLAIN

GROUP = fmt.GROUP_SIZE


class WxA16Linear(nn.Module):
    """y = x @ W^T (+ bias) over packed W; fp16 activations."""

    MODE = A16

    def __init__(self, in_features: int, out_features: int, bit_width: int, group_size: int,
                 packed_indices: torch.Tensor, codebook: torch.Tensor, norms: torch.Tensor, seed: int,
                 rotation: str = "qr", bias=None, orig_dtype: torch.dtype = torch.float16,
                 codebook_type: str = "lloydmax"):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.bit_width, self.group_size = bit_width, group_size
        self.seed, self.rotation = seed, rotation
        self.orig_dtype, self.codebook_type = orig_dtype, codebook_type
        self.register_buffer("packed_indices", packed_indices)
        self.register_buffer("norms", norms)
        self.register_buffer("codebook", codebook)
        if bias is not None:
            self.register_buffer("bias", bias)
        else:
            self.bias = None
        self.n_groups = (in_features + group_size - 1) // group_size
        self._rt = None

    @classmethod
    @torch.no_grad()
    def from_linear(cls, linear: nn.Linear, bit_width: int, group_size=None, seed: int = 42,
                    rotation: str = "qr", keep_on_gpu: bool = True, uniform_codebook: bool = False):
        """Quantise an ``nn.Linear`` (reference: quantization/wxa16/linear.py:83)."""
        group_size = linear.in_features if group_size is None else group_size
        pk = fmt.turboquant_quantize_packed_full(linear.weight.data, bit_width, group_size, seed, rotation,
                                                 keep_on_gpu, uniform_codebook)
        bias = linear.bias.data.clone() if linear.bias is not None else None
        return cls(linear.in_features, linear.out_features, bit_width, group_size, pk["indices_packed"],
                   pk["codebook"], pk["norms"], seed, rotation, bias, linear.weight.dtype, pk["codebook_type"])

    @classmethod
    def from_metadata(cls, meta: dict):
        """Placeholder buffers of the saved shapes; the state dict fills them."""
        bias = torch.empty(meta["bias_shape"], dtype=torch.float16) if meta.get("bias_shape") else None
        dtype = getattr(torch, str(meta.get("orig_dtype", "torch.float16")).split(".")[-1])
        return cls(meta["in_features"], meta["out_features"], meta["bit_width"], meta["group_size"],
                   torch.empty(meta["indices_packed_shape"], dtype=torch.uint8),
                   torch.empty(meta["codebook_shape"], dtype=torch.float16),
                   torch.empty(meta["norms_shape"], dtype=torch.float16), meta["seed"],
                   meta.get("rotation", "qr"), bias, dtype, meta.get("codebook_type", "lloydmax"))

    @classmethod
    def from_wxa16(cls, linear: "WxA16Linear"):
        """In-place switch of the activation mode (zero copy)."""
        if not isinstance(linear, WxA16Linear):
            raise TypeError(f"expected WxA16Linear, got {type(linear)}")
        if cls.MODE == A8 and not (linear.bit_width == 8 and fmt.is_uniform_codebook(linear.codebook)):
            raise ValueError("WxA8Linear needs an 8-bit uniform codebook (weight = index-128)")
        linear.__class__ = cls
        linear._rt = None
        return linear

    def _apply(self, fn, *args, **kwargs):
        ret = super()._apply(fn, *args, **kwargs)
        self._rt = None
        return ret

    def _runtime(self, device):
        rt = self._rt
        if rt is not None and rt["device"] == device:
            return rt
        if self.group_size != GROUP or self.in_features % GROUP or self.out_features % GROUP:
            raise ValueError("packed Linear needs group_size 128 and feature sizes that are multiples of 128")
        from .moe import _group_first_device, _mode_lut, _true_div_half
        lut, act_scale, e0, factor, identity = _mode_lut(self.MODE, self.bit_width, self.codebook, device)
        norms = _true_div_half(self.norms.to(device).t().contiguous(), math.sqrt(GROUP))
        rt = {
            "device": device,
            "idx": _group_first_device(self.packed_indices, self.bit_width, self.in_features, device),
            "norms": norms, "lut": lut, "act_scale": act_scale, "identity": bool(identity),
            "rot": fmt.generate_batch_rotation_matrices(GROUP, int(self.seed), self.in_features // GROUP, GROUP,
                                                        device, torch.float16),
        }
        self._rt = rt
        return rt

    @torch.no_grad()
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        x2 = x.reshape(-1, self.in_features).contiguous()
        rt = self._runtime(x2.device)
        G = self.in_features // GROUP
        n = x2.shape[0]
        if self.MODE == A16:
            codes = torch.empty((n, self.in_features), dtype=torch.float16, device=x2.device)
            scales = None
        else:
            codes = torch.empty((n, self.in_features), dtype=torch.uint8, device=x2.device)
            scales = torch.empty((n, G), dtype=torch.float16, device=x2.device)
        if n:
            K._rotate(self.MODE, x2, rt["rot"], rt["act_scale"], codes, scales)
        info = [(0, n, 0, G)]
        out = K._merged(self.MODE, True, codes, scales, self.in_features, rt["idx"], rt["lut"], rt["norms"], info,
                        GROUP, self.bit_width, True, identity=rt["identity"], epilogue=EPI_PLAIN) if n else \
            torch.empty((0, self.out_features), dtype=torch.float16, device=x2.device)
        if self.bias is not None:
            out = out + self.bias.to(out.device, out.dtype)
        return out.to(x.dtype).reshape(*shape[:-1], self.out_features)

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, bit_width={self.bit_width}, "
                f"group_size={self.group_size}, rotation={self.rotation}")


class WxA8Linear(WxA16Linear):
    """INT8 activations over an 8-bit uniform codebook."""
    MODE = A8


class WxFP8Linear(WxA16Linear):
    """e4m3 activations and an e4m3 codebook LUT."""
    MODE = FP8
