"""Packed-weight format of the rotated-codebook quantizer (host side, torch).

Everything here defines *data layout and load-time constants*; nothing runs per
forward.  It reproduces, value for value, what the reference checkpoint format
stores and what its load-time helpers derive, so a packed checkpoint written by
the reference loads here unchanged:

* index packing                      turboquant_utils/quantize.py:35 / :74
* Lloyd-Max N(0,1) codebooks         turboquant_utils/codebook.py:18 / :77
* seeded Haar rotations              turboquant_utils/rotation.py:53 / :127
* the quantizer (fixture builder)    turboquant_utils/quantize.py:350
* group-first relayout               turboquant_utils/triton_kernels.py:1042
* int8 / e4m3 / e2m1 codebook LUTs   turboquant_utils/triton_kernels_a8.py:526,
                                     triton_kernels_fp8.py:35, triton_kernels_fp4.py:32 / :80
"""

from __future__ import annotations

import math
from typing import Dict, Optional, Tuple

import numpy as np
import torch

GROUP_SIZE = 128
SUPPORTED_BITS = (1, 2, 4, 8)
E4M3_MAX = 448.0
E2M1_GRID = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
E2M1_MAX = 6.0


def _check_bits(bit_width: int) -> None:
    if bit_width not in SUPPORTED_BITS:
        raise ValueError(f"Only {set(SUPPORTED_BITS)} bits are supported, got {bit_width}")


# --------------------------------------------------------------------------- packing

def pack_nbit(indices: torch.Tensor, bit_width: int) -> torch.Tensor:
    """Pack b-bit indices along the last dim, element j of a byte at bits [j*b, j*b+b).

    The last dim is zero-padded up to a whole byte (quantize.py:35-71).
    """
    _check_bits(bit_width)
    per_byte = 8 // bit_width
    n = indices.shape[-1]
    pad = (-n) % per_byte
    if pad:
        indices = torch.nn.functional.pad(indices, (0, pad), value=0)
    lanes = indices.reshape(*indices.shape[:-1], -1, per_byte).to(torch.uint8)
    lanes = lanes & ((1 << bit_width) - 1)
    out = torch.zeros(lanes.shape[:-1], dtype=torch.uint8, device=indices.device)
    for j in range(per_byte):
        out |= lanes[..., j] << (j * bit_width)
    return out


def unpack_nbit(packed: torch.Tensor, bit_width: int, n: int) -> torch.Tensor:
    """Inverse of :func:`pack_nbit`; returns int32 indices of length ``n`` (quantize.py:74-100)."""
    _check_bits(bit_width)
    per_byte = 8 // bit_width
    mask = (1 << bit_width) - 1
    shifts = torch.arange(per_byte, device=packed.device, dtype=torch.uint8) * bit_width
    lanes = (packed.unsqueeze(-1) >> shifts) & mask
    return lanes.reshape(*packed.shape[:-1], -1)[..., :n].to(torch.int32)


def convert_to_group_first(indices_packed: torch.Tensor, norms: torch.Tensor,
                           group_size: int, bit_width: int):
    """(N, K*b/8) row-major bytes -> (G, N, gs*b/8); norms (N, G) -> (G, N).

    triton_kernels.py:1042-1068.  Each group's bytes for all rows become one
    contiguous slab, which is what the streaming kernels read.
    """
    per_group = group_size * bit_width // 8
    n_rows, total = indices_packed.shape
    groups = total // per_group
    gf = indices_packed.reshape(n_rows, groups, per_group).permute(1, 0, 2).contiguous()
    return gf, norms.t().contiguous()


# --------------------------------------------------------------------------- codebooks

_CODEBOOKS: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}


def _lloyd_max_gaussian(levels: int, iters: int = 200):
    """Lloyd-Max quantizer of N(0,1): centroid = E[X | cell], boundary = midpoint.

    Same start (uniform cells on [-3.5, 3.5], outer edges at +-1e10), same
    update order and iteration count as codebook.py:18-71, evaluated in float64
    with scipy's normal cdf/pdf.
    """
    from scipy.stats import norm

    edges = np.linspace(-3.5, 3.5, levels + 1)
    edges[0], edges[-1] = -1e10, 1e10
    cent = np.zeros(levels)
    for _ in range(iters):
        for i in range(levels):
            lo, hi = edges[i], edges[i + 1]
            mass = norm.cdf(hi) - norm.cdf(lo)
            if mass > 1e-15:
                cent[i] = (norm.pdf(lo) - norm.pdf(hi)) / mass
            else:
                cent[i] = (max(lo, -3.5) + min(hi, 3.5)) / 2
        for i in range(1, levels):
            edges[i] = (cent[i - 1] + cent[i]) / 2
    return cent, edges


def get_codebook(bit_width: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """(centroids fp32 (2^b,), inner boundaries fp32 (2^b-1,)), cached (codebook.py:77-100)."""
    if bit_width not in _CODEBOOKS:
        cent, edges = _lloyd_max_gaussian(2 ** bit_width)
        _CODEBOOKS[bit_width] = (torch.tensor(cent, dtype=torch.float32),
                                 torch.tensor(edges[1:-1], dtype=torch.float32))
    return _CODEBOOKS[bit_width]


def uniform8_codebook() -> Tuple[torch.Tensor, torch.Tensor]:
    """Uniform 256-level grid cb[i] = (i-128)*3.5/128 used by dense 8-bit layers (quantize.py:394-402)."""
    step = 3.5 / 128.0
    cent = (torch.arange(256, dtype=torch.float32) - 128) * step
    edges = (torch.arange(255, dtype=torch.float32) - 127.5) * step
    return cent, edges


# --------------------------------------------------------------------------- rotations

_ROT: Dict[Tuple[int, int], torch.Tensor] = {}
_ROT_STACK: Dict[tuple, torch.Tensor] = {}


def generate_rotation_matrix(d: int, seed: int = 42, device=None) -> torch.Tensor:
    """Seeded Haar-distributed orthogonal matrix, fp32 (rotation.py:53-117).

    Always computed on the CPU with ``torch.Generator().manual_seed(seed)`` ->
    ``randn(d, d)`` -> QR -> columns sign-fixed by diag(R), so the quantizer and
    the inference side see the same bits regardless of where they run.
    """
    key = (d, seed)
    base = _ROT.get(key)
    if base is None:
        gen = torch.Generator().manual_seed(seed)
        q, r = torch.linalg.qr(torch.randn(d, d, generator=gen))
        base = (q * torch.sign(torch.diag(r)).unsqueeze(0)).contiguous()
        if len(_ROT) >= 8192:
            _ROT.pop(next(iter(_ROT)))
        _ROT[key] = base
    return base if device is None else base.to(device)


def generate_batch_rotation_matrices(d: int, seed_base: int, num_groups: int, stride: int,
                                     device, dtype: torch.dtype = torch.float16) -> torch.Tensor:
    """Stack (num_groups, d, d): matrix g uses seed ``seed_base + g*stride`` (rotation.py:127-173)."""
    key = (d, seed_base, num_groups, stride, str(device), str(dtype))
    hit = _ROT_STACK.get(key)
    if hit is not None:
        return hit
    stack = torch.stack([generate_rotation_matrix(d, seed_base + g * stride).to(dtype)
                         for g in range(num_groups)]).contiguous().to(device)
    if len(_ROT_STACK) >= 64:
        _ROT_STACK.pop(next(iter(_ROT_STACK)))
    _ROT_STACK[key] = stack
    return stack


def clear_rotation_cache() -> None:
    _ROT.clear()
    _ROT_STACK.clear()


# --------------------------------------------------------------------------- quantizer

@torch.no_grad()
def turboquant_quantize_packed_full(W: torch.Tensor, bit_width: int, group_size: Optional[int] = None,
                                    seed: int = 42, rotation: str = "qr", keep_on_gpu: bool = False,
                                    uniform_codebook: bool = False) -> dict:
    """Quantize ``W (N, K)`` to the packed format (quantize.py:350-472).

    Per ``group_size`` columns: row L2 norm (>=1e-8), normalise, rotate by
    Pi(seed + g_start)^T, scale by sqrt(group), bucket into the codebook's
    cells with ``searchsorted``.  Returns the same dict keys the reference
    writes into a checkpoint.
    """
    _check_bits(bit_width)
    if uniform_codebook and bit_width != 8:
        raise ValueError(f"uniform_codebook requires bit_width=8, got {bit_width}")
    if rotation != "qr":
        raise ValueError("only the 'qr' rotation is part of the MoE hot path")
    n_rows, k = W.shape
    group_size = k if group_size is None else group_size
    cent, edges = uniform8_codebook() if uniform_codebook else get_codebook(bit_width)
    cent_d, edges_d = cent.to(W.device), edges.to(W.device)

    norms, idx = [], []
    for g0 in range(0, k, group_size):
        wg = W[:, g0:g0 + group_size].float()
        nrm = wg.norm(dim=1, keepdim=True).clamp(min=1e-8)
        pi = generate_rotation_matrix(wg.shape[1], seed=seed + g0).to(W.device)
        y = ((wg / nrm) @ pi.T) * math.sqrt(wg.shape[1])
        cell = torch.searchsorted(edges_d, y.reshape(-1)).clamp(0, len(cent_d) - 1)
        idx.append(cell.reshape(n_rows, -1).to(torch.uint8))
        norms.append(nrm.squeeze(1))
    norms_out = torch.stack(norms, dim=1) if len(norms) > 1 else norms[0]
    dev = W.device if keep_on_gpu else "cpu"
    return {
        "indices_packed": pack_nbit(torch.cat(idx, dim=1), bit_width).to(dev),
        "codebook": cent.half().cpu(),
        "norms": norms_out.half().to(dev),
        "seed": seed,
        "group_size": group_size,
        "shape": (n_rows, k),
        "bit_width": bit_width,
        "rotation": rotation,
        "orig_dtype": str(W.dtype),
        "codebook_type": "uniform" if uniform_codebook else "lloydmax",
    }


@torch.no_grad()
def turboquant_dequantize_packed(packed: dict, device=None) -> torch.Tensor:
    """Packed dict -> dense matrix in the original dtype (quantize.py:478-557)."""
    dev = packed["indices_packed"].device if device is None else device
    n_rows, k = packed["shape"]
    gs = packed["group_size"]
    cb = packed["codebook"].to(dev).float()
    norms = packed["norms"].to(dev).float()
    if norms.dim() == 1:
        norms = norms.unsqueeze(1)
    idx = unpack_nbit(packed["indices_packed"].to(dev), packed["bit_width"], k).long()
    out = torch.zeros(n_rows, k, dtype=torch.float32, device=dev)
    for g, g0 in enumerate(range(0, k, gs)):
        y = cb[idx[:, g0:g0 + gs]] / math.sqrt(min(gs, k - g0))
        pi = generate_rotation_matrix(y.shape[1], seed=packed["seed"] + g0).to(dev)
        out[:, g0:g0 + gs] = (y @ pi) * norms[:, g:g + 1]
    dtype = getattr(torch, str(packed.get("orig_dtype", "torch.float16")).split(".")[-1])
    return out.to(dtype)


# --------------------------------------------------------------------------- activation-mode LUTs

def build_int8_codebook(codebook: torch.Tensor):
    """fp16 codebook -> (int8 LUT, step) with codebook[i] ~= lut[i]*step (triton_kernels_a8.py:526-553)."""
    cb = codebook.float()
    top = cb.abs().max()
    if top <= 0:
        raise ValueError("all-zero codebook cannot be mapped to int8")
    step = (top / 127.0).item()
    lut = (cb / step).round().clamp_(-127, 127).to(torch.int8)
    return lut.contiguous(), step


def is_uniform_codebook(codebook: torch.Tensor, rel_tol: float = 1e-2) -> bool:
    """True for the 256-level uniform grid (quantization/wxa8/linear.py:50-62)."""
    if codebook.numel() != 256:
        return False
    d = codebook.float()[1:] - codebook.float()[:-1]
    mean = d.mean().abs()
    return bool(mean > 0 and (d - d.mean()).abs().max() < rel_tol * mean)


def uniform_codebook_step(codebook: torch.Tensor) -> float:
    """Step of a uniform 256-level codebook, (cb[255]-cb[0])/255 (quantization/wxa8/linear.py:35-47)."""
    cb = codebook.float()
    if cb.numel() != 256:
        raise ValueError(f"an 8-bit codebook has 256 levels, got {cb.numel()}")
    step = (cb[-1] - cb[0]) / 255.0
    if step <= 0:
        raise ValueError(f"illegal codebook step {step}")
    return float(step)


def _relerr(cb: torch.Tensor, lut: torch.Tensor, scale: float) -> float:
    return ((lut.float() * scale - cb).norm() / cb.norm()).item()


def build_fp8_codebook(codebook: torch.Tensor, n_coarse: int = 512):
    """fp16 codebook -> (e4m3 LUT, scale) minimising ||lut*scale - cb|| (triton_kernels_fp8.py:35-88).

    One scalar scale is searched: ``n_coarse`` log-spaced points a decade either
    side of max/448, then two 64-point refinements around the best.  The
    candidate lists are produced by the same float operations as the reference
    so the argmin (and therefore the LUT) is identical.
    """
    cb = codebook.float()
    top = cb.abs().max()
    if top <= 0:
        raise ValueError("all-zero codebook cannot be mapped to fp8")

    def lut_at(s: float) -> torch.Tensor:
        return (cb / s).clamp_(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)

    s0 = (top / E4M3_MAX).item()
    mid = torch.log10(torch.tensor(s0))
    coarse = torch.logspace(mid - 1.0, mid + 1.0, n_coarse).tolist()
    best_s, best_err = s0, float("inf")
    for s in coarse:
        err = _relerr(cb, lut_at(s), s)
        if err < best_err:
            best_s, best_err = s, err
    span = (coarse[1] / coarse[0]) if len(coarse) > 1 else 1.0
    for ratio in (span ** 0.5, span ** 0.25):
        for s in [best_s * ratio ** (i / 64.0 - 0.5) for i in range(64)]:
            err = _relerr(cb, lut_at(s), s)
            if err < best_err:
                best_s, best_err = s, err
    return lut_at(best_s).contiguous(), best_s


def build_e2m1_codebook(codebook: torch.Tensor):
    """fp16 codebook -> (nibble LUT, E0, residual, relerr) (triton_kernels_fp4.py:32-77).

    ``codebook[i] ~= e2m1(nib[i]) * 2**E0 * residual``; 2**E0 rides the e8m0
    block-scale channel, the residual is folded into the per-row norms.
    """
    cb = codebook.float()
    top = cb.abs().max()
    if top <= 0:
        raise ValueError("all-zero codebook cannot be mapped to e2m1")
    grid = torch.tensor(E2M1_GRID, device=cb.device)

    def fit(s):
        y = (cb / s).clamp(-E2M1_MAX, E2M1_MAX)
        mag = torch.argmin((y.abs().unsqueeze(-1) - grid).abs(), dim=-1)
        nib = ((mag & 0x7) | (((y < 0).to(torch.uint8) << 3).long())).to(torch.uint8)
        rec = grid[mag] * y.sign() * s
        return nib, ((rec - cb).norm() / cb.norm()).item()

    s0 = top / E2M1_MAX
    best_s, best_err, best_lut = s0, float("inf"), None
    for s in [s0 * (2.0 ** (i / 16.0)) for i in range(-16, 17)]:
        nib, err = fit(s)
        if err < best_err:
            best_s, best_err, best_lut = s, err, nib
    for _ in range(2):
        span = 2.0 ** (1 / 16)
        lo, hi = best_s / span, best_s * span
        for s in [lo * (hi / lo) ** (i / 64.0) for i in range(65)]:
            nib, err = fit(s)
            if err < best_err:
                best_s, best_err, best_lut = s, err, nib
    e0 = math.floor(math.log2(best_s))
    return best_lut.contiguous(), e0, float(best_s / (2.0 ** e0)), best_err


def fold_indices_to_e2m1(indices_packed_gf: torch.Tensor, nib: torch.Tensor,
                         bit_width: int, group_size: int) -> torch.Tensor:
    """(G, N, gs*b/8) codebook indices -> (G, N, gs/2) packed e2m1, even k in the low nibble.

    triton_kernels_fp4.py:80-127.  Done through a 256-entry byte LUT: every
    packed byte expands to ``8/b`` nibbles = ``4/b`` output bytes.
    """
    if bit_width not in (1, 2, 4):
        raise ValueError(f"fold supports bit 1/2/4, got {bit_width}")
    dev = indices_packed_gf.device
    per_byte = 8 // bit_width
    byte = torch.arange(256, dtype=torch.int64)
    nibs = torch.stack([nib.cpu().long()[(byte >> (j * bit_width)) & ((1 << bit_width) - 1)]
                        for j in range(per_byte)], dim=1)            # (256, per_byte)
    lut = (nibs[:, 0::2] | (nibs[:, 1::2] << 4)).to(torch.uint8).to(dev)   # (256, per_byte/2)
    g, n, _ = indices_packed_gf.shape
    out = torch.empty((g, n, group_size // 2), dtype=torch.uint8, device=dev)
    step = max(1, (1 << 24) // max(n * group_size // 2, 1))
    for g0 in range(0, g, step):
        sub = indices_packed_gf[g0:g0 + step]
        out[g0:g0 + step] = lut[sub.long()].reshape(sub.shape[0], n, group_size // 2)
    return out
