"""CPU oracle for the mixed-bit codebook-quantized MoE expert path.  TEST INFRASTRUCTURE ONLY.

This file restates, on the CPU, the algorithm of the reference project's MoE
expert path so that the CUDA kernels can be checked against it.  It is never
imported by the product package: only ``tests/``, ``__graft_entry__.smoke()``
and ``bench.py``'s CPU-baseline legs use it, and only as the checker / the
timed CPU baseline.

Parity pin: every function below is checked in ``tests/test_oracle_golden.py``
against vectors produced by running the reference's own code in the build
container (``tests/golden/make_golden.py`` imports the reference, including its
Triton kernels under the Triton CPU interpreter, and stores inputs + outputs).

Byte/integer stages use numpy; half / bfloat16 / float8 roundings use torch's
CPU conversions; the seeded rotation needs torch's CPU generator and QR because
the format defines the matrices through them.

Citations are paths inside the reference project.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch

GS = 128
E2M1_VALUES = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)


# =========================================================================== format

def pack_nbit(idx: np.ndarray, bit: int) -> np.ndarray:
    """turboquant_utils/quantize.py:35 - element j of a byte sits at bits [j*bit, (j+1)*bit)."""
    per = 8 // bit
    idx = np.asarray(idx)
    pad = (-idx.shape[-1]) % per
    if pad:
        idx = np.concatenate([idx, np.zeros(idx.shape[:-1] + (pad,), idx.dtype)], axis=-1)
    lanes = idx.reshape(idx.shape[:-1] + (-1, per)).astype(np.uint8) & ((1 << bit) - 1)
    out = np.zeros(lanes.shape[:-1], np.uint8)
    for j in range(per):
        out |= (lanes[..., j] << (j * bit)).astype(np.uint8)
    return out


def unpack_nbit(packed: np.ndarray, bit: int, n: int) -> np.ndarray:
    """turboquant_utils/quantize.py:74."""
    per = 8 // bit
    packed = np.asarray(packed, np.uint8)
    lanes = np.stack([(packed >> (j * bit)) & ((1 << bit) - 1) for j in range(per)], axis=-1)
    return lanes.reshape(packed.shape[:-1] + (-1,))[..., :n].astype(np.int32)


def group_first(indices_packed: np.ndarray, norms: np.ndarray, bit: int):
    """turboquant_utils/triton_kernels.py:1042: (N, G*bpg) -> (G, N, bpg); norms (N, G) -> (G, N)."""
    bpg = GS * bit // 8
    n = indices_packed.shape[0]
    g = indices_packed.shape[1] // bpg
    return (np.ascontiguousarray(indices_packed.reshape(n, g, bpg).transpose(1, 0, 2)),
            np.ascontiguousarray(np.asarray(norms).reshape(n, -1).T))


_CB: Dict[int, Tuple[np.ndarray, np.ndarray]] = {}


def lloyd_max(bit: int) -> Tuple[np.ndarray, np.ndarray]:
    """turboquant_utils/codebook.py:18-100: (centroids fp32, inner boundaries fp32) for N(0,1)."""
    if bit in _CB:
        return _CB[bit]
    from scipy.stats import norm
    n = 2 ** bit
    b = np.linspace(-3.5, 3.5, n + 1)
    b[0], b[-1] = -1e10, 1e10
    c = np.zeros(n)
    for _ in range(200):
        for i in range(n):
            lo, hi = b[i], b[i + 1]
            p = norm.cdf(hi) - norm.cdf(lo)
            c[i] = (norm.pdf(lo) - norm.pdf(hi)) / p if p > 1e-15 else (max(lo, -3.5) + min(hi, 3.5)) / 2
        for i in range(1, n):
            b[i] = (c[i - 1] + c[i]) / 2
    _CB[bit] = (c.astype(np.float32), b[1:-1].astype(np.float32))
    return _CB[bit]


def uniform8() -> Tuple[np.ndarray, np.ndarray]:
    """turboquant_utils/quantize.py:394-402."""
    step = np.float32(3.5 / 128.0)
    return ((np.arange(256, dtype=np.float32) - 128) * step,
            (np.arange(255, dtype=np.float32) - np.float32(127.5)) * step)


_ROT: Dict[Tuple[int, int], np.ndarray] = {}


def rotation(d: int, seed: int) -> np.ndarray:
    """turboquant_utils/rotation.py:53: CPU generator -> randn -> QR -> sign fix, fp32."""
    seed = int(seed)
    key = (d, seed)
    if key not in _ROT:
        gen = torch.Generator().manual_seed(seed)
        q, r = torch.linalg.qr(torch.randn(d, d, generator=gen))
        _ROT[key] = (q * torch.sign(torch.diag(r)).unsqueeze(0)).numpy().copy()
        if len(_ROT) > 16384:
            _ROT.pop(next(iter(_ROT)))
    return _ROT[key]


def rotation_stack_f16(seed_base: int, groups: int) -> np.ndarray:
    """turboquant_utils/rotation.py:127: (groups, 128, 128) fp16, seed = base + g*128."""
    return np.stack([rotation(GS, seed_base + g * GS).astype(np.float16) for g in range(groups)])


def quantize_packed(W: np.ndarray, bit: int, seed: int, uniform: bool = False) -> dict:
    """turboquant_utils/quantize.py:350-472 with group_size 128 (fp32 torch math, as the reference)."""
    Wt = torch.as_tensor(np.asarray(W, np.float32))
    n, k = Wt.shape
    cent, edges = uniform8() if uniform else lloyd_max(bit)
    edges_t = torch.from_numpy(edges)
    idx, norms = [], []
    for g0 in range(0, k, GS):
        wg = Wt[:, g0:g0 + GS]
        nrm = wg.norm(dim=1, keepdim=True).clamp(min=1e-8)
        y = ((wg / nrm) @ torch.from_numpy(rotation(GS, seed + g0)).T) * math.sqrt(GS)
        cell = torch.searchsorted(edges_t, y.reshape(-1)).clamp(0, len(cent) - 1)
        idx.append(cell.reshape(n, GS).numpy().astype(np.uint8))
        norms.append(nrm.squeeze(1).numpy())
    return {"indices_packed": pack_nbit(np.concatenate(idx, 1), bit),
            "codebook": cent.astype(np.float16), "norms": np.stack(norms, 1).astype(np.float16),
            "seed": seed, "bit_width": bit, "shape": (n, k), "group_size": GS}


def dequantize_packed(pk: dict) -> np.ndarray:
    """turboquant_utils/quantize.py:478-557: fp32 matrix (before the cast to the original dtype).

    Uses the same torch CPU operations as the reference (unpack by shifts, codebook gather, one
    (N,128)x(128,128) matmul per group), so its run time is representative of the reference's.
    """
    n, k = pk["shape"]
    bit = pk["bit_width"]
    per = 8 // bit
    cb = torch.from_numpy(np.asarray(pk["codebook"], np.float32))
    norms = torch.from_numpy(np.asarray(pk["norms"], np.float32).reshape(n, -1))
    packed = torch.from_numpy(np.ascontiguousarray(pk["indices_packed"]))
    idx = torch.zeros(n, packed.shape[1] * per, dtype=torch.int32)
    for j in range(per):
        idx[:, j::per] = ((packed >> (j * bit)) & ((1 << bit) - 1)).to(torch.int32)
    idx = idx[:, :k]
    out = torch.zeros(n, k, dtype=torch.float32)
    for g, g0 in enumerate(range(0, k, GS)):
        y = cb[idx[:, g0:g0 + GS]] / math.sqrt(GS)
        out[:, g0:g0 + GS] = (y @ torch.from_numpy(rotation(GS, pk["seed"] + g0))) * norms[:, g:g + 1]
    return out.numpy()


# =========================================================================== activation-mode LUTs

def int8_lut(codebook_f16: np.ndarray) -> Tuple[np.ndarray, float]:
    """turboquant_utils/triton_kernels_a8.py:526-553."""
    cb = torch.as_tensor(np.asarray(codebook_f16, np.float16)).float()
    step = (cb.abs().max() / 127.0).item()
    return (cb / step).round().clamp_(-127, 127).to(torch.int8).numpy(), step


def _to_e4m3_bytes(v: torch.Tensor) -> torch.Tensor:
    """fp32 -> e4m3 bytes, round-to-nearest-even, saturating at +-448."""
    return v.clamp(-448.0, 448.0).to(torch.float8_e4m3fn).view(torch.uint8)


def e4m3_to_f32(b: np.ndarray) -> np.ndarray:
    return torch.from_numpy(np.ascontiguousarray(b, np.uint8)).view(torch.float8_e4m3fn).float().numpy()


def fp8_lut(codebook_f16: np.ndarray, n_coarse: int = 512) -> Tuple[np.ndarray, float]:
    """turboquant_utils/triton_kernels_fp8.py:35-88: scale search, same candidate arithmetic."""
    cb = torch.as_tensor(np.asarray(codebook_f16, np.float16)).float()
    top = cb.abs().max()

    def lut_at(s):
        return (cb / s).clamp_(-448.0, 448.0).to(torch.float8_e4m3fn)

    def err(s):
        return ((lut_at(s).float() * s - cb).norm() / cb.norm()).item()

    s0 = (top / 448.0).item()
    mid = torch.log10(torch.tensor(s0))
    coarse = torch.logspace(mid - 1.0, mid + 1.0, n_coarse).tolist()
    best_s, best = s0, float("inf")
    for s in coarse:
        e = err(s)
        if e < best:
            best_s, best = s, e
    span = coarse[1] / coarse[0]
    for ratio in (span ** 0.5, span ** 0.25):
        for s in [best_s * ratio ** (i / 64.0 - 0.5) for i in range(64)]:
            e = err(s)
            if e < best:
                best_s, best = s, e
    return lut_at(best_s).view(torch.uint8).numpy(), best_s


def e2m1_lut(codebook_f16: np.ndarray):
    """turboquant_utils/triton_kernels_fp4.py:32-77: (nibble LUT, E0, residual)."""
    cb = torch.as_tensor(np.asarray(codebook_f16, np.float16)).float()
    grid = torch.tensor(E2M1_VALUES)

    def fit(s):
        y = (cb / s).clamp(-6.0, 6.0)
        mag = torch.argmin((y.abs().unsqueeze(-1) - grid).abs(), dim=-1)
        nib = ((mag & 7) | ((y < 0).long() << 3)).to(torch.uint8)
        rec = grid[mag] * y.sign() * s
        return nib, ((rec - cb).norm() / cb.norm()).item()

    s0 = cb.abs().max() / 6.0
    best_s, best, lut = s0, float("inf"), None
    for s in [s0 * (2.0 ** (i / 16.0)) for i in range(-16, 17)]:
        nib, e = fit(s)
        if e < best:
            best_s, best, lut = s, e, nib
    for _ in range(2):
        span = 2.0 ** (1 / 16)
        lo, hi = best_s / span, best_s * span
        for s in [lo * (hi / lo) ** (i / 64.0) for i in range(65)]:
            nib, e = fit(s)
            if e < best:
                best_s, best, lut = s, e, nib
    e0 = math.floor(math.log2(best_s))
    return lut.numpy(), e0, float(best_s / (2.0 ** e0))


def fold_e2m1(indices_gf: np.ndarray, nib: np.ndarray, bit: int) -> np.ndarray:
    """turboquant_utils/triton_kernels_fp4.py:80-127: (G, N, bpg) indices -> (G, N, 64) packed e2m1."""
    g, n, _ = indices_gf.shape
    idx = unpack_nbit(indices_gf.reshape(g * n, -1), bit, GS)
    nb = np.asarray(nib, np.uint8)[idx]
    return (nb[:, 0::2] | (nb[:, 1::2] << 4)).astype(np.uint8).reshape(g, n, GS // 2)


def e2m1_to_f32(nib: np.ndarray) -> np.ndarray:
    nib = np.asarray(nib, np.uint8)
    return E2M1_VALUES[nib & 7] * np.where(nib & 8, np.float32(-1), np.float32(1))


# =========================================================================== rotation + activation quantisation

def to_f16_values(x: torch.Tensor) -> np.ndarray:
    """x.half() of the reference (quantization/wxa8/bit_partitioned_moe.py:109), as fp32 numpy values."""
    return x.detach().cpu().to(torch.float16).float().numpy()


def rotate_f32(x_f16vals: np.ndarray, rot_f16: np.ndarray) -> np.ndarray:
    """acc[b, g*128+j] = sum_k x[b, g*128+k] * P_g[j, k], sequentially over k in fp32.

    Products of two fp16 values are exact in fp32, so ``acc + x*p`` equals the fused multiply-add
    the GPU performs.  (Reference: tl.dot(x_tile, P^T, out fp32), triton_kernels_a8.py:466-471.)
    """
    b, k = x_f16vals.shape
    g = k // GS
    x = x_f16vals.reshape(b, g, GS).astype(np.float32)
    p = rot_f16.astype(np.float32)               # (g, j, k)
    acc = np.zeros((b, g, GS), np.float32)
    for kk in range(GS):
        acc = acc + x[:, :, kk:kk + 1] * p[None, :, :, kk]
    return acc.reshape(b, k)


def _round_half_away(v: np.ndarray) -> np.ndarray:
    """roundf(): nearest integer, ties away from zero, without the |v|+0.5 double rounding."""
    t = np.trunc(v)
    return t + np.where(np.abs(v - t) >= np.float32(0.5), np.sign(v), 0).astype(v.dtype)


def actquant_int8(acc: np.ndarray, extra_scale: float):
    """triton_kernels_a8.py:473-484: (int8 codes (B,K), fp16 scales (B,G))."""
    b, k = acc.shape
    a = acc.reshape(b, k // GS, GS)
    amax = np.abs(a).max(-1)
    s = np.where(amax < np.float32(1e-8 * 127.0), np.float32(1e-8), amax / np.float32(127.0)).astype(np.float32)
    q = np.clip(_round_half_away((a / s[..., None]).astype(np.float32)), -127, 127).astype(np.int8)
    return q.reshape(b, k), (s * np.float32(extra_scale)).astype(np.float16)


def actquant_e4m3(acc: np.ndarray, extra_scale: float):
    """triton_kernels_fp8.py:176-187: (e4m3 bytes (B,K), fp16 scales (B,G))."""
    b, k = acc.shape
    a = acc.reshape(b, k // GS, GS)
    amax = np.abs(a).max(-1)
    s = np.where(amax < np.float32(1e-8 * 448.0), np.float32(1e-8), amax / np.float32(448.0)).astype(np.float32)
    q = _to_e4m3_bytes(torch.from_numpy((a / s[..., None]).astype(np.float32))).numpy()
    return q.reshape(b, k), (s * np.float32(extra_scale)).astype(np.float16)


def actquant_e2m1(acc: np.ndarray):
    """triton_kernels_fp4.py:1073-1104: (packed (B,K/2) even k low nibble, e8m0 bytes (B,K/32))."""
    b, k = acc.shape
    a = acc.reshape(b, k // 32, 32)
    amax = np.maximum(np.abs(a).max(-1), np.float32(1e-30))
    e = np.ceil(np.log2((amax / np.float32(6.0)).astype(np.float64)).astype(np.float32))
    e = np.clip(e, -127.0, 127.0).astype(np.float32)
    y = np.clip(np.ldexp(a, -e.astype(np.int32)[..., None]).astype(np.float32), -6.0, 6.0)
    ay = np.abs(y)
    mag = np.select([ay < 0.25, ay < 0.75, ay < 1.25, ay < 1.75, ay < 2.5, ay < 3.5, ay < 5.0],
                    [0, 1, 2, 3, 4, 5, 6], 7).astype(np.uint8)
    nib = (mag | ((y < 0).astype(np.uint8) << 3)).reshape(b, k)
    return (nib[:, 0::2] | (nib[:, 1::2] << 4)).astype(np.uint8), (e + 127.0).astype(np.int32).astype(np.uint8)


def unpack_e2m1(packed: np.ndarray) -> np.ndarray:
    p = np.asarray(packed, np.uint8)
    nib = np.stack([p & 15, p >> 4], -1).reshape(p.shape[0], -1)
    return e2m1_to_f32(nib)


# =========================================================================== GEMM stages

def _half(v: np.ndarray) -> np.ndarray:
    return np.asarray(v, np.float32).astype(np.float16)


def weight_codes(indices_gf: np.ndarray, bit: int, rows: slice, groups: slice) -> np.ndarray:
    """Unpacked codebook indices (G_sel, N_sel, 128) of a slice of a group-first tensor."""
    sub = indices_gf[groups, rows]
    g, n, _ = sub.shape
    return unpack_nbit(sub.reshape(g * n, -1), bit, GS).reshape(g, n, GS)


def gemm_int8(x_i8: np.ndarray, xs_f16: np.ndarray, w_i8: np.ndarray, norm_f16: np.ndarray):
    """triton_kernels_a8.py:893-929.  x_i8 (B, G*128), w_i8 (G, N, 128), norm (G, N).

    Returns (fp16 output (B, N), int32 partial sums (B, N, G)); the fp32 total adds
    ((float(acc)*xs)*norm) group by group, unfused.
    """
    b = x_i8.shape[0]
    g, n, _ = w_i8.shape
    # integer group sums through fp32 matrix products: every product and every partial sum is an integer of
    # magnitude <= 128*127*127 < 2^24, so fp32 arithmetic is exact whatever the summation order
    xg = x_i8.reshape(b, g, GS).astype(np.float32)
    part = np.empty((b, n, g), np.int32)
    for gi in range(g):
        part[:, :, gi] = (xg[:, gi] @ w_i8[gi].astype(np.float32).T).astype(np.int32)
    total = np.zeros((b, n), np.float32)
    xs = xs_f16.astype(np.float32)
    nm = norm_f16.astype(np.float32)
    for gi in range(g):
        total = total + (part[:, :, gi].astype(np.float32) * xs[:, gi:gi + 1]) * nm[gi][None, :]
    return _half(total), part


def gemm_scaled_f32(x_vals: np.ndarray, row_scale: Optional[np.ndarray], w_vals: np.ndarray, norm_f16: np.ndarray,
                    block: int = GS) -> np.ndarray:
    """fp32 dot per scale block, then (acc*row_scale)*norm accumulated in block order -> fp16.

    FP8 (triton_kernels_fp8.py:589-626): block 128, row_scale = xs[b, g].
    FP4 (triton_kernels_fp4.py:664-731): block 32, row_scale = 2^(a_e8m0-127+E0) per (b, 32-block).
    A16 (triton_kernels.py:1430-1473): row_scale None (the reference accumulates in fp16; this
    restatement keeps fp32 and rounds once, which is inside the path's 1e-2 tolerance).
    """
    b = x_vals.shape[0]
    g, n, _ = w_vals.shape
    nb = GS // block
    x = x_vals.reshape(b, g, nb, block).astype(np.float32)
    w = w_vals.reshape(g, n, nb, block).astype(np.float32)
    nm = norm_f16.astype(np.float32)
    total = np.zeros((b, n), np.float32)
    for gi in range(g):
        for bi in range(nb):
            acc = x[:, gi, bi] @ w[gi, :, bi].T
            if row_scale is not None:
                acc = acc * row_scale[:, gi * nb + bi][:, None]
            total = total + acc * nm[gi][None, :]
    return _half(total)


def silu_mul_f16(gu_f16: np.ndarray, inter: int) -> np.ndarray:
    """F.silu(gate) * up on fp16 tensors (quantization/wxa8/bit_partitioned_moe.py:336-341)."""
    t = torch.from_numpy(np.ascontiguousarray(gu_f16))
    return (torch.nn.functional.silu(t[:, :inter]) * t[:, inter:]).numpy()


# =========================================================================== whole layer

class Layer:
    """A synthetic or loaded layer in plain numpy form.

    pools: list of dicts {bit, mode, members [expert ids], inter, gu: packed dict, dn: packed dict}
    shared: optional pool-like dict with one member (gate rows then up rows in ``gu``).
    """

    def __init__(self, hidden: int, n_experts: int, top_k: int, pools: List[dict], shared: Optional[dict] = None):
        self.hidden, self.n_experts, self.top_k = hidden, n_experts, top_k
        self.pools, self.shared = pools, shared
        for p in pools + ([shared] if shared else []):
            self._prepare(p)

    @staticmethod
    def _prepare(p: dict) -> None:
        bit = p["bit"]
        for side in ("gu", "dn"):
            pk = p[side]
            idx_gf, norm_gf = group_first(np.asarray(pk["indices_packed"]), np.asarray(pk["norms"]), bit)
            pk["idx_gf"] = idx_gf
            # norms_gf / sqrt(128) in fp16 (quantization/wxa16/bit_partitioned_moe.py:203)
            pk["norm_gf"] = (norm_gf.astype(np.float32) / np.float32(math.sqrt(GS))).astype(np.float16)


def warm_rotations(layer: "Layer") -> None:
    """Fill the rotation cache for every group of every pool (the reference caches them too, rotation.py:33-41)."""
    for p in layer.pools + ([layer.shared] if layer.shared else []):
        for side in ("gu", "dn"):
            k = p[side]["shape"][1]
            for g0 in range(0, k, GS):
                rotation(GS, p[side]["seed"] + g0)


def sort_rows(topk_idx: np.ndarray, topk_w: np.ndarray, n_experts: int):
    """quantization/wxa16/bit_partitioned_moe.py:1125-1138, stable in token order."""
    flat_e = topk_idx.reshape(-1)
    order = np.argsort(flat_e, kind="stable")
    tokens = (np.arange(flat_e.size) // topk_idx.shape[1])[order]
    counts = np.bincount(flat_e, minlength=n_experts)
    starts = np.concatenate([[0], np.cumsum(counts)])
    return tokens.astype(np.int32), topk_w.reshape(-1)[order].astype(np.float32), starts.astype(np.int64), order


def _mode_consts(mode: str, bit: int, codebook_f16: np.ndarray):
    """(weight value table used by the GEMM, act extra scale, E0, norm factor) per activation mode."""
    if mode == "wxa16":
        return np.asarray(codebook_f16, np.float16).astype(np.float32), 1.0, 0, 1.0
    if mode == "wxa8":
        if bit == 8:
            cb = np.asarray(codebook_f16, np.float32)
            return (np.arange(256) - 128).astype(np.int8), float((cb[-1] - cb[0]) / np.float32(255.0)), 0, 1.0
        lut, step = int8_lut(codebook_f16)
        return lut, step, 0, 1.0
    if mode == "wxfp8":
        lut, scale = fp8_lut(codebook_f16)
        return e4m3_to_f32(lut), scale, 0, 1.0
    if mode == "wxfp4":
        nib, e0, resid = e2m1_lut(codebook_f16)
        return e2m1_to_f32(nib), 1.0, e0, resid
    raise ValueError(mode)


def _quant_act(mode: str, acc: np.ndarray, extra: float, e0: int):
    """Returns (values fed to the GEMM, row scales or None, block, raw codes, raw scales)."""
    if mode == "wxa16":
        v = _half(acc)
        return v.astype(np.float32), None, GS, v, None
    if mode == "wxa8":
        q, s = actquant_int8(acc, extra)
        return q, s, GS, q, s
    if mode == "wxfp8":
        q, s = actquant_e4m3(acc, extra)
        return e4m3_to_f32(q), s.astype(np.float32), GS, q, s
    if mode == "wxfp4":
        q, s = actquant_e2m1(acc)
        rs = np.ldexp(np.float32(1.0), s.astype(np.int32) - 127 + e0).astype(np.float32)
        return unpack_e2m1(q), rs, 32, q, s
    raise ValueError(mode)


def _pool_gemm(mode, vals, rs, block, w_idx, table, norm):
    if mode == "wxa8":
        return gemm_int8(vals, rs, table[w_idx], norm)
    return gemm_scaled_f32(vals, rs, table[w_idx], norm, block), None


def moe_forward(layer: Layer, x: torch.Tensor, topk_w: np.ndarray, topk_idx: np.ndarray,
                shared_w: Optional[np.ndarray] = None, keep: bool = False) -> dict:
    """The merged-path forward of the reference modules, stage by stage.

    quantization/wxa16/bit_partitioned_moe.py:856-979 (A16), wxa8/...:283-385 (A8),
    wxfp8/... (FP8), wxfp4/...:288-396 (FP4; pools whose mode is "wxa8" run as int8).
    Returns ``y`` (T, H) fp32 = fp32 sum of the bf16 row contributions (the reference adds them
    in bf16 in an order the GPU does not fix), ``y_bf16seq`` = the same contributions added
    sequentially in bf16, plus the per-stage intermediates when ``keep`` is set.
    """
    T, H = x.shape
    xv = to_f16_values(x)
    tokens, weights, starts, _ = sort_rows(np.asarray(topk_idx), np.asarray(topk_w, np.float32), layer.n_experts)
    y32 = np.zeros((T, H), np.float32)
    yb = torch.zeros(T, H, dtype=torch.bfloat16)
    stages: dict = {}
    pools = list(layer.pools)
    if layer.shared is not None:
        pools.append(layer.shared)
    for p in pools:
        mode, bit, inter = p["mode"], p["bit"], p["inter"]
        shared = p is layer.shared
        if shared:
            rows_tok = np.arange(T, dtype=np.int32)
            rows_w = (np.ones(T, np.float32) if shared_w is None else np.asarray(shared_w, np.float32))
            seg = [(0, 0, T)]
        else:
            seg, tok_l, w_l, cur = [], [], [], 0
            for rank, e in enumerate(p["members"]):
                n = int(starts[e + 1] - starts[e])
                if n:
                    seg.append((rank, cur, n))
                    tok_l.append(tokens[starts[e]:starts[e + 1]])
                    w_l.append(weights[starts[e]:starts[e + 1]])
                    cur += n
            if not seg:
                continue
            rows_tok, rows_w = np.concatenate(tok_l), np.concatenate(w_l)
        gu, dn = p["gu"], p["dn"]
        tab_g, ex_g, e0_g, f_g = _mode_consts(mode, bit, gu["codebook"])
        tab_d, ex_d, e0_d, f_d = _mode_consts(mode, bit, dn["codebook"])
        norm_g = gu["norm_gf"] if f_g == 1.0 else (gu["norm_gf"].astype(np.float32) * np.float32(f_g)).astype(np.float16)
        norm_d = dn["norm_gf"] if f_d == 1.0 else (dn["norm_gf"].astype(np.float32) * np.float32(f_d)).astype(np.float16)
        G_h, G_i = H // GS, inter // GS
        acc = rotate_f32(xv[rows_tok], rotation_stack_f16(gu["seed"], G_h))
        vals, rs, block, codes, scales = _quant_act(mode, acc, ex_g, e0_g)
        n_rows = rows_tok.size
        gu_out = np.zeros((n_rows, 2 * inter), np.float16)
        parts_g = np.zeros((n_rows, 2 * inter, G_h), np.int32) if (mode == "wxa8" and keep) else None
        for rank, r0, n in seg:
            w_idx = weight_codes(gu["idx_gf"], bit, slice(2 * inter * rank, 2 * inter * (rank + 1)), slice(0, G_h))
            o, pt = _pool_gemm(mode, vals[r0:r0 + n], None if rs is None else rs[r0:r0 + n], block, w_idx, tab_g,
                               norm_g[:, 2 * inter * rank:2 * inter * (rank + 1)])
            gu_out[r0:r0 + n] = o
            if parts_g is not None:
                parts_g[r0:r0 + n] = pt
        act = silu_mul_f16(gu_out, inter)
        dn_out = np.zeros((n_rows, H), np.float16)
        parts_d = np.zeros((n_rows, H, G_i), np.int32) if (mode == "wxa8" and keep) else None
        d_codes, d_scales = [], []
        for rank, r0, n in seg:
            rot = rotation_stack_f16(dn["seed"] + rank * inter, G_i)
            acc_d = rotate_f32(act[r0:r0 + n].astype(np.float32), rot)
            v2, rs2, blk2, c2, s2 = _quant_act(mode, acc_d, ex_d, e0_d)
            d_codes.append(c2)
            d_scales.append(s2)
            w_idx = weight_codes(dn["idx_gf"], bit, slice(0, H), slice(rank * G_i, (rank + 1) * G_i))
            o, pt = _pool_gemm(mode, v2, rs2, blk2, w_idx, tab_d, norm_d[rank * G_i:(rank + 1) * G_i])
            dn_out[r0:r0 + n] = o
            if parts_d is not None:
                parts_d[r0:r0 + n] = pt
        # dn.to(bf16); dn.mul_(w); final.index_add_(0, tokens, dn)   (wxa16/...:960-967)
        contrib = torch.from_numpy(dn_out).to(torch.bfloat16)
        contrib = (contrib.float() * torch.from_numpy(rows_w).unsqueeze(1)).to(torch.bfloat16)
        np.add.at(y32, rows_tok, contrib.float().numpy())
        yb.index_add_(0, torch.from_numpy(rows_tok.astype(np.int64)), contrib)
        if keep:
            stages[p.get("key", str(bit))] = dict(
                rows_tok=rows_tok, rows_w=rows_w, seg=seg, codes=codes, scales=scales, gu=gu_out,
                parts_gu=parts_g, act=act, dn_codes=d_codes, dn_scales=d_scales, dn=dn_out, parts_dn=parts_d,
                contrib=contrib.float().numpy())
    return {"y": y32, "y_bf16seq": yb.float().numpy(), "stages": stages}


def dequant_matmul_forward(layer: Layer, x: torch.Tensor, topk_w: np.ndarray, topk_idx: np.ndarray,
                           shared_w: Optional[np.ndarray] = None, dtype=torch.float32,
                           weight_cache: Optional[dict] = None) -> np.ndarray:
    """The reference's dequantize-then-matmul path (turboquant_utils/test_triton_mp_moe_e2e_bench.py:167-272):
    per ACTIVE expert, dequantise its gate_up rows / down columns, x @ W^T, silu*up, @ W_down^T, weight, scatter-add.
    ``dtype`` float16 reproduces the reference's arithmetic type; float32 is the "ideal" answer."""
    T, H = x.shape
    xt = x.detach().cpu().to(dtype)
    tokens, weights, starts, _ = sort_rows(np.asarray(topk_idx), np.asarray(topk_w, np.float32), layer.n_experts)
    y = torch.zeros(T, H, dtype=dtype)

    def expert_weights(p, rank):
        """(gate_up rows, down columns) of one member, dequantised on their own as the reference does per expert and
        bit (turboquant_dequantize_packed_rows / _cols, test_triton_mp_moe_e2e_bench.py:214-238)."""
        key = (id(p), rank)
        if weight_cache is not None and key in weight_cache:
            return weight_cache[key]
        inter, bit = p["inter"], p["bit"]
        gu, dn = p["gu"], p["dn"]
        r0, r1 = 2 * inter * rank, 2 * inter * (rank + 1)
        rows = dict(gu, indices_packed=np.asarray(gu["indices_packed"])[r0:r1], norms=np.asarray(gu["norms"])[r0:r1],
                    shape=(r1 - r0, gu["shape"][1]))
        c0, c1 = inter * rank, inter * (rank + 1)
        cols = dict(dn, indices_packed=np.asarray(dn["indices_packed"])[:, c0 * bit // 8:c1 * bit // 8],
                    norms=np.asarray(dn["norms"])[:, c0 // GS:c1 // GS], shape=(dn["shape"][0], inter),
                    seed=int(dn["seed"]) + c0)
        w = (torch.from_numpy(dequantize_packed(rows)).to(torch.float16).to(dtype),
             torch.from_numpy(dequantize_packed(cols)).to(torch.float16).to(dtype))
        if weight_cache is not None:
            weight_cache[key] = w
        return w

    pools = list(layer.pools) + ([layer.shared] if layer.shared is not None else [])
    for p in pools:
        inter = p["inter"]
        if p is layer.shared:
            members = [(0, np.arange(T), np.ones(T, np.float32) if shared_w is None else np.asarray(shared_w, np.float32))]
        else:
            members = [(rank, tokens[starts[e]:starts[e + 1]], weights[starts[e]:starts[e + 1]])
                       for rank, e in enumerate(p["members"]) if starts[e + 1] > starts[e]]
        for rank, tok, w in members:
            w_gu, w_dn = expert_weights(p, rank)
            xe = xt[torch.from_numpy(tok.astype(np.int64))]
            gu = xe @ w_gu.T
            act = torch.nn.functional.silu(gu[:, :inter]) * gu[:, inter:]
            out = act @ w_dn.T
            out = out * torch.from_numpy(np.asarray(w, np.float32)).to(dtype).unsqueeze(1)
            y.index_add_(0, torch.from_numpy(tok.astype(np.int64)), out)
    return y.float().numpy()
