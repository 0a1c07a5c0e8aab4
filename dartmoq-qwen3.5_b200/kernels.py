"""Function-level operators with the reference wrappers' names and argument meaning.

Each function takes torch CUDA tensors, builds the plain structs of the C ABI
and launches libdmoq kernels on the current stream.  They exist so the stages
of the layer can be driven and checked one at a time, the way the reference
exposes them:

  rotate_quantize_fused            turboquant_utils/triton_kernels_a8.py:487
  rotate_quantize_fused_fp8        turboquant_utils/triton_kernels_fp8.py:190
  rotate_quantize_fused_fp4        turboquant_utils/triton_kernels_fp4.py:1107
  batch_rotate_input               turboquant_utils/rotation.py:176
  *_matmul_merged_rows_gf          triton_kernels.py:1482, _a8.py:959, _fp8.py:641, _fp4.py:740
  *_matmul_merged_in_features_gf   triton_kernels.py:1554, _a8.py:1017, _fp8.py:699, _fp4.py:811
  convert_to_group_first           turboquant_utils/triton_kernels.py:1042

Errors follow the reference: ``ValueError`` for a bad bit width or a K that is
not a multiple of the group size.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Optional, Sequence, Tuple

import torch

from . import _lib
from . import format as fmt
from ._lib import A16, A8, FP8, FP4, EPI_PLAIN, EPI_SILU, EPI_WEIGHTED, MAX_POOLS, TILE_M, Pool, Route, check, ptr

GROUP = fmt.GROUP_SIZE
# None: the function-level GEMMs build a weight image (dmoq_expand_weights) for e2m1 pools only, as the module does
# at load time; True / False force it for every mode / for none
USE_WEIGHT_IMAGES = None


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _need_cuda(t: torch.Tensor) -> None:
    if not t.is_cuda:
        raise _lib.DmoqError("libdmoq operators take CUDA tensors only (no CPU path)")


def _on_tensor_device(fn):
    """Run ``fn`` with the device of its first tensor argument current, so that the stream handed to the
    library and every allocation belong to that device whichever one the caller has selected; all tensor
    arguments must live there."""
    import functools

    @functools.wraps(fn)
    def wrapper(*args, **kwargs):
        tensors = [a for a in list(args) + list(kwargs.values()) if isinstance(a, torch.Tensor)]
        if not tensors or not tensors[0].is_cuda:
            return fn(*args, **kwargs)
        dev = tensors[0].device
        for t in tensors:
            if t.is_cuda and t.device != dev:
                raise ValueError(f"all tensors must be on {dev}, got one on {t.device}")
        with torch.cuda.device(dev):
            return fn(*args, **kwargs)
    return wrapper


def _check_rot(x, rot, group_size, num_groups):
    if group_size != GROUP:
        raise ValueError(f"group_size must be {GROUP}, got {group_size}")
    if x.shape[1] != num_groups * group_size:
        raise ValueError(f"K_total ({x.shape[1]}) != num_groups*group_size ({num_groups * group_size})")
    if tuple(rot.shape) != (num_groups, group_size, group_size):
        raise ValueError(f"rot must have shape {(num_groups, group_size, group_size)}, got {tuple(rot.shape)}")
    if x.dtype not in (torch.float16, torch.bfloat16):
        raise TypeError(f"x must be fp16 or bf16, got {x.dtype}")


@_on_tensor_device
def _rotate(mode: int, x: torch.Tensor, rot: torch.Tensor, extra_scale: float, codes, scales,
            src_row: Optional[torch.Tensor] = None, n_rows: Optional[int] = None) -> None:
    _need_cuda(x)
    lib = _lib.load()
    x = x.contiguous()
    rot = rot.to(torch.float16).contiguous()
    rows = x.shape[0] if n_rows is None else n_rows
    check(lib.dmoq_rotate_quant(mode, ptr(x), int(x.dtype == torch.bfloat16), x.shape[1], ptr(rot), None,
                                ptr(src_row), rows, None, float(extra_scale), ptr(codes), ptr(scales), _stream()),
          "dmoq_rotate_quant")


def rotate_quantize_fused(x: torch.Tensor, rot: torch.Tensor, group_size: int, num_groups: int,
                          extra_scale: float = 1.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """Group rotation + per-token per-group symmetric int8.  Returns (int8 (B, K), fp16 scale (B, G))."""
    _check_rot(x, rot, group_size, num_groups)
    B, K = x.shape
    q = torch.empty((B, K), dtype=torch.int8, device=x.device)
    s = torch.empty((B, num_groups), dtype=torch.float16, device=x.device)
    if B:
        _rotate(A8, x, rot, extra_scale, q, s)
    return q, s


def rotate_quantize_fused_fp8(x: torch.Tensor, rot: torch.Tensor, group_size: int, num_groups: int,
                              extra_scale: float = 1.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """Group rotation + per-token per-group e4m3 (RTNE, saturating).  Returns (e4m3 (B, K), fp16 scale (B, G))."""
    _check_rot(x, rot, group_size, num_groups)
    B, K = x.shape
    q = torch.empty((B, K), dtype=torch.uint8, device=x.device)
    s = torch.empty((B, num_groups), dtype=torch.float16, device=x.device)
    if B:
        _rotate(FP8, x, rot, extra_scale, q, s)
    return q.view(torch.float8_e4m3fn), s


def rotate_quantize_fused_fp4_rowmajor(x: torch.Tensor, rot: torch.Tensor, group_size: int, num_groups: int):
    """Group rotation + e2m1 / per-32 e8m0.  Returns (packed (B, K/2) even k low nibble, e8m0 (B, K/32))."""
    _check_rot(x, rot, group_size, num_groups)
    B, K = x.shape
    q = torch.empty((B, K // 2), dtype=torch.uint8, device=x.device)
    s = torch.empty((B, K // 32), dtype=torch.uint8, device=x.device)
    if B:
        _rotate(FP4, x, rot, 1.0, q, s)
    return q, s


def rotate_quantize_fused_fp4(x: torch.Tensor, rot: torch.Tensor, group_size: int, num_groups: int):
    """As the reference: the packed codes are returned transposed, (K/2, B)."""
    q, s = rotate_quantize_fused_fp4_rowmajor(x, rot, group_size, num_groups)
    return q.t().contiguous(), s


def batch_rotate_input(x: torch.Tensor, group_size: int, seed_base: int) -> torch.Tensor:
    """Group rotation only; fp16 output (fp32 accumulation, one rounding)."""
    if x.shape[1] % group_size:
        raise ValueError(f"K ({x.shape[1]}) must be a multiple of group_size ({group_size})")
    G = x.shape[1] // group_size
    rot = fmt.generate_batch_rotation_matrices(group_size, seed_base, G, group_size, x.device, torch.float16)
    _check_rot(x, rot, group_size, G)
    out = torch.empty(x.shape, dtype=torch.float16, device=x.device)
    if x.shape[0]:
        _rotate(A16, x, rot, 1.0, out, None)
    return out


@_on_tensor_device
def convert_to_group_first(indices_packed: torch.Tensor, norms: torch.Tensor, group_size: int, bit_width: int):
    """(N, K*b/8) -> (G, N, gs*b/8) on the device; norms (N, G) -> (G, N)."""
    if bit_width not in fmt.SUPPORTED_BITS:
        raise ValueError(f"bit_width must be 1/2/4/8, got {bit_width}")
    if group_size != GROUP:
        raise ValueError(f"group_size must be {GROUP}, got {group_size}")
    _need_cuda(indices_packed)
    lib = _lib.load()
    src = indices_packed.contiguous()
    n = src.shape[0]
    k = src.shape[1] * 8 // bit_width
    dst = torch.empty((k // GROUP, n, 16 * bit_width), dtype=torch.uint8, device=src.device)
    check(lib.dmoq_convert_group_first(ptr(src), n, k, bit_width, ptr(dst), _stream()), "dmoq_convert_group_first")
    return dst, norms.t().contiguous()


# --------------------------------------------------------------------------- merged GEMMs

class _HostRoute:
    """Routing tables for rows that are already gathered and grouped by expert (``expert_info``)."""

    def __init__(self, expert_info: Sequence[Sequence[int]], ranks: Sequence[int], n_rows: int, device,
                 weights: Optional[torch.Tensor] = None):
        tiles = []
        for e, (start, count, _s0, _sc) in enumerate(expert_info):
            for m in range(0, count, TILE_M):
                tiles.append((e, start + m, min(TILE_M, count - m), int(ranks[e])))
        i32 = dict(dtype=torch.int32, device=device)
        self.tiles = torch.tensor(tiles if tiles else [(0, 0, 0, 0)], **i32).reshape(-1, 4).contiguous()
        self.n_tiles = torch.tensor([len(tiles)] + [0] * (2 * MAX_POOLS - 1), **i32)
        self.rank = torch.tensor(list(ranks) if len(ranks) else [0], **i32)
        self.pool_of = torch.zeros(max(len(ranks), 1), **i32)
        self.weights = (weights.to(torch.float32).contiguous() if weights is not None
                        else torch.ones(max(n_rows, 1), dtype=torch.float32, device=device))
        self.zeros = torch.zeros(MAX_POOLS, **i32)
        r = Route()
        r.T, r.top_k, r.E, r.has_shared = n_rows, 1, max(len(ranks), 1), 0
        r.tile_m, r.n_pools = TILE_M, 1
        r.expert_pool, r.expert_rank = self.pool_of.data_ptr(), self.rank.data_ptr()
        r.sorted_weights = self.weights.data_ptr()   # a_row stays NULL: the callers' rows are already in routed-row order
        r.tiles, r.n_tiles, r.tile_cap = self.tiles.data_ptr(), self.n_tiles.data_ptr(), max(len(tiles), 1)
        r.pool_hoisted = self.zeros.data_ptr()
        self.c = r


@_on_tensor_device
def router_topk(logits: torch.Tensor, top_k: int, renormalize: bool = False, *, x: Optional[torch.Tensor] = None,
                shared_gate: Optional[torch.nn.Module] = None):
    """fp32 softmax over experts -> top-k probabilities (descending) and indices (int64), optionally renormalised:
    the router stage of the module (quantization/wxa16/bit_partitioned_moe.py:1113-1119) as one launch.
    With ``x`` (T, H) and ``shared_gate`` (a 16-bit ``Linear(H, 1)``) the launch also returns
    ``sigmoid(shared_gate(x))`` per token as fp32 (module :1101-1106); see :func:`fusable_shared_gate`."""
    _need_cuda(logits)
    lg = logits.to(torch.float32).contiguous()
    T, E = lg.shape
    w = torch.empty((T, top_k), dtype=torch.float32, device=lg.device)
    idx = torch.empty((T, top_k), dtype=torch.int64, device=lg.device)
    if shared_gate is None:
        check(_lib.load().dmoq_router_topk(ptr(lg), T, E, top_k, int(renormalize), ptr(w), ptr(idx), _stream()),
              "dmoq_router_topk")
        return w, idx
    sw = torch.empty((T,), dtype=torch.float32, device=lg.device)
    bias = float(shared_gate.bias.float().item()) if shared_gate.bias is not None else 0.0
    check(_lib.load().dmoq_router_topk_gate(ptr(lg), T, E, top_k, int(renormalize), ptr(w), ptr(idx), ptr(x),
                                            int(x.dtype == torch.bfloat16), x.shape[-1], ptr(shared_gate.weight), bias,
                                            ptr(sw), _stream()), "dmoq_router_topk_gate")
    return w, idx, sw


def fusable_shared_gate(gate, x: torch.Tensor) -> bool:
    """True when ``sigmoid(gate(x))`` can ride in the router launch: a bias-free ``Linear(H, 1)`` whose weight has
    the activations' 16-bit type and device, rows of x contiguous and 16-byte aligned."""
    w = getattr(gate, "weight", None)
    return (isinstance(gate, torch.nn.Linear) and gate.out_features == 1 and gate.bias is None and w is not None
            and x.dim() == 2 and x.is_cuda and x.dtype in (torch.bfloat16, torch.float16) and w.dtype == x.dtype
            and w.device == x.device and w.is_contiguous() and x.is_contiguous() and x.shape[1] % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


@_on_tensor_device
def _merged(mode: int, is_down: bool, a_codes: torch.Tensor, a_scales: Optional[torch.Tensor], a_stride: int,
            indices_gf: torch.Tensor, lut: torch.Tensor, norms_gf: torch.Tensor, expert_info, group_size: int,
            bit_width: int, norms_prescaled: bool, *, e0: int = 0, identity: bool = False,
            epilogue: int = EPI_PLAIN, weights: Optional[torch.Tensor] = None,
            partials: Optional[torch.Tensor] = None, out_dtype=torch.float16) -> torch.Tensor:
    if bit_width not in fmt.SUPPORTED_BITS:
        raise ValueError(f"bit_width must be 1/2/4/8, got {bit_width}")
    if group_size != GROUP:
        raise ValueError(f"group_size must be {GROUP}, got {group_size}")
    _need_cuda(a_codes)
    lib = _lib.load()
    info = [tuple(int(v) for v in row) for row in expert_info]
    if not info:
        raise ValueError("merged kernel: empty expert_info (no active experts)")
    widths = {row[3] for row in info}
    if len(widths) != 1:
        raise ValueError(f"merged kernel needs one slice size per pool, got {sorted(widths)}")
    n_rows = a_codes.shape[0]
    dev = a_codes.device
    norms = norms_gf if norms_prescaled else (norms_gf.float() / torch.full((1,), math.sqrt(group_size), device=dev)).half()
    norms = norms.to(torch.float16).contiguous()
    indices_gf = indices_gf.contiguous()
    if is_down:
        g_cnt = widths.pop()
        inter, hidden = g_cnt * GROUP, norms.shape[1]
        ranks = [row[2] // g_cnt for row in info]
        n_members = indices_gf.shape[0] // g_cnt
        n_out = hidden
    else:
        two_i = widths.pop()
        inter, hidden = two_i // 2, indices_gf.shape[0] * GROUP
        ranks = [row[2] // two_i for row in info]
        n_members = indices_gf.shape[1] // two_i
        n_out = two_i if epilogue != EPI_SILU else inter
    if inter % GROUP or hidden % GROUP:
        raise ValueError("slice sizes must be multiples of the group size")
    route = _HostRoute(info, ranks, n_rows, dev, weights)
    pool = (Pool * 1)()
    p = pool[0]
    p.bit, p.mode, p.n_members, p.inter, p.hoisted = bit_width, mode, n_members, inter, 0
    if is_down:
        p.dn_idx, p.dn_norm, p.dn_lut, p.dn_e0 = indices_gf.data_ptr(), norms.data_ptr(), lut.data_ptr(), e0
    else:
        p.gu_idx, p.gu_norm, p.gu_lut, p.gu_e0 = indices_gf.data_ptr(), norms.data_ptr(), lut.data_ptr(), e0
    p.identity_lut = int(identity)
    wide = None
    if bit_width <= 2 and mode in (A16, A8, FP8):   # the tensor-core kernel reads these codes widened to 4-bit fields
        wide = torch.empty(indices_gf.shape[:2] + (64,), dtype=torch.uint8, device=dev)
        check(lib.dmoq_widen_indices(ptr(indices_gf), indices_gf.numel(), bit_width, ptr(wide), _stream()),
              "dmoq_widen_indices")
        if is_down:
            p.dn_idx_wide = wide.data_ptr()
        else:
            p.gu_idx_wide = wide.data_ptr()
    use_img = (mode == FP4) if USE_WEIGHT_IMAGES is None else bool(USE_WEIGHT_IMAGES)
    if use_img and not (mode == FP4 and bit_width == 8):
        side = int(is_down)
        img = torch.empty(max(int(lib.dmoq_weight_image_bytes(C.byref(p), side, hidden)), 16), dtype=torch.uint8, device=dev)
        g_cnt_img = (n_members * inter // GROUP) if is_down else hidden // GROUP
        nimg = torch.empty((g_cnt_img, hidden if is_down else n_members * 2 * inter), dtype=torch.float32, device=dev)
        check(lib.dmoq_expand_weights(C.byref(p), side, hidden, ptr(img), ptr(nimg), _stream()), "dmoq_expand_weights")
        if is_down:
            p.dn_img, p.dn_norm_img = img.data_ptr(), nimg.data_ptr()
        else:
            p.gu_img, p.gu_norm_img = img.data_ptr(), nimg.data_ptr()
    out = torch.empty((n_rows, n_out), dtype=out_dtype, device=dev)
    check(lib.dmoq_grouped_gemm(C.byref(route.c), pool, 0, int(is_down), epilogue, hidden,
                                ptr(a_codes), ptr(a_scales), a_stride, ptr(out), n_out, ptr(partials), _stream()),
          "dmoq_grouped_gemm")
    return out


def triton_fused_matmul_merged_rows_gf(x_rot, indices_packed_gf, codebook, norms_gf, expert_info, group_size,
                                       in_features, bit_width: int = 4, norms_prescaled: bool = False, **kw):
    """A16 gate_up over one pool: (B_total, 2*inter), dtype of ``x_rot`` (name kept from the reference)."""
    if in_features % group_size:
        raise ValueError(f"in_features ({in_features}) must be a multiple of group_size ({group_size})")
    a = x_rot.to(torch.float16).contiguous()
    out = _merged(A16, False, a, None, in_features, indices_packed_gf, codebook.to(torch.float16).contiguous(),
                  norms_gf, expert_info, group_size, bit_width, norms_prescaled, **kw)
    return out.to(x_rot.dtype)


def triton_fused_matmul_merged_in_features_gf(x_rot, indices_packed_gf, codebook, norms_gf, expert_info, group_size,
                                              bit_width: int = 4, norms_prescaled: bool = False, **kw):
    """A16 down over one pool: (B_total, hidden)."""
    a = x_rot.to(torch.float16).contiguous()
    out = _merged(A16, True, a, None, a.shape[1], indices_packed_gf, codebook.to(torch.float16).contiguous(),
                  norms_gf, expert_info, group_size, bit_width, norms_prescaled, **kw)
    return out.to(x_rot.dtype)


def wxa8_matmul_merged_rows_gf(x_i8, x_scale, indices_packed_gf, codebook_i8, norms_gf, expert_info, group_size,
                               in_features, bit_width: int = 2, norms_prescaled: bool = True, **kw):
    """INT8 gate_up over one pool: fp16 (B_total, 2*inter).  ``partials=`` receives int32 (B, 2*inter, G)."""
    if in_features % group_size:
        raise ValueError(f"in_features ({in_features}) must be a multiple of group_size ({group_size})")
    return _merged(A8, False, x_i8.contiguous(), x_scale.to(torch.float16).contiguous(), in_features,
                   indices_packed_gf, codebook_i8.contiguous(), norms_gf, expert_info, group_size, bit_width,
                   norms_prescaled, **kw)


def wxa8_matmul_merged_in_features_gf(x_i8, x_scale, indices_packed_gf, codebook_i8, norms_gf, expert_info,
                                      group_size, bit_width: int = 2, norms_prescaled: bool = True, **kw):
    """INT8 down over one pool: fp16 (B_total, hidden)."""
    return _merged(A8, True, x_i8.contiguous(), x_scale.to(torch.float16).contiguous(), x_i8.shape[1],
                   indices_packed_gf, codebook_i8.contiguous(), norms_gf, expert_info, group_size, bit_width,
                   norms_prescaled, **kw)


def wxfp8_matmul_merged_rows_gf(x_f8, x_scale, indices_packed_gf, codebook_f8, norms_gf, expert_info, group_size,
                                in_features, bit_width: int = 2, norms_prescaled: bool = True, **kw):
    """e4m3 gate_up over one pool: fp16 (B_total, 2*inter)."""
    if in_features % group_size:
        raise ValueError(f"in_features ({in_features}) must be a multiple of group_size ({group_size})")
    return _merged(FP8, False, x_f8.view(torch.uint8).contiguous(), x_scale.to(torch.float16).contiguous(),
                   in_features, indices_packed_gf, codebook_f8.view(torch.uint8).contiguous(), norms_gf,
                   expert_info, group_size, bit_width, norms_prescaled, **kw)


def wxfp8_matmul_merged_in_features_gf(x_f8, x_scale, indices_packed_gf, codebook_f8, norms_gf, expert_info,
                                       group_size, bit_width: int = 2, norms_prescaled: bool = True, **kw):
    """e4m3 down over one pool: fp16 (B_total, hidden)."""
    a = x_f8.view(torch.uint8).contiguous()
    return _merged(FP8, True, a, x_scale.to(torch.float16).contiguous(), a.shape[1], indices_packed_gf,
                   codebook_f8.view(torch.uint8).contiguous(), norms_gf, expert_info, group_size, bit_width,
                   norms_prescaled, **kw)


def _fp4_e0(w_s: torch.Tensor) -> int:
    return int(w_s.reshape(-1)[0].item()) - 127


def wxfp4_matmul_merged_rows_gf(x_f4_t, x_s, indices_packed_gf, nib, w_s, norms_gf, expert_info, group_size,
                                in_features, bit_width: int = 1, norms_prescaled: bool = True,
                                w_e2m1_gf=None, **kw):
    """e2m1 gate_up over one pool.  ``x_f4_t`` is (K/2, B_total) as in the reference; ``w_s`` is the constant
    e8m0 weight block scale 127+E0.  The folded copy ``w_e2m1_gf`` is accepted and ignored (same values)."""
    if in_features % group_size:
        raise ValueError(f"in_features ({in_features}) must be a multiple of group_size ({group_size})")
    a = x_f4_t.t().contiguous()
    return _merged(FP4, False, a, x_s.contiguous(), in_features, indices_packed_gf, nib.contiguous(), norms_gf,
                   expert_info, group_size, bit_width, norms_prescaled, e0=_fp4_e0(w_s), **kw)


def wxfp4_matmul_merged_in_features_gf(x_f4_t, x_s, indices_packed_gf, nib, w_s, norms_gf, expert_info, group_size,
                                       bit_width: int = 1, norms_prescaled: bool = True, w_e2m1_gf=None, **kw):
    """e2m1 down over one pool: fp16 (B_total, hidden)."""
    a = x_f4_t.t().contiguous()
    return _merged(FP4, True, a, x_s.contiguous(), a.shape[1] * 2, indices_packed_gf, nib.contiguous(), norms_gf,
                   expert_info, group_size, bit_width, norms_prescaled, e0=_fp4_e0(w_s), **kw)



@_on_tensor_device
def quantize_packed_full(W: torch.Tensor, bit_width: int, group_size: int = GROUP, seed: int = 42,
                         uniform_codebook: bool = False) -> dict:
    """``format.turboquant_quantize_packed_full`` (turboquant_utils/quantize.py:350) as one library kernel: the same
    dict, tensors on W's device.  Rotation matrices and codebook come from the format module (the reference's own
    CPU generators), the per-element work runs in ``dmoq_quantize_packed``."""
    _need_cuda(W)
    if bit_width not in fmt.SUPPORTED_BITS:
        raise ValueError(f"bit_width must be 1/2/4/8, got {bit_width}")
    if group_size != GROUP or W.shape[1] % GROUP:
        raise ValueError(f"group_size must be {GROUP} and K a multiple of it")
    if uniform_codebook and bit_width != 8:
        raise ValueError(f"uniform_codebook requires bit_width=8, got {bit_width}")
    kind = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}.get(W.dtype)
    if kind is None:
        raise TypeError(f"W must be fp32, fp16 or bf16, got {W.dtype}")
    W = W.contiguous()
    N, K = W.shape
    cent, edges = fmt.uniform8_codebook() if uniform_codebook else fmt.get_codebook(bit_width)
    rot = torch.stack([fmt.generate_rotation_matrix(GROUP, seed=seed + g0) for g0 in range(0, K, GROUP)]).to(W.device).float().contiguous()
    edges_d = edges.to(W.device).float().contiguous()
    idx = torch.empty((N, K * bit_width // 8), dtype=torch.uint8, device=W.device)
    norms = torch.empty((N, K // GROUP), dtype=torch.float16, device=W.device)
    check(_lib.load().dmoq_quantize_packed(ptr(W), kind, N, K, bit_width, ptr(rot), ptr(edges_d), ptr(idx), ptr(norms),
                                           _stream()), "dmoq_quantize_packed")
    return {"indices_packed": idx, "codebook": cent.half().cpu(), "norms": norms, "seed": seed, "group_size": GROUP,
            "shape": (N, K), "bit_width": bit_width, "rotation": "qr", "orig_dtype": str(W.dtype),
            "codebook_type": "uniform" if uniform_codebook else "lloydmax"}
