"""GPU parity: libdmoq kernels (through the C ABI) against the CPU oracle and the reference goldens.

Integer / byte / index stages must match bit for bit; floating-point outputs must be within a relative
Frobenius error of 1e-2 (A16, A8) or 2e-2 (FP8, FP4) of the same-mode oracle.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import dmoq_oracle as O
import dartmoq_b200 as D
from dartmoq_b200 import _lib, format as F, kernels as K, synth
from dartmoq_b200.moe import _Engine
from helpers import rel_fro, routing, to_oracle_layer

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = {"wxa16": 1e-2, "wxa8": 1e-2, "wxfp8": 2e-2, "wxfp4": 2e-2}


def cuda(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    return (t if dtype is None else t.to(dtype)).to(DEV)


# ------------------------------------------------------------------------------------------------ routing

def _run_route(T, k, E, idx, w, pools_of, hoisted, shared_w=None, tile_m=128):
    """Drive dmoq_route_build directly; returns the tables as numpy."""
    lib = _lib.load()
    has_shared = shared_w is not None
    n_ent = E + int(has_shared)
    R = T * k + (T if has_shared else 0)
    i32 = dict(dtype=torch.int32, device=DEV)
    n_pools = max(pools_of) + 1
    members = [sum(1 for p in pools_of if p == q) for q in range(n_pools)]
    rank, seen = [], [0] * n_pools
    for p in pools_of:
        rank.append(seen[p] if p >= 0 else 0)
        if p >= 0:
            seen[p] += 1
    t = dict(expert_pool=torch.tensor(pools_of, **i32), expert_rank=torch.tensor(rank, **i32),
             expert_rows=torch.zeros(n_ent + 1, **i32), sorted_tokens=torch.full((max(R, 1),), -7, **i32),
             sorted_weights=torch.zeros(max(R, 1), dtype=torch.float32, device=DEV),
             row_of=torch.full((max(R, 1),), -9, **i32), a_row=torch.full((max(R, 1),), -5, **i32),
             pool_rows=torch.zeros(8, **i32), n_tiles=torch.zeros(16, **i32))
    caps = [T if hoisted[q] else T * min(k, members[q]) for q in range(n_pools)]
    bases, tot = [], 0
    for q in range(n_pools):
        bases.append(0 if hoisted[q] else tot)
        tot += 0 if hoisted[q] else caps[q]
    t["pool_src"] = torch.full((max(tot, 1),), -3, **i32)
    t["pool_src_base"] = torch.tensor(bases + [0] * (8 - n_pools), **i32)
    t["pool_hoisted"] = torch.tensor([int(h) for h in hoisted] + [0] * (8 - n_pools), **i32)
    tile_cap = (R + tile_m - 1) // tile_m + n_ent
    t["tiles"] = torch.zeros(tile_cap, 4, **i32)
    r = _lib.Route()
    r.T, r.top_k, r.E, r.has_shared, r.tile_m, r.n_pools, r.tile_cap = T, k, E, int(has_shared), tile_m, n_pools, tile_cap
    for name in ("expert_pool", "expert_rank", "expert_rows", "sorted_tokens", "sorted_weights", "row_of", "a_row",
                 "pool_rows", "pool_src", "pool_src_base", "tiles", "n_tiles", "pool_hoisted"):
        setattr(r, name, t[name].data_ptr())
    ws = torch.empty(max(lib.dmoq_route_workspace_bytes(T, k, E), 16), dtype=torch.uint8, device=DEV)
    idx_d, w_d = cuda(idx, torch.int64), cuda(w, torch.float32)
    sw_d = None if shared_w is None else cuda(shared_w, torch.float32)
    _lib.check(lib.dmoq_route_build(C.byref(r), _lib.ptr(idx_d), _lib.ptr(w_d), _lib.ptr(sw_d), _lib.ptr(ws),
                                    ws.numel(), None), "route")
    torch.cuda.synchronize()
    return {k2: v.cpu().numpy() for k2, v in t.items()}, bases


@pytest.mark.parametrize("T,k,E", [(1, 2, 4), (7, 2, 5), (33, 8, 16), (300, 8, 64), (5000, 8, 256), (2048, 6, 128)])
def test_route_build_matches_stable_sort(T, k, E):
    rng = np.random.default_rng(T * 131 + E)
    idx = np.stack([rng.permutation(E)[:k] for _ in range(T)]).astype(np.int64)
    w = rng.random((T, k), dtype=np.float32)
    shared_w = rng.random(T, dtype=np.float32) if T % 2 else None
    pools_of = [int(e % 3) if e % 7 != 6 else -1 for e in range(E)]     # three pools, some experts unused
    pools_of[0], pools_of[1 % E] = 0, 1 if E > 1 else 0
    if max(pools_of) < 2:
        pools_of[-1] = 2
    if shared_w is not None:
        pools_of = pools_of + [max(pools_of) + 1]
    n_pools = max(pools_of) + 1
    hoisted = [q % 2 == 0 for q in range(n_pools)]
    if shared_w is not None:
        hoisted[-1] = True
    got, bases = _run_route(T, k, E, idx, w, pools_of, hoisted, shared_w)

    tokens, weights, starts, order = O.sort_rows(idx, w, E)
    R0 = T * k
    assert np.array_equal(got["expert_rows"][:E + 1], starts)
    assert np.array_equal(got["sorted_tokens"][:R0], tokens)
    assert np.array_equal(got["sorted_weights"][:R0], weights)
    inv = np.empty(R0, np.int64)
    inv[order] = np.arange(R0)
    exp_of_flat = idx.reshape(-1)
    used = np.array([pools_of[e] >= 0 for e in exp_of_flat])
    assert np.array_equal(got["row_of"][:R0][used], inv[used]) and (got["row_of"][:R0][~used] == -1).all()
    if shared_w is not None:
        assert np.array_equal(got["sorted_tokens"][R0:R0 + T], np.arange(T))
        assert np.array_equal(got["sorted_weights"][R0:R0 + T], shared_w)
        assert np.array_equal(got["row_of"][R0:R0 + T], R0 + np.arange(T))
        assert got["expert_rows"][E + 1] == R0 + T
    # tiles: every row of a used expert is covered exactly once, in its pool's list, by tiles of <= 128 rows
    counts = np.diff(got["expert_rows"])
    cover = np.zeros(got["expert_rows"][-1], np.int32)
    rank_of = got["expert_rank"]
    for q in range(n_pools):
        n, base = got["n_tiles"][q], got["n_tiles"][8 + q]
        for e, row0, rows, rank in got["tiles"][base:base + n]:
            assert rank == rank_of[e] and pools_of[e] == q and 0 < rows <= 128
            assert got["expert_rows"][e] <= row0 and row0 + rows <= got["expert_rows"][e + 1]
            cover[row0:row0 + rows] += 1
        assert got["pool_rows"][q] == sum(counts[e] for e in range(len(pools_of)) if pools_of[e] == q)
    for e in range(len(pools_of)):
        lo, hi = got["expert_rows"][e], got["expert_rows"][e + 1]
        assert (cover[lo:hi] == (1 if pools_of[e] >= 0 else 0)).all()
    # activation-table rows: token for hoisted pools, compact per-pool rows (with their source token) otherwise
    for e in range(E):
        q = pools_of[e]
        if q < 0:
            continue
        lo, hi = got["expert_rows"][e], got["expert_rows"][e + 1]
        if hoisted[q]:
            assert np.array_equal(got["a_row"][lo:hi], got["sorted_tokens"][lo:hi])
        else:
            ar = got["a_row"][lo:hi]
            assert np.array_equal(got["pool_src"][bases[q] + ar], got["sorted_tokens"][lo:hi])
    for q in range(n_pools):
        if not hoisted[q]:
            rows = np.concatenate([got["a_row"][got["expert_rows"][e]:got["expert_rows"][e + 1]]
                                   for e in range(E) if pools_of[e] == q] or [np.zeros(0, np.int32)])
            assert np.array_equal(np.sort(rows), np.arange(rows.size))


# ------------------------------------------------------------------------------------------------ rotate + quantise

def test_rotate_quantize_reference_golden(golden):
    """Codes and scales equal the reference kernels' (Triton interpreter) outputs bit for bit."""
    g = golden("actquant")
    x, rot = cuda(g["x_f16"]), cuda(g["rot_f16"])
    q, s = K.rotate_quantize_fused(x, rot, 128, 2, extra_scale=0.0118956)
    assert np.array_equal(q.cpu().numpy(), g["i8_q"]) and np.array_equal(s.cpu().numpy(), g["i8_s"])
    q, s = K.rotate_quantize_fused_fp8(x, rot, 128, 2, extra_scale=0.00472075)
    assert np.array_equal(q.view(torch.uint8).cpu().numpy(), g["f8_q"]) and np.array_equal(s.cpu().numpy(), g["f8_s"])
    q, s = K.rotate_quantize_fused_fp4(x, rot, 128, 2)
    assert np.array_equal(q.cpu().numpy(), g["f4_q_t"]) and np.array_equal(s.cpu().numpy(), g["f4_s"])
    r = K.batch_rotate_input(x, 128, 44)
    assert rel_fro(r.float().cpu().numpy(), g["rot_only_f16"]) < 2e-3


@pytest.mark.parametrize("rows", [1, 63, 64, 65, 200, 1000])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_rotate_quantize_vs_oracle_bit_exact(rows, dtype):
    K_ = 384
    g = torch.Generator().manual_seed(rows)
    x = torch.randn(rows, K_, generator=g)
    x[:, 3] *= 20
    if rows > 2:
        x[1] = 0
        x[2] *= 1e-5
    x = x.to(dtype)
    rot = F.generate_batch_rotation_matrices(128, 46, 3, 128, "cpu", torch.float16)
    acc = O.rotate_f32(O.to_f16_values(x), rot.numpy())
    xd, rd = x.to(DEV), rot.to(DEV)
    q, s = K.rotate_quantize_fused(xd, rd, 128, 3, extra_scale=0.0215151)
    oq, os_ = O.actquant_int8(acc, 0.0215151)
    assert np.array_equal(q.cpu().numpy(), oq) and np.array_equal(s.cpu().numpy(), os_)
    q, s = K.rotate_quantize_fused_fp8(xd, rd, 128, 3, extra_scale=0.0573616)
    oq, os_ = O.actquant_e4m3(acc, 0.0573616)
    assert np.array_equal(q.view(torch.uint8).cpu().numpy(), oq) and np.array_equal(s.cpu().numpy(), os_)
    q, s = K.rotate_quantize_fused_fp4_rowmajor(xd, rd, 128, 3)
    oq, os_ = O.actquant_e2m1(acc)
    assert np.array_equal(q.cpu().numpy(), oq) and np.array_equal(s.cpu().numpy(), os_)
    r = K.batch_rotate_input(xd, 128, 46)      # A16: a floating-point output, tensor-core accumulation order
    assert rel_fro(r.float().cpu().numpy(), acc) < 1e-3


def test_rotate_quantize_gather_and_errors():
    x = synth.make_activations(50, 256, seed=2).to(DEV)
    rot = F.generate_batch_rotation_matrices(128, 44, 2, 128, DEV, torch.float16)
    src = torch.tensor([49, 0, 7, 7, 13], dtype=torch.int32, device=DEV)
    q = torch.empty(5, 256, dtype=torch.int8, device=DEV)
    s = torch.empty(5, 2, dtype=torch.float16, device=DEV)
    K._rotate(_lib.A8, x, rot, 0.01, q, s, src_row=src, n_rows=5)
    qf, sf = K.rotate_quantize_fused(x, rot, 128, 2, extra_scale=0.01)
    assert torch.equal(q, qf[src.long()]) and torch.equal(s, sf[src.long()])
    with pytest.raises(ValueError):
        K.rotate_quantize_fused(x, rot, 128, 3)
    with pytest.raises(ValueError):
        K.rotate_quantize_fused(x, rot[:, :64], 128, 2)
    q0, s0 = K.rotate_quantize_fused(x[:0], rot, 128, 2)
    assert q0.shape == (0, 256) and s0.shape == (0, 2)


@pytest.mark.parametrize("T,E,k,renorm", [(1, 8, 2, True), (37, 256, 8, True), (500, 128, 4, False), (64, 1000, 32, True)])
def test_router_topk_matches_torch(T, E, k, renorm):
    """softmax -> top-k (-> renormalise) in one launch: same experts, weights within a few fp32 ulps of torch's."""
    g = torch.Generator().manual_seed(T + E)
    logits = (torch.randn(T, E, generator=g) * 3).to(DEV)
    w, idx = K.router_topk(logits, k, renormalize=renorm)
    pw, pidx = torch.softmax(logits, dim=-1).topk(k, dim=-1)
    if renorm:
        pw = pw / pw.sum(dim=-1, keepdim=True)
    assert idx.dtype == torch.int64 and torch.equal(idx, pidx)
    assert torch.allclose(w, pw, rtol=2e-6, atol=1e-9)
    lib = _lib.load()
    assert lib.dmoq_router_topk(_lib.ptr(logits), T, E, E + 1, 0, _lib.ptr(w), _lib.ptr(idx), None) == -1


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_router_launch_carries_shared_gate(dtype):
    """sigmoid(shared_expert_gate(x)) from the router launch: the roundings of a 16-bit Linear + sigmoid; a value may
    sit one 16-bit place from torch's where the two dot products (different summation order) round apart."""
    T, H, E, k = 333, 512, 64, 4
    g = torch.Generator().manual_seed(77)
    logits = torch.randn(T, E, generator=g).to(DEV)
    x = torch.randn(T, H, generator=g).to(dtype).to(DEV)
    lin = torch.nn.Linear(H, 1, bias=False, dtype=dtype, device=DEV)
    lin.weight.data.copy_((torch.randn(1, H, generator=g) * 0.05).to(dtype))
    assert K.fusable_shared_gate(lin, x)
    w, idx, sw = K.router_topk(logits, k, x=x, shared_gate=lin)
    pw, pidx = torch.softmax(logits, dim=-1).topk(k, dim=-1)
    assert torch.equal(idx, pidx) and torch.allclose(w, pw, rtol=2e-6, atol=1e-9)
    want = torch.sigmoid(lin(x)).reshape(-1).float()
    assert sw.dtype == torch.float32 and torch.equal(sw.to(dtype).float(), sw)       # values of the 16-bit type
    assert (sw == want).float().mean() > 0.9
    assert float((sw - want).abs().max()) <= (2.0 ** -7 if dtype == torch.bfloat16 else 2.0 ** -9)
    assert not K.fusable_shared_gate(torch.nn.Linear(H, 1, bias=True, dtype=dtype, device=DEV), x)


@pytest.mark.parametrize("bit", [1, 2])
def test_widen_indices(bit):
    """Every 1- or 2-bit code becomes one 4-bit field, low field first."""
    g = torch.Generator().manual_seed(bit)
    packed = torch.randint(0, 256, (3, 40, 16 * bit), dtype=torch.uint8, generator=g)
    codes = F.unpack_nbit(packed.reshape(-1, 16 * bit), bit, 128).reshape(-1)          # one code per entry
    want = (codes[0::2] | (codes[1::2] << 4)).to(torch.uint8).reshape(3, 40, 64)
    src = packed.to(DEV)
    dst = torch.zeros(3, 40, 64, dtype=torch.uint8, device=DEV)
    lib = _lib.load()
    _lib.check(lib.dmoq_widen_indices(_lib.ptr(src), src.numel(), bit, _lib.ptr(dst), None), "dmoq_widen_indices")
    assert torch.equal(dst.cpu(), want)
    assert lib.dmoq_widen_indices(_lib.ptr(src), src.numel(), 4, _lib.ptr(dst), None) == -1


def test_group_first_relayout():
    for b in (1, 2, 4, 8):
        p = torch.randint(0, 256, (40, 3 * 16 * b), dtype=torch.uint8)
        n = torch.randn(40, 3).half()
        gi, gn = K.convert_to_group_first(p.to(DEV), n.to(DEV), 128, b)
        ri, rn = F.convert_to_group_first(p, n, 128, b)
        assert torch.equal(gi.cpu(), ri) and torch.equal(gn.cpu(), rn)


# ------------------------------------------------------------------------------------------------ grouped GEMMs

def _gemm_inputs(g, b):
    gu_i, gu_n = F.convert_to_group_first(torch.from_numpy(g[f"gu_idx_{b}"]), torch.from_numpy(g[f"gu_norms_{b}"]), 128, b)
    dn_i, dn_n = F.convert_to_group_first(torch.from_numpy(g[f"dn_idx_{b}"]), torch.from_numpy(g[f"dn_norms_{b}"]), 128, b)
    pre = lambda n: (n.float() / torch.full((1,), float(np.sqrt(128.0)))).half()
    counts, I = g["counts"], 256
    rows, groups, cur = [], [], 0
    for e, n in enumerate(counts):
        if n:
            rows.append((cur, int(n), 2 * I * e, 2 * I))
            groups.append((cur, int(n), e * I // 128, I // 128))
            cur += int(n)
    return gu_i.to(DEV), pre(gu_n).to(DEV), dn_i.to(DEV), pre(dn_n).to(DEV), rows, groups


def _close_fp16(got, want):
    """INT8 GEMM outputs: the integer group sums are exact; the tensor-core kernel fuses the last multiply-add
    of the fp32 scaling, so a few fp16 outputs may differ from the unfused reference in the last place."""
    got = got.float().cpu().numpy()
    want = want.astype(np.float32)
    assert rel_fro(got, want) < 1e-4 and (got != want).mean() < 5e-3


@pytest.mark.parametrize("images", (False, True))
@pytest.mark.parametrize("b", (1, 2, 4))
def test_merged_gemm_reference_golden(golden, b, images, monkeypatch):
    """Function-level operators on the reference's own inputs: A8 bit-exact (codes, int32 sums, fp16 output).
    ``images``: every mode through the image-fed tensor-core kernel (weights looked up once by dmoq_expand_weights)."""
    monkeypatch.setattr(K, "USE_WEIGHT_IMAGES", True if images else None)
    g = golden("merged_gemm")
    H = I = 256
    gu_i, gu_n, dn_i, dn_n, rows, groups = _gemm_inputs(g, b)
    cb = torch.from_numpy(g[f"cb_{b}"])
    x, a = cuda(g[f"x_{b}"]), cuda(g[f"a_{b}"])
    B = x.shape[0]
    rot_gu = F.generate_batch_rotation_matrices(128, 42 + b, 2, 128, DEV, torch.float16)

    def down_codes(fn, extra=None):
        qs, ss = [], []
        for s0, n, g0, _ in groups:
            rot = F.generate_batch_rotation_matrices(128, 42 + b + 1000 + g0 * 128, 2, 128, DEV, torch.float16)
            q, s = fn(a[s0:s0 + n], rot, 128, 2) if extra is None else fn(a[s0:s0 + n], rot, 128, 2, extra_scale=extra)
            qs.append(q), ss.append(s)
        return qs, ss

    # ---- A8
    lut8, step = F.build_int8_codebook(cb)
    q, s = K.rotate_quantize_fused(x, rot_gu, 128, 2, extra_scale=step)
    assert np.array_equal(q.cpu().numpy(), g[f"a8_xq_{b}"]) and np.array_equal(s.cpu().numpy(), g[f"a8_xs_{b}"])
    part = torch.zeros(B, 2 * I, 2, dtype=torch.int32, device=DEV)
    gu = K.wxa8_matmul_merged_rows_gf(q, s, gu_i, lut8.to(DEV), gu_n, rows, 128, H, bit_width=b, partials=part)
    _close_fp16(gu, g[f"a8_gu_{b}"])
    lut_np = lut8.numpy().astype(np.int32)
    for s0, n, c0, _ in rows:
        w = lut_np[O.weight_codes(gu_i.cpu().numpy(), b, slice(c0, c0 + 2 * I), slice(0, 2))]
        want = np.einsum("bgk,gnk->bng", g[f"a8_xq_{b}"][s0:s0 + n].reshape(n, 2, 128).astype(np.int32), w)
        assert np.array_equal(part[s0:s0 + n].cpu().numpy(), want)
    qs, ss = down_codes(K.rotate_quantize_fused, step)
    assert np.array_equal(torch.cat(qs).cpu().numpy(), g[f"a8_aq_{b}"])
    assert np.array_equal(torch.cat(ss).cpu().numpy(), g[f"a8_as_{b}"])
    dn = K.wxa8_matmul_merged_in_features_gf(torch.cat(qs), torch.cat(ss), dn_i, lut8.to(DEV), dn_n, groups, 128, bit_width=b)
    _close_fp16(dn, g[f"a8_dn_{b}"])
    # ---- A16
    gu = K.triton_fused_matmul_merged_rows_gf(K.batch_rotate_input(x, 128, 42 + b), gu_i, cb.to(DEV), gu_n, rows,
                                              128, H, bit_width=b, norms_prescaled=True)
    assert rel_fro(gu.float().cpu().numpy(), g[f"a16_gu_{b}"]) < 1e-2
    parts = [K.batch_rotate_input(a[s0:s0 + n], 128, 42 + b + 1000 + g0 * 128) for s0, n, g0, _ in groups]
    dn = K.triton_fused_matmul_merged_in_features_gf(torch.cat(parts), dn_i, cb.to(DEV), dn_n, groups, 128,
                                                     bit_width=b, norms_prescaled=True)
    assert rel_fro(dn.float().cpu().numpy(), g[f"a16_dn_{b}"]) < 1e-2
    # ---- FP8
    lutf, sc = F.build_fp8_codebook(cb)
    q, s = K.rotate_quantize_fused_fp8(x, rot_gu, 128, 2, extra_scale=sc)
    gu = K.wxfp8_matmul_merged_rows_gf(q, s, gu_i, lutf.to(DEV), gu_n, rows, 128, H, bit_width=b)
    assert rel_fro(gu.float().cpu().numpy(), g[f"f8_gu_{b}"]) < 2e-2
    qs, ss = down_codes(K.rotate_quantize_fused_fp8, sc)
    dn = K.wxfp8_matmul_merged_in_features_gf(torch.cat(qs), torch.cat(ss), dn_i, lutf.to(DEV), dn_n, groups, 128, bit_width=b)
    assert rel_fro(dn.float().cpu().numpy(), g[f"f8_dn_{b}"]) < 2e-2
    # ---- FP4
    nib, e0, resid, _ = F.build_e2m1_codebook(cb)
    ws = torch.full((1,), 127 + e0, dtype=torch.uint8)
    fold = lambda n: (n.float() * resid).half()
    q, s = K.rotate_quantize_fused_fp4(x, rot_gu, 128, 2)
    assert np.array_equal(q.t().cpu().numpy(), g[f"f4_xq_{b}"]) and np.array_equal(s.cpu().numpy(), g[f"f4_xs_{b}"])
    gu = K.wxfp4_matmul_merged_rows_gf(q, s, gu_i, nib.to(DEV), ws, fold(gu_n), rows, 128, H, b)
    assert rel_fro(gu.float().cpu().numpy(), g[f"f4_gu_{b}"]) < 2e-2
    qs, ss = down_codes(K.rotate_quantize_fused_fp4)
    dn = K.wxfp4_matmul_merged_in_features_gf(torch.cat(qs, dim=1), torch.cat(ss), dn_i, nib.to(DEV), ws, fold(dn_n),
                                              groups, 128, b)
    assert rel_fro(dn.float().cpu().numpy(), g[f"f4_dn_{b}"]) < 2e-2


def test_merged_gemm_argument_errors():
    x = torch.zeros(4, 256, dtype=torch.int8, device=DEV)
    s = torch.ones(4, 2, dtype=torch.float16, device=DEV)
    idx = torch.zeros(2, 512, 32, dtype=torch.uint8, device=DEV)
    nrm = torch.ones(2, 512, dtype=torch.float16, device=DEV)
    lut = torch.zeros(4, dtype=torch.int8, device=DEV)
    with pytest.raises(ValueError):
        K.wxa8_matmul_merged_rows_gf(x, s, idx, lut, nrm, [(0, 4, 0, 512)], 128, 256, bit_width=3)
    with pytest.raises(ValueError):
        K.wxa8_matmul_merged_rows_gf(x, s, idx, lut, nrm, [(0, 4, 0, 512)], 128, 200, bit_width=2)
    with pytest.raises(ValueError):
        K.wxa8_matmul_merged_rows_gf(x, s, idx, lut, nrm, [(0, 2, 0, 512), (2, 2, 0, 256)], 128, 256, bit_width=2)
    with pytest.raises(ValueError):
        K.wxa8_matmul_merged_rows_gf(x, s, idx, lut, nrm, [], 128, 256, bit_width=2)


# ------------------------------------------------------------------------------------------------ whole layer

def _layer(mode, seed=77, **kw):
    cfg = dict(hidden=256, n_experts=10, top_k=3, inter=256, bit_mix={2: 0.6, 1: 0.2, 4: 0.2}, mode=mode,
               shared_inter=256, seed=seed)
    cfg.update(kw)
    return synth.build_layer(**cfg)


@pytest.mark.parametrize("images", ["auto", "always", "never"])
@pytest.mark.parametrize("mode", ["wxa8", "wxa16", "wxfp8", "wxfp4"])
@pytest.mark.parametrize("T", [1, 5, 150, 700])
def test_module_forward_vs_oracle(mode, T, images):
    moe = _layer(mode)
    moe.weight_images = images     # "always": every pool through the image-fed kernel; "never": index expansion per tile
    x = synth.make_activations(T, 256, seed=T)
    tw, ti, sw = routing(moe, x)
    ref = O.moe_forward(to_oracle_layer(moe), x, tw, ti, sw)
    y = moe.to(DEV)(x.to(DEV).unsqueeze(0))[0]
    assert y.dtype == torch.bfloat16 and y.shape == (T, 256)
    assert rel_fro(y.float().cpu().numpy(), ref["y"]) < TOL[mode]


class _LogitsGate(torch.nn.Module):
    """A gate that returns plain logits, the form the module handles with softmax -> topk itself."""

    def __init__(self, n_tokens, n_experts, seed):
        super().__init__()
        g = torch.Generator().manual_seed(seed)
        self.register_buffer("table", torch.randn(n_tokens, n_experts, generator=g) * 2)

    def forward(self, x):
        return self.table[:x.shape[0]]


def test_module_with_logits_gate_uses_fused_router():
    """Gates that return logits go through dmoq_router_topk on the GPU; same result as softmax -> topk in torch."""
    moe = _layer("wxa8", seed=3)
    T = 200
    moe.gate = _LogitsGate(T, moe.num_experts, seed=8)
    x = synth.make_activations(T, 256, seed=2)
    tw, ti, sw = routing(moe, x)
    ref = O.moe_forward(to_oracle_layer(moe), x, tw, ti, sw)
    y = moe.to(DEV)(x.to(DEV).unsqueeze(0))[0]
    assert rel_fro(y.float().cpu().numpy(), ref["y"]) < TOL["wxa8"]


@pytest.mark.parametrize("images", ["never", "always"])
@pytest.mark.parametrize("hoist", [True, False])
def test_a8_stages_bit_exact(hoist, images):
    """INT8 path, stage by stage: activation codes, stored scales and int32 group sums equal the oracle's."""
    moe = _layer("wxa8", seed=5, n_experts=6, top_k=4)
    moe.enable_rotation_hoist = hoist
    moe.weight_images = images
    T = 90
    x = synth.make_activations(T, 256, seed=9)
    tw, ti, sw = routing(moe, x)
    ref = O.moe_forward(to_oracle_layer(moe), x, tw, ti, sw, keep=True)
    moe = moe.to(DEV)
    eng = moe._get_engine(torch.device(DEV))
    R = T * moe.top_k + T
    parts = {("gate_up", p.key): torch.zeros(R, 2 * p.inter, 2, dtype=torch.int32, device=DEV) for p in eng.pools}
    parts.update({("down", p.key): torch.zeros(R, 256, p.inter // 128, dtype=torch.int32, device=DEV) for p in eng.pools})
    y = moe.forward(x.to(DEV).unsqueeze(0), _partials=parts)[0]
    torch.cuda.synchronize()
    ws = eng.workspace(T)
    rows_of_expert = ws.expert_rows.cpu().numpy()
    a_row = ws.a_row.cpu().numpy()
    for i, p in enumerate(eng.pools):
        st = ref["stages"][p.key]
        assert p.hoisted == (p.shared or (hoist and p.n_members * moe.top_k / moe.num_experts > 1.5))
        # global rows of this pool in the oracle's (rank-ordered) row order
        if p.shared:
            rows = np.arange(T * moe.top_k, R)
        else:
            members = [e for e in range(moe.num_experts) if eng.expert_pool[e].item() == i]
            rows = np.concatenate([np.arange(rows_of_expert[e], rows_of_expert[e + 1]) for e in members])
        codes = ws.act_codes[i].view(torch.int8).reshape(-1, 256).cpu().numpy()
        scales = ws.act_scales[i][:codes.shape[0] * 4].view(torch.float16).reshape(-1, 2).cpu().numpy()
        assert np.array_equal(codes[a_row[rows]], st["codes"])
        assert np.array_equal(scales[a_row[rows]], st["scales"])
        assert np.array_equal(parts[("gate_up", p.key)][rows].cpu().numpy(), st["parts_gu"])
        # the fused epilogue's fp16 SiLU may differ from the CPU's in the last place; the integer stages after
        # it are checked on identical inputs in test_merged_gemm_reference_golden
        act = ws.act[rows, :p.inter].float().cpu().numpy()
        assert rel_fro(act, st["act"]) < 1e-3
        same = np.all(act == st["act"].astype(np.float32), axis=1)
        dn_codes = ws.dn_codes.view(torch.int8).reshape(-1, eng.inter_max)[rows, :p.inter].cpu().numpy()
        want = np.concatenate(st["dn_codes"])
        assert same.mean() > 0.9, f"{(~same).sum()} of {same.size} SiLU rows differ from the CPU in the last place"
        assert np.array_equal(dn_codes[same], want[same])
        assert np.array_equal(parts[("down", p.key)][rows].cpu().numpy()[same], st["parts_dn"][same])
    assert rel_fro(y.float().cpu().numpy(), ref["y"]) < 1e-2


def test_multi_bit_experts_and_unused_expert():
    """An expert stored partly in 2 bits and partly in 4 bits (the reference's own test fixture layout)."""
    H, I, E = 256, 128, 4
    moe = D.WxA16BitPartitionedGroupMoE(synth.SyntheticRouter(H, E, 2, seed=1), E, H, 2 * I, 2)
    g = torch.Generator().manual_seed(3)
    for bit, members in ((4, [0, 1, 2, 3]), (2, [0, 2])):
        w = D.WxA16Weights(bit, H)
        n = len(members)
        w.set_packed_data(
            F.turboquant_quantize_packed_full(torch.randn(2 * I * n, H, generator=g) * 0.02, bit, 128, seed=42 + bit),
            F.turboquant_quantize_packed_full(torch.randn(H, I * n, generator=g) * 0.02, bit, 128, seed=1042 + bit))
        moe.bit_weights[str(bit)] = w
        offs, run = [0], 0
        for e in range(E):
            run += I if e in members else 0
            offs.append(run)
        moe.expert_offsets[str(bit)] = torch.tensor(offs)
    moe.bit_list = [4, 2]
    D.WxA8BitPartitionedGroupMoE.from_wxa16(moe)
    x = synth.make_activations(40, H, seed=4)
    tw, ti, _ = routing(moe, x)
    layer = to_oracle_layer(moe)
    ref = O.moe_forward(layer, x, tw, ti)["y"]
    y = moe.to(DEV)(x.to(DEV).unsqueeze(0))[0].float().cpu().numpy()
    assert rel_fro(y, ref) < 1e-2


@pytest.mark.parametrize("mode", ["wxa8", "wxfp4"])
def test_size_independent_properties(mode):
    """At a benchmark-scale token count: determinism, token-permutation equivariance, exact halving with the
    routing weights, zero for an all-zero input."""
    moe = synth.build_layer(hidden=1024, n_experts=32, top_k=4, inter=512, bit_mix={2: 0.9, 1: 0.05, 4: 0.05},
                            mode=mode, shared_inter=512, seed=8, device=DEV)
    T = 4096
    x = synth.make_activations(T, 1024, seed=3, device=DEV)
    _, tw, ti = moe.gate(x)
    sw = torch.sigmoid(moe.shared_expert_gate(x)).reshape(-1)
    eng = moe._get_engine(torch.device(DEV))
    y1 = eng.run(x, tw, ti, sw).clone()
    y2 = eng.run(x, tw, ti, sw).clone()
    assert torch.equal(y1, y2)
    perm = torch.randperm(T, device=DEV)
    yp = eng.run(x[perm].contiguous(), tw[perm], ti[perm], sw[perm]).clone()
    assert torch.equal(yp, y1[perm])
    yh = eng.run(x, tw * 0.5, ti, sw * 0.5).clone()
    assert torch.equal(yh.float() * 2, y1.float())
    y0 = eng.run(torch.zeros_like(x), tw, ti, sw)
    assert float(y0.float().abs().max()) == 0.0
    assert torch.isfinite(y1.float()).all()


def test_packed_linear_vs_dense():
    lin = torch.nn.Linear(256, 384, bias=True)
    x = synth.make_activations(70, 256, seed=6)
    for cls, bit, uni, tol in ((D.WxA16Linear, 4, False, 1e-2), (D.WxA8Linear, 8, True, 1e-2), (D.WxFP8Linear, 8, True, 6e-2)):
        q = D.WxA16Linear.from_linear(lin, bit, 128, seed=11, uniform_codebook=uni)
        dense = F.turboquant_dequantize_packed(dict(indices_packed=q.packed_indices, codebook=q.codebook, norms=q.norms,
                                                    seed=11, group_size=128, shape=(384, 256), bit_width=bit,
                                                    orig_dtype="torch.float32"))
        want = x.float() @ dense.T + lin.bias.float()
        if cls is not D.WxA16Linear:
            cls.from_wxa16(q)
        y = q.to(DEV)(x.to(DEV))
        assert y.dtype == torch.bfloat16 and rel_fro(y.float().cpu().numpy(), want.detach().numpy()) < tol + 1e-2


@pytest.mark.parametrize("mode", ["wxa16", "wxa8"])
def test_small_batch_graph_replay_matches_eager(mode):
    """Decode regime: 32-row tiles and CUDA-graph replay give the eager result, call after call."""
    moe = _layer(mode, seed=31, n_experts=16, top_k=4).to(DEV)
    outs = []
    for call in range(4):
        x = synth.make_activations(6, 256, seed=40 + call % 2, device=DEV)
        y = moe(x.unsqueeze(0))[0].clone()
        moe.enable_cuda_graph = False
        want = moe(x.unsqueeze(0))[0]
        moe.enable_cuda_graph = True
        assert torch.equal(y, want), call
        outs.append(y)
    assert moe._graphs and any(isinstance(v, tuple) for v in moe._graphs.values())
    assert torch.equal(outs[0], outs[2]) and not torch.equal(outs[0], outs[1])
    ref_moe = _layer(mode, seed=31, n_experts=16, top_k=4)
    xc = synth.make_activations(6, 256, seed=40)
    tw, ti, sw = routing(ref_moe, xc)
    ref = O.moe_forward(to_oracle_layer(ref_moe), xc, tw, ti, sw)["y"]
    assert rel_fro(outs[0].float().cpu().numpy(), ref) < TOL[mode]


@pytest.mark.parametrize("mode", ["wxa16", "wxa8"])
def test_weighted_combine_equals_weighted_epilogue(mode):
    """Plain down rows + dmoq_combine_weighted == DMOQ_EPI_WEIGHTED rows + dmoq_combine, bit for bit."""
    moe = _layer(mode, seed=21).to(DEV)
    T = 333
    x = synth.make_activations(T, 256, seed=5, device=DEV)
    y1 = moe(x.unsqueeze(0))[0]
    eng = moe._get_engine(torch.device(DEV))
    ws = eng.workspace(T)
    lib = _lib.load()
    dn2 = torch.zeros_like(ws.dn)
    for i, p in enumerate(eng.pools):   # the workspace still holds this forward's routing tables and activations
        _lib.check(lib.dmoq_rotate_quant_down(C.byref(ws.route), eng.pool_array, i, _lib.ptr(ws.act), eng.inter_max,
                                              _lib.ptr(ws.dn_codes), _lib.ptr(ws.dn_scales), eng.inter_max, None), "rq")
        _lib.check(lib.dmoq_grouped_gemm(C.byref(ws.route), eng.pool_array, i, 1, _lib.EPI_WEIGHTED, eng.hidden,
                                         _lib.ptr(ws.dn_codes), _lib.ptr(ws.dn_scales), eng.inter_max,
                                         _lib.ptr(dn2), eng.hidden, None, None), "gemm")
    y2 = torch.empty_like(y1)
    _lib.check(lib.dmoq_combine(C.byref(ws.route), _lib.ptr(dn2), eng.hidden, _lib.ptr(y2), 1, None), "combine")
    torch.cuda.synchronize()
    assert torch.equal(y1, y2)


def test_host_streamer_matches_direct_calls():
    """Pinned host batches through the three-stream pipeline give the results of plain module calls."""
    from dartmoq_b200.host_io import HostStreamer
    moe = _layer("wxa8", seed=12).to(DEV)
    T = 300
    xs = [synth.make_activations(T, 256, seed=70 + i).pin_memory() for i in range(5)]
    ys = [torch.empty(T, 256, dtype=torch.bfloat16).pin_memory() for _ in xs]
    st = HostStreamer(moe, T, 256, DEV)
    for x, y in zip(xs, ys):
        st.submit(x, y)
    st.join()
    torch.cuda.synchronize()
    for x, y in zip(xs, ys):
        assert torch.equal(y, moe(x.to(DEV).unsqueeze(0))[0].cpu())


@pytest.mark.parametrize("mode", ["wxa8", "wxa16"])
@torch.no_grad()
def test_expert_parallel_building_blocks_on_one_gpu(mode):
    """What the token-gather exchange relies on, without a second GPU: slots masked with -1 are dropped (the two
    halves of the experts add up to the whole layer), and the shared expert as a layer of its own equals the
    shared pool of the full layer bit for bit."""
    from dartmoq_b200 import ep
    moe = _layer(mode, seed=31, n_experts=8).to(DEV)
    x = synth.make_activations(333, 256, seed=5).to(DEV)
    out = moe.gate(x)
    tw, ti = out[1:] if isinstance(out, tuple) else out.softmax(dim=-1).topk(3, dim=-1)
    tw, ti = tw.float(), ti.long()
    sw = torch.sigmoid(moe.shared_expert_gate(x)).reshape(-1).float()
    eng = moe._get_engine(DEV)
    zero_sw = torch.zeros_like(sw)
    whole = eng.run(x, tw, ti, zero_sw).float().cpu()
    halves = [eng.run(x, tw, torch.where((ti >= lo) & (ti < lo + 4), ti, torch.full_like(ti, -1)), zero_sw).float().cpu()
              for lo in (0, 4)]
    assert rel_fro(halves[0] + halves[1], whole) < 4e-3            # each half is rounded to bf16 once
    none = torch.full_like(ti, -1)
    assert torch.count_nonzero(eng.run(x, tw, none, zero_sw)) == 0
    shared_in_layer = eng.run(x, tw, none, sw).clone()
    wrap = ep.ExpertParallelMoE(moe.gate, ep.shard_experts(moe, 0, 8), 8, 3, moe.shared_expert, moe.shared_expert_gate)
    alone = wrap._shared_partial(x)
    assert wrap._shared_layer[0] is not None and torch.equal(alone, shared_in_layer)
    dense = (moe.shared_expert(x) * torch.sigmoid(moe.shared_expert_gate(x))).float().cpu()
    assert rel_fro(alone.float().cpu(), dense) < 2e-2


@pytest.mark.parametrize("b", (1, 2, 4, 8))
def test_quantizer_kernel_vs_reference_golden(golden, b):
    """The quantiser as a library kernel on the reference's own input: norms and indices equal the reference's
    (torch CPU) outputs except where a rotated value sits within fp32 rounding of a cell edge or a norm within rounding
    of an fp16 midpoint (the kernel sums in a fixed order, torch's BLAS in its own); the dequantised matrix agrees."""
    g = golden("quantizer")
    W = torch.from_numpy(g["W"])
    pk = K.quantize_packed_full(W.to(DEV), b, 128, seed=42 + b)
    got = F.unpack_nbit(pk["indices_packed"].cpu(), b, W.shape[1]).numpy()
    want = F.unpack_nbit(torch.from_numpy(g[f"idx_{b}"]), b, W.shape[1]).numpy()
    differ = got != want
    assert differ.mean() < 2e-4, differ.mean()
    assert (np.abs(got.astype(np.int32) - want.astype(np.int32))[differ] <= 1).all()      # only neighbouring cells
    n_got, n_want = pk["norms"].cpu().numpy(), g[f"norms_{b}"]
    assert (n_got != n_want).mean() < 5e-3 and np.allclose(n_got.astype(np.float32), n_want.astype(np.float32), rtol=1e-3)
    assert np.array_equal(pk["codebook"].numpy(), g[f"cb_{b}"])
    deq = F.turboquant_dequantize_packed(dict(pk, orig_dtype="torch.float32"), device="cpu").numpy()
    assert rel_fro(deq, g[f"deq_{b}"]) < 2e-3
    # bf16 input and an input that is not a multiple of the row block
    W2 = synth.make_activations(70, 256, seed=4).to(DEV)
    p2 = K.quantize_packed_full(W2, b, 128, seed=7)
    r2 = F.turboquant_quantize_packed_full(W2.cpu(), b, 128, seed=7)
    i2, j2 = F.unpack_nbit(p2["indices_packed"].cpu(), b, 256), F.unpack_nbit(r2["indices_packed"], b, 256)
    assert (i2 != j2).float().mean() < 2e-4
    with pytest.raises(ValueError):
        K.quantize_packed_full(W2, 3)


def test_zz_tensor_core_status_word_is_clean():
    """No bounded wait of the tcgen05 kernels ran out during this session."""
    import ctypes
    st = ctypes.c_int32(-1)
    _lib.check(_lib.load().dmoq_tc_status(ctypes.byref(st)), "dmoq_tc_status")
    assert st.value == 0
