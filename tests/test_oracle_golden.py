"""The CPU oracle against vectors produced by running the reference (tests/golden/make_golden.py)."""
import numpy as np
import pytest
import torch

import dmoq_oracle as O
from helpers import rel_fro

BITS = (1, 2, 4, 8)


def test_pack_unpack_codebooks_rotation(golden):
    g = golden("format")
    for b in BITS:
        assert np.array_equal(O.pack_nbit(g[f"pack_in_{b}"], b), g[f"pack_out_{b}"])
        assert np.array_equal(O.unpack_nbit(g[f"pack_out_{b}"], b, 45), g[f"unpack_{b}"])
        c, e = O.lloyd_max(b)
        assert np.array_equal(c, g[f"cent_{b}"]) and np.array_equal(e, g[f"edges_{b}"])
    assert np.array_equal(O.rotation(128, 43), g["rot_43"])
    assert np.array_equal(O.rotation_stack_f16(1044, 2), g["rot_1044_stack_f16"])


@pytest.mark.parametrize("b", BITS)
def test_quantizer_dequantizer_luts(golden, b):
    g = golden("quantizer")
    pk = O.quantize_packed(g["W"], b, 42 + b)
    assert np.array_equal(pk["indices_packed"], g[f"idx_{b}"])
    assert np.array_equal(pk["norms"], g[f"norms_{b}"])
    assert np.array_equal(pk["codebook"], g[f"cb_{b}"])
    assert np.array_equal(O.dequantize_packed(pk), g[f"deq_{b}"])
    gi, gn = O.group_first(pk["indices_packed"], pk["norms"], b)
    assert np.array_equal(gi, g[f"gf_idx_{b}"]) and np.array_equal(gn, g[f"gf_norms_{b}"])
    lut, step = O.int8_lut(pk["codebook"])
    assert np.array_equal(lut, g[f"i8_lut_{b}"]) and step == float(g[f"i8_step_{b}"])
    lut, sc = O.fp8_lut(pk["codebook"])
    assert np.array_equal(lut, g[f"f8_lut_{b}"]) and sc == float(g[f"f8_scale_{b}"])
    if b != 8:
        nib, e0, resid = O.e2m1_lut(pk["codebook"])
        assert np.array_equal(nib, g[f"f4_nib_{b}"]) and e0 == int(g[f"f4_e0_{b}"])
        assert resid == float(g[f"f4_resid_{b}"])
        assert np.array_equal(O.fold_e2m1(gi, nib, b), g[f"f4_fold_{b}"])


def test_uniform_8bit_quantizer(golden):
    g = golden("quantizer")
    pk = O.quantize_packed(g["W"], 8, 7, uniform=True)
    assert np.array_equal(pk["indices_packed"], g["u8_idx"])
    assert np.array_equal(pk["norms"], g["u8_norms"]) and np.array_equal(pk["codebook"], g["u8_cb"])


def test_rotate_quantize_codes_bit_exact(golden):
    """int8 / e4m3 / e2m1 codes and stored scales of the reference's fused kernels (Triton interpreter)."""
    g = golden("actquant")
    acc = O.rotate_f32(g["x_f16"].astype(np.float32), g["rot_f16"])
    q, s = O.actquant_int8(acc, 0.0118956)
    assert np.array_equal(q, g["i8_q"]) and np.array_equal(s, g["i8_s"])
    q, s = O.actquant_e4m3(acc, 0.00472075)
    assert np.array_equal(q, g["f8_q"]) and np.array_equal(s, g["f8_s"])
    q, s = O.actquant_e2m1(acc)
    assert np.array_equal(q, g["f4_q_t"].T) and np.array_equal(s, g["f4_s"])
    # rotation only: the reference's bmm accumulates in fp16/fp32 in library order; values agree to fp16 rounding
    assert rel_fro(acc.astype(np.float16), g["rot_only_f16"]) < 2e-3


def _pool_tables(g, b):
    gu_i, gu_n = O.group_first(g[f"gu_idx_{b}"], g[f"gu_norms_{b}"], b)
    dn_i, dn_n = O.group_first(g[f"dn_idx_{b}"], g[f"dn_norms_{b}"], b)
    pre = lambda n: (n.astype(np.float32) / np.float32(np.sqrt(128.0))).astype(np.float16)
    return gu_i, pre(gu_n), dn_i, pre(dn_n)


def _segments(counts, inter):
    segs, cur = [], 0
    for e, n in enumerate(counts):
        if n:
            segs.append((e, cur, int(n)))
            cur += int(n)
    return segs


@pytest.mark.parametrize("b", (1, 2, 4))
def test_merged_gemm_all_modes(golden, b):
    """Per-pool grouped GEMMs: A8 outputs bit-exact, A16/FP8/FP4 within the path's tolerances."""
    g = golden("merged_gemm")
    H = I = 256
    gu_i, gu_n, dn_i, dn_n = _pool_tables(g, b)
    segs = _segments(g["counts"], I)
    cb = g[f"cb_{b}"]
    x, a = g[f"x_{b}"].astype(np.float32), g[f"a_{b}"].astype(np.float32)
    rot_gu = O.rotation_stack_f16(42 + b, H // 128)
    acc_x = O.rotate_f32(x, rot_gu)

    def rot_dn(e):
        return O.rotation_stack_f16(42 + b + 1000 + e * I, I // 128)

    def run(mode, side):
        outs = []
        table, extra, e0, f = O._mode_consts(mode, b, cb)
        for e, r0, n in segs:
            if side == "gu":
                acc = acc_x[r0:r0 + n]
                w_idx = O.weight_codes(gu_i, b, slice(2 * I * e, 2 * I * (e + 1)), slice(0, H // 128))
                norm = gu_n[:, 2 * I * e:2 * I * (e + 1)]
            else:
                acc = O.rotate_f32(a[r0:r0 + n], rot_dn(e))
                w_idx = O.weight_codes(dn_i, b, slice(0, H), slice(e * I // 128, (e + 1) * I // 128))
                norm = dn_n[e * I // 128:(e + 1) * I // 128]
            if f != 1.0:
                norm = (norm.astype(np.float32) * np.float32(f)).astype(np.float16)
            vals, rs, block, codes, scales = O._quant_act(mode, acc, extra, e0)
            o, _ = O._pool_gemm(mode, vals, rs, block, w_idx, table, norm)
            outs.append((o, codes, scales))
        return outs

    o = run("wxa8", "gu")
    assert np.array_equal(np.concatenate([t[1] for t in o]), g[f"a8_xq_{b}"])
    assert np.array_equal(np.concatenate([t[2] for t in o]), g[f"a8_xs_{b}"])
    assert np.array_equal(np.concatenate([t[0] for t in o]), g[f"a8_gu_{b}"])
    o = run("wxa8", "dn")
    assert np.array_equal(np.concatenate([t[1] for t in o]), g[f"a8_aq_{b}"])
    assert np.array_equal(np.concatenate([t[2] for t in o]), g[f"a8_as_{b}"])
    assert np.array_equal(np.concatenate([t[0] for t in o]), g[f"a8_dn_{b}"])
    for mode, key, tol in (("wxa16", "a16", 1e-2), ("wxfp8", "f8", 2e-2), ("wxfp4", "f4", 2e-2)):
        for side in ("gu", "dn"):
            got = np.concatenate([t[0] for t in run(mode, side)])
            assert rel_fro(got, g[f"{key}_{side}_{b}"]) < tol, (mode, side)
    o = run("wxfp4", "gu")
    assert np.array_equal(np.concatenate([t[1] for t in o]), g[f"f4_xq_{b}"])
    assert np.array_equal(np.concatenate([t[2] for t in o]), g[f"f4_xs_{b}"])


def _module_layer(g, mode):
    bits_of = list(g["bits_of"])
    pools = []
    for bit in sorted(set(bits_of), reverse=True):
        members = [e for e in range(len(bits_of)) if bits_of[e] == bit]
        mk = lambda side, seed: dict(indices_packed=g[f"{side}_idx_{bit}"], norms=g[f"{side}_norms_{bit}"],
                                     codebook=g[f"cb_{bit}"], seed=seed, bit_width=bit, group_size=128,
                                     shape=(g[f"{side}_norms_{bit}"].shape[0], g[f"{side}_norms_{bit}"].shape[1] * 128))
        pools.append(dict(key=str(bit), bit=bit, mode=mode, members=members, inter=256,
                          gu=mk("gu", 42 + bit), dn=mk("dn", 42 + bit + 1000)))
    return O.Layer(256, len(bits_of), 2, pools)


@pytest.mark.parametrize("mode,key,tol", [("wxa16", "y_a16", 1e-2), ("wxa8", "y_a8", 1e-2), ("wxfp8", "y_fp8", 2e-2)])
def test_module_forward_vs_reference_modules(golden, mode, key, tol):
    """Whole-layer forward of the reference modules (CPU, Triton interpreter) vs the oracle restatement."""
    g = golden("module")
    layer = _module_layer(g, mode)
    x = torch.from_numpy(g["x"])
    res = O.moe_forward(layer, x, g["topk_w"], g["topk_idx"])
    assert rel_fro(res["y_bf16seq"] if False else res["y"], g[key]) < tol


def test_dequant_matmul_baseline_vs_reference(golden):
    g = golden("module")
    layer = _module_layer(g, "wxa16")
    x = torch.from_numpy(g["x"])
    y = O.dequant_matmul_forward(layer, x, g["topk_w"], g["topk_idx"], dtype=torch.float16)
    assert rel_fro(y, g["y_dequant_fp16"]) < 2e-3
    # and every quantised mode approximates that dense answer
    for mode, tol in (("wxa16", 1e-2), ("wxa8", 3e-2), ("wxfp8", 8e-2)):
        res = O.moe_forward(_module_layer(g, mode), x, g["topk_w"], g["topk_idx"])
        assert rel_fro(res["y"], g["y_dequant_fp16"]) < tol, mode
