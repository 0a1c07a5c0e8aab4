"""Generate the golden fixtures by RUNNING THE REFERENCE in the build container.

Usage (needs the reference checkout; it is not available where the GPU tests run):

    TRITON_INTERPRET=1 PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py /path/to/reference

Everything stored in ``tests/golden/*.npz`` is an input/output pair of the reference's own
functions: its torch format helpers on the CPU, and its Triton kernels executed by the Triton CPU
interpreter (IEEE arithmetic).  Two harness-side substitutions are made for gaps of the
interpreter, not of the reference: the int8 activation-quantisation kernel calls ``libdevice.round``,
which the interpreter lacks (an exact round-half-away-from-zero helper is patched in), and the
interpreter's fp32 -> e4m3 down-cast mishandles the mantissa carry (torch's round-to-nearest-even
saturating conversion, which is what the hardware instruction does, is patched in).  The whole-module goldens run the reference modules' ``forward`` on the CPU.
The reference's FP4 GEMM kernels (``tl.dot_scaled``) do not run in the interpreter, so the FP4 GEMM
golden is built from the reference's own torch operand builders plus a float64 evaluation of the
kernel's documented formula.
"""
import os
import sys

os.environ.setdefault("TRITON_INTERPRET", "1")
os.environ.setdefault("PYTHONDONTWRITEBYTECODE", "1")
REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("DARTMOQ_REFERENCE", "")
if not os.path.isdir(REF):
    sys.exit("usage: make_golden.py <checkout of the reference>   (or set DARTMOQ_REFERENCE)")
sys.path.insert(0, REF)
OUT = os.path.dirname(os.path.abspath(__file__))

import numpy as np  # noqa: E402
import torch  # noqa: E402
import triton  # noqa: E402
import triton.language as tl  # noqa: E402

import turboquant_utils  # noqa: E402,F401
from turboquant_utils import codebook as r_cb  # noqa: E402
from turboquant_utils import quantize as r_q  # noqa: E402
from turboquant_utils import rotation as r_rot  # noqa: E402
from turboquant_utils import triton_kernels as r_k16  # noqa: E402
from turboquant_utils import triton_kernels_a8 as r_k8  # noqa: E402
from turboquant_utils import triton_kernels_fp4 as r_kf4  # noqa: E402
from turboquant_utils import triton_kernels_fp8 as r_kf8  # noqa: E402


@triton.jit
def _round_half_away(x):
    t = tl.where(x >= 0, tl.floor(x), tl.ceil(x))
    d = tl.abs(x - t)
    return t + tl.where(d >= 0.5, tl.where(x >= 0, 1.0, -1.0), 0.0)


tl.extra.cuda.libdevice.round = _round_half_away

# The interpreter's software fp32 -> fp8e4nv down-cast drops the carry when the mantissa rounds up to
# the next power of two (31.6 becomes 16 instead of 32).  The reference's kernel means the hardware
# conversion (round-to-nearest-even, saturating), so that case is routed through torch's conversion.
import triton.runtime.interpreter as _interp  # noqa: E402

_orig_convert_float = _interp._convert_float


def _convert_float_fixed(inp, input_dtype, output_dtype, rounding_mode):
    if input_dtype == tl.float32 and output_dtype == tl.float8e4nv:
        t = torch.from_numpy(np.ascontiguousarray(inp, np.float32)).clamp(-448.0, 448.0)
        return t.to(torch.float8_e4m3fn).view(torch.uint8).numpy().reshape(inp.shape)
    return _orig_convert_float(inp, input_dtype, output_dtype, rounding_mode)


_interp._convert_float = _convert_float_fixed


def save(name, **arrays):
    path = os.path.join(OUT, name + ".npz")
    np.savez_compressed(path, **{k: np.asarray(v) for k, v in arrays.items()})
    print(f"{name}: {os.path.getsize(path) / 1024:.1f} KiB")


def u8(t):
    return t.view(torch.uint8).numpy() if t.dtype == torch.float8_e4m3fn else t.numpy()


def gen_format():
    out = {}
    g = torch.Generator().manual_seed(11)
    for b in (1, 2, 4, 8):
        idx = torch.randint(0, 2 ** b, (3, 45), generator=g)
        out[f"pack_in_{b}"] = idx.numpy()
        out[f"pack_out_{b}"] = r_q.pack_nbit(idx, b).numpy()
        out[f"unpack_{b}"] = r_q.unpack_nbit(r_q.pack_nbit(idx, b), b, 45).numpy()
        c, e = r_cb.get_codebook(b)
        out[f"cent_{b}"], out[f"edges_{b}"] = c.numpy(), e.numpy()
    out["rot_43"] = r_rot.generate_rotation_matrix(128, 43).numpy()
    out["rot_1044_stack_f16"] = r_rot.generate_batch_rotation_matrices(128, 1044, 2, 128, "cpu", torch.float16).numpy()
    save("format", **out)


def gen_quantizer():
    out = {}
    g = torch.Generator().manual_seed(12)
    W = torch.randn(48, 256, generator=g) * 0.02
    out["W"] = W.numpy()
    for b in (1, 2, 4, 8):
        pk = r_q.turboquant_quantize_packed_full(W, b, 128, seed=42 + b)
        out[f"idx_{b}"], out[f"norms_{b}"], out[f"cb_{b}"] = pk["indices_packed"].numpy(), pk["norms"].numpy(), pk["codebook"].numpy()
        out[f"deq_{b}"] = r_q.turboquant_dequantize_packed(dict(pk, orig_dtype="torch.float32")).numpy()
        gf_i, gf_n = r_k16.convert_to_group_first(pk["indices_packed"], pk["norms"], 128, b)
        out[f"gf_idx_{b}"], out[f"gf_norms_{b}"] = gf_i.numpy(), gf_n.numpy()
        lut, step = r_k8.build_int8_codebook(pk["codebook"])
        out[f"i8_lut_{b}"], out[f"i8_step_{b}"] = lut.numpy(), np.float64(step)
        lut, sc = r_kf8.build_fp8_codebook(pk["codebook"])
        out[f"f8_lut_{b}"], out[f"f8_scale_{b}"] = u8(lut), np.float64(sc)
        if b != 8:
            nib, e0, resid, _ = r_kf4.build_e2m1_codebook(pk["codebook"])
            out[f"f4_nib_{b}"], out[f"f4_e0_{b}"], out[f"f4_resid_{b}"] = nib.numpy(), np.int64(e0), np.float64(float(resid))
            out[f"f4_fold_{b}"] = r_kf4.fold_indices_to_e2m1(gf_i, nib, b, 128).numpy()
    pk = r_q.turboquant_quantize_packed_full(W, 8, 128, seed=7, uniform_codebook=True)
    out["u8_idx"], out["u8_norms"], out["u8_cb"] = pk["indices_packed"].numpy(), pk["norms"].numpy(), pk["codebook"].numpy()
    save("quantizer", **out)


def gen_actquant():
    out = {}
    g = torch.Generator().manual_seed(13)
    x = torch.randn(37, 256, generator=g)
    x[:, 5] *= 20.0
    x[3] *= 1e-4
    x[4] = 0.0
    xh = x.to(torch.bfloat16).half()
    rot = r_rot.generate_batch_rotation_matrices(128, 44, 2, 128, "cpu", torch.float16)
    out["x_f16"], out["rot_f16"] = xh.numpy(), rot.numpy()
    q, s = r_k8.rotate_quantize_fused(xh, rot, 128, 2, extra_scale=0.0118956)
    out["i8_q"], out["i8_s"] = q.numpy(), s.numpy()
    q, s = r_kf8.rotate_quantize_fused_fp8(xh, rot, 128, 2, extra_scale=0.00472075)
    out["f8_q"], out["f8_s"] = u8(q), s.numpy()
    q, s = r_kf4.rotate_quantize_fused_fp4(xh, rot, 128, 2)
    out["f4_q_t"], out["f4_s"] = q.numpy(), s.numpy()
    out["rot_only_f16"] = r_rot.batch_rotate_input(xh, 128, 44).numpy()
    save("actquant", **out)


def gen_merged_gemm():
    """Merged (per-pool grouped) GEMM wrappers on a 3-expert pool, hidden 256, inter 256."""
    out = {}
    H, I, n_exp = 256, 256, 3
    g = torch.Generator().manual_seed(14)
    counts = [5, 0, 9]
    info_rows, info_groups, cur = [], [], 0
    for e, n in enumerate(counts):
        if n:
            info_rows.append((cur, n, 2 * I * e, 2 * I))
            info_groups.append((cur, n, e * I // 128, I // 128))
            cur += n
    B = cur
    out["counts"] = np.array(counts)
    for b in (1, 2, 4):
        Wgu = torch.randn(2 * I * n_exp, H, generator=g) * 0.02
        Wdn = torch.randn(H, I * n_exp, generator=g) * 0.02
        gu = r_q.turboquant_quantize_packed_full(Wgu, b, 128, seed=42 + b)
        dn = r_q.turboquant_quantize_packed_full(Wdn, b, 128, seed=42 + b + 1000)
        gu_i, gu_n = r_k16.convert_to_group_first(gu["indices_packed"], gu["norms"], 128, b)
        dn_i, dn_n = r_k16.convert_to_group_first(dn["indices_packed"], dn["norms"], 128, b)
        gu_n, dn_n = gu_n / np.sqrt(128), dn_n / np.sqrt(128)   # fp16 / python float, as _build_group_first
        x = (torch.randn(B, H, generator=g)).half()
        a = (torch.randn(B, I, generator=g) * 0.05).half()
        rot_gu = r_rot.generate_batch_rotation_matrices(128, 42 + b, H // 128, 128, "cpu", torch.float16)
        for k, v in dict(gu_idx=gu["indices_packed"], gu_norms=gu["norms"], dn_idx=dn["indices_packed"],
                         dn_norms=dn["norms"], cb=gu["codebook"], x=x, a=a).items():
            out[f"{k}_{b}"] = v.numpy()
        # A16: rotated fp16 in, fp16 out
        x_rot = r_rot.batch_rotate_input(x, 128, 42 + b)
        out[f"a16_gu_{b}"] = r_k16.triton_fused_matmul_merged_rows_gf(
            x_rot, gu_i, gu["codebook"], gu_n, info_rows, 128, H, bit_width=b, norms_prescaled=True).numpy()
        a_parts = [r_rot.batch_rotate_input(a[s:s + n], 128, 42 + b + 1000 + g0 * 128) for s, n, g0, _ in info_groups]
        out[f"a16_dn_{b}"] = r_k16.triton_fused_matmul_merged_in_features_gf(
            torch.cat(a_parts), dn_i, dn["codebook"], dn_n, info_groups, 128, bit_width=b, norms_prescaled=True).numpy()
        # A8
        lut8, step = r_k8.build_int8_codebook(gu["codebook"])
        q, s = r_k8.rotate_quantize_fused(x, rot_gu, 128, H // 128, extra_scale=step)
        out[f"a8_xq_{b}"], out[f"a8_xs_{b}"] = q.numpy(), s.numpy()
        out[f"a8_gu_{b}"] = r_k8.wxa8_matmul_merged_rows_gf(q, s, gu_i, lut8, gu_n, info_rows, 128, H, bit_width=b).numpy()
        qs, ss = [], []
        for s0, n, g0, _ in info_groups:
            rot = r_rot.generate_batch_rotation_matrices(128, 42 + b + 1000 + g0 * 128, I // 128, 128, "cpu", torch.float16)
            q2, s2 = r_k8.rotate_quantize_fused(a[s0:s0 + n], rot, 128, I // 128, extra_scale=step)
            qs.append(q2), ss.append(s2)
        out[f"a8_aq_{b}"], out[f"a8_as_{b}"] = torch.cat(qs).numpy(), torch.cat(ss).numpy()
        out[f"a8_dn_{b}"] = r_k8.wxa8_matmul_merged_in_features_gf(
            torch.cat(qs), torch.cat(ss), dn_i, lut8, dn_n, info_groups, 128, bit_width=b).numpy()
        # FP8
        lutf, sc = r_kf8.build_fp8_codebook(gu["codebook"])
        q, s = r_kf8.rotate_quantize_fused_fp8(x, rot_gu, 128, H // 128, extra_scale=sc)
        out[f"f8_gu_{b}"] = r_kf8.wxfp8_matmul_merged_rows_gf(q, s, gu_i, lutf, gu_n, info_rows, 128, H, bit_width=b).numpy()
        qs, ss = [], []
        for s0, n, g0, _ in info_groups:
            rot = r_rot.generate_batch_rotation_matrices(128, 42 + b + 1000 + g0 * 128, I // 128, 128, "cpu", torch.float16)
            q2, s2 = r_kf8.rotate_quantize_fused_fp8(a[s0:s0 + n], rot, 128, I // 128, extra_scale=sc)
            qs.append(q2), ss.append(s2)
        out[f"f8_dn_{b}"] = r_kf8.wxfp8_matmul_merged_in_features_gf(
            torch.cat(qs), torch.cat(ss), dn_i, lutf, dn_n, info_groups, 128, bit_width=b).numpy()
        # FP4: operands by the reference's torch builders; the kernel formula
        #   out[b,n] = sum_g norm'[g,n] * sum_k (e2m1(a)*2^(as-127)) * (e2m1(w)*2^E0)     in float64
        nib, e0, resid, _ = r_kf4.build_e2m1_codebook(gu["codebook"])
        grid = torch.tensor(r_kf4.E2M1_GRID, dtype=torch.float64)

        def nib_val(nb):
            return grid[(nb & 7).long()] * torch.where((nb & 8) > 0, -1.0, 1.0)

        out[f"f4_gu_{b}"], out[f"f4_xq_{b}"], out[f"f4_xs_{b}"] = _fp4(
            x, [(s0, n, rot_gu, (0, H // 128), (c0, c0 + 2 * I)) for s0, n, c0, _ in info_rows],
            gu_i, gu_n, nib, e0, resid, b, nib_val)
        out[f"f4_dn_{b}"], out[f"f4_aq_{b}"], out[f"f4_as_{b}"] = _fp4(
            a, [(s0, n, r_rot.generate_batch_rotation_matrices(128, 42 + b + 1000 + g0 * 128, I // 128, 128, "cpu", torch.float16),
                 (g0, g0 + I // 128), (0, H)) for s0, n, g0, _ in info_groups], dn_i, dn_n, nib, e0, resid, b, nib_val)
        out[f"f4_e0_{b}"] = np.int64(e0)
    save("merged_gemm", **out)


def _fp4(xin, segs, idx_gf, norms_gf, nib, e0, resid, b, nib_val):
    """float64 evaluation of the wxfp4 merged kernel formula on operands built by the reference's torch helpers."""
    outs, pqs, pss = [], [], []
    nrm = (norms_gf.float() * resid).half().double()
    for s0, n, rot, (g_lo, g_hi), (r_lo, r_hi) in segs:
        xr = torch.bmm(xin[s0:s0 + n].float().reshape(n, -1, 128).transpose(0, 1), rot.float().transpose(1, 2))
        xr = xr.transpose(0, 1).reshape(n, -1)
        pq, ps = r_kf4.quantize_act_e2m1_per32(xr)
        nibs = torch.stack([pq & 15, pq >> 4], -1).reshape(n, -1)
        av = (nib_val(nibs).reshape(n, -1, 32) * torch.pow(2.0, ps.double() - 127).unsqueeze(-1)).reshape(n, -1, 128)
        sub = idx_gf[g_lo:g_hi, r_lo:r_hi]
        widx = r_q.unpack_nbit(sub.reshape(-1, sub.shape[2]), b, 128)
        wv = nib_val(nib[widx.long()]).reshape(g_hi - g_lo, r_hi - r_lo, 128) * (2.0 ** e0)
        outs.append(torch.einsum("bgk,gnk,gn->bn", av, wv, nrm[g_lo:g_hi, r_lo:r_hi]))
        pqs.append(pq), pss.append(ps)
    return torch.cat(outs).float().numpy(), torch.cat(pqs).numpy(), torch.cat(pss).numpy()


def gen_module():
    """Whole-module forwards of the reference on the CPU (Triton interpreter) + its dequantize-then-matmul path."""
    from quantization.wxa16.bit_partitioned_moe import WxA16BitPartitionedGroupMoE, WxA16Weights
    from quantization.wxa8.bit_partitioned_moe import WxA8BitPartitionedGroupMoE
    from quantization.wxfp8.bit_partitioned_moe import WxFP8BitPartitionedGroupMoE
    from turboquant_utils.test_triton_mp_moe_e2e_bench import reference_forward_fp16
    import torch.nn as nn

    torch.cuda.synchronize = lambda *a, **k: None
    H, I, E, K, T = 256, 256, 6, 2, 24
    bits_of = [2, 2, 4, 2, 1, 2]
    g = torch.Generator().manual_seed(15)
    gate = nn.Linear(H, E, bias=False, dtype=torch.float16)
    gate.weight.data.copy_((torch.randn(E, H, generator=g) * 0.02).half())
    moe = WxA16BitPartitionedGroupMoE(gate=gate, num_experts=E, hidden_size=H, intermediate_size=I, top_k=K)
    moe.enable_timing = False
    out = {"bits_of": np.array(bits_of)}
    for bit in sorted(set(bits_of), reverse=True):
        mem = [e for e in range(E) if bits_of[e] == bit]
        Wgu = torch.randn(2 * I * len(mem), H, generator=g) * 0.02
        Wdn = torch.randn(H, I * len(mem), generator=g) * 0.02
        gu = r_q.turboquant_quantize_packed_full(Wgu, bit, 128, seed=42 + bit, keep_on_gpu=True)
        dn = r_q.turboquant_quantize_packed_full(Wdn, bit, 128, seed=42 + bit + 1000, keep_on_gpu=True)
        w = WxA16Weights(bit, H)
        w.set_packed_data(gu, dn)
        moe.bit_weights[str(bit)] = w
        offs, run = [0], 0
        for e in range(E):
            run += I if bits_of[e] == bit else 0
            offs.append(run)
        moe.expert_offsets[str(bit)] = torch.tensor(offs, dtype=torch.long)
        moe.inter_size_by_bit[bit] = I
        for k, v in dict(gu_idx=gu["indices_packed"], gu_norms=gu["norms"], dn_idx=dn["indices_packed"],
                         dn_norms=dn["norms"], cb=gu["codebook"]).items():
            out[f"{k}_{bit}"] = v.clone().numpy()
    moe.bit_list = sorted(set(bits_of), reverse=True)
    x = torch.randn(1, T, H, generator=g)
    x[..., 7] *= 20
    x = x.half()
    out["x"] = x[0].numpy()
    probs = gate(x[0]).softmax(dim=-1)
    tw, ti = probs.topk(K, dim=-1)
    out["topk_w"], out["topk_idx"] = tw.detach().float().numpy(), ti.numpy()
    with torch.no_grad():
        out["y_dequant_fp16"] = reference_forward_fp16(moe, x)[0].float().numpy()
        out["y_a16"] = moe(x)[0].float().numpy()
        WxA8BitPartitionedGroupMoE.from_wxa16(moe)
        out["y_a8"] = moe(x)[0].float().numpy()
        moe.__class__ = WxA16BitPartitionedGroupMoE
        moe._bit_ctx_cache = None
        WxFP8BitPartitionedGroupMoE.from_wxa16(moe)
        out["y_fp8"] = moe(x)[0].float().numpy()
    save("module", **out)


def gen_checkpoint():
    """The reference's own from_build_block (pool layout + quantisation) and save_quantized_model on a tiny model:
    staged fp16 sub-expert weights -> packed pools, and the meta.json / model.safetensors pair it writes."""
    import shutil
    import torch.nn as nn
    import qwen35_quant_io as r_io
    from quantization.wxa16.bit_partitioned_moe import WxA16BitPartitionedGroupMoE
    from quantization.wxa16.linear import WxA16Linear

    H, E = 128, 4
    g = torch.Generator().manual_seed(23)
    # neurons of every expert per bit width: expert 1 is split over two widths, expert 3 has no 4-bit part
    neurons = {0: {4: 128}, 1: {4: 128, 2: 128}, 2: {2: 256}, 3: {2: 128}}

    class Sub(nn.Module):
        def __init__(self, bit, n):
            super().__init__()
            self._quant_bit = bit
            self.gate_proj, self.up_proj = nn.Linear(H, n, bias=False), nn.Linear(H, n, bias=False)
            self.down_proj = nn.Linear(n, H, bias=False)
            for lin in (self.gate_proj, self.up_proj, self.down_proj):
                lin.weight.data.copy_(torch.randn(lin.weight.shape, generator=g) * 0.02)

    class Wrapper(nn.Module):
        def __init__(self, parts):
            super().__init__()
            self.sub_experts = nn.ModuleList([Sub(b, n) for b, n in parts.items()])

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.gate = nn.Linear(H, E, bias=False)
            self.top_k = 2
            self.experts = nn.ModuleList([Wrapper(neurons[e]) for e in range(E)])
            mk = lambda i, o: WxA16Linear.from_linear(nn.Linear(i, o, bias=False), 8, 128, seed=77, uniform_codebook=True)
            self.shared_expert = nn.Module()
            self.shared_expert.gate_proj, self.shared_expert.up_proj = mk(H, 128), mk(H, 128)
            self.shared_expert.down_proj = mk(128, H)
            self.shared_expert_gate = nn.Linear(H, 1, bias=False)

    torch.manual_seed(5)
    block = Block()
    out = {}
    for e in range(E):
        for sub in block.experts[e].sub_experts:
            for name in ("gate_proj", "up_proj", "down_proj"):
                out[f"w_{e}_{sub._quant_bit}_{name}"] = getattr(sub, name).weight.data.clone().numpy()
    md = {"num_experts": E, "hidden_size": H, "intermediate_size": 256, "bit_list": [4, 2],
          "expert_bit_indices": [{b: list(range(n)) for b, n in neurons[e].items()} for e in range(E)]}
    moe = WxA16BitPartitionedGroupMoE.from_build_block(block, md, group_size=128)
    for bs, w in moe.bit_weights.items():
        for side, pk in (("gate_up", w.gate_up_packed), ("down", w.down_packed)):
            for k in ("indices_packed", "norms", "codebook"):
                out[f"{side}_{k}_{bs}"] = u8(pk[k]) if pk[k].dtype == torch.uint8 else pk[k].clone().numpy()
            out[f"{side}_seed_{bs}"] = np.array(int(pk["seed"]))
        out[f"offsets_{bs}"] = moe.expert_offsets[bs].numpy()
    save("build_block", **out)

    class Layer(nn.Module):
        def __init__(self):
            super().__init__()
            self.mlp = moe
            self.self_attn = nn.Module()
            self.self_attn.q_proj = WxA16Linear.from_linear(nn.Linear(H, 256, bias=True), 8, 128, seed=78,
                                                             uniform_codebook=True)

    model = nn.Module()
    model.model = nn.Module()
    model.model.layers = nn.ModuleList([Layer()])
    ckpt = os.path.join(OUT, "ckpt_ref")
    shutil.rmtree(ckpt, ignore_errors=True)
    r_io.save_quantized_model(model, ckpt, base_model_path=None, quant_args={"seed": 0}, verbose=False)


if __name__ == "__main__":
    which = sys.argv[2:] or ["format", "quantizer", "actquant", "merged_gemm", "module", "checkpoint"]
    for name in which:
        globals()["gen_" + name]()
