"""CPU-side checks: packed-format host logic vs the oracle and the goldens, C-ABI symbols, module plumbing."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

import dmoq_oracle as O
import dartmoq_b200 as D
from dartmoq_b200 import _lib, format as F, synth
from helpers import to_oracle_layer

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BITS = (1, 2, 4, 8)


@pytest.mark.parametrize("b", BITS)
def test_format_matches_reference_goldens(golden, b):
    g = golden("quantizer")
    W = torch.from_numpy(g["W"])
    pk = F.turboquant_quantize_packed_full(W, b, 128, seed=42 + b)
    assert np.array_equal(pk["indices_packed"].numpy(), g[f"idx_{b}"])
    assert np.array_equal(pk["norms"].numpy(), g[f"norms_{b}"])
    assert np.array_equal(pk["codebook"].numpy(), g[f"cb_{b}"])
    assert np.array_equal(F.turboquant_dequantize_packed(dict(pk, orig_dtype="torch.float32")).numpy(), g[f"deq_{b}"])
    gi, gn = F.convert_to_group_first(pk["indices_packed"], pk["norms"], 128, b)
    assert np.array_equal(gi.numpy(), g[f"gf_idx_{b}"]) and np.array_equal(gn.numpy(), g[f"gf_norms_{b}"])
    lut, step = F.build_int8_codebook(pk["codebook"])
    assert np.array_equal(lut.numpy(), g[f"i8_lut_{b}"]) and step == float(g[f"i8_step_{b}"])
    lut, sc = F.build_fp8_codebook(pk["codebook"])
    assert np.array_equal(lut.view(torch.uint8).numpy(), g[f"f8_lut_{b}"]) and sc == float(g[f"f8_scale_{b}"])
    if b != 8:
        nib, e0, resid, _ = F.build_e2m1_codebook(pk["codebook"])
        assert np.array_equal(nib.numpy(), g[f"f4_nib_{b}"]) and e0 == int(g[f"f4_e0_{b}"])
        assert float(resid) == float(g[f"f4_resid_{b}"])
        assert np.array_equal(F.fold_indices_to_e2m1(gi, nib, b, 128).numpy(), g[f"f4_fold_{b}"])


def test_pack_roundtrip_and_edges(golden):
    g = golden("format")
    for b in BITS:
        idx = torch.from_numpy(g[f"pack_in_{b}"])
        p = F.pack_nbit(idx, b)
        assert np.array_equal(p.numpy(), g[f"pack_out_{b}"])
        assert np.array_equal(F.unpack_nbit(p, b, 45).numpy(), g[f"unpack_{b}"])
        assert np.array_equal(O.pack_nbit(idx.numpy(), b), p.numpy())
    assert F.pack_nbit(torch.zeros(2, 0, dtype=torch.long), 2).shape == (2, 0)       # empty
    ragged = torch.arange(7) % 4
    assert F.unpack_nbit(F.pack_nbit(ragged, 2), 2, 7).tolist() == ragged.tolist()    # padded tail
    with pytest.raises(ValueError):
        F.pack_nbit(ragged, 3)
    with pytest.raises(ValueError):
        F.turboquant_quantize_packed_full(torch.zeros(4, 128), 4, 128, uniform_codebook=True)
    assert np.array_equal(F.generate_rotation_matrix(128, 43).numpy(), g["rot_43"])
    assert np.array_equal(F.generate_batch_rotation_matrices(128, 1044, 2, 128, "cpu").numpy(), g["rot_1044_stack_f16"])
    assert F.is_uniform_codebook(F.uniform8_codebook()[0].half()) and not F.is_uniform_codebook(F.get_codebook(8)[0].half())


def test_capi_exports_every_declared_symbol():
    """libdmoq.so loads here (no GPU needed) and exports each function include/dmoq.h declares."""
    header = open(os.path.join(ROOT, "include", "dmoq.h")).read()
    declared = set(re.findall(r"^(?:int|size_t|const char\*)\s+(dmoq_\w+)\s*\(", header, flags=re.M))
    assert declared and declared == set(_lib.EXPORTS), declared ^ set(_lib.EXPORTS)
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for name in declared:
        assert hasattr(lib, name), name
    loaded = _lib.load()
    assert loaded.dmoq_version() == 100
    assert loaded.dmoq_strerror(-1).decode() == "invalid argument"
    assert loaded.dmoq_route_workspace_bytes(64, 8, 256) >= 257 * 4
    # argument validation happens before any CUDA call
    assert loaded.dmoq_combine(None, None, 128, None, 1, None) == -1
    assert loaded.dmoq_convert_group_first(None, 1, 128, 3, None, None) == -1


def test_struct_layout_matches_header():
    """ctypes mirrors have the field order and sizes of the C structs (pointers 8 bytes, ints 4)."""
    assert ctypes.sizeof(_lib.Pool) == 6 * 4 + 6 * 8 + 3 * 4 + 2 * 4 + 4 + 4 * 8 + 2 * 8 + 4 * 8  # includes 4 bytes of padding
    assert ctypes.sizeof(_lib.Route) == 6 * 4 + 12 * 8 + 4 + 4 + 8


def test_module_state_dict_keys_and_mode_switch():
    moe = synth.build_layer(hidden=256, n_experts=6, top_k=2, inter=128, bit_mix={2: 0.6, 4: 0.4}, shared_inter=128)
    keys = set(moe.state_dict().keys())
    want = {"gate.weight", "shared_expert_gate.weight"}
    for p in ("gate_proj", "up_proj", "down_proj"):
        want |= {f"shared_expert.{p}.{k}" for k in ("packed_indices", "norms", "codebook")}
    for b in ("4", "2"):
        for side in ("gate_up", "down"):
            want |= {f"bit_weights.{b}.{side}_{k}" for k in ("indices_packed", "codebook", "norms")}
    assert keys == want
    for cls in (D.WxA8BitPartitionedGroupMoE, D.WxFP8BitPartitionedGroupMoE, D.WxFP4BitPartitionedGroupMoE):
        before = {k: v.data_ptr() for k, v in moe.state_dict().items()}
        assert cls.from_wxa16(moe) is moe and type(moe) is cls
        assert {k: v.data_ptr() for k, v in moe.state_dict().items()} == before   # zero copy
    assert moe._pool_mode(1) == _lib.FP4 and moe._pool_mode(2) == _lib.A8 and moe._pool_mode(4) == _lib.FP4
    with pytest.raises(TypeError):
        D.WxA8BitPartitionedGroupMoE.from_wxa16(torch.nn.Linear(2, 2))
    with pytest.raises(_lib.DmoqError):
        moe(torch.zeros(1, 2, 256, dtype=torch.bfloat16))     # no CPU path


def test_from_metadata_roundtrip():
    """A module rebuilt from metadata + state_dict(assign=True) carries the same tensors (checkpoint load path)."""
    src = synth.build_layer(hidden=256, n_experts=4, top_k=2, inter=128, bit_mix={2: 0.5, 1: 0.5})
    meta = {"num_experts": 4, "hidden_size": 256, "intermediate_size": 128, "top_k": 2, "bit_list": src.bit_list,
            "inter_size_by_bit": {str(k): v for k, v in src.inter_size_by_bit.items()},
            "expert_offsets": {k: v.tolist() for k, v in src.expert_offsets.items()}, "bits": {}}
    for bs, w in src.bit_weights.items():
        meta["bits"][bs] = {}
        for side, pk in (("gate_up", w.gate_up_packed), ("down", w.down_packed)):
            meta["bits"][bs][side] = {"seed": pk["seed"], "group_size": pk["group_size"], "shape": list(pk["shape"]),
                                      "bit_width": pk["bit_width"], "rotation": pk["rotation"],
                                      "orig_dtype": pk["orig_dtype"],
                                      "indices_packed_shape": list(pk["indices_packed"].shape),
                                      "codebook_shape": list(pk["codebook"].shape), "norms_shape": list(pk["norms"].shape)}
    dst = D.WxA16BitPartitionedGroupMoE.from_metadata(meta, src.gate, None, None)
    dst.load_state_dict(src.state_dict(), strict=True, assign=True)
    for bs in src.bit_weights:
        a, b = src.bit_weights[bs].gate_up_packed, dst.bit_weights[bs].gate_up_packed
        assert torch.equal(a["indices_packed"], b["indices_packed"]) and a["seed"] == b["seed"]
    la, lb = to_oracle_layer(src), to_oracle_layer(dst)
    assert [p["members"] for p in la.pools] == [p["members"] for p in lb.pools]


def test_synthetic_bit_assignment_and_router():
    bits = synth.assign_bits(256, {2: 0.98, 1: 0.01, 4: 0.01}, seed=1234)
    assert sorted(set(bits)) == [1, 2, 4] and bits.count(1) == 3 and bits.count(4) == 3
    r = synth.SyntheticRouter(64, 16, 4, seed=3)
    _, w, idx = r(torch.zeros(10, 64, dtype=torch.bfloat16))
    assert w.dtype == torch.float32 and torch.allclose(w.sum(-1), torch.ones(10)) and idx.shape == (10, 4)
    x = synth.make_activations(32, 256, seed=1)
    assert x.dtype == torch.bfloat16 and float(x.float().abs().max()) > 10
