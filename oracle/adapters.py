"""Glue between the product's modules and the CPU oracle.  TEST INFRASTRUCTURE ONLY (see dmoq_oracle.py).

Duck-types the module objects (it imports nothing from the product package): reads their packed
tensors into plain numpy so the oracle can recompute the layer.
"""
import numpy as np
import torch

import dmoq_oracle as O

MODE_OF = {0: "wxa16", 1: "wxa8", 2: "wxfp8", 3: "wxfp4"}


def _np_pack(pk: dict, bit: int) -> dict:
    idx = pk["indices_packed"].detach().cpu().numpy()
    norms = pk["norms"].detach().cpu().numpy()
    return {"indices_packed": idx, "norms": norms, "codebook": pk["codebook"].detach().cpu().numpy(),
            "seed": int(pk["seed"]), "bit_width": bit, "group_size": 128,
            "shape": (idx.shape[0], idx.shape[1] * 8 // bit)}


def to_oracle_layer(moe) -> "O.Layer":
    """Plain-numpy description of a product MoE module for the oracle."""
    pools = []
    for bs, w in moe.bit_weights.items():
        bit = int(bs)
        offs = moe._offsets_lists()[bs]
        members = [e for e in range(moe.num_experts) if offs[e + 1] > offs[e]]
        if not members:
            continue
        inter = offs[members[0] + 1] - offs[members[0]]
        pools.append(dict(key=bs, bit=bit, mode=MODE_OF[moe._pool_mode(bit)], members=members, inter=inter,
                          gu=_np_pack(w.gate_up_packed, bit), dn=_np_pack(w.down_packed, bit)))
    shared = None
    packs = moe._shared_packs()
    if packs is not None:
        gu, dn, bit, inter = packs
        shared = dict(key="shared", bit=bit, mode=MODE_OF[moe._pool_mode(bit, shared=True)], members=[0], inter=inter,
                      gu=_np_pack(gu, bit), dn=_np_pack(dn, bit))
    return O.Layer(moe.hidden_size, moe.num_experts, moe.top_k, pools, shared)


def routing(moe, x):
    """(topk_w fp32, topk_idx, shared_w or None) exactly as the module's forward derives them."""
    out = moe.gate(x)
    if isinstance(out, tuple):
        _, w, idx = out
    else:
        w, idx = out.softmax(dim=-1).topk(moe.top_k, dim=-1)
    sw = None
    if moe.shared_expert is not None and moe.shared_expert_gate is not None:
        sw = torch.sigmoid(moe.shared_expert_gate(x)).detach().reshape(-1).float().cpu().numpy()
    return w.detach().float().cpu().numpy(), idx.cpu().numpy(), sw


def rel_fro(a, b) -> float:
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))
