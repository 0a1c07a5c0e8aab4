"""Expert-parallel exchange logic on CPU ranks (gloo, world_size 2): dispatch, owner compute, return, combine."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from dartmoq_b200 import ep
    E, k, T, H = 8, 3, 11 + rank, 6
    g = torch.Generator().manual_seed(100 + rank)
    x = torch.randn(T, H, generator=g)
    idx = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)])
    if rank == 0:
        idx[:, 0] = 5                     # skew: everything also goes to one remote expert
    w = torch.rand(T, k, generator=g)
    per_rank = E // world

    def local_compute(rows, local_expert, weight):
        # stand-in expert: scale by (global expert id + 1) and the routing weight
        ge = (local_expert + rank * per_rank + 1).to(rows.dtype)
        return rows * ge.unsqueeze(1) * weight.unsqueeze(1)

    y = ep.ep_forward(x, w, idx, per_rank, local_compute)
    want = torch.zeros(T, H)
    for s in range(k):
        want = want + x * (idx[:, s] + 1).float().unsqueeze(1) * w[:, s].unsqueeze(1)
    np.save(os.path.join(out_dir, f"ok_{rank}.npy"), np.array([torch.allclose(y, want, rtol=1e-5, atol=1e-6)]))
    # empty batch on one rank must not hang the exchange
    xe = x[:0] if rank == 1 else x
    ie = idx[:0] if rank == 1 else idx
    we = w[:0] if rank == 1 else w
    ye = ep.ep_forward(xe, we, ie, per_rank, local_compute)
    np.save(os.path.join(out_dir, f"empty_{rank}.npy"), np.array([ye.shape[0] == xe.shape[0]]))
    # token-gather exchange: every rank sees all tokens, computes its own experts' share, partials summed in rank order
    def local_partial(x_all, w_all, local_idx):
        ge = (local_idx + rank * per_rank + 1).to(x_all.dtype)
        coef = torch.where(local_idx >= 0, ge * w_all, torch.zeros_like(w_all)).sum(1)
        return x_all * coef.unsqueeze(1)

    yg = ep.ep_forward_gathered(x, w, idx, per_rank, local_partial)
    yx = ep.ep_forward_gathered(x, w, idx, per_rank, local_partial, extra=0.5 * x)   # one more partial per token
    ok_g = torch.allclose(yg, want, rtol=1e-5, atol=1e-6) and torch.allclose(yx, want + 0.5 * x, rtol=1e-5, atol=1e-6)
    np.save(os.path.join(out_dir, f"gather_{rank}.npy"), np.array([ok_g]))
    yge = ep.ep_forward_gathered(xe, we, ie, per_rank, local_partial)
    ok_e = yge.shape[0] == xe.shape[0] and (rank == 1 or torch.allclose(yge, want, rtol=1e-5, atol=1e-6))
    np.save(os.path.join(out_dir, f"gather_empty_{rank}.npy"), np.array([ok_e]))
    dist.destroy_process_group()


def test_ep_forward_two_cpu_ranks(tmp_path):
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        assert np.load(tmp_path / f"ok_{r}.npy")[0]
        assert np.load(tmp_path / f"empty_{r}.npy")[0]
        assert np.load(tmp_path / f"gather_{r}.npy")[0]
        assert np.load(tmp_path / f"gather_empty_{r}.npy")[0]


def test_dispatch_plan_is_a_stable_permutation():
    sys.path.insert(0, ROOT)
    from dartmoq_b200 import ep
    idx = torch.tensor([[3, 0], [1, 2], [0, 3], [2, 2]])
    plan = ep.DispatchPlan(idx, experts_per_rank=2, world=2)
    assert plan.send_counts.tolist() == [3, 5]
    assert plan.order.tolist() == [1, 2, 4, 0, 3, 5, 6, 7]          # rank 0 pairs first, flat order kept
    assert plan.local_expert.tolist() == [0, 1, 0, 1, 0, 1, 0, 0]
    assert plan.inverse()[plan.order].tolist() == list(range(8))


def test_shard_experts_slices_the_packed_pools():
    sys.path.insert(0, ROOT)
    from dartmoq_b200 import ep, synth
    moe = synth.build_layer(hidden=256, n_experts=8, top_k=2, inter=128, bit_mix={2: 0.5, 4: 0.5}, mode="wxa8", seed=3)
    offs = moe._offsets_lists()
    parts = [ep.shard_experts(moe, 0, 4), ep.shard_experts(moe, 4, 8)]
    for bs, w in moe.bit_weights.items():
        gu = torch.cat([p.bit_weights[bs].gate_up_packed["indices_packed"] for p in parts if bs in p.bit_weights])
        dn = torch.cat([p.bit_weights[bs].down_packed["indices_packed"] for p in parts if bs in p.bit_weights], 1)
        assert torch.equal(gu, w.gate_up_packed["indices_packed"]) and torch.equal(dn, w.down_packed["indices_packed"])
        for i, p in enumerate(parts):
            if bs in p.bit_weights:
                assert p.bit_weights[bs].down_packed["seed"] == w.down_packed["seed"] + offs[bs][4 * i]
                assert p._offsets_lists()[bs][-1] == offs[bs][4 * i + 4] - offs[bs][4 * i]
    assert type(parts[0]) is type(moe) and parts[0].top_k == 1 and parts[0].num_experts == 4
    assert ep.shard_experts(moe, 0, 4, top_k=2).top_k == 2


def test_owner_tile_plan_covers_every_received_row_once():
    """The owner's tile lists, built from the (source, expert) count matrix: every received row is covered exactly
    once, by a tile of its own expert in that expert's pool, inside one (source, expert) segment."""
    sys.path.insert(0, ROOT)
    from dartmoq_b200.ep_codes import owner_tiles
    rng = np.random.default_rng(3)
    n_src, e_loc = 4, 9
    counts = rng.integers(0, 400, size=(n_src, e_loc))
    counts[1, :] = 0                       # a source with an empty batch
    counts[:, 4] = 0                       # an expert nobody routed to
    pool_of = np.array([0, 1, 0, 2, 0, 1, 1, 0, 2])
    rank_of = np.array([0, 0, 1, 0, 2, 1, 2, 3, 1])
    tiles, n_tiles = owner_tiles(counts, pool_of, rank_of, 3)
    total = int(counts.sum())
    cover = np.zeros(total, np.int32)
    starts = np.concatenate([[0], np.cumsum(counts.reshape(-1))])
    for p in range(3):
        n, base = n_tiles[p], n_tiles[8 + p]
        for e, row0, rows, rank in tiles[base:base + n]:
            assert pool_of[e] == p and rank == rank_of[e] and 0 < rows <= 128
            seg = np.searchsorted(starts, row0, side="right") - 1          # the (source, expert) segment of row0
            assert seg % e_loc == e and row0 + rows <= starts[seg + 1]
            cover[row0:row0 + rows] += 1
    assert (cover == 1).all() and n_tiles[:3].sum() == tiles.shape[0]
    empty, n0 = owner_tiles(np.zeros((2, 3), np.int64), np.array([0, 0, 1]), np.array([0, 1, 0]), 2)
    assert empty.shape == (0, 4) and n0.sum() == 0
