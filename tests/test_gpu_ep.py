"""Expert parallelism on two GPUs (NCCL): the sharded layer equals the single-GPU layer on the same tokens
(bit for bit with the per-slot exchange, to bf16 rounding with the token-gather exchange)."""
import os
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out_dir):
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from dartmoq_b200 import ep, synth
    res = {}
    for mode in ("wxa8", "wxfp8", "wxa16"):
        full = synth.build_layer(hidden=256, n_experts=8, top_k=3, inter=256, bit_mix={2: 0.5, 1: 0.25, 4: 0.25},
                                 mode=mode, seed=21, device=dev)
        x = synth.make_activations(200 + 37 * rank, 256, seed=50 + rank, device=dev)
        want = full(x.unsqueeze(0))[0]
        local = ep.shard_experts(full, rank * 4, rank * 4 + 4).to(dev)
        moe = ep.ExpertParallelMoE(full.gate, local, 8, 3)
        got = moe(x.unsqueeze(0))[0]
        res[mode] = bool(torch.equal(got, want))
        # token-gather exchange: per-rank partial sums are rounded to bf16 before the final sum
        local_k = ep.shard_experts(full, rank * 4, rank * 4 + 4, top_k=3).to(dev)
        got_g = ep.ExpertParallelMoE(full.gate, local_k, 8, 3, exchange="gather")(x.unsqueeze(0))[0]
        rel = float((got_g.float() - want.float()).norm() / want.float().norm())
        res[mode] = res[mode] and rel < 4e-3       # bf16 rounding of two partials: about 2**-9 each
        # code exchange: rotated + quantised codes travel, the owner reads them as they arrive: bit-identical
        local_c = ep.shard_experts(full, rank * 4, rank * 4 + 4).to(dev)
        got_c = ep.ExpertParallelMoE(full.gate, local_c, 8, 3, exchange="codes", full_layer=full)(x.unsqueeze(0))[0]
        res[mode] = res[mode] and bool(torch.equal(got_c, want))
    # with a shared expert (token-local: computed by the token's own rank as a layer of its own)
    full = synth.build_layer(hidden=256, n_experts=8, top_k=3, inter=256, shared_inter=256,
                             bit_mix={2: 0.5, 1: 0.25, 4: 0.25}, mode="wxa8", seed=22, device=dev)
    x = synth.make_activations(150 + 21 * rank, 256, seed=60 + rank, device=dev)
    want = full(x.unsqueeze(0))[0].float()
    for exchange, k_local in (("gather", 3), ("rows", 1), ("codes", 1)):
        local = ep.shard_experts(full, rank * 4, rank * 4 + 4, top_k=k_local).to(dev)
        moe = ep.ExpertParallelMoE(full.gate, local, 8, 3, full.shared_expert, full.shared_expert_gate,
                                   exchange=exchange, full_layer=full)
        got = moe(x.unsqueeze(0))[0].float()
        used_engine = moe._shared_layer[0] is not None
        res["wxa8"] = res["wxa8"] and used_engine and float((got - want).norm() / want.norm()) < 4e-3
    dist.barrier()
    np.save(os.path.join(out_dir, f"ep_{rank}.npy"), np.array([res[m] for m in ("wxa8", "wxfp8", "wxa16")]))
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_expert_parallel_equals_single_gpu(tmp_path):
    import torch.multiprocessing as mp
    port = 29600 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        assert np.load(tmp_path / f"ep_{r}.npy").all()


def _worker_one(rank, world, port, out_dir):
    """The whole code-exchange path with a process group of ONE rank (every all-to-all is a copy to itself): route
    over all experts, rotate + quantise, gather, counts, tile plan from the count matrix, owner GEMMs over the
    receive buffer, rows back, combine.  Several token counts, so the owner buffers grow and are reused."""
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    dist.init_process_group("nccl", rank=0, world_size=1, device_id=dev)
    from dartmoq_b200 import ep, synth
    ok = []
    for mode in ("wxa8", "wxfp8", "wxa16"):
        full = synth.build_layer(hidden=512, n_experts=12, top_k=4, inter=256, bit_mix={2: 0.5, 1: 0.25, 4: 0.25},
                                 mode=mode, seed=23, device=dev, zipf=1.1)
        local = ep.shard_experts(full, 0, 12).to(dev)
        moe = ep.ExpertParallelMoE(full.gate, local, 12, 4, exchange="codes", full_layer=full)
        for T in (300, 257, 1500, 300):
            x = synth.make_activations(T, 512, seed=70 + T, device=dev)
            want = full(x.unsqueeze(0))[0]
            got = moe(x.unsqueeze(0))[0]
            ok.append(bool(torch.equal(got, want)))
    np.save(os.path.join(out_dir, "one.npy"), np.array(ok))
    dist.destroy_process_group()


def test_code_exchange_on_one_rank(tmp_path):
    import torch.multiprocessing as mp
    port = 29700 + (os.getpid() % 2000)
    mp.spawn(_worker_one, args=(1, port, str(tmp_path)), nprocs=1, join=True)
    assert np.load(tmp_path / "one.npy").all()
