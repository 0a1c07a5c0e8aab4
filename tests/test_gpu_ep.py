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
    # with a shared expert (token-local: computed by the token's own rank as a layer of its own)
    full = synth.build_layer(hidden=256, n_experts=8, top_k=3, inter=256, shared_inter=256,
                             bit_mix={2: 0.5, 1: 0.25, 4: 0.25}, mode="wxa8", seed=22, device=dev)
    x = synth.make_activations(150 + 21 * rank, 256, seed=60 + rank, device=dev)
    want = full(x.unsqueeze(0))[0].float()
    for exchange, k_local in (("gather", 3), ("rows", 1)):
        local = ep.shard_experts(full, rank * 4, rank * 4 + 4, top_k=k_local).to(dev)
        moe = ep.ExpertParallelMoE(full.gate, local, 8, 3, full.shared_expert, full.shared_expert_gate,
                                   exchange=exchange)
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
