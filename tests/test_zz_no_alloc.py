"""The routing build that brings its own scratch (for callers that may not allocate device memory).

Some hosts cannot hand a kernel a scratch buffer: they run inside a stream capture, or they have frozen
their memory pools, or their framework owns all allocations.  `dmoq_route_build_static` serves them from a
fixed array inside the library.  Checked here, through the C ABI: its tables equal those of the ordinary
`dmoq_route_build` on two calls in a row (the shared scratch keeps the first call's contents), and a
problem larger than the fixed array is refused with a size error instead of overrunning it.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from dartmoq_b200 import _lib

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
OUT_FIELDS = ("expert_rows", "sorted_tokens", "sorted_weights", "row_of", "a_row", "pool_rows", "pool_src",
              "tiles", "n_tiles")


def _tables(T, k, E, seed, has_shared):
    rng = np.random.default_rng(seed)
    idx = torch.from_numpy(np.stack([rng.permutation(E)[:k] for _ in range(T)]).astype(np.int64)).to(DEV)
    w = torch.from_numpy(rng.random((T, k), dtype=np.float32)).to(DEV)
    sw = torch.from_numpy(rng.random(T, dtype=np.float32)).to(DEV) if has_shared else None
    n_ent = E + int(has_shared)
    R = T * k + (T if has_shared else 0)
    i32 = dict(dtype=torch.int32, device=DEV)
    pools = [e % 2 for e in range(E)] + ([2] if has_shared else [])
    rank, seen = [], [0, 0, 0]
    for p in pools:
        rank.append(seen[p])
        seen[p] += 1
    n_pools = 3 if has_shared else 2
    hoisted = [1, 0, 1][:n_pools]
    static = dict(expert_pool=torch.tensor(pools, **i32), expert_rank=torch.tensor(rank, **i32),
                  pool_src_base=torch.zeros(8, **i32), pool_hoisted=torch.tensor(hoisted + [0] * (8 - n_pools), **i32))
    tile_cap = (R + 127) // 128 + n_ent

    def fresh():
        return dict(expert_rows=torch.zeros(n_ent + 1, **i32), sorted_tokens=torch.full((R,), -1, **i32),
                    sorted_weights=torch.zeros(R, dtype=torch.float32, device=DEV), row_of=torch.full((R,), -2, **i32),
                    a_row=torch.full((R,), -3, **i32), pool_rows=torch.zeros(8, **i32),
                    pool_src=torch.full((T * min(k, E // 2 + 1),), -4, **i32), tiles=torch.zeros(tile_cap, 4, **i32),
                    n_tiles=torch.zeros(16, **i32))

    def route(out):
        r = _lib.Route()
        r.T, r.top_k, r.E, r.has_shared, r.tile_m, r.n_pools, r.tile_cap = T, k, E, int(has_shared), 128, n_pools, tile_cap
        for name, t in {**static, **out}.items():
            setattr(r, name, t.data_ptr())
        return r

    return idx, w, sw, fresh, route


@pytest.mark.parametrize("T,k,E,shared", [(50, 2, 8, False), (3000, 8, 64, True)])
def test_static_scratch_route_matches_allocating_route_twice(T, k, E, shared):
    lib = _lib.load()
    assert lib.dmoq_route_static_max_bytes() == 4 << 20
    for call in range(2):                       # second call meets the first call's leftovers in the scratch
        idx, w, sw, fresh, route = _tables(T, k, E, seed=17 + call, has_shared=shared)
        want, got = fresh(), fresh()
        ws = torch.empty(lib.dmoq_route_workspace_bytes(T, k, E), dtype=torch.uint8, device=DEV)
        r1, r2 = route(want), route(got)
        _lib.check(lib.dmoq_route_build(C.byref(r1), _lib.ptr(idx), _lib.ptr(w), _lib.ptr(sw), _lib.ptr(ws),
                                        ws.numel(), None), "dmoq_route_build")
        _lib.check(lib.dmoq_route_build_static(C.byref(r2), _lib.ptr(idx), _lib.ptr(w), _lib.ptr(sw), None),
                   "dmoq_route_build_static")
        torch.cuda.synchronize()
        for name in OUT_FIELDS:
            assert torch.equal(want[name], got[name]), (call, name)
        assert int(got["expert_rows"][-1]) == T * k + (T if shared else 0)


def test_static_scratch_route_allocates_nothing():
    """After a first call on the device, a further call leaves both the framework allocator's and the driver's
    picture of device memory unchanged."""
    lib = _lib.load()
    T, k, E = 700, 4, 32
    idx, w, sw, fresh, route = _tables(T, k, E, seed=5, has_shared=True)
    out = fresh()
    r = route(out)
    for _ in range(2):                          # first call: one-time set-up of the library on this device
        _lib.check(lib.dmoq_route_build_static(C.byref(r), _lib.ptr(idx), _lib.ptr(w), _lib.ptr(sw), None),
                   "dmoq_route_build_static")
    torch.cuda.synchronize()
    before = (torch.cuda.memory_allocated(), torch.cuda.memory_reserved(), torch.cuda.mem_get_info()[0])
    _lib.check(lib.dmoq_route_build_static(C.byref(r), _lib.ptr(idx), _lib.ptr(w), _lib.ptr(sw), None),
               "dmoq_route_build_static")
    torch.cuda.synchronize()
    after = (torch.cuda.memory_allocated(), torch.cuda.memory_reserved(), torch.cuda.mem_get_info()[0])
    assert before == after


def test_static_scratch_route_refuses_oversized_problem():
    lib = _lib.load()
    T, k, E = 1 << 20, 8, 256                   # needs 8192 chunks x 256 experts x 4 B = 8 MiB > 4 MiB
    assert lib.dmoq_route_workspace_bytes(T, k, E) > lib.dmoq_route_static_max_bytes()
    one = torch.zeros(16, dtype=torch.int32, device=DEV)
    r = _lib.Route()
    r.T, r.top_k, r.E, r.has_shared, r.tile_m, r.n_pools, r.tile_cap = T, k, E, 0, 128, 1, 1
    for name in ("expert_pool", "expert_rank", "expert_rows", "sorted_tokens", "sorted_weights", "row_of", "a_row",
                 "pool_rows", "pool_src", "pool_src_base", "tiles", "n_tiles", "pool_hoisted"):
        setattr(r, name, one.data_ptr())
    rc = lib.dmoq_route_build_static(C.byref(r), _lib.ptr(one), _lib.ptr(one), None, None)
    assert rc == -3 and b"size" in lib.dmoq_strerror(rc)
