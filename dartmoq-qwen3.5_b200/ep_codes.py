"""Expert-parallel exchange of rotated + quantised activation codes.

Rank ``r`` owns the experts ``[r*E/N, (r+1)*E/N)``; tokens are data-parallel.  One forward:

  token's rank   route over ALL experts (device-side counting sort: rows grouped by expert = by owner rank)
                 -> hoisted rotation + activation quantisation of the local tokens, once per bit pool (the rotation
                    depends on the expert's bit width only, seed 42+bit, which every rank knows)
                 -> rows gathered into routed order = the send buffer (INT8 / e4m3 codes + fp16 scales: about half
                    the bytes of bf16 rows)
  exchange       per-expert row counts (all-to-all of E/N ints per pair; the one host synchronisation), then codes
                 and scales (all-to-all with those split sizes) into the owner's own memory
  owner          the rows of one (source rank, expert) pair are contiguous in the receive buffer: the host turns the
                 count matrix into tile lists, and the grouped GEMMs read the buffer as it arrived -- no second sort,
                 no gate_up-side rotation on the owner; down-side rotation and down GEMM as on one GPU
  back           fp16 rows in arrival order (all-to-all with the split sizes swapped) = the sender's routed order
  token's rank   the single-GPU combine: routing weights, bf16 rounding chain, fp32 sum in slot order

so the result is bit-identical to the unsharded layer.  The shared expert is token-local and runs on the token's
own rank.  No kernel reads another GPU's memory: every row lands in the receiver's buffer through NCCL first.
The reference has no counterpart (it has no distributed code).
"""
from __future__ import annotations

import ctypes as C
import os
from typing import List, Optional

import numpy as np
import torch
import torch.distributed as dist

from . import _lib
from . import format as fmt
from ._lib import A16, EPI_PLAIN, EPI_SILU, MAX_POOLS, TILE_M, Route, check, ptr

GROUP = fmt.GROUP_SIZE


def owner_tiles(counts: np.ndarray, pool_of: np.ndarray, rank_of: np.ndarray, n_pools: int, tile_m: int = TILE_M,
                expert0: int = 0, row_base: int = 0):
    """Tile lists over a receive buffer laid out source by source, each source's rows sorted by local expert.

    counts (N_src, E_local): rows source s sends for local expert e.  Returns (tiles (n, 4) int32 rows of
    (expert, first row, row count, member rank), pool p's tiles contiguous; n_tiles (2*MAX_POOLS,) = tiles per pool
    then each pool's first tile).  A (source, expert) pair's rows are cut into tiles of at most ``tile_m`` rows.
    ``counts`` may be a column block of the full matrix: its first column is local expert ``expert0`` and its rows
    start at ``row_base`` of the receive buffer."""
    n_src, e_loc = counts.shape
    flat = counts.reshape(-1).astype(np.int64)
    seg_start = row_base + np.concatenate([[0], np.cumsum(flat)[:-1]])   # arrival order: source major, expert minor
    seg_expert = expert0 + np.tile(np.arange(e_loc), n_src)
    seg_tiles = (flat + tile_m - 1) // tile_m
    tiles_out, n_tiles = [], np.zeros(2 * MAX_POOLS, np.int32)
    base = 0
    for p in range(n_pools):
        sel = np.nonzero((pool_of[seg_expert] == p) & (flat > 0))[0]
        # experts in index order, sources in rank order inside an expert (keeps one expert's weights hot in L2)
        sel = sel[np.lexsort((sel // e_loc, seg_expert[sel]))]   # sel // e_loc = source rank
        nt = seg_tiles[sel]
        total = int(nt.sum())
        if total:
            owner = np.repeat(np.arange(sel.size), nt)
            within = np.arange(total) - np.repeat(np.cumsum(nt) - nt, nt)
            row0 = seg_start[sel][owner] + within * tile_m
            rows = np.minimum(tile_m, flat[sel][owner] - within * tile_m)
            e = seg_expert[sel][owner]
            tiles_out.append(np.stack([e, row0, rows, rank_of[e]], 1))
        n_tiles[p], n_tiles[MAX_POOLS + p] = total, base
        base += total
    tiles = np.concatenate(tiles_out, 0).astype(np.int32) if tiles_out else np.zeros((0, 4), np.int32)
    return tiles, n_tiles


class _FrontPool:
    """What the token's rank needs of a bit pool: its mode, rotation stack and activation scale (no weights)."""

    def __init__(self, bit, mode, members, rot, act_scale, hoisted):
        self.bit, self.mode, self.members, self.rot, self.act_scale, self.hoisted = bit, mode, members, rot, act_scale, hoisted

    def code_bytes(self, k):
        return {0: 2 * k, 1: k, 2: k, 3: k // 2}[self.mode]

    def scale_bytes(self, k):
        return {0: 0, 1: 2 * (k // GROUP), 2: 2 * (k // GROUP), 3: k // 32}[self.mode]


class CodesExchange:
    """Sender front end + owner back end of the code exchange for one layer on one rank."""

    def __init__(self, full_layer, local_moe, num_experts: int, top_k: int, group, device):
        from .moe import _mode_lut
        self.group, self.device = group, device
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.E, self.k, self.H = num_experts, top_k, full_layer.hidden_size
        self.E_loc = num_experts // self.world
        self.local_moe = local_moe
        self.lib = _lib.load()
        offsets = full_layer._offsets_lists()
        expert_pool = [-1] * num_experts
        self.pools: List[_FrontPool] = []
        for bs, w in full_layer.bit_weights.items():
            bit, off = int(bs), offsets[bs]
            members = [e for e in range(num_experts) if off[e + 1] > off[e]]
            if not members:
                continue
            for e in members:
                if expert_pool[e] >= 0:
                    raise NotImplementedError("the code exchange needs one bit width per expert")
                expert_pool[e] = len(self.pools)
            mode = full_layer._pool_mode(bit)
            gu = w.gate_up_packed
            _, act_scale, _, _, _ = _mode_lut(mode, bit, gu["codebook"], device)
            rot = fmt.generate_batch_rotation_matrices(GROUP, int(gu["seed"]), self.H // GROUP, GROUP, device, torch.float16)
            hoisted = bool(full_layer.enable_rotation_hoist) and len(members) * top_k / num_experts > float(full_layer.rotation_hoist_threshold)
            self.pools.append(_FrontPool(bit, mode, members, rot, act_scale, hoisted))
        modes = {p.mode for p in self.pools}
        if len(modes) != 1:
            raise NotImplementedError("the code exchange needs one activation mode for all routed pools")
        self.mode = modes.pop()
        i32 = dict(dtype=torch.int32, device=device)
        self.expert_pool = torch.tensor(expert_pool, **i32)
        self.expert_rank = torch.zeros(num_experts, **i32)
        self.pool_hoisted = torch.tensor([int(p.hoisted) for p in self.pools] + [0] * (MAX_POOLS - len(self.pools)), **i32)
        self.stride = (self.H + 511) // 512 * 512                      # elements per row of the exchanged tables
        self._ws = {}
        self._pinned = None
        self._comm_stream = None
        self._pool_of = self._rank_of = None
        # blocks of each owner's experts the exchange is pipelined over (DMOQ_EP_CHUNKS overrides: tuning runs)
        self.n_chunks = int(os.environ.get("DMOQ_EP_CHUNKS", "4"))
        self._owner_cap = 0
        self.last_stage_ms = None
        self.last_launches = 0

    # ------------------------------------------------------------------ per-token-count sender buffers
    def _workspace(self, T: int):
        ws = self._ws.get(T)
        if ws is not None:
            return ws
        if len(self._ws) >= 8:
            self._ws.pop(next(iter(self._ws)))
        dev, k = self.device, self.k
        R = T * k

        class W:
            pass
        ws = W()
        ws.R = R
        i32 = dict(dtype=torch.int32, device=dev)
        u8 = dict(dtype=torch.uint8, device=dev)
        ws.expert_rows = torch.zeros(self.E + 1, **i32)
        ws.sorted_tokens = torch.zeros(max(R, 1), **i32)
        ws.sorted_weights = torch.zeros(max(R, 1), dtype=torch.float32, device=dev)
        ws.row_of = torch.full((max(R, 1),), -1, **i32)
        ws.a_row = torch.zeros(max(R, 1), **i32)
        ws.pool_rows = torch.zeros(MAX_POOLS, **i32)
        ws.n_tiles = torch.zeros(2 * MAX_POOLS, **i32)
        ws.tile_cap = (R + TILE_M - 1) // TILE_M + self.E
        ws.tiles = torch.zeros(ws.tile_cap, 4, **i32)
        bases, total, ws.caps, ws.act_codes, ws.act_scales = [], 0, [], [], []
        for p in self.pools:
            cap = T if p.hoisted else T * min(k, len(p.members))
            bases.append(0 if p.hoisted else total)
            total += 0 if p.hoisted else cap
            ws.caps.append(cap)
            ws.act_codes.append(torch.empty(max(cap, 1) * p.code_bytes(self.H), **u8))
            ws.act_scales.append(torch.empty(max(max(cap, 1) * p.scale_bytes(self.H), 16), **u8))
        ws.pool_src = torch.zeros(max(total, 1), **i32)
        ws.bases = bases
        ws.pool_src_base = torch.tensor(bases + [0] * (MAX_POOLS - len(bases)), **i32)
        ws.route_ws = torch.empty(max(self.lib.dmoq_route_workspace_bytes(T, k, self.E), 16), **u8)
        p0 = self.pools[0]
        ws.send_codes = torch.empty(max(R, 1), p0.code_bytes(self.stride), **u8)
        ws.send_scales = torch.empty(max(R, 1), max(p0.scale_bytes(self.stride), 2), **u8)
        ws.back = torch.empty(max(R, 1), self.H, dtype=torch.float16, device=dev)
        r = Route()
        r.T, r.top_k, r.E, r.has_shared, r.tile_m, r.n_pools = T, k, self.E, 0, TILE_M, len(self.pools)
        r.expert_pool, r.expert_rank = self.expert_pool.data_ptr(), self.expert_rank.data_ptr()
        r.expert_rows = ws.expert_rows.data_ptr()
        r.sorted_tokens, r.sorted_weights = ws.sorted_tokens.data_ptr(), ws.sorted_weights.data_ptr()
        r.row_of, r.a_row = ws.row_of.data_ptr(), ws.a_row.data_ptr()
        r.pool_rows, r.pool_src, r.pool_src_base = ws.pool_rows.data_ptr(), ws.pool_src.data_ptr(), ws.pool_src_base.data_ptr()
        r.tiles, r.n_tiles, r.tile_cap = ws.tiles.data_ptr(), ws.n_tiles.data_ptr(), ws.tile_cap
        r.pool_hoisted = self.pool_hoisted.data_ptr()
        ws.route = r
        self._ws[T] = ws
        return ws

    # ------------------------------------------------------------------ owner side
    def _owner_buffers(self, rows: int):
        """Receive / intermediate buffers of the owner, grown geometrically (row counts vary from step to step)."""
        if rows > self._owner_cap:
            cap = max(rows, int(self._owner_cap * 1.25), 1024)
            dev = self.device
            eng = self.local_moe._get_engine(dev)
            p0 = self.pools[0]
            u8 = dict(dtype=torch.uint8, device=dev)
            self.recv_codes = torch.empty(cap, p0.code_bytes(self.stride), **u8)
            self.recv_scales = torch.empty(cap, max(p0.scale_bytes(self.stride), 2), **u8)
            self.act = torch.empty(cap, eng.inter_max, dtype=torch.float16, device=dev)
            code_b = max(p.code_bytes(eng.inter_max) for p in eng.pools)
            scale_b = max(max(p.scale_bytes(eng.inter_max) for p in eng.pools), 1)
            self.dn_codes = torch.empty(cap * code_b, **u8)
            self.dn_scales = torch.empty(cap * scale_b, **u8)
            self.dn = torch.empty(cap, self.H, dtype=torch.float16, device=dev)
            self.ones = torch.ones(cap, dtype=torch.float32, device=dev)
            self._owner_cap = cap

    def _owner_route(self, counts: np.ndarray, expert0: int, row_base: int, n_rows_total: int):
        """Route struct + tile tensors for the rows of local experts [expert0, expert0 + counts.shape[1]) that start at
        ``row_base`` of the receive buffer."""
        eng = self.local_moe._get_engine(self.device)
        tiles_np, n_tiles_np = owner_tiles(counts, self._pool_of, self._rank_of, len(eng.pools), TILE_M, expert0, row_base)
        tiles = torch.from_numpy(tiles_np if tiles_np.size else np.zeros((1, 4), np.int32)).to(self.device, non_blocking=True)
        n_tiles = torch.from_numpy(n_tiles_np).to(self.device, non_blocking=True)
        r = Route()
        r.T, r.top_k, r.E, r.has_shared, r.tile_m, r.n_pools = n_rows_total, 1, self.E_loc, 0, TILE_M, len(eng.pools)
        r.expert_pool, r.expert_rank = eng.expert_pool.data_ptr(), eng.expert_rank.data_ptr()
        r.sorted_weights = self.ones.data_ptr()
        r.tiles, r.n_tiles, r.tile_cap = tiles.data_ptr(), n_tiles.data_ptr(), max(int(tiles_np.shape[0]), 1)
        r.pool_hoisted = self.pool_hoisted.data_ptr()
        return r, n_tiles_np, (tiles, n_tiles)

    def _owner_compute(self, r, n_tiles_np, s):
        """Grouped GEMMs of the local experts over (a part of) the receive buffer as it arrived."""
        lib = self.lib
        eng = self.local_moe._get_engine(self.device)
        for i, p in enumerate(eng.pools):
            if n_tiles_np[i] == 0:
                continue
            if p.img[0] is not None:
                p.build_norm_images()
                p.c.gu_img, p.c.dn_img = p.img[0].data_ptr(), p.img[1].data_ptr()
            else:
                p.c.gu_img = p.c.dn_img = None
            eng.pool_array[i] = p.c
            check(lib.dmoq_grouped_gemm(C.byref(r), eng.pool_array, i, 0, EPI_SILU, self.H, ptr(self.recv_codes),
                                        ptr(self.recv_scales), self.stride, ptr(self.act), eng.inter_max, None, s),
                  "dmoq_grouped_gemm(gate_up)")
            check(lib.dmoq_rotate_quant_down(C.byref(r), eng.pool_array, i, ptr(self.act), eng.inter_max,
                                             ptr(self.dn_codes), ptr(self.dn_scales), eng.inter_max, s),
                  "dmoq_rotate_quant_down")
            check(lib.dmoq_grouped_gemm(C.byref(r), eng.pool_array, i, 1, EPI_PLAIN, self.H, ptr(self.dn_codes),
                                        ptr(self.dn_scales), eng.inter_max, ptr(self.dn), self.H, None, s),
                  "dmoq_grouped_gemm(down)")
            self.last_launches += 3

    # ------------------------------------------------------------------ one forward
    def forward(self, x: torch.Tensor, topk_w: torch.Tensor, topk_idx: torch.Tensor, profile: bool = False) -> torch.Tensor:
        """x (T, H) local tokens -> routed experts' contribution (T, H), bit-identical to the unsharded layer's.

        The exchange is cut into ``n_chunks`` blocks of each owner's experts.  The collectives run on a second stream:
        while the owner computes block c, block c+1's codes arrive and block c-1's results travel back."""
        lib, dev, N = self.lib, self.device, self.world
        T = x.shape[0]
        ws = self._workspace(T)
        main = torch.cuda.current_stream()
        s = C.c_void_p(main.cuda_stream)
        if self._comm_stream is None:
            self._comm_stream = torch.cuda.Stream(device=dev)
        comm = self._comm_stream
        events, names = [], []

        def mark(name):
            if profile:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                events.append(ev)
                names.append(name)
        mark("start")
        self.last_launches = 0
        is_bf16 = int(x.dtype == torch.bfloat16)
        topk_idx = topk_idx.to(torch.int64).contiguous()
        topk_w = topk_w.to(torch.float32).contiguous()
        # ---- token's rank: route, exchange the per-expert counts, rotate + quantise once per bit pool, rows into routed order
        check(lib.dmoq_route_build(C.byref(ws.route), ptr(topk_idx), ptr(topk_w), None, ptr(ws.route_ws),
                                   ws.route_ws.numel(), s), "dmoq_route_build")
        counts_dev = (ws.expert_rows[1:] - ws.expert_rows[:-1]).reshape(N, self.E_loc).contiguous()
        recv_counts_dev = torch.empty_like(counts_dev)
        dist.all_to_all_single(recv_counts_dev, counts_dev, group=self.group)
        if self._pinned is None:
            self._pinned = torch.empty((2, N, self.E_loc), dtype=torch.int32).pin_memory()
        both = self._pinned
        both.copy_(torch.stack([counts_dev, recv_counts_dev]), non_blocking=True)
        ev_counts = torch.cuda.Event()
        ev_counts.record()
        for i, p in enumerate(self.pools):
            src_row = None if p.hoisted else C.c_void_p(ws.pool_src.data_ptr() + 4 * ws.bases[i])
            n_dev = None if p.hoisted else C.c_void_p(ws.pool_rows.data_ptr() + 4 * i)
            check(lib.dmoq_rotate_quant(p.mode, ptr(x), is_bf16, self.H, ptr(p.rot), None, src_row, ws.caps[i], n_dev,
                                        p.act_scale, ptr(ws.act_codes[i]), ptr(ws.act_scales[i]), s), "dmoq_rotate_quant")
            has_scales = p.scale_bytes(self.H) > 0
            check(lib.dmoq_gather_rows(C.byref(ws.route), i, ptr(ws.act_codes[i]), p.code_bytes(self.H), p.code_bytes(self.H),
                                       ptr(ws.send_codes), p.code_bytes(self.stride),
                                       ptr(ws.act_scales[i]) if has_scales else None, p.scale_bytes(self.H),
                                       p.scale_bytes(self.H), ptr(ws.send_scales) if has_scales else None,
                                       p.scale_bytes(self.stride), s), "dmoq_gather_rows")
            self.last_launches += 2
        mark("route_rotate_gather")
        front_done = torch.cuda.Event()
        front_done.record()
        # ---- split sizes (the one host synchronisation)
        ev_counts.synchronize()
        send_c, recv_c = both[0].numpy().astype(np.int64), both[1].numpy().astype(np.int64)
        n_recv = int(recv_c.sum())
        self._owner_buffers(n_recv)
        eng = self.local_moe._get_engine(dev)
        if self._pool_of is None:
            self._pool_of = eng.expert_pool.cpu().numpy()[:self.E_loc]
            self._rank_of = eng.expert_rank.cpu().numpy()[:self.E_loc]
        # small exchanges go in one piece: a block must be worth its collective's launch latency
        n_chunks = max(1, min(self.n_chunks if ws.R >= 65536 else 1, self.E_loc))
        edges = [self.E_loc * c // n_chunks for c in range(n_chunks + 1)]
        send_start = np.concatenate([[0], np.cumsum(send_c.reshape(-1))])     # first routed row of every global expert
        keep = []
        recv_base = 0
        comm.wait_event(front_done)
        chunks = []
        for c in range(n_chunks):
            c0, c1 = edges[c], edges[c + 1]
            sub_recv = recv_c[:, c0:c1]
            rows_c = int(sub_recv.sum())
            in_codes, in_scales, out_codes, out_scales, back_in, back_out = [], [], [], [], [], []
            off = recv_base
            for peer in range(N):
                a0 = int(send_start[peer * self.E_loc + c0])
                a1 = int(send_start[peer * self.E_loc + c1])
                in_codes.append(ws.send_codes[a0:a1])
                in_scales.append(ws.send_scales[a0:a1])
                back_out.append(ws.back[a0:a1])
                n_from = int(sub_recv[peer].sum())
                out_codes.append(self.recv_codes[off:off + n_from])
                out_scales.append(self.recv_scales[off:off + n_from])
                back_in.append(self.dn[off:off + n_from])
                off += n_from
            chunks.append((c0, sub_recv, recv_base, rows_c, in_codes, in_scales, out_codes, out_scales, back_in, back_out))
            recv_base += rows_c
        arrived = []
        with torch.cuda.stream(comm):
            for ch in chunks:      # all dispatches are queued first: block c+1 travels while block c is computed
                dist.all_to_all(ch[6], ch[4], group=self.group)
                if self.mode != A16:
                    dist.all_to_all(ch[7], ch[5], group=self.group)
                ev = torch.cuda.Event()
                ev.record(comm)
                arrived.append(ev)
        for c, ch in enumerate(chunks):
            c0, sub_recv, base, rows_c = ch[0], ch[1], ch[2], ch[3]
            main.wait_event(arrived[c])
            if c == 0:
                mark("first_block_arrived")
            r, n_tiles_np, alive = self._owner_route(sub_recv, c0, base, n_recv)
            keep.append(alive)
            self._owner_compute(r, n_tiles_np, s)
            done = torch.cuda.Event()
            done.record(main)
            with torch.cuda.stream(comm):      # the block's fp16 rows go back in arrival order = the sender's routed order
                comm.wait_event(done)
                dist.all_to_all(ch[9], ch[8], group=self.group)
        mark("owner_experts")
        back_done = torch.cuda.Event()
        back_done.record(comm)
        main.wait_event(back_done)
        mark("last_block_back")
        self._keep = keep          # tile tensors stay alive until the stream has consumed them
        # ---- token's rank: the single-GPU combine
        y = torch.empty_like(x)
        check(lib.dmoq_combine_weighted(C.byref(ws.route), ptr(ws.back), self.H, ptr(y), is_bf16, s), "dmoq_combine_weighted")
        self.last_launches += 2
        mark("combine")
        if profile:
            torch.cuda.synchronize()
            self.last_stage_ms = {names[i + 1]: round(events[i].elapsed_time(events[i + 1]), 4) for i in range(len(events) - 1)}
        return y
