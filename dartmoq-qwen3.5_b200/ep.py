"""Expert parallelism: experts sharded over the ranks of one node, tokens data-parallel.

The reference has no distributed code; this is the B200 scale-out of the same layer.  Rank ``r`` owns the
experts ``[r*E/N, (r+1)*E/N)``.  One forward is

    route (replicated router, local tokens)  ->  pack rows by destination rank
    ->  all_to_all (counts, then rows)       ->  grouped expert compute on the owner
    ->  all_to_all back                      ->  fixed-order fp32 sum of each token's top-k rows

That is the ``"rows"`` exchange: one row per (token, slot) pair, results bit-identical to the unsharded
layer.  The ``"gather"`` exchange moves each token once per rank instead of once per slot:

    all_gather (tokens, routing)  ->  own experts over ALL tokens, other ranks' slots masked (-1)
    ->  all_to_all of one partial row per token  ->  fp32 sum of the partials in rank order

It rounds each rank's partial sum to the activation dtype before the final sum, so it matches the unsharded
layer to rounding, not bit for bit.

The exchange plumbing below is plain torch + ``torch.distributed`` and device agnostic (NCCL over
NVLink on GPUs, gloo on CPUs for tests); the expert compute is a callback, on GPUs the libdmoq engine.
Rows always land in the receiver's own memory before any kernel touches them.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist


class DispatchPlan:
    """Where every (token, slot) pair goes and how to bring the answers back."""

    def __init__(self, topk_idx: torch.Tensor, experts_per_rank: int, world: int):
        T, k = topk_idx.shape
        flat_e = topk_idx.reshape(-1)
        dest = torch.div(flat_e, experts_per_rank, rounding_mode="floor")
        # stable order: by destination rank, then by flat (token, slot) index -> deterministic
        self.order = torch.sort(dest, stable=True)[1]
        self.send_counts = torch.bincount(dest, minlength=world)
        self.token = torch.div(self.order, k, rounding_mode="floor")
        self.local_expert = flat_e[self.order] - dest[self.order] * experts_per_rank
        self.T, self.k = T, k

    def inverse(self) -> torch.Tensor:
        inv = torch.empty_like(self.order)
        inv[self.order] = torch.arange(self.order.numel(), device=self.order.device)
        return inv


def exchange_counts(send_counts: torch.Tensor, group=None) -> torch.Tensor:
    recv = torch.empty_like(send_counts)
    dist.all_to_all_single(recv, send_counts, group=group)
    return recv


def all_to_all_rows(rows: torch.Tensor, send: list, recv: list, group=None) -> torch.Tensor:
    out = rows.new_empty((sum(recv),) + tuple(rows.shape[1:]))
    dist.all_to_all_single(out, rows.contiguous(), output_split_sizes=recv, input_split_sizes=send, group=group)
    return out


def _sum_slots_torch(back: torch.Tensor, inverse: torch.Tensor, T: int, k: int, dtype) -> torch.Tensor:
    """y[t] = sum over the token's k rows, fp32, slot order (device-agnostic form)."""
    per_pair = back[inverse].reshape(T, k, back.shape[1]).float()
    y = per_pair[:, 0]
    for s in range(1, k):
        y = y + per_pair[:, s]
    return y.to(dtype)


def _sum_slots_cuda(back: torch.Tensor, inverse: torch.Tensor, T: int, k: int, dtype) -> torch.Tensor:
    """The same sum through the library's deterministic combine kernel (one pass over the rows)."""
    import ctypes as C
    from . import _lib
    if back.dtype != torch.bfloat16 or dtype not in (torch.bfloat16, torch.float16):
        return _sum_slots_torch(back, inverse, T, k, dtype)
    row_of = inverse.to(torch.int32).contiguous()
    rows = back.contiguous()
    y = torch.empty((T, rows.shape[1]), dtype=dtype, device=rows.device)
    r = _lib.Route()
    r.T, r.top_k, r.has_shared = T, k, 0
    r.row_of = row_of.data_ptr()
    _lib.check(_lib.load().dmoq_combine(C.byref(r), _lib.ptr(rows), rows.shape[1], _lib.ptr(y),
                                        int(dtype == torch.bfloat16),
                                        C.c_void_p(torch.cuda.current_stream().cuda_stream)), "dmoq_combine")
    return y


def ep_forward(x: torch.Tensor, topk_w: torch.Tensor, topk_idx: torch.Tensor, experts_per_rank: int,
               local_compute: Callable[[torch.Tensor, torch.Tensor, torch.Tensor], torch.Tensor],
               group=None) -> torch.Tensor:
    """x (T, H) local tokens; ``local_compute(rows, local_expert, weight) -> (rows, H)`` runs on the owner and
    returns each row's expert output already multiplied by its routing weight.  Returns (T, H) in x's dtype."""
    world = dist.get_world_size(group)
    plan = DispatchPlan(topk_idx, experts_per_rank, world)
    recv_counts = exchange_counts(plan.send_counts, group)
    send = plan.send_counts.tolist()          # the one host synchronisation of an EP forward
    recv = recv_counts.tolist()
    rows = all_to_all_rows(x[plan.token], send, recv, group)
    meta = torch.stack([plan.local_expert.to(torch.float32), topk_w.reshape(-1)[plan.order].to(torch.float32)], 1)
    meta = all_to_all_rows(meta, send, recv, group)
    out_rows = local_compute(rows, meta[:, 0].to(torch.int64), meta[:, 1])
    back = all_to_all_rows(out_rows, recv, send, group)
    # back[i] answers send row i; put the rows in (token, slot) order and add the k slots in slot order
    if plan.T == 0:
        return x.new_zeros(x.shape)
    sum_slots = _sum_slots_cuda if back.is_cuda else _sum_slots_torch
    return sum_slots(back, plan.inverse(), plan.T, plan.k, x.dtype)


def ep_forward_gathered(x: torch.Tensor, topk_w: torch.Tensor, topk_idx: torch.Tensor, experts_per_rank: int,
                        local_partial: Callable[[torch.Tensor, torch.Tensor, torch.Tensor], torch.Tensor],
                        group=None, extra=None) -> torch.Tensor:
    """Token-gather exchange.  ``local_partial(x_all, w_all, local_idx_all) -> (T_all, H)`` runs this rank's
    experts over every rank's tokens; ``local_idx_all`` holds the local expert id of a slot or -1 where the
    slot belongs to another rank, and the callback returns each token's weighted sum over its local slots
    (zeros where it has none).  Batches may differ in size between ranks (padded to the largest).
    ``extra`` (T, H), e.g. the token-local shared expert's output, is added as one more partial in the same
    fp32 sum; a zero-argument callable is resolved only when the partials have come back (a caller that
    computes it on another stream joins that stream there)."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    T, H = x.shape
    k = topk_idx.shape[1]
    counts = torch.empty(world, dtype=torch.int64, device=x.device)
    dist.all_gather_into_tensor(counts, torch.tensor([T], dtype=torch.int64, device=x.device), group=group)
    t_max = max(counts.tolist())              # the one host synchronisation of this exchange
    if t_max == 0:
        return x.new_zeros(x.shape)
    n_part = world + (1 if extra is not None else 0)

    def padded(t: torch.Tensor, fill: float) -> torch.Tensor:
        if T == t_max:
            return t.contiguous()
        out = t.new_full((t_max,) + tuple(t.shape[1:]), fill)
        out[:T] = t
        return out

    x_all = x.new_empty((world * t_max, H))
    dist.all_gather_into_tensor(x_all, padded(x, 0.0), group=group)
    # expert ids travel as fp32 beside the weights (exact below 2**24); padding rows carry id -1
    meta = torch.cat([topk_w.to(torch.float32), topk_idx.to(torch.float32)], 1)
    meta_all = meta.new_empty((world * t_max, 2 * k))
    dist.all_gather_into_tensor(meta_all, padded(meta, -1.0), group=group)
    w_all = meta_all[:, :k].contiguous()
    idx_all = meta_all[:, k:].to(torch.int64)
    lo = rank * experts_per_rank
    mine = (idx_all >= lo) & (idx_all < lo + experts_per_rank)
    local_idx = torch.where(mine, idx_all - lo, torch.full_like(idx_all, -1))
    part = local_partial(x_all, w_all, local_idx).contiguous()
    back = part.new_empty((n_part * t_max, H))   # chunk r: rank r's partial rows for this rank's tokens
    dist.all_to_all_single(back[:world * t_max], part, group=group)
    if T == 0:
        return x.new_zeros(x.shape)
    if extra is not None:
        back[world * t_max:world * t_max + T] = extra() if callable(extra) else extra
    # row of (token t, partial r) is r * t_max + t; add each token's partials in that order
    row_of = (torch.arange(n_part, device=x.device) * t_max).unsqueeze(0) + torch.arange(T, device=x.device).unsqueeze(1)
    sum_slots = _sum_slots_cuda if back.is_cuda else _sum_slots_torch
    return sum_slots(back, row_of.reshape(-1), T, n_part, x.dtype)


class ExpertParallelMoE(torch.nn.Module):
    """EP wrapper around a local ``Wx*BitPartitionedGroupMoE`` that holds only this rank's experts.

    ``gate`` is the replicated router over ALL experts (tuple-returning or logits, as the local modules
    accept); ``local_moe`` must have ``num_experts == experts_per_rank`` and no shared expert; a shared
    expert, being token-local, is applied here through its packed Linear layers.
    """

    def __init__(self, gate, local_moe, num_experts: int, top_k: int, shared_expert=None,
                 shared_expert_gate=None, group=None, exchange: str = "rows", full_layer=None):
        super().__init__()
        if exchange not in ("rows", "gather", "codes"):
            raise ValueError(f"exchange must be 'rows', 'gather' or 'codes', got {exchange!r}")
        if exchange == "codes" and full_layer is None:
            raise ValueError("exchange='codes' needs full_layer: the unsharded module (its codebooks, seeds and expert "
                             "offsets; the weights themselves are not used)")
        want_k = top_k if exchange == "gather" else 1
        if local_moe.top_k != want_k:
            raise ValueError(f"exchange={exchange!r} needs a local module with top_k={want_k} "
                             f"(shard_experts(..., top_k={want_k})), got {local_moe.top_k}")
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        if num_experts % world:
            raise ValueError(f"num_experts ({num_experts}) must be a multiple of the group size ({world}): "
                             "every rank owns the same number of experts")
        self.gate, self.local_moe = gate, local_moe
        self.num_experts, self.top_k = num_experts, top_k
        self.shared_expert, self.shared_expert_gate = shared_expert, shared_expert_gate
        self.group, self.exchange = group, exchange
        self._shared_layer: list = []         # [module or None] once resolved; a list keeps it out of the submodules
        self._side_stream: list = []
        self._codes: list = []                # the code exchange's state
        self._full_meta = [full_layer] if exchange == "codes" else []
        if exchange == "codes":
            # built now where the device is known: only the unsharded layer's metadata (codebooks, seeds, expert
            # offsets) is read, so the caller may drop that layer's weights right after
            dev = next((b.device for b in local_moe.buffers()), None)
            if dev is not None and dev.type == "cuda":
                from .ep_codes import CodesExchange
                with torch.cuda.device(dev):
                    self._codes.append(CodesExchange(self._full_meta.pop(), local_moe, num_experts, top_k, group, dev))
        self.profile = False                  # codes exchange: per-stage device times into last_stage_ms
        self.last_stage_ms = None
        self.last_launches = 0

    def _local_partial(self, x_all, w_all, local_idx):
        eng = self.local_moe._get_engine(x_all.device)
        return eng.run(x_all, w_all, local_idx, None)

    def _shared_partial(self, x: torch.Tensor) -> Optional[torch.Tensor]:
        """sigmoid(gate(x)) * shared_expert(x) through the library engine: the shared expert as a layer of its
        own with no routed experts.  None when there is none, or it is not three packed linears on a GPU (the
        caller then applies the torch modules)."""
        if self.shared_expert is None or self.shared_expert_gate is None or not x.is_cuda or x.shape[0] == 0:
            return None
        if not self._shared_layer:
            lm = self.local_moe
            layer = type(lm)(None, 1, lm.hidden_size, lm.intermediate_size, 1, self.shared_expert,
                             self.shared_expert_gate)
            layer.enable_timing = False
            self._shared_layer.append(layer if layer._shared_packs() is not None else None)
        layer = self._shared_layer[0]
        if layer is None:
            return None
        T = x.shape[0]
        no_expert = torch.full((T, 1), -1, dtype=torch.int64, device=x.device)
        no_weight = torch.zeros((T, 1), dtype=torch.float32, device=x.device)
        shared_w = torch.sigmoid(self.shared_expert_gate(x)).reshape(-1)
        return layer._get_engine(x.device).run(x, no_weight, no_expert, shared_w)

    def _local(self, rows, local_expert, weight):
        if rows.shape[0] == 0:
            return rows
        eng = self.local_moe._get_engine(rows.device)
        return eng.run(rows.contiguous(), weight.reshape(-1, 1), local_expert.reshape(-1, 1), None)

    @torch.no_grad()
    def forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        b, s, h = hidden_states.shape
        x = hidden_states.reshape(-1, h).contiguous()
        out = self.gate(x)
        if isinstance(out, tuple):
            _, w, idx = out
        else:
            w, idx = out.softmax(dim=-1).topk(self.top_k, dim=-1)
        world = dist.get_world_size(self.group)
        if self.exchange == "gather" and x.is_cuda:
            # the shared expert needs no exchange: it runs on a second stream beside the collectives and the
            # routed experts, and is joined where the partial rows are summed
            main = torch.cuda.current_stream()
            if not self._side_stream:
                self._side_stream.append(torch.cuda.Stream(device=x.device))
            side = self._side_stream[0]
            side.wait_stream(main)
            with torch.cuda.stream(side):
                shared = self._shared_partial(x)

            def joined():
                main.wait_stream(side)
                return shared

            y = ep_forward_gathered(x, w, idx, self.num_experts // world, self._local_partial, self.group,
                                    extra=joined if shared is not None else None)
            main.wait_stream(side)
        elif self.exchange == "codes":
            if not x.is_cuda:
                raise RuntimeError("the code exchange runs on CUDA devices only")
            if not self._codes:
                from .ep_codes import CodesExchange
                self._codes.append(CodesExchange(self._full_meta.pop(), self.local_moe, self.num_experts, self.top_k,
                                                 self.group, x.device))
            main = torch.cuda.current_stream()
            if not self._side_stream:
                self._side_stream.append(torch.cuda.Stream(device=x.device))
            side = self._side_stream[0]
            side.wait_stream(main)
            with torch.cuda.stream(side):       # the token-local shared expert, beside the exchanges
                shared = self._shared_partial(x)
            cx = self._codes[0]
            y = cx.forward(x, w, idx, profile=self.profile)
            main.wait_stream(side)
            if shared is not None:
                y = (y.float() + shared.float()).to(y.dtype)
            self.last_stage_ms, self.last_launches = cx.last_stage_ms, cx.last_launches
        elif self.exchange == "gather":
            shared = None
            y = ep_forward_gathered(x, w, idx, self.num_experts // world, self._local_partial, self.group)
        else:
            shared = self._shared_partial(x)
            y = ep_forward(x, w, idx, self.num_experts // world, self._local, self.group)
            if shared is not None:
                y = y + shared
        if shared is None and self.shared_expert is not None and self.shared_expert_gate is not None:
            y = y + self.shared_expert(x) * torch.sigmoid(self.shared_expert_gate(x))
        return y.reshape(b, s, h)


@torch.no_grad()
def shard_experts(moe, lo: int, hi: int, top_k: int = 1):
    """New module of the same class holding experts ``[lo, hi)`` of ``moe``.  ``top_k`` = 1 for the "rows"
    exchange (on the owner every received row is routed to exactly one local expert), the layer's own top_k
    for the "gather" exchange (every token keeps its k slots, the other ranks' masked).  Packed tensors are sliced, not re-quantised; the
    down-side rotation seed is advanced to the first kept column group, so the rotations stay those of the
    full layer (seed + 128 * global group)."""
    from .moe import WxA16Weights

    cls = type(moe)
    out = cls(None, hi - lo, moe.hidden_size, moe.intermediate_size, top_k, None, None)
    out.enable_timing = False
    out.enable_rotation_hoist = moe.enable_rotation_hoist
    out.rotation_hoist_threshold = moe.rotation_hoist_threshold
    offsets = moe._offsets_lists()
    for bs, w in moe.bit_weights.items():
        bit = int(bs)
        off = offsets[bs]
        s0, s1 = off[lo], off[hi]
        if s1 == s0:
            continue
        gu, dn = w.gate_up_packed, w.down_packed
        col0, col1 = s0 * bit // 8, s1 * bit // 8
        new_gu = dict(gu)
        new_gu.pop("indices_packed_gf", None)
        new_gu["indices_packed"] = gu["indices_packed"][2 * s0:2 * s1].contiguous()
        new_gu["norms"] = gu["norms"][2 * s0:2 * s1].contiguous()
        new_gu["shape"] = (2 * (s1 - s0), gu["shape"][1])
        new_dn = dict(dn)
        new_dn["indices_packed"] = dn["indices_packed"][:, col0:col1].contiguous()
        new_dn["norms"] = dn["norms"][:, s0 // 128:s1 // 128].contiguous()
        new_dn["shape"] = (dn["shape"][0], s1 - s0)
        new_dn["seed"] = int(dn["seed"]) + s0
        nw = WxA16Weights(bit, moe.hidden_size)
        nw.set_packed_data(new_gu, new_dn)
        out.bit_weights[bs] = nw
        local = [o - s0 for o in off[lo:hi + 1]]
        out.expert_offsets[bs] = torch.tensor(local, dtype=torch.long)
        out._expert_offsets_cpu[bs] = local
        out.inter_size_by_bit[bit] = s1 - s0
    out.bit_list = [b for b in moe.bit_list if str(b) in out.bit_weights]
    return out
