"""Drop-in MoE modules over packed mixed-bit weights, executed by libdmoq.

Public surface mirrors the reference modules
    WxA16Weights / WxA16BitPartitionedGroupMoE   quantization/wxa16/bit_partitioned_moe.py:32 / :268
    WxA8BitPartitionedGroupMoE                   quantization/wxa8/bit_partitioned_moe.py:44
    WxFP8BitPartitionedGroupMoE                  quantization/wxfp8/bit_partitioned_moe.py:40
    WxFP4BitPartitionedGroupMoE                  quantization/wxfp4/bit_partitioned_moe.py:42
(same constructor, ``from_metadata`` / ``from_build_block`` / ``from_wxa16``, the
same ``state_dict`` keys and attribute names) so a packed checkpoint loads
unchanged.  What differs is how ``forward`` runs: routing, rotation +
activation quantisation, both grouped GEMMs with their epilogues and the
combine are CUDA kernels behind a C ABI, with no host synchronisation and no
per-expert Python loop.  Derived tensors (group-first indices, LUTs, rotation
stacks) are runtime-only and never enter ``state_dict``.
"""
from __future__ import annotations

import ctypes as C
import math
import os
import time
import weakref
from typing import Dict, List, Optional

import torch
import torch.nn as nn

from . import _lib
from . import format as fmt
from ._lib import A16, A8, FP8, FP4, EPI_PLAIN, EPI_SILU, EPI_WEIGHTED, MAX_POOLS, TILE_M, Pool, Route, check, ptr

GROUP = fmt.GROUP_SIZE
# Device memory this process may spend on resident weight images of the fp16 / INT8 / e4m3 modes (all layers
# together; a 2-bit pool's INT8 image is four times its packed size).  Layers built after it runs out expand
# transient images per forward instead.
IMAGE_BUDGET = {"bytes_left": int(os.environ.get("DMOQ_IMAGE_BUDGET_GB", "96")) << 30}


def _return_image_budget(n: int) -> None:
    IMAGE_BUDGET["bytes_left"] += n


_META_KEYS = ("seed", "group_size", "shape", "bit_width", "rotation", "orig_dtype")


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _as_int(v) -> int:
    return int(v.item()) if torch.is_tensor(v) else int(v)


# =========================================================================== storage

class WxA16Weights(nn.Module):
    """Packed gate_up / down weights of one bit width.

    Buffers ``gate_up_{indices_packed,codebook,norms}`` and ``down_{...}`` are the
    checkpoint payload; the python-valued metadata (seed, group_size, shape, ...)
    lives in attributes, exactly as in the reference class.
    """

    def __init__(self, bit_width: int, hidden_size: int):
        super().__init__()
        self.bit_width = bit_width
        self.hidden_size = hidden_size
        self._cache = {"gate_up": None, "down": None}
        for side in ("gate_up", "down"):
            for key in _META_KEYS:
                setattr(self, f"_{side}_{key}", None)

    def _apply(self, fn, *args, **kwargs):
        ret = super()._apply(fn, *args, **kwargs)
        self._cache = {"gate_up": None, "down": None}
        return ret

    def _packed(self, side: str) -> dict:
        d = self._cache[side]
        if d is None:
            d = {name[len(side) + 1:]: buf for name, buf in self.named_buffers() if name.startswith(side + "_")}
            for key in _META_KEYS:
                val = getattr(self, f"_{side}_{key}")
                if val is not None:
                    d[key] = val
            self._cache[side] = d
        return d

    @property
    def gate_up_packed(self) -> dict:
        return self._packed("gate_up")

    @gate_up_packed.setter
    def gate_up_packed(self, value):
        self._cache["gate_up"] = value

    @property
    def down_packed(self) -> dict:
        return self._packed("down")

    @down_packed.setter
    def down_packed(self, value):
        self._cache["down"] = value

    def set_packed_data(self, gate_up_packed: Optional[dict], down_packed: Optional[dict]) -> None:
        """Register the tensors of both dicts as buffers and keep their metadata."""
        for side, packed in (("gate_up", gate_up_packed), ("down", down_packed)):
            if packed is None:
                continue
            for key, value in packed.items():
                if isinstance(value, torch.Tensor):
                    self.register_buffer(f"{side}_{key}", value)
            for key in _META_KEYS:
                setattr(self, f"_{side}_{key}", packed.get(key))
            self._cache[side] = None

    @classmethod
    def from_metadata(cls, bit_width: int, hidden_size: int, gate_up_meta: dict, down_meta: dict) -> "WxA16Weights":
        """Placeholder buffers of the saved shapes; ``load_state_dict(assign=True)`` fills them."""
        def blank(meta: dict) -> dict:
            return {
                "indices_packed": torch.empty(meta["indices_packed_shape"], dtype=torch.uint8),
                "codebook": torch.empty(meta["codebook_shape"], dtype=torch.float16),
                "norms": torch.empty(meta["norms_shape"], dtype=torch.float16),
                "seed": meta["seed"], "group_size": meta["group_size"], "shape": tuple(meta["shape"]),
                "bit_width": meta["bit_width"], "rotation": meta["rotation"], "orig_dtype": meta["orig_dtype"],
            }
        w = cls(bit_width, hidden_size)
        w.set_packed_data(blank(gate_up_meta), blank(down_meta))
        return w


# =========================================================================== runtime pools

def _true_div_half(norms_gf: torch.Tensor, divisor: float) -> torch.Tensor:
    """fp16 / scalar with an IEEE fp32 division (not a reciprocal multiply), result fp16."""
    d = torch.full((1,), divisor, dtype=torch.float32, device=norms_gf.device)
    return (norms_gf.float() / d).half().contiguous()


def _group_first_device(indices_packed: torch.Tensor, bit: int, k: int, device) -> torch.Tensor:
    """(N, K*bit/8) -> (K/128, N, 16*bit) on the device through the library."""
    lib = _lib.load()
    src = indices_packed.to(device).contiguous()
    n = src.shape[0]
    dst = torch.empty((k // GROUP, n, 16 * bit), dtype=torch.uint8, device=device)
    check(lib.dmoq_convert_group_first(ptr(src), n, k, bit, ptr(dst), _stream()), "dmoq_convert_group_first")
    return dst


def _widen_device(idx_gf: torch.Tensor, bit: int) -> torch.Tensor:
    """Group-first 1- or 2-bit indices (G, N, 16*bit) -> (G, N, 64): one code per 4-bit field."""
    lib = _lib.load()
    dst = torch.empty(idx_gf.shape[:2] + (64,), dtype=torch.uint8, device=idx_gf.device)
    check(lib.dmoq_widen_indices(ptr(idx_gf), idx_gf.numel(), bit, ptr(dst), _stream()), "dmoq_widen_indices")
    return dst


def _mode_lut(mode: int, bit: int, codebook: torch.Tensor, device):
    """(lut tensor, act_scale, e0, norm_factor, identity) for one codebook in one activation mode."""
    cb = codebook.detach().cpu()
    if mode == A16:
        lut16 = cb.half()
        ident = 0
        if bit == 8:   # uniform codebook whose fp16 entries are exactly fp16((i - 128) * step): computable, no table needed
            step = lut16[129].float()
            ident = int(torch.equal(((torch.arange(256, dtype=torch.float32) - 128.0) * step).half(), lut16))
        return lut16.to(device).contiguous(), 1.0, 0, 1.0, ident
    if mode == A8:
        if bit == 8 and fmt.is_uniform_codebook(cb):
            return torch.zeros(256, dtype=torch.int8, device=device), fmt.uniform_codebook_step(cb), 0, 1.0, 1
        lut, step = fmt.build_int8_codebook(cb)
        return lut.to(device), step, 0, 1.0, 0
    if mode == FP8:
        lut, scale = fmt.build_fp8_codebook(cb)
        return lut.view(torch.uint8).to(device), scale, 0, 1.0, 0
    if mode == FP4:
        nib, e0, resid, _ = fmt.build_e2m1_codebook(cb)
        return nib.to(device), 1.0, int(e0), float(resid), 0
    raise ValueError(f"unknown mode {mode}")


class _PoolRuntime:
    """Device tensors of one bit pool plus the dmoq_pool_t that points at them."""

    def __init__(self, *, key: str, bit: int, mode: int, n_members: int, inter: int, hidden: int,
                 gu: dict, dn: dict, device, hoisted: bool, shared: bool = False):
        self.key, self.bit, self.mode = key, bit, mode
        self.n_members, self.inter, self.hidden = n_members, inter, hidden
        self.hoisted, self.shared = hoisted, shared
        gs = int(gu["group_size"])
        if gs != GROUP or int(dn["group_size"]) != GROUP:
            raise ValueError(f"group_size must be {GROUP}, got {gs}/{dn['group_size']}")
        if hidden % GROUP or inter % GROUP:
            raise ValueError("hidden and intermediate sizes must be multiples of 128")
        self.gu_idx = _group_first_device(gu["indices_packed"], bit, hidden, device)
        self.dn_idx = _group_first_device(dn["indices_packed"], bit, n_members * inter, device)
        # the tensor-core GEMM (fp16 / INT8 / e4m3 operand modes) reads 1- and 2-bit codes widened to 4-bit fields;
        # the packed copy stays for the warp-level kernel
        self.gu_idx_wide = self.dn_idx_wide = None
        if bit <= 2 and mode in (A16, A8, FP8):
            self.gu_idx_wide, self.dn_idx_wide = _widen_device(self.gu_idx, bit), _widen_device(self.dn_idx, bit)
        lut_g, s_g, e0_g, f_g, ident_g = _mode_lut(mode, bit, gu["codebook"], device)
        lut_d, s_d, e0_d, f_d, ident_d = _mode_lut(mode, bit, dn["codebook"], device)
        self.gu_lut, self.dn_lut = lut_g, lut_d
        gn = _true_div_half(gu["norms"].to(device).t().contiguous(), math.sqrt(GROUP))
        dnn = _true_div_half(dn["norms"].to(device).t().contiguous(), math.sqrt(GROUP))
        if f_g != 1.0:
            gn = (gn.float() * f_g).half().contiguous()
        if f_d != 1.0:
            dnn = (dnn.float() * f_d).half().contiguous()
        self.gu_norm, self.dn_norm = gn, dnn
        self.gu_rot = fmt.generate_batch_rotation_matrices(GROUP, _as_int(gu["seed"]), hidden // GROUP, GROUP,
                                                           device, torch.float16)
        self.dn_rot = fmt.generate_batch_rotation_matrices(GROUP, _as_int(dn["seed"]), n_members * inter // GROUP,
                                                           GROUP, device, torch.float16)
        self.identity = int(ident_g and ident_d)
        if ident_g != ident_d:
            raise ValueError("gate_up and down must both (or neither) use the uniform 8-bit codebook")
        self.c = Pool()
        c = self.c
        c.bit, c.mode, c.n_members, c.inter = bit, mode, n_members, inter
        c.hoisted = int(hoisted)
        c.gu_idx, c.gu_norm = self.gu_idx.data_ptr(), self.gu_norm.data_ptr()
        c.dn_idx, c.dn_norm = self.dn_idx.data_ptr(), self.dn_norm.data_ptr()
        c.gu_lut, c.dn_lut = self.gu_lut.data_ptr(), self.dn_lut.data_ptr()
        c.identity_lut = self.identity
        c.gu_e0, c.dn_e0 = e0_g, e0_d
        c.gu_act_scale, c.dn_act_scale = s_g, s_d
        c.gu_rot, c.dn_rot = self.gu_rot.data_ptr(), self.dn_rot.data_ptr()
        if self.gu_idx_wide is not None:
            c.gu_idx_wide, c.dn_idx_wide = self.gu_idx_wide.data_ptr(), self.dn_idx_wide.data_ptr()
        # weight images (codewords looked up once, operand-row layout): sizes now, tensors on demand
        lib = _lib.load()
        self.img_bytes = (int(lib.dmoq_weight_image_bytes(C.byref(c), 0, hidden)),
                          int(lib.dmoq_weight_image_bytes(C.byref(c), 1, hidden)))
        self.norm_img = [None, None]     # fp32 column norms in image row order (kept once built)
        self.img = [None, None]          # resident images (FP4: the load-time fold; other modes on request)

    def build_norm_images(self) -> None:
        """fp32 norms in image row order for both projections (small; kept for the life of the pool)."""
        if self.norm_img[0] is not None:
            return
        lib = _lib.load()
        dev = self.gu_idx.device
        for side, (G, N) in enumerate(((self.hidden // GROUP, self.n_members * 2 * self.inter),
                                       (self.n_members * self.inter // GROUP, self.hidden))):
            nimg = torch.empty((G, N), dtype=torch.float32, device=dev)
            scratch = torch.empty(max(self.img_bytes[side], 16), dtype=torch.uint8, device=dev)
            check(lib.dmoq_expand_weights(C.byref(self.c), side, self.hidden, ptr(scratch), ptr(nimg), _stream()),
                  "dmoq_expand_weights")
            self.norm_img[side] = nimg
        self.c.gu_norm_img, self.c.dn_norm_img = self.norm_img[0].data_ptr(), self.norm_img[1].data_ptr()

    def build_resident_images(self) -> None:
        """Both weight images kept in device memory (WxFP4: the reference's load-time fold into e2m1)."""
        if self.img[0] is not None:
            return
        lib = _lib.load()
        dev = self.gu_idx.device
        first = self.norm_img[0] is None
        for side in (0, 1):
            G, N = ((self.hidden // GROUP, self.n_members * 2 * self.inter) if side == 0
                    else (self.n_members * self.inter // GROUP, self.hidden))
            img = torch.empty(max(self.img_bytes[side], 16), dtype=torch.uint8, device=dev)
            nimg = torch.empty((G, N), dtype=torch.float32, device=dev) if first else None
            check(lib.dmoq_expand_weights(C.byref(self.c), side, self.hidden, ptr(img), ptr(nimg), _stream()),
                  "dmoq_expand_weights")
            self.img[side] = img
            if first:
                self.norm_img[side] = nimg
        self.c.gu_norm_img, self.c.dn_norm_img = self.norm_img[0].data_ptr(), self.norm_img[1].data_ptr()

    # bytes per activation-code row / scale row for K columns in this pool's mode
    def code_bytes(self, k: int) -> int:
        return {A16: 2 * k, A8: k, FP8: k, FP4: k // 2}[self.mode]

    def scale_bytes(self, k: int) -> int:
        return {A16: 0, A8: 2 * (k // GROUP), FP8: 2 * (k // GROUP), FP4: k // 32}[self.mode]


class _Workspace:
    """Per-token-count buffers of one forward."""
    pass


class _Engine:
    """Everything a module needs on one device in one activation mode."""

    WORKSPACE_CACHE = 16   # per-token-count buffer sets kept (a serving loop sees many batch sizes)

    def __init__(self, module: "WxA16BitPartitionedGroupMoE", device):
        self.device = device
        self.lib = _lib.load()
        m = module
        self.hidden = m.hidden_size
        self.top_k = m.top_k
        self.E = m.num_experts
        offsets = m._offsets_lists()
        bit_keys = list(m.bit_weights.keys())

        # which bits does each expert use -> virtual experts when more than one
        uses: List[List[int]] = [[] for _ in range(self.E)]
        for pi, bs in enumerate(bit_keys):
            off = offsets[bs]
            for e in range(self.E):
                if off[e + 1] > off[e]:
                    uses[e].append(pi)
        self.mult = max(1, max((len(u) for u in uses), default=1))
        self.E_v = self.E * self.mult
        self.k_v = self.top_k * self.mult

        shared_packs = m._shared_packs()
        self.has_shared = shared_packs is not None
        self.shared_torch = (m.shared_expert is not None and m.shared_expert_gate is not None
                             and shared_packs is None)
        n_entries = self.E_v + (1 if self.has_shared else 0)
        expert_pool = [-1] * n_entries
        expert_rank = [0] * n_entries
        self.slot_valid = None
        if self.mult > 1:
            valid = torch.zeros(self.E, self.mult, dtype=torch.bool)
            for e, u in enumerate(uses):
                valid[e, :len(u)] = True
            self.slot_valid = valid.to(device)

        self.pools: List[_PoolRuntime] = []
        for pi, bs in enumerate(bit_keys):
            w = m.bit_weights[bs]
            bit = int(bs)
            off = offsets[bs]
            members = [e for e in range(self.E) if off[e + 1] > off[e]]
            if not members:
                continue
            sizes = {off[e + 1] - off[e] for e in members}
            if len(sizes) != 1:
                raise NotImplementedError(
                    f"bit pool {bs}: members have different intermediate sizes {sorted(sizes)}; "
                    "the grouped kernels need one size per pool")
            inter = sizes.pop()
            for rank, e in enumerate(members):
                if off[e] != rank * inter:
                    raise NotImplementedError("expert_offsets must be dense (start = rank * inter)")
                v = e * self.mult + uses[e].index(pi)
                expert_pool[v] = len(self.pools)
                expert_rank[v] = rank
            expect = len(members) * self.top_k / max(self.E, 1)
            hoisted = bool(m.enable_rotation_hoist) and expect > float(m.rotation_hoist_threshold)
            self.pools.append(_PoolRuntime(
                key=bs, bit=bit, mode=m._pool_mode(bit), n_members=len(members), inter=inter,
                hidden=self.hidden, gu=w.gate_up_packed, dn=w.down_packed, device=device, hoisted=hoisted))
        if self.has_shared:
            gu, dn, bit, inter = shared_packs
            expert_pool[self.E_v] = len(self.pools)
            expert_rank[self.E_v] = 0
            self.pools.append(_PoolRuntime(
                key="shared", bit=bit, mode=m._pool_mode(bit, shared=True), n_members=1, inter=inter,
                hidden=self.hidden, gu=gu, dn=dn, device=device, hoisted=True, shared=True))
        if len(self.pools) > MAX_POOLS:
            raise NotImplementedError(f"at most {MAX_POOLS} pools are supported")
        self.inter_max = max(p.inter for p in self.pools)
        i32 = dict(dtype=torch.int32, device=device)
        self.expert_pool = torch.tensor(expert_pool, **i32)
        self.expert_rank = torch.tensor(expert_rank, **i32)
        self.pool_hoisted = torch.tensor([int(p.hoisted) for p in self.pools] + [0] * (MAX_POOLS - len(self.pools)), **i32)
        self.pool_array = (Pool * len(self.pools))()
        # small batches: layers whose pools (of more than a few experts) run on the INT8 / e4m3 tcgen05 GEMM keep
        # 128-row tiles, that kernel is the faster one at every batch size; fp16-operand layers go to the warp-level
        # kernel's 32-row tiles (their tcgen05 form needs two operand steps per group and is no faster there)
        def _tc(p):
            if p.mode == A8:
                return p.bit != 8 or bool(p.identity)
            return p.mode == FP8 and p.bit != 8
        self._ws: Dict[int, _Workspace] = {}
        self.last_launches = 0
        # Weight images (dmoq_expand_weights): a pool's codewords looked up once and kept in operand-row layout, so the
        # tensor-core GEMM streams them with TMA copies.  WxFP4 pools need theirs (the reference folds codebooks into
        # e2m1 at load time too, within its byte budget); the other modes trade memory for speed the same way:
        #   "auto"       resident images while the process-wide budget lasts, else a transient image per forward once
        #                an expert expects enough rows to repay the expansion
        #   "transient"  never resident (FP4 excepted): packed weights stay the only copy
        #   "always"     resident regardless of the budget;   "never": index expansion inside the GEMM only
        self.weight_images = getattr(m, "weight_images", "auto")
        self.image_min_rows = int(getattr(m, "weight_image_min_rows", 192))
        fold_budget = int(getattr(m, "_FOLD_BYTES_BUDGET", 16 << 30))
        self._img_scratch = None
        for p in self.pools:
            need = sum(p.img_bytes)
            if need == 0 or self.weight_images == "never":
                continue
            if p.mode == FP4:
                ok = need <= fold_budget
                fold_budget -= need if ok else 0
            elif self.weight_images == "always":
                ok = True
            elif self.weight_images == "auto":
                ok = need <= IMAGE_BUDGET["bytes_left"]
                if ok:
                    IMAGE_BUDGET["bytes_left"] -= need
                    weakref.finalize(self, _return_image_budget, need)   # handed back when this engine goes away
            else:
                ok = False
            if ok:
                p.build_resident_images()
        self.all_tensor_core = all(_tc(p) or p.img[0] is not None or p.n_members < 8 for p in self.pools)
        # small batches of a WxA16 layer take the streaming decode kernels (packed indices, 32-row tiles, one launch for
        # all pools): every pool fp16, 8-bit pools only with the computable uniform codebook
        self.decode_ok = (bool(getattr(m, "enable_decode_kernels", True)) and self.hidden % 256 == 0
                          and all(p.mode == A16 and (p.bit != 8 or p.identity) for p in self.pools))

    def _image_scratch(self) -> torch.Tensor:
        """One buffer for the transient image of whichever pool / projection is being computed."""
        if self._img_scratch is None:
            need = max(max(p.img_bytes) for p in self.pools)
            self._img_scratch = torch.empty(max(need, 16), dtype=torch.uint8, device=self.device)
        return self._img_scratch

    def prepare(self, T: int) -> "_Workspace":
        """Everything a forward of ``T`` tokens allocates or copies from the host, done now: the workspace, the
        routed-order code tables, norm images and the transient image buffer.  A stream capture must find all of it
        in place (allocations and host copies are not capturable)."""
        ws = self.workspace(T)
        for p in self.pools:
            mode = self._image_mode(p, T, ws.tile_m)
            if mode:
                p.build_norm_images()
                self._sorted_tables(ws)
            if mode == 2:
                self._image_scratch()
        return ws

    def _image_mode(self, p: "_PoolRuntime", T: int, tile_m: int) -> int:
        """0: no image (index expansion inside the GEMM), 1: resident image, 2: transient image this forward."""
        if tile_m != TILE_M or self.weight_images == "never":
            return 0
        if p.img[0] is not None:
            return 1
        if p.mode == FP4 or sum(p.img_bytes) == 0:
            return 0
        expect = T if p.shared else T * self.k_v / max(self.E_v, 1)
        return 2 if expect >= self.image_min_rows else 0

    # ------------------------------------------------------------------ per-T buffers
    def workspace(self, T: int) -> _Workspace:
        ws = self._ws.pop(T, None)
        if ws is not None:
            self._ws[T] = ws          # most recently used last
            return ws
        # least recently used first; a captured graph keeps its own reference to the workspace it was
        # captured with, so dropping an entry here never frees memory a graph still replays against
        if len(self._ws) >= self.WORKSPACE_CACHE:
            self._ws.pop(next(iter(self._ws)))
        dev = self.device
        ws = _Workspace()
        R = T * self.k_v + (T if self.has_shared else 0)
        ws.R = R
        n_entries = self.E_v + (1 if self.has_shared else 0)
        i32 = dict(dtype=torch.int32, device=dev)
        u8 = dict(dtype=torch.uint8, device=dev)
        ws.expert_rows = torch.zeros(n_entries + 1, **i32)
        ws.sorted_tokens = torch.zeros(max(R, 1), **i32)
        ws.sorted_weights = torch.zeros(max(R, 1), dtype=torch.float32, device=dev)
        ws.row_of = torch.full((max(R, 1),), -1, **i32)
        ws.a_row = torch.zeros(max(R, 1), **i32)
        ws.pool_rows = torch.zeros(MAX_POOLS, **i32)
        ws.n_tiles = torch.zeros(2 * MAX_POOLS, **i32)
        # small batches (a few rows per expert) use 32-row tiles: every packed weight is still expanded once
        # per expert, but far fewer padded rows go through the MMAs
        # few rows per expert: the warp-level kernel runs 32-row tiles so that the packed weights of an active expert
        # are not padded to 128 rows; pools the tcgen05 kernel covers stay on 128-row tiles, it is the faster one
        # at every batch size (0.53 ms against 0.74 ms at 64 tokens on the 35B-A3B-like INT8 layer)
        small = T <= 256 and T * self.k_v <= 8 * self.E_v
        ws.decode = small and self.decode_ok
        ws.tile_m = 32 if (small and (self.decode_ok or not self.all_tensor_core)) else TILE_M
        ws.tile_cap = (R + ws.tile_m - 1) // ws.tile_m + n_entries
        ws.tiles = torch.zeros(ws.tile_cap, 4, **i32)
        bases, total = [], 0
        ws.act_codes, ws.act_scales = [], []
        for p in self.pools:
            cap = T if p.hoisted else T * min(self.k_v, p.n_members)
            bases.append(total if not p.hoisted else 0)
            if not p.hoisted:
                total += cap
            p_cap = max(cap, 1)
            ws.act_codes.append(torch.empty(p_cap * p.code_bytes(self.hidden), **u8))
            ws.act_scales.append(torch.empty(max(p_cap * p.scale_bytes(self.hidden), 16), **u8))
        ws.caps = [T if p.hoisted else T * min(self.k_v, p.n_members) for p in self.pools]
        ws.pool_src = torch.zeros(max(total, 1), **i32)
        ws.pool_src_base_host = bases
        ws.pool_src_base = torch.tensor(bases + [0] * (MAX_POOLS - len(bases)), **i32)
        ws.route_ws = torch.empty(max(self.lib.dmoq_route_workspace_bytes(T, self.k_v, self.E_v), 16), **u8)
        ws.act = torch.empty(max(R, 1), self.inter_max, dtype=torch.float16, device=dev)
        code_b = max(p.code_bytes(self.inter_max) for p in self.pools)
        scale_b = max(max(p.scale_bytes(self.inter_max) for p in self.pools), 1)
        ws.dn_codes = torch.empty(max(R, 1) * code_b, **u8)
        ws.dn_scales = torch.empty(max(R, 1) * scale_b, **u8)
        ws.dn = torch.empty(max(R, 1), self.hidden, dtype=torch.float16, device=dev)
        r = Route()
        r.T, r.top_k, r.E = T, self.k_v, self.E_v
        r.has_shared, r.tile_m, r.n_pools = int(self.has_shared), ws.tile_m, len(self.pools)
        r.expert_pool, r.expert_rank = self.expert_pool.data_ptr(), self.expert_rank.data_ptr()
        r.expert_rows = ws.expert_rows.data_ptr()
        r.sorted_tokens, r.sorted_weights = ws.sorted_tokens.data_ptr(), ws.sorted_weights.data_ptr()
        r.row_of, r.a_row = ws.row_of.data_ptr(), ws.a_row.data_ptr()
        r.pool_rows, r.pool_src = ws.pool_rows.data_ptr(), ws.pool_src.data_ptr()
        r.pool_src_base = ws.pool_src_base.data_ptr()
        r.tiles, r.n_tiles, r.tile_cap = ws.tiles.data_ptr(), ws.n_tiles.data_ptr(), ws.tile_cap
        r.pool_hoisted = self.pool_hoisted.data_ptr()
        ws.route = r
        # the same tables for GEMMs that read an activation-code table already in routed-row order (a_row = NULL)
        rs = Route.from_buffer_copy(r)
        rs.a_row = None
        ws.route_sorted = rs
        ws.sorted_codes = ws.sorted_scales = None
        self._ws[T] = ws
        return ws

    def _sorted_tables(self, ws: "_Workspace"):
        """Gate_up-side activation codes and scales in routed-row order, shared by the pools of one forward (each
        pool's rows are gathered right before its GEMM).  Row pitch: ``sorted_stride`` elements, a multiple of 512
        so that a row's fp16 scales sit on 8-byte boundaries."""
        if ws.sorted_codes is None:
            stride = (self.hidden + 511) // 512 * 512
            ws.sorted_stride = stride
            rows = max(ws.R, 1)
            ws.sorted_codes = torch.empty(rows * max(p.code_bytes(stride) for p in self.pools), dtype=torch.uint8,
                                          device=self.device)
            ws.sorted_scales = torch.empty(max(rows * max(p.scale_bytes(stride) for p in self.pools), 16),
                                           dtype=torch.uint8, device=self.device)
        return ws.sorted_codes, ws.sorted_scales, ws.sorted_stride

    # ------------------------------------------------------------------ one forward
    def run(self, x: torch.Tensor, topk_w: torch.Tensor, topk_idx: torch.Tensor,
            shared_w: Optional[torch.Tensor], prof=None, partials=None) -> torch.Tensor:
        """x (T, H) bf16/fp16 contiguous -> y (T, H) same dtype."""
        lib = self.lib
        T = x.shape[0]
        ws = self.workspace(T)
        s = _stream()
        is_bf16 = int(x.dtype == torch.bfloat16)
        if self.mult > 1:
            # an expert stored in several bit widths is one virtual expert per width
            lanes = torch.arange(self.mult, device=x.device)
            v_idx = topk_idx.long().unsqueeze(-1) * self.mult + lanes
            ok = self.slot_valid[topk_idx.long()]
            topk_idx = torch.where(ok, v_idx, torch.full_like(v_idx, -1)).reshape(T, -1)
            topk_w = topk_w.unsqueeze(-1).expand(-1, -1, self.mult).reshape(T, -1)
        topk_idx = topk_idx.to(torch.int64).contiguous()
        topk_w = topk_w.to(torch.float32).contiguous()
        if shared_w is not None:
            shared_w = shared_w.to(torch.float32).contiguous()
        mark = prof if prof is not None else (lambda name: None)

        check(lib.dmoq_route_build(C.byref(ws.route), ptr(topk_idx), ptr(topk_w), ptr(shared_w),
                                   ptr(ws.route_ws), ws.route_ws.numel(), s), "dmoq_route_build")
        mark("route")
        # kernels launched by this forward: routing is one fused launch for <= 1024 routed pairs, else three
        self.last_launches = (1 if T * self.k_v <= 1024 and T <= 4096 else 3) + 4 * len(self.pools) + 1
        for i, p in enumerate(self.pools):
            p.c.act_cap_rows = ws.caps[i]
            p.c.act_codes, p.c.act_scales = ws.act_codes[i].data_ptr(), ws.act_scales[i].data_ptr()
            self.pool_array[i] = p.c
        if ws.decode:
            # small batch (WxA16): five launches for all pools -- rotation, gate_up + SiLU, rotation, down, combine
            n = len(self.pools)
            check(lib.dmoq_moe_decode_rotate(C.byref(ws.route), self.pool_array, n, self.hidden, ptr(x), is_bf16, s),
                  "dmoq_moe_decode_rotate")
            mark("decode_rotate")
            check(lib.dmoq_moe_decode_gateup(C.byref(ws.route), self.pool_array, n, self.hidden,
                                             ptr(ws.act), self.inter_max, s), "dmoq_moe_decode_gateup")
            mark("decode_gate_up_silu")
            check(lib.dmoq_moe_decode_rotate_down(C.byref(ws.route), self.pool_array, n, ptr(ws.act), self.inter_max,
                                                  ptr(ws.dn_codes), self.inter_max, s), "dmoq_moe_decode_rotate_down")
            mark("decode_rotate_down")
            check(lib.dmoq_moe_decode_down(C.byref(ws.route), self.pool_array, n, self.hidden,
                                           ptr(ws.dn_codes), self.inter_max, ptr(ws.dn), s), "dmoq_moe_decode_down")
            mark("decode_down")
            self.last_launches = (1 if T * self.k_v <= 1024 and T <= 4096 else 3) + 5
            y = torch.empty_like(x)
            check(lib.dmoq_combine_weighted(C.byref(ws.route), ptr(ws.dn), self.hidden, ptr(y), is_bf16, s),
                  "dmoq_combine_weighted")
            mark("combine")
            return y
        for i, p in enumerate(self.pools):
            src_row = None if p.hoisted else C.c_void_p(ws.pool_src.data_ptr() + 4 * ws.pool_src_base_host[i])
            n_dev = None if p.hoisted else C.c_void_p(ws.pool_rows.data_ptr() + 4 * i)
            check(lib.dmoq_rotate_quant(p.mode, ptr(x), is_bf16, self.hidden, ptr(p.gu_rot), None, src_row,
                                        ws.caps[i], n_dev, p.c.gu_act_scale, ptr(ws.act_codes[i]),
                                        ptr(ws.act_scales[i]), s), "dmoq_rotate_quant")
        mark("rotate_quant")
        img_modes = [self._image_mode(p, T, ws.tile_m) for p in self.pools]
        merged = (partials is None and len(self.pools) > 1 and all(m == 1 for m in img_modes)
                  and len({p.mode for p in self.pools}) == 1 and self.pools[0].mode != FP4)
        if merged:
            # every pool has a resident weight image and the same activation mode: one GEMM launch per projection walks
            # the tile lists of all pools (small pools cost no launches of their own)
            codes, scales, stride = self._sorted_tables(ws)
            for i, p in enumerate(self.pools):
                p.build_norm_images()
                p.c.gu_img, p.c.dn_img = p.img[0].data_ptr(), p.img[1].data_ptr()
                self.pool_array[i] = p.c
                has_scales = p.scale_bytes(self.hidden) > 0
                check(lib.dmoq_gather_rows(C.byref(ws.route), i, ptr(ws.act_codes[i]), p.code_bytes(self.hidden),
                                           p.code_bytes(self.hidden), ptr(codes), p.code_bytes(stride),
                                           ptr(ws.act_scales[i]) if has_scales else None, p.scale_bytes(self.hidden),
                                           p.scale_bytes(self.hidden), ptr(scales) if has_scales else None,
                                           p.scale_bytes(stride), s), "dmoq_gather_rows")
            mark("gather")
            ids = (C.c_int32 * len(self.pools))(*range(len(self.pools)))
            check(lib.dmoq_grouped_gemm_pools(C.byref(ws.route_sorted), self.pool_array, ids, len(self.pools), 0, EPI_SILU,
                                              self.hidden, ptr(codes), ptr(scales), stride, ptr(ws.act), self.inter_max, s),
                  "dmoq_grouped_gemm_pools(gate_up)")
            mark("gate_up_silu:all")
            for i, p in enumerate(self.pools):
                check(lib.dmoq_rotate_quant_down(C.byref(ws.route), self.pool_array, i, ptr(ws.act), self.inter_max,
                                                 ptr(ws.dn_codes), ptr(ws.dn_scales), self.inter_max, s),
                      "dmoq_rotate_quant_down")
            mark("rotate_quant_down")
            check(lib.dmoq_grouped_gemm_pools(C.byref(ws.route), self.pool_array, ids, len(self.pools), 1, EPI_PLAIN,
                                              self.hidden, ptr(ws.dn_codes), ptr(ws.dn_scales), self.inter_max,
                                              ptr(ws.dn), self.hidden, s), "dmoq_grouped_gemm_pools(down)")
            mark("down:all")
            self.last_launches = (1 if T * self.k_v <= 1024 and T <= 4096 else 3) + 3 * len(self.pools) + 3
            y = torch.empty_like(x)
            check(lib.dmoq_combine_weighted(C.byref(ws.route), ptr(ws.dn), self.hidden, ptr(y), is_bf16, s),
                  "dmoq_combine_weighted")
            mark("combine")
            return y
        # pool by pool: gate_up + SiLU, down-side rotation, down.  The down-side code / scale scratch and the transient
        # weight image are shared by all pools; stream order makes each consumer finish before the next producer writes
        for i, p in enumerate(self.pools):
            img = self._image_mode(p, T, ws.tile_m)
            if img:
                p.build_norm_images()
            p.c.gu_img = p.c.dn_img = None
            if img == 1:
                p.c.gu_img, p.c.dn_img = p.img[0].data_ptr(), p.img[1].data_ptr()
            scratch = self._image_scratch() if img == 2 else None
            if img == 2:
                check(lib.dmoq_expand_weights(C.byref(p.c), 0, self.hidden, ptr(scratch), None, s), "dmoq_expand_weights")
                p.c.gu_img = scratch.data_ptr()
                self.last_launches += 2
                mark("expand_gate_up:" + p.key)
            self.pool_array[i] = p.c
            part = None if partials is None else partials.get(("gate_up", p.key))
            if img:
                # the image-fed kernel takes whole tiles of the code table: this pool's rows go into routed-row order
                codes, scales, stride = self._sorted_tables(ws)
                has_scales = p.scale_bytes(self.hidden) > 0
                check(lib.dmoq_gather_rows(C.byref(ws.route), i, ptr(ws.act_codes[i]), p.code_bytes(self.hidden),
                                           p.code_bytes(self.hidden), ptr(codes), p.code_bytes(stride),
                                           ptr(ws.act_scales[i]) if has_scales else None, p.scale_bytes(self.hidden),
                                           p.scale_bytes(self.hidden), ptr(scales) if has_scales else None,
                                           p.scale_bytes(stride), s), "dmoq_gather_rows")
                self.last_launches += 1
                mark("gather:" + p.key)
                check(lib.dmoq_grouped_gemm(C.byref(ws.route_sorted), self.pool_array, i, 0, EPI_SILU, self.hidden,
                                            ptr(codes), ptr(scales), stride,
                                            ptr(ws.act), self.inter_max, ptr(part), s), "dmoq_grouped_gemm(gate_up)")
            else:
                check(lib.dmoq_grouped_gemm(C.byref(ws.route), self.pool_array, i, 0, EPI_SILU, self.hidden,
                                            ptr(ws.act_codes[i]), ptr(ws.act_scales[i]), self.hidden,
                                            ptr(ws.act), self.inter_max, ptr(part), s), "dmoq_grouped_gemm(gate_up)")
            mark("gate_up_silu:" + p.key)
            check(lib.dmoq_rotate_quant_down(C.byref(ws.route), self.pool_array, i, ptr(ws.act), self.inter_max,
                                             ptr(ws.dn_codes), ptr(ws.dn_scales), self.inter_max, s),
                  "dmoq_rotate_quant_down")
            mark("rotate_quant_down:" + p.key)
            if img == 2:
                check(lib.dmoq_expand_weights(C.byref(p.c), 1, self.hidden, ptr(scratch), None, s), "dmoq_expand_weights")
                p.c.dn_img = scratch.data_ptr()
                self.pool_array[i] = p.c
                mark("expand_down:" + p.key)
            part = None if partials is None else partials.get(("down", p.key))
            # plain fp16 rows; the routing weight and its bf16 rounding chain are applied by the combine, which
            # is bound by HBM and has arithmetic to spare
            check(lib.dmoq_grouped_gemm(C.byref(ws.route), self.pool_array, i, 1, EPI_PLAIN, self.hidden,
                                        ptr(ws.dn_codes), ptr(ws.dn_scales), self.inter_max,
                                        ptr(ws.dn), self.hidden, ptr(part), s), "dmoq_grouped_gemm(down)")
            mark("down:" + p.key)
        y = torch.empty_like(x)
        check(lib.dmoq_combine_weighted(C.byref(ws.route), ptr(ws.dn), self.hidden, ptr(y), is_bf16, s),
              "dmoq_combine_weighted")
        mark("combine")
        return y


class _EventProfiler:
    """CUDA-event stage timer: one event per stage boundary, one synchronise at the end."""

    def __init__(self):
        self.names: List[str] = []
        self.events = [torch.cuda.Event(enable_timing=True)]
        self.events[0].record()

    def __call__(self, name: str) -> None:
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self.names.append(name)
        self.events.append(ev)

    def stats(self) -> Dict[str, float]:
        torch.cuda.synchronize()
        out: Dict[str, float] = {}
        for i, name in enumerate(self.names):
            out[name] = out.get(name, 0.0) + self.events[i].elapsed_time(self.events[i + 1])
        return out


# =========================================================================== modules

class WxA16BitPartitionedGroupMoE(nn.Module):
    """Bit-partitioned MoE over packed weights, fp16 activations."""

    MODE = A16
    _DEVICE_CACHE_ATTRS = ("_engine", "_bit_ctx_cache", "_bit_ctx_device", "_graphs")

    def __init__(self, gate, num_experts: int, hidden_size: int, intermediate_size: int, top_k: int = 6,
                 shared_expert=None, shared_expert_gate=None):
        super().__init__()
        self.gate = gate
        self.num_experts = num_experts
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.top_k = top_k
        self.shared_expert = shared_expert
        self.shared_expert_gate = shared_expert_gate
        self.enable_timing = True
        self.last_timings: dict = {}
        self.enable_cuda_profile = False
        self.last_cuda_stats: dict = {}
        self.enable_rotation_hoist = True
        self.rotation_hoist_threshold = 1.5
        self.bit_weights = nn.ModuleDict()
        self.inter_size_by_bit: dict = {}
        self.expert_offsets: dict = {}
        self._expert_offsets_cpu: dict = {}
        self.bit_list: list = []
        self._engine: Optional[_Engine] = None
        # small batches replay a captured CUDA graph of the expert path (no per-launch host cost)
        self.enable_cuda_graph = True
        self.cuda_graph_max_tokens = 256
        self._graphs: Optional[dict] = None

    # ------------------------------------------------------------------ construction
    def _apply(self, fn, *args, **kwargs):
        ret = super()._apply(fn, *args, **kwargs)
        for attr in self._DEVICE_CACHE_ATTRS:
            if hasattr(self, attr):
                setattr(self, attr, None)
        return ret

    @classmethod
    @torch.no_grad()
    def from_build_block(cls, build_block, layer_metadata, group_size: int = GROUP):
        """Quantise a staged fp16 MoE block (reference: quantization/wxa16/bit_partitioned_moe.py:355).

        ``build_block`` must offer ``gate``, ``top_k``, optional ``shared_expert`` /
        ``shared_expert_gate`` and ``experts[e].sub_experts`` with ``_quant_bit``,
        ``gate_proj`` / ``up_proj`` / ``down_proj``; ``layer_metadata`` carries
        ``num_experts, hidden_size, intermediate_size, bit_list, expert_bit_indices``.
        Pool layout follows bit_partitioned_moe.py:120-166, seeds 42+bit / 42+bit+1000.
        """
        md = layer_metadata
        E, H = md["num_experts"], md["hidden_size"]
        moe = cls(gate=build_block.gate, num_experts=E, hidden_size=H,
                  intermediate_size=md["intermediate_size"], top_k=getattr(build_block, "top_k", 6),
                  shared_expert=getattr(build_block, "shared_expert", None),
                  shared_expert_gate=getattr(build_block, "shared_expert_gate", None))
        moe.bit_list = md["bit_list"]
        for bit in md["bit_list"]:
            counts = [len(md["expert_bit_indices"][e].get(bit, [])) for e in range(E)]
            total = sum(counts)
            if total == 0:
                continue
            offs = [0]
            for c in counts:
                offs.append(offs[-1] + c)
            ref = next(build_block.parameters())
            gate_up = torch.zeros(2 * total, H, dtype=ref.dtype, device=ref.device)
            down = torch.zeros(H, total, dtype=ref.dtype, device=ref.device)
            for e in range(E):
                sub = {s._quant_bit: s for s in build_block.experts[e].sub_experts}.get(bit)
                n = counts[e]
                if sub is None or n == 0:
                    continue
                s0 = offs[e]
                gate_up[2 * s0:2 * s0 + n] = sub.gate_proj.weight.data
                gate_up[2 * s0 + n:2 * offs[e + 1]] = sub.up_proj.weight.data
                down[:, s0:offs[e + 1]] = sub.down_proj.weight.data
            w = WxA16Weights(bit, H)
            w.set_packed_data(
                fmt.turboquant_quantize_packed_full(gate_up, bit, group_size, seed=42 + bit, keep_on_gpu=True),
                fmt.turboquant_quantize_packed_full(down, bit, group_size, seed=42 + bit + 1000, keep_on_gpu=True))
            moe.bit_weights[str(bit)] = w
            moe.expert_offsets[str(bit)] = torch.tensor(offs, dtype=torch.long, device=ref.device)
            moe._expert_offsets_cpu[str(bit)] = offs
            moe.inter_size_by_bit[bit] = total
        return moe

    @classmethod
    def from_metadata(cls, meta: dict, gate, shared_expert, shared_expert_gate):
        """Rebuild the module skeleton from ``meta.json`` (reference :462); tensors come from the state dict."""
        moe = cls(gate=gate, num_experts=meta["num_experts"], hidden_size=meta["hidden_size"],
                  intermediate_size=meta["intermediate_size"], top_k=meta["top_k"],
                  shared_expert=shared_expert, shared_expert_gate=shared_expert_gate)
        moe.bit_list = list(meta["bit_list"])
        moe.inter_size_by_bit = {int(k): v for k, v in meta["inter_size_by_bit"].items()}
        moe.expert_offsets = {b: torch.tensor(lst, dtype=torch.long) for b, lst in meta["expert_offsets"].items()}
        moe._expert_offsets_cpu = {b: list(lst) for b, lst in meta["expert_offsets"].items()}
        for bit_str, bm in meta["bits"].items():
            moe.bit_weights[bit_str] = WxA16Weights.from_metadata(int(bit_str), meta["hidden_size"],
                                                                  bm["gate_up"], bm["down"])
        moe.enable_timing = meta.get("enable_timing", True)
        return moe

    @classmethod
    def from_wxa16(cls, moe: "WxA16BitPartitionedGroupMoE"):
        """Switch an already loaded module to this activation mode in place (zero copy)."""
        if not isinstance(moe, WxA16BitPartitionedGroupMoE):
            raise TypeError(f"expected WxA16BitPartitionedGroupMoE, got {type(moe)}")
        moe.__class__ = cls
        moe._engine = None
        moe._graphs = None     # captured graphs belong to the old engine's buffers and activation mode
        return moe

    # ------------------------------------------------------------------ helpers
    def _pool_mode(self, bit: int, shared: bool = False) -> int:
        return self.MODE

    def _offsets_lists(self) -> Dict[str, List[int]]:
        if not self._expert_offsets_cpu:
            for bs, t in self.expert_offsets.items():
                self._expert_offsets_cpu[bs] = t.cpu().tolist()
        return self._expert_offsets_cpu

    def _shared_packs(self):
        """(gate_up dict, down dict, bit, inter) when the shared expert is three packed linears
        with one rotation seed for gate and up; None otherwise."""
        se = self.shared_expert
        if se is None or self.shared_expert_gate is None:
            return None
        parts = [getattr(se, n, None) for n in ("gate_proj", "up_proj", "down_proj")]
        if any(p is None or not hasattr(p, "packed_indices") for p in parts):
            return None
        g, u, d = parts
        same = (g.bit_width == u.bit_width == d.bit_width and g.seed == u.seed
                and g.group_size == u.group_size == d.group_size == GROUP
                and g.bias is None and u.bias is None and d.bias is None
                and torch.equal(g.codebook.cpu(), u.codebook.cpu()))
        if not same:
            return None
        gu = {"indices_packed": torch.cat([g.packed_indices, u.packed_indices.to(g.packed_indices.device)], 0),
              "norms": torch.cat([g.norms, u.norms.to(g.norms.device)], 0), "codebook": g.codebook,
              "seed": g.seed, "group_size": g.group_size}
        dn = {"indices_packed": d.packed_indices, "norms": d.norms, "codebook": d.codebook,
              "seed": d.seed, "group_size": d.group_size}
        return gu, dn, int(g.bit_width), int(g.out_features)

    def _get_engine(self, device) -> _Engine:
        eng = self._engine
        if eng is None or eng.device != device:
            eng = _Engine(self, device)
            self._engine = eng
            self._graphs = None
        return eng

    def _body(self, eng, x, prof=None, partials=None):
        """Router, shared-expert gate and the expert path for x (T, H)."""
        shared_w = None
        fuse_gate = False
        if x.is_cuda and eng.has_shared and hasattr(self.gate, "router_logits"):
            # a gate that can hand out its logits: softmax -> top-k (-> renormalise, as the gate says) and the shared
            # expert's gate share one launch
            from .kernels import fusable_shared_gate
            fuse_gate = fusable_shared_gate(self.shared_expert_gate, x) and self.top_k <= 32
        if fuse_gate:
            from .kernels import router_topk
            lg = self.gate.router_logits(x)
            fuse_gate = lg.is_cuda and lg.shape[-1] <= 1024
        if fuse_gate:
            topk_w, topk_idx, shared_w = router_topk(lg.reshape(-1, lg.shape[-1]), self.top_k,
                                                     renormalize=bool(getattr(self.gate, "norm_topk_prob", False)),
                                                     x=x, shared_gate=self.shared_expert_gate)
            gate_out = None
        else:
            gate_out = self.gate(x)
        if gate_out is None:
            pass
        elif isinstance(gate_out, tuple):
            _, topk_w, topk_idx = gate_out
        elif gate_out.is_cuda and gate_out.shape[-1] <= 1024 and self.top_k <= 32:
            from .kernels import fusable_shared_gate, router_topk
            if eng.has_shared and fusable_shared_gate(self.shared_expert_gate, x):   # the gate rides in the router launch
                topk_w, topk_idx, shared_w = router_topk(gate_out.reshape(-1, gate_out.shape[-1]), self.top_k,
                                                         x=x, shared_gate=self.shared_expert_gate)
            else:
                topk_w, topk_idx = router_topk(gate_out.reshape(-1, gate_out.shape[-1]), self.top_k)
        else:
            topk_w, topk_idx = gate_out.softmax(dim=-1).topk(self.top_k, dim=-1)
        if eng.has_shared and shared_w is None:
            shared_w = torch.sigmoid(self.shared_expert_gate(x)).reshape(-1)
        if prof is not None:
            prof("router")
        return eng.run(x, topk_w, topk_idx, shared_w, prof=prof, partials=partials)

    def _run_graphed(self, eng, x):
        """First call for a token count runs eagerly (also finishes one-time kernel set-up); the second call
        captures router + expert path into a CUDA graph; later calls copy x into the graph's static input and
        replay it.  The router must be capture-safe (no host synchronisation); set ``enable_cuda_graph = False``
        for one that is not."""
        if self._graphs is None:
            self._graphs = {}
        key = (x.shape[0], x.dtype)
        entry = self._graphs.get(key)
        if entry is None:
            self._graphs[key] = "warm"
            return self._body(eng, x)
        if entry == "warm":
            if len(self._graphs) > 8:
                self._graphs = {key: "warm"}
            static_x = x.clone()
            eng.prepare(x.shape[0])          # nothing may be allocated or copied from the host inside the capture
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                static_y = self._body(eng, static_x)
            # the graph replays raw pointers into the engine's tensors and into this token count's workspace:
            # the entry keeps both alive for as long as the graph exists
            entry = (graph, static_x, static_y, eng, eng.workspace(x.shape[0]))
            self._graphs[key] = entry
        graph, static_x, static_y = entry[:3]
        static_x.copy_(x)
        graph.replay()
        return static_y.clone()

    def set_cuda_profile(self, enabled: bool = True):
        """CUDA-event stage timing into ``last_cuda_stats`` (adds one synchronise per forward)."""
        self.enable_cuda_profile = bool(enabled)
        return self

    @torch.no_grad()
    def warmup_kernels(self, seq_len: int = 2048, batch_size: int = 1):
        """Run one dummy forward so load-time work (relayout, LUTs, rotations) is done up front."""
        device = next(self.gate.parameters()).device
        dummy = torch.randn(batch_size, seq_len, self.hidden_size, device=device, dtype=self.gate.weight.dtype)
        self.forward(dummy)
        torch.cuda.synchronize(device)
        with torch.cuda.device(device):
            self.check_device_status()

    @staticmethod
    def check_device_status() -> None:
        """Raise if a bounded wait of the tensor-core kernels ever ran out on the current device (the launch that
        hit it wrote unspecified output).  Synchronises the device; ``forward`` itself never does, so callers that
        want this check poll it at their own synchronisation points."""
        st = C.c_int32(0)
        check(_lib.load().dmoq_tc_status(C.byref(st)), "dmoq_tc_status")
        if st.value != 0:
            raise _lib.DmoqError(f"tensor-core kernel status word is {st.value}: a bounded device-side wait timed out")

    # ------------------------------------------------------------------ forward
    @torch.no_grad()
    def forward(self, hidden_states: torch.Tensor, _partials=None) -> torch.Tensor:
        t0 = time.time()
        if not hidden_states.is_cuda:
            raise _lib.DmoqError("the MoE layer runs on a CUDA device only (no CPU path)")
        if hidden_states.dtype not in (torch.bfloat16, torch.float16):
            raise TypeError(f"activations must be bf16 or fp16, got {hidden_states.dtype}")
        b, s, h = hidden_states.shape
        x = hidden_states.reshape(-1, h).contiguous()
        if x.shape[0] == 0:
            return torch.zeros_like(hidden_states)
        # every launch goes to the current stream of the tensors' own device, whichever device is current
        # for the caller (a model sharded over several GPUs in one process calls layers on all of them)
        with torch.cuda.device(x.device):
            eng = self._get_engine(x.device)
            prof = _EventProfiler() if self.enable_cuda_profile else None

            graphed = (self.enable_cuda_graph and prof is None and _partials is None
                       and x.shape[0] <= self.cuda_graph_max_tokens and not torch.cuda.is_current_stream_capturing())
            if graphed:
                y = self._run_graphed(eng, x)
            else:
                y = self._body(eng, x, prof, _partials)
            if eng.shared_torch:
                y = y + self.shared_expert(x) * torch.sigmoid(self.shared_expert_gate(x))
            if prof is not None:
                self.last_cuda_stats = prof.stats()
                self.check_device_status()    # the profiler has synchronised already
        if self.enable_timing:
            self.last_timings = {"total": time.time() - t0, "active_bits": len(eng.pools)}
        return y.reshape(b, s, h)


class WxA8BitPartitionedGroupMoE(WxA16BitPartitionedGroupMoE):
    """INT8 activations: per-token per-group symmetric codes, int32 group sums."""
    MODE = A8


class WxFP8BitPartitionedGroupMoE(WxA16BitPartitionedGroupMoE):
    """e4m3 activations and e4m3 codebook LUTs, fp32 group sums."""
    MODE = FP8


class WxFP4BitPartitionedGroupMoE(WxA8BitPartitionedGroupMoE):
    """e2m1 activations with per-32 e8m0 scales for the bits in ``FP4_BITS``; other bits run as INT8
    (quantization/wxfp4/bit_partitioned_moe.py:50)."""
    MODE = FP4
    FP4_BITS = {1, 4}

    def _pool_mode(self, bit: int, shared: bool = False) -> int:
        return FP4 if (bit in self.FP4_BITS and not shared) else A8


MODULE_BY_MODE = {
    "wxa16": WxA16BitPartitionedGroupMoE, "wxa8": WxA8BitPartitionedGroupMoE,
    "wxfp8": WxFP8BitPartitionedGroupMoE, "wxfp4": WxFP4BitPartitionedGroupMoE,
}
