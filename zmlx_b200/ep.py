"""Expert-parallel MoE layer across the GPUs of one node (one process per GPU).

Two forms.  ``PeerMoELayer`` (decode, T * ranks <= 8 tokens): ONE ``zmoe_layer_decode`` launch per rank and no
collective -- token rows and projected rows cross NVLink as plain peer stores of tagged words into the home
rank's inbox, inside the kernel.  ``EPMoELayer`` (any token count): NCCL collectives around the separate kernels,
described next.

The reference has no distributed code at all (no collectives anywhere in its tree); this is the sharding
its operator surface allows: experts are independent, so rank r owns experts [r*E/R, (r+1)*E/R) and the router
weight and shared experts are replicated.  Every rank brings its own T decode tokens (data-parallel attention
side); one layer pass is

    all-gather token rows  ->  route all R*T tokens (replicated, identical on every rank)
    -> gate/up + SwiGLU and down projection for the (token, slot) pairs whose expert is local
    -> reduce-scatter of the per-slot rows  ->  ordered combine of the rank's own T tokens.

The per-slot rows of non-local pairs are zero, so the reduce-scatter adds exactly one non-zero bf16 value per
element and zeros: the sum is exact in any order and the combine sees the same rows, in the same slot order, as
the single-GPU layer.  The exchange and the combine thus add no rounding of their own; what can differ from a
1-GPU run is the fp32 summation grouping inside the matmul kernel, which depends on how many rows an expert
receives in one launch (a last-bit effect on a few bf16 outputs).
"""

from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from . import _lib, ops
from .layer import MoELayer
from .synthetic import MoEConfig


def expert_range(n_experts: int, world: int, rank: int) -> tuple[int, int]:
    """[lo, hi) of the experts rank ``rank`` owns; ``world`` must divide the expert count."""
    if n_experts % world != 0:
        raise ValueError(f"{n_experts} experts do not split evenly over {world} ranks")
    per = n_experts // world
    return rank * per, (rank + 1) * per


def shard_params(params: dict, lo: int, hi: int) -> dict:
    """The expert banks restricted to experts [lo, hi); router weight, bias and shared experts stay whole."""
    out = dict(params)
    for k in ("gate", "up", "down"):
        for suffix in ("w", "s", "b"):
            t = params.get(f"{k}_{suffix}")
            if t is None:
                out[f"{k}_{suffix}"] = None
            elif t.dtype == torch.uint32:
                out[f"{k}_{suffix}"] = t.view(torch.int32)[lo:hi].contiguous().view(torch.uint32)
            else:
                out[f"{k}_{suffix}"] = t[lo:hi].contiguous()
    return out


def localize_indices(indices: torch.Tensor, lo: int, hi: int) -> torch.Tensor:
    """Expert ids relative to the local shard; ids outside [lo, hi) become -1 (the plan builder drops them)."""
    idx = indices.to(torch.int32)
    local = idx - lo
    return torch.where((idx >= lo) & (idx < hi), local, torch.full_like(local, -1))


def exchange_slot_rows(y_all: torch.Tensor, world: int, group=None) -> torch.Tensor:
    """Reduce-scatter of the (R*T*K, d) per-slot rows: rank r receives rows [r*T*K, (r+1)*T*K) summed over
    ranks.  Exactly one rank holds a non-zero value per element, so the sum is exact."""
    if world == 1:
        return y_all
    rows = y_all.shape[0] // world
    out = torch.empty((rows, y_all.shape[1]), dtype=y_all.dtype, device=y_all.device)
    if y_all.is_cuda:
        dist.reduce_scatter_tensor(out, y_all, op=dist.ReduceOp.SUM, group=group)
    else:  # gloo has no reduce_scatter: all-reduce and slice (host-logic tests only)
        tmp = y_all.to(torch.float32)
        dist.all_reduce(tmp, op=dist.ReduceOp.SUM, group=group)
        r = dist.get_rank(group)
        out.copy_(tmp[r * rows:(r + 1) * rows].to(y_all.dtype))
    return out


def gather_tokens(x: torch.Tensor, world: int, group=None) -> torch.Tensor:
    """All-gather of the ranks' (T, d) token rows into (R*T, d), rank-major."""
    if world == 1:
        return x
    out = torch.empty((world * x.shape[0], x.shape[1]), dtype=x.dtype, device=x.device)
    if x.is_cuda:
        dist.all_gather_into_tensor(out, x.contiguous(), group=group)
    else:
        parts = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(parts, x.contiguous(), group=group)
        out.copy_(torch.cat(parts))
    return out


class EPMoELayer:
    """One expert-parallel MoE layer; ``params`` are the FULL layer's tensors on this rank's GPU or already the
    shard (``sharded=True``)."""

    def __init__(self, cfg: MoEConfig, params: dict, *, rank: int, world: int, max_tokens: int = 16, group=None,
                 sharded: bool = False, segment_graphs: bool = False):
        self.cfg, self.rank, self.world, self.group = cfg, rank, world, group
        self.lo, self.hi = expert_range(cfg.n_experts, world, rank)
        local = params if sharded else shard_params(params, self.lo, self.hi)
        self.n_local = self.hi - self.lo
        # the single-GPU layer object provides buffers and the replicated router on all R*T tokens
        self.inner = MoELayer(cfg, local, max_tokens=max_tokens * world, fused=False)
        dev = self.inner.device
        TK = max_tokens * world * cfg.top_k
        self.local_idx = torch.empty((TK,), dtype=torch.int32, device=dev)
        self.local_plan = torch.empty(ops.plan_bytes(TK, self.n_local) // 4, dtype=torch.int32, device=dev)
        self.out = torch.empty((max_tokens, cfg.d_model), dtype=torch.bfloat16, device=dev)
        self.x_all = torch.empty((max_tokens * world, cfg.d_model), dtype=torch.bfloat16, device=dev)
        self.y_mine = torch.empty((max_tokens * cfg.top_k, cfg.d_model), dtype=torch.bfloat16, device=dev)
        self.max_tokens = max_tokens
        # segment_graphs: the kernels between the two collectives (router, local plan, gate/up, down: six launches
        # on fixed buffers) are captured in one CUDA graph per token count and replayed; the collectives stay eager
        self.segment_graphs = bool(segment_graphs)
        self._graphs: dict[int, torch.cuda.CUDAGraph] = {}
        self._seen: set[int] = set()

    def _segment(self, TA: int) -> None:
        """Router for all gathered tokens, the plan of the local experts, gate/up + SwiGLU and down projection into
        zeroed per-slot rows: everything between the all-gather and the reduce-scatter."""
        cfg, inner = self.cfg, self.inner
        K = cfg.top_k
        lib = _lib.load()
        p = ops._ptr
        x_all = self.x_all[:TA]
        inner.route(x_all)  # replicated: weights/indices of all R*T tokens (the full-E plan is unused)
        li = self.local_idx[:TA * K]
        torch.sub(inner.indices[:TA].reshape(-1), self.lo, out=li)  # ids outside [0, n_local) are dropped
        st = ops._stream()
        _lib.check(lib.zmoe_build_plan(None, K, p(li), TA * K, 1, self.n_local, p(self.local_plan),
                                       self.local_plan.numel() * 4, st))
        qm = ops.qmode_code(cfg.mode)
        W = inner.p
        y = inner.y[:TA * K]
        y.zero_()
        _lib.check(lib.zmoe_gather_qmm_swiglu(p(x_all), TA, x_all.stride(0), p(W["gate_w"]), p(W["gate_s"]),
                                              p(W["gate_b"]), p(W["up_w"]), p(W["up_s"]), p(W["up_b"]),
                                              self.n_local, cfg.d_ff, cfg.d_model, inner.gs, qm,
                                              p(self.local_plan), TA * K, TA, p(inner.h), inner.swiglu, st))
        _lib.check(lib.zmoe_gather_qmm(p(inner.h), TA * K, cfg.d_ff, p(W["down_w"]), p(W["down_s"]),
                                       p(W["down_b"]), self.n_local, cfg.d_model, cfg.d_ff, inner.gs, qm,
                                       p(self.local_plan), TA * K, TA, 1, p(y), st))

    def _run_segment(self, TA: int) -> None:
        if not self.segment_graphs:
            self._segment(TA)
            return
        g = self._graphs.get(TA)
        if g is None:
            if TA not in self._seen:  # first pass at this size runs eagerly (loads kernels, sizes buffers)
                self._seen.add(TA)
                self._segment(TA)
                return
            cur = torch.cuda.current_stream(self.inner.device)
            side = torch.cuda.Stream(device=self.inner.device)
            side.wait_stream(cur)
            g = torch.cuda.CUDAGraph()
            # thread-local: the process group's watchdog thread may poll CUDA events while this thread captures
            with torch.cuda.graph(g, stream=side, capture_error_mode="thread_local"):
                self._segment(TA)
            cur.wait_stream(side)
            self._graphs[TA] = g
        g.replay()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        cfg, inner, R = self.cfg, self.inner, self.world
        T = x.shape[0]
        if T > self.max_tokens:
            raise ValueError(f"{T} tokens exceed max_tokens={self.max_tokens}")
        K = cfg.top_k
        lib = _lib.load()
        p = ops._ptr
        with torch.cuda.device(inner.device):
            TA = R * T
            if R > 1 and x.is_cuda:
                dist.all_gather_into_tensor(self.x_all[:TA], x.contiguous(), group=self.group)
            else:
                self.x_all[:TA].copy_(gather_tokens(x, R, self.group))
            self._run_segment(TA)
            y = inner.y[:TA * K]
            if R > 1 and y.is_cuda:
                y_mine = self.y_mine[:T * K]
                dist.reduce_scatter_tensor(y_mine, y, op=dist.ReduceOp.SUM, group=self.group)
            else:
                y_mine = exchange_slot_rows(y, R, self.group)  # (T*K, d): complete rows of this rank's tokens
            w_mine = inner.weights[self.rank * T:(self.rank + 1) * T] if R > 1 else inner.weights[:T]
            residual = None
            if cfg.n_shared:
                inner.shared(x)
                residual = inner.sh_y
            _lib.check(lib.zmoe_moe_combine(p(y_mine), _lib.BF16, p(w_mine.contiguous()), _lib.F32, T, K, cfg.d_model,
                                            inner.combine_mode, p(self.out), 3 if cfg.family == "generic" else 1,
                                            p(residual), ops._stream()))
        return self.out[:T]

    __call__ = forward


# ------------------------------------------------------------------ one launch per rank, peer stores
def inbox_layout(T: int, world: int, d_model: int, top_k: int) -> dict:
    """Word offsets inside one rank's inbox (what ``zmoe_layer_decode_inbox_bytes`` sizes): two launch parities of
    token words (T * world rows of d_model) followed by two parities of projected-row words (T * top_k routed rows
    and T shared-expert rows of d_model).  Row ``rank * T + t`` of the token part belongs to rank ``rank``."""
    xwords = T * world * d_model
    ywords = (T * top_k + T) * d_model
    return {"x": [0, xwords], "y": [2 * xwords, 2 * xwords + ywords], "words": 2 * (xwords + ywords),
            "bytes": 8 * (xwords + ywords)}


def home_of_row(row: int, T: int, top_k: int) -> tuple[int, int]:
    """(home rank, row inside the home rank's projected-row part) of routed row ``row`` = token * top_k + slot,
    tokens numbered rank-major (rank r owns tokens r*T .. r*T+T-1)."""
    token, slot = divmod(row, top_k)
    home, local = divmod(token, T)
    return home, local * top_k + slot


def launch_tag(launch_count: int) -> int:
    """Upper half of every hand-over word of launch number ``launch_count`` (counted from 0): never zero, so a
    zeroed inbox holds no valid word, and different from the tag two launches earlier, whose words lie in the same
    parity half of the inbox."""
    return ((launch_count % 65535) + 1) << 16


def pack_words(rows: torch.Tensor, launch_count: int) -> torch.Tensor:
    """bfloat16 rows -> the 32-bit hand-over words the kernel stores into an inbox: {tag : 16 | bfloat16 bits : 16}.
    A word is complete or absent (one 32-bit store), which is what lets the reader poll it without a lock."""
    bits = rows.contiguous().view(torch.int16).to(torch.int64) & 0xFFFF
    return (bits | launch_tag(launch_count)).to(torch.int64)


def unpack_words(words: torch.Tensor, launch_count: int) -> tuple[bool, torch.Tensor]:
    """(all words carry this launch's tag, their bfloat16 payload).  The reader repeats this until it holds, a
    bounded number of times: the kernel gives up after about a second and sets ``ZMOE_ERR_TIMEOUT``."""
    w = words.to(torch.int64)
    ok = bool(((w & 0xFFFF0000) == launch_tag(launch_count)).all())
    return ok, (w & 0xFFFF).to(torch.int16).view(torch.bfloat16) if ok else None


def open_inboxes(nbytes: int, rank: int, world: int, group=None) -> tuple[int, list[int], list[int]]:
    """Allocates this rank's inbox (zeroed, peer-mappable), exchanges handles with the group and maps the peers'.
    Returns (own pointer, pointers of every rank's inbox as seen from here, the mapped peer pointers to unmap)."""
    lib = _lib.load()
    own = ctypes.c_void_p()
    _lib.check(lib.zmoe_ep_alloc(nbytes, ctypes.byref(own)))
    handle = ctypes.create_string_buffer(64)
    _lib.check(lib.zmoe_ep_export(own, handle))
    handles: list = [None] * world
    dist.all_gather_object(handles, bytes(handle.raw), group=group)
    ptrs, mapped = [], []
    for r in range(world):
        if r == rank:
            ptrs.append(own.value)
            continue
        peer = ctypes.c_void_p()
        _lib.check(lib.zmoe_ep_import(ctypes.create_string_buffer(handles[r], 64), ctypes.byref(peer)))
        ptrs.append(peer.value)
        mapped.append(peer.value)
    dist.barrier(group=group)  # every inbox exists, is zero and is mapped everywhere before the first launch
    return own.value, ptrs, mapped


def peer_block_supported(cfg: MoEConfig, tokens: int, world: int) -> bool:
    """Whether the one-launch block takes ``tokens`` rows from each of ``world`` ranks for this shape (its shared
    memory holds the rows of all ranks).  Reads shapes only: no allocation, no exchange."""
    if tokens * world > MoELayer.FUSED_MAX_TOKENS or cfg.n_experts % world != 0:
        return False
    d = _lib.LayerDesc()
    d.E, d.d_model, d.d_ff, d.top_k = cfg.n_experts, cfg.d_model, cfg.d_ff, cfg.top_k
    d.group_size = 32 if cfg.mode == "mxfp4" else cfg.group_size
    d.qmode = _lib.Q_MXFP4 if cfg.mode == "mxfp4" else _lib.Q_AFFINE4
    d.n_shared = int(cfg.n_shared)
    d.ep_world, d.ep_rank = int(world), 0
    return int(_lib.load().zmoe_layer_decode_workspace_bytes(ctypes.byref(d), int(tokens))) > 0


class PeerMoELayer:
    """Expert-parallel block in one launch per rank.  ``params`` hold this rank's shard of the expert banks
    (``shard_params``), the replicated router and shared expert.  Every rank must call ``forward`` the same number
    of times with ``tokens`` rows: the launches of a step find each other through tags derived from the launch
    count."""

    def __init__(self, cfg: MoEConfig, params: dict, *, rank: int, world: int, tokens: int, group=None,
                 launch: str = "cooperative"):
        if tokens * world > MoELayer.FUSED_MAX_TOKENS:
            raise ValueError(f"{tokens} tokens on {world} ranks exceed the {MoELayer.FUSED_MAX_TOKENS} rows of one launch")
        self.cfg, self.rank, self.world, self.tokens, self.group = cfg, rank, world, tokens, group
        self.lo, self.hi = expert_range(cfg.n_experts, world, rank)
        lay = inbox_layout(tokens, world, cfg.d_model, cfg.top_k)
        self._own, ptrs, self._mapped = open_inboxes(lay["bytes"], rank, world, group)
        self.inner = MoELayer(cfg, params, max_tokens=tokens, launch=launch,
                              ep={"rank": rank, "world": world, "inbox": ptrs})
        if self.inner.fused_workspace_bytes(tokens) == 0:
            self.close()
            raise _lib.ZmoeError(_lib.ERR_UNSUPPORTED, "the one-launch block does not cover this shape")

    @property
    def indices(self) -> torch.Tensor:
        return self.inner.indices

    @property
    def weights(self) -> torch.Tensor:
        return self.inner.weights

    @property
    def out(self) -> torch.Tensor:
        return self.inner.out

    def forward(self, x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        if x.shape[0] != self.tokens:
            raise ValueError(f"this layer was set up for {self.tokens} tokens per rank, got {x.shape[0]}")
        with torch.cuda.device(self.inner.device):
            return self.inner.forward_fused(x if x.stride(1) == 1 else x.contiguous(), out)

    __call__ = forward

    def check_status(self) -> None:
        self.inner.check_status()

    def close(self) -> None:
        """Collective over the layer's group: no rank frees its inbox while a peer still has it mapped."""
        lib = _lib.load()
        for ptr in self._mapped:
            lib.zmoe_ep_unmap(ctypes.c_void_p(ptr))
        self._mapped = []
        if dist.is_initialized():
            dist.barrier(group=self.group)
        if self._own:
            lib.zmoe_ep_free(ctypes.c_void_p(self._own))
            self._own = 0
