"""One MoE block forward on the GPU: router -> gate/up + SwiGLU -> down -> combine.

This is the order of the reference's patched block
(src/zmlx/patch/patterns/moe_mlp.py:883-1063) with every step running in a
libzmoe kernel.  ``MoELayer`` owns the packed tensors of one layer and
preallocated work buffers for a fixed maximum token count, so that a forward
pass allocates nothing and can be captured in a CUDA graph.
"""

from __future__ import annotations

import ctypes

import torch

from . import _lib, ops
from .synthetic import MoEConfig

_FAMILY_COMBINE = {"generic": "t", "qwen3": "no_fma", "glm": "fp32_no_fma", "deepseek": "t"}


class MoELayer:
    """Packed weights of one MoE layer plus the buffers of its forward pass."""

    def __init__(self, cfg: MoEConfig, params: dict, *, max_tokens: int = 64, combine: str | None = None,
                 swiglu: str | None = None, fused: bool = True, launch: str = "cooperative",
                 debug_withhold_logit: bool = False, debug_force_inbox: bool = False, ep: dict | None = None):
        self.cfg = cfg
        self.p = params
        dev = params["gate_w"].device
        if dev.type != "cuda":
            raise RuntimeError("MoELayer needs its tensors on a CUDA device (there is no CPU path)")
        self.device = dev
        self.combine_name = combine or _FAMILY_COMBINE[cfg.family]
        self.combine_mode = _lib.COMBINE_MODES[self.combine_name]
        sw = swiglu or ("cpu" if cfg.mode == "affine" else "per_op")
        self.swiglu = _lib.SWIGLU_CPU if sw == "cpu" else _lib.SWIGLU_PER_OP
        self.gs = 32 if cfg.mode == "mxfp4" else cfg.group_size
        self._alloc(max_tokens)
        self.fused = bool(fused)
        if launch not in ("cooperative", "pdl"):
            raise ValueError("launch must be 'cooperative' or 'pdl'")
        # 'pdl': the one-launch block as a regular launch that is set up while the previous kernel still runs
        # (saves the launch gap in a chain of blocks); only when this stream has the GPU to itself
        self.launch = launch
        # test hook of the one-launch block: one router logit is never published, so its bounded waits run out
        self._debug_flags = _lib.DEBUG_WITHHOLD_LOGIT if debug_withhold_logit else 0
        # expert parallel (zmlx_b200.ep.PeerMoELayer): {"rank", "world", "inbox": [device pointers of every rank's
        # inbox as seen from here]}; the banks in `params` are then this rank's shard
        self.ep = ep
        self._inbox: torch.Tensor | None = None
        if debug_force_inbox:  # the expert-parallel data path on one GPU (tests)
            self._debug_flags |= _lib.DEBUG_FORCE_INBOX
        self._stamps: torch.Tensor | None = None
        self._desc = self._describe()
        self._fused_ws: dict[int, torch.Tensor] = {}
        self._fused_ok: dict[int, bool] = {}  # token count -> whether the one-launch path covers this block
        self._side: torch.cuda.Stream | None = None  # second stream for the shared expert (separate-kernel path)
        self._shared_plans: dict[int, torch.Tensor] = {}  # token count -> the shared expert's (constant) plan

    # -- one-launch decode path ---------------------------------------------
    FUSED_MAX_TOKENS = 8

    def _describe(self) -> _lib.LayerDesc:
        """The block as a ``zmoe_layer_desc`` (pointers into this layer's tensors, which it keeps alive)."""
        cfg, W = self.cfg, self.p
        family, bias, renorm = self._route_args()
        d = _lib.LayerDesc()
        d.E, d.d_model, d.d_ff, d.top_k = cfg.n_experts, cfg.d_model, cfg.d_ff, cfg.top_k
        d.group_size, d.qmode = self.gs, ops.qmode_code(cfg.mode)
        d.router_family, d.renorm, d.n_group, d.topk_group = family, renorm, cfg.n_group, cfg.topk_group
        d.routed_scale = float(cfg.routed_scaling_factor) if family == 2 else 1.0
        d.n_shared = int(cfg.n_shared)
        d.swiglu_mode, d.shared_swiglu_mode = self.swiglu, _lib.SWIGLU_PER_OP
        d.combine_mode = self.combine_mode
        d.out_flags = 3 if cfg.family == "generic" else 1
        d.launch_mode = 1 if self.launch == "pdl" else 0
        d.debug_flags = self._debug_flags
        d.debug_stamps = self._stamps.data_ptr() if self._stamps is not None else None
        if self.ep is not None:
            d.ep_world, d.ep_rank = int(self.ep["world"]), int(self.ep["rank"])
            for r, ptr in enumerate(self.ep["inbox"]):
                d.ep_inbox[r] = ptr
        elif self._inbox is not None:
            d.ep_inbox[0] = self._inbox.data_ptr()
        d.router_w = W["router_w"].data_ptr()
        d.router_bias = bias.data_ptr() if bias is not None else None

        def bank(dst, src):
            for proj in ("gate", "up", "down"):
                setattr(dst, f"{proj}_w", src[f"{proj}_w"].data_ptr())
                setattr(dst, f"{proj}_scales", src[f"{proj}_s"].data_ptr())
                b = src.get(f"{proj}_b")
                setattr(dst, f"{proj}_biases", b.data_ptr() if b is not None else None)

        bank(d.routed, W)
        if cfg.n_shared:
            bank(d.shared, W["shared"])
        return d

    def fused_workspace_bytes(self, T: int) -> int:
        """Bytes of workspace the one-launch path needs for T tokens; 0 when the block's shape is outside it."""
        if T < 1 or T > self.FUSED_MAX_TOKENS:
            return 0
        return int(_lib.load().zmoe_layer_decode_workspace_bytes(ctypes.byref(self._desc), T))

    def _chunks(self, T: int) -> list[tuple[int, int]]:
        """(first row, rows) of the one-launch passes that cover T rows."""
        M = self.FUSED_MAX_TOKENS
        return [(r, min(M, T - r)) for r in range(0, T, M)]

    def _chunked_ok(self, T: int) -> bool:
        """More rows than one launch takes, but still fewer than two per expert on average: the block runs as
        consecutive one-launch passes over eight rows each.  Every pass streams only its own rows' experts, and
        measured against the separate kernels it wins up to about that density (c2 T=16: 79 vs 121 us, c5 T=64:
        2.3 vs 3.5 ms per layer); beyond it the experts are shared by enough rows for the grouped matmuls."""
        cfg = self.cfg
        # blocks so wide that the register-fed matmul cannot stage eight token rows (its 96 KB budget) keep the
        # passes up to four rows per expert: measured c5 T=128, 4.6 ms in 16 passes against 5.7 ms
        dense = 4 if cfg.d_model * 2 * 8 > 96 * 1024 else 2
        if self.ep is not None or T <= self.FUSED_MAX_TOKENS or T * cfg.top_k > dense * cfg.n_experts:
            return False
        return all(self.fused_workspace_bytes(n) > 0 for n in {n for _, n in self._chunks(T)})

    def forward_fused(self, x: torch.Tensor, out: torch.Tensor | None = None, *, row0: int = 0,
                      key=None) -> torch.Tensor:
        """The whole block in one launch (``zmoe_layer_decode``); raises if the shape is outside it.  ``row0``:
        first row of ``out``, ``weights`` and ``indices`` this pass writes; ``key``: which workspace it uses (one per
        pass of a chunked call, so that every pass keeps its logits and status)."""
        T = x.shape[0]
        dst = self.out if out is None else out
        key = T if key is None else key
        ws = self._fused_ws.get(key)
        if ws is None:
            if torch.cuda.is_current_stream_capturing():
                # a workspace zeroed inside the graph would be zeroed again at every replay, and with it the launch
                # count that tells this launch's hand-over words from the previous one's
                raise RuntimeError(f"run the block once with {T} token(s) before capturing it in a CUDA graph")
            need = self.fused_workspace_bytes(T)
            if need == 0:
                raise _lib.ZmoeError(_lib.ERR_UNSUPPORTED, f"no one-launch path for this block at T={T}")
            ws = torch.zeros(need, dtype=torch.uint8, device=self.device)  # the sync words start at zero
            self._fused_ws[key] = ws
            if (self._debug_flags & _lib.DEBUG_FORCE_INBOX) and self._inbox is None:
                nb = int(_lib.load().zmoe_layer_decode_inbox_bytes(ctypes.byref(self._desc), self.FUSED_MAX_TOKENS))
                self._inbox = torch.zeros(nb, dtype=torch.uint8, device=self.device)
                self._desc = self._describe()
        p = ops._ptr
        _lib.check(_lib.load().zmoe_layer_decode(ctypes.byref(self._desc), p(x), x.stride(0), T, p(ws), ws.numel(),
                                                 p(self.weights[row0:]), p(self.indices[row0:]), p(dst[row0:]),
                                                 ops._stream()))
        return dst[row0:row0 + T]

    def launch_count(self, T: int) -> int:
        """How many one-launch passes the T-token workspace has seen (the kernel's own launch counter)."""
        ws = self._fused_ws.get(T)
        return 0 if ws is None else int(ws[:32].view(torch.int32)[4].item())

    def router_logits(self, T: int) -> torch.Tensor:
        """The (T, E) bf16 router logits of the last forward pass over T tokens (whichever path ran it)."""
        if self.fused and self._fused_ok.get(T) == "chunks":
            parts = []
            for ci, (_, n) in enumerate(self._chunks(T)):
                words = self._fused_ws[(T, ci)][256:256 + n * self.cfg.n_experts * 32].view(torch.int32)[::8]
                parts.append((words & 0xFFFF).to(torch.int16).view(torch.bfloat16).view(n, self.cfg.n_experts))
            return torch.cat(parts)
        ws = self._fused_ws.get(T) if self.fused else None
        if ws is None:
            return self.logits[:T]
        if self.ep is not None:
            T = T * int(self.ep["world"])  # the kernel routes every rank's tokens
        E = self.cfg.n_experts
        # the kernel keeps each logit in the low half of a 32-bit hand-over word
        words = ws[256:256 + T * E * 32].view(torch.int32)[::8]  # one 32-byte sector per logit
        return (words & 0xFFFF).to(torch.int16).view(torch.bfloat16).view(T, E)

    def fused_status(self, T: int) -> int:
        """The status word of the T-token workspace: non-zero after a bounded wait of the one-launch block ran out."""
        if self._fused_ok.get(T) == "chunks":
            return max(int(self._fused_ws[(T, ci)][:16].view(torch.int32)[3].item())
                       for ci in range(len(self._chunks(T))))
        ws = self._fused_ws.get(T)
        return 0 if ws is None else int(ws[:16].view(torch.int32)[3].item())

    def check_status(self) -> None:
        """Raise ``ZmoeError(ERR_TIMEOUT)`` if a bounded wait ran out in any one-launch pass since the last check
        (the output of that pass is void).  Synchronises the current stream: call it where the caller waits for
        results anyway (end of a decode step, end of a timed region)."""
        lib = _lib.load()
        with torch.cuda.device(self.device):
            for ws in self._fused_ws.values():
                _lib.check(lib.zmoe_layer_decode_status(ops._ptr(ws), 1, ops._stream()))

    def enable_stamps(self) -> torch.Tensor:
        """Debug: make CTA 0 of the one-launch block record its cycle counter at the phase boundaries; returns the
        16 int64 it writes (see ``zmoe_layer_desc.debug_stamps``)."""
        self._stamps = torch.zeros(16, dtype=torch.int64, device=self.device)
        self._desc = self._describe()
        return self._stamps

    def _alloc(self, T: int) -> None:
        cfg, dev = self.cfg, self.device
        K = cfg.top_k
        self.max_tokens = T
        bf, f32, i32 = torch.bfloat16, torch.float32, torch.int32
        self.logits = torch.empty((T, cfg.n_experts), dtype=bf, device=dev)
        self.weights = torch.empty((T, K), dtype=f32, device=dev)
        self.indices = torch.empty((T, K), dtype=i32, device=dev)
        self.plan = torch.empty(ops.plan_bytes(T * K, cfg.n_experts) // 4, dtype=i32, device=dev)
        self.counter = torch.zeros(1, dtype=i32, device=dev)
        self.h = torch.empty((T * K, cfg.d_ff), dtype=bf, device=dev)
        self.y = torch.empty((T * K, cfg.d_model), dtype=bf, device=dev)
        self.out = torch.empty((T, cfg.d_model), dtype=bf, device=dev)
        if cfg.n_shared:
            self.zero_idx = torch.zeros((T,), dtype=i32, device=dev)
            self.shared_plan = torch.empty(ops.plan_bytes(T, 1) // 4, dtype=i32, device=dev)
            self.sh_h = torch.empty((T, cfg.d_ff * cfg.n_shared), dtype=bf, device=dev)
            self.sh_y = torch.empty((T, cfg.d_model), dtype=bf, device=dev)

    # -- steps -------------------------------------------------------------
    def _route_args(self):
        cfg = self.cfg
        bias = self.p.get("expert_bias")
        if cfg.family == "generic":
            if bias is None and cfg.norm_topk_prob:
                return 0, None, 0
            return 1, bias, (1 if cfg.norm_topk_prob else 0)
        if cfg.family == "qwen3":
            return 1, None, (2 if cfg.norm_topk_prob else 0)
        return 2, bias, 0

    def route(self, x: torch.Tensor):
        """Router linear (bf16 logits), the family's top-k and the expert plan, in one launch."""
        cfg = self.cfg
        T = x.shape[0]
        p = ops._ptr
        family, bias, renorm = self._route_args()
        lib = _lib.load()
        if T > 8:
            # many rows: separate launches, one warp per token row across many CTAs
            st = ops._stream()
            _lib.check(lib.zmoe_router_logits(p(x), p(self.p["router_w"]), T, cfg.n_experts, cfg.d_model,
                                              p(self.logits), _lib.BF16, st))
            if family == 2:
                rc = lib.zmoe_router_sigmoid_bias_topk(p(self.logits), _lib.BF16, T, cfg.n_experts, cfg.top_k, p(bias),
                                                       cfg.n_group, cfg.topk_group,
                                                       ctypes.c_float(cfg.routed_scaling_factor), p(self.weights),
                                                       p(self.indices), st)
            else:
                rc = lib.zmoe_router_softmax_topk(p(self.logits), _lib.BF16, T, cfg.n_experts, cfg.top_k,
                                                  _lib.ROUTER_TOPK_THEN_SOFTMAX if family == 0
                                                  else _lib.ROUTER_SOFTMAX_THEN_TOPK, p(bias), renorm,
                                                  p(self.weights), p(self.indices), st)
            _lib.check(rc)
            _lib.check(lib.zmoe_build_plan(None, cfg.top_k, p(self.indices), T * cfg.top_k, 1, cfg.n_experts,
                                           p(self.plan), self.plan.numel() * 4, st))
            return
        _lib.check(lib.zmoe_route(
            p(x), p(self.p["router_w"]), T, cfg.n_experts, cfg.d_model, cfg.top_k, family, p(bias), renorm,
            cfg.n_group, cfg.topk_group, ctypes.c_float(cfg.routed_scaling_factor if family == 2 else 1.0),
            p(self.logits), p(self.weights), p(self.indices), p(self.plan), self.plan.numel() * 4, p(self.counter),
            ops._stream()))

    def experts(self, x: torch.Tensor):
        """Fused gate/up + SwiGLU and the down projection for all (token, slot) pairs (plan from route())."""
        cfg = self.cfg
        T = x.shape[0]
        K = cfg.top_k
        lib = _lib.load()
        st = ops._stream()
        p = ops._ptr
        qm = ops.qmode_code(cfg.mode)
        W = self.p
        _lib.check(lib.zmoe_gather_qmm_swiglu(p(x), T, x.stride(0), p(W["gate_w"]), p(W["gate_s"]), p(W["gate_b"]),
                                              p(W["up_w"]), p(W["up_s"]), p(W["up_b"]), cfg.n_experts, cfg.d_ff,
                                              cfg.d_model, self.gs, qm, p(self.plan), T * K, T, p(self.h),
                                              self.swiglu, st))
        _lib.check(lib.zmoe_gather_qmm(p(self.h), T * K, cfg.d_ff, p(W["down_w"]), p(W["down_s"]), p(W["down_b"]),
                                       cfg.n_experts, cfg.d_model, cfg.d_ff, self.gs, qm, p(self.plan), T * K, T, 3,
                                       p(self.y), st))

    def shared(self, x: torch.Tensor):
        """The always-on shared expert: the same kernels with a one-expert bank."""
        cfg = self.cfg
        T = x.shape[0]
        lib = _lib.load()
        st = ops._stream()
        p = ops._ptr
        qm = ops.qmode_code(cfg.mode)
        S = self.p["shared"]
        f = cfg.d_ff * cfg.n_shared
        # the shared expert's plan depends on the token count only (row t -> expert 0): built once per count and
        # kept, unless this call is being captured in a CUDA graph (a captured launch does not run now)
        plan = self._shared_plans.get(T)
        if plan is None:
            capturing = torch.cuda.is_current_stream_capturing()
            plan = self.shared_plan if capturing else torch.empty(ops.plan_bytes(T, 1) // 4, dtype=torch.int32,
                                                                  device=self.device)
            _lib.check(lib.zmoe_build_plan(None, 1, p(self.zero_idx), T, 1, 1, p(plan), plan.numel() * 4, st))
            if not capturing:
                self._shared_plans[T] = plan
        _lib.check(lib.zmoe_gather_qmm_swiglu(p(x), T, x.stride(0), p(S["gate_w"]), p(S["gate_s"]), p(S["gate_b"]),
                                              p(S["up_w"]), p(S["up_s"]), p(S["up_b"]), 1, f, cfg.d_model, self.gs,
                                              qm, p(plan), T, T, p(self.sh_h), _lib.SWIGLU_PER_OP, st))
        _lib.check(lib.zmoe_gather_qmm(p(self.sh_h), T, f, p(S["down_w"]), p(S["down_s"]), p(S["down_b"]), 1,
                                       cfg.d_model, f, self.gs, qm, p(plan), T, T, 1, p(self.sh_y), st))

    def forward(self, x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """x (T, d_model) bfloat16 on this layer's device -> (T, d_model) bfloat16: ``out`` when given (contiguous,
        at least T rows), else a view of a buffer the layer owns and overwrites on its next call."""
        cfg = self.cfg
        if x.dtype != torch.bfloat16 or x.ndim != 2 or x.shape[1] != cfg.d_model:
            raise ValueError(f"expected (T, {cfg.d_model}) bfloat16 activations, got {tuple(x.shape)} {x.dtype}")
        if x.device != self.device:
            raise RuntimeError(f"activations on {x.device}, layer on {self.device}")
        T = x.shape[0]
        if T > self.max_tokens:
            self._alloc(T)
        if T == 0:
            return self.out[:0]
        if x.stride(1) != 1 or x.stride(0) % 8 != 0 or x.data_ptr() % 16 != 0:
            x = x.contiguous()
        with torch.cuda.device(self.device):
            if self.fused:
                ok = self._fused_ok.get(T)
                if ok is None:
                    ok = self.fused_workspace_bytes(T) > 0 or ("chunks" if self._chunked_ok(T) else False)
                    self._fused_ok[T] = ok
                if ok == "chunks":
                    dst = self.out if out is None else out
                    for ci, (r, n) in enumerate(self._chunks(T)):
                        self.forward_fused(x[r:r + n], dst, row0=r, key=(T, ci))
                    return dst[:T]
                if ok:
                    return self.forward_fused(x, out)
            residual = None
            if cfg.n_shared:
                # the shared expert depends on x only: it runs on a side stream beside the router and the routed
                # experts and joins before the combine (fork and join are events, so a CUDA graph captures them)
                cur = torch.cuda.current_stream(self.device)
                if self._side is None:
                    self._side = torch.cuda.Stream(device=self.device)
                self._side.wait_stream(cur)
                with torch.cuda.stream(self._side):
                    self.shared(x)
                residual = self.sh_y
            self.route(x)
            self.experts(x)
            if cfg.n_shared:
                cur.wait_stream(self._side)
            dst = self.out if out is None else out
            _lib.check(_lib.load().zmoe_moe_combine(
                ops._ptr(self.y), _lib.BF16, ops._ptr(self.weights), _lib.F32, T, cfg.top_k, cfg.d_model,
                self.combine_mode, ops._ptr(dst), 3 if cfg.family == "generic" else 1, ops._ptr(residual),
                ops._stream()))
        return dst[:T]

    __call__ = forward
