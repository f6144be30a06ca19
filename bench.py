"""MoE-layer decode benchmark (one JSON line on stdout).

A *step* is one batch of T decode tokens passing through L stacked MoE layers with distinct
weights.  The default workload is the DeepSeek-V3-shaped layer (d_model 7168, 256 experts + one
shared, top-8 with group-limited sigmoid routing, d_ff 2048, 4-bit affine g64: 227 MB of active
weights per token) at T = 1 through L = 6 layers -- the largest configuration that fits one GPU and
the one where bytes, not latency, decide; ``--config c2`` is the Qwen3-30B-A3B-shaped layer (22 MB
per token, L = 24).  On one GPU every layer is ONE kernel launch (zmoe_layer_decode: router, top-k,
gate/up + SwiGLU, down, combine, shared expert) where the block's shape allows it; larger T, mxfp4
and --no-fused take the separate kernels.  Rotating over L layers means every layer pass streams
its experts from HBM: the bytes touched between two visits of the same layer exceed the 126 MB L2
many times over.  ``value`` = layer-tokens per second = T * L * n_gpus / step time (median of
``--repeats`` timed loops of ``--steps`` steps), inputs resident in HBM; ``e2e`` is the same metric
through the public Python call with the token rows starting in pinned host memory and the result
read back every step.

Multi-GPU (--gpus N under torchrun): expert parallel.  Rank r owns E/N experts of every layer and
brings its own T tokens (zmlx_b200/ep.py).  Per-GPU tokens are fixed as N grows (weak scaling); the
step time is the max over ranks.  ``--replicas`` runs N independent copies instead.

``--impl reference`` times the CPU restatement of the reference's path (the compiled oracle, all
host threads) on a bounded sample of the same workload.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "moe_layer_decode_tokens_per_s"
UNIT = "layer-tokens/s"


def _args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="zmoe", choices=["zmoe", "reference"])
    ap.add_argument("--config", default="c5")
    ap.add_argument("--tokens", type=int, default=1)
    ap.add_argument("--layers", type=int, default=0, help="stacked layers per step (default: 6 for c5, else 24)")
    ap.add_argument("--repeats", type=int, default=5, help="timed loops of --steps steps; the median is reported")
    ap.add_argument("--experts", type=int, default=0,
                    help="trim the routed bank to this many experts (profiling captures on a small footprint)")
    ap.add_argument("--via-patch", action="store_true",
                    help="drive the blocks as nn modules patched by zmlx_b200.patch.patch() instead of MoELayer")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--stamps", action="store_true",
                    help="one GPU, one-launch block: CTA 0 of the middle layer records its cycle counter at the phase "
                         "boundaries; the phase table is printed to stderr after the timed run")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--launch", default="pdl", choices=["pdl", "cooperative"],
                    help="how the one-launch block is launched: 'pdl' = regular launch set up while the previous "
                         "block still runs (this benchmark has the GPU to itself), 'cooperative' = the library default")
    ap.add_argument("--no-fused", action="store_true",
                    help="run every block as separate kernels even where the one-launch decode kernel covers it")
    ap.add_argument("--replicas", action="store_true", help="N>1: independent replicas instead of expert parallel")
    ap.add_argument("--no-ep-segments", dest="ep_segments", action="store_false",
                    help="N>1: launch the kernels between the two collectives of a layer eagerly instead of "
                         "replaying them from one CUDA graph per layer")
    ap.add_argument("--ep-degree", type=int, default=0,
                    help="N>1: ranks per expert-parallel group (the groups run side by side); 0 = choose")
    ap.add_argument("--ep-nccl", action="store_true",
                    help="N>1: NCCL collectives around the separate kernels even where the one-launch peer-store "
                         "form covers the step")
    ap.add_argument("--check", action="store_true", help="N>1: compare the expert-parallel output with a 1-GPU layer")
    return ap.parse_args()


# DRAM bytes per launch of the one-launch block measured with ncu (dram__bytes_read.sum + dram__bytes_write.sum),
# as a ratio to the algorithmic bytes of the captured launches; the summaries that hold the figures are named.
_TRAFFIC_RATIO = {
    (5, 1): (1.020, "profiles/layer_decode_kernel_c5_T1.md: 223.62 MB read + 4.38 MB written per launch over "
                    "223.44 MB algorithmic, 32-expert bank; scaled by the algorithmic bytes of this launch"),
    (2, 1): (1.008, "profiles/layer_decode_kernel_c2_T1.md: 21.54 MB read per launch over 21.37 MB algorithmic, "
                    "32-expert bank; scaled by the algorithmic bytes of this launch"),
}


def _measured_traffic(cfg, T, one_launch, alg_bytes_per_launch):
    rec = _TRAFFIC_RATIO.get((cfg.config_id, T)) if one_launch else None
    if rec is None:
        return None, None
    ratio, source = rec
    return ratio * alg_bytes_per_launch, source


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            with open(path) as f:
                return float(json.load(f)["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    def __init__(self, index: int):
        self.index = index
        self.samples: list[tuple[float, float, list[str]]] = []
        self._stop = threading.Event()
        self._thr = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        try:
            self._run_nvml()
        except Exception:
            self._run_smi()

    def _run_nvml(self):
        """NVML reads (a few microseconds each) every 5 ms: many samples even inside a 30 ms timed region."""
        import pynvml as nv

        nv.nvmlInit()
        try:
            h = nv.nvmlDeviceGetHandleByIndex(self.index)
            mx = float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
            bits = {"hw_slowdown": nv.nvmlClocksEventReasonHwSlowdown if hasattr(nv, "nvmlClocksEventReasonHwSlowdown")
                    else nv.nvmlClocksThrottleReasonHwSlowdown,
                    "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown",
                                                   getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0)),
                    "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown",
                                                   getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0)),
                    "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap",
                                            getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0))}
            get_reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                nv.nvmlDeviceGetCurrentClocksThrottleReasons
            while not self._stop.is_set():
                sm = float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                mask = int(get_reasons(h))
                self.samples.append((sm, mx, [n for n, b in bits.items() if b and (mask & b)]))
                self._stop.wait(0.005)
        finally:
            nv.nvmlShutdown()

    def _run_smi(self):
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits", "-i",
                                      str(self.index)], capture_output=True, text=True, timeout=5).stdout.strip()
                parts = [p.strip() for p in out.split(",")]
                reasons = [n for n, v in zip(names, parts[2:6]) if v.lower().startswith("active")]
                self.samples.append((float(parts[0]), float(parts[1]), reasons))
            except Exception:
                pass
            self._stop.wait(0.1)

    def __enter__(self):
        self._thr.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._thr.join(timeout=6)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        sm = sorted(s[0] for s in self.samples)
        reasons = sorted({r for s in self.samples for r in s[2]})
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": self.samples[0][1], "reasons": reasons,
                "samples": len(self.samples)}


def _cpu_baseline(cfg, tokens: int, budget_s: float = 12.0):
    """Time the compiled oracle (a port of the reference's CPU arithmetic) on a bounded sample:
    whole layer passes of the same shape (router, routed experts, combine, shared expert), repeated
    until ~budget_s of CPU work.  All host threads."""
    import numpy as np
    import torch

    from oracle import fast as F
    from oracle import semantics as S
    from zmlx_b200 import synthetic

    F.set_num_threads(os.cpu_count() or 1)  # torchrun exports OMP_NUM_THREADS=1: choose the count here
    groups = max(cfg.n_group, 1)
    keep = max(cfg.top_k * 2, 16)
    keep = ((keep + groups - 1) // groups) * groups
    small = cfg.scaled(n_experts=min(cfg.n_experts, keep))  # bank trimmed: routing still picks top_k distinct
    p = synthetic.make_layer(small, device="cpu")

    def n(t):
        if t is None:
            return None
        if isinstance(t, dict):
            return {k: n(v) for k, v in t.items()}
        if t.dtype == torch.bfloat16:
            return t.float().numpy()
        if t.dtype == torch.uint32:
            return t.view(torch.int32).numpy().view(np.uint32)
        return t.numpy()

    pn = {k: n(v) for k, v in p.items()}
    x = n(synthetic.make_tokens(small, tokens))
    rw = pn["router_w"]
    gs = 32 if small.mode == "mxfp4" else small.group_size
    sw = "cpu" if small.mode == "affine" else "per_op"
    zero_idx = np.zeros((tokens, 1), dtype=np.int32)

    def one_pass():
        logits = S.bf16(x @ rw.T)
        if small.family == "qwen3":
            idx, w = S.qwen3_gating(logits, small.top_k)
            mode = "no_fma"
        elif small.family == "generic":
            w, idx = S.topk_gating_softmax(logits, small.top_k)
            w, mode = S.bf16(w), "t"
        else:
            w, idx = S.deepseek_router_topk_sigmoid(logits, pn["expert_bias"], k=small.top_k, n_group=small.n_group,
                                                    topk_group=min(small.topk_group, small.n_group))
            w = (w * np.float32(small.routed_scaling_factor)).astype(np.float32)
            mode = "fp32_no_fma" if small.family == "glm" else "t"
        y, _ = F.experts_forward(x, idx.astype(np.int32), pn, group_size=gs, mode=small.mode, swiglu=sw)
        out = S.moe_combine(y, w, mode=mode)
        if small.n_shared:
            ys, _ = F.experts_forward(x, zero_idx, pn["shared"], group_size=gs, mode=small.mode, swiglu="per_op")
            out = S.bf16(S.bf16(out) + ys[:, 0, :])
        return out

    one_pass()
    t0 = time.perf_counter()
    reps = 0
    while True:
        one_pass()
        reps += 1
        dt = time.perf_counter() - t0
        if dt > budget_s or reps >= 2000:
            break
    nbytes = small.algorithmic_bytes(min(small.top_k * tokens, small.n_experts), tokens)
    return {"value": tokens * reps / dt, "unit": UNIT, "cores": F.num_threads(), "kind": "port",
            "achieved_gbs": nbytes * reps / dt / 1e9,
            "sample": f"{reps} passes of one {cfg.name}-shaped layer (expert bank trimmed to {small.n_experts}, "
                      f"top-{small.top_k} active" + (", one shared expert" if small.n_shared else "") +
                      f") at T={tokens}, compiled oracle with OpenMP on {F.num_threads()} threads, {dt:.1f} s; "
                      "a reported baseline, not a target: see roofline.frac for kernel quality"}


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from zmlx_b200 import synthetic

    cfg = synthetic.CONFIGS[args.config]
    if args.experts:
        cfg = cfg.scaled(n_experts=args.experts)
    t0 = time.perf_counter()
    # steps/warmup are honoured as repetitions of a bounded sample
    base = _cpu_baseline(cfg, args.tokens, budget_s=min(20.0, 0.4 * max(args.steps, 1)))
    wall = time.perf_counter() - t0
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * args.tokens / base["value"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"{cfg.name} MoE layer decode, T={args.tokens}; CPU restatement of the reference "
                               "path (MLX itself is not installable here)"},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "wall_s": wall,
    }
    print(json.dumps(line))


def main() -> None:
    args = _args()
    if args.impl == "reference":
        run_reference(args)
        return

    import torch
    import torch.distributed as dist

    from zmlx_b200 import synthetic
    from zmlx_b200.layer import MoELayer

    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the kernels have no CPU fallback")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    cfg = synthetic.CONFIGS[args.config]
    if args.experts:
        cfg = cfg.scaled(n_experts=args.experts)
    if args.layers <= 0:
        args.layers = 6 if cfg.config_id == 5 else 24
    T, L = args.tokens, args.layers
    use_ep = world > 1 and not args.replicas
    ep_peer = False  # expert parallel in one launch per rank (peer stores) instead of collectives around kernels
    if use_ep:
        from zmlx_b200 import _lib as zlib
        from zmlx_b200 import ep

        # Expert-parallel degree: groups of --ep-degree ranks share one set of experts and the groups run side by
        # side as data-parallel replicas.  The default is pairs: a launch then carries 2 T token rows and keeps
        # most of its shared memory for weight stages (measured on 8 GPUs, c5 T=1: ep2 x dp4 80.6k, ep4 x dp2
        # 65.3k, ep8 56.7k layer-tokens/s); wider groups are for models whose experts do not fit in two GPUs.
        ep_deg, ep_group = world, None
        layers = []
        if not args.ep_nccl and not args.no_fused:
            cands = [args.ep_degree] if args.ep_degree else [2, 4, 8]
            for g in [g for g in cands if g >= 2 and world % g == 0]:
                if ep.peer_block_supported(cfg, T, g):
                    # every rank takes part in creating every group
                    groups = [dist.new_group(list(range(b, b + g))) for b in range(0, world, g)] if g < world else [None]
                    ep_peer, ep_deg, ep_group = True, g, groups[rank // g]
                    break
        ep_rank = rank % ep_deg
        for i in range(L):
            full = synthetic.make_layer(cfg, layer=i, device=dev)  # same seed on every rank: one model
            lo, hi = ep.expert_range(cfg.n_experts, ep_deg, ep_rank)
            shard = ep.shard_params(full, lo, hi)
            if ep_peer:
                layers.append(ep.PeerMoELayer(cfg, shard, rank=ep_rank, world=ep_deg, tokens=T, group=ep_group,
                                              launch=args.launch))
            else:
                layers.append(ep.EPMoELayer(cfg, shard, rank=rank, world=world, max_tokens=T, sharded=True,
                                            segment_graphs=args.ep_segments))
            if args.check and i == 0:
                ref_layer = MoELayer(cfg, full, max_tokens=T)
            else:
                del full
        torch.cuda.empty_cache()
    elif args.via_patch:
        # the drop-in surface: torch modules with the attribute contract the reference patches, rewritten by patch()
        from zmlx_b200 import nn as znn
        from zmlx_b200.patch import patch

        class _Stack(torch.nn.Module):
            def __init__(self, blocks):
                super().__init__()
                self.layers = torch.nn.ModuleList(blocks)

        model = _Stack([znn.block_from_params(cfg, synthetic.make_layer(cfg, layer=100 * rank + i, device=dev))
                        for i in range(L)])
        patch(model)

        class _Patched:  # the step loop's view of a patched block
            def __init__(self, blk):
                self.blk, self.fast = blk, blk._zmlx_fast_layer
                if self.fast is None:
                    raise RuntimeError("patch() did not build the fused layer for this block")
                self.fast.launch = args.launch
                self.fast._desc = self.fast._describe()
                self.fused, self.out = True, None

            def forward(self, h):
                self.out = self.blk(h)
                return self.out

            indices = property(lambda self: self.fast.indices)

            def fused_workspace_bytes(self, t):
                return self.fast.fused_workspace_bytes(t)

            def check_status(self):
                self.fast.check_status()

        layers = [_Patched(b) for b in model.layers]
    else:
        layers = [MoELayer(cfg, synthetic.make_layer(cfg, layer=100 * rank + i, device=dev), max_tokens=T,
                           fused=not args.no_fused, launch=args.launch)
                  for i in range(L)]
    stamps = None
    if args.stamps and not args.via_patch and (ep_peer or not use_ep):
        stamps = (layers[L // 2].inner if use_ep else layers[L // 2]).enable_stamps()
    x_host = synthetic.make_tokens(cfg, T, step=rank).pin_memory()
    x_dev = x_host.to(dev)
    out_host = torch.empty((T, cfg.d_model), dtype=torch.bfloat16).pin_memory()
    stream = torch.cuda.Stream(device=dev)
    if use_ep and args.check:
        with torch.cuda.stream(stream):
            got = layers[0].forward(x_dev).clone()
            want = ref_layer.forward(x_dev).clone()
        stream.synchronize()
        diff = (got.float() - want.float()).abs().max().item()
        scale = want.float().abs().max().item()
        rec = {"max_abs_diff": diff, "max_abs": scale, "equal_frac": (got == want).float().mean().item(),
               "indices_equal": bool(torch.equal(layers[0].indices[:T] if ep_peer else
                                                 layers[0].inner.indices[rank * T:(rank + 1) * T],
                                                 ref_layer.indices[:T]))}
        flags = [None] * world
        dist.all_gather_object(flags, rec)
        if rank == 0:
            print(json.dumps({"check": "expert-parallel layer 0 vs the 1-GPU layer on each rank's own tokens",
                              "ranks": flags}), file=sys.stderr)

    def step_eager():
        h = x_dev
        for ly in layers:
            h = ly.forward(h)  # layer i+1 routes and computes on layer i's output: a true dependency chain
        return h

    # --- distinct experts touched per step (for the algorithmic byte count), from one eager pass
    with torch.cuda.stream(stream):
        step_eager()
    stream.synchronize()
    if use_ep:
        distinct = []
        for ly in layers:
            if ep_peer:  # a rank knows the routing of its own tokens: gather the others' (of its group)
                parts = [torch.empty_like(ly.indices[:T]) for _ in range(ep_deg)]
                dist.all_gather(parts, ly.indices[:T].contiguous(), group=ep_group)
                idx = torch.cat(parts).reshape(-1)
            else:
                idx = ly.inner.indices[:T * world].reshape(-1)
            distinct.append(int(torch.unique(idx[(idx >= ly.lo) & (idx < ly.hi)]).numel()))
        # bytes this rank must move: its local experts, the replicated router over all gathered tokens, rows in/out
        alg_bytes_step = sum(dn * cfg.expert_bytes + cfg.n_shared * cfg.expert_bytes + cfg.router_bytes
                             + 4 * T * ep_deg * cfg.d_model for dn in distinct)
        # With collectives between the kernels the step runs eagerly: capturing NCCL calls in a CUDA graph together
        # with the kernels stalled twice on this software stack (default and thread-local capture error mode; both
        # calls ran into their time limit without a GPU fault).  The peer-store form has no collective and is
        # captured like the one-GPU step.
        if not ep_peer:
            args.no_graph = True
    else:
        distinct = [int(torch.unique(ly.indices[:T]).numel()) for ly in layers]
        alg_bytes_step = sum(cfg.algorithmic_bytes(dn, T) for dn in distinct)

    graph = None
    if not args.no_graph:
        with torch.cuda.stream(stream):
            for _ in range(2):
                step_eager()
        stream.synchronize()
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                step_eager()
        except Exception as exc:  # e.g. a collective that cannot be captured: time eager launches instead
            if rank == 0:
                print(f"[bench] CUDA-graph capture failed ({type(exc).__name__}); timing eager launches", file=sys.stderr)
            graph = None
            torch.cuda.synchronize(dev)

    def run_step():
        if graph is not None:
            graph.replay()
        else:
            step_eager()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    # launches per layer: fused router (linear + top-k + plan), gate/up, down, combine (+3 for a shared expert);
    # expert parallel adds the local plan kernel (the NCCL and torch kernels are not counted)
    launches_per_layer = 4 + (3 if cfg.n_shared else 0) + (1 if use_ep else 0)
    one_launch = ep_peer or ((not use_ep) and layers[0].fused and layers[0].fused_workspace_bytes(T) > 0)
    if one_launch:
        launches_per_layer = 1  # zmoe_layer_decode: the whole block, shared expert included
    elif (not use_ep) and layers[0].fused and getattr(layers[0], "_chunked_ok", lambda t: False)(T):
        one_launch = True  # consecutive one-launch passes over eight rows each
        launches_per_layer = len(layers[0]._chunks(T))

    with torch.cuda.stream(stream):
        for _ in range(max(args.warmup, 3)):
            run_step()
    barrier()
    clocks = ClockSampler(local)  # samples over both timed regions (device-timed steps, then end to end)
    clocks.__enter__()
    per_repeat = []
    for _ in range(max(args.repeats, 1)):
        ev0 = torch.cuda.Event(enable_timing=True)
        ev1 = torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            ev0.record(stream)
            for _ in range(args.steps):
                run_step()
            ev1.record(stream)
        barrier()
        ms = ev0.elapsed_time(ev1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        per_repeat.append(ms / args.steps)
    ordered = sorted(per_repeat)
    ms_per_step = ordered[len(ordered) // 2]
    value = T * L * world / (ms_per_step * 1e-3)

    # --- end to end: pinned host rows in, result read back, every step
    barrier()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        for _ in range(3):
            x_dev.copy_(x_host, non_blocking=True)
            run_step()
            out_host.copy_(layers[-1].out[:T], non_blocking=True)
        stream.synchronize()
        e0.record(stream)
        for _ in range(args.steps):
            x_dev.copy_(x_host, non_blocking=True)
            run_step()
            out_host.copy_(layers[-1].out[:T], non_blocking=True)
            stream.synchronize()  # the caller reads the result before issuing the next step
        e1.record(stream)
    barrier()
    clocks.__exit__()
    e2e_ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e_value = T * L * world / (e2e_ms / args.steps * 1e-3)
    # a bounded wait that ran out anywhere in the timed launches voids the numbers: fail loudly
    with torch.cuda.stream(stream):
        for ly in layers:
            getattr(ly, "check_status", lambda: None)()

    if stamps is not None and rank == 0:
        v = stamps.cpu().tolist()
        names = ["push/router linear", "stage x", "logits arrive + scores", "select top-k", "weights + task list",
                 "gate/up + SwiGLU", "stage h", "down", "combine"]
        print(json.dumps({"stamps": "SM cycles of CTA 0, middle layer, last launch",
                          "total_cycles": v[9] - v[0],
                          "phases": {n: v[i + 1] - v[i] for i, n in enumerate(names)},
                          "ns_from_kernel_entry_to_dependency_wait_passed": v[11] - v[10],
                          "ns_kernel_entry_to_exit": v[12] - v[10]}), file=sys.stderr)
    if rank == 0:
        peak, peak_kind = _peaks()
        traffic, traffic_source = _measured_traffic(cfg, T, one_launch, alg_bytes_step / L)
        achieved = alg_bytes_step / (ms_per_step * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
            "ms_per_step_repeats": {"n": len(per_repeat), "min": ordered[0], "median": ms_per_step, "max": ordered[-1]},
            "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"{cfg.name}: d_model={cfg.d_model}, {cfg.n_experts} experts, top-{cfg.top_k}, "
                                   f"d_ff={cfg.d_ff}, {cfg.mode} 4-bit; T={T} decode tokens per step through "
                                   f"L={L} chained layers with distinct weights",
                       "tokens": T, "layers": L, "l2_policy": "inputs larger than L2: each step streams "
                       f"{alg_bytes_step / 1e6:.0f} MB of distinct expert weights across {L} layers",
                       "cuda_graph": graph is not None, "one_launch_block": bool(one_launch),
                       "launches_per_layer": launches_per_layer,
                       "block_launch": args.launch if one_launch else None,
                       "via_patch": bool(args.via_patch),
                       "parallelism": (f"ep{ep_deg}" + (f" x dp{world // ep_deg}" if ep_deg < world else "")
                                       + ": experts sharded; one launch per rank and layer, token rows and "
                                       "projected rows exchanged by peer stores inside the kernel (no collective)"
                                       if ep_peer else
                                       f"ep{world}: experts sharded, tokens all-gathered, per-slot rows "
                                       "reduce-scattered (NCCL)"
                                       + ("; kernels between the collectives replayed from per-layer CUDA graphs"
                                          if args.ep_segments else "")) if use_ep else f"replicas x{world}"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": traffic, "traffic_source": traffic_source,
                         "peak_kind": f"of {peak_kind}",
                         "algorithmic_bytes_per_launch": (alg_bytes_step / L / launches_per_layer) if one_launch else None,
                         "algorithmic_bytes_per_step": alg_bytes_step,
                         "note": ("rank 0's bytes over the step time (per-GPU fraction)" if use_ep else
                                  "whole block in one launch (zmoe_layer_decode)" if one_launch else
                                  "whole layer pass (4 kernels)")},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": T * cfg.d_model * 2,
                    "d2h_bytes_per_step": T * cfg.d_model * 2},
            "gpu_launches": launches_per_layer * L * args.steps,
            "clocks": clocks.summary(),
        }
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = _cpu_baseline(cfg, T)
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
