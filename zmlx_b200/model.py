"""Stacked decode model around the MoE block (the Qwen3-30B-A3B-shaped configuration).

48 decoder layers of: RMSNorm -> GQA attention (32 query heads, 4 KV heads of dim 128, per-head
q/k RMSNorm, RoPE base 1e6, KV cache) -> residual -> RMSNorm -> MoE block -> residual; greedy
sampling.  The reference drives its patched MoE blocks with mlx_lm's decoder and validates
token fidelity with greedy decoding (src/zmlx/validate.py:68-125, 211-225); here the attention side
is plain torch ops -- float32 score/softmax arithmetic, so that a CPU restatement can reproduce it
-- and every MoE block is a :class:`zmlx_b200.layer.MoELayer` (or its expert-parallel form), i.e.
the libzmoe kernels.  Weights are random-init: no checkpoint is involved.

Command line: ``python -m zmlx_b200.model --layers 48 --prompt 4096 --new 256 --batch 1`` prints
prefill and decode rates as one JSON line; under ``python -m torch.distributed.run --nproc-per-node N`` the MoE
blocks run expert-parallel over the N GPUs (every rank decodes its own batch, here the same prompt).
"""

from __future__ import annotations

import json
import math
import time
from dataclasses import dataclass, field

import torch

from . import synthetic
from .layer import MoELayer
from .synthetic import MoEConfig


@dataclass(frozen=True)
class DecoderConfig:
    name: str
    n_layers: int
    d_model: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    vocab: int
    moe: MoEConfig = field(default_factory=lambda: synthetic.CONFIGS["c2"])
    rope_theta: float = 1e6
    rms_eps: float = 1e-6


DECODER_CONFIGS = {
    # stacked decode model of the benchmark list: Qwen3-30B-A3B shapes
    "c4": DecoderConfig("c4-qwen3-30b-a3b-stacked", 48, 2048, 32, 4, 128, 151936),
}


def _randn(shape, seed: int, std: float, device) -> torch.Tensor:
    """Seeded N(0, std) in bfloat16; generated on the CPU so that every device sees the same values."""
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    return (torch.randn(shape, generator=g, dtype=torch.float32) * std).to(torch.bfloat16).to(device)


def make_decoder_params(cfg: DecoderConfig, *, device="cpu", moe_device=None) -> dict:
    """Random-init tensors of the whole model.  ``moe_device`` chooses where the expert banks are generated
    and quantised (their seeded generator is per device: use "cpu" when a CPU restatement must see the
    same weights; the tensors are moved to ``device`` afterwards)."""
    d, hq, hk, hd = cfg.d_model, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim
    moe_device = moe_device or device
    p = {
        "embed": _randn((cfg.vocab, d), 11, 1.0, device),
        "lm_head": _randn((cfg.vocab, d), 13, 0.02, device),
        "final_norm": torch.ones(d, dtype=torch.bfloat16, device=device),
        "layers": [],
    }
    for i in range(cfg.n_layers):
        s = 1000 + 17 * i
        moe = synthetic.make_layer(cfg.moe, layer=i, device=moe_device)
        if str(moe_device) != str(device):
            moe = _to_device(moe, device)
        p["layers"].append({
            "attn_norm": torch.ones(d, dtype=torch.bfloat16, device=device),
            "q_w": _randn((hq * hd, d), s + 1, 0.02, device),
            "k_w": _randn((hk * hd, d), s + 2, 0.02, device),
            "v_w": _randn((hk * hd, d), s + 3, 0.02, device),
            "o_w": _randn((d, hq * hd), s + 4, 0.02, device),
            "q_norm": torch.ones(hd, dtype=torch.bfloat16, device=device),
            "k_norm": torch.ones(hd, dtype=torch.bfloat16, device=device),
            "ffn_norm": torch.ones(d, dtype=torch.bfloat16, device=device),
            "moe": moe,
        })
    return p


def _to_device(tree, device):
    if isinstance(tree, dict):
        return {k: _to_device(v, device) for k, v in tree.items()}
    if isinstance(tree, torch.Tensor):
        return tree.to(device)
    return tree


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """float32 statistics, result in bfloat16."""
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (y * w.float()).to(torch.bfloat16)


def rope_tables(head_dim: int, max_pos: int, theta: float, device) -> tuple[torch.Tensor, torch.Tensor]:
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float64) / head_dim))
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * inv[None, :]
    return ang.cos().float().to(device), ang.sin().float().to(device)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x (B, H, S, hd) bfloat16; cos/sin (S, hd/2) float32; rotate-half convention; result bfloat16."""
    xf = x.float()
    h = xf.shape[-1] // 2
    x1, x2 = xf[..., :h], xf[..., h:]
    c, s = cos[None, None], sin[None, None]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).to(torch.bfloat16)


SDPA_MIN_SEQ = 1024  # prompts at least this long take torch's fused attention in the prefill


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, q_pos0: int, *, q_chunk: int = 512) -> torch.Tensor:
    """Causal grouped-query attention with float32 arithmetic.  q (B, Hq, S, hd); k, v (B, Hk, P, hd) hold
    positions 0..P-1 and the S queries sit at positions q_pos0..q_pos0+S-1.  Returns (B, Hq, S, hd) bfloat16."""
    B, Hq, S, hd = q.shape
    Hk, P = k.shape[1], k.shape[2]
    rep = Hq // Hk
    if q_pos0 == 0 and S == P and S >= SDPA_MIN_SEQ:
        # a long prompt from position 0: torch's fused causal attention (bfloat16 inputs, float32 accumulation
        # inside); the float32 path below stays for everything a CPU restatement is compared with
        return torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
    kf = k.float()
    vf = v.float()
    scale = 1.0 / math.sqrt(hd)
    out = torch.empty((B, Hq, S, hd), dtype=torch.bfloat16, device=q.device)
    kpos = torch.arange(P, device=q.device)
    for s0 in range(0, S, q_chunk):
        s1 = min(S, s0 + q_chunk)
        qf = q[:, :, s0:s1].float().view(B, Hk, rep, s1 - s0, hd)
        sc = torch.einsum("bgrsd,bgpd->bgrsp", qf, kf) * scale
        qpos = torch.arange(q_pos0 + s0, q_pos0 + s1, device=q.device)
        sc = sc.masked_fill(kpos[None, :] > qpos[:, None], float("-inf"))
        pr = torch.softmax(sc, dim=-1)
        o = torch.einsum("bgrsp,bgpd->bgrsd", pr, vf)
        out[:, :, s0:s1] = o.reshape(B, Hq, s1 - s0, hd).to(torch.bfloat16)
    return out


class DequantMoE:
    """GPU-side reference of one MoE block: the packed banks dequantised once to bfloat16, torch ops only (none of
    this package's kernels).  It plays the role of the unpatched model in the reference's fidelity check
    (src/zmlx/validate.py:211-225); its arithmetic follows the per-family recipe the kernels implement (router in
    float32 on bfloat16 logits, gate/up rounded to bfloat16, SwiGLU, down rounded to bfloat16, weighted sum over the
    slots in float32), with two differences that make it an independent check rather than a copy: the weights are
    ROUNDED to bfloat16 (the kernels use q * s + b exactly) and the sums run in cuBLAS order."""

    def __init__(self, cfg: MoEConfig, p: dict):
        from . import quant

        if cfg.mode != "affine":
            raise ValueError("the dequantised reference takes affine banks")
        self.cfg = cfg
        self.router_w = p["router_w"]
        self.bias = p.get("expert_bias")

        def deq(d, name):
            return quant.dequantize_affine(d[f"{name}_w"], d[f"{name}_s"], d[f"{name}_b"], cfg.group_size).to(torch.bfloat16)

        self.w = {n: deq(p, n) for n in ("gate", "up", "down")}  # (E, N, K) bfloat16
        self.shared = {n: deq(p["shared"], n)[0] for n in ("gate", "up", "down")} if p.get("shared") else None

    def _route(self, logits: torch.Tensor):
        cfg = self.cfg
        lg = logits.float()
        if cfg.family == "qwen3":
            probs = torch.softmax(lg, dim=-1)
            w, idx = probs.topk(cfg.top_k, dim=-1)
            if cfg.norm_topk_prob:
                w = w / w.sum(-1, keepdim=True)
            return idx, w
        if cfg.family in ("glm", "deepseek"):
            aff = torch.sigmoid(lg)
            sc = aff + self.bias
            E = sc.shape[-1]
            if cfg.n_group > 1:
                g = sc.reshape(-1, cfg.n_group, E // cfg.n_group)
                gs = g.topk(2, dim=-1).values.sum(-1)
                keep = torch.zeros_like(gs).scatter_(-1, gs.topk(cfg.topk_group, dim=-1).indices, 1.0)
                sc = (g * keep[..., None]).reshape(sc.shape)
            idx = sc.topk(cfg.top_k, dim=-1).indices
            w = torch.gather(aff, -1, idx)
            return idx, w / w.sum(-1, keepdim=True) * cfg.routed_scaling_factor
        w, idx = lg.topk(cfg.top_k, dim=-1)  # generic: top-k of the logits, softmax over the k
        return idx, torch.softmax(w, dim=-1)

    @staticmethod
    def _mlp(x, wg, wu, wd):
        g, u = x @ wg.T, x @ wu.T  # bfloat16 out, float32 accumulation
        h = (torch.nn.functional.silu(g.float()) * u.float()).to(torch.bfloat16)
        return h @ wd.T

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        idx, w = self._route(x @ self.router_w.T)
        T, K = idx.shape
        y = torch.zeros((T, K, cfg.d_model), dtype=torch.bfloat16, device=x.device)
        flat = idx.reshape(-1)
        for e in torch.unique(flat).tolist():  # one expert at a time over all of its rows
            rows = (flat == e).nonzero(as_tuple=True)[0]
            y.view(T * K, -1)[rows] = self._mlp(x[rows // K], self.w["gate"][e], self.w["up"][e], self.w["down"][e])
        out = (y.float() * w[..., None]).sum(1).to(torch.bfloat16)
        if self.shared is not None:
            out = out + self._mlp(x, self.shared["gate"], self.shared["up"], self.shared["down"])
        return out


class StackedDecoder:
    """The model on one GPU (``world == 1``) or with expert-parallel MoE blocks (one process per GPU; every
    rank runs the attention side of its own sequences and the experts are sharded, see zmlx_b200/ep.py)."""

    MOE_CHUNK = 4096  # tokens per MoE call during prefill (bounds the per-layer work buffers)
    EP_CHUNK = 256

    def __init__(self, cfg: DecoderConfig, params: dict, *, max_batch: int, max_seq: int, fused: bool = True,
                 world: int = 1, rank: int = 0, group=None, moe_impl: str = "zmoe"):
        self.cfg = cfg
        self.p = params
        dev = params["embed"].device
        if dev.type != "cuda":
            raise RuntimeError("StackedDecoder needs its tensors on a CUDA device (the MoE kernels have no CPU path)")
        self.device = dev
        self.max_batch, self.max_seq = max_batch, max_seq
        self.world, self.rank = world, rank
        self.cos, self.sin = rope_tables(cfg.head_dim, max_seq, cfg.rope_theta, dev)
        L, hk, hd = cfg.n_layers, cfg.n_kv_heads, cfg.head_dim
        self.k_cache = torch.zeros((L, max_batch, hk, max_seq, hd), dtype=torch.bfloat16, device=dev)
        self.v_cache = torch.zeros_like(self.k_cache)
        self.pos = 0
        self.peer, self.peer_tokens = None, 0
        if moe_impl == "torch":  # the dequantised torch reference in place of the kernels (fidelity check)
            self.chunk = 1 << 30
            self.moe = [DequantMoE(cfg.moe, lp["moe"]) for lp in params["layers"]]
        elif world > 1:
            from . import ep

            self.chunk = self.EP_CHUNK
            self.moe = [ep.EPMoELayer(cfg.moe, lp["moe"], rank=rank, world=world, max_tokens=self.chunk,
                                      group=group) for lp in params["layers"]]
            # decode steps (max_batch rows per rank) take the one-launch block with the peer-store exchange when
            # the rows of all ranks fit one launch; prefill chunks keep the collectives
            if ep.peer_block_supported(cfg.moe, max_batch, world):
                lo, hi = ep.expert_range(cfg.moe.n_experts, world, rank)
                self.peer_tokens = max_batch
                self.peer = [ep.PeerMoELayer(cfg.moe, ep.shard_params(lp["moe"], lo, hi), rank=rank, world=world,
                                             tokens=max_batch, group=group, launch="pdl")
                             for lp in params["layers"]]
        else:
            self.chunk = self.MOE_CHUNK
            self.moe = [MoELayer(cfg.moe, lp["moe"], max_tokens=max(max_batch, 64), fused=fused)
                        for lp in params["layers"]]

    def reset(self) -> None:
        self.pos = 0

    def _moe(self, i: int, x: torch.Tensor) -> torch.Tensor:
        """x (N, d) bfloat16 -> (N, d); long prefills go through in chunks."""
        if self.peer is not None and x.shape[0] == self.peer_tokens:
            return self.peer[i].forward(x if x.is_contiguous() else x.contiguous())
        if x.shape[0] <= self.chunk:
            return self.moe[i].forward(x)
        return torch.cat([self.moe[i].forward(x[s:s + self.chunk]).clone()
                          for s in range(0, x.shape[0], self.chunk)])

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        """ids (B, S) int64 at positions pos..pos+S-1 -> float32 logits (B, vocab) of the last position;
        the KV cache and the position advance."""
        cfg = self.cfg
        B, S = ids.shape
        if B > self.max_batch or self.pos + S > self.max_seq:
            raise ValueError(f"batch {B} / positions {self.pos + S} exceed the cache ({self.max_batch}, {self.max_seq})")
        hq, hk, hd = cfg.n_heads, cfg.n_kv_heads, cfg.head_dim
        p0, p1 = self.pos, self.pos + S
        cos, sin = self.cos[p0:p1], self.sin[p0:p1]
        h = self.p["embed"][ids]  # (B, S, d) bfloat16
        for i, lp in enumerate(self.p["layers"]):
            x = rms_norm(h, lp["attn_norm"], cfg.rms_eps)
            q = (x @ lp["q_w"].T).view(B, S, hq, hd).transpose(1, 2)
            k = (x @ lp["k_w"].T).view(B, S, hk, hd).transpose(1, 2)
            v = (x @ lp["v_w"].T).view(B, S, hk, hd).transpose(1, 2)
            q = apply_rope(rms_norm(q, lp["q_norm"], cfg.rms_eps), cos, sin)
            k = apply_rope(rms_norm(k, lp["k_norm"], cfg.rms_eps), cos, sin)
            self.k_cache[i, :B, :, p0:p1] = k
            self.v_cache[i, :B, :, p0:p1] = v
            a = attention(q, self.k_cache[i, :B, :, :p1], self.v_cache[i, :B, :, :p1], p0)
            a = a.transpose(1, 2).reshape(B, S, hq * hd)
            h = h + (a @ lp["o_w"].T)
            x = rms_norm(h, lp["ffn_norm"], cfg.rms_eps)
            m = self._moe(i, x.reshape(B * S, cfg.d_model))
            h = h + m.view(B, S, cfg.d_model)
        self.pos = p1
        last = rms_norm(h[:, -1], self.p["final_norm"], cfg.rms_eps)
        return (last @ self.p["lm_head"].T).float()

    # -- decode step with static shapes (for CUDA-graph replay) ------------------------------------------
    def _decode_static(self, st: dict) -> None:
        """One greedy step for the B sequences in ``st``: reads the current token ids and the position from
        device buffers, appends to the KV cache, attends over the whole cache with the positions beyond the
        current one masked, and leaves the next ids, the advanced position and the token log in ``st`` --
        no shape or host value depends on the position, so the step can be captured once and replayed."""
        cfg = self.cfg
        ids, pos = st["ids"], st["pos"]
        B = ids.shape[0]
        hq, hk, hd = cfg.n_heads, cfg.n_kv_heads, cfg.head_dim
        rep = hq // hk
        cos, sin = self.cos.index_select(0, pos), self.sin.index_select(0, pos)
        dead = (st["kpos"] > pos)[None, None, None, None, :]  # cache slots after the current position
        scale = 1.0 / math.sqrt(hd)
        h = self.p["embed"].index_select(0, ids).unsqueeze(1)  # (B, 1, d)
        for i, lp in enumerate(self.p["layers"]):
            x = rms_norm(h, lp["attn_norm"], cfg.rms_eps)
            q = (x @ lp["q_w"].T).view(B, 1, hq, hd).transpose(1, 2)
            k = (x @ lp["k_w"].T).view(B, 1, hk, hd).transpose(1, 2)
            v = (x @ lp["v_w"].T).view(B, 1, hk, hd).transpose(1, 2)
            q = apply_rope(rms_norm(q, lp["q_norm"], cfg.rms_eps), cos, sin)
            k = apply_rope(rms_norm(k, lp["k_norm"], cfg.rms_eps), cos, sin)
            self.k_cache[i, :B].index_copy_(2, pos, k)
            self.v_cache[i, :B].index_copy_(2, pos, v)
            sc = torch.einsum("bgrsd,bgpd->bgrsp", q.float().view(B, hk, rep, 1, hd), self.k_cache[i, :B].float())
            pr = torch.softmax((sc * scale).masked_fill(dead, float("-inf")), dim=-1)
            a = torch.einsum("bgrsp,bgpd->bgrsd", pr, self.v_cache[i, :B].float()).to(torch.bfloat16)
            h = h + (a.reshape(B, 1, hq * hd) @ lp["o_w"].T)
            x = rms_norm(h, lp["ffn_norm"], cfg.rms_eps)
            h = h + self._moe(i, x.reshape(B, cfg.d_model)).view(B, 1, cfg.d_model)
        last = rms_norm(h[:, -1], self.p["final_norm"], cfg.rms_eps)
        nxt = (last @ self.p["lm_head"].T).float().argmax(-1)
        st["log"].index_copy_(1, st["n"], nxt[:, None])
        ids.copy_(nxt)
        pos.add_(1)
        st["n"].add_(1)

    @torch.no_grad()
    def generate(self, prompt: torch.Tensor, n_new: int, *, graph: bool = False) -> torch.Tensor:
        """Greedy decoding: prompt (B, S) int64 -> (B, n_new) int64 new tokens.  With ``graph`` the decode step
        is captured in a CUDA graph once and replayed (single-GPU model only)."""
        self.reset()
        B = prompt.shape[0]
        nxt = self.forward(prompt).argmax(-1)
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if not graph or n_new < 4 or self.world > 1:
            out = torch.empty((B, n_new), dtype=torch.int64, device=self.device)
            ev0.record()
            for t in range(n_new):
                out[:, t] = nxt
                if t + 1 < n_new:
                    nxt = self.forward(nxt[:, None]).argmax(-1)
            ev1.record()
            self.last_decode = (ev0, ev1, n_new - 1)  # events around n_new - 1 decode steps
            return out
        dev = self.device
        st = {"ids": nxt.clone(), "pos": torch.tensor([self.pos], dtype=torch.int64, device=dev),
              "kpos": torch.arange(self.max_seq, device=dev), "n": torch.ones(1, dtype=torch.int64, device=dev),
              "log": torch.zeros((B, n_new + 2), dtype=torch.int64, device=dev)}
        st["log"][:, 0] = nxt
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            self._decode_static(st)  # eager: allocates the one-launch workspaces before the capture
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                self._decode_static(st)
            ev0.record(side)
            for _ in range(n_new - 2):
                g.replay()
            ev1.record(side)
        self.last_decode = (ev0, ev1, n_new - 2)  # events around the replayed steps (capture excluded)
        torch.cuda.current_stream(dev).wait_stream(side)
        self.pos += n_new - 1
        return st["log"][:, :n_new].clone()


def _main() -> None:
    import argparse
    from dataclasses import replace

    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="c4")
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--vocab", type=int, default=None)
    ap.add_argument("--prompt", type=int, default=4096)
    ap.add_argument("--new", type=int, default=256)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--no-fused", action="store_true")
    ap.add_argument("--no-graph", action="store_true")
    args = ap.parse_args()
    cfg = DECODER_CONFIGS[args.config]
    if args.layers:
        cfg = replace(cfg, n_layers=args.layers)
    if args.vocab:
        cfg = replace(cfg, vocab=args.vocab)
    import os

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:  # under torch.distributed.run: expert-parallel MoE blocks, every rank its own sequences
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)
    params = make_decoder_params(cfg, device=dev)  # same seeds on every rank: one model
    model = StackedDecoder(cfg, params, max_batch=args.batch, max_seq=args.prompt + args.new,
                           fused=not args.no_fused, world=world, rank=rank)
    g = torch.Generator(device="cpu")
    g.manual_seed(5)
    prompt = torch.randint(0, cfg.vocab, (args.batch, args.prompt), generator=g).to(dev)
    with torch.no_grad():
        model.reset()
        model.forward(prompt[:1])  # untimed, at the timed length: loads the kernels and sizes every work buffer
        torch.cuda.synchronize()
        model.reset()
        t0 = time.perf_counter()
        model.forward(prompt)
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        toks = model.generate(prompt, args.new, graph=not args.no_graph)
        torch.cuda.synchronize()
        ev0, ev1, steps = model.last_decode
        decode_s = ev0.elapsed_time(ev1) * 1e-3
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
        dist.destroy_process_group()
        if rank != 0:
            return
    print(json.dumps({
        "model": cfg.name, "n_gpus": world, "layers": cfg.n_layers, "batch": args.batch, "prompt": args.prompt, "new": args.new,
        "one_launch_block": not args.no_fused,
        "prefill_tokens_per_s": args.batch * args.prompt / (t1 - t0),
        "cuda_graph_decode": not args.no_graph,
        "decode_tokens_per_s": args.batch * steps / max(decode_s, 1e-9),
        "decode_ms_per_step": 1e3 * decode_s / max(steps, 1),
        "decode_steps_timed": steps,
        "first_tokens": toks[0, :16].tolist(),
    }))


if __name__ == "__main__":
    _main()
