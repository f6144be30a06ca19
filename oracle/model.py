"""CPU restatement of the stacked decode model (test infrastructure, not a product path).

NumPy float32 arithmetic on bfloat16-rounded values: RMSNorm -> grouped-query attention with
per-head q/k RMSNorm and rotate-half RoPE -> residual -> RMSNorm -> MoE block (the per-family
recipe of :func:`oracle.semantics.moe_layer`, which follows src/zmlx/patch/patterns/moe_mlp.py:883-1063)
-> residual, greedy sampling as in the reference's fidelity check (src/zmlx/validate.py:211-225: the
patched and the unpatched model must produce the same token ids).  The decoder itself comes from
mlx_lm, which is not part of the reference tree; its published Qwen3 layout is restated here.
Sized for small configurations only (the whole history is recomputed at every step).
"""

from __future__ import annotations

import numpy as np

from . import semantics as S


def _rms(x, w, eps):
    x = np.asarray(x, dtype=np.float32)
    y = x * (1.0 / np.sqrt((x * x).mean(-1, keepdims=True, dtype=np.float32) + np.float32(eps)))
    return S.bf16(y.astype(np.float32) * np.asarray(w, dtype=np.float32))


def _rope(x, pos, theta):
    """x (B, H, S, hd) float32 (bf16 values); rotate-half; returns bf16 values."""
    hd = x.shape[-1]
    inv = 1.0 / (theta ** (np.arange(0, hd, 2, dtype=np.float64) / hd))
    ang = pos.astype(np.float64)[:, None] * inv[None, :]
    c = np.cos(ang).astype(np.float32)[None, None]
    s = np.sin(ang).astype(np.float32)[None, None]
    h = hd // 2
    x1, x2 = x[..., :h], x[..., h:]
    return S.bf16(np.concatenate([x1 * c - x2 * s, x2 * c + x1 * s], axis=-1))


def _linear(x, w):
    """bf16 x (.., K) times bf16 w (N, K), float32 accumulation, result rounded to bf16."""
    return S.bf16(np.asarray(x, dtype=np.float32) @ np.asarray(w, dtype=np.float32).T)


def forward_logits(cfg, p, ids):
    """ids (B, S) -> float32 logits (B, vocab) of the last position (full recompute, causal)."""
    B, Sq = ids.shape
    hq, hk, hd = cfg.n_heads, cfg.n_kv_heads, cfg.head_dim
    rep = hq // hk
    pos = np.arange(Sq)
    h = p["embed"][ids]  # (B, S, d)
    mcfg = cfg.moe
    for lp in p["layers"]:
        x = _rms(h, lp["attn_norm"], cfg.rms_eps)
        q = _linear(x, lp["q_w"]).reshape(B, Sq, hq, hd).transpose(0, 2, 1, 3)
        k = _linear(x, lp["k_w"]).reshape(B, Sq, hk, hd).transpose(0, 2, 1, 3)
        v = _linear(x, lp["v_w"]).reshape(B, Sq, hk, hd).transpose(0, 2, 1, 3)
        q = _rope(_rms(q, lp["q_norm"], cfg.rms_eps), pos, cfg.rope_theta)
        k = _rope(_rms(k, lp["k_norm"], cfg.rms_eps), pos, cfg.rope_theta)
        qg = q.reshape(B, hk, rep, Sq, hd)
        sc = np.einsum("bgrsd,bgpd->bgrsp", qg, k).astype(np.float32) * np.float32(1.0 / np.sqrt(hd))
        mask = pos[None, :] > pos[:, None]
        sc = np.where(mask, -np.inf, sc)
        sc = sc - sc.max(-1, keepdims=True)
        e = np.exp(sc, dtype=np.float32)
        pr = e / e.sum(-1, keepdims=True, dtype=np.float32)
        a = S.bf16(np.einsum("bgrsp,bgpd->bgrsd", pr.astype(np.float32), v).astype(np.float32))
        a = a.reshape(B, hq, Sq, hd).transpose(0, 2, 1, 3).reshape(B, Sq, hq * hd)
        h = S.bf16(h + _linear(a, lp["o_w"]))
        x = _rms(h, lp["ffn_norm"], cfg.rms_eps).reshape(B * Sq, cfg.d_model)
        m = lp["moe"]
        logits = _linear(x, m["router_w"])
        out, _, _ = S.moe_layer(x, logits, m, family=mcfg.family, top_k=mcfg.top_k, group_size=mcfg.group_size,
                                mode=mcfg.mode, expert_bias=m.get("expert_bias"), n_group=mcfg.n_group,
                                topk_group=mcfg.topk_group, routed_scaling_factor=mcfg.routed_scaling_factor,
                                norm_topk_prob=mcfg.norm_topk_prob, shared=m.get("shared"))
        h = S.bf16(h + out.reshape(B, Sq, cfg.d_model))
    last = _rms(h[:, -1], p["final_norm"], cfg.rms_eps)
    return np.asarray(last, dtype=np.float32) @ np.asarray(p["lm_head"], dtype=np.float32).T


def greedy(cfg, p, prompt, n_new):
    """prompt (B, S) int64 -> (tokens (B, n_new), top-2 logit gaps (B, n_new))."""
    ids = np.asarray(prompt)
    toks, gaps = [], []
    for _ in range(n_new):
        lg = forward_logits(cfg, p, ids)
        nxt = lg.argmax(-1)
        srt = np.sort(lg, axis=-1)
        gaps.append(srt[:, -1] - srt[:, -2])
        toks.append(nxt)
        ids = np.concatenate([ids, nxt[:, None]], axis=1)
    return np.stack(toks, 1), np.stack(gaps, 1)
