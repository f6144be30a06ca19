"""Greedy-token fidelity of the stacked decode model: the kernels against a torch reference on the same weights.

The protocol of src/zmlx/validate.py:211-225 (baseline vs patched model, greedy decoding, `matches`, `total`, first
divergence).  The baseline here is :class:`zmlx_b200.model.DequantMoE` -- the expert banks dequantised to bfloat16 and
plain torch ops -- in the same decoder; the candidate runs every MoE block through libzmoe.  Two sequences that
differ at step t are fed different tokens afterwards, so agreement is counted up to the first divergence and the
reference's top-2 logit margin at that step says whether it was a near tie (a bfloat16 ulp of a hidden value moves a
logit by ~1e-3; random-init models have many such ties, trained ones few).  Because a random-init model of this
depth has a median top-2 margin of about two bfloat16 ulps of its logits, the free-running comparison says little at
full size; the teacher-forced one (both models fed the reference's tokens, logits compared step by step) is the
measurement that carries.

    python -m zmlx_b200.validate --layers 48 --prompt 4096 --new 256 --batch 1      # one JSON line
"""

from __future__ import annotations

import json
import time

import torch

from .model import DECODER_CONFIGS, StackedDecoder, make_decoder_params


@torch.no_grad()
def greedy_with_margins(model: StackedDecoder, prompt: torch.Tensor, n_new: int):
    """Free-running greedy decoding; returns (tokens (B, n_new), top-2 logit margins (B, n_new))."""
    model.reset()
    toks, gaps = [], []
    logits = model.forward(prompt)
    for t in range(n_new):
        top = logits.topk(2, dim=-1).values
        gaps.append(top[:, 0] - top[:, 1])
        nxt = logits.argmax(-1)
        toks.append(nxt)
        if t + 1 < n_new:
            logits = model.forward(nxt[:, None])
    return torch.stack(toks, 1), torch.stack(gaps, 1)


@torch.no_grad()
def teacher_forced(ref: StackedDecoder, cand: StackedDecoder, prompt: torch.Tensor, n_new: int) -> dict:
    """Both models consume the REFERENCE's greedy tokens, so every step compares logits on the same history: how
    far the candidate's logits are from the reference's, and whether the arg-max agrees wherever the reference's
    own top-2 margin exceeds that distance (a flip inside the distance says nothing about either model)."""
    ref.reset()
    cand.reset()
    lr, lc = ref.forward(prompt), cand.forward(prompt)
    diffs, gaps, agree = [], [], []
    for t in range(n_new):
        top = lr.topk(2, dim=-1).values
        gaps.append(top[:, 0] - top[:, 1])
        diffs.append((lr - lc).abs().amax(-1))
        nxt = lr.argmax(-1)
        agree.append(nxt == lc.argmax(-1))
        if t + 1 < n_new:
            lr, lc = ref.forward(nxt[:, None]), cand.forward(nxt[:, None])
    gaps, diffs, agree = torch.stack(gaps, 1), torch.stack(diffs, 1), torch.stack(agree, 1)
    noise = float(diffs.max())
    clear = gaps > 2 * noise  # the reference's choice cannot flip under a perturbation of this size
    return {"steps": int(agree.numel()), "argmax_agree": int(agree.sum()),
            "max_abs_logit_diff": noise, "mean_abs_logit_diff": float(diffs.mean()),
            "logit_std": float(lr.std()), "median_ref_margin": float(gaps.median()),
            "steps_with_margin_above_2x_diff": int(clear.sum()),
            "argmax_agree_on_those": int((agree & clear).sum()),
            "disagreements": [{"seq": int(b), "step": int(t), "ref_margin": float(gaps[b, t]),
                               "logit_diff": float(diffs[b, t])} for b, t in (~agree).nonzero().tolist()][:16]}


def compare(ref_tokens: torch.Tensor, got_tokens: torch.Tensor, ref_gaps: torch.Tensor, near_tie: float = 4e-3) -> dict:
    """Per-sequence agreement up to the first divergence, with the reference's margin there."""
    B, N = ref_tokens.shape
    seqs = []
    for b in range(B):
        neq = (ref_tokens[b] != got_tokens[b]).nonzero()
        first = int(neq[0]) if neq.numel() else None
        seqs.append({"matches_before_divergence": N if first is None else first,
                     "first_divergence": first,
                     "ref_margin_at_divergence": None if first is None else float(ref_gaps[b, first]),
                     "near_tie": None if first is None else bool(ref_gaps[b, first] < near_tie),
                     "ref_near_ties_before": int((ref_gaps[b, :N if first is None else first] < near_tie).sum())})
    total = B * N
    matched = sum(s["matches_before_divergence"] for s in seqs)
    return {"total": total, "matches_before_divergence": matched,
            "identical_sequences": sum(s["first_divergence"] is None for s in seqs),
            "divergences_at_near_ties": sum(bool(s["near_tie"]) for s in seqs),
            "divergences_elsewhere": sum(s["first_divergence"] is not None and not s["near_tie"] for s in seqs),
            "min_ref_margin": float(ref_gaps.min()), "median_ref_margin": float(ref_gaps.median()),
            "sequences": seqs}


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
    ap.add_argument("--near-tie", type=float, default=3.2e-2,
                    help="reference margins below this count as ties (two bfloat16 ulps of a logit of magnitude 2..4)")
    ap.add_argument("--separate", action="store_true", help="candidate uses the separate kernels, not the one-launch block")
    args = ap.parse_args()
    cfg = DECODER_CONFIGS[args.config]
    if args.layers:
        cfg = replace(cfg, n_layers=args.layers)
    if args.vocab:
        cfg = replace(cfg, vocab=args.vocab)
    dev = torch.device("cuda", 0)
    params = make_decoder_params(cfg, device=dev)
    g = torch.Generator().manual_seed(1234)
    prompt = torch.randint(0, cfg.vocab, (args.batch, args.prompt), generator=g).to(dev)
    out = {"config": cfg.name, "layers": cfg.n_layers, "prompt": args.prompt, "new": args.new, "batch": args.batch}
    runs, models = {}, {}
    for impl in ("torch", "zmoe"):
        models[impl] = StackedDecoder(cfg, params, max_batch=args.batch, max_seq=args.prompt + args.new + 1,
                                      fused=not args.separate, moe_impl=impl)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        runs[impl] = greedy_with_margins(models[impl], prompt, args.new)
        torch.cuda.synchronize()
        out[f"{impl}_seconds"] = round(time.perf_counter() - t0, 2)
    out["free_running"] = compare(runs["torch"][0].cpu(), runs["zmoe"][0].cpu(), runs["torch"][1].cpu(),
                                  near_tie=args.near_tie)
    out["teacher_forced"] = teacher_forced(models["torch"], models["zmoe"], prompt, args.new)
    print(json.dumps(out))


if __name__ == "__main__":
    _main()
