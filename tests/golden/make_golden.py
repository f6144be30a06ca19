"""Writes tests/golden/known_answers.json.

The reference's tests for this path hold no stored vectors; what they do hold are
known-answer cases whose expected output follows from the case itself.  This
script restates those cases (inputs as compact recipes, expected outputs spelled
out) so that both the CPU oracle and the CUDA kernels can be pinned to them.
MLX cannot be imported on this platform, so nothing here is produced by running
the reference.

Sources (paths relative to the ZMLX tree):
  tests/test_deepseek_router_topk_sigmoid.py:75-104   boosted-bias selection
  tests/test_deepseek_router_topk_sigmoid.py:107-124  zero-logit tie-break
  tests/test_deepseek_router_topk_sigmoid.py:127-180  group-limited selection
  tests/test_fused_ops.py:247-267                     top-2 hand-written rows
  tests/test_gather_qmm_combine.py:149-283            one-hot gate / K = 1 identities

Run: python tests/golden/make_golden.py
"""

import json
import os


def main() -> None:
    cases = []
    for E in (256, 384):
        # all-zero logits and bias: the first 8 experts win, weights are exactly 1/8
        cases.append({
            "name": f"sigmoid_zero_tiebreak_E{E}", "router": "sigmoid", "E": E, "k": 8, "rows": 1,
            "logits": {"kind": "zeros"}, "bias": {"kind": "zeros"}, "n_group": 1, "topk_group": 1,
            "indices": [list(range(8))], "weights": [[0.125] * 8], "weights_exact": True, "ordered": True,
        })
        # logits rise with the expert id, eight experts get +10 bias: exactly those are chosen;
        # with equal bias the larger logit scores higher, so the canonical order is descending id
        boost = [0, 7, 13, 64, 127, 128, E - 2, E - 1]
        cases.append({
            "name": f"sigmoid_boosted_bias_E{E}", "router": "sigmoid", "E": E, "k": 8, "rows": 3,
            "logits": {"kind": "linspace_rows", "lo": -2.0, "hi": 2.0, "row_step": 0.1},
            "bias": {"kind": "sparse", "index": boost, "value": [10.0] * 8}, "n_group": 1, "topk_group": 1,
            "indices": [sorted(boost, reverse=True)] * 3, "weights": None, "ordered": True,
        })
    # group-limited selection: groups 0..3 hold the seven +10 experts, group 7 holds a +9 decoy and is
    # dropped; the eighth pick is the lowest-id remaining expert of a kept group (score 0.5), id 2
    cases.append({
        "name": "sigmoid_group_limited_E256", "router": "sigmoid", "E": 256, "k": 8, "rows": 1,
        "logits": {"kind": "zeros"},
        "bias": {"kind": "sparse", "index": [0, 1, 32, 33, 64, 65, 96, 224],
                 "value": [10.0, 10.0, 10.0, 10.0, 10.0, 10.0, 10.0, 9.0]},
        "n_group": 8, "topk_group": 4,
        "indices": [[0, 1, 32, 33, 64, 65, 96, 2]], "weights": [[0.125] * 8], "weights_exact": True,
        "ordered": True,
    })
    # top-2 of two hand-written rows
    cases.append({
        "name": "softmax_top2_rows", "router": "topk_then_softmax", "E": 8, "k": 2, "rows": 2,
        "logits": {"kind": "explicit", "values": [[0.1, 0.2, 0.3, 0.4, 0.5, 0.6, 0.7, 0.8],
                                                  [0.9, 0.8, 0.7, 0.6, 0.5, 0.4, 0.3, 0.2]]},
        "indices": [[7, 6], [0, 1]], "weights": None, "ordered": True, "weights_sum_to_one": True,
    })
    out = {"note": "known-answer cases restated from the reference's tests; see make_golden.py", "cases": cases}
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "known_answers.json")
    with open(path, "w") as f:
        json.dump(out, f, indent=1)
    print(path, len(cases), "cases")


if __name__ == "__main__":
    main()
