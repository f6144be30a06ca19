"""CPU: MLX-format safetensors ingestion of a MoE block (names and layouts of mlx-community checkpoints)."""

import torch

from zmlx_b200 import checkpoint, quant, synthetic


def _tiny(base="c5"):
    return synthetic.CONFIGS[base].scaled(n_experts=8, d_model=128, d_ff=64, top_k=2, n_group=1, topk_group=1)


def test_round_trip_of_a_block_with_shared_expert_and_bias(tmp_path):
    cfg = _tiny("c5")
    p = synthetic.make_layer(cfg)
    f = str(tmp_path / "model-00001-of-00001.safetensors")
    checkpoint.save_moe_params(p, f, "model.layers.3.mlp")
    assert checkpoint.moe_block_prefixes(str(tmp_path)) == ["model.layers.3.mlp"]
    q = checkpoint.load_moe_params(str(tmp_path), "model.layers.3.mlp")
    for k in ("router_w", "expert_bias", "gate_w", "gate_s", "gate_b", "up_w", "down_b"):
        assert q[k].dtype == p[k].dtype and torch.equal(q[k].view(torch.uint8), p[k].view(torch.uint8)), k
    for k, v in p["shared"].items():
        assert q["shared"][k].shape == v.shape and torch.equal(q["shared"][k].view(torch.uint8), v.view(torch.uint8)), k


def test_blocks_come_back_in_layer_order_and_quantised_routers_are_dequantised(tmp_path):
    from safetensors.torch import load_file, save_file

    cfg = _tiny("c2")
    for i in (10, 2):
        checkpoint.save_moe_params(synthetic.make_layer(cfg, layer=i), str(tmp_path / f"shard{i}.safetensors"),
                                   f"model.layers.{i}.mlp")
    assert checkpoint.moe_block_prefixes(str(tmp_path)) == ["model.layers.2.mlp", "model.layers.10.mlp"]
    # an 8-bit router as some 4-bit conversions keep it: packed (E, d/4) uint32 + scales/biases per 64
    f = str(tmp_path / "shard2.safetensors")
    t = load_file(f)
    rw = t["model.layers.2.mlp.gate.weight"].to(torch.float32)
    g = rw.reshape(rw.shape[0], -1, 64)
    lo, hi = g.amin(-1, keepdim=True), g.amax(-1, keepdim=True)
    scale = ((hi - lo) / 255).clamp_min(1e-8)
    codes = ((g - lo) / scale).round().clamp(0, 255).to(torch.int64).reshape(rw.shape[0], -1, 4)
    packed = (codes[..., 0] | (codes[..., 1] << 8) | (codes[..., 2] << 16) | (codes[..., 3] << 24)).to(torch.uint32)
    t["model.layers.2.mlp.gate.weight"] = packed
    t["model.layers.2.mlp.gate.scales"] = scale.squeeze(-1).to(torch.bfloat16)
    t["model.layers.2.mlp.gate.biases"] = lo.squeeze(-1).to(torch.bfloat16)
    save_file(t, f)
    q = checkpoint.load_moe_params(str(tmp_path), "model.layers.2.mlp")
    assert q["router_w"].dtype == torch.bfloat16 and q["router_w"].shape == rw.shape
    assert (q["router_w"].float() - rw).abs().max() <= 2 * float(scale.max()) + 1e-3
    assert q["shared"] is None and q["expert_bias"] is None
    # the packed banks are what the kernels read: dequantising them gives back the quantiser's values
    w = quant.dequantize_affine(q["gate_w"], q["gate_s"], q["gate_b"], 64)
    assert w.shape == (cfg.n_experts, cfg.d_ff, cfg.d_model)
