"""Pins the CPU oracle to vectors produced by the reference's own code (tests/golden)."""

import dataclasses

import numpy as np
import torch

from oracle import kimi_oracle as K
from oracle import megamoe_oracle as M
from oracle import moe_oracle as O
from vibe_megakernel_b200 import synthetic


def bf16(bits):
    return torch.from_numpy(bits.copy()).view(torch.bfloat16)


def q_bytes(t):
    return t.view(torch.uint8).numpy()


def test_weight_and_activation_block_scales(golden_dir):
    g = np.load(golden_dir / "quantizers.npz")
    value = bf16(g["w_in"])
    for power in (0, 1):
        q, s = O.quantize_weight(value, power_of_two=bool(power))
        assert np.array_equal(q_bytes(q), g[f"w_q_{power}"])
        assert np.array_equal(s.numpy(), g[f"w_s_{power}"])
        assert np.array_equal(O.dequantize_weight(q, s).numpy(), g[f"w_deq_{power}"])
        q, s = O.quantize_activation(value, power_of_two=bool(power))
        assert np.array_equal(q_bytes(q), g[f"wa_q_{power}"])
        assert np.array_equal(s.numpy(), g[f"wa_s_{power}"])
    value = bf16(g["a_in"])
    for power in (0, 1):
        q, s = O.quantize_activation(value, power_of_two=bool(power))
        assert np.array_equal(q_bytes(q), g[f"a_q_{power}"])
        assert np.array_equal(s.numpy(), g[f"a_s_{power}"])
        assert np.array_equal(O.dequantize_activation(q, s).numpy(), g[f"a_deq_{power}"])


def test_scale_edge_values(golden_dir):
    g = np.load(golden_dir / "quantizers.npz")
    value = torch.from_numpy(g["e_in"])
    q, s = O.quantize_activation(value, group=32, scale_format="e8m0")
    assert np.array_equal(q_bytes(q), g["e_q"])
    assert np.array_equal(s.numpy(), g["e_s"])
    assert np.array_equal(O.dequantize_activation(q, s, group=32).numpy(), g["e_deq"])
    q, s = O.quantize_activation(value)
    assert np.array_equal(q_bytes(q), g["ef_q"])
    assert np.array_equal(s.numpy(), g["ef_s"])
    value = torch.from_numpy(g["f_in"])
    q, s = O.quantize_activation(value)
    assert np.array_equal(q_bytes(q), g["f_q"])
    assert np.array_equal(s.numpy(), g["f_s"])
    # an all-zero row takes the 1e-4 floor
    assert float(s[1, 0]) == np.float32(1e-4) / np.float32(448)


def test_sigmoid_group_router(golden_dir):
    g = np.load(golden_dir / "routers.npz")
    for name, (e, k, groups, top_groups), scaling in zip(("ds", "kimi", "small", "pair"), g["sig_cases"], g["sig_scaling"]):
        scores, bias = torch.from_numpy(g[f"{name}_scores"]), torch.from_numpy(g[f"{name}_bias"])
        for t in range(scores.shape[0]):
            ids, w = O.route_sigmoid_grouped(scores[t], bias, int(k), int(groups), int(top_groups), float(scaling))
            assert np.array_equal(ids.numpy(), g[f"{name}_ids"][t])
            assert np.array_equal(w.numpy(), g[f"{name}_w"][t])
    ids, w = O.route_sigmoid_grouped(torch.zeros(8), torch.zeros(8), 2, 2, 1, 2.5)
    assert ids.tolist() == [0, 1] == g["tie_ids"].tolist()
    assert w.tolist() == [1.25, 1.25] == g["tie_w"].tolist()
    scores = torch.from_numpy(g["tie2_scores"])
    ids, w = O.route_sigmoid_grouped(scores, torch.zeros(16), 6, 4, 2, 1.0)
    assert np.array_equal(ids.numpy(), g["tie2_ids"]) and np.array_equal(w.numpy(), g["tie2_w"])
    ids, w = O.route_sigmoid_grouped(scores, torch.zeros(16), 6, 4, 1, 1.0)
    assert np.array_equal(ids.numpy(), g["tie3_ids"]) and np.array_equal(w.numpy(), g["tie3_w"])


def test_softmax_router(golden_dir):
    g = np.load(golden_dir / "routers.npz")
    for name, k in (("sm16", 4), ("sm128", 8), ("sm8", 2)):
        scores = torch.from_numpy(g[f"{name}_scores"])
        for t in range(scores.shape[0]):
            ids, w = O.route_softmax(scores[t], k)
            assert np.array_equal(ids.numpy(), g[f"{name}_ids"][t])
            assert np.array_equal(w.numpy(), g[f"{name}_w"][t])


def test_sqrt_softplus_router(golden_dir):
    # vectors made with the expressions of megabench/tasks/dsv41.py:623-626
    g = np.load(golden_dir / "routers.npz")
    scaling = float(g["sp_scaling"][0])
    for name, k in (("sp256", 6), ("sp32", 4)):
        scores, bias = torch.from_numpy(g[f"{name}_scores"]), torch.from_numpy(g[f"{name}_bias"])
        for t in range(scores.shape[0]):
            ids, w = O.route_sqrt_softplus(scores[t], bias, k, scaling)
            assert np.array_equal(ids.numpy(), g[f"{name}_ids"][t])
            np.testing.assert_allclose(w.numpy(), g[f"{name}_w"][t], rtol=1e-6, atol=0)


def test_biased_softmax_router(golden_dir):
    # vectors made with the expressions of megabench/tasks/gptoss.py:106-109
    g = np.load(golden_dir / "routers.npz")
    for name, k in (("go32", 4), ("go128", 4)):
        logits, bias = torch.from_numpy(g[f"{name}_logits"]), torch.from_numpy(g[f"{name}_bias"])
        for t in range(logits.shape[0]):
            ids, w = O.route_softmax_biased(logits[t], bias, k)
            assert np.array_equal(ids.numpy(), g[f"{name}_ids"][t])
            np.testing.assert_allclose(w.numpy(), g[f"{name}_w"][t], rtol=1e-5, atol=1e-7)


def small_layers():
    return {
        "tiny": synthetic.GEOMETRIES["tiny"],
        "ds_small": dataclasses.replace(synthetic.GEOMETRIES["deepseek_v3"], name="ds_small", hidden=512, inter=256,
                                        experts=32, topk=4, n_group=4, topk_group=2),
        "qwen_small": dataclasses.replace(synthetic.GEOMETRIES["qwen3_30b_a3b"], name="qwen_small", hidden=256,
                                          inter=128, experts=8, topk=2),
    }


def spec_of(geo):
    return O.LayerSpec(geo.hidden, geo.inter, geo.experts, geo.topk, geo.shared, geo.scoring,
                       geo.n_group, geo.topk_group, geo.scaling)


def test_layer_matches_reference_composition(golden_dir):
    g = np.load(golden_dir / "layers.npz")
    for name, geo in small_layers().items():
        tokens, seed = int(g[f"{name}_geo"][7]), int(g[f"{name}_geo"][8])
        values = synthetic.make_inputs(geo, tokens, seed, "cpu")
        sums = np.array([float(values["x"].float().sum()), float(values["router"].sum()),
                         float(values["gate"].float().sum()), float(values["down_scale"].sum())])
        assert np.array_equal(sums, g[f"{name}_x_sum"]), "seeded generator changed"
        got = O.moe_layer(spec_of(geo), values)
        assert np.array_equal(got["expert_ids"].numpy(), g[f"{name}_ids"])
        assert np.array_equal(got["topk_weights"].numpy(), g[f"{name}_w"])
        assert np.array_equal(got["order"].numpy(), g[f"{name}_order"])
        assert np.array_equal(got["y"].view(torch.int16).numpy(), g[f"{name}_y"])
        wide = O.moe_layer(spec_of(geo), values, compute=torch.float32)
        assert np.array_equal(wide["y_fp32"].numpy(), g[f"{name}_y_fp32"])


def test_fp32_operand_convention_matches_frontier_linear(golden_dir):
    # the reference's second operand convention: megabench/tasks/frontier.py:180-186 (`linear`)
    g = np.load(golden_dir / "linears.npz")
    for name in ("a", "b", "ragged"):
        w = torch.from_numpy(g[f"{name}_w"].copy()).view(torch.float8_e4m3fn)
        ws = torch.from_numpy(g[f"{name}_ws"].copy())
        x = bf16(g[f"{name}_x"])
        xq, xs = O.quantize_activation(x)
        got = O.fp8_linear(xq, xs, w, ws, operands="fp32")
        assert np.array_equal(got.view(torch.int16).numpy(), g[f"{name}_y"]), name
        # the other convention rounds the operands first and is a different function
        other = O.fp8_linear(xq, xs, w, ws, operands="bf16")
        assert not torch.equal(other, got), name
    for name in ("tiny", "ds_small"):
        geo = small_layers()[name]
        tokens, seed = int(g[f"{name}_geo"][7]), int(g[f"{name}_geo"][8])
        values = synthetic.make_inputs(geo, tokens, seed, "cpu")
        got = O.moe_layer(spec_of(geo), values, operands="fp32")
        assert np.array_equal(got["expert_ids"].numpy(), g[f"{name}_layer_ids"])
        assert np.array_equal(got["y"].view(torch.int16).numpy(), g[f"{name}_layer_y"]), name


def test_block_matches_reference_composition(golden_dir):
    # RMSNorm (megabench/tasks/common.py:13-21) -> layer -> residual add (megabench/tasks/frontier.py:335-354)
    g = np.load(golden_dir / "blocks.npz")
    for name in ("ds_small", "qwen_small"):
        geo = small_layers()[name]
        tokens, seed, fp32_weight = (int(v) for v in g[f"{name}_geo"][7:10])
        values = synthetic.make_inputs(geo, tokens, seed, "cpu")
        values["x"] = torch.from_numpy(g[f"{name}_x"].copy()).view(torch.bfloat16)
        gamma = torch.from_numpy(g[f"{name}_gamma"].copy()).view(torch.bfloat16)
        got = O.moe_block(spec_of(geo), values, gamma, 1e-6, weight_in_fp32=bool(fp32_weight))
        assert np.array_equal(got["normalized"].view(torch.int16).numpy(), g[f"{name}_normalized"])
        assert np.array_equal(got["expert_ids"].numpy(), g[f"{name}_ids"])
        assert np.array_equal(got["order"].numpy(), g[f"{name}_order"])
        assert np.array_equal(got["x"].view(torch.int16).numpy(), g[f"{name}_x_out"])


def test_megamoe_swiglu_form(golden_dir):
    # megabench/tasks/megamoe.py:116-122 (clamp, routing weight inside SwiGLU) and :176-182 (plain sum)
    g = np.load(golden_dir / "megamoe_swiglu.npz")
    l1 = torch.from_numpy(g["l1"].copy()).view(torch.bfloat16)
    gate, up = l1.chunk(2, dim=-1)
    a = O._silu_mul_clamped(gate, up, 10.0, torch.from_numpy(g["w"]))
    assert np.array_equal(a.numpy(), g["a"])
    for name in ("ds_small", "qwen_small"):
        geo = dataclasses.replace(small_layers()[name], weight_std=0.2)
        tokens, seed = int(g[f"{name}_geo"][7]), int(g[f"{name}_geo"][8])
        values = synthetic.make_inputs(geo, tokens, seed, "cpu")
        spec = dataclasses.replace(spec_of(geo), swiglu_limit=1.0, weight_before_requant=True)
        got = O.moe_layer(spec, values)
        assert np.array_equal(got["expert_ids"].numpy(), g[f"{name}_ids"])
        assert np.array_equal(got["order"].numpy(), g[f"{name}_order"])
        assert np.array_equal(got["y"].view(torch.int16).numpy(), g[f"{name}_y"])


def test_mxfp4_packing(golden_dir):
    # megabench/tasks/quantization.py:13-51; the vectors hold exact ties and all-zero groups
    g = np.load(golden_dir / "megamoe_native.npz")
    blocks, scales = M.pack_mxfp4(torch.from_numpy(g["mx_in"]))
    assert np.array_equal(blocks.numpy(), g["mx_blocks"])
    assert np.array_equal(scales.numpy(), g["mx_scales"])
    back = M.unpack_mxfp4(torch.from_numpy(g["mx_blocks"]), torch.from_numpy(g["mx_scales"]))
    assert np.array_equal(back.numpy(), g["mx_back"])
    bad = torch.from_numpy(g["mx_scales"].copy())
    bad[0, 0] = 255                                   # the E8M0 NaN encoding
    assert torch.isnan(M.unpack_mxfp4(torch.from_numpy(g["mx_blocks"]), bad)[0, :32]).all()


def megamoe_native_inputs(g, name):
    keys = ("x", "x_scales", "topk_idx", "topk_weights", "l1_blocks", "l1_scales", "l2_blocks", "l2_scales")
    values = {k: torch.from_numpy(g[f"{name}_{k}"].copy()) for k in keys}
    values["x"] = values["x"].view(torch.float8_e4m3fn)
    return values


def test_megamoe_native_layer(golden_dir):
    # megabench/tasks/megamoe.py:131-182 with serial=True, on inputs from its own make_inputs
    g = np.load(golden_dir / "megamoe_native.npz")
    for name in ("dev", "wide"):
        tokens, experts, topk, hidden, inter, limit, _ = (int(v) for v in g[f"{name}_geo"])
        values = megamoe_native_inputs(g, name)
        assert values["l1_blocks"].shape == (experts, 2 * inter, hidden // 32, 16)
        assert values["x_scales"].shape == (tokens, hidden // 32)
        got = M.megamoe_layer(values, topk, float(limit))
        assert np.array_equal(got["y"].view(torch.int16).numpy(), g[f"{name}_y"])


def kimi_golden_case(g, name):
    """(values, normalized, topk) of a stored Kimi latent-MoE case."""
    bf = ("router", "latent_down", "latent_up", "latent_norm", "shared_gate", "shared_up", "shared_down")
    raw = ("router_bias", "gate_blocks", "gate_scales", "up_blocks", "up_scales", "down_blocks", "down_scales")
    values = {k: bf16(g[f"{name}_{k}"]) for k in bf}
    values.update({k: torch.from_numpy(g[f"{name}_{k}"].copy()) for k in raw})
    return values, bf16(g[f"{name}_normalized"]), int(g[f"{name}_geo"][2])


def test_kimi_latent_moe_block(golden_dir):
    # megabench/tasks/kimi_layer.py:189-230 (serial) and the situ activation of megabench/tasks/kimi.py:134-135
    g = np.load(golden_dir / "kimi_latent.npz")
    got = K.situ(bf16(g["situ_gate"]), bf16(g["situ_up"]))
    assert np.array_equal(got.view(torch.int16).numpy(), g["situ_out"])
    for name in ("small", "one"):
        values, normalized, topk = kimi_golden_case(g, name)
        out = K.latent_moe(values, normalized, topk)
        assert np.array_equal(out["sorted_ids"].numpy(), g[f"{name}_sorted_ids"])
        assert np.array_equal(out["y"].view(torch.int16).numpy(), g[f"{name}_y"]), name


def test_weight_generator_uses_the_reference_block_format():
    w = torch.randn((256, 384), generator=torch.Generator().manual_seed(2)) * 0.02
    q, s = synthetic.block_quantize_weight(w)
    q2, s2 = O.quantize_weight(w)
    assert torch.equal(q.view(torch.uint8), q2.view(torch.uint8)) and torch.equal(s, s2)


def test_margin_audit_flags_ties():
    geo = small_layers()["ds_small"]
    spec = spec_of(geo)
    x = torch.zeros((1, geo.hidden), dtype=torch.bfloat16)
    router = torch.zeros((geo.experts, geo.hidden))
    assert O.decision_margins(spec, x, router, torch.zeros(geo.experts)) == 0.0
    values = synthetic.make_inputs(geo, 6, 0, "cpu")
    assert O.decision_margins(spec, values["x"], values["router"], values["router_bias"]) > 0
