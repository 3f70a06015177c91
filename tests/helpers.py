"""Shared helpers of the parity tests: geometries, audited seeds, tolerances."""

from __future__ import annotations

import dataclasses

import torch

from oracle import moe_oracle as O
from vibe_megakernel_b200 import synthetic

# A routing decision is "safe" when every boundary gap, computed from fp64 logits, is far above
# the noise of an fp32 GEMV (about 1e-6 at these magnitudes).
MARGIN = 2e-5
# Layer output tolerance: max-abs 2e-2 where the oracle's output is at most 1 in magnitude, else
# 2e-2 of the oracle's largest magnitude (one bf16 ulp there), and cosine similarity above 0.999.
Y_ATOL = 2e-2
Y_COS = 0.999


def spec_of(geo) -> O.LayerSpec:
    return O.LayerSpec(geo.hidden, geo.inter, geo.experts, geo.topk, geo.shared, geo.scoring,
                       geo.n_group, geo.topk_group, geo.scaling)


def small_geometries():
    g = synthetic.GEOMETRIES
    return {
        "tiny": g["tiny"],
        "ds_small": dataclasses.replace(g["deepseek_v3"], name="ds_small", hidden=512, inter=256, experts=32, topk=4,
                                        n_group=4, topk_group=2),
        "qwen_small": dataclasses.replace(g["qwen3_30b_a3b"], name="qwen_small", hidden=256, inter=128, experts=8,
                                          topk=2),
        "kimi_small": dataclasses.replace(g["kimi_k2"], name="kimi_small", hidden=1024, inter=384, experts=48, topk=8,
                                          router_std=1024 ** -0.5),
        "mixtral_small": dataclasses.replace(g["mixtral_8x7b"], name="mixtral_small", hidden=512, inter=1792,
                                             experts=8, topk=2),
        # 66 K blocks in the down projection: the contraction is cut in three parts
        "long_k": dataclasses.replace(g["mixtral_8x7b"], name="long_k", hidden=256, inter=8448, experts=4, topk=2),
    }


def audited_inputs(geo, tokens: int, device="cpu", first_seed: int = 0, max_tries: int = 16):
    """Seeded inputs whose routing margins pass the audit; returns (values, seed)."""
    spec = spec_of(geo)
    for seed in range(first_seed, first_seed + max_tries):
        values = synthetic.make_inputs(geo, tokens, seed, device)
        if O.decision_margins(spec, values["x"], values["router"], values.get("router_bias")) >= MARGIN:
            return values, seed
    raise AssertionError("no seed passed the routing margin audit")


def audited_routing_inputs(geo, tokens: int, device="cpu", first_seed: int = 0, max_tries: int = 16):
    """Only x, router and bias (cheap at full geometry)."""
    spec = spec_of(geo)
    for seed in range(first_seed, first_seed + max_tries):
        x = synthetic.normal_rows(seed, "x", tokens, geo.hidden, 1.0, device).to(torch.bfloat16)
        router = synthetic.normal_rows(seed, "router", geo.experts, geo.hidden, geo.router_std, device)
        bias = synthetic.router_bias(geo, seed, device)
        if O.decision_margins(spec, x, router, bias) >= MARGIN:
            return x, router, bias, seed
    raise AssertionError("no seed passed the routing margin audit")


def to_device(values: dict, device) -> dict:
    return {k: v.to(device) for k, v in values.items()}


def y_error(got: torch.Tensor, want: torch.Tensor):
    g, w = got.double().flatten().cpu(), want.double().flatten().cpu()
    max_abs = float((g - w).abs().max())
    cos = float(torch.dot(g, w) / (g.norm() * w.norm() + 1e-300))
    bound = Y_ATOL * max(1.0, float(w.abs().max()))
    return max_abs, cos, bound


def assert_y_close(got: torch.Tensor, want: torch.Tensor, what: str = "y"):
    """The stated tolerance: max-abs 2e-2 * max(1, max|want|) and cosine > 0.999."""
    max_abs, cos, bound = y_error(got, want)
    assert max_abs <= bound and cos > Y_COS, f"{what}: max-abs {max_abs:.4g} (bound {bound:.4g}), cosine {cos:.6f}"
    return max_abs, cos


# The reference harness' own acceptance band (megabench/harness/correctness.py:64-85 with the
# defaults of megabench/cases.py:33-38 and the MoE-layer case's atol): the candidate's error
# against the fp32-widened oracle may reach noise_factor times the bf16 oracle's own error.
BAND_NOISE_FACTOR = 2.0
BAND_BF16_RTOL = 0.008
BAND_ATOL = 0.003


def assert_y_in_band(got: torch.Tensor, want: torch.Tensor, exact: torch.Tensor, what: str = "y"):
    """Tolerance at large output magnitudes (a bf16 ulp of the output alone exceeds 2e-2 there):
    cosine > 0.999 against the bf16 oracle and the reference harness' band against the fp32 oracle."""
    g, w, x = got.double().cpu(), want.double().cpu(), exact.double().cpu()
    err, ref_err = g - x, w - x
    scale = max(float(x.norm()), 1e-300)
    rel, ref_rel = float(err.norm()) / scale, float(ref_err.norm()) / scale
    peak, ref_peak = float(err.abs().max()), float(ref_err.abs().max())
    cos = float(torch.dot(g.flatten(), w.flatten()) / (g.norm() * w.norm() + 1e-300))
    ok = (cos > Y_COS and rel <= BAND_NOISE_FACTOR * ref_rel + BAND_BF16_RTOL
          and peak <= BAND_NOISE_FACTOR * ref_peak + BAND_ATOL + BAND_BF16_RTOL * float(x.abs().max()))
    detail = (f"{what}: cosine {cos:.6f}, rel-L2 {rel:.5f} (oracle's own {ref_rel:.5f}), max-abs {peak:.4g} "
              f"(oracle's own {ref_peak:.4g}), max-abs vs bf16 oracle {float((g - w).abs().max()):.4g}, "
              f"max|y| {float(x.abs().max()):.3g}")
    assert ok, detail
    return detail


def megamoe_inputs(tokens: int, experts: int, topk: int, hidden: int, inter: int, seed: int) -> dict:
    """Seeded inputs in the formats of megabench/tasks/megamoe.py:86-113 (CPU tensors): E4M3 rows with
    E8M0 scales per 32 channels, distinct experts per token, weights that sum to 2.5, MXFP4 expert
    matrices with linear1 outputs of standard deviation 4 so that some reach the clamp."""
    from oracle import megamoe_oracle as M
    gen = torch.Generator().manual_seed(seed)
    x, x_scales = O.quantize_activation(torch.randn((tokens, hidden), generator=gen), group=32, scale_format="e8m0")
    idx = torch.rand((tokens, experts), generator=gen).topk(topk, dim=-1).indices
    score = torch.nn.functional.softplus(torch.randn((tokens, topk), generator=gen)).sqrt()
    weights = score / score.sum(-1, keepdim=True) * 2.5
    l1 = torch.randn((experts, 2 * inter, hidden), generator=gen) * (4.0 / hidden ** 0.5)
    l2 = torch.randn((experts, hidden, inter), generator=gen) * inter ** -0.5
    l1_blocks, l1_scales = M.pack_mxfp4(l1)
    l2_blocks, l2_scales = M.pack_mxfp4(l2)
    return {"x": x, "x_scales": x_scales, "topk_idx": idx, "topk_weights": weights, "l1_blocks": l1_blocks,
            "l1_scales": l1_scales, "l2_blocks": l2_blocks, "l2_scales": l2_scales}
