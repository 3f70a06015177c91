"""GPU parity of the Kimi-K3 latent MoE block (through the C ABI) against the oracle and the
reference's own vectors (megabench/tasks/kimi_layer.py:189-230, serial form)."""

import numpy as np
import pytest
import torch

from oracle import kimi_oracle as K
from oracle import moe_oracle as O
from tests import helpers as H
from tests.test_oracle_golden import kimi_golden_case
from vibe_megakernel_b200 import synthetic

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def api():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from vibe_megakernel_b200 import kimi_latent
    return kimi_latent


def audited(tokens, experts, topk, hidden, latent, inter, shared, device, first_seed=0):
    """Inputs whose routing decisions all have an fp64 margin far above the error of an fp32 logit."""
    spec = O.LayerSpec(hidden, inter, experts, topk, 0, "sigmoid", 1, 1, 1.0)
    for seed in range(first_seed, first_seed + 16):
        values, normalized = synthetic.kimi_latent_inputs(tokens, experts, topk, hidden, latent, inter, shared, seed, device)
        if O.decision_margins(spec, normalized, values["router"].float(), values["router_bias"]) >= H.MARGIN:
            return values, normalized, seed
    raise AssertionError("no seed passed the routing margin audit")


def test_matches_the_reference_vectors(api, golden_dir):
    g = np.load(golden_dir / "kimi_latent.npz")
    for name in ("small", "one"):
        values, normalized, topk = kimi_golden_case(g, name)
        tokens, experts, _, hidden, latent, inter, shared, _ = (int(v) for v in g[f"{name}_geo"])
        layer = api.LatentMoe(api.LatentMoeConfig(hidden, latent, inter, experts, topk, shared), max_tokens=tokens)
        dev = H.to_device(values, "cuda")
        before = {k: v.clone() for k, v in dev.items()}
        out = layer.forward(dev, normalized.cuda(), check_status=True)
        for k, v in dev.items():
            assert torch.equal(v.view(torch.uint8), before[k].view(torch.uint8)), f"input {k} was modified"
        assert np.array_equal(out["sorted_ids"].cpu().numpy(), g[f"{name}_sorted_ids"])
        want = torch.from_numpy(g[f"{name}_y"].copy()).view(torch.bfloat16)
        max_abs, cos = H.assert_y_close(out["y"], want, name)
        print(f"kimi latent {name}: max-abs {max_abs:.4g}, cosine {cos:.6f}, "
              f"{int((out['y'].cpu() != want).sum())} of {want.numel()} values differ")


@pytest.mark.parametrize("tokens,experts,topk,hidden,latent,inter,shared", [
    (1, 16, 4, 256, 128, 128, 1), (8, 48, 8, 512, 384, 256, 2), (19, 24, 6, 384, 256, 640, 2), (70, 8, 2, 256, 128, 128, 1)])
def test_matches_the_oracle(api, tokens, experts, topk, hidden, latent, inter, shared):
    values, normalized, seed = audited(tokens, experts, topk, hidden, latent, inter, shared, "cpu")
    want = K.latent_moe(values, normalized, topk)
    layer = api.LatentMoe(api.LatentMoeConfig(hidden, latent, inter, experts, topk, shared), max_tokens=tokens)
    out = layer.forward(H.to_device(values, "cuda"), normalized.cuda(), check_status=True)
    assert torch.equal(out["expert_ids"].cpu(), want["expert_ids"]), f"seed {seed}"
    assert torch.equal(out["sorted_ids"].cpu(), want["sorted_ids"])
    torch.testing.assert_close(out["topk_weights"].cpu(), want["topk_weights"], rtol=2e-5, atol=1e-7)
    H.assert_y_close(out["y"], want["y"], f"{tokens} tokens")
    again = layer.forward(H.to_device(values, "cuda"), normalized.cuda(), check_status=True)
    assert torch.equal(again["y"], out["y"])
    # a token's result does not depend on the batch it arrives in
    alone = layer.forward(H.to_device(values, "cuda"), normalized[tokens - 1:].cuda().contiguous(), check_status=True)
    assert torch.equal(alone["y"][0], out["y"][tokens - 1])


def test_catalog_geometry_matches_the_oracle(api):
    # megabench/cases.py:315-324: 896 experts, top-16, hidden 7168, latent 3584, intermediate 3072, two shared
    # experts, 8 sequences per rank; every expert on this GPU, the oracle on CUDA tensors
    tokens, experts, topk, hidden, latent, inter, shared = 8, 896, 16, 7168, 3584, 3072, 2
    values, normalized, seed = audited(tokens, experts, topk, hidden, latent, inter, shared, "cuda")
    want = K.latent_moe(values, normalized, topk)
    layer = api.LatentMoe(api.LatentMoeConfig(hidden, latent, inter, experts, topk, shared), max_tokens=tokens)
    out = layer.forward(values, normalized, check_status=True)
    assert torch.equal(out["expert_ids"], want["expert_ids"]), f"seed {seed}"
    max_abs, cos = H.assert_y_close(out["y"], want["y"], "catalog geometry")
    print(f"kimi latent catalog geometry: max|y| {float(want['y'].float().abs().max()):.3g}, max-abs {max_abs:.4g}, cosine "
          f"{cos:.6f}, {int((out['y'] != want['y']).sum())} of {want['y'].numel()} values differ, {layer.launches()} launches")


def test_bad_arguments_are_refused(api):
    from vibe_megakernel_b200 import _cabi
    with pytest.raises(_cabi.MoeError):
        api.LatentMoe(api.LatentMoeConfig(250, 128, 128, 16, 4), max_tokens=4)       # hidden must be a multiple of 128
    with pytest.raises(_cabi.MoeError):
        api.LatentMoe(api.LatentMoeConfig(256, 128, 128, 16, 4), max_tokens=5000)    # more than 16384 routed rows
    values, normalized = synthetic.kimi_latent_inputs(4, 16, 4, 256, 128, 128, 1, 0, "cuda")
    layer = api.LatentMoe(api.LatentMoeConfig(256, 128, 128, 16, 4, 1), max_tokens=4)
    with pytest.raises(TypeError):
        layer.forward(values, normalized.float())
    with pytest.raises(ValueError):
        layer.forward(values | {"latent_up": values["latent_up"][:, :-32].contiguous()}, normalized)
