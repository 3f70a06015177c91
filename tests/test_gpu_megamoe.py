"""GPU parity of the routed experts in the MegaMoE-native formats (MXFP4 weights, E4M3 rows, E8M0
scales per 32 channels) through the C ABI, against the oracle and the reference's vectors."""

import pytest
import torch

from oracle import megamoe_oracle as M
from tests import helpers as H

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def api():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from vibe_megakernel_b200 import megamoe
    return megamoe


CASES = {
    # tokens, experts, topk, hidden, inter, limit
    "reference_development": (8, 16, 4, 256, 128, 10.0),       # megabench/verify_megamoe.py:32
    "one_token": (1, 16, 4, 256, 128, 10.0),
    "two_chunks_per_expert": (70, 8, 2, 512, 256, 10.0),       # 17.5 rows per expert on tiles of 32
    "ragged_scale_rows": (200, 4, 2, 384, 640, 3.0),           # 3 and 5 K blocks: scale rows of 12 and 20 bytes; tiles of 64
    "idle_experts": (3, 64, 2, 256, 256, 0.0),                 # most experts get no row; no clamp
    "catalog_width": (3, 2, 2, 7168, 3072, 10.0),              # megabench/cases.py:384-385: 56 and 24 K blocks per row
    "rows_on_m": (300, 4, 2, 512, 256, 10.0),                  # 150 rows per expert: 128-row tiles, tokens on the MMA's M side
    "rows_on_m_ragged": (520, 2, 2, 768, 640, 3.0),            # 520 rows per expert (4 full tiles + 8 rows), 6 and 5 K blocks
}


@pytest.mark.parametrize("name", list(CASES))
def test_matches_the_oracle(api, name):
    tokens, experts, topk, hidden, inter, limit = CASES[name]
    values = H.megamoe_inputs(tokens, experts, topk, hidden, inter, seed=len(name))
    want = M.megamoe_layer(values, topk, limit)
    layer = api.MegaMoe(api.MegaMoeConfig(hidden, inter, experts, topk, limit), max_tokens=tokens)
    device = H.to_device(values, "cuda")
    before = {k: v.clone() for k, v in device.items()}
    got = layer.run(device, check_status=True, want_order=True)
    for k, v in device.items():
        assert torch.equal(v.view(torch.uint8), before[k].view(torch.uint8)), f"input {k} was modified"
    assert torch.equal(got["order"].cpu(), want["order"])
    H.assert_y_close(got["y"], want["y"], name)
    again = layer.run(device, check_status=True)
    assert torch.equal(again["y"], got["y"])


def test_a_row_with_an_expert_id_out_of_range_is_dropped(api):
    # the header documents such a row as skipped: it must not be gathered (its source index was never
    # written), the other tokens keep their bits, and the unused tail of `order` reads -1
    tokens, experts, topk, hidden, inter, limit = CASES["reference_development"]
    values = H.to_device(H.megamoe_inputs(tokens, experts, topk, hidden, inter, seed=9), "cuda")
    layer = api.MegaMoe(api.MegaMoeConfig(hidden, inter, experts, topk, limit), max_tokens=tokens)
    layer.workspace.zero_()                  # every index a kernel could read is then in range
    base = layer.run(values, check_status=True, want_order=True)
    bad = dict(values)
    bad["topk_idx"] = values["topk_idx"].clone()
    bad["topk_idx"][2, 1] = -1
    bad["topk_idx"][5, 0] = experts
    layer.workspace.zero_()
    got = layer.run(bad, check_status=True, want_order=True)
    others = [t for t in range(tokens) if t not in (2, 5)]
    assert torch.equal(got["y"][others], base["y"][others])
    flat = bad["topk_idx"].flatten().cpu()
    kept = ((flat >= 0) & (flat < experts)).nonzero().flatten()
    want_order = kept[torch.sort(flat[kept], stable=True).indices]
    assert torch.equal(got["order"].cpu()[: kept.numel()], want_order)
    assert got["order"].cpu()[kept.numel():].tolist() == [-1, -1]


def test_catalog_geometry_matches_the_oracle(api):
    # 384 experts, top-6, hidden 7168, intermediate 3072 (megabench/cases.py:380-388) at 64 tokens, every
    # expert on this GPU; inputs are random codes made on the device and the oracle runs on CUDA tensors
    from vibe_megakernel_b200 import synthetic
    tokens, experts, topk, hidden, inter, limit = 64, 384, 6, 7168, 3072, 10.0
    values = synthetic.megamoe_inputs(tokens, experts, topk, hidden, inter, 0, "cuda")
    want = M.megamoe_layer(values, topk, limit)
    layer = api.MegaMoe(api.MegaMoeConfig(hidden, inter, experts, topk, limit), max_tokens=tokens)
    got = layer.run(values, check_status=True, want_order=True)
    assert torch.equal(got["order"], want["order"])
    max_abs, cos = H.assert_y_close(got["y"], want["y"], "catalog geometry")
    print(f"MXFP4 catalog geometry, 64 tokens: max-abs {max_abs:.4g}, cosine {cos:.6f}, "
          f"{int((got['y'] != want['y']).sum())} of {got['y'].numel()} values differ")


def test_depends_on_every_input(api):
    tokens, experts, topk, hidden, inter, limit = CASES["reference_development"]
    values = H.megamoe_inputs(tokens, experts, topk, hidden, inter, seed=5)
    layer = api.MegaMoe(api.MegaMoeConfig(hidden, inter, experts, topk, limit), max_tokens=tokens)
    base = layer.run(H.to_device(values, "cuda"), check_status=True)["y"]
    # megabench/tests/test_megamoe.py:113-117
    changes = {"x_scales": values["x_scales"] + 1, "l1_blocks": values["l1_blocks"] ^ 0x11,
               "l2_scales": values["l2_scales"] - 1, "topk_weights": values["topk_weights"] * 0.5,
               "topk_idx": (values["topk_idx"] + 1) % experts}
    for key, changed in changes.items():
        other = dict(values)
        other[key] = changed
        got = layer.run(H.to_device(other, "cuda"), check_status=True)["y"]
        assert not torch.equal(got, base), key
        H.assert_y_close(got, M.megamoe_layer(other, topk, limit)["y"], key)


def test_bad_arguments_are_refused(api):
    with pytest.raises(Exception):
        api.MegaMoe(api.MegaMoeConfig(250, 128, 16, 4), max_tokens=4)        # hidden must be a multiple of 128
    with pytest.raises(Exception):
        api.MegaMoe(api.MegaMoeConfig(256, 128, 16, 4), max_tokens=10000)    # more than 32768 routed rows
    layer = api.MegaMoe(api.MegaMoeConfig(256, 128, 16, 4), max_tokens=4)
    values = H.to_device(H.megamoe_inputs(4, 16, 4, 256, 128, seed=1), "cuda")
    values["x_scales"] = values["x_scales"].float()
    with pytest.raises(TypeError):
        layer.run(values)


def test_call_can_be_captured_in_a_cuda_graph(api):
    # no allocation and no synchronisation inside the call: a replay on other token rows and another
    # routing (same buffers) gives the bits of a direct call
    tokens, experts, topk, hidden, inter, limit = CASES["two_chunks_per_expert"]
    values = H.megamoe_inputs(tokens, experts, topk, hidden, inter, seed=21)
    other = dict(values)
    for key in ("x", "x_scales", "topk_idx", "topk_weights"):
        other[key] = H.megamoe_inputs(tokens, experts, topk, hidden, inter, seed=22)[key]
    layer = api.MegaMoe(api.MegaMoeConfig(hidden, inter, experts, topk, limit), max_tokens=tokens)
    want = layer.run(H.to_device(values, "cuda"), check_status=True)["y"].clone()
    want_other = layer.run(H.to_device(other, "cuda"), check_status=True)["y"].clone()
    assert not torch.equal(want, want_other)
    dev = H.to_device(values, "cuda")
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        layer.run(dev)                           # warm-up on the capturing stream
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = layer.run(dev)["y"]
    for inputs, expect in ((values, want), (other, want_other), (values, want)):
        for key in ("x", "x_scales", "topk_idx", "topk_weights"):
            dev[key].view(torch.uint8).copy_(inputs[key].view(torch.uint8))
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, expect)


@pytest.mark.parametrize("name", ["rows_on_m", "rows_on_m_ragged"])
def test_rows_on_the_mma_m_side_give_the_bits_of_the_other_kernel(api, name):
    # more than 64 rows per expert in sight: 128-row tiles with the tokens on M (gemm_mx_wide.cu). The same
    # tokens sixteen at a time meet the kernel with the weights on M: every row must be bit-identical.
    tokens, experts, topk, hidden, inter, limit = CASES[name]
    values = H.to_device(H.megamoe_inputs(tokens, experts, topk, hidden, inter, seed=len(name)), "cuda")
    wide = api.MegaMoe(api.MegaMoeConfig(hidden, inter, experts, topk, limit), max_tokens=tokens)
    full = wide.run(values, check_status=True)
    small = api.MegaMoe(api.MegaMoeConfig(hidden, inter, experts, topk, limit), max_tokens=16)
    per_token = [k for k, v in values.items() if v.shape[0] == tokens]
    assert "x" in per_token or len(per_token) >= 2
    for lo in range(0, tokens, 16):
        few = dict(values)
        for k in per_token:
            few[k] = values[k][lo:lo + 16].contiguous()
        part = small.run(few, check_status=True)
        assert torch.equal(part["y"], full["y"][lo:lo + 16]), lo
