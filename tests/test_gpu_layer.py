"""GPU parity of the whole layer (through the C ABI) against the oracle and the golden vectors."""

import dataclasses

import numpy as np
import pytest
import torch

from oracle import moe_oracle as O
from tests import helpers as H
from vibe_megakernel_b200 import synthetic

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def api():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from vibe_megakernel_b200 import layer
    return layer


def run_layer(api, geo, values_cpu, gemm="tcgen05"):
    tokens = values_cpu["x"].shape[0]
    layer = api.MoeLayer(api.LayerConfig.from_geometry(geo, gemm=gemm), max_tokens=tokens)
    values = H.to_device(values_cpu, "cuda")
    before = {k: v.clone() for k, v in values.items()}
    out = layer.forward(values, check_status=True)
    for k, v in values.items():
        assert torch.equal(v.view(torch.uint8), before[k].view(torch.uint8)), f"input {k} was modified"
    return layer, out


def check_against_oracle(api, geo, values, gemm):
    # every arm is held to the bf16-operand oracle (the graded convention); the tensor-core arithmetic
    # (exact FP8 products, fp32 scaling) must besides sit on the fp32-operand oracle, and the arm that
    # follows the bf16-operand rounding schedule on the bf16-operand one, both far inside the tolerance
    want = O.moe_layer(H.spec_of(geo), values, keep_intermediates=True)
    layer, out = run_layer(api, geo, values, gemm)
    tokens = values["x"].shape[0]
    assert torch.equal(out["expert_ids"].cpu(), want["expert_ids"])
    assert torch.equal(out["order"].cpu(), want["order"])
    torch.testing.assert_close(out["topk_weights"].cpu(), want["topk_weights"], rtol=2e-5, atol=1e-7)
    # grouped activation rows: the quantiser is bit-exact
    routed = tokens * geo.topk
    src = torch.div(want["order"], geo.topk, rounding_mode="floor")
    xq = layer.scratch(tokens, "xq").cpu()
    xs = layer.scratch(tokens, "xs").cpu()
    assert torch.equal(xq[:routed], want["xq"].view(torch.uint8)[src])
    assert torch.equal(xs[:routed], want["xs"][src])
    if geo.shared:
        assert torch.equal(xq[routed:], want["xq"].view(torch.uint8))
    # requantised SwiGLU output. The tensor cores multiply the exact e4m3 values, the oracle
    # multiplies operands rounded to bf16, so gate/up differ by about one bf16 ulp and a share of
    # the e4m3 codes (3 mantissa bits) lands one step away; the dequantised values stay close.
    aq = layer.scratch(tokens, "aq").cpu()
    a_s = layer.scratch(tokens, "as").cpu()
    start, num, den = 0, 0.0, 0.0
    for e, n in enumerate(want["counts"].tolist()):
        if n:
            ref_q, ref_s = want["requant"][e]
            ref = O.dequantize_activation(ref_q, ref_s).double()
            got = O.dequantize_activation(aq[start:start + n].view(torch.float8_e4m3fn), a_s[start:start + n]).double()
            num += float(((got - ref) ** 2).sum())
            den += float((ref ** 2).sum())
            torch.testing.assert_close(a_s[start:start + n], ref_s, rtol=0.04, atol=1e-9)
            start += n
    assert num <= (0.05 ** 2) * den, f"requantised SwiGLU output: relative L2 error {(num / max(den, 1e-300)) ** 0.5:.4f}"
    own = want["y"] if gemm == "simt_bf16" else O.moe_layer(H.spec_of(geo), values, operands="fp32")["y"]
    max_abs, cos, bound = H.y_error(out["y"], own)
    assert max_abs <= bound / 2 and cos > 0.9999, f"{gemm} against the oracle of its own operand convention: {max_abs:.4g}, {cos:.6f}"
    return H.assert_y_close(out["y"], want["y"])


@pytest.mark.parametrize("gemm", ["simt", "simt_bf16", "tcgen05"])
@pytest.mark.parametrize("name", ["tiny", "ds_small", "qwen_small", "kimi_small", "mixtral_small", "long_k"])
def test_small_layers_match_the_oracle(api, name, gemm):
    geo = H.small_geometries()[name]
    # (33 tokens: with top-2 the permutation kernel gets a row count that is no multiple of four)
    for tokens in (1, 4, 19, 33, 40):
        values, _ = H.audited_inputs(geo, tokens)
        check_against_oracle(api, geo, values, gemm)


def test_tiny_layer_matches_the_reference_vectors(api, golden_dir):
    g = np.load(golden_dir / "layers.npz")
    for name in ("tiny", "ds_small", "qwen_small"):
        geo = H.small_geometries()[name]
        tokens, seed = int(g[f"{name}_geo"][7]), int(g[f"{name}_geo"][8])
        values = synthetic.make_inputs(geo, tokens, seed, "cpu")
        _, out = run_layer(api, geo, values)
        assert np.array_equal(out["expert_ids"].cpu().numpy(), g[f"{name}_ids"])
        assert np.array_equal(out["order"].cpu().numpy(), g[f"{name}_order"])
        want = torch.from_numpy(g[f"{name}_y"].copy()).view(torch.bfloat16)
        H.assert_y_close(out["y"], want, name)


@pytest.mark.parametrize("gemm", ["simt", "tcgen05"])
def test_megamoe_swiglu_form(api, golden_dir, gemm):
    # clamp and routing weight inside SwiGLU, plain slot-order sum at the combine
    # (megabench/tasks/megamoe.py:116-122,176-182); vectors made by the reference's own swiglu()
    g = np.load(golden_dir / "megamoe_swiglu.npz")
    for name in ("ds_small", "qwen_small"):
        geo = dataclasses.replace(H.small_geometries()[name], weight_std=0.2)
        tokens, seed = int(g[f"{name}_geo"][7]), int(g[f"{name}_geo"][8])
        values = synthetic.make_inputs(geo, tokens, seed, "cpu")
        config = api.LayerConfig.from_geometry(geo, gemm=gemm, swiglu_limit=1.0, weight_before_requant=True)
        out = api.MoeLayer(config, max_tokens=tokens).forward(H.to_device(values, "cuda"), check_status=True)
        assert np.array_equal(out["expert_ids"].cpu().numpy(), g[f"{name}_ids"])
        assert np.array_equal(out["order"].cpu().numpy(), g[f"{name}_order"])
        H.assert_y_close(out["y"], torch.from_numpy(g[f"{name}_y"].copy()).view(torch.bfloat16), name)
        # each switch alone against the oracle, and both must change the result
        plain = api.MoeLayer(api.LayerConfig.from_geometry(geo, gemm=gemm), max_tokens=tokens).forward(
            H.to_device(values, "cuda"), check_status=True)
        for limit, early in ((1.0, False), (0.0, True), (0.73, True)):
            spec = dataclasses.replace(H.spec_of(geo), swiglu_limit=limit, weight_before_requant=early)
            want = O.moe_layer(spec, values)
            config = api.LayerConfig.from_geometry(geo, gemm=gemm, swiglu_limit=limit, weight_before_requant=early)
            got = api.MoeLayer(config, max_tokens=tokens).forward(H.to_device(values, "cuda"), check_status=True)
            H.assert_y_close(got["y"], want["y"], f"{name} limit {limit} early {early}")
            assert not torch.equal(got["y"], plain["y"])


def test_tensor_core_and_check_arm_agree(api):
    geo = H.small_geometries()["kimi_small"]
    values, _ = H.audited_inputs(geo, 40)
    _, a = run_layer(api, geo, values, "tcgen05")
    _, b = run_layer(api, geo, values, "simt")
    diff = (a["y"].float() - b["y"].float()).abs().max().item()
    assert diff <= 2 * 2e-2, diff


def test_run_twice_is_bit_identical_and_depends_on_every_input(api):
    geo = H.small_geometries()["ds_small"]
    values, _ = H.audited_inputs(geo, 19)
    layer, first = run_layer(api, geo, values)
    again = layer.forward(H.to_device(values, "cuda"), check_status=True)
    for k in first:
        assert torch.equal(first[k], again[k]), k
    for name in values:
        changed = {k: v.clone() for k, v in values.items()}
        t = changed[name]
        if t.dtype == torch.float8_e4m3fn:
            raw = t.view(torch.uint8)
            raw ^= 0x11                      # as megabench/verify_megamoe.py:112-115
        elif name == "router_bias":
            t += torch.linspace(-0.3, 0.3, t.numel())
        else:
            t *= 1.5
        other = layer.forward(H.to_device(changed, "cuda"), check_status=True)
        assert not torch.equal(first["y"], other["y"]), f"output ignores {name}"


@pytest.mark.parametrize("name,tokens", [("ds_small", 40), ("kimi_small", 7), ("mixtral_small", 130), ("long_k", 21),
                                         ("long_k", 5), ("ds_small", 16), ("tiny", 1)])
def test_gemm_handover_and_separate_kernels_agree(api, name, tokens):
    # Stage timing runs the two GEMMs strictly one after the other and the combine as a kernel of its
    # own; a plain call lets the down GEMM start on finished chunks of the gate/up GEMM and, up to 16
    # tokens, do the combine itself (the CTA that stores a token's last row). Same bits either way.
    geo = H.small_geometries()[name]
    values, _ = H.audited_inputs(geo, tokens)
    layer, plain = run_layer(api, geo, values)
    plain_launches = layer.launches()
    dev = H.to_device(values, "cuda")
    layer.profile(True)
    try:
        timed = layer.forward(dev, check_status=True)
        stages = layer.stage_ms()
    finally:
        layer.profile(False)
    assert set(stages) == set(layer.STAGES) and all(v >= 0 for v in stages.values())
    assert layer.launches() == 7 and plain_launches <= (6 if tokens <= 16 else 7)     # no combine launch up to 16 tokens
    for _ in range(3):
        again = layer.forward(dev, check_status=True)
        for k in plain:
            assert torch.equal(plain[k], timed[k]) and torch.equal(plain[k], again[k]), k


@pytest.mark.parametrize("name,tokens,fp32_weight", [("ds_small", 6, True), ("ds_small", 40, True), ("qwen_small", 5, False),
                                                     ("kimi_small", 33, True), ("mixtral_small", 1, False)])
def test_block_with_norm_and_residual(api, golden_dir, name, tokens, fp32_weight):
    # megabench/tasks/frontier.py:335-354: RMSNorm, the layer, the residual add
    geo = H.small_geometries()[name]
    gen = torch.Generator().manual_seed(77 + tokens)
    values = None
    for seed in range(1, 17):            # the router sees the normalised rows: audit those
        candidate = synthetic.make_inputs(geo, tokens, seed, "cpu")
        candidate["x"] = (torch.randn((tokens, geo.hidden), generator=gen) * 3).to(torch.bfloat16)
        gamma = (torch.randn((geo.hidden,), generator=gen) / 100 + 1).to(torch.bfloat16)
        normalized = O.rms_norm(candidate["x"], gamma, 1e-6, weight_in_fp32=fp32_weight)
        if O.decision_margins(H.spec_of(geo), normalized, candidate["router"], candidate.get("router_bias")) >= H.MARGIN:
            values = candidate
            break
    assert values is not None, "no seed passed the routing margin audit"
    want = O.moe_block(H.spec_of(geo), values, gamma, 1e-6, weight_in_fp32=fp32_weight)
    layer = api.MoeLayer(api.LayerConfig.from_geometry(geo), max_tokens=tokens)
    dev = H.to_device(values, "cuda")
    before = dev["x"].clone()
    out = layer.block_forward(dev, gamma.cuda(), 1e-6, weight_in_fp32=fp32_weight, check_status=True)
    assert torch.equal(dev["x"], before), "the residual stream was modified"
    assert torch.equal(out["expert_ids"].cpu(), want["expert_ids"])
    assert torch.equal(out["order"].cpu(), want["order"])
    # The layer's own tolerance (max-abs 2e-2 where max|y| <= 1) plus one bf16 step of the stream,
    # whose rounding after the add may fall the other way.
    def close(got_x, want_x, want_y, x_in):
        tol = 2e-2 * max(1.0, float(want_y.float().abs().max())) + float(x_in.float().abs().max()) * 2.0 ** -7
        assert float((got_x.float() - want_x.float()).abs().max()) <= tol
    close(out["x"].cpu(), want["x"], want["y"], values["x"])
    # golden vectors of the reference's own composition, where this case has them
    g = np.load(golden_dir / "blocks.npz")
    if f"{name}_geo" in g.files and int(g[f"{name}_geo"][7]) == tokens:
        pinned = synthetic.make_inputs(geo, tokens, int(g[f"{name}_geo"][8]), "cpu")
        pinned["x"] = torch.from_numpy(g[f"{name}_x"].copy()).view(torch.bfloat16)
        gamma_g = torch.from_numpy(g[f"{name}_gamma"].copy()).view(torch.bfloat16)
        got = layer.block_forward(H.to_device(pinned, "cuda"), gamma_g.cuda(), 1e-6, weight_in_fp32=fp32_weight,
                                  check_status=True)
        assert np.array_equal(got["expert_ids"].cpu().numpy(), g[f"{name}_ids"])
        assert np.array_equal(got["order"].cpu().numpy(), g[f"{name}_order"])
        want_x = torch.from_numpy(g[f"{name}_x_out"].copy()).view(torch.bfloat16)
        close(got["x"].cpu(), want_x, (want_x.float() - pinned["x"].float()), pinned["x"])


@pytest.mark.parametrize("name,tokens", [("ds_small", 3), ("kimi_small", 40)])
def test_layer_call_can_be_captured_in_a_cuda_graph(api, name, tokens):
    # A decode loop replays the layer from a CUDA graph: the call makes no allocation and no
    # synchronisation, its dependent launches become graph edges, and a replay on new token rows
    # (same buffers) gives the bits of a direct call.
    geo = H.small_geometries()[name]
    values, _ = H.audited_inputs(geo, tokens)
    other = dict(values)                        # other token rows, same weights (the graph holds their addresses)
    other["x"] = (torch.randn(values["x"].shape, generator=torch.Generator().manual_seed(5)) * 0.7).to(torch.bfloat16)
    layer, want = run_layer(api, geo, values)
    want_other = layer.forward(H.to_device(other, "cuda"), check_status=True)
    dev = H.to_device(values, "cuda")
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        layer.forward(dev)                       # warm-up on the capturing stream
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = layer.forward(dev)
    for inputs, expect in ((values, want), (other, want_other), (values, want)):
        dev["x"].copy_(inputs["x"])
        graph.replay()
        torch.cuda.synchronize()
        layer.check_device_status(tokens)
        for k in expect:
            assert torch.equal(out[k], expect[k]), k


def test_experts_with_no_rows_and_one_hot_routing(api):
    # a bias that sends every token to the same experts leaves all others empty
    geo = dataclasses.replace(H.small_geometries()["ds_small"], n_group=1, topk_group=1)
    values, _ = H.audited_inputs(geo, 40)
    values["router_bias"] = torch.zeros(geo.experts)
    values["router_bias"][[3, 7, 8, 30]] = torch.tensor([4.0, 3.0, 2.0, 1.0])
    want = O.moe_layer(H.spec_of(geo), values)
    assert want["expert_ids"].tolist() == [[3, 7, 8, 30]] * 40
    _, out = run_layer(api, geo, values)
    assert torch.equal(out["expert_ids"].cpu(), want["expert_ids"])
    assert torch.equal(out["order"].cpu(), want["order"])
    H.assert_y_close(out["y"], want["y"])


def test_bad_arguments_are_refused(api):
    geo = H.small_geometries()["tiny"]
    values, _ = H.audited_inputs(geo, 4)
    layer = api.MoeLayer(api.LayerConfig.from_geometry(geo), max_tokens=4)
    dev = H.to_device(values, "cuda")
    with pytest.raises(TypeError):
        layer.forward(dev | {"x": dev["x"].float()})
    with pytest.raises(ValueError):
        layer.forward(dev | {"gate": dev["gate"][:, :, :-128].contiguous()})
    with pytest.raises(ValueError):
        layer.forward(dev | {"x": values["x"]})
    from vibe_megakernel_b200 import _cabi
    with pytest.raises(_cabi.MoeError):
        api.MoeLayer(api.LayerConfig(hidden=100, inter=128, experts=8, topk=2), max_tokens=1)


@pytest.mark.parametrize("name,tokens", [("qwen_small", 300), ("mixtral_small", 257), ("ds_small", 128),
                                         ("mixtral_small", 600), ("long_k", 300), ("qwen_small", 1000)])
def test_experts_with_more_rows_than_one_tile(api, name, tokens):
    # several chunks per expert and channel tile (a split contraction in long_k)
    geo = H.small_geometries()[name]
    values, _ = H.audited_inputs(geo, tokens, max_tries=64)
    check_against_oracle(api, geo, values, "tcgen05")
    if tokens >= 600:
        check_against_oracle(api, geo, values, "simt")
        # a row's result does not depend on the tile it was multiplied in: the same tokens, fewer at a time
        full = api.MoeLayer(api.LayerConfig.from_geometry(geo), max_tokens=tokens).forward(H.to_device(values, "cuda"))
        few = dict(values)
        few["x"] = values["x"][:40].contiguous()
        part = api.MoeLayer(api.LayerConfig.from_geometry(geo), max_tokens=40).forward(H.to_device(few, "cuda"))
        assert torch.equal(part["y"], full["y"][:40])


@pytest.mark.parametrize("name,tokens,megamoe_form", [("mixtral_small", 600, False), ("long_k", 300, False),
                                                      ("mixtral_small", 600, True)])
def test_rows_on_the_mma_m_side_give_the_bits_of_the_decode_kernel(api, name, tokens, megamoe_form):
    # With more than 64 rows per expert in sight the tensor-core path multiplies 128-row tiles with the
    # tokens on the MMA's M side (another kernel, another epilogue, divisions without the library's
    # slow path). The same tokens forty at a time meet the decode kernel (16-token tiles, weights on
    # M): every row must come out bit-identical (long_k: a contraction summed in parts).
    # megamoe_form: the clamp and the routing weight inside SwiGLU (megabench/tasks/megamoe.py:116-122), which
    # the 128-row gate/up kernel applies in its closing warps
    geo = H.small_geometries()[name]
    values, _ = H.audited_inputs(geo, tokens, max_tries=64)
    dev = H.to_device(values, "cuda")
    form = dict(swiglu_limit=1.0, weight_before_requant=True) if megamoe_form else {}
    wide = api.MoeLayer(api.LayerConfig.from_geometry(geo, **form), max_tokens=tokens)
    assert wide.workspace(tokens)[1].token_tile == 128
    full = wide.forward(dev, check_status=True)
    small = api.MoeLayer(api.LayerConfig.from_geometry(geo, **form), max_tokens=40)
    assert small.workspace(40)[1].token_tile <= 64
    for lo in range(0, tokens, 40):
        few = dict(dev)
        few["x"] = dev["x"][lo:lo + 40].contiguous()
        part = small.forward(few, check_status=True)
        assert torch.equal(part["expert_ids"], full["expert_ids"][lo:lo + 40])
        assert torch.equal(part["y"], full["y"][lo:lo + 40]), lo


def test_quantising_from_the_token_side_leaves_the_bytes_of_the_gathering_kernel(api):
    # From 8,192 (token, group of 128 channels) pairs on, a layer call quantises each token once and
    # stores the bytes and scales to all of its grouped rows (found through the inverse of the
    # permutation), instead of gathering and quantising every grouped row. The grouped rows left in the
    # workspace must be, byte for byte, what the gathering kernel makes of the same permutation.
    geo = H.small_geometries()["kimi_small"]
    tokens = 1100                                   # x 8 groups of 128 channels
    values = synthetic.make_inputs(geo, tokens, 0, "cpu")    # (not audited: nothing here is compared with the oracle)
    dev = H.to_device(values, "cuda")
    layer = api.MoeLayer(api.LayerConfig.from_geometry(geo), max_tokens=tokens)
    out = layer.forward(dev, check_status=True)
    ws, lay = layer.workspace(tokens)
    rows, groups = int(lay.rows), geo.hidden // 128
    assert rows == tokens * (geo.topk + 1)
    row_token = ws[int(lay.row_token):int(lay.row_token) + 4 * rows].view(torch.int32).clone()
    assert torch.equal(torch.bincount(row_token[:tokens * geo.topk].long(), minlength=tokens),
                       torch.full((tokens,), geo.topk, device="cuda"))
    assert torch.equal(row_token[tokens * geo.topk:], torch.arange(tokens, dtype=torch.int32, device="cuda"))
    xq = ws[int(lay.xq):int(lay.xq) + rows * geo.hidden].view(rows, geo.hidden)
    xs = ws[int(lay.xs):int(lay.xs) + 4 * rows * groups].view(torch.float32).view(rows, groups)
    q, s = api.quantize_rows(dev["x"], gather=row_token)
    assert torch.equal(q.view(torch.uint8), xq)
    assert torch.equal(s, xs)
    # and the call's result is that of the same tokens sixty-four at a time (the small-batch kernels)
    small = api.MoeLayer(api.LayerConfig.from_geometry(geo), max_tokens=64)
    for lo in range(0, tokens, 64):
        few = dict(dev)
        few["x"] = dev["x"][lo:lo + 64].contiguous()
        part = small.forward(few, check_status=True)
        assert torch.equal(part["expert_ids"], out["expert_ids"][lo:lo + 64])
        assert torch.equal(part["y"], out["y"][lo:lo + 64]), lo
