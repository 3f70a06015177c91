"""GPU parity of the single stages (through the C ABI) against the oracle and the golden vectors."""

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


def bf16(bits):
    return torch.from_numpy(bits.copy()).view(torch.bfloat16)


# ---------------------------------------------------------------- quantiser
def test_quantiser_matches_reference_vectors(api, golden_dir):
    g = np.load(golden_dir / "quantizers.npz")
    for key_in, key_q, key_s, as_bf16 in (("w_in", "wa_q_0", "wa_s_0", True), ("a_in", "a_q_0", "a_s_0", True),
                                          ("e_in", "ef_q", "ef_s", False), ("f_in", "f_q", "f_s", False)):
        x = bf16(g[key_in]) if as_bf16 else torch.from_numpy(g[key_in])
        q, s = api.quantize_rows(x.cuda().contiguous())
        assert np.array_equal(q.view(torch.uint8).cpu().numpy(), g[key_q]), key_in
        assert np.array_equal(s.cpu().numpy(), g[key_s]), key_in


@pytest.mark.parametrize("rows,width,dtype", [(1, 128, torch.bfloat16), (7, 7168, torch.bfloat16),
                                              (33, 2048, torch.float32), (5, 259, torch.float32),
                                              (3, 1, torch.bfloat16), (130, 384, torch.bfloat16)])
def test_quantiser_matches_oracle(api, rows, width, dtype):
    gen = torch.Generator().manual_seed(rows * 1000 + width)
    x = (torch.randn((rows, width), generator=gen) * torch.logspace(-5, 2, rows)[:, None]).to(dtype)
    x[0, : min(width, 4)] = 0
    q, s = api.quantize_rows(x.cuda())
    wq, ws = O.quantize_activation(x)
    assert torch.equal(q.view(torch.uint8).cpu(), wq.view(torch.uint8))
    assert torch.equal(s.cpu(), ws)


def test_quantiser_gather(api):
    x = torch.randn((9, 512), generator=torch.Generator().manual_seed(4)).to(torch.bfloat16)
    idx = torch.tensor([8, 0, 0, 3, 5, 5, 5, 1], dtype=torch.int32)
    q, s = api.quantize_rows(x.cuda(), idx.cuda())
    wq, ws = O.quantize_activation(x[idx.long()])
    assert torch.equal(q.view(torch.uint8).cpu(), wq.view(torch.uint8)) and torch.equal(s.cpu(), ws)


# ---------------------------------------------------------------- permutation
@pytest.mark.parametrize("n,experts,kind", [(32, 16, "random"), (1024, 256, "random"), (8192, 384, "random"),
                                            (4096, 8, "random"), (64, 16, "one"), (8, 256, "random"),
                                            (513, 128, "skew"), (1, 4, "random")])
def test_grouping_is_the_stable_sort(api, n, experts, kind):
    gen = torch.Generator().manual_seed(n + experts)
    if kind == "random":
        ids = torch.randint(0, experts, (n,), generator=gen)
    elif kind == "one":
        ids = torch.full((n,), 5, dtype=torch.int64)
    else:
        ids = (torch.rand((n,), generator=gen) ** 4 * experts).long().clamp(max=experts - 1)
    order, counts = api.group_rows(ids.cuda(), experts)
    want_order, want_counts = O.expert_order(ids, experts)
    assert torch.equal(order.cpu(), want_order)
    assert torch.equal(counts.cpu().long(), want_counts)


def test_grouping_keeps_only_local_experts(api):
    gen = torch.Generator().manual_seed(9)
    ids = torch.randint(0, 64, (500,), generator=gen)
    order, counts = api.group_rows(ids.cuda(), 16, id_base=32)     # experts 32..47 live here
    mine = ((ids >= 32) & (ids < 48)).nonzero().flatten()
    want = mine[torch.sort(ids[mine], stable=True).indices]
    assert torch.equal(order.cpu()[: want.numel()], want)
    assert bool((order.cpu()[want.numel():] == -1).all())
    assert torch.equal(counts.cpu().long(), torch.bincount(ids[mine] - 32, minlength=16))


# ---------------------------------------------------------------- router
@pytest.mark.parametrize("name,tokens", [("tiny", 4), ("deepseek_v3", 1), ("deepseek_v3", 64), ("deepseek_v3", 128),
                                         ("kimi_k2", 64), ("qwen3_30b_a3b", 37), ("mixtral_8x7b", 16)])
def test_router_ids_are_bit_exact(api, name, tokens):
    geo = synthetic.GEOMETRIES[name]
    x, router, bias, seed = H.audited_routing_inputs(geo, tokens)
    layer = api.MoeLayer(api.LayerConfig.from_geometry(geo), max_tokens=tokens)
    ids, w = layer.route(x.cuda(), router.cuda(), None if bias is None else bias.cuda())
    want_ids, want_w = O.route_tokens(H.spec_of(geo), x, router, bias)
    assert torch.equal(ids.cpu(), want_ids), f"seed {seed}"
    torch.testing.assert_close(w.cpu(), want_w, rtol=2e-5, atol=1e-7)


@pytest.mark.parametrize("scoring,experts,topk,tokens", [("sqrt_softplus", 256, 6, 1), ("sqrt_softplus", 256, 6, 40),
                                                          ("sqrt_softplus", 48, 8, 19), ("softmax_biased", 128, 4, 1),
                                                          ("softmax_biased", 32, 4, 33), ("softmax_biased", 40, 4, 70)])
def test_other_router_scorings(api, scoring, experts, topk, tokens):
    # sqrt-softplus scores with a selection bias (megabench/tasks/dsv41.py:622-626) and the softmax
    # router with a linear bias (megabench/tasks/gptoss.py:106-109): ids bit-exact, weights to 2e-5
    geo = dataclasses.replace(synthetic.GEOMETRIES["qwen3_30b_a3b"], name=scoring, hidden=512, inter=128,
                              experts=experts, topk=topk, scoring=scoring, scaling=1.5, bias_kind="normal",
                              bias_std=0.05 if scoring == "sqrt_softplus" else 0.3, router_std=0.05)
    x, router, bias, seed = H.audited_routing_inputs(geo, tokens)
    layer = api.MoeLayer(api.LayerConfig.from_geometry(geo), max_tokens=tokens)
    ids, w = layer.route(x.cuda(), router.cuda(), bias.cuda())
    want_ids, want_w = O.route_tokens(H.spec_of(geo), x, router, bias)
    assert torch.equal(ids.cpu(), want_ids), f"seed {seed}"
    torch.testing.assert_close(w.cpu(), want_w, rtol=2e-5, atol=1e-7)


def test_other_router_scorings_through_the_layer(api):
    for scoring in ("sqrt_softplus", "softmax_biased"):
        geo = dataclasses.replace(H.small_geometries()["kimi_small"], name=scoring, scoring=scoring, scaling=1.5,
                                  bias_kind="normal", bias_std=0.05)
        for tokens in (3, 40):
            values, _ = H.audited_inputs(geo, tokens)
            want = O.moe_layer(H.spec_of(geo), values)
            layer = api.MoeLayer(api.LayerConfig.from_geometry(geo), max_tokens=tokens)
            out = layer.forward(H.to_device(values, "cuda"), check_status=True)
            assert torch.equal(out["expert_ids"].cpu(), want["expert_ids"])
            assert torch.equal(out["order"].cpu(), want["order"])
            H.assert_y_close(out["y"], want["y"], scoring)


def test_router_ties_go_to_the_lower_index(api):
    # all-zero logits: megabench/tests/test_frontier.py:297-299 expects ids [0, 1], weights 1.25
    cfg = api.LayerConfig(hidden=128, inter=128, experts=8, topk=2, shared=0, scoring="sigmoid", n_group=2,
                          topk_group=1, scaling=2.5)
    layer = api.MoeLayer(cfg, max_tokens=3)
    x = torch.zeros((3, 128), dtype=torch.bfloat16, device="cuda")
    router = torch.zeros((8, 128), device="cuda")
    ids, w = layer.route(x, router, torch.zeros(8, device="cuda"))
    assert ids.cpu().tolist() == [[0, 1]] * 3
    assert w.cpu().tolist() == [[1.25, 1.25]] * 3
    cfg = api.LayerConfig(hidden=128, inter=128, experts=8, topk=3, shared=0, scoring="softmax")
    ids, w = api.MoeLayer(cfg, max_tokens=3).route(x, router, None)
    assert ids.cpu().tolist() == [[0, 1, 2]] * 3


def test_router_near_ties_follow_the_exact_order_down_to_the_logit_error(api):
    # Two experts whose logits differ by a chosen gap: expert 9's router row is expert 3's plus a
    # multiple of one basis vector, so the gap is delta * x[k] exactly. The kernel's logit error is
    # about 1e-7, so a gap of 1e-6 and more must be decided as exact arithmetic decides it; at an
    # exact tie the lower index wins; below the error either of the two may come first, nothing else.
    geo = dataclasses.replace(synthetic.GEOMETRIES["qwen3_30b_a3b"], name="near_tie", hidden=2048, experts=32, topk=2,
                              router_std=0.01)
    layer = api.MoeLayer(api.LayerConfig.from_geometry(geo), max_tokens=1)
    gen = torch.Generator().manual_seed(17)
    x = torch.randn((1, geo.hidden), generator=gen).to(torch.bfloat16)
    k = int(x[0].float().abs().argmax())
    base = torch.randn((geo.experts, geo.hidden), generator=gen) * geo.router_std
    base[3] += 0.3 * x[0].float() / x[0].float().norm()        # experts 3 and 9 lead the field by a wide margin
    base[3, k] = 0.0                                           # so that adding delta to this entry is exact
    for gap in (1e-4, 1e-5, 1e-6, 0.0, -1e-6, -1e-5, 1e-9, -1e-9):
        router = base.clone()
        router[9] = router[3]
        router[9, k] = float(gap) / float(x[0, k])
        exact = (router.double() @ x[0].double())
        true_gap = float(exact[9] - exact[3])
        ids, _ = layer.route(x.cuda(), router.cuda(), None)
        got = ids.cpu()[0].tolist()
        assert sorted(got) == [3, 9], (gap, got)
        if abs(true_gap) >= 5e-7:
            assert got == ([9, 3] if true_gap > 0 else [3, 9]), (gap, true_gap, got)
        elif true_gap == 0.0:
            assert got == [3, 9], "an exact tie goes to the lower index"


# ---------------------------------------------------------------- experts over quantised rows
@pytest.mark.parametrize("name,n", [("ds_small", 23), ("kimi_small", 150), ("mixtral_small", 70)])
def test_experts_entry_point_matches_the_oracle_and_the_layer(api, name, n):
    geo = H.small_geometries()[name]
    values = synthetic.make_inputs(geo, 8, 3, "cpu")
    gen = torch.Generator().manual_seed(n)
    rows = torch.randn((n, geo.hidden), generator=gen).to(torch.bfloat16)
    ids = torch.randint(0, geo.experts, (n,), generator=gen)
    ids[: min(n, 70)] = 1                                     # one expert with more rows than a tile
    q, s = O.quantize_activation(rows)
    want = torch.empty((n, geo.hidden), dtype=torch.bfloat16)
    for e in ids.unique().tolist():
        sel = (ids == e).nonzero().flatten()
        want[sel], _, _ = O.expert_mlp(q[sel], s[sel], values["gate"][e], values["gate_scale"][e], values["up"][e],
                                       values["up_scale"][e], values["down"][e], values["down_scale"][e])
    dev = H.to_device(values, "cuda")
    config = api.LayerConfig.from_geometry(geo)
    got = api.experts_forward(config, dev, q.cuda(), s.cuda(), ids.to(torch.int32).cuda())
    H.assert_y_close(got, want, "expert rows")
    # a row's result does not depend on its neighbours or its position: any permutation gives the same bits
    perm = torch.randperm(n, generator=gen)
    again = api.experts_forward(config, dev, q[perm].cuda(), s[perm].cuda(), ids[perm].to(torch.int32).cuda())
    assert torch.equal(again.cpu(), got.cpu()[perm])
    if geo.shared:
        want_sh, _, _ = O.expert_mlp(q, s, values["shared_gate"], values["shared_gate_scale"], values["shared_up"],
                                     values["shared_up_scale"], values["shared_down"], values["shared_down_scale"])
        H.assert_y_close(api.experts_forward(config, dev, q.cuda(), s.cuda(), None), want_sh, "shared expert rows")


# ---------------------------------------------------------------- combine
@pytest.mark.parametrize("tokens,topk,hidden,shared", [(1, 8, 7168, True), (19, 4, 512, False), (64, 2, 4096, True)])
def test_combine_is_the_slot_order_fp32_sum(api, tokens, topk, hidden, shared):
    # megabench/tasks/megamoe.py:176-182 (fp32 accumulator, slots in order, one bf16 rounding) with the
    # weights of megabench/tasks/frontier.py:352: bit-exact, the order of the additions is fixed
    gen = torch.Generator().manual_seed(tokens * 31 + topk)
    rows = torch.randn((tokens * topk + (tokens if shared else 0), hidden), generator=gen).to(torch.bfloat16)
    w = torch.rand((tokens, topk), generator=gen) * 2.5
    acc = torch.zeros((tokens, hidden), dtype=torch.float32)
    slots = rows[: tokens * topk].reshape(tokens, topk, hidden)
    for s in range(topk):
        acc = acc + slots[:, s].to(torch.float32) * w[:, s:s + 1]
    if shared:
        acc = acc + rows[tokens * topk:].to(torch.float32)
    got = api.combine(rows.cuda(), w.cuda(), tokens, shared)
    assert torch.equal(got.cpu().view(torch.int16), acc.to(torch.bfloat16).view(torch.int16))


# ---------------------------------------------------------------- power-of-two (UE8M0) scales
def test_ue8m0_quantiser_matches_reference_vectors(api, golden_dir):
    # edge rows of megabench/tests/test_megamoe.py:57-61 (448, its neighbours, the 1e-4 floor, zero, 896)
    g = np.load(golden_dir / "quantizers.npz")
    x = torch.from_numpy(g["e_in"])
    q, s = api.quantize_rows_ue8m0(x.cuda().contiguous(), block=32)
    assert np.array_equal(q.view(torch.uint8).cpu().numpy(), g["e_q"])
    assert np.array_equal(s.cpu().numpy(), g["e_s"])


@pytest.mark.parametrize("rows,width,block,dtype", [(1, 128, 32, torch.bfloat16), (7, 7168, 32, torch.bfloat16),
                                                    (33, 2048, 128, torch.float32), (5, 259, 32, torch.float32),
                                                    (3, 1, 32, torch.bfloat16), (130, 416, 128, torch.bfloat16)])
def test_ue8m0_quantiser_matches_oracle(api, rows, width, block, dtype):
    gen = torch.Generator().manual_seed(rows * 1000 + width)
    x = (torch.randn((rows, width), generator=gen) * torch.logspace(-5, 2, rows)[:, None]).to(dtype)
    x[0, : min(width, 4)] = 0
    q, s = api.quantize_rows_ue8m0(x.cuda(), block=block)
    wq, ws = O.quantize_activation(x, group=block, scale_format="e8m0")
    assert torch.equal(q.view(torch.uint8).cpu(), wq.view(torch.uint8))
    assert torch.equal(s.cpu(), ws)


def test_epilogue_divisions_match_the_library_divisions(api):
    # The tensor-core epilogues divide by a reciprocal plus fused residual corrections instead of the
    # math library's division (no range check, no slow path). Both forms are run on the device over
    # four million value pairs: normal GEMM outputs, zeros of both signs, tiny and huge values, gates
    # far below the point where exp(-g) overflows, group scales at and above their floor.
    import ctypes as C
    from vibe_megakernel_b200 import _cabi
    lib = _cabi.load()
    n = 1 << 22
    gen = torch.Generator(device="cuda").manual_seed(11)
    g = (torch.randn(n, device="cuda", generator=gen) * 3).to(torch.bfloat16).float()
    u = (torch.randn(n, device="cuda", generator=gen) * 3).to(torch.bfloat16).float()
    edge = torch.tensor([0.0, -0.0, 1e-30, -1e-30, 1e-20, -1e-20, 87.0, -87.0, -88.0, -89.0, -100.0, -300.0, 300.0, 1e4,
                         -1e4, 3.0e38, -3.0e38, 1.0, -1.0, 448.0], device="cuda").to(torch.bfloat16).float()
    g[: edge.numel() * edge.numel()] = edge.repeat_interleave(edge.numel())
    u[: edge.numel() * edge.numel()] = edge.repeat(edge.numel())
    act = (g / (1 + torch.exp(-g)) * u).abs()
    amax = torch.maximum(act[0::2], act[1::2])
    amax = torch.where(torch.isfinite(amax), amax, torch.ones_like(amax))
    spread = torch.rand(n // 2, device="cuda", generator=gen) * 4 + 0.25      # some groups saturate, most do not
    scales = torch.clamp(amax * spread, min=1e-4) / torch.tensor(448.0, device="cuda")
    scales = scales.clamp(max=1e30).contiguous()
    counts = torch.zeros(3, dtype=torch.int32, device="cuda")
    rc = lib.moe_selfcheck_divisions(g.data_ptr(), u.data_ptr(), scales.data_ptr(), n, counts.data_ptr(),
                                     torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    differing_values, differing_codes, seen = counts.tolist()
    assert seen == n // 2
    assert differing_values == 0
    assert differing_codes == 0
