"""Generate the golden vectors in this directory by running the REFERENCE's own code.

Run where the reference checkout is available:

    PYTHONDONTWRITEBYTECODE=1 MEGABENCH_ROOT=<reference checkout> python tests/golden/make_golden.py

It imports ``megabench.tasks.{quantization,frontier,megamoe}`` from that checkout and stores
inputs and outputs of its quantisers, routers and of the MoE layer composed from its
primitives. The stored files are what ``tests/test_oracle_golden.py`` pins the oracle to; the
reference is not needed to run the tests.

Layer composition (only reference functions do arithmetic): per token
``frontier.route(router.float() @ x.float(), ...)`` or the stable softmax rule of
``tasks/distributed.py:174-176``; rows grouped per expert with the stable sort of
``megamoe.experts``; per expert ``unpack(pack_fp8_activation(x)).bf16 @ unpack_fp8_weight.bf16.T``,
fp32 ``g/(1+exp(-g))*u``, ``pack/unpack_fp8_activation``, ``@ down.T``; fp32 slot-order weighted
sum plus the shared expert, one bf16 rounding.
"""

from __future__ import annotations

import os
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
REPO = HERE.parent.parent
if "MEGABENCH_ROOT" not in os.environ:
    raise SystemExit("set MEGABENCH_ROOT to the reference checkout (the directory that holds megabench/)")
sys.path.insert(0, os.environ["MEGABENCH_ROOT"])
sys.path.insert(0, str(REPO))

from megabench.tasks import frontier, quantization as Q  # noqa: E402
from megabench.tasks.oracle import WidenBf16  # noqa: E402

from vibe_megakernel_b200 import synthetic  # noqa: E402


def u8(t):
    return t.view(torch.uint8).numpy()


def bf16_bits(t):
    return t.contiguous().view(torch.int16).numpy()


def quantizer_vectors():
    out = {}
    torch.manual_seed(13)
    value = torch.randn(137, 259).to(torch.bfloat16)          # megabench/tests/test_frontier.py:225-226
    out["w_in"] = bf16_bits(value)
    for power in (False, True):
        p, s = Q.pack_fp8_weight(value, power_of_two=power)
        out[f"w_q_{int(power)}"], out[f"w_s_{int(power)}"] = u8(p), s.numpy()
        out[f"w_deq_{int(power)}"] = Q.unpack_fp8_weight(p, s).numpy()
        p, s = Q.pack_fp8_activation(value, power_of_two=power)
        out[f"wa_q_{int(power)}"], out[f"wa_s_{int(power)}"] = u8(p), s.numpy()
    value = torch.randn((3, 300), generator=torch.Generator().manual_seed(5)).to(torch.bfloat16)
    out["a_in"] = bf16_bits(value)                            # megabench/tests/test_megamoe.py:73
    for power in (False, True):
        p, s = Q.pack_fp8_activation(value, power_of_two=power)
        out[f"a_q_{int(power)}"], out[f"a_s_{int(power)}"] = u8(p), s.numpy()
        out[f"a_deq_{int(power)}"] = Q.unpack_fp8_activation(p, s).numpy()
    generator = torch.Generator().manual_seed(3)              # megabench/tests/test_megamoe.py:57-61
    value = torch.randn((64, 256), generator=generator) * torch.logspace(-6, 3, 64)[:, None]
    edges = torch.tensor([448., 448.00003, 447.99997, 224., 1e-4, 1e-6, 0., 2. ** -22 * 448, 896.])
    value[:len(edges), 0] = edges
    out["e_in"] = value.numpy()
    p, s = Q.pack_fp8_activation(value, block=32, scale_format="e8m0")
    out["e_q"], out["e_s"] = u8(p), s.numpy()
    out["e_deq"] = Q.unpack_fp8_activation(p, s, block=32).numpy()
    p, s = Q.pack_fp8_activation(value)                       # float scales on the same edge rows
    out["ef_q"], out["ef_s"] = u8(p), s.numpy()
    # fp32 input (SwiGLU output is fp32 when it is requantised, megamoe.py:125-128)
    value = torch.randn((5, 512), generator=torch.Generator().manual_seed(11)) * 3
    value[1] = 0
    value[2, :128] = 1e-7
    out["f_in"] = value.numpy()
    p, s = Q.pack_fp8_activation(value)
    out["f_q"], out["f_s"] = u8(p), s.numpy()
    np.savez_compressed(HERE / "quantizers.npz", **out)


def softmax_route(scores, topk):
    ids = torch.argsort(scores, descending=True, stable=True)[:topk]   # tasks/distributed.py:175
    return ids, scores[ids].softmax(-1)                                # tasks/distributed.py:176


def router_vectors():
    out = {}
    gen = torch.Generator().manual_seed(21)
    cases = []
    for name, e, topk, groups, top_groups, scaling in (("ds", 256, 8, 8, 4, 2.5), ("kimi", 384, 8, 1, 1, 2.827),
                                                       ("small", 16, 4, 4, 2, 1.0), ("pair", 8, 2, 2, 1, 2.5)):
        scores = torch.randn((12, e), generator=gen)
        bias = torch.randn((e,), generator=gen) * 0.05
        ids = torch.empty((12, topk), dtype=torch.int64)
        ws = torch.empty((12, topk))
        for t in range(12):
            ids[t], ws[t] = frontier.route(scores[t], bias, topk, groups, top_groups, scaling)
        out[f"{name}_scores"], out[f"{name}_bias"] = scores.numpy(), bias.numpy()
        out[f"{name}_ids"], out[f"{name}_w"] = ids.numpy(), ws.numpy()
        cases.append((name, e, topk, groups, top_groups, scaling))
    out["sig_cases"] = np.array([[e, k, g, tg] for _, e, k, g, tg, _ in cases], dtype=np.int64)
    out["sig_scaling"] = np.array([s for *_, s in cases], dtype=np.float64)
    # ties: all-zero scores pick the lowest ids (megabench/tests/test_frontier.py:297-299)
    ids, ws = frontier.route(torch.zeros(8), torch.zeros(8), 2, 2, 1)
    out["tie_ids"], out["tie_w"] = ids.numpy(), ws.numpy()
    # ties inside and across groups, and more picks than live experts
    scores = torch.tensor([0.5, 0.5, -1.0, 0.5, 0.5, 0.5, -1.0, 0.5, 2.0, -3.0, -3.0, -3.0, 0.5, 0.5, 0.5, 0.5])
    ids, ws = frontier.route(scores, torch.zeros(16), 6, 4, 2, 1.0)
    out["tie2_scores"], out["tie2_ids"], out["tie2_w"] = scores.numpy(), ids.numpy(), ws.numpy()
    ids, ws = frontier.route(scores, torch.zeros(16), 6, 4, 1, 1.0)
    out["tie3_ids"], out["tie3_w"] = ids.numpy(), ws.numpy()
    for name, e, topk in (("sm16", 16, 4), ("sm128", 128, 8), ("sm8", 8, 2)):
        scores = torch.randn((12, e), generator=gen)
        scores[3, 1] = scores[3, 5]          # an exact tie
        ids = torch.empty((12, topk), dtype=torch.int64)
        ws = torch.empty((12, topk))
        for t in range(12):
            ids[t], ws[t] = softmax_route(scores[t], topk)
        out[f"{name}_scores"], out[f"{name}_ids"], out[f"{name}_w"] = scores.numpy(), ids.numpy(), ws.numpy()
    # sqrt-softplus scores with a selection bias: the expressions of tasks/dsv41.py:623-626
    from megabench.tasks import dsv41
    for name, e, topk in (("sp256", 256, 6), ("sp32", 32, 4)):
        scores = torch.randn((12, e), generator=gen) * 3
        scores[2, 0] = 25.0                                   # beyond softplus's threshold
        scores[5, 3] = scores[5, 9]                           # an exact tie
        bias = torch.randn((e,), generator=gen) * 0.05
        p = torch.nn.functional.softplus(scores.float()).sqrt()
        ids = dsv41.descending(p + bias, topk)
        ws = p.gather(-1, ids)
        ws = ws / (ws.sum(-1, keepdim=True) + 1e-20) * dsv41.ROUTE_SCALE
        out[f"{name}_scores"], out[f"{name}_bias"] = scores.numpy(), bias.numpy()
        out[f"{name}_ids"], out[f"{name}_w"] = ids.numpy(), ws.numpy()
    out["sp_scaling"] = np.array([dsv41.ROUTE_SCALE], dtype=np.float64)
    # router with a linear-layer bias, stable top-k, softmax over the selection: tasks/gptoss.py:106-109
    for name, e, topk in (("go32", 32, 4), ("go128", 128, 4)):
        x = torch.randn((12, 64), generator=gen)
        router = torch.randn((e, 64), generator=gen) * 0.2
        bias = torch.randn((e,), generator=gen) * 0.3
        ids = torch.empty((12, topk), dtype=torch.int64)
        ws = torch.empty((12, topk))
        for t in range(12):
            scores = torch.nn.functional.linear(x[t], router, bias)
            selected = torch.argsort(scores, descending=True, stable=True)[:topk]
            ids[t], ws[t] = selected, scores[selected].softmax(-1)
        out[f"{name}_logits"] = (x @ router.T).numpy()        # without the bias: the kernels add it themselves
        out[f"{name}_bias"], out[f"{name}_ids"], out[f"{name}_w"] = bias.numpy(), ids.numpy(), ws.numpy()
    np.savez_compressed(HERE / "routers.npz", **out)


def reference_layer(geo, values, *, widen=False, megamoe_swiglu=0.0, fp32_operands=False):
    """The layer composed from reference primitives only. ``megamoe_swiglu`` > 0 switches to the
    MegaMoE form: ``megamoe.swiglu`` (clamp at that bound, routing weight inside, megamoe.py:116-122)
    and an unweighted slot-order sum (megamoe.py:176-182); the shared expert's rows carry weight 1.
    ``fp32_operands`` replaces every expert GEMM by the expression of ``frontier.linear``
    (frontier.py:184-186): fp32 dequantised operands, one rounding of the result to bf16."""
    from types import SimpleNamespace
    from megabench.tasks import megamoe
    case = SimpleNamespace(params={"swiglu_limit": megamoe_swiglu})
    x = values["x"]
    tokens = x.shape[0]
    bf16 = torch.bfloat16
    ids, ws = [], []
    for row in x:
        scores = values["router"].float() @ row.float()                 # frontier.py:343
        if geo.scoring == "sigmoid":
            i, w = frontier.route(scores, values["router_bias"], geo.topk, geo.n_group, geo.topk_group, geo.scaling)
        else:
            i, w = softmax_route(scores, geo.topk)
        ids.append(i)
        ws.append(w)
    ids, ws = torch.stack(ids), torch.stack(ws)
    flat = ids.flatten()
    order = torch.sort(flat, stable=True).indices                       # megamoe.py:137
    counts = torch.bincount(flat, minlength=geo.experts).tolist()       # megamoe.py:138
    source = torch.div(order, geo.topk, rounding_mode="floor")          # megamoe.py:165

    def linear_rows(rows, weight, scale):
        # frontier.py:185-186, row by row as the reference calls it; `rows` may be fp32 (the SwiGLU output)
        return torch.stack([(Q.unpack_fp8_weight(weight, scale) @ Q.unpack_fp8_activation(*Q.pack_fp8_activation(r))).to(bf16)
                            for r in rows])

    def mlp(rows, gate, gs, up, us, down, ds, row_weights=None):
        if fp32_operands:
            g = torch.stack([frontier.linear(r, gate, gs, False) for r in rows])    # frontier.py:180-186
            u = torch.stack([frontier.linear(r, up, us, False) for r in rows])
            g32, u32 = g.float(), u.float()
            return linear_rows(g32 / (1 + torch.exp(-g32)) * u32, down, ds)
        xa = Q.unpack_fp8_activation(*Q.pack_fp8_activation(rows)).to(bf16)      # megamoe.py:146
        g = xa @ Q.unpack_fp8_weight(gate, gs).to(bf16).T                      # megamoe.py:147,149
        u = xa @ Q.unpack_fp8_weight(up, us).to(bf16).T
        if megamoe_swiglu > 0:
            a = megamoe.swiglu(case, torch.cat([g, u], dim=-1), row_weights)    # megamoe.py:116-122
        else:
            g32, u32 = g.float(), u.float()
            a = g32 / (1 + torch.exp(-g32)) * u32                               # megamoe.py:119-122
        a = Q.unpack_fp8_activation(*Q.pack_fp8_activation(a)).to(bf16)         # megamoe.py:125-128
        return a @ Q.unpack_fp8_weight(down, ds).to(bf16).T                     # megamoe.py:148-149

    output = torch.empty((flat.numel(), geo.hidden), dtype=bf16)
    start = 0
    for expert, count in enumerate(counts):
        if not count:
            continue
        selected = order[start:start + count]
        rows = x[source[start:start + count]]
        start += count
        output[selected] = mlp(rows, values["gate"][expert], values["gate_scale"][expert],
                               values["up"][expert], values["up_scale"][expert],
                               values["down"][expert], values["down_scale"][expert],
                               ws.flatten()[selected] if megamoe_swiglu > 0 else None)
    slots = output.view(tokens, geo.topk, -1)
    combined = torch.zeros((tokens, geo.hidden), dtype=torch.float32)
    for slot in range(geo.topk):
        if megamoe_swiglu > 0:
            combined = combined + slots[:, slot].float()                          # megamoe.py:178-181
        else:
            combined = combined + slots[:, slot].float() * ws[:, slot:slot + 1]   # frontier.py:352
    if geo.shared:
        combined = combined + mlp(x, values["shared_gate"], values["shared_gate_scale"],
                                  values["shared_up"], values["shared_up_scale"],
                                  values["shared_down"], values["shared_down_scale"],
                                  torch.ones(tokens) if megamoe_swiglu > 0 else None).float()   # frontier.py:353
    return {"y": combined if widen else combined.to(bf16), "expert_ids": ids, "topk_weights": ws, "order": order}


def layer_vectors():
    """Small layers whose inputs the seeded generator of the package re-creates bit for bit."""
    import dataclasses
    out = {}
    specs = {
        "tiny": (synthetic.GEOMETRIES["tiny"], 4, 0),
        "ds_small": (dataclasses.replace(synthetic.GEOMETRIES["deepseek_v3"], name="ds_small", hidden=512, inter=256,
                                         experts=32, topk=4, n_group=4, topk_group=2), 6, 0),
        "qwen_small": (dataclasses.replace(synthetic.GEOMETRIES["qwen3_30b_a3b"], name="qwen_small", hidden=256,
                                           inter=128, experts=8, topk=2), 5, 0),
    }
    for name, (geo, tokens, seed) in specs.items():
        values = synthetic.make_inputs(geo, tokens, seed, "cpu")
        got = reference_layer(geo, values)
        with torch.no_grad(), WidenBf16():
            wide = reference_layer(geo, values, widen=True)
        out[f"{name}_y"] = bf16_bits(got["y"])
        out[f"{name}_y_fp32"] = wide["y"].float().numpy()
        out[f"{name}_ids"] = got["expert_ids"].numpy()
        out[f"{name}_w"] = got["topk_weights"].numpy()
        out[f"{name}_order"] = got["order"].numpy()
        out[f"{name}_x_sum"] = np.array([float(values["x"].float().sum()), float(values["router"].sum()),
                                         float(values["gate"].float().sum()), float(values["down_scale"].sum())])
        out[f"{name}_geo"] = np.array([geo.hidden, geo.inter, geo.experts, geo.topk, geo.shared,
                                       geo.n_group, geo.topk_group, tokens, seed], dtype=np.int64)
    np.savez_compressed(HERE / "layers.npz", **out)


def linear_vectors():
    """``frontier.linear`` (fp32 dequantised operands, bf16 result; frontier.py:180-186) on its own and
    as the GEMM of small layers: the second operand convention of the reference."""
    import dataclasses
    out = {}
    gen = torch.Generator().manual_seed(61)
    for name, m, k in (("a", 256, 512), ("b", 384, 1024), ("ragged", 137, 259)):
        weight = torch.randn((m, k), generator=gen) * 0.02
        wq, ws = Q.pack_fp8_weight(weight)
        x = torch.randn((5, k), generator=gen).to(torch.bfloat16)
        out[f"{name}_w"], out[f"{name}_ws"], out[f"{name}_x"] = u8(wq), ws.numpy(), bf16_bits(x)
        out[f"{name}_y"] = bf16_bits(torch.stack([frontier.linear(r, wq, ws, False) for r in x]))
    specs = {
        "tiny": (synthetic.GEOMETRIES["tiny"], 4, 0),
        "ds_small": (dataclasses.replace(synthetic.GEOMETRIES["deepseek_v3"], name="ds_small", hidden=512, inter=256,
                                         experts=32, topk=4, n_group=4, topk_group=2), 6, 0),
    }
    for name, (geo, tokens, seed) in specs.items():
        values = synthetic.make_inputs(geo, tokens, seed, "cpu")
        got = reference_layer(geo, values, fp32_operands=True)
        out[f"{name}_layer_y"] = bf16_bits(got["y"])
        out[f"{name}_layer_ids"] = got["expert_ids"].numpy()
        out[f"{name}_geo"] = np.array([geo.hidden, geo.inter, geo.experts, geo.topk, geo.shared,
                                       geo.n_group, geo.topk_group, tokens, seed], dtype=np.int64)
    np.savez_compressed(HERE / "linears.npz", **out)


def megamoe_swiglu_vectors():
    """The MegaMoE SwiGLU form on its own (megabench/tasks/megamoe.py:116-122) and inside small layers."""
    import dataclasses
    from types import SimpleNamespace
    from megabench.tasks import megamoe
    out = {}
    gen = torch.Generator().manual_seed(41)
    l1 = (torch.randn((9, 2 * 256), generator=gen) * 6).to(torch.bfloat16)       # many values beyond the bound
    l1[0, :4] = torch.tensor([10.0, 10.06, -10.06, 0.0]).to(torch.bfloat16)
    w = torch.rand((9,), generator=gen) * 2.5
    out["l1"], out["w"] = bf16_bits(l1), w.numpy()
    out["a"] = megamoe.swiglu(SimpleNamespace(params={"swiglu_limit": 10}), l1, w).numpy()
    specs = {
        "ds_small": (dataclasses.replace(synthetic.GEOMETRIES["deepseek_v3"], name="ds_small", hidden=512, inter=256,
                                         experts=32, topk=4, n_group=4, topk_group=2, weight_std=0.2), 6, 2),
        "qwen_small": (dataclasses.replace(synthetic.GEOMETRIES["qwen3_30b_a3b"], name="qwen_small", hidden=256,
                                           inter=128, experts=8, topk=2, weight_std=0.2), 5, 2),
    }
    for name, (geo, tokens, seed) in specs.items():
        values = synthetic.make_inputs(geo, tokens, seed, "cpu")
        got = reference_layer(geo, values, megamoe_swiglu=1.0)                   # a bound the activations do reach
        out[f"{name}_y"] = bf16_bits(got["y"])
        out[f"{name}_ids"], out[f"{name}_order"] = got["expert_ids"].numpy(), got["order"].numpy()
        out[f"{name}_geo"] = np.array([geo.hidden, geo.inter, geo.experts, geo.topk, geo.shared, geo.n_group,
                                       geo.topk_group, tokens, seed], dtype=np.int64)
    np.savez_compressed(HERE / "megamoe_swiglu.npz", **out)


def megamoe_native_vectors():
    """MXFP4 packing (megabench/tasks/quantization.py:13-51) and the routed experts in their native
    formats: ``megamoe.reference(case, values, serial=True)`` on two reductions of the reference's
    development geometry (megabench/verify_megamoe.py:32-37)."""
    from dataclasses import replace
    from megabench.cases import select_cases
    from megabench.tasks import megamoe
    from megabench.verify_megamoe import development
    out = {}
    gen = torch.Generator().manual_seed(43)
    m = torch.randn((24, 128), generator=gen) * torch.logspace(-3, 3, 24)[:, None]
    # exact ties between neighbouring E2M1 magnitudes (the group's largest value is 6 * 2**k)
    m[0, :9] = torch.tensor([6.0, 0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -2.5])
    m[1, :9] = torch.tensor([6.0, 0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -2.5]) * 2.0 ** -9
    m[2, :4] = torch.tensor([-6.0, -0.75, -1.75, -3.5])
    m[3] = 0.0
    m[4, 32:64] = 0.0
    m[5, :2] = torch.tensor([6.0001, -5.9999])
    out["mx_in"] = m.numpy()
    blocks, scales = Q.pack_mxfp4(m)
    out["mx_blocks"], out["mx_scales"] = blocks.numpy(), scales.numpy()
    out["mx_back"] = Q.unpack_mxfp4(blocks, scales).numpy()
    catalog = [case for case in select_cases("all") if case.family == "megamoe_layer"][0]
    dev = replace(development(catalog, 1), ready=True)
    cases = {      # the development geometry scaled down to keep the fixture small, and a ragged one
        "dev": (replace(dev, params=dev.params | {"hidden": 128, "intermediate": 64}), 7),
        "wide": (replace(dev, params=dev.params | {"tokens": 5, "experts": 12, "topk": 6, "hidden": 160,
                                                   "intermediate": 96, "swiglu_limit": 3}), 11),
    }
    for name, (case, seed) in cases.items():
        values = megamoe.make_inputs(case, seed, "cpu", rank=0)
        for key, value in values.items():
            out[f"{name}_{key}"] = u8(value) if value.dtype == torch.float8_e4m3fn else value.numpy()
        out[f"{name}_y"] = bf16_bits(megamoe.reference(case, values, serial=True)["y"])
        p = case.params
        out[f"{name}_geo"] = np.array([p["tokens"], p["experts"], p["topk"], p["hidden"], p["intermediate"],
                                       p["swiglu_limit"], seed], dtype=np.int64)
    np.savez_compressed(HERE / "megamoe_native.npz", **out)


def kimi_latent_vectors():
    """The MoE block of the Kimi-K3 layer: ``kimi_layer.moe(case, values, normalized, serial=True,
    group=None)`` (megabench/tasks/kimi_layer.py:189-230) on two reductions of the catalog geometry
    (megabench/cases.py:315-324), inputs from the reference's own generator."""
    from dataclasses import replace
    from megabench.cases import select_cases
    from megabench.tasks import kimi_layer
    from megabench.tasks.distributed import matrix
    out = {}
    catalog = [case for case in select_cases("all") if case.id == "kimi-k3-kda-layer-ep8"][0]
    cases = {
        "small": (replace(catalog, gpus=1, ep=1, params=catalog.params | {
            "batch": 5, "experts": 12, "topk": 4, "hidden": 128, "latent_hidden": 128, "intermediate": 128,
            "shared_experts": 2}), 3),
        "one": (replace(catalog, gpus=1, ep=1, params=catalog.params | {
            "batch": 1, "experts": 16, "topk": 6, "hidden": 256, "latent_hidden": 128, "intermediate": 128,
            "shared_experts": 1}), 8),
    }
    keys = ("router", "router_bias", "latent_down", "latent_up", "latent_norm", "gate_blocks", "gate_scales", "up_blocks",
            "up_scales", "down_blocks", "down_scales", "shared_gate", "shared_up", "shared_down")
    for name, (case, seed) in cases.items():
        p = case.params
        # only the tensors of the MoE block (kimi_layer.make_inputs also builds the attention block's)
        values = {k: v for k, v in kimi_layer.make_inputs(case, seed, "cpu", rank=0).items() if k in keys}
        normalized = matrix(seed, "normalized", p["batch"], p["hidden"], 1, "cpu")
        y, sorted_ids = kimi_layer.moe(case, values, normalized, serial=True, group=None)
        for k, v in values.items():
            out[f"{name}_{k}"] = bf16_bits(v) if v.dtype == torch.bfloat16 else v.numpy()
        out[f"{name}_normalized"] = bf16_bits(normalized)
        out[f"{name}_y"], out[f"{name}_sorted_ids"] = bf16_bits(y), sorted_ids.numpy()
        out[f"{name}_geo"] = np.array([p["batch"], p["experts"], p["topk"], p["hidden"], p["latent_hidden"],
                                       p["intermediate"], p["shared_experts"], seed], dtype=np.int64)
    a = (torch.randn((7, 96), generator=torch.Generator().manual_seed(4)) * 8).to(torch.bfloat16)
    b = (torch.randn((7, 96), generator=torch.Generator().manual_seed(5)) * 40).to(torch.bfloat16)
    from megabench.tasks.kimi import situ
    out["situ_gate"], out["situ_up"], out["situ_out"] = bf16_bits(a), bf16_bits(b), bf16_bits(situ(a, b))
    np.savez_compressed(HERE / "kimi_latent.npz", **out)


def block_vectors():
    """RMSNorm -> layer -> residual add, as megabench/tasks/frontier.py:335-354 strings them together."""
    import dataclasses
    from megabench.tasks.common import rms
    out = {}
    specs = {
        "ds_small": (dataclasses.replace(synthetic.GEOMETRIES["deepseek_v3"], name="ds_small", hidden=512, inter=256,
                                         experts=32, topk=4, n_group=4, topk_group=2), 6, 1, True),
        "qwen_small": (dataclasses.replace(synthetic.GEOMETRIES["qwen3_30b_a3b"], name="qwen_small", hidden=256,
                                           inter=128, experts=8, topk=2), 5, 1, False),
    }
    for name, (geo, tokens, seed, fp32_weight) in specs.items():
        values = synthetic.make_inputs(geo, tokens, seed, "cpu")
        gen = torch.Generator().manual_seed(77 + tokens)
        stream = (torch.randn((tokens, geo.hidden), generator=gen) * 3).to(torch.bfloat16)
        gamma = (torch.randn((geo.hidden,), generator=gen) / 100 + 1).to(torch.bfloat16)      # as frontier.py:87
        normalized = rms(stream, gamma, eps=1e-6, weight_in_fp32=fp32_weight)                   # frontier.py:260,335
        got = reference_layer(geo, {**values, "x": normalized})
        new_stream = stream + got["y"].to(stream.dtype)                                        # frontier.py:354
        out[f"{name}_x"], out[f"{name}_gamma"] = bf16_bits(stream), bf16_bits(gamma)
        out[f"{name}_normalized"], out[f"{name}_x_out"] = bf16_bits(normalized), bf16_bits(new_stream)
        out[f"{name}_ids"], out[f"{name}_order"] = got["expert_ids"].numpy(), got["order"].numpy()
        out[f"{name}_geo"] = np.array([geo.hidden, geo.inter, geo.experts, geo.topk, geo.shared, geo.n_group,
                                       geo.topk_group, tokens, seed, int(fp32_weight)], dtype=np.int64)
    np.savez_compressed(HERE / "blocks.npz", **out)


if __name__ == "__main__":
    quantizer_vectors()
    router_vectors()
    layer_vectors()
    block_vectors()
    megamoe_swiglu_vectors()
    megamoe_native_vectors()
    linear_vectors()
    kimi_latent_vectors()
    for f in sorted(HERE.glob("*.npz")):
        print(f.name, f.stat().st_size)
