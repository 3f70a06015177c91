"""CPU oracle for the FP8 MoE decode layer. TEST INFRASTRUCTURE ONLY.

This file restates, in plain torch on the host, the arithmetic that the
reference benchmark (kamahori/vibe-megakernel, package ``megabench``) uses
for its FP8 mixture-of-experts layer. It is the checker for the CUDA path:
only the test-suite, the smoke entry and the CPU-baseline leg of the
benchmark may import it. The product (``vibe_megakernel_b200``) never does.

Parity is pinned: ``tests/golden/`` holds vectors produced by running the
reference's own functions (the generating script sits beside them), and
``tests/test_oracle_golden.py`` checks every function below against them.

Each function cites the reference lines it follows (paths are relative to the
reference project root).
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch

E4M3_MAX = 448.0
AMAX_FLOOR = 1e-4
GROUP = 128


# --------------------------------------------------------------------------
# Quantisation formats  (megabench/tasks/quantization.py:54-131)
# --------------------------------------------------------------------------

def scale_from_amax(amax: torch.Tensor, power_of_two: bool = False) -> torch.Tensor:
    """fp32 scale = max(amax, 1e-4) / 448, optionally rounded up to 2**k.

    megabench/tasks/quantization.py:57-59.
    """
    # The divisor is a tensor on purpose: torch's CUDA kernels replace a division by a Python number
    # with a multiplication by its reciprocal, which is one ulp off for many inputs and then moves
    # payload values that sit exactly on a rounding tie (frequent for bf16 inputs). A tensor divisor
    # is a true IEEE division on every device, as the reference's CPU arithmetic is.
    s = torch.clamp(amax.to(torch.float32), min=AMAX_FLOOR) / torch.tensor(E4M3_MAX, dtype=torch.float32, device=amax.device)
    if power_of_two:
        s = torch.exp2(torch.ceil(torch.log2(s)))
    return s


def ue8m0_exponent(amax: torch.Tensor) -> torch.Tensor:
    """Biased power-of-two exponent (uint8) that maps ``amax`` inside e4m3.

    Integer arithmetic on the fp32 bit pattern: bump the exponent when the
    mantissa is above 1.75 (448 = 1.75 * 2**8), remove 448's exponent, floor
    at the exponent of the 1e-4 clamp. megabench/tasks/quantization.py:62-77.
    """
    bits = amax.to(torch.float32).contiguous().view(torch.int32)
    carry = 0x7FFFFF - 0x600000
    e = (bits + carry) >> 23
    e = torch.clamp(e, min=105 + 8) - 8
    return e.to(torch.uint8)


def ue8m0_value(exp: torch.Tensor, inverse: bool = False) -> torch.Tensor:
    """Exact fp32 2**(e-127) or its reciprocal. quantization.py:80-84."""
    b = exp.to(torch.int32)
    if inverse:
        b = 254 - b
    return (b << 23).view(torch.float32)


def quantize_activation(x: torch.Tensor, *, group: int = GROUP, power_of_two: bool = False,
                        scale_format: str = "float"):
    """Per-row, per-``group``-channel dynamic e4m3 quantisation.

    Returns (payload e4m3 [..., W], scales [..., ceil(W/group)]). A ragged last
    group is padded with zeros for the amax; padding is dropped from the
    payload. megabench/tasks/quantization.py:87-109.
    """
    w = x.shape[-1]
    pad = (-w) % group
    v = x.to(torch.float32)
    if pad:
        v = torch.cat([v, v.new_zeros(*v.shape[:-1], pad)], dim=-1)
    v = v.reshape(*v.shape[:-1], -1, group)
    amax = v.abs().amax(dim=-1)
    if scale_format == "e8m0":
        scales = ue8m0_exponent(amax)
        q = (v * ue8m0_value(scales, inverse=True).unsqueeze(-1)).to(torch.float8_e4m3fn)
    elif scale_format == "float":
        scales = scale_from_amax(amax, power_of_two)
        q = torch.clamp(v / scales.unsqueeze(-1), -E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    else:
        raise ValueError(f"unknown scale format {scale_format!r}")
    q = q.reshape(*q.shape[:-2], -1)[..., :w].contiguous()
    return q, scales


def dequantize_activation(q: torch.Tensor, scales: torch.Tensor, *, group: int = GROUP) -> torch.Tensor:
    """fp32 = payload * per-group scale. quantization.py:112-116."""
    if scales.dtype == torch.uint8:
        scales = ue8m0_value(scales)
    wide = scales.repeat_interleave(group, dim=-1)[..., :q.shape[-1]]
    return q.to(torch.float32) * wide


def quantize_weight(w: torch.Tensor, *, power_of_two: bool = False):
    """e4m3 payload [R, C] with one fp32 scale per 128x128 block.

    megabench/tasks/quantization.py:119-126.
    """
    r, c = w.shape
    pr, pc = (-r) % GROUP, (-c) % GROUP
    v = torch.zeros((r + pr, c + pc), dtype=torch.float32, device=w.device)
    v[:r, :c] = w.to(torch.float32)
    blocks = v.reshape((r + pr) // GROUP, GROUP, (c + pc) // GROUP, GROUP)
    scales = scale_from_amax(blocks.abs().amax(dim=(1, 3)), power_of_two)
    q = torch.clamp(blocks / scales[:, None, :, None], -E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    return q.reshape(r + pr, c + pc)[:r, :c].contiguous(), scales


def dequantize_weight(q: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """fp32 = payload * its block's scale. quantization.py:129-131."""
    wide = scales.repeat_interleave(GROUP, dim=0).repeat_interleave(GROUP, dim=1)
    return q.to(torch.float32) * wide[:q.shape[0], :q.shape[1]]


# --------------------------------------------------------------------------
# Routers
# --------------------------------------------------------------------------

def route_sigmoid_grouped(scores: torch.Tensor, bias: torch.Tensor, topk: int, n_group: int,
                          topk_group: int, scaling: float):
    """One token. Sigmoid scores with a selection-only bias and group limit.

    p = sigmoid(s); c = p + bias. With more than one group, a group's score is
    the sum of its two largest c; the best ``topk_group`` groups survive (ties
    to the lower group index) and the rest become -inf. ids = first ``topk`` of
    a stable descending sort of c; weights = p[ids] / (sum + 1e-20) * scaling.
    megabench/tasks/frontier.py:229-242.
    """
    p = torch.sigmoid(scores)
    c = p + bias
    if n_group > 1:
        g = c.reshape(n_group, -1)
        best_two = torch.sort(g, dim=-1, descending=True, stable=True).values[:, :2].sum(dim=-1)
        keep = torch.argsort(best_two, descending=True, stable=True)[:topk_group]
        alive = torch.zeros(n_group, dtype=torch.bool, device=scores.device)
        alive[keep] = True
        c = torch.where(alive[:, None], g, torch.full_like(g, -math.inf)).reshape(-1)
    ids = torch.argsort(c, descending=True, stable=True)[:topk]
    w = p[ids]
    return ids, w / (w.sum() + 1e-20) * scaling


def route_softmax(scores: torch.Tensor, topk: int):
    """One token. ids = first ``topk`` of a stable descending sort of the
    logits; weights = softmax over the selected logits (softmax over all,
    then renormalised over the selection, is the same number).
    megabench/tasks/distributed.py:174-176; megabench/tasks/references/moe.py:68-70.
    """
    ids = torch.argsort(scores, descending=True, stable=True)[:topk]
    return ids, torch.softmax(scores[ids], dim=-1)


def route_sqrt_softplus(scores: torch.Tensor, bias: torch.Tensor | None, topk: int, scaling: float):
    """One token. p = sqrt(softplus(s)); ids = first ``topk`` of a stable
    descending sort of p + bias; weights = p[ids] / (sum + 1e-20) * scaling.
    megabench/tasks/dsv41.py:622-626 (``descending`` is the stable argsort of
    megabench/tasks/dsv41.py:278-280)."""
    p = torch.nn.functional.softplus(scores.to(torch.float32)).sqrt()
    c = p if bias is None else p + bias
    ids = torch.argsort(c, descending=True, stable=True)[:topk]
    w = p[ids]
    return ids, w / (w.sum() + 1e-20) * scaling


def route_softmax_biased(scores: torch.Tensor, bias: torch.Tensor | None, topk: int):
    """One token. The bias is the router's linear-layer bias: s = logits + bias,
    ids = first ``topk`` of a stable descending sort of s, weights =
    softmax(s[ids]). megabench/tasks/gptoss.py:106-109."""
    s = scores if bias is None else scores + bias
    ids = torch.argsort(s, descending=True, stable=True)[:topk]
    return ids, torch.softmax(s[ids], dim=-1)


# --------------------------------------------------------------------------
# Layer
# --------------------------------------------------------------------------

@dataclass(frozen=True)
class LayerSpec:
    hidden: int
    inter: int
    experts: int
    topk: int
    shared: int = 1                 # number of shared experts (0 or 1)
    scoring: str = "sigmoid"        # "sigmoid" (grouped, biased) or "softmax"
    n_group: int = 1
    topk_group: int = 1
    scaling: float = 1.0
    swiglu_limit: float = 0.0       # > 0: gate clamped above, up clamped both ways (megamoe.py:119-121)
    weight_before_requant: bool = False   # routing weight inside SwiGLU (megamoe.py:122), plain sum at the combine


def router_logits(router: torch.Tensor, x_row: torch.Tensor) -> torch.Tensor:
    """fp32 GEMV per token: router.float() @ x.float().

    megabench/tasks/frontier.py:343; megabench/tasks/kimi_layer.py:200.
    """
    return router.to(torch.float32) @ x_row.to(torch.float32)


def route_tokens(spec: LayerSpec, x: torch.Tensor, router: torch.Tensor, bias: torch.Tensor | None):
    ids, ws = [], []
    for row in x:
        s = router_logits(router, row)
        if spec.scoring == "sigmoid":
            i, w = route_sigmoid_grouped(s, bias, spec.topk, spec.n_group, spec.topk_group, spec.scaling)
        elif spec.scoring == "softmax":
            i, w = route_softmax(s, spec.topk)
        elif spec.scoring == "sqrt_softplus":
            i, w = route_sqrt_softplus(s, bias, spec.topk, spec.scaling)
        elif spec.scoring == "softmax_biased":
            i, w = route_softmax_biased(s, bias, spec.topk)
        else:
            raise ValueError(spec.scoring)
        ids.append(i)
        ws.append(w)
    return torch.stack(ids), torch.stack(ws)


def owner_order(flat_ids: torch.Tensor, experts_per_rank: int) -> torch.Tensor:
    """Stable order of routed rows by owning rank: keeps (token, slot) order
    inside each destination. megabench/tasks/megamoe.py:161-164."""
    owner = torch.div(flat_ids, experts_per_rank, rounding_mode="floor")
    return torch.sort(owner, stable=True).indices


def expert_order(local_ids: torch.Tensor, n_local: int):
    """Stable order of arrived rows by local expert id and the rows per
    expert. megabench/tasks/megamoe.py:137-138."""
    order = torch.sort(local_ids, stable=True).indices
    counts = torch.bincount(local_ids, minlength=n_local)
    return order, counts


def _silu_mul(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """fp32 gate/(1+exp(-gate)) * up on values already rounded to the compute
    dtype of the GEMM output. megabench/tasks/megamoe.py:116-122 (no clamp, no
    weight: the routing weight is applied at the combine, frontier.py:352)."""
    g = gate.to(torch.float32)
    return g / (1 + torch.exp(-g)) * up.to(torch.float32)


def _silu_mul_clamped(gate: torch.Tensor, up: torch.Tensor, bound: float, weights: torch.Tensor | None) -> torch.Tensor:
    """The MegaMoE form: gate clamped above and up clamped both ways in the GEMM
    output dtype, fp32 silu(gate) * up, then times the row's routing weight.
    megabench/tasks/megamoe.py:116-122."""
    if bound > 0:
        gate = gate.clamp(max=bound)
        up = up.clamp(-bound, bound)
    g, u = gate.to(torch.float32), up.to(torch.float32)
    a = g / (1 + torch.exp(-g)) * u
    return a if weights is None else a * weights[:, None]


def fp8_linear(rows_q, rows_s, weight, weight_s, *, compute=torch.bfloat16, operands: str = "bf16") -> torch.Tensor:
    """rows [n, K] (e4m3 + 1x128 fp32 scales) times an FP8 block-scaled matrix [M, K]: [n, M] in ``compute``.

    The reference multiplies dequantised operands in two ways:
      * ``operands="bf16"`` (megabench/tasks/megamoe.py:146-149, deepseek_checkpoint.py:457): both
        operands are rounded to ``compute`` (bf16) first, the GEMM accumulates in fp32 and rounds
        once to ``compute``. This is the graded "dequantize-then-bf16" path.
      * ``operands="fp32"`` (megabench/tasks/frontier.py:184-186, ``linear``): the fp32 dequantised
        operands are multiplied as they are and only the result is rounded to ``compute``. A
        block-scaled tensor-core GEMM (exact FP8 products, fp32 scaling) is numerically this one.
    With ``compute=torch.float32`` the two coincide (the widened noise-floor path, oracle.py:35-53).

    The reference calls ``linear`` token by token (a matrix-vector product); on the CPU, for up to
    64 rows, so does this function, which makes it bit-identical to the reference's vectors. Larger
    or CUDA inputs use one matrix-matrix product: a different fp32 summation order, which moves
    about one bf16 result in a thousand by one ulp.
    """
    xa = dequantize_activation(rows_q, rows_s)
    wd = dequantize_weight(weight, weight_s)
    if operands == "fp32":
        if xa.device.type == "cpu" and xa.dim() == 2 and xa.shape[0] <= 64:
            return torch.stack([wd @ row for row in xa]).to(compute) if xa.shape[0] else (xa @ wd.T).to(compute)
        return (xa @ wd.T).to(compute)
    if operands != "bf16":
        raise ValueError(f"unknown operand convention {operands!r}")
    return xa.to(compute) @ wd.to(compute).T


def expert_mlp(rows_q, rows_s, gate, gate_s, up, up_s, down, down_s, *, compute=torch.bfloat16,
               swiglu_limit: float = 0.0, row_weights: torch.Tensor | None = None, operands: str = "bf16"):
    """One expert over its rows.

    Each GEMM is ``fp8_linear`` (operand convention ``operands``, fp32 accumulation, result in
    ``compute``: bf16 for the graded path, fp32 for the widened noise-floor path); SwiGLU is
    fp32; its result is requantised per row per 128 channels.
    megabench/tasks/megamoe.py:146-149,125-128.
    Returns (rows [n, H] in ``compute``, requantised payload, its scales).
    """
    g = fp8_linear(rows_q, rows_s, gate, gate_s, compute=compute, operands=operands)
    u = fp8_linear(rows_q, rows_s, up, up_s, compute=compute, operands=operands)
    if swiglu_limit > 0 or row_weights is not None:
        a = _silu_mul_clamped(g, u, swiglu_limit, row_weights)
    else:
        a = _silu_mul(g, u)
    aq, a_s = quantize_activation(a)
    return fp8_linear(aq, a_s, down, down_s, compute=compute, operands=operands), aq, a_s


def moe_layer(spec: LayerSpec, values: dict, *, compute=torch.bfloat16, keep_intermediates: bool = False,
              expert_slot: dict | None = None, operands: str = "bf16"):
    """Whole layer on one rank holding every expert.

    values: x bf16 [T,H]; router fp32 [E,H]; router_bias fp32 [E] (sigmoid);
    gate/up e4m3 [E,I,H] + gate_scale/up_scale fp32 [E,I/128,H/128];
    down e4m3 [E,H,I] + down_scale; shared_gate/shared_up [I,H],
    shared_down [H,I] with ``_scale`` (when spec.shared).

    Output keys: y bf16 [T,H]; expert_ids int64 [T,topk] (choice order);
    topk_weights fp32 [T,topk]; order int64 [T*topk] (stable grouping of the
    flattened ids by expert); counts int64 [E].
    ``expert_slot`` maps an expert id to its index in the weight tensors when only
    the experts that are hit were materialised (default: identity).
    ``operands`` is the operand convention of every expert GEMM (see ``fp8_linear``).
    Combine: fp32 sum over slots in slot order of row*weight, then the shared
    expert's row, one rounding to bf16 (frontier.py:349-354, megamoe.py:176-182).
    """
    x = values["x"]
    t, h = x.shape
    ids, ws = route_tokens(spec, x, values["router"], values.get("router_bias"))
    flat = ids.reshape(-1)
    order, counts = expert_order(flat, spec.experts)
    xq, xs = quantize_activation(x.to(torch.bfloat16))
    src = torch.div(order, spec.topk, rounding_mode="floor")
    out_rows = torch.empty((flat.numel(), h), dtype=compute, device=x.device)
    inter = {}
    start = 0
    for e, n in enumerate(counts.tolist()):
        if n == 0:
            continue
        sel = order[start:start + n]
        tok = src[start:start + n]
        start += n
        k = e if expert_slot is None else expert_slot[e]
        res, aq, a_s = expert_mlp(xq[tok], xs[tok], values["gate"][k], values["gate_scale"][k],
                                  values["up"][k], values["up_scale"][k],
                                  values["down"][k], values["down_scale"][k], compute=compute,
                                  swiglu_limit=spec.swiglu_limit, operands=operands,
                                  row_weights=ws.reshape(-1)[sel] if spec.weight_before_requant else None)
        out_rows[sel] = res
        if keep_intermediates:
            inter[e] = (aq, a_s)
    acc = torch.zeros((t, h), dtype=torch.float32, device=x.device)
    slots = out_rows.reshape(t, spec.topk, h)
    for s in range(spec.topk):
        if spec.weight_before_requant:      # the rows are weighted already: plain slot-order sum (megamoe.py:178-181)
            acc = acc + slots[:, s].to(torch.float32)
        else:
            acc = acc + slots[:, s].to(torch.float32) * ws[:, s:s + 1]
    if spec.shared:
        sh, _, _ = expert_mlp(xq, xs, values["shared_gate"], values["shared_gate_scale"],
                              values["shared_up"], values["shared_up_scale"],
                              values["shared_down"], values["shared_down_scale"], compute=compute,
                              swiglu_limit=spec.swiglu_limit, operands=operands)
        acc = acc + sh.to(torch.float32)
    out = {"y": acc.to(torch.bfloat16), "expert_ids": ids, "topk_weights": ws,
           "order": order, "counts": counts}
    if compute is not torch.bfloat16:
        out["y_fp32"] = acc
    if keep_intermediates:
        out["xq"], out["xs"], out["slots"], out["requant"] = xq, xs, slots, inter
    return out


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6, *, weight_in_fp32: bool = False) -> torch.Tensor:
    """RMSNorm in front of the MoE block. n = x.float() * rsqrt(mean(x.float()^2)
    + eps); ``weight_in_fp32`` (DeepSeek family): (n * weight.float()) rounded
    once to x's dtype; otherwise n is rounded to x's dtype and multiplied by
    the weight in that dtype. megabench/tasks/common.py:13-21 (without the
    Gemma offset), called at megabench/tasks/frontier.py:260,335."""
    xf = x.to(torch.float32)
    n = xf * torch.rsqrt(xf.square().mean(-1, keepdim=True) + eps)
    if weight_in_fp32:
        return (n * weight.to(torch.float32)).to(x.dtype)
    return n.to(x.dtype) * weight.to(x.dtype)


def moe_block(spec: LayerSpec, values: dict, norm_weight: torch.Tensor, eps: float = 1e-6, *,
              weight_in_fp32: bool = False, **kwargs) -> dict:
    """The layer with the step either side: ``x + layer(rms(x))`` where the
    layer's output is rounded to x's dtype before the add and the sum is
    rounded again (megabench/tasks/frontier.py:335 ... 354). Returns the
    layer's outputs with ``x`` (the new residual stream) and ``normalized``."""
    x = values["x"]
    normalized = rms_norm(x, norm_weight, eps, weight_in_fp32=weight_in_fp32)
    out = moe_layer(spec, {**values, "x": normalized}, **kwargs)
    out["normalized"] = normalized
    out["x"] = x + out["y"].to(x.dtype)
    return out


def decision_margins(spec: LayerSpec, x: torch.Tensor, router: torch.Tensor, bias: torch.Tensor | None) -> float:
    """Smallest gap at any routing decision boundary, from fp64 logits.

    Used by the input generators: a seed is accepted only when every boundary
    (group cut, top-k cut, in-top-k order) has a gap far above fp32 summation
    noise, so that any correct fp32/fp64 router picks the same ids.
    """
    logits = x.to(torch.float64) @ router.to(torch.float64).T
    worst = math.inf
    for s in logits:
        if spec.scoring == "sigmoid":
            p = torch.sigmoid(s)
            c = p + (bias.to(torch.float64) if bias is not None else 0)
            if spec.n_group > 1:
                g = c.reshape(spec.n_group, -1)
                sc = torch.sort(g, dim=-1, descending=True).values[:, :2].sum(-1)
                ss = torch.sort(sc, descending=True).values
                worst = min(worst, float(ss[spec.topk_group - 1] - ss[spec.topk_group]))
                # within-group top-2 membership does not change ids, only the sum
                keep = torch.argsort(sc, descending=True)[:spec.topk_group]
                alive = torch.zeros(spec.n_group, dtype=torch.bool, device=x.device)
                alive[keep] = True
                c = torch.where(alive[:, None], g, torch.full_like(g, -math.inf)).reshape(-1)
        elif spec.scoring == "sqrt_softplus":
            c = torch.nn.functional.softplus(s).sqrt() + (bias.to(torch.float64) if bias is not None else 0)
        elif spec.scoring == "softmax_biased":
            c = s + (bias.to(torch.float64) if bias is not None else 0)
        else:
            c = s
        top = torch.sort(c, descending=True).values[:spec.topk + 1]
        gaps = top[:-1] - top[1:]
        worst = min(worst, float(gaps.min()))
    return worst
