"""CPU oracle for the MegaMoE-native format of the routed experts. TEST INFRASTRUCTURE ONLY.

Restates, in plain torch on the host, the routed-expert layer of the reference benchmark
(kamahori/vibe-megakernel, ``megabench/tasks/megamoe.py``) in its native number formats:
MXFP4 weights (E2M1 codes, one E8M0 scale per 32 input channels), E4M3 activations with one
E8M0 scale per 32 channels, clamped SwiGLU with the routing weight inside, and a plain
slot-order sum. Routing is an input. Only the test-suite, the smoke entry and the CPU-baseline
leg of the benchmark may import this file; the product never does.

Parity is pinned: ``tests/golden/megamoe_native.npz`` holds inputs and outputs of the
reference's own ``pack_mxfp4``/``unpack_mxfp4`` and of ``megamoe.reference(..., serial=True)``
(the generating script sits beside it) and ``tests/test_oracle_golden.py`` checks the functions
below against them bit for bit.
"""

from __future__ import annotations

import torch

from . import moe_oracle as O

MX_BLOCK = 32          # weights: input channels per E8M0 scale (megabench/tasks/quantization.py:10)
ACT_BLOCK = 32         # activations: channels per E8M0 scale (megabench/tasks/megamoe.py:37)
E2M1_MAGNITUDES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)   # code & 7; code & 8 is the sign


def unpack_mxfp4(blocks: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """uint8 [..., K/32, 16] codes (low nibble = even channel) and uint8 [..., K/32] biased
    exponents -> fp32 [..., K]; value = (+-magnitude) * 2**(scale - 127), scale 255 = NaN.

    megabench/tasks/quantization.py:40-51.
    """
    assert blocks.dtype == torch.uint8 and scales.dtype == torch.uint8
    assert blocks.shape[:-1] == scales.shape and blocks.shape[-1] == MX_BLOCK // 2
    table = torch.tensor(E2M1_MAGNITUDES + tuple(-m for m in E2M1_MAGNITUDES), dtype=torch.float32, device=blocks.device)
    low, high = blocks & 15, blocks >> 4
    codes = torch.stack((low, high), dim=-1).reshape(*blocks.shape[:-1], MX_BLOCK)
    value = torch.ldexp(table[codes.long()], scales.to(torch.int32)[..., None] - 127)
    value = torch.where(scales[..., None] == 255, torch.full_like(value, float("nan")), value)
    return value.reshape(*blocks.shape[:-2], -1)


def pack_mxfp4(matrix: torch.Tensor):
    """fp32/bf16 [..., K] -> (codes uint8 [..., K/32, 16], scales uint8 [..., K/32]).

    Per 32 channels: exponent = ceil(log2(max(amax / 6, 2**-126))) clamped to [-126, 127];
    the values divided by 2**exponent round to the nearest E2M1 magnitude, ties to the even
    code. megabench/tasks/quantization.py:13-37.
    """
    assert matrix.shape[-1] % MX_BLOCK == 0
    groups = matrix.to(torch.float32).reshape(*matrix.shape[:-1], -1, MX_BLOCK)
    amax = groups.abs().amax(-1)
    exponent = torch.ceil(torch.log2(torch.clamp(amax / 6.0, min=2.0 ** -126))).clamp(-126, 127).to(torch.int32)
    scaled = torch.ldexp(groups, -exponent[..., None])
    mag = scaled.abs()
    # midpoints between neighbouring magnitudes; a value on a midpoint goes to the even code
    code = torch.zeros_like(mag, dtype=torch.int64)
    for i, (lo, hi) in enumerate(zip(E2M1_MAGNITUDES[:-1], E2M1_MAGNITUDES[1:])):
        mid = (lo + hi) / 2
        up_on_tie = i % 2 == 1          # lower code i is odd: the tie goes up to the even code i + 1
        code = code + ((mag >= mid) if up_on_tie else (mag > mid)).to(torch.int64)
    code = code | ((scaled < 0).to(torch.int64) << 3)
    code = code.to(torch.uint8)
    return code[..., 0::2] | (code[..., 1::2] << 4), (exponent + 127).to(torch.uint8)


def clamped_swiglu(l1: torch.Tensor, weights: torch.Tensor, limit: float) -> torch.Tensor:
    """bf16 [n, 2I] (gate columns, then up columns) -> fp32 [n, I].

    Gate clamped above and up both ways in bf16, fp32 g/(1+exp(-g))*u, times the row's routing
    weight. megabench/tasks/megamoe.py:116-122.
    """
    gate, up = l1.chunk(2, dim=-1)
    return O._silu_mul_clamped(gate, up, limit, weights)


def requantize(value: torch.Tensor) -> torch.Tensor:
    """fp32 -> E4M3 with E8M0 scales per 32 channels -> bf16. megabench/tasks/megamoe.py:125-128."""
    q, s = O.quantize_activation(value, group=ACT_BLOCK, scale_format="e8m0")
    return O.dequantize_activation(q, s, group=ACT_BLOCK).to(torch.bfloat16)


def experts(values: dict, rows_q, rows_s, local_ids, weights, limit: float, *, keep: dict | None = None):
    """Rows grouped per expert in arrival order, one pair of GEMMs per expert that is hit;
    operands dequantised to bf16, fp32 accumulation, bf16 results.

    megabench/tasks/megamoe.py:131-150. ``keep`` (tests) receives per expert the requantised
    SwiGLU output as bf16.
    """
    n_local = values["l1_blocks"].shape[0]
    hidden = values["l2_blocks"].shape[1]
    out = torch.empty((rows_q.shape[0], hidden), dtype=torch.bfloat16, device=rows_q.device)
    order, counts = O.expert_order(local_ids, n_local)
    start = 0
    for e, n in enumerate(counts.tolist()):
        if not n:
            continue
        sel = order[start:start + n]
        start += n
        x = O.dequantize_activation(rows_q[sel], rows_s[sel], group=ACT_BLOCK).to(torch.bfloat16)
        w1 = unpack_mxfp4(values["l1_blocks"][e], values["l1_scales"][e]).to(torch.bfloat16)
        w2 = unpack_mxfp4(values["l2_blocks"][e], values["l2_scales"][e]).to(torch.bfloat16)
        a = requantize(clamped_swiglu(x @ w1.T, weights[sel], limit))
        if keep is not None:
            keep[e] = a
        out[sel] = a @ w2.T
    return out


def megamoe_layer(values: dict, topk: int, limit: float, *, keep: dict | None = None) -> dict:
    """All experts on one rank (the reference's ``serial=True``).

    values: x e4m3 [T, H] + x_scales uint8 [T, H/32]; topk_idx int64 [T, topk]; topk_weights
    fp32 [T, topk]; l1_blocks uint8 [E, 2I, H/32, 16] + l1_scales [E, 2I, H/32]; l2_blocks
    [E, H, I/32, 16] + l2_scales [E, H, I/32]. Returns y bf16 [T, H] and ``order`` (the stable
    grouping of the flattened ids by expert). megabench/tasks/megamoe.py:153-182.
    """
    tokens = values["x"].shape[0]
    flat = values["topk_idx"].reshape(-1)
    # one rank owns everything: the owner sort is the identity and rows arrive in (token, slot) order
    source = torch.div(torch.arange(flat.numel(), device=flat.device), topk, rounding_mode="floor")
    out = experts(values, values["x"][source], values["x_scales"][source], flat,
                  values["topk_weights"].reshape(-1), limit, keep=keep)
    slots = out.reshape(tokens, topk, -1)
    acc = torch.zeros((tokens, slots.shape[-1]), dtype=torch.float32, device=slots.device)
    for s in range(topk):
        acc = acc + slots[:, s].to(torch.float32)
    return {"y": acc.to(torch.bfloat16), "order": O.expert_order(flat, values["l1_blocks"].shape[0])[0]}
