"""CPU oracle for the Kimi-K3 latent MoE block. TEST INFRASTRUCTURE ONLY.

Restates, in plain torch on the host, the mixture-of-experts block of the reference's Kimi-K3
decoder layer (kamahori/vibe-megakernel, ``megabench/tasks/kimi_layer.py:189-230`` with
``serial=True``): per token a sigmoid top-k router, a bf16 down-projection into a latent width, routed
experts with MXFP4 weights over the bf16 latent rows and the ``situ`` activation
(``megabench/tasks/kimi.py:134-135``), an fp32 slot-order weighted sum, latent RMSNorm and
up-projection, plus shared experts on the full-width token. Only the test-suite, the smoke entry and
the CPU-baseline leg of the benchmark may import this file; the product never does.

Parity is pinned: ``tests/golden/kimi_latent.npz`` holds inputs and outputs of the reference's own
``kimi_layer.moe(case, values, normalized, serial=True, group=None)`` on two reduced geometries (the
generating script sits beside it) and ``tests/test_oracle_golden.py`` checks the functions below
against them bit for bit.
"""

from __future__ import annotations

import torch

from . import megamoe_oracle as M
from . import moe_oracle as O


def situ(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """4*tanh(g/4) * sigmoid(g) * 25*tanh(u/25) in fp32, rounded to the inputs' dtype.
    megabench/tasks/kimi.py:134-135."""
    g, u = gate.float(), up.float()
    return (4 * torch.tanh(g / 4) * g.sigmoid() * (25 * torch.tanh(u / 25))).to(gate.dtype)


def latent_experts(values: dict, rows: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """Local MXFP4 experts over bf16 latent rows: weights dequantised to bf16, bf16 GEMMs with fp32
    accumulation, ``situ`` between them. megabench/tasks/kimi_layer.py:175-186."""
    out = torch.empty_like(rows)
    for expert in ids.unique().tolist():
        sel = (ids == expert).nonzero().flatten()

        def weight(key):
            return M.unpack_mxfp4(values[key + "_blocks"][expert], values[key + "_scales"][expert]).to(torch.bfloat16)
        x = rows[sel]
        out[sel] = situ(x @ weight("gate").T, x @ weight("up").T) @ weight("down").T
    return out


def latent_moe(values: dict, normalized: torch.Tensor, topk: int, latent_eps: float = 1e-5) -> dict:
    """All experts on one rank. ``normalized`` bf16 [T, H] (the layer's post-norm tokens).

    values: router bf16 [E, H]; router_bias fp32 [E]; latent_down bf16 [L, H]; latent_up bf16 [H, L];
    latent_norm bf16 [L]; gate/up MXFP4 [E, I, L/32, 16] + scales [E, I, L/32]; down [E, L, I/32, 16] +
    scales; shared_gate/shared_up bf16 [S*I, H]; shared_down bf16 [H, S*I].
    Returns y bf16 [T, H], expert_ids int64 [T, topk] in choice order, sorted_ids (what the reference
    returns), topk_weights fp32 and ``order`` (stable grouping of the flattened ids by expert).
    megabench/tasks/kimi_layer.py:189-230.
    """
    routes = [O.route_sigmoid_grouped(values["router"].float() @ token.float(), values["router_bias"], topk, 1, 1, 1.0)
              for token in normalized]
    indices = torch.stack([i for i, _ in routes])
    weights = torch.stack([w for _, w in routes])
    latent = torch.stack([values["latent_down"] @ token for token in normalized])
    flat = indices.flatten()
    rows = latent.repeat_interleave(topk, 0)           # one owner: the order by owner is the identity
    output = latent_experts(values, rows, flat)
    combined = output.view(normalized.shape[0], topk, -1)
    results = []
    for row, token in enumerate(normalized):
        expert_sum = torch.zeros(latent.shape[1], device=token.device)
        for slot in range(topk):
            expert_sum = expert_sum + combined[row, slot].float() * weights[row, slot]
        routed = values["latent_up"] @ O.rms_norm(expert_sum.to(torch.bfloat16), values["latent_norm"], latent_eps)
        shared = values["shared_down"] @ situ(values["shared_gate"] @ token, values["shared_up"] @ token)
        results.append(routed + shared)
    return {"y": torch.stack(results), "expert_ids": indices, "sorted_ids": indices.sort(-1).values,
            "topk_weights": weights, "order": O.expert_order(flat, values["gate_blocks"].shape[0])[0],
            "latent": latent, "expert_rows": output}
