"""Expert-parallel CPU oracle. TEST INFRASTRUCTURE ONLY (see moe_oracle.py).

Restates the reference's expert-parallel skeleton with ``torch.distributed`` collectives (Gloo on
CPU): stable order of the routed rows by owning rank, count exchange, variable-size all-to-all of
payload / scales / expert ids, local experts over the arrivals grouped by a stable sort, all-to-all
back, un-permutation, fp32 slot-order weighted sum plus the home rank's shared expert.
megabench/tasks/megamoe.py:153-182, megabench/tasks/parallel.py:52-68, megabench/tasks/kimi_layer.py:189-230.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from . import moe_oracle as O


def _exchange(value: torch.Tensor, send: list[int], receive: list[int], group) -> torch.Tensor:
    """all_to_all_single with host-side split sizes along dim 0 (parallel.py:52-56)."""
    out = value.new_empty((sum(receive), *value.shape[1:]))
    dist.all_to_all_single(out, value.contiguous(), receive, send, group=group)
    return out


def _exchange_counts(owner: torch.Tensor, world: int, group):
    """Rows for every owner and rows arriving from every source (parallel.py:59-68)."""
    send = torch.bincount(owner, minlength=world)
    receive = torch.empty_like(send)
    dist.all_to_all_single(receive, send, group=group)
    return send.tolist(), receive.tolist()


def moe_layer_ep(spec: O.LayerSpec, values: dict, *, group=None, compute=torch.bfloat16) -> dict:
    """One rank's part of the layer. ``values`` holds this rank's token rows and its contiguous
    slice of the routed experts (gate/up/down with their scales), everything else replicated."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    local = spec.experts // world
    x = values["x"]
    t, h = x.shape
    ids, ws = O.route_tokens(spec, x, values["router"], values.get("router_bias"))
    flat = ids.reshape(-1)
    owner = torch.div(flat, local, rounding_mode="floor")
    order = torch.sort(owner, stable=True).indices                         # megamoe.py:164
    source = torch.div(order, spec.topk, rounding_mode="floor")
    xq, xs = O.quantize_activation(x.to(torch.bfloat16))
    send, receive = _exchange_counts(owner, world, group)
    rows = _exchange(xq.view(torch.uint8)[source], send, receive, group).view(torch.float8_e4m3fn)
    scales = _exchange(xs[source], send, receive, group)
    arrived = _exchange(flat[order], send, receive, group) - rank * local
    grouped, counts = O.expert_order(arrived, local)                       # megamoe.py:137-138
    computed = torch.empty((arrived.numel(), h), dtype=compute)
    start = 0
    for e, n in enumerate(counts.tolist()):
        if n == 0:
            continue
        sel = grouped[start:start + n]
        start += n
        computed[sel], _, _ = O.expert_mlp(rows[sel], scales[sel], values["gate"][e], values["gate_scale"][e],
                                           values["up"][e], values["up_scale"][e], values["down"][e],
                                           values["down_scale"][e], compute=compute)
    back = _exchange(computed, receive, send, group)                       # megamoe.py:175
    slots = torch.empty_like(back)
    slots[order] = back
    slots = slots.reshape(t, spec.topk, h)
    acc = torch.zeros((t, h), dtype=torch.float32)
    for s in range(spec.topk):
        acc = acc + slots[:, s].to(torch.float32) * ws[:, s:s + 1]
    if spec.shared:
        sh, _, _ = O.expert_mlp(xq, xs, values["shared_gate"], values["shared_gate_scale"], values["shared_up"],
                                values["shared_up_scale"], values["shared_down"], values["shared_down_scale"],
                                compute=compute)
        acc = acc + sh.to(torch.float32)
    return {"y": acc.to(torch.bfloat16), "expert_ids": ids, "topk_weights": ws, "owner_order": order,
            "received": torch.tensor(receive)}
