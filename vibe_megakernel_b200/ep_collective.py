"""Comparison arm of the expert-parallel layer: the reference's host-driven exchange
(megabench/tasks/megamoe.py:153-182 over megabench/tasks/parallel.py:52-68 — a count exchange with a
host synchronisation, then ``all_to_all_single`` per tensor each way, NCCL on GPUs) around this
library's kernels (router, quantiser, experts). It exists to be measured against the in-kernel
peer-store exchange of ``ep.EpMoeLayer``; results are identical bit for bit.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from .layer import LayerConfig, MoeLayer, experts_forward, quantize_rows


class EpCollectiveLayer:
    def __init__(self, config: LayerConfig, max_tokens: int, group=None, device=None):
        if not dist.is_initialized():
            raise RuntimeError("torch.distributed must be initialised (one process per GPU)")
        self.config = config
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.local = config.experts // self.world
        self._router = MoeLayer(config, max_tokens=max_tokens, device=device)   # router entry point + its scratch

    def _exchange(self, value: torch.Tensor, send: list[int], receive: list[int]) -> torch.Tensor:
        out = value.new_empty((sum(receive), *value.shape[1:]))
        dist.all_to_all_single(out, value.contiguous(), receive, send, group=self.group)
        return out

    def forward(self, values: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
        c = self.config
        x = values["x"]
        tokens = x.shape[0]
        ids, w = self._router.route(x, values["router"], values.get("router_bias"))
        xq, xs = quantize_rows(x)
        flat = ids.reshape(-1)
        owner = torch.div(flat, self.local, rounding_mode="floor")
        order = torch.sort(owner, stable=True).indices
        source = torch.div(order, c.topk, rounding_mode="floor")
        send = torch.bincount(owner, minlength=self.world)
        receive = torch.empty_like(send)
        dist.all_to_all_single(receive, send, group=self.group)
        send, receive = send.tolist(), receive.tolist()                       # the host synchronisation
        rows = self._exchange(xq.view(torch.uint8)[source], send, receive)
        scales = self._exchange(xs[source], send, receive)
        arrived = self._exchange(flat[order], send, receive) - self.rank * self.local
        computed = experts_forward(c, values, rows, scales, arrived.to(torch.int32), world=self.world, rank=self.rank)
        back = self._exchange(computed, receive, send)
        slots = torch.empty_like(back)
        slots[order] = back
        slots = slots.view(tokens, c.topk, c.hidden)
        acc = torch.zeros((tokens, c.hidden), dtype=torch.float32, device=x.device)
        for s in range(c.topk):
            acc = acc + slots[:, s].float() * w[:, s:s + 1]
        if c.shared:
            acc = acc + experts_forward(c, values, xq, xs, None, world=self.world, rank=self.rank).float()
        return {"y": acc.to(torch.bfloat16), "expert_ids": ids, "topk_weights": w}

    __call__ = forward
