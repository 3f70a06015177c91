"""Expert-parallel host side: one process per GPU, experts sharded contiguously over the ranks.

Ownership and token split follow the reference (megabench/tasks/megamoe.py:100-105,
megabench/tasks/parallel.py:25-49): rank r owns experts [r*E/n, (r+1)*E/n) and its own rows of the
batch; router, bias and shared expert are replicated. ``torch.distributed`` is used only to set up
(exchange of the peer-memory handles, barriers); a layer call makes no collective call: rows travel
as peer stores issued by the kernels (csrc/ep.cu).
"""

from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from . import _cabi
from .layer import LayerConfig, _require, weights_struct


def expert_range(experts: int, world: int, rank: int) -> range:
    if experts % world:
        raise ValueError("experts must divide the number of ranks")
    local = experts // world
    return range(rank * local, (rank + 1) * local)


def owner_of(expert_ids: torch.Tensor, experts: int, world: int) -> torch.Tensor:
    """Rank that owns each expert id (megabench/tasks/megamoe.py:162)."""
    return torch.div(expert_ids, experts // world, rounding_mode="floor")


def exchange_capacity(max_tokens: int, topk: int) -> int:
    """Rows one source may send to one owner: every slot of every token."""
    return max_tokens * topk


EXPERT_TENSORS = ("gate", "gate_scale", "up", "up_scale", "down", "down_scale")


def shard_inputs(values: dict[str, torch.Tensor], experts: int, world: int, rank: int, tokens_per_rank: int) -> dict:
    """This rank's slice of a single-rank problem: its token rows and its experts; the rest replicated."""
    mine = expert_range(experts, world, rank)
    out = {}
    for name, t in values.items():
        if name == "x":
            out[name] = t[rank * tokens_per_rank:(rank + 1) * tokens_per_rank].contiguous()
        elif name in EXPERT_TENSORS:
            out[name] = t[mine.start:mine.stop].contiguous()
        else:
            out[name] = t
    return out


class PeerBuffers:
    """One peer-visible exchange buffer per rank and this rank's view of all of them.

    Allocation, CUDA IPC hand-over (the handles travel over ``group``) and release; ``pointers`` is the
    ``void*[world]`` array the C ABI takes. ``close`` is collective."""

    def __init__(self, lib, exchange_bytes: int, group, device: torch.device):
        self.lib, self.group, self.device = lib, group, device
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        with torch.cuda.device(device):
            own = C.c_void_p()
            handle = C.create_string_buffer(64)
            _cabi.check("moe_ep_buffer_alloc", lib.moe_ep_buffer_alloc(int(exchange_bytes), C.byref(own), handle))
            self._own = own.value
            handles: list = [None] * self.world
            dist.all_gather_object(handles, handle.raw, group=group)
            self._opened: list[int] = []
            ptrs = []
            for r, raw in enumerate(handles):
                if r == self.rank:
                    ptrs.append(self._own)
                    continue
                peer = C.c_void_p()
                _cabi.check("moe_ep_buffer_open", lib.moe_ep_buffer_open(C.create_string_buffer(raw, 64), C.byref(peer)))
                self._opened.append(peer.value)
                ptrs.append(peer.value)
            self.pointers = (C.c_void_p * self.world)(*ptrs)

    def close(self) -> None:
        if self._own is None:
            return
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        for p in self._opened:
            self.lib.moe_ep_buffer_close(p)
        dist.barrier(group=self.group)
        self.lib.moe_ep_buffer_free(self._own)
        self._own = None


def aligned_scratch(nbytes: int, device: torch.device) -> torch.Tensor:
    buf = torch.empty(int(nbytes) + 256, dtype=torch.uint8, device=device)
    skew = (-buf.data_ptr()) % 256
    return buf[skew:skew + int(nbytes)]


class EpMoeLayer:
    """The layer of one rank of an expert-parallel group (all ranks on one node, one GPU each)."""

    def __init__(self, config: LayerConfig, max_tokens: int, group=None, device: torch.device | str | None = None):
        if not torch.cuda.is_available():
            raise RuntimeError("vibe_megakernel_b200 needs a CUDA device; there is no CPU path")
        if not dist.is_initialized():
            raise RuntimeError("torch.distributed must be initialised (one process per GPU)")
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.config = config
        self.max_tokens = max_tokens
        self.device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        self.lib = _cabi.load()
        self.cfg = config.c_struct(self.world, self.rank)
        self.layout = _cabi.EpLayout()
        _cabi.check("moe_ep_layout", self.lib.moe_ep_layout(C.byref(self.cfg), max_tokens, C.byref(self.layout)))
        self._peers = PeerBuffers(self.lib, int(self.layout.exchange_bytes), group, self.device)
        self._exchange = self._peers.pointers
        self._local = aligned_scratch(int(self.layout.local_bytes), self.device)
        self.epoch = 0
        torch.cuda.synchronize(self.device)
        dist.barrier(group=group)

    def weights_struct(self, values: dict[str, torch.Tensor]) -> _cabi.Weights:
        return weights_struct(self.config, values, self.config.experts // self.world)

    def forward(self, values: dict[str, torch.Tensor], *, check_status: bool = False) -> dict[str, torch.Tensor]:
        c = self.config
        x = _require(values["x"], "x", torch.bfloat16)
        if x.dim() != 2 or x.shape[1] != c.hidden or not 1 <= x.shape[0] <= self.max_tokens:
            raise ValueError(f"x must be [1..{self.max_tokens}, {c.hidden}]")
        tokens = x.shape[0]
        w = self.weights_struct(values)
        y = torch.empty_like(x)
        ids = torch.empty((tokens, c.topk), dtype=torch.int64, device=x.device)
        tw = torch.empty((tokens, c.topk), dtype=torch.float32, device=x.device)
        order = torch.empty((tokens * c.topk,), dtype=torch.int64, device=x.device)
        self.epoch += 1
        stream = torch.cuda.current_stream(x.device).cuda_stream
        rc = self.lib.moe_ep_forward(C.byref(self.cfg), C.byref(w), x.data_ptr(), tokens, self.max_tokens, y.data_ptr(),
                                     ids.data_ptr(), tw.data_ptr(), order.data_ptr(), self._exchange,
                                     self._local.data_ptr(), self._local.numel(), self.epoch, stream)
        _cabi.check("moe_ep_forward", rc)
        if check_status:
            self.check_device_status()
        return {"y": y, "expert_ids": ids, "topk_weights": tw, "order": order}

    __call__ = forward

    def check_device_status(self) -> None:
        detail = C.c_int32(0)
        stream = torch.cuda.current_stream(self.device).cuda_stream
        rc = self.lib.moe_device_status(self._local.data_ptr(), stream, C.byref(detail))
        if rc != 0:
            raise _cabi.MoeError("device status", rc, detail.value)

    def launches(self) -> int:
        """Kernels the last ``forward`` of this thread launched."""
        return int(self.lib.moe_last_launch_count())

    def close(self) -> None:
        """Collective: every rank must call it, with no layer call in flight."""
        self._peers.close()
