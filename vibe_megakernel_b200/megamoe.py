"""The routed experts in the MegaMoE-native formats (MXFP4 weights, E4M3 rows, E8M0 scales per 32
channels), host side of ``moe_mx_forward``.

Mirrors the reference task ``megabench/tasks/megamoe.py``: ``run(values)`` takes the tensors of its
``make_inputs`` (:86-113) under the same names and returns ``{"y": bf16 [T, H]}`` as its
``reference`` does (:153-182), all experts on one GPU (the reference's ``serial=True``).
"""

from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

from . import _cabi
from .layer import _require


@dataclass(frozen=True)
class MegaMoeConfig:
    hidden: int
    inter: int
    experts: int
    topk: int
    swiglu_limit: float = 10.0      # megabench/tasks/megamoe.py:38

    def c_struct(self, world: int = 1, rank: int = 0) -> _cabi.Config:
        return _cabi.Config(self.hidden, self.inter, self.experts, self.topk, 0, 0, 1, 1, 1.0, world, rank, 0,
                            float(self.swiglu_limit), 1)


class MegaMoe:
    def __init__(self, config: MegaMoeConfig, max_tokens: int, device: torch.device | str | None = None):
        if not torch.cuda.is_available():
            raise RuntimeError("the MegaMoE experts run on a CUDA device only")
        self.config = config
        self.max_tokens = max_tokens
        self.device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        self.lib = _cabi.load()
        self.cfg = config.c_struct()
        need = C.c_uint64(0)
        _cabi.check("moe_mx_workspace", self.lib.moe_mx_workspace(C.byref(self.cfg), max_tokens, C.byref(need)))
        buf = torch.empty(int(need.value) + 256, dtype=torch.uint8, device=self.device)
        skew = (-buf.data_ptr()) % 256
        self._buf = buf
        self.workspace = buf[skew:skew + int(need.value)]

    def run(self, values: dict[str, torch.Tensor], *, check_status: bool = False, want_order: bool = False) -> dict:
        c = self.config
        tokens = values["x"].shape[0]
        if tokens > self.max_tokens:
            raise ValueError(f"{tokens} tokens exceed the {self.max_tokens} this object was sized for")
        h, i, e, k = c.hidden, c.inter, c.experts, c.topk
        u8 = torch.uint8
        x = _require(values["x"].view(u8), "x", u8, (tokens, h))
        xs = _require(values["x_scales"], "x_scales", u8, (tokens, h // 32))
        idx = _require(values["topk_idx"], "topk_idx", torch.int64, (tokens, k))
        tw = _require(values["topk_weights"], "topk_weights", torch.float32, (tokens, k))
        w = _cabi.MxWeights()
        w.l1_blocks = _require(values["l1_blocks"], "l1_blocks", u8, (e, 2 * i, h // 32, 16)).data_ptr()
        w.l1_scales = _require(values["l1_scales"], "l1_scales", u8, (e, 2 * i, h // 32)).data_ptr()
        w.l2_blocks = _require(values["l2_blocks"], "l2_blocks", u8, (e, h, i // 32, 16)).data_ptr()
        w.l2_scales = _require(values["l2_scales"], "l2_scales", u8, (e, h, i // 32)).data_ptr()
        y = torch.empty((tokens, h), dtype=torch.bfloat16, device=self.device)
        order = torch.empty((tokens * k,), dtype=torch.int64, device=self.device) if want_order else None
        stream = torch.cuda.current_stream(self.device).cuda_stream
        rc = self.lib.moe_mx_forward(C.byref(self.cfg), C.byref(w), x.data_ptr(), xs.data_ptr(), idx.data_ptr(),
                                     tw.data_ptr(), tokens, y.data_ptr(), None if order is None else order.data_ptr(),
                                     self.workspace.data_ptr(), self.workspace.numel(), stream)
        _cabi.check("moe_mx_forward", rc)
        if check_status:
            detail = C.c_int32(0)
            rc = self.lib.moe_device_status(self.workspace.data_ptr(), stream, C.byref(detail))
            if rc != _cabi.OK:
                raise _cabi.MoeError("device status", rc, detail.value)
        out = {"y": y}
        if order is not None:
            out["order"] = order
        return out


class MegaMoeEp:
    """One rank of the expert-parallel form (megabench/tasks/megamoe.py:153-182 without ``serial``; the
    reference's cases run it on 8 ranks, megabench/cases.py:380-388). ``run(values)`` takes this rank's
    tensors as ``megamoe.make_inputs(case, seed, device, rank)`` makes them: its token rows with their
    routing (global expert ids) and the MXFP4 matrices of its experts. No collective call inside ``run``:
    rows travel as peer stores issued by the kernels; ``torch.distributed`` only carries the peer-memory
    handles at construction."""

    def __init__(self, config: MegaMoeConfig, max_tokens: int, group=None, device: torch.device | str | None = None):
        import torch.distributed as dist
        from .ep import PeerBuffers, aligned_scratch
        if not torch.cuda.is_available():
            raise RuntimeError("the MegaMoE experts run on a CUDA device only")
        if not dist.is_initialized():
            raise RuntimeError("torch.distributed must be initialised (one process per GPU)")
        self.config = config
        self.max_tokens = max_tokens
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        self.lib = _cabi.load()
        self.cfg = config.c_struct(self.world, self.rank)
        self.layout = _cabi.EpLayout()
        _cabi.check("moe_mx_ep_layout", self.lib.moe_mx_ep_layout(C.byref(self.cfg), max_tokens, C.byref(self.layout)))
        self._peers = PeerBuffers(self.lib, int(self.layout.exchange_bytes), group, self.device)
        self._local = aligned_scratch(int(self.layout.local_bytes), self.device)
        self.epoch = 0
        torch.cuda.synchronize(self.device)
        dist.barrier(group=group)

    def run(self, values: dict[str, torch.Tensor], *, check_status: bool = False, want_order: bool = False) -> dict:
        c = self.config
        tokens = values["x"].shape[0]
        if not 1 <= tokens <= self.max_tokens:
            raise ValueError(f"{tokens} tokens: this object was sized for 1..{self.max_tokens}")
        h, i, e, k = c.hidden, c.inter, c.experts // self.world, c.topk
        u8 = torch.uint8
        x = _require(values["x"].view(u8), "x", u8, (tokens, h))
        xs = _require(values["x_scales"], "x_scales", u8, (tokens, h // 32))
        idx = _require(values["topk_idx"], "topk_idx", torch.int64, (tokens, k))
        tw = _require(values["topk_weights"], "topk_weights", torch.float32, (tokens, k))
        w = _cabi.MxWeights()
        w.l1_blocks = _require(values["l1_blocks"], "l1_blocks", u8, (e, 2 * i, h // 32, 16)).data_ptr()
        w.l1_scales = _require(values["l1_scales"], "l1_scales", u8, (e, 2 * i, h // 32)).data_ptr()
        w.l2_blocks = _require(values["l2_blocks"], "l2_blocks", u8, (e, h, i // 32, 16)).data_ptr()
        w.l2_scales = _require(values["l2_scales"], "l2_scales", u8, (e, h, i // 32)).data_ptr()
        y = torch.empty((tokens, h), dtype=torch.bfloat16, device=self.device)
        order = torch.empty((tokens * k,), dtype=torch.int64, device=self.device) if want_order else None
        self.epoch += 1
        stream = torch.cuda.current_stream(self.device).cuda_stream
        rc = self.lib.moe_mx_ep_forward(C.byref(self.cfg), C.byref(w), x.data_ptr(), xs.data_ptr(), idx.data_ptr(),
                                        tw.data_ptr(), tokens, self.max_tokens, y.data_ptr(),
                                        None if order is None else order.data_ptr(), self._peers.pointers,
                                        self._local.data_ptr(), self._local.numel(), self.epoch, stream)
        _cabi.check("moe_mx_ep_forward", rc)
        if check_status:
            detail = C.c_int32(0)
            rc = self.lib.moe_device_status(self._local.data_ptr(), stream, C.byref(detail))
            if rc != _cabi.OK:
                raise _cabi.MoeError("device status", rc, detail.value)
        out = {"y": y}
        if order is not None:
            out["order"] = order
        return out

    def launches(self) -> int:
        return int(self.lib.moe_last_launch_count())

    def close(self) -> None:
        """Collective: every rank must call it, with no call in flight."""
        self._peers.close()
