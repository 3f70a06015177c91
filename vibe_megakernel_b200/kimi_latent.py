"""The MoE block of the Kimi-K3 decoder layer (latent experts), host side of ``moe_latent_forward``.

Mirrors ``moe(case, values, normalized, serial=True, group=None)`` of the reference
(megabench/tasks/kimi_layer.py:189-230): ``forward(values, normalized)`` takes the tensors of its
``make_inputs`` (:107-125) under the same names and returns what it returns, the block's output rows
and the expert ids sorted per token, plus the ids in choice order and the routing weights.
All experts live on one GPU (the reference's ``serial`` form).
"""

from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

from . import _cabi
from .layer import _require


@dataclass(frozen=True)
class LatentMoeConfig:
    hidden: int
    latent: int
    inter: int
    experts: int
    topk: int
    shared: int = 2
    latent_eps: float = 1e-5       # megabench/tasks/kimi_layer.py:227

    def c_struct(self) -> _cabi.LatentConfig:
        return _cabi.LatentConfig(self.hidden, self.latent, self.inter, self.experts, self.topk, self.shared,
                                  float(self.latent_eps))


class LatentMoe:
    def __init__(self, config: LatentMoeConfig, max_tokens: int, device: torch.device | str | None = None):
        if not torch.cuda.is_available():
            raise RuntimeError("the latent MoE block runs on a CUDA device only")
        self.config = config
        self.max_tokens = max_tokens
        self.device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        self.lib = _cabi.load()
        self.cfg = config.c_struct()
        need = C.c_uint64(0)
        _cabi.check("moe_latent_workspace", self.lib.moe_latent_workspace(C.byref(self.cfg), max_tokens, C.byref(need)))
        buf = torch.empty(int(need.value) + 256, dtype=torch.uint8, device=self.device)
        skew = (-buf.data_ptr()) % 256
        self.workspace = buf[skew:skew + int(need.value)]
        self._router32: tuple[int, torch.Tensor] | None = None

    def _router(self, router: torch.Tensor) -> torch.Tensor:
        """The reference widens its bf16 router per token (``values['router'].float()``); the library takes
        fp32, so the widened copy is made once per router tensor and kept."""
        if router.dtype == torch.float32:
            return router
        key = (router.data_ptr(), router._version)
        if self._router32 is None or self._router32[0] != key:
            self._router32 = (key, router.float())
        return self._router32[1]

    def forward(self, values: dict[str, torch.Tensor], normalized: torch.Tensor, *, check_status: bool = False) -> dict:
        c = self.config
        h, lh, i, e, k, s = c.hidden, c.latent, c.inter, c.experts, c.topk, c.shared
        bf, u8 = torch.bfloat16, torch.uint8
        x = _require(normalized, "normalized", bf)
        if x.dim() != 2 or x.shape[1] != h or not 1 <= x.shape[0] <= self.max_tokens:
            raise ValueError(f"normalized must be [1..{self.max_tokens}, {h}]")
        tokens = x.shape[0]
        w = _cabi.LatentWeights()
        router = self._router(values["router"])
        w.router = _require(router, "router", torch.float32, (e, h)).data_ptr()
        bias = values.get("router_bias")
        w.router_bias = None if bias is None else _require(bias, "router_bias", torch.float32, (e,)).data_ptr()
        w.latent_down = _require(values["latent_down"], "latent_down", bf, (lh, h)).data_ptr()
        w.latent_up = _require(values["latent_up"], "latent_up", bf, (h, lh)).data_ptr()
        w.latent_norm = _require(values["latent_norm"], "latent_norm", bf, (lh,)).data_ptr()
        for name, rows, cols in (("gate", i, lh), ("up", i, lh), ("down", lh, i)):
            setattr(w, name + "_blocks", _require(values[name + "_blocks"], name + "_blocks", u8, (e, rows, cols // 32, 16)).data_ptr())
            setattr(w, name + "_scales", _require(values[name + "_scales"], name + "_scales", u8, (e, rows, cols // 32)).data_ptr())
        w.shared_gate = _require(values["shared_gate"], "shared_gate", bf, (s * i, h)).data_ptr()
        w.shared_up = _require(values["shared_up"], "shared_up", bf, (s * i, h)).data_ptr()
        w.shared_down = _require(values["shared_down"], "shared_down", bf, (h, s * i)).data_ptr()
        y = torch.empty_like(x)
        ids = torch.empty((tokens, k), dtype=torch.int64, device=x.device)
        tw = torch.empty((tokens, k), dtype=torch.float32, device=x.device)
        stream = torch.cuda.current_stream(x.device).cuda_stream
        rc = self.lib.moe_latent_forward(C.byref(self.cfg), C.byref(w), x.data_ptr(), tokens, y.data_ptr(), ids.data_ptr(),
                                         tw.data_ptr(), self.workspace.data_ptr(), self.workspace.numel(), stream)
        _cabi.check("moe_latent_forward", rc)
        if check_status:
            detail = C.c_int32(0)
            rc = self.lib.moe_device_status(self.workspace.data_ptr(), stream, C.byref(detail))
            if rc != _cabi.OK:
                raise _cabi.MoeError("device status", rc, detail.value)
        return {"y": y, "expert_ids": ids, "sorted_ids": ids.sort(-1).values, "topk_weights": tw}

    def launches(self) -> int:
        return int(self.lib.moe_last_launch_count())
