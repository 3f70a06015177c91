"""Host side of the FP8 MoE decode layer: torch owns memory and streams, the C ABI does the work.

The call signature and tensor names follow the reference's MoE-block tensors
(megabench/tasks/frontier.py:157-176) and its plugin protocol (megabench/README.md:83-104).
"""

from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

from . import _cabi


@dataclass(frozen=True)
class LayerConfig:
    hidden: int
    inter: int
    experts: int
    topk: int
    shared: int = 1
    scoring: str = "sigmoid"
    n_group: int = 1
    topk_group: int = 1
    scaling: float = 1.0
    # "tcgen05" (product path); check arms on CUDA cores: "simt" (the same arithmetic) and "simt_bf16"
    # (the reference's dequantize-then-bf16 rounding schedule, megabench/tasks/megamoe.py:146-149)
    gemm: str = "tcgen05"
    # The MegaMoE form of the expert MLP (megabench/tasks/megamoe.py:116-122,176-182): gate/up clamped
    # before SwiGLU, and the routing weight applied before the requantisation instead of at the combine.
    swiglu_limit: float = 0.0
    weight_before_requant: bool = False

    @classmethod
    def from_geometry(cls, geo, **overrides) -> "LayerConfig":
        base = dict(hidden=geo.hidden, inter=geo.inter, experts=geo.experts, topk=geo.topk, shared=geo.shared,
                    scoring=geo.scoring, n_group=geo.n_group, topk_group=geo.topk_group, scaling=geo.scaling)
        base.update(overrides)
        return cls(**base)

    def c_struct(self, world: int = 1, rank: int = 0) -> _cabi.Config:
        return _cabi.Config(self.hidden, self.inter, self.experts, self.topk, self.shared,
                            _cabi.SCORING[self.scoring], self.n_group, self.topk_group, float(self.scaling),
                            world, rank, _cabi.GEMM_IMPL[self.gemm],
                            float(self.swiglu_limit), int(self.weight_before_requant))


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _require(t: torch.Tensor, name: str, dtype, shape=None) -> torch.Tensor:
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor")
    if t.dtype != dtype:
        raise TypeError(f"{name} must be {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    if shape is not None and tuple(t.shape) != tuple(shape):
        raise ValueError(f"{name} must have shape {tuple(shape)}, got {tuple(t.shape)}")
    return t


def weights_struct(c: LayerConfig, values: dict[str, torch.Tensor], n_local: int) -> _cabi.Weights:
    """Checked device pointers of the weight tensors; ``n_local`` experts are held by this rank."""
    e, h, i = n_local, c.hidden, c.inter
    f8, f32 = torch.float8_e4m3fn, torch.float32
    w = _cabi.Weights()
    w.router = _require(values["router"], "router", f32, (c.experts, h)).data_ptr()
    bias = values.get("router_bias")
    w.router_bias = _ptr(_require(bias, "router_bias", f32, (c.experts,))) if bias is not None else None
    for name, shape, sshape in (("gate", (e, i, h), (e, i // 128, h // 128)), ("up", (e, i, h), (e, i // 128, h // 128)),
                                ("down", (e, h, i), (e, h // 128, i // 128))):
        setattr(w, name, _require(values[name], name, f8, shape).data_ptr())
        setattr(w, name + "_scale", _require(values[name + "_scale"], name + "_scale", f32, sshape).data_ptr())
    if c.shared:
        for name, shape, sshape in (("shared_gate", (i, h), (i // 128, h // 128)), ("shared_up", (i, h), (i // 128, h // 128)),
                                    ("shared_down", (h, i), (h // 128, i // 128))):
            setattr(w, name, _require(values[name], name, f8, shape).data_ptr())
            setattr(w, name + "_scale", _require(values[name + "_scale"], name + "_scale", f32, sshape).data_ptr())
    return w


class MoeLayer:
    """One GPU holding every expert. ``forward(values)`` takes the reference's tensor dict."""

    def __init__(self, config: LayerConfig, max_tokens: int = 128, device: torch.device | str | None = None):
        if not torch.cuda.is_available():
            raise RuntimeError("vibe_megakernel_b200 needs a CUDA device; there is no CPU path")
        self.config = config
        self.device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        self.lib = _cabi.load()
        self.cfg = config.c_struct()
        self._workspaces: dict[int, tuple[torch.Tensor, _cabi.Layout]] = {}
        self.max_tokens = max_tokens
        self.workspace(max_tokens)

    def layout(self, tokens: int) -> _cabi.Layout:
        lay = _cabi.Layout()
        _cabi.check("moe_workspace_layout", self.lib.moe_workspace_layout(C.byref(self.cfg), tokens, C.byref(lay)))
        return lay

    def workspace(self, tokens: int) -> tuple[torch.Tensor, _cabi.Layout]:
        got = self._workspaces.get(tokens)
        if got is None:
            lay = self.layout(tokens)
            buf = torch.empty(int(lay.total_bytes) + 256, dtype=torch.uint8, device=self.device)
            skew = (-buf.data_ptr()) % 256
            got = (buf[skew:skew + int(lay.total_bytes)], lay)
            self._workspaces[tokens] = got
        return got

    def weights_struct(self, values: dict[str, torch.Tensor]) -> _cabi.Weights:
        return weights_struct(self.config, values, self.config.experts)

    def forward(self, values: dict[str, torch.Tensor], *, check_status: bool = False) -> dict[str, torch.Tensor]:
        c = self.config
        x = _require(values["x"], "x", torch.bfloat16)
        if x.dim() != 2 or x.shape[1] != c.hidden:
            raise ValueError(f"x must be [tokens, {c.hidden}]")
        tokens = x.shape[0]
        ws, lay = self.workspace(tokens)
        w = self.weights_struct(values)
        y = torch.empty_like(x)
        ids = torch.empty((tokens, c.topk), dtype=torch.int64, device=x.device)
        tw = torch.empty((tokens, c.topk), dtype=torch.float32, device=x.device)
        order = torch.empty((tokens * c.topk,), dtype=torch.int64, device=x.device)
        stream = torch.cuda.current_stream(x.device).cuda_stream
        rc = self.lib.moe_layer_forward(C.byref(self.cfg), C.byref(w), x.data_ptr(), tokens, y.data_ptr(), ids.data_ptr(),
                                        tw.data_ptr(), order.data_ptr(), ws.data_ptr(), ws.numel(), stream)
        _cabi.check("moe_layer_forward", rc)
        if check_status:
            self.check_device_status(tokens)
        return {"y": y, "expert_ids": ids, "topk_weights": tw, "order": order}

    __call__ = forward

    def block_forward(self, values: dict[str, torch.Tensor], norm_weight: torch.Tensor, eps: float = 1e-6, *,
                      weight_in_fp32: bool = False, check_status: bool = False) -> dict[str, torch.Tensor]:
        """The layer between the RMSNorm of the residual stream ``values["x"]`` and the residual add:
        ``x_out = x + layer(rms(x, norm_weight, eps))`` (megabench/tasks/frontier.py:335-354)."""
        c = self.config
        x = _require(values["x"], "x", torch.bfloat16)
        if x.dim() != 2 or x.shape[1] != c.hidden:
            raise ValueError(f"x must be [tokens, {c.hidden}]")
        gamma = _require(norm_weight, "norm_weight", torch.bfloat16, (c.hidden,))
        tokens = x.shape[0]
        ws, lay = self.workspace(tokens)
        w = self.weights_struct(values)
        out = torch.empty_like(x)
        ids = torch.empty((tokens, c.topk), dtype=torch.int64, device=x.device)
        tw = torch.empty((tokens, c.topk), dtype=torch.float32, device=x.device)
        order = torch.empty((tokens * c.topk,), dtype=torch.int64, device=x.device)
        stream = torch.cuda.current_stream(x.device).cuda_stream
        rc = self.lib.moe_block_forward(C.byref(self.cfg), C.byref(w), x.data_ptr(), gamma.data_ptr(), float(eps),
                                        1 if weight_in_fp32 else 0, tokens, out.data_ptr(), ids.data_ptr(),
                                        tw.data_ptr(), order.data_ptr(), ws.data_ptr(), ws.numel(), stream)
        _cabi.check("moe_block_forward", rc)
        if check_status:
            self.check_device_status(tokens)
        return {"x": out, "expert_ids": ids, "topk_weights": tw, "order": order}

    def check_device_status(self, tokens: int) -> None:
        ws, _ = self.workspace(tokens)
        detail = C.c_int32(0)
        stream = torch.cuda.current_stream(self.device).cuda_stream
        rc = self.lib.moe_device_status(ws.data_ptr(), stream, C.byref(detail))
        if rc != 0:
            raise _cabi.MoeError("device status", rc, detail.value)

    def launches(self) -> int:
        return int(self.lib.moe_last_launch_count())

    STAGES = ("router", "permutation", "quantiser", "gate_up_gemm", "down_gemm", "combine")

    def profile(self, on: bool) -> None:
        """Record CUDA events between the stages of later ``forward`` calls made by this thread."""
        self.lib.moe_profile_enable(1 if on else 0)

    def stage_ms(self) -> dict[str, float]:
        """Durations of the stages of the last profiled ``forward`` call (waits for it)."""
        buf = (C.c_float * len(self.STAGES))()
        _cabi.check("moe_profile_read", self.lib.moe_profile_read(buf, len(self.STAGES)))
        return dict(zip(self.STAGES, (float(v) for v in buf)))

    # ---- stage entry points (unit parity) --------------------------------------------
    def route(self, x: torch.Tensor, router: torch.Tensor, bias: torch.Tensor | None):
        c = self.config
        tokens = x.shape[0]
        ws, _ = self.workspace(tokens)
        ids = torch.empty((tokens, c.topk), dtype=torch.int64, device=x.device)
        tw = torch.empty((tokens, c.topk), dtype=torch.float32, device=x.device)
        stream = torch.cuda.current_stream(x.device).cuda_stream
        rc = self.lib.moe_route(C.byref(self.cfg), _require(x, "x", torch.bfloat16).data_ptr(),
                                _require(router, "router", torch.float32).data_ptr(), _ptr(bias), tokens,
                                ids.data_ptr(), tw.data_ptr(), ws.data_ptr(), ws.numel(), stream)
        _cabi.check("moe_route", rc)
        return ids, tw

    def scratch(self, tokens: int, name: str) -> torch.Tensor:
        """A view of one scratch array of the last call with ``tokens`` rows (tests only)."""
        ws, lay = self.workspace(tokens)
        c = self.config
        rows = lay.rows
        spec = {
            "logits": (lay.logits, torch.float32, (tokens, c.experts)),
            "counts": (lay.counts, torch.int32, (c.experts + 1,)),
            "offsets": (lay.offsets, torch.int32, (c.experts + 2,)),
            "n_chunks": (lay.n_chunks, torch.int32, (1,)),
            "chunks": (lay.chunks, torch.int32, (lay.max_chunks, 4)),
            "row_token": (lay.row_token, torch.int32, (rows,)),
            "row_dest": (lay.row_dest, torch.int32, (rows,)),
            "xq": (lay.xq, torch.uint8, (rows, c.hidden)),
            "xs": (lay.xs, torch.float32, (rows, c.hidden // 128)),
            "aq": (lay.aq, torch.uint8, (rows, c.inter)),
            "as": (lay.as_, torch.float32, (rows, c.inter // 128)),
            "slots": (lay.slots, torch.bfloat16, (rows, c.hidden)),
        }[name]
        off, dtype, shape = spec
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        return ws[off:off + nbytes].view(dtype).view(shape)


_experts_scratch: dict = {}


def experts_forward(config: LayerConfig, values: dict[str, torch.Tensor], rows_q: torch.Tensor, rows_scale: torch.Tensor,
                    local_ids: torch.Tensor | None, *, world: int = 1, rank: int = 0) -> torch.Tensor:
    """Local experts over quantised rows (the reference's ``experts()``, megabench/tasks/megamoe.py:131-150):
    bf16 rows [n, H] in input order. ``local_ids`` int32 [n], or None for the shared expert."""
    lib = _cabi.load()
    n = rows_q.shape[0]
    h = config.hidden
    rows_q = _require(rows_q.view(torch.uint8), "rows_q", torch.uint8, (n, h))
    rows_scale = _require(rows_scale, "rows_scale", torch.float32, (n, h // 128))
    if local_ids is not None:
        local_ids = _require(local_ids, "local_ids", torch.int32, (n,))
    out = torch.empty((n, h), dtype=torch.bfloat16, device=rows_q.device)
    if n == 0:
        return out
    cfg = config.c_struct(world, rank)
    need = C.c_uint64(0)
    _cabi.check("moe_experts_workspace", lib.moe_experts_workspace(C.byref(cfg), n, C.byref(need)))
    key = (rows_q.device, int(need.value))
    ws = _experts_scratch.get(key)
    if ws is None:
        buf = torch.empty(int(need.value) + 256, dtype=torch.uint8, device=rows_q.device)
        skew = (-buf.data_ptr()) % 256
        ws = _experts_scratch[key] = buf[skew:skew + int(need.value)]
    n_local = config.experts // world
    w = _cabi.Weights()
    f8, f32 = torch.float8_e4m3fn, torch.float32
    i = config.inter
    names = (("shared_gate", (i, h)), ("shared_up", (i, h)), ("shared_down", (h, i))) if local_ids is None else (
        ("gate", (n_local, i, h)), ("up", (n_local, i, h)), ("down", (n_local, h, i)))
    for name, shape in names:
        setattr(w, name, _require(values[name], name, f8, shape).data_ptr())
        setattr(w, name + "_scale", _require(values[name + "_scale"], name + "_scale", f32).data_ptr())
    rc = lib.moe_experts_forward(C.byref(cfg), C.byref(w), rows_q.data_ptr(), rows_scale.data_ptr(), _ptr(local_ids), n,
                                 out.data_ptr(), ws.data_ptr(), ws.numel(), torch.cuda.current_stream(rows_q.device).cuda_stream)
    _cabi.check("moe_experts_forward", rc)
    return out


STATIC_ROUTE_MAX_TOKENS = 256


def route_static(config: LayerConfig, x: torch.Tensor, router: torch.Tensor, bias: torch.Tensor | None,
                 ids: torch.Tensor, weights: torch.Tensor) -> None:
    """Router into caller-owned ``ids`` (int64 [T, topk]) and ``weights`` (fp32 [T, topk]) without
    any workspace: for hosts that may not allocate device memory. The scratch is a static device
    array inside the library, shared by every call on the GPU (calls that can overlap on the GPU
    race; keep them on one stream), and at most ``STATIC_ROUTE_MAX_TOKENS`` tokens are accepted.
    The first call on a device does a one-time address look-up: make it outside stream capture."""
    lib = _cabi.load()
    tokens = x.shape[0]
    _require(x, "x", torch.bfloat16, (tokens, config.hidden))
    _require(router, "router", torch.float32, (config.experts, config.hidden))
    _require(ids, "ids", torch.int64, (tokens, config.topk))
    _require(weights, "weights", torch.float32, (tokens, config.topk))
    cfg = config.c_struct()
    rc = lib.moe_route_static(C.byref(cfg), x.data_ptr(), router.data_ptr(), _ptr(bias), tokens, ids.data_ptr(),
                              weights.data_ptr(), torch.cuda.current_stream(x.device).cuda_stream)
    _cabi.check("moe_route_static", rc)


def quantize_rows(x: torch.Tensor, gather: torch.Tensor | None = None):
    """e4m3 payload and fp32 scales of ``x`` [rows, width] (bf16 or fp32), per row per 128 channels."""
    lib = _cabi.load()
    if x.dtype not in (torch.bfloat16, torch.float32) or not x.is_cuda or not x.is_contiguous() or x.dim() != 2:
        raise ValueError("x must be a contiguous 2-D CUDA tensor of bf16 or fp32")
    rows = x.shape[0] if gather is None else gather.numel()
    width = x.shape[1]
    q = torch.empty((rows, width), dtype=torch.uint8, device=x.device)
    s = torch.empty((rows, (width + 127) // 128), dtype=torch.float32, device=x.device)
    if gather is not None:
        gather = _require(gather, "gather", torch.int32)
    rc = lib.moe_quantize_rows(x.data_ptr(), 0 if x.dtype == torch.bfloat16 else 1, rows, width, _ptr(gather),
                               q.data_ptr(), s.data_ptr(), torch.cuda.current_stream(x.device).cuda_stream)
    _cabi.check("moe_quantize_rows", rc)
    return q.view(torch.float8_e4m3fn), s


def group_rows(ids: torch.Tensor, n_local: int, id_base: int = 0):
    """Stable grouping of routed rows by expert: (order int64 [n], counts int32 [n_local])."""
    lib = _cabi.load()
    ids = _require(ids.reshape(-1), "ids", torch.int64)
    n = ids.numel()
    order = torch.empty((max(n, 1),), dtype=torch.int64, device=ids.device)
    counts = torch.empty((n_local + 1,), dtype=torch.int32, device=ids.device)
    rc = lib.moe_group_rows(ids.data_ptr(), n, id_base, n_local, order.data_ptr(), counts.data_ptr(),
                            torch.cuda.current_stream(ids.device).cuda_stream)
    _cabi.check("moe_group_rows", rc)
    return order[:n], counts[:n_local]


def combine(rows: torch.Tensor, weights: torch.Tensor, tokens: int, shared: bool) -> torch.Tensor:
    """Slot-order weighted sum of down-projection rows (plus the shared expert's row): bf16 [tokens, H].

    ``rows`` bf16 [tokens*topk (+ tokens), H] in slot order, ``weights`` fp32 [tokens, topk]."""
    lib = _cabi.load()
    rows = _require(rows, "rows", torch.bfloat16)
    weights = _require(weights, "weights", torch.float32)
    topk = weights.numel() // tokens
    if rows.dim() != 2 or rows.shape[0] != tokens * topk + (tokens if shared else 0):
        raise ValueError("rows must be [tokens*topk (+ tokens), H]")
    y = torch.empty((tokens, rows.shape[1]), dtype=torch.bfloat16, device=rows.device)
    rc = lib.moe_combine(rows.data_ptr(), weights.data_ptr(), tokens, topk, rows.shape[1], 1 if shared else 0,
                         y.data_ptr(), torch.cuda.current_stream(rows.device).cuda_stream)
    _cabi.check("moe_combine", rc)
    return y


def quantize_rows_ue8m0(x: torch.Tensor, block: int = 32):
    """e4m3 payload and power-of-two scales as biased exponents, one per ``block`` channels:
    (q float8_e4m3fn [rows, W], scales uint8 [rows, ceil(W/block)])."""
    lib = _cabi.load()
    if x.dtype not in (torch.bfloat16, torch.float32) or x.dim() != 2 or not x.is_cuda or not x.is_contiguous():
        raise TypeError("x must be a contiguous CUDA bf16/fp32 matrix")
    rows, width = x.shape
    q = torch.empty((rows, width), dtype=torch.uint8, device=x.device)
    s = torch.empty((rows, -(-width // block)), dtype=torch.uint8, device=x.device)
    rc = lib.moe_quantize_rows_ue8m0(x.data_ptr(), 0 if x.dtype == torch.bfloat16 else 1, rows, width, block,
                                     q.data_ptr(), s.data_ptr(), torch.cuda.current_stream(x.device).cuda_stream)
    _cabi.check("moe_quantize_rows_ue8m0", rc)
    return q.view(torch.float8_e4m3fn), s
