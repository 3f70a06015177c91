"""ctypes binding of the C ABI declared in include/moe_b200.h (no torch types cross it)."""

from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

from . import build as _build

OK = 0
ERRORS = {-1: "bad argument", -2: "unsupported geometry", -3: "workspace too small",
          -4: "device wait timed out", -5: "tensor-map encode failed", -6: "device index out of range",
          -7: "request exceeds the static scratch limit"}
SCORING = {"softmax": 0, "sigmoid": 1, "sqrt_softplus": 2, "softmax_biased": 3}
GEMM_TCGEN05, GEMM_SIMT, GEMM_SIMT_BF16 = 0, 1, 2
GEMM_IMPL = {"tcgen05": GEMM_TCGEN05, "simt": GEMM_SIMT, "simt_bf16": GEMM_SIMT_BF16}


class Config(C.Structure):
    _fields_ = [("hidden", C.c_int32), ("inter", C.c_int32), ("n_experts", C.c_int32), ("topk", C.c_int32),
                ("n_shared", C.c_int32), ("scoring", C.c_int32), ("n_group", C.c_int32), ("topk_group", C.c_int32),
                ("routed_scaling", C.c_float), ("ep_world", C.c_int32), ("ep_rank", C.c_int32),
                ("gemm_impl", C.c_int32), ("swiglu_limit", C.c_float), ("weight_before_requant", C.c_int32)]


WEIGHT_FIELDS = ("router", "router_bias", "gate", "gate_scale", "up", "up_scale", "down", "down_scale",
                 "shared_gate", "shared_gate_scale", "shared_up", "shared_up_scale", "shared_down",
                 "shared_down_scale")


class Weights(C.Structure):
    _fields_ = [(name, C.c_void_p) for name in WEIGHT_FIELDS]


LAYOUT_OFFSETS = ("total_bytes", "status", "logits", "topk_ids", "topk_weights", "counts", "offsets", "n_chunks",
                  "chunks", "row_token", "row_dest", "xq", "xs", "aq", "as_", "slots")


class MxWeights(C.Structure):
    _fields_ = [(name, C.c_void_p) for name in ("l1_blocks", "l1_scales", "l2_blocks", "l2_scales")]


class LatentConfig(C.Structure):
    _fields_ = [("hidden", C.c_int32), ("latent", C.c_int32), ("inter", C.c_int32), ("n_experts", C.c_int32),
                ("topk", C.c_int32), ("n_shared", C.c_int32), ("latent_eps", C.c_float)]


LATENT_WEIGHT_FIELDS = ("router", "router_bias", "latent_down", "latent_up", "latent_norm", "gate_blocks", "gate_scales",
                        "up_blocks", "up_scales", "down_blocks", "down_scales", "shared_gate", "shared_up", "shared_down")


class LatentWeights(C.Structure):
    _fields_ = [(name, C.c_void_p) for name in LATENT_WEIGHT_FIELDS]


class Layout(C.Structure):
    _fields_ = [(name, C.c_uint64) for name in LAYOUT_OFFSETS] + [
        ("rows", C.c_int32), ("max_chunks", C.c_int32), ("token_tile", C.c_int32), ("reserved", C.c_int32)]


EP_LAYOUT_OFFSETS = ("exchange_bytes", "local_bytes", "flags_dispatch", "flags_return", "recv_count", "recv_expert",
                     "recv_slot", "recv_weight", "recv_q", "recv_s", "slots")


class EpLayout(C.Structure):
    _fields_ = [(name, C.c_uint64) for name in EP_LAYOUT_OFFSETS] + [
        ("cap", C.c_int32), ("rows", C.c_int32), ("max_chunks", C.c_int32), ("token_tile", C.c_int32)]


EXPORTS = {
    "moe_experts_workspace": (C.c_int, [C.POINTER(Config), C.c_int32, C.POINTER(C.c_uint64)]),
    "moe_experts_forward": (C.c_int, [C.POINTER(Config), C.POINTER(Weights), C.c_void_p, C.c_void_p, C.c_void_p,
                                      C.c_int32, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "moe_ep_layout": (C.c_int, [C.POINTER(Config), C.c_int32, C.POINTER(EpLayout)]),
    "moe_ep_forward": (C.c_int, [C.POINTER(Config), C.POINTER(Weights), C.c_void_p, C.c_int32, C.c_int32, C.c_void_p,
                                 C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(C.c_void_p), C.c_void_p, C.c_size_t,
                                 C.c_uint64, C.c_void_p]),
    "moe_mx_ep_layout": (C.c_int, [C.POINTER(Config), C.c_int32, C.POINTER(EpLayout)]),
    "moe_mx_ep_forward": (C.c_int, [C.POINTER(Config), C.POINTER(MxWeights), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                    C.c_int32, C.c_int32, C.c_void_p, C.c_void_p, C.POINTER(C.c_void_p), C.c_void_p,
                                    C.c_size_t, C.c_uint64, C.c_void_p]),
    "moe_ep_wait_flags": (C.c_int, [C.c_void_p, C.c_int32, C.c_uint64, C.c_uint64, C.c_void_p, C.c_void_p]),
    "moe_ep_buffer_alloc": (C.c_int, [C.c_size_t, C.POINTER(C.c_void_p), C.c_void_p]),
    "moe_ep_buffer_open": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p)]),
    "moe_ep_buffer_close": (C.c_int, [C.c_void_p]),
    "moe_ep_buffer_free": (C.c_int, [C.c_void_p]),
    "moe_workspace_layout": (C.c_int, [C.POINTER(Config), C.c_int32, C.POINTER(Layout)]),
    "moe_route": (C.c_int, [C.POINTER(Config), C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p,
                            C.c_void_p, C.c_size_t, C.c_void_p]),
    "moe_route_static": (C.c_int, [C.POINTER(Config), C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p,
                                   C.c_void_p, C.c_void_p]),
    "moe_quantize_rows": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p,
                                    C.c_void_p]),
    "moe_quantize_rows_ue8m0": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p,
                                          C.c_void_p]),
    "moe_group_rows": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p]),
    "moe_combine": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p,
                              C.c_void_p]),
    "moe_layer_forward": (C.c_int, [C.POINTER(Config), C.POINTER(Weights), C.c_void_p, C.c_int32, C.c_void_p,
                                    C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "moe_block_forward": (C.c_int, [C.POINTER(Config), C.POINTER(Weights), C.c_void_p, C.c_void_p, C.c_float, C.c_int32,
                                    C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t,
                                    C.c_void_p]),
    "moe_mx_workspace": (C.c_int, [C.POINTER(Config), C.c_int32, C.POINTER(C.c_uint64)]),
    "moe_mx_forward": (C.c_int, [C.POINTER(Config), C.POINTER(MxWeights), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                 C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "moe_latent_workspace": (C.c_int, [C.POINTER(LatentConfig), C.c_int32, C.POINTER(C.c_uint64)]),
    "moe_latent_forward": (C.c_int, [C.POINTER(LatentConfig), C.POINTER(LatentWeights), C.c_void_p, C.c_int32, C.c_void_p,
                                     C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "moe_device_status": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(C.c_int32)]),
    "moe_last_launch_count": (C.c_int, []),
    "moe_selfcheck_divisions": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p]),
    "moe_profile_enable": (C.c_int, [C.c_int32]),
    "moe_profile_read": (C.c_int, [C.POINTER(C.c_float), C.c_int32]),
}

_lib = None


def library_path() -> Path:
    """The in-tree library, or the one MOE_B200_LIB names (a build with other compile-time options)."""
    override = os.environ.get("MOE_B200_LIB")
    return Path(override) if override else _build.LIB


def load(build_if_missing: bool = True) -> C.CDLL:
    """Load the CUDA library; there is no fallback: a missing library is an error."""
    global _lib
    if _lib is not None:
        return _lib
    path = library_path()
    if not path.exists():
        if not build_if_missing:
            raise RuntimeError(f"{path} is missing: run `python -m vibe_megakernel_b200.build`")
        _build.build()
    lib = C.CDLL(str(path))
    for name, (res, args) in EXPORTS.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    _lib = lib
    return lib


class MoeError(RuntimeError):
    def __init__(self, where: str, code: int, detail: int | None = None):
        what = ERRORS.get(code, f"CUDA error {code}" if code > 0 else f"error {code}")
        super().__init__(f"{where}: {what}" + (f" (detail {detail})" if detail is not None else ""))
        self.code = code
        self.detail = detail


def check(where: str, code: int) -> None:
    if code != OK:
        raise MoeError(where, code)
