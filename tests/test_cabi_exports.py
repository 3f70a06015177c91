"""CPU checks of the boundary: the library builds, loads and exports what include/moe_b200.h declares."""

import ctypes as C
import re
from pathlib import Path

from vibe_megakernel_b200 import _cabi

ROOT = Path(__file__).resolve().parent.parent


def declared_functions():
    text = (ROOT / "include" / "moe_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\bint\s+(moe_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _cabi.load()
    names = declared_functions()
    assert names, "no declarations found"
    for name in names:
        assert hasattr(lib, name), f"{name} is declared but not exported"
    assert sorted(_cabi.EXPORTS) == names, "ctypes binding and header disagree"


def test_struct_sizes_match_the_header():
    # 14 four-byte fields; 14 pointers; 16 uint64 + 4 int32
    assert C.sizeof(_cabi.Config) == 56
    assert C.sizeof(_cabi.Weights) == 14 * C.sizeof(C.c_void_p)
    assert C.sizeof(_cabi.Layout) == 16 * 8 + 16


def test_workspace_layout_and_argument_checks_need_no_gpu():
    lib = _cabi.load()
    cfg = _cabi.Config(7168, 2048, 256, 8, 1, 1, 8, 4, 2.5, 1, 0, 0)
    lay = _cabi.Layout()
    assert lib.moe_workspace_layout(C.byref(cfg), 64, C.byref(lay)) == 0
    assert lay.rows == 64 * 9 and lay.token_tile == 16          # 512 routed rows over 256 experts: narrow tiles
    offsets = [getattr(lay, n) for n in _cabi.LAYOUT_OFFSETS[1:]]
    assert offsets == sorted(offsets) and all(o % 256 == 0 for o in offsets)
    # behind the slot rows: the block entry point's normalised rows and the inverse permutation of large batches
    assert lay.total_bytes >= lay.slots + 2 * lay.rows * 7168 + 2 * 64 * 7168 + 4 * 64 * 8
    assert lib.moe_workspace_layout(C.byref(cfg), 1, C.byref(lay)) == 0 and lay.token_tile == 16
    assert lib.moe_workspace_layout(C.byref(cfg), 1024, C.byref(lay)) == 0 and lay.token_tile == 64   # 32 rows per expert
    dense = _cabi.Config(4096, 14336, 8, 2, 0, 0, 1, 1, 1.0, 1, 0, 0)     # long down contraction: room for partial tiles
    small = _cabi.Config(4096, 8192, 8, 2, 0, 0, 1, 1, 1.0, 1, 0, 0)
    big, ref = _cabi.Layout(), _cabi.Layout()
    assert lib.moe_workspace_layout(C.byref(dense), 16, C.byref(big)) == 0
    assert lib.moe_workspace_layout(C.byref(small), 16, C.byref(ref)) == 0
    assert big.row_token - big.chunks > ref.row_token - ref.chunks + 4 * 32 * 4 * 16 * 128
    bad = _cabi.Config(7000, 2048, 256, 8, 1, 1, 8, 4, 2.5, 1, 0, 0)
    assert lib.moe_workspace_layout(C.byref(bad), 64, None) == -2
    bad = _cabi.Config(7168, 2048, 256, 8, 1, 1, 7, 4, 2.5, 1, 0, 0)      # groups must divide experts
    assert lib.moe_workspace_layout(C.byref(bad), 64, None) == -1
    bad = _cabi.Config(7168, 2048, 256, 8, 2, 1, 8, 4, 2.5, 1, 0, 0)      # at most one shared expert
    assert lib.moe_workspace_layout(C.byref(bad), 64, None) == -2
    mega = _cabi.Config(7168, 2048, 256, 8, 1, 1, 8, 4, 2.5, 1, 0, 0, 7.0, 1)    # clamp, routing weight before the requantisation
    assert lib.moe_workspace_layout(C.byref(mega), 64, None) == 0
    bad = _cabi.Config(7168, 2048, 256, 8, 1, 1, 8, 4, 2.5, 1, 0, 0, -1.0, 0)
    assert lib.moe_workspace_layout(C.byref(bad), 64, None) == -1
    bad = _cabi.Config(7168, 2048, 256, 8, 1, 1, 8, 4, 2.5, 2, 0, 0, 7.0, 1)     # one-GPU entry points only
    assert lib.moe_workspace_layout(C.byref(bad), 64, None) == -2
    assert lib.moe_workspace_layout(None, 64, None) == -1
    assert lib.moe_layer_forward(C.byref(cfg), None, None, 64, None, None, None, None, None, 0, None) == -1


def test_megamoe_native_argument_checks_need_no_gpu():
    lib = _cabi.load()
    need = C.c_uint64(0)
    cfg = _cabi.Config(7168, 3072, 384, 6, 0, 0, 1, 1, 1.0, 1, 0, 0, 10.0, 1)       # megabench/cases.py:384-385
    assert lib.moe_mx_workspace(C.byref(cfg), 512, C.byref(need)) == 0
    rows = 512 * 6
    assert need.value >= rows * (7168 + 3072) + 2 * rows * 7168                       # grouped rows, requantised rows, slot rows
    assert lib.moe_mx_workspace(C.byref(cfg), 5462, C.byref(need)) == -2               # more than 32768 routed rows
    for bad in (_cabi.Config(7168, 3000, 384, 6, 0, 0, 1, 1, 1.0, 1, 0, 0, 10.0, 1),   # intermediate not a multiple of 128
                _cabi.Config(7168, 3072, 384, 6, 1, 0, 1, 1, 1.0, 1, 0, 0, 10.0, 1),   # no shared expert in this task
                _cabi.Config(7168, 3072, 384, 6, 0, 0, 1, 1, 1.0, 2, 0, 0, 10.0, 1)):  # one rank only
        assert lib.moe_mx_workspace(C.byref(bad), 8, C.byref(need)) == -2
    assert lib.moe_mx_workspace(C.byref(_cabi.Config(7168, 3072, 384, 500, 0, 0, 1, 1, 1.0, 1, 0, 0, 10.0, 1)), 8,
                                C.byref(need)) == -1                                   # topk above the expert count
    assert lib.moe_mx_forward(C.byref(cfg), None, None, None, None, None, 8, None, None, None, 0, None) == -1


def test_latent_moe_argument_checks_need_no_gpu():
    lib = _cabi.load()
    need = C.c_uint64(0)
    cfg = _cabi.LatentConfig(7168, 3584, 3072, 896, 16, 2, 1e-5)                       # megabench/cases.py:315-324
    assert lib.moe_latent_workspace(C.byref(cfg), 8, C.byref(need)) == 0
    rows2 = 2 * 8 * 16
    assert need.value >= rows2 * (3584 + 3072) + 2 * 8 * 16 * 3584                       # split rows, requantised rows, slot rows
    assert lib.moe_latent_workspace(C.byref(cfg), 1025, None) == -2                      # more than 16384 routed rows
    assert lib.moe_latent_workspace(C.byref(_cabi.LatentConfig(7168, 3500, 3072, 896, 16, 2, 1e-5)), 8, None) == -2
    assert lib.moe_latent_workspace(C.byref(_cabi.LatentConfig(7168, 3584, 3072, 2000, 16, 2, 1e-5)), 8, None) == -2
    assert lib.moe_latent_workspace(C.byref(_cabi.LatentConfig(7168, 3584, 3072, 896, 16, 0, 1e-5)), 8, None) == -1
    assert lib.moe_latent_forward(C.byref(cfg), None, None, 8, None, None, None, None, 0, None) == -1


def test_product_does_not_import_the_oracle():
    for path in (ROOT / "vibe_megakernel_b200").rglob("*.py"):
        assert "oracle" not in path.read_text().replace("the oracle", ""), path
