"""CPU tests of the expert-parallel path: host-side sharding logic, the exchange-buffer layout
through the C ABI, and a real 2-rank Gloo run of the expert-parallel oracle against the serial one."""

import ctypes as C
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from vibe_megakernel_b200 import _cabi, ep

ROOT = Path(__file__).resolve().parent.parent


def test_contiguous_expert_ownership():
    assert list(ep.expert_range(256, 8, 3)) == list(range(96, 128))
    assert ep.owner_of(torch.tensor([0, 31, 32, 255]), 256, 8).tolist() == [0, 0, 1, 7]
    assert ep.exchange_capacity(16, 8) == 128
    with pytest.raises(ValueError):
        ep.expert_range(10, 4, 0)


def test_shards_are_slices_of_the_serial_problem():
    full = {"x": torch.arange(24.).reshape(6, 4), "gate": torch.arange(8.).reshape(4, 2), "router": torch.ones(4, 4),
            "shared_gate": torch.zeros(2, 2)}
    a = ep.shard_inputs(full, 4, 2, 0, 3)
    b = ep.shard_inputs(full, 4, 2, 1, 3)
    assert torch.equal(torch.cat([a["x"], b["x"]]), full["x"])
    assert torch.equal(torch.cat([a["gate"], b["gate"]]), full["gate"])
    assert a["router"] is full["router"] and b["shared_gate"] is full["shared_gate"]


def test_exchange_layout_through_the_c_abi():
    lib = _cabi.load()
    cfg = _cabi.Config(7168, 2048, 256, 8, 1, 1, 8, 4, 2.5, 8, 3, 0)
    lay = _cabi.EpLayout()
    assert lib.moe_ep_layout(C.byref(cfg), 16, C.byref(lay)) == 0
    # 8 ranks x 16 tokens x top-8 = 1024 routed rows over 256 experts: 4 per expert, narrow tiles
    assert lay.cap == 16 * 8 and lay.rows == 8 * lay.cap + 16 and lay.token_tile == 16
    offsets = [getattr(lay, n) for n in _cabi.EP_LAYOUT_OFFSETS[2:]]
    assert offsets == sorted(offsets) and all(o % 256 == 0 for o in offsets)
    assert lay.exchange_bytes >= lay.slots + 2 * (lay.cap + 16) * 7168
    assert lay.recv_s - lay.recv_q >= 8 * lay.cap * 7168
    too_many = _cabi.Config(7168, 2048, 256, 8, 1, 1, 8, 4, 2.5, 16, 0, 0)
    assert lib.moe_ep_layout(C.byref(too_many), 16, None) == -2
    uneven = _cabi.Config(7168, 2048, 250, 8, 1, 1, 1, 1, 2.5, 8, 0, 0)
    assert lib.moe_ep_layout(C.byref(uneven), 16, None) == -1
    assert lib.moe_ep_forward(C.byref(cfg), None, None, 1, 16, None, None, None, None, None, None, 0, 1, None) == -1
    # epochs start at 1 on a given local buffer: 0 is refused before anything is launched
    w = _cabi.Weights()
    for name in _cabi.WEIGHT_FIELDS:
        setattr(w, name, 256)
    dummy = C.c_void_p(256)
    peers = (C.c_void_p * 8)(*([256] * 8))
    assert lib.moe_ep_forward(C.byref(cfg), C.byref(w), dummy, 1, 16, dummy, None, None, None, peers, dummy, 1 << 40, 0,
                              None) == -1


def test_megamoe_exchange_layout_through_the_c_abi():
    # the reference's expert-parallel cases: 384 experts over 8 ranks, top-6 (megabench/cases.py:380-388)
    lib = _cabi.load()
    cfg = _cabi.Config(7168, 3072, 384, 6, 0, 0, 1, 1, 1.0, 8, 5, 0, 10.0, 1)
    lay = _cabi.EpLayout()
    assert lib.moe_mx_ep_layout(C.byref(cfg), 512, C.byref(lay)) == 0
    assert lay.cap == 512 * 6 and lay.rows == 8 * lay.cap and lay.token_tile == 128
    offsets = [getattr(lay, n) for n in _cabi.EP_LAYOUT_OFFSETS[2:]]
    assert offsets == sorted(offsets) and all(o % 256 == 0 for o in offsets)
    assert lay.recv_s - lay.recv_q >= lay.rows * 7168 and lay.slots - lay.recv_s >= lay.rows * 7168 // 32
    assert lay.recv_q - lay.recv_weight >= 4 * lay.rows
    assert lay.exchange_bytes >= lay.slots + 2 * lay.cap * 7168
    assert lib.moe_mx_ep_layout(C.byref(cfg), 683, None) == -2          # more than 32768 rows could arrive at one rank
    shared = _cabi.Config(7168, 3072, 384, 6, 1, 0, 1, 1, 1.0, 8, 5, 0, 10.0, 1)
    assert lib.moe_mx_ep_layout(C.byref(shared), 16, None) == -2
    assert lib.moe_mx_ep_forward(C.byref(cfg), None, None, None, None, None, 1, 16, None, None, None, None, 0, 1, None) == -1


def test_two_rank_gloo_run_equals_the_serial_oracle(tmp_path):
    out = tmp_path / "report.json"
    env = dict(os.environ, OMP_NUM_THREADS="1", CUDA_VISIBLE_DEVICES="")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--standalone", "--local-addr", "127.0.0.1",
           "--nproc-per-node", "2", str(ROOT / "tests" / "ep_gloo_worker.py"), str(out)]
    done = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-3000:]
    report = json.loads(out.read_text())
    assert set(report) == {"ds_small", "kimi_small", "qwen_small"}
    for name, checks in report.items():
        assert all(checks.values()), (name, checks)
