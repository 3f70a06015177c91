"""GPU tests of the expert-parallel layer.

On one GPU the whole exchange path runs with a single rank (every peer store lands in the rank's
own buffer, every flag is already raised when the waiting kernel starts, so no kernel ever waits on
another): the result must equal the one-GPU layer bit for bit. With two or more GPUs the same is
checked across real ranks, one process per GPU.
"""

import json
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist

from tests import helpers as H
from vibe_megakernel_b200 import synthetic

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def single_rank_group():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    created = False
    if not dist.is_initialized():
        dist.init_process_group("gloo", init_method="tcp://127.0.0.1:29731", rank=0, world_size=1)
        created = True
    yield
    if created:
        dist.destroy_process_group()


@pytest.mark.parametrize("name,tokens", [("tiny", 4), ("ds_small", 19), ("kimi_small", 40), ("qwen_small", 130)])
def test_single_rank_exchange_path_equals_the_one_gpu_layer(single_rank_group, name, tokens):
    from vibe_megakernel_b200 import ep
    from vibe_megakernel_b200.layer import LayerConfig, MoeLayer
    geo = H.small_geometries()[name]
    config = LayerConfig.from_geometry(geo)
    layer = ep.EpMoeLayer(config, max_tokens=tokens)
    single = MoeLayer(config, max_tokens=tokens)
    try:
        for seed in (0, 1, 2):
            n = tokens if seed != 1 else max(1, tokens // 2)          # fewer rows than the buffers were sized for
            values = H.to_device(synthetic.make_inputs(geo, n, seed, "cpu"), "cuda")
            got = layer.forward(values, check_status=True)
            want = single.forward(values, check_status=True)
            assert torch.equal(got["expert_ids"], want["expert_ids"])
            assert torch.equal(got["topk_weights"], want["topk_weights"])
            assert torch.equal(got["y"], want["y"]), f"seed {seed}"
    finally:
        layer.close()


def test_deepseek_shape_single_rank_exchange(single_rank_group):
    from vibe_megakernel_b200 import ep
    from vibe_megakernel_b200.layer import LayerConfig, MoeLayer
    geo = synthetic.GEOMETRIES["deepseek_v3"]
    config = LayerConfig.from_geometry(geo)
    values = synthetic.make_inputs(geo, 64, 0, "cuda")
    layer = ep.EpMoeLayer(config, max_tokens=64)
    try:
        got = layer.forward(values, check_status=True)
        want = MoeLayer(config, max_tokens=64).forward(values, check_status=True)
        assert torch.equal(got["expert_ids"], want["expert_ids"])
        assert torch.equal(got["y"], want["y"])
    finally:
        layer.close()


def test_a_flag_nobody_raises_times_out_with_a_status_not_a_hang():
    """Failure detection without a GPU fault: the wait gives up after its (here 1 ms) limit, the kernel
    returns normally, the status word names the late peer, and the context stays usable."""
    import ctypes as C
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from vibe_megakernel_b200 import _cabi
    lib = _cabi.load()
    flags = torch.zeros(8, dtype=torch.int64, device="cuda")
    flags[:2] = 5                                       # peers 0 and 1 reported epoch 5, peer 2 never did
    status = torch.zeros(8, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.moe_ep_wait_flags(flags.data_ptr(), 3, 5, 1_000_000, status.data_ptr(), stream) == 0
    detail = C.c_int32(0)
    assert lib.moe_device_status(status.data_ptr(), stream, C.byref(detail)) == -4        # MOE_ERR_DEVICE_TIMEOUT
    assert detail.value == 202
    status.zero_()
    flags[2] = 5
    assert lib.moe_ep_wait_flags(flags.data_ptr(), 3, 5, 1_000_000, status.data_ptr(), stream) == 0
    assert lib.moe_device_status(status.data_ptr(), stream, C.byref(detail)) == 0
    assert float(torch.ones(4, device="cuda").sum()) == 4.0                                   # context still fine
    assert lib.moe_ep_wait_flags(flags.data_ptr(), 3, 5, 3_000_000_000, status.data_ptr(), stream) == -1   # limit is 2 s


def test_ranks_on_several_gpus_equal_the_one_gpu_layer(tmp_path):
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs at least two GPUs")
    world = max(n for n in (2, 4, 8) if n <= torch.cuda.device_count())
    out = tmp_path / "report.json"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--standalone", "--local-addr", "127.0.0.1",
           "--nproc-per-node", str(world), str(ROOT / "tests" / "ep_gpu_worker.py"), str(out)]
    done = subprocess.run(cmd, env=dict(os.environ), capture_output=True, text=True, timeout=900)
    assert done.returncode == 0, done.stderr[-3000:]
    report = json.loads(out.read_text())
    assert report, "no geometry ran"
    for name, flags in report.items():
        assert all(flags), (name, flags)
