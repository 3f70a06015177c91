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


def test_plugin_accepts_the_execution_context_of_the_reference_harness(single_rank_group):
    # megabench/harness/distributed.py:68-74 hands build() the case dict with case["execution"]; the
    # run it returns is backed by the expert-parallel layer (here a group of one rank)
    from vibe_megakernel_b200 import submission
    from vibe_megakernel_b200.ep import EpMoeLayer
    from vibe_megakernel_b200.layer import LayerConfig, MoeLayer
    geo = H.small_geometries()["kimi_small"]
    tokens = 24
    case = {"id": "fp8-moe-layer-kimi-small-ep1", "family": "fp8_moe_layer", "model": geo.name, "phase": "moe_layer",
            "gpus": 1, "tp": 1, "ep": 1,
            "params": {"tokens": tokens, "hidden": geo.hidden, "intermediate": geo.inter, "experts": geo.experts,
                       "topk": geo.topk, "shared_experts": geo.shared, "router_groups": geo.n_group,
                       "router_top_groups": geo.topk_group},
            "moe": {"scoring": geo.scoring, "scaling": geo.scaling},
            "execution": {"rank": 0, "world_size": 1, "tp_rank": 0, "ep_rank": 0, "backend": dist.get_backend(),
                          "device": "cuda:0", "tp_group": None, "ep_group": None}}
    run = submission.build(case)
    assert isinstance(run.layer, EpMoeLayer)
    try:
        values = H.to_device(synthetic.make_inputs(geo, tokens, 3, "cpu"), "cuda")
        before = {k: v.clone() for k, v in values.items()}
        got = run(values)
        assert run.layer.launches() == 8       # router 2, dispatch, grouping, gather, two GEMMs (the second sends the rows home), combine
        want = MoeLayer(LayerConfig.from_geometry(geo), max_tokens=tokens).forward(values, check_status=True)
        assert set(got) == {"y", "expert_ids", "order"}
        assert torch.equal(got["y"], want["y"]) and torch.equal(got["expert_ids"], want["expert_ids"])
        # one owner: the stable order by owning rank is the identity (megabench/tasks/megamoe.py:161-164)
        assert torch.equal(got["order"].cpu(), torch.arange(tokens * geo.topk))
        for k, v in values.items():
            assert torch.equal(v.view(torch.uint8), before[k].view(torch.uint8)), f"input {k} was modified"
    finally:
        run.layer.close()
    # without an execution context a case on several GPUs cannot be built
    with pytest.raises(ValueError):
        submission.build({**{k: v for k, v in case.items() if k != "execution"}, "gpus": 2})


@pytest.mark.parametrize("tokens,experts,topk,hidden,inter,limit", [(8, 16, 4, 256, 128, 10.0), (70, 8, 2, 512, 256, 3.0),
                                                                    (3, 64, 2, 256, 256, 0.0)])
def test_megamoe_single_rank_exchange_equals_the_serial_call(single_rank_group, tokens, experts, topk, hidden, inter, limit):
    # the expert-parallel form of the MXFP4 experts with one rank: every peer store lands in the rank's
    # own buffer; bits must equal the serial entry point (megabench/verify_megamoe.py:104-105), also
    # through the plugin file with the family name of the reference's cases
    from vibe_megakernel_b200 import megamoe, submission
    values = H.to_device(H.megamoe_inputs(tokens, experts, topk, hidden, inter, seed=tokens), "cuda")
    config = megamoe.MegaMoeConfig(hidden, inter, experts, topk, limit)
    serial = megamoe.MegaMoe(config, max_tokens=tokens).run(values, check_status=True, want_order=True)
    layer = megamoe.MegaMoeEp(config, max_tokens=tokens + 3)
    case = {"id": "megamoe-layer-test-ep1", "family": "megamoe_layer", "gpus": 1, "tp": 1, "ep": 1,
            "params": {"tokens": tokens, "hidden": hidden, "intermediate": inter, "experts": experts, "topk": topk,
                       "swiglu_limit": limit},
            "execution": {"rank": 0, "world_size": 1, "tp_rank": 0, "ep_rank": 0, "backend": dist.get_backend(),
                          "device": "cuda:0", "tp_group": None, "ep_group": None}}
    try:
        for _ in range(2):                                         # buffers and flags are reused from call to call
            got = layer.run(values, check_status=True, want_order=True)
            assert torch.equal(got["y"], serial["y"])
            assert torch.equal(got["order"].cpu(), torch.arange(tokens * topk))    # one owner: the identity
        assert layer.launches() == 7
        fewer = {k: (v[: max(1, tokens // 2)].contiguous() if k in ("x", "x_scales", "topk_idx", "topk_weights") else v)
                 for k, v in values.items()}
        got = layer.run(fewer, check_status=True)
        assert torch.equal(got["y"], serial["y"][: max(1, tokens // 2)])
    finally:
        layer.close()
    # the plugin file builds the expert-parallel layer from the case and the execution context
    from vibe_megakernel_b200.megamoe import MegaMoeEp
    run = submission.build(case)
    out = run(values)
    assert set(out) == {"y"} and torch.equal(out["y"], serial["y"])
    run_serial = submission.build({k: v for k, v in case.items() if k != "execution"})
    assert torch.equal(run_serial(values)["y"], serial["y"])


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
