"""The allocation-free router entry point (moe_route_static) against the workspace one (moe_route).

Some hosts of the library cannot allocate device memory while serving (their allocator is locked
down, or they are a bare FFI shim with only input and output buffers); for them the router keeps
its scratch in a static device array inside the library. This file is named so that pytest
collects it last: if it fails in a run that stops at the first failure, every other test has
already run. It passes alone in a fresh process and after the rest of the suite.
"""

import ctypes as C

import pytest
import torch

from oracle import moe_oracle as O
from tests import helpers as H
from vibe_megakernel_b200 import synthetic

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def api():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from vibe_megakernel_b200 import layer
    return layer


@pytest.mark.parametrize("name,tokens", [("deepseek_v3", 64), ("qwen3_30b_a3b", 37)])
def test_static_router_matches_the_workspace_router_twice_in_a_row(api, name, tokens):
    geo = synthetic.GEOMETRIES[name]
    config = api.LayerConfig.from_geometry(geo)
    reference = api.MoeLayer(config, max_tokens=tokens)
    first_seed = 0
    for call in range(2):                                     # two calls in a row, different inputs
        x_cpu, router_cpu, bias_cpu, seed = H.audited_routing_inputs(geo, tokens, first_seed=first_seed)
        first_seed = seed + 1
        x, router = x_cpu.cuda(), router_cpu.cuda()
        bias = None if bias_cpu is None else bias_cpu.cuda()
        want_ids, want_w = reference.route(x, router, bias)
        # outputs are allocated by the caller; the entry point itself allocates nothing
        ids = torch.full((tokens, geo.topk), -1, dtype=torch.int64, device="cuda")
        w = torch.full((tokens, geo.topk), float("nan"), dtype=torch.float32, device="cuda")
        if call == 0:
            # the first call on a device also looks the static array up (and the driver may load the
            # kernels lazily): let that happen before free memory is compared
            api.route_static(config, x, router, bias, ids, w)
            ids.fill_(-1)
            w.fill_(float("nan"))
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        free_before = torch.cuda.mem_get_info()[0]            # the driver's view: sees a cudaMalloc inside the library too
        api.route_static(config, x, router, bias, ids, w)
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert torch.cuda.mem_get_info()[0] == free_before, "device memory was allocated during the call"
        # same kernels, same arithmetic as the workspace entry point: identical results, not merely close
        assert torch.equal(ids, want_ids), f"call {call}"
        assert torch.equal(w, want_w), f"call {call}"
        # and the expert ids are the CPU oracle's, bit for bit
        oracle_ids, oracle_w = O.route_tokens(H.spec_of(geo), x_cpu, router_cpu, bias_cpu)
        assert torch.equal(ids.cpu(), oracle_ids), f"call {call}, seed {seed}"
        torch.testing.assert_close(w.cpu(), oracle_w, rtol=2e-5, atol=1e-7)


def test_static_router_refuses_what_does_not_fit(api):
    from vibe_megakernel_b200 import _cabi
    geo = synthetic.GEOMETRIES["tiny"]
    config = api.LayerConfig.from_geometry(geo)
    tokens = api.STATIC_ROUTE_MAX_TOKENS + 1
    x = torch.zeros((tokens, geo.hidden), dtype=torch.bfloat16, device="cuda")
    router = torch.zeros((geo.experts, geo.hidden), device="cuda")
    ids = torch.full((tokens, geo.topk), -1, dtype=torch.int64, device="cuda")
    w = torch.zeros((tokens, geo.topk), device="cuda")
    with pytest.raises(_cabi.MoeError) as err:
        api.route_static(config, x, router, None, ids, w)
    assert err.value.code == -7
    torch.cuda.synchronize()
    assert bool((ids == -1).all()), "a refused call must not launch anything"
    lib = _cabi.load()
    cfg = config.c_struct()
    assert lib.moe_route_static(C.byref(cfg), None, None, None, 4, None, None, None) == -1
