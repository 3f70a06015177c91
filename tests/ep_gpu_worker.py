"""Rank program of the multi-GPU expert-parallel test (one process per GPU, launched by
torch.distributed.run). Every rank also runs the whole problem on its own GPU with the one-GPU
layer; its expert-parallel rows must equal the matching rows of that result bit for bit, for
several calls in a row (fresh inputs every call, exchange buffers reused)."""

import json
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

from tests import helpers as H  # noqa: E402
from vibe_megakernel_b200 import ep, synthetic  # noqa: E402
from vibe_megakernel_b200.ep_collective import EpCollectiveLayer  # noqa: E402
from vibe_megakernel_b200.layer import LayerConfig, MoeLayer  # noqa: E402


def main(out_path: str) -> None:
    rank = int(os.environ["RANK"])
    local_rank = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local_rank)
    dist.init_process_group("cpu:gloo,cuda:nccl")
    world = dist.get_world_size()
    dev = torch.device("cuda", local_rank)
    report = {}
    for name, tokens_per_rank, calls in (("ds_small", 5, 3), ("kimi_small", 16, 2), ("qwen_small", 40, 2), ("tiny", 2, 2)):
        geo = H.small_geometries()[name]
        if geo.experts % world:
            continue
        config = LayerConfig.from_geometry(geo)
        layer = ep.EpMoeLayer(config, max_tokens=tokens_per_rank, device=dev)
        single = MoeLayer(config, max_tokens=tokens_per_rank * world, device=dev)
        collective = EpCollectiveLayer(config, max_tokens=tokens_per_rank, device=dev)   # NCCL all-to-all arm
        ok = True
        for call in range(calls):
            full = {k: v.to(dev) for k, v in synthetic.make_inputs(geo, tokens_per_rank * world, call, "cpu").items()}
            mine = ep.shard_inputs(full, geo.experts, world, rank, tokens_per_rank)
            got = layer.forward(mine, check_status=True)
            want = single.forward(full, check_status=True)
            rows = slice(rank * tokens_per_rank, (rank + 1) * tokens_per_rank)
            ok = ok and torch.equal(got["y"], want["y"][rows]) and torch.equal(got["expert_ids"], want["expert_ids"][rows])
            ok = ok and torch.equal(got["topk_weights"], want["topk_weights"][rows])
            owner = torch.div(got["expert_ids"].flatten(), geo.experts // world, rounding_mode="floor")
            ok = ok and torch.equal(got["order"], torch.sort(owner, stable=True).indices)   # megabench/tasks/megamoe.py:161-164
            alt = collective.forward(mine)
            ok = ok and torch.equal(alt["y"], got["y"]) and torch.equal(alt["expert_ids"], got["expert_ids"])
        flags = [None] * world
        dist.all_gather_object(flags, bool(ok))
        report[name] = flags
        layer.close()
    # the routed experts in the MegaMoE-native formats: expert-parallel == serial, bit for bit
    # (megabench/verify_megamoe.py:44-56,104-105), fresh inputs every call, buffers reused
    from vibe_megakernel_b200 import megamoe
    for name, (tokens_per_rank, experts, topk, hidden, inter, limit) in {
            "megamoe_dev": (8, 16, 4, 256, 128, 10.0), "megamoe_chunks": (40, 8, 2, 512, 256, 3.0)}.items():
        if experts % world:
            continue
        config = megamoe.MegaMoeConfig(hidden, inter, experts, topk, limit)
        layer = megamoe.MegaMoeEp(config, max_tokens=tokens_per_rank, device=dev)
        serial = megamoe.MegaMoe(config, max_tokens=tokens_per_rank * world, device=dev)
        ok = True
        local = experts // world
        for call in range(3):
            full = {k: v.to(dev) for k, v in H.megamoe_inputs(tokens_per_rank * world, experts, topk, hidden, inter,
                                                              seed=100 + call).items()}
            rows = slice(rank * tokens_per_rank, (rank + 1) * tokens_per_rank)
            mine = {k: (v[rows].contiguous() if k in ("x", "x_scales", "topk_idx", "topk_weights")
                        else v[rank * local:(rank + 1) * local].contiguous()) for k, v in full.items()}
            got = layer.run(mine, check_status=True, want_order=True)
            want = serial.run(full, check_status=True)
            ok = ok and torch.equal(got["y"], want["y"][rows])
            owner = torch.div(mine["topk_idx"].flatten(), local, rounding_mode="floor")
            ok = ok and torch.equal(got["order"], torch.sort(owner, stable=True).indices)
        flags = [None] * world
        dist.all_gather_object(flags, bool(ok))
        report[name] = flags
        layer.close()
    if rank == 0:
        Path(out_path).write_text(json.dumps(report))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main(sys.argv[1])
