"""Rank program of the CPU expert-parallel test (launched by torch.distributed.run, Gloo backend).

Every rank builds the same small single-rank problem, keeps its shard (the product's host-side
sharding helper), runs the expert-parallel oracle over real collectives and rank 0 checks that the
union of the ranks' results equals the serial oracle bit for bit, as the reference's verifier does
(megabench/verify_megamoe.py:44-56,104-105).
"""

import json
import sys
from pathlib import Path

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

from oracle import ep_oracle, moe_oracle as O  # noqa: E402
from tests import helpers as H  # noqa: E402
from vibe_megakernel_b200 import ep, synthetic  # noqa: E402


def main(out_path: str) -> None:
    dist.init_process_group("gloo")
    world, rank = dist.get_world_size(), dist.get_rank()
    torch.set_num_threads(1)
    report = {}
    for name, tokens_per_rank in (("ds_small", 5), ("kimi_small", 4), ("qwen_small", 7)):
        geo = H.small_geometries()[name]
        spec = H.spec_of(geo)
        full = synthetic.make_inputs(geo, tokens_per_rank * world, 0, "cpu")
        mine = ep.shard_inputs(full, geo.experts, world, rank, tokens_per_rank)
        # a rank's shard is what the generator makes for that rank directly
        direct = synthetic.make_inputs(geo, tokens_per_rank, 0, "cpu", rank=rank, world=world)
        same = all(torch.equal(mine[k].view(torch.uint8), direct[k].view(torch.uint8)) for k in mine)
        got = ep_oracle.moe_layer_ep(spec, mine)
        ys = [torch.empty_like(got["y"]) for _ in range(world)]
        dist.all_gather(ys, got["y"])
        ids = [torch.empty_like(got["expert_ids"]) for _ in range(world)]
        dist.all_gather(ids, got["expert_ids"])
        received = [torch.empty_like(got["received"]) for _ in range(world)]
        dist.all_gather(received, got["received"])
        if rank == 0:
            serial = O.moe_layer(spec, full)
            owners = ep.owner_of(serial["expert_ids"].reshape(-1), geo.experts, world)
            want_received = torch.stack([torch.bincount(owners[r * tokens_per_rank * geo.topk:(r + 1) * tokens_per_rank * geo.topk],
                                                        minlength=world) for r in range(world)]).T
            report[name] = {
                "shard_equals_direct": bool(same),
                "y_bitwise": bool(torch.equal(torch.cat(ys).view(torch.int16), serial["y"].view(torch.int16))),
                "ids_equal": bool(torch.equal(torch.cat(ids), serial["expert_ids"])),
                "counts_equal": bool(torch.equal(torch.stack(received), want_received)),
            }
    if rank == 0:
        Path(out_path).write_text(json.dumps(report))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main(sys.argv[1])
