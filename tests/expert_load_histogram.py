"""Per-expert load of a synthetic configuration under the oracle's routing (CPU).

    python tests/expert_load_histogram.py kimi_k2 1024 [seed]

Prints how many routed rows each expert receives (summary and a coarse histogram) and the rows each
rank owns when the experts are split over 2, 4 and 8 ranks: the skew the Zipf selection bias of the
Kimi-K2-shaped configuration produces.
"""

import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

from oracle import moe_oracle as O  # noqa: E402
from tests import helpers as H  # noqa: E402
from vibe_megakernel_b200 import synthetic  # noqa: E402


def main(name: str, tokens: int, seed: int = 0) -> None:
    geo = synthetic.GEOMETRIES[name]
    x = synthetic.normal_rows(seed, "x", tokens, geo.hidden, 1.0, "cpu").to(torch.bfloat16)
    router = synthetic.normal_rows(seed, "router", geo.experts, geo.hidden, geo.router_std, "cpu")
    bias = synthetic.router_bias(geo, seed, "cpu")
    ids, _ = O.route_tokens(H.spec_of(geo), x, router, bias)
    load = torch.bincount(ids.flatten(), minlength=geo.experts)
    rows = tokens * geo.topk
    mean = rows / geo.experts
    print(f"{name}, {tokens} tokens, seed {seed}: {rows} routed rows over {geo.experts} experts (mean {mean:.1f})")
    print(f"  experts hit {int((load > 0).sum())}, hottest {int(load.max())} rows ({load.max() / mean:.1f}x mean), "
          f"median {int(load.median())}, coldest {int(load.min())}")
    top = torch.sort(load, descending=True).values
    for share in (1, 5, 10, 25, 50):
        k = max(1, geo.experts * share // 100)
        print(f"  hottest {share:2d} % of the experts ({k:3d}) take {100 * int(top[:k].sum()) / rows:5.1f} % of the rows")
    edges = [0, 1, 2, 4, 8, 16, 32, 64, 128, 256, 1 << 30]
    for lo, hi in zip(edges[:-1], edges[1:]):
        n = int(((load >= lo) & (load < hi)).sum())
        if n:
            print(f"  {lo:4d} <= rows < {hi if hi < (1 << 30) else 'inf':>4}: {n:3d} experts")
    for world in (2, 4, 8):
        per = load.reshape(world, -1).sum(1).tolist()
        hit = (load.reshape(world, -1) > 0).sum(1).tolist()
        print(f"  {world} ranks: rows per rank {per}, experts hit per rank {hit}")


if __name__ == "__main__":
    main(sys.argv[1], int(sys.argv[2]), int(sys.argv[3]) if len(sys.argv) > 3 else 0)
