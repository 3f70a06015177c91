"""Plugin file for the reference harness: ``build(case) -> run(inputs) -> outputs``.

Protocol: megabench/README.md:83-104 and megabench/harness/runner.py:69-87. ``case`` is the
harness' case dict (``Case.to_dict()``, megabench/cases.py:92-108); when the case runs on several GPUs
the harness adds ``case["execution"] = {rank, world_size, tp_rank, ep_rank, backend, device, tp_group,
ep_group}`` with live process-group handles (megabench/harness/distributed.py:68-74) and calls
``build`` once in every rank's process.

Two families are served:

* the FP8 block-scaled MoE layer (any family name but ``megamoe_layer``). Geometry from
  ``case["params"]`` (integers, as the reference's Case admits), the non-integer knobs in
  ``case["moe"]``:

      params: tokens (per rank), hidden, intermediate, experts, topk, shared_experts, router_groups,
              router_top_groups, swiglu_limit (the clamp of megabench/tasks/megamoe.py:43-44,116-122;
              absent or 0 = none)
      moe:    {"scoring": "sigmoid"|"softmax"|"sqrt_softplus"|"softmax_biased", "scaling": float,
               "weight_before_requant": bool (routing weight inside SwiGLU, megamoe.py:122,176-182)}

  ``run`` takes the tensors named in megabench/tasks/frontier.py:157-176 (without the layer prefix;
  with ``execution`` the expert tensors hold this rank's experts, ``x`` its token rows) and returns
  ``y`` (bf16 [T, H]), ``expert_ids`` (int64 [T, topk], choice order) and ``order`` (int64 [T*topk]:
  on one GPU the stable grouping of the flattened ids by expert, megabench/tasks/megamoe.py:137; in
  expert-parallel execution the stable order by owning rank, megabench/tasks/megamoe.py:161-164).

* ``megamoe_layer``: the routed experts in the MegaMoE-native formats, inputs as
  ``megamoe.make_inputs`` (megabench/tasks/megamoe.py:86-113), output ``{"y"}``
  (megabench/integrations/make_agent_workspace.py:109), on one GPU or expert-parallel over the
  ranks of ``execution["ep_group"]`` (megabench/cases.py:380-388).

Inputs are not modified; all work is enqueued on the current torch stream; an expert-parallel
``run`` makes no collective call (rows travel as peer stores issued by the kernels), only ``build``
does (exchange of the peer-memory handles over the given group).
"""

from __future__ import annotations

import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

from vibe_megakernel_b200.layer import LayerConfig, MoeLayer  # noqa: E402


def _layer_config(case: dict) -> LayerConfig:
    p = case["params"]
    extra = case.get("moe", {})
    return LayerConfig(hidden=p["hidden"], inter=p["intermediate"], experts=p["experts"], topk=p["topk"],
                       shared=p.get("shared_experts", 0), scoring=extra.get("scoring", "sigmoid"),
                       n_group=p.get("router_groups", 1), topk_group=p.get("router_top_groups", 1),
                       scaling=float(extra.get("scaling", 1.0)), swiglu_limit=float(p.get("swiglu_limit", 0.0)),
                       weight_before_requant=bool(extra.get("weight_before_requant", False)))


def _ranks(case: dict) -> int:
    execution = case.get("execution")
    return int(execution["world_size"]) if execution else int(case.get("gpus", 1))


def build(case: dict):
    p = case["params"]
    execution = case.get("execution")
    tokens = p.get("tokens", p.get("batch", 1))
    if execution is None and _ranks(case) != 1:
        raise ValueError("a case on several GPUs needs case['execution'] (rank, world_size, device, ep_group)")

    if case.get("family") == "megamoe_layer":
        from vibe_megakernel_b200.megamoe import MegaMoe, MegaMoeConfig, MegaMoeEp
        config = MegaMoeConfig(hidden=p["hidden"], inter=p["intermediate"], experts=p["experts"], topk=p["topk"],
                               swiglu_limit=float(p.get("swiglu_limit", 10)))
        if execution is None:
            mega = MegaMoe(config, max_tokens=tokens)
        else:
            mega = MegaMoeEp(config, max_tokens=tokens, group=execution.get("ep_group"), device=execution.get("device"))

        def run_megamoe(inputs: dict):
            return {"y": mega.run(inputs)["y"]}

        return run_megamoe

    config = _layer_config(case)
    if execution is None:
        layer = MoeLayer(config, max_tokens=tokens)
    else:
        from vibe_megakernel_b200.ep import EpMoeLayer
        layer = EpMoeLayer(config, max_tokens=tokens, group=execution.get("ep_group"), device=execution.get("device"))

    def run(inputs: dict):
        out = layer.forward(inputs)
        return {"y": out["y"], "expert_ids": out["expert_ids"], "order": out["order"]}

    run.layer = layer          # lets a caller release the peer buffers of an expert-parallel layer (layer.close())
    return run
