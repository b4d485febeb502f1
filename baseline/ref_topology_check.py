"""The planner against the reference's own Topology and pipeline schedule, over random layouts.

    python baseline/ref_topology_check.py [--keep DIR] [--layouts 120]

``baseline/ref_topology_check.cc`` dumps, for one layout, what the reference's classes (from the reference library
built by ``baseline/build_ref.py``) say: whether the layout is valid, every rank's coordinates and groups on all
seven axes, pipeline neighbours, layer ranges, the 1F1B action list with its peak of live activations, and the NCCL
environment.  This package's planner (``cverl_b200.parallel.topology`` / ``pipeline``) answers the same questions;
random valid and invalid layouts are compared field by field.  One JSON line; exit code 0 when all agree, 3 when
the reference library is not built.
"""
from __future__ import annotations

import argparse
import json
import random
import subprocess
import sys
import tempfile
from pathlib import Path

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--keep", default="")
    ap.add_argument("--layouts", type=int, default=120)
    a = ap.parse_args(argv)
    import torch

    from cverl_b200.parallel.pipeline import (PipelineActionType, pipeline_1f1b_schedule, pipeline_peers,
                                              pipeline_schedule_max_live_activations)
    from cverl_b200.parallel.topology import ClusterSpec, ParallelDims, Topology
    import ref_common
    try:
        exe = ref_common.link_driver(HERE / "ref_topology_check.cc", "ref_topology_check")
    except ref_common.Unavailable as exc:
        print(json.dumps({"unavailable": str(exc)}))
        return 3
    with tempfile.TemporaryDirectory(prefix="cverl_ref_") as tmp:
        work = Path(a.keep) if a.keep else Path(tmp)
        work.mkdir(parents=True, exist_ok=True)
        rng = random.Random(11)
        valid = invalid = 0
        problems = []
        for _ in range(a.layouts):
            dp, pp, cp, tp, ep = (rng.choice([1, 1, 2, 3, 4]) for _ in range(5))
            sp = rng.choice([1, 1, 1, tp, 2])
            mb = rng.choice([pp, pp, pp + 1, 2 * pp, max(pp - 1, 0), 0])
            gpn = rng.choice([1, 2, 4, 8])
            world = dp * pp * cp * tp * ep + (1 if rng.random() < 0.1 else 0)
            layers = rng.randrange(pp, 70)
            layout = [dp, pp, cp, tp, ep, sp, mb, world, gpn, layers]
            r = subprocess.run([str(exe), *map(str, layout)], capture_output=True, text=True)
            ref = json.loads(r.stdout)
            try:
                topo = Topology(ParallelDims(dp, pp, cp, tp, ep, sp, mb), ClusterSpec(world_size=world, gpus_per_node=gpn))
                mine_ok = True
            except ValueError:
                mine_ok = False
            if ref["valid"] != mine_ok:
                problems.append({"layout": layout, "what": "validity", "reference": ref.get("error", "valid")})
                continue
            if not mine_ok:
                invalid += 1
                continue
            valid += 1
            for rank, want in enumerate(ref["ranks"]):
                info = topo.rank_info(rank)
                peers = pipeline_peers(info.pipeline_group, info.pipeline_rank)
                sched = pipeline_1f1b_schedule(info.pipeline_rank, pp, mb)
                got = {"coords": list(topo.coords_of(rank)), "sequence_rank": info.sequence_rank,
                       "data": info.data_group, "pipeline": info.pipeline_group, "context": info.context_group,
                       "tensor": info.tensor_group, "expert": info.expert_group, "sequence": info.sequence_group,
                       "model": info.model_group, "prev": peers.prev_rank, "next": peers.next_rank,
                       "layers": list(topo.pipeline_layer_range(layers, info.pipeline_rank)),
                       "schedule": [[0 if x.type == PipelineActionType.FORWARD else 1, x.micro_batch] for x in sched],
                       "max_live": pipeline_schedule_max_live_activations(sched, mb)}
                for key, value in got.items():
                    if want[key] != value:
                        problems.append({"layout": layout, "rank": rank, "what": key, "reference": want[key], "ours": value})
            if dict(topo.nccl_env()) != ref["nccl_env"]:
                problems.append({"layout": layout, "what": "nccl_env", "reference": ref["nccl_env"], "ours": dict(topo.nccl_env())})
        ok = not problems
        print(json.dumps({"layouts": a.layouts, "valid": valid, "invalid": invalid, "problems": problems[:5], "agree": ok}))
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
