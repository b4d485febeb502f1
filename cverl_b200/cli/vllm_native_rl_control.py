"""Command-line control of a vLLM server's native RL endpoints (no tensor travels over HTTP).

``python -m cverl_b200.cli.vllm_native_rl_control [--base-url URL] pause | resume | sleep [--level N --mode M] |
wake [--tags ...] | world-size | is-sleeping | init-nccl --master-port P --world-size W | update-nccl --manifest F``

``update-nccl`` posts the ``update_info`` block of a manifest written by ``cverl_b200.cli.vllm_weight_manifest``.
Reference: tools/rollout/vllm_native_rl_control.py.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

from ..rollout.vllm_control import VllmControl


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--base-url", default="http://127.0.0.1:8000")
    ap.add_argument("--timeout", type=float, default=300.0)
    sub = ap.add_subparsers(dest="cmd", required=True)
    sub.add_parser("pause")
    sub.add_parser("resume")
    sl = sub.add_parser("sleep")
    sl.add_argument("--level", type=int, default=1)
    sl.add_argument("--mode", choices=("abort", "wait", "keep"), default="wait")
    wk = sub.add_parser("wake")
    wk.add_argument("--tags", nargs="*", default=None)
    sub.add_parser("world-size")
    sub.add_parser("is-sleeping")
    init = sub.add_parser("init-nccl")
    init.add_argument("--master-address", default="127.0.0.1")
    init.add_argument("--master-port", type=int, required=True)
    init.add_argument("--world-size", type=int, required=True)
    init.add_argument("--rank-offset", type=int, default=1)
    upd = sub.add_parser("update-nccl")
    upd.add_argument("--manifest", required=True)
    a = ap.parse_args(argv)
    c = VllmControl(a.base_url, a.timeout)
    if a.cmd == "pause":
        out = c.pause()
    elif a.cmd == "resume":
        out = c.resume()
    elif a.cmd == "sleep":
        out = c.sleep(a.level, a.mode)
    elif a.cmd == "wake":
        out = c.wake(a.tags)
    elif a.cmd == "world-size":
        out = c.world_size()
    elif a.cmd == "is-sleeping":
        out = c.is_sleeping()
    elif a.cmd == "init-nccl":
        out = c.init_weight_transfer(a.master_address, a.master_port, a.world_size, a.rank_offset)
    else:
        doc = json.loads(Path(a.manifest).read_text())
        out = c.update_weights(doc.get("update_info", doc))
    print(json.dumps(out, indent=2))
    return 0


if __name__ == "__main__":
    sys.exit(main())
