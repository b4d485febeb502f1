"""Sends a model's live parameters to a running vLLM server over NCCL.

``python -m cverl_b200.cli.vllm_nccl_weight_sender --model-dir DIR --master-port P --world-size W [--dry-run]``

Loads the trainable policy (``QwenPolicy``), builds the update manifest from its live tensors, joins the
server's weight-transfer group as rank 0, pauses the server, posts the manifest while ``trainer_send_weights``
moves the tensors in packed buffers (1 GiB x 2 by default), and resumes the server.  ``--dry-run`` stops after
building the tensors and the manifest.  Reference: tools/rollout/vllm_nccl_weight_sender.py.
"""
from __future__ import annotations

import argparse
import json
import sys

from ..rollout.vllm_control import VllmControl, VllmNcclSync, normalize_dtype_name


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--model-dir", required=True)
    ap.add_argument("--tokenizer-path", default="")
    ap.add_argument("--device", default="cuda:0")
    ap.add_argument("--param-dtype", default="float32")
    ap.add_argument("--qwen-max-layers", type=int, default=-1)
    ap.add_argument("--base-url", default="http://127.0.0.1:8000")
    ap.add_argument("--master-address", default="127.0.0.1")
    ap.add_argument("--master-port", type=int, default=0)
    ap.add_argument("--world-size", type=int, default=0, help="trainer rank + all vLLM worker ranks")
    ap.add_argument("--rank-offset", type=int, default=1)
    ap.add_argument("--packed", action=argparse.BooleanOptionalAction, default=True)
    ap.add_argument("--packed-buffer-size-bytes", type=int, default=1 << 30)
    ap.add_argument("--packed-num-buffers", type=int, default=2)
    ap.add_argument("--checkpoint-format", action=argparse.BooleanOptionalAction, default=True)
    ap.add_argument("--timeout", type=float, default=300.0)
    ap.add_argument("--skip-server-init", action="store_true", help="the server's side of the group is opened elsewhere")
    ap.add_argument("--skip-update-metadata", action="store_true", help="the /update_weights request is posted elsewhere")
    ap.add_argument("--skip-pause", action="store_true")
    ap.add_argument("--dry-run", action="store_true")
    a = ap.parse_args(argv)
    from ..rollout.vllm_bridge import QwenPolicy
    policy = QwenPolicy(a.model_dir, a.tokenizer_path, a.device, normalize_dtype_name(a.param_dtype), a.qwen_max_layers)
    params = policy.named_parameters()
    info = policy.update_info(a.packed, a.packed_buffer_size_bytes, a.packed_num_buffers)
    if a.dry_run:
        name, t = params[0]
        print(json.dumps({"params": len(params), "packed": a.packed,
                          "first": {"name": name, "shape": list(t.shape), "device": str(t.device),
                                    "dtype": str(t.dtype).split(".")[-1]}}, indent=2))
        return 0
    if a.master_port <= 0 or a.world_size <= 1:
        print("--master-port and --world-size (>= 2) are required to send", file=sys.stderr)
        return 2
    sync = VllmNcclSync(VllmControl(a.base_url, a.timeout), a.master_address, a.master_port, a.world_size,
                        a.rank_offset, a.packed, a.packed_buffer_size_bytes, a.packed_num_buffers,
                        a.checkpoint_format, pause=not a.skip_pause, server_init=not a.skip_server_init,
                        update_metadata=not a.skip_update_metadata)
    print(json.dumps(sync.sync(params, info), indent=2))
    return 0


if __name__ == "__main__":
    sys.exit(main())
