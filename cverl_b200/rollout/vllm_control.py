"""Control plane of a vLLM server's native RL weight transfer, and the live weight push.

HTTP carries only control and metadata - pause / resume, sleep / wake, engine init, the update manifest
(names, dtypes, shapes).  The tensors themselves travel over NCCL through vLLM's
``NCCLWeightTransferEngine``: the trainer is rank 0 of a group with the server's workers
(``rank_offset`` 1), and ``trainer_send_weights`` broadcasts the live parameters, packed into
fixed-size buffers, while the server's ``/update_weights`` call receives them.  The sequence of one
sync is ``/pause?mode=wait`` -> ``/update_weights`` (on a helper thread, it blocks until the tensors
arrive) in parallel with the NCCL send -> ``/resume``.  Reference: tools/rollout/vllm_online_grpo.py:109-177,
tools/rollout/vllm_native_rl_control.py, tools/rollout/vllm_nccl_weight_sender.py.
"""
from __future__ import annotations

import concurrent.futures
import json
import urllib.error
import urllib.request
from typing import Any, Callable, Dict, Iterable, List, Optional, Tuple

_DTYPE_NAMES = {"float": "float32", "fp32": "float32", "float32": "float32", "bf16": "bfloat16",
                "bfloat16": "bfloat16", "half": "float16", "fp16": "float16", "float16": "float16"}


def normalize_dtype_name(name: str) -> str:
    low = name.replace("torch.", "").lower()
    return _DTYPE_NAMES.get(low, low)


def post_json(base_url: str, path: str, payload: Dict[str, Any], timeout: float = 300.0) -> Dict[str, Any]:
    req = urllib.request.Request(base_url.rstrip("/") + path, data=json.dumps(payload).encode(),
                                 headers={"Content-Type": "application/json"}, method="POST")
    with urllib.request.urlopen(req, timeout=timeout) as resp:
        body = resp.read()
    return json.loads(body) if body else {}


def get_json(base_url: str, path: str, timeout: float = 300.0) -> Dict[str, Any]:
    with urllib.request.urlopen(base_url.rstrip("/") + path, timeout=timeout) as resp:
        return json.loads(resp.read() or b"{}")


class VllmControl:
    """The server's control endpoints."""

    def __init__(self, base_url: str = "http://127.0.0.1:8000", timeout: float = 300.0):
        self.base_url, self.timeout = base_url, timeout

    def pause(self, mode: str = "wait"):
        return post_json(self.base_url, f"/pause?mode={mode}", {}, self.timeout)

    def resume(self):
        return post_json(self.base_url, "/resume", {}, self.timeout)

    def sleep(self, level: int = 1, mode: str = "wait"):
        return post_json(self.base_url, f"/sleep?level={level}&mode={mode}", {}, self.timeout)

    def wake(self, tags: Optional[Iterable[str]] = None):
        suffix = "?" + "&".join(f"tags={t}" for t in tags) if tags else ""
        return post_json(self.base_url, "/wake_up" + suffix, {}, self.timeout)

    def world_size(self):
        return get_json(self.base_url, "/get_world_size?include_dp=true", self.timeout)

    def is_sleeping(self):
        return get_json(self.base_url, "/is_sleeping", self.timeout)

    def init_weight_transfer(self, master_address: str, master_port: int, world_size: int, rank_offset: int = 1):
        return post_json(self.base_url, "/init_weight_transfer_engine",
                         {"init_info": {"master_address": master_address, "master_port": master_port,
                                        "rank_offset": rank_offset, "world_size": world_size}}, self.timeout)

    def update_weights(self, update_info: Dict[str, Any]):
        return post_json(self.base_url, "/update_weights", {"update_info": dict(update_info)}, self.timeout)


def _vllm_engine():
    from vllm.distributed.weight_transfer.nccl_engine import NCCLTrainerSendWeightsArgs, NCCLWeightTransferEngine
    return NCCLWeightTransferEngine, NCCLTrainerSendWeightsArgs


class VllmNcclSync:
    """Pushes a policy's live parameters into a running vLLM server.

    ``engine`` / ``send_args`` default to vLLM's NCCL weight-transfer engine; tests pass fakes.  The first
    ``sync`` opens the NCCL group (the server side joins through ``/init_weight_transfer_engine``, issued on a
    helper thread because both sides block until the group is complete).
    """

    def __init__(self, control: VllmControl, master_address: str, master_port: int, world_size: int,
                 rank_offset: int = 1, packed: bool = True, packed_buffer_size_bytes: int = 1 << 30,
                 packed_num_buffers: int = 2, checkpoint_format: bool = True, pause: bool = True, engine=None,
                 send_args: Optional[Callable[..., Any]] = None, server_init: bool = True,
                 update_metadata: bool = True):
        """``server_init=False``: the server's side of the group was opened by someone else
        (``vllm_native_rl_control init-nccl``), only the trainer's side is opened here.  ``update_metadata=False``:
        the ``/update_weights`` request is posted by someone else; only the tensors are sent."""
        self.control = control
        self.init = dict(master_address=master_address, master_port=master_port, world_size=world_size)
        self.rank_offset = rank_offset
        self.packed, self.buf_bytes, self.num_buf = packed, packed_buffer_size_bytes, packed_num_buffers
        self.checkpoint_format, self.pause = checkpoint_format, pause
        self._engine, self._send_args = engine, send_args
        self.server_init, self.update_metadata = server_init, update_metadata
        self.group = None
        self.syncs = 0

    def _ensure_group(self, pool) -> None:
        if self.group is not None:
            return
        if self._engine is None:
            self._engine, self._send_args = _vllm_engine()
        server = None
        if self.server_init:
            server = pool.submit(self.control.init_weight_transfer, self.init["master_address"],
                                 self.init["master_port"], self.init["world_size"], self.rank_offset)
        self.group = self._engine.trainer_init(dict(self.init))
        if server is not None:
            server.result()

    def sync(self, named_parameters: List[Tuple[str, Any]], update_info: Dict[str, Any]) -> Dict[str, Any]:
        """One weight push.  Returns the byte count and the server's answer to ``/update_weights``."""
        info = dict(update_info)
        info["dtype_names"] = [normalize_dtype_name(x) for x in info.get("dtype_names", [])]
        info["is_checkpoint_format"] = self.checkpoint_format
        with concurrent.futures.ThreadPoolExecutor(max_workers=1) as pool:
            self._ensure_group(pool)
            if self.pause:
                self.control.pause("wait")
            try:
                server = pool.submit(self.control.update_weights, info) if self.update_metadata else None
                self._engine.trainer_send_weights(
                    iter(named_parameters),
                    self._send_args(group=self.group, src=0, packed=self.packed,
                                    packed_buffer_size_bytes=self.buf_bytes, packed_num_buffers=self.num_buf))
                answer = server.result() if server is not None else None
            finally:
                if self.pause:
                    self.control.resume()
        self.syncs += 1
        nbytes = sum(t.numel() * t.element_size() for _, t in named_parameters)
        return {"sent": len(named_parameters), "bytes": nbytes, "server": answer}
