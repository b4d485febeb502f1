"""Text-level rollout transports: request/response records, loopback, shared memory.

``RolloutRequest`` / ``RolloutResponse`` and the two transports follow the reference
(include/cverl/rollout/transport.h:16-102, src/rollout/transport.cc:11-55,
src/rollout/shared_memory_transport.cc).  ``LoopbackRolloutTransport`` echoes
``prompt + suffix`` and synthesises token ids by xorshift of an FNV hash;
``SharedMemoryRolloutTransport`` moves little-endian length-prefixed records through one
shm slot guarded by two named semaphores with timeouts (native code: csrc/shm_transport.cc).
"""
from __future__ import annotations

import abc
import ctypes as C
import struct
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional

from .. import _native as nv


@dataclass
class RolloutRequest:
    prompts: List[str] = field(default_factory=list)
    prompt_token_ids: List[List[int]] = field(default_factory=list)
    n: int = 1
    max_tokens: int = 16
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = 0
    stop: List[str] = field(default_factory=list)
    flags: int = 0
    seed: int = 0
    model: str = ""
    extra_params: Dict[str, str] = field(default_factory=dict)
    request_id: int = 0


@dataclass
class RolloutSequence:
    prompt_index: int = 0
    sample_index: int = 0
    text: str = ""
    token_ids: List[int] = field(default_factory=list)
    logprobs: List[float] = field(default_factory=list)
    finish_reason: str = ""


@dataclass
class RolloutResponse:
    sequences: List[RolloutSequence] = field(default_factory=list)
    metrics: Dict[str, float] = field(default_factory=dict)


class RolloutTransport(abc.ABC):
    @abc.abstractmethod
    def generate(self, request: RolloutRequest) -> RolloutResponse: ...


def _fnv1a(data: bytes) -> int:
    h = 0xCBF29CE484222325
    for b in data:
        h = ((h ^ b) * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    return h


def _xorshift(x: int) -> int:
    x ^= (x << 13) & 0xFFFFFFFFFFFFFFFF
    x ^= x >> 7
    x ^= (x << 17) & 0xFFFFFFFFFFFFFFFF
    return x & 0xFFFFFFFFFFFFFFFF


class LoopbackRolloutTransport(RolloutTransport):
    """Deterministic stand-in for a generation server."""

    def __init__(self, suffix: str = " #### 0", vocab_size: int = 32000):
        self.suffix, self.vocab_size = suffix, vocab_size

    def generate(self, request: RolloutRequest) -> RolloutResponse:
        resp = RolloutResponse()
        for pi, prompt in enumerate(request.prompts):
            for si in range(max(1, request.n)):
                text = prompt + self.suffix
                state = _fnv1a(text.encode()) ^ (si + 1) ^ (request.seed << 1)
                ids, lps = [], []
                for _ in range(max(1, min(request.max_tokens, 8))):
                    state = _xorshift(state or 1)
                    ids.append(state % self.vocab_size)
                    lps.append(-1.0)
                resp.sequences.append(RolloutSequence(pi, si, text, ids, lps, "stop"))
        resp.metrics["num_sequences"] = float(len(resp.sequences))
        return resp


# ---------------------------------------------------------------------------------------------
# little-endian length-prefixed serialisation
# ---------------------------------------------------------------------------------------------
class _W:
    def __init__(self):
        self.b = bytearray()

    def u32(self, v): self.b += struct.pack("<I", v)
    def i64(self, v): self.b += struct.pack("<q", v)
    def f64(self, v): self.b += struct.pack("<d", v)

    def s(self, text: str):
        raw = text.encode()
        self.u32(len(raw))
        self.b += raw

    def i64s(self, xs):
        self.u32(len(xs))
        self.b += struct.pack(f"<{len(xs)}q", *xs)

    def f64s(self, xs):
        self.u32(len(xs))
        self.b += struct.pack(f"<{len(xs)}d", *xs)


class _R:
    def __init__(self, data: bytes):
        self.d, self.o = data, 0

    def _take(self, fmt):
        size = struct.calcsize(fmt)
        if self.o + size > len(self.d):
            raise ValueError("truncated rollout record")
        v = struct.unpack_from(fmt, self.d, self.o)
        self.o += size
        return v

    def u32(self): return self._take("<I")[0]
    def i64(self): return self._take("<q")[0]
    def f64(self): return self._take("<d")[0]

    def s(self) -> str:
        n = self.u32()
        if self.o + n > len(self.d):
            raise ValueError("truncated rollout record")
        v = self.d[self.o:self.o + n].decode()
        self.o += n
        return v

    def i64s(self): return list(self._take(f"<{self.u32()}q"))
    def f64s(self): return list(self._take(f"<{self.u32()}d"))


def serialize_request(r: RolloutRequest) -> bytes:
    w = _W()
    w.u32(len(r.prompts))
    for p in r.prompts:
        w.s(p)
    w.u32(len(r.prompt_token_ids))
    for ids in r.prompt_token_ids:
        w.i64s(ids)
    for v in (r.n, r.max_tokens, r.top_k, r.flags, r.seed, r.request_id):
        w.i64(v)
    w.f64(r.temperature)
    w.f64(r.top_p)
    w.u32(len(r.stop))
    for s in r.stop:
        w.s(s)
    w.s(r.model)
    w.u32(len(r.extra_params))
    for k, v in r.extra_params.items():
        w.s(k)
        w.s(v)
    return bytes(w.b)


def deserialize_request(data: bytes) -> RolloutRequest:
    rd = _R(data)
    r = RolloutRequest()
    r.prompts = [rd.s() for _ in range(rd.u32())]
    r.prompt_token_ids = [rd.i64s() for _ in range(rd.u32())]
    r.n, r.max_tokens, r.top_k, r.flags, r.seed, r.request_id = (rd.i64() for _ in range(6))
    r.temperature, r.top_p = rd.f64(), rd.f64()
    r.stop = [rd.s() for _ in range(rd.u32())]
    r.model = rd.s()
    r.extra_params = {rd.s(): rd.s() for _ in range(rd.u32())}
    return r


def serialize_response(r: RolloutResponse) -> bytes:
    w = _W()
    w.u32(len(r.sequences))
    for s in r.sequences:
        w.i64(s.prompt_index)
        w.i64(s.sample_index)
        w.s(s.text)
        w.i64s(s.token_ids)
        w.f64s(s.logprobs)
        w.s(s.finish_reason)
    w.u32(len(r.metrics))
    for k, v in r.metrics.items():
        w.s(k)
        w.f64(v)
    return bytes(w.b)


def deserialize_response(data: bytes) -> RolloutResponse:
    rd = _R(data)
    r = RolloutResponse()
    for _ in range(rd.u32()):
        s = RolloutSequence()
        s.prompt_index, s.sample_index = rd.i64(), rd.i64()
        s.text = rd.s()
        s.token_ids = rd.i64s()
        s.logprobs = rd.f64s()
        s.finish_reason = rd.s()
        r.sequences.append(s)
    r.metrics = {rd.s(): rd.f64() for _ in range(rd.u32())}
    return r


# ---------------------------------------------------------------------------------------------
# shared memory
# ---------------------------------------------------------------------------------------------
def _lib():
    lib = nv.host()
    if not getattr(lib, "_shm_bound", False):
        p, i64 = C.c_void_p, C.c_int64
        lib.cverl_shm_region_open.restype = p
        lib.cverl_shm_region_open.argtypes = [C.c_char_p, i64, C.c_int]
        lib.cverl_shm_region_addr.restype = p
        lib.cverl_shm_region_addr.argtypes = [p]
        lib.cverl_shm_region_size.restype = i64
        lib.cverl_shm_region_size.argtypes = [p]
        lib.cverl_shm_region_close.argtypes = [p]
        lib.cverl_shm_transport_open.restype = p
        lib.cverl_shm_transport_open.argtypes = [C.c_char_p, i64, C.c_int]
        lib.cverl_shm_transport_close.argtypes = [p]
        lib.cverl_shm_transport_capacity.restype = i64
        lib.cverl_shm_transport_capacity.argtypes = [p]
        lib.cverl_shm_client_call.restype = i64
        lib.cverl_shm_client_call.argtypes = [p, C.c_char_p, i64, C.c_char_p, i64, i64]
        lib.cverl_shm_server_wait.restype = i64
        lib.cverl_shm_server_wait.argtypes = [p, C.c_char_p, i64, i64]
        lib.cverl_shm_server_reply.argtypes = [p, C.c_char_p, i64, C.c_int]
        lib._shm_bound = True
    return lib


class SharedMemoryRegion:
    """RAII POSIX shm mapping; the creating side unlinks the name when closed."""

    def __init__(self, name: str, size: int = 0, create: bool = False):
        self._lib = _lib()
        self._h = self._lib.cverl_shm_region_open(name.encode(), size, int(create))
        if not self._h:
            raise OSError(f"cannot {'create' if create else 'open'} shared memory region {name}")
        self.name = name
        self.size = self._lib.cverl_shm_region_size(self._h)

    def buffer(self):
        return (C.c_ubyte * self.size).from_address(self._lib.cverl_shm_region_addr(self._h))

    def close(self):
        if self._h:
            self._lib.cverl_shm_region_close(self._h)
            self._h = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


class SharedMemoryRolloutTransport(RolloutTransport):
    """Client (``generate``) and server (``serve_one`` / ``serve_loop``) ends of one slot."""

    _ERRORS = {-1: "request larger than the slot", -2: "timed out", -3: "semaphore error",
               -4: "server handler failed", -5: "response larger than the slot", -6: "request id mismatch"}

    def __init__(self, name: str, payload_capacity: int = 1 << 20, create: bool = False, timeout_ms: int = 60000):
        self._lib = _lib()
        self._h = self._lib.cverl_shm_transport_open(name.encode(), payload_capacity, int(create))
        if not self._h:
            raise OSError(f"cannot {'create' if create else 'attach to'} shared-memory transport {name}")
        self.capacity = self._lib.cverl_shm_transport_capacity(self._h)
        self.timeout_ms = timeout_ms

    def generate(self, request: RolloutRequest) -> RolloutResponse:
        raw = serialize_request(request)
        out = C.create_string_buffer(self.capacity)
        n = self._lib.cverl_shm_client_call(self._h, raw, len(raw), out, self.capacity, self.timeout_ms)
        if n < 0:
            if n == -2:
                raise TimeoutError("shared-memory rollout transport: no response within the timeout")
            raise RuntimeError("shared-memory rollout transport: " + self._ERRORS.get(n, f"error {n}"))
        return deserialize_response(out.raw[:n])

    def serve_one(self, handler: Callable[[RolloutRequest], RolloutResponse], timeout_ms: Optional[int] = None) -> bool:
        """Serves one request; returns False when none arrived within the timeout."""
        buf = C.create_string_buffer(self.capacity)
        n = self._lib.cverl_shm_server_wait(self._h, buf, self.capacity, self.timeout_ms if timeout_ms is None
                                            else timeout_ms)
        if n == -2:
            return False
        if n < 0:
            raise RuntimeError("shared-memory rollout transport: server wait failed")
        try:
            raw = serialize_response(handler(deserialize_request(buf.raw[:n])))
        except Exception:
            self._lib.cverl_shm_server_reply(self._h, None, 0, 1)
            return True
        if len(raw) > self.capacity:
            self._lib.cverl_shm_server_reply(self._h, None, 0, 2)
        else:
            self._lib.cverl_shm_server_reply(self._h, raw, len(raw), 0)
        return True

    def serve_loop(self, handler, should_stop: Callable[[], bool], poll_ms: int = 100) -> int:
        served = 0
        while not should_stop():
            if self.serve_one(handler, poll_ms):
                served += 1
        return served

    def close(self):
        if self._h:
            self._lib.cverl_shm_transport_close(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
