"""``Tokenizer`` interface and its two native implementations.

Interface as in the reference (include/cverl/text/tokenizer.h:13-55): ``encode`` with
options (add_bos, add_eos, max_tokens), ``decode(ids, skip_special)``, vocabulary size and
pad / bos / eos / unk ids, ``name``.  The work happens in ``libcverl.so``
(csrc/text_reward.cc, csrc/bpe_tokenizer.cc).
"""
from __future__ import annotations

import abc
import ctypes as C
from dataclasses import dataclass
from typing import List, Sequence

from .. import _native as nv


@dataclass
class EncodeOptions:
    add_bos: bool = False
    add_eos: bool = False
    max_tokens: int = 0  # 0 = unlimited


def _bind():
    lib = nv.host()
    if getattr(lib, "_text_bound", False):
        return lib
    i64, p = C.c_int64, C.c_void_p
    lib.cverl_byte_encode.restype = i64
    lib.cverl_byte_encode.argtypes = [C.c_char_p, i64, C.c_int, C.c_int, i64, C.POINTER(i64), i64]
    lib.cverl_byte_decode.restype = i64
    lib.cverl_byte_decode.argtypes = [C.POINTER(i64), i64, C.c_int, C.c_char_p, i64]
    lib.cverl_bpe_open.restype = p
    lib.cverl_bpe_open.argtypes = [C.c_char_p, C.c_char_p, C.c_int]
    lib.cverl_bpe_close.argtypes = [p]
    lib.cverl_bpe_vocab_size.restype = i64
    lib.cverl_bpe_vocab_size.argtypes = [p]
    lib.cverl_bpe_special_id.restype = i64
    lib.cverl_bpe_special_id.argtypes = [p, C.c_int]
    lib.cverl_bpe_uses_pcre2.argtypes = [p]
    lib.cverl_bpe_encode.restype = i64
    lib.cverl_bpe_encode.argtypes = [p, C.c_char_p, i64, C.POINTER(i64), i64]
    lib.cverl_bpe_uses_jit.argtypes = [p]
    lib.cverl_bpe_uses_id_merges.argtypes = [p]
    lib.cverl_bpe_encode_batch.restype = i64
    lib.cverl_bpe_encode_batch.argtypes = [p, C.POINTER(C.c_char_p), C.POINTER(i64), i64, C.c_int, C.POINTER(i64), i64,
                                           C.POINTER(i64)]
    lib.cverl_bpe_decode.restype = i64
    lib.cverl_bpe_decode.argtypes = [p, C.POINTER(i64), i64, C.c_int, C.c_char_p, i64]
    lib._text_bound = True
    return lib


class Tokenizer(abc.ABC):
    @abc.abstractmethod
    def encode(self, text: str, options: EncodeOptions = EncodeOptions()) -> List[int]: ...

    @abc.abstractmethod
    def decode(self, ids: Sequence[int], skip_special: bool = True) -> str: ...

    @property
    @abc.abstractmethod
    def vocab_size(self) -> int: ...

    pad_id: int = 0
    bos_id: int = -1
    eos_id: int = -1
    unk_id: int = -1

    @abc.abstractmethod
    def name(self) -> str: ...


class ByteTokenizer(Tokenizer):
    """260-entry vocabulary: pad, bos, eos, unk, then the 256 byte values."""

    pad_id, bos_id, eos_id, unk_id = 0, 1, 2, 3

    def __init__(self):
        self._lib = _bind()

    @property
    def vocab_size(self) -> int:
        return 260

    def name(self) -> str:
        return "byte"

    def encode(self, text: str, options: EncodeOptions = EncodeOptions()) -> List[int]:
        raw = text.encode("utf-8")
        cap = len(raw) + 2
        buf = (C.c_int64 * cap)()
        n = self._lib.cverl_byte_encode(raw, len(raw), int(options.add_bos), int(options.add_eos),
                                        options.max_tokens, buf, cap)
        return list(buf[:min(n, cap)])

    def decode(self, ids: Sequence[int], skip_special: bool = True) -> str:
        n = len(ids)
        arr = (C.c_int64 * max(n, 1))(*ids)
        cap = 8 * n + 8
        out = C.create_string_buffer(cap)
        m = self._lib.cverl_byte_decode(arr, n, int(skip_special), out, cap)
        return out.raw[:m].decode("utf-8", errors="replace")


class HfBpeTokenizer(Tokenizer):
    """Byte-level BPE from a Hugging Face ``tokenizer.json``."""

    def __init__(self, tokenizer_json: str):
        self._lib = _bind()
        err = C.create_string_buffer(512)
        self._h = self._lib.cverl_bpe_open(str(tokenizer_json).encode(), err, 512)
        if not self._h:
            raise RuntimeError(f"HfBpeTokenizer: {err.value.decode()}")
        self.pad_id = self._lib.cverl_bpe_special_id(self._h, 0)
        self.bos_id = self._lib.cverl_bpe_special_id(self._h, 1)
        self.eos_id = self._lib.cverl_bpe_special_id(self._h, 2)
        self.unk_id = self._lib.cverl_bpe_special_id(self._h, 3)

    @property
    def vocab_size(self) -> int:
        return self._lib.cverl_bpe_vocab_size(self._h)

    @property
    def uses_pcre2(self) -> bool:
        return bool(self._lib.cverl_bpe_uses_pcre2(self._h))

    @property
    def uses_jit(self) -> bool:
        """The pre-tokenizer pattern runs as JIT-compiled code (a PCRE2 built with JIT support)."""
        return bool(self._lib.cverl_bpe_uses_jit(self._h))

    @property
    def uses_id_merges(self) -> bool:
        """Merges run on symbol ids (every merge's sides and result are vocabulary entries)."""
        return bool(self._lib.cverl_bpe_uses_id_merges(self._h))

    def name(self) -> str:
        return "hf-bpe"      # the reference's spelling (include/cverl/text/hf_bpe_tokenizer.h:71)

    def encode_batch_flat(self, texts: Sequence[str], threads: int = 0):
        """Encodes ``texts`` on ``threads`` native threads (0: one per core, at most 16).  Returns
        ``(ids, offsets)`` as int64 numpy arrays: the ids of text i are ``ids[offsets[i]:offsets[i + 1]]``."""
        import numpy as np
        n = len(texts)
        raws = [t.encode("utf-8") for t in texts]
        arr = (C.c_char_p * max(n, 1))(*raws)
        lens = (C.c_int64 * max(n, 1))(*[len(r) for r in raws])
        if threads <= 0:
            import os
            threads = min(os.cpu_count() or 1, 16)
        offsets = np.zeros(n + 1, dtype=np.int64)
        cap = sum(len(r) for r in raws) + 8        # a token covers at least one byte
        ids = np.empty(cap, dtype=np.int64)
        i64p = C.POINTER(C.c_int64)
        total = self._lib.cverl_bpe_encode_batch(self._h, arr, lens, n, threads, ids.ctypes.data_as(i64p), cap,
                                                 offsets.ctypes.data_as(i64p))
        if total < 0 or total > cap:
            raise RuntimeError("cverl_bpe_encode_batch: output does not fit")
        return ids[:total], offsets

    def encode_batch(self, texts: Sequence[str], options: EncodeOptions = EncodeOptions(),
                     threads: int = 0) -> List[List[int]]:
        ids, offsets = self.encode_batch_flat(texts, threads)
        out = []
        for i in range(len(texts)):
            row = ids[offsets[i]:offsets[i + 1]].tolist()
            if options.add_bos and self.bos_id >= 0:
                row = [self.bos_id] + row
            if options.add_eos and self.eos_id >= 0:
                row = row + [self.eos_id]
            out.append(row[:options.max_tokens] if options.max_tokens > 0 else row)
        return out

    def encode(self, text: str, options: EncodeOptions = EncodeOptions()) -> List[int]:
        raw = text.encode("utf-8")
        cap = len(raw) + 8
        buf = (C.c_int64 * cap)()
        n = self._lib.cverl_bpe_encode(self._h, raw, len(raw), buf, cap)
        ids = list(buf[:min(n, cap)])
        if options.add_bos and self.bos_id >= 0:
            ids = [self.bos_id] + ids
        if options.add_eos and self.eos_id >= 0:
            ids = ids + [self.eos_id]
        if options.max_tokens > 0:
            ids = ids[:options.max_tokens]
        return ids

    def decode(self, ids: Sequence[int], skip_special: bool = True) -> str:
        n = len(ids)
        arr = (C.c_int64 * max(n, 1))(*ids)
        cap = 64 * n + 64
        out = C.create_string_buffer(cap)
        m = self._lib.cverl_bpe_decode(self._h, arr, n, int(skip_special), out, cap)
        return out.raw[:min(m, cap)].decode("utf-8", errors="replace")

    def __del__(self):
        try:
            if self._h:
                self._lib.cverl_bpe_close(self._h)
                self._h = None
        except Exception:
            pass
