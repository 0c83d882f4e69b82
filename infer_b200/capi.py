"""The C handle API's two ends in Python.

``Handle`` is what ``csrc/capi.cpp`` drives: one object per ``ib_engine``, methods that take plain integers and
memory views of the caller's C arrays.  ``CEngine`` is the other side, for Python programs and for the tests: a ctypes
wrapper that goes through the exported C symbols (``ib_engine_create`` ... ``ib_engine_destroy``) exactly as a C
program would, and gives token ids and numpy logits back.  A C or C++ embedder links the library and libpython and
needs neither class.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence

import numpy as np


class Handle:
    """Engine + scheduler behind one C handle (see csrc/capi.cpp for the meaning of every argument)."""

    def __init__(self, model_dir, random_spec, weights_seed, dtype, slots, max_seq, kv_blocks, chunk):
        import torch
        from .engine.generation import LLM
        spec = weights = None
        if random_spec:
            from .config import parse_config
            from .models import load_preset
            from .weights import random_weights
            arch, typed = parse_config(load_preset(random_spec))
            spec = arch.to_spec(typed)
            weights = random_weights(spec, int(weights_seed), torch.bfloat16)
            max_seq = min(int(max_seq), spec.max_positions)
        elif not model_dir:
            raise ValueError("give a model folder or a random-weights spec")
        self.llm = LLM(None if spec is not None else model_dir, dtype=dtype, slots=max(1, int(slots)), max_seq=int(max_seq),
                       kv_blocks=int(kv_blocks), max_batch_tokens=max(1, int(chunk)), spec=spec, weights=weights)
        self.engine = self.llm.engine
        self.logits = None

    def close(self):
        self.logits = None
        self.llm = self.engine = None

    def vocab_size(self) -> int:
        return int(self.engine.spec.vocab_size)

    def add_request(self, rid: int) -> None:
        self.engine.add_request(int(rid))

    def end_request(self, rid: int) -> None:
        self.engine.end_request(int(rid))

    def step(self, n, ids, n_tokens, tokens, n_want, want, ran) -> int:
        from .engine import StepEntry
        ids = np.frombuffer(ids, dtype=np.int64, count=n)
        n_tokens = np.frombuffer(n_tokens, dtype=np.int32, count=n)
        n_want = np.frombuffer(n_want, dtype=np.int32, count=n)
        tokens = np.frombuffer(tokens, dtype=np.int32)
        want = np.frombuffer(want, dtype=np.int32)
        entries, t, w = [], 0, 0
        for i in range(n):
            nt, nw = int(n_tokens[i]), int(n_want[i])
            if nt <= 0 or nw < 0:
                raise ValueError(f"entry {i}: needs at least one token and a non-negative number of wanted places")
            entries.append(StepEntry(int(ids[i]), tokens[t:t + nt].tolist(), want[w:w + nw].tolist()))
            t, w = t + nt, w + nw
        if ran is None:
            self.logits = self.engine.step(entries)
        else:
            res = self.engine.try_step(entries)
            np.frombuffer(ran, dtype=np.int32, count=n)[:] = np.asarray(res.ran, dtype=np.int32)
            self.logits = res.output
        self.engine.check_status()
        return int(self.logits.shape[0])

    def copy_logits(self, out) -> int:
        if self.logits is None:
            raise RuntimeError("no step has run on this handle")
        rows, vocab = self.logits.shape
        dst = np.frombuffer(out, dtype=np.float32)
        if dst.size < rows * vocab:
            raise ValueError(f"the buffer holds {dst.size} floats, the last step's logits are {rows} x {vocab}")
        dst[:rows * vocab] = self.logits.detach().float().cpu().numpy().reshape(-1)
        return int(rows)

    def generate(self, n, lens, tokens, max_new, temperature, seed, eos_id, out_tokens, out_lens) -> None:
        lens = np.frombuffer(lens, dtype=np.int32, count=n)
        tokens = np.frombuffer(tokens, dtype=np.int32)
        prompts, t = [], 0
        for i in range(n):
            prompts.append(tokens[t:t + int(lens[i])].tolist())
            t += int(lens[i])
        outs = self.llm.generate(prompts, max_new=int(max_new), temperature=float(temperature), seed=int(seed),
                                 eos_id=int(eos_id) if eos_id >= 0 else -1)
        dst = np.frombuffer(out_tokens, dtype=np.int32).reshape(n, max_new) if n and max_new else None
        got = np.frombuffer(out_lens, dtype=np.int32, count=n)
        for i, o in enumerate(outs):
            got[i] = len(o)
            if dst is not None:
                dst[i, :len(o)] = o


class CEngineError(RuntimeError):
    pass


class CEngine:
    """The engine through its exported C symbols.

        eng = CEngine(model_dir="/path/to/model", dtype="bfloat16", slots=4, max_seq=256)
        eng.add_request(7); rows = eng.step([(7, [1, 2, 3], [2])]); logits = eng.logits()      # numpy [rows, vocab]
        outs = eng.generate([[1, 2, 3]], max_new=8)
    """

    def __init__(self, model_dir: Optional[str] = None, random_spec: Optional[str] = None, weights_seed: int = 0,
                 dtype: str = "bfloat16", slots: int = 4, max_seq: int = 4096, kv_blocks: int = 0, chunk: int = 512):
        from .csrc.build import load_module
        lib = self._lib = load_module("capi")
        c = ctypes
        lib.ib_api_last_error.restype = c.c_char_p
        lib.ib_engine_create.restype = c.c_void_p
        lib.ib_engine_create.argtypes = [c.c_char_p, c.c_char_p, c.c_uint64, c.c_char_p, c.c_int, c.c_int, c.c_int, c.c_int]
        lib.ib_engine_destroy.argtypes = [c.c_void_p]
        lib.ib_engine_destroy.restype = None
        lib.ib_engine_vocab_size.argtypes = [c.c_void_p]
        lib.ib_engine_vocab_size.restype = c.c_int64
        lib.ib_engine_add_request.argtypes = [c.c_void_p, c.c_int64]
        lib.ib_engine_end_request.argtypes = [c.c_void_p, c.c_int64]
        lib.ib_engine_step.argtypes = [c.c_void_p, c.c_int] + [c.c_void_p] * 6
        lib.ib_engine_step.restype = c.c_int64
        lib.ib_engine_get_logits.argtypes = [c.c_void_p, c.c_void_p, c.c_int64]
        lib.ib_engine_get_logits.restype = c.c_int64
        lib.ib_engine_generate.argtypes = [c.c_void_p, c.c_int, c.c_void_p, c.c_void_p, c.c_int, c.c_float, c.c_uint64, c.c_int64,
                                           c.c_void_p, c.c_void_p]
        self._h = lib.ib_engine_create(model_dir.encode() if model_dir else None, random_spec.encode() if random_spec else None,
                                       weights_seed, dtype.encode(), slots, max_seq, kv_blocks, chunk)
        if not self._h:
            raise CEngineError(self._error())
        self.vocab_size = int(lib.ib_engine_vocab_size(self._h))
        self._rows = 0

    def _error(self) -> str:
        return (self._lib.ib_api_last_error() or b"").decode()

    def _check(self, rc: int) -> int:
        if rc < 0:
            raise CEngineError(self._error())
        return rc

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.ib_engine_destroy(self._h)
            self._h = None

    __del__ = close

    def add_request(self, rid: int) -> None:
        self._check(self._lib.ib_engine_add_request(self._h, rid))

    def end_request(self, rid: int) -> None:
        self._check(self._lib.ib_engine_end_request(self._h, rid))

    def step(self, entries: Sequence, partial: bool = False):
        """entries: (request id, tokens, wanted places). Returns the number of logit rows, or with ``partial`` the pair
        (rows, which entries ran)."""
        ids = np.asarray([e[0] for e in entries], dtype=np.int64)
        n_tokens = np.asarray([len(e[1]) for e in entries], dtype=np.int32)
        n_want = np.asarray([len(e[2]) for e in entries], dtype=np.int32)
        tokens = np.asarray([t for e in entries for t in e[1]], dtype=np.int32)
        want = np.asarray([w for e in entries for w in e[2]], dtype=np.int32)
        ran = np.zeros(len(entries), dtype=np.int32) if partial else None
        p = lambda a: a.ctypes.data if a is not None and a.size else None
        self._rows = self._check(self._lib.ib_engine_step(self._h, len(entries), p(ids), p(n_tokens), p(tokens), p(n_want), p(want), p(ran)))
        return (self._rows, [bool(x) for x in ran]) if partial else self._rows

    def logits(self) -> np.ndarray:
        out = np.empty((self._rows, self.vocab_size), dtype=np.float32)
        rows = self._check(self._lib.ib_engine_get_logits(self._h, out.ctypes.data if out.size else None, out.size))
        return out[:rows]

    def generate(self, prompts: Sequence[Sequence[int]], max_new: int = 16, temperature: float = 0.0, seed: int = 0,
                 eos_id: int = -1) -> List[List[int]]:
        lens = np.asarray([len(p) for p in prompts], dtype=np.int32)
        tokens = np.asarray([t for p in prompts for t in p], dtype=np.int32)
        out = np.zeros((len(prompts), max_new), dtype=np.int32)
        got = np.zeros(len(prompts), dtype=np.int32)
        self._check(self._lib.ib_engine_generate(self._h, len(prompts), lens.ctypes.data, tokens.ctypes.data, max_new,
                                                 float(temperature), seed, eos_id, out.ctypes.data, got.ctypes.data))
        return [out[i, :got[i]].tolist() for i in range(len(prompts))]
