"""Python handle on the native sequence-model engine (wf_seq_* in include/wf_seq.h): weights in, sequences admitted into state slots,
ragged steps of prompt portions and single tokens, logits or sampled tokens out.  numpy and ctypes only."""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence, Tuple

import numpy as np

from . import _lib
from ._lib import SeqConfig, SeqLayer, seq_check, seq_lib


def _i32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.int32)


class SeqEngine:
    def __init__(self, cfg: SeqConfig, layers: Sequence[SeqLayer], build: bool = False):
        L = seq_lib(build=build)
        if not L.wf_seq_available():
            raise _lib.WfError("no compute-capability-10.x CUDA device visible; the sequence-model kernels are sm_100a-only and there is no CPU fallback")
        self.cfg = cfg
        self.layers = list(layers)
        arr = (SeqLayer * len(self.layers))(*self.layers)
        h = C.c_void_p()
        seq_check(L.wf_seq_create(C.byref(cfg), arr, C.byref(h)))
        self._h = h
        self.vocab, self.width = cfg.vocab, cfg.width
        self.float32 = cfg.dtype == _lib.WF_SEQ_F32

    def close(self):
        if getattr(self, "_h", None):
            seq_lib().wf_seq_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- weights
    def expected_tensors(self) -> List[Tuple[str, int, bool]]:
        L = seq_lib()
        out = []
        for i in range(L.wf_seq_tensor_count(self._h)):
            n, ld = C.c_size_t(), C.c_int()
            name = L.wf_seq_tensor_name(self._h, i, C.byref(n), C.byref(ld))
            out.append((name.decode(), int(n.value), bool(ld.value)))
        return out

    def set_tensor(self, name: str, a: np.ndarray) -> None:
        """a: float32 values (float32 engine) or uint16 bfloat16 bit patterns (bfloat16 engine), any shape, C order."""
        want = np.float32 if self.float32 else np.uint16
        if a.dtype != want:
            raise TypeError(f"{name}: engine storage is {np.dtype(want).name}, got {a.dtype}")
        a = np.ascontiguousarray(a)
        seq_check(seq_lib().wf_seq_set_tensor(self._h, name.encode(), a.ctypes.data, a.size, 1))

    def finalize(self) -> None:
        seq_check(seq_lib().wf_seq_finalize(self._h))

    def device_bytes(self) -> int:
        return int(seq_lib().wf_seq_device_bytes(self._h))

    # ---- sequences
    def admit(self) -> int:
        s = C.c_int(-1)
        seq_check(seq_lib().wf_seq_admit(self._h, C.byref(s)))
        return int(s.value)

    def release(self, slot: int) -> None:
        seq_check(seq_lib().wf_seq_release(self._h, slot))

    def length(self, slot: int) -> int:
        return int(seq_lib().wf_seq_length(self._h, slot))

    def free_pages(self) -> int:
        return int(seq_lib().wf_seq_free_pages(self._h))

    def free_slots(self) -> int:
        return int(seq_lib().wf_seq_free_slots(self._h))

    # ---- steps
    def step(self, slots: Sequence[int], counts: Sequence[int], tokens: Sequence[int], want: Sequence[int] = (), fetch: bool = True) -> Optional[np.ndarray]:
        """One ragged step. want: indices into the flat token list; returns float32 [len(want), vocab] (None when nothing is wanted or fetch is off)."""
        s, c, t, w = _i32(slots), _i32(counts), _i32(tokens), _i32(want)
        if t.size != int(c.sum()):
            raise ValueError(f"{t.size} tokens for counts summing to {int(c.sum())}")
        out = np.empty((w.size, self.vocab), dtype=np.float32) if (fetch and w.size) else None
        seq_check(seq_lib().wf_seq_step(self._h, s.size, s.ctypes.data, c.ctypes.data, t.ctypes.data, w.size, w.ctypes.data if w.size else None,
                                        out.ctypes.data if out is not None else None))
        return out

    def sample(self, nrows: int, temperature: float = 0.0, top_k: int = 0, top_p: float = 1.0, uniforms: Optional[np.ndarray] = None) -> np.ndarray:
        nxt = np.empty(nrows, dtype=np.int32)
        u = np.ascontiguousarray(uniforms, dtype=np.float32) if uniforms is not None else None
        seq_check(seq_lib().wf_seq_sample(self._h, nrows, float(temperature), int(top_k), float(top_p), u.ctypes.data if u is not None else None, nxt.ctypes.data))
        return nxt

    def launches_last_step(self) -> int:
        return int(seq_lib().wf_seq_launches_last_step(self._h))

    # ---- parity taps / measurement
    def step_with_layer_tap(self, slots, counts, tokens, want=()):
        n = int(np.sum(counts))
        tap = np.empty((self.cfg.n_layers, n, self.width), dtype=np.float32)
        seq_check(seq_lib().wf_seq_set_layer_tap(self._h, tap.ctypes.data))
        try:
            out = self.step(slots, counts, tokens, want)
        finally:
            seq_check(seq_lib().wf_seq_set_layer_tap(self._h, None))
        return out, tap

    def run_part(self, layer: int, part: int, slots, counts, rows: np.ndarray) -> np.ndarray:
        s, c = _i32(slots), _i32(counts)
        x = np.ascontiguousarray(rows, dtype=np.float32)
        if x.shape != (int(c.sum()), self.width):
            raise ValueError(f"rows must be [{int(c.sum())}, {self.width}]")
        out = np.empty_like(x)
        seq_check(seq_lib().wf_seq_run_part(self._h, layer, part, s.size, s.ctypes.data, c.ctypes.data, x.ctypes.data, out.ctypes.data))
        return out

    def time_step(self, slots, counts, iters: int = 10) -> float:
        s, c = _i32(slots), _i32(counts)
        ms = C.c_float()
        seq_check(seq_lib().wf_seq_time_step(self._h, s.size, s.ctypes.data, c.ctypes.data, iters, C.byref(ms)))
        return float(ms.value)

    def profile_step(self, slots, counts, iters: int = 5) -> dict:
        """{launch group: (ms per step, launch groups per step)} with an event after every launch group (slower than time_step)."""
        import json
        s, c = _i32(slots), _i32(counts)
        buf = C.create_string_buffer(1 << 16)
        seq_check(seq_lib().wf_seq_profile_step(self._h, s.size, s.ctypes.data, c.ctypes.data, iters, buf, len(buf)))
        return {k: tuple(v) for k, v in json.loads(buf.value.decode()).items()}

    def set_length(self, slot: int, length: int) -> None:
        seq_check(seq_lib().wf_seq_set_length(self._h, slot, length))
