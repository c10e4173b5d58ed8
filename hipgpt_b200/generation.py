"""Host-side handle on the library's greedy KV-cache generation (hipgpt_gpt_* in
include/hipgpt_attn.h), the driver that stands where GPTModel::generate's loop stands in the
reference (src/gpt_model.cpp:248-353).  Host numpy arrays in, host numpy arrays out."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _capi


MODE_GRAPH = 0          # one step = a CUDA graph of 52 launches, replayed per token (default)
MODE_PERSISTENT = 1     # one cooperative launch for a run of token steps, phases separated by a barrier over the grid


class GptDecoder:
    def __init__(self, weights: np.ndarray, V: int, S: int, E: int, L: int, H: int, F: int, max_batch: int = 8,
                 mode: int | None = None):
        lib = _capi.lib()
        need = int(lib.hipgpt_gpt_weight_count(V, S, E, L, H, F))
        weights = np.ascontiguousarray(weights, dtype=np.float32)
        if weights.size != need:
            raise ValueError(f"weight blob has {weights.size} floats, the shape needs {need}")
        self.shape = (V, S, E, L, H, F)
        self._h = C.c_void_p()
        _capi.check(lib.hipgpt_gpt_create(C.byref(self._h), weights.ctypes.data, V, S, E, L, H, F, max_batch))
        if mode is not None:
            self.set_mode(mode)

    @classmethod
    def from_checkpoint(cls, path: str, max_batch: int = 8, mode: int | None = None):
        """A HipGPT checkpoint file (GPTModel::save_checkpoint's layout) or, for a path ending in .json, the run
        configuration that names it (src/train_gpt.cpp:60-102); read by the library's native reader."""
        import os
        from . import checkpoint
        lib = _capi.lib()
        self = cls.__new__(cls)
        self._h = C.c_void_p()
        if path.endswith(".json"):
            cfg = checkpoint.read_run_config(path)
            _capi.check(lib.hipgpt_gpt_create_from_run(C.byref(self._h), os.fsencode(path), max_batch))
        else:
            cfg = checkpoint.read_header(path)
            _capi.check(lib.hipgpt_gpt_create_from_checkpoint(C.byref(self._h), os.fsencode(path), max_batch))
        self.shape = (cfg["V"], cfg["S"], cfg["E"], cfg["L"], cfg["H"], cfg["F"])
        if mode is not None:
            self.set_mode(mode)
        return self

    def set_mode(self, mode: int):
        _capi.check(_capi.lib().hipgpt_gpt_set_mode(self._h, int(mode)))

    def generate(self, prompts: np.ndarray, n_new: int):
        """prompts [B, n_prompt] int32 -> (ids [B, n_new], logits of the last step [B, V],
        device ms of the prompt steps, device ms of the remaining n_new-1 steps)."""
        prompts = np.ascontiguousarray(prompts, dtype=np.int32)
        B, n_prompt = prompts.shape
        ids = np.zeros((B, n_new), dtype=np.int32)
        logits = np.zeros((B, self.shape[0]), dtype=np.float32)
        a, b = C.c_float(), C.c_float()
        _capi.check(_capi.lib().hipgpt_gpt_generate(self._h, prompts.ctypes.data, B, n_prompt, n_new, ids.ctypes.data,
                                                    logits.ctypes.data, C.byref(a), C.byref(b)))
        return ids, logits, a.value, b.value

    def close(self):
        if self._h:
            _capi.lib().hipgpt_gpt_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
