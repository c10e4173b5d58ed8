"""HipGPT's checkpoint and run-configuration files from Python: thin bindings over the library's native
reader (hipgpt_checkpoint_* / hipgpt_run_config in include/hipgpt_attn.h), and a writer of the same layout
(GPTModel::save_checkpoint, src/gpt_model.cpp:355-388 with src/transformer_layer.cpp:312-344; save_config,
src/train_gpt.cpp:60-102 in the HipGPT tree) for tests and for handing weights to HipGPT's own classes."""
from __future__ import annotations

import ctypes as C
import json
import os

import numpy as np

from . import _capi


def read_header(path: str) -> dict:
    v = [C.c_int() for _ in range(6)]
    _capi.check(_capi.lib().hipgpt_checkpoint_header(os.fsencode(path), *[C.byref(x) for x in v]))
    return dict(zip(("V", "S", "E", "L", "H", "F"), (x.value for x in v)))


def read_weights(path: str):
    """(shape dict, the tensors in file order without the integer headers: what GptDecoder takes)."""
    lib = _capi.lib()
    cfg = read_header(path)
    n = int(lib.hipgpt_gpt_weight_count(cfg["V"], cfg["S"], cfg["E"], cfg["L"], cfg["H"], cfg["F"]))
    w = np.empty(n, dtype=np.float32)
    _capi.check(lib.hipgpt_checkpoint_weights(os.fsencode(path), w.ctypes.data, n))
    return cfg, w


def read_run_config(path: str) -> dict:
    lib = _capi.lib()
    v = [C.c_int() for _ in range(6)]
    ckpt, tok = C.create_string_buffer(512), C.create_string_buffer(512)
    _capi.check(lib.hipgpt_run_config(os.fsencode(path), *[C.byref(x) for x in v], ckpt, 512, tok, 512))
    out = dict(zip(("V", "S", "E", "H", "F", "L"), (x.value for x in v)))
    out["checkpoint"] = ckpt.value.decode()
    out["tokenizer"] = tok.value.decode()
    return out


def layer_floats(E: int, F: int) -> int:
    return E * 3 * E + E * E + E * F + F * E + 3 * E + E + F + E + 4 * E


def write_layer(f, w: np.ndarray, E: int, H: int, F: int) -> None:
    """One layer as TransformerLayer::save writes it: int32 E, H, F, then its tensors."""
    assert w.dtype == np.float32 and w.size == layer_floats(E, F)
    np.array([E, H, F], dtype=np.int32).tofile(f)
    w.tofile(f)


def write_checkpoint(path: str, weights: np.ndarray, V: int, S: int, E: int, L: int, H: int, F: int) -> None:
    """`weights`: the header-less blob (synth.gpt_weights order) -> a file GPTModel::load_checkpoint reads."""
    weights = np.ascontiguousarray(weights, dtype=np.float32)
    per = layer_floats(E, F)
    assert weights.size == (V + S) * E + L * per + E * V
    with open(path, "wb") as f:
        np.array([V, S, E, L], dtype=np.int32).tofile(f)
        o = (V + S) * E
        weights[:o].tofile(f)
        for _ in range(L):
            write_layer(f, weights[o:o + per], E, H, F)
            o += per
        weights[o:].tofile(f)


def write_run_config(path: str, V: int, S: int, E: int, H: int, F: int, L: int, checkpoint: str, tokenizer: str = "tokenizer.json",
                     step: int = 0) -> None:
    cfg = {"model": {"vocab_size": V, "max_seq_len": S, "embed_dim": E, "num_heads": H, "ff_hidden_dim": F, "num_layers": L},
           "tokenizer": {"path": tokenizer, "tokens_path": "tokens.bin"},
           "training": {"batch_size": 32, "learning_rate": 3e-4, "warmup_steps": 0, "min_lr": 1e-5, "steps": step},
           "checkpoint": {"latest": checkpoint, "step": step}}
    with open(path, "w") as f:
        json.dump(cfg, f, indent=4)
