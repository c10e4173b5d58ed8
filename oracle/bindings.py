"""ctypes bindings for the CPU oracle and, where it was built, the reference's own launchers
compiled for host cores.  TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and
by bench.py's CPU-baseline leg, never by the product package."""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(_HERE, "_build", "libattn_oracle.so")          # pinned: equal to the reference build
ORACLE_FMA_SO = os.path.join(_HERE, "_build", "libattn_oracle_fma.so")  # multiply-accumulates as fmaf, like a GPU
REF_SO = os.path.join(_HERE, "_ref", "libhipgpt_ref.so")

_fp = C.POINTER(C.c_float)
_ip = C.POINTER(C.c_int)


def build(ref_root: str = "/root/reference") -> None:
    """Compile the oracle and, if the reference tree is mounted, oracle/_ref."""
    env = dict(os.environ)
    subprocess.run(["make", "-C", _HERE, f"REF={ref_root}"], check=True, env=env,
                   stdout=subprocess.DEVNULL)


def _f(a):
    if a is None:
        return None
    assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(_fp)


def _i(a):
    assert a.dtype == np.int32 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(_ip)


_oracle = {}
_ref = None


def oracle_lib(fma: bool = False):
    path = ORACLE_FMA_SO if fma else ORACLE_SO
    if path not in _oracle:
        if not os.path.exists(path):
            build()
        _oracle[path] = C.CDLL(path)
    return _oracle[path]


def have_ref() -> bool:
    return os.path.exists(REF_SO)


def ref_lib():
    global _ref
    if _ref is None:
        _ref = C.CDLL(REF_SO)
    return _ref


def num_threads() -> int:
    return int(oracle_lib().oracle_num_threads())


def set_num_threads(n: int) -> None:
    oracle_lib().oracle_set_num_threads(C.c_int(n))


# ---- oracle -----------------------------------------------------------------------------
def mha(qkv: np.ndarray, B: int, S: int, E: int, H: int, causal: bool = False,
        want_probs: bool = False, path: str = "dispatch"):
    """Attention forward on three stacked planes.  path: 'dispatch' follows the launcher's
    rule, 'flash' / 'fallback' force one kernel's arithmetic.  Returns (out, probs|None)."""
    qkv = np.ascontiguousarray(qkv, dtype=np.float32).reshape(3, B * S, E)
    out = np.zeros((B * S, E), dtype=np.float32)
    probs = np.zeros((B, H, S, S), dtype=np.float32) if want_probs else None
    lib = oracle_lib()
    if path == "dispatch":
        rc = lib.oracle_mha_dispatch(_f(qkv), _f(out), _f(probs), B, S, E, H, int(causal))
    else:
        fn = lib.oracle_mha_flash if path == "flash" else lib.oracle_mha_fallback
        rc = fn(_f(qkv[0]), _f(qkv[1]), _f(qkv[2]), _f(out), _f(probs), B, S, E, H, int(causal))
    if rc < 0:
        raise ValueError(f"oracle rejected shape B={B} S={S} E={E} H={H}")
    return out, probs


def sdp(Q: np.ndarray, K: np.ndarray, B: int, S: int, D: int, fma: bool = False) -> np.ndarray:
    scores = np.zeros((B, S, S), dtype=np.float32)
    oracle_lib(fma).oracle_sdp(_f(Q), _f(K), _f(scores), B, S, D)
    return scores


def softmax(scores: np.ndarray, B: int, S: int) -> np.ndarray:
    out = np.zeros((B, S, S), dtype=np.float32)
    oracle_lib().oracle_softmax(_f(scores), _f(out), B, S)
    return out


def weighted_sum(P: np.ndarray, V: np.ndarray, B: int, S: int, D: int, fma: bool = False) -> np.ndarray:
    out = np.zeros((B, S, D), dtype=np.float32)
    oracle_lib(fma).oracle_weighted_sum(_f(P), _f(V), _f(out), B, S, D)
    return out


def decode_row(q, kcache, vcache, B, H, D, ctx, cap) -> np.ndarray:
    out = np.zeros((B, H * D), dtype=np.float32)
    rc = oracle_lib().oracle_decode_row(_f(q), _f(kcache), _f(vcache), _f(out), B, H, D, ctx, cap)
    if rc < 0:
        raise ValueError("oracle rejected decode shape")
    return out


# ---- the reference's own code on host cores ---------------------------------------------
def ref_mha(qkv: np.ndarray, B: int, S: int, E: int, H: int, unique_rows_only: bool = False):
    """launch_multihead_attention of the reference (non-causal, always stores probs)."""
    qkv = np.ascontiguousarray(qkv, dtype=np.float32).reshape(3, B * S, E)
    out = np.zeros((B * S, E), dtype=np.float32)
    probs = np.zeros((B, H, S, S), dtype=np.float32)
    ref_lib().ref_mha(_f(qkv), _f(out), _f(probs), B, S, E, H, int(unique_rows_only))
    return out, probs


def ref_sdp(Q, K, B, S, D):
    scores = np.zeros((B, S, S), dtype=np.float32)
    ref_lib().ref_sdp(_f(Q), _f(K), _f(scores), B, S, D)
    return scores


def ref_softmax(scores, B, S):
    out = np.zeros((B, S, S), dtype=np.float32)
    ref_lib().ref_softmax(_f(scores), _f(out), B, S)
    return out


def ref_weighted_sum(P, V, B, S, D):
    out = np.zeros((B, S, D), dtype=np.float32)
    ref_lib().ref_weighted_sum(_f(P), _f(V), _f(out), B, S, D)
    return out


# ---- whole-model greedy generation (KV-cache form) --------------------------------------
def gpt_weight_count(V, S, E, L, H, F) -> int:
    fn = oracle_lib(True).oracle_gpt_weight_count
    fn.restype = C.c_longlong
    return int(fn(V, S, E, L, H, F))


def gpt_generate(weights: np.ndarray, V, S, E, L, H, F, prompts: np.ndarray, n_new: int, fma: bool = True):
    """Greedy ids [B, n_new] and the logits [B, V] of the last step."""
    B, n_prompt = prompts.shape
    prompts = np.ascontiguousarray(prompts, dtype=np.int32)
    out = np.zeros((B, n_new), dtype=np.int32)
    logits = np.zeros((B, V), dtype=np.float32)
    rc = oracle_lib(fma).oracle_gpt_generate(_f(weights), V, S, E, L, H, F, _i(prompts), B, n_prompt, n_new,
                                             _i(out), _f(logits))
    if rc < 0:
        raise ValueError("oracle rejected the generation request")
    return out, logits


def ref_dropout_forward(x: np.ndarray, p: float, N: int, E: int):
    """The reference's dropout launcher on host cores -> (output, mask)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty_like(x)
    mask = np.empty_like(x)
    lib = ref_lib()
    lib.ref_dropout_forward.restype = None
    lib.ref_dropout_forward.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_int, C.c_int]
    lib.ref_dropout_forward(_f(x), _f(out), _f(mask), p, N, E)
    return out, mask


def ref_embedding_lookup(ids: np.ndarray, tok: np.ndarray, pos: np.ndarray, B: int, S: int, V: int, E: int):
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    out = np.empty((B * S, E), dtype=np.float32)
    lib = ref_lib()
    lib.ref_embedding_lookup.restype = None
    lib.ref_embedding_lookup.argtypes = [C.c_void_p] * 4 + [C.c_int] * 4
    lib.ref_embedding_lookup(_i(ids), _f(tok), _f(pos), _f(out), B, S, V, E)
    return out


def gpt_generate_window(weights: np.ndarray, V, S, E, L, H, F, prompts: np.ndarray, n_new: int, dropout_p: float = 0.1,
                        fma: bool = True):
    """Greedy ids [B, n_new] of the reference's own generation loop (padded window of S ids re-run
    per token) and the logits [B, V] of the last step."""
    B, n_prompt = prompts.shape
    prompts = np.ascontiguousarray(prompts, dtype=np.int32)
    out = np.zeros((B, n_new), dtype=np.int32)
    logits = np.zeros((B, V), dtype=np.float32)
    lib = oracle_lib(fma)
    lib.oracle_gpt_generate_window.restype = C.c_int
    lib.oracle_gpt_generate_window.argtypes = [C.c_void_p] + [C.c_int] * 6 + [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_float,
                                                                              C.c_void_p, C.c_void_p]
    rc = lib.oracle_gpt_generate_window(_f(weights), V, S, E, L, H, F, _i(prompts), B, n_prompt, n_new, dropout_p, _i(out), _f(logits))
    if rc < 0:
        raise ValueError("oracle rejected the generation request")
    return out, logits


def dropout_oracle(x: np.ndarray, p: float):
    """The oracle's restatement of the reference's dropout on a flat array (for the pin against ref_dropout_forward)."""
    x = np.ascontiguousarray(x, dtype=np.float32).ravel()
    out = np.empty_like(x)
    lib = oracle_lib(False)
    lib.oracle_dropout.restype = None
    lib.oracle_dropout.argtypes = [C.c_void_p, C.c_void_p, C.c_longlong, C.c_float]
    lib.oracle_dropout(_f(x), _f(out), x.size, p)
    return out


# ---- the launchers either side of attention (layer norm, projections, embedding, the whole block) ----
def matmul(A: np.ndarray, W: np.ndarray, bias, M: int, N: int, K: int, fma: bool = True) -> np.ndarray:
    """C[M][K] = A[M][N] W[N][K] (+ bias): one accumulator per output, k ascending (fused multiply-add when fma)."""
    out = np.empty((M, K), dtype=np.float32)
    lib = oracle_lib(fma)
    lib.oracle_matmul.restype = None
    lib.oracle_matmul.argtypes = [C.c_void_p] * 4 + [C.c_int] * 3
    lib.oracle_matmul(_f(A), _f(W), _f(bias) if bias is not None else None, _f(out), M, N, K)
    return out


def layer_norm(x: np.ndarray, g: np.ndarray, b: np.ndarray, rows: int, E: int, ref_order: bool = False) -> np.ndarray:
    out = np.empty((rows, E), dtype=np.float32)
    lib = oracle_lib(False)
    lib.oracle_layer_norm.restype = None
    lib.oracle_layer_norm.argtypes = [C.c_void_p] * 4 + [C.c_int] * 3
    lib.oracle_layer_norm(_f(x), _f(out), _f(g), _f(b), rows, E, int(ref_order))
    return out


def embedding(ids: np.ndarray, tok: np.ndarray, pos: np.ndarray, B: int, S: int, V: int, E: int) -> np.ndarray:
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    out = np.empty((B * S, E), dtype=np.float32)
    lib = oracle_lib(False)
    lib.oracle_embedding.restype = None
    lib.oracle_embedding.argtypes = [C.c_void_p] * 4 + [C.c_int] * 4
    lib.oracle_embedding(_i(ids), _f(tok), _f(pos), _f(out), B, S, V, E)
    return out


def layer_forward(x: np.ndarray, w: np.ndarray, B: int, S: int, E: int, H: int, F: int, dropout_p: float = 0.1,
                  fma: bool = True) -> np.ndarray:
    """One HipGPT block (TransformerLayer::forward) on [B*S][E] activations; w = the layer's tensors in checkpoint order."""
    out = np.empty((B * S, E), dtype=np.float32)
    lib = oracle_lib(fma)
    lib.oracle_layer_forward.restype = C.c_int
    lib.oracle_layer_forward.argtypes = [C.c_void_p] * 3 + [C.c_int] * 5 + [C.c_float]
    if lib.oracle_layer_forward(_f(x), _f(w), _f(out), B, S, E, H, F, dropout_p) < 0:
        raise ValueError("oracle rejected the layer")
    return out


# ---- attention backward --------------------------------------------------------------------------------
def mha_backward(gout: np.ndarray, qkv: np.ndarray, probs, B: int, S: int, E: int, H: int, causal: bool = False,
                 fma: bool = False) -> np.ndarray:
    """dQ, dK, dV as three stacked [B*S][E] planes; probs [B][H][S][S] or None (recomputed from Q and K)."""
    out = np.zeros(3 * B * S * E, dtype=np.float32)
    lib = oracle_lib(fma)
    lib.oracle_mha_backward.restype = C.c_int
    lib.oracle_mha_backward.argtypes = [C.c_void_p] * 4 + [C.c_int] * 5
    rc = lib.oracle_mha_backward(_f(gout), _f(qkv), _f(probs) if probs is not None else None, _f(out), B, S, E, H, int(causal))
    if rc < 0:
        raise ValueError("oracle rejected the configuration")
    return out


def ref_mha_backward(gout: np.ndarray, qkv: np.ndarray, probs: np.ndarray, B: int, S: int, E: int, H: int) -> np.ndarray:
    """The reference's own backward launcher on ONE host thread (its atomicAdd is a plain add in the stand-in)."""
    out = np.zeros(3 * B * S * E, dtype=np.float32)
    lib = ref_lib()
    before = lib.ref_num_threads()
    lib.ref_set_num_threads(1)
    try:
        lib.ref_mha_backward.restype = None
        lib.ref_mha_backward.argtypes = [C.c_void_p] * 4 + [C.c_int] * 4
        lib.ref_mha_backward(_f(gout), _f(qkv), _f(probs), _f(out), B, S, E, H)
    finally:
        lib.ref_set_num_threads(before)
    return out
