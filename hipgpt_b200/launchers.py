"""Host-side mirror of the attention group of HipGPT's kernel API (include/hip_kernels.h:38-46
in the HipGPT tree) on top of the C ABI.  Names, argument order and meaning are the
reference's; arguments are CUDA float32 torch tensors (or raw device addresses) and the
calls are asynchronous on torch's current stream.  torch is used for device memory and
streams only; every kernel is the library's own.
"""
from __future__ import annotations

import torch

from . import _capi


def _ptr(t):
    if t is None:
        return None
    if isinstance(t, int):
        return t
    if not (t.is_cuda and t.dtype == torch.float32 and t.is_contiguous()):
        raise ValueError("expected a contiguous CUDA float32 tensor")
    return t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def launch_multihead_attention(d_qkv, d_output, d_attn_probs, B: int, S: int, E: int, H: int, *, causal: bool = False):
    """softmax(Q K^T / sqrt(E/H)) V per (batch, head).  d_qkv: three stacked [B*S, E] planes;
    d_output [B*S, E]; d_attn_probs [B, H, S, S] or None.  Not causal unless asked: the
    reference never masks (src/hip_kernels.cpp:287-319)."""
    if H <= 0 or E % H != 0:
        raise ValueError(f"Bad MHA config: E={E} H={H}")   # the reference aborts here
    _capi.check(_capi.lib().hipgpt_mha_forward_planes(_ptr(d_qkv), _ptr(d_output), _ptr(d_attn_probs),
                                                      B, S, E, H, int(causal), _stream()))


def mha_forward(q, k, v, out, probs, B: int, S: int, E: int, H: int, *, causal: bool = False,
                algo: int = _capi.ALGO_AUTO, warps: int = 0):
    """The same on separate Q, K, V planes, with the kernel selector exposed."""
    _capi.check(_capi.lib().hipgpt_mha_forward_ex(_ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(probs),
                                                  B, S, E, H, int(causal), algo, warps, _stream()))


def mha_forward_bf16(d_qkv, d_output, B: int, S: int, E: int, H: int, *, causal: bool = False, variant: int = 0):
    """The launcher's contract with bf16 storage: d_qkv = three stacked [B*S, E] bf16 planes, d_output
    [B*S, E] bf16 (head_dim 64), fp32 accumulation."""
    for t in (d_qkv, d_output):
        if not (t.is_cuda and t.dtype == torch.bfloat16 and t.is_contiguous()):
            raise ValueError("expected a contiguous CUDA bfloat16 tensor")
    plane = B * S * E * 2                                   # bytes
    p = d_qkv.data_ptr()
    _capi.check(_capi.lib().hipgpt_mha_forward_bf16_ex(p, p + plane, p + 2 * plane, d_output.data_ptr(), B, S, E, H, int(causal),
                                                       int(variant), _stream()))


def launch_scaled_dot_product(Q, K, scores, B: int, S: int, D: int):
    _capi.check(_capi.lib().hipgpt_scaled_dot_product(_ptr(Q), _ptr(K), _ptr(scores), B, S, D, _stream()))


def launch_softmax(scores, softmax_out, B: int, S: int):
    _capi.check(_capi.lib().hipgpt_softmax(_ptr(scores), _ptr(softmax_out), B, S, _stream()))


def launch_attention_weighted_sum(softmax, V, output, B: int, S: int, D: int):
    _capi.check(_capi.lib().hipgpt_attention_weighted_sum(_ptr(softmax), _ptr(V), _ptr(output), B, S, D, _stream()))


def decode_scratch_bytes(B: int, H: int, D: int, ctx: int) -> int:
    return int(_capi.lib().hipgpt_mha_decode_scratch_bytes(B, H, D, ctx))


def mha_decode(q, kcache, vcache, out, scratch, B: int, H: int, D: int, ctx: int, cap: int):
    """One query row per (batch, head) over the first ctx rows of the caches."""
    nbytes = 0 if scratch is None else scratch.numel() * scratch.element_size()
    _capi.check(_capi.lib().hipgpt_mha_decode(_ptr(q), _ptr(kcache), _ptr(vcache), _ptr(out), _ptr(scratch), nbytes,
                                              B, H, D, ctx, cap, _stream()))


def mha_forward_host(h_qkv, h_out, h_probs, B: int, S: int, E: int, H: int, *, causal: bool = False):
    """Host buffers in, host buffers out (numpy float32 arrays or CPU torch tensors, ideally
    pinned): the copies and the kernel run inside the call, which returns when h_out is ready."""
    def hp(a):
        if a is None:
            return None
        if isinstance(a, torch.Tensor):
            assert not a.is_cuda and a.dtype == torch.float32 and a.is_contiguous()
            return a.data_ptr()
        assert a.dtype.name == "float32" and a.flags["C_CONTIGUOUS"]
        return a.ctypes.data
    _capi.check(_capi.lib().hipgpt_mha_forward_host(hp(h_qkv), hp(h_out), hp(h_probs), B, S, E, H, int(causal)))


def mha_forward_bf16_host(h_qkv, h_out, B: int, S: int, E: int, H: int, *, causal: bool = False):
    """The host-buffer call for bf16 planes: CPU torch.bfloat16 tensors (ideally pinned), h_qkv three
    stacked [B*S, E] planes, h_out [B*S, E]; head_dim 64."""
    for t in (h_qkv, h_out):
        if not (isinstance(t, torch.Tensor) and not t.is_cuda and t.dtype == torch.bfloat16 and t.is_contiguous()):
            raise ValueError("expected a contiguous CPU bfloat16 tensor")
    _capi.check(_capi.lib().hipgpt_mha_forward_bf16_host(h_qkv.data_ptr(), h_out.data_ptr(), B, S, E, H, int(causal)))
