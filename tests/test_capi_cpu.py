"""CPU checks of the drop-in boundary: the library loads without a GPU, exports every symbol
that include/hipgpt_attn.h declares and every reference-named launcher, and the host-only
entry points (sharding arithmetic, error text, size queries) behave."""
import ctypes as C
import os
import re

import pytest

from hipgpt_b200 import _capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "hipgpt_attn.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(hipgpt_[a-z0-9_]+)\s*\(", text)))


def test_header_and_bindings_agree():
    assert _declared_symbols() == sorted(_capi.SIGNATURES)


def test_library_exports_every_declared_symbol():
    lib = _capi.lib()
    for name in _declared_symbols():
        assert hasattr(lib, name), name


def test_library_exports_reference_named_launchers():
    raw = C.CDLL(_capi.lib_path())
    for name, mangled in _capi.CXX_LAUNCHERS.items():
        assert getattr(raw, mangled) is not None, name


def test_reference_objects_would_resolve_against_the_library():
    """The mangled names HipGPT's own objects refer to are the ones g++ makes of the
    declarations in include/hip_kernels.h:39-46; check with the compiler, not by hand."""
    import subprocess
    import tempfile
    src = '#include "hipgpt_launchers.hpp"\nvoid f(const float* a, float* b, const int* i){launch_multihead_attention(a,b,b,1,1,1,1);' \
          'launch_scaled_dot_product(a,a,b,1,1,1);launch_softmax(a,b,1,1);launch_attention_weighted_sum(a,a,b,1,1,1);' \
          'launch_multihead_attention_backward(a,a,a,b,1,1,1,1);launch_matmul(a,a,b,1,1,1);launch_matmul_add_bias(a,a,a,b,1,1,1);' \
          'launch_layer_norm_forward(a,b,a,a,1,1);launch_dropout_forward(a,b,b,0.1f,1,1);launch_add_inplace(b,a,1);launch_relu(b,1);' \
          'launch_embedding_lookup(i,a,a,b,1,1,1,1);}\n'
    with tempfile.TemporaryDirectory() as td:
        cpp = os.path.join(td, "t.cpp")
        open(cpp, "w").write(src)
        obj = os.path.join(td, "t.o")
        subprocess.run(["g++", "-c", "-I", os.path.join(ROOT, "include"), cpp, "-o", obj], check=True)
        undefined = subprocess.run(["nm", "-u", obj], check=True, capture_output=True, text=True).stdout
    for mangled in _capi.CXX_LAUNCHERS.values():
        assert mangled in undefined


def test_version_and_error_text():
    lib = _capi.lib()
    assert lib.hipgpt_version() >= 100
    b0, b1 = C.c_int(), C.c_int()
    rc = lib.hipgpt_shard_range(8, 0, 0, C.byref(b0), C.byref(b1))
    assert rc == _capi.ERR_BAD_ARG
    assert b"world=0" in lib.hipgpt_last_error()
    with pytest.raises(_capi.HipGPTError):
        _capi.check(rc)


@pytest.mark.parametrize("B,world", [(64, 8), (32, 1), (10, 4), (3, 8), (0, 2), (7, 7)])
def test_shard_range_partitions_batches(B, world):
    lib = _capi.lib()
    covered = []
    sizes = []
    for r in range(world):
        b0, b1 = C.c_int(), C.c_int()
        assert lib.hipgpt_shard_range(B, world, r, C.byref(b0), C.byref(b1)) == 0
        covered += list(range(b0.value, b1.value))
        sizes.append(b1.value - b0.value)
    assert covered == list(range(B))            # contiguous, ordered, no gaps, no overlap
    assert max(sizes) - min(sizes) <= 1


def test_bad_arguments_are_rejected_before_any_cuda_call():
    lib = _capi.lib()
    # E % H != 0 and H <= 0: the reference aborts (src/hip_kernels.cpp:410-413); the C ABI returns a code
    assert lib.hipgpt_mha_forward(None, None, None, None, None, 1, 4, 30, 4, 0, None) == _capi.ERR_BAD_ARG
    assert b"Bad MHA config" in lib.hipgpt_last_error()
    assert lib.hipgpt_mha_forward(None, None, None, None, None, 1, 4, 32, 0, 0, None) == _capi.ERR_BAD_ARG
    assert lib.hipgpt_mha_forward(None, None, None, None, None, 1, 4, 32, 1, 0, None) == _capi.ERR_NULL
    assert lib.hipgpt_mha_forward(None, None, None, None, None, -1, 4, 32, 1, 0, None) == _capi.ERR_BAD_ARG
    # empty problems succeed without touching a pointer
    assert lib.hipgpt_mha_forward(None, None, None, None, None, 0, 4, 32, 1, 0, None) == 0
    assert lib.hipgpt_mha_forward(None, None, None, None, None, 2, 0, 32, 1, 0, None) == 0
    assert lib.hipgpt_scaled_dot_product(None, None, None, 1, 4, 0, None) == _capi.ERR_BAD_ARG
    assert lib.hipgpt_softmax(None, None, 1, 4, None) == _capi.ERR_NULL
    assert lib.hipgpt_mha_decode(None, None, None, None, None, 0, 1, 1, 32, 5, 4, None) == _capi.ERR_BAD_ARG  # ctx > cap


def test_projection_and_sharding_entry_points_check_their_arguments_first():
    """The entry points added beside attention (tensor-core projections, fused dropout + residual, the sharded driver's
    transports) refuse bad sizes, NULL pointers and in-place use before any CUDA call, so on a box without a GPU too."""
    lib = _capi.lib()
    one = (C.c_float * 4)()
    p = C.cast(one, C.c_void_p)
    assert lib.hipgpt_matmul_tc(None, None, None, None, -1, 4, 4, None) == _capi.ERR_BAD_ARG
    assert lib.hipgpt_matmul_tc(None, None, None, None, 4, 4, 4, None) == _capi.ERR_NULL
    assert lib.hipgpt_matmul_tc(None, None, None, None, 0, 4, 4, None) == 0                       # nothing to do
    assert lib.hipgpt_matmul_tc(p, p, None, p, 2, 2, 2, None) == _capi.ERR_UNSUPPORTED             # in place
    assert b"in place" in lib.hipgpt_last_error()
    h = C.c_void_p()
    assert lib.hipgpt_matmul_tc_prepare(None, 4, 4, C.byref(h), None) == _capi.ERR_NULL
    assert lib.hipgpt_matmul_tc_prepare(p, 0, 4, C.byref(h), None) == _capi.ERR_BAD_ARG
    assert lib.hipgpt_matmul_tc_prepared(p, None, None, p, 2, None) == _capi.ERR_NULL
    assert lib.hipgpt_ln_matmul_tc(p, None, None, p, None, p, 2, 2, 2, None) == _capi.ERR_NULL      # gamma and beta are required
    assert lib.hipgpt_ln_matmul_tc(p, p, p, p, None, p, 2, 0, 2, None) == _capi.ERR_BAD_ARG         # a layer norm over nothing
    lib.hipgpt_matmul_tc_release(None)                                                              # accepted, like free(NULL)
    assert lib.hipgpt_dropout_residual(p, p, p, None, C.c_float(1.0), 1, 4, None) == _capi.ERR_BAD_ARG   # p must be below 1
    assert lib.hipgpt_dropout_residual(None, p, p, None, C.c_float(0.1), 1, 4, None) == _capi.ERR_NULL
    assert lib.hipgpt_dropout_residual(None, None, None, None, C.c_float(0.1), 0, 4, None) == 0
    assert lib.hipgpt_mha_forward_sharded(None, p, p, p, p, 8, 4, 32, 1, 0, 4, 1, 0, None) == _capi.ERR_NULL       # no context
    assert lib.hipgpt_shard_output_buffer(None, 16, C.byref(h)) == _capi.ERR_NULL
    b0, b1 = C.c_int(), C.c_int()
    assert lib.hipgpt_shard_chunk_range(10, 2, 0, 3, 0, C.byref(b0), C.byref(b1)) == _capi.ERR_BAD_ARG      # 10 batches do not split into 2 x 3 runs
    assert lib.hipgpt_shard_chunk_range(12, 2, 1, 3, 2, C.byref(b0), C.byref(b1)) == 0 and (b0.value, b1.value) == (10, 12)


def test_decode_scratch_size_query():
    lib = _capi.lib()
    assert lib.hipgpt_mha_decode_scratch_bytes(8, 8, 32, 256) > 0
    assert lib.hipgpt_mha_decode_scratch_bytes(8, 8, 32, 16) == 0       # one split: no scratch
    assert lib.hipgpt_mha_decode_scratch_bytes(1024, 8, 32, 256) == 0   # enough rows already
    assert lib.hipgpt_mha_decode_scratch_bytes(0, 8, 32, 256) == 0


REFERENCE = os.environ.get("HIPGPT_REFERENCE", "/root/reference")   # the HipGPT tree

# launchers that HipGPT's layer and model sources name but only its training path calls: outside this library
TRAINING_ONLY = {"launch_matmul_backward_bias", "launch_matmul_transpose_A", "launch_matmul_transpose_B", "launch_backprop_activation",
                 "launch_embedding_backward", "launch_adam_update", "launch_layer_norm_backward", "launch_dropout_backward",
                 "launch_l2_accumulate", "launch_scale_inplace"}


@pytest.mark.skipif(not os.path.exists(os.path.join(REFERENCE, "src", "transformer_layer.cpp")), reason="reference tree not mounted")
def test_reference_layer_and_model_resolve_their_forward_path_against_the_library():
    """HipGPT's own src/transformer_layer.cpp and src/gpt_model.cpp, compiled where they lie: every launch_* symbol
    they leave undefined is either exported by this library under exactly that mangled name, or belongs to the
    training path (backward passes, Adam, clipping).  oracle/Makefile links the two objects with the library into
    oracle/_ref/ref_model_run, the program the GPU tests run; nothing is stubbed with an empty function."""
    import subprocess
    import tempfile
    shim = os.path.join(ROOT, "oracle", "ref_shim_cuda")
    exported = subprocess.run(["nm", "-D", "--defined-only", _capi.lib_path()], check=True, capture_output=True, text=True).stdout
    with tempfile.TemporaryDirectory() as td:
        for name in ("transformer_layer", "gpt_model"):
            obj = os.path.join(td, name + ".o")
            subprocess.run(["g++", "-std=c++17", "-O1", "-w", "-I", shim, "-I", os.path.join(REFERENCE, "include"), "-I", "/usr/local/cuda/include",
                            "-c", os.path.join(REFERENCE, "src", name + ".cpp"), "-o", obj], check=True)
            undefined = subprocess.run(["nm", "-u", obj], check=True, capture_output=True, text=True).stdout.split()
            wanted = [u for u in undefined if "launch_" in u]
            assert wanted
            for sym in wanted:
                plain = subprocess.run(["c++filt", sym], check=True, capture_output=True, text=True).stdout.split("(")[0].strip()
                assert sym in exported or plain in TRAINING_ONLY, f"{name}.cpp needs {plain}, which the library does not export"
            if name == "transformer_layer":
                for must in ("launch_multihead_attention", "launch_matmul_add_bias", "launch_layer_norm_forward", "launch_dropout_forward",
                             "launch_multihead_attention_backward"):
                    assert _capi.CXX_LAUNCHERS[must] in wanted and _capi.CXX_LAUNCHERS[must] in exported
    assert os.path.exists(os.path.join(ROOT, "oracle", "_ref", "ref_model_run")), "run `make -C oracle` (or __graft_entry__.build())"
