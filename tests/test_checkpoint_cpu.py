"""CPU tests of the native reader of HipGPT's checkpoint and run-configuration files: a file written in the
reference's layout (GPTModel::save_checkpoint, src/gpt_model.cpp:355-388) reads back to the same tensors, and
damaged files are refused with a reason."""
import os

import numpy as np
import pytest

from hipgpt_b200 import _capi, checkpoint, synth

CFG = dict(V=37, S=12, E=16, L=3, H=4, F=24)


def _write(tmp_path, name="model.bin", **over):
    cfg = dict(CFG, **over)
    w = synth.gpt_weights(5, **cfg)
    w += synth.normal(6, w.shape, 0.01)                   # biases and layer-norm tensors not all 0 / 1
    path = os.path.join(tmp_path, name)
    checkpoint.write_checkpoint(path, w, **cfg)
    return path, w, cfg


def test_checkpoint_round_trip(tmp_path):
    path, w, cfg = _write(tmp_path)
    assert os.path.getsize(path) == 4 * (4 + 3 * cfg["L"] + w.size)
    assert checkpoint.read_header(path) == cfg
    got_cfg, got = checkpoint.read_weights(path)
    assert got_cfg == cfg
    assert np.array_equal(got, w)


def test_run_config_round_trip(tmp_path):
    path, w, cfg = _write(tmp_path, name="run_step40.bin")
    js = os.path.join(tmp_path, "latest_config.json")
    checkpoint.write_run_config(js, cfg["V"], cfg["S"], cfg["E"], cfg["H"], cfg["F"], cfg["L"], "run_step40.bin", "tok.json", step=40)
    got = checkpoint.read_run_config(js)
    assert {k: got[k] for k in "VSEHFL"} == {k: cfg[k] for k in "VSEHFL"}
    assert got["checkpoint"] == "run_step40.bin" and got["tokenizer"] == "tok.json"


def test_damaged_files_are_refused(tmp_path):
    lib = _capi.lib()
    path, w, cfg = _write(tmp_path)
    data = open(path, "rb").read()
    # truncated inside the last layer
    cut = os.path.join(tmp_path, "cut.bin")
    open(cut, "wb").write(data[: len(data) // 2])
    with pytest.raises(_capi.HipGPTError, match="ends"):
        checkpoint.read_weights(cut)
    # trailing bytes
    fat = os.path.join(tmp_path, "fat.bin")
    open(fat, "wb").write(data + b"\x00\x00\x00\x00")
    with pytest.raises(_capi.HipGPTError, match="bytes left"):
        checkpoint.read_weights(fat)
    # a later layer whose header disagrees with the first
    arr = np.frombuffer(data, dtype=np.int32).copy()
    per = checkpoint.layer_floats(cfg["E"], cfg["F"])
    second = 4 + (cfg["V"] + cfg["S"]) * cfg["E"] + 3 + per
    assert arr[second] == cfg["E"] and arr[second + 1] == cfg["H"]
    arr[second + 1] = cfg["H"] * 2
    bad = os.path.join(tmp_path, "bad.bin")
    arr.tofile(bad)
    with pytest.raises(_capi.HipGPTError, match="layer 1 says"):
        checkpoint.read_weights(bad)
    # not a checkpoint at all, a missing file, a buffer of the wrong size
    junk = os.path.join(tmp_path, "junk.bin")
    open(junk, "wb").write(b"\xff" * 64)
    with pytest.raises(_capi.HipGPTError, match="implausible header"):
        checkpoint.read_header(junk)
    with pytest.raises(_capi.HipGPTError, match="cannot open"):
        checkpoint.read_header(os.path.join(tmp_path, "absent.bin"))
    buf = np.empty(10, np.float32)
    assert lib.hipgpt_checkpoint_weights(os.fsencode(path), buf.ctypes.data, 10) == _capi.ERR_BAD_ARG
    # a run configuration without its model keys
    js = os.path.join(tmp_path, "empty.json")
    open(js, "w").write('{"model": {"vocab_size": 3}}')
    with pytest.raises(_capi.HipGPTError, match="missing"):
        checkpoint.read_run_config(js)
