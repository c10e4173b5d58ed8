#!/usr/bin/env python
"""Benchmark of the causal multi-head-attention forward path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload c2|c3|c5] [--causal 0|1] [--probs 0|1] [--gather 0|1]
                    [--kernel auto|whole_head|tiled|split_tf32|rows|generic] [--dtype f32|bf16]

One JSON line on stdout (rank 0).  A *step* is one pass of the attention forward over SETS
different input batches of the workload's shape, one kernel launch per batch; the SETS batches
together are larger than the 126 MB L2, so no launch finds its inputs cached by the one before.
Default workload: B=32 H=8 S=256 head_dim=32, fp32, causal, probabilities not stored.

  value     algorithmic TFLOP/s (2*B*H*D*S*(S+1) per causal batch), inputs resident in HBM,
            CUDA events around the K timed steps, max over ranks
  e2e       the same metric through the host-buffer C-ABI call (pinned host memory in, host
            memory out), copies inside the timed region
  roofline  the attention kernel against the roofline that binds it: the measured HBM copy rate when
            moving the algorithmic bytes takes longer than the tensor pipe needs for the products
            (workload c2), else the measured tensor rate; the fp32 FFMA ceiling timed in the same
            run is reported beside it
  scaling_c5  (default run) the largest workload through the sharded C-ABI driver: compute alone,
            compute in chunks, and with the all-gather of the outputs beside it when N > 1 (NCCL, and
            the library's own transports into the peers' mapped buffers: stores of a copy kernel, copy-engine copies)
  cpu_baseline  the CPU oracle (a port of the reference arithmetic) on this box's host cores
  decode, projections, attention_block  (default run) the greedy generation driver, the matmuls either side of attention, and
            the layer's QKV projection + attention + output projection as one sequence

With N > 1 (torchrun, one rank per GPU) every rank runs the same step on its own batches
(batch-major shards of an N-times larger batch; no kernel reads another GPU's memory), and
--gather 1 adds an NCCL all-gather of the outputs.  `--impl reference` times the reference
arithmetic on the host cores instead (rank 0 only).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from hipgpt_b200 import synth  # noqa: E402

L2_BYTES = 126 * 1024 * 1024
# dram__bytes_read.sum + dram__bytes_write.sum per launch, from the ncu capture that the named summary under
# profiles/ records: (workload, kernel) -> (bytes, summary).  A kernel without a capture of its own reports null.
TRAFFIC = {("c2", "mha_head_kernel"): (25.25e6, "profiles/mha_head_kernel_c2_causal.md")}
FALLBACK_HBM_GBS = 6650.0
# --kernel: name -> (algo, tensor-kernel selector) of hipgpt_mha_forward_ex, and the kernel's name in a launch list
KERNELS = {"auto": None, "whole_head": (3, 6, "mha_head_kernel"), "tiled": (3, 5, "mha_tc16_kernel"),
           "split_tf32": (3, 1, "mha_tc_kernel"), "rows": (2, 0, "mha_rows_kernel"), "generic": (1, 0, "mha_generic_kernel")}


def flops_of(B, H, S, D, causal):
    return 2.0 * B * H * D * S * (S + 1) if causal else 4.0 * B * H * float(S) * S * D


def tiled_launches(B, H, S, D, causal=True):
    """Kernels one call of the tiled fp32 kernel launches: the library cuts the batches into groups whose packed K
    and V (as many bytes as the fp32 K and V) stay below 96 MB, and runs a pack kernel and an attention kernel per group
    (mirrors launch_tc16_cfg in attn_fwd_tc16.cu)."""
    per_batch = H * ((S + 63) // 64) * 64 * 2 * D * 2 * 2
    gb = max(1, (int(os.environ.get("HIPGPT_PACK_GROUP_MB", "96")) << 20) // per_batch)
    env = os.environ.get("HIPGPT_PACK_OVERLAP", "")
    overlap = (not causal) if env == "" else env[:1] != "0"
    if B > gb and gb >= 2 and overlap:
        gb //= 2                                   # several groups: two half-size buffers, group g + 1 packed while g is attended to
    gb = min(gb, B)
    return 2 * ((B + gb - 1) // gb)


def bytes_of(B, H, S, D, probs):
    return 4.0 * B * S * H * D * 4 + (4.0 * B * H * S * S if probs else 0.0)


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=50)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(synth.CONFIGS))
    ap.add_argument("--causal", type=int, default=1)
    ap.add_argument("--dtype", default="f32", choices=["f32", "bf16"], help="storage type of Q, K, V and the output (bf16: head_dim 64)")
    ap.add_argument("--probs", type=int, default=0)
    ap.add_argument("--gather", type=int, default=0)
    ap.add_argument("--strong", type=int, default=0, help="1: the workload's batches are split over the ranks (strong scaling)")
    ap.add_argument("--sets", type=int, default=0, help="input batches per step (0: enough to exceed L2)")
    ap.add_argument("--cpu-seconds", type=float, default=12.0, help="budget of the CPU-baseline leg")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--decode-only", action="store_true", help="run only the greedy-generation leg and print its JSON")
    ap.add_argument("--projections-only", action="store_true", help="run only the projections leg (the matmuls either side of attention) and print its JSON")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-scaling", action="store_true", help="skip the C5 sharded leg (key scaling_c5)")
    ap.add_argument("--kernel", default="auto", choices=sorted(KERNELS),
                    help="fp32 attention kernel: auto is what hipgpt_mha_forward picks; the others go through hipgpt_mha_forward_ex")
    ap.add_argument("--bf16-variant", type=int, default=0, help="--dtype bf16: passed to hipgpt_mha_forward_bf16_ex (0, 1, 2 run the same kernel)")
    return ap.parse_args()


# ------------------------------------------------------------------------------- clocks ----
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU while the timed region runs."""
    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown",
               0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown"}

    def __init__(self, index: int, period: float = 0.02):
        self.index, self.period = index, period
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._nv = None

    def _run(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)))
                try:
                    mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self._h))
                except Exception:
                    mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h))
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(self.period)

    def __enter__(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["unsampled"]}
        return {"sm_mhz": int(np.median(self.samples)), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ---------------------------------------------------------------------------- CPU legs ----
def cpu_leg(cfg, causal, seconds, steps=None, warmup=0):
    """Times the CPU oracle (port of src/hip_kernels.cpp:263-402 with the causal switch) with all
    host threads on a bounded sample: whole batch items of the workload, as many as fit the
    time budget.  Returns (tflops, info dict)."""
    from oracle import bindings as ob
    B, H, S, D = cfg["B"], cfg["H"], cfg["S"], cfg["D"]
    E = H * D
    threads = os.cpu_count() or ob.num_threads()     # every host thread, whatever OMP_NUM_THREADS the launcher set
    ob.set_num_threads(threads)
    one = synth.qkv_planes(cfg["seed"], 1, S, E, cfg["scale"])
    t0 = time.perf_counter()
    ob.mha(one, 1, S, E, H, causal=bool(causal))
    t_item = max(time.perf_counter() - t0, 1e-6)
    n_steps = steps if steps is not None else 3
    items = int(max(1, min(B, seconds / ((n_steps + warmup) * t_item))))
    qkv = np.ascontiguousarray(np.concatenate([one] * items, axis=1)) if items > 1 else one
    for _ in range(warmup):
        ob.mha(qkv, items, S, E, H, causal=bool(causal))
    times = []
    for _ in range(n_steps):
        t0 = time.perf_counter()
        ob.mha(qkv, items, S, E, H, causal=bool(causal))
        times.append(time.perf_counter() - t0)
    t = float(np.mean(times))
    tf = flops_of(items, H, S, D, causal) / t / 1e12
    info = {"value": tf, "unit": "TFLOP/s", "cores": threads, "kind": "port",
            "sample": f"{items} of {B} batch items (all {H} heads, S={S}, D={D}, causal={int(bool(causal))}) per step, "
                      f"{n_steps} steps, mean {t * 1e3:.1f} ms/step",
            "ms_per_step": t * 1e3}
    if ob.have_ref() and S <= 1024:
        # the reference's own launcher on host cores (never causal, always stores probabilities);
        # block rows that repeat the same query are skipped, which changes no result
        ob.ref_lib().ref_set_num_threads(threads)
        t0 = time.perf_counter()
        ob.ref_mha(one, 1, S, E, H, unique_rows_only=True)
        tr = time.perf_counter() - t0
        info["reference_build_noncausal"] = {"tflops": flops_of(1, H, S, D, False) / tr / 1e12,
                                             "sample": "1 batch item, launch_multihead_attention compiled for the host"}
    return tf, info


def projections_leg(lib, fma_peak=None):
    """The projections either side of attention at the default workload's shapes (QKV: [B*S, E] x [E, 3E]; output: [B*S, E] x
    [E, E], bias added): the exact-order kernel (bit-identical to the reference's summation order) and the tensor-core kernel
    (fp32-grade), CUDA-event time per call over input batches that together exceed L2."""
    import torch
    c = synth.CONFIGS["c2"]
    M, E = c["B"] * c["S"], c["H"] * c["D"]
    st = torch.cuda.current_stream().cuda_stream
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        peaks = {}
    tf32_peak = float(peaks.get("bf16_tflops", 1590.0)) / 2.0
    out = {}
    for name, (N, K) in (("qkv", (E, 3 * E)), ("out", (E, E))):
        sets = 8
        A = torch.randn((sets, M, N), device="cuda")
        W = torch.randn((N, K), device="cuda") * 0.05
        b = torch.randn((K,), device="cuda")
        Cc = torch.empty((sets, M, K), device="cuda")
        res = {"M": M, "N_inner": N, "K_out": K, "flops": 2.0 * M * N * K}
        import ctypes
        packed = ctypes.c_void_p()
        _capi_check(lib.hipgpt_matmul_tc_prepare(W.data_ptr(), N, K, ctypes.byref(packed), st))
        for label, fn in (("tensor_core", lib.hipgpt_matmul_tc), ("tensor_core_weights_packed_once", None), ("exact_order", lib.hipgpt_matmul)):
            def step():
                for s in range(sets):
                    if fn is None:
                        rc = lib.hipgpt_matmul_tc_prepared(A[s].data_ptr(), packed, b.data_ptr(), Cc[s].data_ptr(), M, st)
                    else:
                        rc = fn(A[s].data_ptr(), W.data_ptr(), b.data_ptr(), Cc[s].data_ptr(), M, N, K, st)
                    if rc:
                        _capi_check(rc)
            for _ in range(3):
                step()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            reps = 10
            e0.record()
            for _ in range(reps):
                step()
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) / reps / sets * 1e3
            tfl = 2.0 * M * N * K / us / 1e6
            res[label] = {"us_per_call": us, "tflops": tfl}
            # what bounds each kernel: the tensor pipe for the fp16-piece product (three fp16 products per product = 1.5
            # products at the TF32 rate, which is half the measured dense bf16 rate), the FFMA pipe for the exact order
            if fn is not lib.hipgpt_matmul:
                res[label]["roofline"] = {"bound": "tensor", "achieved": 1.5 * tfl, "peak": tf32_peak, "unit": "TFLOP/s", "frac": 1.5 * tfl / tf32_peak,
                                          "peak_source": "half of MEASURED_PEAKS.json bf16_tflops" + ("" if peaks else " (fallback)")}
            elif fma_peak:
                res[label]["roofline"] = {"bound": "fma", "achieved": tfl, "peak": fma_peak, "unit": "TFLOP/s", "frac": tfl / fma_peak,
                                          "peak_source": "fp32 FFMA loop timed in this run"}
        out[name] = res
        torch.cuda.synchronize()
        lib.hipgpt_matmul_tc_release(packed)
        del A, W, b, Cc
    return out


def attention_block_leg(lib):
    """TransformerLayer::self_attention_forward's three launches at the default workload (src/transformer_layer.cpp:214-222:
    QKV projection with bias, launch_multihead_attention on the [T, 3E] output read as three stacked planes, output
    projection with bias), non-causal like the reference: with the exact-order matmul and stored probabilities (what the
    reference's layer asks for, in place output projection), and with the tensor-core matmul, with and without the
    probabilities.  CUDA-event time per block over rotating buffers larger than L2."""
    import torch
    c = synth.CONFIGS["c2"]
    B, H, S, D = c["B"], c["H"], c["S"], c["D"]
    E, T = H * D, B * S
    st = torch.cuda.current_stream().cuda_stream
    sets = 4
    x = torch.randn((sets, T, E), device="cuda")
    wqkv, bqkv = torch.randn((E, 3 * E), device="cuda") * 0.05, torch.randn((3 * E,), device="cuda") * 0.1
    wo, bo = torch.randn((E, E), device="cuda") * 0.05, torch.randn((E,), device="cuda") * 0.1
    qkv = torch.empty((sets, 3, T, E), device="cuda")
    att = torch.empty((sets, T, E), device="cuda")
    y = torch.empty((sets, T, E), device="cuda")
    probs = torch.empty((sets, B, H, S, S), device="cuda")
    plane = T * E * 4

    import ctypes
    pqkv, po = ctypes.c_void_p(), ctypes.c_void_p()
    _capi_check(lib.hipgpt_matmul_tc_prepare(wqkv.data_ptr(), E, 3 * E, ctypes.byref(pqkv), st))
    _capi_check(lib.hipgpt_matmul_tc_prepare(wo.data_ptr(), E, E, ctypes.byref(po), st))

    def block(s, fast, want_probs):
        mm = lib.hipgpt_matmul_tc if fast else lib.hipgpt_matmul
        q = qkv[s].data_ptr()
        if fast == 2:
            rc = lib.hipgpt_matmul_tc_prepared(x[s].data_ptr(), pqkv, bqkv.data_ptr(), q, T, st)
        else:
            rc = mm(x[s].data_ptr(), wqkv.data_ptr(), bqkv.data_ptr(), q, T, E, 3 * E, st)
        rc = rc or lib.hipgpt_mha_forward(q, q + plane, q + 2 * plane, att[s].data_ptr(), probs[s].data_ptr() if want_probs else None, B, S, E, H, 0, st)
        if fast == 2:
            rc = rc or lib.hipgpt_matmul_tc_prepared(att[s].data_ptr(), po, bo.data_ptr(), y[s].data_ptr(), T, st)
        elif fast:
            rc = rc or mm(att[s].data_ptr(), wo.data_ptr(), bo.data_ptr(), y[s].data_ptr(), T, E, E, st)
        else:
            rc = rc or lib.hipgpt_matmul(att[s].data_ptr(), wo.data_ptr(), bo.data_ptr(), att[s].data_ptr(), T, E, E, st)      # in place, like the reference
        if rc:
            _capi_check(rc)
    out = {"config": f"B={B} S={S} E={E} H={H}, non-causal: QKV projection + attention + output projection"}
    for label, fast, want_probs in (("tensor_core_matmul_weights_packed_once_no_probs", 2, False), ("tensor_core_matmul_no_probs", 1, False),
                                    ("tensor_core_matmul_probs_stored", 1, True), ("exact_matmul_probs_stored", 0, True)):
        for _ in range(3):
            for s in range(sets):
                block(s, fast, want_probs)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 10
        e0.record()
        for _ in range(reps):
            for s in range(sets):
                block(s, fast, want_probs)
        e1.record()
        torch.cuda.synchronize()
        out[label] = {"us_per_block": e0.elapsed_time(e1) / reps / sets * 1e3}
    torch.cuda.synchronize()
    lib.hipgpt_matmul_tc_release(pqkv)
    lib.hipgpt_matmul_tc_release(po)
    return out


def _capi_check(rc):
    from hipgpt_b200 import _capi
    _capi.check(rc)


def decode_leg():
    """Greedy KV-cache generation with the default model shape (E=256 L=8 H=8 F=1024 V=5000 S=256,
    random-init weights N(0, 0.02) seed 3, 8 prompts of 16 ids, 128 new tokens): tokens/s of the GPU
    driver, ids checked against the CPU oracle of the same arithmetic, which is timed beside it."""
    from hipgpt_b200.generation import GptDecoder, MODE_PERSISTENT
    from oracle import bindings as ob
    cfg = dict(synth.GPT_DEFAULT)
    B, n_prompt, n_new = 8, 16, 128
    w = synth.gpt_weights(3, **cfg)
    prompts = synth.token_ids(3, (B, n_prompt), cfg["V"])
    dec = GptDecoder(w, **cfg, max_batch=B)
    dec.generate(prompts, n_new)                               # warm-up
    ids, _, ms_prompt, ms_decode = dec.generate(prompts, n_new)
    dec.set_mode(MODE_PERSISTENT)                              # the same steps inside one cooperative launch, for comparison
    dec.generate(prompts, n_new)
    ids_p, _, msp_prompt, msp_decode = dec.generate(prompts, n_new)
    dec.close()
    ob.set_num_threads(os.cpu_count() or 1)
    t0 = time.perf_counter()
    ref_ids, _ = ob.gpt_generate(w, **cfg, prompts=prompts, n_new=n_new, fma=True)
    t_cpu = time.perf_counter() - t0
    return {"metric": "greedy_decode_tokens_per_s", "value": B * n_new / ((ms_prompt + ms_decode) * 1e-3), "unit": "tok/s",
            "steady_state_tokens_per_s": B * (n_new - 1) / (ms_decode * 1e-3), "us_per_step": ms_decode / (n_new - 1) * 1e3,
            "ids_equal_cpu_oracle": bool(np.array_equal(ids, ref_ids)),
            "driver": "one CUDA graph of 52 launches per step",
            "persistent_form": {"value": B * n_new / ((msp_prompt + msp_decode) * 1e-3), "us_per_step": msp_decode / (n_new - 1) * 1e3,
                           "ids_equal_cpu_oracle": bool(np.array_equal(ids_p, ref_ids))},
            "cpu_oracle_tokens_per_s": B * n_new / t_cpu, "cpu_threads": os.cpu_count(),
            "config": {"model": "E=256 L=8 H=8 F=1024 V=5000 S=256, ReLU MLP, fp32", "batch": B, "prompt_len": n_prompt, "new_tokens": n_new,
                       "mode": "causal KV-cache decode (the reference re-runs the padded window per token; not comparable)"}}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cfg = synth.CONFIGS[args.workload]
    tf, info = cpu_leg(cfg, args.causal, seconds=90.0, steps=max(args.steps, 1), warmup=args.warmup)
    line = {"impl": "reference", "metric": "causal_attn_fwd_tflops", "value": tf, "unit": "TFLOP/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": info["ms_per_step"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(args, cfg),
            "timing": {"l2": "host cores: inputs in host memory, no GPU cache involved", "parallelism": "rank 0 only, all host threads"},
            "cpu_baseline": info,
            "e2e": {"value": tf, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    emit(line)


def workload_config(args, cfg):
    """What is computed, in words both arms share (how each arm steps through it is reported beside it, not here)."""
    kind = "causal" if args.causal else "full"
    return {"workload": f"{args.workload}: {kind} MHA forward B={cfg['B']} H={cfg['H']} S={cfg['S']} head_dim={cfg['D']} {args.dtype}",
            "B": cfg["B"], "H": cfg["H"], "S": cfg["S"], "head_dim": cfg["D"], "causal": int(args.causal),
            "probs_stored": int(args.probs)}


def scaling_c5_leg(world, rank, lib):
    """BASELINE.json's scaling configuration (B=64 H=16 S=2048 head_dim=64, causal, fp32 and bf16 storage) with its
    batches split over the ranks by the library's own driver (hipgpt_mha_forward_sharded): compute only, with the
    NCCL all-gather of the outputs chunk by chunk behind the arithmetic, and with the library's own transports into the
    peers' mapped buffers (a small copy kernel's stores; one copy-engine copy per peer and chunk).  Device time per call from CUDA events,
    max over ranks; L2 is flushed between calls (at 8 ranks a rank's bf16 inputs are smaller than L2)."""
    import torch
    import torch.distributed as dist
    from hipgpt_b200 import sharding
    c = synth.CONFIGS["c5"]
    B, H, S, D = c["B"], c["H"], c["S"], c["D"]
    E = H * D
    if B % world:
        return {"skipped": f"{B} batches do not split over {world} ranks"}
    Bl = B // world

    def chunks_for(esz):
        # a chunk should carry at least ~16 MB of output: below that the per-chunk launches and collectives cost
        # more than their overlap saves
        want = max(1, min(16, int(Bl * S * E * esz) // (16 << 20)))
        return next(ch for ch in range(want, 0, -1) if Bl % ch == 0)
    sh = sharding.ShardedAttention()
    stream = torch.cuda.current_stream()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    out = {"config": f"c5: causal MHA forward B={B} H={H} S={S} head_dim={D}, batches split over {world} rank(s)",
           "flops_per_call": flops_of(B, H, S, D, True), "nccl_version": int(lib.hipgpt_shard_nccl_version()),
           "reps": 5}
    for name, dtype in (("f32", torch.float32), ("bf16", torch.bfloat16)):
        g = torch.Generator(device="cuda")
        g.manual_seed(4 + rank)
        loc = torch.randn((3, Bl * S, E), device="cuda", generator=g, dtype=torch.float32).to(dtype)
        # the output lives in the buffer that every rank maps from every other (needed by the peer-store transport)
        full = sh.output_tensor(B * S, E, dtype) if world > 1 else torch.empty((B * S, E), device="cuda", dtype=dtype)
        chunks = chunks_for(full.element_size())

        def call(ch, gather):
            sh.forward(loc[0], loc[1], loc[2], full, B, S, E, H, causal=True, chunks=ch, gather=gather)

        def timed(ch, gather, reps=5):
            for _ in range(2):
                call(ch, gather)
            total = 0.0
            for _ in range(reps):
                flush.fill_(1)
                torch.cuda.synchronize()
                if world > 1:
                    dist.barrier()
                    torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                call(ch, gather)
                e1.record(stream)
                torch.cuda.synchronize()
                ms = e0.elapsed_time(e1)
                if world > 1:
                    tt = torch.tensor([ms], device="cuda")
                    dist.all_reduce(tt, op=dist.ReduceOp.MAX)
                    ms = float(tt.item())
                total += ms
            return total / reps
        res = {}
        few = next(ch for ch in range(min(4, Bl), 0, -1) if Bl % ch == 0)       # the copy-engine transport hides behind fewer, larger chunks
        for label, ch, gather in (("compute_only", 1, 0), ("compute_chunked", chunks, 0), ("with_gather", chunks, sharding.GATHER_NCCL),
                                  ("with_gather_peer_stores", chunks, sharding.GATHER_PEER_STORES),
                                  ("with_gather_peer_copies", few, sharding.GATHER_PEER_COPIES),
                                  ("with_gather_peer_both", chunks, sharding.GATHER_PEER_BOTH)):
            if gather and world == 1:
                continue
            if gather:
                full.zero_()
                torch.cuda.synchronize()
                dist.barrier()
            ms = timed(ch, gather)
            res[label] = {"ms": ms, "tflops": flops_of(B, H, S, D, True) / (ms * 1e-3) / 1e12, "chunks": ch}
            if gather:
                # a size-independent property of the gathered output: every rank holds the same bytes, and their checksum is
                # the sum of the checksums of the parts the ranks computed
                view = full.view(torch.int16 if full.element_size() == 2 else torch.int32).view(ch, world, -1)
                mine = view[:, rank].to(torch.int64).sum()
                whole = view.to(torch.int64).sum()
                parts = mine.clone()
                dist.all_reduce(parts)
                lo, hi = whole.clone(), whole.clone()
                dist.all_reduce(lo, op=dist.ReduceOp.MIN)
                dist.all_reduce(hi, op=dist.ReduceOp.MAX)
                res[label]["gathered_checksums_agree"] = bool(int(lo) == int(hi) == int(parts))
        res["gather_chunks"] = chunks
        res["gathered_bytes_per_rank"] = int((B - Bl) * S * E * full.element_size()) if world > 1 else 0
        out[name] = res
        del loc, full
    sh.close()
    return out


# ----------------------------------------------------------------------------- GPU arm ----
def run_ours(args):
    import torch
    import torch.distributed as dist
    from hipgpt_b200 import _capi

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the product path")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    lib = _capi.lib()
    cfg = dict(synth.CONFIGS[args.workload])
    B_total = cfg["B"]
    if args.strong and world > 1:
        from hipgpt_b200 import sharding
        b0, b1 = sharding.shard_range(B_total, world, rank)      # this rank's slab of the workload's batches
        cfg["B"] = b1 - b0
        if cfg["B"] == 0:
            raise SystemExit("more ranks than batches")
    B, H, S, D = cfg["B"], cfg["H"], cfg["S"], cfg["D"]
    E = H * D
    bf16 = args.dtype == "bf16"
    if bf16 and (args.probs or D != 64):
        raise SystemExit("--dtype bf16: head_dim 64, no stored probabilities")
    esz = 2 if bf16 else 4                                   # bytes per stored element
    tdtype = torch.bfloat16 if bf16 else torch.float32
    per_batch_bytes = bytes_of(B, H, S, D, args.probs) * esz // 4
    sets = args.sets or max(1, int(np.ceil(1.5 * L2_BYTES / per_batch_bytes)))
    plane = B * S * E

    # inputs: `sets` different batches per rank, resident in HBM before the timed region
    h_in = torch.empty((sets, 3, B * S, E), dtype=torch.float32).pin_memory()
    gen = min(sets, 2)                                    # two seeded batches, the rest are rolls of them
    for s in range(gen):
        if 3 * B * S * E <= 64_000_000:
            h_in[s] = torch.from_numpy(synth.qkv_planes(cfg["seed"] + 100 * rank + s, B, S, E, cfg["scale"]))
        else:
            # large workloads: a few seeded batch items, the others are rolls of them along the head dimension
            view = h_in[s].view(3, B, S, E)
            nb = min(B, 4)
            for bi in range(nb):
                view[:, bi] = torch.from_numpy(synth.qkv_planes(cfg["seed"] + 100 * rank + 10 * s + bi, 1, S, E, cfg["scale"])).view(3, S, E)
            for bi in range(nb, B):
                view[:, bi] = torch.roll(view[:, bi % nb], shifts=bi, dims=2)
    for s in range(gen, sets):
        h_in[s] = torch.roll(h_in[s % gen], shifts=s, dims=1)   # other token order: other data, same distribution
    d_in = h_in.cuda(non_blocking=True).to(tdtype)
    d_out = torch.empty((sets, B * S, E), dtype=tdtype, device="cuda")
    d_probs = torch.empty((B, H, S, S), dtype=torch.float32, device="cuda") if args.probs else None
    # --gather: the outputs of all ranks are all-gathered, in chunks of batches, each chunk as soon as
    # its kernel has been enqueued, so that NVLink traffic overlaps the remaining compute
    nchunks = 1
    if args.gather and world > 1:
        if args.strong and B_total % world:
            raise SystemExit("--gather with --strong needs the batch count to divide by the ranks")
        nchunks = 4 if (B % 4 == 0 and B * S * E * esz >= (32 << 20)) else 1
    bc = B // nchunks                                         # batches per chunk
    gathered = (torch.empty((sets, nchunks, world, bc * S, E), dtype=tdtype, device="cuda")
                if (args.gather and world > 1) else None)
    stream = torch.cuda.current_stream()
    st = stream.cuda_stream

    in_ptrs = [d_in[s].data_ptr() for s in range(sets)]
    out_ptrs = [d_out[s].data_ptr() for s in range(sets)]
    probs_ptr = d_probs.data_ptr() if args.probs else None
    if bf16:
        def fwd(q, k, v, out, probs, B_, S_, E_, H_, causal, st_):
            return lib.hipgpt_mha_forward_bf16_ex(q, k, v, out, B_, S_, E_, H_, causal, args.bf16_variant, st_)
    elif KERNELS[args.kernel] is None:
        fwd = lib.hipgpt_mha_forward
    else:
        algo, which = KERNELS[args.kernel][:2]

        def fwd(q, k, v, out, probs, B_, S_, E_, H_, causal, st_):
            return lib.hipgpt_mha_forward_ex(q, k, v, out, probs, B_, S_, E_, H_, causal, algo, which, st_)

    def step():
        handles = []
        for s in range(sets):
            base = in_ptrs[s]
            if gathered is None:
                rc = fwd(base, base + esz * plane, base + 2 * esz * plane, out_ptrs[s], probs_ptr, B, S, E, H, args.causal, st)
                if rc:
                    _capi.check(rc)
                continue
            for c in range(nchunks):
                off = c * bc * S * E * esz                   # byte offset of the chunk inside a plane / the output
                rc = fwd(base + off, base + esz * plane + off, base + 2 * esz * plane + off, out_ptrs[s] + off, None,
                         bc, S, E, H, args.causal, st)
                if rc:
                    _capi.check(rc)
                handles.append(dist.all_gather_into_tensor(gathered[s, c].view(-1), d_out[s].view(nchunks, -1)[c],
                                                           async_op=True))
        for h in handles:
            h.wait()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def timed(fn, n):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record(stream)
        for _ in range(n):
            fn()
        e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    for _ in range(max(args.warmup, 3)):
        step()
    with ClockSampler(local) as clocks:
        ms = timed(step, args.steps)
    ms_per_step = ms / args.steps
    flops_step = flops_of(B, H, S, D, args.causal) * sets
    if args.strong and world > 1:
        value = flops_of(B_total, H, S, D, args.causal) * sets / (ms_per_step * 1e-3) / 1e12
    else:
        value = world * flops_step / (ms_per_step * 1e-3) / 1e12

    # roofline of the attention kernel: FMA-pipe ceiling measured now, on this GPU, at these clocks
    sink = torch.zeros(1, device="cuda")
    import ctypes as C
    fl = C.c_double()
    blocks, iters = 148 * 8, 4096
    for _ in range(3):
        _capi.check(lib.hipgpt_probe_fma(sink.data_ptr(), blocks, iters, C.byref(fl), st))
    probe_ms = timed(lambda: _capi.check(lib.hipgpt_probe_fma(sink.data_ptr(), blocks, iters, C.byref(fl), st)), 20) / 20
    fma_peak = fl.value / (probe_ms * 1e-3) / 1e12
    launch_ms = ms_per_step / sets                        # one launch per batch, back to back
    achieved = flops_of(B, H, S, D, args.causal) / (launch_ms * 1e-3) / 1e12
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    hbm_peak = float(peaks.get("hbm_gbs", FALLBACK_HBM_GBS))
    hbm_achieved = per_batch_bytes / (launch_ms * 1e-3) / 1e9
    # Which roofline binds the kernel that ran: the time HBM needs for the algorithmic bytes against
    # the time the pipe needs for the algorithmic FLOPs.  The tensor-core kernel computes in
    # split-TF32 (three TF32 products per fp32 product); TF32 runs at half the measured dense bf16
    # rate.  With the probabilities stored the kernel forms Q K^T twice (1.5 times the tensor work)
    # and writes B H S S floats more.  Other head dims run the FFMA kernel, measured against the FFMA ceiling.
    tensor_kernel = D in (32, 64) and (KERNELS[args.kernel] is None or KERNELS[args.kernel][0] == 3)
    flops_launch = flops_of(B, H, S, D, args.causal)
    # a kernel timed back to back for seconds is compared with the sustained figure
    bf16_peak = float(peaks.get("bf16_tflops_sustained" if bf16 else "bf16_tflops", 1400.0 if bf16 else 1590.0))
    tf32_peak = bf16_peak / 2.0
    t_hbm = per_batch_bytes / (hbm_peak * 1e9)
    # tensor work per fp32 product, in TF32 products: the default kernel runs one TF32 product and two FP16
    # products (twice the TF32 rate); 3 would be the figure of the split-TF32 variant
    tc16 = tensor_kernel and not bf16
    # tensor work per fp32 product in TF32-rate products: whole-head kernel one TF32 + two FP16 products for Q K^T
    # (2) and three FP16 products for P V (1.5); tiled kernel three FP16 products for both (1.5); split-TF32 three
    whole_head = (KERNELS[args.kernel][2] == "mha_head_kernel") if KERNELS[args.kernel] else (D == 32 and S <= 256)
    tiled = tc16 and not whole_head and args.kernel in ("auto", "tiled")
    tf32_products = (1.5 if tiled else 1.75 if (tc16 and whole_head) else 3.0) * (1.5 if (args.probs and tiled) else 1.0)
    t_pipe = (flops_launch / (bf16_peak * 1e12)) if bf16 else (tf32_products * flops_launch / (tf32_peak * 1e12)) if tensor_kernel else flops_launch / (fma_peak * 1e12)
    src = "measured" if peaks else "fallback"
    if bf16 and t_hbm < t_pipe:
        roofline = {"bound": "tensor", "achieved": achieved, "peak": bf16_peak, "unit": "TFLOP/s", "frac": achieved / bf16_peak,
                    "peak_source": f"MEASURED_PEAKS.json bf16_tflops_sustained ({src}): dense bf16 GEMM rate"}
    elif t_hbm >= t_pipe:
        roofline = {"bound": "hbm", "achieved": hbm_achieved, "peak": hbm_peak, "unit": "GB/s",
                    "frac": hbm_achieved / hbm_peak, "peak_source": f"MEASURED_PEAKS.json hbm_gbs ({src})"}
    elif tensor_kernel:
        roofline = {"bound": "tensor", "achieved": tf32_products * achieved, "peak": tf32_peak, "unit": "TFLOP/s",
                    "frac": tf32_products * achieved / tf32_peak,
                    "peak_source": f"half of MEASURED_PEAKS.json bf16_tflops ({src}): TF32 rate; achieved counts the {tf32_products:g} TF32-equivalent products per fp32 product"}
    else:
        roofline = {"bound": "fma", "achieved": achieved, "peak": fma_peak, "unit": "TFLOP/s", "frac": achieved / fma_peak,
                    "peak_source": "fp32 FFMA loop timed in this run"}
    kernel = ("mha_bf16_kernel" if bf16 else
              KERNELS[args.kernel][2] if KERNELS[args.kernel] else
              "mha_head_kernel" if (D == 32 and S <= 256) else
              "mha_tc16_kernel" if tensor_kernel else "mha_rows_kernel" if D == 128 else "mha_generic_kernel")
    traffic = TRAFFIC.get((args.workload, kernel)) if (args.causal and not args.probs and not bf16) else None
    roofline.update({"kernel": kernel, "traffic": traffic[0] if traffic else None, "traffic_source": traffic[1] if traffic else None,
                     "us_per_launch": launch_ms * 1e3, "kernels_per_launch": tiled_launches(B, H, S, D, bool(args.causal)) if tiled else 1,
                     "algorithmic_bytes_per_launch": per_batch_bytes,
                     "algorithmic_flops_per_launch": flops_launch,
                     "vs_fp32_fma_ceiling": {"achieved_tflops": achieved, "ffma_peak_tflops": fma_peak, "ratio": achieved / fma_peak,
                                             "note": "fp32-grade result rate against the FFMA pipe ceiling measured in this run"},
                     "hbm_time_us": t_hbm * 1e6, "pipe_time_us": t_pipe * 1e6})
    line = {"metric": "causal_attn_fwd_tflops" if args.causal else "attn_fwd_tflops", "value": value, "unit": "TFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "strong" if (args.strong and world > 1) else "weak", "vs_baseline": None,
            "dtype": "bf16 storage, fp32 accumulate" if bf16 else "f32", "data": "synthetic",
            "config": workload_config(args, dict(cfg, B=B_total)),
            "timing": {"batches_per_step": sets,
                       "l2": f"{sets} distinct input batches per step, {sets * per_batch_bytes / 1e6:.0f} MB > 126 MB L2",
                       "parallelism": f"batch-major shards x{world}" + (", NCCL all-gather of outputs in chunks, overlapped" if args.gather else ", no collective")},
            "clocks": clocks.summary(), "roofline": roofline,
            "gpu_launches": args.steps * sets * (tiled_launches(B, H, S, D, bool(args.causal)) if tiled else 1)}

    # the scaling configuration through the library's sharded driver (every N, the default workload only)
    if args.workload == "c2" and not args.no_scaling and not bf16:
        del d_in, d_out
        torch.cuda.empty_cache()
        line["scaling_c5"] = scaling_c5_leg(world, rank, lib)

    # end to end through the host-buffer entry point: pinned host memory in, host memory out
    if not args.no_e2e:
        h_e2e = h_in.to(tdtype).pin_memory() if bf16 else h_in      # bf16: the planes as the caller would hold them
        h_out = torch.empty((B * S, E), dtype=tdtype).pin_memory()
        h_probs = torch.empty((B, H, S, S), dtype=torch.float32).pin_memory() if args.probs else None
        e2e_steps = max(1, min(args.steps, 20))

        def e2e_step():
            for s in range(sets):
                if bf16:
                    rc = lib.hipgpt_mha_forward_bf16_host(h_e2e[s].data_ptr(), h_out.data_ptr(), B, S, E, H, args.causal)
                else:
                    rc = lib.hipgpt_mha_forward_host(h_e2e[s].data_ptr(), h_out.data_ptr(),
                                                     h_probs.data_ptr() if args.probs else None, B, S, E, H, args.causal)
                if rc:
                    _capi.check(rc)
        for _ in range(3):
            e2e_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_step()
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        if world > 1:
            t = torch.tensor([dt], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dt = float(t.item())
        line["e2e"] = {"value": (flops_of(B_total, H, S, D, args.causal) * sets if (args.strong and world > 1) else world * flops_step) * e2e_steps / dt / 1e12,
                       "unit": "TFLOP/s",
                       "h2d_bytes_per_step": int(sets * 3 * plane * esz),
                       "d2h_bytes_per_step": int(sets * (plane * esz + (B * H * S * S * 4 if args.probs else 0))),
                       "ms_per_step": dt / e2e_steps * 1e3, "steps": e2e_steps,
                       "api": ("hipgpt_mha_forward_bf16_host" if bf16 else "hipgpt_mha_forward_host") + " (C ABI, host pointers)"}
        lib.hipgpt_release_workspace()

    if rank == 0 and world == 1 and not args.no_cpu:
        _, info = cpu_leg(cfg, args.causal, seconds=args.cpu_seconds)
        line["cpu_baseline"] = info
        line["decode"] = decode_leg()
        line["projections"] = projections_leg(lib, fma_peak)
        line["attention_block"] = attention_block_leg(lib)
    if rank == 0:
        emit(line)
    if world > 1:
        dist.destroy_process_group()


_REAL_STDOUT = None


def emit(line: dict) -> None:
    """The one JSON line, on the process's real stdout."""
    data = (json.dumps(line) + "\n").encode()
    if _REAL_STDOUT is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_REAL_STDOUT, data)


def main():
    # stdout carries the JSON line only: whatever libraries print there (NCCL's version banner, for
    # one) is sent to stderr by pointing file descriptor 1 at stderr for the duration of the run
    global _REAL_STDOUT
    sys.stdout.flush()
    _REAL_STDOUT = os.dup(1)
    os.dup2(2, 1)
    args = parse()
    if args.decode_only:
        emit(decode_leg())
    elif args.projections_only:
        import torch
        from hipgpt_b200 import _capi
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the product path")
        torch.cuda.set_device(0)
        emit({"projections": projections_leg(_capi.lib()), "attention_block": attention_block_leg(_capi.lib())})
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
