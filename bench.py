#!/usr/bin/env python
"""Benchmark of the FP4 linear path: the four FP4 projections of one GLM-ASR decoder layer at
prefill (M = 10000 tokens, hidden 2048, q/k/v 2048/512/512, ffn 6144) -- benchmark configuration 1.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--mode w4a4|w4a16]

One step = q|k|v GEMM, o GEMM + residual, gate|up GEMM + SiLU-gate, down GEMM + residual
(964.7 GFLOP) on synthetic seeded weights and activations.  Prints ONE JSON line (rank 0).
Under torchrun every rank runs the same workload on its own GPU (data-parallel replicas, no
data-path collective); the value is the whole-job aggregate, time = max over ranks.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from glm_asr_stack_b200 import replicas  # noqa: E402  (host-side rank logic; loads the C-ABI library, no GPU needed)

HIDDEN, FFN, KV, M_TOKENS = 2048, 6144, 512, 10000
METRIC, UNIT = "fp4_linear_tflops", "TFLOP/s"
WORKLOAD = "config1: one decoder layer of FP4 projections at prefill, M=10000, hidden 2048, qkv N=3072, o N=2048, gate-up N=12288 (+SiLU), down K=6144 (+residual)"
NOMINAL_FP4_TFLOPS = 9000.0     # dense FP4, public spec-sheet figure; no measured FP4 peak is available
NOMINAL_BF16_TFLOPS = 2250.0


def layer_flops(M):
    return 2.0 * M * (HIDDEN * (HIDDEN + 2 * KV) + HIDDEN * HIDDEN + 2 * FFN * HIDDEN + HIDDEN * FFN)


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return json.load(f)
    except Exception:
        return None


class ClockSampler:
    """SM clock / throttle-reason samples DURING the timed region (read-only NVML queries; nvidia-smi at 100 ms is
    the fallback).  The layer workload's region lasts a few milliseconds, so besides a background thread that
    polls every 20 ms (frequent NVML queries were measured to cost 2-3 % of the step rate) the main thread takes
    one sample itself between enqueueing the last timed step and the closing barrier, i.e. while the GPU is
    still executing the timed steps."""

    REASONS = ((0x8, "hw_slowdown"), (0x40, "hw_thermal_slowdown"), (0x20, "sw_thermal_slowdown"), (0x4, "sw_power_cap"))

    def __init__(self, index):
        self.index = index
        self.samples = []          # (sm_mhz, reason_bits)
        self.max_mhz = None
        self.proc = None
        self.thread = None
        self.running = False
        self.handle = None
        self.nvml = None

    def _nvml_handle(self):
        import pynvml
        pynvml.nvmlInit()
        self.nvml = pynvml
        try:
            import torch
            uuid = str(torch.cuda.get_device_properties(self.index).uuid)
            return pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid).encode())
        except Exception:
            return pynvml.nvmlDeviceGetHandleByIndex(self.index)

    def _poll(self):
        nv, h = self.nvml, self.handle
        while self.running:
            try:
                mhz = nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)
                try:
                    bits = nv.nvmlDeviceGetCurrentClocksEventReasons(h)
                except Exception:
                    bits = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                self.samples.append((float(mhz), int(bits)))
            except Exception:
                pass
            time.sleep(0.02)

    def sample_now(self):
        """One sample from the calling thread (NVML path only)."""
        if self.handle is None:
            return
        nv, h = self.nvml, self.handle
        try:
            mhz = nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)
            try:
                bits = nv.nvmlDeviceGetCurrentClocksEventReasons(h)
            except Exception:
                bits = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
            self.samples.append((float(mhz), int(bits)))
        except Exception:
            pass

    def start(self):
        try:
            self.handle = self._nvml_handle()
            self.max_mhz = float(self.nvml.nvmlDeviceGetMaxClockInfo(self.handle, self.nvml.NVML_CLOCK_SM))
            self.running = True
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.handle = None
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            f = [x.strip() for x in line.strip().split(",")]
            if len(f) < 6:
                continue
            try:
                bits = 0
                for (bit, _), v in zip(self.REASONS, f[2:6]):
                    if v.lower().startswith("active"):
                        bits |= bit
                self.samples.append((float(f[0]), bits))
                self.max_mhz = float(f[1])
            except ValueError:
                continue

    def stop(self):
        if self.handle is not None:
            self.running = False
            self.thread.join(timeout=1.0)
        elif self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
        else:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["clock query unavailable"], "samples": 0}
        sm = [m for m, _ in self.samples]
        reasons = sorted({name for _, bits in self.samples for bit, name in self.REASONS if bits & bit})
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": self.max_mhz, "reasons": reasons,
                "samples": len(sm), "how": "NVML: one query while the timed steps execute + a 20 ms poll" if self.handle is not None else "nvidia-smi -lms 100"}


def cpu_reference_leg(steps, warmup, sample_rows):
    """The reference's W4A16 fallback arithmetic restated on the host cores (oracle port)."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import cpu_baseline
    sec, threads = cpu_baseline.time_layer(sample_rows, HIDDEN, FFN, KV, steps=steps, warmup=warmup)
    tflops = cpu_baseline.layer_flops(sample_rows, HIDDEN, FFN, KV) / sec / 1e12
    return tflops, sec, threads


def run_reference(args, rank):
    if rank != 0:
        return
    sample = 512
    tflops, sec, threads = cpu_reference_leg(args.steps, max(args.warmup, 1), sample)
    line = {
        "impl": "reference", "metric": METRIC, "value": tflops, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": max(args.warmup, 1), "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16 x fp32-accumulate (weights dequantised from e2m1 every call)",
        "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": f"first {sample} of {M_TOKENS} rows per step"},
        "cpu_baseline": {"value": tflops, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": f"{sample} of {M_TOKENS} rows, all four projections, full weights, torch CPU"},
        "e2e": {"value": tflops, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference has no CPU implementation of this path; this is its fallback arithmetic "
                "(dequantise whole weight each call + fp32-accumulate GEMM) restated with torch on the host cores",
    }
    print(json.dumps(line), flush=True)


def run_decode(args, rank, local_rank, world):
    """Benchmark configuration 2: one batched decode step of the 28-layer decoder + FP4 lm_head + arg-max for
    256 sequences with paged bf16 KV (16-token pages, context 200-450).  tok/s = sequences / step time."""
    os.environ["GLMASR_USE_CUTLASS_NVFP4"] = "1" if args.mode == "w4a4" else "0"
    import torch

    from glm_asr_stack_b200 import engine, ops, workloads

    torch.cuda.set_device(local_rank)
    dist = replicas.init_group("nccl", world, torch.device("cuda", local_rank))
    model = workloads.build_decoder(layers=args.layers)
    state = workloads.build_decode_state(model.cfg, num_seqs=args.seqs)
    cfg, lm, n, vocab = model.cfg, model.lm_head, args.seqs, model.cfg.vocab_size
    gen = torch.Generator(device="cpu").manual_seed(3)
    ids_host = torch.randint(0, vocab, (n,), generator=gen, dtype=torch.int32).pin_memory()
    ids = ids_host.cuda()
    logits = torch.empty((n, vocab), dtype=torch.bfloat16, device="cuda")
    tok_host = torch.empty(n, dtype=torch.int32).pin_memory()

    def step(ids_dev):
        state.reset_lengths()                      # same context every step: the step rewrites the same KV slot
        hidden = ops.embedding_lookup(model.embed, ids_dev)
        engine.decode_step(model.ws, cfg, state.pool, state.bts, hidden, state.d_seq_lens, state.h_seq_lens)
        if args.mode == "w4a4":
            assert ops.nvfp4_linear(logits, hidden, lm.w_packed, lm.w_scales, model.lm_head_input_scale,
                                    lm.w_global_scale) == 0
        else:
            ops.fp4_linear(hidden, lm.w_packed, lm.w_scales, lm.w_global_scale, out=logits)
        return ops.argmax_rows(logits)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step(ids)
    torch.cuda.synchronize()
    _st = ops.status()
    assert _st == 0, f"device status word = {_st} (bounded wait expired or CUDA error)"
    sampler = ClockSampler(local_rank)
    barrier()
    sampler.start()
    l0 = ops.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step(ids)
    e1.record()
    sampler.sample_now()          # the GPU is still working through the timed steps queued above
    barrier()
    ms = e0.elapsed_time(e1) / args.steps
    launches = ops.launch_count() - l0
    clocks = sampler.stop()
    # end to end: token ids from pinned host memory in, next-token ids back to the host
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        tok_host.copy_(step(ids_host.cuda(non_blocking=True)), non_blocking=True)
        torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) / args.steps * 1e3
    ms = replicas.max_over_ranks(ms, dist, "cuda")
    e2e_ms = replicas.max_over_ranks(e2e_ms, dist, "cuda")
    H, KV = cfg.dec_hidden, cfg.dec_kv_heads * cfg.dec_head_dim
    # algorithmic bytes per step: FP4 weights once, K and V of every cached token once, the new token's K/V,
    # embedding rows, logits written then read by the arg-max
    bytes_step = model.weight_bytes + state.kv_read_bytes + n * KV * 2 * 2 * cfg.dec_layers + n * H * 2 + 2 * n * vocab * 2
    peaks = measured_peaks()
    peak = peaks["hbm_gbs"] if peaks else 6650.0
    if rank == 0:
        gbs = bytes_step / (ms * 1e-3) / 1e9
        print(json.dumps({
            "metric": "decode_tok_per_s", "value": replicas.whole_job_rate(n, world, ms * 1e-3), "unit": "tok/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": args.mode, "data": "synthetic",
            "config": {"workload": f"config2: batched decode step, {cfg.dec_layers} layers, {n} sequences, paged bf16 KV "
                                   "(16-token pages, context 200-450), FP4 lm_head over 59264 + arg-max",
                       "l2": f"{bytes_step / 1e9:.2f} GB touched per step > 126 MB L2"},
            "e2e": {"value": replicas.whole_job_rate(n, world, e2e_ms * 1e-3), "unit": "tok/s", "h2d_bytes_per_step": n * 4,
                    "d2h_bytes_per_step": n * 4, "ms_per_step": e2e_ms},
            "gpu_launches": int(launches), "clocks": clocks,
            "roofline": {"bound": "hbm", "kernel": "whole decode step (weights + KV stream)", "achieved": gbs, "peak": peak,
                         "unit": "GB/s", "frac": gbs / peak, "traffic": None, "bytes_per_step": bytes_step,
                         "weight_bytes": model.weight_bytes, "kv_read_bytes": state.kv_read_bytes,
                         "peak_source": "measured HBM copy bandwidth (MEASURED_PEAKS.json)" if peaks else "fallback"},
        }), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def run_prefill(args, rank, local_rank, world):
    """The whole batched prefill the config-1 projections belong to: 28 layers over 25 windows x 400 tokens
    (10000 tokens) through decoder_prefill_paged_batched -- projections, RoPE + paged-cache write, causal
    attention.  tok/s = prefilled tokens / step time; TFLOP/s counts the projections and the attention."""
    os.environ["GLMASR_USE_CUTLASS_NVFP4"] = "1" if args.mode == "w4a4" else "0"
    import torch

    from glm_asr_stack_b200 import engine, ops, synth, workloads

    torch.cuda.set_device(local_rank)
    dist = replicas.init_group("nccl", world, torch.device("cuda", local_rank))
    model = workloads.build_decoder(layers=args.layers)
    cfg = model.cfg
    nseq = max(1, args.rows // 400)
    st = workloads.build_prefill_state(cfg, num_seqs=nseq, seq_len=400)
    T, H = st.total_tokens, cfg.dec_hidden
    xs = [synth.seeded_activation(T, H, 31 + i) for i in range(2)]
    hid = torch.empty_like(xs[0])
    hin = xs[0].cpu().pin_memory()
    hout = torch.empty_like(hin).pin_memory()

    def step(i):
        hid.copy_(xs[i % 2])
        engine.prefill_paged_batched(model.ws, cfg, st.pool, st.bts, hid, st.seq_lens, st.seq_offsets)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        step(i)
    torch.cuda.synchronize()
    _st = ops.status()
    assert _st == 0, f"device status word = {_st} (bounded wait expired or CUDA error)"
    sampler = ClockSampler(local_rank)
    barrier()
    sampler.start()
    l0 = ops.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        step(i)
    e1.record()
    sampler.sample_now()          # the GPU is still working through the timed steps queued above
    barrier()
    ms = e0.elapsed_time(e1) / args.steps
    launches = ops.launch_count() - l0
    clocks = sampler.stop()
    barrier()
    t0 = time.perf_counter()
    for i in range(args.steps):
        hid.copy_(hin, non_blocking=True)
        engine.prefill_paged_batched(model.ws, cfg, st.pool, st.bts, hid, st.seq_lens, st.seq_offsets)
        hout.copy_(hid, non_blocking=True)
        torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) / args.steps * 1e3
    ms = replicas.max_over_ranks(ms, dist, "cuda")
    e2e_ms = replicas.max_over_ranks(e2e_ms, dist, "cuda")
    QH, HD = cfg.dec_heads, cfg.dec_head_dim
    attn_flops = sum(2 * 2 * QH * HD * (ln * (ln + 1) // 2) for ln in st.seq_lens)          # QK^T and PV, causal half
    flops = cfg.dec_layers * (layer_flops(T) + attn_flops)
    if rank == 0:
        print(json.dumps({
            "metric": "prefill_tok_per_s", "value": replicas.whole_job_rate(T, world, ms * 1e-3), "unit": "tok/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": args.mode, "data": "synthetic",
            "config": {"workload": f"batched prefill, {cfg.dec_layers} layers, {nseq} sequences x 400 tokens = {T} tokens, "
                                   "paged bf16 KV (16-token pages)",
                       "l2": "weights of 28 layers (0.76 GB) and 41 MB of activations per layer > 126 MB L2"},
            "tflops": replicas.whole_job_rate(flops, world, ms * 1e-3) / 1e12,
            "e2e": {"value": replicas.whole_job_rate(T, world, e2e_ms * 1e-3), "unit": "tok/s", "h2d_bytes_per_step": T * H * 2,
                    "d2h_bytes_per_step": T * H * 2, "ms_per_step": e2e_ms},
            "gpu_launches": int(launches), "clocks": clocks,
        }), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--mode", default="w4a4", choices=["w4a4", "w4a16"])
    ap.add_argument("--rows", type=int, default=M_TOKENS)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--workload", default="layer", choices=["layer", "decode", "prefill"],
                    help="layer = benchmark configuration 1 (default, the headline); decode = configuration 2; "
                         "prefill = the whole 28-layer batched prefill the config-1 projections belong to")
    ap.add_argument("--seqs", type=int, default=256)
    ap.add_argument("--layers", type=int, default=28)
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank, local_rank, world = replicas.rank_info()

    if args.impl == "reference":
        run_reference(args, rank)
        return

    if args.workload == "decode":
        run_decode(args, rank, local_rank, world)
        return
    if args.workload == "prefill":
        run_prefill(args, rank, local_rank, world)
        return

    import torch

    from glm_asr_stack_b200 import ops, synth

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for this path")
    torch.cuda.set_device(local_rank)
    dist = replicas.init_group("nccl", world, torch.device("cuda", local_rank))

    mode = ops.MODE_W4A4 if args.mode == "w4a4" else ops.MODE_W4A16
    M = args.rows
    # four different layers' weights, used round-robin, so no step finds its weights in L2
    n_sets = 4
    layers = []
    keep = []
    for layer in range(n_sets):
        w = {}
        for i, (n, N, K) in enumerate([("q", HIDDEN, HIDDEN), ("k", KV, HIDDEN), ("v", KV, HIDDEN),
                                       ("o", HIDDEN, HIDDEN), ("gate", FFN, HIDDEN), ("up", FFN, HIDDEN),
                                       ("down", HIDDEN, FFN)]):
            w[n] = synth.seeded_weight(N, K, 1000 * layer + i)
        keep.append(w)
    xs = [synth.seeded_activation(M, HIDDEN, 1 + i) for i in range(2)]
    # per-projection activation scales (static in a real checkpoint): take them from one dry run's inputs
    isc_h = synth.default_input_scale(xs[0])
    for w in keep:
        for n in ("q", "k", "v", "gate", "up"):
            w[n].input_scale = isc_h
        w["o"].input_scale = isc_h * 4.0
        w["down"].input_scale = isc_h * 0.5
        layers.append(ops.make_layer_weights(w["q"], w["k"], w["v"], w["o"], w["gate"], w["up"], w["down"],
                                             HIDDEN, FFN))
    out = torch.empty_like(xs[0])
    hin = [x.cpu().pin_memory() for x in xs]
    hout = torch.empty_like(hin[0]).pin_memory()

    def step(i):
        ops.layer_proj(mode, xs[i % 2], layers[i % n_sets], out)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        step(i)
    torch.cuda.synchronize()
    _st = ops.status()
    assert _st == 0, f"device status word = {_st} (bounded wait expired or CUDA error)"

    # ---- device-resident timing -----------------------------------------------------------
    sampler = ClockSampler(local_rank)
    barrier()
    sampler.start()
    launches0 = ops.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        step(i)
    e1.record()
    sampler.sample_now()          # the GPU is still working through the timed steps queued above
    barrier()
    ms_total = e0.elapsed_time(e1)
    launches = ops.launch_count() - launches0
    clocks = sampler.stop()
    ms_total = replicas.max_over_ranks(ms_total, dist, "cuda")
    ms_step = ms_total / args.steps
    value = replicas.whole_job_rate(layer_flops(M), world, ms_step * 1e-3) / 1e12

    # ---- per-launch kernel timing for the roofline (separate pass, events around each GEMM) ----
    ops.profile_enable(True)
    for i in range(min(args.steps, 8)):
        step(i)
    prof = ops.profile_read()
    ops.profile_enable(False)
    # dominant kernel: the gate|up GEMM (largest flops per launch)
    top_flops = max(f for _, f, _ in prof)
    top = [(ms, f, b) for ms, f, b in prof if f == top_flops]
    top_ms = statistics.mean(ms for ms, _, _ in top)
    achieved = top_flops / (top_ms * 1e-3) / 1e12
    all_ms = sum(ms for ms, _, _ in prof) / max(1, min(args.steps, 8))
    peaks = measured_peaks()
    if args.mode == "w4a4":
        peak, peak_src = NOMINAL_FP4_TFLOPS, "nominal dense FP4 9 PFLOP/s (MEASURED_PEAKS.json holds no FP4 figure)"
    elif peaks:
        peak, peak_src = peaks["bf16_tflops"], "measured bf16 burst (MEASURED_PEAKS.json)"
    else:
        peak, peak_src = 1590.0, "fallback bf16 burst"
    # DRAM bytes of one launch of the dominant kernel (dram__bytes_read.sum + dram__bytes_write.sum of one
    # `ncu --set full` capture of this workload's gate|up launch at M = 10000, W4A4: 25.78 MB read + 0.58 MB
    # written; the quantised output stays in L2).  Not captured for other modes or row counts.
    traffic = 26.36e6 if (args.mode == "w4a4" and M == M_TOKENS) else None
    kname = ("umma_gemm_pair16_kernel (gate|up, SiLU-gate + quantising epilogue)" if args.mode == "w4a4"
             else "umma_gemm_kernel (gate|up, SiLU-gate epilogue)")
    roofline = {"bound": "tensor", "kernel": kname, "achieved": achieved,
                "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak, "peak_source": peak_src,
                "traffic": traffic, "launch_ms": top_ms, "gemm_ms_per_step": all_ms,
                "achieved_gbs": top[0][2] / (top_ms * 1e-3) / 1e9,
                "frac_of_measured_bf16": (achieved / peaks["bf16_tflops"]) if peaks else None}

    # ---- what the tensor pipe delivers to this kernel when nothing else is in the way ----------------
    # MEASURED_PEAKS.json has no FP4 figure, so measure one here: the dominant GEMM (same kernel, same
    # shape) with its operands left resident in shared memory after the first round of the ring and its
    # stores switched off, i.e. the k-loop at the rate of the MMA issue and the tensor pipe alone.
    mma_loop_tflops = None
    if args.mode == "w4a4":
        import ctypes
        from glm_asr_stack_b200 import _lib
        lib = _lib.load()
        w0 = keep[0]
        lib.glmasr_debug_set_flags(ctypes.c_int(4 | 8))
        try:
            for _ in range(3):
                ops.fp4_linear_fused(mode, xs[0], [w0["gate"], w0["up"]], epilogue=ops.EPI_SILU_GATE, input_scale=isc_h)
            ops.profile_enable(True)
            for _ in range(5):
                ops.fp4_linear_fused(mode, xs[0], [w0["gate"], w0["up"]], epilogue=ops.EPI_SILU_GATE, input_scale=isc_h)
            pk = [ms for ms, f, _ in ops.profile_read() if f == top_flops]
            ops.profile_enable(False)
            if pk:
                mma_loop_tflops = top_flops / (statistics.median(pk) * 1e-3) / 1e12
        finally:
            lib.glmasr_debug_set_flags(ctypes.c_int(-1))
        torch.cuda.synchronize()
        ops.status()
        roofline["mma_loop_tflops"] = mma_loop_tflops
        roofline["frac_of_mma_loop"] = (achieved / mma_loop_tflops) if mma_loop_tflops else None
        roofline["mma_loop_how"] = ("same kernel and shape with operands resident in shared memory (no loads after the "
                                    "first ring round) and stores off: the rate of MMA issue + tensor pipe alone")

    # ---- end to end: host buffers in, host buffers out, through the C-ABI host entry point ----
    for i in range(2):
        ops.layer_proj_host(mode, hin[i % 2], hout, layers[i % n_sets])
    barrier()
    t0 = time.perf_counter()
    for i in range(args.steps):
        ops.layer_proj_host(mode, hin[i % 2], hout, layers[i % n_sets])
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    e2e_s = replicas.max_over_ranks(e2e_s, dist, "cuda")
    e2e_val = replicas.whole_job_rate(layer_flops(M), world, e2e_s / args.steps) / 1e12
    bytes_io = M * HIDDEN * 2
    _st = ops.status()
    assert _st == 0, f"device status word = {_st} (bounded wait expired or CUDA error)"

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None,
            "dtype": "e2m1 x e2m1 block-scaled (ue4m3/16), fp32 accumulate" if args.mode == "w4a4" else
                     "bf16 x bf16 (e2m1 weights dequantised in-kernel), fp32 accumulate",
            "data": "synthetic",
            "config": {"workload": WORKLOAD, "rows": M, "arith": args.mode,
                       "l2": "4 weight sets + 2 inputs used round-robin; ~330 MB touched per step > 126 MB L2",
                       "parallelism": f"dp{world} replicas, no collective"},
            "e2e": {"value": e2e_val, "unit": UNIT, "h2d_bytes_per_step": bytes_io, "d2h_bytes_per_step": bytes_io,
                    "ms_per_step": e2e_s / args.steps * 1e3},
            "gpu_launches": int(launches), "clocks": clocks, "roofline": roofline,
        }
        if not args.no_cpu_baseline and world == 1:
            tf, sec, threads = cpu_reference_leg(2, 1, 512)
            line["cpu_baseline"] = {"value": tf, "unit": UNIT, "cores": threads, "kind": "port",
                                    "sample": f"512 of {M_TOKENS} rows, all four projections, full weights, "
                                              f"dequantise-every-call + fp32 GEMM in torch CPU ({sec:.2f} s/step)"}
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
