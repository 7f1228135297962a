#!/usr/bin/env python
"""Benchmark of the B200 operator set: one JSON line per run.

    python bench.py --gpus N --steps K --warmup W            # this library (default N=1)
    python bench.py --impl reference --steps K --warmup W    # the CPU check path on the host cores
    torchrun ... bench.py --gpus N ...                        # one rank per GPU, rows sharded, no collective

Headline workload (`config.workload`): the two BERT-Base row operators the reference's README quotes,
per GPU -- softmax FP32 [196608, 128] (logits N(0, 2^2), seed 0) followed by LayerNorm FP32
[16384, 768] (x ~ N(0,1), gamma ~ U(0.5,1.5), beta ~ N(0,0.1^2), eps 1e-12, seed 1).  One step = one
pass of both over one batch; with N GPUs the rows are sharded (N x the rows, weak scaling) and no data
crosses between GPUs.  `value` = algorithmic bytes of all ranks per step / device time (max over
ranks), inputs resident in HBM; every launch reads a buffer set that is not in L2 (the sets are
rotated and together exceed the 126 MB L2 several times).  `e2e` is the same metric through the
Tensor API with host buffers (pinned H2D before, D2H after, every step).

The GEMMs of the operator set (SGEMM 1024^3; FP16/BF16 tcgen05 GEMM 4096^3 and 16384x3072x768) are
timed in the same run next to cuBLAS and reported under "gemm"; the reference's own kernels recompiled
for sm_100a are timed, when their test-only library is present, under "reference_kernels_on_b200".
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

SOFTMAX_ROWS, SOFTMAX_COLS = 196608, 128
LN_ROWS, LN_COLS, LN_EPS = 16384, 768, 1e-12
SOFTMAX_BYTES = 2 * SOFTMAX_ROWS * SOFTMAX_COLS * 4
LN_BYTES = 2 * LN_ROWS * LN_COLS * 4 + 2 * LN_COLS * 4
STEP_BYTES = SOFTMAX_BYTES + LN_BYTES
METRIC, UNIT = "softmax+layernorm HBM throughput (BERT-Base row ops, FP32)", "GB/s"
WORKLOAD = ("bert_base_row_ops: softmax f32 [196608,128] N(0,4) seed 0 + layernorm f32 [16384,768] affine eps 1e-12 "
            "seed 1, per GPU; rows sharded across GPUs, no collective")
DATA_NOTE = "synthetic (seeded Philox4x32-10 fills of the benchmark shapes and distributions; no dataset involved)"
# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) from the ncu captures summarised in
# profiles/softmax_warp_kernel_196608x128.txt and profiles/layernorm_warp_kernel_16384x768.txt.  "isolated": one
# launch with the caches flushed before it, so the part of the output still dirty in the 126 MB L2 when the kernel ends
# is missing from the write count; "steady": launches back to back over rotating buffer sets with the caches left
# alone, where the write-back of the previous launch's output falls into this launch (mean of three consecutive
# launches of `bench.py --case softmax_c1` / `--case layernorm_c2` under ncu --cache-control none).
NCU_TRAFFIC = {
    "softmax": {"isolated": 145_612_800, "steady": 198_488_900},
    "layernorm": {"isolated": 56_400_000, "steady": 98_592_800},
}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), float(d.get("bf16_tflops", 1590.0)), "measured (MEASURED_PEAKS.json)"
    return 6650.0, 1590.0, "fallback (earlier measurement on this pool)"


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs (read-only)."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz, self._stop = [], set(), None, threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._nv = None

    def _loop(self):
        nv = self._nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
            "hw_power_brake": getattr(nv, "nvmlClocksEventReasonHwPowerBrakeSlowdown", 0x80),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)))
                get = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or nv.nvmlDeviceGetCurrentClocksThrottleReasons
                mask = int(get(self._h))
                for name, bit in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.002)

    def __enter__(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# --------------------------------------------------------------------------------------------------
# CPU check path (the oracle's FP32 ports, all host threads): the reference arm and the cpu_baseline leg
# --------------------------------------------------------------------------------------------------
def host_cores() -> int:
    """Cores this process may run on (torchrun pins OMP_NUM_THREADS to 1, so ask the scheduler instead)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return os.cpu_count() or 1


def cpu_port_step(oracle, xs, xl, g, b, threads):
    """One pass of the FP32 ports over the sample on `threads` host threads; returns seconds."""
    t0 = time.perf_counter()
    oracle.softmax_f32(xs, threads=threads)
    oracle.layernorm_f32(xl, LN_EPS, g, b, threads=threads)
    return time.perf_counter() - t0


def cpu_sample(oracle, fraction: int):
    rs, rl = SOFTMAX_ROWS // fraction, LN_ROWS // fraction
    xs = oracle.fill_normal((rs, SOFTMAX_COLS), 0, 0, 0.0, 2.0)
    xl = oracle.fill_normal((rl, LN_COLS), 1, 0, 0.0, 1.0)
    g, b = oracle.fill_uniform((LN_COLS,), 1, 1, 0.5, 1.5), oracle.fill_normal((LN_COLS,), 1, 2, 0.0, 0.1)
    sample_bytes = 2 * rs * SOFTMAX_COLS * 4 + 2 * rl * LN_COLS * 4 + 2 * LN_COLS * 4
    part = "all rows" if fraction == 1 else f"the first 1/{fraction} of the rows"
    return (xs, xl, g, b), sample_bytes, f"{part} of both operators ({rs} + {rl} rows), FP32 ports, every step"


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return  # the CPU arm runs on rank 0 only
    from oracle import ko_oracle as oracle

    cores = host_cores()
    sample, sample_bytes, what = cpu_sample(oracle, 1)  # every row of both operators: the GPU arm's per-GPU workload
    assert sample_bytes == STEP_BYTES
    for _ in range(max(args.warmup, 1)):
        cpu_port_step(oracle, *sample, cores)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_port_step(oracle, *sample, cores)
    elapsed = time.perf_counter() - t0
    gbs = sample_bytes * args.steps / elapsed / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": elapsed / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": DATA_NOTE,
        "config": {"workload": WORKLOAD},
        "cpu_baseline": {"value": gbs, "unit": UNIT, "cores": cores, "kind": "port", "sample": what},
        "e2e": {"value": gbs, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference project has no CPU implementation; this is the oracle's FP32 restatement of its kernels "
                "(softmax.h:32-58, layernorm.h:13-50/:184-198 with the merge defect removed) on all host threads, "
                "one GPU's worth of rows per step whatever --gpus says (rank 0 only)",
    }
    emit(line)


# --------------------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------------------
E2E_CHUNKS = 6
REPEAT_BATCHES = 10  # the timed batch of --steps steps is repeated this often; value = the median batch


class Rig:
    """One rank: its device, the process group and the timing rules (barrier + synchronize on both sides of a timed
    region, CUDA events on the launch stream, max over ranks)."""

    def __init__(self, args):
        import torch
        import torch.distributed as dist

        from kernel_optimization_b200 import native, sharding

        self.torch, self.dist, self.sharding, self.native = torch, dist, sharding, native
        self.lib = native.lib()  # raises when the CUDA library has not been built: there is no fallback
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        if self.world != args.gpus and self.world == 1 and args.gpus > 1:
            raise SystemExit(f"--gpus {args.gpus} needs torchrun with {args.gpus} ranks (WORLD_SIZE is 1)")
        torch.cuda.set_device(self.local_rank)
        self.dev = torch.device("cuda", self.local_rank)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.dev)
        self.hbm_peak, self.tc_peak, self.peak_kind = measured_peaks()

    def stream(self):
        return self.torch.cuda.current_stream().cuda_stream

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, ms: float) -> float:
        return self.sharding.max_over_ranks(ms, self.dev)

    def timed(self, fn, iters, warm):
        """ms per iteration of fn(i): `warm` untimed calls, then exactly `iters` calls between two events."""
        torch = self.torch
        for i in range(warm):
            fn(i)
        self.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(iters):
            fn(i)
        e1.record()
        self.barrier()
        return self.max_over_ranks(e0.elapsed_time(e1)) / iters

    def per_launch(self, fn, iters, warm):
        """(median, min) microseconds of single launches: an event between every two calls (which also keeps
        consecutive launches from overlapping, unlike the back-to-back figure), max over ranks of each statistic."""
        torch = self.torch
        for i in range(warm):
            fn(i)
        self.barrier()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(iters + 1)]
        ev[0].record()
        for i in range(iters):
            fn(i)
            ev[i + 1].record()
        self.barrier()
        us = sorted(ev[i].elapsed_time(ev[i + 1]) * 1e3 for i in range(iters))
        return self.max_over_ranks(statistics.median(us)), self.max_over_ranks(us[0])

    def close(self):
        if self.world > 1:
            self.dist.destroy_process_group()


def measure_link_ceiling(rig, bytes_each_way: int, iters: int):
    """Plain pinned-memory copies of `bytes_each_way` host->device and device->host at the same time on two streams,
    every rank at once; GB/s summed over both directions and all ranks (wall clock between barriers, max over ranks)."""
    torch = rig.torch
    n = bytes_each_way
    h_in, h_out = torch.empty(n, dtype=torch.uint8).pin_memory(), torch.empty(n, dtype=torch.uint8).pin_memory()
    d_in, d_out = torch.empty(n, dtype=torch.uint8, device=rig.dev), torch.empty(n, dtype=torch.uint8, device=rig.dev)
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()

    def go(h2d: bool, d2h: bool):
        def once():
            if h2d:
                with torch.cuda.stream(s_in):
                    d_in.copy_(h_in, non_blocking=True)
            if d2h:
                with torch.cuda.stream(s_out):
                    h_out.copy_(d_out, non_blocking=True)
        once()
        rig.barrier()
        t0 = time.perf_counter()
        for _ in range(iters):
            once()
        torch.cuda.synchronize()
        dt = rig.max_over_ranks((time.perf_counter() - t0) * 1e3) / iters  # ms
        rig.barrier()
        return n * ((1 if h2d else 0) + (1 if d2h else 0)) * rig.world / (dt * 1e-3) / 1e9

    out = {"h2d_gbs": go(True, False), "d2h_gbs": go(False, True), "both_directions_gbs": go(True, True),
           "bytes_each_way_per_rank": n, "ranks": rig.world,
           "how": "one pinned cudaMemcpyAsync per direction on its own stream, all ranks at once, no kernel"}
    del h_in, h_out, d_in, d_out
    return out


def run_gpu_arm(args):
    import torch

    import kernel_optimization_b200 as ko
    from kernel_optimization_b200 import native, sharding

    rig = Rig(args)
    lib, world, rank, local_rank, dev = rig.lib, rig.world, rig.rank, rig.local_rank, rig.dev
    stream, barrier, timed = rig.stream, rig.barrier, rig.timed
    hbm_peak, tc_peak, peak_kind = rig.hbm_peak, rig.tc_peak, rig.peak_kind

    # ---- inputs: this rank's row shard of the global tensors, seeded by global element index
    sm_off = sharding.weak_scaled_rows(SOFTMAX_ROWS, SOFTMAX_COLS, rank, world).elem_offset
    ln_off = sharding.weak_scaled_rows(LN_ROWS, LN_COLS, rank, world).elem_offset
    xs_host = ko.fill_normal((SOFTMAX_ROWS, SOFTMAX_COLS), 0, 0, 0.0, 2.0, elem_offset=sm_off)
    xl_host = ko.fill_normal((LN_ROWS, LN_COLS), 1, 0, 0.0, 1.0, elem_offset=ln_off)
    g_host, b_host = ko.fill_uniform((LN_COLS,), 1, 1, 0.5, 1.5), ko.fill_normal((LN_COLS,), 1, 2, 0.0, 0.1)
    # default 4 x 201 MB and 8 x 101 MB of distinct addresses: nothing survives in the 126 MB L2
    n_sm_sets, n_ln_sets = (args.row_sets, args.row_sets) if args.row_sets > 0 else (4, 8)
    sm_in = [torch.from_numpy(xs_host).to(dev) for _ in range(n_sm_sets)]
    sm_out = [torch.empty_like(sm_in[0]) for _ in range(n_sm_sets)]
    ln_in = [torch.from_numpy(xl_host).to(dev) for _ in range(n_ln_sets)]
    ln_out = [torch.empty_like(ln_in[0]) for _ in range(n_ln_sets)]
    gamma, beta = torch.from_numpy(g_host).to(dev), torch.from_numpy(b_host).to(dev)

    def softmax_launch(i):
        j = i % n_sm_sets
        native.check(lib.ko_softmax_f32(sm_in[j].data_ptr(), sm_out[j].data_ptr(), SOFTMAX_ROWS, SOFTMAX_COLS, stream()),
                     "ko_softmax_f32")

    def layernorm_launch(i):
        j = i % n_ln_sets
        native.check(lib.ko_layernorm_f32(ln_in[j].data_ptr(), ln_out[j].data_ptr(), LN_ROWS, LN_COLS, LN_EPS,
                                          gamma.data_ptr(), beta.data_ptr(), 0, stream()), "ko_layernorm_f32")

    def step(i):
        softmax_launch(i)
        layernorm_launch(i)

    # ---- headline: K steps of (softmax, layernorm), the batch repeated; the median batch is the reported one
    with ClockSampler(local_rank) as clocks:
        batches = [timed(step, args.steps, args.warmup)]
        batches += [timed(step, args.steps, 0) for _ in range(REPEAT_BATCHES - 1)]
        # per-kernel durations for the roofline, same buffers, same stream
        sm_batches = [timed(softmax_launch, args.steps, args.warmup if b == 0 else 0) for b in range(5)]
        ln_batches = [timed(layernorm_launch, args.steps, args.warmup if b == 0 else 0) for b in range(5)]
        sm_med_us, sm_min_us = rig.per_launch(softmax_launch, max(args.steps, 20), 3)
        ln_med_us, ln_min_us = rig.per_launch(layernorm_launch, max(args.steps, 20), 3)
    ms_per_step = statistics.median(batches)
    ms_softmax, ms_layernorm = statistics.median(sm_batches), statistics.median(ln_batches)
    value = STEP_BYTES * world / (ms_per_step * 1e-3) / 1e9
    softmax_gbs = SOFTMAX_BYTES / (ms_softmax * 1e-3) / 1e9
    layernorm_gbs = LN_BYTES / (ms_layernorm * 1e-3) / 1e9
    repeat = {"batches": len(batches), "steps_per_batch": args.steps, "ms_per_step": batches, "median": ms_per_step,
              "min": min(batches), "max": max(batches), "spread": (max(batches) - min(batches)) / ms_per_step,
              "note": "every batch is exactly --steps steps between two events with a barrier + synchronize on both sides; "
                      "value and ms_per_step are the median batch"}

    # ---- parity spot check of what was just timed (rank 0; the oracle is only the checker here)
    parity = None
    if rank == 0:
        from oracle import ko_oracle as oracle

        pick = np.r_[0:256, SOFTMAX_ROWS - 256:SOFTMAX_ROWS]
        y = sm_out[0][torch.from_numpy(pick).to(dev)].cpu().numpy()
        parity = {"softmax_max_abs": oracle.max_abs_err(y, oracle.softmax_f64(xs_host[pick]))}
        pick = np.r_[0:256, LN_ROWS - 256:LN_ROWS]
        y = ln_out[0][torch.from_numpy(pick).to(dev)].cpu().numpy()
        parity["layernorm_max_rel"] = oracle.max_rel_err(y, oracle.layernorm_f64(xl_host[pick], LN_EPS, g_host, b_host))

    # ---- e2e: host buffers through the Tensor API, H2D + kernels + D2H inside the timed region
    t_sm_in, t_sm_out = ko.Tensor(SOFTMAX_BYTES // 2, local_rank), ko.Tensor(SOFTMAX_BYTES // 2, local_rank)
    t_ln_in, t_ln_out = ko.Tensor(LN_ROWS * LN_COLS * 4, local_rank), ko.Tensor(LN_ROWS * LN_COLS * 4, local_rank)
    t_sm_in.host_ref(np.float32)[:] = xs_host.reshape(-1)
    t_ln_in.host_ref(np.float32)[:] = xl_host.reshape(-1)

    # The two operators of a step are independent, so a caller gives each its own stream: the second call's copies then
    # queue right behind the first call's on the library's copy lanes instead of waiting for its last copy out.
    e2e_streams = (torch.cuda.Stream(), torch.cuda.Stream())
    e2e_joined = (torch.cuda.Event(), torch.cuda.Event())

    def e2e_step(_i):
        # the public host-tensor calls: rows flow through copy-in / kernel / copy-out streams in chunks
        main = torch.cuda.current_stream()
        for st in e2e_streams:
            st.wait_stream(main)
        ko.softmax_host(t_sm_in, t_sm_out, SOFTMAX_ROWS, SOFTMAX_COLS, args.e2e_chunks, stream=e2e_streams[0].cuda_stream)
        ko.layernorm_host(t_ln_in, t_ln_out, LN_ROWS, LN_COLS, LN_EPS, gamma, beta, 0, args.e2e_chunks, stream=e2e_streams[1].cuda_stream)
        for st, ev in zip(e2e_streams, e2e_joined):
            ev.record(st)
            main.wait_event(ev)  # the step ends (and the timing events follow) once both results are on the host

    e2e_steps = max(3, min(args.steps, 20))
    ms_e2e = timed(e2e_step, e2e_steps, 3)
    h2d = SOFTMAX_BYTES // 2 + LN_ROWS * LN_COLS * 4
    e2e = {"value": STEP_BYTES * world / (ms_e2e * 1e-3) / 1e9, "unit": UNIT, "h2d_bytes_per_step": h2d,
           "d2h_bytes_per_step": h2d, "ms_per_step": ms_e2e, "steps": e2e_steps,
           "path": f"ko_softmax_f32_host + ko_layernorm_f32_host on one stream each, {args.e2e_chunks} nominal chunks per call: pinned host -> "
                   "device -> kernel -> pinned host, copies of neighbouring chunks overlap (PCIe is full duplex); every step ends with "
                   "all results on the host"}
    # the host link itself, all ranks at once: the step's bytes as one large pinned copy per direction on two
    # streams, no kernel -- what any pipeline through this host's PCIe fabric could reach at this rank count
    link = measure_link_ceiling(rig, h2d, 5)
    e2e["link_ceiling_gbs"] = link["both_directions_gbs"]
    e2e["of_link_ceiling"] = e2e["value"] / link["both_directions_gbs"]
    e2e["link"] = link
    if rank == 0:
        from oracle import ko_oracle as oracle

        got = t_sm_out.host_ref(np.float32).reshape(SOFTMAX_ROWS, SOFTMAX_COLS)[:256]
        parity["e2e_softmax_max_abs"] = oracle.max_abs_err(got, oracle.softmax_f64(xs_host[:256]))
    del t_sm_in, t_sm_out, t_ln_in, t_ln_out, sm_in, sm_out, ln_in, ln_out

    # ---- GEMMs next to cuBLAS (each rank its own M-block; B replicated by one NCCL broadcast, untimed)
    gemm = {}
    if not args.skip_gemm:
        torch.backends.cuda.matmul.allow_tf32 = False
        torch.backends.cudnn.allow_tf32 = False

        replicate = sharding.replicate_from_rank0

        def bench_gemm(name, fn_ours, fn_cublas, flops, iters=20):
            ms_o = timed(fn_ours, iters, 3)
            ms_c = timed(fn_cublas, iters, 3)
            gemm[name] = {"tflops": flops * world / (ms_o * 1e-3) / 1e12, "us": ms_o * 1e3,
                          "cublas_tflops": flops * world / (ms_c * 1e-3) / 1e12, "cublas_us": ms_c * 1e3,
                          "vs_cublas": ms_c / ms_o}

        M = N = K = 1024
        nset = 8
        a_h, b_h = ko.fill_uniform((M, K), 2, 0, elem_offset=rank * M * K), ko.fill_uniform((K, N), 2, 1)
        As = [torch.from_numpy(a_h).to(dev) for _ in range(nset)]
        Bs = [replicate(torch.from_numpy(b_h).to(dev)) for _ in range(nset)]
        Ds = [torch.empty((M, N), device=dev) for _ in range(nset)]
        bench_gemm("sgemm_f32_1024",
                   lambda i: native.check(lib.ko_sgemm_f32(M, N, K, As[i % nset].data_ptr(), Bs[i % nset].data_ptr(), None,
                                                           Ds[i % nset].data_ptr(), stream()), "ko_sgemm_f32"),
                   lambda i: torch.matmul(As[i % nset], Bs[i % nset], out=Ds[i % nset]), 2.0 * M * N * K, iters=50)
        gemm["sgemm_f32_1024"]["cublas_math"] = "cublasSgemm via torch.matmul, TF32 disabled (FFMA)"
        del As, Bs, Ds
        for kind, tdt, code, fn in (("bf16", torch.bfloat16, 2, lib.ko_gemm_bf16_f32), ("f16", torch.float16, 1, lib.ko_gemm_f16_f32)):
            for tag, (M, N, K) in (("4096", (4096, 4096, 4096)), ("ffn_16384x3072x768", (16384, 3072, 768))):
                nset = 3
                a_h = ko.fill_uniform((M, K), 3, 0, dtype=code, elem_offset=rank * M * K)
                b_h = ko.fill_uniform((N, K), 3, 1, dtype=code)
                As = [torch.from_numpy(a_h.view(np.int16)).to(dev).view(tdt) for _ in range(nset)]
                Bs = [replicate(torch.from_numpy(b_h.view(np.int16)).to(dev).view(tdt)) for _ in range(nset)]
                Ds = [torch.empty((M, N), device=dev) for _ in range(nset)]
                bench_gemm(f"gemm_{kind}_f32_{tag}",
                           lambda i: native.check(fn(M, N, K, As[i % nset].data_ptr(), Bs[i % nset].data_ptr(), None,
                                                     Ds[i % nset].data_ptr(), stream()), "ko_gemm_tc"),
                           lambda i: torch.mm(As[i % nset], Bs[i % nset].t(), out_dtype=torch.float32), 2.0 * M * N * K)
                gemm[f"gemm_{kind}_f32_{tag}"]["of_measured_bf16_peak"] = gemm[f"gemm_{kind}_f32_{tag}"]["tflops"] / world / tc_peak
                del As, Bs, Ds
        torch.cuda.synchronize()
        native.check(lib.ko_poll_device_status(), "ko_poll_device_status")

    # ---- long rows (every rank its own rows): the tiers beyond one block's registers, with a parity spot check
    long_rows = {}
    if not args.skip_gemm:
        lr_rows, lr_cols, lr_sets = 1024, 65536, 2
        lr_bytes = 2.0 * lr_rows * lr_cols * 4
        x_h = ko.fill_normal((lr_rows, lr_cols), 5, 0, 0.0, 2.0, elem_offset=rank * lr_rows * lr_cols)
        g_h, b_h = ko.fill_uniform((lr_cols,), 5, 1, 0.5, 1.5), ko.fill_normal((lr_cols,), 5, 2, 0.0, 0.1)
        xs = [torch.from_numpy(x_h).to(dev) for _ in range(lr_sets)]
        ys = [torch.empty_like(xs[0]) for _ in range(lr_sets)]
        gd, bd = torch.from_numpy(g_h).to(dev), torch.from_numpy(b_h).to(dev)
        ms = timed(lambda i: native.check(lib.ko_softmax_f32(xs[i % lr_sets].data_ptr(), ys[i % lr_sets].data_ptr(), lr_rows, lr_cols,
                                                             stream()), "ko_softmax_f32"), 20, 3)
        err = oracle.max_abs_err(ys[0][:4].cpu().numpy(), oracle.softmax_f64(x_h[:4])) if rank == 0 else None
        long_rows["softmax_f32_1024x65536"] = {"gbs": lr_bytes * world / (ms * 1e-3) / 1e9, "us": ms * 1e3,
                                               "of_peak_per_gpu": lr_bytes / (ms * 1e-3) / 1e9 / hbm_peak, "max_abs_4_rows": err}
        ms = timed(lambda i: native.check(lib.ko_layernorm_f32(xs[i % lr_sets].data_ptr(), ys[i % lr_sets].data_ptr(), lr_rows, lr_cols,
                                                               LN_EPS, gd.data_ptr(), bd.data_ptr(), 0, stream()), "ko_layernorm_f32"), 20, 3)
        err = oracle.max_rel_err(ys[0][:4].cpu().numpy(), oracle.layernorm_f64(x_h[:4], LN_EPS, g_h, b_h)) if rank == 0 else None
        long_rows["layernorm_f32_1024x65536"] = {"gbs": lr_bytes * world / (ms * 1e-3) / 1e9, "us": ms * 1e3,
                                                 "of_peak_per_gpu": lr_bytes / (ms * 1e-3) / 1e9 / hbm_peak, "max_rel_4_rows": err}
        long_rows["note"] = ("rows longer than one block's registers: one row per block in two passes, the second served by the L2; "
                             "2 rotating buffer sets of 537 MB per rank")
        del xs, ys, gd, bd

    # ---- the reference's own kernels, recompiled for sm_100a (test-only library; informational)
    ref_rows = None
    ref_path = os.path.join(ROOT, "oracle", "_ref", "libko_ref_kernels.so")
    if rank == 0 and world == 1 and os.path.exists(ref_path) and not args.skip_gemm:
        ref = C.CDLL(ref_path)
        vp, ll, ci, f32 = C.c_void_p, C.c_longlong, C.c_int, C.c_float
        ref.ko_ref_softmax_f32.argtypes = [vp, vp, ll, ci, vp]
        ref.ko_ref_layernorm_f32.argtypes = [vp, vp, ll, ci, f32, vp, vp, ci, vp]
        xs = [torch.from_numpy(xs_host).to(dev) for _ in range(4)]
        ys = [torch.empty_like(xs[0]) for _ in range(4)]
        ms = timed(lambda i: ref.ko_ref_softmax_f32(xs[i % 4].data_ptr(), ys[i % 4].data_ptr(), SOFTMAX_ROWS, SOFTMAX_COLS, stream()), 30, 3)
        ref_rows = {"softmax_gbs": SOFTMAX_BYTES / (ms * 1e-3) / 1e9}
        del xs, ys
        xl = [torch.from_numpy(xl_host).to(dev) for _ in range(8)]
        yl = [torch.empty_like(xl[0]) for _ in range(8)]
        ms = timed(lambda i: ref.ko_ref_layernorm_f32(xl[i % 8].data_ptr(), yl[i % 8].data_ptr(), LN_ROWS, LN_COLS, 1e-4, None, None, 0, stream()), 30, 3)
        ref_rows["layernorm_gbs"] = LN_BYTES / (ms * 1e-3) / 1e9
        ref_rows["note"] = "SoftMaxWarpImpl / LayerNormWarpImpl at the reference driver's launch geometry; the LayerNorm result is not LayerNorm (its Welford merge divides at every level)"
        del xl, yl

    # ---- CPU baseline beside it (rank 0, single-GPU runs only)
    cpu_baseline = None
    if rank == 0 and world == 1 and not args.skip_cpu:
        from oracle import ko_oracle as oracle

        sample, sample_bytes, what = cpu_sample(oracle, 1)
        cores = host_cores()
        cpu_port_step(oracle, *sample, cores)
        reps = 5
        best = min(cpu_port_step(oracle, *sample, cores) for _ in range(reps))
        cpu_baseline = {"value": sample_bytes / best / 1e9, "unit": UNIT, "cores": cores, "kind": "port",
                        "sample": f"the full per-GPU workload (all rows of both operators), FP32 ports, best of {reps} passes"}

    # ---- benchmark config 5 (the 1/2/4/8-GPU sweep's own shapes, strong scaling) under the same clock
    scaled = None
    if not args.skip_scaled:
        torch.cuda.empty_cache()
        c5_ops, c5_parity = scaled_ops(rig, max(3, min(args.steps, 10)), 3)
        scaled = {"workload": SCALED_WORKLOAD, "scaling": "strong (totals fixed, every rank takes 1/N)", "ops": c5_ops,
                  "parity_worst_over_ranks": c5_parity,
                  "l2": "every per-GPU operand is larger than the 126 MB L2"}

    if rank == 0:
        def roofline_of(kernel, gbs, ms, nbytes, traffic):
            return {"bound": "hbm", "kernel": kernel, "achieved": gbs, "peak": hbm_peak, "unit": "GB/s", "frac": gbs / hbm_peak,
                    "traffic": traffic["steady"] if traffic["steady"] is not None else traffic["isolated"],
                    "traffic_kind": ("steady state: back-to-back launches over rotating buffer sets, caches left alone"
                                     if traffic["steady"] is not None else
                                     "isolated launch, caches flushed before it: part of the output is still dirty in L2 when the "
                                     "kernel ends, so this is below the algorithmic bytes; it shows that nothing is read twice"),
                    "traffic_isolated_launch": traffic["isolated"], "peak_source": peak_kind,
                    "algorithmic_bytes_per_launch": nbytes, "us_per_launch": ms * 1e3}

        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": DATA_NOTE,
            "config": {"workload": WORKLOAD},
            "run": {"rows_per_gpu": {"softmax": SOFTMAX_ROWS, "layernorm": LN_ROWS},
                    "l2": f"inputs and outputs rotate over {n_sm_sets} (softmax) / {n_ln_sets} (layernorm) buffer sets "
                          f"({n_sm_sets * SOFTMAX_BYTES / 1e6:.0f} / {n_ln_sets * LN_BYTES / 1e6:.0f} MB of distinct addresses "
                          "against a 126 MB L2), so every launch reads from HBM",
                    "parallelism": f"rows x{world}, no collective"},
            "repeat": repeat,
            "roofline": roofline_of("softmax_warp_kernel (softmax f32 [196608,128])", softmax_gbs, ms_softmax, SOFTMAX_BYTES,
                                    NCU_TRAFFIC["softmax"]),
            "roofline_layernorm": roofline_of("layernorm_warp_kernel (layernorm f32 [16384,768])", layernorm_gbs, ms_layernorm,
                                              LN_BYTES, NCU_TRAFFIC["layernorm"]),
            "ops": {"softmax": {"gbs": softmax_gbs, "us": ms_softmax * 1e3, "of_peak": softmax_gbs / hbm_peak, "of_nominal_8TBs": softmax_gbs / 8000.0,
                                "us_per_launch_median": sm_med_us, "us_per_launch_min": sm_min_us},
                    "layernorm": {"gbs": layernorm_gbs, "us": ms_layernorm * 1e3, "of_peak": layernorm_gbs / hbm_peak, "of_nominal_8TBs": layernorm_gbs / 8000.0,
                                  "us_per_launch_median": ln_med_us, "us_per_launch_min": ln_min_us},
                    "note": "us / gbs: median of 5 batches of --steps launches back to back (consecutive launches overlap their "
                            "ramps through programmatic dependent launch); us_per_launch_*: single launches with an event between them"},
            "cpu_baseline": cpu_baseline, "e2e": e2e, "gpu_launches": 2 * args.steps, "clocks": clocks.summary(),
            "parity": parity, "gemm": gemm, "long_rows": long_rows, "scaled": scaled, "reference_kernels_on_b200": ref_rows,
        }
        emit(line)
    rig.close()


# --------------------------------------------------------------------------------------------------
# benchmark config 5: the scaled sweep, strong scaling (the totals are fixed, every rank takes 1/N)
# --------------------------------------------------------------------------------------------------
C5_SOFTMAX_ROWS, C5_SOFTMAX_COLS = 8 * 196608, 512
C5_LN_ROWS, C5_LN_COLS = 262144, 4096
C5_M, C5_N, C5_K = 65536, 8192, 8192


def scaled_ops(rig, steps, warmup):
    """Benchmark config 5 on this rank's shard: softmax FP32 [8x196608, 512] causal -1e4, LayerNorm BF16 [262144, 4096],
    BF16 GEMM 65536 x 8192 x 8192 (B replicated by one NCCL broadcast, outside the timed region), seed 4; the totals
    are fixed and rows / M-blocks are sharded over the ranks (strong scaling).  Every rank generates only its own shard.
    Returns (per-operator results, parity worst over ranks)."""
    import kernel_optimization_b200 as ko

    torch, dist, sharding, native, lib = rig.torch, rig.dist, rig.sharding, rig.native, rig.lib
    world, rank, dev = rig.world, rig.rank, rig.dev
    hbm_peak, tc_peak = rig.hbm_peak, rig.tc_peak
    stream, barrier = rig.stream, rig.barrier

    def timed(fn, iters, warm):
        return rig.timed(lambda _i: fn(), iters, warm)

    from oracle import ko_oracle as oracle  # checker for the sampled rows below

    out = {}
    parity = {}
    rng = np.random.default_rng(4 + rank)
    # ---- softmax: shard boundaries on multiples of 512 keep every causal block on one GPU
    sh = sharding.row_shard(C5_SOFTMAX_ROWS, C5_SOFTMAX_COLS, rank, world, multiple_of=512)
    x = ko.fill_normal((sh.rows, sh.cols), 4, 0, 0.0, 2.0, elem_offset=sh.elem_offset)
    ko.fill_causal_mask_(x, sh.begin, 512, -1e4)
    xd = torch.from_numpy(x).to(dev)
    yd = torch.empty_like(xd)
    ms = timed(lambda: native.check(lib.ko_softmax_f32(xd.data_ptr(), yd.data_ptr(), sh.rows, sh.cols, stream()), "softmax"),
               steps, warmup)
    total = 2.0 * C5_SOFTMAX_ROWS * C5_SOFTMAX_COLS * 4
    out["softmax_f32_causal"] = {"gbs": total / (ms * 1e-3) / 1e9, "ms": ms, "of_peak_per_gpu": total / world / (ms * 1e-3) / 1e9 / hbm_peak,
                                 "bytes": total, "rows_per_gpu": sh.rows}
    pick = np.unique(np.r_[0:512, sh.rows - 512:sh.rows, rng.integers(0, sh.rows, 4096)])
    got = yd[torch.from_numpy(pick).to(dev)].cpu().numpy()
    parity["softmax_max_abs"] = oracle.max_abs_err(got, oracle.softmax_f64(x[pick]))
    parity["softmax_rowsum"] = oracle.max_rowsum_err(got)
    del x, xd, yd
    # ---- LayerNorm BF16
    sh = sharding.row_shard(C5_LN_ROWS, C5_LN_COLS, rank, world)
    xb = ko.fill_normal((sh.rows, sh.cols), 4, 1, 0.0, 1.0, dtype=2, elem_offset=sh.elem_offset)
    gb, bb = ko.fill_uniform((sh.cols,), 4, 2, 0.5, 1.5, dtype=2), ko.fill_normal((sh.cols,), 4, 3, 0.0, 0.1, dtype=2)
    to_dev = lambda a: torch.from_numpy(a.view(np.int16)).to(dev)  # noqa: E731
    xd, gd, bd = to_dev(xb), to_dev(gb), to_dev(bb)
    yd = torch.empty_like(xd)
    ms = timed(lambda: native.check(lib.ko_layernorm_bf16(xd.data_ptr(), yd.data_ptr(), sh.rows, sh.cols, LN_EPS, gd.data_ptr(),
                                                          bd.data_ptr(), 0, stream()), "layernorm"), steps, warmup)
    total = 2.0 * C5_LN_ROWS * C5_LN_COLS * 2
    out["layernorm_bf16"] = {"gbs": total / (ms * 1e-3) / 1e9, "ms": ms, "of_peak_per_gpu": total / world / (ms * 1e-3) / 1e9 / hbm_peak,
                             "bytes": total, "rows_per_gpu": sh.rows}
    pick = np.unique(np.r_[0:64, sh.rows - 64:sh.rows, rng.integers(0, sh.rows, 512)])
    got = oracle.from_bf16_bits(yd[torch.from_numpy(pick).to(dev)].cpu().numpy().view(np.uint16))
    want = oracle.layernorm_f64(oracle.from_bf16_bits(xb[pick]), LN_EPS, oracle.from_bf16_bits(gb), oracle.from_bf16_bits(bb))
    parity["layernorm_bf16_max_rel"] = oracle.max_rel_err(got, want)
    del xb, xd, yd
    # ---- BF16 GEMM, M-sharded, B broadcast once (timed separately)
    sh = sharding.row_shard(C5_M, C5_K, rank, world, multiple_of=128)
    ab = ko.fill_uniform((sh.rows, C5_K), 4, 4, dtype=2, elem_offset=sh.elem_offset)
    ad = to_dev(ab)
    bh = ko.fill_uniform((C5_N, C5_K), 4, 5, dtype=2) if rank == 0 else None
    bd = to_dev(bh) if rank == 0 else torch.empty((C5_N, C5_K), dtype=torch.int16, device=dev)
    sharding.replicate_from_rank0(bd)  # the first broadcast also brings the communicator's channels up: not timed
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    sharding.replicate_from_rank0(bd)  # same bytes again, warm: the NVLink figure
    e1.record()
    barrier()
    bcast_ms = rig.max_over_ranks(e0.elapsed_time(e1)) if world > 1 else 0.0
    dd = torch.empty((sh.rows, C5_N), device=dev)
    gsteps = max(2, min(steps, 5))
    ms = timed(lambda: native.check(lib.ko_gemm_bf16_f32(sh.rows, C5_N, C5_K, ad.data_ptr(), bd.data_ptr(), None, dd.data_ptr(), stream()),
                                    "gemm"), gsteps, 1)
    flops = 2.0 * C5_M * C5_N * C5_K
    a_t, b_t = ad.view(torch.bfloat16), bd.view(torch.bfloat16)
    ms_c = timed(lambda: torch.mm(a_t, b_t.t(), out_dtype=torch.float32), gsteps, 1)
    out["gemm_bf16_f32"] = {"tflops": flops / (ms * 1e-3) / 1e12, "ms": ms, "cublas_tflops": flops / (ms_c * 1e-3) / 1e12, "vs_cublas": ms_c / ms,
                            "of_measured_bf16_peak_per_gpu": flops / world / (ms * 1e-3) / 1e12 / tc_peak, "flops": flops,
                            "b_broadcast_ms": bcast_ms, "b_bytes": C5_N * C5_K * 2, "m_per_gpu": sh.rows,
                            "b_broadcast_gbs": (C5_N * C5_K * 2 / (bcast_ms * 1e-3) / 1e9) if bcast_ms > 0 else None,
                            "b_broadcast_note": "second (warm) NCCL broadcast of B from rank 0, device-timed, max over ranks; "
                                                "outside the steady-state timing"}
    native.check(lib.ko_poll_device_status(), "ko_poll_device_status")
    rows = np.unique(np.r_[0:8, sh.rows - 8:sh.rows, rng.integers(0, sh.rows, 16)])
    bfull = oracle.from_bf16_bits(bd.cpu().numpy().view(np.uint16))
    want = oracle.gemm_tn_f64(oracle.from_bf16_bits(ab[rows]), bfull)
    parity["gemm_rel_fro_sampled_rows"] = oracle.rel_frobenius(dd[torch.from_numpy(rows).to(dev)].cpu().numpy(), want)
    del ab, ad, bd, dd, a_t, b_t
    torch.cuda.empty_cache()
    gathered = [None] * world
    if world > 1:
        dist.all_gather_object(gathered, parity)
    else:
        gathered = [parity]
    worst = {k: max(g[k] for g in gathered) for k in parity}
    return out, worst


SCALED_WORKLOAD = ("config5_scaled: softmax f32 [1572864,512] causal -1e4 + layernorm bf16 [262144,4096] + bf16 gemm 65536x8192x8192, "
                   "rows / M-blocks sharded, B replicated by one untimed NCCL broadcast")


def run_scaled(args):
    """`--workload scaled`: benchmark config 5 alone, one JSON line."""
    rig = Rig(args)
    out, worst = scaled_ops(rig, args.steps, args.warmup)
    if rig.rank == 0:
        row_bytes = out["softmax_f32_causal"]["bytes"] + out["layernorm_bf16"]["bytes"]
        row_ms = out["softmax_f32_causal"]["ms"] + out["layernorm_bf16"]["ms"]
        emit({"metric": "scaled sweep (benchmark config 5): softmax+layernorm HBM throughput", "value": row_bytes / (row_ms * 1e-3) / 1e9,
              "unit": UNIT, "n_gpus": rig.world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": row_ms, "higher_is_better": True,
              "scaling": "strong", "vs_baseline": None, "dtype": "f32 softmax / bf16 layernorm (f32 statistics) / bf16 gemm (f32 accumulate)",
              "data": "synthetic (seeded Philox4x32-10, seed 4)",
              "config": {"workload": SCALED_WORKLOAD,
                         "l2": "every per-GPU operand is larger than the 126 MB L2", "parallelism": f"rows and M-blocks x{rig.world}, no data-path collective"},
              "ops": out, "parity_worst_over_ranks": worst, "peak_source": rig.peak_kind})
    rig.close()


CASES = {
    "sgemm_2048": "FP32 SGEMM 2048^3 (48 MB of operands)",
    "sgemm_1024": "FP32 SGEMM 1024^3 (benchmark config 3)",
    "gemm_bf16_4096": "BF16 tcgen05 GEMM 4096^3 (benchmark config 4)",
    "gemm_bf16_ffn": "BF16 tcgen05 GEMM 16384x3072x768 (benchmark config 4, FFN shape)",
    "softmax_c5_shard": "softmax FP32 [196608,512] with the causal -1e4 pattern (1/8 of benchmark config 5)",
    "layernorm_bf16_c5_shard": "LayerNorm BF16 [32768,4096] (1/8 of benchmark config 5)",
    "softmax_long_rows": "softmax FP32 [2048,32768]: one row per block in registers, the next row prefetched by a bulk copy",
    "softmax_cluster_rows": "softmax FP32 [256,131072], cluster tier forced: one row per cluster of 4 blocks, (max, sum) pairs exchanged through DSMEM mailboxes",
    "layernorm_cluster_rows": "LayerNorm FP32 [256,131072] affine, cluster tier forced: one row per cluster of 4 blocks, Welford triples exchanged through DSMEM mailboxes",
    "softmax_reread_rows": "softmax FP32 [1024,65536]: one row per block in two passes, the second served by the L2 (the default for such rows)",
    "layernorm_reread_rows": "LayerNorm FP32 [1024,131072] affine: two rows per block at a time, two passes, gamma / beta loaded once per pair (the default for such rows)",
    "softmax_block_rows": "softmax FP32 [3640,9216]: one row per block in registers, 576 threads of four vectors (exactly what the row needs)",
    "layernorm_c2": "LayerNorm FP32 [16384,768] affine (benchmark config 2), 8 rotating buffer sets",
    "softmax_c1": "softmax FP32 [196608,128] (benchmark config 1), 4 rotating buffer sets",
    "gemm_bf16_ffn_pair": "BF16 GEMM 16384x3072x768 on the two-SM kernel (tcgen05 cta_group::2)",
    "gemm_bf16_4096_pair": "BF16 GEMM 4096^3 on the two-SM kernel (tcgen05 cta_group::2)",
    "gemm_bf16_few_tiles": "BF16 GEMM 1024x384x4096: 24 tiles cut into K slices, partial tiles added by a second kernel (the default for such shapes)",
}


def run_case(args):
    """One operator case, a few launches, one JSON line: small enough for an ncu capture."""
    import torch

    import kernel_optimization_b200 as ko
    from kernel_optimization_b200 import native

    lib = native.lib()
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    s = lambda: torch.cuda.current_stream().cuda_stream  # noqa: E731
    name = args.case
    if name.startswith("sgemm"):
        n = int(name.split("_")[1])
        a = torch.from_numpy(ko.fill_uniform((n, n), 2, 0)).to(dev)
        b = torch.from_numpy(ko.fill_uniform((n, n), 2, 1)).to(dev)
        d = torch.empty((n, n), device=dev)
        launch = lambda: native.check(lib.ko_sgemm_f32(n, n, n, a.data_ptr(), b.data_ptr(), None, d.data_ptr(), s()), name)  # noqa: E731
        work, unit = 2.0 * n ** 3, "TFLOP/s"
    elif name.startswith("gemm_bf16"):
        M, N, K = (1024, 384, 4096) if "few_tiles" in name else (4096, 4096, 4096) if "4096" in name else (16384, 3072, 768)
        a = torch.from_numpy(ko.fill_uniform((M, K), 3, 0, dtype=2).view(np.int16)).to(dev)
        b = torch.from_numpy(ko.fill_uniform((N, K), 3, 1, dtype=2).view(np.int16)).to(dev)
        d = torch.empty((M, N), device=dev)
        if name.endswith("_pair"):
            launch = lambda: native.check(lib.ko_gemm_tc_tuned(1, 0, 0, M, N, K, a.data_ptr(), b.data_ptr(), None, d.data_ptr(), 2048, 0, s()), name)  # noqa: E731
        else:
            launch = lambda: native.check(lib.ko_gemm_bf16_f32(M, N, K, a.data_ptr(), b.data_ptr(), None, d.data_ptr(), s()), name)  # noqa: E731
        work, unit = 2.0 * M * N * K, "TFLOP/s"
    elif name in ("softmax_cluster_rows", "layernorm_cluster_rows", "softmax_reread_rows", "layernorm_reread_rows", "layernorm_c2", "softmax_c1",
                  "softmax_block_rows"):
        rows, cols, nsets = {"softmax_cluster_rows": (256, 131072, 3), "layernorm_cluster_rows": (256, 131072, 3), "softmax_block_rows": (3640, 9216, 3),
                             "softmax_reread_rows": (1024, 65536, 2), "layernorm_reread_rows": (1024, 131072, 2),
                             "layernorm_c2": (LN_ROWS, LN_COLS, 8), "softmax_c1": (SOFTMAX_ROWS, SOFTMAX_COLS, 4)}[name]
        knobs = native.RowKnobs(tier=6) if "cluster" in name else None
        host = ko.fill_normal((rows, cols), 1, 0, 0.0, 1.0)
        xs = [torch.from_numpy(host).to(dev) for _ in range(nsets)]
        ys = [torch.empty_like(xs[0]) for _ in range(nsets)]
        g = torch.from_numpy(ko.fill_uniform((cols,), 1, 1, 0.5, 1.5)).to(dev)
        b = torch.from_numpy(ko.fill_normal((cols,), 1, 2, 0.0, 0.1)).to(dev)
        turn = [0]

        def launch():
            j = turn[0] % nsets
            turn[0] += 1
            if name.startswith("softmax"):
                native.check(lib.ko_softmax_f32_tuned(xs[j].data_ptr(), ys[j].data_ptr(), rows, cols, knobs, s()), name)
            else:
                native.check(lib.ko_layernorm_f32_tuned(xs[j].data_ptr(), ys[j].data_ptr(), rows, cols, LN_EPS, g.data_ptr(), b.data_ptr(), 0,
                                                        knobs, s()), name)
        work, unit = 2.0 * rows * cols * 4, "GB/s"
    elif name == "softmax_long_rows":
        rows, cols = 2048, 32768
        xd = torch.from_numpy(ko.fill_normal((rows, cols), 0, 0, 0.0, 2.0)).to(dev)
        yd = torch.empty_like(xd)
        launch = lambda: native.check(lib.ko_softmax_f32(xd.data_ptr(), yd.data_ptr(), rows, cols, s()), name)  # noqa: E731
        work, unit = 2.0 * rows * cols * 4, "GB/s"
    elif name == "softmax_c5_shard":
        rows, cols = 196608, 512
        x = ko.fill_normal((rows, cols), 4, 0, 0.0, 2.0)
        ko.fill_causal_mask_(x, 0, 512, -1e4)
        xd = torch.from_numpy(x).to(dev)
        yd = torch.empty_like(xd)
        launch = lambda: native.check(lib.ko_softmax_f32(xd.data_ptr(), yd.data_ptr(), rows, cols, s()), name)  # noqa: E731
        work, unit = 2.0 * rows * cols * 4, "GB/s"
    else:
        rows, cols = 32768, 4096
        xd = torch.from_numpy(ko.fill_normal((rows, cols), 4, 0, dtype=2).view(np.int16)).to(dev)
        g = torch.from_numpy(ko.fill_uniform((cols,), 4, 1, 0.5, 1.5, dtype=2).view(np.int16)).to(dev)
        b = torch.from_numpy(ko.fill_normal((cols,), 4, 2, 0.0, 0.1, dtype=2).view(np.int16)).to(dev)
        yd = torch.empty_like(xd)
        launch = lambda: native.check(lib.ko_layernorm_bf16(xd.data_ptr(), yd.data_ptr(), rows, cols, LN_EPS, g.data_ptr(), b.data_ptr(), 0, s()), name)  # noqa: E731
        work, unit = 2.0 * rows * cols * 2, "GB/s"
    for _ in range(max(args.warmup, 1)):
        launch()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        launch()
    e1.record()
    torch.cuda.synchronize()
    native.check(lib.ko_poll_device_status(), "ko_poll_device_status")
    ms = e0.elapsed_time(e1) / args.steps
    scale = 1e12 if unit == "TFLOP/s" else 1e9
    emit({"case": name, "what": CASES[name], "us_per_launch": ms * 1e3, "value": work / (ms * 1e-3) / scale,
          "unit": unit, "steps": args.steps,
          "note": "row-operator cases named *_rows / *_c1 / *_c2 rotate over buffer sets larger than the L2; the others use the same buffers every launch"})


# --------------------------------------------------------------------------------------------------
# --sweep: README-style rows (percent of the copy-bandwidth peak / of the vendor library) in one command
# --------------------------------------------------------------------------------------------------
SWEEP_ROW_SHAPES = {
    # (rows, cols): the benchmark configs, the shape the reference's drivers were written for (49152 x 1024,
    # nn_operators/softmax/main.cu:78-79) and long rows for the block, reread and cluster tiers (512 rows are 3.46
    # rounds of one row per SM; 1024 and 2048 rows fill their rounds; 64 rows go to the cluster tier)
    # (9216 / 10240 / 24576 columns: between the powers of two, where a block brings exactly the threads the row needs)
    "softmax": {"f32": [(196608, 128), (49152, 1024), (196608, 512), (8192, 8192), (3640, 9216), (512, 65536), (1024, 65536),
                        (2048, 131072), (64, 131072)],
                "f16": [(196608, 128), (49152, 1024)], "bf16": [(196608, 512), (49152, 1024), (7281, 9216), (2730, 24576), (2048, 131072)]},
    "layernorm": {"f32": [(16384, 768), (49152, 1024), (8192, 4096), (3125, 10240), (4096, 20480), (512, 65536), (1024, 65536),
                          (2048, 131072), (64, 131072)],
                  "f16": [(16384, 768), (32768, 4096)], "bf16": [(16384, 768), (32768, 4096), (32768, 5120), (2048, 131072)]},
}
SWEEP_SGEMM = [512, 1024, 2048, 4096]
# (the largest case last: its seconds at the power cap would otherwise colour the entries that follow it)
SWEEP_TC = [("bf16", "f32", False, (4096, 4096, 4096)), ("f16", "f32", False, (4096, 4096, 4096)),
            ("bf16", "f32", False, (16384, 3072, 768)),
            ("bf16", "f32", True, (4096, 4096, 4096)), ("bf16", "bf16", False, (4096, 4096, 4096)),
            ("f16", "f16", False, (4096, 4096, 4096)), ("bf16", "bf16", True, (16384, 3072, 768)),
            ("bf16", "f32", False, (8192, 8192, 8192))]


def run_sweep(args):
    """Every operator over a list of shapes next to the vendor library's kernel for the same job
    (torch.softmax / layer_norm / matmul), one JSON line with all rows and a table on stderr."""
    import torch

    from kernel_optimization_b200 import native

    lib = native.lib()
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    s = lambda: torch.cuda.current_stream().cuda_stream  # noqa: E731
    torch.backends.cuda.matmul.allow_tf32 = False
    hbm_peak, tc_peak, peak_kind = measured_peaks()
    tdt = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}
    iters = max(5, min(args.steps, 30))

    def timed(fn, nsets):
        for i in range(3):
            fn(i % nsets)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(iters):
            fn(i % nsets)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters * 1e3  # us

    rows_out = []
    gen = torch.Generator(device=dev)
    gen.manual_seed(7)
    for op, by_type in SWEEP_ROW_SHAPES.items():
        for kind, shapes in by_type.items():
            for rows, cols in shapes:
                esz = 4 if kind == "f32" else 2
                nbytes = 2.0 * rows * cols * esz
                nsets = max(2, min(8, int(300e6 // nbytes) + 1))  # more distinct bytes than the 126 MB L2
                xs = [(torch.randn((rows, cols), device=dev, generator=gen) * 2).to(tdt[kind]) for _ in range(nsets)]
                ys = [torch.empty_like(xs[0]) for _ in range(nsets)]
                if op == "softmax":
                    fn = {"f32": lib.ko_softmax_f32, "f16": lib.ko_softmax_f16, "bf16": lib.ko_softmax_bf16}[kind]
                    ours = lambda i: native.check(fn(xs[i].data_ptr(), ys[i].data_ptr(), rows, cols, s()), "softmax")  # noqa: E731
                    theirs = lambda i: torch.softmax(xs[i], dim=1, out=ys[i])  # noqa: E731
                else:
                    g = (torch.rand(cols, device=dev, generator=gen) + 0.5).to(tdt[kind])
                    b = (torch.randn(cols, device=dev, generator=gen) * 0.1).to(tdt[kind])
                    fn = {"f32": lib.ko_layernorm_f32, "f16": lib.ko_layernorm_f16, "bf16": lib.ko_layernorm_bf16}[kind]
                    ours = lambda i: native.check(fn(xs[i].data_ptr(), ys[i].data_ptr(), rows, cols, 1e-5, g.data_ptr(), b.data_ptr(), 0, s()), "layernorm")  # noqa: E731
                    theirs = lambda i: torch.nn.functional.layer_norm(xs[i], (cols,), g, b, 1e-5)  # noqa: E731
                us_o, us_t = timed(ours, nsets), timed(theirs, nsets)
                gbs = nbytes / us_o / 1e3
                rows_out.append({"op": op, "dtype": kind, "shape": [rows, cols], "us": us_o, "gbs": gbs, "of_hbm_peak": gbs / hbm_peak,
                                 "library_us": us_t, "vs_library": us_t / us_o})
                del xs, ys
    for n in SWEEP_SGEMM:
        nsets = 8 if n <= 1024 else 2
        As = [torch.rand((n, n), device=dev, generator=gen) * 2 - 1 for _ in range(nsets)]
        Bs = [torch.rand((n, n), device=dev, generator=gen) * 2 - 1 for _ in range(nsets)]
        Ds = [torch.empty((n, n), device=dev) for _ in range(nsets)]
        us_o = timed(lambda i: native.check(lib.ko_sgemm_f32(n, n, n, As[i].data_ptr(), Bs[i].data_ptr(), None, Ds[i].data_ptr(), s()), "sgemm"), nsets)
        us_t = timed(lambda i: torch.matmul(As[i], Bs[i], out=Ds[i]), nsets)
        rows_out.append({"op": "sgemm", "dtype": "f32", "shape": [n, n, n], "us": us_o, "tflops": 2.0 * n ** 3 / us_o / 1e6,
                         "library_us": us_t, "vs_library": us_t / us_o})
        del As, Bs, Ds
    for kin, kout, b_row_major, (M, N, K) in SWEEP_TC:
        time.sleep(0.3)  # let the power state of the previous entry settle
        nsets = 3
        As = [(torch.rand((M, K), device=dev, generator=gen) * 2 - 1).to(tdt[kin]) for _ in range(nsets)]
        Bs = [(torch.rand((K, N) if b_row_major else (N, K), device=dev, generator=gen) * 2 - 1).to(tdt[kin]) for _ in range(nsets)]
        Ds = [torch.empty((M, N), device=dev, dtype=tdt[kout]) for _ in range(nsets)]
        fi, fo = (0 if kin == "f16" else 1), {"f32": 0, "f16": 1, "bf16": 2}[kout]
        us_o = timed(lambda i: native.check(lib.ko_gemm_tc(fi, fo, 1 if b_row_major else 0, M, N, K, As[i].data_ptr(), Bs[i].data_ptr(), None,
                                                           Ds[i].data_ptr(), s()), "gemm_tc"), nsets)
        if kout == "f32":
            theirs = lambda i: torch.mm(As[i], Bs[i] if b_row_major else Bs[i].t(), out_dtype=torch.float32)  # noqa: E731
        else:
            theirs = lambda i: torch.mm(As[i], Bs[i] if b_row_major else Bs[i].t(), out=Ds[i])  # noqa: E731
        us_t = timed(theirs, nsets)
        tf = 2.0 * M * N * K / us_o / 1e6
        rows_out.append({"op": "gemm_tc", "dtype": f"{kin}->{kout}", "b": "row-major" if b_row_major else "column-major", "shape": [M, N, K],
                         "us": us_o, "tflops": tf, "of_bf16_peak": tf / tc_peak, "library_us": us_t, "vs_library": us_t / us_o})
        del As, Bs, Ds
    native.check(lib.ko_poll_device_status(), "ko_poll_device_status")
    print(f"{'op':10s} {'dtype':10s} {'shape':22s} {'us':>9s} {'rate':>14s} {'of peak':>8s} {'library us':>11s} {'vs library':>10s}", file=sys.stderr)
    for r in rows_out:
        rate = f"{r['gbs']:.0f} GB/s" if "gbs" in r else f"{r['tflops']:.1f} TFLOP/s"
        frac = r.get("of_hbm_peak", r.get("of_bf16_peak"))
        tag = r["dtype"] + (" rowB" if r.get("b") == "row-major" else "")
        print(f"{r['op']:10s} {tag:10s} {'x'.join(map(str, r['shape'])):22s} {r['us']:9.1f} {rate:>14s} "
              f"{'' if frac is None else format(frac, '.1%'):>8s} {r['library_us']:11.1f} {r['vs_library']:10.2f}", file=sys.stderr)
    emit({"sweep": rows_out, "peaks": {"hbm_gbs": hbm_peak, "bf16_tflops": tc_peak, "source": peak_kind}, "launches_per_row": iters,
          "library": "torch.softmax / torch.nn.functional.layer_norm / torch.matmul (cuBLAS, TF32 off)",
          "l2": "row operators rotate over buffer sets larger than the 126 MB L2"})


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--skip-gemm", action="store_true", help="row operators only")
    ap.add_argument("--skip-cpu", action="store_true", help="do not time the CPU baseline")
    ap.add_argument("--skip-scaled", action="store_true", help="leave benchmark config 5 (the scaled shapes) out of the default run")
    ap.add_argument("--row-sets", type=int, default=0,
                    help="buffer sets to rotate over (0 = default 4/8); 1 keeps a profiler capture small")
    ap.add_argument("--workload", choices=["bert_base", "scaled"], default="bert_base",
                    help="bert_base: configs 1+2 per GPU, weak scaling (default); scaled: config 5 totals, strong scaling")
    ap.add_argument("--e2e-chunks", type=int, default=E2E_CHUNKS,
                    help="row chunks per host-tensor call in the end-to-end leg (copy-in / kernel / copy-out pipeline depth)")
    ap.add_argument("--sweep", action="store_true",
                    help="every operator over a list of shapes next to the vendor library (one JSON line, table on stderr)")
    ap.add_argument("--case", choices=sorted(CASES), default=None,
                    help="run a single operator case a few times instead of the benchmark (for profiler captures)")
    args = ap.parse_args()
    # stdout carries exactly one JSON line: park the real stdout and point fd 1 at stderr meanwhile, so
    # banners printed by libraries (NCCL's version line, for one) cannot end up in front of it
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    try:
        _dispatch(args)
    finally:
        sys.stdout.flush()
        os.dup2(real_stdout, 1)
        os.close(real_stdout)
    for line in _RESULT_LINES:
        print(line, flush=True)


_RESULT_LINES: list = []


def emit(line: dict) -> None:
    _RESULT_LINES.append(json.dumps(line))


def _dispatch(args):
    if args.case:
        run_case(args)
        return
    if args.sweep:
        run_sweep(args)
        return
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.workload == "scaled":
        run_scaled(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
