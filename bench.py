#!/usr/bin/env python
"""Benchmark of the state-once question path (metric: questions/sec at 64 questions per 2048-token state,
d3-turbo-shaped random-init model; whole box = all replicas).

A "step" of the headline is one cold request: capture one 2048-token state, then one ragged question pass of
64 questions (lengths uniform in [48,160]) over it, BF16. One JSON line is printed by rank 0:

  value    : K steps with token ids already resident in HBM (device-pointer C ABI, no host copies), timed with
             CUDA events on the engine stream, max over ranks.
  e2e      : the same steps through the host-buffer C ABI (dcd_capture_state + dcd_readout_state_once_batch):
             pinned H2D of ids, D2H of logits and the error word inside the timed region.
  roofline : the tcgen05 GEMM family, from CUDA-event pairs around every GEMM launch inside the timed region.
  configs  : the other workloads the metric is asked on, each on a bounded, seeded sample through the host-buffer
             C ABI: `w4a16_8states` (int4 group-128 weights, 8 states x 64 questions), `nvfp4_c8` (NVFP4, cold
             requests arriving as a Poisson stream capped at 8 in flight, through the request scheduler),
             `ragged_stress_bf16` / `ragged_stress_nvfp4` (states log-uniform in [256,16384] tokens, 1-256
             questions of 16-512 tokens, seed 7; the first states of the seeded list).

N > 1 (torchrun): independent replicas, one engine per GPU; states are routed to replicas by predicted cost
(decidra_b200.replicas), no data-path collective; NCCL is used for the barriers and the reductions of the timings.

`--impl reference` runs the REFERENCE's own CUDA kernels, FlashInfer shim and cuBLAS (oracle/ref_gpu.py replays its
engine over the binaries compiled from its sources) on the same headline workload on this GPU; when those binaries
are absent it falls back to the CPU restatement on a bounded sample, extrapolated by FLOPs, and says so.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "questions/sec (whole box) at 64 q/state, 2048-tok state"
UNIT = "questions/s"
VOCAB = 248320
# dram__bytes_read.sum + dram__bytes_write.sum of one gate/up (SwiGLU epilogue) GEMM launch, the largest of the step (K = 5120, N = 34816), from
# ncu captures of a 4-layer slice of the same model: with the cold request in one pass the launch has M = 8883 rows (state + questions;
# algorithmic bytes 2*(M*K + N*K + M*N/2) = 756.8 MB), in the two-pass order the question pass's launch has M = 6835 (664.5 MB). The weight
# panel comes from DRAM once per group of 16 M tiles, about four to five times.
GEMM_TRAFFIC_BYTES = {"one_pass": 2180447136, "two_pass": 1747872224}


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=64)
    ap.add_argument("--state-len", type=int, default=2048)
    ap.add_argument("--questions", type=int, default=64)
    ap.add_argument("--qmin", type=int, default=48)
    ap.add_argument("--qmax", type=int, default=160)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--configs", default="all",
                    help="comma list of extra workloads in the line: w4a16,nvfp4,ragged_bf16,ragged_nvfp4 | all | none")
    ap.add_argument("--ragged-states", type=int, default=6, help="states of the seeded ragged-stress list per replica")
    ap.add_argument("--c8-states", type=int, default=24, help="cold requests of the Poisson c8 run per replica")
    ap.add_argument("--two-pass", action="store_true",
                    help="serve a cold request as the reference does, capture then question pass, instead of the one-pass call "
                         "(dcd_capture_and_readout: same bits, the weights stream once per layer for the whole request)")
    ap.add_argument("--box-states", type=int, default=96,
                    help="cold requests of the whole-box run (one process, one engine per GPU behind one router); runs on rank 0 when more than "
                         "one GPU is used, or when --box-replicas is given; 0 = skip")
    ap.add_argument("--box-replicas", type=int, default=0, help="single-GPU runs: this many engines on the one GPU behind the router (a functional check)")
    ap.add_argument("--box-precision", default="nvfp4", choices=["bf16", "fp8", "w4a16", "nvfp4"])
    ap.add_argument("--scheduler-clients", type=int, default=0,
                    help="extra arm: N client threads submit cold requests (a new state each) through the request scheduler; "
                         "adds a 'scheduler' object to the JSON line (not part of the default run)")
    ap.add_argument("--scheduler-warm", action="store_true",
                    help="with --scheduler-clients: every client keeps asking about its own state, captured once before the timed region "
                         "(device-tier hits), as in the reference's published warm-state numbers")
    ap.add_argument("--scheduler-cross-state", action="store_true",
                    help="with --scheduler-clients: let the groups of one coalesced batch share a question pass")
    ap.add_argument("--precision", default="bf16", choices=["bf16", "fp8", "w4a16", "nvfp4"],
                    help="precision of the headline arm; bf16 is the configuration the metric is quoted on")
    return ap.parse_args()


PRECISION_CODE = {"bf16": 0, "w4a16": 1, "fp8": 2, "nvfp4": 3}
PEAK_RATIO = {"bf16": 1.0, "w4a16": 1.0, "fp8": 2.0, "nvfp4": 4.0}
KERNEL_NAME = {"bf16": "gemm_bf16_tc_kernel (tcgen05 kind::f16, all projection/MLP GEMMs)",
               "w4a16": "gemm_w4a16_tc_kernel / gemm_bf16_tc_kernel (tcgen05 kind::f16 on int4 group-128 weights)",
               "fp8": "gemm_bf16_tc_kernel<.,1> (tcgen05 kind::f8f6f4, e4m3 operands; capture pass in bf16)",
               "nvfp4": "gemm_nvfp4_tc_kernel (tcgen05 kind::mxf4nvf4 block-scaled)"}


def headline_workload(args, index):
    """State + questions of global request `index` (seeded; the same request whatever replica serves it)."""
    rng = np.random.Generator(np.random.PCG64(1000 + index))
    state = rng.integers(0, VOCAB, args.state_len, dtype=np.uint32)
    lens = rng.integers(args.qmin, args.qmax + 1, args.questions)
    questions = [rng.integers(0, VOCAB, int(n), dtype=np.uint32) for n in lens]
    return state, questions


def ragged_list(n_states):
    """First n states of the seeded ragged-stress list: S ~ logU[256,16384], 1-256 questions, lengths U[16,512], seed 7."""
    rng = np.random.Generator(np.random.PCG64(7))
    S = np.exp(rng.uniform(np.log(256), np.log(16384), 2048)).astype(np.int64)
    B = rng.integers(1, 257, 2048)
    out = []
    for i in range(n_states):
        r = np.random.Generator(np.random.PCG64(7000 + i))
        lens = r.integers(16, 513, int(B[i]))
        out.append((int(S[i]), [int(x) for x in lens], i))
    return out


def ragged_tokens(S, lens, i):
    r = np.random.Generator(np.random.PCG64(70000 + i))
    return r.integers(0, VOCAB, S, dtype=np.uint32), [r.integers(0, VOCAB, n, dtype=np.uint32) for n in lens]


def config_dict(args, n_gpus):
    return {
        "workload": ("d3-turbo-shaped BF16 random-init" if args.precision == "bf16" else "d3-turbo-shaped, %s weights/GEMMs (not the headline precision)" % args.precision)
                    + ": %d layers 3 GDN:1 full-attn, hidden 5120, 1 state x %d tokens + %d questions len U[%d,%d] per step (cold: capture + question pass)"
                    % (args.layers, args.state_len, args.questions, args.qmin, args.qmax),
        "parallelism": "replicas sharded by state (dp%d), no collective on the data path" % n_gpus,
        "l2": "inputs larger than L2: 48.7 GB of weights are streamed from HBM every step",
        "seed": 0,
        "cold_request": "capture then question pass (two passes)" if getattr(args, "two_pass", False) or args.precision == "fp8"
                        else "state and questions in one pass over the layers (dcd_capture_and_readout; bit-identical to capture + question pass)",
    }


def peak_tflops(precision):
    peaks_path = ROOT / "MEASURED_PEAKS.json"
    if peaks_path.exists():
        peak = float(json.loads(peaks_path.read_text())["bf16_tflops_sustained"])
        src = "measured (MEASURED_PEAKS.json bf16_tflops_sustained: cuBLAS bf16 GEMM loop under the power cap)"
    else:
        peak, src = 1400.0, "fallback (earlier sustained measurement on this pool)"
    ratio = PEAK_RATIO[precision]
    if ratio != 1.0:  # no measured fp8 / fp4 tensor figure exists for this pool
        peak *= ratio
        src += " x %g (nominal dense %s : bf16 ratio; no measured %s figure on this pool)" % (ratio, precision, precision)
    return peak, src


# ---------------------------------------------------------------------------------------------------
# CPU baseline: the CPU restatement on a bounded sample, extrapolated by algorithmic FLOPs
# ---------------------------------------------------------------------------------------------------
def cpu_sample(args, steps=1, warmup=0):
    """Times the CPU restatement on a 2-layer [GDN, full] slice at d3 dimensions (64-token state + 4 questions
    of 48 tokens) with every host thread and scales to the full job by FLOPs. Returns (questions/s, cores, description, times)."""
    os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)  # torchrun exports OMP_NUM_THREADS=1
    sys.path.insert(0, str(ROOT / "tests"))
    from conftest import orc_cfg
    from decidra_b200.config import d3_config
    from oracle import cpu_oracle as O

    small = d3_config(num_layers=2, dtype=1, vocab=4096)
    small.layer_is_full[0], small.layer_is_full[1] = 0, 1
    full = d3_config(num_layers=args.layers, dtype=1)
    rng = np.random.Generator(np.random.PCG64(5))
    S, qlens = 64, [48, 48, 48, 48]
    state = rng.integers(0, 4096, S, dtype=np.uint32)
    qs = [rng.integers(0, 4096, n, dtype=np.uint32) for n in qlens]
    orc = O.Oracle(orc_cfg(O, small), 0)
    f_sample = small.capture_flops(S) + sum(small.question_flops(n, S) for n in qlens)
    mean_len = (args.qmin + args.qmax) / 2.0
    f_full = full.capture_flops(args.state_len) + args.questions * full.question_flops(mean_len, args.state_len)
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        st = orc.capture_state(state)
        orc.readout_state_once_batch(st, qs)
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
    t = statistics.median(times)
    qps = args.questions / (t * f_full / f_sample)
    desc = ("CPU restatement (oracle/, bf16-rounding mode, %d threads) on a 2-layer [GDN,full] slice at d3 dimensions, 64-token state + "
            "4 questions x 48 tokens = %.0f GFLOP in %.2f s (%.1f GFLOP/s); extrapolated by FLOPs x%.0f to the full step"
            % (O.num_threads(), f_sample / 1e9, t, f_sample / 1e9 / t, f_full / f_sample))
    return qps, O.num_threads(), desc, times


def reference_unavailable_reason():
    try:
        import torch
        if not torch.cuda.is_available():
            return "no CUDA device"
    except Exception as ex:  # noqa: BLE001
        return "torch unavailable: %r" % (ex,)
    from oracle import ref_gpu
    if not ref_gpu.available():
        return "oracle/_ref (the reference's kernels and FlashInfer shim compiled for sm_100a) is not built"
    return None


def run_reference(args):
    """Reference arm. Preferred: the reference's own CUDA code on this GPU (full 64-layer model, the headline workload).
    Fallback: the CPU restatement on a bounded sample."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    why_not = reference_unavailable_reason()
    base = {"impl": "reference", "metric": METRIC, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": config_dict(args, args.gpus)}
    if why_not is None:
        import torch
        from decidra_b200.config import d3_config
        from oracle import ref_gpu
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        cfg = d3_config(num_layers=args.layers, dtype=1)
        eng = ref_gpu.RefEngine(cfg, 0)
        times = []
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for i in range(args.warmup + args.steps):
            state, questions = headline_workload(args, i)
            torch.cuda.synchronize()
            ev0.record()
            st = eng.capture_state(state)
            logits = eng.readout_state_once_batch(st, questions)  # ends with a device-to-host copy of the logits
            ev1.record()
            torch.cuda.synchronize()
            if i >= args.warmup:
                times.append(ev0.elapsed_time(ev1) * 1e-3)
            del st
        t = sum(times) / len(times)
        qps = args.questions / t
        sample = ("the reference's own kernels.cu + FlashInfer FA2 shim compiled for sm_100a + cuBLAS (torch.matmul), its engine's launch "
                  "sequence replayed by a Python host on ONE B200 (the reference has no multi-GPU mode); full %d-layer model, every step a cold "
                  "request (capture %d tokens + %d questions), %d kernel launches + %d FlashInfer calls per step; logits finite: %s"
                  % (args.layers, args.state_len, args.questions, eng.k.launches // (args.warmup + args.steps), eng.fi.calls // (args.warmup + args.steps),
                     bool(np.isfinite(logits).all())))
        line = dict(base, value=qps, ms_per_step=t * 1e3,
                    cpu_baseline={"value": qps, "unit": UNIT, "cores": 1, "kind": "reference", "sample": sample},
                    e2e={"value": qps, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                    gpu_launches=0, reference_on="gpu")
        print(json.dumps(line), flush=True)
        return
    qps, cores, desc, times = cpu_sample(args, steps=args.steps, warmup=args.warmup)
    t = statistics.median(times)
    line = dict(base, value=qps, ms_per_step=t * 1e3,
                cpu_baseline={"value": qps, "unit": UNIT, "cores": cores, "kind": "port", "sample": desc + " (reference kernels not used: %s)" % why_not},
                e2e={"value": qps, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, gpu_launches=0, reference_on="cpu")
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.proc = None
        self.index = index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in out.strip().splitlines():
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------------------------------
class Ranks:
    """torch.distributed plumbing of the replicas: barriers and reductions of host scalars (never on the data path)."""

    def __init__(self):
        import torch
        self.torch = torch
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(self.local)
        self.dist = None
        if self.world > 1:
            import torch.distributed as dist
            # rank 0 prints exactly one JSON line on stdout: NCCL's version banner and anything else it logs go to stderr
            if os.environ.get("NCCL_DEBUG", "").upper() in ("VERSION", "WARN"):
                del os.environ["NCCL_DEBUG"]
            os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
            dist.init_process_group("nccl", device_id=torch.device("cuda", self.local))
            self.dist = dist
            self.host_group = dist.new_group(backend="gloo")  # barriers that must not put a kernel on any GPU

    def barrier(self):
        self.torch.cuda.synchronize()
        if self.dist:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def host_barrier(self):
        """A barrier on the host alone. An NCCL barrier is a kernel that spins on the GPUs of the ranks that arrived first; while
        rank 0 drives every GPU of the box from its own process, those kernels would hold SMs that the persistent GEMMs expect."""
        self.torch.cuda.synchronize()
        if self.dist:
            self.dist.barrier(group=self.host_group)

    def _reduce(self, x, op):
        if not self.dist:
            return float(x)
        t = self.torch.tensor([x], dtype=self.torch.float64, device="cuda")
        self.dist.all_reduce(t, op=op)
        return float(t.item())

    def max(self, x):
        return self._reduce(x, self.dist.ReduceOp.MAX) if self.dist else float(x)

    def min(self, x):
        return self._reduce(x, self.dist.ReduceOp.MIN) if self.dist else float(x)

    def sum(self, x):
        return self._reduce(x, self.dist.ReduceOp.SUM) if self.dist else float(x)

    def gather(self, x):
        """All ranks' values of one scalar, in rank order."""
        if not self.dist:
            return [float(x)]
        t = self.torch.zeros(self.world, dtype=self.torch.float64, device="cuda")
        t[self.rank] = x
        self.dist.all_reduce(t)
        return [float(v) for v in t.tolist()]

    def close(self):
        if self.dist:
            self.dist.barrier()
            self.dist.destroy_process_group()


def make_engine(dcd, args, precision, max_pass_tokens, device):
    cfg = dcd.d3_config(num_layers=args.layers, dtype=1)
    opt = dcd.Options()
    opt.max_pass_tokens = max_pass_tokens
    opt.precision = PRECISION_CODE[precision]
    eng = dcd.Engine(cfg, opt, device=device)
    eng.init_random(0)
    return eng, cfg


def gemm_roofline(prof, precision):
    g = prof["gemm"]
    achieved = g["work"] / (g["ms"] * 1e-3) / 1e12 if g["ms"] > 0 else 0.0
    peak, src = peak_tflops(precision)
    return {"kernel": KERNEL_NAME[precision], "bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
            "peak_source": src, "launches": g["launches"], "avg_launch_ms": g["ms"] / max(1, g["launches"])}


def run_requests(eng, R, requests, warm=1, two_pass=False):
    """Serve `requests` (list of (state ids, questions)) through the host-buffer C ABI, one cold request after the other
    (dcd_capture_and_readout, which takes the two-pass order by itself where one pass cannot hold the request).
    Returns a dict of whole-job figures (sums over ranks, time = max over ranks)."""
    def serve(st_ids, qs):
        if two_pass:
            st = eng.capture_state(st_ids)
            eng.readout_state_once_batch(st, qs)
        else:
            st, _ = eng.capture_and_readout(st_ids, qs)
        st.free()

    for st_ids, qs in requests[:warm]:
        serve(st_ids, qs)
    eng.sync()
    eng.profile_read()
    eng.profile_enable(True)
    R.barrier()
    lat = []
    t0 = time.perf_counter()
    for st_ids, qs in requests:
        s0 = time.perf_counter()
        serve(st_ids, qs)
        lat.append(time.perf_counter() - s0)
    eng.sync()
    t = time.perf_counter() - t0
    prof = eng.profile_read()
    eng.profile_enable(False)
    R.barrier()
    nq = sum(len(qs) for _, qs in requests)
    qtok = sum(sum(len(q) for q in qs) for _, qs in requests)
    stok = sum(len(s) for s, _ in requests)
    tmax = R.max(t)
    out = {"value": R.sum(nq) / tmax, "unit": UNIT, "states_per_s": R.sum(len(requests)) / tmax, "seconds": tmax,
           "states": int(R.sum(len(requests))), "questions": int(R.sum(nq)), "question_tokens": int(R.sum(qtok)), "state_tokens": int(R.sum(stok)),
           "p50_request_latency_ms": statistics.median(lat) * 1e3 if lat else None,
           "rank_seconds_min_median_max": None,
           "kernel_time_share_ms": {k: v["ms"] for k, v in prof.items()},
           "timed": "host-buffer C ABI (H2D of ids, D2H of logits inside), wall clock between barriers, max over ranks"}
    ts = sorted(R.gather(t))
    out["rank_seconds_min_median_max"] = [ts[0], ts[len(ts) // 2], ts[-1]]
    return out, prof


def run_poisson_c8(eng, R, args, n_requests, precision):
    """Cold requests (a new 2048-token state + 64 questions each) arriving as a Poisson stream whose in-flight count is capped
    at 8, served through the request scheduler (one worker thread owns the engine). The arrival rate is twice the
    service rate measured on the first requests, so the replica stays saturated; latency is admission to reply."""
    from decidra_b200 import scheduler
    handle = scheduler.BatchHandle(eng, state_cache_entries=0, cold_one_pass=0 if args.two_pass else 1)
    reqs = [headline_workload(args, 500000 + R.rank * 100000 + i) for i in range(n_requests + 2)]
    t0 = time.perf_counter()
    for s, q in reqs[:2]:
        handle.submit_state_once(s, q).result()
    service = (time.perf_counter() - t0) / 2
    rng = np.random.Generator(np.random.PCG64(8000 + R.rank))
    gaps = rng.exponential(service / 2.0, n_requests)
    sem = threading.Semaphore(8)
    lat, errs, threads = [], [], []

    def waiter(ticket, t_in):
        try:
            ticket.result()
            lat.append(time.perf_counter() - t_in)
        except Exception as ex:  # noqa: BLE001
            errs.append(repr(ex))
        finally:
            sem.release()

    R.barrier()
    t0 = time.perf_counter()
    for i in range(n_requests):
        time.sleep(float(gaps[i]))
        sem.acquire()
        s, q = reqs[2 + i]
        t_in = time.perf_counter()
        th = threading.Thread(target=waiter, args=(handle.submit_state_once(s, q), t_in))
        th.start()
        threads.append(th)
    for th in threads:
        th.join()
    t = time.perf_counter() - t0
    stats = handle.stats()
    handle.close()
    R.barrier()
    tmax = R.max(t)
    lat.sort()
    nq = n_requests * args.questions
    return {"value": R.sum(nq) / tmax, "unit": UNIT, "states_per_s": R.sum(n_requests) / tmax, "seconds": tmax, "states": int(R.sum(n_requests)),
            "questions": int(R.sum(nq)), "concurrency_cap": 8, "arrivals": "Poisson, mean gap = half the measured service time (%.0f ms)" % (service * 500),
            "p50_request_latency_ms": lat[len(lat) // 2] * 1e3 if lat else None, "p99_request_latency_ms": lat[min(len(lat) - 1, int(len(lat) * 0.99))] * 1e3 if lat else None,
            "captures": stats["captures"], "errors": errs,
            "sample": "%d cold requests per replica of the 512-state workload (bounded so the default run ends in minutes)" % n_requests,
            "timed": "request scheduler over the host-buffer C ABI, wall clock, max over ranks"}


def run_box(dcd, args, devices, precision, n_states):
    """One process, one engine and one request scheduler per device, one router in front (decidra_b200.box): cold requests (a new
    2048-token state + 64 questions each) arrive as a Poisson stream with at most 8 in flight in the whole box; a cold state goes
    to the replica with the fewest requests in flight. Wall clock from the first arrival to the last reply; latency is admission to
    reply. No process group is involved: the other ranks' processes hold no engine while this runs."""
    from decidra_b200 import box, scheduler
    n = len(devices)
    tm = args.state_len + args.questions * args.qmax   # room for a cold request in one pass
    engines, errs = [None] * n, []

    def mk(i):
        try:
            engines[i] = make_engine(dcd, args, precision, tm, devices[i])[0]
        except Exception as ex:  # noqa: BLE001
            errs.append("replica %d: %r" % (i, ex))

    t_setup = time.perf_counter()
    ths = [threading.Thread(target=mk, args=(i,)) for i in range(n)]
    [t.start() for t in ths]
    [t.join() for t in ths]
    if errs:
        for e in engines:
            if e is not None:
                e.close()
        return {"error": "; ".join(errs)}
    handles = [scheduler.BatchHandle(e, state_cache_entries=0, cold_one_pass=0 if args.two_pass else 1) for e in engines]
    b = box.BoxRunner(handles)
    t_setup = time.perf_counter() - t_setup
    reqs = [headline_workload(args, 900000 + i) for i in range(2 * n_states + 2 * n)]
    # two requests per replica, all replicas at once: warm-up, and the service time of one request while the whole box is busy
    t0 = time.perf_counter()
    for rnd in range(2):
        ts = [handles[i].submit_state_once(*reqs[rnd * n + i]) for i in range(n)]
        [t.result() for t in ts]
    service = (time.perf_counter() - t0) / 2
    def poisson(cap, first, seed):
        rng = np.random.Generator(np.random.PCG64(seed))
        gaps = rng.exponential(service / n / 2.0, n_states)
        sem = threading.Semaphore(cap)
        lat, failures, threads = [], [], []

        def waiter(ticket, t_in):
            try:
                ticket.result()
                lat.append(time.perf_counter() - t_in)
            except Exception as ex:  # noqa: BLE001
                failures.append(repr(ex))
            finally:
                sem.release()

        t0 = time.perf_counter()
        for i in range(n_states):
            time.sleep(float(gaps[i]))
            sem.acquire()
            s, q = reqs[first + i]
            t_in = time.perf_counter()
            th = threading.Thread(target=waiter, args=(b.submit_state_once(s, q), t_in))
            th.start()
            threads.append(th)
        for th in threads:
            th.join()
        t = time.perf_counter() - t0
        lat.sort()
        return {"value": n_states * args.questions / t, "unit": UNIT, "states_per_s": n_states / t, "seconds": t, "concurrency_cap": cap,
                "p50_request_latency_ms": lat[len(lat) // 2] * 1e3 if lat else None,
                "p99_request_latency_ms": lat[min(len(lat) - 1, int(len(lat) * 0.99))] * 1e3 if lat else None, "errors": failures}

    c8 = poisson(8, 2 * n, 8800)                                   # the workload as worded: 8 requests in flight in the whole box
    full = poisson(8 * n, 2 * n + n_states, 8801) if n > 1 else None  # 8 per replica, as each one-GPU process of `nvfp4_c8` has: no replica waits for an arrival
    t, lat_p50, lat_p99, failures = c8["seconds"], c8["p50_request_latency_ms"], c8["p99_request_latency_ms"], c8["errors"]
    st = b.stats()
    b.close()
    for e in engines:
        e.close()
    out = {"value": n_states * args.questions / t, "unit": UNIT, "states_per_s": n_states / t, "seconds": t, "states": n_states,
           "questions": n_states * args.questions, "replicas": n, "devices": list(devices), "precision": precision, "concurrency_cap": 8,
           "arrivals": "Poisson, mean gap = half the box's measured service time per request (%.0f ms per request and replica)" % (service * 1e3),
           "p50_request_latency_ms": lat_p50, "p99_request_latency_ms": lat_p99,
           "requests_per_replica": st["requests"], "stolen_per_replica": st["steals"], "captures": sum(x["captures"] for x in st["schedulers"]),
           "errors": failures, "engine_setup_s": t_setup,
           "sample": "%d cold requests of the 512-state workload per arrival stream (bounded so the default run ends in minutes)" % n_states,
           "timed": "router + request schedulers over the host-buffer C ABI, one process, wall clock; no max over ranks: a replica "
                    "that finishes early takes the next cold state"}
    if full is not None:
        out["eight_in_flight_per_replica"] = full
    return out


def run_ours(args):
    import torch

    import decidra_b200 as dcd
    from decidra_b200 import replicas

    R = Ranks()
    rank, world, local = R.rank, R.world, R.local
    want = {"w4a16", "nvfp4", "ragged_bf16", "ragged_nvfp4"} if args.configs == "all" else set(c for c in args.configs.split(",") if c and c != "none")
    need_ragged_bf16 = "ragged_bf16" in want and args.precision == "bf16"
    tm = max(args.state_len, args.questions * args.qmax)
    if not args.two_pass:  # room for the state and its questions in one pass
        tm = args.state_len + args.questions * args.qmax
    if need_ragged_bf16:
        tm = max(tm, 16384)
    if args.scheduler_cross_state:  # room for one pass over the requests of all clients
        tm = max(tm, min(16384, args.scheduler_clients * args.questions * args.qmax))
    eng, cfg = make_engine(dcd, args, args.precision, tm, local)

    # K * world global requests, routed to replicas by predicted cost (equal here: every replica serves K of them)
    n_req = args.warmup + args.steps
    costs = np.ones(n_req * world)
    mine = replicas.shard_states(costs, world, rank)
    reqs = [headline_workload(args, int(i)) for i in mine]
    dev = []
    B, S = args.questions, args.state_len
    one_pass = not args.two_pass and args.precision != "fp8" and S + args.questions * args.qmax <= tm
    for state, questions in reqs:
        lens = np.array([len(q) for q in questions], dtype=np.int32)
        flat = np.concatenate(questions)
        if one_pass:  # the state is the first sequence of the packed batch
            lens = np.concatenate([[S], lens]).astype(np.int32)
            flat = np.concatenate([state, flat])
        dev.append((torch.from_numpy(state.astype(np.int64)).to(torch.int32).cuda(),  # same 32-bit patterns as uint32 ids
                    torch.from_numpy(flat.astype(np.int64)).to(torch.int32).cuda(), torch.from_numpy(lens).cuda(), int(lens.sum()),
                    int(lens[1:].max() if one_pass else lens.max())))
    d_out_all = torch.empty((B + 1) * cfg.readout_rows, dtype=torch.float32, device="cuda")
    d_out = d_out_all[cfg.readout_rows:] if one_pass else d_out_all[:B * cfg.readout_rows]   # one pass: row 0 is the state's own last token

    def step_device(i):
        d_state, d_flat, d_lens, total, max_len = dev[i]
        if one_pass:
            st = eng.capture_and_readout_device(d_flat.data_ptr(), d_lens.data_ptr(), S, B, total, max_len, d_out_all.data_ptr())
        else:
            st = eng.capture_state_device(d_state.data_ptr(), S)
            eng.readout_state_once_device(st, d_flat.data_ptr(), d_lens.data_ptr(), B, total, max_len, d_out.data_ptr())
        st.free()

    def step_host(i):
        if one_pass:
            st, out = eng.capture_and_readout(reqs[i][0], reqs[i][1])
        else:
            st = eng.capture_state(reqs[i][0])
            out = eng.readout_state_once_batch(st, reqs[i][1])
        st.free()
        return out

    # ---- device-resident arm ------------------------------------------------------------------------
    for i in range(args.warmup):
        step_device(i)
    eng.sync()
    eng.profile_read()
    eng.profile_enable(True)
    launches0 = eng.launch_count()
    clocks = ClockSampler(local)
    R.barrier()
    clocks.start()
    eng.timer_begin()
    for i in range(args.warmup, n_req):
        step_device(i)
    eng.timer_end()
    t_dev_local = eng.timer_seconds()
    R.barrier()
    clock_info = clocks.stop()
    launches = eng.launch_count() - launches0
    prof = eng.profile_read()
    eng.profile_enable(False)
    t_dev = R.max(t_dev_local)
    rank_ms = sorted(v / args.steps * 1e3 for v in R.gather(t_dev_local))
    logits_dev = d_out.cpu().numpy().reshape(B, cfg.readout_rows)

    # ---- end-to-end arm (host buffers through the public C ABI) ----------------------------------------
    for i in range(max(1, args.warmup // 2)):
        step_host(i)
    R.barrier()
    lat = []
    t0 = time.perf_counter()
    for i in range(args.warmup, n_req):
        s0 = time.perf_counter()
        logits_host = step_host(i)
        lat.append(time.perf_counter() - s0)
    eng.sync()
    t_e2e = time.perf_counter() - t0
    R.barrier()
    t_e2e = R.max(t_e2e)
    same = bool(np.array_equal(logits_host, logits_dev))
    total_last = dev[-1][3] - (S if one_pass else 0)
    flops_step = sum(cfg.capture_flops(S) + sum(cfg.question_flops(len(q), S) for q in qs) for _, qs in reqs[args.warmup:]) / args.steps

    # ---- optional: the same cold requests through the request scheduler, from concurrent clients ----------------------
    sched_info = None
    if args.scheduler_clients > 0 and world == 1:
        from decidra_b200 import scheduler
        nc = args.scheduler_clients
        questions = reqs[0][1]
        per_client = []
        for c in range(nc):
            r = np.random.Generator(np.random.PCG64(5000 + c))
            if args.scheduler_warm:
                own = r.integers(0, VOCAB, S, dtype=np.uint32)
                per_client.append([own] * args.steps)
            else:
                per_client.append([r.integers(0, VOCAB, S, dtype=np.uint32) for _ in range(args.steps)])  # a new state per request
        if args.scheduler_warm:   # every client's state fits the device tier and is captured before the clock starts
            handle = scheduler.BatchHandle(eng, state_cache_entries=max(16, nc), state_cache_bytes=64 << 30,
                                           cross_state_pass=int(args.scheduler_cross_state))
            for c in range(nc):
                handle.submit_state_once(per_client[c][0], questions).result()
        else:
            handle = scheduler.BatchHandle(eng, state_cache_entries=0, cross_state_pass=int(args.scheduler_cross_state))   # every request is cold
            handle.submit_state_once(reqs[0][0], questions).result()          # warm
        lat_s, errs = [], []

        def client(c):
            try:
                for st_ids in per_client[c]:
                    t = time.perf_counter()
                    handle.submit_state_once(st_ids, questions).result()
                    lat_s.append(time.perf_counter() - t)
            except Exception as ex:  # noqa: BLE001
                errs.append(repr(ex))

        threads = [threading.Thread(target=client, args=(c,)) for c in range(nc)]
        t0 = time.perf_counter()
        for th in threads:
            th.start()
        for th in threads:
            th.join()
        t_s = time.perf_counter() - t0
        stats = handle.stats()
        handle.close()
        sched_info = {"value": nc * args.steps * B / t_s, "unit": UNIT, "clients": nc, "requests": nc * args.steps,
                      "p50_request_latency_ms": statistics.median(lat_s) * 1e3 if lat_s else None,
                      "max_request_latency_ms": max(lat_s) * 1e3 if lat_s else None, "errors": errs,
                      "captures": stats["captures"], "groups": stats["groups_success"], "questions_answered": stats["questions_answered"],
                      "warm_states": bool(args.scheduler_warm), "cross_state_passes": stats["cross_state_passes"],
                      "gpu_hits": stats["requests_gpu_hit"], "requests_fallback": stats["requests_fallback"]}

    # ---- the other workloads of the metric, each on a bounded seeded sample ---------------------------------------------
    configs = {}

    def ragged_requests():
        n = args.ragged_states * world
        lst = ragged_list(n)
        cost = [cfg.capture_flops(S_) + sum(cfg.question_flops(l, S_) for l in lens_) for S_, lens_, _ in lst]
        own = replicas.shard_states(cost, world, rank)
        return [ragged_tokens(*lst[int(i)]) for i in own], n

    def add_roofline(obj, prof_, precision):
        obj["roofline"] = gemm_roofline(prof_, precision)
        return obj

    if need_ragged_bf16:
        rq, n = ragged_requests()
        obj, p = run_requests(eng, R, rq, warm=1, two_pass=args.two_pass)
        obj["sample"] = "first %d states of the seeded 2048-state list (S ~ logU[256,16384], 1-256 questions of 16-512 tokens, seed 7), routed to replicas by predicted FLOPs" % n
        configs["ragged_stress_bf16"] = add_roofline(obj, p, "bf16")
    eng.close()
    del eng

    if "w4a16" in want and args.precision == "bf16":
        e2, _ = make_engine(dcd, args, "w4a16", tm, local)
        own = replicas.shard_states(np.ones(8), world, rank)       # 8 states in all, whatever the number of replicas
        rq = [headline_workload(args, 200000 + int(i)) for i in own]
        obj, p = run_requests(e2, R, rq, warm=1, two_pass=args.two_pass)                   # a replica without a state idles but joins the barriers and reductions
        obj["sample"] = "8 states x (2048 tokens + 64 questions of 48-160 tokens) in all, int4 group-128 weights with fp16 scales"
        configs["w4a16_8states"] = add_roofline(obj, p, "w4a16")
        e2.close()
        del e2

    if ("nvfp4" in want or "ragged_nvfp4" in want) and args.precision == "bf16":
        e3, _ = make_engine(dcd, args, "nvfp4", 16384 if "ragged_nvfp4" in want else tm, local)
        if "nvfp4" in want:
            # device-timed steps first (the kernel view of this precision), then the Poisson c8 run through the scheduler
            rq = [headline_workload(args, 300000 + rank * 1000 + i) for i in range(4)]
            obj, p = run_requests(e3, R, rq, warm=1, two_pass=args.two_pass)
            c8 = run_poisson_c8(e3, R, args, args.c8_states, "nvfp4")
            c8["sequential_cold_requests"] = {k: obj[k] for k in ("value", "states_per_s", "seconds", "states", "p50_request_latency_ms", "kernel_time_share_ms")}
            configs["nvfp4_c8"] = add_roofline(c8, p, "nvfp4")
        if "ragged_nvfp4" in want:
            rq, n = ragged_requests()
            obj, p = run_requests(e3, R, rq, warm=1, two_pass=args.two_pass)
            obj["sample"] = "first %d states of the seeded 2048-state list (as ragged_stress_bf16), NVFP4 weights and activations" % n
            configs["ragged_stress_nvfp4"] = add_roofline(obj, p, "nvfp4")
        e3.close()
        del e3

    box_info = None
    if args.box_states > 0 and args.precision == "bf16" and (world > 1 or args.box_replicas > 0):
        R.barrier()  # every rank has freed its engines; rank 0 alone now drives all the GPUs from one process
        R.host_barrier()
        if rank == 0:
            try:
                box_info = run_box(dcd, args, list(range(world)) if world > 1 else [local] * args.box_replicas, args.box_precision, args.box_states)
            except Exception as ex:  # noqa: BLE001  (the line of the per-rank arms must survive a failure of this extra arm)
                box_info = {"error": repr(ex)}
        R.host_barrier()

    if rank == 0:
        roof = gemm_roofline(prof, args.precision)
        roof["traffic"] = GEMM_TRAFFIC_BYTES["one_pass" if one_pass else "two_pass"] if args.precision == "bf16" else None
        line = {
            "metric": METRIC, "value": world * B * args.steps / t_dev, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": t_dev / args.steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": {"bf16": "bf16", "fp8": "fp8 e4m3 GEMMs in the question pass (bf16 capture, bf16 activations elsewhere)",
                      "w4a16": "bf16 activations, int4 group-128 weights",
                      "nvfp4": "NVFP4 weights and activations (W4A4 semantics) on the block-scaled FP4 tensor-core GEMM (tcgen05 kind::mxf4nvf4)"}[args.precision],
            "data": "synthetic", "config": config_dict(args, world),
            "states_per_s": world * args.steps / t_dev,
            "rank_ms_per_step_min_median_max": [rank_ms[0], rank_ms[len(rank_ms) // 2], rank_ms[-1]],
            "step_tflop": flops_step / 1e12, "model_tflops_per_gpu": flops_step * args.steps / t_dev_local / 1e12,
            "e2e": {"value": world * B * args.steps / t_e2e, "unit": UNIT, "h2d_bytes_per_step": int(4 * (S + total_last + B + 1)),
                    "d2h_bytes_per_step": int(4 * B * cfg.readout_rows + 8), "p50_request_latency_ms": statistics.median(lat) * 1e3, "max_request_latency_ms": max(lat) * 1e3,
                    "logits_identical_to_device_arm": same},
            "gpu_launches": int(launches),
            "roofline": roof,
            "kernel_time_share_ms_per_step": {k: v["ms"] / args.steps for k, v in prof.items()},
            "clocks": clock_info,
            "configs": configs,
        }
        if sched_info is not None:
            line["scheduler"] = sched_info
        if box_info is not None:
            line["box"] = box_info
        if world == 1 and not args.no_cpu_baseline:
            qps, cores, desc, _ = cpu_sample(args, steps=1, warmup=0)
            line["cpu_baseline"] = {"value": qps, "unit": UNIT, "cores": cores, "kind": "port", "sample": desc}
        print(json.dumps(line), flush=True)
    R.close()


def main():
    args = parse()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
