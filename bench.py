#!/usr/bin/env python
"""Benchmark of the state-once question path (BASELINE metric: questions/sec at 64 questions per
2048-token state, d3-turbo-shaped BF16 random-init model).

A "step" is one cold request: capture one 2048-token state, then one ragged question pass of 64
questions (lengths uniform in [48,160]) over it. Three measurements per run, printed as ONE JSON line:

  value : steps with token ids already resident in HBM (device-pointer C ABI, no host copies), timed with
          CUDA events on the engine stream, max over ranks.
  e2e   : the same steps through the host-buffer C ABI (dcd_capture_state +
          dcd_readout_state_once_batch): pinned H2D of ids, D2H of logits and the error word inside the
          timed region.
  roofline : the tcgen05 GEMM, from CUDA-event pairs around every GEMM launch inside the timed region.

N > 1 (torchrun): independent replicas, one engine per GPU, each rank works on its own states (weak
scaling, no data-path collective); NCCL is used only for the barrier and the max-over-ranks of the time.

`--impl reference` times the CPU restatement of the reference's path (oracle/, all host threads) on a
bounded sample and extrapolates by FLOPs; the reference itself has no CPU implementation and its Rust
host cannot be built here.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "questions/sec (whole box) at 64 q/state, 2048-tok state"
UNIT = "questions/s"
# dram__bytes_read.sum + dram__bytes_write.sum of one gate/up (SwiGLU epilogue) launch at M = 2048, the
# largest GEMM of the step, from the ncu capture summarised in profiles/gemm_bf16_tc_d3_4layer.md
# (algorithmic bytes of that launch: 448.8 MB).
GEMM_TRAFFIC_BYTES = 443.2e6


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
    ap.add_argument("--scheduler-clients", type=int, default=0,
                    help="extra arm: N client threads submit cold requests (a new state each) through the request scheduler; "
                         "adds a 'scheduler' object to the JSON line (not part of the default run)")
    ap.add_argument("--scheduler-warm", action="store_true",
                    help="with --scheduler-clients: every client keeps asking about its own state, captured once before the timed region "
                         "(device-tier hits), as in the reference's published warm-state numbers")
    ap.add_argument("--scheduler-cross-state", action="store_true",
                    help="with --scheduler-clients: let the groups of one coalesced batch share a question pass")
    ap.add_argument("--precision", default="bf16", choices=["bf16", "fp8", "w4a16", "nvfp4"],
                    help="bf16 = BASELINE configs[1] (the headline); fp8 = e4m3 GEMMs in the question pass (extra, not the headline)")
    return ap.parse_args()


def workload(args, rank):
    rng = np.random.Generator(np.random.PCG64(1000 + rank))
    vocab = 248320
    state = rng.integers(0, vocab, args.state_len, dtype=np.uint32)
    lens = rng.integers(args.qmin, args.qmax + 1, args.questions)
    questions = [rng.integers(0, vocab, int(n), dtype=np.uint32) for n in lens]
    return state, questions


def config_dict(args, n_gpus):
    return {
        "workload": ("d3-turbo-shaped BF16 random-init (BASELINE configs[1])" if args.precision == "bf16" else "d3-turbo-shaped, %s weights/GEMMs (not the headline config)" % args.precision) + ": %d layers 3 GDN:1 full-attn, hidden 5120, "
                    "1 state x %d tokens + %d questions len U[%d,%d] per step (cold: capture + question pass)"
                    % (args.layers, args.state_len, args.questions, args.qmin, args.qmax),
        "parallelism": "replicas sharded by state (dp%d), no collective on the data path" % n_gpus,
        "l2": "inputs larger than L2: 48.7 GB of weights are streamed from HBM every step",
        "seed": 0,
    }


# ---------------------------------------------------------------------------------------------------
# CPU baseline: the oracle on a bounded sample, extrapolated by algorithmic FLOPs
# ---------------------------------------------------------------------------------------------------
def cpu_sample(args, steps=1, warmup=0):
    """Times the CPU oracle on a 2-layer [GDN, full] slice at d3 dimensions (64-token state + 4 questions
    of 48 tokens) and scales to the full job by FLOPs. Returns (questions/s, cores, description, times)."""
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
    desc = ("CPU restatement (oracle/, bf16-rounding mode) on a 2-layer [GDN,full] slice at d3 dimensions, 64-token state + "
            "4 questions x 48 tokens = %.0f GFLOP in %.2f s (%.1f GFLOP/s); extrapolated by FLOPs x%.0f to the full step"
            % (f_sample / 1e9, t, f_sample / 1e9 / t, f_full / f_sample))
    return qps, O.num_threads(), desc, times


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    qps, cores, desc, times = cpu_sample(args, steps=args.steps, warmup=args.warmup)
    t = statistics.median(times)
    line = {
        "impl": "reference", "metric": METRIC, "value": qps, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": config_dict(args, args.gpus),
        "cpu_baseline": {"value": qps, "unit": UNIT, "cores": cores, "kind": "port", "sample": desc},
        "e2e": {"value": qps, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
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
def run_ours(args):
    import torch

    import decidra_b200 as dcd

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        # rank 0 prints exactly one JSON line on stdout: NCCL's version banner (printed at every debug level from
        # VERSION up) and anything else it logs go to stderr
        if os.environ.get("NCCL_DEBUG", "").upper() in ("VERSION", "WARN"):
            del os.environ["NCCL_DEBUG"]
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    def barrier():
        torch.cuda.synchronize()
        if dist:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if not dist:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    cfg = dcd.d3_config(num_layers=args.layers, dtype=1)
    opt = dcd.Options()
    opt.max_pass_tokens = max(args.state_len, args.questions * args.qmax)
    if args.scheduler_cross_state:  # room for one pass over the requests of all clients
        opt.max_pass_tokens = max(opt.max_pass_tokens, min(16384, args.scheduler_clients * args.questions * args.qmax))
    opt.precision = {"bf16": 0, "w4a16": 1, "fp8": 2, "nvfp4": 3}[args.precision]
    eng = dcd.Engine(cfg, opt, device=local)
    eng.init_random(0)

    state, questions = workload(args, rank)
    lens = np.array([len(q) for q in questions], dtype=np.int32)
    flat = np.concatenate(questions)
    B, total, max_len, S = len(questions), int(lens.sum()), int(lens.max()), len(state)
    d_state = torch.from_numpy(state.astype(np.int64)).to(torch.int32).cuda()  # same 32-bit patterns as uint32 ids
    d_flat = torch.from_numpy(flat.astype(np.int64)).to(torch.int32).cuda()
    d_lens = torch.from_numpy(lens).cuda()
    d_out = torch.empty(B * cfg.readout_rows, dtype=torch.float32, device="cuda")

    def step_device():
        st = eng.capture_state_device(d_state.data_ptr(), S)
        eng.readout_state_once_device(st, d_flat.data_ptr(), d_lens.data_ptr(), B, total, max_len, d_out.data_ptr())
        st.free()

    def step_host():
        st = eng.capture_state(state)
        out = eng.readout_state_once_batch(st, questions)
        st.free()
        return out

    # ---- device-resident arm ------------------------------------------------------------------------
    for _ in range(args.warmup):
        step_device()
    eng.sync()
    eng.profile_read()
    eng.profile_enable(True)
    launches0 = eng.launch_count()
    clocks = ClockSampler(local)
    barrier()
    clocks.start()
    eng.timer_begin()
    for _ in range(args.steps):
        step_device()
    eng.timer_end()
    t_dev = eng.timer_seconds()
    barrier()
    clock_info = clocks.stop()
    launches = eng.launch_count() - launches0
    prof = eng.profile_read()
    eng.profile_enable(False)
    t_dev = max_over_ranks(t_dev)
    logits_dev = d_out.cpu().numpy().reshape(B, cfg.readout_rows)

    # ---- end-to-end arm (host buffers through the public C ABI) ----------------------------------------
    for _ in range(max(1, args.warmup // 2)):
        step_host()
    barrier()
    lat = []
    t0 = time.perf_counter()
    for _ in range(args.steps):
        s0 = time.perf_counter()
        logits_host = step_host()
        lat.append(time.perf_counter() - s0)
    eng.sync()
    t_e2e = time.perf_counter() - t0
    barrier()
    t_e2e = max_over_ranks(t_e2e)
    same = bool(np.array_equal(logits_host, logits_dev))

    # ---- optional: the same cold requests through the request scheduler, from concurrent clients ----------------------
    sched_info = None
    if args.scheduler_clients > 0 and world == 1:
        import threading
        from decidra_b200 import scheduler
        nc = args.scheduler_clients
        vocab = 248320
        per_client = []
        for c in range(nc):
            r = np.random.Generator(np.random.PCG64(5000 + c))
            if args.scheduler_warm:
                own = r.integers(0, vocab, S, dtype=np.uint32)
                per_client.append([own] * args.steps)
            else:
                per_client.append([r.integers(0, vocab, S, dtype=np.uint32) for _ in range(args.steps)])  # a new state per request
        if args.scheduler_warm:   # every client's state fits the device tier and is captured before the clock starts
            handle = scheduler.BatchHandle(eng, state_cache_entries=max(16, nc), state_cache_bytes=64 << 30,
                                           cross_state_pass=int(args.scheduler_cross_state))
            for c in range(nc):
                handle.submit_state_once(per_client[c][0], questions).result()
        else:
            handle = scheduler.BatchHandle(eng, state_cache_entries=0, cross_state_pass=int(args.scheduler_cross_state))   # every request is cold
            handle.submit_state_once(state, questions).result()          # warm
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

    if rank == 0:
        peaks_path = ROOT / "MEASURED_PEAKS.json"
        if peaks_path.exists():
            peak = float(json.loads(peaks_path.read_text())["bf16_tflops_sustained"])
            peak_src = "measured (MEASURED_PEAKS.json bf16_tflops_sustained: cuBLAS bf16 GEMM loop under the power cap)"
        else:
            peak, peak_src = 1400.0, "fallback (earlier sustained measurement on this pool)"
        # No measured fp8 / fp4 tensor figure exists for this pool: those precisions are set against the measured bf16
        # number times the nominal ratio of the dense peaks (2x, 4x), and say so.
        kernel_name = {"bf16": "gemm_bf16_tc_kernel (tcgen05, all projection/MLP GEMMs)",
                       "w4a16": "gemm_bf16_tc_kernel (tcgen05) on weights dequantised from int4 per call",
                       "fp8": "gemm_bf16_tc_kernel<.,1> (tcgen05 kind::f8f6f4, e4m3 operands; capture pass in bf16)",
                       "nvfp4": "gemm_nvfp4_tc_kernel (tcgen05 kind::mxf4nvf4 block-scaled)"}[args.precision]
        ratio = {"bf16": 1.0, "w4a16": 1.0, "fp8": 2.0, "nvfp4": 4.0}[args.precision]
        if ratio != 1.0:
            peak *= ratio
            peak_src += " x %g (nominal dense %s : bf16 ratio; no measured %s figure on this pool)" % (ratio, args.precision, args.precision)
        g = prof["gemm"]
        achieved = g["work"] / (g["ms"] * 1e-3) / 1e12 if g["ms"] > 0 else 0.0
        flops_step = cfg.capture_flops(S) + sum(cfg.question_flops(int(n), S) for n in lens)
        line = {
            "metric": METRIC, "value": world * B * args.steps / t_dev, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": t_dev / args.steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": {"bf16": "bf16", "fp8": "fp8 e4m3 GEMMs in the question pass (bf16 capture, bf16 activations elsewhere)",
                      "w4a16": "bf16 activations, int4 group-128 weights (BASELINE configs[2] format)",
                      "nvfp4": "NVFP4 weights and activations (W4A4 semantics) on the block-scaled FP4 tensor-core GEMM (tcgen05 kind::mxf4nvf4)"}[args.precision],
            "data": "synthetic", "config": config_dict(args, world),
            "states_per_s": world * args.steps / t_dev,
            "step_tflop": flops_step / 1e12, "model_tflops_per_gpu": flops_step * args.steps / t_dev / 1e12,
            "e2e": {"value": world * B * args.steps / t_e2e, "unit": UNIT, "h2d_bytes_per_step": int(4 * (S + total + B + 1)),
                    "d2h_bytes_per_step": int(4 * B * cfg.readout_rows + 8), "p50_request_latency_ms": statistics.median(lat) * 1e3, "max_request_latency_ms": max(lat) * 1e3,
                    "logits_identical_to_device_arm": same},
            "gpu_launches": int(launches),
            "roofline": {"kernel": kernel_name, "bound": "tensor", "achieved": achieved, "peak": peak,
                         "unit": "TFLOP/s", "frac": achieved / peak, "traffic": GEMM_TRAFFIC_BYTES if args.precision == "bf16" else None, "peak_source": peak_src,
                         "launches": g["launches"], "avg_launch_ms": g["ms"] / max(1, g["launches"])},
            "kernel_time_share_ms_per_step": {k: v["ms"] / args.steps for k, v in prof.items()},
            "clocks": clock_info,
        }
        if sched_info is not None:
            line["scheduler"] = sched_info
        if world == 1 and not args.no_cpu_baseline:
            qps, cores, desc, _ = cpu_sample(args, steps=1, warmup=0)
            line["cpu_baseline"] = {"value": qps, "unit": UNIT, "cores": cores, "kind": "port", "sample": desc}
        print(json.dumps(line), flush=True)
    eng.close()
    if dist:
        dist.barrier()
        dist.destroy_process_group()


def main():
    args = parse()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
