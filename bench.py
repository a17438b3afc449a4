#!/usr/bin/env python
"""Benchmark of the attention hot path.  One JSON line on stdout (rank 0).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg1|cfg2|cfg3|cfg4|cfg5|oproj|rope] [--impl reference]

Workload at N = 1 (default): BASELINE config 2, causal flash-attention prefill, B4 S4096 Hq32 Hkv8 D128,
bf16 inputs, f32 output; metric = attention TFLOP/s from the algorithmic causal FLOPs 4 B Hq D S(S+1)/2.
A "step" is one pass of the kernel over the batch.  With N > 1 (torchrun, one rank per GPU) the kv heads are split
over the ranks (strong scaling, no collective).  `value` is timed with inputs resident in HBM; `e2e` is the same metric
through the host-buffer C-ABI entry point with the copies inside the timed region.  At every N the line also carries
  decode       config 3 (paged GQA decode, kv heads split over the ranks, no collective), KV GB/s
  decode_long  config 4 (131072-key decode, KV sequence split into contiguous chunks over the ranks; the ranks' partial
               records are exchanged over peer memory and merged: the one collective of the path), KV GB/s
  oproj        (N > 1) the head-sharded output projection with the library's all-reduce
each with its own roofline, parity block against the oracle and per-rank times.  In a multi-rank run these extras run
under a deadline (EXTRAS_DEADLINE_S): should one never return, rank 0 still prints the line with the headline
measurement and the extras that finished, names the one that did not, and every rank leaves with exit code 0; the
program's NCCL communicators keep in-switch reduction (NVLS) off unless NCCL_NVLS_ENABLE is set by the caller.
stdout carries the JSON line only; progress and library chatter go to stderr.
`--workload cfg1` runs the CPU-reference configuration (f32, general kernel) with the CPU port timed in full.
`--impl reference` times the CPU restatement of the reference's attention (oracle/) on the host cores instead.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import math
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

METRIC = "attention TFLOP/s (prefill) and KV GB/s (decode) at 1/2/4/8 B200 vs roofline"
DATA = "synthetic (seeded N(0,1) rounded to bf16; random values, no weights)"
EXTRAS_DEADLINE_S = 240  # the extras of a multi-rank run take well under a minute when every collective returns


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm": d["hbm_gbs"], "tensor_burst": d["bf16_tflops"], "tensor_sustained": d["bf16_tflops_sustained"],
                "source": "measured"}
    return {"hbm": 6650.0, "tensor_burst": 1590.0, "tensor_sustained": 1400.0, "source": "fallback"}


# ------------------------------------------------------------------------------------------- workload descriptions
# The `config` object of a line depends on the workload and the number of ranks only, so that both arms print the same one.
def workload_config(name: str, world: int) -> dict:
    if name == "cfg1":
        return {"workload": "cfg1: causal attention B1 S512 Hq32 Hkv8 D64, f32 in, f32 out (the CPU-reference configuration)",
                "flops_per_step": 4.0 * 32 * 64 * 512 * 513 / 2, "sharding": f"kv heads split over {world} rank(s), no collective",
                "l2": "inputs rotate over copies; at 1.3 MB per copy the working set is L2-resident by nature"}
    if name in ("cfg2", "cfg5"):
        B, S, Hq, Hkv = (4, 4096, 32, 8) if name == "cfg2" else (1, 16384, 64, 8)
        return {"workload": f"{name}: causal flash-attention prefill B{B} S{S} Hq{Hq} Hkv{Hkv} D128, bf16 in, f32 out",
                "flops_per_step": 4.0 * B * Hq * 128 * S * (S + 1) / 2, "sharding": f"kv heads split over {world} rank(s), no collective",
                "l2": "inputs rotate over copies larger than L2 in total, so each launch reads HBM-cold data"}
    if name == "cfg3":
        return {"workload": "cfg3: paged GQA decode B64 Hq32 Hkv8 D128, 16-token pages, kv_len ~ U[1024, 8192], permuted page table",
                "sharding": f"kv heads split over {world} rank(s), no collective",
                "l2": "the KV cache rotates over copies larger than L2 in total, so each launch reads HBM-cold data"}
    if name == "cfg4":
        return {"workload": "cfg4: long-context decode B1 Hq64 Hkv8 D128, 131072 keys, 16-token pages",
                "sharding": (f"KV sequence split into {world} contiguous chunks; partial (m, l, O) records stored on every rank over "
                             "peer memory by the decode kernel and merged by log-sum-exp" if world > 1 else "one GPU holds the whole sequence"),
                "l2": "the KV cache rotates over copies larger than L2 in total, so each launch reads HBM-cold data"}
    if name == "oproj":
        return {"workload": "oproj: out = attn[B4,Hq32,S4096,D128] (read in place) x W[4096,4096]^T, bf16 in, f32 out",
                "flops_per_step": 2.0 * 4 * 4096 * 4096 * 32 * 128,
                "sharding": f"query heads split over {world} rank(s)" + (", partial sums all-reduced (NCCL behind the C ABI)" if world > 1 else ""),
                "l2": "the attention input rotates over copies"}
    if name == "rope":
        return {"workload": "rope: fused RoPE + KV-cache append, B4 Hq32 Hkv8 S4096 D128, bf16 in, bf16 pages",
                "sharding": f"heads split over {world} rank(s), no collective",
                "l2": "300 MB buffer written between timed launches; table uploads are inside the timed region"}
    raise ValueError(name)


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled every 50 ms from before the warm-up until after the timed
    region; `stop(t0, t1)` keeps the samples whose timestamp falls inside the busy window [t0, t1] (host clock)."""
    Q = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx, self.proc, self.path = gpu_index, None, f"/tmp/fusor_bench_clocks_{os.getpid()}.csv"

    def start(self):
        try:
            self.f = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50",
                                          "-i", str(self.idx)], stdout=self.f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self, t0: float, t1: float):
        import datetime
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        time.sleep(0.06)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.f.close()
        self.proc = None
        mhz, mx, reasons = [], [], set()
        for line in open(self.path):
            c = [x.strip() for x in line.split(",")]
            if len(c) < 9:
                continue
            try:
                ts = datetime.datetime.strptime(c[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                f = float(c[1])
                m = float(c[2])
            except ValueError:
                continue
            if not (t0 - 0.05 <= ts <= t1 + 0.05):
                continue
            mhz.append(f)
            mx.append(m)
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), c[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        try:
            os.remove(self.path)
        except OSError:
            pass
        if mhz:
            out.update(sm_mhz=statistics.median(mhz), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(mhz))
        out["window_s"] = round(t1 - t0, 3)
        return out


# ------------------------------------------------------------------------------------------- CPU baseline (oracle port)
def cpu_prefill_sample(w):
    """Bounded sample of a prefill workload for the CPU arm: batch 0, kv head 0 with its g query heads, every row,
    evaluated densely with a [S,S] 0/-inf mask tensor exactly as the reference CPU composite does."""
    from oracle import oracle as O
    g = w.q.shape[1] // w.k.shape[1]
    q, k, v = w.q[:1, :g], w.k[:1, :1], w.v[:1, :1]
    S = q.shape[2]
    mask = O.causal_mask(S)
    flops = 4.0 * g * q.shape[3] * S * (S + 1) / 2
    desc = (f"batch 0, kv head 0 ({g} query heads), all {S} rows, dense f32 composite with a [{S},{S}] mask tensor; causal FLOPs are "
            "counted for the dense evaluation the reference performs")
    return (lambda: O.flash_attention(q, k, v, w.scale, mask, O.MASK_QK)), flops, desc


def cpu_full_prefill(w):
    """The whole tensor through the composite, as the reference runs it (config 1)."""
    from oracle import oracle as O
    S = w.q.shape[2]
    mask = O.causal_mask(S)
    return (lambda: O.flash_attention(w.q, w.k, w.v, w.scale, mask, O.MASK_QK)), w.flops, \
        f"the full tensor, dense f32 composite with a [{S},{S}] mask tensor"


def cpu_decode_sample(w, n_seq=8):
    from oracle import oracle as O
    n_seq = min(n_seq, w.q.shape[0])
    Hkv, D = w.k_pages.shape[1], w.k_pages.shape[3]
    nbytes = float(np.sum(w.kv_len[:n_seq])) * 2 * Hkv * D * 2

    def run():
        for b in range(n_seq):
            O.flash_attention(w.q[b:b + 1], w.k_dense[b][None], w.v_dense[b][None], w.scale)
    return run, nbytes, f"first {n_seq} sequence(s), all heads, dense f32 composite on de-paged K/V"


def time_cpu(fn, steps, warmup):
    for _ in range(warmup):
        fn()
    ts = []
    for _ in range(steps):
        t0 = time.perf_counter()
        fn()
        ts.append(time.perf_counter() - t0)
    return sum(ts) / len(ts)


def reference_arm(args, rank):
    """The reference's CPU implementation of the path (oracle port; the Rust sources cannot be built here), on all the
    host cores this process may use.  Imports nothing of the product."""
    if rank != 0:
        return
    from oracle import oracle as O
    from oracle import workloads as W
    O.build()
    cores = O.use_all_cores()
    name = args.workload
    cfg = workload_config(name, args.gpus)
    if name in ("cfg1", "cfg2", "cfg5"):
        w = {"cfg1": W.cfg1, "cfg2": W.cfg2, "cfg5": W.cfg5}[name]()
        fn, work, desc = cpu_full_prefill(w) if name == "cfg1" else cpu_prefill_sample(w)
        unit, div, dtype = "TFLOP/s", 1e12, "f32"
    elif name == "oproj":
        Hq, D, N, rows = 32, 128, 4096, 256
        rng = np.random.default_rng(21)
        x = W.bf16_round(rng.standard_normal((1, Hq, rows, D)).astype(np.float32))
        wt = W.bf16_round((rng.standard_normal((N, Hq * D)) / 64).astype(np.float32))
        fn = lambda: O.out_proj(x, wt)
        work, desc = 2.0 * rows * N * Hq * D, f"{rows} of the 16384 rows, all {N} outputs (f32 transpose + matmul)"
        unit, div, dtype = "TFLOP/s", 1e12, "f32"
    elif name == "rope":
        Hq, Hkv, S, D = 32, 8, 4096, 128
        rng = np.random.default_rng(22)
        x = rng.standard_normal((1, Hq + Hkv, S, D)).astype(np.float32)
        cos, sin = O.rope_tables(D, S, 10000.0)
        fn = lambda: O.rope(x, cos, sin, 0, False)
        work, desc = float(x.nbytes * 2), "one batch entry: all 40 heads rotated, f32 (read + write bytes counted)"
        unit, div, dtype = "GB/s", 1e9, "f32"
    else:
        w = W.cfg3(B=8) if name == "cfg3" else W.cfg4(Skv=16384)
        fn, work, desc = cpu_decode_sample(w)
        if name == "cfg4":
            desc = "the first 16384 of the 131072 keys, all heads, dense f32 composite"
        unit, div, dtype = "GB/s", 1e9, "f32"
    sec = time_cpu(fn, args.steps, args.warmup)
    val = work / sec / div
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": unit, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": dtype, "data": DATA, "config": cfg,
        "cpu_baseline": {"value": val, "unit": unit, "cores": cores, "kind": "port",
                         "sample": desc + "; each step of this arm is one such sample"},
        "e2e": {"value": val, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


# ------------------------------------------------------------------------------------------- GPU arm
def t4(ptr, shape, dtype, strides=None):
    from floneum_b200 import _lib
    t = _lib.Tensor4()
    t.data, t.dtype = ptr, dtype
    acc = 1
    for i in range(3, -1, -1):
        t.shape[i] = shape[i]
        t.stride[i] = strides[i] if strides else acc
        acc *= shape[i]
    return t


def start_exit_timer(seconds, rank, stdout_fd, last_line, where=lambda: None):
    """After `seconds` the process leaves with exit code 0: rank 0 first writes the JSON line `last_line()` returns (unless
    it returns None) to `stdout_fd`.  Returns the timer; cancel() it when the guarded part has finished.  The timer thread
    runs while the main thread sits in a blocking CUDA or NCCL call (those release the interpreter lock)."""
    import threading

    def give_up():
        if rank == 0:
            line = last_line()
            if line is not None:
                os.write(stdout_fd, (json.dumps(line) + "\n").encode())
        sys.stderr.write(f"rank {rank}: ran past the deadline of {seconds} s in {where()}; leaving\n")
        sys.stderr.flush()
        os._exit(0)
    # (the other ranks leave two seconds after rank 0, so that nothing of their going can reach it before the line is out)
    t = threading.Timer(seconds if rank == 0 else seconds + 2.0, give_up)
    t.daemon = True
    t.start()
    return t


def gpu_arm(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist
    import floneum_b200 as fb
    from floneum_b200 import _lib, sharding
    from floneum_b200.cache import lse_combine
    from oracle import oracle as O  # checker + CPU baseline only
    from oracle import workloads as W
    L = _lib.load()
    torch.cuda.set_device(local_rank)
    fake_world = args.shard_of if (world == 1 and args.shard_of > 1) else 0
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # The extras run under a deadline (below): a rank may then leave with a collective of another rank still in flight,
        # which must not happen while its memory is bound to an NVLink multicast object.  In-switch reduction is therefore
        # off for this program's communicators unless the caller asks for it.
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local_rank}"))
    use_dist = world > 1
    if fake_world:
        world = fake_world  # shard sizes as in an N-rank job; no collectives, no cross-rank reductions
    stream = torch.cuda.Stream()
    dev = fb.Device.gpu(local_rank, stream.cuda_stream)
    peaks = load_peaks()
    cuda = torch.device(f"cuda:{local_rank}")
    sampler = ClockSampler(local_rank)

    def barrier():
        if use_dist:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if not use_dist:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=cuda)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def all_ranks(x: float) -> list:
        if not use_dist:
            return [x]
        t = torch.tensor([x], dtype=torch.float64, device=cuda)
        out = torch.empty(world, dtype=torch.float64, device=cuda)
        dist.all_gather_into_tensor(out, t)
        return [float(v) for v in out.cpu()]

    def bf16_dev(a):  # numpy f32 (bf16-representable) -> torch bf16 on the GPU
        return torch.from_numpy(np.ascontiguousarray(a)).to(cuda).to(torch.bfloat16)

    def bf16_pinned(a):
        return torch.from_numpy(np.ascontiguousarray(a)).to(torch.bfloat16).pin_memory()

    def settle_clocks(step, seconds=0.5):
        """Untimed steps until the GPU has been under load for `seconds` (the clocks settle under the power cap)."""
        if args.quick:
            return
        t_end = time.time() + seconds
        i = 0
        while True:
            for _ in range(16):
                step(i)
                i += 1
            torch.cuda.synchronize()
            # every rank must run the same number of steps (a step may hold a collective): the ranks agree on going on
            if max_over_ranks(t_end - time.time()) <= 0.0:
                break

    def timed(step, steps):
        """K steps back to back on the stream between two barriers; returns (total ms max over ranks, this rank's total ms,
        per-step ms of this rank)."""
        barrier()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
        ev[0].record(stream)
        for i in range(steps):
            step(i)
            ev[i + 1].record(stream)
        barrier()
        mine = ev[0].elapsed_time(ev[-1])
        return max_over_ranks(mine), mine, [ev[i].elapsed_time(ev[i + 1]) for i in range(steps)]

    # ======================================================================= prefill (cfg1 / cfg2 / cfg5)
    def run_prefill(w, name, tag=""):
        B, Hq, S, D = w.q.shape
        Hkv = w.k.shape[1]
        f32_in = not w.bf16
        q0, q1 = sharding.q_head_range(Hq, Hkv, rank, world)
        k0, k1 = sharding.kv_head_range(Hkv, rank, world)
        q, k, v = w.q[:, q0:q1], w.k[:, k0:k1], w.v[:, k0:k1]
        esz = 4 if f32_in else 2
        in_bytes = (q.size + k.size + v.size) * esz
        copies = max(1, min(64, int(np.ceil(256e6 / in_bytes))))  # rotate inputs so that the working set exceeds L2
        to_dev = (lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(cuda)) if f32_in else bf16_dev
        dt = _lib.F32 if f32_in else _lib.BF16
        dq, dk, dv = [], [], []
        for _ in range(copies):
            dq.append(to_dev(q)); dk.append(to_dev(k)); dv.append(to_dev(v))
        out = torch.empty(q.shape, dtype=torch.float32, device=cuda)
        cq = [t4(t.data_ptr(), t.shape, dt) for t in dq]
        ck = [t4(t.data_ptr(), t.shape, dt) for t in dk]
        cv = [t4(t.data_ptr(), t.shape, dt) for t in dv]
        co = t4(out.data_ptr(), out.shape, _lib.F32)

        def step(i):
            j = i % copies
            _lib.check(L.fusor_cuda_flash_attention(dev.handle, ctypes.byref(cq[j]), ctypes.byref(ck[j]), ctypes.byref(cv[j]),
                                                    ctypes.c_float(w.scale), None, _lib.MASK_CAUSAL, 0, ctypes.byref(co)), dev.handle)
        with torch.cuda.stream(stream):
            sampler.start()
            time.sleep(0.15)
            t_busy0 = time.time()
            for i in range(args.warmup):
                step(i)
            torch.cuda.synchronize()
            settle_clocks(step)
            launches0 = dev.launch_count()
            total_ms, _, per_launch_ms = timed(step, args.steps)
            clocks = sampler.stop(t_busy0, time.time())
            launches = dev.launch_count() - launches0
            dev.synchronize()
        flops_rank = 4.0 * B * (q1 - q0) * D * S * (S + 1) / 2
        flops_all = w.flops
        value = flops_all * args.steps / (total_ms * 1e-3) / 1e12
        achieved = flops_rank / (statistics.mean(per_launch_ms) * 1e-3) / 1e12
        got = out.cpu().numpy()

        # ---- e2e: host buffers through the C ABI, copies inside the timed region
        if f32_in:
            hq, hk, hv = (torch.from_numpy(np.ascontiguousarray(a)).pin_memory() for a in (q, k, v))
        else:
            hq, hk, hv = bf16_pinned(q), bf16_pinned(k), bf16_pinned(v)
        hout = torch.empty(q.shape, dtype=torch.float32).pin_memory()
        eq, ek, evv = (t4(t.data_ptr(), t.shape, dt) for t in (hq, hk, hv))
        eo = t4(hout.data_ptr(), hout.shape, _lib.F32)

        def e2e_step():
            _lib.check(L.fusor_cuda_flash_attention_host(dev.handle, ctypes.byref(eq), ctypes.byref(ek), ctypes.byref(evv),
                                                         ctypes.c_float(w.scale), None, _lib.MASK_CAUSAL, 0, ctypes.byref(eo)), dev.handle)
        e2e_steps = 1 if args.quick else max(3, min(args.steps, 10))
        with torch.cuda.stream(stream):
            for _ in range(0 if args.quick else 2):
                e2e_step()
            barrier()
            t0 = time.perf_counter()
            for _ in range(e2e_steps):
                e2e_step()
            torch.cuda.synchronize()
            e2e_s = max_over_ranks(time.perf_counter() - t0)
        e2e_val = flops_all * e2e_steps / e2e_s / 1e12
        e2e_ok = bool(np.array_equal(hout.numpy(), got))
        if f32_in:
            # the general kernel runs f32 FMAs on the CUDA cores: 2 x 128 lanes x 148 SMs x clock, against which it is
            # latency- and shared-memory-bound; the fraction says how far a CUDA-core kernel is from that bound
            peak = 2 * 128 * 148 * 1.965e9 / 1e12
            roof = {"bound": "fp32 CUDA cores (no tensor-core path for f32 tensors)", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                    "frac": achieved / peak, "traffic": None, "peak_source": "nominal: 2 flop x 128 lanes x 148 SMs x 1.965 GHz"}
        else:
            # K launches back to back after a 0.5 s busy loop run under the power cap: the sustained cuBLAS figure is the
            # denominator; the fraction of the burst figure is given beside it.
            peak = peaks["tensor_sustained"]
            roof = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                    # no figure: a profiler capture of this kernel ends with most of its f32 output still in L2, so its
                    # DRAM byte count says nothing about re-reads
                    "traffic": None,
                    "peak_source": f"{peaks['source']} (cuBLAS bf16, sustained loop under the power cap)",
                    "frac_of_burst_peak": achieved / peaks["tensor_burst"], "burst_peak": peaks["tensor_burst"],
                    "frac_of_nominal_2250": achieved / 2250.0,
                    "note": "achieved counts the V pre-pass kernel's time as well (both kernels of a step)"}
        cfg = workload_config(name, world)
        if tag:
            cfg = dict(cfg, workload=cfg["workload"] + tag, flops_per_step=flops_all)
        return {
            "value": value, "unit": "TFLOP/s", "ms_per_step": total_ms / args.steps, "gpu_launches": launches,
            "roofline": roof,
            "e2e": {"value": e2e_val, "unit": "TFLOP/s", "h2d_bytes_per_step": int(in_bytes * world),
                    "d2h_bytes_per_step": int(out.numel() * 4 * world), "matches_device_path": e2e_ok},
            "clocks": clocks, "config": cfg, "input_copies": copies,
            "_got": got, "_slice": (q, k, v),
        }

    # ======================================================================= decode (cfg3 / cfg4)
    def run_decode(w, name, chunked, tag="", with_variants=True):
        """cfg3: `w` is the whole workload, this rank takes its kv heads.  cfg4: `w` is this rank's chunk of the keys."""
        B, Hq, _, D = w.q.shape
        Hkv_all = w.k_pages.shape[1]
        if not chunked:
            k0, k1 = sharding.kv_head_range(Hkv_all, rank, world)
            q0, q1 = sharding.q_head_range(Hq, Hkv_all, rank, world)
        else:
            k0, k1, q0, q1 = 0, Hkv_all, 0, Hq
        kp, vp = np.ascontiguousarray(w.k_pages[:, k0:k1]), np.ascontiguousarray(w.v_pages[:, k0:k1])
        qn = np.ascontiguousarray(w.q[:, q0:q1])
        kv_bytes_rank = float(np.sum(w.kv_len)) * 2 * (k1 - k0) * D * 2
        copies = max(1, min(8, int(math.ceil(512e6 / kv_bytes_rank))))  # rotate so that the working set is several x L2
        caches = []
        for _ in range(copies):
            c = fb.PagedKvCache(dev, B, k1 - k0, D, kp.shape[0], w.page_table.shape[1])
            c.write_pages(0, kp, vp)
            c.set_page_table(w.page_table, w.kv_len)
            if args.decode_ctas:
                c.set_decode_ctas(args.decode_ctas)
            caches.append(c)
        dq = bf16_dev(qn)
        out = torch.empty(qn.shape, dtype=torch.float32, device=cuda)
        tq, to = fb.Tensor.from_torch(dev, dq), fb.Tensor.from_torch(dev, out)
        collective = chunked and use_dist
        exchange = None
        if collective:
            part = torch.empty((B, Hq, D + 2), dtype=torch.float32, device=cuda)
            gathered = torch.empty((world, B, Hq, D + 2), dtype=torch.float32, device=cuda)
            out3 = torch.empty((B, Hq, D), dtype=torch.float32, device=cuda)
            tpart, tgath, tout3 = (fb.Tensor.from_torch(dev, t) for t in (part, gathered, out3))
            exchange = sharding.PeerExchange(dev, rank, world, B * Hq * (D + 2))

        def step_main(i):
            c = caches[i % copies]
            if collective:
                exchange.decode(c, tq, w.scale, tout3)  # split-KV kernel, then merge + store on every rank + wait + merge
            else:
                c.decode(tq, w.scale, to)

        def step_local(i):  # this rank's chunk alone, no exchange
            caches[i % copies].decode_partial(tq, w.scale, tpart)

        def step_nccl(i):  # the same step with a library all-gather between the partial and the merge kernels
            caches[i % copies].decode_partial(tq, w.scale, tpart)
            dist.all_gather_into_tensor(gathered, part)
            lse_combine(dev, tgath, tout3)

        def measure(step):
            """Warm-up, one CUDA graph per cache copy (a decode step is launch-bound at small shard sizes), K timed steps."""
            with torch.cuda.stream(stream):
                l0 = dev.launch_count()
                step(0)
                kernels_per_step = dev.launch_count() - l0  # the library's own count of its launches in one step
                for i in range(1, max(args.warmup, copies)):
                    step(i)
                barrier()
                graphs = None
                if not args.no_graph and not args.quick:
                    try:
                        graphs = []
                        for j in range(copies):
                            g = torch.cuda.CUDAGraph()
                            with torch.cuda.graph(g, stream=stream):
                                step(j)
                            graphs.append(g)
                        for g in graphs:
                            g.replay()
                        torch.cuda.synchronize()
                    except Exception as e:  # capture is an optimisation only
                        sys.stderr.write(f"CUDA graph capture failed ({e}); timing eager launches\n")
                        graphs = None
                        torch.cuda.synchronize()
                run = (lambda i: graphs[i % copies].replay()) if graphs is not None else step
                settle_clocks(run, 0.3)
                launches0 = dev.launch_count()
                total_ms, mine_ms, per_step = timed(run, args.steps)
                launches = dev.launch_count() - launches0 if graphs is None else args.steps * kernels_per_step
                dev.synchronize()
            return total_ms / args.steps, mine_ms / args.steps, per_step, launches, graphs is not None

        sampler.start()
        t_busy0 = time.time()
        ms, ms_mine, per_step, launches, graphed = measure(step_main)
        clocks = sampler.stop(t_busy0, time.time())
        res = (out3 if collective else out).float().cpu().numpy().copy()
        bytes_rank = kv_bytes_rank + B * (q1 - q0) * D * 6 + 4 * float(np.sum((w.kv_len + 15) // 16))
        bytes_all = bytes_rank * world
        achieved = bytes_rank / (ms_mine * 1e-3) / 1e9
        r = {"value": bytes_all / (ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": ms, "gpu_launches": launches,
             "rank_ms_per_step": all_ranks(ms_mine),
             "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm"], "unit": "GB/s", "frac": achieved / peaks["hbm"],
                          # profiler capture of a scaled-down case: dram read + write = 1.02 x the algorithmic bytes
                          "traffic": bytes_rank * 1.02, "peak_source": f"{peaks['source']} (device copy)",
                          "frac_of_nominal_8000": achieved / 8000.0},
             "config": workload_config(name, world), "bytes_per_step": bytes_all, "kv_copies": copies,
             "launch": "CUDA graph replay, one step per graph" if graphed else "eager launches", "clocks": clocks,
             "_got": res, "_q": qn, "_krange": (k0, k1)}
        if tag:
            r["config"]["workload"] += tag
        if collective and with_variants:
            phase(f"{name}: the rank's chunk alone")
            loc_ms, _, _, _, _ = measure(step_local)
            r["collective"] = {"local_chunk_only_ms": loc_ms, "step_ms": ms, "share_of_step": max(0.0, 1.0 - loc_ms / ms),
                               "what": "step = split-KV kernel + one kernel that merges the rank's records, stores them on every rank, "
                                       "waits for all ranks and merges; local_chunk_only = the rank's partial record alone, no exchange"}
            phase(f"{name}: NCCL all-gather variant")
            n_ms, _, _, _, _ = measure(step_nccl)
            r["nccl_gather"] = {"value": bytes_all / (n_ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": n_ms,
                                "what": "decode_partial + NCCL all_gather_into_tensor + lse_combine"}
        # e2e: host q up, result down, through the C ABI
        if not args.quick:
            phase(f"{name}: host-buffer steps")
            qh = torch.from_numpy(np.ascontiguousarray(qn, dtype=np.float32)).pin_memory()
            host_out = torch.empty(qn.shape if not collective else (B, Hq, D), dtype=torch.float32).pin_memory()
            if not collective:
                hq4, ho4 = t4(qh.data_ptr(), qh.shape, _lib.F32), t4(host_out.data_ptr(), host_out.shape, _lib.F32)

                def e2e_step():
                    _lib.check(L.fusor_cuda_flash_attention_decode_host(dev.handle, caches[0]._h, ctypes.byref(hq4), ctypes.c_float(w.scale),
                                                                        ctypes.byref(ho4)), dev.handle)
            else:
                dq32 = torch.empty(qn.shape, dtype=torch.float32, device=cuda)
                tq32 = fb.Tensor.from_torch(dev, dq32)

                def e2e_step():
                    _lib.check(L.fusor_cuda_buffer_upload(dev.handle, dq32.data_ptr(), qh.data_ptr(), qh.numel() * 4), dev.handle)
                    exchange.decode(caches[0], tq32, w.scale, tout3)
                    _lib.check(L.fusor_cuda_buffer_download(dev.handle, host_out.data_ptr(), out3.data_ptr(), out3.numel() * 4), dev.handle)
            with torch.cuda.stream(stream):
                for _ in range(2):
                    e2e_step()
                barrier()
                t0 = time.perf_counter()
                n_e2e = max(3, min(args.steps, 20))
                for _ in range(n_e2e):
                    e2e_step()
                torch.cuda.synchronize()
                e2e_s = max_over_ranks(time.perf_counter() - t0)
            r["e2e"] = {"value": bytes_all * n_e2e / e2e_s / 1e9, "unit": "GB/s", "h2d_bytes_per_step": int(qh.numel() * 4 * world),
                        "d2h_bytes_per_step": int(host_out.numel() * 4 * world),
                        "matches_device_path": bool(np.array_equal(host_out.numpy().reshape(-1), res.reshape(-1)))}
        else:
            r["e2e"] = None
        if exchange is not None:
            exchange.close()  # collective: unmap, barrier, free
        for c in caches:
            c.close()
        return r

    def decode_parity(r, w, name, w_full=None):
        got = r.pop("_got"); qn = r.pop("_q"); k0, k1 = r.pop("_krange")
        par = {"finite": bool(np.isfinite(got).all())}
        if rank == 0 and not args.quick:
            if name == "cfg3":
                nb = min(8, qn.shape[0])
                want = np.stack([O.flash_attention(qn[b:b + 1], w.k_dense[b][None, k0:k1], w.v_dense[b][None, k0:k1], w.scale)[0]
                                 for b in range(nb)])
                err = np.abs(got[:nb] - want)
                par["sequences_checked"] = nb
            else:
                wf = w_full if w_full is not None else w  # the whole sequence, whatever the number of chunks
                want = O.flash_attention(wf.q, wf.k_dense[0][None], wf.v_dense[0][None], wf.scale)
                err = np.abs(got.reshape(want.shape) - want)
                par["against"] = "the oracle on the unsplit sequence"
            par.update(max_abs=float(err.max()), mean_abs=float(err.mean()), tolerance="max 2e-3, mean 2e-4")
        r["parity"] = par
        return r

    def load_cfg3():
        return W.cfg3(B=16) if args.small else W.cfg3()

    def load_cfg4():
        """(this rank's chunk, the whole sequence on rank 0 for the parity check)"""
        skv = 16384 if args.small else 131072
        if fake_world:  # one rank's chunk alone on one GPU: it is checked against the attention over that chunk
            mine = W.cfg4(Skv=skv, rank=0, world=fake_world)
            return mine, mine
        full = W.cfg4(Skv=skv) if (rank == 0 or world == 1) else None
        mine = full if world == 1 else W.cfg4(Skv=skv, rank=rank, world=world, keep_dense=False)
        return mine, full

    # ======================================================================= the neighbours of the path
    def time_steps(step):
        for _ in range(args.warmup):
            step(0)
        barrier()
        settle_clocks(step)
        sampler.start()
        t0 = time.time()
        with torch.cuda.stream(stream):
            total_ms, _, _ = timed(step, args.steps)
        clocks = sampler.stop(t0, time.time())
        return total_ms / args.steps, clocks

    def run_oproj():
        B, Hq_all, S, D, N = (2, 16, 2048, 128, 2048) if args.small else (4, 32, 4096, 128, 4096)
        Hq = Hq_all // world
        rng = np.random.default_rng(21)
        n_copies = 2
        gen = torch.Generator(device=cuda)
        gen.manual_seed(21)  # the same attention tensor on every rank: each rank takes its heads of it
        attn_all = [torch.randn((B, Hq_all, S, D), device=cuda, dtype=torch.float32, generator=gen).to(torch.bfloat16) for _ in range(n_copies)]
        attn = [a[:, rank * Hq:(rank + 1) * Hq].contiguous() for a in attn_all]
        full0 = attn_all[0].float().cpu().numpy() if rank == 0 else None
        del attn_all
        w_all = W.bf16_round((rng.standard_normal((N, Hq_all * D)) / np.sqrt(Hq_all * D)).astype(np.float32))
        c0, c1 = (rank * Hq * D, (rank + 1) * Hq * D)
        w_dev = bf16_dev(w_all[:, c0:c1])
        out = torch.empty((B, S, N), device=cuda, dtype=torch.float32)
        ta = [fb.Tensor.from_torch(dev, a) for a in attn]
        tw = fb.Tensor.from_torch(dev, w_dev)
        to = fb.Tensor.from_torch(dev, out)
        comm = sharding.Communicator(dev, rank, world) if use_dist else None

        def step(i):
            if comm is not None:
                comm.out_proj(ta[i % n_copies], tw, None, to)  # GEMM + all-reduce, one library call
            else:
                ta[i % n_copies].out_proj(tw, None, out=to)
        with torch.cuda.stream(stream):
            l0 = dev.launch_count()
            ms, clocks = time_steps(step)
            launches = dev.launch_count() - l0
            gemm_ms = None
            if comm is not None:
                gemm_ms, _ = time_steps(lambda i: ta[i % n_copies].out_proj(tw, None, out=to))
            step(0)
        stream.synchronize()
        got = out.cpu().numpy()
        flops = 2.0 * B * S * N * Hq_all * D
        achieved = flops / world / ((gemm_ms or ms) * 1e-3) / 1e12
        par = {"finite": bool(np.isfinite(got).all())}
        if rank == 0:
            rows = np.random.default_rng(1).integers(0, B * S, 64)
            x = np.stack([full0[r // S, :, r % S, :].reshape(-1) for r in rows])
            want = O.out_proj(x.reshape(len(rows), Hq_all, 1, D), w_all)[:, 0]  # each sampled row as a batch of one token
            err = np.abs(got.reshape(B * S, N)[rows] - want)
            par.update(max_abs=float(err.max()), mean_abs=float(err.mean()), rows_checked=int(len(rows)),
                       tolerance="max 2e-4" if world == 1 else "max 4e-4 (the sum over ranks adds one f32 rounding per rank)")
        if comm is not None:
            comm.close()
        cfg = workload_config("oproj", world)
        if args.small:
            cfg = dict(cfg, workload=cfg["workload"] + " (scaled down: B2 Hq16 S2048 N2048)", flops_per_step=flops)
        r = {"value": flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms, "gpu_launches": launches,
             "clocks": clocks, "parity": par, "e2e": None,
             "roofline": {"bound": "tensor", "achieved": achieved, "peak": peaks["tensor_sustained"], "unit": "TFLOP/s",
                          "frac": achieved / peaks["tensor_sustained"], "traffic": None,
                          "peak_source": f"{peaks['source']} (cuBLAS bf16, sustained loop under the power cap)",
                          "frac_of_burst_peak": achieved / peaks["tensor_burst"],
                          "note": "the GEMM kernel alone; the step's value includes the all-reduce" if comm is not None else None},
             "config": cfg}
        if gemm_ms is not None:
            out_bytes = out.numel() * 4
            r["collective"] = {"gemm_only_ms": gemm_ms, "step_ms": ms, "share_of_step": max(0.0, 1.0 - gemm_ms / ms),
                               "all_reduce_bytes_per_rank": out_bytes, "NCCL_NVLS_ENABLE": os.environ.get("NCCL_NVLS_ENABLE", "unset"),
                               "what": "NCCL all-reduce of the f32 partial sums behind fusor_cuda_attention_out_proj_all_reduce"}
        return r

    def run_rope():
        B, Hq_all, Hkv_all, S, D = (2, 16, 4, 4096, 128) if args.small else (4, 32, 8, 4096, 128)
        Hq, Hkv = Hq_all // world, Hkv_all // world
        rc = fb.RopeCache.new(D, S, 10000.0, dev)
        pages = (S + 15) // 16
        cache = fb.PagedKvCache(dev, B, Hkv, D, num_pages=B * pages, max_pages_per_seq=pages)
        q = torch.randn((B, Hq, S, D), device=cuda, dtype=torch.bfloat16)
        k = torch.randn((B, Hkv, S, D), device=cuda, dtype=torch.bfloat16)
        v = torch.randn((B, Hkv, S, D), device=cuda, dtype=torch.bfloat16)
        qo = torch.empty_like(q)
        tq, tk, tv, tqo = (fb.Tensor.from_torch(dev, t) for t in (q, k, v, qo))
        cq, ck, cv, co = tq._c4(), tk._c4(), tv._c4(), tqo._c4()
        flush = torch.empty(300 << 20, dtype=torch.uint8, device=cuda)

        def step(i):
            cache.reset()
            flush.zero_()  # 300 MB written: the tensors of the next step come from HBM
            rcode = L.fusor_cuda_kvcache_rope_append(cache._h, ctypes.byref(cq), ctypes.byref(ck), ctypes.byref(cv), rc.cos.ptr,
                                                     rc.sin.ptr, S, 0, 0, ctypes.byref(co))
            assert rcode == 0, L.fusor_cuda_last_error(dev.handle)
        # time only the fused kernel: events around the call, after the flush
        for _ in range(args.warmup):
            step(0)
        barrier()
        times = []
        sampler.start()
        t0 = time.time()
        with torch.cuda.stream(stream):
            for i in range(args.steps):
                cache.reset()
                flush.zero_()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(stream)
                rcode = L.fusor_cuda_kvcache_rope_append(cache._h, ctypes.byref(cq), ctypes.byref(ck), ctypes.byref(cv), rc.cos.ptr,
                                                         rc.sin.ptr, S, 0, 0, ctypes.byref(co))
                b.record(stream)
                times.append((a, b))
        barrier()
        t1 = time.time()
        clocks = sampler.stop(t0, t1)
        ms = max_over_ranks(float(np.mean([a.elapsed_time(b) for a, b in times])))
        nbytes_rank = q.numel() * 2 * 2 + k.numel() * 2 * 2 * 2
        # parity: rotated q rows and the gathered K of one (batch, head) against the oracle, bit for bit
        cos, sin = O.rope_tables(D, S, 10000.0)
        qn = q[0, 0].float().cpu().numpy()[None, None]
        want_q = O.bf16_round(O.rope(qn, cos, sin, 0, False))
        got_q = qo[0, 0].float().cpu().numpy()[None, None]
        gk, _ = cache.gather(B, S)
        want_k = O.bf16_round(O.rope(k[0, 0].float().cpu().numpy()[None, None], cos, sin, 0, False))
        par = {"q_bit_exact": bool(np.array_equal(got_q.view(np.uint32), want_q.view(np.uint32))),
               "k_bit_exact": bool(np.array_equal(gk.as_slice()[0, 0].view(np.uint32), want_k[0, 0].view(np.uint32)))}
        achieved = nbytes_rank / (ms * 1e-3) / 1e9
        cfg = dict(workload_config("rope", world), bytes_per_step=nbytes_rank * world)
        if args.small:
            cfg["workload"] += " (scaled down: B2 Hq16 Hkv4)"
        return {"value": nbytes_rank * world / (ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": ms, "gpu_launches": args.steps,
                "clocks": clocks, "parity": par, "e2e": None,
                "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm"], "unit": "GB/s", "frac": achieved / peaks["hbm"],
                             "traffic": None, "peak_source": f"{peaks['source']} (device copy)"},
                "config": cfg}

    # ----------------------------------------------------------------------- run the selected workload
    extras = {}
    t_start = time.time()

    def build_line(r, dtype):
        if fake_world:
            r["config"]["shard_of"] = f"rank 0 of a {fake_world}-rank job on one GPU: value is extrapolated as {fake_world} x this shard"
        line = {"metric": METRIC, "value": r["value"], "unit": r["unit"], "n_gpus": 1 if fake_world else world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": dtype, "data": DATA,
                "config": r["config"], "roofline": r["roofline"], "e2e": r.get("e2e"), "clocks": r.get("clocks"),
                "gpu_launches": r["gpu_launches"], "parity": r.get("parity")}
        for key in ("cpu_baseline", "rank_ms_per_step", "collective", "nccl_gather", "input_copies", "bytes_per_step", "kv_copies", "launch"):
            if key in r:
                line[key] = r[key]
        line.update(extras)
        return line

    # The extras of a multi-rank run hold collectives (record exchange, NCCL).  Should one of them never return, the
    # headline measurement, which is complete by then, must still be reported: after EXTRAS_DEADLINE_S every rank leaves,
    # rank 0 first printing the line with the extras that did finish and the name of the one that did not.
    deadline = None
    pending = {"name": None}

    def phase(name):
        """Names the part that runs next (the deadline reports it) and leaves a trace of progress on stderr."""
        pending["name"] = name
        if rank == 0:
            sys.stderr.write(f"[bench] {name} starts at {time.time() - t_start:.1f} s\n")
            sys.stderr.flush()

    def start_deadline(r, dtype):
        def last_line():
            if pending.get("printed"):
                return None
            extras[pending["name"] or "extras"] = {"error": f"did not finish within {EXTRAS_DEADLINE_S} s; left out"}
            return build_line(r, dtype)
        return start_exit_timer(EXTRAS_DEADLINE_S, rank, args.real_stdout, last_line, lambda: pending["name"])
    name = args.workload
    if name in ("oproj", "rope"):
        r = run_oproj() if name == "oproj" else run_rope()
        dtype = "bf16"
    elif name in ("cfg1", "cfg2", "cfg5"):
        tag = ""
        if args.small and name != "cfg1":
            w = W.cfg2(B=2, Hq=16, Hkv=4) if name == "cfg2" else W.cfg5(S=8192, Hq=8, Hkv=2)
            tag = " (scaled down: B2 Hq16 Hkv4)" if name == "cfg2" else " (scaled down: S8192 Hq8 Hkv2)"
        else:
            w = {"cfg1": W.cfg1, "cfg2": W.cfg2, "cfg5": W.cfg5}[name]()
        r = run_prefill(w, name, tag)
        q, k, v = r.pop("_slice")
        got = r.pop("_got")
        if name == "cfg1":
            want = O.flash_attention(q, k, v, w.scale, mask_kind=O.MASK_CAUSAL)
            err = np.abs(got - want)
            r["parity"] = {"max_abs": float(err.max()), "mean_abs": float(err.mean()), "rows_checked": int(q.shape[1] * q.shape[2]),
                           "tolerance": "max 2e-5, mean 2e-6 (f32 tensors, f32 arithmetic)"}
        else:
            rows = np.unique(np.random.default_rng(0).integers(0, q.shape[0] * q.shape[1] * q.shape[2], 400))
            want = O.flash_attention(q, k, v, w.scale, mask_kind=O.MASK_CAUSAL, rows=rows, skip_masked=True)
            err = np.abs(got.reshape(-1, q.shape[3])[rows] - want)
            r["parity"] = {"max_abs": float(err.max()), "mean_abs": float(err.mean()), "rows_checked": int(rows.size),
                           "tolerance": "max 2e-3, mean 2e-4"}
        dtype = "f32" if name == "cfg1" else "bf16"
        if rank == 0 and world == 1 and not fake_world and not args.no_extras and not args.quick:
            cores = O.use_all_cores()
            fn, flops, desc = cpu_full_prefill(w) if name == "cfg1" else cpu_prefill_sample(w)
            sec = time_cpu(fn, 3, 1)
            r["cpu_baseline"] = {"value": flops / sec / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                                 "sample": desc, "seconds_per_sample": sec}
        if name == "cfg2" and not args.no_extras and not args.quick and not fake_world:
            # the decode configurations and the step after attention ride on the same line, at every N
            if use_dist:
                deadline = start_deadline(r, dtype)
            try:
                phase("decode")
                wd = load_cfg3()
                d = decode_parity(run_decode(wd, "cfg3", chunked=False), wd, "cfg3")
                extras["decode"] = d
                del wd
                phase("decode_long")
                mine, full = load_cfg4()
                d4 = decode_parity(run_decode(mine, "cfg4", chunked=True), mine, "cfg4", full)
                extras["decode_long"] = d4
                del mine, full
                if use_dist:
                    phase("oproj")
                    extras["oproj"] = run_oproj()
            except Exception as e:  # an extra must not take the headline measurement with it
                if not use_dist:
                    raise
                import traceback
                traceback.print_exc()
                extras[pending["name"]] = {"error": f"{type(e).__name__}: {e}"}
    else:
        if name == "cfg3":
            w = load_cfg3()
            r = decode_parity(run_decode(w, "cfg3", chunked=False, tag=" (scaled down: B16)" if args.small else ""), w, "cfg3")
        else:
            mine, full = load_cfg4()
            r = decode_parity(run_decode(mine, "cfg4", chunked=True, tag=" (scaled down: 16384 keys)" if args.small else ""), mine, "cfg4", full)
            w = mine
        if rank == 0 and world == 1 and not fake_world and not args.quick and not args.no_extras:
            cores = O.use_all_cores()
            fn, nbytes, desc = cpu_decode_sample(w, 4 if name == "cfg3" else 1)
            sec = time_cpu(fn, 2, 1)
            r["cpu_baseline"] = {"value": nbytes / sec / 1e9, "unit": "GB/s", "cores": cores, "kind": "port",
                                 "sample": desc, "seconds_per_sample": sec}
        dtype = "bf16"

    line = build_line(r, dtype) if rank == 0 else None
    if use_dist:
        # the line leaves before the teardown, which is a collective of its own and stays under the deadline
        if rank == 0:
            pending["printed"] = True
            os.write(args.real_stdout, (json.dumps(line) + "\n").encode())
            line = None
        if deadline is None:
            deadline = start_deadline(r, dtype)
        dist.destroy_process_group()
    if deadline is not None:
        deadline.cancel()
    return line if rank == 0 else None


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg2", choices=["cfg1", "cfg2", "cfg3", "cfg4", "cfg5", "oproj", "rope"],
                    help="cfg1-cfg5: the attention configurations; oproj / rope: the steps after and before attention "
                    "(output projection GEMM, fused RoPE + cache append) at config 2's sizes")
    ap.add_argument("--no-extras", action="store_true", help="skip the decode / oproj entries and the CPU baseline")
    ap.add_argument("--shard-of", type=int, default=0, help="for profiler captures on one GPU: run rank 0's shard of an "
                    "N-rank job (no process group; the line is marked as a shard)")
    ap.add_argument("--no-graph", action="store_true", help="decode workloads: time eager launches instead of CUDA graph replays")
    ap.add_argument("--decode-ctas", type=int, default=0, help="decode workloads: grid size of the split-KV kernel (0 = automatic)")
    ap.add_argument("--quick", action="store_true", help="for profiler captures: no clock-settling loop, no e2e, no extras")
    ap.add_argument("--small", action="store_true", help="for profiler captures: a scaled-down case of the workload "
                    "(prefill B2 Hq16 Hkv4 S4096; decode B16 / 16384 keys)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        reference_arm(args, rank)
        return
    args.warmup = max(args.warmup, 3)
    # stdout carries the JSON line and nothing else: libraries that print there (NCCL announces its version on stdout when a
    # communicator is first made) are sent to stderr for the duration of the run
    sys.stdout.flush()
    real_stdout = os.dup(1)
    args.real_stdout = real_stdout
    os.dup2(2, 1)
    try:
        line = gpu_arm(args, rank, world, local_rank)
    finally:
        sys.stdout.flush()
        os.dup2(real_stdout, 1)
        os.close(real_stdout)
    if line is not None:
        print(json.dumps(line))
        sys.stdout.flush()


if __name__ == "__main__":
    main()
