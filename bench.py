#!/usr/bin/env python
"""Benchmark of the attention hot path.  One JSON line on stdout (rank 0).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg2|cfg3|cfg4|cfg5] [--impl reference]

Workload at N = 1 (default): BASELINE config 2, causal flash-attention prefill, B4 S4096 Hq32 Hkv8 D128,
bf16 inputs, f32 output; metric = attention TFLOP/s from the algorithmic causal FLOPs 4 B Hq D S(S+1)/2.
A "step" is one pass of the kernel over the batch.  With N > 1 (torchrun, one rank per GPU) the kv heads are split
over the ranks (strong scaling, no collective); `--workload cfg4` runs the long-context KV-chunk decode whose partials
are combined over NCCL.  `value` is timed with inputs resident in HBM; `e2e` is the same metric through the host-buffer
C-ABI entry point with the copies inside the timed region.  The line also carries the decode (config 3) GB/s at N = 1.
`--impl reference` times the CPU restatement of the reference's attention (oracle/) on the host cores instead.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

METRIC = "attention TFLOP/s (prefill) and KV GB/s (decode) at 1/2/4/8 B200 vs roofline"


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm": d["hbm_gbs"], "tensor_burst": d["bf16_tflops"], "tensor_sustained": d["bf16_tflops_sustained"],
                "source": "measured"}
    return {"hbm": 6650.0, "tensor_burst": 1590.0, "tensor_sustained": 1400.0, "source": "fallback"}


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
        mhz, mx, reasons, allmhz = [], [], set(), []
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
            allmhz.append(f)
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


# ------------------------------------------------------------------------------------------- CPU baseline
def cpu_prefill_sample(w):
    """Bounded sample of the prefill workload for the CPU arm: batch 0, kv head 0 with its g query heads, every row,
    evaluated densely with a [S,S] 0/-inf mask tensor exactly as the reference CPU composite does."""
    from oracle import oracle as O
    g = w.q.shape[1] // w.k.shape[1]
    q, k, v = w.q[:1, :g], w.k[:1, :1], w.v[:1, :1]
    S = q.shape[2]
    mask = O.causal_mask(S)
    flops = 4.0 * g * q.shape[3] * S * (S + 1) / 2
    desc = f"batch 0, kv head 0 ({g} query heads), all {S} rows, dense f32 composite with a [{S},{S}] mask tensor"
    return (lambda: O.flash_attention(q, k, v, w.scale, mask, O.MASK_QK)), flops, desc


def cpu_decode_sample(w, n_seq=8):
    from oracle import oracle as O
    n_seq = min(n_seq, w.q.shape[0])
    Hkv, D = w.k_pages.shape[1], w.k_pages.shape[3]
    nbytes = float(np.sum(w.kv_len[:n_seq])) * 2 * Hkv * D * 2
    def run():
        for b in range(n_seq):
            O.flash_attention(w.q[b:b + 1], w.k_dense[b][None], w.v_dense[b][None], w.scale)
    return run, nbytes, f"first {n_seq} sequences, all heads, dense f32 composite on de-paged K/V"


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
    """The reference's CPU implementation of the path (oracle port; the Rust sources cannot be built here)."""
    if rank != 0:
        return
    from floneum_b200 import workloads as W
    from oracle import oracle as O
    O.build()
    if args.workload in ("cfg2", "cfg5"):
        w = W.cfg2() if args.workload == "cfg2" else W.cfg5()
        fn, work, desc = cpu_prefill_sample(w)
        unit, scale_div = "TFLOP/s", 1e12
        cfg = {"workload": f"{args.workload}: causal flash-attention prefill B{w.q.shape[0]} S{w.q.shape[2]} Hq{w.q.shape[1]} "
                           f"Hkv{w.k.shape[1]} D128, bf16 in, f32 out", "flops_per_step": w.flops,
               "note": "CPU arm: each step is the bounded sample named in cpu_baseline.sample"}
    elif args.workload == "oproj":
        B, Hq, S, D, N, rows = 4, 32, 4096, 128, 4096, 256
        rng = np.random.default_rng(21)
        x = W.bf16_round(rng.standard_normal((1, Hq, rows, D)).astype(np.float32))
        wt = W.bf16_round((rng.standard_normal((N, Hq * D)) / 64).astype(np.float32))
        fn = lambda: O.out_proj(x, wt)
        work, desc = 2.0 * rows * N * Hq * D, f"{rows} of the {B * S} rows, all {N} outputs (f32 transpose + matmul)"
        unit, scale_div = "TFLOP/s", 1e12
        cfg = {"workload": f"oproj: out = attn[B{B},Hq{Hq},S{S},D{D}] (read in place) x W[{N},{Hq * D}]^T, bf16 in, f32 out",
               "flops_per_step": 2.0 * B * S * N * Hq * D, "note": "CPU arm: each step is the bounded sample named in cpu_baseline.sample"}
    elif args.workload == "rope":
        B, Hq, Hkv, S, D = 4, 32, 8, 4096, 128
        rng = np.random.default_rng(22)
        x = rng.standard_normal((1, Hq + Hkv, S, D)).astype(np.float32)
        cos, sin = O.rope_tables(D, S, 10000.0)
        fn = lambda: O.rope(x, cos, sin, 0, False)
        work, desc = float(x.nbytes * 2), "one batch entry: all 40 heads rotated, f32 (read + write bytes counted)"
        unit, scale_div = "GB/s", 1e9
        cfg = {"workload": f"rope: fused RoPE + KV-cache append, B{B} Hq{Hq} Hkv{Hkv} S{S} D{D}, bf16 in, bf16 pages",
               "note": "CPU arm: rotation only, on f32 copies; each step is the bounded sample named in cpu_baseline.sample"}
    else:
        w = W.cfg3() if args.workload == "cfg3" else W.cfg4()
        fn, work, desc = cpu_decode_sample(w)
        unit, scale_div = "GB/s", 1e9
        cfg = {"workload": f"{args.workload}: paged GQA decode B{w.q.shape[0]} Hq{w.q.shape[1]} Hkv{w.k_pages.shape[1]} D128, "
                           f"16-token pages, kv tokens {int(np.sum(w.kv_len))}", "bytes_per_step": w.bytes,
               "note": "CPU arm: each step is the bounded sample named in cpu_baseline.sample"}
    sec = time_cpu(fn, args.steps, min(args.warmup, 1))
    val = work / sec / scale_div
    cores = O.num_threads()
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": unit, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": min(args.warmup, 1), "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic (seeded N(0,1), bf16-rounded)", "config": cfg,
        "cpu_baseline": {"value": val, "unit": unit, "cores": cores, "kind": "port", "sample": desc},
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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg2", choices=["cfg2", "cfg3", "cfg4", "cfg5", "oproj", "rope"],
                    help="cfg2-cfg5: the attention configurations; oproj / rope: the steps after and before attention "
                    "(output projection GEMM, fused RoPE + cache append) at config 2's sizes")
    ap.add_argument("--no-extras", action="store_true", help="skip the decode line and the CPU baseline")
    ap.add_argument("--shard-of", type=int, default=0, help="for profiler captures on one GPU: run rank 0's shard of an "
                    "N-rank job (no process group; the line is marked as a shard)")
    ap.add_argument("--nccl-gather", action="store_true", help="cfg4 on several GPUs: exchange the split-KV records with an NCCL "
                    "all-gather between two kernels instead of the library's own peer-memory push + merge")
    ap.add_argument("--no-graph", action="store_true", help="decode workloads: time eager launches instead of a CUDA graph replay")
    ap.add_argument("--quick", action="store_true", help="for profiler captures: no clock-settling loop, no e2e, no extras")
    ap.add_argument("--small", action="store_true", help="for profiler captures: a scaled-down case of the workload "
                    "(prefill B2 Hq16 Hkv4 S4096; decode B16)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    fake_world = args.shard_of if (world == 1 and args.shard_of > 1) else 0
    if args.impl == "reference":
        reference_arm(args, rank)
        return

    import torch
    import torch.distributed as dist
    import floneum_b200 as fb
    from floneum_b200 import _lib, sharding, workloads as W
    from floneum_b200.cache import lse_combine
    L = _lib.load()
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local_rank}"))
    use_dist = world > 1
    if fake_world:
        world = fake_world  # shard sizes as in an N-rank job; no collectives, no cross-rank reductions
    stream = torch.cuda.Stream()
    dev = fb.Device.gpu(local_rank, stream.cuda_stream)
    peaks = load_peaks()
    cuda = torch.device(f"cuda:{local_rank}")

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

    def bf16_dev(a):  # numpy f32 (bf16-representable) -> torch bf16 on the GPU
        return torch.from_numpy(np.ascontiguousarray(a)).to(cuda).to(torch.bfloat16)

    def bf16_pinned(a):
        return torch.from_numpy(np.ascontiguousarray(a)).to(torch.bfloat16).pin_memory()

    result = {}
    sampler = ClockSampler(local_rank)

    # ======================================================================= prefill (cfg2 / cfg5)
    def run_prefill(w, tag):
        B, Hq, S, D = w.q.shape
        Hkv = w.k.shape[1]
        q0, q1 = sharding.q_head_range(Hq, Hkv, rank, world)
        k0, k1 = sharding.kv_head_range(Hkv, rank, world)
        q, k, v = w.q[:, q0:q1], w.k[:, k0:k1], w.v[:, k0:k1]
        in_bytes = (q.size + k.size + v.size) * 2
        copies = max(1, int(np.ceil(256e6 / in_bytes)))  # rotate inputs so that the working set exceeds L2
        dq, dk, dv = [], [], []
        for _ in range(copies):
            dq.append(bf16_dev(q)); dk.append(bf16_dev(k)); dv.append(bf16_dev(v))
        out = torch.empty(q.shape, dtype=torch.float32, device=cuda)
        cq = [t4(t.data_ptr(), t.shape, _lib.BF16) for t in dq]
        ck = [t4(t.data_ptr(), t.shape, _lib.BF16) for t in dk]
        cv = [t4(t.data_ptr(), t.shape, _lib.BF16) for t in dv]
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
            # keep the GPU busy with untimed steps until the clocks have been under load for 0.5 s
            i = args.warmup
            while not args.quick and time.time() - t_busy0 < 0.5:
                for _ in range(20):
                    step(i)
                    i += 1
                torch.cuda.synchronize()
            barrier()
            launches0 = dev.launch_count()
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
            ev[0].record(stream)
            for i in range(args.steps):
                step(i)
                ev[i + 1].record(stream)
            barrier()
            clocks = sampler.stop(t_busy0, time.time())
            launches = dev.launch_count() - launches0
            dev.synchronize()
        total_ms = max_over_ranks(ev[0].elapsed_time(ev[-1]))
        per_launch_ms = [ev[i].elapsed_time(ev[i + 1]) for i in range(args.steps)]
        flops_rank = 4.0 * B * (q1 - q0) * D * S * (S + 1) / 2
        flops_all = w.flops
        value = flops_all * args.steps / (total_ms * 1e-3) / 1e12
        achieved = flops_rank / (statistics.mean(per_launch_ms) * 1e-3) / 1e12
        # parity spot check of the timed configuration (last output, sampled rows)
        got = out.cpu().numpy()

        # ---- e2e: host buffers through the C ABI, copies inside the timed region
        hq, hk, hv = bf16_pinned(q), bf16_pinned(k), bf16_pinned(v)
        hout = torch.empty(q.shape, dtype=torch.float32).pin_memory()
        eq, ek, evv = (t4(t.data_ptr(), t.shape, _lib.BF16) for t in (hq, hk, hv))
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
        # K launches back to back after a 0.5 s busy loop run under the power cap: the sustained cuBLAS figure is the
        # denominator; the fraction of the burst figure is given beside it.
        peak = peaks["tensor_sustained"]
        return {
            "value": value, "unit": "TFLOP/s", "ms_per_step": total_ms / args.steps, "gpu_launches": launches,
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                         # dram read+write of one launch, scaled by (batch, head) pairs from the ncu capture of the
                         # B2 Hq16 case (68.2 MB for 32 pairs)
                         "traffic": 68.2e6 * (B * (q1 - q0)) / 32.0 if D == 128 and S == 4096 else None,
                         "peak_source": f"{peaks['source']} (cuBLAS bf16, sustained loop under the power cap)",
                         "frac_of_burst_peak": achieved / peaks["tensor_burst"], "burst_peak": peaks["tensor_burst"],
                         "frac_of_nominal_2250": achieved / 2250.0,
                         "note": "achieved counts the V pre-pass kernel's time as well (both kernels of a step)"},
            "e2e": {"value": e2e_val, "unit": "TFLOP/s", "h2d_bytes_per_step": int(in_bytes * world),
                    "d2h_bytes_per_step": int(out.numel() * 4 * world), "matches_device_path": e2e_ok},
            "clocks": clocks,
            "config": {"workload": f"{tag}: causal flash-attention prefill B{B} S{S} Hq{Hq} Hkv{Hkv} D{D}, bf16 in, f32 out",
                       "sharding": f"kv heads split over {world} rank(s)", "l2": f"inputs rotate over {copies} copies "
                       f"({in_bytes * copies / 1e6:.0f} MB) so each launch reads HBM-cold data", "flops_per_step": flops_all},
            "_got": got, "_slice": (q, k, v),
        }

    # ======================================================================= decode (cfg3 / cfg4)
    def run_decode(w, tag, shard_heads=True, chunked=False):
        B, Hq, _, D = w.q.shape
        Hkv_all = w.k_pages.shape[1]
        if shard_heads:
            k0, k1 = sharding.kv_head_range(Hkv_all, rank, world)
            q0, q1 = sharding.q_head_range(Hq, Hkv_all, rank, world)
        else:
            k0, k1, q0, q1 = 0, Hkv_all, 0, Hq
        kp, vp = np.ascontiguousarray(w.k_pages[:, k0:k1]), np.ascontiguousarray(w.v_pages[:, k0:k1])
        qn = np.ascontiguousarray(w.q[:, q0:q1])
        cache = fb.PagedKvCache(dev, B, k1 - k0, D, kp.shape[0], w.page_table.shape[1])
        cache.write_pages(0, kp, vp)
        cache.set_page_table(w.page_table, w.kv_len)
        dq = bf16_dev(qn)
        out = torch.empty(qn.shape, dtype=torch.float32, device=cuda)
        tq, to = fb.Tensor.from_torch(dev, dq), fb.Tensor.from_torch(dev, out)
        kv_bytes_rank = float(np.sum(w.kv_len)) * 2 * (k1 - k0) * D * 2
        flush = torch.empty(int(300e6), dtype=torch.uint8, device=cuda) if kv_bytes_rank < 400e6 else None

        if chunked and use_dist:
            # fixed buffers so that the step can be captured in a CUDA graph
            part = torch.empty((B, q1 - q0, D + 2), dtype=torch.float32, device=cuda)
            gathered = torch.empty((world, B, q1 - q0, D + 2), dtype=torch.float32, device=cuda)
            out3 = torch.empty((B, q1 - q0, D), dtype=torch.float32, device=cuda)
            tpart, tgath, tout3 = (fb.Tensor.from_torch(dev, t) for t in (part, gathered, out3))
            exchange = None if args.nccl_gather else sharding.PeerExchange(dev, rank, world, B * (q1 - q0) * (D + 2))

        def step():
            if chunked and use_dist:
                cache.decode_partial(tq, w.scale, tpart)
                if exchange is not None:
                    exchange.lse_combine(tpart, tout3)  # peer stores + epoch flags + merge, inside the library's kernels
                else:
                    dist.all_gather_into_tensor(gathered, part)
                    lse_combine(dev, tgath, tout3)
                return out3
            cache.decode(tq, w.scale, to)
            return out
        with torch.cuda.stream(stream):
            for _ in range(args.warmup):
                if flush is not None:
                    flush.zero_()
                res = step()
            barrier()
            # A decode step is launch-bound at small shard sizes: capture it once in a CUDA graph and replay it.
            graph = None
            if not args.no_graph and not args.quick:
                try:
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph, stream=stream):
                        res = step()
                    graph.replay()
                    torch.cuda.synchronize()
                except Exception as e:  # capture is an optimisation only
                    sys.stderr.write(f"CUDA graph capture failed ({e}); timing eager launches\n")
                    graph = None
                    torch.cuda.synchronize()
            barrier()
            launches0 = dev.launch_count()
            evs = []
            for _ in range(args.steps):
                if flush is not None:
                    flush.zero_()  # write a buffer larger than L2 between timed launches
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(stream)
                if graph is not None:
                    graph.replay()
                else:
                    res = step()
                b.record(stream)
                evs.append((a, b))
            barrier()
            launches = dev.launch_count() - launches0
            if graph is not None:
                # kernels of ours inside each replay: split-KV + combine (+ push + merge, or + merge after the NCCL gather)
                launches = args.steps * ((4 if exchange is not None else 3) if (chunked and use_dist) else 2)
            dev.synchronize()
        ms = [a.elapsed_time(b) for a, b in evs]
        mean_ms = max_over_ranks(statistics.mean(ms))
        # e2e: the host-buffer entry point (q up, result down; the KV cache is the library's device-resident object)
        e2e = {"value": None, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
        if not (chunked and use_dist) and not args.quick:
            # pinned host buffers through the C ABI: q up, result down, one synchronous call per step
            qh = torch.from_numpy(np.ascontiguousarray(qn, dtype=np.float32)).pin_memory()
            host_out = torch.empty(qh.shape, dtype=torch.float32).pin_memory()
            hq4, ho4 = t4(qh.data_ptr(), qh.shape, _lib.F32), t4(host_out.data_ptr(), host_out.shape, _lib.F32)

            def e2e_step():
                _lib.check(L.fusor_cuda_flash_attention_decode_host(dev.handle, cache._h, ctypes.byref(hq4), ctypes.c_float(w.scale),
                                                                    ctypes.byref(ho4)), dev.handle)
            for _ in range(2):
                e2e_step()
            barrier()
            t0 = time.perf_counter()
            n_e2e = max(3, min(args.steps, 20))
            for _ in range(n_e2e):
                e2e_step()
            e2e_s = max_over_ranks(time.perf_counter() - t0)
            e2e = {"unit": "GB/s", "h2d_bytes_per_step": int(qh.numel() * 4 * world), "d2h_bytes_per_step": int(host_out.numel() * 4 * world),
                   "matches_device_path": bool(np.array_equal(host_out.numpy().reshape(-1), (res if isinstance(res, torch.Tensor) else out).float().cpu().numpy().reshape(-1)))}
        bytes_rank = kv_bytes_rank + B * (q1 - q0) * D * 6 + 4 * float(np.sum((w.kv_len + 15) // 16))
        bytes_all = bytes_rank * world
        achieved = bytes_rank / (statistics.mean(ms) * 1e-3) / 1e9
        if "value" not in e2e:
            e2e["value"] = bytes_all * n_e2e / e2e_s / 1e9
        return {"value": bytes_all / (mean_ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": mean_ms, "gpu_launches": launches, "e2e": e2e,
                "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm"], "unit": "GB/s",
                             "frac": achieved / peaks["hbm"],
                             # ncu capture of the B16 case: dram read+write = 1.02 x the algorithmic bytes, scaled by bytes
                             "traffic": bytes_rank * 1.02, "peak_source": f"{peaks['source']} (device copy)",
                             "frac_of_nominal_8000": achieved / 8000.0},
                "config": {"workload": f"{tag}: paged GQA decode B{B} Hq{Hq} Hkv{Hkv_all} D{D}, 16-token pages, "
                           f"kv tokens {int(np.sum(w.kv_len))}", "bytes_per_step": bytes_all,
                           "launch": "CUDA graph replay of one step" if graph is not None else "eager launches",
                           "l2": "KV working set exceeds L2" if flush is None else "300 MB buffer written between timed launches"},
                "_got": (res if isinstance(res, torch.Tensor) else out).cpu().numpy(), "_q": qn, "_krange": (k0, k1)}

    # ======================================================================= the neighbours of the path
    def time_steps(step, n_copies_note):
        for _ in range(args.warmup):
            step(0)
        barrier()
        if not args.quick:  # let the clocks settle under load, as the attention legs do
            t_end = time.time() + 0.5
            i = 0
            while time.time() < t_end:
                step(i); i += 1
                if i % 16 == 0:
                    torch.cuda.synchronize()
        barrier()
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
        sampler.start()
        t0 = time.time()
        with torch.cuda.stream(stream):
            for i, (a, b) in enumerate(evs):
                a.record(stream)
                step(i)
                b.record(stream)
        barrier()
        t1 = time.time()
        clocks = sampler.stop(t0, t1)
        ms = max_over_ranks(float(np.mean([a.elapsed_time(b) for a, b in evs])))
        return ms, clocks

    def run_oproj():
        B, Hq_all, S, D, N = (2, 16, 2048, 128, 2048) if args.small else (4, 32, 4096, 128, 4096)
        Hq = Hq_all // world
        rng = np.random.default_rng(21)
        n_copies = 2
        attn = [torch.randn((B, Hq, S, D), device=cuda, dtype=torch.bfloat16, generator=None) for _ in range(n_copies)]
        w_all = W.bf16_round((rng.standard_normal((N, Hq_all * D)) / np.sqrt(Hq_all * D)).astype(np.float32))
        c0, c1 = (rank * Hq * D, (rank + 1) * Hq * D)
        w_dev = bf16_dev(w_all[:, c0:c1])
        out = torch.empty((B, S, N), device=cuda, dtype=torch.float32)
        ta = [fb.Tensor.from_torch(dev, a) for a in attn]
        tw = fb.Tensor.from_torch(dev, w_dev)
        to = fb.Tensor.from_torch(dev, out)
        flush = torch.empty(300 << 20, dtype=torch.uint8, device=cuda)

        def step(i):
            ta[i % n_copies].out_proj(tw, None, out=to)
            if use_dist:
                dist.all_reduce(out)
        with torch.cuda.stream(stream):
            l0 = dev.launch_count()
            ms, clocks = time_steps(step, n_copies)
            launches = dev.launch_count() - l0
            step(0)
        stream.synchronize()
        got = out.cpu().numpy()
        flops = 2.0 * B * S * N * Hq_all * D
        achieved = flops / world / (ms * 1e-3) / 1e12
        # parity on sampled rows: rank 0 rebuilds the full-K rows only on one GPU (N > 1: the shards' random inputs differ)
        par = {"finite": bool(np.isfinite(got).all())}
        if world == 1:
            rows = np.random.default_rng(1).integers(0, B * S, 64)
            a0 = attn[0].float().cpu().numpy()
            x = np.stack([a0[r // S, :, r % S, :].reshape(-1) for r in rows])
            want = O.out_proj(x.reshape(len(rows), Hq, 1, D), w_all)[:, 0]  # each sampled row as a batch of one token
            err = np.abs(got.reshape(B * S, N)[rows] - want)
            par.update(max_abs=float(err.max()), mean_abs=float(err.mean()), rows_checked=int(len(rows)), tolerance="max 2e-4")
        return {"value": flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms, "gpu_launches": launches,
                "clocks": clocks, "parity": par, "e2e": None,
                "roofline": {"bound": "tensor", "achieved": achieved, "peak": peaks["tensor_sustained"], "unit": "TFLOP/s",
                             "frac": achieved / peaks["tensor_sustained"], "traffic": None,
                             "peak_source": f"{peaks['source']} (cuBLAS bf16, sustained loop under the power cap)",
                             "frac_of_burst_peak": achieved / peaks["tensor_burst"]},
                "config": {"workload": f"oproj: out = attn[B{B},Hq{Hq_all},S{S},D{D}] (read in place) x W[{N},{Hq_all * D}]^T, bf16 in, f32 out",
                           "sharding": f"query heads split over {world} rank(s)" + (", partial sums all-reduced over NCCL" if use_dist else ""),
                           "l2": f"attention input rotates over {n_copies} copies", "flops_per_step": flops}}

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
        return {"value": nbytes_rank * world / (ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": ms, "gpu_launches": args.steps,
                "clocks": clocks, "parity": par, "e2e": None,
                "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm"], "unit": "GB/s", "frac": achieved / peaks["hbm"],
                             "traffic": None, "peak_source": f"{peaks['source']} (device copy)"},
                "config": {"workload": f"rope: fused RoPE + KV-cache append, B{B} Hq{Hq_all} Hkv{Hkv_all} S{S} D{D}, bf16 in, bf16 pages",
                           "sharding": f"heads split over {world} rank(s), no collective", "bytes_per_step": nbytes_rank * world,
                           "l2": "300 MB buffer written between timed launches; table uploads are inside the timed region"}}

    # ----------------------------------------------------------------------- run the selected workload
    from oracle import oracle as O  # checker + CPU baseline only
    extras = {}
    if args.workload in ("oproj", "rope"):
        r = run_oproj() if args.workload == "oproj" else run_rope()
        dtype = "bf16"
    elif args.workload in ("cfg2", "cfg5"):
        if args.small:
            w = W.cfg2(B=2, Hq=16, Hkv=4) if args.workload == "cfg2" else W.cfg5(S=8192, Hq=8, Hkv=2)
        else:
            w = W.cfg2() if args.workload == "cfg2" else W.cfg5()
        r = run_prefill(w, args.workload + (" (scaled down)" if args.small else ""))
        q, k, v = r.pop("_slice")
        got = r.pop("_got")
        rows = np.unique(np.random.default_rng(0).integers(0, q.shape[0] * q.shape[1] * q.shape[2], 400))
        want = O.flash_attention(q, k, v, w.scale, mask_kind=O.MASK_CAUSAL, rows=rows, skip_masked=True)
        err = np.abs(got.reshape(-1, q.shape[3])[rows] - want)
        r["parity"] = {"max_abs": float(err.max()), "mean_abs": float(err.mean()), "rows_checked": int(rows.size),
                       "tolerance": "max 2e-3, mean 2e-4"}
        dtype = "bf16"
        if rank == 0 and world == 1 and not args.no_extras and not args.quick:
            fn, flops, desc = cpu_prefill_sample(w)
            sec = time_cpu(fn, 3, 1)
            r["cpu_baseline"] = {"value": flops / sec / 1e12, "unit": "TFLOP/s", "cores": O.num_threads(), "kind": "port",
                                 "sample": desc, "seconds_per_sample": sec}
            if args.workload == "cfg2":
                wd = W.cfg3()
                d = run_decode(wd, "cfg3")
                gotd = d.pop("_got"); d.pop("_q"); d.pop("_krange")
                wantd = np.stack([O.flash_attention(wd.q[b:b + 1], wd.k_dense[b][None], wd.v_dense[b][None], wd.scale)[0] for b in range(8)])
                errd = np.abs(gotd[:8] - wantd)
                d["parity"] = {"max_abs": float(errd.max()), "mean_abs": float(errd.mean()), "sequences_checked": 8}
                extras["decode"] = d
    else:
        if args.workload == "cfg3":
            w = W.cfg3(B=16) if args.small else W.cfg3()
            r = run_decode(w, "cfg3" + (" (scaled down)" if args.small else ""))
        else:
            w = W.cfg4(rank=rank, world=world)
            r = run_decode(w, "cfg4", shard_heads=False, chunked=True)
            if world > 1:
                r["config"]["sharding"] = (f"KV sequence split into {world} contiguous chunks, " +
                                           ("partials all-gathered over NCCL" if args.nccl_gather else
                                            "partial records pushed to every rank over peer memory and merged (no collective call)"))
                r["value"] = r["value"]  # bytes_all already counts every rank's chunk
        got = r.pop("_got"); qn = r.pop("_q"); k0, k1 = r.pop("_krange")
        r["parity"] = {"finite": bool(np.isfinite(got).all())}
        if rank == 0 and not args.quick:
            if args.workload == "cfg3":
                nb = min(8, qn.shape[0])
                want = np.stack([O.flash_attention(qn[b:b + 1], w.k_dense[b][None, k0:k1], w.v_dense[b][None, k0:k1], w.scale)[0]
                                 for b in range(nb)])
                err = np.abs(got[:nb] - want)
            else:
                wf = w if (world == 1 or fake_world) else W.cfg4()  # rank 0 rebuilds the whole sequence for the check
                want = O.flash_attention(wf.q, wf.k_dense[0][None], wf.v_dense[0][None], wf.scale)
                err = np.abs(got.reshape(want.shape) - want)
            r["parity"].update(max_abs=float(err.max()), mean_abs=float(err.mean()), tolerance="max 2e-3, mean 2e-4")
            if world == 1:
                fn, nbytes, desc = cpu_decode_sample(w, 4 if args.workload == "cfg3" else 1)
                sec = time_cpu(fn, 2, 1)
                r["cpu_baseline"] = {"value": nbytes / sec / 1e9, "unit": "GB/s", "cores": O.num_threads(), "kind": "port",
                                     "sample": desc, "seconds_per_sample": sec}
        dtype = "bf16"

    if rank == 0:
        if fake_world:
            r["config"]["shard_of"] = f"rank 0 of a {fake_world}-rank job on one GPU: value is extrapolated as {fake_world} x this shard"
        line = {"metric": METRIC, "value": r["value"], "unit": r["unit"], "n_gpus": 1 if fake_world else world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": dtype, "data": "synthetic (seeded N(0,1) rounded to bf16; random values, no weights)",
                "config": r["config"], "roofline": r["roofline"], "e2e": r.get("e2e"), "clocks": r.get("clocks"),
                "gpu_launches": r["gpu_launches"], "parity": r.get("parity")}
        if "cpu_baseline" in r:
            line["cpu_baseline"] = r["cpu_baseline"]
        line.update(extras)
        print(json.dumps(line))
    if use_dist:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
