#!/usr/bin/env python
"""Benchmark of the FastNN matmul path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference|reference_gpu]
                    [--workload square8192|linear_gelu|char_lm|attention|mnist_l1]
                    [--scaling weak|strong] [--gather]

One "step" is one pass of the workload's GEMMs over synthetic, seeded operands.  The default
workload is the large square configuration: C = A.B (NN), A.B^T (NT) and A^T.B (TN) with
M = N = K = 8192, FP32 operands ~ N(0,1), TF32 multiply, FP32 accumulate.

* --impl ours       the hand-written sm_100a kernels behind the C ABI (libfastnn_b200.so).
                    `value` is measured with operands resident in HBM; `e2e` goes through the
                    same C ABI starting and ending in pinned host buffers.
* --impl reference  FastNN's CPU matmul (C restatement of its serial loop nest, rows split over
                    all host threads) on a bounded row slab of the same workload.
* --impl reference_gpu  FastNN's own cuda/kernels.cu (cuBLAS TF32) built for sm_100a, when that
                    library has been built; a comparator, never part of the product path.

Multi-GPU (torchrun, one rank per GPU): the output rows M (or the batch) are partitioned over
the ranks with the other operand replicated -- no collective on the data path.  Weak scaling
(default) keeps 8192 rows per rank; --scaling strong splits 8192 rows over the ranks; --gather
adds an NCCL all-gather of the C shards (reported separately, never inside `value`).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

NN, NT, TN = 0, 1, 2
NOMINAL_TF32_TFLOPS = 1100.0     # dense, NVIDIA's per-GPU figure (half the 2:4-sparse number)
FALLBACK_BF16_TFLOPS = 1590.0
FALLBACK_HBM_GBS = 6650.0


# ------------------------------------------------------------------------- workloads ---

def workload_spec(name, rows_scale=1.0):
    """List of GEMMs of one step: dict(layout, m, n, k, batch, bias, act, name).

    FLOPs = 2 m n k batch; algorithmic bytes = each operand once, FP32."""
    def g(layout, m, n, k, batch=1, bias=False, act=0, label=""):
        return dict(layout=layout, m=int(m), n=int(n), k=int(k), batch=batch, bias=bias, act=act,
                    label=label)
    if name == "square8192":
        m = int(8192 * rows_scale)
        return [g(NN, m, 8192, 8192, label="NN"), g(NT, m, 8192, 8192, label="NT"),
                g(TN, m, 8192, 8192, label="TN")]
    if name == "square4096":        # small case of the same kernels, sized for profiler captures
        m = int(4096 * rows_scale)
        return [g(NN, m, 4096, 4096, label="NN"), g(NT, m, 4096, 4096, label="NT"),
                g(TN, m, 4096, 4096, label="TN")]
    if name == "linear_gelu":
        m = int(32768 * rows_scale)
        return [g(NN, m, 16384, 4096, bias=True, act=2, label="fwd NN+bias+GELU"),
                g(NT, m, 4096, 16384, label="dX NT"),
                g(TN, 4096, 16384, m, label="dW TN")]
    if name == "char_lm":
        m = int(8192 * rows_scale)
        out = []
        for k, n, tag in ((256, 768, "qkv"), (256, 256, "o"), (256, 1024, "ff1"), (1024, 256, "ff2")):
            out += [g(NN, m, n, k, label=f"{tag} fwd"), g(NT, m, k, n, label=f"{tag} dX"),
                    g(TN, k, n, m, label=f"{tag} dW")]
        return out
    if name == "attention":
        b = int(512 * rows_scale)
        return [g(NT, 128, 128, 32, batch=b, label="S=Q.K^T"), g(NN, 128, 32, 128, batch=b, label="O=P.V")]
    if name == "mnist_l1":
        return [g(NN, int(512 * rows_scale), 256, 784, bias=True, label="layer1")]
    raise SystemExit(f"unknown workload {name}")


def gemm_flops(s):
    return 2.0 * s["m"] * s["n"] * s["k"] * s["batch"]


def gemm_bytes(s):
    return 4.0 * s["batch"] * (s["m"] * s["k"] + s["k"] * s["n"] + s["m"] * s["n"]) + \
        (4.0 * s["n"] if s["bias"] else 0.0)


L2_TURNOVER_BYTES = 384e6          # three times the 126 MB L2


def ring_count(bytes_per_launch):
    """How many copies of a launch's operands a graph-timed loop rotates over so that the bytes
    touched between two uses of one copy exceed the L2 several times (1 for large launches)."""
    return int(max(1, min(128, -(-L2_TURNOVER_BYTES // max(1.0, bytes_per_launch)))))


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
            p = json.load(fh)
        return dict(source="measured", hbm_gbs=float(p["hbm_gbs"]),
                    bf16_burst=float(p["bf16_tflops"]),
                    bf16_sustained=float(p.get("bf16_tflops_sustained", p["bf16_tflops"])))
    except Exception:
        return dict(source="fallback", hbm_gbs=FALLBACK_HBM_GBS, bf16_burst=FALLBACK_BF16_TFLOPS,
                    bf16_sustained=1400.0)


# -------------------------------------------------------------------- clock sampling ---

class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons every 50 ms on one GPU."""
    FIELDS = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows, self.proc, self.t0 = [], None, None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), line.strip()))

    def stop(self, t_start, t_end):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        inside = [r for t, r in self.rows if t_start <= t <= t_end + 0.12] or [r for _, r in self.rows]
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in inside:
            parts = [x.strip() for x in r.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1])); mx.append(float(parts[2]))
            except ValueError:
                continue
            for nm, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# -------------------------------------------------------------------------- our arm ---

def run_ours(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist
    import fastnn_b200 as f

    torch.cuda.set_device(local_rank)
    f.cuda_init(local_rank)
    if args.policy or args.block_n or args.split_k:
        f.set_policy(args.policy, args.block_n, args.split_k)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    scale = (1.0 / world) if (args.scaling == "strong" and world > 1) else 1.0
    spec = workload_spec(args.workload, scale)
    if args.reverse:
        spec = spec[::-1]

    gen = torch.Generator(device="cuda").manual_seed(1000 + rank)     # this rank's rows / batches
    gen_b = torch.Generator(device="cuda").manual_seed(2000)         # replicated operand
    ops = []
    for s in spec:
        lay, m, n, k, b = s["layout"], s["m"], s["n"], s["k"], s["batch"]
        sa = (k, m) if lay == TN else (m, k)
        sb = (n, k) if lay == NT else (k, n)
        if b > 1:
            sa, sb = (b,) + sa, (b,) + sb
        a = torch.randn(sa, device="cuda", generator=gen)
        bm = torch.randn(sb, device="cuda", generator=gen if b > 1 else gen_b)
        if args.workload in ("char_lm",):
            bm = bm * 0.02
        c = torch.empty(((b,) if b > 1 else ()) + (m, n), device="cuda")
        bias = (torch.rand(n, device="cuda", generator=gen) * 0.02 - 0.01) if s["bias"] else None
        ops.append((s, a, bm, c, bias))

    def launch(s, a, bm, c, bias):
        lay = s["layout"]
        if s["bias"] or s["act"]:
            f.linear_forward(a, bm, bias, act=s["act"], layout=lay, out=c)
        elif lay == NN:
            f.matmul(a, bm, out=c)
        elif lay == NT:
            f.matmul_nt(a, bm, out=c)
        else:
            f.matmul_tn(a, bm, out=c)

    # When one step touches less than a few L2 sizes, successive steps run on different copies of
    # the operands, so that no GEMM of the timed region finds its inputs in L2.
    step_ring = [ops]
    for _ in range(ring_count(sum(gemm_bytes(s) for s in spec)) - 1):
        step_ring.append([(s, a.clone(), bm.clone(), torch.empty_like(c), bias) for s, a, bm, c, bias in ops])
    step_no = [0]

    def step():
        for op in step_ring[step_no[0] % len(step_ring)]:
            launch(*op)
        step_no[0] += 1

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        time.sleep(0.25)
    n0 = f.launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t_start = time.time()
    ev0.record()
    for _ in range(args.steps):
        step()
    ev1.record()
    barrier()
    t_end = time.time()
    launches = f.launch_count() - n0
    ms = torch.tensor([ev0.elapsed_time(ev1)], device="cuda")
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_total = float(ms.item())
    clocks = sampler.stop(t_start, t_end) if sampler else None
    assert f.device_status() == 0, "a kernel reported a bounded-wait timeout"

    # per-GEMM device time (own events, after the headline region) for the roofline entry
    per_gemm = []
    kernel_names = []
    plans = {}
    # Large GEMMs are timed round-robin (one launch of each per turn, an event pair around every
    # launch): timed one GEMM after the other, whichever came last measured 10-15 % slower on this
    # power-capped part, for this library and for cuBLAS alike, whatever its layout.
    round_robin = min(gemm_flops(s) for s in spec) >= 1e11 and len(ops) > 1
    for op in ops:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = max(3, min(20, args.steps))
        launch(*op)
        lp = f.last_path()
        kernel_names.append({1: "gemm_simt_kernel", 2: "gemm_tf32_kernel", 3: "gemm_tf32_pair_kernel",
                             6: "gemm_tf32_clusterk_kernel"}.get(lp["path"], "?"))
        plans[op[0]["label"]] = f"{kernel_names[-1]} bn{lp['block_n']} k/{lp['split_k']} ctas{lp['num_ctas']}"
        if round_robin:
            continue
        torch.cuda.synchronize()
        e0.record()
        for _ in range(reps):
            launch(*op)
        e1.record()
        torch.cuda.synchronize()
        per_gemm.append(e0.elapsed_time(e1) / reps)
    if round_robin:
        reps = max(3, min(20, args.steps))
        pairs = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                  for _ in ops] for _ in range(reps)]
        torch.cuda.synchronize()
        for turn in pairs:
            for op, (e0, e1) in zip(ops, turn):
                e0.record()
                launch(*op)
                e1.record()
        torch.cuda.synchronize()
        per_gemm = [sum(turn[i][0].elapsed_time(turn[i][1]) for turn in pairs) / reps
                    for i in range(len(ops))]

    # the same launches replayed from a CUDA graph: device time without the host's per-call cost
    # (matters for the small, HBM-bound GEMMs, where a Python call outlasts the kernel)
    per_gemm_graph = None
    if not args.no_graph:
        def launch_on(op, stream_ptr):
            s, a, bm, c, bias = op
            m, n, k, b, lay = s["m"], s["n"], s["k"], s["batch"], s["layout"]
            lda = m if lay == TN else k
            ldb = k if lay == NT else n
            f.gemm_ex(lay, a.data_ptr(), bm.data_ptr(), c.data_ptr(), m, n, k, b, lda, ldb, n,
                      m * k, k * n, m * n, 1.0, 0.0, bias.data_ptr() if bias is not None else 0,
                      s["act"], stream_ptr)
        per_gemm_graph = []
        side = torch.cuda.Stream()
        for op in ops:
            # consecutive launches use different copies of the operands, enough of them that no
            # launch finds its inputs (or the lines of its output) still in L2
            s0, a0, b0, c0, bias0 = op
            nring = ring_count(gemm_bytes(s0))
            ring = [op] + [(s0, a0.clone(), b0.clone(), torch.empty_like(c0), bias0)
                           for _ in range(nring - 1)]
            reps = 20 if gemm_flops(op[0]) < 1e11 else 4
            reps = -(-reps // nring) * nring
            with torch.cuda.stream(side):
                launch_on(op, side.cuda_stream)          # split-K workspace of this stream exists
            side.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for i in range(reps):
                    launch_on(ring[i % nring], torch.cuda.current_stream().cuda_stream)
            graph.replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(3):
                graph.replay()
            e1.record()
            torch.cuda.synchronize()
            per_gemm_graph.append(e0.elapsed_time(e1) / (3 * reps))
        assert f.device_status() == 0

    # end to end through the C ABI: pinned host operands -> device -> GEMMs -> host results
    e2e = None
    if not args.no_e2e:
        lib = f.lib()
        import ctypes
        host = []
        for s, a, bm, c, bias in ops:
            host.append((a.cpu().pin_memory(), bm.cpu().pin_memory(),
                         torch.empty(c.shape, dtype=torch.float32).pin_memory()))
        h2d = sum(h[0].numel() + h[1].numel() for h in host) * 4
        d2h = sum(h[2].numel() for h in host) * 4

        def vp(t):
            return ctypes.c_void_p(t.data_ptr())

        def e2e_step():
            for (s, a, bm, c, bias), (ha, hb, hc) in zip(ops, host):
                assert lib.fastnn_cuda_memcpy_h2d(vp(a), vp(ha), ha.numel() * 4) == 0
                assert lib.fastnn_cuda_memcpy_h2d(vp(bm), vp(hb), hb.numel() * 4) == 0
                launch(s, a, bm, c, bias)
                assert lib.fastnn_cuda_memcpy_d2h(vp(hc), vp(c), hc.numel() * 4) == 0

        e2e_steps = max(1, min(args.steps, args.e2e_steps))
        e2e_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_step()
        barrier()
        dt = torch.tensor([time.perf_counter() - t0], device="cuda", dtype=torch.float64)
        if world > 1:
            dist.all_reduce(dt, op=dist.ReduceOp.MAX)
        flops_step = sum(gemm_flops(s) for s in spec) * world
        sync_value = flops_step * e2e_steps / float(dt.item()) / 1e12

        # The same bytes through the stream-ordered entries: upload of GEMM j+1's operands, GEMM j
        # and download of result j-1 run at the same time on three streams over two device slots.
        s_in, s_cmp, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
        slots = [[(torch.empty_like(a), torch.empty_like(bm), torch.empty_like(c)) for _, a, bm, c, _ in ops]
                 for _ in range(2)]
        ev_in = [torch.cuda.Event() for _ in range(2)]
        ev_cmp = [torch.cuda.Event() for _ in range(2)]
        ev_out = [torch.cuda.Event() for _ in range(2)]

        def sp(stream):
            return ctypes.c_void_p(stream.cuda_stream)

        def launch_ex(s, a, bm, c, bias, stream):
            m, n, k, b, lay = s["m"], s["n"], s["k"], s["batch"], s["layout"]
            lda = m if lay == TN else k
            ldb = k if lay == NT else n
            f.gemm_ex(lay, a.data_ptr(), bm.data_ptr(), c.data_ptr(), m, n, k, b, lda, ldb, n,
                      m * k, k * n, m * n, 1.0, 0.0, bias.data_ptr() if bias is not None else 0,
                      s["act"], stream.cuda_stream)

        def e2e_pipelined(nsteps):
            j = 0
            for _ in range(nsteps):
                for i, ((s, _a, _b, _c, bias), (ha, hb, hc)) in enumerate(zip(ops, host)):
                    slot = j & 1
                    da, db, dc = slots[slot][i]
                    if j >= 2:
                        s_in.wait_event(ev_cmp[slot])        # GEMM j-2 has read this slot's operands
                    assert lib.fastnn_b200_memcpy_h2d_async(vp(da), vp(ha), ha.numel() * 4, sp(s_in)) == 0
                    assert lib.fastnn_b200_memcpy_h2d_async(vp(db), vp(hb), hb.numel() * 4, sp(s_in)) == 0
                    ev_in[slot].record(s_in)
                    s_cmp.wait_event(ev_in[slot])
                    if j >= 2:
                        s_cmp.wait_event(ev_out[slot])       # result j-2 has left this slot's C
                    launch_ex(s, da, db, dc, bias, s_cmp)
                    ev_cmp[slot].record(s_cmp)
                    s_out.wait_event(ev_cmp[slot])
                    assert lib.fastnn_b200_memcpy_d2h_async(vp(hc), vp(dc), hc.numel() * 4, sp(s_out)) == 0
                    ev_out[slot].record(s_out)
                    j += 1
            s_out.synchronize()

        e2e_pipelined(1)
        barrier()
        pipe_steps = max(e2e_steps, 8)
        t0 = time.perf_counter()
        e2e_pipelined(pipe_steps)
        barrier()
        dt = torch.tensor([time.perf_counter() - t0], device="cuda", dtype=torch.float64)
        if world > 1:
            dist.all_reduce(dt, op=dist.ReduceOp.MAX)
        e2e = {"value": flops_step * pipe_steps / float(dt.item()) / 1e12, "unit": "TFLOP/s",
               "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h), "steps": pipe_steps,
               "how": "pinned host buffers -> fastnn_b200_memcpy_h2d_async -> GEMM -> "
                      "fastnn_b200_memcpy_d2h_async on three streams, two device slots",
               "sync_value": sync_value,
               "sync_how": "fastnn_cuda_memcpy_h2d -> GEMM -> fastnn_cuda_memcpy_d2h one after the other "
                           "(FastNN's synchronous copies)"}
        del slots

    gather_ms = None
    if args.gather and world > 1:
        s, a, bm, c, bias = ops[0]
        full = torch.empty((world,) + tuple(c.shape), device="cuda")
        for _ in range(3):
            dist.all_gather_into_tensor(full, c)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(10):
            dist.all_gather_into_tensor(full, c)
        e1.record()
        barrier()
        g = torch.tensor([e0.elapsed_time(e1) / 10], device="cuda")
        dist.all_reduce(g, op=dist.ReduceOp.MAX)
        gather_ms = float(g.item())

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    peaks = load_peaks()
    flops_step = sum(gemm_flops(s) for s in spec)
    value = flops_step * world * args.steps / (ms_total * 1e-3) / 1e12
    # Dominant kernel: every GEMM of a step is a launch of the same kernel.  When the launches
    # of a step do equal work (the square workloads) its average duration is the timed region
    # divided by the launch count; otherwise the roofline entry describes the slowest GEMM of the
    # step, timed on its own (graph replay when available, so host call cost is excluded).
    dev_ms = per_gemm_graph or per_gemm
    same_work = len({(s["m"], s["n"], s["k"], s["batch"]) for s in spec}) == 1 and launches == len(spec) * args.steps
    top = max(range(len(spec)), key=lambda i: dev_ms[i])
    ts = spec[top]
    top_ms = (ms_total / launches) if same_work else dev_ms[top]
    ai = gemm_flops(ts) / gemm_bytes(ts)
    tf32_peak = peaks["bf16_sustained"] / 2.0
    ridge = tf32_peak * 1e12 / (peaks["hbm_gbs"] * 1e9)
    if ai >= ridge:
        ach = gemm_flops(ts) / (top_ms * 1e-3) / 1e12
        roof = {"bound": "tensor", "achieved": ach, "peak": tf32_peak, "unit": "TFLOP/s",
                "frac": ach / tf32_peak,
                "peak_source": f"0.5 x {peaks['source']} bf16 sustained {peaks['bf16_sustained']} TFLOP/s",
                "frac_of_nominal_tf32": ach / NOMINAL_TF32_TFLOPS}
    else:
        ach = gemm_bytes(ts) / (top_ms * 1e-3) / 1e9
        roof = {"bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": ach / peaks["hbm_gbs"], "peak_source": f"{peaks['source']} copy bandwidth"}
    roof["kernel"] = kernel_names[top]
    roof["gemm"] = ("all launches of the step" if same_work else
                    f"{ts['label']} m{ts['m']} n{ts['n']} k{ts['k']} b{ts['batch']}")
    roof["ms_per_launch"] = top_ms
    roof["timing"] = ("timed region / launches" if same_work else
                      ("graph replay of that GEMM" if per_gemm_graph else "back-to-back launches of that GEMM"))
    roof["traffic"] = traffic_for(args.workload, kernel_names, [s["label"] for s in spec], same_work, top)

    line = {
        "metric": "gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_total / args.steps,
        "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": "tf32",
        "data": "synthetic",
        "config": {"workload": args.workload,
                   "gemms": [f"{s['label']}:{s['m']}x{s['n']}x{s['k']}" +
                             (f"x{s['batch']}" if s["batch"] > 1 else "") for s in spec],
                   "partition": "rows of C (batch for batched GEMMs) per rank, B replicated",
                   "l2": "operands larger than L2" if max(gemm_bytes(s) for s in spec) > 3 * 126e6
                   else ("a step touches %.0f MB across its GEMMs; graph timings rotate over operand "
                         "copies totalling >= 384 MB between reuses" % (sum(gemm_bytes(s) for s in spec) / 1e6))},
        "per_gemm_ms": {s["label"]: t for s, t in zip(spec, per_gemm)},
        "per_gemm_tflops": {s["label"]: gemm_flops(s) / (t * 1e-3) / 1e12 for s, t in zip(spec, per_gemm)},
        "plans": plans,
        "per_gemm_graph_us": ({s["label"]: t * 1e3 for s, t in zip(spec, per_gemm_graph)}
                              if per_gemm_graph else None),
        "per_gemm_graph_gbs": ({s["label"]: gemm_bytes(s) / (t * 1e-3) / 1e9
                                for s, t in zip(spec, per_gemm_graph)} if per_gemm_graph else None),
        "roofline": roof, "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks,
    }
    if gather_ms is not None:
        line["allgather_ms"] = gather_ms
    if not args.no_cpu_baseline and world == 1:
        line["cpu_baseline"] = cpu_baseline(args.workload, target_s=args.cpu_seconds)
    elif world == 1:
        line["cpu_baseline"] = None
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# ncu-measured DRAM traffic per launch (dram__bytes_read.sum + dram__bytes_write.sum, bytes) of
# the GEMM kernels, from the captures summarised in profiles/; keyed by (workload, kernel, GEMM label)
TRAFFIC_BYTES = {
    ("square8192", "gemm_tf32_kernel", "NN"): 2.278e9 + 0.255e9,
    ("square8192", "gemm_tf32_kernel", "NT"): 2.278e9 + 0.253e9,
    ("square8192", "gemm_tf32_kernel", "TN"): 2.279e9 + 0.253e9,
    ("square8192", "gemm_tf32_pair_kernel", "NN"): 2.280e9 + 0.255e9,
    ("square8192", "gemm_tf32_pair_kernel", "NT"): 2.820e9 + 0.253e9,
    ("square8192", "gemm_tf32_pair_kernel", "TN"): 2.281e9 + 0.252e9,
    ("square4096", "gemm_tf32_pair_kernel", "NN"): 2.98e8 + 0.48e8,
    ("square4096", "gemm_tf32_pair_kernel", "NT"): 2.97e8 + 0.47e8,
    ("square4096", "gemm_tf32_pair_kernel", "TN"): 2.98e8 + 0.48e8,
    ("square4096", "gemm_tf32_kernel", "NN"): 2.93e8 + 0.51e8,
    ("square4096", "gemm_tf32_kernel", "NT"): 2.95e8 + 0.53e8,
    ("square4096", "gemm_tf32_kernel", "TN"): 2.93e8 + 0.51e8,
    # HBM-bound shapes: reads equal the operand bytes; the outputs (8-34 MB) stay in L2 as dirty
    # lines past the end of the launch, so the captured write side is 0
    ("char_lm", "gemm_tf32_kernel", "qkv fwd"): 9257728, ("char_lm", "gemm_tf32_kernel", "qkv dX"): 26034176,
    ("char_lm", "gemm_tf32_kernel", "qkv dW"): 33636096, ("char_lm", "gemm_tf32_kernel", "o fwd"): 8732416,
    ("char_lm", "gemm_tf32_kernel", "o dX"): 8732160, ("char_lm", "gemm_tf32_kernel", "o dW"): 16859136,
    ("char_lm", "gemm_tf32_kernel", "ff1 fwd"): 9519360, ("char_lm", "gemm_tf32_kernel", "ff1 dX"): 34684672,
    ("char_lm", "gemm_tf32_kernel", "ff1 dW"): 42024448 + 768, ("char_lm", "gemm_tf32_kernel", "ff2 fwd"): 34685440,
    ("char_lm", "gemm_tf32_kernel", "ff2 dX"): 9519104, ("char_lm", "gemm_tf32_kernel", "ff2 dW"): 42025216 + 1536,
    ("attention", "gemm_tf32_kernel", "S=Q.K^T"): 16859136, ("attention", "gemm_tf32_kernel", "O=P.V"): 42024960,
    ("mnist_l1", "gemm_tf32_clusterk_kernel", "layer1"): 2459904,
}


def traffic_for(workload, kernels, labels, same_work, top):
    """DRAM bytes per launch for the roofline entry: the mean over the step's launches when the
    entry describes all of them, else the figure of the GEMM it names; None when not captured."""
    idx = range(len(labels)) if same_work else [top]
    vals = [TRAFFIC_BYTES.get((workload, kernels[i], labels[i])) for i in idx]
    if any(v is None for v in vals):
        return None
    return sum(vals) / len(vals)


# -------------------------------------------------------------------- CPU reference ---

def cpu_baseline(workload, target_s=12.0, threads=None):
    """Times the CPU restatement of FastNN's matmul (rows split over host threads) on a row
    slab of the workload's first GEMM, sized for about `target_s` seconds."""
    import numpy as np
    import oracle
    t = threads or oracle.host_threads()
    s = workload_spec(workload)[0]
    m, n, k = s["m"], s["n"], s["k"]
    rng = np.random.default_rng(0)
    probe_rows = max(t, min(m, 2 * t))
    a = rng.standard_normal((max(probe_rows, 1), k), dtype=np.float32)
    b = rng.standard_normal((k, n), dtype=np.float32)
    t0 = time.perf_counter()
    oracle.matmul(a[:probe_rows], b, threads=t)
    dt = time.perf_counter() - t0
    rate = 2.0 * probe_rows * n * k / dt
    rows = int(min(m, max(probe_rows, target_s * rate / (2.0 * n * k))))
    rows = max(t, rows // t * t)
    a = rng.standard_normal((rows, k), dtype=np.float32)
    t0 = time.perf_counter()
    oracle.matmul(a, b, threads=t)
    dt = time.perf_counter() - t0
    val = 2.0 * rows * n * k / dt / 1e12
    return {"value": val, "unit": "TFLOP/s", "cores": t, "kind": "port",
            "sample": f"{rows} of {m} rows of the {s['label']} GEMM (n={n}, k={k}), {dt:.1f} s",
            "seconds": dt}


def run_reference(args, rank, world):
    if rank != 0:
        return
    import numpy as np
    import oracle
    t = oracle.host_threads()
    s = workload_spec(args.workload)[0]
    m, n, k = s["m"], s["n"], s["k"]
    rng = np.random.default_rng(0)
    b = rng.standard_normal((k, n), dtype=np.float32)
    a = rng.standard_normal((2 * t, k), dtype=np.float32)
    t0 = time.perf_counter()
    oracle.matmul(a, b, threads=t)
    rate = 2.0 * a.shape[0] * n * k / (time.perf_counter() - t0)
    budget = 150.0 / max(1, args.steps + args.warmup)          # whole run within a few minutes
    rows = int(min(m, max(t, min(budget, 10.0) * rate / (2.0 * n * k))))
    rows = max(t, rows // t * t)
    a = rng.standard_normal((rows, k), dtype=np.float32)
    for _ in range(args.warmup):
        oracle.matmul(a, b, threads=t)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle.matmul(a, b, threads=t)
    dt = time.perf_counter() - t0
    val = 2.0 * rows * n * k * args.steps / dt / 1e12
    sample = f"{rows} of {m} rows of the {s['label']} GEMM (n={n}, k={k}) per step"
    line = {
        "impl": "reference", "metric": "gemm_tflops", "value": val, "unit": "TFLOP/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": args.scaling,
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "sample": sample},
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": t, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_reference_gpu(args, rank, world, local_rank):
    """FastNN's own GPU library (cuBLAS TF32) on the same workload -- comparator only."""
    if rank != 0:
        return
    import ctypes
    import torch
    import oracle
    path = oracle.ref_gpu_library_path()
    if path is None:
        print(json.dumps({"impl": "reference_gpu", "unavailable": "oracle/_ref/libfastnn_ref.so not built"}))
        return
    torch.cuda.set_device(local_rank)
    lib = ctypes.CDLL(path)
    assert lib.fastnn_cuda_init(local_rank) == 0
    spec = workload_spec(args.workload)
    if args.reverse:
        spec = spec[::-1]
    gen = torch.Generator(device="cuda").manual_seed(1000)
    vp, ci, cf = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    out = {}
    for s in spec:
        lay, m, n, k, b = s["layout"], s["m"], s["n"], s["k"], s["batch"]
        a = torch.randn(b * m * k, device="cuda", generator=gen)
        bm = torch.randn(b * k * n, device="cuda", generator=gen)
        c = torch.empty(b * m * n, device="cuda")
        pa, pb, pc = vp(a.data_ptr()), vp(bm.data_ptr()), vp(c.data_ptr())

        def call():
            if b > 1:
                if lay == NN:
                    return lib.fastnn_cuda_matmul_batched(pa, pb, pc, ci(m), ci(n), ci(k), ci(b), cf(1), cf(0))
                name = "fastnn_cuda_matmul_batched_nt" if lay == NT else "fastnn_cuda_matmul_batched_tn"
                return getattr(lib, name)(pa, pb, pc, ci(m), ci(n), ci(k), ci(b))
            if lay == NN:
                return lib.fastnn_cuda_matmul(pa, pb, pc, ci(m), ci(n), ci(k), ci(k), ci(n), ci(n), cf(1), cf(0))
            name = "fastnn_cuda_matmul_nt" if lay == NT else "fastnn_cuda_matmul_tn"
            return getattr(lib, name)(pa, pb, pc, ci(m), ci(n), ci(k))
        for _ in range(max(3, args.warmup)):
            assert call() == 0
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            call()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / args.steps
        out[s["label"]] = {"ms": ms, "tflops": gemm_flops(s) / (ms * 1e-3) / 1e12,
                           "gbs": gemm_bytes(s) / (ms * 1e-3) / 1e9}
        # cuBLAS TF32 again through torch, replayed from a CUDA graph (no host call cost); the
        # reference's own entry points take no stream, so they cannot be captured
        torch.backends.cuda.matmul.allow_tf32 = True
        shp = ((b,) if b > 1 else ())
        A = a.view(*shp, *((k, m) if lay == TN else (m, k)))
        Bm = bm.view(*shp, *((n, k) if lay == NT else (k, n)))
        Av = A.transpose(-1, -2) if lay == TN else A
        Bv = Bm.transpose(-1, -2) if lay == NT else Bm
        C = c.view(*shp, m, n)
        nring = ring_count(gemm_bytes(s))              # same operand rotation as our own arm
        ring = [(Av, Bv, C)]
        for _ in range(nring - 1):
            A2, B2 = A.clone(), Bm.clone()
            ring.append((A2.transpose(-1, -2) if lay == TN else A2,
                         B2.transpose(-1, -2) if lay == NT else B2, torch.empty_like(C)))
        reps = 20 if gemm_flops(s) < 1e11 else 4
        reps = -(-reps // nring) * nring
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            torch.matmul(Av, Bv, out=C)
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for i in range(reps):
                ra, rb, rc = ring[i % nring]
                torch.matmul(ra, rb, out=rc)
        graph.replay()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(3):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        out[s["label"]]["torch_cublas_graph_us"] = e0.elapsed_time(e1) / (3 * reps) * 1e3
    print(json.dumps({"impl": "reference_gpu", "what": "FastNN cuda/kernels.cu (cuBLAS TF32; bias/activation not included)",
                      "workload": args.workload, "per_gemm": out}), flush=True)


def run_dw_ksharded(args, rank, world, local_rank):
    """Extra arm (needs >= 2 GPUs): the data-parallel weight gradient dW[4096,16384] = X^T . dY with
    the contraction dimension sharded over ranks (32768 rows of X and dY per rank).  Times the fused
    form (GEMM epilogues store partial tiles into the owning rank's symmetric memory over NVLink,
    then a fixed-order reduce) against local GEMM + NCCL all_reduce."""
    import torch
    import torch.distributed as dist
    import fastnn_b200 as f
    from fastnn_b200 import sharding
    torch.cuda.set_device(local_rank)
    f.cuda_init(local_rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    m, n, k = 4096, 16384, 32768
    gen = torch.Generator(device="cuda").manual_seed(1000 + rank)
    x = torch.randn(k, m, device="cuda", generator=gen)
    dy = torch.randn(k, n, device="cuda", generator=gen) * 1e-3
    ws = sharding.KShardedGradWorkspace(m, n)

    def timed(fn):
        for _ in range(args.warmup):
            fn()
        dist.barrier(); torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            fn()
        e1.record()
        dist.barrier(); torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / args.steps], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    fused_ms = timed(lambda: sharding.k_sharded_matmul_tn(x, dy, workspace=ws, fused=True))
    plain_ms = timed(lambda: sharding.k_sharded_matmul_tn(x, dy, fused=False))
    gemm_ms = timed(lambda: f.matmul_tn(x, dy))
    a = sharding.k_sharded_matmul_tn(x, dy, workspace=ws, fused=True)
    b = sharding.k_sharded_matmul_tn(x, dy, fused=False)
    err = ((a - b).norm() / b.norm()).item()
    assert f.device_status() == 0
    if rank == 0:
        flops = 2.0 * m * n * k * world
        print(json.dumps({
            "impl": "dw_ksharded", "n_gpus": world, "m": m, "n": n, "k_per_rank": k,
            "local_gemm_ms": gemm_ms, "fused_ms": fused_ms, "gemm_plus_allreduce_ms": plain_ms,
            "fused_tflops": flops / (fused_ms * 1e-3) / 1e12,
            "gemm_plus_allreduce_tflops": flops / (plain_ms * 1e-3) / 1e12,
            "exchange_bytes_per_rank": 4.0 * m * n * (world - 1) / world,
            "fused_vs_plain_rel_diff": err}), flush=True)
    dist.destroy_process_group()


def run_attention_fused(args, local_rank):
    """Extra arm: the fused attention core (512 heads, T = 128, head_dim 32, causal) against the
    two batched GEMMs it replaces.  Device time from CUDA graphs; bytes = Q, K, V, O once."""
    import torch
    import fastnn_b200 as f
    torch.cuda.set_device(local_rank)
    f.cuda_init(local_rank)
    heads, t, d = 512, 128, 32
    gen = torch.Generator(device="cuda").manual_seed(3000)
    byts = 4.0 * heads * t * d * 4
    # consecutive launches rotate over copies of Q, K, V, O (and of the score matrix for the
    # unfused GEMMs) so that no launch finds its operands in L2
    nring = ring_count(byts)
    sets = []
    for _ in range(nring):
        q = torch.randn(heads, t, d, device="cuda", generator=gen)
        k = torch.randn(heads, t, d, device="cuda", generator=gen)
        v = torch.randn(heads, t, d, device="cuda", generator=gen)
        sets.append((q, k, v, torch.empty_like(q), torch.empty(heads, t, t, device="cuda")))
    scale = 1.0 / d ** 0.5
    side = torch.cuda.Stream()

    def graph_us(fn, reps=2 * nring):
        with torch.cuda.stream(side):
            fn(sets[0], side.cuda_stream)
        side.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            for i in range(reps):
                fn(sets[i % nring], torch.cuda.current_stream().cuda_stream)
        g.replay(); torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(5):
            g.replay()
        e1.record(); torch.cuda.synchronize()
        return e0.elapsed_time(e1) / (5 * reps) * 1e3

    fused = graph_us(lambda x, sp: f.attention_forward(x[0], x[1], x[2], scale=scale, causal=True,
                                                        out=x[3], stream=sp))
    gemm_s = graph_us(lambda x, sp: f.gemm_ex(NT, x[0].data_ptr(), x[1].data_ptr(), x[4].data_ptr(), t, t, d,
                                              heads, d, d, t, t * d, t * d, t * t, 1.0, 0.0, 0, 0, sp))
    gemm_o = graph_us(lambda x, sp: f.gemm_ex(NN, x[4].data_ptr(), x[2].data_ptr(), x[3].data_ptr(), t, d, t,
                                              heads, t, d, d, t * t, t * d, t * d, 1.0, 0.0, 0, 0, sp))
    peaks = load_peaks()
    assert f.device_status() == 0
    print(json.dumps({
        "impl": "attention_fused", "heads": heads, "t": t, "head_dim": d, "causal": True,
        "fused_us": fused, "fused_gbs": byts / fused / 1e3, "fused_frac_of_hbm": byts / fused / 1e3 / peaks["hbm_gbs"],
        "unfused_gemms_only_us": gemm_s + gemm_o,
        "note": "unfused figure omits FastNN's scale, mask-add and softmax launches and their 3 x 33.5 MB temporaries",
        "algorithmic_bytes": byts}), flush=True)


def run_linear_backward(args, local_rank):
    """Extra arm: the fused backward epilogue on the configured transformer block's ff2 backward
    (rows 8192, dy [rows,256], W2 [256,1024], saved pre-activation [rows,1024], GELU): one launch
    (+ a small reduce) against this library's plain GEMM followed by the elementwise derivative
    and the row sum as separate passes (torch ops standing in for FastNN's gelu_backward and
    sum_axis kernels).  Device time from CUDA graphs over rotating operand copies."""
    import torch
    import fastnn_b200 as f
    torch.cuda.set_device(local_rank)
    f.cuda_init(local_rank)
    rows, out_f, in_f = 8192, 256, 1024
    gen = torch.Generator(device="cuda").manual_seed(4000)
    byts = 4.0 * (rows * out_f + out_f * in_f + 2 * rows * in_f + in_f)
    nring = ring_count(byts)
    sets = []
    for _ in range(nring):
        dy = torch.randn(rows, out_f, device="cuda", generator=gen)
        w = torch.randn(out_f, in_f, device="cuda", generator=gen) * 0.05
        pre = torch.randn(rows, in_f, device="cuda", generator=gen)
        sets.append((dy, w, pre, torch.empty(rows, in_f, device="cuda"), torch.empty(in_f, device="cuda")))
    side = torch.cuda.Stream()
    lib = f.lib()
    import ctypes
    vp = lambda t: ctypes.c_void_p(t.data_ptr())

    def fused(x, sp):
        assert lib.fastnn_b200_linear_backward_input(NN, vp(x[0]), vp(x[1]), vp(x[3]), rows, out_f, in_f, 2,
                                                     vp(x[2]), vp(x[4]), ctypes.c_void_p(sp)) == 0

    def fused_no_bias_grad(x, sp):
        assert lib.fastnn_b200_linear_backward_input(NN, vp(x[0]), vp(x[1]), vp(x[3]), rows, out_f, in_f, 2,
                                                     vp(x[2]), ctypes.c_void_p(0), ctypes.c_void_p(sp)) == 0

    def gemm_only(x, sp):
        f.gemm_ex(NN, x[0].data_ptr(), x[1].data_ptr(), x[3].data_ptr(), rows, in_f, out_f, 1,
                  out_f, in_f, in_f, 0, 0, 0, 1.0, 0.0, 0, 0, sp)

    def unfused(x, sp):
        gemm_only(x, sp)
        p = x[2]
        d = 0.5 * (1.0 + torch.erf(p * 0.7071067811865475)) + p * torch.exp(-0.5 * p * p) * 0.3989422804014327
        x[3].mul_(d)
        torch.sum(x[3], dim=0, out=x[4])

    def graph_us(fn, reps=2 * nring):
        with torch.cuda.stream(side):
            fn(sets[0], side.cuda_stream)
        side.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            for i in range(reps):
                fn(sets[i % nring], torch.cuda.current_stream().cuda_stream)
        g.replay(); torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(5):
            g.replay()
        e1.record(); torch.cuda.synchronize()
        return e0.elapsed_time(e1) / (5 * reps) * 1e3

    t_fused, t_gemm, t_unfused = graph_us(fused), graph_us(gemm_only), graph_us(unfused)
    t_fused_nb = graph_us(fused_no_bias_grad)
    peaks = load_peaks()
    assert f.device_status() == 0
    print(json.dumps({
        "impl": "linear_backward", "rows": rows, "out_features": out_f, "in_features": in_f, "act": "gelu",
        "fused_us": t_fused, "fused_gbs": byts / t_fused / 1e3, "fused_frac_of_hbm": byts / t_fused / 1e3 / peaks["hbm_gbs"],
        "fused_without_bias_grad_us": t_fused_nb, "gemm_only_us": t_gemm, "unfused_us": t_unfused,
        "note": "unfused = this library's GEMM + torch elementwise derivative (several kernels) + torch row sum",
        "algorithmic_bytes": byts}), flush=True)


def run_conv2d(args, local_rank):
    """Extra arm: Conv2d forward as an implicit GEMM (batch 32, 64 -> 128 channels, 56 x 56, 3 x 3,
    padding 1, bias) against FastNN's own CUDA entry (im2col + cuBLAS per image, from oracle/_ref
    when built) and cuDNN through torch with TF32 allowed.  Device time, CUDA events around 20
    calls after warm-up (the reference entry takes no stream, so no graph)."""
    import ctypes
    import torch
    import fastnn_b200 as f
    import oracle
    torch.cuda.set_device(local_rank)
    f.cuda_init(local_rank)
    n, ci, co, h, w, kh, kw, pad = 32, 64, 128, 56, 56, 3, 3, 1
    gen = torch.Generator(device="cuda").manual_seed(5000)
    x = torch.randn(n, ci, h, w, device="cuda", generator=gen)
    wt = torch.randn(co, ci, kh, kw, device="cuda", generator=gen) * 0.05
    b = torch.randn(co, device="cuda", generator=gen)
    y = torch.empty(n, co, h, w, device="cuda")
    flops = 2.0 * n * h * w * co * ci * kh * kw

    def timed(fn, reps=20):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record(); torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps * 1e3

    ours = timed(lambda: f.conv2d_forward(x, wt, b, padding=(pad, pad), out=y))
    torch.backends.cudnn.allow_tf32 = True
    cudnn = timed(lambda: torch.nn.functional.conv2d(x, wt, b, padding=pad))
    want = torch.nn.functional.conv2d(x, wt, b, padding=pad)
    rel = float((y - want).norm() / want.norm())
    ref_us = None
    path = oracle.ref_gpu_library_path()
    if path is not None:
        ref = ctypes.CDLL(path)
        assert ref.fastnn_cuda_init(local_rank) == 0
        vp, ci_t = ctypes.c_void_p, ctypes.c_int
        y2 = torch.empty_like(y)
        ref_us = timed(lambda: ref.fastnn_cuda_conv2d_forward(
            vp(x.data_ptr()), vp(wt.data_ptr()), vp(0), vp(y2.data_ptr()), ci_t(n), ci_t(ci), ci_t(co),
            ci_t(h), ci_t(w), ci_t(kh), ci_t(kw), ci_t(1), ci_t(1), ci_t(pad), ci_t(pad)), reps=3)
    # gradients: ours against FastNN's CUDA entries (col2im / im2col + cuBLAS per image) and cuDNN
    go = torch.randn(n, co, h, w, device="cuda", generator=gen)
    gi, gw = torch.empty_like(x), torch.empty_like(wt)
    lib = f.lib()
    vpp = lambda t: ctypes.c_void_p(t.data_ptr())
    dims = (n, ci, co, h, w, h, w, kh, kw, 1, 1, pad, pad)
    bwd_data = timed(lambda: lib.fastnn_b200_conv2d_backward_data(vpp(go), vpp(wt), vpp(gi), *dims, None))
    bwd_weight = timed(lambda: lib.fastnn_b200_conv2d_backward_weight(vpp(x), vpp(go), vpp(gw), *dims, None))
    cudnn_bwd = timed(lambda: torch.ops.aten.convolution_backward(
        go, x, wt, None, [1, 1], [pad, pad], [1, 1], False, [0, 0], 1, [True, True, False]))
    ref_bd = ref_bw = None
    if path is not None:
        ci_t = ctypes.c_int
        idims = [ci_t(v) for v in dims]
        gi2, gw2 = torch.empty_like(x), torch.empty_like(wt)
        ref_bd = timed(lambda: ref.fastnn_cuda_conv2d_backward_data(vpp(go), vpp(wt), vpp(gi2), *idims), reps=3)
        ref_bw = timed(lambda: ref.fastnn_cuda_conv2d_backward_weight(vpp(x), vpp(go), vpp(gw2), *idims), reps=3)
    assert f.device_status() == 0
    print(json.dumps({
        "backward_data_us": bwd_data, "backward_weight_us": bwd_weight,
        "cudnn_backward_both_us": cudnn_bwd, "fastnn_cuda_backward_data_us": ref_bd,
        "fastnn_cuda_backward_weight_us": ref_bw,
        "impl": "conv2d", "shape": f"N{n} C{ci}->{co} {h}x{w} k{kh}x{kw} p{pad}", "ours_us": ours,
        "ours_tflops": flops / ours / 1e6, "cudnn_tf32_us": cudnn, "cudnn_tflops": flops / cudnn / 1e6,
        "fastnn_cuda_entry_us_without_bias": ref_us, "rel_diff_vs_cudnn": rel,
        "note": "FastNN's entry adds bias through one host copy and one launch per channel; timed without bias"}),
        flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=60)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference_gpu"])
    ap.add_argument("--workload", default="square8192")
    ap.add_argument("--reverse", action="store_true",
                    help="run the step's GEMMs in reverse order (separates layout from position effects)")
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"])
    ap.add_argument("--gather", action="store_true")
    ap.add_argument("--policy", type=int, default=0,
                    help="kernel choice for sweeps: 0 planner, 3 single CTAs only, 4 CTA pairs only, "
                         "5 K-split clusters (--split-k = cluster size), 6 planner without them")
    ap.add_argument("--block-n", type=int, default=0, help="tile width for sweeps (0 = planner)")
    ap.add_argument("--split-k", type=int, default=0, help="K split for sweeps (0 = planner)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.workload == "attention_fused":
        if rank == 0:
            run_attention_fused(args, local_rank)
    elif args.workload == "linear_backward":
        if rank == 0:
            run_linear_backward(args, local_rank)
    elif args.workload == "conv2d":
        if rank == 0:
            run_conv2d(args, local_rank)
    elif args.workload == "dw_ksharded":
        if world < 2:
            print(json.dumps({"impl": "dw_ksharded", "unavailable": "needs at least two ranks (torchrun)"}))
            return
        run_dw_ksharded(args, rank, world, local_rank)
    elif args.impl == "reference":
        run_reference(args, rank, world)
    elif args.impl == "reference_gpu":
        run_reference_gpu(args, rank, world, local_rank)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
