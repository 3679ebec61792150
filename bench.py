#!/usr/bin/env python
"""Benchmark of the FastNN matmul path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference|reference_gpu]
                    [--workload square8192|linear_gelu|char_lm|attention|mnist_l1|...]

One "step" is one pass of the workload's GEMMs over synthetic, seeded operands.  The default
workload is the large square configuration: C = A.B (NN), A.B^T (NT) and A^T.B (TN) with
M = N = K = 8192, FP32 operands ~ N(0,1), TF32 multiply, FP32 accumulate.

* --impl ours       the hand-written sm_100a kernels behind the C ABI (libfastnn_b200.so).
                    `value` is measured with operands resident in HBM; `e2e` goes through the
                    same C ABI starting and ending in pinned host buffers.  At one GPU the line
                    also carries `configs`: every other configured GEMM shape, graph-timed.
* --impl reference  FastNN's CPU matmul (C restatement of its serial loop nest, rows split over
                    all host threads) on a bounded row slab of the same workload.
* --impl reference_gpu  FastNN's own cuda/kernels.cu (cuBLAS TF32) built for sm_100a, when that
                    library has been built; a comparator, never part of the product path.

Multi-GPU (torchrun, one rank per GPU).  `value` keeps 8192 rows per rank (weak scaling, no
collective on the data path).  The line of a multi-rank run adds two records:

* `parity`  before anything is timed, every rank checks rows of its shard of one NN, NT and TN
            product (TN through the column-slice shard) and of the K-sharded weight gradient
            against the CPU restatement, and that every rank holds the same gathered C;
* `strong`  the 8192-row problem split along M over the ranks, and the 32768-row fused Linear
            forward likewise: compute only, with the all-gather of C fused into the GEMM epilogue
            (peer stores over NVLink, then one barrier), and with a separate NCCL all-gather after
            the GEMM, each with its efficiency t1 / (N * tN) against the same run's one-GPU time.
"""
from __future__ import annotations

import argparse
import ctypes
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
NVLINK_PEER_GBS = 770.0          # measured peer copy per direction per GPU on this pool
BURST_SECONDS = 1.0              # timed regions shorter than this run at burst clocks
KERNEL_NAMES = {1: "gemm_simt_kernel", 2: "gemm_tf32_kernel", 3: "gemm_tf32_pair_kernel",
                6: "gemm_tf32_clusterk_kernel"}


# ------------------------------------------------------------------------- workloads ---

def workload_spec(name, rows_scale=1.0):
    """List of GEMMs of one step: dict(layout, m, n, k, batch, bias, act, label).

    FLOPs = 2 m n k batch; algorithmic bytes = each operand once, FP32."""
    def g(layout, m, n, k, batch=1, bias=False, act=0, label=""):
        return dict(layout=layout, m=int(m), n=int(n), k=int(k), batch=batch, bias=bias, act=act,
                    label=label)
    if name == "square8192":
        m = int(8192 * rows_scale)
        return [g(NN, m, 8192, 8192, label="NN"), g(NT, m, 8192, 8192, label="NT"),
                g(TN, m, 8192, 8192, label="TN")]
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


def tensor_roofline(flops, seconds_per_launch, region_seconds, peaks):
    """Tensor-bound roofline entry.  TF32 issues at half the BF16 rate, so the measured peak is half
    the measured BF16 GEMM figure: the burst one for a timed region shorter than BURST_SECONDS
    (the part has not yet settled under its power cap), the sustained one for longer regions."""
    ach = flops / seconds_per_launch / 1e12
    burst, sustained = peaks["bf16_burst"] / 2.0, peaks["bf16_sustained"] / 2.0
    use_burst = region_seconds < BURST_SECONDS
    peak = burst if use_burst else sustained
    out = {"bound": "tensor", "achieved": ach, "peak": peak, "unit": "TFLOP/s", "frac": ach / peak,
           "peak_source": (f"0.5 x {peaks['source']} bf16 {'burst' if use_burst else 'sustained'} "
                           f"{peaks['bf16_burst' if use_burst else 'bf16_sustained']} TFLOP/s "
                           f"(timed region {region_seconds:.3f} s {'<' if use_burst else '>='} {BURST_SECONDS} s)"),
           "frac_burst": ach / burst, "frac_sustained": ach / sustained,
           "frac_of_nominal_tf32": ach / NOMINAL_TF32_TFLOPS}
    if out["frac"] > 1.02:
        out["warning"] = "fraction above the roof: the peak does not fit this region's clocks"
    return out


def hbm_roofline(nbytes, seconds_per_launch, peaks):
    ach = nbytes / seconds_per_launch / 1e9
    return {"bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s",
            "frac": ach / peaks["hbm_gbs"], "peak_source": f"{peaks['source']} copy bandwidth"}


def ridge_flop_per_byte(peaks):
    return peaks["bf16_burst"] / 2.0 * 1e12 / (peaks["hbm_gbs"] * 1e9)


def load_traffic_table():
    """DRAM bytes per launch from the ncu captures summarised in profiles/dram_traffic.md: rows
    `| workload | kernel | gemm | plan | read bytes | write bytes | captured at |`.  A launch whose
    kernel or plan is not in the table has no traffic figure (null), never a stale one."""
    table = {}
    try:
        with open(os.path.join(ROOT, "profiles", "dram_traffic.md")) as fh:
            for line in fh:
                cells = [c.strip() for c in line.strip().strip("|").split("|")]
                if len(cells) != 7 or not cells[4].replace(",", "").isdigit():
                    continue
                table[(cells[0], cells[1], cells[2], cells[3])] = (
                    int(cells[4].replace(",", "")) + int(cells[5].replace(",", "")), cells[6])
    except OSError:
        pass
    return table


# -------------------------------------------------------------------- clock sampling ---

class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons every 50 ms on one GPU (read-only query)."""
    FIELDS = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows, self.proc = [], None
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


# ------------------------------------------------------------------ host placement ---

def bind_near_gpu(index):
    """Puts this process's threads and its future host allocations (the pinned staging buffers of
    the end-to-end path) on the NUMA node the GPU's PCIe root hangs off, when the machine says
    which one that is.  Eight ranks whose pinned buffers all sit on one socket share that socket's
    memory controllers and the inter-socket link.  Returns what was done, for the JSON line."""
    info = {"gpu_node": None, "cpus": None, "mempolicy": None}
    try:
        bus = subprocess.run(["nvidia-smi", f"--id={index}", "--query-gpu=pci.bus_id",
                              "--format=csv,noheader"], capture_output=True, text=True, timeout=10).stdout.strip()
        dom, rest = bus.split(":", 1)
        dev = f"{dom[-4:]}:{rest}".lower()
        with open(f"/sys/bus/pci/devices/{dev}/numa_node") as fh:
            node = int(fh.read().strip())
        info["gpu_node"] = node
        if node < 0:
            return info
        with open(f"/sys/devices/system/node/node{node}/cpulist") as fh:
            cpus = set()
            for part in fh.read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = os.sched_getaffinity(0) & cpus
        if allowed:
            os.sched_setaffinity(0, allowed)
            info["cpus"] = len(allowed)
        # set_mempolicy(MPOL_PREFERRED, {node}): new pages come from that node when it has room
        libc = ctypes.CDLL(None, use_errno=True)
        mask = ctypes.c_ulong(1 << node)
        rc = libc.syscall(238, 1, ctypes.byref(mask), ctypes.c_ulong(8 * ctypes.sizeof(mask)))
        info["mempolicy"] = "preferred" if rc == 0 else f"refused (errno {ctypes.get_errno()})"
    except Exception as exc:      # no sysfs entry, no permission: leave placement to the kernel
        info["mempolicy"] = info["mempolicy"] or f"unavailable ({type(exc).__name__})"
    return info


# ---------------------------------------------------------------------- GEMM helpers ---

def make_operands(torch, spec, gen, gen_b, small_weights=False):
    ops = []
    for s in spec:
        lay, m, n, k, b = s["layout"], s["m"], s["n"], s["k"], s["batch"]
        sa = (k, m) if lay == TN else (m, k)
        sb = (n, k) if lay == NT else (k, n)
        if b > 1:
            sa, sb = (b,) + sa, (b,) + sb
        a = torch.randn(sa, device="cuda", generator=gen)
        bm = torch.randn(sb, device="cuda", generator=gen if b > 1 else gen_b)
        if small_weights:
            bm = bm * 0.02
        c = torch.empty(((b,) if b > 1 else ()) + (m, n), device="cuda")
        bias = (torch.rand(n, device="cuda", generator=gen) * 0.02 - 0.01) if s["bias"] else None
        ops.append((s, a, bm, c, bias))
    return ops


def launch_op(f, op):
    s, a, bm, c, bias = op
    lay = s["layout"]
    if s["bias"] or s["act"]:
        f.linear_forward(a, bm, bias, act=s["act"], layout=lay, out=c)
    elif lay == NN:
        f.matmul(a, bm, out=c)
    elif lay == NT:
        f.matmul_nt(a, bm, out=c)
    else:
        f.matmul_tn(a, bm, out=c)


def launch_op_on(f, op, stream_ptr):
    s, a, bm, c, bias = op
    m, n, k, b, lay = s["m"], s["n"], s["k"], s["batch"], s["layout"]
    lda = m if lay == TN else k
    ldb = k if lay == NT else n
    f.gemm_ex(lay, a.data_ptr(), bm.data_ptr(), c.data_ptr(), m, n, k, b, lda, ldb, n,
              m * k, k * n, m * n, 1.0, 0.0, bias.data_ptr() if bias is not None else 0,
              s["act"], stream_ptr)


def plan_of(f):
    lp = f.last_path()
    return KERNEL_NAMES.get(lp["path"], "?"), f"bn{lp['block_n']} k/{lp['split_k']}", lp["num_ctas"]


def graph_time_us(torch, f, op, side):
    """Device time per launch of one GEMM replayed from a CUDA graph (no host call cost).
    Consecutive launches use different copies of the operands, enough of them that no launch
    finds its inputs (or the lines of its output) still in L2.  Every graph is replayed once
    untimed after instantiation (the first replay of a fresh graph uploads it)."""
    s0, a0, b0, c0, bias0 = op
    nring = ring_count(gemm_bytes(s0))
    ring = [op] + [(s0, a0.clone(), b0.clone(), torch.empty_like(c0), bias0) for _ in range(nring - 1)]
    reps = 20 if gemm_flops(s0) < 1e11 else 4
    reps = -(-reps // nring) * nring
    with torch.cuda.stream(side):
        launch_op_on(f, op, side.cuda_stream)          # the stream's split-K workspace exists
    side.synchronize()
    kernel, plan, ctas = plan_of(f)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        for i in range(reps):
            launch_op_on(f, ring[i % nring], torch.cuda.current_stream().cuda_stream)
    for _ in range(2):
        graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(3):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / (3 * reps) * 1e3, kernel, plan, ctas


def time_configs(torch, f, peaks, skip_workload):
    """Every configured GEMM shape outside the headline workload, graph-timed on this GPU:
    microseconds, TFLOP/s, GB/s of algorithmic bytes, the roofline that bounds it and the plan."""
    out = {}
    side = torch.cuda.Stream()
    ridge = ridge_flop_per_byte(peaks)
    for wl, tag in (("mnist_l1", "cfg1"), ("char_lm", "cfg2"), ("attention", "cfg3"),
                    ("square8192", "cfg4"), ("linear_gelu", "cfg5")):
        if wl == skip_workload:
            continue
        gen = torch.Generator(device="cuda").manual_seed(7000)
        spec = workload_spec(wl)
        for s in spec:
            op = make_operands(torch, [s], gen, gen, small_weights=(wl == "char_lm"))[0]
            us, kernel, plan, ctas = graph_time_us(torch, f, op, side)
            sec = us * 1e-6
            tensor = gemm_flops(s) / gemm_bytes(s) >= ridge
            frac = (gemm_flops(s) / sec / 1e12) / (peaks["bf16_burst"] / 2.0) if tensor else \
                (gemm_bytes(s) / sec / 1e9) / peaks["hbm_gbs"]
            out[f"{tag} {s['label']}"] = {
                "shape": f"{s['m']}x{s['n']}x{s['k']}" + (f"x{s['batch']}" if s["batch"] > 1 else ""),
                "us": round(us, 2), "tflops": round(gemm_flops(s) / sec / 1e12, 2),
                "gbs": round(gemm_bytes(s) / sec / 1e9, 1), "bound": "tensor" if tensor else "hbm",
                "frac": round(frac, 4), "plan": f"{kernel} {plan} ctas{ctas}"}
            del op
        torch.cuda.empty_cache()
    return out


# ------------------------------------------------------------- multi-GPU: parity, strong ---

def multi_gpu_parity(torch, dist, f, sharding, oracle, rank, world):
    """Every rank checks, against the CPU restatement, rows of its own shard of one NN, NT and TN
    product of the 8192-row problem (TN through the column-slice shard), rows of other ranks'
    shards as they arrive through the fused gather, and its rows of the K-sharded weight
    gradient.  Returns one dict, the same on every rank (the minimum over ranks decides)."""
    import numpy as np
    m = n = k = 8192
    gen = torch.Generator(device="cuda").manual_seed(4242)          # same operands on every rank
    a = torch.randn(m, k, device="cuda", generator=gen)
    b = torch.randn(k, n, device="cuda", generator=gen)
    b_host = b.cpu().numpy()
    r0, r1 = sharding.row_partition(m, world, rank)
    rows_own = list(range(r0, min(r0 + 32, r1))) + list(range(max(r1 - 32, r0), r1))
    other = (rank + 1) % world
    q0, q1 = sharding.row_partition(m, world, other)
    rows_other = list(range(q0, min(q0 + 8, q1)))
    threads = max(1, oracle.host_threads() // world)
    out = sharding.GatheredOutput((m, n))
    res = {}
    ok_all = True
    worst = 0.0
    rows = rows_own + rows_other
    a_rows = a[rows].cpu().numpy()          # the three layouts store the same A and B differently:
    want = oracle.matmul(a_rows, b_host, threads=threads)      # one expected product serves them all
    bound = 1e-2 * np.sqrt(k) * float(np.abs(a_rows).max()) * float(np.abs(b_host).max())
    for layout, name in ((NN, "NN"), (NT, "NT"), (TN, "TN")):
        # A as stored for this layout: [m,k] for NN/NT, [k,m] for TN; B [k,n], or [n,k] for NT
        a_st = a.t().contiguous() if layout == TN else a
        b_st = b.t().contiguous() if layout == NT else b
        shard = sharding.shard_left_operand(layout, a_st, world, rank)
        out.tensor.fill_(float("nan"))
        out.barrier()
        sharding.sharded_matmul_gathered(layout, shard, b_st, out)
        out.barrier()
        got = out.tensor[rows].cpu().numpy()
        err = np.abs(got.astype(np.float64) - want)
        rel = float(np.linalg.norm(err) / np.linalg.norm(want))
        ok = bool(np.isfinite(got).all() and rel <= 5e-3 and err.max() <= bound)
        # every rank must hold the same C: compare a checksum of the whole buffer across ranks
        chk = out.tensor.double().sum().reshape(1)
        chks = [torch.empty_like(chk) for _ in range(world)]
        dist.all_gather(chks, chk)
        same = all(bool(torch.equal(c, chks[0])) for c in chks) and bool(torch.isfinite(chk).all())
        res[name] = {"rel_fro": rel, "max_abs": float(err.max()), "rows_checked": len(rows)}
        ok_all = ok_all and ok and same
        worst = max(worst, rel)
        del a_st, b_st, shard
    del out, a, b
    # K-sharded weight gradient (the contraction dimension split over ranks, partial tiles stored
    # into the owning rank's memory by the GEMM epilogue, fixed-order reduce)
    gm, gn, kr = 1024, 512, 2048
    gen = torch.Generator(device="cuda").manual_seed(4343)
    x_full = torch.randn(kr * world, gm, device="cuda", generator=gen)
    dy_full = torch.randn(kr * world, gn, device="cuda", generator=gen)
    xl = x_full[rank * kr:(rank + 1) * kr].contiguous()
    dyl = dy_full[rank * kr:(rank + 1) * kr].contiguous()
    ws = sharding.KShardedGradWorkspace(gm, gn)
    mine = sharding.k_sharded_matmul_tn(xl, dyl, workspace=ws, fused=True)
    g0, g1 = sharding.row_partition(gm, world, rank)
    nrows = min(64, g1 - g0)
    x_cols = x_full[:, g0:g0 + nrows].contiguous().cpu().numpy()
    want = oracle.matmul_tn(x_cols, dy_full.cpu().numpy())
    got = mine[:nrows].cpu().numpy()
    err = np.abs(got.astype(np.float64) - want)
    rel = float(np.linalg.norm(err) / np.linalg.norm(want))
    bound = 1e-2 * np.sqrt(kr * world) * float(np.abs(x_cols).max()) * float(dy_full.abs().max())
    ok_all = ok_all and bool(np.isfinite(got).all() and rel <= 5e-3 and err.max() <= bound)
    res["dW_ksharded"] = {"rel_fro": rel, "max_abs": float(err.max()), "rows_checked": nrows}
    del ws, x_full, dy_full
    flag = torch.tensor([1 if ok_all else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    worst_t = torch.tensor([worst], device="cuda")
    dist.all_reduce(worst_t, op=dist.ReduceOp.MAX)
    torch.cuda.empty_cache()
    return {"ok": bool(flag.item() == 1), "ranks": world, "rank0": res,
            "worst_rel_fro_any_rank": float(worst_t.item()),
            "rule": "rel Frobenius <= 5e-3 and max-abs <= 1e-2 sqrt(K) max|A| max|B| on 64 own + 8 gathered rows "
                    "per layout and rank; gathered C checksum identical on all ranks",
            "oracle": "CPU restatement of FastNN's matmul loop"}


def strong_scaling(torch, dist, f, sharding, rank, world, reps=10):
    """The configured multi-GPU cases: a fixed problem split along M over the ranks, every C wanted
    on every rank.  Per GEMM: t1 (the whole problem on one GPU, timed on every rank at the same
    moment, max taken), compute only, the gather fused into the epilogue (+ one barrier among the
    ranks per GEMM), and GEMM followed by an NCCL all-gather.  Device time, max over ranks."""
    def timed(fn, n_rep=reps):
        for _ in range(2):
            fn()
        dist.barrier(); torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n_rep):
            fn()
        e1.record()
        dist.barrier(); torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / n_rep], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    results = {}
    for wl, pick, tag in (("square8192", None, "cfg4"), ("linear_gelu", 0, "cfg5 fwd")):
        spec = workload_spec(wl)
        if pick is not None:
            spec = [spec[pick]]
        gen = torch.Generator(device="cuda").manual_seed(2000)        # same operands on every rank
        per = {}
        for s in spec:
            lay, m, n, k = s["layout"], s["m"], s["n"], s["k"]
            full_op = make_operands(torch, [s], gen, gen)[0]
            _, a, bm, _, bias = full_op
            t1 = timed(lambda: launch_op(f, full_op))
            full_op = None                                  # drops the one-GPU C
            shard = sharding.shard_left_operand(lay, a, world, rank)
            r0, r1 = sharding.row_partition(m, world, rank)
            c_loc = torch.empty(r1 - r0, n, device="cuda")
            lda = a.stride(0)
            ldb = k if lay == NT else n
            stream = f.current_stream_ptr()

            def compute_only():
                f.gemm_ex(lay, shard.data_ptr(), bm.data_ptr(), c_loc.data_ptr(), r1 - r0, n, k, 1, lda, ldb, n,
                          0, 0, 0, 1.0, 0.0, bias.data_ptr() if bias is not None else 0, s["act"], stream)
            t_cmp = timed(compute_only)
            out = sharding.GatheredOutput((m, n))

            def fused(multicast):
                def run():
                    sharding.sharded_matmul_gathered(lay, shard, bm, out, bias=bias, act=s["act"],
                                                     multicast=multicast)
                    out.barrier()
                return run
            t_uni = timed(fused(False))
            t_mc = timed(fused(True)) if out.mc_ptr != 0 else None
            by_switch = False                                # the library's default: unicast peer stores
            t_fused = t_uni
            full = out.tensor          # reuse the buffer as the NCCL destination

            def unfused():
                compute_only()
                dist.all_gather_into_tensor(full, c_loc)
            t_nccl = timed(unfused)

            def gather_only():
                dist.all_gather_into_tensor(full, c_loc)
            t_ag = timed(gather_only)
            flops = gemm_flops(s)
            # every rank takes in the other ranks' shards: (world-1)/world of C over NVLink
            ingest = 4.0 * m * n * (world - 1) / world
            t_link = ingest / (NVLINK_PEER_GBS * 1e9) * 1e3
            per[s["label"]] = {
                "t1_ms": t1, "compute_only_ms": t_cmp, "with_gather_ms": t_fused,
                "gather_by": "multimem.st through the switch" if by_switch else "TMA stores to each peer",
                "peer_stores_ms": t_uni, "multicast_stores_ms": t_mc,
                "gemm_then_nccl_allgather_ms": t_nccl, "allgather_ms": t_ag,
                "compute_only_tflops": flops / (t_cmp * 1e-3) / 1e12,
                "with_gather_tflops": flops / (t_fused * 1e-3) / 1e12,
                "gemm_then_nccl_allgather_tflops": flops / (t_nccl * 1e-3) / 1e12,
                "compute_only_efficiency": t1 / (world * t_cmp),
                "with_gather_efficiency": t1 / (world * t_fused),
                "gemm_then_nccl_allgather_efficiency": t1 / (world * t_nccl),
                "nvlink_ingest_ms_at_770GBs": t_link,
                "with_gather_frac_of_bound": max(t_link, t1 / world) / t_fused,
                "plan": "%s %s ctas%d" % plan_of(f)}
            del out, full, c_loc, shard, a, bm
            torch.cuda.empty_cache()
        tot = {key: sum(v[key] for v in per.values()) for key in
               ("t1_ms", "compute_only_ms", "with_gather_ms", "gemm_then_nccl_allgather_ms")}
        results[tag] = {
            "gemms": per,
            "compute_only_efficiency": tot["t1_ms"] / (world * tot["compute_only_ms"]),
            "with_gather_efficiency": tot["t1_ms"] / (world * tot["with_gather_ms"]),
            "gemm_then_nccl_allgather_efficiency": tot["t1_ms"] / (world * tot["gemm_then_nccl_allgather_ms"]),
            "compute_only_tflops": sum(gemm_flops(s) for s in spec) / (tot["compute_only_ms"] * 1e-3) / 1e12,
            "with_gather_tflops": sum(gemm_flops(s) for s in spec) / (tot["with_gather_ms"] * 1e-3) / 1e12}
    results["how"] = ("rows of C split over the ranks, B replicated; with_gather = every finished tile sent by the GEMM "
                      "epilogue into all ranks' C + one barrier per GEMM: one TMA store per peer (the default, "
                      "peer_stores_ms = with_gather_ms); the optional form, one multimem.st through the NVSwitch, "
                      "is timed beside it (multicast_stores_ms); efficiency = t1 / (N * tN), t1 timed in "
                      "this run; bound = max(t1 / N, NVLink ingest)")
    return results


# -------------------------------------------------------------------------- our arm ---

def run_ours(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist
    import fastnn_b200 as f
    from fastnn_b200 import sharding

    affinity0 = os.sched_getaffinity(0)
    numa = bind_near_gpu(local_rank) if not args.no_e2e else None
    torch.cuda.set_device(local_rank)
    f.cuda_init(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    spec = workload_spec(args.workload)

    parity = None
    if world > 1 and not args.no_strong:
        import oracle
        parity = multi_gpu_parity(torch, dist, f, sharding, oracle, rank, world)

    gen = torch.Generator(device="cuda").manual_seed(1000 + rank)     # this rank's rows / batches
    gen_b = torch.Generator(device="cuda").manual_seed(2000)         # replicated operand
    ops = make_operands(torch, spec, gen, gen_b, small_weights=(args.workload == "char_lm"))

    # When one step touches less than a few L2 sizes, successive steps run on different copies of
    # the operands, so that no GEMM of the timed region finds its inputs in L2.
    step_ring = [ops]
    for _ in range(ring_count(sum(gemm_bytes(s) for s in spec)) - 1):
        step_ring.append([(s, a.clone(), bm.clone(), torch.empty_like(c), bias) for s, a, bm, c, bias in ops])
    step_no = [0]

    def step():
        for op in step_ring[step_no[0] % len(step_ring)]:
            launch_op(f, op)
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

    # which kernel and plan every GEMM of the step takes, and per-GEMM device time: large GEMMs
    # round-robin (one launch of each per turn, an event pair around every launch; timed one after
    # the other, whichever came last measured 10-15 % slower on this power-capped part, for this
    # library and for cuBLAS alike), small ones back to back
    kernel_names, plans, plan_keys, per_gemm = [], {}, [], []
    round_robin = min(gemm_flops(s) for s in spec) >= 1e11 and len(ops) > 1
    reps = max(3, min(20, args.steps))
    for op in ops:
        launch_op(f, op)
        kernel, plan, ctas = plan_of(f)
        kernel_names.append(kernel)
        plan_keys.append(plan)
        plans[op[0]["label"]] = f"{kernel} {plan} ctas{ctas}"
        if round_robin:
            continue
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(reps):
            launch_op(f, op)
        e1.record()
        torch.cuda.synchronize()
        per_gemm.append(e0.elapsed_time(e1) / reps)
    if round_robin:
        pairs = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                  for _ in ops] for _ in range(reps)]
        torch.cuda.synchronize()
        for turn in pairs:
            for op, (e0, e1) in zip(ops, turn):
                e0.record()
                launch_op(f, op)
                e1.record()
        torch.cuda.synchronize()
        per_gemm = [sum(turn[i][0].elapsed_time(turn[i][1]) for turn in pairs) / reps
                    for i in range(len(ops))]

    # the same launches replayed from a CUDA graph: device time without the host's per-call cost
    per_gemm_graph = None
    if not args.no_graph:
        side = torch.cuda.Stream()
        per_gemm_graph = [graph_time_us(torch, f, op, side)[0] * 1e-3 for op in ops]
        assert f.device_status() == 0

    e2e = None
    if not args.no_e2e:
        e2e = run_e2e(torch, dist, f, ops, spec, args, world, barrier)
        e2e["host_placement"] = numa
    os.sched_setaffinity(0, affinity0)                # the CPU baseline uses every core again

    strong = None
    if world > 1 and not args.no_strong:
        del step_ring
        torch.cuda.empty_cache()
        strong = strong_scaling(torch, dist, f, sharding, rank, world)
        assert f.device_status() == 0

    configs = None
    if world == 1 and not args.no_configs and rank == 0:
        peaks = load_peaks()
        try:
            del step_ring
        except NameError:
            pass
        torch.cuda.empty_cache()
        configs = time_configs(torch, f, peaks, args.workload)
        assert f.device_status() == 0

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    peaks = load_peaks()
    flops_step = sum(gemm_flops(s) for s in spec)
    value = flops_step * world * args.steps / (ms_total * 1e-3) / 1e12
    # Dominant kernel: every GEMM of a step is a launch of the same kernel.  When the launches
    # of a step do equal work (the square workload) its average duration is the timed region
    # divided by the launch count, measured live above; otherwise the roofline entry describes the
    # slowest GEMM of the step, timed on its own (graph replay when available).
    dev_ms = per_gemm_graph or per_gemm
    same_work = len({(s["m"], s["n"], s["k"], s["batch"]) for s in spec}) == 1 and launches == len(spec) * args.steps
    top = max(range(len(spec)), key=lambda i: dev_ms[i])
    ts = spec[top]
    top_ms = (ms_total / launches) if same_work else dev_ms[top]
    region_s = ms_total * 1e-3 if same_work else 0.0      # a graph replay of one GEMM is a burst
    if gemm_flops(ts) / gemm_bytes(ts) >= ridge_flop_per_byte(peaks):
        roof = tensor_roofline(gemm_flops(ts), top_ms * 1e-3, region_s, peaks)
    else:
        roof = hbm_roofline(gemm_bytes(ts), top_ms * 1e-3, peaks)
    roof["kernel"] = kernel_names[top]
    roof["gemm"] = ("all launches of the step" if same_work else
                    f"{ts['label']} m{ts['m']} n{ts['n']} k{ts['k']} b{ts['batch']}")
    roof["ms_per_launch"] = top_ms
    roof["timing"] = ("timed region / launches" if same_work else
                      ("graph replay of that GEMM" if per_gemm_graph else "back-to-back launches of that GEMM"))
    table = load_traffic_table()
    idx = range(len(spec)) if same_work else [top]
    hits = [table.get((args.workload, kernel_names[i], spec[i]["label"], plan_keys[i])) for i in idx]
    if all(h is not None for h in hits):
        roof["traffic"] = sum(h[0] for h in hits) / len(hits)
        roof["traffic_source"] = "ncu dram__bytes_read.sum + dram__bytes_write.sum, profiles/dram_traffic.md, " \
                                 "captured at " + ", ".join(sorted({h[1] for h in hits}))
    else:
        roof["traffic"] = None
        roof["traffic_source"] = "no capture of this kernel and plan in profiles/dram_traffic.md"
    roof["algorithmic_bytes"] = gemm_bytes(ts)
    if roof["bound"] == "tensor" and same_work and clocks and clocks.get("sm_mhz"):
        # what the tensor cores can do at the clock the power cap left during the timed region:
        # SMs x 4096 dense TF32 flop per clock x the median sampled SM clock
        sms = torch.cuda.get_device_properties(local_rank).multi_processor_count
        at_clock = sms * 4096 * clocks["sm_mhz"] * 1e6 / 1e12
        roof["tensor_peak_at_sampled_clock"] = at_clock
        roof["frac_of_peak_at_sampled_clock"] = roof["achieved"] / at_clock

    line = {
        "metric": "gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_total / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "tf32",
        "data": "synthetic",
        "config": {"workload": args.workload,
                   "gemms": [f"{s['label']}:{s['m']}x{s['n']}x{s['k']}" +
                             (f"x{s['batch']}" if s["batch"] > 1 else "") for s in spec],
                   "partition": "rows of C (batch for batched GEMMs) per rank, B replicated; "
                                "8192 rows per rank in `value`, the 8192-row problem split over the ranks in `strong`",
                   "l2": "operands larger than L2" if max(gemm_bytes(s) for s in spec) > 3 * 126e6
                   else ("a step touches %.0f MB across its GEMMs; graph timings rotate over operand "
                         "copies totalling >= 384 MB between reuses" % (sum(gemm_bytes(s) for s in spec) / 1e6))},
        "per_gemm_ms": {s["label"]: t for s, t in zip(spec, per_gemm)},
        "per_gemm_tflops": {s["label"]: gemm_flops(s) / (t * 1e-3) / 1e12 for s, t in zip(spec, per_gemm)},
        "plans": plans,
        "per_gemm_graph_us": ({s["label"]: t * 1e3 for s, t in zip(spec, per_gemm_graph)}
                              if per_gemm_graph else None),
        "roofline": roof, "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks,
    }
    if parity is not None:
        line["parity"] = parity
    if strong is not None:
        line["strong"] = strong
    if configs is not None:
        line["configs"] = configs
    if world == 1:
        line["cpu_baseline"] = None if args.no_cpu_baseline else cpu_baseline(args.workload, target_s=args.cpu_seconds)
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_e2e(torch, dist, f, ops, spec, args, world, barrier):
    """End to end through the C ABI: pinned host operands -> device -> GEMMs -> host results."""
    lib = f.lib()
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
            launch_op(f, (s, a, bm, c, bias))
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
                launch_op_on(f, (s, da, db, dc, bias), s_cmp.cuda_stream)
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
    seconds = float(dt.item())
    return {"value": flops_step * pipe_steps / seconds / 1e12, "unit": "TFLOP/s",
            "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h), "steps": pipe_steps,
            "host_gbs_all_ranks": (h2d + d2h) * world * pipe_steps / seconds / 1e9,
            "how": "pinned host buffers -> fastnn_b200_memcpy_h2d_async -> GEMM -> "
                   "fastnn_b200_memcpy_d2h_async on three streams, two device slots",
            "sync_value": sync_value,
            "sync_how": "fastnn_cuda_memcpy_h2d -> GEMM -> fastnn_cuda_memcpy_d2h one after the other "
                        "(FastNN's synchronous copies)"}


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
        "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
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
        for _ in range(2):
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
    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
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


def _graph_us(torch, fn, sets, side, reps):
    nring = len(sets)
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
    fused = _graph_us(torch, lambda x, sp: f.attention_forward(x[0], x[1], x[2], scale=scale, causal=True,
                                                               out=x[3], stream=sp), sets, side, 2 * nring)
    gemm_s = _graph_us(torch, lambda x, sp: f.gemm_ex(NT, x[0].data_ptr(), x[1].data_ptr(), x[4].data_ptr(), t, t, d,
                                                      heads, d, d, t, t * d, t * d, t * t, 1.0, 0.0, 0, 0, sp),
                       sets, side, 2 * nring)
    gemm_o = _graph_us(torch, lambda x, sp: f.gemm_ex(NN, x[4].data_ptr(), x[2].data_ptr(), x[3].data_ptr(), t, d, t,
                                                      heads, t, d, d, t * t, t * d, t * d, 1.0, 0.0, 0, 0, sp),
                       sets, side, 2 * nring)
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

    t_fused, t_gemm, t_unfused = (_graph_us(torch, fn, sets, side, 2 * nring) for fn in (fused, gemm_only, unfused))
    t_fused_nb = _graph_us(torch, fused_no_bias_grad, sets, side, 2 * nring)
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
    padding 1, bias) and its two gradients against FastNN's own CUDA entries (im2col / col2im +
    cuBLAS per image, from oracle/_ref when built) and cuDNN through torch with TF32 allowed.
    Device time, CUDA events around 20 calls after warm-up (the reference entries take no stream)."""
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
    ci_t = ctypes.c_int
    vpp = lambda t: ctypes.c_void_p(t.data_ptr())
    if path is not None:
        ref = ctypes.CDLL(path)
        assert ref.fastnn_cuda_init(local_rank) == 0
        y2 = torch.empty_like(y)
        ref_us = timed(lambda: ref.fastnn_cuda_conv2d_forward(
            vpp(x), vpp(wt), ctypes.c_void_p(0), vpp(y2), ci_t(n), ci_t(ci), ci_t(co),
            ci_t(h), ci_t(w), ci_t(kh), ci_t(kw), ci_t(1), ci_t(1), ci_t(pad), ci_t(pad)), reps=3)
    go = torch.randn(n, co, h, w, device="cuda", generator=gen)
    gi, gw = torch.empty_like(x), torch.empty_like(wt)
    lib = f.lib()
    dims = (n, ci, co, h, w, h, w, kh, kw, 1, 1, pad, pad)
    bwd_data = timed(lambda: lib.fastnn_b200_conv2d_backward_data(vpp(go), vpp(wt), vpp(gi), *dims, None))
    bwd_weight = timed(lambda: lib.fastnn_b200_conv2d_backward_weight(vpp(x), vpp(go), vpp(gw), *dims, None))
    cudnn_bwd = timed(lambda: torch.ops.aten.convolution_backward(
        go, x, wt, None, [1, 1], [pad, pad], [1, 1], False, [0, 0], 1, [True, True, False]))
    cudnn_bwd_data = timed(lambda: torch.ops.aten.convolution_backward(
        go, x, wt, None, [1, 1], [pad, pad], [1, 1], False, [0, 0], 1, [True, False, False]))
    cudnn_bwd_weight = timed(lambda: torch.ops.aten.convolution_backward(
        go, x, wt, None, [1, 1], [pad, pad], [1, 1], False, [0, 0], 1, [False, True, False]))
    # stride 2 (the gather-form input gradient): 64 -> 128 channels, 56 x 56 -> 28 x 28
    go2 = torch.randn(n, co, 28, 28, device="cuda", generator=gen)
    dims2 = (n, ci, co, h, w, 28, 28, kh, kw, 2, 2, pad, pad)
    bwd_data_s2 = timed(lambda: lib.fastnn_b200_conv2d_backward_data(vpp(go2), vpp(wt), vpp(gi), *dims2, None))
    cudnn_bwd_data_s2 = timed(lambda: torch.ops.aten.convolution_backward(
        go2, x, wt, None, [2, 2], [pad, pad], [1, 1], False, [0, 0], 1, [True, False, False]))
    ref_bd = ref_bw = None
    if path is not None:
        idims = [ci_t(v) for v in dims]
        gi2, gw2 = torch.empty_like(x), torch.empty_like(wt)
        ref_bd = timed(lambda: ref.fastnn_cuda_conv2d_backward_data(vpp(go), vpp(wt), vpp(gi2), *idims), reps=3)
        ref_bw = timed(lambda: ref.fastnn_cuda_conv2d_backward_weight(vpp(x), vpp(go), vpp(gw2), *idims), reps=3)
    assert f.device_status() == 0
    print(json.dumps({
        "impl": "conv2d", "shape": f"N{n} C{ci}->{co} {h}x{w} k{kh}x{kw} p{pad}", "ours_us": ours,
        "ours_tflops": flops / ours / 1e6, "cudnn_tf32_us": cudnn, "cudnn_tflops": flops / cudnn / 1e6,
        "fastnn_cuda_entry_us_without_bias": ref_us, "rel_diff_vs_cudnn": rel,
        "backward_data_us": bwd_data, "backward_weight_us": bwd_weight,
        "cudnn_backward_both_us": cudnn_bwd, "cudnn_backward_data_us": cudnn_bwd_data,
        "cudnn_backward_weight_us": cudnn_bwd_weight,
        "backward_data_stride2_us": bwd_data_s2, "cudnn_backward_data_stride2_us": cudnn_bwd_data_s2,
        "fastnn_cuda_backward_data_us": ref_bd, "fastnn_cuda_backward_weight_us": ref_bw,
        "note": "FastNN's entry adds bias through one host copy and one launch per channel; timed without bias"}),
        flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=60)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference_gpu"])
    ap.add_argument("--workload", default="square8192")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-configs", action="store_true", help="skip the per-configuration table (one GPU)")
    ap.add_argument("--no-strong", action="store_true", help="skip parity and strong scaling (several GPUs)")
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
