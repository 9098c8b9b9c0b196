#!/usr/bin/env python
"""Benchmark of the hot path.  Headline: float x binary GEMM  C = A (alpha * sign(W)),  M = N = K = 16384.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--size n]

One "step" is one GEMM over the whole activation matrix (activation split + tensor-core kernel; on N > 1 GPUs
the weight columns are sharded over the ranks and the all-gather of the result is fused into the kernel's
epilogue, closed by a cross-GPU barrier).  The packed weights are prepared once before the timed region, as the
reference Session caches them.  Rank 0 prints ONE JSON line.  N > 1 is launched with torchrun (one rank per GPU,
NCCL): strong scaling of the fixed 16384^3 problem.

Besides the headline the line carries one block per benchmark configuration, each with its roofline fraction
and (at N = 1) the reference's CPU implementation timed on the host beside it:
  ternary_mlp_projection   float x ternary 4096 x 4096 x 11008, column-sharded at N > 1
  cnn.conv_layer_*         binary 3x3 convolution 64x14x14 -> 128, batch 4096 (batch-sharded) and batch 1
  cnn.resnet18_binary_224  binary ResNet-18-style network, the whole batch of 8192 images in micro-batches
  lenet_batch_sweep        the LeNet-style binary CNN through the C++ tbn::Session, batch 1 ... 65536 (N = 1)
  gemm_ladder              the square GEMM at 128 ... 4096 (N = 1)
  declared_fp16            the declared one-pass variant (fp16 activations, <= 1e-3), never the headline
Every multi-GPU result is compared with the CPU oracle on sampled rows (`parity`), outside the timed region.

`--impl reference` times the reference's own CPU code for this path (compiled from its sources as
oracle/_ref/libtbn_ref.so) on the host cores, on a bounded row sample of the same workload.
"""
import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# DRAM bytes of one gemm_tc_kernel launch measured with ncu (a profiler cannot run inside the benchmark):
# key = (size, mode, GPUs).
MEASURED_TRAFFIC = {(16384, "x2", 1): 5.45e9, (8192, "x2", 1): 0.648e9}

METRIC = "float x binary GEMM throughput (2*M*N*K / time)"
UNIT = "TFLOP/s"
PARITY_TOL = 1e-5


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons while the timed region runs.

    Reads only (NVML queries from a thread of this process every 5 ms, so that even a timed region of a few
    tens of milliseconds is covered); when NVML cannot be loaded, an `nvidia-smi -lms` child is used instead."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    REASON_BITS = (("sw_power_cap", 0x4), ("hw_slowdown", 0x8), ("sw_thermal_slowdown", 0x20),
                   ("hw_thermal_slowdown", 0x40))

    def __init__(self, gpu_index, pci_bus_id=None):
        self.gpu = gpu_index
        self.pci = pci_bus_id
        self.proc = None
        self.path = None
        self.thread = None
        self.stop_flag = threading.Event()
        self.sm, self.reasons, self.sm_max = [], set(), None

    def _nvml_loop(self, nv, handle):
        while not self.stop_flag.is_set():
            try:
                self.sm.append(float(nv.nvmlDeviceGetClockInfo(handle, nv.NVML_CLOCK_SM)))
                mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(handle))
                for name, bit in self.REASON_BITS:
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.005)

    def start(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            handle = None
            if self.pci:
                try:
                    handle = nv.nvmlDeviceGetHandleByPciBusId(self.pci.encode() if hasattr(self.pci, "encode") else self.pci)
                except Exception:
                    handle = None
            if handle is None:
                handle = nv.nvmlDeviceGetHandleByIndex(self.gpu)
            self.sm_max = float(nv.nvmlDeviceGetMaxClockInfo(handle, nv.NVML_CLOCK_SM))
            self.thread = threading.Thread(target=self._nvml_loop, args=(nv, handle), daemon=True)
            self.thread.start()
            return
        except Exception:
            self.thread = None
        fd, self.path = tempfile.mkstemp(suffix=".csv")
        os.close(fd)
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0, "source": None}
        if self.thread is not None:
            self.stop_flag.set()
            self.thread.join(timeout=2)
            if self.sm:
                out.update(sm_mhz=float(np.median(self.sm)), sm_max_mhz=self.sm_max, reasons=sorted(self.reasons),
                           samples=len(self.sm), source="nvml")
            return out
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for line in open(self.path):
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        if sm:
            out.update(sm_mhz=float(np.median(sm)), sm_max_mhz=float(max(mx)), reasons=sorted(reasons), samples=len(sm),
                       source="nvidia-smi")
        return out


# ======================================================================================================
# Host-side pieces: inputs, the oracle as checker, the reference as CPU baseline
# ======================================================================================================

def normal(seed, shape, sigma=1.0):
    """N(0, sigma) fp32 from numpy's default_rng(seed): the generator every configuration names."""
    a = np.random.default_rng(seed).standard_normal(shape, dtype=np.float32)
    return a if sigma == 1.0 else (a * np.float32(sigma)).astype(np.float32)


def oracle_rows(A_rows, W_deq, threads=None):
    """oracle.gemm_f32(A_rows, W_deq) with the rows spread over host threads (the C call releases the GIL)."""
    from oracle import cpu_oracle
    orc = cpu_oracle.Oracle()
    threads = max(1, min(threads or (os.cpu_count() or 1), A_rows.shape[0]))
    parts = np.array_split(np.arange(A_rows.shape[0]), threads)
    out = np.empty((A_rows.shape[0], W_deq.shape[1]), dtype=np.float32)

    def work(idx):
        if len(idx):
            out[idx] = orc.gemm_f32(np.ascontiguousarray(A_rows[idx]), W_deq)

    ts = [threading.Thread(target=work, args=(p,)) for p in parts]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    return out


def dequantise_binary(W, inplace=False):
    """alpha * sign(W) of a [K, N] weight matrix: sign by w > 0 (everything else -1, as tbn::quantize_to_binary),
    alpha = mean |W| per column summed sequentially in fp32 over k, the order of model.hpp:388-394 (vectorised
    across the columns, so every column sees exactly the sequential sum).  `inplace` overwrites W."""
    acc = np.zeros(W.shape[1], dtype=np.float32)
    for k in range(W.shape[0]):
        acc += np.abs(W[k])
    alpha = (acc / np.float32(W.shape[0])).astype(np.float32)
    out = W if inplace else np.empty_like(W)
    step = 1024
    for k0 in range(0, W.shape[0], step):
        blk = W[k0:k0 + step]
        out[k0:k0 + step] = np.where(blk > 0, alpha[None, :], -alpha[None, :])
    return out


def rel_l2(got, expect):
    got, expect = np.asarray(got, dtype=np.float64), np.asarray(expect, dtype=np.float64)
    return float(np.linalg.norm(got - expect) / max(np.linalg.norm(expect), 1e-300))


def check_sharded_result(sg, A_d, A_h, W_deq_fn, rows_seed, n_rows, torch, dist):
    """Parity of the sharded product with the CPU oracle, outside every timed region.  Every rank's result
    matrix is first filled with NaN; after ONE step plus the barrier, rank 0 and the last rank compare `n_rows`
    seeded rows of their own copy of C (all N columns: every rank's slab, i.e. what arrived over NVLink as well
    as what was computed locally) with oracle.gemm_f32 on the dequantised weights.  Returns the block printed
    as `parity` (rank 0 holds the merged result)."""
    world, rank = sg.world, sg.rank
    sg.C.fill_(float("nan"))
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    out = sg.run(A_d)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    rows = np.sort(np.random.default_rng(rows_seed).choice(sg.M, size=n_rows, replace=False))
    err, checked = -1.0, 0
    if rank in (0, world - 1):
        got = out[torch.from_numpy(rows).to(out.device)].cpu().numpy()
        expect = oracle_rows(A_h[rows], W_deq_fn())
        err = rel_l2(got, expect) if np.isfinite(got).all() else float("inf")
        checked = 1
    if world > 1:
        t = torch.tensor([err, float(checked)], dtype=torch.float64, device=out.device)
        every = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(every, t)
        errs = [float(e[0]) for e in every if float(e[1]) > 0]
    else:
        errs = [err]
    worst = max(errs)
    return {"rel_l2": worst, "rows": int(n_rows), "ranks_checked": len(errs), "tolerance": PARITY_TOL,
            "ok": bool(worst <= PARITY_TOL),
            "how": "C filled with NaN, one step + barrier, seeded rows of the full C on rank 0 and the last rank "
                   "against oracle.gemm_f32(A[rows], dequantised W)"}


def timed_host(fn, min_s=0.3, max_reps=1000):
    """Wall time of a host function: seconds per call, repeated until min_s has passed."""
    fn()
    reps, t0 = 0, time.perf_counter()
    while True:
        fn()
        reps += 1
        dt = time.perf_counter() - t0
        if dt >= min_s or reps >= max_reps:
            return dt / reps


def cpu_reference_arm(n, steps, warmup, threads, rows_per_thread):
    """Times the reference's CPU path on a row sample: per step, `threads` host threads each run
    tbn::qlinear_matmul_binary_blocked_packed on `rows_per_thread` rows of A against the full
    cached packed weight matrix (the reference itself is single-threaded; independent row blocks
    are the only way to use more cores without touching its code)."""
    from oracle import cpu_oracle
    ref = cpu_oracle.Reference()
    W = normal(1, (n, n))
    qb = ref.quantize_to_binary(W, 0.0)
    del W
    handle = ref.pack_binary_weights(qb)
    del qb
    rows = threads * rows_per_thread
    A = normal(0, (rows, n))
    blocks = [A[i * rows_per_thread:(i + 1) * rows_per_thread] for i in range(threads)]

    def one_step():
        ts = [threading.Thread(target=ref.qlinear_matmul_binary_packed, args=(b, handle, 1.0)) for b in blocks]
        for t in ts:
            t.start()
        for t in ts:
            t.join()

    for _ in range(warmup):
        one_step()
    t0 = time.perf_counter()
    for _ in range(steps):
        one_step()
    dt = time.perf_counter() - t0
    # The same sample through the reference's float GEMM (its exact fp32 evaluation of the product).
    Wd = np.where(normal(1, (n, n)) > 0, np.float32(1), np.float32(-1))
    frows = max(1, min(rows, 8))
    t1 = time.perf_counter()
    ref.gemm_f32(A[:frows], Wd)
    dtf = time.perf_counter() - t1
    ref.free_binary_weights(handle)
    return {
        "tflops": 2.0 * rows * n * n * steps / dt / 1e12,
        "ms_per_step": dt / steps * 1e3,
        "rows_per_step": rows,
        "float_gemm_tflops_1core": 2.0 * frows * n * n / dtf / 1e12,
    }


def cpu_baselines_other_configs():
    """The reference's own CPU code (oracle/_ref, one core like the reference) on the other configurations,
    each on a bounded sample.  Returns {config: cpu_baseline block}."""
    from oracle import cpu_oracle, graphs
    if not cpu_oracle.reference_available():
        return {}
    ref = cpu_oracle.Reference()
    out = {}
    # conv layer, batch 1: float tbn::conv2d on the dequantised weights, and the Session's quantised (S1) path
    net = graphs.conv_layer(batch=1)
    x = normal(0, (1, 64, 14, 14))
    wq = graphs.dequantise(net["inits"]["w"])
    p = (1, 1, 1, 1, 1, 1)
    s_float = timed_host(lambda: ref.conv2d_f32(x, wq, net["inits"]["b"], p), 0.5)
    spec, blob, iblob = graphs.to_spec(net, dequantised=True)
    shape = (1, 128, 14, 14)
    base = timed_host(lambda: ref.session_run(spec, blob, iblob, "input", x, "output", shape, True, repeats=1), 0.3)
    many = timed_host(lambda: ref.session_run(spec, blob, iblob, "input", x, "output", shape, True, repeats=21), 0.3)
    s_s1 = max((many - base) / 20.0, 1e-9)
    out["conv_layer"] = {
        "value": 1.0 / s_float, "unit": "images/s", "cores": 1, "kind": "reference",
        "sample": "batch 1 (the loops are linear in the batch): tbn::conv2d float on alpha*sign(W); beside it the "
                  "Session with quantisation on (cached packed weights, ternarised activations), per run after the first",
        "float_conv2d_ms_per_image": s_float * 1e3, "session_tbn_mode_ms_per_image": s_s1 * 1e3,
        "session_tbn_mode_images_per_s": 1.0 / s_s1}
    # LeNet through the reference Session, both modes, batch 1
    net = graphs.lenet(batch=1, seed=1)
    xin = np.random.default_rng(0).random((1, 1, 28, 28), dtype=np.float32)
    spec, blob, iblob = graphs.to_spec(net, dequantised=True)
    res = {}
    for quant in (False, True):
        base = timed_host(lambda: ref.session_run(spec, blob, iblob, "input", xin, "output", (1, 10), quant, repeats=1), 0.2)
        many = timed_host(lambda: ref.session_run(spec, blob, iblob, "input", xin, "output", (1, 10), quant, repeats=101), 0.2)
        res[quant] = max((many - base) / 100.0, 1e-9)
    out["lenet"] = {"value": 1.0 / res[False], "unit": "images/s", "cores": 1, "kind": "reference",
                    "sample": "batch 1 through the reference TBNModel::Session, per run after the first (weights cached): "
                              "quantisation off (float operators) = value; quantisation on beside it",
                    "session_float_ms": res[False] * 1e3, "session_tbn_mode_ms": res[True] * 1e3,
                    "session_tbn_mode_images_per_s": 1.0 / res[True]}
    # float x ternary projection: the reference has no true ternary product (its qlinear_matmul_ternary maps 0 to
    # +1), so the baseline is its float GEMM on the dequantised ternary weights, 8 rows of A
    M, K, N = 4096, 4096, 11008
    W = normal(1, (K, N))
    delta = np.float32(0.7) * np.abs(W).mean(dtype=np.float32)
    T = np.where(W > delta, np.float32(1), np.where(W < -delta, np.float32(-1), np.float32(0)))
    A = normal(0, (8, K))
    t0 = time.perf_counter()
    ref.gemm_f32(A, T)
    dt = time.perf_counter() - t0
    out["ternary_mlp_projection"] = {"value": 2.0 * 8 * K * N / dt / 1e12, "unit": UNIT, "cores": 1, "kind": "reference",
                                     "sample": "8 rows of A (of 4096) against the full 4096 x 11008 ternary weights "
                                               "through the reference's float tbn::gemm"}
    del W, T
    # ResNet-18: the reference Session with quantisation off on ONE 224 x 224 image (about 3.6 GFLOP of naive loops)
    net = graphs.resnet18(batch=1, seed=2, image=224, classes=1000)
    xin = normal(0, (1, 3, 224, 224))
    spec, blob, iblob = graphs.to_spec(net, dequantised=True)
    t0 = time.perf_counter()
    ref.session_run(spec, blob, iblob, "input", xin, "output", (1, 1000), False, repeats=1)
    dt = time.perf_counter() - t0
    out["resnet18"] = {"value": 1.0 / dt, "unit": "images/s", "cores": 1, "kind": "reference",
                       "sample": "one 224 x 224 image through the reference TBNModel::Session, quantisation off, "
                                 "including its one-time weight handling (a single run)", "s_per_image": dt}
    return out


# ======================================================================================================
# GPU blocks
# ======================================================================================================

class Ctx:
    pass


def device_timer(ctx):
    """-> timed(fn, reps): milliseconds per call on the device (CUDA events), max over ranks."""
    torch, dist = ctx.torch, ctx.dist
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def timed(fn, reps, warm=1):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        if ctx.world > 1:
            dist.barrier()
        ev0.record()
        for _ in range(reps):
            fn()
        ev1.record()
        torch.cuda.synchronize()
        ms = torch.tensor([ev0.elapsed_time(ev1) / reps], device=ctx.dev)
        if ctx.world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    return timed


def tensor_roofline(flops, ms, passes, peaks, note):
    """Roofline block of a tensor-pipe-bound kernel sequence: logical FLOP rate against pipe peak / passes."""
    peak = peaks["bf16_tflops"] / passes
    ach = flops / (ms * 1e-3) / 1e12
    return {"bound": "tensor", "achieved": ach, "peak": peak, "unit": "TFLOP/s", "frac": ach / peak,
            "peak_source": f"{peaks['source']} cuBLAS bf16 burst {peaks['bf16_tflops']} TFLOP/s / {passes} passes", "note": note}


def resnet_flops(net):
    """(binary-conv FLOPs, float-layer FLOPs) per image of a graph recipe, from its node list and shapes."""
    shapes = {k: tuple(v) for k, v in net["inputs"].items()}
    fb = ff = 0.0
    for n in net["nodes"]:
        op, a = n["op"], n["attrs"]
        x = shapes[n["inputs"][0]]
        if op == "Conv":
            w = net["inits"][n["inputs"][1]].shape
            st, pd = a.get("strides", [1, 1]), a.get("pads", [0, 0, 0, 0])
            oh = (x[2] + 2 * pd[0] - w[2]) // st[0] + 1
            ow = (x[3] + 2 * pd[1] - w[3]) // st[1] + 1
            fl = 2.0 * oh * ow * w[0] * w[1] * w[2] * w[3]
            if n["inputs"][1] in net["binary"]:
                fb += fl
            else:
                ff += fl
            shapes[n["outputs"][0]] = (x[0], w[0], oh, ow)
        elif op in ("MaxPool", "AveragePool"):
            ks, st, pd = a.get("kernel_shape", [2, 2]), a.get("strides", [2, 2]), a.get("pads", [0, 0, 0, 0])
            shapes[n["outputs"][0]] = (x[0], x[1], (x[2] + 2 * pd[0] - ks[0]) // st[0] + 1, (x[3] + 2 * pd[1] - ks[1]) // st[1] + 1)
        elif op == "GlobalAveragePool":
            shapes[n["outputs"][0]] = (x[0], x[1], 1, 1)
        elif op == "Flatten":
            shapes[n["outputs"][0]] = (x[0], int(np.prod(x[1:])))
        elif op == "Gemm":
            w = net["inits"][n["inputs"][1]].shape
            fl = 2.0 * w[0] * w[1]
            if n["inputs"][1] in net["binary"]:
                fb += fl
            else:
                ff += fl
            shapes[n["outputs"][0]] = (x[0], w[1])
        else:
            shapes[n["outputs"][0]] = x
    return fb, ff


def cnn_block(args, ctx):
    """Binary-CNN throughput, batch-sharded over the ranks with no collective: the 64x14x14 -> 128 3x3 conv layer
    at batch 4096 (and batch 1 for latency) and the binary ResNet-18-style network at 224x224 over the WHOLE batch
    of 8192 images in micro-batches.  Whole-job images/s = images of all ranks / max-over-ranks device time."""
    from fast_arm_tbcnn_b200 import graphs, sharding
    from fast_arm_tbcnn_b200.session import Session
    torch, capi, L, dev, rank, world = ctx.torch, ctx.capi, ctx.L, ctx.dev, ctx.rank, ctx.world
    timed = device_timer(ctx)
    peaks = ctx.peaks
    out = {}

    # ---- single conv layer, batch 4096 split across the ranks; inputs N(0,1) seed 0, weights N(0,0.05) seed 1
    net = graphs.conv_layer(batch=1)
    b0, b1 = sharding.batch_block(rank, world, 4096)
    x_all = normal(0, (4096, 64, 14, 14))
    x = torch.from_numpy(x_all[b0:b1]).to(dev)
    x1 = torch.from_numpy(x_all[:1]).to(dev)
    del x_all
    w = torch.from_numpy(net["inits"]["w"]).to(dev)
    bias = torch.from_numpy(net["inits"]["b"]).to(dev)
    order = capi.CONV_WEIGHTS_TAP_MAJOR
    words, alpha = L.quant_pack_binary(L.permute_filters(w), capi.LAYOUT_NK)
    ws, _ = L.conv_workspace(x.shape, 128, 3, 3, dev, order)
    y = torch.empty((b1 - b0, 128, 14, 14), device=dev)
    p = (1, 1, 1, 1, 1, 1)
    conv_call = lambda: L.conv2d_fxb(x, words, w.shape, p, alpha=alpha, bias=bias, workspace=ws, out=y, order=order)  # noqa: E731
    for _ in range(2):   # first launches (code upload) stay outside the per-kernel events
        conv_call()
    torch.cuda.synchronize()
    L.profile_read()
    L.profile_enable(True)
    ms = timed(conv_call, 10, warm=0)
    prof = L.profile_read()
    L.profile_enable(False)
    flops = 2.0 * 4096 * 196 * 128 * 576
    bytes_alg = 4096.0 * (64 + 128) * 196 * 4
    blk = {"images_per_s": 4096 / (ms * 1e-3), "ms": ms, "tflops": flops / (ms * 1e-3) / 1e12,
           "kernel_ms": prof["gemm_ms"] / max(prof["gemm_launches"], 1),
           "prepass_ms": prof["split_ms"] / max(prof["split_launches"], 1),
           "algorithmic_gbs": bytes_alg / (ms * 1e-3) / 1e9,
           "roofline": tensor_roofline(flops / world, ms, 2, peaks,
                                       "whole layer call per GPU (channels-last pre-pass + implicit-GEMM kernel), two bf16 "
                                       "terms; the HBM fraction of the same call is given beside it (the layer sits near the ridge)"),
           "data": "x N(0,1) default_rng(0), w N(0,0.05) default_rng(1)"}
    blk["roofline"]["hbm_frac"] = bytes_alg / world / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"]
    out["conv_layer_64x14x14_to_128_batch4096"] = blk
    # batch 1: latency of one call (device time between events, back-to-back calls)
    ws1, _ = L.conv_workspace(x1.shape, 128, 3, 3, dev, order)
    y1 = torch.empty((1, 128, 14, 14), device=dev)
    ms1 = timed(lambda: L.conv2d_fxb(x1, words, w.shape, p, alpha=alpha, bias=bias, workspace=ws1, out=y1, order=order), 50, warm=3)
    out["conv_layer_64x14x14_to_128_batch1"] = {
        "ms": ms1, "images_per_s": 1.0 / (ms1 * 1e-3), "bound": "launch latency (two short launches per call)",
        "roofline": {"bound": "hbm", "achieved": 160768 / (ms1 * 1e-3) / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": 160768 / (ms1 * 1e-3) / 1e9 / peaks["hbm_gbs"],
                     "tensor_frac": 2.890e7 / (ms1 * 1e-3) / 1e12 / (peaks["bf16_tflops"] / 2)}}
    del x, y, x1, y1

    # ---- binary ResNet-18-style CNN, 3x224x224, the whole batch of 8192 in micro-batches of `micro` images
    micro = args.resnet_microbatch
    total = args.resnet_batch
    b0, b1 = sharding.batch_block(rank, world, total)
    n_micro = max(1, (b1 - b0) // micro)
    net = graphs.resnet18(batch=micro, seed=2, image=224, classes=1000)
    fb, ff = resnet_flops(graphs.resnet18(batch=1, seed=2, image=224, classes=1000))
    sess = Session(net)
    sess.keep_intermediates = False
    # inputs: micro-batch j of this rank is drawn N(0,1) from default_rng(1000 + global micro-batch index)
    first = b0 // micro
    xs = torch.empty((n_micro, micro, 3, 224, 224), device=dev)
    for j in range(n_micro):
        xs[j].copy_(torch.from_numpy(normal(1000 + first + j, (micro, 3, 224, 224))))
    sess.set_input("input", xs[0])
    sess.run()          # prepares and caches the packed weights, grows the workspaces
    logits = torch.empty((n_micro, micro, 1000), device=dev)

    def eager_pass():
        for j in range(n_micro):
            sess.set_input("input", xs[j])
            sess.run()
            logits[j].copy_(sess.get_output("output"))

    ms_eager = timed(eager_pass, 1)
    ms_pass, how, ms_graph = ms_eager, "eager launches", None
    try:
        # One captured Session.run per micro-batch, each reading its images where they lie; the graphs run one after
        # the other and share one memory pool for their intermediates.
        graphs_, outs, pool = [], [], None
        for j in range(n_micro):
            sess.set_input("input", xs[j])
            g = torch.cuda.CUDAGraph()
            torch.cuda.synchronize()
            with torch.cuda.graph(g, pool=pool):
                sess.run()
            if pool is None:
                pool = g.pool()
            graphs_.append(g)
            outs.append(sess.get_output("output"))

        def graph_pass():
            for j in range(n_micro):
                graphs_[j].replay()
                logits[j].copy_(outs[j])

        ms_graph = timed(graph_pass, 1)
        if ms_graph < ms_pass:
            ms_pass, how = ms_graph, "CUDA graph replay: one captured Session.run per micro-batch, reading its images in place"
    except Exception as exc:  # noqa: BLE001 -- capture is an optimisation; the eager number stands
        how = "eager launches (graph capture failed: %r)" % (exc,)
    images = n_micro * micro * world
    # Roofline of the mix: binary convolutions run 2 passes (two bf16 activation terms), the float stem / 1x1
    # shortcuts / FC run 3 (hi*hi + hi*lo + lo*hi): time at the pipe peak = sum(flops_i * passes_i) / peak.
    exec_flops = (2.0 * fb + 3.0 * ff) * n_micro * micro
    roof_ms = exec_flops / (peaks["bf16_tflops"] * 1e12) * 1e3
    out["resnet18_binary_224"] = {
        "images_per_s": images / (ms_pass * 1e-3), "batch": images, "ms_per_batch": ms_pass, "ms_per_batch_eager": ms_eager, "ms_per_batch_graph": ms_graph,
        "ms_per_microbatch": ms_pass / n_micro, "launch_mode": how, "microbatch_per_gpu": micro, "microbatches_per_gpu": n_micro,
        "tflops": (fb + ff) * images / (ms_pass * 1e-3) / 1e12, "flops_per_image": fb + ff,
        "roofline": {"bound": "tensor", "achieved": (fb + ff) * n_micro * micro / (ms_pass * 1e-3) / 1e12,
                     "peak": (fb + ff) * n_micro * micro / (roof_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "frac": roof_ms / ms_pass,
                     "note": f"mix: {fb / (fb + ff):.3f} of the FLOPs are binary convolutions at 2 passes, the rest float layers "
                             f"at 3 passes, against {peaks['source']} cuBLAS bf16 burst {peaks['bf16_tflops']} TFLOP/s; "
                             "pools, adds and the input pre-pass are HBM work on top"},
        "data": "images N(0,1) default_rng(1000 + micro-batch index), weights default_rng(2)",
        "topology": "fp32 stem 7x7/2 + maxpool; 4 stages x 2 basic blocks (64/128/256/512), "
                    "stride 2 + fp32 1x1 shortcut at the entry of stages 2-4; GAP; fp32 FC 1000"}
    return out


def ternary_block(args, ctx):
    """Float x ternary GEMM of the MLP-projection shape: A 4096 x 4096 (seed 0), W 4096 x 11008 (seed 1) ternarised
    at 0.7 * mean|W|, per-column scale = mean |W| over the non-zero entries; two bf16 terms; the columns sharded
    over the ranks with the all-gather of C fused into the epilogue, as for the headline product."""
    from fast_arm_tbcnn_b200.sharded import ShardedGemm
    torch, capi, L, dev, dist = ctx.torch, ctx.capi, ctx.L, ctx.dev, ctx.dist
    M, K, N = 4096, 4096, 11008
    A_h = normal(0, (M, K))
    W_h = normal(1, (K, N))
    delta = float(np.float32(0.7) * np.abs(W_h).mean(dtype=np.float32))
    sg = ShardedGemm(M, K, N, dev, mode=capi.MODE_TC_BF16X2, fused=not args.no_fused_gather, barrier=args.barrier)
    W_d = torch.from_numpy(np.ascontiguousarray(W_h[:, sg.c0:sg.c1])).to(dev)
    timed = device_timer(ctx)
    pack_ms = timed(lambda: sg.set_weights_ternary(W_d, -delta, delta), 5, warm=2)
    del W_d
    A_d = torch.from_numpy(A_h).to(dev)
    L.profile_read()
    L.profile_enable(True)
    ms = timed(lambda: sg.run(A_d), 10, warm=3)
    prof = L.profile_read()
    L.profile_enable(False)

    def w_deq():
        from oracle import cpu_oracle
        orc = cpu_oracle.Oracle()
        t = orc.quantize_to_ternary(W_h, -delta, delta).astype(np.float32)
        return t * orc.column_abs_mean_nonzero(W_h, -delta, delta)[None, :]

    parity = check_sharded_result(sg, A_d, A_h, w_deq, 5, 32, torch, dist)
    flops = 2.0 * M * K * N
    kernel_ms = prof["gemm_ms"] / 13.0   # per product (3 warm-up + 10 timed; a product may be two launches)
    res = {"shape": [M, K, N], "ms": ms, "tflops": flops / (ms * 1e-3) / 1e12, "mode": "x2", "kernel_ms_rank0": kernel_ms,
           "split_ms_rank0": prof["split_ms"] / 13.0,
           "zeros_fraction": float((np.abs(W_h) <= delta).mean()), "pack_ms": pack_ms,
           "pack_note": "this rank's slab: sign planes + per-column scale",
           "parallelism": "single GPU" if ctx.world == 1 else
           f"columns sharded x{ctx.world} ({N // ctx.world} per rank), " + ("all-gather fused into the GEMM epilogue"
                                                                            if sg.fused else "NCCL all-gather + interleave"),
           "parity": parity,
           "roofline": tensor_roofline(flops / ctx.world, kernel_ms, 2, ctx.peaks,
                                       "gemm_tc_kernel of rank 0 (its column slab), two bf16 terms"),
           "data": "A N(0,1) default_rng(0), W N(0,1) default_rng(1), one global threshold 0.7 mean|W|"}
    return res


def fp16_block(args, ctx):
    """The declared one-pass variant (fp16 activations, bar 1e-3) on the headline shape.  Reported beside the
    headline, never as it."""
    torch, capi, L, dev = ctx.torch, ctx.capi, ctx.L, ctx.dev
    if not hasattr(capi, "MODE_TC_FP16X1"):
        return None
    n = args.size
    A_h, W_h = normal(0, (n, n)), normal(1, (n, n))
    W_d = torch.from_numpy(W_h).to(dev)
    words, alpha = L.quant_pack_binary(W_d)
    del W_d
    A_d = torch.from_numpy(A_h).to(dev)
    ws, _ = L.gemm_workspace(n, n, capi.MODE_TC_FP16X1, dev)
    out = torch.empty((n, n), device=dev)
    timed = device_timer(ctx)
    L.profile_read()
    L.profile_enable(True)
    ms = timed(lambda: L.gemm_fxb(A_d, words, n, alpha=alpha, mode=capi.MODE_TC_FP16X1, out=out, workspace=ws), 10, warm=3)
    prof = L.profile_read()
    L.profile_enable(False)
    rows = np.sort(np.random.default_rng(11).choice(n, size=16, replace=False))
    expect = oracle_rows(A_h[rows], dequantise_binary(W_h))
    err = rel_l2(out[torch.from_numpy(rows).to(dev)].cpu().numpy(), expect)
    flops = 2.0 * n * n * n
    kernel_ms = prof["gemm_ms"] / max(prof["gemm_launches"], 1)
    return {"workload": f"float x binary GEMM M=N=K={n}", "mode": "fp16 activations, one pass (declared lower-precision variant)",
            "ms": ms, "tflops": flops / (ms * 1e-3) / 1e12, "kernel_ms": kernel_ms,
            "parity": {"rel_l2": err, "rows": 16, "tolerance": 1e-3, "ok": bool(err <= 1e-3)},
            "roofline": tensor_roofline(flops, kernel_ms, 1, ctx.peaks, "gemm_tc_kernel, one fp16 term")}


def gemm_ladder(args, ctx):
    """The square float x binary GEMM at n = 128 ... 4096 (AUTO mode: the library's per-shape choice): ms per call,
    both roofline fractions, and the error against the oracle on sampled rows."""
    torch, capi, L, dev = ctx.torch, ctx.capi, ctx.L, ctx.dev
    timed = device_timer(ctx)
    res = []
    for n in (128, 256, 512, 1024, 4096):
        A_h, W_h = normal(0, (n, n)), normal(1, (n, n))
        A_d = torch.from_numpy(A_h).to(dev)
        words, alpha = L.quant_pack_binary(torch.from_numpy(W_h).to(dev))
        ws, _ = L.gemm_workspace(n, n, capi.MODE_TC_BF16X2, dev)
        out = torch.empty((n, n), device=dev)
        ms = timed(lambda: L.gemm_fxb(A_d, words, n, alpha=alpha, mode=capi.MODE_AUTO, out=out, workspace=ws), 50 if n <= 1024 else 20, warm=3)
        rows = np.sort(np.random.default_rng(3).choice(n, size=min(n, 16), replace=False))
        err = rel_l2(out[torch.from_numpy(rows).to(dev)].cpu().numpy(), oracle_rows(A_h[rows], dequantise_binary(W_h)))
        flops, byts = 2.0 * n ** 3, 8.125 * n * n + 4 * n
        res.append({"n": n, "ms": ms, "tflops": flops / (ms * 1e-3) / 1e12,
                    "tensor_frac": flops / (ms * 1e-3) / 1e12 / (ctx.peaks["bf16_tflops"] / 2),
                    "hbm_frac": byts / (ms * 1e-3) / 1e9 / ctx.peaks["hbm_gbs"], "rel_l2": err,
                    "kernel": L.describe_choice(n, n, n) if hasattr(L, "describe_choice") else None})
    return res


def lenet_sweep(args, ctx):
    """LeNet-style binary CNN through the C++ tbn::Session (host/bin/run_graph): wall time per synchronous
    Session::run after the first (weights cached, input resident), batch 1 ... 65536."""
    from fast_arm_tbcnn_b200 import graphs, host_build
    driver = host_build.RUN_GRAPH
    if not os.path.exists(driver):
        return {"error": "host/bin/run_graph is not built"}
    res = []
    with tempfile.TemporaryDirectory() as tmp:
        for batch, reps in ((1, 200), (256, 100), (4096, 30), (65536, 6)):
            net = graphs.lenet(batch=batch, seed=1)
            spec, blob, _ = graphs.to_spec(net)
            open(os.path.join(tmp, "spec.txt"), "w").write(spec)
            blob.tofile(os.path.join(tmp, "blob.f32"))
            np.random.default_rng(0).random((batch, 1, 28, 28), dtype=np.float32).tofile(os.path.join(tmp, "x.f32"))
            proc = subprocess.run([driver, os.path.join(tmp, "spec.txt"), os.path.join(tmp, "blob.f32"),
                                   os.path.join(tmp, "x.f32"), "input", "output", "0", os.path.join(tmp, "out.f32"), str(reps)],
                                  capture_output=True, text=True, timeout=600)
            ms = None
            for line in proc.stdout.splitlines():
                if line.startswith("ms_per_run"):
                    ms = float(line.split()[1])
            if proc.returncode != 0 or ms is None:
                res.append({"batch": batch, "error": (proc.stderr or proc.stdout)[-300:]})
                continue
            byts = batch * (3136.0 + 40.0)
            adds = batch * 242560.0   # 6*576*25 + 16*64*150 + 256*10 signed adds per image
            res.append({"batch": batch, "ms": ms, "images_per_s": batch / (ms * 1e-3),
                        "hbm_frac_of_compulsory_bytes": byts / (ms * 1e-3) / 1e9 / ctx.peaks["hbm_gbs"],
                        "cuda_core_add_frac": adds / (ms * 1e-3) / (148 * 128 * 1.965e9)})
    return {"through": "C++ tbn::TBNModel::Session (host/bin/run_graph), float x binary mode, wall time per synchronous run; "
                       "the Session runs this graph as one whole-network kernel (add / subtract by sign on the CUDA cores)",
            "roofline_note": "cuda_core_add_frac = signed adds per second / (148 SMs x 128 lanes x 1.965 GHz); the kernel reads only "
                             "the image and writes only the logits, so the HBM fraction of the compulsory bytes is given as well",
            "data": "input U[0,1) default_rng(0), weights N(0,0.1) default_rng(1)", "sweep": res,
            "bound": "launch latency at small batches, the CUDA cores' add rate at large ones"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import cpu_oracle
    n = args.size
    if not cpu_oracle.reference_available():
        print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref/libtbn_ref.so is not present"}))
        return
    threads = os.cpu_count() or 1
    # ~1.5 s per step per thread at ~30 GFLOP-equivalent/s per core.
    rows_per_thread = max(1, int(1.5 * 30e9 / (2.0 * n * n)) // 16 * 16 or 16)
    rows_per_thread = max(1, min(rows_per_thread, n // threads))
    r = cpu_reference_arm(n, args.steps, args.warmup, threads, rows_per_thread)
    sample = (f"per step: {threads} host threads x {rows_per_thread} rows of A (of {n}) against the full {n}x{n} "
              f"cached packed weights through tbn::qlinear_matmul_binary_blocked_packed "
              f"(ternarised activations, scalar popcount: the portable branch, host is not ARM)")
    line = {
        "impl": "reference", "metric": METRIC, "value": r["tflops"], "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "int1 x int2 popcount (reference TBN mode)",
        "data": "synthetic N(0,1), numpy default_rng seeds 0/1",
        "config": {"workload": f"float x binary GEMM {n}^3 (row sample of {r['rows_per_step']} rows per step)"},
        "cpu_baseline": {"value": r["tflops"], "unit": UNIT, "cores": threads, "kind": "reference", "sample": sample,
                         "float_gemm_tflops_1core": r["float_gemm_tflops_1core"]},
        "e2e": {"value": r["tflops"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def guarded(fn, *a):
    """Runs one block; an exception becomes {"error": ...} so that the headline line is still printed."""
    try:
        return fn(*a)
    except Exception as exc:  # noqa: BLE001
        import traceback
        return {"error": repr(exc), "where": traceback.format_exc(limit=3)[-400:]}


def run_ours(args):
    import torch
    import torch.distributed as dist
    from fast_arm_tbcnn_b200 import capi
    from fast_arm_tbcnn_b200.sharded import ShardedGemm

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU fallback)"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    L = capi.lib
    L.init(local)
    ctx = Ctx()
    ctx.torch, ctx.dist, ctx.capi, ctx.L, ctx.dev, ctx.rank, ctx.world, ctx.peaks = torch, dist, capi, L, dev, rank, world, load_peaks()
    if args.only_cnn:
        # Profiling aid: only the binary-CNN block (conv layer batch 4096 + ResNet-18), one JSON line.
        cnn = cnn_block(args, ctx)
        if rank == 0:
            print(json.dumps({"metric": "binary-CNN images/s", "n_gpus": world, "cnn": cnn}))
        if world > 1:
            dist.destroy_process_group()
        return
    n = args.size
    mode = {"x1": capi.MODE_TC_BF16X1, "x2": capi.MODE_TC_BF16X2, "x3": capi.MODE_TC_BF16X3}[args.mode]
    npass = {"x1": 1, "x2": 2, "x3": 3}[args.mode]
    A_h, W_h = normal(0, (n, n)), normal(1, (n, n))
    sg = ShardedGemm(n, n, n, dev, mode=mode, fused=not args.no_fused_gather, barrier=args.barrier)
    col0, col1, nc = sg.c0, sg.c1, sg.nc
    fused = sg.fused
    if world > 1 and not fused and rank == 0:
        sys.stderr.write(f"symmetric memory unavailable ({sg.fallback_reason}); using NCCL all-gather\n")

    # ---- one-time weight preparation (outside the timed region; timed separately) -------------
    W_d = torch.from_numpy(np.ascontiguousarray(W_h[:, col0:col1])).to(dev)
    timed = device_timer(ctx)
    pack_ms = timed(lambda: sg.set_weights_binary(W_d), 5, warm=3)   # back-to-back calls hide the host-side call overhead
    pack_bytes = 4.0 * n * nc + n * nc / 8.0 + 4.0 * nc
    del W_d

    A_pin = torch.from_numpy(A_h).pin_memory()
    A_d = A_pin.to(dev, non_blocking=True)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    span_events = None  # N > 1: [after GEMM, after barrier] per timed step, to report what the barrier costs

    def step():
        if span_events is None or world == 1:
            sg.run(A_d)
            return
        sg._multiply(A_d)
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        span_events.append(ev)
        sg._barrier()
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        span_events.append(ev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    L.sync()
    L.profile_enable(True)
    L.profile_read()
    props = torch.cuda.get_device_properties(dev)
    try:
        pci = "%08x:%02x:%02x.0" % (props.pci_domain_id, props.pci_bus_id, props.pci_device_id)
    except AttributeError:
        pci = None
    sampler = ClockSampler(local, pci)
    if rank == 0:
        sampler.start()   # before the barrier: its start-up (NVML initialisation) must not delay rank 0 into the timed loop
    barrier()
    launches0 = L.launch_count()
    if world > 1 and fused:
        span_events = []
    ev0.record()
    for _ in range(args.steps):
        step()
    ev1.record()
    torch.cuda.synchronize()
    barrier_ms = None
    if span_events:
        pairs = list(zip(span_events[0::2], span_events[1::2]))
        mine = [sum(a.elapsed_time(b) for a, b in pairs) / len(pairs)]
        # barrier end of step i -> GEMM end of step i+1: split + GEMM + whatever separates them on the stream
        nxt = list(zip(span_events[1::2][:-1], span_events[2::2]))
        mine.append(sum(a.elapsed_time(b) for a, b in nxt) / max(len(nxt), 1))
        both = torch.tensor(mine, device=dev)
        every = torch.empty(world * 2, device=dev)
        dist.all_gather_into_tensor(every, both)
        vals = [round(float(v), 4) for v in every.tolist()]
        barrier_ms = {"barrier_ms_ranks": vals[0::2], "split_plus_gemm_span_ms_ranks": vals[1::2]}
    span_events = None
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    launches = L.launch_count() - launches0
    prof = L.profile_read()
    L.profile_enable(False)
    ms_total = torch.tensor([ev0.elapsed_time(ev1)], device=dev)
    if world > 1:
        dist.all_reduce(ms_total, op=dist.ReduceOp.MAX)
    ms_total = float(ms_total.item())
    L.sync()

    # ---- parity of what was just timed, against the CPU oracle (outside the timed region) --------------
    def w_deq():
        return dequantise_binary(W_h, inplace=True)   # W_h is not needed again: the slabs are packed on the device

    parity = guarded(check_sharded_result, sg, A_d, A_h, w_deq, 7, args.parity_rows, torch, dist)

    # ---- end to end through the product API with host buffers ---------------------------------------
    C_pin = torch.empty((sg.host_rows(), n), dtype=torch.float32).pin_memory()
    e2e_steps = max(1, min(args.steps, 5))
    a_bytes, c_bytes = A_pin.numel() * 4, C_pin.numel() * 4   # c_bytes: this rank's share
    sg.run_host(A_pin, C_pin)
    barrier()
    ev0.record()
    for _ in range(e2e_steps):
        sg.run_host(A_pin, C_pin)
    ev1.record()
    torch.cuda.synchronize()
    barrier()
    e2e_ms = torch.tensor([ev0.elapsed_time(ev1)], device=dev)
    if world > 1:
        dist.all_reduce(e2e_ms, op=dist.ReduceOp.MAX)
    e2e_ms = float(e2e_ms.item())
    # the rows that came back through the host path, against the device-resident result checked above
    my_rows = np.concatenate([np.arange(r0, r1) for r0, r1 in sg.plan["my_rows"]]) if world > 1 else np.arange(n)
    pick = np.sort(np.random.default_rng(13).choice(len(my_rows), size=min(64, len(my_rows)), replace=False))
    same = bool(torch.equal(C_pin[torch.from_numpy(pick)], sg.C[torch.from_numpy(my_rows[pick]).to(dev)].cpu()))
    e2e_agree = torch.tensor([1.0 if same else 0.0], device=dev)
    if world > 1:
        dist.all_reduce(e2e_agree, op=dist.ReduceOp.MIN)
    e2e_agree = bool(e2e_agree.item() > 0)

    kernel_ms_ranks = None
    if world > 1:
        mine = torch.tensor([prof["gemm_ms"] / args.steps], device=dev)   # per product (a product may be two launches)
        every = torch.empty(world, device=dev)
        dist.all_gather_into_tensor(every, mine)
        kernel_ms_ranks = [round(float(v), 4) for v in every.tolist()]
    del A_d, A_pin, C_pin, sg
    torch.cuda.empty_cache()

    cnn = ternary = ladder = lenet = fp16 = None
    if not args.no_cnn:
        ternary = guarded(ternary_block, args, ctx)
        cnn = guarded(cnn_block, args, ctx)
        if world == 1:
            fp16 = guarded(fp16_block, args, ctx)
            ladder = guarded(gemm_ladder, args, ctx)
            lenet = guarded(lenet_sweep, args, ctx)
    if rank == 0:
        peaks = ctx.peaks
        flops_step = 2.0 * n * n * n
        value = flops_step * args.steps / (ms_total * 1e-3) / 1e12
        e2e_value = flops_step * e2e_steps / (e2e_ms * 1e-3) / 1e12
        gemm_ms = prof["gemm_ms"] / args.steps   # GEMM kernel time per product: large products run as two row blocks
        kernel_flops = 2.0 * n * nc * n
        achieved = kernel_flops / (gemm_ms * 1e-3) / 1e12
        sustained = ms_total >= 500.0
        pipe_peak = peaks["bf16_tflops_sustained"] if sustained else peaks["bf16_tflops"]
        peak = pipe_peak / npass
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_total / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": f"bf16 x{npass} split of fp32 activations, +-1 weights, fp32 accumulate", "data":
            "synthetic N(0,1), numpy default_rng seeds 0 (A) / 1 (W)",
            "config": {"workload": f"float x binary GEMM M=N=K={n}, per-column scale mean|W|", "mode": args.mode,
                       "parallelism": "single GPU" if world == 1 else (
                           f"weight columns sharded x{world}; " + ("all-gather fused into the GEMM epilogue (peer stores over "
                           f"NVLink) + {args.barrier} barrier" if fused else "one NCCL all-gather of C + interleave kernel")),
                       "l2": "inputs (1 GiB A per step) larger than the 126 MB L2; no flush needed"},
            "parity": parity,
            "clocks": {k: clocks[k] for k in ("sm_mhz", "sm_max_mhz", "reasons")},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": a_bytes, "d2h_bytes_per_step": c_bytes * world,
                    "bytes_note": "whole job: A crosses PCIe once per step (1/N of every row block per rank), C comes back once",
                    "steps": e2e_steps, "ms_per_step": e2e_ms / e2e_steps, "matches_device_result": e2e_agree,
                    "call": "ShardedGemm.run_host (N = 1: one tbn_gemm_fxb_host call)"},
            "gpu_launches": int(launches),
            "roofline": {
                "bound": "tensor", "kernel": "gemm_tc_kernel", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                "frac": achieved / peak, "traffic": MEASURED_TRAFFIC.get((n, args.mode, world)),
                "traffic_note": "dram__bytes_read.sum + dram__bytes_write.sum of one launch at this size, from a one-pass "
                                "ncu capture summarised with the repository's profiler notes; algorithmic bytes "
                                f"{(2.0 * npass * n * n + n * nc / 8.0 + 4.0 * nc + 4.0 * n * nc):.4g}",
                "peak_source": f"{peaks['source']} cuBLAS bf16 {'sustained' if sustained else 'burst'} "
                               f"{pipe_peak} TFLOP/s / {npass} passes",
                "executed_tflops": achieved * npass, "frac_of_pipe_raw": achieved / pipe_peak,
                "kernel_ms": gemm_ms, "kernel_ms_ranks": kernel_ms_ranks, "barrier_ms": barrier_ms, "barrier": (
                    None if world == 1 else args.barrier), "activation_split": (
                    "separate kernel" if prof["split_launches"] else "inside the GEMM kernel (fp32 rows split in registers)"),
                "split_kernel_ms": prof["split_ms"] / args.steps,
                "launches_per_product": {"gemm": prof["gemm_launches"] / args.steps, "split": prof["split_launches"] / args.steps},
                "hbm_algorithmic_gbs": (4.0 * n * n + n * nc / 8.0 + 4.0 * n * nc) / (gemm_ms * 1e-3) / 1e9,
            },
            "weight_pack": {"ms": pack_ms, "algorithmic_gbs": pack_bytes / (pack_ms * 1e-3) / 1e9,
                            "frac_of_hbm": pack_bytes / (pack_ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                            "roofline": {"bound": "hbm", "achieved": pack_bytes / (pack_ms * 1e-3) / 1e9, "peak": peaks["hbm_gbs"],
                                         "unit": "GB/s", "frac": pack_bytes / (pack_ms * 1e-3) / 1e9 / peaks["hbm_gbs"]},
                            "peak_source": f"{peaks['source']} copy {peaks['hbm_gbs']} GB/s"},
        }
        line["cnn"] = cnn
        line["ternary_mlp_projection"] = ternary
        line["declared_fp16"] = fp16
        line["gemm_ladder"] = ladder
        line["lenet_batch_sweep"] = lenet
        if world == 1 and not args.no_cpu_baseline:
            from oracle import cpu_oracle
            if cpu_oracle.reference_available():
                r = cpu_reference_arm(n, 3, 1, 1, 64)
                line["cpu_baseline"] = {
                    "value": r["tflops"], "unit": UNIT, "cores": 1, "kind": "reference",
                    "sample": f"3 steps of 64 rows of A (of {n}) against the full cached packed weights through the "
                              "reference's tbn::qlinear_matmul_binary_blocked_packed (single-threaded like the "
                              "reference; portable scalar-popcount branch; its float tbn::gemm on 8 rows is given beside)",
                    "float_gemm_tflops_1core": r["float_gemm_tflops_1core"], "host_cores": os.cpu_count()}
                others = guarded(cpu_baselines_other_configs)
                if isinstance(others, dict) and "error" not in others:
                    if isinstance(cnn, dict):
                        if "conv_layer" in others and "conv_layer_64x14x14_to_128_batch4096" in cnn:
                            cnn["conv_layer_64x14x14_to_128_batch4096"]["cpu_baseline"] = others["conv_layer"]
                            cnn["conv_layer_64x14x14_to_128_batch1"]["cpu_baseline"] = others["conv_layer"]
                        if "resnet18" in others and "resnet18_binary_224" in cnn:
                            cnn["resnet18_binary_224"]["cpu_baseline"] = others["resnet18"]
                    if isinstance(ternary, dict) and "ternary_mlp_projection" in others:
                        ternary["cpu_baseline"] = others["ternary_mlp_projection"]
                    if isinstance(lenet, dict) and "lenet" in others:
                        lenet["cpu_baseline"] = others["lenet"]
                else:
                    line["cpu_baseline_other_configs"] = others
            else:
                line["cpu_baseline"] = {"value": None, "unit": UNIT, "cores": 0, "kind": "reference",
                                        "sample": "oracle/_ref/libtbn_ref.so not present"}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    if isinstance(parity, dict) and parity.get("ok") is False:
        sys.exit(3)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--size", type=int, default=16384)
    ap.add_argument("--mode", default="x2", choices=["x1", "x2", "x3"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-cnn", action="store_true", help="skip every block but the headline GEMM")
    ap.add_argument("--only-cnn", action="store_true", help="run only the binary-CNN images/s block")
    ap.add_argument("--resnet-microbatch", type=int, default=1024, help="images per GPU and Session.run in the ResNet-18 block")
    ap.add_argument("--resnet-batch", type=int, default=8192, help="whole-job batch of the ResNet-18 block")
    ap.add_argument("--parity-rows", type=int, default=32, help="rows of C compared with the CPU oracle after the timed region")
    ap.add_argument("--barrier", choices=["nccl", "symm"], default="nccl",
                    help="N > 1, fused path: step-closing barrier = tiny NCCL all-reduce or the symmetric-memory signal barrier")
    ap.add_argument("--no-fused-gather", action="store_true", help="N > 1: use NCCL all-gather instead of peer stores")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
