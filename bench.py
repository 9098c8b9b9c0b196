#!/usr/bin/env python
"""Benchmark of the hot path: float x binary GEMM  C = A (alpha * sign(W)),  M = N = K = 16384.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--size n]

One "step" is one GEMM over the whole activation matrix (activation split + tensor-core kernel;
on N > 1 GPUs additionally the all-gather of the column slabs and the interleave).  The packed
weights are prepared once before the timed region, as the reference Session caches them.
Rank 0 prints ONE JSON line.  N > 1 is launched with torchrun (one rank per GPU, NCCL): the
weight columns are sharded across ranks (strong scaling of the fixed 16384^3 problem).

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
MEASURED_TRAFFIC = {(16384, "x2", 1): 5.09e9, (8192, "x2", 1): 0.639e9}

METRIC = "float x binary GEMM throughput (2*M*N*K / time)"
UNIT = "TFLOP/s"


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


def make_inputs(n, rank_cols=None):
    """A from seed 0, W from seed 1, both N(0,1) fp32 (numpy default_rng), generated on the host."""
    A = np.random.default_rng(0).standard_normal((n, n), dtype=np.float32)
    W = np.random.default_rng(1).standard_normal((n, n), dtype=np.float32)
    if rank_cols is not None:
        W = np.ascontiguousarray(W[:, rank_cols[0]:rank_cols[1]])
    return A, W


def cpu_reference_arm(n, steps, warmup, threads, rows_per_thread):
    """Times the reference's CPU path on a row sample: per step, `threads` host threads each run
    tbn::qlinear_matmul_binary_blocked_packed on `rows_per_thread` rows of A against the full
    cached packed weight matrix (the reference itself is single-threaded; independent row blocks
    are the only way to use more cores without touching its code)."""
    from oracle import cpu_oracle
    ref = cpu_oracle.Reference()
    rng = np.random.default_rng(1)
    W = rng.standard_normal((n, n), dtype=np.float32)
    qb = ref.quantize_to_binary(W, 0.0)
    del W
    handle = ref.pack_binary_weights(qb)
    del qb
    rows = threads * rows_per_thread
    A = np.random.default_rng(0).standard_normal((rows, n), dtype=np.float32)
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
    Wd = np.random.default_rng(1).standard_normal((n, n), dtype=np.float32)
    Wd = np.where(Wd > 0, np.float32(1), np.float32(-1))
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


def cnn_block(args, L, capi, torch, dist, dev, rank, world):
    """Binary-CNN throughput, batch-sharded over the ranks with no collective: the 64x14x14 -> 128 3x3 conv
    layer at batch 4096 and the binary ResNet-18-style network at 224x224 (micro-batches of 512 images per
    GPU).  Whole-job images/s = images of all ranks / max-over-ranks device time."""
    from fast_arm_tbcnn_b200 import sharding
    from fast_arm_tbcnn_b200.session import Session
    from fast_arm_tbcnn_b200 import graphs
    out = {}
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def timed(fn, reps):
        fn()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        ev0.record()
        for _ in range(reps):
            fn()
        ev1.record()
        torch.cuda.synchronize()
        ms = torch.tensor([ev0.elapsed_time(ev1) / reps], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    # ---- single conv layer, batch 4096 split across the ranks
    b0, b1 = sharding.batch_block(rank, world, 4096)
    g = torch.Generator(device=dev).manual_seed(rank)
    x = torch.randn((b1 - b0, 64, 14, 14), generator=g, device=dev)
    w = torch.randn((128, 64, 3, 3), generator=g, device=dev) * 0.05
    bias = torch.randn(128, generator=g, device=dev) * 0.05
    order = capi.CONV_WEIGHTS_TAP_MAJOR
    words, alpha = L.quant_pack_binary(L.permute_filters(w), capi.LAYOUT_NK)
    ws, _ = L.conv_workspace(x.shape, 128, 3, 3, dev, order)
    y = torch.empty((b1 - b0, 128, 14, 14), device=dev)
    p = (1, 1, 1, 1, 1, 1)
    ms = timed(lambda: L.conv2d_fxb(x, words, w.shape, p, alpha=alpha, bias=bias, workspace=ws, out=y, order=order), 10)
    flops = 2.0 * 4096 * 196 * 128 * 576
    out["conv_layer_64x14x14_to_128_batch4096"] = {
        "images_per_s": 4096 / (ms * 1e-3), "ms": ms, "tflops": flops / (ms * 1e-3) / 1e12,
        "algorithmic_gbs": 4096 * (64 + 128) * 196 * 4 / (ms * 1e-3) / 1e9}
    del x, y

    # ---- binary ResNet-18-style CNN, 3x224x224
    micro = args.resnet_microbatch
    net = graphs.resnet18(batch=micro, seed=2, image=224, classes=1000)
    sess = Session(net)
    sess.keep_intermediates = False
    xin = torch.randn((micro, 3, 224, 224), generator=g, device=dev)
    sess.set_input("input", xin)
    sess.run()          # prepares and caches the packed weights, grows the workspaces
    ms_eager = timed(sess.run, 5)
    # One Session.run is about sixty short launches: replaying it as a CUDA graph takes the host's per-launch
    # cost out of the loop.  The eager figure is kept beside it.
    ms, how = ms_eager, "eager launches"
    try:
        graph = torch.cuda.CUDAGraph()
        torch.cuda.synchronize()
        with torch.cuda.graph(graph):
            sess.run()
        ms_graph = timed(graph.replay, 10)
        if ms_graph < ms:
            ms, how = ms_graph, "CUDA graph replay of one Session.run"
    except Exception as exc:  # noqa: BLE001 -- capture is an optimisation; the eager number stands
        how = "eager launches (graph capture failed: %r)" % (exc,)
    out["resnet18_binary_224"] = {"images_per_s": micro * world / (ms * 1e-3), "ms_per_microbatch": ms,
                                  "ms_per_microbatch_eager": ms_eager, "launch_mode": how,
                                  "microbatch_per_gpu": micro, "tflops": 3.63e9 * micro * world / (ms * 1e-3) / 1e12,
                                  "topology": "fp32 stem 7x7/2 + maxpool; 4 stages x 2 basic blocks (64/128/256/512), "
                                              "stride 2 + fp32 1x1 shortcut at the entry of stages 2-4; GAP; fp32 FC 1000"}
    return out


def ternary_block(L, capi, torch, dev):
    """Float x ternary GEMM of the MLP-projection shape: A 4096 x 4096, W 4096 x 11008 ternarised at 0.7 * mean|W|,
    per-column scale = mean |W| over the non-zero entries; two bf16 terms.  One GPU, inputs resident."""
    M, K, N = 4096, 4096, 11008
    g = torch.Generator(device=dev).manual_seed(0)
    A = torch.randn((M, K), generator=g, device=dev)
    W = torch.randn((K, N), generator=g, device=dev)
    delta = 0.7 * float(W.abs().mean())
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(2):
        codes, pos, neg, alpha = L.quant_pack_ternary(W, -delta, delta)
    torch.cuda.synchronize()
    ev0.record()
    for _ in range(5):
        codes, pos, neg, alpha = L.quant_pack_ternary(W, -delta, delta)
    ev1.record()
    torch.cuda.synchronize()
    pack_ms = ev0.elapsed_time(ev1) / 5
    ws, _ = L.gemm_workspace(M, K, capi.MODE_TC_BF16X2, dev)
    out = torch.empty((M, N), device=dev)
    for _ in range(3):
        L.gemm_fxb(A, neg, N, pos=pos, alpha=alpha, mode=capi.MODE_TC_BF16X2, out=out, workspace=ws)
    torch.cuda.synchronize()
    ev0.record()
    for _ in range(10):
        L.gemm_fxb(A, neg, N, pos=pos, alpha=alpha, mode=capi.MODE_TC_BF16X2, out=out, workspace=ws)
    ev1.record()
    torch.cuda.synchronize()
    ms = ev0.elapsed_time(ev1) / 10
    return {"shape": [M, K, N], "ms": ms, "tflops": 2.0 * M * K * N / (ms * 1e-3) / 1e12, "mode": "x2",
            "zeros_fraction": float((W.abs() <= delta).float().mean()), "pack_ms": pack_ms,
            "pack_note": "sign planes + 2-bit reference codes + per-column scale"}


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


def run_ours(args):
    import torch
    import torch.distributed as dist
    from fast_arm_tbcnn_b200 import capi

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
    if args.only_cnn:
        # Profiling aid: only the binary-CNN block (conv layer batch 4096 + ResNet-18), one JSON line.
        cnn = cnn_block(args, L, capi, torch, dist, dev, rank, world)
        if rank == 0:
            print(json.dumps({"metric": "binary-CNN images/s", "n_gpus": world, "cnn": cnn}))
        if world > 1:
            dist.destroy_process_group()
        return
    n = args.size
    mode = {"x1": capi.MODE_TC_BF16X1, "x2": capi.MODE_TC_BF16X2, "x3": capi.MODE_TC_BF16X3}[args.mode]
    npass = {"x1": 1, "x2": 2, "x3": 3}[args.mode]
    from fast_arm_tbcnn_b200 import sharding
    col0, col1 = sharding.column_slab(rank, world, n)
    nc = col1 - col0
    A_h, W_h = make_inputs(n, (col0, col1))

    # ---- one-time weight preparation (outside the timed region; timed separately) -------------
    W_d = torch.from_numpy(W_h).to(dev)
    L.quant_pack_binary(W_d)
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    pack_reps = 5   # back-to-back calls, so that the host-side call overhead hides behind the previous kernel
    for _ in range(2):  # settle the caching allocator (two result buffers alternate)
        words, alpha = L.quant_pack_binary(W_d)
    torch.cuda.synchronize()
    ev0.record()
    for _ in range(pack_reps):
        words, alpha = L.quant_pack_binary(W_d)
    ev1.record()
    torch.cuda.synchronize()
    pack_ms = ev0.elapsed_time(ev1) / pack_reps
    pack_bytes = 4.0 * n * nc + n * nc / 8.0 + 4.0 * nc
    del W_d, W_h

    A_pin = torch.from_numpy(A_h).pin_memory()
    A_d = A_pin.to(dev, non_blocking=True)
    C_slab = torch.empty((n, nc), dtype=torch.float32, device=dev)
    ws, _ = L.gemm_workspace(n, n, mode, dev)
    # N > 1: the epilogue of each rank's GEMM writes its column slab straight into every rank's result
    # matrix (peer-mapped symmetric memory, plain stores over NVLink) -- compute and all-gather in one kernel;
    # a tiny NCCL all-reduce closes the step as the cross-GPU barrier.  If symmetric memory cannot be set up,
    # fall back to one NCCL all-gather of the slabs plus the interleave kernel.
    gathered, dests, fused, flag = None, None, False, None
    C_full = C_slab
    if world > 1:
        flag = torch.zeros(1, device=dev)
        if not args.no_fused_gather:
            try:
                import torch.distributed._symmetric_memory as symm_mem
                C_full = symm_mem.empty((n, n), dtype=torch.float32, device=dev)
                hdl = symm_mem.rendezvous(C_full, dist.group.WORLD)
                ptrs = [int(p) for p in hdl.buffer_ptrs]
                order = [(rank + i) % world for i in range(world)]
                dests = [ptrs[r] + col0 * 4 for r in order]
                fused = True
            except Exception as exc:  # noqa: BLE001
                sys.stderr.write(f"[rank {rank}] symmetric memory unavailable ({exc}); using NCCL all-gather\n")
        ok = torch.tensor([1.0 if fused else 0.0], device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        fused = bool(ok.item() > 0)
        if not fused:
            gathered = torch.empty((world, n, nc), dtype=torch.float32, device=dev)
            C_full = torch.empty((n, n), dtype=torch.float32, device=dev)

    span_events = None  # N > 1: [after GEMM, after barrier] per timed step, to report what the barrier costs

    def step():
        if world == 1:
            L.gemm_fxb(A_d, words, nc, alpha=alpha, mode=mode, out=C_slab, workspace=ws)
        elif fused:
            L.gemm_fxb_multi(A_d, words, nc, dests, n, alpha=alpha, mode=mode, workspace=ws)
            if span_events is not None:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                span_events.append(ev)
            if args.barrier == "symm":
                hdl.barrier(channel=0)
            else:
                dist.all_reduce(flag)
            if span_events is not None:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                span_events.append(ev)
        else:
            L.gemm_fxb(A_d, words, nc, alpha=alpha, mode=mode, out=C_slab, workspace=ws)
            dist.all_gather_into_tensor(gathered.view(world * n, nc), C_slab)
            L.gather_cols_permute(gathered, out=C_full)

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

    # Every rank must hold the same full result: compare a checksum of C across ranks.
    replicas_agree = None
    if world > 1:
        cs = C_full.double().sum().reshape(1)
        lo, hi = cs.clone(), cs.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        replicas_agree = bool((lo == hi).item()) and bool(torch.isfinite(cs).item())

    # ---- end to end through the C ABI with host buffers ---------------------------------------
    # Each rank returns its block of result rows (contiguous in the row-major C), so that the host holds
    # the whole product once.
    rows0, rows1 = rank * (n // world), (rank + 1) * (n // world)
    C_out_view = C_full[rows0:rows1] if world > 1 else C_slab
    C_pin = torch.empty(tuple(C_out_view.shape), dtype=torch.float32).pin_memory()
    e2e_steps = max(1, min(args.steps, 5))
    h = L.h
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    a_bytes, c_bytes = A_pin.numel() * 4, C_pin.numel() * 4   # c_bytes: this rank's share

    host_ws = None
    if world == 1:
        host_ws = torch.empty(h.tbn_gemm_fxb_host_workspace_bytes(n, n, nc, mode), dtype=torch.uint8, device=dev)

    def e2e_step():
        if world == 1:
            # One C-ABI call on host buffers: chunked upload / multiply / download, overlapped.
            L.gemm_fxb_host(A_pin, words, nc, C_pin, alpha=alpha, mode=mode, workspace=host_ws)
            return
        # N > 1: the host matrix is uploaded ONCE per step across the job -- every rank copies its block of rows
        # over its own PCIe link -- and the blocks are exchanged over NVLink (one in-place NCCL all-gather), which
        # is an order of magnitude faster than sending the whole of A to every GPU from the host.  Then the sharded
        # multiply, and every rank returns its block of result rows.
        a_blk, a_pin_blk = A_d[rows0:rows1], A_pin[rows0:rows1]
        capi.check(h.tbn_cuda_h2d(C.c_void_p(a_blk.data_ptr()), C.c_void_p(a_pin_blk.data_ptr()), a_blk.numel() * 4, stream))
        dist.all_gather_into_tensor(A_d, a_blk)
        step()
        capi.check(h.tbn_cuda_d2h(C.c_void_p(C_pin.data_ptr()), C.c_void_p(C_out_view.data_ptr()), c_bytes, stream))

    e2e_step()
    barrier()
    ev0.record()
    for _ in range(e2e_steps):
        e2e_step()
    ev1.record()
    torch.cuda.synchronize()
    barrier()
    e2e_ms = torch.tensor([ev0.elapsed_time(ev1)], device=dev)
    if world > 1:
        dist.all_reduce(e2e_ms, op=dist.ReduceOp.MAX)
    e2e_ms = float(e2e_ms.item())

    kernel_ms_ranks = None
    if world > 1:
        mine = torch.tensor([prof["gemm_ms"] / max(prof["gemm_launches"], 1)], device=dev)
        every = torch.empty(world, device=dev)
        dist.all_gather_into_tensor(every, mine)
        kernel_ms_ranks = [round(float(v), 4) for v in every.tolist()]

    cnn = None
    if not args.no_cnn:
        try:
            cnn = cnn_block(args, L, capi, torch, dist, dev, rank, world)
        except Exception as exc:  # noqa: BLE001  -- the GEMM line must still be printed
            cnn = {"error": repr(exc)}
    ternary = None
    if not args.no_cnn and world == 1:
        try:
            ternary = ternary_block(L, capi, torch, dev)
        except Exception as exc:  # noqa: BLE001
            ternary = {"error": repr(exc)}
    if rank == 0:
        peaks = load_peaks()
        flops_step = 2.0 * n * n * n
        value = flops_step * args.steps / (ms_total * 1e-3) / 1e12
        e2e_value = flops_step * e2e_steps / (e2e_ms * 1e-3) / 1e12
        gemm_ms = prof["gemm_ms"] / max(prof["gemm_launches"], 1)
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
                           "NVLink) + NCCL barrier" if fused else "one NCCL all-gather of C + interleave kernel")),
                       "replicas_agree": replicas_agree,
                       "l2": "inputs (1 GiB A per step) larger than the 126 MB L2; no flush needed"},
            "clocks": {k: clocks[k] for k in ("sm_mhz", "sm_max_mhz", "reasons")},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": a_bytes, "d2h_bytes_per_step": c_bytes * world,
                    "bytes_note": "whole job: A crosses PCIe once per step (1/N of its rows per rank), C comes back once",
                    "steps": e2e_steps, "ms_per_step": e2e_ms / e2e_steps},
            "gpu_launches": int(launches),
            "roofline": {
                "bound": "tensor", "kernel": "gemm_tc_kernel", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                "frac": achieved / peak, "traffic": MEASURED_TRAFFIC.get((n, args.mode, world)),
                "traffic_note": "dram__bytes_read.sum + dram__bytes_write.sum of one launch at this size, one-pass ncu "
                                "capture (profiles/gemm_tc_kernel_fxb_16384_x2_dram_traffic.md); algorithmic bytes "
                                f"{(2.0 * npass * n * n + n * nc / 8.0 + 4.0 * nc + 4.0 * n * nc):.4g}",
                "peak_source": f"{peaks['source']} cuBLAS bf16 {'sustained' if sustained else 'burst'} "
                               f"{pipe_peak} TFLOP/s / {npass} passes",
                "executed_tflops": achieved * npass, "frac_of_pipe_raw": achieved / pipe_peak,
                "kernel_ms": gemm_ms, "kernel_ms_ranks": kernel_ms_ranks, "barrier_ms": barrier_ms, "barrier": (
                    None if world == 1 else args.barrier), "activation_split": (
                    "separate kernel" if prof["split_launches"] else "inside the GEMM kernel (fp32 rows split in registers)"),
                "split_kernel_ms": prof["split_ms"] / max(prof["split_launches"], 1),
                "hbm_algorithmic_gbs": (4.0 * n * n + n * nc / 8.0 + 4.0 * n * nc) / (gemm_ms * 1e-3) / 1e9,
            },
            "weight_pack": {"ms": pack_ms, "algorithmic_gbs": pack_bytes / (pack_ms * 1e-3) / 1e9,
                            "frac_of_hbm": pack_bytes / (pack_ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                            "peak_source": f"{peaks['source']} copy {peaks['hbm_gbs']} GB/s"},
        }
        line["cnn"] = cnn
        line["ternary_mlp_projection"] = ternary
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
            else:
                line["cpu_baseline"] = {"value": None, "unit": UNIT, "cores": 0, "kind": "reference",
                                        "sample": "oracle/_ref/libtbn_ref.so not present"}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--size", type=int, default=16384)
    ap.add_argument("--mode", default="x2", choices=["x1", "x2", "x3"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-cnn", action="store_true", help="skip the binary-CNN images/s block")
    ap.add_argument("--only-cnn", action="store_true", help="run only the binary-CNN images/s block")
    ap.add_argument("--resnet-microbatch", type=int, default=512, help="images per GPU and Session.run in the ResNet-18 block")
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
