"""Column-sharded float x {binary, ternary} GEMM across the GPUs of one box (one process per GPU).

The reference is single-device; this is the multi-GPU form of its GEMM path (the product defined by
tbn::qlinear_matmul_binary_naive, tbn-runtime/src/operators/quantized_gemm_neon.cpp:63-90, on weights packed as
BinaryMatrix::pack does, GeMM/05-final/GeMM.cpp:114-151).  Rank g owns the weight columns
[g*N/G, (g+1)*N/G) -- in the packed layout one contiguous range of words, so every rank packs only its own
slab -- the activations A are replicated, and every rank ends a step holding the whole C[M, N].

`ShardedGemm` owns everything a step needs:
  * the rendezvous of the result matrices in symmetric memory (every rank's C mapped into every rank's
    address space) and the per-rank destination list (own matrix first, then the peers in ring order, each
    pointer already offset to this rank's column slab);
  * the step itself: ONE kernel per rank (tbn_gemm_fxb_multi) whose epilogue stores each finished tile into
    every rank's C over NVLink -- compute and all-gather fused -- followed by the cross-GPU barrier that makes
    the peers' stores visible (a one-element NCCL all-reduce, or the symmetric-memory signal barrier);
  * the fallback when symmetric memory cannot be set up: one NCCL all-gather of the [M, N/G] slabs plus the
    interleave kernel (tbn_gather_cols_permute);
  * `run_host`: the same product for HOST buffers -- the call a user of the reference's host-tensor operators
    makes.  A is uploaded ONCE across the job (each rank copies 1/G of every row block over its own PCIe link
    and an NCCL all-gather spreads it over NVLink), row block by row block, so that upload, multiply and
    download of successive blocks overlap on three streams; every rank returns its share of the result rows.

World size 1 is the plain single-GPU GEMM behind the same interface.  The bookkeeping (slabs, destination
order, row blocks) is plain Python and is exercised on CPU by `plan()` without a GPU.
"""
import ctypes as C

from . import sharding


def destination_order(rank, world):
    """Ranks in the order this rank's epilogue writes them: itself first, then the ring rank+1, rank+2, ...
    so that at any moment the G ranks target G different peers."""
    return [(rank + i) % world for i in range(world)]


def row_blocks(M, world, blocks):
    """Row blocks of the host-buffer pipeline: [(m0, m1)] with every block a multiple of 128*world rows (whole
    GEMM tiles per rank share) except possibly the last."""
    unit = 128 * world
    per = max(unit, ((M + blocks - 1) // blocks + unit - 1) // unit * unit)
    return [(m0, min(M, m0 + per)) for m0 in range(0, M, per)]


def rank_rows(m0, m1, rank, world):
    """The part of row block [m0, m1) that `rank` uploads and downloads: contiguous, 1/world of it (the last rank
    takes the remainder)."""
    per = (m1 - m0 + world - 1) // world
    lo = min(m1, m0 + rank * per)
    return lo, min(m1, lo + per)


def plan(M, K, N, rank, world, host_blocks=8):
    """Everything index-like a step uses, as plain numbers (no torch, no CUDA): checked on CPU."""
    c0, c1 = sharding.column_slab(rank, world, N)
    blocks = row_blocks(M, world, host_blocks)
    return {
        "columns": (c0, c1),
        "dest_ranks": destination_order(rank, world),
        "dest_byte_offset": c0 * 4,
        "row_blocks": blocks,
        "my_rows": [rank_rows(m0, m1, rank, world) for m0, m1 in blocks],
        "packed_word_rows": (c0, c1),          # rows of the [N_pad][K_pad/32] word matrix this rank owns
    }


class ShardedGemm:
    """C[M, N] = A[M, K] (alpha * w) with the columns of w sharded over the ranks of `group`.

    mode: a tensor-core mode of the C ABI (capi.MODE_TC_BF16X2 by default).  barrier: "nccl" | "symm".
    fused=False forces the NCCL all-gather fallback."""

    def __init__(self, M, K, N, device, group=None, mode=None, fused=True, barrier="nccl"):
        import torch
        import torch.distributed as dist
        from . import capi
        self.torch, self.dist, self.capi = torch, dist, capi
        self.L = capi.lib
        self.L.init(device.index if device.index is not None else torch.cuda.current_device())
        self.M, self.K, self.N, self.device = M, K, N, device
        self.mode = capi.MODE_TC_BF16X2 if mode is None else mode
        self.barrier_kind = barrier
        self.world = dist.get_world_size(group) if (dist.is_available() and dist.is_initialized()) else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        self.group = group if group is not None else (dist.group.WORLD if self.world > 1 else None)
        self.plan = plan(M, K, N, self.rank, self.world)
        self.c0, self.c1 = self.plan["columns"]
        self.nc = self.c1 - self.c0
        self.neg = self.pos = self.alpha = self.bias = None
        self.ws, _ = self.L.gemm_workspace(M, K, self.mode, device)
        self.fused = False
        self.handle = None
        self.gathered = None
        self.flag = None
        self._host = None
        if self.world == 1:
            self.C = torch.empty((M, N), dtype=torch.float32, device=device)
            self.dests = None
            return
        self.flag = torch.zeros(1, device=device)
        why = "disabled by the caller"
        if fused:
            try:
                import torch.distributed._symmetric_memory as symm_mem
                self.C = symm_mem.empty((M, N), dtype=torch.float32, device=device)
                self.handle = symm_mem.rendezvous(self.C, self.group)
                ptrs = [int(p) for p in self.handle.buffer_ptrs]
                self.dests = [ptrs[r] + self.plan["dest_byte_offset"] for r in self.plan["dest_ranks"]]
                self.fused = True
            except Exception as exc:  # noqa: BLE001 -- the fallback below is a complete implementation
                why = repr(exc)
        ok = torch.tensor([1.0 if self.fused else 0.0], device=device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=self.group)
        self.fused = bool(ok.item() > 0)
        self.fallback_reason = None if self.fused else why
        if not self.fused:
            self.handle, self.dests = None, None
            self.C = torch.empty((M, N), dtype=torch.float32, device=device)
            self.gathered = torch.empty((self.world, M, self.nc), dtype=torch.float32, device=device)
            self.c_slab = torch.empty((M, self.nc), dtype=torch.float32, device=device)

    # ---- weights ------------------------------------------------------------------------------
    def set_weights_binary(self, w_slab, thr=0.0):
        """w_slab: this rank's columns of W, fp32 [K, N/G] on the device.  Packs the sign words and the
        per-column scale mean|W| of the slab."""
        assert tuple(w_slab.shape) == (self.K, self.nc)
        self.neg, self.alpha = self.L.quant_pack_binary(w_slab, thr=thr)
        self.pos = None

    def set_weights_ternary(self, w_slab, lo, hi):
        """Ternary slab: planes for w < lo (-1) and w > hi (+1); scale = mean |W| over the non-zero entries."""
        assert tuple(w_slab.shape) == (self.K, self.nc)
        _, self.pos, self.neg, self.alpha = self.L.quant_pack_ternary(w_slab, lo, hi, want_codes=False)

    def set_bias(self, bias_slab):
        self.bias = bias_slab

    # ---- one step on resident activations -----------------------------------------------------------
    def _multiply(self, a, m0=0):
        """Enqueues the multiply of the rows `a` = A[m0 : m0 + a.shape[0]] on the current stream (no barrier)."""
        L, world = self.L, self.world
        rows = a.shape[0]
        if world == 1:
            L.gemm_fxb(a, self.neg, self.nc, pos=self.pos, alpha=self.alpha, bias=self.bias, mode=self.mode,
                       out=self.C[m0:m0 + rows], workspace=self.ws)
        elif self.fused:
            off = m0 * self.N * 4
            L.gemm_fxb_multi(a, self.neg, self.nc, [d + off for d in self.dests], self.N, pos=self.pos, alpha=self.alpha,
                             bias=self.bias, mode=self.mode, workspace=self.ws)
        else:
            slab = self.c_slab[:rows]
            L.gemm_fxb(a, self.neg, self.nc, pos=self.pos, alpha=self.alpha, bias=self.bias, mode=self.mode, out=slab,
                       workspace=self.ws)
            g = self.gathered.view(-1)[: world * rows * self.nc].view(world * rows, self.nc)
            self.dist.all_gather_into_tensor(g, slab, group=self.group)
            L.gather_cols_permute(g.view(world, rows, self.nc), out=self.C[m0:m0 + rows])

    def _barrier(self):
        """Closes a step: after it (in stream order) every peer's stores into this rank's C have landed."""
        if self.world == 1 or not self.fused:
            return      # the fallback's all-gather already orders the exchange
        if self.barrier_kind == "symm":
            self.handle.barrier(channel=0)
        else:
            self.dist.all_reduce(self.flag, group=self.group)

    def run(self, a):
        """a: A [M, K] fp32 resident on this rank's GPU (the same on every rank).  Returns C [M, N] (this rank's
        copy; complete, in stream order, when the call returns)."""
        self._multiply(a)
        self._barrier()
        return self.C

    # ---- host buffers ---------------------------------------------------------------------------------
    def _host_state(self):
        if self._host is None:
            t = self.torch
            self._host = {
                "a": t.empty((self.M, self.K), dtype=t.float32, device=self.device) if self.world > 1 else None,
                "h2d": t.cuda.Stream(device=self.device), "d2h": t.cuda.Stream(device=self.device),
                "ws1": None,
            }
        return self._host

    def run_host(self, a_host, c_host):
        """a_host: A [M, K] in (pinned) host memory, the same array on every rank.  c_host: host buffer that
        receives this rank's share of the result rows, in the order of plan["my_rows"] (world 1: the whole C).
        Asynchronous with respect to the host: synchronise the current stream before reading c_host."""
        t, capi, h = self.torch, self.capi, self.L.h
        st = self._host_state()
        if self.world == 1:
            if st["ws1"] is None:
                st["ws1"] = t.empty(h.tbn_gemm_fxb_host_workspace_bytes(self.M, self.K, self.nc, self.mode), dtype=t.uint8,
                                    device=self.device)
            self.L.gemm_fxb_host(a_host, self.neg, self.nc, c_host, pos=self.pos, alpha=self.alpha, bias=self.bias,
                                 mode=self.mode, workspace=st["ws1"])
            return c_host
        main = t.cuda.current_stream()
        h2d, d2h = st["h2d"], st["d2h"]
        h2d.wait_stream(main)
        d2h.wait_stream(main)
        a_dev = st["a"]
        out_row = 0
        for (m0, m1), (r0, r1) in zip(self.plan["row_blocks"], self.plan["my_rows"]):
            # upload this rank's part of the block over its own PCIe link
            with t.cuda.stream(h2d):
                if r1 > r0:
                    capi.check(h.tbn_cuda_h2d(C.c_void_p(a_dev[r0:r1].data_ptr()), C.c_void_p(a_host[r0:r1].data_ptr()),
                                              (r1 - r0) * self.K * 4, C.c_void_p(h2d.cuda_stream)))
                up = t.cuda.Event()
                up.record(h2d)
            main.wait_event(up)
            # spread the parts over NVLink (in place), multiply the block, close it with the barrier
            per = (m1 - m0 + self.world - 1) // self.world
            if per * self.world == m1 - m0:
                self.dist.all_gather_into_tensor(a_dev[m0:m1], a_dev[r0:r1], group=self.group)
            else:   # ragged last block: gather whole padded parts through a list of views
                parts = [a_dev[min(m1, m0 + r * per):min(m1, m0 + (r + 1) * per)] for r in range(self.world)]
                for r, part in enumerate(parts):
                    if part.numel():
                        self.dist.broadcast(part, src=self.dist.get_global_rank(self.group, r), group=self.group)
            self._multiply(a_dev[m0:m1], m0)
            self._barrier()
            done = t.cuda.Event()
            done.record(main)
            # download this rank's share of the finished rows
            with t.cuda.stream(d2h):
                d2h.wait_event(done)
                if r1 > r0:
                    capi.check(h.tbn_cuda_d2h(C.c_void_p(c_host[out_row:out_row + (r1 - r0)].data_ptr()),
                                              C.c_void_p(self.C[r0:r1].data_ptr()), (r1 - r0) * self.N * 4,
                                              C.c_void_p(d2h.cuda_stream)))
            out_row += r1 - r0
        main.wait_stream(d2h)
        main.wait_stream(h2d)
        return c_host

    def host_rows(self):
        """Number of result rows `run_host` returns on this rank."""
        if self.world == 1:
            return self.M
        return sum(r1 - r0 for r0, r1 in self.plan["my_rows"])
