"""Multi-rank host logic on CPU: two gloo ranks run the column-sharded GEMM orchestration
(slab ownership, one all-gather, interleave) with the oracle standing in for the device GEMM,
and batch sharding with no collective."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, M, K, N, result_dir):
    sys.path.insert(0, ROOT)
    from fast_arm_tbcnn_b200 import sharding
    from oracle import cpu_oracle, graphs
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        orc = cpu_oracle.Oracle()
        A = np.random.default_rng(0).standard_normal((M, K), dtype=np.float32)
        W = np.random.default_rng(1).standard_normal((K, N), dtype=np.float32)
        lo, hi = sharding.column_slab(rank, world, N)
        # Each rank packs only its own columns: the slab of the full packed matrix is the packing of the slab.
        full_words = orc.binary_pack_padded(orc.quantize_to_binary(W))
        slab_words = orc.binary_pack_padded(orc.quantize_to_binary(W[:, lo:hi]))
        assert np.array_equal(full_words[lo:hi], slab_words[: hi - lo])
        c_slab = torch.from_numpy(orc.gemm_f32(A, graphs.dequantise(W[:, lo:hi])))
        gathered = torch.empty((world * M, hi - lo), dtype=torch.float32)
        dist.all_gather_into_tensor(gathered, c_slab)
        c_full = sharding.interleave_slabs(gathered.numpy().reshape(world, M, hi - lo))
        if rank == 0:
            np.save(os.path.join(result_dir, "c_full.npy"), c_full)
        # Batch sharding: blocks tile the batch without a collective.
        blocks = [sharding.batch_block(r, world, 11) for r in range(world)]
        assert blocks[0][0] == 0 and blocks[-1][1] == 11
        assert all(blocks[i][1] == blocks[i + 1][0] for i in range(world - 1))
    finally:
        dist.destroy_process_group()


def _plan_worker(rank, world, port, M, K, N, result_dir):
    """The bookkeeping of ShardedGemm (sharded.plan) driven by two gloo ranks: each rank computes its column slab
    with the oracle and "stores" it into every rank's result matrix (a memory-mapped file per rank stands in for
    the peer-mapped symmetric memory) at the byte offsets and in the destination order the plan gives -- exactly
    what the fused epilogue does with the pointers built from the same plan.  After the barrier every rank must
    hold the full product, and the row shares of the host-buffer path must tile the matrix."""
    sys.path.insert(0, ROOT)
    from fast_arm_tbcnn_b200 import sharded
    from oracle import cpu_oracle, graphs
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        orc = cpu_oracle.Oracle()
        A = np.random.default_rng(0).standard_normal((M, K), dtype=np.float32)
        W = np.random.default_rng(1).standard_normal((K, N), dtype=np.float32)
        pl = sharded.plan(M, K, N, rank, world, host_blocks=3)
        c0, c1 = pl["columns"]
        mine = np.lib.format.open_memmap(os.path.join(result_dir, f"c_{rank}.npy"), mode="w+", dtype=np.float32, shape=(M, N))
        mine[:] = np.nan
        mine.flush()
        dist.barrier()
        slab = orc.gemm_f32(A, graphs.dequantise(W[:, c0:c1]))
        assert pl["dest_ranks"][0] == rank and sorted(pl["dest_ranks"]) == list(range(world))
        for r in pl["dest_ranks"]:
            dest = np.load(os.path.join(result_dir, f"c_{r}.npy"), mmap_mode="r+")
            flat = dest.reshape(-1).view(np.uint8)
            for m in range(M):  # row stride ldc = N, first byte of the slab = dest_byte_offset
                start = pl["dest_byte_offset"] + m * N * 4
                flat[start:start + (c1 - c0) * 4] = slab[m].view(np.uint8)
            dest.flush()
        dist.barrier()
        full = np.load(os.path.join(result_dir, f"c_{rank}.npy"))
        assert np.array_equal(full, orc.gemm_f32(A, graphs.dequantise(W)))
        # host-buffer path: row blocks tile [0, M); the ranks' shares tile every block
        shares = [None] * world
        dist.all_gather_object(shares, pl["my_rows"])
        blocks = pl["row_blocks"]
        assert blocks[0][0] == 0 and blocks[-1][1] == M and all(a[1] == b[0] for a, b in zip(blocks, blocks[1:]))
        for i, (m0, m1) in enumerate(blocks):
            parts = [shares[r][i] for r in range(world)]
            assert parts[0][0] == m0 and parts[-1][1] == m1 and all(a[1] == b[0] for a, b in zip(parts, parts[1:]))
    finally:
        dist.destroy_process_group()


def test_sharded_gemm_plan_two_ranks(tmp_path):
    M, K, N = 40, 96, 48
    mp.spawn(_plan_worker, args=(2, _free_port(), M, K, N, str(tmp_path)), nprocs=2, join=True)


def test_plan_arithmetic():
    from fast_arm_tbcnn_b200 import sharded
    assert sharded.destination_order(5, 8) == [5, 6, 7, 0, 1, 2, 3, 4]
    pl = sharded.plan(16384, 16384, 16384, 3, 8)
    assert pl["columns"] == (6144, 8192) and pl["dest_byte_offset"] == 6144 * 4
    assert pl["row_blocks"] == [(i * 2048, (i + 1) * 2048) for i in range(8)]
    assert pl["my_rows"][1] == (2048 + 3 * 256, 2048 + 4 * 256)
    # ragged: 1000 rows over 2 ranks in blocks of whole 256-row units, the last block shorter
    pl = sharded.plan(1000, 64, 64, 1, 2, host_blocks=3)
    assert pl["row_blocks"] == [(0, 512), (512, 1000)]
    assert pl["my_rows"] == [(256, 512), (756, 1000)]
    assert sharded.plan(4096, 4096, 11008, 7, 8)["columns"] == (9632, 11008)


@pytest.mark.parametrize("world", [2])
def test_column_sharded_gemm_two_ranks(tmp_path, world):
    M, K, N = 24, 200, 64
    mp.spawn(_worker, args=(world, _free_port(), M, K, N, str(tmp_path)), nprocs=world, join=True)
    sys.path.insert(0, ROOT)
    from oracle import cpu_oracle, graphs
    orc = cpu_oracle.Oracle()
    A = np.random.default_rng(0).standard_normal((M, K), dtype=np.float32)
    W = np.random.default_rng(1).standard_normal((K, N), dtype=np.float32)
    expect = orc.gemm_f32(A, graphs.dequantise(W))
    got = np.load(tmp_path / "c_full.npy")
    assert np.array_equal(got, expect)


def test_slab_arithmetic():
    from fast_arm_tbcnn_b200 import sharding
    assert sharding.column_slab(3, 8, 16384) == (6144, 8192)
    with pytest.raises(ValueError):
        sharding.column_slab(0, 3, 16384)
    with pytest.raises(ValueError):
        sharding.column_slab(2, 2, 8)
    assert [sharding.batch_block(r, 4, 10) for r in range(4)] == [(0, 3), (3, 6), (6, 8), (8, 10)]
    g = np.arange(2 * 3 * 4, dtype=np.float32).reshape(2, 3, 4)
    out = sharding.interleave_slabs(g)
    assert out.shape == (3, 8) and np.array_equal(out[1], np.concatenate([g[0, 1], g[1, 1]]))
