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
