"""Host-side partitioning of the path across the GPUs of one box (one process per GPU).

Large GEMM: the weight columns are sharded.  In the packed layout a column slab is one contiguous
range of words, so a rank packs (or slices) only its own columns; A is replicated; after ONE
all-gather the per-rank slabs [M, N/G] sit as [G, M, N/G] and are interleaved into row-major C.
Conv / CNN batches: images are independent, each rank takes a contiguous block, no collective.

Pure index arithmetic (no torch, no CUDA) so that the CPU tests can exercise it with gloo ranks.
"""


def column_slab(rank, world, n_cols):
    """[begin, end) of the weight/output columns owned by `rank`.  Requires n_cols % world == 0
    (equal slabs keep the all-gather a plain, unpadded collective)."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    if n_cols % world != 0:
        raise ValueError(f"{n_cols} columns do not divide evenly over {world} ranks")
    per = n_cols // world
    return rank * per, (rank + 1) * per


def batch_block(rank, world, batch):
    """[begin, end) of the images owned by `rank`; the first batch % world ranks take one more."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    base, extra = divmod(batch, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def interleave_slabs(gathered):
    """numpy statement of tbn_gather_cols_permute: [G, M, Nc] -> [M, G*Nc]."""
    g, m, nc = gathered.shape
    return gathered.transpose(1, 0, 2).reshape(m, g * nc)
