"""Column (N) sharding of a fused GEMM stage over the GPUs of one box.

Each output column depends on one weight column, the full activation rows and the per-row
scalars, so a stage shards on N with no exchange: rank g owns columns [g*N/G, (g+1)*N/G) of the
weights, of every per-column vector and of the output; activations, per-row vectors and the RoPE
table are replicated.  The only collective is an all-gather of output shards where the next stage
contracts over those columns (gate/up -> down projection).  The gathered buffer keeps the shards
as G slabs [G][M, N/G]; the consumer GEMM reads it in place through the K-slab layout of its A
operand (xf_gemm_desc.a_k_slab), so nothing is re-interleaved.
"""

SLAB_MULTIPLE = 256  # the K-slab layout needs slab widths that are multiples of 256 elements


def shard_columns(n_cols, world, rank, multiple=2):
    """[start, stop) of the columns rank owns.  Shards are equal and `multiple`-aligned: 2 for
    pair ops, 128 for RoPE heads, the CTA tile width to avoid ragged tiles."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError(f"bad rank {rank} of {world}")
    if n_cols % world != 0:
        raise ValueError(f"{n_cols} columns do not split evenly over {world} ranks")
    per = n_cols // world
    if per % multiple != 0:
        raise ValueError(f"shard width {per} is not a multiple of {multiple}")
    return rank * per, (rank + 1) * per


def stage_multiple(preset, compact=False):
    """Alignment a shard boundary needs for a preset's epilogue."""
    if preset in ("k3", "k4", "k4v2"):
        return 128            # whole heads: the RoPE table repeats every head_dim columns
    if preset in ("k2", "k2_geglu"):
        return 2 * SLAB_MULTIPLE if compact else 2   # compact output shard feeds a K-slab consumer
    return 2


def gathered_shape(m_rows, shard_cols, world):
    """Shape of the all-gathered output: G slabs of [M, N/G]."""
    return (world, m_rows, shard_cols)


def all_gather_shards(dist, shard, gathered, group=None):
    """All-gathers this rank's [M, Ns] output shard into gathered[G][M, Ns] (slab g = rank g's
    columns).  `shard` and `gathered` are contiguous torch tensors on the same device."""
    if tuple(gathered.shape) != (dist.get_world_size(group), *shard.shape):
        raise ValueError(f"gathered buffer {tuple(gathered.shape)} does not match shard {tuple(shard.shape)}")
    if dist.get_backend(group) == "nccl":
        dist.all_gather_into_tensor(gathered, shard, group=group)     # one ncclAllGather, in place
    else:
        dist.all_gather(list(gathered.unbind(0)), shard, group=group)  # gloo (CPU tests)
    return gathered


def slabs_to_matrix(gathered):
    """[G][M, Ns] -> the logical [M, G*Ns] matrix (host-side check helper; copies)."""
    g, m, ns = gathered.shape
    return gathered.permute(1, 0, 2).reshape(m, g * ns)


class GatherBuffer:
    """The [G][M, Ns] gathered buffer of a column-sharded stage in symmetric (peer-mapped) memory.

    Every rank allocates the same buffer and exchanges handles once; afterwards rank r's producer
    GEMM stores each output tile into slab r of EVERY rank's buffer straight from its epilogue
    (xf_gemm_desc.D_peer), so the all-gather overlaps the GEMM instead of following it.  A
    stream-ordered barrier across the ranks then releases the consumer stage, which reads only its
    own (local) copy.  Collective: all ranks construct it, and call barrier(), in the same order.
    """

    def __init__(self, dist, m_rows, shard_cols, dtype, device, group=None):
        import torch
        import torch.distributed._symmetric_memory as symm
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.tensor = symm.empty((self.world, m_rows, shard_cols), dtype=dtype, device=device)
        self.handle = symm.rendezvous(self.tensor, group=self.group)
        self.slab_bytes = m_rows * shard_cols * self.tensor.element_size()
        self.base_ptrs = [int(p) for p in self.handle.buffer_ptrs]
        if len(self.base_ptrs) != self.world:
            raise RuntimeError("symmetric memory rendezvous returned %d pointers for %d ranks"
                               % (len(self.base_ptrs), self.world))

    @property
    def local_shard(self):
        """This rank's slab of its own buffer: the producer stage's D."""
        return self.tensor[self.rank]

    def peer_slab_ptrs(self):
        """Device pointers of slab `rank` in every OTHER rank's buffer (mapped into this process)."""
        off = self.rank * self.slab_bytes
        return [p + off for g, p in enumerate(self.base_ptrs) if g != self.rank]

    def barrier(self):
        """Stream-ordered barrier: returns (on the current stream) once every rank's work enqueued
        before its own barrier() has finished, i.e. once all slabs of the local buffer are complete."""
        self.handle.barrier(channel=0)
