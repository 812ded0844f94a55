"""N-sharded GEMM across the GPUs of one box, one process per GPU.

The reference library is single-GPU (it never calls cudaSetDevice); this is
the multi-GPU form of the same operation.  Output columns are independent:

    C[:, j0:j1] = alpha * A @ B[:, j0:j1] + beta * C[:, j0:j1]

so rank r owns a contiguous block of columns of B and C, A is replicated, and
no data moves between GPUs while computing.  Only when the caller wants the
whole C on every rank is there a collective: one all-gather of the column
blocks (NCCL over NVLink) followed by a copy kernel that interleaves the
gathered [rank][row][col] blocks into row-major [row][all cols].

`torch.distributed` supplies the process group; the GEMM and the interleave are
this library's CUDA kernels, reached through the C ABI.  The two callables can
be replaced (tests on CPU ranks inject host stand-ins to exercise the shard
arithmetic and the collective without a GPU); the defaults have no fallback.

Two further operations go through the library's own communicator (`ckl.Comm`,
NCCL bound inside the C library) and need no process group at all:
`ShardedGemm.gathered` assembles C with the library's copy kernel writing each
row panel straight into every rank's C while the next panel multiplies, and
`ShardedGemm.run_host` is the whole operation on host buffers, every rank
uploading only its own rows of A.  `make_comm` builds the communicator from a
`torch.distributed` group when there is one.
"""

from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class ColumnShard:
    rank: int
    world: int
    col0: int    # first column owned
    width: int   # columns owned (0 for a rank past the end)
    block: int   # nominal block width: every rank but the last non-empty one owns this many


def column_shard(n: int, world: int, rank: int, align: int = 8) -> ColumnShard:
    """Contiguous column block of rank `rank` among `world` ranks.  Block widths are
    multiples of `align` columns (8 keeps every block's first element 16-byte aligned
    for 16-bit types, which the TMA path needs); the tail block takes what is left."""
    if world <= 0 or not (0 <= rank < world) or n < 0 or align <= 0:
        raise ValueError(f"bad shard request n={n} world={world} rank={rank} align={align}")
    per = -(-n // world)                # ceil(n / world)
    block = -(-per // align) * align    # rounded up to the alignment
    col0 = min(rank * block, n)
    width = min(block, n - col0)
    return ColumnShard(rank, world, col0, width, block)


def even_shards(n: int, world: int, align: int = 8) -> bool:
    """True when every rank owns the same number of columns (needed for the gather)."""
    return n % world == 0 and (n // world) % align == 0


class ShardedGemm:
    """One rank's view of an N-sharded GEMM.

    b_shard is the rank's k x width block (row-major, leading dimension `ldb`, which is
    `width` for a packed shard or the full n when the block is a view into the whole B);
    c_shard likewise m x width.  `run` enqueues the local GEMM; `gather` assembles the
    whole C on every rank.
    """

    def __init__(self, ckl, m: int, n: int, k: int, ab_dtype: int, c_dtype: int, world: int,
                 rank: int, local_gemm=None, assemble=None):
        self.ckl = ckl
        self.m, self.n, self.k = m, n, k
        self.ab_dtype, self.c_dtype = ab_dtype, c_dtype
        self.shard = column_shard(n, world, rank)
        self._local_gemm = local_gemm or self._abi_gemm
        self._assemble = assemble or self._abi_assemble

    # -- defaults: the CUDA kernels behind the C ABI -------------------------------
    def _abi_gemm(self, a, b_shard, c_shard, lda, ldb, ldc, alpha, beta, algo, stream):
        self.ckl.gemm_ex(self.ab_dtype, a, b_shard, c_shard, self.c_dtype, self.m,
                         self.shard.width, self.k, lda, ldb, ldc, alpha, beta, algo, stream)

    def _abi_assemble(self, dst, src, elem_size, m, width, parts, stream):
        self.ckl.assemble_column_blocks(dst, src, elem_size, m, width, parts, stream)

    # -- operations -------------------------------------------------------------------
    def run(self, a, b_shard, c_shard, alpha: float, beta: float, *, lda=None, ldb=None, ldc=None,
            algo: int = 0, stream=None) -> None:
        w = self.shard.width
        if w == 0:
            return
        self._local_gemm(a, b_shard, c_shard, self.k if lda is None else lda,
                         w if ldb is None else ldb, w if ldc is None else ldc, alpha, beta, algo,
                         stream)

    def gather(self, c_shard, staging, out_full, group=None, stream=None) -> None:
        """All ranks end with the row-major m x n matrix in `out_full`.  `c_shard` must be the
        packed m x width block, `staging` a world x m x width buffer."""
        import torch.distributed as dist

        if not even_shards(self.n, self.shard.world):
            raise ValueError(
                f"gather needs equal column blocks: n={self.n} is not a multiple of "
                f"world*8={self.shard.world * 8}")
        # [world][m][width] is the row-wise concatenation of the ranks' [m][width] blocks.
        # The collective is ordered against torch's CURRENT stream only, so it is issued with
        # `stream` current: behind the GEMM that wrote c_shard, ahead of the interleave.
        flat = staging.view(self.shard.world * self.m, self.shard.width)
        if stream is not None and hasattr(stream, "cuda_stream"):
            import torch
            with torch.cuda.stream(stream):
                dist.all_gather_into_tensor(flat, c_shard, group=group)
        else:
            if stream is not None and c_shard.is_cuda:
                import torch
                if int(stream) != torch.cuda.current_stream().cuda_stream:
                    raise ValueError("gather: pass a torch stream, or make `stream` the current "
                                     "stream; a raw handle of another stream cannot be ordered "
                                     "against the collective")
            dist.all_gather_into_tensor(flat, c_shard, group=group)
        self._assemble(out_full, staging, c_shard.element_size(), self.m, self.shard.width,
                       self.shard.world, stream)

    def gathered(self, comm, a, b_shard, c_shard, c_full, alpha: float, beta: float, *, lda=None,
                 ldb=None, stream=None) -> None:
        """GEMM and assembly in one call of the C library (ckl_gemm_gathered): `c_full` is a
        buffer from `comm.alloc_shared`; every rank ends with the row-major m x n matrix."""
        comm.gemm_gathered(self.ab_dtype, a, b_shard, c_shard, c_full, self.c_dtype, self.m, self.n,
                           self.k, self.k if lda is None else lda,
                           self.shard.width if ldb is None else ldb, alpha, beta, stream)

    def run_host(self, comm, a_rows_host, b_shard_host, c_shard_host, alpha: float, beta: float) -> None:
        """The whole operation on HOST buffers (ckl_gemm_host_sharded): `a_rows_host` holds only
        the rows of A that `ckl.plan_host_sharded(m, world, rank)` assigns to this rank."""
        comm.gemm_host_sharded(self.ab_dtype, a_rows_host, b_shard_host, c_shard_host, self.c_dtype,
                               self.m, self.shard.width, self.k, alpha, beta)


def make_comm(ckl, world: int, rank: int, group=None, device=None):
    """A `ckl.Comm` for the ranks of a torch.distributed group: rank 0 draws the id, a
    broadcast carries it.  With world == 1 no process group is needed."""
    if world == 1:
        return ckl.Comm(1, 0, None)
    import torch
    import torch.distributed as dist
    uid = torch.zeros(ckl.COMM_ID_BYTES, dtype=torch.uint8)
    if rank == 0:
        uid = torch.frombuffer(bytearray(ckl.comm_unique_id()), dtype=torch.uint8).clone()
    if device is not None:
        uid = uid.to(device)
    dist.broadcast(uid, src=0, group=group)
    return ckl.Comm(world, rank, bytes(uid.cpu().numpy().tobytes()))
