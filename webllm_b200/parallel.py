"""Multi-GPU use of the quantized linear, one process per GPU (``torch.distributed``: NCCL on GPUs, gloo in
the CPU tests). The reference has a single device (src/gpu/device.ts:40-98); both modes below are new.

* replicas: independent sequences, replicated weights, no communication — nothing to write beyond
  ``replica_share``.
* output-column shards: rank r owns columns ``[r*N/G, (r+1)*N/G)`` of a GPTQ linear (its slice of
  ``qweight[:, cols]``, ``scales[:, cols]``, ``qzeros[:, cols/8]``), the activation is replicated, and one
  all-gather reassembles ``y``. Shard width must be a multiple of 8 so that no qzeros word is split.

The exchange itself sits behind the C ABI: ``wb_comm_init`` + ``wb_linear_colshard`` (an NCCL all-gather that the
library enqueues on its own stream) or ``wb_linear_gather_barrier`` (the product's own stores into the peers' slabs
plus the library's barrier kernel). torch is plumbing here: it provides the process group over which the ranks
exchange the communicator id and the IPC handles, and the CPU (gloo) tests of the reassembly.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from .synthetic import GptqTensors


def replica_share(n_items: int, rank: int, world: int) -> range:
    """Round-robin share of ``n_items`` independent sequences for ``rank``."""
    return range(rank, n_items, world)


@dataclass
class ColumnShard:
    begin: int
    count: int


def column_shard(N: int, rank: int, world: int) -> ColumnShard:
    """Equal column shards; refuses widths that would split a qzeros word (8 columns)."""
    if N % world != 0 or (N // world) % 8 != 0:
        raise ValueError(f"N={N} cannot be split into {world} column shards that are multiples of 8")
    return ColumnShard(rank * (N // world), N // world)


def slice_gptq_columns(t: GptqTensors, begin: int, count: int) -> GptqTensors:
    """Host-side slice of a GPTQ linear to output columns [begin, begin+count) (multiples of 8). The C ABI
    can also slice while uploading (``wb_gptq_register_cols``); this is the same cut on numpy arrays."""
    if begin % 8 or count % 8 or begin < 0 or begin + count > t.out_features:
        raise ValueError("column slices must start and end on a multiple of 8 inside the matrix")
    qz = None if t.qzeros is None else np.ascontiguousarray(t.qzeros[:, begin // 8:(begin + count) // 8])
    return GptqTensors(np.ascontiguousarray(t.qweight[:, begin:begin + count]), qz,
                       np.ascontiguousarray(t.scales[:, begin:begin + count]), t.in_features, count, t.group_size)


def gather_columns(y_local, M: int, group=None):
    """All-gathers per-rank ``[M, N/G]`` pieces into the full ``[M, N]`` (torch tensors, any backend).
    The collective delivers rank-major ``[G, M, N/G]``; for M == 1 that already is ``[1, N]``, otherwise the
    pieces are interleaved back to row-major."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    piece = y_local.reshape(M, -1).contiguous()
    out = torch.empty((world, M, piece.shape[1]), dtype=piece.dtype, device=piece.device)
    if dist.get_backend(group) == "nccl":
        dist.all_gather_into_tensor(out, piece, group=group)
    else:  # gloo (CPU tests) has no single-tensor all-gather
        dist.all_gather(list(out.unbind(0)), piece, group=group)
    if M == 1:
        return out.reshape(1, -1)
    return out.permute(1, 0, 2).reshape(M, -1).contiguous()


class ShardGroup:
    """One rank of a column-sharded group: a ``Gpu`` whose activation slab every other rank has mapped (CUDA IPC, one
    node) and, on request, an NCCL communicator owned by the library (``wb_comm_init``).

    Tensors are ``(slab, byte offset)`` on every rank: the ranks must make the same sequence of arena allocations, so
    that one offset names the same tensor everywhere. The slab is made ``WB_PEER_FLAG_BYTES`` larger than asked: those
    last bytes are the flag words of the library's peer barrier (keep arena allocations within ``act_bytes``). Kernels go to torch's current stream so that CUDA events recorded there time them."""

    def __init__(self, device: int, weight_bytes: int, act_bytes: int, group=None, nccl: bool = True, peers: bool = True,
                 comm_timeout_ms: int = 0):
        import torch
        import torch.distributed as dist

        from . import _lib as L
        from .buffer import Tensor
        from .device import Gpu
        self.torch, self.group = torch, group
        self.device = torch.device(f"cuda:{device}")
        torch.cuda.set_device(self.device)
        act_bytes = (act_bytes + 255) // 256 * 256
        self.gpu = Gpu(device, weight_bytes=weight_bytes, act_bytes=act_bytes + L.WB_PEER_FLAG_BYTES)
        self.gpu.set_stream(torch.cuda.current_stream(self.device).cuda_stream)
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.peer_bases: list[int] = []
        self.flags = Tensor(act_bytes, L.WB_PEER_FLAG_BYTES // 4, [L.WB_PEER_FLAG_BYTES // 4], "f32")
        self.has_comm = False
        if peers:
            handles = [None] * self.world
            dist.all_gather_object(handles, self.gpu.ipc_export(), group=group)
            self.peer_bases = [self.gpu.peer_open(h) for r, h in enumerate(handles) if r != self.rank]
            self.gpu.peer_barrier_init(self.flags)
            dist.barrier(group=group)  # every rank's flags are zero before any peer stores into them
        if nccl:
            box = [self.gpu.comm_unique_id() if self.rank == 0 else None]
            dist.broadcast_object_list(box, src=0, group=group)
            self.gpu.comm_init(self.rank, self.world, box[0], comm_timeout_ms)
            self.has_comm = True

    def barrier(self, timeout_us: int = 0) -> None:
        """Stream-ordered barrier across the ranks by the library's own kernel (bounded wait, see ``wb_peer_barrier``)."""
        self.gpu.peer_barrier(self.flags, self.rank, self.peer_bases, timeout_us)

    def close(self) -> None:
        if self.has_comm:
            self.gpu.comm_destroy()
            self.has_comm = False
        for b in self.peer_bases:
            self.gpu.peer_close(b)
        self.peer_bases = []
        self.gpu.close()


class ColumnShardedLinear:
    """One GPTQ linear split by output columns over the ranks of a ``ShardGroup``: rank r registers columns
    ``[r*N/G, (r+1)*N/G)`` and runs the library's kernels on its slice (GEMV for small M, tcgen05 GEMM for large M)."""

    def __init__(self, host: ShardGroup, name: str, t: GptqTensors, bias: np.ndarray | None = None):
        self.host = host
        self.rank, self.world = host.rank, host.world
        self.N, self.K = t.out_features, t.in_features
        self.shard = column_shard(self.N, self.rank, self.world)
        gpu = host.gpu
        self.weight = gpu.gptq_register(name, t.qweight, t.qzeros, t.scales, t.in_features, t.out_features, t.group_size,
                                        4, cols=(self.shard.begin, self.shard.count))
        self.bias = None
        if bias is not None:
            self.bias = gpu.f32_upload(name + ".bias", bias[self.shard.begin:self.shard.begin + self.shard.count])

    def scratch_elems(self, M: int, row_major: bool = True) -> int:
        """Elements of the scratch tensor ``forward`` needs (the local piece, plus the gathered pieces when they have
        to be rearranged to row-major)."""
        piece = M * self.shard.count
        return (piece + 127) // 128 * 128 + (self.world * piece if row_major and M > 1 and self.world > 1 else 0)

    def local(self, A, C_local, M: int, exact: bool = False) -> None:
        self.host.gpu.linear(self.weight, A, C_local, self.bias, M, exact=exact)

    def forward(self, A, C_full, scratch, M: int, row_major: bool = True) -> None:
        """Local product + NCCL all-gather behind the C ABI (``wb_linear_colshard``). A: arena tensor [M, K]
        (replicated); C_full: arena tensor that receives [M, N] row-major (or the rank-major pieces [G, M, N/G] with
        ``row_major=False``); scratch: ``scratch_elems(M, row_major)`` elements of C_full's dtype."""
        self.host.gpu.linear_colshard(self.weight, A, C_full, scratch, self.bias, M, row_major)

    def forward_fused(self, A, C_full, tmp, M: int, timeout_us: int = 0) -> None:
        """The all-gather as the kernels' own stores: every rank's kernel stores its columns into all ranks' C_full
        (same offset everywhere) and the library's barrier kernel follows, so that at this point of the stream every
        rank holds the full, row-major [M, N]. tmp: arena tensor [M, N/G] (decode-size calls only). The caller must not
        let any rank reuse C_full for another result before all ranks have read it (``host.barrier()``)."""
        self.host.gpu.linear_gather_barrier(self.weight, A, C_full, tmp, self.bias, M, self.N, self.shard.begin,
                                            self.host.peer_bases, self.host.flags, self.rank, timeout_us)
