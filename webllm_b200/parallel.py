"""Multi-GPU use of the quantized linear, one process per GPU (``torch.distributed``: NCCL on GPUs, gloo in
the CPU tests). The reference has a single device (src/gpu/device.ts:40-98); both modes below are new.

* replicas: independent sequences, replicated weights, no communication — nothing to write beyond
  ``replica_share``.
* output-column shards: rank r owns columns ``[r*N/G, (r+1)*N/G)`` of a GPTQ linear (its slice of
  ``qweight[:, cols]``, ``scales[:, cols]``, ``qzeros[:, cols/8]``), the activation is replicated, and one
  all-gather reassembles ``y``. Shard width must be a multiple of 8 so that no qzeros word is split.

torch is plumbing here: it owns the activation slab that the context adopts (``wb_arena_adopt``), so that NCCL
can run on arena tensors in place, and it provides the process group.
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


class TorchSlabGpu:
    """A ``Gpu`` whose activation slab is a torch tensor, so that collectives can run on arena tensors
    without a copy, and whose kernels are enqueued on torch's current stream."""

    def __init__(self, device: int, weight_bytes: int, act_bytes: int):
        import torch

        from .device import Gpu
        self.torch = torch
        self.device = torch.device(f"cuda:{device}")
        torch.cuda.set_device(self.device)
        self.slab = torch.empty(act_bytes, dtype=torch.uint8, device=self.device)
        self.gpu = Gpu(device, weight_bytes=weight_bytes, act_slab=(self.slab.data_ptr(), act_bytes))
        self.gpu.set_stream(torch.cuda.current_stream(self.device).cuda_stream)

    def view(self, t, dtype=None):
        """torch view of an arena tensor."""
        torch = self.torch
        dtype = dtype or (torch.float32 if t.dtype == "f32" else torch.float16)
        return self.slab[t.offset:t.offset + t.nbytes].view(dtype)

    def close(self):
        self.gpu.close()


class PeerSlabGpu:
    """A ``Gpu`` whose activation slab the library allocated itself and that has every other rank's activation slab
    mapped (CUDA IPC, one node), so that ``ColumnShardedLinear.forward_fused`` can store results straight into the
    peers. Tensors are ``(slab, byte offset)`` on every rank: the ranks must make the same sequence of arena
    allocations, so that one offset names the same tensor everywhere. Kernels go to torch's current stream, which
    is also where the barrier's collective is enqueued."""

    def __init__(self, device: int, weight_bytes: int, act_bytes: int, group=None):
        import torch
        import torch.distributed as dist

        from .device import Gpu
        self.torch, self.group = torch, group
        self.device = torch.device(f"cuda:{device}")
        torch.cuda.set_device(self.device)
        self.gpu = Gpu(device, weight_bytes=weight_bytes, act_bytes=act_bytes)
        self.gpu.set_stream(torch.cuda.current_stream(self.device).cuda_stream)
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        handles = [None] * self.world
        dist.all_gather_object(handles, self.gpu.ipc_export(), group=group)
        self.peer_bases = [self.gpu.peer_open(h) for r, h in enumerate(handles) if r != self.rank]
        self._flag = torch.zeros(1, dtype=torch.int32, device=self.device)

    def barrier(self) -> None:
        """Stream-ordered barrier across the ranks: a one-element all-reduce behind the kernels already enqueued."""
        import torch.distributed as dist
        dist.all_reduce(self._flag, group=self.group)

    def close(self) -> None:
        for b in self.peer_bases:
            self.gpu.peer_close(b)
        self.peer_bases = []
        self.gpu.close()


class ColumnShardedLinear:
    """One GPTQ linear split by output columns over the ranks of a process group.

    ``forward(x_tensor, M)`` runs the local ``[M, N/G]`` product with the library's kernels (GEMV for small M,
    tcgen05 GEMM for large M) and all-gathers the pieces over NCCL/NVLink.
    """

    def __init__(self, host: TorchSlabGpu, name: str, t: GptqTensors, bias: np.ndarray | None = None, group=None):
        import torch.distributed as dist
        self.host, self.group = host, group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.N, self.K = t.out_features, t.in_features
        self.shard = column_shard(self.N, self.rank, self.world)
        gpu = host.gpu
        self.weight = gpu.gptq_register(name, t.qweight, t.qzeros, t.scales, t.in_features, t.out_features, t.group_size,
                                        4, cols=(self.shard.begin, self.shard.count))
        self.bias = None
        if bias is not None:
            self.bias = gpu.f32_upload(name + ".bias", bias[self.shard.begin:self.shard.begin + self.shard.count])

    def local(self, A, C_local, M: int, exact: bool = False) -> None:
        self.host.gpu.linear(self.weight, A, C_local, self.bias, M, exact=exact)

    def forward_fused(self, A, C_full, tmp, M: int) -> None:
        """A: arena tensor [M, K] (replicated); C_full: arena tensor [M, N] at the same offset on every rank; tmp:
        arena tensor [M, N/G] (used by decode-size calls only). ``host`` must be a ``PeerSlabGpu``. The kernel of
        every rank stores its columns into all ranks' C_full; after the barrier every rank holds the full, row-major
        [M, N]. The caller must not let any rank reuse C_full for another result before all ranks have read it."""
        self.host.gpu.linear_gather(self.weight, A, C_full, tmp, self.bias, M, self.N, self.shard.begin,
                                    self.host.peer_bases)
        self.host.barrier()

    def forward(self, A, C_local, M: int, exact: bool = False):
        """A: arena tensor [M, K] (replicated), C_local: arena tensor [M, N/G]. Returns a torch tensor [M, N]."""
        self.local(A, C_local, M, exact)
        return gather_columns(self.host.view(C_local), M, self.group)
