"""One GPU context: slabs, transfers, weights, linear calls. The role of ``GpuContext`` + ``Arena`` +
the upload helpers of the reference (src/gpu/device.ts, src/gpu/arena.ts, src/gpu/buffer.ts)."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib as L
from .buffer import Tensor


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


class Gpu:
    """``initGpu`` (src/gpu/device.ts:40-98): opens CUDA device ``device`` and two slabs — weights and
    activations (the reference's documented group0 / group1 split)."""

    def __init__(self, device: int = 0, weight_bytes: int = 1 << 30, act_bytes: int = 256 << 20,
                 weight_slab: tuple[int, int] | None = None, act_slab: tuple[int, int] | None = None):
        self._lib = L.load()
        self._ctx = C.c_void_p()
        L.check(self._lib.wb_context_create(device, C.byref(self._ctx)))
        self.device = device
        for arena, slab, size in ((L.WB_ARENA_WEIGHTS, weight_slab, weight_bytes), (L.WB_ARENA_ACT, act_slab, act_bytes)):
            if slab is not None:  # (device pointer, bytes) owned by the caller, e.g. a torch tensor
                L.check(self._lib.wb_arena_adopt(self._ctx, arena, C.c_void_p(slab[0]), slab[1]))
            else:
                L.check(self._lib.wb_arena_create(self._ctx, arena, size))
        self.arena = Arena(self)

    # -- lifetime
    def close(self) -> None:
        if self._ctx:
            self._lib.wb_context_destroy(self._ctx)
            self._ctx = C.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def ctx(self):
        return self._ctx

    def synchronize(self) -> None:
        L.check(self._lib.wb_synchronize(self._ctx))

    def set_stream(self, cuda_stream: int | None) -> None:
        L.check(self._lib.wb_set_stream(self._ctx, C.c_void_p(cuda_stream or 0)))

    @property
    def stream(self) -> int:
        s = C.c_void_p()
        L.check(self._lib.wb_get_stream(self._ctx, C.byref(s)))
        return s.value or 0

    @property
    def launch_count(self) -> int:
        n = C.c_uint64()
        L.check(self._lib.wb_launch_count(self._ctx, C.byref(n)))
        return n.value

    def arena_base(self, arena: int = L.WB_ARENA_ACT) -> int:
        p = C.c_void_p()
        L.check(self._lib.wb_arena_base(self._ctx, arena, C.byref(p)))
        return p.value or 0

    # -- transfers (writeF32 / readbackF32, src/gpu/buffer.ts:37-52,123-145)
    def write(self, t: Tensor, data: np.ndarray, elem_offset: int = 0) -> None:
        want = np.float32 if t.dtype == "f32" else np.float16
        a = np.ascontiguousarray(data, dtype=want).ravel()
        if elem_offset + a.size > t.length:
            raise L.WebllmError(L.WB_ERR_BAD_ARG, f"write of {a.size} elements at {elem_offset} exceeds tensor of {t.length}")
        L.check(self._lib.wb_upload(self._ctx, L.WB_ARENA_ACT, t.offset + elem_offset * t.itemsize, _ptr(a), a.nbytes))

    def write_bytes(self, offset: int, data: np.ndarray) -> None:
        a = np.ascontiguousarray(data)
        L.check(self._lib.wb_upload(self._ctx, L.WB_ARENA_ACT, offset, _ptr(a), a.nbytes))

    def read(self, t: Tensor, elem_offset: int = 0, count: int | None = None) -> np.ndarray:
        count = t.length - elem_offset if count is None else count
        if elem_offset < 0 or elem_offset + count > t.length:
            raise L.WebllmError(L.WB_ERR_BAD_ARG, "read outside tensor")
        out = np.empty(count, np.float32 if t.dtype == "f32" else np.float16)
        L.check(self._lib.wb_download(self._ctx, L.WB_ARENA_ACT, t.offset + elem_offset * t.itemsize, _ptr(out), out.nbytes))
        return out

    # -- weights
    def gptq_register(self, name: str, qweight, qzeros, scales_f16, in_features: int, out_features: int,
                      group_size: int = 128, bits: int = 4, cols: tuple[int, int] | None = None) -> int:
        qw = np.ascontiguousarray(qweight).view(np.uint8).ravel()
        qz = None if qzeros is None else np.ascontiguousarray(qzeros).view(np.uint8).ravel()
        sc = np.ascontiguousarray(scales_f16)
        if sc.dtype != np.float16 and sc.dtype != np.uint16:
            raise L.WebllmError(L.WB_ERR_BAD_ARG, "scales must be fp16 (np.float16 or raw uint16 bits)")
        sc = sc.view(np.uint16).ravel()
        h = C.c_int32(-1)
        args = [self._ctx, name.encode(), _ptr(qw), qw.size, None if qz is None else _ptr(qz),
                0 if qz is None else qz.size, _ptr(sc), sc.size, in_features, out_features, group_size, bits]
        if cols is None:
            L.check(self._lib.wb_gptq_register(*args, C.byref(h)))
        else:
            L.check(self._lib.wb_gptq_register_cols(*args, cols[0], cols[1], C.byref(h)))
        return h.value

    def f16_alloc(self, name: str, rows: int, cols: int) -> int:
        h = C.c_int32(-1)
        L.check(self._lib.wb_f16_alloc(self._ctx, name.encode(), rows, cols, C.byref(h)))
        return h.value

    def f16_write_chunk(self, h: int, elem_offset: int, data) -> None:
        a = np.ascontiguousarray(data, dtype=np.float32).ravel()
        L.check(self._lib.wb_f16_write_chunk(self._ctx, h, elem_offset, _ptr(a), a.size))

    def f16_write_bits(self, h: int, elem_offset: int, bits) -> None:
        a = np.ascontiguousarray(bits).view(np.uint16).ravel()
        L.check(self._lib.wb_f16_write_bits(self._ctx, h, elem_offset, _ptr(a), a.size))

    def f32_upload(self, name: str, data) -> int:
        a = np.ascontiguousarray(data, dtype=np.float32).ravel()
        h = C.c_int32(-1)
        L.check(self._lib.wb_f32_upload(self._ctx, name.encode(), _ptr(a), a.size, C.byref(h)))
        return h.value

    def weight(self, name: str) -> int:
        h = C.c_int32(-1)
        L.check(self._lib.wb_weight_lookup(self._ctx, name.encode(), C.byref(h)))
        return h.value

    def weight_pop(self) -> None:
        L.check(self._lib.wb_weight_pop(self._ctx))

    def read_weight_f16(self, h: int, elem_offset: int, count: int) -> np.ndarray:
        out = np.empty(count, np.uint16)
        L.check(self._lib.wb_read_weight_f16(self._ctx, h, elem_offset, count, _ptr(out)))
        return out

    @property
    def weight_bytes(self) -> int:
        n = C.c_uint64()
        L.check(self._lib.wb_weight_bytes(self._ctx, C.byref(n)))
        return n.value

    # -- kernels
    def gptq_dequant(self, h: int, out: Tensor) -> None:
        fn = self._lib.wb_gptq_dequant_f32 if out.dtype == "f32" else self._lib.wb_gptq_dequant_f16
        L.check(fn(self._ctx, h, out.offset))

    def linear(self, weight: int, A: Tensor, Cout: Tensor, bias: int | None, M: int, exact: bool = False) -> None:
        L.check(self._lib.wb_linear(self._ctx, weight, A.offset, Cout.offset, -1 if bias is None else bias, M,
                                    L.WB_F32 if A.dtype == "f32" else L.WB_F16,
                                    L.WB_F32 if Cout.dtype == "f32" else L.WB_F16, 1 if exact else 0))

    def linear_gather(self, weight: int, A: Tensor, C_full: Tensor, tmp: Tensor, bias: int | None, M: int, n_total: int,
                      col_begin: int, peer_bases: list[int]) -> None:
        """Column-sharded linear whose kernel stores its columns of the ``[M, n_total]`` result into this GPU's
        slab and into every peer slab (``wb_linear_gather``); the caller barriers across the ranks afterwards."""
        arr = (C.c_void_p * max(1, len(peer_bases)))(*peer_bases)
        L.check(self._lib.wb_linear_gather(self._ctx, weight, A.offset, C_full.offset, tmp.offset,
                                           -1 if bias is None else bias, M,
                                           L.WB_F32 if A.dtype == "f32" else L.WB_F16,
                                           L.WB_F32 if C_full.dtype == "f32" else L.WB_F16, n_total, col_begin, arr,
                                           len(peer_bases)))

    def linear_gather_barrier(self, weight: int, A: Tensor, C_full: Tensor, tmp: Tensor, bias: int | None, M: int,
                              n_total: int, col_begin: int, peer_bases: list[int], flags: Tensor, rank: int,
                              timeout_us: int = 0) -> None:
        """``linear_gather`` followed by the library's own peer barrier (``wb_linear_gather_barrier``): when the
        stream reaches the end of this call, every rank's columns are in this GPU's ``C_full``."""
        arr = (C.c_void_p * max(1, len(peer_bases)))(*peer_bases)
        L.check(self._lib.wb_linear_gather_barrier(self._ctx, weight, A.offset, C_full.offset, tmp.offset,
                                                   -1 if bias is None else bias, M,
                                                   L.WB_F32 if A.dtype == "f32" else L.WB_F16,
                                                   L.WB_F32 if C_full.dtype == "f32" else L.WB_F16, n_total, col_begin,
                                                   arr, len(peer_bases), flags.offset, rank, timeout_us))

    def peer_barrier_init(self, flags: Tensor) -> None:
        """Zeroes the barrier's flag words (``WB_PEER_FLAG_BYTES`` of the activation slab) and the epoch counter."""
        L.check(self._lib.wb_peer_barrier_init(self._ctx, flags.offset))

    def peer_barrier(self, flags: Tensor, rank: int, peer_bases: list[int], timeout_us: int = 0) -> None:
        """Stream-ordered barrier across the ranks by the library's own kernel (``wb_peer_barrier``); a wait that
        runs out surfaces as WB_ERR_TIMEOUT from the next ``synchronize``."""
        arr = (C.c_void_p * max(1, len(peer_bases)))(*peer_bases)
        L.check(self._lib.wb_peer_barrier(self._ctx, flags.offset, rank, arr, len(peer_bases), timeout_us))

    # -- NCCL communicator behind the C ABI (loaded with dlopen on first use)
    def comm_unique_id(self) -> bytes:
        buf = C.create_string_buffer(L.WB_COMM_ID_BYTES)
        L.check(self._lib.wb_comm_unique_id(buf))
        return buf.raw

    def comm_init(self, rank: int, nranks: int, unique_id: bytes, timeout_ms: int = 0) -> None:
        L.check(self._lib.wb_comm_init(self._ctx, rank, nranks, C.c_char_p(unique_id), timeout_ms))

    def comm_destroy(self) -> None:
        L.check(self._lib.wb_comm_destroy(self._ctx))

    def linear_colshard(self, weight: int, A: Tensor, C_full: Tensor, scratch: Tensor, bias: int | None, M: int,
                        row_major: bool = True) -> None:
        """Local product of this rank's columns + NCCL all-gather of the pieces (``wb_linear_colshard``)."""
        L.check(self._lib.wb_linear_colshard(self._ctx, weight, A.offset, C_full.offset, scratch.offset,
                                             -1 if bias is None else bias, M,
                                             L.WB_F32 if A.dtype == "f32" else L.WB_F16,
                                             L.WB_F32 if C_full.dtype == "f32" else L.WB_F16, 1 if row_major else 0))

    def ipc_export(self, arena: int = L.WB_ARENA_ACT) -> bytes:
        """Handle of a slab of this context for another process on the same node (``wb_arena_ipc_export``)."""
        buf = C.create_string_buffer(L.WB_IPC_HANDLE_BYTES)
        L.check(self._lib.wb_arena_ipc_export(self._ctx, arena, buf))
        return buf.raw

    def peer_open(self, handle: bytes) -> int:
        base = C.c_void_p()
        L.check(self._lib.wb_peer_open(self._ctx, C.c_char_p(handle), C.byref(base)))
        return base.value

    def peer_close(self, base: int) -> None:
        L.check(self._lib.wb_peer_close(self._ctx, C.c_void_p(base)))

    def read_sweep(self, offset: int, nbytes: int, ctas: int, arena: int = L.WB_ARENA_WEIGHTS) -> None:
        """One pass of plain reads over a byte range of a slab (``wb_read_sweep``), for bandwidth comparisons."""
        L.check(self._lib.wb_read_sweep(self._ctx, arena, offset, nbytes, ctas))

    def hint_next(self, weight: int | None) -> None:
        """The next ``linear`` call also asks the L2 to fetch ``weight``, which a later call will stream."""
        L.check(self._lib.wb_linear_hint_next(self._ctx, -1 if weight is None else weight))

    def plan(self, weight: int, M: int, act_dtype: str = "f32", exact: bool = False) -> dict:
        p = L.Plan()
        L.check(self._lib.wb_plan_query(self._ctx, weight, M, L.WB_F32 if act_dtype == "f32" else L.WB_F16,
                                        1 if exact else 0, C.byref(p)))
        return p.as_dict()

    def batch(self) -> "CommandBatch":
        return CommandBatch(self)

    def plan_override(self, kernel: int = 0, split_k: int = 0) -> None:
        L.check(self._lib.wb_plan_override(self._ctx, kernel, split_k))


class CommandBatch:
    """``CommandBatch`` (src/gpu/pipeline.ts:55-117): ``with gpu.batch() as b: gpu.linear(...)`` records the
    calls; ``b.submit()`` enqueues the whole recording at once and can be repeated."""

    def __init__(self, gpu: "Gpu"):
        self._gpu, self._handle = gpu, C.c_void_p()

    def __enter__(self):
        L.check(self._gpu._lib.wb_batch_begin(self._gpu.ctx))
        return self

    def __exit__(self, exc_type, exc, tb):
        rc = self._gpu._lib.wb_batch_end(self._gpu.ctx, C.byref(self._handle))
        if exc_type is None:
            L.check(rc)
        return False

    def submit(self) -> None:
        L.check(self._gpu._lib.wb_batch_submit(self._handle))

    def destroy(self) -> None:
        if self._handle:
            self._gpu._lib.wb_batch_destroy(self._handle)
            self._handle = C.c_void_p()


class Arena:
    """``Arena`` (src/gpu/arena.ts:17-59) over one device slab: bump allocation with 256-byte alignment,
    ``reset()`` recycles everything since the last reset."""

    def __init__(self, gpu: Gpu, which: int = L.WB_ARENA_ACT):
        self._gpu, self._which = gpu, which

    @property
    def used_bytes(self) -> int:
        u, c = C.c_uint64(), C.c_uint64()
        L.check(self._gpu._lib.wb_arena_used(self._gpu.ctx, self._which, C.byref(u), C.byref(c)))
        return u.value

    @property
    def capacity(self) -> int:
        u, c = C.c_uint64(), C.c_uint64()
        L.check(self._gpu._lib.wb_arena_used(self._gpu.ctx, self._which, C.byref(u), C.byref(c)))
        return c.value

    def reset(self) -> None:
        L.check(self._gpu._lib.wb_arena_reset(self._gpu.ctx, self._which))

    def rewind(self, mark: int) -> None:
        """Hands back everything allocated since ``used_bytes`` was ``mark``."""
        L.check(self._gpu._lib.wb_arena_rewind(self._gpu.ctx, self._which, mark))

    def alloc(self, length: int, shape=None, dtype: str = "f32") -> Tensor:
        off = C.c_uint64()
        L.check(self._gpu._lib.wb_arena_alloc(self._gpu.ctx, self._which, length * (4 if dtype == "f32" else 2), C.byref(off)))
        return Tensor(off.value, length, list(shape) if shape is not None else [length], dtype)

    def alloc_float32(self, length: int, shape=None) -> Tensor:
        """``allocFloat32(length, shape)``."""
        return self.alloc(length, shape, "f32")
