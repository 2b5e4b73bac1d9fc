"""ctypes binding of ``libwebllm_b200.so`` — the Python stand-in for the N-API/FFI binding a TypeScript
host would use. Every signature below is the one declared in ``include/webllm_b200.h``.

There is no CPU fallback: if the library is missing, or no B200 is visible when a context is created,
the call raises.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libwebllm_b200.so"

WB_OK = 0
WB_ERR_BAD_ARG, WB_ERR_OOM, WB_ERR_CUDA, WB_ERR_NCCL = -1, -2, -3, -4
WB_ERR_TIMEOUT, WB_ERR_NOT_FOUND, WB_ERR_EXISTS, WB_ERR_UNSUPPORTED = -5, -6, -7, -8
WB_F32, WB_F16 = 0, 1
WB_ARENA_WEIGHTS, WB_ARENA_ACT = 0, 1
WB_IPC_HANDLE_BYTES = 64
WB_PEER_FLAG_BYTES = 256
WB_COMM_ID_BYTES = 128
WB_KERNEL_GEMV_MMA, WB_KERNEL_GEMM_TC, WB_KERNEL_GENERIC, WB_KERNEL_DENSE_GEMV, WB_KERNEL_GEMV_STREAM = 1, 2, 3, 4, 5
WB_KERNEL_GEMM_TC_PAIR = 6
KERNEL_NAMES = {1: "gemv_mma", 2: "gemm_tc", 3: "generic", 4: "dense_gemv", 5: "gemv_stream", 6: "gemm_tc_pair"}


class WebllmError(RuntimeError):
    """A non-zero wb_status; ``.status`` is the code, the message is ``wb_last_error()``."""

    def __init__(self, status: int, message: str):
        super().__init__(message)
        self.status = status


class Plan(C.Structure):
    _fields_ = [("kernel", C.c_int32), ("split_k", C.c_int32), ("grid_x", C.c_int32), ("grid_y", C.c_int32),
                ("grid_z", C.c_int32), ("block", C.c_int32), ("tile_m", C.c_int32), ("tile_n", C.c_int32),
                ("launches", C.c_int32), ("scratch_bytes", C.c_uint64)]

    def as_dict(self) -> dict:
        d = {n: getattr(self, n) for n, _ in self._fields_}
        d["kernel_name"] = KERNEL_NAMES.get(self.kernel, "?")
        return d


class QwenConfigC(C.Structure):
    _fields_ = [("vocab_size", C.c_int32), ("n_layer", C.c_int32), ("n_head", C.c_int32), ("n_kv_head", C.c_int32),
                ("n_embd", C.c_int32), ("intermediate", C.c_int32), ("max_t", C.c_int32), ("kv_dtype", C.c_int32),
                ("rms_eps", C.c_float), ("rope_theta", C.c_float)]


_vp, _u64, _i64, _i32 = C.c_void_p, C.c_uint64, C.c_int64, C.c_int

# name -> argtypes (restype is int unless listed in _RESTYPES). Kept in one table so that the test that
# compares exported symbols with the header has a single place to look.
SIGNATURES = {
    "wb_last_error": [],
    "wb_version": [],
    "wb_context_create": [_i32, C.POINTER(_vp)],
    "wb_context_destroy": [_vp],
    "wb_set_stream": [_vp, _vp],
    "wb_get_stream": [_vp, C.POINTER(_vp)],
    "wb_synchronize": [_vp],
    "wb_launch_count": [_vp, C.POINTER(_u64)],
    "wb_arena_create": [_vp, _i32, _u64],
    "wb_arena_adopt": [_vp, _i32, _vp, _u64],
    "wb_arena_alloc": [_vp, _i32, _u64, C.POINTER(_u64)],
    "wb_arena_reset": [_vp, _i32],
    "wb_arena_used": [_vp, _i32, C.POINTER(_u64), C.POINTER(_u64)],
    "wb_arena_rewind": [_vp, _i32, _u64],
    "wb_arena_base": [_vp, _i32, C.POINTER(_vp)],
    "wb_upload": [_vp, _i32, _u64, _vp, _u64],
    "wb_download": [_vp, _i32, _u64, _vp, _u64],
    "wb_gptq_register": [_vp, C.c_char_p, _vp, _u64, _vp, _u64, _vp, _u64, _i64, _i64, _i64, _i32,
                         C.POINTER(C.c_int32)],
    "wb_gptq_register_cols": [_vp, C.c_char_p, _vp, _u64, _vp, _u64, _vp, _u64, _i64, _i64, _i64, _i32, _i64, _i64,
                              C.POINTER(C.c_int32)],
    "wb_f16_alloc": [_vp, C.c_char_p, _i64, _i64, C.POINTER(C.c_int32)],
    "wb_f16_write_chunk": [_vp, C.c_int32, _i64, _vp, _i64],
    "wb_f16_write_bits": [_vp, C.c_int32, _i64, _vp, _i64],
    "wb_f32_upload": [_vp, C.c_char_p, _vp, _i64, C.POINTER(C.c_int32)],
    "wb_weight_lookup": [_vp, C.c_char_p, C.POINTER(C.c_int32)],
    "wb_weight_pop": [_vp],
    "wb_read_weight_f16": [_vp, C.c_int32, _i64, _i64, _vp],
    "wb_weight_bytes": [_vp, C.POINTER(_u64)],
    "wb_gptq_dequant_f32": [_vp, C.c_int32, _u64],
    "wb_gptq_dequant_f16": [_vp, C.c_int32, _u64],
    "wb_linear": [_vp, C.c_int32, _u64, _u64, C.c_int32, _i64, _i32, _i32, _i32],
    "wb_linear_gather": [_vp, C.c_int32, _u64, _u64, _u64, C.c_int32, _i64, _i32, _i32, _i64, _i64, C.POINTER(_vp), _i32],
    "wb_arena_ipc_export": [_vp, _i32, _vp],
    "wb_peer_open": [_vp, _vp, C.POINTER(_vp)],
    "wb_peer_close": [_vp, _vp],
    "wb_peer_barrier_init": [_vp, _u64],
    "wb_peer_barrier": [_vp, _u64, _i32, C.POINTER(_vp), _i32, C.c_uint32],
    "wb_linear_gather_barrier": [_vp, C.c_int32, _u64, _u64, _u64, C.c_int32, _i64, _i32, _i32, _i64, _i64, C.POINTER(_vp), _i32,
                                 _u64, _i32, C.c_uint32],
    "wb_comm_unique_id": [_vp],
    "wb_comm_init": [_vp, _i32, _i32, _vp, _i32],
    "wb_comm_destroy": [_vp],
    "wb_linear_colshard": [_vp, C.c_int32, _u64, _u64, _u64, C.c_int32, _i64, _i32, _i32, _i32],
    "wb_read_sweep": [_vp, _i32, _u64, _u64, _i32],
    "wb_plan_query": [_vp, C.c_int32, _i64, _i32, _i32, C.POINTER(Plan)],
    "wb_plan_override": [_vp, _i32, _i32],
    "wb_linear_hint_next": [_vp, _i32],
    "wb_batch_begin": [_vp],
    "wb_batch_end": [_vp, C.POINTER(_vp)],
    "wb_batch_submit": [_vp],
    "wb_batch_destroy": [_vp],
    "wb_qwen_create": [_vp, C.POINTER(QwenConfigC), C.POINTER(_vp)],
    "wb_qwen_destroy": [_vp],
    "wb_qwen_reset_cache": [_vp],
    "wb_qwen_cache_len": [_vp, C.POINTER(_i64)],
    "wb_qwen_set_exact": [_vp, _i32],
    "wb_qwen_forward": [_vp, _vp, _i64, _i64, C.POINTER(_u64)],
    "wb_qwen_prefill": [_vp, _vp, _i64, _i32, C.POINTER(_u64)],
    "wb_qwen_decode_step": [_vp, C.c_uint32, C.POINTER(_u64)],
    "wb_qwen_decode_greedy": [_vp, C.c_uint32, _i64, _vp],
    "wb_qwen_last_logits": [_vp, _vp],
    "wb_gptq_gemv_static": [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i32, _i32, _i32, _vp],
}
_RESTYPES = {"wb_last_error": C.c_char_p}

_lib = None


def load():
    """Loads the shared library (once). Raises if it has not been built: there is nothing to fall back to."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise WebllmError(WB_ERR_UNSUPPORTED,
                              f"{LIB_PATH} is missing: build it with `python -m webllm_b200.build` "
                              "(this package has no CPU or eager fallback)")
        lib = C.CDLL(str(LIB_PATH))
        for name, argtypes in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = _RESTYPES.get(name, C.c_int)
        _lib = lib
    return _lib


def check(status: int) -> None:
    if status != WB_OK:
        raise WebllmError(status, load().wb_last_error().decode("utf-8", "replace"))
