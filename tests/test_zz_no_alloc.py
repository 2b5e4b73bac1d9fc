"""GPU test of wb_gptq_gemv_static, the GEMV entry point for hosts that are not allowed to allocate device
memory where they run the kernel (a real-time loop, a sandboxed plugin that only receives input and output
buffers, an application that owns the whole GPU). Its split-K scratch is a fixed array inside the library
instead of the context workspace, so the call takes nothing but the caller's own device pointers.

The file name sorts last on purpose: a run that stops at the first failure has then already run every
other test. The test needs nothing from the others and also passes alone in a fresh process.

It stages the tensors in device memory owned by the test (torch, standing in for the host application),
calls the entry point through the C ABI twice in a row, and compares each result with the regular
context-based entry point (wb_linear) on the same inputs and with the CPU oracle, within the tolerance the
other linear tests use (the two GPU paths run the same kernel with the same split, so they normally agree bit
for bit). The second call must leave the amount of free device memory unchanged.
"""
import ctypes as C

import numpy as np
import pytest

from helpers import assert_close, oracle_weight, register, run_linear
from webllm_b200 import _lib, synthetic

pytestmark = pytest.mark.gpu

F32_RTOL = 1e-5


def _dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("K,N,M,split,act", [(4864, 896, 1, 8, "f32"), (896, 4864, 3, 2, "f16"), (3584, 512, 8, 0, "f32")])
def test_static_scratch_gemv_matches_context_path(gpu, oracle, K, N, M, split, act):
    import torch
    lib = _lib.load()
    t = synthetic.random_gptq(K, N, 128, seed=K + N + M, zeros="any")
    bias = np.random.default_rng(N).standard_normal(N).astype(np.float32)
    np_act = np.float32 if act == "f32" else np.float16
    xs = [np.random.default_rng(s).standard_normal((M, K)).astype(np_act) for s in (1, 2)]

    W = oracle_weight(oracle, t)
    oracle_ref = [oracle.gemm_nt_ref(x.astype(np.float32), W, M, N, K, bias, threads=oracle.max_threads()) for x in xs]

    # regular path: context, registered weight, workspace scratch, same split
    h = register(gpu, f"static_ref_{K}x{N}x{M}", t)
    hb = gpu.f32_upload(f"static_refb_{K}x{N}x{M}", bias)
    gpu.plan_override(_lib.WB_KERNEL_GEMV_MMA, split)
    try:
        want = [run_linear(gpu, h, x, M, N, hb, act=act) for x in xs]
        used_split = gpu.plan(h, M, act)["split_k"]
    finally:
        gpu.plan_override(0, 0)

    # allocation-free path: the test owns every buffer, the library brings only its static array
    d_qw, d_qz, d_sc, d_b = _dev(torch, t.qweight), _dev(torch, t.qzeros), _dev(torch, t.scales.view(np.int16)), _dev(torch, bias)
    d_y = torch.empty((M, N), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    free_after_first = None
    for call, (x, ref, oref) in enumerate(zip(xs, want, oracle_ref)):  # two calls in a row share (and must each re-initialise) the scratch
        d_x = _dev(torch, x.view(np.int16) if act == "f16" else x)
        d_y.fill_(float("nan"))
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        rc = lib.wb_gptq_gemv_static(d_qw.data_ptr(), d_qz.data_ptr(), d_sc.data_ptr(), d_x.data_ptr(), d_y.data_ptr(),
                                     d_b.data_ptr(), K, N, 128, M, _lib.WB_F32 if act == "f32" else _lib.WB_F16,
                                     _lib.WB_F32, used_split, None)
        assert rc == 0, lib.wb_last_error().decode()
        torch.cuda.synchronize()
        if call == 1:  # the first call on a device may set up the module; from then on nothing is allocated
            assert torch.cuda.mem_get_info()[0] == free_before
        got = d_y.cpu().numpy()
        assert_close(oracle, got, ref, F32_RTOL, f"static K={K} N={N} M={M} split={used_split}")
        assert_close(oracle, got, oref, F32_RTOL if act == "f32" else 1e-3, f"static vs oracle K={K} N={N} M={M}")


def test_static_scratch_limits_are_refused_not_truncated(built_lib):
    import torch
    lib = _lib.load()
    buf = torch.zeros(1 << 20, dtype=torch.int32, device="cuda")
    p = buf.data_ptr()
    # split_k * M * N * 4 beyond the 4 MiB of static partial sums
    rc = lib.wb_gptq_gemv_static(p, None, p, p, p, None, 3584, 16384, 128, 32, _lib.WB_F16, _lib.WB_F32, 8, None)
    assert rc == _lib.WB_ERR_UNSUPPORTED and b"exceed the static scratch" in lib.wb_last_error()
    rc = lib.wb_gptq_gemv_static(p, None, p, p, p, None, 896, 4864, 128, 33, _lib.WB_F16, _lib.WB_F32, 0, None)
    assert rc == _lib.WB_ERR_UNSUPPORTED and b"M <= 32" in lib.wb_last_error()
    rc = lib.wb_gptq_gemv_static(None, None, p, p, p, None, 896, 4864, 128, 1, _lib.WB_F16, _lib.WB_F32, 0, None)
    assert rc == _lib.WB_ERR_BAD_ARG
    # pointers into the middle of a buffer that break the kernel's vector accesses are refused on the host:
    # (argument index, byte offset that breaks its rule) for qweight, qzeros, scales, x, y, bias
    for arg, off, word in ((0, 4, b"16-byte"), (3, 8, b"16-byte"), (4, 4, b"16-byte"), (2, 4, b"8-byte"), (1, 2, b"4-byte"),
                           (5, 2, b"4-byte")):
        ptrs = [p, p, p, p, p, p]
        ptrs[arg] = p + off
        rc = lib.wb_gptq_gemv_static(ptrs[0], ptrs[1], ptrs[2], ptrs[3], ptrs[4], ptrs[5], 896, 4864, 128, 1, _lib.WB_F16,
                                     _lib.WB_F32, 0, None)
        assert rc == _lib.WB_ERR_BAD_ARG and word in lib.wb_last_error(), (arg, off, lib.wb_last_error())
