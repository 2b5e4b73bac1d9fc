"""GPU tests of the output-column-sharded linear: device-side slicing (wb_gptq_register_cols) on one GPU, and the
NCCL all-gather across ranks when at least two GPUs are visible."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest

from helpers import assert_close, oracle_weight, run_linear
from webllm_b200 import WebllmError, parallel, synthetic

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("M", [1, 64])
def test_column_slices_reassemble_to_the_full_product(gpu, oracle, M):
    """Four column shards of a 7B-class k/v projection (3584 -> 512) registered with wb_gptq_register_cols on one
    GPU; their outputs side by side equal the unsharded product (streaming kernel at M=1, tensor cores at M=64)."""
    K, N, G = 3584, 512, 4
    t = synthetic.random_gptq(K, N, 128, seed=21, zeros="any")
    W = oracle_weight(oracle, t)
    x = np.random.default_rng(M).standard_normal((M, K)).astype(np.float16)
    parts = []
    for r in range(G):
        sh = parallel.column_shard(N, r, G)
        name = f"shard{r}_of{G}"
        try:
            h = gpu.weight(name)
        except WebllmError:
            h = gpu.gptq_register(name, t.qweight, t.qzeros, t.scales, K, N, 128, 4, cols=(sh.begin, sh.count))
        parts.append(run_linear(gpu, h, x, M, sh.count, None, act="f16"))
    got = np.concatenate(parts, axis=1)
    Wref = oracle.round_f16(W).reshape(N, K) if M > 16 else W
    ref = oracle.gemm_nt_ref(x.astype(np.float32), Wref, M, N, K, threads=oracle.max_threads())
    assert_close(oracle, got, ref, 1e-3, f"sharded M={M}")
    with pytest.raises(WebllmError, match="multiple of 8"):
        gpu.gptq_register("bad_slice", t.qweight, t.qzeros, t.scales, K, N, 128, 4, cols=(4, 64))


@pytest.mark.parametrize("M", [1, 64, 300])
def test_gather_placement_on_one_gpu(gpu, oracle, M):
    """wb_linear_gather without peers: four column shards of a 3584 -> 512 projection each store their columns of one
    [M, 512] tensor (scatter launch behind the GEMV at M=1, the tensor-core kernel's own epilogue at M=64, its split-K
    reduce at M=300); the tensor equals the unsharded product and the columns next to a shard are left alone."""
    K, N, G = 3584, 512, 4
    t = synthetic.random_gptq(K, N, 128, seed=22, zeros="any")
    W = oracle_weight(oracle, t)
    x = np.random.default_rng(M).standard_normal((M, K)).astype(np.float16)
    bias = np.random.default_rng(3).standard_normal(N).astype(np.float32)
    gpu.arena.reset()
    A = gpu.arena.alloc(M * K, [M, K], "f16")
    Cf = gpu.arena.alloc(M * N, [M, N], "f32")
    tmp = gpu.arena.alloc(M * (N // G), [M, N // G], "f32")
    gpu.write(A, x)
    gpu.write(Cf, np.full(M * N, -7.0, np.float32))
    Wref = oracle.round_f16(W).reshape(N, K) if M > 16 else W
    ref = oracle.gemm_nt_ref(x.astype(np.float32), Wref, M, N, K, bias, threads=oracle.max_threads())
    for r in (2, 0, 3, 1):
        sh = parallel.column_shard(N, r, G)
        name = f"gshard{r}_of{G}"
        try:
            h, hb = gpu.weight(name), gpu.weight(name + ".bias")
        except WebllmError:
            h = gpu.gptq_register(name, t.qweight, t.qzeros, t.scales, K, N, 128, 4, cols=(sh.begin, sh.count))
            hb = gpu.f32_upload(name + ".bias", bias[sh.begin:sh.begin + sh.count])
        gpu.linear_gather(h, A, Cf, tmp, hb, M, N, sh.begin, [])
        got = gpu.read(Cf).reshape(M, N)
        if r == 2:  # first shard written: everything else still holds the fill value
            assert np.all(got[:, :sh.begin] == -7.0) and np.all(got[:, sh.begin + sh.count:] == -7.0)
    assert_close(oracle, got, ref, 1e-3, f"gather placement M={M}")
    with pytest.raises(WebllmError, match="do not fit"):
        gpu.linear_gather(h, A, Cf, tmp, None, M, N, N - 8, [])


def test_gather_from_the_persistent_tile_loop(gpu, oracle):
    """Two column shards of the 0.5B gate projection at M = 2048, enough tiles per shard for the planner to consider
    the persistent tensor-core kernel, whose epilogue warps then do the placement into the [2048, 4864] tensor."""
    K, N, G, M = 896, 4864, 2, 2048
    t = synthetic.random_gptq(K, N, 128, seed=23, zeros="any")
    W = oracle.round_f16(oracle_weight(oracle, t)).reshape(N, K)
    x = np.random.default_rng(7).standard_normal((M, K)).astype(np.float16)
    gpu.arena.reset()
    A = gpu.arena.alloc(M * K, [M, K], "f16")
    Cf = gpu.arena.alloc(M * N, [M, N], "f16")
    tmp = gpu.arena.alloc(M * (N // G), [M, N // G], "f16")
    gpu.write(A, x)
    for r in range(G):
        sh = parallel.column_shard(N, r, G)
        h = gpu.gptq_register(f"pshard{r}", t.qweight, t.qzeros, t.scales, K, N, 128, 4, cols=(sh.begin, sh.count))
        p = gpu.plan(h, M, "f16")
        assert p["kernel_name"] in ("gemm_tc", "gemm_tc_pair") and p["split_k"] == 1
        gpu.linear_gather(h, A, Cf, tmp, None, M, N, sh.begin, [])
    rows = sorted(set(np.random.default_rng(1).integers(0, M, 94).tolist()) | {0, M - 1})  # sampled: the host is slow
    got = gpu.read(Cf).reshape(M, N)[rows].astype(np.float32)
    ref = oracle.gemm_nt_ref(np.ascontiguousarray(x[rows]).astype(np.float32), W, len(rows), N, K, threads=oracle.max_threads())
    ref16 = ref.astype(np.float16).astype(np.float32)  # the output tensor is fp16: round both sides
    assert_close(oracle, got, ref16, 1e-3, "gather from the persistent kernel")
    for _ in range(G):
        gpu.weight_pop()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _nccl_rank(rank, world, port, tmp):
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests"))
    import torch
    import torch.distributed as dist
    from oracle import oracle
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device(f"cuda:{rank}"))
    host = parallel.ShardGroup(rank, weight_bytes=256 << 20, act_bytes=256 << 20)
    gpu = host.gpu
    try:
        K, N = 3584, 3584
        t = synthetic.random_gptq(K, N, 128, seed=5, zeros="any")
        bias = np.random.default_rng(2).standard_normal(N).astype(np.float32)
        lin = parallel.ColumnShardedLinear(host, "q7", t, bias)
        W = oracle.dequantize_gptq_int4(t.qweight, t.qzeros, oracle.f16_bits_to_f32(t.scales.view(np.uint16)), K, N, 128)
        for M in (1, 48, 300):
            x = np.random.default_rng(10 + M).standard_normal((M, K)).astype(np.float16)  # same on every rank
            Wref = oracle.round_f16(W).reshape(N, K) if M > 16 else W
            ref = oracle.gemm_nt_ref(x.astype(np.float32), Wref, M, N, K, bias, threads=4)
            rms = float(np.sqrt(np.mean(ref.astype(np.float64) ** 2)))
            gpu.arena.reset()
            A = gpu.arena.alloc(M * K, [M, K], "f16")
            Cf = gpu.arena.alloc(M * N, [M, N], "f32")
            scratch = gpu.arena.alloc(lin.scratch_elems(M), dtype="f32")
            tmpc = gpu.arena.alloc(M * lin.shard.count, [M, lin.shard.count], "f32")
            gpu.write(A, x)
            # (1) local product + NCCL all-gather enqueued by the library (wb_linear_colshard), row-major result
            lin.forward(A, Cf, scratch, M)
            got = gpu.read(Cf).reshape(M, N)
            r = oracle.check_tolerance(got, ref, 1e-3 * rms, 1e-3)
            assert r.ok, ("colshard", rank, M, r)
            # (2) the all-gather as the kernels' own stores into the peers' slabs + the library's barrier kernel
            gpu.write(Cf, np.zeros(M * N, np.float32))
            gpu.synchronize()
            dist.barrier()  # every rank's tensor is cleared before any peer stores into it
            lin.forward_fused(A, Cf, tmpc, M)
            got = gpu.read(Cf).reshape(M, N)
            r = oracle.check_tolerance(got, ref, 1e-3 * rms, 1e-3)
            assert r.ok, ("fused", rank, M, r)
            dist.barrier()  # nobody clears its tensor for the next M while a peer is still storing
        Path(tmp, f"ok{rank}").write_text("ok")
    finally:
        host.close()
        dist.destroy_process_group()


def test_column_sharded_linear_over_nccl(tmp_path, built_lib, oracle):
    """7B-class 3584 -> 3584 projection split over every visible GPU (2, 4 or 8), decode (M=1) and a batch that
    takes the tensor-core kernel; every rank must end with the same full [M, N] as the unsharded oracle."""
    import torch
    world = torch.cuda.device_count()
    world = 8 if world >= 8 else 4 if world >= 4 else 2 if world >= 2 else 1
    if world < 2:
        pytest.skip("needs at least two GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_nccl_rank, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))


def test_peer_barrier_gives_up_instead_of_hanging(gpu):
    """The wait of the library's barrier kernel is bounded: with a flag word that nobody writes (this GPU stands in for
    its own peer, so only slot 0 is ever stored) it records its code after the time limit, the kernel returns, the next
    synchronize reports WB_ERR_TIMEOUT, and the context keeps working. With both slots served it passes."""
    from webllm_b200 import _lib
    gpu.arena.reset()
    flags = gpu.arena.alloc(_lib.WB_PEER_FLAG_BYTES // 4)
    gpu.peer_barrier_init(flags)
    own = gpu.arena_base()
    gpu.peer_barrier(flags, 0, [own], timeout_us=2000)  # waits for rank 1, which does not exist
    with pytest.raises(WebllmError) as e:
        gpu.synchronize()
    assert e.value.status == _lib.WB_ERR_TIMEOUT
    gpu.synchronize()  # the status word was consumed; the context is usable
    # both "ranks" played by this GPU in turn: rank 1 stores its epoch first, then rank 0 finds it and passes
    gpu.peer_barrier_init(flags)
    words = np.zeros(_lib.WB_PEER_FLAG_BYTES // 4, np.uint32)
    words[1] = 1  # what rank 1's barrier number 1 would have stored into this GPU's flags
    gpu.write_bytes(flags.offset, words)
    gpu.peer_barrier(flags, 0, [own], timeout_us=200000)
    gpu.synchronize()
    with pytest.raises(WebllmError, match="rank"):
        gpu.peer_barrier(flags, 3, [own])


@pytest.mark.parametrize("M", [1, 48])
def test_colshard_entry_point_on_a_one_rank_communicator(gpu, oracle, M):
    """wb_comm_init / wb_linear_colshard through the C ABI with a communicator of one rank (NCCL loaded with dlopen,
    the all-gather of one piece is a copy): the call's bookkeeping, scratch layout and result against the oracle."""
    from webllm_b200 import _lib
    K, N = 3584, 512
    t = synthetic.random_gptq(K, N, 128, seed=31, zeros="any")
    try:
        h = gpu.weight("cs1")
    except WebllmError:
        h = gpu.gptq_register("cs1", t.qweight, t.qzeros, t.scales, K, N, 128)
    with pytest.raises(WebllmError, match="wb_comm_init first"):
        gpu.arena.reset()
        A = gpu.arena.alloc(M * K, [M, K], "f16")
        Cf = gpu.arena.alloc(M * N, [M, N], "f32")
        gpu.linear_colshard(h, A, Cf, Cf, None, M)
    gpu.comm_init(0, 1, gpu.comm_unique_id(), 20000)
    try:
        with pytest.raises(WebllmError) as e:
            gpu.comm_init(0, 1, gpu.comm_unique_id())
        assert e.value.status == _lib.WB_ERR_EXISTS
        W = oracle_weight(oracle, t)
        x = np.random.default_rng(M).standard_normal((M, K)).astype(np.float16)
        gpu.arena.reset()
        A = gpu.arena.alloc(M * K, [M, K], "f16")
        Cf = gpu.arena.alloc(M * N, [M, N], "f32")
        scratch = gpu.arena.alloc(M * N + 64)
        gpu.write(A, x)
        gpu.linear_colshard(h, A, Cf, scratch, None, M)
        got = gpu.read(Cf).reshape(M, N)
        Wref = oracle.round_f16(W).reshape(N, K) if M > 16 else W
        ref = oracle.gemm_nt_ref(x.astype(np.float32), Wref, M, N, K, threads=oracle.max_threads())
        assert_close(oracle, got, ref, 1e-3, f"colshard one rank M={M}")
    finally:
        gpu.comm_destroy()
