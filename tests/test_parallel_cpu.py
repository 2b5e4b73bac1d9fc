"""CPU tests of the multi-GPU host logic: shard planning, host-side GPTQ column slicing against the oracle,
and the all-gather reassembly on a world_size-2 gloo group (the N > 1 path without GPUs)."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

from webllm_b200 import parallel, synthetic  # noqa: E402


def test_replica_share_partitions_sequences():
    shares = [list(parallel.replica_share(256, r, 8)) for r in range(8)]
    assert sorted(sum(shares, [])) == list(range(256)) and all(len(s) == 32 for s in shares)
    assert list(parallel.replica_share(5, 1, 2)) == [1, 3]


def test_column_shard_rules():
    # 7B-class widths split over 1/2/4/8 ranks: 3584, 512 and 18944 all stay multiples of 8
    for N in (3584, 512, 18944):
        for G in (1, 2, 4, 8):
            s = [parallel.column_shard(N, r, G) for r in range(G)]
            assert s[0].begin == 0 and s[-1].begin + s[-1].count == N and all(x.count % 8 == 0 for x in s)
    with pytest.raises(ValueError):
        parallel.column_shard(900, 0, 8)   # not divisible
    with pytest.raises(ValueError):
        parallel.column_shard(128, 0, 32)  # 4 columns per rank would split a qzeros word


def test_slice_matches_slice_of_dequantised_weight(oracle):
    t = synthetic.random_gptq(256, 64, 128, seed=4, zeros="any")
    full = oracle.dequantize_gptq_int4(t.qweight, t.qzeros, t.scales.astype(np.float32), 256, 64, 128)
    for begin, count in ((0, 16), (16, 24), (40, 24)):
        s = parallel.slice_gptq_columns(t, begin, count)
        part = oracle.dequantize_gptq_int4(s.qweight, s.qzeros, s.scales.astype(np.float32), 256, count, 128)
        assert np.array_equal(part.view(np.uint32), full[begin:begin + count].view(np.uint32))
    with pytest.raises(ValueError):
        parallel.slice_gptq_columns(t, 4, 16)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _gloo_rank(rank, world, port, K, N, tmp):
    import torch
    import torch.distributed as dist
    from oracle import oracle
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        t = synthetic.random_gptq(K, N, 128, seed=9, zeros="any")
        W = oracle.dequantize_gptq_int4(t.qweight, t.qzeros, t.scales.astype(np.float32), K, N, 128)
        sh = parallel.column_shard(N, rank, world)
        s = parallel.slice_gptq_columns(t, sh.begin, sh.count)
        Ws = oracle.dequantize_gptq_int4(s.qweight, s.qzeros, s.scales.astype(np.float32), K, sh.count, 128)
        for M in (1, 3):
            x = np.random.default_rng(M).standard_normal((M, K)).astype(np.float32)  # replicated activation
            y_local = oracle.gemm_nt_ref(x, Ws, M, sh.count, K)
            y = parallel.gather_columns(torch.from_numpy(y_local), M).numpy()
            want = oracle.gemm_nt_ref(x, W, M, N, K)
            assert y.shape == (M, N)
            assert np.array_equal(y.view(np.uint32), want.view(np.uint32)), f"rank {rank} M={M}"
        Path(tmp, f"ok{rank}").write_text("ok")
    finally:
        dist.destroy_process_group()


def test_all_gather_reassembly_on_gloo_world2(tmp_path, oracle):
    """Each rank computes its column shard with the oracle; the gathered result equals the unsharded one on
    every rank, for M = 1 (rank-major already row-major) and M = 3 (interleave needed)."""
    import torch.multiprocessing as mp
    port = _free_port()
    mp.spawn(_gloo_rank, args=(2, port, 256, 64, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok0").exists() and (tmp_path / "ok1").exists()
