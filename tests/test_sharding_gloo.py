"""N-sharded linears on two CPU ranks (gloo): shard + oracle product + all-gather == unsharded oracle."""

import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import lqq_oracle as O
from tests.helpers import random_lqq, random_tokens, to_torch_qw


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from liquidgemm_b200 import sharding
        N, K, M = 512, 256, 6
        qw = random_lqq(N, K, 64, seed=5)
        x, ascale = random_tokens(M, K, seed=6)
        full = O.w4a8_matmul(x, ascale, qw)
        tq = to_torch_qw(qw, device="cpu")
        sh = sharding.shard_weight(tq, rank, world)
        lo, hi = sharding.shard_range(N, rank, world)
        assert (sh.N, sh.K) == (N // world, K) and sh.s_u8.shape == (N // world, K // 64)
        # quantising the shard alone equals slicing the quantised matrix (all statistics are per row)
        W = O.synth_weight(N, K, seed=9).astype(np.float32)
        q_full, q_part = O.quantize_weight(W, 64), O.quantize_weight(W[lo:hi], 64)
        assert np.array_equal(q_full.qweight_u4[lo:hi], q_part.qweight_u4)
        assert np.array_equal(q_full.s1[lo:hi], q_part.s1)
        part = O.LQQWeight(sh.qweight_u4.numpy(), sh.s_u8.numpy(), sh.offset_a.numpy(), sh.s1.numpy(), 64)
        y_local = torch.from_numpy(O.w4a8_matmul(x, ascale, part))
        y = sharding.gather_columns(y_local)
        assert y.shape == (M, N)
        ret[rank] = bool(np.array_equal(y.numpy().view(np.uint32), full.view(np.uint32)))
    finally:
        dist.destroy_process_group()


def test_two_rank_column_sharding_matches_unsharded():
    world = 2
    port = _free_port()
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
        assert dict(ret) == {0: True, 1: True}


def test_shard_range_rejects_uneven_splits():
    from liquidgemm_b200 import sharding
    import pytest
    assert sharding.shard_range(10240, 3, 8) == (3840, 5120)
    with pytest.raises(ValueError):
        sharding.shard_range(1000, 0, 8)
