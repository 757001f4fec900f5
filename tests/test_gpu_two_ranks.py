"""Two ranks on two GPUs: the N-sharded decode linear whose epilogue stores its slice into both ranks'
full-width outputs (symmetric memory) against the unsharded CPU oracle.  Skipped on hosts with fewer
than two GPUs; no rank leaves early and nothing here can wait on a rank that is gone."""

import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, M, N, K, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
    try:
        import torch.distributed._symmetric_memory as symm_mem
        from liquidgemm_b200 import ops
        from liquidgemm_b200.sharding import shard_range
        from oracle import lqq_oracle as O
        from tests.helpers import random_lqq, random_tokens, to_torch_qw, bits, expected_bits
        qw = random_lqq(N, K, 64, seed=5)                      # the same full layer on every rank
        x, ascale = random_tokens(M, K, seed=6)
        lo, hi = shard_range(N, rank, world)
        shard = O.LQQWeight(qw.qweight_u4[lo:hi], qw.s_u8[lo:hi], qw.offset_a[lo:hi], qw.s1[lo:hi], 64)
        tq = to_torch_qw(shard, device=f"cuda:{rank}")
        blob = ops.repack_rs_weight(tq).reshape(-1)
        full = symm_mem.empty((M, N), dtype=torch.bfloat16, device=torch.device("cuda", rank))
        full.fill_(-1.0)
        hdl = symm_mem.rendezvous(full, dist.group.WORLD.group_name)
        hdl.barrier(channel=0)
        ops.gemm_fused_scatter(torch.from_numpy(x).cuda(), blob, torch.from_numpy(ascale).cuda(), tq.s1,
                               hdl.buffer_ptrs, N, lo, hi - lo, K, 0)
        hdl.barrier(channel=0)
        torch.cuda.synchronize()
        want = expected_bits(O.w4a8_matmul(x, ascale, qw), 0)
        q.put((rank, bool(np.array_equal(bits(full), want))))
        hdl.barrier(channel=0)
    except Exception as exc:  # report instead of leaving the other rank waiting for a message
        q.put((rank, repr(exc)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("M", [1, 8])
def test_sharded_decode_linear_gathers_by_stores(M):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, M, 1024, 2048, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(results) == [(0, True), (1, True)], results
