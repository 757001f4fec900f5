"""Every GPU of the host as one rank: the N-sharded linear whose epilogue stores its slice into every rank's
full-width output (symmetric memory, plain peer stores, no multicast objects) against the unsharded CPU
oracle -- through each kernel route of the dispatch (dp4a GEMV, one-launch tensor-core decode kernel, tile
kernel with split-K planes + finish pass, tile kernel with the fused epilogue, CTA-pair kernel), with a barrier between the
ranks and with the kernels' own flags.  Skipped on hosts with fewer than two GPUs; no rank leaves early and
nothing here can wait on a rank that is gone."""

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


def _worker(rank, world, port, cases, q):
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
        dev = torch.device("cuda", rank)
        flags = symm_mem.empty(64, dtype=torch.int32, device=dev)
        fh = symm_mem.rendezvous(flags, dist.group.WORLD.group_name)
        results = []
        for M, N, K in cases:
            # the last case runs on the CTA-pair kernel wherever the shard has whole 256-channel blocks (the
            # library reads the switch at every call)
            if (M, N, K) == cases[-1]:
                os.environ["LQ_PAIR_ALWAYS"] = "1"
            else:
                os.environ.pop("LQ_PAIR_ALWAYS", None)
            qw = random_lqq(N, K, 64, seed=5 + M)                  # the same full layer on every rank
            x, ascale = random_tokens(M, K, seed=6 + M)
            lo, hi = shard_range(N, rank, world)
            shard = O.LQQWeight(qw.qweight_u4[lo:hi], qw.s_u8[lo:hi], qw.offset_a[lo:hi], qw.s1[lo:hi], 64)
            tq = to_torch_qw(shard, device=f"cuda:{rank}")
            blob = ops.repack_rs_weight(tq).reshape(-1)
            full = symm_mem.empty((M, N), dtype=torch.bfloat16, device=dev)
            hdl = symm_mem.rendezvous(full, dist.group.WORLD.group_name)
            want = expected_bits(O.w4a8_matmul(x, ascale, qw), 0)
            xt, at = torch.from_numpy(x).cuda(), torch.from_numpy(ascale).cuda()
            # (1) ranks ordered by a barrier after the stores
            full.fill_(-1.0)
            hdl.barrier(channel=0)
            ops.gemm_fused_scatter(xt, blob, at, tq.s1, hdl.buffer_ptrs, N, lo, hi - lo, K, 0)
            hdl.barrier(channel=0)
            torch.cuda.synchronize()
            ok_barrier = bool(np.array_equal(bits(full), want))
            # (2) ranks ordered by the kernels' flags: every writing CTA of every rank signals word 0 of every
            # rank; a second launch (of the same linear) waits for that count before it reads its tokens
            full.fill_(-1.0)
            flags.zero_()
            torch.cuda.synchronize()
            fh.barrier(channel=1)
            ops.gemm_fused_scatter(xt, blob, at, tq.s1, hdl.buffer_ptrs, N, lo, hi - lo, K, 0,
                                   flag_ptrs=fh.buffer_ptrs, flag_index=0)
            grid = ops.decode_grid(M, hi - lo, K)
            ops.gemm_fused_scatter(xt, blob, at, tq.s1, hdl.buffer_ptrs, N, lo, hi - lo, K, 0,
                                   flag_ptrs=fh.buffer_ptrs, flag_index=1, wait_ptr=flags.data_ptr(),
                                   wait_value=world * grid)
            torch.cuda.synchronize()
            fh.barrier(channel=1)
            torch.cuda.synchronize()
            ok_flags = bool(np.array_equal(bits(full), want)) and int(flags[0]) == world * grid
            ops.poll_status()
            results.append((M, ok_barrier, ok_flags))
            hdl.barrier(channel=0)
        q.put((rank, results))
    except Exception as exc:  # report instead of leaving the other ranks waiting for a message
        import traceback
        q.put((rank, repr(exc) + traceback.format_exc()[-1500:]))
    finally:
        dist.destroy_process_group()


def test_sharded_linear_gathers_by_stores_on_every_gpu():
    world = min(torch.cuda.device_count(), 8)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    while 1024 % (world * 128):       # shards stay multiples of the 128-row tile
        world -= 1
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    # token counts that take the GEMV, the decode tensor-core kernel, tile + finish, the fused tile epilogue, and
    # the CTA-pair kernel's multi-destination epilogue
    cases = [(1, 1024, 2048), (8, 1024, 2048), (64, 1024, 2048), (300, 2048, 512), (600, 1024, 1024)]
    procs = [ctx.Process(target=_worker, args=(r, world, port, cases, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=600) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    want = [(M, True, True) for M, _, _ in cases]
    for rank, res in sorted(results, key=lambda r: r[0]):
        assert res == want, (rank, res)
