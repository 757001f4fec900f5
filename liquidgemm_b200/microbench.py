"""Pipeline microbenchmarks for the sm_100a building blocks of the W4A8 kernels.

    python -m liquidgemm_b200.build --debug           # once: the measurement kernels, a library of their own
    python -m liquidgemm_b200.microbench mma_rate     # tcgen05.mma kind::i8 issue-to-issue cost
    python -m liquidgemm_b200.microbench mma_rate2    # the same for cta_group::2 (CTA pairs)
    python -m liquidgemm_b200.microbench sync_cost    # mbarrier / commit / bulk-copy instruction costs
    python -m liquidgemm_b200.microbench handover     # end of one kernel -> griddepcontrol.wait returns in the next
    python -m liquidgemm_b200.microbench tma_stream   # HBM streaming rate of ring-buffered bulk copies
    python -m liquidgemm_b200.microbench l2_stream    # the same stream when the data is L2-resident
    python -m liquidgemm_b200.microbench tma_stream2  # two producer threads with a ring each in one CTA
    python -m liquidgemm_b200.microbench tma_rows     # the same with one bulk copy per weight row

    python -m liquidgemm_b200.build --trace           # once: the product sources with -DLQ_PIPELINE_TRACE
    python -m liquidgemm_b200.microbench decode_trace gate_up 8   # per-CTA cycle counters of the decode kernel
    python -m liquidgemm_b200.microbench pair_trace gate_up 8192  # the same for the CTA-pair prefill kernel
    python -m liquidgemm_b200.microbench tile_trace gate_up 8     # time stamps of every CTA of the tile kernel

All but the last launch measurement-only kernels (``lq_debug_*`` in ``csrc/dbg/lq_debug.cu``); none of them is
in the product library.  ``decode_trace`` and ``pair_trace`` run the real decode tensor-core kernel and the CTA-pair prefill kernel
from the trace build and print where each role's cycles go.  They need a B200; every device-side wait in them is bounded.
"""

from __future__ import annotations

import ctypes
import os
import sys

import numpy as np
import torch

_HERE = os.path.dirname(os.path.abspath(__file__))


class _Lazy:
    """The debug library, loaded on first use (it is not built by default)."""

    _lib = None

    def __getattr__(self, name):
        if _Lazy._lib is None:
            path = os.path.join(_HERE, "_lq_b200_dbg.so")
            if not os.path.exists(path):
                raise ImportError(f"{path} is missing: build it with `python -m liquidgemm_b200.build --debug`")
            _Lazy._lib = ctypes.CDLL(path)
        return getattr(_Lazy._lib, name)


lib = _Lazy()

_I, _P, _L = ctypes.c_int, ctypes.c_void_p, ctypes.c_long


def _stream():
    return torch.cuda.current_stream().cuda_stream


def mma_rate(iters: int = 2000) -> None:
    """Cycles between back-to-back 128 x N x 32 int8 MMAs, A in tensor memory (TS) or shared (SS)."""
    fn = lib.lq_debug_mma_rate
    fn.argtypes, fn.restype = [_I] * 4 + [_P, _P], _I
    for ctas in (1, 148):
        for ts in (1, 0):
            for n in (16, 64, 128, 192, 256):
                out = torch.zeros(ctas * 2, dtype=torch.int64, device="cuda")
                for _ in range(2):
                    assert fn(n, iters, ts, ctas, out.data_ptr(), _stream()) == 0
                torch.cuda.synchronize()
                o = out.cpu().numpy().reshape(ctas, 2)
                cyc = float(np.median(o[:, 0])) / (iters * 4)
                issue = float(np.median(o[:, 1])) / (iters * 4)
                print(f"ctas={ctas:3d} {'TS' if ts else 'SS'} N={n:3d}: {cyc:7.1f} cycles/MMA (issue {issue:6.1f})"
                      f"  -> {128 * n * 32 / cyc:7.0f} MAC/clk/SM", flush=True)
    # the issue loop walked by the whole warp with one elected lane issuing, against `if (thread 0) loop`; both
    # with an operand address that changes from group to group, as in a real main loop
    for mode, what in [(1, "thread 0 alone"), (9, "warp-uniform loop, elected lane")]:
        for n in (16, 64, 128, 192, 256):
            out = torch.zeros(148 * 2, dtype=torch.int64, device="cuda")
            for _ in range(2):
                assert fn(n, iters, mode, 148, out.data_ptr(), _stream()) == 0
            torch.cuda.synchronize()
            cyc = float(np.median(out.cpu().numpy().reshape(148, 2)[:, 0])) / (iters * 4)
            print(f"ctas=148 TS N={n:3d} {what}: {cyc:7.1f} cycles/MMA", flush=True)
    # two accumulators taken in turn: is the floor a dependent-accumulate latency?
    for n in (16, 64, 128):
        out = torch.zeros(148 * 2, dtype=torch.int64, device="cuda")
        for _ in range(2):
            assert fn(n, iters, 5, 148, out.data_ptr(), _stream()) == 0
        torch.cuda.synchronize()
        cyc = float(np.median(out.cpu().numpy().reshape(148, 2)[:, 0])) / (iters * 4)
        print(f"ctas=148 TS N={n:3d} two accumulators in turn: {cyc:7.1f} cycles/MMA", flush=True)
    # two CTAs per SM (256 tensor-memory columns each): do their MMA streams overlap?
    for n in (16, 128):
        out = torch.zeros(296 * 2, dtype=torch.int64, device="cuda")
        for _ in range(2):
            assert fn(n, iters, 3, 296, out.data_ptr(), _stream()) == 0
        torch.cuda.synchronize()
        cyc = float(np.median(out.cpu().numpy().reshape(296, 2)[:, 0])) / (iters * 4)
        print(f"ctas=296 (2 per SM) TS N={n:3d}: {cyc:7.1f} cycles/MMA per CTA", flush=True)


def mma_rate2(iters: int = 2000) -> None:
    """The same for tcgen05.mma.cta_group::2: one 256 x N x 32 MMA per CTA pair (128 x N per SM); then what the
    issuing thread's other per-k-step work adds: one or two multicast commits per group of four MMAs, a wait
    on a completed barrier with its fence."""
    fn = lib.lq_debug_mma_rate2
    fn.argtypes, fn.restype = [_I] * 5 + [_P, _P], _I

    def run(n, ts, extra, ctas):
        out = torch.zeros(ctas * 2, dtype=torch.int64, device="cuda")
        for _ in range(2):
            assert fn(n, iters, ts, extra, ctas, out.data_ptr(), _stream()) == 0
        torch.cuda.synchronize()
        o = out.cpu().numpy().reshape(ctas, 2)
        return float(np.median(o[:, 0])) / (iters * 4), int(o[:, 1].sum())

    for ctas in (2, 148):
        for ts in (1, 0):
            for n in (64, 128, 192, 256):
                cyc, bad = run(n, ts, 0, ctas)
                print(f"ctas={ctas:3d} pair {'TS' if ts else 'SS'} N={n:3d}: {cyc:7.1f} cycles/MMA  -> "
                      f"{128 * n * 32 / cyc:7.0f} MAC/clk/SM  (waits that ran out: {bad})", flush=True)
    for n in (128, 192, 256):
        for extra, what in [(0, "four MMAs"), (1, "+ one commit"), (2, "+ two commits"), (4, "+ wait and fence"),
                            (5, "+ one commit, wait and fence"), (6, "+ two commits, wait and fence")]:
            cyc, bad = run(n, 1, extra, 148)
            print(f"pair TS N={n:3d} per group: {what:32s} {4 * cyc:7.1f} cycles  (waits that ran out: {bad})", flush=True)


def tma_stream2(total_bytes: int = 2_000_000_000) -> None:
    """Two producer threads per CTA, each with its own ring, reading L2-resident data: is the fixed cost of a
    bulk copy paid per issuing thread or per CTA?"""
    fn = lib.lq_debug_tma_stream2
    fn.argtypes, fn.restype = [_P, _I, _I, _I, _I, _I, _P, _P], _I
    src = torch.zeros(1 << 28, dtype=torch.uint8, device="cuda")
    cyc = torch.zeros(296, dtype=torch.int64, device="cuda")
    for stage, ns in [(8704, 8), (16384, 5), (24576, 4), (32768, 3)]:
        wrap = max(1, (32 << 20) // (296 * stage))
        steps = total_bytes // (296 * stage)
        for _ in range(2):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            assert fn(src.data_ptr(), stage, ns, steps, wrap, 148, cyc.data_ptr(), None) == 0
            e1.record()
            torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3
        clk = float(np.median(cyc.cpu().numpy())) / steps
        print(f"148 CTAs x 2 rings, stage {stage:6d} B x {ns:2d} buffers: {us:8.1f} us  "
              f"{296 * steps * stage / us / 1e6:6.2f} TB/s  {clk:6.1f} cycles per copy per ring  "
              f"{2 * stage / clk:5.1f} B/clk/SM", flush=True)


def handover() -> None:
    """Time from the end of a kernel's last CTA to the return of griddepcontrol.wait in the next kernel of the
    stream (both launched with programmatic stream serialisation), with and without tensor memory in the first
    kernel, for several output sizes and shared-memory footprints."""
    fn = lib.lq_debug_handover
    fn.argtypes, fn.restype = [_I, _I, _I, _I, _P, _P, _P], _I
    out = torch.zeros(148 * (1 << 20), dtype=torch.uint8, device="cuda")
    stamps = torch.zeros(4, dtype=torch.int64, device="cuda")
    big = torch.iinfo(torch.int64).max
    for smem_kb in (95, 150):
        for use_tmem in (0, 1):
            for out_kb in (0, 4, 64, 1024):
                ctas = 296 if smem_kb < 110 else 148
                gaps = []
                for rep in range(12):
                    stamps.copy_(torch.tensor([0, big, 0, 0], dtype=torch.int64))
                    torch.cuda.synchronize()
                    assert fn(use_tmem, out_kb * 1024 // 2 if ctas == 296 else out_kb * 1024, smem_kb * 1024, ctas,
                              out.data_ptr(), stamps.data_ptr(), _stream()) == 0
                    torch.cuda.synchronize()
                    s = stamps.cpu().numpy()
                    if rep >= 2:
                        gaps.append(int(s[1]) - int(s[0]))
                print(f"{ctas} CTAs, {smem_kb:3d} KB shared memory per CTA, tensor memory {'yes' if use_tmem else 'no '}, "
                      f"{out_kb:5d} KB written per SM: last CTA's end -> wait returns: median {int(np.median(gaps)):6d} ns  "
                      f"(min {min(gaps)}, max {max(gaps)})", flush=True)


def sync_cost() -> None:
    """Cycle cost of the synchronisation instructions the GEMM pipeline is built from."""
    fn = lib.lq_debug_sync_cost
    fn.argtypes, fn.restype = [_P] * 3, _I
    src = torch.zeros(1 << 20, dtype=torch.uint8, device="cuda")
    out = torch.zeros(16, dtype=torch.int64, device="cuda")
    names = ["loop64", "clock64", "trywait_fresh", "arrive", "trywait_done", "bulk8k_roundtrip", "commit",
             "bulk_issue", "ok"]
    for _ in range(3):
        assert fn(src.data_ptr(), out.data_ptr(), None) == 0
        torch.cuda.synchronize()
        print(dict(zip(names, out.cpu().tolist())), flush=True)


def tma_stream(total_bytes: int = 400_000_000) -> None:
    """One producer thread per CTA streams contiguous stages through a ring of `ns` buffers."""
    fn = lib.lq_debug_tma_stream
    fn.argtypes, fn.restype = [_P, _I, _I, _I, _I, _P, _P], _I
    src = torch.zeros(1 << 30, dtype=torch.uint8, device="cuda")
    cyc = torch.zeros(148, dtype=torch.int64, device="cuda")
    for stage, ns in [(8704, 16), (8704, 8), (8704, 4), (17408, 8), (32768, 5), (4352, 32), (8704, 20)]:
        steps = total_bytes // (148 * stage)
        for _ in range(2):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            assert fn(src.data_ptr(), stage, ns, steps, 148, cyc.data_ptr(), None) == 0
            e1.record()
            torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3
        nbytes = 148 * steps * stage
        print(f"stage {stage:6d} B x {ns:2d} buffers: {us:8.1f} us  {nbytes / us / 1e6:6.2f} TB/s  "
              f"cycles/stage {float(np.median(cyc.cpu().numpy())) / steps:7.1f}", flush=True)


def l2_stream(total_bytes: int = 2_000_000_000) -> None:
    """The bulk-copy stream out of L2: every group of `share` CTAs re-reads a region small enough that all
    regions together stay L2-resident (what the token tiles of a prefill GEMM look like to the memory system).
    296 CTAs are two per SM: whether the cost of a copy is paid per issuing CTA or per SM."""
    fn = lib.lq_debug_tma_stream_l2
    fn.argtypes, fn.restype = [_P, _I, _I, _I, _I, _I, _I, _P, _P], _I
    src = torch.zeros(1 << 28, dtype=torch.uint8, device="cuda")
    cyc = torch.zeros(296, dtype=torch.int64, device="cuda")
    for stage, ns, footprint_mb, share, ctas in [
            (32768, 5, 32, 1, 148), (32768, 5, 32, 8, 148), (16384, 10, 32, 1, 148), (24576, 6, 32, 4, 148),
            (8704, 16, 32, 1, 148), (8704, 8, 32, 1, 296), (16384, 5, 32, 1, 296), (32768, 3, 32, 1, 296),
            (49152, 4, 32, 1, 148), (65536, 3, 32, 1, 148), (65536, 3, 32, 8, 148), (4352, 16, 32, 1, 148)]:
        groups = -(-ctas // share)
        wrap = max(1, (footprint_mb << 20) // (groups * stage))
        steps = total_bytes // (ctas * stage)
        for _ in range(2):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            assert fn(src.data_ptr(), stage, ns, steps, wrap, share, ctas, cyc.data_ptr(), None) == 0
            e1.record()
            torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3
        nbytes = ctas * steps * stage
        clk = float(np.median(cyc[:ctas].cpu().numpy())) / steps
        print(f"{ctas} CTAs, stage {stage:6d} B x {ns:2d} buffers, {footprint_mb:3d} MB footprint, {share} CTAs per region: "
              f"{us:8.1f} us  {nbytes / us / 1e6:6.2f} TB/s  {clk:6.1f} cycles per copy per CTA  "
              f"{stage / clk * (ctas / 148):5.1f} B/clk/SM", flush=True)


def tma_rows(total_bytes: int = 400_000_000) -> None:
    """A stage made of `rows` separate bulk copies of `row_bytes` each (a row-major weight slice)
    instead of one contiguous copy; `pieces` splits every row into that many copies."""
    fn = lib.lq_debug_tma_rows
    fn.argtypes, fn.restype = [_P, _I, _I, _L, _I, _I, _I, _I, _P, _P], _I
    src = torch.zeros(1 << 30, dtype=torch.uint8, device="cuda")
    cyc = torch.zeros(148, dtype=torch.int64, device="cuda")
    for rows, row_bytes, stride, ns, pieces in [(8, 2048, 2048, 9, 1), (8, 1024, 2048, 18, 2), (16, 1024, 2048, 9, 2),
                                                (8, 2048, 7168, 9, 3), (32, 512, 2048, 9, 4), (4, 4096, 4096, 9, 1),
                                                (16, 512, 2048, 18, 4)]:
        stage = rows * row_bytes
        steps = total_bytes // (148 * stage)
        for _ in range(2):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            rc = fn(src.data_ptr(), rows, row_bytes, stride, ns, steps, pieces, 148, cyc.data_ptr(), None)
            e1.record()
            torch.cuda.synchronize()
            assert rc == 0, rc
        us = e0.elapsed_time(e1) * 1e3
        print(f"{rows:2d} rows x {row_bytes:4d} B (stride {stride}, {pieces} copies/row) x {ns:2d} buffers: "
              f"{us:8.1f} us  {148 * steps * stage / us / 1e6:6.2f} TB/s  "
              f"cycles/stage {float(np.median(cyc.cpu().numpy())) / steps:7.1f}", flush=True)


def decode_trace(shape: str = "gate_up", M: int = 8) -> None:
    """Per-CTA cycle counters of ``w4a8_decode_tc_kernel`` on one Llama-3.1-8B shape (trace build of the
    library): median / 10th / 90th percentile over the CTAs of the last launch of a graph of back-to-back
    launches over rotating weight copies.  Counters are sums over the k-tiles a role handled."""
    if os.environ.get("LIQUIDGEMM_B200_TRACE") != "1":
        import subprocess
        env = dict(os.environ, LIQUIDGEMM_B200_TRACE="1")
        sys.exit(subprocess.call([sys.executable, "-m", "liquidgemm_b200.microbench", "decode_trace", shape, str(M)],
                                 env=env))
    from . import benchlib as B
    from ._lib import lib as plib
    N, K = B.SHAPES[shape]
    C = 6
    layers = [B.device_lqq(N, K, seed=31 * c + 1, want_gp=False) for c in range(C)]
    x, sc = B.device_tokens(M, K, seed=M)
    t = B.graph_time_us(lambda i: B.linear_call(layers[i % C], x, sc, M), C, 3)
    buf = (ctypes.c_longlong * (1024 * 16))()
    plib.lq_debug_read_decode_trace.argtypes = [ctypes.c_void_p]
    assert plib.lq_debug_read_decode_trace(buf) == 0
    a = np.frombuffer(buf, dtype=np.int64).reshape(1024, 16)[:plib.lq_decode_grid(M, N, K)]
    names = {0: "producer: waiting for a free weight stage", 1: "producer: whole loop",
             3: "MMA thread: waiting for operands", 4: "MMA thread: whole loop", 10: "MMA thread: issuing 4 MMAs",
             11: "MMA thread: commit", 5: "dequant thread: waiting for the weight tile",
             12: "dequant thread: shared loads + unpack", 7: "dequant thread: tcgen05.st + token store + wait::st",
             2: "dequant thread: proxy fence + arrive", 6: "dequant thread: waiting for the operand stage",
             9: "dequant thread: epilogues", 8: "dequant thread: whole role (incl. wait for the previous kernel)"}
    print(f"{shape} {N}x{K}, M = {M}: {t:.2f} us per launch (trace build), {len(a)} CTAs; cycles per CTA")
    for slot, label in names.items():
        col = a[:, slot]
        print(f"  {label:62s} median {int(np.median(col)):7d}   p10 {int(np.percentile(col, 10)):7d}   "
              f"p90 {int(np.percentile(col, 90)):7d}")
    t0 = a[:, 13].min()
    for label, col in (("CTA start", a[:, 13]), ("CTA end", a[:, 14])):
        c = col - t0
        print(f"  {label:10s} ns after the first CTA's start: min {int(c.min())}  median {int(np.median(c))}  "
              f"max {int(c.max())}")


def tile_trace(shape: str = "gate_up", M: int = 8) -> None:
    """%globaltimer stamps of every CTA of ``w4a8_tile_kernel`` (trace build) for the last launch of a graph of
    back-to-back launches over rotating weight copies: nanoseconds after the launch's first CTA started."""
    if os.environ.get("LIQUIDGEMM_B200_TRACE") != "1":
        import subprocess
        env = dict(os.environ, LIQUIDGEMM_B200_TRACE="1")
        sys.exit(subprocess.call([sys.executable, "-m", "liquidgemm_b200.microbench", "tile_trace", shape, str(M)],
                                 env=env))
    from . import benchlib as B
    from ._lib import lib as plib
    N, K = B.SHAPES[shape]
    C = 6
    layers = [B.device_lqq(N, K, seed=31 * c + 1, want_gp=False) for c in range(C)]
    x, sc = B.device_tokens(M, K, seed=M)
    t = B.graph_time_us(lambda i: B.linear_call(layers[i % C], x, sc, M), C, 3)
    buf = (ctypes.c_longlong * (1024 * 8))()
    plib.lq_debug_read_tile_trace.argtypes = [ctypes.c_void_p]
    assert plib.lq_debug_read_tile_trace(buf) == 0
    a = np.frombuffer(buf, dtype=np.int64).reshape(1024, 8)
    a = a[a[:, 0] > 0]
    t0 = a[:, 0].min()
    names = {0: "CTA start", 1: "first weight copies issued", 2: "previous kernel complete (griddepcontrol.wait returned)",
             3: "first stage landed (weights + tokens)", 4: "last stage landed", 5: "accumulator final",
             6: "all roles done"}
    print(f"{shape} {N}x{K}, M = {M}: {t:.2f} us per launch (trace build), {len(a)} CTAs; ns after the first CTA's start")
    for slot, label in names.items():
        col = a[:, slot] - t0
        print(f"  {label:58s} min {int(col.min()):6d}   median {int(np.median(col)):6d}   p90 {int(np.percentile(col, 90)):6d}"
              f"   max {int(col.max()):6d}")
    for (i, j), label in {(0, 2): "start -> previous kernel complete", (2, 3): "-> first stage landed",
                          (3, 4): "-> last stage landed (the stream)", (4, 5): "-> accumulator final",
                          (5, 6): "-> done (epilogue)"}.items():
        d = a[:, j] - a[:, i]
        print(f"  per CTA {label:40s} median {int(np.median(d)):6d}   p10 {int(np.percentile(d, 10)):6d}   p90 "
              f"{int(np.percentile(d, 90)):6d}")


def pair_trace(shape: str = "gate_up", M: int = 8192) -> None:
    """Per-CTA cycle counters of ``w4a8_pair_kernel`` (trace build of the library) on one Llama-3.1-8B shape:
    median / min / max over the CTAs of either rank of the last launch.  Counters are sums over the k-steps
    (or tiles) a role handled; divide by the k-steps the MMA warp reports."""
    if os.environ.get("LIQUIDGEMM_B200_TRACE") != "1":
        import subprocess
        env = dict(os.environ, LIQUIDGEMM_B200_TRACE="1", LQ_PAIR_ALWAYS="1")
        sys.exit(subprocess.call([sys.executable, "-m", "liquidgemm_b200.microbench", "pair_trace", shape, str(M)],
                                 env=env))
    from . import benchlib as B
    from ._lib import lib as plib
    N, K = B.SHAPES[shape]
    layer = B.device_lqq(N, K, seed=1, want_gp=False)
    x, sc = B.device_tokens(M, K, seed=M)
    for _ in range(3):
        B.linear_call(layer, x, sc, M)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    B.linear_call(layer, x, sc, M)
    e1.record()
    torch.cuda.synchronize()
    buf = (ctypes.c_longlong * (256 * 32))()
    plib.lq_debug_read_pair_trace.argtypes = [ctypes.c_void_p]
    assert plib.lq_debug_read_pair_trace(buf) == 0
    a = np.frombuffer(buf, dtype=np.int64).reshape(256, 32)[:plib.lq_decode_grid(M, N, K)]
    names = {0: "weight producer: waiting for a free stage", 1: "weight producer: whole loop",
             2: "token producer: waiting for a free stage", 3: "token producer: whole loop",
             4: "MMA warp: waiting for a free accumulator", 5: "MMA warp: waiting for operands",
             6: "MMA warp: issuing 4 MMAs", 7: "MMA warp: commits", 8: "MMA warp: whole loop", 9: "MMA warp: k-steps",
             10: "dequant thread: waiting for the stage", 11: "dequant thread: shared loads + unpack",
             12: "dequant thread: waiting for the operand stage", 13: "dequant thread: tcgen05.st + wait::st + arrive",
             14: "dequant thread: whole role", 16: "epilogue thread: waiting for an accumulator",
             19: "epilogue thread: token scales + barrier", 21: "epilogue thread: tcgen05.ld, convert, store",
             17: "epilogue thread: whole role", 18: "epilogue thread: tiles",
             22: "epilogue thread, first k-range of a cut tile: sums to the plane", 23: "... fence, barrier, counter"}
    print(f"{shape} {N}x{K}, M = {M}: {e0.elapsed_time(e1) * 1e3:.1f} us (trace build), {len(a)} CTAs; cycles per CTA")
    for rank in (0, 1):
        rows = a[rank::2]
        print(f"rank {rank} of the pair")
        for slot, label in names.items():
            col = rows[:, slot]
            if col.any():
                print(f"  {label:48s} median {int(np.median(col)):9d}   min {int(col.min()):9d}   max {int(col.max()):9d}")


_CASES = {"mma_rate": mma_rate, "mma_rate2": mma_rate2, "sync_cost": sync_cost, "handover": handover, "tma_stream": tma_stream,
          "l2_stream": l2_stream, "tma_stream2": tma_stream2, "tma_rows": tma_rows}

if __name__ == "__main__":
    torch.cuda.set_device(0)
    if len(sys.argv) > 1 and sys.argv[1] in ("decode_trace", "pair_trace", "tile_trace"):
        fn = {"decode_trace": decode_trace, "pair_trace": pair_trace, "tile_trace": tile_trace}[sys.argv[1]]
        fn(*(sys.argv[2:3] or ["gate_up"]), *(int(v) for v in sys.argv[3:4]))
        sys.exit(0)
    which = sys.argv[1:] or list(_CASES)
    for name in which:
        print(f"== {name}", flush=True)
        _CASES[name]()
