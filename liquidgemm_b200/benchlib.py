"""Secondary measurements printed under ``extras`` by ``bench.py``.

Everything here is timed on the device with CUDA events around CUDA-graph replays, walks rotating
weight copies larger than L2, and uses seeded synthetic LQQ data generated on the device (timing
does not depend on the values; parity is the test-suite's job).

* ``sweep``   : per (shape, M) time of the W4A8 op, weight GB/s, TOPS, roofline fraction, and cuBLAS
                bf16 (``x @ w.T``) on the same GPU -- the comparison the reference publishes
                (bench/rs_bench.py:44, bench/RESULTS.md:218-224).
* ``splitk``  : decode-tile GEMM M in {32, 64, 128} on down / gate_up for split-K 1, 2, 4, 8.
* ``tp70b``   : Llama-3-70B-shape linears column-sharded along N over the ranks, 80 layers x 4
                linears: without exchange, with an NCCL all-gather of every output (on the compute stream and
                overlapped on a second stream), and with the gather done by the linears' own store epilogues.
"""

from __future__ import annotations

import os

import torch

from . import ops

SHAPES = {"qkv": (6144, 4096), "o": (4096, 4096), "gate_up": (28672, 4096), "down": (4096, 14336)}
SHAPES_70B = {"qkv": (10240, 8192), "o": (8192, 8192), "gate_up": (57344, 8192), "down": (8192, 28672)}
INT8_DENSE_TOPS = 4500.0   # B200 datasheet, dense


def device_lqq(N, K, seed, want_gp=True, want_rs=True):
    """Random valid LQQ layer generated on the device: codes, steps 1..16, offsets with u <= 255."""
    from .quant import LiquidQuantWeight
    g = torch.Generator(device="cuda").manual_seed(seed)
    codes = torch.randint(0, 16, (N, K), dtype=torch.uint8, device="cuda", generator=g)
    step = torch.randint(1, 17, (N, K // 64), dtype=torch.int32, device="cuda", generator=g)
    off = (torch.rand((N, K // 64), device="cuda", generator=g) * (256 - 15 * step).float()).to(torch.int32)
    off = torch.minimum(off, 255 - 15 * step)
    s1 = torch.rand(N, device="cuda", generator=g) * 0.01 + 1e-4
    qw = LiquidQuantWeight(codes, step.to(torch.uint8), off.to(torch.uint8), s1, 64)
    out = {"s_u8": qw.s_u8, "offset_a": qw.offset_a, "s1": qw.s1, "N": N, "K": K}
    if want_gp:
        out["gp"] = ops.pack_gemv_interleaved(qw)
    if want_rs:
        out["rs"] = ops.repack_rs_weight(qw).reshape(-1)
    return out


def device_tokens(M, K, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randint(-127, 128, (M, K), dtype=torch.int8, device="cuda", generator=g)
    sc = torch.rand(M, device="cuda", generator=g) * 0.02 + 0.01
    return x, sc


def graph_time_us(fn, n_items, reps=5):
    """fn(i) enqueues one launch on weight copy i; returns microseconds per launch under graph replay."""
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        for i in range(min(n_items, 3)):
            fn(i)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            for i in range(n_items):
                fn(i)
        g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(s)
        for _ in range(reps):
            g.replay()
        e1.record(s)
        torch.cuda.synchronize()
    return e0.elapsed_time(e1) / (reps * n_items) * 1e3


def linear_call(L, x, sc, M, splitk=None, out_dtype=0):
    if ops.use_gemv(M, L["N"], L["K"], "gp" in L, "rs" in L):
        return torch.ops.liquidgemm.w4a8_gemv2(x, L["gp"], L["s_u8"], L["offset_a"], sc, L["s1"], L["N"], L["K"], 64,
                                               out_dtype)
    return ops.gemm_fused(x, L["rs"], sc, L["s1"], L["N"], L["K"], out_dtype, splitk=splitk)


def algorithmic_bytes(M, N, K):
    return N * K // 2 + 2 * N * K // 64 + 4 * N + M * K + 4 * M + M * N * 2


def run_sweep(peaks, Ms=(1, 4, 8, 16, 32, 64, 128, 512, 2048, 8192)):
    rows = []
    for name, (N, K) in SHAPES.items():
        C = max(3, -(-400_000_000 // (N * K // 2)))
        layers = [device_lqq(N, K, seed=31 * c + len(name), want_gp=False) for c in range(C)]
        Cb = max(3, -(-300_000_000 // (N * K * 2)))
        wbf = [torch.randn(N, K, device="cuda", dtype=torch.bfloat16) for _ in range(Cb)]
        for M in Ms:
            x, sc = device_tokens(M, K, seed=M)
            xb = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
            reps = 5 if M < 2048 else 2
            t = graph_time_us(lambda i: linear_call(layers[i % C], x, sc, M), C, reps)
            tb = graph_time_us(lambda i: torch.matmul(xb, wbf[i % Cb].t()), Cb, reps)
            tops = 2.0 * M * N * K / t / 1e6
            gbs = algorithmic_bytes(M, N, K) / t / 1e3
            rows.append({"shape": name, "M": M, "us": round(t, 2), "weight_GBps": round(N * K / 2 / t / 1e3, 1),
                         "alg_GBps": round(gbs, 1), "hbm_frac": round(gbs / peaks["hbm_gbs"], 3),
                         "TOPS": round(tops, 1), "int8_frac_of_4500": round(tops / INT8_DENSE_TOPS, 3),
                         "cublas_bf16_us": round(tb, 2), "speedup_vs_cublas_bf16": round(tb / t, 2),
                         "int8_frac_of_2x_bf16": round(tops / (2.0 * peaks.get("bf16_tflops", 1685.0)), 3)})
        del layers, wbf
        torch.cuda.empty_cache()
    return rows


def run_quant(peaks, K=4096):
    """The per-token activation quantiser alone (fp16 in): time and fraction of the HBM copy rate
    for its algorithmic bytes (read 2 B, write 1 B per element + one scale per token)."""
    rows = []
    for M in (1, 16, 128, 2048, 8192):
        C = max(3, -(-300_000_000 // (M * K * 3)))
        C = min(C, 64)
        xs = [torch.randn(M, K, device="cuda", dtype=torch.float16) for _ in range(C)]
        t = graph_time_us(lambda i: torch.ops.liquidgemm.quant_per_token(xs[i % C]), C)
        nbytes = M * K * 3 + 4 * M
        rows.append({"M": M, "K": K, "us": round(t, 2), "GBps": round(nbytes / t / 1e3, 1),
                     "hbm_frac": round(nbytes / t / 1e3 / peaks["hbm_gbs"], 3)})
        del xs
    torch.cuda.empty_cache()
    return rows


def run_splitk(peaks):
    rows = []
    for name in ("down", "gate_up"):
        N, K = SHAPES[name]
        C = max(3, -(-400_000_000 // (N * K // 2)))
        layers = [device_lqq(N, K, seed=77 * c + 1, want_gp=False) for c in range(C)]
        for M in (32, 64, 128):
            x, sc = device_tokens(M, K, seed=M)
            for S in (0, 1, 2, 4, 8):
                t = graph_time_us(lambda i: linear_call(layers[i % C], x, sc, M, splitk=S), C)
                gbs = algorithmic_bytes(M, N, K) / t / 1e3
                rows.append({"shape": name, "M": M, "splitk": S, "us": round(t, 2), "alg_GBps": round(gbs, 1),
                             "hbm_frac": round(gbs / peaks["hbm_gbs"], 3)})
        del layers
        torch.cuda.empty_cache()
    return rows


def _symmetric_outputs(world, M, names):
    """Full-width [M, N] bf16 outputs allocated as symmetric memory: every rank can store into every
    rank's buffer.  Returns {name: (tensor, handle)} or None where symmetric memory is unavailable."""
    import torch.distributed as dist
    try:
        import torch.distributed._symmetric_memory as symm_mem
        out = {}
        for n in names:
            t = symm_mem.empty((M, SHAPES_70B[n][0]), dtype=torch.bfloat16, device=torch.device("cuda", torch.cuda.current_device()))
            out[n] = (t, symm_mem.rendezvous(t, dist.group.WORLD.group_name))
        return out
    except Exception:
        return None


def _symmetric_flags(words):
    """A uint32 flag array in symmetric memory (every rank's kernels can add to every rank's words).  Returns
    (tensor, handle) or None."""
    import torch.distributed as dist
    try:
        import torch.distributed._symmetric_memory as symm_mem
        t = symm_mem.empty(max(words, 64), dtype=torch.int32, device=torch.device("cuda", torch.cuda.current_device()))
        t.zero_()
        return t, symm_mem.rendezvous(t, dist.group.WORLD.group_name)
    except Exception:
        return None


def run_tp70b(world, rank, Ms=(1, 64, 2048), layers_in_stack=80, distinct_layers=3):
    """80-layer stack of the four 70B-shape linears, each column-sharded along N over `world` ranks, timed
    (CUDA events around graph replays, max over ranks) in up to four ways:

    * ``no_gather``     sharded linears only;
    * ``nccl``          an NCCL all-gather of every output on the compute stream (the stated baseline);
    * ``nccl_overlap``  the same collective on a second stream, so that the gather of linear i runs under the
                        GEMM of linear i + 1 (each output has its own buffer; joined at the end of the stack);
    * ``stores``        gather by stores: the linear's own epilogue writes its slice into every rank's
                        full-width output over NVLink (plain peer stores into symmetric memory), and the
                        ranks are ordered ONCE PER LAYER by a symmetric-memory barrier on the stream, i.e.
                        the four outputs of a layer are complete on every rank when the next layer starts;
    * ``stores_flags``  the same stores ordered by the kernels' own flags instead of a barrier per layer: every
                        writing CTA of layer l adds 1 to word l of every rank's flag array after its last store,
                        and the first linear of layer l + 1 waits (bounded) until its own word l has reached the
                        number of writing CTAs of all ranks before it reads its tokens.  Outputs alternate
                        between two sets of buffers by layer parity (a rank starts the stores of layer l + 2 only
                        after every rank has finished the kernels of layer l + 1, which are the readers of layer
                        l's buffers); the flags are cleared, between two barriers, once per stack.

    On one rank the unsharded stack is ``single_gpu_ms``; with more ranks every rank also times that
    unsharded stack on its own GPU, so that the strong-scaling efficiency t1 / (N * tN) of each mode comes
    from one run."""
    import torch.distributed as dist
    rows = []
    names = list(SHAPES_70B)
    stack = []
    for l in range(distinct_layers):
        stack.append({n: device_lqq(SHAPES_70B[n][0] // world, SHAPES_70B[n][1], seed=1000 * rank + 10 * l + i,
                                    want_gp=False)
                      for i, n in enumerate(names)})
    full_stack = stack
    if world > 1:
        full_stack = [{n: device_lqq(SHAPES_70B[n][0], SHAPES_70B[n][1], seed=10 * l + i, want_gp=False)
                       for i, n in enumerate(names)} for l in range(distinct_layers)]
    for M in Ms:
        toks = {n: device_tokens(M, SHAPES_70B[n][1], seed=M + i) for i, n in enumerate(names)}
        gathered = {n: torch.empty((world * M, SHAPES_70B[n][0] // world), dtype=torch.bfloat16, device="cuda")
                    for n in names} if world > 1 else None
        symm = _symmetric_outputs(world, M, names) if world > 1 else None
        symm2 = _symmetric_outputs(world, M, names) if symm is not None else None
        flags = _symmetric_flags(layers_in_stack) if symm2 is not None else None
        layer_ctas = world * sum(ops.decode_grid(M, SHAPES_70B[n][0] // world, SHAPES_70B[n][1]) for n in names) \
            if flags is not None else 0
        comm = torch.cuda.Stream() if world > 1 else None

        def one_stack(mode):
            lays = full_stack if mode == "single" else stack
            done = []
            if mode == "stores_flags":
                symm[names[0]][1].barrier(channel=1)    # every rank is done with the previous stack's flags
                flags[0].zero_()
                symm[names[0]][1].barrier(channel=1)    # every rank's flags are clear before anyone signals
            for l in range(layers_in_stack):
                lay = lays[l % distinct_layers]
                for i, n in enumerate(names):
                    L = lay[n]
                    if mode == "stores_flags":
                        full, hdl = (symm if (layers_in_stack - 1 - l) % 2 == 0 else symm2)[n]   # the last layer writes `symm`
                        first = i == 0 and l > 0
                        ops.gemm_fused_scatter(toks[n][0], L["rs"], toks[n][1], L["s1"], hdl.buffer_ptrs, full.shape[1],
                                               rank * L["N"], L["N"], L["K"], 0, flag_ptrs=flags[1].buffer_ptrs,
                                               flag_index=l,
                                               wait_ptr=(flags[0].data_ptr() + 4 * (l - 1)) if first else None,
                                               wait_value=layer_ctas if first else 0)
                    elif mode == "stores":
                        full, hdl = symm[n]
                        ops.gemm_fused_scatter(toks[n][0], L["rs"], toks[n][1], L["s1"], hdl.buffer_ptrs, full.shape[1],
                                               rank * L["N"], L["N"], L["K"], 0)
                    else:
                        y = linear_call(L, toks[n][0], toks[n][1], M)
                        if mode == "nccl":
                            dist.all_gather_into_tensor(gathered[n], y)
                        elif mode == "nccl_overlap":
                            cur = torch.cuda.current_stream()
                            comm.wait_stream(cur)
                            with torch.cuda.stream(comm):
                                out = torch.empty_like(gathered[n])
                                dist.all_gather_into_tensor(out, y)
                                y.record_stream(comm)
                            done.append(out)
                            if len(done) > 8:
                                done.pop(0)
                if mode == "stores":
                    symm[names[0]][1].barrier(channel=0)   # one ordering point per layer
            if mode == "stores_flags":
                symm[names[0]][1].barrier(channel=1)    # the last layer's outputs are complete everywhere
            if mode == "nccl_overlap":
                torch.cuda.current_stream().wait_stream(comm)

        res = {"M": M}
        modes = (["no_gather"] if world > 1 else ["single"]) + \
                (["nccl"] if world > 1 else []) + (["nccl_overlap"] if world > 1 and M >= 512 else []) + \
                (["stores"] if symm is not None else []) + (["stores_flags"] if flags is not None else []) + \
                (["single"] if world > 1 else [])
        for mode in modes:
            s = torch.cuda.Stream()
            with torch.cuda.stream(s):
                one_stack(mode)
                torch.cuda.synchronize()
                use_graph = mode != "nccl_overlap"
                run = lambda: one_stack(mode)
                if use_graph:
                    try:
                        g = torch.cuda.CUDAGraph()
                        with torch.cuda.graph(g, stream=s):
                            one_stack(mode)
                        run = g.replay
                    except Exception:
                        use_graph = False
                        torch.cuda.synchronize()
                run()
                if world > 1:
                    dist.barrier()
                torch.cuda.synchronize()
                reps = 3 if M <= 64 else 2
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(s)
                for _ in range(reps):
                    run()
                e1.record(s)
                torch.cuda.synchronize()
                ms = e0.elapsed_time(e1) / reps
            t = torch.tensor([ms], dtype=torch.float64, device="cuda")
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            res[mode + "_ms"] = round(float(t[0]), 3)
            if not use_graph:
                res[mode + "_graph"] = False
        if world > 1:
            t1 = res["single_ms"]
            for mode in ("no_gather", "nccl", "nccl_overlap", "stores", "stores_flags"):
                if mode + "_ms" in res:
                    res[mode + "_eff"] = round(t1 / (world * res[mode + "_ms"]), 3)
        if symm is not None:
            # the stores really arrived: the last layer's full-width output equals the NCCL gather of the slices
            lay = stack[(layers_in_stack - 1) % distinct_layers]
            ok = True
            for n in names:
                y = linear_call(lay[n], toks[n][0], toks[n][1], M)
                parts = [torch.empty_like(y) for _ in range(world)]
                dist.all_gather(parts, y)
                ok = ok and torch.equal(torch.cat(parts, dim=1), symm[n][0])
            res["stores_match_nccl"] = bool(ok)
            if flags is not None:
                # the flag-ordered stack ran last (its final layer's outputs are what was just compared with NCCL):
                # every layer's flag word holds exactly the writing CTAs of all ranks, no bounded wait ran out
                ok2 = bool((flags[0][:layers_in_stack] == layer_ctas).all())
                try:
                    ops.poll_status()
                except Exception:
                    ok2 = False
                res["stores_flags_ok"] = bool(ok2)
        rows.append(res)
        del symm, symm2, flags, gathered
        torch.cuda.empty_cache()
    return rows


def run_extras(world, rank, local_rank, peaks):
    out = {}
    if world == 1:
        out["sweep"] = run_sweep(peaks)
        out["splitk"] = run_splitk(peaks)
        out["quant_per_token"] = run_quant(peaks)
        out["int8_mode"] = [run_one_i8(name, M) for name in SHAPES for M in (2048, 8192)]
    out["tp70b"] = {"ranks": world, "layers": 80, "rows": run_tp70b(world, rank)}
    return out


def run_one(name, M, reps=3):
    """One (shape, M) point of the sweep: microseconds, TOPS, algorithmic GB/s (for profiling a single kernel)."""
    N, K = SHAPES[name]
    C = max(3, -(-400_000_000 // (N * K // 2)))
    layers = [device_lqq(N, K, seed=31 * c + 1, want_gp=False) for c in range(C)]
    x, sc = device_tokens(M, K, seed=M)
    t = graph_time_us(lambda i: linear_call(layers[i % C], x, sc, M), C, reps)
    return {"shape": name, "M": M, "us": round(t, 2), "TOPS": round(2.0 * M * N * K / t / 1e6, 1),
            "alg_GBps": round(algorithmic_bytes(M, N, K) / t / 1e3, 1)}


def run_one_i8(name, M, reps=3):
    """One (shape, M) point of the INT8 x INT8 operator (``i8_gemm_scaled``, the plugin's INT8-weights mode) beside
    cuBLASLt's INT8 GEMM (``torch._int_mm``: int32 outputs, no scaling): microseconds and TOPS of either."""
    N, K = SHAPES[name]
    a = torch.randint(-127, 128, (M, K), dtype=torch.int8, device="cuda")
    ws = [torch.randint(-127, 128, (N, K), dtype=torch.int8, device="cuda") for _ in range(3)]
    sa = torch.rand(M, device="cuda") + 0.5
    sb = torch.rand(N, device="cuda") + 0.5
    t = graph_time_us(lambda i: torch.ops.liquidgemm.i8_gemm_scaled(a, ws[i % 3], sa, sb, 0), 3, reps)
    wt = [w.t() for w in ws]
    t2 = graph_time_us(lambda i: torch._int_mm(a, wt[i % 3]), 3, reps)
    ops_ = 2.0 * M * N * K / 1e6
    return {"shape": name, "M": M, "us": round(t, 2), "TOPS": round(ops_ / t, 1), "cublaslt_int8_us": round(t2, 2),
            "cublaslt_int8_TOPS": round(ops_ / t2, 1)}


if __name__ == "__main__":
    # ``python -m liquidgemm_b200.benchlib <hbm_gbs>``: single-GPU extras as one JSON object on stdout
    # (bench.py runs this in a child process so that the headline numbers never depend on it);
    # ``python -m liquidgemm_b200.benchlib one <qkv|gate_up|down> <M>``: a single point of the sweep;
    # ``... one_i8 <shape> <M>``: the same for the INT8 x INT8 operator beside cuBLASLt's INT8 GEMM.
    import json
    import sys
    torch.cuda.set_device(0)
    if len(sys.argv) > 1 and sys.argv[1] == "one":
        print(json.dumps(run_one(sys.argv[2], int(sys.argv[3]))))
        sys.exit(0)
    if len(sys.argv) > 1 and sys.argv[1] == "one_i8":
        from . import ops as _ops  # noqa: F401  (registers torch.ops.liquidgemm)
        print(json.dumps(run_one_i8(sys.argv[2], int(sys.argv[3]))))
        sys.exit(0)
    print(json.dumps(run_extras(1, 0, 0, {"hbm_gbs": float(sys.argv[1]) if len(sys.argv) > 1 else 6451.8,
                                          "bf16_tflops": float(sys.argv[2]) if len(sys.argv) > 2 else 1685.0})))
