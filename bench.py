#!/usr/bin/env python
"""Benchmark of the W4A8 linear hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--no-extras]

One *step* is one pass of the decode sweep: M in {1, 4, 8, 16} over the three Llama-3.1-8B linear
shapes (qkv 6144x4096, gate_up 28672x4096, down 4096x14336) = 12 linears through the decode
dispatch of the plugin (``torch.ops.liquidgemm.w4a8_wgmma_rs_fused`` on the tile blob, which picks the
streaming GEMV or a tensor-core kernel by M).  Weights are seeded synthetic LQQ data of those shapes
(no checkpoint is read).  Four weight copies rotate per launch: the linear of shape s at the i-th M
of step t reads copy (t + i) mod 4, so a copy is read again only after three other copies of the
same shape plus the rest of the sweep (more than 300 MB, over twice the 126 MB L2) went by.
Before anything is timed, every (shape, M) of the sweep runs once and a 16-channel slice of its
output, and its quantised tokens, are compared bit for bit with the CPU oracle (``parity`` in the line).

The JSON line printed by rank 0 carries
  value     weight GB/s (packed weight bytes N*K/2 per launch / device time), whole job
  e2e       the same metric from host buffers (ops.HostStepPlan over lq_w4a8_linear_host): per linear a pinned
            fp16 activation copy to the device, quant_per_token + linear, and the result copied back
  roofline  algorithmic bytes of the sweep / device time, against the measured HBM copy rate
  cpu_baseline  the CPU oracle (C, OpenMP) on the same sweep, timed on this host
  extras    the other benchmark configurations (split-K decode tiles, prefill TOPS, cuBLAS bf16
            beside every shape, the N-sharded 70B-shape stack when run on several GPUs)

With ``--impl reference`` rank 0 times the CPU restatement of the reference's own pure-PyTorch
path (the reference tree itself is not present on the GPU host) and prints the same line with
``"impl": "reference"``.
"""

from __future__ import annotations

import argparse
import ctypes
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SHAPES = {"qkv": (6144, 4096), "gate_up": (28672, 4096), "down": (4096, 14336)}
SHAPES_70B = {"qkv": (10240, 8192), "o": (8192, 8192), "gate_up": (57344, 8192), "down": (8192, 28672)}
SWEEP_M = (1, 4, 8, 16)
METRIC = "w4a8_decode_weight_GBps"
UNIT = "GB/s"
OUT_BF16 = 0


def algorithmic_bytes(M, N, K, out_bytes=2):
    """Packed codes + step/offset bytes + row scales + int8 tokens + token scales + output."""
    return N * K // 2 + 2 * N * K // 64 + 4 * N + M * K + 4 * M + M * N * out_bytes


def weight_bytes(N, K):
    return N * K // 2


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d.get("bf16_tflops", 1590.0)),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", 1400.0)), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# ----------------------------------------------------------------------------------------------
# synthetic LQQ data (seeded, generated on the host with numpy)
# ----------------------------------------------------------------------------------------------

def synth_lqq_codes(N, K, seed):
    """Seeded LQQ weight in code space (codes 0..15, steps 1..16, offsets keeping u <= 255).

    Quantising a 28672x4096 fp16 matrix on the host takes longer than the whole benchmark; the
    kernels' time does not depend on the values, so the benchmark draws valid codes directly and
    the parity tests cover quantised Gaussian + outlier weights."""
    rng = np.random.default_rng(seed)
    G = K // 64
    codes = rng.integers(0, 16, (N, K), dtype=np.uint8)
    step = rng.integers(1, 17, (N, G), dtype=np.int32)
    room = 255 - 15 * step
    off = np.minimum((rng.random((N, G)) * (room + 1)).astype(np.int32), room)
    s1 = (rng.random(N, dtype=np.float32) * np.float32(0.01) + np.float32(1e-4)).astype(np.float32)
    return codes, step.astype(np.uint8), off.astype(np.uint8), s1


# ----------------------------------------------------------------------------------------------
# clocks
# ----------------------------------------------------------------------------------------------

class ClockSampler:
    """Background ``nvidia-smi`` sampling (every 50 ms, with timestamps) started at program start;
    ``summary(t0, t1)`` keeps the samples whose wall-clock time falls inside the timed region (or,
    if the region was shorter than one period, the nearest ones)."""

    FIELDS = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")
    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.gpu_index)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def summary(self, t0, t1):
        import datetime
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0, "power_w": None}
        if self.proc is None:
            return out
        time.sleep(0.12)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        rows = []
        try:
            with open(self.path) as f:
                for line in f:
                    c = [x.strip() for x in line.split(",")]
                    if len(c) < 8:
                        continue
                    try:
                        ts = datetime.datetime.strptime(c[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                        rows.append((ts, float(c[1]), float(c[2]), float(c[3]), c[4:8]))
                    except ValueError:
                        continue
            os.unlink(self.path)
        except OSError:
            pass
        if not rows:
            return out
        inside = [r for r in rows if t0 - 0.03 <= r[0] <= t1 + 0.03]
        if not inside:
            mid = 0.5 * (t0 + t1)
            inside = sorted(rows, key=lambda r: abs(r[0] - mid))[:2]
        reasons = set()
        for r in inside:
            for name, val in zip(self.NAMES, r[4]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        out.update(sm_mhz=float(np.median([r[1] for r in inside])), sm_max_mhz=float(max(r[2] for r in inside)),
                   power_w=float(np.median([r[3] for r in inside])), samples=len(inside), reasons=sorted(reasons))
        return out


# ----------------------------------------------------------------------------------------------
# reference arm / CPU baseline
# ----------------------------------------------------------------------------------------------

def host_threads():
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return os.cpu_count() or 1


def cpu_sweep(reps):
    """Time the C oracle on the decode sweep.  Returns (seconds per sweep, threads used)."""
    from oracle import build_oracle
    lib = build_oracle.load()
    # all host cores whatever the launcher exported (torchrun sets OMP_NUM_THREADS=1 for its children)
    lib.lqo_set_num_threads(host_threads())
    threads = lib.lqo_num_threads()
    p = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    data = {}
    for i, (name, (N, K)) in enumerate(SHAPES.items()):
        data[name] = synth_lqq_codes(N, K, seed=7 + i)
    rng = np.random.default_rng(0)
    xs = {(name, M): rng.standard_normal((M, SHAPES[name][1]), dtype=np.float32) for name in SHAPES for M in SWEEP_M}
    ys = {(name, M): np.empty((M, SHAPES[name][0]), np.float32) for name in SHAPES for M in SWEEP_M}
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        for M in SWEEP_M:
            for name, (N, K) in SHAPES.items():
                codes, step, off, s1 = data[name]
                lib.lqo_w4a8_linear(p(xs[(name, M)]), p(codes), p(step), p(off), p(s1), p(ys[(name, M)]), M, N, K, 64)
        times.append(time.perf_counter() - t0)
    return times, threads


def sweep_weight_bytes():
    return sum(weight_bytes(*SHAPES[n]) for n in SHAPES) * len(SWEEP_M)


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    times, threads = cpu_sweep(args.warmup + args.steps)
    timed = times[args.warmup:]
    total = sum(timed)
    val = sweep_weight_bytes() * len(timed) / total / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": total / len(timed) * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8 x uint4 -> int32",
        "data": "synthetic",
        "config": {"workload": "decode GEMV sweep M in {1,4,8,16} x Llama-3.1-8B qkv/gate_up/down (configs[1])",
                   "group_size": 64, "out": "fp32"},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": "C/OpenMP restatement of quantize_activation + w4a8_matmul on the full sweep, "
                                   "one sweep per step"},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------------------------

PARITY_ROWS = 16


def build_device_sets(torch, ops, n_sets, seed_base):
    """n_sets independent copies of the three quantised layers on the device (tile blob only: the one
    weight format the dispatch reads).  Of every layer a 16-channel slice stays on the host for the
    parity gate."""
    from liquidgemm_b200.quant import LiquidQuantWeight
    sets = []
    for c in range(n_sets):
        layer = {}
        for name, (N, K) in SHAPES.items():
            codes, step, off, s1 = synth_lqq_codes(N, K, seed=seed_base + 17 * c + len(name))
            qw = LiquidQuantWeight(torch.from_numpy(codes).cuda(), torch.from_numpy(step).cuda(),
                                   torch.from_numpy(off).cuda(), torch.from_numpy(s1).cuda(), 64)
            rows = np.sort(np.random.default_rng(c).choice(N, PARITY_ROWS, replace=False))
            layer[name] = {"rs": ops.repack_rs_weight(qw).reshape(-1),
                           "s_u8": qw.s_u8, "offset_a": qw.offset_a, "s1": qw.s1, "N": N, "K": K,
                           "check": (rows, codes[rows].copy(), step[rows].copy(), off[rows].copy(), s1[rows].copy())}
            del qw, codes
        sets.append(layer)
    return sets


def parity_gate(torch, sets, acts, launches, run_linear):
    """Every (shape, M) of the sweep once on every weight copy: quantised tokens and a 16-channel slice of
    the bf16 output against the numpy oracle, bit for bit.  Returns (ok, cases checked)."""
    from oracle import lqq_oracle as O
    ok, n = True, 0
    for name, M in launches:
        a = acts[(name, M)]
        xq_want, sc_want = O.quantize_activation(a["host"].float().numpy())
        ok &= bool(np.array_equal(a["xq"].cpu().numpy(), xq_want))
        ok &= bool(np.array_equal(a["sc"].cpu().numpy().view(np.uint32), sc_want.view(np.uint32)))
        for layer_set in sets:
            L = layer_set[name]
            rows, codes, step, off, s1 = L["check"]
            y = run_linear(L, a["xq"], a["sc"], M, OUT_BF16)
            got = y[:, torch.from_numpy(rows).cuda()].cpu().view(torch.int16).numpy().view(np.uint16)
            want = O.w4a8_linear(xq_want, sc_want, O.LQQWeight(codes, step, off, s1, 64), O.OUT_BF16)
            ok &= bool(np.array_equal(got, want))
            n += 1
    return ok, n


# DRAM read+write bytes per launch / algorithmic bytes per launch, mean over the ncu captures of the decode
# kernels summarised under profiles/ (taken on single launches of the same shapes; the benchmark itself
# never runs under a profiler, so `roofline.traffic` is that measured ratio times the step's algorithmic bytes).
NCU_TRAFFIC_RATIO = 1.007


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--no-extras", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "native" else args.warmup

    if args.impl == "reference":
        run_reference_arm(args)
        return

    # peer stores only: symmetric memory is used without NVLink multicast objects
    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    from liquidgemm_b200 import ops  # loads the CUDA library; raises if it is not built
    from liquidgemm_b200._lib import lib

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    peaks = measured_peaks()
    n_sets = 4
    sets = build_device_sets(torch, ops, n_sets, seed_base=1000 * rank)

    gen = torch.Generator().manual_seed(rank)
    acts = {}
    for name, (N, K) in SHAPES.items():
        for M in SWEEP_M:
            x16 = torch.randn(M, K, generator=gen).to(torch.float16)
            xq, sc = torch.ops.liquidgemm.quant_per_token(x16.cuda())
            acts[(name, M)] = {"host": x16.pin_memory(), "dev16": x16.cuda(), "xq": xq, "sc": sc,
                               "out_host": torch.empty(M, N, dtype=torch.float16).pin_memory()}
    launches = [(name, M) for M in SWEEP_M for name in SHAPES]

    def decode_linear(L, xq, sc, M, out_dtype):
        """The op the plugin's forward calls (liquidgemm_b200.vllm_plugin.apply_layer): the fused linear on
        the tile blob, which dispatches on M inside the library."""
        return torch.ops.liquidgemm.w4a8_wgmma_rs_fused(xq, L["rs"], L["s_u8"], L["offset_a"], sc, L["s1"], L["N"],
                                                        L["K"], 64, out_dtype)

    def copy_for(step, name, M):
        return sets[(step + SWEEP_M.index(M)) % n_sets][name]

    def enqueue_sweep(c):
        for name, M in launches:
            a = acts[(name, M)]
            decode_linear(copy_for(c, name, M), a["xq"], a["sc"], M, OUT_BF16)

    parity_ok, parity_cases = parity_gate(torch, sets, acts, launches, decode_linear)

    stream = torch.cuda.Stream()
    graphs = []
    with torch.cuda.stream(stream):
        for c in range(n_sets):
            enqueue_sweep(c)
        torch.cuda.synchronize()
        for c in range(n_sets):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                enqueue_sweep(c)
            graphs.append(g)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    with torch.cuda.stream(stream):
        for i in range(args.warmup):
            graphs[i % n_sets].replay()
        barrier()
        wall0 = time.time()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for i in range(args.steps):
            graphs[i % n_sets].replay()
        e1.record(stream)
        barrier()
        wall1 = time.time()
        ms = e0.elapsed_time(e1)
    clocks = sampler.summary(wall0, wall1) if rank == 0 else None

    # ---- e2e: host buffers in, host buffers out, through the public API
    # One step = the same 12 linears as host-buffer requests (liquidgemm_b200.ops.HostStepPlan): per linear
    # a pinned fp16 activation copy to the device, quant_per_token, the linear, and the output copied back
    # to pinned host memory -- recorded once per weight rotation and replayed with one call per step.  The
    # requests of a step are independent and spread over three streams inside the plan.
    def requests_for(c):
        return [(acts[(name, M)]["host"], copy_for(c, name, M), acts[(name, M)]["out_host"]) for name, M in launches]

    e2e_stream = torch.cuda.Stream()          # one stream: the steps run strictly one after the other
    plans = [ops.HostStepPlan(requests_for(c), stream=e2e_stream) for c in range(n_sets)]
    e2e_steps = max(3, min(args.steps, 100))
    for i in range(3):
        plans[i % n_sets].run()
    for p in plans:
        p.synchronize()
    barrier()
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        plans[i % n_sets].run()
    for p in plans:
        p.synchronize()
    barrier()                                  # device-wide synchronise: every stream has drained
    e2e_ms = (time.perf_counter() - t0) * 1e3
    # the outputs that came back are the right ones (last replay of every plan)
    e2e_ok = True
    for name, M in launches:
        a = acts[(name, M)]
        c_last = (e2e_steps - 1) % n_sets
        want = decode_linear(copy_for(c_last, name, M), a["xq"], a["sc"], M, 1)
        e2e_ok &= bool(torch.equal(want.cpu(), a["out_host"]))

    t_ms = torch.tensor([ms, e2e_ms], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t_ms, op=dist.ReduceOp.MAX)
    ms, e2e_ms = float(t_ms[0]), float(t_ms[1])
    status = lib.lq_poll_status(torch.cuda.current_stream().cuda_stream)

    def kernels_of(name, M):
        """Kernel launches of one linear: 2 when the tile kernel splits K (planes + finish pass), else 1."""
        N, K = SHAPES[name]
        return lib.lq_gemm_launches(M, N, K, 0)
    launches_per_step = sum(kernels_of(n, M) for n, M in launches)
    wbytes = sweep_weight_bytes()
    abytes = sum(algorithmic_bytes(M, *SHAPES[n]) for n, M in launches)
    step_s = ms / 1e3 / args.steps
    value = world * wbytes / step_s / 1e9
    e2e_value = world * wbytes / (e2e_ms / 1e3 / e2e_steps) / 1e9
    achieved = abytes / step_s / 1e9

    extras = {}
    if not args.no_extras:
        if world == 1:
            # the secondary configurations run in a child process: nothing they do can touch the
            # numbers measured above
            try:
                env = dict(os.environ, CUDA_VISIBLE_DEVICES=os.environ.get("CUDA_VISIBLE_DEVICES", str(local_rank)))
                out = subprocess.run([sys.executable, "-m", "liquidgemm_b200.benchlib", str(peaks["hbm_gbs"]),
                                      str(peaks["bf16_tflops"])], cwd=ROOT,
                                     env=env, capture_output=True, text=True, timeout=900)
                extras = json.loads(out.stdout.strip().splitlines()[-1]) if out.returncode == 0 else {
                    "error": (out.stderr or "")[-400:]}
            except Exception as exc:
                extras = {"error": repr(exc)}
        else:
            try:
                from liquidgemm_b200 import benchlib
                extras = benchlib.run_extras(world, rank, local_rank, peaks)
            except Exception as exc:
                extras = {"error": repr(exc)}

    # A compact copy of the secondary results inside `config` (the full tables stay under `extras`).
    summary = {}
    try:
        if "sweep" in extras:
            summary["prefill"] = [
                {"shape": r["shape"], "M": r["M"], "TOPS": r["TOPS"], "of_4500": r["int8_frac_of_4500"],
                 "of_2x_measured_bf16": r.get("int8_frac_of_2x_bf16"), "x_cublas_bf16": r["speedup_vs_cublas_bf16"]}
                for r in extras["sweep"] if r["M"] in (512, 2048, 8192)]
            summary["decode_us"] = {f'{r["shape"]}:{r["M"]}': [r["us"], r["hbm_frac"], r["speedup_vs_cublas_bf16"]]
                                    for r in extras["sweep"] if r["M"] <= 128}
            summary["decode_us_columns"] = ["us per launch", "fraction of measured HBM rate", "x cuBLAS bf16"]
        if "int8_mode" in extras:
            # the plugin's INT8-weights mode (i8_gemm_scaled) beside cuBLASLt's INT8 GEMM: [TOPS, cuBLASLt TOPS]
            summary["int8_mode_tops"] = {f'{r["shape"]}:{r["M"]}': [r["TOPS"], r["cublaslt_int8_TOPS"]]
                                         for r in extras["int8_mode"]}
        if "tp70b" in extras:
            summary["tp70b_stack_ms"] = extras["tp70b"]["rows"]
    except Exception as exc:
        summary["error"] = repr(exc)

    cpu = None
    if rank == 0 and world == 1:
        times, threads = cpu_sweep(3)
        best = min(times)
        cpu = {"value": wbytes / best / 1e9, "unit": UNIT, "cores": threads, "kind": "port",
               "sample": "C/OpenMP oracle (quantize_activation + w4a8_matmul) on the full 12-launch sweep, best of 3"}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "int8 x uint4 -> int32", "data": "synthetic",
            "config": {"workload": "decode GEMV sweep M in {1,4,8,16} x Llama-3.1-8B qkv/gate_up/down (configs[1])",
                       "group_size": 64, "out": "bf16", "launches_per_step": len(launches),
                       "l2": f"{n_sets} weight copies rotate per launch (a copy is re-read after > 300 MB of other "
                             "weights, over 2 x L2); step captured in a CUDA graph",
                       "sharding": "each rank owns a full set of output channels (N-sharded, no collective)",
                       "summary": summary},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": achieved / peaks["hbm_gbs"], "traffic": NCU_TRAFFIC_RATIO * abytes,
                         "of": peaks["source"], "traffic_source": f"ncu DRAM bytes / algorithmic bytes = {NCU_TRAFFIC_RATIO} on single launches "
                                           "(profiles/decode_kernels_ncu_full.md) x this step's algorithmic bytes",
                         "kernel": "w4a8_tile_kernel (gate_up and down at M = 4, 8, 16; down with finish_kernel), "
                                   "w4a8_decode_tc_kernel (qkv at M = 4, 8, 16), gemv_blob_kernel (M = 1): the 12-op sweep",
                         "algorithmic_bytes_per_step": abytes},
            "cpu_baseline": cpu,
            "e2e": {"value": e2e_value, "unit": UNIT,
                    "h2d_bytes_per_step": sum(M * SHAPES[n][1] * 2 for n, M in launches),
                    "d2h_bytes_per_step": sum(M * SHAPES[n][0] * 2 for n, M in launches),
                    "steps": e2e_steps, "ms_per_step": e2e_ms / e2e_steps, "outputs_match_device_path": bool(e2e_ok),
                    "api": "liquidgemm_b200.ops.HostStepPlan.run(): pinned fp16 tokens -> H2D -> quant_per_token -> "
                           "linear -> D2H of every output, one recorded step per call"},
            "gpu_launches": launches_per_step * args.steps,
            "parity": bool(parity_ok and status == 0), "parity_cases": parity_cases,
            "clocks": clocks, "device_status": status, "extras": extras,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
