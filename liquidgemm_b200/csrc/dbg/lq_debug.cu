// Measurement-only kernels (no product path calls them): the issue/execute rate of
// tcgen05.mma kind::i8 for a given N, with the A operand in tensor memory or in shared memory.
#include "../lq_common.cuh"
#include "../lq_tc_ptx.cuh"

namespace lq {
__device__ __forceinline__ bool dbg_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}"
               : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// One lane of the (converged) warp, the same one every time.
__device__ __forceinline__ bool dbg_elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}
// Bounded: gives up after ~2^22 polls so that a wrong experiment ends instead of hanging.
__device__ __forceinline__ void dbg_wait(uint32_t bar, uint32_t parity, int mode) {
  for (int i = 0; i < (1 << 22); ++i) {
    if ((mode & 64) ? dbg_test_wait(bar, parity) : ptx::mbar_try_wait(bar, parity)) return;
  }
}
}  // namespace lq

namespace lq {

// One CTA: `iters` groups of four 128 x N x 32 MMAs into the same accumulator, one commit per group
// (like one k-step of the GEMM main loop), then a wait for the last commit.  out[blockIdx.x] =
// cycles from the first issue to the completion of the last MMA.
__global__ void __launch_bounds__(128, 1)
mma_rate_kernel(int n, int iters, int a_in_tmem, long long* out) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_slot;
  const uint32_t bar_addr = smem_u32(&bar);
  if (threadIdx.x == 0) {
    ptx::mbar_init(bar_addr, 1);
    ptx::fence_mbar_init();
  }
  // operands: B tile (256 rows x 128 B) at base, A tile (128 x 128 B) behind it; contents are
  // whatever the memory holds after this fill (values do not change the timing)
  for (int i = threadIdx.x; i < (1024 + 32768 + 16384) / 4; i += blockDim.x)
    reinterpret_cast<uint32_t*>(smem_raw + (base - raw_addr))[i] = 0x01020304u * (i + 1);
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  // a_in_tmem bit 1: allocate 256 columns (accumulator <= 128 wide) so two CTAs share an SM
  const uint32_t cols = (a_in_tmem & 2) ? 256u : 512u;
  const uint32_t a_col = cols / 2;
  // bit 2: alternate between two accumulators (columns [0, n) and [n, 2n)) from one MMA to the next, to tell a
  // dependent-accumulate latency from an issue limit
  const uint32_t alt = (a_in_tmem & 4) ? (uint32_t)n : 0u;
  // bit 3: the whole warp walks the issue loop and one elected lane issues (instead of `if (thread 0) loop`)
  const bool uniform_issue = (a_in_tmem & 8) != 0;
  a_in_tmem &= 1;
  if (threadIdx.x < 32) {
    ptx::tmem_alloc(smem_u32(&tmem_slot), cols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  if (uniform_issue) {
    // The whole warp walks the loop (operands stay warp-uniform values); one elected lane issues.
    if (threadIdx.x < 32) {
      const uint32_t idesc = ptx::idesc_i8(n);
      const bool leader = dbg_elect_one();
      const long long t0 = clock64();
      for (int i = 0; i < iters; ++i) {
        // a stage-dependent operand address, as in a real main loop
        const uint32_t sbase = base + (uint32_t)(i & 1) * 1024u;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint64_t bdesc = ptx::smem_desc_sw128(sbase + j * 32);
          const uint32_t acc = tmem_base + ((j & 1) ? alt : 0u);
          if (leader) {
            if (a_in_tmem) ptx::mma_i8_ts(acc, tmem_base + a_col + j * 8, bdesc, idesc, 1u);
            else ptx::mma_i8_ss(acc, ptx::smem_desc_sw128(sbase + 32768 + j * 32), bdesc, idesc, 1u);
          }
        }
        __syncwarp();
      }
      if (leader) {
        const long long t_issue = clock64();
        ptx::tc_commit(bar_addr);
        ptx::mbar_wait_bounded(bar_addr, 0u, 2000000000ull);
        const long long t1 = clock64();
        out[blockIdx.x * 2] = t1 - t0;
        out[blockIdx.x * 2 + 1] = t_issue - t0;
      }
      __syncwarp();
    }
  } else if (threadIdx.x == 0) {
    const uint32_t idesc = ptx::idesc_i8(n);
    const long long t0 = clock64();
    for (int i = 0; i < iters; ++i) {
      const uint32_t sbase = base + (uint32_t)(i & 1) * 1024u;   // a stage-dependent operand address
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint64_t bdesc = ptx::smem_desc_sw128(sbase + j * 32);
        const uint32_t acc = tmem_base + ((j & 1) ? alt : 0u);
        if (a_in_tmem) ptx::mma_i8_ts(acc, tmem_base + a_col + j * 8, bdesc, idesc, 1u);
        else ptx::mma_i8_ss(acc, ptx::smem_desc_sw128(sbase + 32768 + j * 32), bdesc, idesc, 1u);
      }
    }
    const long long t_issue = clock64();
    ptx::tc_commit(bar_addr);
    ptx::mbar_wait_bounded(bar_addr, 0u, 2000000000ull);
    const long long t1 = clock64();
    out[blockIdx.x * 2] = t1 - t0;
    out[blockIdx.x * 2 + 1] = t_issue - t0;
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (threadIdx.x < 32) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, cols);
  }
}

}  // namespace lq

// out: device buffer of 2 x ctas int64: total cycles and cycles spent issuing, per CTA.
extern "C" LQ_API int lq_debug_mma_rate(int n, int iters, int a_in_tmem, int ctas, long long* out, void* stream) {
  if (n < 16 || n > 256 || n % 16 || iters <= 0 || ctas <= 0 || !out) return LQ_ERR_BAD_ARG;
  if ((a_in_tmem & 2) && n > 128) return LQ_ERR_BAD_ARG;
  if ((a_in_tmem & 4) && n > ((a_in_tmem & 2) ? 64 : 128)) return LQ_ERR_BAD_ARG;
  const int smem = 2048 + 32768 + 16384;
  static bool attr_done = false;
  if (!attr_done) {
    cudaFuncSetAttribute(lq::mma_rate_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    attr_done = true;
  }
  lq::mma_rate_kernel<<<ctas, 128, smem, lq::as_stream(stream)>>>(n, iters, a_in_tmem, out);
  return lq::check_launch("mma_rate_kernel");
}

namespace lq {
// Cost (cycles per operation, one thread, back to back) of the synchronisation primitives the GEMM
// roles execute once per k-step.  out[0..]: clock64 pair, try_wait on a completed phase, arrive,
// arrive.expect_tx (with matching bulk copy of 16 bytes), tcgen05.commit, bulk copy issue of 8 KB.
__global__ void __launch_bounds__(32, 1) sync_cost_kernel(const uint8_t* src, long long* out) {
  __shared__ uint64_t bar[4];
  __shared__ __align__(128) uint8_t buf[8192 + 128];
  const uint32_t b0 = smem_u32(&bar[0]), b1 = smem_u32(&bar[1]), b2 = smem_u32(&bar[2]);
  if (threadIdx.x == 0) {
    ptx::mbar_init(b0, 1);
    ptx::mbar_init(b1, 1);
    ptx::mbar_init(b2, 1);
    ptx::fence_mbar_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const int R = 64;
    long long t0, t1;
    t0 = clock64();
    for (int i = 0; i < R; ++i) asm volatile("" ::: "memory");
    t1 = clock64();
    out[0] = t1 - t0;                                   // empty loop + clock pair
    t0 = clock64();
    long long acc = 0;
    for (int i = 0; i < R; ++i) acc += clock64();
    t1 = clock64();
    out[1] = (t1 - t0) / R + (acc & 0);                 // clock64
    t0 = clock64();
    int okc = 0;
    for (int i = 0; i < R; ++i) okc += ptx::mbar_try_wait(b0, 1u) ? 1 : 0;   // fresh barrier, previous phase
    t1 = clock64();
    out[2] = (t1 - t0) / R;
    out[8] = okc;
    t0 = clock64();
    for (int i = 0; i < R; ++i) {                        // arrive completes a phase each time (count 1)
      ptx::mbar_arrive(b1);
    }
    t1 = clock64();
    out[3] = (t1 - t0) / R;
    t0 = clock64();
    okc = 0;
    for (int i = 0; i < R; ++i) okc += ptx::mbar_try_wait(b1, 1u) ? 1 : 0;   // completed phases
    t1 = clock64();
    out[4] = (t1 - t0) / R;
    t0 = clock64();
    for (int i = 0; i < 16; ++i) {
      ptx::mbar_expect_tx(b2, 8192);
      ptx::bulk_load(smem_u32(buf), src + (size_t)i * 8192, 8192, b2);
      dbg_wait(b2, (uint32_t)i & 1u, 0);
    }
    t1 = clock64();
    out[5] = (t1 - t0) / 16;                             // expect_tx + 8 KB bulk copy round trip
    t0 = clock64();
    for (int i = 0; i < 16; ++i) ptx::tc_commit(b0);   // nothing outstanding: arrives at once
    t1 = clock64();
    out[6] = (t1 - t0) / 16;
    // issue cost only: 8 copies in flight on one barrier
    ptx::mbar_expect_tx(b2, 8 * 1024);
    t0 = clock64();
    for (int i = 0; i < 8; ++i) ptx::bulk_load(smem_u32(buf) + i * 1024, src + (size_t)i * 1024, 1024, b2);
    t1 = clock64();
    out[7] = (t1 - t0) / 8;
    dbg_wait(b2, 0u, 0);
  }
  __syncthreads();
}
}  // namespace lq

extern "C" LQ_API int lq_debug_sync_cost(const void* src_128k, long long* out16, void* stream) {
  lq::sync_cost_kernel<<<1, 32, 0, lq::as_stream(stream)>>>(static_cast<const uint8_t*>(src_128k), out16);
  return lq::check_launch("sync_cost_kernel");
}

namespace lq {
// Pure streaming test: each CTA pulls `steps` blocks of `stage_bytes` (contiguous, CTA-private
// region of `src`) through a ring of `ns` shared-memory stages with bulk copies; one thread
// produces, one thread consumes (wait full -> arrive empty).  Upper bound for any TMA-fed kernel.
__global__ void __launch_bounds__(64, 1)
tma_stream_kernel(const uint8_t* src, int stage_bytes, int ns, int steps, int wrap, int share, long long* cycles) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 127u) & ~127u;
  __shared__ uint64_t bars[64];
  if (threadIdx.x == 0) {
    for (int i = 0; i < ns; ++i) {
      ptx::mbar_init(smem_u32(&bars[i]), 1);
      ptx::mbar_init(smem_u32(&bars[32 + i]), 1);
    }
    ptx::fence_mbar_init();
  }
  __syncthreads();
  const long long t0 = clock64();
  // wrap > 0: the CTA re-reads a region of `wrap` stages (an L2-resident stream when the regions of all CTAs
  // fit there); share > 1: that many consecutive CTAs read the same region (tiles shared between CTAs).
  const int span = wrap > 0 ? wrap : steps;
  const uint8_t* my = src + (size_t)(blockIdx.x / share) * span * stage_bytes;
  if (threadIdx.x == 0) {
    int s = 0, w = 0;
    uint32_t ph = 0;
    for (int i = 0; i < steps; ++i) {
      dbg_wait(smem_u32(&bars[32 + s]), ph ^ 1u, 0);
      ptx::mbar_expect_tx(smem_u32(&bars[s]), stage_bytes);
      ptx::bulk_load(base + s * stage_bytes, my + (size_t)w * stage_bytes, stage_bytes, smem_u32(&bars[s]));
      if (++w == span) w = 0;
      if (++s == ns) { s = 0; ph ^= 1u; }
    }
  } else if (threadIdx.x == 32) {
    int s = 0;
    uint32_t ph = 0;
    for (int i = 0; i < steps; ++i) {
      dbg_wait(smem_u32(&bars[s]), ph, 0);
      ptx::mbar_arrive(smem_u32(&bars[32 + s]));
      if (++s == ns) { s = 0; ph ^= 1u; }
    }
    cycles[blockIdx.x] = clock64() - t0;
  }
  __syncthreads();
}
}  // namespace lq

static int launch_tma_stream(const void* src, int stage_bytes, int ns, int steps, int wrap, int share, int ctas,
                             long long* cycles, void* stream) {
  if (ns < 1 || ns > 32 || stage_bytes % 16 || stage_bytes * ns > 200 * 1024 || share < 1 || wrap < 0) return LQ_ERR_BAD_ARG;
  const int smem = stage_bytes * ns + 256;
  cudaFuncSetAttribute(lq::tma_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 201 * 1024);
  lq::tma_stream_kernel<<<ctas, 64, smem, lq::as_stream(stream)>>>(static_cast<const uint8_t*>(src), stage_bytes, ns,
                                                                   steps, wrap, share, cycles);
  return lq::check_launch("tma_stream_kernel");
}

extern "C" LQ_API int lq_debug_tma_stream(const void* src, int stage_bytes, int ns, int steps, int ctas,
                                          long long* cycles, void* stream) {
  return launch_tma_stream(src, stage_bytes, ns, steps, 0, 1, ctas, cycles, stream);
}

// The same stream out of L2: every group of `share` CTAs re-reads its own region of `wrap` stages.
extern "C" LQ_API int lq_debug_tma_stream_l2(const void* src, int stage_bytes, int ns, int steps, int wrap, int share,
                                             int ctas, long long* cycles, void* stream) {
  return launch_tma_stream(src, stage_bytes, ns, steps, wrap, share, ctas, cycles, stream);
}

namespace lq {
// Skeleton of the GEMM hand-offs without any arithmetic, to cost the synchronisation structure:
//   thread 0      producer: wait empty -> expect_tx + bulk copy
//   warps 4..7    "dequant": lane 0 waits full, all 128 threads read 64 bytes, arrive empty,
//                 (mode & 2) wait afree, arrive aready
//   thread 32     (mode & 2) "MMA": wait full, wait aready, then release empty/afree either with
//                 tcgen05.commit (mode & 4) or with plain arrives
// empty count = 128 (+1 with the MMA thread).  nt = operand ring depth.
__global__ void __launch_bounds__(256, 1)
skeleton_kernel(const uint8_t* src, int stage_bytes, int ns, int nt, int steps, int mode, long long* cycles,
                unsigned* sink) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 127u) & ~127u;
  const uint8_t* gen = smem_raw + (base - raw_addr);
  __shared__ uint64_t bars[128];   // full[32], empty[32], aready[32], afree[32]
  const bool with_mma = mode & 2;
  if (threadIdx.x == 0) {
    for (int i = 0; i < ns; ++i) {
      ptx::mbar_init(smem_u32(&bars[i]), 1);
      ptx::mbar_init(smem_u32(&bars[32 + i]), ((mode & 8) ? 4 : 128) + (with_mma ? 1 : 0));
    }
    for (int i = 0; i < nt; ++i) {
      ptx::mbar_init(smem_u32(&bars[64 + i]), (mode & 8) ? 4 : 128);
      ptx::mbar_init(smem_u32(&bars[96 + i]), 1);
    }
    ptx::fence_mbar_init();
  }
  __syncthreads();
  const long long t0 = clock64();
  const uint8_t* my = (mode & 32) ? src + (size_t)(blockIdx.x & 7) * 64 * stage_bytes
                                  : src + (size_t)blockIdx.x * steps * stage_bytes;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if ((mode & 256) ? warp == 0 : threadIdx.x == 0) {
    int s = 0; uint32_t ph = 0;
    for (int i = 0; i < steps; ++i) {
      dbg_wait(smem_u32(&bars[32 + s]), ph ^ 1u, mode);
      if (lane == 0) ptx::mbar_expect_tx(smem_u32(&bars[s]), stage_bytes);
      const size_t off = (mode & 32) ? (size_t)(i & 63) * stage_bytes : (size_t)i * stage_bytes;
      if (lane == 0) ptx::bulk_load(base + s * stage_bytes, my + off, stage_bytes, smem_u32(&bars[s]));
      if (mode & 256) __syncwarp();
      if (++s == ns) { s = 0; ph ^= 1u; }
    }
  } else if (((mode & 256) ? warp == 1 : threadIdx.x == 32) && with_mma) {
    int s = 0, t = 0; uint32_t ph = 0, pht = 0;
    for (int i = 0; i < steps; ++i) {
      dbg_wait(smem_u32(&bars[s]), ph, mode);
      dbg_wait(smem_u32(&bars[64 + t]), pht, mode);
      if (lane == 0) {
        if (mode & 4) {
          ptx::tc_commit(smem_u32(&bars[32 + s]));
          ptx::tc_commit(smem_u32(&bars[96 + t]));
        } else {
          ptx::mbar_arrive(smem_u32(&bars[32 + s]));
          ptx::mbar_arrive(smem_u32(&bars[96 + t]));
        }
      }
      if (mode & 256) __syncwarp();
      if (++s == ns) { s = 0; ph ^= 1u; }
      if (++t == nt) { t = 0; pht ^= 1u; }
    }
    if (lane == 0) cycles[blockIdx.x] = clock64() - t0;
  } else if (warp >= 4) {
    int s = 0, t = 0; uint32_t ph = 0, pht = 0;
    unsigned acc = 0;
    const int row = threadIdx.x - 128;
    for (int i = 0; i < steps; ++i) {
      if (mode & 128) dbg_wait(smem_u32(&bars[s]), ph, mode);
      else { if (lane == 0) dbg_wait(smem_u32(&bars[s]), ph, mode); __syncwarp(); }
      const uint4 v = *reinterpret_cast<const uint4*>(gen + s * stage_bytes + row * 16);
      acc += v.x ^ v.y ^ v.z ^ v.w;
      if (mode & 8) { __syncwarp(); if (lane == 0) ptx::mbar_arrive(smem_u32(&bars[32 + s])); }
      else ptx::mbar_arrive(smem_u32(&bars[32 + s]));
      if (with_mma) {
        if (mode & 128) dbg_wait(smem_u32(&bars[96 + t]), pht ^ 1u, mode);
        else { if (lane == 0) dbg_wait(smem_u32(&bars[96 + t]), pht ^ 1u, mode); __syncwarp(); }
        if (mode & 8) { if (lane == 0) ptx::mbar_arrive(smem_u32(&bars[64 + t])); }
        else ptx::mbar_arrive(smem_u32(&bars[64 + t]));
      }
      if (++s == ns) { s = 0; ph ^= 1u; }
      if (++t == nt) { t = 0; pht ^= 1u; }
    }
    if (!with_mma && threadIdx.x == 128) cycles[blockIdx.x] = clock64() - t0;
    if (acc == 0x12345678u) sink[0] = acc;
  }
  __syncthreads();
}
}  // namespace lq

extern "C" LQ_API int lq_debug_skeleton(const void* src, int stage_bytes, int ns, int nt, int steps, int mode,
                                        int ctas, long long* cycles, void* stream) {
  if (ns < 1 || ns > 32 || nt < 1 || nt > 32 || stage_bytes % 16 || stage_bytes * ns > 200 * 1024) return LQ_ERR_BAD_ARG;
  const int smem = stage_bytes * ns + 256;
  cudaFuncSetAttribute(lq::skeleton_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 201 * 1024);
  lq::skeleton_kernel<<<ctas, 256, smem, lq::as_stream(stream)>>>(static_cast<const uint8_t*>(src), stage_bytes, ns, nt,
                                                                  steps, mode, cycles,
                                                                  reinterpret_cast<unsigned*>(cycles + ctas));
  return lq::check_launch("skeleton_kernel");
}

namespace lq {
// Streaming test with each stage assembled from `rows` separate bulk copies (one per producer lane)
// of `row_bytes` each, taken from rows that are `row_stride` bytes apart: the access pattern of a
// row-major weight matrix fetched as short row pieces.  One consumer thread releases the stages.
__global__ void __launch_bounds__(64, 1)
tma_rows_kernel(const uint8_t* src, int rows, int row_bytes, long row_stride, int ns, int steps, int pieces_per_row,
                long long* cycles) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 127u) & ~127u;
  __shared__ uint64_t bars[64];
  const int stage_bytes = rows * row_bytes;
  if (threadIdx.x == 0) {
    for (int i = 0; i < ns; ++i) {
      ptx::mbar_init(smem_u32(&bars[i]), 1);
      ptx::mbar_init(smem_u32(&bars[32 + i]), 1);
    }
    ptx::fence_mbar_init();
  }
  __syncthreads();
  const long long t0 = clock64();
  const int lane = threadIdx.x & 31;
  if (threadIdx.x < 32) {
    int s = 0;
    uint32_t ph = 0;
    for (int i = 0; i < steps; ++i) {
      dbg_wait(smem_u32(&bars[32 + s]), ph ^ 1u, 0);
      if (lane == 0) ptx::mbar_expect_tx(smem_u32(&bars[s]), stage_bytes);
      __syncwarp();
      if (lane < rows) {
        // unit u = blockIdx.x * steps + i: row group u / pieces_per_row, piece u % pieces_per_row
        const long u = (long)blockIdx.x * steps + i;
        const long grp = u / pieces_per_row, piece = u % pieces_per_row;
        const uint8_t* p = src + (grp * rows + lane) * row_stride + piece * row_bytes;
        ptx::bulk_load(base + s * stage_bytes + lane * row_bytes, p, row_bytes, smem_u32(&bars[s]));
      }
      if (++s == ns) { s = 0; ph ^= 1u; }
    }
  } else if (threadIdx.x == 32) {
    int s = 0;
    uint32_t ph = 0;
    for (int i = 0; i < steps; ++i) {
      dbg_wait(smem_u32(&bars[s]), ph, 0);
      ptx::mbar_arrive(smem_u32(&bars[32 + s]));
      if (++s == ns) { s = 0; ph ^= 1u; }
    }
    cycles[blockIdx.x] = clock64() - t0;
  }
  __syncthreads();
}
}  // namespace lq

extern "C" LQ_API int lq_debug_tma_rows(const void* src, int rows, int row_bytes, long row_stride, int ns, int steps,
                                        int pieces_per_row, int ctas, long long* cycles, void* stream) {
  if (rows < 1 || rows > 32 || ns < 1 || ns > 32 || row_bytes % 16 || (long)rows * row_bytes * ns > 200 * 1024)
    return LQ_ERR_BAD_ARG;
  const int smem = rows * row_bytes * ns + 256;
  cudaFuncSetAttribute(lq::tma_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 201 * 1024);
  lq::tma_rows_kernel<<<ctas, 64, smem, lq::as_stream(stream)>>>(static_cast<const uint8_t*>(src), rows, row_bytes,
                                                                 row_stride, ns, steps, pieces_per_row, cycles);
  return lq::check_launch("tma_rows_kernel");
}

namespace lq {
// Two independent bulk-copy rings inside one CTA (producers: threads 0 and 64, consumers: threads 32 and 96):
// whether the fixed cost of a bulk copy is paid per issuing thread or per CTA.
__global__ void __launch_bounds__(128, 1)
tma_stream2_kernel(const uint8_t* src, int stage_bytes, int ns, int steps, int wrap, long long* cycles) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 127u) & ~127u;
  __shared__ uint64_t bars[128];
  const int ring = threadIdx.x >> 6;            // 0 or 1
  const int role = (threadIdx.x >> 5) & 1;      // 0 producer warp, 1 consumer warp
  if (threadIdx.x == 0) {
    for (int i = 0; i < 2 * ns; ++i) {
      ptx::mbar_init(smem_u32(&bars[i]), 1);
      ptx::mbar_init(smem_u32(&bars[64 + i]), 1);
    }
    ptx::fence_mbar_init();
  }
  __syncthreads();
  const long long t0 = clock64();
  const int span = wrap > 0 ? wrap : steps;
  const uint8_t* my = src + (size_t)(blockIdx.x * 2 + ring) * span * stage_bytes;
  const uint32_t ring_smem = base + ring * ns * stage_bytes;
  uint64_t* full = &bars[ring * ns];
  uint64_t* empty = &bars[64 + ring * ns];
  if ((threadIdx.x & 31) == 0) {
    int s = 0, w = 0;
    uint32_t ph = 0;
    for (int i = 0; i < steps; ++i) {
      if (role == 0) {
        dbg_wait(smem_u32(&empty[s]), ph ^ 1u, 0);
        ptx::mbar_expect_tx(smem_u32(&full[s]), stage_bytes);
        ptx::bulk_load(ring_smem + s * stage_bytes, my + (size_t)w * stage_bytes, stage_bytes, smem_u32(&full[s]));
        if (++w == span) w = 0;
      } else {
        dbg_wait(smem_u32(&full[s]), ph, 0);
        ptx::mbar_arrive(smem_u32(&empty[s]));
      }
      if (++s == ns) { s = 0; ph ^= 1u; }
    }
    if (role == 1) cycles[blockIdx.x * 2 + ring] = clock64() - t0;
  }
  __syncthreads();
}
}  // namespace lq

extern "C" LQ_API int lq_debug_tma_stream2(const void* src, int stage_bytes, int ns, int steps, int wrap, int ctas,
                                           long long* cycles, void* stream) {
  if (ns < 1 || ns > 32 || stage_bytes % 16 || 2 * stage_bytes * ns > 200 * 1024 || wrap < 0) return LQ_ERR_BAD_ARG;
  const int smem = 2 * stage_bytes * ns + 256;
  cudaFuncSetAttribute(lq::tma_stream2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 201 * 1024);
  lq::tma_stream2_kernel<<<ctas, 128, smem, lq::as_stream(stream)>>>(static_cast<const uint8_t*>(src), stage_bytes, ns,
                                                                     steps, wrap, cycles);
  return lq::check_launch("tma_stream2_kernel");
}

namespace lq {
// tcgen05.mma.cta_group::2 (a pair of CTAs on two SMs issues one 256 x N x 32 MMA; each CTA holds 128 rows of A
// and of the accumulator in its own tensor memory and N / 2 rows of B in its own shared memory): the issue
// rate seen by the leader CTA, like mma_rate_kernel.  out[2 * cta] = cycles to completion, [2 * cta + 1] = status
// (0 ok, 1 the wait for the commit ran out).
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(128, 1)
mma_rate2_kernel(int n, int iters, int a_in_tmem, int extra, long long* out) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  __shared__ uint64_t bar;
  __shared__ uint64_t side_bar[3];   // extra & 1 / & 2: one / two more commits per group of four MMAs go here;
                                     // [2] is a completed barrier for the extra & 4 wait
  __shared__ uint32_t tmem_slot;
  const uint32_t bar_addr = smem_u32(&bar);
  uint32_t rank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  if (threadIdx.x == 0) {
    ptx::mbar_init(bar_addr, 1);
    for (int i = 0; i < 3; ++i) ptx::mbar_init(smem_u32(&side_bar[i]), 1);
    ptx::fence_mbar_init();
    ptx::mbar_arrive(smem_u32(&side_bar[2]));   // phase 0 of [2] is complete
  }
  for (int i = threadIdx.x; i < (1024 + 16384 + 16384) / 4; i += blockDim.x)
    reinterpret_cast<uint32_t*>(smem_raw + (base - raw_addr))[i] = 0x01020304u * (i + 1);
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  if (threadIdx.x < 32) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  ptx::tc_fence_before();
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  ptx::tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  long long t0 = clock64();
  if (rank == 0 && threadIdx.x < 32) {
    // the whole warp walks the loop, one elected lane issues (see ptx::elect_one)
    const bool leader = ptx::elect_one();
    const uint32_t idesc = ptx::idesc_i8_pair(n);
    t0 = clock64();
    for (int i = 0; i < iters; ++i) {
      const uint32_t sbase = base + (uint32_t)(i & 1) * 1024u;   // a stage-dependent operand address
      if (leader) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint64_t bdesc = ptx::smem_desc_sw128(sbase + j * 32);
          if (a_in_tmem) {
            ptx::mma_i8_ts_pair(tmem_base, tmem_base + 256u + j * 8, bdesc, idesc, 1u);
          } else {
            const uint64_t adesc = ptx::smem_desc_sw128(sbase + 16384 + j * 32);
            asm volatile(
                "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_base),
                "l"(adesc), "l"(bdesc), "r"(idesc), "r"(1u)
                : "memory");
          }
        }
        if (extra & 3) ptx::tc_commit_pair(smem_u32(&side_bar[0]));
        if (extra & 2) ptx::tc_commit_pair(smem_u32(&side_bar[1]));
      }
      if (extra & 4) {
        ptx::mbar_wait_bounded(smem_u32(&side_bar[2]), 0u, 1000000ull);
        ptx::tc_fence_after();
      }
      __syncwarp();
    }
    if (leader) ptx::tc_commit_pair(bar_addr);
  }
  if (threadIdx.x == 0) {
    const bool ok = ptx::mbar_wait_bounded(bar_addr, 0u, 2000000000ull);
    out[blockIdx.x * 2] = clock64() - t0;
    out[blockIdx.x * 2 + 1] = ok ? 0 : 1;
  }
  ptx::tc_fence_before();
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  if (threadIdx.x < 32) {
    ptx::tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}
}  // namespace lq

extern "C" LQ_API int lq_debug_mma_rate2(int n, int iters, int a_in_tmem, int extra, int ctas, long long* out,
                                         void* stream) {
  if (n < 32 || n > 256 || n % 32 || iters <= 0 || ctas <= 0 || (ctas & 1) || !out) return LQ_ERR_BAD_ARG;
  const int smem = 2048 + 16384 + 16384;
  cudaFuncSetAttribute(lq::mma_rate2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  lq::mma_rate2_kernel<<<ctas, 128, smem, lq::as_stream(stream)>>>(n, iters, a_in_tmem, extra, out);
  return lq::check_launch("mma_rate2_kernel");
}

namespace lq {
// Hand-over between two kernels launched with programmatic stream serialisation: kernel "first" (one CTA per SM)
// optionally allocates tensor memory and writes `out_bytes_per_cta` bytes, stamps %globaltimer just before it
// ends; kernel "second" stamps %globaltimer when griddepcontrol.wait returns.  stamps[0] = latest end stamp of the
// first kernel (atomicMax), stamps[1] = earliest return of the wait in the second (atomicMin).
__global__ void __launch_bounds__(320, 1)
handover_first_kernel(int use_tmem, int out_bytes_per_cta, uint8_t* out, unsigned long long* stamps, int smem_dummy) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint32_t tmem_slot;
  (void)smem_dummy;
  allow_dependents();
  dependency_wait();
  uint32_t tmem_base = 0;
  if (use_tmem) {
    if (threadIdx.x < 32) {
      ptx::tmem_alloc(smem_u32(&tmem_slot), 256);
      ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    tmem_base = tmem_slot;
  }
  // some work: stream the CTA's share of `out`
  uint4* dst = reinterpret_cast<uint4*>(out + (size_t)blockIdx.x * out_bytes_per_cta);
  for (int i = threadIdx.x; i < out_bytes_per_cta / 16; i += blockDim.x) dst[i] = make_uint4(i, i, i, i);
  if (smem_raw[threadIdx.x] == 0xff) dst[0] = make_uint4(0, 0, 0, 0);   // keeps the dynamic shared memory referenced
  __syncthreads();
  if (threadIdx.x == 0) atomicMax(stamps, (unsigned long long)ptx::globaltimer_ns());
  if (use_tmem) {
    ptx::tc_fence_before();
    __syncthreads();
    if (threadIdx.x < 32) {
      ptx::tc_fence_after();
      ptx::tmem_dealloc(tmem_base, 256);
    }
  }
}
__global__ void __launch_bounds__(320, 1) handover_second_kernel(unsigned long long* stamps, int smem_dummy) {
  extern __shared__ uint8_t smem_raw[];
  (void)smem_dummy;
  allow_dependents();
  dependency_wait();
  if (threadIdx.x == 0) atomicMin(stamps + 1, (unsigned long long)ptx::globaltimer_ns());
  if (smem_raw[threadIdx.x] == 0xff) stamps[2] = 1;
}
}  // namespace lq

// Launches first + second `pairs` times back to back; after each pair the host reads nothing - the caller reads
// stamps[0..1] after synchronising (they hold the LAST pair's values only if it resets them between pairs, so
// the Python side launches one pair at a time after a warm-up).  smem_bytes: dynamic shared memory per CTA of
// both kernels (occupancy: with more than half of the SM's shared memory the second kernel's CTAs cannot be
// resident beside the first's).
extern "C" LQ_API int lq_debug_handover(int use_tmem, int out_bytes_per_cta, int smem_bytes, int ctas, void* out,
                                        unsigned long long* stamps, void* stream) {
  if (ctas <= 0 || out_bytes_per_cta % 16 || smem_bytes < 512 || smem_bytes > 200 * 1024 || !out || !stamps)
    return LQ_ERR_BAD_ARG;
  cudaStream_t st = lq::as_stream(stream);
  cudaFuncSetAttribute(lq::handover_first_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 201 * 1024);
  cudaFuncSetAttribute(lq::handover_second_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 201 * 1024);
  cudaError_t e = lq::launch_overlapped(lq::handover_first_kernel, dim3(ctas), dim3(320), (size_t)smem_bytes, st, use_tmem,
                                        out_bytes_per_cta, static_cast<uint8_t*>(out), stamps, 0);
  if (e != cudaSuccess) return LQ_ERR_CUDA;
  e = lq::launch_overlapped(lq::handover_second_kernel, dim3(ctas), dim3(320), (size_t)smem_bytes, st, stamps, 0);
  if (e != cudaSuccess) return LQ_ERR_CUDA;
  return lq::check_launch("handover kernels");
}
