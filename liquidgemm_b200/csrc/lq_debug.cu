// Measurement-only kernels (no product path calls them): the issue/execute rate of
// tcgen05.mma kind::i8 for a given N, with the A operand in tensor memory or in shared memory.
#include "lq_common.cuh"
#include "lq_tc_ptx.cuh"

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
  for (int i = threadIdx.x; i < (32768 + 16384) / 4; i += blockDim.x)
    reinterpret_cast<uint32_t*>(smem_raw + (base - raw_addr))[i] = 0x01020304u * (i + 1);
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  if (threadIdx.x < 32) {
    ptx::tmem_alloc(smem_u32(&tmem_slot), 512);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  if (threadIdx.x == 0) {
    const uint32_t idesc = ptx::idesc_i8(n);
    const long long t0 = clock64();
    for (int i = 0; i < iters; ++i) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint64_t bdesc = ptx::smem_desc_sw128(base + j * 32);
        if (a_in_tmem) ptx::mma_i8_ts(tmem_base, tmem_base + 256 + j * 8, bdesc, idesc, 1u);
        else ptx::mma_i8_ss(tmem_base, ptx::smem_desc_sw128(base + 32768 + j * 32), bdesc, idesc, 1u);
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
    ptx::tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace lq

// out: device buffer of 2 x ctas int64: total cycles and cycles spent issuing, per CTA.
extern "C" LQ_API int lq_debug_mma_rate(int n, int iters, int a_in_tmem, int ctas, long long* out, void* stream) {
  if (n < 16 || n > 256 || n % 16 || iters <= 0 || ctas <= 0 || !out) return LQ_ERR_BAD_ARG;
  const int smem = 1024 + 32768 + 16384;
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
      while (!ptx::mbar_try_wait(b2, (uint32_t)i & 1u)) {}
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
    while (!ptx::mbar_try_wait(b2, 0u)) {}
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
tma_stream_kernel(const uint8_t* src, int stage_bytes, int ns, int steps, long long* cycles) {
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
  const uint8_t* my = src + (size_t)blockIdx.x * steps * stage_bytes;
  if (threadIdx.x == 0) {
    int s = 0;
    uint32_t ph = 0;
    for (int i = 0; i < steps; ++i) {
      while (!ptx::mbar_try_wait(smem_u32(&bars[32 + s]), ph ^ 1u)) {}
      ptx::mbar_expect_tx(smem_u32(&bars[s]), stage_bytes);
      ptx::bulk_load(base + s * stage_bytes, my + (size_t)i * stage_bytes, stage_bytes, smem_u32(&bars[s]));
      if (++s == ns) { s = 0; ph ^= 1u; }
    }
  } else if (threadIdx.x == 32) {
    int s = 0;
    uint32_t ph = 0;
    for (int i = 0; i < steps; ++i) {
      while (!ptx::mbar_try_wait(smem_u32(&bars[s]), ph)) {}
      ptx::mbar_arrive(smem_u32(&bars[32 + s]));
      if (++s == ns) { s = 0; ph ^= 1u; }
    }
    cycles[blockIdx.x] = clock64() - t0;
  }
  __syncthreads();
}
}  // namespace lq

extern "C" LQ_API int lq_debug_tma_stream(const void* src, int stage_bytes, int ns, int steps, int ctas,
                                          long long* cycles, void* stream) {
  if (ns < 1 || ns > 32 || stage_bytes % 16 || stage_bytes * ns > 200 * 1024) return LQ_ERR_BAD_ARG;
  const int smem = stage_bytes * ns + 256;
  cudaFuncSetAttribute(lq::tma_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 201 * 1024);
  lq::tma_stream_kernel<<<ctas, 64, smem, lq::as_stream(stream)>>>(static_cast<const uint8_t*>(src), stage_bytes, ns,
                                                                   steps, cycles);
  return lq::check_launch("tma_stream_kernel");
}
