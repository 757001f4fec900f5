// INT8 x INT8 GEMM for large token counts on CTA pairs: C[M,N] = A[M,K] * B[N,K]^T with int32 sums, optionally
// scaled by a per-row and a per-column factor (the reference's CUTLASS INT8 GEMM, csrc/liquid_gemm/wgmma_i8_gemm.cu,
// which its vLLM plugin uses when the weights stay INT8: liquidgemm/vllm_plugin.py:160-176).
//
// Nothing is unpacked here, so both operands go from global memory to shared memory by TMA and from there to the
// tensor cores: one tcgen05.mma.cta_group::2 covers 256 output channels (128 from the shared memory of each CTA of
// the pair) x 256 tokens (128 rows staged by each CTA) x 32 of k; the 256 x 256 int32 tile lives in the tensor
// memory of both CTAs, two accumulators of 256 columns each, so that the epilogue of a tile overlaps the main
// loop of the next.  No load uses cluster multicast.
//
// Per CTA (640 threads), connected by mbarrier rings; rank = CTA's rank in its pair:
//   warp 0        weight producer: 128 channels x 128 bytes of k per k-step (rows 256 * block + 128 * rank ...)
//   warp 2        token producer: 128 token rows x 128 bytes of k per k-step (rows 256 * tile + 128 * rank ...)
//   warp 3        relay: when both copies of a stage have landed HERE it tells the leader CTA (whose MMA reads the
//                 shared memory of both CTAs); one arrival per CTA and stage
//   warp 1        tensor-memory allocation (both CTAs); on rank 0 the MMA issue: four MMAs per k-step, then one
//                 commit that frees the stage in both CTAs
//   warps 4..19   four epilogue groups sharing every tile (16-token chunks g, g + 4, ...)
// Work: tile = 256 channels x 256 tokens, pair p of P takes tiles p, p + P, ... whole (the INT8 entry points take
// no workspace).  Every wait is bounded; the status codes are 141-146.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <mutex>
#include <type_traits>

#include "lq_common.cuh"
#include "lq_pair_common.cuh"
#include "lq_sched.cuh"
#include "lq_tc_ptx.cuh"

namespace lq {

int make_byte_matrix_map(CUtensorMap* map, const void* ptr, long rows, long row_bytes, int box_rows, int box_bytes);   // lq_gemm_tc.cu

namespace i8pair {

using namespace pairc;

constexpr int kBN = 256;                 // tokens per tile
constexpr int kHalf = kBN / 2;           // token rows staged by each CTA
constexpr int kNS = 6;                   // shared-memory stages
constexpr int kGroups = 4;               // epilogue groups of four warps
constexpr int kThreads = 128 + 128 * kGroups;
constexpr int kAStage = 128 * 128;       // 128 channels x 128 bytes of k
constexpr int kXStage = kHalf * 128;
constexpr int kTmemCols = 512;           // two 256-column accumulators
constexpr int kNumBars = 3 * kNS + 4;
constexpr int kBarBytes = kNumBars * 8 + 64;
constexpr int kSmemBytes = 1024 /* alignment slack */ + kNS * (kAStage + kXStage) + ((kBarBytes + 15) & ~15) +
                           kGroups * 2 * kBN * 4;
constexpr uint64_t kWaitLimitNs = 2000000000ull;
constexpr int kOutI32 = kEpiI32;

struct Args {
  const float* ascale;     // [M] or null (raw int32)
  const float* s1;         // [N] or null
  const void* bias;        // [N] in the output dtype, or null
  void* out;               // [M, N]
  int* status;
  int out_mode;            // LQ_DT_* or kOutI32
  int M, N, K;
  int kt_total;            // K / 128
  int n2_tiles, m_tiles;   // 256-channel blocks, 256-token blocks
  int pairs;               // CTA pairs of the launch
  int tail_s;              // always 1: whole tiles
};

__device__ __forceinline__ void group_bar(int g) { asm volatile("bar.sync %0, 128;" ::"r"(g + 1) : "memory"); }

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
i8_pair_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w, const Args args) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw_addr);

  const uint32_t xs = base;                                  // kNS token stages (1024-aligned, 128-byte swizzle)
  const uint32_t as = xs + kNS * kXStage;                    // kNS weight stages
  const uint32_t bars = as + kNS * kAStage;
  const uint32_t bar_full = bars;                            // [kNS] both copies of the stage landed (this CTA)
  const uint32_t bar_empty = bar_full + kNS * 8;             // [kNS] the MMAs that read the stage are done
  const uint32_t bar_ready = bar_empty + kNS * 8;            // [kNS] used on rank 0: the stage landed in both CTAs
  const uint32_t bar_accfull = bar_ready + kNS * 8;          // [2] accumulator final
  const uint32_t bar_accfree = bar_accfull + 2 * 8;          // [2] accumulator drained; used on rank 0
  const uint32_t tmem_slot = bar_accfree + 2 * 8;
  uint8_t* gen_bars = smem + (bars - base);
  volatile uint32_t* tmem_slot_p = reinterpret_cast<volatile uint32_t*>(gen_bars + kNumBars * 8);
  volatile int* wait_flag = reinterpret_cast<volatile int*>(gen_bars + kNumBars * 8 + 8);   // [group][2]
  float* tok_scale = reinterpret_cast<float*>(gen_bars + ((kBarBytes + 15) & ~15));          // [group][2][kBN]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = ptx::cluster_ctarank();
  const int pair = (int)ptx::cluster_id_x();

  if (threadIdx.x == 0) {
    for (int s = 0; s < kNS; ++s) {
      ptx::mbar_init(bar_full + 8 * s, 2);       // one expect_tx arrival per producer
      ptx::mbar_init(bar_empty + 8 * s, 1);      // the MMA thread's commit
      ptx::mbar_init(bar_ready + 8 * s, 2);      // one relay arrival per CTA
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(bar_accfull + 8 * b, 1);
      ptx::mbar_init(bar_accfree + 8 * b, 2 * 4 * kGroups);   // one arrival per epilogue warp, both CTAs
    }
    ptx::fence_mbar_init();
    ptx::prefetch_tensormap(&tmap_x);
    ptx::prefetch_tensormap(&tmap_w);
  }
  if (warp == 1) {
    ptx::tmem_alloc_pair(tmem_slot, kTmemCols);
    ptx::tmem_relinquish_pair();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync_all();   // the barriers of both CTAs exist before anything arrives on them from the peer
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_p;
  const uint32_t leader_ready = ptx::map_to_cta(bar_ready, 0);
  const uint32_t leader_accfree = ptx::map_to_cta(bar_accfree, 0);

  if (warp == 0 || warp == 2) {
    // ------------------------------------------------------------------ producers (one thread each)
    if (lane == 0) {
      const bool weights = (warp == 0);
      PairWalk walk(args, pair);
      Segment sg;
      Ring<kNS> ring;
      int issued = 0;
      bool ok = true;
      while (ok && walk.next(sg)) {
        int n2, mt;
        tile_coords(sg.tile, args.n2_tiles, args.m_tiles, kGroupM, n2, mt);
        const int row0 = weights ? (2 * n2 + (int)rank) * 128 : mt * kBN + (int)rank * kHalf;
        for (int kt = sg.kb; kt < sg.ke; ++kt) {
          if (!ptx::mbar_wait_bounded(bar_empty + 8 * ring.s, ring.ph ^ 1u, kWaitLimitNs)) {
            atomicExch(args.status, 141);
            ok = false;
            break;
          }
          const uint32_t full = bar_full + 8 * ring.s;
          if (weights) {
            ptx::mbar_expect_tx(full, kAStage);
            ptx::tensor_load_2d(as + ring.s * kAStage, &tmap_w, kt * 128, row0, full);
          } else {
            ptx::mbar_expect_tx(full, kXStage);
            ptx::tensor_load_2d(xs + ring.s * kXStage, &tmap_x, kt * 128, row0, full);
          }
          ring.advance();
          ++issued;
        }
      }
      if (!ok) {
        // copies already issued still write shared memory: let them land before the CTA exits
        Ring<kNS> back;
        const int first = issued > kNS ? issued - kNS : 0;
        for (int i = 0; i < issued; ++i) {
          if (i >= first) ptx::mbar_wait_bounded(bar_full + 8 * back.s, back.ph, kWaitLimitNs);
          back.advance();
        }
      }
    }
  } else if (warp == 3) {
    // ------------------------------------------------------------------ relay (one thread)
    if (lane == 0) {
      PairWalk walk(args, pair);
      Segment sg;
      Ring<kNS> ring;
      bool ok = true;
      while (ok && walk.next(sg)) {
        for (int kt = sg.kb; kt < sg.ke; ++kt) {
          if (!ptx::mbar_wait_bounded(bar_full + 8 * ring.s, ring.ph, kWaitLimitNs)) {
            atomicExch(args.status, 142);
            ok = false;
            break;
          }
          if (rank == 0) ptx::mbar_arrive(bar_ready + 8 * ring.s);
          else ptx::mbar_arrive_remote(leader_ready + 8 * ring.s);
          ring.advance();
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issue (leader CTA)
    // The whole warp walks the loop; one elected lane issues (see ptx::elect_one).
    if (rank == 0) {
      const bool leader = ptx::elect_one();
      constexpr uint32_t idesc = ptx::idesc_i8_pair(kBN);
      PairWalk walk(args, pair);
      Segment sg;
      Ring<kNS> ring;
      Ring<2> accring;
      bool ok = true;
      while (ok && walk.next(sg)) {
        if (!ptx::mbar_wait_bounded(bar_accfree + 8 * accring.s, accring.ph ^ 1u, kWaitLimitNs)) {
          if (leader) atomicExch(args.status, 143);
          ok = false;
        }
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        ptx::tc_fence_after();
        const uint32_t tmem_acc = tmem_base + accring.s * kBN;
        for (int kt = sg.kb; kt < sg.ke; ++kt) {
          if (!ptx::mbar_wait_bounded(bar_ready + 8 * ring.s, ring.ph, kWaitLimitNs)) {
            if (leader) atomicExch(args.status, 144);
            ok = false;
          }
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          ptx::tc_fence_after();
          const uint32_t xb = xs + ring.s * kXStage;
          const uint32_t ab = as + ring.s * kAStage;
          if (leader) {
#pragma unroll
            for (int j = 0; j < 4; ++j)
              ptx::mma_i8_ss_pair(tmem_acc, ptx::smem_desc_sw128(ab + j * 32), ptx::smem_desc_sw128(xb + j * 32), idesc,
                                  (kt > sg.kb || j > 0) ? 1u : 0u);
            ptx::tc_commit_pair(bar_empty + 8 * ring.s);
          }
          ring.advance();
        }
        if (ok && leader) ptx::tc_commit_pair(bar_accfull + 8 * accring.s);
        accring.advance();
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 4..19, four groups)
    const int g = (warp - 4) >> 2;
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
    const int et = (threadIdx.x & 127);        // 0..127 inside the group (the groups start at multiples of 128)
    const bool raw = args.out_mode == kOutI32;
    const bool has_bias = !raw && args.bias != nullptr;
    volatile int* wflag = wait_flag + 2 * g;
    PairWalk walk(args, pair);
    Segment sg;
    Ring<2> accring;
    int seg = 0;
    bool ok = true;
    while (ok && walk.next(sg)) {
      const int b = accring.s;
      const uint32_t phb = accring.ph;
      accring.advance();
      // One thread of the group performs the bounded wait and publishes the outcome, so that its 128 threads
      // always agree on it (they meet at a named barrier and must never split up).
      const int fslot = seg & 1;
      ++seg;
      if (et == 0) {
        const bool done = ptx::mbar_wait_bounded(bar_accfull + 8 * b, phb, kWaitLimitNs);
        if (!done) atomicExch(args.status, 145);
        wflag[fslot] = done ? 1 : 0;
      }
      int n2, mt;
      tile_coords(sg.tile, args.n2_tiles, args.m_tiles, kGroupM, n2, mt);
      const int m0 = mt * kBN;
      const long n = (long)(2 * n2 + (int)rank) * 128 + row;
      const int cols = (args.M - m0) < kBN ? (args.M - m0) : kBN;   // valid token columns of this tile
      float* tsc = tok_scale + (2 * g + fslot) * kBN;
      if (!raw) {
        for (int i = et; i < kBN; i += 128) tsc[i] = (i < cols) ? __ldg(args.ascale + m0 + i) : 0.f;
      }
      group_bar(g);
      if (wflag[fslot] == 0) {
        ok = false;
        break;
      }
      ptx::tc_fence_after();
      const uint32_t tmem_acc = tmem_base + b * kBN + lane_addr;
      const float w_scale = raw ? 0.f : __ldg(args.s1 + n);
      const float bias = has_bias ? load_bias(args.bias, n, args.out_mode) : 0.f;
#pragma unroll 1
      for (int c0 = 16 * g; c0 < cols; c0 += 16 * kGroups) {
        int v[16];
        ptx::tmem_ld16(tmem_acc + c0, v);
        float sc[16];
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const float4 f = *reinterpret_cast<const float4*>(tsc + c0 + 4 * q4);
          sc[4 * q4] = f.x; sc[4 * q4 + 1] = f.y; sc[4 * q4 + 2] = f.z; sc[4 * q4 + 3] = f.w;
        }
        ptx::tc_wait_ld();
        // lane = channel: a warp's store covers 32 consecutive channels of one token row
        epi_store_cols(args.out, args.out_mode, (size_t)(m0 + c0) * args.N + n, args.N, v, sc, w_scale, bias, has_bias,
                       cols - c0);
      }
      // this warp's reads of the accumulator are complete: the MMA warp may reuse it
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (rank == 0) ptx::mbar_arrive(bar_accfree + 8 * b);
        else ptx::mbar_arrive_remote(leader_accfree + 8 * b);
      }
    }
  }

  // Both CTAs are done with each other's shared and tensor memory before either releases anything.
  __syncwarp();
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync_all();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

static int max_pairs() {
  static int cached[64] = {};
  static std::mutex mu;
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> lock(mu);
  int& v = cached[dev & 63];
  if (v == 0) {
    v = sm_count() / 2;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * v);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = kSmemBytes;
    int clusters = 0;
    cudaFuncSetAttribute(i8_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (cudaOccupancyMaxActiveClusters(&clusters, i8_pair_kernel, &cfg) == cudaSuccess && clusters > 0 && clusters < v)
      v = clusters;
    cudaGetLastError();
    if (v < 1) v = 1;
  }
  return v;
}

}  // namespace i8pair

// Shapes the INT8 pair kernel takes: whole 256-channel blocks and at least 60 tiles of 256 x 256 for the 74 pairs.
// Measured against the one-CTA persistent kernel on the Llama-3.1-8B shapes at 128..4096 tokens: from 64 tiles
// up it is 1.3-1.6x faster (and within 2 % of cuBLASLt's INT8 GEMM at every point), at 96 tiles level, with
// 16-48 tiles 0-4 % slower.
bool i8_pair_serves(int M, int N, int K) {
  if (M < 256 || N < 256 || N % 256 || K < 128 || K % 128) return false;
  const long tiles = (long)(N / 256) * ((M + i8pair::kBN - 1) / i8pair::kBN);
  return tiles >= 60;
}

int run_i8_pair_gemm(const int8_t* x, const int8_t* w, const float* ascale, const float* s1, const void* bias, void* out,
                     int out_mode, int M, int N, int K, cudaStream_t st) {
  using namespace i8pair;
  if (out_mode < 0 || out_mode > kOutI32) return LQ_ERR_BAD_ARG;
  CUtensorMap tx, tw;
  if (int rc = make_byte_matrix_map(&tx, x, M, K, kHalf, 128)) return rc;
  if (int rc = make_byte_matrix_map(&tw, w, N, K, 128, 128)) return rc;
  Args a;
  a.ascale = ascale;
  a.s1 = s1;
  a.bias = bias;
  a.out = out;
  a.status = status_word();
  a.out_mode = out_mode;
  a.M = M;
  a.N = N;
  a.K = K;
  a.kt_total = K / 128;
  a.n2_tiles = N / 256;
  a.m_tiles = (M + kBN - 1) / kBN;
  const long tiles = (long)a.n2_tiles * a.m_tiles;
  const int cap = max_pairs();
  a.pairs = (int)(tiles < cap ? tiles : cap);
  a.tail_s = 1;
  if (!a.status) return LQ_ERR_CUDA;
  static std::once_flag once[64];
  int dev = 0;
  cudaGetDevice(&dev);
  cudaError_t attr_err = cudaSuccess;
  std::call_once(once[dev & 63], [&]() {
    attr_err = cudaFuncSetAttribute(i8_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
  });
  if (attr_err != cudaSuccess) {
    record_cuda_error(attr_err, "cudaFuncSetAttribute(i8_pair_kernel)");
    return LQ_ERR_CUDA;
  }
  i8_pair_kernel<<<2 * a.pairs, kThreads, kSmemBytes, st>>>(tx, tw, a);
  return check_launch("i8_pair_kernel");
}

}  // namespace lq
