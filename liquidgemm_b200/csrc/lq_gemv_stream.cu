// Decode GEMV (M <= 16) as a persistent weight-streaming kernel.
//
// The tensor-core GEMM is a poor fit for a handful of tokens: every tcgen05.mma costs about a
// hundred cycles of issue whatever its N, which caps weight streaming below HBM speed.  Here the
// weights stay on the CUDA-core / warp-level tensor path instead, and the structure is built
// around what a microsecond-scale bandwidth-bound kernel needs:
//   * one CTA per SM; the (row-block, k-stage) units of the whole matrix are dealt out in equal
//     contiguous ranges (stream-K), so every SM pulls the same number of bytes;
//   * a producer warp keeps a ring of NS stages full with TMA: a 128-row x 128-byte box of the
//     row-major interleaved nibble pack (256 k, 16 KB) and two token boxes per stage, all with
//     the 128-byte swizzle;
//   * eight consumer warps own 16 rows each.  A lane (g = lane/4, q = lane%4) reads the 32 codes
//     k = 32q..32q+31 of rows g and g+8 for each 128-k half (conflict-free 16-byte loads),
//     reconstructs INT8 with AND / SHR+AND, multiply-add, XOR and accumulates with dp4a against the
//     matching 32 bytes of every token (broadcast shared loads).  On this GPU the warp-level
//     mma.sync INT8 path measured ~130 cycles per m16n8k32, far slower than dp4a, so it is not
//     used.  Sums stay in registers for the whole k-range of a row block and the four lanes that
//     share a row are combined with two shuffles per value at the end;
//   * a k-range that covers the block's whole K is scaled and stored directly; otherwise the
//     partial int32 sums are added into a workspace slot and the CTA that completes the block
//     finishes it and re-zeroes the slot (same protocol as the tensor-core GEMM).
// All waits are bounded and report through the status word.
#include <cuda.h>

#include <mutex>

#include "lq_common.cuh"
#include "lq_tc_ptx.cuh"
#include "lq_sched.cuh"

namespace lq {

int make_byte_matrix_map(CUtensorMap* map, const void* ptr, long rows, long row_bytes, int box_rows,
                         int box_bytes);  // lq_gemm_tc.cu

constexpr int kGsThreads = 288;          // warp 0 producer, warps 1..8 consumers
constexpr int kGsWStage = 16384;         // 128 rows x 128 bytes of nibbles = 256 k
constexpr uint64_t kGsWaitNs = 2000000000ull;

struct GemvArgs {
  const uint8_t* s_u8;    // [N, K/64]
  const uint8_t* off_a;   // [N, K/64]
  const float* ascale;    // [M]
  const float* s1;        // [N]
  void* out;              // [M, N]
  int32_t* slots;         // [grid][16][128] int32 partial sums, all zero between launches
  int32_t* counters;      // [grid]
  int* status;
  int out_dtype;
  int M, N, K;
  SchedArgs sched;        // kt_total = stages of 256 k per row block
};

__device__ __forceinline__ void consumer_barrier() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

// MT: tokens held in registers (>= M; 1, 2, 4, 8 or 16).  NS: ring stages.
template <int MT, int NS>
__global__ void __launch_bounds__(kGsThreads, 1)
gemv_stream_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                   const GemvArgs args) {
  constexpr int TS = MT > 8 ? 2 : 1;
  constexpr int kXBox = TS * 8 * 128;                 // one token box: 8 or 16 rows x 128 bytes
  constexpr int kStage = kGsWStage + 2 * kXBox;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw_addr);
  const uint32_t bars = base + NS * kStage;
  const uint32_t bar_full = bars, bar_empty = bars + NS * 8;
  volatile int* flags = reinterpret_cast<volatile int*>(smem + NS * kStage + 2 * NS * 8);   // [0] last, [1..2] ok

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < NS; ++s) {
      ptx::mbar_init(bar_full + 8 * s, 1);
      ptx::mbar_init(bar_empty + 8 * s, 256);
    }
    ptx::fence_mbar_init();
    ptx::prefetch_tensormap(&tmap_w);
    ptx::prefetch_tensormap(&tmap_x);
  }
  __syncthreads();

  const int kt_total = args.sched.kt_total;
  if (warp == 0) {
    // ------------------------------------------------------------------ producer (whole warp walks, lane 0 issues)
    SegmentWalk walk(args.sched, blockIdx.x, gridDim.x);
    Segment sg;
    Ring<NS> ring;
    int issued = 0;
    bool ok = true;
    while (ok && walk.next(sg)) {
      for (int kt = sg.kb; kt < sg.ke; ++kt) {
        if (!ptx::mbar_wait_bounded(bar_empty + 8 * ring.s, ring.ph ^ 1u, kGsWaitNs)) {
          atomicExch(args.status, 201);
          ok = false;
          break;
        }
        if (lane == 0) {
          const uint32_t full = bar_full + 8 * ring.s;
          const uint32_t st = base + ring.s * kStage;
          ptx::mbar_expect_tx(full, kStage);
          ptx::tensor_load_2d(st, &tmap_w, kt * 128, sg.tile * 128, full);
          ptx::tensor_load_2d(st + kGsWStage, &tmap_x, kt * 256, 0, full);
          ptx::tensor_load_2d(st + kGsWStage + kXBox, &tmap_x, kt * 256 + 128, 0, full);
        }
        ring.advance();
        ++issued;
      }
    }
    if (!ok) {
      Ring<NS> back;
      const int first = issued > NS ? issued - NS : 0;
      for (int i = 0; i < issued; ++i) {
        if (i >= first) ptx::mbar_wait_bounded(bar_full + 8 * back.s, back.ph, kGsWaitNs);
        back.advance();
      }
    }
  } else {
    // ------------------------------------------------------------------ consumers
    const int cw = warp - 1;                   // 0..7: rows 16 cw .. 16 cw + 15 of the block
    const int g = lane >> 2, q = lane & 3;
    const int rA = cw * 16 + g, rB = rA + 8;   // rows inside the 128-row block
    const int ct = threadIdx.x - 32;           // 0..255 inside the consumer group
    const int G = args.K >> 6;
    const int k_groups_total = G;
    SegmentWalk walk(args.sched, blockIdx.x, gridDim.x);
    Segment sg;
    Ring<NS> ring;
    bool ok = true;
    int seg = 0;
    while (ok && walk.next(sg)) {
      const long nA = (long)sg.tile * 128 + rA, nB = nA + 8;
      const bool okA = nA < args.N, okB = nB < args.N;
      const uint8_t* sA = args.s_u8 + (okA ? nA : 0) * G;
      const uint8_t* sB = args.s_u8 + (okB ? nB : 0) * G;
      const uint8_t* oA = args.off_a + (okA ? nA : 0) * G;
      const uint8_t* oB = args.off_a + (okB ? nB : 0) * G;
      int accA[MT], accB[MT];
#pragma unroll
      for (int m = 0; m < MT; ++m) accA[m] = accB[m] = 0;

      for (int kt = sg.kb; kt < sg.ke; ++kt) {
        // (step, offset) of this lane's two rows for both 128-k halves: fetched before the wait
        uint32_t stp[2][2], abc[2][2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int grp = 4 * kt + 2 * h + (q >> 1);
          const bool in_k = grp < k_groups_total;
          stp[h][0] = (okA && in_k) ? __ldg(sA + grp) : 0u;
          stp[h][1] = (okB && in_k) ? __ldg(sB + grp) : 0u;
          abc[h][0] = ((okA && in_k) ? (uint32_t)__ldg(oA + grp) : 128u) * 0x01010101u;
          abc[h][1] = ((okB && in_k) ? (uint32_t)__ldg(oB + grp) : 128u) * 0x01010101u;
        }
        if (!ptx::mbar_wait_bounded(bar_full + 8 * ring.s, ring.ph, kGsWaitNs)) {
          atomicExch(args.status, 202);
          ok = false;
          break;
        }
        const uint8_t* st = smem + ring.s * kStage;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int c = 4 * h + q;               // 16-byte chunk of the 128-byte row
          const uint4 wa = *reinterpret_cast<const uint4*>(st + rA * 128 + ((c ^ (rA & 7)) << 4));
          const uint4 wb = *reinterpret_cast<const uint4*>(st + rB * 128 + ((c ^ (rB & 7)) << 4));
          const uint32_t pa[4] = {wa.x, wa.y, wa.z, wa.w};
          const uint32_t pb[4] = {wb.x, wb.y, wb.z, wb.w};
          int qa[8], qb[8];                      // word 2j: k = 8j..8j+3, word 2j+1: k = 8j+4..8j+7
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            qa[2 * j] = (int)lqq_dequant4(pa[j] & 0x0F0F0F0Fu, stp[h][0], abc[h][0]);
            qa[2 * j + 1] = (int)lqq_dequant4((pa[j] >> 4) & 0x0F0F0F0Fu, stp[h][0], abc[h][0]);
            qb[2 * j] = (int)lqq_dequant4(pb[j] & 0x0F0F0F0Fu, stp[h][1], abc[h][1]);
            qb[2 * j + 1] = (int)lqq_dequant4((pb[j] >> 4) & 0x0F0F0F0Fu, stp[h][1], abc[h][1]);
          }
#pragma unroll
          for (int m = 0; m < MT; ++m) {
            const uint8_t* xb = st + kGsWStage + h * kXBox + m * 128;
            const int4 x0 = *reinterpret_cast<const int4*>(xb + (((2 * q) ^ (m & 7)) << 4));
            const int4 x1 = *reinterpret_cast<const int4*>(xb + (((2 * q + 1) ^ (m & 7)) << 4));
            const int xs[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
            int a = accA[m], b2 = accB[m];
#pragma unroll
            for (int w = 0; w < 8; ++w) {
              a = __dp4a(xs[w], qa[w], a);
              b2 = __dp4a(xs[w], qb[w], b2);
            }
            accA[m] = a;
            accB[m] = b2;
          }
        }
        ptx::mbar_arrive(bar_empty + 8 * ring.s);   // every shared load of the stage was issued above
        ring.advance();
      }
      if (!ok) break;

      // ---- combine the four lanes (q = 0..3) that share rows rA / rB; lane q then owns tokens m = q mod 4
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        accA[m] += __shfl_xor_sync(0xffffffffu, accA[m], 1);
        accA[m] += __shfl_xor_sync(0xffffffffu, accA[m], 2);
        accB[m] += __shfl_xor_sync(0xffffffffu, accB[m], 1);
        accB[m] += __shfl_xor_sync(0xffffffffu, accB[m], 2);
      }
      if (sg.whole) {
        const float wsA = okA ? __ldg(args.s1 + nA) : 0.f, wsB = okB ? __ldg(args.s1 + nB) : 0.f;
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          if ((m & 3) == q && m < args.M) {
            const float as = __ldg(args.ascale + m);
            if (okA) store_out(args.out, (size_t)m * args.N + nA, lqq_scale(accA[m], as, wsA), args.out_dtype);
            if (okB) store_out(args.out, (size_t)m * args.N + nB, lqq_scale(accB[m], as, wsB), args.out_dtype);
          }
        }
      } else {
        int32_t* slot = args.slots + (size_t)sg.slot * (128 * 16);
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          if ((m & 3) == q && m < args.M) {
            atomicAdd(slot + m * 128 + rA, accA[m]);
            atomicAdd(slot + m * 128 + rB, accB[m]);
          }
        }
        __threadfence();
        consumer_barrier();
        if (ct == 0) {
          const int add = sg.ke - sg.kb;
          const int before = atomicAdd(args.counters + sg.slot, add);
          flags[0] = (before + add == kt_total) ? 1 : 0;
        }
        consumer_barrier();
        const bool last = flags[0] != 0;
        consumer_barrier();
        if (last) {
          __threadfence();
          // 256 threads, 128 rows: thread ct finishes row (ct & 127) for tokens of parity (ct >> 7)
          const int r = ct & 127;
          const long n = (long)sg.tile * 128 + r;
          if (n < args.N) {
            const float ws = __ldg(args.s1 + n);
            for (int m = ct >> 7; m < args.M; m += 2) {
              int32_t* p = slot + m * 128 + r;
              const int v = __ldcg(p);
              __stcg(p, 0);
              store_out(args.out, (size_t)m * args.N + n, lqq_scale(v, __ldg(args.ascale + m), ws), args.out_dtype);
            }
          } else {
            for (int m = ct >> 7; m < args.M; m += 2) __stcg(slot + m * 128 + r, 0);
          }
          if (ct == 0) args.counters[sg.slot] = 0;
        }
      }
      ++seg;
    }
  }
  __syncthreads();
}

template <int MT, int NS>
static int launch_stream(const CUtensorMap& tw, const CUtensorMap& tx, const GemvArgs& a, int grid, cudaStream_t st) {
  constexpr int TS = MT > 8 ? 2 : 1;
  constexpr int smem = 1024 + NS * (kGsWStage + 2 * TS * 8 * 128) + 2 * NS * 8 + 64;
  static_assert(smem <= 232448 && smem > 116 * 1024, "ring must fill most of the SM so that one CTA is resident");
  auto kern = &gemv_stream_kernel<MT, NS>;
  static std::once_flag once[64];
  int dev = 0;
  cudaGetDevice(&dev);
  cudaError_t e = cudaSuccess;
  std::call_once(once[dev & 63], [&]() { e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); });
  if (e != cudaSuccess) {
    record_cuda_error(e, "cudaFuncSetAttribute(gemv_stream_kernel)");
    return LQ_ERR_CUDA;
  }
  kern<<<grid, kGsThreads, smem, st>>>(tw, tx, a);
  return check_launch("gemv_stream_kernel");
}

static int stream_grid(int N, int K, int* kt_out, int* tiles_out) {
  const int kt = (K + 255) / 256, tiles = (N + 127) / 128;
  const long units = (long)kt * tiles;
  const int sms = sm_count();
  *kt_out = kt;
  *tiles_out = tiles;
  return (int)(units < sms ? units : sms);
}

}  // namespace lq

using namespace lq;

extern "C" {

size_t lq_gemv_workspace_bytes(int N, int K) {
  if (N <= 0 || K < 128) return 0;
  int kt, tiles;
  const int grid = stream_grid(N, K, &kt, &tiles);
  return (size_t)grid * (128 * 16 * 4) + (((size_t)grid * 4 + 255) / 256) * 256;
}

int lq_w4a8_gemv_stream(const int8_t* x_i8, const uint8_t* gpack, const uint8_t* s_u8, const uint8_t* offset_a,
                        const float* ascale, const float* s1, void* y, int out_dtype, int M, int N, int K,
                        void* workspace, size_t workspace_bytes, void* stream) {
  if (!x_i8 || !gpack || !s_u8 || !offset_a || !ascale || !s1 || !y) return LQ_ERR_BAD_ARG;
  if (M < 0 || N <= 0 || K <= 0 || out_dtype < 0 || out_dtype > 2) return LQ_ERR_BAD_ARG;
  if (M > 16 || K % 128) return LQ_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(x_i8) | reinterpret_cast<uintptr_t>(gpack)) % 16) return LQ_ERR_BAD_ARG;
  if (M == 0) return LQ_OK;
  if (!workspace || workspace_bytes < lq_gemv_workspace_bytes(N, K)) return LQ_ERR_WORKSPACE;
  int kt, tiles;
  const int grid = stream_grid(N, K, &kt, &tiles);
  const int ts = M <= 8 ? 1 : 2;
  CUtensorMap tw, tx;
  int rc = make_byte_matrix_map(&tw, gpack, N, K / 2, 128, 128);
  if (rc) return rc;
  rc = make_byte_matrix_map(&tx, x_i8, M, K, 8 * ts, 128);
  if (rc) return rc;
  GemvArgs a;
  a.s_u8 = s_u8;
  a.off_a = offset_a;
  a.ascale = ascale;
  a.s1 = s1;
  a.out = y;
  a.slots = static_cast<int32_t*>(workspace);
  a.counters = reinterpret_cast<int32_t*>(static_cast<uint8_t*>(workspace) + (size_t)grid * (128 * 16 * 4));
  a.status = status_word();
  a.out_dtype = out_dtype;
  a.M = M;
  a.N = N;
  a.K = K;
  a.sched = SchedArgs{kt, tiles, 1, 0};
  if (!a.status) return LQ_ERR_CUDA;
  cudaStream_t st = as_stream(stream);
  if (M <= 1) return launch_stream<1, 10>(tw, tx, a, grid, st);
  if (M <= 2) return launch_stream<2, 10>(tw, tx, a, grid, st);
  if (M <= 4) return launch_stream<4, 10>(tw, tx, a, grid, st);
  if (M <= 8) return launch_stream<8, 10>(tw, tx, a, grid, st);
  return launch_stream<16, 9>(tw, tx, a, grid, st);
}

}  // extern "C"
