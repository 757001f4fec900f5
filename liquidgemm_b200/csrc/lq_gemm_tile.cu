// Tile W4A8 GEMM (3 tokens and more; up to 128 tokens per tile): one 128-channel x BN-token tile per CTA, two CTAs
// per SM.  Serves decode on the large matrices (whole 16-token tiles of a 28672-channel layer stream at 0.65 of
// the HBM rate with no cross-CTA join at all), every batch from 17 tokens, and prefill where the CTA-pair kernel's
// large tiles quantise badly.
//
// The persistent stream-K kernel keeps one CTA per SM; for a handful of k-steps per CTA its
// cross-CTA reduction tail dominates.  With small token tiles the
// shared-memory and tensor-memory footprint of a tile is small enough for two CTAs per SM, whose
// load, dequant, MMA-issue and epilogue latencies overlap each other, which measured 1.5-2x
// faster in this range.  Long-K shapes are cut into `splits` k-ranges (blockIdx.z); each CTA then
// writes an int32 partial plane and one finish kernel reduces the planes and applies
// (float)acc * ascale[m] * s1[n] (the reference's design, csrc/liquid_gemm/w4a8_wgmma.cu:39-56,
// 523-534); with one split the epilogue is fused in the GEMM kernel.
//
// Per CTA: warp 0 = TMA producer (8704-byte bulk copy of the weight tile + BN x 128 token box per
// k-step), warp 1 = TMEM allocation and tcgen05.mma issue (the warp walks the loop, one elected lane issues; A
// operand from tensor memory), warps
// 2..5 and 6..9 = two dequant sets taking alternate k-steps (thread r of a set owns weight row r ->
// TMEM lane r; one set alone needs ~800 cycles per k-step, more than the MMAs of two CTAs), then
// epilogue, the sets sharing the accumulator's columns.  All waits are bounded.
#include <cuda.h>

#include <cstdlib>
#include <mutex>
#include <type_traits>

#include "lq_common.cuh"
#include "lq_tc_ptx.cuh"

namespace lq {

int launch_finish(const int32_t* acc, const float* ascale, const float* s1, const void* bias, const OutSpec& out,
                  const PeerSync* sync, int out_dtype, int planes, int M, int N, cudaStream_t st);  // lq_elementwise.cu
int make_byte_matrix_map(CUtensorMap* map, const void* ptr, long rows, long row_bytes, int box_rows,
                         int box_bytes);  // lq_gemm_tc.cu

namespace tile {

constexpr int kTileBytes = 8704;
constexpr int kI8TileBytes = 16384;
// Dequant sets of 128 threads, taking k-tiles round-robin.  Two keep up with the MMAs of two CTAs per
// SM.  A build with three (448 threads per CTA) ended its first benchmark run with an unspecified launch
// failure whose cause reading the code did not show; it is not used and must not be tried again
// without an explanation.
constexpr int kSets = 2;
constexpr int kThreads = 64 + 128 * kSets;
constexpr uint64_t kWaitLimitNs = 2000000000ull;
constexpr int kOutI32 = kEpiI32;

// Pipeline studies (-DLQ_PIPELINE_TRACE, a build of its own): %globaltimer stamps of every CTA's milestones, read
// back with lq_debug_read_tile_trace().  The product build compiles none of it.
#ifdef LQ_PIPELINE_TRACE
__device__ long long g_trace[1024 * 8];
#define TT_STAMP(slot)                                                                              \
  do {                                                                                              \
    const unsigned cta_ = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);           \
    if (cta_ < 1024u) g_trace[cta_ * 8 + (slot)] = (long long)ptx::globaltimer_ns();               \
  } while (0)
#else
#define TT_STAMP(slot) ((void)0)
#endif

struct GemmArgs {
  const uint8_t* blob;   // W4: tile blob
  const float* ascale;   // [M]
  const float* s1;       // [N]
  const void* bias;      // [N] in the output dtype, or null (fused epilogue only)
  void* out;             // scaled output [M,N] or int32 planes [splits][M][N]
  int* status;
  int out_mode;          // LQ_DT_* or kOutI32
  int M, N, K;
  int kt_total;          // K / 128
  int vec_out;           // 2-byte outputs whose rows allow 16-byte stores: stage the tile through shared memory
};

template <int BN, int NS, int NT, bool W4>
struct TcCfg {
  static constexpr int kXStage = BN * 128;
  static constexpr int kWStage = W4 ? kTileBytes : kI8TileBytes;
  static constexpr int kAccCols = BN;
  static constexpr int kACols = W4 ? 32 * NT : 0;
  static constexpr int kColsNeeded = kAccCols + kACols;
  static constexpr int kTmemCols = kColsNeeded <= 32 ? 32 : kColsNeeded <= 64 ? 64 : kColsNeeded <= 128 ? 128
                                   : kColsNeeded <= 256 ? 256 : 512;
  static constexpr int kBarBytes = (2 * NS + 2 * NT + 1) * 8 + 8;
  static constexpr int kOutStage = 16 * 128 * 2;   // per dequant set: 16 tokens x 128 channels of 2-byte outputs
  static constexpr int kSmemBytes = 1024 /* alignment slack */ + NS * (kXStage + kWStage) + kBarBytes + 16 +
                                    kSets * kOutStage;
  static_assert(kColsNeeded <= 512, "tensor memory budget exceeded");
};

template <int BN, int NS, int NT, bool W4, bool MULTI>
__global__ void __launch_bounds__(kThreads, 1)
w4a8_tile_kernel(const __grid_constant__ CUtensorMap tmap_x, const GemmArgs args,
                 const std::conditional_t<MULTI, MultiOut, NoMultiOut> multi) {
  // Only the blob-fed form exists, so the kernel takes one tensor map (the tokens).
  static_assert(W4, "the tile kernel reads its weights from the tile blob");
  using Cfg = TcCfg<BN, NS, NT, W4>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw_addr);

  const uint32_t xs = base;                                  // NS activation stages (1024-aligned)
  const uint32_t ws = xs + NS * Cfg::kXStage;                // NS weight stages
  const uint32_t bars = ws + NS * Cfg::kWStage;              // barriers
  const uint32_t bar_full = bars;                            // [NS] TMA landed
  const uint32_t bar_empty = bars + NS * 8;                  // [NS] stage may be overwritten
  const uint32_t bar_aready = bars + 2 * NS * 8;             // [NT] dequantised operand in TMEM
  const uint32_t bar_afree = bars + (2 * NS + NT) * 8;       // [NT] MMAs that read the operand are done
  const uint32_t bar_acc = bars + (2 * NS + 2 * NT) * 8;     // accumulators final
  const uint32_t tmem_slot = bar_acc + 8;
  uint8_t* gen = smem + (bars - base);
  volatile uint32_t* tmem_slot_p = reinterpret_cast<volatile uint32_t*>(gen + (2 * NS + 2 * NT + 1) * 8);
  uint8_t* out_stage = gen + ((Cfg::kBarBytes + 15) & ~15);   // 16-byte aligned (`bars` is)


  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nt = blockIdx.x, mt = blockIdx.y, z = blockIdx.z, splits = gridDim.z;
  if (threadIdx.x == 0) TT_STAMP(0);   // CTA start
  const int kt_begin = (int)(((long)z * args.kt_total) / splits);
  const int kt_end = (int)(((long)(z + 1) * args.kt_total) / splits);
  const int nk = kt_end - kt_begin;
  const int m0 = mt * BN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < NS; ++s) {
      ptx::mbar_init(bar_full + 8 * s, 1);
      ptx::mbar_init(bar_empty + 8 * s, W4 ? 129 : 1);
    }
    for (int t = 0; t < NT; ++t) {
      ptx::mbar_init(bar_aready + 8 * t, 128);
      ptx::mbar_init(bar_afree + 8 * t, 1);
    }
    ptx::mbar_init(bar_acc, 1);
    ptx::fence_mbar_init();
    ptx::prefetch_tensormap(&tmap_x);
  }
  if (warp == 1) {
    ptx::tmem_alloc(tmem_slot, Cfg::kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  allow_dependents();   // the next kernel of the stream may start prefetching its weights
  const uint32_t tmem_base = *tmem_slot_p;
  const uint32_t tmem_acc = tmem_base;             // columns [0, BN)
  const uint32_t tmem_a = tmem_base + BN;          // NT operand stages of 32 columns

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      constexpr uint32_t kTx = Cfg::kXStage + Cfg::kWStage;
      int issued = 0;
      bool ok = true;
      // Weight tiles never depend on the previous kernel of the stream, the tokens do: the first NS
      // weight tiles are requested at once, then comes the wait for that kernel, then the token boxes.
      const int early = nk < NS ? nk : NS;
      for (int i = 0; i < early; ++i) {
        ptx::mbar_expect_tx(bar_full + 8 * i, kTx);
        const uint8_t* src = args.blob + ((size_t)nt * args.kt_total + kt_begin + i) * kTileBytes;
        ptx::bulk_load(ws + i * Cfg::kWStage, src, kTileBytes, bar_full + 8 * i);
      }
      TT_STAMP(1);   // first weight copies issued
      dependency_wait();
      TT_STAMP(2);   // the previous kernel is complete
      if constexpr (MULTI) {
        if (!peer_wait(multi.sync, 1000000000ull)) atomicExch(args.status, 109);   // tokens gathered from peers
      }
      for (int i = 0; i < early; ++i)
        ptx::tensor_load_2d(xs + i * Cfg::kXStage, &tmap_x, (kt_begin + i) * 128, m0, bar_full + 8 * i);
      issued = early;
      for (int i = early; i < nk; ++i) {
        const int s = i % NS;
        const uint32_t ph = (uint32_t)(i / NS) & 1u;
        if (!ptx::mbar_wait_bounded(bar_empty + 8 * s, ph ^ 1u, kWaitLimitNs)) {
          atomicExch(args.status, 101);
          ok = false;
          break;
        }
        ptx::mbar_expect_tx(bar_full + 8 * s, kTx);
        const int kt = kt_begin + i;
        const uint8_t* src = args.blob + ((size_t)nt * args.kt_total + kt) * kTileBytes;
        ptx::bulk_load(ws + s * Cfg::kWStage, src, kTileBytes, bar_full + 8 * s);
        ptx::tensor_load_2d(xs + s * Cfg::kXStage, &tmap_x, kt * 128, m0, bar_full + 8 * s);
        ++issued;
      }
      if (!ok) {
        // copies already issued still write shared memory: let them land before the CTA exits
        for (int i = issued > NS ? issued - NS : 0; i < issued; ++i)
          ptx::mbar_wait_bounded(bar_full + 8 * (i % NS), (uint32_t)(i / NS) & 1u, kWaitLimitNs);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issue
    // The whole warp walks the loop; one elected lane issues (see ptx::elect_one).
    {
      const bool leader = ptx::elect_one();
      constexpr uint32_t idesc = ptx::idesc_i8(BN);
      bool ok = true;
      for (int i = 0; i < nk; ++i) {
        const int s = i % NS;
        const uint32_t ph = (uint32_t)(i / NS) & 1u;
        const int t = i % NT;
        const uint32_t pht = (uint32_t)(i / NT) & 1u;
        ok = ptx::mbar_wait_bounded(bar_full + 8 * s, ph, kWaitLimitNs);
        if (ok && W4) ok = ptx::mbar_wait_bounded(bar_aready + 8 * t, pht, kWaitLimitNs);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          if (leader) atomicExch(args.status, 102);
          break;
        }
        ptx::tc_fence_after();
        const uint32_t xb = xs + s * Cfg::kXStage;
        const uint32_t ab = tmem_a + t * 32;
        const uint32_t wb = ws + s * Cfg::kWStage;
        if (leader) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint64_t bdesc = ptx::smem_desc_sw128(xb + j * 32);
            const uint32_t accumulate = (i > 0 || j > 0) ? 1u : 0u;
            if (W4) ptx::mma_i8_ts(tmem_acc, ab + j * 8, bdesc, idesc, accumulate);
            else ptx::mma_i8_ss(tmem_acc, ptx::smem_desc_sw128(wb + j * 32), bdesc, idesc, accumulate);
          }
          ptx::tc_commit(bar_empty + 8 * s);
          if (W4) ptx::tc_commit(bar_afree + 8 * t);
        }
      }
      if (ok && leader) ptx::tc_commit(bar_acc);
    }
  } else {
    // ------------------------------------------------------------------ dequant, then epilogue
    const int quad = warp & 3;               // TMEM lane quadrant this warp may access
    const int row = quad * 32 + lane;        // weight row inside the tile == TMEM lane
    const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
    const int set = (threadIdx.x - 64) >> 7;
    bool ok = true;
    if (W4) {
      for (int i = set; i < nk; i += kSets) {
        const int s = i % NS;
        const uint32_t ph = (uint32_t)(i / NS) & 1u;
        const int t = i % NT;
        const uint32_t pht = (uint32_t)(i / NT) & 1u;
        if (!ptx::mbar_wait_bounded(bar_full + 8 * s, ph, kWaitLimitNs)) {
          atomicExch(args.status, 103);
          ok = false;
          break;
        }
        if (i == 0 && threadIdx.x == 64) TT_STAMP(3);   // first stage (weights and tokens) landed
        if (i + kSets >= nk && (threadIdx.x & 127) == 64 % 128 && set == ((nk - 1) % kSets)) TT_STAMP(4);   // last stage landed
        const uint8_t* wst = smem + (ws - base) + s * Cfg::kWStage;
        uint4 ch[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) ch[c] = *reinterpret_cast<const uint4*>(wst + (c * 128 + row) * 16);
        const uint32_t meta = *reinterpret_cast<const uint32_t*>(wst + 8192 + row * 4);
        ptx::mbar_arrive(bar_empty + 8 * s);

        // Unpack into registers first, wait for the operand stage afterwards: the arithmetic of this k-step
        // overlaps the MMAs that still read the stage.  (Leaving the operand store in flight during the NEXT
        // unpack, as the decode kernel does, was measured here and lost 10-30 % at prefill sizes: the MMAs of
        // a 128-token tile are long enough to starve when "operand ready" comes one unpack later.)
        const uint32_t step0 = meta & 0xffu, a0 = ((meta >> 8) & 0xffu) * 0x01010101u;
        const uint32_t step1 = (meta >> 16) & 0xffu, a1 = (meta >> 24) * 0x01010101u;
        uint32_t v[4][8];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const uint32_t step = c < 2 ? step0 : step1;
          const uint32_t ab = c < 2 ? a0 : a1;
          const uint32_t pk[4] = {ch[c].x, ch[c].y, ch[c].z, ch[c].w};
#pragma unroll
          for (int h = 0; h < 4; ++h) {
            v[c][2 * h] = lqq_dequant4(pk[h] & 0x0F0F0F0Fu, step, ab);
            v[c][2 * h + 1] = lqq_dequant4((pk[h] >> 4) & 0x0F0F0F0Fu, step, ab);
          }
        }
        if (!ptx::mbar_wait_bounded(bar_afree + 8 * t, pht ^ 1u, kWaitLimitNs)) {
          atomicExch(args.status, 104);
          ok = false;
          break;
        }
        __syncwarp();   // lanes leave the poll loops one by one; tcgen05.st / wait::st need the warp converged
        ptx::tc_fence_after();
#pragma unroll
        for (int c = 0; c < 4; ++c) ptx::tmem_st8(tmem_a + lane_addr + t * 32 + c * 8, v[c]);
        ptx::tc_wait_st();
        ptx::tc_fence_before();
        ptx::mbar_arrive(bar_aready + 8 * t);
      }
    }
    if (ok && !ptx::mbar_wait_bounded(bar_acc, 0u, kWaitLimitNs)) {
      atomicExch(args.status, 105);
      ok = false;
    }
    __syncwarp();
    if (threadIdx.x == 64) TT_STAMP(5);   // accumulator final
    dependency_wait();   // outputs, planes and token scales belong to earlier kernels until here
    if (ok) {
      ptx::tc_fence_after();
      const long n = (long)nt * 128 + row;
      const bool n_ok = n < args.N;
      const float w_scale = (n_ok && args.out_mode != kOutI32) ? args.s1[n] : 0.f;
      const bool has_bias = args.out_mode != kOutI32 && args.bias != nullptr;
      const float bias = (has_bias && n_ok) ? load_bias(args.bias, n, args.out_mode) : 0.f;
      int32_t* plane = reinterpret_cast<int32_t*>(args.out) + (size_t)z * args.M * args.N;
      const bool vec = args.vec_out != 0;   // uniform over the CTA
      const bool sc_vec = (reinterpret_cast<uintptr_t>(args.ascale) & 15u) == 0;   // 16-byte loads of the token scales
      const int q_in_set = (threadIdx.x - 64) & 127;
      uint8_t* stage = out_stage + set * Cfg::kOutStage;
#pragma unroll 1
      for (int c0 = 16 * set; c0 < BN; c0 += 16 * kSets) {   // the sets share the accumulator's columns
        if (m0 + c0 >= args.M) break;  // uniform over the set
        int v[16];
        ptx::tmem_ld16(tmem_acc + lane_addr + c0, v);
        // token scales of the chunk, fetched while the tensor-memory load is in flight
        float sc[16];
        if (args.out_mode == kOutI32) {
#pragma unroll
          for (int j = 0; j < 16; ++j) sc[j] = 0.f;
        } else if (sc_vec && m0 + c0 + 16 <= args.M) {
          const float4* sp = reinterpret_cast<const float4*>(args.ascale + m0 + c0);
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            const float4 f = __ldg(sp + q4);
            sc[4 * q4] = f.x; sc[4 * q4 + 1] = f.y; sc[4 * q4 + 2] = f.z; sc[4 * q4 + 3] = f.w;
          }
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) sc[j] = (m0 + c0 + j < args.M) ? __ldg(args.ascale + m0 + c0 + j) : 0.f;
        }
        ptx::tc_wait_ld();
        if (vec) {
          // A thread holds 16 tokens of ONE channel, the output rows run along the channels: stored
          // directly, a warp writes 64 contiguous bytes per token.  Through shared memory the set writes
          // whole 256-byte rows with 16-byte stores instead (local HBM and NVLink alike prefer those).
          // (rows past N hold values nobody copies out: w_scale and bias are zero there)
          epi_stage_cols(reinterpret_cast<uint16_t*>(stage) + row, args.out_mode, v, sc, w_scale, bias, has_bias);
          if (set == 0) asm volatile("bar.sync 1, 128;" ::: "memory");
          else asm volatile("bar.sync 2, 128;" ::: "memory");
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            const int vi = q_in_set + 128 * q;
            const int j = vi >> 4, chunk = vi & 15;
            const int m = m0 + c0 + j;
            const long ncol = (long)nt * 128 + chunk * 8;
            if (m < args.M && ncol < args.N) {
              const uint4 val = *reinterpret_cast<const uint4*>(stage + j * 256 + chunk * 16);
              if constexpr (MULTI) {
                const size_t idx = (size_t)m * multi.out.ld + multi.out.col0 + ncol;
#pragma unroll
                for (int r = 0; r < 8; ++r)   // constant indices into the kernel parameter
                  if (r < multi.out.n) *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(multi.out.ptr[r]) + idx) = val;
              } else {
                *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(args.out) + (size_t)m * args.N + ncol) = val;
              }
            }
          }
          if (set == 0) asm volatile("bar.sync 1, 128;" ::: "memory");   // the stage is rewritten by the next chunk
          else asm volatile("bar.sync 2, 128;" ::: "memory");
        } else if (n_ok) {
          const size_t idx0 = (size_t)(m0 + c0) * args.N + n;
          const int valid = args.M - (m0 + c0);
          if (args.out_mode == kOutI32) {
            epi_store_cols(plane, kEpiI32, idx0, args.N, v, sc, w_scale, bias, false, valid);
          } else if constexpr (MULTI) {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (j < valid)
                store_out_all(multi.out, m0 + c0 + j, n, lqq_scale(v[j], sc[j], w_scale), bias, has_bias, args.out_mode);
          } else {
            epi_store_cols(args.out, args.out_mode, idx0, args.N, v, sc, w_scale, bias, has_bias, valid);
          }
        }
      }
    }
    if constexpr (MULTI) {
      // every output store of this CTA, peer memory included, is ordered before the flags (see lq_common.cuh)
      asm volatile("bar.sync 3, %0;" ::"n"(128 * kSets) : "memory");
      if (threadIdx.x == 64 && args.out_mode != kOutI32) peer_signal(multi.sync);
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) TT_STAMP(6);   // all roles done
  if (warp == 1) {
    __syncwarp();
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

template <int BN, int NS, int NT, bool W4, bool MULTI>
static int launch_one(const CUtensorMap& tx, const GemmArgs& a, const MultiOut* multi, int splits, cudaStream_t st) {
  using Cfg = TcCfg<BN, NS, NT, W4>;
  auto kern = &w4a8_tile_kernel<BN, NS, NT, W4, MULTI>;
  static std::once_flag once[64];
  int dev = 0;
  cudaGetDevice(&dev);
  cudaError_t attr_err = cudaSuccess;
  std::call_once(once[dev & 63], [&]() {
    attr_err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
  });
  if (attr_err != cudaSuccess) {
    record_cuda_error(attr_err, "cudaFuncSetAttribute(w4a8_tile_kernel)");
    return LQ_ERR_CUDA;
  }
  dim3 grid((a.N + 127) / 128, (a.M + BN - 1) / BN, splits);
  cudaError_t le;
  if constexpr (MULTI) le = launch_overlapped(kern, grid, dim3(kThreads), (size_t)Cfg::kSmemBytes, st, tx, a, *multi);
  else le = launch_overlapped(kern, grid, dim3(kThreads), (size_t)Cfg::kSmemBytes, st, tx, a, NoMultiOut{});
  if (le != cudaSuccess) {
    record_cuda_error(le, "w4a8_tile_kernel launch");
    return LQ_ERR_CUDA;
  }
  return check_launch("w4a8_tile_kernel");
}

template <int BN, int NS, int NT, bool W4>
static int launch_cfg(const CUtensorMap& tx, const GemmArgs& a, const MultiOut* multi, int splits, cudaStream_t st) {
  if (multi) return launch_one<BN, NS, NT, W4, true>(tx, a, multi, splits, st);
  return launch_one<BN, NS, NT, W4, false>(tx, a, nullptr, splits, st);
}

// Token-tile widths: the smallest that holds a decode batch, 128 tokens for prefill.  A 192-token
// configuration (three shared-memory stages, two operand stages, otherwise this kernel) would do 1.5x the
// tensor-core work per unpacked weight byte; it passed the parity tests on three full-size shapes and then
// raised an unspecified launch failure on a fourth (28672 x 4096, 8192 tokens) and in back-to-back graph
// replays.  Reading the index arithmetic, the barrier counts and the tensor-memory budget (192 + 2 x 32 =
// 256 columns, two CTAs per SM) did not show the cause, so the configuration is not built.
// Between 65 and 128 tokens a small matrix (up to 32 M weights: the qkv and o projections of an 8B model)
// takes 64-token tiles: twice the CTAs, so the split factor halves and so do the int32 planes each CTA
// writes (measured at 128 tokens: 6144 x 4096 15.7 -> 14.4 us, 4096 x 4096 13.5 -> 11.7 us; 28672 x 4096
// and 4096 x 14336, which fill the machine without it, lose 38 % and 7 %).
static int tile_bn(int M, int N, int K) {
  if (M > 64 && M <= 128 && (long)N * K <= (1L << 25)) return 64;
  // A few hundred tokens on a small matrix: where 64-token tiles fill the two CTA slots of every SM in exactly
  // one wave (between 80 % and 100 % of them) they beat 128-token tiles cut along k with their planes and finish
  // pass (4096 x 4096 at 512 tokens 15.7 -> 14.5 us, 6144 x 4096 at 384 tokens 16.5 -> 15.2 us); with fewer
  // tiles the cut tiles win, with more a second wave starts.
  if (M > 128 && M <= 1024 && (long)N * K <= (1L << 25)) {
    const long tiles64 = (long)((N + 127) / 128) * ((M + 63) / 64), slots = 2L * sm_count();
    if (tiles64 <= slots && tiles64 * 5 >= slots * 4) return 64;
  }
  return M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : 128;
}

}  // namespace tile

// Split factor for the tile kernel: fill about two CTAs per SM, at least 5 k-steps per split (measured
// on 6144 x 4096 at 8 tokens: S = 4 / 5 / 6 / 8 give 8.35 / 7.95 / 8.03 / 10.9 us).
int tile_pick_splits(int M, int N, int K) {
  const int kt = K / 128;
  const int bn = tile::tile_bn(M, N, K);
  const long tiles = (long)((N + 127) / 128) * ((M + bn - 1) / bn);
  const long slots = 2L * sm_count();
  int S = 1;
  if (tiles * 2 <= slots) {
    S = (int)(slots / tiles);
    const int max_by_k = kt / 5 > 0 ? kt / 5 : 1;
    if (S > max_by_k) S = max_by_k;
    if (S > 16) S = 16;
  }
  return S < 1 ? 1 : (S > kt ? kt : S);
}

size_t tile_workspace_bytes(int M, int N, int splits) {
  return splits <= 1 ? 0 : (size_t)splits * (size_t)M * (size_t)N * sizeof(int32_t);
}

// CTAs of the launch that writes the outputs (and signals the peers): the tile grid, or the finish pass.
int finish_grid(int M, int N);   // lq_elementwise.cu
int tile_output_grid(int M, int N, int K, int splits) {
  if (splits > 1) return finish_grid(M, N);
  const int bn = tile::tile_bn(M, N, K);
  return ((N + 127) / 128) * ((M + bn - 1) / bn);
}

// out_mode: LQ_DT_* or 3 (raw int32).  Any M.  `ws` holds `splits` int32 planes (need not be zeroed).
// `out`: one or several destinations (gather by stores); `sync`: optional cross-GPU flags.
int run_tile_gemm(const int8_t* x, const uint8_t* blob, const float* ascale, const float* s1, const void* bias,
                  const OutSpec& out, const PeerSync* sync, int out_mode, int M, int N, int K, int splits, void* ws,
                  size_t ws_bytes, cudaStream_t st) {
  using namespace tile;
  if (splits > 1 && (!ws || ws_bytes < tile_workspace_bytes(M, N, splits))) return LQ_ERR_WORKSPACE;
  const int bn = tile_bn(M, N, K);
  CUtensorMap tx;
  int rc = make_byte_matrix_map(&tx, x, M, K, bn, 128);
  if (rc) return rc;
  const bool multi = out.n != 1 || out.ld != N || out.col0 != 0 || (sync && (sync->n_signal > 0 || sync->wait));
  if (multi && out_mode == kOutI32) return LQ_ERR_BAD_ARG;
  GemmArgs a;
  a.blob = blob;
  a.ascale = splits > 1 ? nullptr : ascale;
  a.s1 = splits > 1 ? nullptr : s1;
  a.bias = splits > 1 ? nullptr : bias;
  a.out = splits > 1 ? ws : out.ptr[0];
  a.status = status_word();
  a.out_mode = splits > 1 ? kOutI32 : out_mode;
  a.M = M;
  a.N = N;
  a.K = K;
  a.kt_total = K / 128;
  bool vec = splits <= 1 && (out_mode == LQ_DT_BF16 || out_mode == LQ_DT_F16) && N % 8 == 0 && out.ld % 8 == 0 &&
             out.col0 % 8 == 0;
  for (int r = 0; r < out.n; ++r) vec = vec && (reinterpret_cast<uintptr_t>(out.ptr[r]) % 16 == 0);
  a.vec_out = vec ? 1 : 0;
  if (!a.status) return LQ_ERR_CUDA;
  MultiOut mo;
  const MultiOut* mop = nullptr;
  if (multi && splits <= 1) {
    mo.out = out;
    mo.sync = sync ? *sync : PeerSync{};
    mop = &mo;
  } else if (multi && sync && sync->wait) {
    // the planes kernel only waits for the tokens; the finish pass writes and signals
    mo.out = single_out(ws, N);
    mo.sync = PeerSync{};
    mo.sync.wait = sync->wait;
    mo.sync.wait_value = sync->wait_value;
    mop = &mo;
  }
  switch (bn) {
    // 16 tokens: 8 stages, 4 operand stages (95 KB, two CTAs per SM).  Five stages and two operand stages, so
    // that three CTAs fit an SM and the next launch's CTAs can start beside this one's, measured 30 % slower
    // on 28672 x 4096 (19.2 vs 14.8 us) and 9 % slower on 4096 x 14336.
    case 16: rc = launch_cfg<16, 8, 4, true>(tx, a, mop, splits, st); break;
    case 32: rc = launch_cfg<32, 8, 4, true>(tx, a, mop, splits, st); break;
    case 64: rc = launch_cfg<64, 6, 4, true>(tx, a, mop, splits, st); break;
    default: rc = launch_cfg<128, 4, 4, true>(tx, a, mop, splits, st); break;
  }
  if (rc || splits <= 1) return rc;
  PeerSync fsync = {};
  if (sync) {
    fsync = *sync;
    fsync.wait = nullptr;   // the planes kernel already waited
  }
  return launch_finish(static_cast<const int32_t*>(ws), ascale, s1, bias, out, sync ? &fsync : nullptr, out_mode, splits,
                       M, N, st);
}

}  // namespace lq

#ifdef LQ_PIPELINE_TRACE
// Copies the per-CTA stamps of the last launch (1024 CTAs x 8 slots of int64) to host memory.
extern "C" LQ_API int lq_debug_read_tile_trace(long long* host_dst) {
  return cudaMemcpyFromSymbol(host_dst, lq::tile::g_trace, sizeof(long long) * 1024 * 8) == cudaSuccess ? 0 : -4;
}
#endif
