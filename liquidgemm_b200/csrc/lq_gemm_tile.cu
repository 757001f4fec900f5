// Tile W4A8 GEMM (M >= 17; up to 128 tokens per tile): one 128-channel x BN-token tile per CTA, two CTAs per SM.
//
// The persistent stream-K kernel keeps one CTA per SM; for a handful of k-steps per CTA its
// single MMA-issuing thread and the cross-CTA reduction tail dominate.  With small token tiles the
// shared-memory and tensor-memory footprint of a tile is small enough for two CTAs per SM, whose
// load, dequant, MMA-issue and epilogue latencies overlap each other, which measured 1.5-2x
// faster in this range.  Long-K shapes are cut into `splits` k-ranges (blockIdx.z); each CTA then
// writes an int32 partial plane and one finish kernel reduces the planes and applies
// (float)acc * ascale[m] * s1[n] (the reference's design, csrc/liquid_gemm/w4a8_wgmma.cu:39-56,
// 523-534); with one split the epilogue is fused in the GEMM kernel.
//
// Per CTA: warp 0 = TMA producer (8704-byte bulk copy of the weight tile + BN x 128 token box per
// k-step), warp 1 = TMEM allocation and tcgen05.mma issue (A operand from tensor memory), warps
// 2..5 and 6..9 = two dequant sets taking alternate k-steps (thread r of a set owns weight row r ->
// TMEM lane r; one set alone needs ~800 cycles per k-step, more than the MMAs of two CTAs), then
// epilogue, the sets sharing the accumulator's columns.  All waits are bounded.
#include <cuda.h>

#include <cstdlib>
#include <mutex>

#include "lq_common.cuh"
#include "lq_tc_ptx.cuh"

namespace lq {

int launch_finish(const int32_t* acc, const float* ascale, const float* s1, const void* bias, void* y, int out_dtype,
                  int planes, int M, int N, cudaStream_t st);  // lq_elementwise.cu
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
constexpr int kOutI32 = 3;

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
  static constexpr int kSmemBytes = 1024 /* alignment slack */ + NS * (kXStage + kWStage) + kBarBytes + BN * 4;
  static_assert(kColsNeeded <= 512, "tensor memory budget exceeded");
};

template <int BN, int NS, int NT, bool W4>
__global__ void __launch_bounds__(kThreads, 1)
w4a8_tile_kernel(const __grid_constant__ CUtensorMap tmap_x, const GemmArgs args) {
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

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nt = blockIdx.x, mt = blockIdx.y, z = blockIdx.z, splits = gridDim.z;
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
      dependency_wait();
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
    if (lane == 0) {
      constexpr uint32_t idesc = ptx::idesc_i8(BN);
      bool ok = true;
      for (int i = 0; i < nk && ok; ++i) {
        const int s = i % NS;
        const uint32_t ph = (uint32_t)(i / NS) & 1u;
        const int t = i % NT;
        const uint32_t pht = (uint32_t)(i / NT) & 1u;
        ok = ptx::mbar_wait_bounded(bar_full + 8 * s, ph, kWaitLimitNs);
        if (ok && W4) ok = ptx::mbar_wait_bounded(bar_aready + 8 * t, pht, kWaitLimitNs);
        if (!ok) {
          atomicExch(args.status, 102);
          break;
        }
        ptx::tc_fence_after();
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint64_t bdesc = ptx::smem_desc_sw128(xs + s * Cfg::kXStage + j * 32);
          const uint32_t accumulate = (i > 0 || j > 0) ? 1u : 0u;
          if (W4) {
            ptx::mma_i8_ts(tmem_acc, tmem_a + t * 32 + j * 8, bdesc, idesc, accumulate);
          } else {
            const uint64_t adesc = ptx::smem_desc_sw128(ws + s * Cfg::kWStage + j * 32);
            ptx::mma_i8_ss(tmem_acc, adesc, bdesc, idesc, accumulate);
          }
        }
        ptx::tc_commit(bar_empty + 8 * s);
        if (W4) ptx::tc_commit(bar_afree + 8 * t);
      }
      if (ok) ptx::tc_commit(bar_acc);
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
        const uint8_t* wst = smem + (ws - base) + s * Cfg::kWStage;
        uint4 ch[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) ch[c] = *reinterpret_cast<const uint4*>(wst + (c * 128 + row) * 16);
        const uint32_t meta = *reinterpret_cast<const uint32_t*>(wst + 8192 + row * 4);
        ptx::mbar_arrive(bar_empty + 8 * s);

        // Unpack into registers first, wait for the operand stage afterwards: the arithmetic of this k-step
        // overlaps the MMAs that still read the stage.
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
    dependency_wait();   // outputs, planes and token scales belong to earlier kernels until here
    if (ok) {
      ptx::tc_fence_after();
      const long n = (long)nt * 128 + row;
      const bool n_ok = n < args.N;
      const float w_scale = (n_ok && args.out_mode != kOutI32) ? args.s1[n] : 0.f;
      const bool has_bias = args.out_mode != kOutI32 && args.bias != nullptr;
      const float bias = (has_bias && n_ok) ? load_bias(args.bias, n, args.out_mode) : 0.f;
      int32_t* plane = reinterpret_cast<int32_t*>(args.out) + (size_t)z * args.M * args.N;
#pragma unroll 1
      for (int c0 = 16 * set; c0 < BN; c0 += 16 * kSets) {   // the sets share the accumulator's columns
        if (m0 + c0 >= args.M) break;  // uniform over the warp
        int v[16];
        ptx::tmem_ld16(tmem_acc + lane_addr + c0, v);
        ptx::tc_wait_ld();
        if (n_ok) {
          float sc[16];
#pragma unroll
          for (int j = 0; j < 16; ++j)   // all loads of the chunk first: one round trip
            sc[j] = (args.out_mode != kOutI32 && m0 + c0 + j < args.M) ? __ldg(args.ascale + m0 + c0 + j) : 0.f;
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int m = m0 + c0 + j;
            if (m < args.M) {
              const size_t idx = (size_t)m * args.N + n;
              if (args.out_mode == kOutI32) plane[idx] = v[j];
              else store_out_bias(args.out, idx, lqq_scale(v[j], sc[j], w_scale), bias, has_bias, args.out_mode);
            }
          }
        }
      }
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

template <int BN, int NS, int NT, bool W4>
static int launch_cfg(const CUtensorMap& tx, const GemmArgs& a, int splits, cudaStream_t st) {
  using Cfg = TcCfg<BN, NS, NT, W4>;
  auto kern = &w4a8_tile_kernel<BN, NS, NT, W4>;
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
  cudaError_t le = launch_overlapped(kern, grid, dim3(kThreads), (size_t)Cfg::kSmemBytes, st, tx, a);
  if (le != cudaSuccess) {
    record_cuda_error(le, "w4a8_tile_kernel launch");
    return LQ_ERR_CUDA;
  }
  return check_launch("w4a8_tile_kernel");
}

// Token-tile widths: the smallest that holds a decode batch; for prefill 128 or 192 tokens.  A dequantised
// weight tile costs the same whatever it is multiplied with, so wider token tiles do more tensor-core
// work per unpacked byte (192 tokens: 1.5x); but tiles are not split further, so the width that leaves
// the last wave of two CTAs per SM fullest wins.
static int wide_tiles() {
  static const int v = []() {
    const char* e = getenv("LQ_TILE_WIDE");
    return e ? atoi(e) : 0;
  }();
  return v;
}
static int tile_bn_for(int M, int N) {
  if (M <= 128) return M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : 128;
  if (!wide_tiles()) return 128;
  const long slots = 2L * sm_count();
  const long nt = (N + 127) / 128;
  double best = 0;
  int best_bn = 128;
  const int cand[2] = {128, 192};
  for (int bn : cand) {
    const long tiles = nt * ((M + bn - 1) / bn);
    const long waves = (tiles + slots - 1) / slots;
    // useful token columns per unit of time: a wave of 192-token tiles takes about 1.25x a wave of 128
    const double rate = (double)M / ((double)waves * (bn == 192 ? 1.25 : 1.0));
    if (rate > best * 1.0001) {
      best = rate;
      best_bn = bn;
    }
  }
  return best_bn;
}
static int tile_bn(int M) { return M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : 128; }

}  // namespace tile

// Split factor for the tile kernel: fill about two CTAs per SM, at least 5 k-steps per split (measured
// on 6144 x 4096 at 8 tokens: S = 4 / 5 / 6 / 8 give 8.35 / 7.95 / 8.03 / 10.9 us).
int tile_pick_splits(int M, int N, int K) {
  const int kt = K / 128;
  const long tiles = (long)((N + 127) / 128) * ((M + tile::tile_bn(M) - 1) / tile::tile_bn(M));
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

// out_mode: LQ_DT_* or 3 (raw int32).  Any M.  `ws` holds `splits` int32 planes (need not be zeroed).
int run_tile_gemm(const int8_t* x, const uint8_t* blob, const float* ascale, const float* s1, const void* bias,
                  void* out, int out_mode, int M, int N, int K, int splits, void* ws, size_t ws_bytes,
                  cudaStream_t st) {
  using namespace tile;
  if (splits > 1 && (!ws || ws_bytes < tile_workspace_bytes(M, N, splits))) return LQ_ERR_WORKSPACE;
  const int bn = splits > 1 ? tile_bn(M) : tile_bn_for(M, N);
  CUtensorMap tx;
  int rc = make_byte_matrix_map(&tx, x, M, K, bn, 128);
  if (rc) return rc;
  GemmArgs a;
  a.blob = blob;
  a.ascale = splits > 1 ? nullptr : ascale;
  a.s1 = splits > 1 ? nullptr : s1;
  a.bias = splits > 1 ? nullptr : bias;
  a.out = splits > 1 ? ws : out;
  a.status = status_word();
  a.out_mode = splits > 1 ? kOutI32 : out_mode;
  a.M = M;
  a.N = N;
  a.K = K;
  a.kt_total = K / 128;
  if (!a.status) return LQ_ERR_CUDA;
  switch (bn) {
    case 16: rc = launch_cfg<16, 8, 4, true>(tx, a, splits, st); break;
    case 32: rc = launch_cfg<32, 8, 4, true>(tx, a, splits, st); break;
    case 64: rc = launch_cfg<64, 6, 4, true>(tx, a, splits, st); break;
    case 192: rc = launch_cfg<192, 3, 2, true>(tx, a, splits, st); break;
    default: rc = launch_cfg<128, 4, 4, true>(tx, a, splits, st); break;
  }
  if (rc || splits <= 1) return rc;
  return launch_finish(static_cast<const int32_t*>(ws), ascale, s1, bias, out, out_mode, splits, M, N, st);
}

}  // namespace lq
