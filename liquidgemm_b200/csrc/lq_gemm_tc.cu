// W4A8 tensor-core GEMM for sm_100a: TMA -> in-register LQQ dequant -> TMEM -> tcgen05.mma kind::i8.
//
// Orientation.  The weights are the MMA "A" operand (128 output channels per CTA, the full
// tensor-core M), the tokens are the "B" operand (BN = 16..256 per CTA, the MMA N), so small
// token counts waste nothing on the 128-wide dimension: Y^T[n, m] = sum_k q_hat[n, k] * x[m, k].
//
// One CTA = 6 warps with fixed roles, connected by mbarrier rings:
//   warp 0      producer : one thread issues, per 128-k step, one bulk copy of the 8704-byte
//                          weight tile (nibbles + per-row step/offset pairs, contiguous in the
//                          blob) and one tiled TMA load of the BN x 128 activation box
//                          (128-byte swizzle; token rows past M are zero-filled by the TMA unit).
//   warps 2..5  dequant  : thread r owns weight row r of the tile.  It reads its 64 bytes of
//                          nibbles (4 conflict-free 16-byte shared loads) and its two
//                          (step, offset) pairs, reconstructs 128 INT8 values with
//                          AND / SHR+AND + multiply-add + XOR on 32-bit words, and writes them with
//                          tcgen05.st into TMEM lane r (4 consecutive k per 32-bit column),
//                          which is exactly the layout tcgen05.mma expects for an A operand
//                          taken from tensor memory.
//   warp 1      MMA      : one thread issues four 128 x BN x 32 tcgen05.mma per step (A from
//                          TMEM, B through a shared-memory descriptor), accumulating int32 in
//                          TMEM, and commits to the barriers that recycle the stages.
//   warps 2..5  epilogue : tcgen05.ld of the accumulators (lane = output channel, column = token),
//                          then either int32 stores (exact accumulators / split-K partial
//                          planes) or (float)acc * ascale[m] * s1[n] and the cast.
// Dequant of step i+1..i+NT-1 overlaps the MMAs of step i (NT TMEM operand stages), and the
// TMA ring runs NS steps ahead of both.
//
// The same kernel with W4 = false takes INT8 weights through a second tensor map and issues the
// shared-memory form of the MMA; that is the plain INT8 GEMM entry point.
//
// Every wait is bounded: when a barrier does not complete within kWaitLimitNs the thread writes
// a site code to the status word, leaves its loop, and the CTA still reaches the common exit
// where tensor memory is released.
#include <cuda.h>

#include <mutex>

#include "lq_common.cuh"
#include "lq_tc_ptx.cuh"

namespace lq {

int launch_finish(const int32_t* acc, const float* ascale, const float* s1, void* y, int out_dtype,
                  int planes, int M, int N, cudaStream_t st);  // lq_elementwise.cu
int launch_gemv_plain_f32(const int8_t* x, const uint8_t* nibbles, const uint8_t* s_u8,
                          const uint8_t* off_a, const float* ascale, const float* s1, float* y, int M,
                          int N, int K, int G, cudaStream_t st);  // lq_gemv.cu

constexpr int kTileBytes = 8704;     // weight tile in the blob: 8192 nibble bytes + 512 metadata bytes
constexpr int kI8TileBytes = 16384;  // INT8 weight tile: 128 rows x 128 bytes
constexpr int kThreads = 192;
constexpr uint64_t kWaitLimitNs = 2000000000ull;
constexpr int kOutI32 = 3;           // internal output mode: raw int32 (plane z of acc_out)

struct GemmArgs {
  const uint8_t* blob;   // W4: tile blob
  const float* ascale;   // [M]
  const float* s1;       // [N]
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
w4a8_tc_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
               const GemmArgs args) {
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
  float* ascale_s = reinterpret_cast<float*>(gen + Cfg::kBarBytes);

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
    if (!W4) ptx::prefetch_tensormap(&tmap_w);
  }
  if (warp == 1) {
    ptx::tmem_alloc(tmem_slot, Cfg::kTmemCols);
    ptx::tmem_relinquish();
  }
  if (warp >= 2 && args.out_mode != kOutI32) {
    for (int j = threadIdx.x - 64; j < BN; j += 128) ascale_s[j] = (m0 + j < args.M) ? args.ascale[m0 + j] : 0.f;
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_p;
  const uint32_t tmem_acc = tmem_base;             // columns [0, BN)
  const uint32_t tmem_a = tmem_base + BN;          // NT operand stages of 32 columns

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      constexpr uint32_t kTx = Cfg::kXStage + Cfg::kWStage;
      int issued = 0;
      bool ok = true;
      for (int i = 0; i < nk; ++i) {
        const int s = i % NS;
        const uint32_t ph = (uint32_t)(i / NS) & 1u;
        if (!ptx::mbar_wait_bounded(bar_empty + 8 * s, ph ^ 1u, kWaitLimitNs)) {
          atomicExch(args.status, 101);
          ok = false;
          break;
        }
        ptx::mbar_expect_tx(bar_full + 8 * s, kTx);
        const int kt = kt_begin + i;
        if (W4) {
          const uint8_t* src = args.blob + ((size_t)nt * args.kt_total + kt) * kTileBytes;
          ptx::bulk_load(ws + s * Cfg::kWStage, src, kTileBytes, bar_full + 8 * s);
        } else {
          ptx::tensor_load_2d(ws + s * Cfg::kWStage, &tmap_w, kt * 128, nt * 128, bar_full + 8 * s);
        }
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
    bool ok = true;
    if (W4) {
      for (int i = 0; i < nk; ++i) {
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

        if (!ptx::mbar_wait_bounded(bar_afree + 8 * t, pht ^ 1u, kWaitLimitNs)) {
          atomicExch(args.status, 104);
          ok = false;
          break;
        }
        ptx::tc_fence_after();
        const uint32_t step0 = meta & 0xffu, a0 = ((meta >> 8) & 0xffu) * 0x01010101u;
        const uint32_t step1 = (meta >> 16) & 0xffu, a1 = (meta >> 24) * 0x01010101u;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const uint32_t step = c < 2 ? step0 : step1;
          const uint32_t ab = c < 2 ? a0 : a1;
          const uint32_t pk[4] = {ch[c].x, ch[c].y, ch[c].z, ch[c].w};
          uint32_t v[8];
#pragma unroll
          for (int h = 0; h < 4; ++h) {
            v[2 * h] = lqq_dequant4(pk[h] & 0x0F0F0F0Fu, step, ab);
            v[2 * h + 1] = lqq_dequant4((pk[h] >> 4) & 0x0F0F0F0Fu, step, ab);
          }
          ptx::tmem_st8(tmem_a + lane_addr + t * 32 + c * 8, v);
        }
        ptx::tc_wait_st();
        ptx::tc_fence_before();
        ptx::mbar_arrive(bar_aready + 8 * t);
      }
    }
    if (ok && !ptx::mbar_wait_bounded(bar_acc, 0u, kWaitLimitNs)) {
      atomicExch(args.status, 105);
      ok = false;
    }
    if (ok) {
      ptx::tc_fence_after();
      const long n = (long)nt * 128 + row;
      const bool n_ok = n < args.N;
      const float w_scale = (n_ok && args.out_mode != kOutI32) ? args.s1[n] : 0.f;
      int32_t* plane = reinterpret_cast<int32_t*>(args.out) + (size_t)z * args.M * args.N;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 16) {
        if (m0 + c0 >= args.M) break;  // uniform over the CTA
        int v[16];
        ptx::tmem_ld16(tmem_acc + lane_addr + c0, v);
        ptx::tc_wait_ld();
        if (n_ok) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int m = m0 + c0 + j;
            if (m < args.M) {
              const size_t idx = (size_t)m * args.N + n;
              if (args.out_mode == kOutI32) plane[idx] = v[j];
              else store_out(args.out, idx, lqq_scale(v[j], ascale_s[c0 + j], w_scale), args.out_mode);
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

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, []() {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// Tensor map over a row-major int8 matrix [rows, K] with a (box_rows x 128-byte) box, 128-byte
// swizzle and zero fill for out-of-range rows.
static int make_rowmajor_i8_map(CUtensorMap* map, const void* ptr, int rows, int K, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) {
    record_cuda_error(cudaErrorUnknown, "cuTensorMapEncodeTiled entry point not found");
    return LQ_ERR_CUDA;
  }
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)K};
  const cuuint32_t box[2] = {128u, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1u, 1u};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    record_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled failed");
    return LQ_ERR_CUDA;
  }
  return LQ_OK;
}

template <int BN, int NS, int NT, bool W4>
static int launch_cfg(const CUtensorMap& tx, const CUtensorMap& tw, const GemmArgs& a, int splits, cudaStream_t st) {
  using Cfg = TcCfg<BN, NS, NT, W4>;
  auto kern = &w4a8_tc_kernel<BN, NS, NT, W4>;
  static std::once_flag once[64];
  int dev = 0;
  cudaGetDevice(&dev);
  cudaError_t attr_err = cudaSuccess;
  std::call_once(once[dev & 63], [&]() {
    attr_err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
  });
  if (attr_err != cudaSuccess) {
    record_cuda_error(attr_err, "cudaFuncSetAttribute(w4a8_tc_kernel)");
    return LQ_ERR_CUDA;
  }
  dim3 grid((a.N + 127) / 128, (a.M + BN - 1) / BN, splits);
  kern<<<grid, kThreads, Cfg::kSmemBytes, st>>>(tx, tw, a);
  return check_launch("w4a8_tc_kernel");
}

static int pick_bn(int M) {
  if (M <= 16) return 16;
  if (M <= 32) return 32;
  if (M <= 64) return 64;
  if (M <= 128) return 128;
  const int rem = M % 256;
  if (M < 1024 && rem > 0 && rem <= 128) return 128;
  return 256;
}

// x: [M,K] int8 tokens.  w: W4 blob or [N,K] int8 weights.
template <bool W4>
static int run_gemm(const int8_t* x, const void* w, const float* ascale, const float* s1, void* out, int out_mode,
                    int M, int N, int K, int splits, cudaStream_t st) {
  const int bn = pick_bn(M);
  CUtensorMap tx, tw;
  int rc = make_rowmajor_i8_map(&tx, x, M, K, bn);
  if (rc) return rc;
  if (W4) tw = tx;
  else if ((rc = make_rowmajor_i8_map(&tw, w, N, K, 128))) return rc;
  GemmArgs a;
  a.blob = W4 ? static_cast<const uint8_t*>(w) : nullptr;
  a.ascale = ascale;
  a.s1 = s1;
  a.out = out;
  a.status = status_word();
  a.out_mode = out_mode;
  a.M = M;
  a.N = N;
  a.K = K;
  a.kt_total = K / 128;
  if (!a.status) return LQ_ERR_CUDA;
  if (W4) {
    switch (bn) {
      case 16: return launch_cfg<16, 8, 4, true>(tx, tw, a, splits, st);
      case 32: return launch_cfg<32, 8, 4, true>(tx, tw, a, splits, st);
      case 64: return launch_cfg<64, 6, 4, true>(tx, tw, a, splits, st);
      case 128: return launch_cfg<128, 4, 4, true>(tx, tw, a, splits, st);
      default: return launch_cfg<256, 5, 4, true>(tx, tw, a, splits, st);
    }
  } else {
    switch (bn) {
      case 16: return launch_cfg<16, 5, 1, false>(tx, tw, a, splits, st);
      case 32: return launch_cfg<32, 5, 1, false>(tx, tw, a, splits, st);
      case 64: return launch_cfg<64, 4, 1, false>(tx, tw, a, splits, st);
      case 128: return launch_cfg<128, 3, 1, false>(tx, tw, a, splits, st);
      default: return launch_cfg<256, 4, 1, false>(tx, tw, a, splits, st);
    }
  }
}

static int clamp_splits(int splitk, int M, int N, int K) {
  if (splitk <= 0) splitk = lq_gemm_pick_splitk(M, N, K, 0);
  const int kt = K / 128;
  if (splitk > kt) splitk = kt;
  return splitk < 1 ? 1 : splitk;
}

static int w4_common(const int8_t* x, const uint8_t* blob, const float* ascale, const float* s1, void* out,
                     int out_mode, int M, int N, int K, int splitk, void* ws, size_t ws_bytes, cudaStream_t st) {
  if (!x || !blob || !out || M < 0 || N <= 0 || K <= 0) return LQ_ERR_BAD_ARG;
  if (K % 128) return LQ_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(blob)) % 16) return LQ_ERR_BAD_ARG;
  if (M == 0) return LQ_OK;
  if (int rc = lq_check_device()) return rc;
  const int S = clamp_splits(splitk, M, N, K);
  if (S == 1) return run_gemm<true>(x, blob, ascale, s1, out, out_mode, M, N, K, 1, st);
  if (!ws || ws_bytes < lq_gemm_workspace_bytes(M, N, K, S)) return LQ_ERR_WORKSPACE;
  int rc = run_gemm<true>(x, blob, nullptr, nullptr, ws, kOutI32, M, N, K, S, st);
  if (rc) return rc;
  return launch_finish(static_cast<const int32_t*>(ws), ascale, s1, out, out_mode, S, M, N, st);
}

}  // namespace lq

using namespace lq;

extern "C" {

int lq_gemm_pick_splitk(int M, int N, int K, int env_override) {
  if (M <= 0 || N <= 0 || K < 128) return 1;
  const int kt = K / 128;
  int S = 1;
  if (env_override > 0 && M <= 128) {
    S = env_override;
  } else {
    // Fill the machine: with T output tiles and 2 resident CTAs per SM, split K until there are
    // about 2 x SM-count CTAs, keeping at least 8 k-steps per split.
    const int bn = pick_bn(M);
    const long tiles = (long)((N + 127) / 128) * ((M + bn - 1) / bn);
    const long slots = 2L * sm_count();
    if (tiles * 2 <= slots) {
      S = (int)(slots / tiles);
      const int max_by_k = kt / 8 > 0 ? kt / 8 : 1;
      if (S > max_by_k) S = max_by_k;
      if (S > 16) S = 16;
    }
  }
  if (S > kt) S = kt;
  return S < 1 ? 1 : S;
}

size_t lq_gemm_workspace_bytes(int M, int N, int K, int splitk) {
  (void)K;
  if (splitk <= 1 || M <= 0 || N <= 0) return 0;
  return (size_t)splitk * (size_t)M * (size_t)N * sizeof(int32_t);
}

int lq_w4a8_gemm_i32(const int8_t* x_i8, const uint8_t* blob, int32_t* acc, int M, int N, int K, int splitk,
                     void* workspace, size_t workspace_bytes, void* stream) {
  return w4_common(x_i8, blob, nullptr, nullptr, acc, kOutI32, M, N, K, splitk, workspace, workspace_bytes,
                   as_stream(stream));
}

int lq_w4a8_gemm_fused(const int8_t* x_i8, const uint8_t* blob, const float* ascale, const float* s1, void* y,
                       int out_dtype, int M, int N, int K, int splitk, void* workspace, size_t workspace_bytes,
                       void* stream) {
  if (!ascale || !s1 || out_dtype < 0 || out_dtype > 2) return LQ_ERR_BAD_ARG;
  return w4_common(x_i8, blob, ascale, s1, y, out_dtype, M, N, K, splitk, workspace, workspace_bytes,
                   as_stream(stream));
}

size_t lq_gemm_v1_workspace_bytes(int M, int N, int K) {
  if (M <= 16) return 0;
  const size_t blob = lq_tile_blob_bytes(N, K);
  const int S = lq_gemm_pick_splitk(M, N, K, 0);
  return ((blob + 255) / 256) * 256 + lq_gemm_workspace_bytes(M, N, K, S);
}

int lq_w4a8_gemm_v1(const int8_t* x_i8, const uint8_t* nibbles, const uint8_t* s_u8, const uint8_t* offset_a,
                    const float* s1, const float* ascale, float* y, int M, int N, int K, int group_size,
                    void* workspace, size_t workspace_bytes, void* stream) {
  if (!x_i8 || !nibbles || !s_u8 || !offset_a || !s1 || !ascale || !y || M < 0 || N <= 0 || K <= 0)
    return LQ_ERR_BAD_ARG;
  if (group_size != 64 || K % 64) return LQ_ERR_SHAPE;
  if (M == 0) return LQ_OK;
  cudaStream_t st = as_stream(stream);
  if (M <= 16) {
    if ((reinterpret_cast<uintptr_t>(x_i8) | reinterpret_cast<uintptr_t>(nibbles)) % 16) return LQ_ERR_BAD_ARG;
    return launch_gemv_plain_f32(x_i8, nibbles, s_u8, offset_a, ascale, s1, y, M, N, K, K / 64, st);
  }
  if (K % 128) return LQ_ERR_SHAPE;
  if (!workspace || workspace_bytes < lq_gemm_v1_workspace_bytes(M, N, K)) return LQ_ERR_WORKSPACE;
  uint8_t* blob = static_cast<uint8_t*>(workspace);
  const size_t blob_bytes = ((lq_tile_blob_bytes(N, K) + 255) / 256) * 256;
  int rc = lq_repack_tiles(nibbles, LQ_SRC_NIBBLES, s_u8, offset_a, blob, N, K, group_size, stream);
  if (rc) return rc;
  const int S = lq_gemm_pick_splitk(M, N, K, 0);
  return w4_common(x_i8, blob, ascale, s1, y, LQ_DT_F32, M, N, K, S, blob + blob_bytes,
                   workspace_bytes - blob_bytes, st);
}

static int i8_common(const int8_t* a, const int8_t* b, const float* a_scale, const float* b_scale, void* out,
                     int out_mode, int M, int N, int K, void* stream) {
  if (!a || !b || !out || M < 0 || N <= 0 || K <= 0) return LQ_ERR_BAD_ARG;
  if (K % 128) return LQ_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b)) % 16) return LQ_ERR_BAD_ARG;
  if (M == 0) return LQ_OK;
  if (int rc = lq_check_device()) return rc;
  return run_gemm<false>(a, b, a_scale, b_scale, out, out_mode, M, N, K, 1, as_stream(stream));
}

int lq_i8_gemm_i32(const int8_t* a, const int8_t* b, int32_t* c, int M, int N, int K, void* stream) {
  return i8_common(a, b, nullptr, nullptr, c, kOutI32, M, N, K, stream);
}

int lq_i8_gemm_scaled(const int8_t* a, const int8_t* b, const float* a_scale, const float* b_scale, void* y,
                      int out_dtype, int M, int N, int K, void* stream) {
  if (!a_scale || !b_scale || out_dtype < 0 || out_dtype > 2) return LQ_ERR_BAD_ARG;
  return i8_common(a, b, a_scale, b_scale, y, out_dtype, M, N, K, stream);
}

}  // extern "C"
