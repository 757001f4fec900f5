// Memory-bound helpers of the W4A8 path: standalone dequant, per-token activation quantiser,
// scale epilogue, split-K finish and the weight re-tiling kernels.  All of them are sized as a
// grid-stride sweep over a multiple of the SM count and move 16 bytes per thread per access.
#include <type_traits>

#include "lq_common.cuh"

namespace lq {

// ---------------------------------------------------------------------------------------------
// dequant_weight: [N,K] one code per byte -> int8 [N,K]
// ---------------------------------------------------------------------------------------------
// One thread handles 16 consecutive codes (one uint4 in, one uint4 out); 16 divides every legal
// group size that is a multiple of 16, otherwise the 4-code path below is used.
template <int VEC_WORDS>
__global__ void __launch_bounds__(256)
dequant_weight_kernel(const uint32_t* __restrict__ q, const uint8_t* __restrict__ s_u8,
                      const uint8_t* __restrict__ off_a, uint32_t* __restrict__ out,
                      long total_vec, int K, int group_size) {
  const int vec_codes = VEC_WORDS * 4;
  const int vec_per_row = K / vec_codes;
  const int G = K / group_size;
  for (long v = (long)blockIdx.x * blockDim.x + threadIdx.x; v < total_vec;
       v += (long)gridDim.x * blockDim.x) {
    const long n = v / vec_per_row;
    const int k = (int)(v - n * vec_per_row) * vec_codes;
    const int g = k / group_size;
    const uint32_t step = s_u8[n * G + g];
    const uint32_t a = off_a[n * G + g] * 0x01010101u;
    if (VEC_WORDS == 4) {
      uint4 w = reinterpret_cast<const uint4*>(q)[v];
      w.x = lqq_dequant4(w.x, step, a);
      w.y = lqq_dequant4(w.y, step, a);
      w.z = lqq_dequant4(w.z, step, a);
      w.w = lqq_dequant4(w.w, step, a);
      reinterpret_cast<uint4*>(out)[v] = w;
    } else {
      out[v] = lqq_dequant4(q[v], step, a);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// quant_per_token
// ---------------------------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

__device__ __forceinline__ float block_max(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = lane < (blockDim.x >> 5) ? red[lane] : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) r = fmaxf(r, __shfl_xor_sync(0xffffffffu, r, o));
  return r;
}

__device__ __forceinline__ int quant1(float x, float scale) {
  // IEEE division, round half to even, clamp: liquidgemm/quant.py:140 of the reference.
  int q = __float2int_rn(__fdiv_rn(x, scale));
  return max(-127, min(127, q));
}

// One CTA per token row.  Elements are read in 16-byte vectors; the row is visited twice
// (amax, then quantise) and the second visit is served by L1/L2.
template <typename T>
__global__ void __launch_bounds__(256)
quant_per_token_kernel(const T* __restrict__ x, int8_t* __restrict__ xq, float* __restrict__ ascale,
                       int K) {
  __shared__ float red[32];
  // The linear that consumes these tokens is launched with programmatic stream serialisation: let it
  // start streaming its weights now; it waits for this grid before it reads the tokens.
  allow_dependents();
  // This grid itself may have been started while the previous kernel of the stream was still running:
  // that kernel may still write the activations or read the buffers written here.
  dependency_wait();
  const long m = blockIdx.x;
  const T* xr = x + m * K;
  int8_t* qr = xq + m * K;
  constexpr int VEC = 16 / sizeof(T);
  const bool vec_ok = (K % 16 == 0) && ((reinterpret_cast<uintptr_t>(xr) & 15) == 0) &&
                      ((reinterpret_cast<uintptr_t>(qr) & 15) == 0);
  float amax = 0.f;
  if (vec_ok) {
    for (int k = threadIdx.x * VEC; k < K; k += blockDim.x * VEC) {
      uint4 raw = *reinterpret_cast<const uint4*>(xr + k);
      const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int i = 0; i < VEC; ++i) amax = fmaxf(amax, fabsf(to_f32<T>(e[i])));
    }
  } else {
    for (int k = threadIdx.x; k < K; k += blockDim.x) amax = fmaxf(amax, fabsf(to_f32<T>(xr[k])));
  }
  amax = block_max(amax, red);
  const float scale = __fdiv_rn(fmaxf(amax, 1e-12f), 127.0f);
  if (threadIdx.x == 0) ascale[m] = scale;
  if (vec_ok) {
    // 16 outputs (one uint4 of int8) per thread per step
    for (int k = threadIdx.x * 16; k < K; k += blockDim.x * 16) {
      uint32_t packed[4];
#pragma unroll
      for (int v = 0; v < 16 / VEC; ++v) {
        uint4 raw = *reinterpret_cast<const uint4*>(xr + k + v * VEC);
        const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
          const int idx = v * VEC + i;
          const uint32_t b = static_cast<uint32_t>(quant1(to_f32<T>(e[i]), scale)) & 0xffu;
          if ((idx & 3) == 0) packed[idx >> 2] = b;
          else packed[idx >> 2] |= b << (8 * (idx & 3));
        }
      }
      *reinterpret_cast<uint4*>(qr + k) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    }
  } else {
    for (int k = threadIdx.x; k < K; k += blockDim.x) qr[k] = (int8_t)quant1(to_f32<T>(xr[k]), scale);
  }
}

// ---------------------------------------------------------------------------------------------
// Tile blob -> row-major INT8 weights [N, K] (the level-2 dequantisation of the whole matrix), for very large
// token counts where unpacking once and running the INT8 x INT8 pair kernel beats unpacking inside the main
// loop.  One CTA of 128 threads per 128 x 128 tile; thread = weight row, which it writes as one 128-byte line.
__global__ void __launch_bounds__(128)
unpack_blob_i8_kernel(const uint8_t* __restrict__ blob, int8_t* __restrict__ w, int N, int K) {
  const int kt = blockIdx.x, nt = blockIdx.y, row = threadIdx.x;
  const uint8_t* tile = blob + ((size_t)nt * (K / 128) + kt) * 8704;
  uint4 ch[4];
#pragma unroll
  for (int c = 0; c < 4; ++c) ch[c] = __ldg(reinterpret_cast<const uint4*>(tile + (c * 128 + row) * 16));
  const uint32_t meta = __ldg(reinterpret_cast<const uint32_t*>(tile + 8192 + row * 4));
  const uint32_t step0 = meta & 0xffu, a0 = ((meta >> 8) & 0xffu) * 0x01010101u;
  const uint32_t step1 = (meta >> 16) & 0xffu, a1 = (meta >> 24) * 0x01010101u;
  const long n = (long)nt * 128 + row;
  if (n >= N) return;
  uint4* dst = reinterpret_cast<uint4*>(w + n * K + (long)kt * 128);
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
    dst[2 * c] = make_uint4(v[0], v[1], v[2], v[3]);
    dst[2 * c + 1] = make_uint4(v[4], v[5], v[6], v[7]);
  }
}

// Enqueue the unpack of a whole blob (N a multiple of 128 rows in the blob; K % 128 == 0; `w` 16-byte aligned).
int run_unpack_blob_i8(const uint8_t* blob, int8_t* w, int N, int K, cudaStream_t st) {
  dim3 grid(K / 128, (N + 127) / 128);
  unpack_blob_i8_kernel<<<grid, 128, 0, st>>>(blob, w, N, K);
  return check_launch("unpack_blob_i8_kernel");
}

// ---------------------------------------------------------------------------------------------
// scale_epilogue and split-K finish
// ---------------------------------------------------------------------------------------------
// out_dtype 0..2 select the scaled output type; 3 writes the exact int32 sum of the planes.
// planes == 1: plain epilogue.  planes > 1: sum of `planes` int32 partial planes [planes][M][N]
// first (exact in any order), then the same formula
// (reference csrc/liquid_gemm/w4a8_wgmma.cu:39-56).
// MULTI: the outputs go to several row-major matrices with their own row stride and column offset (gather by
// stores over NVLink, see OutSpec), element by element, and every CTA signals the peers' flags at its end.
template <bool MULTI>
__global__ void __launch_bounds__(256)
finish_kernel(const int32_t* __restrict__ acc, const float* __restrict__ ascale,
              const float* __restrict__ s1, const void* __restrict__ bias, void* __restrict__ y, int out_dtype,
              int planes, int M, int N, bool vec, const std::conditional_t<MULTI, MultiOut, NoMultiOut> multi) {
  // Launched with programmatic stream serialisation behind the kernel that writes the planes: let the
  // kernel after this one start (it prefetches weights, and waits for this grid before it touches
  // tokens, planes or outputs), then wait for the planes to be complete.
  allow_dependents();
  dependency_wait();
  const long total = (long)M * N;
  const long quads = total >> 2;
  if (vec) {
    for (long qd = (long)blockIdx.x * blockDim.x + threadIdx.x; qd < quads;
         qd += (long)gridDim.x * blockDim.x) {
      const long idx = qd << 2;
      const int m = (int)(idx / N);
      const int n = (int)(idx - (long)m * N);
      int4 v = *reinterpret_cast<const int4*>(acc + idx);
      for (int p = 1; p < planes; ++p) {
        const int4 w = *reinterpret_cast<const int4*>(acc + (long)p * total + idx);
        v.x += w.x; v.y += w.y; v.z += w.z; v.w += w.w;
      }
      if (out_dtype == 3) {  // exact int32 sum, no scaling
        *reinterpret_cast<int4*>(reinterpret_cast<int32_t*>(y) + idx) = v;
        continue;
      }
      const float a = ascale[m];
      const float4 w1 = *reinterpret_cast<const float4*>(s1 + n);
      float r0 = lqq_scale(v.x, a, w1.x), r1 = lqq_scale(v.y, a, w1.y);
      float r2 = lqq_scale(v.z, a, w1.z), r3 = lqq_scale(v.w, a, w1.w);
      if (bias) {
        // bias joins the value already rounded to the output type (PyTorch's `y + bias`); the stores
        // below round the sum once more
        const float b0 = load_bias(bias, n, out_dtype), b1 = load_bias(bias, n + 1, out_dtype);
        const float b2 = load_bias(bias, n + 2, out_dtype), b3 = load_bias(bias, n + 3, out_dtype);
        if (out_dtype == LQ_DT_BF16) {
          r0 = __bfloat162float(__float2bfloat16_rn(r0)); r1 = __bfloat162float(__float2bfloat16_rn(r1));
          r2 = __bfloat162float(__float2bfloat16_rn(r2)); r3 = __bfloat162float(__float2bfloat16_rn(r3));
        } else if (out_dtype == LQ_DT_F16) {
          r0 = __half2float(__float2half_rn(r0)); r1 = __half2float(__float2half_rn(r1));
          r2 = __half2float(__float2half_rn(r2)); r3 = __half2float(__float2half_rn(r3));
        }
        r0 = __fadd_rn(r0, b0); r1 = __fadd_rn(r1, b1); r2 = __fadd_rn(r2, b2); r3 = __fadd_rn(r3, b3);
      }
      if (out_dtype == LQ_DT_F32) {
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(y) + idx) = make_float4(r0, r1, r2, r3);
      } else if (out_dtype == LQ_DT_BF16) {
        __nv_bfloat162 lo = __halves2bfloat162(__float2bfloat16_rn(r0), __float2bfloat16_rn(r1));
        __nv_bfloat162 hi = __halves2bfloat162(__float2bfloat16_rn(r2), __float2bfloat16_rn(r3));
        uint2 o;
        o.x = *reinterpret_cast<uint32_t*>(&lo);
        o.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(y) + idx) = o;
      } else {
        __half2 lo = __halves2half2(__float2half_rn(r0), __float2half_rn(r1));
        __half2 hi = __halves2half2(__float2half_rn(r2), __float2half_rn(r3));
        uint2 o;
        o.x = *reinterpret_cast<uint32_t*>(&lo);
        o.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(y) + idx) = o;
      }
    }
  } else {
    for (long idx = (long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (long)gridDim.x * blockDim.x) {
      const int m = (int)(idx / N);
      const int n = (int)(idx - (long)m * N);
      int v = acc[idx];
      for (int p = 1; p < planes; ++p) v += acc[(long)p * total + idx];
      if (out_dtype == 3) reinterpret_cast<int32_t*>(y)[idx] = v;
      else if constexpr (MULTI)
        store_out_all(multi.out, m, n, lqq_scale(v, ascale[m], s1[n]), bias ? load_bias(bias, n, out_dtype) : 0.f,
                      bias != nullptr, out_dtype);
      else store_out_bias(y, idx, lqq_scale(v, ascale[m], s1[n]), bias ? load_bias(bias, n, out_dtype) : 0.f,
                          bias != nullptr, out_dtype);
    }
  }
  if constexpr (MULTI) {
    __syncthreads();   // every store of the CTA before the flags (release is cumulative over what the barrier ordered)
    if (threadIdx.x == 0) peer_signal(multi.sync);
  }
}

// ---------------------------------------------------------------------------------------------
// weight re-tiling for the tensor-core GEMM
// ---------------------------------------------------------------------------------------------
// Blob tile (nt, kt), 8704 bytes at ((nt * KT) + kt) * 8704:
//   bytes [0, 8192): chunk c (32 k each), row r, 16 bytes at (c*128 + r)*16; 32-bit word h of the
//     chunk holds the octet k = 32c + 8h .. +7 of row r: byte b = code[8h+b] | code[8h+4+b] << 4,
//     so `word & 0x0F0F0F0F` is four consecutive k in byte lanes and `(word >> 4) & 0x0F..` the next
//     four (the mask/shift-only unpack of liquidgemm/ops.py:143-149 of the reference).
//   bytes [8192, 8704): row r, 4 bytes (step, offset) of k 0..63 then (step, offset) of k 64..127.
// Rows past N are written as code 0, step 1, offset 128, which reconstructs to q_hat = 0.
// One thread produces one 16-byte chunk entry, or (threads 512..639 of a tile) one metadata word.
constexpr int kTileBytes = 8704;

__global__ void __launch_bounds__(128)
repack_tiles_kernel(const uint8_t* __restrict__ src, int src_layout,
                    const uint8_t* __restrict__ s_u8, const uint8_t* __restrict__ off_a,
                    uint8_t* __restrict__ blob, int N, int K, int group_size, long total_tiles) {
  const int KT = K >> 7;
  const int G = K / group_size;
  for (long tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
    const int nt = (int)(tile / KT), kt = (int)(tile - (long)nt * KT);
    uint8_t* out = blob + tile * kTileBytes;
    const int r = threadIdx.x;
    const long n = (long)nt * 128 + r;
    const int k0 = kt * 128;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t words[4] = {0u, 0u, 0u, 0u};
      if (n < N) {
        if (src_layout == LQ_SRC_CODES) {
          const uint4* p = reinterpret_cast<const uint4*>(src + n * K + k0 + c * 32);
          const uint4 lo = p[0], hi = p[1];
          const uint32_t cw[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
          for (int h = 0; h < 4; ++h) words[h] = (cw[2 * h] & 0x0F0F0F0Fu) | ((cw[2 * h + 1] & 0x0F0F0F0Fu) << 4);
        } else {
          // pack_nibbles order: byte j = code[2j] | code[2j+1] << 4; 16 bytes cover this chunk
          const uint4 v = *reinterpret_cast<const uint4*>(src + n * (K >> 1) + ((k0 + c * 32) >> 1));
          const uint32_t nw[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
          for (int h = 0; h < 4; ++h) {
            const uint32_t w = nw[h];  // codes 8h .. 8h+7, code i in nibble i
            uint32_t o = 0;
#pragma unroll
            for (int b = 0; b < 4; ++b) {
              const uint32_t lo4 = (w >> (4 * b)) & 0xFu;         // code 8h + b
              const uint32_t hi4 = (w >> (4 * (b + 4))) & 0xFu;   // code 8h + 4 + b
              o |= (lo4 | (hi4 << 4)) << (8 * b);
            }
            words[h] = o;
          }
        }
      }
      *reinterpret_cast<uint4*>(out + (c * 128 + r) * 16) = make_uint4(words[0], words[1], words[2], words[3]);
    }
    uint32_t meta = 0x80018001u;  // step 1, offset 128 twice
    if (n < N) {
      const int g0 = k0 / group_size, g1 = (k0 + 64) / group_size;
      meta = (uint32_t)s_u8[n * G + g0] | ((uint32_t)off_a[n * G + g0] << 8) |
             ((uint32_t)s_u8[n * G + g1] << 16) | ((uint32_t)off_a[n * G + g1] << 24);
    }
    reinterpret_cast<uint32_t*>(out + 8192)[r] = meta;
  }
}

static int grid_for(long work_items, int threads, int waves) {
  long blocks = (work_items + threads - 1) / threads;
  long cap = (long)sm_count() * waves;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

static long finish_items(int M, int N, bool vec) { return vec ? ((long)M * N) >> 2 : (long)M * N; }

// CTAs of the (multi-destination, element-wise) finish pass: what a peer has to see arrive.
int finish_grid(int M, int N) { return grid_for(finish_items(M, N, false), 256, 8); }

int launch_finish(const int32_t* acc, const float* ascale, const float* s1, const void* bias, const OutSpec& out,
                  const PeerSync* sync, int out_dtype, int planes, int M, int N, cudaStream_t st) {
  const bool multi = out.n != 1 || out.ld != N || out.col0 != 0 || (sync && (sync->n_signal > 0 || sync->wait));
  void* y = out.ptr[0];
  // four outputs per thread when every row start stays 16-byte aligned (single destination only)
  const uintptr_t align_bits = reinterpret_cast<uintptr_t>(acc) | reinterpret_cast<uintptr_t>(y) |
                               reinterpret_cast<uintptr_t>(s1) | reinterpret_cast<uintptr_t>(bias);
  const bool vec = !multi && (N % 4 == 0) && (align_bits % 16 == 0);
  const int grid = grid_for(finish_items(M, N, vec), 256, 8);
  cudaError_t e;
  if (multi) {
    MultiOut mo;
    mo.out = out;
    mo.sync = sync ? *sync : PeerSync{};
    e = launch_overlapped(finish_kernel<true>, dim3(grid), dim3(256), (size_t)0, st, acc, ascale, s1, bias, y, out_dtype,
                          planes, M, N, vec, mo);
  } else {
    e = launch_overlapped(finish_kernel<false>, dim3(grid), dim3(256), (size_t)0, st, acc, ascale, s1, bias, y,
                          out_dtype, planes, M, N, vec, NoMultiOut{});
  }
  if (e != cudaSuccess) {
    record_cuda_error(e, "finish_kernel launch");
    return LQ_ERR_CUDA;
  }
  return check_launch("finish_kernel");
}

}  // namespace lq

using namespace lq;

extern "C" {

int lq_dequant_weight(const uint8_t* q_u4, const uint8_t* s_u8, const uint8_t* offset_a,
                      int8_t* out_i8, int N, int K, int group_size, void* stream) {
  if (!q_u4 || !s_u8 || !offset_a || !out_i8 || N <= 0 || K <= 0 || group_size <= 0) return LQ_ERR_BAD_ARG;
  if (K % 4 || group_size % 4 || K % group_size) return LQ_ERR_SHAPE;
  const bool v16 = (K % 16 == 0) && (group_size % 16 == 0) &&
                   ((reinterpret_cast<uintptr_t>(q_u4) | reinterpret_cast<uintptr_t>(out_i8)) % 16 == 0);
  cudaStream_t st = as_stream(stream);
  if (v16) {
    const long total = (long)N * (K / 16);
    dequant_weight_kernel<4><<<grid_for(total, 256, 8), 256, 0, st>>>(
        reinterpret_cast<const uint32_t*>(q_u4), s_u8, offset_a, reinterpret_cast<uint32_t*>(out_i8),
        total, K, group_size);
  } else {
    const long total = (long)N * (K / 4);
    dequant_weight_kernel<1><<<grid_for(total, 256, 8), 256, 0, st>>>(
        reinterpret_cast<const uint32_t*>(q_u4), s_u8, offset_a, reinterpret_cast<uint32_t*>(out_i8),
        total, K, group_size);
  }
  return check_launch("dequant_weight_kernel");
}

int lq_quant_per_token(const void* x, int in_dtype, int8_t* xq, float* ascale, int M, int K,
                       void* stream) {
  if (!x || !xq || !ascale || M < 0 || K <= 0) return LQ_ERR_BAD_ARG;
  if (M == 0) return LQ_OK;
  cudaStream_t st = as_stream(stream);
  cudaError_t e;
  switch (in_dtype) {
    case LQ_DT_BF16:
      e = launch_overlapped(quant_per_token_kernel<__nv_bfloat16>, dim3(M), dim3(256), (size_t)0, st,
                            static_cast<const __nv_bfloat16*>(x), xq, ascale, K);
      break;
    case LQ_DT_F16:
      e = launch_overlapped(quant_per_token_kernel<__half>, dim3(M), dim3(256), (size_t)0, st,
                            static_cast<const __half*>(x), xq, ascale, K);
      break;
    case LQ_DT_F32:
      e = launch_overlapped(quant_per_token_kernel<float>, dim3(M), dim3(256), (size_t)0, st,
                            static_cast<const float*>(x), xq, ascale, K);
      break;
    default:
      return LQ_ERR_BAD_ARG;
  }
  if (e != cudaSuccess) {
    record_cuda_error(e, "quant_per_token_kernel launch");
    return LQ_ERR_CUDA;
  }
  return check_launch("quant_per_token_kernel");
}

int lq_scale_epilogue(const int32_t* acc, const float* ascale, const float* s1, void* y,
                      int out_dtype, int M, int N, void* stream) {
  if (!acc || !ascale || !s1 || !y || M < 0 || N <= 0) return LQ_ERR_BAD_ARG;
  if (out_dtype < 0 || out_dtype > 2) return LQ_ERR_BAD_ARG;
  if (M == 0) return LQ_OK;
  return launch_finish(acc, ascale, s1, nullptr, single_out(y, N), nullptr, out_dtype, 1, M, N, as_stream(stream));
}

size_t lq_tile_blob_bytes(int N, int K) {
  if (N <= 0 || K <= 0 || K % 128) return 0;
  return (size_t)((N + 127) / 128) * (size_t)(K / 128) * kTileBytes;
}

int lq_repack_tiles(const uint8_t* src, int src_layout, const uint8_t* s_u8,
                    const uint8_t* offset_a, uint8_t* blob, int N, int K, int group_size,
                    void* stream) {
  if (!src || !s_u8 || !offset_a || !blob || N <= 0 || K <= 0) return LQ_ERR_BAD_ARG;
  if (src_layout != LQ_SRC_CODES && src_layout != LQ_SRC_NIBBLES) return LQ_ERR_BAD_ARG;
  if (K % 128 || group_size < 64 || group_size % 64 || K % group_size) return LQ_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(blob)) % 16) return LQ_ERR_BAD_ARG;
  const long tiles = (long)((N + 127) / 128) * (K / 128);
  long blocks = tiles < (long)sm_count() * 16 ? tiles : (long)sm_count() * 16;
  repack_tiles_kernel<<<(int)blocks, 128, 0, as_stream(stream)>>>(src, src_layout, s_u8, offset_a, blob, N, K,
                                                                 group_size, tiles);
  return check_launch("repack_tiles_kernel");
}

}  // extern "C"
