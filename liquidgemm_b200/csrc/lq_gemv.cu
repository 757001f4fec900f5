// Decode GEMV (M <= 16) of the W4A8 path: HBM-bandwidth bound weight streaming.
//
// Two kernels read the same row-major interleaved pack (byte b of octet h of a row is
// code[8h+b] | code[8h+4+b] << 4, liquidgemm/ops.py:68-75 of the reference):
//
//  * gemv_dp4a_kernel  -- a warp owns R output rows; every lane streams 16-byte pieces of them
//    (32 codes), unpacks with AND / SHR+AND, reconstructs INT8 with one multiply-add and one XOR
//    per four codes, and feeds dp4a.  Several 16-byte loads per lane are in flight before the
//    first is consumed, which is what lets a 2-10 microsecond kernel approach HBM speed.
//  * gemv_mma_kernel   -- for 5..16 tokens the dp4a count outgrows the memory time, so the
//    reconstructed INT8 words are used directly as the A fragment of mma.sync m16n8k32 (a warp
//    owns 16 rows); the k permutation implied by the 16-byte-per-lane loads is applied to the
//    activation fragment as well, so the integer sum is unchanged.
//
// Both produce exact int32 sums and apply (float)acc * ascale[m] * s1[n] before the cast, i.e.
// the result is bit-identical to the reference formula for every M.
#include "lq_common.cuh"

namespace lq {

// pack_nibbles word (code i in nibble i, 8 codes) -> the interleaved form used everywhere else.
__device__ __forceinline__ uint32_t spread4(uint32_t x16) {
  uint32_t t = (x16 | (x16 << 8)) & 0x00FF00FFu;
  return (t | (t << 4)) & 0x0F0F0F0Fu;
}
template <bool PLAIN>
__device__ __forceinline__ void unpack8(uint32_t w, uint32_t& lo, uint32_t& hi) {
  if (PLAIN) {
    lo = spread4(w & 0xFFFFu);
    hi = spread4(w >> 16);
  } else {
    lo = w & 0x0F0F0F0Fu;
    hi = (w >> 4) & 0x0F0F0F0Fu;
  }
}

// Sum V per-lane values over the warp with V - 1 + (5 - log2 V) shuffles: every step halves the
// number of values a lane carries.  Afterwards v[0] of lane L is the total of value
// index_of(L); lanes that differ only in their low (5 - log2 V) bits hold the same total.
template <int V>
__device__ __forceinline__ void warp_sum_many(int (&v)[V], int lane) {
  static_assert(V >= 1 && V <= 32 && (V & (V - 1)) == 0, "V must be a power of two <= 32");
  int off = 16;
#pragma unroll
  for (int cnt = V; cnt > 1; cnt >>= 1) {
    const int half = cnt >> 1;
    const bool upper = (lane & off) != 0;
#pragma unroll
    for (int i = 0; i < half; ++i) {
      const int send = upper ? v[i] : v[i + half];
      const int keep = upper ? v[i + half] : v[i];
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
    }
    off >>= 1;
  }
#pragma unroll
  for (; off > 0; off >>= 1) v[0] += __shfl_xor_sync(0xffffffffu, v[0], off);
}
template <int V>
__device__ __forceinline__ int warp_sum_many_index(int lane) {
  int idx = 0, bit = 16;
#pragma unroll
  for (int cnt = V; cnt > 1; cnt >>= 1) {
    if (lane & bit) idx += cnt >> 1;
    bit >>= 1;
  }
  return idx;
}
template <int V>
__device__ __forceinline__ bool warp_sum_many_writer(int lane) {
  int low_bits = 5;
#pragma unroll
  for (int cnt = V; cnt > 1; cnt >>= 1) --low_bits;
  return (lane & ((1 << low_bits) - 1)) == 0;
}

// MT: tokens held in registers (>= M), R: rows per warp, U: 1024-k steps in flight per lane.
template <int MT, int R, int U, bool PLAIN>
__global__ void __launch_bounds__(256)
gemv_dp4a_kernel(const int8_t* __restrict__ X, const uint8_t* __restrict__ Wp,
                 const uint8_t* __restrict__ s_u8, const uint8_t* __restrict__ off_a,
                 const float* __restrict__ ascale, const float* __restrict__ s1,
                 void* __restrict__ Y, int out_dtype, int M, int N, int K, int G) {
  const int lane = threadIdx.x & 31;
  const long warp = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long n0 = warp * R;
  if (n0 >= N) return;
  const int Kh = K >> 1;

  int acc[R * MT];
#pragma unroll
  for (int i = 0; i < R * MT; ++i) acc[i] = 0;

  for (int base = 0; base < K; base += 1024 * U) {
    uint4 w[U][R];
    uint32_t step[U][R], abc[U][R];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int kc = base + u * 1024 + lane * 32;
      const int g = kc >> 6;
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const long n = n0 + r;
        if (kc < K && n < N) {
          w[u][r] = ldg_stream_v4(Wp + n * Kh + (kc >> 1));
          step[u][r] = __ldg(s_u8 + n * G + g);
          abc[u][r] = __ldg(off_a + n * G + g) * 0x01010101u;
        } else {
          w[u][r] = make_uint4(0, 0, 0, 0);
          step[u][r] = 0;
          abc[u][r] = 0x80808080u;  // reconstructs to zero
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int kc = base + u * 1024 + lane * 32;
      if (kc >= K) continue;
      int wq[R][8];
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const uint32_t pk[4] = {w[u][r].x, w[u][r].y, w[u][r].z, w[u][r].w};
#pragma unroll
        for (int h = 0; h < 4; ++h) {
          uint32_t lo, hi;
          unpack8<PLAIN>(pk[h], lo, hi);
          wq[r][2 * h] = (int)lqq_dequant4(lo, step[u][r], abc[u][r]);
          wq[r][2 * h + 1] = (int)lqq_dequant4(hi, step[u][r], abc[u][r]);
        }
      }
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        if (m < M) {
          const int4* xp = reinterpret_cast<const int4*>(X + (long)m * K + kc);
          const int4 x0 = __ldg(xp), x1 = __ldg(xp + 1);
          const int xs[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
          for (int r = 0; r < R; ++r) {
            int a = acc[r * MT + m];
#pragma unroll
            for (int j = 0; j < 8; ++j) a = __dp4a(xs[j], wq[r][j], a);
            acc[r * MT + m] = a;
          }
        }
      }
    }
  }

  warp_sum_many<R * MT>(acc, lane);
  if (warp_sum_many_writer<R * MT>(lane)) {
    const int idx = warp_sum_many_index<R * MT>(lane);
    const int r = idx / MT, m = idx - r * MT;
    const long n = n0 + r;
    if (m < M && n < N) store_out(Y, (size_t)m * N + n, lqq_scale(acc[0], ascale[m], s1[n]), out_dtype);
  }
}

__device__ __forceinline__ void mma_s8_16x8x32(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// A warp owns 16 rows.  Lane (g = lane/4, q = lane%4) streams rows n0+g and n0+g+8; within a
// 128-k block it owns k = 32q..32q+31 of both rows (one 16-byte load each) and of token g
// (+8 for the second token set).  MMA j of the block (j = 0..3) places the lane's octet
// 32q+8j..+7 in fragment k-slots {4q..4q+3, 16+4q..16+4q+3} for A and B alike.
// TS = token sets of 8 (1 or 2).  U = 128-k blocks in flight per lane.
template <int TS, int U>
__global__ void __launch_bounds__(256)
gemv_mma_kernel(const int8_t* __restrict__ X, const uint8_t* __restrict__ Wp,
                const uint8_t* __restrict__ s_u8, const uint8_t* __restrict__ off_a,
                const float* __restrict__ ascale, const float* __restrict__ s1,
                void* __restrict__ Y, int out_dtype, int M, int N, int K, int G) {
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2, q = lane & 3;
  const long warp = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long n0 = warp * 16;
  if (n0 >= N) return;
  const int Kh = K >> 1;
  const long rowA = n0 + g, rowB = n0 + g + 8;
  const bool okA = rowA < N, okB = rowB < N;
  const uint8_t* wA = Wp + (okA ? rowA : 0) * Kh;
  const uint8_t* wB = Wp + (okB ? rowB : 0) * Kh;
  const uint8_t* sA = s_u8 + (okA ? rowA : 0) * G;
  const uint8_t* sB = s_u8 + (okB ? rowB : 0) * G;
  const uint8_t* oA = off_a + (okA ? rowA : 0) * G;
  const uint8_t* oB = off_a + (okB ? rowB : 0) * G;
  const int8_t* xrow[TS];
  bool xok[TS];
#pragma unroll
  for (int t = 0; t < TS; ++t) {
    xok[t] = (g + 8 * t) < M;
    xrow[t] = X + (long)(xok[t] ? g + 8 * t : 0) * K;
  }

  int acc[TS][4];
#pragma unroll
  for (int t = 0; t < TS; ++t)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[t][i] = 0;

  for (int base = 0; base < K; base += 128 * U) {
    uint4 wa[U], wb[U];
    uint32_t st[U][2], ab[U][2];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int kc = base + u * 128 + q * 32;
      if (kc < K) {
        wa[u] = ldg_stream_v4(wA + (kc >> 1));
        wb[u] = ldg_stream_v4(wB + (kc >> 1));
        const int grp = kc >> 6;
        st[u][0] = __ldg(sA + grp);
        st[u][1] = __ldg(sB + grp);
        ab[u][0] = __ldg(oA + grp) * 0x01010101u;
        ab[u][1] = __ldg(oB + grp) * 0x01010101u;
      } else {
        wa[u] = wb[u] = make_uint4(0, 0, 0, 0);
        st[u][0] = st[u][1] = 0;
        ab[u][0] = ab[u][1] = 0x80808080u;
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int kc = base + u * 128 + q * 32;
      if (base + u * 128 >= K) continue;  // uniform over the warp
      int4 xv[TS][2];
#pragma unroll
      for (int t = 0; t < TS; ++t) {
        if (xok[t]) {
          const int4* xp = reinterpret_cast<const int4*>(xrow[t] + kc);
          xv[t][0] = __ldg(xp);
          xv[t][1] = __ldg(xp + 1);
        } else {
          xv[t][0] = xv[t][1] = make_int4(0, 0, 0, 0);
        }
      }
      const uint32_t pa[4] = {wa[u].x, wa[u].y, wa[u].z, wa[u].w};
      const uint32_t pb[4] = {wb[u].x, wb[u].y, wb[u].z, wb[u].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t a0 = okA ? lqq_dequant4(pa[j] & 0x0F0F0F0Fu, st[u][0], ab[u][0]) : 0u;
        const uint32_t a2 = okA ? lqq_dequant4((pa[j] >> 4) & 0x0F0F0F0Fu, st[u][0], ab[u][0]) : 0u;
        const uint32_t a1 = okB ? lqq_dequant4(pb[j] & 0x0F0F0F0Fu, st[u][1], ab[u][1]) : 0u;
        const uint32_t a3 = okB ? lqq_dequant4((pb[j] >> 4) & 0x0F0F0F0Fu, st[u][1], ab[u][1]) : 0u;
#pragma unroll
        for (int t = 0; t < TS; ++t) {
          const int* xw = reinterpret_cast<const int*>(&xv[t][0]);
          mma_s8_16x8x32(acc[t], a0, a1, a2, a3, (uint32_t)xw[2 * j], (uint32_t)xw[2 * j + 1]);
        }
      }
    }
  }

  // c0,c1: (row g, tokens 2q, 2q+1); c2,c3: (row g+8, same tokens)
#pragma unroll
  for (int t = 0; t < TS; ++t) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int m = 8 * t + 2 * q + (i & 1);
      const long n = (i & 2) ? rowB : rowA;
      if (m < M && n < N) store_out(Y, (size_t)m * N + n, lqq_scale(acc[t][i], ascale[m], s1[n]), out_dtype);
    }
  }
}

// dp4a kernel up to four tokens, warp-MMA kernel above (measured crossover on B200)
template <bool PLAIN>
static int launch_gemv(const int8_t* x, const uint8_t* wp, const uint8_t* s_u8, const uint8_t* off_a,
                       const float* ascale, const float* s1, void* y, int out_dtype, int M, int N,
                       int K, int G, cudaStream_t st) {
  const int warps_per_block = 8;
  const bool use_mma = !PLAIN && M > 4;
  if (use_mma) {
    const long warps = ((long)N + 15) / 16;
    const int blocks = (int)((warps + warps_per_block - 1) / warps_per_block);
    if (M <= 8)
      gemv_mma_kernel<1, 4><<<blocks, 256, 0, st>>>(x, wp, s_u8, off_a, ascale, s1, y, out_dtype, M, N, K, G);
    else
      gemv_mma_kernel<2, 4><<<blocks, 256, 0, st>>>(x, wp, s_u8, off_a, ascale, s1, y, out_dtype, M, N, K, G);
    return check_launch("gemv_mma_kernel");
  }
#define LQ_GEMV_DP4A(MT, R, U)                                                                     \
  {                                                                                                \
    const long warps = ((long)N + (R) - 1) / (R);                                                  \
    const int blocks = (int)((warps + warps_per_block - 1) / warps_per_block);                     \
    gemv_dp4a_kernel<MT, R, U, PLAIN><<<blocks, 256, 0, st>>>(x, wp, s_u8, off_a, ascale, s1, y,   \
                                                              out_dtype, M, N, K, G);              \
  }
  if (M <= 1) LQ_GEMV_DP4A(1, 2, 4)
  else if (M <= 2) LQ_GEMV_DP4A(2, 2, 4)
  else if (M <= 4) LQ_GEMV_DP4A(4, 2, 2)
  else if (M <= 8) LQ_GEMV_DP4A(8, 2, 2)
  else LQ_GEMV_DP4A(16, 2, 1)
#undef LQ_GEMV_DP4A
  return check_launch("gemv_dp4a_kernel");
}

int launch_gemv_plain_f32(const int8_t* x, const uint8_t* nibbles, const uint8_t* s_u8,
                          const uint8_t* off_a, const float* ascale, const float* s1, float* y, int M,
                          int N, int K, int G, cudaStream_t st) {
  return launch_gemv<true>(x, nibbles, s_u8, off_a, ascale, s1, y, LQ_DT_F32, M, N, K, G, st);
}

}  // namespace lq

using namespace lq;

extern "C" int lq_w4a8_gemv(const int8_t* x_i8, const uint8_t* gpack, const uint8_t* s_u8,
                            const uint8_t* offset_a, const float* ascale, const float* s1, void* y,
                            int out_dtype, int M, int N, int K, int group_size, void* stream) {
  if (!x_i8 || !gpack || !s_u8 || !offset_a || !ascale || !s1 || !y) return LQ_ERR_BAD_ARG;
  if (M < 0 || N <= 0 || K <= 0 || out_dtype < 0 || out_dtype > 2) return LQ_ERR_BAD_ARG;
  if (M > 16 || K % 128 || group_size != 64) return LQ_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(x_i8) | reinterpret_cast<uintptr_t>(gpack)) % 16) return LQ_ERR_BAD_ARG;
  if (M == 0) return LQ_OK;
  return launch_gemv<false>(x_i8, gpack, s_u8, offset_a, ascale, s1, y, out_dtype, M, N, K, K / 64,
                            as_stream(stream));
}
