// Decode GEMV over the tile blob (the GEMM's weight format): y[m,n] = scale * sum_k x[m,k] * q^[n,k]
// for 1..8 tokens, replacing the reference's fused GEMV (csrc/liquid_gemm/gemv2.cu:21-120) without a
// second copy of the weights in a GEMV-specific layout.
//
// HBM-bound streaming design:
//  * the (n-tile, k-tile) grid of 8704-byte blob tiles is cut into equal contiguous ranges, one per
//    CTA, two CTAs per SM ("stream-K"): every SM streams the same number of bytes whatever N and K;
//  * one producer thread per CTA keeps a ring of NS tiles in flight with contiguous bulk copies
//    (cp.async.bulk + mbarrier complete_tx), plus one 128-byte copy per token for the activations;
//  * 256 consumer threads: thread (row r, group h) reconstructs the 64 weights of row r in 64-wide
//    group h of the k-tile (AND / SHR+AND / IMAD / XOR on words of 4 lanes) and feeds dp4a against the
//    tokens' words, which every lane reads from shared memory at the same address (broadcast);
//  * the partial sums of an n-tile cut by a range boundary meet in a zeroed workspace word per
//    output element through ONE returning 64-bit atomic add that carries the k-tile count along with
//    the sum; whoever completes the count stores the output and re-zeroes the word.  Integer addition
//    commutes, so the result is bit-identical for every grid size.  A CTA whose range starts inside one
//    tile and ends inside the next issues the atomics of the first tile and reads their results only
//    after its last tile, so their round trip through L2 is hidden behind the stream.
// Every wait is bounded: on expiry the thread records a site code in the status word, stops waiting
// and runs the rest of its control flow (barriers included) so the CTA still exits.

#include <stdint.h>

#include <cstdlib>
#include <mutex>
#include <type_traits>

#include "lq_common.cuh"
#include "lq_sched.cuh"
#include "lq_tc_ptx.cuh"

namespace lq {
namespace gblob {

constexpr int kTileBytes = 8704;   // 4 chunks x [128 rows][16 B] + [128 rows][step0, off0, step1, off1]
constexpr int kConsumers = 256;
constexpr int kThreads = 32 + kConsumers;
constexpr uint64_t kWaitLimitNs = 2000000000ull;
// The wait for tokens gathered from peer GPUs gives up well before the barrier waits of the threads that
// depend on it, so that one late peer is reported once (by the producer) and the rest of the CTA still
// finishes its reduction and leaves the workspace clean.
constexpr uint64_t kPeerWaitLimitNs = 1000000000ull;

struct Args {
  const uint8_t* blob;
  const int8_t* x;       // [M, K]
  const float* ascale;   // [M]
  const float* s1;       // [N]
  void* out;             // [M, N] (single-destination kernels; the others get a MultiOut parameter)
  unsigned long long* slots;   // [grid][MT][128] packed (k-tile count, biased partial sum), zero between launches
  int* status;
  int out_dtype;
  int M, N, K, fixed_split;
  const void* bias;      // [N] in the output dtype, or null
};

template <int MT, int NS>
struct Cfg {
  static constexpr int kXStage = MT * 128;
  static constexpr int kStage = kTileBytes + kXStage;
  static constexpr int kRedBytes = MT * 128 * 4;
  static constexpr int kUsedBytes = 128 + NS * kStage + 2 * NS * 8 + kRedBytes + 16;
  // Never three CTAs on one SM: with programmatic dependent launch the next kernel's CTAs fill whatever
  // fits, and an SM that holds three streams while its neighbour holds one makes the slowest CTA
  // (hence the kernel) much later than the average one.  Asking for more than a third of the SM's
  // shared memory caps residency at two.  (Sizing the CTAs so that four fit, in the hope that the next
  // launch's two CTAs per SM would sit beside this launch's and have their first ring of tiles loaded
  // early, measured 5-30 % slower on every shape: the grids are not all exactly two CTAs per SM, so some
  // SMs end up with three streams of one launch.)
  static constexpr int kSmemBytes = kUsedBytes > 78 * 1024 ? kUsedBytes : 78 * 1024;
};

__device__ __forceinline__ void consumer_barrier() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

__device__ __forceinline__ int dp4a_s8(uint32_t w, uint32_t x, int acc) {
  int d;
  asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(w), "r"(x), "r"(acc));
  return d;
}

template <int MT, int NS, bool MULTI>
__global__ void __launch_bounds__(kThreads, 2)
gemv_blob_kernel(const Args args, const std::conditional_t<MULTI, MultiOut, NoMultiOut> multi) {
  const int kt_total = args.K >> 7;
  using C = Cfg<MT, NS>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 127u) & ~127u;
  uint8_t* smem = smem_raw + (base - raw);

  const uint32_t ws = base;                                // NS weight tiles
  const uint32_t xs = ws + NS * kTileBytes;                // NS token slices [MT][128 B]
  const uint32_t bar_full = xs + NS * C::kXStage;
  const uint32_t bar_empty = bar_full + NS * 8;
  int32_t* red = reinterpret_cast<int32_t*>(smem + (bar_empty + NS * 8 - base));   // [MT][128]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int M = args.M;

  if (threadIdx.x == 0) {
    for (int s = 0; s < NS; ++s) {
      ptx::mbar_init(bar_full + 8 * s, 1);
      ptx::mbar_init(bar_empty + 8 * s, kConsumers);
    }
    ptx::fence_mbar_init();
  }
  __syncthreads();

  allow_dependents();   // the next kernel of the stream may start prefetching its weights

  SchedArgs sa;
  sa.kt_total = kt_total;
  sa.n_tiles = (args.N + 127) >> 7;
  sa.m_tiles = 1;
  sa.fixed_split = args.fixed_split;
  SegmentWalk walk(sa, blockIdx.x, gridDim.x);
  Segment sg;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      // One plain 128-byte copy per token and k-tile.  (A single tensor-map box of MT rows x 128 bytes per
      // k-tile instead was measured: equal at two tokens, 10-15 % slower at four.)
      const uint32_t tx = (uint32_t)(kTileBytes + M * 128);
      Ring<NS> ring;
      int issued = 0;
      bool ok = true;
      // The weights never depend on the previous kernel of the stream, the tokens do: the first NS
      // weight tiles are requested at once, the wait for the previous kernel comes after that, and
      // only then the token slices of those stages.
      int early_kt[NS];
      bool dependency_met = false;
      auto meet_dependency = [&]() {
        dependency_wait();
        if constexpr (MULTI) {
          if (!peer_wait(multi.sync, kPeerWaitLimitNs)) atomicExch(args.status, 303);   // tokens gathered from peers
        }
        dependency_met = true;
        const int n = issued < NS ? issued : NS;
        for (int j = 0; j < n; ++j) {
          const int8_t* xsrc = args.x + (size_t)early_kt[j] * 128;
          for (int m = 0; m < M; ++m)
            ptx::bulk_load(xs + j * C::kXStage + m * 128, xsrc + (size_t)m * args.K, 128, bar_full + 8 * j);
        }
      };
      // (Asking the tiles behind the first ring into L2 with cp.async.bulk.prefetch while the CTA waits for
      // the previous kernel was measured and lost 5-25 %: the requests compete with the demand copies of
      // this ring and of the previous kernel's last CTAs, which are the critical path.)
      while (ok && walk.next(sg)) {
        const uint8_t* src = args.blob + ((size_t)sg.tile * kt_total + sg.kb) * kTileBytes;
        for (int kt = sg.kb; kt < sg.ke; ++kt, src += kTileBytes) {
          if (issued == NS) meet_dependency();
          if (!ptx::mbar_wait_bounded(bar_empty + 8 * ring.s, ring.ph ^ 1u, kWaitLimitNs)) {
            atomicExch(args.status, 301);
            ok = false;
            break;
          }
          const uint32_t full = bar_full + 8 * ring.s;
          ptx::mbar_expect_tx(full, tx);
          ptx::bulk_load(ws + ring.s * kTileBytes, src, kTileBytes, full);
          if (issued < NS) {
            early_kt[issued] = kt;
          } else {
            const int8_t* xsrc = args.x + (size_t)kt * 128;
            for (int m = 0; m < M; ++m)
              ptx::bulk_load(xs + ring.s * C::kXStage + m * 128, xsrc + (size_t)m * args.K, 128, full);
          }
          ring.advance();
          ++issued;
        }
      }
      if (!dependency_met) meet_dependency();
      // Copies in flight write shared memory: they must have landed before the CTA may exit.  On
      // the normal path the consumers have waited for every one of them already.
      const int pending = issued < NS ? issued : NS;
      for (int j = 0; j < pending; ++j) {
        const int i = issued - pending + j;
        ptx::mbar_wait_bounded(bar_full + 8 * (i % NS), (uint32_t)(i / NS) & 1u, kWaitLimitNs);
      }
    }
  } else {
    // ------------------------------------------------------------------ consumers
    const int c = threadIdx.x - 32;
    const int row = c & 127;
    const int h = c >> 7;   // 64-wide group of the k-tile handled by this thread
    const uint32_t w_off = (uint32_t)((2 * h) * 128 + row) * 16;
    const uint32_t meta_off = 8192u + (uint32_t)row * 4 + 2 * h;
    Ring<NS> ring;
    bool ok = true;
    dependency_wait();   // outputs, the reduction workspace and the tokens belong to earlier kernels until here
    const bool has_bias = args.bias != nullptr;
    auto emit = [&](long m, long n, float v, float bias) {
      if constexpr (MULTI) store_out_all(multi.out, m, n, v, bias, has_bias, args.out_dtype);
      else store_out_bias(args.out, (size_t)m * args.N + n, v, bias, has_bias, args.out_dtype);
    };
    float a_scale[MT];   // token scales: read once, they are needed right after the last tile
#pragma unroll
    for (int m = 0; m < MT; ++m) a_scale[m] = (m < M) ? __ldg(args.ascale + m) : 0.f;

    // A partial segment whose atomics are in flight while the CTA streams its next segment.
    bool pend = false;
    unsigned long long pend_old[MT];
    int pend_acc[MT];
    long pend_n = 0;
    long long pend_nk = 0;
    float pend_w = 0.f;
    unsigned long long* pend_slot = nullptr;
    // The thread whose add completed the tile's k-tile count holds the full sum in the value it got back:
    // it re-zeroes the word and stores the output.
    auto finish_partial = [&](const unsigned long long (&old)[MT], const int (&part)[MT], long n, long long nk,
                              float w_scale, unsigned long long* slot) {
      const float bias = has_bias ? load_bias(args.bias, n, args.out_dtype) : 0.f;
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        if (m < M && (long long)(old[m] >> 40) + nk == (long long)kt_total) {
          const long long total = (long long)(old[m] & ((1ull << 40) - 1)) + (long long)part[m] + (nk << 21) -
                                  ((long long)kt_total << 21);
          __stcg(slot + m * 128 + row, 0ull);
          emit(m, n, lqq_scale((int)total, a_scale[m], w_scale), bias);
        }
      }
    };

    while (walk.next(sg)) {
      const long n = (long)sg.tile * 128 + row;
      const float w_scale = (n < args.N) ? __ldg(args.s1 + n) : 0.f;   // a weight: fetched ahead of the loop
      int acc[MT];
#pragma unroll
      for (int m = 0; m < MT; ++m) acc[m] = 0;

#pragma unroll 1
      for (int kt = sg.kb; kt < sg.ke; ++kt) {
        if (ok && !ptx::mbar_wait_bounded(bar_full + 8 * ring.s, ring.ph, kWaitLimitNs)) {
          atomicExch(args.status, 302);
          ok = false;
        }
        const uint8_t* wst = smem + (ws - base) + ring.s * kTileBytes;
        const uint4 c0 = *reinterpret_cast<const uint4*>(wst + w_off);
        const uint4 c1 = *reinterpret_cast<const uint4*>(wst + w_off + 2048);
        const uint32_t meta = *reinterpret_cast<const uint16_t*>(wst + meta_off);
        const uint32_t step = meta & 0xffu;
        const uint32_t ab = (meta >> 8) * 0x01010101u;
        const uint32_t pk[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
        uint32_t v[16];   // v[2j], v[2j+1]: weights k = 8j..8j+3, 8j+4..8j+7 of the group
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          v[2 * j] = lqq_dequant4(pk[j] & 0x0F0F0F0Fu, step, ab);
          v[2 * j + 1] = lqq_dequant4((pk[j] >> 4) & 0x0F0F0F0Fu, step, ab);
        }
        const uint8_t* xst = smem + (xs - base) + ring.s * C::kXStage + 64 * h;
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          const uint4* xp = reinterpret_cast<const uint4*>(xst + m * 128);
          int a = acc[m], b = 0;   // two chains: dp4a latency, not issue, would bound one
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const uint4 xv = xp[q];
            a = dp4a_s8(v[4 * q], xv.x, a);
            b = dp4a_s8(v[4 * q + 1], xv.y, b);
            a = dp4a_s8(v[4 * q + 2], xv.z, a);
            b = dp4a_s8(v[4 * q + 3], xv.w, b);
          }
          acc[m] = a + b;
        }
        ptx::mbar_arrive(bar_empty + 8 * ring.s);
        ring.advance();
      }

      // ---- reduce the two k-groups of every row, then finish or publish the partial sums
      if (h == 1) {
#pragma unroll
        for (int m = 0; m < MT; ++m) red[m * 128 + row] = acc[m];
      }
      consumer_barrier();
      const bool mine = (h == 0) && n < args.N;
      if (h == 0) {
#pragma unroll
        for (int m = 0; m < MT; ++m) acc[m] += red[m * 128 + row];
      }
      if (sg.whole) {
        if (mine) {
          const float bias = has_bias ? load_bias(args.bias, n, args.out_dtype) : 0.f;
#pragma unroll
          for (int m = 0; m < MT; ++m)
            if (m < M) emit(m, n, lqq_scale(acc[m], a_scale[m], w_scale), bias);
        }
      } else if (mine) {
        // One returning 64-bit atomic per element does the whole cross-CTA reduction: the word holds
        // the number of k-tiles added so far (bits 40..) and the sum of the contributions, each
        // biased by 2^21 per k-tile so that it is non-negative and never borrows from the count:
        // no fence, no counter, no read-back.
        unsigned long long* slot = args.slots + (size_t)sg.slot * (MT * 128);
        const long long nk = sg.ke - sg.kb;
        unsigned long long old[MT];
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          const unsigned long long add = (unsigned long long)((long long)acc[m] + (nk << 21)) |
                                         ((unsigned long long)nk << 40);
          old[m] = (m < M) ? atomicAdd(slot + m * 128 + row, add) : 0ull;
        }
        if (walk.has_more() && !pend) {
          // more tiles follow: look at the returned values after them
          pend = true;
#pragma unroll
          for (int m = 0; m < MT; ++m) {
            pend_old[m] = old[m];
            pend_acc[m] = acc[m];
          }
          pend_n = n;
          pend_nk = nk;
          pend_w = w_scale;
          pend_slot = slot;
        } else {
          finish_partial(old, acc, n, nk, w_scale, slot);
        }
      }
      consumer_barrier();   // `red` may be rewritten by the next segment
    }
    if (pend) finish_partial(pend_old, pend_acc, pend_n, pend_nk, pend_w, pend_slot);
    if constexpr (MULTI) {
      // Every output store of this CTA, including those into peer memory, is ordered before the flags:
      // the barrier makes the other threads' stores visible to thread 0 (CTA scope), and the release of
      // its system-scope reduction is cumulative over them.
      consumer_barrier();
      if (c == 0) {
        peer_signal(multi.sync);   // red.release.sys: ordered after everything the barrier made visible
      }
    }
  }
  __syncthreads();
}

template <int MT, int NS, bool MULTI>
static int launch(const Args& a, const MultiOut* multi, int grid, cudaStream_t st) {
  using C = Cfg<MT, NS>;
  auto kern = &gemv_blob_kernel<MT, NS, MULTI>;
  static std::once_flag once[64];
  int dev = 0;
  cudaGetDevice(&dev);
  cudaError_t e = cudaSuccess;
  std::call_once(once[dev & 63], [&]() {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
  });
  if (e != cudaSuccess) {
    record_cuda_error(e, "cudaFuncSetAttribute(gemv_blob_kernel)");
    return LQ_ERR_CUDA;
  }
  if constexpr (MULTI) e = launch_overlapped(kern, dim3(grid), dim3(kThreads), (size_t)C::kSmemBytes, st, a, *multi);
  else e = launch_overlapped(kern, dim3(grid), dim3(kThreads), (size_t)C::kSmemBytes, st, a, NoMultiOut{});
  if (e != cudaSuccess) {
    record_cuda_error(e, "gemv_blob_kernel launch");
    return LQ_ERR_CUDA;
  }
  return check_launch("gemv_blob_kernel");
}

static DecodePlan plan_for(int N, int K) { return decode_plan((N + 127) / 128, K / 128, 2 * sm_count(), false); }
static int grid_for(int N, int K) { return plan_for(N, K).grid; }

}  // namespace gblob

// Workspace bytes for a launch grid of `grid` CTAs: one 64-bit word per (token <= 8, row) of a slot.
static size_t gemv_blob_ws_bytes(int grid) { return (size_t)grid * (8 * 128 * 8); }

int gemv_blob_grid(int N, int K) { return gblob::grid_for(N, K); }   // CTAs a launch of this shape uses

size_t gemv_blob_workspace_bytes(int N, int K) {
  (void)N;
  (void)K;
  return gemv_blob_ws_bytes(2 * sm_count());   // one slot per resident CTA
}

// Same call with a size-checked workspace, for the GEMM entry points.
int run_gemv_blob_ws(const int8_t* x, const uint8_t* blob, const float* ascale, const float* s1, const void* bias,
                     const OutSpec& out, const PeerSync* sync, int out_dtype, int M, int N, int K, void* ws,
                     size_t ws_bytes, cudaStream_t st);

int run_gemv_blob(const int8_t* x, const uint8_t* blob, const float* ascale, const float* s1, const void* bias,
                  const OutSpec& out, const PeerSync* sync, int out_dtype, int M, int N, int K,
                  unsigned long long* slots, cudaStream_t st) {
  using namespace gblob;
  Args a;
  a.blob = blob;
  a.x = x;
  a.ascale = ascale;
  a.s1 = s1;
  // one plain destination with nothing to signal or wait for: the small-parameter kernels
  const bool multi = out.n != 1 || out.ld != N || out.col0 != 0 || (sync && (sync->n_signal > 0 || sync->wait));
  a.out = out.ptr[0];
  a.slots = slots;
  a.status = status_word();
  a.out_dtype = out_dtype;
  a.M = M;
  a.N = N;
  a.K = K;
  a.fixed_split = plan_for(N, K).fixed_split;
  a.bias = bias;
  if (!a.status) return LQ_ERR_CUDA;
  const int grid = grid_for(N, K);
  if (!multi) {
    if (M <= 1) return launch<1, 8, false>(a, nullptr, grid, st);
    if (M <= 2) return launch<2, 8, false>(a, nullptr, grid, st);
    if (M <= 4) return launch<4, 8, false>(a, nullptr, grid, st);
    return launch<8, 7, false>(a, nullptr, grid, st);
  }
  MultiOut mo;
  mo.out = out;
  mo.sync = sync ? *sync : PeerSync{};
  if (M <= 1) return launch<1, 8, true>(a, &mo, grid, st);
  if (M <= 2) return launch<2, 8, true>(a, &mo, grid, st);
  if (M <= 4) return launch<4, 8, true>(a, &mo, grid, st);
  return launch<8, 7, true>(a, &mo, grid, st);
}

int run_gemv_blob_ws(const int8_t* x, const uint8_t* blob, const float* ascale, const float* s1, const void* bias,
                     const OutSpec& out, const PeerSync* sync, int out_dtype, int M, int N, int K, void* ws,
                     size_t ws_bytes, cudaStream_t st) {
  const int grid = gblob::grid_for(N, K);
  if (!ws || ws_bytes < gemv_blob_ws_bytes(grid)) return LQ_ERR_WORKSPACE;
  return run_gemv_blob(x, blob, ascale, s1, bias, out, sync, out_dtype, M, N, K,
                       static_cast<unsigned long long*>(ws), st);
}

}  // namespace lq

using namespace lq;

extern "C" {

LQ_API size_t lq_gemv_blob_workspace_bytes(void) { return gemv_blob_ws_bytes(2 * sm_count()); }

LQ_API int lq_w4a8_gemv_blob(const void* x_i8, const void* blob, const void* ascale, const void* s1, void* out,
                             int out_dtype, int M, int N, int K, void* workspace, size_t workspace_bytes,
                             void* stream) {
  if (!x_i8 || !blob || !ascale || !s1 || !out) return LQ_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(x_i8) | reinterpret_cast<uintptr_t>(blob)) & 15u) return LQ_ERR_BAD_ARG;
  if (out_dtype < LQ_DT_BF16 || out_dtype > LQ_DT_F32) return LQ_ERR_BAD_ARG;
  if (M < 1 || M > 8 || N < 1 || K < 128 || K % 128) return LQ_ERR_SHAPE;
  const int grid = gblob::grid_for(N, K);
  if (!workspace || workspace_bytes < gemv_blob_ws_bytes(grid)) return LQ_ERR_WORKSPACE;
  return run_gemv_blob(static_cast<const int8_t*>(x_i8), static_cast<const uint8_t*>(blob),
                       static_cast<const float*>(ascale), static_cast<const float*>(s1), nullptr, single_out(out, N),
                       nullptr, out_dtype, M, N, K, static_cast<unsigned long long*>(workspace), as_stream(stream));
}

// ---------------------------------------------------------------------------------------------
// The same GEMV with its reduction scratch inside the library image instead of a caller buffer.
// ---------------------------------------------------------------------------------------------
}  // extern "C"

namespace lq {
namespace gblob {

// Room for 512 CTAs (two per SM on up to 256 SMs): 512 x (8 tokens x 128 rows x 8 B) reduction
// words, 4 194 304 bytes of device memory that exist as long as the library is loaded.  The loader
// zero-fills it; every kernel that completes leaves it zero-filled.
constexpr int kStaticMaxCtas = 512;
constexpr size_t kStaticBytes = (size_t)kStaticMaxCtas * 8 * 128 * 8;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticBytes];

static void* g_static_ptr[64];
static cudaError_t g_static_err[64];
static std::once_flag g_static_once[64];

// First use on a device (that device current): resolve the array's address and clear it once.  The host
// name `g_static_scratch` is only a handle for the runtime; the kernel needs the device address that
// cudaGetSymbolAddress returns for the current device.  cudaMemset on device memory returns before the
// fill has run and is ordered only against the legacy default stream, so the set-up ends with a device-wide
// synchronise: when it returns the array is zero for a kernel on ANY stream, blocking or not.
static void* static_scratch_for_current_device() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::call_once(g_static_once[dev], [dev]() {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e == cudaSuccess) e = cudaMemset(p, 0, kStaticBytes);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    g_static_err[dev] = e;
    g_static_ptr[dev] = e == cudaSuccess ? p : nullptr;
    if (e != cudaSuccess) record_cuda_error(e, "static GEMV scratch set-up");
  });
  return g_static_ptr[dev];
}

}  // namespace gblob
}  // namespace lq

extern "C" {

LQ_API int lq_w4a8_gemv_blob_static(const void* x_i8, const void* blob, const void* ascale, const void* s1,
                                    void* out, int out_dtype, int M, int N, int K, void* stream) {
  if (!x_i8 || !blob || !ascale || !s1 || !out) return LQ_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(x_i8) | reinterpret_cast<uintptr_t>(blob)) & 15u) return LQ_ERR_BAD_ARG;
  if (out_dtype < LQ_DT_BF16 || out_dtype > LQ_DT_F32) return LQ_ERR_BAD_ARG;
  if (M < 1 || M > 8 || N < 1 || K < 128 || K % 128) return LQ_ERR_SHAPE;
  const int grid = gblob::grid_for(N, K);
  if (grid > gblob::kStaticMaxCtas) {
    record_cuda_error(cudaErrorInvalidValue,
                      "lq_w4a8_gemv_blob_static: the built-in scratch holds 512 CTAs (devices up to 256 SMs)");
    return LQ_ERR_WORKSPACE;
  }
  void* p = gblob::static_scratch_for_current_device();
  if (!p) return LQ_ERR_CUDA;
  return run_gemv_blob(static_cast<const int8_t*>(x_i8), static_cast<const uint8_t*>(blob),
                       static_cast<const float*>(ascale), static_cast<const float*>(s1), nullptr, single_out(out, N),
                       nullptr, out_dtype, M, N, K, static_cast<unsigned long long*>(p), as_stream(stream));
}

// Clears the built-in scratch of the current device on `stream` (a cudaMemsetAsync: nothing is allocated,
// nothing is synchronised).  Needed only after a call whose kernel gave up a bounded wait (lq_poll_status
// returned LQ_ERR_TIMEOUT): such a kernel can leave partial sums behind, and every later call would add to them.
LQ_API int lq_w4a8_gemv_blob_static_reset(void* stream) {
  void* p = gblob::static_scratch_for_current_device();
  if (!p) return LQ_ERR_CUDA;
  cudaError_t e = cudaMemsetAsync(p, 0, gblob::kStaticBytes, as_stream(stream));
  if (e != cudaSuccess) {
    record_cuda_error(e, "lq_w4a8_gemv_blob_static_reset");
    return LQ_ERR_CUDA;
  }
  return LQ_OK;
}

}  // extern "C"
