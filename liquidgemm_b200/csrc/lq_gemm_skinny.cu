// W4A8 tensor-core GEMM for decode batches (M <= 128 tokens): HBM-bound, so built like a streaming
// copy with tensor cores attached.  Replaces the reference's split-K WGMMA path for small M
// (csrc/liquid_gemm/w4a8_wgmma.cu:333-503 with the split rule at :523-534 and the finish kernel :39-56).
//
//  * Work = the (n-tile, k-tile) grid of 8704-byte blob tiles, cut into equal contiguous ranges, one
//    per CTA, two CTAs per SM (stream-K): every SM streams the same number of weight bytes whatever
//    N and K are, in ONE launch (no second reduction kernel).
//  * warp 0  producer: one thread keeps a ring of NS stages in flight: a contiguous bulk copy of the
//            weight tile and a 128-byte-swizzled tensor-map box of the BN x 128 token slice.
//  * warps 2..9  two dequant sets taking alternate k-tiles; thread r of a set owns weight row r:
//            64 bytes of nibbles -> 128 INT8 (AND / SHR+AND / IMAD / XOR on 4-lane words) ->
//            tcgen05.st into tensor-memory lane r (the MMA's A operand, 4 consecutive k per column).
//  * warp 1  MMA: one thread issues four 128 x BN x 32 tcgen05.mma kind::i8 per k-tile (A from tensor
//            memory, B = tokens through a shared-memory descriptor); its commit recycles the stage.
//            A single CTA cannot issue these faster than one per ~94 cycles, two CTAs per SM overlap.
//  * Epilogue by the dequant warps: tcgen05.ld (lane = channel, column = token); a segment that
//    covers its tile's whole K is scaled and stored directly; otherwise the partial sums of the CTAs
//    that share the tile meet in a zeroed workspace word per output element through ONE returning
//    64-bit atomic add that carries the k-tile count along with the sum, and whoever completes the
//    count stores the output and re-zeroes the word.  Integer sums are exact in any order.
//  * Launched with programmatic stream serialisation: weight tiles are requested before the wait for
//    the previous kernel of the stream, tokens / outputs / workspace are touched only after it.
// Every wait is bounded; a thread whose wait expires records a site code, stops waiting and still
// runs the rest of its control flow, so the CTA reaches the exit where tensor memory is released.

#include <cuda.h>
#include <stdint.h>

#include <cstdlib>
#include <mutex>
#include <type_traits>

#ifndef LQ_SKINNY_SETS
#define LQ_SKINNY_SETS 2
#endif

#include "lq_common.cuh"
#include "lq_sched.cuh"
#include "lq_tc_ptx.cuh"

namespace lq {

int make_byte_matrix_map(CUtensorMap* map, const void* ptr, long rows, long row_bytes, int box_rows,
                         int box_bytes);   // lq_gemm_tc.cu

namespace skinny {

constexpr int kTileBytes = 8704;
constexpr int kSets = LQ_SKINNY_SETS;       // dequant sets of 128 threads, taking k-tiles round-robin
constexpr int kDequant = 128 * kSets;
constexpr int kThreads = 64 + kDequant;
constexpr uint64_t kWaitLimitNs = 2000000000ull;
constexpr int kOutI32 = 3;

struct Args {
  const uint8_t* blob;
  const float* ascale;   // [M]
  const float* s1;       // [N]
  void* out;             // [M, N] (single-destination kernels; the others get a MultiOut parameter)
  unsigned long long* slots;   // [grid][BN][128] packed (k-tile count, biased partial sum), zero between launches
  int* status;
  int out_mode;          // LQ_DT_* or kOutI32
  int M, N, K, fixed_split;
  long long* trace;      // pipeline studies: [grid][4] globaltimer stamps, or null
  int debug_skip;        // pipeline studies only (results become wrong): 1 no tcgen05.st, 2 no MMA, 4 no dequant ALU
};

// One ring of NS stages couples shared memory (weight tile + token box) and the tensor-memory operand
// stage: three barriers per k-tile (full, operand ready, empty) is the cheapest protocol measured;
// every extra handshake per k-tile costs more than the buffer space it frees earlier.  Measured on
// B200: about 70-100 KB of copies in flight per SM saturate HBM, deeper rings are slower.
template <int BN, int NS>
struct Cfg {
  static constexpr int kXStage = BN * 128;
  static constexpr int kACols = 32 * NS;   // one operand stage per shared-memory stage
  static constexpr int kColsNeeded = BN + kACols;
  static constexpr int kTmemCols = kColsNeeded <= 128 ? 128 : kColsNeeded <= 256 ? 256 : 512;
  static constexpr int kNumBars = 3 * NS + 2;
  static constexpr int kUsedBytes = 1024 + NS * (kXStage + kTileBytes) + kNumBars * 8 + 16;
  // more than a third of the SM's shared memory, so that never three CTAs (of this and of the next
  // kernel, under programmatic dependent launch) share an SM while another SM holds one
  static constexpr int kSmemBytes = kUsedBytes > 78 * 1024 ? kUsedBytes : 78 * 1024;
  static_assert(kColsNeeded <= 256, "two CTAs per SM share 512 tensor-memory columns");
  static_assert(kSmemBytes <= 113 * 1024, "two CTAs per SM share the shared memory");
};


template <int BN, int NS, bool MULTI>
__global__ void __launch_bounds__(kThreads, 2)
w4a8_skinny_kernel(const __grid_constant__ CUtensorMap tmap_x, const Args args,
                   const std::conditional_t<MULTI, MultiOut, NoMultiOut> multi) {
  const int kt_total = args.K >> 7;
  using C = Cfg<BN, NS>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);

  const uint32_t xs = base;                          // NS token boxes (1024-aligned for the swizzle)
  const uint32_t ws = xs + NS * C::kXStage;          // NS weight tiles
  const uint32_t bar_full = ws + NS * kTileBytes;    // [NS] both copies of the stage landed
  const uint32_t bar_empty = bar_full + NS * 8;      // [NS] the stage's MMAs are done
  const uint32_t bar_aready = bar_empty + NS * 8;    // [NS] dequantised operand is in tensor memory
  const uint32_t bar_accfull = bar_aready + NS * 8;  // the segment's accumulator is final
  const uint32_t bar_accfree = bar_accfull + 8;      // the accumulator has been read
  const uint32_t tmem_slot = bar_accfree + 8;
  volatile uint32_t* tmem_slot_p = reinterpret_cast<volatile uint32_t*>(smem + (tmem_slot - base));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < NS; ++s) {
      ptx::mbar_init(bar_full + 8 * s, 1);
      ptx::mbar_init(bar_empty + 8 * s, 1);
      ptx::mbar_init(bar_aready + 8 * s, 128);
    }
    ptx::mbar_init(bar_accfull, 1);
    ptx::mbar_init(bar_accfree, kDequant);
    ptx::fence_mbar_init();
    ptx::prefetch_tensormap(&tmap_x);
  }
  __syncthreads();
  allow_dependents();   // the next kernel of the stream may start prefetching its weights

  SegmentWalk walk(SchedArgs{kt_total, (args.N + 127) >> 7, 1, args.fixed_split}, blockIdx.x, gridDim.x);
  Segment sg;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      constexpr uint32_t kTx = (uint32_t)(kTileBytes + C::kXStage);
      Ring<NS> ring;
      int issued = 0;
      bool ok = true;
      long long p_wait = 0;
      // Weight tiles do not depend on the previous kernel of the stream, the tokens do: the first NS
      // weight tiles are requested at once, then comes the wait for the previous kernel, then the
      // token boxes of those stages.
      int early_kt[NS];
      bool dependency_met = false;
      auto meet_dependency = [&]() {
        dependency_wait();
        if constexpr (MULTI) {
          if (!peer_wait(multi.sync, kWaitLimitNs)) atomicExch(args.status, 409);   // tokens gathered from peers
        }
        dependency_met = true;
        const int n = issued < NS ? issued : NS;
        for (int j = 0; j < n; ++j)
          ptx::tensor_load_2d(xs + j * C::kXStage, &tmap_x, early_kt[j] * 128, 0, bar_full + 8 * j);
      };
      while (ok && walk.next(sg)) {
        const uint8_t* src = args.blob + ((size_t)sg.tile * kt_total + sg.kb) * kTileBytes;
        for (int kt = sg.kb; kt < sg.ke; ++kt, src += kTileBytes) {
          if (issued == NS) meet_dependency();
          const long long p0 = args.trace ? clock64() : 0;
          if (!ptx::mbar_wait_bounded(bar_empty + 8 * ring.s, ring.ph ^ 1u, kWaitLimitNs)) {
            atomicExch(args.status, 401);
            ok = false;
            break;
          }
          if (args.trace) p_wait += clock64() - p0;
          const uint32_t full = bar_full + 8 * ring.s;
          ptx::mbar_expect_tx(full, kTx);
          ptx::bulk_load(ws + ring.s * kTileBytes, src, kTileBytes, full);
          if (issued < NS) early_kt[issued] = kt;
          else ptx::tensor_load_2d(xs + ring.s * C::kXStage, &tmap_x, kt * 128, 0, full);
          ring.advance();
          ++issued;
        }
      }
      if (!dependency_met) meet_dependency();
      if (args.trace) args.trace[blockIdx.x * 8 + 7] = p_wait;
      // Copies in flight write shared memory: they must have landed before the CTA may exit.
      const int pending = issued < NS ? issued : NS;
      for (int j = 0; j < pending; ++j) {
        const int i = issued - pending + j;
        ptx::mbar_wait_bounded(bar_full + 8 * (i % NS), (uint32_t)(i / NS) & 1u, kWaitLimitNs);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ tensor memory + MMA issue
    ptx::tmem_alloc(tmem_slot, C::kTmemCols);
    ptx::tmem_relinquish();
    ptx::tc_fence_before();
    asm volatile("bar.sync 2, %0;" ::"n"(32 + kDequant) : "memory");   // publishes the allocation to the dequant warps
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot_p;
    const uint32_t tmem_acc = tmem_base;
    const uint32_t tmem_a = tmem_base + BN;
    if (lane == 0) {
      constexpr uint32_t idesc = ptx::idesc_i8(BN);
      Ring<NS> ring;
      bool ok = true;
      uint32_t seg = 0;
      while (walk.next(sg)) {
        if (seg > 0 && ok && !ptx::mbar_wait_bounded(bar_accfree, (seg - 1) & 1u, kWaitLimitNs)) {
          atomicExch(args.status, 402);
          ok = false;
        }
        for (int kt = sg.kb; kt < sg.ke; ++kt) {
          // "operand ready" implies "token box landed": the dequant set saw the stage's full barrier
          if (ok && !ptx::mbar_wait_bounded(bar_aready + 8 * ring.s, ring.ph, kWaitLimitNs)) {
            atomicExch(args.status, 403);
            ok = false;
          }
          ptx::tc_fence_after();
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint64_t bdesc = ptx::smem_desc_sw128(xs + ring.s * C::kXStage + j * 32);
            if (!(args.debug_skip & 2))
              ptx::mma_i8_ts(tmem_acc, tmem_a + ring.s * 32 + j * 8, bdesc, idesc, (kt > sg.kb || j > 0) ? 1u : 0u);
          }
          ptx::tc_commit(bar_empty + 8 * ring.s);
          ring.advance();
        }
        ptx::tc_commit(bar_accfull);
        ++seg;
      }
    }
    __syncwarp();
    // tensor memory is released after every role is done
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, C::kTmemCols);
    return;
  } else {
    // ------------------------------------------------------------------ dequant sets, then epilogue
    const int d = threadIdx.x - 64;
    const int set = d >> 7;                   // takes the k-tiles whose running index is set (mod kSets)
    const int quad = warp & 3;                // tensor-memory lane quadrant this warp may access
    const int row = quad * 32 + lane;         // weight row inside the tile == tensor-memory lane
    const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
    asm volatile("bar.sync 2, %0;" ::"n"(32 + kDequant) : "memory");
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot_p;
    const uint32_t tmem_acc = tmem_base + lane_addr;
    const uint32_t tmem_a = tmem_base + BN + lane_addr;
    Ring<NS> ring;
    bool ok = true;
    uint32_t step = 0;   // running k-tile index of this CTA
    uint32_t seg = 0;
    bool waited_dependency = false;
    const bool tracing = args.trace != nullptr && d == 0;
    long long e_wait = 0, e_load = 0, e_store = 0, d_wait = 0;
    bool first = true;
    if (tracing) args.trace[blockIdx.x * 8 + 0] = (long long)ptx::globaltimer_ns();

    while (walk.next(sg)) {
      // the channel scale is a weight: fetch it now, it is needed right after the last MMA
      const long n = (long)sg.tile * 128 + row;
      const bool n_ok = n < args.N;
      const bool scaled = args.out_mode != kOutI32;
      const float w_scale = (n_ok && scaled) ? __ldg(args.s1 + n) : 0.f;
#pragma unroll 1
      for (int kt = sg.kb; kt < sg.ke; ++kt, ++step, ring.advance()) {
        if ((int)(step % (uint32_t)kSets) != set) continue;
        const long long w0 = tracing ? clock64() : 0;
        if (ok && !ptx::mbar_wait_bounded(bar_full + 8 * ring.s, ring.ph, kWaitLimitNs)) {
          atomicExch(args.status, 404);
          ok = false;
        }
        if (tracing) d_wait += clock64() - w0;
        if (first) {
          // The stage holds tokens, so the producer is past its wait for the previous kernel: pull the
          // token scales (that kernel's output) into L1 now, the epilogue reads them under time pressure.
          if (tracing) args.trace[blockIdx.x * 8 + 1] = (long long)ptx::globaltimer_ns();
          first = false;
          dependency_wait();
          waited_dependency = true;
          if (scaled && d * 32 < args.M) asm volatile("prefetch.global.L1 [%0];" ::"l"(args.ascale + d * 32));
        }
        const uint8_t* wst = smem + (ws - base) + ring.s * kTileBytes;
        uint4 ch[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) ch[c] = *reinterpret_cast<const uint4*>(wst + (c * 128 + row) * 16);
        const uint32_t meta = *reinterpret_cast<const uint32_t*>(wst + 8192 + row * 4);
        __syncwarp();   // lanes leave the poll loop one by one; tcgen05.st / wait::st need the warp converged
        const uint32_t step0 = meta & 0xffu, a0 = ((meta >> 8) & 0xffu) * 0x01010101u;
        const uint32_t step1 = (meta >> 16) & 0xffu, a1 = (meta >> 24) * 0x01010101u;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const uint32_t st = c < 2 ? step0 : step1;
          const uint32_t ab = c < 2 ? a0 : a1;
          const uint32_t pk[4] = {ch[c].x, ch[c].y, ch[c].z, ch[c].w};
          uint32_t v[8];
#pragma unroll
          for (int h = 0; h < 4; ++h) {
            if (args.debug_skip & 4) {
              v[2 * h] = pk[h];
              v[2 * h + 1] = pk[h] + st;
            } else {
              v[2 * h] = lqq_dequant4(pk[h] & 0x0F0F0F0Fu, st, ab);
              v[2 * h + 1] = lqq_dequant4((pk[h] >> 4) & 0x0F0F0F0Fu, st, ab);
            }
          }
          if (!(args.debug_skip & 1)) ptx::tmem_st8(tmem_a + ring.s * 32 + c * 8, v);
          else if (v[0] + v[3] == 0x12345u) atomicExch(args.status, 499);
        }
        ptx::tc_wait_st();
        ptx::tc_fence_before();
        ptx::mbar_arrive(bar_aready + 8 * ring.s);
      }

      if (tracing) args.trace[blockIdx.x * 8 + 2] = (long long)ptx::globaltimer_ns();   // last dequant done
      // ---- epilogue of the segment: set g takes the 16-column chunks g, g+2, ...
      const long long e0 = tracing ? clock64() : 0;
      if (ok && !ptx::mbar_wait_bounded(bar_accfull, seg & 1u, kWaitLimitNs)) {
        atomicExch(args.status, 405);
        ok = false;
      }
      __syncwarp();
      ptx::tc_fence_after();
      if (!waited_dependency) {
        dependency_wait();   // outputs and the reduction workspace belong to earlier kernels until here
        waited_dependency = true;
      }
      unsigned long long* slot = args.slots + (size_t)sg.slot * (BN * 128);
      const long long nk = sg.ke - sg.kb;
      const long long e1 = tracing ? clock64() : 0;
      long long e2 = e1;
#pragma unroll 1
      for (int c0 = set * 16; c0 < BN; c0 += 16 * kSets) {
        if (c0 >= args.M) break;   // uniform over the warp
        int v[16];
        ptx::tmem_ld16(tmem_acc + c0, v);
        ptx::tc_wait_ld();
        if (c0 + 16 * kSets >= BN || c0 + 16 * kSets >= args.M) {   // last chunk of this set: the accumulator may be reused
          __syncwarp();
          ptx::tc_fence_before();
          ptx::mbar_arrive(bar_accfree);
        }
        if (!n_ok) continue;
        float sc[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) sc[j] = (scaled && c0 + j < args.M) ? __ldg(args.ascale + c0 + j) : 0.f;
        if (tracing) {
          if (sc[0] == 123.456f) atomicExch(args.status, 498);   // forces the loads to complete here
          e2 = clock64();
        }
        if (!sg.whole) {
          // One returning 64-bit atomic per element does the cross-CTA reduction: the word holds the
          // k-tiles added so far (bits 40..) and the sum of the contributions, each biased by 2^21 per
          // k-tile so that it is non-negative and never borrows from the count.  The thread whose add
          // completes the tile's count holds the full sum in the value it got back: it stores the
          // output and re-zeroes the word.  No fence, no counter, no read-back.
          unsigned long long old[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const unsigned long long add = (unsigned long long)((long long)v[j] + (nk << 21)) |
                                           ((unsigned long long)nk << 40);
            old[j] = (c0 + j < args.M) ? atomicAdd(slot + (c0 + j) * 128 + row, add) : 0ull;
          }
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const bool done = (c0 + j < args.M) && ((long long)(old[j] >> 40) + nk == (long long)kt_total);
            if (done) {
              __stcg(slot + (c0 + j) * 128 + row, 0ull);
              v[j] = (int)((long long)(old[j] & ((1ull << 40) - 1)) + (long long)v[j] + (nk << 21) -
                           ((long long)kt_total << 21));
            } else {
              sc[j] = __int_as_float(0x7fc00000);   // marks "not finished here"
            }
          }
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          if (c0 + j < args.M && (sg.whole || sc[j] == sc[j])) {
            if (!scaled) {
              reinterpret_cast<int32_t*>(args.out)[(size_t)(c0 + j) * args.N + n] = v[j];
            } else {
              const float y = lqq_scale(v[j], sc[j], w_scale);
              if constexpr (MULTI) store_out_all(multi.out, c0 + j, n, y, args.out_mode);
              else store_out(args.out, (size_t)(c0 + j) * args.N + n, y, args.out_mode);
            }
          }
        }
      }
      if (tracing) {
        const long long e3 = clock64();
        e_wait += e1 - e0;
        e_load += e2 - e1;
        e_store += e3 - e2;
      }
      if (set * 16 >= BN || set * 16 >= args.M) {   // this set had no chunk: it still releases the accumulator
        __syncwarp();
        ptx::tc_fence_before();
        ptx::mbar_arrive(bar_accfree);
      }
      ++seg;
    }
    if constexpr (MULTI) {
      // Every output store of this CTA, including those into peer memory, is ordered before the flags:
      // the barrier makes the other threads' stores visible to thread 0 (CTA scope), and the release of
      // its system-scope reduction is cumulative over them.
      asm volatile("bar.sync 1, %0;" ::"n"(kDequant) : "memory");
      if (d == 0) {
        peer_signal(multi.sync);   // red.release.sys: ordered after everything the barrier made visible
      }
    }
    if (tracing) {
      args.trace[blockIdx.x * 8 + 3] = (long long)ptx::globaltimer_ns();
      args.trace[blockIdx.x * 8 + 4] = e_wait;
      args.trace[blockIdx.x * 8 + 5] = e_load + e_store;
      args.trace[blockIdx.x * 8 + 6] = d_wait;
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
}

template <int BN, int NS, bool MULTI>
static int launch(const CUtensorMap& tx, const Args& a, const MultiOut* multi, int grid, cudaStream_t st) {
  using C = Cfg<BN, NS>;
  auto kern = &w4a8_skinny_kernel<BN, NS, MULTI>;
  static std::once_flag once[64];
  int dev = 0;
  cudaGetDevice(&dev);
  cudaError_t e = cudaSuccess;
  std::call_once(once[dev & 63], [&]() {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
  });
  if (e == cudaSuccess) {
    if constexpr (MULTI) e = launch_overlapped(kern, dim3(grid), dim3(kThreads), (size_t)C::kSmemBytes, st, tx, a, *multi);
    else e = launch_overlapped(kern, dim3(grid), dim3(kThreads), (size_t)C::kSmemBytes, st, tx, a, NoMultiOut{});
  }
  if (e != cudaSuccess) {
    record_cuda_error(e, "w4a8_skinny_kernel launch");
    return LQ_ERR_CUDA;
  }
  return check_launch("w4a8_skinny_kernel");
}

static int g_debug_skip = 0;
static long long* g_trace = nullptr;

static int bn_for(int M) { return M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : 128; }

static DecodePlan plan_for(int N, int K) { return decode_plan((N + 127) / 128, K / 128, 2 * sm_count(), true); }

}  // namespace skinny

// CTAs a launch of this shape uses: what a consumer of the gather-by-stores epilogue must see arrive
// from every rank.
int skinny_grid(int N, int K) { return skinny::plan_for(N, K).grid; }

size_t skinny_workspace_bytes(int M, int N, int K) {
  (void)N;
  (void)K;
  return (size_t)(2 * sm_count()) * (size_t)(skinny::bn_for(M) * 128 * 8);   // one slot per resident CTA
}

// out_mode: LQ_DT_* or 3 (raw int32).  M <= 128.  `ws`: skinny_workspace_bytes(), all zero, left all zero.
int run_skinny_gemm(const int8_t* x, const uint8_t* blob, const float* ascale, const float* s1, const OutSpec& out,
                    const PeerSync* sync, int out_mode, int M, int N, int K, void* ws, size_t ws_bytes, cudaStream_t st) {
  using namespace skinny;
  if (!ws || ws_bytes < skinny_workspace_bytes(M, N, K)) return LQ_ERR_WORKSPACE;
  const int bn = bn_for(M);
  const DecodePlan plan = plan_for(N, K);
  const int grid = plan.grid;
  CUtensorMap tx;
  int rc = make_byte_matrix_map(&tx, x, M, K, bn, 128);
  if (rc) return rc;
  Args a;
  a.blob = blob;
  a.ascale = ascale;
  a.s1 = s1;
  // one plain destination with nothing to signal or wait for: the small-parameter kernels
  const bool multi = out.n != 1 || out.ld != N || out.col0 != 0 || (sync && (sync->n_signal > 0 || sync->wait));
  if (multi && out_mode == kOutI32) return LQ_ERR_BAD_ARG;
  a.out = out.ptr[0];
  a.slots = static_cast<unsigned long long*>(ws);
  a.status = status_word();
  a.out_mode = out_mode;
  a.M = M;
  a.N = N;
  a.K = K;
  a.fixed_split = plan.fixed_split;
  a.debug_skip = g_debug_skip;
  a.trace = g_trace;
  if (!a.status) return LQ_ERR_CUDA;
  if (!multi) {
    switch (bn) {
      case 16: return launch<16, 6, false>(tx, a, nullptr, grid, st);
      case 32: return launch<32, 6, false>(tx, a, nullptr, grid, st);
      case 64: return launch<64, 5, false>(tx, a, nullptr, grid, st);
      default: return launch<128, 4, false>(tx, a, nullptr, grid, st);
    }
  }
  MultiOut mo;
  mo.out = out;
  mo.sync = sync ? *sync : PeerSync{};
  if (bn != 16) return LQ_ERR_SHAPE;   // the gather-by-stores variant is a decode path (M <= 16)
  return launch<16, 6, true>(tx, a, &mo, grid, st);
}

}  // namespace lq

// Pipeline-study hook (timing experiments only; results become wrong when non-zero).
extern "C" LQ_API void lq_debug_set_skinny_skip(int mask) { lq::skinny::g_debug_skip = mask; }

// Pipeline-study hook: device buffer of 4 x int64 per CTA receiving globaltimer stamps of dequant
// thread 0 (start, first tile landed, last dequant done, exit); null switches it off.
extern "C" LQ_API void lq_debug_set_skinny_trace(void* device_buffer) {
  lq::skinny::g_trace = static_cast<long long*>(device_buffer);
}
