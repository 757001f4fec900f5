// W4A8 tensor-core linear for decode batches (up to 32 tokens; the dispatch uses it for 3..16 tokens on matrices
// up to 32 M weights, where its single launch beats the tile kernel's planes + finish pass): HBM-bound, so built like a streaming
// copy with tensor cores attached, in ONE launch.  Replaces the reference's split-K WGMMA path for small
// M (csrc/liquid_gemm/w4a8_wgmma.cu:333-503 with the split rule at :523-534 and the finish kernel :39-56).
//
//  * Work = the (n-tile, k-tile) grid of 8704-byte blob tiles, cut into equal contiguous ranges, one
//    per CTA, two CTAs per SM (stream-K; layers with few n-tiles are cut into equal k-ranges per tile):
//    every SM streams the same number of weight bytes whatever N and K are.
//  * warp 0  producer: one thread keeps a ring of NW weight tiles in flight, one contiguous bulk copy
//            each.  The dequant threads release a stage as soon as they hold the tile in registers, so
//            the ring only has to cover the memory latency.  The tokens do NOT come through the copy
//            engine: measured on B200, a second (tensor-map) copy per k-tile made the copy engine the
//            bottleneck -- the producer was never idle, its copy instructions blocked on a full queue, the
//            MMAs waited for token boxes a third of the time and the stream ran at 60 % of the dp4a GEMV's
//            rate.  The 128 threads of the dequant set that owns a k-tile fetch its BN x 128-byte token
//            slice themselves (16 bytes each, an L2 hit issued before the wait for the weights) and store
//            it into the operand stage in the 128-byte-swizzled layout the MMA's descriptor expects.
//  * warps 2..9  two dequant sets taking alternate k-tiles; thread r of a set owns weight row r:
//            64 bytes of nibbles -> 128 INT8 (AND / SHR+AND / IMAD / XOR on 4-lane words) ->
//            tcgen05.st into tensor-memory lane r (the MMA's A operand, 4 consecutive k per column).
//  * warp 1  MMA: the warp walks the loop, one elected lane issues four 128 x BN x 32 tcgen05.mma kind::i8 per k-tile (A from tensor
//            memory, B = tokens through a shared-memory descriptor); its commit recycles the operand
//            stage (NT stages: 32 tensor-memory columns + the token slice in shared memory).
//  * Two accumulators in tensor memory, taken in turn by the segments (tile, k-range) of the CTA's
//    range.  Set p owns accumulator p and runs the epilogue of a segment only when that accumulator is
//    needed again, or at the very end -- where the two sets finish the CTA's (at most two) partial
//    segments side by side.  Nothing stalls in the middle of the stream: measured on B200, an epilogue
//    between two segments (tensor-memory load, atomics, stores: one to two microseconds during which
//    no operand is produced) cost more than the imbalance stream-K removes.
//  * Epilogue: tcgen05.ld (lane = channel, column = token); a segment that covers its tile's whole K
//    is scaled and stored directly; otherwise the partial sums of the CTAs that share the tile meet in
//    a zeroed workspace word per output element through ONE returning 64-bit atomic add that carries
//    the k-tile count along with the sum, and whoever completes the count stores the output and
//    re-zeroes the word.  Integer sums are exact in any order, so results do not depend on the split.
//    The optional bias is added to the value already rounded to the output type, as PyTorch's
//    `y + bias` after the reference's operator does (liquidgemm/vllm_plugin.py:205-206).
//  * Launched with programmatic stream serialisation: weight tiles are requested before the wait for
//    the previous kernel of the stream, tokens / outputs / workspace are touched only after it.
// Every wait is bounded; a thread whose wait expires records a site code, stops waiting and still
// runs the rest of its control flow, so the CTA reaches the exit where tensor memory is released.

#include <stdint.h>

#include <cstdlib>
#include <mutex>
#include <type_traits>

#include "lq_common.cuh"
#include "lq_sched.cuh"
#include "lq_tc_ptx.cuh"

namespace lq {

namespace dtc {

// Pipeline studies (-DLQ_PIPELINE_TRACE, a build of its own): per-CTA cycle counters of every role, read
// back with lq_debug_read_decode_trace().  The product build compiles none of it.
#ifdef LQ_PIPELINE_TRACE
__device__ long long g_trace[1024 * 16];
#define TR_NOW() clock64()
#define TR_ADD(acc, t0) (acc) += clock64() - (t0)
#define TR_SET(slot, v) g_trace[(blockIdx.x & 1023) * 16 + (slot)] = (long long)(v)
#define TR_VAR(name) long long name = 0
#else
#define TR_NOW() 0ll
#define TR_ADD(acc, t0) ((void)(t0))
#define TR_SET(slot, v) ((void)(v))
#define TR_VAR(name) const long long name = 0
#endif

constexpr int kTileBytes = 8704;
constexpr int kSets = 2;                    // dequant sets of 128 threads; set p also owns accumulator p
constexpr int kDequant = 128 * kSets;
constexpr int kThreads = 64 + kDequant;
constexpr uint64_t kWaitLimitNs = 2000000000ull;
// The wait for tokens gathered from peer GPUs gives up well before the barrier waits of the threads that
// depend on it, so that one late peer is reported once (by the producer) and the rest of the CTA still
// finishes its reduction and leaves the workspace clean.
constexpr uint64_t kPeerWaitLimitNs = 1000000000ull;
constexpr int kOutI32 = 3;

struct Args {
  const uint8_t* blob;
  const int8_t* x;       // [M, K]
  const float* ascale;   // [M]
  const float* s1;       // [N]
  const void* bias;      // [N] in the output dtype, or null
  void* out;             // [M, N] (single-destination kernels; the others get a MultiOut parameter)
  unsigned long long* slots;   // [grid][BN][128] packed (k-tile count, biased partial sum), zero between launches
  int* status;
  int out_mode;          // LQ_DT_* or kOutI32
  int M, N, K, fixed_split;
};

template <int BN, int NW, int NT>
struct Cfg {
  static constexpr int kXStage = BN * 128;
  static constexpr int kAccCols = 2 * BN;   // two accumulators
  static constexpr int kACols = 32 * NT;    // one tensor-memory operand stage per token box
  static constexpr int kColsNeeded = kAccCols + kACols;
  static constexpr int kTmemCols = kColsNeeded <= 128 ? 128 : 256;
  static constexpr int kNumBars = 2 * NW + 2 * NT + 4;
  static constexpr int kUsedBytes = 1024 + NT * kXStage + NW * kTileBytes + kNumBars * 8 + 16 + 2 * BN * 4;
  // more than a third of the SM's shared memory, so that never three CTAs (of this and of the next
  // kernel, under programmatic dependent launch) share an SM while another SM holds one
  static constexpr int kSmemBytes = kUsedBytes > 78 * 1024 ? kUsedBytes : 78 * 1024;
  static_assert(kColsNeeded <= 256, "two CTAs per SM share 512 tensor-memory columns");
  static_assert(kSmemBytes <= 113 * 1024, "two CTAs per SM share the shared memory");
};

// What the epilogue needs to know about a segment after the walk has moved on.
struct SegInfo {
  int tile, nk, slot;
  bool whole;
  float w_scale, bias;   // of this thread's output channel: weights, fetched when the segment starts
};

template <int BN, int NW, int NT, bool MULTI>
__global__ void __launch_bounds__(kThreads, 2)
w4a8_decode_tc_kernel(const Args args, const std::conditional_t<MULTI, MultiOut, NoMultiOut> multi) {
  const int kt_total = args.K >> 7;
  using C = Cfg<BN, NW, NT>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);

  const uint32_t xs = base;                          // NT token slices (1024-aligned for the swizzle)
  const uint32_t ws = xs + NT * C::kXStage;          // NW weight tiles
  const uint32_t bar_wfull = ws + NW * kTileBytes;   // [NW] weight tile landed
  const uint32_t bar_wfree = bar_wfull + NW * 8;     // [NW] a dequant set holds the tile in registers
  const uint32_t bar_aready = bar_wfree + NW * 8;    // [NT] dequantised operand and token slice are in place
  const uint32_t bar_afree = bar_aready + NT * 8;    // [NT] the MMAs that read operand and token slice are done
  const uint32_t bar_accfull = bar_afree + NT * 8;   // [2] the accumulator's segment is final
  const uint32_t bar_accfree = bar_accfull + 16;     // [2] the accumulator has been read
  const uint32_t tmem_slot = bar_accfree + 16;
  volatile uint32_t* tmem_slot_p = reinterpret_cast<volatile uint32_t*>(smem + (tmem_slot - base));
  float* tok_scale = reinterpret_cast<float*>(smem + (tmem_slot + 16 - base));   // [2 sets][BN] token scales

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < NW; ++s) {
      ptx::mbar_init(bar_wfull + 8 * s, 1);
      ptx::mbar_init(bar_wfree + 8 * s, 128);
    }
    for (int t = 0; t < NT; ++t) {
      ptx::mbar_init(bar_aready + 8 * t, 128);
      ptx::mbar_init(bar_afree + 8 * t, 1);
    }
    for (int p = 0; p < 2; ++p) {
      ptx::mbar_init(bar_accfull + 8 * p, 1);
      ptx::mbar_init(bar_accfree + 8 * p, 128);
    }
    ptx::fence_mbar_init();
  }
  __syncthreads();
  allow_dependents();   // the next kernel of the stream may start prefetching its weights

  const SchedArgs sched{kt_total, (args.N + 127) >> 7, 1, args.fixed_split};
  SegmentWalk walk(sched, blockIdx.x, gridDim.x);
  Segment sg;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      Ring<NW> ring;
      int issued = 0;
      bool ok = true;
      TR_VAR(tr_idle);
      const long long tr_p0 = TR_NOW();
      // Weight tiles do not depend on the previous kernel of the stream, so they are requested at once.
      while (ok && walk.next(sg)) {
        const uint8_t* src = args.blob + ((size_t)sg.tile * kt_total + sg.kb) * kTileBytes;
        for (int kt = sg.kb; kt < sg.ke; ++kt, src += kTileBytes) {
          const long long tr_i0 = TR_NOW();
          if (!ptx::mbar_wait_bounded(bar_wfree + 8 * ring.s, ring.ph ^ 1u, kWaitLimitNs)) {
            atomicExch(args.status, 401);
            ok = false;
            break;
          }
          TR_ADD(tr_idle, tr_i0);
          ptx::mbar_expect_tx(bar_wfull + 8 * ring.s, kTileBytes);
          ptx::bulk_load(ws + ring.s * kTileBytes, src, kTileBytes, bar_wfull + 8 * ring.s);
          ring.advance();
          ++issued;
        }
      }
      TR_SET(0, tr_idle);
      TR_SET(1, TR_NOW() - tr_p0);
      if (!ok) {
        // Copies in flight write shared memory: they must have landed before the CTA may exit.  (On the
        // normal path the dequant sets have waited for every one of them.)
        for (int i = issued > NW ? issued - NW : 0; i < issued; ++i)
          ptx::mbar_wait_bounded(bar_wfull + 8 * (i % NW), (uint32_t)(i / NW) & 1u, kWaitLimitNs);
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
    const uint32_t tmem_a = tmem_base + C::kAccCols;
    {
      // The whole warp walks the loop; one elected lane issues (see ptx::elect_one).
      const bool leader = ptx::elect_one();
      constexpr uint32_t idesc = ptx::idesc_i8(BN);
      Ring<NT> ring;
      bool ok = true;
      uint32_t seg = 0;
      TR_VAR(tr_wa);
      TR_VAR(tr_issue);
      TR_VAR(tr_commit);
      const long long tr_m0 = TR_NOW();
      while (walk.next(sg)) {
        const uint32_t p = seg & 1u;
        // the accumulator's previous segment (two back) must have been read out by its set
        if (seg >= 2 && ok && !ptx::mbar_wait_bounded(bar_accfree + 8 * p, ((seg >> 1) - 1u) & 1u, kWaitLimitNs)) {
          if (leader) atomicExch(args.status, 402);
          ok = false;
        }
        const uint32_t tmem_acc = tmem_base + p * BN;
        for (int kt = sg.kb; kt < sg.ke; ++kt) {
          const long long tr_a1 = TR_NOW();
          if (ok && !ptx::mbar_wait_bounded(bar_aready + 8 * ring.s, ring.ph, kWaitLimitNs)) {
            if (leader) atomicExch(args.status, 403);
            ok = false;
          }
          TR_ADD(tr_wa, tr_a1);
          __syncwarp();
          ptx::tc_fence_after();
          const long long tr_i1 = TR_NOW();
          const uint32_t xb = xs + ring.s * C::kXStage;
          const uint32_t ab = tmem_a + ring.s * 32;
          if (leader) {
#pragma unroll
            for (int j = 0; j < 4; ++j)
              ptx::mma_i8_ts(tmem_acc, ab + j * 8, ptx::smem_desc_sw128(xb + j * 32), idesc, (kt > sg.kb || j > 0) ? 1u : 0u);
          }
          TR_ADD(tr_issue, tr_i1);
          const long long tr_i2 = TR_NOW();
          if (leader) ptx::tc_commit(bar_afree + 8 * ring.s);   // frees the operand stage and its token slice
          TR_ADD(tr_commit, tr_i2);
          ring.advance();
        }
        if (leader) ptx::tc_commit(bar_accfull + 8 * p);
        ++seg;
      }
      if (leader) {
        TR_SET(3, tr_wa);
        TR_SET(4, TR_NOW() - tr_m0);
        TR_SET(10, tr_issue);
        TR_SET(11, tr_commit);
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
    // ------------------------------------------------------------------ dequant sets, then epilogues
    const int d = threadIdx.x - 64;
    const int set = d >> 7;                   // takes the k-tiles whose running index is set (mod 2); owns accumulator `set`
    const int quad = warp & 3;                // tensor-memory lane quadrant this warp may access
    const int row = quad * 32 + lane;         // weight row inside the tile == tensor-memory lane
    const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
    asm volatile("bar.sync 2, %0;" ::"n"(32 + kDequant) : "memory");
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot_p;
    const uint32_t tmem_a = tmem_base + C::kAccCols + lane_addr;
    // Token slice of a k-tile: BN rows of 128 bytes.  Thread j of the owning set moves 16-byte chunk
    // (j & 7) of token rows (j >> 3) + 16 q; in the 128-byte swizzle chunk c of row r sits at chunk
    // c ^ (r & 7) of that row.  Rows past M are zero.
    const int jx = d & 127;
    const int x_row = jx >> 3;
    const uint32_t x_off = (uint32_t)(x_row * 128 + (((jx & 7) ^ (x_row & 7)) << 4));
    const int8_t* x_src = args.x + (size_t)x_row * args.K + (jx & 7) * 16;
    Ring<NW> rw;   // weight ring position
    Ring<NT> rt;   // operand ring position
    bool ok = true;
    TR_VAR(tr_wfull);
    TR_VAR(tr_flush);
    TR_VAR(tr_unpack);
    TR_VAR(tr_afree);
    TR_VAR(tr_st);
    TR_VAR(tr_epi);
    const long long tr_d0 = TR_NOW();
    if (d == 0) {
      TR_SET(13, ptx::globaltimer_ns());
      uint32_t smid;
      asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
      TR_SET(15, smid);
    }
    uint32_t step = 0;   // running k-tile index of this CTA
    uint32_t seg = 0;
    bool waited_dependency = false;
    SegInfo mine = {0, 0, 0, true, 0.f, 0.f};   // the last segment that went into this set's accumulator
    const bool scaled = args.out_mode != kOutI32;
    const bool has_bias = scaled && args.bias != nullptr;

    // Epilogue of segment number `s` (accumulator s & 1 == set), described by `si`.
    auto epilogue = [&](const SegInfo& si, uint32_t s) {
      const uint32_t p = s & 1u;
      if (ok && !ptx::mbar_wait_bounded(bar_accfull + 8 * p, (s >> 1) & 1u, kWaitLimitNs)) {
        atomicExch(args.status, 405);
        ok = false;
      }
      __syncwarp();
      ptx::tc_fence_after();
      if (!waited_dependency) {
        dependency_wait();   // token scales, outputs and the reduction workspace belong to earlier kernels until here
        waited_dependency = true;
      }
      const long n = (long)si.tile * 128 + row;
      const bool n_ok = n < args.N;
      const float w_scale = si.w_scale, bias = si.bias;
      unsigned long long* slot = args.slots + (size_t)si.slot * (BN * 128);
      const long long nk = si.nk;
      const uint32_t tmem_acc = tmem_base + p * BN + lane_addr;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 16) {
        if (c0 >= args.M) break;   // uniform over the warp
        int v[16];
        ptx::tmem_ld16(tmem_acc + c0, v);
        ptx::tc_wait_ld();
        if (c0 + 16 >= BN || c0 + 16 >= args.M) {   // last chunk: the accumulator may be reused
          __syncwarp();
          ptx::tc_fence_before();
          ptx::mbar_arrive(bar_accfree + 8 * p);
        }
        if (!n_ok) continue;
        float sc[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) sc[j] = tok_scale[set * BN + c0 + j];   // staged at the set's first k-tile
        if (!si.whole) {
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
          if (c0 + j < args.M && (si.whole || sc[j] == sc[j])) {
            if (!scaled) {
              reinterpret_cast<int32_t*>(args.out)[(size_t)(c0 + j) * args.N + n] = v[j];
            } else {
              const float y = lqq_scale(v[j], sc[j], w_scale);
              if constexpr (MULTI) store_out_all(multi.out, c0 + j, n, y, bias, has_bias, args.out_mode);
              else store_out_bias(args.out, (size_t)(c0 + j) * args.N + n, y, bias, has_bias, args.out_mode);
            }
          }
        }
      }
    };

    for (;;) {
      const bool more = walk.next(sg);
      // One place decides which finished segment this set reads out now.  While the stream runs: the
      // segment two back, just before its accumulator (this set's) takes a new one.  After the last
      // segment: whichever of the last two segments sits in this set's accumulator -- the two sets
      // finish the CTA's last two segments side by side.
      uint32_t epi = 0xffffffffu;
      if (more) {
        if (seg >= 2 && (int)(seg & 1u) == set) epi = seg - 2;
      } else if (seg >= 1 && (int)((seg - 1u) & 1u) == set) {
        epi = seg - 1;
      } else if (seg >= 2) {
        epi = seg - 2;
      }
      if (epi != 0xffffffffu) {
        const long long tr_e1 = TR_NOW();
        epilogue(mine, epi);
        TR_ADD(tr_epi, tr_e1);
      }
      if (!more) break;
      if ((int)(seg & 1u) == set) {
        // channel scale and bias are weights: fetched here, far from the epilogue that needs them
        const long n = (long)sg.tile * 128 + row;
        const bool n_ok = n < args.N;
        mine = SegInfo{sg.tile, sg.ke - sg.kb, sg.slot, sg.whole, (n_ok && scaled) ? __ldg(args.s1 + n) : 0.f,
                       (n_ok && has_bias) ? load_bias(args.bias, n, args.out_mode) : 0.f};
      }
#pragma unroll 1
      for (int kt = sg.kb; kt < sg.ke; ++kt, ++step, rw.advance(), rt.advance()) {
        if ((int)(step & 1u) != set) continue;
        if (!waited_dependency) {
          dependency_wait();   // the tokens (and later the outputs) belong to earlier kernels until here
          waited_dependency = true;
          // Token scales (an earlier kernel's output) go to shared memory once per set; the epilogue, which
          // this set runs much later and under time pressure, reads them from there.
          if (jx < BN) tok_scale[set * BN + jx] = (scaled && jx < args.M) ? __ldg(args.ascale + jx) : 0.f;
          if (set == 0) asm volatile("bar.sync 5, 128;" ::: "memory");
          else asm volatile("bar.sync 6, 128;" ::: "memory");
          if constexpr (MULTI) {
            // tokens gathered from peer GPUs: one thread waits for their flags on behalf of its set
            if ((d & 127) == 0 && !peer_wait(multi.sync, kPeerWaitLimitNs)) atomicExch(args.status, 409);
            if (set == 0) asm volatile("bar.sync 3, 128;" ::: "memory");
            else asm volatile("bar.sync 4, 128;" ::: "memory");
          }
        }
        // request this k-tile's tokens now (L2 hits); they are stored after the unpack
        uint4 xv[BN / 16];
#pragma unroll
        for (int q = 0; q < BN / 16; ++q)
          xv[q] = (x_row + 16 * q < args.M) ? ldg_stream_v4(x_src + (size_t)(16 * q) * args.K + (size_t)kt * 128)
                                            : make_uint4(0u, 0u, 0u, 0u);
        const long long tr_w0 = TR_NOW();
        if (ok && !ptx::mbar_wait_bounded(bar_wfull + 8 * rw.s, rw.ph, kWaitLimitNs)) {
          atomicExch(args.status, 404);
          ok = false;
        }
        TR_ADD(tr_wfull, tr_w0);
        const long long tr_u0 = TR_NOW();
        const uint8_t* wst = smem + (ws - base) + rw.s * kTileBytes;
        uint4 ch[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) ch[c] = *reinterpret_cast<const uint4*>(wst + (c * 128 + row) * 16);
        const uint32_t meta = *reinterpret_cast<const uint32_t*>(wst + 8192 + row * 4);
        ptx::mbar_arrive(bar_wfree + 8 * rw.s);   // the tile is in registers: its stage may be refilled
        // unpack into registers first, wait for the operand stage afterwards
        const uint32_t step0 = meta & 0xffu, a0 = ((meta >> 8) & 0xffu) * 0x01010101u;
        const uint32_t step1 = (meta >> 16) & 0xffu, a1 = (meta >> 24) * 0x01010101u;
        uint32_t v[32];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const uint32_t st = c < 2 ? step0 : step1;
          const uint32_t ab = c < 2 ? a0 : a1;
          const uint32_t pk[4] = {ch[c].x, ch[c].y, ch[c].z, ch[c].w};
#pragma unroll
          for (int h = 0; h < 4; ++h) {
            v[8 * c + 2 * h] = lqq_dequant4(pk[h] & 0x0F0F0F0Fu, st, ab);
            v[8 * c + 2 * h + 1] = lqq_dequant4((pk[h] >> 4) & 0x0F0F0F0Fu, st, ab);
          }
        }
#ifdef LQ_PIPELINE_TRACE
        if (v[0] == 0x12345678u && v[31] == 0x9abcdef0u) TR_SET(8, 1);   // pins the arithmetic before the timer
#endif
        TR_ADD(tr_unpack, tr_u0);
        const long long tr_f0 = TR_NOW();
        if (ok && !ptx::mbar_wait_bounded(bar_afree + 8 * rt.s, rt.ph ^ 1u, kWaitLimitNs)) {
          atomicExch(args.status, 406);
          ok = false;
        }
        TR_ADD(tr_afree, tr_f0);
        __syncwarp();
        ptx::tc_fence_after();
        const long long tr_s0 = TR_NOW();
        ptx::tmem_st32(tmem_a + rt.s * 32, v);   // one store instruction for the whole operand stage row
#pragma unroll
        for (int q = 0; q < BN / 16; ++q)
          *reinterpret_cast<uint4*>(smem + rt.s * C::kXStage + x_off + q * 2048) = xv[q];
        // Wait for the operand store at once.  (Leaving it in flight during the next unpack and arriving
        // afterwards was measured: 1-3 % slower here, 10-30 % slower in the prefill kernel -- "operand ready"
        // one unpack later starves the MMAs more than the store's latency costs the thread.)
        ptx::tc_wait_st();
        TR_ADD(tr_st, tr_s0);
        const long long tr_s2 = TR_NOW();
        // the token slice was written with ordinary stores: make it visible to the tensor core's reads
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        ptx::tc_fence_before();
        ptx::mbar_arrive(bar_aready + 8 * rt.s);
        TR_ADD(tr_flush, tr_s2);
      }
      ++seg;
    }

    if (d == 0) {
      TR_SET(2, tr_flush);
      TR_SET(12, tr_unpack);
      TR_SET(5, tr_wfull);
      TR_SET(6, tr_afree);
      TR_SET(7, tr_st);
      TR_SET(8, TR_NOW() - tr_d0);
      TR_SET(9, tr_epi);
      TR_SET(14, ptx::globaltimer_ns());
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
  }
  ptx::tc_fence_before();
  __syncthreads();
}

template <int BN, int NW, int NT, bool MULTI>
static int launch(const Args& a, const MultiOut* multi, int grid, cudaStream_t st) {
  using C = Cfg<BN, NW, NT>;
  auto kern = &w4a8_decode_tc_kernel<BN, NW, NT, MULTI>;
  static std::once_flag once[64];
  int dev = 0;
  cudaGetDevice(&dev);
  cudaError_t e = cudaSuccess;
  std::call_once(once[dev & 63], [&]() {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
  });
  if (e == cudaSuccess) {
    if constexpr (MULTI) e = launch_overlapped(kern, dim3(grid), dim3(kThreads), (size_t)C::kSmemBytes, st, a, *multi);
    else e = launch_overlapped(kern, dim3(grid), dim3(kThreads), (size_t)C::kSmemBytes, st, a, NoMultiOut{});
  }
  if (e != cudaSuccess) {
    record_cuda_error(e, "w4a8_decode_tc_kernel launch");
    return LQ_ERR_CUDA;
  }
  return check_launch("w4a8_decode_tc_kernel");
}

static int bn_for(int M) { return M <= 16 ? 16 : 32; }

static DecodePlan plan_for(int N, int K) { return decode_plan((N + 127) / 128, K / 128, 2 * sm_count(), false); }

}  // namespace dtc

// CTAs a launch of this shape uses: what a consumer of the gather-by-stores epilogue must see arrive
// from every rank.
int decode_tc_grid(int N, int K) { return dtc::plan_for(N, K).grid; }

size_t decode_tc_workspace_bytes(int M, int N, int K) {
  (void)N;
  (void)K;
  return (size_t)(2 * sm_count()) * (size_t)(dtc::bn_for(M) * 128 * 8);   // one slot per resident CTA
}

// out_mode: LQ_DT_* or 3 (raw int32).  M <= 32.  `ws`: decode_tc_workspace_bytes(), all zero, left all zero.
int run_decode_tc(const int8_t* x, const uint8_t* blob, const float* ascale, const float* s1, const void* bias,
                  const OutSpec& out, const PeerSync* sync, int out_mode, int M, int N, int K, void* ws,
                  size_t ws_bytes, cudaStream_t st) {
  using namespace dtc;
  if (M < 1 || M > 32) return LQ_ERR_SHAPE;
  if (!ws || ws_bytes < decode_tc_workspace_bytes(M, N, K)) return LQ_ERR_WORKSPACE;
  const int bn = bn_for(M);
  const DecodePlan plan = plan_for(N, K);
  const int grid = plan.grid;
  Args a;
  a.blob = blob;
  a.x = x;
  a.ascale = ascale;
  a.s1 = s1;
  a.bias = bias;
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
  if (!a.status) return LQ_ERR_CUDA;
  if (!multi) {
    if (bn == 16) return launch<16, 8, 7, false>(a, nullptr, grid, st);
    return launch<32, 8, 6, false>(a, nullptr, grid, st);
  }
  MultiOut mo;
  mo.out = out;
  mo.sync = sync ? *sync : PeerSync{};
  if (bn == 16) return launch<16, 8, 7, true>(a, &mo, grid, st);
  return launch<32, 8, 6, true>(a, &mo, grid, st);
}

}  // namespace lq

#ifdef LQ_PIPELINE_TRACE
// Copies the per-CTA counters of the last launches (1024 CTAs x 16 slots of int64) to host memory.
extern "C" LQ_API int lq_debug_read_decode_trace(long long* host_dst) {
  return cudaMemcpyFromSymbol(host_dst, lq::dtc::g_trace, sizeof(long long) * 1024 * 16) == cudaSuccess ? 0 : -4;
}
#endif
