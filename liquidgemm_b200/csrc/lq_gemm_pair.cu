// Prefill W4A8 GEMM on CTA pairs (a few hundred tokens and more): tcgen05.mma.cta_group::2.
//
// Why pairs.  A 128-channel x 192-token tile needs, per 128-wide k-step, 8.7 KB of packed weights and 24 KB
// of tokens for 424 cycles of tensor-core work: 78 bytes per clock into every SM, which is what the L2 of
// this part delivers to 148 SMs that all read different lines (measured with the library's bulk-copy
// stream: 75 B/clk/SM out of L2, 18 TB/s in total).  A one-CTA kernel would sit on that limit as soon as its
// tensor cores ran at their full rate.  Two CTAs on neighbouring SMs that issue ONE 256-channel x 192-token
// MMA share the token tile: each stages only 96 of the 192 token rows (12 KB per k-step) and the tensor
// cores of both read both halves, so the traffic per SM drops to 49 B/clk at the same tensor-core rate
// (measured: 106 cycles per 256 x 192 x 32 MMA, the same as the one-CTA 128 x 192 x 32).
//
// Work.  Tile = 256 channels x 192 tokens, pair p of P takes tiles p, p + P, ... (channel blocks fastest, so
// the pairs of a wave share one or two token tiles and walk k in step: their weight and token lines hit in
// L2).  The tiles of the last, partial wave are taken whole by as many pairs, or, when they are long and few,
// cut into equal k-ranges over the pairs; a pair that holds one of the first k-ranges of a tile takes that unit
// FIRST and writes its int32 sums to a plane of the workspace; the pair with the last k-range takes it last, adds
// the planes (exact in any order) to the sums in its tensor memory, applies the epilogue and re-zeroes them.
//
// Per CTA (768 threads), connected by mbarrier rings; rank = CTA's rank in its pair:
//   warp 0        weight producer: one 8704-byte bulk copy per k-step (tile 2 * block + rank of the blob)
//   warp 2        token producer: one 96-row x 128-byte tensor-map box per k-step (rows 96 * rank ...)
//   warp 1        tensor-memory allocation; on rank 0 it issues (one elected lane) four 256 x 192 x 32 MMAs per k-step
//                 (A from the tensor memory of both CTAs, B from the shared memory of both) and commits to the
//                 barriers of BOTH CTAs (stage free, operand free, accumulator full)
//   warps 8..19   three dequant sets taking the k-steps in turn (two measured 3-4 % slower: a set spends half of
//                 its k-step in the tensor-memory store and its wait): thread r owns weight row r of its CTA's tile,
//                 unpacks 128 INT8 into tensor-memory lane r, then arrives on rank 0's "operand ready"
//                 barrier (one arrival per warp, both CTAs)
//   warps 4..7,   epilogue of the CTA's 128 channels, two groups sharing every tile's token chunks: tcgen05.ld,
//   20..23        scale, optional bias, stores (straight to global memory for one destination, staged through
//                 shared memory as 16-byte stores for several), while the MMAs of the next tile fill the other
//                 accumulator; every warp arrives on rank 0's "accumulator free" barrier
// Tensor memory (512 columns per CTA): two 192-column accumulators + four 32-column operand stages.
// Every wait is bounded; a wait that runs out records a site code (121..129) and the CTA unwinds to the common
// exit, where the pair synchronises before tensor memory is released.  No load uses cluster multicast.
#include <cuda.h>

#include <cstdlib>
#include <mutex>
#include <type_traits>

#include "lq_common.cuh"
#include "lq_tc_ptx.cuh"
#include "lq_sched.cuh"
#include "lq_pair_common.cuh"

namespace lq {

int make_byte_matrix_map(CUtensorMap* map, const void* ptr, long rows, long row_bytes, int box_rows,
                         int box_bytes);  // lq_gemm_tc.cu

namespace pairk {

using namespace pairc;

constexpr int kTileBytes = 8704;
constexpr int kBN = 192;                 // tokens per tile
constexpr int kHalf = kBN / 2;           // token rows staged by each CTA
constexpr int kSets = 3;                 // dequant sets of four warps, taking the k-steps in turn
constexpr int kThreads = 256 + 128 * kSets + 128;   // 24 warps: see the role list above
constexpr int kNS = 9;                   // shared-memory stages (weights + token half)
constexpr int kNT = 4;                   // operand stages in tensor memory
constexpr int kXStage = kHalf * 128;     // 12288
constexpr int kWStage = kTileBytes;
constexpr int kTmemCols = 512;           // 2 x 192 accumulator columns + 4 x 32 operand columns
constexpr int kNumBars = 2 * kNS + 2 * kNT + 4;
constexpr int kBarBytes = kNumBars * 8 + 32;
constexpr int kOutStage = 16 * 128 * 2;  // 16 tokens x 128 channels of 2-byte outputs
constexpr int kScaleBytes = 4 * kBN * 4;  // token scales of the current and the next tile, per epilogue group
constexpr int kSmemBytes = 1024 /* alignment slack */ + kNS * (kXStage + kWStage) + ((kBarBytes + 15) & ~15) + 2 * kOutStage +
                           kScaleBytes;
constexpr uint64_t kWaitLimitNs = 2000000000ull;
constexpr int kOutI32 = kEpiI32;              // internal output mode: raw int32
static_assert(kSmemBytes <= 232448, "shared memory budget exceeded");
static_assert(2 * kBN + 32 * kNT <= kTmemCols, "tensor memory budget exceeded");

// Pipeline studies (-DLQ_PIPELINE_TRACE, a build of its own): per-CTA cycle counters of every role, read back
// with lq_debug_read_pair_trace().  The product build compiles none of it.
#ifdef LQ_PIPELINE_TRACE
__device__ long long g_trace[256 * 32];
#define TR_NOW() clock64()
#define TR_ADD(acc, t0) (acc) += clock64() - (t0)
#define TR_SET(slot, v) g_trace[(blockIdx.x & 255) * 32 + (slot)] = (long long)(v)
#define TR_VAR(name) long long name = 0
#else
#define TR_NOW() 0ll
#define TR_ADD(acc, t0) ((void)(t0))
#define TR_SET(slot, v) ((void)(v))
#define TR_VAR(name) const long long name = 0
#endif

struct Args {
  const uint8_t* blob;     // tile blob
  const float* ascale;     // [M]
  const float* s1;         // [N]
  const void* bias;        // [N] in the output dtype, or null
  void* out;               // [M, N] in out_mode's type (single destination)
  int32_t* slots;          // workspace: per (partial tile, k-range but the last, rank) a plane of 192 x 128 int32 sums, all zero between launches
  int32_t* counters;       // workspace: per (partial tile, rank, epilogue group) planes written so far, all zero between launches
  int* status;
  int out_mode;            // LQ_DT_* or kOutI32
  int M, N, K;
  int kt_total;            // K / 128
  int n2_tiles, m_tiles;   // 256-channel blocks, 192-token blocks
  int pairs;               // CTA pairs of the launch
  int group_m;             // tile order: 0 channel blocks fastest, else groups of this many token tiles (see tile_coords)
  int tail_s;              // k-ranges each tile of the last, partial wave is cut into (1: whole tiles)
  int vec_out;             // several destinations, 2-byte outputs whose rows allow 16-byte stores: stage through smem
};

constexpr int kGroupsLast = 2 + kSets;   // warps groups sharing the epilogue of a pair's last tile

template <bool MULTI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
w4a8_pair_kernel(const __grid_constant__ CUtensorMap tmap_x, const Args args,
                 const std::conditional_t<MULTI, MultiOut, NoMultiOut> multi) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw_addr);

  const uint32_t xs = base;                                  // kNS token stages (1024-aligned, 128-byte swizzle)
  const uint32_t ws = xs + kNS * kXStage;                    // kNS weight stages
  const uint32_t bars = ws + kNS * kWStage;
  const uint32_t bar_full = bars;                            // [kNS] both copies of the stage landed (this CTA)
  const uint32_t bar_empty = bar_full + kNS * 8;             // [kNS] weights read by the dequant set + MMAs done
  const uint32_t bar_aready = bar_empty + kNS * 8;           // [kNT] operand in tensor memory; used on rank 0: 256 arrivals
  const uint32_t bar_afree = bar_aready + kNT * 8;           // [kNT] MMAs that read the operand stage are done
  const uint32_t bar_accfull = bar_afree + kNT * 8;          // [2] accumulator final
  const uint32_t bar_accfree = bar_accfull + 2 * 8;          // [2] accumulator drained; used on rank 0: 256 arrivals
  const uint32_t tmem_slot = bar_accfree + 2 * 8;
  uint8_t* gen_bars = smem + (bars - base);
  volatile uint32_t* tmem_slot_p = reinterpret_cast<volatile uint32_t*>(gen_bars + kNumBars * 8);
  volatile int* wait_flag = reinterpret_cast<volatile int*>(gen_bars + kNumBars * 8 + 8);   // [group][2]
  volatile int* last_flag = reinterpret_cast<volatile int*>(gen_bars + kNumBars * 8 + 24);  // [group]
  uint8_t* out_stage = gen_bars + ((kBarBytes + 15) & ~15);
  float* tok_scale = reinterpret_cast<float*>(out_stage + 2 * kOutStage);   // [group][2][kBN]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = ptx::cluster_ctarank();
  const int pair = (int)ptx::cluster_id_x();

  if (threadIdx.x == 0) {
    for (int s = 0; s < kNS; ++s) {
      ptx::mbar_init(bar_full + 8 * s, 2);       // one expect_tx arrival per producer
      ptx::mbar_init(bar_empty + 8 * s, 129);    // 128 dequant threads + the MMA thread's commit
    }
    for (int t = 0; t < kNT; ++t) {
      ptx::mbar_init(bar_aready + 8 * t, 8);     // one arrival per warp of the owning dequant set, both CTAs
      ptx::mbar_init(bar_afree + 8 * t, 1);
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(bar_accfull + 8 * b, 1);
      ptx::mbar_init(bar_accfree + 8 * b, 16);   // one arrival per epilogue warp (eight per CTA), both CTAs
    }
    ptx::fence_mbar_init();
    ptx::prefetch_tensormap(&tmap_x);
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
  const uint32_t tmem_a = tmem_base + 2 * kBN;   // kNT operand stages behind the two accumulators
  const uint32_t leader_aready = ptx::map_to_cta(bar_aready, 0);
  const uint32_t leader_accfree = ptx::map_to_cta(bar_accfree, 0);

  if (warp == 0 || warp == 2) {
    // ------------------------------------------------------------------ producers (one thread each)
    if (lane == 0) {
      const bool weights = (warp == 0);
      if (!weights) {
        if constexpr (MULTI) {
          if (!peer_wait(multi.sync, 1000000000ull)) atomicExch(args.status, 129);   // tokens gathered from peers
        }
      }
      PairWalk walk(args, pair);
      Segment sg;
      Ring<kNS> ring;
      int issued = 0;
      bool ok = true;
      TR_VAR(tr_empty);
      const long long tr_p0 = TR_NOW();
      while (ok && walk.next(sg)) {
        int n2, mt;
        tile_coords(sg.tile, args.n2_tiles, args.m_tiles, args.group_m, n2, mt);
        const uint8_t* wsrc = args.blob + ((size_t)(2 * n2 + (int)rank) * args.kt_total + sg.kb) * kTileBytes;
        const int row0 = mt * kBN + (int)rank * kHalf;
        for (int kt = sg.kb; kt < sg.ke; ++kt) {
          const long long tr_e0 = TR_NOW();
          if (!ptx::mbar_wait_bounded(bar_empty + 8 * ring.s, ring.ph ^ 1u, kWaitLimitNs)) {
            atomicExch(args.status, 121);
            ok = false;
            break;
          }
          TR_ADD(tr_empty, tr_e0);
          const uint32_t full = bar_full + 8 * ring.s;
          if (weights) {
            ptx::mbar_expect_tx(full, kWStage);
            ptx::bulk_load(ws + ring.s * kWStage, wsrc, kTileBytes, full);
            wsrc += kTileBytes;
          } else {
            ptx::mbar_expect_tx(full, kXStage);
            ptx::tensor_load_2d(xs + ring.s * kXStage, &tmap_x, kt * 128, row0, full);
          }
          ring.advance();
          ++issued;
        }
      }
      TR_SET(weights ? 0 : 2, tr_empty);
      TR_SET(weights ? 1 : 3, TR_NOW() - tr_p0);
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
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issue (leader CTA)
    // The whole warp walks the loop; one elected lane issues (see ptx::elect_one).
    if (rank == 0) {
      const bool leader = ptx::elect_one();
      constexpr uint32_t idesc = ptx::idesc_i8_pair(kBN);
      PairWalk walk(args, pair);
      Segment sg;
      Ring<kNS> ring;
      Ring<kNT> tring;
      Ring<2> accring;
      bool ok = true;
      TR_VAR(tr_accfree);
      TR_VAR(tr_aready);
      TR_VAR(tr_issue);
      TR_VAR(tr_commit);
      long long tr_steps = 0;
      const long long tr_m0 = TR_NOW();
      while (ok && walk.next(sg)) {
        const long long tr_a0 = TR_NOW();
        if (!ptx::mbar_wait_bounded(bar_accfree + 8 * accring.s, accring.ph ^ 1u, kWaitLimitNs)) {
          if (leader) atomicExch(args.status, 126);
          ok = false;
        }
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        TR_ADD(tr_accfree, tr_a0);
        ptx::tc_fence_after();
        const uint32_t tmem_acc = tmem_base + accring.s * kBN;
        for (int kt = sg.kb; kt < sg.ke; ++kt) {
          // "operand ready" from both CTAs implies that the token halves of both have landed: every dequant
          // thread saw its stage's full barrier (weights and tokens) before it produced the operand
          const long long tr_r0 = TR_NOW();
          if (!ptx::mbar_wait_bounded(bar_aready + 8 * tring.s, tring.ph, kWaitLimitNs)) {
            if (leader) atomicExch(args.status, 122);
            ok = false;
          }
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          TR_ADD(tr_aready, tr_r0);
          ++tr_steps;
          const long long tr_i0 = TR_NOW();
          ptx::tc_fence_after();
          const uint32_t xb = xs + ring.s * kXStage;
          const uint32_t ab = tmem_a + tring.s * 32;
          if (leader) {
#pragma unroll
            for (int j = 0; j < 4; ++j)
              ptx::mma_i8_ts_pair(tmem_acc, ab + j * 8, ptx::smem_desc_sw128(xb + j * 32), idesc,
                                  (kt > sg.kb || j > 0) ? 1u : 0u);
          }
          TR_ADD(tr_issue, tr_i0);
          const long long tr_c0 = TR_NOW();
          if (leader) {
            ptx::tc_commit_pair(bar_empty + 8 * ring.s);
            ptx::tc_commit_pair(bar_afree + 8 * tring.s);
          }
          TR_ADD(tr_commit, tr_c0);
          ring.advance();
          tring.advance();
        }
        if (ok && leader) ptx::tc_commit_pair(bar_accfull + 8 * accring.s);
        accring.advance();
      }
      if (leader) {
        TR_SET(4, tr_accfree);
        TR_SET(5, tr_aready);
        TR_SET(6, tr_issue);
        TR_SET(7, tr_commit);
        TR_SET(8, TR_NOW() - tr_m0);
        TR_SET(9, tr_steps);
      }
    }
  } else if (warp >= 8 && warp < 8 + 4 * kSets) {
    // ------------------------------------------------------------------ dequant (kSets sets, k-steps in turn)
    const int my_set = (warp - 8) >> 2;
    int step_set = 0;
    const int quad = warp & 3;               // TMEM lane quadrant this warp may access
    const int row = quad * 32 + lane;        // weight row inside the CTA's tile == TMEM lane
    const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
    PairWalk walk(args, pair);
    Segment sg;
    Ring<kNS> ring;
    Ring<kNT> tring;
    bool ok = true;
    TR_VAR(tr_full);
    TR_VAR(tr_unpack);
    TR_VAR(tr_afree);
    TR_VAR(tr_store);
    const long long tr_d0 = TR_NOW();
    while (ok && walk.next(sg)) {
      for (int kt = sg.kb; kt < sg.ke; ++kt) {
        const bool mine = step_set == my_set;
        step_set = step_set + 1 == kSets ? 0 : step_set + 1;
        if (!mine) {
          ring.advance();
          tring.advance();
          continue;
        }
        const long long tr_f0 = TR_NOW();
        if (!ptx::mbar_wait_bounded(bar_full + 8 * ring.s, ring.ph, kWaitLimitNs)) {
          atomicExch(args.status, 123);
          ok = false;
          break;
        }
        TR_ADD(tr_full, tr_f0);
        const long long tr_u0 = TR_NOW();
        const uint8_t* wst = smem + (ws - base) + ring.s * kWStage;
        uint4 ch[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) ch[c] = *reinterpret_cast<const uint4*>(wst + (c * 128 + row) * 16);
        const uint32_t meta = *reinterpret_cast<const uint32_t*>(wst + 8192 + row * 4);
        ptx::mbar_arrive(bar_empty + 8 * ring.s);
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
#ifdef LQ_PIPELINE_TRACE
        if (v[0][0] == 0x12345678u && v[3][7] == 0x9abcdef0u) TR_SET(31, 1);   // pins the arithmetic before the timer
#endif
        TR_ADD(tr_unpack, tr_u0);
        const long long tr_w0 = TR_NOW();
        if (!ptx::mbar_wait_bounded(bar_afree + 8 * tring.s, tring.ph ^ 1u, kWaitLimitNs)) {
          atomicExch(args.status, 124);
          ok = false;
          break;
        }
        TR_ADD(tr_afree, tr_w0);
        const long long tr_s0 = TR_NOW();
        __syncwarp();   // lanes leave the poll loops one by one; tcgen05.st / wait::st need the warp converged
        ptx::tc_fence_after();
#pragma unroll
        for (int c = 0; c < 4; ++c) ptx::tmem_st8(tmem_a + lane_addr + tring.s * 32 + c * 8, v[c]);
        // Waited for at once (leaving the stores in flight during the next unpack measured 5 % slower).  The
        // store and its wait are what a dequant set's k-step mostly consists of (about 435 of 830 cycles); feeding
        // the MMA unsigned operands (no XOR in the unpack above, 128 x the token row sums subtracted in the
        // epilogue) was measured too: bit-exact, within +-4 % on every shape, not kept.
        ptx::tc_wait_st();
        ptx::tc_fence_before();
        // One arrival per warp; the peer's goes over the SM-to-SM network with the default (CTA-scope) release
        // (a cluster-scope release cost the arriving thread about 1000 cycles when measured).
        __syncwarp();
        if (lane == 0) {
          if (rank == 0) ptx::mbar_arrive(bar_aready + 8 * tring.s);
          else ptx::mbar_arrive_remote(leader_aready + 8 * tring.s);
        }
        TR_ADD(tr_store, tr_s0);
        ring.advance();
        tring.advance();
      }
    }
    // The pair's last tile: nothing is left to unpack, and the two epilogue groups alone would take as long over
    // it as over any other (a converting, storing warp gets a memory instruction through per ~130 cycles; this
    // last epilogue is the one nothing hides).  The dequant sets join as groups 2..4 of kGroupsLast, with the
    // direct-store form only (one destination, or rows that do not allow 16-byte stores).
    if (!MULTI && args.vec_out == 0 && ok && walk.last_shared()) {
      const int last = walk.segments() - 1;            // sg still holds that segment
      const int b = last & 1;
      const uint32_t phb = (uint32_t)(last >> 1) & 1u;
      bool done = true;
      if (lane == 0) {
        done = ptx::mbar_wait_bounded(bar_accfull + 8 * b, phb, kWaitLimitNs);
        if (!done) atomicExch(args.status, 126);
      }
      constexpr size_t kPlane4 = (size_t)128 * kBN / 4;
      const int S = walk.S;
      const bool completes = !sg.whole;                // the last k-range of a cut tile: add the other pairs' planes
      int4* planes = reinterpret_cast<int4*>(args.slots) + ((size_t)walk.rt * (S - 1) * 2 + rank) * kPlane4;
      if (done && completes && lane == 0) {
        done = planes_ready(args.counters + 2 * ((size_t)walk.rt * 2 + rank), S - 1, kWaitLimitNs);
        if (!done) atomicExch(args.status, 130);
      }
      done = __shfl_sync(0xffffffffu, done ? 1 : 0, 0) != 0;
      if (done) {
        if (completes) __threadfence();
        ptx::tc_fence_after();
        const bool raw = args.out_mode == kOutI32;
        const bool has_bias = !raw && args.bias != nullptr;
        int n2, mt;
        tile_coords(sg.tile, args.n2_tiles, args.m_tiles, args.group_m, n2, mt);
        const int m0 = mt * kBN;
        const long n = (long)(2 * n2 + (int)rank) * 128 + row;
        const int cols = (args.M - m0) < kBN ? (args.M - m0) : kBN;
        const uint32_t tmem_acc = tmem_base + b * kBN + lane_addr;
        const float w_scale = raw ? 0.f : __ldg(args.s1 + n);
        const float bias = has_bias ? load_bias(args.bias, n, args.out_mode) : 0.f;
#pragma unroll 1
        for (int c0 = 16 * (2 + my_set); c0 < cols; c0 += 16 * kGroupsLast) {
          int v[16];
          ptx::tmem_ld16(tmem_acc + c0, v);
          float sc[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) sc[j] = (!raw && c0 + j < cols) ? __ldg(args.ascale + m0 + c0 + j) : 0.f;
          ptx::tc_wait_ld();
          if (completes) add_planes(v, planes, 2 * kPlane4, S - 1, c0, cols, row);
          epi_store_cols(args.out, args.out_mode, (size_t)(m0 + c0) * args.N + n, args.N, v, sc, w_scale, bias, has_bias,
                         cols - c0);
        }
        if (completes) {
#pragma unroll 1
          for (int c0 = 16 * (2 + my_set); c0 < cols; c0 += 16 * kGroupsLast) zero_planes(planes, 2 * kPlane4, S - 1, c0, cols, row);
        }
        ptx::tc_fence_before();
      }
    }
    if (threadIdx.x == 256) {
      TR_SET(10, tr_full);
      TR_SET(11, tr_unpack);
      TR_SET(12, tr_afree);
      TR_SET(13, tr_store);
      TR_SET(14, TR_NOW() - tr_d0);
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ epilogue (warps 4..7 and 20..23)
    // Two groups of four warps share every tile: group g takes the 16-token chunks g, g + 2, ...  (One warp
    // converting and storing runs at a fraction of an instruction per cycle; the tile's 192 x 128 outputs need
    // eight of them to finish inside the next tile's main loop.)
    const int g = warp >= 8 + 4 * kSets ? 1 : 0;
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
    const int et = (threadIdx.x & 127);        // 0..127 inside the group (both groups start at a multiple of 128)
    const bool raw = args.out_mode == kOutI32;
    const bool has_bias = !raw && args.bias != nullptr;
    const bool vec = args.vec_out != 0;
    uint8_t* stage = out_stage + g * kOutStage;
    volatile int* wflag = wait_flag + 2 * g;
    PairWalk walk(args, pair);
    const int nseg = walk.segments();
    const bool helped = !MULTI && !vec && walk.last_shared();
    Segment sg;
    Ring<2> accring;
    int seg = 0;
    bool ok = true;
    TR_VAR(tr_accfull);
    TR_VAR(tr_tsc);
    TR_VAR(tr_out);
    TR_VAR(tr_p1);
    TR_VAR(tr_psync);
    const long long tr_g0 = TR_NOW();
    while (ok && walk.next(sg)) {
      const int b = accring.s;
      const uint32_t phb = accring.ph;
      accring.advance();
      const long long tr_x0 = TR_NOW();
      // One thread of the group performs the bounded wait and publishes the outcome, so that its 128 threads
      // always agree on it (they meet at named barriers below and must never split up).
      const int fslot = seg & 1;
      ++seg;
      if (et == 0) {
        const bool done = ptx::mbar_wait_bounded(bar_accfull + 8 * b, phb, kWaitLimitNs);
        if (!done) atomicExch(args.status, 125);
        wflag[fslot] = done ? 1 : 0;
      }
      group_barrier(g);
      if (wflag[fslot] == 0) {
        ok = false;
        break;
      }
      ptx::tc_fence_after();
      TR_ADD(tr_accfull, tr_x0);
      int n2, mt;
        tile_coords(sg.tile, args.n2_tiles, args.m_tiles, args.group_m, n2, mt);
      const int m0 = mt * kBN;
      const long nbase = (long)(2 * n2 + (int)rank) * 128;
      const long n = nbase + row;
      const bool n_ok = n < args.N;
      const int cols = (args.M - m0) < kBN ? (args.M - m0) : kBN;   // valid token columns of this tile
      const uint32_t tmem_acc = tmem_base + b * kBN + lane_addr;
      const float w_scale = (n_ok && !raw) ? __ldg(args.s1 + n) : 0.f;
      const float bias = (has_bias && n_ok) ? load_bias(args.bias, n, args.out_mode) : 0.f;
      // A tile cut along k between S pairs: every pair but the one with the last k-range writes its sums to a
      // plane of its own in the workspace (plain 16-byte stores; int32 atomics on whole tiles from every pair at
      // once were measured at a fraction of that rate) and counts itself in; the pair with the last k-range
      // adds those planes to the sums it holds in tensor memory, applies the epilogue and leaves the planes zero
      // again (the counters are cleared at the end of the kernel).  The writers' two groups count separately.
      constexpr size_t kPlane4 = (size_t)128 * kBN / 4;   // int4 units: [token / 4][channel]
      const int S = walk.S;
      const bool completes = !sg.whole && walk.part == S - 1;
      int4* planes = reinterpret_cast<int4*>(args.slots) + ((size_t)walk.rt * (S - 1) * 2 + rank) * kPlane4;   // k-range q: + q * 2 * kPlane4
      int32_t* counters2 = args.counters + 2 * ((size_t)walk.rt * 2 + rank);   // one per epilogue group of the writers
      if (sg.whole || completes) {
        // Token scales of the tile, once, through shared memory (two buffers per group: a warp may be one tile
        // ahead of the slowest; this barrier is the only one of a tile whose outputs go straight to global memory).
        float* tsc = tok_scale + (2 * g + fslot) * kBN;
        const long long tr_t0 = TR_NOW();
        if (!raw) {
          for (int i = et; i < kBN; i += 128) tsc[i] = (i < cols) ? __ldg(args.ascale + m0 + i) : 0.f;
        }
        if (completes && et == 0) {
          // the other pairs took their k-ranges first of all: their sums have been there for a long time
          const bool there = planes_ready(counters2, S - 1, kWaitLimitNs);
          if (!there) atomicExch(args.status, 130);
          last_flag[g] = there ? 1 : 0;
        }
        group_barrier(g);
        if (completes) {
          if (last_flag[g] == 0) {
            ok = false;
            break;
          }
          __threadfence();
        }
        TR_ADD(tr_tsc, tr_t0);
        const long long tr_o0 = TR_NOW();
        // the pair's last tile, its main loop over: the dequant warps take three of every five chunks (below)
        const int cstep = (helped && seg == nseg) ? 16 * kGroupsLast : 32;
#pragma unroll 1
        for (int c0 = 16 * g; c0 < cols; c0 += cstep) {
          int v[16];
          ptx::tmem_ld16(tmem_acc + c0, v);
          if (completes) {
            // (Loading these one chunk ahead was measured: it saves a microsecond here and costs every whole tile
            // of short-K layers 8 % through the registers it holds.)
            ptx::tc_wait_ld();
            add_planes(v, planes, 2 * kPlane4, S - 1, c0, cols, row);
          }
          float sc[16];
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            const float4 f = *reinterpret_cast<const float4*>(tsc + c0 + 4 * q4);
            sc[4 * q4] = f.x; sc[4 * q4 + 1] = f.y; sc[4 * q4 + 2] = f.z; sc[4 * q4 + 3] = f.w;
          }
          ptx::tc_wait_ld();
          const int valid = cols - c0;
          if (!vec) {
            // lane = channel: a warp's store covers 32 consecutive channels of one token row
            if (n_ok) {
              const size_t idx0 = (size_t)(m0 + c0) * args.N + n;
              if constexpr (MULTI) {
                // several destinations whose type or alignment rules out the staged form
#pragma unroll
                for (int j = 0; j < 16; ++j)
                  if (j < valid)
                    store_out_all(multi.out, m0 + c0 + j, n, lqq_scale(v[j], sc[j], w_scale), bias, has_bias, args.out_mode);
              } else {
                epi_store_cols(args.out, args.out_mode, idx0, args.N, v, sc, w_scale, bias, has_bias, valid);
              }
            }
          } else {
            // Several destinations (peers over NVLink prefer whole 256-byte rows written with 16-byte stores):
            // through shared memory.  A thread holds 16 tokens of ONE channel, the output rows run along the channels.
            epi_stage_cols(reinterpret_cast<uint16_t*>(stage) + row, args.out_mode, v, sc, w_scale, bias, has_bias);
            group_barrier(g);
#pragma unroll
            for (int q = 0; q < 2; ++q) {
              const int vi = et + 128 * q;
              const int j = vi >> 4, chunk = vi & 15;
              const int m = m0 + c0 + j;
              const long ncol = nbase + chunk * 8;
              if (j < valid && ncol < args.N) {
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
            group_barrier(g);   // the stage is rewritten by the next chunk
          }
        }
        // this warp's reads of the accumulator are complete: the MMA warp may reuse it
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if (rank == 0) ptx::mbar_arrive(bar_accfree + 8 * b);
          else ptx::mbar_arrive_remote(leader_accfree + 8 * b);
        }
        if (completes) {
#pragma unroll 1
          for (int c0 = 16 * g; c0 < cols; c0 += cstep) zero_planes(planes, 2 * kPlane4, S - 1, c0, cols, row);
        }
        TR_ADD(tr_out, tr_o0);
      } else {
        // One of the first S - 1 k-ranges of a split tile: sums to this pair's plane.
        int4* own = planes + (size_t)walk.part * 2 * kPlane4 + row;
        const long long tr_a0 = TR_NOW();
#pragma unroll 1
        for (int c0 = 16 * g; c0 < cols; c0 += 32) {
          int v[16];
          ptx::tmem_ld16(tmem_acc + c0, v);
          ptx::tc_wait_ld();
#pragma unroll
          for (int jj = 0; jj < 4; ++jj)
            if (c0 + 4 * jj < cols)
              __stcg(own + (size_t)((c0 >> 2) + jj) * 128, make_int4(v[4 * jj], v[4 * jj + 1], v[4 * jj + 2], v[4 * jj + 3]));
        }
        TR_ADD(tr_p1, tr_a0);
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if (rank == 0) ptx::mbar_arrive(bar_accfree + 8 * b);
          else ptx::mbar_arrive_remote(leader_accfree + 8 * b);
        }
        const long long tr_b0 = TR_NOW();
        __threadfence();
        group_barrier(g);
        if (et == 0) atomicAdd(counters2 + g, 1);
        TR_ADD(tr_psync, tr_b0);
      }
    }
    if (et == 0 && g == 0) {
      TR_SET(16, tr_accfull);
      TR_SET(17, TR_NOW() - tr_g0);
      TR_SET(18, seg);
      TR_SET(19, tr_tsc);
      TR_SET(21, tr_out);
      TR_SET(22, tr_p1);
      TR_SET(23, tr_psync);
    }
    if constexpr (MULTI) {
      // every output store of this CTA, peer memory included, is ordered before the flags (see lq_common.cuh):
      // the two groups meet, then one thread signals for the CTA
      asm volatile("bar.sync 3, 256;" ::: "memory");
      if (et == 0 && g == 0) peer_signal(multi.sync);
    }
  }

  // Both CTAs are done with each other's shared and tensor memory before either releases anything.
  __syncwarp();
  ptx::tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) {
    // every warp of this CTA is done with the planes of the tile it completed: the counters are zero for the next launch
    const PairWalk w(args, pair);
    if (w.completes_tile()) {
      int32_t* c = args.counters + 2 * ((size_t)w.rt * 2 + rank);
      c[0] = 0;
      c[1] = 0;
    }
  }
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
    cudaFuncSetAttribute(w4a8_pair_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (cudaOccupancyMaxActiveClusters(&clusters, w4a8_pair_kernel<false>, &cfg) == cudaSuccess && clusters > 0 &&
        clusters < v)
      v = clusters;
    cudaGetLastError();
    if (v < 1) v = 1;
  }
  return v;
}

template <bool MULTI>
static int launch(const CUtensorMap& tx, const Args& a, const MultiOut* multi, cudaStream_t st) {
  auto kern = &w4a8_pair_kernel<MULTI>;
  static std::once_flag once[64];
  int dev = 0;
  cudaGetDevice(&dev);
  cudaError_t attr_err = cudaSuccess;
  std::call_once(once[dev & 63], [&]() {
    attr_err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
  });
  if (attr_err != cudaSuccess) {
    record_cuda_error(attr_err, "cudaFuncSetAttribute(w4a8_pair_kernel)");
    return LQ_ERR_CUDA;
  }
  if constexpr (MULTI) kern<<<2 * a.pairs, kThreads, kSmemBytes, st>>>(tx, a, *multi);
  else kern<<<2 * a.pairs, kThreads, kSmemBytes, st>>>(tx, a, NoMultiOut{});
  return check_launch("w4a8_pair_kernel");
}

struct PairPlan {
  int n2_tiles, m_tiles, pairs, partial_tiles, tail_s;
  size_t ws_bytes;
};
static PairPlan plan(int M, int N, int K) {
  PairPlan p;
  p.n2_tiles = N / 256;
  p.m_tiles = (M + kBN - 1) / kBN;
  const long tiles = (long)p.n2_tiles * p.m_tiles;
  const int cap = max_pairs();
  p.pairs = (int)(tiles < cap ? tiles : cap);
  const int r = (int)(tiles % p.pairs);
  p.tail_s = tail_split(r, p.pairs, K / 128);
  p.partial_tiles = p.tail_s > 1 ? r : 0;   // tiles whose K is shared between pairs
  // per partial tile, k-range but the last and rank: 192 x 128 int32 sums; then one counter per tile, rank and
  // epilogue group, padded to 256 bytes
  p.ws_bytes = p.partial_tiles == 0 ? 0
                                    : (size_t)p.partial_tiles * (p.tail_s - 1) * 2 * (128 * kBN * 4) +
                                          (((size_t)p.partial_tiles * 2 * 2 * 4 + 255) / 256) * 256;
  return p;
}

}  // namespace pairk

// Shapes the pair kernel serves: whole 256-channel blocks.
bool pair_serves(int M, int N, int K) { return M >= 1 && N >= 256 && N % 256 == 0 && K >= 128 && K % 128 == 0; }

// Whether the pair kernel is expected to beat the two-CTAs-per-SM tile kernel on this shape.  Both run whole
// waves of tiles, so the comparison is between (waves x k-steps x time per k-step) of either, with the times
// per k-step measured on B200 over the Llama-3.1-8B shapes at 256..8192 tokens in one run (microseconds: pair
// 0.335, or 0.30 for K >= 8192, plus 3 for the prologue and the last epilogue, a tile cut in S costing 1/S of
// a wave plus 20 k-steps (8 for K < 8192); tile 0.53, 0.45 for K >= 8192, 0.40 when there is at most one CTA per SM).  The
// model reproduces the measured winner at every point of that sweep except ties within 4 %.
bool pair_prefers(int M, int N, int K) {
  if (!pair_serves(M, N, K)) return false;
  const int kt = K / 128;
  const int sms = sm_count();
  const long tiles_t = (long)(N / 128) * ((M + 127) / 128);
  if (tiles_t * 2 <= 2L * sms) return false;   // the tile kernel splits K here: a small problem, it wins
  const double waves_t = (double)((tiles_t + 2L * sms - 1) / (2L * sms));
  const double est_tile = waves_t * kt * (tiles_t <= sms ? 0.40 : kt >= 64 ? 0.45 : 0.53);
  const pairk::PairPlan p = pairk::plan(M, N, K);
  const long tiles_p = (long)p.n2_tiles * p.m_tiles;
  const int r = (int)(tiles_p % p.pairs);
  const int S = p.tail_s;
  const double tail = r == 0 ? 0.0 : S > 1 ? 1.0 / S + (kt >= 64 ? 20.0 : 8.0) / kt : 1.0;   // a split tile costs its reduction too
  const double est_pair = ((double)(tiles_p / p.pairs) + tail) * kt * (kt >= 64 ? 0.30 : 0.335) + 3.0;
  return est_pair < 0.97 * est_tile;
}

size_t pair_workspace_bytes(int M, int N, int K) { return pairk::plan(M, N, K).ws_bytes; }

// CTAs of the launch (each signals the peers once in the gather-by-stores form).
int pair_grid(int M, int N, int K) { return 2 * pairk::plan(M, N, K).pairs; }

// out_mode: LQ_DT_* or 3 (raw int32).  `ws` (all zero on entry, all zero again on exit) holds the slots of the last partial wave.
int run_pair_gemm(const int8_t* x, const uint8_t* blob, const float* ascale, const float* s1, const void* bias,
                  const OutSpec& out, const PeerSync* sync, int out_mode, int M, int N, int K, void* ws, size_t ws_bytes,
                  cudaStream_t st) {
  using namespace pairk;
  if (!pair_serves(M, N, K) || out_mode < 0 || out_mode > kOutI32) return LQ_ERR_BAD_ARG;
  const PairPlan p = plan(M, N, K);
  if (p.ws_bytes && (!ws || ws_bytes < p.ws_bytes)) return LQ_ERR_WORKSPACE;
  CUtensorMap tx;
  if (int rc = make_byte_matrix_map(&tx, x, M, K, kHalf, 128)) return rc;
  const bool multi = out.n != 1 || out.ld != N || out.col0 != 0 || (sync && (sync->n_signal > 0 || sync->wait));
  if (multi && out_mode == kOutI32) return LQ_ERR_BAD_ARG;
  Args a;
  a.blob = blob;
  a.ascale = ascale;
  a.s1 = s1;
  a.bias = bias;
  a.out = out.ptr[0];
  a.slots = static_cast<int32_t*>(ws);
  a.counters = p.ws_bytes ? reinterpret_cast<int32_t*>(static_cast<uint8_t*>(ws) +
                                                      (size_t)p.partial_tiles * (p.tail_s - 1) * 2 * (128 * kBN * 4))
                          : nullptr;
  a.status = status_word();
  a.out_mode = out_mode;
  a.M = M;
  a.N = N;
  a.K = K;
  a.kt_total = K / 128;
  a.n2_tiles = p.n2_tiles;
  a.m_tiles = p.m_tiles;
  a.pairs = p.pairs;
  a.tail_s = p.tail_s;
  // Weights that do not stay in L2 beside tokens and outputs (more than 48 MB of 4-bit tiles: the 70B-model layers
  // on one GPU) are walked in groups of token tiles: 57344 x 8192 10 % faster at 2048 and 8192 tokens, 8192 x 28672
  // 15-25 % at 2048; the 8B-model layers, which fit, are 1-2 % better channel blocks first.
  a.group_m = (size_t)N * K / 2 > ((size_t)48 << 20) ? kGroupM : 0;
  // staged 16-byte stores for the gather-by-stores form; one local destination is written directly
  bool vec = multi && (out_mode == LQ_DT_BF16 || out_mode == LQ_DT_F16) && out.ld % 8 == 0 && out.col0 % 8 == 0;
  for (int r = 0; r < out.n; ++r) vec = vec && (reinterpret_cast<uintptr_t>(out.ptr[r]) % 16 == 0);
  a.vec_out = vec ? 1 : 0;
  if (!a.status) return LQ_ERR_CUDA;
  if (multi) {
    MultiOut mo;
    mo.out = out;
    mo.sync = sync ? *sync : PeerSync{};
    return launch<true>(tx, a, &mo, st);
  }
  return launch<false>(tx, a, nullptr, st);
}

}  // namespace lq

#ifdef LQ_PIPELINE_TRACE
// Copies the per-CTA counters of the last launch (256 CTAs x 32 slots of int64) to host memory.
extern "C" LQ_API int lq_debug_read_pair_trace(long long* host_dst) {
  return cudaMemcpyFromSymbol(host_dst, lq::pairk::g_trace, sizeof(long long) * 256 * 32) == cudaSuccess ? 0 : -4;
}
#endif
