// W4A8 tensor-core GEMM for sm_100a: TMA -> in-register LQQ dequant -> TMEM -> tcgen05.mma kind::i8,
// as one persistent, warp-specialised kernel with stream-K scheduling.
//
// Orientation.  The weights are the MMA "A" operand (128 output channels per tile, the full
// tensor-core M), the tokens are the "B" operand (BN = 16..256 per tile, the MMA N), so small
// token counts waste nothing on the 128-wide dimension: Y^T[n, m] = sum_k q_hat[n, k] * x[m, k].
//
// Work.  An output tile is 128 channels x BN tokens; it needs KT = K/128 "k-steps".  The grid is
// one CTA per SM.  All T*KT k-steps of the problem are laid end to end (tile-major) and cut into
// equal contiguous ranges, one per CTA ("stream-K"): every SM streams the same number of weight
// bytes whatever the tile count, which is what a bandwidth-bound decode GEMM needs, and prefill
// loses nothing to wave quantisation.  A CTA's range is a sequence of segments (tile, k-range).
// A segment that covers its tile's whole K is finished by that CTA alone.  Otherwise the CTA adds
// its int32 partial sums into a per-tile workspace slot with red.global.add (integer addition is
// exact in any order, so the result is bit-identical however the tile was cut); the CTA whose
// contribution completes the tile (a per-slot k-step counter reaches KT) reads the sums back,
// applies the epilogue and re-zeroes slot and counter, so the workspace is all-zero again when
// the kernel ends.  A fixed split-K factor can be requested instead (tile = S equal k-ranges).
//
// Roles inside a CTA (16 warps), connected by mbarrier rings:
//   warps 0, 2   producers: per k-step, warp 0 issues the weight tile (one 8704-byte bulk copy from
//                           the tile blob, or a tensor-map box of INT8 weights) and warp 2 the
//                           BN x 128 activation box (128-byte swizzle; token rows past M are
//                           zero-filled by the TMA unit).
//   warps 4..7,  dequant  : two sets take alternate k-steps; thread r owns weight row r of the tile:
//   12..15                  64 bytes of nibbles (four
//                           conflict-free 16-byte shared loads) + two (step, offset) pairs ->
//                           128 INT8 values by AND / SHR+AND, multiply-add, XOR on 32-bit words ->
//                           tcgen05.st into TMEM lane r, 4 consecutive k per 32-bit column, which
//                           is the layout tcgen05.mma reads an A operand from tensor memory in.
//   warp 1       MMA      : one thread issues four 128 x BN x 32 tcgen05.mma per k-step (A from
//                           TMEM, B through a shared-memory descriptor) into one of NACC
//                           accumulators, and commits to the barriers that recycle the stages.
//   warps 8..11  epilogue : tcgen05.ld (lane = channel, column = token) of a finished
//                           accumulator while the MMAs of the next segment fill the other one;
//                           (float)acc * ascale[m] * s1[n] + cast, int32 stores, or the partial
//                           reduction described above.
// The TMA ring runs NS k-steps ahead of the MMAs; operand stage s in tensor memory is tied to
// shared-memory stage s.
//
// Every wait is bounded: when a barrier does not complete within kWaitLimitNs the thread writes
// a site code to the status word, leaves its loop, and the CTA still reaches the common exit
// where tensor memory is released.
#include <cuda.h>

#include <cstdlib>
#include <mutex>

#include "lq_common.cuh"
#include "lq_tc_ptx.cuh"
#include "lq_sched.cuh"

namespace lq {

int tile_pick_splits(int M, int N, int K);                                   // lq_gemm_tile.cu
size_t tile_workspace_bytes(int M, int N, int splits);                       // lq_gemm_tile.cu
int run_tile_gemm(const int8_t* x, const uint8_t* blob, const float* ascale, const float* s1, const void* bias,
                  const OutSpec& out, const PeerSync* sync, int out_mode, int M, int N, int K, int splits, void* ws,
                  size_t ws_bytes, cudaStream_t st);  // lq_gemm_tile.cu
int tile_output_grid(int M, int N, int K, int splits);                            // lq_gemm_tile.cu
size_t decode_tc_workspace_bytes(int M, int N, int K);                       // lq_decode_tc.cu
int run_decode_tc(const int8_t* x, const uint8_t* blob, const float* ascale, const float* s1, const void* bias,
                  const OutSpec& out, const PeerSync* sync, int out_mode, int M, int N, int K, void* ws,
                  size_t ws_bytes, cudaStream_t st);  // lq_decode_tc.cu
size_t gemv_blob_workspace_bytes(int N, int K);                              // lq_gemv_blob.cu
int run_gemv_blob_ws(const int8_t* x, const uint8_t* blob, const float* ascale, const float* s1, const void* bias,
                     const OutSpec& out, const PeerSync* sync, int out_dtype, int M, int N, int K, void* ws,
                     size_t ws_bytes, cudaStream_t st);  // lq_gemv_blob.cu
int decode_tc_grid(int N, int K);                                            // lq_decode_tc.cu
bool pair_serves(int M, int N, int K);                                       // lq_gemm_pair.cu
bool i8_pair_serves(int M, int N, int K);                                    // lq_i8_pair.cu
int run_i8_pair_gemm(const int8_t* x, const int8_t* w, const float* ascale, const float* s1, const void* bias, void* out,
                     int out_mode, int M, int N, int K, cudaStream_t st);
int run_unpack_blob_i8(const uint8_t* blob, int8_t* w, int N, int K, cudaStream_t st);   // lq_elementwise.cu
bool pair_prefers(int M, int N, int K);                                      // lq_gemm_pair.cu
size_t pair_workspace_bytes(int M, int N, int K);                                // lq_gemm_pair.cu
int pair_grid(int M, int N, int K);                                              // lq_gemm_pair.cu
int run_pair_gemm(const int8_t* x, const uint8_t* blob, const float* ascale, const float* s1, const void* bias,
                  const OutSpec& out, const PeerSync* sync, int out_mode, int M, int N, int K, void* ws, size_t ws_bytes,
                  cudaStream_t st);  // lq_gemm_pair.cu
int gemv_blob_grid(int N, int K);                                            // lq_gemv_blob.cu
int launch_gemv_plain_f32(const int8_t* x, const uint8_t* nibbles, const uint8_t* s_u8,
                          const uint8_t* off_a, const float* ascale, const float* s1, float* y, int M,
                          int N, int K, int G, cudaStream_t st);  // lq_gemv.cu

constexpr int kTileBytes = 8704;     // weight tile in the blob: 8192 nibble bytes + 512 metadata bytes
constexpr int kI8TileBytes = 16384;  // INT8 weight tile: 128 rows x 128 bytes
constexpr int kThreads = 512;
constexpr uint64_t kWaitLimitNs = 2000000000ull;
constexpr int kOutI32 = 3;           // internal output mode: raw int32

enum WeightSource { kBlob = 0, kInt8 = 1 };

struct GemmArgs {
  const uint8_t* blob;     // kBlob: tile blob
  const float* ascale;     // [M]
  const float* s1;         // [N]
  void* out;               // [M, N] in out_mode's type
  int32_t* slots;          // workspace: per-slot 128 x BN int32 partial sums (all zero between launches)
  int32_t* counters;       // workspace: per-slot k-steps received so far (all zero between launches)
  int* status;
  int out_mode;            // LQ_DT_* or kOutI32
  int M, N, K;
  int kt_total;            // K / 128
  int n_tiles, m_tiles;
  int fixed_split;         // 0: stream-K ranges; S >= 1: every tile is cut into S equal k-ranges
};

template <int BN, int NS, int NT, int NACC, int WSRC>
struct TcCfg {
  static constexpr int kXStage = BN * 128;
  static constexpr int kWStage = WSRC == kBlob ? kTileBytes : kI8TileBytes;
  static constexpr int kACols = WSRC == kInt8 ? 0 : 32 * NS;   // one operand stage per shared-memory stage
  static constexpr int kColsNeeded = NACC * BN + kACols;
  static constexpr int kTmemCols = kColsNeeded <= 32 ? 32 : kColsNeeded <= 64 ? 64 : kColsNeeded <= 128 ? 128
                                   : kColsNeeded <= 256 ? 256 : 512;
  static constexpr int kNumBars = 3 * NS + 2 * NACC;
  static constexpr int kBarBytes = kNumBars * 8 + 16;
  static constexpr int kSmemBytes = 1024 /* alignment slack */ + NS * (kXStage + kWStage) + kBarBytes;
  static_assert(kColsNeeded <= 512, "tensor memory budget exceeded");
  static_assert(kSmemBytes <= 232448, "shared memory budget exceeded");
  static_assert(kSmemBytes > 116 * 1024, "one CTA per SM is assumed (tensor memory is allocated whole)");
};

// Bounded barrier wait performed by lane 0 on behalf of a converged warp.
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, int lane) {
  int done = 1;
  if (lane == 0) done = ptx::mbar_wait_bounded(bar, parity, kWaitLimitNs) ? 1 : 0;
  done = __shfl_sync(0xffffffffu, done, 0);
  return done != 0;
}

__device__ __forceinline__ void epilogue_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

template <int BN, int NS, int NT, int NACC, int WSRC>
__global__ void __launch_bounds__(kThreads, 1)
w4a8_tc_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
               const GemmArgs args) {
  using Cfg = TcCfg<BN, NS, NT, NACC, WSRC>;
  constexpr bool kDequant = WSRC != kInt8;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw_addr);

  const uint32_t xs = base;                                  // NS activation stages (1024-aligned)
  const uint32_t ws = xs + NS * Cfg::kXStage;                // NS weight stages
  const uint32_t bars = ws + NS * Cfg::kWStage;
  const uint32_t bar_full = bars;                            // [NS] both TMA copies of the stage landed
  const uint32_t bar_empty = bar_full + NS * 8;              // [NS] stage may be overwritten
  const uint32_t bar_aready = bar_empty + NS * 8;            // [NS] dequantised operand is in TMEM
  const uint32_t bar_accfull = bar_aready + NS * 8;          // [NACC] accumulator final
  const uint32_t bar_accempty = bar_accfull + NACC * 8;      // [NACC] accumulator drained
  const uint32_t tmem_slot = bar_accempty + NACC * 8;
  uint8_t* gen_bars = smem + (bars - base);
  volatile uint32_t* tmem_slot_p = reinterpret_cast<volatile uint32_t*>(gen_bars + Cfg::kNumBars * 8);
  volatile int* last_flag = reinterpret_cast<volatile int*>(gen_bars + Cfg::kNumBars * 8 + 4);
  volatile int* wait_flag = reinterpret_cast<volatile int*>(gen_bars + Cfg::kNumBars * 8 + 8);  // [2]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < NS; ++s) {
      ptx::mbar_init(bar_full + 8 * s, 2);                   // one expect_tx arrival per producer thread
      ptx::mbar_init(bar_empty + 8 * s, 1);                    // the MMA warp's commit
      ptx::mbar_init(bar_aready + 8 * s, 128);                 // the 128 threads of one dequant set
    }
    for (int b = 0; b < NACC; ++b) {
      ptx::mbar_init(bar_accfull + 8 * b, 1);
      ptx::mbar_init(bar_accempty + 8 * b, 128);
    }
    ptx::fence_mbar_init();
    ptx::prefetch_tensormap(&tmap_x);
    if (WSRC != kBlob) ptx::prefetch_tensormap(&tmap_w);
  }
  if (warp == 1) {
    ptx::tmem_alloc(tmem_slot, Cfg::kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_p;
  const uint32_t tmem_a = tmem_base + NACC * BN;   // NS operand stages of 32 columns behind the accumulators

  if (warp == 0 || warp == 2) {
    // ------------------------------------------------------------------ producers
    // warp 0 streams the weight tiles, warp 2 the activation boxes.  The whole warp walks the loop
    // and polls (a warp that stays converged costs far less than one lane spinning while 31 wait);
    // lane 0 alone announces the byte count and issues the copy.
    const bool weights = (warp == 0);
    SegmentWalk walk(SchedArgs{args.kt_total, args.n_tiles, args.m_tiles, args.fixed_split}, blockIdx.x, gridDim.x);
    Segment sg;
    Ring<NS> ring;
    int issued = 0;
    bool ok = true;
    while (ok && walk.next(sg)) {
      const int nt = sg.tile % args.n_tiles, mt = sg.tile / args.n_tiles;
      const uint8_t* wsrc = WSRC == kBlob ? args.blob + ((size_t)nt * args.kt_total + sg.kb) * kTileBytes : nullptr;
      for (int kt = sg.kb; kt < sg.ke; ++kt) {
        if (!ptx::mbar_wait_bounded(bar_empty + 8 * ring.s, ring.ph ^ 1u, kWaitLimitNs)) {
          atomicExch(args.status, 101);
          ok = false;
          break;
        }
        const uint32_t full = bar_full + 8 * ring.s;
        if (lane == 0) {
          if (weights) {
            ptx::mbar_expect_tx(full, Cfg::kWStage);
            if (WSRC == kBlob) {
              ptx::bulk_load(ws + ring.s * Cfg::kWStage, wsrc, kTileBytes, full);
            } else {
              ptx::tensor_load_2d(ws + ring.s * Cfg::kWStage, &tmap_w, kt * 128, nt * 128, full);
            }
          } else {
            ptx::mbar_expect_tx(full, Cfg::kXStage);
            ptx::tensor_load_2d(xs + ring.s * Cfg::kXStage, &tmap_x, kt * 128, mt * BN, full);
          }
        }
        if (WSRC == kBlob) wsrc += kTileBytes;
        ring.advance();
        ++issued;
      }
    }
    if (!ok) {
      // copies already issued still write shared memory: let them land before the CTA exits
      Ring<NS> back;
      const int first = issued > NS ? issued - NS : 0;
      for (int i = 0; i < issued; ++i) {
        if (i >= first) ptx::mbar_wait_bounded(bar_full + 8 * back.s, back.ph, kWaitLimitNs);
        back.advance();
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issue
    // The whole warp walks the loop; one elected lane issues (see ptx::elect_one).  With dequantisation the only wait per k-step is on the
    // operand barrier: the dequant warps saw the stage's full barrier (weights and activations)
    // before they produced the operand, so "operand ready" implies "activations landed".
    constexpr uint32_t idesc = ptx::idesc_i8(BN);
    const bool leader = ptx::elect_one();
    SegmentWalk walk(SchedArgs{args.kt_total, args.n_tiles, args.m_tiles, args.fixed_split}, blockIdx.x, gridDim.x);
    Segment sg;
    Ring<NS> ring;
    Ring<NACC> accring;
    bool ok = true;
    while (ok && walk.next(sg)) {
      ok = __all_sync(0xffffffffu, ptx::mbar_wait_bounded(bar_accempty + 8 * accring.s, accring.ph ^ 1u, kWaitLimitNs));
      if (!ok) {
        if (leader) atomicExch(args.status, 106);
        break;
      }
      ptx::tc_fence_after();
      const uint32_t tmem_acc = tmem_base + accring.s * BN;
      for (int kt = sg.kb; kt < sg.ke; ++kt) {
        ok = __all_sync(0xffffffffu, ptx::mbar_wait_bounded((kDequant ? bar_aready : bar_full) + 8 * ring.s, ring.ph,
                                                            kWaitLimitNs));
        if (!ok) {
          if (leader) atomicExch(args.status, 102);
          break;
        }
        ptx::tc_fence_after();
        const uint32_t xb = xs + ring.s * Cfg::kXStage;
        const uint32_t ab = tmem_a + ring.s * 32;
        const uint32_t wb = ws + ring.s * Cfg::kWStage;
        if (leader) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint64_t bdesc = ptx::smem_desc_sw128(xb + j * 32);
            const uint32_t accumulate = (kt > sg.kb || j > 0) ? 1u : 0u;
            if (kDequant) ptx::mma_i8_ts(tmem_acc, ab + j * 8, bdesc, idesc, accumulate);
            else ptx::mma_i8_ss(tmem_acc, ptx::smem_desc_sw128(wb + j * 32), bdesc, idesc, accumulate);
          }
          // one commit recycles the shared-memory stage and the tensor-memory operand stage: the
          // dequant warps have finished with both before they signalled "operand ready"
          ptx::tc_commit(bar_empty + 8 * ring.s);
        }
        ring.advance();
      }
      if (ok && leader) ptx::tc_commit(bar_accfull + 8 * accring.s);
      accring.advance();
    }
  } else if ((warp >= 4 && warp < 8) || warp >= 12) {
    // ------------------------------------------------------------------ dequant
    // Two sets of four warps (4..7 and 12..15) take alternate k-steps, so each set has two k-step
    // periods to hide its shared-load and tcgen05.st latencies.  Operand stage s lives in tensor
    // memory columns [32 s, 32 s + 32) and is tied to shared-memory stage s: when the stage's full
    // barrier fires for k-step i, the producer had seen the commit of k-step i - NS, so the MMAs
    // that read the previous contents of both are complete and no separate "operand free"
    // barrier is needed.
    if (kDequant) {
      const int my_set = warp < 8 ? 0 : 1;
      int step_set = 0;   // set that owns the current k-step
      const int quad = warp & 3;               // TMEM lane quadrant this warp may access
      const int row = quad * 32 + lane;        // weight row inside the tile == TMEM lane
      const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
      SegmentWalk walk(SchedArgs{args.kt_total, args.n_tiles, args.m_tiles, args.fixed_split}, blockIdx.x, gridDim.x);
      Segment sg;
      Ring<NS> ring;
      bool ok = true;
      while (ok && walk.next(sg)) {
        for (int kt = sg.kb; kt < sg.ke; ++kt) {
          const bool mine = step_set == my_set;
          step_set ^= 1;
          if (!mine) {                           // another set's k-step
            ring.advance();
            continue;
          }
          if (!ptx::mbar_wait_bounded(bar_full + 8 * ring.s, ring.ph, kWaitLimitNs)) {
            atomicExch(args.status, 103);
            ok = false;
            break;
          }
          __syncwarp();   // lanes leave the poll loop one by one; tcgen05.st / wait::st need the warp converged
          ptx::tc_fence_after();
          const uint8_t* wst = smem + (ws - base) + ring.s * Cfg::kWStage;
          uint4 ch[4];
#pragma unroll
          for (int c = 0; c < 4; ++c) ch[c] = *reinterpret_cast<const uint4*>(wst + (c * 128 + row) * 16);
          const uint32_t meta = *reinterpret_cast<const uint32_t*>(wst + 8192 + row * 4);
          const uint32_t step0 = meta & 0xffu, a0 = ((meta >> 8) & 0xffu) * 0x01010101u;
          const uint32_t step1 = (meta >> 16) & 0xffu, a1 = (meta >> 24) * 0x01010101u;
          uint32_t v[32];
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const uint32_t step = c < 2 ? step0 : step1;
            const uint32_t ab = c < 2 ? a0 : a1;
            const uint32_t pk[4] = {ch[c].x, ch[c].y, ch[c].z, ch[c].w};
#pragma unroll
            for (int h = 0; h < 4; ++h) {
              v[8 * c + 2 * h] = lqq_dequant4(pk[h] & 0x0F0F0F0Fu, step, ab);
              v[8 * c + 2 * h + 1] = lqq_dequant4((pk[h] >> 4) & 0x0F0F0F0Fu, step, ab);
            }
          }
          ptx::tmem_st32(tmem_a + lane_addr + ring.s * 32, v);
          // Publish at once: the other dequant set covers the next k-step while these stores drain.
          // (Deferring this to the set's next iteration would tie MMA i to the arrival of the TMA
          // data of k-step i + 2 and eat two stages of prefetch depth.)
          ptx::tc_wait_st();
          ptx::tc_fence_before();
          ptx::mbar_arrive(bar_aready + 8 * ring.s);
          ring.advance();
        }
      }
    }
  } else if (warp >= 8 && warp < 12) {
    // ------------------------------------------------------------------ epilogue
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
    const int et = threadIdx.x - 256;          // 0..127 inside the epilogue group
    SegmentWalk walk(SchedArgs{args.kt_total, args.n_tiles, args.m_tiles, args.fixed_split}, blockIdx.x, gridDim.x);
    Segment sg;
    Ring<NACC> accring;
    int seg = 0;
    bool ok = true;
    while (ok && walk.next(sg)) {
      const int b = accring.s;
      const uint32_t phb = accring.ph;
      accring.advance();
      // One thread performs the bounded wait and publishes the outcome, so that the 128 threads
      // always agree on it (they meet at named barriers below and must never split up).
      const int fslot = seg & 1;
      ++seg;
      if (et == 0) {
        const bool done = ptx::mbar_wait_bounded(bar_accfull + 8 * b, phb, kWaitLimitNs);
        if (!done) atomicExch(args.status, 105);
        wait_flag[fslot] = done ? 1 : 0;
      }
      epilogue_barrier();
      if (wait_flag[fslot] == 0) {
        ok = false;
        break;
      }
      ptx::tc_fence_after();
      const int nt = sg.tile % args.n_tiles, mt = sg.tile / args.n_tiles;
      const int m0 = mt * BN;
      const long n = (long)nt * 128 + row;
      const bool n_ok = n < args.N;
      const int cols = (args.M - m0) < BN ? (args.M - m0) : BN;   // valid token columns of this tile
      const uint32_t tmem_acc = tmem_base + b * BN + lane_addr;
      const float w_scale = (n_ok && args.out_mode != kOutI32) ? __ldg(args.s1 + n) : 0.f;
      if (sg.whole) {
#pragma unroll 1
        for (int c0 = 0; c0 < cols; c0 += 16) {
          int v[16];
          ptx::tmem_ld16(tmem_acc + c0, v);
          // token scales of the chunk, fetched while the tensor-memory load is in flight
          float sc[16];
          if (args.out_mode != kOutI32) {
            if (c0 + 16 <= cols) {
              const float4* sp = reinterpret_cast<const float4*>(args.ascale + m0 + c0);
#pragma unroll
              for (int q4 = 0; q4 < 4; ++q4) {
                const float4 f = __ldg(sp + q4);
                sc[4 * q4] = f.x; sc[4 * q4 + 1] = f.y; sc[4 * q4 + 2] = f.z; sc[4 * q4 + 3] = f.w;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 16; ++j) sc[j] = (c0 + j < cols) ? __ldg(args.ascale + m0 + c0 + j) : 0.f;
            }
          }
          ptx::tc_wait_ld();
          if (c0 + 16 >= cols) {          // last chunk read: the MMA warp may reuse the accumulator
            ptx::tc_fence_before();
            ptx::mbar_arrive(bar_accempty + 8 * b);
          }
          if (n_ok)
            epi_store_cols(args.out, args.out_mode, (size_t)(m0 + c0) * args.N + n, args.N, v, sc, w_scale, 0.f, false,
                           cols - c0);
        }
      } else {
        int32_t* slot = args.slots + (size_t)sg.slot * (128 * BN);
#pragma unroll 1
        for (int c0 = 0; c0 < cols; c0 += 16) {
          int v[16];
          ptx::tmem_ld16(tmem_acc + c0, v);
          ptx::tc_wait_ld();
          if (c0 + 16 >= cols) {
            ptx::tc_fence_before();
            ptx::mbar_arrive(bar_accempty + 8 * b);
          }
          if (n_ok) {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (c0 + j < cols) atomicAdd(slot + (c0 + j) * 128 + row, v[j]);
          }
        }
        __threadfence();
        epilogue_barrier();
        if (et == 0) {
          const int add = sg.ke - sg.kb;
          const int before = atomicAdd(args.counters + sg.slot, add);
          *last_flag = (before + add == args.kt_total) ? 1 : 0;
        }
        epilogue_barrier();
        const bool last = *last_flag != 0;
        epilogue_barrier();                      // everyone has read the flag before it can be rewritten
        if (last) {
          __threadfence();
          if (n_ok) {
#pragma unroll 1
            for (int c0 = 0; c0 < cols; c0 += 16) {
              int v[16];
              float sc[16];
#pragma unroll
              for (int j = 0; j < 16; ++j) {       // all loads of the chunk first: one L2 round trip
                int32_t* p = slot + (c0 + j) * 128 + row;
                v[j] = (c0 + j < cols) ? __ldcg(p) : 0;
                sc[j] = (c0 + j < cols && args.out_mode != kOutI32) ? __ldg(args.ascale + m0 + c0 + j) : 0.f;
              }
              epi_store_cols(args.out, args.out_mode, (size_t)(m0 + c0) * args.N + n, args.N, v, sc, w_scale, 0.f, false,
                             cols - c0);
            }
            // Zeroed in a pass of its own: a load issued behind a store to the same slot waits for it, chunk
            // after chunk (measured in the CTA-pair kernel: 2.5 x the time of the whole pass).
#pragma unroll 1
            for (int c0 = 0; c0 < cols; c0 += 16) {
#pragma unroll
              for (int j = 0; j < 16; ++j)
                if (c0 + j < cols) __stcg(slot + (c0 + j) * 128 + row, 0);
            }
          }
          if (et == 0) args.counters[sg.slot] = 0;
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

// Tensor map over a row-major byte matrix [rows, row_bytes] with a (box_rows x box_bytes) box whose
// rows are stored with the swizzle that matches their length; rows out of range read as zero.
int make_byte_matrix_map(CUtensorMap* map, const void* ptr, long rows, long row_bytes, int box_rows,
                                int box_bytes) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) {
    record_cuda_error(cudaErrorUnknown, "cuTensorMapEncodeTiled entry point not found");
    return LQ_ERR_CUDA;
  }
  const cuuint64_t dims[2] = {(cuuint64_t)row_bytes, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
  const cuuint32_t box[2] = {(cuuint32_t)box_bytes, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1u, 1u};
  const CUtensorMapSwizzle sw = box_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    record_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled failed");
    return LQ_ERR_CUDA;
  }
  return LQ_OK;
}

static int pick_bn(int M, int K = 0) {
  (void)K;
  if (M <= 16) return 16;
  if (M <= 32) return 32;
  if (M <= 64) return 64;
  if (M <= 128) return 128;
  // Two 192-token accumulators.  A single 256-token accumulator (5 stages) measured 20-40 % faster
  // on long-K shapes but produced intermittent launch failures on a 8192 x 28672 layer; it stays
  // off until the cause is understood.
  return 192;
}

struct Plan {
  int cfg;   // kernel configuration key (differs from bn only in experiments)
  int bn, n_tiles, m_tiles, grid, fixed_split;
  long tiles;
  size_t slots, ws_bytes;
};

// splitk: 0 = stream-K over one CTA per SM, 1 = whole tiles only, S > 1 = every tile cut into S ranges.
static Plan make_plan(int M, int N, int K, int splitk) {
  Plan p;
  p.bn = pick_bn(M, K);
  p.cfg = p.bn;
  p.n_tiles = (N + 127) / 128;
  p.m_tiles = (M + p.bn - 1) / p.bn;
  p.tiles = (long)p.n_tiles * p.m_tiles;
  const int kt = K / 128;
  const int sms = sm_count();
  if (splitk > kt) splitk = kt;
  p.fixed_split = splitk < 0 ? 0 : splitk;
  const long units = p.fixed_split == 0 ? p.tiles * kt : p.tiles * p.fixed_split;
  p.grid = (int)(units < sms ? units : sms);
  p.slots = p.fixed_split == 0 ? (size_t)p.grid : p.fixed_split == 1 ? 0 : (size_t)p.tiles;
  // slots of 128 x BN int32 followed by one counter per slot (padded to 256 bytes)
  p.ws_bytes = p.slots == 0 ? 0 : p.slots * (size_t)(128 * p.bn * 4) + ((p.slots * 4 + 255) / 256) * 256;
  return p;
}

template <int BN, int NS, int NT, int NACC, int WSRC>
static int launch_cfg(const CUtensorMap& tx, const CUtensorMap& tw, const GemmArgs& a, int grid, cudaStream_t st) {
  using Cfg = TcCfg<BN, NS, NT, NACC, WSRC>;
  auto kern = &w4a8_tc_kernel<BN, NS, NT, NACC, WSRC>;
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
  kern<<<grid, kThreads, Cfg::kSmemBytes, st>>>(tx, tw, a);
  return check_launch("w4a8_tc_kernel");
}

template <int WSRC>
static int dispatch_bn(int bn, const CUtensorMap& tx, const CUtensorMap& tw, const GemmArgs& a, int grid,
                       cudaStream_t st) {
  constexpr int NT = 1;   // unused: operand stages follow the shared-memory ring
  if constexpr (WSRC == kInt8) {
    switch (bn) {
      case 16: return launch_cfg<16, 9, NT, 2, WSRC>(tx, tw, a, grid, st);
      case 32: return launch_cfg<32, 9, NT, 2, WSRC>(tx, tw, a, grid, st);
      case 64: return launch_cfg<64, 8, NT, 2, WSRC>(tx, tw, a, grid, st);
      case 128: return launch_cfg<128, 6, NT, 2, WSRC>(tx, tw, a, grid, st);
      default: return launch_cfg<192, 5, NT, 2, WSRC>(tx, tw, a, grid, st);
    }
  } else {
    // tensor memory: 2 * BN accumulator columns + 32 * NS operand columns <= 512
    switch (bn) {
      case 16: return launch_cfg<16, 14, NT, 2, WSRC>(tx, tw, a, grid, st);
      case 32: return launch_cfg<32, 14, NT, 2, WSRC>(tx, tw, a, grid, st);
      case 64: return launch_cfg<64, 12, NT, 2, WSRC>(tx, tw, a, grid, st);
      case 128: return launch_cfg<128, 8, NT, 2, WSRC>(tx, tw, a, grid, st);
      default: return launch_cfg<192, 4, NT, 2, WSRC>(tx, tw, a, grid, st);
    }
  }
}

// x: [M,K] int8 tokens.  w: tile blob, or [N,K] int8 weights.
template <int WSRC>
static int run_gemm(const int8_t* x, const void* w, const float* ascale,
                    const float* s1, void* out, int out_mode, int M, int N, int K, int splitk, void* wsp,
                    size_t ws_bytes, cudaStream_t st) {
  if (int rc = lq_check_device()) return rc;
  const Plan p = make_plan(M, N, K, splitk);
  if (p.ws_bytes && (!wsp || ws_bytes < p.ws_bytes)) return LQ_ERR_WORKSPACE;
  CUtensorMap tx, tw;
  int rc = make_byte_matrix_map(&tx, x, M, K, p.bn, 128);
  if (rc) return rc;
  if (WSRC == kBlob) tw = tx;
  else rc = make_byte_matrix_map(&tw, w, N, K, 128, 128);
  if (rc) return rc;
  GemmArgs a;
  a.blob = WSRC == kBlob ? static_cast<const uint8_t*>(w) : nullptr;
  a.ascale = ascale;
  a.s1 = s1;
  a.out = out;
  a.slots = static_cast<int32_t*>(wsp);
  a.counters = p.slots ? reinterpret_cast<int32_t*>(static_cast<uint8_t*>(wsp) + p.slots * (size_t)(128 * p.bn * 4))
                       : nullptr;
  a.status = status_word();
  a.out_mode = out_mode;
  a.M = M;
  a.N = N;
  a.K = K;
  a.kt_total = K / 128;
  a.n_tiles = p.n_tiles;
  a.m_tiles = p.m_tiles;
  a.fixed_split = p.fixed_split;
  if (!a.status) return LQ_ERR_CUDA;
  return dispatch_bn<WSRC>(p.cfg, tx, tw, a, p.grid, st);
}

}  // namespace lq

using namespace lq;

extern "C" {

int lq_gemm_pick_splitk(int M, int N, int K, int env_override) {
  // 0 selects stream-K scheduling, which balances any shape over the SMs; an explicit
  // LIQUIDGEMM_SPLITK only applies to the decode range, as in the reference.
  if (M <= 0 || N <= 0 || K < 128) return 0;
  if (env_override > 0 && M <= 128) {
    const int kt = K / 128;
    return env_override > kt ? kt : env_override;
  }
  return 0;
}

// Which kernel serves (M, splitk).
enum RouteKind {
  kRoutePersistent,   // one CTA per SM, stream-K or a fixed split (explicit requests above 128 tokens, splitk -1)
  kRouteTile,         // two CTAs per SM, one tile each, `splits` int32 planes + finish pass when splits > 1
  kRouteGemv,         // streaming dp4a GEMV over the blob (scaled outputs only)
  kRouteDecodeTc,     // streaming tensor-core kernel, one launch, atomic join
  kRoutePair,         // CTA pairs, 256 channels x 192 tokens per tile (prefill)
  kRouteUnpackI8,     // very large token counts: unpack the blob to INT8 once, then the INT8 x INT8 pair kernel
};
struct Route {
  RouteKind kind;
  int splits;
};
// The dp4a streaming GEMV over the blob serves one token, two on matrices up to 64 M weights (28672 x 4096 at two
// tokens: 15.7 us against the tile kernel's 14.8) and three or four on matrices up to 16 M weights (measured on
// the Llama-3.1-8B shapes against the tensor-core decode kernel: 4096 x 4096 5.2 vs 5.7 us at three tokens;
// 6144 x 4096 equal; 4096 x 14336 11.2 vs 10.5 us); it only produces scaled outputs, the int32 entry point always
// uses tensor cores.
constexpr int kGemvBlobMaxM = 4;

// Largest decode batch of the single-launch streaming tensor-core kernel: its one-atomic-per-element
// join is cheap only while a CTA holds few tokens.  LQ_DECODE_TC_MAX_M (16 or 32) moves the limit for
// measurements.
static int decode_tc_max_m() {
  static const int v = []() {
    const char* e = getenv("LQ_DECODE_TC_MAX_M");
    const int n = e ? atoi(e) : 16;
    return n <= 0 ? 0 : n >= 32 ? 32 : 16;
  }();
  return v;
}

// From this many tokens on, shapes with whole 256-channel blocks go to the CTA-pair kernel where it is expected
// to win (pair_prefers).  LQ_PAIR_MIN_M moves the limit for measurements; 0 switches the kernel off.
static int pair_min_m() {
  static const int v = []() {
    const char* e = getenv("LQ_PAIR_MIN_M");
    const int n = e ? atoi(e) : 256;
    return n <= 0 ? (1 << 30) : n < 129 ? 129 : n;
  }();
  return v;
}

// LQ_PAIR_ALWAYS=1: every shape the pair kernel serves goes to it (tests and measurements).
static bool pair_forced() {   // read at every call: a test sets and clears it inside one process
  const char* e = getenv("LQ_PAIR_ALWAYS");
  return e && atoi(e) != 0;
}

static bool gemv_serves(int M, int N, int K) {
  static const int cap = []() {   // LQ_GEMV_MAX_M (0..4) lowers the limit for measurements
    const char* e = getenv("LQ_GEMV_MAX_M");
    return e ? atoi(e) : kGemvBlobMaxM;
  }();
  if (M > cap) return false;
  const long w = (long)N * K;
  return M == 1 || (M == 2 && w <= (1L << 26)) || (M <= kGemvBlobMaxM && w <= (1L << 24));
}

// Large token counts on layers the INT8 pair kernel serves: unpacking the whole blob to INT8 once (a pass over
// N x K bytes of scratch: 38 us for 28672 x 4096) and running the INT8 x INT8 pair kernel, which keeps the tensor
// pipe 95 % busy, beats unpacking inside the main loop (71 %).  Measured in one process: at 8192 tokens qkv 158.6
// -> 144.0 us, o 108.9 -> 93.8, gate_up 720.6 -> 660.4; at 5120 tokens 6 / 3 / 2.5 %; at 3072 tokens qkv 6 %, o
// 2 %, gate_up 5 % slower; at 2048 all slower.  down (K = 14336, where the W4 kernel's epilogues weigh least) is
// level at every size: layers with K >= 8192 stay on the W4 pair kernel, and so do layers above 256 MB of INT8
// weights (the scratch would be larger than that).  LQ_UNPACK_I8_MIN_M replaces both limits (0 switches the route
// off).  Running the two kernels overlapped (the GEMM launched programmatically behind a persistent unpack kernel,
// waiting per channel block on counts of finished tiles) was measured as well: bit-exact, 3-7 % SLOWER than one after
// the other (the unpack's memory traffic slows the GEMM it runs beside); not kept.
static bool unpack_i8_serves(int M, int N, int K) {
  const char* e = getenv("LQ_UNPACK_I8_MIN_M");   // read at every call: a measurement switch
  const int lim = e ? atoi(e) : ((size_t)N * K <= ((size_t)1 << 25) ? 3072 : 5120);
  return lim > 0 && M >= lim && K < 8192 && (size_t)N * K <= ((size_t)256 << 20) && i8_pair_serves(M, N, K);
}

static Route route_for(int M, int N, int K, int splitk, bool scaled, bool single_dest = true) {
  const int kt = K / 128;
  if (splitk == -1) return {kRoutePersistent, 0};
  if (M <= 128) {
    if (splitk == 0) {
      if (scaled && gemv_serves(M, N, K)) return {kRouteGemv, 0};
      // Small matrices (up to 32 M weights) only: on larger ones the tile kernel's whole tiles (or its planes
      // and finish pass) are ahead since the MMA issue became cheap (28672 x 4096 at 8 tokens: 14.7 vs 16.7 us,
      // 4096 x 14336: 10.4 vs 10.8 us; 6144 x 4096: 7.3 vs 7.0 us, 4096 x 4096: 6.6 vs 6.0 us).
      if (M <= decode_tc_max_m() && (long)N * K <= (1L << 25)) return {kRouteDecodeTc, 0};
    }
    int S = splitk > 0 ? splitk : tile_pick_splits(M, N, K);
    if (S > kt) S = kt;
    return {kRouteTile, S < 1 ? 1 : S};
  }
  // Automatic choice above 128 tokens: the CTA-pair kernel where its cost model expects it to win (large
  // M x N on layers with whole 256-channel blocks), else the two-CTAs-per-SM tile kernel; the persistent
  // stream-K kernel stays reachable through an explicit split argument.
  if (splitk == 0) {
    if (single_dest && !pair_forced() && unpack_i8_serves(M, N, K)) return {kRouteUnpackI8, 0};
    if (M >= pair_min_m() && (pair_forced() ? pair_serves(M, N, K) : pair_prefers(M, N, K))) return {kRoutePair, 0};
    return {kRouteTile, tile_pick_splits(M, N, K)};
  }
  return {kRoutePersistent, splitk};
}

static size_t route_ws_bytes(const Route& r, int M, int N, int K) {
  switch (r.kind) {
    case kRouteGemv: return gemv_blob_workspace_bytes(N, K);
    case kRouteDecodeTc: return decode_tc_workspace_bytes(M, N, K);
    case kRouteTile: return tile_workspace_bytes(M, N, r.splits);
    case kRoutePair: return pair_workspace_bytes(M, N, K);
    case kRouteUnpackI8: return (size_t)N * K;   // scratch: the INT8 weights
    default: return make_plan(M, N, K, r.splits).ws_bytes;
  }
}

// The size does not know whether the caller wants scaled or int32 outputs: the larger of the two routes.
size_t lq_gemm_workspace_bytes(int M, int N, int K, int splitk) {
  if (M <= 0 || N <= 0 || K < 128) return 0;
  const size_t a = route_ws_bytes(route_for(M, N, K, splitk, true), M, N, K);
  const size_t b = route_ws_bytes(route_for(M, N, K, splitk, false), M, N, K);
  return a > b ? a : b;
}

// 0: none, 1: scratch (split-K planes; any content), 2: the shared buffer that is all zero between calls.
int lq_gemm_workspace_kind(int M, int N, int K, int splitk) {
  if (lq_gemm_workspace_bytes(M, N, K, splitk) == 0) return 0;
  const RouteKind k = route_for(M, N, K, splitk, true).kind;
  return (k == kRouteTile || k == kRouteUnpackI8) ? 1 : 2;   // 1: scratch, 2: all-zero reduction buffer
}

// Kernel launches one call makes (for callers that count them).
int lq_gemm_launches(int M, int N, int K, int splitk) {
  if (M <= 0 || N <= 0 || K < 128) return 0;
  const Route r = route_for(M, N, K, splitk, true);
  return ((r.kind == kRouteTile && r.splits > 1) || r.kind == kRouteUnpackI8) ? 2 : 1;
}

static int blob_gemm(const int8_t* x, const uint8_t* blob, const float* ascale, const float* s1, const void* bias,
                     void* out, int out_mode, int M, int N, int K, int splitk, void* ws, size_t ws_bytes,
                     cudaStream_t st) {
  if (!x || !blob || !out || M < 0 || N <= 0 || K <= 0) return LQ_ERR_BAD_ARG;
  if (K % 128) return LQ_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(blob)) % 16) return LQ_ERR_BAD_ARG;
  if (M == 0) return LQ_OK;
  const Route r = route_for(M, N, K, splitk, out_mode != kOutI32);
  if (r.kind != kRoutePersistent) {
    if (int rc = lq_check_device()) return rc;
  }
  switch (r.kind) {
    case kRouteGemv:
      return run_gemv_blob_ws(x, blob, ascale, s1, bias, single_out(out, N), nullptr, out_mode, M, N, K, ws, ws_bytes, st);
    case kRouteDecodeTc:
      return run_decode_tc(x, blob, ascale, s1, bias, single_out(out, N), nullptr, out_mode, M, N, K, ws, ws_bytes, st);
    case kRouteTile:
      return run_tile_gemm(x, blob, ascale, s1, bias, single_out(out, N), nullptr, out_mode, M, N, K, r.splits, ws,
                           ws_bytes, st);
    case kRoutePair:
      return run_pair_gemm(x, blob, ascale, s1, bias, single_out(out, N), nullptr, out_mode, M, N, K, ws, ws_bytes, st);
    case kRouteUnpackI8: {
      if (!ws || ws_bytes < (size_t)N * K || (reinterpret_cast<uintptr_t>(ws) & 15)) return LQ_ERR_WORKSPACE;
      int8_t* w8 = static_cast<int8_t*>(ws);
      if (int rc = run_unpack_blob_i8(blob, w8, N, K, st)) return rc;
      return run_i8_pair_gemm(x, w8, ascale, s1, bias, out, out_mode, M, N, K, st);
    }
    default:
      if (bias) return LQ_ERR_BAD_ARG;   // the persistent kernel has no bias epilogue
      return run_gemm<kBlob>(x, blob, ascale, s1, out, out_mode, M, N, K, r.splits, ws, ws_bytes, st);
  }
}

int lq_w4a8_gemm_i32(const int8_t* x_i8, const uint8_t* blob, int32_t* acc, int M, int N, int K, int splitk,
                     void* workspace, size_t workspace_bytes, void* stream) {
  return blob_gemm(x_i8, blob, nullptr, nullptr, nullptr, acc, kOutI32, M, N, K, splitk, workspace, workspace_bytes,
                   as_stream(stream));
}

int lq_w4a8_gemm_fused(const int8_t* x_i8, const uint8_t* blob, const float* ascale, const float* s1, void* y,
                       int out_dtype, int M, int N, int K, int splitk, void* workspace, size_t workspace_bytes,
                       void* stream) {
  if (!ascale || !s1 || out_dtype < 0 || out_dtype > 2) return LQ_ERR_BAD_ARG;
  return blob_gemm(x_i8, blob, ascale, s1, nullptr, y, out_dtype, M, N, K, splitk, workspace, workspace_bytes,
                   as_stream(stream));
}

int lq_w4a8_linear_bias(const int8_t* x_i8, const uint8_t* blob, const float* ascale, const float* s1,
                        const void* bias, void* y, int out_dtype, int M, int N, int K, void* workspace,
                        size_t workspace_bytes, void* stream) {
  if (!ascale || !s1 || out_dtype < 0 || out_dtype > 2) return LQ_ERR_BAD_ARG;
  if (bias && (reinterpret_cast<uintptr_t>(bias) % (out_dtype == LQ_DT_F32 ? 4 : 2))) return LQ_ERR_BAD_ARG;
  return blob_gemm(x_i8, blob, ascale, s1, bias, y, out_dtype, M, N, K, 0, workspace, workspace_bytes,
                   as_stream(stream));
}

int lq_w4a8_gemm_fused_scatter_sync(const int8_t* x_i8, const uint8_t* blob, const float* ascale, const float* s1,
                                    void* const* outs, int n_outs, long ld_out, long col0, int out_dtype, int M,
                                    int N, int K, unsigned* const* peer_flags, int flag_index,
                                    const unsigned* wait_flag, unsigned wait_value, void* workspace,
                                    size_t workspace_bytes, void* stream) {
  if (!x_i8 || !blob || !ascale || !s1 || !outs || n_outs < 1 || n_outs > 8) return LQ_ERR_BAD_ARG;
  if (out_dtype < 0 || out_dtype > 2 || ld_out < N || col0 < 0 || col0 + N > ld_out) return LQ_ERR_BAD_ARG;
  if (M < 1 || N <= 0 || K < 128 || K % 128) return LQ_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(x_i8) | reinterpret_cast<uintptr_t>(blob)) % 16) return LQ_ERR_BAD_ARG;
  if (flag_index < 0) return LQ_ERR_BAD_ARG;
  OutSpec o = {};
  PeerSync ps = {};
  for (int r = 0; r < n_outs; ++r) {
    if (!outs[r] || (peer_flags && !peer_flags[r])) return LQ_ERR_BAD_ARG;
    o.ptr[r] = outs[r];
    if (peer_flags) ps.signal[r] = peer_flags[r];
  }
  o.n = n_outs;
  o.ld = ld_out;
  o.col0 = col0;
  ps.n_signal = peer_flags ? n_outs : 0;
  ps.signal_index = flag_index;
  ps.wait = wait_flag;
  ps.wait_value = wait_value;
  if (int rc = lq_check_device()) return rc;
  const Route r = route_for(M, N, K, 0, true, false);
  switch (r.kind) {
    case kRouteGemv:
      return run_gemv_blob_ws(x_i8, blob, ascale, s1, nullptr, o, &ps, out_dtype, M, N, K, workspace, workspace_bytes,
                              as_stream(stream));
    case kRouteDecodeTc:
      return run_decode_tc(x_i8, blob, ascale, s1, nullptr, o, &ps, out_dtype, M, N, K, workspace, workspace_bytes,
                           as_stream(stream));
    case kRoutePair:
      return run_pair_gemm(x_i8, blob, ascale, s1, nullptr, o, &ps, out_dtype, M, N, K, workspace, workspace_bytes,
                           as_stream(stream));
    default:
      return run_tile_gemm(x_i8, blob, ascale, s1, nullptr, o, &ps, out_dtype, M, N, K, r.splits, workspace,
                           workspace_bytes, as_stream(stream));
  }
}

int lq_w4a8_gemm_fused_scatter(const int8_t* x_i8, const uint8_t* blob, const float* ascale, const float* s1,
                               void* const* outs, int n_outs, long ld_out, long col0, int out_dtype, int M, int N,
                               int K, void* workspace, size_t workspace_bytes, void* stream) {
  return lq_w4a8_gemm_fused_scatter_sync(x_i8, blob, ascale, s1, outs, n_outs, ld_out, col0, out_dtype, M, N, K,
                                         nullptr, 0, nullptr, 0u, workspace, workspace_bytes, stream);
}

size_t lq_scatter_workspace_bytes(int M, int N, int K) {
  if (M < 1 || N <= 0 || K < 128 || K % 128) return 0;
  return route_ws_bytes(route_for(M, N, K, 0, true, false), M, N, K);
}

int lq_scatter_workspace_kind(int M, int N, int K) {
  if (lq_scatter_workspace_bytes(M, N, K) == 0) return 0;
  return route_for(M, N, K, 0, true, false).kind == kRouteTile ? 1 : 2;
}

int lq_decode_grid(int M, int N, int K) {
  if (M < 1 || N <= 0 || K < 128 || K % 128) return 0;
  const Route r = route_for(M, N, K, 0, true, false);
  switch (r.kind) {
    case kRouteGemv: return gemv_blob_grid(N, K);
    case kRouteDecodeTc: return decode_tc_grid(N, K);
    case kRoutePair: return pair_grid(M, N, K);
    default: return tile_output_grid(M, N, K, r.splits);
  }
}

size_t lq_gemm_v1_workspace_bytes(int M, int N, int K) {
  if (M <= 16) return 0;
  const size_t blob = lq_tile_blob_bytes(N, K);
  return ((blob + 255) / 256) * 256 + lq_gemm_workspace_bytes(M, N, K, 1);
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
  // scratch = re-tiled weights only; whole-tile scheduling (splitk 1) needs no reduction slots
  uint8_t* blob = static_cast<uint8_t*>(workspace);
  int rc = lq_repack_tiles(nibbles, LQ_SRC_NIBBLES, s_u8, offset_a, blob, N, K, group_size, stream);
  if (rc) return rc;
  return run_gemm<kBlob>(x_i8, blob, ascale, s1, y, LQ_DT_F32, M, N, K, 1, nullptr, 0, st);
}

// LQ_I8_PAIR=0 keeps every INT8 GEMM on the one-CTA persistent kernel (read at every call: a measurement switch).
static bool i8_pair_enabled() {
  const char* e = getenv("LQ_I8_PAIR");
  return !(e && e[0] == '0');
}

static int i8_common(const int8_t* a, const int8_t* b, const float* a_scale, const float* b_scale, void* out,
                     int out_mode, int M, int N, int K, void* stream) {
  if (!a || !b || !out || M < 0 || N <= 0 || K <= 0) return LQ_ERR_BAD_ARG;
  if (K % 128) return LQ_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b)) % 16) return LQ_ERR_BAD_ARG;
  if (M == 0) return LQ_OK;
  // whole-tile scheduling: the plain INT8 entry points take no workspace
  if (i8_pair_serves(M, N, K) && i8_pair_enabled())
    return run_i8_pair_gemm(a, b, a_scale, b_scale, nullptr, out, out_mode, M, N, K, as_stream(stream));
  return run_gemm<kInt8>(a, b, a_scale, b_scale, out, out_mode, M, N, K, 1, nullptr, 0,
                         as_stream(stream));
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
