// Pieces shared by the CTA-pair kernels (lq_gemm_pair.cu: 4-bit weights unpacked into tensor memory;
// lq_i8_pair.cu: INT8 weights read from shared memory): the walk of a pair over its tiles, the cut of the last
// wave's tiles along k and the planes through which the pairs of a cut tile add up.
#pragma once

#include <cstdint>
#include <cstdlib>

#include "lq_common.cuh"
#include "lq_sched.cuh"
#include "lq_tc_ptx.cuh"

namespace lq {
namespace pairc {

// Split factor of the tiles of the last, partial wave (r tiles on P pairs): when at least half of the pairs would
// otherwise idle, each tile is cut into equal k-ranges of 16 k-steps or more.  A cut costs the pair that
// completes the tile a read of the other pairs' sums in its last, exposed epilogue, and more pairs working in
// the last wave run at a lower clock under the power limit than the few that would otherwise finish it alone.
// Measured against whole tiles: 4096 x 14336 (112 k-steps) 16 % faster at 1024 tokens, 6 % at 2048, 4 % at 3072
// and 8192; layers of 32 k-steps 1-3 % faster where it applies.
inline int tail_split(int r, int P, int kt) {
  if (r == 0 || 2 * r > P || kt < 32) return 1;
  int S = P / r;
  if (S > kt / 16) S = kt / 16;
  return S < 1 ? 1 : S;
}

// The segments of one pair: the whole tiles of the full waves and at most one unit of the last, partial wave (a
// whole tile, or one of the S equal k-ranges of a tile).  The pair with the last k-range of a split tile completes
// it from the other pairs' sums; it takes that unit last, the others take theirs FIRST, so that their sums are in
// memory long before they are wanted and nobody's last segment waits for anybody else's.
struct PairWalk {
  int kt, P, p, full_waves, wave, S, rt, part;
  bool has_tail, tail_left, tail_first;
  template <class A>
  __device__ PairWalk(const A& a, int pair) {
    kt = a.kt_total;
    P = a.pairs;
    p = pair;
    const int tiles = a.n2_tiles * a.m_tiles;
    full_waves = tiles / P;
    wave = 0;
    const int r = tiles - full_waves * P;
    S = a.tail_s;
    has_tail = tail_left = p < r * S;
    rt = p / S;
    part = p - rt * S;
    tail_first = tail_left && part < S - 1;
  }
  __device__ int segments() const { return full_waves + (has_tail ? 1 : 0); }
  // Whether the dequant warps share the epilogue of the pair's last segment: a whole tile or the last k-range of
  // a cut one (at least 16 k-steps), long enough that a dequant warp done with it (at most seven k-steps
  // ahead of the MMA warp) cannot meet the accumulator barrier a whole use behind, where the parity it waits
  // for would read as complete.
  __device__ bool last_shared() const { return kt >= 8 && ((has_tail && !tail_first) || full_waves > 0); }
  // whether this pair holds the last k-range of a cut tile
  __device__ bool completes_tile() const { return has_tail && S > 1 && part == S - 1; }
  __device__ void tail(Segment& s) {
    tail_left = false;
    s.tile = full_waves * P + rt;
    s.kb = (part * kt) / S;
    s.ke = ((part + 1) * kt) / S;
    s.whole = (S == 1);
    s.slot = p;   // unit index: tile rt, k-range part
  }
  __device__ bool next(Segment& s) {
    if (tail_first && tail_left) {
      tail(s);
      return true;
    }
    if (wave < full_waves) {
      s.tile = wave * P + p;
      s.kb = 0;
      s.ke = kt;
      s.whole = true;
      s.slot = 0;
      ++wave;
      return true;
    }
    if (!tail_left) return false;
    tail(s);
    return true;
  }
};

// Tile index -> (channel block, token tile).  Tiles are numbered in groups of kGroupM token tiles, token tiles
// fastest inside a group, so that the 74 tiles the pairs work on at one time share 8 token tiles and about 9
// channel blocks: 17 MB of operands per wave instead of the 75 MB of a wave along one token tile (the weights
// of a wide layer do not stay in L2 beside the outputs: INT8 28672 x 4096 ran DRAM-bound at 2.57 POPS before,
// 2.98 after).
constexpr int kGroupM = 8;
// group_m = 0: channel blocks fastest (the pairs of a wave share one or two token tiles; 1-2 % better while the
// weights stay in L2).
__device__ __forceinline__ void tile_coords(int tile, int n2_tiles, int m_tiles, int group_m, int& n2, int& mt) {
  if (group_m == 0) {
    n2 = tile % n2_tiles;
    mt = tile / n2_tiles;
    return;
  }
  const int per_group = group_m * n2_tiles;
  const int group = tile / per_group, in_group = tile - group * per_group;
  const int first = group * group_m;
  const int gm = (m_tiles - first) < group_m ? (m_tiles - first) : group_m;
  mt = first + in_group % gm;
  n2 = in_group / gm;
}

// Bounded wait for the planes of a cut tile: both epilogue groups of each of the `need` other pairs have counted
// themselves in.  Relaxed polls; the caller fences before it reads the planes.
__device__ __forceinline__ bool planes_ready(const int32_t* counters2, int need, uint64_t limit_ns) {
  const uint64_t t0 = ptx::globaltimer_ns();
  for (;;) {
    int a, b;
    asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(a) : "l"(counters2) : "memory");
    asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(b) : "l"(counters2 + 1) : "memory");
    if (a >= need && b >= need) return true;
    if (ptx::globaltimer_ns() - t0 > limit_ns) return false;
    __nanosleep(100);
  }
}

// Adds the other pairs' sums of one 16-token chunk (planes of int4: [token / 4][channel]).  The planes are zeroed
// in a pass of their own afterwards (zero_planes): a load issued behind a store to the same plane waited for
// it, chunk after chunk, which made the completing epilogue 2.5 times as long as an ordinary one (trace build:
// 79 000 cycles against 30 000 without the loads and 36 000 without the stores).
__device__ __forceinline__ void add_planes(int (&v)[16], const int4* planes, size_t plane_stride, int others, int c0,
                                           int cols, int row) {
#pragma unroll 1
  for (int q = 0; q < others; ++q) {
    const int4* pl = planes + (size_t)q * plane_stride + (size_t)(c0 >> 2) * 128 + row;
    int4 t[4];
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) t[jj] = (c0 + 4 * jj < cols) ? __ldcg(pl + jj * 128) : make_int4(0, 0, 0, 0);
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {
      v[4 * jj] += t[jj].x; v[4 * jj + 1] += t[jj].y; v[4 * jj + 2] += t[jj].z; v[4 * jj + 3] += t[jj].w;
    }
  }
}
__device__ __forceinline__ void zero_planes(int4* planes, size_t plane_stride, int others, int c0, int cols, int row) {
#pragma unroll 1
  for (int q = 0; q < others; ++q) {
    int4* pl = planes + (size_t)q * plane_stride + (size_t)(c0 >> 2) * 128 + row;
#pragma unroll
    for (int jj = 0; jj < 4; ++jj)
      if (c0 + 4 * jj < cols) __stcg(pl + jj * 128, make_int4(0, 0, 0, 0));
  }
}

// The 128 threads of epilogue group g (named barriers 1 and 2).
__device__ __forceinline__ void group_barrier(int g) {
  if (g == 0) asm volatile("bar.sync 1, 128;" ::: "memory");
  else asm volatile("bar.sync 2, 128;" ::: "memory");
}


}  // namespace pairc
}  // namespace lq
