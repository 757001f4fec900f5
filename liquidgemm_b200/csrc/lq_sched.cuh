// Work scheduling shared by the persistent kernels: segments of (tile, k-range) per CTA, either as
// equal contiguous ranges of all k-steps ("stream-K") or as a fixed split of every tile.
#pragma once

namespace lq {

struct SchedArgs {
  int kt_total;      // k-steps per tile
  int n_tiles, m_tiles;
  int fixed_split;   // 0: stream-K ranges; S >= 1: every tile is cut into S equal k-ranges
};

// One unit of a CTA's work: k-steps [kb, ke) of output tile `tile`.
struct Segment {
  int tile, kb, ke, slot;
  bool whole;   // covers the tile's full K: no cross-CTA reduction
};

// Enumerates the segments of this CTA; every role walks the same sequence.  32-bit arithmetic
// throughout (tiles * k-steps stays far below 2^31 for any problem that fits the GPU).
struct SegmentWalk {
  int kt, split, grid;
  unsigned u, u_end;   // stream-K: current / last k-step of the range
  unsigned q, r;       // stream-K: base range length and number of CTAs with one extra k-step
  unsigned w, w_end;   // fixed split: current / last work item

  __device__ SegmentWalk(const SchedArgs& a, unsigned cta, unsigned grid_) {
    kt = a.kt_total;
    split = a.fixed_split;
    grid = (int)grid_;
    const unsigned tiles = (unsigned)(a.n_tiles * a.m_tiles);
    if (split == 0) {
      const unsigned total = tiles * (unsigned)kt;
      q = total / grid_;
      r = total - q * grid_;
      u = cta * q + (cta < r ? cta : r);
      u_end = u + q + (cta < r ? 1u : 0u);
      w = w_end = 0;
    } else {
      w = cta;
      w_end = tiles * (unsigned)split;
      u = u_end = q = r = 0;
    }
  }
  __device__ int owner_of(unsigned unit) const {   // CTA whose stream-K range contains `unit`
    const unsigned big = r * (q + 1);
    return unit < big ? (int)(unit / (q + 1)) : (int)(r + (unit - big) / q);
  }
  __device__ bool has_more() const { return split == 0 ? u < u_end : w < w_end; }   // after next(): segments left
  __device__ bool next(Segment& s) {
    if (split == 0) {
      if (u >= u_end) return false;
      s.tile = (int)(u / (unsigned)kt);
      s.kb = (int)(u - (unsigned)s.tile * (unsigned)kt);
      const int left = (int)(u_end - u);
      s.ke = (kt - s.kb) < left ? kt : s.kb + left;
      s.whole = (s.kb == 0 && s.ke == kt);
      s.slot = s.whole ? 0 : owner_of((unsigned)s.tile * (unsigned)kt);
      u += (unsigned)(s.ke - s.kb);
      return true;
    }
    if (w >= w_end) return false;
    s.tile = (int)(w / (unsigned)split);
    const int si = (int)(w - (unsigned)s.tile * (unsigned)split);
    s.kb = (si * kt) / split;
    s.ke = ((si + 1) * kt) / split;
    s.whole = (split == 1);
    s.slot = s.tile;
    w += (unsigned)grid;
    return true;
  }
};

// Work split of the streaming decode kernels over `slots` resident CTAs.  With few output tiles every
// tile is cut into S equal k-ranges, one CTA each: a CTA then has exactly one segment, so no CTA pays
// the segment epilogue twice.  With many tiles the k-tiles of all tiles are laid end to end and cut
// into equal contiguous ranges (stream-K): perfectly balanced bytes, at the price of a second
// segment in most CTAs.  Between slots/2 and slots tiles the choice is the kernel's: whole tiles
// leave some SMs with one CTA (measured better for the tensor-core kernel, whose segment epilogue is
// expensive), stream-K keeps all CTAs equal (measured better for the dp4a GEMV).
struct DecodePlan {
  int grid, fixed_split;
};
inline DecodePlan decode_plan(int n_tiles, int kt, int slots, bool whole_tiles_up_to_slots) {
  if (n_tiles * 2 <= slots || (whole_tiles_up_to_slots && n_tiles <= slots)) {
    int S = slots / n_tiles;
    if (S > kt) S = kt;
    return {n_tiles * S, S};
  }
  const long units = (long)n_tiles * kt;
  return {(int)(units < slots ? units : slots), 0};
}

// Position in a ring of N stages: stage index and the parity of the pass over the ring.
template <int N>
struct Ring {
  int s = 0;
  uint32_t ph = 0;
  __device__ __forceinline__ void advance() {
    if (++s == N) {
      s = 0;
      ph ^= 1u;
    }
  }
};

}  // namespace lq
