// Pieces shared by the paged decode kernels: the walk over (row, block) segments, the cut of the
// global block sequence into one range per CTA, and the fold of the partial results of a row that
// several CTAs worked on.
#pragma once

#include "paged_decode.cuh"

namespace nvj {

constexpr int kDecodeThreads = 256;
constexpr int kMinBlocksPerCta = 6;
constexpr int kRing = 1024;  // block-id look-ahead window (two halves of 512 iterations)
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kNegBig = -1.0e30f;

// What a CTA pays for every row that ends in its range, in units of the time one block takes to stream: the hand-over
// of the row (exchange between the warps, output or partial, fence and counter, perhaps the fold) and the start of the
// next one.  The sequence that is cut into equal ranges therefore holds, behind the blocks of every non-empty row,
// kRowEndCost phantom blocks that nobody reads: a range with more row ends gets fewer real blocks.  (With ranges of
// equal real blocks the CTAs of a 256-row batch finished 21 us apart, and the time a CTA finished followed the number
// of rows in its range with a correlation of 0.85: 205.8 / 210.9 / 214.6 / 220.9 us for 2 / 3 / 4 / 5 rows.)
constexpr int kRowEndCost = 6;  // the mma.sync and the CUDA-core kernel; the tcgen05 wide kernel has its own figure
__device__ __forceinline__ int blocks_in_sequence(const DecodeParams& p, int nb) { return nb > 0 ? nb + p.row_end_cost : 0; }

struct Seg {
  int b, j0, j1, nb, len;  // real blocks [j0, j1) of row b, which has nb blocks
  long long g0;            // index of block j0 in the sequence (phantom blocks counted)
};

// Next row segment with real blocks in this CTA's range [g, g1) of the sequence.
__device__ __forceinline__ bool next_seg(const DecodeParams& p, int& b, int& j, long long& g,
                                         long long g1, Seg& s) {
  while (g < g1 && b < p.batch) {
    const int len = decode_row_len(p, b);
    const int nb = (len + kBlk - 1) / kBlk;
    const int nbv = blocks_in_sequence(p, nb);
    if (j >= nbv) { ++b; j = 0; continue; }
    const long long room = g1 - g;
    const int take = (long long)(nbv - j) < room ? (nbv - j) : (int)room;
    const int j0 = j, j1 = j + take < nb ? j + take : nb, row = b;
    const long long at = g;
    g += take; ++b; j = 0;  // either the row is finished or the range is
    if (j1 <= j0) continue;  // only phantom blocks of the row lie here
    s.b = row; s.j0 = j0; s.j1 = j1; s.nb = nb; s.len = len; s.g0 = at;
    return true;
  }
  return false;
}

// Real blocks in the range [g, g1) that starts at position j of row b.
__device__ __forceinline__ int blocks_in_range(const DecodeParams& p, int b, int j, long long g, long long g1) {
  Seg s;
  int n = 0;
  while (next_seg(p, b, j, g, g1, s)) n += s.j1 - s.j0;
  return n;
}

// Inclusive scan of one int per thread over the whole CTA (kDecodeThreads).
__device__ __forceinline__ int cta_inclusive_scan(int v, int* warp_sums, int& total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int n = __shfl_up_sync(kFullMask, v, o);
    if (lane >= o) v += n;
  }
  __syncthreads();
  if (lane == 31) warp_sums[warp] = v;
  __syncthreads();
  int before = 0, all = 0;
#pragma unroll
  for (int w = 0; w < kDecodeThreads / 32; ++w) {
    const int x = warp_sums[w];
    if (w < warp) before += x;
    all += x;
  }
  total = all;
  return v + before;
}

// Look-ahead walker that fills the block-id ring.
struct FillState {
  Seg s;
  int b, jn;      // walker position after s
  long long g;
  int j;          // next block of s to emit
  int nsegs;
  bool has;
};

// Emits ring entries for the CTA's iterations [n0, n0 + count): block id and the
// number of attended tokens in the block (0 for a block id outside the pool).
// All kDecodeThreads threads call this with identical arguments; the caller
// separates it from the readers of the ring with CTA barriers.
// (A thread waits for memory once per row segment here, and CTAs whose range holds three rows instead of two issue
// their first K/V copies later than the others.  Asynchronous 4-byte copies of the ids with a second walk that checks
// them were measured: the late CTAs gained 1.8 us, the others lost 0.8, the kernel's time did not change; an L1
// prefetch of the next segment's ids ahead of every segment cost 3 us at kernel level.)
template <class Smem>
__device__ __forceinline__ void fill_ring(const DecodeParams& p, Smem& sm, FillState& f,
                                          long long g1, int n0, int count) {
  while (count > 0) {
    if (!f.has || f.j >= f.s.j1) {
      if (!next_seg(p, f.b, f.jn, f.g, g1, f.s)) break;
      f.j = f.s.j0;
      f.has = true;
      ++f.nsegs;
    }
    const int take = count < f.s.j1 - f.j ? count : f.s.j1 - f.j;
    const long long tbase = decode_table_base(p, f.s.b);
    for (int i = threadIdx.x; i < take; i += kDecodeThreads) {
      const int jj = f.j + i;
      const int blk = p.block_tables[tbase + jj];
      int rows = (jj == f.s.nb - 1) ? f.s.len - kBlk * (f.s.nb - 1) : kBlk;
      if (blk < 0 || blk >= p.num_blocks) {
        atomicOr(p.status, NVJ_DEV_BAD_BLOCK_ID);
        rows = 0;
      }
      sm.ring_blk[(n0 + i) & (kRing - 1)] = blk;
      sm.ring_rows[(n0 + i) & (kRing - 1)] = (signed char)rows;
    }
    n0 += take;
    f.j += take;
    count -= take;
  }
}

// How the sequence [0, total) of real and phantom blocks is cut into one contiguous range per CTA: CTA c
// of n gets [c * total / n, (c + 1) * total / n).  With fewer blocks than CTAs only `total`
// CTAs take part (one block each), so every CTA id inside a row's span delivers a partial.
// (Giving the CTA that arrives first on an SM a larger share was measured and does not
// help: the two CTAs of an SM share its bandwidth, so the SM finishes at the same time.)
struct Partition {
  long long total;
  int n;

  __device__ __forceinline__ long long start(int c) const { return (long long)c * total / n; }
  // The CTA whose range holds global block g (the last CTA whose start is <= g).
  __device__ __forceinline__ int cta_of(long long g) const { return (int)(((g + 1) * n - 1) / total); }
};

__device__ __forceinline__ Partition make_partition(long long total, int grid) {
  Partition pt;
  pt.total = total;
  // at least kMinBlocksPerCta blocks per CTA: with fewer, a short batch is cut into so many partials that the
  // CTA that merges a row becomes the long pole (8 rows of ~65 blocks: 51 us with one block per CTA, 31 us so)
  const long long cap = (total + kMinBlocksPerCta - 1) / kMinBlocksPerCta;
  pt.n = cap < grid ? (int)cap : grid;
  return pt;
}

// Where a CTA parks its partial result for a row it shares with other CTAs: a
// CTA holds at most one segment that continues a row begun elsewhere (slot 2c)
// and at most one that begins a row finished elsewhere (slot 2c + 1).
__device__ __forceinline__ int partial_slot(int cta, bool begins_row) { return 2 * cta + (begins_row ? 1 : 0); }

// Folds n <= 32 partial results into one.  Part i sits in slot base + 2 * (first + i), plus one if
// first + i == row_first (the slot pairing of partial_slot).  kFinal: the normalised result goes to
// output row dst; otherwise the un-normalised sum and its (max, sum) go to partial slot dst.
// Two phases, so that no load depends on another: (a) thread (part, head) reads the part's (max, sum),
// the CTA reduces them to the head's max and sum and leaves one weight per (part, head) in shared
// memory; (b) thread (head, 8 dims) sums weight * accumulator over the parts, eight parts (sixteen
// 16-byte loads from L2, never L1) in flight at a time.  A fold of 16 parts costs about three memory
// round trips.  A slot holds slot_rows rows of (kD accumulators, (max, sum)); the fold covers the kHq rows
// from row_off on, so a kernel with several query tokens per row folds each token's heads in turn.
// dst: kFinal, first of the kHq output rows; otherwise the destination slot.  All 256 threads call it;
// `red` is shared-memory scratch of 384 floats.  kBatch parts' accumulators are in flight at a time (4 * kBatch
// registers): 8 in the kernel that runs two CTAs per SM, 16 where a thread has 255 registers.
template <bool kFinal, int kBatch = 8>
__device__ __forceinline__ void fold_parts(const DecodeParams& p, float* red, int tid, long long base, int first,
                                           int row_first, int n, long long dst, int slot_rows = kHq, int row_off = 0) {
  float* m_sh = red + 64;         // [8 heads]
  float* w_sh = red + 128;        // [32 parts][8 heads]
  const int warp = tid >> 5, lane = tid & 31;
  // the first batch of accumulators is requested before the (max, sum) round trip, not after it
  float4 x[kBatch][2];
#pragma unroll
  for (int k = 0; k < kBatch; ++k) {
    const bool ok = k < n;
    const int c = first + (ok ? k : 0);
    const long long sl = base + 2 * c + (c == row_first ? 1 : 0);
    const float4* src = reinterpret_cast<const float4*>(p.part_acc + (sl * slot_rows + row_off + warp) * kD + lane * 8);
    x[k][0] = ok ? __ldcg(src) : make_float4(0.f, 0.f, 0.f, 0.f);
    x[k][1] = ok ? __ldcg(src + 1) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  {
    const int i = tid >> 3, h = tid & 7;
    const bool ok = i < n;
    const int c = first + (ok ? i : 0);
    const long long sl = base + 2 * c + (c == row_first ? 1 : 0);
    const float2 e = ok ? __ldcg(reinterpret_cast<const float2*>(p.part_ml + (sl * slot_rows + row_off + h) * 2)) : make_float2(kNegBig, 0.f);
    float m = e.x;
    m = fmaxf(m, __shfl_xor_sync(kFullMask, m, 8));
    m = fmaxf(m, __shfl_xor_sync(kFullMask, m, 16));
    if (lane < 8) red[warp * 8 + lane] = m;
    named_bar_sync(1, kDecodeThreads);
    float M = red[h];
#pragma unroll
    for (int w = 1; w < kDecodeThreads / 32; ++w) M = fmaxf(M, red[w * 8 + h]);
    const float wgt = ok ? ex2_approx(e.x - M) : 0.f;
    w_sh[i * 8 + h] = wgt;
    if (i == 0) m_sh[h] = M;
    float l = e.y * wgt;
    l += __shfl_xor_sync(kFullMask, l, 8);
    l += __shfl_xor_sync(kFullMask, l, 16);
    named_bar_sync(1, kDecodeThreads);  // every thread has read the maxima
    if (lane < 8) red[warp * 8 + lane] = l;
    named_bar_sync(1, kDecodeThreads);
  }
  const int h = warp, d0 = lane * 8;
  float L = 0.f;
#pragma unroll
  for (int w = 0; w < kDecodeThreads / 32; ++w) L += red[w * 8 + h];
  float acc[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) acc[k] = 0.f;
#pragma unroll 1
  for (int i0 = 0; i0 < n; i0 += kBatch) {
#pragma unroll
    for (int k = 0; k < kBatch; ++k) {
      if (i0 == 0) break;  // loaded above
      const bool ok = i0 + k < n;
      const int c = first + (ok ? i0 + k : 0);
      const long long sl = base + 2 * c + (c == row_first ? 1 : 0);
      const float4* src = reinterpret_cast<const float4*>(p.part_acc + (sl * slot_rows + row_off + h) * kD + d0);
      x[k][0] = ok ? __ldcg(src) : make_float4(0.f, 0.f, 0.f, 0.f);
      x[k][1] = ok ? __ldcg(src + 1) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int k = 0; k < kBatch; ++k) {
      const float wgt = i0 + k < n ? w_sh[(i0 + k) * 8 + h] : 0.f;
      acc[0] = fmaf(x[k][0].x, wgt, acc[0]); acc[1] = fmaf(x[k][0].y, wgt, acc[1]);
      acc[2] = fmaf(x[k][0].z, wgt, acc[2]); acc[3] = fmaf(x[k][0].w, wgt, acc[3]);
      acc[4] = fmaf(x[k][1].x, wgt, acc[4]); acc[5] = fmaf(x[k][1].y, wgt, acc[5]);
      acc[6] = fmaf(x[k][1].z, wgt, acc[6]); acc[7] = fmaf(x[k][1].w, wgt, acc[7]);
    }
  }
  const long long row = kFinal ? dst + h : dst * slot_rows + row_off + h;
  if (kFinal) {
    const float inv = L > 0.f ? 1.f / L : 0.f;
    float4* o = reinterpret_cast<float4*>(p.out + row * kD + d0);
    o[0] = make_float4(acc[0] * inv, acc[1] * inv, acc[2] * inv, acc[3] * inv);
    o[1] = make_float4(acc[4] * inv, acc[5] * inv, acc[6] * inv, acc[7] * inv);
  } else {
    float4* o = reinterpret_cast<float4*>(p.part_acc + row * kD + d0);
    o[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
    o[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
    if (lane == 0) *reinterpret_cast<float2*>(p.part_ml + row * 2) = make_float2(m_sh[h], L);
  }
}

}  // namespace nvj
