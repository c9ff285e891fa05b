// Paged GQA decode attention for rows of several query tokens (speculative verification, widths up to 16) on the
// 5th-generation tensor cores: tcgen05.mma with the scores and the output accumulators in tensor memory.
//
// Why a second wide kernel.  decode_wide_kernel (mma.sync) holds one 16-row tile of query rows per warp; rows of
// 5..8 tokens are two tiles per KV head, every warp then walks every block, and the kernel takes 1.9x its width-1
// time: 512 mma.sync per block and SM are more than the legacy tensor path issues in the HBM time of a block.  Here
// the 4 x width <= 64 query rows of one KV head sit in lanes 0..63 of a 128-row UMMA tile (the other lanes compute
// on whatever they hold and are never read; up to 8 tokens per row only lanes 0..31 are used): per tile of 64 keys
// and KV head 16 MMAs of N = 64 for the scores and eight of N = 256 for the weighted sum, ~1500 tensor cycles against ~3000 cycles of HBM time.  (Scores block by
// block, 64 MMAs of N = 16 per tile, were measured first: 345 us on C2 shapes, the small MMAs cost more to issue
// than they compute.)
//
// Work split.  The blocks of all rows form one sequence cut into equal ranges as in the other decode kernels
// (decode_parts.cuh), but a range belongs to a PAIR of CTAs, one per KV head: CTA 2c + h streams head h's half of
// every block of range c, so every K/V byte still crosses HBM once.  Keys are walked in tiles of up to four blocks
// that never straddle a row; a tile's K lands as [64-d chunk][64 keys][128 B] (one 2 KiB TMA box per block and
// chunk, so that the whole tile is one N = 64 operand), its V block by block as [chunk][16 keys][128 B] (one 8 KiB
// box per block: P V contracts 16 keys per MMA anyway).  One CTA per SM (192 KiB of shared memory: three tiles in
// flight; 512 TMEM columns).
//   warp 0   (and warp 1 for rows of more than 8 tokens: a warp may only touch the 32 TMEM lanes of its quarter)
//            softmax and epilogue: lane r = query row r = token * 4 + head of the group.  Per row segment it stages
//            the query rows into tensor memory, per tile of up to four blocks (64 keys) reads the scores
//            (tcgen05.ld), masks (key < length, key <= the token's position), keeps the running maximum lazily (O in
//            tensor memory is rescaled only when a tile exceeds it by 2^8) and writes the weights back over the
//            scores as two bf16 terms (hi + lo); at the end of the segment it reads O and stores the row (whole row
//            in this range) or the un-normalised partial with its (max, sum).
//   warp 3   producer: block ids straight from the block table (32 at a time), TMA boxes into the ring.
//   warp 2   MMA issue: S(t) = Q K(t)^T into one of two score buffers, O += P(t) V(t) once the weights are
//            written; S(t + 2) follows P V (t).  tcgen05.commit releases ring stages and signals the softmax warp.
// A row cut over several ranges is folded afterwards by decode_umma_merge_kernel (one CTA per row, stream order
// instead of counters and fences): the merge costs a second small launch, which rows of this width can afford.
// Every wait is bounded; on a timeout the kernel flags NVJ_DEV_TIMEOUT, stops issuing, lets copies in flight land
// and still frees its tensor memory.  A block id outside the pool is flagged and its box is fetched from beyond the
// tensor (zeros), so nothing foreign is read; the row's result is then meaningless but finite.
// Semantics: nanovllm_jax/kv_cache.py:852-998 with query width > 1 (key p of row b is visible to token t when
// p < seq_lens[b] and, with positions given, p <= positions[b, t]).

#include <cuda.h>

#include "decode_parts.cuh"
#include "umma.cuh"

namespace nvj {

constexpr int kUdStages = 3;      // tiles (K and V of one KV head for up to 64 keys: 64 KiB) in flight
constexpr int kUdTileBlocks = 4;  // blocks per tile: 64 keys
constexpr int kUdTmemCols = 512;
constexpr int kUdColQ = 0;        // query rows as the A operand: 256 bf16 per row = 128 columns
constexpr int kUdColS = 128;      // two score buffers of 64 columns; the weights (hi: 32 columns, lo: 32) overwrite theirs
constexpr int kUdColO = 256;      // output accumulator: columns [256, 512)
constexpr int kUdHalfBlock = kBlk * kD * 2;  // K (or V) of one KV head of one block: 8 KiB
constexpr float kUdRescaleGap = 8.f;
constexpr int kUdMaxWidth = 16;  // 64 query rows per KV head: two softmax warps
constexpr int kUdRowEndCost = 6;  // what a row end costs a CTA here, in blocks (6 and 12 measured alike, 18 and 24 worse)

struct UdSmem {
  alignas(1024) char k[kUdStages][4][kUdTileBlocks * kBlk * 128];  // [stage][64-d chunk][64 keys][128 B], swizzled
  alignas(1024) char v[kUdStages][kUdTileBlocks][kUdHalfBlock];    // [stage][block][64-d chunk][16 keys][128 B], swizzled
  alignas(8) unsigned long long full_bar[kUdStages], empty_bar[kUdStages], q_full, s_full[2], p_full, pv_done, o_free;
  float red[384];
  int scan[16];
  int start_b, start_j, abort_flag;
  uint32_t tmem_base;
};

// One box of the 4-D view {64 dims, token, 64-dim chunk, kv head} of a cache layer: with the V map all four chunks of
// one KV head's half of a block (8 KiB), with the K map one chunk of it (2 KiB).
__device__ __forceinline__ void ud_tma_box(uint32_t dst, const CUtensorMap* map, int token, int chunk, int kvh, uint32_t bar,
                                           uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3, %4, %5}], [%6], %7;"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(0), "r"(token), "r"(chunk), "r"(kvh), "r"(bar), "l"(policy)
      : "memory");
}

// ---- warp 3: TMA loads --------------------------------------------------------------------------
__device__ __forceinline__ void ud_producer(const CUtensorMap* k_map, const CUtensorMap* v_map, const DecodeParams& p,
                                            UdSmem& sm, int kvh, int b, int j, long long g, long long g1, int lane) {
  const int oob = (int)(p.num_blocks * kBlk);  // a box that starts here is filled with zeros
  uint64_t policy;  // every block is read once: do not let it displace what the L2 is good for
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
  Seg s;
  uint32_t gt = 0;  // tiles so far, over all segments
  while (next_seg(p, b, j, g, g1, s)) {
    const long long tbase = decode_table_base(p, s.b);
    for (int jb = s.j0; jb < s.j1; jb += 32) {  // 32 block ids = 8 tiles at a time
      const int n = s.j1 - jb < 32 ? s.j1 - jb : 32;
      int id = -1;
      if (lane < n) {
        id = p.block_tables[tbase + jb + lane];
        if (id < 0 || id >= p.num_blocks) {
          atomicOr(p.status, NVJ_DEV_BAD_BLOCK_ID);
          id = -1;
        }
      }
      for (int i0 = 0; i0 < n; i0 += kUdTileBlocks, ++gt) {
        const int cnt = n - i0 < kUdTileBlocks ? n - i0 : kUdTileBlocks;
        const int stage = (int)(gt % kUdStages);
        if (gt >= kUdStages && !um_wait(&sm.empty_bar[stage], ((gt / kUdStages) - 1) & 1u, &sm.abort_flag, p.status)) return;
        const uint32_t fb = smem_u32(&sm.full_bar[stage]);
        if (lane == 0) mbar_arrive_expect_tx(fb, (uint32_t)cnt * 2u * kUdHalfBlock);
        __syncwarp();
        for (int i = 0; i < cnt; ++i) {
          const int blk = __shfl_sync(kFullMask, id, i0 + i);
          const int token = blk >= 0 ? blk * kBlk : oob;
          if (lane < 4) ud_tma_box(smem_u32(&sm.k[stage][lane][0]) + i * (kBlk * 128), k_map, token, lane, kvh, fb, policy);
          else if (lane == 4) ud_tma_box(smem_u32(&sm.v[stage][i][0]), v_map, token, 0, kvh, fb, policy);
        }
        __syncwarp();
      }
    }
  }
}

// ---- warp 2: MMA issue --------------------------------------------------------------------------
// Scores of tile `gt` (stage gt % kUdStages) into score buffer gt & 1: columns of blocks the tile does not have are
// computed from whatever the stage holds there and masked by the softmax warp.
__device__ __forceinline__ bool ud_issue_s(UdSmem& sm, const DecodeParams& p, uint32_t tmem, uint64_t k_desc0, uint32_t gt) {
  const int stage = (int)(gt % kUdStages);
  if (!um_wait(&sm.full_bar[stage], (gt / kUdStages) & 1u, &sm.abort_flag, p.status)) return false;
  tc_fence_after_sync();
  if (um_elect_one()) {
    constexpr uint32_t idesc = umma_idesc(kUdTileBlocks * kBlk, false);
    const uint64_t k_desc = k_desc0 + (uint64_t)((stage * 4 * kUdTileBlocks * kBlk * 128) >> 4);
    const uint32_t d = tmem + kUdColS + (gt & 1u) * 64;
#pragma unroll
    for (int ks = 0; ks < 16; ++ks)  // 16 dims per MMA: 8 columns of Q; K chunk ks / 4, 32 bytes into its swizzled rows
      umma_bf16_ts(d, tmem + kUdColQ + ks * 8, k_desc + (uint64_t)(((ks >> 2) * (kUdTileBlocks * kBlk * 128) + (ks & 3) * 32) >> 4),
                   idesc, ks > 0 ? 1u : 0u);
    umma_commit(smem_u32(&sm.s_full[gt & 1u]));
  }
  __syncwarp();
  return true;
}

__device__ __forceinline__ void ud_mma_warp(UdSmem& sm, const DecodeParams& p, uint32_t tmem, int b, int j, long long g,
                                            long long g1) {
  const uint64_t k_desc0 = umma_desc(smem_u32(&sm.k[0][0][0]), 16, 1024);          // K: keys are rows, dims contracted
  const uint64_t v_desc0 = umma_desc(smem_u32(&sm.v[0][0][0]), kBlk * 128, 1024);  // V: 64-d chunks 2 KiB apart, keys contracted
  Seg s;
  uint32_t gt = 0;  // tiles so far, over all segments: picks the stage, the score buffer and the barrier phases
  uint32_t seg = 0;
  while (next_seg(p, b, j, g, g1, s)) {
    const int nblk = s.j1 - s.j0, nt = (nblk + kUdTileBlocks - 1) / kUdTileBlocks;
    if (!um_wait(&sm.q_full, seg & 1u, &sm.abort_flag, p.status)) return;
    for (int t = 0; t < 2 && t < nt; ++t)
      if (!ud_issue_s(sm, p, tmem, k_desc0, gt + t)) return;
    for (int t = 0; t < nt; ++t, ++gt) {
      const int cnt = nblk - t * kUdTileBlocks < kUdTileBlocks ? nblk - t * kUdTileBlocks : kUdTileBlocks;
      const int stage = (int)(gt % kUdStages);
      if (!um_wait(&sm.p_full, gt & 1u, &sm.abort_flag, p.status)) return;
      // the first P V of a segment overwrites O: the segment before must have been read out
      if (t == 0 && seg > 0 && !um_wait(&sm.o_free, (seg - 1) & 1u, &sm.abort_flag, p.status)) return;
      tc_fence_after_sync();
      if (um_elect_one()) {
        constexpr uint32_t idesc = umma_idesc(kD, true);
        const uint32_t pa = tmem + kUdColS + (gt & 1u) * 64;
        for (int i = 0; i < cnt; ++i) {  // 16 keys per MMA: 8 columns of P, the block's two 8-key groups of V
          const uint64_t dv = v_desc0 + (uint64_t)(((stage * kUdTileBlocks + i) * kUdHalfBlock) >> 4);
          umma_bf16_ts(tmem + kUdColO, pa + i * 8, dv, idesc, (t > 0 || i > 0) ? 1u : 0u);
          umma_bf16_ts(tmem + kUdColO, pa + 32 + i * 8, dv, idesc, 1u);
        }
        umma_commit(smem_u32(&sm.empty_bar[stage]));
        umma_commit(smem_u32(&sm.pv_done));
      }
      __syncwarp();
      // S(t + 2) overwrites the columns P V (t) reads P(t) from, and every phase of pv_done is observed in turn
      if (!um_wait(&sm.pv_done, gt & 1u, &sm.abort_flag, p.status)) return;
      if (t + 2 < nt && !ud_issue_s(sm, p, tmem, k_desc0, gt + 2)) return;
    }
    ++seg;
  }
}

// Query rows of one table row into tensor memory: lane = row (token * 4 + head), 256 dims -> 128 columns, two bf16 per
// column; sixteen 16-byte loads in flight at a time (one at a time, the eight round trips to memory cost a segment
// more than its epilogue).  `tmem` addresses this warp's lanes; `row` = 32 * warp + lane.  Arrives on q_full.
__device__ __forceinline__ void ud_stage_q(UdSmem& sm, const DecodeParams& p, uint32_t tmem, int kvh, int row_b, int row) {
  const int tok = row >> 2, head = row & 3;
  const bool real = tok < p.width;
  const uint4* src = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(p.q) +
                                                    (((long long)row_b * p.width + (real ? tok : 0)) * kHq + kvh * kG + head) * kD);
#pragma unroll 1
  for (int half = 0; half < 2; ++half) {
    uint4 u[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) u[i] = real ? ld_nc_u4(src + half * 16 + i) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
    for (int part = 0; part < 4; ++part) {  // 32 dims = 16 columns at a time
      uint32_t w[16];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        w[4 * i] = u[part * 4 + i].x; w[4 * i + 1] = u[part * 4 + i].y; w[4 * i + 2] = u[part * 4 + i].z; w[4 * i + 3] = u[part * 4 + i].w;
      }
      tmem_st16(tmem + kUdColQ + half * 64 + part * 16, w);
    }
  }
  tmem_st_wait();
  tc_fence_before_sync();
  mbar_arrive(smem_u32(&sm.q_full));
}

// ---- warps 0 and 1: query staging, softmax, epilogue ----------------------------------------------------
__device__ __forceinline__ void ud_softmax_warp(UdSmem& sm, const DecodeParams& p, uint32_t tmem, int kvh, int b, int j,
                                                long long g, long long g1, int range, int row) {
  const int tok = row >> 2, head = row & 3;
  const bool real = tok < p.width;
  const float scale_log2 = p.scale * kLog2e;
  const int slot_rows = p.width * kHq;
  Seg s, nxt;
  uint32_t gt = 0;
  bool have = next_seg(p, b, j, g, g1, s);
  if (have) ud_stage_q(sm, p, tmem, kvh, s.b, row);
  while (have) {
    const long long qbase = (long long)s.b * p.width;
    bool have_next = false;
    const int my_pos = real ? (p.positions ? p.positions[qbase + tok] : 0x7fffffff) : -1;
    const int last_key = my_pos < s.len - 1 ? my_pos : s.len - 1;  // last key this row may see
    float m_row = -INFINITY, l_row = 0.f;                           // m_row in units of log2(e) * scale
    const int nblk = s.j1 - s.j0, nt = (nblk + kUdTileBlocks - 1) / kUdTileBlocks;
    for (int t = 0; t < nt; ++t, ++gt) {
      const uint32_t s_tmem = tmem + kUdColS + (gt & 1u) * 64;
      if (!um_wait(&sm.s_full[gt & 1u], (gt >> 1) & 1u, &sm.abort_flag, p.status)) return;
      tc_fence_after_sync();
      float sc[64];
      {
        float a[32];
        tmem_ld32(s_tmem, a);
#pragma unroll
        for (int i = 0; i < 32; ++i) sc[i] = a[i];
        tmem_ld32(s_tmem + 32, a);
#pragma unroll
        for (int i = 0; i < 32; ++i) sc[32 + i] = a[i];
      }
      const int cnt = nblk - t * kUdTileBlocks < kUdTileBlocks ? nblk - t * kUdTileBlocks : kUdTileBlocks;
      int lim = last_key - (s.j0 + t * kUdTileBlocks) * kBlk;  // columns [0, lim] are visible
      lim = lim < cnt * kBlk - 1 ? lim : cnt * kBlk - 1;       // columns of blocks the tile does not have hold old scores
      float tmax = -INFINITY;
#pragma unroll
      for (int i = 0; i < 64; ++i) {
        sc[i] = i <= lim ? sc[i] : -INFINITY;
        tmax = fmaxf(tmax, sc[i]);
      }
      tmax *= scale_log2;  // scale > 0
      if (t == 0) {
        m_row = tmax;
      } else if (__any_sync(kFullMask, tmax > m_row + kUdRescaleGap)) {
        // rare: raise the maxima and rescale O, once the last P V has landed
        if (!um_wait(&sm.pv_done, (gt - 1) & 1u, &sm.abort_flag, p.status)) return;
        tc_fence_after_sync();
        const float m_new = fmaxf(m_row, tmax);
        const float f = m_new == -INFINITY ? 1.f : ex2_approx(m_row - m_new);
        m_row = m_new;
        l_row *= f;
#pragma unroll 1
        for (int cc = 0; cc < kD / 32; ++cc) {
          float o[32];
          tmem_ld32(tmem + kUdColO + cc * 32, o);
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] *= f;
          tmem_st32(tmem + kUdColO + cc * 32, o);
        }
      }
      const float neg_m = m_row == -INFINITY ? 0.f : -m_row;
      uint32_t hi[32], lo[32];
#pragma unroll
      for (int e = 0; e < 32; ++e) {
        const float p0 = ex2_approx(fmaf(sc[2 * e], scale_log2, neg_m)), p1 = ex2_approx(fmaf(sc[2 * e + 1], scale_log2, neg_m));
        l_row += p0 + p1;
        const __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
        const __nv_bfloat162 r2 = __floats2bfloat162_rn(p0 - __low2float(h), p1 - __high2float(h));
        hi[e] = *reinterpret_cast<const uint32_t*>(&h);
        lo[e] = *reinterpret_cast<const uint32_t*>(&r2);
      }
      // every phase of pv_done is observed in turn (a parity wait tells only two consecutive phases apart)
      if (gt >= 1 && !um_wait(&sm.pv_done, (gt - 1) & 1u, &sm.abort_flag, p.status)) return;
      {  // P(t) as the A operand of P V: keys 2j, 2j + 1 in column j; hi in columns [0, 32), lo in [32, 64)
        uint32_t w[16];
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
#pragma unroll
          for (int i = 0; i < 16; ++i) w[i] = q4 < 2 ? hi[(q4 & 1) * 16 + i] : lo[(q4 & 1) * 16 + i];
          tmem_st16(s_tmem + q4 * 16, w);
        }
      }
      tmem_st_wait();
      tc_fence_before_sync();
      mbar_arrive(smem_u32(&sm.p_full));
      if (t == nt - 1) {
        // The segment's last scores have been read, so all of its S products have retired and the query columns are
        // free: the next row's queries go in now, and its first scores are computed while this segment's output is
        // still being read out below (the MMA warp holds the next P V back until o_free).
        have_next = next_seg(p, b, j, g, g1, nxt);
        if (have_next) ud_stage_q(sm, p, tmem, kvh, nxt.b, row);
      }
    }
    // ---- end of the segment: O -> the output row (the whole row lies in this range) or this range's partial
    if (!um_wait(&sm.pv_done, (gt - 1) & 1u, &sm.abort_flag, p.status)) return;
    tc_fence_after_sync();
    const bool whole_row = (s.j0 == 0 && s.j1 == s.nb);
    const float inv = whole_row ? (l_row > 0.f ? 1.f / l_row : 0.f) : 1.f;
    const int slot = partial_slot(range, s.j0 == 0);
    const int row_in_slot = tok * kHq + kvh * kG + head;
    float* dst = whole_row ? p.out + ((qbase + tok) * kHq + kvh * kG + head) * kD
                           : p.part_acc + ((long long)slot * slot_rows + row_in_slot) * kD;
#pragma unroll 1
    for (int cc = 0; cc < kD / 32; ++cc) {
      float o[32];
      tmem_ld32(tmem + kUdColO + cc * 32, o);
      if (real) {
#pragma unroll
        for (int i = 0; i < 32; i += 4)
          *reinterpret_cast<float4*>(dst + cc * 32 + i) = make_float4(o[i] * inv, o[i + 1] * inv, o[i + 2] * inv, o[i + 3] * inv);
      }
    }
    if (real && !whole_row)
      *reinterpret_cast<float2*>(p.part_ml + ((long long)slot * slot_rows + row_in_slot) * 2) =
          make_float2(m_row == -INFINITY ? kNegBig : m_row, l_row);
    tc_fence_before_sync();  // the next segment's first P V overwrites what was just read
    if (have_next) mbar_arrive(smem_u32(&sm.o_free));
    s = nxt;
    have = have_next;
  }
}

__global__ void __launch_bounds__(kDecodeThreads, 1)
decode_umma_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map, DecodeParams p) {
  extern __shared__ unsigned char ud_smem_raw[];
  UdSmem& sm = *reinterpret_cast<UdSmem*>((reinterpret_cast<uintptr_t>(ud_smem_raw) + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kvh = blockIdx.x & 1, range = blockIdx.x >> 1, ranges = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&k_map)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&v_map)) : "memory");
    sm.start_b = p.batch; sm.start_j = 0; sm.abort_flag = 0;
  }
  // ---- pass 1: total number of blocks; zero the output of inactive rows
  int mine = 0;
  for (int base = 0; base < p.batch; base += kDecodeThreads) {
    const int b = base + threadIdx.x;
    int len = 0;
    if (b < p.batch) len = decode_row_len(p, b);
    mine += blocks_in_sequence(p, (len + kBlk - 1) / kBlk);
    const unsigned idle = __ballot_sync(kFullMask, b < p.batch && len <= 0 && (b % (int)gridDim.x) == (int)blockIdx.x);
    for (unsigned m = idle; m; m &= m - 1) {
      const int bb = base + (warp << 5) + (__ffs(m) - 1);
      float4* o = reinterpret_cast<float4*>(p.out + (long long)bb * p.width * kHq * kD);
      for (int i = lane; i < p.width * kHq * kD / 4; i += 32) o[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
  int total = 0;
  cta_inclusive_scan(mine, sm.scan, total);
  if (total == 0) return;
  const Partition pt = make_partition(total, ranges);
  if (range >= pt.n) return;
  const long long g0 = pt.start(range);
  const long long g1 = pt.start(range + 1);
  if (g0 == g1) return;

  // ---- pass 2: locate (row, block) of g0
  long long carry = 0;
  for (int base = 0; base < p.batch && carry <= g0; base += kDecodeThreads) {
    const int b = base + threadIdx.x;
    int n = 0;
    if (b < p.batch) n = blocks_in_sequence(p, (decode_row_len(p, b) + kBlk - 1) / kBlk);
    int chunk_total = 0;
    const long long excl = carry + cta_inclusive_scan(n, sm.scan, chunk_total) - n;
    if (n > 0 && excl <= g0 && g0 < excl + n) { sm.start_b = b; sm.start_j = (int)(g0 - excl); }
    carry += chunk_total;
  }
  if (warp == 2) tmem_alloc(smem_u32(&sm.tmem_base), kUdTmemCols);
  if (threadIdx.x == 0) {
    for (int i = 0; i < kUdStages; ++i) {
      mbar_init(smem_u32(&sm.full_bar[i]), 1);
      mbar_init(smem_u32(&sm.empty_bar[i]), 1);
    }
    const uint32_t softmax_threads = p.width > 8 ? 64u : 32u;
    mbar_init(smem_u32(&sm.q_full), softmax_threads);
    mbar_init(smem_u32(&sm.s_full[0]), 1);
    mbar_init(smem_u32(&sm.s_full[1]), 1);
    mbar_init(smem_u32(&sm.p_full), softmax_threads);
    mbar_init(smem_u32(&sm.pv_done), 1);
    mbar_init(smem_u32(&sm.o_free), softmax_threads);
    mbar_fence_init();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = sm.tmem_base;
  const int b0 = sm.start_b, j0 = sm.start_j;

  if (warp == 0 || (warp == 1 && p.width > 8))  // this warp's quarter of the TMEM lanes: rows 32 * warp ..
    ud_softmax_warp(sm, p, tmem + ((uint32_t)(warp * 32) << 16), kvh, b0, j0, g0, g1, range, warp * 32 + lane);
  else if (warp == 2) ud_mma_warp(sm, p, tmem, b0, j0, g0, g1);
  else if (warp == 3) ud_producer(&k_map, &v_map, p, sm, kvh, b0, j0, g0, g1, lane);

  tc_fence_before_sync();
  __syncthreads();
  if (sm.abort_flag) {  // give copies and MMAs in flight time to land before the CTA's memory is released
    const unsigned long long t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 2) tmem_dealloc(tmem, kUdTmemCols);
}

// One CTA per (row, query token): a row whose blocks were cut over several ranges is folded from the ranges' partials.
// Runs behind decode_umma_kernel in stream order, so it needs neither counters nor fences.  (One CTA per row that
// folded its tokens in turn took 8.2 us for 64 rows of 8 tokens: every fold is three round trips to the L2.)
__global__ void __launch_bounds__(kDecodeThreads)
decode_umma_merge_kernel(DecodeParams p, int ranges) {
  __shared__ float red[384];
  __shared__ long long sums[2][kDecodeThreads / 32];
  const int b = blockIdx.x, tok = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // blocks (real and phantom: the sequence the tile kernel cut into ranges) in front of row b and in all rows
  long long before = 0, all = 0;
  for (int r = tid; r < p.batch; r += kDecodeThreads) {
    const int n = blocks_in_sequence(p, (decode_row_len(p, r) + kBlk - 1) / kBlk);
    all += n;
    if (r < b) before += n;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    before += __shfl_xor_sync(kFullMask, before, o);
    all += __shfl_xor_sync(kFullMask, all, o);
  }
  if (lane == 0) { sums[0][warp] = before; sums[1][warp] = all; }
  __syncthreads();
  before = 0; all = 0;
#pragma unroll
  for (int w = 0; w < kDecodeThreads / 32; ++w) { before += sums[0][w]; all += sums[1][w]; }
  const int nb = (decode_row_len(p, b) + kBlk - 1) / kBlk;
  if (nb == 0 || all == 0) return;
  const Partition pt = make_partition(all, ranges);
  const int c_lo = pt.cta_of(before), c_hi = pt.cta_of(before + nb - 1);
  if (c_lo == c_hi) return;  // the range's CTAs wrote the row themselves
  const int slot_rows = p.width * kHq;
  const long long qbase = (long long)b * p.width;
  int first = c_lo, n = c_hi - c_lo + 1;
  if (n <= 32) {
    fold_parts<true>(p, red, tid, 0, first, c_lo, n, (qbase + tok) * kHq, slot_rows, tok * kHq);
    return;
  }
  // more than 32 parts (a few very long rows): a plain running fold, thread = (head, 8 dims), four parts in flight
  const int h = warp, d0 = lane * 8;
  {
    float M = kNegBig, L = 0.f, acc[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = 0.f;
    for (int i0 = 0; i0 < n; i0 += 4) {
      float2 e[4];
      float4 x[4][2];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const bool ok = i0 + k < n;
        const int c = c_lo + (ok ? i0 + k : 0);
        const long long row = ((long long)(2 * c + (c == c_lo ? 1 : 0)) * slot_rows + tok * kHq + h);
        e[k] = ok ? __ldcg(reinterpret_cast<const float2*>(p.part_ml + row * 2)) : make_float2(kNegBig, 0.f);
        const float4* src = reinterpret_cast<const float4*>(p.part_acc + row * kD + d0);
        x[k][0] = ok ? __ldcg(src) : make_float4(0.f, 0.f, 0.f, 0.f);
        x[k][1] = ok ? __ldcg(src + 1) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float Mn = fmaxf(M, e[k].x);
        const float fo = ex2_approx(M - Mn), fn = ex2_approx(e[k].x - Mn);
        M = Mn;
        L = L * fo + e[k].y * fn;
        acc[0] = acc[0] * fo + x[k][0].x * fn; acc[1] = acc[1] * fo + x[k][0].y * fn;
        acc[2] = acc[2] * fo + x[k][0].z * fn; acc[3] = acc[3] * fo + x[k][0].w * fn;
        acc[4] = acc[4] * fo + x[k][1].x * fn; acc[5] = acc[5] * fo + x[k][1].y * fn;
        acc[6] = acc[6] * fo + x[k][1].z * fn; acc[7] = acc[7] * fo + x[k][1].w * fn;
      }
    }
    const float inv = L > 0.f ? 1.f / L : 0.f;
    float4* o = reinterpret_cast<float4*>(p.out + ((qbase + tok) * kHq + h) * kD + d0);
    o[0] = make_float4(acc[0] * inv, acc[1] * inv, acc[2] * inv, acc[3] * inv);
    o[1] = make_float4(acc[4] * inv, acc[5] * inv, acc[6] * inv, acc[7] * inv);
  }
}

typedef CUresult (*UdEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static UdEncodeTiledFn ud_encode_fn() {
  static UdEncodeTiledFn fn = [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult res;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &res) != cudaSuccess ||
        res != cudaDriverEntryPointSuccess)
      ptr = nullptr;
    return reinterpret_cast<UdEncodeTiledFn>(ptr);
  }();
  return fn;
}

// A cache layer [token, kv head, 256] bf16 seen as {64 dims, token, 64-dim chunk, kv head}: one box of {64, 16, 4, 1}
// is one KV head's half of a block and lands as [chunk][16 tokens][128 B] with the 128-byte swizzle in every panel;
// a box of {64, 16, 1, 1} is one such panel.
template <int kChunks>
static bool ud_make_map(CUtensorMap* map, const void* base, uint64_t tokens) {
  const cuuint64_t dims[4] = {64, tokens, 4, (cuuint64_t)kHkv};
  const cuuint64_t strides[3] = {(cuuint64_t)kTokenBytes, 128, (cuuint64_t)kRowBytes};
  const cuuint32_t box[4] = {64, (cuuint32_t)kBlk, kChunks, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  return ud_encode_fn()(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// p as launch_decode_wide takes it (width 1..8, carved workspace whose partial area holds ws_slots(decode_wide_num_ctas())
// slots of width * kHq rows).  NVJ_ERR_UNSUPPORTED: no tensor-map encoder, a scale that is not positive (row maxima are
// taken before scaling), the packed or the appending form.
int launch_decode_umma(const DecodeParams& p, cudaStream_t stream) {
  if (p.width < 1 || p.width > kUdMaxWidth || p.num_blocks < 1 || (p.num_blocks + 1) * kBlk > 0x7fffffffLL || !ud_encode_fn() ||
      !(p.scale > 0.f) || p.packed_rows || p.new_k || p.kv_indptr)
    return NVJ_ERR_UNSUPPORTED;
  const int ctas = decode_wide_num_ctas();
  if (ctas < 2) return NVJ_ERR_LAUNCH;
  const int ranges = ctas / 2;
  CUtensorMap k_map, v_map;
  if (!tensor_map_cached(&k_map, 4, p.k_cache, (uint64_t)p.num_blocks * kBlk, ud_make_map<1>) ||
      !tensor_map_cached(&v_map, 3, p.v_cache, (uint64_t)p.num_blocks * kBlk, ud_make_map<4>))
    return NVJ_ERR_UNSUPPORTED;
  static PerDeviceFlags smem_opted_in;
  constexpr int kSmemBytes = (int)sizeof(UdSmem) + 1024;
  static_assert(kSmemBytes <= 232448, "the tile ring exceeds the shared memory of one CTA");
  if (!once_per_device(smem_opted_in, [](int) {
        return cudaFuncSetAttribute(decode_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) == cudaSuccess;
      }))
    return NVJ_ERR_LAUNCH;
  DecodeParams q = p;
  q.row_end_cost = kUdRowEndCost;
  decode_umma_kernel<<<2 * ranges, kDecodeThreads, kSmemBytes, stream>>>(k_map, v_map, q);
  if (cudaGetLastError() != cudaSuccess) return NVJ_ERR_LAUNCH;
  decode_umma_merge_kernel<<<dim3(p.batch, p.width), kDecodeThreads, 0, stream>>>(q, ranges);
  return cudaGetLastError() == cudaSuccess ? NVJ_OK : NVJ_ERR_LAUNCH;
}

}  // namespace nvj
