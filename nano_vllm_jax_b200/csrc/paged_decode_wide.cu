// Paged GQA decode attention with the products on tensor-core tiles, for rows of 1..8 query tokens:
// the decode step proper (width 1, with the optional fused append of the step's new K/V row) and
// the verification of speculated tokens / multi-token prediction (width 2..8).  Cache shape of the
// model's full-attention layer: bf16, 16-token blocks, 2 KV heads x 4 query heads, head_dim 256.
//
// The kernel is HBM-bound: every K/V byte is read from HBM exactly once.  On the CUDA cores the dot
// products take half of the issue slots at width 1 and would make the kernel compute-bound beyond
// it, so the scores and the weighted sums run on the tensor cores (mma.sync m16n8k16, bf16 in, fp32
// accumulate): the width * 4 query rows of one KV head fill one 16-row tile.  Around the arithmetic
// the scheme is the CUDA-core kernel's (paged_decode.cu, decode_parts.cuh): all blocks of all
// rows form one sequence cut into equal ranges, one per CTA (one CTA per SM here, the accumulators
// need the registers); a ring of (K, V) blocks is kept in flight; a row that straddles CTAs is
// finished by the CTA that arrives last, in two levels when it was cut into many partials.
//   * Staging: one TMA tiled copy per 16 KiB block of K and of V, over a 4-D view of the cache whose box
//     lands as [kv head][64-dim chunk][16 tokens][128 B] with the 128-byte swizzle, so that ldmatrix reads
//     the tiles without bank conflicts.
//   * Warp w = (block parity w & 1, kv head (w >> 1) & 1, dim half w >> 2).  The four warps of a
//     parity take every other block: each computes the 16 x 16 scores of its KV head over all 256
//     dims (the two dim halves repeat this; it is a quarter of the work) and accumulates its 128
//     output dims.  The softmax weights enter the second product as two bf16 terms (hi + lo), which
//     keeps the result within 2e-3 of an fp32 evaluation.
//   * The two parities of a (kv head, dim half) merge through shared memory at the end of a row
//     segment.
//   * Rows of 5..8 query tokens need two 16-row tiles per KV head, and a warp has registers for one
//     (64 of query fragments + 64 of accumulators).  The kernel is then built in its second form
//     (kDual): the two warps of a (kv head, dim half) no longer split the blocks by parity but the
//     ROWS: both read every staged block, one for tokens 0..3, the other for tokens 4..7, and
//     nothing is merged between them.  K/V still cross HBM once; the tensor work per block doubles
//     and every warp now walks every block, which makes this form bound by a warp's chain of dependent
//     tile products (width 8 takes ~1.9x the width-1 time; entering the softmax weights as one bf16
//     term instead of two was measured: 11% faster at 4e-3 instead of 2e-3 error, not taken).
// Semantics: nanovllm_jax/kv_cache.py:852-998 (key p of row b is visible to token t when
// p < seq_lens[b] and, at width > 1 with positions given, p <= positions[b, t]); the fused append
// follows nanovllm_jax/kernels/full_attention_triton.py:373-485 (positions are then the slots the
// new rows go to).

#include <cuda.h>

#include <mutex>

#include "decode_parts.cuh"
#include "umma.cuh"

namespace nvj {

// Development aid, compiled in only with -DNVJ_PHASE_TIMING: thread 0 of every CTA stamps the global timer at the
// kernel's phase boundaries, and nvj_debug_phase_ns copies the stamps out.
#ifdef NVJ_PHASE_TIMING
__device__ unsigned long long g_phase_ns[256][12];  // slots 0-7: stamps; 8: the SM the CTA ran on; 9: its number of blocks; 10: ns spent finishing segments; 11: folds it did
#define NVJ_PHASE(i) do { if (threadIdx.x == 0) g_phase_ns[blockIdx.x][i] = global_timer_ns(); } while (0)
#define NVJ_PHASE_NOTE(i, v) do { if (threadIdx.x == 0) g_phase_ns[blockIdx.x][i] = (v); } while (0)
#else
#define NVJ_PHASE(i) do { } while (0)
#define NVJ_PHASE_NOTE(i, v) do { } while (0)
#endif

// An even number, so that a stage always holds blocks of the same parity and is read by the same four warps: a
// parity wait can only tell two consecutive phases of an mbarrier apart, and a warp that waited for every other
// phase of a stage's barrier could take an unfinished phase for the one after it, release the stage early and
// leave a copy in flight when the CTA exits (seen as a launch failure with five stages).
constexpr int kWStages = 4;
static_assert(kWStages % 2 == 0, "each stage must belong to one block parity");
constexpr int kWMaxWidth = 8;   // 1..4: one row tile per warp; 5..8: the dual form
constexpr int kWideMaxWidth = 16;  // what nvj_paged_decode_wide takes; beyond kWMaxWidth on the tcgen05 form only
constexpr int kWPad = 136;                    // row pitch (floats) of the parity exchange buffer

struct WideSmem {
  alignas(1024) char tiles[kWStages][2][kTileBytes];  // [stage][K|V][kv head][chunk][16 tokens][128 B]
  alignas(16) float xo[4][16][kWPad];                 // accumulators of the odd-parity warps
  float xm[4][16], xl[4][16];                         // their running max and sum
  float red[384];                                     // scratch of fold_parts
  alignas(8) unsigned long long full_bar[kWStages];
  alignas(8) unsigned long long empty_bar[kWStages];
  int ring_blk[kRing];
  signed char ring_rows[kRing];
  int scan[16];
  int start_b, start_j;
  int is_last;
  int abort_flag;
};

// One whole block (16 KiB) of the 4-D view {64 dims, token, 64-dim chunk, kv head} of a cache layer.
__device__ __forceinline__ void w_tma_block(uint32_t dst, const CUtensorMap* map, int token, uint32_t bar) {
  uint64_t policy;  // every block is read once: do not let it displace what the L2 is good for
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3, %4, %5}], [%6], %7;"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(0), "r"(token), "r"(0), "r"(0), "r"(bar), "l"(policy)
      : "memory");
}

__device__ __forceinline__ void w_ldsm4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void w_ldsm4_t(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void w_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// (lo, hi) -> packed bf16 pair, and what the rounding left over
__device__ __forceinline__ uint32_t w_pack_hi_lo(float x, float y, uint32_t& lo) {
  const __nv_bfloat16 hx = __float2bfloat16_rn(x), hy = __float2bfloat16_rn(y);
  const __nv_bfloat16 lx = __float2bfloat16_rn(x - __bfloat162float(hx)), ly = __float2bfloat16_rn(y - __bfloat162float(hy));
  lo = (uint32_t)__bfloat16_as_ushort(lx) | ((uint32_t)__bfloat16_as_ushort(ly) << 16);
  return (uint32_t)__bfloat16_as_ushort(hx) | ((uint32_t)__bfloat16_as_ushort(hy) << 16);
}

// One lane refills ring stage n % kWStages with the K and V block of iteration n, after
// (wait_first) the four warps that read the stage's previous occupant have released it.
__device__ __forceinline__ void w_issue_block(const DecodeParams& p, WideSmem& sm, const CUtensorMap* k_map,
                                              const CUtensorMap* v_map, int n, bool wait_first) {
  const int stage = n % kWStages;
  if (wait_first) {
    if (!mbar_wait(smem_u32(&sm.empty_bar[stage]), (uint32_t)((n / kWStages) - 1) & 1u, &sm.abort_flag, p.status)) return;
  }
  const uint32_t full = smem_u32(&sm.full_bar[stage]);
  const int blk = sm.ring_blk[n & (kRing - 1)];
  if (sm.ring_rows[n & (kRing - 1)] > 0) {
    mbar_arrive_expect_tx(full, 2u * kTileBytes);
    w_tma_block(smem_u32(sm.tiles[stage][0]), k_map, blk * kBlk, full);
    w_tma_block(smem_u32(sm.tiles[stage][1]), v_map, blk * kBlk, full);
  } else {
    mbar_arrive(full);
  }
}

// Per-warp state: the query rows as A fragments, the output accumulators of the warp's 128 dims,
// running max (log2 units) and this lane's share of the sum for rows g and g + 8.
struct WideState {
  uint32_t qa[16][4];
  float o[16][4];
  float m[2], l[2];
  int pos[2];  // last visible key of rows g, g + 8 (-1: the row is padding)
};

// One block (16 keys) of the warp's KV head: scores over all 256 dims, online softmax, weighted
// sum into the warp's 128 output dims.  kt / vt: the KV head's part of the staged K / V tile;
// `rows` keys of the block exist, the block starts at key `key0` of the row.
__device__ __forceinline__ void w_process_block(uint32_t kt, uint32_t vt, int lane, int dh, int rows, int key0, float c,
                                                WideState& st) {
  const int g = lane >> 2, t = lane & 3;
  // ---- scores
  float s[2][4];
#pragma unroll
  for (int j = 0; j < 2; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) s[j][e] = 0.f;
  {
    const int key = ((lane >> 4) & 1) * 8 + (lane & 7), hi = (lane >> 3) & 1;
    const uint32_t base = kt + key * 128;
#pragma unroll
    for (int ks = 0; ks < 16; ++ks) {
      uint32_t b[4];
      w_ldsm4(base + (ks >> 2) * 2048 + ((((ks & 3) * 2 + hi) ^ (lane & 7)) << 4), b);
      w_mma(s[0], st.qa[ks], b[0], b[1]);
      w_mma(s[1], st.qa[ks], b[2], b[3]);
    }
  }
  // ---- mask, running max, weights
  float mx[2] = {kNegBig, kNegBig};
#pragma unroll
  for (int j = 0; j < 2; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int kb = 8 * j + 2 * t + (e & 1), r = e >> 1;
      const bool ok = kb < rows && key0 + kb <= st.pos[r];
      s[j][e] = ok ? s[j][e] * c : kNegBig;
      mx[r] = fmaxf(mx[r], s[j][e]);
    }
  float alpha[2], mu[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    mx[r] = fmaxf(mx[r], __shfl_xor_sync(kFullMask, mx[r], 1));
    mx[r] = fmaxf(mx[r], __shfl_xor_sync(kFullMask, mx[r], 2));
    const float mn = fmaxf(st.m[r], mx[r]);
    alpha[r] = ex2_approx(st.m[r] - mn);
    st.m[r] = mn;
    mu[r] = mn <= kNegBig ? 0.f : mn;  // nothing visible yet: the weights below come out as 0
    st.l[r] *= alpha[r];
  }
  uint32_t ph[4], pl[4];
#pragma unroll
  for (int j = 0; j < 2; ++j)
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const float p0 = ex2_approx(s[j][2 * r] - mu[r]), p1 = ex2_approx(s[j][2 * r + 1] - mu[r]);
      st.l[r] += p0 + p1;
      ph[2 * j + r] = w_pack_hi_lo(p0, p1, pl[2 * j + r]);
    }
  if (__any_sync(kFullMask, alpha[0] != 1.f || alpha[1] != 1.f)) {
#pragma unroll
    for (int n = 0; n < 16; ++n) {
      st.o[n][0] *= alpha[0]; st.o[n][1] *= alpha[0];
      st.o[n][2] *= alpha[1]; st.o[n][3] *= alpha[1];
    }
  }
  // ---- weighted sum of the V rows
  {
    const int key = ((lane >> 3) & 1) * 8 + (lane & 7), hi = lane >> 4;
    const uint32_t base = vt + dh * 4096 + key * 128;
#pragma unroll
    for (int n2 = 0; n2 < 8; ++n2) {
      uint32_t b[4];
      w_ldsm4_t(base + (n2 >> 2) * 2048 + ((((n2 & 3) * 2 + hi) ^ (lane & 7)) << 4), b);
      w_mma(st.o[2 * n2], ph, b[0], b[1]);
      w_mma(st.o[2 * n2], pl, b[0], b[1]);
      w_mma(st.o[2 * n2 + 1], ph, b[2], b[3]);
      w_mma(st.o[2 * n2 + 1], pl, b[2], b[3]);
    }
  }
}

// End of a row segment: the two block parities of every (kv head, dim half) merge through shared
// memory, then the even-parity warps write either the final output rows (the segment covered the
// whole row) or this CTA's partial; the CTA that delivers a row's last partial folds them all,
// token by token (see the width-1 kernel for the two-level scheme).  (A CTA whose range goes on behind a shared
// segment could put the count and the fold off until its last block is done, so that its copies in flight do not run
// dry meanwhile.  Measured: worse, 41.5 -> 44.0 us on 16 rows x 4096 tokens and 227.5 -> 230.9 us on 256 rows, because
// the row then completes later and two counts queue up at the end of the CTA.)
template <bool kDual>
__device__ __forceinline__ void w_finish_segment(const DecodeParams& p, WideSmem& sm, const Seg& s, WideState& st, int warp,
                                                 int lane, const Partition& pt) {
  const int g = lane >> 2, t = lane & 3, tid = warp * 32 + lane;
  const int par = warp & 1, kvh = (warp >> 1) & 1, dh = warp >> 2, grp = warp >> 1;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    st.l[r] += __shfl_xor_sync(kFullMask, st.l[r], 1);
    st.l[r] += __shfl_xor_sync(kFullMask, st.l[r], 2);
  }
  if (!kDual && par == 1) {
#pragma unroll
    for (int n = 0; n < 16; ++n) {
      *reinterpret_cast<float2*>(&sm.xo[grp][g][n * 8 + 2 * t]) = make_float2(st.o[n][0], st.o[n][1]);
      *reinterpret_cast<float2*>(&sm.xo[grp][g + 8][n * 8 + 2 * t]) = make_float2(st.o[n][2], st.o[n][3]);
    }
    if (t == 0) {
      sm.xm[grp][g] = st.m[0]; sm.xm[grp][g + 8] = st.m[1];
      sm.xl[grp][g] = st.l[0]; sm.xl[grp][g + 8] = st.l[1];
    }
  }
  named_bar_sync(1, kDecodeThreads);
  const bool whole_row = (s.j0 == 0 && s.j1 == s.nb);
  const long long qbase = p.packed_rows ? (long long)p.query_start_loc[s.b] : (long long)s.b * p.width;  // first query token
  const int slot = partial_slot(blockIdx.x, s.j0 == 0);
  const int slot_rows = p.width * kHq;  // rows of one partial slot: [token][head]
  if (kDual || par == 0) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int row = g + 8 * r, tok = (kDual ? 4 * par : 0) + (row >> 2);
      // dual form: this warp alone holds the row's state; else the odd-parity warp's share comes from shared memory
      const float m1 = kDual ? kNegBig : sm.xm[grp][row], l1 = kDual ? 0.f : sm.xl[grp][row];
      const float M = fmaxf(st.m[r], m1);
      const float f0 = ex2_approx(st.m[r] - M), f1 = ex2_approx(m1 - M);
      const float L = st.l[r] * f0 + l1 * f1;
      if (tok >= p.width) continue;
      const int head = kvh * kG + (row & 3);
      const float inv = whole_row ? (L > 0.f ? 1.f / L : 0.f) : 1.f;
      float* dst = whole_row ? p.out + ((qbase + tok) * kHq + head) * kD
                             : p.part_acc + ((long long)slot * slot_rows + tok * kHq + head) * kD;
      dst += dh * 128 + 2 * t;
#pragma unroll
      for (int n = 0; n < 16; ++n) {
        const float2 x = kDual ? make_float2(0.f, 0.f) : *reinterpret_cast<const float2*>(&sm.xo[grp][row][n * 8 + 2 * t]);
        *reinterpret_cast<float2*>(dst + n * 8) =
            make_float2((st.o[n][2 * r] * f0 + x.x * f1) * inv, (st.o[n][2 * r + 1] * f0 + x.y * f1) * inv);
      }
      if (!whole_row && dh == 0 && t == 0)
        *reinterpret_cast<float2*>(p.part_ml + ((long long)slot * slot_rows + tok * kHq + head) * 2) = make_float2(M, L);
    }
  }
  if (whole_row) {
    named_bar_sync(1, kDecodeThreads);  // the exchange buffer is free again
    return;
  }
  // ---- cross-CTA: count this partial in; the last arrival folds
  const long long row_g0 = s.g0 - s.j0;
  const int c_lo = pt.cta_of(row_g0);
  const int c_hi = pt.cta_of(row_g0 + s.nb - 1);
  const int grid = gridDim.x;
  const bool tree = c_hi - c_lo + 1 > kTreeMergeMin;
  const int cg = blockIdx.x / kMergeGroup, g_lo = c_lo / kMergeGroup, g_hi = c_hi / kMergeGroup;
  const int first = tree ? max(c_lo, cg * kMergeGroup) : c_lo;
  const int last = tree ? min(c_hi, cg * kMergeGroup + kMergeGroup - 1) : c_hi;
  int32_t* counter = tree ? p.group_counters + 2 * cg + (cg == g_lo ? 1 : 0) : p.counters + s.b;
  __threadfence();
  named_bar_sync(1, kDecodeThreads);
  if (tid == 0) sm.is_last = (atomicAdd(counter, 1) == last - first) ? 1 : 0;
  named_bar_sync(1, kDecodeThreads);
  NVJ_PHASE(7);
  if (!sm.is_last) return;
  __threadfence();
  if (!tree) {
    for (int tok = 0; tok < p.width; ++tok) {
      fold_parts<true, 13>(p, sm.red, tid, 0, c_lo, c_lo, c_hi - c_lo + 1, (qbase + tok) * kHq, slot_rows, tok * kHq);
      named_bar_sync(1, kDecodeThreads);
    }
    if (tid == 0) *counter = 0;
    return;
  }
  for (int tok = 0; tok < p.width; ++tok) {
    fold_parts<false, 13>(p, sm.red, tid, 0, first, c_lo, last - first + 1, 2LL * grid + 2 * cg + (cg == g_lo ? 1 : 0), slot_rows,
                      tok * kHq);
    named_bar_sync(1, kDecodeThreads);
  }
  if (tid == 0) *counter = 0;
  __threadfence();
  named_bar_sync(1, kDecodeThreads);
  if (tid == 0) sm.is_last = (atomicAdd(p.counters + s.b, 1) == g_hi - g_lo) ? 1 : 0;
  named_bar_sync(1, kDecodeThreads);
  if (!sm.is_last) return;
  __threadfence();
  for (int tok = 0; tok < p.width; ++tok) {
    fold_parts<true, 13>(p, sm.red, tid, 2LL * grid, g_lo, g_lo, g_hi - g_lo + 1, (qbase + tok) * kHq, slot_rows,
                     tok * kHq);
    named_bar_sync(1, kDecodeThreads);
  }
  if (tid == 0) p.counters[s.b] = 0;
}

template <bool kDual>
__global__ void __launch_bounds__(kDecodeThreads, 1)
decode_wide_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map, DecodeParams p) {
  extern __shared__ unsigned char w_smem_raw[];
  WideSmem& sm = *reinterpret_cast<WideSmem*>((reinterpret_cast<uintptr_t>(w_smem_raw) + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int grid = gridDim.x;

  NVJ_PHASE(0);
  // The kernel opens with three dependent trips to memory (lengths -> block ids -> K/V blocks).  While the first is
  // under way, pull what the others will need towards the SM: the tensor maps, and this CTA's share of the block
  // tables into the L2 (all CTAs together cover the tables, so the second trip ends in the L2 for everyone).
  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&k_map)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&v_map)) : "memory");
  }
  if (!p.kv_indptr) {
    const long long lines = ((long long)p.batch * p.table_width * (long long)sizeof(int32_t) + 127) / 128;
    const long long line = (long long)blockIdx.x * kDecodeThreads + threadIdx.x;
    if (line < lines) asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const char*>(p.block_tables) + line * 128));
  }
  if (threadIdx.x == 0) { sm.start_b = p.batch; sm.start_j = 0; sm.abort_flag = 0; sm.is_last = 0; }  // the scan below has the barrier
  // ---- pass 1: total number of blocks; zero the output of inactive rows
  int mine = 0, first_n = 0;
  for (int base = 0; base < p.batch; base += kDecodeThreads) {
    const int b = base + threadIdx.x;
    int len = 0;
    if (b < p.batch) len = decode_row_len(p, b);
    if (base == 0) first_n = blocks_in_sequence(p, (len + kBlk - 1) / kBlk);
    mine += blocks_in_sequence(p, (len + kBlk - 1) / kBlk);
    // rows without keys get zeros; in a packed batch only the rows this pass owns (one query token) are touched
    const bool mine_to_zero = b < p.batch && len <= 0 && (b % grid) == (int)blockIdx.x &&
                              (!p.packed_rows || p.query_start_loc[b + 1] - p.query_start_loc[b] == 1);
    const unsigned idle = __ballot_sync(kFullMask, mine_to_zero);
    for (unsigned m = idle; m; m &= m - 1) {
      const int bb = base + (warp << 5) + (__ffs(m) - 1);
      float4* o = reinterpret_cast<float4*>(p.out + (p.packed_rows ? (long long)p.query_start_loc[bb] : (long long)bb * p.width) * kHq * kD);
      for (int i = lane; i < p.width * kHq * kD / 4; i += 32) o[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
  int total = 0;
  const int incl = cta_inclusive_scan(mine, sm.scan, total);
  if (total == 0) return;
  const Partition pt = make_partition(total, grid);
  if ((int)blockIdx.x >= pt.n) return;
  const long long g0 = pt.start(blockIdx.x);
  const long long g1 = pt.start(blockIdx.x + 1);
  if (g0 == g1) return;
  NVJ_PHASE(1);

  // ---- pass 2: locate (row, block) of g0
  long long carry = 0;
  if (p.batch <= kDecodeThreads) {  // one row per thread: the scan of pass 1 has the answer already
    const long long excl = incl - first_n;
    if (first_n > 0 && excl <= g0 && g0 < excl + first_n) { sm.start_b = threadIdx.x; sm.start_j = (int)(g0 - excl); }
    carry = g0 + 1;  // skips the loop below
  }
  for (int base = 0; base < p.batch && carry <= g0; base += kDecodeThreads) {
    const int b = base + threadIdx.x;
    int n = 0;
    if (b < p.batch) n = blocks_in_sequence(p, (decode_row_len(p, b) + kBlk - 1) / kBlk);
    int chunk_total = 0;
    const long long excl = carry + cta_inclusive_scan(n, sm.scan, chunk_total) - n;
    if (n > 0 && excl <= g0 && g0 < excl + n) { sm.start_b = b; sm.start_j = (int)(g0 - excl); }
    carry += chunk_total;
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < kWStages; ++s) {
      mbar_init(smem_u32(&sm.full_bar[s]), 1);
      mbar_init(smem_u32(&sm.empty_bar[s]), kDual ? 8 : 4);
    }
    mbar_fence_init();
  }
  __syncthreads();
  NVJ_PHASE(2);
  const int n_iters = blocks_in_range(p, sm.start_b, sm.start_j, g0, g1);  // the range's real blocks
  if (n_iters == 0) return;
#ifdef NVJ_PHASE_TIMING
  {
    unsigned smid;
    asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
    NVJ_PHASE_NOTE(8, (unsigned long long)smid);
    NVJ_PHASE_NOTE(9, (unsigned long long)n_iters);
    NVJ_PHASE_NOTE(10, 0ull);
    NVJ_PHASE_NOTE(11, 0ull);
  }
#endif

  FillState fs;
  fs.b = sm.start_b; fs.jn = sm.start_j; fs.g = g0; fs.j = 0; fs.nsegs = 0; fs.has = false;
  fill_ring(p, sm, fs, g1, 0, n_iters < kRing ? n_iters : kRing);
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int n = 0; n < kWStages && n < n_iters; ++n) w_issue_block(p, sm, &k_map, &v_map, n, false);
  }
  NVJ_PHASE(3);

  int b = sm.start_b, j = sm.start_j;
  long long g = g0;
  Seg s;
  int it = 0;
  const int par = warp & 1, kvh = (warp >> 1) & 1, dh = warp >> 2;
  const int fg = lane >> 2, ft = lane & 3;
  const float c = p.scale * kLog2e;
  WideState st;
  while (next_seg(p, b, j, g, g1, s)) {
    // query rows of this KV head as A fragments: row = token * 4 + head of the group; rows past the width are zero
    // (packed_rows: the row's single query token sits at query_start_loc[b]; its length is already capped by its position)
    const long long qbase = p.packed_rows ? (long long)p.query_start_loc[s.b] : (long long)s.b * p.width;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int row = fg + 8 * r, tok = (kDual ? 4 * par : 0) + (row >> 2);
      const bool real = tok < p.width;
      const __nv_bfloat16* qrow =
          static_cast<const __nv_bfloat16*>(p.q) + ((qbase + (real ? tok : 0)) * kHq + kvh * kG + (row & 3)) * kD;
#pragma unroll
      for (int ks = 0; ks < 16; ++ks) {
        st.qa[ks][r] = real ? *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 2 * ft) : 0u;
        st.qa[ks][r + 2] = real ? *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 8 + 2 * ft) : 0u;
      }
      st.pos[r] = real ? (p.positions && !p.new_k ? p.positions[qbase + tok] : 0x7fffffff) : -1;
      st.m[r] = kNegBig;
      st.l[r] = 0.f;
    }
#pragma unroll
    for (int n = 0; n < 16; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) st.o[n][e] = 0.f;

    // Fused append (width 1).  The CTA that owns block min(pos / 16, nb - 1) of the row writes the new K/V row
    // (one warp per KV head); its copy of that block may race with the store, so every warp that reads the block
    // overwrites the row in the staged tile, from the same source, once the copy has landed: no fence is needed
    // and nothing waits for the store.
    int patch_j = -1, patch_t = 0;
    if (p.new_k) {
      const int pos = p.pre_append ? p.seq_lens[s.b] : p.positions[s.b];
      const int jt = pos >> 4;
      const int jw = jt < s.nb - 1 ? jt : s.nb - 1;
      if (pos >= 0 && jw >= s.j0 && jw < s.j1) {
        const long long tgt = jt < p.table_width ? (long long)p.block_tables[decode_table_base(p, s.b) + jt] : -1;
        if (tgt >= 0 && tgt < p.num_blocks) {
          if (par == 0 && dh == 0) {
            const long long src = (long long)s.b * kTokenBytes + kvh * kRowBytes + lane * 16;
            const long long dst = (tgt * kBlk + (pos & 15)) * kTokenBytes + kvh * kRowBytes + lane * 16;
            *reinterpret_cast<uint4*>(const_cast<char*>(p.k_cache) + dst) =
                *reinterpret_cast<const uint4*>(static_cast<const char*>(p.new_k) + src);
            *reinterpret_cast<uint4*>(const_cast<char*>(p.v_cache) + dst) =
                *reinterpret_cast<const uint4*>(static_cast<const char*>(p.new_v) + src);
          }
          if (jt == jw && pos < s.len) { patch_j = jw; patch_t = pos & 15; }
        } else if (warp == 0 && lane == 0) {
          atomicOr(p.status, NVJ_DEV_BAD_BLOCK_ID);
        }
      }
    }
    for (int jb = s.j0; jb < s.j1; ++jb, ++it) {
      if ((it & (kRing / 2 - 1)) == 0 && it > 0) {
        named_bar_sync(1, kDecodeThreads);
        const int n0 = it + kRing / 2;
        if (n0 < n_iters) fill_ring(p, sm, fs, g1, n0, n_iters - n0 < kRing / 2 ? n_iters - n0 : kRing / 2);
        named_bar_sync(1, kDecodeThreads);
      }
      if (!kDual && (it & 1) != par) continue;
      const int stage = it % kWStages;
      mbar_wait(smem_u32(&sm.full_bar[stage]), (uint32_t)(it / kWStages) & 1u, &sm.abort_flag, p.status);
      const int rows = sm.ring_rows[it & (kRing - 1)];
      if (it == 0) NVJ_PHASE(4);
      if (jb == patch_j) {  // lane l carries 16-byte piece l of the KV head's 512-byte row; the source is cache-hot
        const long long src = (long long)s.b * kTokenBytes + kvh * kRowBytes + lane * 16;
        const uint32_t off = kvh * 8192 + (lane >> 3) * 2048 + patch_t * 128 + (((lane & 7) ^ (patch_t & 7)) << 4);
        *reinterpret_cast<uint4*>(sm.tiles[stage][0] + off) = *reinterpret_cast<const uint4*>(static_cast<const char*>(p.new_k) + src);
        *reinterpret_cast<uint4*>(sm.tiles[stage][1] + off) = *reinterpret_cast<const uint4*>(static_cast<const char*>(p.new_v) + src);
        __syncwarp();
      }
      if (rows > 0)
        w_process_block(smem_u32(sm.tiles[stage][0]) + kvh * 8192, smem_u32(sm.tiles[stage][1]) + kvh * 8192, lane, dh, rows,
                        jb * kBlk, c, st);
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(smem_u32(&sm.empty_bar[stage]));
        // the warps that read the stage take turns to refill it: the four warps of a parity, or all eight (dual form)
        if ((kDual ? warp == (it & 7) : (warp >> 1) == ((it >> 1) & 3)) && it + kWStages < n_iters)
          w_issue_block(p, sm, &k_map, &v_map, it + kWStages, true);
      }
      __syncwarp();
    }
    NVJ_PHASE(5);
#ifdef NVJ_PHASE_TIMING
    const unsigned long long fin0 = global_timer_ns();
#endif
    w_finish_segment<kDual>(p, sm, s, st, warp, lane, pt);
#ifdef NVJ_PHASE_TIMING
    if (threadIdx.x == 0) {
      g_phase_ns[blockIdx.x][10] += global_timer_ns() - fin0;
      g_phase_ns[blockIdx.x][11] += (unsigned long long)sm.is_last;
    }
#endif
    NVJ_PHASE(6);
  }
  // Only after a timeout can copies still be in flight with nobody waiting for them: hold the
  // CTA's shared memory until they have landed.
  __syncthreads();
  if (threadIdx.x == 0 && sm.abort_flag) {
    const unsigned long long t0 = global_timer_ns();
    for (int back = 1; back <= kWStages && back <= n_iters; ++back) {
      const int i = n_iters - back;
      while (!mbar_try_wait(smem_u32(&sm.full_bar[i % kWStages]), (uint32_t)(i / kWStages) & 1u) &&
             global_timer_ns() - t0 < kWaitLimitNs) {
      }
    }
  }
  __syncthreads();
}

typedef CUresult (*WEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static WEncodeTiledFn w_encode_fn() {
  static WEncodeTiledFn fn = [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult res;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &res) != cudaSuccess ||
        res != cudaDriverEntryPointSuccess)
      ptr = nullptr;
    return reinterpret_cast<WEncodeTiledFn>(ptr);
  }();
  return fn;
}

// A cache layer [token, kv head, 256] bf16 seen as {64 dims, token, 64-dim chunk, kv head}: one box of
// {64, 16, 4, 2} is a whole block, and lands in shared memory as [kv head][chunk][16 tokens][128 B] with the
// 128-byte swizzle inside every [token][128 B] panel.
static bool w_make_map(CUtensorMap* map, const void* base, uint64_t tokens) {
  const cuuint64_t dims[4] = {64, tokens, 4, (cuuint64_t)kHkv};
  const cuuint64_t strides[3] = {(cuuint64_t)kTokenBytes, 128, (cuuint64_t)kRowBytes};
  const cuuint32_t box[4] = {64, (cuuint32_t)kBlk, 4, (cuuint32_t)kHkv};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  return w_encode_fn()(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                       CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

struct MapEntry {
  int kind;
  const void* base;
  uint64_t extent;
  CUtensorMap map;
};
static std::mutex g_map_mutex;
static MapEntry g_map_cache[128];
static unsigned g_map_next;

bool tensor_map_cached(CUtensorMap* map, int kind, const void* base, uint64_t extent, TensorMapMaker make) {
  std::lock_guard<std::mutex> lock(g_map_mutex);
  for (const MapEntry& e : g_map_cache)
    if (e.base == base && e.extent == extent && e.kind == kind && e.base != nullptr) {
      *map = e.map;
      return true;
    }
  if (!make(map, base, extent)) return false;
  MapEntry& e = g_map_cache[g_map_next++ % 128];
  e.kind = kind;
  e.base = base;
  e.extent = extent;
  e.map = *map;
  return true;
}

static PerDeviceFlags g_wide_ctas;  // 0 = not queried yet

int decode_wide_num_ctas() {  // one per SM of the current device
  const int dev = current_device();
  if (dev < 0) return 0;
  int n = g_wide_ctas.v[dev].load(std::memory_order_acquire);
  if (n == 0) {
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    n = sms < kMergeGroup * kGroupCounters / 2 ? sms : kMergeGroup * kGroupCounters / 2;
    g_wide_ctas.v[dev].store(n, std::memory_order_release);
  }
  return n;
}

static size_t wide_ml_bytes(int n, int width) { return ws_round(sizeof(float) * ws_slots(n) * width * kHq * 2); }
static size_t wide_acc_bytes(int n, int width) { return ws_round(sizeof(float) * ws_slots(n) * width * kHq * kD); }

// p carries everything but the tensor maps: pointers, shapes, width (1..4) and the carved workspace, whose
// partial area holds ws_slots(decode_wide_num_ctas()) slots of width * kHq rows.
int launch_decode_wide(const DecodeParams& p, cudaStream_t stream) {
  if (p.width < 1 || p.width > kWideMaxWidth || p.num_blocks < 1 || p.num_blocks * kBlk > 0x7fffffffLL || !w_encode_fn())
    return NVJ_ERR_UNSUPPORTED;
  int n = decode_wide_num_ctas();
  if (n <= 0) return NVJ_ERR_LAUNCH;
  // rows of 5 and more query tokens: the tcgen05 form (two 16-row tiles per warp pair make the mma.sync form
  // compute-bound, and it ends at 8 tokens)
  if (p.wide_form == 2 || (p.wide_form == 0 && p.width > 4)) {
    const int rc = launch_decode_umma(p, stream);
    if (rc != NVJ_ERR_UNSUPPORTED || p.wide_form == 2) return rc;
  }
  if (p.width > kWMaxWidth) return NVJ_ERR_UNSUPPORTED;
  if (p.cta_limit > 0 && p.cta_limit < n) n = p.cta_limit;
  DecodeParams q = p;
  q.row_end_cost = kRowEndCost;
  CUtensorMap k_map, v_map;
  if (!tensor_map_cached(&k_map, 0, p.k_cache, (uint64_t)p.num_blocks * kBlk, w_make_map) ||
      !tensor_map_cached(&v_map, 0, p.v_cache, (uint64_t)p.num_blocks * kBlk, w_make_map))
    return NVJ_ERR_UNSUPPORTED;
  static PerDeviceFlags smem_opted_in;
  const int smem = (int)sizeof(WideSmem) + 1024;
  if (!once_per_device(smem_opted_in, [smem](int) {
        return cudaFuncSetAttribute(decode_wide_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) == cudaSuccess &&
               cudaFuncSetAttribute(decode_wide_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) == cudaSuccess;
      }))
    return NVJ_ERR_LAUNCH;
  if (p.width > 4) decode_wide_kernel<true><<<n, kDecodeThreads, smem, stream>>>(k_map, v_map, q);
  else decode_wide_kernel<false><<<n, kDecodeThreads, smem, stream>>>(k_map, v_map, q);
  return cudaGetLastError() == cudaSuccess ? NVJ_OK : NVJ_ERR_LAUNCH;
}

}  // namespace nvj

#ifdef NVJ_PHASE_TIMING
extern "C" int nvj_debug_phase_ns(unsigned long long* host_out) {  // [256][8]
  return cudaMemcpyFromSymbol(host_out, nvj::g_phase_ns, sizeof(nvj::g_phase_ns)) == cudaSuccess ? 0 : 1;
}
#endif

extern "C" size_t nvj_paged_decode_wide_workspace_bytes(int max_batch) {
  using namespace nvj;
  if (max_batch < 0) return 0;
  const int n = decode_wide_num_ctas();
  if (n <= 0) return 0;
  return ws_header_bytes(max_batch) + wide_ml_bytes(n, kWMaxWidth) + wide_acc_bytes(n, kWMaxWidth);
}

extern "C" int nvj_paged_decode_wide(const void* q, const void* k_cache_layer, const void* v_cache_layer, int64_t num_blocks,
                                     const int32_t* block_tables, int table_width, const int32_t* seq_lens,
                                     const int32_t* positions, int batch, int width, float scale, float* out,
                                     void* workspace, size_t workspace_bytes, nvj_stream_t stream) {
  return nvj_paged_decode_wide_form(q, k_cache_layer, v_cache_layer, num_blocks, block_tables, table_width, seq_lens, positions,
                                    batch, width, scale, out, workspace, workspace_bytes, 0, stream);
}

extern "C" int nvj_paged_decode_wide_form(const void* q, const void* k_cache_layer, const void* v_cache_layer, int64_t num_blocks,
                                          const int32_t* block_tables, int table_width, const int32_t* seq_lens,
                                          const int32_t* positions, int batch, int width, float scale, float* out,
                                          void* workspace, size_t workspace_bytes, int form, nvj_stream_t stream) {
  using namespace nvj;
  if (batch < 0 || table_width < 0 || num_blocks < 0 || width < 1 || form < 0 || form > 2) return NVJ_ERR_INVALID_ARGUMENT;
  if (width > kWideMaxWidth || (form == 1 && width > kWMaxWidth)) return NVJ_ERR_UNSUPPORTED;
  if (batch == 0) return NVJ_OK;
  if (!q || !k_cache_layer || !v_cache_layer || !block_tables || !seq_lens || !out) return NVJ_ERR_INVALID_ARGUMENT;
  const uintptr_t al = reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k_cache_layer) |
                       reinterpret_cast<uintptr_t>(v_cache_layer) | reinterpret_cast<uintptr_t>(out) |
                       reinterpret_cast<uintptr_t>(workspace);
  if ((al & 15u) != 0) return NVJ_ERR_UNSUPPORTED;
  const int n = decode_wide_num_ctas();
  if (n <= 0) return NVJ_ERR_LAUNCH;
  DecodeParams p{};
  p.batch = batch;
  // rows of more than 8 tokens run on the tcgen05 form only, which parks two partials per pair of CTAs: n slots
  const size_t ml_bytes = width > kWMaxWidth ? ws_round(sizeof(float) * n * width * kHq * 2) : wide_ml_bytes(n, width);
  const size_t acc_bytes = width > kWMaxWidth ? ws_round(sizeof(float) * n * width * kHq * kD) : wide_acc_bytes(n, width);
  const int carved = carve_decode_workspace(p, workspace, workspace_bytes, ml_bytes, acc_bytes);
  if (carved != NVJ_OK) return carved;
  p.q = q;
  p.k_cache = static_cast<const char*>(k_cache_layer);
  p.v_cache = static_cast<const char*>(v_cache_layer);
  p.block_tables = block_tables;
  p.seq_lens = seq_lens;
  p.positions = positions;
  p.width = width;
  p.wide_form = form;
  p.out = out;
  p.num_blocks = num_blocks;
  p.table_width = table_width;
  p.block_size = kBlk;
  p.num_kv_heads = kHkv;
  p.num_q_heads = kHq;
  p.head_dim = kD;
  p.q_dtype = NVJ_BF16;
  p.kv_dtype = NVJ_BF16;
  p.scale = scale;
  return launch_decode_wide(p, static_cast<cudaStream_t>(stream));
}
