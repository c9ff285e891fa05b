// Paged GQA decode attention for the model's full-attention shape (bf16 cache,
// 16-token blocks, 2 KV heads x 4 query heads, head_dim 256), with the optional
// fused append of the step's new K/V row.
//
// The kernel is HBM-bound: every K/V byte is read from HBM exactly once.
//   * The cache layout [block, slot, kv_head, head_dim] makes one block of K (and
//     of V) one contiguous 16 KiB span, so a single 1-D bulk async copy
//     (cp.async.bulk -> shared memory, completion on an mbarrier) stages it; a
//     ring of kStages (K, V) block pairs is kept in flight, the eight warps
//     taking turns to refill the stage they have all just released.
//   * All blocks of all rows form one global sequence that is cut into equal
//     contiguous ranges, one per CTA (two CTAs per SM), so every CTA moves the
//     same number of bytes whatever the mix of context lengths.  A row that
//     straddles CTAs is finished by whichever of them arrives last (arrival
//     counter; nobody waits).
//   * Eight consumer warps split a block: warp w takes KV head (w & 1) and tokens
//     4*(w>>1) .. +3, covering all four query heads of the group.  Lane l owns
//     head_dim elements 8l..8l+7 of every row (one 16-byte shared-memory load),
//     the 16 (token, head) partial dot products are reduced across the warp by a
//     shuffle butterfly, and each warp keeps its own online-softmax state; states
//     are merged once per row segment.
// Arithmetic is fp32 (packed FFMA2), scores in log2 units, output fp32.
// Semantics: nanovllm_jax/kv_cache.py:852-998 for width-1 queries, and
// nanovllm_jax/kernels/full_attention_triton.py:373-485 for the fused append.

#include "decode_parts.cuh"

namespace nvj {

constexpr int kConsumerWarps = 8;
constexpr int kConsumerThreads = kConsumerWarps * 32;
static_assert(kDecodeThreads == kConsumerThreads, "every thread of the CTA is a consumer");
constexpr int kStages = 3;

struct DecodeSmem {
  alignas(128) char tiles[kStages][2][kTileBytes];  // [stage][K|V]
  alignas(16) float merge[kConsumerWarps][kD];      // one query-head slot of every warp
  alignas(16) float pbuf[kConsumerWarps][2][16];    // softmax weights of a unit, [token][head]
  float2 ml[kConsumerWarps][kG];                    // per warp (max, sum) per head slot
  float2 ML[kHkv][kG];                              // merged (max, sum) per head
  alignas(8) unsigned long long full_bar[kStages];
  alignas(8) unsigned long long empty_bar[kStages];
  int ring_blk[kRing];            // physical block id of the CTA's iteration n, at n % kRing
  signed char ring_rows[kRing];   // tokens of that block that are attended (0: skip the block)
  int scan[16];
  int start_b, start_j;
  int is_last;
  int abort_flag;
};

// Per-warp online-softmax state.  q2 / acc2 hold packed fp32 pairs of the lane's
// eight head_dim elements.  q2 is indexed by head *slot*: slot h of lane l holds
// query head h ^ hperm(l), which is what lets the score butterfly run without
// selects.  acc2 and m4 are indexed by the real head of the group.
struct WarpState {
  float2 q2[kG][4];
  float2 acc2[kG][4];
  float m4[kG];
  float m_own;   // running max of the head this lane's score belongs to
  float l_part;  // partial sum of weights for this lane's (token, head) position
};

__device__ __forceinline__ void unpack8(const uint4& r, float2 (&o)[4]) {
  o[0] = bf16x2_to_float2(r.x);
  o[1] = bf16x2_to_float2(r.y);
  o[2] = bf16x2_to_float2(r.z);
  o[3] = bf16x2_to_float2(r.w);
}

// One unit = 4 tokens of one KV head: scores for 4 tokens x 4 heads, online
// softmax update, weighted sum of the 4 V rows.  kt/vt point at this warp's
// first row of the staged K/V block (token stride kTokenBytes); `nvalid` (1..4)
// tokens are real when kMasked.
template <bool kMasked>
__device__ __forceinline__ void process_unit(const char* kt, const char* vt, int lane, int nvalid,
                                             WarpState& st, float* pbuf) {
  const int rperm = lane >> 3;        // token of the lane's final score
  const int h_own = (lane >> 1) & 3;  // head of the lane's final score
  // ---- scores: s[slot r][slot h], partial over the lane's 8 elements
  float s[16];
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int row = r ^ rperm;
    uint4 kr = *reinterpret_cast<const uint4*>(kt + row * kTokenBytes + lane * 16);
    if (kMasked && row >= nvalid) kr = make_uint4(0u, 0u, 0u, 0u);
    float2 k2[4];
    unpack8(kr, k2);
#pragma unroll
    for (int h = 0; h < kG; ++h) {
      float2 a = fma2(st.q2[h][0], k2[0], make_float2(0.f, 0.f));
      a = fma2(st.q2[h][1], k2[1], a);
      a = fma2(st.q2[h][2], k2[2], a);
      a = fma2(st.q2[h][3], k2[3], a);
      s[r * 4 + h] = a.x + a.y;
    }
  }
  // ---- butterfly reduce-scatter over the 32 lanes (no selects: see WarpState)
#pragma unroll
  for (int i = 0; i < 8; ++i) s[i] += __shfl_xor_sync(kFullMask, s[i + 8], 16);
#pragma unroll
  for (int i = 0; i < 4; ++i) s[i] += __shfl_xor_sync(kFullMask, s[i + 4], 8);
#pragma unroll
  for (int i = 0; i < 2; ++i) s[i] += __shfl_xor_sync(kFullMask, s[i + 2], 4);
  s[0] += __shfl_xor_sync(kFullMask, s[1], 2);
  float sc = s[0] + __shfl_xor_sync(kFullMask, s[0], 1);  // score of (token rperm, head h_own)
  if (kMasked && rperm >= nvalid) sc = -INFINITY;
  // ---- online softmax: unit maximum per head, rescale only when it grows
  float bm = fmaxf(sc, __shfl_xor_sync(kFullMask, sc, 8));
  bm = fmaxf(bm, __shfl_xor_sync(kFullMask, bm, 16));
  if (__any_sync(kFullMask, bm > st.m_own)) {
#pragma unroll
    for (int j = 0; j < kG; ++j) {
      const float bj = __shfl_sync(kFullMask, bm, j * 2);
      const float mn = fmaxf(st.m4[j], bj);
      const float a = ex2_approx(st.m4[j] - mn);
      st.m4[j] = mn;
#pragma unroll
      for (int c = 0; c < 4; ++c) { st.acc2[j][c].x *= a; st.acc2[j][c].y *= a; }
      if (h_own == j) { st.l_part *= a; st.m_own = mn; }
    }
  }
  const float pw = ex2_approx(sc - st.m_own);
  st.l_part += pw;
  if ((lane & 1) == 0) pbuf[lane >> 1] = pw;  // [token][head]
  __syncwarp();
  // ---- weighted V rows
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    if (kMasked && r >= nvalid) break;
    const uint4 vr = *reinterpret_cast<const uint4*>(vt + r * kTokenBytes + lane * 16);
    const float4 pr = *reinterpret_cast<const float4*>(pbuf + r * 4);
    float2 v2[4];
    unpack8(vr, v2);
    const float ph[4] = {pr.x, pr.y, pr.z, pr.w};
#pragma unroll
    for (int h = 0; h < kG; ++h) {
      const float2 pp = make_float2(ph[h], ph[h]);
#pragma unroll
      for (int c = 0; c < 4; ++c) st.acc2[h][c] = fma2(pp, v2[c], st.acc2[h][c]);
    }
  }
}

// Loads the lane's slice of the row's query heads, pre-multiplied by
// scale * log2(e), into head slots (slot h <- head h ^ hperm).
__device__ __forceinline__ void load_query(const DecodeParams& p, int b, int kvh, int lane,
                                           WarpState& st) {
  const int hperm = (lane >> 1) & 3;
  const float c = p.scale * kLog2e;
  const long long qi = decode_query_index(p, b);
#pragma unroll
  for (int h = 0; h < kG; ++h) {
    const long long off = (qi * kHq + kvh * kG + (h ^ hperm)) * kD + lane * 8;
    if (p.q_dtype == NVJ_BF16) {
      const uint4 w = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(p.q) + off);
      unpack8(w, st.q2[h]);
    } else {
      const float4 a = *reinterpret_cast<const float4*>(static_cast<const float*>(p.q) + off);
      const float4 d = *reinterpret_cast<const float4*>(static_cast<const float*>(p.q) + off + 4);
      st.q2[h][0] = make_float2(a.x, a.y);
      st.q2[h][1] = make_float2(a.z, a.w);
      st.q2[h][2] = make_float2(d.x, d.y);
      st.q2[h][3] = make_float2(d.z, d.w);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) { st.q2[h][i].x *= c; st.q2[h][i].y *= c; }
  }
}

__device__ __forceinline__ void reset_state(WarpState& st) {
#pragma unroll
  for (int h = 0; h < kG; ++h) {
    st.m4[h] = kNegBig;
#pragma unroll
    for (int i = 0; i < 4; ++i) st.acc2[h][i] = make_float2(0.f, 0.f);
  }
  st.m_own = kNegBig;
  st.l_part = 0.f;
}

// One lane refills ring stage n % kStages with the K and V block of iteration n,
// after (wait_first) every warp has released the stage's previous occupant.
__device__ __forceinline__ void issue_block(const DecodeParams& p, DecodeSmem& sm, int n,
                                            bool wait_first) {
  const int stage = n % kStages;
  if (wait_first) {
    // previous occupant was iteration n - kStages; its release completes phase ((n / kStages) - 1) & 1
    if (!mbar_wait(smem_u32(&sm.empty_bar[stage]), (uint32_t)((n / kStages) - 1) & 1u, &sm.abort_flag, p.status))
      return;
  }
  const uint32_t full = smem_u32(&sm.full_bar[stage]);
  const long long blk = sm.ring_blk[n & (kRing - 1)];
  const int rows = sm.ring_rows[n & (kRing - 1)];
  if (rows > 0) {
    const uint32_t bytes = (uint32_t)rows * kTokenBytes;
    mbar_arrive_expect_tx(full, 2u * bytes);
    bulk_g2s(smem_u32(sm.tiles[stage][0]), p.k_cache + blk * kTileBytes, bytes, full);
    bulk_g2s(smem_u32(sm.tiles[stage][1]), p.v_cache + blk * kTileBytes, bytes, full);
  } else {
    mbar_arrive(full);
  }
}

// Merge the eight warp states of a finished segment and write either the final
// output row (the segment covered the whole row) or this CTA's partial; the CTA
// that delivers a row's last partial combines all of them.
__device__ __forceinline__ void finish_segment(const DecodeParams& p, DecodeSmem& sm, const Seg& s,
                                               WarpState& st, int warp, int lane, const Partition& pt) {
  const int kvh = warp & 1;
  const int tid = warp * 32 + lane;
  // per-head sum of weights: add the four token positions
  float lh = st.l_part;
  lh += __shfl_xor_sync(kFullMask, lh, 8);
  lh += __shfl_xor_sync(kFullMask, lh, 16);
  float l4[kG];
#pragma unroll
  for (int j = 0; j < kG; ++j) l4[j] = __shfl_sync(kFullMask, lh, j * 2);
  if (lane == 0) {
#pragma unroll
    for (int j = 0; j < kG; ++j) sm.ml[warp][j] = make_float2(st.m4[j], l4[j]);
  }
  named_bar_sync(1, kConsumerThreads);
  float f[kG];
#pragma unroll
  for (int j = 0; j < kG; ++j) {
    float M = kNegBig;
#pragma unroll
    for (int i = 0; i < kConsumerWarps / 2; ++i) M = fmaxf(M, sm.ml[kvh + 2 * i][j].x);
    float L = 0.f;
#pragma unroll
    for (int i = 0; i < kConsumerWarps / 2; ++i) {
      const float2 e = sm.ml[kvh + 2 * i][j];
      L += e.y * ex2_approx(e.x - M);
    }
    f[j] = ex2_approx(st.m4[j] - M);
    if (warp < 2 && lane == 0) sm.ML[kvh][j] = make_float2(M, L);
  }
  const bool whole_row = (s.j0 == 0 && s.j1 == s.nb);
  const long long out_row = decode_query_index(p, s.b);
  const int slot = partial_slot(blockIdx.x, s.j0 == 0);
  const int o_kvh = tid >> 7, o_d = (tid & 127) * 2;
#pragma unroll
  for (int j = 0; j < kG; ++j) {
    float4 a = make_float4(st.acc2[j][0].x * f[j], st.acc2[j][0].y * f[j], st.acc2[j][1].x * f[j], st.acc2[j][1].y * f[j]);
    float4 c = make_float4(st.acc2[j][2].x * f[j], st.acc2[j][2].y * f[j], st.acc2[j][3].x * f[j], st.acc2[j][3].y * f[j]);
    *reinterpret_cast<float4*>(&sm.merge[warp][lane * 8]) = a;
    *reinterpret_cast<float4*>(&sm.merge[warp][lane * 8 + 4]) = c;
    named_bar_sync(1, kConsumerThreads);
    float2 o = make_float2(0.f, 0.f);
#pragma unroll
    for (int i = 0; i < kConsumerWarps / 2; ++i) {
      const float2 x = *reinterpret_cast<const float2*>(&sm.merge[o_kvh + 2 * i][o_d]);
      o.x += x.x; o.y += x.y;
    }
    const int head = o_kvh * kG + j;
    const float2 MLv = sm.ML[o_kvh][j];
    if (whole_row) {
      const float inv = MLv.y > 0.f ? 1.f / MLv.y : 0.f;
      *reinterpret_cast<float2*>(p.out + (out_row * kHq + head) * kD + o_d) = make_float2(o.x * inv, o.y * inv);
    } else {
      *reinterpret_cast<float2*>(p.part_acc + ((long long)slot * kHq + head) * kD + o_d) = o;
      if (o_d == 0) *reinterpret_cast<float2*>(p.part_ml + ((long long)slot * kHq + head) * 2) = MLv;
    }
    named_bar_sync(1, kConsumerThreads);
  }
  if (whole_row) return;
  // ---- cross-CTA: count this partial in; the last arrival combines them.  One CTA can take in ~60 GB/s, and a
  // partial is 8 KiB (296 partials of one 32k-token row: 40 us for what took 10 us to stream), so a row cut
  // into more than kTreeMergeMin partials is folded in two levels: per group of kMergeGroup consecutive CTA ids by
  // the group's last arrival, then the group partials by the row's last group.  A group's CTAs lie inside at most
  // two such rows (one ending, one beginning in it: a row lying wholly inside has at most kMergeGroup partials),
  // which is why two counters and two partial slots per group are enough.
  const long long row_g0 = s.g0 - s.j0;
  const int c_lo = pt.cta_of(row_g0);
  const int c_hi = pt.cta_of(row_g0 + s.nb - 1);
  const int grid = gridDim.x;
  const bool tree = c_hi - c_lo + 1 > kTreeMergeMin;
  const int grp = blockIdx.x / kMergeGroup, g_lo = c_lo / kMergeGroup, g_hi = c_hi / kMergeGroup;
  const int first = tree ? max(c_lo, grp * kMergeGroup) : c_lo;
  const int last = tree ? min(c_hi, grp * kMergeGroup + kMergeGroup - 1) : c_hi;
  int32_t* counter = tree ? p.group_counters + 2 * grp + (grp == g_lo ? 1 : 0) : p.counters + s.b;
  __threadfence();
  named_bar_sync(1, kConsumerThreads);
  if (tid == 0) sm.is_last = (atomicAdd(counter, 1) == last - first) ? 1 : 0;
  named_bar_sync(1, kConsumerThreads);
  if (!sm.is_last) return;
  __threadfence();
  if (!tree) {
    fold_parts<true>(p, &sm.merge[0][0], tid, 0, c_lo, c_lo, c_hi - c_lo + 1, out_row * kHq);
    if (tid == 0) *counter = 0;
    return;
  }
  fold_parts<false>(p, &sm.merge[0][0], tid, 0, first, c_lo, last - first + 1, 2LL * grid + 2 * grp + (grp == g_lo ? 1 : 0));
  if (tid == 0) *counter = 0;
  __threadfence();
  named_bar_sync(1, kConsumerThreads);
  if (tid == 0) sm.is_last = (atomicAdd(p.counters + s.b, 1) == g_hi - g_lo) ? 1 : 0;
  named_bar_sync(1, kConsumerThreads);
  if (!sm.is_last) return;
  __threadfence();
  fold_parts<true>(p, &sm.merge[0][0], tid, 2LL * grid, g_lo, g_lo, g_hi - g_lo + 1, out_row * kHq);
  if (tid == 0) p.counters[s.b] = 0;
}

__global__ void __launch_bounds__(kDecodeThreads, 2) decode_pipelined_kernel(DecodeParams p) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  DecodeSmem& sm = *reinterpret_cast<DecodeSmem*>(smem_raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int grid = gridDim.x;

  // ---- pass 1: total number of blocks; zero the output of inactive rows
  int mine = 0;
  for (int base = 0; base < p.batch; base += kDecodeThreads) {
    const int b = base + threadIdx.x;
    int len = 0;
    if (b < p.batch) len = decode_row_len(p, b);
    mine += blocks_in_sequence(p, (len + kBlk - 1) / kBlk);
    // rows without keys get zeros; in a packed batch only the rows this pass owns (one query token) are touched
    const bool mine_to_zero = b < p.batch && len <= 0 && (b % grid) == (int)blockIdx.x &&
                              (!p.packed_rows || p.query_start_loc[b + 1] - p.query_start_loc[b] == 1);
    const unsigned idle = __ballot_sync(kFullMask, mine_to_zero);
    for (unsigned m = idle; m; m &= m - 1) {
      const int bb = base + (warp << 5) + (__ffs(m) - 1);
      float4* o = reinterpret_cast<float4*>(p.out + (p.packed_rows ? (long long)p.query_start_loc[bb] : (long long)bb) * kHq * kD);
      for (int i = lane; i < kHq * kD / 4; i += 32) o[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
  int total = 0;
  cta_inclusive_scan(mine, sm.scan, total);
  if (total == 0) return;
  const Partition pt = make_partition(total, grid);
  if ((int)blockIdx.x >= pt.n) return;
  const long long g0 = pt.start(blockIdx.x);
  const long long g1 = pt.start(blockIdx.x + 1);
  if (g0 == g1) return;

  // ---- pass 2: locate (row, block) of g0
  if (threadIdx.x == 0) { sm.start_b = p.batch; sm.start_j = 0; sm.abort_flag = 0; sm.is_last = 0; }
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
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&sm.full_bar[s]), 1);
      mbar_init(smem_u32(&sm.empty_bar[s]), kConsumerWarps);
    }
    mbar_fence_init();
  }
  __syncthreads();
  const int n_iters = blocks_in_range(p, sm.start_b, sm.start_j, g0, g1);  // the range's real blocks
  if (n_iters == 0) return;

  // ---- block-id look-ahead ring, first fill, first kStages copies
  FillState fs;
  fs.b = sm.start_b; fs.jn = sm.start_j; fs.g = g0; fs.j = 0; fs.nsegs = 0; fs.has = false;
  fill_ring(p, sm, fs, g1, 0, n_iters < kRing ? n_iters : kRing);
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int n = 0; n < kStages && n < n_iters; ++n) issue_block(p, sm, n, false);
  }

  int b = sm.start_b, j = sm.start_j;
  long long g = g0;
  Seg s;
  int it = 0;
  const int kvh = warp & 1, tok0 = (warp >> 1) * 4;
  WarpState st;
  while (next_seg(p, b, j, g, g1, s)) {
    load_query(p, s.b, kvh, lane, st);
    reset_state(st);
    // Fused append.  The CTA that owns block min(pos / 16, nb - 1) of the row writes the new
    // K/V row; inside it the two warps (one per KV head) that handle the row's token group
    // each store their 512-byte half.  The bulk copy of that block may race with the store,
    // so the same warps overwrite the row in the staged tile from registers once the copy
    // has landed: no fence is needed and nothing waits for the store.
    int patch_j = -1, patch_t = 0;
    if (p.new_k) {
      const int pos = p.pre_append ? p.seq_lens[s.b] : p.positions[s.b];
      const int jt = pos >> 4;
      const int jw = jt < s.nb - 1 ? jt : s.nb - 1;
      if (pos >= 0 && jw >= s.j0 && jw < s.j1 && (warp >> 1) == ((pos & 15) >> 2)) {
        const long long tgt = jt < p.table_width ? (long long)p.block_tables[decode_table_base(p, s.b) + jt] : -1;
        if (tgt >= 0 && tgt < p.num_blocks) {
          const long long src = (long long)s.b * kTokenBytes + kvh * kRowBytes + lane * 16;
          const uint4 new_k16 = *reinterpret_cast<const uint4*>(static_cast<const char*>(p.new_k) + src);
          const uint4 new_v16 = *reinterpret_cast<const uint4*>(static_cast<const char*>(p.new_v) + src);
          const long long dst = (tgt * kBlk + (pos & 15)) * kTokenBytes + kvh * kRowBytes + lane * 16;
          *reinterpret_cast<uint4*>(const_cast<char*>(p.k_cache) + dst) = new_k16;
          *reinterpret_cast<uint4*>(const_cast<char*>(p.v_cache) + dst) = new_v16;
          if (jt == jw && pos < s.len) { patch_j = jw; patch_t = pos & 3; }
        } else if (lane == 0) {
          atomicOr(p.status, NVJ_DEV_BAD_BLOCK_ID);
        }
      }
    }
    for (int jb = s.j0; jb < s.j1; ++jb, ++it) {
      if ((it & (kRing / 2 - 1)) == 0 && it > 0) {
        // every thread is done with ring entries below `it`: refill the half behind us
        named_bar_sync(1, kDecodeThreads);
        const int n0 = it + kRing / 2;
        if (n0 < n_iters) fill_ring(p, sm, fs, g1, n0, n_iters - n0 < kRing / 2 ? n_iters - n0 : kRing / 2);
        named_bar_sync(1, kDecodeThreads);
      }
      const int stage = it % kStages;
      mbar_wait(smem_u32(&sm.full_bar[stage]), (uint32_t)(it / kStages) & 1u, &sm.abort_flag, p.status);
      const int rows = sm.ring_rows[it & (kRing - 1)];
      char* kt = sm.tiles[stage][0] + tok0 * kTokenBytes + kvh * kRowBytes;
      char* vt = sm.tiles[stage][1] + tok0 * kTokenBytes + kvh * kRowBytes;
      if (jb == patch_j) {  // only this warp reads these two rows of the tile; the source is cache-hot
        const long long src = (long long)s.b * kTokenBytes + kvh * kRowBytes + lane * 16;
        *reinterpret_cast<uint4*>(kt + patch_t * kTokenBytes + lane * 16) =
            *reinterpret_cast<const uint4*>(static_cast<const char*>(p.new_k) + src);
        *reinterpret_cast<uint4*>(vt + patch_t * kTokenBytes + lane * 16) =
            *reinterpret_cast<const uint4*>(static_cast<const char*>(p.new_v) + src);
        __syncwarp();
      }
      float* pb = sm.pbuf[warp][it & 1];
      if (rows >= tok0 + 4) process_unit<false>(kt, vt, lane, 4, st, pb);
      else if (rows > tok0) process_unit<true>(kt, vt, lane, rows - tok0, st, pb);
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(smem_u32(&sm.empty_bar[stage]));
        // the warps take turns to refill the stage that iteration `it` just used
        if (warp == (it & (kConsumerWarps - 1)) && it + kStages < n_iters) issue_block(p, sm, it + kStages, true);
      }
      __syncwarp();  // lane 0 may have waited for the other warps; reconverge before any CTA barrier
    }
    finish_segment(p, sm, s, st, warp, lane, pt);
  }
  // Only after a timeout can copies still be in flight with nobody waiting for
  // them: hold the CTA's shared memory until they have landed.
  __syncthreads();
  if (threadIdx.x == 0 && sm.abort_flag) {
    const unsigned long long t0 = global_timer_ns();
    for (int back = 1; back <= kStages && back <= n_iters; ++back) {
      const int i = n_iters - back;
      while (!mbar_try_wait(smem_u32(&sm.full_bar[i % kStages]), (uint32_t)(i / kStages) & 1u) &&
             global_timer_ns() - t0 < kWaitLimitNs) {
      }
    }
  }
  __syncthreads();
}

static PerDeviceFlags g_num_ctas;  // 0 = not queried yet

int decode_num_ctas() {
  const int dev = current_device();
  if (dev < 0) return 0;
  int n = g_num_ctas.v[dev].load(std::memory_order_acquire);
  if (n == 0) {
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    // no more CTAs than the group counters of the workspace header cover
    n = 2 * sms < kMergeGroup * kGroupCounters / 2 ? 2 * sms : kMergeGroup * kGroupCounters / 2;
    g_num_ctas.v[dev].store(n, std::memory_order_release);
  }
  return n;
}

int launch_decode_pipelined(const DecodeParams& p, int num_ctas, cudaStream_t stream) {
  static_assert(sizeof(DecodeSmem) <= 113 * 1024, "two CTAs must fit one SM");
  static PerDeviceFlags smem_opted_in;
  if (!once_per_device(smem_opted_in, [](int) {
        return cudaFuncSetAttribute(decode_pipelined_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    (int)sizeof(DecodeSmem)) == cudaSuccess;
      }))
    return NVJ_ERR_LAUNCH;
  DecodeParams q = p;
  q.row_end_cost = kRowEndCost;
  decode_pipelined_kernel<<<num_ctas, kDecodeThreads, sizeof(DecodeSmem), stream>>>(q);
  return cudaGetLastError() == cudaSuccess ? NVJ_OK : NVJ_ERR_LAUNCH;
}

}  // namespace nvj
