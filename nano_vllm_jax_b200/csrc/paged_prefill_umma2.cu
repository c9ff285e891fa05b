// Ragged packed prefill attention on CTA pairs: the tcgen05 tile kernel with `cta_group::2`.
//
// The single-CTA kernel (paged_prefill_umma.cu) is bound by what one SM can take in from L2:
// every 64-key tile costs it 64 KiB for 128 query rows.  Here two CTAs of a cluster (the two
// SMs of a TPC) work on two neighbouring 32-token tiles of the same table row and KV head =
// 256 query rows, and every K/V tile is loaded once for the pair: CTA r keeps keys
// [32 r, 32 r + 32) of the K tile and head dims [128 r, 128 r + 128) of the V tile, 32 KiB per
// tile and SM instead of 64.  `tcgen05.mma.cta_group::2` (issued by CTA 0 alone) multiplies the
// 128 rows each CTA holds in its own tensor memory (Q, later P) with the B operand assembled
// from both halves, and leaves each CTA's 128 x N result in that CTA's tensor memory.
//   S:   M 256 (2 x 128), N 64 keys (2 x 32),  K 16 dims  x 16 per tile
//   P V: M 256,           N 256 dims (2 x 128), K 16 keys x 4 per tile, P as hi + lo
// Roles per CTA as in the single-CTA kernel (warp 0 TMA producer, warp 1 MMA issue in CTA 0,
// warps 2-9 softmax); what crosses the pair:
//   * both producers' TMA loads complete on CTA 0's full barriers (cp.async.bulk.tensor with
//     .cta_group::2 and the barrier address of rank 0); no load is a multicast;
//   * `tcgen05.commit` with a two-CTA mask releases K/V stages and S buffers in both CTAs;
//   * the softmax threads of both CTAs arrive on CTA 0's "Q staged" and "P written" barriers.
// A cluster barrier after set-up and one before the tensor memory is freed fence the pair.
// Every mbarrier wait is bounded; a timeout flags NVJ_DEV_TIMEOUT and both CTAs still reach
// the final cluster barrier and free their tensor memory.
// Short batches (a 512-token chunk is 16 CTA pairs on 74 pair slots) split every tile's key range over up to
// kU2MaxSplits pairs (blockIdx.z): each split writes its un-normalised rows and their (max, sum) to a workspace and
// is done; prefill_umma2_merge_kernel, launched behind this kernel, folds the splits of every tile into the output
// with the whole GPU (a first build let the pair that arrived last fold its tile alone: ~10 us of round trips to
// the L2 on two SMs, so that only key ranges of 16 tiles or more were worth splitting).
// Semantics: nanovllm_jax/kv_cache.py:831-849, nanovllm_jax/kernels/full_attention_triton.py:51-145.

#include <cstddef>

#include "paged_decode.cuh"
#include "umma.cuh"

namespace nvj {

constexpr int kU2Tokens = 32;    // query tokens per CTA (64 per pair)
constexpr int kU2Rows = 128;     // query rows per CTA
constexpr int kU2Keys = 64;      // keys per tile
constexpr int kU2Stages = 4;
constexpr int kU2Threads = 320;
constexpr int kU2SoftmaxThreads = 256;
constexpr int kU2TmemCols = 512;
constexpr int kU2ColQ = 0, kU2ColS = 128, kU2ColO = 256;
constexpr uint32_t kU2TileBytes = kU2Keys * kRowBytes;  // a whole K (or V) tile: both CTAs' halves, 32 KiB
constexpr uint32_t kU2LeaderMask = 0xFEFFFFFFu;         // clears the CTA-rank bit of a shared::cluster address
constexpr float kU2Log2e = 1.4426950408889634f;
constexpr float kU2RescaleGap = 8.f;
constexpr int kU2MaxSplits = 4;
// What a split costs: its rows go out to the workspace (~1 us) and the merge launch behind the kernel (~5 us for the
// batch, whatever the number of splits).  A key tile costs a pair ~1 us.  Key ranges of kU2SplitFrom tiles or more
// are split into pieces of at least kU2MinSplitTiles tiles.
constexpr int kU2SplitFrom = 8;
constexpr int kU2MinSplitTiles = 3;
constexpr int kU2MergeThreads = 256;
constexpr int kU2MergeParts = 8;  // CTAs of the merge launch per CTA tile: 4 of its 32 tokens each

// Development aid, compiled in only with -DNVJ_PHASE_TIMING: the first softmax thread of every CTA stamps the global
// timer at the kernel's phase boundaries (slot 7: the number of key tiles), nvj_debug_prefill_phase_ns copies them out.
#ifdef NVJ_PHASE_TIMING
__device__ unsigned long long g_u2_phase_ns[512][8];
#define NVJ_U2_PHASE(i) do { if (threadIdx.x == 64) g_u2_phase_ns[(blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x & 511][i] = global_timer_ns(); } while (0)
#define NVJ_U2_NOTE(i, v) do { if (threadIdx.x == 64) g_u2_phase_ns[(blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x & 511][i] = (v); } while (0)
#else
#define NVJ_U2_PHASE(i) do { } while (0)
#define NVJ_U2_NOTE(i, v) do { } while (0)
#endif

struct Umma2Params {
  const void* q;
  const int32_t* block_tables;
  const int32_t* kv_lens;
  const int32_t* positions;
  const int32_t* query_start_loc;
  float* out;
  int32_t* status;
  long long num_blocks;
  int rows, token_bucket, table_width, skip_single, q_dtype;
  int zero_fill;  // 1: the kernel itself zeroes what no tile writes (padding tokens, rows of several tokens without keys)
  int split_p;  // 1: P enters P V as two bf16 terms (hi + lo), 0: as one (the weights are then bf16-rounded)
  float scale;
  // key-range splits (gridDim.z > 1): un-normalised rows [split][token][head][kD], their (max, sum)
  // [split][token][head][2]; pair slots of the device
  float* part_o;
  float* part_ml;
  int4* tile_info;  // per (CTA of the x grid, KV head): {first token, tokens, splits, 0}, written by split 0 for the merge launch
  int pair_slots;
};

struct Umma2Smem {
  alignas(1024) char k[kU2Stages][4][32 * 128];  // [stage][64-d chunk][this CTA's 32 keys][128 B]
  alignas(1024) char v[kU2Stages][2][64 * 128];  // [stage][this CTA's two 64-d chunks][64 keys][128 B]
  // used in CTA 0 only: q_full, k_full, v_full, p_full; used in both: the rest
  alignas(8) unsigned long long q_full, k_full[kU2Stages], v_full[kU2Stages], k_empty[kU2Stages], v_empty[kU2Stages],
      s_full[2], p_full, pv_done, x_full;
  float xchg[2][2][kU2Rows];
  // this CTA's query rows on their way into tensor memory: [token][head of the group][32 pieces of 16 B], the pieces
  // of token t stored at (piece ^ (t & 7)) so that both the row-wise fill and the token-wise read are conflict-free
  alignas(16) char qstage[kU2Tokens * kG * kD * 2];
  float own_ml[2][kU2Rows];  // this split's (max, sum) per row, for the fold
  uint32_t tmem_base;
  int row, tok0, ntok, pair_last_tok, idle_index, abort_flag, total_pairs;
};

// ---- cta_group::2 wrappers ---------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem2_alloc(uint32_t smem_dst, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem2_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// D[256 x N] (+)= A[256 x 16] B[16 x N] over the CTA pair: each CTA's 128 rows of A and D in its own tensor
// memory at the same addresses, each CTA's N / 2 columns of B in its own shared memory at the same offsets
__device__ __forceinline__ void umma2_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
// arrives, once the MMAs issued so far have retired, on the barrier at this offset in both CTAs of the pair
__device__ __forceinline__ void umma2_commit_pair(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"((uint16_t)3) : "memory");
}
// One box into this CTA's shared memory; the bytes are counted on CTA 0's barrier at `bar`'s offset.
__device__ __forceinline__ void tma2_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(z), "r"(bar & kU2LeaderMask)
      : "memory");
}
__device__ __forceinline__ void mbar_arrive_leader(uint32_t bar) {
  // default semantics (release at CTA scope): what the arrival publishes lives in tensor memory and is ordered by
  // tcgen05.wait::st + tcgen05.fence; a cluster-scope release here cost ~1700 cycles per arrival
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar & kU2LeaderMask) : "memory");
}
// Instruction descriptor, kind::f16, fp32 accumulate, bf16 A and B, M = 256 over the pair.
__device__ __forceinline__ constexpr uint32_t umma2_idesc(int n, bool b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) | ((256u >> 4) << 24);
}

// ---- warp 0 of both CTAs: TMA loads of this CTA's halves ------------------------------------
__device__ __forceinline__ void u2_producer(const CUtensorMap* k_map, const CUtensorMap* v_map, const Umma2Params& p,
                                            Umma2Smem& sm, int row, int kvh, int kv_len, int tile0, int n_tiles, int rank,
                                            int lane, int first_ids) {
  const int need_blocks = (kv_len + kBlk - 1) / kBlk;
  const int oob = (int)(p.num_blocks * kBlk);  // a box that starts here is filled with zeros
  int ids = -1;
  for (int t = 0; t < n_tiles; ++t) {
    const int s = t % kU2Stages;
    const uint32_t reuse_parity = ((t / kU2Stages) - 1) & 1;
    if ((t & 7) == 0) {  // block ids of the next 8 tiles, one per lane
      const int bi = (tile0 + t) * 4 + lane;
      ids = -1;
      if (bi < need_blocks && bi < p.table_width) {
        ids = t == 0 ? first_ids : p.block_tables[(long long)row * p.table_width + bi];  // the first eight tiles' came early
        if (ids < 0 || ids >= p.num_blocks) {
          if (rank == 0) atomicOr(p.status, NVJ_DEV_BAD_BLOCK_ID);
          ids = -1;
        }
      }
    }
    int z[4];
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const int id = __shfl_sync(0xffffffffu, ids, (t & 7) * 4 + b);
      z[b] = id >= 0 ? id * kBlk : oob;
    }
    if (t >= kU2Stages && !um_wait(&sm.k_empty[s], reuse_parity, &sm.abort_flag, p.status)) break;
    if (lane == 0) {
      const uint32_t kb = smem_u32(&sm.k_full[s]);
      if (rank == 0) mbar_arrive_expect_tx(kb, kU2TileBytes);  // both CTAs' halves are counted here
#pragma unroll
      for (int b2 = 0; b2 < 2; ++b2)  // this CTA's keys: cache blocks 2 rank, 2 rank + 1 of the tile
#pragma unroll
        for (int c = 0; c < 4; ++c)
          tma2_load_3d(smem_u32(&sm.k[s][c][0]) + b2 * (kBlk * 128), k_map, c * 64, kvh, rank ? z[2 + b2] : z[b2], kb);
    }
    if (t >= kU2Stages && !um_wait(&sm.v_empty[s], reuse_parity, &sm.abort_flag, p.status)) break;
    if (lane == 0) {
      const uint32_t vb = smem_u32(&sm.v_full[s]);
      if (rank == 0) mbar_arrive_expect_tx(vb, kU2TileBytes);
#pragma unroll
      for (int b = 0; b < 4; ++b)  // all keys, this CTA's head dims: 64-d chunks 2 rank, 2 rank + 1
#pragma unroll
        for (int c2 = 0; c2 < 2; ++c2)
          tma2_load_3d(smem_u32(&sm.v[s][c2][0]) + b * (kBlk * 128), v_map, (2 * rank + c2) * 64, kvh, z[b], vb);
    }
    __syncwarp();
  }
}

// ---- warp 1 of CTA 0: MMA issue for the pair -------------------------------------------------
__device__ __forceinline__ bool u2_issue_s(Umma2Smem& sm, const Umma2Params& p, uint32_t tmem, uint64_t k_desc0, int t,
                                           int stage, uint32_t full_parity) {
  if (!um_wait(&sm.k_full[stage], full_parity, &sm.abort_flag, p.status)) return false;
  tc_fence_after_sync();
  if (um_elect_one()) {
    constexpr uint32_t idesc = umma2_idesc(kU2Keys, false);
    const uint64_t k_desc = k_desc0 + (uint64_t)((stage * 4 * 32 * 128) >> 4);
    const uint32_t d = tmem + kU2ColS + (t & 1) * kU2Keys;
#pragma unroll
    for (int ks = 0; ks < 16; ++ks)  // 16 dims per MMA: 8 columns of Q; K chunk ks / 4, 32 bytes into its swizzled rows
      umma2_bf16_ts(d, tmem + kU2ColQ + ks * 8, k_desc + (uint64_t)(((ks >> 2) * (32 * 128) + (ks & 3) * 32) >> 4), idesc,
                    ks > 0 ? 1u : 0u);
    umma2_commit_pair(smem_u32(&sm.s_full[t & 1]));
    umma2_commit_pair(smem_u32(&sm.k_empty[stage]));
  }
  __syncwarp();
  return true;
}

__device__ __forceinline__ void u2_mma_warp(Umma2Smem& sm, const Umma2Params& p, uint32_t tmem, int n_tiles) {
  const uint64_t k_desc0 = umma_desc(smem_u32(&sm.k[0][0][0]), 16, 1024);
  const uint64_t v_desc0 = umma_desc(smem_u32(&sm.v[0][0][0]), kU2Keys * 128, 1024);
  if (!um_wait(&sm.q_full, 0, &sm.abort_flag, p.status)) return;
  if (!u2_issue_s(sm, p, tmem, k_desc0, 0, 0, 0)) return;
  if (n_tiles > 1 && !u2_issue_s(sm, p, tmem, k_desc0, 1, 1, 0)) return;
  int sv = 0, sk = 2 % kU2Stages;
  uint32_t pv = 0, pk = 2 / kU2Stages;
  for (int t = 0; t < n_tiles; ++t) {
    if (!um_wait(&sm.v_full[sv], pv, &sm.abort_flag, p.status)) return;
    if (!um_wait(&sm.p_full, t & 1, &sm.abort_flag, p.status)) return;
    tc_fence_after_sync();
    if (um_elect_one()) {
      constexpr uint32_t idesc = umma2_idesc(kD, true);
      const uint64_t v_desc = v_desc0 + (uint64_t)((sv * 2 * kU2Keys * 128) >> 4);
      const uint32_t pa = tmem + kU2ColS + (t & 1) * kU2Keys;
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {  // 16 keys per MMA: 8 columns of P, two 8-key groups of V
        const uint64_t dv = v_desc + (uint64_t)((kk * 2048) >> 4);
        umma2_bf16_ts(tmem + kU2ColO, pa + kk * 8, dv, idesc, (t > 0 || kk > 0) ? 1u : 0u);
        if (p.split_p) umma2_bf16_ts(tmem + kU2ColO, pa + 32 + kk * 8, dv, idesc, 1u);
      }
      umma2_commit_pair(smem_u32(&sm.v_empty[sv]));
      umma2_commit_pair(smem_u32(&sm.pv_done));
    }
    __syncwarp();
    // S(t + 2) overwrites the columns P V (t) reads P(t) from; MMAs of different shapes are not
    // ordered against each other, so wait for P V (t) to retire first
    if (t + 2 < n_tiles) {
      if (!um_wait(&sm.pv_done, t & 1, &sm.abort_flag, p.status)) return;
      if (!u2_issue_s(sm, p, tmem, k_desc0, t + 2, sk, pk)) return;
    }
    if (++sv == kU2Stages) { sv = 0; pv ^= 1u; }
    if (++sk == kU2Stages) { sk = 0; pk ^= 1u; }
  }
}

// The walk over the key tiles for one softmax thread (row r, column half): scores out of tensor memory, mask, running
// max shared with the other half, weights back into tensor memory.  False when a wait ran out (the caller still
// joins its barriers).
__device__ __forceinline__ bool u2_softmax_tiles(Umma2Smem& sm, const Umma2Params& p, uint32_t my_tmem, int tok0, int ntok,
                                                 int kv_len, int tile0, int n_tiles, int half, int r, int token, float& m_row,
                                                 float& l_row) {
  const int my_pos = token < ntok ? p.positions[tok0 + token] : -1;
  const int last_key = my_pos < kv_len - 1 ? my_pos : kv_len - 1;
  const float scale_log2 = p.scale * kU2Log2e;
  for (int t = 0; t < n_tiles; ++t) {
    const int b = t & 1;
    const uint32_t s_tmem = my_tmem + kU2ColS + b * kU2Keys;
    if (!um_wait(&sm.s_full[b], (t >> 1) & 1, &sm.abort_flag, p.status)) return false;
    if (t == 0) NVJ_U2_PHASE(3);
    tc_fence_after_sync();
    float s[32];
    tmem_ld32(s_tmem + half * 32, s);
    const int lim = last_key - (tile0 + t) * kU2Keys - half * 32;
    float hmax = -INFINITY;
    if (lim >= 31) {
#pragma unroll
      for (int i = 0; i < 32; i += 2) hmax = fmaxf(hmax, fmaxf(s[i], s[i + 1]));
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) { s[i] = i <= lim ? s[i] : -INFINITY; hmax = fmaxf(hmax, s[i]); }
    }
    sm.xchg[b][half][r] = hmax;
    mbar_arrive(smem_u32(&sm.x_full));
    if (!um_wait(&sm.x_full, t & 1, &sm.abort_flag, p.status)) return false;
    const float tmax = fmaxf(hmax, sm.xchg[b][half ^ 1][r]) * scale_log2;  // scale > 0
    if (t == 0) {
      m_row = tmax;
    } else if (__any_sync(0xffffffffu, tmax > m_row + kU2RescaleGap)) {
      if (!um_wait(&sm.pv_done, (t - 1) & 1, &sm.abort_flag, p.status)) return false;
      tc_fence_after_sync();
      const float m_new = fmaxf(m_row, tmax);
      const float f = m_new == -INFINITY ? 1.f : ex2_approx(m_row - m_new);
      m_row = m_new;
      l_row *= f;
#pragma unroll 1
      for (int cc = 0; cc < kD / 64; ++cc) {
        float o[32];
        tmem_ld32(my_tmem + kU2ColO + half * (kD / 2) + cc * 32, o);
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] *= f;
        tmem_st32(my_tmem + kU2ColO + half * (kD / 2) + cc * 32, o);
      }
    }
    const float neg_m = m_row == -INFINITY ? 0.f : -m_row;
    uint32_t hi[16], lo[16];
#pragma unroll
    for (int e = 0; e < 16; ++e) {
      const float p0 = ex2_approx(fmaf(s[2 * e], scale_log2, neg_m)), p1 = ex2_approx(fmaf(s[2 * e + 1], scale_log2, neg_m));
      l_row += p0 + p1;
      const __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
      const __nv_bfloat162 g = __floats2bfloat162_rn(p0 - __low2float(h), p1 - __high2float(h));
      hi[e] = *reinterpret_cast<const uint32_t*>(&h);
      lo[e] = *reinterpret_cast<const uint32_t*>(&g);
    }
    // every phase of pv_done is observed in turn (parity waits tell only two phases apart)
    if (t >= 1 && !um_wait(&sm.pv_done, (t - 1) & 1, &sm.abort_flag, p.status)) return false;
    tmem_st16(s_tmem + half * 16, hi);
    if (p.split_p) tmem_st16(s_tmem + 32 + half * 16, lo);
    tmem_st_wait();
    tc_fence_before_sync();
    mbar_arrive_leader(smem_u32(&sm.p_full));
  }
  return true;
}

// The tile's query rows, 2 KiB per token (the group's four heads lie side by side), as whole 512-byte rows per warp
// instruction, all sixteen loads of a thread in flight at once: softmax warp sw takes tokens 4 sw .. 4 sw + 3.
__device__ __forceinline__ void u2_request_q(const Umma2Params& p, int tok0, int ntok, int kvh, int warp, int lane, uint4 (&u)[4][4]) {
  const int sw = (warp - 2) & 7;
#pragma unroll
  for (int a = 0; a < 4; ++a) {
    const int tk = sw * 4 + a;
    const uint4* src = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(p.q) +
                                                      ((long long)(tok0 + tk) * kHq + kvh * kG) * kD) + lane;
#pragma unroll
    for (int h = 0; h < 4; ++h) u[a][h] = tk < ntok ? ld_nc_u4(src + h * 32) : make_uint4(0u, 0u, 0u, 0u);
  }
}

// ---- warps 2-9 of both CTAs: Q staging, softmax, epilogue for this CTA's 128 rows -------------
__device__ __forceinline__ void u2_softmax_warps(Umma2Smem& sm, const Umma2Params& p, uint32_t tmem, int tok0, int ntok,
                                                 int kvh, int kv_len, int tile0, int n_tiles, int splits, int warp, int lane,
                                                 const uint4 (&u)[4][4]) {
  const int quarter = warp & 3, half = (warp - 2) >> 2;
  const int r = quarter * 32 + lane, token = lane, hl = quarter;
  const uint32_t my_tmem = tmem + ((uint32_t)(quarter * 32) << 16);
  if (p.q_dtype == NVJ_BF16) {
    // The tile's query rows (`u`, requested by u2_request_q before the pair was set up) go through shared memory: a
    // thread that fetched its own row directly would touch 32 lines per instruction and wait for memory four times
    // in a row (4.4 us of a 30 us kernel on a 512-token chunk).
    const int sw = (warp - 2) & 7;  // 0..7: four tokens each
#pragma unroll
    for (int a = 0; a < 4; ++a) {
      const int tk = sw * 4 + a;
#pragma unroll
      for (int h = 0; h < 4; ++h)
        *reinterpret_cast<uint4*>(sm.qstage + tk * 2048 + h * 512 + ((lane ^ (tk & 7)) << 4)) = u[a][h];
    }
    named_bar_sync(1, kU2SoftmaxThreads);
    // this row's half of Q (128 dims) -> 64 TMEM columns, two bf16 per column
    const char* mine = sm.qstage + token * 2048 + hl * 512;
#pragma unroll 1
    for (int part = 0; part < 4; ++part) {
      uint32_t w[16];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint4 x = *reinterpret_cast<const uint4*>(mine + (((half * 16 + part * 4 + i) ^ (token & 7)) << 4));
        w[4 * i] = x.x; w[4 * i + 1] = x.y; w[4 * i + 2] = x.z; w[4 * i + 3] = x.w;
      }
      tmem_st16(my_tmem + kU2ColQ + half * 64 + part * 16, w);
    }
    tmem_st_wait();
    tc_fence_before_sync();
    mbar_arrive_leader(smem_u32(&sm.q_full));
    NVJ_U2_PHASE(2);
  } else {  // fp32 queries: every thread converts its own row
    const long long qrow = ((long long)(tok0 + token) * kHq + kvh * kG + hl) * kD + half * (kD / 2);
#pragma unroll 1
    for (int part = 0; part < 4; ++part) {
      uint32_t w[16];
      if (token >= ntok) {
#pragma unroll
        for (int i = 0; i < 16; ++i) w[i] = 0u;
      } else {
        const float4* src = reinterpret_cast<const float4*>(static_cast<const float*>(p.q) + qrow + part * 32);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float4 f = src[i];
          const __nv_bfloat162 a = __floats2bfloat162_rn(f.x, f.y), b2 = __floats2bfloat162_rn(f.z, f.w);
          w[2 * i] = *reinterpret_cast<const uint32_t*>(&a);
          w[2 * i + 1] = *reinterpret_cast<const uint32_t*>(&b2);
        }
      }
      tmem_st16(my_tmem + kU2ColQ + half * 64 + part * 16, w);
    }
    tmem_st_wait();
    tc_fence_before_sync();
    mbar_arrive_leader(smem_u32(&sm.q_full));
    NVJ_U2_PHASE(2);
  }
  float m_row = -INFINITY, l_row = 0.f;
  bool alive = u2_softmax_tiles(sm, p, my_tmem, tok0, ntok, kv_len, tile0, n_tiles, half, r, token, m_row, l_row);
  // ---- epilogue.  From here on the softmax threads meet at CTA-wide named barriers, so a thread whose wait ran out
  // does not leave: it skips the work and everybody returns together once the barrier has made the flag visible.
  NVJ_U2_PHASE(4);
  if (alive) {
    sm.xchg[n_tiles & 1][half][r] = l_row;
    mbar_arrive(smem_u32(&sm.x_full));
    alive = um_wait(&sm.x_full, n_tiles & 1, &sm.abort_flag, p.status);
  }
  if (alive) {
    l_row += sm.xchg[n_tiles & 1][half ^ 1][r];
    alive = um_wait(&sm.pv_done, (n_tiles - 1) & 1, &sm.abort_flag, p.status);
  }
  tc_fence_after_sync();
  const float inv = splits > 1 ? 1.f : (l_row > 0.f ? 1.f / l_row : 0.f);  // a split leaves its rows un-normalised
  if (splits > 1 && half == 0) { sm.own_ml[0][r] = m_row; sm.own_ml[1][r] = l_row; }
  // The K and V stages (128 KiB, contiguous) are free now: every copy has landed and every product has retired.  The
  // normalised rows are laid down there, [row][256 floats] with the 16-byte pieces of row r stored at (piece ^ (r & 7))
  // inside their group of eight, and leave as whole 512-byte runs per warp instruction.  (Stored straight from the
  // registers, a warp instruction touched 32 lines: 5.4 us of a 30 us kernel on a 512-token chunk.)
  float* stage = reinterpret_cast<float*>(&sm.k[0][0][0]);
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the stages were last written by bulk copies
  static_assert(sizeof(sm.k) + sizeof(sm.v) >= (size_t)kU2Rows * kD * sizeof(float) && offsetof(Umma2Smem, v) == sizeof(sm.k),
                "the output tile is staged across the K and V stages");
#pragma unroll 1
  for (int cc = 0; cc < kD / 64 && alive; ++cc) {
    float o[32];
    tmem_ld32(my_tmem + kU2ColO + half * (kD / 2) + cc * 32, o);
    const int c0 = (half * (kD / 2) + cc * 32) >> 2;  // first 16-byte piece of these 32 floats within the row
#pragma unroll
    for (int i = 0; i < 8; ++i)
      *reinterpret_cast<float4*>(stage + r * kD + ((c0 + (i ^ (r & 7))) << 2)) =
          make_float4(o[4 * i] * inv, o[4 * i + 1] * inv, o[4 * i + 2] * inv, o[4 * i + 3] * inv);
  }
  named_bar_sync(1, kU2SoftmaxThreads);
  if (*reinterpret_cast<volatile int*>(&sm.abort_flag)) return;  // somebody gave up: the same answer in every thread
  const int sw = (warp - 2) & 7;
  const long long split_rows = (long long)p.token_bucket * kHq;  // rows of one split's partial area
  {
    float* base = splits > 1 ? p.part_o + (long long)blockIdx.z * split_rows * kD : p.out;
#pragma unroll 4
    for (int a = 0; a < kU2Rows / 8; ++a) {
      const int rr = sw * (kU2Rows / 8) + a, tk = rr & 31, hd = rr >> 5;
      if (tk >= ntok) continue;
      const long long g = (long long)(tok0 + tk) * kHq + kvh * kG + hd;
#pragma unroll
      for (int h2 = 0; h2 < 2; ++h2) {
        const int c = h2 * 32 + lane;
        reinterpret_cast<float4*>(base + g * kD)[c] = *reinterpret_cast<const float4*>(stage + rr * kD + (((c & ~7) | ((c ^ rr) & 7)) << 2));
      }
      if (splits > 1 && lane == 0)
        *reinterpret_cast<float2*>(p.part_ml + ((long long)blockIdx.z * split_rows + g) * 2) = make_float2(sm.own_ml[0][rr], sm.own_ml[1][rr]);
    }
  }
  NVJ_U2_PHASE(5);  // a split is done here: the merge launch folds the splits
}

// Which (table row, 32-token tile) the CTA with cluster index `cluster` of `clusters` and rank `rank` serves: the
// heaviest pairs (the last tokens of a row see the most keys) get the lowest cluster indices.  One thread runs this.
// row < 0: no tile (`idle` then numbers the clusters beyond the last pair 0, 1, ...).  `total` (the batch's number
// of pairs) is complete only when `need_total`.
struct U2Tile {
  int row, tok0, ntok, pair_last_tok, idle, total;
};
__device__ __forceinline__ U2Tile u2_find_tile(const Umma2Params& p, int cluster, int clusters, int rank, bool need_total) {
  U2Tile t{-1, 0, 0, 0, -1, 0};
  int idx = clusters - 1 - cluster;
  for (int r = 0; r < p.rows; ++r) {
    const int lo = p.query_start_loc[r];
    int hi = p.query_start_loc[r + 1];
    hi = hi < p.token_bucket ? hi : p.token_bucket;
    int pairs = hi > lo ? (hi - lo + 2 * kU2Tokens - 1) / (2 * kU2Tokens) : 0;
    if (p.skip_single && p.query_start_loc[r + 1] - lo == 1) pairs = 0;
    t.total += pairs;
    if (t.row < 0 && idx < pairs) {
      t.row = r;
      t.tok0 = lo + (2 * idx + rank) * kU2Tokens;
      t.ntok = hi - t.tok0 < kU2Tokens ? hi - t.tok0 : kU2Tokens;
      if (t.ntok < 0) t.ntok = 0;
      const int pair_end = lo + (2 * idx + 2) * kU2Tokens;
      t.pair_last_tok = (pair_end < hi ? pair_end : hi) - 1;
      if (!need_total) break;
    }
    if (t.row < 0) idx -= pairs;
  }
  if (t.row < 0) t.idle = idx;
  return t;
}
// Key tiles of the pair (warp-collective; the same in every warp of both CTAs): the token of the pair that sees the most
// keys bounds the key range (positions need not grow along the tiles).  `kv_len` comes back clipped to the table.
__device__ __forceinline__ int u2_key_tiles(const Umma2Params& p, int row, int tok0, int rank, int pair_last_tok, int lane,
                                            int& kv_len, bool flag) {
  kv_len = p.kv_lens[row];
  if (kv_len > p.table_width * kBlk) {
    if (flag) atomicOr(p.status, NVJ_DEV_BAD_LENGTH);
    kv_len = p.table_width * kBlk;
  }
  const int pair_tok0 = tok0 - rank * kU2Tokens, pair_n = pair_last_tok - pair_tok0 + 1;
  int seen = lane < pair_n ? p.positions[pair_tok0 + lane] : -1;
  if (lane + 32 < pair_n) seen = max(seen, p.positions[pair_tok0 + lane + 32]);
  const int max_pos = __reduce_max_sync(0xffffffffu, seen);
  const int key_end = kv_len < max_pos + 1 ? kv_len : max_pos + 1;
  return key_end > 0 ? (key_end + kU2Keys - 1) / kU2Keys : 0;
}
// Key-range splits of a pair: as many as leave every split kU2MinSplitTiles tiles, as the batch's pairs leave pair
// slots for, and as the launch has.
__device__ __forceinline__ int u2_split_count(const Umma2Params& p, int n_tiles, int total_pairs, int launched) {
  const int room = p.pair_slots / (total_pairs * kHkv > 0 ? total_pairs * kHkv : 1);
  int splits = n_tiles >= kU2SplitFrom ? n_tiles / kU2MinSplitTiles : 1;
  splits = splits < room ? splits : room;
  splits = splits < launched ? splits : launched;
  return splits > 1 ? splits : 1;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kU2Threads, 1)
prefill_umma2_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
                     const Umma2Params p) {
  extern __shared__ unsigned char u2_smem_raw[];
  Umma2Smem& sm = *reinterpret_cast<Umma2Smem*>((reinterpret_cast<uintptr_t>(u2_smem_raw) + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kvh = blockIdx.y;
  const int rank = (int)cluster_ctarank();  // == blockIdx.x & 1
  NVJ_U2_PHASE(0);
  NVJ_U2_NOTE(7, 0ull);
  // a merge launch follows a launch with splits: let its CTAs take their places now (they wait for this grid to finish)
  if (gridDim.z > 1) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (blockIdx.z > 0) {  // the extra splits leave at once when no row's key range is long enough to be split
    int any = 0;
    for (int rr = threadIdx.x; rr < p.rows; rr += kU2Threads) any |= p.kv_lens[rr] > (kU2SplitFrom - 1) * kU2Keys ? 1 : 0;
    if (!__syncthreads_or(any)) return;
  }

  // ---- which (table row, pair of 32-token tiles) this cluster serves; both CTAs compute the same
  if (threadIdx.x == 0) {
    const U2Tile t = u2_find_tile(p, blockIdx.x >> 1, gridDim.x >> 1, rank, gridDim.z > 1);
    sm.row = t.row; sm.tok0 = t.tok0; sm.ntok = t.ntok; sm.pair_last_tok = t.pair_last_tok; sm.abort_flag = 0;
    sm.total_pairs = t.total; sm.idle_index = t.idle;
  }
  __syncthreads();
  const int row = sm.row, tok0 = sm.tok0, ntok = sm.ntok;
  int4* info = gridDim.z > 1 && blockIdx.z == 0 && threadIdx.x == 0 ? p.tile_info + blockIdx.x * kHkv + kvh : nullptr;
  if (row < 0) {  // the whole cluster leaves: nothing has been allocated or shared yet
    if (info) *info = make_int4(0, 0, 0, 0);
    if (p.zero_fill && sm.idle_index == 0 && blockIdx.z == 0) {
      // the first idle cluster (there is always one) zeroes the padding tokens, a quarter per CTA of the cluster pair x KV head
      int real = p.query_start_loc[p.rows];
      real = real < p.token_bucket ? real : p.token_bucket;
      const long long n4 = (long long)(p.token_bucket - real) * kHq * kD / 4;
      float4* pad = reinterpret_cast<float4*>(p.out + (long long)real * kHq * kD);
      const int part = rank * kHkv + kvh;
      for (long long i = (long long)part * kU2Threads + threadIdx.x; i < n4; i += 2LL * kHkv * kU2Threads)
        pad[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    return;
  }

  int kv_len;
  const int n_tiles = u2_key_tiles(p, row, tok0, rank, sm.pair_last_tok, lane, kv_len, threadIdx.x == 0 && rank == 0);
  if (n_tiles == 0) {  // same decision in both CTAs; a row without keys produces zeros
    if (info) *info = make_int4(tok0, ntok, 0, 0);
    if (p.zero_fill && blockIdx.z == 0) {
      for (int i = threadIdx.x; i < ntok * kG * (kD / 4); i += kU2Threads) {
        const int t = i / (kG * (kD / 4)), rest = i - t * (kG * (kD / 4));
        reinterpret_cast<float4*>(p.out + ((long long)(tok0 + t) * kHq + kvh * kG) * kD)[rest] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
    return;
  }

  // Key-range splits of this pair: as many as leave every split kU2MinSplitTiles tiles and as the batch's pairs
  // leave pair slots for; the splits beyond that leave at once (both CTAs decide alike).
  int splits = 1, tile0 = 0, my_tiles = n_tiles;
  if (gridDim.z > 1) {
    splits = u2_split_count(p, n_tiles, sm.total_pairs, (int)gridDim.z);
    if (info) *info = make_int4(tok0, ntok, splits, 0);
    if ((int)blockIdx.z >= splits) return;
    tile0 = (int)blockIdx.z * n_tiles / splits;
    my_tiles = ((int)blockIdx.z + 1) * n_tiles / splits - tile0;
  }

  // the query rows, and the block ids of the producer's first eight tiles, are asked for now and arrive while the
  // pair is being set up
  uint4 qv[4][4];
  if (warp >= 2 && p.q_dtype == NVJ_BF16) u2_request_q(p, tok0, ntok, kvh, warp, lane, qv);
  int first_ids = -1;
  if (warp == 0) {
    const int bi = tile0 * 4 + lane;
    if (bi < (kv_len + kBlk - 1) / kBlk && bi < p.table_width) first_ids = p.block_tables[(long long)row * p.table_width + bi];
  }

  if (warp == 1) tmem2_alloc(smem_u32(&sm.tmem_base), kU2TmemCols);
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&sm.q_full), 2 * kU2SoftmaxThreads);
    for (int i = 0; i < kU2Stages; ++i) {
      mbar_init(smem_u32(&sm.k_full[i]), 1);
      mbar_init(smem_u32(&sm.v_full[i]), 1);
      mbar_init(smem_u32(&sm.k_empty[i]), 1);
      mbar_init(smem_u32(&sm.v_empty[i]), 1);
    }
    mbar_init(smem_u32(&sm.s_full[0]), 1);
    mbar_init(smem_u32(&sm.s_full[1]), 1);
    mbar_init(smem_u32(&sm.p_full), 2 * kU2SoftmaxThreads);
    mbar_init(smem_u32(&sm.pv_done), 1);
    mbar_init(smem_u32(&sm.x_full), kU2SoftmaxThreads);
    mbar_fence_init();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers exist before anything is sent to them
  tc_fence_after_sync();
  const uint32_t tmem = sm.tmem_base;
  NVJ_U2_PHASE(1);
  NVJ_U2_NOTE(7, (unsigned long long)my_tiles);

  if (warp == 0) u2_producer(&k_map, &v_map, p, sm, row, kvh, kv_len, tile0, my_tiles, rank, lane, first_ids);
  else if (warp == 1) { if (rank == 0) u2_mma_warp(sm, p, tmem, my_tiles); }
  else u2_softmax_warps(sm, p, tmem, tok0, ntok, kvh, kv_len, tile0, my_tiles, splits, warp, lane, qv);

  tc_fence_before_sync();
  __syncthreads();
  if (sm.abort_flag) {  // give copies and MMAs in flight time to land before memory is released
    const unsigned long long t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  cluster_sync_all();  // CTA 0's MMAs read this CTA's shared and tensor memory until its last commit
  NVJ_U2_PHASE(6);
  if (warp == 1) tmem2_dealloc(tmem, kU2TmemCols);
}

// Behind prefill_umma2_kernel in stream order (no counters, no fences): folds the key-range splits of every tile into the
// output.  Grid = the tile kernel's (x, y) with kU2MergeParts CTAs per CTA tile (4 of its 32 tokens each).  Split 0 of
// every tile left {first token, tokens, splits} in the workspace, so a CTA is two trips to memory: that record, then
// every split's (max, sum) and both 16-byte pieces per lane of its rows, all requested before anything is used.  (A
// build that found its tile and its splits again from the batch's metadata took 8.8 us: five trips.)
// Warp w folds token 4 part + w / 2, heads 2 (w & 1) and 2 (w & 1) + 1 of the group.
static_assert(kU2MaxSplits == 4 && kU2Tokens % kU2MergeParts == 0 && kU2MergeThreads == 64 * (kU2Tokens / kU2MergeParts),
              "the merge launch maps a warp to (token, two heads) and reduces over four lanes");
__global__ void __launch_bounds__(kU2MergeThreads)
prefill_umma2_merge_kernel(const Umma2Params p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kvh = blockIdx.y, part = blockIdx.z;
  // launched with programmatic stream serialization: the CTAs may be resident before the tile kernel has finished, and
  // wait here until all of it has completed and its writes are visible
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int4 info = __ldcg(p.tile_info + blockIdx.x * kHkv + kvh);
  const int tok0 = info.x, ntok = info.y, splits = info.z;
  if (splits <= 1) return;
  const int tk = part * (kU2Tokens / kU2MergeParts) + (warp >> 1);
  if (tk >= ntok) return;
  const long long split_rows = (long long)p.token_bucket * kHq;
  float2 e[2];
  float4 x[2][kU2MaxSplits][2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const long long g = (long long)(tok0 + tk) * kHq + kvh * kG + (warp & 1) * 2 + h;
    e[h] = make_float2(-INFINITY, 0.f);  // lane s2 < splits: that split's (max, sum) of the row
    if (lane < splits) e[h] = __ldcg(reinterpret_cast<const float2*>(p.part_ml + ((long long)lane * split_rows + g) * 2));
#pragma unroll
    for (int s2 = 0; s2 < kU2MaxSplits; ++s2) {
      const float4* src = reinterpret_cast<const float4*>(p.part_o + ((long long)s2 * split_rows + g) * kD);
      x[h][s2][0] = s2 < splits ? __ldcg(src + lane) : make_float4(0.f, 0.f, 0.f, 0.f);
      x[h][s2][1] = s2 < splits ? __ldcg(src + 32 + lane) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const long long g = (long long)(tok0 + tk) * kHq + kvh * kG + (warp & 1) * 2 + h;
    float big = e[h].x;
#pragma unroll
    for (int o = 1; o < kU2MaxSplits; o <<= 1) big = fmaxf(big, __shfl_xor_sync(0xffffffffu, big, o));
    float w = e[h].x == -INFINITY ? 0.f : ex2_approx(e[h].x - big);
    float total = w * e[h].y;
#pragma unroll
    for (int o = 1; o < kU2MaxSplits; o <<= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
    w = total > 0.f ? w / total : 0.f;  // lanes 0 .. kU2MaxSplits - 1 hold their split's normalised weight
    float4 acc[2] = {make_float4(0.f, 0.f, 0.f, 0.f), make_float4(0.f, 0.f, 0.f, 0.f)};
#pragma unroll
    for (int s2 = 0; s2 < kU2MaxSplits; ++s2) {
      const float ws = __shfl_sync(0xffffffffu, w, s2);
#pragma unroll
      for (int h2 = 0; h2 < 2; ++h2) {
        acc[h2].x = fmaf(x[h][s2][h2].x, ws, acc[h2].x); acc[h2].y = fmaf(x[h][s2][h2].y, ws, acc[h2].y);
        acc[h2].z = fmaf(x[h][s2][h2].z, ws, acc[h2].z); acc[h2].w = fmaf(x[h][s2][h2].w, ws, acc[h2].w);
      }
    }
    float4* dst = reinterpret_cast<float4*>(p.out + g * kD);
    dst[lane] = acc[0];
    dst[32 + lane] = acc[1];
  }
}

typedef CUresult (*U2EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static U2EncodeTiledFn u2_encode_fn() {
  static U2EncodeTiledFn fn = [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult res;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &res) != cudaSuccess ||
        res != cudaDriverEntryPointSuccess)
      ptr = nullptr;
    return reinterpret_cast<U2EncodeTiledFn>(ptr);
  }();
  return fn;
}

static int u2_pair_slots() {  // CTA pairs that run at once: half the SMs of the current device
  static PerDeviceFlags slots;
  const int dev = current_device();
  if (dev < 0) return 0;
  int n = slots.v[dev].load(std::memory_order_acquire);
  if (n == 0) {
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    n = sms / 2;
    slots.v[dev].store(n, std::memory_order_release);
  }
  return n;
}

// Room for the un-normalised rows and (max, sum) pairs of the splits of the largest batch that is split at all:
// splits x tokens never exceeds the pair slots x 64 tokens (plus one pair per split of rounding).
size_t prefill_split_bytes() {
  const int slots = u2_pair_slots();
  const size_t tokens = (size_t)(slots > 0 ? slots : 74) * 2 * kU2Tokens / kHkv + (size_t)kU2MaxSplits * 2 * kU2Tokens;
  return ws_round(sizeof(float) * tokens * kHq * (kD + 2)) + ws_round(sizeof(int4) * 2 * (tokens / (2 * kU2Tokens) + 4096) * kHkv);
}

static bool u2_make_map(CUtensorMap* map, const void* base, uint64_t outer) {
  const cuuint64_t dims[3] = {(cuuint64_t)kD, (cuuint64_t)kHkv, outer};
  const cuuint64_t strides[2] = {(cuuint64_t)kRowBytes, (cuuint64_t)kRowBytes * kHkv};
  const cuuint32_t box[3] = {64, 1, (cuuint32_t)kBlk};
  const cuuint32_t estr[3] = {1, 1, 1};
  return u2_encode_fn()(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Whether launch_prefill_umma2 will take a batch with these parameters (a caller that knows so need not zero the output).
bool prefill_umma2_usable(float scale, long long num_blocks) { return scale > 0.f && num_blocks >= 1 && u2_encode_fn() != nullptr; }

// Returns NVJ_ERR_UNSUPPORTED when the driver offers no tensor-map encoder or the scale is not positive.
int launch_prefill_umma2(const void* q, int q_dtype, const char* k_cache, const char* v_cache,
                         long long num_blocks, const int32_t* block_tables, int table_width,
                         const int32_t* kv_lens, const int32_t* positions, const int32_t* query_start_loc,
                         int rows, int token_bucket, float scale, float* out, int32_t* status,
                         int skip_single, int split_p, float* split_area, size_t split_bytes, cudaStream_t stream) {
  static PerDeviceFlags opted_in;
  constexpr int kSmemBytes = (int)sizeof(Umma2Smem) + 1024;
  static_assert(kSmemBytes <= 232448, "tiles exceed the shared memory of one CTA");
  if (!(scale > 0.f) || num_blocks < 1 || !u2_encode_fn()) return NVJ_ERR_UNSUPPORTED;
  if (!once_per_device(opted_in, [](int) {
        return cudaFuncSetAttribute(prefill_umma2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) == cudaSuccess;
      }))
    return NVJ_ERR_LAUNCH;
  CUtensorMap k_map, v_map;
  if (!tensor_map_cached(&k_map, 2, k_cache, (uint64_t)num_blocks * kBlk, u2_make_map) ||
      !tensor_map_cached(&v_map, 2, v_cache, (uint64_t)num_blocks * kBlk, u2_make_map))
    return NVJ_ERR_UNSUPPORTED;
  // The kernel zeroes what no tile writes itself (padding tokens, rows of several tokens without keys), and the
  // decode-row pass of a mixed batch does the same for its rows: no memset launch in front of a batch.
  Umma2Params p{};
  p.zero_fill = 1;
  p.q = q; p.q_dtype = q_dtype;
  p.block_tables = block_tables; p.kv_lens = kv_lens; p.positions = positions; p.query_start_loc = query_start_loc;
  p.out = out; p.status = status; p.num_blocks = num_blocks; p.rows = rows; p.token_bucket = token_bucket;
  p.table_width = table_width; p.skip_single = skip_single; p.scale = scale; p.split_p = split_p;
  const int pairs = (token_bucket + 2 * kU2Tokens - 1) / (2 * kU2Tokens) + rows;
  // Key-range splits: only while the batch leaves pair slots free, as many as the lent area holds; the kernel settles
  // the number per pair from what the batch really holds.
  int splits = 1;
  const int slots = u2_pair_slots();
  if (split_area && slots > 0) {
    // by the most clusters the batch can hold (a batch of many short rows is launched whole: its extra splits would
    // only scan the rows and leave, 200 us on 256 rows of 4 tokens)
    const int most = pairs * kHkv;
    splits = slots / most < kU2MaxSplits ? slots / most : kU2MaxSplits;
    const size_t per_split = sizeof(float) * (size_t)token_bucket * kHq * (kD + 2);
    const size_t info_bytes = ws_round(sizeof(int4) * 2 * (size_t)pairs * kHkv);
    const size_t room = split_bytes < prefill_split_bytes() ? split_bytes : prefill_split_bytes();
    while (splits > 1 && ws_round(per_split * splits) + info_bytes > room) --splits;
    if (splits < 1) splits = 1;
    // The partials end where the lent area ends: its low end borders arrival counters of calls with more rows.
    split_area = reinterpret_cast<float*>(reinterpret_cast<char*>(split_area) + split_bytes - ws_round(per_split * splits) - info_bytes);
  }
  if (splits > 1) {
    p.part_o = split_area;
    p.part_ml = split_area + (size_t)splits * token_bucket * kHq * kD;
    p.tile_info = reinterpret_cast<int4*>(reinterpret_cast<char*>(split_area) + ws_round(sizeof(float) * (size_t)splits * token_bucket * kHq * (kD + 2)));
    p.pair_slots = slots;
  }
  dim3 grid(2 * pairs, kHkv, splits);
  prefill_umma2_kernel<<<grid, kU2Threads, kSmemBytes, stream>>>(k_map, v_map, p);
  if (cudaGetLastError() != cudaSuccess) return NVJ_ERR_LAUNCH;
  if (splits > 1) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs, kHkv, kU2MergeParts);
    cfg.blockDim = dim3(kU2MergeThreads, 1, 1);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, prefill_umma2_merge_kernel, p) != cudaSuccess) return NVJ_ERR_LAUNCH;
  }
  return cudaGetLastError() == cudaSuccess ? NVJ_OK : NVJ_ERR_LAUNCH;
}

}  // namespace nvj

#ifdef NVJ_PHASE_TIMING
extern "C" int nvj_debug_prefill_phase_ns(unsigned long long* host_out) {  // [512][8]
  return cudaMemcpyFromSymbol(host_out, nvj::g_u2_phase_ns, sizeof(nvj::g_u2_phase_ns)) == cudaSuccess ? 0 : 1;
}
#endif
