// Ragged packed prefill attention on the 5th-generation tensor cores: tcgen05.mma with both
// accumulators and the left-hand operands (Q, P) in tensor memory (TMEM), K and V staged by TMA,
// for the model's full-attention shape (bf16 cache, 16-token blocks, 2 KV heads x 4 query heads,
// head_dim 256).
//
// One CTA = 32 consecutive query tokens of one table row x the 4 query heads of one KV head
// = 128 query rows (UMMA M = 128, TMEM lane = row = head * 32 + token).  Keys are walked once,
// in tiles of 64, through the row's block table.  Ten warps, three roles:
//   warp 0     producer: TMA tile loads (cp.async.bulk.tensor, 128-byte swizzle) of K and V per
//              key tile (one box of 16 keys x 64 dims per cache block and 64-dim chunk) into
//              3-stage rings; a K stage is released when its S product retires, a V stage when
//              its P V product does;
//   warp 1     one elected lane issues the MMAs: S(t) = Q K(t)^T (M128 N64 K16 x 16, A = Q from
//              TMEM) into one of two S buffers, and O += P(t) V(t) (M128 N256 K16 x 4, A = P
//              from TMEM as two bf16 terms hi + lo, V read as an MN-major operand); S(t + 2) is
//              issued as soon as P V (t) has retired, so it overlaps the softmax of tile t + 1;
//   warps 2-9  two threads per query row (a warp may only touch TMEM lanes 32 * (warp % 4) ..
//              + 31, so the two halves of a row's columns sit in warps w and w + 4).  They stage
//              Q into TMEM once (global -> registers -> tcgen05.st), then per tile read S
//              (tcgen05.ld), mask, exchange half maxima through shared memory, and write
//              P = exp2(S - m) over the S columns they came from.  The running maximum m is
//              only raised when a tile exceeds it by more than 2^8; then the warp rescales its
//              lanes of O in TMEM (tcgen05.ld/st), which is rare.  At the end O / l -> global.
// TMEM columns: Q [0, 128) (two bf16 per column), S/P buffers [128, 192) and [192, 256),
// O [256, 512).
// Shared-memory operands use the canonical 128-byte-swizzle layouts of the UMMA descriptors:
// rows of 128 bytes (64 bf16), 16-byte chunk j of row r stored at chunk j ^ (r & 7), 8-row
// groups 1024 bytes apart.  K and V tiles share one physical layout ([64-d chunk][key][128 B]);
// only the descriptor says which dimension is contracted.
// What bounds it: every 64-key tile costs 64 KiB of L2 -> shared memory traffic per CTA for
// 12.6 MFLOP of tensor work; an SM takes in about 20-30 bytes per clock through TMA, so a tile
// takes ~2850 cycles while its MMAs need ~1540.
// mbarrier parity waits can only tell two consecutive phases apart: every waiter here observes
// every phase of the barriers it uses, in order.
// Rows of the cache that were never written must hold finite values (the allocator zero-fills):
// a masked key has weight 0, and 0 x NaN would still poison the row.
// Every wait is bounded; on a timeout the kernel flags NVJ_DEV_TIMEOUT, stops issuing, lets
// copies in flight land, and still frees its TMEM.
// Semantics: nanovllm_jax/kv_cache.py:831-849, nanovllm_jax/kernels/full_attention_triton.py:51-145.

#include "paged_decode.cuh"
#include "umma.cuh"

namespace nvj {

constexpr int kUmTokens = 32;    // query tokens per CTA
constexpr int kUmRows = 128;     // query rows = tokens x 4 heads
constexpr int kUmKeys = 64;      // keys per tile
constexpr int kUmStages = 3;     // K and V tiles in flight
constexpr int kUmThreads = 320;  // producer warp, MMA warp, 8 softmax warps
constexpr int kUmSoftmaxThreads = 256;
constexpr int kUmTmemCols = 512;
constexpr int kUmColQ = 0;       // Q as the A operand: 256 bf16 per row = 128 columns
constexpr int kUmColS = 128;     // two S accumulators of 64 columns; P (hi: 32 columns, lo: 32) overwrites its S
constexpr int kUmColO = 256;     // O accumulator: columns [256, 512)
constexpr uint32_t kUmTileBytes = kUmKeys * kRowBytes;  // one K (or V) tile of one KV head: 32 KiB
constexpr float kUmLog2e = 1.4426950408889634f;
constexpr float kUmRescaleGap = 8.f;  // log2 units a tile may exceed the running maximum before O is rescaled

struct UmmaPrefillParams {
  const void* q;
  const int32_t* block_tables;
  const int32_t* kv_lens;
  const int32_t* positions;
  const int32_t* query_start_loc;
  float* out;
  int32_t* status;
  long long num_blocks;
  int rows, token_bucket, table_width, skip_single, q_dtype;
  float scale;
};

struct UmmaSmem {
  alignas(1024) char k[kUmStages][4][kUmKeys * 128];  // [stage][64-d chunk][key][128 B], swizzled
  alignas(1024) char v[kUmStages][4][kUmKeys * 128];
  alignas(8) unsigned long long q_full, k_full[kUmStages], v_full[kUmStages], k_empty[kUmStages], v_empty[kUmStages],
      s_full[2], p_full, pv_done, x_full;
  float xchg[2][2][kUmRows];  // [tile parity][column half][row]: half maxima, at the end half sums
  uint32_t tmem_base;
  int row, tok0, ntok, abort_flag;
};

// ---- warp 0: TMA loads ------------------------------------------------------------------------
__device__ __forceinline__ void um_producer(const CUtensorMap* k_map, const CUtensorMap* v_map, const UmmaPrefillParams& p,
                                            UmmaSmem& sm, int row, int kvh, int kv_len, int n_tiles, int lane) {
  const int need_blocks = (kv_len + kBlk - 1) / kBlk;
  const int oob = (int)(p.num_blocks * kBlk);  // a box that starts here is filled with zeros
  int ids = -1;
  for (int t = 0; t < n_tiles; ++t) {
    const int s = t % kUmStages;
    const uint32_t reuse_parity = ((t / kUmStages) - 1) & 1;  // phase in which the stage's previous tile (t - 3) released it
    if ((t & 7) == 0) {  // block ids of the next 8 tiles, one per lane
      const int bi = t * 4 + lane;
      ids = -1;
      if (bi < need_blocks && bi < p.table_width) {
        ids = p.block_tables[(long long)row * p.table_width + bi];
        if (ids < 0 || ids >= p.num_blocks) {
          atomicOr(p.status, NVJ_DEV_BAD_BLOCK_ID);
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
    // K is released as soon as S(t - 3) has been computed, V only after P V (t - 3)
    if (t >= kUmStages && !um_wait(&sm.k_empty[s], reuse_parity, &sm.abort_flag, p.status)) break;
    if (lane == 0) {
      const uint32_t kb = smem_u32(&sm.k_full[s]);
      mbar_arrive_expect_tx(kb, kUmTileBytes);
#pragma unroll
      for (int b = 0; b < 4; ++b)
#pragma unroll
        for (int c = 0; c < 4; ++c) tma_load_3d(smem_u32(&sm.k[s][c][0]) + b * (kBlk * 128), k_map, c * 64, kvh, z[b], kb);
    }
    if (t >= kUmStages && !um_wait(&sm.v_empty[s], reuse_parity, &sm.abort_flag, p.status)) break;
    if (lane == 0) {
      const uint32_t vb = smem_u32(&sm.v_full[s]);
      mbar_arrive_expect_tx(vb, kUmTileBytes);
#pragma unroll
      for (int b = 0; b < 4; ++b)
#pragma unroll
        for (int c = 0; c < 4; ++c) tma_load_3d(smem_u32(&sm.v[s][c][0]) + b * (kBlk * 128), v_map, c * 64, kvh, z[b], vb);
    }
    __syncwarp();
  }
}

// ---- warp 1: MMA issue ----------------------------------------------------------------------
// One lane issues everything.
// Descriptors are built once; stepping through a tile only adds to the 14-bit start-address field
// (shared-memory addresses are below 256 KiB, so the sum never carries out of the field).
__device__ __forceinline__ bool um_issue_s(UmmaSmem& sm, const UmmaPrefillParams& p, uint32_t tmem, uint64_t k_desc0, int t,
                                           int stage, uint32_t full_parity, int lane) {
  if (!um_wait(&sm.k_full[stage], full_parity, &sm.abort_flag, p.status)) return false;
  tc_fence_after_sync();
  if (um_elect_one()) {
    constexpr uint32_t idesc = umma_idesc(kUmKeys, false);
    const uint64_t k_desc = k_desc0 + (uint64_t)((stage * 4 * kUmKeys * 128) >> 4);
    const uint32_t d = tmem + kUmColS + (t & 1) * kUmKeys;
#pragma unroll
    for (int ks = 0; ks < 16; ++ks)  // 16 dims per MMA: 8 columns of Q; K chunk ks / 4, 32 bytes into its swizzled rows
      umma_bf16_ts(d, tmem + kUmColQ + ks * 8, k_desc + (uint64_t)(((ks >> 2) * (kUmKeys * 128) + (ks & 3) * 32) >> 4), idesc,
                   ks > 0 ? 1u : 0u);
    umma_commit(smem_u32(&sm.s_full[t & 1]));
    umma_commit(smem_u32(&sm.k_empty[stage]));
  }
  __syncwarp();
  return true;
}

__device__ __forceinline__ void um_mma_warp(UmmaSmem& sm, const UmmaPrefillParams& p, uint32_t tmem, int n_tiles, int lane) {
  const uint64_t k_desc0 = umma_desc(smem_u32(&sm.k[0][0][0]), 16, 1024);
  const uint64_t v_desc0 = umma_desc(smem_u32(&sm.v[0][0][0]), kUmKeys * 128, 1024);
  if (!um_wait(&sm.q_full, 0, &sm.abort_flag, p.status)) return;
  if (!um_issue_s(sm, p, tmem, k_desc0, 0, 0, 0, lane)) return;
  if (n_tiles > 1 && !um_issue_s(sm, p, tmem, k_desc0, 1, 1, 0, lane)) return;
  int sv = 0, sk = 2 % kUmStages;      // stage of V(t) and of K(t + 2)
  uint32_t pv = 0, pk = 2 / kUmStages;  // parities of their full barriers
  for (int t = 0; t < n_tiles; ++t) {
    if (!um_wait(&sm.v_full[sv], pv, &sm.abort_flag, p.status)) return;
    if (!um_wait(&sm.p_full, t & 1, &sm.abort_flag, p.status)) return;
    tc_fence_after_sync();
    if (um_elect_one()) {
      constexpr uint32_t idesc = umma_idesc(kD, true);
      const uint64_t v_desc = v_desc0 + (uint64_t)((sv * 4 * kUmKeys * 128) >> 4);
      const uint32_t pa = tmem + kUmColS + (t & 1) * kUmKeys;
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {  // 16 keys per MMA: 8 columns of P, two 8-key groups of V
        const uint64_t dv = v_desc + (uint64_t)((kk * 2048) >> 4);
        umma_bf16_ts(tmem + kUmColO, pa + kk * 8, dv, idesc, (t > 0 || kk > 0) ? 1u : 0u);
        umma_bf16_ts(tmem + kUmColO, pa + 32 + kk * 8, dv, idesc, 1u);
      }
      umma_commit(smem_u32(&sm.v_empty[sv]));
      umma_commit(smem_u32(&sm.pv_done));
    }
    __syncwarp();
    // S(t + 2) overwrites the columns P V (t) reads P(t) from; MMAs of different shapes are not
    // ordered against each other, so wait for P V (t) to retire first
    if (t + 2 < n_tiles) {
      if (!um_wait(&sm.pv_done, t & 1, &sm.abort_flag, p.status)) return;
      if (!um_issue_s(sm, p, tmem, k_desc0, t + 2, sk, pk, lane)) return;
    }
    if (++sv == kUmStages) { sv = 0; pv ^= 1u; }
    if (++sk == kUmStages) { sk = 0; pk ^= 1u; }
  }
}

// ---- warps 2-9: Q staging, softmax, epilogue ------------------------------------------------
// Two threads per query row: warp w works on TMEM lanes [32 * (w % 4), +32) (the only ones it may
// touch) and on half (w - 2) / 4 of the columns.  The halves exchange their tile maxima through
// shared memory so that both keep the same running maximum.
__device__ __forceinline__ void um_softmax_warps(UmmaSmem& sm, const UmmaPrefillParams& p, uint32_t tmem, int tok0,
                                                 int ntok, int kvh, int kv_len, int n_tiles, int warp, int lane) {
  const int quarter = warp & 3, half = (warp - 2) >> 2;
  const int r = quarter * 32 + lane, token = lane, hl = quarter;
  const uint32_t my_tmem = tmem + ((uint32_t)(quarter * 32) << 16);
  // ---- this row's half of Q (128 dims) -> 64 TMEM columns, two bf16 per column
  {
    const long long qrow = ((long long)(tok0 + token) * kHq + kvh * kG + hl) * kD + half * (kD / 2);
#pragma unroll 1
    for (int part = 0; part < 4; ++part) {  // 32 dims = 16 columns at a time
      uint32_t w[16];
      if (token >= ntok) {
#pragma unroll
        for (int i = 0; i < 16; ++i) w[i] = 0u;
      } else if (p.q_dtype == NVJ_BF16) {
        const uint4* src = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(p.q) + qrow + part * 32);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint4 u = ld_nc_u4(src + i);
          w[4 * i] = u.x; w[4 * i + 1] = u.y; w[4 * i + 2] = u.z; w[4 * i + 3] = u.w;
        }
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
      tmem_st16(my_tmem + kUmColQ + half * 64 + part * 16, w);
    }
    tmem_st_wait();
    tc_fence_before_sync();
    mbar_arrive(smem_u32(&sm.q_full));
  }
  const int my_pos = token < ntok ? p.positions[tok0 + token] : -1;
  const int last_key = my_pos < kv_len - 1 ? my_pos : kv_len - 1;  // last key this row may see
  const float scale_log2 = p.scale * kUmLog2e;
  float m_row = -INFINITY, l_row = 0.f;  // m_row in units of log2(e) * scale, the same in both halves

  for (int t = 0; t < n_tiles; ++t) {
    const int b = t & 1;
    const uint32_t s_tmem = my_tmem + kUmColS + b * kUmKeys;
    if (!um_wait(&sm.s_full[b], (t >> 1) & 1, &sm.abort_flag, p.status)) return;
    tc_fence_after_sync();
    float s[32];
    tmem_ld32(s_tmem + half * 32, s);
    const int lim = last_key - t * kUmKeys - half * 32;  // columns [0, lim] of this half are visible
    float hmax = -INFINITY;
    if (lim >= 31) {
#pragma unroll
      for (int i = 0; i < 32; i += 2) hmax = fmaxf(hmax, fmaxf(s[i], s[i + 1]));
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) { s[i] = i <= lim ? s[i] : -INFINITY; hmax = fmaxf(hmax, s[i]); }
    }
    sm.xchg[b][half][r] = hmax;
    mbar_arrive(smem_u32(&sm.x_full));  // release; the bounded wait below acquires the partner's value
    if (!um_wait(&sm.x_full, t & 1, &sm.abort_flag, p.status)) return;
    // from here on both halves have read their S columns: P may overwrite them
    const float tmax = fmaxf(hmax, sm.xchg[b][half ^ 1][r]) * scale_log2;  // scale > 0
    if (t == 0) {
      m_row = tmax;
    } else if (__any_sync(0xffffffffu, tmax > m_row + kUmRescaleGap)) {
      // rare: raise the maxima of this warp's rows and rescale their O, once the last P V has landed
      if (!um_wait(&sm.pv_done, (t - 1) & 1, &sm.abort_flag, p.status)) return;
      tc_fence_after_sync();
      const float m_new = fmaxf(m_row, tmax);
      const float f = m_new == -INFINITY ? 1.f : ex2_approx(m_row - m_new);
      m_row = m_new;
      l_row *= f;
#pragma unroll 1
      for (int cc = 0; cc < kD / 64; ++cc) {
        float o[32];
        tmem_ld32(my_tmem + kUmColO + half * (kD / 2) + cc * 32, o);
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] *= f;
        tmem_st32(my_tmem + kUmColO + half * (kD / 2) + cc * 32, o);
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
    // A parity wait only tells two consecutive phases apart, so every phase of pv_done has to be
    // observed in turn (the rescaling above and the epilogue rely on it); P V (t - 1) has
    // normally retired by now.
    if (t >= 1 && !um_wait(&sm.pv_done, (t - 1) & 1, &sm.abort_flag, p.status)) return;
    // P(t) as the A operand of P V: keys 2j, 2j + 1 of this half in column half * 16 + j; hi then lo
    tmem_st16(s_tmem + half * 16, hi);
    tmem_st16(s_tmem + 32 + half * 16, lo);
    tmem_st_wait();
    tc_fence_before_sync();
    mbar_arrive(smem_u32(&sm.p_full));
  }
  // ---- epilogue: O / l -> global, each half its 128 columns
  sm.xchg[n_tiles & 1][half][r] = l_row;
  mbar_arrive(smem_u32(&sm.x_full));
  if (!um_wait(&sm.x_full, n_tiles & 1, &sm.abort_flag, p.status)) return;
  l_row += sm.xchg[n_tiles & 1][half ^ 1][r];
  if (!um_wait(&sm.pv_done, (n_tiles - 1) & 1, &sm.abort_flag, p.status)) return;
  tc_fence_after_sync();
  const float inv = l_row > 0.f ? 1.f / l_row : 0.f;
  float* dst = p.out + ((long long)(tok0 + token) * kHq + kvh * kG + hl) * kD + half * (kD / 2);
#pragma unroll 1
  for (int cc = 0; cc < kD / 64; ++cc) {
    float o[32];
    tmem_ld32(my_tmem + kUmColO + half * (kD / 2) + cc * 32, o);
    if (token < ntok) {
#pragma unroll
      for (int i = 0; i < 32; i += 4)
        *reinterpret_cast<float4*>(dst + cc * 32 + i) = make_float4(o[i] * inv, o[i + 1] * inv, o[i + 2] * inv, o[i + 3] * inv);
    }
  }
}

__global__ void __launch_bounds__(kUmThreads, 1)
prefill_umma_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
                    const UmmaPrefillParams p) {
  extern __shared__ unsigned char um_smem_raw[];
  UmmaSmem& sm = *reinterpret_cast<UmmaSmem*>((reinterpret_cast<uintptr_t>(um_smem_raw) + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kvh = blockIdx.y;

  // ---- set-up: TMEM, barriers, which (table row, 32-token tile) this CTA serves
  if (warp == 1) tmem_alloc(smem_u32(&sm.tmem_base), kUmTmemCols);
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&sm.q_full), kUmSoftmaxThreads);
    for (int i = 0; i < kUmStages; ++i) {
      mbar_init(smem_u32(&sm.k_full[i]), 1);
      mbar_init(smem_u32(&sm.v_full[i]), 1);
      mbar_init(smem_u32(&sm.k_empty[i]), 1);
      mbar_init(smem_u32(&sm.v_empty[i]), 1);
    }
    mbar_init(smem_u32(&sm.s_full[0]), 1);
    mbar_init(smem_u32(&sm.s_full[1]), 1);
    mbar_init(smem_u32(&sm.p_full), kUmSoftmaxThreads);
    mbar_init(smem_u32(&sm.pv_done), 1);
    mbar_init(smem_u32(&sm.x_full), kUmSoftmaxThreads);
    mbar_fence_init();
    sm.abort_flag = 0;
    // heaviest tiles (the last tokens of a row see the most keys) get the lowest block indices
    int idx = gridDim.x - 1 - blockIdx.x, row = -1, tok0 = 0, ntok = 0;
    for (int r = 0; r < p.rows; ++r) {
      const int lo = p.query_start_loc[r];
      int hi = p.query_start_loc[r + 1];
      hi = hi < p.token_bucket ? hi : p.token_bucket;
      int tiles = hi > lo ? (hi - lo + kUmTokens - 1) / kUmTokens : 0;
      if (p.skip_single && p.query_start_loc[r + 1] - lo == 1) tiles = 0;
      if (idx < tiles) {
        row = r;
        tok0 = lo + idx * kUmTokens;
        ntok = hi - tok0 < kUmTokens ? hi - tok0 : kUmTokens;
        break;
      }
      idx -= tiles;
    }
    sm.row = row; sm.tok0 = tok0; sm.ntok = ntok;
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = sm.tmem_base;
  const int row = sm.row, tok0 = sm.tok0, ntok = sm.ntok;

  int kv_len = row >= 0 ? p.kv_lens[row] : 0;
  if (kv_len > p.table_width * kBlk) {
    if (threadIdx.x == 0) atomicOr(p.status, NVJ_DEV_BAD_LENGTH);
    kv_len = p.table_width * kBlk;
  }
  // the token of the tile that sees the most keys bounds the key range (positions need not grow along the tile:
  // a rectangular batch pads rows with position 0)
  const int max_pos = __reduce_max_sync(0xffffffffu, (row >= 0 && lane < ntok) ? p.positions[tok0 + lane] : -1);
  const int key_end = kv_len < max_pos + 1 ? kv_len : max_pos + 1;
  const int n_tiles = key_end > 0 ? (key_end + kUmKeys - 1) / kUmKeys : 0;

  if (n_tiles > 0) {
    if (warp == 0) um_producer(&k_map, &v_map, p, sm, row, kvh, kv_len, n_tiles, lane);
    else if (warp == 1) um_mma_warp(sm, p, tmem, n_tiles, lane);
    else um_softmax_warps(sm, p, tmem, tok0, ntok, kvh, kv_len, n_tiles, warp, lane);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (sm.abort_flag) {  // give copies and MMAs in flight time to land before the CTA's memory is released
    const unsigned long long t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) tmem_dealloc(tmem, kUmTmemCols);
}

typedef CUresult (*UmEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static UmEncodeTiledFn um_encode_fn() {
  static UmEncodeTiledFn fn = [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult res;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &res) != cudaSuccess ||
        res != cudaDriverEntryPointSuccess)
      ptr = nullptr;
    return reinterpret_cast<UmEncodeTiledFn>(ptr);
  }();
  return fn;
}

// bf16 tensor [outer, mid, 256] (row pitch 512 B), boxes of [box_outer, 1, 64], 128-byte swizzle
static bool um_make_map(CUtensorMap* map, const void* base, uint64_t mid, uint64_t outer, uint32_t box_outer) {
  const cuuint64_t dims[3] = {(cuuint64_t)kD, mid, outer};
  const cuuint64_t strides[2] = {(cuuint64_t)kRowBytes, (cuuint64_t)kRowBytes * mid};
  const cuuint32_t box[3] = {64, 1, box_outer};
  const cuuint32_t estr[3] = {1, 1, 1};
  return um_encode_fn()(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Returns NVJ_ERR_UNSUPPORTED when the driver offers no tensor-map encoder or the scale is not
// positive (row maxima are taken before scaling); the caller then takes the mma.sync kernel.
int launch_prefill_umma(const void* q, int q_dtype, const char* k_cache, const char* v_cache,
                        long long num_blocks, const int32_t* block_tables, int table_width,
                        const int32_t* kv_lens, const int32_t* positions, const int32_t* query_start_loc,
                        int rows, int token_bucket, float scale, float* out, int32_t* status,
                        int skip_single, cudaStream_t stream) {
  static PerDeviceFlags opted_in;
  constexpr int kSmemBytes = (int)sizeof(UmmaSmem) + 1024;
  static_assert(kSmemBytes <= 232448, "tiles exceed the shared memory of one CTA");
  if (!(scale > 0.f) || num_blocks < 1 || !um_encode_fn()) return NVJ_ERR_UNSUPPORTED;
  if (!once_per_device(opted_in, [](int) {
        return cudaFuncSetAttribute(prefill_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) == cudaSuccess;
      }))
    return NVJ_ERR_LAUNCH;
  CUtensorMap k_map, v_map;
  const TensorMapMaker make = [](CUtensorMap* m, const void* base, uint64_t tokens) { return um_make_map(m, base, kHkv, tokens, kBlk); };
  if (!tensor_map_cached(&k_map, 1, k_cache, (uint64_t)num_blocks * kBlk, make) ||
      !tensor_map_cached(&v_map, 1, v_cache, (uint64_t)num_blocks * kBlk, make))
    return NVJ_ERR_UNSUPPORTED;
  if (!skip_single &&
      cudaMemsetAsync(out, 0, sizeof(float) * (size_t)token_bucket * kHq * kD, stream) != cudaSuccess)
    return NVJ_ERR_LAUNCH;
  UmmaPrefillParams p{};
  p.q = q; p.q_dtype = q_dtype;
  p.block_tables = block_tables; p.kv_lens = kv_lens; p.positions = positions; p.query_start_loc = query_start_loc;
  p.out = out; p.status = status; p.num_blocks = num_blocks; p.rows = rows; p.token_bucket = token_bucket;
  p.table_width = table_width; p.skip_single = skip_single; p.scale = scale;
  dim3 grid((token_bucket + kUmTokens - 1) / kUmTokens + rows, kHkv, 1);
  prefill_umma_kernel<<<grid, kUmThreads, kSmemBytes, stream>>>(k_map, v_map, p);
  return cudaGetLastError() == cudaSuccess ? NVJ_OK : NVJ_ERR_LAUNCH;
}

}  // namespace nvj
