// Ragged packed prefill attention over the paged cache with tensor-core tiles
// (bf16 mma.sync m16n8k16, fp32 accumulate) for the model's full-attention shape:
// bf16 cache, 16-token blocks, 2 KV heads x 4 query heads, head_dim 256.
//
// One CTA = 16 consecutive query tokens of one table row, all 8 query heads
// (warp w = head w, so both KV heads' blocks are used whole).  Keys are walked in
// tiles of 32 (two cache blocks) through the row's block table; K/V tiles are
// staged with 16-byte cp.async into a 2-stage ring, rows ordered [head][token] /
// [kv head][key] and padded to 528 bytes so that ldmatrix is bank-conflict free.  Per tile: S = Q K^T (16 x 32 per warp),
// mask p < kv_len and p <= position(token), online softmax in log2 units,
// O += P V with P carried as two bf16 terms (hi + lo).  Output fp32; tokens at or beyond
// query_start_loc[rows] are left at the zero the launcher wrote.
// Semantics: nanovllm_jax/kv_cache.py:831-849 and
// nanovllm_jax/kernels/full_attention_triton.py:51-145.

#include "paged_decode.cuh"

namespace nvj {

constexpr int kPfTokens = 16;
constexpr int kPfKeys = 32;
constexpr int kPfRowBytes = 528;  // 512 + 16: consecutive rows start 4 banks apart
constexpr int kPfThreads = 256;
constexpr float kPfLog2e = 1.4426950408889634f;

struct PrefillParams {
  const void* q;
  const char* k_cache;
  const char* v_cache;
  const int32_t* block_tables;
  const int32_t* kv_lens;
  const int32_t* positions;
  const int32_t* query_start_loc;
  float* out;
  int32_t* status;
  long long num_blocks;
  int rows, token_bucket, table_width, q_dtype;
  int skip_single;  // rows with exactly one query token are served by the decode kernel
  float scale;
};

struct PrefillSmem {
  alignas(16) char q[kPfTokens * kHq][kPfRowBytes];
  alignas(16) char k[2][kPfKeys * kHkv][kPfRowBytes];
  alignas(16) char v[2][kPfKeys * kHkv][kPfRowBytes];
  int row, tok0, ntok;
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2_bf16(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

// Stage the K and V rows of key tile `tile` (32 keys, both KV heads) of table row `row`.
// V rows of keys at or beyond kv_len are zero-filled: their weights are exactly 0, and
// 0 x (whatever bits the pool holds) must stay 0.
__device__ __forceinline__ void load_kv_tile(const PrefillParams& p, PrefillSmem& sm, int stage, int row,
                                             int tile, int kv_len) {
  for (int c = threadIdx.x; c < kPfKeys * kHkv * 32; c += kPfThreads) {
    const int r = c >> 5, chunk = c & 31;  // r = kv head * 32 + key: consecutive keys are adjacent rows
    const int key = tile * kPfKeys + (r & 31);
    const long long blk = p.block_tables[(long long)row * p.table_width + (key >> 4)];
    const bool ok = key < kv_len && blk >= 0 && blk < p.num_blocks;
    const long long src = (blk * kBlk + (key & 15)) * kTokenBytes + (r >> 5) * kRowBytes + chunk * 16;
    const uint32_t dk = smem_u32(&sm.k[stage][r][chunk * 16]);
    const uint32_t dv = smem_u32(&sm.v[stage][r][chunk * 16]);
    if (ok) {
      cp_async16(dk, p.k_cache + src);
      cp_async16(dv, p.v_cache + src);
    } else {
      *reinterpret_cast<uint4*>(&sm.k[stage][r][chunk * 16]) = make_uint4(0u, 0u, 0u, 0u);
      *reinterpret_cast<uint4*>(&sm.v[stage][r][chunk * 16]) = make_uint4(0u, 0u, 0u, 0u);
      if (key < kv_len && chunk == 0) atomicOr(p.status, NVJ_DEV_BAD_BLOCK_ID);
    }
  }
}

__global__ void __launch_bounds__(kPfThreads, 1) prefill_mma_kernel(PrefillParams p) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  PrefillSmem& sm = *reinterpret_cast<PrefillSmem*>(smem_raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;

  // ---- which (table row, 16-token tile) is this CTA?
  if (threadIdx.x == 0) {
    int idx = blockIdx.x, row = -1, tok0 = 0, ntok = 0;
    for (int r = 0; r < p.rows; ++r) {
      const int lo = p.query_start_loc[r];
      int hi = p.query_start_loc[r + 1];
      hi = hi < p.token_bucket ? hi : p.token_bucket;
      int tiles = hi > lo ? (hi - lo + kPfTokens - 1) / kPfTokens : 0;
      if (p.skip_single && p.query_start_loc[r + 1] - lo == 1) tiles = 0;
      if (idx < tiles) {
        row = r;
        tok0 = lo + idx * kPfTokens;
        ntok = hi - tok0 < kPfTokens ? hi - tok0 : kPfTokens;
        break;
      }
      idx -= tiles;
    }
    sm.row = row; sm.tok0 = tok0; sm.ntok = ntok;
  }
  __syncthreads();
  const int row = sm.row, tok0 = sm.tok0, ntok = sm.ntok;
  if (row < 0) return;

  int kv_len = p.kv_lens[row];
  const int cap = p.table_width * kBlk;
  if (kv_len > cap) {
    if (threadIdx.x == 0) atomicOr(p.status, NVJ_DEV_BAD_LENGTH);
    kv_len = cap;
  }
  // positions of this thread's two query rows (token g and g + 8); -1 = no such token
  const int pos_a = g < ntok ? p.positions[tok0 + g] : -1;
  const int pos_b = g + 8 < ntok ? p.positions[tok0 + g + 8] : -1;
  int max_pos = pos_a > pos_b ? pos_a : pos_b;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) max_pos = max(max_pos, __shfl_xor_sync(kFullMask, max_pos, o));
  const int key_end = kv_len < max_pos + 1 ? kv_len : max_pos + 1;
  if (key_end <= 0) return;  // nothing visible: the rows stay zero
  const int n_tiles = (key_end + kPfKeys - 1) / kPfKeys;

  // ---- stage Q (all 8 heads of the 16 tokens) and the first K/V tile
  for (int c = threadIdx.x; c < kPfTokens * kHq * 32; c += kPfThreads) {
    const int r = c >> 5, chunk = c & 31;  // r = head * 16 + token: consecutive tokens are adjacent rows
    const int tok = r & 15, hd = r >> 4;
    char* dst = &sm.q[r][chunk * 16];
    if (tok >= ntok) {
      *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
    } else if (p.q_dtype == NVJ_BF16) {
      cp_async16(smem_u32(dst), static_cast<const char*>(p.q) + ((long long)(tok0 + tok) * kHq + hd) * kRowBytes + chunk * 16);
    } else {
      const float* src = static_cast<const float*>(p.q) + ((long long)(tok0 + tok) * kHq + hd) * kD + chunk * 8;
      const float4 a = *reinterpret_cast<const float4*>(src), b = *reinterpret_cast<const float4*>(src + 4);
      *reinterpret_cast<uint4*>(dst) = make_uint4(pack2_bf16(a.x, a.y), pack2_bf16(a.z, a.w), pack2_bf16(b.x, b.y), pack2_bf16(b.z, b.w));
    }
  }
  load_kv_tile(p, sm, 0, row, 0, kv_len);
  cp_async_commit();

  const int head = warp, kvh = warp >> 2;
  const float scale_log2 = p.scale * kPfLog2e;
  float o[32][4];
#pragma unroll
  for (int i = 0; i < 32; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;

  // per-lane ldmatrix row addresses (bytes), see the fragment layouts of mma.m16n8k16
  const uint32_t q_addr = smem_u32(&sm.q[head * kPfTokens + (lane & 7) + 8 * ((lane >> 3) & 1)][16 * (lane >> 4)]);
  const int k_row = kvh * kPfKeys + (lane & 7) + 8 * (lane >> 4);  // + 16 rows for the second 16 keys
  const int k_col = 16 * ((lane >> 3) & 1);
  const int v_row = kvh * kPfKeys + (lane & 7) + 8 * ((lane >> 3) & 1);
  const int v_col = 16 * (lane >> 4);

  for (int tile = 0; tile < n_tiles; ++tile) {
    const int stage = tile & 1;
    if (tile + 1 < n_tiles) load_kv_tile(p, sm, stage ^ 1, row, tile + 1, kv_len);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();

    // ---- S = Q K^T for 32 keys
    float s[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll
    for (int ks = 0; ks < 16; ++ks) {
      uint32_t a[4], b0[4], b1[4];
      ldsm_x4(a, q_addr + ks * 32);
      ldsm_x4(b0, smem_u32(&sm.k[stage][k_row][k_col + ks * 32]));
      ldsm_x4(b1, smem_u32(&sm.k[stage][k_row + 16][k_col + ks * 32]));
      mma_bf16(s[0], a, b0[0], b0[1]);
      mma_bf16(s[1], a, b0[2], b0[3]);
      mma_bf16(s[2], a, b1[0], b1[1]);
      mma_bf16(s[3], a, b1[2], b1[3]);
    }
    // ---- mask, online softmax (log2 units)
    float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int key = tile * kPfKeys + nt * 8 + 2 * t + e;
        const bool in_len = key < kv_len;
        s[nt][e] = (in_len && key <= pos_a) ? s[nt][e] * scale_log2 : -INFINITY;
        s[nt][2 + e] = (in_len && key <= pos_b) ? s[nt][2 + e] * scale_log2 : -INFINITY;
        mx_a = fmaxf(mx_a, s[nt][e]);
        mx_b = fmaxf(mx_b, s[nt][2 + e]);
      }
    }
    mx_a = fmaxf(mx_a, __shfl_xor_sync(kFullMask, mx_a, 1));
    mx_a = fmaxf(mx_a, __shfl_xor_sync(kFullMask, mx_a, 2));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(kFullMask, mx_b, 1));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(kFullMask, mx_b, 2));
    const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
    const float ms_a = mn_a == -INFINITY ? 0.f : mn_a, ms_b = mn_b == -INFINITY ? 0.f : mn_b;
    const float al_a = ex2_approx(m_a - ms_a), al_b = ex2_approx(m_b - ms_b);
    m_a = mn_a; m_b = mn_b;
    l_a *= al_a; l_b *= al_b;
#pragma unroll
    for (int i = 0; i < 32; ++i) { o[i][0] *= al_a; o[i][1] *= al_a; o[i][2] *= al_b; o[i][3] *= al_b; }
    // The weights enter the P x V product as two bf16 terms, P = hi + lo with lo = bf16(P - hi):
    // their sum carries 16 mantissa bits, so the product matches fp32 weights far inside the
    // tolerance instead of losing bf16's 2^-9 per weight.
    uint32_t pa[2][4], pl[2][4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      const float p0 = ex2_approx(s[nt][0] - ms_a), p1 = ex2_approx(s[nt][1] - ms_a);
      const float p2 = ex2_approx(s[nt][2] - ms_b), p3 = ex2_approx(s[nt][3] - ms_b);
      l_a += p0 + p1;
      l_b += p2 + p3;
      const __nv_bfloat162 h01 = __floats2bfloat162_rn(p0, p1), h23 = __floats2bfloat162_rn(p2, p3);
      pa[nt >> 1][(nt & 1) * 2] = *reinterpret_cast<const uint32_t*>(&h01);      // row g,   keys of this n-tile
      pa[nt >> 1][(nt & 1) * 2 + 1] = *reinterpret_cast<const uint32_t*>(&h23);  // row g+8
      pl[nt >> 1][(nt & 1) * 2] = pack2_bf16(p0 - __low2float(h01), p1 - __high2float(h01));
      pl[nt >> 1][(nt & 1) * 2 + 1] = pack2_bf16(p2 - __low2float(h23), p3 - __high2float(h23));
    }
    // ---- O += P V
#pragma unroll
    for (int s2 = 0; s2 < 2; ++s2) {
#pragma unroll
      for (int dn = 0; dn < 16; ++dn) {
        uint32_t b[4];
        ldsm_x4_trans(b, smem_u32(&sm.v[stage][v_row + s2 * 16][v_col + dn * 32]));
        mma_bf16(o[2 * dn], pa[s2], b[0], b[1]);
        mma_bf16(o[2 * dn + 1], pa[s2], b[2], b[3]);
        mma_bf16(o[2 * dn], pl[s2], b[0], b[1]);
        mma_bf16(o[2 * dn + 1], pl[s2], b[2], b[3]);
      }
    }
    __syncthreads();  // the next iteration's prefetch overwrites this stage's neighbour only after everyone left it
  }

  // ---- normalise and store
  l_a += __shfl_xor_sync(kFullMask, l_a, 1);
  l_a += __shfl_xor_sync(kFullMask, l_a, 2);
  l_b += __shfl_xor_sync(kFullMask, l_b, 1);
  l_b += __shfl_xor_sync(kFullMask, l_b, 2);
  const float inv_a = l_a > 0.f ? 1.f / l_a : 0.f, inv_b = l_b > 0.f ? 1.f / l_b : 0.f;
  if (g < ntok) {
    float* dst = p.out + ((long long)(tok0 + g) * kHq + head) * kD + 2 * t;
#pragma unroll
    for (int nt = 0; nt < 32; ++nt) *reinterpret_cast<float2*>(dst + nt * 8) = make_float2(o[nt][0] * inv_a, o[nt][1] * inv_a);
  }
  if (g + 8 < ntok) {
    float* dst = p.out + ((long long)(tok0 + g + 8) * kHq + head) * kD + 2 * t;
#pragma unroll
    for (int nt = 0; nt < 32; ++nt) *reinterpret_cast<float2*>(dst + nt * 8) = make_float2(o[nt][2] * inv_b, o[nt][3] * inv_b);
  }
}

int launch_prefill_mma(const void* q, int q_dtype, const char* k_cache, const char* v_cache,
                       long long num_blocks, const int32_t* block_tables, int table_width,
                       const int32_t* kv_lens, const int32_t* positions, const int32_t* query_start_loc,
                       int rows, int token_bucket, float scale, float* out, int32_t* status,
                       int skip_single, cudaStream_t stream) {
  static PerDeviceFlags opted_in;
  if (!once_per_device(opted_in, [](int) {
        return cudaFuncSetAttribute(prefill_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    (int)sizeof(PrefillSmem)) == cudaSuccess;
      }))
    return NVJ_ERR_LAUNCH;
  // padded tokens (and rows that see no key) are defined to be zero; with skip_single the caller
  // has already cleared the output and the decode kernel has written the single-token rows
  if (!skip_single &&
      cudaMemsetAsync(out, 0, sizeof(float) * (size_t)token_bucket * kHq * kD, stream) != cudaSuccess)
    return NVJ_ERR_LAUNCH;
  PrefillParams p{};
  p.q = q; p.k_cache = k_cache; p.v_cache = v_cache; p.block_tables = block_tables; p.kv_lens = kv_lens;
  p.positions = positions; p.query_start_loc = query_start_loc; p.out = out; p.status = status;
  p.num_blocks = num_blocks; p.rows = rows; p.token_bucket = token_bucket; p.table_width = table_width;
  p.q_dtype = q_dtype; p.scale = scale; p.skip_single = skip_single;
  const int grid = (token_bucket + kPfTokens - 1) / kPfTokens + rows;
  prefill_mma_kernel<<<grid, kPfThreads, sizeof(PrefillSmem), stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? NVJ_OK : NVJ_ERR_LAUNCH;
}

}  // namespace nvj
