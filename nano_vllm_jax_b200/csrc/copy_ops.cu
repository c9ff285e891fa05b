// Index-list copies on the path: whole cache blocks (prefix reuse by copy) and
// GDN hybrid-state rows (snapshot into / restore from a pool keyed by prefix
// hash), plus the per-row argmax that stands in for the sampler.
//
// All three copies are HBM-bound: 16-byte vector accesses, four independent
// loads in flight per thread, a 2-D grid of (chunk group, row pair).  The
// algorithmic traffic is 2 x bytes moved (one read, one write).

#include "nvj_common.cuh"
#include "row_argmax.cuh"

namespace nvj {

constexpr int kCopyThreads = 256;
constexpr int kCopyUnroll = 4;
constexpr long long kCopyTileBytes = (long long)kCopyThreads * kCopyUnroll * 16;  // 16 KiB

__device__ __forceinline__ void st_cs_u4(void* p, uint4 v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

// Copies `bytes` (multiple of 16, both pointers 16-byte aligned) with CTA `block` of `nblocks`
// moving the 16 KiB tiles block, block + nblocks, ...
__device__ __forceinline__ void copy_span16(const char* src, char* dst, long long bytes, int block, int nblocks) {
  const long long chunks = bytes >> 4;
  for (long long base = (long long)block * kCopyThreads * kCopyUnroll; base < chunks;
       base += (long long)nblocks * kCopyThreads * kCopyUnroll) {
    uint4 v[kCopyUnroll];
#pragma unroll
    for (int u = 0; u < kCopyUnroll; ++u) {
      const long long c = base + u * kCopyThreads + threadIdx.x;
      if (c < chunks) v[u] = ld_nc_u4(src + (c << 4));
    }
#pragma unroll
    for (int u = 0; u < kCopyUnroll; ++u) {
      const long long c = base + u * kCopyThreads + threadIdx.x;
      if (c < chunks) st_cs_u4(dst + (c << 4), v[u]);
    }
  }
}

__device__ __forceinline__ void copy_span1(const char* src, char* dst, long long bytes, int block, int nblocks) {
  for (long long c = (long long)block * kCopyThreads + threadIdx.x; c < bytes; c += (long long)nblocks * kCopyThreads)
    dst[c] = src[c];
}

// The (source, destination) row indices of a copy: two device arrays, or, for a handful of pairs that the host knows
// (the usual case: one restore per prefix hit), the values themselves, carried in the kernel's parameters so that no
// host-to-device copy has to run in front of the launch.
constexpr int kInlinePairs = 24;
struct SlotLists {
  const int32_t* src;
  const int32_t* dst;
  int32_t inline_src[kInlinePairs];
  int32_t inline_dst[kInlinePairs];
  __device__ __forceinline__ long long source(int i) const { return src ? src[i] : inline_src[i]; }
  __device__ __forceinline__ long long destination(int i) const { return dst ? dst[i] : inline_dst[i]; }
};

// One table of rows that are copied by index: dst_base[dst_idx[i]] <- src_base[src_idx[i]].
struct RowTable {
  const char* src_base;
  char* dst_base;
  long long row_bytes;
  int vec16;
  int blocks;  // CTAs of grid.x that work on this table
};

// Both tables of a hybrid state (recurrent and conv) in one launch; grid.y = pair, grid.x = a.blocks + b.blocks.
__global__ void __launch_bounds__(kCopyThreads)
copy_rows_kernel(RowTable a, RowTable b, long long src_rows, long long dst_rows, const __grid_constant__ SlotLists slots,
                 int32_t* status) {
  const int i = blockIdx.y;
  const long long s = slots.source(i), d = slots.destination(i);
  if (s < 0 || s >= src_rows || d < 0 || d >= dst_rows) {
    if (threadIdx.x == 0 && blockIdx.x == 0 && status) atomicOr(status, NVJ_DEV_BAD_BLOCK_ID);
    return;
  }
  const bool first = (int)blockIdx.x < a.blocks;
  const RowTable& t = first ? a : b;
  const int block = first ? blockIdx.x : blockIdx.x - a.blocks;
  const char* src = t.src_base + s * t.row_bytes;
  char* dst = t.dst_base + d * t.row_bytes;
  if (t.vec16) copy_span16(src, dst, t.row_bytes, block, t.blocks);
  else copy_span1(src, dst, t.row_bytes, block, t.blocks);
}

// The same row copy for rows whose size is a multiple of 16 bytes, moved by the bulk-copy engine: one warp per
// CTA, a ring of kBulkStages chunks of kBulkChunk bytes in shared memory, every chunk loaded by one
// cp.async.bulk (global -> shared, completion on an mbarrier) and written back by one cp.async.bulk
// (shared -> global, tracked by a bulk group).  A thread keeps 64 KiB in flight instead of 64 bytes, which is
// what a copy of one 19 MB state row needs to reach the memory system's bandwidth: with 16-byte vector loads
// the same copy is bound by the latency of its few loads per thread.  Chunks of all (pair, table) combinations
// form one sequence dealt round-robin to the CTAs.
constexpr int kBulkChunk = 16 * 1024;
constexpr int kBulkStages = 4;

struct BulkSmem {
  alignas(128) unsigned char stage[kBulkStages][kBulkChunk];
  alignas(8) unsigned long long full[kBulkStages];
  int abort_flag;
};

__device__ __forceinline__ void bulk_s2g(void* gmem_dst, uint32_t smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gmem_dst), "r"(smem_src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory"); }

__global__ void __launch_bounds__(32)
copy_rows_bulk_kernel(RowTable a, RowTable b, long long src_rows, long long dst_rows, const __grid_constant__ SlotLists slots,
                      int n_pairs, int32_t* status) {
  extern __shared__ unsigned char bulk_smem_raw[];
  BulkSmem& sm = *reinterpret_cast<BulkSmem*>((reinterpret_cast<uintptr_t>(bulk_smem_raw) + 127) & ~(uintptr_t)127);
  if (threadIdx.x != 0) return;  // one thread drives the copy engine; the warp exists only to own the shared memory
  const long long chunks_a = (a.row_bytes + kBulkChunk - 1) / kBulkChunk, chunks_b = (b.row_bytes + kBulkChunk - 1) / kBulkChunk;
  const long long per_pair = chunks_a + chunks_b, total = per_pair * n_pairs;
  sm.abort_flag = 0;
  for (int s = 0; s < kBulkStages; ++s) mbar_init(smem_u32(&sm.full[s]), 1);
  mbar_fence_init();

  // chunk c of this CTA's subsequence -> (source, destination, bytes); bytes = 0 for a pair with a bad index
  auto locate = [&](long long c, const char*& src, char*& dst) -> uint32_t {
    const int pair = (int)(c / per_pair);
    long long r = c - (long long)pair * per_pair;
    const long long si = slots.source(pair), di = slots.destination(pair);
    if (si < 0 || si >= src_rows || di < 0 || di >= dst_rows) {
      if (status) atomicOr(status, NVJ_DEV_BAD_BLOCK_ID);
      return 0;
    }
    const RowTable& t = r < chunks_a ? a : b;
    if (r >= chunks_a) r -= chunks_a;
    const long long off = r * kBulkChunk;
    src = t.src_base + si * t.row_bytes + off;
    dst = t.dst_base + di * t.row_bytes + off;
    const long long left = t.row_bytes - off;
    return (uint32_t)(left < kBulkChunk ? left : kBulkChunk);
  };

  const long long first = blockIdx.x, stride = gridDim.x;
  const long long mine = first < total ? (total - first + stride - 1) / stride : 0;
  char* dsts[kBulkStages];
  uint32_t sizes[kBulkStages];
  auto issue_load = [&](long long k) {
    const int s = (int)(k % kBulkStages);
    const char* src = nullptr;
    sizes[s] = locate(first + k * stride, src, dsts[s]);
    const uint32_t bar = smem_u32(&sm.full[s]);
    if (sizes[s] > 0) {
      mbar_arrive_expect_tx(bar, sizes[s]);
      bulk_g2s(smem_u32(sm.stage[s]), src, sizes[s], bar);
    } else {
      mbar_arrive(bar);
    }
  };
  long long issued = 0;
  for (; issued < mine && issued < kBulkStages; ++issued) issue_load(issued);
  for (long long k = 0; k < mine; ++k) {
    const int s = (int)(k % kBulkStages);
    if (!mbar_wait(smem_u32(&sm.full[s]), (uint32_t)(k / kBulkStages) & 1u, &sm.abort_flag, status)) break;
    if (sizes[s] > 0) {
      fence_proxy_async_all();
      bulk_s2g(dsts[s], smem_u32(sm.stage[s]), sizes[s]);
    }
    bulk_commit();
    if (issued < mine) {
      bulk_wait_read<0>();  // the store has read the stage: it can take the next chunk
      issue_load(issued++);
    }
  }
  bulk_wait_all<0>();
  if (sm.abort_flag) {  // only after a timeout can loads still be in flight: hold the shared memory until they have landed
    const unsigned long long t0 = global_timer_ns();
    for (long long k = issued > kBulkStages ? issued - kBulkStages : 0; k < issued; ++k)
      while (!mbar_try_wait(smem_u32(&sm.full[k % kBulkStages]), (uint32_t)(k / kBulkStages) & 1u) &&
             global_timer_ns() - t0 < kWaitLimitNs) {
      }
  }
}

// Block copy across layers and K/V: grid.y = pair, grid.z = layer * 2 + (0: K, 1: V).
__global__ void __launch_bounds__(kCopyThreads)
copy_blocks_kernel(char* k_cache, char* v_cache, long long num_blocks, long long block_bytes,
                   long long layer_stride, const int32_t* src_ids, const int32_t* dst_ids, int vec16,
                   int32_t* status) {
  const int i = blockIdx.y;
  const long long s = src_ids[i], d = dst_ids[i];
  if (s < 0 || s >= num_blocks || d < 0 || d >= num_blocks) {
    if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.z == 0 && status)
      atomicOr(status, NVJ_DEV_BAD_BLOCK_ID);
    return;
  }
  if (s == d) return;
  char* base = (blockIdx.z & 1) ? v_cache : k_cache;
  base += (long long)(blockIdx.z >> 1) * layer_stride;
  if (vec16) copy_span16(base + s * block_bytes, base + d * block_bytes, block_bytes, blockIdx.x, gridDim.x);
  else copy_span1(base + s * block_bytes, base + d * block_bytes, block_bytes, blockIdx.x, gridDim.x);
}

// One CTA per row.  With seq_lens the row's resident decode metadata is advanced in the same launch, as
// advance_decode_metadata_kernel would (the tail of a decode step whose attention ran in pre-append form).
__global__ void __launch_bounds__(kArgmaxThreads)
row_argmax_kernel(const float* x, int row_len, int32_t* tokens, int32_t* seq_lens, int32_t* positions, long long capacity,
                  int32_t* status) {
  const int token = row_argmax_cta(x + (long long)blockIdx.x * row_len, row_len);
  if (threadIdx.x == 0) {
    tokens[blockIdx.x] = token;
    if (seq_lens) advance_row(seq_lens, positions, blockIdx.x, capacity, status);
  }
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Opt the bulk row-copy kernel into its 64 KiB of dynamic shared memory, once per device.
static bool bulk_copy_ready() {
  static PerDeviceFlags opted_in;
  return once_per_device(opted_in, [](int) {
    return cudaFuncSetAttribute(copy_rows_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                (int)sizeof(BulkSmem) + 128) == cudaSuccess;
  });
}

static int sm_count() {
  static PerDeviceFlags cached;  // 0 = not queried yet
  const int dev = current_device();
  if (dev < 0) return 0;
  int n = cached.v[dev].load(std::memory_order_acquire);
  if (n == 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    cached.v[dev].store(n, std::memory_order_release);
  }
  return n;
}

static int grid_x_for(long long bytes, int pairs) {
  // Enough CTAs to fill the machine a few times over, never more than one per tile.
  long long tiles = (bytes + kCopyTileBytes - 1) / kCopyTileBytes;
  long long want = (148LL * 16 + pairs - 1) / pairs;
  long long gx = tiles < want ? tiles : want;
  return gx < 1 ? 1 : (int)gx;
}

static RowTable row_table(const void* src, void* dst, long long row_bytes, int pairs) {
  RowTable t{};
  if (!src || !dst || row_bytes == 0) return t;  // blocks = 0: no CTA works on it
  t.src_base = static_cast<const char*>(src);
  t.dst_base = static_cast<char*>(dst);
  t.row_bytes = row_bytes;
  t.vec16 = aligned16(src) && aligned16(dst) && row_bytes % 16 == 0;
  t.blocks = grid_x_for(row_bytes, pairs);
  return t;
}

// One decode step of the batch metadata, on the device: every active row (seq_len > 0) grows by
// the token it is about to append; its position is the old length.  Rows that would outgrow
// their block table are flagged and left alone.
__global__ void advance_decode_metadata_kernel(int32_t* seq_lens, int32_t* positions, int batch, long long capacity,
                                               int32_t* status) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= batch) return;
  advance_row(seq_lens, positions, b, capacity, status);
}

}  // namespace nvj

extern "C" int nvj_abi_version(void) { return NVJ_ABI_VERSION; }

extern "C" const char* nvj_status_string(int status) {
  switch (status) {
    case NVJ_OK: return "ok";
    case NVJ_ERR_INVALID_ARGUMENT: return "invalid argument";
    case NVJ_ERR_UNSUPPORTED: return "unsupported shape or dtype";
    case NVJ_ERR_LAUNCH: return "kernel launch failed";
    case NVJ_ERR_WORKSPACE: return "workspace missing or too small";
    case NVJ_ERR_TOO_LARGE: return "size exceeds a built-in limit of this entry point";
    default: return "unknown status";
  }
}

extern "C" int nvj_copy_blocks(void* k_cache, void* v_cache, int num_layers, int64_t num_blocks,
                               int64_t block_bytes, int64_t layer_stride_bytes,
                               const int32_t* src_ids, const int32_t* dst_ids, int n_pairs,
                               int32_t* status, nvj_stream_t stream) {
  using namespace nvj;
  if (num_layers < 0 || num_blocks < 0 || block_bytes < 0 || n_pairs < 0 || layer_stride_bytes < 0)
    return NVJ_ERR_INVALID_ARGUMENT;
  if (n_pairs == 0 || num_layers == 0 || block_bytes == 0) return NVJ_OK;
  if (!k_cache || !v_cache || !src_ids || !dst_ids) return NVJ_ERR_INVALID_ARGUMENT;
  if (n_pairs > 65535 || num_layers * 2 > 65535) return NVJ_ERR_UNSUPPORTED;
  const int vec16 = aligned16(k_cache) && aligned16(v_cache) && block_bytes % 16 == 0 &&
                    layer_stride_bytes % 16 == 0;
  dim3 grid(grid_x_for(block_bytes, n_pairs * num_layers * 2), n_pairs, num_layers * 2);
  copy_blocks_kernel<<<grid, kCopyThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<char*>(k_cache), static_cast<char*>(v_cache), num_blocks, block_bytes,
      layer_stride_bytes, src_ids, dst_ids, vec16, status);
  return cudaGetLastError() == cudaSuccess ? NVJ_OK : NVJ_ERR_LAUNCH;
}

static int hybrid_copy(const void* conv_src, void* conv_dst, int64_t conv_row_bytes,
                       const void* rec_src, void* rec_dst, int64_t rec_row_bytes,
                       int64_t src_rows, int64_t dst_rows, const int32_t* src_slots,
                       const int32_t* dst_slots, int n, bool slots_on_host, int32_t* status, nvj_stream_t stream) {
  using namespace nvj;
  if (n < 0 || conv_row_bytes < 0 || rec_row_bytes < 0 || src_rows < 0 || dst_rows < 0)
    return NVJ_ERR_INVALID_ARGUMENT;
  if (n == 0) return NVJ_OK;
  if (!src_slots || !dst_slots) return NVJ_ERR_INVALID_ARGUMENT;
  if (n > 65535) return NVJ_ERR_UNSUPPORTED;
  SlotLists slots{};
  if (slots_on_host) {
    if (n > kInlinePairs) return NVJ_ERR_TOO_LARGE;
    for (int i = 0; i < n; ++i) { slots.inline_src[i] = src_slots[i]; slots.inline_dst[i] = dst_slots[i]; }
  } else {
    slots.src = src_slots;
    slots.dst = dst_slots;
  }
  if ((conv_src == nullptr) != (conv_dst == nullptr) || (rec_src == nullptr) != (rec_dst == nullptr))
    return NVJ_ERR_INVALID_ARGUMENT;
  const RowTable rec = row_table(rec_src, rec_dst, rec_row_bytes, n);
  const RowTable conv = row_table(conv_src, conv_dst, conv_row_bytes, n);
  if (rec.blocks + conv.blocks == 0) return NVJ_OK;
  // rows that the bulk-copy engine can move (16-byte aligned, sizes multiples of 16 bytes) go through it
  const bool bulk_ok = (rec.blocks == 0 || rec.vec16) && (conv.blocks == 0 || conv.vec16) && bulk_copy_ready();
  if (bulk_ok) {
    const long long chunks = ((rec.row_bytes + kBulkChunk - 1) / kBulkChunk + (conv.row_bytes + kBulkChunk - 1) / kBulkChunk) * n;
    const int sms = sm_count();
    const long long cap = (long long)(sms > 0 ? sms : 148) * 3;  // three CTAs of 64 KiB shared memory per SM
    const int ctas = (int)(chunks < cap ? chunks : cap);
    copy_rows_bulk_kernel<<<ctas, 32, sizeof(BulkSmem) + 128, static_cast<cudaStream_t>(stream)>>>(
        rec, conv, src_rows, dst_rows, slots, n, status);
    return cudaGetLastError() == cudaSuccess ? NVJ_OK : NVJ_ERR_LAUNCH;
  }
  dim3 grid(rec.blocks + conv.blocks, n, 1);
  copy_rows_kernel<<<grid, kCopyThreads, 0, static_cast<cudaStream_t>(stream)>>>(rec, conv, src_rows, dst_rows, slots, status);
  return cudaGetLastError() == cudaSuccess ? NVJ_OK : NVJ_ERR_LAUNCH;
}

extern "C" int nvj_hybrid_snapshot(const void* conv_table, void* conv_pool, int64_t conv_row_bytes,
                                   const void* rec_table, void* rec_pool, int64_t rec_row_bytes,
                                   int64_t table_rows, int64_t pool_rows,
                                   const int32_t* table_slots, const int32_t* pool_slots, int n,
                                   int32_t* status, nvj_stream_t stream) {
  return hybrid_copy(conv_table, conv_pool, conv_row_bytes, rec_table, rec_pool, rec_row_bytes,
                     table_rows, pool_rows, table_slots, pool_slots, n, false, status, stream);
}

extern "C" int nvj_hybrid_snapshot_host_slots(const void* conv_table, void* conv_pool, int64_t conv_row_bytes,
                                              const void* rec_table, void* rec_pool, int64_t rec_row_bytes,
                                              int64_t table_rows, int64_t pool_rows,
                                              const int32_t* table_slots, const int32_t* pool_slots, int n,
                                              int32_t* status, nvj_stream_t stream) {
  return hybrid_copy(conv_table, conv_pool, conv_row_bytes, rec_table, rec_pool, rec_row_bytes,
                     table_rows, pool_rows, table_slots, pool_slots, n, true, status, stream);
}

extern "C" int nvj_hybrid_restore(void* conv_table, const void* conv_pool, int64_t conv_row_bytes,
                                  void* rec_table, const void* rec_pool, int64_t rec_row_bytes,
                                  int64_t table_rows, int64_t pool_rows,
                                  const int32_t* table_slots, const int32_t* pool_slots, int n,
                                  int32_t* status, nvj_stream_t stream) {
  return hybrid_copy(conv_pool, conv_table, conv_row_bytes, rec_pool, rec_table, rec_row_bytes,
                     pool_rows, table_rows, pool_slots, table_slots, n, false, status, stream);
}

extern "C" int nvj_hybrid_restore_host_slots(void* conv_table, const void* conv_pool, int64_t conv_row_bytes,
                                             void* rec_table, const void* rec_pool, int64_t rec_row_bytes,
                                             int64_t table_rows, int64_t pool_rows,
                                             const int32_t* table_slots, const int32_t* pool_slots, int n,
                                             int32_t* status, nvj_stream_t stream) {
  return hybrid_copy(conv_pool, conv_table, conv_row_bytes, rec_pool, rec_table, rec_row_bytes,
                     pool_rows, table_rows, pool_slots, table_slots, n, true, status, stream);
}

extern "C" int nvj_advance_decode_metadata(int32_t* seq_lens, int32_t* positions, int batch,
                                           int table_width, int block_size, int32_t* status,
                                           nvj_stream_t stream) {
  using namespace nvj;
  if (batch < 0 || table_width < 0 || block_size <= 0) return NVJ_ERR_INVALID_ARGUMENT;
  if (batch == 0) return NVJ_OK;
  if (!seq_lens || !positions) return NVJ_ERR_INVALID_ARGUMENT;
  advance_decode_metadata_kernel<<<(batch + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      seq_lens, positions, batch, (long long)table_width * block_size, status);
  return cudaGetLastError() == cudaSuccess ? NVJ_OK : NVJ_ERR_LAUNCH;
}

extern "C" int nvj_copy_many_async(void* const* dst, const void* const* src, const size_t* bytes, int n,
                                   nvj_stream_t stream) {
  if (n < 0 || (n > 0 && (!dst || !src || !bytes))) return NVJ_ERR_INVALID_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  for (int i = 0; i < n; ++i) {
    if (bytes[i] == 0) continue;
    if (!dst[i] || !src[i]) return NVJ_ERR_INVALID_ARGUMENT;
    if (cudaMemcpyAsync(dst[i], src[i], bytes[i], cudaMemcpyDefault, s) != cudaSuccess) return NVJ_ERR_LAUNCH;
  }
  return NVJ_OK;
}

extern "C" int nvj_row_argmax(const float* x, int rows, int row_len, int32_t* tokens,
                              nvj_stream_t stream) {
  using namespace nvj;
  if (rows < 0 || row_len <= 0) return NVJ_ERR_INVALID_ARGUMENT;
  if (rows == 0) return NVJ_OK;
  if (!x || !tokens) return NVJ_ERR_INVALID_ARGUMENT;
  row_argmax_kernel<<<rows, kArgmaxThreads, 0, static_cast<cudaStream_t>(stream)>>>(x, row_len, tokens, nullptr, nullptr, 0, nullptr);
  return cudaGetLastError() == cudaSuccess ? NVJ_OK : NVJ_ERR_LAUNCH;
}

extern "C" int nvj_row_argmax_advance(const float* x, int rows, int row_len, int32_t* tokens, int32_t* seq_lens,
                                      int32_t* positions, int table_width, int block_size, int32_t* status,
                                      nvj_stream_t stream) {
  using namespace nvj;
  if (rows < 0 || row_len <= 0 || table_width < 0 || block_size <= 0) return NVJ_ERR_INVALID_ARGUMENT;
  if (rows == 0) return NVJ_OK;
  if (!x || !tokens || !seq_lens) return NVJ_ERR_INVALID_ARGUMENT;
  row_argmax_kernel<<<rows, kArgmaxThreads, 0, static_cast<cudaStream_t>(stream)>>>(x, row_len, tokens, seq_lens, positions,
                                                                                   (long long)table_width * block_size, status);
  return cudaGetLastError() == cudaSuccess ? NVJ_OK : NVJ_ERR_LAUNCH;
}
