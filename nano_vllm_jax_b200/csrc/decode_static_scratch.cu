// Paged decode for callers that cannot allocate device memory.
//
// Some hosts of this library only ever see buffers that a framework hands them
// for the duration of one call: an XLA custom-call handler gets its operands and
// results and nothing else, and a plugin running inside another runtime's stream
// callback or memory pool must not call cudaMalloc (it would synchronise the
// device, or break the runtime's accounting).  Such callers have nowhere to keep
// the decode workspace that nvj_paged_decode asks for.  This entry point runs the
// same kernels with the workspace taken from a fixed array that is part of the
// library image, so the call itself allocates nothing.
//
// The array, the per-device set-up that resolves its device address, and the
// entry point live in this one file on purpose: in host code the array's name is
// only a handle for the runtime, not a device address.  The address a kernel can
// use comes from cudaGetSymbolAddress, queried once per device with that device
// current, and that pointer is what the kernels receive.

#include <mutex>

#include "paged_decode.cuh"

namespace nvj {

constexpr int kStaticMaxBatch = NVJ_STATIC_SCRATCH_MAX_BATCH;
constexpr int kStaticMaxCtas = 320;  // two CTAs per SM up to 160 SMs; a larger device runs 320 CTAs
constexpr size_t kStaticSlots = 2ull * kStaticMaxCtas + 2ull * ((kStaticMaxCtas + kMergeGroup - 1) / kMergeGroup);
constexpr size_t kStaticHeaderBytes = (64 + sizeof(int32_t) * ((size_t)kStaticMaxBatch + kGroupCounters) + 255) / 256 * 256;
constexpr size_t kStaticMlBytes = (sizeof(float) * kStaticSlots * kHq * 2 + 255) / 256 * 256;
constexpr size_t kStaticAccBytes = (sizeof(float) * kStaticSlots * kHq * kD + 255) / 256 * 256;
constexpr size_t kStaticScratchBytes = kStaticHeaderBytes + kStaticMlBytes + kStaticAccBytes;
static_assert(kStaticScratchBytes == NVJ_STATIC_SCRATCH_BYTES, "header and library disagree on the scratch size");

// The scratch itself: status word, arrival counters, per-CTA and per-group partial
// results.  Every GPU that loads the library holds these ~5 MiB until exit.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

static std::mutex g_setup_mutex;
static void* g_scratch_ptr[64];  // device address of g_static_scratch, per device ordinal

// Device address of the scratch array on the current device (nullptr on failure).
static void* static_scratch_for_current_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_static_scratch) != cudaSuccess || ptr == nullptr) {
      (void)cudaGetLastError();
      return nullptr;
    }
    g_scratch_ptr[dev] = ptr;
  }
  return g_scratch_ptr[dev];
}

static bool ptr16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace nvj

extern "C" int nvj_paged_decode_static_scratch(const void* q, int q_dtype, const void* k_cache_layer,
                                               const void* v_cache_layer, int kv_dtype,
                                               int64_t num_blocks, int block_size, int num_kv_heads,
                                               int head_dim, int num_q_heads,
                                               const int32_t* block_tables, int table_width,
                                               const int32_t* seq_lens, int batch, float scale,
                                               float* out, int32_t* status_out, nvj_stream_t stream) {
  using namespace nvj;
  if (batch < 0 || table_width < 0 || num_blocks < 0 || block_size <= 0 || num_kv_heads <= 0 ||
      num_q_heads <= 0 || head_dim <= 0 || num_q_heads % num_kv_heads != 0)
    return NVJ_ERR_INVALID_ARGUMENT;
  if (batch > kStaticMaxBatch) return NVJ_ERR_TOO_LARGE;
  if (batch == 0) return NVJ_OK;
  if (!q || !k_cache_layer || !v_cache_layer || !block_tables || !seq_lens || !out)
    return NVJ_ERR_INVALID_ARGUMENT;
  char* scratch = static_cast<char*>(static_scratch_for_current_device());
  if (!scratch) return NVJ_ERR_WORKSPACE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);

  DecodeParams p{};
  p.q = q;
  p.k_cache = static_cast<const char*>(k_cache_layer);
  p.v_cache = static_cast<const char*>(v_cache_layer);
  p.block_tables = block_tables;
  p.seq_lens = seq_lens;
  p.out = out;
  p.status = reinterpret_cast<int32_t*>(scratch);
  p.group_counters = reinterpret_cast<int32_t*>(scratch + 64);
  p.counters = reinterpret_cast<int32_t*>(scratch + 64 + sizeof(int32_t) * kGroupCounters);
  p.part_ml = reinterpret_cast<float*>(scratch + kStaticHeaderBytes);
  p.part_acc = reinterpret_cast<float*>(scratch + kStaticHeaderBytes + kStaticMlBytes);
  p.num_blocks = num_blocks;
  p.batch = batch;
  p.table_width = table_width;
  p.block_size = block_size;
  p.num_kv_heads = num_kv_heads;
  p.num_q_heads = num_q_heads;
  p.head_dim = head_dim;
  p.q_dtype = q_dtype;
  p.kv_dtype = kv_dtype;
  p.scale = scale;

  // The array keeps whatever the previous call left.  The partial results are
  // always written before they are read, but the status word and the arrival
  // counters must start at zero, and a call that was flagged may have left them
  // dirty: clear the header every time (a memset node on the stream, no allocation).
  if (cudaMemsetAsync(scratch, 0, 64 + sizeof(int32_t) * ((size_t)batch + kGroupCounters), s) != cudaSuccess)
    return NVJ_ERR_LAUNCH;

  int num_ctas = decode_num_ctas();
  if (num_ctas <= 0) return NVJ_ERR_LAUNCH;
  if (num_ctas > kStaticMaxCtas) num_ctas = kStaticMaxCtas;
  const bool fast = kv_dtype == NVJ_BF16 && block_size == kBlk && num_kv_heads == kHkv &&
                    num_q_heads == kHq && head_dim == kD && (q_dtype == NVJ_BF16 || q_dtype == NVJ_F32) &&
                    ptr16(q) && ptr16(k_cache_layer) && ptr16(v_cache_layer) && ptr16(out);
  int rc = NVJ_ERR_UNSUPPORTED;
  // tensor-core streaming kernel, one CTA per SM: its partials fit the slots as long as the device has at most 320 SMs
  if (fast && q_dtype == NVJ_BF16 && decode_wide_num_ctas() <= kStaticMaxCtas) {
    p.width = 1;
    rc = launch_decode_wide(p, s);
    p.width = 0;
  }
  if (rc == NVJ_ERR_UNSUPPORTED) rc = fast ? launch_decode_pipelined(p, num_ctas, s) : launch_decode_generic(p, s);
  if (rc != NVJ_OK) return rc;
  if (status_out &&
      cudaMemcpyAsync(status_out, scratch, sizeof(int32_t), cudaMemcpyDeviceToDevice, s) != cudaSuccess)
    return NVJ_ERR_LAUNCH;
  return NVJ_OK;
}
