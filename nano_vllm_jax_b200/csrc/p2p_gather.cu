// All-gather of each rank's per-step tokens over NVLink peer stores, for one process per GPU on one node.
//
// The only exchange on the path is a few hundred int32 per rank and step; a library all-gather
// spends 7-20 us on it (launch + protocol).  Here every rank owns an exchange buffer that its
// peers map through CUDA IPC:
//
//   header   published, consumed (uint64 epoch counters of this rank), arrivals (uint32)
//   data     [3][world][n] words of 64 bits = (epoch << 32 | token), three sets used in turn (epoch % 3)
//
// A token travels together with the epoch it belongs to in ONE 8-byte store, so the receiver needs no flag and the
// sender no fence: a word whose upper half carries the awaited epoch is the awaited token (the aligned 8-byte store
// is indivisible).  No step of the protocol waits for an NVLink round trip before it can go on.
//
// Two forms use it.
//
// (1) nvj_p2p_allgather_i32, one blocking kernel per rank and step: store the words into slot `rank` of every
//     peer's set, wait (bounded) until all words of the own set carry the epoch, copy the tokens out.
//
// (2) the split form for a pipelined decode step, where the wait must not sit between two steps:
//     nvj_p2p_argmax_publish   token pick of the step fused with the publish: every CTA takes a row's argmax and
//                              stores the word into every peer's set.  The same CTAs can collect the step before
//                              (below), one word per thread.  The publish waits for nobody.
//     nvj_p2p_collect          waits (bounded) for the oldest published epoch that has not been collected yet and
//                              copies its tokens out; does nothing when there is none.
//     A step k + 1 runs  append + decode,  then one launch that collects step k and publishes step k + 1: step k's
//     tokens have had a whole step to arrive, so a peer that is late by less than one step costs nothing, and no
//     launch of the step waits beside the attention kernel (which fills every SM's register file: a waiting kernel
//     that got an SM first delayed the attention's last CTA).  Three sets suffice: a peer overwrites set k % 3 when it
//     publishes k + 3, which it does after collecting k + 2, hence after this rank's launch k + 2 has started, hence
//     (stream order) after this rank's launch k + 1, the one that collects k, has finished.
//
// Every wait has a time limit (nvj_set_wait_limit_ns, default 1 s); on a timeout the kernel flags
// NVJ_DEV_TIMEOUT and returns, and the call can be issued again.  Plain peer stores only: no multicast.
// The reference is single-device and has no counterpart.

#include <atomic>
#include <cstring>

#include "nvj_common.cuh"
#include "row_argmax.cuh"

namespace nvj {

constexpr int kP2pMaxWorld = 16;
constexpr int kP2pSets = 3;

struct P2pHeader {
  unsigned long long published;  // last epoch this rank published (device-kept epochs)
  unsigned long long consumed;   // last epoch this rank collected
  unsigned int arrivals;         // CTAs of the running publish / collect kernel that are done
  unsigned int failed;           // a wait of the running kernel ran out
  unsigned int pad[2];
};
static_assert(sizeof(P2pHeader) % 16 == 0, "the data sets start 16-byte aligned");

struct P2pPeers {
  char* base[kP2pMaxWorld];
};

__device__ __forceinline__ P2pHeader* p2p_header(char* base) { return reinterpret_cast<P2pHeader*>(base); }
__device__ __forceinline__ unsigned long long* p2p_set(char* base, unsigned long long epoch, int world, int n) {
  return reinterpret_cast<unsigned long long*>(base + sizeof(P2pHeader)) + (long long)(epoch % kP2pSets) * world * n;
}
__device__ __forceinline__ unsigned long long p2p_word(int32_t token, unsigned long long epoch) {
  return (epoch << 32) | (unsigned long long)(uint32_t)token;
}
__device__ __forceinline__ void st_word(unsigned long long* p, unsigned long long v) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_word(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

// One thread waits (bounded) until `word` carries `epoch` and returns the token; `*ok` is cleared when the limit
// ran out (or another thread of the CTA has given up already: `failed_sh`).  `first` is the value of a load issued
// earlier, so that callers can put other work between the load and the check.
__device__ __forceinline__ int32_t p2p_await_word(const unsigned long long* word, unsigned long long first, unsigned long long epoch,
                                                  unsigned long long wait_ns, volatile int* failed_sh, bool* ok) {
  const unsigned long long want = epoch & 0xffffffffull;
  unsigned long long w = first;
  if ((w >> 32) != want) {
    const unsigned long long t0 = global_timer_ns();
    for (uint32_t spins = 0;; ++spins) {
      w = ld_word(word);
      if ((w >> 32) == want) break;
      if ((spins & 63u) == 63u && (*failed_sh || global_timer_ns() - t0 > wait_ns)) {
        *failed_sh = 1;
        *ok = false;
        return 0;
      }
    }
  }
  return (int32_t)(uint32_t)w;
}

__global__ void __launch_bounds__(256) p2p_allgather_kernel(P2pPeers peers, const int32_t* local, int n, int rank, int world,
                                                           unsigned long long epoch, unsigned long long wait_ns, int32_t* out,
                                                           int32_t* status) {
  __shared__ unsigned long long epoch_sh;
  __shared__ int failed;
  P2pHeader* own = p2p_header(peers.base[rank]);
  if (threadIdx.x == 0) {
    failed = 0;
    if (epoch == 0) {  // epoch kept on the device: the same launch can then be replayed from a CUDA graph
      epoch = own->published + 1;
      own->published = epoch;
      own->consumed = epoch;
    }
    epoch_sh = epoch;
  }
  __syncthreads();
  epoch = epoch_sh;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const unsigned long long w = p2p_word(local[i], epoch);
    for (int r = 0; r < world; ++r) st_word(p2p_set(peers.base[r], epoch, world, n) + rank * n + i, w);
  }
  // eight independent loads per thread in flight, then the checks: the words arrive together, so after the first
  // wait the others cost no round trip each
  const unsigned long long* set = p2p_set(peers.base[rank], epoch, world, n);
  const int count = world * n;
  bool ok = true;
  for (int base = threadIdx.x; base < count; base += 8 * blockDim.x) {
    unsigned long long w[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = base + u * blockDim.x;
      w[u] = i < count ? ld_word(set + i) : 0ull;
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = base + u * blockDim.x;
      if (i < count && ok) {
        const int32_t token = p2p_await_word(set + i, w[u], epoch, wait_ns, &failed, &ok);
        if (ok) out[i] = token;
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0 && failed && status) atomicOr(status, NVJ_DEV_TIMEOUT);
}

// Token pick fused with the publish (and, optionally, with the collect of the step before).  CTA r takes the argmax
// of row r (first maximum wins, as row_argmax_kernel), stores the token locally and sends its word to every peer
// (thread t to peer t).  With collect_out the same threads first fetch row r's tokens of the oldest epoch that has
// not been collected, one word per thread, loaded before the argmax and checked after it.  The CTA that finishes last
// advances this rank's epoch counters (local stores: nothing here waits for the links unless a peer is a step late).
__global__ void __launch_bounds__(kArgmaxThreads) p2p_argmax_publish_kernel(P2pPeers peers, const float* x, int row_len, int n, int rank,
                                                                            int world, int32_t* tokens, int32_t* collect_out,
                                                                            int32_t* seq_lens, int32_t* positions, long long capacity,
                                                                            unsigned long long wait_ns, int32_t* status) {
  P2pHeader* own = p2p_header(peers.base[rank]);
  // the counters are advanced by the last CTA only, after every CTA of the launch has read them
  const unsigned long long published = *reinterpret_cast<volatile unsigned long long*>(&own->published);
  const unsigned long long consumed = *reinterpret_cast<volatile unsigned long long*>(&own->consumed);
  const unsigned long long epoch = published + 1, wanted = consumed + 1;
  const bool collecting = collect_out != nullptr && wanted <= published;
  __shared__ int token_sh, failed_sh;
  const int r = blockIdx.x;
  const unsigned long long* word = nullptr;
  unsigned long long first = 0;
  if (threadIdx.x == 0) failed_sh = 0;
  if (collecting && (int)threadIdx.x < world) {
    word = p2p_set(peers.base[rank], wanted, world, n) + threadIdx.x * n + r;
    first = ld_word(word);
  }
  const int token = row_argmax_cta(x + (long long)r * row_len, row_len);
  if (threadIdx.x == 0) {
    token_sh = token;
    tokens[r] = token;
    // the step's resident metadata, for the next step; a row without room was flagged by the decode pass already
    // (this launch's status word reports waits that ran out, nothing else)
    if (seq_lens) advance_row(seq_lens, positions, r, capacity, nullptr);
  }
  __syncthreads();
  if ((int)threadIdx.x < world) {
    st_word(p2p_set(peers.base[threadIdx.x], epoch, world, n) + rank * n + r, p2p_word(token_sh, epoch));
    if (collecting) {
      bool ok = true;
      const int32_t got = p2p_await_word(word, first, wanted, wait_ns, &failed_sh, &ok);
      if (ok) collect_out[threadIdx.x * n + r] = got;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (failed_sh) {
      atomicOr(&own->failed, 1u);
      if (status) atomicOr(status, NVJ_DEV_TIMEOUT);
    }
    __threadfence();
    if (atomicAdd(&own->arrivals, 1u) == gridDim.x - 1u) {
      __threadfence();
      const unsigned int failed = *reinterpret_cast<volatile unsigned int*>(&own->failed);
      own->arrivals = 0;
      own->failed = 0;
      own->published = epoch;
      if (collecting && !failed) own->consumed = wanted;  // after a timeout the same epoch is collected again
    }
  }
}

// The collect alone: one word per thread; the CTA that finishes last advances `consumed` unless a wait ran out.
__global__ void __launch_bounds__(kArgmaxThreads) p2p_collect_kernel(char* own_base, int n, int world, unsigned long long wait_ns,
                                                                     int32_t* out, int32_t* status) {
  P2pHeader* own = p2p_header(own_base);
  const unsigned long long epoch = *reinterpret_cast<volatile unsigned long long*>(&own->consumed) + 1;
  if (epoch > *reinterpret_cast<volatile unsigned long long*>(&own->published)) return;  // nothing to collect
  __shared__ int failed_sh;
  if (threadIdx.x == 0) failed_sh = 0;
  __syncthreads();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < world * n) {
    const unsigned long long* word = p2p_set(own_base, epoch, world, n) + i;
    bool ok = true;
    const int32_t got = p2p_await_word(word, ld_word(word), epoch, wait_ns, &failed_sh, &ok);
    if (ok) out[i] = got;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (failed_sh) {
      atomicOr(&own->failed, 1u);
      if (status) atomicOr(status, NVJ_DEV_TIMEOUT);
    }
    __threadfence();
    if (atomicAdd(&own->arrivals, 1u) == gridDim.x - 1u) {
      __threadfence();
      const unsigned int failed = *reinterpret_cast<volatile unsigned int*>(&own->failed);
      own->arrivals = 0;
      own->failed = 0;
      if (!failed) own->consumed = epoch;
    }
  }
}

static std::atomic<unsigned long long> g_wait_limit_ns{kWaitLimitNs};

unsigned long long wait_limit_ns() { return g_wait_limit_ns.load(std::memory_order_relaxed); }

// A barrier that nobody arrives on, waited for with the limit: exercises the timeout branch of the bounded
// mbarrier wait that every pipelined kernel uses, without a fault and without a second party.
__global__ void __launch_bounds__(64) bounded_wait_selftest_kernel(unsigned long long wait_ns, int32_t* status, int32_t* returned) {
  __shared__ alignas(8) unsigned long long bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&bar), 1);
    mbar_fence_init();
  }
  __syncthreads();
  const bool ok = mbar_wait(smem_u32(&bar), 0u, &abort_flag, status, wait_ns);
  if (!ok) atomicAdd(returned, 1);
}

static bool p2p_args_ok(int rank, int world, void* const* peer_buffers, P2pPeers& peers) {
  if (world <= 0 || world > kP2pMaxWorld || rank < 0 || rank >= world || !peer_buffers) return false;
  for (int r = 0; r < world; ++r) {
    if (!peer_buffers[r]) return false;
    peers.base[r] = static_cast<char*>(peer_buffers[r]);
  }
  return true;
}

}  // namespace nvj

extern "C" void nvj_set_wait_limit_ns(uint64_t ns) { nvj::g_wait_limit_ns.store(ns ? ns : nvj::kWaitLimitNs, std::memory_order_relaxed); }

extern "C" uint64_t nvj_get_wait_limit_ns(void) { return nvj::wait_limit_ns(); }

extern "C" int nvj_selftest_bounded_wait(int32_t* status, int32_t* returned, nvj_stream_t stream) {
  if (!status || !returned) return NVJ_ERR_INVALID_ARGUMENT;
  nvj::bounded_wait_selftest_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(nvj::wait_limit_ns(), status, returned);
  return cudaGetLastError() == cudaSuccess ? NVJ_OK : NVJ_ERR_LAUNCH;
}

extern "C" size_t nvj_p2p_gather_buffer_bytes(int world, int n) {
  if (world <= 0 || world > nvj::kP2pMaxWorld || n < 0) return 0;
  return sizeof(nvj::P2pHeader) + sizeof(unsigned long long) * nvj::kP2pSets * (size_t)world * n;
}

extern "C" int nvj_p2p_buffer_create(size_t bytes, void** dev_ptr, unsigned char* handle64) {
  if (!dev_ptr || !handle64 || bytes == 0) return NVJ_ERR_INVALID_ARGUMENT;
  void* p = nullptr;
  if (cudaMalloc(&p, bytes) != cudaSuccess) return NVJ_ERR_LAUNCH;
  if (cudaMemset(p, 0, bytes) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) { cudaFree(p); return NVJ_ERR_LAUNCH; }
  cudaIpcMemHandle_t h;
  static_assert(sizeof(h) == 64, "IPC handles are exchanged as 64 bytes");
  if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) { cudaFree(p); return NVJ_ERR_UNSUPPORTED; }
  memcpy(handle64, &h, 64);
  *dev_ptr = p;
  return NVJ_OK;
}

extern "C" int nvj_p2p_buffer_open(const unsigned char* handle64, void** dev_ptr) {
  if (!dev_ptr || !handle64) return NVJ_ERR_INVALID_ARGUMENT;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  void* p = nullptr;
  if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
    (void)cudaGetLastError();
    return NVJ_ERR_UNSUPPORTED;
  }
  *dev_ptr = p;
  return NVJ_OK;
}

extern "C" int nvj_p2p_buffer_close(void* dev_ptr) {
  return dev_ptr && cudaIpcCloseMemHandle(dev_ptr) == cudaSuccess ? NVJ_OK : NVJ_ERR_INVALID_ARGUMENT;
}

extern "C" int nvj_p2p_buffer_destroy(void* dev_ptr) {
  return dev_ptr && cudaFree(dev_ptr) == cudaSuccess ? NVJ_OK : NVJ_ERR_INVALID_ARGUMENT;
}

extern "C" int nvj_p2p_allgather_i32(const int32_t* local, int n, int rank, int world, void* const* peer_buffers,
                                     uint32_t epoch, int32_t* out, int32_t* status, nvj_stream_t stream) {
  using namespace nvj;
  if (n < 0) return NVJ_ERR_INVALID_ARGUMENT;
  P2pPeers peers{};
  if (!p2p_args_ok(rank, world, peer_buffers, peers)) return NVJ_ERR_INVALID_ARGUMENT;
  if (n == 0) return NVJ_OK;
  if (!local || !out) return NVJ_ERR_INVALID_ARGUMENT;
  p2p_allgather_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(peers, local, n, rank, world, epoch, wait_limit_ns(), out,
                                                                         status);
  return cudaGetLastError() == cudaSuccess ? NVJ_OK : NVJ_ERR_LAUNCH;
}

extern "C" int nvj_p2p_argmax_publish(const float* x, int rows, int row_len, int32_t* tokens, int rank, int world,
                                      void* const* peer_buffers, int32_t* collect_out, int32_t* seq_lens, int32_t* positions,
                                      int table_width, int block_size, int32_t* status, nvj_stream_t stream) {
  using namespace nvj;
  if (rows < 0 || row_len <= 0 || (seq_lens && (table_width < 0 || block_size <= 0))) return NVJ_ERR_INVALID_ARGUMENT;
  P2pPeers peers{};
  if (!p2p_args_ok(rank, world, peer_buffers, peers)) return NVJ_ERR_INVALID_ARGUMENT;
  if (rows == 0) return NVJ_OK;
  if (!x || !tokens) return NVJ_ERR_INVALID_ARGUMENT;
  p2p_argmax_publish_kernel<<<rows, kArgmaxThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      peers, x, row_len, rows, rank, world, tokens, collect_out, seq_lens, positions, (long long)table_width * block_size,
      wait_limit_ns(), status);
  return cudaGetLastError() == cudaSuccess ? NVJ_OK : NVJ_ERR_LAUNCH;
}

extern "C" int nvj_p2p_collect(void* own_buffer, int n, int world, int32_t* out, int32_t* status, nvj_stream_t stream) {
  using namespace nvj;
  if (world <= 0 || world > kP2pMaxWorld || n < 0 || !own_buffer) return NVJ_ERR_INVALID_ARGUMENT;
  if (n == 0) return NVJ_OK;
  if (!out) return NVJ_ERR_INVALID_ARGUMENT;
  const int ctas = (world * n + kArgmaxThreads - 1) / kArgmaxThreads;
  p2p_collect_kernel<<<ctas, kArgmaxThreads, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<char*>(own_buffer), n, world,
                                                                                    wait_limit_ns(), out, status);
  return cudaGetLastError() == cudaSuccess ? NVJ_OK : NVJ_ERR_LAUNCH;
}
