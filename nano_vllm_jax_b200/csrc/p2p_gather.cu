// All-gather of each rank's per-step tokens over NVLink peer stores, for one process per GPU on one node.
//
// The only exchange on the path is a few hundred int32 per rank and step; a library all-gather
// spends 7-20 us on it (launch + protocol).  Here every rank owns an exchange buffer that its
// peers map through CUDA IPC:
//
//   header   flags[2][16] (uint64: the epoch each rank last published into data set 0 / 1),
//            published, consumed (uint64 epoch counters of this rank), arrivals (uint32)
//   data     [2][world][n] int32, two sets that alternate by epoch parity
//
// Two forms use it.
//
// (1) nvj_p2p_allgather_i32, one blocking kernel per rank and step: store the tokens into slot `rank` of
//     every peer's set, publish the epoch into every peer's flag (system-scope release), wait (bounded)
//     until all flags in the own buffer carry the epoch, copy the set out.
//
// (2) the split form for a pipelined decode step, where the wait must not sit between two steps:
//     nvj_p2p_argmax_publish   token pick of the step fused with the publish: every CTA takes a row's
//                              argmax; the CTA that finishes last copies the tokens into every peer's set
//                              and publishes the epoch.  One more CTA of the same launch can collect the
//                              step before (below).  The publish waits for nobody.
//     nvj_p2p_collect          waits (bounded) for the oldest published epoch that has not been collected
//                              yet and copies its set out; does nothing when there is none.
//     A step k + 1 runs  append + decode,  then one launch that collects step k and publishes step k + 1:
//     step k's tokens have had a whole step to arrive, so a peer that is late by less than one step costs
//     nothing, and no launch of the step waits beside the attention kernel (which fills every SM's register
//     file: a waiting kernel that got an SM first delayed the attention's last CTA).  Because every rank collects epoch k
//     before it publishes k + 1, and a peer publishes k + 2 only after it has seen this rank's flag k + 1
//     (it collects k + 1 first), nobody overwrites set (k & 1) before everyone has read it: two sets are
//     enough and a flag is either the awaited epoch or an older one.
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

struct P2pHeader {
  unsigned long long flags[2][kP2pMaxWorld];
  unsigned long long published;  // last epoch this rank published (device-kept epochs)
  unsigned long long consumed;   // last epoch this rank collected
  unsigned int arrivals;         // CTAs of the running publish kernel that are done
  unsigned int pad[3];
};
static_assert(sizeof(P2pHeader) % 16 == 0, "the data sets start 16-byte aligned");

struct P2pPeers {
  char* base[kP2pMaxWorld];
};

__device__ __forceinline__ P2pHeader* p2p_header(char* base) { return reinterpret_cast<P2pHeader*>(base); }
__device__ __forceinline__ int32_t* p2p_data(char* base, int parity, int world, int n) {
  return reinterpret_cast<int32_t*>(base + sizeof(P2pHeader)) + (long long)parity * world * n;
}
__device__ __forceinline__ void st_release_sys(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

// Thread r < world waits until rank r's flag of `parity` in the own buffer reaches `epoch`.  Returns false
// (and flags the status word) when the limit ran out.
__device__ __forceinline__ bool p2p_wait_flag(const unsigned long long* flag, unsigned long long epoch,
                                              unsigned long long wait_ns, int32_t* status) {
  const unsigned long long t0 = global_timer_ns();
  for (uint32_t spins = 0;; ++spins) {
    if (ld_acquire_sys(flag) >= epoch) return true;
    if ((spins & 63u) == 63u && global_timer_ns() - t0 > wait_ns) {
      if (status) atomicOr(status, NVJ_DEV_TIMEOUT);
      return false;
    }
  }
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
  const int parity = (int)(epoch & 1u);
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int32_t v = local[i];
    for (int r = 0; r < world; ++r) p2p_data(peers.base[r], parity, world, n)[rank * n + i] = v;
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < world) {
    st_release_sys(&p2p_header(peers.base[threadIdx.x])->flags[parity][rank], epoch);
    if (!p2p_wait_flag(&own->flags[parity][threadIdx.x], epoch, wait_ns, status)) failed = 1;
  }
  __syncthreads();
  if (failed) return;
  const int32_t* gathered = p2p_data(peers.base[rank], parity, world, n);
  for (int i = threadIdx.x; i < world * n; i += blockDim.x) out[i] = gathered[i];
}

// Waits (bounded) for the oldest published epoch this rank has not collected and copies its data set out.
// Called by all threads of one CTA.  Returns without doing anything when there is no such epoch; on a timeout the
// status word is flagged, nothing is consumed, and a later call tries the same epoch again.
__device__ __forceinline__ void p2p_collect_cta(char* own_base, int n, int world, unsigned long long wait_ns, int32_t* out,
                                                int32_t* status) {
  __shared__ int failed;
  P2pHeader* own = p2p_header(own_base);
  const unsigned long long epoch = *reinterpret_cast<volatile unsigned long long*>(&own->consumed) + 1;
  if (epoch > *reinterpret_cast<volatile unsigned long long*>(&own->published)) return;
  if (threadIdx.x == 0) failed = 0;
  __syncthreads();
  const int parity = (int)(epoch & 1u);
  if ((int)threadIdx.x < world && !p2p_wait_flag(&own->flags[parity][threadIdx.x], epoch, wait_ns, status)) failed = 1;
  __syncthreads();
  if (failed) return;
  const int32_t* gathered = p2p_data(own_base, parity, world, n);
  for (int i = threadIdx.x; i < world * n; i += blockDim.x) out[i] = gathered[i];
  __syncthreads();
  if (threadIdx.x == 0) own->consumed = epoch;
}

// Token pick fused with the publish (and, optionally, with the collect of the step before).  CTA r < n takes the
// argmax of row r (first maximum wins, as row_argmax_kernel) and stores the token locally; CTA n, present when
// collect_out is given, collects the previous epoch.  The CTA that finishes last copies the n tokens into every
// peer's data set with coalesced stores and then publishes the epoch: one system-scope fence per launch, and the
// publish comes after this rank's own collect, which is what lets two data sets suffice.
__global__ void __launch_bounds__(kArgmaxThreads) p2p_argmax_publish_kernel(P2pPeers peers, const float* x, int row_len, int n, int rank,
                                                                            int world, int32_t* tokens, int32_t* collect_out,
                                                                            unsigned long long wait_ns, int32_t* status) {
  P2pHeader* own = p2p_header(peers.base[rank]);
  __shared__ int last_sh;
  if ((int)blockIdx.x < n) {
    const int token = row_argmax_cta(x + (long long)blockIdx.x * row_len, row_len);
    if (threadIdx.x == 0) tokens[blockIdx.x] = token;
  } else {
    p2p_collect_cta(peers.base[rank], n, world, wait_ns, collect_out, status);
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) last_sh = (atomicAdd(&own->arrivals, 1u) == gridDim.x - 1u) ? 1 : 0;
  __syncthreads();
  if (!last_sh) return;
  __threadfence();
  // `published` is advanced here and nowhere else, after every CTA of the launch is done with it
  const unsigned long long epoch = *reinterpret_cast<volatile unsigned long long*>(&own->published) + 1;
  const int parity = (int)(epoch & 1u);
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int32_t v = __ldcg(tokens + i);
    for (int r = 0; r < world; ++r) p2p_data(peers.base[r], parity, world, n)[rank * n + i] = v;
  }
  __threadfence_system();
  __syncthreads();
  if ((int)threadIdx.x < world) st_release_sys(&p2p_header(peers.base[threadIdx.x])->flags[parity][rank], epoch);
  if (threadIdx.x == 0) {
    own->arrivals = 0;
    own->published = epoch;
  }
}

__global__ void __launch_bounds__(kArgmaxThreads) p2p_collect_kernel(char* own_base, int n, int world, unsigned long long wait_ns,
                                                                     int32_t* out, int32_t* status) {
  p2p_collect_cta(own_base, n, world, wait_ns, out, status);
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
  return sizeof(nvj::P2pHeader) + sizeof(int32_t) * 2 * (size_t)world * n;
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
                                      void* const* peer_buffers, int32_t* collect_out, int32_t* status, nvj_stream_t stream) {
  using namespace nvj;
  if (rows < 0 || row_len <= 0) return NVJ_ERR_INVALID_ARGUMENT;
  P2pPeers peers{};
  if (!p2p_args_ok(rank, world, peer_buffers, peers)) return NVJ_ERR_INVALID_ARGUMENT;
  if (rows == 0) return NVJ_OK;
  if (!x || !tokens) return NVJ_ERR_INVALID_ARGUMENT;
  p2p_argmax_publish_kernel<<<rows + (collect_out ? 1 : 0), kArgmaxThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      peers, x, row_len, rows, rank, world, tokens, collect_out, wait_limit_ns(), status);
  return cudaGetLastError() == cudaSuccess ? NVJ_OK : NVJ_ERR_LAUNCH;
}

extern "C" int nvj_p2p_collect(void* own_buffer, int n, int world, int32_t* out, int32_t* status, nvj_stream_t stream) {
  using namespace nvj;
  if (world <= 0 || world > kP2pMaxWorld || n < 0 || !own_buffer) return NVJ_ERR_INVALID_ARGUMENT;
  if (n == 0) return NVJ_OK;
  if (!out) return NVJ_ERR_INVALID_ARGUMENT;
  p2p_collect_kernel<<<1, kArgmaxThreads, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<char*>(own_buffer), n, world,
                                                                                 wait_limit_ns(), out, status);
  return cudaGetLastError() == cudaSuccess ? NVJ_OK : NVJ_ERR_LAUNCH;
}
