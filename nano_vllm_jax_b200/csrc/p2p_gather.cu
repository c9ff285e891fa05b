// All-gather of each rank's per-step tokens over NVLink peer stores, for one process per GPU on one node.
//
// The only exchange on the path is a few hundred int32 per rank and step; a library all-gather
// spends 7-20 us on it (launch + protocol).  Here every rank owns an exchange buffer that its
// peers map through CUDA IPC.  One single-CTA kernel per rank and step
//   1. stores its tokens into slot `rank` of every peer's buffer (plain peer stores, no multicast),
//   2. publishes them with a system-scope release store of the step's epoch into its flag in every
//      peer's buffer,
//   3. waits, bounded, until the flags of all ranks in its own buffer carry this epoch, and
//   4. copies the gathered tokens out.
// Two data/flag sets alternate by epoch parity: a rank can be at most one step ahead of a peer
// (step k + 1 cannot complete before every peer has published step k + 1, which a peer does only
// after it has consumed step k on its stream), so set (k & 1) is free again at step k + 2.
// The epoch is either passed by the host or (epoch argument 0) kept in the rank's own buffer and advanced by the
// kernel, which makes the launch replayable from a CUDA graph.  The wait has a 1 s limit; on a timeout the kernel flags NVJ_DEV_TIMEOUT and returns.
// The reference is single-device and has no counterpart.

#include <cstring>

#include "nvj_common.cuh"

namespace nvj {

constexpr int kP2pMaxWorld = 16;

struct P2pPeers {
  char* base[kP2pMaxWorld];
};

__device__ __forceinline__ int32_t* p2p_data(char* base, int parity, int world, int n) {
  return reinterpret_cast<int32_t*>(base) + (long long)parity * world * n;
}
__device__ __forceinline__ uint32_t* p2p_flags(char* base, int parity, int world, int n) {
  return reinterpret_cast<uint32_t*>(base) + 2LL * world * n + parity * kP2pMaxWorld;
}

__global__ void __launch_bounds__(256) p2p_allgather_kernel(P2pPeers peers, const int32_t* local, int n, int rank, int world,
                                                           uint32_t epoch, int32_t* out, int32_t* status) {
  __shared__ uint32_t epoch_sh;
  __shared__ int failed;
  if (threadIdx.x == 0) {
    failed = 0;
    if (epoch == 0) {  // epoch kept on the device: the same launch can then be replayed from a CUDA graph
      uint32_t* counter = p2p_flags(peers.base[rank], 0, world, n) + 2 * kP2pMaxWorld;
      epoch = *counter + 1;
      if (epoch == 0) epoch = 2;  // 0 is reserved; 2 keeps the parity sequence alternating after the wrap
      *counter = epoch;
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
    uint32_t* theirs = p2p_flags(peers.base[threadIdx.x], parity, world, n) + rank;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(theirs), "r"(epoch) : "memory");
    const uint32_t* mine = p2p_flags(peers.base[rank], parity, world, n) + threadIdx.x;
    const unsigned long long t0 = global_timer_ns();
    for (uint32_t spins = 0;; ++spins) {
      uint32_t seen;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
      if (seen == epoch) break;
      if ((spins & 63u) == 63u && global_timer_ns() - t0 > kWaitLimitNs) {
        failed = 1;
        if (status) atomicOr(status, NVJ_DEV_TIMEOUT);
        break;
      }
    }
  }
  __syncthreads();
  if (failed) return;
  const int32_t* gathered = p2p_data(peers.base[rank], parity, world, n);
  for (int i = threadIdx.x; i < world * n; i += blockDim.x) out[i] = gathered[i];
}

}  // namespace nvj

extern "C" size_t nvj_p2p_gather_buffer_bytes(int world, int n) {
  if (world <= 0 || world > nvj::kP2pMaxWorld || n < 0) return 0;
  return sizeof(int32_t) * 2 * (size_t)world * n + sizeof(uint32_t) * (2 * nvj::kP2pMaxWorld + 4);  // data, flags, epoch counter
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
  if (world <= 0 || world > kP2pMaxWorld || rank < 0 || rank >= world || n < 0) return NVJ_ERR_INVALID_ARGUMENT;
  if (n == 0) return NVJ_OK;
  if (!local || !peer_buffers || !out) return NVJ_ERR_INVALID_ARGUMENT;
  P2pPeers peers{};
  for (int r = 0; r < world; ++r) {
    if (!peer_buffers[r]) return NVJ_ERR_INVALID_ARGUMENT;
    peers.base[r] = static_cast<char*>(peer_buffers[r]);
  }
  p2p_allgather_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(peers, local, n, rank, world, epoch, out, status);
  return cudaGetLastError() == cudaSuccess ? NVJ_OK : NVJ_ERR_LAUNCH;
}
