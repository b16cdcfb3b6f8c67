// Peer-memory plumbing for the sequence-parallel (Ulysses) path on one NVSwitch box:
//   * an exchange arena per rank, allocated once with cudaMalloc and shared with the other
//     ranks' processes through CUDA IPC handles, so that the q/k/v assembly kernel and the
//     attention kernel can store their results straight into the consuming rank's memory;
//   * a signal / wait pair of one-warp kernels that orders those stores between GPUs through
//     flags in the arenas (epoch counters, release/acquire at system scope, bounded waits).
// No load ever targets peer memory and no TMA instruction touches it: peers are only written
// with plain global stores.  The reference has no multi-GPU path; nothing here has a
// counterpart in it.
#include <string.h>

#include "common.cuh"

namespace fluxb {
namespace peer {

constexpr int MAX_RANKS = 8;
constexpr int BARRIERS = 2;
// Arena header (first 512 bytes): flags[BARRIERS][MAX_RANKS] written by the peers, then this
// rank's own epoch counters.
constexpr int FLAGS_OFFSET = 0;
constexpr int SIGNAL_EPOCH_OFFSET = 256;
constexpr int WAIT_EPOCH_OFFSET = 256 + 4 * BARRIERS;

struct PeerFlags {
  uint32_t* flag[MAX_RANKS];  // address of this rank's slot in every rank's flag array
};

__device__ __forceinline__ void store_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t load_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Tells every rank that everything this rank's stream ran before this kernel is done.
__global__ void signal_kernel(PeerFlags peers, int n_ranks, uint32_t* epoch) {
  uint32_t e = 0;
  if (threadIdx.x == 0) {
    e = *epoch + 1;
    *epoch = e;
  }
  e = __shfl_sync(0xffffffffu, e, 0);
  __threadfence_system();
  if ((int)threadIdx.x < n_ranks) store_release_sys(peers.flag[threadIdx.x], e);
}

// Returns once every rank has signalled this barrier as often as this rank has waited on it.
__global__ void wait_kernel(const uint32_t* flags, int n_ranks, uint32_t* epoch, DeviceStatus* status, int where) {
  uint32_t e = 0;
  if (threadIdx.x == 0) {
    e = *epoch + 1;
    *epoch = e;
  }
  e = __shfl_sync(0xffffffffu, e, 0);
  if ((int)threadIdx.x < n_ranks) {
    const uint64_t t0 = global_timer_ns();
    uint32_t spins = 0;
    while ((int32_t)(load_acquire_sys(flags + threadIdx.x) - e) < 0) {
      if ((++spins & 0xffu) == 0 && global_timer_ns() - t0 > FLUXB_WAIT_LIMIT_NS) {
        report_error(status, FLUXB_ERR_TIMEOUT, where);
        break;
      }
    }
  }
  __threadfence_system();
}

}  // namespace peer
}  // namespace fluxb

using namespace fluxb;

extern "C" int fluxb_peer_header_bytes(void) { return 512; }

extern "C" int fluxb_peer_alloc(int64_t bytes, void** ptr) {
  if (!ptr || bytes < 512) return set_error(FLUXB_ERR_BAD_ARG, "peer_alloc: need an output pointer and at least the 512-byte header");
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, (size_t)bytes);
  if (e != cudaSuccess) return set_error(FLUXB_ERR_CUDA, "peer_alloc: cudaMalloc(%lld): %s", (long long)bytes, cudaGetErrorString(e));
  e = cudaMemset(p, 0, (size_t)bytes);
  if (e != cudaSuccess) {
    cudaFree(p);
    return set_error(FLUXB_ERR_CUDA, "peer_alloc: cudaMemset: %s", cudaGetErrorString(e));
  }
  *ptr = p;
  return FLUXB_OK;
}

extern "C" int fluxb_peer_free(void* ptr) {
  if (!ptr) return FLUXB_OK;
  cudaError_t e = cudaFree(ptr);
  if (e != cudaSuccess) return set_error(FLUXB_ERR_CUDA, "peer_free: %s", cudaGetErrorString(e));
  return FLUXB_OK;
}

extern "C" int fluxb_peer_export(const void* ptr, void* handle64) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  if (!ptr || !handle64) return set_error(FLUXB_ERR_BAD_ARG, "peer_export: null pointer");
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, const_cast<void*>(ptr));
  if (e != cudaSuccess) return set_error(FLUXB_ERR_CUDA, "peer_export: cudaIpcGetMemHandle: %s", cudaGetErrorString(e));
  memcpy(handle64, &h, 64);
  return FLUXB_OK;
}

extern "C" int fluxb_peer_open(const void* handle64, void** ptr) {
  if (!ptr || !handle64) return set_error(FLUXB_ERR_BAD_ARG, "peer_open: null pointer");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return set_error(FLUXB_ERR_CUDA, "peer_open: cudaIpcOpenMemHandle: %s", cudaGetErrorString(e));
  *ptr = p;
  return FLUXB_OK;
}

extern "C" int fluxb_peer_close(void* ptr) {
  if (!ptr) return FLUXB_OK;
  cudaError_t e = cudaIpcCloseMemHandle(ptr);
  if (e != cudaSuccess) return set_error(FLUXB_ERR_CUDA, "peer_close: %s", cudaGetErrorString(e));
  return FLUXB_OK;
}

static int check_barrier_args(const void* const* arenas, int n_ranks, int rank, int barrier, const char* what) {
  using namespace fluxb::peer;
  if (!arenas || n_ranks < 1 || n_ranks > MAX_RANKS || rank < 0 || rank >= n_ranks || barrier < 0 || barrier >= BARRIERS)
    return set_error(FLUXB_ERR_BAD_ARG, "%s: need 1..%d ranks, a rank among them and barrier 0..%d", what, MAX_RANKS, BARRIERS - 1);
  for (int i = 0; i < n_ranks; ++i)
    if (!arenas[i] || (reinterpret_cast<uintptr_t>(arenas[i]) & 255))
      return set_error(FLUXB_ERR_BAD_ARG, "%s: arena %d is null or not 256-byte aligned", what, i);
  return FLUXB_OK;
}

extern "C" int fluxb_peer_signal(const void* const* arenas, int n_ranks, int rank, int barrier,
                                 fluxb_stream_t stream) {
  using namespace fluxb::peer;
  int rc = check_barrier_args(arenas, n_ranks, rank, barrier, "peer_signal");
  if (rc != FLUXB_OK) return rc;
  PeerFlags pf;
  for (int i = 0; i < MAX_RANKS; ++i) pf.flag[i] = nullptr;
  for (int i = 0; i < n_ranks; ++i) {
    uint8_t* a = static_cast<uint8_t*>(const_cast<void*>(arenas[i]));
    pf.flag[i] = reinterpret_cast<uint32_t*>(a + FLAGS_OFFSET) + barrier * MAX_RANKS + rank;
  }
  uint8_t* mine = static_cast<uint8_t*>(const_cast<void*>(arenas[rank]));
  uint32_t* epoch = reinterpret_cast<uint32_t*>(mine + SIGNAL_EPOCH_OFFSET) + barrier;
  signal_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(pf, n_ranks, epoch);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(FLUXB_ERR_CUDA, "peer_signal: launch failed: %s", cudaGetErrorString(e));
  return FLUXB_OK;
}

extern "C" int fluxb_peer_wait(const void* const* arenas, int n_ranks, int rank, int barrier,
                               fluxb_stream_t stream) {
  using namespace fluxb::peer;
  int rc = check_barrier_args(arenas, n_ranks, rank, barrier, "peer_wait");
  if (rc != FLUXB_OK) return rc;
  uint8_t* mine = static_cast<uint8_t*>(const_cast<void*>(arenas[rank]));
  const uint32_t* flags = reinterpret_cast<const uint32_t*>(mine + FLAGS_OFFSET) + barrier * MAX_RANKS;
  uint32_t* epoch = reinterpret_cast<uint32_t*>(mine + WAIT_EPOCH_OFFSET) + barrier;
  wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(flags, n_ranks, epoch, device_status_ptr(), 61 + barrier);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(FLUXB_ERR_CUDA, "peer_wait: launch failed: %s", cudaGetErrorString(e));
  return FLUXB_OK;
}
