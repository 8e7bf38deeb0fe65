// Plumbing for the head-sharded prefill across the GPUs of one box: device memory that other processes can map
// (CUDA IPC), and a device-side rendezvous of the ranks through flag words in that memory.  The reference has
// nothing like it (its runtime is single-GPU); the entry points are declared as additive in include/rib200.h.

#include "common.hpp"

#include <cuda_runtime.h>

#include <cstdint>
#include <cstring>

namespace rib200 {

constexpr long long kRendezvousLimitCycles = 1LL << 31; // about a second

namespace {

struct RendezvousParams {
  std::uint32_t *flags[8];
  std::uint32_t world;
  std::uint32_t rank;
  std::uint32_t epoch;
  unsigned int *status;
  long long limit_cycles;
};

// One warp.  Lane r < world publishes this rank's epoch in rank r's array, then waits for rank r's epoch in this
// rank's own array.  The kernels before this one on the stream have completed, so their peer stores are visible
// before the flag is.
__global__ void peer_rendezvous_kernel(const RendezvousParams p) {
  const std::uint32_t lane = threadIdx.x;
  if (lane >= p.world) {
    return;
  }
  __threadfence_system();
  volatile std::uint32_t *theirs = p.flags[lane] + p.rank;
  *theirs = p.epoch;
  __threadfence_system();
  volatile std::uint32_t *mine = p.flags[p.rank] + lane;
  const long long started = clock64();
  // epochs are compared as a signed difference, so they may wrap
  while (static_cast<std::int32_t>(*mine - p.epoch) < 0) {
    if (clock64() - started > p.limit_cycles) {
      atomicOr(p.status, static_cast<unsigned int>(RIB200_DEVICE_WAIT_TIMED_OUT));
      return;
    }
  }
  __threadfence_system();
}

} // namespace

void launch_peer_rendezvous(std::uint32_t *const *flags, std::uint32_t world, std::uint32_t rank, std::uint32_t epoch,
                            cudaStream_t stream, long long limit_cycles) {
  RendezvousParams p{};
  for (std::uint32_t r = 0; r < world; ++r) {
    p.flags[r] = flags[r];
  }
  p.world = world;
  p.rank = rank;
  p.epoch = epoch;
  p.status = device_status_word();
  p.limit_cycles = limit_cycles > 0 ? limit_cycles : kRendezvousLimitCycles;
  peer_rendezvous_kernel<<<1, 32, 0, stream>>>(p);
  cuda_ok(cudaGetLastError(), "peer rendezvous launch");
}

} // namespace rib200

using namespace rib200;

extern "C" Rib200Status rib200_peer_rendezvous_bounded(uint32_t *const *flags, size_t world, size_t rank,
                                                       uint32_t epoch, uint64_t limit_cycles, void *stream) {
  return guarded([&] {
    require(limit_cycles >= 1 && limit_cycles <= (1ULL << 40), "peer rendezvous: limit_cycles is out of range");
    require(flags != nullptr, "peer rendezvous: flag array list is null");
    require(world >= 1 && world <= 8, "peer rendezvous: world must be between 1 and 8");
    require(rank < world, "peer rendezvous: rank is out of range");
    require(stream != nullptr, "peer rendezvous: CUDA stream is null");
    for (std::size_t r = 0; r < world; ++r) {
      require(flags[r] != nullptr, "peer rendezvous: a flag array is null");
    }
    launch_peer_rendezvous(flags, static_cast<std::uint32_t>(world), static_cast<std::uint32_t>(rank), epoch,
                           static_cast<cudaStream_t>(stream), static_cast<long long>(limit_cycles));
  });
}

extern "C" Rib200Status rib200_peer_rendezvous(uint32_t *const *flags, size_t world, size_t rank, uint32_t epoch,
                                               void *stream) {
  return rib200_peer_rendezvous_bounded(flags, world, rank, epoch, static_cast<uint64_t>(kRendezvousLimitCycles),
                                        stream);
}

extern "C" Rib200Status rib200_shared_alloc(size_t bytes, void **pointer, uint8_t handle[64]) {
  return guarded([&] {
    require(pointer != nullptr && handle != nullptr, "shared alloc: output pointer is null");
    require(bytes > 0, "shared alloc: size must be positive");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    void *ptr = nullptr;
    cuda_ok(cudaMalloc(&ptr, bytes), "shared alloc: cudaMalloc");
    cudaIpcMemHandle_t ipc{};
    cudaError_t err = cudaMemset(ptr, 0, bytes);
    if (err == cudaSuccess) {
      err = cudaDeviceSynchronize();
    }
    if (err == cudaSuccess) {
      err = cudaIpcGetMemHandle(&ipc, ptr);
    }
    if (err != cudaSuccess) {
      cudaFree(ptr);
      cuda_ok(err, "shared alloc: handle export");
    }
    std::memcpy(handle, &ipc, 64);
    *pointer = ptr;
  });
}

extern "C" Rib200Status rib200_shared_open(const uint8_t handle[64], void **pointer) {
  return guarded([&] {
    require(pointer != nullptr && handle != nullptr, "shared open: pointer is null");
    cudaIpcMemHandle_t ipc{};
    std::memcpy(&ipc, handle, 64);
    void *ptr = nullptr;
    cuda_ok(cudaIpcOpenMemHandle(&ptr, ipc, cudaIpcMemLazyEnablePeerAccess), "shared open: cudaIpcOpenMemHandle");
    *pointer = ptr;
  });
}

extern "C" Rib200Status rib200_shared_close(void *pointer) {
  return guarded([&] {
    require(pointer != nullptr, "shared close: pointer is null");
    cuda_ok(cudaIpcCloseMemHandle(pointer), "shared close: cudaIpcCloseMemHandle");
  });
}

extern "C" Rib200Status rib200_shared_free(void *pointer) {
  return guarded([&] {
    require(pointer != nullptr, "shared free: pointer is null");
    cuda_ok(cudaFree(pointer), "shared free: cudaFree");
  });
}
