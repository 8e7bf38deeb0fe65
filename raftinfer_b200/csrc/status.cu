// Status plumbing of librib200: the thread-local message buffer behind Rib200Status and the
// per-device status word that kernels set instead of trapping
// (the reference traps at cpp/kernels/qwen35_online_attention.cu:714-717).

#include "common.hpp"

#include <cuda_runtime.h>

#include <mutex>

namespace rib200 {
namespace {

__device__ unsigned int g_device_status = 0;

thread_local std::string t_message;

} // namespace

Rib200Status ok_status() { return Rib200Status{RIB200_STATUS_OK, ""}; }

Rib200Status fail_status(int32_t code, const std::string &message) {
  t_message = message;
  return Rib200Status{code, t_message.c_str()};
}

unsigned int *device_status_word() {
  static std::mutex lock;
  static unsigned int *address[64] = {};
  int device = 0;
  cuda_ok(cudaGetDevice(&device), "cudaGetDevice");
  require(device >= 0 && device < 64, "device ordinal out of range", RIB200_STATUS_INTERNAL);
  std::lock_guard<std::mutex> guard(lock);
  if (address[device] == nullptr) {
    void *ptr = nullptr;
    cuda_ok(cudaGetSymbolAddress(&ptr, g_device_status), "status word address");
    address[device] = static_cast<unsigned int *>(ptr);
  }
  return address[device];
}

} // namespace rib200

extern "C" Rib200Status rib200_device_status(void *stream, uint32_t *bits) {
  return rib200::guarded([&] {
    rib200::require(bits != nullptr, "status output pointer is null");
    rib200::require(stream != nullptr, "CUDA stream is null");
    auto *s = static_cast<cudaStream_t>(stream);
    unsigned int *word = rib200::device_status_word();
    unsigned int host = 0;
    rib200::cuda_ok(cudaMemcpyAsync(&host, word, sizeof(host), cudaMemcpyDeviceToHost, s), "status read");
    rib200::cuda_ok(cudaMemsetAsync(word, 0, sizeof(host), s), "status clear");
    rib200::cuda_ok(cudaStreamSynchronize(s), "status synchronize");
    *bits = host;
  });
}

extern "C" const char *rib200_version(void) { return "rib200 0.1 sm_100a"; }
