#include "common.hpp"
namespace rib200 {
void launch_prefill_attention(const PrefillArgs &, cudaStream_t) {
  unsupported(false, "prefill attention kernel is not built yet");
}
} // namespace rib200
