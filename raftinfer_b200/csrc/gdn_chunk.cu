#include "common.hpp"
namespace rib200 {
std::size_t gdn_chunk_workspace_bytes(std::size_t, std::size_t, std::size_t) { return 0; }
void launch_gdn_chunked(const GdnCoreArgs &args, void *, cudaStream_t stream) { launch_gdn_recurrent(args, stream); }
} // namespace rib200
