// placeholder until the tcgen05 kernel lands
#include "launch.cuh"
namespace b2a {
bool sdpa_tc_supported(const b2a_sdpa_desc&, const int64_t (&)[4], const int64_t (&)[4], const int64_t (&)[4],
                       const int64_t (&)[4], const void*, const void*, const void*, const void*) { return false; }
int sdpa_tc_launch(const b2a_sdpa_desc&, const int64_t (&)[4], const int64_t (&)[4], const int64_t (&)[4],
                   const int64_t (&)[4], const void*, const void*, const void*, void*, int32_t*, cudaStream_t) {
    return B2A_ERR_UNSUPPORTED;
}
}  // namespace b2a
