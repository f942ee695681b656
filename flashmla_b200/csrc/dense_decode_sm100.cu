// tcgen05 dense decode kernel (placeholder until the kernel lands).
#include "common.cuh"
namespace mla {
bool dense_decode_sm100_supports(const mla_dense_decode_args_t&) { return false; }
int launch_dense_decode_sm100(const mla_dense_decode_args_t&) {
    return set_error(MLA_ERR_UNSUPPORTED, "tcgen05 dense decode kernel is not built");
}
}  // namespace mla
