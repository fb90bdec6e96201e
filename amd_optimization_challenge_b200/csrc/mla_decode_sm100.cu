// tcgen05 / TMEM stage-1 kernel (placeholder until the kernel lands: reports "not applicable").
#include "mla_common.cuh"

namespace b200mla {

bool sm100_supported(const MlaParams&) { return false; }
int sm100_rows_per_cta(const MlaParams&) { return 16; }
cudaError_t launch_sm100(const MlaParams&, cudaStream_t) { return cudaErrorNotSupported; }

}  // namespace b200mla
