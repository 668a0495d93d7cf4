// Grouped expert projections on tcgen05.  Placeholder translation unit: until the grouped
// tensor-core kernel is in place every shape goes to the portable kernels in moe.cu.
#include "common.cuh"

namespace nml_sm100 {

bool experts_umma_supported(const ExpertArgs&) { return false; }

int32_t launch_experts_umma(const ExpertArgs&, const DeviceInfo&, char* message,
                            size_t capacity) {
  return fail(NML_SM100_LAUNCH_FAILURE, "the tcgen05 expert kernel is not built", message,
              capacity);
}

}  // namespace nml_sm100
