// placeholder until the tcgen05 kernel lands
#include "common.cuh"
namespace caifq
{
bool umma_supported(const LinearArgs &) { return false; }
int launch_linear_umma(const LinearArgs &, cudaStream_t)
{
  set_error("umma path not built");
  return CAIFQ_ERR_UNSUPPORTED;
}
}  // namespace caifq
