// Tensor-core (tcgen05 / TMEM) appearance MLP -- placeholder until the kernel lands.
#include "gnr_internal.cuh"

int gnr_mlp_tc_prepare(GnrModel*, const float*, const float*, const float*, const float*, const float*, const float*,
                       cudaStream_t) {
  gnr_set_error("mlp_mode != 0 (tensor-core MLP) is not available in this build");
  return -1;
}

int launch_mlp_tc(const GnrModel*, const GnrSampleParams&, const float*, char*, const GnrWs&, int64_t, cudaStream_t) {
  gnr_set_error("mlp_mode != 0 (tensor-core MLP) is not available in this build");
  return -1;
}
