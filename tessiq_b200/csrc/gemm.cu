// GEMM + bias + activation. Placeholder until the tcgen05 kernel lands: every call declines.
#include "common.h"

extern "C" tq_status tq_gemm_bias_act_launch(tq_dtype, tq_activation, const void*, int64_t, int32_t,
                                             const void*, int64_t, int32_t, const void*, void*, int64_t,
                                             int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t,
                                             int32_t, void*) {
  return tq::fail(TQ_UNSUPPORTED, "the GEMM kernel is not built yet");
}
