// SageSLA quantized forward (placeholder translation unit until the kernels land).
#include "common.cuh"
#include "kernels.h"
#include "workspace.h"

extern "C" int sage_sla_fwd(const sla_shape*, const void*, const void*, const void*, const int32_t*,
                            const float*, const float*, void*, void*, void*, size_t, sla_stream_t) {
  return SLA_ERR_UNSUPPORTED;
}
