// placeholder until the tensor-core kernel lands in this file
#include "common.cuh"
extern "C" int b200_matmul_tc8_launch(const b200_matmul_params_t *p, b200_stream_t stream) {
    (void)p; (void)stream;
    return B200_ERR_UNSUPPORTED;
}
