// Glue between the reference's test driver (tests/benchdnn in the reference tree) and this
// library.  TEST INFRASTRUCTURE: compiled only into the driver binary that oracle/build_benchdnn.py
// builds where the reference tree is present; nothing of the product includes or links it.
//
// The driver is written against the reference's public C API plus a handful of the reference
// library's internals.  The public API is served by libonednn_b200.so itself; the internals the
// matmul driver reaches are answered here:
//   * dnnl::impl::is_pd_in_cache / is_primitive_in_cache / set_primitive_cache_capacity_without_clearing
//     (src/common/primitive_cache.hpp) -> this library's C-ABI forms of the same questions;
//   * dnnl::impl::cpu::platform::* (src/cpu/platform.hpp): properties of the host the driver uses
//     to size its cold-cache buffers and to decide what a CPU engine could run -- this library's
//     host engine computes nothing, so the data-type questions answer "no";
//   * try_cvt_float_to_bfloat16 (src/cpu/bfloat16.cpp, a JIT routine): "not available", which
//     sends src/common/bfloat16.cpp to its portable conversion;
//   * conv_dw_fusion::get_fused_conv_dst_dims (a post-op of the convolution driver that a matmul
//     never carries).
#include <thread>

#include "oneapi/dnnl/dnnl.h"

#include "common/bfloat16.hpp"
#include "common/primitive_cache.hpp"
#include "cpu/platform.hpp"

#include "dnn_types.hpp"

extern "C" dnnl_status_t dnnl_b200_primitive_cache_contains(const_dnnl_primitive_desc_t pd, const_dnnl_primitive_t primitive,
        int *result);
extern "C" dnnl_status_t dnnl_b200_set_primitive_cache_capacity_without_clearing(int capacity);

namespace dnnl {
namespace impl {

bool is_pd_in_cache(const primitive_desc_iface_t *pd) {
    int r = 0;
    return dnnl_b200_primitive_cache_contains((const_dnnl_primitive_desc_t)pd, nullptr, &r) == dnnl_success && r != 0;
}
bool is_primitive_in_cache(const primitive_iface_t *p) {
    int r = 0;
    return dnnl_b200_primitive_cache_contains(nullptr, (const_dnnl_primitive_t)p, &r) == dnnl_success && r != 0;
}
size_t set_primitive_cache_capacity_without_clearing(size_t capacity) {
    int old = 0;
    dnnl_get_primitive_cache_capacity(&old);
    dnnl_b200_set_primitive_cache_capacity_without_clearing((int)capacity);
    return (size_t)old;
}

bool try_cvt_float_to_bfloat16(bfloat16_t *, const float *) {
    return false;
}

namespace cpu {
namespace platform {
bool has_data_type_support(data_type_t) {
    return false;
}
bool has_training_support(data_type_t) {
    return false;
}
unsigned get_per_core_cache_size(int level) {
    return level == 1 ? 48u * 1024 : level == 2 ? 2u * 1024 * 1024 : 4u * 1024 * 1024;
}
unsigned get_num_cores() {
    const unsigned n = std::thread::hardware_concurrency();
    return n ? n : 1;
}
float s8s8_weights_scale_factor() {
    return 1.f;
}
} // namespace platform
} // namespace cpu

} // namespace impl
} // namespace dnnl

namespace conv_dw_fusion {
void get_fused_conv_dst_dims(const int, const attr_t::post_ops_t::entry_t &, const dnnl_dims_t, dnnl_dims_t) {}
} // namespace conv_dw_fusion
