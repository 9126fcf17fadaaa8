// Generic matmul kernel: one thread per destination element, scalar loop over
// K.  It accepts everything the reference's two scalar implementations accept
// (any strides, every scale / zero-point mask and group size, every post-op)
// and performs the same operations in the same order, so its results are
// bit-identical to theirs.  It is the engine's fallback implementation
// ("cuda:generic") and the on-device yardstick for the fast kernels.
//   int8 sources:  src/cpu/matmul/ref_matmul_int8.cpp:154-261
//   other sources: src/cpu/matmul/ref_matmul.cpp:130-233
#include "common.cuh"
#include "launch.hpp"

namespace b200 {

__global__ void __launch_bounds__(256) matmul_generic_kernel(const __grid_constant__ b200_matmul_params_t p) {
    const int64_t total = p.M * p.N;
    const bool int8_path = p.src_dt == B200_DT_S8 || p.src_dt == B200_DT_U8;
    const float dst_inv = dst_scale_reciprocal(p);
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
            idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t m = idx / p.N, n = idx % p.N;
        float d;
        if (int8_path) {
            // The reference cuts the K loop into the smallest group among the four scale /
            // zero-point arguments, and an argument without explicit groups (set or not)
            // counts as group size 1 (ref_matmul_int8.cpp:83-144,
            // primitive_attr_quant.hpp:83-90): unless every argument is explicitly
            // grouped, each product is converted to f32, scaled and accumulated in f32.
            int64_t ng = 1;
            {
                const int64_t a = (p.src_zp.ptr && p.src_zp.g1 > 1) ? p.K / p.src_zp.g1 : p.K;
                const int64_t b = (p.wei_zp.ptr && p.wei_zp.g0 > 1) ? p.K / p.wei_zp.g0 : p.K;
                const int64_t c = (p.src_scale.ptr && p.src_scale.g1 > 1) ? p.K / p.src_scale.g1 : p.K;
                const int64_t e = (p.wei_scale.ptr && p.wei_scale.g0 > 1) ? p.K / p.wei_scale.g0 : p.K;
                ng = a > b ? a : b;
                ng = c > ng ? c : ng;
                ng = e > ng ? e : ng;
            }
            const int64_t gk = p.K / ng;
            d = 0.f;
            for (int64_t g = 0; g < ng; ++g) {
                int acc = 0;
                for (int64_t kk = 0; kk < gk; ++kk) {
                    const int64_t k = g * gk + kk;
                    int s = load_int(p.src_dt, p.src, m * p.src_sm + k * p.src_sk);
                    int w = load_int(p.wei_dt, p.wei, k * p.wei_sk + n * p.wei_sn);
                    if (p.src_zp.ptr) s -= load_int(p.src_zp.dt, p.src_zp.ptr, quant_off(p.src_zp, m, k));
                    if (p.wei_zp.ptr) w -= load_int(p.wei_zp.dt, p.wei_zp.ptr, quant_off(p.wei_zp, k, n));
                    acc += s * w;
                }
                float a = (float)acc;
                if (p.src_scale.ptr)
                    a = __fmul_rn(a, load_f32(p.src_scale.dt, p.src_scale.ptr, quant_off(p.src_scale, m, g * gk)));
                if (p.wei_scale.ptr)
                    a = __fmul_rn(a, load_f32(p.wei_scale.dt, p.wei_scale.ptr, quant_off(p.wei_scale, g * gk, n)));
                d = __fadd_rn(d, a);
            }
        } else {
            const bool decomp = dt_is_int(p.wei_dt) && p.wei_dt != B200_DT_S32 && p.apply_to_int;
            float acc = 0.f;
            for (int64_t k = 0; k < p.K; ++k) {
                const float s = load_f32(p.src_dt, p.src, m * p.src_sm + k * p.src_sk);
                float w = load_f32(p.wei_dt, p.wei, k * p.wei_sk + n * p.wei_sn);
                if (decomp) {
                    if (p.wei_zp.ptr)
                        w = __fsub_rn(w, (float)load_int(p.wei_zp.dt, p.wei_zp.ptr, quant_off(p.wei_zp, k, n)));
                    if (p.wei_scale.ptr)
                        w = __fmul_rn(w, load_f32(p.wei_scale.dt, p.wei_scale.ptr, quant_off(p.wei_scale, k, n)));
                }
                acc = __fadd_rn(acc, __fmul_rn(s, w));
            }
            d = acc;
            if (p.src_scale.ptr) d = __fmul_rn(d, load_f32(p.src_scale.dt, p.src_scale.ptr, 0));
            if (p.wei_scale.ptr && !decomp)
                d = __fmul_rn(d, load_f32(p.wei_scale.dt, p.wei_scale.ptr, quant_off(p.wei_scale, 0, n)));
        }
        finish_element(p, d, m, n, int8_path, dst_inv);
    }
}

} // namespace b200

extern "C" int b200_matmul_generic_launch(const b200_matmul_params_t *p, b200_stream_t stream) {
    if (!p || !p->src || !p->wei || !p->dst) return B200_ERR_BAD_ARG;
    if (p->M < 0 || p->N < 0 || p->K < 0 || p->npo < 0 || p->npo > B200_MAX_POSTOPS) return B200_ERR_BAD_ARG;
    if (p->M == 0 || p->N == 0 || p->K == 0) return 0; // a zero dim: dst is left untouched
    if (p->wei_layout != B200_WEI_PLAIN || p->n_dst_peers) return B200_ERR_UNSUPPORTED;
    const int64_t total = p->M * p->N;
    int64_t blocks = (total + 255) / 256;
    if (blocks > 148 * 64) blocks = 148 * 64;
    b200::matmul_generic_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(*p);
    return b200::after_launch();
}
