// Device-side numerics shared by every kernel of the matmul path: typed loads
// and stores, the eltwise / binary formulas, and the epilogue
//   bias -> post-ops -> dst scale -> dst zero-point -> saturate + round-to-nearest-even
// in the exact operation order of the reference's scalar implementations
// (src/cpu/matmul/ref_matmul_int8.cpp:234-261, src/cpu/matmul/ref_matmul.cpp:196-231,
//  src/cpu/primitive_attr_postops.cpp:278-347, src/cpu/ref_io_helper.hpp:33-154,
//  src/cpu/simple_q10n.hpp:33-81, src/common/math_utils.hpp:134-420).
//
// Every f32 operation is written with a round-to-nearest intrinsic
// (__fmul_rn / __fadd_rn / __fdiv_rn) so that the compiler cannot contract a
// multiply and an add into one FMA: integer destinations are then a bit-exact
// function of the s32 accumulator, identical to the CPU result.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "onednn_b200_kernels.h"

namespace b200 {

// dnnl_alg_kind_t values (include/oneapi/dnnl/dnnl_types.h:2043-2110 in the reference)
enum : int {
    ALG_RELU = 0x20, ALG_TANH = 0x21, ALG_ELU = 0x22, ALG_SQUARE = 0x23, ALG_ABS = 0x24, ALG_SQRT = 0x25,
    ALG_LINEAR = 0x26, ALG_SOFT_RELU = 0x27, ALG_HARDSIGMOID = 0x28, ALG_LOGISTIC = 0x29, ALG_EXP = 0x2a,
    ALG_GELU_TANH = 0x2b, ALG_SWISH = 0x2c, ALG_LOG = 0x2d, ALG_CLIP = 0x2e, ALG_CLIP_V2 = 0x2f,
    ALG_POW = 0x30, ALG_GELU_ERF = 0x31, ALG_ROUND = 0x32, ALG_MISH = 0x33, ALG_HARDSWISH = 0x34,
    ALG_RELU_DST = 0x100, ALG_TANH_DST = 0x101, ALG_ELU_DST = 0x102, ALG_SQRT_DST = 0x103,
    ALG_LOGISTIC_DST = 0x104, ALG_EXP_DST = 0x105, ALG_CLIP_V2_DST = 0x106,
    ALG_BIN_ADD = 0x1fff0, ALG_BIN_MUL = 0x1fff1, ALG_BIN_MAX = 0x1fff2, ALG_BIN_MIN = 0x1fff3,
    ALG_BIN_DIV = 0x1fff4, ALG_BIN_SUB = 0x1fff5, ALG_BIN_GE = 0x1fff6, ALG_BIN_GT = 0x1fff7,
    ALG_BIN_LE = 0x1fff8, ALG_BIN_LT = 0x1fff9, ALG_BIN_EQ = 0x1fffa, ALG_BIN_NE = 0x1fffb,
    ALG_BIN_SELECT = 0x1fffc
};

__host__ __device__ inline bool dt_is_int(int dt) {
    return dt == B200_DT_S32 || dt == B200_DT_S8 || dt == B200_DT_U8 || dt == B200_DT_S4 || dt == B200_DT_U4;
}
__host__ __device__ inline int dt_bits(int dt) {
    switch (dt) {
        case B200_DT_F32: case B200_DT_S32: return 32;
        case B200_DT_F16: case B200_DT_BF16: return 16;
        case B200_DT_S8: case B200_DT_U8: case B200_DT_F8_E4M3: case B200_DT_F8_E5M2: return 8;
        case B200_DT_S4: case B200_DT_U4: return 4;
        default: return 0;
    }
}

// ---- typed loads -----------------------------------------------------------

__device__ __forceinline__ float e4m3_to_f32(uint8_t raw) {
    __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)raw, __NV_E4M3);
    return __half2float(__half(h));
}
__device__ __forceinline__ float e5m2_to_f32(uint8_t raw) {
    __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)raw, __NV_E5M2);
    return __half2float(__half(h));
}

// 4-bit types: two values per byte, even index in the low nibble
__device__ __forceinline__ int load_int(int dt, const void *ptr, int64_t idx) {
    switch (dt) {
        case B200_DT_S32: return ((const int32_t *)ptr)[idx];
        case B200_DT_S8: return ((const int8_t *)ptr)[idx];
        case B200_DT_U8: return ((const uint8_t *)ptr)[idx];
        case B200_DT_S4: {
            uint32_t b = ((const uint8_t *)ptr)[idx >> 1];
            int v = (idx & 1) ? (b >> 4) : (b & 0xf);
            return (v & 8) ? v - 16 : v;
        }
        case B200_DT_U4: {
            uint32_t b = ((const uint8_t *)ptr)[idx >> 1];
            return (idx & 1) ? (b >> 4) : (b & 0xf);
        }
        default: return 0x7fffffff;
    }
}

__device__ __forceinline__ float load_f32(int dt, const void *ptr, int64_t idx) {
    switch (dt) {
        case B200_DT_F32: return ((const float *)ptr)[idx];
        case B200_DT_BF16: return __uint_as_float((uint32_t)((const uint16_t *)ptr)[idx] << 16);
        case B200_DT_F16: return __half2float(((const __half *)ptr)[idx]);
        case B200_DT_F8_E4M3: return e4m3_to_f32(((const uint8_t *)ptr)[idx]);
        case B200_DT_F8_E5M2: return e5m2_to_f32(((const uint8_t *)ptr)[idx]);
        default: return (float)load_int(dt, ptr, idx);
    }
}

// ---- typed stores ----------------------------------------------------------

// f32 -> bf16, round to nearest even; f32 denormals become signed zero as in
// the reference's conversion (src/common/bfloat16.cpp:22-51)
__device__ __forceinline__ uint16_t f32_to_bf16_bits(float v) {
    uint32_t u = __float_as_uint(v);
    uint32_t e = (u >> 23) & 0xff;
    if (e == 0) return (uint16_t)((u >> 16) & 0x8000);
    if (e == 0xff) return (uint16_t)((u & 0x7fffff) ? ((u >> 16) | 0x40) : (u >> 16));
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

// f32 -> e4m3 through f16 (two roundings, overflow above 464 gives NaN 0x7f),
// as src/common/float8.cpp:96-147 does
__device__ __forceinline__ uint8_t f32_to_e4m3_bits(float v) {
    __half h = __float2half_rn(v);
    return (uint8_t)__nv_cvt_halfraw_to_fp8(__half_raw(h), __NV_NOSAT, __NV_E4M3);
}
__device__ __forceinline__ uint8_t f32_to_e5m2_bits(float v) {
    __half h = __float2half_rn(v);
    return (uint8_t)__nv_cvt_halfraw_to_fp8(__half_raw(h), __NV_NOSAT, __NV_E5M2);
}

// integer destinations: clamp in f32, then round to nearest even, then narrow.
// Comparisons (not fmaxf/fminf) so that NaN passes through the clamp as on the
// CPU, where it then converts to INT_MIN: low byte 0 for s8/u8.
__device__ __forceinline__ int sat_rne_s8(float v) {
    v = v < -128.f ? -128.f : v;
    v = v > 127.f ? 127.f : v;
    return __float2int_rn(v);
}
__device__ __forceinline__ int sat_rne_u8(float v) {
    v = v < 0.f ? 0.f : v;
    v = v > 255.f ? 255.f : v;
    return __float2int_rn(v);
}
__device__ __forceinline__ int sat_rne_s32(float v) {
    if (v != v) return (int)0x80000000;
    v = v < -2147483648.f ? -2147483648.f : v;
    v = v > 2147483520.f ? 2147483520.f : v;
    return __float2int_rn(v);
}

// f32 -> s8 / u8: round to nearest even and saturate in one instruction.  Rounding and
// clamping to integer bounds commute, so this equals the reference's clamp-then-round; NaN
// gives 0 in both.  The result is the byte, zero-extended.
__device__ __forceinline__ uint32_t cvt_sat_s8(float v) {
    int r;
    asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(r) : "f"(v));
    return (uint32_t)r & 0xffu;
}
__device__ __forceinline__ uint32_t cvt_sat_u8(float v) {
    uint32_t r;
    asm("cvt.rni.sat.u8.f32 %0, %1;" : "=r"(r) : "f"(v));
    return r & 0xffu;
}

__device__ __forceinline__ void store_f32(int dt, float v, void *ptr, int64_t idx) {
    switch (dt) {
        case B200_DT_F32: ((float *)ptr)[idx] = v; break;
        case B200_DT_BF16: ((uint16_t *)ptr)[idx] = f32_to_bf16_bits(v); break;
        case B200_DT_F16: ((__half *)ptr)[idx] = __float2half_rn(v); break;
        case B200_DT_F8_E4M3: ((uint8_t *)ptr)[idx] = f32_to_e4m3_bits(v); break;
        case B200_DT_F8_E5M2: ((uint8_t *)ptr)[idx] = f32_to_e5m2_bits(v); break;
        case B200_DT_S32: ((int32_t *)ptr)[idx] = sat_rne_s32(v); break;
        case B200_DT_S8: ((int8_t *)ptr)[idx] = (int8_t)sat_rne_s8(v); break;
        case B200_DT_U8: ((uint8_t *)ptr)[idx] = (uint8_t)sat_rne_u8(v); break;
        default: break;
    }
}

// ---- portable tanh ---------------------------------------------------------
// Double-precision tanh made of + - * / only, each rounded to nearest, in a
// fixed order; the CPU side of the tests runs the same sequence, so float
// results agree bit for bit.  |error| ~ 1e-15, i.e. its float rounding is the
// correctly rounded tanhf except on near-ties.
__device__ __forceinline__ double exp_portable(double y) { // y in [0, 40]
    const double log2e = 1.4426950408889634074;
    const double ln2_hi = 6.93147180369123816490e-01;
    const double ln2_lo = 1.90821492927058770002e-10;
    double t = __dadd_rn(__dmul_rn(y, log2e), 0.5);
    long long n = (long long)t;
    double dn = (double)n;
    double r = __dsub_rn(__dsub_rn(y, __dmul_rn(dn, ln2_hi)), __dmul_rn(dn, ln2_lo));
    double p = 1.0 / 6227020800.0;
    p = __dadd_rn(__dmul_rn(p, r), 1.0 / 479001600.0);
    p = __dadd_rn(__dmul_rn(p, r), 1.0 / 39916800.0);
    p = __dadd_rn(__dmul_rn(p, r), 1.0 / 3628800.0);
    p = __dadd_rn(__dmul_rn(p, r), 1.0 / 362880.0);
    p = __dadd_rn(__dmul_rn(p, r), 1.0 / 40320.0);
    p = __dadd_rn(__dmul_rn(p, r), 1.0 / 5040.0);
    p = __dadd_rn(__dmul_rn(p, r), 1.0 / 720.0);
    p = __dadd_rn(__dmul_rn(p, r), 1.0 / 120.0);
    p = __dadd_rn(__dmul_rn(p, r), 1.0 / 24.0);
    p = __dadd_rn(__dmul_rn(p, r), 1.0 / 6.0);
    p = __dadd_rn(__dmul_rn(p, r), 0.5);
    p = __dadd_rn(__dmul_rn(p, r), 1.0);
    p = __dadd_rn(__dmul_rn(p, r), 1.0);
    double scale = __longlong_as_double((long long)(n + 1023) << 52);
    return __dmul_rn(p, scale);
}

__device__ __forceinline__ double tanh_portable(double x) {
    double ax = fabs(x);
    double r;
    if (!(ax == ax)) return x;
    if (ax >= 20.0) {
        r = 1.0;
    } else if (ax < 0.03125) {
        double x2 = __dmul_rn(ax, ax);
        double p = 62.0 / 2835.0;
        p = __dsub_rn(__dmul_rn(p, x2), 17.0 / 315.0);
        p = __dadd_rn(__dmul_rn(p, x2), 2.0 / 15.0);
        p = __dsub_rn(__dmul_rn(p, x2), 1.0 / 3.0);
        p = __dmul_rn(p, x2);
        r = __dadd_rn(ax, __dmul_rn(ax, p));
    } else {
        double e = exp_portable(__dmul_rn(2.0, ax));
        r = __dsub_rn(1.0, __ddiv_rn(2.0, __dadd_rn(e, 1.0)));
    }
    return x < 0 ? -r : r;
}

__device__ __forceinline__ float tanh_f32(float s) { return (float)tanh_portable((double)s); }

// ---- eltwise / binary ------------------------------------------------------
// Transcendentals other than tanh are evaluated in double and rounded once to
// float, which is what a correctly rounded float libm returns.

__device__ __forceinline__ float exp_f32(float x) { return (float)exp((double)x); }

__device__ __forceinline__ float logistic_f32(float s) {
    const float bound = 88.72283172607421875f;
    float in = -s;
    return in < bound ? __fdiv_rn(1.f, __fadd_rn(1.f, exp_f32(in))) : 0.f;
}
__device__ __forceinline__ float soft_relu_f32(float s, float alpha) {
    const float bound = 88.72283172607421875f;
    float in = __fmul_rn(s, alpha);
    float v = in < bound ? (float)log1p((double)exp_f32(in)) : in;
    return __fdiv_rn(v, alpha);
}
__device__ __forceinline__ float hardsigmoid_f32(float s, float alpha, float beta) {
    float v = __fadd_rn(__fmul_rn(alpha, s), beta);
    return v <= 0.f ? 0.f : v >= 1.f ? 1.f : v;
}

__device__ __forceinline__ float gelu_tanh_f32(float s) {
    const float sqrt_2_over_pi = 0.79788458347320556640625f;
    const float fitting_const = 0.044715f;
    float g = __fmul_rn(__fmul_rn(sqrt_2_over_pi, s),
            __fadd_rn(1.f, __fmul_rn(__fmul_rn(fitting_const, s), s)));
    float v = tanh_f32(g);
    // the reference finishes in double: 0.5 * s * (1. + v)
    return (float)__dmul_rn(__dmul_rn(0.5, (double)s), __dadd_rn(1.0, (double)v));
}

__device__ __forceinline__ float eltwise_fwd(int alg, float s, float alpha, float beta) {
    switch (alg) {
        case ALG_RELU: case ALG_RELU_DST: return s > 0 ? s : __fmul_rn(s, alpha);
        case ALG_TANH: case ALG_TANH_DST: return tanh_f32(s);
        case ALG_ELU: case ALG_ELU_DST: return s > 0 ? s : __fmul_rn(alpha, (float)expm1((double)s));
        case ALG_SQUARE: return __fmul_rn(s, s);
        case ALG_ABS: return s > 0 ? s : -s;
        case ALG_SQRT: case ALG_SQRT_DST: return __fsqrt_rn(s);
        case ALG_LINEAR: return __fadd_rn(__fmul_rn(alpha, s), beta);
        case ALG_SOFT_RELU: return soft_relu_f32(s, alpha);
        case ALG_HARDSIGMOID: return hardsigmoid_f32(s, alpha, beta);
        case ALG_LOGISTIC: case ALG_LOGISTIC_DST: return logistic_f32(s);
        case ALG_EXP: case ALG_EXP_DST: return exp_f32(s);
        case ALG_GELU_TANH: return gelu_tanh_f32(s);
        case ALG_SWISH: return __fmul_rn(s, logistic_f32(__fmul_rn(alpha, s)));
        case ALG_LOG: return (float)log((double)s);
        case ALG_CLIP: { s = s > alpha ? s : alpha; return s > beta ? beta : s; }
        case ALG_CLIP_V2: case ALG_CLIP_V2_DST: { s = s > alpha ? s : alpha; return s < beta ? s : beta; }
        case ALG_POW: return __fmul_rn(alpha, (float)pow((double)s, (double)beta));
        case ALG_GELU_ERF: {
            const float sqrt_2_over_2 = 0.707106769084930419921875f;
            float v = __fmul_rn(s, sqrt_2_over_2);
            return __fmul_rn(__fmul_rn(0.5f, s), __fadd_rn(1.f, (float)erf((double)v)));
        }
        case ALG_ROUND: return rintf(s);
        case ALG_MISH: return __fmul_rn(s, tanh_f32(soft_relu_f32(s, 1.f)));
        case ALG_HARDSWISH: return __fmul_rn(s, hardsigmoid_f32(s, alpha, beta));
        default: return __int_as_float(0x7fc00000);
    }
}

__device__ __forceinline__ float binary_fwd(int alg, float x, float y) {
    switch (alg) {
        case ALG_BIN_ADD: return __fadd_rn(x, y);
        case ALG_BIN_MUL: return __fmul_rn(x, y);
        case ALG_BIN_MAX: return x > y ? x : y;
        case ALG_BIN_MIN: return x < y ? x : y;
        case ALG_BIN_DIV: return __fdiv_rn(x, y);
        case ALG_BIN_SUB: return __fsub_rn(x, y);
        case ALG_BIN_GE: return x >= y;
        case ALG_BIN_GT: return x > y;
        case ALG_BIN_LE: return x <= y;
        case ALG_BIN_LT: return x < y;
        case ALG_BIN_EQ: return x == y;
        case ALG_BIN_NE: return x != y;
        case ALG_BIN_SELECT: return y;
        default: return __int_as_float(0x7fc00000);
    }
}

// ---- epilogue --------------------------------------------------------------

__device__ __forceinline__ int64_t quant_off(const b200_quant_t &q, int64_t i0, int64_t i1) {
    return (i0 / q.g0) * q.s0 + (i1 / q.g1) * q.s1;
}

__device__ __forceinline__ int sum_dt_of(const b200_matmul_params_t &p) {
    for (int i = 0; i < p.npo; ++i)
        if (p.po[i].kind == B200_PO_SUM && p.po[i].dt != B200_DT_UNDEF) return p.po[i].dt;
    return p.dst_dt;
}

__device__ __forceinline__ bool has_sum(const b200_matmul_params_t &p) {
    for (int i = 0; i < p.npo; ++i)
        if (p.po[i].kind == B200_PO_SUM) return true;
    return false;
}

// the post-op chain on one value; dst_old is the prior destination value read as the sum type
__device__ __forceinline__ float apply_post_ops(const b200_matmul_params_t &p, float x, float dst_old, int64_t m,
        int64_t n) {
    for (int i = 0; i < p.npo; ++i) {
        const b200_postop_t &e = p.po[i];
        switch (e.kind) {
            case B200_PO_SUM:
                x = __fadd_rn(x, __fmul_rn(e.scale, __fsub_rn(dst_old, (float)e.zero_point)));
                break;
            case B200_PO_ELTWISE: x = __fmul_rn(eltwise_fwd(e.alg, x, e.alpha, e.beta), e.scale); break;
            case B200_PO_BINARY: x = binary_fwd(e.alg, x, load_f32(e.dt, e.ptr, m * e.sm + n * e.sn)); break;
            case B200_PO_PRELU:
                if (!(x >= 0)) x = __fmul_rn(((const float *)e.ptr)[m * e.sm + n * e.sn], x);
                break;
            default: break;
        }
    }
    return x;
}

// Everything after the scaled accumulator for the element (m, n): bias,
// post-ops, destination scale (a multiply by the f32 reciprocal), destination
// zero-point, conversion and store.  int8_path selects the tail of the int8
// implementation (which adds the zero-point, 0 when unset, whenever any
// attribute is set) or of the floating-point one (no zero-point).
__device__ __forceinline__ void finish_element(const b200_matmul_params_t &p, float d, int64_t m, int64_t n,
        bool int8_path, float dst_scale_inv) {
    if (p.bias) d = __fadd_rn(d, load_f32(p.bias_dt, p.bias, m * p.bias_sm + n * p.bias_sn));
    const int64_t doff = m * p.dst_sm + n * p.dst_sn;
    if (p.npo > 0) {
        float dst_old = has_sum(p) ? load_f32(sum_dt_of(p), p.dst, doff) : 0.f;
        d = apply_post_ops(p, d, dst_old, m, n);
    }
    if (p.dst_scale.ptr) d = __fmul_rn(d, dst_scale_inv);
    if (int8_path) {
        const bool non_default = p.npo > 0 || p.src_scale.ptr || p.wei_scale.ptr || p.dst_scale.ptr
                || p.src_zp.ptr || p.wei_zp.ptr || p.dst_zp.ptr;
        if (non_default)
            d = __fadd_rn(d, p.dst_zp.ptr ? (float)load_int(B200_DT_S32, p.dst_zp.ptr, quant_off(p.dst_zp, m, n)) : 0.f);
    }
    store_f32(p.dst_dt, d, p.dst, doff);
}

__device__ __forceinline__ float dst_scale_reciprocal(const b200_matmul_params_t &p) {
    return p.dst_scale.ptr ? __fdiv_rn(1.f, load_f32(p.dst_scale.dt, p.dst_scale.ptr, 0)) : 1.f;
}

} // namespace b200
