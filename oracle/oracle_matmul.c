/*
 * CPU oracle for the quantized matmul path -- TEST INFRASTRUCTURE ONLY.
 * See oracle_matmul.h.  Build: gcc -O2 -ffp-contract=off -fopenmp -fPIC -shared.
 * -ffp-contract=off matters: every float operation below is rounded on its
 * own, as in the reference build (no FMA contraction).
 *
 * Each function names the reference code it restates (paths relative to the
 * reference project root).
 */
#include "oracle_matmul.h"

#include <math.h>
#include <stddef.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* ---- 16-bit and 8-bit float encodings ---------------------------------- */

/* src/common/float16.hpp:100-128 */
static float f16_to_f32(uint16_t raw) {
    uint32_t s = raw >> 15, e = (raw >> 10) & 0x1f, m = raw & 0x3ff;
    if (e == 0) {
        if (m == 0) return u2f(s << 31);
        float v = ldexpf((float)m, -24);
        return s ? -v : v;
    }
    if (e == 0x1f) {
        uint32_t mm = m << 13;
        if (mm) mm |= 0x400000;
        return u2f((s << 31) | 0x7f800000u | mm);
    }
    return u2f((s << 31) | ((e - 15 + 127) << 23) | (m << 13));
}

/* src/common/float16.hpp:52-98: round to nearest even; f32 denormals flush to
 * zero; results below the f16 normal range are rounded on the 2^-24 grid. */
static uint16_t f32_to_f16(float f) {
    uint32_t i = f2u(f), s = i >> 31, e = (i >> 23) & 0xff, m = i & 0x7fffff;
    uint32_t mm = m >> 13, r = m & 0x1fff, ee = 0;
    int32_t eee = (int32_t)e - 127 + 15;
    if (e == 0) {
        ee = 0; mm = 0;
    } else if (e == 0xff) {
        ee = 0x1f;
        if (m != 0) mm |= 0x200;
    } else if (eee > 0 && eee < 0x1f) {
        ee = (uint32_t)eee;
        if (r > (0x1000 - (mm & 1))) {
            mm++;
            if (mm == 0x400) { mm = 0; ee++; }
        }
    } else if (eee >= 0x1f) {
        ee = 0x1f; mm = 0;
    } else {
        /* |f| + 0.5f places the 2^-24 grid at the bottom of the mantissa,
         * so the float addition itself performs the rounding */
        float ff = fabsf(f) + 0.5f;
        ee = 0;
        mm = f2u(ff) & 0x7ff;
    }
    return (uint16_t)((s << 15) | (ee << 10) | mm);
}

/* src/common/bfloat16.cpp:22-51 */
static uint16_t f32_to_bf16(float f) {
    uint32_t u = f2u(f);
    uint32_t e = (u >> 23) & 0xff, m = u & 0x7fffff;
    if (e == 0) return (uint16_t)((u >> 16) & 0x8000);
    if (e == 0xff) {
        if (m == 0) return (uint16_t)(u >> 16);
        return (uint16_t)((u >> 16) | (1u << 6));
    }
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
static float bf16_to_f32(uint16_t r) { return u2f((uint32_t)r << 16); }

/* src/common/float8.cpp:150-188 (e4m3 -> f16 -> f32) */
static float e4m3_to_f32(uint8_t raw) {
    uint32_t s = raw >> 7, e = (raw >> 3) & 0xf, m = raw & 7;
    float v;
    if (e == 0xf && m == 7) return u2f((s << 31) | 0x7fc00000u);
    if (e == 0) v = ldexpf((float)m, -9);
    else v = ldexpf((float)(8 + m), (int)e - 10);
    return s ? -v : v;
}

/* src/common/float8.cpp:96-147: the value is first rounded to f16, then to
 * three mantissa bits (nearest even); above 464 it becomes NaN (0x7f), at or
 * below 2^-10 it becomes zero; the sub-normal grid is 2^-9. */
static uint8_t f32_to_e4m3(float f) {
    uint16_t h = f32_to_f16(f);
    uint32_t s8 = (h & 0x8000) >> 8;
    uint32_t a = h & 0x7fff;
    if (a > 0x5f40) return (uint8_t)(s8 | 0x7f);
    if (a <= 0x1400) return (uint8_t)s8;
    float v = f16_to_f32((uint16_t)a);
    int ex;
    (void)frexpf(v, &ex);      /* v = frac * 2^ex, frac in [0.5, 1) */
    int e = ex - 1;            /* v in [2^e, 2^(e+1)) */
    int q = e - 3;             /* quantum 2^q keeps 3 mantissa bits */
    if (q < -9) q = -9;
    float scaled = ldexpf(v, -q);           /* exact */
    float r = nearbyintf(scaled);           /* ties to even */
    float rv = ldexpf(r, q);
    /* encode rv (exactly representable) */
    if (rv < ldexpf(1.0f, -6)) {
        uint32_t m8 = (uint32_t)ldexpf(rv, 9);
        return (uint8_t)(s8 | m8);
    }
    (void)frexpf(rv, &ex);
    e = ex - 1;
    uint32_t m8 = (uint32_t)(ldexpf(rv, 3 - e)) - 8;
    return (uint8_t)(s8 | ((uint32_t)(e + 7) << 3) | m8);
}

/* src/common/float8.cpp:69-86 (e5m2 is the top byte of an f16) */
static float e5m2_to_f32(uint8_t raw) {
    uint8_t r = ((raw & 0x7d) == 0x7d) ? (uint8_t)(raw | 0x02) : raw;
    return f16_to_f32((uint16_t)((uint16_t)r << 8));
}
static uint8_t f32_to_e5m2(float f) {
    uint16_t fraw = f32_to_f16(f);
    int special = (fraw & 0x7c00) == 0x7c00;
    if (special && (fraw & 0x03ff)) return (uint8_t)((fraw >> 8) | 0x02);
    if (special) return (uint8_t)(fraw >> 8);
    fraw = (uint16_t)(fraw + 0x007f + ((fraw & 0x0100) >> 8));
    return (uint8_t)(fraw >> 8);
}

/* ---- typed loads and stores -------------------------------------------- */

/* src/cpu/ref_io_helper.hpp:33-62; 4-bit types hold two values per byte,
 * even index in the low nibble (src/common/utils.hpp nibble2_t). */
int32_t orc_load_int(int32_t dt, const void *ptr, int64_t idx) {
    switch (dt) {
        case ORC_S32: return ((const int32_t *)ptr)[idx];
        case ORC_S8: return ((const int8_t *)ptr)[idx];
        case ORC_U8: return ((const uint8_t *)ptr)[idx];
        case ORC_S4: {
            uint8_t b = ((const uint8_t *)ptr)[idx / 2];
            int v = (idx % 2) ? (b >> 4) : (b & 0xf);
            return (v & 8) ? v - 16 : v;
        }
        case ORC_U4: {
            uint8_t b = ((const uint8_t *)ptr)[idx / 2];
            return (idx % 2) ? (b >> 4) : (b & 0xf);
        }
        default: return INT32_MAX;
    }
}

/* src/cpu/ref_io_helper.hpp:64-113 */
float orc_load_float(int32_t dt, const void *ptr, int64_t idx) {
    switch (dt) {
        case ORC_F32: return ((const float *)ptr)[idx];
        case ORC_BF16: return bf16_to_f32(((const uint16_t *)ptr)[idx]);
        case ORC_F16: return f16_to_f32(((const uint16_t *)ptr)[idx]);
        case ORC_F8_E4M3: return e4m3_to_f32(((const uint8_t *)ptr)[idx]);
        case ORC_F8_E5M2: return e5m2_to_f32(((const uint8_t *)ptr)[idx]);
        case ORC_S32: case ORC_S8: case ORC_U8: case ORC_S4: case ORC_U4:
            return (float)orc_load_int(dt, ptr, idx);
        default: return NAN;
    }
}

/* src/cpu/ref_io_helper.hpp:115-154 with src/cpu/simple_q10n.hpp:33-81:
 * integer types saturate in f32 to [lowest, max] (s32's upper bound is
 * 2147483520.f, src/common/type_helpers.hpp:219-229), then round to nearest
 * even (nearbyintf under the default rounding mode), then narrow. */
void orc_store_float(int32_t dt, float v, void *ptr, int64_t idx) {
    switch (dt) {
        case ORC_F32: ((float *)ptr)[idx] = v; break;
        case ORC_BF16: ((uint16_t *)ptr)[idx] = f32_to_bf16(v); break;
        case ORC_F16: ((uint16_t *)ptr)[idx] = f32_to_f16(v); break;
        case ORC_F8_E4M3: ((uint8_t *)ptr)[idx] = f32_to_e4m3(v); break;
        case ORC_F8_E5M2: ((uint8_t *)ptr)[idx] = f32_to_e5m2(v); break;
        case ORC_S32: {
            float lo = -2147483648.f, hi = 2147483520.f;
            if (v < lo) v = lo;
            if (v > hi) v = hi;
            ((int32_t *)ptr)[idx] = (int32_t)nearbyintf(v);
        } break;
        case ORC_S8: {
            if (v < -128.f) v = -128.f;
            if (v > 127.f) v = 127.f;
            ((int8_t *)ptr)[idx] = (int8_t)(int32_t)nearbyintf(v);
        } break;
        case ORC_U8: {
            if (v < 0.f) v = 0.f;
            if (v > 255.f) v = 255.f;
            ((uint8_t *)ptr)[idx] = (uint8_t)(int32_t)nearbyintf(v);
        } break;
        /* 4-bit types (src/common/int4.hpp, src/common/nstl.hpp numeric_limits of int4_t / uint4_t,
         * src/cpu/ref_io_helper.hpp:84-97): saturate to [-8, 7] / [0, 15], round to nearest even,
         * keep the low four bits; two values per byte, even index in the low nibble */
        case ORC_S4: case ORC_U4: {
            const float lo = dt == ORC_S4 ? -8.f : 0.f, hi = dt == ORC_S4 ? 7.f : 15.f;
            if (v < lo) v = lo;
            if (v > hi) v = hi;
            const uint8_t q = (uint8_t)((int32_t)nearbyintf(v) & 0xf);
            uint8_t *b = (uint8_t *)ptr + (idx >> 1);
            *b = (idx & 1) ? (uint8_t)((*b & 0x0f) | (q << 4)) : (uint8_t)((*b & 0xf0) | q);
        } break;
        default: break;
    }
}

/* ---- portable tanh ------------------------------------------------------
 * Double-precision tanh built only from + - * / in a fixed order, so that a
 * CUDA kernel executing the same sequence with round-to-nearest operations
 * gives the same bits.  Accuracy is ~1e-15 relative, so its float rounding
 * equals the correctly rounded tanhf except on near-ties. */
static double exp_portable(double y) {
    /* y in [0, 40]: y = n ln2 + r, exp(r) by a degree-13 Taylor polynomial */
    const double log2e = 1.4426950408889634074;
    const double ln2_hi = 6.93147180369123816490e-01;
    const double ln2_lo = 1.90821492927058770002e-10;
    double t = y * log2e + 0.5;
    long long n = (long long)t; /* y >= 0: truncation is floor */
    double dn = (double)n;
    double r = (y - dn * ln2_hi) - dn * ln2_lo;
    double p = 1.0 / 6227020800.0;
    p = p * r + 1.0 / 479001600.0;
    p = p * r + 1.0 / 39916800.0;
    p = p * r + 1.0 / 3628800.0;
    p = p * r + 1.0 / 362880.0;
    p = p * r + 1.0 / 40320.0;
    p = p * r + 1.0 / 5040.0;
    p = p * r + 1.0 / 720.0;
    p = p * r + 1.0 / 120.0;
    p = p * r + 1.0 / 24.0;
    p = p * r + 1.0 / 6.0;
    p = p * r + 0.5;
    p = p * r + 1.0;
    p = p * r + 1.0;
    uint64_t bits = (uint64_t)(n + 1023) << 52;
    double scale;
    memcpy(&scale, &bits, 8);
    return p * scale;
}

double orc_tanh_portable(double x) {
    double ax = x < 0 ? -x : x;
    double r;
    if (!(ax == ax)) return x; /* NaN */
    if (ax >= 20.0) {
        r = 1.0;
    } else if (ax < 0.03125) {
        double x2 = ax * ax;
        double p = 62.0 / 2835.0;
        p = p * x2 - 17.0 / 315.0;
        p = p * x2 + 2.0 / 15.0;
        p = p * x2 - 1.0 / 3.0;
        p = p * x2;
        r = ax + ax * p;
    } else {
        double e = exp_portable(2.0 * ax);
        r = 1.0 - 2.0 / (e + 1.0);
    }
    return x < 0 ? -r : r;
}

static float tanh_sel(float s, int mode) {
    if (mode == 1) return (float)orc_tanh_portable((double)s);
    return tanhf(s);
}

/* ---- eltwise ------------------------------------------------------------
 * src/common/math_utils.hpp:134-420 (forward formulas) and the dispatcher in
 * src/cpu/primitive_attr_postops.cpp:48-86. */
static float logistic_fwd(float s) {
    float bound = 88.72283172607421875f;
    float in = -s;
    return in < bound ? (1.f / (1.f + expf(in))) : 0.f;
}
static float soft_relu_fwd(float s, float alpha) {
    float bound = 88.72283172607421875f;
    float in = s * alpha;
    float v = in < bound ? log1pf(expf(in)) : in;
    return v / alpha;
}
static float hardsigmoid_fwd(float s, float alpha, float beta) {
    float v = alpha * s + beta;
    return v <= 0.f ? 0.f : v >= 1.f ? 1.f : v;
}

float orc_eltwise(int32_t alg, float s, float alpha, float beta, int32_t tanh_mode) {
    switch (alg) {
        case 0x20: case 0x100: /* relu */
            return s > 0 ? s : s * alpha;
        case 0x21: case 0x101: return tanh_sel(s, tanh_mode);
        case 0x22: case 0x102: return s > 0 ? s : alpha * expm1f(s);
        case 0x23: return s * s;
        case 0x24: return s > 0 ? s : -s;
        case 0x25: case 0x103: return sqrtf(s);
        case 0x26: return alpha * s + beta;
        case 0x27: return soft_relu_fwd(s, alpha);
        case 0x28: return hardsigmoid_fwd(s, alpha, beta);
        case 0x29: case 0x104: return logistic_fwd(s);
        case 0x2a: case 0x105: return expf(s);
        case 0x2b: { /* gelu_tanh, math_utils.hpp:309-314: the last product is double */
            const float sqrt_2_over_pi = 0.79788458347320556640625f;
            const float fitting_const = 0.044715f;
            float v = tanh_sel(sqrt_2_over_pi * s * (1 + fitting_const * s * s), tanh_mode);
            return (float)(0.5 * s * (1. + v));
        }
        case 0x2c: return s * logistic_fwd(alpha * s);
        case 0x2d: return logf(s);
        case 0x2e: { s = s > alpha ? s : alpha; return s > beta ? beta : s; }
        case 0x2f: case 0x106: { s = s > alpha ? s : alpha; return s < beta ? s : beta; }
        case 0x30: return alpha * powf(s, beta);
        case 0x31: { /* gelu_erf */
            const float sqrt_2_over_2 = 0.707106769084930419921875f;
            float v = s * sqrt_2_over_2;
            return 0.5f * s * (1.f + erff(v));
        }
        case 0x32: return nearbyintf(s);
        case 0x33: return s * tanh_sel(soft_relu_fwd(s, 1.f), tanh_mode);
        case 0x34: return s * hardsigmoid_fwd(s, alpha, beta);
        default: return NAN;
    }
}

/* src/cpu/primitive_attr_postops.cpp:29-46 */
static float binary_op(int alg, float x, float y) {
    switch (alg) {
        case 0x1fff0: return x + y;
        case 0x1fff1: return x * y;
        case 0x1fff2: return x > y ? x : y; /* nstl::max(x, y) */
        case 0x1fff3: return x < y ? x : y; /* nstl::min(x, y) */
        case 0x1fff4: return x / y;
        case 0x1fff5: return x - y;
        case 0x1fff6: return x >= y;
        case 0x1fff7: return x > y;
        case 0x1fff8: return x <= y;
        case 0x1fff9: return x < y;
        case 0x1fffa: return x == y;
        case 0x1fffb: return x != y;
        case 0x1fffc: return y; /* select with a false condition */
        default: return NAN;
    }
}

/* src/cpu/primitive_attr_postops.cpp:278-347 */
static float post_ops(const orc_problem_t *p, float res, float dst_val, int64_t m, int64_t n) {
    for (int i = 0; i < p->npo; ++i) {
        const orc_postop_t *e = &p->po[i];
        switch (e->kind) {
            case ORC_PO_SUM:
                res += e->scale * (dst_val - (float)e->zero_point);
                break;
            case ORC_PO_ELTWISE:
                res = orc_eltwise(e->alg, res, e->alpha, e->beta, p->tanh_mode) * e->scale;
                break;
            case ORC_PO_BINARY: {
                float y = orc_load_float(e->dt, e->ptr, m * e->sm + n * e->sn);
                res = binary_op(e->alg, res, y);
            } break;
            case ORC_PO_PRELU:
                if (res >= 0) break;
                res = ((const float *)e->ptr)[m * e->sm + n * e->sn] * res;
                break;
            default: break;
        }
    }
    return res;
}

static inline int64_t qoff(const orc_quant_t *q, int64_t i0, int64_t i1) {
    return (i0 / q->g0) * q->s0 + (i1 / q->g1) * q->s1;
}

static int sum_dt_of(const orc_problem_t *p) {
    for (int i = 0; i < p->npo; ++i)
        if (p->po[i].kind == ORC_PO_SUM && p->po[i].dt != ORC_UNDEF) return p->po[i].dt;
    return p->dst_dt;
}

/* the reference converts a one-element scale to f32 up front and inverts a
 * destination scale (src/cpu/cpu_primitive.hpp:32-66) */
static float single_scale(const orc_quant_t *q) { return orc_load_float(q->dt, q->ptr, 0); }

/* src/cpu/matmul/ref_matmul_int8.cpp:154-261 */
static void matmul_int8(const orc_problem_t *p) {
    const int64_t M = p->M, N = p->N, K = p->K;
    /* ref_matmul_int8.cpp:83-144: the number of K groups is the largest among the
     * four arguments, and quant_entry_t::get_group returns 1 when no groups were
     * requested (primitive_attr_quant.hpp:83-90) -- for arguments that are not set
     * at all, too -- so without explicit groups the loop runs in K groups of 1. */
    int64_t src_zp_ng = K, wei_zp_ng = K, src_sc_ng = K, wei_sc_ng = K;
    if (p->src_zp.ptr && p->src_zp.g1 > 1) src_zp_ng = K / p->src_zp.g1;
    if (p->wei_zp.ptr && p->wei_zp.g0 > 1) wei_zp_ng = K / p->wei_zp.g0;
    if (p->src_scale.ptr && p->src_scale.g1 > 1) src_sc_ng = K / p->src_scale.g1;
    if (p->wei_scale.ptr && p->wei_scale.g0 > 1) wei_sc_ng = K / p->wei_scale.g0;
    if (p->exact_acc) {
        /* only explicit groups count */
        if (!(p->src_zp.ptr && p->src_zp.g1 > 1)) src_zp_ng = 1;
        if (!(p->wei_zp.ptr && p->wei_zp.g0 > 1)) wei_zp_ng = 1;
        if (!(p->src_scale.ptr && p->src_scale.g1 > 1)) src_sc_ng = 1;
        if (!(p->wei_scale.ptr && p->wei_scale.g0 > 1)) wei_sc_ng = 1;
    }
    int64_t ng = src_zp_ng;
    if (wei_zp_ng > ng) ng = wei_zp_ng;
    if (src_sc_ng > ng) ng = src_sc_ng;
    if (wei_sc_ng > ng) ng = wei_sc_ng;
    const int64_t gk = K / ng;
    const float src_scale0 = (p->src_scale.ptr && p->src_scale.nelems_is_one) ? single_scale(&p->src_scale) : 1.f;
    const float wei_scale0 = (p->wei_scale.ptr && p->wei_scale.nelems_is_one) ? single_scale(&p->wei_scale) : 1.f;
    const float dst_scale_inv = p->dst_scale.ptr ? 1.f / single_scale(&p->dst_scale) : 1.f;
    const int sum_dt = sum_dt_of(p);
    const int non_default = p->npo > 0 || p->src_scale.ptr || p->wei_scale.ptr || p->dst_scale.ptr
            || p->src_zp.ptr || p->wei_zp.ptr || p->dst_zp.ptr;
    const int64_t ms = p->m_step > 0 ? p->m_step : 1, ns = p->n_step > 0 ? p->n_step : 1;
    const int64_t nm = (M - p->m0 + ms - 1) / ms, nn = (N - p->n0 + ns - 1) / ns;

#pragma omp parallel for collapse(2) schedule(static)
    for (int64_t im = 0; im < nm; ++im)
        for (int64_t in = 0; in < nn; ++in) {
            const int64_t m = p->m0 + im * ms, n = p->n0 + in * ns;
            float d = 0;
            for (int64_t g = 0; g < ng; ++g) {
                int acc = 0;
                for (int64_t kk = 0; kk < gk; ++kk) {
                    const int64_t k = kk + g * gk;
                    int s = orc_load_int(p->src_dt, p->src, m * p->src_sm + k * p->src_sk);
                    int w = orc_load_int(p->wei_dt, p->wei, k * p->wei_sk + n * p->wei_sn);
                    if (p->src_zp.ptr) s -= orc_load_int(p->src_zp.dt, p->src_zp.ptr, qoff(&p->src_zp, m, k));
                    if (p->wei_zp.ptr) w -= orc_load_int(p->wei_zp.dt, p->wei_zp.ptr, qoff(&p->wei_zp, k, n));
                    acc += s * w;
                }
                float acc_f = (float)acc;
                if (p->src_scale.ptr) {
                    float sc = p->src_scale.nelems_is_one
                            ? src_scale0
                            : orc_load_float(p->src_scale.dt, p->src_scale.ptr, qoff(&p->src_scale, m, g * gk));
                    acc_f *= sc;
                }
                if (p->wei_scale.ptr) {
                    float sc = p->wei_scale.nelems_is_one
                            ? wei_scale0
                            : orc_load_float(p->wei_scale.dt, p->wei_scale.ptr, qoff(&p->wei_scale, g * gk, n));
                    acc_f *= sc;
                }
                d += acc_f;
            }
            if (p->bias) d += orc_load_float(p->bias_dt, p->bias, m * p->bias_sm + n * p->bias_sn);
            const int64_t doff = m * p->dst_sm + n * p->dst_sn;
            if (non_default) {
                float dst_val = orc_load_float(sum_dt, p->dst, doff);
                d = post_ops(p, d, dst_val, m, n);
                if (p->dst_scale.ptr) d *= dst_scale_inv;
                /* the reference adds the zero-point even when it is not set (its
                 * default is a pointer to 0), which turns -0.f into +0.f */
                d += p->dst_zp.ptr ? (float)orc_load_int(ORC_S32, p->dst_zp.ptr, qoff(&p->dst_zp, m, n)) : 0.f;
            }
            orc_store_float(p->dst_dt, d, p->dst, doff);
        }
}

/* src/cpu/matmul/ref_matmul.cpp:130-233 */
static void matmul_fp(const orc_problem_t *p) {
    const int64_t M = p->M, N = p->N, K = p->K;
    const int wei_is_int = p->wei_dt == ORC_S8 || p->wei_dt == ORC_U8 || p->wei_dt == ORC_S4 || p->wei_dt == ORC_U4;
    const int decomp = wei_is_int && p->apply_to_int;
    const float src_scale0 = p->src_scale.ptr ? single_scale(&p->src_scale) : 1.f;
    const float wei_scale0 = (p->wei_scale.ptr && p->wei_scale.nelems_is_one) ? single_scale(&p->wei_scale) : 1.f;
    const float dst_scale_inv = p->dst_scale.ptr ? 1.f / single_scale(&p->dst_scale) : 1.f;
    const int sum_dt = sum_dt_of(p);
    const int64_t ms = p->m_step > 0 ? p->m_step : 1, ns = p->n_step > 0 ? p->n_step : 1;
    const int64_t nm = (M - p->m0 + ms - 1) / ms, nn = (N - p->n0 + ns - 1) / ns;

#pragma omp parallel for collapse(2) schedule(static)
    for (int64_t im = 0; im < nm; ++im)
        for (int64_t in = 0; in < nn; ++in) {
            const int64_t m = p->m0 + im * ms, n = p->n0 + in * ns;
            float acc = 0;
            for (int64_t k = 0; k < K; ++k) {
                const float s = orc_load_float(p->src_dt, p->src, m * p->src_sm + k * p->src_sk);
                float w = orc_load_float(p->wei_dt, p->wei, k * p->wei_sk + n * p->wei_sn);
                if (decomp) {
                    if (p->wei_zp.ptr)
                        w -= orc_load_int(p->wei_zp.dt, p->wei_zp.ptr, qoff(&p->wei_zp, k, n));
                    if (p->wei_scale.ptr) {
                        float sc = p->wei_scale.nelems_is_one
                                ? wei_scale0
                                : orc_load_float(p->wei_scale.dt, p->wei_scale.ptr, qoff(&p->wei_scale, k, n));
                        w *= sc;
                    }
                }
                acc += s * w;
            }
            float d = acc;
            if (p->src_scale.ptr) d *= src_scale0;
            if (p->wei_scale.ptr && !decomp) {
                float sc = p->wei_scale.nelems_is_one
                        ? wei_scale0
                        : orc_load_float(p->wei_scale.dt, p->wei_scale.ptr, qoff(&p->wei_scale, 0, n));
                d *= sc;
            }
            if (p->bias) d += orc_load_float(p->bias_dt, p->bias, m * p->bias_sm + n * p->bias_sn);
            const int64_t doff = m * p->dst_sm + n * p->dst_sn;
            if (p->npo > 0) {
                float dst_val = orc_load_float(sum_dt, p->dst, doff);
                d = post_ops(p, d, dst_val, m, n);
            }
            if (p->dst_scale.ptr) d *= dst_scale_inv;
            orc_store_float(p->dst_dt, d, p->dst, doff);
        }
}

int orc_matmul(const orc_problem_t *p) {
    if (!p || !p->src || !p->wei || !p->dst) return 1;
    if (p->M <= 0 || p->N <= 0 || p->K <= 0) return 0; /* a zero dim: the reference returns without touching dst */
#ifdef _OPENMP
    int saved = omp_get_max_threads();
    if (p->nthreads > 0) omp_set_num_threads(p->nthreads);
#endif
    if (p->src_dt == ORC_S8 || p->src_dt == ORC_U8)
        matmul_int8(p);
    else
        matmul_fp(p);
#ifdef _OPENMP
    if (p->nthreads > 0) omp_set_num_threads(saved);
#endif
    return 0;
}

/* src/cpu/reorder/simple_reorder.hpp:2551-2635 (the generic "simple:any" reorder) with
 * src/cpu/reorder/cpu_reorder_pd.hpp:83-109: the destination scale is inverted up front;
 * an integer source minus its zero-point is an integer subtraction, converted to f32
 * afterwards; scale, sum and zero-point are separate f32 operations (no fused
 * multiply-add); the store saturates, then rounds to nearest even. */
int orc_reorder(const orc_reorder_t *r) {
    if (!r || !r->src || !r->dst) return 1;
    if (r->rows <= 0 || r->cols <= 0) return 0;
    const int int_src = r->src_dt == ORC_S32 || r->src_dt == ORC_S8 || r->src_dt == ORC_U8 || r->src_dt == ORC_S4 || r->src_dt == ORC_U4;
    const int32_t dst_zp = r->dst_zp.ptr ? orc_load_int(r->dst_zp.dt, r->dst_zp.ptr, 0) : 0;
#ifdef _OPENMP
    int saved = omp_get_max_threads();
    if (r->nthreads > 0) omp_set_num_threads(r->nthreads);
#pragma omp parallel for schedule(static)
#endif
    for (int64_t i = 0; i < r->rows; ++i)
        for (int64_t j = 0; j < r->cols; ++j) {
            float ss = 1.f, ds = 1.f;
            if (r->src_scale.ptr)
                ss = r->src_scale.nelems_is_one ? single_scale(&r->src_scale)
                                                : orc_load_float(r->src_scale.dt, r->src_scale.ptr, qoff(&r->src_scale, i, j));
            if (r->dst_scale.ptr)
                ds = 1.f / orc_load_float(r->dst_scale.dt, r->dst_scale.ptr,
                                          r->dst_scale.nelems_is_one ? 0 : qoff(&r->dst_scale, i, j));
            int zp = 0;
            if (r->src_zp.ptr)
                zp = (int)orc_load_float(r->src_zp.dt, r->src_zp.ptr, r->src_zp.nelems_is_one ? 0 : qoff(&r->src_zp, i, j));
            const int64_t ioff = i * r->src_s0 + j * r->src_s1, ooff = i * r->dst_s0 + j * r->dst_s1;
            float d; /* built with -ffp-contract=off: the steps below stay separate */
            if (int_src)
                d = ss * (float)(orc_load_int(r->src_dt, r->src, ioff) - zp);
            else
                d = ss * (orc_load_float(r->src_dt, r->src, ioff) - (float)zp);
            if (r->beta != 0.f) {
                d += r->beta * orc_load_float(r->dst_dt, r->dst, ooff);
            }
            d = d * ds + (float)dst_zp;
            orc_store_float(r->dst_dt, d, r->dst, ooff);
        }
#ifdef _OPENMP
    if (r->nthreads > 0) omp_set_num_threads(saved);
#endif
    return 0;
}
