/*
 * CPU oracle for the quantized matmul path -- TEST INFRASTRUCTURE ONLY.
 *
 * This is a plain-C restatement of the arithmetic of the reference library's
 * two scalar matmul implementations ("ref_int8:any" and "ref:any") and of the
 * helpers they call.  It exists so that tests can check the CUDA path, and so
 * that bench.py can time a CPU baseline.  Nothing in the shipped library links
 * to, loads or calls this file.
 *
 * Parity status: PINNED.  tests/test_oracle_vs_reference.py compares this code
 * bit for bit with the reference library itself (built from its own sources by
 * oracle/build_ref.py) and tests/golden/ holds outputs of the reference
 * library that this code must reproduce.
 */
#ifndef ORACLE_MATMUL_H
#define ORACLE_MATMUL_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* data type codes: the numeric values of dnnl_data_type_t
 * (include/oneapi/dnnl/dnnl_common_types.h:78-110 in the reference). */
enum {
    ORC_UNDEF = 0, ORC_F16 = 1, ORC_BF16 = 2, ORC_F32 = 3, ORC_S32 = 4,
    ORC_S8 = 5, ORC_U8 = 6, ORC_F8_E5M2 = 9, ORC_F8_E4M3 = 10, ORC_S4 = 11,
    ORC_U4 = 12
};

/* post-op kinds */
enum { ORC_PO_SUM = 1, ORC_PO_ELTWISE = 2, ORC_PO_BINARY = 3, ORC_PO_PRELU = 4 };

/* A scale or zero-point argument.  The element used for logical index
 * (i0, i1) is ptr[(i0 / g0) * s0 + (i1 / g1) * s1]; (i0, i1) is (m, k) for a
 * source argument, (k, n) for a weights argument and (m, n) for a destination
 * argument.  ptr == NULL means "not set" (scale 1, zero-point 0). */
typedef struct {
    const void *ptr;
    int32_t dt;
    int32_t nelems_is_one; /* the reference converts a single scale up front */
    int64_t s0, s1;
    int64_t g0, g1;
} orc_quant_t;

typedef struct {
    int32_t kind;       /* ORC_PO_* */
    int32_t alg;        /* dnnl_alg_kind_t value for eltwise / binary */
    float alpha, beta;  /* eltwise */
    float scale;        /* eltwise scale or sum scale */
    int32_t zero_point; /* sum */
    int32_t dt;         /* sum: type dst is read as; binary: type of src1 */
    const void *ptr;    /* binary src1 or prelu weights (f32) */
    int64_t sm, sn;     /* element strides of ptr over (m, n); 0 = broadcast */
} orc_postop_t;

#define ORC_MAX_POSTOPS 32

typedef struct {
    int64_t M, N, K;
    const void *src; int32_t src_dt; int32_t pad0; int64_t src_sm, src_sk;
    const void *wei; int32_t wei_dt; int32_t pad1; int64_t wei_sk, wei_sn;
    const void *bias; int32_t bias_dt; int32_t pad2; int64_t bias_sm, bias_sn;
    void *dst; int32_t dst_dt; int32_t pad3; int64_t dst_sm, dst_sn;
    orc_quant_t src_scale, wei_scale, dst_scale;
    orc_quant_t src_zp, wei_zp, dst_zp;
    int32_t apply_to_int; /* fpmath_mode apply_to_int flag (weights decompression) */
    int32_t npo;
    orc_postop_t po[ORC_MAX_POSTOPS];
    /* 0: tanhf from libm, exactly as the reference does;
     * 1: the portable double-precision tanh below, which is the one the CUDA
     *    kernels can reproduce bit for bit. */
    int32_t tanh_mode;
    int32_t nthreads; /* 0 = OpenMP default */
    /* only rows m0, m0+m_step, ... < M and columns n0, n0+n_step, ... < N are
     * computed (step 1 and origin 0 = everything); other dst elements are left
     * untouched.  Lets a test sample a problem that is too large to compute
     * in full on the CPU. */
    int64_t m0, m_step, n0, n_step;
    /* int8 sources only.  0: exactly what the reference's scalar implementation
     * does -- its K loop is cut into groups of the smallest group size among
     * the scale / zero-point arguments, and an argument without explicit
     * groups counts as group size 1, so that in practice every product s*w is
     * converted to f32, scaled and accumulated in f32.
     * 1: "exact accumulation": only explicitly requested groups cut the K
     * loop; within a group the products are summed exactly in s32 and scaled
     * once.  This is the library's documented formula and what its optimised
     * (JIT) implementation and the tensor-core kernel compute. */
    int32_t exact_acc;
    int32_t pad4;
} orc_problem_t;

/* returns 0 on success, non-zero for an unsupported combination */
int orc_matmul(const orc_problem_t *p);

/* Quantising reorder of a 2-D tensor (plain layouts): the reference's generic reorder
 * implementation "simple:any" (src/cpu/reorder/simple_reorder.hpp:2551-2635).
 * Scale / zero-point elements are addressed as in orc_quant_t with (i0, i1) the
 * element's (row, column). */
typedef struct {
    int64_t rows, cols;
    const void *src; int32_t src_dt; int32_t pad0; int64_t src_s0, src_s1;
    void *dst; int32_t dst_dt; int32_t pad1; int64_t dst_s0, dst_s1;
    orc_quant_t src_scale, dst_scale; /* dst scale: f32 */
    orc_quant_t src_zp, dst_zp;       /* dst zero-point: one s32 value */
    float beta;                       /* scale of a sum post-op (0 = none): d += beta * dst */
    int32_t nthreads;                 /* 0 = OpenMP default */
} orc_reorder_t;

int orc_reorder(const orc_reorder_t *r);

/* scalar helpers, exported for the data-type tests */
float orc_load_float(int32_t dt, const void *ptr, int64_t idx);
int32_t orc_load_int(int32_t dt, const void *ptr, int64_t idx);
void orc_store_float(int32_t dt, float v, void *ptr, int64_t idx);
float orc_eltwise(int32_t alg, float s, float alpha, float beta, int32_t tanh_mode);
double orc_tanh_portable(double x);

#ifdef __cplusplus
}
#endif
#endif
