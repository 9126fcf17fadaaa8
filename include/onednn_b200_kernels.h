/*
 * Inner kernel launch ABI of the B200 matmul engine.
 *
 * Every device kernel of the library is reached through one extern "C"
 * launcher that takes a plain parameter block (pointers, sizes, strides,
 * quantisation modes, the post-op chain) and a CUDA stream.  The host library
 * lowers a matmul primitive descriptor + its runtime arguments into this block;
 * the launchers can equally be bound directly over FFI (ctypes, cgo, JNI) by a
 * caller that already holds device pointers.
 *
 * The block describes what the reference library's matmul implementations read
 * from their execution context: src/weights/bias/dst memories with their
 * memory descriptors, DNNL_ARG_ATTR_SCALES | arg and DNNL_ARG_ATTR_ZERO_POINTS
 * | arg memories, and the post-op list of the primitive attribute
 * (reference: src/cpu/matmul/ref_matmul_int8.cpp:38-152,
 *  src/cpu/matmul/ref_matmul.cpp:38-128, src/common/primitive_attr.hpp:274-521).
 *
 * All launchers return 0 on success, a negative B200_ERR_* code when the
 * parameter block is not supported by that kernel (nothing was launched), or a
 * positive cudaError_t value when the launch itself failed.  Launches are
 * asynchronous on the given stream; pointers are device pointers unless a
 * comment says otherwise.
 */
#ifndef ONEDNN_B200_KERNELS_H
#define ONEDNN_B200_KERNELS_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_API __attribute__((visibility("default")))

/* opaque stream handle: a cudaStream_t */
typedef void *b200_stream_t;

/* data type codes = numeric values of dnnl_data_type_t
 * (reference: include/oneapi/dnnl/dnnl_common_types.h:78-110) */
enum {
    B200_DT_UNDEF = 0, B200_DT_F16 = 1, B200_DT_BF16 = 2, B200_DT_F32 = 3,
    B200_DT_S32 = 4, B200_DT_S8 = 5, B200_DT_U8 = 6, B200_DT_F8_E5M2 = 9,
    B200_DT_F8_E4M3 = 10, B200_DT_S4 = 11, B200_DT_U4 = 12
};

enum {
    B200_ERR_UNSUPPORTED = -1, /* this kernel cannot run this block */
    B200_ERR_BAD_ARG = -2,     /* null pointer / negative size / misalignment */
    B200_ERR_TOO_LARGE = -3    /* a size exceeds a fixed-capacity resource */
};

enum { B200_PO_SUM = 1, B200_PO_ELTWISE = 2, B200_PO_BINARY = 3, B200_PO_PRELU = 4 };

/* A scale or zero-point argument.  Element for logical index (i0, i1) is
 * ptr[(i0 / g0) * s0 + (i1 / g1) * s1] with (i0, i1) = (m, k) for src,
 * (k, n) for weights and (m, n) for dst arguments; a stride of 0 broadcasts.
 * This is the offset rule of the reference's get_quant_off
 * (src/cpu/matmul/matmul_utils.hpp:156-196).  ptr == NULL: argument not set. */
typedef struct {
    const void *ptr;
    int32_t dt;
    int32_t reserved;
    int64_t s0, s1;
    int64_t g0, g1;
} b200_quant_t;

/* One post-op (reference: dnnl_post_ops::entry_t, primitive_attr.hpp:274-420;
 * applied in list order by ref_post_ops_t::execute,
 * src/cpu/primitive_attr_postops.cpp:278-347). */
typedef struct {
    int32_t kind;       /* B200_PO_* */
    int32_t alg;        /* dnnl_alg_kind_t value (eltwise_* / binary_*) */
    float alpha, beta;  /* eltwise parameters */
    float scale;        /* eltwise scale, or sum scale */
    int32_t zero_point; /* sum zero-point */
    int32_t dt;         /* sum: type the old dst is read as; binary: src1 type */
    int32_t reserved;
    const void *ptr;    /* binary src1, or prelu weights (f32) */
    int64_t sm, sn;     /* element strides of ptr over (m, n); 0 = broadcast */
} b200_postop_t;

#define B200_MAX_DST_PEERS 7
#define B200_MAX_POSTOPS 32

/* packed weights layouts produced by b200_pack_weights */
enum {
    B200_WEI_PLAIN = 0,      /* strided (k, n) as given by wei_sk / wei_sn */
    B200_WEI_KMAJOR = 1,     /* 8-bit weights transposed to [N][Kp] (K contiguous,
                                Kp = K rounded up to 16) followed by the s32 column
                                sums: the tcgen05 operand layout */
    B200_WEI_WC8_TC = 4,     /* 8-bit weights, same blocks (8 KiB), one byte per weight */
    B200_WEI_WC4_TC = 3,     /* 4-bit weights in blocks of 128 n x 64 k (4 KiB), row-major inside,
                              * for the tensor-core weight-decompression kernel (matmul_wctc.cu) */
    B200_WEI_WC4_TILED = 2   /* 4-bit weights in tiles of 16 n x 64 k (512 bytes),
                                nibbles ordered as mma.m16n8k16 A fragments; s4
                                values stored offset by 8 */
};

typedef struct {
    int64_t M, N, K;
    const void *src; int32_t src_dt; int32_t reserved0; int64_t src_sm, src_sk;
    const void *wei; int32_t wei_dt; int32_t wei_layout; int64_t wei_sk, wei_sn;
    const void *bias; int32_t bias_dt; int32_t reserved1; int64_t bias_sm, bias_sn;
    void *dst; int32_t dst_dt; int32_t reserved2; int64_t dst_sm, dst_sn;
    b200_quant_t src_scale, wei_scale, dst_scale;
    b200_quant_t src_zp, wei_zp, dst_zp;
    /* s32 column sums of the weights, sum_k w[k][n], length N (int8 path with a
     * source zero-point; produced by b200_pack_weights or b200_colsum) */
    const int32_t *wei_colsum;
    int32_t apply_to_int; /* fpmath apply_to_int: integer weights are decompressed */
    int32_t npo;
    b200_postop_t po[B200_MAX_POSTOPS];
    /* device status word (may be NULL): kernels OR a non-zero code into it when
     * a bounded wait ran out; the stream's wait() reports it */
    uint32_t *status;
    /* scratch for kernels that need it (split-K partials); sized by
     * b200_matmul_scratch_bytes */
    void *scratch; size_t scratch_bytes;
    /* non-zero: the caller guarantees that the accumulation part of the scratch
     * is all zero on entry (kernels that use it leave it zeroed on exit) */
    int32_t scratch_zeroed; int32_t reserved3;
    /* N-split over the GPUs of a node: besides dst, every finished element is also stored at
     * the same offset from each of these bases -- the same (M, N_full) destination in the
     * memory of the other GPUs, mapped into this process (peer / symmetric memory) -- so that
     * the exchange of column slices rides on the epilogue's stores instead of a collective
     * afterwards (each warp re-reads its finished block from the local L2 and sends whole row
     * segments).  Plain stores only; nothing is ever loaded from a peer.  Honoured by
     * b200_matmul_tc8_launch; the other kernels return B200_ERR_UNSUPPORTED when it is set. */
    int32_t n_dst_peers; int32_t reserved4;
    void *dst_peer[B200_MAX_DST_PEERS];
    /* s32 row sums of src, sum_k src[m][k], length M: needed by b200_matmul_tc8_launch when
     * weights zero-points are set (b200_colsum_launch on src seen as its transpose gives them) */
    const int32_t *src_rowsum;
} b200_matmul_params_t;

/* ---- matmul kernels ----------------------------------------------------- */

/* Generic kernel: any dtype combination of the reference's ref_int8 / ref
 * implementations, any strides, any quantisation mode, any post-op chain.
 * One thread per dst element.  (ref_matmul_int8.cpp:154-261, ref_matmul.cpp:130-233) */
B200_API int b200_matmul_generic_launch(const b200_matmul_params_t *p, b200_stream_t stream);

/* Dense 8-bit GEMM on the 5th-generation tensor cores (tcgen05.mma kind::i8 for
 * u8/s8 x s8, kind::f8f6f4 for e4m3 x e4m3; TMA-fed, mbarrier-pipelined, TMEM
 * accumulators) with the whole epilogue fused.  Needs row-major src (src_sk == 1),
 * weights in B200_WEI_KMAJOR layout, row-major dst, K % 16 == 0, per-tensor or
 * per-N scales, a per-tensor source zero-point at most.  Replaces the
 * reference's brgemm_matmul_t execute (src/cpu/x64/matmul/brgemm_matmul.cpp:383-496)
 * for these shapes. */
B200_API int b200_matmul_tc8_launch(const b200_matmul_params_t *p, b200_stream_t stream);

/* Weight-compressed decode GEMV / skinny GEMM: bf16 (or f16/f32) activations
 * times u4/s4/s8/u8 weights with K-grouped scales and zero-points, f32
 * accumulation, 32 activation rows per pass; HBM-bound.  Weights in
 * B200_WEI_WC4_TILED layout (or plain dense ab, packed into the scratch first).  (ref_matmul.cpp:130-233 with
 * with_wei_decompression; brgemm_matmul_copy_utils.cpp:2861-2880 is the
 * reference's JIT decompression.) */
B200_API int b200_matmul_wc_launch(const b200_matmul_params_t *p, b200_stream_t stream);

/* The weight-compressed kernel for callers that may not allocate device memory.
 * This entry point has no counterpart in the reference.
 *
 * b200_matmul_wc_launch accumulates partial sums in a scratch buffer that the
 * caller (or the host library, for its primitives) has to allocate.  Code that
 * runs where allocation is off limits -- a plugin inside a host runtime that
 * owns all device memory and only passes pointers in, a decode loop inside a
 * serving engine's captured or latency-critical section, a callback of a
 * memory pool -- can call this variant instead: its scratch is a fixed 2 MiB
 * array inside the library's device image, held by every GPU that loads the
 * library until the process exits.  It calls neither cudaMalloc nor cudaFree
 * nor any allocating library routine; src, weights, scales, zero-points, bias
 * and dst are still passed in by the caller (p->scratch is ignored).
 *
 * Limits: bf16 activations (src_dt == B200_DT_BF16), weights already in
 * B200_WEI_WC4_TILED layout, and the partial sums plus the per-strip counters
 * must fit the array: M * N * 4 bytes rounded up to 256, plus N / 16 * 4 bytes
 * rounded up to 256, at most b200_matmul_wc_noalloc_max_bytes() (2 MiB) -- for
 * N = 14336 that is M <= 36, and M * N = 524288 itself does not fit because the
 * counters share the array.  Anything larger returns B200_ERR_TOO_LARGE,
 * anything else unsupported B200_ERR_UNSUPPORTED, and nothing is launched.
 *
 * The first call on a device looks up the array's device address
 * (cudaGetSymbolAddress) with that device current; make that first call before
 * any stream capture begins.  All calls on a device share the one array and it
 * keeps the last call's contents: each call clears the part it uses on the
 * given stream first, and two calls whose kernels overlap on the GPU (different
 * streams without ordering between them) race on it -- serialise them. */
B200_API int b200_matmul_wc_noalloc_launch(const b200_matmul_params_t *p, b200_stream_t stream);
B200_API size_t b200_matmul_wc_noalloc_max_bytes(void);

/* Weight-decompression matmul for more than a few activation rows: the weights are
 * converted to bf16 in shared memory and multiplied on the tensor cores (tcgen05, f32
 * accumulation in tensor memory).  bf16 activations, u4 / s4 weights in the
 * B200_WEI_WC4_TC layout (or plain dense ab, packed into the scratch first), bf16 scales
 * (per tensor, per column or K-grouped) or none, u4 / s4 zero-points or none; or s8 / u8
 * weights in the B200_WEI_WC8_TC layout (or plain, any strides) with f32 / bf16 / f16 scales
 * and s8 / u8 / s32 / 4-bit zero-points.  K groups multiples of 64.  Same semantics as b200_matmul_wc_launch
 * (ref_matmul.cpp:130-233 with_wei_decompression) with each decompressed weight rounded to
 * bf16, which fpmath mode bf16 with apply_to_int permits. */
B200_API int b200_matmul_wc_tc_launch(const b200_matmul_params_t *p, b200_stream_t stream);
/* plain dense (K, N) 4-bit weights -> B200_WEI_WC4_TC, and the size of the result */
B200_API int b200_wc_tc_pack_launch(const void *src, void *dst, int64_t K, int64_t N, int32_t dt, b200_stream_t stream);
/* plain (K, N) s8 / u8 weights with element strides sk, sn -> B200_WEI_WC8_TC */
B200_API int b200_wc_tc_pack8_launch(const void *src, int64_t sk, int64_t sn, void *dst, int64_t K, int64_t N, int32_t dt,
        b200_stream_t stream);
B200_API size_t b200_wc_tc_packed_bytes(int64_t K, int64_t N, int32_t dt);

/* plain dense (K, N) 4-bit weights (two per byte along N) -> B200_WEI_WC4_TILED;
 * needs K % 64 == 0 and N % 16 == 0 */
B200_API int b200_wc_pack_launch(const void *src, void *dst, int64_t K, int64_t N, int32_t dt, b200_stream_t stream);

/* bytes of scratch the given block needs for the given kernel
 * (0 = generic, 1 = tc8, 2 = wc) */
B200_API size_t b200_matmul_scratch_bytes(const b200_matmul_params_t *p, int kernel);

/* ---- weights reorder / pack kernels -------------------------------------- */

typedef struct {
    int64_t K, N;
    const void *src; int32_t src_dt; int32_t src_layout; int64_t src_sk, src_sn;
    void *dst; int32_t dst_dt; int32_t dst_layout; int64_t dst_sk, dst_sn;
    /* optional quantising reorder: dst = sat_rne(src * scale[n] ... ) is not part
     * of this ABI yet; scale pointers must be NULL */
    const void *scale; int32_t scale_dt; int32_t scale_mask;
} b200_reorder_params_t;

/* bytes a packed weights buffer occupies (data + column sums) */
B200_API size_t b200_packed_weights_bytes(int64_t K, int64_t N, int32_t dt, int32_t layout);
/* byte offset of the s32 column sums inside a B200_WEI_KMAJOR buffer */
B200_API size_t b200_packed_colsum_offset(int64_t K, int64_t N, int32_t dt);

/* plain (strided) -> plain or packed, same element type or a plain conversion
 * between f32 / bf16 / f16 / s32 / s8 / u8 (saturate + round-to-nearest-even
 * for integer destinations, as the reference's simple_reorder does).
 * Replaces dnnl_reorder for the weights of this path
 * (src/common/reorder.cpp:63-220, src/cpu/reorder/simple_reorder.hpp). */
B200_API int b200_reorder_launch(const b200_reorder_params_t *p, b200_stream_t stream);

/* Quantising reorder of a plain 2-D tensor (any element strides):
 *   d = src_scale * (src - src_zp);  d += beta * dst (sum post-op);
 *   d = d * (1 / dst_scale) + dst_zp;  dst = saturate + round-to-nearest-even (integer
 *   destinations) or a plain conversion of d
 * with every step a separate f32 operation and the subtraction done in s32 for integer
 * sources -- the arithmetic of the reference's generic reorder
 * (src/cpu/reorder/simple_reorder.hpp:2551-2635, destination scale inverted up front as in
 * src/cpu/reorder/cpu_reorder_pd.hpp:83-109).  Scale / zero-point elements are addressed as
 * b200_quant_t describes with (i0, i1) = (row, column); the destination zero-point is one
 * s32 value.  8 / 16 / 32-bit element types.  Replaces dnnl_reorder with scales and
 * zero-points attributes (src/common/reorder.cpp:63-160) for the tensors of this path:
 * quantising activations before an int8 matmul, dequantising its result. */
typedef struct {
    int64_t rows, cols;
    const void *src; int32_t src_dt; int32_t reserved0; int64_t src_s0, src_s1;
    void *dst; int32_t dst_dt; int32_t reserved1; int64_t dst_s0, dst_s1;
    b200_quant_t src_scale, dst_scale, src_zp, dst_zp;
    float beta; int32_t reserved2;
} b200_reorder_quant_params_t;

B200_API int b200_reorder_quant_launch(const b200_reorder_quant_params_t *p, b200_stream_t stream);

/* s32 column sums of plain 8-bit weights: out[n] = sum_k w[k][n]
 * (the zero-point compensation the reference computes at reorder time,
 * src/cpu/x64/matmul/brgemm_matmul.cpp:1184-1200) */
B200_API int b200_colsum_launch(const void *wei, int32_t wei_dt, int64_t K, int64_t N, int64_t sk, int64_t sn,
        int32_t *out, b200_stream_t stream);

/* ---- multi-GPU ----------------------------------------------------------- */

/* N-split matmul: every rank computes the columns [r*N/parts, (r+1)*N/parts) of dst
 * (its slice of the weights, per-N scales and bias; src replicated), the slices are
 * all-gathered rank by rank into `staged` = [parts][M][N/parts], and this kernel
 * lays them out as one row-major (M, N) matrix.  The reference has no multi-device
 * matmul; the split follows from dst elements being independent given a full K
 * reduction (ref_matmul_int8.cpp:154-261 computes each (m, n) on its own). */
B200_API int b200_gather_columns_launch(const void *staged, void *dst, int64_t M, int64_t N, int32_t parts,
        int32_t elem_bytes, b200_stream_t stream);

/* ---- utilities ----------------------------------------------------------- */

/* Test hook for the bounded-wait mechanism every kernel here uses: one warp polls an
 * mbarrier that is never completed, at most max_polls (<= 2^20) times 100 ns, then ORs
 * B200_STATUS_SELFTEST_WAIT into *status and returns.  The context stays usable. */
#define B200_STATUS_SELFTEST_WAIT 0x80000000u
B200_API int b200_selftest_bounded_wait_launch(uint32_t *status, uint32_t max_polls, b200_stream_t stream);

/* The tensor-pipe peak as measured with this library's own instruction: one CTA per SM issues
 * `iters` groups of four tcgen05.mma (kind::i8, or kind::f8f6f4 when fp8 != 0; 128 x 256 x 32 each)
 * on operands resident in shared memory -- no copies, no epilogue.  The caller times the launch
 * with CUDA events; *ops_out receives the operations it performs (2 x MACs).  The denominator the
 * dense kernels' roofline fraction can be quoted against besides the bf16-derived proxy.  No
 * counterpart in the reference. */
B200_API int b200_tc8_mma_peak_launch(int32_t fp8, uint32_t iters, uint32_t *status, uint64_t *ops_out, b200_stream_t stream);

/* number of kernel launches issued by this library since load (for benchmarks) */
B200_API uint64_t b200_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif
