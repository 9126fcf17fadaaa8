// The matmul primitive descriptor: validation, implementation dispatch, and the
// lowering of (descriptor, attribute, runtime arguments) into the kernel
// parameter block.
//
// Validation restates the rules of the reference's matmul_desc_init and
// matmul_attr_check (src/common/matmul.cpp:284-409 and :40-278) with the same
// status codes: inconsistent descriptors are dnnl_invalid_arguments, valid but
// unsupported attribute combinations are dnnl_unimplemented.  Dispatch walks
// this engine's implementation list the way the reference's
// primitive_desc_iterator_t walks an impl_list_item_t[]
// (src/common/primitive_desc_iterator.hpp:67-94): the first implementation whose
// init accepts the problem wins, dnnl_primitive_desc_next_impl resumes after it.
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>

#include "internal.hpp"

namespace b200 {

#define INVALID_IF(cond) \
    do { \
        if (cond) return dnnl_invalid_arguments; \
    } while (0)
#define UNIMPL_IF(cond) \
    do { \
        if (cond) return dnnl_unimplemented; \
    } while (0)

static bool one_of(int64_t v, int64_t a, int64_t b) { return v == a || v == b; }

dnnl_status_t matmul_validate(const dnnl_memory_desc &src, const dnnl_memory_desc &wei, const dnnl_memory_desc *bias,
        const dnnl_memory_desc &dst, const dnnl_primitive_attr &attr) {
    const bool with_bias = bias && bias->ndims != 0;
    const int ndims = dst.ndims;
    INVALID_IF(ndims < 2 || ndims > DNNL_MAX_NDIMS);
    INVALID_IF(src.ndims != ndims || wei.ndims != ndims);
    INVALID_IF(with_bias && bias->ndims != ndims);
    const int m_idx = ndims - 2, n_idx = ndims - 1;
    INVALID_IF(dst.dims[m_idx] != src.dims[m_idx]);
    INVALID_IF(dst.dims[n_idx] != wei.dims[n_idx]);
    INVALID_IF(src.dims[n_idx] != wei.dims[m_idx]);
    INVALID_IF(with_bias && !one_of(bias->dims[n_idx], 1, dst.dims[n_idx]));
    INVALID_IF(with_bias && !one_of(bias->dims[m_idx], 1, dst.dims[m_idx]));
    INVALID_IF(dt_is_int4(wei.data_type) && wei.dims[n_idx] % 2 != 0);
    INVALID_IF(dt_is_int4(src.data_type) && src.dims[n_idx] % 2 != 0);
    for (int d = 0; d < ndims - 2; ++d) {
        const int64_t s = src.dims[d], w = wei.dims[d], o = dst.dims[d];
        if (s == DNNL_RUNTIME_DIM_VAL || w == DNNL_RUNTIME_DIM_VAL || o == DNNL_RUNTIME_DIM_VAL) {
            INVALID_IF(!(s == DNNL_RUNTIME_DIM_VAL && w == DNNL_RUNTIME_DIM_VAL && o == DNNL_RUNTIME_DIM_VAL));
            continue;
        }
        INVALID_IF(!(s == w && w == o) && !(s == 1 || w == 1));
        INVALID_IF(s == 1 && o != w);
        INVALID_IF(w == 1 && o != s);
        INVALID_IF(with_bias && !one_of(bias->dims[d], 1, o));
    }
    // accumulation type must exist for the (src, weights) pair (type_helpers.hpp:444-460)
    const int sdt = src.data_type, wdt = wei.data_type, ddt = dst.data_type;
    const bool src_int8 = dt_is_int8(sdt), src_fp8 = dt_is_fp8(sdt);
    const bool wei_int = dt_is_int8(wdt) || dt_is_int4(wdt);
    const bool src_fp = sdt == dnnl_f32 || sdt == dnnl_bf16 || sdt == dnnl_f16;
    INVALID_IF(!dt_known(sdt) || !dt_known(wdt) || !dt_known(ddt));
    UNIMPL_IF(!dt_valid(sdt) || !dt_valid(wdt) || !dt_valid(ddt)); // f64, e8m0, f4: descriptors only
    INVALID_IF(!(src_int8 || src_fp8 || src_fp));

    // ---- attribute rules ----
    const int src_qmask_M = 1 << (ndims - 2), src_qmask_K = 1 << (ndims - 1);
    const int wei_qmask_K = 1 << (ndims - 2), wei_qmask_N = 1 << (ndims - 1);
    const bool wei_fp8 = dt_is_fp8(wdt);
    for (auto &kv : attr.zero_points)
        if (kv.second.set) {
            // zero-points need an int8 / fp8 source, or integer / fp8 weights
            // (the latter is weights decompression)
            UNIMPL_IF(!(src_int8 || src_fp8 || wei_int || wei_fp8));
            UNIMPL_IF(kv.first != DNNL_ARG_SRC && kv.first != DNNL_ARG_WEIGHTS && kv.first != DNNL_ARG_DST);
        }
    for (auto &kv : attr.scales)
        if (kv.second.set)
            UNIMPL_IF(kv.first != DNNL_ARG_SRC && kv.first != DNNL_ARG_WEIGHTS && kv.first != DNNL_ARG_DST);

    int64_t src_sc_gk = 1, wei_sc_gk = 1;
    const quant_entry_t &ss = attr.scale(DNNL_ARG_SRC);
    if (ss.set) {
        UNIMPL_IF(!(ss.mask == 0 || ss.mask == src_qmask_K || ss.mask == src_qmask_M + src_qmask_K));
        if (ss.group_ndims && (ss.mask & src_qmask_K)) src_sc_gk = ss.groups[1];
        UNIMPL_IF(src_sc_gk > 1 && src_sc_gk % 32 != 0);
    }
    const quant_entry_t &ws = attr.scale(DNNL_ARG_WEIGHTS);
    if (ws.set) {
        int64_t gn = 1;
        if (ws.group_ndims) {
            if (ws.mask & wei_qmask_K) wei_sc_gk = ws.groups[0];
            if (ws.mask & wei_qmask_N) gn = ws.groups[1];
        }
        UNIMPL_IF(gn > 1 && !attr.apply_to_int);
        UNIMPL_IF(wei_sc_gk > 1 && wei_sc_gk % 32 != 0);
        UNIMPL_IF(gn > 1 && gn % 32 != 0);
        UNIMPL_IF(!wei_int && !wei_fp8 && ws.group_ndims && (wei_sc_gk > 1 || gn > 1));
    }
    const quant_entry_t &ds = attr.scale(DNNL_ARG_DST);
    if (ds.set) {
        const int dst_qmask_M = src_qmask_M, dst_qmask_N = wei_qmask_N;
        UNIMPL_IF(!(ds.mask == 0 || ds.mask == dst_qmask_N || ds.mask == dst_qmask_M
                || ds.mask == dst_qmask_N + dst_qmask_M));
    }
    if (src_sc_gk > 1) {
        UNIMPL_IF(!(src_int8 || src_fp8));
        UNIMPL_IF(wei_sc_gk > 1 && !(src_sc_gk % wei_sc_gk == 0 || wei_sc_gk % src_sc_gk == 0));
    }

    int64_t src_zp_gk = 1, wei_zp_gk = 1;
    const quant_entry_t &sz = attr.zp(DNNL_ARG_SRC);
    if (sz.set) {
        UNIMPL_IF(!(sz.mask == 0 || sz.mask == src_qmask_K || sz.mask == src_qmask_M + src_qmask_K));
        if (sz.group_ndims && (sz.mask & src_qmask_K)) src_zp_gk = sz.groups[1];
        UNIMPL_IF(src_zp_gk > 1 && src_zp_gk % 32 != 0);
    }
    const quant_entry_t &wz = attr.zp(DNNL_ARG_WEIGHTS);
    if (wz.set) {
        int64_t gn = 1;
        if (wz.group_ndims) {
            if (wz.mask & wei_qmask_K) wei_zp_gk = wz.groups[0];
            if (wz.mask & wei_qmask_N) gn = wz.groups[1];
        }
        UNIMPL_IF(gn > 1 && !attr.apply_to_int);
        UNIMPL_IF(wei_zp_gk > 1 && wei_zp_gk % 32 != 0);
        UNIMPL_IF(gn > 1 && gn % 32 != 0);
        if (dt_is_int4(wz.dt)) {
            UNIMPL_IF((wz.mask & wei_qmask_K) && wei.dims[m_idx] % 2 != 0);
            UNIMPL_IF((wz.mask & wei_qmask_N) && wei.dims[n_idx] % 2 != 0);
        }
    }
    const quant_entry_t &dz = attr.zp(DNNL_ARG_DST);
    if (dz.set) UNIMPL_IF(!(dz.mask == 0 || (ndims == 2 && dz.mask == 2)));
    if (src_zp_gk > 1) {
        UNIMPL_IF(!src_int8);
        UNIMPL_IF(wei_zp_gk > 1 && !(src_zp_gk % wei_zp_gk == 0 || wei_zp_gk % src_zp_gk == 0));
    }

    // post-ops: sum consistency (primitive_attr.cpp:289-329) and binary broadcast
    bool seen_sum_dt = false;
    int sum_dt = dnnl_data_type_undef;
    for (auto &e : attr.post_ops.entries) {
        if (e.kind == dnnl_sum) {
            const int sdt_eff = e.dt == dnnl_data_type_undef ? ddt : e.dt;
            UNIMPL_IF(dt_nbits(sdt_eff) != dt_nbits(ddt));
            UNIMPL_IF(e.zero_point != 0 && !src_int8);
            UNIMPL_IF(seen_sum_dt && sum_dt != e.dt);
            seen_sum_dt = true;
            sum_dt = e.dt;
        } else if (e.kind == dnnl_binary) {
            INVALID_IF(e.src1.ndims != ndims);
            // (a dst dim known only at execution is checked then, on the concrete descriptors)
            for (int d = 0; d < ndims; ++d)
                INVALID_IF(dst.dims[d] != DNNL_RUNTIME_DIM_VAL && !one_of(e.src1.dims[d], 1, dst.dims[d]));
        } else if (e.kind != dnnl_eltwise && e.kind != dnnl_prelu) {
            return dnnl_unimplemented;
        }
    }
    return dnnl_success;
}

// ---- implementation acceptance ---------------------------------------------------

static void make_plain(dnnl_memory_desc &md, bool transposed = false) {
    md.format_kind = dnnl_blocked;
    md.packed_layout = B200_WEI_PLAIN;
    int64_t s = 1;
    if (transposed && md.ndims >= 2) {
        const int a = md.ndims - 2, b = md.ndims - 1;
        md.strides[a] = 1;
        md.strides[b] = md.dims[a];
        s = md.dims[a] * md.dims[b];
        for (int i = md.ndims - 3; i >= 0; --i) {
            md.strides[i] = s;
            s *= md.dims[i] > 0 ? md.dims[i] : 1;
        }
        return;
    }
    for (int i = md.ndims - 1; i >= 0; --i) {
        md.strides[i] = s;
        s *= md.dims[i] > 0 ? md.dims[i] : 1;
    }
}

static bool quant_simple(const quant_entry_t &q, int allowed_masks_bits) {
    if (!q.set) return true;
    if (q.mask & ~allowed_masks_bits) return false;
    if (q.group_ndims && (q.groups[0] > 1 || q.groups[1] > 1)) return false;
    return true;
}

static const char *reject(const char *impl, const char *why) {
    verbose_dispatch(impl, why);
    return why;
}

// How the tensor-core kernel gets at 8-bit weights.  One rule for dispatch, scratchpad sizing and
// execution: plain weights are read in place only when they are K-major with a pitch and an
// offset the TMA descriptor accepts (multiples of 16 bytes); N-major weights -- which includes
// a single column, whose two strides are both 1 -- are transposed into the scratchpad.
enum tc8_wei_class_t { TC8_WEI_PACKED, TC8_WEI_INPLACE_KMAJOR, TC8_WEI_PACK_NMAJOR, TC8_WEI_UNSUPPORTED };
static tc8_wei_class_t tc8_weights_class(const dnnl_memory_desc &wei) {
    if (wei.format_kind == dnnl_format_kind_opaque)
        return wei.packed_layout == B200_WEI_KMAJOR ? TC8_WEI_PACKED : TC8_WEI_UNSUPPORTED;
    if (!wei.is_plain()) return TC8_WEI_PACKED; // format_tag::any resolves to the packed layout
    if (wei.strides[0] == 1 && wei.strides[1] % 16 == 0 && wei.offset0 % 16 == 0) return TC8_WEI_INPLACE_KMAJOR;
    if (wei.strides[1] == 1) return TC8_WEI_PACK_NMAJOR;
    return TC8_WEI_UNSUPPORTED;
}

// dense 8-bit tensor-core GEMM
static bool accept_tc8(dnnl_primitive_desc *pd) {
    const char *name = "cuda:sm100:tcgen05";
    const dnnl_memory_desc &src = pd->user_src, &wei = pd->user_wei, &dst = pd->user_dst;
    const dnnl_primitive_attr &a = pd->attr;
    if (src.ndims != 2) return reject(name, "only 2-D problems"), false;
    const int sdt = src.data_type, wdt = wei.data_type;
    const bool i8 = dt_is_int8(sdt) && dt_is_int8(wdt);
    const bool f8 = dt_is_fp8(sdt) && dt_is_fp8(wdt);
    if (!i8 && !f8) return reject(name, "needs 8-bit src and weights"), false;
    const int64_t M = src.dims[0], K = src.dims[1], N = wei.dims[1];
    if (M == 0 || N == 0 || K == 0) return reject(name, "zero dim"), false;
    if (K % 16 != 0) return reject(name, "K must be a multiple of 16 (TMA row pitch)"), false;
    if (src.is_plain() && !(src.strides[1] == 1 && src.strides[0] % 16 == 0 && src.offset0 % 16 == 0))
        return reject(name, "src must be row-major with a 16-byte pitch"), false;
    if (dst.is_plain() && dst.strides[1] != 1) return reject(name, "dst must be row-major"), false;
    if (tc8_weights_class(wei) == TC8_WEI_UNSUPPORTED)
        return reject(name, wei.format_kind == dnnl_format_kind_opaque ? "unknown packed weights layout" : "weights strides not supported"), false;
    // source scales: one per tensor, or one per row -- what dynamic (per-token) quantisation of the
    // activations produces; the API spells it mask M+K with one group spanning all of K
    const quant_entry_t &ssc = a.scale(DNNL_ARG_SRC);
    const bool src_per_row = i8 && ssc.set && ssc.mask == 3 && ssc.group_ndims == 2 && ssc.groups[0] == 1 && ssc.groups[1] == K
            && ssc.dt == dnnl_f32;
    if (!src_per_row && !quant_simple(ssc, 0)) return reject(name, "src scales must be per-tensor or per-row"), false;
    if (!quant_simple(a.scale(DNNL_ARG_WEIGHTS), 2)) return reject(name, "weights scales must be per-tensor or per-N"), false;
    if (!quant_simple(a.scale(DNNL_ARG_DST), 0)) return reject(name, "dst scales must be per-tensor"), false;
    if (!quant_simple(a.zp(DNNL_ARG_SRC), 0)) return reject(name, "src zero-point must be per-tensor"), false;
    // weights zero-points, one per tensor or per column: folded in by the epilogue from the row sums of src
    if (!quant_simple(a.zp(DNNL_ARG_WEIGHTS), 2)) return reject(name, "weights zero-points must be per-tensor or per-N"), false;
    if (!quant_simple(a.zp(DNNL_ARG_DST), 2)) return reject(name, "dst zero-point mask"), false;
    if (f8 && (a.zp(DNNL_ARG_SRC).set || a.zp(DNNL_ARG_WEIGHTS).set)) return reject(name, "fp8 with zero-points"), false;
    // resolve layouts
    pd->src = src;
    if (src.is_any()) make_plain(pd->src);
    pd->dst = dst;
    if (dst.is_any()) make_plain(pd->dst);
    pd->wei = wei;
    if (wei.is_any()) {
        pd->wei.format_kind = dnnl_format_kind_opaque;
        pd->wei.packed_layout = B200_WEI_KMAJOR;
    }
    pd->impl_str = i8 ? "cuda:sm100:tcgen05_i8" : "cuda:sm100:tcgen05_f8";
    return true;
}

// weight-compressed GEMV / skinny GEMM
static bool accept_wc(dnnl_primitive_desc *pd) {
    const char *name = "cuda:sm100:wc_gemv";
    const dnnl_memory_desc &src = pd->user_src, &wei = pd->user_wei, &dst = pd->user_dst;
    const dnnl_primitive_attr &a = pd->attr;
    if (src.ndims != 2) return reject(name, "only 2-D problems"), false;
    const int sdt = src.data_type, wdt = wei.data_type;
    if (!(sdt == dnnl_bf16 || sdt == dnnl_f16 || sdt == dnnl_f32)) return reject(name, "src must be bf16/f16/f32"), false;
    const bool w8 = wdt == dnnl_s8 || wdt == dnnl_u8;
    if (!(dt_is_int4(wdt) || w8) || !a.apply_to_int) return reject(name, "needs 4- or 8-bit weights with fpmath apply_to_int"), false;
    const int64_t M = src.dims[0], K = src.dims[1], N = wei.dims[1];
    if (M == 0 || N == 0 || K == 0) return reject(name, "zero dim"), false;
    if ((!w8 && N % 16 != 0) || K % 64 != 0) return reject(name, "needs N % 16 == 0 and K % 64 == 0"), false;
    if (src.is_plain() && !(src.strides[1] == 1 && src.strides[0] % 8 == 0 && src.offset0 % 8 == 0))
        return reject(name, "src must be row-major with 16-byte aligned rows"), false;
    if (dst.is_plain() && dst.strides[1] != 1) return reject(name, "dst must be row-major"), false;
    if (!w8 && wei.is_plain() && !(wei.strides[1] == 1 && wei.strides[0] == N && wei.offset0 == 0))
        return reject(name, "weights must be dense ab"), false;
    if (wei.format_kind == dnnl_format_kind_opaque && wei.packed_layout != B200_WEI_WC4_TILED
            && wei.packed_layout != B200_WEI_WC4_TC && wei.packed_layout != B200_WEI_WC8_TC)
        return reject(name, "unknown packed weights layout"), false;
    if (!quant_simple(a.scale(DNNL_ARG_SRC), 0)) return reject(name, "src scales must be per-tensor"), false;
    if (!quant_simple(a.scale(DNNL_ARG_DST), 0)) return reject(name, "dst scales must be per-tensor"), false;
    int64_t gks[2] = {K, K};
    int gi = 0;
    for (const quant_entry_t *q : {&a.scale(DNNL_ARG_WEIGHTS), &a.zp(DNNL_ARG_WEIGHTS)}) {
        const int i = gi++;
        if (!q->set) continue;
        if (q->group_ndims && (q->mask & 2) && q->groups[1] != 1) return reject(name, "groups along N not supported"), false;
        const int64_t gk = (q->mask & 1) ? (q->group_ndims ? q->groups[0] : 1) : K;
        if (gk % 64 != 0 || K % gk != 0) return reject(name, "K group must be a multiple of 64 that divides K"), false;
        gks[i] = gk;
    }
    if (gks[0] % gks[1] != 0 && gks[1] % gks[0] != 0) return reject(name, "scale and zero-point groups must nest"), false;
    if (a.zp(DNNL_ARG_SRC).set || a.zp(DNNL_ARG_DST).set) return reject(name, "src/dst zero-points"), false;
    pd->src = src;
    if (src.is_any()) make_plain(pd->src);
    pd->dst = dst;
    if (dst.is_any()) make_plain(pd->dst);
    // More activation rows than one pass of the decode kernel takes (32): the tensor-core kernel
    // (weights converted to bf16 in shared memory; its time hardly depends on M, the decode
    // kernel's grows with every pass), when it can take the problem: bf16 src, bf16 scales,
    // 4-bit zero-points.
    const quant_entry_t &ws = a.scale(DNNL_ARG_WEIGHTS), &wz = a.zp(DNNL_ARG_WEIGHTS);
    bool tc = M > 32 && sdt == dnnl_bf16 && (!ws.set || ws.dt == dnnl_bf16) && (!wz.set || dt_is_int4(wz.dt))
            && !(wz.set && wz.mask == 0); // a 4-bit zero-point needs a mask (the attribute check says so too)
    if (w8) {
        // 8-bit weights: the tensor-core kernel for any M (there is no 8-bit decode kernel); it converts
        // in f32, so any float scale and any integer zero-point type will do
        tc = sdt == dnnl_bf16 && (!ws.set || ws.dt == dnnl_bf16 || ws.dt == dnnl_f16 || ws.dt == dnnl_f32)
                && (!wz.set || dt_is_int4(wz.dt) || wz.dt == dnnl_s8 || wz.dt == dnnl_u8 || wz.dt == dnnl_s32);
        if (!tc) return reject(name, "8-bit weights need bf16 src and float scales"), false;
    }
    if (const char *v = std::getenv("ONEDNN_CUDA_DISABLE_IMPL"))
        if (std::string(v).find("wc_tc") != std::string::npos) tc = false;
    if (const char *v = std::getenv("ONEDNN_CUDA_DISABLE_IMPL"))
        if (w8 && std::string(v).find("wc_tc") != std::string::npos) return reject(name, "disabled"), false;
    if (!tc && M > 512) return reject(name, "M too large for the decode kernel"), false;
    if (wei.format_kind == dnnl_format_kind_opaque) {
        // the layout was fixed when the weights were packed: it decides
        const bool packed_tc = wei.packed_layout == B200_WEI_WC4_TC || wei.packed_layout == B200_WEI_WC8_TC;
        if (packed_tc && !tc) return reject(name, "weights packed for the tensor-core kernel"), false;
        if ((wei.packed_layout == B200_WEI_WC8_TC) != w8) return reject(name, "packed layout of another weight width"), false;
        tc = packed_tc;
    }
    pd->wei = wei;
    if (wei.is_any()) {
        pd->wei.format_kind = dnnl_format_kind_opaque;
        pd->wei.packed_layout = w8 ? B200_WEI_WC8_TC : (tc ? B200_WEI_WC4_TC : B200_WEI_WC4_TILED);
    }
    pd->impl_str = tc ? "cuda:sm100:wc_tcgen05" : "cuda:sm100:wc_gemv";
    return true;
}

static bool accept_generic(dnnl_primitive_desc *pd) {
    const char *name = "cuda:generic";
    if (pd->user_src.ndims != 2) return reject(name, "only 2-D problems"), false;
    if (pd->user_wei.format_kind == dnnl_format_kind_opaque) return reject(name, "packed weights"), false;
    const int sdt = pd->user_src.data_type, wdt = pd->user_wei.data_type;
    const bool src_int8 = dt_is_int8(sdt);
    const bool wei_int = dt_is_int8(wdt) || dt_is_int4(wdt);
    // the (src, weights) type pairs of the reference's two scalar implementations
    if (src_int8 && !wei_int) return reject(name, "int8 src needs integer weights"), false;
    if (!src_int8 && wei_int && !pd->attr.apply_to_int && !dt_is_fp8(sdt))
        return reject(name, "integer weights with a float src need fpmath apply_to_int"), false;
    // group sizes must divide K / N
    const int64_t K = pd->user_src.dims[1], N = pd->user_wei.dims[1];
    for (int arg : {DNNL_ARG_SRC, DNNL_ARG_WEIGHTS}) {
        for (const quant_entry_t *q : {&pd->attr.scale(arg), &pd->attr.zp(arg)}) {
            if (!q->set || !q->group_ndims) continue;
            const int64_t gk = arg == DNNL_ARG_SRC ? q->groups[1] : q->groups[0];
            const int64_t gn = arg == DNNL_ARG_SRC ? 1 : q->groups[1];
            if (gk <= 0 || gn <= 0 || K % gk != 0 || N % gn != 0) return reject(name, "group must divide the dim"), false;
        }
    }
    if (!src_int8) {
        if (pd->attr.zp(DNNL_ARG_SRC).set || pd->attr.zp(DNNL_ARG_DST).set)
            return reject(name, "src/dst zero-points need an int8 src"), false;
        if (pd->attr.scale(DNNL_ARG_SRC).set && pd->attr.scale(DNNL_ARG_SRC).mask != 0)
            return reject(name, "src scale mask"), false;
    }
    if (pd->attr.scale(DNNL_ARG_DST).set && pd->attr.scale(DNNL_ARG_DST).mask != 0)
        return reject(name, "dst scale mask"), false;
    pd->src = pd->user_src;
    if (pd->src.is_any()) make_plain(pd->src);
    pd->wei = pd->user_wei;
    if (pd->wei.is_any()) make_plain(pd->wei);
    pd->dst = pd->user_dst;
    if (pd->dst.is_any()) make_plain(pd->dst);
    pd->impl_str = "cuda:generic";
    return true;
}

// tcgen05 8-bit implementation: the part of the scratchpad that holds weights-side data (the
// row sums of src, needed with weights zero-points, follow it at a 256-byte boundary)
static size_t tc8_weights_scratch_bytes(const dnnl_primitive_desc *pd) {
    const int64_t K = pd->K(), N = pd->N();
    size_t bytes = 0;
    // plain N-major weights are transposed into the packed layout on every
    // execution; plain K-major weights only need the column sums
    const tc8_wei_class_t wc = tc8_weights_class(pd->wei);
    if (wc == TC8_WEI_PACK_NMAJOR)
        bytes = b200_packed_weights_bytes(K, N, pd->wei.data_type, B200_WEI_KMAJOR);
    else if (wc == TC8_WEI_INPLACE_KMAJOR && pd->attr.zp(DNNL_ARG_SRC).set)
        bytes = (size_t)N * sizeof(int32_t);
    return (bytes + 255) / 256 * 256;
}

static size_t scratch_bytes_for(const dnnl_primitive_desc *pd) {
    size_t bytes = 0;
    if (pd->impl == IMPL_TC8) {
        bytes = tc8_weights_scratch_bytes(pd);
        if (pd->attr.zp(DNNL_ARG_WEIGHTS).set) bytes += (size_t)pd->M() * sizeof(int32_t);
    }
    if (pd->impl == IMPL_WC) {
        b200_matmul_params_t q;
        std::memset(&q, 0, sizeof(q));
        q.M = pd->M();
        q.N = pd->N();
        q.K = pd->K();
        q.src_dt = pd->src.data_type;
        q.wei_layout = pd->wei.format_kind == dnnl_format_kind_opaque ? pd->wei.packed_layout : B200_WEI_PLAIN;
        if (pd->impl_str.find("tcgen05") != std::string::npos)
            bytes = q.wei_layout == B200_WEI_PLAIN ? b200_wc_tc_packed_bytes(q.K, q.N, pd->wei.data_type) : 0; // plain weights are packed per execution
        else
            bytes = b200_matmul_scratch_bytes(&q, 2);
    }
    return (bytes + 255) / 256 * 256;
}

// debugging knob: ONEDNN_CUDA_DISABLE_IMPL=tc8,wc takes implementations out of the list
static bool impl_disabled(int id) {
    const char *v = std::getenv("ONEDNN_CUDA_DISABLE_IMPL");
    if (!v) return false;
    const std::string s(v);
    return (id == IMPL_TC8 && s.find("tc8") != std::string::npos) || (id == IMPL_WC && s.find("wc") != std::string::npos);
}

// ---- batched problems -------------------------------------------------------------------
// The reference's matmul takes any number of leading batch dims, each equal in src, weights
// and dst or 1 (broadcast) in src or weights (src/common/matmul.cpp:374-401); every batch
// index is an independent 2-D problem (ref_matmul_int8.cpp:154-170 loops over it).  Here the
// descriptor of one 2-D slice goes through the ordinary dispatch, and execution runs it once
// per batch index on the same stream.

// the last two dims of md as a 2-D descriptor
static dnnl_memory_desc slice_2d(const dnnl_memory_desc &md) {
    dnnl_memory_desc r = md;
    if (r.is_any()) make_plain(r);
    dnnl_memory_desc o;
    o.ndims = 2;
    o.data_type = r.data_type;
    o.format_kind = r.format_kind;
    o.packed_layout = r.packed_layout;
    for (int i = 0; i < 2; ++i) {
        o.dims[i] = r.dims[r.ndims - 2 + i];
        o.strides[i] = r.strides[r.ndims - 2 + i];
    }
    return o;
}

// (batch..., R, C) seen as (prod(batch) * R, C): possible when the batch dims and R form one dense run of rows
static bool collapse_rows(const dnnl_memory_desc &md, int nb, dnnl_memory_desc &out) {
    dnnl_memory_desc r = md;
    if (r.is_any()) make_plain(r);
    if (!r.is_plain()) return false;
    const int nd = r.ndims;
    int64_t rows = r.dims[nd - 2];
    for (int d = nb - 1; d >= 0; --d) {
        if (r.strides[d] != r.strides[d + 1] * r.dims[d + 1]) return false;
        rows *= r.dims[d];
    }
    out = dnnl_memory_desc();
    out.ndims = 2;
    out.data_type = r.data_type;
    out.format_kind = r.format_kind;
    out.packed_layout = r.packed_layout;
    out.offset0 = r.offset0;
    out.dims[0] = rows;
    out.dims[1] = r.dims[nd - 1];
    out.strides[0] = r.strides[nd - 2];
    out.strides[1] = r.strides[nd - 1];
    return true;
}

// A batched problem whose weights are the same for every batch index (all their batch dims 1) and
// whose src and dst rows run densely through the batch dims is one 2-D matmul with
// prod(batch) * M rows: one launch instead of one per batch index.  Everything that varies with
// the row inside a batch index (per-row quantisation, a prelu mask over M, a binary operand that
// is neither per-column nor a full dense tensor) keeps the per-index form.
static bool collapsible(const dnnl_primitive_desc *pd, int nb, dnnl_memory_desc &src2, dnnl_memory_desc &dst2,
        std::vector<dnnl_memory_desc> &src1_2d) {
    for (int d = 0; d < nb; ++d)
        if (pd->user_wei.dims[d] != 1) return false;
    if (pd->user_src.is_any() || pd->user_dst.is_any()) return false; // `any` would be dense, but keep the given-layout rule simple
    if (!collapse_rows(pd->user_src, nb, src2) || !collapse_rows(pd->user_dst, nb, dst2)) return false;
    if (dt_nbits(src2.data_type) == 4 || dt_nbits(dst2.data_type) == 4) return false;
    if (pd->user_bias.ndims)
        for (int d = 0; d <= nb; ++d)
            if (pd->user_bias.dims[d] != 1) return false;
    for (auto *m : {&pd->attr.scales, &pd->attr.zero_points})
        for (auto &kv : *m)
            if (kv.second.set && kv.first != DNNL_ARG_WEIGHTS && (kv.second.mask & (1 << nb))) return false; // varies along M
    const auto &po = pd->attr.post_ops.entries;
    src1_2d.assign(po.size(), dnnl_memory_desc());
    for (size_t i = 0; i < po.size(); ++i) {
        if (po[i].kind == dnnl_prelu && (po[i].mask & (1 << nb))) return false;
        if (po[i].kind != dnnl_binary) continue;
        const dnnl_memory_desc &s1 = po[i].src1;
        bool all_one = true, all_full = true;
        for (int d = 0; d <= nb; ++d) {
            all_one = all_one && s1.dims[d] == 1;
            all_full = all_full && s1.dims[d] == pd->user_dst.dims[d];
        }
        if (all_one) src1_2d[i] = slice_2d(s1);
        else if (!(all_full && !s1.is_any() && collapse_rows(s1, nb, src1_2d[i]))) return false;
    }
    return true;
}

static dnnl_status_t select_batched(dnnl_primitive_desc *pd, int first) {
    const int nd = pd->user_dst.ndims, nb = nd - 2;
    if (pd->user_src.format_kind == dnnl_format_kind_opaque || pd->user_dst.format_kind == dnnl_format_kind_opaque)
        return first == 0 ? dnnl_unimplemented : dnnl_last_impl_reached; // packed layouts are for weights
    auto in = std::make_shared<dnnl_primitive_desc>();
    in->kind = dnnl_matmul;
    in->engine = pd->engine; // not counted: the slice descriptor lives and dies with this one
    in->attr = pd->attr;
    // scales / zero-points: the mask's bits over the last two dims move down with them; bits over batch
    // dims mean one set of values per index of those dims, handed to the slice's execution part by part
    pd->batch_quant.clear();
    for (auto *m : {&in->attr.scales, &in->attr.zero_points})
        for (auto &kv : *m) {
            if (!kv.second.set) continue;
            const int bmask = kv.second.mask & ((1 << nb) - 1);
            if (bmask) {
                if (kv.second.group_ndims) return first == 0 ? dnnl_unimplemented : dnnl_last_impl_reached; // groups are over the last two dims
                dnnl_primitive_desc::batch_quant_t q;
                q.exec_arg = (m == &in->attr.scales ? DNNL_ARG_ATTR_SCALES : DNNL_ARG_ATTR_ZERO_POINTS) | kv.first;
                q.tensor_arg = kv.first;
                q.batch_mask = bmask;
                q.is_zp = m != &in->attr.scales;
                pd->batch_quant.push_back(q);
            }
            kv.second.mask >>= nb;
        }
    for (auto &e : in->attr.post_ops.entries)
        if (e.kind == dnnl_binary && e.src1.ndims != nd) return dnnl_invalid_arguments;
    dnnl_memory_desc src2, dst2;
    std::vector<dnnl_memory_desc> src1_2d;
    const bool collapse = pd->batch_quant.empty() && collapsible(pd, nb, src2, dst2, src1_2d);
    for (size_t i = 0; i < in->attr.post_ops.entries.size(); ++i) {
        auto &e = in->attr.post_ops.entries[i];
        if (e.kind == dnnl_binary) {
            e.src1 = collapse ? src1_2d[i] : slice_2d(e.src1);
        } else if (e.kind == dnnl_prelu) {
            if (e.mask & ((1 << nb) - 1)) return first == 0 ? dnnl_unimplemented : dnnl_last_impl_reached;
            e.mask >>= nb;
        }
    }
    in->user_src = collapse ? src2 : slice_2d(pd->user_src);
    // weights given as `any` take the implementation's packed layout slice by slice: every batch
    // index's (K, N) matrix packed on its own, the slices one after the other (packed_slice_stride)
    if (pd->user_wei.is_any()) {
        in->user_wei = dnnl_memory_desc();
        in->user_wei.ndims = 2;
        in->user_wei.data_type = pd->user_wei.data_type;
        in->user_wei.format_kind = dnnl_format_kind_any;
        in->user_wei.dims[0] = pd->user_wei.dims[nd - 2];
        in->user_wei.dims[1] = pd->user_wei.dims[nd - 1];
    } else {
        in->user_wei = slice_2d(pd->user_wei);
    }
    in->user_dst = collapse ? dst2 : slice_2d(pd->user_dst);
    if (pd->user_bias.ndims) in->user_bias = slice_2d(pd->user_bias);
    // every batch index must start a 4-bit tensor on a byte: the 2-D slices are addressed by pointer
    for (const dnnl_memory_desc *md : {&pd->user_src, &pd->user_wei, &pd->user_dst}) {
        if (dt_nbits(md->data_type) != 4 || !md->is_plain()) continue;
        for (int d = 0; d < nb; ++d)
            if (md->dims[d] > 1 && (md->strides[d] & 1)) return first == 0 ? dnnl_unimplemented : dnnl_last_impl_reached;
    }
    const dnnl_status_t st = matmul_select_impl(in.get(), first);
    if (st != dnnl_success) return st;
    pd->src = pd->user_src;
    if (pd->src.is_any()) make_plain(pd->src);
    pd->wei = pd->user_wei;
    if (pd->wei.is_any()) {
        if (in->wei.format_kind == dnnl_format_kind_opaque) {
            pd->wei.format_kind = dnnl_format_kind_opaque;
            pd->wei.packed_layout = in->wei.packed_layout;
        } else {
            make_plain(pd->wei);
        }
    }
    pd->dst = pd->user_dst;
    if (pd->dst.is_any()) make_plain(pd->dst);
    pd->bias = pd->user_bias;
    if (pd->bias.ndims && pd->bias.is_any()) make_plain(pd->bias);
    pd->impl = in->impl;
    pd->impl_str = in->impl_str;
    pd->scratchpad = in->scratchpad;
    pd->inner = in;
    pd->collapsed = collapse;
    return dnnl_success;
}

// element offset of batch index `idx` (over dst's batch dims) in a tensor whose batch dims are 1 or dst's
static int64_t batch_offset(const dnnl_memory_desc &md, const int64_t *idx, int nb) {
    int64_t off = 0;
    for (int d = 0; d < nb; ++d)
        if (md.dims[d] != 1) off += idx[d] * md.strides[d];
    return off;
}

static dnnl_status_t batched_execute(const dnnl_primitive *prim, dnnl_stream *stream, const std::map<int, dnnl_memory *> &args) {
    const dnnl_primitive_desc *pd = prim->pd.get();
    const dnnl_primitive_desc *in = pd->inner.get();
    const int nb = pd->dst.ndims - 2;
    int64_t total = 1;
    for (int d = 0; d < nb; ++d) total *= pd->dst.dims[d];
    if (total == 0 || pd->dst.has_zero_dim() || pd->src.has_zero_dim() || pd->wei.has_zero_dim()) return dnnl_success;
    if (pd->collapsed) total = 1; // the inner descriptor is the whole problem: one execution from the tensors' starts
    // the tensors that move with the batch index, their N-D descriptors and their 2-D slices
    struct moving_t { int arg; const dnnl_memory_desc *full; dnnl_memory_desc slice; dnnl_memory mem; };
    std::vector<moving_t> mv;
    auto add = [&](int arg, const dnnl_memory_desc &full, const dnnl_memory_desc &slice) -> bool {
        auto it = args.find(arg);
        if (it == args.end() || !it->second->handle) return false;
        moving_t m;
        m.arg = arg;
        m.full = &full;
        m.slice = slice;
        m.mem = *it->second;
        mv.push_back(m);
        return true;
    };
    if (!add(DNNL_ARG_SRC, pd->src, in->src) || !add(DNNL_ARG_WEIGHTS, pd->wei, in->wei) || !add(DNNL_ARG_DST, pd->dst, in->dst))
        return dnnl_invalid_arguments;
    if (pd->bias.ndims && !add(DNNL_ARG_BIAS, pd->bias, in->bias)) return dnnl_invalid_arguments;
    const auto &po = pd->attr.post_ops.entries;
    std::vector<dnnl_memory_desc> po_full(po.size());
    for (size_t i = 0; i < po.size(); ++i)
        if (po[i].kind == dnnl_binary) {
            po_full[i] = po[i].src1;
            if (po_full[i].is_any()) make_plain(po_full[i]);
            if (!add(DNNL_ARG_ATTR_MULTIPLE_POST_OP((int)i) | DNNL_ARG_SRC_1, po_full[i], in->attr.post_ops.entries[i].src1))
                return dnnl_invalid_arguments;
        }
    // quantisation arguments that vary over batch dims: the part of batch index idx starts
    // (row-major index of idx over the masked batch dims of the argument's tensor) x (values per slice) in
    struct moving_quant_t { dnnl_memory mem; const dnnl_memory_desc *tensor; int batch_mask; int64_t per_slice; void *base0; int bits; };
    std::vector<moving_quant_t> mq;
    for (const auto &bq : pd->batch_quant) {
        auto it = args.find(bq.exec_arg);
        if (it == args.end() || !it->second->handle) return dnnl_invalid_arguments;
        const dnnl_memory_desc *t = bq.tensor_arg == DNNL_ARG_SRC ? &pd->src : bq.tensor_arg == DNNL_ARG_WEIGHTS ? &pd->wei : &pd->dst;
        const quant_entry_t &qe = bq.is_zp ? in->attr.zp(bq.tensor_arg) : in->attr.scale(bq.tensor_arg);
        moving_quant_t q;
        q.mem = *it->second;
        q.tensor = t;
        q.batch_mask = bq.batch_mask;
        q.per_slice = ((qe.mask & 1) ? t->dims[nb] : 1) * ((qe.mask & 2) ? t->dims[nb + 1] : 1);
        q.bits = dt_nbits(q.mem.md.data_type);
        q.base0 = (char *)q.mem.handle + q.mem.md.offset0 * q.bits / 8;
        int64_t sets = 1;
        for (int d = 0; d < nb; ++d)
            if (bq.batch_mask & (1 << d)) sets *= t->dims[d];
        if (q.mem.md.nelems() < sets * q.per_slice) return dnnl_invalid_arguments;
        // the slice's own descriptor: a 1-D run of per_slice values
        dnnl_memory_desc one;
        one.ndims = 1;
        one.data_type = q.mem.md.data_type;
        one.format_kind = dnnl_blocked;
        one.dims[0] = q.per_slice;
        one.strides[0] = 1;
        q.mem.md = one;
        q.mem.owned = false;
        q.mem.mapped = nullptr;
        mq.push_back(q);
    }
    std::vector<void *> base(mv.size());
    for (size_t i = 0; i < mv.size(); ++i) {
        base[i] = (char *)mv[i].mem.handle + mv[i].full->offset0 * dt_nbits(mv[i].full->data_type) / 8;
        mv[i].mem.md = mv[i].slice;
        mv[i].mem.owned = false;
        mv[i].mem.mapped = nullptr;
    }
    // a primitive of the slice descriptor that borrows this primitive's scratchpad
    dnnl_primitive tmp;
    tmp.pd = pd->inner;
    tmp.lib_scratch = prim->lib_scratch;
    tmp.lib_scratch_bytes = prim->lib_scratch_bytes;
    tmp.scratch_owner = prim->scratch_owner ? prim->scratch_owner : prim;
    std::map<int, dnnl_memory *> a2 = args;
    for (size_t i = 0; i < mv.size(); ++i) a2[mv[i].arg] = &mv[i].mem;
    for (size_t i = 0; i < mq.size(); ++i) a2[pd->batch_quant[i].exec_arg] = &mq[i].mem;
    dnnl_status_t st = dnnl_success;
    int64_t idx[DNNL_MAX_NDIMS] = {0};
    for (int64_t b = 0; b < total && st == dnnl_success; ++b) {
        int64_t rem = b;
        for (int d = nb - 1; d >= 0; --d) {
            idx[d] = rem % pd->dst.dims[d];
            rem /= pd->dst.dims[d];
        }
        for (size_t i = 0; i < mv.size(); ++i) {
            if (mv[i].full->format_kind == dnnl_format_kind_opaque) {
                // packed weights: slices in row-major order of the weights' own batch dims
                int64_t flat = 0;
                for (int d = 0; d < nb; ++d) flat = flat * mv[i].full->dims[d] + (mv[i].full->dims[d] != 1 ? idx[d] : 0);
                mv[i].mem.handle = (char *)base[i] + (size_t)flat * mv[i].full->packed_slice_stride();
                continue;
            }
            const int64_t off = batch_offset(*mv[i].full, idx, nb);
            const int bits = dt_nbits(mv[i].full->data_type);
            if ((off * bits) % 8 != 0) { st = dnnl_unimplemented; break; } // a 4-bit slice starting inside a byte
            mv[i].mem.handle = (char *)base[i] + off * bits / 8;
        }
        for (auto &q : mq) {
            int64_t flat = 0;
            for (int d = 0; d < nb; ++d)
                if (q.batch_mask & (1 << d)) flat = flat * q.tensor->dims[d] + (q.tensor->dims[d] != 1 ? idx[d] : 0);
            const int64_t off_bits = flat * q.per_slice * q.bits;
            if (off_bits % 8 != 0) { st = dnnl_unimplemented; break; } // a 4-bit part starting inside a byte
            q.mem.handle = (char *)q.base0 + off_bits / 8;
        }
        if (st == dnnl_success) st = matmul_execute(&tmp, stream, a2);
    }
    tmp.lib_scratch = nullptr; // borrowed
    tmp.pd.reset();
    return st;
}

// a descriptor with runtime dims admits the concrete one of a memory argument
static bool runtime_md_matches(const dnnl_memory_desc &decl, const dnnl_memory_desc &actual) {
    if (decl.ndims != actual.ndims || decl.data_type != actual.data_type || actual.has_runtime_dims()) return false;
    for (int i = 0; i < decl.ndims; ++i) {
        if (decl.dims[i] != DNNL_RUNTIME_DIM_VAL && decl.dims[i] != actual.dims[i]) return false;
        if (decl.is_plain() && actual.is_plain() && decl.strides[i] != DNNL_RUNTIME_DIM_VAL && decl.strides[i] != actual.strides[i])
            return false;
    }
    return true;
}

// Execution of a primitive created with runtime dims: the sizes come from the memory
// arguments; validation and dispatch run now, on a descriptor that lives for this call.
static dnnl_status_t runtime_execute(const dnnl_primitive *prim, dnnl_stream *stream, const std::map<int, dnnl_memory *> &args) {
    const dnnl_primitive_desc *pd = prim->pd.get();
    auto get = [&](int a) -> dnnl_memory * {
        auto it = args.find(a);
        return it == args.end() ? nullptr : it->second;
    };
    dnnl_memory *src = get(DNNL_ARG_SRC), *wei = get(DNNL_ARG_WEIGHTS), *dst = get(DNNL_ARG_DST), *bias = get(DNNL_ARG_BIAS);
    if (!src || !wei || !dst || (pd->bias.ndims && !bias)) return dnnl_invalid_arguments;
    if (!runtime_md_matches(pd->src, src->md) || !runtime_md_matches(pd->wei, wei->md) || !runtime_md_matches(pd->dst, dst->md)
            || (pd->bias.ndims && !runtime_md_matches(pd->bias, bias->md)))
        return dnnl_invalid_arguments;
    auto now = std::make_shared<dnnl_primitive_desc>();
    now->kind = dnnl_matmul;
    now->engine = pd->engine;
    now->attr = pd->attr;
    now->attr.scratchpad_mode = dnnl_scratchpad_mode_library;
    now->user_src = src->md;
    now->user_wei = wei->md;
    now->user_dst = dst->md;
    if (pd->bias.ndims) now->user_bias = bias->md;
    dnnl_status_t st = matmul_validate(now->user_src, now->user_wei, pd->bias.ndims ? &now->user_bias : nullptr, now->user_dst, now->attr);
    if (st != dnnl_success) return st;
    st = matmul_select_impl(now.get(), 0);
    if (st != dnnl_success) return st;
    dnnl_primitive tmp;
    tmp.pd = now;
    const size_t sb = now->scratchpad.ndims ? (size_t)now->scratchpad.dims[0] : 0;
    cudaStream_t cs = (cudaStream_t)stream->cuda_stream;
    if (sb) { // stream-ordered: no synchronisation, released after the kernels queued below
        if (device_alloc_async(&tmp.lib_scratch, sb, cs) != cudaSuccess) {
            (void)cudaGetLastError();
            tmp.lib_scratch = nullptr;
            tmp.pd.reset();
            return dnnl_out_of_memory;
        }
        if (cudaMemsetAsync(tmp.lib_scratch, 0, sb, cs) != cudaSuccess) st = dnnl_runtime_error;
        tmp.lib_scratch_bytes = sb;
    }
    if (st == dnnl_success) st = matmul_execute(&tmp, stream, args);
    if (tmp.lib_scratch) cudaFreeAsync(tmp.lib_scratch, cs);
    tmp.lib_scratch = nullptr;
    tmp.pd.reset();
    return st;
}

dnnl_status_t matmul_select_impl(dnnl_primitive_desc *pd, int first) {
    if (pd->runtime) return dnnl_last_impl_reached; // nothing to iterate over before the sizes are known
    // layouts of other engines (blocked tags such as AB16b16a arrive as opaque descriptors that only
    // record the tag was foreign): no implementation here reads them
    for (const dnnl_memory_desc *md : {&pd->user_src, &pd->user_wei, &pd->user_bias, &pd->user_dst})
        if (md->format_kind == dnnl_format_kind_opaque && md->packed_layout == B200_LAYOUT_FOREIGN)
            return first == 0 ? dnnl_unimplemented : dnnl_last_impl_reached;
    if (pd->user_src.format_kind == dnnl_format_kind_opaque || pd->user_dst.format_kind == dnnl_format_kind_opaque
            || pd->user_bias.format_kind == dnnl_format_kind_opaque)
        return first == 0 ? dnnl_unimplemented : dnnl_last_impl_reached;
    if (pd->user_dst.ndims > 2) return select_batched(pd, first);
    for (int id = first; id <= IMPL_GENERIC; ++id) {
        bool ok = false;
        if (impl_disabled(id)) continue;
        switch (id) {
            case IMPL_TC8: ok = accept_tc8(pd); break;
            case IMPL_WC: ok = accept_wc(pd); break;
            case IMPL_GENERIC: ok = accept_generic(pd); break;
        }
        if (!ok) continue;
        pd->impl = id;
        pd->bias = pd->user_bias;
        if (pd->bias.ndims && pd->bias.is_any()) make_plain(pd->bias);
        pd->scratchpad = dnnl_memory_desc();
        const size_t sb = scratch_bytes_for(pd);
        if (sb) {
            pd->scratchpad.ndims = 1;
            pd->scratchpad.dims[0] = (int64_t)sb;
            pd->scratchpad.strides[0] = 1;
            pd->scratchpad.data_type = dnnl_u8;
            pd->scratchpad.format_kind = dnnl_blocked;
        }
        return dnnl_success;
    }
    return first == 0 ? dnnl_unimplemented : dnnl_last_impl_reached;
}

// ---- lowering + execution ---------------------------------------------------------

static inline const void *base_ptr(const dnnl_memory *m) {
    if (!m || !m->handle) return nullptr;
    return (const char *)m->handle + m->md.offset0 * dt_nbits(m->md.data_type) / 8;
}

static void lower_quant(b200_quant_t &out, const quant_entry_t &q, const dnnl_memory *mem, int64_t d0, int64_t d1) {
    out = b200_quant_t();
    out.g0 = out.g1 = 1;
    if (!q.set || !mem) return;
    out.ptr = base_ptr(mem);
    out.dt = mem->md.data_type;
    const int64_t g0 = (q.mask & 1) ? (q.group_ndims ? q.groups[0] : 1) : 1;
    const int64_t g1 = (q.mask & 2) ? (q.group_ndims ? q.groups[1] : 1) : 1;
    const int64_t n1 = (q.mask & 2) ? d1 / g1 : 1;
    out.s0 = (q.mask & 1) ? n1 : 0;
    out.s1 = (q.mask & 2) ? 1 : 0;
    out.g0 = g0;
    out.g1 = g1;
    (void)d0;
}

static void bcast_strides(const dnnl_memory_desc &md, int64_t &sm, int64_t &sn) {
    sm = md.dims[0] > 1 ? md.strides[0] : 0;
    sn = md.dims[1] > 1 ? md.strides[1] : 0;
}

dnnl_status_t matmul_execute(const dnnl_primitive *prim, dnnl_stream *stream, const std::map<int, dnnl_memory *> &args) {
    const dnnl_primitive_desc *pd = prim->pd.get();
    auto get = [&](int a) -> dnnl_memory * {
        auto it = args.find(a);
        return it == args.end() ? nullptr : it->second;
    };
    if (pd->runtime) return runtime_execute(prim, stream, args);
    if (pd->inner) return batched_execute(prim, stream, args);
    dnnl_memory *src = get(DNNL_ARG_SRC), *wei = get(DNNL_ARG_WEIGHTS), *dst = get(DNNL_ARG_DST), *bias = get(DNNL_ARG_BIAS);
    if (!src || !wei || !dst) return dnnl_invalid_arguments;
    if (pd->bias.ndims && !bias) return dnnl_invalid_arguments;
    if (pd->src.has_zero_dim() || pd->wei.has_zero_dim() || pd->dst.has_zero_dim()) return dnnl_success;
    if (!src->handle || !wei->handle || !dst->handle) return dnnl_invalid_arguments;

    b200_matmul_params_t p;
    std::memset(&p, 0, sizeof(p));
    p.M = pd->M();
    p.N = pd->N();
    p.K = pd->K();
    p.src = base_ptr(src);
    p.src_dt = pd->src.data_type;
    p.src_sm = pd->src.strides[0];
    p.src_sk = pd->src.strides[1];
    p.wei = base_ptr(wei);
    p.wei_dt = pd->wei.data_type;
    if (pd->wei.format_kind == dnnl_format_kind_opaque) {
        p.wei_layout = pd->wei.packed_layout;
    } else {
        p.wei_layout = B200_WEI_PLAIN;
        p.wei_sk = pd->wei.strides[0];
        p.wei_sn = pd->wei.strides[1];
    }
    if (bias && pd->bias.ndims) {
        p.bias = base_ptr(bias);
        p.bias_dt = pd->bias.data_type;
        bcast_strides(pd->bias, p.bias_sm, p.bias_sn);
    }
    p.dst = const_cast<void *>(base_ptr(dst));
    p.dst_dt = pd->dst.data_type;
    p.dst_sm = pd->dst.strides[0];
    p.dst_sn = pd->dst.strides[1];
    // mirrors of dst on other GPUs (extension arguments): same descriptor, peer-mapped handles
    for (int i = 0; i < B200_MAX_DST_PEERS; ++i) {
        dnnl_memory *peer = get(DNNL_ARG_B200_DST_PEER(i));
        if (!peer) break;
        if (!peer->handle || !peer->md.equal(dst->md)) return dnnl_invalid_arguments;
        p.dst_peer[p.n_dst_peers++] = const_cast<void *>(base_ptr(peer));
    }

    const dnnl_primitive_attr &a = pd->attr;
    struct { const quant_entry_t *q; int arg; b200_quant_t *out; int64_t d0, d1; } qs[6] = {
            {&a.scale(DNNL_ARG_SRC), DNNL_ARG_ATTR_SCALES | DNNL_ARG_SRC, &p.src_scale, p.M, p.K},
            {&a.scale(DNNL_ARG_WEIGHTS), DNNL_ARG_ATTR_SCALES | DNNL_ARG_WEIGHTS, &p.wei_scale, p.K, p.N},
            {&a.scale(DNNL_ARG_DST), DNNL_ARG_ATTR_SCALES | DNNL_ARG_DST, &p.dst_scale, p.M, p.N},
            {&a.zp(DNNL_ARG_SRC), DNNL_ARG_ATTR_ZERO_POINTS | DNNL_ARG_SRC, &p.src_zp, p.M, p.K},
            {&a.zp(DNNL_ARG_WEIGHTS), DNNL_ARG_ATTR_ZERO_POINTS | DNNL_ARG_WEIGHTS, &p.wei_zp, p.K, p.N},
            {&a.zp(DNNL_ARG_DST), DNNL_ARG_ATTR_ZERO_POINTS | DNNL_ARG_DST, &p.dst_zp, p.M, p.N}};
    for (auto &e : qs) {
        dnnl_memory *m = get(e.arg);
        if (e.q->set && (!m || !m->handle)) return dnnl_invalid_arguments; // runtime quantisation argument missing
        lower_quant(*e.out, *e.q, m, e.d0, e.d1);
        if (e.q->set) {
            // the memory must hold at least the elements the mask implies
            const int64_t need = (e.out->s0 ? e.d0 / e.out->g0 : 1) * (e.out->s1 ? e.d1 / e.out->g1 : 1);
            if (m->md.nelems() < need) return dnnl_invalid_arguments;
        }
    }
    p.apply_to_int = a.apply_to_int;
    p.npo = (int)a.post_ops.entries.size();
    for (int i = 0; i < p.npo; ++i) {
        const post_op_t &e = a.post_ops.entries[i];
        b200_postop_t &o = p.po[i];
        o.alg = e.alg;
        o.alpha = e.alpha;
        o.beta = e.beta;
        o.scale = e.scale;
        o.zero_point = e.zero_point;
        if (e.kind == dnnl_sum) {
            o.kind = B200_PO_SUM;
            o.dt = e.dt;
        } else if (e.kind == dnnl_eltwise) {
            o.kind = B200_PO_ELTWISE;
        } else if (e.kind == dnnl_binary) {
            o.kind = B200_PO_BINARY;
            dnnl_memory *m = get(DNNL_ARG_ATTR_MULTIPLE_POST_OP(i) | DNNL_ARG_SRC_1);
            if (!m || !m->handle) return dnnl_invalid_arguments;
            o.ptr = base_ptr(m);
            o.dt = e.src1.data_type;
            dnnl_memory_desc s1 = e.src1;
            if (s1.is_any()) make_plain(s1);
            bcast_strides(s1, o.sm, o.sn);
        } else {
            o.kind = B200_PO_PRELU;
            dnnl_memory *m = get(DNNL_ARG_ATTR_MULTIPLE_POST_OP(i) | DNNL_ARG_WEIGHTS);
            if (!m || !m->handle) return dnnl_invalid_arguments;
            o.ptr = base_ptr(m);
            o.dt = dnnl_f32;
            // weights are a dense tensor over the dims selected by the mask
            const bool pm = e.mask & 1, pn = e.mask & 2;
            o.sn = pn ? 1 : 0;
            o.sm = pm ? (pn ? p.N : 1) : 0;
        }
    }
    p.status = stream->status;

    // scratchpad
    void *scratch = nullptr;
    size_t scratch_bytes = pd->scratchpad.ndims ? (size_t)pd->scratchpad.dims[0] : 0;
    if (scratch_bytes) {
        if (a.scratchpad_mode == dnnl_scratchpad_mode_user) {
            dnnl_memory *m = get(DNNL_ARG_SCRATCHPAD);
            if (!m || !m->handle) return dnnl_invalid_arguments;
            scratch = m->handle;
        } else {
            scratch = prim->lib_scratch;
        }
        if (!scratch) return dnnl_out_of_memory;
    }
    p.scratch = scratch;
    p.scratch_bytes = scratch_bytes;
    // the library-owned scratchpad is zeroed when the primitive is created and every kernel
    // leaves its accumulation area zeroed -- unless an execution went wrong since (g_scratch_epoch)
    p.scratch_zeroed = 0;
    if (scratch && a.scratchpad_mode == dnnl_scratchpad_mode_library) {
        const dnnl_primitive *owner = prim->scratch_owner ? prim->scratch_owner : prim;
        const uint64_t now = g_scratch_epoch.load();
        if (owner->scratch_epoch.exchange(now) == now) p.scratch_zeroed = 1;
        else g_scratch_reclears.fetch_add(1);
    }

    b200_stream_t cs = stream->cuda_stream;
    int rc = 0;
    switch (pd->impl) {
        case IMPL_GENERIC: rc = b200_matmul_generic_launch(&p, cs); break;
        case IMPL_WC:
            rc = pd->impl_str.find("tcgen05") != std::string::npos ? b200_matmul_wc_tc_launch(&p, cs) : b200_matmul_wc_launch(&p, cs);
            break;
        case IMPL_TC8: {
            if (p.wei_layout == B200_WEI_KMAJOR) {
                if (p.src_zp.ptr)
                    p.wei_colsum = (const int32_t *)((const char *)p.wei + b200_packed_colsum_offset(p.K, p.N, p.wei_dt));
            } else if (tc8_weights_class(pd->wei) == TC8_WEI_INPLACE_KMAJOR) {
                // plain K-major weights: usable in place; column sums into the scratchpad
                if (p.src_zp.ptr) {
                    rc = b200_colsum_launch(p.wei, p.wei_dt, p.K, p.N, p.wei_sk, p.wei_sn, (int32_t *)scratch, cs);
                    p.wei_colsum = (const int32_t *)scratch;
                }
            } else {
                // plain N-major weights: pack into the scratchpad first
                b200_reorder_params_t r;
                std::memset(&r, 0, sizeof(r));
                r.K = p.K;
                r.N = p.N;
                r.src = p.wei;
                r.src_dt = p.wei_dt;
                r.src_layout = B200_WEI_PLAIN;
                r.src_sk = p.wei_sk;
                r.src_sn = p.wei_sn;
                r.dst = scratch;
                r.dst_dt = p.wei_dt;
                r.dst_layout = B200_WEI_KMAJOR;
                rc = b200_reorder_launch(&r, cs);
                p.wei = scratch;
                p.wei_layout = B200_WEI_KMAJOR;
                p.wei_colsum = (const int32_t *)((const char *)scratch + b200_packed_colsum_offset(p.K, p.N, p.wei_dt));
            }
            if (rc == 0 && p.wei_zp.ptr) {
                // sum over k of src[m][k]: the column sums of src seen as its own transpose
                int32_t *rowsum = (int32_t *)((char *)scratch + tc8_weights_scratch_bytes(pd));
                rc = b200_colsum_launch(p.src, p.src_dt, p.K, p.M, p.src_sk, p.src_sm, rowsum, cs);
                p.src_rowsum = rowsum;
            }
            if (rc == 0) rc = b200_matmul_tc8_launch(&p, cs);
        } break;
        default: return dnnl_runtime_error;
    }
    if (rc == 0) return dnnl_success;
    if (rc == B200_ERR_BAD_ARG) return dnnl_invalid_arguments;
    if (rc == B200_ERR_UNSUPPORTED) return dnnl_unimplemented;
    return dnnl_runtime_error;
}

} // namespace b200

using namespace b200;

dnnl_status_t dnnl_matmul_primitive_desc_create(dnnl_primitive_desc_t *primitive_desc, dnnl_engine_t engine,
        const_dnnl_memory_desc_t src_desc, const_dnnl_memory_desc_t weights_desc, const_dnnl_memory_desc_t bias_desc,
        const_dnnl_memory_desc_t dst_desc, const_dnnl_primitive_attr_t attr) {
    if (!primitive_desc || !engine || !src_desc || !weights_desc || !dst_desc) return dnnl_invalid_arguments;
    const double t0 = now_ms();
    static const dnnl_primitive_attr default_attr;
    const dnnl_primitive_attr &a = attr ? *attr : default_attr;
    dnnl_status_t st = matmul_validate(*src_desc, *weights_desc, bias_desc, *dst_desc, a);
    if (st != dnnl_success) return st;
    if (engine->host) return dnnl_unimplemented; // the host engine holds memory and reorders; it computes nothing
    const bool runtime = src_desc->has_runtime_dims() || weights_desc->has_runtime_dims() || dst_desc->has_runtime_dims()
            || (bias_desc && bias_desc->has_runtime_dims());
    auto pd = std::unique_ptr<dnnl_primitive_desc>(new dnnl_primitive_desc());
    pd->kind = dnnl_matmul;
    pd->engine = engine;
    pd->attr = a; // copied: later changes to the caller's attr have no effect
    // a binary post-op operand left to the implementation (format_tag::any) is dense row-major here;
    // the resolved descriptor is what dnnl_query_exec_arg_md returns for it
    for (auto &e : pd->attr.post_ops.entries)
        if (e.kind == dnnl_binary && e.src1.is_any() && !e.src1.has_runtime_dims()) make_plain(e.src1);
    pd->user_src = *src_desc;
    pd->user_wei = *weights_desc;
    if (bias_desc) pd->user_bias = *bias_desc;
    pd->user_dst = *dst_desc;
    if (runtime) {
        // Sizes known only at execution (DNNL_RUNTIME_DIM_VAL, src/common/matmul.cpp:374-401):
        // nothing can be dispatched yet.  Layouts must be given (no format_tag::any); the
        // implementation is selected per execution from the memory arguments' descriptors.
        if (src_desc->is_any() || weights_desc->is_any() || dst_desc->is_any()) return dnnl_unimplemented;
        // a bias of known size may be left to the implementation: dense row-major
        if (bias_desc && bias_desc->is_any() && bias_desc->has_runtime_dims()) return dnnl_unimplemented;
        if (a.scratchpad_mode == dnnl_scratchpad_mode_user) return dnnl_unimplemented; // its size is not known here
        pd->src = pd->user_src;
        pd->wei = pd->user_wei;
        pd->dst = pd->user_dst;
        pd->bias = pd->user_bias;
        if (pd->bias.is_any()) make_plain(pd->bias);
        pd->impl = IMPL_GENERIC;
        pd->impl_str = "cuda:runtime_dims";
        pd->runtime = true;
        st = dnnl_success;
    } else {
        st = matmul_select_impl(pd.get(), 0);
    }
    if (st != dnnl_success) return st;
    engine->refs.fetch_add(1);
    verbose_create(pd.get(), now_ms() - t0, false);
    *primitive_desc = pd.release();
    return dnnl_success;
}

// ---- inner product (forward) as a view of the matmul -----------------------------------------
// dst(N, OC) = src(N, IC) x weights(OC, IC)^T + bias(OC)  (src/common/inner_product.cpp:37-120).
// The weights' (OC, IC) descriptor read with its two strides exchanged is the matmul's (K, N)
// weights; row-major (OC, IC) -- what format_tag::any resolves to here -- is K-contiguous per
// output channel, the operand layout of the tensor-core kernels, so nothing is repacked.

dnnl_status_t dnnl_inner_product_forward_primitive_desc_create(dnnl_primitive_desc_t *primitive_desc, dnnl_engine_t engine,
        dnnl_prop_kind_t prop_kind, const_dnnl_memory_desc_t src_desc, const_dnnl_memory_desc_t weights_desc,
        const_dnnl_memory_desc_t bias_desc, const_dnnl_memory_desc_t dst_desc, const_dnnl_primitive_attr_t attr) {
    if (!primitive_desc || !engine || !src_desc || !weights_desc || !dst_desc) return dnnl_invalid_arguments;
    if (prop_kind != dnnl_forward_training && prop_kind != dnnl_forward_inference) return dnnl_invalid_arguments;
    if (engine->host) return dnnl_unimplemented;
    const dnnl_memory_desc &s = *src_desc, &w = *weights_desc, &d = *dst_desc;
    if (s.ndims != w.ndims || d.ndims != 2) return dnnl_invalid_arguments;
    if (s.ndims != 2) return dnnl_unimplemented; // spatial dims: not on this path
    if (s.has_runtime_dims() || w.has_runtime_dims() || d.has_runtime_dims()) return dnnl_unimplemented;
    if (s.dims[0] != d.dims[0] || s.dims[1] != w.dims[1] || w.dims[0] != d.dims[1]) return dnnl_invalid_arguments;
    const bool with_bias = bias_desc && bias_desc->ndims != 0;
    if (with_bias && (bias_desc->ndims != 1 || bias_desc->dims[0] != d.dims[1])) return dnnl_invalid_arguments;
    if (w.format_kind == dnnl_format_kind_opaque) return dnnl_unimplemented;
    static const dnnl_primitive_attr default_attr;
    const dnnl_primitive_attr &a = attr ? *attr : default_attr;

    auto in = std::make_shared<dnnl_primitive_desc>();
    in->kind = dnnl_matmul;
    in->engine = engine;
    in->attr = a;
    // weights masks and groups follow the exchange of the weights' two dims
    for (auto *m : {&in->attr.scales, &in->attr.zero_points}) {
        auto it = m->find(DNNL_ARG_WEIGHTS);
        if (it == m->end() || !it->second.set) continue;
        b200::quant_entry_t &q = it->second;
        q.mask = ((q.mask & 1) << 1) | ((q.mask & 2) >> 1);
        std::swap(q.groups[0], q.groups[1]);
    }
    dnnl_memory_desc wplain = w;
    if (wplain.is_any()) make_plain(wplain);
    in->user_src = s;
    in->user_wei = wplain;
    std::swap(in->user_wei.dims[0], in->user_wei.dims[1]);
    std::swap(in->user_wei.strides[0], in->user_wei.strides[1]);
    in->user_dst = d;
    if (with_bias) {
        dnnl_memory_desc b;
        b.ndims = 2;
        b.dims[0] = 1;
        b.dims[1] = bias_desc->dims[0];
        b.data_type = bias_desc->data_type;
        b.format_kind = dnnl_blocked;
        b.strides[1] = bias_desc->is_any() ? 1 : bias_desc->strides[0];
        b.strides[0] = b.dims[1] * b.strides[1];
        in->user_bias = b;
    }
    dnnl_status_t st = b200::matmul_validate(in->user_src, in->user_wei, with_bias ? &in->user_bias : nullptr, in->user_dst, in->attr);
    if (st != dnnl_success) return st;
    st = b200::matmul_select_impl(in.get(), 0);
    if (st != dnnl_success) return st;

    auto pd = std::unique_ptr<dnnl_primitive_desc>(new dnnl_primitive_desc());
    pd->kind = dnnl_inner_product;
    pd->engine = engine;
    pd->attr = a;
    pd->user_src = s;
    pd->user_wei = w;
    pd->user_dst = d;
    pd->src = in->src;
    pd->wei = wplain;
    pd->dst = in->dst;
    if (with_bias) {
        pd->user_bias = *bias_desc;
        pd->bias = *bias_desc;
        if (pd->bias.is_any()) make_plain(pd->bias);
    }
    pd->impl = in->impl;
    pd->impl_str = in->impl_str;
    pd->scratchpad = in->scratchpad;
    pd->inner = in;
    pd->ip = true;
    engine->refs.fetch_add(1);
    *primitive_desc = pd.release();
    return dnnl_success;
}

namespace b200 {

dnnl_status_t inner_product_execute(const dnnl_primitive *prim, dnnl_stream *stream, const std::map<int, dnnl_memory *> &args) {
    const dnnl_primitive_desc *pd = prim->pd.get();
    const dnnl_primitive_desc *in = pd->inner.get();
    std::map<int, dnnl_memory *> a2 = args;
    dnnl_memory wei, bias;
    auto wi = args.find(DNNL_ARG_WEIGHTS);
    if (wi == args.end()) return dnnl_invalid_arguments;
    wei = *wi->second;
    wei.md = in->wei;          // the same bytes, dims and strides exchanged
    wei.md.offset0 = wi->second->md.offset0;
    wei.owned = false;
    a2[DNNL_ARG_WEIGHTS] = &wei;
    if (pd->bias.ndims) {
        auto bi = args.find(DNNL_ARG_BIAS);
        if (bi == args.end()) return dnnl_invalid_arguments;
        bias = *bi->second;
        bias.md = in->bias;
        bias.md.offset0 = bi->second->md.offset0;
        bias.owned = false;
        a2[DNNL_ARG_BIAS] = &bias;
    }
    dnnl_primitive tmp;
    tmp.pd = pd->inner;
    tmp.lib_scratch = prim->lib_scratch; // borrowed
    tmp.lib_scratch_bytes = prim->lib_scratch_bytes;
    tmp.scratch_owner = prim->scratch_owner ? prim->scratch_owner : prim;
    const dnnl_status_t st = matmul_execute(&tmp, stream, a2);
    tmp.lib_scratch = nullptr;
    tmp.pd.reset();
    return st;
}

} // namespace b200
