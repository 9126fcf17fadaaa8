// Primitive descriptor queries / iteration, the reorder primitive descriptor,
// primitive creation (through a small LRU cache) and execution.  Replaces the
// reference's src/common/primitive_desc_iface.cpp, primitive_iface.cpp:147-217,
// primitive_exec_types.cpp:27-92 (argument classification), reorder.cpp:63-220
// and primitive_cache.cpp for the two primitive kinds of this path.
#include <cuda_runtime.h>

#include <list>

#include <iterator>

#include "internal.hpp"

using namespace b200;

dnnl_primitive::~dnnl_primitive() {
    if (lib_scratch && pd && pd->engine && pd->engine->usable()) {
        cudaSetDevice(pd->engine->device);
        cudaFree(lib_scratch);
    }
}

// ---- reorder primitive descriptor -----------------------------------------------

// Attributes of a quantising reorder: what src/common/reorder.cpp:96-146 and the generic
// implementation's own check (src/cpu/reorder/simple_reorder.hpp:2498-2547) admit, for the
// plain 1-D / 2-D tensors this engine reorders with scales.
static dnnl_status_t reorder_quant_validate(const dnnl_memory_desc &s, const dnnl_memory_desc &d,
        const dnnl_primitive_attr &attr) {
    if (!s.is_plain() || !d.is_plain()) return dnnl_unimplemented;
    if (s.ndims < 1) return dnnl_unimplemented;
    if (s.ndims > 2) {
        // more dims: dense row-major tensors whose scales / zero-points are per tensor or per element of
        // the last dim fold into (prod(leading dims), last dim) -- activations of any rank quantised per
        // tensor or per channel; anything else is not taken
        if (!s.is_dense_row_major() || !d.is_dense_row_major()) return dnnl_unimplemented;
        if (dt_nbits(s.data_type) == 4 || dt_nbits(d.data_type) == 4) return dnnl_unimplemented;
        const int last = 1 << (s.ndims - 1);
        for (auto *m : {&attr.scales, &attr.zero_points})
            for (const auto &kv : *m) {
                if (!kv.second.set) continue;
                if (kv.first != DNNL_ARG_SRC && kv.first != DNNL_ARG_DST) return dnnl_unimplemented;
                if (kv.second.mask & ~((1 << s.ndims) - 1)) return dnnl_invalid_arguments;
                if ((kv.second.mask != 0 && kv.second.mask != last) || kv.second.group_ndims) return dnnl_unimplemented;
            }
        auto is_int_nd = [](int dt) { return dt == dnnl_s32 || dt == dnnl_s8 || dt == dnnl_u8; };
        if (attr.zp(DNNL_ARG_SRC).set && !is_int_nd(s.data_type)) return dnnl_invalid_arguments;
        if (attr.zp(DNNL_ARG_DST).set && !is_int_nd(d.data_type)) return dnnl_invalid_arguments;
        if (attr.zp(DNNL_ARG_DST).set && (attr.zp(DNNL_ARG_DST).mask != 0 || attr.zp(DNNL_ARG_DST).dt != dnnl_s32)) return dnnl_unimplemented;
        if (attr.scale(DNNL_ARG_DST).set && attr.scale(DNNL_ARG_DST).dt != dnnl_f32) return dnnl_unimplemented;
        const auto &po_nd = attr.post_ops.entries;
        if (po_nd.size() > 1 || (po_nd.size() == 1 && !(po_nd[0].kind == dnnl_sum && po_nd[0].zero_point == 0))) return dnnl_unimplemented;
        return dnnl_success;
    }
    const bool s4 = dt_nbits(s.data_type) == 4, d4 = dt_nbits(d.data_type) == 4;
    if (s4 || d4) {
        // decompressing a 4-bit tensor into f32 / bf16 / f16 with source-side scales and zero-points;
        // nothing else (src/cpu/reorder/cpu_reorder_regular_s4.cpp, _u4.cpp list what the reference has)
        if (!s4 || d4) return dnnl_unimplemented;
        if (!(d.data_type == dnnl_f32 || d.data_type == dnnl_bf16 || d.data_type == dnnl_f16)) return dnnl_unimplemented;
        if (attr.scale(DNNL_ARG_DST).set || attr.zp(DNNL_ARG_DST).set || !attr.post_ops.entries.empty()) return dnnl_unimplemented;
        // a 4-bit source takes no scale common to the whole tensor (src/common/reorder.cpp:117-120)
        if (attr.scale(DNNL_ARG_SRC).set && attr.scale(DNNL_ARG_SRC).mask == 0) return dnnl_invalid_arguments;
    }
    const int full = (1 << s.ndims) - 1;
    for (const auto &kv : attr.scales) {
        if (!kv.second.set) continue;
        if (kv.first != DNNL_ARG_SRC && kv.first != DNNL_ARG_DST) return dnnl_unimplemented;
        if (kv.second.mask & ~full) return dnnl_invalid_arguments;
    }
    for (const auto &kv : attr.zero_points) {
        if (!kv.second.set) continue;
        if (kv.first != DNNL_ARG_SRC && kv.first != DNNL_ARG_DST) return dnnl_unimplemented;
        if (kv.second.mask & ~full) return dnnl_invalid_arguments;
    }
    // zero-points go with integer tensors only
    auto is_int = [](int dt) { return dt == dnnl_s32 || dt == dnnl_s8 || dt == dnnl_u8 || dt == dnnl_s4 || dt == dnnl_u4; };
    if (attr.zp(DNNL_ARG_SRC).set && !is_int(s.data_type)) return dnnl_invalid_arguments;
    if (attr.zp(DNNL_ARG_DST).set && !is_int(d.data_type)) return dnnl_invalid_arguments;
    if (attr.zp(DNNL_ARG_DST).set && (attr.zp(DNNL_ARG_DST).mask != 0 || attr.zp(DNNL_ARG_DST).dt != dnnl_s32))
        return dnnl_unimplemented;
    const b200::quant_entry_t &ss = attr.scale(DNNL_ARG_SRC), &ds = attr.scale(DNNL_ARG_DST);
    if (ds.set && (ds.group_ndims != 0 || ds.dt != dnnl_f32)) return dnnl_unimplemented;
    if (ss.set && ds.set && ss.mask > 0 && ds.mask > 0 && ss.mask != ds.mask) return dnnl_invalid_arguments;
    for (const b200::quant_entry_t *q : {&ss, &attr.zp(DNNL_ARG_SRC)}) {
        if (!q->set || q->group_ndims == 0) continue;
        if (s.ndims != 2 || q->group_ndims != 2 || q->mask != 3) return dnnl_invalid_arguments;
        for (int i = 0; i < 2; ++i)
            if (q->groups[i] < 1 || s.dims[i] % q->groups[i] != 0) return dnnl_invalid_arguments;
    }
    const auto &po = attr.post_ops.entries;
    if (po.size() > 1) return dnnl_unimplemented;
    if (po.size() == 1 && !(po[0].kind == dnnl_sum && po[0].zero_point == 0)) return dnnl_unimplemented;
    return dnnl_success;
}

dnnl_status_t dnnl_reorder_primitive_desc_create(dnnl_primitive_desc_t *reorder_primitive_desc,
        const_dnnl_memory_desc_t src_desc, dnnl_engine_t src_engine, const_dnnl_memory_desc_t dst_desc,
        dnnl_engine_t dst_engine, const_dnnl_primitive_attr_t attr) {
    if (!reorder_primitive_desc || !src_desc || !dst_desc || !src_engine || !dst_engine) return dnnl_invalid_arguments;
    const bool with_host = src_engine->host || dst_engine->host;
    if (!with_host && src_engine != dst_engine && src_engine->device != dst_engine->device) return dnnl_unimplemented;
    const dnnl_memory_desc &s = *src_desc, &d = *dst_desc;
    if (s.is_any() || d.is_any()) return dnnl_invalid_arguments;
    if (s.ndims != d.ndims) return dnnl_invalid_arguments;
    for (int i = 0; i < s.ndims; ++i)
        if (s.dims[i] != d.dims[i]) return dnnl_invalid_arguments;
    if (s.has_runtime_dims()) return dnnl_unimplemented;
    if (with_host) return host_reorder_pd_create(reorder_primitive_desc, s, src_engine, d, dst_engine, attr);
    bool quantising = attr && (!attr->scales.empty() || !attr->zero_points.empty() || !attr->post_ops.entries.empty());
    // a 4-bit tensor and a float one: the conversion runs on the quantising reorder's kernel, attributes or not
    // (4-bit -> f32 / bf16 / f16, and f32 -> 4-bit without attributes)
    const bool conv4 = s.is_plain() && d.is_plain() && s.ndims <= 2 && dt_nbits(s.data_type) != dt_nbits(d.data_type)
            && (dt_nbits(s.data_type) == 4 || dt_nbits(d.data_type) == 4);
    if (conv4) {
        static const dnnl_primitive_attr no_attr;
        if (dt_nbits(d.data_type) == 4) {
            if (quantising || s.data_type != dnnl_f32) return dnnl_unimplemented;
        } else {
            const dnnl_status_t st = reorder_quant_validate(s, d, attr ? *attr : no_attr);
            if (st != dnnl_success) return st;
        }
        // dense rows that start on a byte
        const dnnl_memory_desc &q = dt_nbits(s.data_type) == 4 ? s : d;
        if (q.strides[q.ndims - 1] != 1 || (q.dims[q.ndims - 1] & 1) || (q.offset0 & 1) || (q.ndims == 2 && q.dims[0] > 1 && (q.strides[0] & 1)))
            return dnnl_unimplemented;
        quantising = true;
    } else if (quantising) {
        const dnnl_status_t st = reorder_quant_validate(s, d, *attr);
        if (st != dnnl_success) return st;
    }
    if (!s.is_plain()) return dnnl_unimplemented; // unpacking is not needed by the matmul path
    if (d.format_kind == dnnl_format_kind_opaque) {
        // packed weights: a (K, N) matrix, or batch dims in front of one (every slice packed on its own)
        if (s.ndims < 2 || s.data_type != d.data_type) return dnnl_unimplemented;
        const int64_t K = s.dims[s.ndims - 2], N = s.dims[s.ndims - 1];
        const bool slice_dense = s.strides[s.ndims - 1] == 1 && s.strides[s.ndims - 2] == N;
        if (d.packed_layout == B200_WEI_KMAJOR && !(dt_is_int8(s.data_type) || dt_is_fp8(s.data_type)))
            return dnnl_unimplemented;
        if (d.packed_layout == B200_WEI_WC4_TILED && !(dt_is_int4(s.data_type) && slice_dense && K % 64 == 0 && N % 16 == 0))
            return dnnl_unimplemented;
        if (d.packed_layout == B200_WEI_WC4_TC && !(dt_is_int4(s.data_type) && slice_dense && K % 64 == 0 && N % 2 == 0))
            return dnnl_unimplemented;
        if (d.packed_layout == B200_WEI_WC8_TC && !(dt_is_int8(s.data_type) && K % 64 == 0)) return dnnl_unimplemented;
        // a 4-bit slice must start on a byte
        if (dt_is_int4(s.data_type))
            for (int i = 0; i < s.ndims - 2; ++i)
                if (s.dims[i] > 1 && (s.strides[i] & 1)) return dnnl_unimplemented;
    } else {
        if (s.ndims > 6) return dnnl_unimplemented;
        const int sb = dt_nbits(s.data_type), db = dt_nbits(d.data_type);
        // 4-bit tensors: dense copies of the same type (conversions to and from float types went above)
        if (!conv4 && (sb == 4 || db == 4) && !(s.data_type == d.data_type && s.equal(d) && s.is_dense_row_major()))
            return dnnl_unimplemented;
    }
    auto pd = std::unique_ptr<dnnl_primitive_desc>(new dnnl_primitive_desc());
    pd->kind = dnnl_reorder;
    pd->engine = dst_engine;
    if (attr) pd->attr = *attr;
    pd->user_src = pd->src = s;
    pd->user_dst = pd->dst = d;
    pd->impl = IMPL_REORDER;
    pd->impl_str = d.format_kind == dnnl_format_kind_opaque ? "cuda:pack_weights"
                                                            : (quantising ? "cuda:reorder_quant" : "cuda:reorder");
    dst_engine->refs.fetch_add(1);
    *reorder_primitive_desc = pd.release();
    return dnnl_success;
}

namespace b200 {

static dnnl_status_t reorder_quant_execute(const dnnl_primitive_desc *pd, dnnl_stream *stream, const dnnl_memory *from,
        const dnnl_memory *to, const std::map<int, dnnl_memory *> &args) {
    const dnnl_memory_desc &s = pd->src, &d = pd->dst;
    b200_reorder_quant_params_t r;
    std::memset(&r, 0, sizeof(r));
    r.src = (const char *)from->handle + s.offset0 * dt_nbits(s.data_type) / 8;
    r.dst = (char *)to->handle + d.offset0 * dt_nbits(d.data_type) / 8;
    r.src_dt = s.data_type;
    r.dst_dt = d.data_type;
    // a 1-D tensor is one row; its only dim then is mask bit 1 below.  More than two dims (dense
    // row-major, validated at creation): the leading dims fold into the rows, and the only mask
    // bit that can be set, the last dim's, becomes bit 1 as well.
    const int sh = s.ndims == 1 ? 1 : s.ndims > 2 ? s.ndims - 2 : 0;
    r.cols = s.dims[s.ndims - 1];
    if (s.ndims > 2) {
        r.rows = 1;
        for (int i = 0; i < s.ndims - 1; ++i) r.rows *= s.dims[i];
        r.src_s0 = r.dst_s0 = r.cols;
    } else {
        r.rows = sh ? 1 : s.dims[0];
        r.src_s0 = sh ? 0 : s.strides[0];
        r.dst_s0 = sh ? 0 : d.strides[0];
    }
    r.src_s1 = s.strides[s.ndims - 1];
    r.dst_s1 = d.strides[s.ndims - 1];
    const dnnl_primitive_attr &a = pd->attr;
    struct { const quant_entry_t *q; int arg; b200_quant_t *out; } qs[4] = {
            {&a.scale(DNNL_ARG_SRC), DNNL_ARG_ATTR_SCALES | DNNL_ARG_SRC, &r.src_scale},
            {&a.scale(DNNL_ARG_DST), DNNL_ARG_ATTR_SCALES | DNNL_ARG_DST, &r.dst_scale},
            {&a.zp(DNNL_ARG_SRC), DNNL_ARG_ATTR_ZERO_POINTS | DNNL_ARG_SRC, &r.src_zp},
            {&a.zp(DNNL_ARG_DST), DNNL_ARG_ATTR_ZERO_POINTS | DNNL_ARG_DST, &r.dst_zp}};
    for (auto &e : qs) {
        b200_quant_t &o = *e.out;
        o.g0 = o.g1 = 1;
        if (!e.q->set) continue;
        auto it = args.find(e.arg);
        if (it == args.end() || !it->second->handle) return dnnl_invalid_arguments; // runtime argument missing
        const dnnl_memory *m = it->second;
        const int mask = s.ndims > 2 ? (e.q->mask >> sh) : (e.q->mask << sh);
        o.ptr = (const char *)m->handle + m->md.offset0 * dt_nbits(m->md.data_type) / 8;
        o.dt = m->md.data_type;
        if (o.dt != e.q->dt) return dnnl_invalid_arguments;
        o.g0 = (mask & 1) && e.q->group_ndims ? e.q->groups[0] : 1;
        o.g1 = (mask & 2) && e.q->group_ndims ? e.q->groups[1] : 1;
        const int64_t n1 = (mask & 2) ? r.cols / o.g1 : 1, n0 = (mask & 1) ? r.rows / o.g0 : 1;
        o.s0 = (mask & 1) ? n1 : 0;
        o.s1 = (mask & 2) ? 1 : 0;
        if (m->md.nelems() < n0 * n1) return dnnl_invalid_arguments;
    }
    if (!a.post_ops.entries.empty()) r.beta = a.post_ops.entries[0].scale;
    const int rc = b200_reorder_quant_launch(&r, stream->cuda_stream);
    if (rc == 0) return dnnl_success;
    if (rc == B200_ERR_UNSUPPORTED) return dnnl_unimplemented;
    if (rc == B200_ERR_BAD_ARG) return dnnl_invalid_arguments;
    return dnnl_runtime_error;
}

dnnl_status_t reorder_execute(const dnnl_primitive *prim, dnnl_stream *stream, const std::map<int, dnnl_memory *> &args) {
    const dnnl_primitive_desc *pd = prim->pd.get();
    auto f = args.find(DNNL_ARG_FROM), t = args.find(DNNL_ARG_TO);
    if (f == args.end() || t == args.end()) return dnnl_invalid_arguments;
    const dnnl_memory *from = f->second, *to = t->second;
    if (pd->src.has_zero_dim()) return dnnl_success;
    if (!from->handle || !to->handle) return dnnl_invalid_arguments;
    if (pd->impl_str.compare(0, 5, "host:") == 0) return host_reorder_execute(prim, stream, from, to);
    const dnnl_memory_desc &s = pd->src, &d = pd->dst;
    if (pd->impl_str == "cuda:reorder_quant") return reorder_quant_execute(pd, stream, from, to, args);
    b200_reorder_params_t r;
    std::memset(&r, 0, sizeof(r));
    r.src = (const char *)from->handle + s.offset0 * dt_nbits(s.data_type) / 8;
    r.dst = (char *)to->handle + d.offset0 * dt_nbits(d.data_type) / 8;
    r.src_dt = s.data_type;
    r.dst_dt = d.data_type;
    int rc;
    if (d.format_kind == dnnl_format_kind_opaque && s.ndims > 2) {
        // batched weights into the packed layout: one pack per batch index, slices at packed_slice_stride
        const int nd = s.ndims;
        int64_t outer = 1;
        for (int i = 0; i < nd - 2; ++i) outer *= s.dims[i];
        const size_t stride = d.packed_slice_stride();
        rc = 0;
        for (int64_t o = 0; o < outer && rc == 0; ++o) {
            int64_t rem = o, so = 0;
            for (int i = nd - 3; i >= 0; --i) {
                so += (rem % s.dims[i]) * s.strides[i];
                rem /= s.dims[i];
            }
            b200_reorder_params_t q = r;
            q.src = (const char *)r.src + so * dt_nbits(s.data_type) / 8;
            q.dst = (char *)r.dst + (size_t)o * stride;
            q.K = s.dims[nd - 2];
            q.N = s.dims[nd - 1];
            q.src_sk = s.strides[nd - 2];
            q.src_sn = s.strides[nd - 1];
            q.src_layout = B200_WEI_PLAIN;
            q.dst_layout = d.packed_layout;
            rc = b200_reorder_launch(&q, stream->cuda_stream);
        }
    } else if (s.ndims == 2 || d.format_kind == dnnl_format_kind_opaque) {
        r.K = s.dims[0];
        r.N = s.dims[1];
        r.src_sk = s.strides[0];
        r.src_sn = s.strides[1];
        r.src_layout = B200_WEI_PLAIN;
        if (d.format_kind == dnnl_format_kind_opaque) {
            r.dst_layout = d.packed_layout;
        } else {
            r.dst_layout = B200_WEI_PLAIN;
            r.dst_sk = d.strides[0];
            r.dst_sn = d.strides[1];
        }
        rc = b200_reorder_launch(&r, stream->cuda_stream);
    } else {
        // N-D plain tensors: fold into batches of 2-D slices over the two innermost dims
        const int nd = s.ndims;
        if (nd == 1) {
            r.K = 1;
            r.N = s.dims[0];
            r.src_sk = 0;
            r.src_sn = s.strides[0];
            r.dst_sk = 0;
            r.dst_sn = d.strides[0];
            rc = b200_reorder_launch(&r, stream->cuda_stream);
        } else {
            int64_t outer = 1;
            for (int i = 0; i < nd - 2; ++i) outer *= s.dims[i];
            rc = 0;
            for (int64_t o = 0; o < outer && rc == 0; ++o) {
                int64_t rem = o, so = 0, dof = 0;
                for (int i = nd - 3; i >= 0; --i) {
                    const int64_t idx = rem % s.dims[i];
                    rem /= s.dims[i];
                    so += idx * s.strides[i];
                    dof += idx * d.strides[i];
                }
                b200_reorder_params_t q = r;
                q.src = (const char *)r.src + so * dt_nbits(s.data_type) / 8;
                q.dst = (char *)r.dst + dof * dt_nbits(d.data_type) / 8;
                q.K = s.dims[nd - 2];
                q.N = s.dims[nd - 1];
                q.src_sk = s.strides[nd - 2];
                q.src_sn = s.strides[nd - 1];
                q.dst_sk = d.strides[nd - 2];
                q.dst_sn = d.strides[nd - 1];
                rc = b200_reorder_launch(&q, stream->cuda_stream);
            }
        }
    }
    if (rc == 0) return dnnl_success;
    if (rc == B200_ERR_UNSUPPORTED) return dnnl_unimplemented;
    if (rc == B200_ERR_BAD_ARG) return dnnl_invalid_arguments;
    return dnnl_runtime_error;
}

} // namespace b200

// ---- primitive descriptor API --------------------------------------------------------

dnnl_status_t dnnl_primitive_desc_next_impl(dnnl_primitive_desc_t pd) {
    if (!pd) return dnnl_invalid_arguments;
    if (pd->kind != dnnl_matmul) return dnnl_last_impl_reached; // reorder, inner product: one implementation
    dnnl_primitive_desc trial = *pd;
    dnnl_status_t st = matmul_select_impl(&trial, pd->impl + 1);
    if (st != dnnl_success) return dnnl_last_impl_reached;
    trial.arg_mds.clear();
    *pd = trial;
    return dnnl_success;
}

dnnl_status_t dnnl_primitive_desc_clone(dnnl_primitive_desc_t *primitive_desc, const_dnnl_primitive_desc_t existing) {
    if (!primitive_desc || !existing) return dnnl_invalid_arguments;
    *primitive_desc = new dnnl_primitive_desc(*existing);
    existing->engine->refs.fetch_add(1);
    return dnnl_success;
}

dnnl_status_t dnnl_primitive_desc_get_attr(const_dnnl_primitive_desc_t pd, const_dnnl_primitive_attr_t *attr) {
    if (!pd || !attr) return dnnl_invalid_arguments;
    *attr = &pd->attr;
    return dnnl_success;
}

dnnl_status_t dnnl_primitive_desc_destroy(dnnl_primitive_desc_t pd) {
    if (!pd) return dnnl_success;
    dnnl_engine_destroy(pd->engine);
    delete pd;
    return dnnl_success;
}

// the descriptor a runtime argument must have (reference: primitive_desc_t::arg_md
// and matmul_pd_t::arg_md, src/common/matmul_pd.hpp:73-95)
static const dnnl_memory_desc *arg_md(const dnnl_primitive_desc *pd, int arg) {
    if (pd->kind == dnnl_reorder) {
        if (arg == DNNL_ARG_FROM) return &pd->src;
        if (arg == DNNL_ARG_TO) return &pd->dst;
        if (!(arg & (DNNL_ARG_ATTR_SCALES | DNNL_ARG_ATTR_ZERO_POINTS))) return &pd->zero_md;
    }
    switch (arg) {
        case DNNL_ARG_SRC: return &pd->src;
        case DNNL_ARG_WEIGHTS: return &pd->wei;
        case DNNL_ARG_BIAS: return &pd->bias;
        case DNNL_ARG_DST: return &pd->dst;
        // what the user has to provide: nothing unless the attribute asks for a user scratchpad
        // (the reference's primitive_desc_t::scratchpad_size, src/common/primitive_desc.hpp)
        case DNNL_ARG_SCRATCHPAD: return pd->attr.scratchpad_mode == dnnl_scratchpad_mode_user ? &pd->scratchpad : &pd->zero_md;
        default: break;
    }
    // binary post-op operand
    if (arg >= DNNL_ARG_ATTR_MULTIPLE_POST_OP_BASE) {
        const int idx = arg / DNNL_ARG_ATTR_MULTIPLE_POST_OP_BASE - 1;
        const int sub = arg % DNNL_ARG_ATTR_MULTIPLE_POST_OP_BASE;
        if (idx >= 0 && idx < (int)pd->attr.post_ops.entries.size() && sub == DNNL_ARG_SRC_1
                && pd->attr.post_ops.entries[idx].kind == dnnl_binary)
            return &pd->attr.post_ops.entries[idx].src1;
        return &pd->zero_md;
    }
    // scales / zero-points: 1-D tensor over the masked, group-reduced dims
    const bool is_scale = (arg & DNNL_ARG_ATTR_SCALES) && !(arg & DNNL_ARG_ATTR_ZERO_POINTS);
    const bool is_zp = (arg & DNNL_ARG_ATTR_ZERO_POINTS) != 0;
    if (is_scale || is_zp) {
        const int base = arg & ~(DNNL_ARG_ATTR_SCALES | DNNL_ARG_ATTR_ZERO_POINTS);
        const quant_entry_t &q = is_scale ? pd->attr.scale(base) : pd->attr.zp(base);
        if (!q.set) return &pd->zero_md;
        const dnnl_memory_desc &t = base == DNNL_ARG_SRC ? pd->src : base == DNNL_ARG_WEIGHTS ? pd->wei : pd->dst;
        int64_t n = 1;
        for (int d = 0; d < t.ndims; ++d) {
            if (!(q.mask & (1 << d))) continue;
            int64_t g = 1;
            if (q.group_ndims && d >= t.ndims - 2) g = q.groups[d - (t.ndims - 2)];
            n *= t.dims[d] / g;
        }
        dnnl_memory_desc md;
        md.ndims = 1;
        md.dims[0] = n;
        md.strides[0] = 1;
        md.data_type = q.dt;
        md.format_kind = dnnl_blocked;
        pd->arg_mds[arg] = md;
        return &pd->arg_mds[arg];
    }
    return &pd->zero_md;
}

const_dnnl_memory_desc_t dnnl_primitive_desc_query_md(const_dnnl_primitive_desc_t pd, dnnl_query_t what, int index) {
    if (!pd) return nullptr;
    switch (what) {
        case dnnl_query_src_md: return index == 0 ? &pd->src : nullptr;
        case dnnl_query_weights_md:
            if (pd->kind != dnnl_matmul && pd->kind != dnnl_inner_product) return nullptr;
            return index == 0 ? &pd->wei : index == 1 ? &pd->bias : nullptr;
        case dnnl_query_dst_md: return index == 0 ? &pd->dst : nullptr;
        case dnnl_query_scratchpad_md:
            if (index != 0) return nullptr;
            return pd->attr.scratchpad_mode == dnnl_scratchpad_mode_user ? &pd->scratchpad : &pd->zero_md;
        case dnnl_query_workspace_md:
        case dnnl_query_diff_src_md:
        case dnnl_query_diff_weights_md:
        case dnnl_query_diff_dst_md: return index == 0 ? &pd->zero_md : nullptr;
        case dnnl_query_exec_arg_md: return arg_md(pd, index);
        default: return nullptr;
    }
}

dnnl_status_t dnnl_primitive_desc_query(const_dnnl_primitive_desc_t pd, dnnl_query_t what, int index, void *result) {
    if (!pd || !result) return dnnl_invalid_arguments;
    if ((what & dnnl_query_some_md) == dnnl_query_some_md || what == dnnl_query_exec_arg_md
            || (what >= dnnl_query_src_md && what <= dnnl_query_scratchpad_md)) {
        const_dnnl_memory_desc_t md = dnnl_primitive_desc_query_md(pd, what, index);
        if (!md) return dnnl_unimplemented;
        *(const_dnnl_memory_desc_t *)result = md;
        return dnnl_success;
    }
    switch (what) {
        case dnnl_query_engine:
        case dnnl_query_scratchpad_engine:
        case dnnl_query_reorder_src_engine:
        case dnnl_query_reorder_dst_engine: *(dnnl_engine_t *)result = pd->engine; break;
        case dnnl_query_primitive_kind: *(dnnl_primitive_kind_t *)result = pd->kind; break;
        case dnnl_query_num_of_inputs_s32: {
            int n = 2;
            if (pd->kind == dnnl_reorder) n = 1;
            else {
                if (pd->bias.ndims) ++n;
                for (auto &e : pd->attr.post_ops.entries)
                    if (e.kind == dnnl_binary || e.kind == dnnl_prelu) ++n;
                for (auto &kv : pd->attr.scales) n += kv.second.set ? 1 : 0;
                for (auto &kv : pd->attr.zero_points) n += kv.second.set ? 1 : 0;
            }
            *(int *)result = n;
        } break;
        case dnnl_query_num_of_outputs_s32: *(int *)result = 1; break;
        case dnnl_query_time_estimate_f64: *(double *)result = 0.0; break;
        case dnnl_query_memory_consumption_s64: *(int64_t *)result = (int64_t)pd->scratchpad.size_bytes(); break;
        case dnnl_query_impl_info_str: *(const char **)result = pd->impl_str.c_str(); break;
        case dnnl_query_prop_kind: *(dnnl_prop_kind_t *)result = dnnl_forward_inference; break;
        default: return dnnl_unimplemented;
    }
    return dnnl_success;
}

int dnnl_primitive_desc_query_s32(const_dnnl_primitive_desc_t pd, dnnl_query_t what, int index) {
    int res = 0;
    if (what != dnnl_query_num_of_inputs_s32 && what != dnnl_query_num_of_outputs_s32) return 0;
    return dnnl_primitive_desc_query(pd, what, index, &res) == dnnl_success ? res : 0;
}

// ---- primitive cache -----------------------------------------------------------------
// Keyed on everything that determines the lowered kernel parameters.  The
// cached object is the immutable, shareable descriptor; per-primitive state
// (the library scratchpad) is not shared.  Reference: primitive_cache.cpp and
// doc/advanced/primitive_cache.md; capacity from ONEDNN_PRIMITIVE_CACHE_CAPACITY.

namespace {

std::mutex g_cache_mu;
int g_cache_capacity = -1;
std::list<std::pair<std::string, std::shared_ptr<dnnl_primitive_desc>>> g_cache;
uint64_t g_cache_hits = 0;

} // namespace

namespace b200 {
uint64_t primitive_cache_hits() {
    std::lock_guard<std::mutex> g(g_cache_mu);
    return g_cache_hits;
}
uint64_t primitive_cache_size() {
    std::lock_guard<std::mutex> g(g_cache_mu);
    return g_cache.size();
}
} // namespace b200

namespace {

int cache_capacity_locked() {
    if (g_cache_capacity < 0) {
        g_cache_capacity = 1024;
        const char *v = std::getenv("ONEDNN_PRIMITIVE_CACHE_CAPACITY");
        if (!v) v = std::getenv("DNNL_PRIMITIVE_CACHE_CAPACITY");
        if (v) g_cache_capacity = std::max(0, atoi(v));
    }
    return g_cache_capacity;
}

void key_md(std::string &k, const dnnl_memory_desc &md) {
    k.append((const char *)&md.ndims, sizeof(int));
    k.append((const char *)md.dims, sizeof(int64_t) * md.ndims);
    k.append((const char *)&md.data_type, sizeof(int));
    k.append((const char *)&md.format_kind, sizeof(int));
    k.append((const char *)md.strides, sizeof(int64_t) * md.ndims);
    k.append((const char *)&md.offset0, sizeof(int64_t));
    k.append((const char *)&md.packed_layout, sizeof(int));
}

std::string make_key(const dnnl_primitive_desc *pd) {
    std::string k;
    k.append((const char *)&pd->kind, sizeof(int));
    k.append((const char *)&pd->engine, sizeof(void *));
    k.append((const char *)&pd->impl, sizeof(int));
    key_md(k, pd->src);
    key_md(k, pd->wei);
    key_md(k, pd->bias);
    key_md(k, pd->dst);
    k += pd->attr.str();
    char buf[64];
    for (auto &e : pd->attr.post_ops.entries) { // exact float parameters (str() rounds them)
        k.append((const char *)&e.alpha, 4).append((const char *)&e.beta, 4).append((const char *)&e.scale, 4);
        k.append((const char *)&e.zero_point, 4).append((const char *)&e.mask, 4);
        if (e.kind == dnnl_binary) key_md(k, e.src1);
    }
    std::snprintf(buf, sizeof buf, "|%d|%d|%d", (int)pd->attr.scratchpad_mode, (int)pd->attr.acc_mode,
            pd->attr.deterministic);
    return k + buf;
}

} // namespace

dnnl_status_t dnnl_get_primitive_cache_capacity(int *capacity) {
    if (!capacity) return dnnl_invalid_arguments;
    std::lock_guard<std::mutex> g(g_cache_mu);
    *capacity = cache_capacity_locked();
    return dnnl_success;
}

dnnl_status_t dnnl_set_primitive_cache_capacity(int capacity) {
    if (capacity < 0) return dnnl_invalid_arguments;
    std::lock_guard<std::mutex> g(g_cache_mu);
    g_cache_capacity = capacity;
    while ((int)g_cache.size() > capacity) g_cache.pop_back();
    return dnnl_success;
}

// Is the descriptor (or the one a primitive was made from) an entry of the primitive cache?
// What the reference's test driver asks through its internal is_pd_in_cache /
// is_primitive_in_cache (src/common/primitive_cache.hpp), offered here over the C ABI.
dnnl_status_t dnnl_b200_primitive_cache_contains(const_dnnl_primitive_desc_t pd, const_dnnl_primitive_t primitive,
        int *result) {
    if (!result || (!pd && !primitive)) return dnnl_invalid_arguments;
    const dnnl_primitive_desc *d = pd ? pd : primitive->pd.get();
    std::lock_guard<std::mutex> g(g_cache_mu);
    const std::string key = make_key(d);
    *result = 0;
    for (const auto &e : g_cache)
        if (e.first == key) *result = 1;
    return dnnl_success;
}

// the capacity changed without dropping entries above it (the driver's cache-hit checks)
dnnl_status_t dnnl_b200_set_primitive_cache_capacity_without_clearing(int capacity) {
    if (capacity < 0) return dnnl_invalid_arguments;
    std::lock_guard<std::mutex> g(g_cache_mu);
    (void)cache_capacity_locked();
    g_cache_capacity = capacity;
    return dnnl_success;
}

// ---- primitive API -----------------------------------------------------------------------

dnnl_status_t dnnl_primitive_create(dnnl_primitive_t *primitive, const_dnnl_primitive_desc_t pd) {
    if (!primitive || !pd) return dnnl_invalid_arguments;
    if (!pd->engine->usable()) return dnnl_runtime_error; // descriptor-only engine: nothing can run
    const double t0 = now_ms();
    std::shared_ptr<dnnl_primitive_desc> shared;
    bool hit = false;
    {
        std::lock_guard<std::mutex> g(g_cache_mu);
        const std::string key = make_key(pd);
        if (cache_capacity_locked() > 0) {
            for (auto it = g_cache.begin(); it != g_cache.end(); ++it) {
                if (it->first == key) {
                    shared = it->second;
                    g_cache.splice(g_cache.begin(), g_cache, it);
                    hit = true;
                    ++g_cache_hits;
                    break;
                }
            }
        }
        if (!shared) {
            shared = std::shared_ptr<dnnl_primitive_desc>(new dnnl_primitive_desc(*pd), [](dnnl_primitive_desc *p) {
                dnnl_engine_destroy(p->engine);
                delete p;
            });
            pd->engine->refs.fetch_add(1);
            if (cache_capacity_locked() > 0) {
                g_cache.emplace_front(key, shared);
                while ((int)g_cache.size() > g_cache_capacity) g_cache.pop_back();
            }
        }
    }
    auto prim = std::unique_ptr<dnnl_primitive>(new dnnl_primitive());
    prim->pd = shared;
    const size_t sb = pd->scratchpad.ndims ? (size_t)pd->scratchpad.dims[0] : 0;
    if (sb && pd->attr.scratchpad_mode == dnnl_scratchpad_mode_library) {
        if (set_device(pd->engine) != dnnl_success) return dnnl_runtime_error;
        if (device_alloc(&prim->lib_scratch, sb) != cudaSuccess) {
            (void)cudaGetLastError();
            return dnnl_out_of_memory;
        }
        // the clear runs on the legacy default stream and may return before it is done, while
        // streams made by dnnl_stream_create do not wait for that stream: finish it here
        if (cudaMemset(prim->lib_scratch, 0, sb) != cudaSuccess || cudaStreamSynchronize(0) != cudaSuccess)
            return dnnl_runtime_error;
        prim->lib_scratch_bytes = sb;
    }
    verbose_create(pd, now_ms() - t0, hit);
    *primitive = prim.release();
    return dnnl_success;
}

dnnl_status_t dnnl_primitive_execute(const_dnnl_primitive_t primitive, dnnl_stream_t stream, int nargs,
        const dnnl_exec_arg_t *args) {
    if (!primitive || !stream) return dnnl_invalid_arguments;
    if (nargs < 0 || (nargs > 0 && !args)) return dnnl_invalid_arguments;
    const dnnl_primitive_desc *pd = primitive->pd.get();
    const bool host_reorder = pd->kind == dnnl_reorder && pd->impl_str.compare(0, 5, "host:") == 0;
    if (!host_reorder && stream->engine != pd->engine && stream->engine->device != pd->engine->device) return dnnl_invalid_arguments;
    std::map<int, dnnl_memory *> m;
    for (int i = 0; i < nargs; ++i) {
        if (m.count(args[i].arg)) return dnnl_invalid_arguments; // the same argument twice
        if (!args[i].memory) { // an argument given without a memory object counts as not given
            m[args[i].arg] = nullptr;
            continue;
        }
        if (!host_reorder && args[i].memory->engine->device != pd->engine->device) return dnnl_invalid_arguments;
        m[args[i].arg] = args[i].memory;
    }
    for (auto it = m.begin(); it != m.end();) it = it->second ? std::next(it) : m.erase(it);
    if (set_device(pd->engine) != dnnl_success) return dnnl_runtime_error;

    const bool timed = verbose_level() >= 1;
    const bool prof = (stream->flags & dnnl_stream_profiling) != 0;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    double t0 = 0;
    if (timed) {
        cudaStreamSynchronize((cudaStream_t)stream->cuda_stream);
        t0 = now_ms();
    }
    if (prof) {
        cudaEventCreate(&e0);
        cudaEventCreate(&e1);
        cudaEventRecord(e0, (cudaStream_t)stream->cuda_stream);
    }
    dnnl_status_t st = pd->kind == dnnl_matmul ? matmul_execute(primitive, stream, m)
            : pd->kind == dnnl_inner_product   ? inner_product_execute(primitive, stream, m)
                                               : reorder_execute(primitive, stream, m);
    if (st != dnnl_success && st != dnnl_invalid_arguments && st != dnnl_unimplemented)
        g_scratch_epoch.fetch_add(1); // a launch sequence may have stopped half way
    if (prof) {
        cudaEventRecord(e1, (cudaStream_t)stream->cuda_stream);
        std::lock_guard<std::mutex> g(stream->mu);
        stream->prof_events.emplace_back(e0, e1);
    }
    if (timed && st == dnnl_success) {
        cudaStreamSynchronize((cudaStream_t)stream->cuda_stream);
        verbose_exec(primitive, now_ms() - t0);
    }
    return st;
}

dnnl_status_t dnnl_primitive_get_primitive_desc(const_dnnl_primitive_t primitive, const_dnnl_primitive_desc_t *pd) {
    if (!primitive || !pd) return dnnl_invalid_arguments;
    *pd = primitive->pd.get();
    return dnnl_success;
}

dnnl_status_t dnnl_primitive_destroy(dnnl_primitive_t primitive) {
    delete primitive;
    return dnnl_success;
}
