// Runs ONE matmul problem through the reference library's own public C API on
// its CPU engine -- TEST INFRASTRUCTURE ONLY (never linked into the product).
//
// The problem is described by the same orc_problem_t the C oracle takes, so a
// test can hand identical buffers to both.  Restrictions of this runner: plain
// 2-D tensors (any strides), scales/zero-points with the masks the matmul
// primitive admits, and the post-op kinds sum / eltwise / binary / prelu.
//
// refrun_matmul(problem, impl_filter, weights_any, iters, *ms_min, *ms_avg, impl_out)
//   impl_filter: "" = first implementation the library dispatches (its JIT),
//                otherwise iterate dnnl_primitive_desc_next_impl until the
//                implementation name contains the filter (e.g. "ref").
//   weights_any: 1 = let the library choose its packed weights layout and
//                reorder the plain weights into it once (not timed).
//   iters > 0:   time `iters` executions after one warm-up.
#include "oracle_matmul.h"

#include <chrono>
#include <cstdio>
#include <cstring>
#include <vector>

#include "oneapi/dnnl/dnnl.h"

#define CK(x) \
    do { \
        dnnl_status_t s_ = (x); \
        if (s_ != dnnl_success) { \
            std::fprintf(stderr, "refrun: %s failed with %d (line %d)\n", #x, (int)s_, __LINE__); \
            return 100 + (int)s_; \
        } \
    } while (0)

namespace {

struct md_guard {
    dnnl_memory_desc_t md = nullptr;
    ~md_guard() { if (md) dnnl_memory_desc_destroy(md); }
};

dnnl_status_t make_md(dnnl_memory_desc_t *md, int nd, const int64_t *dims, int dt, const int64_t *strides) {
    return dnnl_memory_desc_create_with_strides(md, nd, dims, (dnnl_data_type_t)dt, strides);
}

// number of elements a scale/zero-point argument spans
int64_t quant_count(const orc_quant_t &q, int64_t d0, int64_t d1) {
    int64_t n0 = q.s0 ? d0 / q.g0 : 1;
    int64_t n1 = q.s1 ? d1 / q.g1 : 1;
    return n0 * n1;
}

int quant_mask(const orc_quant_t &q) { return (q.s0 ? 1 : 0) | (q.s1 ? 2 : 0); }

} // namespace

extern "C" __attribute__((visibility("default"))) int refrun_version(int *major, int *minor, int *patch) {
    const dnnl_version_t *v = dnnl_version();
    *major = v->major; *minor = v->minor; *patch = v->patch;
    return 0;
}

extern "C" __attribute__((visibility("default"))) int refrun_matmul(const orc_problem_t *p, const char *impl_filter,
        int weights_any, int iters, double *ms_min, double *ms_avg, char *impl_out, int impl_out_len) {
    dnnl_engine_t eng;
    CK(dnnl_engine_create(&eng, dnnl_cpu, 0));
    dnnl_stream_t strm;
    CK(dnnl_stream_create(&strm, eng, dnnl_stream_default_flags));

    const int64_t sdims[2] = {p->M, p->K}, wdims[2] = {p->K, p->N}, ddims[2] = {p->M, p->N};
    const int64_t sstr[2] = {p->src_sm, p->src_sk}, wstr[2] = {p->wei_sk, p->wei_sn}, dstr[2] = {p->dst_sm, p->dst_sn};
    dnnl_memory_desc_t src_md, wei_md, wei_any_md = nullptr, dst_md, bia_md = nullptr;
    CK(make_md(&src_md, 2, sdims, p->src_dt, sstr));
    CK(make_md(&wei_md, 2, wdims, p->wei_dt, wstr));
    CK(make_md(&dst_md, 2, ddims, p->dst_dt, dstr));
    if (weights_any)
        CK(dnnl_memory_desc_create_with_tag(&wei_any_md, 2, wdims, (dnnl_data_type_t)p->wei_dt, dnnl_format_tag_any));
    int64_t bdims[2] = {1, 1};
    if (p->bias) {
        bdims[0] = p->bias_sm ? p->M : 1;
        bdims[1] = p->bias_sn ? p->N : 1;
        const int64_t bstr[2] = {p->bias_sm ? p->bias_sm : bdims[1], p->bias_sn ? p->bias_sn : 1};
        CK(make_md(&bia_md, 2, bdims, p->bias_dt, bstr));
    }

    dnnl_primitive_attr_t attr;
    CK(dnnl_primitive_attr_create(&attr));
    CK(dnnl_primitive_attr_set_scratchpad_mode(attr, dnnl_scratchpad_mode_library));
    if (p->apply_to_int) CK(dnnl_primitive_attr_set_fpmath_mode_v2(attr, dnnl_fpmath_mode_bf16, 1));

    struct qarg { const orc_quant_t *q; int arg; bool is_zp; int64_t d0, d1; };
    const qarg qs[6] = {
        {&p->src_scale, DNNL_ARG_SRC, false, p->M, p->K}, {&p->wei_scale, DNNL_ARG_WEIGHTS, false, p->K, p->N},
        {&p->dst_scale, DNNL_ARG_DST, false, p->M, p->N}, {&p->src_zp, DNNL_ARG_SRC, true, p->M, p->K},
        {&p->wei_zp, DNNL_ARG_WEIGHTS, true, p->K, p->N}, {&p->dst_zp, DNNL_ARG_DST, true, p->M, p->N}};
    for (const qarg &a : qs) {
        if (!a.q->ptr) continue;
        const int mask = quant_mask(*a.q);
        const bool grouped = a.q->g0 > 1 || a.q->g1 > 1;
        const int64_t groups[2] = {a.q->g0, a.q->g1};
        if (a.is_zp)
            CK(dnnl_primitive_attr_set_zero_points(attr, a.arg, mask, grouped ? 2 : 0, groups, (dnnl_data_type_t)a.q->dt));
        else
            CK(dnnl_primitive_attr_set_scales(attr, a.arg, mask, grouped ? 2 : 0, groups, (dnnl_data_type_t)a.q->dt));
    }

    std::vector<dnnl_memory_desc_t> po_mds;
    if (p->npo > 0) {
        dnnl_post_ops_t po;
        CK(dnnl_post_ops_create(&po));
        for (int i = 0; i < p->npo; ++i) {
            const orc_postop_t &e = p->po[i];
            if (e.kind == ORC_PO_SUM) {
                CK(dnnl_post_ops_append_sum(po, e.scale, e.zero_point, (dnnl_data_type_t)e.dt));
            } else if (e.kind == ORC_PO_ELTWISE) {
                CK(dnnl_post_ops_append_eltwise(po, (dnnl_alg_kind_t)e.alg, e.alpha, e.beta));
            } else if (e.kind == ORC_PO_BINARY) {
                const int64_t d[2] = {e.sm ? p->M : 1, e.sn ? p->N : 1};
                const int64_t st[2] = {e.sm ? e.sm : d[1], e.sn ? e.sn : 1};
                dnnl_memory_desc_t md;
                CK(make_md(&md, 2, d, e.dt, st));
                po_mds.push_back(md);
                CK(dnnl_post_ops_append_binary(po, (dnnl_alg_kind_t)e.alg, md));
            } else if (e.kind == ORC_PO_PRELU) {
                CK(dnnl_post_ops_append_prelu(po, (e.sm ? 1 : 0) | (e.sn ? 2 : 0)));
            }
        }
        CK(dnnl_primitive_attr_set_post_ops(attr, po));
        CK(dnnl_post_ops_destroy(po));
    }

    dnnl_primitive_desc_t pd;
    CK(dnnl_matmul_primitive_desc_create(&pd, eng, src_md, weights_any ? wei_any_md : wei_md, bia_md, dst_md, attr));
    const char *impl = nullptr;
    for (;;) {
        CK(dnnl_primitive_desc_query(pd, dnnl_query_impl_info_str, 0, &impl));
        if (!impl_filter || !impl_filter[0] || std::strstr(impl, impl_filter)) break;
        dnnl_status_t s = dnnl_primitive_desc_next_impl(pd);
        if (s != dnnl_success) {
            std::fprintf(stderr, "refrun: no implementation matching '%s'\n", impl_filter);
            return 3;
        }
    }
    if (impl_out && impl_out_len > 0) std::snprintf(impl_out, impl_out_len, "%s", impl);

    dnnl_primitive_t prim;
    CK(dnnl_primitive_create(&prim, pd));

    std::vector<dnnl_exec_arg_t> args;
    std::vector<dnnl_memory_t> mems;
    auto add = [&](int arg, const_dnnl_memory_desc_t md, const void *ptr) -> dnnl_status_t {
        dnnl_memory_t m;
        dnnl_status_t s = dnnl_memory_create(&m, md, eng, const_cast<void *>(ptr));
        if (s != dnnl_success) return s;
        mems.push_back(m);
        args.push_back({arg, m});
        return dnnl_success;
    };
    CK(add(DNNL_ARG_SRC, src_md, p->src));
    const_dnnl_memory_desc_t wei_q = dnnl_primitive_desc_query_md(pd, dnnl_query_weights_md, 0);
    if (weights_any && !dnnl_memory_desc_equal(wei_q, wei_md)) {
        dnnl_memory_t plain, packed;
        CK(dnnl_memory_create(&plain, wei_md, eng, const_cast<void *>(p->wei)));
        CK(dnnl_memory_create(&packed, wei_q, eng, DNNL_MEMORY_ALLOCATE));
        dnnl_primitive_desc_t rpd;
        // the packed layout of an int8 matmul with a source zero-point carries
        // compensation; the reorder needs the same attr only when it quantises
        CK(dnnl_reorder_primitive_desc_create(&rpd, wei_md, eng, wei_q, eng, nullptr));
        dnnl_primitive_t r;
        CK(dnnl_primitive_create(&r, rpd));
        dnnl_exec_arg_t ra[2] = {{DNNL_ARG_FROM, plain}, {DNNL_ARG_TO, packed}};
        CK(dnnl_primitive_execute(r, strm, 2, ra));
        CK(dnnl_stream_wait(strm));
        dnnl_primitive_destroy(r);
        dnnl_primitive_desc_destroy(rpd);
        dnnl_memory_destroy(plain);
        mems.push_back(packed);
        args.push_back({DNNL_ARG_WEIGHTS, packed});
    } else {
        CK(add(DNNL_ARG_WEIGHTS, wei_q, p->wei));
    }
    if (p->bias) CK(add(DNNL_ARG_BIAS, bia_md, p->bias));
    CK(add(DNNL_ARG_DST, dst_md, p->dst));

    std::vector<md_guard> qmds(6);
    for (int i = 0; i < 6; ++i) {
        const qarg &a = qs[i];
        if (!a.q->ptr) continue;
        const int64_t n = quant_count(*a.q, a.d0, a.d1);
        const int64_t one = 1;
        CK(make_md(&qmds[i].md, 1, &n, a.q->dt, &one));
        CK(add((a.is_zp ? DNNL_ARG_ATTR_ZERO_POINTS : DNNL_ARG_ATTR_SCALES) | a.arg, qmds[i].md, a.q->ptr));
    }
    std::vector<md_guard> pmds(p->npo);
    size_t bi = 0;
    for (int i = 0; i < p->npo; ++i) {
        const orc_postop_t &e = p->po[i];
        if (e.kind == ORC_PO_BINARY) {
            CK(add(DNNL_ARG_ATTR_MULTIPLE_POST_OP(i) | DNNL_ARG_SRC_1, po_mds[bi++], e.ptr));
        } else if (e.kind == ORC_PO_PRELU) {
            const int64_t d[2] = {e.sm ? p->M : 1, e.sn ? p->N : 1};
            const int64_t st[2] = {d[1], 1};
            CK(make_md(&pmds[i].md, 2, d, dnnl_f32, st));
            CK(add(DNNL_ARG_ATTR_MULTIPLE_POST_OP(i) | DNNL_ARG_WEIGHTS, pmds[i].md, e.ptr));
        }
    }

    CK(dnnl_primitive_execute(prim, strm, (int)args.size(), args.data()));
    CK(dnnl_stream_wait(strm));
    if (iters > 0) {
        double tmin = 1e30, tsum = 0;
        for (int it = 0; it < iters; ++it) {
            auto t0 = std::chrono::steady_clock::now();
            CK(dnnl_primitive_execute(prim, strm, (int)args.size(), args.data()));
            CK(dnnl_stream_wait(strm));
            double ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
            tmin = ms < tmin ? ms : tmin;
            tsum += ms;
        }
        if (ms_min) *ms_min = tmin;
        if (ms_avg) *ms_avg = tsum / iters;
    }

    for (dnnl_memory_t m : mems) dnnl_memory_destroy(m);
    for (dnnl_memory_desc_t m : po_mds) dnnl_memory_desc_destroy(m);
    dnnl_primitive_destroy(prim);
    dnnl_primitive_desc_destroy(pd);
    dnnl_primitive_attr_destroy(attr);
    dnnl_memory_desc_destroy(src_md);
    dnnl_memory_desc_destroy(wei_md);
    dnnl_memory_desc_destroy(dst_md);
    if (wei_any_md) dnnl_memory_desc_destroy(wei_any_md);
    if (bia_md) dnnl_memory_desc_destroy(bia_md);
    dnnl_stream_destroy(strm);
    dnnl_engine_destroy(eng);
    return 0;
}

// refrun_reorder(problem, impl_filter, impl_out): one quantising reorder of a plain 2-D
// tensor through dnnl_reorder_primitive_desc_create on the CPU engine, with the scales,
// zero-points and the optional sum post-op of orc_reorder_t as attributes.
extern "C" __attribute__((visibility("default"))) int refrun_reorder(const orc_reorder_t *r, const char *impl_filter,
        char *impl_out, int impl_out_len) {
    dnnl_engine_t eng;
    CK(dnnl_engine_create(&eng, dnnl_cpu, 0));
    dnnl_stream_t strm;
    CK(dnnl_stream_create(&strm, eng, dnnl_stream_default_flags));
    const int64_t dims[2] = {r->rows, r->cols};
    const int64_t sstr[2] = {r->src_s0, r->src_s1}, dstr[2] = {r->dst_s0, r->dst_s1};
    dnnl_memory_desc_t src_md, dst_md;
    CK(make_md(&src_md, 2, dims, r->src_dt, sstr));
    CK(make_md(&dst_md, 2, dims, r->dst_dt, dstr));

    dnnl_primitive_attr_t attr;
    CK(dnnl_primitive_attr_create(&attr));
    struct qarg { const orc_quant_t *q; int arg; bool is_zp; };
    const qarg qs[4] = {{&r->src_scale, DNNL_ARG_SRC, false}, {&r->dst_scale, DNNL_ARG_DST, false},
            {&r->src_zp, DNNL_ARG_SRC, true}, {&r->dst_zp, DNNL_ARG_DST, true}};
    for (const qarg &a : qs) {
        if (!a.q->ptr) continue;
        const int mask = quant_mask(*a.q);
        const bool grouped = a.q->g0 > 1 || a.q->g1 > 1;
        const int64_t groups[2] = {a.q->g0, a.q->g1};
        if (a.is_zp)
            CK(dnnl_primitive_attr_set_zero_points(attr, a.arg, mask, grouped ? 2 : 0, groups, (dnnl_data_type_t)a.q->dt));
        else
            CK(dnnl_primitive_attr_set_scales(attr, a.arg, mask, grouped ? 2 : 0, groups, (dnnl_data_type_t)a.q->dt));
    }
    if (r->beta != 0.f) {
        dnnl_post_ops_t po;
        CK(dnnl_post_ops_create(&po));
        CK(dnnl_post_ops_append_sum(po, r->beta, 0, dnnl_data_type_undef));
        CK(dnnl_primitive_attr_set_post_ops(attr, po));
        CK(dnnl_post_ops_destroy(po));
    }

    dnnl_primitive_desc_t pd;
    CK(dnnl_reorder_primitive_desc_create(&pd, src_md, eng, dst_md, eng, attr));
    const char *impl = nullptr;
    for (;;) {
        CK(dnnl_primitive_desc_query(pd, dnnl_query_impl_info_str, 0, &impl));
        if (!impl_filter || !impl_filter[0] || std::strstr(impl, impl_filter)) break;
        if (dnnl_primitive_desc_next_impl(pd) != dnnl_success) {
            std::fprintf(stderr, "refrun: no reorder implementation matching '%s'\n", impl_filter);
            return 3;
        }
    }
    if (impl_out && impl_out_len > 0) std::snprintf(impl_out, impl_out_len, "%s", impl);
    dnnl_primitive_t prim;
    CK(dnnl_primitive_create(&prim, pd));

    std::vector<dnnl_exec_arg_t> args;
    std::vector<dnnl_memory_t> mems;
    auto add = [&](int arg, const_dnnl_memory_desc_t md, const void *ptr) -> dnnl_status_t {
        dnnl_memory_t m;
        dnnl_status_t s = dnnl_memory_create(&m, md, eng, const_cast<void *>(ptr));
        if (s != dnnl_success) return s;
        mems.push_back(m);
        args.push_back({arg, m});
        return dnnl_success;
    };
    CK(add(DNNL_ARG_FROM, src_md, r->src));
    CK(add(DNNL_ARG_TO, dst_md, r->dst));
    std::vector<md_guard> qmds(4);
    for (int i = 0; i < 4; ++i) {
        const qarg &a = qs[i];
        if (!a.q->ptr) continue;
        const int64_t n = quant_count(*a.q, r->rows, r->cols);
        const int64_t one = 1;
        CK(make_md(&qmds[i].md, 1, &n, a.q->dt, &one));
        CK(add((a.is_zp ? DNNL_ARG_ATTR_ZERO_POINTS : DNNL_ARG_ATTR_SCALES) | a.arg, qmds[i].md, a.q->ptr));
    }
    CK(dnnl_primitive_execute(prim, strm, (int)args.size(), args.data()));
    CK(dnnl_stream_wait(strm));

    for (dnnl_memory_t m : mems) dnnl_memory_destroy(m);
    dnnl_primitive_destroy(prim);
    dnnl_primitive_desc_destroy(pd);
    dnnl_primitive_attr_destroy(attr);
    dnnl_memory_desc_destroy(src_md);
    dnnl_memory_desc_destroy(dst_md);
    dnnl_stream_destroy(strm);
    dnnl_engine_destroy(eng);
    return 0;
}
