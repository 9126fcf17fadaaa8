// Primitive attributes and post-ops: scales / zero-points (mask, data type,
// group sizes) per argument, fpmath mode with apply_to_int, accumulation and
// scratchpad modes, rounding, and the ordered post-op list.  Argument checks
// and status codes follow the reference's C API
// (src/common/primitive_attr.cpp:150-265 append rules, :408-804 setters/getters).
#include <cmath>
#include <cstdio>

#include "internal.hpp"

using namespace b200;

namespace b200 {
const quant_entry_t default_quant_entry;
static std::mutex g_fpmath_mu;
static dnnl_fpmath_mode_t g_default_fpmath = dnnl_fpmath_mode_strict;
static bool g_default_fpmath_init = false;

static dnnl_fpmath_mode_t default_fpmath() {
    std::lock_guard<std::mutex> g(g_fpmath_mu);
    if (!g_default_fpmath_init) {
        g_default_fpmath_init = true;
        const char *v = std::getenv("ONEDNN_DEFAULT_FPMATH_MODE");
        if (!v) v = std::getenv("DNNL_DEFAULT_FPMATH_MODE");
        if (v) {
            std::string s(v);
            for (auto &c : s) c = (char)tolower(c);
            if (s == "bf16") g_default_fpmath = dnnl_fpmath_mode_bf16;
            else if (s == "f16") g_default_fpmath = dnnl_fpmath_mode_f16;
            else if (s == "tf32") g_default_fpmath = dnnl_fpmath_mode_tf32;
            else if (s == "any") g_default_fpmath = dnnl_fpmath_mode_any;
        }
    }
    return g_default_fpmath;
}
} // namespace b200

const quant_entry_t &dnnl_primitive_attr::scale(int arg) const {
    auto it = scales.find(arg);
    return it == scales.end() ? default_quant_entry : it->second;
}
const quant_entry_t &dnnl_primitive_attr::zp(int arg) const {
    auto it = zero_points.find(arg);
    return it == zero_points.end() ? default_quant_entry : it->second;
}

static const char *arg_name(int arg) {
    switch (arg) {
        case DNNL_ARG_SRC: return "src";
        case DNNL_ARG_WEIGHTS: return "wei";
        case DNNL_ARG_DST: return "dst";
        case DNNL_ARG_SRC_1: return "src1";
        default: return "arg";
    }
}

static const char *alg_name(int alg) {
    switch (alg) {
        case dnnl_eltwise_relu: return "eltwise_relu";
        case dnnl_eltwise_tanh: return "eltwise_tanh";
        case dnnl_eltwise_elu: return "eltwise_elu";
        case dnnl_eltwise_square: return "eltwise_square";
        case dnnl_eltwise_abs: return "eltwise_abs";
        case dnnl_eltwise_sqrt: return "eltwise_sqrt";
        case dnnl_eltwise_linear: return "eltwise_linear";
        case dnnl_eltwise_soft_relu: return "eltwise_soft_relu";
        case dnnl_eltwise_hardsigmoid: return "eltwise_hardsigmoid";
        case dnnl_eltwise_logistic: return "eltwise_logistic";
        case dnnl_eltwise_exp: return "eltwise_exp";
        case dnnl_eltwise_gelu_tanh: return "eltwise_gelu_tanh";
        case dnnl_eltwise_swish: return "eltwise_swish";
        case dnnl_eltwise_log: return "eltwise_log";
        case dnnl_eltwise_clip: return "eltwise_clip";
        case dnnl_eltwise_clip_v2: return "eltwise_clip_v2";
        case dnnl_eltwise_pow: return "eltwise_pow";
        case dnnl_eltwise_gelu_erf: return "eltwise_gelu_erf";
        case dnnl_eltwise_round: return "eltwise_round";
        case dnnl_eltwise_mish: return "eltwise_mish";
        case dnnl_eltwise_hardswish: return "eltwise_hardswish";
        case dnnl_binary_add: return "binary_add";
        case dnnl_binary_mul: return "binary_mul";
        case dnnl_binary_max: return "binary_max";
        case dnnl_binary_min: return "binary_min";
        case dnnl_binary_div: return "binary_div";
        case dnnl_binary_sub: return "binary_sub";
        case dnnl_binary_ge: return "binary_ge";
        case dnnl_binary_gt: return "binary_gt";
        case dnnl_binary_le: return "binary_le";
        case dnnl_binary_lt: return "binary_lt";
        case dnnl_binary_eq: return "binary_eq";
        case dnnl_binary_ne: return "binary_ne";
        default: return "alg";
    }
}

// the attribute as the reference's verbose line prints it, e.g.
// attr-scales:src0:0:f32+wei:2:f32 attr-zero-points:src0:0:s32 attr-post-ops:eltwise_relu
std::string dnnl_primitive_attr::str() const {
    std::string s;
    char buf[160];
    auto quant = [&](const char *name, const std::map<int, quant_entry_t> &m) {
        std::string q;
        for (auto &kv : m) {
            if (!kv.second.set) continue;
            if (!q.empty()) q += "+";
            std::snprintf(buf, sizeof buf, "%s:%d:%s", arg_name(kv.first), kv.second.mask, dt_name(kv.second.dt));
            q += buf;
            if (kv.second.group_ndims) {
                std::snprintf(buf, sizeof buf, ":%lldx%lld", (long long)kv.second.groups[0],
                        (long long)kv.second.groups[1]);
                q += buf;
            }
        }
        if (!q.empty()) s += std::string(s.empty() ? "" : " ") + name + q;
    };
    if (fpmath != dnnl_fpmath_mode_strict || apply_to_int) {
        const char *fm[] = {"strict", "bf16", "f16", "any", "tf32"};
        std::snprintf(buf, sizeof buf, "attr-fpmath:%s%s", fm[(int)fpmath], apply_to_int ? ":true" : "");
        s += buf;
    }
    quant("attr-scales:", scales);
    quant("attr-zero-points:", zero_points);
    if (!post_ops.entries.empty()) {
        std::string q;
        for (auto &e : post_ops.entries) {
            if (!q.empty()) q += "+";
            if (e.kind == dnnl_sum) {
                std::snprintf(buf, sizeof buf, "sum:%g:%d:%s", e.scale, e.zero_point, dt_name(e.dt));
            } else if (e.kind == dnnl_eltwise) {
                std::snprintf(buf, sizeof buf, "%s:%g:%g", alg_name(e.alg), e.alpha, e.beta);
            } else if (e.kind == dnnl_binary) {
                std::snprintf(buf, sizeof buf, "%s:%s", alg_name(e.alg), dt_name(e.src1.data_type));
            } else {
                std::snprintf(buf, sizeof buf, "prelu:%d", e.mask);
            }
            q += buf;
        }
        s += std::string(s.empty() ? "" : " ") + "attr-post-ops:" + q;
    }
    return s;
}

// ---- attribute API -----------------------------------------------------------

dnnl_status_t dnnl_primitive_attr_create(dnnl_primitive_attr_t *attr) {
    if (!attr) return dnnl_invalid_arguments;
    dnnl_primitive_attr *a = new dnnl_primitive_attr();
    a->fpmath = default_fpmath();
    *attr = a;
    return dnnl_success;
}

dnnl_status_t dnnl_primitive_attr_clone(dnnl_primitive_attr_t *attr, const_dnnl_primitive_attr_t existing) {
    if (!attr || !existing) return dnnl_invalid_arguments;
    *attr = new dnnl_primitive_attr(*existing);
    return dnnl_success;
}

dnnl_status_t dnnl_primitive_attr_destroy(dnnl_primitive_attr_t attr) {
    delete attr;
    return dnnl_success;
}

static bool fpmath_ok(int m) { return m >= dnnl_fpmath_mode_strict && m <= dnnl_fpmath_mode_tf32; }

dnnl_status_t dnnl_primitive_attr_get_fpmath_mode(const_dnnl_primitive_attr_t attr, dnnl_fpmath_mode_t *mode) {
    if (!attr || !mode) return dnnl_invalid_arguments;
    *mode = attr->fpmath;
    return dnnl_success;
}
dnnl_status_t dnnl_primitive_attr_set_fpmath_mode(dnnl_primitive_attr_t attr, dnnl_fpmath_mode_t mode) {
    if (!attr || !fpmath_ok(mode)) return dnnl_invalid_arguments;
    attr->fpmath = mode;
    attr->apply_to_int = 0;
    return dnnl_success;
}
dnnl_status_t dnnl_primitive_attr_get_fpmath_mode_v2(const_dnnl_primitive_attr_t attr, dnnl_fpmath_mode_t *mode,
        int *apply_to_int) {
    if (!attr) return dnnl_invalid_arguments;
    if (mode) *mode = attr->fpmath;
    if (apply_to_int) *apply_to_int = attr->apply_to_int;
    return dnnl_success;
}
dnnl_status_t dnnl_primitive_attr_set_fpmath_mode_v2(dnnl_primitive_attr_t attr, dnnl_fpmath_mode_t mode,
        int apply_to_int) {
    if (!attr || !fpmath_ok(mode)) return dnnl_invalid_arguments;
    attr->fpmath = mode;
    attr->apply_to_int = apply_to_int ? 1 : 0;
    return dnnl_success;
}
dnnl_status_t dnnl_primitive_attr_get_deterministic(const_dnnl_primitive_attr_t attr, int *value) {
    if (!attr || !value) return dnnl_invalid_arguments;
    *value = attr->deterministic;
    return dnnl_success;
}
dnnl_status_t dnnl_primitive_attr_set_deterministic(dnnl_primitive_attr_t attr, int value) {
    if (!attr) return dnnl_invalid_arguments;
    attr->deterministic = value ? 1 : 0;
    return dnnl_success;
}
dnnl_status_t dnnl_primitive_attr_get_accumulation_mode(const_dnnl_primitive_attr_t attr, dnnl_accumulation_mode_t *mode) {
    if (!attr || !mode) return dnnl_invalid_arguments;
    *mode = attr->acc_mode;
    return dnnl_success;
}
dnnl_status_t dnnl_primitive_attr_set_accumulation_mode(dnnl_primitive_attr_t attr, dnnl_accumulation_mode_t mode) {
    if (!attr || mode < dnnl_accumulation_mode_strict || mode > dnnl_accumulation_mode_f16) return dnnl_invalid_arguments;
    attr->acc_mode = mode;
    return dnnl_success;
}
dnnl_status_t dnnl_primitive_attr_get_scratchpad_mode(const_dnnl_primitive_attr_t attr, dnnl_scratchpad_mode_t *mode) {
    if (!attr || !mode) return dnnl_invalid_arguments;
    *mode = attr->scratchpad_mode;
    return dnnl_success;
}
dnnl_status_t dnnl_primitive_attr_set_scratchpad_mode(dnnl_primitive_attr_t attr, dnnl_scratchpad_mode_t mode) {
    if (!attr) return dnnl_invalid_arguments;
    if (mode != dnnl_scratchpad_mode_library && mode != dnnl_scratchpad_mode_user) return dnnl_invalid_arguments;
    attr->scratchpad_mode = mode;
    return dnnl_success;
}

static dnnl_status_t set_quant(std::map<int, quant_entry_t> &m, int arg, int mask, int ndims, const dnnl_dims_t groups,
        int dt) {
    if (ndims > 2) return dnnl_invalid_arguments;
    quant_entry_t e;
    e.set = true;
    e.mask = mask;
    e.dt = dt;
    e.group_ndims = ndims;
    if (ndims > 0) {
        if (!groups) return dnnl_invalid_arguments;
        for (int i = 0; i < ndims; ++i)
            if (groups[i] <= 0) return dnnl_invalid_arguments;
        if (ndims == 2) {
            e.groups[0] = groups[0];
            e.groups[1] = groups[1];
        } else {
            e.groups[1] = groups[0];
        }
    }
    m[arg] = e;
    return dnnl_success;
}

dnnl_status_t dnnl_primitive_attr_set_scales_mask(dnnl_primitive_attr_t attr, int arg, int mask) {
    if (!attr || mask < 0 || arg < 0) return dnnl_invalid_arguments;
    return set_quant(attr->scales, arg, mask, 0, nullptr, dnnl_f32);
}

dnnl_status_t dnnl_primitive_attr_set_scales(dnnl_primitive_attr_t attr, int arg, int mask, int ndims,
        const dnnl_dims_t group_dims, dnnl_data_type_t data_type) {
    if (!attr || mask < 0 || arg < 0 || ndims < 0) return dnnl_invalid_arguments;
    if (data_type != dnnl_f32 && data_type != dnnl_bf16 && data_type != dnnl_f16 && data_type != dnnl_e8m0
            && data_type != dnnl_f8_e5m2 && data_type != dnnl_f8_e4m3)
        return dnnl_invalid_arguments;
    return set_quant(attr->scales, arg, mask, ndims, group_dims, data_type);
}

dnnl_status_t dnnl_primitive_attr_set_zero_points_mask(dnnl_primitive_attr_t attr, int arg, int mask) {
    if (!attr || mask < 0) return dnnl_invalid_arguments;
    return set_quant(attr->zero_points, arg, mask, 0, nullptr, dnnl_s32);
}

dnnl_status_t dnnl_primitive_attr_set_zero_points(dnnl_primitive_attr_t attr, int arg, int mask, int ndims,
        const dnnl_dims_t group_dims, dnnl_data_type_t data_type) {
    if (!attr || mask < 0 || arg < 0 || ndims < 0) return dnnl_invalid_arguments;
    if (data_type != dnnl_s32 && data_type != dnnl_s8 && data_type != dnnl_u8 && data_type != dnnl_s4
            && data_type != dnnl_u4)
        return dnnl_invalid_arguments;
    if ((data_type == dnnl_s4 || data_type == dnnl_u4) && mask == 0) return dnnl_invalid_arguments;
    if (arg != DNNL_ARG_SRC && arg != DNNL_ARG_WEIGHTS && !(data_type == dnnl_s32 && ndims == 0))
        return dnnl_invalid_arguments;
    return set_quant(attr->zero_points, arg, mask, ndims, group_dims, data_type);
}

dnnl_status_t dnnl_primitive_attr_set_rounding(dnnl_primitive_attr_t attr, int arg, dnnl_rounding_mode_t mode) {
    if (!attr) return dnnl_invalid_arguments;
    if (mode != dnnl_rounding_mode_environment && mode != dnnl_rounding_mode_stochastic) return dnnl_invalid_arguments;
    attr->rounding[arg] = mode;
    return dnnl_success;
}
dnnl_status_t dnnl_primitive_attr_get_rounding(dnnl_primitive_attr_t attr, int arg, dnnl_rounding_mode_t *mode) {
    if (!attr || !mode) return dnnl_invalid_arguments;
    auto it = attr->rounding.find(arg);
    *mode = it == attr->rounding.end() ? dnnl_rounding_mode_environment : (dnnl_rounding_mode_t)it->second;
    return dnnl_success;
}

dnnl_status_t dnnl_primitive_attr_get_post_ops(const_dnnl_primitive_attr_t attr, const_dnnl_post_ops_t *post_ops) {
    if (!attr || !post_ops) return dnnl_invalid_arguments;
    *post_ops = &attr->post_ops;
    return dnnl_success;
}
dnnl_status_t dnnl_primitive_attr_set_post_ops(dnnl_primitive_attr_t attr, const_dnnl_post_ops_t post_ops) {
    if (!attr || !post_ops) return dnnl_invalid_arguments;
    attr->post_ops = *post_ops;
    return dnnl_success;
}

// ---- post-ops API --------------------------------------------------------------

static const int post_ops_limit = 32;

dnnl_status_t dnnl_post_ops_create(dnnl_post_ops_t *post_ops) {
    if (!post_ops) return dnnl_invalid_arguments;
    *post_ops = new dnnl_post_ops();
    return dnnl_success;
}
dnnl_status_t dnnl_post_ops_clone(dnnl_post_ops_t *post_ops, const_dnnl_post_ops_t existing) {
    if (!post_ops || !existing) return dnnl_invalid_arguments;
    *post_ops = new dnnl_post_ops(*existing);
    return dnnl_success;
}
dnnl_status_t dnnl_post_ops_destroy(dnnl_post_ops_t post_ops) {
    delete post_ops;
    return dnnl_success;
}
int dnnl_post_ops_len(const_dnnl_post_ops_t post_ops) {
    return post_ops ? (int)post_ops->entries.size() : 0;
}
dnnl_primitive_kind_t dnnl_post_ops_get_kind(const_dnnl_post_ops_t post_ops, int index) {
    if (!post_ops || index < 0 || index >= (int)post_ops->entries.size()) return dnnl_undefined_primitive;
    return (dnnl_primitive_kind_t)post_ops->entries[index].kind;
}

dnnl_status_t dnnl_post_ops_append_sum(dnnl_post_ops_t post_ops, float scale, int32_t zero_point,
        dnnl_data_type_t data_type) {
    if (!post_ops) return dnnl_invalid_arguments;
    if ((int)post_ops->entries.size() == post_ops_limit) return dnnl_out_of_memory;
    if (std::isnan(scale)) return dnnl_invalid_arguments;
    post_op_t e;
    e.kind = dnnl_sum;
    e.scale = scale;
    e.zero_point = zero_point;
    e.dt = data_type;
    post_ops->entries.push_back(e);
    return dnnl_success;
}
dnnl_status_t dnnl_post_ops_get_params_sum(const_dnnl_post_ops_t post_ops, int index, float *scale,
        int32_t *zero_point, dnnl_data_type_t *data_type) {
    if (!post_ops || index < 0 || index >= (int)post_ops->entries.size()) return dnnl_invalid_arguments;
    const post_op_t &e = post_ops->entries[index];
    if (e.kind != dnnl_sum) return dnnl_invalid_arguments;
    if (scale) *scale = e.scale;
    if (zero_point) *zero_point = e.zero_point;
    if (data_type) *data_type = (dnnl_data_type_t)e.dt;
    return dnnl_success;
}

static bool eltwise_alg_ok(int alg, float alpha, float beta) {
    const bool known = (alg >= dnnl_eltwise_relu && alg <= dnnl_eltwise_hardswish)
            || (alg >= dnnl_eltwise_relu_use_dst_for_bwd && alg <= dnnl_eltwise_clip_v2_use_dst_for_bwd);
    if (!known) return false;
    // parameter rules of math::is_eltwise_ok (src/common/math_utils.hpp:420-460)
    if (alg == dnnl_eltwise_clip || alg == dnnl_eltwise_clip_v2 || alg == dnnl_eltwise_clip_v2_use_dst_for_bwd)
        return beta >= alpha;
    if (alg == dnnl_eltwise_relu_use_dst_for_bwd || alg == dnnl_eltwise_elu_use_dst_for_bwd) return alpha >= 0;
    if (alg == dnnl_eltwise_soft_relu) return alpha != 0.f;
    return true;
}

dnnl_status_t dnnl_post_ops_append_eltwise(dnnl_post_ops_t post_ops, dnnl_alg_kind_t alg_kind, float alpha, float beta) {
    if (!post_ops) return dnnl_invalid_arguments;
    if ((int)post_ops->entries.size() == post_ops_limit) return dnnl_out_of_memory;
    if (!eltwise_alg_ok(alg_kind, alpha, beta) || std::isnan(alpha) || std::isnan(beta)) return dnnl_invalid_arguments;
    post_op_t e;
    e.kind = dnnl_eltwise;
    e.alg = alg_kind;
    e.alpha = alpha;
    e.beta = beta;
    e.scale = 1.f;
    post_ops->entries.push_back(e);
    return dnnl_success;
}
dnnl_status_t dnnl_post_ops_get_params_eltwise(const_dnnl_post_ops_t post_ops, int index, dnnl_alg_kind_t *alg_kind,
        float *alpha, float *beta) {
    if (!post_ops || index < 0 || index >= (int)post_ops->entries.size()) return dnnl_invalid_arguments;
    const post_op_t &e = post_ops->entries[index];
    if (e.kind != dnnl_eltwise) return dnnl_invalid_arguments;
    if (alg_kind) *alg_kind = (dnnl_alg_kind_t)e.alg;
    if (alpha) *alpha = e.alpha;
    if (beta) *beta = e.beta;
    return dnnl_success;
}

dnnl_status_t dnnl_post_ops_append_binary(dnnl_post_ops_t post_ops, dnnl_alg_kind_t alg_kind,
        const_dnnl_memory_desc_t src1_desc) {
    if (!post_ops || !src1_desc) return dnnl_invalid_arguments;
    if ((int)post_ops->entries.size() == post_ops_limit) return dnnl_out_of_memory;
    if (alg_kind < dnnl_binary_add || alg_kind > dnnl_binary_ne) return dnnl_invalid_arguments;
    if (src1_desc->ndims == 0 || src1_desc->has_runtime_dims()) return dnnl_invalid_arguments;
    post_op_t e;
    e.kind = dnnl_binary;
    e.alg = alg_kind;
    e.src1 = *src1_desc;
    post_ops->entries.push_back(e);
    return dnnl_success;
}
dnnl_status_t dnnl_post_ops_get_params_binary(const_dnnl_post_ops_t post_ops, int index, dnnl_alg_kind_t *alg_kind,
        const_dnnl_memory_desc_t *src1_desc) {
    if (!post_ops || index < 0 || index >= (int)post_ops->entries.size()) return dnnl_invalid_arguments;
    const post_op_t &e = post_ops->entries[index];
    if (e.kind != dnnl_binary) return dnnl_invalid_arguments;
    if (alg_kind) *alg_kind = (dnnl_alg_kind_t)e.alg;
    if (src1_desc) *src1_desc = &e.src1;
    return dnnl_success;
}

dnnl_status_t dnnl_post_ops_append_prelu(dnnl_post_ops_t post_ops, int mask) {
    if (!post_ops) return dnnl_invalid_arguments;
    if ((int)post_ops->entries.size() == post_ops_limit) return dnnl_out_of_memory;
    post_op_t e;
    e.kind = dnnl_prelu;
    e.mask = mask;
    post_ops->entries.push_back(e);
    return dnnl_success;
}
dnnl_status_t dnnl_post_ops_get_params_prelu(const_dnnl_post_ops_t post_ops, int index, int *mask) {
    if (!post_ops || index < 0 || index >= (int)post_ops->entries.size()) return dnnl_invalid_arguments;
    const post_op_t &e = post_ops->entries[index];
    if (e.kind != dnnl_prelu) return dnnl_invalid_arguments;
    if (mask) *mask = e.mask;
    return dnnl_success;
}

// ---- process-wide defaults ---------------------------------------------------

dnnl_status_t dnnl_get_default_fpmath_mode(dnnl_fpmath_mode_t *mode) {
    if (!mode) return dnnl_invalid_arguments;
    *mode = default_fpmath();
    return dnnl_success;
}
dnnl_status_t dnnl_set_default_fpmath_mode(dnnl_fpmath_mode_t mode) {
    if (!fpmath_ok(mode)) return dnnl_invalid_arguments;
    (void)default_fpmath();
    std::lock_guard<std::mutex> g(g_fpmath_mu);
    g_default_fpmath = mode;
    return dnnl_success;
}
