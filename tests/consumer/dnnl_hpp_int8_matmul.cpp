// A user program written against the reference library's own C++ header (dnnl.hpp), linked
// against libonednn_b200.so instead of libdnnl.so: int8 matmul with per-tensor source scale and
// zero-point, per-column weights scales, bias, relu and a destination scale into u8, weights
// reordered into the layout the implementation asks for (format_tag::any) -- the flow of the
// reference's examples/tutorials/matmul/inference_int8_matmul.cpp, with data moved through
// map_data / unmap_data because the engine is neither SYCL nor OpenCL.
//
// Prints one line: "OK <impl> max_abs_diff=<d>" and exits 0, or a message and a non-zero code.
// TEST INFRASTRUCTURE: built by oracle/build_ref.py where the reference headers are present.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <random>
#include <unordered_map>
#include <vector>

#include "oneapi/dnnl/dnnl.hpp"

using namespace dnnl;

template <typename T>
static void write_mem(memory &m, const std::vector<T> &v) {
    void *p = m.map_data();
    std::memcpy(p, v.data(), v.size() * sizeof(T));
    m.unmap_data(p);
}
template <typename T>
static std::vector<T> read_mem(memory &m, size_t n) {
    std::vector<T> v(n);
    void *p = m.map_data();
    std::memcpy(v.data(), p, n * sizeof(T));
    m.unmap_data(p);
    return v;
}

int main() {
    try {
        const memory::dim M = 96, K = 128, N = 80;
        engine eng(engine::kind::gpu, 0);
        stream strm(eng);

        std::mt19937 rng(7);
        std::vector<uint8_t> src(M * K);
        std::vector<int8_t> wei(K * N);
        std::vector<float> bias(N), wscale(N), sscale {0.02f}, dscale {0.5f};
        std::vector<int32_t> szp {120}, dzp {10};
        for (auto &x : src) x = (uint8_t)(rng() % 256);
        for (auto &x : wei) x = (int8_t)((int)(rng() % 255) - 127);
        for (auto &x : bias) x = (float)((int)(rng() % 2001) - 1000) / 500.f;
        for (auto &x : wscale) x = 0.001f + (float)(rng() % 1000) * 3e-6f;

        memory::desc src_md({M, K}, memory::data_type::u8, memory::format_tag::ab);
        memory::desc wei_plain_md({K, N}, memory::data_type::s8, memory::format_tag::ab);
        memory::desc wei_any_md({K, N}, memory::data_type::s8, memory::format_tag::any);
        memory::desc bias_md({1, N}, memory::data_type::f32, memory::format_tag::ab);
        memory::desc dst_md({M, N}, memory::data_type::u8, memory::format_tag::ab);

        primitive_attr attr;
        attr.set_scales_mask(DNNL_ARG_SRC, 0);
        attr.set_scales_mask(DNNL_ARG_WEIGHTS, 1 << 1);
        attr.set_scales_mask(DNNL_ARG_DST, 0);
        attr.set_zero_points_mask(DNNL_ARG_SRC, 0);
        attr.set_zero_points_mask(DNNL_ARG_DST, 0);
        post_ops po;
        po.append_eltwise(algorithm::eltwise_relu, 0.f, 0.f);
        attr.set_post_ops(po);

        matmul::primitive_desc pd(eng, src_md, wei_any_md, bias_md, dst_md, attr);
        matmul prim(pd);

        memory src_m(src_md, eng), wei_plain_m(wei_plain_md, eng), bias_m(bias_md, eng), dst_m(dst_md, eng);
        write_mem(src_m, src);
        write_mem(wei_plain_m, wei);
        write_mem(bias_m, bias);
        memory wei_m = wei_plain_m;
        if (pd.weights_desc() != wei_plain_md) {
            wei_m = memory(pd.weights_desc(), eng);
            reorder(wei_plain_m, wei_m).execute(strm, wei_plain_m, wei_m);
        }
        memory sscale_m({{1}, memory::data_type::f32, memory::format_tag::a}, eng);
        memory wscale_m({{N}, memory::data_type::f32, memory::format_tag::a}, eng);
        memory dscale_m({{1}, memory::data_type::f32, memory::format_tag::a}, eng);
        memory szp_m({{1}, memory::data_type::s32, memory::format_tag::a}, eng);
        memory dzp_m({{1}, memory::data_type::s32, memory::format_tag::a}, eng);
        write_mem(sscale_m, sscale);
        write_mem(wscale_m, wscale);
        write_mem(dscale_m, dscale);
        write_mem(szp_m, szp);
        write_mem(dzp_m, dzp);

        prim.execute(strm,
                {{DNNL_ARG_SRC, src_m}, {DNNL_ARG_WEIGHTS, wei_m}, {DNNL_ARG_BIAS, bias_m}, {DNNL_ARG_DST, dst_m},
                        {DNNL_ARG_ATTR_SCALES | DNNL_ARG_SRC, sscale_m}, {DNNL_ARG_ATTR_SCALES | DNNL_ARG_WEIGHTS, wscale_m},
                        {DNNL_ARG_ATTR_SCALES | DNNL_ARG_DST, dscale_m}, {DNNL_ARG_ATTR_ZERO_POINTS | DNNL_ARG_SRC, szp_m},
                        {DNNL_ARG_ATTR_ZERO_POINTS | DNNL_ARG_DST, dzp_m}});
        strm.wait();
        std::vector<uint8_t> got = read_mem<uint8_t>(dst_m, (size_t)(M * N));

        // the library's documented formula on the host
        int max_diff = 0;
        for (memory::dim m = 0; m < M; ++m)
            for (memory::dim n = 0; n < N; ++n) {
                int32_t acc = 0;
                for (memory::dim k = 0; k < K; ++k) acc += ((int)src[m * K + k] - szp[0]) * (int)wei[k * N + n];
                float d = (float)acc * sscale[0] * wscale[n] + bias[n];
                d = d > 0.f ? d : 0.f;
                d = d * (1.f / dscale[0]) + (float)dzp[0];
                d = std::min(255.f, std::max(0.f, d));
                const int want = (int)std::nearbyint(d);
                max_diff = std::max(max_diff, std::abs(want - (int)got[m * N + n]));
            }
        if (max_diff > 1) {
            std::printf("MISMATCH max_abs_diff=%d\n", max_diff);
            return 2;
        }
        std::printf("OK %s max_abs_diff=%d\n", pd.impl_info_str(), max_diff);
        return 0;
    } catch (const dnnl::error &e) {
        std::printf("dnnl::error status=%d: %s\n", (int)e.status, e.what());
        return 3;
    }
}
