// A user program written against the reference library's own C++ header (dnnl.hpp), linked
// against libonednn_b200.so: weights decompression as in the reference's
// examples/tutorials/matmul/weights_decompression_matmul.cpp -- C = A * ((B_u4 - zp) * scale)
// with bf16 activations, u4 weights given as format_tag::any and reordered once, bf16 scales
// and u4 zero-points per group of 128 along K, fpmath mode bf16 applied to integer weights --
// for one activation row (the decode GEMV) and for 64 rows (the tensor-core path).
//
// Prints "OK <impl for 1 row> <impl for 64 rows>" and exits 0, or a message and a non-zero code.
// TEST INFRASTRUCTURE: built by oracle/build_ref.py where the reference headers are present.
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <random>
#include <string>
#include <vector>

#include "oneapi/dnnl/dnnl.hpp"

using namespace dnnl;

static uint16_t to_bf16(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
static float from_bf16(uint16_t h) {
    uint32_t u = (uint32_t)h << 16;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}
template <typename T>
static void write_mem(memory &m, const std::vector<T> &v) {
    void *p = m.map_data();
    std::memcpy(p, v.data(), v.size() * sizeof(T));
    m.unmap_data(p);
}

int main() {
    try {
        const memory::dim K = 512, N = 256, G = 128, NG = K / G;
        engine eng(engine::kind::gpu, 0);
        stream strm(eng);
        std::mt19937 rng(11);
        std::vector<uint8_t> wq(K * N), wpacked(K * N / 2), zq(NG * N), zpacked(NG * N / 2);
        std::vector<uint16_t> scale(NG * N);
        for (auto &x : wq) x = (uint8_t)(rng() % 16);
        for (auto &x : zq) x = (uint8_t)(rng() % 16);
        for (memory::dim i = 0; i < K * N / 2; ++i) wpacked[i] = (uint8_t)(wq[2 * i] | (wq[2 * i + 1] << 4));
        for (memory::dim i = 0; i < NG * N / 2; ++i) zpacked[i] = (uint8_t)(zq[2 * i] | (zq[2 * i + 1] << 4));
        for (auto &x : scale) x = to_bf16(0.01f + (float)(rng() % 100) * 1e-4f);

        memory::desc wei_plain_md({K, N}, memory::data_type::u4, memory::format_tag::ab);
        memory wei_plain(wei_plain_md, eng);
        write_mem(wei_plain, wpacked);
        memory sc_m({{NG * N}, memory::data_type::bf16, memory::format_tag::a}, eng);
        memory zp_m({{NG * N}, memory::data_type::u4, memory::format_tag::a}, eng);
        write_mem(sc_m, scale);
        write_mem(zp_m, zpacked);

        primitive_attr attr;
        attr.set_scales(DNNL_ARG_WEIGHTS, (1 << 0) + (1 << 1), {G, 1}, memory::data_type::bf16);
        attr.set_zero_points(DNNL_ARG_WEIGHTS, (1 << 0) + (1 << 1), {G, 1}, memory::data_type::u4);
        attr.set_fpmath_mode(fpmath_mode::bf16, true);

        std::string impls;
        for (memory::dim M : {1, 64}) {
            std::vector<uint16_t> a(M * K);
            for (auto &x : a) x = to_bf16((float)((int)(rng() % 2001) - 1000) / 1000.f);
            memory::desc a_md({M, K}, memory::data_type::bf16, memory::format_tag::ab);
            memory::desc b_md({K, N}, memory::data_type::u4, memory::format_tag::any);
            memory::desc c_md({M, N}, memory::data_type::bf16, memory::format_tag::ab);
            matmul::primitive_desc pd(eng, a_md, b_md, c_md, attr);
            memory a_m(a_md, eng), c_m(c_md, eng);
            write_mem(a_m, a);
            memory wei = wei_plain;
            if (pd.weights_desc() != wei_plain_md) {
                wei = memory(pd.weights_desc(), eng);
                reorder(wei_plain, wei).execute(strm, wei_plain, wei);
            }
            matmul(pd).execute(strm,
                    {{DNNL_ARG_SRC, a_m}, {DNNL_ARG_WEIGHTS, wei}, {DNNL_ARG_DST, c_m},
                            {DNNL_ARG_ATTR_SCALES | DNNL_ARG_WEIGHTS, sc_m}, {DNNL_ARG_ATTR_ZERO_POINTS | DNNL_ARG_WEIGHTS, zp_m}});
            strm.wait();
            std::vector<uint16_t> got(M * N);
            void *p = c_m.map_data();
            std::memcpy(got.data(), p, got.size() * 2);
            c_m.unmap_data(p);
            double max_err = 0, max_ref = 0;
            for (memory::dim m = 0; m < M; ++m)
                for (memory::dim n = 0; n < N; ++n) {
                    double acc = 0;
                    for (memory::dim k = 0; k < K; ++k) {
                        const memory::dim g = k / G;
                        acc += (double)from_bf16(a[m * K + k]) * ((double)wq[k * N + n] - (double)zq[g * N + n])
                                * (double)from_bf16(scale[g * N + n]);
                    }
                    max_err = std::fmax(max_err, std::fabs(acc - (double)from_bf16(got[m * N + n])));
                    max_ref = std::fmax(max_ref, std::fabs(acc));
                }
            if (max_err > 0.02 * max_ref) {
                std::printf("MISMATCH M=%d max_err=%g max_ref=%g\n", (int)M, max_err, max_ref);
                return 2;
            }
            impls += std::string(" ") + pd.impl_info_str();
        }
        std::printf("OK%s\n", impls.c_str());
        return 0;
    } catch (const dnnl::error &e) {
        std::printf("dnnl::error status=%d: %s\n", (int)e.status, e.what());
        return 3;
    }
}
