// The host side of the library: a dnnl_cpu engine that owns plain host memory and reorders.
//
// It exists for the callers either side of the matmul, not as a compute fallback: programs such
// as the reference's own test driver keep their reference tensors in f32 on a CPU engine, fill
// the tensors under test through reorders from that engine (f32 -> any data type, any plain
// layout or this engine's packed weights) and read results back the same way
// (tests/benchdnn/dnnl_memory.cpp:103-179, dnnl_common.hpp:132).  So this engine offers
//   * memory objects over malloc'ed (or user) host memory; map / unmap are the pointer itself;
//   * reorders host -> host, host -> CUDA engine and CUDA engine -> host between plain strided
//     tensors of any supported data type, element by element with the conversions of the
//     reference's generic reorder (src/cpu/reorder/simple_reorder.hpp:2551-2635 without
//     attributes: integers saturate and round to nearest even, floats convert with one
//     rounding), and host -> packed weights of the CUDA engine (converted to the plain layout of
//     the target type on the host, copied, then packed by the device kernel);
//   * no matmul: dnnl_matmul_primitive_desc_create on it returns dnnl_unimplemented.
// Copies to and from the device are synchronous; this is a fill / read-back path, not a hot one.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdlib>
#include <vector>

#include "internal.hpp"

namespace b200 {

// ---- element conversions on the host ----------------------------------------------------

static inline float host_bf16_to_f32(uint16_t b) {
    uint32_t u = (uint32_t)b << 16;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}
// round to nearest even; denormal results flush to signed zero as the reference's conversion
// does (src/common/bfloat16.cpp:22-51)
static inline uint16_t host_f32_to_bf16(float v) {
    uint32_t u;
    std::memcpy(&u, &v, 4);
    const uint32_t e = (u >> 23) & 0xff;
    if (e == 0) return (uint16_t)((u >> 16) & 0x8000);
    if (e == 0xff) return (uint16_t)((u & 0x7fffff) ? ((u >> 16) | 0x40) : (u >> 16));
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

// the value of element `idx` (an element offset: 4-bit types hold two per byte, even in the low nibble)
static float host_load(int dt, const void *p, int64_t idx) {
    switch (dt) {
        case dnnl_f32: return ((const float *)p)[idx];
        case dnnl_s32: return (float)((const int32_t *)p)[idx];
        case dnnl_s8: return (float)((const int8_t *)p)[idx];
        case dnnl_u8: return (float)((const uint8_t *)p)[idx];
        case dnnl_bf16: return host_bf16_to_f32(((const uint16_t *)p)[idx]);
        case dnnl_f16: return __half2float(((const __half *)p)[idx]);
        case dnnl_f8_e4m3: {
            const __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)((const uint8_t *)p)[idx], __NV_E4M3);
            return __half2float(__half(h));
        }
        case dnnl_f8_e5m2: {
            const __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)((const uint8_t *)p)[idx], __NV_E5M2);
            return __half2float(__half(h));
        }
        case dnnl_s4: {
            const int v = (((const uint8_t *)p)[idx >> 1] >> ((idx & 1) * 4)) & 0xf;
            return (float)((v & 8) ? v - 16 : v);
        }
        case dnnl_u4: return (float)((((const uint8_t *)p)[idx >> 1] >> ((idx & 1) * 4)) & 0xf);
        default: return NAN;
    }
}

static inline float sat_round(float v, float lo, float hi) {
    if (v != v) return 0.f; // the reference's conversion of NaN ends in 0 for 8-bit types
    v = v < lo ? lo : v;
    v = v > hi ? hi : v;
    return std::nearbyintf(v);
}

static void host_store(int dt, void *p, int64_t idx, float v) {
    switch (dt) {
        case dnnl_f32: ((float *)p)[idx] = v; break;
        case dnnl_s32:
            ((int32_t *)p)[idx] = v != v ? (int32_t)0x80000000 : (int32_t)sat_round(v, -2147483648.f, 2147483520.f);
            break;
        case dnnl_s8: ((int8_t *)p)[idx] = (int8_t)sat_round(v, -128.f, 127.f); break;
        case dnnl_u8: ((uint8_t *)p)[idx] = (uint8_t)sat_round(v, 0.f, 255.f); break;
        case dnnl_bf16: ((uint16_t *)p)[idx] = host_f32_to_bf16(v); break;
        case dnnl_f16: ((__half *)p)[idx] = __float2half_rn(v); break;
        case dnnl_f8_e4m3: // through f16, as src/common/float8.cpp:96-147
            ((uint8_t *)p)[idx] = (uint8_t)__nv_cvt_halfraw_to_fp8(__half_raw(__float2half_rn(v)), __NV_NOSAT, __NV_E4M3);
            break;
        case dnnl_f8_e5m2:
            ((uint8_t *)p)[idx] = (uint8_t)__nv_cvt_halfraw_to_fp8(__half_raw(__float2half_rn(v)), __NV_NOSAT, __NV_E5M2);
            break;
        case dnnl_s4:
        case dnnl_u4: {
            const int q = dt == dnnl_s4 ? (int)sat_round(v, -8.f, 7.f) : (int)sat_round(v, 0.f, 15.f);
            uint8_t &b = ((uint8_t *)p)[idx >> 1];
            const int sh = (int)(idx & 1) * 4;
            b = (uint8_t)((b & ~(0xf << sh)) | ((q & 0xf) << sh));
            break;
        }
        default: break;
    }
}

static bool host_dt_ok(int dt) {
    switch (dt) {
        case dnnl_f32: case dnnl_s32: case dnnl_s8: case dnnl_u8: case dnnl_bf16: case dnnl_f16: case dnnl_f8_e4m3:
        case dnnl_f8_e5m2: case dnnl_s4: case dnnl_u4: return true;
        default: return false;
    }
}

// dst[i] = convert(src[i]) over all logical indices; both descriptors plain, same dims.
// Raw pointers are the starts of the buffers (offset0 is applied here).
void host_reorder_plain(const dnnl_memory_desc &s, const void *src, const dnnl_memory_desc &d, void *dst) {
    const int nd = s.ndims;
    const int64_t total = s.nelems();
    if (nd == 0 || total == 0) return;
    // same type and both dense in the same order: one copy
    if (s.data_type == d.data_type && s.equal(d) && s.is_dense_row_major() && s.offset0 == 0
            && (dt_nbits(s.data_type) >= 8 || total % 2 == 0)) {
        std::memcpy(dst, src, (size_t)(total * dt_nbits(s.data_type) / 8));
        return;
    }
    int64_t idx[DNNL_MAX_NDIMS] = {0};
    int64_t so = s.offset0, dof = d.offset0;
    for (int64_t i = 0; i < total; ++i) {
        host_store(d.data_type, dst, dof, host_load(s.data_type, src, so));
        // odometer over the logical dims, innermost last
        for (int k = nd - 1; k >= 0; --k) {
            ++idx[k];
            so += s.strides[k];
            dof += d.strides[k];
            if (idx[k] < s.dims[k]) break;
            so -= idx[k] * s.strides[k];
            dof -= idx[k] * d.strides[k];
            idx[k] = 0;
        }
    }
}

static const char *md_base(const dnnl_memory *m) { return (const char *)m->handle; }

// ---- reorders that involve the host engine ----------------------------------------------

dnnl_status_t host_reorder_pd_create(dnnl_primitive_desc_t *out, const dnnl_memory_desc &s, dnnl_engine *se,
        const dnnl_memory_desc &d, dnnl_engine *de, const dnnl_primitive_attr *attr) {
    if (attr && (!attr->scales.empty() || !attr->zero_points.empty() || !attr->post_ops.entries.empty()))
        return dnnl_unimplemented; // quantising reorders belong to the CUDA engine
    if (!s.is_plain()) return dnnl_unimplemented; // packed weights are never read back
    if (!host_dt_ok(s.data_type) || !host_dt_ok(d.data_type)) return dnnl_unimplemented;
    if (d.format_kind == dnnl_format_kind_opaque) {
        if (de->host || s.ndims != 2) return dnnl_unimplemented;
        if (dt_nbits(d.data_type) == 4 && s.dims[1] % 2 != 0) return dnnl_unimplemented;
    } else if (!d.is_plain()) {
        return dnnl_unimplemented;
    }
    auto pd = std::unique_ptr<dnnl_primitive_desc>(new dnnl_primitive_desc());
    pd->kind = dnnl_reorder;
    // the CUDA engine when one is involved: its stream orders the copies
    pd->engine = !de->host ? de : (!se->host ? se : de);
    if (attr) pd->attr = *attr;
    pd->user_src = pd->src = s;
    pd->user_dst = pd->dst = d;
    pd->impl = IMPL_REORDER;
    pd->impl_str = se->host && de->host ? "host:reorder" : (se->host ? "host:convert+copy_in" : "host:copy_out+convert");
    pd->engine->refs.fetch_add(1);
    *out = pd.release();
    return dnnl_success;
}

dnnl_status_t host_reorder_execute(const dnnl_primitive *prim, dnnl_stream *stream, const dnnl_memory *from,
        const dnnl_memory *to) {
    const dnnl_primitive_desc *pd = prim->pd.get();
    const dnnl_memory_desc &s = pd->src, &d = pd->dst;
    if (s.has_zero_dim()) return dnnl_success;
    if (!from->handle || !to->handle) return dnnl_invalid_arguments;
    const bool sh = from->engine->host, dh = to->engine->host;
    if (sh && dh) {
        host_reorder_plain(s, md_base(from), d, (void *)md_base(to));
        return dnnl_success;
    }
    dnnl_engine *gpu = sh ? to->engine : from->engine;
    if (set_device(gpu) != dnnl_success) return dnnl_runtime_error;
    if (cudaDeviceSynchronize() != cudaSuccess) return dnnl_runtime_error; // whatever wrote either buffer has finished
    if (!sh) {
        // device -> host: the raw bytes of the plain source, then the conversion
        const size_t bytes = s.size_bytes();
        std::vector<unsigned char> raw(bytes + 16);
        if (cudaMemcpy(raw.data(), md_base(from), bytes, cudaMemcpyDeviceToHost) != cudaSuccess) return dnnl_runtime_error;
        host_reorder_plain(s, raw.data(), d, (void *)md_base(to));
        return dnnl_success;
    }
    if (d.is_plain()) {
        // host -> device, plain: convert into a host image of the destination (what lies between
        // the elements of a strided destination is kept), then one copy
        const size_t bytes = d.size_bytes();
        std::vector<unsigned char> img(bytes + 16);
        if (!d.is_dense_row_major() || d.offset0 != 0 || dt_nbits(d.data_type) == 4) {
            if (cudaMemcpy(img.data(), md_base(to), bytes, cudaMemcpyDeviceToHost) != cudaSuccess) return dnnl_runtime_error;
        }
        host_reorder_plain(s, md_base(from), d, img.data());
        return cudaMemcpy((void *)md_base(to), img.data(), bytes, cudaMemcpyHostToDevice) == cudaSuccess ? dnnl_success
                                                                                                         : dnnl_runtime_error;
    }
    // host -> packed weights: the plain (K, N) image of the target type on the host, a temporary
    // device copy of it, and the device kernel that packs
    dnnl_memory_desc plain;
    plain.ndims = 2;
    plain.data_type = d.data_type;
    plain.format_kind = dnnl_blocked;
    plain.dims[0] = d.dims[0];
    plain.dims[1] = d.dims[1];
    plain.strides[0] = d.dims[1];
    plain.strides[1] = 1;
    const size_t bytes = plain.size_bytes();
    std::vector<unsigned char> img(bytes + 16, 0);
    host_reorder_plain(s, md_base(from), plain, img.data());
    void *tmp = nullptr;
    if (device_alloc(&tmp, bytes ? bytes : 1) != cudaSuccess) return dnnl_out_of_memory;
    dnnl_status_t st = dnnl_runtime_error;
    if (cudaMemcpy(tmp, img.data(), bytes, cudaMemcpyHostToDevice) == cudaSuccess) {
        dnnl_primitive_desc_t rpd = nullptr;
        st = dnnl_reorder_primitive_desc_create(&rpd, &plain, gpu, &d, gpu, nullptr);
        if (st == dnnl_success) {
            dnnl_primitive inner;
            inner.pd = std::shared_ptr<dnnl_primitive_desc>(rpd, [](dnnl_primitive_desc *p) { dnnl_primitive_desc_destroy(p); });
            dnnl_memory src_mem;
            src_mem.md = plain;
            src_mem.engine = gpu;
            src_mem.handle = tmp;
            std::map<int, dnnl_memory *> args;
            args[DNNL_ARG_FROM] = &src_mem;
            args[DNNL_ARG_TO] = const_cast<dnnl_memory *>(to);
            // on the caller's stream when it belongs to the CUDA engine, else on the default stream
            dnnl_stream local;
            local.engine = gpu;
            dnnl_stream *use = (stream && !stream->engine->host) ? stream : &local;
            st = reorder_execute(&inner, use, args);
            if (cudaDeviceSynchronize() != cudaSuccess) st = dnnl_runtime_error;
        }
    }
    cudaFree(tmp);
    return st;
}

} // namespace b200
