// Entry points of the reference's C API that a matmul program's surroundings touch but this
// engine does not implement, so that such programs link: each returns the status the reference
// itself returns for a feature that was not built (dnnl_unimplemented).  Plus the two hidden
// entry points the reference's test driver declares for itself
// (tests/benchdnn/dnnl_memory.cpp:44-50): dnnl_memory_desc_create_with_string_tag and
// dnnl_memory_desc_set_data_type, and the descriptor blob pair
// (include/oneapi/dnnl/dnnl.h, dnnl_memory_desc_get_blob / _create_with_blob).
#include <cctype>
#include <cstring>

#include "internal.hpp"

extern "C" {

DNNL_API dnnl_status_t dnnl_sgemm(char, char, int64_t, int64_t, int64_t, float, const float *, int64_t, const float *, int64_t,
        float, float *, int64_t) {
    return dnnl_unimplemented; // no CPU compute in this library
}

DNNL_API dnnl_status_t dnnl_set_cpu_isa_hints(int) { return dnnl_unimplemented; }

DNNL_API dnnl_status_t dnnl_primitive_get_cache_blob(const_dnnl_primitive_t, size_t *, uint8_t *) { return dnnl_unimplemented; }
DNNL_API dnnl_status_t dnnl_primitive_create_from_cache_blob(dnnl_primitive_t *, const_dnnl_primitive_desc_t, size_t,
        const uint8_t *) {
    return dnnl_unimplemented;
}

DNNL_API dnnl_status_t dnnl_primitive_attr_set_dropout(dnnl_primitive_attr_t, const_dnnl_memory_desc_t) { return dnnl_unimplemented; }
DNNL_API dnnl_status_t dnnl_post_ops_append_dw(dnnl_post_ops_t, dnnl_data_type_t, dnnl_data_type_t, dnnl_data_type_t, int64_t,
        int64_t, int64_t) {
    return dnnl_unimplemented;
}

// other primitive kinds: the descriptor constructors exist, nothing implements them
DNNL_API dnnl_status_t dnnl_eltwise_forward_primitive_desc_create(dnnl_primitive_desc_t *, dnnl_engine_t, dnnl_prop_kind_t,
        dnnl_alg_kind_t, const_dnnl_memory_desc_t, const_dnnl_memory_desc_t, float, float, const_dnnl_primitive_attr_t) {
    return dnnl_unimplemented;
}
DNNL_API dnnl_status_t dnnl_eltwise_backward_primitive_desc_create(dnnl_primitive_desc_t *, dnnl_engine_t, dnnl_alg_kind_t,
        const_dnnl_memory_desc_t, const_dnnl_memory_desc_t, const_dnnl_memory_desc_t, float, float,
        const_dnnl_primitive_desc_t, const_dnnl_primitive_attr_t) {
    return dnnl_unimplemented;
}

// A memory descriptor as an opaque byte string and back (same process, same library build).
DNNL_API dnnl_status_t dnnl_memory_desc_get_blob(uint8_t *blob, size_t *size, const_dnnl_memory_desc_t md) {
    if (!size || !md) return dnnl_invalid_arguments;
    if (blob) std::memcpy(blob, md, sizeof(dnnl_memory_desc));
    *size = sizeof(dnnl_memory_desc);
    return dnnl_success;
}
DNNL_API dnnl_status_t dnnl_memory_desc_create_with_blob(dnnl_memory_desc_t *md, const uint8_t *blob) {
    if (!md || !blob) return dnnl_invalid_arguments;
    dnnl_memory_desc *out = new dnnl_memory_desc();
    std::memcpy((void *)out, blob, sizeof(dnnl_memory_desc));
    *md = out;
    return dnnl_success;
}

// The element type of a descriptor replaced in place; strides count elements and stay.
DNNL_API dnnl_status_t dnnl_memory_desc_set_data_type(dnnl_memory_desc_t md, dnnl_data_type_t dt) {
    if (!md || !b200::dt_known(dt)) return dnnl_invalid_arguments;
    md->data_type = dt;
    return dnnl_success;
}

// Plain layouts named by a permutation string ("ab", "acb", "ba" ...): letter i is logical dim
// i, the string lists the dims from outermost to innermost.  "any" and "undef" as in
// dnnl_memory_desc_create_with_tag.  Blocked tags (capital letters, digits) belong to other
// engines: dnnl_unimplemented.
DNNL_API dnnl_status_t dnnl_memory_desc_create_with_string_tag(dnnl_memory_desc_t *md, int ndims, const dnnl_dims_t dims,
        dnnl_data_type_t dt, const char *tag) {
    if (!md || !tag) return dnnl_invalid_arguments;
    if (std::strcmp(tag, "any") == 0) return dnnl_memory_desc_create_with_tag(md, ndims, dims, dt, dnnl_format_tag_any);
    if (std::strcmp(tag, "undef") == 0) return dnnl_memory_desc_create_with_tag(md, ndims, dims, dt, dnnl_format_tag_undef);
    const int len = (int)std::strlen(tag);
    if (ndims <= 0 || ndims > DNNL_MAX_NDIMS) return dnnl_invalid_arguments;
    bool seen[DNNL_MAX_NDIMS] = {false};
    bool foreign = false;
    for (int i = 0; i < len; ++i) foreign |= !std::islower((unsigned char)tag[i]);
    if (foreign) {
        // a blocked layout of another engine: a descriptor that records only that (every dim padded
        // to a multiple of 64 bounds its size from above); no implementation here accepts it
        for (int i = 0; i < ndims; ++i)
            if (dims[i] < 0) return dnnl_invalid_arguments;
        if (!b200::dt_known(dt)) return dnnl_invalid_arguments;
        dnnl_memory_desc *out = new dnnl_memory_desc();
        out->ndims = ndims;
        out->data_type = dt;
        out->format_kind = dnnl_format_kind_opaque;
        out->packed_layout = B200_LAYOUT_FOREIGN;
        for (int i = 0; i < ndims; ++i) out->dims[i] = dims[i];
        *md = out;
        return dnnl_success;
    }
    for (int i = 0; i < len; ++i) {
        const int d = tag[i] - 'a';
        if (d < 0 || d >= ndims || seen[d]) return dnnl_invalid_arguments;
        seen[d] = true;
    }
    if (len != ndims) return dnnl_invalid_arguments;
    dnnl_dims_t strides;
    int64_t s = 1;
    bool rt = false; // strides that depend on a runtime dim are runtime values themselves
    for (int j = ndims - 1; j >= 0; --j) {
        const int d = tag[j] - 'a';
        strides[d] = rt ? DNNL_RUNTIME_DIM_VAL : s;
        if (dims[d] == DNNL_RUNTIME_DIM_VAL) rt = true;
        else s *= dims[d] > 0 ? dims[d] : 1;
    }
    return dnnl_memory_desc_create_with_strides(md, ndims, dims, dt, strides);
}

// Device memory of a CUDA engine: total bytes and the largest single allocation the driver would
// grant now (what a test driver sizes its problems against; the reference's driver asks its
// OpenCL / SYCL runtime the same, tests/benchdnn/dnnl_common.cpp:1003-1036).
DNNL_API dnnl_status_t dnnl_b200_engine_get_memory_info(dnnl_engine_t engine, size_t *total_bytes, size_t *max_alloc_bytes,
        size_t *l2_bytes) {
    if (!engine || engine->host || !engine->usable()) return dnnl_invalid_arguments;
    if (b200::set_device(engine) != dnnl_success) return dnnl_runtime_error;
    size_t free_b = 0, total_b = 0;
    if (cudaMemGetInfo(&free_b, &total_b) != cudaSuccess) return dnnl_runtime_error;
    int l2 = 0;
    cudaDeviceGetAttribute(&l2, cudaDevAttrL2CacheSize, engine->device);
    if (total_bytes) *total_bytes = total_b;
    if (max_alloc_bytes) *max_alloc_bytes = free_b;
    if (l2_bytes) *l2_bytes = (size_t)l2;
    return dnnl_success;
}

} // extern "C"
