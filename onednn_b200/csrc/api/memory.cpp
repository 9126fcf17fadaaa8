// Memory descriptors and memory objects.  Replaces the reference's
// src/common/memory_desc.cpp (create_with_tag / strides, submemory, reshape,
// permute, query, equal, size) and src/common/memory.cpp:139-307 (create, data
// handles, map / unmap) for the plain strided layouts and the packed weights
// layouts this engine uses.  Device buffers come from cudaMalloc; map_data
// stages through pinned host memory because device memory is not host
// addressable.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdio>

#include <cstdlib>

#include "internal.hpp"

using namespace b200;

namespace b200 {

const char *dt_name(int dt) {
    switch (dt) {
        case dnnl_f16: return "f16";
        case dnnl_bf16: return "bf16";
        case dnnl_f32: return "f32";
        case dnnl_s32: return "s32";
        case dnnl_s8: return "s8";
        case dnnl_u8: return "u8";
        case dnnl_f8_e5m2: return "f8_e5m2";
        case dnnl_f8_e4m3: return "f8_e4m3";
        case dnnl_s4: return "s4";
        case dnnl_u4: return "u4";
        default: return "undef";
    }
}

} // namespace b200

size_t dnnl_memory_desc::size_bytes() const {
    if (ndims == 0 || is_any() || has_runtime_dims()) return 0;
    if (has_zero_dim()) return 0;
    if (format_kind == dnnl_format_kind_opaque && packed_layout == B200_LAYOUT_FOREIGN) {
        int64_t n = 1; // an upper bound: every dim padded to a multiple of 64
        for (int i = 0; i < ndims; ++i) n *= (dims[i] + 63) / 64 * 64;
        return (size_t)((n * dt_nbits(data_type) + 7) / 8);
    }
    if (format_kind == dnnl_format_kind_opaque) {
        if (ndims <= 2) return b200_packed_weights_bytes(dims[ndims - 2], dims[ndims - 1], data_type, packed_layout);
        size_t batch = 1;
        for (int i = 0; i < ndims - 2; ++i) batch *= (size_t)dims[i];
        return batch * packed_slice_stride();
    }
    int64_t span = 1;
    for (int i = 0; i < ndims; ++i) span += (dims[i] - 1) * strides[i];
    const int bits = dt_nbits(data_type);
    return (size_t)((span * bits + 7) / 8);
}

size_t dnnl_memory_desc::packed_slice_stride() const {
    const size_t b = b200_packed_weights_bytes(dims[ndims - 2], dims[ndims - 1], data_type, packed_layout);
    return (b + 255) / 256 * 256;
}

bool dnnl_memory_desc::equal(const dnnl_memory_desc &o) const {
    if (ndims != o.ndims) return false;
    if (ndims == 0) return true;
    if (data_type != o.data_type || format_kind != o.format_kind || offset0 != o.offset0) return false;
    for (int i = 0; i < ndims; ++i)
        if (dims[i] != o.dims[i]) return false;
    if (format_kind == dnnl_blocked) {
        for (int i = 0; i < ndims; ++i)
            if (dims[i] != 1 && strides[i] != o.strides[i]) return false;
    }
    if (format_kind == dnnl_format_kind_opaque && packed_layout != o.packed_layout) return false;
    return true;
}

bool dnnl_memory_desc::is_dense_row_major() const {
    if (!is_plain()) return false;
    int64_t s = 1;
    for (int i = ndims - 1; i >= 0; --i) {
        if (dims[i] != 1 && strides[i] != s) return false;
        s *= dims[i];
    }
    return true;
}

std::string dnnl_memory_desc::layout_str() const {
    if (ndims == 0) return "undef";
    if (is_any()) return "any";
    if (format_kind == dnnl_format_kind_opaque)
        return packed_layout == B200_WEI_KMAJOR ? "packed:kmajor_colsum"
                : packed_layout == B200_WEI_WC4_TC ? "packed:wc4_tc"
                : packed_layout == B200_WEI_WC8_TC ? "packed:wc8_tc" : "packed:wc4_tiled";
    // order dims by decreasing stride and print them as letters
    std::vector<int> idx(ndims);
    for (int i = 0; i < ndims; ++i) idx[i] = i;
    std::stable_sort(idx.begin(), idx.end(), [&](int a, int b) { return strides[a] > strides[b]; });
    std::string s;
    for (int i : idx) s += (char)('a' + i);
    // dense?
    int64_t expect = 1;
    bool dense = true;
    for (int j = ndims - 1; j >= 0; --j) {
        if (dims[idx[j]] != 1 && strides[idx[j]] != expect) dense = false;
        expect *= dims[idx[j]];
    }
    if (!dense) s += ":strided";
    return s;
}

static dnnl_status_t check_dims(int ndims, const dnnl_dims_t dims, dnnl_data_type_t dt) {
    if (ndims < 0 || ndims > DNNL_MAX_NDIMS) return dnnl_invalid_arguments;
    if (ndims == 0) return dnnl_success;
    if (!dims) return dnnl_invalid_arguments;
    if (!dt_known(dt)) return dnnl_invalid_arguments;
    for (int i = 0; i < ndims; ++i)
        if (dims[i] < 0 && dims[i] != DNNL_RUNTIME_DIM_VAL) return dnnl_invalid_arguments;
    return dnnl_success;
}

dnnl_status_t dnnl_memory_desc_destroy(dnnl_memory_desc_t md) {
    delete md;
    return dnnl_success;
}

dnnl_status_t dnnl_memory_desc_clone(dnnl_memory_desc_t *md, const_dnnl_memory_desc_t existing) {
    if (!md || !existing) return dnnl_invalid_arguments;
    *md = new dnnl_memory_desc(*existing);
    return dnnl_success;
}

dnnl_status_t dnnl_memory_desc_create_with_strides(dnnl_memory_desc_t *memory_desc, int ndims, const dnnl_dims_t dims,
        dnnl_data_type_t data_type, const dnnl_dims_t strides) {
    if (!memory_desc) return dnnl_invalid_arguments;
    dnnl_status_t st = check_dims(ndims, dims, data_type);
    if (st != dnnl_success) return st;
    auto md = std::unique_ptr<dnnl_memory_desc>(new dnnl_memory_desc());
    if (ndims == 0) {
        *memory_desc = md.release();
        return dnnl_success;
    }
    md->ndims = ndims;
    md->data_type = data_type;
    md->format_kind = dnnl_blocked;
    bool runtime = false;
    for (int i = 0; i < ndims; ++i) {
        md->dims[i] = dims[i];
        runtime |= dims[i] == DNNL_RUNTIME_DIM_VAL;
    }
    if (!strides) {
        int64_t s = 1;
        for (int i = ndims - 1; i >= 0; --i) {
            md->strides[i] = runtime ? DNNL_RUNTIME_DIM_VAL : s;
            if (!runtime) s *= std::max<int64_t>(dims[i], 1);
        }
    } else {
        for (int i = 0; i < ndims; ++i) {
            if (strides[i] < 0 && strides[i] != DNNL_RUNTIME_DIM_VAL) return dnnl_invalid_arguments;
            md->strides[i] = strides[i];
        }
        if (!runtime) {
            // dims sorted by stride must not overlap (reference: memory_desc_init_by_strides)
            std::vector<int> idx;
            for (int i = 0; i < ndims; ++i)
                if (dims[i] > 1) idx.push_back(i);
            std::sort(idx.begin(), idx.end(), [&](int a, int b) { return strides[a] < strides[b]; });
            int64_t min_next = 1;
            for (int i : idx) {
                if (strides[i] < min_next) return dnnl_invalid_arguments;
                min_next = strides[i] * dims[i];
            }
        }
    }
    *memory_desc = md.release();
    return dnnl_success;
}

dnnl_status_t dnnl_memory_desc_create_with_tag(dnnl_memory_desc_t *memory_desc, int ndims, const dnnl_dims_t dims,
        dnnl_data_type_t data_type, dnnl_format_tag_t tag) {
    if (!memory_desc) return dnnl_invalid_arguments;
    dnnl_status_t st = check_dims(ndims, dims, data_type);
    if (st != dnnl_success) return st;
    if (ndims == 0) {
        *memory_desc = new dnnl_memory_desc();
        return dnnl_success;
    }
    if (tag == dnnl_format_tag_undef) return dnnl_invalid_arguments;
    if (tag == dnnl_format_tag_any) {
        dnnl_memory_desc *md = new dnnl_memory_desc();
        md->ndims = ndims;
        md->data_type = data_type;
        md->format_kind = dnnl_format_kind_any;
        for (int i = 0; i < ndims; ++i) md->dims[i] = dims[i];
        *memory_desc = md;
        return dnnl_success;
    }
    // outer-to-inner order of the logical dims for each plain tag
    std::vector<int> order;
    switch (tag) {
        case dnnl_a: order = {0}; break;
        case dnnl_ab: order = {0, 1}; break;
        case dnnl_ba: order = {1, 0}; break;
        case dnnl_abc: order = {0, 1, 2}; break;
        case dnnl_acb: order = {0, 2, 1}; break;
        case dnnl_bac: order = {1, 0, 2}; break;
        case dnnl_abcd: order = {0, 1, 2, 3}; break;
        case dnnl_abdc: order = {0, 1, 3, 2}; break;
        case dnnl_abcde: order = {0, 1, 2, 3, 4}; break;
        default: return dnnl_unimplemented; // blocked tags of other engines
    }
    if ((int)order.size() != ndims) return dnnl_invalid_arguments;
    dnnl_dims_t strides;
    int64_t s = 1;
    // a stride that depends on a dim known only at execution is itself known only then
    // (reference: memory_desc_init_by_tag with runtime dims, src/common/memory_desc.cpp)
    bool rt = false;
    for (int j = ndims - 1; j >= 0; --j) {
        strides[order[j]] = rt ? DNNL_RUNTIME_DIM_VAL : s;
        if (dims[order[j]] == DNNL_RUNTIME_DIM_VAL) rt = true;
        else s *= std::max<int64_t>(dims[order[j]], 1);
    }
    return dnnl_memory_desc_create_with_strides(memory_desc, ndims, dims, data_type, strides);
}

dnnl_status_t dnnl_memory_desc_create_submemory(dnnl_memory_desc_t *memory_desc, const_dnnl_memory_desc_t parent,
        const dnnl_dims_t dims, const dnnl_dims_t offsets) {
    if (!memory_desc || !parent || !dims || !offsets) return dnnl_invalid_arguments;
    if (!parent->is_plain() || parent->has_runtime_dims()) return dnnl_unimplemented;
    dnnl_memory_desc md = *parent;
    for (int i = 0; i < md.ndims; ++i) {
        if (dims[i] < 0 || offsets[i] < 0 || offsets[i] + dims[i] > parent->dims[i]) return dnnl_invalid_arguments;
        md.dims[i] = dims[i];
        md.offset0 += offsets[i] * parent->strides[i];
    }
    if (dt_nbits(md.data_type) == 4 && (md.offset0 & 1)) return dnnl_unimplemented;
    *memory_desc = new dnnl_memory_desc(md);
    return dnnl_success;
}

dnnl_status_t dnnl_memory_desc_reshape(dnnl_memory_desc_t *out, const_dnnl_memory_desc_t in, int ndims,
        const dnnl_dims_t dims) {
    if (!out || !in || !dims || ndims <= 0 || ndims > DNNL_MAX_NDIMS) return dnnl_invalid_arguments;
    if (!in->is_plain() || in->has_runtime_dims()) return dnnl_invalid_arguments;
    int64_t n = 1;
    for (int i = 0; i < ndims; ++i) {
        if (dims[i] < 0) return dnnl_invalid_arguments;
        n *= dims[i];
    }
    if (n != in->nelems()) return dnnl_invalid_arguments;
    dnnl_memory_desc md;
    md.ndims = ndims;
    md.data_type = in->data_type;
    md.format_kind = dnnl_blocked;
    md.offset0 = in->offset0;
    if (in->is_dense_row_major()) {
        int64_t s = 1;
        for (int i = ndims - 1; i >= 0; --i) {
            md.dims[i] = dims[i];
            md.strides[i] = s;
            s *= std::max<int64_t>(dims[i], 1);
        }
    } else {
        // only insertion / removal of unit dims keeps a strided layout expressible
        int j = 0;
        for (int i = 0; i < ndims; ++i) {
            md.dims[i] = dims[i];
            while (j < in->ndims && in->dims[j] == 1 && dims[i] != 1) ++j;
            if (dims[i] == 1 && !(j < in->ndims && in->dims[j] == 1)) {
                md.strides[i] = 1;
                continue;
            }
            if (j >= in->ndims || in->dims[j] != dims[i]) return dnnl_invalid_arguments;
            md.strides[i] = in->strides[j++];
        }
        for (int i = ndims - 1, last = 1; i >= 0; --i) { // give unit dims a consistent stride
            if (md.dims[i] == 1) md.strides[i] = last;
            else last = (int)(md.strides[i] * md.dims[i]);
        }
    }
    *out = new dnnl_memory_desc(md);
    return dnnl_success;
}

dnnl_status_t dnnl_memory_desc_permute_axes(dnnl_memory_desc_t *out, const_dnnl_memory_desc_t in, const int *perm) {
    if (!out || !in || !perm) return dnnl_invalid_arguments;
    if (!in->is_plain() && !in->is_any()) return dnnl_invalid_arguments;
    std::vector<bool> seen(in->ndims, false);
    for (int i = 0; i < in->ndims; ++i) {
        if (perm[i] < 0 || perm[i] >= in->ndims || seen[perm[i]]) return dnnl_invalid_arguments;
        seen[perm[i]] = true;
    }
    dnnl_memory_desc md = *in;
    for (int i = 0; i < in->ndims; ++i) {
        md.dims[perm[i]] = in->dims[i];
        md.strides[perm[i]] = in->strides[i];
    }
    *out = new dnnl_memory_desc(md);
    return dnnl_success;
}

dnnl_status_t dnnl_memory_desc_query(const_dnnl_memory_desc_t md, dnnl_query_t what, void *result) {
    if (!md || !result) return dnnl_invalid_arguments;
    static const dnnl_dims_t zeros = {0};
    switch (what) {
        case dnnl_query_ndims_s32: *(int32_t *)result = md->ndims; break;
        case dnnl_query_dims: *(const int64_t **)result = md->dims; break;
        case dnnl_query_data_type: *(dnnl_data_type_t *)result = (dnnl_data_type_t)md->data_type; break;
        case dnnl_query_submemory_offset_s64: *(int64_t *)result = md->offset0; break;
        case dnnl_query_padded_dims: *(const int64_t **)result = md->dims; break;
        case dnnl_query_padded_offsets: *(const int64_t **)result = zeros; break;
        case dnnl_query_format_kind: *(dnnl_format_kind_t *)result = (dnnl_format_kind_t)md->format_kind; break;
        case dnnl_query_strides:
            if (!md->is_plain()) return dnnl_invalid_arguments;
            *(const int64_t **)result = md->strides;
            break;
        case dnnl_query_inner_nblks_s32:
            if (!md->is_plain()) return dnnl_invalid_arguments;
            *(int32_t *)result = 0;
            break;
        case dnnl_query_inner_blks:
        case dnnl_query_inner_idxs:
            if (!md->is_plain()) return dnnl_invalid_arguments;
            *(const int64_t **)result = zeros;
            break;
        default: return dnnl_unimplemented;
    }
    return dnnl_success;
}

int dnnl_memory_desc_equal(const_dnnl_memory_desc_t lhs, const_dnnl_memory_desc_t rhs) {
    if (lhs == rhs) return 1;
    if (!lhs || !rhs) return 0;
    return lhs->equal(*rhs) ? 1 : 0;
}

size_t dnnl_memory_desc_get_size(const_dnnl_memory_desc_t md) {
    return md ? md->size_bytes() : 0;
}

size_t dnnl_data_type_size(dnnl_data_type_t dt) {
    const int bits = dt_nbits(dt);
    return bits >= 8 ? (size_t)bits / 8 : (bits == 4 ? 1 : 0);
}

// ---- memory objects ---------------------------------------------------------

dnnl_status_t dnnl_memory_create(dnnl_memory_t *memory, const_dnnl_memory_desc_t md, dnnl_engine_t engine, void *handle) {
    if (!memory || !md || !engine) return dnnl_invalid_arguments;
    if (md->is_any() || md->has_runtime_dims()) return dnnl_invalid_arguments;
    auto m = std::unique_ptr<dnnl_memory>(new dnnl_memory());
    m->md = *md;
    m->engine = engine;
    if (handle == DNNL_MEMORY_ALLOCATE && engine->host) {
        const size_t bytes = md->size_bytes();
        if (bytes && !(m->handle = std::aligned_alloc(64, (bytes + 63) / 64 * 64))) return dnnl_out_of_memory;
        m->owned = true;
    } else if (handle == DNNL_MEMORY_ALLOCATE) {
        if (set_device(engine) != dnnl_success) return dnnl_runtime_error;
        const size_t bytes = md->size_bytes();
        if (bytes) {
            if (device_alloc(&m->handle, bytes) != cudaSuccess) {
                (void)cudaGetLastError();
                return dnnl_out_of_memory;
            }
        }
        m->owned = true;
    } else {
        m->handle = handle;
    }
    engine->refs.fetch_add(1);
    *memory = m.release();
    return dnnl_success;
}

dnnl_status_t dnnl_memory_get_memory_desc(const_dnnl_memory_t memory, const_dnnl_memory_desc_t *md) {
    if (!memory || !md) return dnnl_invalid_arguments;
    *md = &memory->md;
    return dnnl_success;
}

dnnl_status_t dnnl_memory_get_engine(const_dnnl_memory_t memory, dnnl_engine_t *engine) {
    if (!memory || !engine) return dnnl_invalid_arguments;
    *engine = memory->engine;
    return dnnl_success;
}

dnnl_status_t dnnl_memory_map_data(const_dnnl_memory_t cmem, void **mapped_ptr) {
    if (!cmem || !mapped_ptr) return dnnl_invalid_arguments;
    dnnl_memory *mem = const_cast<dnnl_memory *>(cmem);
    if (mem->mapped) return dnnl_invalid_arguments;
    const size_t bytes = mem->md.size_bytes();
    if (!mem->handle || bytes == 0) {
        *mapped_ptr = nullptr;
        return dnnl_success;
    }
    if (mem->engine->host) { // host memory is its own mapping
        *mapped_ptr = mem->handle;
        return dnnl_success;
    }
    if (set_device(mem->engine) != dnnl_success) return dnnl_runtime_error;
    void *host = nullptr;
    if (pinned_alloc(&host, bytes) != cudaSuccess) return dnnl_out_of_memory;
    // every stream that may have written the buffer must have finished
    if (cudaDeviceSynchronize() != cudaSuccess
            || cudaMemcpy(host, (const char *)mem->handle + mem->md.offset0 * dt_nbits(mem->md.data_type) / 8, bytes,
                       cudaMemcpyDeviceToHost)
                    != cudaSuccess) {
        cudaFreeHost(host);
        return dnnl_runtime_error;
    }
    mem->mapped = host;
    *mapped_ptr = host;
    return dnnl_success;
}

dnnl_status_t dnnl_memory_unmap_data(const_dnnl_memory_t cmem, void *mapped_ptr) {
    if (!cmem) return dnnl_invalid_arguments;
    dnnl_memory *mem = const_cast<dnnl_memory *>(cmem);
    if (mem->engine->host) return dnnl_success;
    if (!mem->mapped) return mapped_ptr ? dnnl_invalid_arguments : dnnl_success;
    if (mapped_ptr != mem->mapped) return dnnl_invalid_arguments;
    if (set_device(mem->engine) != dnnl_success) return dnnl_runtime_error;
    const size_t bytes = mem->md.size_bytes();
    cudaError_t e = cudaMemcpy((char *)mem->handle + mem->md.offset0 * dt_nbits(mem->md.data_type) / 8, mem->mapped,
            bytes, cudaMemcpyHostToDevice);
    cudaFreeHost(mem->mapped);
    mem->mapped = nullptr;
    return e == cudaSuccess ? dnnl_success : dnnl_runtime_error;
}

dnnl_status_t dnnl_memory_get_data_handle(const_dnnl_memory_t memory, void **handle) {
    if (!memory || !handle) return dnnl_invalid_arguments;
    *handle = memory->handle;
    return dnnl_success;
}

dnnl_status_t dnnl_memory_set_data_handle(dnnl_memory_t memory, void *handle) {
    if (!memory) return dnnl_invalid_arguments;
    if (memory->owned && memory->handle) {
        if (memory->engine->host) {
            std::free(memory->handle);
        } else {
            cudaSetDevice(memory->engine->device);
            cudaFree(memory->handle);
        }
    }
    memory->owned = false;
    memory->handle = handle;
    return dnnl_success;
}

dnnl_status_t dnnl_memory_destroy(dnnl_memory_t memory) {
    if (!memory) return dnnl_success; // like delete: nothing to do
    if (memory->engine->host) {
        if (memory->owned && memory->handle) std::free(memory->handle);
    } else if (memory->engine->usable()) {
        cudaSetDevice(memory->engine->device);
        if (memory->mapped) cudaFreeHost(memory->mapped);
        if (memory->owned && memory->handle) cudaFree(memory->handle);
    }
    dnnl_engine_destroy(memory->engine);
    delete memory;
    return dnnl_success;
}
