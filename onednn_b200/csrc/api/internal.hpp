// Internal object model of the host library: what stands behind the opaque
// handles of onednn_b200.h.  The roles mirror the reference's common runtime
// (src/common/engine.hpp:49-178, stream.hpp:29-94, memory.hpp:44-120,
// memory_desc.hpp:262-345, primitive_attr.hpp:274-727, primitive_desc.hpp,
// primitive.hpp:42-135) but the design is specific to this engine: one
// descriptor type for plain strided tensors and for the packed weights
// layouts of the sm_100a kernels, a flat attribute record that lowers directly
// into the kernel parameter block, and an implementation list of four kernels.
#pragma once

#include <atomic>
#include <cstdint>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include <cuda_runtime.h>

#include "onednn_b200.h"
#include "onednn_b200_kernels.h"

// packed_layout value of an opaque descriptor that stands for a blocked layout of another engine
// (created from a blocked format tag): it can be described, compared and sized, nothing reads it
#define B200_LAYOUT_FOREIGN 100

namespace b200 {

// a data type a memory descriptor may carry (the whole enum of the reference); which of them a
// primitive here computes with is dt_valid below
inline bool dt_known(int dt) {
    return dt >= dnnl_f16 && dt <= dnnl_f4_e3m0;
}
inline bool dt_valid(int dt) {
    switch (dt) {
        case dnnl_f16: case dnnl_bf16: case dnnl_f32: case dnnl_s32: case dnnl_s8: case dnnl_u8:
        case dnnl_f8_e5m2: case dnnl_f8_e4m3: case dnnl_s4: case dnnl_u4: return true;
        default: return false;
    }
}
inline int dt_nbits(int dt) {
    switch (dt) {
        case dnnl_f32: case dnnl_s32: return 32;
        case dnnl_f16: case dnnl_bf16: return 16;
        case dnnl_s8: case dnnl_u8: case dnnl_f8_e5m2: case dnnl_f8_e4m3: case dnnl_boolean: case dnnl_e8m0: return 8;
        case dnnl_s4: case dnnl_u4: case dnnl_f4_e2m1: case dnnl_f4_e3m0: return 4;
        case dnnl_f64: return 64;
        default: return 0;
    }
}
inline bool dt_is_int8(int dt) { return dt == dnnl_s8 || dt == dnnl_u8; }
inline bool dt_is_int4(int dt) { return dt == dnnl_s4 || dt == dnnl_u4; }
inline bool dt_is_fp8(int dt) { return dt == dnnl_f8_e4m3 || dt == dnnl_f8_e5m2; }
const char *dt_name(int dt);

} // namespace b200

// A memory descriptor: logical dims + data type + one of
//   any     : layout to be chosen by the primitive descriptor,
//   blocked : plain strided layout (no inner blocks in this engine),
//   opaque  : a packed weights layout of this engine (B200_WEI_*), addressed
//             only by the kernels; `packed_layout` says which.
struct dnnl_memory_desc {
    int ndims = 0;
    int64_t dims[DNNL_MAX_NDIMS] = {0};
    int data_type = dnnl_data_type_undef;
    int format_kind = dnnl_format_kind_undef;
    int64_t strides[DNNL_MAX_NDIMS] = {0};
    int64_t offset0 = 0;
    int packed_layout = B200_WEI_PLAIN;

    int64_t nelems() const {
        if (ndims == 0) return 0;
        int64_t n = 1;
        for (int i = 0; i < ndims; ++i) n *= dims[i];
        return n;
    }
    bool has_zero_dim() const { return ndims > 0 && nelems() == 0; }
    bool has_runtime_dims() const {
        for (int i = 0; i < ndims; ++i)
            if (dims[i] == DNNL_RUNTIME_DIM_VAL) return true;
        return false;
    }
    bool is_plain() const { return format_kind == dnnl_blocked; }
    bool is_any() const { return format_kind == dnnl_format_kind_any; }
    bool is_zero() const { return ndims == 0; }
    size_t size_bytes() const;
    // opaque (packed weights) descriptors with batch dims: every 2-D slice is packed on its own and
    // slices follow one another at this distance (a multiple of 256 bytes), batch index row-major
    size_t packed_slice_stride() const;
    bool equal(const dnnl_memory_desc &o) const;
    bool is_dense_row_major() const; // strides of tag a / ab / abc ...
    std::string layout_str() const;  // "ab", "ba", "a:strided", "packed:kmajor", "any"
};

struct dnnl_engine {
    dnnl_engine_kind_t kind = dnnl_gpu;
    int device = -1; // CUDA ordinal; -1 = descriptor-only engine (no device present)
    bool host = false; // the dnnl_cpu engine: host memory and reorders only (host_engine.cpp)
    std::atomic<int> refs {1};
    int sm_major = 0, sm_minor = 0, sm_count = 0;
    bool usable() const { return host || device >= 0; }
};

struct dnnl_stream {
    dnnl_engine *engine = nullptr;
    void *cuda_stream = nullptr; // cudaStream_t
    bool owns_stream = false;
    unsigned flags = dnnl_stream_default_flags;
    uint32_t *status = nullptr; // device word the kernels flag bounded-wait failures in
    // profiling: one (start, stop) event pair per executed primitive
    std::vector<std::pair<void *, void *>> prof_events;
    std::mutex mu;
};

struct dnnl_memory {
    dnnl_memory_desc md;
    dnnl_engine *engine = nullptr;
    void *handle = nullptr;
    bool owned = false;
    void *mapped = nullptr; // pinned host copy while mapped
};

namespace b200 {

// one scales / zero-points entry of an attribute (reference: quant_entry_t,
// src/common/primitive_attr_quant.hpp:45-140)
struct quant_entry_t {
    bool set = false;
    int mask = 0;
    int dt = dnnl_f32;
    int group_ndims = 0;
    int64_t groups[2] = {1, 1};
    bool operator==(const quant_entry_t &o) const {
        return set == o.set && mask == o.mask && dt == o.dt && groups[0] == o.groups[0] && groups[1] == o.groups[1];
    }
};

struct post_op_t {
    int kind = 0; // dnnl_sum / dnnl_eltwise / dnnl_binary / dnnl_prelu
    int alg = 0;
    float alpha = 0.f, beta = 0.f, scale = 1.f;
    int32_t zero_point = 0;
    int dt = dnnl_data_type_undef; // sum data type
    dnnl_memory_desc src1;         // binary
    int mask = 0;                  // prelu
};

} // namespace b200

struct dnnl_post_ops {
    std::vector<b200::post_op_t> entries;
};

struct dnnl_primitive_attr {
    dnnl_fpmath_mode_t fpmath = dnnl_fpmath_mode_strict;
    int apply_to_int = 0;
    int deterministic = 0;
    dnnl_accumulation_mode_t acc_mode = dnnl_accumulation_mode_strict;
    dnnl_scratchpad_mode_t scratchpad_mode = dnnl_scratchpad_mode_library;
    std::map<int, b200::quant_entry_t> scales, zero_points;
    std::map<int, int> rounding;
    dnnl_post_ops post_ops;

    const b200::quant_entry_t &scale(int arg) const;
    const b200::quant_entry_t &zp(int arg) const;
    std::string str() const; // verbose representation
};

namespace b200 {

// the matmul implementations of this engine, in dispatch order
enum impl_id_t { IMPL_TC8 = 0, IMPL_WC = 1, IMPL_GENERIC = 2, IMPL_REORDER = 3, IMPL_COUNT };
const char *impl_name(int id, const dnnl_primitive_desc *pd);

} // namespace b200

struct dnnl_primitive_desc {
    dnnl_primitive_kind_t kind = dnnl_undefined_primitive;
    dnnl_engine *engine = nullptr;
    dnnl_primitive_attr attr;
    // descriptors as the user gave them (weights may be `any`) ...
    dnnl_memory_desc user_src, user_wei, user_bias, user_dst;
    // ... and as resolved by the selected implementation
    dnnl_memory_desc src, wei, bias, dst;
    dnnl_memory_desc scratchpad; // 1-D u8
    dnnl_memory_desc zero_md;
    int impl = -1;
    std::string impl_str;
    // scratch md returned for DNNL_ARG_ATTR_* queries
    mutable std::map<int, dnnl_memory_desc> arg_mds;
    // batched problems (more than two dims): the descriptor of one 2-D slice, which the
    // selected implementation runs once per batch index
    std::shared_ptr<dnnl_primitive_desc> inner;
    bool collapsed = false; // batched with broadcast weights and dense rows: `inner` is the whole problem as one 2-D matmul
    // batched: scales / zero-points whose mask reaches into the batch dims -- the argument's memory then holds one
    // set of values per index of those dims, and every batch index is executed with its own part of it
    struct batch_quant_t {
        int exec_arg;   // DNNL_ARG_ATTR_SCALES | arg or DNNL_ARG_ATTR_ZERO_POINTS | arg
        int tensor_arg; // DNNL_ARG_SRC / WEIGHTS / DST: whose dims the mask is over
        int batch_mask; // the mask's bits over the batch dims
        bool is_zp;
    };
    std::vector<batch_quant_t> batch_quant;
    // some dims are DNNL_RUNTIME_DIM_VAL: the implementation is chosen at execution, from the
    // descriptors of the memory arguments
    bool runtime = false;
    // kind == dnnl_inner_product: `inner` is the matmul it runs as; weights / bias keep the
    // descriptors the caller gave, (OC, IC) and (OC)
    bool ip = false;

    int64_t M() const { return dst.dims[dst.ndims - 2]; }
    int64_t N() const { return dst.dims[dst.ndims - 1]; }
    int64_t K() const { return src.dims[src.ndims - 1]; }
};

namespace b200 {
// Kernels that accumulate in the library-owned scratchpad rely on finding it zeroed and leave it
// zeroed.  A kernel that gave up a bounded wait, or a launch sequence that failed half way, may
// not have: every such event advances this epoch, and a primitive whose scratchpad was last
// known clean in an older epoch has it cleared on the stream before its next execution.
extern std::atomic<uint64_t> g_scratch_epoch;
extern std::atomic<uint64_t> g_scratch_reclears; // how often that clearing was asked for (tests)

// Every device / pinned-host allocation of the host library goes through these, so that an
// allocation failure can be injected on the host (dnnl_b200_debug_fail_allocations) and the
// dnnl_out_of_memory paths tested without exhausting a GPU.  The reference surfaces the same
// status from its engine's allocator (src/common/engine.cpp:87-120, memory.cpp:159-163).
cudaError_t device_alloc(void **ptr, size_t bytes);
cudaError_t device_alloc_async(void **ptr, size_t bytes, cudaStream_t stream);
cudaError_t pinned_alloc(void **ptr, size_t bytes);
} // namespace b200

struct dnnl_primitive {
    std::shared_ptr<dnnl_primitive_desc> pd;
    void *lib_scratch = nullptr; // library-mode scratchpad (device)
    size_t lib_scratch_bytes = 0;
    mutable std::atomic<uint64_t> scratch_epoch {b200::g_scratch_epoch.load()}; // epoch in which lib_scratch was last known clean
    const dnnl_primitive *scratch_owner = nullptr; // set when lib_scratch is borrowed from another primitive
    ~dnnl_primitive();
};

namespace b200 {

// ---- validation + dispatch (matmul_pd.cpp) ----
dnnl_status_t matmul_validate(const dnnl_memory_desc &src, const dnnl_memory_desc &wei, const dnnl_memory_desc *bias,
        const dnnl_memory_desc &dst, const dnnl_primitive_attr &attr);
// tries implementations starting at `first`; fills pd->impl and resolved mds
dnnl_status_t matmul_select_impl(dnnl_primitive_desc *pd, int first);
dnnl_status_t matmul_execute(const dnnl_primitive *prim, dnnl_stream *stream, const std::map<int, dnnl_memory *> &args);
dnnl_status_t reorder_execute(const dnnl_primitive *prim, dnnl_stream *stream, const std::map<int, dnnl_memory *> &args);
// ---- host engine (host_engine.cpp) ----
dnnl_status_t host_reorder_pd_create(dnnl_primitive_desc_t *out, const dnnl_memory_desc &s, dnnl_engine *se,
        const dnnl_memory_desc &d, dnnl_engine *de, const dnnl_primitive_attr *attr);
dnnl_status_t host_reorder_execute(const dnnl_primitive *prim, dnnl_stream *stream, const dnnl_memory *from,
        const dnnl_memory *to);
dnnl_status_t inner_product_execute(const dnnl_primitive *prim, dnnl_stream *stream, const std::map<int, dnnl_memory *> &args);

// ---- verbose (service.cpp) ----
int verbose_level();
void verbose_exec(const dnnl_primitive *prim, double ms);
void verbose_create(const dnnl_primitive_desc *pd, double ms, bool cache_hit);
void verbose_dispatch(const char *impl, const char *why);
std::string md_verbose(const char *tag, const dnnl_memory_desc &md);

// ---- CUDA helpers (engine.cpp) ----
dnnl_status_t set_device(const dnnl_engine *e);
double now_ms();

// default attribute entries
extern const quant_entry_t default_quant_entry;

} // namespace b200
