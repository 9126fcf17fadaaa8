// Verbose tracing and version.  The verbose line has the shape of the
// reference's (doc/performance_considerations/verbose.md:22-45,
// src/common/verbose.cpp):
//   onednn_verbose,v1,primitive,exec,gpu:0,matmul,<impl>,undef,<mds>,<attr>,,<problem>,<ms>
// controlled by ONEDNN_VERBOSE / DNNL_VERBOSE (0, 1, 2, or "dispatch") and
// dnnl_set_verbose.
#include <cstdio>
#include <cstdlib>

#include "internal.hpp"

namespace b200 {

static std::mutex g_verbose_mu;
static int g_verbose = -1;
static bool g_verbose_dispatch = false;
static bool g_header_printed = false;

int verbose_level() {
    std::lock_guard<std::mutex> g(g_verbose_mu);
    if (g_verbose < 0) {
        g_verbose = 0;
        const char *v = std::getenv("ONEDNN_VERBOSE");
        if (!v) v = std::getenv("DNNL_VERBOSE");
        if (v) {
            std::string s(v);
            if (s.find("dispatch") != std::string::npos || s.find("all") != std::string::npos) g_verbose_dispatch = true;
            if (s.find("profile_exec") != std::string::npos || s.find("all") != std::string::npos) g_verbose = 1;
            if (s.find("profile_create") != std::string::npos || s.find("all") != std::string::npos) g_verbose = 2;
            if (!s.empty() && s[0] >= '0' && s[0] <= '9') g_verbose = atoi(v);
        }
    }
    return g_verbose;
}

static void header() {
    if (g_header_printed) return;
    g_header_printed = true;
    const dnnl_version_t *v = dnnl_version();
    std::printf("onednn_verbose,v1,info,oneDNN-compatible B200 matmul engine v%d.%d.%d\n", v->major, v->minor, v->patch);
    std::printf("onednn_verbose,v1,info,gpu,runtime:CUDA\n");
    std::printf("onednn_verbose,v1,primitive,info,template:operation,engine,primitive,implementation,prop_kind,"
                "memory_descriptors,attributes,auxiliary,problem_desc,exec_time\n");
}

std::string md_verbose(const char *tag, const dnnl_memory_desc &md) {
    if (md.ndims == 0) return "";
    char buf[64];
    std::string s = std::string(tag) + ":" + dt_name(md.data_type) + "::";
    s += md.format_kind == dnnl_format_kind_opaque ? "opaque:" : md.is_any() ? "any:" : "blocked:";
    s += md.layout_str() + "::f0";
    (void)buf;
    return s;
}

static std::string problem(const dnnl_primitive_desc *pd) {
    char buf[128];
    if (pd->kind == dnnl_matmul)
        std::snprintf(buf, sizeof buf, "%lldx%lld:%lldx%lld", (long long)pd->M(), (long long)pd->K(), (long long)pd->K(),
                (long long)pd->N());
    else {
        std::string s;
        for (int i = 0; i < pd->src.ndims; ++i) s += (i ? "x" : "") + std::to_string(pd->src.dims[i]);
        return s;
    }
    return buf;
}

static void line(const char *what, const dnnl_primitive_desc *pd, double ms, const char *extra) {
    std::lock_guard<std::mutex> g(g_verbose_mu);
    header();
    std::string mds;
    if (pd->kind == dnnl_matmul) {
        mds = md_verbose("src", pd->src) + " " + md_verbose("wei", pd->wei);
        if (pd->bias.ndims) mds += " " + md_verbose("bia", pd->bias);
        mds += " " + md_verbose("dst", pd->dst);
    } else {
        mds = md_verbose("src", pd->src) + " " + md_verbose("dst", pd->dst);
    }
    std::printf("onednn_verbose,v1,primitive,%s%s,gpu:%d,%s,%s,undef,%s,%s,,%s,%g\n", what, extra, pd->engine->device,
            pd->kind == dnnl_matmul ? "matmul" : "reorder", pd->impl_str.c_str(), mds.c_str(), pd->attr.str().c_str(),
            problem(pd).c_str(), ms);
    std::fflush(stdout);
}

void verbose_exec(const dnnl_primitive *prim, double ms) {
    if (verbose_level() >= 1) line("exec", prim->pd.get(), ms, "");
}

void verbose_create(const dnnl_primitive_desc *pd, double ms, bool cache_hit) {
    if (verbose_level() >= 2) line("create", pd, ms, cache_hit ? ":cache_hit" : ":cache_miss");
}

void verbose_dispatch(const char *impl, const char *why) {
    (void)verbose_level();
    if (!g_verbose_dispatch) return;
    std::lock_guard<std::mutex> g(g_verbose_mu);
    std::printf("onednn_verbose,v1,primitive,create:dispatch,matmul,%s,skipping: %s\n", impl, why);
    std::fflush(stdout);
}

std::atomic<uint64_t> g_scratch_epoch {1};
std::atomic<uint64_t> g_scratch_reclears {0};

// allocation-failure injection: the next g_fail_allocs allocations report out of memory
static std::atomic<int> g_fail_allocs {0};
static bool inject_failure() {
    int n = g_fail_allocs.load();
    while (n > 0)
        if (g_fail_allocs.compare_exchange_weak(n, n - 1)) return true;
    return false;
}
cudaError_t device_alloc(void **ptr, size_t bytes) {
    if (inject_failure()) return cudaErrorMemoryAllocation;
    return cudaMalloc(ptr, bytes);
}
cudaError_t device_alloc_async(void **ptr, size_t bytes, cudaStream_t stream) {
    if (inject_failure()) return cudaErrorMemoryAllocation;
    return cudaMallocAsync(ptr, bytes, stream);
}
cudaError_t pinned_alloc(void **ptr, size_t bytes) {
    if (inject_failure()) return cudaErrorMemoryAllocation;
    return cudaMallocHost(ptr, bytes);
}

uint64_t primitive_cache_hits();
uint64_t primitive_cache_size();

} // namespace b200

dnnl_status_t dnnl_b200_debug_fail_allocations(int count) {
    if (count < 0) return dnnl_invalid_arguments;
    b200::g_fail_allocs.store(count);
    return dnnl_success;
}

dnnl_status_t dnnl_b200_debug_mark_scratchpads_dirty(void) {
    b200::g_scratch_epoch.fetch_add(1);
    return dnnl_success;
}

dnnl_status_t dnnl_b200_debug_counter(int which, uint64_t *value) {
    if (!value) return dnnl_invalid_arguments;
    switch (which) {
        case DNNL_B200_COUNTER_CACHE_HITS: *value = b200::primitive_cache_hits(); break;
        case DNNL_B200_COUNTER_CACHE_SIZE: *value = b200::primitive_cache_size(); break;
        case DNNL_B200_COUNTER_SCRATCH_RECLEARS: *value = b200::g_scratch_reclears.load(); break;
        case DNNL_B200_COUNTER_KERNEL_LAUNCHES: *value = b200_launch_count(); break;
        default: return dnnl_invalid_arguments;
    }
    return dnnl_success;
}

dnnl_status_t dnnl_set_verbose(int level) {
    if (level < 0 || level > 2) return dnnl_invalid_arguments;
    (void)b200::verbose_level();
    std::lock_guard<std::mutex> g(b200::g_verbose_mu);
    b200::g_verbose = level;
    return dnnl_success;
}

const dnnl_version_t *dnnl_version(void) {
    // major.minor follow the API level this library is a drop-in for
    static const dnnl_version_t v = {3, 8, 0, "b200-native", 0u /* no CPU runtime */, 1024u /* CUDA */};
    return &v;
}
