// Weights reorder / pack kernels and small utilities.
//
//  * plain strided 2-D copy with data-type conversion (saturate + round to
//    nearest even for integer destinations), the counterpart of the
//    reference's simple_reorder (src/cpu/reorder/simple_reorder.hpp);
//  * pack of 8-bit (K, N) weights into the tensor-core layout B200_WEI_KMAJOR:
//    [N][K] with K contiguous, followed (256-byte aligned) by the s32 column
//    sums sum_k w[k][n] that the int8 kernel multiplies by the source
//    zero-point -- the compensation the reference computes when it reorders
//    into its own blocked layout (src/cpu/x64/matmul/brgemm_matmul.cpp:1184-1200,
//    src/cpu/reorder/cpu_reorder.hpp compensation flags).
#include "common.cuh"
#include "launch.hpp"

namespace b200 {

std::atomic<unsigned long long> g_launches {0};

// ---- plain copy / convert -------------------------------------------------------

__global__ void __launch_bounds__(256) reorder_plain_kernel(const void *__restrict__ src, int src_dt, int64_t ssk,
        int64_t ssn, void *__restrict__ dst, int dst_dt, int64_t dsk, int64_t dsn, int64_t K, int64_t N) {
    const int64_t total = K * N;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t k = i / N, n = i % N;
        const int64_t so = k * ssk + n * ssn, dof = k * dsk + n * dsn;
        if (src_dt == dst_dt) {
            switch (dt_bits(src_dt)) {
                case 32: ((uint32_t *)dst)[dof] = ((const uint32_t *)src)[so]; break;
                case 16: ((uint16_t *)dst)[dof] = ((const uint16_t *)src)[so]; break;
                default: ((uint8_t *)dst)[dof] = ((const uint8_t *)src)[so]; break;
            }
        } else if (dt_is_int(src_dt) && dt_is_int(dst_dt)) {
            // integer to integer: saturate without a float round trip
            long long v = load_int(src_dt, src, so);
            switch (dst_dt) {
                case B200_DT_S32: ((int32_t *)dst)[dof] = (int32_t)v; break;
                case B200_DT_S8: ((int8_t *)dst)[dof] = (int8_t)(v < -128 ? -128 : v > 127 ? 127 : v); break;
                case B200_DT_U8: ((uint8_t *)dst)[dof] = (uint8_t)(v < 0 ? 0 : v > 255 ? 255 : v); break;
                default: break;
            }
        } else {
            store_f32(dst_dt, load_f32(src_dt, src, so), dst, dof);
        }
    }
}

// ---- pack to K-major + column sums ------------------------------------------------

// 64 x 64 byte tiles through shared memory: coalesced reads along whichever
// source dim is contiguous, coalesced 16-byte writes along K.
__global__ void __launch_bounds__(256) pack_kmajor_kernel(const uint8_t *__restrict__ src, int64_t ssk, int64_t ssn,
        uint8_t *__restrict__ dst, int64_t K, int64_t N) {
    __shared__ uint8_t tile[64][64 + 4];
    const int64_t k0 = (int64_t)blockIdx.x * 64, n0 = (int64_t)blockIdx.y * 64;
    const int t = threadIdx.x;
    if (ssn == 1) {
        // source rows are k, contiguous in n
        for (int i = t; i < 64 * 64; i += 256) {
            const int kk = i / 64, nn = i % 64;
            const int64_t k = k0 + kk, n = n0 + nn;
            tile[kk][nn] = (k < K && n < N) ? src[k * ssk + n] : 0;
        }
    } else {
        for (int i = t; i < 64 * 64; i += 256) {
            const int nn = i / 64, kk = i % 64;
            const int64_t k = k0 + kk, n = n0 + nn;
            tile[kk][nn] = (k < K && n < N) ? src[k * ssk + n * ssn] : 0;
        }
    }
    __syncthreads();
    for (int i = t; i < 64 * 64; i += 256) {
        const int nn = i / 64, kk = i % 64;
        const int64_t k = k0 + kk, n = n0 + nn;
        if (k < K && n < N) dst[n * K + k] = tile[kk][nn];
    }
}

// out[n] = sum_k w[k][n]; one warp per column when K is contiguous, one thread
// per column when N is contiguous (both coalesced)
__global__ void __launch_bounds__(256) colsum_kernel(const void *__restrict__ w, int dt, int64_t K, int64_t N,
        int64_t sk, int64_t sn, int32_t *__restrict__ out) {
    if (sk == 1) {
        const int lane = threadIdx.x & 31;
        const int64_t n = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
        if (n >= N) return;
        int acc = 0;
        for (int64_t k = lane; k < K; k += 32) acc += load_int(dt, w, k + n * sn);
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (lane == 0) out[n] = acc;
    } else {
        const int64_t n = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
        if (n >= N) return;
        int acc = 0;
        for (int64_t k = 0; k < K; ++k) acc += load_int(dt, w, k * sk + n * sn);
        out[n] = acc;
    }
}

} // namespace b200

using namespace b200;

static inline size_t align256(size_t x) { return (x + 255) / 256 * 256; }

extern "C" size_t b200_packed_colsum_offset(int64_t K, int64_t N, int32_t dt) {
    (void)dt;
    return align256((size_t)K * (size_t)N);
}

extern "C" size_t b200_packed_weights_bytes(int64_t K, int64_t N, int32_t dt, int32_t layout) {
    if (layout == B200_WEI_KMAJOR) return b200_packed_colsum_offset(K, N, dt) + align256((size_t)N * sizeof(int32_t));
    if (layout == B200_WEI_WC4_TC || layout == B200_WEI_WC8_TC) return b200_wc_tc_packed_bytes(K, N, dt);
    return (size_t)((K * N * dt_bits(dt) + 7) / 8);
}

// Column-split results gathered rank by rank ([parts][M][N / parts], what an all-gather of
// contiguous slices produces) -> one row-major (M, N) matrix.  16 bytes per thread.
__global__ void __launch_bounds__(256) gather_columns_kernel(const uint4 *__restrict__ staged, uint4 *__restrict__ dst,
        int64_t M, int64_t row_vecs, int parts) {
    // row_vecs = 16-byte vectors per row of one part
    const int64_t total = M * row_vecs * parts;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t v = i % row_vecs, m = (i / row_vecs) % M, part = i / (row_vecs * M);
        dst[(m * parts + part) * row_vecs + v] = staged[i];
    }
}

extern "C" int b200_colsum_launch(const void *wei, int32_t wei_dt, int64_t K, int64_t N, int64_t sk, int64_t sn,
        int32_t *out, b200_stream_t stream) {
    if (!wei || !out || K < 0 || N < 0) return B200_ERR_BAD_ARG;
    if (wei_dt != B200_DT_S8 && wei_dt != B200_DT_U8) return B200_ERR_UNSUPPORTED;
    if (N == 0) return 0;
    const int64_t threads = sk == 1 ? N * 32 : N;
    colsum_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, (cudaStream_t)stream>>>(wei, wei_dt, K, N, sk, sn, out);
    return after_launch();
}

extern "C" int b200_reorder_launch(const b200_reorder_params_t *p, b200_stream_t stream) {
    if (!p || !p->src || !p->dst || p->K < 0 || p->N < 0) return B200_ERR_BAD_ARG;
    if (p->scale) return B200_ERR_UNSUPPORTED;
    if (p->K == 0 || p->N == 0) return 0;
    if (p->src_layout != B200_WEI_PLAIN) return B200_ERR_UNSUPPORTED;
    cudaStream_t cs = (cudaStream_t)stream;
    if (p->dst_layout == B200_WEI_KMAJOR) {
        if (p->src_dt != p->dst_dt || dt_bits(p->src_dt) != 8) return B200_ERR_UNSUPPORTED;
        dim3 grid((unsigned)((p->K + 63) / 64), (unsigned)((p->N + 63) / 64));
        pack_kmajor_kernel<<<grid, 256, 0, cs>>>((const uint8_t *)p->src, p->src_sk, p->src_sn, (uint8_t *)p->dst, p->K,
                p->N);
        int rc = after_launch();
        if (rc) return rc;
        int32_t *colsum = (int32_t *)((char *)p->dst + b200_packed_colsum_offset(p->K, p->N, p->dst_dt));
        if (p->src_dt == B200_DT_S8 || p->src_dt == B200_DT_U8)
            return b200_colsum_launch(p->src, p->src_dt, p->K, p->N, p->src_sk, p->src_sn, colsum, stream);
        return cudaMemsetAsync(colsum, 0, (size_t)p->N * sizeof(int32_t), cs) == cudaSuccess ? 0 : (int)cudaGetLastError();
    }
    if (p->dst_layout == B200_WEI_WC8_TC) {
        if (p->src_dt != p->dst_dt) return B200_ERR_UNSUPPORTED;
        return b200_wc_tc_pack8_launch(p->src, p->src_sk, p->src_sn, p->dst, p->K, p->N, p->src_dt, stream);
    }
    if (p->dst_layout == B200_WEI_WC4_TC) {
        if (p->src_dt != p->dst_dt || p->src_sn != 1 || p->src_sk != p->N) return B200_ERR_UNSUPPORTED;
        return b200_wc_tc_pack_launch(p->src, p->dst, p->K, p->N, p->src_dt, stream);
    }
    if (p->dst_layout == B200_WEI_WC4_TILED) {
        if (p->src_dt != p->dst_dt || p->src_sn != 1 || p->src_sk != p->N) return B200_ERR_UNSUPPORTED;
        return b200_wc_pack_launch(p->src, p->dst, p->K, p->N, p->src_dt, stream);
    }
    if (p->dst_layout != B200_WEI_PLAIN) return B200_ERR_UNSUPPORTED;
    if (dt_bits(p->src_dt) == 4 || dt_bits(p->dst_dt) == 4) {
        // 4-bit tensors: dense same-type copies only (two values per byte)
        if (p->src_dt != p->dst_dt || p->src_sn != 1 || p->dst_sn != 1 || p->src_sk != p->N || p->dst_sk != p->N
                || (p->N & 1))
            return B200_ERR_UNSUPPORTED;
        return cudaMemcpyAsync(p->dst, p->src, (size_t)(p->K * p->N / 2), cudaMemcpyDeviceToDevice, cs) == cudaSuccess
                ? 0
                : (int)cudaGetLastError();
    }
    const int64_t total = p->K * p->N;
    int64_t blocks = (total + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    reorder_plain_kernel<<<(unsigned)blocks, 256, 0, cs>>>(p->src, p->src_dt, p->src_sk, p->src_sn, p->dst, p->dst_dt,
            p->dst_sk, p->dst_sn, p->K, p->N);
    return after_launch();
}

// The kernels of this library never wait without a bound: a wait that runs out ORs a code
// into the status word and the kernel winds down.  This kernel is that mechanism on its
// own, for tests: one warp polls an mbarrier that nothing will ever complete, at most
// max_polls times, then reports through the status word like the matmul kernels do.
__global__ void bounded_wait_selftest_kernel(uint32_t *status, uint32_t max_polls) {
    __shared__ uint64_t bar;
    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(&bar);
    if (threadIdx.x == 0) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(addr));
    __syncwarp();
    bool done = false;
    for (uint32_t i = 0; i < max_polls && !done; ++i) {
        uint32_t ok;
        asm volatile(
                "{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], 0;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                : "=r"(ok)
                : "r"(addr)
                : "memory");
        done = ok != 0;
        if (!done) __nanosleep(100);
    }
    if (!done && threadIdx.x == 0 && status) atomicOr(status, B200_STATUS_SELFTEST_WAIT);
}

extern "C" int b200_selftest_bounded_wait_launch(uint32_t *status, uint32_t max_polls, b200_stream_t stream) {
    if (!status || max_polls == 0 || max_polls > (1u << 20)) return B200_ERR_BAD_ARG; // at most ~0.1 s
    bounded_wait_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(status, max_polls);
    return after_launch();
}

extern "C" uint64_t b200_launch_count(void) {
    return g_launches.load();
}

extern "C" int b200_gather_columns_launch(const void *staged, void *dst, int64_t M, int64_t N, int32_t parts,
        int32_t elem_bytes, b200_stream_t stream) {
    if (!staged || !dst || M < 0 || N < 0 || parts <= 0 || elem_bytes <= 0) return B200_ERR_BAD_ARG;
    if (N % parts != 0 || ((N / parts) * elem_bytes) % 16 != 0) return B200_ERR_UNSUPPORTED;
    if ((((uintptr_t)staged) | ((uintptr_t)dst)) & 15) return B200_ERR_BAD_ARG;
    if (M == 0 || N == 0) return 0;
    const int64_t row_vecs = (N / parts) * elem_bytes / 16;
    int64_t blocks = (M * row_vecs * parts + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    gather_columns_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>((const uint4 *)staged, (uint4 *)dst, M,
            row_vecs, parts);
    return after_launch();
}
