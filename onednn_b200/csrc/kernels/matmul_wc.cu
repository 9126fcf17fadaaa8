// Weight-compressed decode GEMV / skinny GEMM: bf16 activations (M rows) times
// 4-bit weights with K-grouped scales and zero-points, f32 accumulation.
// Semantics: the reference's weights-decompression matmul
// (src/cpu/matmul/ref_matmul.cpp:130-233, with_wei_decompression), i.e.
//   dst[m][n] = epilogue( sum_k x[m][k] * (q[k][n] - zp[k/Gz][n]) * s[k/Gs][n] ).
//
// The kernel is HBM-bound (M = 1: 0.5 byte of weights per multiply-add), so
// the design goal is to stream the packed weights once with 128-bit loads and
// keep the per-byte instruction count low:
//
//  * Weights are read in the B200_WEI_WC4_TILED layout written by the pack
//    kernel below: the matrix is cut into tiles of 16 output columns x 64 k;
//    each tile is 512 contiguous bytes, 16 bytes per lane, ordered so that one
//    32-bit word of a lane holds exactly the eight 4-bit values that lane owns
//    in the A fragment of one mma.m16n8k16 (output columns play the role of the
//    MMA's M dimension, activations rows the role of its N dimension).
//  * A nibble becomes a bf16 with one logic op: (w >> 4i) & 0x000f000f | 0x43004300
//    gives the pair (128 + q_lo, 128 + q_hi) exactly.  No subtraction and no
//    multiply is spent per weight: the MMA accumulates sum_k x*(128+q) in f32,
//    a second MMA with an all-ones A tile accumulates sum_k x, and at every
//    quantisation-group boundary the fold
//        total += s * (acc - (128 + zp) * xsum)
//    applies scale and zero-point to a whole group at once (4 FMAs per thread
//    per group).  s4 weights are stored offset by 8, so they fold with 136 + zp.
//  * Work is split by bytes, not by tiles: the S = (N/16)*(K/64) tile steps are
//    dealt out in equal contiguous ranges to every warp of a grid sized to the
//    SM count, each warp streams its range with a 3-deep register prefetch ring
//    and adds its partial sums into an f32 scratch [M][N] with red.global.add;
//    a small second kernel applies the epilogue and leaves the scratch zeroed.
#include <mutex>

#include "common.cuh"
#include "launch.hpp"

namespace b200 {

constexpr int WC_WARPS = 8;           // warps per CTA
constexpr int WC_TILE_N = 16;         // output columns per tile (MMA M)
constexpr int WC_TILE_K = 64;         // k per 512-byte tile step

struct wc_args_t {
    const uint4 *wei;       // packed tiles
    const __nv_bfloat16 *x; // activations, row-major, converted to bf16 if needed
    int64_t x_ld;
    float *acc;             // scratch [M][N] f32, zero on entry
    int64_t M, N, K;
    int m0;                 // first activation row of this pass
    const void *scale; int scale_dt; int64_t scale_s0, scale_s1; uint32_t scale_g0; // g0: K-group size (K if none)
    const void *zp; int zp_dt; int64_t zp_s0, zp_s1; uint32_t zp_g0;
    uint32_t fold_k;        // fold period in k (multiple of 16)
    float nibble_offset;    // 128 (u4) or 136 (s4 stored offset by 8)
};

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg_stream(const uint4 *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// Scale and zero-point of output column n for K group `grp` (FASTQ) or for the group that
// contains k (generic).  FASTQ: bf16 scales and u4 zero-points, both [K / group][N] with
// the same group (the common decode configuration): two direct loads.
template <bool FASTQ>
__device__ __forceinline__ void wc_group_params(const wc_args_t &a, uint32_t grp, uint32_t k, uint32_t n, float &s,
        float &c) {
    if (FASTQ) {
        const uint32_t row = grp * (uint32_t)a.N + n;
        s = __uint_as_float((uint32_t)((const uint16_t *)a.scale)[row] << 16);
        const uint32_t byte = ((const uint8_t *)a.zp)[row >> 1];
        c = a.nibble_offset + (float)((byte >> ((row & 1) * 4)) & 0xf);
    } else {
        s = 1.f;
        c = a.nibble_offset;
        if (a.scale) s = load_f32(a.scale_dt, a.scale, (int64_t)(k / a.scale_g0) * a.scale_s0 + (int64_t)n * a.scale_s1);
        if (a.zp) c += (float)load_int(a.zp_dt, a.zp, (int64_t)(k / a.zp_g0) * a.zp_s0 + (int64_t)n * a.zp_s1);
    }
}

// MB   = number of 8-row activation blocks handled per pass (1, 2 or 4)
// XTAB = single activation row: sum_k x per tile step comes from a table the CTA builds
//        in shared memory; otherwise a second MMA with an all-ones A tile accumulates it.
//
// One tile step = 16 output columns x 64 k = 512 bytes of weights = four MMA k-steps.  Within
// a step the MMA's k slots are permuted so that everything a lane needs is contiguous in
// memory: lane (g, t) owns k = 16 t + 4 j + {0,1,2,3} of MMA step j, i.e. 32 contiguous
// bytes of its activation row per tile step (two 128-bit loads), and the pack kernel lays
// the weight nibbles out for the same permutation.  A dot product does not care in which
// order k is visited, as long as both operands agree.
template <int MB, bool FASTQ, bool XTAB>
__global__ void __launch_bounds__(WC_WARPS * 32) wc_gemv_kernel(const __grid_constant__ wc_args_t a) {
    __shared__ float xtab[XTAB ? 1024 : 1]; // sum of the activation row over each tile step (K <= 65536)
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t g = lane >> 2, t = lane & 3;
    const uint32_t kchunks = (uint32_t)(a.K / WC_TILE_K);
    if (XTAB) {
        // thread i sums 16 consecutive activations; four neighbours make one tile step
        const __nv_bfloat16 *xr = a.x + (int64_t)a.m0 * a.x_ld;
        for (uint32_t i = threadIdx.x; i < kchunks * 4; i += blockDim.x) {
            const uint4 *xp = reinterpret_cast<const uint4 *>(xr + i * 16);
            const uint4 u0 = xp[0], u1 = xp[1];
            const uint32_t w[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
            float sum = 0.f;
#pragma unroll
            for (int q = 0; q < 8; ++q) sum += __uint_as_float(w[q] << 16) + __uint_as_float(w[q] & 0xffff0000u);
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            if ((i & 3) == 0) xtab[i >> 2] = sum;
        }
        __syncthreads();
    }
    // equal contiguous ranges of tile steps: the first (steps % nwarps) warps take one more
    const uint32_t warp = blockIdx.x * WC_WARPS + (threadIdx.x >> 5);
    const uint32_t nwarps = gridDim.x * WC_WARPS;
    const uint32_t steps = (uint32_t)(a.N / WC_TILE_N) * kchunks;
    const uint32_t base = steps / nwarps, rem = steps % nwarps;
    const uint32_t s_begin = warp * base + (warp < rem ? warp : rem);
    const uint32_t count = base + (warp < rem ? 1 : 0);
    if (count == 0) return;

    const uint32_t ones[4] = {0x3f803f80u, 0x3f803f80u, 0x3f803f80u, 0x3f803f80u};
    float acc[MB][4], xs[MB][4], tot[MB][4];
#pragma unroll
    for (int mb = 0; mb < MB; ++mb)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[mb][i] = xs[mb][i] = tot[mb][i] = 0.f;

    // activation rows this lane feeds into the B fragments (MMA column g of each block),
    // already offset to this lane's 16 k of a tile step
    const __nv_bfloat16 *xrow[MB];
    bool xok[MB];
#pragma unroll
    for (int mb = 0; mb < MB; ++mb) {
        const int64_t m = a.m0 + mb * 8 + g;
        xok[mb] = m < a.M;
        xrow[mb] = a.x + (xok[mb] ? m : 0) * a.x_ld + 16 * t;
    }

    uint32_t strip = s_begin / kchunks;
    uint32_t kc = s_begin - strip * kchunks;
    const uint32_t fold_steps = a.fold_k / WC_TILE_K;  // tile steps per quantisation group
    uint32_t grp = kc / fold_steps;                    // current K group (FASTQ)
    uint32_t kin = kc - grp * fold_steps;              // tile steps done inside it

    // FASTQ: the raw scale and zero-point bytes of the group being accumulated are requested
    // one group ahead (right after the previous fold), so that their latency is not paid at
    // the fold itself.
    uint32_t q_s0 = 0, q_s1 = 0, q_z0 = 0, q_z1 = 0;
    auto request_group = [&]() {
        if (FASTQ) {
            const uint32_t row = grp * (uint32_t)a.N + strip * WC_TILE_N + g;
            q_s0 = ((const uint16_t *)a.scale)[row];
            q_s1 = ((const uint16_t *)a.scale)[row + 8];
            q_z0 = ((const uint8_t *)a.zp)[row >> 1];
            q_z1 = ((const uint8_t *)a.zp)[(row + 8) >> 1];
        }
    };
    request_group();
    auto fold = [&]() {
        const uint32_t n0 = strip * WC_TILE_N + g;
        float s0, s1, c0, c1;
        if (FASTQ) {
            // n0 and n0 + 8 have the same parity: the same nibble of their bytes
            const uint32_t sh = (n0 & 1) * 4;
            s0 = __uint_as_float(q_s0 << 16);
            s1 = __uint_as_float(q_s1 << 16);
            c0 = a.nibble_offset + (float)((q_z0 >> sh) & 0xf);
            c1 = a.nibble_offset + (float)((q_z1 >> sh) & 0xf);
        } else {
            const uint32_t k_in_group = grp * a.fold_k; // any k of the group being closed
            wc_group_params<false>(a, grp, k_in_group, n0, s0, c0);
            wc_group_params<false>(a, grp, k_in_group, n0 + 8, s1, c1);
        }
#pragma unroll
        for (int mb = 0; mb < MB; ++mb) {
            tot[mb][0] = fmaf(s0, fmaf(-c0, xs[mb][0], acc[mb][0]), tot[mb][0]);
            tot[mb][1] = fmaf(s0, fmaf(-c0, xs[mb][1], acc[mb][1]), tot[mb][1]);
            tot[mb][2] = fmaf(s1, fmaf(-c1, xs[mb][2], acc[mb][2]), tot[mb][2]);
            tot[mb][3] = fmaf(s1, fmaf(-c1, xs[mb][3], acc[mb][3]), tot[mb][3]);
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[mb][i] = xs[mb][i] = 0.f;
        }
    };
    auto flush = [&]() {
        float *out = a.acc + (size_t)strip * WC_TILE_N + g;
#pragma unroll
        for (int mb = 0; mb < MB; ++mb) {
            const int64_t mA = a.m0 + mb * 8 + 2 * t, mB = mA + 1;
            if (mA < a.M) {
                atomicAdd(out + mA * a.N, tot[mb][0]);
                atomicAdd(out + mA * a.N + 8, tot[mb][2]);
            }
            if (mB < a.M) {
                atomicAdd(out + mB * a.N, tot[mb][1]);
                atomicAdd(out + mB * a.N + 8, tot[mb][3]);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) tot[mb][i] = 0.f;
        }
    };
    // one tile step on the 16 bytes of weights w4
    auto step = [&](const uint4 &w4) {
        uint4 xa[MB], xb[MB];
#pragma unroll
        for (int mb = 0; mb < MB; ++mb) {
            xa[mb] = make_uint4(0, 0, 0, 0);
            xb[mb] = xa[mb];
            if (xok[mb]) {
                const uint4 *xp = reinterpret_cast<const uint4 *>(xrow[mb] + kc * WC_TILE_K);
                xa[mb] = xp[0];
                xb[mb] = xp[1];
            }
        }
        if (XTAB) {
            // the row's sum over this step; only MMA column 0 (accumulator slots 0 and 2) is real
            const float sx = xtab[kc];
            xs[0][0] += sx;
            xs[0][2] += sx;
        }
        const uint32_t words[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t w = words[j];
            uint32_t af[4];
            af[0] = (w & 0x000f000fu) | 0x43004300u;
            af[1] = ((w >> 4) & 0x000f000fu) | 0x43004300u;
            af[2] = ((w >> 8) & 0x000f000fu) | 0x43004300u;
            af[3] = ((w >> 12) & 0x000f000fu) | 0x43004300u;
#pragma unroll
            for (int mb = 0; mb < MB; ++mb) {
                const uint32_t b0 = j == 0 ? xa[mb].x : j == 1 ? xa[mb].z : j == 2 ? xb[mb].x : xb[mb].z;
                const uint32_t b1 = j == 0 ? xa[mb].y : j == 1 ? xa[mb].w : j == 2 ? xb[mb].y : xb[mb].w;
                mma_bf16_16816(acc[mb], af, b0, b1);
                if (!XTAB) mma_bf16_16816(xs[mb], ones, b0, b1);
            }
        }
        const bool group_done = ++kin == fold_steps;
        if (group_done) {
            fold();
            kin = 0;
            ++grp;
        }
        if (++kc == kchunks) {
            // the last fold of the strip has happened (the fold period divides K)
            flush();
            kc = 0;
            grp = 0;
            ++strip;
        }
        if (group_done) request_group(); // for the group that starts now
    };

    // Four tile steps per iteration with the weights of the next four already requested:
    // 2 KiB in flight per warp, no register shuffling.
    const uint4 *wp = a.wei + (size_t)s_begin * 32 + lane;
    auto fetch = [&](uint32_t i, uint4 &r) {
        if (i < count) r = ldg_stream(wp + (size_t)i * 32);
    };
    uint4 r0 = make_uint4(0, 0, 0, 0), r1 = r0, r2 = r0, r3 = r0;
    fetch(0, r0);
    fetch(1, r1);
    fetch(2, r2);
    fetch(3, r3);
    uint32_t s = 0;
#pragma unroll 1
    for (; s + 4 <= count; s += 4) {
        step(r0);
        fetch(s + 4, r0);
        step(r1);
        fetch(s + 5, r1);
        step(r2);
        fetch(s + 6, r2);
        step(r3);
        fetch(s + 7, r3);
    }
    if (s < count) step(r0);
    if (s + 1 < count) step(r1);
    if (s + 2 < count) step(r2);
    if (kc != 0) {
        // the range ended inside a strip: close the open group, then publish
        if (kin != 0) fold();
        flush();
    }
}

// epilogue over the f32 partial sums: src scale, bias, post-ops, dst scale, store;
// leaves the scratch zeroed for the next execution
__global__ void __launch_bounds__(256) wc_epilogue_kernel(const __grid_constant__ b200_matmul_params_t p, float *acc) {
    const int64_t total = p.M * p.N;
    const float dst_inv = dst_scale_reciprocal(p);
    const float src_scale = p.src_scale.ptr ? load_f32(p.src_scale.dt, p.src_scale.ptr, 0) : 1.f;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        float d = acc[i];
        acc[i] = 0.f;
        if (p.src_scale.ptr) d = __fmul_rn(d, src_scale);
        finish_element(p, d, i / p.N, i % p.N, false, dst_inv);
    }
}

// activations of another float type -> bf16 rows (fpmath bf16 permits the down-conversion)
__global__ void __launch_bounds__(256) wc_convert_x_kernel(const void *src, int dt, int64_t ld, int64_t M, int64_t K,
        __nv_bfloat16 *dst) {
    const int64_t total = M * K;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t m = i / K, k = i % K;
        ((uint16_t *)dst)[i] = f32_to_bf16_bits(load_f32(dt, src, m * ld + k));
    }
}

// plain (K, N) 4-bit weights, two per byte along N -> B200_WEI_WC4_TILED.
// One thread per 32-bit output word.
__global__ void __launch_bounds__(256) wc_pack_kernel(const uint8_t *__restrict__ src, uint32_t *__restrict__ dst,
        int64_t K, int64_t N, int is_signed) {
    const int64_t nwords = K * N / 8;
    const int64_t kchunks = K / WC_TILE_K;
    for (int64_t wi = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; wi < nwords; wi += (int64_t)gridDim.x * blockDim.x) {
        const int j = (int)(wi & 3);
        const int lane = (int)((wi >> 2) & 31);
        const int64_t tile = wi >> 7;
        const int64_t kc = tile % kchunks, strip = tile / kchunks;
        const int g = lane >> 2, t = lane & 3;
        uint32_t word = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int p = i & 3, half = i >> 2;
            const int64_t n = strip * WC_TILE_N + g + 8 * (p & 1);
            const int64_t k = kc * WC_TILE_K + 16 * t + 4 * j + 2 * (p >> 1) + half;
            const int64_t e = k * N + n;
            uint32_t q = (src[e >> 1] >> ((e & 1) * 4)) & 0xf;
            if (is_signed) q ^= 8u; // two's complement nibble -> offset binary (value + 8)
            // nibble p goes to bits [4p, 4p+4) of the low half (even k) or the high half (odd k)
            word |= q << (4 * p + 16 * half);
        }
        dst[wi] = word;
    }
}

static inline size_t align256(size_t x) { return (x + 255) / 256 * 256; }

} // namespace b200

using namespace b200;

// bf16 scales and u4 zero-points, both [K / group][N] over the same K groups
static bool wc_fast_quant(const b200_matmul_params_t *p, int64_t gs, int64_t gz) {
    return p->wei_scale.ptr && p->wei_zp.ptr && p->wei_scale.dt == B200_DT_BF16 && p->wei_zp.dt == B200_DT_U4 && gs == gz
            && p->wei_scale.s0 == p->N && p->wei_scale.s1 == 1 && p->wei_zp.s0 == p->N && p->wei_zp.s1 == 1
            && p->N * (p->K / gs) < ((int64_t)1 << 31);
}

static void wc_launch_pass(const wc_args_t &a, int64_t rows, bool fastq, unsigned ctas, cudaStream_t cs) {
    const unsigned threads = WC_WARPS * 32;
    const bool xtab = rows == 1 && a.K <= 65536;
    if (fastq) {
        if (xtab) wc_gemv_kernel<1, true, true><<<ctas, threads, 0, cs>>>(a);
        else if (rows <= 8) wc_gemv_kernel<1, true, false><<<ctas, threads, 0, cs>>>(a);
        else if (rows <= 16) wc_gemv_kernel<2, true, false><<<ctas, threads, 0, cs>>>(a);
        else wc_gemv_kernel<4, true, false><<<ctas, threads, 0, cs>>>(a);
    } else {
        if (xtab) wc_gemv_kernel<1, false, true><<<ctas, threads, 0, cs>>>(a);
        else if (rows <= 8) wc_gemv_kernel<1, false, false><<<ctas, threads, 0, cs>>>(a);
        else if (rows <= 16) wc_gemv_kernel<2, false, false><<<ctas, threads, 0, cs>>>(a);
        else wc_gemv_kernel<4, false, false><<<ctas, threads, 0, cs>>>(a);
    }
}

// scratch layout of the wc kernel: [f32 acc M*N][bf16 x copy M*K if src is not bf16][packed weights if plain]
static void wc_scratch_layout(const b200_matmul_params_t *p, size_t *acc, size_t *xcopy, size_t *packed) {
    *acc = align256((size_t)p->M * p->N * sizeof(float));
    *xcopy = p->src_dt == B200_DT_BF16 ? 0 : align256((size_t)p->M * p->K * 2);
    *packed = p->wei_layout == B200_WEI_WC4_TILED ? 0 : align256((size_t)(p->K * p->N / 2));
}

extern "C" size_t b200_matmul_scratch_bytes(const b200_matmul_params_t *p, int kernel) {
    if (!p) return 0;
    if (kernel == 2) {
        size_t a, x, w;
        wc_scratch_layout(p, &a, &x, &w);
        return a + x + w;
    }
    return 0;
}

extern "C" int b200_wc_pack_launch(const void *src, void *dst, int64_t K, int64_t N, int32_t dt, b200_stream_t stream) {
    if (!src || !dst) return B200_ERR_BAD_ARG;
    if ((dt != B200_DT_U4 && dt != B200_DT_S4) || K % WC_TILE_K != 0 || N % WC_TILE_N != 0) return B200_ERR_UNSUPPORTED;
    const int64_t nwords = K * N / 8;
    if (nwords == 0) return 0;
    int64_t blocks = (nwords + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    wc_pack_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>((const uint8_t *)src, (uint32_t *)dst, K, N,
            dt == B200_DT_S4);
    return after_launch();
}

extern "C" int b200_matmul_wc_launch(const b200_matmul_params_t *p, b200_stream_t stream) {
    if (!p || !p->src || !p->wei || !p->dst) return B200_ERR_BAD_ARG;
    if (p->M <= 0 || p->N <= 0 || p->K <= 0) return p->M < 0 || p->N < 0 || p->K < 0 ? B200_ERR_BAD_ARG : 0;
    if (p->wei_dt != B200_DT_U4 && p->wei_dt != B200_DT_S4) return B200_ERR_UNSUPPORTED;
    if (!p->apply_to_int) return B200_ERR_UNSUPPORTED;
    if (p->src_dt != B200_DT_BF16 && p->src_dt != B200_DT_F16 && p->src_dt != B200_DT_F32) return B200_ERR_UNSUPPORTED;
    if (p->N % WC_TILE_N != 0 || p->K % WC_TILE_K != 0 || p->src_sk != 1 || p->dst_sn != 1) return B200_ERR_UNSUPPORTED;
    if (p->K > (int64_t)1 << 30 || (p->N / WC_TILE_N) * (p->K / WC_TILE_K) >= ((int64_t)1 << 31)) return B200_ERR_TOO_LARGE;
    if (p->wei_layout == B200_WEI_PLAIN && !(p->wei_sn == 1 && p->wei_sk == p->N)) return B200_ERR_UNSUPPORTED;
    if (p->wei_layout != B200_WEI_PLAIN && p->wei_layout != B200_WEI_WC4_TILED) return B200_ERR_UNSUPPORTED;
    if (p->src_zp.ptr || p->dst_zp.ptr) return B200_ERR_UNSUPPORTED;
    if (p->src_scale.ptr && (p->src_scale.s0 || p->src_scale.s1)) return B200_ERR_UNSUPPORTED;
    // K-group sizes: multiples of 16 that divide K, and one must divide the other
    int64_t gs = p->K, gz = p->K;
    if (p->wei_scale.ptr) {
        if (p->wei_scale.g1 != 1) return B200_ERR_UNSUPPORTED;
        if (p->wei_scale.s0) gs = p->wei_scale.g0;
    }
    if (p->wei_zp.ptr) {
        if (p->wei_zp.g1 != 1) return B200_ERR_UNSUPPORTED;
        if (p->wei_zp.s0) gz = p->wei_zp.g0;
    }
    // a tile step covers 64 k in a permuted order, so groups must be whole tile steps
    if (gs % WC_TILE_K || gz % WC_TILE_K || p->K % gs || p->K % gz) return B200_ERR_UNSUPPORTED;
    const int64_t fold_k = gs < gz ? gs : gz;
    if (gs % fold_k || gz % fold_k) return B200_ERR_UNSUPPORTED;
    // activations are read 16 bytes at a time
    if (p->src_dt == B200_DT_BF16 && (((uintptr_t)p->src & 15) || (p->src_sm & 7))) return B200_ERR_BAD_ARG;

    size_t acc_b, x_b, w_b;
    wc_scratch_layout(p, &acc_b, &x_b, &w_b);
    if (!p->scratch || p->scratch_bytes < acc_b + x_b + w_b) return B200_ERR_BAD_ARG;
    cudaStream_t cs = (cudaStream_t)stream;
    char *sc = (char *)p->scratch;
    float *acc = (float *)sc;
    const __nv_bfloat16 *x = (const __nv_bfloat16 *)p->src;
    int64_t x_ld = p->src_sm;
    if (x_b) {
        __nv_bfloat16 *xc = (__nv_bfloat16 *)(sc + acc_b);
        int64_t blocks = (p->M * p->K + 255) / 256;
        if (blocks > 148 * 8) blocks = 148 * 8;
        wc_convert_x_kernel<<<(unsigned)blocks, 256, 0, cs>>>(p->src, p->src_dt, p->src_sm, p->M, p->K, xc);
        int rc = after_launch();
        if (rc) return rc;
        x = xc;
        x_ld = p->K;
    }
    const void *wei = p->wei;
    if (w_b) {
        void *wp = sc + acc_b + x_b;
        int rc = b200_wc_pack_launch(p->wei, wp, p->K, p->N, p->wei_dt, stream);
        if (rc) return rc;
        wei = wp;
    }
    if (((uintptr_t)wei & 15)) return B200_ERR_BAD_ARG;
    if (!p->scratch_zeroed) {
        if (cudaMemsetAsync(acc, 0, (size_t)p->M * p->N * sizeof(float), cs) != cudaSuccess) return (int)cudaGetLastError();
    }

    wc_args_t a;
    a.wei = (const uint4 *)wei;
    a.x = x;
    a.x_ld = x_ld;
    a.acc = acc;
    a.M = p->M;
    a.N = p->N;
    a.K = p->K;
    a.scale = p->wei_scale.ptr;
    a.scale_dt = p->wei_scale.dt;
    a.scale_s0 = p->wei_scale.s0;
    a.scale_s1 = p->wei_scale.s1;
    a.scale_g0 = (uint32_t)gs;
    a.zp = p->wei_zp.ptr;
    a.zp_dt = p->wei_zp.dt;
    a.zp_s0 = p->wei_zp.s0;
    a.zp_s1 = p->wei_zp.s1;
    a.zp_g0 = (uint32_t)gz;
    a.fold_k = (uint32_t)fold_k;
    a.nibble_offset = p->wei_dt == B200_DT_S4 ? 136.f : 128.f;

    const bool fastq = wc_fast_quant(p, gs, gz);
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int64_t steps = (p->N / WC_TILE_N) * (p->K / WC_TILE_K);
    int64_t ctas = (int64_t)sms * 3;
    if (ctas * WC_WARPS > steps) ctas = (steps + WC_WARPS - 1) / WC_WARPS;
    // activation rows in passes of up to 32 (the weights are re-read from L2)
    for (int64_t m0 = 0; m0 < p->M; m0 += 32) {
        a.m0 = (int)m0;
        const int64_t rows = p->M - m0;
        wc_launch_pass(a, rows, fastq, (unsigned)ctas, cs);
        int rc = after_launch();
        if (rc) return rc;
    }
    int64_t eblocks = (p->M * p->N + 255) / 256;
    if (eblocks > (int64_t)sms * 8) eblocks = (int64_t)sms * 8;
    wc_epilogue_kernel<<<(unsigned)eblocks, 256, 0, cs>>>(*p, acc);
    return after_launch();
}

// ---- entry point that allocates nothing ---------------------------------------------------
//
// b200_matmul_wc_launch needs an f32 accumulation scratch that somebody has to
// allocate.  Some callers cannot: code that runs inside another framework's
// CUDA-graph capture or inside its memory-pool callbacks, plugins that are only
// handed device pointers by a host runtime that owns every allocation, and
// real-time decode loops that must not touch the allocator.  For them the same
// kernels are offered with the scratch in a fixed array that lives in the
// library's device image: every GPU that loads the library holds these 2 MiB
// until the process exits.
static constexpr size_t WC_STATIC_SCRATCH_BYTES = (size_t)2 << 20; // room for M * N <= 524288 partial sums
static __device__ __align__(256) unsigned char g_wc_static_scratch[WC_STATIC_SCRATCH_BYTES];

// In host code the array's name is only a handle for the runtime, not a device
// address.  The address is looked up once per device, with that device current.
static int wc_static_scratch_ptr(float **out) {
    static std::mutex mu;
    static float *ptrs[64] = {nullptr};
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return (int)cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> g(mu);
    if (!ptrs[dev]) {
        void *p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_wc_static_scratch);
        if (e != cudaSuccess) return (int)e;
        ptrs[dev] = (float *)p;
    }
    *out = ptrs[dev];
    return 0;
}

extern "C" size_t b200_matmul_wc_noalloc_max_bytes(void) {
    return WC_STATIC_SCRATCH_BYTES;
}

extern "C" int b200_matmul_wc_noalloc_launch(const b200_matmul_params_t *p, b200_stream_t stream) {
    if (!p || !p->src || !p->wei || !p->dst) return B200_ERR_BAD_ARG;
    if (p->M <= 0 || p->N <= 0 || p->K <= 0) return p->M < 0 || p->N < 0 || p->K < 0 ? B200_ERR_BAD_ARG : 0;
    // only the forms that need no other scratch: bf16 activations, weights already packed
    if (p->wei_dt != B200_DT_U4 && p->wei_dt != B200_DT_S4) return B200_ERR_UNSUPPORTED;
    if (!p->apply_to_int || p->src_dt != B200_DT_BF16 || p->wei_layout != B200_WEI_WC4_TILED) return B200_ERR_UNSUPPORTED;
    if (p->N % WC_TILE_N != 0 || p->K % WC_TILE_K != 0 || p->src_sk != 1 || p->dst_sn != 1) return B200_ERR_UNSUPPORTED;
    if (p->K > (int64_t)1 << 30 || (p->N / WC_TILE_N) * (p->K / WC_TILE_K) >= ((int64_t)1 << 31)) return B200_ERR_TOO_LARGE;
    if (p->src_zp.ptr || p->dst_zp.ptr) return B200_ERR_UNSUPPORTED;
    if (p->src_scale.ptr && (p->src_scale.s0 || p->src_scale.s1)) return B200_ERR_UNSUPPORTED;
    int64_t gs = p->K, gz = p->K;
    if (p->wei_scale.ptr) {
        if (p->wei_scale.g1 != 1) return B200_ERR_UNSUPPORTED;
        if (p->wei_scale.s0) gs = p->wei_scale.g0;
    }
    if (p->wei_zp.ptr) {
        if (p->wei_zp.g1 != 1) return B200_ERR_UNSUPPORTED;
        if (p->wei_zp.s0) gz = p->wei_zp.g0;
    }
    // a tile step covers 64 k in a permuted order, so groups must be whole tile steps
    if (gs % WC_TILE_K || gz % WC_TILE_K || p->K % gs || p->K % gz) return B200_ERR_UNSUPPORTED;
    const int64_t fold_k = gs < gz ? gs : gz;
    if (gs % fold_k || gz % fold_k) return B200_ERR_UNSUPPORTED;
    if (((uintptr_t)p->src & 15) || (p->src_sm & 7) || ((uintptr_t)p->wei & 15)) return B200_ERR_BAD_ARG;
    // the fixed array bounds the problem: M * N partial sums of 4 bytes
    if ((uint64_t)p->M * (uint64_t)p->N * sizeof(float) > WC_STATIC_SCRATCH_BYTES) return B200_ERR_TOO_LARGE;

    float *acc = nullptr;
    int rc = wc_static_scratch_ptr(&acc);
    if (rc) return rc;
    cudaStream_t cs = (cudaStream_t)stream;
    // the array keeps whatever the last call left behind: clear the part used now
    if (cudaMemsetAsync(acc, 0, (size_t)p->M * p->N * sizeof(float), cs) != cudaSuccess) return (int)cudaGetLastError();

    wc_args_t a;
    a.wei = (const uint4 *)p->wei;
    a.x = (const __nv_bfloat16 *)p->src;
    a.x_ld = p->src_sm;
    a.acc = acc;
    a.M = p->M;
    a.N = p->N;
    a.K = p->K;
    a.scale = p->wei_scale.ptr;
    a.scale_dt = p->wei_scale.dt;
    a.scale_s0 = p->wei_scale.s0;
    a.scale_s1 = p->wei_scale.s1;
    a.scale_g0 = (uint32_t)gs;
    a.zp = p->wei_zp.ptr;
    a.zp_dt = p->wei_zp.dt;
    a.zp_s0 = p->wei_zp.s0;
    a.zp_s1 = p->wei_zp.s1;
    a.zp_g0 = (uint32_t)gz;
    a.fold_k = (uint32_t)fold_k;
    a.nibble_offset = p->wei_dt == B200_DT_S4 ? 136.f : 128.f;

    const bool fastq = wc_fast_quant(p, gs, gz);
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int64_t steps = (p->N / WC_TILE_N) * (p->K / WC_TILE_K);
    int64_t ctas = (int64_t)sms * 3;
    if (ctas * WC_WARPS > steps) ctas = (steps + WC_WARPS - 1) / WC_WARPS;
    for (int64_t m0 = 0; m0 < p->M; m0 += 32) {
        a.m0 = (int)m0;
        const int64_t rows = p->M - m0;
        wc_launch_pass(a, rows, fastq, (unsigned)ctas, cs);
        rc = after_launch();
        if (rc) return rc;
    }
    int64_t eblocks = (p->M * p->N + 255) / 256;
    if (eblocks > (int64_t)sms * 8) eblocks = (int64_t)sms * 8;
    wc_epilogue_kernel<<<(unsigned)eblocks, 256, 0, cs>>>(*p, acc);
    return after_launch();
}
