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
//  * Work is split by bytes, not by tiles.  A unit is one or two tile steps (one
//    quantisation group where the group is 128 k).  Each CTA of a grid of one CTA
//    per SM takes a contiguous range of units -- whole strips of 16 output
//    columns when there are enough strips, an even share of all units otherwise
//    -- and each of its 16 warps a contiguous part of that range.
//  * Every warp streams its part through a private ring in shared memory filled
//    by asynchronous copies (cp.async, 16 bytes per lane and tile step, one commit
//    group per unit): about 100 KiB of weights in flight per SM without spending
//    registers on them.  Each lane copies exactly the bytes it will feed to the
//    MMAs itself, so a lane waits for its own copies only and the ring needs no
//    barrier.  A stage is refilled as soon as its unit has been folded in.
//  * A strip is usually shared by a few neighbouring warps.  Each leaves its
//    partial sums in its own slab of shared memory and adds its unit count to
//    the strip's counter; the warp that completes the count adds the slabs up and
//    applies the epilogue, so nobody waits for anybody.  A strip shared between
//    CTAs goes one level further the same way: red.global.add into the f32
//    scratch [M][N] plus a global per-strip counter, and the CTA that completes
//    it applies the epilogue and leaves scratch and counter zeroed.
#include <cstdlib>
#include <mutex>
#include <utility>
#include <vector>

#include "common.cuh"
#include "launch.hpp"

namespace b200 {

// warps per CTA (one CTA per SM): a single block of 8 rows leaves registers for 24
__host__ __device__ constexpr int wc_warps(int mb) { return mb == 1 ? 24 : 16; }
constexpr int WC_TILE_N = 16;         // output columns per tile (MMA M)
constexpr int WC_TILE_K = 64;         // k per 512-byte tile step
constexpr int WC_TILE_BYTES = 512;
constexpr int WC_MAX_STAGES = 16;     // ring stages per warp (512-byte units)
constexpr int WC_XTAB_MAX_BYTES = 40960;
__host__ __device__ constexpr int wc_ring_bytes(int mb) { return mb == 2 ? 8192 : 4096; } // per warp: 96 / 128 / 64 KiB per CTA

// n / d for any 32-bit n with one multiply-high, one subtract, two shifts and one add
// (round-up method of Granlund and Montgomery)
struct wc_div_t {
    uint32_t m, s1, s2;
};
__device__ __forceinline__ uint32_t wc_div(uint32_t n, const wc_div_t &d) {
    const uint32_t t = __umulhi(n, d.m);
    return (t + ((n - t) >> d.s1)) >> d.s2;
}

struct wc_args_t {
    const uint4 *wei;       // packed tiles
    const __nv_bfloat16 *x; // activations, row-major, converted to bf16 if needed
    int64_t x_ld;
    float *acc;             // scratch [M][N] f32, zero on entry
    uint32_t *done;         // scratch [N / 16]: units folded in per strip shared between CTAs, zero on entry
    int64_t M, N, K;
    int m0;                 // first activation row of this pass
    const void *scale; int scale_dt; int64_t scale_s0, scale_s1; uint32_t scale_g0; // g0: K-group size (K if none)
    const void *zp; int zp_dt; int64_t zp_s0, zp_s1; uint32_t zp_g0;
    float nibble_offset;    // 128 (u4) or 136 (s4 stored offset by 8)
    uint32_t kchunks;       // K / 64
    uint32_t ups;           // units per strip = kchunks / U
    uint32_t units;         // total units = (N / 16) * ups
    wc_div_t div_ups;       // division by ups
    wc_div_t div_fu;        // division by the number of units per quantisation group
    int group_is_unit;      // that number is 1
    int whole_strips;       // CTA ranges are whole strips
    uint32_t max_segs;      // upper bound of the strips one CTA touches (size of its counter array)
};

// d += a * b
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t wc_smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
// 16 bytes global -> shared, asynchronously, not kept in L1
__device__ __forceinline__ void wc_copy16(uint32_t dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void wc_copy_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int PENDING>
__device__ __forceinline__ void wc_copy_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(PENDING) : "memory");
}

// Scale and (128 + zero-point) of output column n for the K group that contains k: the
// general form, any supported type and group combination.
__device__ __forceinline__ void wc_group_params(const wc_args_t &a, uint32_t k, uint32_t n, float &s, float &c) {
    s = 1.f;
    c = a.nibble_offset;
    if (a.scale) s = load_f32(a.scale_dt, a.scale, (int64_t)(k / a.scale_g0) * a.scale_s0 + (int64_t)n * a.scale_s1);
    if (a.zp) c += (float)load_int(a.zp_dt, a.zp, (int64_t)(k / a.zp_g0) * a.zp_s0 + (int64_t)n * a.zp_s1);
}

// How a CTA's range of units [begin, begin + T) is cut into the contiguous parts of its warps.
struct wc_split_t {
    uint32_t begin, base, rem; // warp w: base + (w < rem) units from begin + w * base + min(w, rem)
    __device__ __forceinline__ uint32_t first(uint32_t w) const { return begin + w * base + (w < rem ? w : rem); }
    __device__ __forceinline__ uint32_t count(uint32_t w) const { return base + (w < rem ? 1 : 0); }
};

// Epilogue of the part [seg_lo, seg_hi) of strip `strip` that lies in this CTA's range, run
// by the warp that completed it.  Every warp whose part overlaps it has left its sums in one
// of its three slabs: slab 0 if the strip is the first one the warp touches, slab 1 if it is
// the last, slab 2 for a strip in between (which it then owns alone).  A slab is
// [MB][32 lanes][4], the accumulator fragment as it sat in registers: lane (g, t), slot e =
// row 2t + (e & 1) of the 8-row block, column 2g + (e >> 1) of the strip.
// If the part is the whole strip it is finished here: src scale, bias, post-ops, dst scale,
// conversion, store.  Otherwise the sums go into the global scratch, and the CTA that brings
// the strip's global unit count to a.ups finishes it from there and leaves scratch and
// counter zeroed.  Kept out of line so that its registers do not weigh on the streaming loop.
__device__ __noinline__ void wc_strip_epilogue(const b200_matmul_params_t &p, const wc_args_t &a, const float *slabs,
        uint32_t slab_floats, const uint2 *wspan, uint32_t nwarps, uint32_t strip, uint32_t seg_lo, uint32_t seg_hi,
        uint32_t rows, uint32_t lane) {
    // wspan[w] = (first, last) strip warp w touches, first > last if it has no units: one
    // lane per warp finds out who has a slab for this strip
    uint32_t who;
    {
        const uint2 span = lane < nwarps ? wspan[lane] : make_uint2(1, 0);
        who = __ballot_sync(0xffffffffu, span.x <= strip && strip <= span.y);
    }
    const float dst_inv = dst_scale_reciprocal(p);
    const float src_scale = p.src_scale.ptr ? load_f32(p.src_scale.dt, p.src_scale.ptr, 0) : 1.f;
    const uint32_t cells = rows * WC_TILE_N;
    const bool whole = seg_hi - seg_lo == a.ups;
    float *out = a.acc + (int64_t)a.m0 * a.N + (int64_t)strip * WC_TILE_N;
    for (uint32_t i = lane; i < cells; i += 32) {
        const uint32_t row = i / WC_TILE_N, col = i % WC_TILE_N;
        const uint32_t at = (((row >> 3) * 32 + (col >> 1) * 4 + ((row & 7) >> 1)) << 2) + (row & 1) + 2 * (col & 1);
        float d = 0.f;
        for (uint32_t m = who; m; m &= m - 1) {
            const uint32_t w = __ffs(m) - 1;
            const uint2 span = wspan[w];
            const uint32_t slot = strip == span.x ? 0 : (strip == span.y ? 1 : 2);
            d += slabs[(w * 3 + slot) * slab_floats + at];
        }
        if (whole) {
            if (p.src_scale.ptr) d = __fmul_rn(d, src_scale);
            finish_element(p, d, a.m0 + row, (int64_t)strip * WC_TILE_N + col, false, dst_inv);
        } else {
            atomicAdd(out + (int64_t)row * a.N + col, d);
        }
    }
    if (whole) return;
    __threadfence(); // the sums above are visible before the count below
    __syncwarp();
    uint32_t before = 0;
    if (lane == 0) before = atomicAdd(a.done + strip, seg_hi - seg_lo);
    before = __shfl_sync(0xffffffffu, before, 0);
    if (before + (seg_hi - seg_lo) != a.ups) return;
    __threadfence();
    for (uint32_t i = lane; i < cells; i += 32) {
        float *cell = out + (int64_t)(i / WC_TILE_N) * a.N + i % WC_TILE_N;
        float d = __ldcg(cell);
        *cell = 0.f;
        if (p.src_scale.ptr) d = __fmul_rn(d, src_scale);
        finish_element(p, d, a.m0 + i / WC_TILE_N, (int64_t)strip * WC_TILE_N + i % WC_TILE_N, false, dst_inv);
    }
    if (lane == 0) a.done[strip] = 0;
}

// MB    = number of 8-row activation blocks handled per pass (1, 2 or 4)
// FASTQ = bf16 scales and u4 zero-points, both [K / group][N] over the same groups (the
//         common decode configuration): one 32-bit and one 8-bit load per lane and unit
// XTAB  = sum_k x of every activation row over every tile step comes from a table the CTA
//         builds in shared memory; otherwise a second MMA with an all-ones A tile
//         accumulates it (K too large for the table)
// U     = tile steps per unit (2 when the quantisation group is a multiple of 128 k)
//
// One tile step = 16 output columns x 64 k = 512 bytes of weights = four MMA k-steps.  Within
// a step the MMA's k slots are permuted so that everything a lane needs is contiguous in
// memory: lane (g, t) owns k = 16 t + 4 j + {0,1,2,3} of MMA step j, i.e. 32 contiguous
// bytes of its activation row per tile step (two 128-bit loads), and the pack kernel lays
// the weight nibbles out for the same permutation.  A dot product does not care in which
// order k is visited, as long as both operands agree.  The MMA's rows g and g + 8 are output
// columns 2g and 2g + 1 of the strip, so that a lane's two scales are one 32-bit word and its
// two zero-points one byte.
//
// Dynamic shared memory: [rings W x RING][slabs W x 3 x SLAB][strip spans W]
// [strip counters max_segs][activation-sum table kchunks x R].
template <int MB, bool FASTQ, bool XTAB, int U>
__global__ void __launch_bounds__(wc_warps(MB) * 32, 1)
        wc_gemv_kernel(const __grid_constant__ wc_args_t a, const __grid_constant__ b200_matmul_params_t p) {
    constexpr int R = MB * 8;                         // activation rows per pass
    constexpr uint32_t W = wc_warps(MB);
    constexpr uint32_t RING = wc_ring_bytes(MB);      // bytes of weights in flight per warp
    constexpr uint32_t UNIT_BYTES = U * WC_TILE_BYTES;
    constexpr uint32_t S = RING / UNIT_BYTES;         // ring stages (a power of two)
    constexpr uint32_t SLAB = MB * 32 * 4;            // floats per slab
    static_assert(S <= WC_MAX_STAGES && (S & (S - 1)) == 0, "ring stages");
    extern __shared__ __align__(128) unsigned char wc_smem[];
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t g = lane >> 2, t = lane & 3;
    unsigned char *ring = wc_smem + warp * RING;
    float *slabs = reinterpret_cast<float *>(wc_smem + W * RING);                         // [W][3][SLAB]
    uint2 *wspan = reinterpret_cast<uint2 *>(slabs + W * 3 * SLAB);                       // [W]
    uint32_t *segcnt = reinterpret_cast<uint32_t *>(wspan + W);                           // [max_segs]
    float *xtab = reinterpret_cast<float *>(segcnt + a.max_segs);                         // [kchunks][R]
    const uint32_t rows = a.M - a.m0 < R ? (uint32_t)(a.M - a.m0) : (uint32_t)R;

    // This CTA's range of units [c_begin, c_begin + T), T >= 1.  a.whole_strips: the ranges are
    // whole strips (the grid has at most one CTA per strip); otherwise the units are split
    // evenly and a range may start and end inside a strip.
    uint32_t c_begin, T;
    {
        const uint32_t n = a.whole_strips ? a.units / a.ups : a.units;
        const uint32_t base = n / gridDim.x, rem = n % gridDim.x;
        c_begin = blockIdx.x * base + (blockIdx.x < rem ? blockIdx.x : rem);
        T = base + (blockIdx.x < rem ? 1 : 0);
        if (a.whole_strips) {
            c_begin *= a.ups;
            T *= a.ups;
        }
    }
    const uint32_t c_end = c_begin + T;
    const uint32_t first_strip = wc_div(c_begin, a.div_ups);
    // this warp's contiguous part [wb, wb + cw)
    wc_split_t split;
    split.begin = c_begin;
    split.base = T / W;
    split.rem = T % W;
    const uint32_t wb = split.first(warp), cw = split.count(warp);
    const uint32_t my_first = wc_div(wb, a.div_ups), my_last = cw ? wc_div(wb + cw - 1, a.div_ups) : my_first;
    if (lane == 0) wspan[warp] = cw ? make_uint2(my_first, my_last) : make_uint2(1, 0);

    // Ring: every lane copies, asynchronously, the 16 bytes of each tile step that it will
    // itself feed to the MMAs, so a lane only ever waits for its own copies and no barrier
    // is involved.  One commit group per unit, S units ahead.
    const unsigned char *wsrc = reinterpret_cast<const unsigned char *>(a.wei) + (size_t)wb * UNIT_BYTES + lane * 16;
    const uint32_t ring_s = wc_smem_u32(ring) + lane * 16;
    auto request = [&](uint32_t unit_index) {
        if (unit_index < cw) {
            const uint32_t dst = ring_s + (unit_index & (S - 1)) * UNIT_BYTES;
            const unsigned char *src = wsrc + (size_t)unit_index * UNIT_BYTES;
#pragma unroll
            for (int s = 0; s < U; ++s) wc_copy16(dst + s * WC_TILE_BYTES, src + s * WC_TILE_BYTES);
        }
        wc_copy_commit(); // also when nothing was requested: the group count is what the waits rely on
    };
#pragma unroll
    for (uint32_t s = 0; s < S; ++s) request(s);

    // while those copies fly: clear the strip counters, build the activation-sum table
    for (uint32_t i = threadIdx.x; i < a.max_segs; i += blockDim.x) segcnt[i] = 0;
    if (XTAB) {
        // thread i sums 16 consecutive activations of one row; four neighbours make one tile step
        const uint32_t pieces = rows * a.kchunks * 4;
        for (uint32_t i = threadIdx.x; i < (uint32_t)R * a.kchunks; i += blockDim.x)
            if (i >= rows * a.kchunks) xtab[(i % a.kchunks) * R + i / a.kchunks] = 0.f; // rows past the last
        for (uint32_t i = threadIdx.x; i < pieces; i += blockDim.x) {
            const uint32_t cell = i >> 2, row = cell / a.kchunks, kc = cell - row * a.kchunks;
            const uint4 *xp = reinterpret_cast<const uint4 *>(
                    a.x + (int64_t)(a.m0 + row) * a.x_ld + (int64_t)kc * WC_TILE_K + (i & 3) * 16);
            const uint4 u0 = xp[0], u1 = xp[1];
            const uint32_t w[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
            float sum = 0.f;
#pragma unroll
            for (int q = 0; q < 8; ++q) sum += __uint_as_float(w[q] << 16) + __uint_as_float(w[q] & 0xffff0000u);
            // pieces is a multiple of 4, not of 32: only the four lanes of a tile step take part
            const uint32_t quad = 0xfu << (lane & 28);
            sum += __shfl_xor_sync(quad, sum, 1);
            sum += __shfl_xor_sync(quad, sum, 2);
            if ((i & 3) == 0) xtab[kc * R + row] = sum;
        }
    }
    __syncthreads();

    // activation rows this lane feeds into the B fragments (MMA column g of each block),
    // already offset to this lane's 16 k of a tile step.  Columns past the last row re-read
    // the last row: an MMA column only ever reaches its own accumulator column, and those
    // are never stored.
    const __nv_bfloat16 *xrow[MB];
#pragma unroll
    for (int mb = 0; mb < MB; ++mb) {
        const int64_t m = a.m0 + mb * 8 + g;
        xrow[mb] = a.x + (m < a.M ? m : a.M - 1) * a.x_ld + 16 * t;
    }

    float tot[MB][4];
#pragma unroll
    for (int mb = 0; mb < MB; ++mb)
#pragma unroll
        for (int i = 0; i < 4; ++i) tot[mb][i] = 0.f;

    uint32_t strip = my_first, kq = wb - my_first * a.ups; // position of the unit being consumed
    uint32_t in_strip = 0;                                  // units of `strip` folded into tot

    // Publish this warp's sums of `strip`; the warp that completes the strip's count inside
    // the CTA adds all slabs up and runs the epilogue.
    auto close_strip = [&]() {
        const uint32_t slot = strip == my_first ? 0 : (strip == my_last ? 1 : 2);
        float4 *mine = reinterpret_cast<float4 *>(slabs + (warp * 3 + slot) * SLAB) + lane;
#pragma unroll
        for (int mb = 0; mb < MB; ++mb) {
            mine[mb * 32] = make_float4(tot[mb][0], tot[mb][1], tot[mb][2], tot[mb][3]);
#pragma unroll
            for (int i = 0; i < 4; ++i) tot[mb][i] = 0.f;
        }
        __threadfence_block();
        __syncwarp();
        const uint32_t s_lo = strip * a.ups, s_hi = s_lo + a.ups;
        const uint32_t seg_lo = s_lo > c_begin ? s_lo : c_begin, seg_hi = s_hi < c_end ? s_hi : c_end;
        uint32_t before = 0;
        if (lane == 0) before = atomicAdd(&segcnt[strip - first_strip], in_strip);
        before = __shfl_sync(0xffffffffu, before, 0);
        if (before + in_strip == seg_hi - seg_lo) {
            __threadfence_block();
            wc_strip_epilogue(p, a, slabs, SLAB, wspan, W, strip, seg_lo, seg_hi, rows, lane);
        }
        in_strip = 0;
    };

    const uint32_t ones[4] = {0x3f803f80u, 0x3f803f80u, 0x3f803f80u, 0x3f803f80u};

    // raw scale / zero-point words of a unit (FASTQ)
    auto load_q = [&](uint32_t qstrip, uint32_t qkq, uint32_t &qs, uint32_t &qz) {
        if (FASTQ) {
            const uint32_t grp = a.group_is_unit ? qkq : wc_div(qkq, a.div_fu);
            const uint32_t row = grp * (uint32_t)a.N + qstrip * WC_TILE_N + 2 * g; // even
            qs = *reinterpret_cast<const uint32_t *>((const uint16_t *)a.scale + row);
            qz = ((const uint8_t *)a.zp)[row >> 1];
        }
    };
    // position one unit further
    auto step_pos = [&](uint32_t &ps, uint32_t &pk) {
        if (++pk == a.ups) {
            pk = 0;
            ++ps;
        }
    };

    // scale / zero-point words are requested two units ahead
    uint32_t qs0 = 0, qz0 = 0, qs1 = 0, qz1 = 0;
    uint32_t pstrip = strip, pkq = kq; // position of the unit whose words are requested next
    if (cw > 0) load_q(pstrip, pkq, qs0, qz0);
    step_pos(pstrip, pkq);
    if (cw > 1) load_q(pstrip, pkq, qs1, qz1);
    step_pos(pstrip, pkq);

    uint32_t n = 0;
    // one unit: wait for its stage, U tile steps of MMAs, fold, refill the stage
    auto unit = [&](uint32_t qs, uint32_t qz) {
        const uint32_t stage = n & (S - 1);
        wc_copy_wait<S - 1>(); // all but the S - 1 newest groups have landed: unit n is there
        const uint4 *sp = reinterpret_cast<const uint4 *>(ring + stage * UNIT_BYTES) + lane;
        float acc[MB][4], xs[MB][4]; // xs: [0] = sum of row 2t, [1] = sum of row 2t + 1 (XTAB)
#pragma unroll
        for (int mb = 0; mb < MB; ++mb)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[mb][e] = xs[mb][e] = 0.f;
        auto tile_step = [&](const uint4 wv, const uint32_t kc) {
            uint4 xa[MB], xb[MB];
#pragma unroll
            for (int mb = 0; mb < MB; ++mb) {
                const uint4 *xp = reinterpret_cast<const uint4 *>(xrow[mb] + (size_t)kc * WC_TILE_K);
                xa[mb] = xp[0];
                xb[mb] = xp[1];
                if (XTAB) {
                    const float2 sx = *reinterpret_cast<const float2 *>(xtab + kc * R + mb * 8 + 2 * t);
                    xs[mb][0] += sx.x;
                    xs[mb][1] += sx.y;
                }
            }
            // four MMA k-steps: word q of the lane's 16 bytes against activation words 2q and 2q + 1
#define WC_MMA_STEP(WORD, B0, B1)                                              \
    {                                                                          \
        const uint32_t v = (WORD);                                             \
        uint32_t af[4];                                                        \
        af[0] = (v & 0x000f000fu) | 0x43004300u;                               \
        af[1] = ((v >> 4) & 0x000f000fu) | 0x43004300u;                        \
        af[2] = ((v >> 8) & 0x000f000fu) | 0x43004300u;                        \
        af[3] = ((v >> 12) & 0x000f000fu) | 0x43004300u;                       \
        _Pragma("unroll") for (int mb = 0; mb < MB; ++mb) {                    \
            mma_bf16_16816(acc[mb], af, (B0), (B1));                           \
            if (!XTAB) mma_bf16_16816(xs[mb], ones, (B0), (B1));               \
        }                                                                      \
    }
            WC_MMA_STEP(wv.x, xa[mb].x, xa[mb].y)
            WC_MMA_STEP(wv.y, xa[mb].z, xa[mb].w)
            WC_MMA_STEP(wv.z, xb[mb].x, xb[mb].y)
            WC_MMA_STEP(wv.w, xb[mb].z, xb[mb].w)
#undef WC_MMA_STEP
        };
        tile_step(sp[0], kq * U);
        if (U == 2) tile_step(sp[32 * (U - 1)], kq * U + 1);

        float s0, s1, c0, c1;
        if (FASTQ) {
            s0 = __uint_as_float(qs << 16);
            s1 = __uint_as_float(qs & 0xffff0000u);
            c0 = a.nibble_offset + (float)(qz & 0xf);
            c1 = a.nibble_offset + (float)((qz >> 4) & 0xf);
        } else {
            const uint32_t n0 = strip * WC_TILE_N + 2 * g, k = kq * (U * WC_TILE_K);
            wc_group_params(a, k, n0, s0, c0);
            wc_group_params(a, k, n0 + 1, s1, c1);
        }
#pragma unroll
        for (int mb = 0; mb < MB; ++mb) {
            // accumulator slots: [0] (row 2t, col 2g), [1] (row 2t+1, col 2g), [2] (row 2t, col 2g+1), [3] (row 2t+1, col 2g+1);
            // without the table the all-ones MMA left the row sums in xs[.][0] and xs[.][1] as well
            const float xe = xs[mb][0], xo = xs[mb][1];
            tot[mb][0] = fmaf(s0, fmaf(-c0, xe, acc[mb][0]), tot[mb][0]);
            tot[mb][1] = fmaf(s0, fmaf(-c0, xo, acc[mb][1]), tot[mb][1]);
            tot[mb][2] = fmaf(s1, fmaf(-c1, xe, acc[mb][2]), tot[mb][2]);
            tot[mb][3] = fmaf(s1, fmaf(-c1, xo, acc[mb][3]), tot[mb][3]);
        }
        // the stage's bytes have been consumed by the MMAs above: request the unit S further on
        request(n + S);
        ++n;
        ++in_strip;
        if (++kq == a.ups) {
            close_strip();
            kq = 0;
            ++strip;
        }
    };

#pragma unroll 1
    while (n < cw) {
        unit(qs0, qz0);
        if (n + 1 < cw) load_q(pstrip, pkq, qs0, qz0); // for unit n + 1 after the increment above, i.e. two ahead
        step_pos(pstrip, pkq);
        if (n >= cw) break;
        unit(qs1, qz1);
        if (n + 1 < cw) load_q(pstrip, pkq, qs1, qz1);
        step_pos(pstrip, pkq);
    }
    wc_copy_wait<0>();
    if (in_strip) close_strip();
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
            const int64_t n = strip * WC_TILE_N + 2 * g + (p & 1);
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


// ---- streaming form of the decode kernel ------------------------------------------------------
//
// The kernel above has every lane fetch its own weights with cp.async: correct and simple, but
// 40 % of its instructions are copy bookkeeping, and at one byte of weights per two multiply-adds
// the instruction issue rate, not HBM, bounds it.  This form moves the stream to the copy engine
// and fixes every warp's K range, so that the activations and everything derived from them stay
// in registers:
//
//  * A chunk is one strip of 16 output columns x C = 16 * TPW tile steps of K (TPW = 4, 2 or 1:
//    8 to 32 KiB, contiguous in the tiled layout).  When K is longer than a chunk the strip has
//    several parts; chunks are numbered part-major, so a CTA's contiguous range of chunks keeps
//    the same part (the same K range) almost throughout.
//  * One producer thread streams the CTA's chunks with cp.async.bulk into a ring of shared-memory
//    stages (full / empty mbarriers), a few copies of 8 KiB per chunk.
//  * Consumer warp w of 16 owns tile steps [w * TPW, (w + 1) * TPW) of every chunk: its
//    activation fragments (MB * TPW * 8 registers), their row sums per quantisation group and the
//    group indices are loaded once per K part.  Per tile step it issues one 128-bit shared-memory
//    load, the nibble unpack (7 logic operations per 8 weights) and the MMAs -- no addressing, no
//    activation loads, no copy instructions.
//  * The 16 partial sums of a strip (one per warp) go through double-buffered slabs to one
//    epilogue warp per 8 activation rows, which adds them up and finishes the strip, so a
//    consumer never waits for another consumer.
//  * The CTA's range is cut in quarter chunks (4 warps' worth), which balances the grid to within
//    one quarter chunk; a strip that is not wholly inside one CTA (range ends, several K parts) is
//    completed through the f32 scratch and the per-strip counter like in the kernel above.
constexpr int WS_WARPS = 16;
constexpr int WS_MAX_STAGES = 16;
constexpr uint32_t WS_WAIT_TRIES = 1u << 20; // bounded waits: a million suspended waits of up to a microsecond
constexpr uint32_t WS_ST_FULL = 0x100, WS_ST_EMPTY = 0x200, WS_ST_SLAB_FULL = 0x400, WS_ST_SLAB_EMPTY = 0x800;
__host__ __device__ constexpr int ws_threads(int mb) { return (WS_WARPS + 1 + mb) * 32; }

struct ws_ctrl_t {
    uint64_t full[WS_MAX_STAGES], empty[WS_MAX_STAGES];
    uint64_t slab_full[2], slab_empty[2];
    volatile uint32_t abort;
};

struct ws_args_t {
    const unsigned char *wei;
    const __nv_bfloat16 *x;
    int64_t x_ld;
    float *acc;
    uint32_t *done;
    int64_t M, N;
    int m0;
    const void *scale; int scale_dt; int64_t scale_s0, scale_s1; uint32_t scale_g0;
    const void *zp; int zp_dt; int64_t zp_s0, zp_s1; uint32_t zp_g0;
    float nibble_offset;
    uint32_t kchunks;   // tile steps per strip
    uint32_t strips;    // N / 16
    uint32_t parts;     // K parts per strip
    uint32_t quarters;  // strips * parts * 4: the units the grid divides
    uint32_t stages;    // ring depth
    int plain_bf16;     // dst is bf16 with even pitch and nothing between the sum and the store: two columns per 32-bit store
    int simple;         // no post-ops, f32 / bf16 bias or none, f32 / bf16 dst: ws_finish_simple applies
    wc_div_t div_strips, div_fold; // division by strips and by the tile steps of a quantisation group
};

__device__ __forceinline__ void ws_mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(wc_smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void ws_mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(wc_smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void ws_mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(wc_smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool ws_mbar_try(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(wc_smem_u32(bar)), "r"(parity), "r"(1000u)
            : "memory");
    return ok != 0;
}
// bounded wait (of the order of a second); false when it ran out or another role gave up.
// The loop is out of line: the common case is one successful try.
__device__ __noinline__ bool ws_wait_slow(uint64_t *bar, uint32_t parity, ws_ctrl_t *c, uint32_t *status, uint32_t code) {
    for (uint32_t i = 0; i < WS_WAIT_TRIES; ++i) {
        if (ws_mbar_try(bar, parity)) return true;
        if (c->abort) return false;
    }
    c->abort = 1;
    if (status) atomicOr(status, code);
    return false;
}
__device__ __forceinline__ bool ws_wait(uint64_t *bar, uint32_t parity, ws_ctrl_t *c, uint32_t *status, uint32_t code) {
    if (ws_mbar_try(bar, parity)) return true;
    return ws_wait_slow(bar, parity, c, status, code);
}
// contiguous global -> shared copy by the copy engine; its bytes are counted on the barrier
__device__ __forceinline__ void ws_bulk_copy(uint32_t dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
                 "r"(bytes), "r"(wc_smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ void ws_group_params(const ws_args_t &a, uint32_t k, uint32_t n, float &s, float &c) {
    s = 1.f;
    c = a.nibble_offset;
    if (a.scale) s = load_f32(a.scale_dt, a.scale, (int64_t)(k / a.scale_g0) * a.scale_s0 + (int64_t)n * a.scale_s1);
    if (a.zp) c += (float)load_int(a.zp_dt, a.zp, (int64_t)(k / a.zp_g0) * a.zp_s0 + (int64_t)n * a.zp_s1);
}

// Everything behind the sum of one dst element in its general form (bias, any post-op chain,
// destination scale, any destination type).  One out-of-line copy: inlined at every call site the
// interpreter of the post-op chain -- some 40 KiB of code -- made the kernel a quarter of a megabyte,
// and a kernel that runs for a few microseconds pays for every instruction-cache line it touches.
__device__ __noinline__ void ws_finish(const b200_matmul_params_t &p, float d, int64_t m, int64_t n, float src_scale,
        float dst_inv) {
    if (p.src_scale.ptr) d = __fmul_rn(d, src_scale);
    finish_element(p, d, m, n, false, dst_inv);
}

// The same for the configurations a decode layer usually has -- no post-ops, f32 / bf16 bias or
// none, f32 / bf16 destination: a handful of instructions, inlined.
__device__ __forceinline__ void ws_finish_simple(const b200_matmul_params_t &p, float d, int64_t m, int64_t n, float src_scale,
        float dst_inv) {
    if (p.src_scale.ptr) d = __fmul_rn(d, src_scale);
    if (p.bias) {
        const int64_t bo = m * p.bias_sm + n * p.bias_sn;
        d = __fadd_rn(d, p.bias_dt == B200_DT_F32 ? ((const float *)p.bias)[bo]
                                                   : __uint_as_float((uint32_t)((const uint16_t *)p.bias)[bo] << 16));
    }
    if (p.dst_scale.ptr) d = __fmul_rn(d, dst_inv);
    const int64_t doff = m * p.dst_sm + n * p.dst_sn;
    if (p.dst_dt == B200_DT_F32) ((float *)p.dst)[doff] = d;
    else ((uint16_t *)p.dst)[doff] = f32_to_bf16_bits(d);
}

// the chunk sequence of one CTA: chunk i of its range -> (part, strip) and the quarters [qlo, qhi) it owns
struct ws_range_t {
    uint32_t b, e;        // quarter units [b, e)
    uint32_t first, n;    // first chunk index, number of chunks
    __device__ __forceinline__ void init(const ws_args_t &a) {
        const uint32_t base = a.quarters / gridDim.x, rem = a.quarters % gridDim.x;
        b = blockIdx.x * base + (blockIdx.x < rem ? blockIdx.x : rem);
        e = b + base + (blockIdx.x < rem ? 1 : 0);
        first = b >> 2;
        n = e > b ? ((e - 1) >> 2) - first + 1 : 0;
    }
    // quarters [qlo, qhi) of the k-th chunk of the range that belong to this CTA
    __device__ __forceinline__ uint32_t qlo(uint32_t k) const { return k == 0 ? (b & 3) : 0; }
    __device__ __forceinline__ uint32_t qhi(uint32_t k) const { return k + 1 == n ? ((e - 1) & 3) + 1 : 4; }
};

// Order in which a CTA takes the chunks of its range: the last one first, then the others in
// ascending order.  The chunks a range shares with its neighbours are its first and its last;
// their sums travel through global memory (atomics, a fence, a counter round trip), and taken
// first that latency passes while the whole chunks are processed instead of ending the kernel.
struct ws_walk_t {
    uint32_t k;    // index of the current chunk inside the range
    uint32_t q, s; // its K part and strip
    __device__ __forceinline__ void start(const ws_args_t &a, const ws_range_t &rg) {
        k = rg.n ? rg.n - 1 : 0;
        const uint32_t idx = rg.first + k;
        q = wc_div(idx, a.div_strips);
        s = idx - q * a.strips;
    }
    // the position after this one (step i -> i + 1 of the walk)
    __device__ __forceinline__ ws_walk_t next(const ws_args_t &a, const ws_range_t &rg, uint32_t i) const {
        ws_walk_t r;
        if (i == 0) {
            r.k = 0;
            r.q = wc_div(rg.first, a.div_strips);
            r.s = rg.first - r.q * a.strips;
        } else {
            r.k = k + 1;
            r.q = q;
            r.s = s + 1;
            if (r.s == a.strips) {
                r.s = 0;
                ++r.q;
            }
        }
        return r;
    }
};

// MB: 8-row activation blocks per pass; TPW: tile steps per warp and chunk; FE: tile steps per
// fold (the quantisation group, or all TPW when the group is longer); FASTQ: bf16 scales and u4
// zero-points over the same groups, fetched as one 32-bit and one 8-bit load per lane and fold.
template <int MB, int TPW, int FE, bool FASTQ>
__global__ void __launch_bounds__(ws_threads(MB), 1)
        wc_stream_kernel(const __grid_constant__ ws_args_t a, const __grid_constant__ b200_matmul_params_t p) {
    constexpr uint32_t C = WS_WARPS * TPW;              // tile steps per chunk
    constexpr uint32_t CH = C * WC_TILE_BYTES;          // bytes per chunk = per ring stage
    constexpr uint32_t QB = CH / 4;                     // bytes per quarter chunk
    constexpr int NF = TPW / FE;                        // folds per warp and chunk
    extern __shared__ __align__(128) unsigned char wc_smem[];
    const uint32_t S = a.stages;
    unsigned char *ring = wc_smem;
    float4 *slabs = reinterpret_cast<float4 *>(wc_smem + (size_t)S * CH);                       // [2][16][MB][32]
    ws_ctrl_t *ctrl = reinterpret_cast<ws_ctrl_t *>(wc_smem + (size_t)S * CH + 2 * WS_WARPS * MB * 32 * sizeof(float4));
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t rows = a.M - a.m0 < MB * 8 ? (uint32_t)(a.M - a.m0) : (uint32_t)(MB * 8);
    const uint32_t nblk = (rows + 7) / 8;

    ws_range_t rg;
    rg.init(a);
    // The consumers' activation fragments.  The loads of the first K part are issued before
    // anything else in the kernel -- ahead of the barrier set-up and of the producer's flood of
    // weight requests, behind which they would otherwise queue.
    uint32_t xr[MB][TPW][8];
    auto fetch_x = [&](uint32_t q) {
        const uint32_t g = lane >> 2, t = lane & 3;
#pragma unroll
        for (int mb = 0; mb < MB; ++mb) {
            const int64_t m = a.m0 + mb * 8 + g;
            const __nv_bfloat16 *xrow = a.x + (m < a.M ? m : a.M - 1) * a.x_ld + 16 * t;
#pragma unroll
            for (int j = 0; j < TPW; ++j) {
                const uint4 *xp = reinterpret_cast<const uint4 *>(xrow + (size_t)(q * C + warp * TPW + j) * WC_TILE_K);
                const uint4 u0 = xp[0], u1 = xp[1];
                xr[mb][j][0] = u0.x; xr[mb][j][1] = u0.y; xr[mb][j][2] = u0.z; xr[mb][j][3] = u0.w;
                xr[mb][j][4] = u1.x; xr[mb][j][5] = u1.y; xr[mb][j][6] = u1.z; xr[mb][j][7] = u1.w;
            }
        }
    };
    uint32_t cur_q = 0xffffffffu;
    if (warp < WS_WARPS && rg.n > 0) {
        ws_walk_t w0;
        w0.start(a, rg);
        fetch_x(w0.q);
        cur_q = w0.q;
    }

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < S; ++s) {
            ws_mbar_init(&ctrl->full[s], 1);
            ws_mbar_init(&ctrl->empty[s], WS_WARPS);
        }
        for (int i = 0; i < 2; ++i) {
            ws_mbar_init(&ctrl->slab_full[i], WS_WARPS);
            ws_mbar_init(&ctrl->slab_empty[i], MB);
        }
        ctrl->abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    if (warp == WS_WARPS) {
        // ---------------- producer ----------------
        if (lane == 0) {
            uint32_t issued = 0;
            ws_walk_t w;
            w.start(a, rg);
            uint32_t st = 0, ph = 1; // stage of step i and the parity of its previous release
            for (uint32_t i = 0; i < rg.n; ++i) {
                if (i >= S && !ws_wait(&ctrl->empty[st], ph, ctrl, p.status, WS_ST_EMPTY)) break;
                const uint32_t qlo = rg.qlo(w.k), qhi = rg.qhi(w.k), q = w.q, s = w.s;
                const unsigned char *src = a.wei + ((size_t)s * a.kchunks + (size_t)q * C) * WC_TILE_BYTES + (size_t)qlo * QB;
                const uint32_t dst = wc_smem_u32(ring + (size_t)st * CH) + qlo * QB;
                ws_mbar_expect_tx(&ctrl->full[st], (qhi - qlo) * QB);
                if (QB >= 4096) {
                    for (uint32_t h = 0; h < qhi - qlo; ++h) ws_bulk_copy(dst + h * QB, src + (size_t)h * QB, QB, &ctrl->full[st]);
                } else {
                    ws_bulk_copy(dst, src, (qhi - qlo) * QB, &ctrl->full[st]);
                }
                issued = i + 1;
                w = w.next(a, rg, i);
                if (++st == S) {
                    st = 0;
                    ph ^= 1;
                }
            }
            // every copy issued must have landed before the CTA may exit
            for (uint32_t j = issued > S ? issued - S : 0; j < issued; ++j) {
                const uint32_t st = j % S, par = (j / S) & 1;
                for (uint32_t t = 0; t < WS_WAIT_TRIES; ++t)
                    if (ws_mbar_try(&ctrl->full[st], par)) break;
            }
        }
    } else if (warp < WS_WARPS) {
        // ---------------- consumers ----------------
        const uint32_t g = lane >> 2, t = lane & 3;
        float xf[MB][NF][2];       // sums of the fragments per fold: rows 2t and 2t + 1 of the block
        uint32_t kfold[NF];        // first k of each fold
        uint32_t sum_q = 0xffffffffu; // the K part xf and kfold belong to
        auto sum_x = [&](uint32_t q) {
#pragma unroll
            for (int f = 0; f < NF; ++f) kfold[f] = (q * C + warp * TPW + f * FE) * WC_TILE_K;
#pragma unroll
            for (int mb = 0; mb < MB; ++mb) {
                float part[TPW];
#pragma unroll
                for (int j = 0; j < TPW; ++j) {
                    float sum = 0.f;
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        sum += __uint_as_float(xr[mb][j][i] << 16) + __uint_as_float(xr[mb][j][i] & 0xffff0000u);
                    // the four lanes of a group hold the four quarters of the row's 64 k
                    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
                    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
                    part[j] = sum; // sum of row g of the block over tile step j
                }
#pragma unroll
                for (int f = 0; f < NF; ++f) {
                    float fs = 0.f;
#pragma unroll
                    for (int j = 0; j < FE; ++j) fs += part[f * FE + j];
                    // accumulator slots of this lane belong to rows 2t and 2t + 1
                    xf[mb][f][0] = __shfl_sync(0xffffffffu, fs, (2 * t) * 4);
                    xf[mb][f][1] = __shfl_sync(0xffffffffu, fs, (2 * t + 1) * 4);
                }
            }
        };
        // scale / zero-point words of a chunk's folds (FASTQ), requested one chunk ahead
        uint32_t qs[NF], qz[NF], qs_n[NF], qz_n[NF], grow_n[NF]; // grow_n: (group index) * N + 2g of each fold of part gq
        uint32_t gq = 0xffffffffu;
        auto load_q = [&](uint32_t q, uint32_t s, uint32_t (&os)[NF], uint32_t (&oz)[NF]) {
            if (!FASTQ) return;
            if (q != gq) {
#pragma unroll
                for (int f = 0; f < NF; ++f) grow_n[f] = wc_div(q * C + warp * TPW + f * FE, a.div_fold) * (uint32_t)a.N + 2 * g;
                gq = q;
            }
#pragma unroll
            for (int f = 0; f < NF; ++f) {
                const uint32_t row = grow_n[f] + s * WC_TILE_N; // even
                os[f] = *reinterpret_cast<const uint32_t *>((const uint16_t *)a.scale + row);
                oz[f] = ((const uint8_t *)a.zp)[row >> 1];
            }
        };
        ws_walk_t w;
        w.start(a, rg);
#pragma unroll
        for (int f = 0; f < NF; ++f) qs[f] = qz[f] = qs_n[f] = qz_n[f] = grow_n[f] = 0;
        if (rg.n > 0) load_q(w.q, w.s, qs_n, qz_n);
        const uint32_t quarter = warp >> 2;
        bool ok = true;
        uint32_t st = 0, ph = 0; // ring stage of chunk i and the parity of its arrival
#pragma unroll 1
        for (uint32_t i = 0; i < rg.n; ++i) {
            const uint32_t q = w.q, s = w.s;
            if (q != cur_q) {
                fetch_x(q);
                cur_q = q;
            }
            if (q != sum_q) {
                sum_x(q);
                sum_q = q;
            }
#pragma unroll
            for (int f = 0; f < NF; ++f) {
                qs[f] = qs_n[f];
                qz[f] = qz_n[f];
            }
            // position of the next chunk, and its group parameters
            const ws_walk_t wn = w.next(a, rg, i);
            if (i + 1 < rg.n) load_q(wn.q, wn.s, qs_n, qz_n);
            const bool active = quarter >= rg.qlo(w.k) && quarter < rg.qhi(w.k);
            ok = ws_wait(&ctrl->full[st], ph, ctrl, p.status, WS_ST_FULL);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            float tot[MB][4];
#pragma unroll
            for (int mb = 0; mb < MB; ++mb)
#pragma unroll
                for (int e = 0; e < 4; ++e) tot[mb][e] = 0.f;
            if (active) {
                const uint4 *sp = reinterpret_cast<const uint4 *>(ring + (size_t)st * CH + (size_t)(warp * TPW) * WC_TILE_BYTES) + lane;
#pragma unroll
                for (int f = 0; f < NF; ++f) {
                    // The MMAs of a fold go to NA independent accumulators (one per word of a
                    // lane's 16 bytes while registers allow): a single accumulator would chain all
                    // of them, and the latency of that chain, not any pipe, then sets the pace.
                    constexpr int NA = MB == 1 ? 4 : (MB == 2 ? 2 : 1);
                    float accs[NA][MB][4];
#pragma unroll
                    for (int u = 0; u < NA; ++u)
#pragma unroll
                        for (int mb = 0; mb < MB; ++mb)
#pragma unroll
                            for (int e = 0; e < 4; ++e) accs[u][mb][e] = 0.f;
#pragma unroll
                    for (int jj = 0; jj < FE; ++jj) {
                        const int j = f * FE + jj;
                        const uint4 wv = sp[j * 32];
#define WS_MMA_STEP(WORD, I0)                                                  \
    {                                                                          \
        const uint32_t v = (WORD);                                             \
        uint32_t af[4];                                                        \
        af[0] = (v & 0x000f000fu) | 0x43004300u;                               \
        af[1] = ((v >> 4) & 0x000f000fu) | 0x43004300u;                        \
        af[2] = ((v >> 8) & 0x000f000fu) | 0x43004300u;                        \
        af[3] = ((v >> 12) & 0x000f000fu) | 0x43004300u;                       \
        _Pragma("unroll") for (int mb = 0; mb < MB; ++mb)                      \
                mma_bf16_16816(accs[((I0) / 2) % NA][mb], af, xr[mb][j][I0], xr[mb][j][(I0) + 1]); \
    }
                        WS_MMA_STEP(wv.x, 0)
                        WS_MMA_STEP(wv.y, 2)
                        WS_MMA_STEP(wv.z, 4)
                        WS_MMA_STEP(wv.w, 6)
#undef WS_MMA_STEP
                    }
                    float acc[MB][4];
#pragma unroll
                    for (int mb = 0; mb < MB; ++mb)
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            float t2 = accs[0][mb][e];
#pragma unroll
                            for (int u = 1; u < NA; ++u) t2 += accs[u][mb][e];
                            acc[mb][e] = t2;
                        }
                    float s0, s1, c0, c1;
                    if (FASTQ) {
                        s0 = __uint_as_float(qs[f] << 16);
                        s1 = __uint_as_float(qs[f] & 0xffff0000u);
                        // 2^23 + nibble as a float, minus (2^23 - offset): offset + nibble, exactly
                        c0 = __uint_as_float(0x4b000000u | (qz[f] & 0xfu)) - (8388608.f - a.nibble_offset);
                        c1 = __uint_as_float(0x4b000000u | (qz[f] >> 4)) - (8388608.f - a.nibble_offset);
                    } else {
                        const uint32_t n0 = s * WC_TILE_N + 2 * g;
                        ws_group_params(a, kfold[f], n0, s0, c0);
                        ws_group_params(a, kfold[f], n0 + 1, s1, c1);
                    }
#pragma unroll
                    for (int mb = 0; mb < MB; ++mb) {
                        const float xe = xf[mb][f][0], xo = xf[mb][f][1];
                        tot[mb][0] = fmaf(s0, fmaf(-c0, xe, acc[mb][0]), tot[mb][0]);
                        tot[mb][1] = fmaf(s0, fmaf(-c0, xo, acc[mb][1]), tot[mb][1]);
                        tot[mb][2] = fmaf(s1, fmaf(-c1, xe, acc[mb][2]), tot[mb][2]);
                        tot[mb][3] = fmaf(s1, fmaf(-c1, xo, acc[mb][3]), tot[mb][3]);
                    }
                }
            }
            // the stage's bytes are in registers or consumed: hand it back to the producer
            __syncwarp();
            if (lane == 0) ws_mbar_arrive(&ctrl->empty[st]);
            // partial sums of the strip into this warp's slab of buffer i & 1
            const uint32_t buf = i & 1, use = i >> 1;
            if (use > 0) {
                ok = ws_wait(&ctrl->slab_empty[buf], (use - 1) & 1, ctrl, p.status, WS_ST_SLAB_EMPTY);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
            }
            if (active) {
                float4 *mine = slabs + ((size_t)(buf * WS_WARPS + warp) * MB) * 32 + lane;
#pragma unroll
                for (int mb = 0; mb < MB; ++mb) mine[mb * 32] = make_float4(tot[mb][0], tot[mb][1], tot[mb][2], tot[mb][3]);
            }
            __syncwarp();
            if (lane == 0) ws_mbar_arrive(&ctrl->slab_full[buf]);
            w = wn;
            if (++st == S) {
                st = 0;
                ph ^= 1;
            }
        }
    } else {
        // ---------------- epilogue warps: one per 8-row block ----------------
        const uint32_t mb = warp - WS_WARPS - 1;
        const uint32_t g = lane >> 2, t = lane & 3;
        const float dst_inv = dst_scale_reciprocal(p);
        const float src_scale = p.src_scale.ptr ? load_f32(p.src_scale.dt, p.src_scale.ptr, 0) : 1.f;
        ws_walk_t w;
        w.start(a, rg);
        bool ok = true;
#pragma unroll 1
        for (uint32_t i = 0; i < rg.n; ++i) {
            const uint32_t buf = i & 1, use = i >> 1;
            const uint32_t qlo = rg.qlo(w.k), qhi = rg.qhi(w.k);
            ok = ws_wait(&ctrl->slab_full[buf], use & 1, ctrl, p.status, WS_ST_SLAB_FULL);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
            const float4 *sl = slabs + ((size_t)(buf * WS_WARPS) * MB + mb) * 32 + lane;
            for (uint32_t w = 4 * qlo; w < 4 * qhi; ++w) {
                const float4 v = sl[(size_t)w * MB * 32];
                sum.x += v.x;
                sum.y += v.y;
                sum.z += v.z;
                sum.w += v.w;
            }
            __syncwarp();
            if (lane == 0) ws_mbar_arrive(&ctrl->slab_empty[buf]);
            const uint32_t strip = w.s;
            w = w.next(a, rg, i);
            if (mb >= nblk) continue; // no valid row in this block (the barriers above still count this warp)
            const uint32_t r0 = mb * 8 + 2 * t;             // rows r0, r0 + 1 of the pass
            const int64_t n0 = (int64_t)strip * WC_TILE_N + 2 * g; // columns n0, n0 + 1
            const float v[4] = {sum.x, sum.y, sum.z, sum.w}; // (r0, n0) (r0+1, n0) (r0, n0+1) (r0+1, n0+1)
            if (a.parts == 1 && qlo == 0 && qhi == 4) {
                // the whole strip was summed here
                if (a.plain_bf16) {
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const uint32_t r = r0 + e;
                        if (r < rows)
                            *reinterpret_cast<uint32_t *>((uint16_t *)p.dst + (a.m0 + r) * p.dst_sm + n0)
                                    = (uint32_t)f32_to_bf16_bits(v[e]) | ((uint32_t)f32_to_bf16_bits(v[e + 2]) << 16);
                    }
                } else if (a.simple) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const uint32_t r = r0 + (e & 1);
                        if (r < rows) ws_finish_simple(p, v[e], a.m0 + r, n0 + (e >> 1), src_scale, dst_inv);
                    }
                } else {
#pragma unroll 1
                    for (int e = 0; e < 4; ++e) {
                        const uint32_t r = r0 + (e & 1);
                        if (r < rows) ws_finish(p, v[e], a.m0 + r, n0 + (e >> 1), src_scale, dst_inv);
                    }
                }
                continue;
            }
            // part of a strip: into the scratch; whoever completes the strip's count finishes it
            float *out = a.acc + (int64_t)a.m0 * a.N;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const uint32_t r = r0 + (e & 1);
                if (r < rows) atomicAdd(out + (int64_t)r * a.N + n0 + (e >> 1), v[e]);
            }
            __threadfence(); // the sums above are visible before the count below
            __syncwarp();
            const uint32_t cnt = (qhi - qlo) * (C / 4);
            uint32_t before = 0;
            if (lane == 0) before = atomicAdd(a.done + strip, cnt);
            before = __shfl_sync(0xffffffffu, before, 0);
            if (before + cnt != a.kchunks * nblk) continue;
            __threadfence();
            const uint32_t cells = rows * WC_TILE_N;
            for (uint32_t c = lane; c < cells; c += 32) {
                const uint32_t r = c / WC_TILE_N, col = c % WC_TILE_N;
                float *cell = out + (int64_t)r * a.N + (int64_t)strip * WC_TILE_N + col;
                const float d = __ldcg(cell);
                *cell = 0.f;
                if (a.simple) ws_finish_simple(p, d, a.m0 + r, (int64_t)strip * WC_TILE_N + col, src_scale, dst_inv);
                else ws_finish(p, d, a.m0 + r, (int64_t)strip * WC_TILE_N + col, src_scale, dst_inv);
            }
            if (lane == 0) a.done[strip] = 0;
        }
    }
}

static inline size_t align256(size_t x) { return (x + 255) / 256 * 256; }

} // namespace b200

using namespace b200;

// bf16 scales and u4 zero-points, both [K / group][N] over the same K groups
static bool wc_fast_quant(const b200_matmul_params_t *p, int64_t gs, int64_t gz) {
    return p->wei_scale.ptr && p->wei_zp.ptr && p->wei_scale.dt == B200_DT_BF16 && p->wei_zp.dt == B200_DT_U4 && gs == gz
            && p->wei_scale.s0 == p->N && p->wei_scale.s1 == 1 && p->wei_zp.s0 == p->N && p->wei_zp.s1 == 1
            && p->N * (p->K / gs) < ((int64_t)1 << 31) && ((uintptr_t)p->wei_scale.ptr & 3) == 0;
}

static wc_div_t wc_make_div(uint32_t d) {
    uint32_t l = 0;
    while (((uint64_t)1 << l) < d) ++l;
    wc_div_t f;
    f.m = (uint32_t)((((uint64_t)1 << 32) * (((uint64_t)1 << l) - d)) / d + 1);
    f.s1 = l < 1 ? l : 1;
    f.s2 = l > 0 ? l - 1 : 0;
    return f;
}

template <int MB, bool FASTQ>
static void wc_launch_variant(const wc_args_t &a, const b200_matmul_params_t &p, bool xtab, int unit_steps, unsigned ctas,
        size_t smem, cudaStream_t cs) {
    const unsigned threads = wc_warps(MB) * 32;
    // rings, slabs and table exceed the 48 KiB a kernel gets without asking
    static std::once_flag once[64];
    int dev = 0;
    cudaGetDevice(&dev);
    std::call_once(once[dev & 63], [] {
        const int max_smem = 227 * 1024;
        cudaFuncSetAttribute(wc_gemv_kernel<MB, FASTQ, true, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
        cudaFuncSetAttribute(wc_gemv_kernel<MB, FASTQ, true, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
        cudaFuncSetAttribute(wc_gemv_kernel<MB, FASTQ, false, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
        cudaFuncSetAttribute(wc_gemv_kernel<MB, FASTQ, false, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
    });
    if (xtab) {
        if (unit_steps == 2) wc_gemv_kernel<MB, FASTQ, true, 2><<<ctas, threads, smem, cs>>>(a, p);
        else wc_gemv_kernel<MB, FASTQ, true, 1><<<ctas, threads, smem, cs>>>(a, p);
    } else {
        if (unit_steps == 2) wc_gemv_kernel<MB, FASTQ, false, 2><<<ctas, threads, smem, cs>>>(a, p);
        else wc_gemv_kernel<MB, FASTQ, false, 1><<<ctas, threads, smem, cs>>>(a, p);
    }
}

// ---- launch of the streaming form ----
typedef void (*ws_kernel_t)(const ws_args_t, const b200_matmul_params_t);
template <int MB, int TPW, int FE>
static ws_kernel_t ws_pick(bool fastq) {
    return fastq ? wc_stream_kernel<MB, TPW, FE, true> : wc_stream_kernel<MB, TPW, FE, false>;
}
static ws_kernel_t ws_kernel_for(int mb, int tpw, int fe, bool fastq) {
    const int key = mb * 100 + tpw * 10 + fe;
    switch (key) {
        case 144: return ws_pick<1, 4, 4>(fastq);
        case 142: return ws_pick<1, 4, 2>(fastq);
        case 141: return ws_pick<1, 4, 1>(fastq);
        case 122: return ws_pick<1, 2, 2>(fastq);
        case 121: return ws_pick<1, 2, 1>(fastq);
        case 111: return ws_pick<1, 1, 1>(fastq);
        case 222: return ws_pick<2, 2, 2>(fastq);
        case 221: return ws_pick<2, 2, 1>(fastq);
        case 211: return ws_pick<2, 1, 1>(fastq);
        case 411: return ws_pick<4, 1, 1>(fastq);
        default: return nullptr;
    }
}

// One pass (up to 32 activation rows from a.m0) with the streaming kernel.  Returns
// B200_ERR_UNSUPPORTED when the shape does not fit its chunking: K must be a multiple of
// 1024 x TPW with MB x TPW <= 4, and the quantisation groups must nest with a warp's tile steps.
static int ws_run_pass(const wc_args_t &w, const b200_matmul_params_t &p, int mb, uint32_t fold_steps, bool fastq, int sms,
        cudaStream_t cs) {
    int tpw = 0, fe = 0;
    for (int cand = 4 / mb; cand >= 1; cand /= 2) {
        if (w.kchunks % (uint32_t)(WS_WARPS * cand) != 0) continue;
        const bool nests = fold_steps >= (uint32_t)cand ? fold_steps % cand == 0 : cand % fold_steps == 0;
        if (!nests) continue;
        tpw = cand;
        fe = fold_steps >= (uint32_t)cand ? cand : (int)fold_steps;
        break;
    }
    if (!tpw) return B200_ERR_UNSUPPORTED;
    ws_kernel_t kern = ws_kernel_for(mb, tpw, fe, fastq);
    if (!kern) return B200_ERR_UNSUPPORTED;
    ws_args_t a;
    a.wei = (const unsigned char *)w.wei;
    a.x = w.x;
    a.x_ld = w.x_ld;
    a.acc = w.acc;
    a.done = w.done;
    a.M = w.M;
    a.N = w.N;
    a.m0 = w.m0;
    a.scale = w.scale; a.scale_dt = w.scale_dt; a.scale_s0 = w.scale_s0; a.scale_s1 = w.scale_s1; a.scale_g0 = w.scale_g0;
    a.zp = w.zp; a.zp_dt = w.zp_dt; a.zp_s0 = w.zp_s0; a.zp_s1 = w.zp_s1; a.zp_g0 = w.zp_g0;
    a.nibble_offset = w.nibble_offset;
    a.kchunks = w.kchunks;
    a.strips = (uint32_t)(w.N / WC_TILE_N);
    const uint32_t chunk_steps = (uint32_t)(WS_WARPS * tpw);
    a.parts = w.kchunks / chunk_steps;
    // Several K parts per strip send every strip's sums through the global scratch (atomics, a
    // fence and a counter round trip per chunk on one epilogue warp): measured several times slower
    // than the per-lane copy form, which is therefore kept for those shapes.
    if (a.parts != 1) return B200_ERR_UNSUPPORTED;
    const uint64_t quarters = (uint64_t)a.strips * a.parts * 4;
    if (quarters >= ((uint64_t)1 << 31)) return B200_ERR_TOO_LARGE;
    a.quarters = (uint32_t)quarters;
    a.div_strips = wc_make_div(a.strips);
    a.div_fold = wc_make_div(fold_steps);
    a.simple = p.npo == 0 && (!p.bias || p.bias_dt == B200_DT_F32 || p.bias_dt == B200_DT_BF16)
            && (p.dst_dt == B200_DT_F32 || p.dst_dt == B200_DT_BF16);
    a.plain_bf16 = p.dst_dt == B200_DT_BF16 && !p.bias && p.npo == 0 && !p.src_scale.ptr && !p.dst_scale.ptr && p.dst_sm % 2 == 0
            && ((uintptr_t)p.dst & 3) == 0;
    const size_t chunk_bytes = (size_t)chunk_steps * WC_TILE_BYTES;
    const size_t slab_bytes = (size_t)2 * WS_WARPS * mb * 32 * sizeof(float4);
    const size_t budget = (size_t)227 * 1024 - 1024 - slab_bytes - sizeof(ws_ctrl_t);
    size_t stages = budget / chunk_bytes;
    if (stages > WS_MAX_STAGES) stages = WS_MAX_STAGES;
    if (stages < 2) return B200_ERR_UNSUPPORTED;
    a.stages = (uint32_t)stages;
    const size_t smem = stages * chunk_bytes + slab_bytes + sizeof(ws_ctrl_t);
    // opt in to the large dynamic shared memory once per kernel and device
    static std::mutex mu;
    static std::vector<std::pair<int, const void *>> done_attr;
    int dev = 0;
    cudaGetDevice(&dev);
    {
        std::lock_guard<std::mutex> g(mu);
        bool seen = false;
        for (auto &e : done_attr) seen |= e.first == dev && e.second == (const void *)kern;
        if (!seen) {
            const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
            if (e != cudaSuccess) return (int)e;
            done_attr.emplace_back(dev, (const void *)kern);
        }
    }
    const unsigned ctas = a.quarters < (uint32_t)sms ? a.quarters : (unsigned)sms;
    kern<<<ctas, ws_threads(mb), smem, cs>>>(a, p);
    return after_launch();
}

// Checks shared by the two entry points; on success the K-group sizes of scales and
// zero-points and the fold period are returned.
static int wc_validate(const b200_matmul_params_t *p, int64_t *gs_out, int64_t *gz_out, int64_t *fold_out) {
    if (p->wei_dt != B200_DT_U4 && p->wei_dt != B200_DT_S4) return B200_ERR_UNSUPPORTED;
    if (!p->apply_to_int) return B200_ERR_UNSUPPORTED;
    if (p->N % WC_TILE_N != 0 || p->K % WC_TILE_K != 0 || p->src_sk != 1 || p->dst_sn != 1 || p->n_dst_peers) return B200_ERR_UNSUPPORTED;
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
    // a tile step covers 64 k in a permuted order, so groups must be whole tile steps;
    // one group size must divide the other
    if (gs % WC_TILE_K || gz % WC_TILE_K || p->K % gs || p->K % gz) return B200_ERR_UNSUPPORTED;
    const int64_t fold_k = gs < gz ? gs : gz;
    if (gs % fold_k || gz % fold_k) return B200_ERR_UNSUPPORTED;
    *gs_out = gs;
    *gz_out = gz;
    *fold_out = fold_k;
    return 0;
}

// All passes over the activation rows.  acc: zeroed f32 [M][N]; done: zeroed [N / 16].
static int wc_run(const b200_matmul_params_t *p, const uint4 *wei, const __nv_bfloat16 *x, int64_t x_ld, float *acc,
        uint32_t *done, int64_t gs, int64_t gz, int64_t fold_k, cudaStream_t cs) {
    wc_args_t a;
    a.wei = wei;
    a.x = x;
    a.x_ld = x_ld;
    a.acc = acc;
    a.done = done;
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
    a.nibble_offset = p->wei_dt == B200_DT_S4 ? 136.f : 128.f;
    // a unit never straddles a quantisation group: two tile steps where the groups allow it
    const uint32_t fold_steps = (uint32_t)(fold_k / WC_TILE_K);
    const int unit_steps = fold_steps % 2 == 0 ? 2 : 1;
    a.kchunks = (uint32_t)(p->K / WC_TILE_K);
    a.ups = a.kchunks / unit_steps;
    a.units = (uint32_t)(p->N / WC_TILE_N) * a.ups;
    a.div_ups = wc_make_div(a.ups);
    a.div_fu = wc_make_div(fold_steps / unit_steps);

    const bool fastq = wc_fast_quant(p, gs, gz);
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    a.group_is_unit = fold_steps / unit_steps == 1;
    unsigned ctas = a.units < (uint32_t)sms ? a.units : (unsigned)sms;
    // Whole strips per CTA need no exchange between CTAs but leave some SMs one strip short of
    // others; taken when that costs less than the exchange would (about two microseconds at
    // the rate one GPU streams weights).
    const uint32_t strips = (uint32_t)(p->N / WC_TILE_N);
    a.whole_strips = 0;
    if (strips >= ctas) {
        const double avg = (double)strips / ctas, most = (double)((strips + ctas - 1) / ctas);
        const double stream_us = (double)p->K * p->N / 2 / 5e6;
        if ((most - avg) / avg * stream_us < 2.0) a.whole_strips = 1;
    }
    // strips one CTA can touch: those of its share of the units plus one cut at either end
    {
        const uint32_t share = a.whole_strips ? (strips + ctas - 1) / ctas * a.ups : (a.units + ctas - 1) / ctas;
        a.max_segs = (share / a.ups + 2 + 3) / 4 * 4;
        if (a.max_segs > 8192) return B200_ERR_TOO_LARGE;
    }
    // the streaming form where the shape fits its chunking (ONEDNN_B200_WC_STREAM=0 keeps the per-lane copy form)
    const char *se = std::getenv("ONEDNN_B200_WC_STREAM");
    const bool use_stream = !(se && se[0] == '0');
    // activation rows in passes of up to 32 (the weights are re-read from L2)
    for (int64_t m0 = 0; m0 < p->M; m0 += 32) {
        a.m0 = (int)m0;
        const int64_t rows = p->M - m0;
        const int mb = rows <= 8 ? 1 : rows <= 16 ? 2 : 4;
        if (use_stream) {
            const int rc = ws_run_pass(a, *p, mb, fold_steps, fastq, sms, cs);
            if (rc != B200_ERR_UNSUPPORTED) {
                if (rc) return rc;
                continue;
            }
        }
        const size_t table = (size_t)a.kchunks * mb * 8 * sizeof(float);
        const bool xtab = table <= WC_XTAB_MAX_BYTES;
        const size_t nw = wc_warps(mb);
        const size_t smem = nw * wc_ring_bytes(mb) + nw * 3 * mb * 128 * sizeof(float) + nw * sizeof(uint2)
                + (size_t)a.max_segs * sizeof(uint32_t) + (xtab ? table : 0);
        if (fastq) {
            if (mb == 1) wc_launch_variant<1, true>(a, *p, xtab, unit_steps, ctas, smem, cs);
            else if (mb == 2) wc_launch_variant<2, true>(a, *p, xtab, unit_steps, ctas, smem, cs);
            else wc_launch_variant<4, true>(a, *p, xtab, unit_steps, ctas, smem, cs);
        } else {
            if (mb == 1) wc_launch_variant<1, false>(a, *p, xtab, unit_steps, ctas, smem, cs);
            else if (mb == 2) wc_launch_variant<2, false>(a, *p, xtab, unit_steps, ctas, smem, cs);
            else wc_launch_variant<4, false>(a, *p, xtab, unit_steps, ctas, smem, cs);
        }
        const int rc = after_launch();
        if (rc) return rc;
    }
    return 0;
}

// scratch layout of the wc kernel: [f32 acc M*N][bf16 x copy M*K if src is not bf16][packed weights if plain]
static void wc_scratch_layout(const b200_matmul_params_t *p, size_t *acc, size_t *xcopy, size_t *packed) {
    // partial sums [M][N] followed by one counter per strip of 16 columns
    *acc = align256((size_t)p->M * p->N * sizeof(float)) + align256((size_t)(p->N / WC_TILE_N) * sizeof(uint32_t));
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
    if (p->src_dt != B200_DT_BF16 && p->src_dt != B200_DT_F16 && p->src_dt != B200_DT_F32) return B200_ERR_UNSUPPORTED;
    if (p->wei_layout == B200_WEI_PLAIN && !(p->wei_sn == 1 && p->wei_sk == p->N)) return B200_ERR_UNSUPPORTED;
    if (p->wei_layout != B200_WEI_PLAIN && p->wei_layout != B200_WEI_WC4_TILED) return B200_ERR_UNSUPPORTED;
    int64_t gs, gz, fold_k;
    int rc = wc_validate(p, &gs, &gz, &fold_k);
    if (rc) return rc;
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
        rc = after_launch();
        if (rc) return rc;
        x = xc;
        x_ld = p->K;
    }
    const void *wei = p->wei;
    if (w_b) {
        void *wp = sc + acc_b + x_b;
        rc = b200_wc_pack_launch(p->wei, wp, p->K, p->N, p->wei_dt, stream);
        if (rc) return rc;
        wei = wp;
    }
    if (((uintptr_t)wei & 15)) return B200_ERR_BAD_ARG;
    if (!p->scratch_zeroed) {
        if (cudaMemsetAsync(acc, 0, acc_b, cs) != cudaSuccess) return (int)cudaGetLastError();
    }
    uint32_t *done = (uint32_t *)((char *)acc + align256((size_t)p->M * p->N * sizeof(float)));
    return wc_run(p, (const uint4 *)wei, x, x_ld, acc, done, gs, gz, fold_k, cs);
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
static constexpr size_t WC_STATIC_SCRATCH_BYTES = (size_t)2 << 20; // partial sums (4 bytes per dst element) + strip counters
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
    if (p->src_dt != B200_DT_BF16 || p->wei_layout != B200_WEI_WC4_TILED) return B200_ERR_UNSUPPORTED;
    int64_t gs, gz, fold_k;
    int rc = wc_validate(p, &gs, &gz, &fold_k);
    if (rc) return rc;
    if (((uintptr_t)p->src & 15) || (p->src_sm & 7) || ((uintptr_t)p->wei & 15)) return B200_ERR_BAD_ARG;
    // the fixed array bounds the problem: M * N partial sums of 4 bytes plus the strip counters
    const size_t used = align256((size_t)p->M * p->N * sizeof(float)) + align256((size_t)(p->N / WC_TILE_N) * sizeof(uint32_t));
    if ((uint64_t)p->M * (uint64_t)p->N > ((uint64_t)1 << 40) || used > WC_STATIC_SCRATCH_BYTES) return B200_ERR_TOO_LARGE;

    float *acc = nullptr;
    rc = wc_static_scratch_ptr(&acc);
    if (rc) return rc;
    cudaStream_t cs = (cudaStream_t)stream;
    // the array keeps whatever the last call left behind: clear the part used now
    if (cudaMemsetAsync(acc, 0, used, cs) != cudaSuccess) return (int)cudaGetLastError();
    uint32_t *done = (uint32_t *)((char *)acc + align256((size_t)p->M * p->N * sizeof(float)));
    return wc_run(p, (const uint4 *)p->wei, (const __nv_bfloat16 *)p->src, p->src_sm, acc, done, gs, gz, fold_k, cs);
}
