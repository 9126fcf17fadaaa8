// Quantising reorder: dst = convert((src_scale * (src - src_zp) [+ beta * dst]) * (1 / dst_scale) + dst_zp)
// over a plain 2-D tensor -- what a user runs on the activations before an int8 matmul and on
// its result afterwards.  Arithmetic follows the reference's generic reorder step for step
// (src/cpu/reorder/simple_reorder.hpp:2551-2635; destination scale inverted up front,
// src/cpu/reorder/cpu_reorder_pd.hpp:83-109): an integer source minus its zero-point is an
// s32 subtraction, every other step one f32 operation rounded on its own (no fused
// multiply-add), integer destinations saturate and then round to nearest even.
//
// The work is pure streaming: 1-4 bytes read and 1-4 bytes written per element, so the bound
// is HBM bandwidth.  The fast kernel handles rows that are contiguous in both tensors.  One
// work item is V consecutive elements of a row, V chosen so that the narrower of the two
// tensors moves 16 bytes per item (V = 16 with an 8-bit side, 8 with a 16-bit side, else 4);
// a thread owns one item position and walks down the rows, keeping at least 64 bytes of
// loads in flight.  Everything else (transposing strides, odd sizes, a sum post-op, group
// sizes that cut an item, f16 / f8 tensors, scales that are not f32) goes through the
// element-wise kernel.
#include "common.cuh"
#include "launch.hpp"

namespace b200 {

namespace {

// how a scale / zero-point argument varies, as the row kernel sees it
enum {
    K_NONE = 0,  // not set
    K_CONST = 1, // one value per thread: per tensor, or column groups that contain the item
    K_ROW = 2,   // one value per (row, item): fetched with the row's data
    K_COL = 3    // one value per column, the same for every row: held in registers
};

struct rq_args_t {
    b200_reorder_quant_params_t p;
    uint32_t items; // items per row
    int kind_ss, kind_ds, kind_sz;
};

template <int DT>
struct dt_bytes {
    static constexpr int value
            = (DT == B200_DT_F32 || DT == B200_DT_S32) ? 4 : (DT == B200_DT_BF16 || DT == B200_DT_F16) ? 2 : 1;
};

// W 32-bit words from / to a row, in the widest pieces the item's size allows; streaming
// hints: nothing is read twice
template <int W>
__device__ __forceinline__ void load_words(const void *ptr, uint32_t (&w)[W]) {
    if (W >= 4) {
#pragma unroll
        for (int i = 0; i < W / 4; ++i) {
            const uint4 v = __ldcs((const uint4 *)ptr + i);
            w[4 * i] = v.x; w[4 * i + 1] = v.y; w[4 * i + 2] = v.z; w[4 * i + 3] = v.w;
        }
    } else if (W == 2) {
        const uint2 v = __ldcs((const uint2 *)ptr);
        w[0] = v.x; w[1] = v.y;
    } else {
        w[0] = __ldcs((const uint32_t *)ptr);
    }
}

template <int W>
__device__ __forceinline__ void store_words(void *ptr, const uint32_t (&w)[W]) {
    if (W >= 4) {
#pragma unroll
        for (int i = 0; i < W / 4; ++i)
            __stcs((uint4 *)ptr + i, make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]));
    } else if (W == 2) {
        __stcs((uint2 *)ptr, make_uint2(w[0], w[1]));
    } else {
        __stcs((uint32_t *)ptr, w[0]);
    }
}

// element e of packed words -> f32 value of (src - zp): integer sources subtract in s32 first
template <int DT, int W>
__device__ __forceinline__ float decode_minus_zp(const uint32_t (&w)[W], int e, int zp) {
    switch (DT) {
        case B200_DT_F32: return __fsub_rn(__uint_as_float(w[e]), (float)zp);
        case B200_DT_BF16:
            return __fsub_rn(__uint_as_float((e & 1) ? (w[e >> 1] & 0xffff0000u) : (w[e >> 1] << 16)), (float)zp);
        case B200_DT_S32: return (float)((int)w[e] - zp);
        case B200_DT_S8: return (float)(((int)(w[e >> 2] << (24 - 8 * (e & 3))) >> 24) - zp);
        default: return (float)((int)((w[e >> 2] >> (8 * (e & 3))) & 0xffu) - zp); // u8
    }
}

template <int DT>
__device__ __forceinline__ uint32_t encode(float d) {
    switch (DT) {
        case B200_DT_F32: return __float_as_uint(d);
        case B200_DT_BF16: return f32_to_bf16_bits(d);
        case B200_DT_S32: return (uint32_t)sat_rne_s32(d);
        case B200_DT_S8: return cvt_sat_s8(d);
        default: return cvt_sat_u8(d); // u8
    }
}

__device__ __forceinline__ uint32_t quant_word(const b200_quant_t &q, uint32_t row, uint32_t col) {
    int64_t off = 0;
    if (q.s0) off = (int64_t)(q.g0 == 1 ? row : row / (uint32_t)q.g0) * q.s0;
    if (q.s1) off += (int64_t)(q.g1 == 1 ? col : col / (uint32_t)q.g1) * q.s1;
    return __ldg((const uint32_t *)q.ptr + off);
}

// Thread (x, y) of a block owns the V columns of item x for the rows y, y + Y, ... (Y = rows in
// flight over the grid): no index division, and what does not depend on the row -- per-tensor
// and per-column scales, their reciprocals, zero-points -- is fetched once per thread.
// COLQ: some argument has one value per column (otherwise all three are scalars per row).
// Scales are f32 and zero-points s32 here, i.e. 4-byte words.
template <int SDT, int DDT, int V, bool COLQ>
__global__ void __launch_bounds__(256) reorder_quant_rows_kernel(const __grid_constant__ rq_args_t a) {
    constexpr int SB = dt_bytes<SDT>::value, DB = dt_bytes<DDT>::value;
    constexpr int SW = V * SB / 4, DW = V * DB / 4;          // words per item
    constexpr int UNROLL = SW >= 16 ? 1 : (SW >= 8 ? 2 : (SW >= 4 ? 4 : 8)); // rows per step: >= 64 bytes of loads in flight
    const b200_reorder_quant_params_t &p = a.p;
    const uint32_t item = blockIdx.x * blockDim.x + threadIdx.x;
    if (item >= a.items) return;
    const uint32_t col = item * V;
    const float dzp = p.dst_zp.ptr ? (float)__ldg((const int *)p.dst_zp.ptr) : 0.f;
    float s_ss = 1.f, s_rds = 1.f;
    int s_zp = 0;
    if (a.kind_ss == K_CONST) s_ss = __uint_as_float(quant_word(p.src_scale, 0, col));
    if (a.kind_ds == K_CONST) s_rds = __fdiv_rn(1.f, __uint_as_float(quant_word(p.dst_scale, 0, col)));
    if (a.kind_sz == K_CONST) s_zp = (int)quant_word(p.src_zp, 0, col);
    float v_ss[COLQ ? V : 1], v_rds[COLQ ? V : 1];
    int v_zp[COLQ ? V : 1];
    if (COLQ) {
#pragma unroll
        for (int e = 0; e < V; ++e) {
            v_ss[e] = a.kind_ss == K_COL ? __uint_as_float(quant_word(p.src_scale, 0, col + e)) : s_ss;
            v_rds[e] = a.kind_ds == K_COL ? __fdiv_rn(1.f, __uint_as_float(quant_word(p.dst_scale, 0, col + e))) : s_rds;
            v_zp[e] = a.kind_sz == K_COL ? (int)quant_word(p.src_zp, 0, col + e) : s_zp;
        }
    }
    const uint32_t rows = (uint32_t)p.rows, ystep = gridDim.y * blockDim.y;
    const char *src = (const char *)p.src + (int64_t)col * SB;
    char *dst = (char *)p.dst + (int64_t)col * DB;
    for (uint32_t r0 = blockIdx.y * blockDim.y + threadIdx.y; r0 < rows; r0 += ystep * UNROLL) {
        uint32_t raw[UNROLL][SW], q_ss[UNROLL], q_ds[UNROLL], q_sz[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const uint32_t r = r0 + u * ystep;
            if (r < rows) {
                load_words<SW>(src + (int64_t)r * p.src_s0 * SB, raw[u]);
                if (a.kind_ss == K_ROW) q_ss[u] = quant_word(p.src_scale, r, col);
                if (a.kind_ds == K_ROW) q_ds[u] = quant_word(p.dst_scale, r, col);
                if (a.kind_sz == K_ROW) q_sz[u] = quant_word(p.src_zp, r, col);
            }
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const uint32_t r = r0 + u * ystep;
            if (r >= rows) continue;
            if (a.kind_ss == K_ROW) s_ss = __uint_as_float(q_ss[u]);
            if (a.kind_ds == K_ROW) s_rds = __fdiv_rn(1.f, __uint_as_float(q_ds[u]));
            if (a.kind_sz == K_ROW) s_zp = (int)q_sz[u];
            if (COLQ && (a.kind_ss == K_ROW || a.kind_ds == K_ROW || a.kind_sz == K_ROW)) {
#pragma unroll
                for (int e = 0; e < V; ++e) {
                    if (a.kind_ss == K_ROW) v_ss[e] = s_ss;
                    if (a.kind_ds == K_ROW) v_rds[e] = s_rds;
                    if (a.kind_sz == K_ROW) v_zp[e] = s_zp;
                }
            }
            uint32_t out[DW];
#pragma unroll
            for (int i = 0; i < DW; ++i) out[i] = 0;
#pragma unroll
            for (int e = 0; e < V; ++e) {
                const float ss = COLQ ? v_ss[e] : s_ss, rds = COLQ ? v_rds[e] : s_rds;
                const int zp = COLQ ? v_zp[e] : s_zp;
                const float d = __fmul_rn(ss, decode_minus_zp<SDT, SW>(raw[u], e, zp));
                const uint32_t bits = encode<DDT>(__fadd_rn(__fmul_rn(d, rds), dzp));
                if (DB == 4) out[e] = bits;
                else if (DB == 2) out[e >> 1] |= bits << (16 * (e & 1));
                else out[e >> 2] |= bits << (8 * (e & 3));
            }
            store_words<DW>(dst + (int64_t)r * p.dst_s0 * DB, out);
        }
    }
}

// any strides, any group sizes, any 8 / 16 / 32-bit types, optional sum post-op: one element
// per thread step
__global__ void __launch_bounds__(256) reorder_quant_elem_kernel(const __grid_constant__ b200_reorder_quant_params_t p) {
    const int64_t total = p.rows * p.cols;
    const float dzp = p.dst_zp.ptr ? (float)load_int(p.dst_zp.dt, p.dst_zp.ptr, 0) : 0.f;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / p.cols, c = i - r * p.cols;
        const float ss = p.src_scale.ptr ? load_f32(p.src_scale.dt, p.src_scale.ptr, quant_off(p.src_scale, r, c)) : 1.f;
        const float rds = p.dst_scale.ptr
                ? __fdiv_rn(1.f, load_f32(p.dst_scale.dt, p.dst_scale.ptr, quant_off(p.dst_scale, r, c)))
                : 1.f;
        const int zp = p.src_zp.ptr ? (int)load_f32(p.src_zp.dt, p.src_zp.ptr, quant_off(p.src_zp, r, c)) : 0;
        const int64_t so = r * p.src_s0 + c * p.src_s1, dof = r * p.dst_s0 + c * p.dst_s1;
        float v;
        if (dt_is_int(p.src_dt))
            v = (float)(load_int(p.src_dt, p.src, so) - zp);
        else
            v = __fsub_rn(load_f32(p.src_dt, p.src, so), (float)zp);
        float d = __fmul_rn(ss, v);
        if (p.beta != 0.f) d = __fadd_rn(d, __fmul_rn(p.beta, load_f32(p.dst_dt, p.dst, dof)));
        d = __fadd_rn(__fmul_rn(d, rds), dzp);
        store_f32(p.dst_dt, d, p.dst, dof);
    }
}

// 4-bit tensors on either side (two values per byte, even index in the low nibble; dense rows
// that start on a byte): one thread per pair of neighbouring columns, so that a destination
// byte has one writer.  s4 / u4 -> f32 / bf16 / f16 with source scales and zero-points of any
// mask and grouping (decompressing weights), f32 -> s4 / u4 saturating, round to nearest even
// (src/common/int4.hpp, src/cpu/ref_io_helper.hpp:84-97; the reference's own f32 -> 4-bit
// reorder accepts a common destination scale and does not apply it: not mirrored, the launcher
// takes no attributes on that side).
__global__ void __launch_bounds__(256) reorder_quant_int4_kernel(const __grid_constant__ b200_reorder_quant_params_t p) {
    const int64_t pairs = p.cols / 2, total = p.rows * pairs;
    const bool dst4 = p.dst_dt == B200_DT_S4 || p.dst_dt == B200_DT_U4;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / pairs, c0 = 2 * (i - r * pairs);
        float d[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int64_t c = c0 + e;
            const float ss = p.src_scale.ptr ? load_f32(p.src_scale.dt, p.src_scale.ptr, quant_off(p.src_scale, r, c)) : 1.f;
            const int zp = p.src_zp.ptr ? (int)load_f32(p.src_zp.dt, p.src_zp.ptr, quant_off(p.src_zp, r, c)) : 0;
            const int64_t so = r * p.src_s0 + c * p.src_s1;
            const float v = dt_is_int(p.src_dt) || p.src_dt == B200_DT_S4 || p.src_dt == B200_DT_U4
                    ? (float)(load_int(p.src_dt, p.src, so) - zp)
                    : __fsub_rn(load_f32(p.src_dt, p.src, so), (float)zp);
            d[e] = __fmul_rn(ss, v);
        }
        if (dst4) {
            const float lo = p.dst_dt == B200_DT_S4 ? -8.f : 0.f, hi = p.dst_dt == B200_DT_S4 ? 7.f : 15.f;
            const uint32_t q0 = (uint32_t)__float2int_rn(fminf(fmaxf(d[0], lo), hi)) & 0xfu;
            const uint32_t q1 = (uint32_t)__float2int_rn(fminf(fmaxf(d[1], lo), hi)) & 0xfu;
            ((uint8_t *)p.dst)[(r * p.dst_s0 + c0) >> 1] = (uint8_t)(q0 | (q1 << 4));
        } else {
            store_f32(p.dst_dt, d[0], p.dst, r * p.dst_s0 + c0 * p.dst_s1);
            store_f32(p.dst_dt, d[1], p.dst, r * p.dst_s0 + (c0 + 1) * p.dst_s1);
        }
    }
}

bool dt_ok(int dt) {
    switch (dt) {
        case B200_DT_F32: case B200_DT_BF16: case B200_DT_F16: case B200_DT_F8_E4M3: case B200_DT_F8_E5M2:
        case B200_DT_S32: case B200_DT_S8: case B200_DT_U8: return true;
        default: return false;
    }
}

bool fast_dt(int dt) {
    return dt == B200_DT_F32 || dt == B200_DT_BF16 || dt == B200_DT_S32 || dt == B200_DT_S8 || dt == B200_DT_U8;
}

// how the row kernel with items of v columns would address this argument; -1: it cannot
int quant_kind(const b200_quant_t &q, int want_dt, int v) {
    if (!q.ptr) return K_NONE;
    if (q.dt != want_dt) return -1;
    const bool item_uniform = q.s1 == 0 || q.g1 % v == 0;
    if (item_uniform) return q.s0 == 0 ? K_CONST : K_ROW;
    if (q.g1 == 1 && q.s0 == 0) return K_COL;
    return -1;
}

template <int SDT, int DDT>
int launch_rows(const rq_args_t &a, int v, bool colq, dim3 grid, dim3 block, cudaStream_t cs) {
    constexpr int SB = dt_bytes<SDT>::value, DB = dt_bytes<DDT>::value;
    constexpr int VW = 16 / (SB < DB ? SB : DB); // the wide item of this pair of types
    constexpr int VC = VW > 8 ? 8 : VW;          // with per-column values held in registers
    if (colq) {
        if (v == VC && VC != 4)
            reorder_quant_rows_kernel<SDT, DDT, VC, true><<<grid, block, 0, cs>>>(a);
        else
            reorder_quant_rows_kernel<SDT, DDT, 4, true><<<grid, block, 0, cs>>>(a);
    } else {
        if (v == VW && VW != 4)
            reorder_quant_rows_kernel<SDT, DDT, VW, false><<<grid, block, 0, cs>>>(a);
        else
            reorder_quant_rows_kernel<SDT, DDT, 4, false><<<grid, block, 0, cs>>>(a);
    }
    return after_launch();
}

template <int SDT>
int launch_rows_src(const rq_args_t &a, int v, bool colq, dim3 grid, dim3 block, cudaStream_t cs) {
    switch (a.p.dst_dt) {
        case B200_DT_F32: return launch_rows<SDT, B200_DT_F32>(a, v, colq, grid, block, cs);
        case B200_DT_BF16: return launch_rows<SDT, B200_DT_BF16>(a, v, colq, grid, block, cs);
        case B200_DT_S32: return launch_rows<SDT, B200_DT_S32>(a, v, colq, grid, block, cs);
        case B200_DT_S8: return launch_rows<SDT, B200_DT_S8>(a, v, colq, grid, block, cs);
        default: return launch_rows<SDT, B200_DT_U8>(a, v, colq, grid, block, cs);
    }
}

} // namespace

} // namespace b200

using namespace b200;

extern "C" int b200_reorder_quant_launch(const b200_reorder_quant_params_t *p, b200_stream_t stream) {
    if (!p || p->rows < 0 || p->cols < 0) return B200_ERR_BAD_ARG;
    if (p->rows == 0 || p->cols == 0) return 0;
    if (!p->src || !p->dst) return B200_ERR_BAD_ARG;
    const bool s4 = p->src_dt == B200_DT_S4 || p->src_dt == B200_DT_U4, d4 = p->dst_dt == B200_DT_S4 || p->dst_dt == B200_DT_U4;
    if (s4 || d4) {
        // one side 4-bit, the other a float type; dense rows that start on a byte; no sum, nothing on the dst side
        if (s4 == d4 || p->beta != 0.f || p->dst_scale.ptr || p->dst_zp.ptr) return B200_ERR_UNSUPPORTED;
        if (s4 && !(p->dst_dt == B200_DT_F32 || p->dst_dt == B200_DT_BF16 || p->dst_dt == B200_DT_F16)) return B200_ERR_UNSUPPORTED;
        if (d4 && (p->src_dt != B200_DT_F32 || p->src_scale.ptr || p->src_zp.ptr)) return B200_ERR_UNSUPPORTED;
        const int64_t s0_4 = s4 ? p->src_s0 : p->dst_s0, s1_4 = s4 ? p->src_s1 : p->dst_s1;
        if ((p->cols & 1) || s1_4 != 1 || (p->rows > 1 && (s0_4 & 1))) return B200_ERR_UNSUPPORTED;
        for (const b200_quant_t *q : {&p->src_scale, &p->src_zp})
            if (q->ptr && (q->g0 <= 0 || q->g1 <= 0 || !dt_ok(q->dt))) return B200_ERR_BAD_ARG;
        int64_t blocks = (p->rows * (p->cols / 2) + 255) / 256;
        if (blocks > 148 * 32) blocks = 148 * 32;
        reorder_quant_int4_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(*p);
        return after_launch();
    }
    if (!dt_ok(p->src_dt) || !dt_ok(p->dst_dt)) return B200_ERR_UNSUPPORTED;
    const b200_quant_t *qs[4] = {&p->src_scale, &p->dst_scale, &p->src_zp, &p->dst_zp};
    for (const b200_quant_t *q : qs)
        if (q->ptr && (q->g0 <= 0 || q->g1 <= 0 || !dt_ok(q->dt))) return B200_ERR_BAD_ARG;
    // the reference admits zero-points for integer tensors only (src/common/reorder.cpp:96-103)
    if (p->src_zp.ptr && !dt_is_int(p->src_dt)) return B200_ERR_BAD_ARG;
    if (p->dst_zp.ptr && (!dt_is_int(p->dst_dt) || p->dst_zp.dt != B200_DT_S32)) return B200_ERR_BAD_ARG;
    cudaStream_t cs = (cudaStream_t)stream;

    const int sb = dt_bits(p->src_dt) / 8, db = dt_bits(p->dst_dt) / 8;
    const bool rows_shape = fast_dt(p->src_dt) && fast_dt(p->dst_dt) && p->src_s1 == 1 && p->dst_s1 == 1 && p->beta == 0.f
            && p->cols < (int64_t)1 << 31 && p->rows < (int64_t)1 << 31;
    // the widest item whose pieces are aligned in both tensors and whose columns the
    // scale / zero-point arguments can follow
    const int widths[3] = {16 / (sb < db ? sb : db), 8, 4};
    for (int v : widths) {
        if (!rows_shape) break;
        if (v > widths[0]) continue;
        const int sa = v * sb < 16 ? v * sb : 16, da = v * db < 16 ? v * db : 16; // bytes of one load / store
        if (p->cols % v != 0 || (p->src_s0 * sb) % sa != 0 || (p->dst_s0 * db) % da != 0 || (uintptr_t)p->src % sa != 0
                || (uintptr_t)p->dst % da != 0)
            continue;
        rq_args_t a;
        a.p = *p;
        a.kind_ss = quant_kind(p->src_scale, B200_DT_F32, v);
        a.kind_ds = quant_kind(p->dst_scale, B200_DT_F32, v);
        a.kind_sz = quant_kind(p->src_zp, B200_DT_S32, v);
        if (a.kind_ss < 0 || a.kind_ds < 0 || a.kind_sz < 0) continue;
        const bool colq = a.kind_ss == K_COL || a.kind_ds == K_COL || a.kind_sz == K_COL;
        if (v == 16 && colq) continue;                 // per-column values: items of at most 8
        if (v == 8 && widths[0] != 8 && !colq) continue; // 8 is this pair's width only in that case
        a.items = (uint32_t)(p->cols / v);
        // block: x over the items of a row (a power of two up to 256), y over rows
        unsigned bx = 1;
        while (bx < 256 && bx < a.items) bx <<= 1;
        const dim3 block(bx, 256 / bx);
        const unsigned gx = (a.items + bx - 1) / bx;
        // rows in flight: about eight blocks per SM, but no more blocks than there are rows
        int64_t gy = (p->rows + block.y - 1) / block.y;
        const int64_t want = (148 * 8 + gx - 1) / gx;
        if (gy > want) gy = want;
        if (gy < 1) gy = 1;
        if (gy > 65535) gy = 65535;
        const dim3 grid(gx, (unsigned)gy);
        switch (p->src_dt) {
            case B200_DT_F32: return launch_rows_src<B200_DT_F32>(a, v, colq, grid, block, cs);
            case B200_DT_BF16: return launch_rows_src<B200_DT_BF16>(a, v, colq, grid, block, cs);
            case B200_DT_S32: return launch_rows_src<B200_DT_S32>(a, v, colq, grid, block, cs);
            case B200_DT_S8: return launch_rows_src<B200_DT_S8>(a, v, colq, grid, block, cs);
            default: return launch_rows_src<B200_DT_U8>(a, v, colq, grid, block, cs);
        }
    }
    int64_t blocks = (p->rows * p->cols + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    reorder_quant_elem_kernel<<<(unsigned)blocks, 256, 0, cs>>>(*p);
    return after_launch();
}
