// Dense 8-bit GEMM on the Blackwell tensor cores with the whole matmul epilogue fused.
//
//   dst = epilogue( A[M,K] (u8/s8 or e4m3/e5m2, row-major) x W[N,K] (K-major packed weights) )
//
// Computes what the reference's int8 matmul computes per element
// (src/cpu/matmul/ref_matmul_int8.cpp:154-261: s32 accumulation of (s - zp_src) * w,
// f32 scale by src_scale then wei_scale[n], bias, post-ops, dst scale, dst
// zero-point, saturate + round-to-nearest-even), and for fp8 what its
// floating-point matmul computes (src/cpu/matmul/ref_matmul.cpp:130-233), in the
// place of the reference's AMX brgemm kernel
// (src/cpu/x64/matmul/brgemm_matmul.cpp:383-496, jit_brgemm_amx_uker.cpp:1286-1445).
//
// Structure (one persistent CTA per SM, 576 threads):
//   warp 0      TMA producer: cp.async.bulk.tensor 2-D loads (no multicast) of a
//               128 x 128-byte A tile and a 256 x 128-byte W tile per k-block into a
//               4-stage ring of 128-byte-swizzled shared memory, completion on
//               "full" mbarriers.
//   warp 1      MMA issuer: one lane issues tcgen05.mma.cta_group::1 (kind::i8 or
//               kind::f8f6f4), 128 x 256 x 32 per instruction, four per k-block,
//               accumulating in tensor memory; tcgen05.commit releases the smem
//               stage ("empty" mbarrier) and, after the last k-block, publishes the
//               accumulator ("tmem_full").  Also owns the TMEM allocation (512
//               columns = two 128 x 256 x 32-bit accumulators).
//   warps 2-17  epilogue (four per TMEM lane quarter, each converts a quarter of the
//               tile's columns): tcgen05.ld 32 lanes x 16 columns at a time, exact s32
//               zero-point compensation (acc - zp_src * colsum_W[n]), the f32
//               epilogue chain, packed 16-byte stores.  With two accumulator
//               stages the epilogue of tile i overlaps the main loop of tile i+1.
//
// Every mbarrier wait is bounded: when a wait runs out the kernel raises a flag
// in the stream's status word, every role stops at its next wait, the producer
// waits (bounded) for its own copies in flight, the TMEM allocation is released
// and the kernel returns; dnnl_stream_wait then reports dnnl_runtime_error.
#include <cuda.h>

#include <cstddef>
#include <cstdlib>
#include <mutex>

#include "common.cuh"
#include "launch.hpp"

namespace b200 {

constexpr int BM = 128;          // rows of dst per tile (= TMEM lanes)
constexpr int BN = 256;          // columns of dst per tile (= one MMA's N)
constexpr int BK = 128;          // bytes of K per stage (= one 128-byte swizzle row)
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK; // 16 KiB
constexpr int B_BYTES = BN * BK; // 32 KiB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
// Pair kernel (two CTAs of a cluster on one 256 x 256 tile, tcgen05 cta_group::2): each CTA
// stages its 128 rows of A and its half of the tile's weight rows, so a stage is 32 KiB and six
// of them fit where the single-CTA kernel has four.
constexpr int PAIR_STAGES = 6;
constexpr int PAIR_B_BYTES = B_BYTES / 2;
constexpr int PAIR_STAGE_BYTES = A_BYTES + PAIR_B_BYTES;
constexpr int MAX_STAGES = 6;
constexpr int B_BOX_ROWS = 128;     // rows of one weights copy (TMA box) of the single-CTA kernel; a second map has 64-row boxes
constexpr int B_BOX_ROWS_SMALL = 64; // ... for units of BN / 4 columns and for the pair kernel (a CTA's share is half of the unit)
static_assert(PAIR_STAGES * PAIR_STAGE_BYTES == STAGES * STAGE_BYTES, "both kernels use the same shared memory");
constexpr int EPI_WARPS = 16;                 // four per TMEM lane quarter, each takes a quarter of the columns
constexpr int NUM_THREADS = 64 + 32 * EPI_WARPS;
constexpr int EPI_COLS = BN / (EPI_WARPS / 4); // columns per epilogue warp
constexpr int CH = 16;                        // columns per epilogue chunk (held in registers)
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t WAIT_TRIES = 1u << 20; // bounded wait: a million suspended waits of up to a microsecond
constexpr uint32_t WAIT_SPINS = 1u << 22; // drain loop of the producer: polls 64 ns apart
constexpr uint32_t POLL_TRIES = 1u << 26; // polling waits of the two issuing threads

enum : uint32_t { ST_WAIT_FULL = 0x1, ST_WAIT_EMPTY = 0x2, ST_WAIT_TMEM_FULL = 0x4, ST_WAIT_TMEM_EMPTY = 0x8 };

struct smem_ctrl_t {
    uint64_t full[MAX_STAGES];
    uint64_t empty[MAX_STAGES];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint32_t tmem_base;
    volatile uint32_t abort;
    // per epilogue warp: per-column vectors of its half of the current tile
    // (16-byte aligned: the epilogue reads these four columns at a time)
    alignas(16) float wscale[EPI_WARPS][EPI_COLS];   // weights scale, 1 when unset
    alignas(16) float wsx[EPI_WARPS][EPI_COLS];      // src scale x weights scale (approximate paths only)
    alignas(16) float bias[EPI_WARPS][EPI_COLS];     // bias, -0 when unset (x + -0 == x for every x)
    alignas(16) int32_t comp[EPI_WARPS][EPI_COLS];   // zp_src * colsum_W[n], 0 when unset
    alignas(16) float zp[EPI_WARPS][EPI_COLS];       // destination zero-point addend
    // gelu-into-8-bit fast path: constant term of the fused output expression and the
    // constant part of its error bound, per column
    alignas(16) float cq[EPI_WARPS][EPI_COLS];
    alignas(16) float hq[EPI_WARPS][EPI_COLS];
};

static_assert(offsetof(smem_ctrl_t, wscale) % 16 == 0 && offsetof(smem_ctrl_t, wsx) % 16 == 0 && offsetof(smem_ctrl_t, bias) % 16 == 0
                && offsetof(smem_ctrl_t, comp) % 16 == 0 && offsetof(smem_ctrl_t, zp) % 16 == 0
                && offsetof(smem_ctrl_t, cq) % 16 == 0 && offsetof(smem_ctrl_t, hq) % 16 == 0,
        "per-column vectors are read with 128-bit loads");
static_assert((EPI_COLS * sizeof(float)) % 16 == 0 && (CH * sizeof(float)) % 16 == 0, "chunk offsets keep the alignment");

constexpr size_t SMEM_BYTES = 1024 /* alignment slack */ + (size_t)STAGES * STAGE_BYTES + sizeof(smem_ctrl_t);

// ---- PTX wrappers ---------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(smem_u32(bar)), "r"(parity)
            : "memory");
    return ok != 0;
}
// one wait of at most about a microsecond, suspended in hardware: a waiting thread issues
// no instructions and makes no shared-memory accesses until the phase completes or the time
// runs out
__device__ __forceinline__ bool mbar_try(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(smem_u32(bar)), "r"(parity), "r"(1000u)
            : "memory");
    return ok != 0;
}
// bounded wait (of the order of a second); false when it ran out or another role already gave up
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, smem_ctrl_t *c, uint32_t *status, uint32_t code) {
    for (uint32_t i = 0; i < WAIT_TRIES; ++i) {
        if (mbar_try(bar, parity)) return true;
        if (c->abort) return false;
    }
    c->abort = 1;
    if (status) atomicOr(status, code);
    return false;
}

// The same wait by polling, for the copy-issuing and the MMA-issuing thread: their waits are
// part of every stage's round trip, and a poll sees the phase flip sooner than a suspended
// waiter is woken (C1: 2 us per launch).  Two single threads: the polls cost nothing else.
// Bounded like the other: 2^26 polls, of the order of a second.
__device__ __forceinline__ bool mbar_wait_poll(uint64_t *bar, uint32_t parity, smem_ctrl_t *c, uint32_t *status, uint32_t code) {
    for (uint32_t i = 0; i < POLL_TRIES; ++i) {
        if (mbar_test(bar, parity)) return true;
        if ((i & 63) == 63) {
            if (c->abort) return false;
            __nanosleep(20);
        }
    }
    c->abort = 1;
    if (status) atomicOr(status, code);
    return false;
}

__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, int c0, int c1, uint64_t *bar) {
    asm volatile(
            "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
            :
            : "r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
            : "memory");
}

__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tcgen05_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

// ---- two-CTA (cluster) forms ---------------------------------------------------------------

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// address of the same shared-memory location in the CTA with the given rank of this cluster
__device__ __forceinline__ uint32_t cluster_map(uint32_t saddr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load of the pair kernel: the bytes land in this CTA's shared memory, their count is
// reported to the barrier at bar_cluster_addr (the leader CTA's)
__device__ __forceinline__ void tma_load_2d_pair(void *dst, const CUtensorMap *map, int c0, int c1, uint32_t bar_cluster_addr) {
    asm volatile(
            "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
            :
            : "r"(smem_u32(dst)), "l"(map), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
            : "memory");
}
// completion of the leader's earlier MMAs arrives on the barrier at this offset in both CTAs
__device__ __forceinline__ void tcgen05_commit_pair(uint64_t *bar) {
    const uint16_t both = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
                         smem_u32(bar)),
                 "h"(both)
                 : "memory");
}
template <bool FP8>
__device__ __forceinline__ void tcgen05_mma_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
    const uint32_t z = 0;
    if (FP8) {
        asm volatile(
                "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
                :
                : "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc), "r"(z)
                : "memory");
    } else {
        asm volatile(
                "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
                :
                : "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc), "r"(z)
                : "memory");
    }
}

template <bool FP8>
__device__ __forceinline__ void tcgen05_mma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
    if (FP8) {
        asm volatile(
                "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
                :
                : "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
                : "memory");
    } else {
        asm volatile(
                "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
                :
                : "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
                : "memory");
    }
}

// 16 consecutive 32-bit columns of this thread's TMEM lane.  The load is asynchronous:
// the registers are valid only after tmem_ld_wait, which names them as operands so that
// the compiler cannot move a use above the wait.
__device__ __forceinline__ void tmem_ld16_issue(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
            : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
            "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
            : "r"(taddr)
            : "memory");
}
__device__ __forceinline__ void tmem_ld_wait(uint32_t (&v)[16]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7]), "+r"(v[8]),
                 "+r"(v[9]), "+r"(v[10]), "+r"(v[11]), "+r"(v[12]), "+r"(v[13]), "+r"(v[14]), "+r"(v[15])
                 :
                 : "memory");
}

// one 32-bit column of this thread's TMEM lane (interpreted epilogue, exact recomputation)
__device__ __forceinline__ uint32_t tmem_ld1(uint32_t taddr) {
    uint32_t v;
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(v) : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" : "+r"(v) : : "memory");
    return v;
}

// shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows of 128
// bytes, 8-row groups 1024 bytes apart (tile base 1024-byte aligned)
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3ffff) >> 4);  // start address, 16-byte units
    d |= (uint64_t)1 << 16;                   // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;         // stride byte offset
    d |= (uint64_t)1 << 46;                   // descriptor version for sm_100
    d |= (uint64_t)2 << 61;                   // SWIZZLE_128B
    return d;
}

struct tc8_args_t {
    b200_matmul_params_t p;
    int m_tiles, n_tiles, k_blocks;
    // Work units: unit u < full_units is tile u (BM x BN); the tiles after that -- those of a
    // last wave that fills at most half of the SMs, or all tiles of a problem that small -- are
    // each cut into `split` (2 or 4) units of BN / split columns, so that the work spreads
    // over that many more CTAs.
    int full_units, units, split;
    uint32_t idesc, idesc_tail; // instruction descriptors for N = BN and N = BN / split
};

struct unit_t {
    int m0, n0;   // origin of the unit in dst
    int width;    // columns: BN, BN / 2 or BN / 4
};

// rows: dst rows per tile (BM, or 2 * BM in the pair kernel)
__device__ __forceinline__ unit_t decode_unit(const tc8_args_t &a, int u, int rows) {
    unit_t r;
    int tile = u, off = 0;
    r.width = BN;
    if (u >= a.full_units) {
        const int h = u - a.full_units;
        r.width = BN / a.split;
        tile = a.full_units + h / a.split;
        off = (h % a.split) * r.width;
    }
    r.m0 = (tile % a.m_tiles) * rows; // m fastest
    r.n0 = (tile / a.m_tiles) * BN + off;
    return r;
}

// ---- epilogue on CH columns of one row ---------------------------------------------------
//
// The post-op chain is evaluated in one of four ways, chosen on the host:
//   EPI_NONE    no post-ops;
//   EPI_SIMPLE  only sum and non-transcendental eltwise kinds;
//   EPI_GELU_Q  [gelu_tanh] or [gelu_tanh, sum] into an s8 / u8 destination: see below;
//   EPI_GENERIC anything else: the interpreter shared with the generic kernel.
//
// The first three keep the CH values of a chunk in registers and are written
// without per-element branches, so that the compiler can interleave the CH
// independent dependency chains: an epilogue warp has at most one other warp on
// its scheduler to hide latency behind.  Unset scales / bias / zero-points are
// neutral elements (x * 1, x + -0) instead of branches.
//   EPI_SIMPLE_WZ  EPI_SIMPLE (or an empty chain) with weights zero-points: a kernel of its own so
//               that the others carry neither the extra registers nor the branch.
enum { EPI_NONE = 0, EPI_SIMPLE = 1, EPI_GELU_Q = 2, EPI_GENERIC = 3, EPI_SIMPLE_WZ = 4 };

// Coefficients of the error bound of the gelu-into-8-bit fast path, in units of the quantities
// they multiply (u = 2^-24 is one rounding):
//   TAU_G x |A x|: fast tanh (5e-7 |x|), x within 3 ulp (2e-7 |x| through gelu' <= 1.13),
//                  4 u from roundings of terms as large as the gelu term: 9.7e-7 needed;
//   TAU_S x |B old|: 4 u = 2.4e-7 needed (B, the sum term on both paths, its addition);
//   TAU_R x (range edge + |zp| + |B zp_sum|): 2 u = 1.2e-7 needed (the two last additions).
constexpr float TAU_G = 1.5e-6f, TAU_S = 3e-7f, TAU_R = 2e-7f;

struct epi_consts_t {
    float src_scale;   // 1 when unset; with per-row scales: this lane's row's
    bool src_per_row;  // the combined scale vector then holds the weights scales alone
    float dst_inv;     // 1 when unset
    bool any_sum;
    int sum_dt;
    bool int8_nondefault; // the int8 path adds the destination zero-point (0 when unset) whenever any attribute is set
    bool has_comp;        // a source zero-point is set: the per-column compensation vector is not all zero
    bool zp_uniform;      // the destination zero-point does not vary over columns: cq / hq below apply to every column
    float cq, hq;         // gelu-into-8-bit fast path with a uniform zero-point: its two per-column constants as scalars
    // Weights zero-points (int8): sum_k (s - zs)(w - zw[n]) = acc - zs colsum[n] - zw[n] rowsum[m] + zs zw[n] K.
    // The two terms that depend on the column alone are in the compensation vector; the epilogue
    // subtracts zw[n] * rowsum[m] (the zero-points travel in the cq[] vector, as integers: the
    // gelu-into-8-bit path, its only other user, is not chosen together with them).
    bool has_wzp;
    int rowsum;           // this lane's row's sum of src
};

// the exact gelu_tanh, kept out of line: it is needed for about one element in ten thousand
// and would otherwise sit in the middle of the hot epilogue code
__device__ __noinline__ float gelu_tanh_exact(float x) { return gelu_tanh_f32(x); }

// one non-transcendental eltwise kind applied to the CH values in registers
__device__ __forceinline__ void eltwise_simple_chunk(const b200_postop_t &e, float (&y)[CH]) {
    const float al = e.alpha, be = e.beta, sc = e.scale;
    switch (e.alg) {
        case ALG_RELU: case ALG_RELU_DST:
#pragma unroll
            for (int j = 0; j < CH; ++j) y[j] = __fmul_rn(y[j] > 0 ? y[j] : __fmul_rn(y[j], al), sc);
            break;
        case ALG_SQUARE:
#pragma unroll
            for (int j = 0; j < CH; ++j) y[j] = __fmul_rn(__fmul_rn(y[j], y[j]), sc);
            break;
        case ALG_ABS:
#pragma unroll
            for (int j = 0; j < CH; ++j) y[j] = __fmul_rn(y[j] > 0 ? y[j] : -y[j], sc);
            break;
        case ALG_SQRT: case ALG_SQRT_DST:
#pragma unroll
            for (int j = 0; j < CH; ++j) y[j] = __fmul_rn(__fsqrt_rn(y[j]), sc);
            break;
        case ALG_LINEAR:
#pragma unroll
            for (int j = 0; j < CH; ++j) y[j] = __fmul_rn(__fadd_rn(__fmul_rn(al, y[j]), be), sc);
            break;
        case ALG_HARDSIGMOID:
#pragma unroll
            for (int j = 0; j < CH; ++j) y[j] = __fmul_rn(hardsigmoid_f32(y[j], al, be), sc);
            break;
        case ALG_HARDSWISH:
#pragma unroll
            for (int j = 0; j < CH; ++j) y[j] = __fmul_rn(__fmul_rn(y[j], hardsigmoid_f32(y[j], al, be)), sc);
            break;
        case ALG_CLIP:
#pragma unroll
            for (int j = 0; j < CH; ++j) {
                const float t = y[j] > al ? y[j] : al;
                y[j] = __fmul_rn(t > be ? be : t, sc);
            }
            break;
        case ALG_ROUND:
#pragma unroll
            for (int j = 0; j < CH; ++j) y[j] = __fmul_rn(rintf(y[j]), sc);
            break;
        default: // clip_v2
#pragma unroll
            for (int j = 0; j < CH; ++j) {
                const float t = y[j] > al ? y[j] : al;
                y[j] = __fmul_rn(t < be ? t : be, sc);
            }
            break;
    }
}

// pack CH final f32 values of one row and store them (or the valid part of them)
__device__ __forceinline__ void store_row_at(const b200_matmul_params_t &p, const float (&y)[CH], char *drow, int64_t nvalid) {
    const bool aligned = nvalid == CH && ((uintptr_t)drow & 15) == 0;
    if (aligned && (p.dst_dt == B200_DT_S8 || p.dst_dt == B200_DT_U8)) {
        const bool is_s8 = p.dst_dt == B200_DT_S8;
        uint32_t w[CH / 4];
#pragma unroll
        for (int q = 0; q < CH / 4; ++q) {
            uint32_t r = 0;
#pragma unroll
            for (int b = 0; b < 4; ++b) r |= (is_s8 ? cvt_sat_s8(y[q * 4 + b]) : cvt_sat_u8(y[q * 4 + b])) << (8 * b);
            w[q] = r;
        }
        ((uint4 *)drow)[0] = make_uint4(w[0], w[1], w[2], w[3]);
    } else if (aligned && p.dst_dt == B200_DT_BF16) {
#pragma unroll
        for (int q = 0; q < CH / 8; ++q) {
            uint32_t w[4];
#pragma unroll
            for (int b = 0; b < 4; ++b)
                w[b] = (uint32_t)f32_to_bf16_bits(y[q * 8 + 2 * b]) | ((uint32_t)f32_to_bf16_bits(y[q * 8 + 2 * b + 1]) << 16);
            ((uint4 *)drow)[q] = make_uint4(w[0], w[1], w[2], w[3]);
        }
    } else if (aligned && p.dst_dt == B200_DT_F32) {
#pragma unroll
        for (int q = 0; q < CH / 4; ++q)
            ((float4 *)drow)[q] = make_float4(y[q * 4], y[q * 4 + 1], y[q * 4 + 2], y[q * 4 + 3]);
    } else {
#pragma unroll
        for (int j = 0; j < CH; ++j)
            if (j < nvalid) store_f32(p.dst_dt, y[j], drow, j);
    }
}

template <bool PEERS>
__device__ __forceinline__ void store_row(const b200_matmul_params_t &p, const float (&y)[CH], char *drow, int64_t nvalid) {
    if (nvalid <= 0) return;
    store_row_at(p, y, drow, nvalid);
}

// Kernels built for a destination mirrored on other GPUs: once a warp has stored its block of
// the tile (32 rows x EPI_COLS columns) locally, it reads the block back from L2 row by row
// and stores it at the same offset from every peer base, 16 bytes per lane with the lanes
// running along the row, so that what crosses NVLink are whole 64- to 256-byte row segments
// (one row of the block per store instruction for f32, two for bf16, four for 8-bit types)
// rather than the 16-byte pieces per row a lane holds after the epilogue.
__device__ __forceinline__ void mirror_block(const b200_matmul_params_t &p, int64_t row0, int64_t n0, int cols_max, int lane) {
    const int64_t rows = p.M - row0 < 32 ? p.M - row0 : 32;
    const int64_t cols = p.N - n0 < cols_max ? p.N - n0 : cols_max;
    if (rows <= 0 || cols <= 0) return;
    const int eb = dt_bits(p.dst_dt) / 8;
    const int64_t pitch = p.dst_sm * eb, row_bytes = cols * eb;
    const int64_t off0 = (row0 * p.dst_sm + n0) * eb;
    const char *base = (const char *)p.dst + off0;
    __syncwarp(); // the lanes' stores of this block are ordered before the reads below
    if ((((uintptr_t)base | (uintptr_t)pitch | (uintptr_t)row_bytes) & 15) == 0) {
        const int vecs = (int)(row_bytes >> 4);
        const int total = (int)rows * vecs;
        for (int i = lane; i < total; i += 32) {
            const int r = i / vecs, v = i - r * vecs;
            const int64_t off = r * pitch + v * 16;
            const uint4 val = __ldcg(reinterpret_cast<const uint4 *>(base + off));
            for (int q = 0; q < p.n_dst_peers; ++q) *reinterpret_cast<uint4 *>((char *)p.dst_peer[q] + off0 + off) = val;
        }
    } else {
        const int64_t total = rows * row_bytes;
        for (int64_t i = lane; i < total; i += 32) {
            const int64_t r = i / row_bytes, off = r * pitch + (i - r * row_bytes);
            const unsigned char val = __ldcg(reinterpret_cast<const unsigned char *>(base + off));
            for (int q = 0; q < p.n_dst_peers; ++q) ((unsigned char *)p.dst_peer[q])[off0 + off] = val;
        }
    }
}

// SUM: how the sum post-op's prior destination values are obtained
//   0 no sum;  1 the sum type is s8 / u8: 16 bytes per chunk, kept packed in four registers;
//   2 any other sum type: converted to f32 up front.
enum { SUM_NONE = 0, SUM_8BIT = 1, SUM_OTHER = 2 };

template <bool FP8, int EPI, int SUM, bool PEERS>
__device__ __forceinline__ void epilogue_chunk(const b200_matmul_params_t &p, const uint32_t (&v)[CH], int64_t m,
        int64_t n0, const float *wscale, const float *wsx, const float *bias, const int32_t *comp, const float *zp, const float *cq,
        const float *hq, const epi_consts_t &k, uint32_t taddr, int lane, uint4 old_raw, bool old_prefetched) {
    const int64_t nvalid = m < p.M ? (p.N - n0 < CH ? p.N - n0 : CH) : 0;
    char *drow = (char *)p.dst + (size_t)((m < p.M ? m : 0) * p.dst_sm + n0) * (dt_bits(p.dst_dt) / 8);

    // Prior destination values.  All control flow happens here, once per chunk; the element
    // loops below are straight-line so that the compiler can interleave the CH chains.
    uint32_t ow[4] = {old_raw.x, old_raw.y, old_raw.z, old_raw.w};
    float oldf[SUM == SUM_OTHER ? CH : 1];
    if (SUM == SUM_8BIT && !old_prefetched) {
        // ragged or unaligned row: gather the bytes one by one into the same packed form
#pragma unroll
        for (int q = 0; q < 4; ++q) ow[q] = 0;
#pragma unroll
        for (int j = 0; j < CH; ++j) // unrolled: a run-time index would push the array to local memory
            if (j < nvalid) ow[j >> 2] |= (uint32_t)((const uint8_t *)drow)[j] << ((j & 3) * 8);
    }
    if (SUM == SUM_OTHER) {
#pragma unroll
        for (int j = 0; j < CH; ++j) oldf[j] = j < nvalid ? load_f32(k.sum_dt, drow, j) : 0.f;
    }
    // byte b of a packed word, sign- or zero-extended by one byte permute: selector nibble
    // 8|b replicates the byte's sign bit, nibble 4 picks a zero byte of the second operand
    // Byte b of a packed word as a float without an int-to-float conversion (those share a
    // quarter-rate pipe with the exponentials and the final conversions of this epilogue): s8
    // bytes are biased to 0..255 by flipping their sign bits, one byte permute drops the byte
    // into the low mantissa bits of 2^23, and subtracting 2^23 (+ 128) leaves its value, exactly.
    if (SUM == SUM_8BIT && k.sum_dt == B200_DT_S8) {
#pragma unroll
        for (int q = 0; q < 4; ++q) ow[q] ^= 0x80808080u;
    }
    const float unbias = k.sum_dt == B200_DT_S8 ? 8388736.f : 8388608.f;
    auto old_val = [&](int j) -> float {
        if (SUM == SUM_OTHER) return oldf[j];
        uint32_t e;
        asm("prmt.b32 %0, %1, %2, %3;" : "=r"(e) : "r"(ow[j >> 2]), "r"(0x4b000000u), "r"(0x7440u | (uint32_t)(j & 3)));
        return __uint_as_float(e) - unbias;
    };

    // per-column vectors of the chunk as 128-bit shared-memory reads
    if (EPI == EPI_GENERIC) {
        // interpreted chain: one copy of the code in a rolled loop over the chunk; each
        // column of the accumulator is read from tensor memory when its turn comes
#pragma unroll 1
        for (int j = 0; j < CH; ++j) {
            const uint32_t raw = tmem_ld1(taddr + j);
            if (j >= nvalid) continue;
            const float acc = FP8 ? __uint_as_float(raw)
                                  : (float)((int)raw - comp[j] - (k.has_wzp ? __float_as_int(cq[j]) * k.rowsum : 0));
            float x = __fadd_rn(__fmul_rn(__fmul_rn(acc, k.src_scale), wscale[j]), bias[j]);
            if (p.bias && p.bias_sm) // a bias that varies along M is not part of the per-column vector
                x = __fadd_rn(x, load_f32(p.bias_dt, p.bias, m * p.bias_sm + (n0 + j) * p.bias_sn));
            const float o = k.any_sum ? load_f32(k.sum_dt, drow, j) : 0.f;
            x = __fmul_rn(apply_post_ops(p, x, o, m, n0 + j), k.dst_inv);
            if (!FP8) x = __fadd_rn(x, zp[j]);
            store_f32(p.dst_dt, x, drow, j);
        }
        return;
    }

    if (EPI == EPI_GELU_Q) {
        // gelu_tanh (then optionally sum) into an s8 / u8 destination, bit-exact.  The exact
        // value needs a double-precision tanh; almost always it is not needed: evaluate a fast
        // value o with a fast tanh (ex2 / rcp: 1 / (exp(2g) + 1) with absolute error below 1e-6
        // on the whole range, 0 and 1 at the far ends) and fused multiply-adds, bound its
        // distance tau from the exact value, and convert both o + tau and o - tau with the
        // saturating round-to-nearest-even conversion.  If the two bytes agree, the exact value
        // -- which lies between them -- converts to the same byte, saturation included; only
        // elements where they differ are recomputed exactly (one warp vote per chunk).
        // The chunk is handled as two independent halves of eight columns, each a sequence
        // of passes of eight independent operations, ending in packed bytes: short live
        // ranges, no per-element control flow.
        // Fast value: with A = elt_scale / dst_scale, B = sum_scale / dst_scale and the per-column
        // constant C = zp_dst - B * zp_sum (cq[]), o = gelu(x) * A + old * B + C in two fused
        // multiply-adds.  Its distance from the exact value is at most
        //   tau = TAU_G |A| |x| + TAU_S |B| |old| + TAU_R (R + |zp_dst| + |B| |zp_sum|)   (last term: hq[])
        // with R the edge of the destination range: beyond it both conversions saturate to the
        // same byte whatever tau is.
        const float elt_scale = p.po[0].scale;
        const float sum_scale = SUM != SUM_NONE ? p.po[1].scale : 0.f;
        const float sum_zp = SUM != SUM_NONE ? (float)p.po[1].zero_point : 0.f;
        const float A = elt_scale * k.dst_inv, B = sum_scale * k.dst_inv;
        const float inv_abs = TAU_G * fabsf(A), c2 = TAU_S * fabsf(B);
        const bool is_s8 = p.dst_dt == B200_DT_S8;
        // 2 log2(e) folded into the polynomial: exp(2 g) = 2^(gl x + gc x^3)
        const float gl = 2.885390081777927f * 0.79788458347320556640625f, gc = gl * 0.044715f;
        static_assert(CH == 16, "four packed words per chunk");
        uint32_t packed[4];
        uint32_t risky = 0;
#pragma unroll
        for (int hb = 0; hb < CH; hb += 8) {
            float x[8], t[8], o[8], tau[8];
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                const float4 a = ((const float4 *)wsx)[hb / 4 + q], b = ((const float4 *)bias)[hb / 4 + q];
                const float ws[4] = {a.x, a.y, a.z, a.w}, bs[4] = {b.x, b.y, b.z, b.w};
                int cs[4] = {0, 0, 0, 0};
                if (!FP8 && k.has_comp) { // warp-uniform: the vector is read only when a source zero-point exists
                    const int4 c = ((const int4 *)comp)[hb / 4 + q];
                    cs[0] = c.x; cs[1] = c.y; cs[2] = c.z; cs[3] = c.w;
                }
                float accf[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) accf[i] = FP8 ? __uint_as_float(v[hb + 4 * q + i]) : (float)((int)v[hb + 4 * q + i] - cs[i]);
                if (k.src_per_row) { // the row's scale is not part of the combined vector
#pragma unroll
                    for (int i = 0; i < 4; ++i) accf[i] *= k.src_scale;
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) x[4 * q + i] = fmaf(accf[i], ws[i], bs[i]); // within 3 ulp of the reference's unfused value
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float e2 = x[j] * fmaf(gc, x[j] * x[j], gl);
                float ex;
                asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(ex) : "f"(e2));
                asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(t[j]) : "f"(ex + 1.f)); // r = 1 / (exp(2g) + 1): tanh(g) = 1 - 2r
            }
            float cv[8], hv[8];
            if (k.zp_uniform) {
#pragma unroll
                for (int j = 0; j < 8; ++j) cv[j] = k.cq, hv[j] = k.hq;
            } else {
                const float4 c0 = ((const float4 *)cq)[hb / 4], c1 = ((const float4 *)cq)[hb / 4 + 1];
                const float4 h0 = ((const float4 *)hq)[hb / 4], h1 = ((const float4 *)hq)[hb / 4 + 1];
                cv[0] = c0.x; cv[1] = c0.y; cv[2] = c0.z; cv[3] = c0.w; cv[4] = c1.x; cv[5] = c1.y; cv[6] = c1.z; cv[7] = c1.w;
                hv[0] = h0.x; hv[1] = h0.y; hv[2] = h0.z; hv[3] = h0.w; hv[4] = h1.x; hv[5] = h1.y; hv[6] = h1.z; hv[7] = h1.w;
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float gelu = fmaf(-x[j], t[j], x[j]); // 0.5 x (1 + tanh) = x - x r
                float s = cv[j];
                tau[j] = fmaf(inv_abs, fabsf(x[j]), hv[j]);
                if (SUM != SUM_NONE) {
                    const float old = old_val(hb + j);
                    s = fmaf(old, B, s);
                    tau[j] = fmaf(c2, fabsf(old), tau[j]);
                }
                o[j] = fmaf(gelu, A, s);
            }
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                int up[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int j = 4 * q + i;
                    int dn;
                    if (is_s8) {
                        asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(up[i]) : "f"(o[j] + tau[j]));
                        asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(dn) : "f"(o[j] - tau[j]));
                    } else {
                        asm("cvt.rni.sat.u8.f32 %0, %1;" : "=r"(up[i]) : "f"(o[j] + tau[j]));
                        asm("cvt.rni.sat.u8.f32 %0, %1;" : "=r"(dn) : "f"(o[j] - tau[j]));
                    }
                    if (up[i] != dn) risky |= 1u << (hb + j);
                }
                // low bytes of the four results into one word
                uint32_t lo, hi, w;
                asm("prmt.b32 %0, %1, %2, 0x0040;" : "=r"(lo) : "r"(up[0]), "r"(up[1]));
                asm("prmt.b32 %0, %1, %2, 0x0040;" : "=r"(hi) : "r"(up[2]), "r"(up[3]));
                asm("prmt.b32 %0, %1, %2, 0x5410;" : "=r"(w) : "r"(lo), "r"(hi));
                packed[hb / 4 + q] = w;
            }
        }
        if (__any_sync(0xffffffffu, risky != 0)) {
            // Exact recomputation of the flagged columns (column index known only at run
            // time).  The accumulator is still in tensor memory: it is read again, one column
            // at a time, by the whole warp; lanes that did not flag the column discard it.
            const uint32_t any_mask = __reduce_or_sync(0xffffffffu, risky);
#pragma unroll 1
            for (int j = 0; j < CH; ++j) {
                if (!(any_mask & (1u << j))) continue;
                const uint32_t raw = tmem_ld1(taddr + j);
                if (!(risky & (1u << j))) continue;
                const float acc = FP8 ? __uint_as_float(raw) : (float)((int)raw - comp[j]);
                const float xj = __fadd_rn(__fmul_rn(__fmul_rn(acc, k.src_scale), wscale[j]), bias[j]);
                float r = __fmul_rn(gelu_tanh_exact(xj), elt_scale);
                if (SUM != SUM_NONE)
                    r = __fadd_rn(r, __fmul_rn(sum_scale, __fsub_rn(j < nvalid ? load_f32(k.sum_dt, drow, j) : 0.f, sum_zp)));
                r = __fmul_rn(r, k.dst_inv);
                if (!FP8) r = __fadd_rn(r, zp[j]);
                const uint32_t byte = is_s8 ? cvt_sat_s8(r) : cvt_sat_u8(r);
                const int sh = (j & 3) * 8;
                const uint32_t keep = ~(0xffu << sh), put = byte << sh;
                const int q = j >> 2;
                packed[0] = q == 0 ? (packed[0] & keep) | put : packed[0];
                packed[1] = q == 1 ? (packed[1] & keep) | put : packed[1];
                packed[2] = q == 2 ? (packed[2] & keep) | put : packed[2];
                packed[3] = q == 3 ? (packed[3] & keep) | put : packed[3];
            }
        }
        if (nvalid == CH && ((uintptr_t)drow & 15) == 0) {
            ((uint4 *)drow)[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
        } else {
#pragma unroll
            for (int j = 0; j < CH; ++j)
                if (j < nvalid) ((uint8_t *)drow)[j] = (uint8_t)(packed[j >> 2] >> ((j & 3) * 8));
        }
        return;
    }

    // accumulator -> scaled value + bias (neutral elements where unset), four columns per
    // 128-bit shared-memory read of each per-column vector
    float y[CH];
#pragma unroll
    for (int q = 0; q < CH / 4; ++q) {
        const float4 a = ((const float4 *)wscale)[q], b = ((const float4 *)bias)[q];
        const int4 c = ((const int4 *)comp)[q];
        const float ws[4] = {a.x, a.y, a.z, a.w}, bs[4] = {b.x, b.y, b.z, b.w};
        int cs[4] = {c.x, c.y, c.z, c.w};
        if (!FP8 && EPI == EPI_SIMPLE_WZ) {
            const int4 z = ((const int4 *)cq)[q];
            cs[0] += z.x * k.rowsum; cs[1] += z.y * k.rowsum; cs[2] += z.z * k.rowsum; cs[3] += z.w * k.rowsum;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int j = 4 * q + i;
            const float x = FP8 ? __uint_as_float(v[j]) : (float)((int)v[j] - cs[i]);
            y[j] = __fadd_rn(__fmul_rn(__fmul_rn(x, k.src_scale), ws[i]), bs[i]);
        }
    }
    // destination scale and zero-point (zp[] holds -0 when no zero-point is to be added)
    auto tail = [&](float x, int j) -> float {
        x = __fmul_rn(x, k.dst_inv);
        return FP8 ? x : __fadd_rn(x, zp[j]);
    };

    if (EPI == EPI_NONE) {
#pragma unroll
        for (int j = 0; j < CH; ++j) y[j] = tail(y[j], j);
    } else if (EPI == EPI_SIMPLE || EPI == EPI_SIMPLE_WZ) {
        for (int i = 0; i < p.npo; ++i) {
            const b200_postop_t &e = p.po[i];
            if (e.kind == B200_PO_SUM) {
                if (SUM != SUM_NONE) {
                    const float sc = e.scale, z = (float)e.zero_point;
#pragma unroll
                    for (int j = 0; j < CH; ++j) y[j] = __fadd_rn(y[j], __fmul_rn(sc, __fsub_rn(old_val(j), z)));
                }
            } else {
                eltwise_simple_chunk(e, y);
            }
        }
#pragma unroll
        for (int j = 0; j < CH; ++j) y[j] = tail(y[j], j);
    }
    store_row<PEERS>(p, y, drow, nvalid);
}

// ---- the kernel -------------------------------------------------------------------------

// 18 warps land 5 + 5 + 4 + 4 on the four schedulers, so a thread may use at most
// 16384 / (5 * 32) = 102 registers; declaring 640 threads makes ptxas stay within that.
//
// PAIR: the two CTAs of a cluster compute one tile of 2 * BM rows together (tcgen05
// cta_group::2).  CTA r stages rows [r * BM, +BM) of the tile's activations and half r of its
// weight rows; all copies report to the leader's (rank 0) full barriers; the leader's thread
// issues the MMAs, which read both CTAs' shared memory and write each CTA's rows into that
// CTA's tensor memory; its commits arrive on the empty / accumulator-ready barriers of both
// CTAs; each CTA's epilogue warps convert its own rows and arrive on the leader's
// accumulator-free barrier.  Per tile this moves 2/3 of the bytes from L2 to shared memory.
template <bool FP8, int EPI, int SUM, bool PEERS = false, bool PAIR = false>
__global__ void __launch_bounds__(640, 1) matmul_tc8_kernel(const __grid_constant__ CUtensorMap tmap_a,
        const __grid_constant__ CUtensorMap tmap_b, const __grid_constant__ CUtensorMap tmap_b_small,
        const __grid_constant__ tc8_args_t args) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    smem_ctrl_t *ctrl = (smem_ctrl_t *)(smem + (size_t)STAGES * STAGE_BYTES);
    const b200_matmul_params_t &p = args.p;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int KB = args.k_blocks;
    constexpr int NST = PAIR ? PAIR_STAGES : STAGES;
    constexpr int SBYTES = PAIR ? PAIR_STAGE_BYTES : STAGE_BYTES;   // one stage
    constexpr int BBYTES = PAIR ? PAIR_B_BYTES : B_BYTES;           // its weights part (wide unit)
    const uint32_t rank = PAIR ? cluster_ctarank() : 0;             // 0: leader
    // this CTA's (pair's) first unit and the stride over units
    const int unit0 = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x, ustep = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
    constexpr int TILE_ROWS = PAIR ? 2 * BM : BM;

    if (threadIdx.x == 0) {
        for (int s = 0; s < NST; ++s) {
            mbar_init(&ctrl->full[s], 1);
            mbar_init(&ctrl->empty[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&ctrl->tmem_full[a], 1);
            mbar_init(&ctrl->tmem_empty[a], PAIR ? 2 * EPI_WARPS : EPI_WARPS); // the pair's leader hears from both CTAs
        }
        ctrl->abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        if (PAIR) { // the same warp of both CTAs, together
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctrl->tmem_base)),
                         "r"(TMEM_COLS)
                         : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctrl->tmem_base)),
                         "r"(TMEM_COLS)
                         : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (PAIR) cluster_sync_all(); // both CTAs' barriers exist before either signals the other's
    tcgen05_fence_after();
    const uint32_t tmem_base = ctrl->tmem_base;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int u = unit0; u < args.units && ok; u += ustep) {
                const unit_t un = decode_unit(args, u, TILE_ROWS);
                for (int kb = 0; kb < KB; ++kb, ++it) {
                    const uint32_t s = it % NST, r = it / NST;
                    if (!(ok = mbar_wait_poll(&ctrl->empty[s], (r & 1) ^ 1, ctrl, p.status, ST_WAIT_EMPTY))) break;
                    uint8_t *sa = smem + (size_t)s * SBYTES;
                    // This CTA's share of the unit's weight rows (all of them, or half in the pair
                    // kernel) is one or two boxes: of 128 rows, or of 64 (second map) where the share
                    // is 64 rows and in the pair kernel.  Straight-line code: in the pair kernel the
                    // time this thread takes per stage is part of the stage's round trip.
                    if (PAIR) {
                        // the leader's barrier counts the bytes of both CTAs
                        const uint32_t bar = cluster_map(smem_u32(&ctrl->full[s]), 0);
                        const bool two = un.width == BN; // 128 rows per CTA: two boxes of 64
                        if (rank == 0) mbar_expect_tx(&ctrl->full[s], 2 * (A_BYTES + (two ? 2 : 1) * B_BOX_ROWS_SMALL * BK));
                        tma_load_2d_pair(sa, &tmap_a, kb * BK, un.m0 + (int)rank * BM, bar);
                        const int nb = un.n0 + (int)rank * (un.width / 2);
                        tma_load_2d_pair(sa + A_BYTES, &tmap_b_small, kb * BK, nb, bar);
                        if (two) tma_load_2d_pair(sa + A_BYTES + B_BOX_ROWS_SMALL * BK, &tmap_b_small, kb * BK, nb + B_BOX_ROWS_SMALL, bar);
                    } else {
                        mbar_expect_tx(&ctrl->full[s], A_BYTES + (uint32_t)un.width * BK);
                        tma_load_2d(sa, &tmap_a, kb * BK, un.m0, &ctrl->full[s]);
                        if (un.width >= B_BOX_ROWS) {
                            tma_load_2d(sa + A_BYTES, &tmap_b, kb * BK, un.n0, &ctrl->full[s]);
                            if (un.width == BN) tma_load_2d(sa + A_BYTES + B_BOX_ROWS * BK, &tmap_b, kb * BK, un.n0 + B_BOX_ROWS, &ctrl->full[s]);
                        } else {
                            tma_load_2d(sa + A_BYTES, &tmap_b_small, kb * BK, un.n0, &ctrl->full[s]);
                        }
                    }
                }
            }
            // drain: every copy issued must have landed before the CTA may exit.  In the pair
            // kernel the leader's barriers cover both CTAs' copies, and the other CTA stays
            // until the leader has passed the cluster barrier at the end.
            const uint32_t issued = it;
            for (uint32_t j = issued > NST ? issued - NST : 0; j < issued && rank == 0; ++j) {
                const uint32_t s = j % NST, r = j / NST;
                for (uint32_t i = 0; i < WAIT_SPINS; ++i) {
                    if (mbar_test(&ctrl->full[s], r & 1)) break;
                    __nanosleep(64);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0 && rank == 0) {
            uint32_t tile_i = 0;
            bool ok = true;
            bool early = false;       // the early look's answer for the k-block at hand
            uint32_t st = 0, par = 0; // stage of the k-block at hand and the parity of its fill
            // descriptors of stage 0; a stage further on is STAGE_BYTES / 16 more in the address field,
            // a k-step of 32 bytes 2 more
            const uint64_t adesc0 = make_smem_desc(smem_u32(smem)), bdesc0 = make_smem_desc(smem_u32(smem) + A_BYTES);
            constexpr bool FULLDESC = NST <= 4;
            constexpr int DK = FULLDESC ? BK / 32 : 1;
            uint64_t adesc[NST][DK], bdesc[NST][DK];
#pragma unroll
            for (int s = 0; s < NST; ++s)
#pragma unroll
                for (int k = 0; k < DK; ++k) {
                    adesc[s][k] = adesc0 + (uint64_t)(s * (SBYTES >> 4) + 2 * k);
                    bdesc[s][k] = bdesc0 + (uint64_t)(s * (SBYTES >> 4) + 2 * k);
                }
            for (int u = unit0; u < args.units && ok; u += ustep, ++tile_i) {
                const uint32_t a = tile_i & 1, use = tile_i >> 1;
                const uint32_t idesc = u < args.full_units ? args.idesc : args.idesc_tail;
                if (!(ok = mbar_wait_poll(&ctrl->tmem_empty[a], (use & 1) ^ 1, ctrl, p.status, ST_WAIT_TMEM_EMPTY))) break;
                tcgen05_fence_after();
                const uint32_t tmem_d = tmem_base + a * BN;
                // This thread's loop is what the tensor pipe waits for, and it shares its scheduler with
                // four epilogue warps: once those are busy every instruction here takes about twice as
                // long, and a k-block whose four MMAs keep the pipe busy for 550 cycles took 900 to issue.
                // So the loop is unrolled over the stages of the ring, with the operand descriptors of
                // every stage and k-step held in registers (the single-CTA kernel; the pair kernel, with
                // six stages, keeps one per stage and adds the k-step): no index or descriptor arithmetic
                // is left per k-block.  And since a look at a barrier costs a few hundred cycles even when
                // its phase completed long ago, the look for k-block i + 1 is issued before the MMAs of
                // k-block i and its answer read after them; the thread polls only when that early look
                // said "not yet" (the look is unambiguous: the phase before the one asked about belongs to
                // a block this thread has already consumed; looking two blocks ahead was slower again).
                // No tcgen05 fence per k-block: the operands are in shared memory, written through the
                // async proxy and ordered by the barrier; the fence belongs where tensor memory changes
                // hands (above).
                for (int kb = 0; kb < KB && ok;) {
#pragma unroll
                    for (int s = 0; s < NST; ++s) {
                        if (st == (uint32_t)s && kb < KB && ok) {
                            if (!early) ok = mbar_wait_poll(&ctrl->full[s], par, ctrl, p.status, ST_WAIT_FULL);
                            if (ok) {
                                const int s2 = (s + 1) % NST; // a constant in each unrolled copy
                                const uint32_t par2 = s2 == 0 ? par ^ 1u : par;
                                const bool next_early = mbar_test(&ctrl->full[s2], par2);
#pragma unroll
                                for (int k = 0; k < BK / 32; ++k) { // 32 bytes of K per instruction: +2 in 16-byte units
                                    const uint64_t ad = FULLDESC ? adesc[s][k] : adesc[s][0] + 2 * k;
                                    const uint64_t bd = FULLDESC ? bdesc[s][k] : bdesc[s][0] + 2 * k;
                                    if (PAIR) tcgen05_mma_pair<FP8>(tmem_d, ad, bd, idesc, (kb | k) != 0);
                                    else tcgen05_mma<FP8>(tmem_d, ad, bd, idesc, (kb | k) != 0);
                                }
                                if (PAIR) tcgen05_commit_pair(&ctrl->empty[s]);
                                else tcgen05_commit(&ctrl->empty[s]);
                                early = next_early;
                                st = (uint32_t)s2;
                                par = par2;
                                ++kb;
                            }
                        }
                    }
                }
                if (ok) {
                    if (PAIR) tcgen05_commit_pair(&ctrl->tmem_full[a]);
                    else tcgen05_commit(&ctrl->tmem_full[a]);
                }
            }
        }
    } else {
        // ---------------- epilogue warps ----------------
        const int ew = warp - 2;           // 0..15
        const int quarter = warp & 3;      // TMEM lanes this warp may read: 32*quarter .. +31
        const int half = ew >> 2;          // which quarter of the tile's columns this warp converts
        float *wscale = ctrl->wscale[ew], *wsx = ctrl->wsx[ew], *bias = ctrl->bias[ew], *zpv = ctrl->zp[ew];
        int32_t *comp = ctrl->comp[ew];
        float *cqv = ctrl->cq[ew], *hqv = ctrl->hq[ew];
        const bool has_comp = !FP8 && p.src_zp.ptr && p.wei_colsum;
        const int zp_src = has_comp ? load_int(p.src_zp.dt, p.src_zp.ptr, 0) : 0;
        epi_consts_t k;
        k.src_per_row = p.src_scale.ptr && p.src_scale.s0 != 0;
        const float src_scale_all = (p.src_scale.ptr && !k.src_per_row) ? load_f32(p.src_scale.dt, p.src_scale.ptr, 0) : 1.f;
        k.src_scale = src_scale_all;
        k.dst_inv = dst_scale_reciprocal(p);
        k.any_sum = has_sum(p);
        k.sum_dt = sum_dt_of(p);
        k.int8_nondefault = !FP8
                && (p.npo > 0 || p.src_scale.ptr || p.wei_scale.ptr || p.dst_scale.ptr || p.src_zp.ptr || p.wei_zp.ptr
                        || p.dst_zp.ptr);
        const bool bias_per_col = p.bias && !p.bias_sm;
        k.has_comp = has_comp;
        k.has_wzp = !FP8 && (EPI == EPI_SIMPLE_WZ || EPI == EPI_GENERIC) && p.wei_zp.ptr && p.src_rowsum;
        k.rowsum = 0;
        k.zp_uniform = !(p.dst_zp.ptr && p.dst_zp.s1);
        k.cq = k.hq = 0.f;
        if (EPI == EPI_GELU_Q && k.zp_uniform) {
            const float z = !k.int8_nondefault ? -0.f : p.dst_zp.ptr ? (float)((const int32_t *)p.dst_zp.ptr)[0] : 0.f;
            const float bz = SUM != SUM_NONE ? p.po[1].scale * k.dst_inv * (float)p.po[1].zero_point : 0.f;
            k.cq = z - bz;
            k.hq = TAU_R * ((p.dst_dt == B200_DT_S8 ? 130.f : 258.f) + fabsf(z) + fabsf(bz));
        }
        uint32_t tile_i = 0;
        bool ok = true;
        for (int u = unit0; u < args.units && ok; u += ustep, ++tile_i) {
            const unit_t un = decode_unit(args, u, TILE_ROWS);
            if (SUM != SUM_NONE && u + ustep < args.units) {
                // The prior destination bytes of the NEXT unit, asked into L2 now: when the epilogue
                // is the slower side the accumulator is already waiting at the top of a unit, and
                // the first read of those bytes would otherwise sit in the open with its DRAM latency.
                const unit_t nx = decode_unit(args, u + ustep, TILE_ROWS);
                const int64_t nm = nx.m0 + (int64_t)rank * BM + quarter * 32 + lane;
                const int64_t nn = (int64_t)nx.n0 + half * (nx.width / 4);
                if (nm < p.M && nn < p.N) {
                    const char *pf = (const char *)p.dst + (size_t)(nm * p.dst_sm + nn) * (dt_bits(sum_dt_of(p)) / 8);
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(pf));
                }
            }
            // this warp's share of the unit's columns: a quarter of them, in chunks of CH
            const int ecols = un.width / 4, nch = ecols / CH;
            const int64_t m0 = un.m0 + (int64_t)rank * BM;
            const int64_t n0 = (int64_t)un.n0 + half * ecols;
            const uint32_t a = tile_i & 1, use = tile_i >> 1;
            // per-column vectors of this warp's columns
            __syncwarp();
            for (int j = lane; j < ecols; j += 32) {
                const int64_t n = n0 + j;
                const bool in = n < p.N;
                wscale[j] = (in && p.wei_scale.ptr) ? load_f32(p.wei_scale.dt, p.wei_scale.ptr, n * p.wei_scale.s1) : 1.f;
                wsx[j] = wscale[j] * src_scale_all;
                bias[j] = (in && bias_per_col) ? load_f32(p.bias_dt, p.bias, n * p.bias_sn) : -0.f;
                comp[j] = (in && has_comp) ? zp_src * p.wei_colsum[n] : 0;
                if ((EPI == EPI_SIMPLE_WZ || EPI == EPI_GENERIC) && k.has_wzp) {
                    const int zw = in ? load_int(p.wei_zp.dt, p.wei_zp.ptr, n * p.wei_zp.s1) : 0;
                    cqv[j] = __int_as_float(zw);
                    comp[j] -= zp_src * zw * (int)p.K; // wraps like the sum it is part of; the total is exact whenever it fits 32 bits
                }
                // the int8 path adds the zero-point (+0 when unset) whenever any attribute is set; -0 adds nothing
                zpv[j] = !k.int8_nondefault ? -0.f
                        : (in && p.dst_zp.ptr) ? (float)((const int32_t *)p.dst_zp.ptr)[p.dst_zp.s1 ? n : 0] : 0.f;
                if (EPI == EPI_GELU_Q) {
                    const float bz = SUM != SUM_NONE ? p.po[1].scale * k.dst_inv * (float)p.po[1].zero_point : 0.f;
                    cqv[j] = zpv[j] - bz;
                    hqv[j] = TAU_R * ((p.dst_dt == B200_DT_S8 ? 130.f : 258.f) + fabsf(zpv[j]) + fabsf(bz));
                }
            }
            __syncwarp();
            const int64_t m = m0 + quarter * 32 + lane;
            if (k.src_per_row) k.src_scale = m < p.M ? ((const float *)p.src_scale.ptr)[m] : 1.f;
            if ((EPI == EPI_SIMPLE_WZ || EPI == EPI_GENERIC) && k.has_wzp) k.rowsum = m < p.M ? p.src_rowsum[m] : 0;
            const uint32_t trow = tmem_base + ((uint32_t)(quarter * 32) << 16) + a * BN + half * ecols;
            // Prior destination bytes of this warp's columns (sum post-op): requested now, for
            // the whole tile, so that the DRAM latency passes while the accumulator is still
            // being computed.  One aligned 16-byte read per chunk where that is possible.
            constexpr int NCH = EPI_COLS / CH;
            const char *drow0 = (const char *)p.dst + (size_t)((m < p.M ? m : 0) * p.dst_sm + n0) * (dt_bits(p.dst_dt) / 8);
            const bool sum8 = SUM == SUM_8BIT && EPI != EPI_GENERIC && m < p.M && (((uintptr_t)drow0) & 15) == 0;
            static_assert(NCH == 4, "the prefetch registers below are named for four chunks");
            uint4 ob0 = make_uint4(0, 0, 0, 0), ob1 = ob0, ob2 = ob0, ob3 = ob0;
            const bool of0 = sum8 && n0 + 1 * CH <= p.N, of1 = sum8 && n0 + 2 * CH <= p.N;
            const bool of2 = sum8 && nch > 2 && n0 + 3 * CH <= p.N, of3 = sum8 && nch > 2 && n0 + 4 * CH <= p.N;
            if (of0) ob0 = *(const uint4 *)(drow0);
            if (of1) ob1 = *(const uint4 *)(drow0 + CH);
            if (of2) ob2 = *(const uint4 *)(drow0 + 2 * CH);
            if (of3) ob3 = *(const uint4 *)(drow0 + 3 * CH);
            uint32_t ofbits = (of0 ? 1u : 0u) | (of1 ? 2u : 0u) | (of2 ? 4u : 0u) | (of3 ? 8u : 0u);
            ok = mbar_wait(&ctrl->tmem_full[a], use & 1, ctrl, p.status, ST_WAIT_TMEM_FULL);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tcgen05_fence_after();
            // one copy of the chunk code, executed once per chunk (the unrolled form does not fit
            // the instruction cache); the prefetched bytes rotate through named registers
#pragma unroll 1
            for (int c = 0; c < nch; ++c) {
                uint32_t v[CH];
                tmem_ld16_issue(trow + c * CH, v);
                tmem_ld_wait(v);
                epilogue_chunk<FP8, EPI, SUM, PEERS>(p, v, m, n0 + c * CH, wscale + c * CH, wsx + c * CH, bias + c * CH, comp + c * CH, zpv + c * CH,
                        cqv + c * CH, hqv + c * CH, k, trow + c * CH, lane, ob0, (ofbits & 1u) != 0);
                ob0 = ob1;
                ob1 = ob2;
                ob2 = ob3;
                ofbits >>= 1;
            }
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (PAIR && rank != 0) mbar_arrive_cluster(cluster_map(smem_u32(&ctrl->tmem_empty[a]), 0));
                else mbar_arrive(&ctrl->tmem_empty[a]);
            }
            if (PEERS) mirror_block(p, m0 + quarter * 32, n0, ecols, lane); // after the accumulator is handed back
        }
    }

    __syncwarp();
    tcgen05_fence_before();
    __syncthreads();
    if (PAIR) cluster_sync_all(); // neither CTA leaves (or frees tensor memory) while the other may still reach into it
    if (warp == 1) {
        tcgen05_fence_after();
        if (PAIR)
            asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
        else
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// ---- measured tensor-pipe peak -------------------------------------------------------------
//
// The denominator of the dense kernels' roofline: how fast this GPU's tensor cores run the very
// instruction the kernel above issues (tcgen05.mma cta_group::1, kind::i8 or kind::f8f6f4,
// 128 x 256 x 32) when nothing else is in the way -- operands resident in shared memory (whatever
// bytes are there: the arithmetic does not depend on the values), no copies, no epilogue.  One CTA
// per SM, one thread issues `iters` groups of four MMAs over two operand stages and two accumulators
// and commits after each group; the kernel ends when the last commit has arrived.  Timed by
// the caller with CUDA events; ops = 2 * 128 * 256 * 32 * 4 * iters * CTAs.
template <bool FP8>
__global__ void __launch_bounds__(128, 1) tc8_mma_peak_kernel(uint32_t iters, uint32_t idesc, uint32_t *status) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    __shared__ uint64_t done_bar;
    __shared__ uint32_t tmem_base_s;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        mbar_init(&done_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = tmem_base_s;
    if (warp == 0 && lane == 0) {
        const uint64_t adesc0 = make_smem_desc(smem_u32(smem)), bdesc0 = make_smem_desc(smem_u32(smem) + A_BYTES);
        for (uint32_t it = 0; it < iters; ++it) {
            const uint32_t s = it & 1;
            const uint64_t adesc = adesc0 + (uint64_t)(s * (STAGE_BYTES >> 4)), bdesc = bdesc0 + (uint64_t)(s * (STAGE_BYTES >> 4));
#pragma unroll
            for (int k = 0; k < BK / 32; ++k) tcgen05_mma<FP8>(tmem_base + s * BN, adesc + 2 * k, bdesc + 2 * k, idesc, (it > 1) || k != 0);
        }
        tcgen05_commit(&done_bar);
        // bounded like every wait here: a few seconds at most
        bool ok = false;
        for (uint32_t i = 0; i < (1u << 26) && !ok; ++i) {
            ok = mbar_test(&done_bar, 0);
            if (!ok) __nanosleep(64);
        }
        if (!ok && status) atomicOr(status, ST_WAIT_TMEM_FULL);
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 0) {
        tcgen05_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// ---- host side ------------------------------------------------------------------------------

typedef CUresult (*encode_tiled_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
        const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
        CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static encode_tiled_fn get_encode_fn() {
    static encode_tiled_fn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess
                && q == cudaDriverEntryPointSuccess)
            fn = (encode_tiled_fn)sym;
    });
    return fn;
}

// rows x K bytes, row pitch in bytes; box = 128 bytes of K x box_rows rows, 128-byte swizzle;
// out-of-range parts of a box read as zero
static bool make_tmap(CUtensorMap *map, const void *base, int64_t rows, int64_t K, int64_t pitch, uint32_t box_rows) {
    encode_tiled_fn fn = get_encode_fn();
    if (!fn) return false;
    const cuuint64_t gdim[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t gstride[1] = {(cuuint64_t)pitch};
    const cuuint32_t box[2] = {(cuuint32_t)BK, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), gdim, gstride, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE)
            == CUDA_SUCCESS;
}

static uint32_t make_idesc(bool fp8, int a_dt, int b_dt, int n, int m) {
    uint32_t d = 0;
    if (fp8) {
        d |= 1u << 4;                                       // accumulator f32
        d |= (a_dt == B200_DT_F8_E5M2 ? 1u : 0u) << 7;      // A format: 0 = e4m3, 1 = e5m2
        d |= (b_dt == B200_DT_F8_E5M2 ? 1u : 0u) << 10;     // B format
    } else {
        d |= 2u << 4;                                       // accumulator s32
        d |= (a_dt == B200_DT_S8 ? 1u : 0u) << 7;           // A format: 0 = u8, 1 = s8
        d |= (b_dt == B200_DT_S8 ? 1u : 0u) << 10;          // B format
    }
    // bits 15 / 16: A and B are K-major (0)
    d |= (uint32_t)(n >> 3) << 17;
    d |= (uint32_t)(m >> 4) << 24;
    return d;
}

} // namespace b200

using namespace b200;

extern "C" int b200_tc8_mma_peak_launch(int32_t fp8, uint32_t iters, uint32_t *status, uint64_t *ops_out, b200_stream_t stream) {
    if (iters == 0 || iters > (1u << 20)) return B200_ERR_BAD_ARG;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const size_t smem = 1024 + 2 * (size_t)STAGE_BYTES;
    const uint32_t idesc = make_idesc(fp8 != 0, fp8 ? B200_DT_F8_E4M3 : B200_DT_S8, fp8 ? B200_DT_F8_E4M3 : B200_DT_S8, BN, BM);
    auto kern = fp8 ? tc8_mma_peak_kernel<true> : tc8_mma_peak_kernel<false>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return (int)cudaGetLastError();
    kern<<<sms, 128, smem, (cudaStream_t)stream>>>(iters, idesc, status);
    if (ops_out) *ops_out = (uint64_t)2 * BM * BN * 32 * (BK / 32) * iters * (uint64_t)sms;
    return after_launch();
}

extern "C" int b200_matmul_tc8_launch(const b200_matmul_params_t *p, b200_stream_t stream) {
    if (!p || !p->src || !p->wei || !p->dst) return B200_ERR_BAD_ARG;
    if (p->M < 0 || p->N < 0 || p->K < 0 || p->npo < 0 || p->npo > B200_MAX_POSTOPS) return B200_ERR_BAD_ARG;
    if (p->M == 0 || p->N == 0 || p->K == 0) return 0;
    const bool i8 = (p->src_dt == B200_DT_S8 || p->src_dt == B200_DT_U8) && (p->wei_dt == B200_DT_S8 || p->wei_dt == B200_DT_U8);
    const bool f8 = (p->src_dt == B200_DT_F8_E4M3 || p->src_dt == B200_DT_F8_E5M2)
            && (p->wei_dt == B200_DT_F8_E4M3 || p->wei_dt == B200_DT_F8_E5M2);
    if (!i8 && !f8) return B200_ERR_UNSUPPORTED;
    if (p->K % 16 != 0 || p->src_sk != 1 || p->dst_sn != 1) return B200_ERR_UNSUPPORTED;
    if (p->n_dst_peers < 0 || p->n_dst_peers > B200_MAX_DST_PEERS) return B200_ERR_BAD_ARG;
    for (int i = 0; i < p->n_dst_peers; ++i)
        if (!p->dst_peer[i] || (((uintptr_t)p->dst_peer[i] ^ (uintptr_t)p->dst) & 15)) return B200_ERR_BAD_ARG; // same 16-byte phase as dst
    // weights: packed K-major, or plain with K contiguous
    int64_t wpitch;
    if (p->wei_layout == B200_WEI_KMAJOR) wpitch = p->K;
    else if (p->wei_layout == B200_WEI_PLAIN && p->wei_sk == 1) wpitch = p->wei_sn;
    else return B200_ERR_UNSUPPORTED;
    // source scales: per tensor, or per row (one K group covering all of K; f32)
    if (p->src_scale.ptr && (p->src_scale.s0 || p->src_scale.s1)
            && !(i8 && p->src_scale.s0 == 1 && p->src_scale.g0 == 1 && p->src_scale.g1 >= p->K && p->src_scale.dt == B200_DT_F32))
        return B200_ERR_UNSUPPORTED;
    if (p->wei_scale.ptr && (p->wei_scale.s0 || p->wei_scale.g1 != 1)) return B200_ERR_UNSUPPORTED;
    if (p->dst_scale.ptr && (p->dst_scale.s0 || p->dst_scale.s1)) return B200_ERR_UNSUPPORTED;
    if (p->src_zp.ptr && (p->src_zp.s0 || p->src_zp.s1 || !p->wei_colsum || f8)) return B200_ERR_UNSUPPORTED;
    // weights zero-points: per tensor or per column, with the row sums of src supplied
    if (p->wei_zp.ptr && (p->wei_zp.s0 || p->wei_zp.g0 != 1 || p->wei_zp.g1 != 1 || !p->src_rowsum || f8)) return B200_ERR_UNSUPPORTED;
    if (p->dst_zp.ptr && (p->dst_zp.s0 || p->dst_zp.dt != B200_DT_S32 || f8)) return B200_ERR_UNSUPPORTED;
    if (((uintptr_t)p->src & 15) || ((uintptr_t)p->wei & 15) || (p->src_sm & 15) || (wpitch & 15)) return B200_ERR_BAD_ARG;
    if (p->M > INT32_MAX || p->N > INT32_MAX || p->K > INT32_MAX) return B200_ERR_TOO_LARGE;

    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    // Two CTAs per tile of 2 * BM rows (cta_group::2): a third fewer bytes from L2 per tile, but
    // a longer round trip per pipeline stage (both CTAs' copies report to the leader, its
    // commits travel back to both) and work units twice as large.  Measured on 148 SMs it wins
    // from about eight waves of single-CTA tiles upwards (8192^3: +4 %, 16384 x 28672 x 8192:
    // +8 %) and loses below (4096^3: -3 %).  ONEDNN_B200_TC8_PAIR=0 / 1 forces the choice.
    // Mirrored destinations (N-split over GPUs) use the single-CTA kernel.
    const char *pe = std::getenv("ONEDNN_B200_TC8_PAIR");
    const int64_t single_tiles = ((p->M + BM - 1) / BM) * ((p->N + BN - 1) / BN);
    const bool pair_wanted = pe && (pe[0] == '0' || pe[0] == '1') ? pe[0] == '1' : single_tiles >= (int64_t)8 * sms;
    const bool pair = pair_wanted && p->M > BM && p->n_dst_peers == 0 && sms >= 2;
    const int tile_rows = pair ? 2 * BM : BM;
    const int workers = pair ? sms / 2 : sms; // CTAs or CTA pairs working at the same time

    CUtensorMap ta, tb, tbs;
    if (!make_tmap(&ta, p->src, p->M, p->K, p->src_sm, BM)) return (int)cudaErrorUnknown;
    if (!make_tmap(&tb, p->wei, p->N, p->K, wpitch, B_BOX_ROWS)) return (int)cudaErrorUnknown;
    if (!make_tmap(&tbs, p->wei, p->N, p->K, wpitch, B_BOX_ROWS_SMALL)) return (int)cudaErrorUnknown;

    tc8_args_t a;
    a.p = *p;
    a.m_tiles = (int)((p->M + tile_rows - 1) / tile_rows);
    a.n_tiles = (int)((p->N + BN - 1) / BN);
    a.k_blocks = (int)((p->K + BK - 1) / BK);
    a.idesc = make_idesc(f8, p->src_dt, p->wei_dt, BN, tile_rows);

    const int64_t tiles = (int64_t)a.m_tiles * a.n_tiles;
    if (tiles > INT32_MAX / 4) return B200_ERR_TOO_LARGE;
    // Narrower units where whole tiles would leave SMs idle: all tiles of a problem with at
    // most half (a quarter) as many tiles as workers are cut in 2 (4); otherwise the tiles of a
    // last wave that fills at most half of the workers are cut in 2.
    const int max_split = pair ? 2 : 4; // a CTA of a pair holds half of the unit's weight rows: at least one box
    int64_t tail = 0;
    a.split = 1;
    if (tiles * 2 <= workers) {
        tail = tiles;
        a.split = (tiles * 4 <= workers && max_split >= 4) ? 4 : 2;
    } else if (tiles > workers && tiles % workers != 0 && 2 * (tiles % workers) <= workers) {
        tail = tiles % workers;
        a.split = 2;
    }
    a.full_units = (int)(tiles - tail);
    a.units = (int)(tiles - tail + tail * a.split);
    a.idesc_tail = make_idesc(f8, p->src_dt, p->wei_dt, BN / a.split, tile_rows);
    const unsigned grid = (unsigned)(a.units < workers ? a.units : workers) * (pair ? 2u : 1u);

    // epilogue evaluation mode
    int epi = EPI_NONE;
    if (p->npo > 0) {
        bool simple = true;
        for (int i = 0; i < p->npo; ++i) {
            const b200_postop_t &e = p->po[i];
            const bool elt_ok = e.kind == B200_PO_ELTWISE
                    && (e.alg == ALG_RELU || e.alg == ALG_RELU_DST || e.alg == ALG_SQUARE || e.alg == ALG_ABS
                            || e.alg == ALG_LINEAR || e.alg == ALG_HARDSIGMOID || e.alg == ALG_CLIP || e.alg == ALG_CLIP_V2
                            || e.alg == ALG_CLIP_V2_DST || e.alg == ALG_ROUND || e.alg == ALG_HARDSWISH
                            || e.alg == ALG_SQRT || e.alg == ALG_SQRT_DST);
            if (!(e.kind == B200_PO_SUM || elt_ok)) simple = false;
        }
        const bool int_dst = p->dst_dt == B200_DT_S8 || p->dst_dt == B200_DT_U8;
        const bool gelu_q = int_dst && p->po[0].kind == B200_PO_ELTWISE && p->po[0].alg == ALG_GELU_TANH
                && (p->npo == 1 || (p->npo == 2 && p->po[1].kind == B200_PO_SUM));
        epi = simple ? EPI_SIMPLE : gelu_q ? EPI_GELU_Q : EPI_GENERIC;
    }
    if (p->bias && p->bias_sm) epi = EPI_GENERIC; // a bias that varies along M is added by the interpreted path
    if (p->wei_zp.ptr) {
        // the straight-line path with an empty or simple chain, the interpreted one otherwise
        if (epi == EPI_NONE || epi == EPI_SIMPLE) epi = EPI_SIMPLE_WZ;
        else if (epi == EPI_GELU_Q) epi = EPI_GENERIC;
    }

    // how the sum post-op reads the prior destination
    int sum = SUM_NONE;
    if (epi == EPI_SIMPLE || epi == EPI_SIMPLE_WZ || epi == EPI_GELU_Q) {
        for (int i = 0; i < p->npo; ++i)
            if (p->po[i].kind == B200_PO_SUM) {
                const int sdt = p->po[i].dt != B200_DT_UNDEF ? p->po[i].dt : p->dst_dt;
                sum = (sdt == B200_DT_S8 || sdt == B200_DT_U8) ? SUM_8BIT : SUM_OTHER;
            }
        if (epi == EPI_GELU_Q && sum == SUM_OTHER) epi = EPI_GENERIC, sum = SUM_NONE;
    }

    typedef void (*kernel_t)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const tc8_args_t);
#define TC8_ROW(F, P) \
    {{matmul_tc8_kernel<F, EPI_NONE, SUM_NONE, false, P>, nullptr, nullptr}, \
            {matmul_tc8_kernel<F, EPI_SIMPLE, SUM_NONE, false, P>, matmul_tc8_kernel<F, EPI_SIMPLE, SUM_8BIT, false, P>, \
                    matmul_tc8_kernel<F, EPI_SIMPLE, SUM_OTHER, false, P>}, \
            {matmul_tc8_kernel<F, EPI_GELU_Q, SUM_NONE, false, P>, matmul_tc8_kernel<F, EPI_GELU_Q, SUM_8BIT, false, P>, nullptr}, \
            {matmul_tc8_kernel<F, EPI_GENERIC, SUM_NONE, false, P>, nullptr, nullptr}, \
            {F ? nullptr : (kernel_t)matmul_tc8_kernel<false, EPI_SIMPLE_WZ, SUM_NONE, false, P>, \
                    F ? nullptr : (kernel_t)matmul_tc8_kernel<false, EPI_SIMPLE_WZ, SUM_8BIT, false, P>, \
                    F ? nullptr : (kernel_t)matmul_tc8_kernel<false, EPI_SIMPLE_WZ, SUM_OTHER, false, P>}}
    static const kernel_t table[2][2][5][3] = {{TC8_ROW(false, false), TC8_ROW(true, false)}, {TC8_ROW(false, true), TC8_ROW(true, true)}};
#undef TC8_ROW
    kernel_t kern = table[pair ? 1 : 0][f8 ? 1 : 0][epi][sum];
    if (p->n_dst_peers) {
        // mirrored destinations: built for the epilogues an N-split layer has (bias, simple eltwise), no sum
        kern = nullptr;
        if (sum == SUM_NONE && epi == EPI_NONE)
            kern = f8 ? matmul_tc8_kernel<true, EPI_NONE, SUM_NONE, true> : matmul_tc8_kernel<false, EPI_NONE, SUM_NONE, true>;
        if (sum == SUM_NONE && epi == EPI_SIMPLE)
            kern = f8 ? matmul_tc8_kernel<true, EPI_SIMPLE, SUM_NONE, true> : matmul_tc8_kernel<false, EPI_SIMPLE, SUM_NONE, true>;
    }
    if (!kern) return B200_ERR_UNSUPPORTED;
    // opt in to the large dynamic shared memory once per kernel and device
    static std::mutex attr_mu;
    static bool attr_done[64][2][2][5][3] = {};
    {
        std::lock_guard<std::mutex> g(attr_mu);
        static bool attr_done_peers[64][2][5] = {};
        bool &done = p->n_dst_peers ? attr_done_peers[dev & 63][f8 ? 1 : 0][epi] : attr_done[dev & 63][pair ? 1 : 0][f8 ? 1 : 0][epi][sum];
        if (dev < 64 && !done) {
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
            if (e != cudaSuccess) return (int)e;
            done = true;
        }
    }
    if (!pair) {
        kern<<<grid, NUM_THREADS, SMEM_BYTES, (cudaStream_t)stream>>>(ta, tb, tbs, a);
        return after_launch();
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t le = cudaLaunchKernelEx(&cfg, kern, ta, tb, tbs, a);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    if (le != cudaSuccess) {
        (void)cudaGetLastError();
        return (int)le;
    }
    return 0;
}
