// Weight-compressed matmul on the tensor cores: bf16 activations (up to 128 rows per
// pass) times 4-bit or 8-bit integer weights with K-grouped scales and zero-points.
// Semantics: the reference's weights-decompression matmul
// (src/cpu/matmul/ref_matmul.cpp:130-233, with_wei_decompression) under fpmath bf16
// with apply_to_int: every weight is decompressed to w' = (q - zp) * scale and rounded
// to bf16 -- exactly the bf16 rounding of the reference's f32 w' (4-bit weights: (q - zp) is
// formed exactly in bf16 and multiplied by the bf16 scale with one rounding; 8-bit weights:
// the reference's own f32 arithmetic, then one rounding) -- and products are accumulated
// in f32.
//
// Where the decode kernel (matmul_wc.cu) spends its issue slots on register-level MMAs,
// this one only converts: per stage of 64 k, a group of four warps (one thread per output
// column) turns the packed weights of 128 columns into a 128-column x 64-k bf16 tile in
// shared memory, laid out as the 128-byte-swizzled K-major operand tile a TMA load would
// have produced; the activations of the same 64 k arrive by TMA into a ring of their own; two
// threads issue tcgen05.mma (kind::f16, 128 x NB x 16) for alternate k-blocks, each into its
// own accumulator, with the weights as the A operand (128 output columns = the TMEM lanes)
// and the activations as B (NB = activation rows rounded up to 16), accumulating in TMEM over
// the whole K.  The epilogue adds the two accumulators and reads TMEM with one output column
// per lane, so that stores of a dst row are coalesced.  Block i uses barrier pair i mod SA
// (SA = stages of converted weights: 4, 6 or 8; SB <= SA stages of activations).
//
//   warp 0        TMA producer (activations)           waits empty[i - SB] -> full_a[i] (tx bytes)
//   warps 1, 2    MMA issuers (warp 1 owns TMEM):      wait full_a[i]      -> empty[i], acc_full
//                 issuer j takes the tile's k-blocks
//                 j, j + 2, ... into accumulator j
//   warps 3..18   four dequantising groups (group g    wait empty[i - SA]  -> full_a[i]; acc_full -> acc_empty
//                 converts blocks g, g + 4, ...), then
//                 the epilogue
//
// Weights are read in the layouts written by the pack kernels below.  B200_WEI_WC4_TC:
// blocks of 128 output columns x 64 k = 4 KiB, block (nt, kb) at ((nt * K/64) + kb) * 4096,
// inside a block row-major [128 columns][64 k] nibbles, 32 bytes per column; inside each
// 32-bit word (8 consecutive k) nibble i holds k 2i and nibble i + 4 holds k 2i + 1, so that
// (w >> 4i) & 0x000f000f | 0x43004300 is the bf16 pair (128 + q[2i], 128 + q[2i + 1]);
// s4 values are stored offset by 8.  B200_WEI_WC8_TC: the same blocks with one byte per
// weight (8 KiB, 64 bytes per column, k ascending).  Columns past N are stored as zeros.
//
// Every wait is bounded; a wait that runs out sets a bit in the stream's status word,
// every role stops at its next wait, copies in flight are drained and TMEM is released.
#include <cuda.h>
#include <cuda_bf16.h>

#include <cstdlib>
#include <mutex>

#include "common.cuh"
#include "launch.hpp"

namespace b200 {
namespace wctc {

constexpr int TN = 128;              // output columns per tile (UMMA M, TMEM lanes)
constexpr int TK = 64;               // k per stage: 128 bytes of bf16 = one swizzle row
constexpr int GROUPS = 4;            // dequantising warp groups, each converts every fourth k-block
constexpr int MAX_STAGES = 8;        // ring depths are 4, 6 or 8: converted weights SA, activations SB <= SA
constexpr int GROUP_WARPS = TN / 32; // one thread per output column of the tile
constexpr int DQ_WARPS = GROUPS * GROUP_WARPS;
// per weight width (4 or 8 bits): packed bytes of one column in one k-block, of a whole block,
// and the number of its own k-blocks a group requests ahead (64 KiB of ring either way)
__host__ __device__ constexpr int pf_bytes(int wbits) { return TK * wbits / 8; }
__host__ __device__ constexpr int block_bytes(int wbits) { return TN * TK * wbits / 8; }
__host__ __device__ constexpr int pfs(int wbits) { return 2; }
// One thread issuing a k-block's four MMAs and its commit, with one look at a barrier, takes about
// 800 cycles per block however small the MMAs are, three times what the tensor pipe needs for them
// at 128 activation rows -- so two threads issue alternate k-blocks, each into an accumulator of
// its own (f32 partial sums added by the epilogue), and together keep the pipe fed.
constexpr int ISSUERS = 2;
constexpr int FIRST_DQ_WARP = 1 + ISSUERS;
constexpr int NUM_THREADS = (FIRST_DQ_WARP + DQ_WARPS) * 32;
constexpr int A_BYTES = TN * TK * 2; // dequantised weights tile, 16 KiB
constexpr uint32_t WAIT_SPINS = 1u << 24; // polls of the drain loop
constexpr uint32_t WAIT_TRIES = 1u << 19; // hardware-suspended waits of up to ~2 us each
enum : uint32_t { ST_WAIT_FULL = 0x1000, ST_WAIT_EMPTY = 0x2000, ST_WAIT_ACC = 0x4000 };

// One pair of barriers per k-block modulo the depth SA of the weights ring (4, 6 or 8; the
// activations ring has SB <= SA stages): full[i] collects the four warp arrivals of the converted
// weights and the bytes of the activations' copy of block i; done[i] ("empty" below) is the
// arrival of the commit behind block i's MMAs.  The converters wait on done for block i - SA,
// the copy-issuing thread for block i - SB: one look and one commit per block for an MMA-issuing
// thread.  Both rings want depth: a copy of 128-byte row pieces from L2 takes about 1.4 us to
// land, and a group may only refill a weights stage when the MMAs that read it have retired, a
// microsecond after they were issued; at 128 activation rows six stages of each fit.
struct ctrl_t {
    uint64_t full_a[MAX_STAGES];
    uint64_t empty[MAX_STAGES];
    uint64_t acc_full, acc_empty;
    uint32_t tmem_base;
    volatile uint32_t abort;
};

struct args_t {
    b200_matmul_params_t p;
    const uint8_t *wei;      // packed weights
    int nb;                  // activation rows per pass, rounded up to 16 (UMMA N)
    int m_passes, n_tiles, k_blocks;
    int64_t rows_per_pass;
    uint32_t idesc;
    uint32_t tmem_cols;
    uint32_t gs_blocks, gz_blocks; // K-group sizes of scales and zero-points in k-blocks of 64 (K / 64 when not grouped)
    uint32_t gs_shift, gz_shift;   // their base-2 logarithms (the FASTQ instantiation requires powers of two)
    uint32_t a_stages, b_stages;   // ring depths (4, 6 or 8): converted weights, activations (b_stages <= a_stages)
    float nibble_offset;     // 4-bit weights: 128 (u4) or 136 (s4 stored offset by 8)
    uint32_t byte_xor;       // 8-bit weights: 0x80808080 for s8 (to offset binary), 0 for u8
};

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
// one wait of at most about two microseconds, suspended in hardware
__device__ __forceinline__ bool mbar_try(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(smem_u32(bar)), "r"(parity), "r"(2000u)
            : "memory");
    return ok != 0;
}
// bounded wait (about a second); false when it ran out or another role already gave up
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, ctrl_t *c, uint32_t *status, uint32_t code) {
    for (uint32_t i = 0; i < WAIT_TRIES; ++i) {
        if (mbar_try(bar, parity)) return true;
        if (c->abort) return false;
    }
    c->abort = 1;
    if (status) atomicOr(status, code);
    return false;
}
// The same wait by polling, for the copy-issuing and the MMA-issuing thread, whose waits are
// part of every stage's round trip: a poll sees the phase flip sooner than a suspended waiter
// is woken.  Bounded as well: 2^26 polls, of the order of a second.
__device__ __forceinline__ bool mbar_wait_poll(uint64_t *bar, uint32_t parity, ctrl_t *c, uint32_t *status, uint32_t code) {
    for (uint32_t i = 0; i < (1u << 26); ++i) {
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
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tc_mma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
    asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
            :
            : "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
            : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
            : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
            "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
            : "r"(taddr)
            : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7]), "+r"(v[8]),
                 "+r"(v[9]), "+r"(v[10]), "+r"(v[11]), "+r"(v[12]), "+r"(v[13]), "+r"(v[14]), "+r"(v[15])
                 :
                 : "memory");
}
// shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows of 128 bytes,
// 8-row groups 1024 bytes apart (tile base 1024-byte aligned)
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3ffff) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// Epilogue of 16 activation rows of one output column: src scale, bias, post-ops, dst
// scale, conversion, store.  Out of line and not unrolled: the interpreter behind
// finish_element is large, and the conversion loop should keep the instruction cache.
__device__ __noinline__ void finish_chunk(const b200_matmul_params_t &p, const uint32_t (&v)[16], int64_t m_first, int64_t m_end,
        int64_t n) {
    if (n >= p.N) return;
    const float dst_inv = dst_scale_reciprocal(p);
    const float src_scale = p.src_scale.ptr ? load_f32(p.src_scale.dt, p.src_scale.ptr, 0) : 1.f;
#pragma unroll 1
    for (int j = 0; j < 16; ++j) {
        const int64_t m = m_first + j;
        if (m >= m_end) break;
        float dv = __uint_as_float(v[j]);
        if (p.src_scale.ptr) dv = __fmul_rn(dv, src_scale);
        finish_element(p, dv, m, n, false, dst_inv);
    }
}

// ---- the kernel -------------------------------------------------------------------------

// FASTQ (4-bit weights only): bf16 (or no) scales, 4-bit (or no) zero-points, K groups that are
// powers of two in k-blocks, all indices within 32 bits -- what the benchmark's configuration
// and most weight-only-quantised checkpoints have.  The per-block scale / zero-point fetch is then
// a shift, a multiply-add and a 16-bit load instead of two divisions and a chain of type tests.
template <int WBITS, bool FASTQ>
__global__ void __launch_bounds__(NUM_THREADS, 1)
        wc_tc_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ args_t args) {
    constexpr int PFS = pfs(WBITS), PF_BYTES = pf_bytes(WBITS), BLOCK_BYTES = block_bytes(WBITS);
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const b200_matmul_params_t &p = args.p;
    const int nb = args.nb;
    const uint32_t b_bytes = (uint32_t)nb * (TK * 2); // a multiple of 2 KiB: every stage of either ring starts on a 1 KiB boundary
    // block index -> stage and use count; the depths are 4, 6 or 8 so that this is a mask and a shift or
    // a division by a constant (the loops of the issuing threads set the pace: a division by a
    // run-time value there costs more than the MMAs' issue)
    const uint32_t SA = args.a_stages, SB = args.b_stages;
    auto rmod = [](uint32_t x, uint32_t n) -> uint32_t { return n == 8 ? (x & 7u) : n == 6 ? x % 6u : (x & 3u); };
    auto rdiv = [](uint32_t x, uint32_t n) -> uint32_t { return n == 8 ? (x >> 3) : n == 6 ? x / 6u : (x >> 2); };
    uint8_t *smem_b = smem + (size_t)SA * A_BYTES;                             // [SB][nb][128 bytes] activations
    uint8_t *pf_ring = smem_b + (size_t)SB * b_bytes;                          // [PFS][threads][PF_BYTES] packed weights in flight
    ctrl_t *ctrl = (ctrl_t *)(pf_ring + (size_t)PFS * DQ_WARPS * 32 * PF_BYTES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_tiles = args.n_tiles * args.m_passes;
    const int KB = args.k_blocks;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < SA; ++s) {
            mbar_init(&ctrl->full_a[s], GROUP_WARPS + 1); // the group's warps and the activations' copy
            mbar_init(&ctrl->empty[s], 1);
        }
        mbar_init(&ctrl->acc_full, ISSUERS);
        mbar_init(&ctrl->acc_empty, DQ_WARPS);
        ctrl->abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctrl->tmem_base)),
                     "r"(args.tmem_cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = ctrl->tmem_base;

    if (warp == 0) {
        // ---------------- TMA producer: activations of each k-block ----------------
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            // stage indices and the parity to wait for are carried along and wrapped by hand: this
            // loop and the issuers' set the pace, and every instruction in them counts
            uint32_t sa = 0, sb = 0;          // barrier / activations stage of block `it`
            uint32_t pa = 0, ppar = 0;        // barrier of block it - SB and the parity of its commit (valid once it >= SB)
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                const int row0 = (int)((tile / args.n_tiles) * args.rows_per_pass);
                for (int kb = 0; kb < KB; ++kb, ++it) {
                    // this block's stage of the activations ring was last read by block it - SB
                    if (it >= SB) {
                        if (!(ok = mbar_wait_poll(&ctrl->empty[pa], ppar, ctrl, p.status, ST_WAIT_EMPTY))) break;
                        if (++pa == SA) pa = 0, ppar ^= 1;
                    }
                    uint64_t *full = &ctrl->full_a[sa];
                    mbar_expect_tx(full, b_bytes);
                    tma_load_2d(smem_b + (size_t)sb * b_bytes, &tmap_x, kb * (TK * 2), row0, full); // byte coordinates
                    if (++sa == SA) sa = 0;
                    if (++sb == SB) sb = 0;
                }
            }
            // drain: every copy this thread issued must have landed before the CTA may exit
            const uint32_t issued = it;
            for (uint32_t j = issued > SB ? issued - SB : 0; j < issued; ++j) {
                const uint32_t s = rmod(j, SA), r = rdiv(j, SA);
                for (uint32_t i = 0; i < WAIT_SPINS; ++i) {
                    if (mbar_test(&ctrl->full_a[s], r & 1)) break;
                    __nanosleep(64);
                }
            }
        }
    } else if (warp <= ISSUERS) {
        // ---------------- MMA issuers ----------------
        if (lane == 0) {
            const int me = warp - 1;                                 // this issuer's k-blocks: me, me + ISSUERS, ...
            const uint32_t tmem_d = tmem_base + (uint32_t)(me * nb); // and its accumulator: nb columns of tensor memory
            uint32_t it0 = 0, tile_i = 0;
            bool ok = true;
            // descriptors of stage 0; a stage further on is stage_bytes / 16 more in the address field
            const uint64_t adesc0 = make_smem_desc(smem_u32(smem)), bdesc0 = make_smem_desc(smem_u32(smem_b));
            // This thread's loop sets the pace of the kernel: per k-block one look at a barrier, four
            // MMAs, one commit.  A look at a barrier costs about 200 cycles even when the phase has long
            // completed, so the look for block i + 1 is issued before the MMAs of block i and its
            // answer read after them; only when that early look says "not yet" does the thread poll.
            // No tcgen05 fence inside the loop: the operands are in shared memory, written through
            // the async proxy (the copies) or published with fence.proxy.async (the converters), and
            // ordered by the barrier; the fence belongs where tensor memory changes hands (below).
            // (The look ISSUERS blocks ahead is unambiguous: the phase before the one asked about, on
            // the same barrier, belongs to one of this thread's own earlier blocks -- the ring depth is
            // a multiple of ISSUERS.)
            bool early = false; // the early look's answer for the block at hand
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++tile_i, it0 += (uint32_t)KB) {
                if (!(ok = mbar_wait_poll(&ctrl->acc_empty, (tile_i & 1) ^ 1, ctrl, p.status, ST_WAIT_ACC))) break;
                tc_fence_after();
                early = false; // looks do not cross tiles: the next tile's first block is another distance away
                // stage, parity and activations stage of this thread's first block of the tile; from
                // there on they advance by ISSUERS with a wrap (SA and SB are multiples of ISSUERS)
                uint32_t s = rmod(it0 + (uint32_t)me, SA), par = rdiv(it0 + (uint32_t)me, SA) & 1, sb = rmod(it0 + (uint32_t)me, SB);
                for (int kb = me; kb < KB; kb += ISSUERS) {
                    // one barrier per block: converted weights (four warps) and activations (copy bytes)
                    if (!early && !(ok = mbar_wait_poll(&ctrl->full_a[s], par, ctrl, p.status, ST_WAIT_FULL))) break;
                    uint32_t s2 = s + ISSUERS, par2 = par;
                    if (s2 >= SA) s2 -= SA, par2 ^= 1;
                    const bool next_early = kb + ISSUERS < KB && mbar_test(&ctrl->full_a[s2], par2);
                    const uint64_t adesc = adesc0 + (uint64_t)(s * (A_BYTES >> 4)), bdesc = bdesc0 + (uint64_t)(sb * (b_bytes >> 4));
#pragma unroll
                    for (int k = 0; k < TK / 16; ++k) // 16 bf16 = 32 bytes of K per instruction: +2 in 16-byte units
                        tc_mma_bf16(tmem_d, adesc + 2 * k, bdesc + 2 * k, args.idesc, (kb >= ISSUERS) | (k != 0));
                    tc_commit(&ctrl->empty[s]);
                    early = next_early;
                    s = s2, par = par2;
                    sb += ISSUERS;
                    if (sb >= SB) sb -= SB;
                }
                if (ok) tc_commit(&ctrl->acc_full);
            }
        }
    } else {
        // ---------------- dequantisers, then epilogue ----------------
        // Warp group g (four warps, one thread per column of the tile) converts the k-blocks that
        // land in operand stage g, i.e. every fourth one: a thread then has a quarter of the
        // iterations, each with a whole 64-k row to convert, and the four groups work on four
        // different stages at the same time.
        const int dq = threadIdx.x - FIRST_DQ_WARP * 32; // 0 .. 511
        const int grp = dq >> 7, r = dq & 127;
        const int quarter = warp & 3;       // TMEM lanes this warp may read: 32*quarter .. +31
        const int which = (warp - FIRST_DQ_WARP) >> 2; // four warps share a quarter and split the chunks of columns
        const uint32_t sw = (uint32_t)(r & 7);
        const bool simple_epilogue = p.npo == 0 && !p.dst_scale.ptr && (!p.bias || p.bias_sm == 0)
                && (p.dst_dt == B200_DT_BF16 || p.dst_dt == B200_DT_F32);
        const float src_scale = p.src_scale.ptr ? load_f32(p.src_scale.dt, p.src_scale.ptr, 0) : 1.f;
        uint8_t *const row_a = smem + (uint32_t)r * 128; // this thread's row in stage 0
        uint8_t *my_ring = pf_ring + (size_t)dq * PF_BYTES;
        const uint32_t my_ring_s = smem_u32(my_ring);
        constexpr uint32_t RING_STRIDE = DQ_WARPS * 32 * PF_BYTES;
        uint32_t tile_i = 0;
        bool ok = true;

        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++tile_i) {
            const int nt = tile % args.n_tiles;
            const int64_t ncol = (int64_t)nt * TN + r;
            const bool col_ok = ncol < p.N;
            // the k-blocks of this tile that fall into this group's stage
            const uint32_t it0 = tile_i * (uint32_t)KB; // running index of the tile's first k-block
            const int first_kb = (int)((grp + GROUPS - it0 % GROUPS) % GROUPS);
            const int iters = first_kb < KB ? (KB - first_kb + GROUPS - 1) / GROUPS : 0;
            const uint8_t *wsrc = args.wei + ((size_t)nt * KB + first_kb) * BLOCK_BYTES + (size_t)r * PF_BYTES;
            auto request = [&](int j) { // packed row of this thread's j-th k-block, 16-byte copies
                if (j < iters) {
                    const uint8_t *src = wsrc + (size_t)j * (GROUPS * BLOCK_BYTES);
                    const uint32_t dst = my_ring_s + (uint32_t)(j % PFS) * RING_STRIDE;
#pragma unroll
                    for (int q = 0; q < PF_BYTES; q += 16)
                        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + q), "l"(src + q) : "memory");
                }
                asm volatile("cp.async.commit_group;" ::: "memory"); // also when empty: the waits count groups
            };
#pragma unroll 1
            for (int j = 0; j < PFS; ++j) request(j);
            // scale / zero-point of the column: the raw bits for the next iteration are requested
            // while this one is converted
            const bool has_s = col_ok && p.wei_scale.ptr, has_zp = col_ok && p.wei_zp.ptr;
            const int64_t sbase = ncol * p.wei_scale.s1, zbase = ncol * p.wei_zp.s1;
            uint32_t sraw = 0, zraw = 0, zshift = 0;
            const uint32_t sbase32 = (uint32_t)sbase, zbase32 = (uint32_t)zbase, ss0 = (uint32_t)p.wei_scale.s0, zs0 = (uint32_t)p.wei_zp.s0;
            auto load_q = [&](int kb) {
                if (kb >= KB) return;
                if (FASTQ) {
                    if (has_s) sraw = ((const uint16_t *)p.wei_scale.ptr)[((uint32_t)kb >> args.gs_shift) * ss0 + sbase32];
                    if (has_zp) {
                        const uint32_t e = ((uint32_t)kb >> args.gz_shift) * zs0 + zbase32;
                        zraw = ((const uint8_t *)p.wei_zp.ptr)[e >> 1];
                        zshift = (e & 1u) * 4u;
                    }
                    return;
                }
                if (has_s) {
                    const int64_t e = (int64_t)((uint32_t)kb / args.gs_blocks) * p.wei_scale.s0 + sbase;
                    sraw = p.wei_scale.dt == B200_DT_F32 ? ((const uint32_t *)p.wei_scale.ptr)[e] : ((const uint16_t *)p.wei_scale.ptr)[e];
                }
                if (has_zp) {
                    const int64_t e = (int64_t)((uint32_t)kb / args.gz_blocks) * p.wei_zp.s0 + zbase;
                    if (p.wei_zp.dt == B200_DT_S32) {
                        zraw = ((const uint32_t *)p.wei_zp.ptr)[e];
                    } else if (p.wei_zp.dt == B200_DT_S8 || p.wei_zp.dt == B200_DT_U8) {
                        zraw = ((const uint8_t *)p.wei_zp.ptr)[e];
                    } else { // u4 / s4: the byte that holds the nibble
                        zraw = ((const uint8_t *)p.wei_zp.ptr)[e >> 1];
                        zshift = (uint32_t)(e & 1) * 4;
                    }
                }
            };
            auto scale_f32 = [&]() -> float { // of the bits load_q fetched
                if (!col_ok) return 0.f;      // padding columns convert to zeros
                if (!has_s) return 1.f;
                if (p.wei_scale.dt == B200_DT_F32) return __uint_as_float(sraw);
                if (p.wei_scale.dt == B200_DT_BF16) return __uint_as_float(sraw << 16);
                return __half2float(__ushort_as_half((unsigned short)sraw));
            };
            auto zp_int = [&]() -> int {
                if (!has_zp) return 0;
                if (p.wei_zp.dt == B200_DT_S32) return (int)zraw;
                if (p.wei_zp.dt == B200_DT_S8) return (int)(int8_t)zraw;
                if (p.wei_zp.dt == B200_DT_U8) return (int)zraw;
                const int z = (int)((zraw >> zshift) & 0xf);
                return p.wei_zp.dt == B200_DT_S4 ? (z ^ 8) - 8 : z;
            };
            load_q(first_kb);
            for (int j = 0; j < iters; ++j) {
                const int kb = first_kb + j * GROUPS;
                const uint32_t it = it0 + (uint32_t)kb, stage = rmod(it, SA); // the block's running index and its stage of the weights ring
                uint8_t *tile_a = row_a + (size_t)stage * A_BYTES;
                // decode this block's scale and zero-point, then ask for the next block's
                const float sf = FASTQ ? 0.f : scale_f32();
                const int zpi = FASTQ ? 0 : zp_int();
                // FASTQ: the scale's own bits (zeros for a padding column, 1.0 when unset) and the
                // zero-point nibble, sign-extended for s4 -- taken before the next block's are requested
                uint32_t sbits = 0;
                int zq = 0;
                if (FASTQ) {
                    sbits = !col_ok ? 0u : has_s ? sraw : 0x3f80u;
                    zq = has_zp ? (int)((zraw >> zshift) & 0xfu) : 0;
                    if (p.wei_zp.dt == B200_DT_S4) zq = (zq ^ 8) - 8;
                }
                load_q(kb + GROUPS);
                asm volatile("cp.async.wait_group %0;" ::"n"(PFS - 1) : "memory"); // this thread's j-th row has landed
                const uint4 *slot = reinterpret_cast<const uint4 *>(my_ring + (size_t)(j % PFS) * RING_STRIDE);
                uint32_t words[PF_BYTES / 4];
#pragma unroll
                for (int q = 0; q < PF_BYTES / 16; ++q) {
                    const uint4 t4 = slot[q];
                    words[4 * q] = t4.x, words[4 * q + 1] = t4.y, words[4 * q + 2] = t4.z, words[4 * q + 3] = t4.w;
                }
                // the stage was last read by the MMAs of block it - 4
                const uint32_t prev = it - SA;
                if (it >= SA && !(ok = mbar_wait(&ctrl->empty[stage], rdiv(prev, SA) & 1, ctrl, p.status, ST_WAIT_EMPTY))) {
                    asm volatile("cp.async.wait_group 0;" ::: "memory");
                    break;
                }
                if (WBITS == 4) {
                    // bf16 arithmetic: (128 + q) - (128 + zp) is exact, the product with the bf16 scale is
                    // rounded once: the bf16 rounding of the reference's f32 (q - zp) * scale
                    __nv_bfloat162 sc, cc;
                    if (FASTQ) {
                        const uint32_t sb2 = sbits | (sbits << 16);
                        sc = *reinterpret_cast<const __nv_bfloat162 *>(&sb2);
                        cc = __float2bfloat162_rn(args.nibble_offset + (float)zq);
                    } else {
                        sc = __float2bfloat162_rn(sf);                                // exact: the scale is bf16
                        cc = __float2bfloat162_rn(args.nibble_offset + (float)zpi);   // exact: an integer below 256
                    }
#pragma unroll
                    for (int c = 0; c < 8; ++c) { // 16-byte chunk c of the row: k 8c .. 8c + 7
                        const uint32_t v = words[c];
                        uint32_t o[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const uint32_t bits = ((v >> (4 * i)) & 0x000f000fu) | 0x43004300u; // (128 + q, 128 + q')
                            __nv_bfloat162 x = *reinterpret_cast<const __nv_bfloat162 *>(&bits);
                            x = __hmul2(__hsub2(x, cc), sc);
                            o[i] = *reinterpret_cast<const uint32_t *>(&x);
                        }
                        *reinterpret_cast<uint4 *>(tile_a + (((uint32_t)c ^ sw) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
                    }
                } else {
                    // f32 arithmetic: byte b (s8 as offset binary) inside the float 2^23 + b, minus
                    // 2^23 + offset + zp is (q - zp) exactly; times the scale in f32 as the reference
                    // does; then one rounding to bf16
                    const float cf = 8388608.f + (args.byte_xor ? 128.f : 0.f) + (float)zpi;
#pragma unroll
                    for (int c = 0; c < 8; ++c) { // 16-byte chunk c of the row: k 8c .. 8c + 7 = two words of four bytes
                        uint32_t o[4];
#pragma unroll
                        for (int hw = 0; hw < 2; ++hw) {
                            const uint32_t v = words[2 * c + hw] ^ args.byte_xor;
                            float f[4];
#pragma unroll
                            for (int i = 0; i < 4; ++i)
                                f[i] = (__uint_as_float(__byte_perm(v, 0x4B000000u, 0x7540u + i)) - cf) * sf;
                            const __nv_bfloat162 lo = __floats2bfloat162_rn(f[0], f[1]), hi = __floats2bfloat162_rn(f[2], f[3]);
                            o[2 * hw] = *reinterpret_cast<const uint32_t *>(&lo);
                            o[2 * hw + 1] = *reinterpret_cast<const uint32_t *>(&hi);
                        }
                        *reinterpret_cast<uint4 *>(tile_a + (((uint32_t)c ^ sw) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
                    }
                }
                // generic-proxy writes -> visible to the tensor core's (async proxy) reads
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(&ctrl->full_a[stage]);
                request(j + PFS); // the ring slot of iteration j is free again
            }
            if (!ok) break;

            // epilogue: lane = output column, TMEM columns = activation rows of this pass
            ok = mbar_wait(&ctrl->acc_full, tile_i & 1, ctrl, p.status, ST_WAIT_ACC);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const int64_t n = (int64_t)nt * TN + quarter * 32 + lane;
            const int64_t m0 = (int64_t)(tile / args.n_tiles) * args.rows_per_pass;
            const int64_t m_end = m0 + args.rows_per_pass < p.M ? m0 + args.rows_per_pass : p.M;
            const uint32_t trow = tmem_base + ((uint32_t)(quarter * 32) << 16);
            const float bias_n = simple_epilogue && p.bias && n < p.N ? load_f32(p.bias_dt, p.bias, n * p.bias_sn) : 0.f;
            for (int c = which; c * 16 < nb; c += DQ_WARPS / 4) {
                if (m0 + c * 16 >= m_end) break; // warp-uniform: nothing but padding from here on
                uint32_t v[16];
                tmem_ld16(trow + c * 16, v);
                if (KB > 1) { // the second issuer's partial sums (it has none when the tile is a single k-block)
                    uint32_t w[16];
                    tmem_ld16(trow + nb + c * 16, w);
#pragma unroll
                    for (int j = 0; j < 16; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) + __uint_as_float(w[j]));
                }
                if (simple_epilogue) {
                    // no post-ops, no dst scale, bias per column or none, bf16 / f32 dst: a handful of
                    // instructions per element, lanes along a dst row
                    if (n < p.N) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int64_t m = m0 + c * 16 + j;
                            if (m < m_end) {
                                float dv = __uint_as_float(v[j]);
                                if (p.src_scale.ptr) dv = __fmul_rn(dv, src_scale);
                                if (p.bias) dv = __fadd_rn(dv, bias_n);
                                if (p.dst_dt == B200_DT_BF16) ((uint16_t *)p.dst)[m * p.dst_sm + n] = f32_to_bf16_bits(dv);
                                else ((float *)p.dst)[m * p.dst_sm + n] = dv;
                            }
                        }
                    }
                } else {
                    finish_chunk(p, v, m0 + c * 16, m_end, n);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&ctrl->acc_empty);
        }
    }

    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(args.tmem_cols) : "memory");
    }
}

// plain (K, N) 4-bit weights, two per byte along N -> B200_WEI_WC4_TC.  One thread per
// 32-bit output word (8 consecutive k of one column).
__global__ void __launch_bounds__(256) wc_tc_pack_kernel(const uint8_t *__restrict__ src, uint32_t *__restrict__ dst,
        int64_t K, int64_t N, int is_signed) {
    constexpr int BLOCK_BYTES = block_bytes(4);
    const int64_t KB = K / TK, n_tiles = (N + TN - 1) / TN;
    const int64_t nwords = n_tiles * KB * (BLOCK_BYTES / 4);
    for (int64_t wi = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; wi < nwords; wi += (int64_t)gridDim.x * blockDim.x) {
        const int64_t block = wi / (BLOCK_BYTES / 4);
        const int in_block = (int)(wi % (BLOCK_BYTES / 4));
        const int r = in_block >> 3, j = in_block & 7;
        const int64_t nt = block / KB, kb = block % KB;
        const int64_t n = nt * TN + r, k8 = kb * TK + j * 8;
        uint32_t word = 0;
        if (n < N) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int64_t k = k8 + (i < 4 ? 2 * i : 2 * (i - 4) + 1);
                const int64_t e = k * N + n;
                uint32_t q = (src[e >> 1] >> ((e & 1) * 4)) & 0xf;
                if (is_signed) q ^= 8u; // two's complement nibble -> offset binary (value + 8)
                word |= q << (4 * i);
            }
        }
        dst[wi] = word;
    }
}

// plain (K, N) 8-bit weights, any strides -> B200_WEI_WC8_TC: blocks of 128 columns x 64 k,
// row-major [128][64] bytes inside (k contiguous), columns past N zero.  One thread per byte.
__global__ void __launch_bounds__(256) wc_tc_pack8_kernel(const uint8_t *__restrict__ src, int64_t sk, int64_t sn,
        uint8_t *__restrict__ dst, int64_t K, int64_t N) {
    constexpr int BLOCK_BYTES = block_bytes(8);
    const int64_t KB = K / TK, n_tiles = (N + TN - 1) / TN;
    const int64_t total = n_tiles * KB * BLOCK_BYTES;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t block = i / BLOCK_BYTES;
        const int in_block = (int)(i % BLOCK_BYTES);
        const int r = in_block / TK, kk = in_block % TK;
        const int64_t n = (block / KB) * TN + r, k = (block % KB) * TK + kk;
        dst[i] = n < N ? src[k * sk + n * sn] : (uint8_t)0;
    }
}

} // namespace wctc
} // namespace b200

using namespace b200;
using namespace b200::wctc;

typedef CUresult (*wctc_encode_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
        const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
        CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static wctc_encode_fn wctc_get_encode_fn() {
    static wctc_encode_fn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess
                && q == cudaDriverEntryPointSuccess)
            fn = (wctc_encode_fn)sym;
    });
    return fn;
}

static inline size_t wctc_align256(size_t x) { return (x + 255) / 256 * 256; }

extern "C" size_t b200_wc_tc_packed_bytes(int64_t K, int64_t N, int32_t dt) {
    if (K <= 0 || N <= 0) return 0;
    const int bits = dt_bits(dt);
    if (bits != 4 && bits != 8) return 0;
    return (size_t)((N + TN - 1) / TN) * (size_t)(K / TK) * (size_t)block_bytes(bits);
}

extern "C" int b200_wc_tc_pack8_launch(const void *src, int64_t sk, int64_t sn, void *dst, int64_t K, int64_t N, int32_t dt,
        b200_stream_t stream) {
    if (!src || !dst) return B200_ERR_BAD_ARG;
    if ((dt != B200_DT_U8 && dt != B200_DT_S8) || K % TK != 0) return B200_ERR_UNSUPPORTED;
    const int64_t total = (int64_t)b200_wc_tc_packed_bytes(K, N, dt);
    if (total == 0) return 0;
    int64_t blocks = (total + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    wc_tc_pack8_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>((const uint8_t *)src, sk, sn, (uint8_t *)dst, K, N);
    return after_launch();
}

extern "C" int b200_wc_tc_pack_launch(const void *src, void *dst, int64_t K, int64_t N, int32_t dt, b200_stream_t stream) {
    if (!src || !dst) return B200_ERR_BAD_ARG;
    if ((dt != B200_DT_U4 && dt != B200_DT_S4) || K % TK != 0 || (N & 1)) return B200_ERR_UNSUPPORTED;
    const int64_t nwords = (int64_t)(b200_wc_tc_packed_bytes(K, N, dt) / 4);
    if (nwords == 0) return 0;
    int64_t blocks = (nwords + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    wc_tc_pack_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>((const uint8_t *)src, (uint32_t *)dst, K, N,
            dt == B200_DT_S4);
    return after_launch();
}

extern "C" int b200_matmul_wc_tc_launch(const b200_matmul_params_t *p, b200_stream_t stream) {
    if (!p || !p->src || !p->wei || !p->dst) return B200_ERR_BAD_ARG;
    if (p->M <= 0 || p->N <= 0 || p->K <= 0) return p->M < 0 || p->N < 0 || p->K < 0 ? B200_ERR_BAD_ARG : 0;
    const int wbits = dt_bits(p->wei_dt);
    const bool w4 = p->wei_dt == B200_DT_U4 || p->wei_dt == B200_DT_S4, w8 = p->wei_dt == B200_DT_U8 || p->wei_dt == B200_DT_S8;
    if (!w4 && !w8) return B200_ERR_UNSUPPORTED;
    if (!p->apply_to_int || p->src_dt != B200_DT_BF16) return B200_ERR_UNSUPPORTED;
    if (p->K % TK != 0 || (w4 && (p->N & 1)) || p->src_sk != 1 || p->dst_sn != 1 || p->n_dst_peers) return B200_ERR_UNSUPPORTED;
    if (p->M > INT32_MAX || p->N > INT32_MAX || p->K > INT32_MAX) return B200_ERR_TOO_LARGE;
    if (w4 && p->wei_layout == B200_WEI_PLAIN && !(p->wei_sn == 1 && p->wei_sk == p->N)) return B200_ERR_UNSUPPORTED;
    if (p->wei_layout != B200_WEI_PLAIN && p->wei_layout != (w4 ? B200_WEI_WC4_TC : B200_WEI_WC8_TC)) return B200_ERR_UNSUPPORTED;
    if (p->src_zp.ptr || p->dst_zp.ptr) return B200_ERR_UNSUPPORTED;
    if (p->src_scale.ptr && (p->src_scale.s0 || p->src_scale.s1)) return B200_ERR_UNSUPPORTED;
    // 4-bit weights are converted with bf16 arithmetic: the scale must be bf16 to begin with, and
    // 128 + zero-point must be exact in bf16, which 4-bit zero-points guarantee.  8-bit weights
    // are converted in f32: any float scale, any integer zero-point.
    int64_t gs = p->K, gz = p->K;
    if (p->wei_scale.ptr) {
        const int sdt = p->wei_scale.dt;
        if (w4 ? sdt != B200_DT_BF16 : (sdt != B200_DT_BF16 && sdt != B200_DT_F16 && sdt != B200_DT_F32)) return B200_ERR_UNSUPPORTED;
        if (p->wei_scale.g1 != 1) return B200_ERR_UNSUPPORTED;
        if (p->wei_scale.s0) gs = p->wei_scale.g0;
    }
    if (p->wei_zp.ptr) {
        const int zdt = p->wei_zp.dt;
        const bool z4 = zdt == B200_DT_U4 || zdt == B200_DT_S4;
        if (w4 ? !z4 : !(z4 || zdt == B200_DT_S8 || zdt == B200_DT_U8 || zdt == B200_DT_S32)) return B200_ERR_UNSUPPORTED;
        if (p->wei_zp.g1 != 1) return B200_ERR_UNSUPPORTED;
        if (p->wei_zp.s0) gz = p->wei_zp.g0;
    }
    if (gs % TK || gz % TK || p->K % gs || p->K % gz) return B200_ERR_UNSUPPORTED;
    // activations arrive by TMA: 16-byte aligned base and row pitch
    if (((uintptr_t)p->src & 15) || ((p->src_sm * 2) & 15)) return B200_ERR_BAD_ARG;

    cudaStream_t cs = (cudaStream_t)stream;
    const void *wei = p->wei;
    if (p->wei_layout == B200_WEI_PLAIN) {
        const size_t need = wctc_align256(b200_wc_tc_packed_bytes(p->K, p->N, p->wei_dt));
        if (!p->scratch || p->scratch_bytes < need) return B200_ERR_BAD_ARG;
        int rc = w4 ? b200_wc_tc_pack_launch(p->wei, p->scratch, p->K, p->N, p->wei_dt, stream)
                    : b200_wc_tc_pack8_launch(p->wei, p->wei_sk, p->wei_sn, p->scratch, p->K, p->N, p->wei_dt, stream);
        if (rc) return rc;
        wei = p->scratch;
    }
    if ((uintptr_t)wei & 15) return B200_ERR_BAD_ARG;

    args_t a;
    a.p = *p;
    a.wei = (const uint8_t *)wei;
    a.rows_per_pass = p->M <= 128 ? p->M : 128;
    a.nb = (int)((a.rows_per_pass + 15) / 16 * 16);
    a.m_passes = (int)((p->M + a.rows_per_pass - 1) / a.rows_per_pass);
    a.n_tiles = (int)((p->N + TN - 1) / TN);
    a.k_blocks = (int)(p->K / TK);
    a.gs_blocks = (uint32_t)(gs / TK);
    a.gz_blocks = (uint32_t)(gz / TK);
    auto pow2 = [](uint32_t v) { return v && !(v & (v - 1)); };
    auto log2u = [](uint32_t v) { uint32_t l = 0; while ((1u << l) < v) ++l; return l; };
    a.gs_shift = log2u(a.gs_blocks);
    a.gz_shift = log2u(a.gz_blocks);
    const bool z4 = p->wei_zp.ptr && (p->wei_zp.dt == B200_DT_U4 || p->wei_zp.dt == B200_DT_S4);
    const bool fastq = w4 && pow2(a.gs_blocks) && pow2(a.gz_blocks) && (!p->wei_scale.ptr || p->wei_scale.dt == B200_DT_BF16)
            && (!p->wei_zp.ptr || z4) && (p->K / TK + 1) * (p->N + 1) < ((int64_t)1 << 31);
    a.nibble_offset = p->wei_dt == B200_DT_S4 ? 136.f : 128.f;
    a.byte_xor = p->wei_dt == B200_DT_S8 ? 0x80808080u : 0u;
    a.tmem_cols = 32;
    while ((int)a.tmem_cols < ISSUERS * a.nb) a.tmem_cols *= 2; // one accumulator of nb columns per issuing thread
    // instruction descriptor: D f32, A and B bf16, both K-major, N = nb, M = 128
    a.idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(a.nb >> 3) << 17) | ((uint32_t)(TN >> 4) << 24);

    wctc_encode_fn fn = wctc_get_encode_fn();
    if (!fn) return (int)cudaErrorUnknown;
    CUtensorMap tx;
    {
        // bytes: rows of K * 2 bytes; box = 128 bytes of K x nb rows, 128-byte swizzle; rows past M read as zero
        const cuuint64_t gdim[2] = {(cuuint64_t)p->K * 2, (cuuint64_t)p->M};
        const cuuint64_t gstride[1] = {(cuuint64_t)p->src_sm * 2};
        const cuuint32_t box[2] = {(cuuint32_t)(TK * 2), (cuuint32_t)a.nb};
        const cuuint32_t estr[2] = {1, 1};
        if (fn(&tx, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(p->src), gdim, gstride, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE)
                != CUDA_SUCCESS)
            return (int)cudaErrorUnknown;
    }

    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int64_t tiles = (int64_t)a.n_tiles * a.m_passes;
    const unsigned grid = (unsigned)(tiles < sms ? tiles : sms);
    // shared memory: the packed-weights ring, then the deepest pair of rings that fits
    const size_t b_bytes = (size_t)a.nb * TK * 2;
    const size_t fixed = 1024 + (size_t)pfs(wbits) * DQ_WARPS * 32 * pf_bytes(wbits) + sizeof(ctrl_t);
    static const int depths[][2] = {{8, 8}, {8, 6}, {6, 6}, {6, 4}, {4, 4}};
    a.a_stages = a.b_stages = 0;
    for (const auto &d : depths)
        if (fixed + (size_t)d[0] * A_BYTES + (size_t)d[1] * b_bytes <= 227 * 1024) {
            a.a_stages = (uint32_t)d[0];
            a.b_stages = (uint32_t)d[1];
            break;
        }
    if (!a.a_stages) return B200_ERR_UNSUPPORTED;
    const size_t smem = fixed + (size_t)a.a_stages * A_BYTES + (size_t)a.b_stages * b_bytes;
    static std::mutex mu;
    static bool attr_done[64] = {};
    {
        std::lock_guard<std::mutex> g(mu);
        if (dev < 64 && !attr_done[dev]) {
            cudaError_t e = cudaFuncSetAttribute(wc_tc_kernel<4, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
            if (e == cudaSuccess) e = cudaFuncSetAttribute(wc_tc_kernel<4, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
            if (e == cudaSuccess) e = cudaFuncSetAttribute(wc_tc_kernel<8, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
            if (e != cudaSuccess) return (int)e;
            attr_done[dev] = true;
        }
    }
    if (w4 && fastq) wc_tc_kernel<4, true><<<grid, NUM_THREADS, smem, cs>>>(tx, a);
    else if (w4) wc_tc_kernel<4, false><<<grid, NUM_THREADS, smem, cs>>>(tx, a);
    else wc_tc_kernel<8, false><<<grid, NUM_THREADS, smem, cs>>>(tx, a);
    return after_launch();
}
