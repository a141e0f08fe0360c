// Pieces shared by the tensor-core kernels that stream the packed weights (the decode GEMV and the small-batch kernel):
// tcgen05 / TMA wrappers, the split of the work list over the CTAs, and bounded barrier waits.
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace sbvr {

constexpr int TS_HDR = 1024;                    // barriers, flags, tensor-memory base
constexpr int TS_TMEM_COLS = 512;
constexpr int TS_SF_COL = 480;                  // 32 columns of unit scale factors
constexpr int TS_MAX_STAGES = 8;
constexpr int TS_STAGE_WORDS = 4096;            // bytes of packed words per 256-k block of a stage

__host__ __device__ constexpr int ts_sp(int S) { return S == 2 ? 2 : 4; }            // MMA rows per output row
__host__ __device__ constexpr int ts_tn(int S) { return 128 / ts_sp(S); }            // output rows per tile
__host__ __device__ inline int ts_round_up(int v, int a) { return (v + a - 1) / a * a; }

// Tensor map of the packed words, uint32 [K/32 rows][N * S], box 8 KS rows x TN * S words (cached per weight).
int ts_tensor_map(const PackedW& w, int KS, CUtensorMap* out);

// ---------------------------------------------------------------------------------------------
// tcgen05 / TMA wrappers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void ts_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void ts_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ uint64_t ts_bdesc(uint32_t saddr, uint32_t sbo = 1024u) {
    // K-major, no swizzle: core matrices of 8 rows x 16 B; 128 B between the two K chunks of one MMA,
    // `sbo` bytes between groups of 8 rows; descriptor version 1 (sm_100)
    return (uint64_t)((saddr & 0x3FFFF) >> 4) | ((uint64_t)(128 >> 4) << 16) | ((uint64_t)(sbo >> 4) << 32) |
           ((uint64_t)1 << 46);
}

__device__ __forceinline__ void ts_mma(uint32_t d_t, uint32_t a_t, uint64_t bdesc, uint32_t idesc, uint32_t sfa,
                                       uint32_t sfb, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.scale_vec::2X [%0], [%1], %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(d_t), "r"(a_t), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
        : "memory");
}

__device__ __forceinline__ void ts_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ void ts_st32(uint32_t taddr, const uint32_t (&a)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
        "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(a[4]), "r"(a[5]), "r"(a[6]), "r"(a[7]), "r"(a[8]), "r"(a[9]),
        "r"(a[10]), "r"(a[11]), "r"(a[12]), "r"(a[13]), "r"(a[14]), "r"(a[15]), "r"(a[16]), "r"(a[17]), "r"(a[18]),
        "r"(a[19]), "r"(a[20]), "r"(a[21]), "r"(a[22]), "r"(a[23]), "r"(a[24]), "r"(a[25]), "r"(a[26]), "r"(a[27]),
        "r"(a[28]), "r"(a[29]), "r"(a[30]), "r"(a[31])
        : "memory");
}
__device__ __forceinline__ void ts_st8(uint32_t taddr, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t a4, uint32_t a5,
                                       uint32_t a6, uint32_t a7) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr), "r"(a0), "r"(a1), "r"(a2),
                 "r"(a3), "r"(a4), "r"(a5), "r"(a6), "r"(a7)
                 : "memory");
}
__device__ __forceinline__ void ts_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// Waits for this thread's tensor-memory loads; the registers are operands so that nothing uses them earlier.
__device__ __forceinline__ void ts_wait_ld(uint32_t (&r)[8]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7])
                 :
                 : "memory");
}

// Sixteen columns of this thread's tensor-memory lane; valid after ts_wait_ld() on both halves.
__device__ __forceinline__ void ts_ld16_issue(uint32_t taddr, uint32_t (&lo)[8], uint32_t (&hi)[8]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(lo[0]), "=r"(lo[1]), "=r"(lo[2]), "=r"(lo[3]), "=r"(lo[4]), "=r"(lo[5]), "=r"(lo[6]), "=r"(lo[7]), "=r"(hi[0]),
          "=r"(hi[1]), "=r"(hi[2]), "=r"(hi[3]), "=r"(hi[4]), "=r"(hi[5]), "=r"(hi[6]), "=r"(hi[7])
        : "r"(taddr)
        : "memory");
}

// Eight columns of this thread's tensor-memory lane; the values are valid after ts_wait_ld().
__device__ __forceinline__ void ts_ld8_issue(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
}

// One box of a 2-D tensor map, global -> shared, completion counted on an mbarrier.  No multicast.
__device__ __forceinline__ void ts_tma_2d(void* dst_smem, const CUtensorMap* tmap, int c0, int c1, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(dst_smem)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(c0), "r"(c1), "r"(smem_u32(bar))
        : "memory");
}

__device__ __forceinline__ void ts_bar_arrive(int id, int nthreads) {
    asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// ---------------------------------------------------------------------------------------------
// The steps of a CTA, in the order it processes them.
//
// A step is KS 256-k blocks of one row tile; a row tile has KBS steps.  With G CTAs and NT row tiles every CTA owns
// base = NT / G WHOLE tiles (tiles c base .. c base + base - 1); the R = NT % G tiles left over are cut into their
// R KBS steps, and CTA c takes steps [c R KBS / G, (c + 1) R KBS / G) of that list: one or two steps each, so every SM
// gets the same work to within a step.  A CTA therefore has at most two "shared" segments (parts of left-over tiles,
// finished together with other CTAs) and they come first, then its whole tiles.
// ---------------------------------------------------------------------------------------------
struct TsSegs {
    int KBS, base, rem_tile0, own_tile0;
    int r0, r1, rt_first, nrs, nseg, steps;
    unsigned int RS, G;
    // RS * G < 2^32 is checked by the host (linear_tcs_supported)
    __host__ __device__ void init(int NT, int KBS_, unsigned int G_, unsigned int c) {
        KBS = KBS_;
        G = G_;
        base = NT / (int)G;
        const int R = NT - base * (int)G;
        RS = (unsigned int)(R * KBS);
        rem_tile0 = base * (int)G;
        own_tile0 = (int)c * base;
        r0 = (int)(c * RS / G);
        r1 = (int)((c + 1u) * RS / G);
        rt_first = r0 / KBS;
        nrs = (r1 > r0) ? (r1 - 1) / KBS - rt_first + 1 : 0;
        nseg = nrs + base;
        steps = base * KBS + (r1 - r0);
    }
    __host__ __device__ int tile(int q) const { return q < nrs ? rem_tile0 + rt_first + q : own_tile0 + (q - nrs); }
    __host__ __device__ int k0(int q) const { return (q < nrs && q == 0) ? r0 - rt_first * KBS : 0; }
    __host__ __device__ int k1(int q) const { return (q < nrs && q == nrs - 1) ? r1 - (rt_first + q) * KBS : KBS; }
    __host__ __device__ bool shared(int q) const { return k1(q) - k0(q) < KBS; }
    // the CTA that owns step r of the left-over list
    __host__ __device__ int cta_of(unsigned int r) const { return (int)(((r + 1u) * G - 1u) / RS); }
    // which of its two exchange slots CTA cc uses for left-over tile rt
    __host__ __device__ int slot_of(unsigned int cc, int rt) const { return (rt == (int)(cc * RS / G) / KBS) ? 0 : 1; }
};

// Position in that list, advanced by a fixed stride (the number of warpgroups).
struct TsCursor {
    int q, k, k_end;              // segment, k block inside its tile, end of the segment's k range
    __device__ void start(const TsSegs& sg, int pos) {
        q = 0;
        k = 0, k_end = 0;
        if (sg.nseg > 0) {
            k = sg.k0(0) + pos;
            k_end = sg.k1(0);
            norm(sg);
        }
    }
    __device__ void norm(const TsSegs& sg) {
        while (q < sg.nseg && k >= k_end) {
            const int over = k - k_end;
            ++q;
            if (q < sg.nseg) {
                k = sg.k0(q) + over;
                k_end = sg.k1(q);
            }
        }
    }
    __device__ void advance(const TsSegs& sg, int n) {
        k += n;
        norm(sg);
    }
    __device__ bool done(const TsSegs& sg) const { return q >= sg.nseg; }
};


// ---------------------------------------------------------------------------------------------
// bounded waits
// ---------------------------------------------------------------------------------------------
// Slow path of ts_wait: polls until the phase completes or about a second of SM clock has passed.  A time-out is
// recorded in the status words and in the CTA's abort flag; the caller then carries on as if the phase had completed
// (its results are garbage, the host sees SBVR_ERR_TIMEOUT), and every later wait of the CTA gives up at once, so
// that the barrier protocol of the CTA runs to its end instead of hanging.
template <int UNUSED = 0>      // a template only so that the header can be included by several translation units
__device__ __noinline__ void ts_wait_slow(uint32_t bar, uint32_t parity, volatile int* abort_flag, unsigned int* status,
                                          uint32_t where, bool heed_abort) {
    const long long t0 = clock64();
    for (;;) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.b32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(bar), "r"(parity)
            : "memory");
        if (ok) return;
        if (heed_abort && *abort_flag) return;
        if (clock64() - t0 > 2000000000LL) {
            *abort_flag = 1;
            atomicExch(status, 1u);
            atomicExch(status + 1, where);
            return;
        }
    }
}
__device__ __forceinline__ void ts_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, unsigned int* status,
                                        uint32_t where, bool heed_abort = true) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    if (!ok) ts_wait_slow(bar, parity, abort_flag, status, where, heed_abort);
}

}  // namespace sbvr
