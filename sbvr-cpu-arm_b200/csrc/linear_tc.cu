// Decode-time SBVR linear (M <= 4 activation rows) on the 5th-generation tensor cores, one launch.
//
//   y[n] = sum_g sum_s c[g,n,s] * ( sum_{k in g} x[k] * bit_s[n,k] )
//
// The inner sum is a dot product of the activations with a 0/1 vector, evaluated by
// tcgen05.mma kind::mxf4 (packed 4-bit E2M1 operands, fp32 accumulation in tensor memory):
//
//  A operand (weights)  One MMA row per (output row n, plane s).  A packed word w holds 32 k of one
//      row.  E2M1 codes 1, 2, 4 are the values 0.5, 1, 2, so `w & 0x11111111`, `w & 0x22222222`,
//      `w & 0x44444444` and `(w >> 1) & 0x44444444` are four words of eight 4-bit elements each,
//      holding the bits k = j, j+4, ..., j+28 (j = 0..3) as {0, 0.5}, {0, 1}, {0, 2}, {0, 2}: five
//      integer instructions expand 32 plane bits.  The words go straight from registers into
//      tensor memory (tcgen05.st) and the MMA reads A from there: the expanded form (4x the packed
//      bytes) never touches shared memory.
//  B operand (activations)  Each group of 256 activations is block fixed point, q = x / step in
//      16-bit two's complement with a power-of-two step per group of G; q is written as eight
//      radix-4 digits, digits 0..6 in {0,1,2,3}, digit 7 in {-2,-1,0,1}, pre-multiplied by 2, 1,
//      0.5, 0.5 for k = 0, 1, 2, 3 (mod 4) to undo A's weights; all of these are exact E2M1 values.
//      The 8 digits of an activation row are 8 columns of the MMA's N dimension, stored in the same
//      k permutation as A.  Every CTA quantises x itself into shared memory (no separate launch).
//  D  128 rows x (8 digits x rows of x) fp32 per 256 k, exact small integers.  The epilogue reads it
//      with tcgen05.ld, forms sum_d 4^d D[d] (exact, < 2^24), multiplies by the row's fp16
//      coefficient and the group's step and accumulates in fp32.
//  The block scale factors the instruction requires are all set to 2^0 once per CTA.
//
// The only deviation from an fp32-accumulated product of the fp16 inputs is the block
// fixed-point rounding of activations more than 2^4 below their group's maximum: at most 2^-16 of
// that maximum per element.
//
// Replaces cuda_1xtN_rd_WP8_TBW4_NS4 / cuda_row_deq_mm_T (reference sbvr/kernels/sbvr_kernel.cu:284-359,
// :121-191), whose per-bit select + FMA needs 3-5x more issue slots than HBM3e leaves per element.
//
// Structure: one CTA per SM, 21 warps.  A CTA owns whole row tiles (128 MMA rows = 32 output rows
// for S = 3, 4; 64 for S = 2) and takes them round-robin; inside a row tile the four compute
// warpgroups split K into four contiguous quarters, so no partial sum ever leaves the SM.
// Thread r of a warpgroup owns MMA row r: the 8 packed words of its row per 256 k come from global
// memory through a per-warp cp.async ring in shared memory (a warp reads 128 contiguous bytes per
// word row; loads run three tiles ahead of their use); it expands them, stores them to its
// tensor-memory lane and signals an mbarrier.  Four issuer warps (one per warpgroup) wait on those
// barriers and issue the four K = 64 MMAs of a tile from one elected lane of a converged warp (a lone divergent thread
// needs about twice as long per tcgen05.mma).  A and D are double buffered in tensor memory so that
// the MMAs of a tile overlap the expansion of the next and the epilogue of the previous one.
// When a warpgroup has finished its quarter of a row tile it leaves its fp32 sums in shared memory;
// a finisher warp adds the four quarters and the planes in a fixed order (deterministic), adds the
// bias and writes fp16.  Every wait is bounded; on time-out the kernel records it in the status
// word, frees its tensor memory and leaves.
#include "common.cuh"

namespace sbvr {

constexpr int TC_WGS = 4;                       // warpgroups that compute
constexpr int TC_CTHREADS = TC_WGS * 128;
constexpr int TC_IWARPS = 4;                    // MMA issuer warps, each serves TC_WGS / TC_IWARPS warpgroups
constexpr int TC_FWARP = TC_WGS * 4 + TC_IWARPS;            // the finisher warp
constexpr int TC_THREADS = TC_CTHREADS + 32 * TC_IWARPS + 32;
constexpr int TC_HDR = 1024;                    // barriers, flags, tensor-memory base
constexpr int TC_TMEM_COLS = 512;
constexpr int TC_WG_COLS = 112;                 // tensor-memory columns per warpgroup: A 2 x 32, D 3 x 16 (or 32 + 64)
constexpr int TC_SF_COL = 448;                  // 32 columns of unit scale factors
constexpr int TC_BSLACK = 4096;                 // MMA columns beyond M read (and ignore) what follows
constexpr int TC_STAGES = 4;                    // packed words of the next three tiles are in flight per warpgroup
constexpr int TC_STAGE_BYTES = 1152;              // per warp and stage: 8 x 128 B of packed words + 128 B of coefficient data
constexpr int TC_RING_BYTES = TC_WGS * 4 * TC_STAGES * TC_STAGE_BYTES;

struct TcParams {
    const __half* x;
    const uint32_t* bvr;
    const void* idx;
    const __half* coeff;
    const __half* bias;
    __half* y;
    unsigned int* status;
    int N, K, KB, NT, C, cache_in_smem;
    // what the activations are made of while they are brought in (XOp): nothing, SiLU(gate) * up, or
    // RMSNorm(h + delta) * weight with the new residual written once
    int x_op;
    const __half* delta;
    const __half* norm_w;
    __half* h_out;
    float eps;
};

__host__ __device__ constexpr int tc_sp(int S) { return S == 2 ? 2 : 4; }            // MMA rows per output row
__host__ __device__ constexpr int tc_tn(int S) { return 128 / tc_sp(S); }            // output rows per tile
__host__ __device__ constexpr int tc_mpad(int M) { return M <= 2 ? 2 : 4; }
__host__ __device__ inline int tc_round_up(int v, int a) { return (v + a - 1) / a * a; }

// ---------------------------------------------------------------------------------------------
// tcgen05 wrappers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ uint64_t tc_bdesc(uint32_t saddr) {
    // K-major, no swizzle: core matrices of 8 rows x 16 B; 128 B between the two K chunks of one MMA,
    // 1024 B between groups of 8 rows; descriptor version 1 (sm_100)
    return (uint64_t)((saddr & 0x3FFFF) >> 4) | ((uint64_t)(128 >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46);
}

__device__ __forceinline__ void tc_mma(uint32_t d_t, uint32_t a_t, uint64_t bdesc, uint32_t idesc, uint32_t sfa,
                                       uint32_t sfb, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.scale_vec::2X [%0], [%1], %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(d_t), "r"(a_t), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
        : "memory");
}

__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ void tc_st32(uint32_t taddr, const uint32_t (&a)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
        "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(a[4]), "r"(a[5]), "r"(a[6]), "r"(a[7]), "r"(a[8]), "r"(a[9]),
        "r"(a[10]), "r"(a[11]), "r"(a[12]), "r"(a[13]), "r"(a[14]), "r"(a[15]), "r"(a[16]), "r"(a[17]), "r"(a[18]),
        "r"(a[19]), "r"(a[20]), "r"(a[21]), "r"(a[22]), "r"(a[23]), "r"(a[24]), "r"(a[25]), "r"(a[26]), "r"(a[27]),
        "r"(a[28]), "r"(a[29]), "r"(a[30]), "r"(a[31])
        : "memory");
}
__device__ __forceinline__ void tc_st_fill32(uint32_t taddr, uint32_t v) {
    uint32_t a[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) a[i] = v;
    tc_st32(taddr, a);
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void tc_ld8(uint32_t taddr, float (&d)[8]) {
    uint32_t r[8];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
    tc_wait_ld();
#pragma unroll
    for (int i = 0; i < 8; ++i) d[i] = __uint_as_float(r[i]);
}

// Optional timestamp trace of thread 0 of CTA 0 (development builds only, -DSBVR_PROFILE).
#ifdef SBVR_PROFILE
__device__ long long g_tc_prof[8 * 64 + 16];
__device__ long long g_tc_iprof[4 * 64];
#define TC_PROF(slot)                                                                                             \
    do {                                                                                                          \
        if (blockIdx.x == 0 && threadIdx.x == 0 && prof_tile < 64) g_tc_prof[prof_tile * 8 + (slot)] = clock64(); \
    } while (0)
#define TC_PROF_NEXT() ++prof_tile
#define TC_IPROF(slot)                                                                                              \
    do {                                                                                                            \
        if (blockIdx.x == 0 && threadIdx.x == TC_WGS * 128 && prof_tile < 64) g_tc_iprof[prof_tile * 4 + (slot)] = clock64(); \
    } while (0)
#define TC_PROF_MARK(k)                                                               \
    do {                                                                              \
        if (blockIdx.x == 0 && threadIdx.x == 0) g_tc_prof[8 * 64 + (k)] = clock64(); \
    } while (0)
#else
#define TC_PROF(slot) do { } while (0)
#define TC_PROF_NEXT() do { } while (0)
#define TC_IPROF(slot) do { } while (0)
#define TC_PROF_MARK(k) do { } while (0)
#endif

// ---------------------------------------------------------------------------------------------
// the product
// ---------------------------------------------------------------------------------------------
template <int S, int NSUB, int M, int IDXB>
__global__ void __launch_bounds__(TC_THREADS, 1) linear_tc_kernel(const TcParams p) {
#ifdef SBVR_PROFILE
    int prof_tile = 0;
#endif
    TC_PROF_MARK(0);
    pdl_launch_dependents();                       // the next kernel on the stream may be scheduled as SMs free up
    extern __shared__ __align__(128) unsigned char smem[];
    constexpr int SP = tc_sp(S);
    constexpr int TN = tc_tn(S);
    constexpr int MPAD = tc_mpad(M);
    constexpr int NMMA = 8 * MPAD;                 // MMA N: 8 digits per activation row
    constexpr bool PIPE = (NSUB * NMMA <= 16);     // room in tensor memory for two D buffers
    // instruction descriptor: A, B = E2M1 (1), scales UE8M0, M = 128, N = NMMA, K-major both, K = 64
    constexpr uint32_t IDESC = (1u << 7) | (1u << 10) | ((uint32_t)(NMMA >> 3) << 17) | (1u << 23) | (8u << 24);

    uint64_t* mma_bar = reinterpret_cast<uint64_t*>(smem);                            // [TC_WGS][3] MMAs of a tile done
    uint64_t* a_ready = mma_bar + 3 * TC_WGS;                                         // [TC_WGS][2] A of a tile stored
    uint64_t* red_full = a_ready + 2 * TC_WGS;                                        // [2] sums of a row tile deposited
    uint64_t* red_empty = red_full + 2;                                               // [2] ... and consumed
    uint64_t* b_ready = red_empty + 2;                                                // [1] activation digits written
    uint64_t* tmem_ready = b_ready + 1;                                               // [1] tensor memory allocated
    uint64_t* cache_bar = tmem_ready + 1;                                             // [1] codebook copied
    volatile int* flags = reinterpret_cast<volatile int*>(cache_bar + 1);             // [0] abort
    uint32_t* tmem_base_s = reinterpret_cast<uint32_t*>(smem + TC_HDR - 16);

    const int KB = p.KB, N = p.N;
    const int sbytes = tc_round_up(M * KB * NSUB * 4, 16);
    const int cbytes = p.cache_in_smem ? tc_round_up(p.C * S * 2, 16) : 0;
    float* xsc = reinterpret_cast<float*>(smem + TC_HDR);                            // [M][KB][NSUB] steps
    float* red = reinterpret_cast<float*>(smem + TC_HDR + sbytes);                   // [2][TC_WGS][M][128]
    __half* cache_s = reinterpret_cast<__half*>(smem + TC_HDR + sbytes + 2 * TC_WGS * M * 128 * 4);
    uint32_t* wring = reinterpret_cast<uint32_t*>(
        smem + tc_round_up(TC_HDR + sbytes + 2 * TC_WGS * M * 128 * 4 + cbytes, 128));  // [TC_WGS][TC_STAGES][8][128]
    unsigned char* Bs = smem + tc_round_up(tc_round_up(TC_HDR + sbytes + 2 * TC_WGS * M * 128 * 4 + cbytes, 128) +
                                               TC_RING_BYTES, 1024);                      // [KB][M][1024]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = (int)gridDim.x;
    const int n_units = ((int)blockIdx.x < p.NT) ? (p.NT - 1 - (int)blockIdx.x) / G + 1 : 0;   // row tiles of this CTA

    if (threadIdx.x < 5 * TC_WGS + 7) {            // one barrier per thread: the barriers are contiguous
        const int i = threadIdx.x;
        const uint32_t count = (i < 3 * TC_WGS)       ? 1u
                               : (i < 5 * TC_WGS)     ? 4u
                               : (i < 5 * TC_WGS + 2) ? (uint32_t)(TC_WGS * 4)
                               : (i < 5 * TC_WGS + 4) ? 1u
                               : (i == 5 * TC_WGS + 4) ? (uint32_t)(TC_WGS * 4)
                                                       : 1u;
        mbar_init(&mma_bar[i], count);
        if (i == 0) flags[0] = 0;
        fence_mbar_init();
    }
    __syncthreads();                               // barriers are initialised; nothing else is waited for here
    TC_PROF_MARK(1);

    // k blocks [lo, hi) of warpgroup j inside every row tile
    auto kb_lo = [&](int j) { return (KB * j) / TC_WGS; };
    // Tensor memory is allocated by the finisher warp while the others already load and quantise;
    // whoever needs the base address waits for `tmem_ready` first.
    auto wait_tmem = [&]() -> bool {
        const bool ok = mbar_wait_timed(tmem_ready, 0u);
        tc_fence_after();
        return ok;
    };
    const bool bulk_cache = p.cache_in_smem && ((p.C * S * 2) % 16 == 0);

    if (warp == TC_FWARP) {
        // ------------------------------ finisher warp ------------------------------
        if (bulk_cache && lane == 0) {             // codebook -> shared memory, one asynchronous copy
            mbar_arrive_expect_tx(cache_bar, (uint32_t)(p.C * S * 2));
            bulk_g2s(cache_s, p.coeff, (uint32_t)(p.C * S * 2), cache_bar);
        }
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_base_s)),
                     "r"((uint32_t)TC_TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tmem_ready);
        uint32_t fph[2] = {0u, 0u};
        bool ok = true;
        for (int ui = 0; ui < n_units && ok; ++ui) {
            const int ub = ui & 1;
            if (flags[0] || !mbar_wait_timed(&red_full[ub], fph[ub])) {
                ok = false;
                flags[0] = 1;
                break;
            }
            fph[ub] ^= 1u;
            const int n0 = ((int)blockIdx.x + ui * G) * TN;
            const float* rs = red + (size_t)ub * TC_WGS * M * 128;
            for (int i = lane; i < M * TN; i += 32) {
                const int m = i / TN, nl = i % TN;
                float v = 0.0f;
#pragma unroll
                for (int j = 0; j < TC_WGS; ++j)
#pragma unroll
                    for (int s = 0; s < SP; ++s) v += rs[(j * M + m) * 128 + nl * SP + s];
                const float b = p.bias ? __half2float(p.bias[n0 + nl]) : 0.0f;
                p.y[(size_t)m * N + n0 + nl] = __float2half_rn(v + b);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&red_empty[ub]);
        }
        if (!ok && lane == 0) {
            atomicExch(p.status, 1u);
            atomicExch(p.status + 1, 0x300u + blockIdx.x);
        }
    } else if (warp >= TC_WGS * 4) {
        // ------------------------------ issuer warps ------------------------------
        const int iw = warp - TC_WGS * 4;
        constexpr int PER = TC_WGS / TC_IWARPS;
        int lo[PER], hi[PER], kbs[PER], units[PER], cnt[PER], dbufs[PER];
        uint32_t aph[PER][2];
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            lo[j] = kb_lo(iw * PER + j);
            hi[j] = kb_lo(iw * PER + j + 1);
            kbs[j] = lo[j];
            units[j] = (hi[j] > lo[j]) ? n_units : 0;      // row tiles still to do
            cnt[j] = 0;
            dbufs[j] = 0;
            aph[j][0] = aph[j][1] = 0u;
        }
        bool ok = wait_tmem() && mbar_wait_timed(b_ready, 0u);   // tensor memory is there, the digits are written
        const uint32_t tbase = *tmem_base_s;
        const uint32_t sfa = tbase + TC_SF_COL, sfb = sfa;       // every scale byte is 2^0: one region serves both
        bool any = true;
        while (ok && any) {
            any = false;
#pragma unroll
            for (int j = 0; j < PER; ++j) {
                if (!ok || units[j] <= 0) continue;
                any = true;
                const int wgj = iw * PER + j;
                const int buf = PIPE ? (cnt[j] & 1) : 0;        // A buffer
                const int dbuf = PIPE ? dbufs[j] : 0;           // D buffer (three of them when pipelined)
                const int kb = kbs[j];
                const uint32_t a_col = tbase + wgj * TC_WG_COLS;
                const uint32_t d_col = a_col + (PIPE ? 64 : 32);
                TC_IPROF(0);
                if (flags[0] || !mbar_wait_timed(&a_ready[wgj * 2 + buf], aph[j][buf])) {
                    ok = false;
                    continue;
                }
                aph[j][buf] ^= 1u;
                TC_IPROF(1);
                tc_fence_after();
                const uint32_t bs = smem_u32(Bs + (size_t)kb * M * 1024);
                if (elect_one()) {
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const int sub = (NSUB == 2) ? (q >> 1) : 0;
                        const uint32_t accum = (NSUB == 2) ? (uint32_t)(q & 1) : (uint32_t)(q > 0);
                        tc_mma(d_col + dbuf * NMMA + sub * NMMA, a_col + buf * 32 + q * 8, tc_bdesc(bs + q * 256), IDESC,
                               sfa, sfb, accum);
                    }
                    tc_commit(&mma_bar[wgj * 3 + dbuf]);
                }
                __syncwarp();
                TC_IPROF(2);
                TC_PROF_NEXT();
                cnt[j] += 1;
                dbufs[j] = (dbuf == 2) ? 0 : dbuf + 1;
                if (kb + 1 == hi[j]) {
                    kbs[j] = lo[j];
                    units[j] -= 1;
                } else {
                    kbs[j] = kb + 1;
                }
            }
        }
        if (!ok) {
            flags[0] = 1;
            if (lane == 0) {
                atomicExch(p.status, 1u);
                atomicExch(p.status + 1, 0x100u + blockIdx.x);
            }
        }
    } else {
        // ------------------------------ compute warpgroups ------------------------------
        const int ctid = threadIdx.x;              // 0 .. 511
        const int wg = warp >> 2, wl = warp & 3;
        const int r = wl * 32 + lane;              // MMA row = tensor-memory lane
        const int nl = r / SP, s = r % SP;         // output row inside the tile, plane
        const bool live_row = s < S;
        const uint32_t lane_sel = (uint32_t)(wl * 32) << 16;
        const int my_lo = kb_lo(wg), my_hi = kb_lo(wg + 1);
        const int per_unit = my_hi - my_lo;
        const int n_tiles = per_unit * n_units;

        // ---- loads run three tiles ahead, global -> shared memory with cp.async, one ring per warp.  A warp
        // needs, per 256-k tile, 8 rows (one per 32 k) of 128 contiguous bytes (96 for S = 3) and the coefficient
        // indices (or direct coefficients) of its 32 MMA rows: 64 (48) pieces of 16 bytes, two per lane, plus up
        // to 8 pieces of 8 bytes.  Lanes copy for each other, so a __syncwarp follows the wait; no register
        // scoreboard is tied up for a memory latency.  Byte offsets are 32-bit and advance by constants.
        constexpr int CPR = (S == 3) ? 6 : 8;                  // 16-byte pieces per 32-k row of a warp
        constexpr int WROW = CPR * 16;                         // bytes of such a row
        constexpr int CI_PIECES = (IDXB == 0) ? (32 / SP) * S * 2 / 8 : ((32 / SP) * IDXB + 7) / 8;   // 8-byte pieces per sub
        constexpr int CI_BYTES = (IDXB == 0) ? (32 / SP) * S * 2 : (32 / SP) * IDXB;
        constexpr int STAGE_B = TC_STAGE_BYTES;                // 1024 B of words + 128 B of coefficient data
        const uint32_t ROWB = (uint32_t)N * S * 4;             // bytes between the rows of consecutive 32-k words
        const uint32_t KSTEP_B = 8u * ROWB;
        const uint32_t CIROW = (IDXB == 0) ? (uint32_t)N * S * 2 : (uint32_t)N * IDXB;     // bytes per coefficient group
        const uint32_t ISTEP_B = (uint32_t)NSUB * CIROW;
        // from the last tile of a row tile to the first tile of this CTA's next row tile
        const uint32_t WRAP_B = (uint32_t)G * TN * S * 4 - (uint32_t)(per_unit - 1) * KSTEP_B;
        const uint32_t IWRAP_B = (uint32_t)G * TN * (CIROW / N) - (uint32_t)(per_unit - 1) * ISTEP_B;
        int kb_l = my_lo, loaded = 0;
        uint32_t off_l = ((uint32_t)(my_lo * 8) * N + (uint32_t)blockIdx.x * TN) * S * 4;
        uint32_t ioff_l = (uint32_t)(my_lo * NSUB) * CIROW + (uint32_t)blockIdx.x * TN * (CIROW / N);
        unsigned char* ring_w = reinterpret_cast<unsigned char*>(wring) + (size_t)warp * TC_STAGES * STAGE_B;
        const uint32_t ring_s = smem_u32(ring_w);
        const int c1 = lane + 32;                              // second 16-byte piece of this lane
        const bool two = c1 < 8 * CPR;
        const uint32_t rel0 = (uint32_t)(lane / CPR) * ROWB + (uint32_t)wl * WROW + (uint32_t)(lane % CPR) * 16;
        const uint32_t rel1 = (uint32_t)(c1 / CPR) * ROWB + (uint32_t)wl * WROW + (uint32_t)(c1 % CPR) * 16;
        const bool ci_lane = lane < NSUB * CI_PIECES;
        const int ci_sub = lane / CI_PIECES, ci_pc = lane % CI_PIECES;
        const uint32_t irel = (uint32_t)ci_sub * CIROW + (uint32_t)wl * CI_BYTES + (uint32_t)ci_pc * 8;
        const unsigned char* wbytes = reinterpret_cast<const unsigned char*>(p.bvr);
        const unsigned char* cbytes_g = (IDXB == 0) ? reinterpret_cast<const unsigned char*>(p.coeff)
                                                    : reinterpret_cast<const unsigned char*>(p.idx);
        auto load_tile = [&]() {
            if (loaded < n_tiles) {
                const uint32_t dst = ring_s + (uint32_t)(loaded % TC_STAGES) * STAGE_B;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + lane * 16), "l"(wbytes + (off_l + rel0))
                             : "memory");
                if (two)
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + c1 * 16),
                                 "l"(wbytes + (off_l + rel1))
                                 : "memory");
                if (ci_lane)
                    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst + 1024 + ci_sub * 64 + ci_pc * 8),
                                 "l"(cbytes_g + (ioff_l + irel))
                                 : "memory");
            }
            asm volatile("cp.async.commit_group;" ::: "memory");      // one group per tile, empty or not
            ++loaded;
            const bool wrap = (++kb_l == my_hi);   // on to this warpgroup's quarter of the CTA's next row tile
            off_l += wrap ? WRAP_B : KSTEP_B;
            ioff_l += wrap ? IWRAP_B : ISTEP_B;
            if (wrap) kb_l = my_lo;
        };
        // ---- set-up shared by the CTA.  The packed words of the first three tiles are requested first: weights do
        // not depend on the previous kernel of the stream, so this (like the barrier set-up, the codebook copy and
        // the tensor-memory allocation) overlaps that kernel's tail.  The activations do: wait for it, then copy
        // them as they are into the first half of each block's digit area.
        load_tile();
        TC_PROF_MARK(11);
        load_tile();
        load_tile();
        pdl_wait();
        if (p.x_op == SBVR_XOP_NONE) {
            const int nchunk = M * KB * 32;        // 16-byte pieces
            for (int c = ctid; c < nchunk; c += TC_CTHREADS) {
                const int part = c & 31, blk = c >> 5;     // blk = m * KB + kb
                const int m = blk / KB, kb = blk - m * KB;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(
                                 smem_u32(Bs + ((size_t)kb * M + m) * 1024 + part * 16)),
                             "l"(p.x + (size_t)m * p.K + (size_t)kb * 256 + part * 8)
                             : "memory");
            }
        } else if (p.x_op == SBVR_XOP_SILU_MUL) {
            // x[m][k] = fp16(silu(g[m][k])) * u[m][k] with rows [g (K) | u (K)]: the activation of the MLP, formed here
            // instead of in a kernel of its own (every CTA needs all of x anyway)
            const int nchunk = M * KB * 32;
            for (int c = ctid; c < nchunk; c += TC_CTHREADS) {
                const int part = c & 31, blk = c >> 5;
                const int m = blk / KB, kb = blk - m * KB;
                const __half* gp = p.x + (size_t)m * 2 * p.K + (size_t)kb * 256 + part * 8;
                const uint4 g = __ldg(reinterpret_cast<const uint4*>(gp));
                const uint4 u = __ldg(reinterpret_cast<const uint4*>(gp + p.K));
                const __half2* gh = reinterpret_cast<const __half2*>(&g);
                const __half2* uh = reinterpret_cast<const __half2*>(&u);
                uint4 o;
                __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 f = __half22float2(gh[e]);
                    oh[e] = __hmul2(__floats2half2_rn(f.x / (1.0f + expf(-f.x)), f.y / (1.0f + expf(-f.y))), uh[e]);
                }
                *reinterpret_cast<uint4*>(Bs + ((size_t)kb * M + m) * 1024 + part * 16) = o;
            }
        } else {
            // x[m] = weight * fp16((h[m] + delta[m]) * rsqrt(mean((h[m] + delta[m])^2) + eps)): the residual add and the
            // RMSNorm in front of the linear.  Pass 1 leaves h + delta in the staging area and sums the squares, pass 2
            // scales in place; CTA 0 also writes the new residual (to a buffer other than h: other CTAs still read h).
            float ss[M];
#pragma unroll
            for (int m = 0; m < M; ++m) ss[m] = 0.0f;
            const int nchunk = M * KB * 32;
            for (int c = ctid; c < nchunk; c += TC_CTHREADS) {
                const int part = c & 31, blk = c >> 5;
                const int m = blk / KB, kb = blk - m * KB;
                const size_t off = (size_t)m * p.K + (size_t)kb * 256 + part * 8;
                uint4 a = __ldg(reinterpret_cast<const uint4*>(p.x + off));
                __half2* ah = reinterpret_cast<__half2*>(&a);
                if (p.delta) {
                    const uint4 b = __ldg(reinterpret_cast<const uint4*>(p.delta + off));
                    const __half2* bh = reinterpret_cast<const __half2*>(&b);
#pragma unroll
                    for (int e = 0; e < 4; ++e) ah[e] = __hadd2(ah[e], bh[e]);
                }
                float sq = 0.0f;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 f = __half22float2(ah[e]);
                    sq += f.x * f.x + f.y * f.y;
                }
#pragma unroll
                for (int mm = 0; mm < M; ++mm) ss[mm] += (mm == m) ? sq : 0.0f;
                *reinterpret_cast<uint4*>(Bs + ((size_t)kb * M + m) * 1024 + part * 16) = a;
                if (p.h_out && blockIdx.x == 0) *reinterpret_cast<uint4*>(p.h_out + off) = a;
            }
            float* ssum = red;                     // [16 warps][M]: the hand-over area is not in use yet
#pragma unroll
            for (int m = 0; m < M; ++m) {
                float v = ss[m];
#pragma unroll
                for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                if (lane == 0) ssum[warp * M + m] = v;
            }
            named_bar_sync(2, TC_CTHREADS);
            float rs[M];
#pragma unroll
            for (int m = 0; m < M; ++m) {
                float tot = 0.0f;
                for (int w = 0; w < TC_WGS * 4; ++w) tot += ssum[w * M + m];
                rs[m] = rsqrtf(tot / (float)p.K + p.eps);
            }
            for (int c = ctid; c < nchunk; c += TC_CTHREADS) {       // the same pieces this thread wrote above
                const int part = c & 31, blk = c >> 5;
                const int m = blk / KB, kb = blk - m * KB;
                uint4* sp = reinterpret_cast<uint4*>(Bs + ((size_t)kb * M + m) * 1024 + part * 16);
                const uint4 a = *sp;
                const uint4 wv = __ldg(reinterpret_cast<const uint4*>(p.norm_w + (size_t)kb * 256 + part * 8));
                const __half2* ah = reinterpret_cast<const __half2*>(&a);
                const __half2* wh = reinterpret_cast<const __half2*>(&wv);
                float r1 = 0.0f;
#pragma unroll
                for (int mm = 0; mm < M; ++mm) r1 = (mm == m) ? rs[mm] : r1;
                uint4 o;
                __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 f = __half22float2(ah[e]);
                    oh[e] = __hmul2(wh[e], __floats2half2_rn(f.x * r1, f.y * r1));
                }
                *sp = o;
            }
            named_bar_sync(2, TC_CTHREADS);        // `red` is free again before anybody hands sums over
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        TC_PROF_MARK(10);
        TC_PROF_MARK(5);
        asm volatile("cp.async.wait_group 0;" ::: "memory");       // this thread's pieces of x have landed
        named_bar_sync(2, TC_CTHREADS);                            // ... and everybody else's
        TC_PROF_MARK(6);
        {
            // Activations -> radix-4 E2M1 digits.  One warp per 256-k block; lane (kw, j) owns the eight
            // elements k = 32 kw + j + 4 e, which are exactly one 32-bit word of every digit plane.
            const int kw = lane >> 2, j = lane & 3;
            // E2M1 codes of digit value t = 0..3 as bytes, scaled by 2, 1, 0.5, 0.5 for j = 0..3; the low digits
            // take t as {0,1,2,3}, the top digit as {0,1,-2,-1}
            const uint32_t pool_lo = (j == 0) ? 0x07060400u : (j == 1) ? 0x05040200u : 0x03020100u;
            const uint32_t pool_hi = (j == 0) ? 0x0C0E0400u : (j == 1) ? 0x0A0C0200u : 0x090A0100u;
            // Digit words are stored rotated by kw (word i of this lane is digit (i + kw) & 7) so that the eight
            // kw of a warp hit different banks; the rotation is applied to the digits themselves, which keeps
            // every register index static.  `top` marks the nibble that holds digit 7 after the rotation.
            const uint32_t rot = 4u * (uint32_t)kw;
            const uint32_t top = 4u << (4u * (uint32_t)(7 - kw));
            for (int blk = warp; blk < M * KB; blk += TC_WGS * 4) {
                const int m = blk / KB, kb = blk - m * KB;
                unsigned char* area = Bs + ((size_t)kb * M + m) * 1024;
                const __half* xp = reinterpret_cast<const __half*>(area) + 32 * kw + j;
                float v[8];
                float a = 0.0f;
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    v[e] = __half2float(xp[4 * e]);
                    float av = fabsf(v[e]);
                    if (!(av == av)) av = __int_as_float(0x7f800000);     // NaN counts as infinity
                    a = fmaxf(a, av);
                }
                __syncwarp();                      // all lanes hold their elements: the area may be overwritten
                TC_PROF_MARK(12);
#pragma unroll
                for (int o = (NSUB == 2 ? 8 : 16); o; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
                TC_PROF_MARK(13);
                float step = 0.0f, inv = 0.0f;
                bool poison = false;
                if (a >= __int_as_float(0x7f800000)) {                    // non-finite activations poison the group
                    step = __int_as_float(0x7fc00000);
                    poison = true;
                } else if (a > 0.0f) {
                    const int ex = (int)((__float_as_uint(a) >> 23) & 0xFF) - 127;   // a = 1.f * 2^ex, ex in [-24, 15]
                    step = __uint_as_float((uint32_t)(ex - 14 + 127) << 23);
                    inv = __uint_as_float((uint32_t)(14 - ex + 127) << 23);
                }
                if (NSUB == 1) {
                    if (lane == 0) xsc[m * KB + kb] = step;
                } else {
                    if ((lane & 15) == 0) xsc[(m * KB + kb) * 2 + (lane >> 4)] = step;
                }
                // per element: 16-bit two's complement -> its 8 radix-4 digits, one per nibble -> rotate -> codes
                uint32_t c_lo[8], c_hi[8];         // bytes i = 0..3 / 4..7: code of rotated digit i
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const uint32_t q = poison ? 1u : (uint32_t)__float2int_rn(v[e] * inv);     // |q| < 2^15
                    uint32_t sp = __byte_perm(q, 0u, 0x4140);                 // bytes [q0, 0, q1, 0]
                    sp = (sp | (sp << 4)) & 0x0F0F0F0Fu;
                    sp = (sp | (sp << 2)) & 0x33333333u;                      // nibble d = digit d
                    sp = __funnelshift_r(sp, sp, rot) | top;                  // nibble i = digit (i + kw) & 7; top digit + 4
                    c_lo[e] = __byte_perm(pool_lo, pool_hi, sp);
                    c_hi[e] = __byte_perm(pool_lo, pool_hi, sp >> 16);
                }
                TC_PROF_MARK(14);
                // element pairs share a byte (low nibble = even element), then a 4 x 4 byte transpose per half
                uint32_t* dstw = reinterpret_cast<uint32_t*>(area) + kw * 32 + j;
#pragma unroll
                for (int hf = 0; hf < 2; ++hf) {
                    uint32_t R[4];
#pragma unroll
                    for (int pr = 0; pr < 4; ++pr)
                        R[pr] = hf ? (c_hi[2 * pr] | (c_hi[2 * pr + 1] << 4)) : (c_lo[2 * pr] | (c_lo[2 * pr + 1] << 4));
                    const uint32_t t0 = __byte_perm(R[0], R[1], 0x5140), t1 = __byte_perm(R[2], R[3], 0x5140);
                    const uint32_t t2 = __byte_perm(R[0], R[1], 0x7362), t3 = __byte_perm(R[2], R[3], 0x7362);
                    const uint32_t T[4] = {__byte_perm(t0, t1, 0x5410), __byte_perm(t0, t1, 0x7632),
                                           __byte_perm(t2, t3, 0x5410), __byte_perm(t2, t3, 0x7632)};
#pragma unroll
                    for (int i = 0; i < 4; ++i) dstw[(((hf * 4 + i) + kw) & 7) * 4] = T[i];   // [kw][digit][16 B], word j
                }
            }
            TC_PROF_MARK(7);
            fence_proxy_async();                   // generic writes of the digits -> visible to the MMA's reads
            __syncwarp();
            if (lane == 0) mbar_arrive(b_ready);
        }
        if (p.cache_in_smem && !bulk_cache) {      // codebook whose byte size is not a multiple of 16: copy by hand
            const int nvec = (p.C * S * 2) / 16;
            const uint4* src = reinterpret_cast<const uint4*>(p.coeff);
            uint4* dst = reinterpret_cast<uint4*>(cache_s);
            for (int i = ctid; i < nvec; i += TC_CTHREADS) dst[i] = __ldg(src + i);
            for (int i = nvec * 8 + ctid; i < p.C * S; i += TC_CTHREADS) cache_s[i] = p.coeff[i];
        }
        bool dead = !wait_tmem();
        dead = __any_sync(0xffffffffu, dead);
        TC_PROF_MARK(8);
        const uint32_t tbase = *tmem_base_s;
        const uint32_t a_col = tbase + wg * TC_WG_COLS;
        const uint32_t d_col = a_col + (PIPE ? 64 : 32);
        if (wg == 0 && !dead) {                    // unit scale factors, every byte 2^0
            tc_st_fill32(tbase + lane_sel + TC_SF_COL, 0x7F7F7F7Fu);
            tc_wait_st();
        }
        tc_fence_before();
        named_bar_sync(1, TC_CTHREADS);            // scale factors, steps, hand-copied codebook and digits are in place
        tc_fence_after();
        TC_PROF_MARK(9);
        if (bulk_cache && !mbar_wait_async(cache_bar, 0u)) dead = true;
        dead = __any_sync(0xffffffffu, dead);
        if (dead) flags[0] = 1;
        TC_PROF_MARK(2);

        float acc[M];
#pragma unroll
        for (int m = 0; m < M; ++m) acc[m] = 0.0f;
        uint32_t mph = 0u;                         // bit d: phase of this warpgroup's MMA barrier of D buffer d
        uint32_t eph = 0u;                         // bit b: phase of "sums consumed" barrier b
        // epilogues run two tiles behind (PIPE): what they need of tiles ti-1 (s1) and ti-2 (s2)
        float s1[NSUB][M], s2[NSUB][M];
        bool last1 = false, last2 = false;
        int ui1 = 0, ui2 = 0;
        int kb_c = my_lo, ui_c = 0, dmod = 0;      // dmod = ti % 3 = D buffer of tile ti
#pragma unroll
        for (int sub = 0; sub < NSUB; ++sub)
#pragma unroll
            for (int m = 0; m < M; ++m) s1[sub][m] = s2[sub][m] = 0.0f;

        // D of one finished tile -> fp32 sums.  `dbuf` selects the D buffer.
        auto epilogue = [&](int dbuf, const float (&scale)[NSUB][M]) {
#pragma unroll
            for (int sub = 0; sub < NSUB; ++sub) {
#pragma unroll
                for (int m = 0; m < M; ++m) {
                    float d[8];
                    tc_ld8(d_col + lane_sel + dbuf * NMMA + sub * NMMA + m * 8, d);
                    float pv = 0.0f;
#pragma unroll
                    for (int dg = 7; dg >= 0; --dg) pv = fmaf(pv, 4.0f, d[dg]);
                    acc[m] = fmaf(pv, scale[sub][m], acc[m]);
                }
            }
            tc_fence_before();     // order these tensor-memory reads before later writes of the buffer
        };
        auto wait_mma = [&](int dbuf) {
            if (!dead && !mbar_wait_async(&mma_bar[wg * 3 + dbuf], (mph >> dbuf) & 1u)) {
                dead = true;
                flags[0] = 1;
            }
            dead = __any_sync(0xffffffffu, dead);  // warp-uniform: tcgen05.st/ld are .aligned
            if (!dead) {
                mph ^= 1u << dbuf;
                tc_fence_after();
            }
        };
        // This warpgroup's quarter of row tile `ui` is summed: hand it to the finisher warp.
        auto deposit = [&](int ui) {
            const int ub = ui & 1;
            if (ui >= 2) {                         // the finisher must have consumed row tile ui - 2
                if (!dead && !mbar_wait_timed(&red_empty[ub], (eph >> ub) & 1u)) {
                    dead = true;
                    flags[0] = 1;
                }
                dead = __any_sync(0xffffffffu, dead);
                eph ^= 1u << ub;
            }
            float* rs = red + (size_t)ub * TC_WGS * M * 128;
#pragma unroll
            for (int m = 0; m < M; ++m) {
                rs[(wg * M + m) * 128 + r] = acc[m];
                acc[m] = 0.0f;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&red_full[ub]);
        };

        if (per_unit == 0) {
            // fewer k blocks than warpgroups: nothing to add, but the finisher still counts this warpgroup
            for (int ui = 0; ui < n_units; ++ui) deposit(ui);
        }
        // word index of this thread's row inside a 32-k row of its warp's ring
        const int wpos = (S == 3) ? 3 * (lane >> 2) + (lane & 3) : lane;
        for (int ti = 0; ti < n_tiles; ++ti) {
            TC_PROF(0);
            // The state of the MMA barrier of tile ti-2 is requested before the copies of tile ti+3 are issued and
            // looked at after them: a barrier poll costs a couple of hundred cycles on a busy SM even when the phase is
            // complete, and this way that latency hides behind the copy requests (measured: -5.6 % at 14336 x 4096).
            const int db_e = (dmod == 2) ? 0 : dmod + 1;
            bool early = false;
            if (PIPE && ti >= 2 && !dead) early = mbar_test(&mma_bar[wg * 3 + db_e], (mph >> db_e) & 1u);
            load_tile();                           // tile ti + 3
            const int abuf = PIPE ? (ti & 1) : 0;
            TC_PROF(1);
            TC_PROF(2);
            // Tile ti-2: its MMAs were issued two tile times ago, so this wait rarely stalls; it also frees A
            // buffer `abuf`, which those MMAs read.
            if (PIPE && ti >= 2) {
                const int db = (dmod == 2) ? 0 : dmod + 1;
                early = __all_sync(0xffffffffu, early);
                if (early) {
                    mph ^= 1u << db;
                    tc_fence_after();
                } else {
                    wait_mma(db);
                }
                if (!dead) epilogue(db, s2);
                if (last2) deposit(ui2);
            }
            TC_PROF(3);
            // the copies of tile ti (issued three steps ago) have landed; three younger groups may be in flight
            asm volatile("cp.async.wait_group 3;" ::: "memory");
            __syncwarp();
            const unsigned char* stg = ring_w + (size_t)(ti % TC_STAGES) * STAGE_B;
            float scale[NSUB][M];
#pragma unroll
            for (int sub = 0; sub < NSUB; ++sub) {
                float c = 0.0f;
                if (live_row) {
                    const unsigned char* cs = stg + 1024 + sub * 64;
                    if constexpr (IDXB == 0) {
                        c = __half2float(reinterpret_cast<const __half*>(cs)[(lane / SP) * S + s]);
                    } else {
                        const uint32_t ci = (IDXB == 1) ? (uint32_t)cs[lane / SP]
                                                        : (uint32_t)reinterpret_cast<const unsigned short*>(cs)[lane / SP];
                        c = __half2float((p.cache_in_smem ? cache_s : p.coeff)[(size_t)ci * S + s]);
                    }
                }
#pragma unroll
                for (int m = 0; m < M; ++m) scale[sub][m] = c * xsc[(m * KB + kb_c) * NSUB + sub];
            }
            if (!dead) {
                // ---- packed words of this thread's row -> 32 words of 4-bit elements {0, 0.5 | 1 | 2 | 2}
                const uint32_t* wsrc = reinterpret_cast<const uint32_t*>(stg) + wpos;
                uint32_t a[32];
#pragma unroll
                for (int kw = 0; kw < 8; ++kw) {
                    const uint32_t w = (S == 3 && !live_row) ? 0u : wsrc[kw * (WROW / 4)];
                    a[4 * kw + 0] = w & 0x11111111u;
                    a[4 * kw + 1] = w & 0x22222222u;
                    a[4 * kw + 2] = w & 0x44444444u;
                    a[4 * kw + 3] = (w >> 1) & 0x44444444u;
                }
                TC_PROF(4);
                tc_st32(a_col + lane_sel + abuf * 32, a);
                tc_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&a_ready[wg * 2 + abuf]);  // 4 warps release the issuer
            }
            TC_PROF(5);
            const bool last_of_unit = (kb_c + 1 == my_hi);
            if (PIPE) {
#pragma unroll
                for (int sub = 0; sub < NSUB; ++sub)
#pragma unroll
                    for (int m = 0; m < M; ++m) {
                        s2[sub][m] = s1[sub][m];
                        s1[sub][m] = scale[sub][m];
                    }
                last2 = last1, last1 = last_of_unit;
                ui2 = ui1, ui1 = ui_c;
            } else {
                wait_mma(0);
                if (!dead) epilogue(0, scale);
                if (last_of_unit) deposit(ui_c);
            }
            TC_PROF(6);
            TC_PROF_NEXT();
            dmod = (dmod == 2) ? 0 : dmod + 1;
            if (last_of_unit) {
                kb_c = my_lo;
                ++ui_c;
            } else {
                ++kb_c;
            }
            if ((ti & 7) == 7) {                   // notice a time-out elsewhere in the CTA now and then
                if (flags[0]) dead = true;
                dead = __any_sync(0xffffffffu, dead);
            }
        }
        if (PIPE) {                                // the last two tiles are still in the tensor pipe
            if (n_tiles >= 2) {
                const int db = (n_tiles - 2) % 3;
                wait_mma(db);
                if (!dead) epilogue(db, s2);
                if (last2) deposit(ui2);
            }
            if (n_tiles >= 1) {
                const int db = (n_tiles - 1) % 3;
                wait_mma(db);
                if (!dead) epilogue(db, s1);
                if (last1) deposit(ui1);
            }
        }
        asm volatile("cp.async.wait_all;" ::: "memory");
        if (dead) {
            flags[0] = 1;
            if (lane == 0) {
                atomicExch(p.status, 1u);
                atomicExch(p.status + 1, 0x200u + blockIdx.x);
            }
        }
    }
    // ------------------------------ teardown ------------------------------
    TC_PROF_MARK(3);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == TC_FWARP)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(*tmem_base_s),
                     "r"((uint32_t)TC_TMEM_COLS)
                     : "memory");
    TC_PROF_MARK(4);
}

// ---------------------------------------------------------------------------------------------
// host
// ---------------------------------------------------------------------------------------------
struct TcPlan {
    int KB, NT, grid, cache_in_smem, smem;
};

static int tc_plan(const PackedW& w, int M, const DeviceInfo& di, TcPlan* pl) {
    const int NSUB = 256 / w.G, TN = tc_tn(w.S);
    pl->KB = w.K / 256;
    pl->NT = w.N / TN;
    pl->grid = pl->NT < di.sm_count ? pl->NT : di.sm_count;
    const int sbytes = tc_round_up(M * pl->KB * NSUB * 4, 16);
    const int red_bytes = 2 * TC_WGS * M * 128 * 4;
    const int bbytes = pl->KB * M * 1024 + TC_BSLACK;
    const int cache_bytes = w.idx_bytes ? tc_round_up(w.C * w.S * 2, 16) : 0;
    const int base = TC_HDR + sbytes + red_bytes;
    // the codebook goes to shared memory if it still fits next to the digits
    auto total = [&](int cb) { return tc_round_up(tc_round_up(base + cb, 128) + TC_RING_BYTES, 1024) + bbytes; };
    pl->cache_in_smem = (w.idx_bytes && cache_bytes <= 65536 && total(cache_bytes) <= di.smem_optin) ? 1 : 0;
    pl->smem = total(pl->cache_in_smem ? cache_bytes : 0);
    if (pl->smem > di.smem_optin) return SBVR_ERR_UNSUPPORTED;      // K * M too large for resident digits
    return SBVR_OK;
}

bool linear_tc_supported(const PackedW& w, int M) {
    if (w.S < 2 || w.S > 4) return false;
    if (w.G != 256 && w.G != 128) return false;
    if (M < 1 || M > 4) return false;
    if (w.N % tc_tn(w.S) || w.K % 256) return false;
    if (w.idx_bytes < 0 || w.idx_bytes > 2) return false;
    if (reinterpret_cast<uintptr_t>(w.coeff) & 15) return false;
    if (reinterpret_cast<uintptr_t>(w.bvr) & 15) return false;                  // 16-byte cp.async of the packed words
    if (w.idx_bytes && (reinterpret_cast<uintptr_t>(w.idx) & 7)) return false;   // 8-byte cp.async of the indices
    if ((size_t)w.N * w.K / 32 * w.S >= ((size_t)1 << 32)) return false;      // 32-bit word offsets
    // the activation digits of the whole K stay resident in shared memory: K/256 * M KB
    const int KB = w.K / 256, NSUB = 256 / w.G;
    const int base = TC_HDR + tc_round_up(M * KB * NSUB * 4, 16) + 2 * TC_WGS * M * 128 * 4;
    if ((size_t)tc_round_up(tc_round_up(base, 128) + TC_RING_BYTES, 1024) + (size_t)KB * M * 1024 + TC_BSLACK > 227 * 1024)
        return false;
    return true;
}

template <int S, int NSUB, int M, int IDXB>
static int tc_launch_inst(const TcParams& p, int grid, int smem, cudaStream_t st) {
    static int configured_for = -1;   // device whose attribute was set last
    int dev = 0;
    SBVR_CUDA_TRY(cudaGetDevice(&dev));
    if (configured_for != dev) {
        SBVR_CUDA_TRY(cudaFuncSetAttribute(linear_tc_kernel<S, NSUB, M, IDXB>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        configured_for = dev;
    }
    SBVR_CUDA_TRY(launch_pdl(linear_tc_kernel<S, NSUB, M, IDXB>, dim3(grid), dim3(TC_THREADS), (size_t)smem, st, p));
    return SBVR_OK;
}
template <int S, int NSUB, int M>
static int tc_launch_idx(const TcParams& p, int idxb, int grid, int smem, cudaStream_t st) {
    switch (idxb) {
        case 0: return tc_launch_inst<S, NSUB, M, 0>(p, grid, smem, st);
        case 1: return tc_launch_inst<S, NSUB, M, 1>(p, grid, smem, st);
        default: return tc_launch_inst<S, NSUB, M, 2>(p, grid, smem, st);
    }
}
template <int S, int NSUB>
static int tc_launch_m(const TcParams& p, int M, int idxb, int grid, int smem, cudaStream_t st) {
    switch (M) {
        case 1: return tc_launch_idx<S, NSUB, 1>(p, idxb, grid, smem, st);
        case 2: return tc_launch_idx<S, NSUB, 2>(p, idxb, grid, smem, st);
        case 3: return tc_launch_idx<S, NSUB, 3>(p, idxb, grid, smem, st);
        default: return tc_launch_idx<S, NSUB, 4>(p, idxb, grid, smem, st);
    }
}
template <int S>
static int tc_launch_g(const TcParams& p, int G, int M, int idxb, int grid, int smem, cudaStream_t st) {
    return G == 256 ? tc_launch_m<S, 1>(p, M, idxb, grid, smem, st) : tc_launch_m<S, 2>(p, M, idxb, grid, smem, st);
}

int launch_linear_tc(const __half* x, const PackedW& w, const __half* bias, __half* y, int M, sbvr_workspace* ws,
                     cudaStream_t st, const XOp* xop) {
    if (!linear_tc_supported(w, M)) return SBVR_ERR_UNSUPPORTED;
    if (!ws) return SBVR_ERR_WORKSPACE;
    if (reinterpret_cast<uintptr_t>(x) & 15) return SBVR_ERR_ALIGN;      // x is fetched with 16-byte cp.async
    DeviceInfo di;
    int rc = device_info(ws->device, &di);
    if (rc) return rc;
    if (di.cc_major != 10) return SBVR_ERR_UNSUPPORTED;
    TcPlan pl;
    rc = tc_plan(w, M, di, &pl);
    if (rc) return rc;
    TcParams p;
    p.x = x, p.bvr = w.bvr, p.idx = w.idx, p.coeff = w.coeff, p.bias = bias, p.y = y;
    p.status = ws->status;
    p.x_op = xop ? xop->op : SBVR_XOP_NONE;
    p.delta = xop ? xop->delta : nullptr, p.norm_w = xop ? xop->norm_w : nullptr, p.h_out = xop ? xop->h_out : nullptr;
    p.eps = xop ? xop->eps : 0.0f;
    if (p.x_op == SBVR_XOP_ADD_RMSNORM) {
        if (!p.norm_w || p.h_out == x) return SBVR_ERR_BAD_ARG;
        if ((reinterpret_cast<uintptr_t>(p.delta) | reinterpret_cast<uintptr_t>(p.norm_w) |
             reinterpret_cast<uintptr_t>(p.h_out)) & 15)
            return SBVR_ERR_ALIGN;
    }
    p.N = w.N, p.K = w.K, p.KB = pl.KB, p.NT = pl.NT, p.C = w.C, p.cache_in_smem = pl.cache_in_smem;
    switch (w.S) {
        case 2: return tc_launch_g<2>(p, w.G, M, w.idx_bytes, pl.grid, pl.smem, st);
        case 3: return tc_launch_g<3>(p, w.G, M, w.idx_bytes, pl.grid, pl.smem, st);
        default: return tc_launch_g<4>(p, w.G, M, w.idx_bytes, pl.grid, pl.smem, st);
    }
}

}  // namespace sbvr

#ifdef SBVR_PROFILE
extern "C" __attribute__((visibility("default"))) int sbvr_debug_read_profile(long long* out, int n) {
    long long tmp[8 * 64 + 16];
    if (cudaMemcpyFromSymbol(tmp, sbvr::g_tc_prof, sizeof(tmp)) != cudaSuccess) return -1;
    for (int i = 0; i < n && i < 8 * 64 + 16; ++i) out[i] = tmp[i];
    return 0;
}
extern "C" __attribute__((visibility("default"))) int sbvr_debug_read_iprofile(long long* out, int n) {
    long long tmp[4 * 64];
    if (cudaMemcpyFromSymbol(tmp, sbvr::g_tc_iprof, sizeof(tmp)) != cudaSuccess) return -1;
    for (int i = 0; i < n && i < 4 * 64; ++i) out[i] = tmp[i];
    return 0;
}
#endif
