// Decode-time SBVR linear (M <= 4 activation rows): streamed weights, FP4 tensor-core dot products, balanced split.
//
//   y[n] = sum_g sum_s c[g,n,s] * ( sum_{k in g} x[k] * bit_s[n,k] )
//
// Arithmetic (shared with the older one-kernel form): the inner sum is a tcgen05.mma kind::mxf4 product of
//   A  one MMA row per (output row n, plane s); a packed word w becomes four words of eight E2M1 elements
//      (`w & 0x1111..`, `w & 0x2222..`, `w & 0x4444..`, `(w >> 1) & 0x4444..`: plane bits as {0, 0.5 | 1 | 2 | 2}),
//      written from registers straight into tensor memory (tcgen05.st), and
//   B  the activations as eight radix-4 E2M1 digits of a 16-bit block-fixed-point value per group (xdigits.cuh),
// accumulated exactly in fp32 in tensor memory; per 256 k the epilogue reads the 128 x 8 sums, forms
// sum_d 4^d D[d], multiplies by the row's fp16 coefficient and the group's step, and accumulates in fp32.
//
// What is different here, and why:
//   * The digits are produced ONCE per call by a small kernel (xquant_kernel, which also applies the op in front of
//     the linear: nothing, SiLU(gate) * up, or residual add + RMSNorm) and copied into every CTA with one bulk copy,
//     instead of every CTA spending ~2 500 cycles of its integer pipe on the same activations.
//   * Weights reach shared memory through TMA tensor copies (one 8 x TN*S-word box per 256-k step and warpgroup,
//     issued by that warpgroup's issuer warp as soon as the stage is free), not through per-thread cp.async.
//   * The hand-over compute warps -> issuer is a named hardware barrier (bar.arrive / bar.sync), not an mbarrier poll.
//   * Work is split by 256-k STEPS, not by row tiles: CTA c owns steps [c T / G, (c + 1) T / G) of the (row tile, k
//     block) list, so every SM streams the same number of bytes whatever N / 32 mod #SM is.  A CTA's warpgroups take its
//     steps round-robin.  Per row tile the warpgroups' sums meet in shared memory.  Every CTA owns NT / #CTA whole row
//     tiles; the tiles left over are cut into steps and spread over the CTAs, and finished by the first CTA of each such
//     tile, which collects the others' sums from tagged 8-byte slots in scratch in CTA order (the same bits on every
//     run).  These shared parts are processed first, so their exchange is over long before the CTA ends.
//   * Every wait is bounded; after a time-out a thread keeps the barrier protocol going but skips the work.
//
// Replaces cuda_1xtN_rd_WP8_TBW4_NS4 / cuda_row_deq_mm_T (reference sbvr/kernels/sbvr_kernel.cu:284-359, :121-191).
#include <cuda.h>

#include <mutex>

#include "common.cuh"
#include "tc_stream.cuh"
#include "xdigits.cuh"

namespace sbvr {

constexpr int TS_BSLACK = 4096;                 // MMA columns beyond M read (and ignore) what follows the digits

__host__ __device__ constexpr int ts_mpad(int M) { return M <= 2 ? 2 : 4; }
// KS = 256-k blocks per step (1 or 2).  Two blocks per step halve the per-step bookkeeping per weight byte; the sums of
// the two blocks then share one 16-column D (block 0 in columns 0-7, block 1 in 8-15, see the MMA issue), which is only
// possible for a single activation row and one group per block.
__host__ __device__ constexpr int ts_dcols(int NSUB, int M, int KS) { return KS == 2 ? 16 : NSUB * 8 * ts_mpad(M); }
__host__ __device__ constexpr int ts_wgcols(int NSUB, int M, int KS) { return 64 * KS + 2 * ts_dcols(NSUB, M, KS); }
__host__ __device__ constexpr int ts_nwg(int NSUB, int M, int KS) {
    return (TS_SF_COL / ts_wgcols(NSUB, M, KS)) > 5 ? 5 : (TS_SF_COL / ts_wgcols(NSUB, M, KS));
}
__host__ __device__ constexpr int ts_stage_bytes(int KS) { return KS * TS_STAGE_WORDS + 512; }   // + the step's coefficient data
// Warp roles: warps 0 .. NWG-1 issue (MMAs and copies), warp NWG finishes, compute warps start at the next multiple of
// four (a warp reaches the tensor-memory lanes 32 (warp % 4) ...).  The issuers have the lowest warp numbers on purpose:
// the schedulers favour older warps, and an issuer behind twenty ALU-bound compute warps waited 700-1000 cycles for
// its first issue slot after every hand-over.
__host__ __device__ constexpr int ts_cw0(int NSUB, int M, int KS) { return (ts_nwg(NSUB, M, KS) + 1 + 3) / 4 * 4; }
__host__ __device__ constexpr int ts_threads(int NSUB, int M, int KS) {
    return (ts_cw0(NSUB, M, KS) + 4 * ts_nwg(NSUB, M, KS)) * 32;
}

struct TsParams {
    const __half* x;              // activations [M][K] when the CTAs quantise them themselves (x_in_kernel), else unused
    int x_in_kernel;
    const unsigned char* xq;      // digits [KB][M][1024] then steps float [M][KB * NSUB] (written by xquant_kernel)
    const void* idx;
    const __half* coeff;
    const __half* bias;
    __half* y;                    // the pushing form of the kernel finds an sbvr_push_desc_t (device memory) here instead
    unsigned int* status;
    unsigned long long* xchg;     // [grid][2][M * TN] (fp32 sum | tag << 32) of the shared segments; all zero between calls
    int N, K, KB, NT, C, cache_in_smem, stages;
    int pre_stages;               // stages requested before the activations are fetched
    int steps_bytes;              // bytes of the steps, rounded up to a multiple of 16
    int off_red, off_cache, off_ring, off_b;      // shared-memory carve-up; at off_b: [1 KB zeros][digits][1 KB zeros][steps]
};

struct XqParams {
    const __half* x;
    unsigned char* xq;
    int K, KB, M;
    int x_op;
    const __half* delta;
    const __half* norm_w;
    __half* h_out;
    float eps;
};

// ---------------------------------------------------------------------------------------------
// activations -> digits, once per call
// ---------------------------------------------------------------------------------------------
template <int NSUB>
__global__ void __launch_bounds__(512) xquant_kernel(const XqParams p) {
    __shared__ __align__(16) unsigned char area[16][1024];
    __shared__ float ssum[16];
    pdl_launch_dependents();
    pdl_wait();                                    // the activations come from the previous kernel of the stream
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m = blockIdx.y;
    const int kb = blockIdx.x * 16 + warp;
    const int K = p.K;
    float rs = 0.0f;
    if (p.x_op == SBVR_XOP_ADD_RMSNORM) {
        // mean of (h + delta)^2 over the whole row, the sum formed in fp16 like the separate kernel does
        float sq = 0.0f;
        for (int c = threadIdx.x; c < K / 8; c += 512) {
            uint4 a = __ldg(reinterpret_cast<const uint4*>(p.x + (size_t)m * K) + c);
            __half2* ah = reinterpret_cast<__half2*>(&a);
            if (p.delta) {
                const uint4 b = __ldg(reinterpret_cast<const uint4*>(p.delta + (size_t)m * K) + c);
                const __half2* bh = reinterpret_cast<const __half2*>(&b);
#pragma unroll
                for (int e = 0; e < 4; ++e) ah[e] = __hadd2(ah[e], bh[e]);
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __half22float2(ah[e]);
                sq += f.x * f.x + f.y * f.y;
            }
        }
#pragma unroll
        for (int o = 16; o; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
        if (lane == 0) ssum[warp] = sq;
        __syncthreads();
        float tot = 0.0f;
#pragma unroll
        for (int w = 0; w < 16; ++w) tot += ssum[w];
        rs = rsqrtf(tot / (float)K + p.eps);
    }
    if (kb >= p.KB) return;
    // this warp's 256 activations: lane l brings elements 8 l .. 8 l + 7
    const size_t off = (size_t)m * K + (size_t)kb * 256 + lane * 8;
    uint4 o;
    __half2* oh = reinterpret_cast<__half2*>(&o);
    if (p.x_op == SBVR_XOP_SILU_MUL) {
        const __half* gp = p.x + (size_t)m * 2 * K + (size_t)kb * 256 + lane * 8;
        const uint4 g = __ldg(reinterpret_cast<const uint4*>(gp));
        const uint4 u = __ldg(reinterpret_cast<const uint4*>(gp + K));
        const __half2* gh = reinterpret_cast<const __half2*>(&g);
        const __half2* uh = reinterpret_cast<const __half2*>(&u);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = __half22float2(gh[e]);
            oh[e] = __hmul2(__floats2half2_rn(f.x / (1.0f + expf(-f.x)), f.y / (1.0f + expf(-f.y))), uh[e]);
        }
    } else if (p.x_op == SBVR_XOP_ADD_RMSNORM) {
        uint4 a = __ldg(reinterpret_cast<const uint4*>(p.x + off));
        __half2* ah = reinterpret_cast<__half2*>(&a);
        if (p.delta) {
            const uint4 b = __ldg(reinterpret_cast<const uint4*>(p.delta + off));
            const __half2* bh = reinterpret_cast<const __half2*>(&b);
#pragma unroll
            for (int e = 0; e < 4; ++e) ah[e] = __hadd2(ah[e], bh[e]);
        }
        if (p.h_out) *reinterpret_cast<uint4*>(p.h_out + off) = a;
        const uint4 wv = __ldg(reinterpret_cast<const uint4*>(p.norm_w + (size_t)kb * 256 + lane * 8));
        const __half2* wh = reinterpret_cast<const __half2*>(&wv);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = __half22float2(ah[e]);
            oh[e] = __hmul2(wh[e], __floats2half2_rn(f.x * rs, f.y * rs));
        }
    } else {
        o = __ldg(reinterpret_cast<const uint4*>(p.x + off));
    }
    unsigned char* ar = area[warp];
    reinterpret_cast<uint4*>(ar)[lane] = o;
    __syncwarp();
    float* steps = reinterpret_cast<float*>(p.xq + (size_t)p.KB * p.M * 1024) + ((size_t)m * p.KB + kb) * NSUB;
    xdigits_block<NSUB>(ar, steps, lane);
    __syncwarp();
    uint4* dst = reinterpret_cast<uint4*>(p.xq + ((size_t)kb * p.M + m) * 1024);
    dst[lane] = reinterpret_cast<const uint4*>(ar)[lane];
    dst[lane + 32] = reinterpret_cast<const uint4*>(ar)[lane + 32];
}


// ---------------------------------------------------------------------------------------------
// the product
// ---------------------------------------------------------------------------------------------
template <int S, int NSUB, int M, int IDXB, int KS, bool PUSH>
__global__ void __launch_bounds__(ts_threads(NSUB, M, KS), 1)
    linear_tcs_kernel(const __grid_constant__ CUtensorMap tmap, const TsParams p) {
    static_assert(KS == 1 || (KS == 2 && NSUB == 1 && M == 1), "two blocks per step: one activation row, one group per block");
    // The next kernel on the stream may be scheduled as SMs free up.  The pushing form lets it go later, from the finisher
    // warp once this kernel's own dependency wait has returned: its consumer (sbvr_ll_reduce_add_rmsnorm_f16) then knows
    // that everything in front of this kernel is complete and does not wait for this kernel to end.
    if (!PUSH) pdl_launch_dependents();
    extern __shared__ __align__(1024) unsigned char smem[];
    constexpr int SP = ts_sp(S);
    constexpr int TN = ts_tn(S);
    constexpr int MPAD = ts_mpad(M);
    constexpr int NMMA = 8 * MPAD;                 // MMA N: 8 digits per activation row
    constexpr int DCOLS = ts_dcols(NSUB, M, KS);   // columns of one D buffer
    constexpr int ACOLS = 32 * KS;                 // columns of one A buffer
    constexpr int WGCOLS = ts_wgcols(NSUB, M, KS); // A 2 x ACOLS, D 2 x DCOLS
    constexpr int NWG = ts_nwg(NSUB, M, KS);
    constexpr int CW0 = ts_cw0(NSUB, M, KS);       // first compute warp
    constexpr int NWARPS = CW0 + 4 * NWG;
    constexpr int NGRP = KS * NSUB;                // coefficient groups per step
    constexpr int STAGE_B = ts_stage_bytes(KS);
    constexpr int COEF_OFF = KS * TS_STAGE_WORDS;  // the step's coefficient data inside a stage
    constexpr int WROW = TN * S * 4;               // bytes of one 32-k row of a stage
    constexpr int CI_BYTES = (IDXB == 0) ? TN * S * 2 : TN * IDXB;     // coefficient data per group of a row tile
    constexpr uint32_t STEP_TX = KS * 8 * WROW + NGRP * CI_BYTES;
    // instruction descriptor: A, B = E2M1 (1), scales UE8M0, M = 128, N = NMMA, K-major both, K = 64
    constexpr uint32_t IDESC = (1u << 7) | (1u << 10) | ((uint32_t)(NMMA >> 3) << 17) | (1u << 23) | (8u << 24);

    uint64_t* full = reinterpret_cast<uint64_t*>(smem);                              // [NWG][TS_MAX_STAGES] stage landed
    uint64_t* mma_bar = full + NWG * TS_MAX_STAGES;                                  // [NWG][2] MMAs of a step done
    uint64_t* red_full = mma_bar + 2 * NWG;                                          // [2] sums of a segment deposited
    uint64_t* red_empty = red_full + 2;                                              // [2] ... and consumed
    uint64_t* b_ready = red_empty + 2;                                               // [1] digits copied
    uint64_t* cache_bar = b_ready + 1;                                               // [1] codebook copied
    uint64_t* tmem_ready = cache_bar + 1;                                            // [1] tensor memory allocated
    uint64_t* sf_ready = tmem_ready + 1;                                             // [1] unit scale factors written
    // [NWG][TS_MAX_STAGES] what the compute warps need to know about the step in a stage: k block | (deposit-up-to + 1) << 16
    volatile uint32_t* steptab = reinterpret_cast<volatile uint32_t*>(smem + 512);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + TS_HDR - 64);  // a wait of this CTA ran out
    uint32_t* tmem_base_s = reinterpret_cast<uint32_t*>(smem + TS_HDR - 16);

    const int KB = p.KB, N = p.N;
    float* red = reinterpret_cast<float*>(smem + p.off_red);                         // [2][NWG][M][128]
    __half* cache_s = reinterpret_cast<__half*>(smem + p.off_cache);
    unsigned char* ring = smem + p.off_ring;                                         // [NWG][stages][STAGE_B]
    unsigned char* Z0 = smem + p.off_b;                                              // 1 KB of zeros
    unsigned char* Bs = Z0 + 1024;                                                   // [KB][M][1024] digits
    unsigned char* Z1 = Bs + (size_t)KB * M * 1024;                                  // 1 KB of zeros
    float* xsc = reinterpret_cast<float*>(Z1 + 1024);                                // [M][KB * NSUB] steps
    const int KBS = KB / KS;                       // steps per row tile
    const int ST = p.stages;

    // The warp index comes from a broadcast so that the compiler knows it (and everything derived from it: roles, tensor-memory
    // addresses, barrier numbers, the operands of tcgen05.mma and of the TMA copies) to be warp-uniform and keeps it in uniform
    // registers.  Measured: an MMA whose operands are formed in divergent code costs its issuer about 200 cycles, 13-17 otherwise.
    const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
    TsSegs sg;
    sg.init(p.NT, KBS, gridDim.x, blockIdx.x);
    const int cta_steps = sg.steps;

    {
        // one barrier per thread (they are contiguous): a single thread needed ~1 800 cycles for all of them
        constexpr int NB_FULL = NWG * TS_MAX_STAGES, NB_MMA = 2 * NWG;
        const int i = threadIdx.x;
        if (i < NB_FULL + NB_MMA + 8) {
            uint32_t count = 1u;                                                     // full, mma_bar, red_empty, cache, tmem
            if (i >= NB_FULL + NB_MMA && i < NB_FULL + NB_MMA + 2) count = (uint32_t)(NWG * 4);            // red_full
            if (i == NB_FULL + NB_MMA + 4) count = (uint32_t)NWARPS + (p.x_in_kernel ? 0u : 1u);          // b_ready
            if (i == NB_FULL + NB_MMA + 7) count = 4u;                                                     // sf_ready
            mbar_init(&full[i], count);
            if (i == 0) *abort_flag = 0;
            fence_mbar_init();
        }
    }
    __syncthreads();                               // (A) barriers are initialised

    const bool bulk_cache = p.cache_in_smem && ((p.C * S * 2) % 16 == 0);

    // Every warp of the CTA calls this once, when it has nothing else to do before the digits exist.  Short activation
    // rows are quantised here, by every CTA for itself, one 256-k block per warp: cheaper than a launch of its own in
    // front of this one (a kernel boundary costs more than the ~1 us this takes).  Only the k blocks this CTA's steps
    // touch are done.  Either way the warp then reports on b_ready (its generic writes made visible to the MMA's reads).
    // `after_fetch` runs once this warp's activations have arrived (the issuers request the rest of their first stages
    // there: requested earlier, those 100+ KB per SM queue in front of the activations and delay them by over a microsecond).
    auto digits_share = [&](auto after_fetch) {
        if (warp == CW0) {                         // the two zero blocks beside the digits
            reinterpret_cast<uint4*>(Z0)[lane] = make_uint4(0u, 0u, 0u, 0u);
            reinterpret_cast<uint4*>(Z0)[lane + 32] = make_uint4(0u, 0u, 0u, 0u);
            reinterpret_cast<uint4*>(Z1)[lane] = make_uint4(0u, 0u, 0u, 0u);
            reinterpret_cast<uint4*>(Z1)[lane + 32] = make_uint4(0u, 0u, 0u, 0u);
        }
        if (p.x_in_kernel) {
            pdl_wait();                            // the activations belong to the stream's earlier kernels until now
            // all k blocks if the CTA owns a whole tile, else the blocks of its one or two shared segments
            int kb_lo = 0, nkb = KB;
            if (sg.base == 0 && sg.nrs == 1) {
                kb_lo = sg.k0(0) * KS;
                nkb = (sg.k1(0) - sg.k0(0)) * KS;
            }
            const int blk = warp;                  // M * nkb <= NWARPS: at most one block per warp
            const bool mine = blk < M * nkb;
            const int m = mine ? blk / nkb : 0, kb = mine ? kb_lo + (blk - m * nkb) : 0;
            unsigned char* area = Bs + ((size_t)kb * M + m) * 1024;
            if (mine)
                reinterpret_cast<uint4*>(area)[lane] =
                    __ldg(reinterpret_cast<const uint4*>(p.x + (size_t)m * p.K + (size_t)kb * 256) + lane);
            __syncwarp();
            after_fetch();
            if (mine) xdigits_block<NSUB>(area, xsc + ((size_t)m * KB + kb) * NSUB, lane);
        } else {
            after_fetch();
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(b_ready);
    };

    if (warp == NWG) {
        // ------------------------------ finisher warp ------------------------------
        if (bulk_cache && lane == 0) {             // codebook -> shared memory, one asynchronous copy
            mbar_arrive_expect_tx(cache_bar, (uint32_t)(p.C * S * 2));
            bulk_g2s(cache_s, p.coeff, (uint32_t)(p.C * S * 2), cache_bar);
        }
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_base_s)),
                     "r"((uint32_t)TS_TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        ts_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tmem_ready);    // whoever needs tensor memory waits for this
        pdl_wait();                                // digits, scratch and y belong to the stream's earlier kernels until now
        if (PUSH) pdl_launch_dependents();
        digits_share([] {});
        if (lane == 0 && !p.x_in_kernel) {
            const uint32_t dig = (uint32_t)(KB * M * 1024);
            mbar_arrive_expect_tx(b_ready, dig + (uint32_t)p.steps_bytes);
            bulk_g2s(Bs, p.xq, dig, b_ready);
            bulk_g2s(xsc, p.xq + dig, (uint32_t)p.steps_bytes, b_ready);
        }
        uint32_t fph = 0u;                         // bit b: phase of red_full[b]
#pragma unroll 1
        for (int q = 0; q < sg.nseg; ++q) {
            const int ub = q & 1;
            ts_wait(smem_u32(&red_full[ub]), (fph >> ub) & 1u, abort_flag, p.status, 0x330u);
            fph ^= 1u << ub;
            const int tile = sg.tile(q);
            const int n0 = tile * TN;
            const float* rs = red + (size_t)ub * NWG * M * 128;
            constexpr int PER = (M * TN + 31) / 32;
            float v[PER];
#pragma unroll
            for (int e = 0; e < PER; ++e) {
                const int i = lane + 32 * e;
                v[e] = 0.0f;
                if (i < M * TN) {
                    const int m = i / TN, nl = i % TN;
#pragma unroll
                    for (int j = 0; j < NWG; ++j)
#pragma unroll
                        for (int s = 0; s < SP; ++s) v[e] += rs[(j * M + m) * 128 + nl * SP + s];
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&red_empty[ub]);          // the warpgroups may deposit segment q + 2
            bool fin = true;                                     // this CTA writes y for the tile
            if (sg.shared(q)) {
                // A left-over tile: its steps are spread over a few CTAs.  Every CTA but the first leaves its sums in its
                // slot, each value in one 8-byte store with a tag beside it (no fence, no atomic, nothing to wait for);
                // the first CTA collects the slots in CTA order as their tags appear, clears them, and writes y.
                const int rt = tile - sg.rem_tile0;
                const int c_first = sg.cta_of((unsigned int)(rt * KBS));
                if ((int)blockIdx.x != c_first) {
                    fin = false;
                    unsigned long long* mine = p.xchg + ((size_t)blockIdx.x * 2 + sg.slot_of(blockIdx.x, rt)) * (M * TN);
#pragma unroll
                    for (int e = 0; e < PER; ++e) {
                        const int i = lane + 32 * e;
                        if (i < M * TN) {
                            const unsigned long long pk = (unsigned long long)__float_as_uint(v[e]) | (1ull << 32);
                            asm volatile("st.relaxed.gpu.global.b64 [%0], %1;" ::"l"(mine + i), "l"(pk) : "memory");
                        }
                    }
                } else {
                    // The contributors are the distinct owners of the tile's steps, in step order (not every CTA in
                    // between owns a step of the left-over list).  Their slots are polled four contributors at a time, all
                    // loads of a round in flight together: one dependent round trip per slot made a 16-way tile cost 30 us.
                    int prev = c_first, k = 1;
#pragma unroll 1
                    while (k < KBS) {
                        int ccs[4] = {0, 0, 0, 0}, n = 0;
                        while (k < KBS && n < 4) {
                            const int cc = sg.cta_of((unsigned int)(rt * KBS + k));
                            ++k;
                            if (cc != prev) {
                                prev = cc;
#pragma unroll
                                for (int j = 0; j < 4; ++j)
                                    if (j == n) ccs[j] = cc;
                                ++n;
                            }
                        }
                        unsigned long long pk[4][PER];
                        const unsigned long long* slot[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            slot[j] = p.xchg + ((size_t)ccs[j] * 2 + sg.slot_of((unsigned int)ccs[j], rt)) * (M * TN);
#pragma unroll
                            for (int e = 0; e < PER; ++e) pk[j][e] = 0ull;
                        }
                        const long long t0 = clock64();
                        for (;;) {
                            bool missing = false;
#pragma unroll
                            for (int j = 0; j < 4; ++j)
#pragma unroll
                                for (int e = 0; e < PER; ++e) {
                                    const int i = lane + 32 * e;
                                    if (j < n && i < M * TN && !(pk[j][e] >> 32))
                                        asm volatile("ld.relaxed.gpu.global.b64 %0, [%1];" : "=l"(pk[j][e]) : "l"(slot[j] + i) : "memory");
                                }
#pragma unroll
                            for (int j = 0; j < 4; ++j)
#pragma unroll
                                for (int e = 0; e < PER; ++e) {
                                    const int i = lane + 32 * e;
                                    if (j < n && i < M * TN && !(pk[j][e] >> 32)) missing = true;
                                }
                            if (!missing || *abort_flag) break;
                            if (clock64() - t0 > 2000000000LL) {              // a contributor never delivered
                                *abort_flag = 1;
                                atomicExch(p.status, 1u);
                                atomicExch(p.status + 1, 0x340u);
                                break;
                            }
                        }
#pragma unroll
                        for (int j = 0; j < 4; ++j)
#pragma unroll
                            for (int e = 0; e < PER; ++e) {
                                const int i = lane + 32 * e;
                                if (j < n && i < M * TN) {
                                    v[e] += __uint_as_float((unsigned int)pk[j][e]);
                                    asm volatile("st.relaxed.gpu.global.b64 [%0], %1;" ::"l"(slot[j] + i), "l"(0ull) : "memory");
                                }
                            }
                    }
                }
            }
            if (PUSH && fin) {
                // Tensor parallel: (two fp16 outputs | epoch << 32) to slot [epoch parity][this rank] of every rank's receive
                // area (M * TN is a multiple of 32: a warp's 32 values are valid together).
                const sbvr_push_desc_t* pd = reinterpret_cast<const sbvr_push_desc_t*>(p.y);
                const int world = pd->world;
                const unsigned int epoch = (unsigned int)(*pd->step) * (unsigned int)pd->calls_per_step + (unsigned int)pd->call_idx + 1u;
                const size_t slot = ((size_t)(pd->call_idx & 1) * world + pd->rank) * pd->rows_max;
#pragma unroll
                for (int e = 0; e < PER; ++e) {
                    const int i = lane + 32 * e;
                    if (i < M * TN) {
                        const int m = i / TN, nl = i % TN;
                        const float b = p.bias ? __half2float(p.bias[n0 + nl]) : 0.0f;
                        // four neighbouring outputs meet in one lane: two packets, one 16-byte store per peer
                        const unsigned int h = __half_as_ushort(__float2half_rn(v[e] + b));
                        const unsigned int h1 = __shfl_down_sync(0xffffffffu, h, 1);
                        const unsigned int h2 = __shfl_down_sync(0xffffffffu, h, 2);
                        const unsigned int h3 = __shfl_down_sync(0xffffffffu, h, 3);
                        if ((lane & 3) == 0) {
                            const unsigned long long pk0 = (unsigned long long)(h | (h1 << 16)) | ((unsigned long long)epoch << 32);
                            const unsigned long long pk1 = (unsigned long long)(h2 | (h3 << 16)) | ((unsigned long long)epoch << 32);
                            const size_t at = (slot + m) * (size_t)(N / 2) + (size_t)((n0 + nl) >> 1);
                            for (int r = 0; r < world; ++r)
                                asm volatile("st.volatile.global.v2.u64 [%0], {%1, %2};" ::"l"(
                                                 reinterpret_cast<unsigned long long*>(pd->peer_recv[r]) + at),
                                             "l"(pk0), "l"(pk1)
                                             : "memory");
                        }
                    }
                }
            } else if (!PUSH && fin) {
#pragma unroll
                for (int e = 0; e < PER; ++e) {
                    const int i = lane + 32 * e;
                    if (i < M * TN) {
                        const int m = i / TN, nl = i % TN;
                        const float b = p.bias ? __half2float(p.bias[n0 + nl]) : 0.0f;
                        p.y[(size_t)m * N + n0 + nl] = __float2half_rn(v[e] + b);
                    }
                }
            }
        }
        if (lane == 0) {                           // the copies this warp asked for have landed before the CTA leaves
            if (bulk_cache) ts_wait(smem_u32(cache_bar), 0u, abort_flag, p.status, 0x331u, false);
            ts_wait(smem_u32(b_ready), 0u, abort_flag, p.status, 0x332u, false);
        }
    } else if (warp < NWG) {
        // ------------------------------ issuer warps ------------------------------
        const int w = warp;
        const int n_w = (cta_steps > w) ? (cta_steps - w + NWG - 1) / NWG : 0;     // steps of this warpgroup
        const uint32_t ring_ws = smem_u32(ring + (size_t)w * ST * STAGE_B);
        const uint32_t full_ws = smem_u32(full + w * TS_MAX_STAGES);
        const unsigned char* cbytes_g = (IDXB == 0) ? reinterpret_cast<const unsigned char*>(p.coeff)
                                                    : reinterpret_cast<const unsigned char*>(p.idx);
        constexpr int CIROW_PER_N = (IDXB == 0) ? S * 2 : IDXB;                    // coefficient bytes per (group, row)
        TsCursor lc;                               // the step whose loads are issued next
        lc.start(sg, w);
        int issued = 0, lslot = 0;
        // Weights box + coefficient data of one step.  The whole (converged) warp forms the operands, one elected lane
        // issues the copies.
        auto load_step = [&]() {
            const int tile = sg.tile(lc.q), kb = lc.k * KS, q_i = lc.q;
            lc.advance(sg, NWG);
            const int q_next = lc.done(sg) ? sg.nseg : lc.q;
            // after the sums of this step have been read, the warpgroup deposits its segments up to q_next (if it moves on)
            const uint32_t entry = (uint32_t)kb | ((q_next != q_i) ? (uint32_t)(q_next + 1) << 16 : 0u);
            const uint32_t stg = ring_ws + (uint32_t)lslot * STAGE_B;
            const uint32_t bar = full_ws + (uint32_t)lslot * 8u;
            const int c0 = tile * TN * S, c1 = kb * 8;
            const unsigned char* csrc = cbytes_g + ((size_t)(kb * NSUB) * N + (size_t)tile * TN) * CIROW_PER_N;
            if (elect_one()) {
                steptab[w * TS_MAX_STAGES + lslot] = entry;      // published by the arrive below (release), read after the wait
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(STEP_TX) : "memory");
                asm volatile(
                    "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                    ::"r"(stg), "l"(reinterpret_cast<uint64_t>(&tmap)), "r"(c0), "r"(c1), "r"(bar)
                    : "memory");
#pragma unroll
                for (int sub = 0; sub < NGRP; ++sub)
                    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                                     stg + COEF_OFF + sub * CI_BYTES),
                                 "l"(csrc + (size_t)sub * N * CIROW_PER_N), "r"((uint32_t)CI_BYTES), "r"(bar)
                                 : "memory");
            }
            __syncwarp();
            ++issued;
            lslot = (lslot + 1 == ST) ? 0 : lslot + 1;
        };
        // weights do not depend on the previous kernel of the stream: the first stages are requested at once
        {
            const int first = n_w < p.pre_stages ? n_w : p.pre_stages;
#pragma unroll 1
            for (int i = 0; i < first; ++i) load_step();
        }
        digits_share([&] {
            const int first = n_w < ST ? n_w : ST;
#pragma unroll 1
            while (issued < first) load_step();
        });
        ts_wait(smem_u32(tmem_ready), 0u, abort_flag, p.status, 0x312u);                  // tensor memory is allocated
        ts_wait(smem_u32(sf_ready), 0u, abort_flag, p.status, 0x313u);                    // ... and holds the scale factors
        ts_fence_after();
        const uint32_t tbase = __shfl_sync(0xffffffffu, *tmem_base_s, 0);
        if (n_w > 0) ts_wait(smem_u32(b_ready), 0u, abort_flag, p.status, 0x310u);        // the digits are in shared memory
        const uint32_t sfa = tbase + TS_SF_COL, sfb = sfa;                    // every scale byte is 2^0
        const uint32_t a_col = tbase + w * WGCOLS;
        const uint32_t d_col = a_col + 2 * ACOLS;
        const uint32_t bs0 = smem_u32(Bs), z0 = smem_u32(Z0), z1 = smem_u32(Z1);
        const uint64_t bdesc0 = ts_bdesc(bs0);
        const uint32_t mbar0 = smem_u32(&mma_bar[w * 2]);
        TsCursor mc;                               // the step whose MMAs are issued next
        mc.start(sg, w);
#pragma unroll 1
        for (int i = 0; i < n_w; ++i) {
            const int buf = i & 1;
            const int kb = mc.k * KS;
            const uint64_t bd = bdesc0 + (uint64_t)((uint32_t)(kb * M * 1024) >> 4);
            const uint32_t dc = d_col + buf * DCOLS, ac = a_col + buf * ACOLS;
            // Two blocks per step: block 0 multiplies [digits of kb | zeros] (rows 8-15 of B point at the zero block behind
            // the digits), block 1 multiplies [zeros | digits of kb + 1] (rows 0-7 are the zero block in front): the first
            // MMA overwrites all 16 columns, the others accumulate, and the two blocks' sums end up side by side.
            const uint32_t x0 = bs0 + (uint32_t)kb * 1024u, x1 = x0 + 1024u;
            const uint64_t bd_a = ts_bdesc(x0, z1 - x0), bd_b = ts_bdesc(z0, x1 - z0);
            named_bar_sync(1 + 2 * w + buf, 160);                             // A of step i is in tensor memory
            ts_fence_after();
            if (elect_one()) {
                if constexpr (KS == 2) {
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4)
                        ts_mma(dc, ac + q4 * 8, bd_a + (uint64_t)((q4 * 256) >> 4), IDESC, sfa, sfb, (uint32_t)(q4 > 0));
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4)
                        ts_mma(dc, ac + 32 + q4 * 8, bd_b + (uint64_t)((q4 * 256) >> 4), IDESC, sfa, sfb, 1u);
                } else {
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        const int sub = (NSUB == 2) ? (q4 >> 1) : 0;
                        const uint32_t accum = (NSUB == 2) ? (uint32_t)(q4 & 1) : (uint32_t)(q4 > 0);
                        ts_mma(dc + sub * NMMA, ac + q4 * 8, bd + (uint64_t)((q4 * 256) >> 4), IDESC, sfa, sfb, accum);
                    }
                }
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mbar0 + buf * 8)
                             : "memory");
            }
            __syncwarp();
            // every compute warp has read the stage of step i: refill it
            if (issued < n_w) {
                fence_proxy_async();
                load_step();
            }
            mc.advance(sg, NWG);
        }
        if (lane == 0) {                           // no copy of this warp is in flight when the CTA leaves
            const int firstj = issued > ST ? issued - ST : 0;
#pragma unroll 1
            for (int j = firstj; j < issued; ++j)
                ts_wait(full_ws + (uint32_t)(j % ST) * 8u, (uint32_t)((j / ST) & 1), abort_flag, p.status, 0x311u, false);
        }
    } else if (warp < CW0) {
        // ------------------------------ spare warps: their share of the digits, then nothing until the teardown ----
        digits_share([] {});
    } else {
        // ------------------------------ compute warpgroups ------------------------------
        const int w = (warp - CW0) >> 2, wl = warp & 3;
        const int r = wl * 32 + lane;              // MMA row = tensor-memory lane
        const int nl = r / SP, s = r % SP;         // output row inside the tile, plane
        const bool live_row = (S != 3) || (s < S);
        const uint32_t lane_sel = (uint32_t)(wl * 32) << 16;
        const int n_w = (cta_steps > w) ? (cta_steps - w + NWG - 1) / NWG : 0;
        const unsigned char* ring_w = ring + (size_t)w * ST * STAGE_B;
        const uint32_t full_ws = smem_u32(full + w * TS_MAX_STAGES);
        const uint32_t mbar0 = smem_u32(&mma_bar[w * 2]);

        if (p.cache_in_smem && !bulk_cache) {      // codebook whose byte size is not a multiple of 16: copy by hand
            const int tid = threadIdx.x - CW0 * 32;
            for (int i = tid; i < p.C * S; i += NWG * 128) cache_s[i] = p.coeff[i];
        }
        ts_wait(smem_u32(tmem_ready), 0u, abort_flag, p.status, 0x327u);                  // tensor memory is allocated
        ts_fence_after();
        const uint32_t tbase = __shfl_sync(0xffffffffu, *tmem_base_s, 0);
        if (w == 0) {                              // unit scale factors, every byte 2^0
            uint32_t f[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) f[i] = 0x7F7F7F7Fu;
            ts_st32(tbase + lane_sel + TS_SF_COL, f);
            ts_wait_st();
            ts_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(sf_ready);  // the issuers wait for the four warps
        }
        if (p.cache_in_smem && !bulk_cache) named_bar_sync(15, NWG * 128);                // the hand-copied codebook is complete
        digits_share([] {});
        if (bulk_cache) ts_wait(smem_u32(cache_bar), 0u, abort_flag, p.status, 0x320u);
        ts_wait(smem_u32(b_ready), 0u, abort_flag, p.status, 0x321u);                      // digits and steps are in place

        const uint32_t a_addr = tbase + w * WGCOLS + lane_sel;      // this thread's lane of the A buffers
        const uint32_t d_addr = a_addr + 2 * ACOLS;
        float acc[M];
#pragma unroll
        for (int m = 0; m < M; ++m) acc[m] = 0.0f;
        uint32_t eph = 0u;                         // bit b: phase of "sums consumed" barrier b
        int qdep = 0;                              // next segment this warpgroup deposits

        // This warpgroup's sums of segment qdep -> shared memory for the finisher; segments in which it has no step
        // are deposited as zeros (the finisher counts every warp).
        auto deposit_until = [&](int qnext) {
#pragma unroll 1
            while (qdep < qnext) {
                const int ub = qdep & 1;
                if (qdep >= 2) {                   // the finisher must have consumed segment qdep - 2
                    ts_wait(smem_u32(&red_empty[ub]), (eph >> ub) & 1u, abort_flag, p.status, 0x322u);
                    eph ^= 1u << ub;
                }
                float* rsd = red + (size_t)ub * NWG * M * 128;
#pragma unroll
                for (int m = 0; m < M; ++m) {
                    rsd[(w * M + m) * 128 + r] = acc[m];
                    acc[m] = 0.0f;
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&red_full[ub]);
                ++qdep;
            }
        };
        // non-blocking look at a barrier phase (1 = complete)
        auto test = [](uint32_t bar, uint32_t parity) -> uint32_t {
            uint32_t ok;
            asm volatile(
                "{\n\t.reg .pred p;\n\t"
                "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                "selp.b32 %0, 1, 0, p;\n\t}"
                : "=r"(ok)
                : "r"(bar), "r"(parity)
                : "memory");
            return ok;
        };

        {
            TsCursor cc;
            cc.start(sg, w);
            deposit_until(cc.done(sg) ? sg.nseg : cc.q);      // segments before this warpgroup's first step
        }
        // The warpgroups would all start their first step in the same cycle: warpgroup w starts 200 w cycles late.  Measured
        // (graph over rotating weights, M = 1): 5.97 -> 5.72 us at 4096 x 4096, 5.27 -> 5.01 at 1024 x 4096, 11.91 -> 11.47 at
        // 4096 x 14336, 10.71 -> 10.66 at 14336 x 4096; 100 and 300 cycles gain about half of that, 800 cycles lose 3 %.
        if (w > 0 && n_w > 1) {
            const long long t0 = clock64();
            while (clock64() - t0 < (long long)w * 200) {
            }
        }
        float s1[NGRP][M], s2[NGRP][M];            // scales of steps i-1, i-2
        int dep1 = -1, dep2 = -1;                  // deposit up to this segment after step i-1 / i-2 (-1: nothing)
#pragma unroll
        for (int sub = 0; sub < NGRP; ++sub)
#pragma unroll
            for (int m = 0; m < M; ++m) s1[sub][m] = s2[sub][m] = 0.0f;
        const int wpos = nl * S + s;               // word of this thread's row inside a 32-k row of the stage
        int slot = 0;                              // stage of step i
        uint32_t fpar = 0u;                        // its parity
        uint32_t okf = 0u, okm = 0u;               // the phases iteration i waits for were seen complete during iteration i - 1
        // Iteration i loads, expands and hands over step i (if there is one) and reads the sums of step i - 2 (if there
        // is one): the tensor pipe works two steps behind, and the loop body exists once.  Inside an iteration the
        // independent latencies overlap: the tensor-memory read of step i - 2 is issued before the expansion of step i
        // and consumed after it, and the barriers of iteration i + 1 are looked at while the stores of step i drain.
#pragma unroll 1
        for (int i = 0; i < n_w + 2; ++i) {
            const int buf = i & 1;
            const bool front = i < n_w, back = i >= 2;
            uint32_t wv[8 * KS];
            uint32_t craw[NGRP];                   // coefficient index (or the coefficient itself, direct form)
            int kb = 0, dep_i = -1;
            const unsigned char* stg = ring_w + (size_t)slot * STAGE_B;
            if (front) {
                // ---- the step's packed words and coefficient data have landed
                if (!okf) ts_wait(full_ws + (uint32_t)slot * 8u, fpar, abort_flag, p.status, 0x323u);
                const uint32_t entry = steptab[w * TS_MAX_STAGES + slot];
                kb = (int)(entry & 0xFFFFu);
                dep_i = (int)(entry >> 16) - 1;
                const uint32_t* wsrc = reinterpret_cast<const uint32_t*>(stg) + wpos;
#pragma unroll
                for (int kw = 0; kw < 8 * KS; ++kw) wv[kw] = live_row ? wsrc[kw * (WROW / 4)] : 0u;
#pragma unroll
                for (int sub = 0; sub < NGRP; ++sub) {
                    const unsigned char* cs = stg + COEF_OFF + sub * CI_BYTES;
                    if constexpr (IDXB == 0) craw[sub] = live_row ? (uint32_t)reinterpret_cast<const unsigned short*>(cs)[nl * S + s] : 0u;
                    else if constexpr (IDXB == 1) craw[sub] = (uint32_t)cs[nl];
                    else craw[sub] = (uint32_t)reinterpret_cast<const unsigned short*>(cs)[nl];
                }
            }
            // ---- step i-2 is through the tensor pipe: its sums are requested, and A buffer i & 1 is free again
            uint32_t d[NGRP][M][8];
            if (back) {
                if (!okm) ts_wait(mbar0 + buf * 8, (uint32_t)(((i >> 1) - 1) & 1), abort_flag, p.status, 0x324u);
                ts_fence_after();
                if constexpr (KS == 2) {
                    ts_ld16_issue(d_addr + buf * DCOLS, d[0][0], d[1][0]);
                } else {
#pragma unroll
                    for (int sub = 0; sub < NSUB; ++sub)
#pragma unroll
                        for (int m = 0; m < M; ++m) ts_ld8_issue(d_addr + buf * DCOLS + sub * NMMA + m * 8, d[sub][m]);
                }
            }
            float scale[NGRP][M];
            if (front) {
#pragma unroll
                for (int sub = 0; sub < NGRP; ++sub) {
                    float c = 0.0f;
                    if constexpr (IDXB == 0) {
                        c = __half2float(__ushort_as_half((unsigned short)craw[sub]));
                    } else {
                        if (live_row) c = __half2float((p.cache_in_smem ? cache_s : p.coeff)[(size_t)craw[sub] * S + s]);
                    }
#pragma unroll
                    for (int m = 0; m < M; ++m) scale[sub][m] = c * xsc[(m * KB + kb) * NSUB + sub];
                }
                // ---- packed words of this thread's row -> 32 words of 4-bit elements {0, 0.5 | 1 | 2 | 2}
#pragma unroll
                for (int h = 0; h < 4 * KS; ++h) { // eight columns = one K = 64 MMA
                    const uint32_t w0 = wv[2 * h], w1 = wv[2 * h + 1];
                    ts_st8(a_addr + buf * ACOLS + h * 8, w0 & 0x11111111u, w0 & 0x22222222u, w0 & 0x44444444u,
                           (w0 >> 1) & 0x44444444u, w1 & 0x11111111u, w1 & 0x22222222u, w1 & 0x44444444u,
                           (w1 >> 1) & 0x44444444u);
                }
                if (++slot == ST) {
                    slot = 0;
                    fpar ^= 1u;
                }
            }
            // ---- a look at the barriers of iteration i + 1 while the stores drain
            okf = (i + 1 < n_w) ? test(full_ws + (uint32_t)slot * 8u, fpar) : 0u;
            okm = (i + 1 >= 2) ? test(mbar0 + (buf ^ 1) * 8, (uint32_t)((((i + 1) >> 1) - 1) & 1)) : 0u;
            if (back) {
                // ---- D of step i-2 -> fp32 sums
#pragma unroll
                for (int sub = 0; sub < NGRP; ++sub)
#pragma unroll
                    for (int m = 0; m < M; ++m) ts_wait_ld(d[sub][m]);
#pragma unroll
                for (int sub = 0; sub < NGRP; ++sub)
#pragma unroll
                    for (int m = 0; m < M; ++m) {
                        float pv = 0.0f;
#pragma unroll
                        for (int dg = 7; dg >= 0; --dg) pv = fmaf(pv, 4.0f, __uint_as_float(d[sub][m][dg]));
                        acc[m] = fmaf(pv, s2[sub][m], acc[m]);
                    }
                if (dep2 >= 0) deposit_until(dep2);
            }
            if (front) {
                ts_wait_st();
                ts_fence_before();
                ts_bar_arrive(1 + 2 * w + buf, 160);   // releases the issuer; also: the stage of step i has been read
            }
#pragma unroll
            for (int sub = 0; sub < NGRP; ++sub)
#pragma unroll
                for (int m = 0; m < M; ++m) {
                    s2[sub][m] = s1[sub][m];
                    if (front) s1[sub][m] = scale[sub][m];
                }
            dep2 = dep1;
            dep1 = dep_i;
        }
        deposit_until(sg.nseg);
    }
    // ------------------------------ teardown ------------------------------
    ts_fence_before();
    __syncthreads();
    ts_fence_after();
    if (warp == NWG)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(*tmem_base_s),
                     "r"((uint32_t)TS_TMEM_COLS)
                     : "memory");
}

// ---------------------------------------------------------------------------------------------
// host
// ---------------------------------------------------------------------------------------------
struct TsPlan {
    int KB, NT, KS, grid, cache_in_smem, stages, smem;
    int off_red, off_cache, off_ring, off_b;
    int steps_bytes, xq_bytes;
};

// Two 256-k blocks per step where the kernel has that form: one activation row, one group per block, an even number of blocks.
static int ts_choose_ks(const PackedW& w, int M) { return (M == 1 && w.G == 256 && (w.K / 256) % 2 == 0) ? 2 : 1; }

static int ts_plan(const PackedW& w, int M, const DeviceInfo& di, TsPlan* pl) {
    const int NSUB = 256 / w.G, TN = ts_tn(w.S);
    const int KS = ts_choose_ks(w, M);
    const int NWG = ts_nwg(NSUB, M, KS);
    pl->KS = KS;
    pl->KB = w.K / 256;
    pl->NT = w.N / TN;
    // Up to one row tile per SM: a CTA owns whole tiles and nothing is exchanged between CTAs (measured: the exchange at the
    // end of a CTA that owns no whole tile costs 2.5-4.5 us).  More tiles than SMs: every SM takes the same number of
    // steps; tiles that straddle CTAs are exchanged early, behind the whole tiles' work.
    pl->grid = pl->NT <= di.sm_count ? pl->NT : di.sm_count;
    pl->steps_bytes = ts_round_up(M * pl->KB * NSUB * 4, 16);
    pl->xq_bytes = pl->KB * M * 1024 + pl->steps_bytes;
    const int red_bytes = 2 * NWG * M * 128 * 4;
    const int cache_bytes = w.idx_bytes ? ts_round_up(w.C * w.S * 2, 16) : 0;
    const int bbytes = 1024 + pl->KB * M * 1024 + 1024 + pl->steps_bytes + TS_BSLACK;     // zeros, digits, zeros, steps, slack
    auto layout = [&](int cb, int stages) {
        pl->off_red = TS_HDR;
        pl->off_cache = pl->off_red + red_bytes;
        pl->off_ring = ts_round_up(pl->off_cache + cb, 128);
        pl->off_b = ts_round_up(pl->off_ring + NWG * stages * ts_stage_bytes(KS), 1024);
        return pl->off_b + bbytes;
    };
    // the codebook goes to shared memory if at least four stages per warpgroup still fit next to it
    pl->cache_in_smem = (w.idx_bytes && cache_bytes <= 65536 && layout(cache_bytes, 4) <= di.smem_optin) ? 1 : 0;
    const int cb = pl->cache_in_smem ? cache_bytes : 0;
    int stages = TS_MAX_STAGES;
    while (stages > 2 && layout(cb, stages) > di.smem_optin) --stages;
    pl->stages = stages;
    pl->smem = layout(cb, stages);
    if (pl->smem > di.smem_optin) return SBVR_ERR_UNSUPPORTED;      // K * M too large for resident digits
    return SBVR_OK;
}

bool linear_tcs_supported(const PackedW& w, int M) {
    if (w.S < 2 || w.S > 4) return false;
    if (w.G != 256 && w.G != 128) return false;
    if (M < 1 || M > 4) return false;
    if (w.N % ts_tn(w.S) || w.K % 256) return false;
    if (w.idx_bytes < 0 || w.idx_bytes > 2) return false;
    if (reinterpret_cast<uintptr_t>(w.coeff) & 15) return false;                 // bulk copies
    if (reinterpret_cast<uintptr_t>(w.bvr) & 15) return false;                   // tensor map base
    if (w.idx_bytes && (reinterpret_cast<uintptr_t>(w.idx) & 15)) return false;
    if ((size_t)(w.N / ts_tn(w.S)) * (size_t)(w.K / 256) >= ((size_t)1 << 24)) return false;   // 32-bit step arithmetic (steps x CTAs)
    if ((size_t)w.N * w.S >= ((size_t)1 << 31)) return false;                    // 32-bit tensor coordinates
    // the activation digits of the whole K stay resident in shared memory: K/256 * M KB, beside two stages at least
    const int NSUB = 256 / w.G, KB = w.K / 256, KS = ts_choose_ks(w, M), NWG = ts_nwg(NSUB, M, KS);
    const int need = ts_round_up(ts_round_up(TS_HDR + 2 * NWG * M * 128 * 4, 128) + NWG * 2 * ts_stage_bytes(KS), 1024) + 2048 +
                     KB * M * 1024 + ts_round_up(M * KB * NSUB * 4, 16) + TS_BSLACK;
    return need <= 227 * 1024;
}

size_t linear_tcs_workspace_bytes(const PackedW& w, int M, int sm_count) {
    (void)sm_count;
    const int NSUB = 256 / w.G, KB = w.K / 256;
    const size_t xq = (size_t)KB * M * 1024 + (size_t)ts_round_up(M * KB * NSUB * 4, 16);
    return ((xq + 255) / 256) * 256;
}

// ---- tensor maps of the packed words: uint32 [K/32 rows][N * S], box 8 KS rows x TN * S words
typedef CUresult (*TsEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int ts_tensor_map(const PackedW& w, int KS, CUtensorMap* out) {
    static std::mutex mu;
    static TsEncodeFn encode = nullptr;
    struct Entry {
        const void* bvr;
        int N, K, S, KS, valid;
        CUtensorMap map;
    };
    static Entry cache[64];
    std::lock_guard<std::mutex> lock(mu);
    if (!encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        SBVR_CUDA_TRY(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
        if (!fn || qres != cudaDriverEntryPointSuccess) return SBVR_ERR_UNSUPPORTED;
        encode = reinterpret_cast<TsEncodeFn>(fn);
    }
    const size_t h = (reinterpret_cast<uintptr_t>(w.bvr) >> 8) * 0x9E3779B97F4A7C15ull;
    Entry& e = cache[(h >> 40) & 63];
    if (!(e.valid && e.bvr == w.bvr && e.N == w.N && e.K == w.K && e.S == w.S && e.KS == KS)) {
        const cuuint64_t dims[2] = {(cuuint64_t)w.N * w.S, (cuuint64_t)w.K / 32};
        const cuuint64_t strides[1] = {(cuuint64_t)w.N * w.S * 4};
        const cuuint32_t box[2] = {(cuuint32_t)(ts_tn(w.S) * w.S), (cuuint32_t)(8 * KS)};
        const cuuint32_t estr[2] = {1u, 1u};
        const CUresult r = encode(&e.map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<uint32_t*>(w.bvr), dims, strides, box,
                                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) {
            e.valid = 0;
            g_last_cuda_error = (int)r;
            return SBVR_ERR_CUDA;
        }
        e.bvr = w.bvr, e.N = w.N, e.K = w.K, e.S = w.S, e.KS = KS, e.valid = 1;
    }
    *out = e.map;
    return SBVR_OK;
}

template <int S, int NSUB, int M, int IDXB, int KS, bool PUSH>
static int ts_launch_inst(const CUtensorMap& tm, const TsParams& p, int grid, int smem, cudaStream_t st) {
    static SmemOnce once;
    const int rc = set_max_smem_once(once, linear_tcs_kernel<S, NSUB, M, IDXB, KS, PUSH>, 227 * 1024);
    if (rc) return rc;
    SBVR_CUDA_TRY(launch_pdl(linear_tcs_kernel<S, NSUB, M, IDXB, KS, PUSH>, dim3(grid), dim3(ts_threads(NSUB, M, KS)),
                             (size_t)smem, st, tm, p));
    return SBVR_OK;
}
template <int S, int NSUB, int M, bool PUSH>
static int ts_launch_idx(const CUtensorMap& tm, const TsParams& p, int idxb, int KS, int grid, int smem, cudaStream_t st) {
    if constexpr (NSUB == 1 && M == 1) {
        if (KS == 2) {
            switch (idxb) {
                case 0: return ts_launch_inst<S, NSUB, M, 0, 2, PUSH>(tm, p, grid, smem, st);
                case 1: return ts_launch_inst<S, NSUB, M, 1, 2, PUSH>(tm, p, grid, smem, st);
                default: return ts_launch_inst<S, NSUB, M, 2, 2, PUSH>(tm, p, grid, smem, st);
            }
        }
    }
    switch (idxb) {
        case 0: return ts_launch_inst<S, NSUB, M, 0, 1, PUSH>(tm, p, grid, smem, st);
        case 1: return ts_launch_inst<S, NSUB, M, 1, 1, PUSH>(tm, p, grid, smem, st);
        default: return ts_launch_inst<S, NSUB, M, 2, 1, PUSH>(tm, p, grid, smem, st);
    }
}
template <int S, int NSUB, bool PUSH>
static int ts_launch_m(const CUtensorMap& tm, const TsParams& p, int M, int idxb, int KS, int grid, int smem,
                       cudaStream_t st) {
    switch (M) {
        case 1: return ts_launch_idx<S, NSUB, 1, PUSH>(tm, p, idxb, KS, grid, smem, st);
        case 2: return ts_launch_idx<S, NSUB, 2, PUSH>(tm, p, idxb, KS, grid, smem, st);
        case 3: return ts_launch_idx<S, NSUB, 3, PUSH>(tm, p, idxb, KS, grid, smem, st);
        default: return ts_launch_idx<S, NSUB, 4, PUSH>(tm, p, idxb, KS, grid, smem, st);
    }
}
// The pushing form (tensor-parallel decode) is a kernel of its own, so that the plain one carries none of its code; it is
// built for group length 256 only.
template <int S>
static int ts_launch_g(const CUtensorMap& tm, const TsParams& p, bool push, int G, int M, int idxb, int KS, int grid, int smem,
                       cudaStream_t st) {
    if (push) {
        if (G != 256) return SBVR_ERR_UNSUPPORTED;
        return ts_launch_m<S, 1, true>(tm, p, M, idxb, KS, grid, smem, st);
    }
    return G == 256 ? ts_launch_m<S, 1, false>(tm, p, M, idxb, KS, grid, smem, st)
                    : ts_launch_m<S, 2, false>(tm, p, M, idxb, KS, grid, smem, st);
}

// `scratch` (256-byte aligned, linear_tcs_workspace_bytes long), `status` and `xchg` (SBVR_WS_XCHG_BYTES of exchange slots,
// all zero between calls: the kernel leaves them zero) are the caller's: the workspace form and the no-allocation form
// carve them differently.
int launch_linear_tcs(const __half* x, const PackedW& w, const __half* bias, __half* y, int M, int device,
                      unsigned int* status, unsigned long long* xchg, char* scratch, size_t scratch_bytes, cudaStream_t st,
                      const XOp* xop, const sbvr_push_desc_t* push) {
    if (!linear_tcs_supported(w, M)) return SBVR_ERR_UNSUPPORTED;
    if (!status || !xchg || !scratch) return SBVR_ERR_WORKSPACE;
    if (reinterpret_cast<uintptr_t>(x) & 15) return SBVR_ERR_ALIGN;      // x is fetched 16 bytes at a time
    if (reinterpret_cast<uintptr_t>(scratch) & 255) return SBVR_ERR_ALIGN;
    DeviceInfo di;
    int rc = device_info(device, &di);
    if (rc) return rc;
    if (di.cc_major != 10) return SBVR_ERR_UNSUPPORTED;
    TsPlan pl;
    rc = ts_plan(w, M, di, &pl);
    if (rc) return rc;
    if (linear_tcs_workspace_bytes(w, M, di.sm_count) > scratch_bytes) return SBVR_ERR_WORKSPACE;
    if ((size_t)pl.grid * 2 * M * ts_tn(w.S) * 8 > SBVR_WS_XCHG_BYTES) return SBVR_ERR_UNSUPPORTED;
    XqParams xp;
    xp.x = x, xp.xq = reinterpret_cast<unsigned char*>(scratch), xp.K = w.K, xp.KB = pl.KB, xp.M = M;
    xp.x_op = xop ? xop->op : SBVR_XOP_NONE;
    xp.delta = xop ? xop->delta : nullptr, xp.norm_w = xop ? xop->norm_w : nullptr, xp.h_out = xop ? xop->h_out : nullptr;
    xp.eps = xop ? xop->eps : 0.0f;
    if (xp.x_op == SBVR_XOP_ADD_RMSNORM) {
        // h_out is written while other blocks still read x and delta for the row's mean square
        if (!xp.norm_w) return SBVR_ERR_BAD_ARG;
        if (xp.h_out) {
            const uintptr_t n = (uintptr_t)M * w.K * 2, ho = reinterpret_cast<uintptr_t>(xp.h_out);
            auto overlaps = [&](const void* q) {
                const uintptr_t a = reinterpret_cast<uintptr_t>(q);
                return q && ho < a + n && a < ho + n;
            };
            if (overlaps(x) || overlaps(xp.delta)) return SBVR_ERR_BAD_ARG;
        }
        if ((reinterpret_cast<uintptr_t>(xp.delta) | reinterpret_cast<uintptr_t>(xp.norm_w) |
             reinterpret_cast<uintptr_t>(xp.h_out)) & 15)
            return SBVR_ERR_ALIGN;
    }
    CUtensorMap tm;
    rc = ts_tensor_map(w, pl.KS, &tm);
    if (rc) return rc;
    // one block per compute warp at most: the CTAs quantise for themselves; longer rows (and rows with an op in front)
    // get the separate kernel
    const int NWG = ts_nwg(256 / w.G, M, pl.KS);
    const bool in_kernel = (xp.x_op == SBVR_XOP_NONE) && (M * pl.KB <= ts_cw0(256 / w.G, M, pl.KS) + 4 * NWG);
    // SBVR_XOP_DIGITS: the digits are in the scratch already (written by the reduce kernel in front of this call)
    if (xp.x_op == SBVR_XOP_DIGITS && w.G != 256) return SBVR_ERR_UNSUPPORTED;
    if (!in_kernel && xp.x_op != SBVR_XOP_DIGITS) {
        const dim3 qgrid((pl.KB + 15) / 16, M);
        if (w.G == 256) SBVR_CUDA_TRY(launch_pdl(xquant_kernel<1>, qgrid, dim3(512), 0, st, xp));
        else SBVR_CUDA_TRY(launch_pdl(xquant_kernel<2>, qgrid, dim3(512), 0, st, xp));
    }
    TsParams p;
    p.x = x, p.x_in_kernel = in_kernel ? 1 : 0;
    p.xq = xp.xq, p.idx = w.idx, p.coeff = w.coeff, p.bias = bias, p.y = y;
    p.status = status, p.xchg = xchg;
    p.N = w.N, p.K = w.K, p.KB = pl.KB, p.NT = pl.NT, p.C = w.C, p.cache_in_smem = pl.cache_in_smem, p.stages = pl.stages;
    p.steps_bytes = pl.steps_bytes;
    p.pre_stages = pl.stages < 3 ? pl.stages : 3;
    p.off_red = pl.off_red, p.off_cache = pl.off_cache, p.off_ring = pl.off_ring, p.off_b = pl.off_b;
    if (push) {
        if (w.N & 3) return SBVR_ERR_SHAPE;
        p.y = reinterpret_cast<__half*>(const_cast<sbvr_push_desc_t*>(push));
    }
    switch (w.S) {
        case 2: return ts_launch_g<2>(tm, p, push != nullptr, w.G, M, w.idx_bytes, pl.KS, pl.grid, pl.smem, st);
        case 3: return ts_launch_g<3>(tm, p, push != nullptr, w.G, M, w.idx_bytes, pl.KS, pl.grid, pl.smem, st);
        default: return ts_launch_g<4>(tm, p, push != nullptr, w.G, M, w.idx_bytes, pl.KS, pl.grid, pl.smem, st);
    }
}

}  // namespace sbvr
