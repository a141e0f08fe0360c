// SBVR linear for small activation batches (2 .. 32 rows): FP4 tensor-core dot products of plane bits with activation
// digits, like the decode GEMV, but with the digits' weights and the activations' block scale carried by the MMA's own
// block scale factors, so that the tensor pipe sums over digits and nothing but one multiply-add per (row, plane,
// activation row, 256-k block) is left for the CUDA cores.
//
//   y[m, n] = sum_g sum_s c[g, n, s] * sum_{k in g} x[m, k] * bit_s[n, k]
//
// Operands of tcgen05.mma kind::mxf4.block_scale.scale_vec::2X (K = 64 per instruction, fp32 accumulation in tensor memory):
//
//  A (tensor memory)  128 lanes = TN output rows x their planes; a lane's 256 plane bits of a k block are expanded to 4-bit
//      E2M1 codes by six integer instructions per packed word (`(w << 1) & 0x2222.., w & 0x2222.., w & 0x4444..,
//      (w >> 1) & 0x4444..`): a set bit becomes 1, 1, 2, 2 for k % 4 = 0 .. 3.
//  B (shared memory)  x is quantised per (activation row, 256-k block) to 16-bit block fixed point q = round(x / step),
//      step a power of two, and q + 0x24924 is cut into six 3-bit fields t, digit = t - 4 in {-4 .. 3}, so that
//      q = sum_d 8^d digit_d.  Every digit is an exact E2M1 value (halved where the plane bit counts 2).  One MMA
//      multiplies the plane bits by ONE digit of all activation rows (M > 16: N = 32 rows) or by two digits of up to
//      16 rows (N = 2 x 16), with the scale factor 8^d * step of that digit and row as the B block scale (UE8M0, a power
//      of two): the accumulator column of an activation row then holds sum_k bit * x^ directly, whatever the digit.
//      M <= 16 leaves two columns per activation row (even and odd digits), added on the way out.
//
// Structure: persistent CTAs; NWG compute warpgroups work on NWG neighbouring row tiles in lockstep through the k blocks, so
// that one copy of a k block's digits (12 or 24 KB, fetched by a producer warp with one bulk copy per block from the
// blob the quantiser kernel wrote) serves all of them.  Per warpgroup an issuer warp streams the packed words (TMA) and
// issues the MMAs; the compute warps expand step i, write its B scale factors to tensor memory, and read the sums of
// step i - 2.  Work is split by (tile group, k block) steps over the CTAs like the decode GEMV's; a tile group whose k
// blocks are spread over several CTAs is finished by the first of them, after its own steps, from fp32 partial sums in
// scratch, summed in CTA order (the same bits on every run) once per-slot arrival counters (zero between calls) show
// them complete.  Every wait is bounded.
//
// Measured (B200, rotating weights larger than L2, CUDA graph, quantiser kernel included): 14336 x 4096, S = 4:
// 24 us at M = 2, 26.3 us at M = 16, 34.6 us at M = 32 (the fp16 GEMM with in-kernel dequantisation: 34-35 us); a step of
// three tiles takes about 1 500 cycles, bound by the latency chain of a compute warp (barrier, tensor-memory load,
// expansion, store drain), not by the tensor pipe (12 or 24 MMAs of 17 cycles) nor by memory.
//
// Replaces the M > 1 use of `_sbvr_row_deq_mm_T` (reference sbvr/kernels/sbvr_kernel.cu:121-191) for 2 .. 32 rows.
#include <cuda.h>

#include <mutex>

#include "common.cuh"
#include "tc_stream.cuh"

namespace sbvr {


constexpr int TB_SF_BYTES = 512;                // 32 rows x 16 B of B scale factors (and the poison mask) per k block
constexpr int TB_CW0 = 4;                       // first compute warp
constexpr int TB_ASTAGE = TS_STAGE_WORDS + 512; // packed words of a 256-k block of one tile + its coefficient data
constexpr int TB_MAX_BSTAGES = 8;
constexpr int TB_HDR = 2048;                    // barriers, the contributor list of a shared tile group, flags, tensor-memory base
__host__ __device__ constexpr int tb_nwg(int NSUB) { return NSUB == 2 ? 2 : 3; }
__host__ __device__ constexpr int tb_threads(int NSUB) { return (TB_CW0 + 4 * tb_nwg(NSUB)) * 32; }
__host__ __device__ constexpr int tb_bstage(int NJ) { return NJ * 4096 + TB_SF_BYTES; }
// Tensor-memory columns of a warpgroup: A x 2 (32 each), B scale factors x 2 (three 4-column blocks each, padded to 16: the
// scale-factor address of an MMA designates a 4-column block and must be aligned to one), D x 2
__host__ __device__ constexpr int tb_wgcols(int NSUB) { return 64 + 32 + 2 * NSUB * 32; }

struct TbParams {
    const unsigned char* xb;      // [KB][NJ * 4096 digits + 512 scale factors] written by xq8_kernel
    const void* idx;
    const __half* coeff;
    const __half* bias;
    __half* y;
    unsigned int* status;
    unsigned int* flags;          // [grid][2] arrival counters of the partial sums; all zero between calls
    float* part;                  // [grid][2][NWG][MP][TN] partial sums of tile groups shared between CTAs
    int M, N, K, KB, NT, NTG, C, cache_in_smem, a_stages, b_stages;
    int off_cache, off_aring, off_bring;
};

// ---------------------------------------------------------------------------------------------
// activations -> digit blob, once per call
// ---------------------------------------------------------------------------------------------
// One block per 256-k block, one warp per (padded) activation row.  Lane (kw, j) owns the eight elements
// k = 32 kw + j + 4 e, which are one 32-bit word (nibble e) of every digit: the K order in which the weight expansion
// leaves the plane bits.  Blob of a k block: [MMA j (NJ)][row group (4)][kw (8)][row (8)][16 B], then 32 rows x 16 B:
// words 0 .. 2 hold the scale bytes of MMA 2 i (bytes 0, 1) and 2 i + 1 (bytes 2, 3) for that B row, word 3 the mask of
// activation rows of this block that hold a non-finite value.
template <int NJ>
__global__ void __launch_bounds__(NJ == 3 ? 512 : 1024) xq8_kernel(const __half* __restrict__ x, unsigned char* __restrict__ xb,
                                                                     int M, int K) {
    __shared__ __align__(16) unsigned char sf[32][16];
    __shared__ unsigned int poison_s;
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kb = blockIdx.x;
    if (threadIdx.x < 128) reinterpret_cast<uint32_t*>(sf)[threadIdx.x] = ((threadIdx.x & 3) == 3) ? 0u : 0x7F7F7F7Fu;
    if (threadIdx.x == 0) poison_s = 0u;
    __syncthreads();
    pdl_wait();                                    // the activations come from the previous kernel of the stream
    const int m = warp;
    const int kw = lane >> 2, j = lane & 3;
    uint32_t words[6] = {0u, 0u, 0u, 0u, 0u, 0u};
    int ex = 14;
    if (m < M) {
        const __half* xp = x + (size_t)m * K + (size_t)kb * 256 + 32 * kw + j;
        float v[8];
        float a = 0.0f;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            v[e] = __half2float(xp[4 * e]);
            float av = fabsf(v[e]);
            if (!(av == av)) av = __int_as_float(0x7f800000);     // NaN counts as infinity
            a = fmaxf(a, av);
        }
#pragma unroll
        for (int o = 16; o; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
        float inv = 0.0f;
        bool poison = false;
        if (a >= __int_as_float(0x7f800000)) {
            poison = true;
            if (lane == 0) atomicOr(&poison_s, 1u << m);
        } else if (a > 0.0f) {
            ex = (int)((__float_as_uint(a) >> 23) & 0xFF) - 127;              // a = 1.f * 2^ex, ex in [-24, 15]
            inv = __uint_as_float((uint32_t)(14 - ex + 127) << 23);
        }
        // E2M1 codes of digit t - 4 (t = 0 .. 7), one nibble each: the value itself for j = 0, 1, half of it for j = 2, 3
        const uint32_t lut = (j < 2) ? 0x5420ACDEu : 0x32109ABCu;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const int q = poison ? 0 : __float2int_rn(v[e] * inv);            // |q| <= 2^15
            const uint32_t u = (uint32_t)(q + 0x24924);
#pragma unroll
            for (int d = 0; d < 6; ++d) {
                const uint32_t t = (u >> (3 * d)) & 7u;
                words[d] |= ((lut >> (4u * t)) & 0xFu) << (4 * e);
            }
        }
    }
    unsigned char* blob = xb + (size_t)kb * tb_bstage(NJ);
#pragma unroll
    for (int d = 0; d < 6; ++d) {
        const int jm = (NJ == 6) ? d : (d >> 1);
        const int row = (NJ == 6) ? m : ((d & 1) * 16 + m);
        *reinterpret_cast<uint32_t*>(blob + jm * 4096 + (row >> 3) * 1024 + kw * 128 + (row & 7) * 16 + j * 4) = words[d];
        if (m < M && lane == 0) {
            const unsigned char sb = (unsigned char)(127 + 3 * d + ex - 14);
            unsigned char* dst = &sf[row][(jm >> 1) * 4 + (jm & 1) * 2];
            dst[0] = sb;
            dst[1] = sb;
        }
    }
    __syncthreads();
    if (threadIdx.x < 32) {
        uint4 v = reinterpret_cast<const uint4*>(sf)[threadIdx.x];
        v.w = poison_s;
        reinterpret_cast<uint4*>(blob + NJ * 4096)[threadIdx.x] = v;
    }
}

// ---------------------------------------------------------------------------------------------
// the product
// ---------------------------------------------------------------------------------------------
template <int S, int NSUB, int NJ, int IDXB>
__global__ void __launch_bounds__(tb_threads(NSUB), 1)
    linear_tcb_kernel(const __grid_constant__ CUtensorMap tmap, const TbParams p) {
    pdl_launch_dependents();
    extern __shared__ __align__(1024) unsigned char smem[];
    constexpr int SP = ts_sp(S);
    constexpr int TN = ts_tn(S);
    constexpr int MP = (NJ == 3) ? 16 : 32;        // activation rows the accumulators cover
    constexpr int NV = MP / SP;                    // ... and how many of them one thread finishes
    constexpr int NWG = tb_nwg(NSUB);
    constexpr int CW0 = TB_CW0;
    constexpr int WGCOLS = tb_wgcols(NSUB);
    constexpr int DCOLS = NSUB * 32;
    constexpr int BSTAGE = tb_bstage(NJ);
    constexpr int WROW = TN * S * 4;               // bytes of one 32-k row of a stage
    constexpr int CI_BYTES = (IDXB == 0) ? TN * S * 2 : TN * IDXB;
    constexpr uint32_t A_TX = 8 * WROW + NSUB * CI_BYTES;
    constexpr int COEF_OFF = TS_STAGE_WORDS;
    // instruction descriptor: A, B = E2M1, scales UE8M0, M = 128, N = 32, K-major both; the scale-factor byte pair is added per MMA
    constexpr uint32_t IDESC = (1u << 7) | (1u << 10) | ((uint32_t)(32 >> 3) << 17) | (1u << 23) | (8u << 24);

    uint64_t* a_full = reinterpret_cast<uint64_t*>(smem);                            // [NWG][TS_MAX_STAGES]
    uint64_t* mma_bar = a_full + NWG * TS_MAX_STAGES;                                // [NWG][2]
    uint64_t* b_full = mma_bar + 2 * NWG;                                            // [TB_MAX_BSTAGES]
    // [NWG][TB_MAX_BSTAGES]: one barrier per warpgroup and stage, so that every barrier has a single arriving commit (three
    // issuers' tcgen05.commit on one barrier of count three is the one construct this kernel did not share with the decode GEMV)
    uint64_t* b_empty = b_full + TB_MAX_BSTAGES;
    uint64_t* cache_bar = b_empty + NWG * TB_MAX_BSTAGES;
    uint64_t* tmem_ready = cache_bar + 1;
    uint64_t* sf_ready = tmem_ready + 1;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + TB_HDR - 64);
    volatile int* done_cnt = reinterpret_cast<volatile int*>(smem + TB_HDR - 48);     // [2] compute warps done with a shared tile group
    volatile int* ctab = reinterpret_cast<volatile int*>(smem + 1024);                 // [128] who contributed to a shared tile group
    uint32_t* tmem_base_s = reinterpret_cast<uint32_t*>(smem + TB_HDR - 16);

    const int KB = p.KB, N = p.N, M = p.M;
    __half* cache_s = reinterpret_cast<__half*>(smem + p.off_cache);
    unsigned char* aring = smem + p.off_aring;                                       // [NWG][a_stages][TB_ASTAGE]
    unsigned char* bring = smem + p.off_bring;                                       // [b_stages][BSTAGE]
    const int AST = p.a_stages, BST = p.b_stages;

    const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
    TsSegs sg;
    sg.init(p.NTG, KB, gridDim.x, blockIdx.x);
    const int n_steps = sg.steps;

    {
        constexpr int NB_A = NWG * TS_MAX_STAGES, NB_M = 2 * NWG;
        constexpr int NB = NB_A + NB_M + (1 + NWG) * TB_MAX_BSTAGES + 3;
        const int i = threadIdx.x;
        if (i < NB) {
            uint32_t count = 1u;
            if (i == NB - 1) count = 4u;                                                                           // sf_ready
            mbar_init(&a_full[i], count);
            if (i == 0) {
                *abort_flag = 0;
                done_cnt[0] = 0;
                done_cnt[1] = 0;
            }
            fence_mbar_init();
        }
    }
    __syncthreads();

    const bool bulk_cache = p.cache_in_smem && ((p.C * S * 2) % 16 == 0);

    if (warp == NWG) {
        // ------------------------------ producer of the activation digits ------------------------------
        if (bulk_cache && lane == 0) {
            mbar_arrive_expect_tx(cache_bar, (uint32_t)(p.C * S * 2));
            bulk_g2s(cache_s, p.coeff, (uint32_t)(p.C * S * 2), cache_bar);
        }
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_base_s)),
                     "r"((uint32_t)TS_TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        ts_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tmem_ready);
        pdl_wait();                                // the blob is written by the kernel in front of this one
        TsCursor pc;
        pc.start(sg, 0);
#pragma unroll 1
        for (int i = 0; i < n_steps; ++i) {
            const int slot = i % BST;
            // the slot's previous occupant (step i - BST) has been multiplied by every warpgroup
            if (i >= BST) {
#pragma unroll
                for (int wq = 0; wq < NWG; ++wq)
                    ts_wait(smem_u32(&b_empty[wq * TB_MAX_BSTAGES + slot]), (uint32_t)((i / BST - 1) & 1), abort_flag, p.status, 0x410u);
            }
            if (lane == 0) {
                mbar_arrive_expect_tx(&b_full[slot], (uint32_t)BSTAGE);
                bulk_g2s(bring + (size_t)slot * BSTAGE, p.xb + (size_t)pc.k * BSTAGE, (uint32_t)BSTAGE, &b_full[slot]);
            }
            __syncwarp();
            pc.advance(sg, 1);
        }
        if (lane == 0) {                           // no copy of this warp is in flight when the CTA leaves
            if (bulk_cache) ts_wait(smem_u32(cache_bar), 0u, abort_flag, p.status, 0x411u, false);
            const int firstj = n_steps > BST ? n_steps - BST : 0;
#pragma unroll 1
            for (int jx = firstj; jx < n_steps; ++jx)
                ts_wait(smem_u32(&b_full[jx % BST]), (uint32_t)((jx / BST) & 1), abort_flag, p.status, 0x412u, false);
        }
    } else if (warp < NWG) {
        // ------------------------------ issuer warps ------------------------------
        const int w = warp;
        const uint32_t ring_ws = smem_u32(aring + (size_t)w * AST * TB_ASTAGE);
        const uint32_t full_ws = smem_u32(a_full + w * TS_MAX_STAGES);
        const unsigned char* cbytes_g = (IDXB == 0) ? reinterpret_cast<const unsigned char*>(p.coeff)
                                                    : reinterpret_cast<const unsigned char*>(p.idx);
        constexpr int CIROW_PER_N = (IDXB == 0) ? S * 2 : IDXB;
        TsCursor lc;
        lc.start(sg, 0);
        int issued = 0, lslot = 0;
        auto load_step = [&]() {
            int tile = sg.tile(lc.q) * NWG + w;    // a warpgroup without a tile of its own repeats the last one and drops the result
            tile = tile < p.NT ? tile : p.NT - 1;
            const int kb = lc.k;
            lc.advance(sg, 1);
            const uint32_t stg = ring_ws + (uint32_t)lslot * TB_ASTAGE;
            const uint32_t bar = full_ws + (uint32_t)lslot * 8u;
            const int c0 = tile * TN * S, c1 = kb * 8;
            const unsigned char* csrc = cbytes_g + ((size_t)(kb * NSUB) * N + (size_t)tile * TN) * CIROW_PER_N;
            if (elect_one()) {
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(A_TX) : "memory");
                asm volatile(
                    "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                    ::"r"(stg), "l"(reinterpret_cast<uint64_t>(&tmap)), "r"(c0), "r"(c1), "r"(bar)
                    : "memory");
#pragma unroll
                for (int sub = 0; sub < NSUB; ++sub)
                    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                                     stg + COEF_OFF + sub * CI_BYTES),
                                 "l"(csrc + (size_t)sub * N * CIROW_PER_N), "r"((uint32_t)CI_BYTES), "r"(bar)
                                 : "memory");
            }
            __syncwarp();
            ++issued;
            lslot = (lslot + 1 == AST) ? 0 : lslot + 1;
        };
        {
            const int first = n_steps < AST ? n_steps : AST;       // the weights do not depend on the kernel in front
#pragma unroll 1
            for (int i = 0; i < first; ++i) load_step();
        }
        ts_wait(smem_u32(tmem_ready), 0u, abort_flag, p.status, 0x420u);
        ts_wait(smem_u32(sf_ready), 0u, abort_flag, p.status, 0x421u);
        ts_fence_after();
        const uint32_t tbase = __shfl_sync(0xffffffffu, *tmem_base_s, 0);
        const uint32_t sfa = tbase + TS_SF_COL;
        const uint32_t a_col = tbase + w * WGCOLS;
        const uint32_t sfb_col = a_col + 64;
        const uint32_t d_col = a_col + 96;
        const uint32_t bring_s = smem_u32(bring);
        const uint32_t mbar0 = smem_u32(&mma_bar[w * 2]);
        int bslot = 0;
        uint32_t bpar = 0u;
#pragma unroll 1
        for (int i = 0; i < n_steps; ++i) {
            const int buf = i & 1;
            const uint64_t bd = ts_bdesc(bring_s + (uint32_t)bslot * BSTAGE);
            const uint32_t dc = d_col + buf * DCOLS, ac = a_col + buf * 32, sc = sfb_col + buf * 16;
            named_bar_sync(1 + 2 * w + buf, 160);                             // A and the B scales of step i are in tensor memory
            ts_wait(smem_u32(&b_full[bslot]), bpar, abort_flag, p.status, 0x422u);   // ... and its digits in shared memory
            ts_fence_after();
            if (elect_one()) {
#pragma unroll
                for (int c = 0; c < 4; ++c)
#pragma unroll
                    for (int jm = 0; jm < NJ; ++jm) {
                        const int sub = (NSUB == 2) ? (c >> 1) : 0;
                        const bool first = (jm == 0) && ((NSUB == 2) ? ((c & 1) == 0) : (c == 0));
                        const uint32_t sfid = (uint32_t)((jm & 1) * 2);
                        ts_mma(dc + sub * 32, ac + c * 8, bd + (uint64_t)((jm * 4096 + c * 256) >> 4),
                               IDESC | (sfid << 4) | (sfid << 29), sfa, sc + 4 * (jm >> 1), (uint32_t)!first);
                    }
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mbar0 + buf * 8)
                             : "memory");
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                                 smem_u32(&b_empty[w * TB_MAX_BSTAGES + bslot]))
                             : "memory");
            }
            __syncwarp();
            if (issued < n_steps) {                // every compute warp has read the stage of step i: refill it
                fence_proxy_async();
                load_step();
            }
            if (++bslot == BST) {
                bslot = 0;
                bpar ^= 1u;
            }
        }
        if (lane == 0) {
            const int firstj = issued > AST ? issued - AST : 0;
#pragma unroll 1
            for (int jx = firstj; jx < issued; ++jx)
                ts_wait(full_ws + (uint32_t)(jx % AST) * 8u, (uint32_t)((jx / AST) & 1), abort_flag, p.status, 0x423u, false);
        }
    } else if (warp < CW0) {
        // spare warp (two warpgroups): nothing until the teardown
    } else {
        // ------------------------------ compute warpgroups ------------------------------
        const int w = (warp - CW0) >> 2, wl = warp & 3;
        const int r = wl * 32 + lane;              // MMA row = tensor-memory lane
        const int nl = r / SP, s = r % SP;
        const bool live_row = (S != 3) || (s < S);
        const uint32_t lane_sel = (uint32_t)(wl * 32) << 16;
        const unsigned char* ring_w = aring + (size_t)w * AST * TB_ASTAGE;
        const uint32_t full_ws = smem_u32(a_full + w * TS_MAX_STAGES);
        const uint32_t mbar0 = smem_u32(&mma_bar[w * 2]);

        if (p.cache_in_smem && !bulk_cache) {
            const int tid = threadIdx.x - CW0 * 32;
            for (int i = tid; i < p.C * S; i += NWG * 128) cache_s[i] = p.coeff[i];
        }
        ts_wait(smem_u32(tmem_ready), 0u, abort_flag, p.status, 0x430u);
        ts_fence_after();
        const uint32_t tbase = __shfl_sync(0xffffffffu, *tmem_base_s, 0);
        if (w == 0) {                              // unit scale factors for A, every byte 2^0
            uint32_t f[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) f[i] = 0x7F7F7F7Fu;
            ts_st32(tbase + lane_sel + TS_SF_COL, f);
            ts_wait_st();
            ts_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(sf_ready);
        }
        if (p.cache_in_smem && !bulk_cache) named_bar_sync(15, NWG * 128);
        if (bulk_cache) ts_wait(smem_u32(cache_bar), 0u, abort_flag, p.status, 0x431u);

        const uint32_t a_addr = tbase + w * WGCOLS + lane_sel;
        const uint32_t sfb_addr = a_addr + 64;
        const uint32_t d_addr = a_addr + 96;
        float acc[MP];
#pragma unroll
        for (int m = 0; m < MP; ++m) acc[m] = 0.0f;
        uint32_t pm = 0u;                          // activation rows seen with a non-finite value
        int shq0 = -1, shq1 = -1;                  // this CTA's shared segments it has to finish at the end
        const int wpos = nl * S + s;

        // Sums of segment q (this warpgroup's tile of the group): planes added by shuffles, every thread of a row's
        // planes keeps the activation rows m = s (mod SP).
        auto finish = [&](int q) {
            float outv[NV];
#pragma unroll
            for (int m = 0; m < MP; ++m) {
                float v = acc[m];
                acc[m] = 0.0f;
                v += __shfl_xor_sync(0xffffffffu, v, 1);
                if (SP == 4) v += __shfl_xor_sync(0xffffffffu, v, 2);
                if ((pm >> m) & 1u) v = __int_as_float(0x7fc00000);
                if ((m % SP) == s) outv[m / SP] = v;
            }
            const int tile = sg.tile(q) * NWG + w;
            const bool valid = tile < p.NT;
            if (!sg.shared(q)) {
                if (valid) {
                    const int n = tile * TN + nl;
                    const float b = p.bias ? __half2float(p.bias[n]) : 0.0f;
#pragma unroll
                    for (int e = 0; e < NV; ++e) {
                        const int m = e * SP + s;
                        if (m < M) p.y[(size_t)m * N + n] = __float2half_rn(outv[e] + b);
                    }
                }
            } else {
                const int rt = sg.tile(q) - sg.rem_tile0;
                const int sl = sg.slot_of(blockIdx.x, rt);
                float* dst = p.part + (((size_t)blockIdx.x * 2 + sl) * NWG + w) * (MP * TN);
#pragma unroll
                for (int e = 0; e < NV; ++e) dst[(e * SP + s) * TN + nl] = outv[e];
                if (sg.cta_of((unsigned int)(rt * KB)) != (int)blockIdx.x) {
                    __threadfence();
                    __syncwarp();
                    if (lane == 0) atomicAdd(p.flags + blockIdx.x * 2 + sl, 1u);
                } else {
                    if (shq0 < 0) shq0 = q;
                    else shq1 = q;
                }
            }
        };

        int seg_q = 0, seg_left = sg.nseg > 0 ? sg.k1(0) - sg.k0(0) : 0;      // current segment, steps left in it
        float c1[NSUB], c2[NSUB];
        int fin1 = -1, fin2 = -1;
#pragma unroll
        for (int sub = 0; sub < NSUB; ++sub) c1[sub] = c2[sub] = 0.0f;
        int aslot = 0, bslot = 0;
        uint32_t apar = 0u, bpar = 0u;
        // What step i needs from shared memory is fetched during iteration i - 1, behind the tensor-memory stores of
        // step i - 1 that have to drain anyway: packed words, coefficients, this lane's B scale factors.
        uint32_t wv_n[8];
        float cf_n[NSUB];
        uint4 sf_n = make_uint4(0u, 0u, 0u, 0u);
        auto fetch_next = [&](int i) {
            ts_wait(full_ws + (uint32_t)aslot * 8u, apar, abort_flag, p.status, 0x432u);
            const unsigned char* stg = ring_w + (size_t)aslot * TB_ASTAGE;
            const uint32_t* wsrc = reinterpret_cast<const uint32_t*>(stg) + wpos;
#pragma unroll
            for (int kw = 0; kw < 8; ++kw) wv_n[kw] = live_row ? wsrc[kw * (WROW / 4)] : 0u;
#pragma unroll
            for (int sub = 0; sub < NSUB; ++sub) {
                const unsigned char* cs = stg + COEF_OFF + sub * CI_BYTES;
                float c = 0.0f;
                if constexpr (IDXB == 0) {
                    if (live_row) c = __half2float(reinterpret_cast<const __half*>(cs)[nl * S + s]);
                } else {
                    const uint32_t ci = (IDXB == 1) ? (uint32_t)cs[nl] : (uint32_t)reinterpret_cast<const unsigned short*>(cs)[nl];
                    if (live_row) c = __half2float((p.cache_in_smem ? cache_s : p.coeff)[(size_t)ci * S + s]);
                }
                cf_n[sub] = c;
            }
            ts_wait(smem_u32(&b_full[bslot]), bpar, abort_flag, p.status, 0x433u);
            sf_n = reinterpret_cast<const uint4*>(bring + (size_t)bslot * BSTAGE + NJ * 4096)[lane];
            if (++aslot == AST) {
                aslot = 0;
                apar ^= 1u;
            }
            if (++bslot == BST) {
                bslot = 0;
                bpar ^= 1u;
            }
        };
        if (n_steps > 0) fetch_next(0);
#pragma unroll 1
        for (int i = 0; i < n_steps + 2; ++i) {
            const int buf = i & 1;
            const bool front = i < n_steps, back = i >= 2;
            int fin_i = -1;
            uint32_t d[NSUB][4][8];
            if (back) {
                ts_wait(mbar0 + buf * 8, (uint32_t)(((i >> 1) - 1) & 1), abort_flag, p.status, 0x434u);
                ts_fence_after();
#pragma unroll
                for (int sub = 0; sub < NSUB; ++sub) {
                    ts_ld16_issue(d_addr + buf * DCOLS + sub * 32, d[sub][0], d[sub][1]);
                    ts_ld16_issue(d_addr + buf * DCOLS + sub * 32 + 16, d[sub][2], d[sub][3]);
                }
            }
            float cf[NSUB];
            if (front) {
                if (--seg_left == 0) {               // last step of a segment: its sums are finished two iterations later
                    fin_i = seg_q;
                    ++seg_q;
                    seg_left = seg_q < sg.nseg ? sg.k1(seg_q) - sg.k0(seg_q) : 0;
                }
#pragma unroll
                for (int sub = 0; sub < NSUB; ++sub) cf[sub] = cf_n[sub];
                // packed words of this thread's row -> 32 words of 4-bit elements {0, 1 | 1 | 2 | 2}
#pragma unroll
                for (int h = 0; h < 4; ++h) {
                    const uint32_t w0 = wv_n[2 * h], w1 = wv_n[2 * h + 1];
                    ts_st8(a_addr + buf * 32 + h * 8, (w0 << 1) & 0x22222222u, w0 & 0x22222222u, w0 & 0x44444444u,
                           (w0 >> 1) & 0x44444444u, (w1 << 1) & 0x22222222u, w1 & 0x22222222u, w1 & 0x44444444u,
                           (w1 >> 1) & 0x44444444u);
                }
                // this B row's scale bytes: word i (MMAs 2 i, 2 i + 1) goes to column 0 of the i-th 4-column block
                asm volatile(
                    "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%4,%4,%4,%2,%4,%4,%4,%3,%4,%4,%4,%4,%4,%4,%4};" ::"r"(
                        sfb_addr + buf * 16),
                    "r"(sf_n.x), "r"(sf_n.y), "r"(sf_n.z), "r"(0x7F7F7F7Fu)
                    : "memory");
                pm |= sf_n.w;
                if (i + 1 < n_steps) fetch_next(i + 1);
            }
            if (back) {
#pragma unroll
                for (int sub = 0; sub < NSUB; ++sub)
#pragma unroll
                    for (int g4 = 0; g4 < 4; ++g4) ts_wait_ld(d[sub][g4]);
#pragma unroll
                for (int sub = 0; sub < NSUB; ++sub)
#pragma unroll
                    for (int m = 0; m < MP; ++m) {
                        float v = __uint_as_float(d[sub][m >> 3][m & 7]);
                        if (NJ == 3) v += __uint_as_float(d[sub][2 + (m >> 3)][m & 7]);
                        acc[m] = fmaf(v, c2[sub], acc[m]);
                    }
                if (fin2 >= 0) finish(fin2);
            }
            if (front) {
                ts_wait_st();
                ts_fence_before();
                ts_bar_arrive(1 + 2 * w + buf, 160);
            }
#pragma unroll
            for (int sub = 0; sub < NSUB; ++sub) {
                c2[sub] = c1[sub];
                if (front) c1[sub] = cf[sub];
            }
            fin2 = fin1;
            fin1 = fin_i;
        }

        // ---- tile groups shared with other CTAs that this CTA finishes: every contributor's sums, in step order
#pragma unroll 1
        for (int h = 0; h < 2; ++h) {
            const int q = h ? shq1 : shq0;
            if (q < 0) continue;
            const int rt = sg.tile(q) - sg.rem_tile0;
            const int tile = sg.tile(q) * NWG + w;
            // Who contributed: the first compute warp works out the owners of the tile group's steps, one step per lane
            // and round (the divisions of cta_of / slot_of cost about 200 cycles each), leaves slot index + 1 of a step's
            // owner in shared memory (0 where the owner is that of the step before), waits until every contributor has
            // delivered, and releases the other compute warps.  All lanes stay converged: a warp that had diverged in
            // per-lane polling loops needed about 800 cycles for every later shuffle.
            const int self_ent = (int)blockIdx.x * 2 + sg.slot_of(blockIdx.x, rt) + 1;
            if (warp == CW0) {
                for (int k = lane; k < KB; k += 32) {
                    const int cc = sg.cta_of((unsigned int)(rt * KB + k));
                    const int cp = k > 0 ? sg.cta_of((unsigned int)(rt * KB + k - 1)) : -1;
                    ctab[k] = (cc != cp) ? cc * 2 + sg.slot_of((unsigned int)cc, rt) + 1 : 0;
                }
                __syncwarp();
                const long long t0 = clock64();
                for (;;) {
                    bool ok = true;
                    for (int k = lane; k < KB; k += 32) {
                        const int en = ctab[k];
                        if (en != 0 && en != self_ent) {
                            unsigned int got;
                            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(got) : "l"(p.flags + (en - 1)) : "memory");
                            ok = ok && got >= (unsigned int)(4 * NWG);
                        }
                    }
                    if (__all_sync(0xffffffffu, ok) || *abort_flag) break;
                    if (clock64() - t0 > 2000000000LL) {
                        *abort_flag = 1;
                        atomicExch(p.status, 1u);
                        atomicExch(p.status + 1, 0x440u);
                        break;
                    }
                }
                __threadfence();
            }
            named_bar_sync(14, NWG * 128);         // the list is complete and every contributor's sums are visible
            // The sums are added in step order, eight contributors at a time with all their loads in flight.  This code
            // runs once per kernel, so its instructions come from L2: a batch of sixteen (twice the code) took 10 000 cycles.
            float v[NV];
#pragma unroll
            for (int e = 0; e < NV; ++e) v[e] = 0.0f;
            int k = 0;
#pragma unroll 1
            while (k < KB) {
                const float* src[8];
                int n = 0;
#pragma unroll
                for (int j = 0; j < 8; ++j) src[j] = p.part;
#pragma unroll 1
                while (k < KB && n < 8) {
                    const int en = ctab[k];
                    ++k;
                    if (en != 0) {
                        const float* sp = p.part + ((size_t)(en - 1) * NWG + w) * (MP * TN);
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            if (j == n) src[j] = sp;
                        ++n;
                    }
                }
                float t[8][NV];
#pragma unroll
                for (int j = 0; j < 8; ++j)
#pragma unroll
                    for (int e = 0; e < NV; ++e) t[j][e] = (j < n) ? __ldcg(src[j] + (e * SP + s) * TN + nl) : 0.0f;
#pragma unroll
                for (int j = 0; j < 8; ++j)
#pragma unroll
                    for (int e = 0; e < NV; ++e)
                        if (j < n) v[e] += t[j][e];
            }
            if (tile < p.NT) {
                const int n = tile * TN + nl;
                const float b = p.bias ? __half2float(p.bias[n]) : 0.0f;
#pragma unroll
                for (int e = 0; e < NV; ++e) {
                    const int m = e * SP + s;
                    if (m < M) p.y[(size_t)m * N + n] = __float2half_rn(v[e] + b);
                }
            }
            // the counters go back to zero: the last of this CTA's compute warps to be done with them clears them (plain
            // stores, one lane per step owner; a returning atomic per contributor from one lane cost a round trip each)
            __syncwarp();
            int old = 0;
            if (lane == 0) old = atomicAdd(const_cast<int*>(done_cnt) + h, 1);
            old = __shfl_sync(0xffffffffu, old, 0);
            if (old == 4 * NWG - 1) {
                for (int k2 = lane; k2 < KB; k2 += 32) {
                    const int en = ctab[k2];
                    if (en != 0 && en != self_ent)
                        asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(p.flags + (en - 1)), "r"(0u) : "memory");
                }
            }
            named_bar_sync(14, NWG * 128);         // the list may be overwritten for the next tile group
        }
    }
    // ------------------------------ teardown ------------------------------
    if (threadIdx.x == 0 && *abort_flag) {         // which problem gave up: N, and K / 256 | M | CTA (for the host's message)
        atomicExch(p.status + 2, (unsigned int)p.N);
        atomicExch(p.status + 3, ((unsigned int)KB << 16) | ((unsigned int)M << 8) | (blockIdx.x & 0xFFu));
    }
    ts_fence_before();
    __syncthreads();
    ts_fence_after();
    if (warp == NWG)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(*tmem_base_s), "r"((uint32_t)TS_TMEM_COLS)
                     : "memory");
}

// ---------------------------------------------------------------------------------------------
// host
// ---------------------------------------------------------------------------------------------
struct TbPlan {
    int KB, NT, NTG, NJ, NWG, grid, cache_in_smem, a_stages, b_stages, smem;
    int off_cache, off_aring, off_bring;
    size_t blob_bytes, part_bytes;
};

static int tb_plan(const PackedW& w, int M, const DeviceInfo& di, TbPlan* pl) {
    const int NSUB = 256 / w.G, TN = ts_tn(w.S);
    pl->NJ = M <= 16 ? 3 : 6;
    pl->NWG = tb_nwg(NSUB);
    pl->KB = w.K / 256;
    pl->NT = w.N / TN;
    pl->NTG = (pl->NT + pl->NWG - 1) / pl->NWG;
    const long long steps = (long long)pl->NTG * pl->KB;
    pl->grid = steps < di.sm_count ? (int)steps : di.sm_count;
    const int MP = pl->NJ == 3 ? 16 : 32;
    pl->blob_bytes = (size_t)pl->KB * tb_bstage(pl->NJ);
    pl->part_bytes = (size_t)pl->grid * 2 * pl->NWG * MP * TN * 4;
    const int cache_bytes = w.idx_bytes ? ts_round_up(w.C * w.S * 2, 16) : 0;
    auto layout = [&](int cb, int ast, int bst) {
        pl->off_cache = TB_HDR;
        pl->off_aring = ts_round_up(pl->off_cache + cb, 128);
        pl->off_bring = ts_round_up(pl->off_aring + pl->NWG * ast * TB_ASTAGE, 128);
        return pl->off_bring + bst * tb_bstage(pl->NJ);
    };
    pl->cache_in_smem = (w.idx_bytes && cache_bytes <= 65536 && layout(cache_bytes, 3, 3) <= di.smem_optin) ? 1 : 0;
    const int cb = pl->cache_in_smem ? cache_bytes : 0;
    int ast = 6, bst = 6;
    while ((ast > 2 || bst > 2) && layout(cb, ast, bst) > di.smem_optin) {
        if (bst >= ast && bst > 2) --bst;
        else if (ast > 2) --ast;
        else --bst;
    }
    pl->a_stages = ast, pl->b_stages = bst;
    pl->smem = layout(cb, ast, bst);
    if (pl->smem > di.smem_optin) return SBVR_ERR_UNSUPPORTED;
    return SBVR_OK;
}

bool linear_tcb_supported(const PackedW& w, int M) {
    if (w.S < 2 || w.S > 4) return false;
    if (w.G != 256 && w.G != 128) return false;
    if (M < 2 || M > 32) return false;
    if (w.G == 128 && M > 16) return false;                                      // tensor-memory columns
    if (w.N % ts_tn(w.S) || w.K % 256 || w.K > 32768) return false;              // at most 128 k blocks (contributor lists)
    if (w.idx_bytes < 0 || w.idx_bytes > 2) return false;
    if (reinterpret_cast<uintptr_t>(w.coeff) & 15) return false;                 // bulk copies
    if (reinterpret_cast<uintptr_t>(w.bvr) & 15) return false;                   // tensor map base
    if (w.idx_bytes && (reinterpret_cast<uintptr_t>(w.idx) & 15)) return false;
    if ((size_t)(w.N / ts_tn(w.S)) * (size_t)(w.K / 256) >= ((size_t)1 << 24)) return false;   // 32-bit step arithmetic
    if ((size_t)w.N * w.S >= ((size_t)1 << 31)) return false;                    // 32-bit tensor coordinates
    return true;
}

size_t linear_tcb_workspace_bytes(const PackedW& w, int M, int sm_count) {
    const int NSUB = 256 / w.G, TN = ts_tn(w.S), NJ = M <= 16 ? 3 : 6, MP = NJ == 3 ? 16 : 32;
    const size_t blob = ((size_t)(w.K / 256) * tb_bstage(NJ) + 255) / 256 * 256;
    const size_t part = (size_t)sm_count * 2 * tb_nwg(NSUB) * MP * TN * 4;
    return blob + part;
}

template <int S, int NSUB, int NJ, int IDXB>
static int tb_launch_inst(const CUtensorMap& tm, const TbParams& p, int grid, int smem, cudaStream_t st) {
    static SmemOnce once;
    const int rc = set_max_smem_once(once, linear_tcb_kernel<S, NSUB, NJ, IDXB>, 227 * 1024);
    if (rc) return rc;
    SBVR_CUDA_TRY(launch_pdl(linear_tcb_kernel<S, NSUB, NJ, IDXB>, dim3(grid), dim3(tb_threads(NSUB)), (size_t)smem, st, tm, p));
    return SBVR_OK;
}
template <int S, int NSUB, int NJ>
static int tb_launch_idx(const CUtensorMap& tm, const TbParams& p, int idxb, int grid, int smem, cudaStream_t st) {
    switch (idxb) {
        case 0: return tb_launch_inst<S, NSUB, NJ, 0>(tm, p, grid, smem, st);
        case 1: return tb_launch_inst<S, NSUB, NJ, 1>(tm, p, grid, smem, st);
        default: return tb_launch_inst<S, NSUB, NJ, 2>(tm, p, grid, smem, st);
    }
}
template <int S>
static int tb_launch_g(const CUtensorMap& tm, const TbParams& p, int G, int NJ, int idxb, int grid, int smem, cudaStream_t st) {
    if (G == 128) return tb_launch_idx<S, 2, 3>(tm, p, idxb, grid, smem, st);
    return NJ == 3 ? tb_launch_idx<S, 1, 3>(tm, p, idxb, grid, smem, st) : tb_launch_idx<S, 1, 6>(tm, p, idxb, grid, smem, st);
}

// `flags` are the first words of the workspace's zeroed exchange region (the kernel leaves them zero); `scratch`
// (256-byte aligned, linear_tcb_workspace_bytes long) holds the digit blob and the partial sums.
int launch_linear_tcb(const __half* x, const PackedW& w, const __half* bias, __half* y, int M, int device,
                      unsigned int* status, unsigned long long* xchg, char* scratch, size_t scratch_bytes, cudaStream_t st) {
    if (!linear_tcb_supported(w, M)) return SBVR_ERR_UNSUPPORTED;
    if (!status || !xchg || !scratch) return SBVR_ERR_WORKSPACE;
    if (reinterpret_cast<uintptr_t>(x) & 1) return SBVR_ERR_ALIGN;
    if (reinterpret_cast<uintptr_t>(scratch) & 255) return SBVR_ERR_ALIGN;
    DeviceInfo di;
    int rc = device_info(device, &di);
    if (rc) return rc;
    if (di.cc_major != 10) return SBVR_ERR_UNSUPPORTED;
    TbPlan pl;
    rc = tb_plan(w, M, di, &pl);
    if (rc) return rc;
    if (linear_tcb_workspace_bytes(w, M, di.sm_count) > scratch_bytes) return SBVR_ERR_WORKSPACE;
    if ((size_t)pl.grid * 2 * 4 > SBVR_WS_XCHG_BYTES) return SBVR_ERR_UNSUPPORTED;
    CUtensorMap tm;
    rc = ts_tensor_map(w, 1, &tm);
    if (rc) return rc;
    unsigned char* blob = reinterpret_cast<unsigned char*>(scratch);
    if (pl.NJ == 3)
        SBVR_CUDA_TRY(launch_pdl(xq8_kernel<3>, dim3(pl.KB), dim3(512), 0, st, x, blob, M, w.K));
    else
        SBVR_CUDA_TRY(launch_pdl(xq8_kernel<6>, dim3(pl.KB), dim3(1024), 0, st, x, blob, M, w.K));
    TbParams p;
    p.xb = blob;
    p.idx = w.idx, p.coeff = w.coeff, p.bias = bias, p.y = y, p.status = status;
    p.flags = reinterpret_cast<unsigned int*>(xchg);
    p.part = reinterpret_cast<float*>(scratch + (pl.blob_bytes + 255) / 256 * 256);
    p.M = M, p.N = w.N, p.K = w.K, p.KB = pl.KB, p.NT = pl.NT, p.NTG = pl.NTG, p.C = w.C;
    p.cache_in_smem = pl.cache_in_smem, p.a_stages = pl.a_stages, p.b_stages = pl.b_stages;
    p.off_cache = pl.off_cache, p.off_aring = pl.off_aring, p.off_bring = pl.off_bring;
    switch (w.S) {
        case 2: return tb_launch_g<2>(tm, p, w.G, pl.NJ, w.idx_bytes, pl.grid, pl.smem, st);
        case 3: return tb_launch_g<3>(tm, p, w.G, pl.NJ, w.idx_bytes, pl.grid, pl.smem, st);
        default: return tb_launch_g<4>(tm, p, w.G, pl.NJ, w.idx_bytes, pl.grid, pl.smem, st);
    }
}

}  // namespace sbvr
