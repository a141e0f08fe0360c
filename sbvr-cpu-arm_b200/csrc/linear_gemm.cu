// SBVR linear for more than four activation rows (small batches and prefill): a tcgen05 fp16 GEMM whose
// weight operand is dequantised inside the kernel and never exists in memory.
//
//   y[m, n] = sum_k x[m, k] * W[n, k] (+ bias[n]),   W[n, k] = sum_s c[k/G, n, s] * bit_s[n, k]
//
// Operands of tcgen05.mma kind::f16 (fp32 accumulation in tensor memory), D[128 weight rows, NX activation rows]:
//
//  A (weights, from tensor memory)  Decoder thread r of a warpgroup owns weight row r of the tile.  Per 64 k it
//      loads its 2 x S packed words, turns them into 64 fp16 values and stores them to its tensor-memory lane
//      (tcgen05.st): decoded weights never touch shared or global memory.  The value of an element is the sum of
//      the c_s whose plane bit is set, formed two elements at a time in half2: a lone bit at position 10 .. 14 of a
//      half is a power of two, so `word & (0x04000400 << i)` is (2^e * bit_j, 2^e * bit_{j+16}) and one HFMA2 with
//      c_s / 2^e adds c_s where the bits are set: a mask and an HFMA2 per plane per pair of elements, plus three
//      shifted copies per word (rows with |c_s| >= 3.9 use sign flips around sum_s c_s / 2 instead: shift, LOP3,
//      HADD2).  Elements j and j + 16 of a word share a 32-bit column, so the K order inside each 32-k word is
//      permuted (position p <-> k = p/2 + 16 (p & 1)).
//  B (activations, from shared memory)  x is first re-tiled by a small kernel into the blocked layout the MMA
//      reads (8-row x 16-byte core matrices, K-major, no swizzle) with the same K permutation, one contiguous
//      block per (NX rows, 64 k); the GEMM fetches a block with a single bulk asynchronous copy.
//
// Replaces `x @ decode().T` of the reference's Llama flow for prefill (reference sbvr_utils/utils_llama.py:147,
// sbvr/core.py:926-949) and the M > 1 use of `_sbvr_row_deq_mm_T` (sbvr/kernels/sbvr_kernel.cu:121-191).
// Accuracy: weights are formed in fp16 with one rounding per plane (not the single rounding of decode()), which
// perturbs a weight by at most a few fp16 ulps of its partial sums; products accumulate in fp32.
//
// Structure: persistent CTAs of 18 warps.  Warps 0-15 are four decoder warpgroups that take the 64-k stages
// round-robin and, once the MMAs of a work item have finished, read D from tensor memory, add the bias and
// write fp16 (or fp32 partial sums when K is split over several CTAs: small activation batches on wide GPUs;
// the last CTA to arrive adds the parts in a fixed order, so results do not depend on timing).  Warp 16 issues
// the MMAs from one elected lane; warp 17 streams the activation blocks.  At M = 2048 the tensor pipe is busy about
// half of the time: a stage costs the decoders about 630 issue slots per scheduler against 512 tensor cycles, and
// the serial work of the issuer warp (barrier polls, four MMAs, three commits per stage) sits on the same path.  Every wait is bounded; on a time-out
// the kernel records it in the status word, skips the remaining work without skipping a barrier, frees its
// tensor memory and returns.
#include "common.cuh"

namespace sbvr {

constexpr int GM_DWGS = 4;
constexpr int GM_DTHREADS = GM_DWGS * 128;
constexpr int GM_IWARP = GM_DWGS * 4;
constexpr int GM_PWARP = GM_IWARP + 1;
constexpr int GM_THREADS = (GM_PWARP + 1) * 32;
constexpr int GM_ASLOTS = 6;                    // decoded 128 x 64 weight tiles resident in tensor memory
constexpr int GM_A_COL = 256;                   // D occupies columns [0, NX), the A ring [256, 256 + 32 slots)
constexpr int GM_TMEM_COLS = 512;
constexpr int GM_XSTAGES = 6;
constexpr int GM_HDR = 1024;

struct GmParams {
    const __half* xt;            // re-tiled activations [MT][K/64][NX*64]
    const uint32_t* bvr;
    const void* idx;
    const __half* coeff;
    const __half* bias;
    __half* y;
    float* part;                 // [KS][MT*NX][N] fp32 partial sums (KS > 1)
    unsigned int* counters;      // one per output tile, zero between launches
    unsigned int* status;
    int M, N, K, C, G, idx_bytes;
    int NT, MT, KS, SPP, items;  // weight-row tiles, activation-row tiles, k parts, 64-k stages per part
};

__device__ __forceinline__ void gm_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void gm_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ uint64_t gm_bdesc(uint32_t saddr) {
    // K-major, no swizzle: 128 B between core matrices along K, 1024 B between 8-row groups; version 1
    return (uint64_t)((saddr & 0x3FFFF) >> 4) | ((uint64_t)(128 >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46);
}
__device__ __forceinline__ void gm_mma(uint32_t d_t, uint32_t a_t, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_t),
        "r"(a_t), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void gm_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void gm_st32(uint32_t taddr, const uint32_t (&a)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
        "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(a[4]), "r"(a[5]), "r"(a[6]), "r"(a[7]), "r"(a[8]), "r"(a[9]),
        "r"(a[10]), "r"(a[11]), "r"(a[12]), "r"(a[13]), "r"(a[14]), "r"(a[15]), "r"(a[16]), "r"(a[17]), "r"(a[18]),
        "r"(a[19]), "r"(a[20]), "r"(a[21]), "r"(a[22]), "r"(a[23]), "r"(a[24]), "r"(a[25]), "r"(a[26]), "r"(a[27]),
        "r"(a[28]), "r"(a[29]), "r"(a[30]), "r"(a[31])
        : "memory");
}
__device__ __forceinline__ void gm_ld32(uint32_t taddr, float (&d)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) d[i] = __uint_as_float(r[i]);
}

// ---------------------------------------------------------------------------------------------
// activations -> blocked, K-permuted layout
// ---------------------------------------------------------------------------------------------
// One thread per 16-byte chunk: chunk (mt, kst, rg, kc, rr) holds row mt*NX + rg*8 + rr, positions kc*8 .. kc*8+7
// of 64-k stage kst; position p of a stage is k = 64 kst + 32 (p / 32) + (p % 32) / 2 + 16 (p & 1).
__global__ void gemm_retile_x_kernel(const __half* __restrict__ x, __half* __restrict__ xt, int M, int K, int NX,
                                     int MT) {
    pdl_launch_dependents();
    pdl_wait();
    const int KST = K / 64;
    const size_t chunks = (size_t)MT * KST * NX * 8;
    for (size_t c = (size_t)blockIdx.x * blockDim.x + threadIdx.x; c < chunks; c += (size_t)gridDim.x * blockDim.x) {
        const int rr = (int)(c & 7), kc = (int)((c >> 3) & 7);
        size_t rest = c >> 6;
        const int rg = (int)(rest % (NX / 8));
        rest /= (NX / 8);
        const int kst = (int)(rest % KST), mt = (int)(rest / KST);
        const int m = mt * NX + rg * 8 + rr;
        __align__(16) __half v[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const int p = kc * 8 + e;
            const int k = kst * 64 + (p & 32) + ((p & 31) >> 1) + 16 * (p & 1);
            v[e] = (m < M) ? x[(size_t)m * K + k] : __float2half(0.0f);
        }
        *reinterpret_cast<uint4*>(xt + c * 8) = *reinterpret_cast<const uint4*>(v);
    }
}

// ---------------------------------------------------------------------------------------------
// the GEMM
// ---------------------------------------------------------------------------------------------
template <int S, int NX>
__global__ void __launch_bounds__(GM_THREADS, 1) linear_gemm_kernel(const GmParams p) {
    extern __shared__ __align__(1024) unsigned char smem[];
    constexpr uint32_t IDESC = (1u << 4) | ((uint32_t)(NX >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
    constexpr int STAGE_BYTES = NX * 128;

    uint64_t* x_full = reinterpret_cast<uint64_t*>(smem);        // [GM_XSTAGES] activation block landed
    uint64_t* x_empty = x_full + GM_XSTAGES;                     // [GM_XSTAGES] ... and read by its MMAs
    uint64_t* a_full = x_empty + GM_XSTAGES;                     // [GM_ASLOTS]  weight tile stored
    uint64_t* a_empty = a_full + GM_ASLOTS;                      // [GM_ASLOTS]  ... and read by its MMAs
    uint64_t* d_full = a_empty + GM_ASLOTS;                      // [1] all MMAs of a work item done
    uint64_t* d_empty = d_full + 1;                              // [1] D read out
    volatile int* flags = reinterpret_cast<volatile int*>(d_empty + 1);     // [0] abort, [1] "last part" flag
    uint32_t* tmem_base_s = reinterpret_cast<uint32_t*>(smem + GM_HDR - 16);
    unsigned char* xs = smem + GM_HDR;                           // [GM_XSTAGES][STAGE_BYTES]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_launch_dependents();
    pdl_wait();                                    // the re-tiled activations come from the previous kernel
    if (threadIdx.x == 0) {
        for (int i = 0; i < GM_XSTAGES; ++i) {
            mbar_init(&x_full[i], 1);
            mbar_init(&x_empty[i], 1);
        }
        for (int i = 0; i < GM_ASLOTS; ++i) {
            mbar_init(&a_full[i], 4);
            mbar_init(&a_empty[i], 1);
        }
        mbar_init(d_full, 1);
        mbar_init(d_empty, GM_DWGS * 4);
        flags[0] = 0;
        flags[1] = 0;
        fence_mbar_init();
    }
    if (warp == GM_PWARP) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_base_s)),
                     "r"((uint32_t)GM_TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        gm_fence_before();
    }
    __syncthreads();
    gm_fence_after();
    const uint32_t tbase = *tmem_base_s;
    const int grid = (int)gridDim.x;
    const int SPP = p.SPP;

    if (warp == GM_PWARP) {
        // ------------------------------ activation producer ------------------------------
        if (lane == 0) {
            int it = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < p.items && ok; item += grid) {
                const int kp = item % p.KS, mt = (item / p.KS) % p.MT;
                const unsigned char* src = reinterpret_cast<const unsigned char*>(p.xt) +
                                           ((size_t)mt * (p.K / 64) + (size_t)kp * SPP) * STAGE_BYTES;
                for (int ks = 0; ks < SPP; ++ks, ++it) {
                    const int st = it % GM_XSTAGES;
                    const uint32_t ph = (uint32_t)(it / GM_XSTAGES) & 1u;
                    if (flags[0] || !mbar_wait_async(&x_empty[st], ph ^ 1u)) {
                        ok = false;
                        break;
                    }
                    mbar_arrive_expect_tx(&x_full[st], (uint32_t)STAGE_BYTES);
                    bulk_g2s(xs + (size_t)st * STAGE_BYTES, src + (size_t)ks * STAGE_BYTES, (uint32_t)STAGE_BYTES,
                             &x_full[st]);
                }
            }
            if (!ok) {
                flags[0] = 1;
                atomicExch(p.status, 1u);
                atomicExch(p.status + 1, 0x500u + blockIdx.x);
            }
        }
    } else if (warp == GM_IWARP) {
        // ------------------------------ MMA issuer ------------------------------
        // A barrier poll costs a couple of hundred cycles on a busy SM even when the phase is complete, and two polls
        // per stage in front of four MMAs made this warp the kernel's serial bottleneck.  So the lanes poll the
        // barriers of the next LOOK stages in one go and the warp issues every stage found complete.
        constexpr int LOOK = GM_XSTAGES < GM_ASLOTS ? GM_XSTAGES : GM_ASLOTS;
        int it = 0, seq = 0, ready = 0;            // stages [it, ready) are known to have both operands in place
        bool ok = true;
        for (int item = blockIdx.x; item < p.items && ok; item += grid, ++seq) {
            if (seq > 0) {                          // D of the previous item must have been read out
                if (flags[0] || !mbar_wait_timed(d_empty, (uint32_t)(seq - 1) & 1u)) {
                    ok = false;
                    break;
                }
                gm_fence_after();
            }
            for (int ks = 0; ks < SPP; ++ks, ++it) {
                const int st = it % GM_XSTAGES, slot = it % GM_ASLOTS;
                if (it >= ready) {
                    long long t0 = 0;
                    for (;;) {
                        const int s = it + lane;   // lane l looks at stage it + l
                        bool okl = false;
                        if (lane < LOOK)
                            okl = mbar_test(&x_full[s % GM_XSTAGES], (uint32_t)(s / GM_XSTAGES) & 1u) &&
                                  mbar_test(&a_full[s % GM_ASLOTS], (uint32_t)(s / GM_ASLOTS) & 1u);
                        const uint32_t mask = __ballot_sync(0xffffffffu, okl);
                        const int n = __ffs((int)~mask) - 1;       // stages complete in a row, starting at `it`
                        if (n > 0) {
                            ready = it + n;
                            break;
                        }
                        if (t0 == 0) t0 = clock64();
                        else if (flags[0] || clock64() - t0 > 2000000000LL) {
                            ok = false;
                            break;
                        }
                    }
                    if (!ok) break;
                    gm_fence_after();
                }
                const uint32_t bs = smem_u32(xs + (size_t)st * STAGE_BYTES);
                if (elect_one()) {
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        gm_mma(tbase, tbase + GM_A_COL + slot * 32 + q * 8, gm_bdesc(bs + q * 256), IDESC,
                               (uint32_t)((ks | q) != 0));
                    gm_commit(&a_empty[slot]);
                    gm_commit(&x_empty[st]);
                    if (ks == SPP - 1) gm_commit(d_full);
                }
                __syncwarp();
            }
        }
        if (!ok) {
            flags[0] = 1;
            if (lane == 0) {
                atomicExch(p.status, 1u);
                atomicExch(p.status + 1, 0x600u + blockIdx.x);
            }
        }
    } else {
        // ------------------------------ decoder warpgroups ------------------------------
        const int wg = warp >> 2, wl = warp & 3;
        const int r = wl * 32 + lane;
        const int dtid = threadIdx.x;              // 0 .. 383
        const uint32_t lane_sel = (uint32_t)(wl * 32) << 16;
        const int N = p.N;
        bool dead = false;

        // The stages of all work items of this CTA form one sequence; this warpgroup takes every third one.
        struct Pos {
            int item, ks, it;
            int kst0, n;                           // first 64-k stage of the item's k part; this thread's weight row
        };
        auto set_item = [&](Pos& q) {              // the divisions happen once per work item, not per stage
            q.kst0 = (q.item % p.KS) * SPP;
            q.n = (q.item / (p.KS * p.MT)) * 128 + r;
        };
        auto advance = [&](Pos& q, int by) {
            q.ks += by;
            q.it += by;
            if (q.ks >= SPP) {
                do {
                    q.ks -= SPP;
                    q.item += grid;
                } while (q.ks >= SPP);
                set_item(q);
            }
        };
        const int group_shift = (p.G == 256) ? 2 : 1;      // 64-k stages per coefficient group, as a shift
        auto load_words = [&](const Pos& q, uint32_t (&w)[2][S]) {
            if (q.item >= p.items) return;
            const uint32_t* src = p.bvr + ((size_t)(2 * (q.kst0 + q.ks)) * N + q.n) * S;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint32_t* g = src + (size_t)h * N * S;
                if constexpr (S == 4) {
                    const uint4 v = __ldg(reinterpret_cast<const uint4*>(g));
                    w[h][0] = v.x, w[h][1] = v.y, w[h][2] = v.z, w[h][3] = v.w;
                } else if constexpr (S == 2) {
                    const uint2 v = __ldg(reinterpret_cast<const uint2*>(g));
                    w[h][0] = v.x, w[h][1] = v.y;
                } else {
#pragma unroll
                    for (int s = 0; s < S; ++s) w[h][s] = __ldg(g + s);
                }
            }
        };
        // D of one finished work item -> y (or fp32 parts); every decoder warp takes part, also when dead.
        int ep_item = blockIdx.x, ep_seq = 0;
        auto epilogue = [&]() {
            const int item = ep_item;
            const int kp = item % p.KS, mt = (item / p.KS) % p.MT, nt = item / (p.KS * p.MT);
            const int n = nt * 128 + r;
            if (!dead && !mbar_wait_async(d_full, (uint32_t)ep_seq & 1u)) {
                dead = true;
                flags[0] = 1;
            }
            dead = __any_sync(0xffffffffu, dead);
            const int m0 = mt * NX;
            if (!dead) {
                gm_fence_after();
                const float bias = (p.bias && p.KS == 1) ? __half2float(p.bias[n]) : 0.0f;
                for (int c = wg; c < NX / 32; c += GM_DWGS) {
                    float d[32];
                    gm_ld32(tbase + lane_sel + c * 32, d);
                    if (p.KS == 1) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const int m = m0 + c * 32 + i;
                            if (m < p.M) p.y[(size_t)m * N + n] = __float2half_rn(d[i] + bias);
                        }
                    } else {
                        float* dst = p.part + ((size_t)kp * p.MT * NX + m0 + c * 32) * N + n;
#pragma unroll
                        for (int i = 0; i < 32; ++i) dst[(size_t)i * N] = d[i];
                    }
                }
                gm_fence_before();
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(d_empty);
            if (p.KS > 1) {
                // split K: the CTA that delivers the last part adds all parts in part order
                __threadfence();
                named_bar_sync(1, GM_DTHREADS);
                if (dtid == 0) {
                    const unsigned int tile = (unsigned int)(mt * p.NT + nt);
                    const unsigned int old = dead ? 0u : atomicAdd(p.counters + tile, 1u);
                    const int last = (!dead && old == (unsigned int)(p.KS - 1)) ? 1 : 0;
                    if (last) p.counters[tile] = 0u;           // ready for the next launch
                    flags[1] = last;
                }
                named_bar_sync(1, GM_DTHREADS);
                const bool last = flags[1] != 0;
                named_bar_sync(1, GM_DTHREADS);                // everyone has read the flag before it is rewritten
                if (last) {
                    __threadfence();
                    const size_t plane = (size_t)p.MT * NX * N;
                    for (int e = dtid; e < NX * 128; e += GM_DTHREADS) {
                        const int mm = e >> 7, nn = e & 127;
                        const int m = m0 + mm;
                        if (m >= p.M) continue;
                        const size_t o = (size_t)m * N + nt * 128 + nn;
                        float v = 0.0f;
                        for (int q = 0; q < p.KS; ++q) v += __ldcg(p.part + (size_t)q * plane + o);
                        if (p.bias) v += __half2float(p.bias[nt * 128 + nn]);
                        p.y[o] = __float2half_rn(v);
                    }
                }
            }
            ep_item += grid;
            ++ep_seq;
        };

        // Coefficients are fetched ahead as well: the line index of a stage two steps before its use, the
        // coefficient line itself one step before (it needs the index), so neither latency is exposed.
        auto line_of = [&](const Pos& q) -> uint32_t {
            if (q.item >= p.items) return 0u;
            const int g = (q.kst0 + q.ks) >> group_shift;
            const size_t e = (size_t)g * N + q.n;
            if (p.idx_bytes == 1) return __ldg(reinterpret_cast<const uint8_t*>(p.idx) + e);
            if (p.idx_bytes == 2) return __ldg(reinterpret_cast<const uint16_t*>(p.idx) + e);
            return (uint32_t)e;
        };
        auto load_coef = [&](const Pos& q, uint32_t line, unsigned short (&c)[S]) {
            if (q.item >= p.items) return;
            const unsigned short* src = reinterpret_cast<const unsigned short*>(p.coeff) + (size_t)line * S;
#pragma unroll
            for (int s = 0; s < S; ++s) c[s] = __ldg(src + s);
        };

        Pos cur{(int)blockIdx.x, 0, 0, 0, 0};
        set_item(cur);
        advance(cur, wg);
        Pos nxt = cur;
        advance(nxt, GM_DWGS);
        Pos nn = nxt;
        advance(nn, GM_DWGS);
        uint32_t w0[2][S], w1[2][S];               // packed words of `cur` and `nxt`: loads run one stage ahead
        unsigned short c0[S], c1[S];               // their coefficient lines (fp16 bits)
        load_words(cur, w0);
        load_words(nxt, w1);
        {
            const uint32_t lc = line_of(cur), ln = line_of(nxt);
            load_coef(cur, lc, c0);
            load_coef(nxt, ln, c1);
        }
        uint32_t l_nn = line_of(nn);

        auto decode_stage = [&](const Pos& q, const uint32_t (&w)[2][S], const unsigned short (&c)[S]) {
            while (ep_item < q.item) epilogue();   // items whose stages have all been handed to the issuer
            // A lone bit at position 10 .. 14 of a half is the number 2^-14, 2^-13, 2^-11, 2^-7, 2^1: masking a packed
            // word with 0x04000400 << i leaves (bit, bit + 16) as such a half2, and one HFMA2 with c_s divided by that
            // number adds c_s where the bit is set.  Three shifted copies of the word bring all 16 bit pairs into the
            // window, so an element pair costs one mask and one HFMA2 per plane (the integer pipe, half as wide as the
            // fp16 pipe, was this kernel's limit with a shift and a mask-xor per pair).  |c_s| >= 4 would overflow the
            // largest multiplier: such a row takes the sign-flip form below instead.
            bool big = false;
            __half2 mul[S][5];
#pragma unroll
            for (int s = 0; s < S; ++s) {
                const __half ch = __ushort_as_half(c[s]);
                big |= !(__habs(ch) < __float2half_rn(3.9f));
                const __half2 c2 = __half2half2(ch);
                mul[s][0] = __hmul2(c2, __float2half2_rn(16384.0f));
                mul[s][1] = __hmul2(c2, __float2half2_rn(8192.0f));
                mul[s][2] = __hmul2(c2, __float2half2_rn(2048.0f));
                mul[s][3] = __hmul2(c2, __float2half2_rn(128.0f));
                mul[s][4] = __hmul2(c2, __float2half2_rn(0.5f));
            }
            const int slot = q.it % GM_ASLOTS;
            if (!dead && !mbar_wait_async(&a_empty[slot], ((uint32_t)(q.it / GM_ASLOTS) & 1u) ^ 1u)) {
                dead = true;
                flags[0] = 1;
            }
            dead = __any_sync(0xffffffffu, dead);
            if (dead) return;
            gm_fence_after();
            uint32_t a[32];
            if (!__any_sync(0xffffffffu, big)) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    __half2 acc[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) acc[j] = __float2half2_rn(0.0f);
#pragma unroll
                    for (int s = 0; s < S; ++s) {
                        // window copies: bits 0..4 / 5..9 / 10..14 / 15 of each half at positions 10..14 / 10..14 / 10..14 / 14
                        const uint32_t v0 = w[h][s] << 10, v1 = w[h][s] << 5, v2 = w[h][s], v3 = w[h][s] >> 1;
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const uint32_t v = (j < 5) ? v0 : (j < 10) ? v1 : (j < 15) ? v2 : v3;
                            const int pos = (j < 15) ? j % 5 : 4;
                            const uint32_t t = v & (0x04000400u << pos);
                            acc[j] = __hfma2(*reinterpret_cast<const __half2*>(&t), mul[s][pos], acc[j]);
                        }
                    }
#pragma unroll
                    for (int j = 0; j < 16; ++j) a[16 * h + j] = *reinterpret_cast<const uint32_t*>(&acc[j]);
                }
            } else {
                uint32_t hc[S];                    // (c_s / 2, c_s / 2)
                float sum = 0.0f;
#pragma unroll
                for (int s = 0; s < S; ++s) {
                    const float chf = __half2float(__ushort_as_half(c[s])) * 0.5f;
                    sum += chf;
                    const uint32_t hb = (uint32_t)__half_as_ushort(__float2half_rn(chf));
                    hc[s] = hb | (hb << 16);
                }
                const uint32_t bb = (uint32_t)__half_as_ushort(__float2half_rn(sum));
                const uint32_t base2 = bb | (bb << 16);
#pragma unroll
                for (int h = 0; h < 2; ++h) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        __half2 acc = *reinterpret_cast<const __half2*>(&base2);
#pragma unroll
                        for (int s = 0; s < S; ++s) {
                            const uint32_t v = w[h][s] << (15 - j);
                            const uint32_t t = (~v & 0x80008000u) ^ hc[s];
                            acc = __hadd2(acc, *reinterpret_cast<const __half2*>(&t));
                        }
                        a[16 * h + j] = *reinterpret_cast<const uint32_t*>(&acc);
                    }
                }
            }
            gm_st32(tbase + lane_sel + GM_A_COL + slot * 32, a);
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            gm_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&a_full[slot]);
        };

        while (cur.item < p.items) {
            decode_stage(cur, w0, c0);
            cur = nxt, nxt = nn;
            advance(nn, GM_DWGS);
            {
                const uint32_t ln = l_nn;          // index of the new look-ahead stage, loaded a step ago
                l_nn = line_of(nn);
                load_words(nxt, w0);               // the set just used is free: it becomes the look-ahead set
                load_coef(nxt, ln, c0);
            }
            if (cur.item >= p.items) break;
            decode_stage(cur, w1, c1);
            cur = nxt, nxt = nn;
            advance(nn, GM_DWGS);
            {
                const uint32_t ln = l_nn;
                l_nn = line_of(nn);
                load_words(nxt, w1);
                load_coef(nxt, ln, c1);
            }
        }
        while (ep_item < p.items) epilogue();

        if (dead) {
            flags[0] = 1;
            if (lane == 0) {
                atomicExch(p.status, 1u);
                atomicExch(p.status + 1, 0x400u + blockIdx.x);
            }
        }
    }
    // ------------------------------ teardown ------------------------------
    gm_fence_before();
    __syncthreads();
    gm_fence_after();
    if (warp == GM_PWARP)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tbase), "r"((uint32_t)GM_TMEM_COLS)
                     : "memory");
}

// ---------------------------------------------------------------------------------------------
// host
// ---------------------------------------------------------------------------------------------
struct GmPlan {
    int NX, MT, NT, KS, SPP, items, grid, smem;
    size_t xt_bytes, part_bytes;
};

static int gm_nx(int M) { return M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256; }

bool linear_gemm_supported(const PackedW& w, int M) {
    if (w.S < 2 || w.S > 4) return false;
    if (w.G != 256 && w.G != 128) return false;
    if (M < 1) return false;
    if (w.N % 128 || w.K % 64) return false;
    if (w.idx_bytes < 0 || w.idx_bytes > 2) return false;
    if (w.S != 3 && (reinterpret_cast<uintptr_t>(w.bvr) & (w.S * 4 - 1))) return false;   // vector loads of a row's planes
    return true;
}

static void gm_plan(const PackedW& w, int M, int sm_count, GmPlan* pl) {
    pl->NX = gm_nx(M);
    pl->MT = (M + pl->NX - 1) / pl->NX;
    pl->NT = w.N / 128;
    const int KST = w.K / 64;
    int ks = 1;
    const int tiles = pl->NT * pl->MT;
    if (tiles < sm_count && tiles <= SBVR_WS_COUNTERS) {
        // split K so that more SMs work, keeping at least 4 stages per part
        for (int cand = 2; cand <= KST / 4; ++cand) {
            if (KST % cand) continue;
            if (tiles * cand > sm_count) break;
            ks = cand;
        }
    }
    pl->KS = ks;
    pl->SPP = KST / ks;
    pl->items = tiles * ks;
    pl->grid = pl->items < sm_count ? pl->items : sm_count;
    pl->smem = GM_HDR + GM_XSTAGES * pl->NX * 128;
    pl->xt_bytes = ((size_t)pl->MT * pl->NX * w.K * 2 + 255) / 256 * 256;
    pl->part_bytes = ks > 1 ? (size_t)ks * pl->MT * pl->NX * w.N * 4 : 0;
}

size_t linear_gemm_workspace_bytes(const PackedW& w, int M, int sm_count) {
    GmPlan pl;
    gm_plan(w, M, sm_count, &pl);
    return pl.xt_bytes + pl.part_bytes;
}

template <int S, int NX>
static int gm_launch_inst(const GmParams& p, int grid, int smem, cudaStream_t st) {
    static SmemOnce once;
    const int rc = set_max_smem_once(once, linear_gemm_kernel<S, NX>, 227 * 1024);
    if (rc) return rc;
    SBVR_CUDA_TRY(launch_pdl(linear_gemm_kernel<S, NX>, dim3(grid), dim3(GM_THREADS), (size_t)smem, st, p));
    return SBVR_OK;
}
template <int S>
static int gm_launch_nx(const GmParams& p, int NX, int grid, int smem, cudaStream_t st) {
    switch (NX) {
        case 32: return gm_launch_inst<S, 32>(p, grid, smem, st);
        case 64: return gm_launch_inst<S, 64>(p, grid, smem, st);
        case 128: return gm_launch_inst<S, 128>(p, grid, smem, st);
        default: return gm_launch_inst<S, 256>(p, grid, smem, st);
    }
}

int launch_linear_gemm(const __half* x, const PackedW& w, const __half* bias, __half* y, int M, sbvr_workspace* ws,
                       cudaStream_t st) {
    if (!linear_gemm_supported(w, M)) return SBVR_ERR_UNSUPPORTED;
    if (!ws) return SBVR_ERR_WORKSPACE;
    DeviceInfo di;
    int rc = device_info(ws->device, &di);
    if (rc) return rc;
    if (di.cc_major != 10) return SBVR_ERR_UNSUPPORTED;
    GmPlan pl;
    gm_plan(w, M, di.sm_count, &pl);
    if (pl.xt_bytes + pl.part_bytes > ws->dyn_bytes) return SBVR_ERR_WORKSPACE;
    __half* xt = reinterpret_cast<__half*>(ws->dyn);
    {
        const size_t chunks = (size_t)pl.MT * pl.NX * w.K / 8;
        const int blocks = (int)((chunks + 255) / 256 < (size_t)di.sm_count * 8 ? (chunks + 255) / 256
                                                                               : (size_t)di.sm_count * 8);
        SBVR_CUDA_TRY(launch_pdl(gemm_retile_x_kernel, dim3(blocks), dim3(256), 0, st, x, xt, M, w.K, pl.NX, pl.MT));
    }
    GmParams p;
    p.xt = xt, p.bvr = w.bvr, p.idx = w.idx, p.coeff = w.coeff, p.bias = bias, p.y = y;
    p.part = reinterpret_cast<float*>(ws->dyn + pl.xt_bytes);
    p.counters = ws->counters, p.status = ws->status;
    p.M = M, p.N = w.N, p.K = w.K, p.C = w.C, p.G = w.G, p.idx_bytes = w.idx_bytes;
    p.NT = pl.NT, p.MT = pl.MT, p.KS = pl.KS, p.SPP = pl.SPP, p.items = pl.items;
    switch (w.S) {
        case 2: return gm_launch_nx<2>(p, pl.NX, pl.grid, pl.smem, st);
        case 3: return gm_launch_nx<3>(p, pl.NX, pl.grid, pl.smem, st);
        default: return gm_launch_nx<4>(p, pl.NX, pl.grid, pl.smem, st);
    }
}

}  // namespace sbvr
