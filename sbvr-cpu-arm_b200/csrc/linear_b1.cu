// Decode-time SBVR linear (M <= 4 activation rows) as a bit-serial tensor-core product.
//
//   y[n] = sum_g sum_s c[g,n,s] * ( sum_{k in g} x[k] * bit_s[n,k] )
//
// The inner sum is a dot product of the activations with a 0/1 vector.  The activations of each
// 256-long block of K are turned into 16-bit block fixed point (one power-of-two step per group of
// G, two's complement), i.e. 16 bit-planes, once per call by `xquant_kernel`.  Then
//   sum_k x[k]*bit[k] = step * sum_b w_b * popc(bitplane_b(x) & bit)      w_b = 2^b, w_15 = -2^15
// and `mma.sync.m16n8k256 ... b1.b1 .and.popc` evaluates 16 weight rows x 8 activation planes x 256
// k per instruction DIRECTLY ON THE PACKED WORDS as they lie in memory: no bit is ever expanded.
// Popcounts are exact integers; they are combined in integer arithmetic, converted to fp32 (exact,
// < 2^24), scaled by the fp16 coefficient and the step and accumulated in fp32.  The only error
// against the fp32-accumulated reference product is the block fixed-point rounding of activations
// more than 2^4 below their group's maximum: at most 2^-16 of the group maximum per element.
//
// Replaces cuda_1xtN_rd_WP8_TBW4_NS4 / cuda_row_deq_mm_T (reference sbvr/kernels/sbvr_kernel.cu:284-359,
// :121-191), whose per-bit select + FMA needs 3-5x more issue slots than HBM3e leaves per element.
//
// Structure: persistent grid, one CTA per SM.  Work is cut into tiles of 64 rows x 256 k
// (8 rows of the [K/32, N*S] word matrix, 64*S*4 contiguous bytes each), numbered row-tile major, and
// every CTA takes one contiguous run of tiles, so that all SMs stream the same number of bytes.
// A producer warp feeds a ring of shared-memory stages with bulk asynchronous copies
// (cp.async.bulk, completion on an mbarrier); eight consumer warps each own 8 of the 64 rows:
// two 128-bit shared loads give a thread its A fragments, four MMAs give the popcounts.
// A row tile whose K range is split over several CTAs is finished by whichever CTA arrives last:
// every contributor stores its fp32 partial sums into its own slot, bumps the tile's counter, and
// the last one adds the slots in a fixed order (deterministic), adds the bias and writes fp16.
// Every wait is bounded; on time-out the kernel records it in the workspace status word and leaves.
#include "common.cuh"

namespace sbvr {

constexpr int B1_TN = 64;                 // rows per tile
constexpr int B1_CW = 8;                  // consumer warps (8 rows each)
constexpr int B1_THREADS = (B1_CW + 1) * 32;
constexpr int B1_MAXD = 16;               // ring stages (upper bound)
constexpr int B1_HDR = 512;               // barriers + flags

struct B1Params {
    const uint32_t* bvr;
    const void* idx;
    const __half* coeff;
    const __half* bias;
    __half* y;
    const uint32_t* xq;       // [M][KB][16 planes][4 tig][2]   words {tig, tig+4} of each plane adjacent
    const float* xscale;      // [M][KB][NSUB]
    float* partial;           // [NT][maxc][M][64]
    unsigned int* counters;   // [NT]
    unsigned int* status;
    int N, K, KB, NT, T, C, maxc, D, cache_in_smem;
};

__host__ __device__ constexpr int b1_rowbytes(int S) { return B1_TN * S * 4; }
// Row pitch in shared memory: the four k-rows a quarter-warp touches must fall into different banks.
__host__ __device__ constexpr int b1_pitch(int S) { return b1_rowbytes(S) + (S == 3 ? 96 : 32); }
__host__ __device__ constexpr int b1_coefbytes(int S, int IDXB) { return IDXB ? B1_TN * IDXB : B1_TN * S * 2; }
__host__ __device__ constexpr int b1_stage(int S, int NSUB, int IDXB) {
    return ((8 * b1_pitch(S) + NSUB * b1_coefbytes(S, IDXB) + 127) / 128) * 128;
}
__host__ __device__ inline int round_up(int v, int a) { return (v + a - 1) / a * a; }

// Tile run of CTA c out of P:  [c*T/P, (c+1)*T/P).  owner(t) is its inverse.
__host__ __device__ inline int b1_tile_begin(int c, int T, int P) { return (int)(((long long)c * T) / P); }
__host__ __device__ inline int b1_tile_owner(int t, int T, int P) { return (int)((((long long)t + 1) * P - 1) / T); }

// ---------------------------------------------------------------------------------------------
// activations -> 16 bit-planes of block fixed point
// ---------------------------------------------------------------------------------------------
template <int NSUB>
__global__ void __launch_bounds__(256) xquant_kernel(const __half* __restrict__ x, uint32_t* __restrict__ xq,
                                                     float* __restrict__ xscale, int K, int KB) {
    __shared__ float wmax[8];
    const int kb = blockIdx.x, m = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float v = __half2float(x[(size_t)m * K + (size_t)kb * 256 + tid]);
    float a = fabsf(v);
    if (!(a == a)) a = __int_as_float(0x7f800000);      // NaN counts as infinity for the maximum
#pragma unroll
    for (int o = 16; o; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
    if (lane == 0) wmax[warp] = a;
    __syncthreads();
    const int sub = (NSUB == 2) ? (warp >> 2) : 0;
    float gm = 0.0f;
#pragma unroll
    for (int i = 0; i < 8 / NSUB; ++i) gm = fmaxf(gm, wmax[sub * (8 / NSUB) + i]);

    int q = 0;
    float step = 0.0f;
    if (gm >= __int_as_float(0x7f800000)) {              // non-finite activations poison the group
        step = __int_as_float(0x7fc00000);
        q = 1;
    } else if (gm > 0.0f) {
        const int e = (int)((__float_as_uint(gm) >> 23) & 0xFF) - 127;    // gm = 1.f * 2^e, e in [-24, 15]
        step = __uint_as_float((uint32_t)(e - 14 + 127) << 23);
        const float inv = __uint_as_float((uint32_t)(14 - e + 127) << 23);
        q = __float2int_rn(v * inv);                     // |q| < 2^15
    }
    uint32_t mine = 0;
#pragma unroll
    for (int b = 0; b < 16; ++b) {
        const uint32_t wv = __ballot_sync(0xffffffffu, (q >> b) & 1);
        if (lane == b) mine = wv;
    }
    if (lane < 16) xq[(((size_t)m * KB + kb) * 16 + lane) * 8 + (warp & 3) * 2 + (warp >> 2)] = mine;
    if ((tid & (256 / NSUB - 1)) == 0) xscale[((size_t)m * KB + kb) * NSUB + sub] = step;
}

// ---------------------------------------------------------------------------------------------
// the product
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void mma_b1(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k256.row.col.s32.b1.b1.s32.and.popc {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%10,%10,%10};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

template <int S, int NSUB, int M, int IDXB>
__global__ void __launch_bounds__(B1_THREADS, 1) linear_b1_kernel(const B1Params p) {
    extern __shared__ __align__(128) unsigned char smem[];
    constexpr int ROWB = b1_rowbytes(S);
    constexpr int PITCH = b1_pitch(S);
    constexpr int CB = b1_coefbytes(S, IDXB);
    constexpr int STAGE = b1_stage(S, NSUB, IDXB);
    constexpr int NPAIR = (S + 1) / 2;

    uint64_t* full = reinterpret_cast<uint64_t*>(smem);
    uint64_t* empty = full + B1_MAXD;
    volatile int* flags = reinterpret_cast<volatile int*>(smem + 2 * B1_MAXD * 8);   // [0] abort, [1] last arriver

    const int KB = p.KB, N = p.N, D = p.D;
    const int xbytes = M * KB * 512;
    const int sbytes = round_up(M * KB * NSUB * 4, 16);
    const int cbytes = p.cache_in_smem ? round_up(p.C * S * 2, 16) : 0;
    uint32_t* xpl = reinterpret_cast<uint32_t*>(smem + B1_HDR);
    float* xsc = reinterpret_cast<float*>(smem + B1_HDR + xbytes);
    __half* cache_s = reinterpret_cast<__half*>(smem + B1_HDR + xbytes + sbytes);
    unsigned char* ring = smem + round_up(B1_HDR + xbytes + sbytes + cbytes, 128);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t0 = b1_tile_begin(blockIdx.x, p.T, gridDim.x);
    const int t1 = b1_tile_begin(blockIdx.x + 1, p.T, gridDim.x);

    if (threadIdx.x == 0) {
        for (int i = 0; i < B1_MAXD; ++i) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], B1_CW);
        }
        flags[0] = 0;
        flags[1] = 0;
        fence_mbar_init();
    }
    __syncthreads();

    if (warp == B1_CW) {
        // ------------------------------ producer ------------------------------
        int i = 0;
        bool gave_up = false;
        for (int t = t0; t < t1; ++t, ++i) {
            const int st = i % D, rnd = i / D;
            if (rnd > 0 && !mbar_wait_bounded(&empty[st], (uint32_t)((rnd - 1) & 1))) {
                gave_up = true;
                break;
            }
            if (flags[0]) break;
            const int nt = t / KB, kb = t - nt * KB, n0 = nt * B1_TN;
            unsigned char* sp = ring + (size_t)st * STAGE;
            if (lane == 0) mbar_arrive_expect_tx(&full[st], 8 * ROWB + NSUB * CB);
            __syncwarp();
            if (lane < 8) {
                bulk_g2s(sp + lane * PITCH, p.bvr + ((size_t)(kb * 8 + lane) * N + n0) * S, ROWB, &full[st]);
            } else if (lane < 8 + NSUB) {
                const int sub = lane - 8, g = kb * NSUB + sub;
                const unsigned char* src =
                    IDXB ? reinterpret_cast<const unsigned char*>(p.idx) + ((size_t)g * N + n0) * IDXB
                         : reinterpret_cast<const unsigned char*>(p.coeff) + ((size_t)g * N + n0) * S * 2;
                bulk_g2s(sp + 8 * PITCH + sub * CB, src, CB, &full[st]);
            }
        }
        if (gave_up) {
            flags[0] = 1;
            if (lane == 0) {
                atomicExch(p.status, 1u);
                atomicExch(p.status + 1, 0x100u + blockIdx.x);
            }
        }
        if (gave_up || flags[0]) {
            // copies already issued still land in this CTA's shared memory: wait for them (bounded)
            const int issued = i;
            for (int j = max(0, issued - D); j < issued; ++j) (void)mbar_wait_bounded(&full[j % D], (uint32_t)((j / D) & 1), 20000u);
        }
        return;
    }

    // ------------------------------ consumers ------------------------------
    const int ctid = threadIdx.x;                  // 0 .. 255
    const int gid = lane >> 2, tig = lane & 3;
    {
        const uint4* src = reinterpret_cast<const uint4*>(p.xq);
        uint4* dst = reinterpret_cast<uint4*>(xpl);
        for (int i = ctid; i < xbytes / 16; i += B1_CW * 32) dst[i] = __ldcg(src + i);
        for (int i = ctid; i < M * KB * NSUB; i += B1_CW * 32) xsc[i] = __ldcg(p.xscale + i);
        if (p.cache_in_smem)
            for (int i = ctid; i < p.C * S; i += B1_CW * 32) cache_s[i] = p.coeff[i];
    }
    named_bar_sync(1, B1_CW * 32);

    float acc[M];
#pragma unroll
    for (int m = 0; m < M; ++m) acc[m] = 0.0f;
    const float f4 = (float)(1 << (2 * tig));
    const int hm = (tig == 3) ? -512 : 512;        // 256 * (+-2): weight of the odd high plane
    const int row = warp * 8 + gid;                // row inside the tile
    int cur_nt = -1, ks_a = 0, kb_last = 0;
    bool aborted = false;

    // Write one finished or partial row tile.  All consumer threads call it together.
    auto flush = [&](int nt, int ka, int kbe) {
        float v[M];
#pragma unroll
        for (int m = 0; m < M; ++m) {
            float a = acc[m];
            a += __shfl_xor_sync(0xffffffffu, a, 1);
            a += __shfl_xor_sync(0xffffffffu, a, 2);
            v[m] = a;
        }
        const int n = nt * B1_TN + row;
        if (ka == 0 && kbe == KB) {
            if (tig == 0) {
                const float b = p.bias ? __half2float(p.bias[n]) : 0.0f;
#pragma unroll
                for (int m = 0; m < M; ++m) p.y[(size_t)m * N + n] = __float2half_rn(v[m] + b);
            }
            return;
        }
        const int cfirst = b1_tile_owner(nt * KB, p.T, gridDim.x);
        const int clast = b1_tile_owner(nt * KB + KB - 1, p.T, gridDim.x);
        const int ci = (int)blockIdx.x - cfirst, ncontrib = clast - cfirst + 1;
        float* slot = p.partial + ((size_t)nt * p.maxc + ci) * M * B1_TN;
        if (tig == 0) {
#pragma unroll
            for (int m = 0; m < M; ++m) slot[m * B1_TN + row] = v[m];
        }
        __threadfence();
        named_bar_sync(1, B1_CW * 32);
        if (ctid == 0) {
            const unsigned int old = atomicAdd(p.counters + nt, 1u);
            const int last = (old == (unsigned int)(ncontrib - 1));
            if (last) p.counters[nt] = 0u;         // every contributor has arrived: ready for the next call
            flags[1] = last;
        }
        named_bar_sync(1, B1_CW * 32);
        if (flags[1]) {
            __threadfence();
            const float* base = p.partial + (size_t)nt * p.maxc * M * B1_TN;
            for (int i = ctid; i < M * B1_TN; i += B1_CW * 32) {
                float s = 0.0f;
                for (int c = 0; c < ncontrib; ++c) s += __ldcg(base + (size_t)c * M * B1_TN + i);
                const int m = i / B1_TN, r = i % B1_TN;
                const int nn = nt * B1_TN + r;
                const float b = p.bias ? __half2float(p.bias[nn]) : 0.0f;
                p.y[(size_t)m * N + nn] = __float2half_rn(s + b);
            }
        }
        named_bar_sync(1, B1_CW * 32);             // flags[1] is rewritten by the next flush
    };

    int i = 0;
    for (int t = t0; t < t1; ++t, ++i) {
        const int st = i % D, rnd = i / D;
        const int nt = t / KB, kb = t - nt * KB;
        if (nt != cur_nt) {
            if (cur_nt >= 0) flush(cur_nt, ks_a, KB);
            cur_nt = nt;
            ks_a = kb;
#pragma unroll
            for (int m = 0; m < M; ++m) acc[m] = 0.0f;
        }
        kb_last = kb;
        if (flags[0] || !mbar_wait_bounded(&full[st], (uint32_t)(rnd & 1))) {
            aborted = true;
            break;
        }
        const unsigned char* sp = ring + (size_t)st * STAGE;
        const unsigned char* rl = sp + tig * PITCH + row * (S * 4);
        const unsigned char* rh = rl + 4 * PITCH;
        uint32_t wl[4] = {0, 0, 0, 0}, wh[4] = {0, 0, 0, 0};
        if constexpr (S == 4) {
            const uint4 a = *reinterpret_cast<const uint4*>(rl), b = *reinterpret_cast<const uint4*>(rh);
            wl[0] = a.x, wl[1] = a.y, wl[2] = a.z, wl[3] = a.w;
            wh[0] = b.x, wh[1] = b.y, wh[2] = b.z, wh[3] = b.w;
        } else if constexpr (S == 2) {
            const uint2 a = *reinterpret_cast<const uint2*>(rl), b = *reinterpret_cast<const uint2*>(rh);
            wl[0] = a.x, wl[1] = a.y;
            wh[0] = b.x, wh[1] = b.y;
        } else {
#pragma unroll
            for (int s = 0; s < S; ++s) {
                wl[s] = reinterpret_cast<const uint32_t*>(rl)[s];
                wh[s] = reinterpret_cast<const uint32_t*>(rh)[s];
            }
        }
        float cf[NSUB][4];
#pragma unroll
        for (int sub = 0; sub < NSUB; ++sub) {
            const unsigned char* ca = sp + 8 * PITCH + sub * CB;
            const __half* cl;
            if constexpr (IDXB == 0) {
                cl = reinterpret_cast<const __half*>(ca) + row * S;
            } else {
                const unsigned int line = (IDXB == 1) ? (unsigned int)ca[row]
                                                      : (unsigned int)reinterpret_cast<const uint16_t*>(ca)[row];
                cl = (p.cache_in_smem ? cache_s : p.coeff) + (size_t)line * S;
            }
#pragma unroll
            for (int s = 0; s < 4; ++s) cf[sub][s] = (s < S) ? __half2float(cl[s]) : 0.0f;
        }
#pragma unroll
        for (int m = 0; m < M; ++m) {
            const uint2* xp = reinterpret_cast<const uint2*>(xpl) + ((size_t)(m * KB + kb) * 16) * 4;
            const uint2 blo = xp[gid * 4 + tig], bhi = xp[(8 + gid) * 4 + tig];
            float g[NSUB];
#pragma unroll
            for (int sub = 0; sub < NSUB; ++sub) g[sub] = 0.0f;
#pragma unroll
            for (int pr = 0; pr < NPAIR; ++pr) {
                const uint32_t a0 = wl[2 * pr], a1 = wl[2 * pr + 1], a2 = wh[2 * pr], a3 = wh[2 * pr + 1];
#pragma unroll
                for (int sub = 0; sub < NSUB; ++sub) {
                    // G = 128: the low half of the k block belongs to one group, the high half to the next
                    const uint32_t l0 = (NSUB == 2 && sub == 1) ? 0u : blo.x, l1 = (NSUB == 2 && sub == 0) ? 0u : blo.y;
                    const uint32_t h0 = (NSUB == 2 && sub == 1) ? 0u : bhi.x, h1 = (NSUB == 2 && sub == 0) ? 0u : bhi.y;
                    int c[4], d[4];
                    mma_b1(c, a0, a1, a2, a3, l0, l1);
                    mma_b1(d, a0, a1, a2, a3, h0, h1);
                    const int p0 = c[0] + 2 * c[1] + 256 * d[0] + hm * d[1];
                    const int p1 = c[2] + 2 * c[3] + 256 * d[2] + hm * d[3];
                    g[sub] = fmaf((float)p0, cf[sub][2 * pr], g[sub]);
                    g[sub] = fmaf((float)p1, cf[sub][2 * pr + 1], g[sub]);
                }
            }
#pragma unroll
            for (int sub = 0; sub < NSUB; ++sub)
                acc[m] = fmaf(g[sub], xsc[(m * KB + kb) * NSUB + sub] * f4, acc[m]);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[st]);
    }
    if (aborted) {
        flags[0] = 1;
        if (lane == 0) {
            atomicExch(p.status, 1u);
            atomicExch(p.status + 1, 0x200u + blockIdx.x);
        }
        return;
    }
    if (cur_nt >= 0) flush(cur_nt, ks_a, kb_last + 1);
}

// ---------------------------------------------------------------------------------------------
// host
// ---------------------------------------------------------------------------------------------
bool linear_b1_supported(const PackedW& w, int M) {
    if (w.S < 2 || w.S > 4) return false;
    if (w.G != 256 && w.G != 128) return false;
    if (M < 1 || M > 4) return false;
    if (w.N % B1_TN || w.K % 256) return false;
    if (w.N / B1_TN > SBVR_WS_COUNTERS) return false;
    if (w.idx_bytes < 0 || w.idx_bytes > 2) return false;
    if ((reinterpret_cast<uintptr_t>(w.bvr) & 15) || (reinterpret_cast<uintptr_t>(w.coeff) & 15)) return false;
    if (w.idx_bytes && (reinterpret_cast<uintptr_t>(w.idx) & 15)) return false;
    return true;
}

struct B1Plan {
    int KB, NT, T, grid, maxc, D, cache_in_smem, smem;
    size_t xq_bytes, xs_bytes, partial_bytes;
};

static int b1_plan(const PackedW& w, int M, const DeviceInfo& di, B1Plan* pl) {
    const int NSUB = 256 / w.G;
    pl->KB = w.K / 256;
    pl->NT = w.N / B1_TN;
    pl->T = pl->KB * pl->NT;
    pl->grid = pl->T < di.sm_count ? pl->T : di.sm_count;
    const int per = pl->T / pl->grid;
    int maxc = (pl->KB + per - 1) / per + 1;
    pl->maxc = maxc < pl->KB ? maxc : pl->KB;
    if (pl->maxc < 1) pl->maxc = 1;
    const int xbytes = M * pl->KB * 512, sbytes = round_up(M * pl->KB * NSUB * 4, 16);
    const int cache_bytes = w.idx_bytes ? round_up(w.C * w.S * 2, 16) : 0;
    pl->cache_in_smem = (w.idx_bytes && cache_bytes <= 32768) ? 1 : 0;
    const int fixed = round_up(B1_HDR + xbytes + sbytes + (pl->cache_in_smem ? cache_bytes : 0), 128);
    const int stage = b1_stage(w.S, NSUB, w.idx_bytes);
    int D = (di.smem_optin - fixed) / stage;
    if (D > B1_MAXD) D = B1_MAXD;
    if (D < 2) return SBVR_ERR_UNSUPPORTED;
    pl->D = D;
    pl->smem = fixed + D * stage;
    pl->xq_bytes = (size_t)xbytes;
    pl->xs_bytes = (size_t)sbytes;
    pl->partial_bytes = (size_t)pl->NT * pl->maxc * M * B1_TN * 4;
    return SBVR_OK;
}

template <int S, int NSUB, int M, int IDXB>
static int b1_launch_inst(const B1Params& p, int grid, int smem, cudaStream_t st) {
    static int configured_for = -1;   // device whose attribute was set last
    int dev = 0;
    SBVR_CUDA_TRY(cudaGetDevice(&dev));
    if (configured_for != dev) {
        SBVR_CUDA_TRY(cudaFuncSetAttribute(linear_b1_kernel<S, NSUB, M, IDXB>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        configured_for = dev;
    }
    linear_b1_kernel<S, NSUB, M, IDXB><<<grid, B1_THREADS, smem, st>>>(p);
    SBVR_CUDA_TRY(cudaGetLastError());
    return SBVR_OK;
}

template <int S, int NSUB, int M>
static int b1_launch_idx(const B1Params& p, int idxb, int grid, int smem, cudaStream_t st) {
    switch (idxb) {
        case 0: return b1_launch_inst<S, NSUB, M, 0>(p, grid, smem, st);
        case 1: return b1_launch_inst<S, NSUB, M, 1>(p, grid, smem, st);
        default: return b1_launch_inst<S, NSUB, M, 2>(p, grid, smem, st);
    }
}
template <int S, int NSUB>
static int b1_launch_m(const B1Params& p, int M, int idxb, int grid, int smem, cudaStream_t st) {
    switch (M) {
        case 1: return b1_launch_idx<S, NSUB, 1>(p, idxb, grid, smem, st);
        case 2: return b1_launch_idx<S, NSUB, 2>(p, idxb, grid, smem, st);
        case 3: return b1_launch_idx<S, NSUB, 3>(p, idxb, grid, smem, st);
        default: return b1_launch_idx<S, NSUB, 4>(p, idxb, grid, smem, st);
    }
}
template <int S>
static int b1_launch_g(const B1Params& p, int G, int M, int idxb, int grid, int smem, cudaStream_t st) {
    return G == 256 ? b1_launch_m<S, 1>(p, M, idxb, grid, smem, st) : b1_launch_m<S, 2>(p, M, idxb, grid, smem, st);
}

static inline size_t round_up_sz(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Activation planes buffer: [bit-planes: M*KB*512 bytes, padded to 256][steps: M*KB*NSUB floats]
size_t act_planes_bytes(int M, int K, int G) {
    const size_t KB = (size_t)K / 256, NSUB = 256 / (size_t)G;
    return round_up_sz((size_t)M * KB * 512, 256) + round_up_sz((size_t)M * KB * NSUB * 4, 256);
}

int launch_xquant(const __half* x, void* planes, int M, int K, int G, cudaStream_t st) {
    if ((G != 256 && G != 128) || K % 256 || M < 1 || M > 65535) return SBVR_ERR_UNSUPPORTED;
    if (reinterpret_cast<uintptr_t>(planes) & 255) return SBVR_ERR_ALIGN;
    const int KB = K / 256;
    uint32_t* xq = reinterpret_cast<uint32_t*>(planes);
    float* xs = reinterpret_cast<float*>(reinterpret_cast<char*>(planes) + round_up_sz((size_t)M * KB * 512, 256));
    dim3 qgrid(KB, M);
    if (G == 256)
        xquant_kernel<1><<<qgrid, 256, 0, st>>>(x, xq, xs, K, KB);
    else
        xquant_kernel<2><<<qgrid, 256, 0, st>>>(x, xq, xs, K, KB);
    SBVR_CUDA_TRY(cudaGetLastError());
    return SBVR_OK;
}

int launch_linear_b1_planes(const void* planes, const PackedW& w, const __half* bias, __half* y, int M,
                            sbvr_workspace* ws, cudaStream_t st) {
    if (!linear_b1_supported(w, M)) return SBVR_ERR_UNSUPPORTED;
    if (!ws) return SBVR_ERR_WORKSPACE;
    if (reinterpret_cast<uintptr_t>(planes) & 255) return SBVR_ERR_ALIGN;
    DeviceInfo di;
    int rc = device_info(ws->device, &di);
    if (rc) return rc;
    B1Plan pl;
    rc = b1_plan(w, M, di, &pl);
    if (rc) return rc;
    if (pl.partial_bytes > ws->dyn_bytes) return SBVR_ERR_WORKSPACE;

    B1Params p;
    p.bvr = w.bvr, p.idx = w.idx, p.coeff = w.coeff, p.bias = bias, p.y = y;
    p.xq = reinterpret_cast<const uint32_t*>(planes);
    p.xscale = reinterpret_cast<const float*>(reinterpret_cast<const char*>(planes) +
                                              round_up_sz((size_t)M * pl.KB * 512, 256));
    p.partial = reinterpret_cast<float*>(ws->dyn);
    p.counters = ws->counters, p.status = ws->status;
    p.N = w.N, p.K = w.K, p.KB = pl.KB, p.NT = pl.NT, p.T = pl.T, p.C = w.C, p.maxc = pl.maxc, p.D = pl.D;
    p.cache_in_smem = pl.cache_in_smem;
    switch (w.S) {
        case 2: return b1_launch_g<2>(p, w.G, M, w.idx_bytes, pl.grid, pl.smem, st);
        case 3: return b1_launch_g<3>(p, w.G, M, w.idx_bytes, pl.grid, pl.smem, st);
        default: return b1_launch_g<4>(p, w.G, M, w.idx_bytes, pl.grid, pl.smem, st);
    }
}

// x -> planes (at the end of the workspace) -> product
int launch_linear_b1(const __half* x, const PackedW& w, const __half* bias, __half* y, int M, sbvr_workspace* ws,
                     cudaStream_t st) {
    if (!linear_b1_supported(w, M)) return SBVR_ERR_UNSUPPORTED;
    if (!ws) return SBVR_ERR_WORKSPACE;
    const size_t pb = act_planes_bytes(M, w.K, w.G);
    if (pb + ((size_t)1 << 20) > ws->dyn_bytes) return SBVR_ERR_WORKSPACE;
    char* planes = ws->dyn + ((ws->dyn_bytes - pb) & ~(size_t)255);
    int rc = launch_xquant(x, planes, M, w.K, w.G, st);
    if (rc) return rc;
    sbvr_workspace shrunk = *ws;
    shrunk.dyn_bytes = (size_t)(planes - ws->dyn);
    return launch_linear_b1_planes(planes, w, bias, y, M, &shrunk, st);
}

}  // namespace sbvr

// Exposed for the host-side unit test of the tile partition (no GPU needed).
extern "C" int sbvr_debug_b1_partition(int T, int P, int c, int* begin, int* end, int t, int* owner) {
    if (begin) *begin = sbvr::b1_tile_begin(c, T, P);
    if (end) *end = sbvr::b1_tile_begin(c + 1, T, P);
    if (owner) *owner = sbvr::b1_tile_owner(t, T, P);
    return 0;
}
