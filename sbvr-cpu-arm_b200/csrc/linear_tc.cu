// Decode-time SBVR linear (M <= 4 activation rows) on the 5th-generation tensor cores.
//
//   y[n] = sum_g sum_s c[g,n,s] * ( sum_{k in g} x[k] * bit_s[n,k] )
//
// The inner sum is a dot product of the activations with a 0/1 vector, evaluated by
// tcgen05.mma kind::mxf4 (packed 4-bit E2M1 operands, fp32 accumulation in tensor memory):
//
//  A operand (weights)  One MMA row per (output row n, plane s).  A packed word holds 32 k of one
//      row; `(w >> j) & 0x11111111` (here shifted to 0x22222222 so that a set bit reads as the E2M1
//      code of 1.0) turns it into a word of eight 4-bit elements with values {0, 1} for
//      k = j, j+4, ..., j+28.  Seven integer instructions expand 32 plane bits; the result goes
//      straight from registers into tensor memory with tcgen05.st and is read by the MMA from
//      there, so the expanded form (4x the packed bytes) never touches shared memory.
//  B operand (activations)  Each group of 256 activations is block fixed point, q = x / step in
//      16-bit two's complement with a power-of-two step per group of G; q is written as eight
//      radix-4 digits, digits 0..6 in {0,1,2,3}, digit 7 in {-2,-1,0,1}, all exact E2M1 values.
//      The 8 digits of an activation row are 8 columns of the MMA's N dimension, stored in the
//      same k permutation as A (`xdigits_kernel`), resident in shared memory for the whole K.
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
// Structure: persistent grid, one CTA per SM, 18 warps.  Work is cut into tiles of 128 MMA rows
// (32 output rows for S = 3, 4; 64 for S = 2) x 256 k, numbered row-tile major; every CTA takes one
// contiguous run of tiles so that all SMs stream the same number of bytes.  Four warpgroups take
// the tiles of a row tile round-robin.  Thread r of a warpgroup owns MMA row r: it loads the 8
// packed words of its row straight from global memory (a warp reads 128 contiguous bytes per
// word row; loads run two tiles ahead of their use), expands them and stores them to its tensor-
// memory lane, then signals an mbarrier.  Two issuer warps (each serving two warpgroups) wait on
// those barriers and issue the four K = 64 MMAs of a tile from one elected lane of a converged
// warp (a lone divergent thread needs about twice as long per tcgen05.mma).  A and D are double
// buffered in tensor memory so that the MMAs of a tile overlap the expansion of the next and the
// epilogue of the previous one.  The first issuer warp also brings the activation digits into
// shared memory with bulk asynchronous copies.  At the end of a row tile the warpgroups' fp32 sums are added in a fixed
// order; a row tile whose K range is split over several CTAs is finished by whichever CTA arrives
// last (per-contributor slots, fixed order: results are deterministic).
// Every wait is bounded; on time-out the kernel records it in the workspace status word, frees its
// tensor memory and leaves.
#include "common.cuh"

namespace sbvr {

constexpr int TC_WGS = 4;                       // warpgroups that compute
constexpr int TC_CTHREADS = TC_WGS * 128;
constexpr int TC_IWARPS = 2;                    // MMA issuer warps, each serves TC_WGS / TC_IWARPS warpgroups
constexpr int TC_THREADS = TC_CTHREADS + 32 * TC_IWARPS;
constexpr int TC_HDR = 1024;                    // barriers, flags, tensor-memory base
constexpr int TC_TMEM_COLS = 512;
constexpr int TC_SF_COL = 448;                  // 64 columns of unit scale factors
constexpr int TC_MAXCHUNK = 16;                 // activation digits arrive in at most 16 bulk copies
constexpr int TC_BSLACK = 4096;                 // MMA columns beyond M read (and ignore) what follows

struct TcParams {
    const uint32_t* bvr;
    const void* idx;
    const __half* coeff;
    const __half* bias;
    __half* y;
    const uint8_t* xd;        // [KB][M][8 kw][8 digits][16 B]
    const float* xscale;      // [M][KB][NSUB]
    float* partial;           // [NT][maxc][M][TN]
    unsigned int* counters;   // [NT]
    unsigned int* status;
    int N, K, KB, NT, T, C, maxc, cache_in_smem, chunk;   // chunk: k blocks per digit copy
};

__host__ __device__ constexpr int tc_sp(int S) { return S == 2 ? 2 : 4; }            // MMA rows per output row
__host__ __device__ constexpr int tc_tn(int S) { return 128 / tc_sp(S); }            // output rows per tile
__host__ __device__ constexpr int tc_mpad(int M) { return M <= 2 ? 2 : 4; }
__host__ __device__ inline int tc_round_up(int v, int a) { return (v + a - 1) / a * a; }
__host__ __device__ inline int tc_tile_begin(int c, int T, int P) { return (int)(((long long)c * T) / P); }
__host__ __device__ inline int tc_tile_owner(int t, int T, int P) { return (int)((((long long)t + 1) * P - 1) / T); }

// ---------------------------------------------------------------------------------------------
// activations -> radix-4 E2M1 digits of 16-bit block fixed point
// ---------------------------------------------------------------------------------------------
template <int NSUB>
__global__ void __launch_bounds__(256) xdigits_kernel(const __half* __restrict__ x, uint8_t* __restrict__ xd,
                                                      float* __restrict__ xscale, int M, int K, int KB) {
    __shared__ float wmax[8];
    __shared__ uint8_t nib[8][8][32];          // [kw][digit][position]
    const int kb = blockIdx.x, m = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float v = __half2float(x[(size_t)m * K + (size_t)kb * 256 + tid]);
    float a = fabsf(v);
    if (!(a == a)) a = __int_as_float(0x7f800000);       // NaN counts as infinity for the maximum
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
    if (gm >= __int_as_float(0x7f800000)) {               // non-finite activations poison the group
        step = __int_as_float(0x7fc00000);
        q = 1;
    } else if (gm > 0.0f) {
        const int e = (int)((__float_as_uint(gm) >> 23) & 0xFF) - 127;   // gm = 1.f * 2^e, e in [-24, 15]
        step = __uint_as_float((uint32_t)(e - 14 + 127) << 23);
        const float inv = __uint_as_float((uint32_t)(14 - e + 127) << 23);
        q = __float2int_rn(v * inv);                      // |q| < 2^15
    }
    if ((tid & (256 / NSUB - 1)) == 0) xscale[((size_t)m * KB + kb) * NSUB + sub] = step;
    // E2M1 codes of the digit values 0, 1, 2, 3 and of -2, -1 (top digit)
    const int pos = 8 * (lane & 3) + (lane >> 2);              // k = 32 kw + j + 4 e  ->  position 8 j + e
#pragma unroll
    for (int d = 0; d < 8; ++d) {
        const int t = (d < 7) ? ((q >> (2 * d)) & 3) : (q >> 14);    // arithmetic shift: -2 .. 1
        uint8_t code;
        if (t >= 0) code = (t == 0) ? 0x0 : (t == 1) ? 0x2 : (t == 2) ? 0x4 : 0x5;
        else code = (t == -1) ? 0xA : 0xC;
        nib[warp][d][pos] = code;
    }
    __syncthreads();
    // 1024 output bytes: [kw][digit][16 B], position p at byte p/2, low nibble first
    uint32_t* out = reinterpret_cast<uint32_t*>(xd + ((size_t)kb * M + m) * 1024);
    const uint8_t* src = &nib[0][0][0] + tid * 8;
    uint32_t wv = 0;
#pragma unroll
    for (int b = 0; b < 4; ++b) wv |= (uint32_t)(src[2 * b] | (src[2 * b + 1] << 4)) << (8 * b);
    out[tid] = wv;
}

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

__device__ __forceinline__ void tc_ld16(uint32_t taddr, float (&d)[16]) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
    tc_wait_ld();
#pragma unroll
    for (int i = 0; i < 16; ++i) d[i] = __uint_as_float(r[i]);
}

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
__device__ long long g_tc_prof[8 * 64 + 8];
#define TC_PROF(slot)                                                                                             \
    do {                                                                                                          \
        if (blockIdx.x == 0 && threadIdx.x == 0 && prof_tile < 64) g_tc_prof[prof_tile * 8 + (slot)] = clock64(); \
    } while (0)
#define TC_PROF_NEXT() ++prof_tile
#define TC_PROF_MARK(k)                                                               \
    do {                                                                              \
        if (blockIdx.x == 0 && threadIdx.x == 0) g_tc_prof[8 * 64 + (k)] = clock64(); \
    } while (0)
#else
#define TC_PROF(slot) do { } while (0)
#define TC_PROF_NEXT() do { } while (0)
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
    extern __shared__ __align__(128) unsigned char smem[];
    constexpr int SP = tc_sp(S);
    constexpr int TN = tc_tn(S);
    constexpr int MPAD = tc_mpad(M);
    constexpr int NMMA = 8 * MPAD;                 // MMA N: 8 digits per activation row
    constexpr bool PIPE = (NSUB * NMMA <= 16);     // room in tensor memory for two D buffers
    // instruction descriptor: A, B = E2M1 (1), scales UE8M0, M = 128, N = NMMA, K-major both, K = 64
    constexpr uint32_t IDESC = (1u << 7) | (1u << 10) | ((uint32_t)(NMMA >> 3) << 17) | (1u << 23) | (8u << 24);

    uint64_t* bbar = reinterpret_cast<uint64_t*>(smem);                               // [TC_MAXCHUNK] digits arrived
    uint64_t* mma_bar = bbar + TC_MAXCHUNK;                                           // [TC_WGS][2] MMAs of a tile done
    uint64_t* a_ready = mma_bar + 2 * TC_WGS;                                         // [TC_WGS][2] A of a tile stored
    volatile int* flags = reinterpret_cast<volatile int*>(a_ready + 2 * TC_WGS);      // [0] abort, [1 + wg] last arriver
    uint32_t* tmem_base_s = reinterpret_cast<uint32_t*>(smem + TC_HDR - 16);

    const int KB = p.KB, N = p.N;
    const int sbytes = tc_round_up(M * KB * NSUB * 4, 16);
    const int cbytes = p.cache_in_smem ? tc_round_up(p.C * S * 2, 16) : 0;
    float* xsc = reinterpret_cast<float*>(smem + TC_HDR);
    __half* cache_s = reinterpret_cast<__half*>(smem + TC_HDR + sbytes);
    unsigned char* Bs = smem + tc_round_up(TC_HDR + sbytes + cbytes, 1024);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // every warpgroup is a worker with its own run of tiles; with fewer tiles than warpgroups only the
    // first T workers get one (so that every worker counted by the split-K protocol does contribute)
    const int P = min((int)gridDim.x * TC_WGS, p.T);
    const int nchunks = (KB + p.chunk - 1) / p.chunk;

    if (threadIdx.x == 0) {
        for (int i = 0; i < TC_MAXCHUNK; ++i) mbar_init(&bbar[i], 1);
        for (int i = 0; i < 2 * TC_WGS; ++i) mbar_init(&mma_bar[i], 1);
        for (int i = 0; i < 2 * TC_WGS; ++i) mbar_init(&a_ready[i], 4);
        for (int i = 0; i < 1 + TC_WGS; ++i) flags[i] = 0;
        fence_mbar_init();
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_base_s)),
                     "r"((uint32_t)TC_TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tbase = *tmem_base_s;
    TC_PROF_MARK(1);

    if (warp >= TC_WGS * 4) {
        // ------------------------------ issuer warps ------------------------------
        const int iw = warp - TC_WGS * 4;
        if (iw == 0 && lane < nchunks) {           // activation digits -> shared memory, one copy per lane
            const int kb_lo = lane * p.chunk;
            const int nkb = min(p.chunk, KB - kb_lo);
            const uint32_t bytes = (uint32_t)nkb * M * 1024;
            mbar_arrive_expect_tx(&bbar[lane], bytes);
            bulk_g2s(Bs + (size_t)kb_lo * M * 1024, p.xd + (size_t)kb_lo * M * 1024, bytes, &bbar[lane]);
        }
        __syncwarp();
        constexpr int PER = TC_WGS / TC_IWARPS;
        const uint32_t sfa = tbase + TC_SF_COL, sfb = tbase + TC_SF_COL + 32;
        int left[PER], kbs[PER], cnt[PER];
        uint32_t aph[PER][2];
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            const int vw = (int)blockIdx.x * TC_WGS + iw * PER + j;
            const int b = vw < P ? tc_tile_begin(vw, p.T, P) : 0;
            left[j] = vw < P ? tc_tile_begin(vw + 1, p.T, P) - b : 0;
            kbs[j] = b % KB;
            cnt[j] = 0;
            aph[j][0] = aph[j][1] = 0u;
        }
        bool ok = true, any = true;
        while (ok && any) {
            any = false;
#pragma unroll
            for (int j = 0; j < PER; ++j) {
                if (!ok || left[j] <= 0) continue;
                any = true;
                const int wgj = iw * PER + j;
                const int buf = PIPE ? (cnt[j] & 1) : 0;
                const int kb = kbs[j];
                const uint32_t a_col = tbase + wgj * 96;
                const uint32_t d_col = a_col + (PIPE ? 64 : 32);
                if (flags[0] || !mbar_wait_timed(&a_ready[wgj * 2 + buf], aph[j][buf]) ||
                    !mbar_wait_timed(&bbar[kb / p.chunk], 0u)) {
                    ok = false;
                    flags[0] = 1;
                    continue;
                }
                aph[j][buf] ^= 1u;
                tc_fence_after();
                const uint32_t bs = smem_u32(Bs + (size_t)kb * M * 1024);
                if (elect_one()) {
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const int sub = (NSUB == 2) ? (q >> 1) : 0;
                        const uint32_t accum = (NSUB == 2) ? (uint32_t)(q & 1) : (uint32_t)(q > 0);
                        tc_mma(d_col + buf * NMMA + sub * NMMA, a_col + buf * 32 + q * 8, tc_bdesc(bs + q * 256), IDESC,
                               sfa, sfb, accum);
                    }
                    tc_commit(&mma_bar[wgj * 2 + buf]);
                }
                __syncwarp();
                left[j] -= 1;
                cnt[j] += 1;
                kbs[j] = (kb + 1 == KB) ? 0 : kb + 1;
            }
        }
        if (!ok && lane == 0) {
            atomicExch(p.status, 1u);
            atomicExch(p.status + 1, 0x100u + blockIdx.x);
        }
    } else {
        // ------------------------------ compute warpgroups ------------------------------
        const int ctid = threadIdx.x;              // 0 .. 511
        const int wg = warp >> 2, wl = warp & 3;
        const int wtid = ctid & 127;               // thread inside the warpgroup
        const int r = wl * 32 + lane;              // MMA row = tensor-memory lane
        const int nl = r / SP, s = r % SP;         // output row inside the tile, plane
        const bool live_row = s < S;
        const uint32_t lane_sel = (uint32_t)(wl * 32) << 16;
        const uint32_t a_col = tbase + wg * 96;
        const uint32_t d_col = a_col + (PIPE ? 64 : 32);

        // ---- this warpgroup's run of tiles
        const int vw = (int)blockIdx.x * TC_WGS + wg;
        const int t0 = vw < P ? tc_tile_begin(vw, p.T, P) : 0;
        const int n_tiles = vw < P ? tc_tile_begin(vw + 1, p.T, P) - t0 : 0;
        int nt_c = n_tiles > 0 ? t0 / KB : 0;      // position of the tile being processed
        int kb_c = t0 - nt_c * KB;

        // ---- loads run two tiles ahead; all offsets are 32-bit element offsets, advanced incrementally
        struct Raw {
            uint32_t w[8];
            uint32_t ci[NSUB];
        };
        const uint32_t NS = (uint32_t)N * S, KSTEP = 8u * NS, ISTEP = (uint32_t)NSUB * N;
        int nt_l = nt_c, kb_l = kb_c, loaded = 0;
        uint32_t off_l = ((uint32_t)(kb_l * 8) * N + nt_l * TN + nl) * S + s;       // word offset into bvr
        uint32_t ioff_l = (uint32_t)(kb_l * NSUB) * N + nt_l * TN + nl;              // (group, row) offset
        auto load_tile = [&](Raw& q) {
            if (loaded < n_tiles && live_row) {
#pragma unroll
                for (int kw = 0; kw < 8; ++kw) q.w[kw] = __ldcs(p.bvr + (off_l + kw * NS));
#pragma unroll
                for (int sub = 0; sub < NSUB; ++sub) {
                    const uint32_t io = ioff_l + sub * N;
                    if constexpr (IDXB == 0)
                        q.ci[sub] = __ldcs(reinterpret_cast<const unsigned short*>(p.coeff) + ((size_t)io * S + s));
                    else if constexpr (IDXB == 1)
                        q.ci[sub] = __ldcs(reinterpret_cast<const unsigned char*>(p.idx) + io);
                    else
                        q.ci[sub] = __ldcs(reinterpret_cast<const unsigned short*>(p.idx) + io);
                }
            } else {
#pragma unroll
                for (int kw = 0; kw < 8; ++kw) q.w[kw] = 0u;
#pragma unroll
                for (int sub = 0; sub < NSUB; ++sub) q.ci[sub] = 0u;
            }
            ++loaded;
            ++kb_l;
            off_l += KSTEP;
            ioff_l += ISTEP;
            if (kb_l == KB) {
                kb_l = 0;
                ++nt_l;
                off_l = (uint32_t)(nt_l * TN + nl) * S + s;
                ioff_l = (uint32_t)(nt_l * TN + nl);
            }
        };
        Raw X0, X1, X2;
        load_tile(X0);
        load_tile(X1);

        for (int i = ctid; i < M * KB * NSUB; i += TC_CTHREADS) xsc[i] = __ldcg(p.xscale + i);
        if (p.cache_in_smem) {
            const int nvec = (p.C * S * 2) / 16;
            const uint4* src = reinterpret_cast<const uint4*>(p.coeff);
            uint4* dst = reinterpret_cast<uint4*>(cache_s);
            for (int i = ctid; i < nvec; i += TC_CTHREADS) dst[i] = __ldg(src + i);
            for (int i = nvec * 8 + ctid; i < p.C * S; i += TC_CTHREADS) cache_s[i] = p.coeff[i];
        }
        if (wg == 0) {                             // unit scale factors, every byte 2^0
            tc_st_fill32(tbase + lane_sel + TC_SF_COL, 0x7F7F7F7Fu);
            tc_st_fill32(tbase + lane_sel + TC_SF_COL + 32, 0x7F7F7F7Fu);
            tc_wait_st();
        }
        tc_fence_before();
        named_bar_sync(1, TC_CTHREADS);            // scale factors, steps and codebook are in place
        tc_fence_after();
        TC_PROF_MARK(2);

        float acc[M];
#pragma unroll
        for (int m = 0; m < M; ++m) acc[m] = 0.0f;
        uint32_t ph[2] = {0u, 0u};                 // phases of this warpgroup's two MMA barriers
        bool dead = false;
        bool pend = false;                         // deferred epilogue of the previous tile (PIPE only)
        int pend_buf = 0;
        float pend_scale[NSUB][M];
        int seg_ka = kb_c;                         // first k block of the row tile segment being summed
        int ti = 0;                                // tiles done

        // D of one finished tile -> fp32 sums.  `buf` selects the D buffer.
        auto epilogue = [&](int buf, const float (&scale)[NSUB][M]) {
#pragma unroll
            for (int sub = 0; sub < NSUB; ++sub) {
#pragma unroll
                for (int m = 0; m < M; ++m) {
                    float d[8];
                    tc_ld8(d_col + lane_sel + buf * NMMA + sub * NMMA + m * 8, d);
                    float pv = 0.0f;
#pragma unroll
                    for (int dg = 7; dg >= 0; --dg) pv = fmaf(pv, 4.0f, d[dg]);
                    acc[m] = fmaf(pv, scale[sub][m], acc[m]);
                }
            }
            tc_fence_before();     // order these tensor-memory reads before later writes of the buffer
        };
        auto wait_mma = [&](int buf) {
            if (!dead && !mbar_wait_timed(&mma_bar[wg * 2 + buf], ph[buf])) {
                dead = true;
                flags[0] = 1;
            }
            dead = __any_sync(0xffffffffu, dead);  // warp-uniform: tcgen05.st/ld are .aligned
            if (!dead) {
                ph[buf] ^= 1u;
                tc_fence_after();
            }
        };

        // Finish the rows of one row tile with the sums of k blocks [ka, kbe).  All 128 threads of the
        // warpgroup call it together; it contains barriers and is never skipped.
        auto flush = [&](int nt, int ka, int kbe) {
            float v[M];
#pragma unroll
            for (int m = 0; m < M; ++m) {
                float a = acc[m];
                a += __shfl_xor_sync(0xffffffffu, a, 1);
                if (SP == 4) a += __shfl_xor_sync(0xffffffffu, a, 2);
                v[m] = a;
                acc[m] = 0.0f;
            }
            const int n = nt * TN + nl;
            if (ka == 0 && kbe == KB) {
                if (s == 0) {
                    const float b = p.bias ? __half2float(p.bias[n]) : 0.0f;
#pragma unroll
                    for (int m = 0; m < M; ++m) p.y[(size_t)m * N + n] = __float2half_rn(v[m] + b);
                }
                return;
            }
            const int cfirst = tc_tile_owner(nt * KB, p.T, P);
            const int clast = tc_tile_owner(nt * KB + KB - 1, p.T, P);
            const int ci = vw - cfirst, ncontrib = clast - cfirst + 1;
            float* slot = p.partial + ((size_t)nt * p.maxc + ci) * M * TN;
            if (s == 0) {
#pragma unroll
                for (int m = 0; m < M; ++m) slot[m * TN + nl] = v[m];
            }
            __threadfence();
            named_bar_sync(2 + wg, 128);
            if (wtid == 0) {
                const unsigned int old = atomicAdd(p.counters + nt, 1u);
                const int last = (old == (unsigned int)(ncontrib - 1));
                if (last) p.counters[nt] = 0u;     // every contributor has arrived: ready for the next call
                flags[1 + wg] = last;
            }
            named_bar_sync(2 + wg, 128);
            if (flags[1 + wg]) {
                __threadfence();
                const float* base = p.partial + (size_t)nt * p.maxc * M * TN;
                for (int i = wtid; i < M * TN; i += 128) {
                    float sum = 0.0f;
                    for (int c = 0; c < ncontrib; ++c) sum += __ldcg(base + (size_t)c * M * TN + i);
                    const int m = i / TN, rr = i % TN;
                    const int nn = nt * TN + rr;
                    const float b = p.bias ? __half2float(p.bias[nn]) : 0.0f;
                    p.y[(size_t)m * N + nn] = __float2half_rn(sum + b);
                }
            }
        };

        // One tile: `cur` holds its words (loaded two steps ago), `fill` is the register set to refill.
        auto step = [&](Raw& cur, Raw& fill) {
            TC_PROF(0);
            load_tile(fill);                       // tile ti + 2
            const int buf = PIPE ? (ti & 1) : 0;
            if (flags[0]) dead = true;
            dead = __any_sync(0xffffffffu, dead);
            TC_PROF(1);
            float scale[NSUB][M];
#pragma unroll
            for (int sub = 0; sub < NSUB; ++sub) {
                float c = 0.0f;
                if (live_row) {
                    if constexpr (IDXB == 0) c = __half2float(__ushort_as_half((unsigned short)cur.ci[sub]));
                    else c = __half2float((p.cache_in_smem ? cache_s : p.coeff)[(size_t)cur.ci[sub] * S + s]);
                }
#pragma unroll
                for (int m = 0; m < M; ++m) scale[sub][m] = c * xsc[(m * KB + kb_c) * NSUB + sub];
            }
            if (!dead) {
                // ---- packed words of this thread's row -> 32 words of 4-bit {0, 1.0} elements
                uint32_t a[32];
#pragma unroll
                for (int kw = 0; kw < 8; ++kw) {
                    const uint32_t w = cur.w[kw];
                    a[4 * kw + 0] = (w << 1) & 0x22222222u;
                    a[4 * kw + 1] = w & 0x22222222u;
                    a[4 * kw + 2] = (w >> 1) & 0x22222222u;
                    a[4 * kw + 3] = (w >> 2) & 0x22222222u;
                }
                TC_PROF(2);
                // buffer `buf` is free: the MMAs that read it two tiles ago were waited for last step
                tc_st32(a_col + lane_sel + buf * 32, a);
            }
            TC_PROF(3);
            if (PIPE && pend) {                    // the previous tile's epilogue overlaps the store
                wait_mma(pend_buf);
                TC_PROF(4);
                if (!dead) epilogue(pend_buf, pend_scale);
                pend = false;
            }
            TC_PROF(5);
            if (!dead) {
                tc_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&a_ready[wg * 2 + buf]);   // 4 warps release the issuer
            }
            const bool seg_end = (kb_c + 1 == KB) || (ti + 1 == n_tiles);
            if (PIPE && !seg_end) {
                pend = true;
                pend_buf = buf;
#pragma unroll
                for (int sub = 0; sub < NSUB; ++sub)
#pragma unroll
                    for (int m = 0; m < M; ++m) pend_scale[sub][m] = scale[sub][m];
            } else {
                wait_mma(buf);
                if (!dead) epilogue(buf, scale);
            }
            if (seg_end) {
                flush(nt_c, seg_ka, kb_c + 1);
                seg_ka = 0;
            }
            TC_PROF(6);
            TC_PROF_NEXT();
            ++ti;
            ++kb_c;
            if (kb_c == KB) {
                kb_c = 0;
                ++nt_c;
            }
        };

        while (ti < n_tiles) {
            step(X0, X2);
            if (ti < n_tiles) step(X1, X0);
            if (ti < n_tiles) step(X2, X1);
        }
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
    if (warp == TC_WGS * 4 && lane < nchunks) {
        // the digit copies must have landed before this CTA's shared memory is given up
        if (!mbar_wait_timed(&bbar[lane], 0u)) atomicExch(p.status, 1u);
    }
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tbase), "r"((uint32_t)TC_TMEM_COLS)
                     : "memory");
    TC_PROF_MARK(4);
}


// ---------------------------------------------------------------------------------------------
// host
// ---------------------------------------------------------------------------------------------
struct TcPlan {
    int KB, NT, T, grid, maxc, cache_in_smem, chunk, smem;
    size_t partial_bytes;
};

static int tc_plan(const PackedW& w, int M, const DeviceInfo& di, TcPlan* pl) {
    const int NSUB = 256 / w.G, TN = tc_tn(w.S);
    pl->KB = w.K / 256;
    pl->NT = w.N / TN;
    pl->T = pl->KB * pl->NT;
    const int want = (pl->T + TC_WGS - 1) / TC_WGS;          // CTAs needed to give every warpgroup a tile
    pl->grid = want < di.sm_count ? want : di.sm_count;
    const int workers = pl->grid * TC_WGS < pl->T ? pl->grid * TC_WGS : pl->T;
    const int per = pl->T / workers;                          // tiles per warpgroup, rounded down (>= 1)
    int maxc = (pl->KB + per - 1) / per + 1;
    pl->maxc = maxc < pl->KB ? maxc : pl->KB;
    if (pl->maxc < 1) pl->maxc = 1;
    pl->chunk = (pl->KB + TC_MAXCHUNK - 1) / TC_MAXCHUNK;
    const int sbytes = tc_round_up(M * pl->KB * NSUB * 4, 16);
    const int red_bytes = 0;
    const int bbytes = pl->KB * M * 1024 + TC_BSLACK;
    const int cache_bytes = w.idx_bytes ? tc_round_up(w.C * w.S * 2, 16) : 0;
    const int base = TC_HDR + sbytes + red_bytes;
    // the codebook goes to shared memory if it still fits next to the digits
    pl->cache_in_smem = (w.idx_bytes && cache_bytes <= 65536 &&
                         tc_round_up(base + cache_bytes, 1024) + bbytes <= di.smem_optin) ? 1 : 0;
    pl->smem = tc_round_up(base + (pl->cache_in_smem ? cache_bytes : 0), 1024) + bbytes;
    if (pl->smem > di.smem_optin) return SBVR_ERR_UNSUPPORTED;      // K * M too large for resident digits
    pl->partial_bytes = (size_t)pl->NT * pl->maxc * M * TN * 4;
    return SBVR_OK;
}

bool linear_tc_supported(const PackedW& w, int M) {
    if (w.S < 2 || w.S > 4) return false;
    if (w.G != 256 && w.G != 128) return false;
    if (M < 1 || M > 4) return false;
    if (w.N % tc_tn(w.S) || w.K % 256) return false;
    if (w.N / tc_tn(w.S) > SBVR_WS_COUNTERS) return false;
    if (w.idx_bytes < 0 || w.idx_bytes > 2) return false;
    if (reinterpret_cast<uintptr_t>(w.coeff) & 15) return false;
    // the activation digits of the whole K stay resident in shared memory: K/256 * M KB
    const int KB = w.K / 256, NSUB = 256 / w.G;
    const int base = TC_HDR + tc_round_up(M * KB * NSUB * 4, 16);
    if ((size_t)tc_round_up(base, 1024) + (size_t)KB * M * 1024 + TC_BSLACK > 227 * 1024) return false;
    return true;
}

static inline size_t tc_round_up_sz(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Activation digits buffer: [digits: KB * M * 1024 bytes, padded to 256][steps: M * KB * NSUB floats, padded to 256]
size_t act_digits_bytes(int M, int K, int G) {
    const size_t KB = (size_t)K / 256, NSUB = 256 / (size_t)G;
    return tc_round_up_sz(KB * M * 1024, 256) + tc_round_up_sz((size_t)M * KB * NSUB * 4, 256);
}

int launch_xdigits(const __half* x, void* buf, int M, int K, int G, cudaStream_t st) {
    if ((G != 256 && G != 128) || K % 256 || M < 1 || M > 4) return SBVR_ERR_UNSUPPORTED;
    if (reinterpret_cast<uintptr_t>(buf) & 255) return SBVR_ERR_ALIGN;
    const int KB = K / 256;
    uint8_t* xd = reinterpret_cast<uint8_t*>(buf);
    float* xs = reinterpret_cast<float*>(xd + tc_round_up_sz((size_t)KB * M * 1024, 256));
    dim3 grid(KB, M);
    if (G == 256)
        xdigits_kernel<1><<<grid, 256, 0, st>>>(x, xd, xs, M, K, KB);
    else
        xdigits_kernel<2><<<grid, 256, 0, st>>>(x, xd, xs, M, K, KB);
    SBVR_CUDA_TRY(cudaGetLastError());
    return SBVR_OK;
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
    linear_tc_kernel<S, NSUB, M, IDXB><<<grid, TC_THREADS, smem, st>>>(p);
    SBVR_CUDA_TRY(cudaGetLastError());
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

int launch_linear_tc_digits(const void* buf, const PackedW& w, const __half* bias, __half* y, int M,
                            sbvr_workspace* ws, cudaStream_t st) {
    if (!linear_tc_supported(w, M)) return SBVR_ERR_UNSUPPORTED;
    if (!ws) return SBVR_ERR_WORKSPACE;
    if (reinterpret_cast<uintptr_t>(buf) & 255) return SBVR_ERR_ALIGN;
    DeviceInfo di;
    int rc = device_info(ws->device, &di);
    if (rc) return rc;
    if (di.cc_major != 10) return SBVR_ERR_UNSUPPORTED;
    TcPlan pl;
    rc = tc_plan(w, M, di, &pl);
    if (rc) return rc;
    if (pl.partial_bytes > ws->dyn_bytes) return SBVR_ERR_WORKSPACE;

    TcParams p;
    p.bvr = w.bvr, p.idx = w.idx, p.coeff = w.coeff, p.bias = bias, p.y = y;
    p.xd = reinterpret_cast<const uint8_t*>(buf);
    p.xscale = reinterpret_cast<const float*>(p.xd + tc_round_up_sz((size_t)pl.KB * M * 1024, 256));
    p.partial = reinterpret_cast<float*>(ws->dyn);
    p.counters = ws->counters, p.status = ws->status;
    p.N = w.N, p.K = w.K, p.KB = pl.KB, p.NT = pl.NT, p.T = pl.T, p.C = w.C, p.maxc = pl.maxc;
    p.cache_in_smem = pl.cache_in_smem, p.chunk = pl.chunk;
    switch (w.S) {
        case 2: return tc_launch_g<2>(p, w.G, M, w.idx_bytes, pl.grid, pl.smem, st);
        case 3: return tc_launch_g<3>(p, w.G, M, w.idx_bytes, pl.grid, pl.smem, st);
        default: return tc_launch_g<4>(p, w.G, M, w.idx_bytes, pl.grid, pl.smem, st);
    }
}

// x -> digits (at the end of the workspace) -> product
int launch_linear_tc(const __half* x, const PackedW& w, const __half* bias, __half* y, int M, sbvr_workspace* ws,
                     cudaStream_t st) {
    if (!linear_tc_supported(w, M)) return SBVR_ERR_UNSUPPORTED;
    if (!ws) return SBVR_ERR_WORKSPACE;
    const size_t pb = act_digits_bytes(M, w.K, w.G);
    if (pb + ((size_t)1 << 20) > ws->dyn_bytes) return SBVR_ERR_WORKSPACE;
    char* buf = ws->dyn + ((ws->dyn_bytes - pb) & ~(size_t)255);
    int rc = launch_xdigits(x, buf, M, w.K, w.G, st);
    if (rc) return rc;
    sbvr_workspace shrunk = *ws;
    shrunk.dyn_bytes = (size_t)(buf - ws->dyn);
    return launch_linear_tc_digits(buf, w, bias, y, M, &shrunk, st);
}

}  // namespace sbvr

#ifdef SBVR_PROFILE
extern "C" __attribute__((visibility("default"))) int sbvr_debug_read_profile(long long* out, int n) {
    long long tmp[8 * 64 + 8];
    if (cudaMemcpyFromSymbol(tmp, sbvr::g_tc_prof, sizeof(tmp)) != cudaSuccess) return -1;
    for (int i = 0; i < n && i < 8 * 64 + 8; ++i) out[i] = tmp[i];
    return 0;
}
#endif
