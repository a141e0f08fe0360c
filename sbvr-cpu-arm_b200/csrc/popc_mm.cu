// SBVR x SBVR product: both operands are bit-plane encoded, the inner products are popcounts.
//
//   y[m][n] = sum_g sum_{a < LS} sum_{b < RS} popc( l_a[m, g] & r_b[n, g] ) * cl[g, m, a] * cr[g, n, b]  (+ bias[n])
//
// l_a[m, g], r_b[n, g] = the 256 bits of plane a / b of row m / n in group g; cl, cr = the fp16 coefficient lines
// the index tensors select.  Replaces `_sbvr_mm_T` / cuda_1xtN_sbvr_mm_T of the reference
// (sbvr/kernels/sbvr_ops.cpp:35-76, sbvr/kernels/sbvr_kernel.cu:464-562, launch :914-1023) on the same layouts:
//   l_bvr u32 [K/32, M, LS], l_idx u8|u16 [K/256, M], l_cache f16 [Cl, LS];   r_* likewise with N, RS.
// Differences from the reference kernel, both on the side of accuracy: popcounts are kept in 32-bit counters (the
// reference's uchar counters wrap at 256, sbvr_kernel.cu:486-487) and the coefficient products and sums are fp32
// (the reference multiplies in half2).
//
// The right operand (the weight) is streamed once: a warp owns 32 / RP weight rows (RP = planes per row, 4 for
// RS = 3) and a quarter of K; lane = (row, plane) reads one packed word per 32 k, 128 contiguous bytes per warp.
// The left operand (the encoded activations, at most 8 rows per pass) sits in shared memory with its coefficients.
#include "common.cuh"

namespace sbvr {

constexpr int PM_MT = 8;               // left rows per pass
constexpr int PM_KQ = 4;               // K quarters per row block (one warp each)
constexpr int PM_RB = 2;               // row blocks per CTA
constexpr int PM_THREADS = 32 * PM_KQ * PM_RB;

template <int LS, int RS, int GU>
__global__ void __launch_bounds__(PM_THREADS) popc_mm_kernel(const uint32_t* __restrict__ l_bvr, const void* __restrict__ l_idx,
                                                             int l_idx_bytes, const __half* __restrict__ l_cache,
                                                             const uint32_t* __restrict__ r_bvr, const void* __restrict__ r_idx,
                                                             int r_idx_bytes, const __half* __restrict__ r_cache,
                                                             const __half* __restrict__ bias, __half* __restrict__ y, int M,
                                                             int m0, int N, int K) {
    extern __shared__ __align__(16) unsigned char smem[];
    constexpr int RP = (RS == 3) ? 4 : RS;
    constexpr int ROWS = 32 / RP;                       // weight rows per warp
    const int KW = K / 32, KB = K / 256;
    const int mt = min(PM_MT, M - m0);
    uint32_t* lw = reinterpret_cast<uint32_t*>(smem);                       // [KW][mt][LS]
    float* lc = reinterpret_cast<float*>(smem + (size_t)KW * PM_MT * LS * 4);   // [KB][mt][LS]
    float* red = lc + (size_t)KB * PM_MT * LS;                               // [PM_RB][PM_KQ][PM_MT][ROWS]
    pdl_launch_dependents();
    pdl_wait();
    for (int i = threadIdx.x; i < KW * mt * LS; i += PM_THREADS) {
        const int a = i % LS, m = (i / LS) % mt, kw = i / (LS * mt);
        lw[(kw * PM_MT + m) * LS + a] = l_bvr[((size_t)kw * M + m0 + m) * LS + a];
    }
    for (int i = threadIdx.x; i < KB * mt * LS; i += PM_THREADS) {
        const int a = i % LS, m = (i / LS) % mt, g = i / (LS * mt);
        const size_t e = (size_t)g * M + m0 + m;
        const size_t line = (l_idx_bytes == 1) ? reinterpret_cast<const uint8_t*>(l_idx)[e]
                                               : reinterpret_cast<const uint16_t*>(l_idx)[e];
        lc[(g * PM_MT + m) * LS + a] = __half2float(l_cache[line * LS + a]);
    }
    __syncthreads();

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rb = warp / PM_KQ, kq = warp % PM_KQ;
    const int n = ((int)blockIdx.x * PM_RB + rb) * ROWS + lane / RP, b = lane % RP;
    const bool live = (n < N) && (b < RS);
    const int g0 = (KB * kq) / PM_KQ, g1 = (KB * (kq + 1)) / PM_KQ;
    float acc[PM_MT];
#pragma unroll
    for (int m = 0; m < PM_MT; ++m) acc[m] = 0.0f;
    // GU groups per iteration: their packed words and coefficients are requested before the first popcount.  Two groups
    // in flight help when the grid is small (one group per warp in flight left the weight stream latency-bound:
    // 10.2 -> 8.3 us at 4096 x 4096); with many CTAs the extra registers cost occupancy (17.7 -> 26 us at 14336 x 4096).
    for (int g = g0; g < g1; g += GU) {
        uint32_t rw[GU][8];
        float cr[GU];
#pragma unroll
        for (int u = 0; u < GU; ++u) {
            const bool on = live && (g + u < g1);
#pragma unroll
            for (int kw = 0; kw < 8; ++kw) rw[u][kw] = on ? __ldcs(r_bvr + ((size_t)((g + u) * 8 + kw) * N + n) * RS + b) : 0u;
            cr[u] = 0.0f;
            if (on) {
                const size_t e = (size_t)(g + u) * N + n;
                const size_t line = (r_idx_bytes == 1) ? reinterpret_cast<const uint8_t*>(r_idx)[e]
                                                       : reinterpret_cast<const uint16_t*>(r_idx)[e];
                cr[u] = __half2float(r_cache[line * RS + b]);
            }
        }
#pragma unroll
        for (int u = 0; u < GU; ++u) {
            if (g + u < g1) {
#pragma unroll
                for (int m = 0; m < PM_MT; ++m) {
                    if (m < mt) {
                        float s = 0.0f;
#pragma unroll
                        for (int a = 0; a < LS; ++a) {
                            int cnt = 0;
#pragma unroll
                            for (int kw = 0; kw < 8; ++kw) cnt += __popc(lw[(((g + u) * 8 + kw) * PM_MT + m) * LS + a] & rw[u][kw]);
                            s += lc[((g + u) * PM_MT + m) * LS + a] * (float)cnt;
                        }
                        acc[m] += cr[u] * s;
                    }
                }
            }
        }
    }
    // planes of a row sit in neighbouring lanes; then the K quarters meet in shared memory, in a fixed order
#pragma unroll
    for (int m = 0; m < PM_MT; ++m) {
#pragma unroll
        for (int o = RP / 2; o; o >>= 1) acc[m] += __shfl_xor_sync(0xffffffffu, acc[m], o);
        if (b == 0) red[((rb * PM_KQ + kq) * PM_MT + m) * ROWS + lane / RP] = acc[m];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < PM_RB * mt * ROWS; i += PM_THREADS) {
        const int r = i % ROWS, m = (i / ROWS) % mt, rbb = i / (ROWS * mt);
        const int nn = ((int)blockIdx.x * PM_RB + rbb) * ROWS + r;
        if (nn >= N) continue;
        float v = 0.0f;
#pragma unroll
        for (int q = 0; q < PM_KQ; ++q) v += red[((rbb * PM_KQ + q) * PM_MT + m) * ROWS + r];
        if (bias) v += __half2float(bias[nn]);
        y[(size_t)(m0 + m) * N + nn] = __float2half_rn(v);
    }
}

template <int LS, int RS>
static int popc_launch(const uint32_t* l_bvr, const void* l_idx, int lib, const __half* l_cache, const uint32_t* r_bvr,
                       const void* r_idx, int rib, const __half* r_cache, const __half* bias, __half* y, int M, int N, int K,
                       cudaStream_t st) {
    constexpr int RP = (RS == 3) ? 4 : RS;
    constexpr int ROWS = 32 / RP;
    const size_t smem = (size_t)(K / 32) * PM_MT * LS * 4 + (size_t)(K / 256) * PM_MT * LS * 4 +
                        (size_t)PM_RB * PM_KQ * PM_MT * ROWS * 4;
    if (smem > 200 * 1024) return SBVR_ERR_UNSUPPORTED;
    static SmemOnce once1, once2;
    int rc_once = set_max_smem_once(once1, popc_mm_kernel<LS, RS, 1>, 200 * 1024);
    if (rc_once) return rc_once;
    rc_once = set_max_smem_once(once2, popc_mm_kernel<LS, RS, 2>, 200 * 1024);
    if (rc_once) return rc_once;
    const int blocks = (N + PM_RB * ROWS - 1) / (PM_RB * ROWS);
    int dev = 0;
    SBVR_CUDA_TRY(cudaGetDevice(&dev));
    DeviceInfo di;
    const int rc_di = device_info(dev, &di);
    if (rc_di) return rc_di;
    const bool two = blocks <= 3 * di.sm_count;
    for (int m0 = 0; m0 < M; m0 += PM_MT) {
        if (two)
            SBVR_CUDA_TRY(launch_pdl(popc_mm_kernel<LS, RS, 2>, dim3(blocks), dim3(PM_THREADS), smem, st, l_bvr, l_idx, lib, l_cache,
                                     r_bvr, r_idx, rib, r_cache, bias, y, M, m0, N, K));
        else
            SBVR_CUDA_TRY(launch_pdl(popc_mm_kernel<LS, RS, 1>, dim3(blocks), dim3(PM_THREADS), smem, st, l_bvr, l_idx, lib, l_cache,
                                     r_bvr, r_idx, rib, r_cache, bias, y, M, m0, N, K));
    }
    return SBVR_OK;
}

}  // namespace sbvr

using namespace sbvr;

extern "C" int sbvr_popc_mm_f16(const uint32_t* l_bvr, const void* l_idx, int l_idx_bytes, const void* l_cache, int Cl, int LS,
                                 const uint32_t* r_bvr, const void* r_idx, int r_idx_bytes, const void* r_cache, int Cr, int RS,
                                 const void* bias, void* y, int M, int N, int K, sbvr_stream_t stream) {
    if (!l_bvr || !l_idx || !l_cache || !r_bvr || !r_idx || !r_cache || !y) return SBVR_ERR_BAD_ARG;
    if (M < 1 || N < 1 || K < 1 || Cl < 1 || Cr < 1) return SBVR_ERR_BAD_ARG;
    if ((l_idx_bytes != 1 && l_idx_bytes != 2) || (r_idx_bytes != 1 && r_idx_bytes != 2)) return SBVR_ERR_BAD_ARG;
    if ((l_idx_bytes == 1 && Cl > 256) || (r_idx_bytes == 1 && Cr > 256) || Cl > 65536 || Cr > 65536) return SBVR_ERR_BAD_ARG;
    if (K % 256) return SBVR_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(l_bvr) | reinterpret_cast<uintptr_t>(r_bvr)) & 3) return SBVR_ERR_ALIGN;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const __half* lc = reinterpret_cast<const __half*>(l_cache);
    const __half* rc = reinterpret_cast<const __half*>(r_cache);
    const __half* bh = reinterpret_cast<const __half*>(bias);
    __half* yh = reinterpret_cast<__half*>(y);
#define SBVR_PM(L_, R_)                                                                                              \
    if (LS == L_ && RS == R_)                                                                                        \
        return popc_launch<L_, R_>(l_bvr, l_idx, l_idx_bytes, lc, r_bvr, r_idx, r_idx_bytes, rc, bh, yh, M, N, K, st)
    SBVR_PM(2, 2);
    SBVR_PM(2, 3);
    SBVR_PM(2, 4);
    SBVR_PM(3, 2);
    SBVR_PM(3, 3);
    SBVR_PM(3, 4);
    SBVR_PM(4, 2);
    SBVR_PM(4, 3);
    SBVR_PM(4, 4);
#undef SBVR_PM
    return SBVR_ERR_UNSUPPORTED;
}
