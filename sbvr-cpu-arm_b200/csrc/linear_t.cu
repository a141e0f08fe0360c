// SBVR linear on the TRANSPOSED ("row-dequant") weight encoding: the weight was encoded as W^T, so a packed word
// holds 32 consecutive OUTPUT columns n of one input k and the groups of G run along n:
//
//     bvr_t  uint32 [N/32, K, S]      bit (n % 32) of word (n / 32, k, s) = plane s of element (k, n)
//     idx_t  u8|u16 [N/G, K]          codebook line of (group of G outputs, k)
//     y[m, n] = fp16( bias[n] + sum_k x[m, k] * sum_s c[idx_t[n / G, k]][s] * bit_s[n, k] )        (fp32 throughout)
//
// Replaces cuda_row_deq_mm_T / cuda_row_deq_wo_shfl_mm_T / cuda_1xtN_rd_WP8_TBW4_NS4 (reference
// sbvr/kernels/sbvr_kernel.cu:121-191, :193-254, :284-359; launcher :876-912, binding sbvr/kernels/sbvr_ops.cpp:79-120)
// with the same arithmetic: the dequantised element is the fp32 sum of its selected coefficients (not rounded to
// fp16), products and sums are fp32, the bias is added in fp32 and the result converted once.
//
// Mapping.  The reference gives a warp one word and lets every lane pick its bit, so each k costs a broadcast and the
// word is read once per lane.  Here a THREAD owns one k at a time and all 32 outputs of the word: the lanes of a warp
// read 32 consecutive k of one word row (S * 128 contiguous bytes, one 16-byte load per lane for S = 4), the codebook
// index of (group, k) and the activation, and add x * c_s to the accumulators whose bit is set: one predicated add per
// plane bit, no shifts (with several activation rows the element is dequantised once and costs one FMA per row).
// 32 fp32 accumulators per activation row live in registers; at the end a butterfly
// reduce-scatter over the lanes (31 shuffles per row, a fixed tree) leaves the sum of output n = lane in each lane, the
// warps of the block are added in order through shared memory.  A block covers one word row (32 outputs) and a
// contiguous part of K; when K is split over several blocks (small N), the partial sums go to the workspace and the
// block that arrives last at the word row's counter adds them in part order: the result never depends on timing.
// The loop is bound by instruction issue (2 * S * 32 thread instructions per packed word), not by HBM.
#include "common.cuh"

namespace sbvr {

constexpr int LT_THREADS = 256;
constexpr int LT_WARPS = LT_THREADS / 32;

struct LtParams {
    const __half* x;          // [M, K]
    const uint32_t* bvr;      // [N/32, K, S]
    const void* idx;          // [N/G, K]
    const __half* coeff;      // [C, S]
    const __half* bias;       // [N] or NULL
    __half* y;                // [M, N]
    float* part;              // [KS, MT, N] partial sums (KS > 1)
    unsigned int* counters;   // [N/32], zero between launches (KS > 1)
    int rows;                 // activation rows of this launch (<= MT)
    int N, K, g32, kchunk, KS;
};

template <int S>
__device__ __forceinline__ void lt_load_words(const uint32_t* p, uint32_t (&w)[S]) {
    if constexpr (S == 4) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(p));
        w[0] = v.x, w[1] = v.y, w[2] = v.z, w[3] = v.w;
    } else if constexpr (S == 2) {
        const uint2 v = __ldg(reinterpret_cast<const uint2*>(p));
        w[0] = v.x, w[1] = v.y;
    } else {
#pragma unroll
        for (int s = 0; s < S; ++s) w[s] = __ldg(p + s);
    }
}

template <int S>
__device__ __forceinline__ void lt_load_coef(const __half* line, float (&c)[S]) {
    if constexpr (S == 4) {
        const uint2 v = __ldg(reinterpret_cast<const uint2*>(line));
        const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&v.x));
        const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&v.y));
        c[0] = a.x, c[1] = a.y, c[2] = b.x, c[3] = b.y;
    } else if constexpr (S == 2) {
        const uint32_t v = __ldg(reinterpret_cast<const uint32_t*>(line));
        const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&v));
        c[0] = a.x, c[1] = a.y;
    } else {
#pragma unroll
        for (int s = 0; s < S; ++s) c[s] = __half2float(__ldg(line + s));
    }
}

template <int S, int MT, int IDXB>
__global__ void __launch_bounds__(LT_THREADS) linear_t_kernel(const LtParams p) {
    __shared__ float red[LT_WARPS][MT][32];
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nw = blockIdx.x, ks = blockIdx.y;
    const int K = p.K;
    const int k0 = ks * p.kchunk, k1 = min(K, k0 + p.kchunk);
    const uint32_t* wrow = p.bvr + (size_t)nw * K * S;
    const size_t irow = (size_t)(nw / p.g32) * K;

    float acc[MT][32];
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int n = 0; n < 32; ++n) acc[m][n] = 0.0f;

    // what one k needs; the next k's loads are issued before the current one is used
    uint32_t w[S], wn[S];
    uint32_t ci = 0, cin = 0;
    auto load_idx = [&](int k) -> uint32_t {
        return (IDXB == 1) ? (uint32_t)__ldg(reinterpret_cast<const uint8_t*>(p.idx) + irow + k)
                           : (uint32_t)__ldg(reinterpret_cast<const uint16_t*>(p.idx) + irow + k);
    };
    int k = k0 + (int)threadIdx.x;
    if (k < k1) {                                  // weights and indices do not depend on the previous kernel
        lt_load_words<S>(wrow + (size_t)k * S, w);
        ci = load_idx(k);
    }
    pdl_wait();                                    // the activations may come from the previous kernel on the stream
    for (; k < k1; k += LT_THREADS) {
        const int kn = k + LT_THREADS;
        if (kn < k1) {
            lt_load_words<S>(wrow + (size_t)kn * S, wn);
            cin = load_idx(kn);
        }
        float c[S];
        lt_load_coef<S>(p.coeff + (size_t)ci * S, c);
        float xv[MT];
#pragma unroll
        for (int m = 0; m < MT; ++m) xv[m] = __half2float(p.x[(size_t)min(m, p.rows - 1) * K + k]);
        if constexpr (MT == 1) {                   // one row: add x * c_s where the bit is set, S predicated adds per output
#pragma unroll
            for (int s = 0; s < S; ++s) {
                const float xc = xv[0] * c[s];
#pragma unroll
                for (int n = 0; n < 32; ++n)
                    if (w[s] & (1u << n)) acc[0][n] += xc;
            }
        } else {                                   // several rows: dequantise the element once, one FMA per row
#pragma unroll
            for (int n = 0; n < 32; ++n) {
                float wv = 0.0f;
#pragma unroll
                for (int s = 0; s < S; ++s)
                    if (w[s] & (1u << n)) wv += c[s];
#pragma unroll
                for (int m = 0; m < MT; ++m) acc[m][n] = fmaf(xv[m], wv, acc[m][n]);
            }
        }
#pragma unroll
        for (int s = 0; s < S; ++s) w[s] = wn[s];
        ci = cin;
    }

    // lanes -> outputs: after the step with offset o a lane keeps the accumulators whose bit o of n equals its own
#pragma unroll
    for (int m = 0; m < MT; ++m) {
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) {
            const bool up = (lane & o) != 0;
#pragma unroll
            for (int i = 0; i < o; ++i) {
                const float keep = up ? acc[m][i + o] : acc[m][i];
                const float send = up ? acc[m][i] : acc[m][i + o];
                acc[m][i] = keep + __shfl_xor_sync(0xffffffffu, send, o);
            }
        }
        red[warp][m][lane] = acc[m][0];            // output n = nw * 32 + lane
    }
    __syncthreads();
    if (warp != 0) return;
    const int n = nw * 32 + lane;
    const float b = p.bias ? __half2float(p.bias[n]) : 0.0f;
    float v[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        v[m] = 0.0f;
#pragma unroll
        for (int wi = 0; wi < LT_WARPS; ++wi) v[m] += red[wi][m][lane];
    }
    if (p.KS == 1) {
#pragma unroll
        for (int m = 0; m < MT; ++m)
            if (m < p.rows) p.y[(size_t)m * p.N + n] = __float2half_rn(v[m] + b);
        return;
    }
#pragma unroll
    for (int m = 0; m < MT; ++m) p.part[((size_t)ks * MT + m) * p.N + n] = v[m];
    __threadfence();
    __syncwarp();
    unsigned int last = 0;
    if (lane == 0) last = (atomicAdd(p.counters + nw, 1u) == (unsigned int)(p.KS - 1)) ? 1u : 0u;
    last = __shfl_sync(0xffffffffu, last, 0);
    if (!last) return;
    __threadfence();
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        if (m >= p.rows) break;
        float t = 0.0f;
        for (int q = 0; q < p.KS; ++q) t += __ldcg(p.part + ((size_t)q * MT + m) * p.N + n);
        p.y[(size_t)m * p.N + n] = __float2half_rn(t + b);
    }
    if (lane == 0) p.counters[nw] = 0u;            // ready for the next launch
}

template <int S, int MT>
static int lt_launch_idx(const LtParams& p, int idxb, dim3 grid, cudaStream_t st) {
    if (idxb == 1)
        SBVR_CUDA_TRY(launch_pdl(linear_t_kernel<S, MT, 1>, grid, dim3(LT_THREADS), 0, st, p));
    else
        SBVR_CUDA_TRY(launch_pdl(linear_t_kernel<S, MT, 2>, grid, dim3(LT_THREADS), 0, st, p));
    return SBVR_OK;
}
template <int S>
static int lt_launch_m(const LtParams& p, int mt, int idxb, dim3 grid, cudaStream_t st) {
    switch (mt) {
        case 1: return lt_launch_idx<S, 1>(p, idxb, grid, st);
        case 2: return lt_launch_idx<S, 2>(p, idxb, grid, st);
        default: return lt_launch_idx<S, 4>(p, idxb, grid, st);
    }
}

}  // namespace sbvr

using namespace sbvr;

extern "C" int sbvr_linear_t_f16(const void* x, const uint32_t* bvr_t, const void* coeff_idx, int idx_bytes,
                                  const void* coeff, int C, const void* bias, void* y, int M, int N, int K, int S, int G,
                                  sbvr_workspace_t* ws, sbvr_stream_t stream) {
    if (!x || !bvr_t || !coeff_idx || !coeff || !y || !ws) return SBVR_ERR_BAD_ARG;
    if (M < 1 || N < 1 || K < 1 || C < 1 || C > 65536) return SBVR_ERR_BAD_ARG;
    if ((idx_bytes != 1 && idx_bytes != 2) || (idx_bytes == 1 && C > 256)) return SBVR_ERR_BAD_ARG;
    if (S < 2 || S > 4) return SBVR_ERR_UNSUPPORTED;
    if (G < 32 || G % 32 || N % G) return SBVR_ERR_SHAPE;
    const uintptr_t walign = (S == 4) ? 15 : (S == 2) ? 7 : 3;
    const uintptr_t calign = (S == 4) ? 7 : (S == 2) ? 3 : 1;
    if ((reinterpret_cast<uintptr_t>(bvr_t) & walign) || (reinterpret_cast<uintptr_t>(coeff) & calign) ||
        (reinterpret_cast<uintptr_t>(x) & 1) || (reinterpret_cast<uintptr_t>(y) & 1) ||
        (idx_bytes == 2 && (reinterpret_cast<uintptr_t>(coeff_idx) & 1)))
        return SBVR_ERR_ALIGN;
    DeviceInfo di;
    const int rc = device_info(ws->device, &di);
    if (rc) return rc;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const int nwords = N / 32;
    // K is split over blocks while at most four blocks per SM exist (one resident wave at 64 registers per thread; measured
    // best on the Llama-3-8B layer shapes); parts are multiples of the block's 256 k
    const int mt_all = M >= 3 ? 4 : M;            // rows per launch as instantiated: 1, 2 or 4
    int KS = 4 * di.sm_count / nwords;             // rounded down: all blocks resident at once
    if (KS < 1) KS = 1;
    int kchunk = ((K + KS - 1) / KS + LT_THREADS - 1) / LT_THREADS * LT_THREADS;
    if (kchunk < 2 * LT_THREADS) kchunk = 2 * LT_THREADS;
    KS = (K + kchunk - 1) / kchunk;
    if (KS > 1 && (nwords > SBVR_WS_COUNTERS || (size_t)KS * mt_all * N * sizeof(float) > ws->dyn_bytes)) {
        KS = 1;
        kchunk = K;
    }
    LtParams p;
    p.bvr = bvr_t, p.idx = coeff_idx, p.coeff = reinterpret_cast<const __half*>(coeff);
    p.bias = reinterpret_cast<const __half*>(bias);
    p.part = reinterpret_cast<float*>(ws->dyn), p.counters = ws->counters;
    p.N = N, p.K = K, p.g32 = G / 32, p.kchunk = kchunk, p.KS = KS;
    const dim3 grid(nwords, KS);
    for (int m0 = 0; m0 < M; m0 += 4) {
        const int rows = (M - m0 < 4) ? M - m0 : 4;
        const int mt = rows >= 3 ? 4 : rows;
        p.x = reinterpret_cast<const __half*>(x) + (size_t)m0 * K;
        p.y = reinterpret_cast<__half*>(y) + (size_t)m0 * N;
        p.rows = rows;
        int r;
        switch (S) {
            case 2: r = lt_launch_m<2>(p, mt, idx_bytes, grid, st); break;
            case 3: r = lt_launch_m<3>(p, mt, idx_bytes, grid, st); break;
            default: r = lt_launch_m<4>(p, mt, idx_bytes, grid, st); break;
        }
        if (r) return r;
    }
    return SBVR_OK;
}
