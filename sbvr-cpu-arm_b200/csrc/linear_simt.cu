// General SBVR linear on CUDA cores: y[M, N] = fp16(x . W^T + bias) for any S <= 8, G a multiple of
// 32, any index form, any M.  It is the path for shapes the tensor-core kernels do not cover and
// the in-library cross-check for them.  Replaces cuda_row_deq_mm_T (reference
// sbvr/kernels/sbvr_kernel.cu:121-191): same arithmetic (dequantise an element as the fp32 sum of
// its selected coefficients, multiply by the activation, accumulate in fp32, bias, convert last),
// but on the non-transposed weight layout and with coalesced plane loads.
//
// Block = 32 output rows (one per lane) x 8 warps that split K; activations of up to MB rows are
// staged in shared memory in chunks of KC elements and read as broadcasts.
#include "common.cuh"

namespace sbvr {

constexpr int SIMT_KC = 2048;   // activation elements staged per chunk
constexpr int SIMT_MB = 4;      // activation rows per block

template <int S>
__global__ void __launch_bounds__(256) linear_simt_kernel(const __half* __restrict__ x, const uint32_t* __restrict__ bvr,
                                                          const void* __restrict__ idx, int idx_bytes,
                                                          const __half* __restrict__ coeff,
                                                          const __half* __restrict__ bias, __half* __restrict__ y,
                                                          int M, int N, int K, int G) {
    __shared__ __align__(16) __half xs[SIMT_MB][SIMT_KC];
    __shared__ float red[8][SIMT_MB][32];

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n = blockIdx.x * 32 + lane;
    const int m0 = blockIdx.y * SIMT_MB;
    const bool live = n < N;

    float acc[SIMT_MB];
#pragma unroll
    for (int m = 0; m < SIMT_MB; ++m) acc[m] = 0.0f;

    for (int kc0 = 0; kc0 < K; kc0 += SIMT_KC) {
        const int kc = min(SIMT_KC, K - kc0);
        __syncthreads();
        for (int i = threadIdx.x; i < SIMT_MB * (SIMT_KC / 2); i += 256) {
            const int m = i / (SIMT_KC / 2), k2 = (i % (SIMT_KC / 2)) * 2;
            __half2 v = __float2half2_rn(0.0f);
            if (m0 + m < M && k2 < kc) v = *reinterpret_cast<const __half2*>(x + (size_t)(m0 + m) * K + kc0 + k2);
            *reinterpret_cast<__half2*>(&xs[m][k2]) = v;
        }
        __syncthreads();
        if (!live) continue;
        for (int kwl = warp; kwl < kc / 32; kwl += 8) {
            const int kw = kc0 / 32 + kwl;
            uint32_t w[S];
            const uint32_t* src = bvr + ((size_t)kw * N + n) * S;
#pragma unroll
            for (int s = 0; s < S; ++s) w[s] = __ldg(src + s);
            const __half* line = coeff_line(idx, idx_bytes, coeff, (kw * 32) / G, n, N, S);
            float c[S];
#pragma unroll
            for (int s = 0; s < S; ++s) c[s] = __half2float(line[s]);
#pragma unroll 4
            for (int j = 0; j < 32; j += 2) {
                float w0 = 0.0f, w1 = 0.0f;
#pragma unroll
                for (int s = 0; s < S; ++s) {
                    if ((w[s] >> j) & 1u) w0 += c[s];
                    if ((w[s] >> (j + 1)) & 1u) w1 += c[s];
                }
#pragma unroll
                for (int m = 0; m < SIMT_MB; ++m) {
                    const float2 xv = __half22float2(*reinterpret_cast<const __half2*>(&xs[m][kwl * 32 + j]));
                    acc[m] = fmaf(xv.x, w0, acc[m]);
                    acc[m] = fmaf(xv.y, w1, acc[m]);
                }
            }
        }
    }
#pragma unroll
    for (int m = 0; m < SIMT_MB; ++m) red[warp][m][lane] = acc[m];
    __syncthreads();
    if (warp == 0 && live) {
        const float b = bias ? __half2float(bias[n]) : 0.0f;
#pragma unroll
        for (int m = 0; m < SIMT_MB; ++m) {
            if (m0 + m >= M) break;
            float v = 0.0f;
#pragma unroll
            for (int wi = 0; wi < 8; ++wi) v += red[wi][m][lane];
            y[(size_t)(m0 + m) * N + n] = __float2half_rn(v + b);
        }
    }
}

int launch_linear_simt(const __half* x, const PackedW& w, const __half* bias, __half* y, int M, cudaStream_t st) {
    dim3 grid((w.N + 31) / 32, (M + SIMT_MB - 1) / SIMT_MB);
    dim3 block(256);
    if (grid.y > 65535) return SBVR_ERR_SHAPE;
#define SBVR_SIMT_CASE(SS)                                                                                           \
    case SS:                                                                                                         \
        linear_simt_kernel<SS><<<grid, block, 0, st>>>(x, w.bvr, w.idx, w.idx_bytes, w.coeff, bias, y, M, w.N, w.K,  \
                                                       w.G);                                                         \
        break;
    switch (w.S) {
        SBVR_SIMT_CASE(1)
        SBVR_SIMT_CASE(2)
        SBVR_SIMT_CASE(3)
        SBVR_SIMT_CASE(4)
        SBVR_SIMT_CASE(5)
        SBVR_SIMT_CASE(6)
        SBVR_SIMT_CASE(7)
        SBVR_SIMT_CASE(8)
        default:
            return SBVR_ERR_UNSUPPORTED;
    }
#undef SBVR_SIMT_CASE
    SBVR_CUDA_TRY(cudaGetLastError());
    return SBVR_OK;
}

}  // namespace sbvr
