// sbvr_decode_f16: packed bit-planes + coefficients -> dense fp16 weight, bit-exact with the
// reference decoder (`sbvr.decode`, reference sbvr/core.py:926-949): for every element the
// coefficients of its set planes are summed in fp32 in plane order (products with 0/1 are exact)
// and rounded to fp16 once (round-to-nearest-even).  No fast-math, no flush-to-zero: about 0.5 %
// of N(0, 0.01) coefficients are fp16 subnormals and must survive.
//
// HBM-bound: reads S/8 + idx bytes per element, writes 2 bytes per element.
// One thread decodes the 32 elements of one (row n, word kw) pair.  A warp takes 32 consecutive
// rows at one kw, so its plane loads are one contiguous run of 32*S words; each lane then writes
// 64 contiguous bytes (two full 32-byte sectors) of its own row.
#include "common.cuh"

namespace sbvr {

template <int S>
__global__ void __launch_bounds__(256) decode_kernel(const uint32_t* __restrict__ bvr, const void* __restrict__ idx,
                                                     int idx_bytes, const __half* __restrict__ coeff,
                                                     __half* __restrict__ W, int ldw, int N, int K, int Kout, int G) {
    const int n = blockIdx.x * 32 + (threadIdx.x & 31);
    const int kw = blockIdx.y * 8 + (threadIdx.x >> 5);
    const int KW = K / 32;
    if (n >= N || kw >= KW || kw * 32 >= Kout) return;

    uint32_t w[S];
    const uint32_t* src = bvr + ((size_t)kw * N + n) * S;
#pragma unroll
    for (int s = 0; s < S; ++s) w[s] = __ldg(src + s);

    const int g = (kw * 32) / G;
    const __half* line = coeff_line(idx, idx_bytes, coeff, g, n, N, S);
    float c[S];
#pragma unroll
    for (int s = 0; s < S; ++s) c[s] = __half2float(line[s]);   // exact, subnormals included

    __half* dst = W + (size_t)n * ldw + (size_t)kw * 32;
    const bool vec = ((((size_t)n * ldw + (size_t)kw * 32) & 7) == 0) && ((reinterpret_cast<uintptr_t>(W) & 15) == 0);
#pragma unroll
    for (int j8 = 0; j8 < 4; ++j8) {
        __half2 out[4];
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
            float v[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int j = j8 * 8 + jj * 2 + e;
                float acc = 0.0f;
#pragma unroll
                for (int s = 0; s < S; ++s)
                    if ((w[s] >> j) & 1u) acc = __fadd_rn(acc, c[s]);
                v[e] = acc;
            }
            out[jj] = __halves2half2(__float2half_rn(v[0]), __float2half_rn(v[1]));
        }
        if (vec && kw * 32 + j8 * 8 + 8 <= Kout) {
            *reinterpret_cast<uint4*>(dst + j8 * 8) = *reinterpret_cast<uint4*>(out);
        } else {
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
                const int k = kw * 32 + j8 * 8 + jj * 2;
                if (k < Kout) dst[j8 * 8 + jj * 2] = __low2half(out[jj]);
                if (k + 1 < Kout) dst[j8 * 8 + jj * 2 + 1] = __high2half(out[jj]);
            }
        }
    }
}

int launch_decode(const PackedW& w, __half* W, int ldw, int Kout, cudaStream_t st) {
    dim3 grid((w.N + 31) / 32, (w.K / 32 + 7) / 8);
    dim3 block(256);
#define SBVR_DECODE_CASE(SS)                                                                                        \
    case SS:                                                                                                         \
        decode_kernel<SS><<<grid, block, 0, st>>>(w.bvr, w.idx, w.idx_bytes, w.coeff, W, ldw, w.N, w.K, Kout,  \
                                                  w.G);        \
        break;
    switch (w.S) {
        SBVR_DECODE_CASE(1)
        SBVR_DECODE_CASE(2)
        SBVR_DECODE_CASE(3)
        SBVR_DECODE_CASE(4)
        SBVR_DECODE_CASE(5)
        SBVR_DECODE_CASE(6)
        SBVR_DECODE_CASE(7)
        SBVR_DECODE_CASE(8)
        default:
            return SBVR_ERR_UNSUPPORTED;
    }
#undef SBVR_DECODE_CASE
    SBVR_CUDA_TRY(cudaGetLastError());
    return SBVR_OK;
}

}  // namespace sbvr
