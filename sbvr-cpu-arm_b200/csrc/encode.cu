// The arithmetic core of the SBVR encoder: for groups of 256 fp16 values and candidate coefficient lines, the mean
// squared error of representing every value by the nearest of the 2^S sums a line can form, the selector of that
// nearest sum, and the packing of selectors into bit-planes.
//
// The reference evaluates a candidate set by materialising diff[c, e, j] = (data[e] - point[c, j])^2 as an fp16 tensor,
// taking the minimum over j and the fp32 mean over e (sbvr/core.py:485-500, `_data_diff_min_mse`; points =
// search_matrix @ bin_combs^T, :520-521), one group at a time in a Python loop.  Here one thread owns one (group,
// candidate) pair, keeps the 2^S points in registers and streams the group from shared memory: nothing of size
// candidates x 256 x 2^S ever exists, and many groups are evaluated against the codebook in one launch.
//
// Arithmetic, step for step as the reference's tensor ops round:
//   point[j] = fp16( fp32 sum over s, in order, of line[s] * bit_s(j) ),  bit_s(j) = (j >> (S-1-s)) & 1  (bin_combs, :345-351)
//   diff     = fp16( fp16(d - point)^2 )                                  (fp16 subtraction, fp16 square)
//   m[e]     = min over j of diff (the first j on ties)                   (fp16 min)
//   mse      = (fp32 sum over e of m[e]) / 256                            (`.to(float32).mean`)
#include "common.cuh"

namespace sbvr {

constexpr int ENC_G = 256;            // group length (the reference enforces 256, sbvr/core.py:222)
constexpr int ENC_THREADS = 128;

template <int S>
__device__ __forceinline__ void enc_points(const __half* line, __half2 (&pt)[1 << S]) {
    float c[S];
#pragma unroll
    for (int s = 0; s < S; ++s) c[s] = __half2float(line[s]);
#pragma unroll
    for (int j = 0; j < (1 << S); ++j) {
        float v = 0.0f;
#pragma unroll
        for (int s = 0; s < S; ++s)
            if ((j >> (S - 1 - s)) & 1) v += c[s];
        pt[j] = __half2half2(__float2half_rn(v));
    }
}

// mse[b, c] for b < B groups and c < L lines.  grid = (ceil(L / 128), B).
template <int S>
__global__ void __launch_bounds__(ENC_THREADS) encode_mse_kernel(const __half* __restrict__ data,
                                                                 const __half* __restrict__ lines, int L,
                                                                 float* __restrict__ mse) {
    __shared__ __align__(16) __half2 ds[ENC_G / 2];
    const int b = blockIdx.y;
    for (int i = threadIdx.x; i < ENC_G / 2; i += ENC_THREADS)
        ds[i] = reinterpret_cast<const __half2*>(data + (size_t)b * ENC_G)[i];
    __syncthreads();
    const int c = blockIdx.x * ENC_THREADS + threadIdx.x;
    if (c >= L) return;
    __half2 pt[1 << S];
    enc_points<S>(lines + (size_t)c * S, pt);
    float s0 = 0.0f, s1 = 0.0f;
#pragma unroll 4
    for (int i = 0; i < ENC_G / 2; ++i) {
        const __half2 d = ds[i];
        __half2 t = __hsub2(d, pt[0]);
        __half2 m = __hmul2(t, t);
#pragma unroll
        for (int j = 1; j < (1 << S); ++j) {
            t = __hsub2(d, pt[j]);
            m = __hmin2(m, __hmul2(t, t));
        }
        const float2 f = __half22float2(m);
        s0 += f.x, s1 += f.y;
    }
    mse[(size_t)b * L + c] = (s0 + s1) * (1.0f / ENC_G);
}

// sel[b, e] = first j minimising fp16((d - point_j)^2) for the line `which[b]` of `lines`.  grid = B, block = 256.
template <int S>
__global__ void __launch_bounds__(ENC_G) encode_select_kernel(const __half* __restrict__ data,
                                                              const __half* __restrict__ lines,
                                                              const int* __restrict__ which, uint8_t* __restrict__ sel) {
    const int b = blockIdx.x, e = threadIdx.x;
    __half2 pt[1 << S];
    enc_points<S>(lines + (size_t)which[b] * S, pt);
    const __half d = data[(size_t)b * ENC_G + e];
    int best = 0;
    __half t = __hsub(d, __low2half(pt[0]));
    __half bm = __hmul(t, t);
#pragma unroll
    for (int j = 1; j < (1 << S); ++j) {
        t = __hsub(d, __low2half(pt[j]));
        const __half v = __hmul(t, t);
        if (__hlt(v, bm)) bm = v, best = j;
    }
    sel[(size_t)b * ENC_G + e] = (uint8_t)best;
}

// Selectors [N, Kp] -> bit-planes bvr[Kp/32, N, S]: bit i of word (kw, n, s) = bit (S-1-s) of sel[n, 32 kw + i]
// (`_change_coeff_sel_to_bvr` + layout change, sbvr/core.py:842-876, :783).  One warp per word position.
__global__ void encode_pack_kernel(const uint8_t* __restrict__ sel, int N, int KW, int S, uint32_t* __restrict__ bvr) {
    const int lane = threadIdx.x & 31;
    const size_t word = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);     // kw * N + n
    if (word >= (size_t)KW * N) return;
    const int kw = (int)(word / N), n = (int)(word % N);
    const uint32_t v = sel[((size_t)n * KW + kw) * 32 + lane];
    uint32_t mine = 0;
    for (int s = 0; s < S; ++s) {
        const uint32_t w = __ballot_sync(0xffffffffu, (v >> (S - 1 - s)) & 1u);
        if (lane == s) mine = w;
    }
    if (lane < S) bvr[word * S + lane] = mine;
}

}  // namespace sbvr

using namespace sbvr;

extern "C" int sbvr_encode_mse_f16(const void* data, int groups, const void* lines, int L, int S, float* mse,
                                    sbvr_stream_t stream) {
    if (!data || !lines || !mse || groups < 1 || L < 1) return SBVR_ERR_BAD_ARG;
    if (groups > 65535) return SBVR_ERR_SHAPE;
    if (reinterpret_cast<uintptr_t>(data) & 3) return SBVR_ERR_ALIGN;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const dim3 grid((L + ENC_THREADS - 1) / ENC_THREADS, groups);
    const __half* d = reinterpret_cast<const __half*>(data);
    const __half* l = reinterpret_cast<const __half*>(lines);
    switch (S) {
        case 1: encode_mse_kernel<1><<<grid, ENC_THREADS, 0, st>>>(d, l, L, mse); break;
        case 2: encode_mse_kernel<2><<<grid, ENC_THREADS, 0, st>>>(d, l, L, mse); break;
        case 3: encode_mse_kernel<3><<<grid, ENC_THREADS, 0, st>>>(d, l, L, mse); break;
        case 4: encode_mse_kernel<4><<<grid, ENC_THREADS, 0, st>>>(d, l, L, mse); break;
        default: return SBVR_ERR_UNSUPPORTED;
    }
    SBVR_CUDA_TRY(cudaGetLastError());
    return SBVR_OK;
}

extern "C" int sbvr_encode_select_f16(const void* data, int groups, const void* lines, const int* which, int S,
                                       uint8_t* sel, sbvr_stream_t stream) {
    if (!data || !lines || !which || !sel || groups < 1) return SBVR_ERR_BAD_ARG;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const __half* d = reinterpret_cast<const __half*>(data);
    const __half* l = reinterpret_cast<const __half*>(lines);
    switch (S) {
        case 1: encode_select_kernel<1><<<groups, ENC_G, 0, st>>>(d, l, which, sel); break;
        case 2: encode_select_kernel<2><<<groups, ENC_G, 0, st>>>(d, l, which, sel); break;
        case 3: encode_select_kernel<3><<<groups, ENC_G, 0, st>>>(d, l, which, sel); break;
        case 4: encode_select_kernel<4><<<groups, ENC_G, 0, st>>>(d, l, which, sel); break;
        default: return SBVR_ERR_UNSUPPORTED;
    }
    SBVR_CUDA_TRY(cudaGetLastError());
    return SBVR_OK;
}

extern "C" int sbvr_encode_pack(const uint8_t* sel, int N, int Kp, int S, uint32_t* bvr, sbvr_stream_t stream) {
    if (!sel || !bvr || N < 1 || Kp < 32 || S < 1 || S > 8) return SBVR_ERR_BAD_ARG;
    if (Kp % 32) return SBVR_ERR_SHAPE;
    const int KW = Kp / 32;
    const size_t words = (size_t)KW * N;
    const size_t blocks = (words + 7) / 8;
    if (blocks > 0x7fffffffu) return SBVR_ERR_SHAPE;
    encode_pack_kernel<<<(unsigned int)blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(sel, N, KW, S, bvr);
    SBVR_CUDA_TRY(cudaGetLastError());
    return SBVR_OK;
}
