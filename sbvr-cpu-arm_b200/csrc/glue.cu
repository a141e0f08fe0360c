// The small kernels between the SBVR linears of a Llama decoder layer, each one launch where the reference runs
// a chain of eager PyTorch ops (reference models/sbvr_llama.py): RMSNorm with the residual add folded in
// (:118-123, :395-406), rotary embedding + KV-cache append (:169-224, :330-336), attention over the cache for
// decode and prefill (:243-278), SiLU(gate) * up (:238-240), embedding lookup, greedy argmax.
// Rounding follows the reference where it is visible in fp16: RMSNorm multiplies by the weight after the cast
// to fp16; the rotary products and their sum are separate fp16 operations; SiLU is rounded to fp16 before the
// multiplication.  Attention keeps scores and probabilities in fp32 (the reference rounds the scores and the
// probabilities to fp16), which is inside the 1e-2 tolerance of the layer outputs.
#include "common.cuh"

namespace sbvr {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// ---------------------------------------------------------------------------------------------
// h_out = h_in (+ delta);  y = weight * fp16( h_out * rsqrt(mean(h_out^2) + eps) )        one CTA per row
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) add_rmsnorm_kernel(const __half* h_in, const __half* __restrict__ delta,
                                                          const __half* __restrict__ weight, __half* h_out,
                                                          __half* __restrict__ y, int hidden, float eps) {
    __shared__ float red[8];
    pdl_launch_dependents();
    pdl_wait();
    const size_t row = (size_t)blockIdx.x * hidden;
    const int nvec = hidden / 8;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
        uint4 a = *reinterpret_cast<const uint4*>(h_in + row + (size_t)i * 8);
        __half2* ah = reinterpret_cast<__half2*>(&a);
        if (delta) {
            const uint4 b = *reinterpret_cast<const uint4*>(delta + row + (size_t)i * 8);
            const __half2* bh = reinterpret_cast<const __half2*>(&b);
#pragma unroll
            for (int e = 0; e < 4; ++e) ah[e] = __hadd2(ah[e], bh[e]);
        }
        if (h_out) *reinterpret_cast<uint4*>(h_out + row + (size_t)i * 8) = a;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = __half22float2(ah[e]);
            ss += f.x * f.x + f.y * f.y;
        }
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int w = 0; w < 8; ++w) tot += (w < (int)(blockDim.x >> 5)) ? red[w] : 0.0f;
    const float rs = rsqrtf(tot / (float)hidden + eps);
    const __half* src = h_out ? h_out : h_in;      // written above by this same thread when h_out is set
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
        uint4 a = *reinterpret_cast<const uint4*>(src + row + (size_t)i * 8);
        if (!h_out && delta) {
            const uint4 b = *reinterpret_cast<const uint4*>(delta + row + (size_t)i * 8);
            __half2* ah2 = reinterpret_cast<__half2*>(&a);
            const __half2* bh = reinterpret_cast<const __half2*>(&b);
#pragma unroll
            for (int e = 0; e < 4; ++e) ah2[e] = __hadd2(ah2[e], bh[e]);
        }
        const uint4 wv = *reinterpret_cast<const uint4*>(weight + (size_t)i * 8);
        const __half2* ah = reinterpret_cast<const __half2*>(&a);
        const __half2* wh = reinterpret_cast<const __half2*>(&wv);
        uint4 o;
        __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = __half22float2(ah[e]);
            oh[e] = __hmul2(wh[e], __floats2half2_rn(f.x * rs, f.y * rs));
        }
        *reinterpret_cast<uint4*>(y + (size_t)blockIdx.x * hidden + (size_t)i * 8) = o;
    }
}

// ---------------------------------------------------------------------------------------------
// rotary embedding of q and k in place + append of k, v to the cache            one CTA per token
//   qkv row: [n_heads * d | n_kv * d | n_kv * d];  cache [seq, n_kv, max_ctx, d]
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) rope_append_kernel(__half* __restrict__ qkv, const int* __restrict__ positions,
                                                          const float* __restrict__ inv_freq, float attn_scaling,
                                                          __half* __restrict__ kcache, __half* __restrict__ vcache,
                                                          int tokens_per_seq, int n_heads, int n_kv, int d, int max_ctx) {
    __shared__ __half cs_s[2][256];                // cos, sin of this token's position for i < head_dim / 2 <= 256
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int seq = t / tokens_per_seq;
    const int half_d = d / 2;
    __half* row = qkv + (size_t)t * (n_heads + 2 * n_kv) * d;
    for (int i = threadIdx.x; i < half_d; i += blockDim.x) {       // the accurate cosf / sinf are the expensive part
        const float ang = (float)pos * inv_freq[i];
        cs_s[0][i] = __float2half_rn(cosf(ang) * attn_scaling);
        cs_s[1][i] = __float2half_rn(sinf(ang) * attn_scaling);
    }
    __syncthreads();
    const int rot_items = (n_heads + n_kv) * half_d;
    for (int it = threadIdx.x; it < rot_items; it += blockDim.x) {
        const int head = it / half_d, i = it - head * half_d;
        const __half c = cs_s[0][i], s = cs_s[1][i];
        __half* hp = row + (size_t)head * d;
        const __half x1 = hp[i], x2 = hp[i + half_d];
        const __half o1 = __hadd(__hmul(x1, c), __hmul(__hneg(x2), s));
        const __half o2 = __hadd(__hmul(x2, c), __hmul(x1, s));
        hp[i] = o1, hp[i + half_d] = o2;
        if (head >= n_heads && pos < max_ctx) {
            __half* kc = kcache + (((size_t)seq * n_kv + (head - n_heads)) * max_ctx + pos) * d;
            kc[i] = o1, kc[i + half_d] = o2;
        }
    }
    if (pos < max_ctx) {
        const __half* vrow = row + (size_t)(n_heads + n_kv) * d;
        for (int it = threadIdx.x; it < n_kv * d; it += blockDim.x) {
            const int head = it / d, i = it - head * d;
            vcache[(((size_t)seq * n_kv + head) * max_ctx + pos) * d + i] = vrow[it];
        }
    }
}

// ---------------------------------------------------------------------------------------------
// attention of one query token over cache positions [0, pos]; head_dim 128; grouped-query: the R = n_heads / n_kv
// query heads of a KV head are served together.   grid (tokens * n_kv, nsplit), 128 threads
//   nsplit == 1: writes out[t, head, :] fp16.   nsplit > 1: writes (max, sum, unnormalised acc) per split.
// ---------------------------------------------------------------------------------------------
constexpr int AT_D = 128;
constexpr int AT_RMAX = 8;

// `inv_freq` != NULL (decode, one token per sequence): the rotary embedding is applied here -- q on its way into shared
// memory; the token's own k by the CTA whose positions include it, which also appends k and v to the cache and
// takes them from shared memory (the cache rows are read through the read-only path).
template <int R>
__global__ void __launch_bounds__(128) attention_kernel(const __half* __restrict__ qkv, __half* kcache, __half* vcache,
                                                        const int* __restrict__ positions, __half* __restrict__ out,
                                                        float* __restrict__ part, int tokens_per_seq, int n_heads, int n_kv, int max_ctx, float scale,
                                                        int nsplit, const float* __restrict__ inv_freq, float attn_scaling) {
    __shared__ float qs[R][AT_D];
    __shared__ float wm[4][R], wl[4][R];
    __shared__ float wacc[4][R][AT_D];
    __shared__ __half cs_s[2][AT_D / 2];
    __shared__ __align__(16) __half knew[AT_D], vnew[AT_D];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x / n_kv, kvh = blockIdx.x - t * n_kv;
    const int split = blockIdx.y;
    const int seq = t / tokens_per_seq;
    const int pos = positions[t];
    const int ctx = min(pos + 1, max_ctx);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const __half* tok = qkv + (size_t)t * (n_heads + 2 * n_kv) * AT_D;
    const __half* qrow = tok + (size_t)kvh * R * AT_D;
    const int per = (ctx + nsplit - 1) / nsplit;
    const int p0 = split * per, p1 = min(ctx, p0 + per);
    __half* kb = kcache + ((size_t)seq * n_kv + kvh) * max_ctx * AT_D;
    __half* vb = vcache + ((size_t)seq * n_kv + kvh) * max_ctx * AT_D;
    const bool rope = inv_freq != nullptr;
    // position of the row that comes from shared memory instead of the cache (-1: none)
    const int own = (rope && pos < max_ctx && pos >= p0 && pos < p1) ? pos : -1;
    if (rope) {
        if (threadIdx.x < AT_D / 2) {
            const float ang = (float)pos * inv_freq[threadIdx.x];
            cs_s[0][threadIdx.x] = __float2half_rn(cosf(ang) * attn_scaling);
            cs_s[1][threadIdx.x] = __float2half_rn(sinf(ang) * attn_scaling);
        }
        __syncthreads();
        for (int i = threadIdx.x; i < R * AT_D; i += 128) {
            const int r = i / AT_D, dd = i % AT_D, i2 = dd % (AT_D / 2);
            const __half c = cs_s[0][i2], sn = cs_s[1][i2];
            const __half x = qrow[i];
            const __half y = (dd < AT_D / 2) ? __hneg(qrow[r * AT_D + dd + AT_D / 2]) : qrow[r * AT_D + dd - AT_D / 2];
            qs[r][dd] = __half2float(__hadd(__hmul(x, c), __hmul(y, sn))) * scale;
        }
        if (own >= 0) {                            // this CTA holds the new token's position
            const __half* krow = tok + (size_t)(n_heads + kvh) * AT_D;
            const __half* vrow = tok + (size_t)(n_heads + n_kv + kvh) * AT_D;
            const int dd = threadIdx.x, i2 = dd % (AT_D / 2);
            const __half c = cs_s[0][i2], sn = cs_s[1][i2];
            const __half y = (dd < AT_D / 2) ? __hneg(krow[dd + AT_D / 2]) : krow[dd - AT_D / 2];
            const __half kr1 = __hadd(__hmul(krow[dd], c), __hmul(y, sn));
            knew[dd] = kr1, vnew[dd] = vrow[dd];
            kb[(size_t)pos * AT_D + dd] = kr1;
            vb[(size_t)pos * AT_D + dd] = vrow[dd];
        }
    } else {
        for (int i = threadIdx.x; i < R * AT_D; i += 128) qs[i / AT_D][i % AT_D] = __half2float(qrow[i]) * scale;
    }
    __syncthreads();

    float m[R], l[R], acc[R][4];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        m[r] = -INFINITY, l[r] = 0.0f;
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[r][e] = 0.0f;
    }
    // The CTA's positions are cut into four contiguous quarters, one per warp; a warp takes up to 32 consecutive
    // positions at a time: lane <-> position for the scores, lane <-> 4 dims for P.V.
    const int quarter = (p1 - p0 + 3) / 4;
    const int w0 = min(p1, p0 + warp * quarter), w1 = min(p1, w0 + quarter);
    for (int base = w0; base < w1; base += 32) {
        const int p = base + lane;
        const int p1 = w1;                         // this warp's end (shadows the CTA's)
        float sc[R];
#pragma unroll
        for (int r = 0; r < R; ++r) sc[r] = 0.0f;
        if (p < p1) {
            const uint4* kr = reinterpret_cast<const uint4*>(kb + (size_t)p * AT_D);
            const uint4* ks = reinterpret_cast<const uint4*>(knew);
#pragma unroll
            for (int c = 0; c < AT_D / 8; ++c) {
                const uint4 kv = (p == own) ? ks[c] : __ldg(kr + c);
                const __half2* kh = reinterpret_cast<const __half2*>(&kv);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 f = __half22float2(kh[e]);
#pragma unroll
                    for (int r = 0; r < R; ++r) sc[r] += f.x * qs[r][c * 8 + 2 * e] + f.y * qs[r][c * 8 + 2 * e + 1];
                }
            }
        } else {
#pragma unroll
            for (int r = 0; r < R; ++r) sc[r] = -INFINITY;
        }
        // online softmax: new running maximum per head, rescale, then this chunk's weights
        float w[R];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            float cm = sc[r];
#pragma unroll
            for (int o = 16; o; o >>= 1) cm = fmaxf(cm, __shfl_xor_sync(0xffffffffu, cm, o));
            const float nm = fmaxf(m[r], cm);
            const float corr = (m[r] == -INFINITY) ? 0.0f : __expf(m[r] - nm);
            w[r] = (p < p1) ? __expf(sc[r] - nm) : 0.0f;
            l[r] = l[r] * corr + warp_sum(w[r]);
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[r][e] *= corr;
            m[r] = nm;
        }
        const int np = min(32, p1 - base);
        for (int j0 = 0; j0 < np; j0 += 8) {       // eight V rows in flight; rows past the end carry weight 0
            uint2 vv[8];
#pragma unroll
            for (int u = 0; u < 8; ++u)
                vv[u] = (base + j0 + u == own)
                            ? reinterpret_cast<const uint2*>(vnew)[lane]
                            : __ldg(reinterpret_cast<const uint2*>(vb + (size_t)min(base + j0 + u, max_ctx - 1) * AT_D) + lane);
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const __half2* vh = reinterpret_cast<const __half2*>(&vv[u]);
                const float2 f0 = __half22float2(vh[0]), f1 = __half22float2(vh[1]);
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const float wj = __shfl_sync(0xffffffffu, w[r], j0 + u);
                    acc[r][0] += wj * f0.x, acc[r][1] += wj * f0.y, acc[r][2] += wj * f1.x, acc[r][3] += wj * f1.y;
                }
            }
        }
    }
    // merge the four warps
#pragma unroll
    for (int r = 0; r < R; ++r) {
        if (lane == 0) wm[warp][r] = m[r], wl[warp][r] = l[r];
#pragma unroll
        for (int e = 0; e < 4; ++e) wacc[warp][r][lane * 4 + e] = acc[r][e];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < R * AT_D; i += 128) {
        const int r = i / AT_D, dd = i % AT_D;
        float gm = -INFINITY;
#pragma unroll
        for (int w4 = 0; w4 < 4; ++w4) gm = fmaxf(gm, wm[w4][r]);
        float gl = 0.0f, ga = 0.0f;
#pragma unroll
        for (int w4 = 0; w4 < 4; ++w4) {
            const float c = (wm[w4][r] == -INFINITY) ? 0.0f : __expf(wm[w4][r] - gm);
            gl += wl[w4][r] * c;
            ga += wacc[w4][r][dd] * c;
        }
        const int head = kvh * R + r;
        if (nsplit == 1) {
            out[((size_t)t * n_heads + head) * AT_D + dd] = __float2half_rn(gl > 0.0f ? ga / gl : 0.0f);
        } else {
            float* pp = part + (((size_t)t * n_heads + head) * nsplit + split) * (AT_D + 2);
            pp[2 + dd] = ga;
            if (dd == 0) pp[0] = gm, pp[1] = gl;
        }
    }
}

// merges the splits of one (token, head)                                   grid tokens * n_heads, 128 threads
__global__ void __launch_bounds__(128) attention_combine_kernel(const float* __restrict__ part, __half* __restrict__ out,
                                                                int nsplit) {
    pdl_launch_dependents();
    pdl_wait();
    const float* pp = part + (size_t)blockIdx.x * nsplit * (AT_D + 2);
    // all loads of a batch of eight splits are issued before any is used (one L2 latency per batch, not per split)
    float gm = -INFINITY;
    for (int s0 = 0; s0 < nsplit; s0 += 8) {
        float mv[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) mv[u] = (s0 + u < nsplit) ? pp[(size_t)(s0 + u) * (AT_D + 2)] : -INFINITY;
#pragma unroll
        for (int u = 0; u < 8; ++u) gm = fmaxf(gm, mv[u]);
    }
    float gl = 0.0f, ga = 0.0f;
    for (int s0 = 0; s0 < nsplit; s0 += 8) {
        float mv[8], lv[8], av[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const bool on = s0 + u < nsplit;
            const float* q = pp + (size_t)(on ? s0 + u : 0) * (AT_D + 2);
            mv[u] = on ? q[0] : -INFINITY;
            lv[u] = on ? q[1] : 0.0f;
            av[u] = on ? q[2 + threadIdx.x] : 0.0f;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const float c = (mv[u] == -INFINITY) ? 0.0f : __expf(mv[u] - gm);
            gl += lv[u] * c;
            ga += av[u] * c;
        }
    }
    out[(size_t)blockIdx.x * AT_D + threadIdx.x] = __float2half_rn(gl > 0.0f ? ga / gl : 0.0f);
}

// ---------------------------------------------------------------------------------------------
// Causal prefill: QB consecutive tokens of a sequence share a CTA, so that a K or V row is fetched once for
// 16 = QB * R (query token, query head) pairs instead of once per token.  grid sequences * n_kv * ceil(tps / QB).
// Same arithmetic as attention_kernel: scores and probabilities in fp32, running maximum per pair.
// ---------------------------------------------------------------------------------------------
template <int R>
__global__ void __launch_bounds__(128) attention_block_kernel(const __half* __restrict__ qkv, const __half* __restrict__ kcache,
                                                              const __half* __restrict__ vcache,
                                                              const int* __restrict__ positions, __half* __restrict__ out,
                                                              int tokens_per_seq, int n_heads, int n_kv, int max_ctx,
                                                              float scale) {
    constexpr int QB = 16 / R, NQ = 16;
    __shared__ float qs[NQ][AT_D];
    __shared__ float wm[4][NQ], wl[4][NQ];
    __shared__ float wacc[4][NQ][AT_D];
    __shared__ int ctx_s[QB];
    pdl_launch_dependents();
    pdl_wait();
    const int nblk = (tokens_per_seq + QB - 1) / QB;
    // the blocks with the longest context are scheduled first (they finish last otherwise)
    const int rest = blockIdx.x % ((int)gridDim.x / nblk), qblk = nblk - 1 - (int)blockIdx.x / ((int)gridDim.x / nblk);
    const int kvh = rest % n_kv, seq = rest / n_kv;
    const int t0 = seq * tokens_per_seq + qblk * QB;
    const int nq = min(QB, tokens_per_seq - qblk * QB);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x < QB) ctx_s[threadIdx.x] = (threadIdx.x < nq) ? min(positions[t0 + threadIdx.x] + 1, max_ctx) : 0;
    for (int i = threadIdx.x; i < NQ * AT_D; i += 128) {
        const int q = i / AT_D, dd = i % AT_D, j = q / R, r = q % R;
        qs[q][dd] = (j < nq) ? __half2float(qkv[(size_t)(t0 + j) * (n_heads + 2 * n_kv) * AT_D +
                                                 (size_t)(kvh * R + r) * AT_D + dd]) * scale
                             : 0.0f;
    }
    __syncthreads();
    int P = 0;
#pragma unroll
    for (int j = 0; j < QB; ++j) P = max(P, ctx_s[j]);
    const __half* kb = kcache + ((size_t)seq * n_kv + kvh) * max_ctx * AT_D;
    const __half* vb = vcache + ((size_t)seq * n_kv + kvh) * max_ctx * AT_D;

    float m[NQ], l[NQ], acc[NQ][4];
#pragma unroll
    for (int q = 0; q < NQ; ++q) {
        m[q] = -INFINITY, l[q] = 0.0f;
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[q][e] = 0.0f;
    }
    for (int base = warp * 32; base < P; base += 128) {
        const int p = base + lane;
        float sc[NQ];
#pragma unroll
        for (int q = 0; q < NQ; ++q) sc[q] = 0.0f;
        if (p < P) {
            const uint4* kr = reinterpret_cast<const uint4*>(kb + (size_t)p * AT_D);
#pragma unroll 4
            for (int c = 0; c < AT_D / 8; ++c) {
                const uint4 kv = __ldg(kr + c);
                const __half2* kh = reinterpret_cast<const __half2*>(&kv);
                float kf[8];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 f = __half22float2(kh[e]);
                    kf[2 * e] = f.x, kf[2 * e + 1] = f.y;
                }
#pragma unroll
                for (int q = 0; q < NQ; ++q) {
                    const float4 a = *reinterpret_cast<const float4*>(&qs[q][c * 8]);
                    const float4 b = *reinterpret_cast<const float4*>(&qs[q][c * 8 + 4]);
                    sc[q] += kf[0] * a.x + kf[1] * a.y + kf[2] * a.z + kf[3] * a.w + kf[4] * b.x + kf[5] * b.y +
                             kf[6] * b.z + kf[7] * b.w;
                }
            }
        }
        float w[NQ];
#pragma unroll
        for (int q = 0; q < NQ; ++q) {
            const bool on = p < ctx_s[q / R];      // causal: token j sees positions up to its own
            float cm = on ? sc[q] : -INFINITY;
#pragma unroll
            for (int o = 16; o; o >>= 1) cm = fmaxf(cm, __shfl_xor_sync(0xffffffffu, cm, o));
            const float nm = fmaxf(m[q], cm);
            const float corr = (m[q] == -INFINITY) ? 0.0f : __expf(m[q] - nm);
            w[q] = on ? __expf(sc[q] - nm) : 0.0f;
            l[q] = l[q] * corr + warp_sum(w[q]);
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[q][e] *= corr;
            m[q] = nm;
        }
        const int np = min(32, P - base);
        for (int j0 = 0; j0 < np; j0 += 4) {       // four V rows in flight; rows past the end carry weight 0
            uint2 vv[4];
#pragma unroll
            for (int u = 0; u < 4; ++u)
                vv[u] = __ldg(reinterpret_cast<const uint2*>(vb + (size_t)min(base + j0 + u, max_ctx - 1) * AT_D) + lane);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const __half2* vh = reinterpret_cast<const __half2*>(&vv[u]);
                const float2 f0 = __half22float2(vh[0]), f1 = __half22float2(vh[1]);
#pragma unroll
                for (int q = 0; q < NQ; ++q) {
                    const float wj = __shfl_sync(0xffffffffu, w[q], j0 + u);
                    acc[q][0] += wj * f0.x, acc[q][1] += wj * f0.y, acc[q][2] += wj * f1.x, acc[q][3] += wj * f1.y;
                }
            }
        }
    }
#pragma unroll
    for (int q = 0; q < NQ; ++q) {
        if (lane == 0) wm[warp][q] = m[q], wl[warp][q] = l[q];
#pragma unroll
        for (int e = 0; e < 4; ++e) wacc[warp][q][lane * 4 + e] = acc[q][e];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < NQ * AT_D; i += 128) {
        const int q = i / AT_D, dd = i % AT_D, j = q / R, r = q % R;
        if (j >= nq) continue;
        float gm = -INFINITY;
#pragma unroll
        for (int w4 = 0; w4 < 4; ++w4) gm = fmaxf(gm, wm[w4][q]);
        float gl = 0.0f, ga = 0.0f;
#pragma unroll
        for (int w4 = 0; w4 < 4; ++w4) {
            const float c = (wm[w4][q] == -INFINITY) ? 0.0f : __expf(wm[w4][q] - gm);
            gl += wl[w4][q] * c;
            ga += wacc[w4][q][dd] * c;
        }
        out[((size_t)(t0 + j) * n_heads + kvh * R + r) * AT_D + dd] = __float2half_rn(gl > 0.0f ? ga / gl : 0.0f);
    }
}

// ---------------------------------------------------------------------------------------------
// out[t, i] = fp16(silu(gate[t, i])) * up[t, i];   gu row = [gate (inter) | up (inter)]
// ---------------------------------------------------------------------------------------------
__global__ void silu_mul_kernel(const __half* __restrict__ gu, __half* __restrict__ out, int rows, int inter) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t nvec = (size_t)rows * inter / 8;
    for (size_t v = (size_t)blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += (size_t)gridDim.x * blockDim.x) {
        const size_t e0 = v * 8;
        const size_t t = e0 / inter, i = e0 - t * inter;
        const uint4 g = *reinterpret_cast<const uint4*>(gu + t * 2 * inter + i);
        const uint4 u = *reinterpret_cast<const uint4*>(gu + t * 2 * inter + inter + i);
        const __half2* gh = reinterpret_cast<const __half2*>(&g);
        const __half2* uh = reinterpret_cast<const __half2*>(&u);
        uint4 o;
        __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = __half22float2(gh[e]);
            const __half2 a = __floats2half2_rn(f.x / (1.0f + expf(-f.x)), f.y / (1.0f + expf(-f.y)));
            oh[e] = __hmul2(a, uh[e]);
        }
        *reinterpret_cast<uint4*>(out + e0) = o;
    }
}

__global__ void embedding_kernel(const int* __restrict__ ids, const __half* __restrict__ table, __half* __restrict__ out,
                                 int hidden) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t src = (size_t)ids[blockIdx.x] * hidden, dst = (size_t)blockIdx.x * hidden;
    for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x)
        *reinterpret_cast<uint4*>(out + dst + (size_t)i * 8) = *reinterpret_cast<const uint4*>(table + src + (size_t)i * 8);
}

// index of the first maximum of each row (torch.argmax's tie rule); NaN wins like in torch.
// grid (rows, parts): part `blockIdx.y` scans its slice of the row and leaves (value, index) in `partial`
// (or, with one part, writes the result); argmax_final_kernel picks the winner of the parts.
__global__ void __launch_bounds__(1024) argmax_kernel(const __half* __restrict__ logits, int* __restrict__ out, int vocab,
                                                      float* __restrict__ pval, int* __restrict__ pidx) {
    __shared__ float bv[32];
    __shared__ int bi[32];
    pdl_launch_dependents();
    pdl_wait();
    const __half* row = logits + (size_t)blockIdx.x * vocab;
    const int parts = (int)gridDim.y;
    const int per = (vocab + parts - 1) / parts;
    const int i0 = (int)blockIdx.y * per, i1 = min(vocab, i0 + per);
    float best = -INFINITY;
    int idx = 0x7fffffff;
    for (int i = i0 + (int)threadIdx.x; i < i1; i += blockDim.x) {
        float v = __half2float(row[i]);
        if (v != v) v = INFINITY;
        if (v > best || (v == best && i < idx)) best = v, idx = i;
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > best || (ov == best && oi < idx)) best = ov, idx = oi;
    }
    if ((threadIdx.x & 31) == 0) bv[threadIdx.x >> 5] = best, bi[threadIdx.x >> 5] = idx;
    __syncthreads();
    if (threadIdx.x < 32) {
        best = (threadIdx.x < (blockDim.x >> 5)) ? bv[threadIdx.x] : -INFINITY;
        idx = (threadIdx.x < (blockDim.x >> 5)) ? bi[threadIdx.x] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (ov > best || (ov == best && oi < idx)) best = ov, idx = oi;
        }
        if (threadIdx.x == 0) {
            if (parts == 1) {
                out[blockIdx.x] = idx;
            } else {
                pval[(size_t)blockIdx.x * parts + blockIdx.y] = best;
                pidx[(size_t)blockIdx.x * parts + blockIdx.y] = idx;
            }
        }
    }
}

__global__ void __launch_bounds__(32) argmax_final_kernel(const float* __restrict__ pval, const int* __restrict__ pidx,
                                                          int* __restrict__ out, int parts) {
    pdl_launch_dependents();
    pdl_wait();
    float best = -INFINITY;
    int idx = 0x7fffffff;
    for (int i = threadIdx.x; i < parts; i += 32) {
        const float v = pval[(size_t)blockIdx.x * parts + i];
        const int j = pidx[(size_t)blockIdx.x * parts + i];
        if (v > best || (v == best && j < idx)) best = v, idx = j;
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > best || (ov == best && oi < idx)) best = ov, idx = oi;
    }
    if (threadIdx.x == 0) out[blockIdx.x] = idx;
}

}  // namespace sbvr

using namespace sbvr;

extern "C" {

int sbvr_add_rmsnorm_f16(const void* h_in, const void* delta, const void* weight, void* h_out, void* y, int rows,
                         int hidden, float eps, sbvr_stream_t stream) {
    if (!h_in || !weight || !y || rows < 1 || hidden < 8) return SBVR_ERR_BAD_ARG;
    if (hidden % 8) return SBVR_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(h_in) | reinterpret_cast<uintptr_t>(delta) | reinterpret_cast<uintptr_t>(weight) |
         reinterpret_cast<uintptr_t>(h_out) | reinterpret_cast<uintptr_t>(y)) & 15)
        return SBVR_ERR_ALIGN;
    SBVR_CUDA_TRY(launch_pdl(add_rmsnorm_kernel, dim3(rows), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream),
                             reinterpret_cast<const __half*>(h_in), reinterpret_cast<const __half*>(delta),
                             reinterpret_cast<const __half*>(weight), reinterpret_cast<__half*>(h_out),
                             reinterpret_cast<__half*>(y), hidden, eps));
    return SBVR_OK;
}

int sbvr_rope_append_f16(void* qkv, const int* positions, const float* inv_freq, float attn_scaling, void* kcache,
                         void* vcache, int tokens, int tokens_per_seq, int n_heads, int n_kv, int head_dim, int max_ctx,
                         sbvr_stream_t stream) {
    if (!qkv || !positions || !inv_freq || !kcache || !vcache) return SBVR_ERR_BAD_ARG;
    if (tokens < 1 || tokens_per_seq < 1 || tokens % tokens_per_seq || n_heads < 1 || n_kv < 1 || head_dim < 2 ||
        head_dim % 2 || max_ctx < 1)
        return SBVR_ERR_BAD_ARG;
    SBVR_CUDA_TRY(launch_pdl(rope_append_kernel, dim3(tokens), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream),
                             reinterpret_cast<__half*>(qkv), positions, inv_freq, attn_scaling,
                             reinterpret_cast<__half*>(kcache), reinterpret_cast<__half*>(vcache), tokens_per_seq, n_heads,
                             n_kv, head_dim, max_ctx));
    return SBVR_OK;
}

static int attention_launch(const void* qkv, void* kcache, void* vcache, const int* positions, void* out, float* scratch,
                            int tokens, int tokens_per_seq, int n_heads, int n_kv, int head_dim, int max_ctx, float scale,
                            int nsplit, const float* inv_freq, float attn_scaling, sbvr_stream_t stream) {
    if (!qkv || !kcache || !vcache || !positions || !out) return SBVR_ERR_BAD_ARG;
    if (tokens < 1 || tokens_per_seq < 1 || tokens % tokens_per_seq || n_kv < 1 || n_heads % n_kv || max_ctx < 1 ||
        nsplit < 1 || nsplit > 64)
        return SBVR_ERR_BAD_ARG;
    if (head_dim != AT_D) return SBVR_ERR_UNSUPPORTED;
    if (nsplit > 1 && !scratch) return SBVR_ERR_WORKSPACE;
    if ((reinterpret_cast<uintptr_t>(kcache) | reinterpret_cast<uintptr_t>(vcache)) & 15) return SBVR_ERR_ALIGN;
    const int R = n_heads / n_kv;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const dim3 grid((unsigned)(tokens * n_kv), (unsigned)nsplit);
    const __half* q = reinterpret_cast<const __half*>(qkv);
    __half* kc = reinterpret_cast<__half*>(kcache);
    __half* vc = reinterpret_cast<__half*>(vcache);
    __half* o = reinterpret_cast<__half*>(out);
    if (!inv_freq && nsplit == 1 && tokens_per_seq >= 8) {      // prefill: tokens of a sequence share K / V fetches
        const int QB = 16 / R, nblk = (tokens_per_seq + QB - 1) / QB;
        const dim3 bgrid((unsigned)((tokens / tokens_per_seq) * n_kv * nblk));
#define SBVR_ATTB(RR)                                                                                               \
    SBVR_CUDA_TRY(launch_pdl(attention_block_kernel<RR>, bgrid, dim3(128), 0, st, q, static_cast<const __half*>(kc), \
                             static_cast<const __half*>(vc), positions, o, tokens_per_seq, n_heads, n_kv, max_ctx, scale))
        switch (R) {
            case 1: SBVR_ATTB(1); break;
            case 2: SBVR_ATTB(2); break;
            case 4: SBVR_ATTB(4); break;
            case 8: SBVR_ATTB(8); break;
            default: return SBVR_ERR_UNSUPPORTED;
        }
#undef SBVR_ATTB
        return SBVR_OK;
    }
#define SBVR_ATT(RR)                                                                                              \
    SBVR_CUDA_TRY(launch_pdl(attention_kernel<RR>, grid, dim3(128), 0, st, q, kc, vc, positions, o, scratch,     \
                             tokens_per_seq, n_heads, n_kv, max_ctx, scale, nsplit, inv_freq, attn_scaling))
    switch (R) {
        case 1: SBVR_ATT(1); break;
        case 2: SBVR_ATT(2); break;
        case 4: SBVR_ATT(4); break;
        case 8: SBVR_ATT(8); break;
        default: return SBVR_ERR_UNSUPPORTED;
    }
#undef SBVR_ATT
    if (nsplit > 1)
        SBVR_CUDA_TRY(launch_pdl(attention_combine_kernel, dim3(tokens * n_heads), dim3(128), 0, st,
                                 static_cast<const float*>(scratch), o, nsplit));
    return SBVR_OK;
}

int sbvr_attention_f16(const void* qkv, const void* kcache, const void* vcache, const int* positions, void* out,
                       float* scratch, int tokens, int tokens_per_seq, int n_heads, int n_kv, int head_dim, int max_ctx,
                       float scale, int nsplit, sbvr_stream_t stream) {
    return attention_launch(qkv, const_cast<void*>(kcache), const_cast<void*>(vcache), positions, out, scratch, tokens,
                            tokens_per_seq, n_heads, n_kv, head_dim, max_ctx, scale, nsplit, nullptr, 1.0f, stream);
}

int sbvr_rope_attention_f16(const void* qkv, const int* positions, const float* inv_freq, float attn_scaling, void* kcache,
                            void* vcache, void* out, float* scratch, int tokens, int n_heads, int n_kv, int head_dim,
                            int max_ctx, float scale, int nsplit, sbvr_stream_t stream) {
    if (!inv_freq) return SBVR_ERR_BAD_ARG;
    return attention_launch(qkv, kcache, vcache, positions, out, scratch, tokens, 1, n_heads, n_kv, head_dim, max_ctx, scale,
                            nsplit, inv_freq, attn_scaling, stream);
}

int sbvr_silu_mul_f16(const void* gate_up, void* out, int rows, int inter, sbvr_stream_t stream) {
    if (!gate_up || !out || rows < 1 || inter < 8) return SBVR_ERR_BAD_ARG;
    if (inter % 8) return SBVR_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(gate_up) | reinterpret_cast<uintptr_t>(out)) & 15) return SBVR_ERR_ALIGN;
    const size_t nvec = (size_t)rows * inter / 8;
    const int blocks = (int)((nvec + 255) / 256 < 4096 ? (nvec + 255) / 256 : 4096);
    SBVR_CUDA_TRY(launch_pdl(silu_mul_kernel, dim3(blocks), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream),
                             reinterpret_cast<const __half*>(gate_up), reinterpret_cast<__half*>(out), rows, inter));
    return SBVR_OK;
}

int sbvr_embedding_f16(const int* ids, const void* table, void* out, int tokens, int hidden, sbvr_stream_t stream) {
    if (!ids || !table || !out || tokens < 1 || hidden < 8) return SBVR_ERR_BAD_ARG;
    if (hidden % 8) return SBVR_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(table) | reinterpret_cast<uintptr_t>(out)) & 15) return SBVR_ERR_ALIGN;
    SBVR_CUDA_TRY(launch_pdl(embedding_kernel, dim3(tokens), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream), ids,
                             reinterpret_cast<const __half*>(table), reinterpret_cast<__half*>(out), hidden));
    return SBVR_OK;
}

int sbvr_argmax_f16(const void* logits, int* out, float* scratch, int rows, int vocab, sbvr_stream_t stream) {
    if (!logits || !out || rows < 1 || vocab < 1) return SBVR_ERR_BAD_ARG;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    // few rows of a large vocabulary: cut every row into up to 64 parts so that more than one SM scans it
    int parts = 1;
    if (scratch && vocab >= 16384) {
        parts = 128 / rows;
        if (parts > 64) parts = 64;
        if (parts < 1) parts = 1;
    }
    float* pval = scratch;
    int* pidx = reinterpret_cast<int*>(scratch) + (size_t)rows * parts;
    SBVR_CUDA_TRY(launch_pdl(argmax_kernel, dim3((unsigned)rows, (unsigned)parts), dim3(1024), 0, st,
                             reinterpret_cast<const __half*>(logits), out, vocab, pval, pidx));
    if (parts > 1)
        SBVR_CUDA_TRY(launch_pdl(argmax_final_kernel, dim3(rows), dim3(32), 0, st, static_cast<const float*>(pval),
                                 static_cast<const int*>(pidx), out, parts));
    return SBVR_OK;
}

}  // extern "C"
