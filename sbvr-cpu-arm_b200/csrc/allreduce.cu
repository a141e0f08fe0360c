// One-shot all-reduce of the partial outputs of a row-parallel SBVR linear, fused with the residual add and the
// RMSNorm that follow it in a Llama decoder layer:
//
//     delta = fp16( sum over ranks r = 0 .. world-1 of partial_r )      (fp32 sum, fixed rank order: every rank gets
//     h_out = h_in + delta                                               the same bits, run after run)
//     y     = weight * fp16( h_out * rsqrt(mean(h_out^2) + eps) )
//
// Replaces, for decode-sized batches, the NCCL all-reduce + residual add + LlamaRMSNorm of the tensor-parallel
// model (reference models/sbvr_llama.py:118-123, :395-406; the reference itself has no tensor-parallel path).
//
// Every rank's linear writes its partial [rows, hidden] into its own buffer of a symmetric allocation that all
// ranks have mapped (peer pointers are plain device pointers; the loads below are ordinary loads over NVLink, no
// multicast).  Protocol per call, identified by a monotonically increasing epoch:
//   1. block 0 publishes "my partial of this epoch is complete" by storing the epoch into slot [my rank] of every
//      peer's flag array (system-scope release; the partial was written by the previous kernel on this stream);
//   2. every block waits until all slots of its own flag array have reached the epoch (system-scope acquire),
//      with a bounded number of polls: on time-out the status word is set and the block returns;
//   3. every block reads its row from all ranks' buffers and finishes the three formulas above locally.
// Two buffers alternate between consecutive calls: a rank can start call e + 2 (which overwrites the buffer of
// call e) only after call e + 1, which needs every peer's flag of e + 1, which a peer raises only after its call e
// has finished reading.  The epoch is step * calls_per_step + call + 1 with `step` read from device memory, so a
// captured CUDA graph can be replayed: the host bumps `step` once per decode step inside the graph.
#include <cooperative_groups.h>

#include "common.cuh"
#include "xdigits.cuh"

namespace sbvr {

constexpr int AR_MAX_WORLD = 16;
constexpr int AR_CLUSTER = 8;                           // CTAs that share a row (thread-block cluster, sums meet in shared memory)

// A row is split by columns over the CTAs of a cluster (one SM moved a row of 8192 at about 64 B per clock: 2-3 us of a
// 9 us all-reduce); the sum of squares of the row is the sum of the CTAs' parts, read from each other's shared memory.
__device__ __forceinline__ float cluster_row_sum(float part, float* red /* [33] shared */) {
    namespace cg = cooperative_groups;
#pragma unroll
    for (int o = 16; o; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = part;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.0f;
        for (int w = 0; w < (int)((blockDim.x + 31) >> 5); ++w) t += red[w];
        red[32] = t;
    }
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();                                     // every CTA's part is in its shared memory
    float tot = 0.0f;
    for (unsigned int r = 0; r < cluster.num_blocks(); ++r) tot += *cluster.map_shared_rank(&red[32], r);
    cluster.sync();                                     // nobody leaves while its part may still be read
    return tot;
}

constexpr unsigned int AR_POLL_LIMIT = 1u << 22;        // polls of about 50 ns each

__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}


// The normalised row as activation digits of the decode GEMV (layout of xquant_kernel in linear_tcs.cu: [k block][row][1024 B]
// then one fp32 step per (row, k block)), written next to y: a warp's 32 chunks of 8 values are one 256-k block.  `area` is
// this warp's 1 KB of shared memory.
__device__ __forceinline__ void ar_emit_digits(unsigned char* area, const uint4& o, int chunk, int row, int rows, int KB,
                                               unsigned char* xq) {
    const int lane = threadIdx.x & 31;
    const int kb = chunk >> 5;
    reinterpret_cast<uint4*>(area)[lane] = o;
    __syncwarp();
    float* steps = reinterpret_cast<float*>(xq + (size_t)KB * rows * 1024) + ((size_t)row * KB + kb);
    xdigits_block<1>(area, steps, lane);
    __syncwarp();
    uint4* dst = reinterpret_cast<uint4*>(xq + ((size_t)kb * rows + row) * 1024);
    dst[lane] = reinterpret_cast<const uint4*>(area)[lane];
    dst[lane + 32] = reinterpret_cast<const uint4*>(area)[lane + 32];
}

__global__ void __launch_bounds__(1024) allreduce_add_rmsnorm_kernel(
    const unsigned long long* __restrict__ peer_bufs,    // [world] base address of every rank's buffer area
    const unsigned long long* __restrict__ peer_flags,   // [world] base address of every rank's flag array
    const int* __restrict__ step_ptr, int calls_per_step, int call_idx, int rank, int world, size_t buf_elems,
    const __half* h_in, const __half* __restrict__ weight, __half* h_out, __half* __restrict__ y, int hidden, float eps,
    unsigned int* status, unsigned char* xq) {
    __shared__ float red[33];
    __shared__ int ok_s;
    // 1 KB per warp, present only in launches that emit digits (a fixed 16 KB would keep this kernel from becoming resident
    // beside the pushing GEMV, whose CTA leaves about 11 KB of an SM's shared memory free)
    extern __shared__ __align__(16) unsigned char dig_area[];
    pdl_launch_dependents();
    pdl_wait();                                    // the partial of this rank (previous kernel) is complete from here on
    const unsigned int epoch = (unsigned int)(*step_ptr) * (unsigned int)calls_per_step + (unsigned int)call_idx + 1u;
    const size_t parity_off = (size_t)(call_idx & 1) * buf_elems;
    const int nslice = (int)cooperative_groups::this_cluster().num_blocks();
    const int row_idx = blockIdx.x / nslice, slice = blockIdx.x % nslice;
    if (blockIdx.x == 0 && threadIdx.x < world) {
        __threadfence_system();
        st_release_sys(reinterpret_cast<unsigned int*>(peer_flags[threadIdx.x]) + rank, epoch);
    }
    if (threadIdx.x == 0) ok_s = 1;
    __syncthreads();
    if (threadIdx.x < world) {
        const unsigned int* mine = reinterpret_cast<const unsigned int*>(peer_flags[rank]) + threadIdx.x;
        unsigned int n = 0;
        // epochs only grow; a peer that is already one call ahead shows a larger value
        while ((int)(ld_acquire_sys(mine) - epoch) < 0) {
            if (++n > AR_POLL_LIMIT) {
                ok_s = 0;
                atomicExch(status, 1u);
                atomicExch(status + 1, 0x700u + (unsigned int)rank);
                break;
            }
            __nanosleep(40);
        }
    }
    __syncthreads();
    // a CTA whose wait ran out carries on with what it has (the host sees the time-out): the cluster barriers below
    // need every CTA

    const size_t row = (size_t)row_idx * hidden;
    const int nvec = hidden / 8;
    const int v0 = slice * (nvec / nslice), v1 = v0 + nvec / nslice;
    float ss = 0.0f;
    for (int i = v0 + threadIdx.x; i < v1; i += blockDim.x) {
        float acc[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = 0.0f;
        // the loads of up to eight ranks are all issued before the first is used: one NVLink round trip per batch,
        // not one per rank; the sum still runs in rank order
        for (int r0 = 0; r0 < world; r0 += 8) {
            uint4 v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int r = (r0 + u < world) ? r0 + u : rank;
                const __half* src = reinterpret_cast<const __half*>(peer_bufs[r]) + parity_off + row + (size_t)i * 8;
                v[u] = __ldcv(reinterpret_cast<const uint4*>(src));
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                if (r0 + u < world) {
                    const __half2* vh = reinterpret_cast<const __half2*>(&v[u]);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float2 f = __half22float2(vh[e]);
                        acc[2 * e] += f.x, acc[2 * e + 1] += f.y;
                    }
                }
            }
        }
        uint4 a = *reinterpret_cast<const uint4*>(h_in + row + (size_t)i * 8);
        __half2* ah = reinterpret_cast<__half2*>(&a);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            ah[e] = __hadd2(ah[e], __floats2half2_rn(acc[2 * e], acc[2 * e + 1]));
            const float2 f = __half22float2(ah[e]);
            ss += f.x * f.x + f.y * f.y;
        }
        *reinterpret_cast<uint4*>(h_out + row + (size_t)i * 8) = a;
    }
    const float tot = cluster_row_sum(ss, red);
    const float rs = rsqrtf(tot / (float)hidden + eps);
    for (int i = v0 + threadIdx.x; i < v1; i += blockDim.x) {
        const uint4 a = *reinterpret_cast<const uint4*>(h_out + row + (size_t)i * 8);     // written above by this thread
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
        *reinterpret_cast<uint4*>(y + row + (size_t)i * 8) = o;
        if (xq) ar_emit_digits(dig_area + (threadIdx.x >> 5) * 1024, o, i, row_idx, (int)(gridDim.x / nslice), hidden / 256, xq);
    }
}

// ---------------------------------------------------------------------------------------------
// The receiving side of the pushed form: every rank's row-parallel decode GEMV has stored its partial result into slot
// [call parity][rank] of THIS rank's receive area as 8-byte packets (two fp16 values | epoch << 32), so nothing is read
// over NVLink here and no flag is exchanged: a thread polls its own packets of every rank until their epochs match
// (bounded), adds them in rank order (the same bits on every rank and run), and finishes residual add + RMSNorm like
// the kernel above.  A slot is overwritten two calls later, which a peer can only reach after this rank has pushed the
// call in between, i.e. after this kernel has finished (stream order).
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ ulonglong2 ld_volatile_v2(const unsigned long long* p) {
    ulonglong2 v;
    asm volatile("ld.volatile.global.v2.u64 {%0, %1}, [%2];" : "=l"(v.x), "=l"(v.y) : "l"(p) : "memory");
    return v;
}

__global__ void __launch_bounds__(1024) ll_reduce_add_rmsnorm_kernel(
    const unsigned long long* __restrict__ recv,      // [2][world][rows_max][hidden / 2]
    const int* __restrict__ step_ptr, int calls_per_step, int call_idx, int world, int rows_max, const __half* h_in,
    const __half* __restrict__ weight, __half* h_out, __half* __restrict__ y, int hidden, float eps, unsigned int* status,
    int follows_push, unsigned char* xq) {
    __shared__ float red[33];
    // 1 KB per warp, present only in launches that emit digits (a fixed 16 KB would keep this kernel from becoming resident
    // beside the pushing GEMV, whose CTA leaves about 11 KB of an SM's shared memory free)
    extern __shared__ __align__(16) unsigned char dig_area[];
    pdl_launch_dependents();
    // Directly behind the pushing GEMV of the same call this kernel is only let go once that GEMV's own dependency wait
    // has returned: the residual and the step counter are final, the packets announce themselves, and nothing else of
    // the GEMV is read, so its end (and the acknowledgement of its stores to the peers) need not be waited for.
    if (!follows_push) pdl_wait();
    const unsigned int epoch = (unsigned int)(*step_ptr) * (unsigned int)calls_per_step + (unsigned int)call_idx + 1u;
    const int nslice = (int)cooperative_groups::this_cluster().num_blocks();
    const int row_idx = blockIdx.x / nslice, slice = blockIdx.x % nslice;
    const size_t row = (size_t)row_idx * hidden;
    const int nvec = hidden / 8;
    const int v0 = slice * (nvec / nslice), v1 = v0 + nvec / nslice;
    float ss = 0.0f;
    for (int i = v0 + threadIdx.x; i < v1; i += blockDim.x) {
        float acc[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = 0.0f;
        for (int r0 = 0; r0 < world; r0 += 8) {
            ulonglong2 a[8], b[8];
            const long long t0 = clock64();
            for (;;) {
                // the packets of up to eight ranks are all requested before the first is looked at
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int r = (r0 + u < world) ? r0 + u : r0;
                    const unsigned long long* src =
                        recv + (((size_t)(call_idx & 1) * world + r) * rows_max + row_idx) * (size_t)(hidden / 2) + (size_t)i * 4;
                    a[u] = ld_volatile_v2(src);
                    b[u] = ld_volatile_v2(src + 2);
                }
                bool done = true;
#pragma unroll
                for (int u = 0; u < 8; ++u)
                    if (r0 + u < world)
                        done = done && (unsigned int)(a[u].x >> 32) == epoch && (unsigned int)(a[u].y >> 32) == epoch &&
                               (unsigned int)(b[u].x >> 32) == epoch && (unsigned int)(b[u].y >> 32) == epoch;
                if (done) break;
                if (clock64() - t0 > 600000000LL) {           // about a third of a second: a rank never delivered
                    atomicExch(status, 1u);
                    atomicExch(status + 1, 0x710u);
                    break;
                }
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                if (r0 + u < world) {
                    const unsigned int w4[4] = {(unsigned int)a[u].x, (unsigned int)a[u].y, (unsigned int)b[u].x, (unsigned int)b[u].y};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w4[e]));
                        acc[2 * e] += f.x, acc[2 * e + 1] += f.y;
                    }
                }
            }
        }
        uint4 hv = *reinterpret_cast<const uint4*>(h_in + row + (size_t)i * 8);
        __half2* ah = reinterpret_cast<__half2*>(&hv);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            ah[e] = __hadd2(ah[e], __floats2half2_rn(acc[2 * e], acc[2 * e + 1]));
            const float2 f = __half22float2(ah[e]);
            ss += f.x * f.x + f.y * f.y;
        }
        *reinterpret_cast<uint4*>(h_out + row + (size_t)i * 8) = hv;
    }
    const float tot = cluster_row_sum(ss, red);
    const float rs = rsqrtf(tot / (float)hidden + eps);
    for (int i = v0 + threadIdx.x; i < v1; i += blockDim.x) {
        const uint4 hv = *reinterpret_cast<const uint4*>(h_out + row + (size_t)i * 8);    // written above by this thread
        const uint4 wv = *reinterpret_cast<const uint4*>(weight + (size_t)i * 8);
        const __half2* ah = reinterpret_cast<const __half2*>(&hv);
        const __half2* wh = reinterpret_cast<const __half2*>(&wv);
        uint4 o;
        __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = __half22float2(ah[e]);
            oh[e] = __hmul2(wh[e], __floats2half2_rn(f.x * rs, f.y * rs));
        }
        *reinterpret_cast<uint4*>(y + row + (size_t)i * 8) = o;
        if (xq) ar_emit_digits(dig_area + (threadIdx.x >> 5) * 1024, o, i, row_idx, (int)(gridDim.x / nslice), hidden / 256, xq);
    }
}

}  // namespace sbvr

using namespace sbvr;

// Where the digits go: the start of the workspace's dynamic region, which is where the decode GEMV looks for them.
static int ar_digits_target(sbvr_workspace_t* ws, int rows, int hidden, int emit_digits, unsigned char** xq) {
    *xq = nullptr;
    if (!emit_digits) return SBVR_OK;
    const int nvec = hidden / 8;
    if (rows > 4 || hidden % 2048 || nvec % AR_CLUSTER || (nvec / AR_CLUSTER) % 32 || nvec / AR_CLUSTER > 512) return SBVR_ERR_UNSUPPORTED;
    const size_t need = (size_t)(hidden / 256) * rows * 1024 + (((size_t)rows * (hidden / 256) * 4 + 15) / 16) * 16;
    if (need > ws->dyn_bytes) return SBVR_ERR_WORKSPACE;
    *xq = reinterpret_cast<unsigned char*>(ws->dyn);
    return SBVR_OK;
}

extern "C" int sbvr_allreduce_add_rmsnorm_digits_f16(const void* peer_bufs_dev, const void* peer_flags_dev, const int* step_dev,
                                                      int calls_per_step, int call_idx, int rank, int world, size_t buf_elems,
                                                      const void* h_in, const void* weight, void* h_out, void* y, int rows,
                                                      int hidden, float eps, int emit_digits, sbvr_workspace_t* ws,
                                                      sbvr_stream_t stream) {
    if (!peer_bufs_dev || !peer_flags_dev || !step_dev || !h_in || !weight || !h_out || !y || !ws) return SBVR_ERR_BAD_ARG;
    if (world < 1 || world > AR_MAX_WORLD || rank < 0 || rank >= world || rows < 1 || calls_per_step < 1 || call_idx < 0 ||
        call_idx >= calls_per_step || (calls_per_step & 1))
        return SBVR_ERR_BAD_ARG;
    if (hidden < 8 || hidden % 8) return SBVR_ERR_SHAPE;
    if ((size_t)rows * hidden > buf_elems) return SBVR_ERR_WORKSPACE;
    if ((reinterpret_cast<uintptr_t>(h_in) | reinterpret_cast<uintptr_t>(weight) | reinterpret_cast<uintptr_t>(h_out) |
         reinterpret_cast<uintptr_t>(y)) & 15)
        return SBVR_ERR_ALIGN;
    unsigned char* xq = nullptr;
    const int rc = ar_digits_target(ws, rows, hidden, emit_digits, &xq);
    if (rc) return rc;
    // a row is shared by a cluster of CTAs where its 16-byte chunks divide evenly
    const int nvec = hidden / 8, cs = (nvec % AR_CLUSTER == 0) ? AR_CLUSTER : 1;
    const int per = nvec / cs, threads = per >= 512 ? 512 : (per + 31) / 32 * 32;
    SBVR_CUDA_TRY(launch_pdl_cluster(allreduce_add_rmsnorm_kernel, dim3(rows * cs), dim3(threads), cs, xq ? (size_t)(threads / 32) * 1024 : 0, reinterpret_cast<cudaStream_t>(stream),
                             reinterpret_cast<const unsigned long long*>(peer_bufs_dev),
                             reinterpret_cast<const unsigned long long*>(peer_flags_dev), step_dev, calls_per_step, call_idx,
                             rank, world, buf_elems, reinterpret_cast<const __half*>(h_in),
                             reinterpret_cast<const __half*>(weight), reinterpret_cast<__half*>(h_out),
                             reinterpret_cast<__half*>(y), hidden, eps, ws->status, xq));
    return SBVR_OK;
}

extern "C" int sbvr_allreduce_add_rmsnorm_f16(const void* peer_bufs_dev, const void* peer_flags_dev, const int* step_dev,
                                               int calls_per_step, int call_idx, int rank, int world, size_t buf_elems,
                                               const void* h_in, const void* weight, void* h_out, void* y, int rows,
                                               int hidden, float eps, sbvr_workspace_t* ws, sbvr_stream_t stream) {
    return sbvr_allreduce_add_rmsnorm_digits_f16(peer_bufs_dev, peer_flags_dev, step_dev, calls_per_step, call_idx, rank, world,
                                                 buf_elems, h_in, weight, h_out, y, rows, hidden, eps, 0, ws, stream);
}

extern "C" int sbvr_ll_reduce_add_rmsnorm_digits_f16(const void* recv_local, const int* step_dev, int calls_per_step,
                                                      int call_idx, int world, int rows_max, const void* h_in,
                                                      const void* weight, void* h_out, void* y, int rows, int hidden, float eps,
                                                      int follows_push, int emit_digits, sbvr_workspace_t* ws,
                                                      sbvr_stream_t stream) {
    if (!recv_local || !step_dev || !h_in || !weight || !h_out || !y || !ws) return SBVR_ERR_BAD_ARG;
    if (world < 1 || world > AR_MAX_WORLD || rows < 1 || rows > rows_max || calls_per_step < 1 || call_idx < 0 ||
        call_idx >= calls_per_step || (calls_per_step & 1))
        return SBVR_ERR_BAD_ARG;
    if (hidden < 8 || hidden % 8) return SBVR_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(recv_local) | reinterpret_cast<uintptr_t>(h_in) | reinterpret_cast<uintptr_t>(weight) |
         reinterpret_cast<uintptr_t>(h_out) | reinterpret_cast<uintptr_t>(y)) & 15)
        return SBVR_ERR_ALIGN;
    unsigned char* xq = nullptr;
    const int rc = ar_digits_target(ws, rows, hidden, emit_digits, &xq);
    if (rc) return rc;
    const int nvec = hidden / 8, cs = (nvec % AR_CLUSTER == 0) ? AR_CLUSTER : 1;
    const int per = nvec / cs, threads = per >= 512 ? 512 : (per + 31) / 32 * 32;
    SBVR_CUDA_TRY(launch_pdl_cluster(ll_reduce_add_rmsnorm_kernel, dim3(rows * cs), dim3(threads), cs, xq ? (size_t)(threads / 32) * 1024 : 0,
                             reinterpret_cast<cudaStream_t>(stream), reinterpret_cast<const unsigned long long*>(recv_local),
                             step_dev, calls_per_step, call_idx, world, rows_max, reinterpret_cast<const __half*>(h_in),
                             reinterpret_cast<const __half*>(weight), reinterpret_cast<__half*>(h_out),
                             reinterpret_cast<__half*>(y), hidden, eps, ws->status, follows_push ? 1 : 0, xq));
    return SBVR_OK;
}

extern "C" int sbvr_ll_reduce_add_rmsnorm_f16(const void* recv_local, const int* step_dev, int calls_per_step, int call_idx,
                                               int world, int rows_max, const void* h_in, const void* weight, void* h_out,
                                               void* y, int rows, int hidden, float eps, int follows_push,
                                               sbvr_workspace_t* ws, sbvr_stream_t stream) {
    return sbvr_ll_reduce_add_rmsnorm_digits_f16(recv_local, step_dev, calls_per_step, call_idx, world, rows_max, h_in, weight,
                                                 h_out, y, rows, hidden, eps, follows_push, 0, ws, stream);
}
