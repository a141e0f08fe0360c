// Shared declarations of the sbvr_b200 library: status codes, the workspace, launch helpers and
// the few PTX wrappers (mbarrier, bulk asynchronous copy, programmatic dependent launch) the
// kernels use.  sm_100a only.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

#include "../../include/sbvr_b200.h"

namespace sbvr {

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
extern thread_local int g_last_cuda_error;

#define SBVR_CUDA_TRY(expr)                                   \
    do {                                                      \
        cudaError_t e__ = (expr);                             \
        if (e__ != cudaSuccess) {                             \
            ::sbvr::g_last_cuda_error = (int)e__;             \
            (void)cudaGetLastError();                         \
            return SBVR_ERR_CUDA;                             \
        }                                                     \
    } while (0)

struct DeviceInfo {
    int sm_count;
    int smem_optin;
    int l2_bytes;
    int cc_major, cc_minor;
};
int device_info(int device, DeviceInfo* out);      // cached per device, read-only after first call

// How a weight's coefficients are addressed.
struct PackedW {
    const uint32_t* bvr;     // [K/32, N, S]
    const void* idx;         // [K/G, N] u8/u16, or unused
    const __half* coeff;     // [C, S] codebook or [K/G, N, S] direct
    int idx_bytes;           // 0 direct, 1, 2
    int C;
    int N, K, S, G;
};

}  // namespace sbvr

// The workspace: one device allocation carved into regions.
struct sbvr_workspace {
    int device;
    size_t bytes;
    char* base;               // device
    // fixed regions at the start of `base`
    unsigned int* status;     // [4]   word 0: 0 ok / 1 a bounded wait ran out; word 1: where
    unsigned int* counters;   // [SBVR_WS_COUNTERS] reserved for kernels that count arrivals; all zero between calls
    unsigned long long* xchg; // [SBVR_WS_XCHG_BYTES / 8] tagged exchange slots of the decode kernel; all zero between calls
    char* dyn;                // rest: staging buffers of the host-pointer entry point, future scratch
    size_t dyn_bytes;
    void* pinned_status;      // host, 16 bytes
};
#define SBVR_WS_COUNTERS 8192
#define SBVR_WS_XCHG_BYTES (1u << 20)
// bytes of the fixed regions in front of `dyn`: status (256), counters, exchange slots
#define SBVR_WS_FIXED_BYTES (256u + SBVR_WS_COUNTERS * 4u + SBVR_WS_XCHG_BYTES)

namespace sbvr {

// Launch with programmatic stream serialization: the grid may be scheduled while its predecessor on the stream is
// still running; every such kernel executes griddepcontrol.wait before it touches what the predecessor produced.
// SBVR_NO_PDL=1 in the environment turns the attribute off (plain stream order).
bool pdl_enabled();
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid, cfg.blockDim = block, cfg.dynamicSmemBytes = smem, cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// The same with thread-block clusters of `cluster_x` CTAs along x (the grid's x must be a multiple of it).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, int cluster_x, size_t smem,
                                      cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid, cfg.blockDim = block, cfg.dynamicSmemBytes = smem, cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned int)cluster_x, attr[0].val.clusterDim.y = 1, attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) once per device for one kernel instantiation: the caller keeps one
// static SmemOnce per instantiation.  Safe from several host threads and with several devices in turn.
struct SmemOnce {
    std::mutex mu;
    bool done[64] = {false};
};
template <typename Kernel>
inline int set_max_smem_once(SmemOnce& once, Kernel kernel, int bytes) {
    int dev = 0;
    SBVR_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return SBVR_ERR_BAD_ARG;
    std::lock_guard<std::mutex> lock(once.mu);
    if (!once.done[dev]) {
        SBVR_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
        once.done[dev] = true;
    }
    return SBVR_OK;
}

int launch_decode(const PackedW& w, __half* W, int ldw, int Kout, cudaStream_t st);
int launch_linear_simt(const __half* x, const PackedW& w, const __half* bias, __half* y, int M, cudaStream_t st);
// What the decode GEMV makes its activations of while it brings them in.
struct XOp {
    int op;                  // SBVR_XOP_*
    const __half* delta;     // ADD_RMSNORM: added to x first (may be NULL)
    const __half* norm_w;    // ADD_RMSNORM: RMSNorm weight [K]
    __half* h_out;           // ADD_RMSNORM: x + delta is stored here (may be NULL; must not be x)
    float eps;
};
// The decode GEMV can push its result to the ranks of a tensor-parallel model instead of storing y: `push` is an
// sbvr_push_desc_t in device memory (include/sbvr_b200.h), read by the kernel only.
// The decode GEMV (linear_tcs.cu): FP4 tensor-core dot products, weights through TMA, work split by 256-k steps.
// The caller hands it its scratch: a status word pair, the zeroed exchange slots (SBVR_WS_XCHG_BYTES) and
// `scratch_bytes` >= linear_tcs_workspace_bytes() of 256-byte aligned memory.
bool linear_tcs_supported(const PackedW& w, int M);
size_t linear_tcs_workspace_bytes(const PackedW& w, int M, int sm_count);
int launch_linear_tcs(const __half* x, const PackedW& w, const __half* bias, __half* y, int M, int device,
                      unsigned int* status, unsigned long long* xchg, char* scratch, size_t scratch_bytes, cudaStream_t st,
                      const XOp* xop = nullptr, const sbvr_push_desc_t* push = nullptr);
// The small-batch kernel (linear_tcb.cu), 2 .. 32 activation rows: same scratch rules; it uses the first words of the
// exchange region as arrival counters and leaves them zero.
bool linear_tcb_supported(const PackedW& w, int M);
size_t linear_tcb_workspace_bytes(const PackedW& w, int M, int sm_count);
int launch_linear_tcb(const __half* x, const PackedW& w, const __half* bias, __half* y, int M, int device,
                      unsigned int* status, unsigned long long* xchg, char* scratch, size_t scratch_bytes, cudaStream_t st);
bool linear_gemm_supported(const PackedW& w, int M);
size_t linear_gemm_workspace_bytes(const PackedW& w, int M, int sm_count);
int launch_linear_gemm(const __half* x, const PackedW& w, const __half* bias, __half* y, int M,
                       sbvr_workspace* ws, cudaStream_t st);

// ---------------------------------------------------------------------------------------------
// device side
// ---------------------------------------------------------------------------------------------
#ifdef __CUDACC__

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(2000u)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after `limit` tries (each try may suspend for about 2 us) and reports it.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, uint32_t limit = 400000u) {
    for (uint32_t i = 0; i < limit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}

// Bounded wait by elapsed time.  Each try lets the hardware suspend the warp (no issue slots burnt
// while it sleeps) for up to the hint; the loop gives up after about a second of SM clock.
__device__ __forceinline__ bool mbar_wait_timed(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    const uint32_t a = smem_u32(bar);
    long long t0 = 0;
    for (;;) {
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
            "selp.b32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(a), "r"(parity), "r"(100000u)
            : "memory");
        if (ok) return true;
        if (t0 == 0) t0 = clock64();
        else if (clock64() - t0 > 2000000000LL) return false;
    }
}

// Bounded wait for barriers completed by ASYNCHRONOUS arrivals (tcgen05.commit, bulk-copy complete_tx).
// Measured on B200: a waiter parked by try_wait with a long suspend hint is woken promptly by a
// thread's mbarrier.arrive, but sleeps on for thousands of cycles when the phase is completed by an
// asynchronous arrival.  So these barriers are polled with the default (short) time limit.
__device__ __forceinline__ bool mbar_wait_async(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    const uint32_t a = smem_u32(bar);
    long long t0 = 0;
    for (;;) {
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.b32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(a), "r"(parity)
            : "memory");
        if (ok) return true;
        if (t0 == 0) t0 = clock64();
        else if (clock64() - t0 > 2000000000LL) return false;
    }
}

// Non-blocking test of a phase (true = complete).
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// 1-D bulk asynchronous copy global -> shared; both addresses 16-byte aligned, bytes % 16 == 0.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// Programmatic dependent launch: let the next kernel in the stream start its prologue / wait for
// the previous kernel's memory to be visible.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// One lane of a converged warp; the compiler keeps the operands of what it guards in uniform registers.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred = 0, laneid = 0;
    asm volatile(
        "{\n\t.reg .b32 %%rx;\n\t.reg .pred %%px;\n\t"
        "elect.sync %%rx|%%px, %2;\n\t"
        "@%%px mov.s32 %1, 1;\n\t"
        "mov.s32 %0, %%rx;\n\t}"
        : "+r"(laneid), "+r"(pred)
        : "r"(0xFFFFFFFFu));
    return pred != 0;
}

__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// Coefficient line of (group g, row n) as a pointer to S halves.
__device__ __forceinline__ const __half* coeff_line(const void* idx, int idx_bytes, const __half* coeff, int g, int n,
                                                    int N, int S) {
    if (idx_bytes == 0) return coeff + ((size_t)g * N + n) * S;
    size_t line = (idx_bytes == 1) ? (size_t)((const uint8_t*)idx)[(size_t)g * N + n]
                                   : (size_t)((const uint16_t*)idx)[(size_t)g * N + n];
    return coeff + line * S;
}

#endif  // __CUDACC__
}  // namespace sbvr
