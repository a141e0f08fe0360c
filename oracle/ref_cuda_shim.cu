// TEST INFRASTRUCTURE - a thin C-ABI shim over the REFERENCE's own CUDA kernels, compiled from where they lie.
//
// `make -C oracle ref REF=<reference checkout>` compiles <REF>/sbvr/kernels/sbvr_kernel.cu (untouched) together with
// this file into oracle/_ref/libsbvr_ref_cuda.so.  This file supplies the two globals the reference kernels expect from
// their torch binding (sbvr/kernels/sbvr_ops.cpp:31-32, filled by sbvr_cuda_init :122-150) and extern "C" wrappers over
// the reference's two launchers (sbvr/kernels/sbvr_kernel.cu:876-912 and :914-1023), so that tests and the benchmark's
// comparator leg can call them with raw device pointers (no torch extension build is needed).  Nothing in the product
// links or loads this library.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

int device_count;
cudaDeviceProp cuda_prop_list[16];

void launch_cuda_sbvr_mm_T(uint32_t* l_bvr, void* l_coeff_idx, __half* l_coeff_cache, uint32_t* r_bvr, void* r_coeff_idx,
                           __half* r_coeff_cache, __half* bias, __half* out, int M, int N, int K, int l_num_sums,
                           int r_num_sums, int l_cache_size, int r_cache_size, int device_id);
void launch_cuda_sbvr_row_deq_mm_T(__half* l_w, uint32_t* r_bvr, void* r_coeff_idx, __half* r_coeff_cache, __half* bias,
                                   __half* out, int M, int N, int K, int r_num_sums, int r_cache_size, int use_shfl,
                                   int device_id);

extern "C" {

// what sbvr_cuda_init does, without the printing; returns the device count or a negative cudaError
__attribute__((visibility("default"))) int sbvr_ref_init(void) {
    cudaError_t e = cudaGetDeviceCount(&device_count);
    if (e != cudaSuccess) return -(int)e;
    for (int d = 0; d < device_count && d < 16; ++d) {
        e = cudaGetDeviceProperties(&cuda_prop_list[d], d);
        if (e != cudaSuccess) return -(int)e;
    }
    return device_count;
}

// out[M, N] = l_w[M, K] @ W^T + bias on the transposed ("row-dequant") encoding: r_bvr uint32 [N/32, K, S],
// r_coeff_idx [N/256, K], r_coeff_cache [C, S].  The reference's S = 4 kernel computes row 0 of l_w only.
// Runs on the default stream of `device`; returns the cudaError of the synchronisation that follows.
__attribute__((visibility("default"))) int sbvr_ref_row_deq_mm_T(void* l_w, void* r_bvr, void* r_coeff_idx, void* r_coeff_cache,
                                                                 void* bias, void* out, int M, int N, int K, int S, int C,
                                                                 int use_shfl, int device) {
    try {
        launch_cuda_sbvr_row_deq_mm_T((__half*)l_w, (uint32_t*)r_bvr, r_coeff_idx, (__half*)r_coeff_cache, (__half*)bias,
                                      (__half*)out, M, N, K, S, C, use_shfl, device);
    } catch (...) {
        return -1;
    }
    return (int)cudaDeviceSynchronize();
}

// out[M, N] = decode(l) @ decode(r)^T + bias with both operands encoded: l_bvr uint32 [Kw, M, LS], r_bvr [Kw, N, RS]
// (Kw = K / 32 words, a multiple of 8), indices [Kw/8, M] / [Kw/8, N], codebooks [Cl, LS] / [Cr, RS].
__attribute__((visibility("default"))) int sbvr_ref_mm_T(void* l_bvr, void* l_idx, void* l_cache, void* r_bvr, void* r_idx,
                                                         void* r_cache, void* bias, void* out, int M, int N, int Kw, int LS,
                                                         int RS, int Cl, int Cr, int device) {
    try {
        launch_cuda_sbvr_mm_T((uint32_t*)l_bvr, l_idx, (__half*)l_cache, (uint32_t*)r_bvr, r_idx, (__half*)r_cache,
                              (__half*)bias, (__half*)out, M, N, Kw, LS, RS, Cl, Cr, device);
    } catch (...) {
        return -1;
    }
    return (int)cudaDeviceSynchronize();
}

// average microseconds of `reps` back-to-back launches of either call above (which = 0 row_deq, 1 mm_T), CUDA events on
// the default stream; the arguments are those of the respective wrapper (unused ones ignored)
__attribute__((visibility("default"))) float sbvr_ref_time_us(int which, int reps, void* a0, void* a1, void* a2, void* a3,
                                                               void* a4, void* a5, void* bias, void* out, int M, int N, int K,
                                                               int S0, int S1, int C0, int C1, int device) {
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    float ms = -1.0f;
    try {
        for (int r = -3; r < reps; ++r) {
            if (r == 0) cudaEventRecord(e0, 0);
            if (which == 0)
                launch_cuda_sbvr_row_deq_mm_T((__half*)a0, (uint32_t*)a1, a2, (__half*)a3, (__half*)bias, (__half*)out, M, N, K,
                                              S0, C0, 0, device);
            else
                launch_cuda_sbvr_mm_T((uint32_t*)a0, a1, (__half*)a2, (uint32_t*)a3, a4, (__half*)a5, (__half*)bias,
                                      (__half*)out, M, N, K, S0, S1, C0, C1, device);
        }
        cudaEventRecord(e1, 0);
        if (cudaEventSynchronize(e1) == cudaSuccess) cudaEventElapsedTime(&ms, e0, e1);
    } catch (...) {
        ms = -1.0f;
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    return ms < 0 ? -1.0f : ms * 1000.0f / reps;
}

}  // extern "C"
