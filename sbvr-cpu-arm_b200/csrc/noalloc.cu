// sbvr_linear_f16_noalloc: the SBVR linear for callers that are not allowed to allocate device memory.
//
// Who needs this.  Some hosts hand a plugin a fixed set of buffers and forbid it to touch the
// allocator: an inference server that carved up the whole GPU at start-up and treats any later
// cudaMalloc as a bug (it synchronises the device and can fail under memory pressure in the middle
// of serving); a real-time loop whose latency budget has no room for the allocator's implicit
// synchronisation; code that runs while another thread of the process has a stream capture open
// in global mode, where an allocation call would break that capture.  Such callers cannot create
// the `sbvr_workspace_t` the regular entry point wants, because creating it is a cudaMalloc.
//
// What it does instead.  The scratch the kernels need (the time-out status word, the arrival counters,
// the quantised activations and partial sums of the decode kernel, the re-tiled activations and the
// split-K partial sums of the batched kernel) lives in ONE
// fixed array that is part of this library's device image, `g_noalloc_scratch` below: SBVR_NOALLOC_BYTES = 4 MiB per
// GPU that loads the library, held until the process exits.  Nothing is allocated or freed here,
// by this file or by anything it calls.
//
// Rules that follow from sharing one array:
//   * Every call on a device uses the same bytes.  Two calls that can overlap on that GPU (different
//     streams, different host threads) race on it and corrupt each other's result: serialise them.
//   * The array keeps what the previous call left.  The part that must be zero when a kernel starts
//     (status word and arrival counters) is cleared on the stream at the beginning of every call.
//   * The first call on each device looks up the array's device address (cudaGetSymbolAddress, which
//     may load the module); the first call of each kernel variant (S, G, M, index width) on a device sets
//     that kernel's shared-memory attribute and may encode a tensor map.  Make such first calls outside
//     any stream capture, with the device current; later calls only enqueue work.
//   * A problem whose scratch does not fit is refused with SBVR_ERR_NOALLOC_LIMIT before anything is
//     launched.  The decode kernel (M <= 4) needs about 4 K M bytes for the activation digits plus 150 KB of
//     partial sums: every shape it serves fits.  Batches (M > 4) run on the tensor-core GEMM, whose re-tiled
//     activations take M K 2 bytes (M rounded up to its tile): M = 128 at K = 14336 fits, M = 2048 does not
//     and is refused.  Shapes neither kernel serves run on the SIMT kernel, which needs no scratch.
//   * A time-out of a bounded device wait is recorded in the array but this entry point has no
//     synchronising call to report it; use the workspace form if you need that.
#include <mutex>

#include "common.cuh"

#define SBVR_NOALLOC_BYTES (4u << 20)

// The scratch itself.  In host code this name is only a handle for cudaGetSymbolAddress: it is NOT a
// device pointer, and passing it to a kernel would make the kernel read host memory or fault.
static __device__ __align__(256) unsigned char g_noalloc_scratch[SBVR_NOALLOC_BYTES];

namespace {

std::mutex g_mu;
void* g_dev_ptr[64];
bool g_have[64];

// Device address of the array on the current device, looked up once per device.
int scratch_for_current_device(void** ptr, int* device) {
    int dev = 0;
    SBVR_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return SBVR_ERR_BAD_ARG;
    std::lock_guard<std::mutex> lock(g_mu);
    if (!g_have[dev]) {
        void* p = nullptr;
        SBVR_CUDA_TRY(cudaGetSymbolAddress(&p, g_noalloc_scratch));
        if (!p || (reinterpret_cast<uintptr_t>(p) & 255)) return SBVR_ERR_ALIGN;
        g_dev_ptr[dev] = p;
        g_have[dev] = true;
    }
    *ptr = g_dev_ptr[dev];
    *device = dev;
    return SBVR_OK;
}

}  // namespace

extern "C" int sbvr_linear_f16_noalloc(const void* x, const uint32_t* bvr, const void* coeff_idx, int idx_bytes,
                                       const void* coeff, int C, const void* bias, void* y, int M, int N, int K, int S,
                                       int G, sbvr_stream_t stream) {
    using namespace sbvr;
    // same argument rules as sbvr_linear_f16
    if (!x || !y || !bvr || !coeff || M < 1 || N < 1 || K < 1 || S < 1 || S > 8) return SBVR_ERR_BAD_ARG;
    if (idx_bytes != 0 && idx_bytes != 1 && idx_bytes != 2) return SBVR_ERR_BAD_ARG;
    if (idx_bytes != 0 && (!coeff_idx || C < 1 || C > 65536 || (idx_bytes == 1 && C > 256))) return SBVR_ERR_BAD_ARG;
    if (G < 32 || G % 32) return SBVR_ERR_BAD_ARG;
    if (K % G) return SBVR_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(bvr) & 3) || (reinterpret_cast<uintptr_t>(coeff) & 1) ||
        (reinterpret_cast<uintptr_t>(x) & 3) || (reinterpret_cast<uintptr_t>(y) & 1) ||
        (idx_bytes == 2 && (reinterpret_cast<uintptr_t>(coeff_idx) & 1)))
        return SBVR_ERR_ALIGN;
    PackedW w;
    w.bvr = bvr, w.idx = coeff_idx, w.coeff = reinterpret_cast<const __half*>(coeff);
    w.idx_bytes = idx_bytes, w.C = C, w.N = N, w.K = K, w.S = S, w.G = G;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const __half* xh = reinterpret_cast<const __half*>(x);
    const __half* bh = reinterpret_cast<const __half*>(bias);
    __half* yh = reinterpret_cast<__half*>(y);

    void* base = nullptr;
    int dev = 0;
    int rc = scratch_for_current_device(&base, &dev);
    if (rc) return rc;
    DeviceInfo di;
    rc = device_info(dev, &di);
    if (rc) return rc;
    // carve the static array exactly like an allocated workspace
    const size_t fixed = SBVR_WS_FIXED_BYTES;
    sbvr_workspace ws;
    ws.device = dev;
    ws.bytes = SBVR_NOALLOC_BYTES;
    ws.base = reinterpret_cast<char*>(base);
    ws.status = reinterpret_cast<unsigned int*>(ws.base);
    ws.counters = reinterpret_cast<unsigned int*>(ws.base + 256);
    ws.xchg = reinterpret_cast<unsigned long long*>(ws.base + 256 + (size_t)SBVR_WS_COUNTERS * 4);
    ws.dyn = ws.base + fixed;
    ws.dyn_bytes = SBVR_NOALLOC_BYTES - fixed;
    ws.pinned_status = nullptr;
    const bool aligned_x = !(reinterpret_cast<uintptr_t>(x) & 15);
    // which kernel serves the call, and how much of the array it needs
    int kind = 0;                                  // 0: SIMT kernel (no scratch), 1: decode GEMV, 2: batched GEMM
    size_t need = 0;
    if (di.cc_major == 10 && aligned_x && linear_tcs_supported(w, M)) {
        kind = 1;
        need = linear_tcs_workspace_bytes(w, M, di.sm_count);       // activation digits + partial sums of shared row tiles
    } else if (di.cc_major == 10 && linear_gemm_supported(w, M)) {
        kind = 2;
        need = linear_gemm_workspace_bytes(w, M, di.sm_count);      // re-tiled activations + fp32 parts of a split K
    }
    if (kind == 0) return launch_linear_simt(xh, w, bh, yh, M, st);
    if (need > ws.dyn_bytes) return SBVR_ERR_NOALLOC_LIMIT;         // nothing has been launched
    // whatever the previous call (possibly an aborted one) left in the status word and the counters must go
    SBVR_CUDA_TRY(cudaMemsetAsync(ws.base, 0, fixed, st));
    if (kind == 1)
        rc = launch_linear_tcs(xh, w, bh, yh, M, dev, ws.status, ws.xchg, ws.dyn, ws.dyn_bytes, st);
    else
        rc = launch_linear_gemm(xh, w, bh, yh, M, &ws, st);
    if (rc == SBVR_ERR_WORKSPACE) return SBVR_ERR_NOALLOC_LIMIT;
    return rc;
}
