// noalloc.cu -- Q8 block-quantized mul_mat for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc on the path where they need the product: code
// running inside a memory-planned executor whose arena was sized up front (the reference's graph
// allocator plans every buffer before the first node runs), code that is being replayed under a
// fixed memory budget, or a process that handed all free device memory to another allocator.  The
// regular entry point, ppml_b200_mul_mat_q8, may grow a device scratch buffer on its CUDA-core path
// (the quantized activations go through global memory there).  This variant never allocates: the
// scratch is a fixed array that is part of the library image on every device that loads it.
//
// Cost and limits: every GPU that loads the library holds kNoAllocScratchBytes (4 MiB) until the
// process exits; a call needs N * (K / 32) * 36 bytes of it and is refused (status 9) beyond that.
// All calls share the one array: it keeps the previous call's blocks (every byte a call reads is
// written by that same call first, so nothing has to be cleared), and two calls that overlap in time
// on the GPU -- different streams, different host threads -- race on it.  Issue them on one stream.
//
// The first call on each device looks up the device address of the array (cudaGetSymbolAddress, with
// that device current).  That lookup is not a stream operation; make the first call on a device
// before starting any stream capture on it.  It is also the moment at which the CUDA runtime may load
// this library's device code onto that device and back the array with memory (module loading is lazy
// by default), so the free-memory figure can drop once, by about the size of the array and the code,
// during that first call and never afterwards: make it before the memory is capped or handed to
// another allocator.  Later calls change nothing on the device but the caller's C.
#include <cuda_runtime.h>

#include <atomic>
#include <cstdio>

#include "../../include/ppml_b200.h"
#include "kernels.h"

namespace {

constexpr size_t kNoAllocScratchBytes = PPML_B200_NOALLOC_SCRATCH_BYTES;

// In host code this name is only a handle for cudaGetSymbolAddress, never a pointer a kernel may use.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

constexpr int kMaxDevices = 64;
std::atomic<void*> g_scratch_addr[kMaxDevices];      // zero-initialised; two threads may both look up, same answer

// Device address of the scratch array on the current device (looked up once per device).
void* scratch_for_current_device() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) { cudaGetLastError(); return nullptr; }
    void* known = g_scratch_addr[dev].load(std::memory_order_acquire);
    if (known == nullptr) {
        void* ptr = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
        if (e != cudaSuccess || ptr == nullptr) {
            std::fprintf(stderr, "[ppml_b200] no-alloc scratch: cudaGetSymbolAddress failed on device %d: %s\n", dev,
                         cudaGetErrorString(e));
            cudaGetLastError();
            return nullptr;
        }
        g_scratch_addr[dev].store(ptr, std::memory_order_release);
        known = ptr;
    }
    return known;
}

}  // namespace

extern "C" {

int ppml_b200_mul_mat_q8_noalloc(const void* W, const float* X, float* C, int M, int N, int K, int wtype, int c_trans,
                                 const float* bias, void* stream) {
    using namespace ppml_b200;
    if (!W || !X || !C || M <= 0 || N <= 0 || K <= 0) return ST_BAD_ARGS;
    if ((K % 32) != 0) return ST_BAD_K;
    if (wtype < 0 || wtype > 2) return ST_WTYPE;
    const size_t need = static_cast<size_t>(N) * static_cast<size_t>(K / 32) * 36u;
    if (need > kNoAllocScratchBytes) {
        std::fprintf(stderr,
                     "[ppml_b200] mul_mat_q8_noalloc: %d tokens x K=%d need %zu bytes of scratch, the fixed array holds %zu; "
                     "split the token rows or use ppml_b200_mul_mat_q8\n", N, K, need, kNoAllocScratchBytes);
        return ST_TOO_LARGE;
    }
    void* scratch = scratch_for_current_device();
    if (!scratch) return ST_SCRATCH;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (launch_quantize_q8_1(X, scratch, static_cast<long long>(K) * N, st) != ST_OK) return ST_QUANT;
    return launch_q8_dp4a(W, scratch, C, M, N, K / 32, wtype, c_trans, bias, nullptr, st);
}

}  // extern "C"
