// Allocation-free variant of the ROSA suffix-automaton match.
//
// Who needs it: callers that must not allocate device memory while they run.
// Examples: a serving process whose host application handed it a fixed device
// memory budget and owns every byte itself; a latency-critical thread for
// which cudaMalloc / cudaFree are unacceptable because they may synchronise
// the whole device and take unbounded time; a plugin loaded into a process
// that has already reserved all of the GPU's memory for its own pool, so any
// further cudaMalloc simply fails.  Such callers already own their input and
// output buffers; what they cannot supply is the automaton's per-stream
// state, which the regular entry point (ullis_cuda_rosa_qkv_1bit_fwd) takes
// from a cudaMalloc'd pool that grows on demand.  Here that state lives in a
// fixed 64 MiB array that is part of the library image on every GPU that
// loads it, so the call neither allocates nor frees anything - not through
// the CUDA runtime and not on the host heap (errors are formatted into a
// fixed buffer).
//
// Consequences the caller must know:
//  * streams * state_bytes(time) must fit the 64 MiB; larger requests are
//    refused with ULLIS_CUDA_ERR_NOMEM, never split or spilled elsewhere.
//  * The first call on each device looks up the array's device address
//    (cudaGetSymbolAddress) and caches it.  Every call waits for `cuda_stream`
//    to drain before it returns, so it must never be issued on a stream that
//    is being captured - and the first call on a device, which also does the
//    look-up, should come before any capture starts anywhere in the process.
//  * The caller's current device is the same after the call as before it.
//  * Every call uses the same array and leaves its last contents behind.  The
//    kernel writes each field of a state block before reading it, so nothing
//    has to be cleared between calls - but two calls whose kernels overlap on
//    the GPU (different streams or host threads) would overwrite each
//    other's state: serialise them.
#include <cstdio>
#include <mutex>

#include "kernels.hpp"
#include "sam_core.cuh"

namespace {

constexpr size_t STATIC_SCRATCH_BYTES = (size_t)64 << 20;
constexpr int MAX_DEVICES = 64;

// File-scope device array: in host code this name is only a handle for
// cudaGetSymbolAddress, never a pointer a kernel could dereference.
static __device__ __align__(256) unsigned char g_sam_static_scratch[STATIC_SCRATCH_BYTES];

std::mutex g_setup_mutex;
unsigned char* g_scratch_addr[MAX_DEVICES] = {};

template <typename Ix>
__global__ void __launch_bounds__(128)
rosa_sam_static_kernel(unsigned char* __restrict__ scratch, size_t stride, const uint32_t* __restrict__ q_sw,
                       const uint32_t* __restrict__ k_sw, const uint32_t* __restrict__ v_sw,
                       uint32_t* __restrict__ idx_sw, size_t streams, uint32_t T, size_t wps) {
    // 4 streams per warp, as in the pooled kernel
    const int lane = threadIdx.x & 31;
    if (lane & 7) return;
    const size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const size_t s = warp * 4 + (lane >> 3);
    if (s >= streams) return;
    // run_euler reports "more states than 2T + 2" through its return value; an automaton over T symbols
    // never has that many, and the host has already checked that every block fits the array, so there is
    // nothing to report here
    (void)ullis::sam::run_euler<Ix>(scratch + s * stride, q_sw + s * wps, k_sw + s * wps, v_sw + s * wps,
                                    idx_sw + s * wps, T, nullptr);
}

int32_t refuse(int32_t code, const char* msg) {
    ullis::set_global_error(msg);
    return code;
}

int32_t refuse_cuda(const char* what, cudaError_t e) {
    char buf[256];
    snprintf(buf, sizeof(buf), "%s: %s", what, cudaGetErrorString(e));
    cudaGetLastError();   // the error is reported here: the next launch check of this thread must not see it again
    return refuse(ULLIS_CUDA_ERR_CUDA, buf);
}

// Puts the caller's current device back when the call leaves, whichever way.
struct DeviceRestore {
    int previous = -1;
    ~DeviceRestore() {
        if (previous >= 0) cudaSetDevice(previous);
    }
};

}  // namespace

extern "C" {

int32_t ullis_cuda_rosa_sam_static(int32_t device, void* cuda_stream, const uint32_t* q_sw, const uint32_t* k_sw,
                                   const uint32_t* v_sw, uint32_t* idx_sw, size_t streams, size_t time) {
    if (device < 0 || device >= MAX_DEVICES) return refuse(ULLIS_CUDA_ERR_ARG, "device index out of range");
    if (streams == 0 || time == 0) return refuse(ULLIS_CUDA_ERR_SHAPE, "ROSA dispatch dimensions must be non-zero");
    if (!q_sw || !k_sw || !v_sw || !idx_sw) return refuse(ULLIS_CUDA_ERR_ARG, "a device buffer pointer is null");
    if (time > 0x3FFFFFFFu) return refuse(ULLIS_CUDA_ERR_SHAPE, "ROSA time does not fit 32-bit state ids");
    const size_t stride = ullis::k::rosa_sam_scratch_bytes_per_stream(ULLIS_CUDA_SAM_EULER, time);
    if (streams > STATIC_SCRATCH_BYTES / stride) {
        char buf[256];
        snprintf(buf, sizeof(buf),
                 "request needs %zu x %zu bytes of automaton state; the built-in array holds %zu "
                 "(at most %zu streams at this length)",
                 streams, stride, STATIC_SCRATCH_BYTES, STATIC_SCRATCH_BYTES / stride);
        return refuse(ULLIS_CUDA_ERR_NOMEM, buf);
    }
    DeviceRestore restore;
    cudaError_t e = cudaGetDevice(&restore.previous);
    if (e != cudaSuccess) {
        restore.previous = -1;
        return refuse_cuda("cudaGetDevice", e);
    }
    e = cudaSetDevice(device);
    if (e != cudaSuccess) return refuse_cuda("cudaSetDevice", e);
    unsigned char* scratch = nullptr;
    {
        // once per device, with that device current
        std::lock_guard<std::mutex> lock(g_setup_mutex);
        if (!g_scratch_addr[device]) {
            void* p = nullptr;
            e = cudaGetSymbolAddress(&p, g_sam_static_scratch);
            if (e != cudaSuccess || !p)
                return refuse_cuda("cudaGetSymbolAddress", e);
            g_scratch_addr[device] = static_cast<unsigned char*>(p);
        }
        scratch = g_scratch_addr[device];
    }
    cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
    const size_t wps = (time + 31) / 32;
    const size_t warps = (streams + 3) / 4;
    const unsigned grid = (unsigned)((warps * 32 + 127) / 128);
    if (ullis::sam::node_capacity((uint32_t)time) <= 0xFFFFu)
        rosa_sam_static_kernel<uint16_t><<<grid, 128, 0, st>>>(scratch, stride, q_sw, k_sw, v_sw, idx_sw, streams,
                                                             (uint32_t)time, wps);
    else
        rosa_sam_static_kernel<uint32_t><<<grid, 128, 0, st>>>(scratch, stride, q_sw, k_sw, v_sw, idx_sw, streams,
                                                             (uint32_t)time, wps);
    e = cudaGetLastError();
    if (e != cudaSuccess) return refuse_cuda("kernel launch", e);
    e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return refuse_cuda("cudaStreamSynchronize", e);
    return ULLIS_CUDA_OK;
}

}  // extern "C"
