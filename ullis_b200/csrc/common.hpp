// Host-side plumbing shared by the CUDA backend: status/exception type, the
// runtime object behind `ullis_cuda_runtime`, and grow-only device buffers.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>
#include <vector>

#include "../../include/ullis_cuda.h"

struct ullis_cuda_runtime;

namespace ullis {

struct Error {
    int32_t code;
    std::string msg;
};

[[noreturn]] inline void fail(int32_t code, const std::string& msg) { throw Error{code, msg}; }

#define ULLIS_CUDA_CHECK(expr)                                                                   \
    do {                                                                                         \
        cudaError_t _e = (expr);                                                                 \
        if (_e != cudaSuccess)                                                                   \
            ::ullis::fail(ULLIS_CUDA_ERR_CUDA, std::string(#expr) + ": " + cudaGetErrorString(_e)); \
    } while (0)

// Grow-only device allocation (cudaMalloc'd; freed with the owner).
class DeviceBuffer {
   public:
    DeviceBuffer() = default;
    DeviceBuffer(const DeviceBuffer&) = delete;
    DeviceBuffer& operator=(const DeviceBuffer&) = delete;
    ~DeviceBuffer() { release(); }
    void release() {
        if (ptr_) cudaFree(ptr_);
        ptr_ = nullptr;
        bytes_ = 0;
    }
    void* ensure(size_t bytes) {
        if (bytes > bytes_) {
            release();
            size_t want = (bytes + 255) / 256 * 256;
            cudaError_t e = cudaMalloc(&ptr_, want);
            if (e != cudaSuccess) {
                ptr_ = nullptr;
                cudaGetLastError();
                fail(ULLIS_CUDA_ERR_NOMEM, "cudaMalloc of " + std::to_string(want) + " bytes failed: " +
                                               cudaGetErrorString(e));
            }
            bytes_ = want;
        }
        return ptr_;
    }
    template <typename T>
    T* as(size_t count) {
        return static_cast<T*>(ensure(count * sizeof(T)));
    }
    void* get() const { return ptr_; }
    size_t bytes() const { return bytes_; }

   private:
    void* ptr_ = nullptr;
    size_t bytes_ = 0;
};

struct NcclState;  // dp.cpp

// Sums `count` doubles at `dev` (device memory) over the ranks of the runtime's data-parallel group, in
// place, on the runtime stream; no host synchronisation.  Throws without a group.  (dp.cpp)
void dp_allreduce_device(ullis_cuda_runtime* rt, double* dev, size_t count);

// Message returned by ullis_cuda_last_error(NULL); copied into a fixed buffer.
void set_global_error(const char* msg);

}  // namespace ullis

// Device-side status word layout (one per runtime, zeroed before each call
// that uses it): 0 = ok, otherwise a kernel-specific code; slots 1..3 hold
// details (e.g. the offending row / stream).
enum { ULLIS_DEV_OK = 0, ULLIS_DEV_BAD_TOKEN = 1, ULLIS_DEV_SAM_CAPACITY = 2, ULLIS_DEV_SAM_NOMATCH = 3,
       ULLIS_DEV_WAIT_TIMEOUT = 4, ULLIS_DEV_FP16_RANGE = 5 };

struct ullis_cuda_runtime {
    int device = 0;
    cudaStream_t stream = nullptr;
    // a second stream for a kernel that has nothing to wait for on `stream` and that a latency-bound kernel there
    // leaves room for (the constant-q closed form beside the automaton pass); forked and joined with the two events
    cudaStream_t side_stream = nullptr;
    cudaEvent_t side_fork = nullptr, side_join = nullptr;
    bool sam_side = true;               // false: everything on `stream`
    int sm_count = 0;
    int cc_major = 0, cc_minor = 0;
    int mode = ULLIS_CUDA_MODE_FAST;
    int sam_algo = ULLIS_CUDA_SAM_EULER;
    bool sam_coop = true;               // warp-cooperative tour / pass 2 when the stream fits shared memory
    bool sam_coop_ready = false;
    bool sam_lanes_fixed = false;       // ULLIS_CUDA_SAM_LANES was given: no per-launch choice in pass 1
    uint32_t sam_sparse_per_sm = 40;    // pass 1 carries one stream per warp below this many streams per SM
    int sam_coop_threads = 0;           // threads per stream in the tour / pass 2 kernel (256, 512, 1024); 0 = from the shared memory a stream needs
    bool sam_words = true;              // pass 1 on packed state words (sam_core.cuh euler_pass1_words); false: the field-wise form
    bool sam_split = false;             // pass 1 as two kernels, extend chain then query walk, and the climb inside the tour kernel
                                        // (off: measured slower than the interleaved single-thread form at every stream count)
    int tc_ln_rows = 0;                 // rows per warp (1, 2, 4) in the LayerNorm + mix + operand kernel; 0 = by the number of rows
    int sam_smem_waves = 1;             // serial pass with the states in shared memory when the streams are expected to fit in this many rounds of resident CTAs; 0 = never, >= 1000 = always
    bool rowvec_smem_ready = false;     // the staged few-row FP16 matvec has been allowed its dynamic shared memory
    bool sam_smem_ready = false;        // that kernel has been allowed its dynamic shared memory
    // Streams that reached the automaton at each call site's last call, written by the serial-pass kernels straight
    // into pinned host memory (slot 0: callers without a site); 0xFFFFFFFF = no call yet.  Children share the parent's.
    static constexpr int SAM_HINT_SLOTS = 257;
    uint32_t* sam_hints = nullptr;
    uint32_t* sam_hint_slot(int site) {
        ullis_cuda_runtime* owner = parent ? parent : this;
        if (!owner->sam_hints) return nullptr;
        return owner->sam_hints + ((site >= 0 && site < SAM_HINT_SLOTS - 1) ? site + 1 : 0);
    }
    bool sam_reload_w = true;           // serial pass: load the query state's words once per step instead of carrying a patched copy
    bool sam_defer_climb = true;        // interleaved pass 1 records where each query walk ended; the climb to the state it reads runs in the tour kernel
    bool sam_walk_chunked = false;      // the query walk of the split form with eight lanes per stream (guessed pieces, then put right)
    int sam_lanes = 4;                  // streams carried per warp by the suffix-automaton kernel (1,2,4,...,32)
    uint64_t launches = 0;
    std::string last_error;
    uint32_t* dev_status = nullptr;     // 4 words, device
    uint32_t* host_status = nullptr;    // 4 words, pinned
    ullis::DeviceBuffer pool[24];       // op-level scratch slots
    size_t sam_budget_bytes = (size_t)12 << 30;   // cap of sam_scratch; more streams than fit run in waves
    ullis::DeviceBuffer sam_scratch;    // suffix-automaton state blocks
    ullis::DeviceBuffer sam_list;       // ids of the streams that need the automaton + their count
    size_t sam_last_streams = 0;        // streams of the last suffix-automaton call (where its counters sit in sam_list)
    ullis::DeviceBuffer tc_ws[16];      // 16-bit operands / partials of the tensor-core stages
    int tc_stages = 2, tc_stages2 = 2;  // GEMM pipeline depth with one / two activation operands
    bool tc_ws_kernel = true;           // weight-stationary persistent kernel for packed weights with K <= 512
    bool tc_ws2_kernel = true;          // ... and its CTA-pair form (256 x 256 tiles) for large M and N % 256 == 0
    size_t tc_ws2_min_rows = 4096;      // fewer rows than this stay with the single-CTA form (more, smaller row tiles)
    int tc_ws2_dense_clusters[2] = {0, 0};      // the same for dense weights (store, residual)
    int tc_ws2_clusters[5] = {0, 0, 0, 0, 0};   // CTA pairs of that kernel the device holds at once, per epilogue
    bool tc_fuse_ln = true;             // LayerNorm folded into the kernel that writes the 16-bit operands of the next GEMM
    bool tc_fix_list = true;            // exact sign recomputation from a compact list of the flagged outputs (one thread each)
    int tc_ready = 0;                   // 0 = not probed, 1 = usable, -1 = unusable on this device
    ullis::NcclState* nccl = nullptr;

    // Lanes: a model forward splits its batch into shares that run the whole pass on streams of their own, so
    // that one share's suffix-automaton kernels (bound by the latency of a serial chain, most issue slots idle)
    // run beside another share's GEMMs.  A share runs through a child runtime: its own stream, scratch buffers
    // and timing marks, the parent's settings and status words.  Children are created on demand, owned by the
    // parent and only ever used from inside a model call on the parent.
    int lanes = 1;                                   // shares a forward may use (1 = everything on `stream`, the default: see enqueue_hidden)
    ullis_cuda_runtime* parent = nullptr;            // set on a child
    std::vector<ullis_cuda_runtime*> children;
    cudaEvent_t lane_event = nullptr;                // parent: the fork point; child: the end of its share
    ullis_cuda_runtime* child(size_t i);             // child i (0-based), created on first use with the parent's settings
    size_t lanes_last = 1;                           // shares of the last suffix-automaton call (1 + children used)

    // Per-kernel device times: while enabled, an event is recorded behind every
    // launch; the stream is in order, so consecutive events bracket one kernel
    // (plus any small copy queued just before it).
    struct LaunchMark { const char* name; cudaEvent_t done; cudaEvent_t begin; bool side; };   // side: a kernel on side_stream, timed begin -> done
    bool kernel_timing = false;
    std::vector<LaunchMark> marks;
    size_t marks_used = 0;
    cudaEvent_t marks_start = nullptr;
    void kernel_timing_begin();
    void mark(const char* what);   // closes the current bracket under the name `what`
    void side_begin();             // kernel timing on: records the start of a side-stream kernel ...
    void side_end(const char* what);   // ... and its end, as an entry of its own in the table
    // total milliseconds and launches of the kernels recorded under `name` (all kernels when name is empty)
    void kernel_time(const char* name, float* total_ms, uint32_t* n_launches);
    size_t kernel_names(char* buf, size_t len);  // newline-separated distinct names; returns bytes needed

    void bind() const { ULLIS_CUDA_CHECK(cudaSetDevice(device)); }
    void sync() { ULLIS_CUDA_CHECK(cudaStreamSynchronize(stream)); }
    void h2d(void* dst, const void* src, size_t bytes) {
        if (bytes) ULLIS_CUDA_CHECK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, stream));
    }
    void d2h(void* dst, const void* src, size_t bytes) {
        if (bytes) ULLIS_CUDA_CHECK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, stream));
    }
    void zero(void* dst, size_t bytes) {
        if (bytes) ULLIS_CUDA_CHECK(cudaMemsetAsync(dst, 0, bytes, stream));
    }
    void clear_status() { zero(dev_status, 16); }
    // Synchronises and throws when a kernel reported a problem.
    void check_status();
    // Throws when host_status (already copied back and synchronised) holds a kernel's report.
    void throw_on_status();
    void launched(const char* what);  // counts a launch and checks the launch error
};
