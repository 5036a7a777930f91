// extern "C" surface declared in include/ullis_cuda.h: runtime lifecycle,
// the device-resident model entry points and the op-level calls that mirror
// the reference's MetalRuntime methods.  No C++ exception leaves this file.
#include <algorithm>
#include <cstdio>
#include <cstring>
#include <exception>
#include <new>

#include "kernels.hpp"
#include "linear_tc.hpp"
#include "generate.hpp"
#include "train.hpp"
#include "model.hpp"

using namespace ullis;

namespace {

char g_global_error[512] = "";  // last failure of a call that had no runtime to blame (fixed buffer: no allocation)

template <typename F>
int32_t guard(ullis_cuda_runtime* rt, F&& body) {
    if (!rt) {
        set_global_error("runtime handle is null");
        return ULLIS_CUDA_ERR_ARG;
    }
    try {
        rt->bind();
        body();
        return ULLIS_CUDA_OK;
    } catch (const Error& e) {
        rt->last_error = e.msg;
        return e.code;
    } catch (const std::bad_alloc&) {
        rt->last_error = "host allocation failed";
        return ULLIS_CUDA_ERR_NOMEM;
    } catch (const std::exception& e) {
        rt->last_error = e.what();
        return ULLIS_CUDA_ERR_ARG;
    }
}

template <typename F>
int32_t guard_model(ullis_cuda_model* m, F&& body) {
    if (!m) {
        set_global_error("model handle is null");
        return ULLIS_CUDA_ERR_ARG;
    }
    return guard(m->rt, body);
}

void need_ptr(const void* p, const char* name) {
    if (!p) fail(ULLIS_CUDA_ERR_ARG, std::string(name) + " is null");
}

size_t mul_or_fail(size_t a, size_t b, const char* what) {
    if (b != 0 && a > SIZE_MAX / b) fail(ULLIS_CUDA_ERR_SHAPE, std::string(what) + " shape overflow");
    return a * b;
}

template <typename T>
T* stage(ullis_cuda_runtime* rt, int slot, const T* host, size_t count) {
    T* dev = rt->pool[slot].as<T>(count ? count : 1);
    rt->h2d(dev, host, count * sizeof(T));
    return dev;
}

void packed_linear_dev(ullis_cuda_runtime* rt, const float* x, const uint32_t* bits, const uint16_t* scale,
                       const uint16_t* bias, float* y, size_t rows, size_t K, size_t N) {
    if (rt->mode == ULLIS_CUDA_MODE_EXACT || !tc::binary_linear(rt, x, bits, scale, bias, y, rows, K, N))
        k::binary_linear_exact(rt, x, bits, scale, bias, y, rows, K, N, false);
}

void dense_linear_dev(ullis_cuda_runtime* rt, const float* x, const uint16_t* w, float* y, size_t rows, size_t K,
                      size_t N) {
    if (rt->mode == ULLIS_CUDA_MODE_EXACT || !tc::fp16_linear(rt, x, w, y, rows, K, N))
        k::fp16_linear_exact(rt, x, w, y, rows, K, N, false);
}

}  // namespace

namespace ullis {
void set_global_error(const char* msg) {
    snprintf(g_global_error, sizeof(g_global_error), "%s", msg ? msg : "");
}
}  // namespace ullis

// Child runtime i of a lane-splitting forward: a stream, scratch and timing marks of its own; everything that
// configures kernels is copied from the parent on every request, and the status words are the parent's.
ullis_cuda_runtime* ullis_cuda_runtime::child(size_t i) {
    while (children.size() <= i) {
        ullis_cuda_runtime* c = new ullis_cuda_runtime();
        children.push_back(c);
        c->parent = this;
        c->device = device;
        c->sm_count = sm_count;
        c->cc_major = cc_major;
        c->cc_minor = cc_minor;
        c->dev_status = dev_status;     // shared: a kernel of any share reports into the parent's words
        c->host_status = host_status;
        c->lanes = 1;
        ULLIS_CUDA_CHECK(cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking));
        ULLIS_CUDA_CHECK(cudaEventCreateWithFlags(&c->lane_event, cudaEventDisableTiming));
    }
    ullis_cuda_runtime* c = children[i];
    c->mode = mode;
    c->sam_algo = sam_algo;
    c->sam_coop = sam_coop;
    c->sam_side = sam_side;
    c->sam_lanes = sam_lanes;
    c->sam_lanes_fixed = sam_lanes_fixed;
    c->sam_sparse_per_sm = sam_sparse_per_sm;
    c->sam_coop_threads = sam_coop_threads;
    c->sam_words = sam_words;
    c->sam_split = sam_split;
    c->sam_defer_climb = sam_defer_climb;
    c->sam_reload_w = sam_reload_w;
    c->sam_smem_waves = sam_smem_waves;
    c->tc_ln_rows = tc_ln_rows;
    c->sam_walk_chunked = sam_walk_chunked;
    c->sam_budget_bytes = sam_budget_bytes / (children.size() + 1);
    c->tc_fix_list = tc_fix_list;
    c->tc_fuse_ln = tc_fuse_ln;
    c->tc_stages = tc_stages;
    c->tc_stages2 = tc_stages2;
    c->tc_ws2_min_rows = tc_ws2_min_rows;
    if (c->kernel_timing != kernel_timing) {
        c->kernel_timing = kernel_timing;
        if (kernel_timing) c->kernel_timing_begin();
    }
    return c;
}

void ullis_cuda_runtime::launched(const char* what) {
    ++launches;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) fail(ULLIS_CUDA_ERR_CUDA, std::string("launch of ") + what + ": " + cudaGetErrorString(e));
    if (kernel_timing) mark(what);
}

static void ensure_mark(ullis_cuda_runtime* rt) {
    if (rt->marks_used == rt->marks.size()) {
        ullis_cuda_runtime::LaunchMark m{"", nullptr, nullptr, false};
        ULLIS_CUDA_CHECK(cudaEventCreate(&m.done));
        rt->marks.push_back(m);
    }
}

void ullis_cuda_runtime::mark(const char* what) {
    ensure_mark(this);
    marks[marks_used].name = what;
    marks[marks_used].side = false;
    ULLIS_CUDA_CHECK(cudaEventRecord(marks[marks_used].done, stream));
    ++marks_used;
}

void ullis_cuda_runtime::side_begin() {
    ensure_mark(this);
    if (!marks[marks_used].begin) ULLIS_CUDA_CHECK(cudaEventCreate(&marks[marks_used].begin));
    ULLIS_CUDA_CHECK(cudaEventRecord(marks[marks_used].begin, side_stream));
}

void ullis_cuda_runtime::side_end(const char* what) {
    marks[marks_used].name = what;
    marks[marks_used].side = true;
    ULLIS_CUDA_CHECK(cudaEventRecord(marks[marks_used].done, side_stream));
    ++marks_used;
}

void ullis_cuda_runtime::kernel_timing_begin() {
    if (!marks_start) ULLIS_CUDA_CHECK(cudaEventCreate(&marks_start));
    marks_used = 0;
    ULLIS_CUDA_CHECK(cudaEventRecord(marks_start, stream));
}

void ullis_cuda_runtime::kernel_time(const char* name, float* total_ms, uint32_t* n_launches) {
    sync();
    float total = 0.f;
    uint32_t n = 0;
    for (ullis_cuda_runtime* c : children) {   // the shares of a lane-splitting forward ran on these
        float t = 0.f;
        uint32_t k = 0;
        if (c->kernel_timing) c->kernel_time(name, &t, &k);
        total += t;
        n += k;
    }
    if (side_stream) ULLIS_CUDA_CHECK(cudaStreamSynchronize(side_stream));
    cudaEvent_t previous = marks_start;   // end of the last kernel on `stream`
    for (size_t i = 0; i < marks_used; ++i) {
        const cudaEvent_t from = marks[i].side ? marks[i].begin : previous;
        if (!marks[i].side) previous = marks[i].done;
        if (name && name[0] && std::strcmp(name, marks[i].name) != 0) continue;
        float t = 0.f;
        ULLIS_CUDA_CHECK(cudaEventElapsedTime(&t, from, marks[i].done));
        total += t;
        ++n;
    }
    if (total_ms) *total_ms = total;
    if (n_launches) *n_launches = n;
}

size_t ullis_cuda_runtime::kernel_names(char* buf, size_t len) {
    std::vector<const char*> seen;
    std::string out;
    auto collect = [&](const ullis_cuda_runtime* r) {
        for (size_t i = 0; i < r->marks_used; ++i) {
            bool dup = false;
            for (const char* s : seen) dup = dup || std::strcmp(s, r->marks[i].name) == 0;
            if (dup) continue;
            seen.push_back(r->marks[i].name);
            out += r->marks[i].name;
            out += '\n';
        }
    };
    collect(this);
    for (const ullis_cuda_runtime* c : children)
        if (c->kernel_timing) collect(c);
    if (buf && len) {
        const size_t n = out.size() < len - 1 ? out.size() : len - 1;
        std::memcpy(buf, out.data(), n);
        buf[n] = 0;
    }
    return out.size() + 1;
}

void ullis_cuda_runtime::check_status() {
    d2h(host_status, dev_status, 16);
    sync();
    throw_on_status();
}

void ullis_cuda_runtime::throw_on_status() {
    const uint32_t code = host_status[0];
    if (code == ULLIS_DEV_OK) return;
    if (code == ULLIS_DEV_BAD_TOKEN)
        fail(ULLIS_CUDA_ERR_TOKEN, "token id exceeds vocabulary (row " + std::to_string(host_status[1]) + ")");
    if (code == ULLIS_DEV_FP16_RANGE)
        fail(ULLIS_CUDA_ERR_DEVICE_CHECK,
             "an activation exceeds the FP16 range of the tensor-core operands (row " + std::to_string(host_status[1]) +
                 "); use ULLIS_CUDA_MODE_EXACT for this input");
    if (code == ULLIS_DEV_WAIT_TIMEOUT)
        fail(ULLIS_CUDA_ERR_TIMEOUT, "a kernel gave up waiting (site " + std::to_string(host_status[1]) + ")");
    fail(ULLIS_CUDA_ERR_DEVICE_CHECK, "device-side check failed, code " + std::to_string(code) + " detail " +
                                          std::to_string(host_status[1]));
}

extern "C" {

int32_t ullis_cuda_runtime_create(int32_t device, ullis_cuda_runtime** out) {
    if (!out) {
        set_global_error("out is null");
        return ULLIS_CUDA_ERR_ARG;
    }
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0) {
        cudaGetLastError();
        set_global_error((std::string("--backend cuda requires a CUDA device: ") +
                          (e != cudaSuccess ? cudaGetErrorString(e) : "no device found")).c_str());
        return ULLIS_CUDA_ERR_CUDA;
    }
    if (device < 0 || device >= count) {
        set_global_error("device index out of range");
        return ULLIS_CUDA_ERR_ARG;
    }
    ullis_cuda_runtime* rt = new (std::nothrow) ullis_cuda_runtime();
    if (!rt) {
        set_global_error("host allocation failed");
        return ULLIS_CUDA_ERR_NOMEM;
    }
    rt->device = device;
    try {
        rt->bind();
        cudaDeviceProp prop;
        ULLIS_CUDA_CHECK(cudaGetDeviceProperties(&prop, device));
        rt->sm_count = prop.multiProcessorCount;
        rt->cc_major = prop.major;
        rt->cc_minor = prop.minor;
        ULLIS_CUDA_CHECK(cudaStreamCreateWithFlags(&rt->stream, cudaStreamNonBlocking));
        ULLIS_CUDA_CHECK(cudaMalloc(&rt->dev_status, 16));
        ULLIS_CUDA_CHECK(cudaMallocHost(&rt->host_status, 16));
        {   // mapped pinned memory: the kernels store into it, the host reads it without a copy or a wait
            void* hints = nullptr;
            ULLIS_CUDA_CHECK(cudaHostAlloc(&hints, ullis_cuda_runtime::SAM_HINT_SLOTS * sizeof(uint32_t), cudaHostAllocMapped));
            rt->sam_hints = static_cast<uint32_t*>(hints);
            for (int i = 0; i < ullis_cuda_runtime::SAM_HINT_SLOTS; ++i) rt->sam_hints[i] = 0xFFFFFFFFu;
            void* dev_view = nullptr;
            ULLIS_CUDA_CHECK(cudaHostGetDevicePointer(&dev_view, hints, 0));
            if (dev_view != hints) {   // no unified addressing of host memory: the kernels cannot be handed the host pointer
                cudaFreeHost(hints);
                rt->sam_hints = nullptr;
            }
        }
        rt->clear_status();
        rt->sync();
        if (const char* env = getenv("ULLIS_CUDA_TC_STAGES")) {
            const int a = atoi(env) / 10, b = atoi(env) % 10;   // e.g. 32 = 3 stages (one operand), 2 stages (two)
            if (a >= 2 && a <= 4 && b >= 2 && b <= 4) { rt->tc_stages = a; rt->tc_stages2 = b; }
        }
        if (const char* env = getenv("ULLIS_CUDA_SAM_COOP")) rt->sam_coop = atoi(env) != 0;
        if (const char* env = getenv("ULLIS_CUDA_SAM_BUDGET_MB")) {
            const long mb = atol(env);
            if (mb > 0) rt->sam_budget_bytes = (size_t)mb << 20;
        }
        if (const char* env = getenv("ULLIS_CUDA_SAM_SPARSE")) rt->sam_sparse_per_sm = (uint32_t)std::max(0, atoi(env));
        if (const char* env = getenv("ULLIS_CUDA_SAM_WORDS")) rt->sam_words = atoi(env) != 0;
        if (const char* env = getenv("ULLIS_CUDA_FUSE_LN")) rt->tc_fuse_ln = atoi(env) != 0;
        if (const char* env = getenv("ULLIS_CUDA_FIX_LIST")) rt->tc_fix_list = atoi(env) != 0;
        if (const char* env = getenv("ULLIS_CUDA_SAM_WALK_CHUNKED")) rt->sam_walk_chunked = atoi(env) != 0;
        if (const char* env = getenv("ULLIS_CUDA_LN_ROWS")) rt->tc_ln_rows = atoi(env);
        if (const char* env = getenv("ULLIS_CUDA_SAM_SMEM_WAVES")) rt->sam_smem_waves = std::max(0, atoi(env));
        if (const char* env = getenv("ULLIS_CUDA_SAM_RELOAD_W")) rt->sam_reload_w = atoi(env) != 0;
        if (const char* env = getenv("ULLIS_CUDA_SAM_DEFER_CLIMB")) rt->sam_defer_climb = atoi(env) != 0;
        if (const char* env = getenv("ULLIS_CUDA_SAM_SPLIT")) rt->sam_split = atoi(env) != 0;
        if (const char* env = getenv("ULLIS_CUDA_SAM_SIDE")) rt->sam_side = atoi(env) != 0;
        if (const char* env = getenv("ULLIS_CUDA_LANES")) rt->lanes = std::min(16, std::max(1, atoi(env)));
        if (const char* env = getenv("ULLIS_CUDA_SAM_COOP_THREADS")) {
            const int v = atoi(env);
            if (v == 256 || v == 512 || v == 1024) rt->sam_coop_threads = v;
        }
        if (const char* env = getenv("ULLIS_CUDA_SAM_LANES")) {
            const int v = atoi(env);
            if (v == 1 || v == 2 || v == 4 || v == 8 || v == 16 || v == 32) {
                rt->sam_lanes = v;
                rt->sam_lanes_fixed = true;
            }
        }
    } catch (const Error& err) {
        set_global_error(err.msg.c_str());
        ullis_cuda_runtime_destroy(rt);
        return err.code;
    }
    *out = rt;
    return ULLIS_CUDA_OK;
}

void ullis_cuda_runtime_destroy(ullis_cuda_runtime* rt) {
    if (!rt) return;
    cudaSetDevice(rt->device);
    for (ullis_cuda_runtime* c : rt->children) {
        c->dev_status = nullptr;    // the parent's
        c->host_status = nullptr;
        ullis_cuda_runtime_destroy(c);
    }
    rt->children.clear();
    if (rt->lane_event) cudaEventDestroy(rt->lane_event);
    ullis_cuda_dp_finalize(rt);
    if (rt->stream) {
        cudaStreamSynchronize(rt->stream);
        cudaStreamDestroy(rt->stream);
    }
    if (rt->side_stream) {
        cudaStreamSynchronize(rt->side_stream);
        cudaStreamDestroy(rt->side_stream);
    }
    if (rt->side_fork) cudaEventDestroy(rt->side_fork);
    if (rt->side_join) cudaEventDestroy(rt->side_join);
    if (rt->dev_status) cudaFree(rt->dev_status);
    if (rt->host_status) cudaFreeHost(rt->host_status);
    if (rt->sam_hints) cudaFreeHost(rt->sam_hints);
    for (auto& m : rt->marks) {
        cudaEventDestroy(m.done);
        if (m.begin) cudaEventDestroy(m.begin);
    }
    if (rt->marks_start) cudaEventDestroy(rt->marks_start);
    delete rt;
}

const char* ullis_cuda_last_error(const ullis_cuda_runtime* rt) {
    return rt ? rt->last_error.c_str() : g_global_error;
}

int32_t ullis_cuda_runtime_set_mode(ullis_cuda_runtime* rt, int32_t mode) {
    return guard(rt, [&] {
        if (mode != ULLIS_CUDA_MODE_FAST && mode != ULLIS_CUDA_MODE_EXACT) fail(ULLIS_CUDA_ERR_ARG, "unknown mode");
        rt->mode = mode;
    });
}

int32_t ullis_cuda_runtime_set_sam(ullis_cuda_runtime* rt, int32_t sam_algo) {
    return guard(rt, [&] {
        if (sam_algo != ULLIS_CUDA_SAM_EULER && sam_algo != ULLIS_CUDA_SAM_EAGER)
            fail(ULLIS_CUDA_ERR_ARG, "unknown suffix-automaton schedule");
        rt->sam_algo = sam_algo;
    });
}

int32_t ullis_cuda_runtime_synchronize(ullis_cuda_runtime* rt) {
    return guard(rt, [&] { rt->sync(); });
}

void* ullis_cuda_runtime_stream(ullis_cuda_runtime* rt) { return rt ? (void*)rt->stream : nullptr; }

uint64_t ullis_cuda_runtime_launch_count(const ullis_cuda_runtime* rt) {
    if (!rt) return 0;
    uint64_t n = rt->launches;
    for (const ullis_cuda_runtime* c : rt->children) n += c->launches;
    return n;
}

int32_t ullis_cuda_runtime_kernel_timing(ullis_cuda_runtime* rt, int32_t enabled) {
    return guard(rt, [&] {
        rt->bind();
        rt->kernel_timing = enabled != 0;
        if (rt->kernel_timing) rt->kernel_timing_begin();
        for (size_t i = 0; i < rt->children.size(); ++i) {
            rt->children[i]->kernel_timing = false;   // re-armed (from a fresh start event) when a forward next uses it
            rt->children[i]->marks_used = 0;
        }
    });
}

int32_t ullis_cuda_runtime_kernel_time(ullis_cuda_runtime* rt, const char* name, float* total_ms, uint32_t* launches) {
    return guard(rt, [&] {
        rt->bind();
        rt->kernel_time(name, total_ms, launches);
    });
}

int32_t ullis_cuda_runtime_kernel_names(ullis_cuda_runtime* rt, char* buf, size_t len, size_t* needed) {
    return guard(rt, [&] {
        const size_t n = rt->kernel_names(buf, len);
        if (needed) *needed = n;
    });
}

int32_t ullis_cuda_runtime_sam_counts(ullis_cuda_runtime* rt, uint64_t* total, uint64_t* automaton,
                                      uint64_t* constant_q) {
    return guard(rt, [&] {
        uint64_t sum[3] = {0, 0, 0};
        for (size_t lane = 0; lane < rt->lanes_last; ++lane) {
            ullis_cuda_runtime* r = lane == 0 ? rt : rt->children.at(lane - 1);
            uint32_t host[2] = {0, 0};
            if (r->sam_last_streams) {
                // the two counters sit behind the automaton list (k::rosa_sam)
                r->d2h(host, r->sam_list.as<uint32_t>(2 * r->sam_last_streams + 2) + r->sam_last_streams, 8);
                r->sync();
            }
            sum[0] += r->sam_last_streams;
            sum[1] += host[0];
            sum[2] += host[1];
        }
        if (total) *total = sum[0];
        if (automaton) *automaton = sum[1];
        if (constant_q) *constant_q = sum[2];
    });
}

int32_t ullis_cuda_runtime_wait_selftest(ullis_cuda_runtime* rt, uint32_t polls) {
    return guard(rt, [&] {
        if (polls == 0 || polls > (1u << 20)) fail(ULLIS_CUDA_ERR_ARG, "polls must be in 1..2^20");
        rt->clear_status();
        tc::wait_selftest(rt, polls);
        rt->check_status();   // throws ULLIS_CUDA_ERR_TIMEOUT: that is the expected outcome
        fail(ULLIS_CUDA_ERR_DEVICE_CHECK, "the wait did not time out");
    });
}

int32_t ullis_cuda_runtime_is_sm100(const ullis_cuda_runtime* rt) { return rt && rt->cc_major == 10 ? 1 : 0; }

// ------------------------------------------------------------------ model

int32_t ullis_cuda_model_load_safetensors(ullis_cuda_runtime* rt, const uint8_t* bytes, size_t len,
                                          ullis_cuda_model** out) {
    return guard(rt, [&] {
        need_ptr(out, "out");
        *out = nullptr;
        need_ptr(bytes, "bytes");
        ullis_cuda_model* m = new ullis_cuda_model();
        m->rt = rt;
        try {
            m->load(bytes, len);
        } catch (...) {
            delete m;
            throw;
        }
        *out = m;
    });
}

void ullis_cuda_model_destroy(ullis_cuda_model* model) {
    if (!model) return;
    cudaSetDevice(model->rt->device);
    cudaStreamSynchronize(model->rt->stream);
    delete model;
}

int32_t ullis_cuda_model_dims(const ullis_cuda_model* model, size_t dims[6]) {
    if (!model || !dims) return ULLIS_CUDA_ERR_ARG;
    dims[0] = model->d;
    dims[1] = model->layers;
    dims[2] = model->vocab;
    dims[3] = model->context_len;
    dims[4] = model->batch_size;
    dims[5] = model->ffn;
    return ULLIS_CUDA_OK;
}

int32_t ullis_cuda_model_forward_ce(ullis_cuda_model* model, const uint32_t* tokens, const uint32_t* labels,
                                    uint32_t ignore_id, size_t batch, size_t time, float* mean_loss,
                                    double* loss_sum, uint64_t* n_valid, float* row_loss) {
    return guard_model(model, [&] {
        need_ptr(labels, "labels");
        model->upload_tokens(tokens, labels, batch, time);
        model->enqueue_forward_ce(ignore_id, batch, time);
        model->read_loss(mean_loss, loss_sum, n_valid, row_loss, batch * time);
    });
}

int32_t ullis_cuda_model_upload_tokens(ullis_cuda_model* model, const uint32_t* tokens, const uint32_t* labels,
                                       size_t batch, size_t time) {
    return guard_model(model, [&] { model->upload_tokens(tokens, labels, batch, time); });
}

int32_t ullis_cuda_model_enqueue_forward_ce(ullis_cuda_model* model, uint32_t ignore_id, size_t batch,
                                            size_t time) {
    return guard_model(model, [&] { model->enqueue_forward_ce(ignore_id, batch, time); });
}

int32_t ullis_cuda_model_read_loss_global(ullis_cuda_model* model, float* mean_loss, double* loss_sum,
                                          uint64_t* n_valid) {
    return guard_model(model, [&] { model->read_loss_global(mean_loss, loss_sum, n_valid); });
}

int32_t ullis_cuda_model_read_loss(ullis_cuda_model* model, float* mean_loss, double* loss_sum,
                                   uint64_t* n_valid, float* row_loss, size_t rows) {
    return guard_model(model, [&] { model->read_loss(mean_loss, loss_sum, n_valid, row_loss, rows); });
}

int32_t ullis_cuda_model_logits(ullis_cuda_model* model, const uint32_t* tokens, size_t batch, size_t time,
                                float* logits) {
    return guard_model(model, [&] {
        need_ptr(logits, "logits");
        model->upload_tokens(tokens, nullptr, batch, time);
        model->enqueue_logits(batch, time, logits);
    });
}

int32_t ullis_cuda_model_hidden(ullis_cuda_model* model, const uint32_t* tokens, size_t batch, size_t time,
                                float* hidden) {
    return guard_model(model, [&] {
        need_ptr(hidden, "hidden");
        model->upload_tokens(tokens, nullptr, batch, time);
        model->enqueue_hidden(batch, time);
        model->rt->d2h(hidden, model->a.get(), batch * time * model->d * 4);
        model->rt->check_status();
    });
}

int32_t ullis_cuda_model_set_taps(ullis_cuda_model* model, int32_t enabled) {
    return guard_model(model, [&] {
        model->taps_enabled = enabled != 0;
        if (!enabled) {
            model->tap_bufs.clear();
            model->tap_rows = 0;
        }
    });
}

int32_t ullis_cuda_model_tap(ullis_cuda_model* model, int32_t layer, int32_t which, void* out, size_t bytes) {
    return guard_model(model, [&] {
        need_ptr(out, "out");
        model->tap(layer, which, out, bytes);
    });
}

int32_t ullis_cuda_model_set_profile(ullis_cuda_model* model, int32_t enabled) {
    return guard_model(model, [&] {
        model->profile = enabled != 0;
        model->spans_used = 0;
    });
}

int32_t ullis_cuda_model_phase_ms(ullis_cuda_model* model, float ms[6]) {
    return guard_model(model, [&] {
        need_ptr(ms, "ms");
        model->phase_ms(ms);
    });
}

// ---------------------------------------------------------------- op level

// ------------------------------------------------------------------ generate

int32_t ullis_cuda_generate_state_create(ullis_cuda_model* model, size_t batch, ullis_cuda_generate_state** out) {
    return guard_model(model, [&] {
        need_ptr(out, "out");
        *out = nullptr;
        *out = new ullis_cuda_generate_state(model, batch);
    });
}

void ullis_cuda_generate_state_destroy(ullis_cuda_generate_state* state) {
    if (!state) return;
    if (state->model && state->model->rt) cudaSetDevice(state->model->rt->device);
    delete state;
}

int32_t ullis_cuda_generate_state_reset(ullis_cuda_generate_state* state) {
    if (!state) {
        set_global_error("generate state handle is null");
        return ULLIS_CUDA_ERR_ARG;
    }
    return guard_model(state->model, [&] { state->reset(); });
}

size_t ullis_cuda_generate_state_time(const ullis_cuda_generate_state* state) { return state ? state->time : 0; }

int32_t ullis_cuda_generate_step(ullis_cuda_generate_state* state, const uint32_t* tokens, float* logits) {
    if (!state) {
        set_global_error("generate state handle is null");
        return ULLIS_CUDA_ERR_ARG;
    }
    return guard_model(state->model, [&] {
        need_ptr(tokens, "tokens");
        need_ptr(logits, "logits");
        state->step(tokens, logits);
    });
}

int32_t ullis_cuda_rosa_pushers_create(ullis_cuda_runtime* rt, size_t streams, size_t capacity,
                                       ullis_cuda_rosa_pushers** out) {
    return guard(rt, [&] {
        need_ptr(out, "out");
        *out = nullptr;
        *out = new ullis_cuda_rosa_pushers(rt, streams, capacity);
    });
}

void ullis_cuda_rosa_pushers_destroy(ullis_cuda_rosa_pushers* pushers) {
    if (!pushers) return;
    if (pushers->rt) cudaSetDevice(pushers->rt->device);
    delete pushers;
}

int32_t ullis_cuda_rosa_pushers_reset(ullis_cuda_rosa_pushers* pushers) {
    if (!pushers) {
        set_global_error("ROSA pushers handle is null");
        return ULLIS_CUDA_ERR_ARG;
    }
    return guard(pushers->rt, [&] { pushers->reset(); });
}

int32_t ullis_cuda_rosa_pushers_push(ullis_cuda_rosa_pushers* pushers, const uint8_t* q, const uint8_t* k,
                                     const uint8_t* v, size_t steps, uint8_t* idx) {
    if (!pushers) {
        set_global_error("ROSA pushers handle is null");
        return ULLIS_CUDA_ERR_ARG;
    }
    return guard(pushers->rt, [&] {
        need_ptr(q, "q"); need_ptr(k, "k"); need_ptr(v, "v"); need_ptr(idx, "idx");
        pushers->push(q, k, v, steps, idx);
    });
}

// --------------------------------------------------------------------- train

int32_t ullis_cuda_train_state_create(ullis_cuda_model* model, const uint8_t* checkpoint, size_t len,
                                      ullis_cuda_train_state** out) {
    return guard_model(model, [&] {
        need_ptr(out, "out");
        *out = nullptr;
        *out = new ullis_cuda_train_state(model, checkpoint, len);
    });
}

void ullis_cuda_train_state_destroy(ullis_cuda_train_state* state) {
    if (!state) return;
    if (state->rt) cudaSetDevice(state->rt->device);
    delete state;
}

int32_t ullis_cuda_model_train_step(ullis_cuda_train_state* state, const uint32_t* tokens, const uint32_t* labels,
                                    uint32_t ignore_id, size_t batch, size_t time, float learning_rate,
                                    ullis_cuda_train_result* result) {
    if (!state) {
        set_global_error("train state handle is null");
        return ULLIS_CUDA_ERR_ARG;
    }
    return guard_model(state->m, [&] { state->step(tokens, labels, ignore_id, batch, time, learning_rate, result); });
}

int32_t ullis_cuda_train_state_read(ullis_cuda_train_state* state, const char* name, void* dst, size_t bytes) {
    if (!state) {
        set_global_error("train state handle is null");
        return ULLIS_CUDA_ERR_ARG;
    }
    return guard_model(state->m, [&] {
        need_ptr(dst, "dst");
        state->read(name, dst, bytes);
    });
}

int32_t ullis_cuda_train_state_install_head_unigram_prior(ullis_cuda_train_state* state, const uint32_t* labels,
                                                          size_t n, uint32_t ignore_id,
                                                          ullis_cuda_head_unigram_install* result) {
    if (!state) {
        set_global_error("train state handle is null");
        return ULLIS_CUDA_ERR_ARG;
    }
    return guard_model(state->m, [&] { state->install_head_unigram_prior(labels, n, ignore_id, result); });
}

namespace {
// clipped (ste_scale < 0) or BinaryConnect step of n elements through pool slots 0..3
void sgd_op(ullis_cuda_runtime* rt, const uint16_t* parameters, const float* residual, const float* gradient, float lr,
            float ste_scale, size_t n, uint16_t* next_parameters, float* next_residual, uint32_t* next_bits,
            const char* what) {
    if (n == 0) return;
    need_ptr(parameters, "parameters"); need_ptr(residual, "residual"); need_ptr(gradient, "gradient");
    need_ptr(next_parameters, "next_parameters"); need_ptr(next_residual, "next_residual");
    (void)what;
    uint16_t* dw = stage(rt, 0, parameters, n);
    float* dr = stage(rt, 1, residual, n);
    float* dg = stage(rt, 2, gradient, n);
    uint32_t* dbits = next_bits ? rt->pool[3].as<uint32_t>((n + 31) / 32) : nullptr;
    if (ste_scale < 0.0f)
        k::clipped_sgd(rt, dw, dr, dg, lr, n);
    else
        k::latent_sgd(rt, dw, dr, dg, lr, ste_scale, dbits, n);
    rt->d2h(next_parameters, dw, n * 2);
    rt->d2h(next_residual, dr, n * 4);
    if (next_bits) rt->d2h(next_bits, dbits, (n + 31) / 32 * 4);
    rt->sync();
}
}  // namespace

int32_t ullis_cuda_clipped_sgd_fp16(ullis_cuda_runtime* rt, const uint16_t* parameters, const float* residual,
                                    const float* gradient, float learning_rate, size_t n, uint16_t* next_parameters,
                                    float* next_residual) {
    return guard(rt, [&] {
        sgd_op(rt, parameters, residual, gradient, learning_rate, -1.0f, n, next_parameters, next_residual, nullptr,
               "clipped");
    });
}

int32_t ullis_cuda_binaryconnect_sgd_fp16(ullis_cuda_runtime* rt, const uint16_t* parameters, const float* residual,
                                          const float* gradient, float learning_rate, size_t n,
                                          uint16_t* next_parameters, float* next_residual) {
    return guard(rt, [&] {
        sgd_op(rt, parameters, residual, gradient, learning_rate, 1.0f, n, next_parameters, next_residual, nullptr,
               "binaryconnect");
    });
}

int32_t ullis_cuda_apply_latent_sgd(ullis_cuda_runtime* rt, const uint16_t* latent, const float* residual,
                                    const float* gradient, float learning_rate, float ste_scale, size_t n,
                                    uint16_t* next_latent, float* next_residual, uint32_t* next_bits) {
    return guard(rt, [&] {
        if (n) need_ptr(next_bits, "next_bits");
        if (!(ste_scale >= 0.0f)) fail(ULLIS_CUDA_ERR_ARG, "ste_scale must be non-negative");
        sgd_op(rt, latent, residual, gradient, learning_rate, ste_scale, n, next_latent, next_residual, next_bits,
               "latent");
    });
}

int32_t ullis_cuda_rosa_qkv_1bit_bwd_e(ullis_cuda_runtime* rt, const float* output_gradient, const uint8_t* idx,
                                       size_t batch, size_t time, size_t channels, float* g_e) {
    return guard(rt, [&] {
        if (channels == 0) fail(ULLIS_CUDA_ERR_SHAPE, "ROSA g_e shape mismatch");
        const size_t rows = mul_or_fail(batch, time, "ROSA g_e"), n = mul_or_fail(rows, channels, "ROSA g_e");
        need_ptr(g_e, "g_e");
        float* dge = rt->pool[2].as<float>(channels);
        if (n == 0) {
            rt->zero(dge, channels * 4);
        } else {
            need_ptr(output_gradient, "output_gradient"); need_ptr(idx, "idx");
            float* dgy = stage(rt, 0, output_gradient, n);
            uint8_t* didx = stage(rt, 1, idx, n);
            k::rosa_e_grad(rt, dgy, didx, dge, rows, channels, rt->pool[3]);
        }
        rt->d2h(g_e, dge, channels * 4);
        rt->sync();
    });
}

int32_t ullis_cuda_cmix_relu2_backward(ullis_cuda_runtime* rt, const float* input, const float* output_gradient,
                                       float* gx, size_t n) {
    return guard(rt, [&] {
        if (n == 0) return;
        need_ptr(input, "input"); need_ptr(output_gradient, "output_gradient"); need_ptr(gx, "gx");
        float* din = stage(rt, 0, input, n);
        float* dg = stage(rt, 1, output_gradient, n);
        k::relu2_backward(rt, din, dg, n);
        rt->d2h(gx, dg, n * 4);
        rt->sync();
    });
}

int32_t ullis_cuda_layer_norm_backward(ullis_cuda_runtime* rt, const float* input, const float* output_gradient,
                                       const uint16_t* weight, size_t rows, size_t channels, float* gx, float* gw,
                                       float* gb) {
    return guard(rt, [&] {
        if (channels == 0) fail(ULLIS_CUDA_ERR_SHAPE, "LayerNorm backward shape mismatch");
        const size_t n = mul_or_fail(rows, channels, "LayerNorm backward");
        need_ptr(weight, "weight"); need_ptr(gw, "gw"); need_ptr(gb, "gb");
        float* dsmall = rt->pool[5].as<float>(2 * channels);
        if (n == 0) {
            rt->zero(dsmall, 2 * channels * 4);
        } else {
            need_ptr(input, "input"); need_ptr(output_gradient, "output_gradient"); need_ptr(gx, "gx");
            float* dx = stage(rt, 0, input, n);
            float* dgy = stage(rt, 1, output_gradient, n);
            uint16_t* dw = stage(rt, 2, weight, channels);
            float* dgx = rt->pool[3].as<float>(n);
            float* dxh = rt->pool[4].as<float>(n);
            k::layer_norm_backward(rt, dx, dgy, dw, dgx, dxh, dsmall, dsmall + channels, rows, channels, rt->pool[6]);
            rt->d2h(gx, dgx, n * 4);
        }
        rt->d2h(gw, dsmall, channels * 4);
        rt->d2h(gb, dsmall + channels, channels * 4);
        rt->sync();
    });
}

int32_t ullis_cuda_layer_norm(ullis_cuda_runtime* rt, const float* x, const uint16_t* weight,
                              const uint16_t* bias, float* y, size_t rows, size_t channels) {
    return guard(rt, [&] {
        if (channels == 0) fail(ULLIS_CUDA_ERR_SHAPE, "LayerNorm input shape mismatch");
        const size_t n = mul_or_fail(rows, channels, "LayerNorm");
        if (n == 0) return;
        need_ptr(x, "x"); need_ptr(weight, "weight"); need_ptr(bias, "bias"); need_ptr(y, "y");
        float* dx = stage(rt, 0, x, n);
        uint16_t* dw = stage(rt, 1, weight, channels);
        uint16_t* db = stage(rt, 2, bias, channels);
        float* dy = rt->pool[3].as<float>(n);
        k::layer_norm(rt, dx, dw, db, dy, rows, channels, rt->mode == ULLIS_CUDA_MODE_EXACT);
        rt->d2h(y, dy, n * 4);
        rt->sync();
    });
}

int32_t ullis_cuda_time_shift_delta(ullis_cuda_runtime* rt, const float* x, float* xx, size_t rows, size_t time,
                                    size_t channels) {
    return guard(rt, [&] {
        if (time == 0 || channels == 0 || rows % time != 0) fail(ULLIS_CUDA_ERR_SHAPE, "time-shift input shape mismatch");
        const size_t n = mul_or_fail(rows, channels, "time-shift");
        if (n == 0) return;
        need_ptr(x, "x"); need_ptr(xx, "xx");
        float* dx = stage(rt, 0, x, n);
        float* dy = rt->pool[1].as<float>(n);
        k::time_shift_delta(rt, dx, dy, rows, time, channels);
        rt->d2h(xx, dy, n * 4);
        rt->sync();
    });
}

int32_t ullis_cuda_binary_linear(ullis_cuda_runtime* rt, const float* x, const uint32_t* bits,
                                 const uint16_t* scale, const uint16_t* bias, float* y, size_t rows,
                                 size_t in_features, size_t out_features) {
    return guard(rt, [&] {
        if (in_features == 0 || out_features == 0) fail(ULLIS_CUDA_ERR_SHAPE, "packed linear input shape mismatch");
        const size_t nx = mul_or_fail(rows, in_features, "packed linear");
        const size_t ny = mul_or_fail(rows, out_features, "packed linear");
        const size_t words = (mul_or_fail(in_features, out_features, "packed linear") + 31) / 32;
        if (rows == 0) return;
        need_ptr(x, "x"); need_ptr(bits, "bits"); need_ptr(scale, "scale"); need_ptr(y, "y");
        float* dx = stage(rt, 0, x, nx);
        uint32_t* dbits = stage(rt, 1, bits, words);
        uint16_t* ds = stage(rt, 2, scale, out_features);
        uint16_t* db = bias ? stage(rt, 3, bias, out_features) : nullptr;
        float* dy = rt->pool[4].as<float>(ny);
        rt->clear_status();
        packed_linear_dev(rt, dx, dbits, ds, db, dy, rows, in_features, out_features);
        rt->d2h(y, dy, ny * 4);
        rt->check_status();
    });
}

int32_t ullis_cuda_fp16_linear(ullis_cuda_runtime* rt, const float* x, const uint16_t* weight, float* y,
                               size_t rows, size_t in_features, size_t out_features) {
    return guard(rt, [&] {
        if (in_features == 0 || out_features == 0) fail(ULLIS_CUDA_ERR_SHAPE, "FP16 linear shape mismatch");
        const size_t nx = mul_or_fail(rows, in_features, "FP16 linear");
        const size_t ny = mul_or_fail(rows, out_features, "FP16 linear");
        const size_t nw = mul_or_fail(in_features, out_features, "FP16 linear");
        if (rows == 0) return;
        need_ptr(x, "x"); need_ptr(weight, "weight"); need_ptr(y, "y");
        float* dx = stage(rt, 0, x, nx);
        uint16_t* dw = stage(rt, 1, weight, nw);
        float* dy = rt->pool[2].as<float>(ny);
        rt->clear_status();
        dense_linear_dev(rt, dx, dw, dy, rows, in_features, out_features);
        rt->d2h(y, dy, ny * 4);
        rt->check_status();
    });
}

int32_t ullis_cuda_sign_pack_bits(ullis_cuda_runtime* rt, const float* x, uint32_t* bits, size_t n) {
    return guard(rt, [&] {
        if (n == 0) return;
        need_ptr(x, "x"); need_ptr(bits, "bits");
        float* dx = stage(rt, 0, x, n);
        uint32_t* dw = rt->pool[1].as<uint32_t>((n + 31) / 32);
        k::sign_pack_flat(rt, dx, dw, n);
        rt->d2h(bits, dw, ((n + 31) / 32) * 4);
        rt->sync();
    });
}

int32_t ullis_cuda_cmix_relu2(ullis_cuda_runtime* rt, const float* x, float* y, size_t n) {
    return guard(rt, [&] {
        if (n == 0) return;
        need_ptr(x, "x"); need_ptr(y, "y");
        float* dx = stage(rt, 0, x, n);
        float* dy = rt->pool[1].as<float>(n);
        k::relu2(rt, dx, dy, n);
        rt->d2h(y, dy, n * 4);
        rt->sync();
    });
}

int32_t ullis_cuda_residual_add(ullis_cuda_runtime* rt, const float* residual, const float* update, float* out,
                                size_t n) {
    return guard(rt, [&] {
        if (n == 0) return;
        need_ptr(residual, "residual"); need_ptr(update, "update"); need_ptr(out, "out");
        float* da = stage(rt, 0, residual, n);
        float* db = stage(rt, 1, update, n);
        float* dy = rt->pool[2].as<float>(n);
        k::residual_add(rt, da, db, dy, n);
        rt->d2h(out, dy, n * 4);
        rt->sync();
    });
}

int32_t ullis_cuda_rosa_qkv_1bit_fwd(ullis_cuda_runtime* rt, const uint32_t* q_bits, const uint32_t* k_bits,
                                     const uint32_t* v_bits, const uint16_t* e, uint8_t* idx, float* out,
                                     size_t batch, size_t time, size_t channels) {
    return guard(rt, [&] {
        // reference: MetalDispatchShape::new rejects zero dims (src/metal.rs:36-53)
        if (batch == 0 || time == 0 || channels == 0) fail(ULLIS_CUDA_ERR_SHAPE, "ROSA dispatch dimensions must be non-zero");
        const size_t n = mul_or_fail(mul_or_fail(batch, time, "ROSA"), channels, "ROSA");
        need_ptr(q_bits, "q_bits"); need_ptr(k_bits, "k_bits"); need_ptr(v_bits, "v_bits"); need_ptr(e, "e");
        const size_t words = (n + 31) / 32, wps = (time + 31) / 32, sw = batch * channels * wps;
        uint32_t* dq = stage(rt, 0, q_bits, words);
        uint32_t* dk = stage(rt, 1, k_bits, words);
        uint32_t* dv = stage(rt, 2, v_bits, words);
        uint16_t* de = stage(rt, 3, e, channels);
        uint32_t* qs = rt->pool[4].as<uint32_t>(sw);
        uint32_t* ks = rt->pool[5].as<uint32_t>(sw);
        uint32_t* vs = rt->pool[6].as<uint32_t>(sw);
        uint32_t* is = rt->pool[7].as<uint32_t>(sw);
        k::planes_to_streams(rt, dq, qs, batch, time, channels);
        k::planes_to_streams(rt, dk, ks, batch, time, channels);
        k::planes_to_streams(rt, dv, vs, batch, time, channels);
        rt->clear_status();
        k::rosa_sam(rt, qs, ks, vs, is, batch * channels, time);
        uint8_t* didx = idx ? rt->pool[8].as<uint8_t>(n) : nullptr;
        float* dout = out ? rt->pool[9].as<float>(n) : nullptr;
        if (idx || out) k::rosa_emit(rt, is, de, didx, dout, batch, time, channels);
        if (idx) rt->d2h(idx, didx, n);
        if (out) rt->d2h(out, dout, n * 4);
        rt->check_status();
    });
}

int32_t ullis_cuda_rosa_block_forward(ullis_cuda_runtime* rt, const float* x, const uint16_t* mix_q,
                                      const uint16_t* mix_k, const uint16_t* mix_v, const uint32_t* q_bits,
                                      const uint16_t* q_scale, const uint16_t* q_bias, const uint32_t* k_bits,
                                      const uint16_t* k_scale, const uint16_t* k_bias, const uint32_t* v_bits,
                                      const uint16_t* v_scale, const uint16_t* v_bias, const uint16_t* e,
                                      const uint32_t* o_bits, const uint16_t* o_scale, const uint16_t* o_bias,
                                      size_t batch, size_t time, size_t channels, uint32_t* q_plane,
                                      uint32_t* k_plane, uint32_t* v_plane, uint8_t* idx, float* y, float* out) {
    return guard(rt, [&] {
        if (batch == 0 || time == 0 || channels == 0) fail(ULLIS_CUDA_ERR_SHAPE, "ROSA dispatch dimensions must be non-zero");
        const size_t rows = mul_or_fail(batch, time, "ROSA block");
        const size_t n = mul_or_fail(rows, channels, "ROSA block");
        const size_t d = channels, words = (d * d + 31) / 32, wps = (time + 31) / 32, sw = batch * d * wps;
        const void* req[] = {x, mix_q, mix_k, mix_v, q_bits, q_scale, q_bias, k_bits, k_scale, k_bias,
                             v_bits, v_scale, v_bias, e, o_bits, o_scale, o_bias};
        for (const void* p : req) need_ptr(p, "ROSA block argument");
        LayerWeights L;
        float* dx = stage(rt, 0, x, n);
        L.x_q = stage(rt, 1, mix_q, d);
        L.x_k = stage(rt, 2, mix_k, d);
        L.x_v = stage(rt, 3, mix_v, d);
        L.e = stage(rt, 4, e, d);
        auto lin = [&](PackedWeights& w, int slot, const uint32_t* b, const uint16_t* s, const uint16_t* bi) {
            w.out = d; w.in = d;
            w.bits = stage(rt, slot, b, words);
            w.scale = stage(rt, slot + 1, s, d);
            w.bias = stage(rt, slot + 2, bi, d);
        };
        lin(L.q, 5, q_bits, q_scale, q_bias);
        lin(L.k, 8, k_bits, k_scale, k_bias);
        lin(L.v, 11, v_bits, v_scale, v_bias);
        lin(L.o, 14, o_bits, o_scale, o_bias);
        // one allocation for the activations of this call
        float* work = rt->pool[17].as<float>(n * 5);
        float *bq = work, *bk = work + n, *bv = work + 2 * n, *w = work + 3 * n, *dout = work + 4 * n;
        uint32_t* sws = rt->pool[18].as<uint32_t>(sw * 4);
        uint32_t *qs = sws, *ks = sws + sw, *vs = sws + 2 * sw, *is = sws + 3 * sw;
        rt->clear_status();
        const bool exact = rt->mode == ULLIS_CUDA_MODE_EXACT;
        if (exact || !tc::rosa_qkv_bits(rt, dx, L, qs, ks, vs, batch, time, d)) {
            k::shift_mix(rt, dx, L.x_q, L.x_k, L.x_v, bq, bk, bv, rows, time, d);
            k::binary_linear_exact(rt, bq, L.q.bits, L.q.scale, L.q.bias, w, rows, d, d, false);
            k::sign_pack_streams(rt, w, qs, batch, time, d);
            k::binary_linear_exact(rt, bk, L.k.bits, L.k.scale, L.k.bias, w, rows, d, d, false);
            k::sign_pack_streams(rt, w, ks, batch, time, d);
            k::binary_linear_exact(rt, bv, L.v.bits, L.v.scale, L.v.bias, w, rows, d, d, false);
            k::sign_pack_streams(rt, w, vs, batch, time, d);
        }
        k::rosa_sam(rt, qs, ks, vs, is, batch * d, time);
        uint8_t* didx = rt->pool[19].as<uint8_t>(n);
        k::rosa_emit(rt, is, L.e, didx, w, batch, time, d);  // w <- y
        packed_linear_dev(rt, w, L.o.bits, L.o.scale, L.o.bias, dout, rows, d, d);
        const size_t plane_words = (n + 31) / 32;
        uint32_t* dplane = rt->pool[20].as<uint32_t>(plane_words);
        uint32_t* planes_out[3] = {q_plane, k_plane, v_plane};
        uint32_t* planes_in[3] = {qs, ks, vs};
        for (int i = 0; i < 3; ++i) {
            if (!planes_out[i]) continue;
            k::streams_to_planes(rt, planes_in[i], dplane, batch, time, d);
            rt->d2h(planes_out[i], dplane, plane_words * 4);
            rt->sync();  // dplane is reused
        }
        if (idx) rt->d2h(idx, didx, n);
        if (y) rt->d2h(y, w, n * 4);
        if (out) rt->d2h(out, dout, n * 4);
        rt->check_status();
    });
}

int32_t ullis_cuda_cmix_block_forward(ullis_cuda_runtime* rt, const float* x, const uint16_t* mix,
                                      const uint32_t* key_bits, const uint16_t* key_scale,
                                      const uint16_t* value, size_t batch, size_t time, size_t d_model,
                                      size_t dim_ffn, float* out) {
    return guard(rt, [&] {
        if (batch == 0 || time == 0 || d_model == 0 || dim_ffn == 0) fail(ULLIS_CUDA_ERR_SHAPE, "CMix shape mismatch");
        const size_t rows = mul_or_fail(batch, time, "CMix");
        const size_t n = mul_or_fail(rows, d_model, "CMix");
        const size_t nf = mul_or_fail(rows, dim_ffn, "CMix");
        const size_t nw = mul_or_fail(d_model, dim_ffn, "CMix");
        need_ptr(x, "x"); need_ptr(mix, "mix"); need_ptr(key_bits, "key_bits"); need_ptr(key_scale, "key_scale");
        need_ptr(value, "value"); need_ptr(out, "out");
        float* dx = stage(rt, 0, x, n);
        uint16_t* dm = stage(rt, 1, mix, d_model);
        uint32_t* dkb = stage(rt, 2, key_bits, (nw + 31) / 32);
        uint16_t* dks = stage(rt, 3, key_scale, dim_ffn);
        uint16_t* dv = stage(rt, 4, value, nw);
        float* sh = rt->pool[5].as<float>(n);
        float* key = rt->pool[6].as<float>(nf);
        float* dout = rt->pool[7].as<float>(n);
        rt->clear_status();
        k::shift_mix(rt, dx, dm, nullptr, nullptr, sh, nullptr, nullptr, rows, time, d_model);
        packed_linear_dev(rt, sh, dkb, dks, nullptr, key, rows, d_model, dim_ffn);
        k::relu2(rt, key, key, nf);
        dense_linear_dev(rt, key, dv, dout, rows, dim_ffn, d_model);
        rt->d2h(out, dout, n * 4);
        rt->check_status();
    });
}

int32_t ullis_cuda_streamed_ce(ullis_cuda_runtime* rt, const float* hidden, const uint32_t* bits,
                               const uint16_t* scale, const uint16_t* bias, const uint32_t* labels,
                               uint32_t ignore_id, size_t rows, size_t time, size_t channels, size_t vocab,
                               float* row_loss, float* mean_loss, uint64_t* n_valid) {
    return guard(rt, [&] {
        // reference: src/metal.rs:2932-2941
        if (time == 0 || rows % time != 0 || channels == 0 || vocab == 0) fail(ULLIS_CUDA_ERR_SHAPE, "streamed CE shape mismatch");
        const size_t nh = mul_or_fail(rows, channels, "streamed CE");
        const size_t words = (mul_or_fail(vocab, channels, "streamed CE") + 31) / 32;
        if (rows == 0) {
            if (mean_loss) *mean_loss = 0.0f;
            if (n_valid) *n_valid = 0;
            return;
        }
        need_ptr(hidden, "hidden"); need_ptr(bits, "bits"); need_ptr(scale, "scale"); need_ptr(labels, "labels");
        float* dh = stage(rt, 0, hidden, nh);
        PackedWeights head;
        head.out = vocab; head.in = channels;
        head.bits = stage(rt, 1, bits, words);
        head.scale = stage(rt, 2, scale, vocab);
        head.bias = bias ? stage(rt, 3, bias, vocab) : nullptr;
        uint32_t* dl = stage(rt, 4, labels, rows);
        float* rl = rt->pool[5].as<float>(rows);
        uint8_t* res = static_cast<uint8_t*>(rt->pool[6].ensure(16));
        rt->clear_status();
        if (rt->mode == ULLIS_CUDA_MODE_EXACT ||
            !tc::head_ce(rt, dh, head, dl, ignore_id, rows, time, channels, vocab, rl)) {
            const size_t chunk = std::max<size_t>(1, std::min<size_t>(rows, ((size_t)256 << 20) / (vocab * 4)));
            float* lg = rt->pool[7].as<float>(chunk * vocab);
            for (size_t r0 = 0; r0 < rows; r0 += chunk) {
                const size_t nr = std::min(chunk, rows - r0);
                k::binary_linear_exact(rt, dh + r0 * channels, head.bits, head.scale, head.bias, lg, nr, channels,
                                       vocab, false);
                k::ce_rows_from_logits(rt, lg, dl, ignore_id, r0, nr, rows, time, vocab, rl);
            }
        }
        k::ce_reduce(rt, rl, dl, ignore_id, rows, time, reinterpret_cast<double*>(res),
                     reinterpret_cast<unsigned long long*>(res + 8));
        struct { double sum; unsigned long long n; } host;
        rt->d2h(&host, res, 16);
        if (row_loss) rt->d2h(row_loss, rl, rows * 4);
        rt->check_status();
        if (mean_loss) *mean_loss = host.n == 0 ? 0.0f : (float)(host.sum / (double)host.n);
        if (n_valid) *n_valid = host.n;
    });
}

}  // extern "C"
