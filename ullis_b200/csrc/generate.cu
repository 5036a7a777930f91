// Incremental generation: one token per sequence and call, with the automata
// of every (sequence, layer, channel) kept on the device between calls
// (reference UllisHeron::generate_state / generate_step, src/model.rs:2691-2753;
// per-block forward_one src/model.rs:2243-2262, ROSA 1320-1352, CMix 1003-1016).
//
// A step is a handful of [batch, d_model] row operations, so it runs on the
// CUDA-core kernels in the reference's summation order: the logits of step t
// are bit-identical to row t of the one-shot forward in EXACT mode, which is
// what the reference's own test asserts (src/model.rs:4991-5004).  The automata
// follow the reference's eager schedule (push stamps the whole suffix-link chain
// of the new state), because the O(T log T) form needs the whole sequence in
// advance; the chain is kept as an array and stamped by a warp, 32 states per
// round, instead of one dependent load per state.  A stream whose key bits have
// all been equal so far is answered in closed form and its automaton written
// only when that ends.
//
// Nothing in a step depends on the host except the tokens, so after the first
// use the ~150 small launches of a step are replayed as one CUDA graph (two
// graphs: before and after the first token, which has no time-shift history).
#include "generate.hpp"

#include <cuda_fp16.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "kernels.hpp"
#include "sam_core.cuh"

namespace ullis {
namespace {

inline unsigned blocks_for(size_t n, unsigned per) { return (unsigned)((n + per - 1) / per); }

__device__ __forceinline__ float h2f(uint16_t b) { return __half2float(__ushort_as_half(b)); }

// empty automaton per stream (src/rosa.rs:66-74)
template <typename Ix>
__global__ void gen_init_kernel(uint8_t* __restrict__ blocks, size_t stride, sam::WalkerState* __restrict__ ws,
                                size_t streams, uint32_t T) {
    const size_t s = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= streams) return;
    // no pushes yet; the automaton is written lazily (sam::gen_push), not even the root is needed
    sam::WalkerState st;
    st.u = 1; st.g = 0; st.w = 0; st.gmax = 0; st.gfail = 0; st.h = 0; st.steps = 0; st.pad = 0;
    ws[s] = st;
    (void)blocks; (void)stride; (void)T;
}

// time_shift_one + mixes (src/model.rs:214-228, 1331-1340, 1008-1012): xx = prev - x, or -x before the
// first token; out_m = x + xx*mix_m, unfused; then x becomes the layer's new time-shift history
__global__ void gen_shift_mix_kernel(const float* __restrict__ x, float* __restrict__ prev, int has_prev,
                                     const uint16_t* __restrict__ m0, const uint16_t* __restrict__ m1,
                                     const uint16_t* __restrict__ m2, float* __restrict__ o0, float* __restrict__ o1,
                                     float* __restrict__ o2, size_t n, size_t C) {
    const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= n) return;
    const size_t c = e % C;
    const float xt = x[e];
    const float xx = has_prev ? __fsub_rn(prev[e], xt) : -xt;
    o0[e] = __fadd_rn(xt, __fmul_rn(xx, h2f(m0[c])));
    if (o1) o1[e] = __fadd_rn(xt, __fmul_rn(xx, h2f(m1[c])));
    if (o2) o2[e] = __fadd_rn(xt, __fmul_rn(xx, h2f(m2[c])));
    prev[e] = xt;
}

// LayerNorm of one row and the time-shift mixes of that row in one launch (the two kernels above it in a step,
// for the few rows of a step): the reference's LayerNorm arithmetic (src/model.rs:259-276: the sum, then the sum
// of the squared deviations, each added one value after the other) is a chain one thread has to run, 2·C
// dependent additions; it runs from shared memory, and the rest of the CTA does the affine part, the mixes and
// the new time-shift history.  `ln_out` (nullable) receives the normalised row.
__global__ void __launch_bounds__(128)
gen_ln_shift_mix_kernel(const float* __restrict__ x, const uint16_t* __restrict__ lw, const uint16_t* __restrict__ lb,
                        float* __restrict__ ln_out, float* __restrict__ prev, int has_prev,
                        const uint16_t* __restrict__ m0, const uint16_t* __restrict__ m1,
                        const uint16_t* __restrict__ m2, float* __restrict__ o0, float* __restrict__ o1,
                        float* __restrict__ o2, size_t C) {
    extern __shared__ __align__(16) float gen_row[];
    __shared__ float s_mean, s_inv;
    const size_t r = blockIdx.x;
    for (size_t c = threadIdx.x; c < C; c += blockDim.x) gen_row[c] = x[r * C + c];
    __syncthreads();
    if (threadIdx.x == 0) {
        // the additions are one chain; the loads are not: sixteen values are fetched (four 16-byte loads) before
        // they are added, so that the chain waits for arithmetic only
        float acc = 0.0f;
        size_t c = 0;
        for (; c + 16 <= C; c += 16) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) v[u] = *reinterpret_cast<const float4*>(gen_row + c + 4 * u);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                acc = __fadd_rn(acc, v[u].x); acc = __fadd_rn(acc, v[u].y);
                acc = __fadd_rn(acc, v[u].z); acc = __fadd_rn(acc, v[u].w);
            }
        }
        for (; c < C; ++c) acc = __fadd_rn(acc, gen_row[c]);
        const float mean = __fdiv_rn(acc, (float)C);
        acc = 0.0f;
        for (c = 0; c + 16 <= C; c += 16) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) v[u] = *reinterpret_cast<const float4*>(gen_row + c + 4 * u);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const float d0 = __fsub_rn(v[u].x, mean), d1 = __fsub_rn(v[u].y, mean);
                const float d2 = __fsub_rn(v[u].z, mean), d3 = __fsub_rn(v[u].w, mean);
                acc = __fadd_rn(acc, __fmul_rn(d0, d0)); acc = __fadd_rn(acc, __fmul_rn(d1, d1));
                acc = __fadd_rn(acc, __fmul_rn(d2, d2)); acc = __fadd_rn(acc, __fmul_rn(d3, d3));
            }
        }
        for (; c < C; ++c) {
            const float dlt = __fsub_rn(gen_row[c], mean);
            acc = __fadd_rn(acc, __fmul_rn(dlt, dlt));
        }
        s_mean = mean;
        s_inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(acc, (float)C), 1e-5f)));
    }
    __syncthreads();
    const float mean = s_mean, inv = s_inv;
    for (size_t c = threadIdx.x; c < C; c += blockDim.x) {
        const size_t e = r * C + c;
        const float n = __fmul_rn(__fsub_rn(gen_row[c], mean), inv);
        const float xt = __fadd_rn(__fmul_rn(n, h2f(lw[c])), h2f(lb[c]));
        if (ln_out) ln_out[e] = xt;
        // time_shift_one + mixes (src/model.rs:214-228, 1331-1340, 1008-1012), as gen_shift_mix_kernel
        const float xx = has_prev ? __fsub_rn(prev[e], xt) : -xt;
        o0[e] = __fadd_rn(xt, __fmul_rn(xx, h2f(m0[c])));
        if (o1) o1[e] = __fadd_rn(xt, __fmul_rn(xx, h2f(m1[c])));
        if (o2) o2[e] = __fadd_rn(xt, __fmul_rn(xx, h2f(m2[c])));
        prev[e] = xt;
    }
}

// one RosaSam::push per (sequence, channel) of one layer and y = (2*idx - 1)*e (src/model.rs:1344-1351).
// One warp per stream: lane 0 runs the query and the extend, all lanes the stamping of the suffix-link chain
// (sam::gen_push), which is what a late position costs.
template <typename Ix>
__global__ void __launch_bounds__(128)
gen_push_kernel(uint8_t* __restrict__ blocks, size_t stride, sam::WalkerState* __restrict__ ws,
                uint32_t* __restrict__ vhist, size_t wps, const float* __restrict__ q, const float* __restrict__ k,
                const float* __restrict__ v, const uint16_t* __restrict__ e, float* __restrict__ y, size_t streams,
                size_t C, uint32_t T, uint32_t* __restrict__ status) {
    const size_t s = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const uint32_t lane = threadIdx.x & 31u;
    if (s >= streams) return;   // the whole warp
    sam::GenLayout<Ix> L(T);
    uint8_t* blk = blocks + s * stride;
    sam::WalkerState st = ws[s];
    const uint32_t i = st.steps;
    if (i >= T) {  // the host checks the context length first; never write past the state block
        if (lane == 0 && atomicCAS(status, ULLIS_DEV_OK, ULLIS_DEV_SAM_CAPACITY) == ULLIS_DEV_OK) status[1] = (uint32_t)s;
        return;
    }
    // src/rosa.rs:372-374: bit = activation > 0
    const uint32_t qb = q[s] > 0.0f, kb = k[s] > 0.0f, vb = v[s] > 0.0f;
    uint32_t* vh = vhist + s * wps;
    if (lane == 0) {   // only lane 0 reads the v history
        const uint32_t word = (i & 31u) ? vh[i >> 5] : 0u;   // a new word starts empty
        vh[i >> 5] = word | (vb << (i & 31u));
    }
    // constant key so far: O(1); otherwise RosaSam::push with the chain stamped by the warp
    const uint32_t idx = sam::gen_push<Ix>(reinterpret_cast<sam::Node<Ix>*>(blk + L.nodes), reinterpret_cast<Ix*>(blk + L.last),
                                           reinterpret_cast<Ix*>(blk + L.path), vh, &st, qb, kb);
    if (lane == 0) {
        ws[s] = st;
        const float ev = h2f(e[s % C]);
        y[s] = idx ? ev : -ev;
    }
}

}  // namespace
}  // namespace ullis

using namespace ullis;

ullis_cuda_generate_state::ullis_cuda_generate_state(ullis_cuda_model* m, size_t batch_) : model(m), batch(batch_) {
    if (batch == 0) fail(ULLIS_CUDA_ERR_SHAPE, "generate needs at least one sequence");
    const uint32_t T = (uint32_t)m->context_len;
    narrow = sam::node_capacity(T) <= 0xFFFFu;
    stride = narrow ? sam::GenLayout<uint16_t>(T).total : sam::GenLayout<uint32_t>(T).total;
    wps = (m->context_len + 31) / 32;
    const size_t per_layer = batch * m->d;
    if (per_layer / m->d != batch || m->layers > SIZE_MAX / per_layer) fail(ULLIS_CUDA_ERR_SHAPE, "generate state shape overflow");
    streams = m->layers * per_layer;
    if (streams > SIZE_MAX / stride) fail(ULLIS_CUDA_ERR_SHAPE, "generate state shape overflow");
    m->rt->bind();
    k::rowvec_prepare(m->rt);   // before any step is recorded into a graph
    blocks.ensure(streams * stride);
    walkers.ensure(streams * sizeof(sam::WalkerState));
    vhist.ensure(streams * wps * 4);
    prev.ensure(m->layers * 2 * per_layer * 4);
    ids.ensure(batch * 4);
    for (ullis::DeviceBuffer* buf : {&x, &a, &bq, &bk, &bv}) buf->ensure(per_layer * 4);
    wide.ensure(batch * std::max(m->ffn, 3 * m->d) * 4);
    logits.ensure(batch * m->vocab * 4);
    ULLIS_CUDA_CHECK(cudaMallocHost(&h_tokens, batch * 4));
    ULLIS_CUDA_CHECK(cudaMallocHost(&h_logits, batch * m->vocab * 4));
    use_graph = !getenv("ULLIS_CUDA_NO_GRAPH");
    if (const char* env = getenv("ULLIS_CUDA_INJECT_GENERATE_FAILURE")) inject_failure_at = (size_t)std::max(0, atoi(env));
    reset();
}

ullis_cuda_generate_state::~ullis_cuda_generate_state() {
    for (cudaGraphExec_t g : graph)
        if (g) cudaGraphExecDestroy(g);
    if (h_tokens) cudaFreeHost(h_tokens);
    if (h_logits) cudaFreeHost(h_logits);
}

void ullis_cuda_generate_state::reset() {
    ullis_cuda_runtime* rt = model->rt;
    rt->bind();
    const uint32_t T = (uint32_t)model->context_len;
    auto* ws = static_cast<sam::WalkerState*>(walkers.get());
    auto* blk = static_cast<uint8_t*>(blocks.get());
    if (narrow) gen_init_kernel<uint16_t><<<blocks_for(streams, 256), 256, 0, rt->stream>>>(blk, stride, ws, streams, T);
    else gen_init_kernel<uint32_t><<<blocks_for(streams, 256), 256, 0, rt->stream>>>(blk, stride, ws, streams, T);
    rt->launched("gen_init");
    rt->sync();
    time = 0;
    poisoned = false;
}

void ullis_cuda_generate_state::step(const uint32_t* tokens, float* logits_out) {
    ullis_cuda_model* m = model;
    ullis_cuda_runtime* rt = m->rt;
    // src/model.rs:2718-2723
    for (size_t b = 0; b < batch; ++b)
        if (tokens[b] >= m->vocab) fail(ULLIS_CUDA_ERR_TOKEN, "token id exceeds vocabulary");
    if (time >= m->context_len)
        fail(ULLIS_CUDA_ERR_SHAPE, "generate exceeded context_len (" + std::to_string(m->context_len) + ")");
    if (poisoned)
        fail(ULLIS_CUDA_ERR_ARG, "generate state is unusable after a failed step: reset it (ullis_cuda_generate_state_reset)");
    rt->bind();
    if (rt->kernel_timing) rt->mark("(between steps)");
    std::memcpy(h_tokens, tokens, batch * 4);
    const int has_prev = time != 0;
    // From here on the device-side automata, v history and time-shift inputs may have moved on by one position
    // while `time` has not: a failure below leaves the state out of step with itself, and a retry would push the
    // same position twice.  The state stays refused until reset() (which rebuilds it from scratch).
    struct Poison {
        bool* flag;
        bool armed = true;
        ~Poison() { if (armed) *flag = true; }
    } poison{&poisoned};

    if (use_graph && !rt->kernel_timing) {
        // Replay the step as one graph launch; per-kernel timing needs the plain launches.
        if (!graph[has_prev]) {
            cudaGraph_t captured = nullptr;
            const uint64_t before = rt->launches;
            ULLIS_CUDA_CHECK(cudaStreamBeginCapture(rt->stream, cudaStreamCaptureModeThreadLocal));
            try {
                enqueue(has_prev);
            } catch (...) {
                cudaStreamEndCapture(rt->stream, &captured);
                if (captured) cudaGraphDestroy(captured);
                rt->launches = before;
                throw;
            }
            ULLIS_CUDA_CHECK(cudaStreamEndCapture(rt->stream, &captured));
            graph_launches = rt->launches - before;
            rt->launches = before;   // counted per replay below
            const cudaError_t e = cudaGraphInstantiate(&graph[has_prev], captured, 0);
            cudaGraphDestroy(captured);
            ULLIS_CUDA_CHECK(e);
        }
        ULLIS_CUDA_CHECK(cudaGraphLaunch(graph[has_prev], rt->stream));
        rt->launches += graph_launches;
    } else {
        enqueue(has_prev);
    }
    rt->sync();
    rt->throw_on_status();
    if (inject_failure_at && time + 1 == inject_failure_at) {   // host-injected: what a CUDA error after the launches does
        inject_failure_at = 0;
        fail(ULLIS_CUDA_ERR_CUDA, "injected failure after the step's kernels ran");
    }
    std::memcpy(logits_out, h_logits, batch * m->vocab * 4);
    time += 1;
    poison.armed = false;
}

void ullis_cuda_generate_state::enqueue(int has_prev) {
    ullis_cuda_model* m = model;
    ullis_cuda_runtime* rt = m->rt;
    const size_t d = m->d, ffn = m->ffn, rows = batch, n = rows * d;
    const uint32_t T = (uint32_t)m->context_len;
    uint32_t* IDS = static_cast<uint32_t*>(ids.get());
    float* X = static_cast<float*>(x.get());
    float* A = static_cast<float*>(a.get());
    float* Bq = static_cast<float*>(bq.get());
    float* Bk = static_cast<float*>(bk.get());
    float* Bv = static_cast<float*>(bv.get());
    float* W = static_cast<float*>(wide.get());
    float* LG = static_cast<float*>(logits.get());
    rt->clear_status();
    rt->h2d(IDS, h_tokens, rows * 4);
    k::embed(rt, IDS, m->embedding, X, rows, d, m->vocab);
    const bool fused_ln = d * 4 <= 48 * 1024 && !getenv("ULLIS_CUDA_GEN_UNFUSED");   // a row in shared memory
    for (size_t l = 0; l < m->layers; ++l) {
        const LayerWeights& L = m->blocks[l];
        float* rosa_prev = static_cast<float*>(prev.get()) + (l * 2) * n;
        float* cmix_prev = rosa_prev + n;
        const size_t s0 = l * n;  // first stream of this layer
        if (l == 0) {  // ln0 REPLACES x on layer 0 (src/model.rs:2244-2248)
            k::layer_norm(rt, X, L.ln0.weight, L.ln0.bias, A, rows, d, true);
            ULLIS_CUDA_CHECK(cudaMemcpyAsync(X, A, n * 4, cudaMemcpyDeviceToDevice, rt->stream));
        }
        // ROSA (src/model.rs:1320-1352)
        if (fused_ln) {
            gen_ln_shift_mix_kernel<<<(unsigned)rows, 128, d * 4, rt->stream>>>(X, L.ln3.weight, L.ln3.bias, nullptr, rosa_prev,
                                                                                has_prev, L.x_q, L.x_k, L.x_v, Bq, Bk, Bv, d);
            rt->launched("gen_ln_shift_mix");
        } else {
            k::layer_norm(rt, X, L.ln3.weight, L.ln3.bias, A, rows, d, true);
            gen_shift_mix_kernel<<<blocks_for(n, 256), 256, 0, rt->stream>>>(A, rosa_prev, has_prev, L.x_q, L.x_k, L.x_v, Bq,
                                                                           Bk, Bv, n, d);
            rt->launched("gen_shift_mix");
        }
        {   // Q, K and V in one launch when the shape allows
            const float* xs[3] = {Bq, Bk, Bv};
            const uint32_t* bs[3] = {L.q.bits, L.k.bits, L.v.bits};
            const uint16_t* ss[3] = {L.q.scale, L.k.scale, L.v.scale};
            const uint16_t* bi[3] = {L.q.bias, L.k.bias, L.v.bias};
            float* ys[3] = {W, W + n, W + 2 * n};
            if (!fused_ln || !k::binary_rowvec_multi(rt, 3, xs, bs, ss, bi, ys, rows, d, d, false)) {
                k::binary_linear_exact(rt, Bq, L.q.bits, L.q.scale, L.q.bias, W, rows, d, d, false);
                k::binary_linear_exact(rt, Bk, L.k.bits, L.k.scale, L.k.bias, W + n, rows, d, d, false);
                k::binary_linear_exact(rt, Bv, L.v.bits, L.v.scale, L.v.bias, W + 2 * n, rows, d, d, false);
            }
        }
        {
            auto* ws = static_cast<sam::WalkerState*>(walkers.get()) + s0;
            uint8_t* blk = static_cast<uint8_t*>(blocks.get()) + s0 * stride;
            uint32_t* vh = static_cast<uint32_t*>(vhist.get()) + s0 * wps;
            if (narrow)
                gen_push_kernel<uint16_t><<<blocks_for(n * 32, 128), 128, 0, rt->stream>>>(blk, stride, ws, vh, wps, W, W + n, W + 2 * n,
                                                                                     L.e, A, n, d, T, rt->dev_status);
            else
                gen_push_kernel<uint32_t><<<blocks_for(n * 32, 128), 128, 0, rt->stream>>>(blk, stride, ws, vh, wps, W, W + n, W + 2 * n,
                                                                                     L.e, A, n, d, T, rt->dev_status);
            rt->launched("gen_push");
        }
        k::binary_linear_exact(rt, A, L.o.bits, L.o.scale, L.o.bias, X, rows, d, d, true);  // h += rosa out
        // CMix (src/model.rs:1003-1016)
        if (fused_ln) {
            gen_ln_shift_mix_kernel<<<(unsigned)rows, 128, d * 4, rt->stream>>>(X, L.ln2.weight, L.ln2.bias, nullptr, cmix_prev,
                                                                                has_prev, L.ffn_x_k, nullptr, nullptr, Bq, nullptr,
                                                                                nullptr, d);
            rt->launched("gen_ln_shift_mix");
        } else {
            k::layer_norm(rt, X, L.ln2.weight, L.ln2.bias, A, rows, d, true);
            gen_shift_mix_kernel<<<blocks_for(n, 256), 256, 0, rt->stream>>>(A, cmix_prev, has_prev, L.ffn_x_k, nullptr, nullptr,
                                                                           Bq, nullptr, nullptr, n, d);
            rt->launched("gen_shift_mix");
        }
        {   // key and relu^2 in one launch when the shape allows
            const float* xs[1] = {Bq};
            const uint32_t* bs[1] = {L.key.bits};
            const uint16_t* ss[1] = {L.key.scale};
            const uint16_t* bi[1] = {nullptr};
            float* ys[1] = {W};
            if (!fused_ln || !k::binary_rowvec_multi(rt, 1, xs, bs, ss, bi, ys, rows, d, ffn, true)) {
                k::binary_linear_exact(rt, Bq, L.key.bits, L.key.scale, nullptr, W, rows, d, ffn, false);
                k::relu2(rt, W, W, rows * ffn);
            }
        }
        k::fp16_linear_exact(rt, W, L.value, X, rows, ffn, d, true);  // h += cmix out
    }
    // src/model.rs:2750-2752
    k::layer_norm(rt, X, m->ln_out.weight, m->ln_out.bias, A, rows, d, true);
    k::binary_linear_exact(rt, A, m->head.bits, m->head.scale, m->head.bias, LG, rows, d, m->vocab, false);
    rt->d2h(h_logits, LG, rows * m->vocab * 4);
    rt->d2h(rt->host_status, rt->dev_status, 16);
}

// ------------------------------------------------------------------ op level: RosaSam::push for many streams

ullis_cuda_rosa_pushers::ullis_cuda_rosa_pushers(ullis_cuda_runtime* rt_, size_t streams_, size_t capacity_)
    : rt(rt_), streams(streams_), capacity(capacity_) {
    if (streams == 0 || capacity == 0) fail(ULLIS_CUDA_ERR_SHAPE, "ROSA pushers need at least one stream and one position");
    if (capacity > 0x7FFFFFF0u) fail(ULLIS_CUDA_ERR_SHAPE, "ROSA pushers: capacity too large");
    const uint32_t T = (uint32_t)capacity;
    narrow = sam::node_capacity(T) <= 0xFFFFu;
    stride = narrow ? sam::GenLayout<uint16_t>(T).total : sam::GenLayout<uint32_t>(T).total;
    wps = (capacity + 31) / 32;
    if (streams > SIZE_MAX / stride) fail(ULLIS_CUDA_ERR_SHAPE, "ROSA pushers: shape overflow");
    rt->bind();
    blocks.ensure(streams * stride);
    walkers.ensure(streams * sizeof(sam::WalkerState));
    vhist.ensure(streams * wps * 4);
    reset();
}

void ullis_cuda_rosa_pushers::reset() {
    rt->bind();
    auto* ws = static_cast<sam::WalkerState*>(walkers.get());
    auto* blk = static_cast<uint8_t*>(blocks.get());
    gen_init_kernel<uint16_t><<<blocks_for(streams, 256), 256, 0, rt->stream>>>(blk, stride, ws, streams, (uint32_t)capacity);
    rt->launched("gen_init");
    rt->sync();
    time = 0;
}

void ullis_cuda_rosa_pushers::push(const uint8_t* q, const uint8_t* k, const uint8_t* v, size_t steps, uint8_t* idx) {
    // RosaSam has no capacity (src/rosa.rs:55-64 grows its vectors); here it is fixed when the state is made
    if (steps > capacity - time) fail(ULLIS_CUDA_ERR_SHAPE, "ROSA pushers: more pushes than the capacity given at creation");
    if (steps == 0) return;
    if (steps > SIZE_MAX / streams / 20) fail(ULLIS_CUDA_ERR_SHAPE, "ROSA pushers: shape overflow");
    rt->bind();
    const size_t n = steps * streams;
    // the generation kernel takes activations (bit = x > 0) and writes (2*idx - 1)*e: feed it +-1 and e = 1
    std::vector<float> h(3 * n);
    for (size_t i = 0; i < n; ++i) {
        h[i] = q[i] ? 1.0f : -1.0f;
        h[n + i] = k[i] ? 1.0f : -1.0f;
        h[2 * n + i] = v[i] ? 1.0f : -1.0f;
    }
    io.ensure(4 * n * 4 + 16);
    float* d = static_cast<float*>(io.get());
    uint16_t* one = reinterpret_cast<uint16_t*>(d + 4 * n);
    const uint16_t h_one = 0x3C00u;   // FP16 1.0
    rt->clear_status();
    rt->h2d(d, h.data(), 3 * n * 4);
    rt->h2d(one, &h_one, 2);
    auto* ws = static_cast<sam::WalkerState*>(walkers.get());
    auto* blk = static_cast<uint8_t*>(blocks.get());
    uint32_t* vh = static_cast<uint32_t*>(vhist.get());
    for (size_t t = 0; t < steps; ++t) {
        const float* row = d + t * streams;
        if (narrow)
            gen_push_kernel<uint16_t><<<blocks_for(streams * 32, 128), 128, 0, rt->stream>>>(
                blk, stride, ws, vh, wps, row, row + n, row + 2 * n, one, d + 3 * n + t * streams, streams, 1, (uint32_t)capacity,
                rt->dev_status);
        else
            gen_push_kernel<uint32_t><<<blocks_for(streams * 32, 128), 128, 0, rt->stream>>>(
                blk, stride, ws, vh, wps, row, row + n, row + 2 * n, one, d + 3 * n + t * streams, streams, 1, (uint32_t)capacity,
                rt->dev_status);
        rt->launched("gen_push");
    }
    std::vector<float> y(n);
    rt->d2h(y.data(), d + 3 * n, n * 4);
    rt->d2h(rt->host_status, rt->dev_status, 16);
    rt->sync();
    time += steps;   // the automata have moved on whatever the status says
    rt->throw_on_status();
    for (size_t i = 0; i < n; ++i) idx[i] = y[i] > 0.0f;
}
