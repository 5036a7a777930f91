// Device-resident state of incremental generation (reference HeronGenerateState,
// src/model.rs:2433-2454): per layer one suffix automaton per (sequence,
// channel) and the two time-shift inputs; `batch` independent sequences advance
// in lock step.
#pragma once
#include "model.hpp"

struct ullis_cuda_generate_state {
    ullis_cuda_model* model = nullptr;
    size_t batch = 0, time = 0;
    bool narrow = true;          // 16-bit state ids (context_len <= 32766)
    size_t stride = 0, wps = 0;  // bytes of one automaton block, v-history words per stream
    size_t streams = 0;          // layers * batch * d_model
    ullis::DeviceBuffer blocks, walkers, vhist, prev;
    // activations of one step (owned here, so that a captured graph's pointers stay valid)
    ullis::DeviceBuffer ids, x, a, bq, bk, bv, wide, logits;
    uint32_t* h_tokens = nullptr;   // pinned staging of the step's inputs / outputs
    float* h_logits = nullptr;
    // The step as a CUDA graph: [0] before the first token (no time-shift history), [1] afterwards.
    bool use_graph = true;
    cudaGraphExec_t graph[2] = {nullptr, nullptr};
    uint64_t graph_launches = 0;    // kernels inside one replay
    // A step that fails after its kernels were enqueued leaves the device-side automata one position ahead of
    // `time`; the state then refuses further steps until reset().
    bool poisoned = false;
    // Test hook (ULLIS_CUDA_INJECT_GENERATE_FAILURE=n when the state is created): step n fails on the host after
    // its kernels have run, the way a CUDA error reported at the synchronisation would.
    size_t inject_failure_at = 0;

    ullis_cuda_generate_state(ullis_cuda_model* m, size_t batch);
    ~ullis_cuda_generate_state();
    ullis_cuda_generate_state(const ullis_cuda_generate_state&) = delete;
    ullis_cuda_generate_state& operator=(const ullis_cuda_generate_state&) = delete;
    void reset();
    void enqueue(int has_prev);   // copies in, every kernel of one step, copies out; no synchronisation
    // tokens [batch] (host) -> logits [batch, vocab] (host); advances time by one
    void step(const uint32_t* tokens, float* logits);
};

// `streams` independent RosaSam automata (src/rosa.rs:55-176) kept on the device between calls: the op-level form
// of what a generate state holds per layer.  push() advances every stream by `steps` positions.
struct ullis_cuda_rosa_pushers {
    ullis_cuda_runtime* rt = nullptr;
    size_t streams = 0, capacity = 0, time = 0;
    bool narrow = true;
    size_t stride = 0, wps = 0;
    ullis::DeviceBuffer blocks, walkers, vhist, io;

    ullis_cuda_rosa_pushers(ullis_cuda_runtime* rt, size_t streams, size_t capacity);
    void reset();
    // q, k, v, idx: [steps, streams] bytes of 0 / 1 on the host
    void push(const uint8_t* q, const uint8_t* k, const uint8_t* v, size_t steps, uint8_t* idx);
};
