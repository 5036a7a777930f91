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

    ullis_cuda_generate_state(ullis_cuda_model* m, size_t batch);
    void reset();
    // tokens [batch] (host) -> logits [batch, vocab] (host); advances time by one
    void step(const uint32_t* tokens, float* logits);
};
