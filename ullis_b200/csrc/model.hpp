// Device-resident Heron model: weights parsed from a v2 checkpoint into one
// device arena, activation buffers sized on first use, and the forward + CE
// schedule (reference src/model.rs:2644-2688, 2224-2241, 3205-3228).
#pragma once
#include <string>
#include <vector>

#include "common.hpp"

namespace ullis {

struct PackedWeights {  // PackedBinaryLinear, src/model.rs:560-567 (forward fields)
    const uint32_t* bits = nullptr;
    const uint16_t* scale = nullptr;
    const uint16_t* bias = nullptr;  // null when the matrix has none (CMix key)
    size_t out = 0, in = 0;
};

struct LayerNormWeights {  // src/model.rs:232-235
    const uint16_t* weight = nullptr;
    const uint16_t* bias = nullptr;
};

struct LayerWeights {  // HeronBlock, src/model.rs:2215-2221
    LayerNormWeights ln0, ln2, ln3;  // ln0 only on layer 0
    const uint16_t *x_q = nullptr, *x_k = nullptr, *x_v = nullptr, *e = nullptr;
    PackedWeights q, k, v, o;
    const uint16_t* ffn_x_k = nullptr;
    PackedWeights key;
    const uint16_t* value = nullptr;  // [d_model, dim_ffn] FP16
};

enum Phase { PH_EMBED_LN = 0, PH_QKV, PH_SAM, PH_O, PH_CMIX, PH_HEAD_CE, PH_COUNT };

}  // namespace ullis

struct ullis_cuda_model {
    ullis_cuda_runtime* rt = nullptr;
    size_t d = 0, layers = 0, vocab = 0, context_len = 0, batch_size = 0, ffn = 0;
    ullis::DeviceBuffer arena;  // all weights
    const uint16_t* embedding = nullptr;
    ullis::LayerNormWeights ln_out;
    ullis::PackedWeights head;
    std::vector<ullis::LayerWeights> blocks;

    // activations (grow-only)
    ullis::DeviceBuffer ids, labels, x, a, b, c, dd, wide, q_sw, k_sw, v_sw, idx_sw, logits, row_loss, result;
    size_t cur_batch = 0, cur_time = 0;
    bool have_result = false;
    bool have_pair = false;   // result also holds {sum, count} as two doubles that no all-reduce has consumed yet

    // training tape: the residual stream after each ROSA block and the idx bits, kept per layer
    bool train_tape = false;
    std::vector<ullis::DeviceBuffer> tape_after, tape_idx;

    // taps
    bool taps_enabled = false;
    size_t tap_rows = 0;
    std::vector<ullis::DeviceBuffer> tap_bufs;  // layers * 8 + 1

    // phase profile
    bool profile = false;
    struct Span { int phase; cudaEvent_t start, stop; };
    std::vector<Span> spans;
    size_t spans_used = 0;

    ~ullis_cuda_model();
    void load(const uint8_t* bytes, size_t len);
    void upload_tokens(const uint32_t* tokens, const uint32_t* labels, size_t batch, size_t time);
    void check_shape(size_t batch, size_t time) const;
    // A share of the batch (whole sequences) and the runtime - the model's own or one of its children - whose
    // stream and scratch carry it.
    struct Lane { ullis_cuda_runtime* rt; size_t seq0, nseq; };
    std::vector<Lane> lanes;          // of the forward being enqueued (lane 0 runs on the model's runtime)
    bool lanes_open = false;          // other shares may still be running: nothing on rt->stream has waited for them
    // x <- hidden() ; leaves ln_out output in buffer `a` as f32 [rows, d].  With join = false the shares are
    // left running on their streams (the caller appends per-share work and calls join_lanes()).
    void enqueue_hidden(size_t batch, size_t time, bool join = true);
    void join_lanes();                // the model's stream waits for every share
    void enqueue_forward_ce(uint32_t ignore_id, size_t batch, size_t time);
    void enqueue_logits(size_t batch, size_t time, float* host_logits);
    void read_loss(float* mean_loss, double* loss_sum, uint64_t* n_valid, float* row_loss, size_t rows);
    void read_loss_global(float* mean_loss, double* loss_sum, uint64_t* n_valid);
    void tap(int layer, int which, void* out, size_t bytes);
    void phase_ms(float ms[6]);

   private:
    void begin(int phase, ullis_cuda_runtime* on = nullptr);
    void end(ullis_cuda_runtime* on = nullptr);
    void enqueue_layer(const Lane& lane, size_t l, size_t time);
    void save_tap(int layer, int which, const void* src, size_t bytes);
    void save_tap_bits(int layer, int which, const uint32_t* sw, size_t batch, size_t time);
};
