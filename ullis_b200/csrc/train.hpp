// Optimiser carry and scratch of a device-resident training step in
// rosa_grad = stop_grad_bits mode (reference src/model.rs:2827-3020): the FP16
// BinaryConnect latents of the packed matrices that learn (head, ROSA O, CMix
// key), the f32 carry of every FP16 tensor that is stepped
// (src/precision.rs:106-134), and the gradient buffers of one step.
#pragma once
#include <map>
#include <string>
#include <vector>

#include "model.hpp"

namespace ullis {

struct Fp16Param {      // an FP16 tensor of the model with its f32 carry
    uint16_t* w = nullptr;
    float* residual = nullptr;
    size_t n = 0;
};

struct PackedParam {    // PackedBinaryLinear with its latent (src/model.rs:560-567)
    PackedWeights* weights = nullptr;
    uint16_t* latent = nullptr;
    float* latent_residual = nullptr;
    Fp16Param scale, bias;   // bias.w null when the matrix has none
};

}  // namespace ullis

struct ullis_cuda_train_state {
    ullis_cuda_model* m = nullptr;
    ullis_cuda_runtime* rt = nullptr;
    ullis::DeviceBuffer carry;   // latents + residuals, one allocation
    ullis::PackedParam head;
    ullis::Fp16Param embedding, ln_out_w, ln_out_b;
    struct Layer {
        ullis::Fp16Param ln0_w, ln0_b, ln2_w, ln2_b, e, x_k, value;
        ullis::PackedParam o, key;
    };
    std::vector<Layer> layers;
    struct Named { void* ptr; size_t bytes; };
    std::map<std::string, Named> named;   // every tensor a caller may read back, by checkpoint name

    // step scratch (grow-only)
    ullis::DeviceBuffer gx, t1, t2, t3, wide1, wide2, logits, a16, b16, gmat, part, small, counters, order, starts,
        toks;
    uint64_t steps = 0;

    ullis_cuda_train_state(ullis_cuda_model* model, const uint8_t* checkpoint, size_t len);
    void step(const uint32_t* tokens, const uint32_t* labels, uint32_t ignore_id, size_t batch, size_t time,
              float learning_rate, ullis_cuda_train_result* out);
    void read(const char* name, void* dst, size_t bytes);
    void install_head_unigram_prior(const uint32_t* labels, size_t n, uint32_t ignore_id,
                                    ullis_cuda_head_unigram_install* out);
};
