// Tensor-core (tcgen05 / TMEM) stages of the forward pass.  Each function
// returns false without launching anything when it does not take the request
// (validation mode, or a shape outside its tiling), in which case the caller
// runs the CUDA-core kernels instead; nothing here ever computes on the host.
#pragma once
#include "model.hpp"

namespace ullis {
namespace tc {

// y = bias + scale * (x . sign^T), x f32 [rows,K] on the device.
bool binary_linear(ullis_cuda_runtime* rt, const float* x, const uint32_t* bits, const uint16_t* scale,
                   const uint16_t* bias, float* y, size_t rows, size_t in_features, size_t out_features);
// y = x . W^T, W FP16 [out,in].
bool fp16_linear(ullis_cuda_runtime* rt, const float* x, const uint16_t* w, float* y, size_t rows,
                 size_t in_features, size_t out_features);
// y [M,N] f32 = a . b^T with both operands already FP16: a [M,K], b [N,K] (K a multiple of 64).
bool dense_nt(ullis_cuda_runtime* rt, const uint16_t* a16, const uint16_t* b16, float* y, size_t M, size_t K,
              size_t N);
// ln3 output -> time-shift mixes -> packed Q,K,V -> stream-major sign bits.  With `x_before_ln` the LayerNorm
// itself is part of the call (L.ln3 over x_before_ln, folded into the operand kernel where the width allows) and
// its output is left in `ln3_write`, which must be the buffer `ln3_out` names.
bool rosa_qkv_bits(ullis_cuda_runtime* rt, const float* ln3_out, const LayerWeights& L, uint32_t* q_sw,
                   uint32_t* k_sw, uint32_t* v_sw, size_t batch, size_t time, size_t d,
                   const float* x_before_ln = nullptr, float* ln3_write = nullptr);
// x += O((2*idx-1)*e)
bool rosa_out_residual(ullis_cuda_runtime* rt, const uint32_t* idx_sw, const LayerWeights& L, float* x,
                       size_t batch, size_t time, size_t d);
// x += value(relu(key(mix(ln2(x))))^2)
bool cmix_residual(ullis_cuda_runtime* rt, const LayerWeights& L, float* x, size_t batch, size_t time, size_t d,
                   size_t ffn);
// row_loss from hidden without materialising logits.
bool head_ce(ullis_cuda_runtime* rt, const float* hidden, const PackedWeights& head, const uint32_t* labels,
             uint32_t ignore_id, size_t rows, size_t time, size_t d, size_t vocab, float* row_loss);

// Makes a bounded device wait run out on purpose (a barrier nothing arrives on, `polls` polls): the kernel
// returns by itself and leaves ULLIS_DEV_WAIT_TIMEOUT in the runtime's status words.
void wait_selftest(ullis_cuda_runtime* rt, uint32_t polls);

// True when every stage above takes a model of these dimensions at `rows` rows per call (so that a forward
// can count on none of the CUDA-core fall-backs, which share buffers, being reached).
bool takes_model(ullis_cuda_runtime* rt, size_t rows, size_t time, size_t d, size_t ffn, size_t vocab);

}  // namespace tc
}  // namespace ullis
