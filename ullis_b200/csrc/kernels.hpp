// Launchers of the backend's kernels. All pointers are DEVICE pointers; every
// launcher enqueues on rt->stream and counts itself in rt->launches.
#pragma once
#include "common.hpp"

namespace ullis {
namespace k {

// ---- elementwise.cu
// x[row,:] = f32(embedding[id*D ..]); ids >= vocab set the device status word.
void embed(ullis_cuda_runtime* rt, const uint32_t* ids, const uint16_t* emb, float* x, size_t rows, size_t d,
           size_t vocab);
// LayerNorm, eps 1e-5, FP16 affine. exact: reference summation order.
void layer_norm(ullis_cuda_runtime* rt, const float* x, const uint16_t* w, const uint16_t* b, float* y,
                size_t rows, size_t channels, bool exact);
void time_shift_delta(ullis_cuda_runtime* rt, const float* x, float* xx, size_t rows, size_t time,
                      size_t channels);
// out_m = x + xx*mix_m with xx = x[t-1]-x[t] (first step of a sequence: -x),
// unfused multiply/add; m1/m2 (and o1/o2) may be null.
void shift_mix(ullis_cuda_runtime* rt, const float* x, const uint16_t* m0, const uint16_t* m1,
               const uint16_t* m2, float* o0, float* o1, float* o2, size_t rows, size_t time, size_t channels);
void sign_pack_flat(ullis_cuda_runtime* rt, const float* x, uint32_t* words, size_t n);
// Stream-major bit words: stream s = b*C + c owns words [s*wps, (s+1)*wps),
// wps = ceil(T/32), bit t of the stream at word t/32, bit t%32.
void sign_pack_streams(ullis_cuda_runtime* rt, const float* x, uint32_t* sw, size_t batch, size_t time,
                       size_t channels);
void planes_to_streams(ullis_cuda_runtime* rt, const uint32_t* plane, uint32_t* sw, size_t batch, size_t time,
                       size_t channels);
void streams_to_planes(ullis_cuda_runtime* rt, const uint32_t* sw, uint32_t* plane, size_t batch, size_t time,
                       size_t channels);
void relu2(ullis_cuda_runtime* rt, const float* x, float* y, size_t n);
void residual_add(ullis_cuda_runtime* rt, const float* a, const float* b, float* out, size_t n);
// From stream-major idx bits: idx u8 [B,T,C] (nullable) and y = (2*idx-1)*e f32 (nullable).
void rosa_emit(ullis_cuda_runtime* rt, const uint32_t* idx_sw, const uint16_t* e, uint8_t* idx, float* y,
               size_t batch, size_t time, size_t channels);

// ---- linear_exact.cu  (CUDA-core f32, reference summation order)
void binary_linear_exact(ullis_cuda_runtime* rt, const float* x, const uint32_t* bits, const uint16_t* scale,
                         const uint16_t* bias, float* y, size_t rows, size_t in_features, size_t out_features,
                         bool accumulate);
void fp16_linear_exact(ullis_cuda_runtime* rt, const float* x, const uint16_t* w, float* y, size_t rows,
                       size_t in_features, size_t out_features, bool accumulate);
// `count` (1 to 3) packed matvecs of one shape in one launch, for few rows (a generation step): y[z] = x[z] W[z]^T
// with W[z]'s scale and bias (bias[z] nullable), optionally followed by relu^2; the sums of binary_linear_exact.
// Returns false (nothing launched) when the shape is not one it takes.
bool binary_rowvec_multi(ullis_cuda_runtime* rt, int count, const float* const* x, const uint32_t* const* bits,
                         const uint16_t* const* scale, const uint16_t* const* bias, float* const* y, size_t rows,
                         size_t in_features, size_t out_features, bool relu2);
// One-time set-up of the few-row kernels (shared-memory allowance); the linears do it on first use, a caller that
// is about to record them into a CUDA graph does it beforehand.
void rowvec_prepare(ullis_cuda_runtime* rt);

// ---- sam.cu
// idx_sw <- suffix-automaton match of each stream; uses rt->sam_scratch.  `site` names the caller's call site (a
// model passes its layer): calls of one site are expected to send a similar number of streams to the automaton,
// which picks the kernel of the serial pass; -1 = a site shared by every other caller.
void rosa_sam(ullis_cuda_runtime* rt, const uint32_t* q_sw, const uint32_t* k_sw, const uint32_t* v_sw,
              uint32_t* idx_sw, size_t streams, size_t time, int site = -1);
size_t rosa_sam_scratch_bytes_per_stream(int algo, size_t time);

// ---- ce.cu
// Per-row CE from materialised logits [rows,V]; rows whose target is ignored
// or past the sequence end get 0. Targets >= vocab set the status word.
void ce_rows_from_logits(ullis_cuda_runtime* rt, const float* logits, const uint32_t* labels, uint32_t ignore_id,
                         size_t row0, size_t rows, size_t total_rows, size_t time, size_t vocab, float* row_loss);
// loss_sum (f64) and n_valid over row_loss / labels, fixed-order reduction.  `pair` (nullable, device)
// receives the same two numbers as doubles, the form the data-parallel all-reduce sums.
void ce_reduce(ullis_cuda_runtime* rt, const float* row_loss, const uint32_t* labels, uint32_t ignore_id,
               size_t rows, size_t time, double* loss_sum, unsigned long long* n_valid, double* pair = nullptr);


// ---- train.cu  (op-level forms of the training kernels)
// Fp16Storage::apply_clipped_sgd element by element (src/precision.rs:106-113), in place.
void clipped_sgd(ullis_cuda_runtime* rt, uint16_t* w, float* residual, const float* g, float lr, size_t n);
// apply_binaryconnect_sgd on g * ste_scale (src/precision.rs:124-134), in place; bits (nullable) <- latent >= 0.
void latent_sgd(ullis_cuda_runtime* rt, uint16_t* latent, float* residual, const float* g, float lr, float ste_scale,
                uint32_t* bits, size_t n);
// g_e[c] = sum over rows of gy * (2*idx - 1)   (src/model.rs:1608-1634)
void rosa_e_grad(ullis_cuda_runtime* rt, const float* gy, const uint8_t* idx, float* g_e, size_t rows, size_t channels,
                 DeviceBuffer& scratch);
// g <- input > 0 ? 2*input*g : 0   (src/model.rs:1189-1204)
void relu2_backward(ullis_cuda_runtime* rt, const float* input, float* g, size_t n);
// LayerNorm::backward (src/model.rs:270-315); xhat is scratch of the input's size.
void layer_norm_backward(ullis_cuda_runtime* rt, const float* x, const float* gy, const uint16_t* w, float* gx,
                         float* xhat, float* gw, float* gb, size_t rows, size_t channels, DeviceBuffer& scratch);

}  // namespace k
}  // namespace ullis
