/*
 * ullis_cuda.h - C ABI of the B200 (sm_100a) `cuda` backend for the Heron
 * forward + next-token cross-entropy path of Ullis.
 *
 * This is the drop-in boundary beside the reference's Metal backend: the
 * entry points are what a `src/cuda.rs` sitting next to `src/metal.rs` binds
 * over FFI.  Conventions shared by every function:
 *
 *  - plain pointers and sizes only; FP16 parameters cross as raw IEEE
 *    binary16 bit patterns (`uint16_t`), packed +/-1 weights as `uint32_t`
 *    words in the checkpoint's order (row-major [out,in], bit (o*in+i) of an
 *    LSB-first word stream, 1 => +1, 0 => -1; reference src/model.rs:146-148,
 *    2267-2268);
 *  - op-level calls take HOST pointers for inputs and caller-allocated HOST
 *    outputs, are synchronous, and mirror the `MetalRuntime` method of the
 *    same name (reference src/metal.rs, cited per function);
 *  - every call returns an `int32_t` status (0 = ok); the message of the last
 *    failure is available from ullis_cuda_last_error();
 *  - a runtime handle is bound to one device and one host thread at a time;
 *  - there is no CPU fallback: without a CUDA device runtime creation fails.
 */
#ifndef ULLIS_CUDA_H
#define ULLIS_CUDA_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define ULLIS_CUDA_API __attribute__((visibility("default")))
#else
#define ULLIS_CUDA_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef struct ullis_cuda_runtime ullis_cuda_runtime;
typedef struct ullis_cuda_model ullis_cuda_model;
typedef struct ullis_cuda_generate_state ullis_cuda_generate_state;
typedef struct ullis_cuda_rosa_pushers ullis_cuda_rosa_pushers;
typedef struct ullis_cuda_train_state ullis_cuda_train_state;

enum {
    ULLIS_CUDA_OK = 0,
    ULLIS_CUDA_ERR_SHAPE = 1,        /* dimension / length mismatch (reference: bail!("... mismatch")) */
    ULLIS_CUDA_ERR_CHECKPOINT = 2,   /* unparsable, v1, or shape-inconsistent checkpoint */
    ULLIS_CUDA_ERR_CUDA = 3,         /* CUDA runtime error (reference: command buffer error, src/metal.rs:736-738) */
    ULLIS_CUDA_ERR_DEVICE_CHECK = 4, /* a kernel's own bounds / progress check failed */
    ULLIS_CUDA_ERR_NCCL = 5,
    ULLIS_CUDA_ERR_TIMEOUT = 6,
    ULLIS_CUDA_ERR_ARG = 7,          /* null handle / pointer, unknown option */
    ULLIS_CUDA_ERR_TOKEN = 8,        /* token or target id >= vocabulary (src/model.rs:2662-2664) */
    ULLIS_CUDA_ERR_NOMEM = 9
};

/* Arithmetic mode of the linears / LayerNorm.
 * FAST  : tensor-core (tcgen05) GEMMs, warp-shuffle LayerNorm; results within
 *         the stated tolerances of the reference CPU backend.
 * EXACT : f32 accumulation in the reference's summation order on CUDA cores;
 *         every +,-,*,/,sqrt result is bit-identical to the reference CPU
 *         backend (validation mode, much slower). */
enum { ULLIS_CUDA_MODE_FAST = 0, ULLIS_CUDA_MODE_EXACT = 1 };

/* Suffix-automaton schedule. Both give identical idx.
 * EULER : O(T log T) per stream for any input (default).
 * EAGER : the reference's per-step chain stamping, O(T^2) on constant streams. */
enum { ULLIS_CUDA_SAM_EULER = 0, ULLIS_CUDA_SAM_EAGER = 1 };

/* Which per-layer intermediate ullis_cuda_model_tap returns (all row-major
 * [B*T, C] unless noted; f32 = float, u8 = one byte per element). */
enum {
    ULLIS_CUDA_TAP_BLOCK_IN = 0,   /* f32 residual stream entering the layer (after ln0 on layer 0) */
    ULLIS_CUDA_TAP_LN3_OUT = 1,    /* f32 */
    ULLIS_CUDA_TAP_Q_BITS = 2,     /* u8 0/1 */
    ULLIS_CUDA_TAP_K_BITS = 3,     /* u8 0/1 */
    ULLIS_CUDA_TAP_V_BITS = 4,     /* u8 0/1 */
    ULLIS_CUDA_TAP_IDX = 5,        /* u8 0/1 */
    ULLIS_CUDA_TAP_AFTER_ROSA = 6, /* f32 residual stream after the ROSA branch */
    ULLIS_CUDA_TAP_BLOCK_OUT = 7,  /* f32 residual stream leaving the layer */
    ULLIS_CUDA_TAP_HIDDEN = 8      /* f32 ln_out output (layer argument ignored) */
};

/* ---------------------------------------------------------------- lifecycle
 * Replaces MetalRuntime::new (src/metal.rs:466) and the `--backend` runtime
 * construction in train() (src/main.rs:650-678). */
ULLIS_CUDA_API int32_t ullis_cuda_runtime_create(int32_t device, ullis_cuda_runtime** out);
ULLIS_CUDA_API void ullis_cuda_runtime_destroy(ullis_cuda_runtime* rt);
/* Message of the last failed call on `rt` (or of the last failed
 * ullis_cuda_runtime_create when rt is NULL). Never NULL. */
ULLIS_CUDA_API const char* ullis_cuda_last_error(const ullis_cuda_runtime* rt);
ULLIS_CUDA_API int32_t ullis_cuda_runtime_set_mode(ullis_cuda_runtime* rt, int32_t mode);
ULLIS_CUDA_API int32_t ullis_cuda_runtime_set_sam(ullis_cuda_runtime* rt, int32_t sam_algo);
/* MetalRuntime::synchronize (src/metal.rs:598). */
ULLIS_CUDA_API int32_t ullis_cuda_runtime_synchronize(ullis_cuda_runtime* rt);
/* The CUDA stream (cudaStream_t) every kernel of this runtime is launched on. */
ULLIS_CUDA_API void* ullis_cuda_runtime_stream(ullis_cuda_runtime* rt);
/* Number of this library's kernels launched through `rt` so far. */
ULLIS_CUDA_API uint64_t ullis_cuda_runtime_launch_count(const ullis_cuda_runtime* rt);
/* Per-kernel device times (no counterpart in the reference; the Metal runtime
 * is timed from the host, src/main.rs:706-736).  While enabled, an event is
 * recorded behind every launch of this runtime; `kernel_time` synchronises the
 * stream and returns the total milliseconds and the number of launches recorded
 * under `name` since timing was enabled (all kernels when `name` is NULL or
 * empty).  `kernel_names` writes the distinct names, newline-separated and
 * NUL-terminated, into `buf` (truncated to `len`) and the size needed into
 * `*needed`. */
ULLIS_CUDA_API int32_t ullis_cuda_runtime_kernel_timing(ullis_cuda_runtime* rt, int32_t enabled);
ULLIS_CUDA_API int32_t ullis_cuda_runtime_kernel_time(ullis_cuda_runtime* rt, const char* name, float* total_ms,
                                                      uint32_t* launches);
ULLIS_CUDA_API int32_t ullis_cuda_runtime_kernel_names(ullis_cuda_runtime* rt, char* buf, size_t len, size_t* needed);
/* How the last suffix-automaton call on `rt` (op-level or inside a model forward: the last layer's) split its
 * streams: `automaton` streams went through the automaton kernels, `constant_q` were settled by the
 * constant-query closed form, and the rest of `total` by the other closed forms (constant key or value bits).
 * No counterpart in the reference, which runs every stream through RosaSam.  Synchronises. */
ULLIS_CUDA_API int32_t ullis_cuda_runtime_sam_counts(ullis_cuda_runtime* rt, uint64_t* total, uint64_t* automaton,
                                                     uint64_t* constant_q);
/* Error-path self-test: one small kernel waits - with the bounded mbarrier wait that every tensor-core kernel of
 * the library uses, cut to `polls` polls (1..2^20) - on a barrier nothing ever arrives on, gives up, returns by
 * itself and reports through the device status words.  The expected result is ULLIS_CUDA_ERR_TIMEOUT with
 * "a kernel gave up waiting" as the message; the runtime stays usable.  The reference's counterpart of the path
 * is the command-buffer error check after waitUntilCompleted (src/metal.rs:736-738). */
ULLIS_CUDA_API int32_t ullis_cuda_runtime_wait_selftest(ullis_cuda_runtime* rt, uint32_t polls);
/* Compute capability check: 1 when the device is sm_100 class. */
ULLIS_CUDA_API int32_t ullis_cuda_runtime_is_sm100(const ullis_cuda_runtime* rt);

/* -------------------------------------------------------------------- model
 * Device-resident whole-model path.  `bytes` is a v2 checkpoint.safetensors
 * exactly as ModelCheckpoint::to_safetensors_bytes writes it
 * (src/model.rs:3426-3468); loading follows from_safetensors_bytes /
 * validate_checkpoint_shapes / heron_from_checkpoint (src/model.rs:3470-3553,
 * 4402-4456, 4258-4309): format_version must be 2, a missing head bias loads
 * as zeros, train-carry tensors are ignored. */
ULLIS_CUDA_API int32_t ullis_cuda_model_load_safetensors(ullis_cuda_runtime* rt, const uint8_t* bytes, size_t len,
                                          ullis_cuda_model** out);
ULLIS_CUDA_API void ullis_cuda_model_destroy(ullis_cuda_model* model);
/* d_model, n_layers, vocab_size, context_len, batch_size, dim_ffn (resolved). */
ULLIS_CUDA_API int32_t ullis_cuda_model_dims(const ullis_cuda_model* model, size_t dims[6]);

/* Forward + next-token CE: UllisHeron::hidden (src/model.rs:2644-2683) followed
 * by the CE forward of apply_head_ce (src/model.rs:3205-3228, 3253-3257) with
 * the valid-row rule of causal_ce_row_valid (src/model.rs:27-39), horizon 1.
 * tokens, labels: [batch*time] host; ignore_id = UINT32_MAX supervises every
 * in-range target.  Outputs (each nullable): mean_loss = loss_sum / n_valid
 * (0 when n_valid is 0), loss_sum, n_valid, row_loss [batch*time] (0 on
 * invalid rows).  Rejects batch > config.batch_size, time > context_len and
 * ids >= vocab like the reference. */
ULLIS_CUDA_API int32_t ullis_cuda_model_forward_ce(ullis_cuda_model* model, const uint32_t* tokens, const uint32_t* labels,
                                    uint32_t ignore_id, size_t batch, size_t time, float* mean_loss,
                                    double* loss_sum, uint64_t* n_valid, float* row_loss);
/* The same step split for device-resident timing: copy ids in, enqueue every
 * kernel on the runtime stream without synchronising, read the result. */
ULLIS_CUDA_API int32_t ullis_cuda_model_upload_tokens(ullis_cuda_model* model, const uint32_t* tokens, const uint32_t* labels,
                                       size_t batch, size_t time);
ULLIS_CUDA_API int32_t ullis_cuda_model_enqueue_forward_ce(ullis_cuda_model* model, uint32_t ignore_id, size_t batch,
                                            size_t time);
ULLIS_CUDA_API int32_t ullis_cuda_model_read_loss(ullis_cuda_model* model, float* mean_loss, double* loss_sum,
                                   uint64_t* n_valid, float* row_loss, size_t rows);

/* read_loss for a rank of a data-parallel group (ullis_cuda_dp_init on the model's runtime): the
 * {loss_sum, n_valid} pair of the last forward is summed over the ranks on the device (one 16-byte
 * all-reduce on the runtime stream) and read back once; mean_loss = sum / count over ALL ranks, which is the
 * reference's single-process mean over every valid position (src/model.rs:3253-3257).  One call per forward. */
ULLIS_CUDA_API int32_t ullis_cuda_model_read_loss_global(ullis_cuda_model* model, float* mean_loss, double* loss_sum,
                                                         uint64_t* n_valid);

/* UllisHeron::logits (src/model.rs:2685-2688): logits [batch*time*vocab] host. */
ULLIS_CUDA_API int32_t ullis_cuda_model_logits(ullis_cuda_model* model, const uint32_t* tokens, size_t batch, size_t time,
                                float* logits);
/* UllisHeron::hidden (src/model.rs:2644-2683): hidden [batch*time*d_model] host. */
ULLIS_CUDA_API int32_t ullis_cuda_model_hidden(ullis_cuda_model* model, const uint32_t* tokens, size_t batch, size_t time,
                                float* hidden);
/* Keep per-layer intermediates of the next forward (costs memory; for parity
 * tests) and read one of them back. `bytes` must equal the tap's size. */
ULLIS_CUDA_API int32_t ullis_cuda_model_set_taps(ullis_cuda_model* model, int32_t enabled);
ULLIS_CUDA_API int32_t ullis_cuda_model_tap(ullis_cuda_model* model, int32_t layer, int32_t which, void* out, size_t bytes);
/* Milliseconds of the last enqueue_forward_ce spent in each phase, measured
 * with CUDA events when profiling is enabled (same phase idea as the
 * reference's TrainStepProfile, src/model.rs:101-124):
 * [embed_ln, qkv, sam, o, cmix, head_ce]. */
ULLIS_CUDA_API int32_t ullis_cuda_model_set_profile(ullis_cuda_model* model, int32_t enabled);
ULLIS_CUDA_API int32_t ullis_cuda_model_phase_ms(ullis_cuda_model* model, float ms[6]);

/* ----------------------------------------------------------------- generate
 * Incremental generation with the state on the device (HeronGenerateState,
 * src/model.rs:2433-2454): per layer one suffix automaton per (sequence,
 * channel) plus the ROSA and CMix time-shift inputs.  The reference generates
 * one sequence; here `batch` independent sequences advance in lock step.
 * Arithmetic is the reference's (CUDA cores, its summation order), whatever
 * the runtime's mode: the logits of step t are bit-identical to row t of
 * ullis_cuda_model_logits in ULLIS_CUDA_MODE_EXACT (src/model.rs:4991-5004). */

/* UllisHeron::generate_state (src/model.rs:2691-2715): empty automata sized for
 * the model's context_len, no time-shift history, time 0.  The state borrows
 * `model`; destroy it before the model. */
ULLIS_CUDA_API int32_t ullis_cuda_generate_state_create(ullis_cuda_model* model, size_t batch,
                                                        ullis_cuda_generate_state** out);
ULLIS_CUDA_API void ullis_cuda_generate_state_destroy(ullis_cuda_generate_state* state);
/* Back to time 0 without reallocating (RosaSam::reset, src/rosa.rs:66-74). */
ULLIS_CUDA_API int32_t ullis_cuda_generate_state_reset(ullis_cuda_generate_state* state);
/* HeronGenerateState::time (src/model.rs:2449-2453): tokens consumed so far. */
ULLIS_CUDA_API size_t ullis_cuda_generate_state_time(const ullis_cuda_generate_state* state);
/* UllisHeron::generate_step (src/model.rs:2717-2753): one token per sequence
 * (tokens [batch]) -> last-token logits [batch, vocab].  ULLIS_CUDA_ERR_TOKEN
 * for a token id >= vocab, ULLIS_CUDA_ERR_SHAPE once time == context_len; in
 * both cases the state is unchanged. */
ULLIS_CUDA_API int32_t ullis_cuda_generate_step(ullis_cuda_generate_state* state, const uint32_t* tokens,
                                                float* logits);

/* RosaSam (src/rosa.rs:55-176) for `streams` independent 1-bit streams, kept on
 * the device between calls: what a generate state holds per layer, at op
 * level.  `capacity` is the number of pushes a stream can take (RosaSam grows
 * without bound; here the memory is sized once).  RosaSam::push
 * (src/rosa.rs:100-176) for every stream, `steps` times: q, k, v and idx are
 * host arrays [steps, streams] of 0 / 1 bytes; idx[s, c] is what the
 * reference's push returns for stream c at its position time + s.
 * ULLIS_CUDA_ERR_SHAPE (nothing pushed) when time + steps > capacity. */
ULLIS_CUDA_API int32_t ullis_cuda_rosa_pushers_create(ullis_cuda_runtime* rt, size_t streams, size_t capacity,
                                                      ullis_cuda_rosa_pushers** out);
ULLIS_CUDA_API void ullis_cuda_rosa_pushers_destroy(ullis_cuda_rosa_pushers* pushers);
/* RosaSam::reset (src/rosa.rs:66-74). */
ULLIS_CUDA_API int32_t ullis_cuda_rosa_pushers_reset(ullis_cuda_rosa_pushers* pushers);
ULLIS_CUDA_API int32_t ullis_cuda_rosa_pushers_push(ullis_cuda_rosa_pushers* pushers, const uint8_t* q, const uint8_t* k,
                                                    const uint8_t* v, size_t steps, uint8_t* idx);

/* -------------------------------------------------------------------- train
 * One optimiser step with the weights, the BinaryConnect latents and the f32
 * carry on the device: UllisHeron::train_step_with_labels
 * (src/model.rs:2773-2785, train_step_on 2827-3020) in rosa_grad =
 * stop_grad_bits mode, the only mode the reference wires.  Q/K/V, their
 * time-shift mixes and ln3 are frozen; the head, ROSA O and e, CMix, the other
 * LayerNorms and the embedding rows are stepped (clipped SGD with an f32 carry,
 * BinaryConnect for the packed latents, src/precision.rs:106-134).  The loss
 * and the flip counts are exact restatements; the gradients are FP16-operand
 * tensor-core products with f32 accumulation, so updated tensors agree with the
 * reference's CPU step to gradient rounding, not bit for bit. */

/* Optimiser state for `model` (which it borrows and MODIFIES).  `checkpoint`
 * (nullable) is the safetensors file the model was loaded from: its
 * "<name>.latent" / "<name>.residual" tensors restore a resumed run's carry
 * (src/model.rs:3461-3466); without them latents start at +/-0.01 by the sign
 * bit (src/model.rs:640-649) and residuals at zero. */
ULLIS_CUDA_API int32_t ullis_cuda_train_state_create(ullis_cuda_model* model, const uint8_t* checkpoint, size_t len,
                                                     ullis_cuda_train_state** out);
ULLIS_CUDA_API void ullis_cuda_train_state_destroy(ullis_cuda_train_state* state);
/* CausalLoss fields the step itself produces (src/model.rs:60-83). */
typedef struct ullis_cuda_train_result {
    float mean_loss;      /* next_token */
    uint64_t n_valid;     /* next_token_count */
    uint64_t flips_head, flips_cmix, flips_rosa_o;
} ullis_cuda_train_result;
/* tokens, labels [batch*time] on the host.  ULLIS_CUDA_ERR_ARG unless
 * learning_rate is finite and positive and time >= 2; ULLIS_CUDA_ERR_SHAPE
 * for a shape or id the reference rejects (src/model.rs:2849-2861). */
ULLIS_CUDA_API int32_t ullis_cuda_model_train_step(ullis_cuda_train_state* state, const uint32_t* tokens,
                                                   const uint32_t* labels, uint32_t ignore_id, size_t batch,
                                                   size_t time, float learning_rate,
                                                   ullis_cuda_train_result* result);
/* Copies a tensor of the trained model or of its carry to the host by its
 * checkpoint name ("head.bits", "blocks.0.rosa.o.latent", "embedding.residual",
 * ...; src/model.rs:3428-3466); `bytes` must be the tensor's size. */
ULLIS_CUDA_API int32_t ullis_cuda_train_state_read(ullis_cuda_train_state* state, const char* name, void* dst,
                                                   size_t bytes);

/* UllisHeron::install_head_unigram_prior (src/model.rs:3034-3110): bias[v] =
 * log((count_v + 1) / (n + V)) minus its mean over the vocabulary, from the
 * supervised labels, and the row scales times 0.25 if their mean is still
 * within a factor two of 1/sqrt(d_model).  Skipped (applied = 0) when mean
 * |bias| already exceeds 0.05.  ULLIS_CUDA_ERR_ARG without any supervised label. */
typedef struct ullis_cuda_head_unigram_install {
    int32_t applied;
    uint64_t n_targets;
    float bias_rms, scale_rms;
    int32_t shrunk_kaiming_scale;
} ullis_cuda_head_unigram_install;
ULLIS_CUDA_API int32_t ullis_cuda_train_state_install_head_unigram_prior(ullis_cuda_train_state* state,
                                                                         const uint32_t* labels, size_t n,
                                                                         uint32_t ignore_id,
                                                                         ullis_cuda_head_unigram_install* result);

/* ------------------------------------------------------------------ op level
 * Host pointers in, caller-allocated host buffers out; one synchronous call
 * each, like the MetalRuntime methods they mirror. */

/* MetalRuntime::layer_norm (src/metal.rs:1590); LayerNorm::forward
 * (src/model.rs:259-276), eps 1e-5. weight/bias are FP16 bits. */
ULLIS_CUDA_API int32_t ullis_cuda_layer_norm(ullis_cuda_runtime* rt, const float* x, const uint16_t* weight,
                              const uint16_t* bias, float* y, size_t rows, size_t channels);
/* MetalRuntime::time_shift_delta (src/metal.rs:1103); src/model.rs:186-212. */
ULLIS_CUDA_API int32_t ullis_cuda_time_shift_delta(ullis_cuda_runtime* rt, const float* x, float* xx, size_t rows, size_t time,
                                    size_t channels);
/* MetalRuntime::binary_linear (src/metal.rs:1705); PackedBinaryLinear::forward
 * (src/model.rs:724-742). bias nullable. y [rows*out]. */
ULLIS_CUDA_API int32_t ullis_cuda_binary_linear(ullis_cuda_runtime* rt, const float* x, const uint32_t* bits,
                                 const uint16_t* scale, const uint16_t* bias, float* y, size_t rows,
                                 size_t in_features, size_t out_features);
/* MetalRuntime::fp16_linear (src/metal.rs:2790); Fp16Linear::forward
 * (src/model.rs:419-436). weight FP16 bits [out*in]. */
ULLIS_CUDA_API int32_t ullis_cuda_fp16_linear(ullis_cuda_runtime* rt, const float* x, const uint16_t* weight, float* y,
                               size_t rows, size_t in_features, size_t out_features);
/* MetalRuntime::sign_pack_bits (src/metal.rs:1142); bit = x > 0, 32 per word
 * LSB-first (src/rosa.rs:372-374, 400-411). bits [(n+31)/32]. */
ULLIS_CUDA_API int32_t ullis_cuda_sign_pack_bits(ullis_cuda_runtime* rt, const float* x, uint32_t* bits, size_t n);
/* MetalRuntime::cmix_relu2 (src/metal.rs:1542): max(v,0)^2. */
ULLIS_CUDA_API int32_t ullis_cuda_cmix_relu2(ullis_cuda_runtime* rt, const float* x, float* y, size_t n);
/* MetalRuntime::residual_add (src/metal.rs:1078): out = residual + update. */
ULLIS_CUDA_API int32_t ullis_cuda_residual_add(ullis_cuda_runtime* rt, const float* residual, const float* update, float* out,
                                size_t n);

/* MetalRuntime::clipped_sgd_fp16 (src/metal.rs:3053): Fp16Storage::apply_clipped_sgd
 * (src/precision.rs:106-113) on every element; FP16 bits and f32 carry in and out.
 * Bit-identical to the reference's CPU step. */
ULLIS_CUDA_API int32_t ullis_cuda_clipped_sgd_fp16(ullis_cuda_runtime* rt, const uint16_t* parameters,
                                                   const float* residual, const float* gradient, float learning_rate,
                                                   size_t n, uint16_t* next_parameters, float* next_residual);
/* MetalRuntime::binaryconnect_sgd_fp16 (src/metal.rs:3069): apply_binaryconnect_sgd
 * (src/precision.rs:124-134). Bit-identical to the reference's CPU step. */
ULLIS_CUDA_API int32_t ullis_cuda_binaryconnect_sgd_fp16(ullis_cuda_runtime* rt, const uint16_t* parameters,
                                                         const float* residual, const float* gradient,
                                                         float learning_rate, size_t n, uint16_t* next_parameters,
                                                         float* next_residual);
/* MetalRuntime::apply_latent_sgd (src/metal.rs:3006): the BinaryConnect step on
 * gradient * ste_scale, then next_bits [(n+31)/32] = latent >= 0 (rebinarize,
 * src/model.rs:878-884). */
ULLIS_CUDA_API int32_t ullis_cuda_apply_latent_sgd(ullis_cuda_runtime* rt, const uint16_t* latent, const float* residual,
                                                   const float* gradient, float learning_rate, float ste_scale, size_t n,
                                                   uint16_t* next_latent, float* next_residual, uint32_t* next_bits);
/* MetalRuntime::rosa_qkv_1bit_bwd_e (src/metal.rs:1258); rosa_e_grad
 * (src/model.rs:1608-1634): g_e[c] = sum over (b,t) of gy * (2*idx - 1). */
ULLIS_CUDA_API int32_t ullis_cuda_rosa_qkv_1bit_bwd_e(ullis_cuda_runtime* rt, const float* output_gradient,
                                                      const uint8_t* idx, size_t batch, size_t time, size_t channels,
                                                      float* g_e);
/* MetalRuntime::cmix_relu2_backward (src/metal.rs:1546): gx = input > 0 ? 2*input*gy : 0. */
ULLIS_CUDA_API int32_t ullis_cuda_cmix_relu2_backward(ullis_cuda_runtime* rt, const float* input,
                                                      const float* output_gradient, float* gx, size_t n);
/* MetalRuntime::layer_norm_backward (src/metal.rs:1628); LayerNorm::backward
 * (src/model.rs:270-315). weight as FP16 bits; gx [rows*channels], gw, gb [channels]. */
ULLIS_CUDA_API int32_t ullis_cuda_layer_norm_backward(ullis_cuda_runtime* rt, const float* input,
                                                      const float* output_gradient, const uint16_t* weight, size_t rows,
                                                      size_t channels, float* gx, float* gw, float* gb);

/* MetalRuntime::rosa_qkv_1bit_fwd (src/metal.rs:1168); rosa_qkv_batch_packed +
 * rosa_qkv_out_batched (src/rosa.rs:459-481, 585-609).  q/k/v_bits: packed
 * planes over the flat [B,T,C] index; e: FP16 bits [C]; idx u8 [B,T,C]
 * (nullable), out f32 [B,T,C] = (2*idx-1)*e (nullable). */
ULLIS_CUDA_API int32_t ullis_cuda_rosa_qkv_1bit_fwd(ullis_cuda_runtime* rt, const uint32_t* q_bits, const uint32_t* k_bits,
                                     const uint32_t* v_bits, const uint16_t* e, uint8_t* idx, float* out,
                                     size_t batch, size_t time, size_t channels);
/* MetalRuntime::rosa_block_forward (src/metal.rs:1334); RwkvRosaQkv1Bit::forward
 * (src/model.rs:1284-1318).  x f32 [B*T*C]; mixes/e FP16 [C]; each linear is
 * {bits [C*C/32], scale [C], bias [C]}.  Outputs (nullable): q/k/v planes
 * packed over [B,T,C], idx u8, y = (2*idx-1)*e f32, out f32 (after O). */
ULLIS_CUDA_API int32_t ullis_cuda_rosa_block_forward(ullis_cuda_runtime* rt, const float* x, const uint16_t* mix_q,
                                      const uint16_t* mix_k, const uint16_t* mix_v, const uint32_t* q_bits,
                                      const uint16_t* q_scale, const uint16_t* q_bias, const uint32_t* k_bits,
                                      const uint16_t* k_scale, const uint16_t* k_bias, const uint32_t* v_bits,
                                      const uint16_t* v_scale, const uint16_t* v_bias, const uint16_t* e,
                                      const uint32_t* o_bits, const uint16_t* o_scale, const uint16_t* o_bias,
                                      size_t batch, size_t time, size_t channels, uint32_t* q_plane,
                                      uint32_t* k_plane, uint32_t* v_plane, uint8_t* idx, float* y, float* out);
/* MetalRuntime::cmix_block_forward (src/metal.rs:1891); RwkvCMixX070::forward
 * (src/model.rs:987-1001). value FP16 [d_model*dim_ffn] (out=d_model). */
ULLIS_CUDA_API int32_t ullis_cuda_cmix_block_forward(ullis_cuda_runtime* rt, const float* x, const uint16_t* mix,
                                      const uint32_t* key_bits, const uint16_t* key_scale,
                                      const uint16_t* value, size_t batch, size_t time, size_t d_model,
                                      size_t dim_ffn, float* out);
/* MetalRuntime::streamed_cross_entropy_fp16 (src/metal.rs:2921), forward part,
 * with the head bias the CPU model applies (src/model.rs:737, 4244); CE as in
 * apply_head_ce (src/model.rs:3205-3228, 3253-3257).  Logits never reach
 * host or (in FAST mode) device memory.  row_loss [rows] nullable. */
ULLIS_CUDA_API int32_t ullis_cuda_streamed_ce(ullis_cuda_runtime* rt, const float* hidden, const uint32_t* bits,
                               const uint16_t* scale, const uint16_t* bias, const uint32_t* labels,
                               uint32_t ignore_id, size_t rows, size_t time, size_t channels, size_t vocab,
                               float* row_loss, float* mean_loss, uint64_t* n_valid);

/* Allocation-free form of the suffix-automaton match.  It has no counterpart
 * in the reference.  For callers that may not allocate device memory while
 * they run (a fixed memory budget owned by the host application, a
 * latency-critical thread that cannot afford cudaMalloc's device-wide
 * synchronisation, a process whose own pool already holds all GPU memory).
 * The caller passes DEVICE buffers: q_sw / k_sw / v_sw / idx_sw hold one row
 * of ceil(time/32) words per stream (stream s = sequence*channels + channel;
 * bit t of the stream at word t/32, bit t%32); idx_sw receives the idx bits
 * in the same layout.  Per-stream automaton state lives in a 64 MiB array
 * built into the library (ULLIS_CUDA_SAM_STATIC_BYTES, resident on every GPU
 * that loads it): 74368 bytes per stream at time 2048, so at most 902
 * streams there; requests beyond it fail with ULLIS_CUDA_ERR_NOMEM.  No
 * cudaMalloc / cudaFree / host allocation happens.  The call is synchronous
 * (it returns after `cuda_stream` has drained), so never issue it on a stream
 * that is being captured; the first call on a device also resolves the array's
 * address and should come before any capture starts.  The caller's current
 * device is left as it was.
 * All calls share the array (nothing needs clearing between calls, every
 * field is written before it is read), so calls that overlap on the GPU race:
 * serialise them.  The kernel is enqueued on `cuda_stream` (a cudaStream_t,
 * NULL = default stream).
 * Failure text: ullis_cuda_last_error(NULL). */
#define ULLIS_CUDA_SAM_STATIC_BYTES ((size_t)64 << 20)
ULLIS_CUDA_API int32_t ullis_cuda_rosa_sam_static(int32_t device, void* cuda_stream, const uint32_t* q_sw,
                                                  const uint32_t* k_sw, const uint32_t* v_sw, uint32_t* idx_sw,
                                                  size_t streams, size_t time);

/* ------------------------------------------------------------ data parallel
 * Sequences are independent; ranks own disjoint blocks of sequences and only
 * {loss_sum, n_valid} is summed across ranks (NCCL all-reduce, 16 bytes).
 * No counterpart in the reference (single process, single device). */
ULLIS_CUDA_API int32_t ullis_cuda_dp_unique_id(uint8_t id[128]);
/* Host-side rendezvous with a deadline, to be called before ullis_cuda_dp_init (whose NCCL bootstrap waits
 * for every rank without one): each rank announces itself with a file `<dir>/<tag>.<rank>` in a directory all
 * ranks of the node share and waits until all `world` files exist.  ULLIS_CUDA_ERR_TIMEOUT when a rank has not
 * shown up within timeout_ms - no NCCL or CUDA call has been made at that point.  `tag` names the group (use a
 * fresh one per job).  Failure text: ullis_cuda_last_error(NULL). */
ULLIS_CUDA_API int32_t ullis_cuda_dp_rendezvous(const char* dir, const char* tag, int32_t rank, int32_t world,
                                                uint32_t timeout_ms);
ULLIS_CUDA_API int32_t ullis_cuda_dp_init(ullis_cuda_runtime* rt, int32_t rank, int32_t world, const uint8_t id[128]);
ULLIS_CUDA_API int32_t ullis_cuda_dp_allreduce_loss(ullis_cuda_runtime* rt, double* loss_sum, uint64_t* n_valid);
ULLIS_CUDA_API int32_t ullis_cuda_dp_finalize(ullis_cuda_runtime* rt);

#ifdef __cplusplus
}
#endif
#endif /* ULLIS_CUDA_H */
