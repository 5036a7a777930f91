/*
 * CPU oracle for the Heron forward + next-token cross-entropy path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is a plain-C restatement of the
 * reference crate's CPU arithmetic (ullis 0.10.0, Rust) for the one hot path
 * the CUDA backend accelerates.  It is linked/loaded only by the parity tests,
 * the smoke check and the CPU-baseline leg of the benchmark; the CUDA product
 * library never calls into it and has no CPU fallback.
 *
 * Every function keeps the reference's loop nesting and f32 summation order
 * (no -ffast-math, no FMA contraction), so results are comparable bit for bit
 * where the arithmetic is integer or uses only +,-,*,/ and sqrt, and to libm
 * accuracy where exp/ln are involved.
 *
 * Parity status: the kernel-level semantics are pinned against every golden
 * vector the reference's own tests hold for this path (tests/rosa.rs,
 * tests/binary_linear.rs, tests/cmix.rs, src/metal.rs test module).  Whole
 * model numeric values (hidden / logits / mean CE) are "parity unpinned" by
 * the reference: it stores no such numbers, and the Rust crate cannot be
 * built where this oracle is developed (no rustc).  They are pinned only by
 * this restatement.
 *
 * Each function cites the reference file:line it follows.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define UO_API __attribute__((visibility("default")))

static int g_threads = 1; /* the reference CPU model path is single-threaded */

UO_API void uo_set_threads(int n) { g_threads = n < 1 ? 1 : n; }
UO_API int uo_get_threads(void) { return g_threads; }
UO_API int uo_max_threads(void) {
#ifdef _OPENMP
    return omp_get_num_procs();
#else
    return 1;
#endif
}

/* ------------------------------------------------------------------ fp16 */

/* src/precision.rs:23-55  Fp16::from_f32 — round to nearest even, subnormals,
 * overflow to inf, NaN -> 0x7e00. */
UO_API uint16_t uo_fp16_from_f32(float value) {
    uint32_t bits;
    memcpy(&bits, &value, 4);
    uint16_t sign = (uint16_t)((bits >> 16) & 0x8000u);
    int32_t exponent = (int32_t)((bits >> 23) & 0xffu);
    uint32_t mantissa = bits & 0x007fffffu;
    if (exponent == 0xff) return (uint16_t)(sign | (mantissa == 0 ? 0x7c00u : 0x7e00u));
    int32_t half_exponent = exponent - 127 + 15;
    if (half_exponent >= 31) return (uint16_t)(sign | 0x7c00u);
    if (half_exponent <= 0) {
        if (half_exponent < -10) return sign;
        uint32_t significand = mantissa | 0x00800000u;
        uint32_t shift = (uint32_t)(14 - half_exponent);
        uint32_t rounded = significand >> shift;
        uint32_t remainder = significand & ((1u << shift) - 1u);
        uint32_t halfway = 1u << (shift - 1u);
        if (remainder > halfway || (remainder == halfway && (rounded & 1u))) rounded += 1u;
        return (uint16_t)(sign | (uint16_t)rounded);
    }
    uint16_t rounded = (uint16_t)(sign | ((uint16_t)half_exponent << 10) | (uint16_t)(mantissa >> 13));
    uint32_t remainder = mantissa & 0x1fffu;
    if (remainder > 0x1000u || (remainder == 0x1000u && (rounded & 1u))) rounded = (uint16_t)(rounded + 1u);
    return rounded;
}

/* src/precision.rs:57-76  Fp16::to_f32 */
UO_API float uo_fp16_to_f32(uint16_t h) {
    uint32_t sign = ((uint32_t)(h & 0x8000u)) << 16;
    uint32_t exponent = (uint32_t)((h >> 10) & 0x1fu);
    uint32_t mantissa = (uint32_t)(h & 0x03ffu);
    uint32_t bits;
    if (exponent == 0) {
        if (mantissa == 0) {
            bits = sign;
        } else {
            uint32_t significand = mantissa;
            int32_t e = -14;
            while ((significand & 0x0400u) == 0) {
                significand <<= 1;
                e -= 1;
            }
            bits = sign | ((uint32_t)(e + 127) << 23) | ((significand & 0x03ffu) << 13);
        }
    } else if (exponent == 31) {
        bits = sign | 0x7f800000u | (mantissa << 13);
    } else {
        bits = sign | ((exponent + 112u) << 23) | (mantissa << 13);
    }
    float out;
    memcpy(&out, &bits, 4);
    return out;
}

UO_API void uo_fp16_from_f32_n(const float* x, uint16_t* out, size_t n) {
    for (size_t i = 0; i < n; ++i) out[i] = uo_fp16_from_f32(x[i]);
}
UO_API void uo_fp16_to_f32_n(const uint16_t* x, float* out, size_t n) {
    for (size_t i = 0; i < n; ++i) out[i] = uo_fp16_to_f32(x[i]);
}

static float* widen(const uint16_t* h, size_t n) {
    float* f = (float*)malloc((n ? n : 1) * sizeof(float));
    for (size_t i = 0; i < n; ++i) f[i] = uo_fp16_to_f32(h[i]);
    return f;
}

/* ------------------------------------------------------------- LayerNorm */

/* src/model.rs:259-276  LayerNorm::forward, eps = LAYER_NORM_EPS = 1e-5
 * (model.rs:132): sequential sum / C, sequential sum of squared deviations
 * / C (population variance), inv = 1/sqrt(var+eps),
 * y = (x-mean)*inv*w + b with w,b widened from FP16. */
UO_API int uo_layer_norm(const float* x, const uint16_t* w_bits, const uint16_t* b_bits, float* y,
                         size_t rows, size_t channels) {
    if (channels == 0) return 1;
    float* w = widen(w_bits, channels);
    float* b = widen(b_bits, channels);
#pragma omp parallel for num_threads(g_threads) schedule(static)
    for (long row = 0; row < (long)rows; ++row) {
        const float* src = x + (size_t)row * channels;
        float* dst = y + (size_t)row * channels;
        float sum = 0.0f;
        for (size_t c = 0; c < channels; ++c) sum += src[c];
        float mean = sum / (float)channels;
        float sq = 0.0f;
        for (size_t c = 0; c < channels; ++c) sq += (src[c] - mean) * (src[c] - mean);
        float var = sq / (float)channels;
        float inv = 1.0f / sqrtf(var + 1e-5f);
        for (size_t c = 0; c < channels; ++c) dst[c] = (src[c] - mean) * inv * w[c] + b[c];
    }
    free(w);
    free(b);
    return 0;
}

/* ------------------------------------------------------------ time shift */

/* src/model.rs:186-212  time_shift_delta: xx[t] = x[t-1] - x[t]; the first
 * step of each sequence has no predecessor and yields -x[0]. */
UO_API int uo_time_shift_delta(const float* x, float* xx, size_t batch, size_t time, size_t channels) {
    if (time == 0 || channels == 0) return 1;
    for (size_t b = 0; b < batch; ++b)
        for (size_t t = 0; t < time; ++t) {
            size_t row = (b * time + t) * channels;
            for (size_t c = 0; c < channels; ++c) {
                float xt = x[row + c];
                xx[row + c] = (t == 0) ? -xt : x[row - channels + c] - xt;
            }
        }
    return 0;
}

/* src/model.rs:1291-1298 (ROSA) and 992-997 (CMix): in = x + xx * mix[c]. */
UO_API void uo_shift_mix(const float* x, const float* xx, const uint16_t* mix_bits, float* out, size_t rows,
                         size_t channels) {
    float* mix = widen(mix_bits, channels);
    for (size_t i = 0; i < rows; ++i)
        for (size_t c = 0; c < channels; ++c) {
            size_t index = i * channels + c;
            out[index] = x[index] + xx[index] * mix[c];
        }
    free(mix);
}

/* --------------------------------------------------------- packed linear */

/* src/model.rs:146-148  bit_is_plus: LSB-first u32 words, bit (o*K+i). */
static inline int bit_is_plus(const uint32_t* bits, size_t index) {
    return (bits[index / 32] & (1u << (index % 32))) != 0;
}

/* src/model.rs:724-742  PackedBinaryLinear::forward, literal loop nest:
 * sum += sign(o,i) * x[row,i] for i ascending, then y = bias + scale*sum
 * (separate multiply and add). bias may be NULL (CMix key). */
UO_API int uo_binary_linear_scalar(const float* x, const uint32_t* bits, const uint16_t* scale_bits,
                                   const uint16_t* bias_bits, float* y, size_t rows, size_t in_features,
                                   size_t out_features) {
    for (size_t row = 0; row < rows; ++row) {
        const float* x_row = x + row * in_features;
        for (size_t o = 0; o < out_features; ++o) {
            float sum = 0.0f;
            size_t base = o * in_features;
            for (size_t i = 0; i < in_features; ++i) {
                float sign = bit_is_plus(bits, base + i) ? 1.0f : -1.0f;
                sum += sign * x_row[i];
            }
            float bias = bias_bits ? uo_fp16_to_f32(bias_bits[o]) : 0.0f;
            y[row * out_features + o] = bias + uo_fp16_to_f32(scale_bits[o]) * sum;
        }
    }
    return 0;
}

/* Same arithmetic as uo_binary_linear_scalar, arranged so the compiler can
 * vectorise ACROSS outputs: each output's partial sum still receives
 * (+/-1)*x[i] for i = 0..K-1 in ascending order, so every result is bit
 * identical to the literal loop (the product by +/-1 is exact). */
UO_API int uo_binary_linear(const float* x, const uint32_t* bits, const uint16_t* scale_bits,
                            const uint16_t* bias_bits, float* y, size_t rows, size_t in_features,
                            size_t out_features) {
    const size_t K = in_features, N = out_features;
    if (K == 0 || N == 0) return 1;
    float* st = (float*)malloc(K * N * sizeof(float)); /* signs transposed [K][N] */
    for (size_t o = 0; o < N; ++o)
        for (size_t i = 0; i < K; ++i) st[i * N + o] = bit_is_plus(bits, o * K + i) ? 1.0f : -1.0f;
    float* scale = widen(scale_bits, N);
    float* bias = bias_bits ? widen(bias_bits, N) : NULL;
    enum { RB = 4, OB = 32 };
    long row_blocks = (long)((rows + RB - 1) / RB);
#pragma omp parallel for num_threads(g_threads) schedule(static)
    for (long rb = 0; rb < row_blocks; ++rb) {
        size_t r0 = (size_t)rb * RB;
        size_t nr = rows - r0 < RB ? rows - r0 : RB;
        for (size_t o0 = 0; o0 < N; o0 += OB) {
            size_t no = N - o0 < OB ? N - o0 : OB;
            float acc[RB][OB];
            for (size_t r = 0; r < RB; ++r)
                for (size_t o = 0; o < OB; ++o) acc[r][o] = 0.0f;
            if (no == OB && nr == RB) {
                for (size_t i = 0; i < K; ++i) {
                    const float* s = st + i * N + o0;
                    for (size_t r = 0; r < RB; ++r) {
                        float xv = x[(r0 + r) * K + i];
                        for (size_t o = 0; o < OB; ++o) acc[r][o] += s[o] * xv;
                    }
                }
            } else {
                for (size_t i = 0; i < K; ++i) {
                    const float* s = st + i * N + o0;
                    for (size_t r = 0; r < nr; ++r) {
                        float xv = x[(r0 + r) * K + i];
                        for (size_t o = 0; o < no; ++o) acc[r][o] += s[o] * xv;
                    }
                }
            }
            for (size_t r = 0; r < nr; ++r)
                for (size_t o = 0; o < no; ++o) {
                    float b = bias ? bias[o0 + o] : 0.0f;
                    y[(r0 + r) * N + o0 + o] = b + scale[o0 + o] * acc[r][o];
                }
        }
    }
    free(st);
    free(scale);
    free(bias);
    return 0;
}

/* ----------------------------------------------------------- fp16 linear */

/* src/model.rs:419-436  Fp16Linear::forward: y[r,o] = sum_i W[o,i]*x[r,i],
 * i ascending, product then add (no fused multiply-add), no bias. */
UO_API int uo_fp16_linear_scalar(const float* x, const uint16_t* w_bits, float* y, size_t rows,
                                 size_t in_features, size_t out_features) {
    for (size_t row = 0; row < rows; ++row) {
        const float* x_row = x + row * in_features;
        for (size_t o = 0; o < out_features; ++o) {
            float sum = 0.0f;
            size_t w_row = o * in_features;
            for (size_t i = 0; i < in_features; ++i) sum += uo_fp16_to_f32(w_bits[w_row + i]) * x_row[i];
            y[row * out_features + o] = sum;
        }
    }
    return 0;
}

/* Order-preserving vectorisable form of uo_fp16_linear_scalar. */
UO_API int uo_fp16_linear(const float* x, const uint16_t* w_bits, float* y, size_t rows, size_t in_features,
                          size_t out_features) {
    const size_t K = in_features, N = out_features;
    if (K == 0 || N == 0) return 1;
    float* wt = (float*)malloc(K * N * sizeof(float)); /* W transposed [K][N] */
    for (size_t o = 0; o < N; ++o)
        for (size_t i = 0; i < K; ++i) wt[i * N + o] = uo_fp16_to_f32(w_bits[o * K + i]);
    enum { RB = 4, OB = 32 };
    long row_blocks = (long)((rows + RB - 1) / RB);
#pragma omp parallel for num_threads(g_threads) schedule(static)
    for (long rb = 0; rb < row_blocks; ++rb) {
        size_t r0 = (size_t)rb * RB;
        size_t nr = rows - r0 < RB ? rows - r0 : RB;
        for (size_t o0 = 0; o0 < N; o0 += OB) {
            size_t no = N - o0 < OB ? N - o0 : OB;
            float acc[RB][OB];
            for (size_t r = 0; r < RB; ++r)
                for (size_t o = 0; o < OB; ++o) acc[r][o] = 0.0f;
            for (size_t i = 0; i < K; ++i) {
                const float* w = wt + i * N + o0;
                for (size_t r = 0; r < nr; ++r) {
                    float xv = x[(r0 + r) * K + i];
                    for (size_t o = 0; o < no; ++o) {
                        float prod = w[o] * xv;
                        acc[r][o] += prod;
                    }
                }
            }
            for (size_t r = 0; r < nr; ++r)
                for (size_t o = 0; o < no; ++o) y[(r0 + r) * N + o0 + o] = acc[r][o];
        }
    }
    free(wt);
    return 0;
}

/* ------------------------------------------------------------- bit plane */

/* src/rosa.rs:372-374  bit_from_activation: value > 0.0 (0.0, -0.0, NaN -> 0);
 * src/rosa.rs:400-411  pack_bitplane: 32 per word, LSB = lowest index. */
UO_API void uo_bits_from_activation(const float* x, uint8_t* bits, size_t n) {
    for (size_t i = 0; i < n; ++i) bits[i] = (uint8_t)(x[i] > 0.0f);
}
UO_API void uo_pack_bitplane(const uint8_t* bits, uint32_t* words, size_t n) {
    size_t nw = (n + 31) / 32;
    for (size_t w = 0; w < nw; ++w) words[w] = 0;
    for (size_t i = 0; i < n; ++i)
        if (bits[i]) words[i / 32] |= 1u << (i % 32);
}
UO_API void uo_sign_pack_bits(const float* x, uint32_t* words, size_t n) {
    size_t nw = (n + 31) / 32;
    for (size_t w = 0; w < nw; ++w) words[w] = 0;
    for (size_t i = 0; i < n; ++i)
        if (x[i] > 0.0f) words[i / 32] |= 1u << (i % 32);
}

/* ------------------------------------------------------------------- SAM */

/* src/rosa.rs:28-43  SamNode */
typedef struct {
    int32_t trans[2];
    int32_t fail;
    int32_t maxlen;
    int32_t last;
} SamNode;

/* src/rosa.rs:15-26  RosaSam */
typedef struct {
    SamNode* nodes;
    size_t n_nodes;
    uint8_t* v_hist;
    size_t v_len, v_cap;
    int32_t u, g, w, h, i;
    uint64_t walk_steps; /* instrumentation only: iterations of the last-propagation loop */
} UoSam;

static const SamNode SAM_EMPTY = {{-1, -1}, -1, 0, -1};

static void sam_grow_to(UoSam* s, size_t len) { /* src/rosa.rs:92-97 */
    if (len <= s->n_nodes) return;
    s->nodes = (SamNode*)realloc(s->nodes, len * sizeof(SamNode));
    for (size_t k = s->n_nodes; k < len; ++k) s->nodes[k] = SAM_EMPTY;
    s->n_nodes = len;
}

/* src/rosa.rs:47-58  with_max_time: 2*T+1 nodes (rosa.rs:377-379) */
UO_API UoSam* uo_sam_new(size_t max_time) {
    UoSam* s = (UoSam*)calloc(1, sizeof(UoSam));
    size_t nodes = 2 * max_time + 1;
    s->nodes = (SamNode*)malloc(nodes * sizeof(SamNode));
    s->n_nodes = nodes;
    for (size_t k = 0; k < nodes; ++k) s->nodes[k] = SAM_EMPTY;
    s->v_cap = max_time ? max_time : 1;
    s->v_hist = (uint8_t*)malloc(s->v_cap);
    s->v_len = 0;
    s->u = 1;
    s->g = s->w = s->h = s->i = 0;
    return s;
}

/* src/rosa.rs:66-74  reset */
UO_API void uo_sam_reset(UoSam* s) {
    for (size_t k = 0; k < s->n_nodes; ++k) s->nodes[k] = SAM_EMPTY;
    s->v_len = 0;
    s->u = 1;
    s->g = s->w = s->h = s->i = 0;
    s->walk_steps = 0;
}

UO_API void uo_sam_free(UoSam* s) {
    if (!s) return;
    free(s->nodes);
    free(s->v_hist);
    free(s);
}

UO_API uint64_t uo_sam_walk_steps(const UoSam* s) { return s->walk_steps; }

static inline int32_t sam_child(const UoSam* s, int32_t p, uint8_t bit) { /* src/rosa.rs:76-82 */
    if (p < 0) return -1;
    return s->nodes[p].trans[bit];
}

/* src/rosa.rs:100-176  RosaSam::push — one step of rosa_qkv_ref, transcribed
 * statement by statement: record v; query with q from the saved state (w,h);
 * normalise to the state whose length range holds x; skip root / never-seen
 * states; read v_hist[last+1]; save (w,h); extend the automaton with k
 * (standard suffix-automaton extend, the clone copies every field including
 * `last`); stamp `last = i` along the suffix-link chain of the new state. */
UO_API uint8_t uo_sam_push(UoSam* s, uint8_t q_bit, uint8_t k_bit, uint8_t v_bit) {
    if (s->v_len == s->v_cap) {
        s->v_cap *= 2;
        s->v_hist = (uint8_t*)realloc(s->v_hist, s->v_cap);
    }
    s->v_hist[s->v_len++] = v_bit;
    int32_t i = s->i;
    int32_t p = s->w;
    int32_t x = s->h;
    while (p != -1 && sam_child(s, p, q_bit) < 0) {
        int32_t mp = s->nodes[p].maxlen;
        if (x > mp) x = mp;
        p = s->nodes[p].fail;
    }
    if (p == -1) {
        p = 0;
        x = 0;
    } else {
        p = sam_child(s, p, q_bit);
        x += 1;
    }
    int32_t v = p;
    while (s->nodes[v].fail != -1 && s->nodes[s->nodes[v].fail].maxlen >= x) v = s->nodes[v].fail;
    while (v != -1 && (s->nodes[v].maxlen <= 0 || s->nodes[v].last < 0)) v = s->nodes[v].fail;
    int32_t y;
    if (v == -1) {
        y = -1;
    } else {
        size_t pos = (size_t)(s->nodes[v].last + 1);
        y = (int32_t)s->v_hist[pos];
    }
    uint8_t idx = (uint8_t)(y > 0 ? y : 0);
    s->w = p;
    s->h = x;

    int32_t j = s->u;
    s->u += 1;
    sam_grow_to(s, (size_t)s->u + 2);
    s->nodes[j].maxlen = s->nodes[s->g].maxlen + 1;
    p = s->g;
    while (p != -1 && sam_child(s, p, k_bit) < 0) {
        s->nodes[p].trans[k_bit] = j;
        p = s->nodes[p].fail;
    }
    if (p == -1) {
        s->nodes[j].fail = 0;
    } else {
        int32_t d = sam_child(s, p, k_bit);
        if (s->nodes[p].maxlen + 1 == s->nodes[d].maxlen) {
            s->nodes[j].fail = d;
        } else {
            int32_t b = s->u;
            s->u += 1;
            sam_grow_to(s, (size_t)s->u);
            s->nodes[b] = s->nodes[d];
            s->nodes[b].maxlen = s->nodes[p].maxlen + 1;
            s->nodes[d].fail = b;
            s->nodes[j].fail = b;
            while (p != -1 && sam_child(s, p, k_bit) == d) {
                s->nodes[p].trans[k_bit] = b;
                p = s->nodes[p].fail;
            }
        }
    }
    v = j;
    s->g = j;
    while (v != -1 && s->nodes[v].last < i) {
        s->nodes[v].last = i;
        v = s->nodes[v].fail;
        s->walk_steps += 1;
    }
    s->i += 1;
    return idx;
}

/* src/rosa.rs:180-193  rosa_qkv_ref; returns non-zero on a bit > 1. */
UO_API int uo_rosa_qkv_ref(const uint8_t* q, const uint8_t* k, const uint8_t* v, size_t n, uint8_t* idx) {
    for (size_t t = 0; t < n; ++t)
        if (q[t] > 1 || k[t] > 1 || v[t] > 1) return 1;
    UoSam* s = uo_sam_new(n);
    for (size_t t = 0; t < n; ++t) idx[t] = uo_sam_push(s, q[t], k[t], v[t]);
    uo_sam_free(s);
    return 0;
}

/* src/rosa.rs:204-285  rosa(): the distinct single-stream routine; raw y with
 * -1 for "unmatched".  Only used to pin the T=5,C=3 fixture. */
UO_API int uo_rosa(const uint8_t* bits, size_t n, int32_t* y) {
    for (size_t t = 0; t < n; ++t)
        if (bits[t] > 1) return 1;
    size_t nodes = 2 * n + 1;
    int32_t* trans0 = (int32_t*)malloc(nodes * 4);
    int32_t* trans1 = (int32_t*)malloc(nodes * 4);
    int32_t* fail = (int32_t*)malloc(nodes * 4);
    int32_t* maxlen = (int32_t*)malloc(nodes * 4);
    int32_t* last = (int32_t*)malloc(nodes * 4);
    for (size_t k = 0; k < nodes; ++k) {
        trans0[k] = trans1[k] = fail[k] = last[k] = -1;
        maxlen[k] = 0;
    }
#define CHILD(p, bit) ((p) < 0 ? -1 : ((bit) == 0 ? trans0[(p)] : trans1[(p)]))
    int32_t g = 0, z = 1;
    for (size_t i = 0; i < n; ++i) {
        uint8_t token = bits[i];
        y[i] = -1;
        int32_t r = z++;
        maxlen[r] = maxlen[g] + 1;
        int32_t p = g;
        while (p != -1 && CHILD(p, token) < 0) {
            if (token == 0) trans0[p] = r; else trans1[p] = r;
            p = fail[p];
        }
        if (p == -1) {
            fail[r] = 0;
        } else {
            int32_t q = CHILD(p, token);
            if (maxlen[p] + 1 == maxlen[q]) {
                fail[r] = q;
            } else {
                int32_t u = z++;
                trans0[u] = trans0[q];
                trans1[u] = trans1[q];
                maxlen[u] = maxlen[p] + 1;
                fail[u] = fail[q];
                last[u] = last[q];
                while (p != -1 && CHILD(p, token) == q) {
                    if (token == 0) trans0[p] = u; else trans1[p] = u;
                    p = fail[p];
                }
                fail[q] = u;
                fail[r] = u;
            }
        }
        g = r;
        int32_t v = g, a = -1;
        while (v != -1) {
            if (maxlen[v] > 0 && last[v] >= 0) {
                a = (int32_t)bits[last[v] + 1];
                break;
            }
            v = fail[v];
        }
        y[i] = a;
        v = g;
        int32_t time = (int32_t)i;
        while (v != -1 && last[v] < time) {
            last[v] = time;
            v = fail[v];
        }
    }
#undef CHILD
    free(trans0); free(trans1); free(fail); free(maxlen); free(last);
    return 0;
}

static inline uint8_t packed_bit_at(const uint32_t* words, size_t index) { /* src/rosa.rs:413-415 */
    return (uint8_t)((words[index / 32] >> (index % 32)) & 1u);
}

/* src/rosa.rs:459-481 (+540-582)  rosa_qkv_batch_packed: q/k/v are LSB-packed
 * bit planes over the flat [B,T,C] index; idx comes back row-major [B,T,C].
 * One fresh automaton per (b,c) stream.  walk_total (nullable) receives the
 * summed last-propagation iterations (instrumentation). */
UO_API int uo_rosa_qkv_batch_packed(const uint32_t* q_bits, const uint32_t* k_bits, const uint32_t* v_bits,
                                    size_t batch, size_t time, size_t channels, uint8_t* idx,
                                    uint64_t* walk_total) {
    if (batch == 0 || time == 0 || channels == 0) return 1;
    long jobs = (long)(batch * channels);
    uint64_t walks = 0;
#pragma omp parallel num_threads(g_threads) reduction(+ : walks)
    {
        UoSam* s = uo_sam_new(time);
#pragma omp for schedule(dynamic, 8)
        for (long job = 0; job < jobs; ++job) {
            size_t b = (size_t)job / channels, c = (size_t)job % channels;
            uo_sam_reset(s);
            for (size_t t = 0; t < time; ++t) {
                size_t index = (b * time + t) * channels + c;
                idx[index] = uo_sam_push(s, packed_bit_at(q_bits, index), packed_bit_at(k_bits, index),
                                         packed_bit_at(v_bits, index));
            }
            walks += s->walk_steps;
        }
        uo_sam_free(s);
    }
    if (walk_total) *walk_total = walks;
    return 0;
}

/* Unpacked form, src/rosa.rs:429-456 rosa_qkv_batch. */
UO_API int uo_rosa_qkv_batch(const uint8_t* q, const uint8_t* k, const uint8_t* v, size_t batch, size_t time,
                             size_t channels, uint8_t* idx) {
    if (batch == 0 || time == 0 || channels == 0) return 1;
    size_t n = batch * time * channels;
    for (size_t i = 0; i < n; ++i)
        if (q[i] > 1 || k[i] > 1 || v[i] > 1) return 1;
    long jobs = (long)(batch * channels);
#pragma omp parallel num_threads(g_threads)
    {
        UoSam* s = uo_sam_new(time);
#pragma omp for schedule(dynamic, 8)
        for (long job = 0; job < jobs; ++job) {
            size_t b = (size_t)job / channels, c = (size_t)job % channels;
            uo_sam_reset(s);
            for (size_t t = 0; t < time; ++t) {
                size_t index = (b * time + t) * channels + c;
                idx[index] = uo_sam_push(s, q[index], k[index], v[index]);
            }
        }
        uo_sam_free(s);
    }
    return 0;
}

/* Stream-major driver: stream s owns words [s*wps, (s+1)*wps) of each plane,
 * bit t at word t/32, bit t%32; idx bits are written in the same layout.
 * Each stream is T pushes of a fresh automaton (src/rosa.rs:180-193). */
UO_API int uo_rosa_qkv_streams(const uint32_t* qw, const uint32_t* kw, const uint32_t* vw, size_t n_streams,
                               size_t time, size_t wps, uint32_t* out, uint64_t* walk_total) {
    uint64_t walks = 0;
#pragma omp parallel num_threads(g_threads) reduction(+ : walks)
    {
        UoSam* s = uo_sam_new(time);
#pragma omp for schedule(dynamic, 8)
        for (long job = 0; job < (long)n_streams; ++job) {
            const uint32_t *q = qw + (size_t)job * wps, *k = kw + (size_t)job * wps, *v = vw + (size_t)job * wps;
            uint32_t* o = out + (size_t)job * wps;
            uo_sam_reset(s);
            for (size_t w = 0; w < wps; ++w) o[w] = 0;
            for (size_t t = 0; t < time; ++t) {
                uint8_t id = uo_sam_push(s, packed_bit_at(q, t), packed_bit_at(k, t), packed_bit_at(v, t));
                o[t / 32] |= (uint32_t)id << (t % 32);
            }
            walks += s->walk_steps;
        }
        uo_sam_free(s);
    }
    if (walk_total) *walk_total = walks;
    return 0;
}

/* src/rosa.rs:585-609  rosa_qkv_out_batched: out = (2*idx-1)*e[c], e given as
 * FP16 bits and widened (model.rs:1313 uses self.e.get(c)). */
UO_API void uo_rosa_qkv_out_batched(const uint8_t* idx, const uint16_t* e_bits, float* out, size_t batch,
                                    size_t time, size_t channels) {
    float* e = widen(e_bits, channels);
    for (size_t r = 0; r < batch * time; ++r)
        for (size_t c = 0; c < channels; ++c) {
            size_t index = r * channels + c;
            out[index] = (2.0f * (float)idx[index] - 1.0f) * e[c];
        }
    free(e);
}

/* ------------------------------------------------------------ ROSA block */

/* src/model.rs:1284-1318  RwkvRosaQkv1Bit::forward.  Optional taps (any may
 * be NULL): q/k/v pre-activations [rows,C], their bits [rows,C] (u8), idx
 * [rows,C] (u8), y = (2*idx-1)*e [rows,C]. */
UO_API int uo_rosa_block_forward(const float* x, const uint16_t* mix_q, const uint16_t* mix_k,
                                 const uint16_t* mix_v, const uint32_t* q_bits, const uint16_t* q_scale,
                                 const uint16_t* q_bias, const uint32_t* k_bits, const uint16_t* k_scale,
                                 const uint16_t* k_bias, const uint32_t* v_bits, const uint16_t* v_scale,
                                 const uint16_t* v_bias, const uint16_t* e_bits, const uint32_t* o_bits,
                                 const uint16_t* o_scale, const uint16_t* o_bias, size_t batch, size_t time,
                                 size_t channels, float* tap_q, float* tap_k, float* tap_v, uint8_t* tap_qb,
                                 uint8_t* tap_kb, uint8_t* tap_vb, uint8_t* tap_idx, float* tap_y, float* out,
                                 uint64_t* walk_total) {
    size_t d = channels, rows = batch * time, n = rows * d;
    float* xx = (float*)malloc(n * 4);
    float* in = (float*)malloc(n * 4);
    float* q = (float*)malloc(n * 4);
    float* k = (float*)malloc(n * 4);
    float* v = (float*)malloc(n * 4);
    float* y = (float*)malloc(n * 4);
    uint8_t* idx = (uint8_t*)malloc(n);
    uo_time_shift_delta(x, xx, batch, time, d);
    uo_shift_mix(x, xx, mix_q, in, rows, d);
    uo_binary_linear(in, q_bits, q_scale, q_bias, q, rows, d, d);
    uo_shift_mix(x, xx, mix_k, in, rows, d);
    uo_binary_linear(in, k_bits, k_scale, k_bias, k, rows, d, d);
    uo_shift_mix(x, xx, mix_v, in, rows, d);
    uo_binary_linear(in, v_bits, v_scale, v_bias, v, rows, d, d);
    float* e = widen(e_bits, d);
    long jobs = (long)(batch * d);
    uint64_t walks = 0;
#pragma omp parallel num_threads(g_threads) reduction(+ : walks)
    {
        UoSam* s = uo_sam_new(time);
#pragma omp for schedule(dynamic, 8)
        for (long job = 0; job < jobs; ++job) {
            size_t b = (size_t)job / d, c = (size_t)job % d;
            uo_sam_reset(s);
            for (size_t t = 0; t < time; ++t) {
                size_t index = (b * time + t) * d + c;
                uint8_t id = uo_sam_push(s, (uint8_t)(q[index] > 0.0f), (uint8_t)(k[index] > 0.0f),
                                         (uint8_t)(v[index] > 0.0f));
                idx[index] = id;
                y[index] = (2.0f * (float)id - 1.0f) * e[c];
            }
            walks += s->walk_steps;
        }
        uo_sam_free(s);
    }
    if (walk_total) *walk_total = walks;
    uo_binary_linear(y, o_bits, o_scale, o_bias, out, rows, d, d);
    if (tap_q) memcpy(tap_q, q, n * 4);
    if (tap_k) memcpy(tap_k, k, n * 4);
    if (tap_v) memcpy(tap_v, v, n * 4);
    if (tap_qb) uo_bits_from_activation(q, tap_qb, n);
    if (tap_kb) uo_bits_from_activation(k, tap_kb, n);
    if (tap_vb) uo_bits_from_activation(v, tap_vb, n);
    if (tap_idx) memcpy(tap_idx, idx, n);
    if (tap_y) memcpy(tap_y, y, n * 4);
    free(xx); free(in); free(q); free(k); free(v); free(y); free(idx); free(e);
    return 0;
}

/* ------------------------------------------------------------------ CMix */

/* src/model.rs:987-1001  RwkvCMixX070::forward: shift-mix with x_k, packed
 * key (no bias), relu(v)^2 written as max(v,0)*max(v,0), dense FP16 value.
 * tap_relu2 (nullable) receives the [rows,F] hidden activations. */
UO_API int uo_cmix_forward(const float* x, const uint16_t* mix, const uint32_t* key_bits,
                           const uint16_t* key_scale, const uint16_t* value_bits, size_t batch, size_t time,
                           size_t d_model, size_t dim_ffn, float* tap_relu2, float* out) {
    size_t rows = batch * time;
    float* xx = (float*)malloc(rows * d_model * 4);
    float* shifted = (float*)malloc(rows * d_model * 4);
    float* key = (float*)malloc(rows * dim_ffn * 4);
    uo_time_shift_delta(x, xx, batch, time, d_model);
    uo_shift_mix(x, xx, mix, shifted, rows, d_model);
    uo_binary_linear(shifted, key_bits, key_scale, NULL, key, rows, d_model, dim_ffn);
    for (size_t i = 0; i < rows * dim_ffn; ++i) {
        float m = fmaxf(key[i], 0.0f);
        key[i] = m * m;
    }
    if (tap_relu2) memcpy(tap_relu2, key, rows * dim_ffn * 4);
    uo_fp16_linear(key, value_bits, out, rows, dim_ffn, d_model);
    free(xx); free(shifted); free(key);
    return 0;
}

/* ----------------------------------------------------------------- embed */

/* src/model.rs:2660-2669  embedding gather; returns 2 on id >= vocab. */
UO_API int uo_embed(const uint32_t* ids, const uint16_t* embedding, float* x, size_t rows, size_t d_model,
                    size_t vocab) {
    for (size_t row = 0; row < rows; ++row) {
        if ((size_t)ids[row] >= vocab) return 2;
        size_t offset = (size_t)ids[row] * d_model;
        for (size_t c = 0; c < d_model; ++c) x[row * d_model + c] = uo_fp16_to_f32(embedding[offset + c]);
    }
    return 0;
}

/* -------------------------------------------------------------------- CE */

/* src/model.rs:27-39  causal_ce_row_valid with horizon 1. */
static int ce_row_valid(size_t row, size_t time, const uint32_t* targets, size_t n_targets, uint32_t ignore_id) {
    if (time == 0 || row % time + 1 >= time) return 0;
    size_t target_row = row + 1;
    return target_row < n_targets && targets[target_row] != ignore_id;
}

/* src/model.rs:3144-3149 (count), 3212-3228 (per-row CE), 3253-3257 (mean):
 * per valid row logits = head.forward(h,1); max; exps summed sequentially;
 * ce = max + ln(sum) - logits[target]; f32 running loss_sum;
 * mean = loss_sum / n_valid (0 when nothing is valid).  row_loss is 0 on
 * invalid rows.  logits_out (nullable, [rows,V]) receives every row's logits
 * (src/model.rs:2685-2688). */
UO_API int uo_head_ce(const float* hidden, const uint32_t* head_bits, const uint16_t* head_scale,
                      const uint16_t* head_bias, const uint32_t* targets, uint32_t ignore_id, size_t rows,
                      size_t time, size_t d_model, size_t vocab, float* row_loss, float* mean_loss,
                      uint64_t* n_valid_out, float* logits_out) {
    float* logits = logits_out ? logits_out : (float*)malloc(rows * vocab * 4);
    uo_binary_linear(hidden, head_bits, head_scale, head_bias, logits, rows, d_model, vocab);
    uint64_t n_valid = 0;
    float loss_sum = 0.0f;
    for (size_t row = 0; row < rows; ++row) {
        row_loss[row] = 0.0f;
        if (!ce_row_valid(row, time, targets, rows, ignore_id)) continue;
        n_valid += 1;
        size_t target = targets[row + 1];
        if (target >= vocab) {
            if (!logits_out) free(logits);
            return 2;
        }
        const float* l = logits + row * vocab;
        float max = -INFINITY;
        for (size_t v = 0; v < vocab; ++v) max = fmaxf(max, l[v]);
        float exp_sum = 0.0f;
        for (size_t v = 0; v < vocab; ++v) exp_sum += expf(l[v] - max);
        float ce = max + logf(exp_sum) - l[target];
        row_loss[row] = ce;
        loss_sum += ce;
    }
    *mean_loss = n_valid == 0 ? 0.0f : loss_sum / (float)n_valid;
    *n_valid_out = n_valid;
    if (!logits_out) free(logits);
    return 0;
}

UO_API void uo_add_inplace(float* dst, const float* src, size_t n) { /* src/model.rs:2232-2234 */
    for (size_t i = 0; i < n; ++i) dst[i] += src[i];
}
