// One training step on the device, rosa_grad = stop_grad_bits: the tensor-core
// forward keeps a small tape (the residual stream after each ROSA block and
// the idx bits), the backward recomputes the CMix activations from it and
// runs every gradient matrix product as an FP16 x FP16 -> f32 tcgen05 GEMM on
// operands that small kernels cast / transpose, and the optimiser kernels
// apply the reference's clipped SGD and BinaryConnect steps element by element.
//
// Reference: train_step_on (src/model.rs:2827-3020), apply_head_ce
// (3132-3275), backward_ste (745-796), flip_after_gradients (838-876),
// CMix backward_update (1138-1177), backward_stop_grad (1494-1521),
// rosa_e_grad (1608-1634), LayerNorm::backward (270-315),
// Fp16Storage::apply_clipped_sgd / apply_binaryconnect_sgd (src/precision.rs:106-134).
//
// Gradients travel multiplied by P = 2^ceil(log2(T-1)): the loss scale is
// 1/(T-1), so P*g is O(1) where the 16-bit GEMM operands are formed, and the
// optimiser kernels multiply by 1/P (exact) before they clip.
#include "train.hpp"

#include <cuda_fp16.h>

#include <algorithm>
#include <cmath>
#include <cstring>

#include "kernels.hpp"
#include "linear_tc.hpp"
#include "safetensors.hpp"

using namespace ullis;

namespace {

constexpr float LN_EPS = 1e-5f;              // src/model.rs:22
constexpr float HEAD_BIAS_LR_MULT = 8.0f;    // src/model.rs:97
constexpr uint16_t LATENT_PLUS = 0x211F;     // FP16(0.01), BINARYCONNECT_INIT_ABS (src/model.rs:550)

__device__ __forceinline__ float h2f(uint16_t b) { return __half2float(__ushort_as_half(b)); }

// f32 -> FP16 bits; a finite value beyond the FP16 range is reported, not turned into inf
__device__ __forceinline__ uint16_t to_f16(float v, uint32_t* status, size_t row) {
    const float a = fabsf(v);
    if (a > 65504.0f && a <= 3.4028234e38f) {
        if (atomicCAS(status, ULLIS_DEV_OK, ULLIS_DEV_FP16_RANGE) == ULLIS_DEV_OK) status[1] = (uint32_t)row;
        v = copysignf(65504.0f, v);
    }
    return __half_as_ushort(__float2half_rn(v));
}

inline unsigned blocks_for(size_t n, unsigned per) { return (unsigned)((n + per - 1) / per); }
inline size_t pad64(size_t n) { return (n + 63) / 64 * 64; }

// ------------------------------------------------------------ GEMM operands
// the same for C == Cp, C % 4 == 0: four elements per thread
__global__ void cast_rows4_kernel(const float* __restrict__ x, const uint16_t* __restrict__ colscale,
                                  uint16_t* __restrict__ out, size_t R, size_t C, uint32_t* status) {
    const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= R * C) return;
    const size_t r = i / C, c = i % C;
    const float4 v = *reinterpret_cast<const float4*>(x + i);
    float f[4] = {v.x, v.y, v.z, v.w};
    if (colscale) {
        const uint2 sw = *reinterpret_cast<const uint2*>(colscale + c);
        f[0] = __fmul_rn(f[0], h2f((uint16_t)(sw.x & 0xFFFFu)));
        f[1] = __fmul_rn(f[1], h2f((uint16_t)(sw.x >> 16)));
        f[2] = __fmul_rn(f[2], h2f((uint16_t)(sw.y & 0xFFFFu)));
        f[3] = __fmul_rn(f[3], h2f((uint16_t)(sw.y >> 16)));
    }
    const uint32_t lo = to_f16(f[0], status, r) | ((uint32_t)to_f16(f[1], status, r) << 16);
    const uint32_t hi = to_f16(f[2], status, r) | ((uint32_t)to_f16(f[3], status, r) << 16);
    *reinterpret_cast<uint2*>(out + i) = make_uint2(lo, hi);
}

// out [R, Cp] = FP16(x [R, C] * colscale[c]), columns C..Cp zero
__global__ void cast_rows_kernel(const float* __restrict__ x, const uint16_t* __restrict__ colscale,
                                 uint16_t* __restrict__ out, size_t R, size_t C, size_t Cp, uint32_t* status) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= R * Cp) return;
    const size_t r = i / Cp, c = i % Cp;
    float v = 0.0f;
    if (c < C) {
        v = x[r * C + c];
        if (colscale) v = __fmul_rn(v, h2f(colscale[c]));
    }
    out[i] = to_f16(v, status, r);
}

// out [C, Rp] = FP16(op(x [R, C]))^T, columns R..Rp zero (Rp % 64 == 0).  op 1: relu(x)^2
// A CTA moves 64 rows x 64 columns: 16-byte loads along a row, 16-byte stores of eight consecutive
// rows of one column.
__global__ void __launch_bounds__(256)
transpose_cast_kernel(const float* __restrict__ x, uint16_t* __restrict__ out, size_t R, size_t C, size_t Rp, int op,
                      uint32_t* status) {
    __shared__ float tile[64][65];
    const size_t r0 = (size_t)blockIdx.x * 64, c0 = (size_t)blockIdx.y * 64;
    const bool vec = (C & 3) == 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int slot = threadIdx.x + k * 256;      // 64 rows x 16 groups of four columns
        const int j = slot >> 4, q = (slot & 15) * 4;
        const size_t r = r0 + j, c = c0 + q;
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        if (r < R) {
            if (vec && c + 3 < C) {
                const float4 t = *reinterpret_cast<const float4*>(x + r * C + c);
                v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
            } else {
                for (int e = 0; e < 4; ++e) if (c + e < C) v[e] = x[r * C + c + e];
            }
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            float t = v[e];
            if (op == 1) { t = fmaxf(t, 0.0f); t *= t; }
            tile[j][q + e] = t;
        }
    }
    __syncthreads();
    const int cl = threadIdx.x >> 2, seg = (threadIdx.x & 3) * 16;   // column, first of its sixteen rows
    const size_t c = c0 + cl;
    if (c >= C) return;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        uint32_t w[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int j = seg + h * 8 + e * 2;
            w[e] = (uint32_t)to_f16(tile[j][cl], status, r0 + j) | ((uint32_t)to_f16(tile[j + 1][cl], status, r0 + j + 1) << 16);
        }
        // r0 + seg + 8h + 7 < Rp: Rp is a multiple of 64
        *reinterpret_cast<uint4*>(out + c * Rp + r0 + seg + h * 8) = make_uint4(w[0], w[1], w[2], w[3]);
    }
}

// packed signs [out, in] -> FP16 +/-1 [in, outp], columns out..outp zero
__global__ void unpack_transpose_kernel(const uint32_t* __restrict__ bits, uint16_t* __restrict__ b16, size_t out_f,
                                        size_t in_f, size_t outp) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= in_f * outp) return;
    const size_t k = i / outp, o = i % outp;
    uint16_t v = 0;
    if (o < out_f) {
        const size_t bit = o * in_f + k;
        v = (bits[bit >> 5] >> (bit & 31)) & 1u ? 0x3C00 : 0xBC00;
    }
    b16[i] = v;
}

// w [R, C] FP16 -> [C, Rp], columns R..Rp zero
__global__ void transpose16_kernel(const uint16_t* __restrict__ w, uint16_t* __restrict__ out, size_t R, size_t C,
                                   size_t Rp) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= C * Rp) return;
    const size_t c = i / Rp, r = i % Rp;
    out[i] = r < R ? w[r * C + c] : (uint16_t)0;
}

// y [M, N] = a [M, K] . b [N, K]^T, f32 accumulation of the same FP16 operands the
// tensor-core kernel takes (shapes outside its tiling, validation mode)
__global__ void gemm_nt_plain_kernel(const uint16_t* __restrict__ a, const uint16_t* __restrict__ b,
                                     float* __restrict__ y, size_t M, size_t K, size_t N) {
    __shared__ float sa[16][17], sb[16][17];
    const size_t m = (size_t)blockIdx.y * 16 + threadIdx.y, n = (size_t)blockIdx.x * 16 + threadIdx.x;
    float acc = 0.0f;
    for (size_t k0 = 0; k0 < K; k0 += 16) {
        const size_t ka = k0 + threadIdx.x;
        sa[threadIdx.y][threadIdx.x] = (m < M && ka < K) ? h2f(a[m * K + ka]) : 0.0f;
        const size_t nb = (size_t)blockIdx.x * 16 + threadIdx.y;
        sb[threadIdx.y][threadIdx.x] = (nb < N && ka < K) ? h2f(b[nb * K + ka]) : 0.0f;
        __syncthreads();
#pragma unroll
        for (int k = 0; k < 16; ++k) acc = fmaf(sa[threadIdx.y][k], sb[threadIdx.x][k], acc);
        __syncthreads();
    }
    if (m < M && n < N) y[m * N + n] = acc;
}

// ------------------------------------------------------------ head
// logits [rows, V] -> row_loss and, in place, gy * P with gy = loss_scale * (softmax - onehot)
// (src/model.rs:3204-3236; valid-row rule 27-39).  One CTA per row.
__global__ void __launch_bounds__(256)
ce_grad_kernel(float* __restrict__ logits, const uint32_t* __restrict__ labels, uint32_t ignore_id, size_t rows,
               size_t time, size_t vocab, float loss_scale, float P, float* __restrict__ row_loss,
               uint32_t* status) {
    __shared__ float red[8];
    __shared__ float bcast;
    const size_t m = blockIdx.x;
    float* lg = logits + m * vocab;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    bool valid = (m % time) + 1 < time && m + 1 < rows && labels[m + 1] != ignore_id;
    const uint32_t target = valid ? labels[m + 1] : 0u;
    if (valid && target >= vocab) {
        if (threadIdx.x == 0 && atomicCAS(status, ULLIS_DEV_OK, ULLIS_DEV_BAD_TOKEN) == ULLIS_DEV_OK)
            status[1] = (uint32_t)m;
        valid = false;
    }
    if (!valid) {
        for (size_t v = threadIdx.x; v < vocab; v += 256) lg[v] = 0.0f;
        if (threadIdx.x == 0) row_loss[m] = 0.0f;
        return;
    }
    float mx = -INFINITY;
    for (size_t v = threadIdx.x; v < vocab; v += 256) mx = fmaxf(mx, lg[v]);
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) red[warp] = mx;
    __syncthreads();
    if (threadIdx.x == 0) {
        float v = red[0];
        for (int w = 1; w < 8; ++w) v = fmaxf(v, red[w]);
        bcast = v;
    }
    __syncthreads();
    mx = bcast;
    float sum = 0.0f;
    for (size_t v = threadIdx.x; v < vocab; v += 256) sum += expf(lg[v] - mx);
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    __syncthreads();
    if (lane == 0) red[warp] = sum;
    __syncthreads();
    if (threadIdx.x == 0) {
        float v = 0.0f;
        for (int w = 0; w < 8; ++w) v += red[w];
        bcast = v;
        row_loss[m] = mx + logf(v) - lg[target];
    }
    __syncthreads();
    sum = bcast;
    for (size_t v = threadIdx.x; v < vocab; v += 256) {
        const float p = expf(lg[v] - mx) / sum;
        lg[v] = loss_scale * (p - (v == target ? 1.0f : 0.0f)) * P;
    }
}

// ------------------------------------------------------------ reductions over rows
// part[chunk, c] = sum over the chunk's 256 rows of f(a, b); mode 0: a, 1: a*b (b f32), 2: a*(2*b-1) (b u8)
__global__ void __launch_bounds__(256)
col_partial_kernel(const float* __restrict__ a, const void* __restrict__ b, float* __restrict__ part, size_t R,
                   size_t C, int mode) {
    const size_t c = (size_t)blockIdx.x * 256 + threadIdx.x;
    if (c >= C) return;
    const size_t r0 = (size_t)blockIdx.y * 256, r1 = min(r0 + 256, R);
    float acc = 0.0f;
    for (size_t r = r0; r < r1; ++r) {
        const float av = a[r * C + c];
        if (mode == 0) acc += av;
        else if (mode == 1) acc += av * static_cast<const float*>(b)[r * C + c];
        else acc += static_cast<const uint8_t*>(b)[r * C + c] ? av : -av;
    }
    part[(size_t)blockIdx.y * C + c] = acc;
}

__global__ void col_final_kernel(const float* __restrict__ part, float* __restrict__ out, size_t chunks, size_t C) {
    const size_t c = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    float acc = 0.0f;
    for (size_t k = 0; k < chunks; ++k) acc += part[k * C + c];
    out[c] = acc;
}

// ------------------------------------------------------------ LayerNorm backward
// gx (+)= d/dx, xhat out (for g_w = sum gy*xhat); one warp per row (src/model.rs:270-315)
__global__ void __launch_bounds__(256)
ln_backward_kernel(const float* __restrict__ x, const float* __restrict__ gy, const uint16_t* __restrict__ w,
                   float* __restrict__ gx, float* __restrict__ xhat_out, size_t rows, size_t C, int accumulate) {
    const int lane = threadIdx.x & 31;
    const size_t row = (size_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= rows) return;
    const float* xr = x + row * C;
    const float* gr = gy + row * C;
    float s = 0.0f;
    for (size_t c = lane; c < C; c += 32) s += xr[c];
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    const float mean = s / (float)C;
    float v = 0.0f;
    for (size_t c = lane; c < C; c += 32) { const float dlt = xr[c] - mean; v += dlt * dlt; }
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const float inv = 1.0f / sqrtf(v / (float)C + LN_EPS);
    float s1 = 0.0f, s2 = 0.0f;
    for (size_t c = lane; c < C; c += 32) {
        const float xh = (xr[c] - mean) * inv, dx = gr[c] * h2f(w[c]);
        s1 += dx;
        s2 += dx * xh;
    }
    for (int o = 16; o > 0; o >>= 1) {
        s1 += __shfl_xor_sync(0xffffffffu, s1, o);
        s2 += __shfl_xor_sync(0xffffffffu, s2, o);
    }
    const float inv_n = inv / (float)C;
    for (size_t c = lane; c < C; c += 32) {
        const float xh = (xr[c] - mean) * inv, dx = gr[c] * h2f(w[c]);
        const float g = inv_n * ((float)C * dx - s1 - xh * s2);
        xhat_out[row * C + c] = xh;
        gx[row * C + c] = accumulate ? gx[row * C + c] + g : g;
    }
}

// ------------------------------------------------------------ CMix pieces
// g <- key > 0 ? 2*key*g : 0   (relu2_bwd_on, src/model.rs:1189-1204)
__global__ void relu2_bwd_kernel(const float* __restrict__ key, float* __restrict__ g, size_t n) {
    const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= n) return;
    if (i + 4 <= n) {
        const float4 k = *reinterpret_cast<const float4*>(key + i);
        float4 v = *reinterpret_cast<const float4*>(g + i);
        v.x = k.x > 0.0f ? 2.0f * k.x * v.x : 0.0f;
        v.y = k.y > 0.0f ? 2.0f * k.y * v.y : 0.0f;
        v.z = k.z > 0.0f ? 2.0f * k.z * v.z : 0.0f;
        v.w = k.w > 0.0f ? 2.0f * k.w * v.w : 0.0f;
        *reinterpret_cast<float4*>(g + i) = v;
        return;
    }
    for (size_t j = i; j < n; ++j) g[j] = key[j] > 0.0f ? 2.0f * key[j] * g[j] : 0.0f;
}

// lerp_shift_backward (src/model.rs:1206-1240): out[t] = (g[t] - g[t]*mix) + g[t+1]*mix
__global__ void lerp_bwd_kernel(const float* __restrict__ g, const uint16_t* __restrict__ mix, float* __restrict__ out,
                                size_t rows, size_t time, size_t C) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * C) return;
    const size_t row = i / C, c = i % C;
    const float mv = h2f(mix[c]);
    float v = __fsub_rn(g[i], __fmul_rn(g[i], mv));
    if (row % time + 1 < time) v = __fadd_rn(v, __fmul_rn(g[i + C], mv));
    out[i] = v;
}

// ------------------------------------------------------------ optimiser
// Fp16Storage::apply_clipped_sgd (src/precision.rs:106-113) on g * gmul
__device__ __forceinline__ void clipped_step(uint16_t& w, float& residual, float g, float lr) {
    const float current = h2f(w);
    const float update = __fmul_rn(lr, fminf(fmaxf(g, -1.0f), 1.0f));
    const float desired = __fadd_rn(__fsub_rn(current, update), residual);
    const uint16_t rounded = __half_as_ushort(__float2half_rn(desired));
    residual = __fsub_rn(desired, h2f(rounded));
    w = rounded;
}

__global__ void clipped_sgd_kernel(uint16_t* __restrict__ w, float* __restrict__ residual, const float* __restrict__ g,
                                   float gmul, float lr, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    uint16_t wb = w[i];
    float r = residual[i];
    clipped_step(wb, r, __fmul_rn(g[i], gmul), lr);
    w[i] = wb;
    residual[i] = r;
}

// Latent step of a packed matrix (apply_binaryconnect_sgd, src/precision.rs:124-134, on
// g_w = scale[o] * G[o,i] * gmul * ste_scale), re-packing of the sign bits (rebinarize,
// src/model.rs:878-884) and the count of bits that changed.  One warp per 32-bit word.
__global__ void __launch_bounds__(256)
latent_sgd_kernel(uint16_t* __restrict__ latent, float* __restrict__ residual, const float* __restrict__ G,
                  const uint16_t* __restrict__ scale, uint32_t* __restrict__ bits, size_t out_f, size_t in_f,
                  float gmul, float ste_scale, float lr, unsigned long long* flips) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t n = out_f * in_f;
    bool plus = false;
    if (i < n) {
        const float g = __fmul_rn(__fmul_rn(__fmul_rn(scale ? h2f(scale[i / in_f]) : 1.0f, G[i]), gmul), ste_scale);
        uint16_t lb = latent[i];
        if (g != 0.0f && fabsf(g) <= 3.4028234e38f) {
            const float current = h2f(lb);
            const float update = __fmul_rn(lr, fminf(fmaxf(g, -1.0f), 1.0f));
            const float desired = fminf(fmaxf(__fadd_rn(__fsub_rn(current, update), residual[i]), -1.0f), 1.0f);
            lb = __half_as_ushort(__float2half_rn(desired));
            residual[i] = __fsub_rn(desired, h2f(lb));
            latent[i] = lb;
        }
        plus = h2f(lb) >= 0.0f;
    }
    const uint32_t word = __ballot_sync(0xffffffffu, plus);
    if (bits && (threadIdx.x & 31) == 0 && i < n) {
        const uint32_t old = bits[i >> 5];
        bits[i >> 5] = word;
        const uint32_t diff = __popc(old ^ word);
        if (diff && flips) atomicAdd(flips, (unsigned long long)diff);
    }
}

// g_scale[o] = sum_i sign[o,i] * G[o,i]   (g_scale of backward_ste, src/model.rs:784-790, with the
// row sum taken first).  One warp per output row.
__global__ void __launch_bounds__(256)
g_scale_kernel(const float* __restrict__ G, const uint32_t* __restrict__ bits, float* __restrict__ out, size_t out_f,
               size_t in_f) {
    const int lane = threadIdx.x & 31;
    const size_t o = (size_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (o >= out_f) return;
    float acc = 0.0f;
    for (size_t i = lane; i < in_f; i += 32) {
        const size_t bit = o * in_f + i;
        const float g = G[bit];
        acc += (bits[bit >> 5] >> (bit & 31)) & 1u ? g : -g;
    }
    for (int k = 16; k > 0; k >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, k);
    if (lane == 0) out[o] = acc;
}

// Embedding rows: one clipped step per ROW in row order (src/model.rs:2980-2987), so a token that
// occurs n times is stepped n times.  A thread per (distinct token, channel).
__global__ void embed_sgd_kernel(uint16_t* __restrict__ emb, float* __restrict__ residual, const float* __restrict__ gx,
                                 const uint32_t* __restrict__ toks, const uint32_t* __restrict__ starts,
                                 const uint32_t* __restrict__ order, size_t d, float gmul, float lr) {
    const uint32_t tok = toks[blockIdx.x], r0 = starts[blockIdx.x], r1 = starts[blockIdx.x + 1];
    const size_t c = (size_t)blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= d) return;
    uint16_t wb = emb[(size_t)tok * d + c];
    float r = residual[(size_t)tok * d + c];
    for (uint32_t k0 = r0; k0 < r1; k0 += 8) {
        float g[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) g[j] = k0 + j < r1 ? gx[(size_t)order[k0 + j] * d + c] : 0.0f;   // loads go out together
#pragma unroll
        for (int j = 0; j < 8; ++j)
            if (k0 + j < r1) clipped_step(wb, r, __fmul_rn(g[j], gmul), lr);                       // steps stay in row order
    }
    emb[(size_t)tok * d + c] = wb;
    residual[(size_t)tok * d + c] = r;
}

__global__ void init_latent_kernel(const uint32_t* __restrict__ bits, uint16_t* __restrict__ latent, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    latent[i] = (bits[i >> 5] >> (i & 31)) & 1u ? LATENT_PLUS : (uint16_t)(LATENT_PLUS | 0x8000u);
}

void col_reduce_launch(ullis_cuda_runtime* rt, const float* a, const void* b, float* out, size_t R, size_t C, int mode,
                       DeviceBuffer& scratch) {
    const size_t chunks = (R + 255) / 256;
    float* part = scratch.as<float>(chunks * C);
    dim3 grid(blocks_for(C, 256), (unsigned)chunks);
    col_partial_kernel<<<grid, 256, 0, rt->stream>>>(a, b, part, R, C, mode);
    rt->launched("col_partial");
    col_final_kernel<<<blocks_for(C, 256), 256, 0, rt->stream>>>(part, out, chunks, C);
    rt->launched("col_final");
}

// ------------------------------------------------------------ host helpers
struct Step {
    ullis_cuda_train_state* st;
    ullis_cuda_runtime* rt;
    float gmul, lr, ste;

    // y [M,N] = a16 [M,K] . b16 [N,K]^T
    void gemm(const uint16_t* a, const uint16_t* b, float* y, size_t M, size_t K, size_t N) {
        if (tc::dense_nt(rt, a, b, y, M, K, N)) return;
        dim3 grid(blocks_for(N, 16), blocks_for(M, 16)), block(16, 16);
        gemm_nt_plain_kernel<<<grid, block, 0, rt->stream>>>(a, b, y, M, K, N);
        rt->launched("gemm_nt_plain");
    }
    void cast_rows(const float* x, const uint16_t* colscale, uint16_t* out, size_t R, size_t C, size_t Cp) {
        if (C == Cp && C % 4 == 0 && (reinterpret_cast<uintptr_t>(colscale) & 7) == 0)
            cast_rows4_kernel<<<blocks_for(R * C / 4, 256), 256, 0, rt->stream>>>(x, colscale, out, R, C, rt->dev_status);
        else
            cast_rows_kernel<<<blocks_for(R * Cp, 256), 256, 0, rt->stream>>>(x, colscale, out, R, C, Cp, rt->dev_status);
        rt->launched("cast_rows");
    }
    void transpose_cast(const float* x, uint16_t* out, size_t R, size_t C, size_t Rp, int op = 0) {
        dim3 grid(blocks_for(Rp, 64), blocks_for(C, 64));
        transpose_cast_kernel<<<grid, 256, 0, rt->stream>>>(x, out, R, C, Rp, op, rt->dev_status);
        rt->launched("transpose_cast");
    }
    void unpack_transpose(const uint32_t* bits, uint16_t* out, size_t out_f, size_t in_f, size_t outp) {
        unpack_transpose_kernel<<<blocks_for(in_f * outp, 256), 256, 0, rt->stream>>>(bits, out, out_f, in_f, outp);
        rt->launched("unpack_transpose");
    }
    // out[c] = sum_r f(a[r,c], b[r,c])
    void col_reduce(const float* a, const void* b, float* out, size_t R, size_t C, int mode) {
        col_reduce_launch(rt, a, b, out, R, C, mode, st->part);
    }
    void sgd(const Fp16Param& p, const float* g, float rate) {
        clipped_sgd_kernel<<<blocks_for(p.n, 256), 256, 0, rt->stream>>>(p.w, p.residual, g, gmul, rate, p.n);
        rt->launched("clipped_sgd");
    }
    // gx_out (+)= LN backward of (x, gy); steps the LayerNorm's weight and bias
    void ln_backward(const float* x, const float* gy, const Fp16Param& w, const Fp16Param& b, float* gx_out,
                     bool accumulate, float* xhat, float* small, size_t rows, size_t d) {
        ln_backward_kernel<<<blocks_for(rows, 8), 256, 0, rt->stream>>>(x, gy, w.w, gx_out, xhat, rows, d,
                                                                       accumulate ? 1 : 0);
        rt->launched("ln_backward");
        col_reduce(gy, xhat, small, rows, d, 1);
        col_reduce(gy, nullptr, small + d, rows, d, 0);
        sgd(w, small, lr);
        sgd(b, small + d, lr);
    }
    // Packed matrix: G = gy^T . x (unscaled by the row scale), then scale / bias / latent steps.
    // gy16t: FP16(gy)^T [out, rows_p]; x16t: FP16(x)^T [in, rows_p].  g_bias (or null) is already reduced.
    void packed_update(PackedParam& p, const uint16_t* gy16t, const uint16_t* x16t, size_t rows_p, const float* g_bias,
                       float bias_lr, unsigned long long* flips, float* small) {
        const size_t out_f = p.weights->out, in_f = p.weights->in;
        float* G = st->gmat.as<float>(out_f * in_f);
        gemm(gy16t, x16t, G, out_f, rows_p, in_f);
        g_scale_kernel<<<blocks_for(out_f, 8), 256, 0, rt->stream>>>(G, p.weights->bits, small, out_f, in_f);
        rt->launched("g_scale");
        latent_sgd_kernel<<<blocks_for((out_f * in_f + 31) / 32 * 32, 256), 256, 0, rt->stream>>>(
            p.latent, p.latent_residual, G, p.scale.w, const_cast<uint32_t*>(p.weights->bits), out_f, in_f, gmul, ste,
            lr, flips);
        rt->launched("latent_sgd");
        sgd(p.scale, small, lr);
        if (p.bias.w && g_bias) sgd(p.bias, g_bias, bias_lr);
    }
};

}  // namespace

// ------------------------------------------------------------ op-level launchers (kernels.hpp)
namespace ullis {
namespace k {

void clipped_sgd(ullis_cuda_runtime* rt, uint16_t* w, float* residual, const float* g, float lr, size_t n) {
    clipped_sgd_kernel<<<blocks_for(n, 256), 256, 0, rt->stream>>>(w, residual, g, 1.0f, lr, n);
    rt->launched("clipped_sgd");
}

void latent_sgd(ullis_cuda_runtime* rt, uint16_t* latent, float* residual, const float* g, float lr, float ste_scale,
                uint32_t* bits, size_t n) {
    latent_sgd_kernel<<<blocks_for((n + 31) / 32 * 32, 256), 256, 0, rt->stream>>>(latent, residual, g, nullptr, bits, 1,
                                                                                  n, 1.0f, ste_scale, lr, nullptr);
    rt->launched("latent_sgd");
}

void rosa_e_grad(ullis_cuda_runtime* rt, const float* gy, const uint8_t* idx, float* g_e, size_t rows, size_t channels,
                 DeviceBuffer& scratch) {
    col_reduce_launch(rt, gy, idx, g_e, rows, channels, 2, scratch);
}

void relu2_backward(ullis_cuda_runtime* rt, const float* input, float* g, size_t n) {
    relu2_bwd_kernel<<<blocks_for((n + 3) / 4, 256), 256, 0, rt->stream>>>(input, g, n);
    rt->launched("relu2_bwd");
}

void layer_norm_backward(ullis_cuda_runtime* rt, const float* x, const float* gy, const uint16_t* w, float* gx,
                         float* xhat, float* gw, float* gb, size_t rows, size_t channels, DeviceBuffer& scratch) {
    ln_backward_kernel<<<blocks_for(rows, 8), 256, 0, rt->stream>>>(x, gy, w, gx, xhat, rows, channels, 0);
    rt->launched("ln_backward");
    col_reduce_launch(rt, gy, xhat, gw, rows, channels, 1, scratch);
    col_reduce_launch(rt, gy, nullptr, gb, rows, channels, 0, scratch);
}

}  // namespace k
}  // namespace ullis

// ------------------------------------------------------------ state
ullis_cuda_train_state::ullis_cuda_train_state(ullis_cuda_model* model, const uint8_t* checkpoint, size_t len)
    : m(model), rt(model->rt) {
    rt->bind();
    const size_t d = m->d, f = m->ffn, v = m->vocab;
    layers.assign(m->layers, Layer{});
    // plan: every latent (u16) and residual (f32) in one zeroed allocation
    struct Slot { void** at; size_t bytes; size_t offset; };
    std::vector<Slot> slots;
    size_t total = 0;
    auto want = [&](void** at, size_t bytes) {
        slots.push_back({at, bytes, total});
        total = (total + bytes + 255) / 256 * 256;
    };
    auto fp16 = [&](Fp16Param& p, const uint16_t* w, size_t n, const std::string& name) {
        p.w = const_cast<uint16_t*>(w);
        p.n = n;
        want(reinterpret_cast<void**>(&p.residual), n * 4);
        named[name] = Named{p.w, n * 2};
    };
    auto packed = [&](PackedParam& p, PackedWeights& w, const std::string& name) {
        p.weights = &w;
        const size_t n = w.out * w.in;
        want(reinterpret_cast<void**>(&p.latent), n * 2);
        want(reinterpret_cast<void**>(&p.latent_residual), n * 4);
        fp16(p.scale, w.scale, w.out, name + ".scale");
        if (w.bias) fp16(p.bias, w.bias, w.out, name + ".bias");
        named[name + ".bits"] = Named{const_cast<uint32_t*>(w.bits), (n + 31) / 32 * 4};
    };
    fp16(embedding, m->embedding, v * d, "embedding");
    fp16(ln_out_w, m->ln_out.weight, d, "ln_out.weight");
    fp16(ln_out_b, m->ln_out.bias, d, "ln_out.bias");
    packed(head, m->head, "head");
    for (size_t l = 0; l < m->layers; ++l) {
        LayerWeights& L = m->blocks[l];
        Layer& T = layers[l];
        const std::string pre = "blocks." + std::to_string(l);
        if (l == 0) {
            fp16(T.ln0_w, L.ln0.weight, d, pre + ".ln0.weight");
            fp16(T.ln0_b, L.ln0.bias, d, pre + ".ln0.bias");
        }
        fp16(T.ln2_w, L.ln2.weight, d, pre + ".ln2.weight");
        fp16(T.ln2_b, L.ln2.bias, d, pre + ".ln2.bias");
        fp16(T.e, L.e, d, pre + ".rosa.e");
        fp16(T.x_k, L.ffn_x_k, d, pre + ".ffn.x_k");
        fp16(T.value, L.value, f * d, pre + ".ffn.value");
        packed(T.o, L.o, pre + ".rosa.o");
        packed(T.key, L.key, pre + ".ffn.key");
        // frozen in this mode, readable all the same
        named[pre + ".rosa.q.bits"] = Named{const_cast<uint32_t*>(L.q.bits), (d * d + 31) / 32 * 4};
        named[pre + ".rosa.k.bits"] = Named{const_cast<uint32_t*>(L.k.bits), (d * d + 31) / 32 * 4};
        named[pre + ".rosa.v.bits"] = Named{const_cast<uint32_t*>(L.v.bits), (d * d + 31) / 32 * 4};
        named[pre + ".ln3.weight"] = Named{const_cast<uint16_t*>(L.ln3.weight), d * 2};
        named[pre + ".rosa.x_q"] = Named{const_cast<uint16_t*>(L.x_q), d * 2};
    }
    uint8_t* base = static_cast<uint8_t*>(carry.ensure(total ? total : 256));
    rt->zero(base, total);
    for (const Slot& s : slots) *s.at = base + s.offset;

    // latents: +/-0.01 by the sign bit (src/model.rs:640-649) unless the checkpoint carries them
    auto init_latent = [&](PackedParam& p, const std::string& name) {
        const size_t n = p.weights->out * p.weights->in;
        init_latent_kernel<<<blocks_for(n, 256), 256, 0, rt->stream>>>(p.weights->bits, p.latent, n);
        rt->launched("init_latent");
        named[name + ".latent"] = Named{p.latent, n * 2};
        named[name + ".latent.residual"] = Named{p.latent_residual, n * 4};
    };
    init_latent(head, "head");
    for (size_t l = 0; l < m->layers; ++l) {
        init_latent(layers[l].o, "blocks." + std::to_string(l) + ".rosa.o");
        init_latent(layers[l].key, "blocks." + std::to_string(l) + ".ffn.key");
    }
    auto residual_name = [&](const Fp16Param& p, const std::string& name) {
        named[name + ".residual"] = Named{p.residual, p.n * 4};
    };
    residual_name(embedding, "embedding");
    residual_name(ln_out_w, "ln_out.weight");
    residual_name(ln_out_b, "ln_out.bias");
    residual_name(head.scale, "head.scale");
    if (head.bias.w) residual_name(head.bias, "head.bias");
    for (size_t l = 0; l < m->layers; ++l) {
        Layer& T = layers[l];
        const std::string pre = "blocks." + std::to_string(l);
        if (l == 0) {
            residual_name(T.ln0_w, pre + ".ln0.weight");
            residual_name(T.ln0_b, pre + ".ln0.bias");
        }
        residual_name(T.ln2_w, pre + ".ln2.weight");
        residual_name(T.ln2_b, pre + ".ln2.bias");
        residual_name(T.e, pre + ".rosa.e");
        residual_name(T.x_k, pre + ".ffn.x_k");
        residual_name(T.value, pre + ".ffn.value");
        residual_name(T.o.scale, pre + ".rosa.o.scale");
        if (T.o.bias.w) residual_name(T.o.bias, pre + ".rosa.o.bias");
        residual_name(T.key.scale, pre + ".ffn.key.scale");
    }
    // carry of a resumed run: "<name>.latent" (F16) and "<name>.residual" (F32) tensors
    // (src/model.rs:3461-3466, 3724-3740)
    if (checkpoint && len) {
        SafeTensors stf = parse_safetensors(checkpoint, len);
        for (const auto& kv : stf.tensors) {
            const std::string& name = kv.first;
            const bool is_latent = name.size() > 7 && name.compare(name.size() - 7, 7, ".latent") == 0;
            const bool is_residual = name.size() > 9 && name.compare(name.size() - 9, 9, ".residual") == 0;
            if (!is_latent && !is_residual) continue;
            auto it = named.find(name);
            if (it == named.end()) continue;   // carry of a tensor this mode does not step
            if (kv.second.dtype != (is_latent ? "F16" : "F32") || kv.second.bytes != it->second.bytes)
                fail(ULLIS_CUDA_ERR_CHECKPOINT, "checkpoint carry shape mismatch (" + name + ")");
            rt->h2d(it->second.ptr, kv.second.data, kv.second.bytes);
        }
    }
    rt->sync();
}

void ullis_cuda_train_state::read(const char* name, void* dst, size_t bytes) {
    auto it = named.find(name ? name : "");
    if (it == named.end()) fail(ULLIS_CUDA_ERR_ARG, std::string("unknown tensor ") + (name ? name : "(null)"));
    if (bytes != it->second.bytes)
        fail(ULLIS_CUDA_ERR_SHAPE, "tensor size mismatch: expected " + std::to_string(it->second.bytes) + " bytes");
    rt->bind();
    rt->d2h(dst, it->second.ptr, bytes);
    rt->sync();
}

// ------------------------------------------------------------ the step
void ullis_cuda_train_state::step(const uint32_t* tokens, const uint32_t* labels_h, uint32_t ignore_id, size_t batch,
                                  size_t time, float learning_rate, ullis_cuda_train_result* out) {
    // src/model.rs:2837-2861
    if (!std::isfinite(learning_rate) || learning_rate <= 0.0f || time < 2)
        fail(ULLIS_CUDA_ERR_ARG, "train step requires a positive learning rate and time >= 2");
    if (!tokens || !labels_h) fail(ULLIS_CUDA_ERR_ARG, "tokens or labels is null");
    m->check_shape(batch, time);
    const size_t d = m->d, f = m->ffn, vocab = m->vocab, rows = batch * time;
    for (size_t r = 0; r < rows; ++r)
        if (tokens[r] >= vocab || (labels_h[r] != ignore_id && labels_h[r] >= vocab))
            fail(ULLIS_CUDA_ERR_SHAPE, "token shape or context length is invalid");
    rt->bind();

    // rows of each distinct token, in row order, for the embedding step
    std::vector<uint32_t> count(vocab + 1, 0), h_order(rows), h_toks, h_starts;
    for (size_t r = 0; r < rows; ++r) ++count[tokens[r] + 1];
    for (size_t t = 0; t < vocab; ++t) count[t + 1] += count[t];
    {
        std::vector<uint32_t> at(count.begin(), count.end() - 1);
        for (size_t r = 0; r < rows; ++r) h_order[at[tokens[r]]++] = (uint32_t)r;
    }
    for (size_t t = 0; t < vocab; ++t)
        if (count[t + 1] != count[t]) {
            h_toks.push_back((uint32_t)t);
            h_starts.push_back(count[t]);
        }
    h_starts.push_back((uint32_t)rows);
    rt->h2d(order.as<uint32_t>(rows), h_order.data(), rows * 4);
    rt->h2d(toks.as<uint32_t>(h_toks.size()), h_toks.data(), h_toks.size() * 4);
    rt->h2d(starts.as<uint32_t>(h_starts.size()), h_starts.data(), h_starts.size() * 4);

    // forward with the tape
    m->upload_tokens(tokens, labels_h, batch, time);
    m->train_tape = true;
    try {
        m->enqueue_hidden(batch, time);
    } catch (...) {
        m->train_tape = false;
        throw;
    }
    m->train_tape = false;

    const size_t n = rows * d, rows_p = pad64(rows), vocab_p = pad64(vocab), d_p = pad64(d), f_p = pad64(f);
    const bool exact = rt->mode == ULLIS_CUDA_MODE_EXACT;
    float P = 1.0f;
    while (P < (float)(time - 1)) P *= 2.0f;
    Step s{this, rt, 1.0f / P, learning_rate, (float)(time - 1)};
    float* X = m->x.as<float>(n);        // residual stream before ln_out
    float* H = m->a.as<float>(n);        // ln_out(X)
    float* GX = gx.as<float>(n);
    float* T1 = t1.as<float>(n);
    float* T2 = t2.as<float>(n);
    float* T3 = t3.as<float>(n);
    float* W1 = wide1.as<float>(rows * f);
    float* W2 = wide2.as<float>(rows * f);
    float* LG = logits.as<float>(rows * vocab);
    const size_t widest = std::max({f_p, vocab_p, d_p});
    uint16_t* A16 = a16.as<uint16_t>(std::max(rows * widest, std::max({f, vocab, d}) * rows_p));
    uint16_t* B16 = b16.as<uint16_t>(std::max(std::max(f, d) * rows_p, widest * std::max(f, d)));
    float* SM = small.as<float>(4 * std::max({f, vocab, d}));
    unsigned long long* CNT = counters.as<unsigned long long>(3);
    const uint32_t* lab = m->labels.as<uint32_t>(rows);
    float* RL = m->row_loss.as<float>(rows);
    uint8_t* res = static_cast<uint8_t*>(m->result.ensure(16));
    rt->zero(CNT, 24);
    gmat.as<float>(std::max({d * f, vocab * d, d * d}));                        // sized once: no growth mid-step
    part.as<float>((rows + 255) / 256 * std::max({f, vocab, d}));

    // ---- head: logits, loss, gy (src/model.rs:3204-3257)
    if (!tc::binary_linear(rt, H, m->head.bits, m->head.scale, m->head.bias, LG, rows, d, vocab))
        k::binary_linear_exact(rt, H, m->head.bits, m->head.scale, m->head.bias, LG, rows, d, vocab, false);
    ce_grad_kernel<<<(unsigned)rows, 256, 0, rt->stream>>>(LG, lab, ignore_id, rows, time, vocab,
                                                          1.0f / (float)(time - 1), P, RL, rt->dev_status);
    rt->launched("ce_grad");
    k::ce_reduce(rt, RL, lab, ignore_id, rows, time, reinterpret_cast<double*>(res),
                 reinterpret_cast<unsigned long long*>(res + 8));
    m->have_result = true;
    s.col_reduce(LG, nullptr, SM + 2 * vocab, rows, vocab, 0);                      // g_bias
    s.cast_rows(LG, m->head.scale, A16, rows, vocab, vocab_p);                      // (gy*scale) [rows, V]
    s.unpack_transpose(m->head.bits, B16, vocab, d, vocab_p);                       // S^T [d, V]
    s.gemm(A16, B16, GX, rows, vocab_p, d);                                         // g_hidden
    s.transpose_cast(LG, A16, rows, vocab, rows_p);                                 // gy^T [V, rows]
    s.transpose_cast(H, B16, rows, d, rows_p);                                      // hidden^T [d, rows]
    s.packed_update(head, A16, B16, rows_p, SM + 2 * vocab, learning_rate * HEAD_BIAS_LR_MULT, CNT + 0, SM);

    // ---- ln_out
    s.ln_backward(X, GX, ln_out_w, ln_out_b, T1, false, T2, SM, rows, d);
    std::swap(GX, T1);

    for (size_t li = m->layers; li-- > 0;) {
        LayerWeights& L = m->blocks[li];
        Layer& T = layers[li];
        const float* AR = m->tape_after[li].as<float>(n);   // residual stream after the ROSA block
        // ---- CMix: recompute ln2 -> shifted -> key from the tape (src/model.rs:1050-1061)
        k::layer_norm(rt, AR, L.ln2.weight, L.ln2.bias, T1, rows, d, exact);
        k::shift_mix(rt, T1, L.ffn_x_k, nullptr, nullptr, T2, nullptr, nullptr, rows, time, d);     // shifted
        if (!tc::binary_linear(rt, T2, L.key.bits, L.key.scale, nullptr, W1, rows, d, f))
            k::binary_linear_exact(rt, T2, L.key.bits, L.key.scale, nullptr, W1, rows, d, f, false);  // key
        // value: g_relu2 = gy . W (before W is stepped), g_W = gy^T . relu2 (src/model.rs:1138-1140)
        s.cast_rows(GX, nullptr, A16, rows, d, d_p);
        {
            uint16_t* wt = B16;
            transpose16_kernel<<<blocks_for(f * d_p, 256), 256, 0, rt->stream>>>(L.value, wt, d, f, d_p);
            rt->launched("transpose16");
            s.gemm(A16, wt, W2, rows, d_p, f);                                                        // g_relu2
        }
        s.transpose_cast(GX, A16, rows, d, rows_p);                                                   // gy^T
        s.transpose_cast(W1, B16, rows, f, rows_p, 1);                                                // relu2^T
        {
            float* G = gmat.as<float>(d * f);
            s.gemm(A16, B16, G, d, rows_p, f);
            s.sgd(T.value, G, learning_rate);
        }
        relu2_bwd_kernel<<<blocks_for((rows * f + 3) / 4, 256), 256, 0, rt->stream>>>(W1, W2, rows * f);        // g_key
        rt->launched("relu2_bwd");
        // key (src/model.rs:1141-1163)
        s.cast_rows(W2, L.key.scale, A16, rows, f, f_p);
        s.unpack_transpose(L.key.bits, B16, f, d, f_p);
        s.gemm(A16, B16, T3, rows, f_p, d);                                                           // g_shifted
        s.transpose_cast(W2, A16, rows, f, rows_p);
        s.transpose_cast(T2, B16, rows, d, rows_p);
        s.packed_update(T.key, A16, B16, rows_p, nullptr, 0.0f, CNT + 1, SM);
        // time-shift mix (src/model.rs:1164-1176)
        k::time_shift_delta(rt, T1, T2, rows, time, d);                                               // xx
        s.col_reduce(T3, T2, SM, rows, d, 1);                                                         // g_mix
        lerp_bwd_kernel<<<blocks_for(n, 256), 256, 0, rt->stream>>>(T3, L.ffn_x_k, T1, rows, time, d);
        rt->launched("lerp_bwd");
        s.sgd(T.x_k, SM, learning_rate);                                                              // after its last use
        s.ln_backward(AR, T1, T.ln2_w, T.ln2_b, GX, true, T2, SM, rows, d);

        // ---- ROSA: gradients stop at the q/k/v bits (src/model.rs:1494-1521)
        uint8_t* IDX = reinterpret_cast<uint8_t*>(T3);
        k::rosa_emit(rt, m->tape_idx[li].as<uint32_t>(1), L.e, IDX, T1, batch, time, d);               // idx, y = +/-e
        s.col_reduce(GX, nullptr, SM + 2 * d, rows, d, 0);                                            // g_bias
        s.cast_rows(GX, L.o.scale, A16, rows, d, d_p);
        s.unpack_transpose(L.o.bits, B16, d, d, d_p);
        s.gemm(A16, B16, T2, rows, d_p, d);                                                           // g_y
        s.col_reduce(T2, IDX, SM + 3 * d, rows, d, 2);                                                // g_e
        s.transpose_cast(GX, A16, rows, d, rows_p);
        s.transpose_cast(T1, B16, rows, d, rows_p);
        s.packed_update(T.o, A16, B16, rows_p, SM + 2 * d, learning_rate, CNT + 2, SM);
        s.sgd(T.e, SM + 3 * d, learning_rate);

        if (li == 0) {   // ln0 replaced x on layer 0: its input is the embedded rows (src/model.rs:2972-2977)
            k::embed(rt, m->ids.as<uint32_t>(rows), m->embedding, T1, rows, d, vocab);
            s.ln_backward(T1, GX, T.ln0_w, T.ln0_b, T2, false, T3, SM, rows, d);
            std::swap(GX, T2);
        }
    }
    // ---- embedding rows (src/model.rs:2980-2987)
    embed_sgd_kernel<<<dim3((unsigned)h_toks.size(), blocks_for(d, 128)), 128, 0, rt->stream>>>(embedding.w, embedding.residual, GX,
                                                                      toks.as<uint32_t>(1), starts.as<uint32_t>(1),
                                                                      order.as<uint32_t>(1), d, s.gmul, learning_rate);
    rt->launched("embed_sgd");

    unsigned long long h_cnt[3] = {0, 0, 0};
    rt->d2h(h_cnt, CNT, 24);
    float mean = 0.0f;
    uint64_t n_valid = 0;
    m->read_loss(&mean, nullptr, &n_valid, nullptr, 0);   // synchronises and checks the status word
    ++steps;
    if (out) *out = ullis_cuda_train_result{mean, n_valid, h_cnt[0], h_cnt[1], h_cnt[2]};
}

// install_head_unigram_prior (src/model.rs:3034-3085) with shrink_head_kaiming_scale (3087-3110): a
// one-shot host computation over the labels and two vocabulary-sized tensors.
void ullis_cuda_train_state::install_head_unigram_prior(const uint32_t* labels, size_t n, uint32_t ignore_id,
                                                        ullis_cuda_head_unigram_install* out) {
    if (!labels && n) fail(ULLIS_CUDA_ERR_ARG, "labels is null");
    const size_t vocab = m->vocab, d = m->d;
    rt->bind();
    std::vector<uint16_t> bias(vocab), scale(vocab);
    rt->d2h(bias.data(), head.bias.w, vocab * 2);
    rt->d2h(scale.data(), head.scale.w, vocab * 2);
    rt->sync();
    auto to_f32 = [](uint16_t b) { return __half2float(__ushort_as_half(b)); };
    auto to_f16 = [](float v) { return __half_as_ushort(__float2half_rn(v)); };
    auto rms = [&](const std::vector<uint16_t>& v) {
        float sum_sq = 0.0f;
        for (uint16_t b : v) sum_sq += to_f32(b) * to_f32(b);
        return v.empty() ? 0.0f : std::sqrt(sum_sq / (float)v.size());
    };
    float abs_sum = 0.0f;
    for (uint16_t b : bias) abs_sum += std::fabs(to_f32(b));
    ullis_cuda_head_unigram_install r{};
    if (abs_sum / (float)vocab > 0.05f) {   // HEAD_BIAS_PRIOR_ABS_EPS: a fitted prior is left alone
        r.bias_rms = rms(bias);
        r.scale_rms = rms(scale);
        if (out) *out = r;
        return;
    }
    std::vector<uint64_t> counts(vocab, 0);
    uint64_t n_targets = 0;
    for (size_t i = 0; i < n; ++i) {
        if (labels[i] == ignore_id || labels[i] >= vocab) continue;
        ++counts[labels[i]];
        ++n_targets;
    }
    if (n_targets == 0) fail(ULLIS_CUDA_ERR_ARG, "head unigram prior needs at least one supervised label");
    const float log_denom = std::log((float)n_targets + (float)vocab);
    std::vector<float> logs(vocab);
    float log_sum = 0.0f;
    for (size_t v = 0; v < vocab; ++v) {
        logs[v] = std::log1p((float)counts[v]) - log_denom;
        log_sum += logs[v];
    }
    const float log_mean = log_sum / (float)vocab;
    for (size_t v = 0; v < vocab; ++v) bias[v] = to_f16(logs[v] - log_mean);
    std::vector<float> zeros(vocab, 0.0f);
    rt->h2d(head.bias.w, bias.data(), vocab * 2);
    rt->h2d(head.bias.residual, zeros.data(), vocab * 4);   // Fp16Storage::set clears the carry (src/precision.rs:208-211)
    const float kaiming = 1.0f / std::sqrt((float)d);
    float mean = 0.0f;
    for (uint16_t b : scale) mean += to_f32(b);
    mean /= (float)vocab;
    if (mean > kaiming * 0.5f && mean < kaiming * 2.0f) {
        for (uint16_t& b : scale) b = to_f16(to_f32(b) * 0.25f);   // HEAD_KAIMING_SCALE_SHRINK
        rt->h2d(head.scale.w, scale.data(), vocab * 2);
        rt->h2d(head.scale.residual, zeros.data(), vocab * 4);
        r.shrunk_kaiming_scale = 1;
    }
    rt->sync();
    r.applied = 1;
    r.n_targets = n_targets;
    r.bias_rms = rms(bias);
    r.scale_rms = rms(scale);
    if (out) *out = r;
}
