// HBM-bound elementwise / row kernels of the Heron forward path: embedding
// gather, LayerNorm, time-shift mixing, sign-threshold bit packing, relu^2,
// residual add and the ROSA +/-e emit.  Arithmetic that the reference performs
// as separate f32 operations is written with the _rn intrinsics so the
// compiler cannot contract it into fused multiply-adds.
#include <cuda_fp16.h>

#include "kernels.hpp"

namespace ullis {
namespace k {

namespace {

__device__ __forceinline__ float h2f(uint16_t bits) { return __half2float(__ushort_as_half(bits)); }

inline unsigned blocks_for(size_t n, unsigned per_block) { return (unsigned)((n + per_block - 1) / per_block); }

// ------------------------------------------------------------------ embed
// reference src/model.rs:2660-2669
__global__ void embed_kernel(const uint32_t* __restrict__ ids, const uint16_t* __restrict__ emb,
                             float* __restrict__ x, size_t rows, size_t d, size_t vocab, uint32_t* status) {
    size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= rows * d) return;
    size_t row = e / d, c = e % d;
    uint32_t id = ids[row];
    if (id >= vocab) {
        if (c == 0 && atomicCAS(status, ULLIS_DEV_OK, ULLIS_DEV_BAD_TOKEN) == ULLIS_DEV_OK) status[1] = (uint32_t)row;
        x[e] = 0.0f;
        return;
    }
    x[e] = h2f(emb[(size_t)id * d + c]);
}

// -------------------------------------------------------------- LayerNorm
// Reference order (src/model.rs:259-276): sequential sum, /C, sequential sum
// of squared deviations, /C, 1/sqrt(var+eps), ((x-mean)*inv)*w + b.
// One CTA normalises 32 rows; a row's sequential sums are carried by one
// thread reading a transposed shared-memory tile that the whole CTA loads
// with coalesced accesses.
constexpr int LNX_ROWS = 32, LNX_CHUNK = 128, LNX_THREADS = 256;

__global__ void __launch_bounds__(LNX_THREADS)
ln_exact_kernel(const float* __restrict__ x, const uint16_t* __restrict__ w, const uint16_t* __restrict__ b,
                float* __restrict__ y, size_t rows, size_t C) {
    __shared__ float tile[LNX_ROWS][LNX_CHUNK + 1];
    __shared__ float s_mean[LNX_ROWS], s_inv[LNX_ROWS];
    const size_t row0 = (size_t)blockIdx.x * LNX_ROWS;
    const int tid = threadIdx.x;
    float acc = 0.0f;
    for (int pass = 0; pass < 2; ++pass) {
        acc = 0.0f;
        const float mean = (pass == 1 && tid < LNX_ROWS) ? s_mean[tid] : 0.0f;
        for (size_t c0 = 0; c0 < C; c0 += LNX_CHUNK) {
            for (int e = tid; e < LNX_ROWS * LNX_CHUNK; e += LNX_THREADS) {
                int r = e / LNX_CHUNK, c = e % LNX_CHUNK;
                float v = 0.0f;
                if (row0 + r < rows && c0 + c < C) v = x[(row0 + r) * C + c0 + c];
                tile[r][c] = v;
            }
            __syncthreads();
            if (tid < LNX_ROWS) {
                const int lim = (int)((C - c0) < (size_t)LNX_CHUNK ? (C - c0) : (size_t)LNX_CHUNK);
                if (pass == 0) {
                    for (int c = 0; c < lim; ++c) acc = __fadd_rn(acc, tile[tid][c]);
                } else {
                    for (int c = 0; c < lim; ++c) {
                        float dlt = __fsub_rn(tile[tid][c], mean);
                        acc = __fadd_rn(acc, __fmul_rn(dlt, dlt));
                    }
                }
            }
            __syncthreads();
        }
        if (tid < LNX_ROWS) {
            if (pass == 0) {
                s_mean[tid] = __fdiv_rn(acc, (float)C);
            } else {
                float var = __fdiv_rn(acc, (float)C);
                s_inv[tid] = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(var, 1e-5f)));
            }
        }
        __syncthreads();
    }
    for (size_t e = tid; e < (size_t)LNX_ROWS * C; e += LNX_THREADS) {
        size_t r = e / C, c = e % C;
        if (row0 + r >= rows) break;
        float v = x[(row0 + r) * C + c];
        float n = __fmul_rn(__fsub_rn(v, s_mean[r]), s_inv[r]);
        y[(row0 + r) * C + c] = __fadd_rn(__fmul_rn(n, h2f(w[c])), h2f(b[c]));
    }
}

// Fast path: one warp per row, the row is read once with 128-bit loads and
// kept in registers (C <= 1024, C % 128 == 0); mean and variance by warp
// shuffles. Other widths take the generic re-reading loop.
template <int VEC_PER_LANE>
__global__ void __launch_bounds__(256)
ln_warp_kernel(const float* __restrict__ x, const uint16_t* __restrict__ w, const uint16_t* __restrict__ b,
               float* __restrict__ y, size_t rows, int C) {
    const int lane = threadIdx.x & 31;
    const size_t row = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const float4* src = reinterpret_cast<const float4*>(x + row * C);
    float4 v[VEC_PER_LANE];
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < VEC_PER_LANE; ++i) {
        v[i] = src[lane + 32 * i];
        sum += (v[i].x + v[i].y) + (v[i].z + v[i].w);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float mean = sum / (float)C;
    float sq = 0.0f;
#pragma unroll
    for (int i = 0; i < VEC_PER_LANE; ++i) {
        float a = v[i].x - mean, bb = v[i].y - mean, c = v[i].z - mean, d = v[i].w - mean;
        sq += (a * a + bb * bb) + (c * c + d * d);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
    const float inv = 1.0f / sqrtf(sq / (float)C + 1e-5f);
    float4* dst = reinterpret_cast<float4*>(y + row * C);
    const uint2* w4 = reinterpret_cast<const uint2*>(w);
    const uint2* b4 = reinterpret_cast<const uint2*>(b);
#pragma unroll
    for (int i = 0; i < VEC_PER_LANE; ++i) {
        uint2 wb = w4[lane + 32 * i], bb = b4[lane + 32 * i];
        float4 o;
        o.x = (v[i].x - mean) * inv * h2f((uint16_t)(wb.x & 0xffff)) + h2f((uint16_t)(bb.x & 0xffff));
        o.y = (v[i].y - mean) * inv * h2f((uint16_t)(wb.x >> 16)) + h2f((uint16_t)(bb.x >> 16));
        o.z = (v[i].z - mean) * inv * h2f((uint16_t)(wb.y & 0xffff)) + h2f((uint16_t)(bb.y & 0xffff));
        o.w = (v[i].w - mean) * inv * h2f((uint16_t)(wb.y >> 16)) + h2f((uint16_t)(bb.y >> 16));
        dst[lane + 32 * i] = o;
    }
}

__global__ void __launch_bounds__(256)
ln_warp_generic_kernel(const float* __restrict__ x, const uint16_t* __restrict__ w,
                       const uint16_t* __restrict__ b, float* __restrict__ y, size_t rows, size_t C) {
    const int lane = threadIdx.x & 31;
    const size_t row = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const float* src = x + row * C;
    float sum = 0.0f;
    for (size_t c = lane; c < C; c += 32) sum += src[c];
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float mean = sum / (float)C;
    float sq = 0.0f;
    for (size_t c = lane; c < C; c += 32) {
        float d = src[c] - mean;
        sq += d * d;
    }
    for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
    const float inv = 1.0f / sqrtf(sq / (float)C + 1e-5f);
    for (size_t c = lane; c < C; c += 32) y[row * C + c] = (src[c] - mean) * inv * h2f(w[c]) + h2f(b[c]);
}

// ------------------------------------------------------------- time shift
// reference src/model.rs:186-212
__global__ void time_shift_delta_kernel(const float* __restrict__ x, float* __restrict__ xx, size_t n, size_t time,
                                        size_t C) {
    size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= n) return;
    size_t row = e / C;
    float xt = x[e];
    xx[e] = (row % time == 0) ? -xt : __fsub_rn(x[e - C], xt);
}

// reference src/model.rs:1291-1298, 992-997: in = x + xx*mix (multiply, then add)
__global__ void shift_mix_kernel(const float* __restrict__ x, const uint16_t* __restrict__ m0,
                                 const uint16_t* __restrict__ m1, const uint16_t* __restrict__ m2,
                                 float* __restrict__ o0, float* __restrict__ o1, float* __restrict__ o2, size_t n,
                                 size_t time, size_t C) {
    size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= n) return;
    size_t row = e / C, c = e % C;
    float xt = x[e];
    float xx = (row % time == 0) ? -xt : __fsub_rn(x[e - C], xt);
    o0[e] = __fadd_rn(xt, __fmul_rn(xx, h2f(m0[c])));
    if (o1) o1[e] = __fadd_rn(xt, __fmul_rn(xx, h2f(m1[c])));
    if (o2) o2[e] = __fadd_rn(xt, __fmul_rn(xx, h2f(m2[c])));
}

// ------------------------------------------------------------- bit planes
// reference src/rosa.rs:372-374 (bit = v > 0) and 400-411 (LSB-first words)
__global__ void sign_pack_flat_kernel(const float* __restrict__ x, uint32_t* __restrict__ words, size_t n) {
    size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    bool bit = e < n && x[e] > 0.0f;
    uint32_t word = __ballot_sync(0xffffffffu, bit);
    if ((threadIdx.x & 31) == 0 && e < n) words[e >> 5] = word;
}

// x [B,T,C] f32 -> stream-major sign words. Block = 32 steps x 32 channels.
__global__ void __launch_bounds__(1024)
sign_pack_streams_kernel(const float* __restrict__ x, uint32_t* __restrict__ sw, size_t T, size_t C, size_t wps) {
    __shared__ uint8_t sm[32][33];
    const size_t b = blockIdx.z, t0 = (size_t)blockIdx.x * 32, c0 = (size_t)blockIdx.y * 32;
    const int tx = threadIdx.x, ty = threadIdx.y;
    bool bit = false;
    if (t0 + ty < T && c0 + tx < C) bit = x[((b * T + t0 + ty) * C) + c0 + tx] > 0.0f;
    sm[ty][tx] = bit;
    __syncthreads();
    uint32_t word = __ballot_sync(0xffffffffu, sm[tx][ty] != 0);  // lanes = steps, warp = channel ty
    if (tx == 0 && c0 + ty < C) sw[(b * C + c0 + ty) * wps + blockIdx.x] = word;
}

// flat [B,T,C] plane words -> stream-major words (any T, C)
__global__ void planes_to_streams_kernel(const uint32_t* __restrict__ plane, uint32_t* __restrict__ sw, size_t B,
                                         size_t T, size_t C, size_t wps) {
    size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= B * C * wps) return;
    size_t s = e / wps, wd = e % wps, b = s / C, c = s % C;
    uint32_t word = 0;
    for (int tt = 0; tt < 32; ++tt) {
        size_t t = wd * 32 + tt;
        if (t >= T) break;
        size_t idx = (b * T + t) * C + c;
        word |= ((plane[idx >> 5] >> (idx & 31)) & 1u) << tt;
    }
    sw[e] = word;
}

// The same for C % 32 == 0, where a step's channels are whole words: a warp takes one word column (32 channels)
// of one sequence and eight blocks of 32 steps.  Lane l reads the word of step l; 32 ballots turn the 32 x 32 bit
// block (lane i keeps the word of channel i), and after eight blocks lane i writes eight consecutive words of its
// stream.  The warps of a CTA take neighbouring word columns of the same steps, so the 4-byte reads of a row
// share their sectors in L1.
constexpr int P2S_BLOCKS = 8;
__global__ void __launch_bounds__(512)
planes_to_streams_words_kernel(const uint32_t* __restrict__ plane, uint32_t* __restrict__ sw, size_t T, size_t C,
                               size_t wps) {
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5, cwords = (uint32_t)(C >> 5);
    const size_t b = blockIdx.z, tb0 = (size_t)blockIdx.x * P2S_BLOCKS;
    const uint32_t cw = blockIdx.y * (blockDim.x >> 5) + warp;
    if (cw >= cwords) return;
    uint32_t mine[P2S_BLOCKS];
#pragma unroll
    for (int k = 0; k < P2S_BLOCKS; ++k) {
        const size_t t = (tb0 + k) * 32 + lane;
        const uint32_t x = t < T ? plane[(b * T + t) * cwords + cw] : 0u;
        uint32_t keep = 0;
#pragma unroll
        for (uint32_t i = 0; i < 32; ++i) {
            const uint32_t word = __ballot_sync(0xffffffffu, (x >> i) & 1u);
            if (lane == i) keep = word;
        }
        mine[k] = keep;
    }
    uint32_t* dst = sw + (b * C + (size_t)cw * 32 + lane) * wps + tb0;
#pragma unroll
    for (int k = 0; k < P2S_BLOCKS; ++k)
        if (tb0 + k < wps) dst[k] = mine[k];
}

__global__ void streams_to_planes_kernel(const uint32_t* __restrict__ sw, uint32_t* __restrict__ plane, size_t B,
                                         size_t T, size_t C, size_t wps) {
    size_t wd = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t n = B * T * C;
    if (wd >= (n + 31) / 32) return;
    uint32_t word = 0;
    for (int k = 0; k < 32; ++k) {
        size_t idx = wd * 32 + k;
        if (idx >= n) break;
        size_t c = idx % C, row = idx / C, t = row % T, b = row / T;
        word |= ((sw[(b * C + c) * wps + (t >> 5)] >> (t & 31)) & 1u) << k;
    }
    plane[wd] = word;
}

// reference src/model.rs:999: max(v,0)*max(v,0)
__global__ void relu2_kernel(const float* __restrict__ x, float* __restrict__ y, size_t n) {
    size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= n) return;
    float m = fmaxf(x[e], 0.0f);
    y[e] = __fmul_rn(m, m);
}

__global__ void residual_add_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                    float* __restrict__ out, size_t n) {
    size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e < n) out[e] = __fadd_rn(a[e], b[e]);
}

// reference src/model.rs:1313 / src/rosa.rs:585-609: y = (2*idx-1)*e, i.e. +e or -e
__global__ void __launch_bounds__(1024)
rosa_emit_kernel(const uint32_t* __restrict__ idx_sw, const uint16_t* __restrict__ e, uint8_t* __restrict__ idx,
                 float* __restrict__ y, size_t T, size_t C, size_t wps) {
    __shared__ uint32_t wsm[32];
    const size_t b = blockIdx.z, t0 = (size_t)blockIdx.x * 32, c0 = (size_t)blockIdx.y * 32;
    const int tx = threadIdx.x, ty = threadIdx.y;
    if (ty == 0) wsm[tx] = (c0 + tx < C) ? idx_sw[(b * C + c0 + tx) * wps + blockIdx.x] : 0u;
    __syncthreads();
    if (t0 + ty >= T || c0 + tx >= C) return;
    const uint32_t bit = (wsm[tx] >> ty) & 1u;
    const size_t o = (b * T + t0 + ty) * C + c0 + tx;
    if (idx) idx[o] = (uint8_t)bit;
    if (y) {
        float ev = h2f(e[c0 + tx]);
        y[o] = bit ? ev : -ev;
    }
}

}  // namespace

void embed(ullis_cuda_runtime* rt, const uint32_t* ids, const uint16_t* emb, float* x, size_t rows, size_t d,
           size_t vocab) {
    if (rows * d == 0) return;
    embed_kernel<<<blocks_for(rows * d, 256), 256, 0, rt->stream>>>(ids, emb, x, rows, d, vocab, rt->dev_status);
    rt->launched("embed");
}

void layer_norm(ullis_cuda_runtime* rt, const float* x, const uint16_t* w, const uint16_t* b, float* y,
                size_t rows, size_t channels, bool exact) {
    if (rows == 0) return;
    if (exact) {
        ln_exact_kernel<<<blocks_for(rows, LNX_ROWS), LNX_THREADS, 0, rt->stream>>>(x, w, b, y, rows, channels);
        rt->launched("ln_exact");
        return;
    }
    const unsigned grid = blocks_for(rows, 8);
    const bool vec = channels % 128 == 0 && channels <= 1024 &&
                     (reinterpret_cast<uintptr_t>(x) % 16 == 0) && (reinterpret_cast<uintptr_t>(y) % 16 == 0) &&
                     (reinterpret_cast<uintptr_t>(w) % 8 == 0) && (reinterpret_cast<uintptr_t>(b) % 8 == 0);
    if (vec) {
        switch (channels / 128) {
            case 1: ln_warp_kernel<1><<<grid, 256, 0, rt->stream>>>(x, w, b, y, rows, (int)channels); break;
            case 2: ln_warp_kernel<2><<<grid, 256, 0, rt->stream>>>(x, w, b, y, rows, (int)channels); break;
            case 3: ln_warp_kernel<3><<<grid, 256, 0, rt->stream>>>(x, w, b, y, rows, (int)channels); break;
            case 4: ln_warp_kernel<4><<<grid, 256, 0, rt->stream>>>(x, w, b, y, rows, (int)channels); break;
            case 5: ln_warp_kernel<5><<<grid, 256, 0, rt->stream>>>(x, w, b, y, rows, (int)channels); break;
            case 6: ln_warp_kernel<6><<<grid, 256, 0, rt->stream>>>(x, w, b, y, rows, (int)channels); break;
            case 7: ln_warp_kernel<7><<<grid, 256, 0, rt->stream>>>(x, w, b, y, rows, (int)channels); break;
            default: ln_warp_kernel<8><<<grid, 256, 0, rt->stream>>>(x, w, b, y, rows, (int)channels); break;
        }
    } else {
        ln_warp_generic_kernel<<<grid, 256, 0, rt->stream>>>(x, w, b, y, rows, channels);
    }
    rt->launched("ln_warp");
}

void time_shift_delta(ullis_cuda_runtime* rt, const float* x, float* xx, size_t rows, size_t time,
                      size_t channels) {
    const size_t n = rows * channels;
    if (!n) return;
    time_shift_delta_kernel<<<blocks_for(n, 256), 256, 0, rt->stream>>>(x, xx, n, time, channels);
    rt->launched("time_shift_delta");
}

void shift_mix(ullis_cuda_runtime* rt, const float* x, const uint16_t* m0, const uint16_t* m1,
               const uint16_t* m2, float* o0, float* o1, float* o2, size_t rows, size_t time, size_t channels) {
    const size_t n = rows * channels;
    if (!n) return;
    shift_mix_kernel<<<blocks_for(n, 256), 256, 0, rt->stream>>>(x, m0, m1, m2, o0, o1, o2, n, time, channels);
    rt->launched("shift_mix");
}

void sign_pack_flat(ullis_cuda_runtime* rt, const float* x, uint32_t* words, size_t n) {
    if (!n) return;
    sign_pack_flat_kernel<<<blocks_for(n, 256), 256, 0, rt->stream>>>(x, words, n);
    rt->launched("sign_pack_flat");
}

void sign_pack_streams(ullis_cuda_runtime* rt, const float* x, uint32_t* sw, size_t batch, size_t time,
                       size_t channels) {
    if (batch * time * channels == 0) return;
    const size_t wps = (time + 31) / 32;
    dim3 grid((unsigned)wps, (unsigned)((channels + 31) / 32), (unsigned)batch);
    sign_pack_streams_kernel<<<grid, dim3(32, 32), 0, rt->stream>>>(x, sw, time, channels, wps);
    rt->launched("sign_pack_streams");
}

void planes_to_streams(ullis_cuda_runtime* rt, const uint32_t* plane, uint32_t* sw, size_t batch, size_t time,
                       size_t channels) {
    const size_t wps = (time + 31) / 32, n = batch * channels * wps;
    if (!n) return;
    if (channels % 32 == 0 && batch <= 65535) {
        const unsigned cwords = (unsigned)(channels / 32), warps = cwords < 16 ? cwords : 16;
        dim3 grid((unsigned)((wps + P2S_BLOCKS - 1) / P2S_BLOCKS), (cwords + warps - 1) / warps, (unsigned)batch);
        planes_to_streams_words_kernel<<<grid, warps * 32, 0, rt->stream>>>(plane, sw, time, channels, wps);
        rt->launched("planes_to_streams");
        return;
    }
    planes_to_streams_kernel<<<blocks_for(n, 256), 256, 0, rt->stream>>>(plane, sw, batch, time, channels, wps);
    rt->launched("planes_to_streams");
}

void streams_to_planes(ullis_cuda_runtime* rt, const uint32_t* sw, uint32_t* plane, size_t batch, size_t time,
                       size_t channels) {
    const size_t wps = (time + 31) / 32, n = (batch * time * channels + 31) / 32;
    if (!n) return;
    streams_to_planes_kernel<<<blocks_for(n, 256), 256, 0, rt->stream>>>(sw, plane, batch, time, channels, wps);
    rt->launched("streams_to_planes");
}

void relu2(ullis_cuda_runtime* rt, const float* x, float* y, size_t n) {
    if (!n) return;
    relu2_kernel<<<blocks_for(n, 256), 256, 0, rt->stream>>>(x, y, n);
    rt->launched("relu2");
}

void residual_add(ullis_cuda_runtime* rt, const float* a, const float* b, float* out, size_t n) {
    if (!n) return;
    residual_add_kernel<<<blocks_for(n, 256), 256, 0, rt->stream>>>(a, b, out, n);
    rt->launched("residual_add");
}

void rosa_emit(ullis_cuda_runtime* rt, const uint32_t* idx_sw, const uint16_t* e, uint8_t* idx, float* y,
               size_t batch, size_t time, size_t channels) {
    if (batch * time * channels == 0) return;
    const size_t wps = (time + 31) / 32;
    dim3 grid((unsigned)wps, (unsigned)((channels + 31) / 32), (unsigned)batch);
    rosa_emit_kernel<<<grid, dim3(32, 32), 0, rt->stream>>>(idx_sw, e, idx, y, time, channels, wps);
    rt->launched("rosa_emit");
}

}  // namespace k
}  // namespace ullis
