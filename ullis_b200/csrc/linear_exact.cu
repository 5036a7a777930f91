// Validation-mode linears on CUDA cores: f32 accumulation in exactly the
// reference's order, so every output is bit-identical to the CPU backend.
//
//  packed:  y[r,o] = bias[o] + scale[o] * sum_{i ascending} s(o,i) * x[r,i]
//           (reference src/model.rs:724-742; s = +1 iff bit o*K+i is set,
//           src/model.rs:146-148).  s*x is exact, so fmaf(s, x, acc) rounds
//           once, exactly like the reference's `sum += sign * x`.
//  dense :  y[r,o] = sum_{i ascending} W[o,i] * x[r,i], product rounded, then
//           added (reference src/model.rs:419-436; Rust does not contract).
//
// Tiling: a 256-thread CTA computes a 64x64 output tile, 4x4 outputs per
// thread, stepping K in chunks of 32 through shared memory.  Any rows/K/N.
#include <cuda_fp16.h>

#include "kernels.hpp"

namespace ullis {
namespace k {

namespace {

constexpr int TM = 64, TN = 64, TK = 32;

__device__ __forceinline__ float h2f(uint16_t bits) { return __half2float(__ushort_as_half(bits)); }

template <bool PACKED>
__global__ void __launch_bounds__(256)
linear_exact_kernel(const float* __restrict__ x, const uint32_t* __restrict__ bits,
                    const uint16_t* __restrict__ wdense, const uint16_t* __restrict__ scale,
                    const uint16_t* __restrict__ bias, float* __restrict__ y, size_t rows, size_t K, size_t N,
                    int accumulate) {
    __shared__ float xs[TM][TK + 1];
    __shared__ float ws[TK][TN + 1];
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const size_t r0 = (size_t)blockIdx.y * TM, o0 = (size_t)blockIdx.x * TN;
    float acc[4][4];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) acc[a][b] = 0.0f;

    for (size_t k0 = 0; k0 < K; k0 += TK) {
        const int kmax = (int)((K - k0) < (size_t)TK ? (K - k0) : (size_t)TK);
        for (int e = tid; e < TM * TK; e += 256) {
            int r = e / TK, kk = e % TK;
            float v = 0.0f;
            if (r0 + r < rows && kk < kmax) v = x[(r0 + r) * K + k0 + kk];
            xs[r][kk] = v;
        }
        for (int e = tid; e < TK * TN; e += 256) {
            int o = e / TK, kk = e % TK;  // consecutive threads walk K: adjacent weight bits / halves
            float v = 0.0f;
            if (o0 + o < N && kk < kmax) {
                size_t index = (o0 + o) * K + k0 + kk;
                if (PACKED)
                    v = (bits[index >> 5] >> (index & 31)) & 1u ? 1.0f : -1.0f;
                else
                    v = h2f(wdense[index]);
            }
            ws[kk][o] = v;
        }
        __syncthreads();
        for (int kk = 0; kk < kmax; ++kk) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = xs[ty * 4 + i][kk];
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (PACKED)
                        acc[i][j] = __fmaf_rn(w[j], a[i], acc[i][j]);
                    else
                        acc[i][j] = __fadd_rn(acc[i][j], __fmul_rn(w[j], a[i]));
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const size_t r = r0 + ty * 4 + i;
        if (r >= rows) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const size_t o = o0 + tx * 4 + j;
            if (o >= N) continue;
            float v = acc[i][j];
            if (PACKED) {
                const float bv = bias ? h2f(bias[o]) : 0.0f;
                v = __fadd_rn(bv, __fmul_rn(h2f(scale[o]), v));
            }
            float* dst = y + r * N + o;
            *dst = accumulate ? __fadd_rn(*dst, v) : v;
        }
    }
}

// Few rows (incremental generation): one thread per output, the row of x in
// shared memory, the same i-ascending f32 sum as above.  A thread's 32 weight
// bits come with one load; every lane reads the same x[i] (broadcast).
template <bool PACKED>
__global__ void __launch_bounds__(128)
rowvec_exact_kernel(const float* __restrict__ x, const uint32_t* __restrict__ bits,
                    const uint16_t* __restrict__ wdense, const uint16_t* __restrict__ scale,
                    const uint16_t* __restrict__ bias, float* __restrict__ y, size_t K, size_t N, int accumulate) {
    extern __shared__ float xrow[];
    const size_t r = blockIdx.y, o = (size_t)blockIdx.x * 128 + threadIdx.x;
    for (size_t i = threadIdx.x; i < K; i += 128) xrow[i] = x[r * K + i];
    __syncthreads();
    if (o >= N) return;
    float sum = 0.0f;
    if (PACKED) {
        if (K % 32 == 0) {
            const uint32_t* wrow = bits + (o * K >> 5);
            for (size_t i0 = 0; i0 < K; i0 += 32) {
                const uint32_t w = wrow[i0 >> 5];
#pragma unroll
                for (int b = 0; b < 32; ++b) sum = __fmaf_rn((w >> b) & 1u ? 1.0f : -1.0f, xrow[i0 + b], sum);
            }
        } else {
            for (size_t i = 0; i < K; ++i) {
                const size_t index = o * K + i;
                sum = __fmaf_rn((bits[index >> 5] >> (index & 31)) & 1u ? 1.0f : -1.0f, xrow[i], sum);
            }
        }
        const float bv = bias ? h2f(bias[o]) : 0.0f;
        sum = __fadd_rn(bv, __fmul_rn(h2f(scale[o]), sum));
    } else {
        const uint16_t* wrow = wdense + o * K;
        if (K % 8 == 0) {
            for (size_t i0 = 0; i0 < K; i0 += 8) {
                const uint4 w8 = *reinterpret_cast<const uint4*>(wrow + i0);
                const uint32_t w[4] = {w8.x, w8.y, w8.z, w8.w};
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const uint16_t hb = (uint16_t)(e & 1 ? w[e >> 1] >> 16 : w[e >> 1] & 0xFFFFu);
                    sum = __fadd_rn(sum, __fmul_rn(h2f(hb), xrow[i0 + e]));
                }
            }
        } else {
            for (size_t i = 0; i < K; ++i) sum = __fadd_rn(sum, __fmul_rn(h2f(wrow[i]), xrow[i]));
        }
    }
    float* dst = y + r * N + o;
    *dst = accumulate ? __fadd_rn(*dst, sum) : sum;
}

constexpr size_t ROWVEC_MAX_ROWS = 128, ROWVEC_MAX_K = 12288;   // x row within the default 48 KiB of shared memory

}  // namespace

void binary_linear_exact(ullis_cuda_runtime* rt, const float* x, const uint32_t* bits, const uint16_t* scale,
                         const uint16_t* bias, float* y, size_t rows, size_t in_features, size_t out_features,
                         bool accumulate) {
    if (rows == 0 || out_features == 0) return;
    if (rows <= ROWVEC_MAX_ROWS && in_features <= ROWVEC_MAX_K) {
        dim3 g((unsigned)((out_features + 127) / 128), (unsigned)rows);
        rowvec_exact_kernel<true><<<g, 128, in_features * 4, rt->stream>>>(x, bits, nullptr, scale, bias, y, in_features,
                                                                          out_features, accumulate ? 1 : 0);
        rt->launched("binary_rowvec_exact");
        return;
    }
    dim3 grid((unsigned)((out_features + TN - 1) / TN), (unsigned)((rows + TM - 1) / TM));
    linear_exact_kernel<true><<<grid, 256, 0, rt->stream>>>(x, bits, nullptr, scale, bias, y, rows, in_features,
                                                           out_features, accumulate ? 1 : 0);
    rt->launched("binary_linear_exact");
}

void fp16_linear_exact(ullis_cuda_runtime* rt, const float* x, const uint16_t* w, float* y, size_t rows,
                       size_t in_features, size_t out_features, bool accumulate) {
    if (rows == 0 || out_features == 0) return;
    if (rows <= ROWVEC_MAX_ROWS && in_features <= ROWVEC_MAX_K) {
        dim3 g((unsigned)((out_features + 127) / 128), (unsigned)rows);
        rowvec_exact_kernel<false><<<g, 128, in_features * 4, rt->stream>>>(x, nullptr, w, nullptr, nullptr, y, in_features,
                                                                           out_features, accumulate ? 1 : 0);
        rt->launched("fp16_rowvec_exact");
        return;
    }
    dim3 grid((unsigned)((out_features + TN - 1) / TN), (unsigned)((rows + TM - 1) / TM));
    linear_exact_kernel<false><<<grid, 256, 0, rt->stream>>>(x, nullptr, w, nullptr, nullptr, y, rows, in_features,
                                                            out_features, accumulate ? 1 : 0);
    rt->launched("fp16_linear_exact");
}

}  // namespace k
}  // namespace ullis
