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
    extern __shared__ __align__(16) float xrow[];
    const size_t r = blockIdx.y, o = (size_t)blockIdx.x * 128 + threadIdx.x;
    for (size_t i = threadIdx.x; i < K; i += 128) xrow[i] = x[r * K + i];
    __syncthreads();
    if (o >= N) return;
    float sum = 0.0f;
    if (PACKED) {
        if (K % 32 == 0) {
            const uint32_t* wrow = bits + (o * K >> 5);
            uint32_t w = wrow[0];
            for (size_t i0 = 0; i0 < K; i0 += 32) {
                const uint32_t w_next = i0 + 32 < K ? wrow[(i0 >> 5) + 1] : 0u;   // on its way while this word's terms are added
                float4 xv[8];   // the 32 inputs of the word: eight 16-byte loads ahead of the chain of additions
#pragma unroll
                for (int u = 0; u < 8; ++u) xv[u] = *reinterpret_cast<const float4*>(xrow + i0 + 4 * u);
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    sum = __fmaf_rn((w >> (4 * u + 0)) & 1u ? 1.0f : -1.0f, xv[u].x, sum);
                    sum = __fmaf_rn((w >> (4 * u + 1)) & 1u ? 1.0f : -1.0f, xv[u].y, sum);
                    sum = __fmaf_rn((w >> (4 * u + 2)) & 1u ? 1.0f : -1.0f, xv[u].z, sum);
                    sum = __fmaf_rn((w >> (4 * u + 3)) & 1u ? 1.0f : -1.0f, xv[u].w, sum);
                }
                w = w_next;
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

// Up to three packed matvecs of the same shape in one launch (the Q, K and V of a step: blockIdx.z picks the
// matrix and its input row), and an optional relu^2 on the way out (the CMix key: src/model.rs:999).  Same sums as
// rowvec_exact_kernel<true>.  K % 32 == 0.
struct RowvecSet {
    const float* x[3];
    const uint32_t* bits[3];
    const uint16_t* scale[3];
    const uint16_t* bias[3];
    float* y[3];
};
__global__ void __launch_bounds__(128)
rowvec_packed_multi_kernel(RowvecSet set, size_t K, size_t N, int relu2) {
    extern __shared__ __align__(16) float xrow[];
    const int z = blockIdx.z;
    const size_t r = blockIdx.y, o = (size_t)blockIdx.x * 128 + threadIdx.x;
    // picked with selects: indexing the parameter arrays with z would copy them to local memory
    auto pick = [z](auto a0, auto a1, auto a2) { return z == 0 ? a0 : z == 1 ? a1 : a2; };
    const float* x = pick(set.x[0], set.x[1], set.x[2]);
    const uint32_t* bits = pick(set.bits[0], set.bits[1], set.bits[2]);
    const uint16_t* scale = pick(set.scale[0], set.scale[1], set.scale[2]);
    const uint16_t* bias = pick(set.bias[0], set.bias[1], set.bias[2]);
    float* y = pick(set.y[0], set.y[1], set.y[2]);
    for (size_t i = threadIdx.x; i < K; i += 128) xrow[i] = x[r * K + i];
    __syncthreads();
    if (o >= N) return;
    float sum = 0.0f;
    const uint32_t* wrow = bits + (o * K >> 5);
    uint32_t w = wrow[0];
    for (size_t i0 = 0; i0 < K; i0 += 32) {
        const uint32_t w_next = i0 + 32 < K ? wrow[(i0 >> 5) + 1] : 0u;   // on its way while this word's terms are added
        float4 xv[8];   // the 32 inputs of the word: eight 16-byte loads ahead of the chain of additions
#pragma unroll
        for (int u = 0; u < 8; ++u) xv[u] = *reinterpret_cast<const float4*>(xrow + i0 + 4 * u);
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            sum = __fmaf_rn((w >> (4 * u + 0)) & 1u ? 1.0f : -1.0f, xv[u].x, sum);
            sum = __fmaf_rn((w >> (4 * u + 1)) & 1u ? 1.0f : -1.0f, xv[u].y, sum);
            sum = __fmaf_rn((w >> (4 * u + 2)) & 1u ? 1.0f : -1.0f, xv[u].z, sum);
            sum = __fmaf_rn((w >> (4 * u + 3)) & 1u ? 1.0f : -1.0f, xv[u].w, sum);
        }
        w = w_next;
    }
    const float bv = bias ? h2f(bias[o]) : 0.0f;
    sum = __fadd_rn(bv, __fmul_rn(h2f(scale[o]), sum));
    if (relu2) {
        const float m = fmaxf(sum, 0.0f);
        sum = __fmul_rn(m, m);
    }
    y[r * N + o] = sum;
}

// The same for a dense FP16 matrix with long rows (the CMix value: K = 2048).  One thread per output still adds
// its K products one after the other, but it no longer fetches its own row from global memory (threads of a warp
// 2K bytes apart: 32 sectors per load instruction, and the sum waited for each): the CTA's 64 weight rows come
// through shared memory in pieces of 128 columns, copied asynchronously three pieces ahead with every request
// covering whole 256-byte row pieces.  A row piece is stored with its 16-byte granules permuted by the row
// number, so that the eight lanes of a quarter warp read eight different granules: no bank conflict.
constexpr int RVS_OUT = 64, RVS_KC = 128, RVS_STAGES = 4;
constexpr size_t RVS_STAGE_BYTES = (size_t)RVS_OUT * RVS_KC * 2;

__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__global__ void __launch_bounds__(RVS_OUT)
rowvec_fp16_staged_kernel(const float* __restrict__ x, const uint16_t* __restrict__ w, float* __restrict__ y, size_t K,
                          size_t N, int accumulate) {
    extern __shared__ __align__(16) uint8_t rvs_smem[];
    uint8_t* tiles = rvs_smem;                                                     // RVS_STAGES pieces
    float* xrow = reinterpret_cast<float*>(rvs_smem + RVS_STAGES * RVS_STAGE_BYTES);   // K floats
    const size_t r = blockIdx.y, o0 = (size_t)blockIdx.x * RVS_OUT;
    const int t = threadIdx.x;
    const uint32_t pieces = (uint32_t)(K / RVS_KC);
    auto fetch = [&](uint32_t piece) {
        uint8_t* dst = tiles + (piece % RVS_STAGES) * RVS_STAGE_BYTES;
#pragma unroll
        for (int i = 0; i < RVS_KC / 8 * RVS_OUT / RVS_OUT; ++i) {   // 16 granules of 16 bytes per row, 64 rows: 16 per thread
            const int idx = t + RVS_OUT * i, row = idx >> 4, g = idx & 15;
            cp_async_16(dst + row * (RVS_KC * 2) + ((g ^ (row & 7)) << 4),
                        w + (o0 + row) * K + (size_t)piece * RVS_KC + g * 8);
        }
    };
    for (uint32_t pc = 0; pc < RVS_STAGES - 1 && pc < pieces; ++pc) { fetch(pc); cp_async_commit(); }
    for (size_t i = t; i < K; i += RVS_OUT) xrow[i] = x[r * K + i];
    float sum = 0.0f;
    for (uint32_t pc = 0; pc < pieces; ++pc) {
        // exactly one group is committed per round (an empty one at the end), so "all but the newest
        // RVS_STAGES - 2 groups have landed" always means: piece pc is here
        if (pc + RVS_STAGES - 1 < pieces) fetch(pc + RVS_STAGES - 1);
        cp_async_commit();
        cp_async_wait<RVS_STAGES - 1>();
        __syncthreads();   // everybody's copies of piece pc (and, the first time, the x row)
        const uint8_t* row = tiles + (pc % RVS_STAGES) * RVS_STAGE_BYTES + t * (RVS_KC * 2);
        const float* xs = xrow + (size_t)pc * RVS_KC;
#pragma unroll 4
        for (int g = 0; g < RVS_KC / 8; ++g) {
            const uint4 w8 = *reinterpret_cast<const uint4*>(row + ((g ^ (t & 7)) << 4));
            const uint32_t ww[4] = {w8.x, w8.y, w8.z, w8.w};
            const float4 xa = *reinterpret_cast<const float4*>(xs + g * 8), xb = *reinterpret_cast<const float4*>(xs + g * 8 + 4);
            const float xe[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
            for (int e = 0; e < 8; ++e) {   // i ascending, as the reference adds (src/model.rs:419-436)
                const uint16_t hb = (uint16_t)(e & 1 ? ww[e >> 1] >> 16 : ww[e >> 1] & 0xFFFFu);
                sum = __fadd_rn(sum, __fmul_rn(h2f(hb), xe[e]));
            }
        }
        __syncthreads();   // the piece's buffer is refilled RVS_STAGES - 1 rounds later at the earliest: next round
    }
    float* dst = y + r * N + o0 + t;
    *dst = accumulate ? __fadd_rn(*dst, sum) : sum;
}

}  // namespace

void rowvec_prepare(ullis_cuda_runtime* rt) {
    if (rt->rowvec_smem_ready) return;   // the attribute belongs to the function and the device: always the same value
    ULLIS_CUDA_CHECK(cudaFuncSetAttribute(rowvec_fp16_staged_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int)(RVS_STAGES * RVS_STAGE_BYTES + ROWVEC_MAX_K * 4)));
    rt->rowvec_smem_ready = true;
}

bool binary_rowvec_multi(ullis_cuda_runtime* rt, int count, const float* const* x, const uint32_t* const* bits,
                         const uint16_t* const* scale, const uint16_t* const* bias, float* const* y, size_t rows,
                         size_t in_features, size_t out_features, bool relu2) {
    if (count < 1 || count > 3 || rows == 0 || rows > ROWVEC_MAX_ROWS || in_features > ROWVEC_MAX_K || in_features % 32 ||
        out_features == 0)
        return false;
    RowvecSet set{};
    for (int z = 0; z < count; ++z) {
        set.x[z] = x[z]; set.bits[z] = bits[z]; set.scale[z] = scale[z]; set.bias[z] = bias[z]; set.y[z] = y[z];
    }
    dim3 g((unsigned)((out_features + 127) / 128), (unsigned)rows, (unsigned)count);
    rowvec_packed_multi_kernel<<<g, 128, in_features * 4, rt->stream>>>(set, in_features, out_features, relu2 ? 1 : 0);
    rt->launched("binary_rowvec_exact");
    return true;
}

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
    if (rows <= ROWVEC_MAX_ROWS && in_features <= ROWVEC_MAX_K && in_features % RVS_KC == 0 && in_features >= 4 * RVS_KC &&
        out_features % RVS_OUT == 0 && reinterpret_cast<uintptr_t>(w) % 16 == 0) {
        const size_t smem = RVS_STAGES * RVS_STAGE_BYTES + in_features * 4;
        rowvec_prepare(rt);
        dim3 g((unsigned)(out_features / RVS_OUT), (unsigned)rows);
        rowvec_fp16_staged_kernel<<<g, RVS_OUT, smem, rt->stream>>>(x, w, y, in_features, out_features, accumulate ? 1 : 0);
        rt->launched("fp16_rowvec_exact");
        return;
    }
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
