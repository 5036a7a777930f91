// Host side of the tensor-core stages: TMA descriptors, the small kernels that
// prepare 16-bit operands (time-shift mixes with a hi+lo FP16 split, +/-e
// emit, f32 -> 16-bit casts), the exact fix-up of sign bits that fall inside
// the tensor-core error band, the CE finishing reduction, and the launch of
// the tcgen05 GEMM (tc_gemm.cuh) with the epilogue each stage needs.
#include "linear_tc.hpp"

#include <cudaTypedefs.h>

#include <algorithm>
#include <cstring>

#include "kernels.hpp"
#include "tc_gemm.cuh"
#include "tc_gemm_ws.cuh"
#include "tc_gemm_ws2.cuh"

namespace ullis {
namespace tc {

namespace {

// ------------------------------------------------------------ TMA descriptors
PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
    static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        ULLIS_CUDA_CHECK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q));
        if (!p || q != cudaDriverEntryPointSuccess) fail(ULLIS_CUDA_ERR_CUDA, "cuTensorMapEncodeTiled is unavailable");
        fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
    }
    return fn;
}

// [rows, K] 16-bit row-major matrix, 64 x 128 boxes, 128-byte swizzle, zero fill
CUtensorMap make_map(const void* ptr, size_t rows, size_t K, bool bf16) {
    CUtensorMap m;
    cuuint64_t dims[2] = {K, rows};
    cuuint64_t strides[1] = {K * 2};
    cuuint32_t box[2] = {BK, BM};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = encode_fn()(&m, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                             const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) fail(ULLIS_CUDA_ERR_CUDA, "cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
    return m;
}

__device__ __forceinline__ float h2f(uint16_t b) { return __half2float(__ushort_as_half(b)); }

// ------------------------------------------------------------ operand kernels
// f32 -> f16 / bf16
// (FP16 ends at 65504: a larger finite input is reported through the status word, not turned into inf)
__global__ void cast16_kernel(const float* __restrict__ x, uint16_t* __restrict__ y, size_t n, int bf16, size_t K,
                              uint32_t* __restrict__ status) {
    size_t e = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (e >= n) return;
    float v[4];
    for (int k = 0; k < 4; ++k) v[k] = e + k < n ? x[e + k] : 0.0f;
    for (int k = 0; k < 4; ++k) {
        if (e + k >= n) break;
        if (!bf16 && fabsf(v[k]) > 65504.0f && fabsf(v[k]) <= 3.4028234e38f &&
            atomicCAS(status, ULLIS_DEV_OK, ULLIS_DEV_FP16_RANGE) == ULLIS_DEV_OK)
            status[1] = (uint32_t)((e + k) / K);
        y[e + k] = bf16 ? __bfloat16_as_ushort(__float2bfloat16_rn(v[k])) : __half_as_ushort(__float2half_rn(v[k]));
    }
}

// Time-shift mixes of one LayerNorm output (reference src/model.rs:1291-1298:
// in = x + (x[t-1]-x[t])*mix, unfused) written as FP16 hi and lo = FP16(in - hi)
// for up to three mixes, plus the row's sum |in| that scales the sign-bit error
// band. One warp per row.
__global__ void __launch_bounds__(256)
mix_split_kernel(const float* __restrict__ x, const uint16_t* __restrict__ m0, const uint16_t* __restrict__ m1,
                 const uint16_t* __restrict__ m2, uint16_t* __restrict__ hi0, uint16_t* __restrict__ lo0,
                 uint16_t* __restrict__ hi1, uint16_t* __restrict__ lo1, uint16_t* __restrict__ hi2,
                 uint16_t* __restrict__ lo2, float* __restrict__ s1, size_t rows, size_t time, size_t C) {
    const int lane = threadIdx.x & 31;
    const size_t row = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const bool first = row % time == 0;
    const uint16_t* mix[3] = {m0, m1, m2};
    uint16_t* hi[3] = {hi0, hi1, hi2};
    uint16_t* lo[3] = {lo0, lo1, lo2};
    float sum[3] = {0.0f, 0.0f, 0.0f};
    // four channels per lane and step (C % 4 == 0 on this path): 16-byte loads, 8-byte stores
    for (size_t c = (size_t)lane * 4; c < C; c += 128) {
        const float4 cur = *reinterpret_cast<const float4*>(x + row * C + c);
        float4 prev = make_float4(0.f, 0.f, 0.f, 0.f);
        if (!first) prev = *reinterpret_cast<const float4*>(x + (row - 1) * C + c);
        const float xt[4] = {cur.x, cur.y, cur.z, cur.w}, pt[4] = {prev.x, prev.y, prev.z, prev.w};
        float xx[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) xx[e] = first ? -xt[e] : __fsub_rn(pt[e], xt[e]);
#pragma unroll
        for (int k = 0; k < 3; ++k) {
            if (!mix[k]) continue;
            const uint2 mw = *reinterpret_cast<const uint2*>(mix[k] + c);
            const uint16_t mb[4] = {(uint16_t)(mw.x & 0xFFFFu), (uint16_t)(mw.x >> 16), (uint16_t)(mw.y & 0xFFFFu),
                                    (uint16_t)(mw.y >> 16)};
            uint16_t hb[4], lb[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float v = __fadd_rn(xt[e], __fmul_rn(xx[e], h2f(mb[e])));
                const __half h = __float2half_rn(v);
                hb[e] = __half_as_ushort(h);
                lb[e] = __half_as_ushort(__float2half_rn(v - __half2float(h)));
                sum[k] += fabsf(v);
            }
            *reinterpret_cast<uint2*>(hi[k] + row * C + c) =
                make_uint2(hb[0] | ((uint32_t)hb[1] << 16), hb[2] | ((uint32_t)hb[3] << 16));
            if (lo[k])
                *reinterpret_cast<uint2*>(lo[k] + row * C + c) =
                    make_uint2(lb[0] | ((uint32_t)lb[1] << 16), lb[2] | ((uint32_t)lb[3] << 16));
        }
    }
    if (s1) {
#pragma unroll
        for (int k = 0; k < 3; ++k) {
            float s = sum[k];
            for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
            if (lane == 0 && mix[k]) s1[k * rows + row] = s;
        }
    }
}

// LayerNorm and mix_split_kernel in one pass over the residual stream: a warp normalises its row and the row
// before it (the same arithmetic as the stand-alone warp LayerNorm, so both warps that need a row get the same
// values), forms the mixes and writes the 16-bit operands; the LayerNorm output itself is only written when
// something downstream reads it as f32 (`ln_out`: the exact sign fix-up).  Saves the round trip of the
// LayerNorm output through HBM.  C = 128 * VEC channels, VEC <= 8.
template <int VEC, int ROWS>
__global__ void __launch_bounds__(256)
ln_mix_split_kernel(const float* __restrict__ x, const uint16_t* __restrict__ lw, const uint16_t* __restrict__ lb,
                    float* __restrict__ ln_out, const uint16_t* __restrict__ m0, const uint16_t* __restrict__ m1,
                    const uint16_t* __restrict__ m2, uint16_t* __restrict__ hi0, uint16_t* __restrict__ lo0,
                    uint16_t* __restrict__ hi1, uint16_t* __restrict__ lo1, uint16_t* __restrict__ hi2,
                    uint16_t* __restrict__ lo2, float* __restrict__ s1, size_t rows, size_t time) {
    constexpr int C = 128 * VEC;
    const int lane = threadIdx.x & 31;
    // a warp takes ROWS consecutive rows: the LayerNorm of a row is then computed once and handed on as the next
    // row's "row before" (with ROWS = 1 every row is normalised twice, by its own warp and by its successor's)
    const size_t row0 = ((size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * ROWS;
    if (row0 >= rows) return;
    const uint2* w4 = reinterpret_cast<const uint2*>(lw);
    const uint2* b4 = reinterpret_cast<const uint2*>(lb);
    // normalised values of one row, in place
    auto layer_norm_row = [&](float4 (&v)[VEC]) {
        float sum = 0.0f;
#pragma unroll
        for (int i = 0; i < VEC; ++i) sum += (v[i].x + v[i].y) + (v[i].z + v[i].w);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        const float mean = sum / (float)C;
        float sq = 0.0f;
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
            float a = v[i].x - mean, bb = v[i].y - mean, c = v[i].z - mean, d = v[i].w - mean;
            sq += (a * a + bb * bb) + (c * c + d * d);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
        const float inv = 1.0f / sqrtf(sq / (float)C + 1e-5f);
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
            const uint2 wb = w4[lane + 32 * i], bb = b4[lane + 32 * i];
            v[i].x = (v[i].x - mean) * inv * h2f((uint16_t)(wb.x & 0xffff)) + h2f((uint16_t)(bb.x & 0xffff));
            v[i].y = (v[i].y - mean) * inv * h2f((uint16_t)(wb.x >> 16)) + h2f((uint16_t)(bb.x >> 16));
            v[i].z = (v[i].z - mean) * inv * h2f((uint16_t)(wb.y & 0xffff)) + h2f((uint16_t)(bb.y & 0xffff));
            v[i].w = (v[i].w - mean) * inv * h2f((uint16_t)(wb.y >> 16)) + h2f((uint16_t)(bb.y >> 16));
        }
    };
    float4 cur[VEC], prev[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) prev[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    const uint16_t* mix[3] = {m0, m1, m2};
    uint16_t* hi[3] = {hi0, hi1, hi2};
    uint16_t* lo[3] = {lo0, lo1, lo2};
#pragma unroll 1
    for (int r = 0; r < ROWS; ++r) {
    const size_t row = row0 + r;
    if (row >= rows) break;
    const bool first = row % time == 0;   // the same for the whole warp
    const float4* src = reinterpret_cast<const float4*>(x + row * C);
#pragma unroll
    for (int i = 0; i < VEC; ++i) cur[i] = src[lane + 32 * i];
    if (r == 0 && !first) {
#pragma unroll
        for (int i = 0; i < VEC; ++i) prev[i] = (src - C / 4)[lane + 32 * i];
        layer_norm_row(prev);
    }
    layer_norm_row(cur);
    if (ln_out) {
        float4* dst = reinterpret_cast<float4*>(ln_out + row * C);
#pragma unroll
        for (int i = 0; i < VEC; ++i) dst[lane + 32 * i] = cur[i];
    }
    float sum[3] = {0.0f, 0.0f, 0.0f};
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
        const size_t c = (size_t)(lane + 32 * i) * 4;
        const float xt[4] = {cur[i].x, cur[i].y, cur[i].z, cur[i].w}, pt[4] = {prev[i].x, prev[i].y, prev[i].z, prev[i].w};
        float xx[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) xx[e] = first ? -xt[e] : __fsub_rn(pt[e], xt[e]);
#pragma unroll
        for (int k = 0; k < 3; ++k) {
            if (!mix[k]) continue;
            const uint2 mw = *reinterpret_cast<const uint2*>(mix[k] + c);
            const uint16_t mb[4] = {(uint16_t)(mw.x & 0xFFFFu), (uint16_t)(mw.x >> 16), (uint16_t)(mw.y & 0xFFFFu),
                                    (uint16_t)(mw.y >> 16)};
            uint16_t hb[4], lbt[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float v = __fadd_rn(xt[e], __fmul_rn(xx[e], h2f(mb[e])));
                const __half h = __float2half_rn(v);
                hb[e] = __half_as_ushort(h);
                lbt[e] = __half_as_ushort(__float2half_rn(v - __half2float(h)));
                sum[k] += fabsf(v);
            }
            *reinterpret_cast<uint2*>(hi[k] + row * C + c) =
                make_uint2(hb[0] | ((uint32_t)hb[1] << 16), hb[2] | ((uint32_t)hb[3] << 16));
            if (lo[k])
                *reinterpret_cast<uint2*>(lo[k] + row * C + c) =
                    make_uint2(lbt[0] | ((uint32_t)lbt[1] << 16), lbt[2] | ((uint32_t)lbt[3] << 16));
        }
    }
    if (s1) {
#pragma unroll
        for (int k = 0; k < 3; ++k) {
            float s = sum[k];
            for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
            if (lane == 0 && mix[k]) s1[k * rows + row] = s;
        }
    }
#pragma unroll
    for (int i = 0; i < VEC; ++i) prev[i] = cur[i];
    }
}

// idx bits (stream-major) -> y = +/-e as FP16 [B*T, C] (reference src/model.rs:1313)
// One CTA: 32 steps x 256 channels; a thread writes eight channels (16 bytes) of four steps.
__global__ void __launch_bounds__(256)
emit_f16_kernel(const uint32_t* __restrict__ idx_sw, const uint16_t* __restrict__ e, uint16_t* __restrict__ y,
                size_t T, size_t C, size_t wps) {
    __shared__ __align__(16) uint32_t wsm[256];
    const size_t b = blockIdx.z, t0 = (size_t)blockIdx.x * 32, c0 = (size_t)blockIdx.y * 256;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    wsm[threadIdx.x] = (c0 + threadIdx.x < C) ? idx_sw[(b * C + c0 + threadIdx.x) * wps + blockIdx.x] : 0u;
    __syncthreads();
    const size_t c = c0 + (size_t)tx * 8;
    if (c >= C) return;   // C % 8 == 0 on this path
    const uint4 ev = *reinterpret_cast<const uint4*>(e + c);
    const uint32_t eb[8] = {ev.x & 0xFFFFu, ev.x >> 16, ev.y & 0xFFFFu, ev.y >> 16,
                            ev.z & 0xFFFFu, ev.z >> 16, ev.w & 0xFFFFu, ev.w >> 16};
    const uint4 wa = reinterpret_cast<const uint4*>(wsm)[tx * 2], wb = reinterpret_cast<const uint4*>(wsm)[tx * 2 + 1];
    const uint32_t words[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const uint32_t tt = ty * 4 + k;
        if (t0 + tt >= T) break;
        uint32_t h[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) h[j] = eb[j] ^ (((words[j] >> tt) & 1u) ? 0u : 0x8000u);  // flip the FP16 sign for idx 0
        *reinterpret_cast<uint4*>(y + (b * T + t0 + tt) * C + c) =
            make_uint4(h[0] | (h[1] << 16), h[2] | (h[3] << 16), h[4] | (h[5] << 16), h[6] | (h[7] << 16));
    }
}

// Exact pre-activation sign of one output of a packed linear over the time-shift mix of x, as the reference
// computes it (src/model.rs:1291-1298 then 724-742): in_i = x_i + (x[t-1]_i - x_i) * mix_i (unfused), the sum of
// +/- in_i for i ascending in f32, then bias + scale * sum.  R inputs per round: the 2R/4 row loads of a round go
// out together, then the sum is taken in order.
template <int R>
__device__ __forceinline__ bool exact_mixed_sign(const float* __restrict__ xr, bool first_step,
                                                 const uint16_t* __restrict__ mix, const uint32_t* __restrict__ wbits,
                                                 float scale, float bias, size_t C) {
    float sum = 0.0f;
    for (size_t i0 = 0; i0 < C; i0 += R) {
        float4 cur[R / 4], prev[R / 4];
#pragma unroll
        for (int u = 0; u < R / 4; ++u) {
            cur[u] = *reinterpret_cast<const float4*>(xr + i0 + 4 * u);
            prev[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (!first_step) prev[u] = *reinterpret_cast<const float4*>(xr - C + i0 + 4 * u);
        }
        const uint32_t wword = wbits[i0 >> 5] >> (i0 & 31);
#pragma unroll
        for (int u = 0; u < R / 4; ++u) {
            const float xs[4] = {cur[u].x, cur[u].y, cur[u].z, cur[u].w};
            const float ps[4] = {prev[u].x, prev[u].y, prev[u].z, prev[u].w};
            const uint2 mw = *reinterpret_cast<const uint2*>(mix + i0 + 4 * u);
            const uint16_t mb[4] = {(uint16_t)(mw.x & 0xFFFFu), (uint16_t)(mw.x >> 16), (uint16_t)(mw.y & 0xFFFFu),
                                    (uint16_t)(mw.y >> 16)};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float xt = xs[k];
                const float xx = first_step ? -xt : __fsub_rn(ps[k], xt);
                const float in = __fadd_rn(xt, __fmul_rn(xx, h2f(mb[k])));
                sum = __fmaf_rn((wword >> (4 * u + k)) & 1u ? 1.0f : -1.0f, in, sum);
            }
        }
    }
    return __fadd_rn(bias, __fmul_rn(scale, sum)) > 0.0f;
}

// The flagged outputs of one Q/K/V launch as a compact list, so that the exact recomputation runs over the whole
// device instead of a few busy threads per window.  An entry names the sign bit to redo: (index of its word among
// the 3 * sw stream-major bit words of the launch) * 32 + bit.  A warp takes one (sequence, block of 32 steps, matrix) at
// a time, reads that block's flag word of every channel and appends all the bits it found with ONE addition to the
// list's counter (an addition per word would queue a hundred thousand of them on one address).  Entries of a
// block lie together in the list and read the same 33 rows of x.  More flags than the list holds (never on
// realistic inputs: the list takes one output in 64) raise `ctrl[1]`, and the window kernel below then redoes the
// whole launch.  C <= 32 * FIXQ_MAX_WORDS channels.
constexpr int FIXQ_MAX_WORDS = 32;
__global__ void __launch_bounds__(256)
fix_collect_kernel(const uint32_t* __restrict__ flags, size_t sw, size_t batch, size_t C, size_t wps,
                   uint32_t* __restrict__ list, uint32_t cap, uint32_t* __restrict__ ctrl) {
    const int lane = threadIdx.x & 31;
    const size_t warps = ((size_t)gridDim.x * blockDim.x) >> 5;
    const size_t buckets = batch * wps * 3;
    const int rounds = (int)((C + 31) / 32);
    for (size_t bk = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; bk < buckets; bk += warps) {
        const size_t m = bk % 3, word = (bk / 3) % wps, b = bk / (3 * wps);
        const size_t base = m * sw + b * C * wps + word;     // bit word of channel ch: base + ch * wps (stream-major)
        const uint32_t* fl = flags + m * sw + (b * wps + word) * C;   // its flag word: fl[ch] (channels side by side)
        uint32_t f[FIXQ_MAX_WORDS];
        uint32_t mine = 0;
#pragma unroll
        for (int r = 0; r < FIXQ_MAX_WORDS; ++r) {
            const size_t ch = (size_t)r * 32 + lane;
            f[r] = (r < rounds && ch < C) ? fl[ch] : 0u;
            mine += __popc(f[r]);
        }
        uint32_t incl = mine;                                  // inclusive prefix sum over the lanes
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t up = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += up;
        }
        const uint32_t total = __shfl_sync(0xffffffffu, incl, 31);
        if (total == 0) continue;
        uint32_t at = 0;
        if (lane == 31) at = atomicAdd(&ctrl[0], total);
        at = __shfl_sync(0xffffffffu, at, 31);
        if (at + total > cap) {
            if (lane == 0) ctrl[1] = 1u;
            continue;
        }
        at += incl - mine;
#pragma unroll
        for (int r = 0; r < FIXQ_MAX_WORDS; ++r) {
            uint32_t g = f[r];
            while (g) {
                const uint32_t tt = __ffs(g) - 1;
                g &= g - 1;
                list[at++] = (uint32_t)(base + ((size_t)r * 32 + lane) * wps) * 32u + tt;
            }
        }
    }
}

// The exact recomputation of the listed outputs, a warp for 32 entries at a time.  The terms +/- in_i of an
// output have to be added one after the other in f32 (that order is what makes the sign exact), which only a
// single thread can do; everything before it is shared: for 128 input columns at a time the whole warp loads the
// rows of one entry after the other side by side (512 bytes per request instead of 32 requests into 32 rows),
// forms the signed terms and leaves them in shared memory, and then lane e adds up the 128 terms of entry e.
constexpr int FIXQ_WARPS = 2, FIXQ_COLS = 128, FIXQ_PITCH = FIXQ_COLS + 1, FIXQ_BATCH = 8;

__global__ void __launch_bounds__(FIXQ_WARPS * 32)
fix_apply_kernel(const float* __restrict__ x, const uint16_t* __restrict__ mq, const uint16_t* __restrict__ mk,
                 const uint16_t* __restrict__ mv, PackedWeights wq, PackedWeights wk, PackedWeights wv,
                 uint32_t* __restrict__ bq, uint32_t* __restrict__ bk, uint32_t* __restrict__ bv,
                 const uint32_t* __restrict__ list, uint32_t cap, const uint32_t* __restrict__ ctrl, size_t sw, size_t T,
                 size_t C, size_t wps) {
    __shared__ float terms[FIXQ_WARPS][32 * FIXQ_PITCH];
    // what the whole warp needs to know about entry e, written by lane e once per task
    __shared__ const float* e_row[FIXQ_WARPS][32];
    __shared__ const uint32_t* e_w[FIXQ_WARPS][32];
    __shared__ const uint16_t* e_mix[FIXQ_WARPS][32];
    __shared__ uint32_t e_flags[FIXQ_WARPS][32];   // 1: first step of its sequence (no row before it)
    if (ctrl[1]) return;   // the list overflowed: the window kernel redoes everything
    const uint32_t count = min(ctrl[0], cap);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float* mine = terms[warp];
    const uint32_t tasks = (count + 31u) / 32u;
    for (uint32_t task = blockIdx.x * FIXQ_WARPS + warp; task < tasks; task += gridDim.x * FIXQ_WARPS) {
        const uint32_t i = task * 32u + lane;
        const bool live = i < count;
        const uint32_t entry = live ? list[i] : 0u, tt = entry & 31u;
        const size_t wi = entry >> 5, m = wi / sw, rem = wi % sw;
        const size_t s = rem / wps, word = rem % wps, b = s / C, ch = s % C, t = word * 32 + tt;
        const PackedWeights& W = m == 0 ? wq : m == 1 ? wk : wv;
        // a lane without an entry (the tail of the list) stands in with row 0 of x: every load below is then
        // unconditional, and only the final write looks at `live`
        e_row[warp][lane] = live ? x + (b * T + t) * C : x;
        e_w[warp][lane] = W.bits + (ch * C >> 5);               // C % 32 == 0 on this path
        e_mix[warp][lane] = m == 0 ? mq : m == 1 ? mk : mv;
        e_flags[warp][lane] = (t == 0 || !live) ? 1u : 0u;     // 1: no row before it
        __syncwarp();
        float sum = 0.0f;
        for (size_t i0 = 0; i0 < C; i0 += FIXQ_COLS) {
            const size_t c = i0 + 4 * lane;
            // FIXQ_BATCH entries at a time: first every load of the batch (they do not depend on each other, and the
            // compiler will not move a load above a store to shared memory by itself), then the arithmetic
            for (int e0 = 0; e0 < 32; e0 += FIXQ_BATCH) {
                float4 cur[FIXQ_BATCH], prev[FIXQ_BATCH];
                uint2 mw[FIXQ_BATCH];
                uint32_t ww[FIXQ_BATCH], fl[FIXQ_BATCH];
#pragma unroll
                for (int u = 0; u < FIXQ_BATCH; ++u) {
                    const int e = e0 + u;
                    fl[u] = e_flags[warp][e];
                    const float* row = e_row[warp][e];
                    cur[u] = *reinterpret_cast<const float4*>(row + c);
                    // the row before it, or (first step of a sequence) the row itself: its value is not used then
                    prev[u] = *reinterpret_cast<const float4*>((fl[u] & 1u) ? row + c : row - C + c);
                    mw[u] = *reinterpret_cast<const uint2*>(e_mix[warp][e] + c);
                    ww[u] = e_w[warp][e][c >> 5] >> (c & 31);
                }
#pragma unroll
                for (int u = 0; u < FIXQ_BATCH; ++u) {
                    const int e = e0 + u;
                    const bool first_step = (fl[u] & 1u) != 0;
                    const float xs[4] = {cur[u].x, cur[u].y, cur[u].z, cur[u].w};
                    const float ps[4] = {prev[u].x, prev[u].y, prev[u].z, prev[u].w};
                    const uint16_t mb[4] = {(uint16_t)(mw[u].x & 0xFFFFu), (uint16_t)(mw[u].x >> 16),
                                            (uint16_t)(mw[u].y & 0xFFFFu), (uint16_t)(mw[u].y >> 16)};
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const float xx = first_step ? -xs[k] : __fsub_rn(ps[k], xs[k]);
                        const float in = __fadd_rn(xs[k], __fmul_rn(xx, h2f(mb[k])));
                        // column 4 * lane + k of the chunk is kept at k * 32 + lane: no bank conflict here (lanes side
                        // by side) nor in the sums below (rows 129 words apart)
                        mine[e * FIXQ_PITCH + k * 32 + lane] = ((ww[u] >> k) & 1u) ? in : -in;
                    }
                }
            }
            __syncwarp();
            if (live) {
#pragma unroll 8
                for (int k = 0; k < FIXQ_COLS; ++k)   // i ascending
                    sum = __fadd_rn(sum, mine[lane * FIXQ_PITCH + (k & 3) * 32 + (k >> 2)]);
            }
            __syncwarp();
        }
        if (live) {
            const float y = __fadd_rn(W.bias ? h2f(W.bias[ch]) : 0.0f, __fmul_rn(h2f(W.scale[ch]), sum));
            uint32_t* bits = m == 0 ? bq : m == 1 ? bk : bv;
            if (y > 0.0f) atomicOr(&bits[rem], 1u << tt); else atomicAnd(&bits[rem], ~(1u << tt));
        }
        __syncwarp();   // the entry table is rewritten by the next task
    }
}

// Sign bits whose tensor-core pre-activation fell inside the error band are
// recomputed exactly as the reference does (src/model.rs:724-742 on the
// time-shift mix of x): sequential f32 sum over i, then bias + scale*sum.
// Flags are sparse (a few per thousand).  A CTA owns a window of 64 steps of
// one sequence for ALL channels of Q, K and V, so the 65 rows of x its exact
// dot products read stay in L1 / L2 and every row is fetched from HBM about
// once per launch; it gathers the flagged (matrix, channel, step) triples into
// a shared queue and spreads them over its threads, one dot product each.
constexpr int FIX_THREADS = 256, FIX_WIN = 2 /* flag words (of 32 steps) per window */, FIX_QUEUE = 12288, FIX_BATCH = 8;
static_assert(FIX_QUEUE >= FIX_THREADS * 32, "the flag bits of one word per thread must fit the queue");

__global__ void __launch_bounds__(FIX_THREADS)
sign_fixup_kernel(const float* __restrict__ x, const uint16_t* __restrict__ mq, const uint16_t* __restrict__ mk,
                  const uint16_t* __restrict__ mv, PackedWeights wq, PackedWeights wk, PackedWeights wv,
                  uint32_t* __restrict__ bq, uint32_t* __restrict__ bk, uint32_t* __restrict__ bv,
                  const uint32_t* __restrict__ fq, const uint32_t* __restrict__ fk, const uint32_t* __restrict__ fv,
                  size_t batch, size_t T, size_t C, size_t wps, const uint32_t* __restrict__ only_if) {
    if (only_if && *only_if == 0u) return;   // the compact list took every flag: nothing left for the windows
    extern __shared__ uint32_t fix_queue[];  // entries: matrix << 28 | channel << 8 | word in window << 5 | bit
    __shared__ uint32_t q_count, announced;   // entries queued; flag bits announced so far (never reset)
    const size_t windows = (wps + FIX_WIN - 1) / FIX_WIN;
    const size_t b = blockIdx.x / windows, w0 = (blockIdx.x % windows) * FIX_WIN;
    const uint32_t per_matrix = (uint32_t)C * FIX_WIN, items = 3u * per_matrix;
    if (threadIdx.x == 0) { q_count = 0; announced = 0; }
    __syncthreads();

    // one exact dot product per queued entry, spread over the CTA's threads; empties the queue
    auto drain = [&]() {
        __syncthreads();
        const uint32_t count = q_count;
        for (uint32_t i = threadIdx.x; i < count; i += FIX_THREADS) {
            const uint32_t entry = fix_queue[i], tt = entry & 31u, m = entry >> 28;
            const size_t ch = (entry >> 8) & 0xFFFFFu, word = w0 + ((entry >> 5) & 7u);
            const size_t ew = (b * C + ch) * wps + word;
            const size_t t = word * 32 + tt, row = b * T + t;
            const float* xr = x + row * C;
            const uint16_t* mix = m == 0 ? mq : m == 1 ? mk : mv;
            const uint32_t* wb = m == 0 ? wq.bits : m == 1 ? wk.bits : wv.bits;
            const uint16_t* wscale = m == 0 ? wq.scale : m == 1 ? wk.scale : wv.scale;
            const uint16_t* wbias = m == 0 ? wq.bias : m == 1 ? wk.bias : wv.bias;
            uint32_t* bits = m == 0 ? bq : m == 1 ? bk : bv;
            const uint32_t* wbits = wb + (ch * C >> 5);  // C % 32 == 0 on this path
            const bool plus = exact_mixed_sign<32>(xr, t == 0, mix, wbits, h2f(wscale[ch]), wbias ? h2f(wbias[ch]) : 0.0f, C);
            if (plus) atomicOr(&bits[ew], 1u << tt); else atomicAnd(&bits[ew], ~(1u << tt));
        }
        __syncthreads();
        if (threadIdx.x == 0) q_count = 0;
        __syncthreads();
    };
    auto push = [&](uint32_t f, uint32_t it) {
        const uint32_t which = it / per_matrix, rem = it % per_matrix;
        const uint32_t at = atomicAdd(&q_count, (uint32_t)__popc(f));
        uint32_t k = 0;
        while (f) {
            const uint32_t tt = __ffs(f) - 1;
            f &= f - 1;
            fix_queue[at + k++] = which << 28 | (rem / FIX_WIN) << 8 | (rem % FIX_WIN) << 5 | tt;
        }
    };

    // Flag words are read FIX_BATCH per thread at a time, all loads in flight together; the CTA first
    // announces how many bits the batch holds so that every thread takes the same decision about the queue.
    uint32_t seen = 0;   // value of `announced` before this batch (the same in every thread)
    for (uint32_t base = 0; base < items; base += FIX_THREADS * FIX_BATCH) {
        uint32_t f[FIX_BATCH], mine = 0;
#pragma unroll
        for (int k = 0; k < FIX_BATCH; ++k) {
            const uint32_t it = base + k * FIX_THREADS + threadIdx.x;
            f[k] = 0;
            if (it < items) {
                const uint32_t which = it / per_matrix, rem = it % per_matrix;
                const uint32_t* flags = which == 0 ? fq : which == 1 ? fk : fv;
                const size_t word = w0 + rem % FIX_WIN;
                if (word < wps) f[k] = flags[(b * wps + word) * C + rem / FIX_WIN];
            }
        }
#pragma unroll
        for (int k = 0; k < FIX_BATCH; ++k) mine += (uint32_t)__popc(f[k]);
        if (mine) atomicAdd(&announced, mine);
        __syncthreads();
        const uint32_t batch_bits = announced - seen, queued = q_count;
        seen = announced;
        __syncthreads();   // everyone has read both counters before either moves again
        if (queued + batch_bits > FIX_QUEUE) drain();
        if (batch_bits <= FIX_QUEUE) {
#pragma unroll
            for (int k = 0; k < FIX_BATCH; ++k)
                if (f[k]) push(f[k], base + k * FIX_THREADS + threadIdx.x);
        } else {   // dense flags: one word per thread at a time (at most 32 * FIX_THREADS entries)
#pragma unroll
            for (int k = 0; k < FIX_BATCH; ++k) {
                if (f[k]) push(f[k], base + k * FIX_THREADS + threadIdx.x);
                drain();
            }
        }
    }
    drain();
}

// Merge the per-tile (max, sum exp) partials of a row and subtract the target
// logit (reference src/model.rs:3219-3227; valid-row rule 27-39).
__global__ void ce_finish_kernel(const float2* __restrict__ part, const float* __restrict__ target_logit,
                                 const uint32_t* __restrict__ labels, uint32_t ignore_id, size_t rows, size_t time,
                                 size_t vocab, uint32_t n_tiles, float* __restrict__ row_loss, uint32_t* status) {
    const size_t m = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (m >= rows) return;
    const bool valid = time != 0 && (m % time) + 1 < time && m + 1 < rows && labels[m + 1] != ignore_id;
    if (!valid) {
        row_loss[m] = 0.0f;
        return;
    }
    if (labels[m + 1] >= vocab) {
        if (atomicCAS(status, ULLIS_DEV_OK, ULLIS_DEV_BAD_TOKEN) == ULLIS_DEV_OK) status[1] = (uint32_t)m;
        row_loss[m] = 0.0f;
        return;
    }
    float gmax = -INFINITY;
    for (uint32_t i = 0; i < n_tiles; ++i) gmax = fmaxf(gmax, part[m * n_tiles + i].x);
    float sum = 0.0f;
    for (uint32_t i = 0; i < n_tiles; ++i) {
        const float2 pr = part[m * n_tiles + i];
        sum += pr.y * expf(pr.x - gmax);
    }
    row_loss[m] = gmax + logf(sum) - target_logit[m];
}

inline unsigned blocks_for(size_t n, unsigned per) { return (unsigned)((n + per - 1) / per); }

}  // namespace

namespace {

// How many CTA pairs of the pair kernel the device holds at once (0 = clusters of two cannot be placed).
template <int EPI, bool RESIDENT_W = true>
int ws2_resident_clusters(ullis_cuda_runtime* rt) {
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.gridDim = dim3(2u * (unsigned)rt->sm_count);
    cfg.blockDim = dim3(WS2_THREADS);
    cfg.dynamicSmemBytes = WS_SMEM_LIMIT;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_ws2_kernel<EPI, RESIDENT_W>, &cfg) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

bool usable(ullis_cuda_runtime* rt) {
    if (rt->mode == ULLIS_CUDA_MODE_EXACT) return false;
    if (rt->tc_ready == 0) {
        rt->tc_ready = -1;
        if (rt->cc_major == 10 && !getenv("ULLIS_CUDA_NO_TC")) {
            encode_fn();
            const int smem = (int)gemm_smem_bytes(2, MAX_STAGES);
#define ULLIS_SET_SMEM(EPI, PACKED) \
    ULLIS_CUDA_CHECK(cudaFuncSetAttribute(gemm_kernel<EPI, PACKED>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem))
            ULLIS_SET_SMEM(EPI_STORE, true);
            ULLIS_SET_SMEM(EPI_STORE, false);
            ULLIS_SET_SMEM(EPI_RESIDUAL, true);
            ULLIS_SET_SMEM(EPI_RESIDUAL, false);
            ULLIS_SET_SMEM(EPI_RELU2, true);
            ULLIS_SET_SMEM(EPI_SIGNBITS, true);
            ULLIS_SET_SMEM(EPI_CE, true);
#undef ULLIS_SET_SMEM
#define ULLIS_SET_SMEM_WS(EPI) \
    ULLIS_CUDA_CHECK(cudaFuncSetAttribute(gemm_ws_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)WS_SMEM_LIMIT))
            ULLIS_SET_SMEM_WS(EPI_STORE);
            ULLIS_SET_SMEM_WS(EPI_RESIDUAL);
            ULLIS_SET_SMEM_WS(EPI_RELU2);
            ULLIS_SET_SMEM_WS(EPI_SIGNBITS);
            ULLIS_SET_SMEM_WS(EPI_CE);
#undef ULLIS_SET_SMEM_WS
            ULLIS_CUDA_CHECK(cudaFuncSetAttribute(gemm_ws_kernel<EPI_STORE, false>,
                                                  cudaFuncAttributeMaxDynamicSharedMemorySize, (int)WS_SMEM_LIMIT));
            ULLIS_CUDA_CHECK(cudaFuncSetAttribute(gemm_ws_kernel<EPI_RESIDUAL, false>,
                                                  cudaFuncAttributeMaxDynamicSharedMemorySize, (int)WS_SMEM_LIMIT));
            rt->tc_ws_kernel = !getenv("ULLIS_CUDA_NO_WS");
#define ULLIS_SET_SMEM_WS2(EPI)                                                                                    \
    ULLIS_CUDA_CHECK(cudaFuncSetAttribute(gemm_ws2_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize,       \
                                          (int)WS_SMEM_LIMIT));                                                    \
    rt->tc_ws2_clusters[EPI] = ws2_resident_clusters<EPI>(rt)
            ULLIS_SET_SMEM_WS2(EPI_STORE);
            ULLIS_SET_SMEM_WS2(EPI_RESIDUAL);
            ULLIS_SET_SMEM_WS2(EPI_RELU2);
            ULLIS_SET_SMEM_WS2(EPI_SIGNBITS);
            ULLIS_SET_SMEM_WS2(EPI_CE);
#undef ULLIS_SET_SMEM_WS2
            ULLIS_CUDA_CHECK(cudaFuncSetAttribute(gemm_ws2_kernel<EPI_STORE, false>,
                                                  cudaFuncAttributeMaxDynamicSharedMemorySize, (int)WS_SMEM_LIMIT));
            ULLIS_CUDA_CHECK(cudaFuncSetAttribute(gemm_ws2_kernel<EPI_RESIDUAL, false>,
                                                  cudaFuncAttributeMaxDynamicSharedMemorySize, (int)WS_SMEM_LIMIT));
            rt->tc_ws2_dense_clusters[0] = ws2_resident_clusters<EPI_STORE, false>(rt);
            rt->tc_ws2_dense_clusters[1] = ws2_resident_clusters<EPI_RESIDUAL, false>(rt);
            rt->tc_ws2_kernel = rt->tc_ws_kernel && !getenv("ULLIS_CUDA_NO_WS2");
            if (const char* env = getenv("ULLIS_CUDA_WS2_MIN_ROWS")) rt->tc_ws2_min_rows = (size_t)std::max(1, atoi(env));
            ULLIS_CUDA_CHECK(cudaFuncSetAttribute(sign_fixup_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                  FIX_QUEUE * 4));
            rt->tc_ready = 1;
        }
    }
    return rt->tc_ready == 1;
}

bool shape_ok(size_t M, size_t K, size_t N) {
    return M > 0 && K >= BK && K % BK == 0 && N >= 8 && N % 8 == 0 && M < (1u << 30) && N < (1u << 30) &&
           (M + BM - 1) / BM <= 65535;
}

// packed weights with a short K go to the weight-stationary kernel
bool takes_ws(const ullis_cuda_runtime* rt, size_t K, uint32_t n_a) {
    return rt->tc_ws_kernel && K / BK <= WS_MAX_KB && ws_shape((uint32_t)K, n_a, true).stages >= 2;
}

// ... and, with enough rows and whole 256-column tiles, to its CTA-pair form
bool takes_ws2(const ullis_cuda_runtime* rt, int epi, size_t M, size_t K, size_t N, uint32_t n_a) {
    return rt->tc_ws2_kernel && takes_ws(rt, K, n_a) && N % WS2_BN == 0 && M >= rt->tc_ws2_min_rows &&
           rt->tc_ws2_clusters[epi] >= 8 && ws2_shape((uint32_t)K, n_a, epi).stages >= 2;
}

// one (problem, 256-column tile) per CTA pair; the pairs with the same one share the 256-row tiles
template <int EPI, bool RESIDENT_W>
void launch_ws2(ullis_cuda_runtime* rt, const GemmMaps& maps, const GemmParams& p, unsigned n_prob, int resident,
                const char* what) {
    const WsShape shape = ws2_shape(p.K, p.n_a, EPI, RESIDENT_W);
    GemmParams q = p;
    q.stages = shape.stages;
    const uint32_t pairs = n_prob * (p.N / WS2_BN), m_tiles = (p.M + WS2_BM - 1) / WS2_BM;
    uint32_t members = (uint32_t)resident / pairs;
    if (members < 1) members = 1;
    if (members > m_tiles) members = m_tiles;
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.gridDim = dim3(2u * pairs * members);
    cfg.blockDim = dim3(WS2_THREADS);
    cfg.dynamicSmemBytes = shape.smem;
    cfg.stream = rt->stream;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    if (rt->kernel_timing) rt->mark("(cta_pair)");   // a zero-length entry in the timing table: which form ran
    ULLIS_CUDA_CHECK(cudaLaunchKernelEx(&cfg, gemm_ws2_kernel<EPI, RESIDENT_W>, maps, q, pairs));
    rt->launched(what);
}

template <int EPI, bool PACKED>
void launch(ullis_cuda_runtime* rt, const GemmMaps& maps, const GemmParams& p, unsigned n_prob, const char* what) {
    if (PACKED && takes_ws2(rt, EPI, p.M, p.K, p.N, p.n_a)) {
        launch_ws2<EPI, true>(rt, maps, p, n_prob, rt->tc_ws2_clusters[EPI], what);
        return;
    }
    if (PACKED && takes_ws(rt, p.K, p.n_a)) {
        // one (problem, column tile) pair per CTA, the CTAs of a pair share the row tiles
        const WsShape shape = ws_shape(p.K, p.n_a, EPI == EPI_STORE || EPI == EPI_RESIDUAL);
        {
            GemmParams q = p;
            q.stages = shape.stages;
            const uint32_t pairs = n_prob * ((p.N + BN - 1) / BN), m_tiles = (p.M + BM - 1) / BM;
            uint32_t members = (uint32_t)rt->sm_count / pairs;
            if (members < 1) members = 1;
            if (members > m_tiles) members = m_tiles;
            gemm_ws_kernel<EPI><<<pairs * members, WS_THREADS, shape.smem, rt->stream>>>(maps, q, pairs);
            rt->launched(what);
            return;
        }
    }
    if constexpr (!PACKED && (EPI == EPI_STORE || EPI == EPI_RESIDUAL)) {
        // dense weights: the persistent kernel with the weight tile in the ring (large M only: a CTA needs
        // several row tiles to amortise its set-up)
        const uint32_t m_tiles = (p.M + BM - 1) / BM, pairs = n_prob * ((p.N + BN - 1) / BN);
        if (rt->tc_ws2_kernel && m_tiles * pairs >= 4u * (uint32_t)rt->sm_count && p.N % WS2_BN == 0 &&
            p.M >= rt->tc_ws2_min_rows && rt->tc_ws2_dense_clusters[EPI] >= 8 &&
            ws2_shape(p.K, p.n_a, EPI, false).stages >= 2) {
            launch_ws2<EPI, false>(rt, maps, p, n_prob, rt->tc_ws2_dense_clusters[EPI], what);
            return;
        }
        if (rt->tc_ws_kernel && m_tiles * pairs >= 4u * (uint32_t)rt->sm_count) {
            const WsShape shape = ws_shape(p.K, p.n_a, true, false);
            GemmParams q = p;
            q.stages = shape.stages;
            uint32_t members = (uint32_t)rt->sm_count / pairs;
            if (members < 1) members = 1;
            if (members > m_tiles) members = m_tiles;
            gemm_ws_kernel<EPI, false><<<pairs * members, WS_THREADS, shape.smem, rt->stream>>>(maps, q, pairs);
            rt->launched(what);
            return;
        }
    }
    dim3 grid((p.N + BN - 1) / BN, (p.M + BM - 1) / BM, n_prob);
    gemm_kernel<EPI, PACKED><<<grid, GEMM_THREADS, gemm_smem_bytes(p.n_a, p.stages), rt->stream>>>(maps, p);
    rt->launched(what);
}

GemmParams base_params(ullis_cuda_runtime* rt, size_t M, size_t N, size_t K) {
    GemmParams p;
    memset(&p, 0, sizeof(p));
    p.M = (uint32_t)M;
    p.N = (uint32_t)N;
    p.K = (uint32_t)K;
    p.n_a = 1;
    p.stages = rt->tc_stages;   // shallow pipeline, several CTAs per SM: one CTA's epilogue runs under another's MMAs
    p.status = rt->dev_status;
    return p;
}

// LayerNorm + mixes + 16-bit operands in one kernel when the width allows (a multiple of 128 up to 1024 channels);
// returns false when it does not, and the caller runs the two kernels one after the other.
bool launch_ln_mix_split(ullis_cuda_runtime* rt, const float* x, const LayerNormWeights& ln, float* ln_out,
                         const uint16_t* m0, const uint16_t* m1, const uint16_t* m2, uint16_t* hi0, uint16_t* lo0,
                         uint16_t* hi1, uint16_t* lo1, uint16_t* hi2, uint16_t* lo2, float* s1, size_t rows, size_t time,
                         size_t d, const char* what) {
    if (!rt->tc_fuse_ln || d % 128 != 0 || d > 1024) return false;
    // rows per warp: several once there are enough rows to fill the device with warps anyway
    // (measured at 131 072 rows: the Q/K/V form, bound by its 0.8 GB of stores, is best with two; the one-operand
    // form, bound by instruction issue, with four)
    const int per_warp = rt->tc_ln_rows > 0 ? rt->tc_ln_rows : rows < 32768 ? 1 : m1 ? 2 : 4;
    const unsigned grid = blocks_for(rows, 8 * (per_warp == 4 ? 4 : per_warp == 2 ? 2 : 1));
#define ULLIS_LN_MIX(V)                                                                                                  \
    do {                                                                                                                 \
        if (per_warp == 4)                                                                                               \
            ln_mix_split_kernel<V, 4><<<grid, 256, 0, rt->stream>>>(x, ln.weight, ln.bias, ln_out, m0, m1, m2, hi0, lo0, \
                                                                    hi1, lo1, hi2, lo2, s1, rows, time);                 \
        else if (per_warp == 2)                                                                                          \
            ln_mix_split_kernel<V, 2><<<grid, 256, 0, rt->stream>>>(x, ln.weight, ln.bias, ln_out, m0, m1, m2, hi0, lo0, \
                                                                    hi1, lo1, hi2, lo2, s1, rows, time);                 \
        else                                                                                                             \
            ln_mix_split_kernel<V, 1><<<grid, 256, 0, rt->stream>>>(x, ln.weight, ln.bias, ln_out, m0, m1, m2, hi0, lo0, \
                                                                    hi1, lo1, hi2, lo2, s1, rows, time);                 \
    } while (0)
    switch (d / 128) {
        case 1: ULLIS_LN_MIX(1); break;
        case 2: ULLIS_LN_MIX(2); break;
        case 3: ULLIS_LN_MIX(3); break;
        case 4: ULLIS_LN_MIX(4); break;
        case 5: ULLIS_LN_MIX(5); break;
        case 6: ULLIS_LN_MIX(6); break;
        case 7: ULLIS_LN_MIX(7); break;
        default: ULLIS_LN_MIX(8); break;
    }
#undef ULLIS_LN_MIX
    rt->launched(what);
    return true;
}

// x [rows, K] f32 -> 16-bit operand
void cast16(ullis_cuda_runtime* rt, const float* x, uint16_t* y, size_t rows, size_t K, bool bf16) {
    const size_t n = rows * K;
    cast16_kernel<<<blocks_for((n + 3) / 4, 256), 256, 0, rt->stream>>>(x, y, n, bf16 ? 1 : 0, K, rt->dev_status);
    rt->launched("cast16");
}

}  // namespace

bool binary_linear(ullis_cuda_runtime* rt, const float* x, const uint32_t* bits, const uint16_t* scale,
                   const uint16_t* bias, float* y, size_t rows, size_t in_features, size_t out_features) {
    if (!usable(rt) || !shape_ok(rows, in_features, out_features) || out_features % 4) return false;
    uint16_t* a = rt->tc_ws[0].as<uint16_t>(rows * in_features);
    cast16(rt, x, a, rows, in_features, false);
    GemmMaps maps;
    memset(&maps, 0, sizeof(maps));
    maps.a[0][0] = make_map(a, rows, in_features, false);
    GemmParams p = base_params(rt, rows, out_features, in_features);
    p.prob[0] = GemmProblem{bits, scale, bias, y, nullptr, nullptr};
    launch<EPI_STORE, true>(rt, maps, p, 1, "gemm_packed_store");
    return true;
}

bool fp16_linear(ullis_cuda_runtime* rt, const float* x, const uint16_t* w, float* y, size_t rows,
                 size_t in_features, size_t out_features) {
    if (!usable(rt) || !shape_ok(rows, in_features, out_features)) return false;
    // both operands FP16: the weights as stored (no second rounding), the activations with 11 significant
    // bits; an activation beyond the FP16 range is reported by cast16
    uint16_t* a = rt->tc_ws[0].as<uint16_t>(rows * in_features);
    cast16(rt, x, a, rows, in_features, false);
    GemmMaps maps;
    memset(&maps, 0, sizeof(maps));
    maps.a[0][0] = make_map(a, rows, in_features, false);
    maps.b[0] = make_map(w, out_features, in_features, false);
    GemmParams p = base_params(rt, rows, out_features, in_features);
    p.prob[0] = GemmProblem{nullptr, nullptr, nullptr, y, nullptr, nullptr};
    launch<EPI_STORE, false>(rt, maps, p, 1, "gemm_dense_store");
    return true;
}

namespace {
// y = sum of the split-K partials, in split order
__global__ void splitk_reduce_kernel(const float* __restrict__ part, float* __restrict__ y, uint32_t splits, size_t n) {
    const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= n) return;   // n % 4 == 0 (N % 8 == 0)
    float4 acc = *reinterpret_cast<const float4*>(part + i);
    for (uint32_t s = 1; s < splits; ++s) {
        const float4 v = *reinterpret_cast<const float4*>(part + (size_t)s * n + i);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    *reinterpret_cast<float4*>(y + i) = acc;
}
}  // namespace

bool dense_nt(ullis_cuda_runtime* rt, const uint16_t* a16, const uint16_t* b16, float* y, size_t M, size_t K,
              size_t N) {
    if (!usable(rt) || !shape_ok(M, K, N)) return false;
    GemmMaps maps;
    memset(&maps, 0, sizeof(maps));
    maps.a[0][0] = make_map(a16, M, K, false);
    maps.b[0] = make_map(b16, N, K, false);
    GemmParams p = base_params(rt, M, N, K);
    p.prob[0] = GemmProblem{nullptr, nullptr, nullptr, y, nullptr, nullptr};
    // A long K under a few output tiles (a weight gradient: K = rows of the batch) is split over
    // blockIdx.z so that the whole GPU works on it; the partials are then summed in split order.
    const uint32_t tiles = (uint32_t)(((M + BM - 1) / BM) * ((N + BN - 1) / BN)), kb = (uint32_t)(K / BK);
    if (tiles < (uint32_t)rt->sm_count && kb >= 32) {
        uint32_t want = (2u * (uint32_t)rt->sm_count + tiles - 1) / tiles;
        want = std::min(std::min(want, kb / 8), 64u);
        const uint32_t per = (kb + want - 1) / want, splits = (kb + per - 1) / per;
        if (splits > 1) {
            float* part = rt->tc_ws[8].as<float>((size_t)splits * M * N);
            p.split_k = splits;
            p.prob[0].out = part;
            dim3 grid((unsigned)((N + BN - 1) / BN), (unsigned)((M + BM - 1) / BM), splits);
            gemm_kernel<EPI_STORE, false><<<grid, GEMM_THREADS, gemm_smem_bytes(p.n_a, p.stages), rt->stream>>>(maps, p);
            rt->launched("gemm_dense_nt_splitk");
            const size_t n = M * N;
            splitk_reduce_kernel<<<blocks_for((n + 3) / 4, 256), 256, 0, rt->stream>>>(part, y, splits, n);
            rt->launched("splitk_reduce");
            return true;
        }
    }
    launch<EPI_STORE, false>(rt, maps, p, 1, "gemm_dense_nt");
    return true;
}

bool rosa_qkv_bits(ullis_cuda_runtime* rt, const float* ln3_out, const LayerWeights& L, uint32_t* q_sw,
                   uint32_t* k_sw, uint32_t* v_sw, size_t batch, size_t time, size_t d, const float* x_before_ln,
                   float* ln3_write) {
    const size_t rows = batch * time;
    if (!usable(rt) || !shape_ok(rows, d, d) || time % 32) return false;
    const size_t n = rows * d, wps = time / 32, sw = batch * d * wps;
    uint16_t* op = rt->tc_ws[1].as<uint16_t>(6 * n);   // q/k/v hi, then q/k/v lo
    float* s1 = rt->tc_ws[2].as<float>(3 * rows);
    uint32_t* flags = rt->tc_ws[3].as<uint32_t>(3 * sw);
    // x_before_ln: ln3 has not run yet - it is folded into the operand kernel, which leaves its output in ln3_write
    // (= ln3_out) for the exact fix-up below
    if (!(x_before_ln && launch_ln_mix_split(rt, x_before_ln, L.ln3, ln3_write, L.x_q, L.x_k, L.x_v, op, op + 3 * n, op + n,
                                             op + 4 * n, op + 2 * n, op + 5 * n, s1, rows, time, d, "ln_mix_split"))) {
        if (x_before_ln) k::layer_norm(rt, x_before_ln, L.ln3.weight, L.ln3.bias, ln3_write, rows, d, false);
        mix_split_kernel<<<blocks_for(rows, 8), 256, 0, rt->stream>>>(ln3_out, L.x_q, L.x_k, L.x_v, op, op + 3 * n, op + n,
                                                                     op + 4 * n, op + 2 * n, op + 5 * n, s1, rows, time, d);
        rt->launched("mix_split");
    }
    GemmMaps maps;
    memset(&maps, 0, sizeof(maps));
    for (int z = 0; z < 3; ++z) {
        maps.a[z][0] = make_map(op + z * n, rows, d, false);
        maps.a[z][1] = make_map(op + (3 + z) * n, rows, d, false);
    }
    GemmParams p = base_params(rt, rows, d, d);
    p.n_a = 2;
    p.stages = rt->tc_stages2;
    p.time = (uint32_t)time;
    p.wps = (uint32_t)wps;
    const PackedWeights* W[3] = {&L.q, &L.k, &L.v};
    uint32_t* outs[3] = {q_sw, k_sw, v_sw};
    for (int z = 0; z < 3; ++z)
        p.prob[z] = GemmProblem{W[z]->bits, W[z]->scale, W[z]->bias, outs[z], flags + z * sw, s1 + z * rows};
    launch<EPI_SIGNBITS, true>(rt, maps, p, 3, "gemm_qkv_signbits");
    const unsigned grid = (unsigned)(((wps + FIX_WIN - 1) / FIX_WIN) * batch);   // rows < 2^30, so this fits
    const uint32_t* only_if = nullptr;
    if (rt->tc_fix_list && 3 * sw < ((size_t)1 << 27) && d % FIXQ_COLS == 0 && d <= 32 * FIXQ_MAX_WORDS) {
        // one thread per flagged output, from a compact list; room for one output in 64
        const size_t cap = std::max<size_t>(65536, 3 * sw * 32 / 64);
        uint32_t* ctrl = rt->tc_ws[9].as<uint32_t>(2 + cap);
        uint32_t* list = ctrl + 2;
        rt->zero(ctrl, 8);
        fix_collect_kernel<<<4 * (unsigned)rt->sm_count, 256, 0, rt->stream>>>(flags, sw, batch, d, wps, list, (uint32_t)cap, ctrl);
        rt->launched("fix_collect");
        fix_apply_kernel<<<12 * (unsigned)rt->sm_count, FIXQ_WARPS * 32, 0, rt->stream>>>(
            ln3_out, L.x_q, L.x_k, L.x_v, L.q, L.k, L.v, q_sw, k_sw, v_sw, list, (uint32_t)cap, ctrl, sw, time, d, wps);
        rt->launched("fix_apply");
        only_if = ctrl + 1;
    }
    sign_fixup_kernel<<<grid, FIX_THREADS, FIX_QUEUE * 4, rt->stream>>>(ln3_out, L.x_q, L.x_k, L.x_v, L.q, L.k, L.v, q_sw, k_sw, v_sw, flags,
                                                   flags + sw, flags + 2 * sw, batch, time, d, wps, only_if);
    rt->launched("sign_fixup");
    return true;
}

bool rosa_out_residual(ullis_cuda_runtime* rt, const uint32_t* idx_sw, const LayerWeights& L, float* x, size_t batch,
                       size_t time, size_t d) {
    const size_t rows = batch * time;
    if (!usable(rt) || !shape_ok(rows, d, d) || d % 4) return false;
    uint16_t* y16 = rt->tc_ws[0].as<uint16_t>(rows * d);
    const size_t wps = (time + 31) / 32;
    dim3 grid((unsigned)wps, (unsigned)((d + 255) / 256), (unsigned)batch);
    emit_f16_kernel<<<grid, 256, 0, rt->stream>>>(idx_sw, L.e, y16, time, d, wps);
    rt->launched("emit_f16");
    GemmMaps maps;
    memset(&maps, 0, sizeof(maps));
    maps.a[0][0] = make_map(y16, rows, d, false);
    GemmParams p = base_params(rt, rows, d, d);
    p.prob[0] = GemmProblem{L.o.bits, L.o.scale, L.o.bias, x, nullptr, nullptr};
    launch<EPI_RESIDUAL, true>(rt, maps, p, 1, "gemm_o_residual");
    return true;
}

bool cmix_residual(ullis_cuda_runtime* rt, const LayerWeights& L, float* x, size_t batch, size_t time, size_t d,
                   size_t ffn) {
    const size_t rows = batch * time;
    if (!usable(rt) || !shape_ok(rows, d, ffn) || !shape_ok(rows, ffn, d) || d % 4) return false;
    float* ln = rt->tc_ws[4].as<float>(rows * d);
    uint16_t* a16 = rt->tc_ws[0].as<uint16_t>(rows * d);
    uint16_t* k16 = rt->tc_ws[5].as<uint16_t>(rows * ffn);
    if (!launch_ln_mix_split(rt, x, L.ln2, nullptr, L.ffn_x_k, nullptr, nullptr, a16, nullptr, nullptr, nullptr, nullptr,
                             nullptr, nullptr, rows, time, d, "ln_mix_f16")) {
        k::layer_norm(rt, x, L.ln2.weight, L.ln2.bias, ln, rows, d, false);
        mix_split_kernel<<<blocks_for(rows, 8), 256, 0, rt->stream>>>(ln, L.ffn_x_k, nullptr, nullptr, a16, nullptr,
                                                                     nullptr, nullptr, nullptr, nullptr, nullptr, rows, time, d);
        rt->launched("mix_f16");
    }
    GemmMaps maps;
    memset(&maps, 0, sizeof(maps));
    maps.a[0][0] = make_map(a16, rows, d, false);
    GemmParams p = base_params(rt, rows, ffn, d);
    p.out_fmt = 0;  // FP16: three more significant bits than bf16; the epilogue reports values past 65504
    p.prob[0] = GemmProblem{L.key.bits, L.key.scale, nullptr, k16, nullptr, nullptr};
    launch<EPI_RELU2, true>(rt, maps, p, 1, "gemm_key_relu2");
    memset(&maps, 0, sizeof(maps));
    maps.a[0][0] = make_map(k16, rows, ffn, false);
    maps.b[0] = make_map(L.value, d, ffn, false);   // the FP16 weights as stored
    GemmParams pv = base_params(rt, rows, d, ffn);
    pv.prob[0] = GemmProblem{nullptr, nullptr, nullptr, x, nullptr, nullptr};
    launch<EPI_RESIDUAL, false>(rt, maps, pv, 1, "gemm_value_residual");
    return true;
}

namespace {
// One CTA waits, with the bounded mbarrier wait every tensor-core kernel here uses, on a barrier that nothing
// ever arrives on, and reports the give-up through the runtime's status words like those kernels do.
__global__ void wait_selftest_kernel(uint32_t polls, uint32_t* status) {
    __shared__ __align__(8) uint64_t bar;
    if (threadIdx.x == 0) {
        ptx::mbar_init(&bar, 1);
        ptx::fence_mbar_init();
    }
    __syncthreads();
    if (threadIdx.x == 0 && !ptx::mbar_wait(&bar, 0, polls)) {
        if (atomicCAS(status, ULLIS_DEV_OK, ULLIS_DEV_WAIT_TIMEOUT) == ULLIS_DEV_OK) status[1] = 99u;   // site: self-test
    }
}
}  // namespace

void wait_selftest(ullis_cuda_runtime* rt, uint32_t polls) {
    wait_selftest_kernel<<<1, 32, 0, rt->stream>>>(polls, rt->dev_status);
    rt->launched("wait_selftest");
}

bool takes_model(ullis_cuda_runtime* rt, size_t rows, size_t time, size_t d, size_t ffn, size_t vocab) {
    return usable(rt) && shape_ok(rows, d, d) && time % 32 == 0 && d % 4 == 0 && shape_ok(rows, d, ffn) &&
           shape_ok(rows, ffn, d) && shape_ok(rows, d, vocab);
}

bool head_ce(ullis_cuda_runtime* rt, const float* hidden, const PackedWeights& head, const uint32_t* labels,
             uint32_t ignore_id, size_t rows, size_t time, size_t d, size_t vocab, float* row_loss) {
    if (!usable(rt) || !shape_ok(rows, d, vocab)) return false;
    // partials per row: one per vocabulary tile and epilogue warp group of the kernel that will run
    const uint32_t n_tiles = (uint32_t)((vocab + BN - 1) / BN) * (takes_ws(rt, d, 1) ? WS_EPI_GROUPS : 1u);
    uint16_t* a16 = rt->tc_ws[0].as<uint16_t>(rows * d);
    float2* part = rt->tc_ws[6].as<float2>(rows * n_tiles);
    float* tl = rt->tc_ws[7].as<float>(rows);
    cast16(rt, hidden, a16, rows, d, false);
    GemmMaps maps;
    memset(&maps, 0, sizeof(maps));
    maps.a[0][0] = make_map(a16, rows, d, false);
    GemmParams p = base_params(rt, rows, vocab, d);
    p.labels = labels;
    p.ignore_id = ignore_id;
    p.n_tiles = n_tiles;
    p.time = (uint32_t)time;
    p.prob[0] = GemmProblem{head.bits, head.scale, head.bias, part, tl, nullptr};
    launch<EPI_CE, true>(rt, maps, p, 1, "gemm_head_ce");
    ce_finish_kernel<<<blocks_for(rows, 256), 256, 0, rt->stream>>>(part, tl, labels, ignore_id, rows, time, vocab, n_tiles,
                                                                  row_loss, rt->dev_status);
    rt->launched("ce_finish");
    return true;
}

}  // namespace tc
}  // namespace ullis
