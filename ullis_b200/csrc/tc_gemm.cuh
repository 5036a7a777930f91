// Tensor-core GEMM for the Heron linears on sm_100a: D[M,N] = A[M,K] . W[N,K]^T
// with f32 accumulation in TMEM (tcgen05.mma, kind::f16) and a fused epilogue.
//
//  * A (activations, 16-bit, K-major) arrives by TMA into 128-byte-swizzled
//    shared tiles; an optional second A operand ("lo" part of a hi+lo split of
//    f32 activations) is multiplied into the same accumulator.
//  * W is either packed +/-1 bits - expanded inside the kernel from 32-bit
//    words into FP16 +/-1.0 rows written straight into the swizzled layout the
//    MMA reads (reference weight order: bit o*K+i, LSB first, 1 => +1,
//    src/model.rs:146-148) - or a dense FP16 [N,K] matrix loaded by TMA.
//  * One CTA computes one 128x128 tile: warp 0 issues TMA, warp 1 owns TMEM and
//    issues the MMAs, warps 2-5 expand weight bits during the main loop and
//    then run the epilogue, one TMEM lane (= output row) per thread.
//  * Pipeline: STAGES shared-memory stages guarded by full/empty mbarriers;
//    every wait is bounded and reports through the status word.
//
// Epilogues (y = bias + scale * acc, FP16 row scale / bias, either may be null):
//   EPI_STORE     f32 store                      (src/model.rs:724-742)
//   EPI_RESIDUAL  out += y                       (src/model.rs:2232-2239)
//   EPI_RELU2     16-bit store of max(y,0)^2     (src/model.rs:999)
//   EPI_SIGNBITS  sign bit y > 0 per element, 32 consecutive steps of a channel
//                 per word (stream-major), plus a "too close to zero to trust
//                 the tensor-core sum" flag word  (src/rosa.rs:372-374)
//   EPI_CE        per-row partial (max, sum exp, target logit) over the tile's
//                 vocabulary slice               (src/model.rs:3219-3226)
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.hpp"
#include "tc_ptx.cuh"

namespace ullis {
namespace tc {

enum { EPI_STORE = 0, EPI_RESIDUAL = 1, EPI_RELU2 = 2, EPI_SIGNBITS = 3, EPI_CE = 4 };

constexpr int BM = 128, BN = 128, BK = 64, MAX_STAGES = 4;
constexpr int TILE_BYTES = BM * BK * 2;  // 16 KiB, also the B tile (BN == BM)
constexpr int GEMM_THREADS = 192;
constexpr int STAGE_STRIDE = 20;                         // floats per row of an epilogue warp's 32 x 16 transposition buffer
constexpr int STAGE_BYTES = 32 * STAGE_STRIDE * 4;       // per epilogue warp

struct GemmProblem {
    const uint32_t* bits;   // packed weights (PACKED kernels)
    const uint16_t* scale;  // FP16 [N] or null (= 1)
    const uint16_t* bias;   // FP16 [N] or null (= 0)
    void* out;
    void* out2;
    const float* aux;       // EPI_SIGNBITS: per-row sum |a| ; EPI_CE: unused
};

struct GemmMaps {
    CUtensorMap a[3][2];  // [problem][hi, lo]
    CUtensorMap b[3];     // dense weights
};

struct GemmParams {
    GemmProblem prob[3];
    uint32_t M, N, K;
    uint32_t n_a;            // 1 or 2 A operands
    uint32_t stages;         // shared-memory pipeline depth, 2..MAX_STAGES
    uint32_t a_fmt, b_fmt;   // 0 = f16, 1 = bf16
    uint32_t out_fmt;        // EPI_RELU2: 0 = f16, 1 = bf16
    uint32_t time, wps;      // EPI_SIGNBITS / EPI_CE: steps per sequence, words per stream
    const uint32_t* labels;  // EPI_CE
    uint32_t ignore_id;      // EPI_CE
    uint32_t n_tiles;        // EPI_CE: (max, sum exp) partials per row: one per vocabulary tile and epilogue warp group
    uint32_t split_k;        // > 1 (gemm_kernel, one problem): blockIdx.z owns a K range and writes its own [M,N] partial
    uint32_t* status;
};

inline size_t gemm_smem_bytes(uint32_t n_a, uint32_t stages) {
    return 1024 /*alignment slack*/ + (size_t)stages * (n_a + 1) * TILE_BYTES + 256 * 16 /*LUT*/ + 2 * BN * 4 + 256;
}

__device__ __forceinline__ float h2f_bits(uint16_t b) { return __half2float(__ushort_as_half(b)); }

// row scale / bias of the tile's columns as the kernel keeps them in shared memory: f32, or the FP16 they came from
__device__ __forceinline__ float sb_load(const float* p, uint32_t i) { return p[i]; }
__device__ __forceinline__ float sb_load(const __half* p, uint32_t i) { return __half2float(p[i]); }
// entries i and i + 1 (i even) with one shared-memory load
__device__ __forceinline__ float2 sb_load2(const float* p, uint32_t i) { return *reinterpret_cast<const float2*>(p + i); }
__device__ __forceinline__ float2 sb_load2(const __half* p, uint32_t i) {
    return __half22float2(*reinterpret_cast<const __half2*>(p + i));
}

// One output row (TMEM lane) per thread, the 32-column chunks [c_begin, c_end) of the tile's 128 columns.
// `part` = index of this call's partial among the row's p.n_tiles partials (EPI_CE).
// The TMEM loads are warp-collective, so row / column guards only wrap stores.
template <int EPI, typename SB = float, bool STAGED16 = false>
__device__ __forceinline__ void epilogue(const GemmParams& p, const GemmProblem& pr, uint32_t taddr, uint32_t m,
                                         uint32_t n0, const SB* s_scale, const SB* s_bias, int lane, uint32_t part,
                                         uint32_t c_begin = 0, uint32_t c_end = BN / 32, float* stage = nullptr) {
    const bool row_ok = m < p.M;
    // EPI_SIGNBITS: the 32 rows of this warp are 32 consecutive steps of one sequence (M, time % 32 == 0)
    const uint32_t m_warp = m - lane;
    const float s1 = (EPI == EPI_SIGNBITS && row_ok) ? pr.aux[m] : 0.0f;
    // EPI_CE running state
    float run_max = -INFINITY, run_sum = 0.0f;
    uint32_t target = 0xFFFFFFFFu;
    if (EPI == EPI_CE && m + 1 < p.M) target = p.labels[m + 1];
#pragma unroll 1
    for (uint32_t c = c_begin; c < c_end; ++c) {
        const uint32_t nc = n0 + c * 32;
        // EPI_RESIDUAL: the chunk's eight 16-byte pieces of the old rows are asked for before anything else, so
        // that they travel while the accumulator is read, converted and transposed (a load placed next to its
        // store cannot be moved up by the compiler, and each then waited for the one before it)
        float4 old_rows[2][4];
        if (EPI == EPI_RESIDUAL) {
            const float* out = static_cast<const float*>(pr.out);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const uint32_t gm = m_warp + i * 8 + (lane >> 2), col = nc + h * 16 + (lane & 3) * 4;
                    old_rows[h][i] = (gm < p.M && col < p.N) ? *reinterpret_cast<const float4*>(out + (size_t)gm * p.N + col)
                                                             : make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
        }
        uint32_t r[32];
        ptx::tmem_ld_32x32(taddr + c * 32, r);
        ptx::tmem_ld_wait();
        if (EPI == EPI_STORE || EPI == EPI_RESIDUAL) {
            // A thread holds one row of the accumulator, so a direct store touches 32
            // different rows per instruction.  The chunk goes through a small
            // shared-memory transposition instead (16 columns at a time): afterwards
            // four lanes cover 64 contiguous bytes of one row and an instruction
            // covers eight rows.
            float* out = static_cast<float*>(pr.out);
            const uint32_t m_first = m - lane;   // first row of this warp
#pragma unroll
            for (int h = 0; h < 2; ++h) {
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int j = h * 16 + q * 4;
                    float4 v;
                    v.x = sb_load(s_bias, c * 32 + j + 0) + sb_load(s_scale, c * 32 + j + 0) * __uint_as_float(r[j + 0]);
                    v.y = sb_load(s_bias, c * 32 + j + 1) + sb_load(s_scale, c * 32 + j + 1) * __uint_as_float(r[j + 1]);
                    v.z = sb_load(s_bias, c * 32 + j + 2) + sb_load(s_scale, c * 32 + j + 2) * __uint_as_float(r[j + 2]);
                    v.w = sb_load(s_bias, c * 32 + j + 3) + sb_load(s_scale, c * 32 + j + 3) * __uint_as_float(r[j + 3]);
                    *reinterpret_cast<float4*>(stage + lane * STAGE_STRIDE + q * 4) = v;
                }
                __syncwarp();
                const uint32_t col = nc + h * 16 + (lane & 3) * 4;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const uint32_t row = i * 8 + (lane >> 2);
                    const uint32_t gm = m_first + row;
                    float4 v = *reinterpret_cast<const float4*>(stage + row * STAGE_STRIDE + (lane & 3) * 4);
                    if (gm < p.M && col < p.N) {            // N is a multiple of 4: the whole float4 is in range
                        float4* dst = reinterpret_cast<float4*>(out + (size_t)gm * p.N + col);
                        if (EPI == EPI_RESIDUAL) {
                            const float4 o = old_rows[h][i];
                            v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
                        }
                        *dst = v;
                    }
                }
                __syncwarp();
            }
        } else if (EPI == EPI_RELU2) {
            uint16_t* out = static_cast<uint16_t*>(pr.out) + (size_t)m * p.N + nc;
            float top = 0.0f;   // largest output of this row's chunk, for the FP16 range check
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
                uint32_t w[4];
#pragma unroll
                for (int e = 0; e < 8; e += 2) {
                    const float2 sc = sb_load2(s_scale, c * 32 + j + e), bi = sb_load2(s_bias, c * 32 + j + e);
                    float a = fmaxf(bi.x + sc.x * __uint_as_float(r[j + e]), 0.0f);
                    float b = fmaxf(bi.y + sc.y * __uint_as_float(r[j + e + 1]), 0.0f);
                    a *= a; b *= b;
                    if (p.out_fmt == 1) {
                        __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
                        w[e / 2] = *reinterpret_cast<uint32_t*>(&h);
                    } else {
                        // FP16 keeps 11 significant bits (bf16: 8) but ends at 65504: report, do not emit inf
                        top = fmaxf(top, fmaxf(a, b));
                        __half2 h = __floats2half2_rn(fminf(a, 65504.0f), fminf(b, 65504.0f));
                        w[e / 2] = *reinterpret_cast<uint32_t*>(&h);
                    }
                }
                if (STAGED16) {
                    // 16-byte granule q = j / 8 of this lane's row, at (q ^ f(row)) so that neither the
                    // row-wise writes nor the reads below meet a bank conflict (rows are 64 bytes apart)
                    reinterpret_cast<uint4*>(stage)[lane * 4 + ((j >> 3) ^ ((lane >> 1) & 3))] =
                        make_uint4(w[0], w[1], w[2], w[3]);
                } else if (row_ok && nc + j + 7 < p.N) {
                    *reinterpret_cast<uint4*>(out + j) = make_uint4(w[0], w[1], w[2], w[3]);
                }
            }
            if (row_ok && top > 65504.0f && atomicCAS(p.status, ULLIS_DEV_OK, ULLIS_DEV_FP16_RANGE) == ULLIS_DEV_OK)
                p.status[1] = m;
            if (STAGED16) {
                // a thread holds 64 bytes of ONE row, so direct stores touch 32 rows per instruction; through
                // the warp's 32 x 64-byte buffer four lanes cover a row's 64 bytes and an instruction eight rows
                __syncwarp();
                uint16_t* base = static_cast<uint16_t*>(pr.out);
                const uint32_t col = nc + (lane & 3) * 8;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const uint32_t row = i * 8 + (lane >> 2);
                    const uint4 v = reinterpret_cast<const uint4*>(stage)[row * 4 + ((lane & 3) ^ ((row >> 1) & 3))];
                    const uint32_t gm = m_warp + row;
                    if (gm < p.M && col + 7 < p.N) *reinterpret_cast<uint4*>(base + (size_t)gm * p.N + col) = v;
                }
                __syncwarp();
            }
        } else if (EPI == EPI_SIGNBITS) {
            uint32_t my_bits = 0, my_flags = 0;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                const float2 sc2 = sb_load2(s_scale, c * 32 + (j & ~1)), bi2 = sb_load2(s_bias, c * 32 + (j & ~1));
                const float sc = (j & 1) ? sc2.y : sc2.x, bi = (j & 1) ? bi2.y : bi2.x;
                const float t = sc * __uint_as_float(r[j]);
                const float y = bi + t;
                // error bound of the tensor-core sum against the reference's sequential f32 sum
                const float guard = fabsf(sc) * (s1 * 1.3e-4f + 1e-4f) + 1e-6f * (fabsf(bi) + fabsf(t));
                const uint32_t wb = __ballot_sync(0xffffffffu, row_ok && y > 0.0f);
                const uint32_t wf = __ballot_sync(0xffffffffu, row_ok && fabsf(y) <= guard);
                if (lane == j) { my_bits = wb; my_flags = wf; }
            }
            const uint32_t n = nc + lane;
            if (m_warp < p.M && n < p.N) {
                const uint32_t b = m_warp / p.time, word = (m_warp % p.time) >> 5;
                const size_t o = ((size_t)b * p.N + n) * p.wps + word;
                static_cast<uint32_t*>(pr.out)[o] = my_bits;      // stream-major, as the automaton reads them
                // the flag words of one block of 32 steps lie side by side over the channels: the warp writes 128
                // consecutive bytes, and the kernel that lists the flags reads them the same way
                static_cast<uint32_t*>(pr.out2)[((size_t)b * p.wps + word) * p.N + n] = my_flags;
            }
        } else if (EPI == EPI_CE) {
            // whole chunks (the usual case: the vocabulary is a multiple of 32) skip the per-column range test,
            // and the target's logit is picked out only in the one chunk of the row that holds it
            const bool whole = nc + 32u <= p.N;
            float cmax = -INFINITY;
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
                const float2 sc2 = sb_load2(s_scale, c * 32 + j), bi2 = sb_load2(s_bias, c * 32 + j);
                const float y0 = bi2.x + sc2.x * __uint_as_float(r[j]);
                const float y1 = bi2.y + sc2.y * __uint_as_float(r[j + 1]);
                r[j] = __float_as_uint(y0);
                r[j + 1] = __float_as_uint(y1);
                if (whole || nc + j < p.N) cmax = fmaxf(cmax, y0);
                if (whole || nc + j + 1 < p.N) cmax = fmaxf(cmax, y1);
            }
            if (row_ok && target - nc < 32u) {
                const uint32_t tj = target - nc;
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    if ((uint32_t)j == tj) static_cast<float*>(pr.out2)[m] = __uint_as_float(r[j]);
            }
            if (cmax > -INFINITY) {
                const float nmax = fmaxf(run_max, cmax);
                float add = 0.0f;
                if (whole) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) add += __expf(__uint_as_float(r[j]) - nmax);
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (nc + j < p.N) add += __expf(__uint_as_float(r[j]) - nmax);
                }
                run_sum = run_sum * __expf(run_max - nmax) + add;
                run_max = nmax;
            }
        }
    }
    if (EPI == EPI_CE && row_ok)
        static_cast<float2*>(pr.out)[(size_t)m * p.n_tiles + part] = make_float2(run_max, run_sum);
}

template <int EPI, bool PACKED>
__global__ void __launch_bounds__(GEMM_THREADS, 3)
gemm_kernel(const __grid_constant__ GemmMaps maps, const GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t stage_bytes = (p.n_a + 1) * TILE_BYTES;
    const uint32_t STAGES = p.stages;
    uint8_t* tiles = smem;
    uint4* lut = reinterpret_cast<uint4*>(smem + STAGES * stage_bytes);
    float* s_scale = reinterpret_cast<float*>(lut + 256);
    float* s_bias = s_scale + BN;
    uint64_t* bars = reinterpret_cast<uint64_t*>(s_bias + BN);
    uint64_t* full_a = bars;                 // [STAGES] TMA bytes landed
    uint64_t* full_b = bars + MAX_STAGES;        // [STAGES] weight tile expanded
    uint64_t* empty = bars + 2 * MAX_STAGES;     // [STAGES] MMAs that read the stage are done
    uint64_t* tmem_full = bars + 3 * MAX_STAGES; // accumulator complete
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3 * MAX_STAGES + 1);
    uint32_t* s_error = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t z = p.split_k > 1 ? 0u : blockIdx.z;
    GemmProblem pr = p.prob[z];
    const uint32_t n0 = blockIdx.x * BN, m0 = blockIdx.y * BM;
    uint32_t KB = p.K / BK, kb0 = 0;
    if (p.split_k > 1) {   // the host sizes the grid so that every split owns at least one k-block
        const uint32_t per = (KB + p.split_k - 1) / p.split_k;
        kb0 = blockIdx.z * per;
        KB = min(per, KB - kb0);
        pr.out = static_cast<float*>(pr.out) + (size_t)blockIdx.z * p.M * p.N;
    }

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < STAGES; ++s) {
            ptx::mbar_init(&full_a[s], 1);
            ptx::mbar_init(&full_b[s], 128);
            ptx::mbar_init(&empty[s], 1);
        }
        ptx::mbar_init(tmem_full, 1);
        *s_error = 0;
        ptx::fence_mbar_init();
        ptx::tma_prefetch_desc(&maps.a[z][0]);
        if (p.n_a == 2) ptx::tma_prefetch_desc(&maps.a[z][1]);
        if (!PACKED) ptx::tma_prefetch_desc(&maps.b[z]);
    }
    if (PACKED) {
        // 8 weight bits -> 8 FP16 values (+1.0 = 0x3C00, -1.0 = 0xBC00), bit i -> element i
        for (int b = threadIdx.x; b < 256; b += GEMM_THREADS) {
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t lo = (b >> (2 * j)) & 1u, hi = (b >> (2 * j + 1)) & 1u;
                w[j] = (lo ? 0x3C00u : 0xBC00u) | ((hi ? 0x3C00u : 0xBC00u) << 16);
            }
            lut[b] = make_uint4(w[0], w[1], w[2], w[3]);
        }
    }
    if (warp >= 2) {
        const int c = threadIdx.x - 64;  // 0..127: column of the tile
        const uint32_t n = n0 + c;
        s_scale[c] = (pr.scale && n < p.N) ? h2f_bits(pr.scale[n]) : 1.0f;
        s_bias[c] = (pr.bias && n < p.N) ? h2f_bits(pr.bias[n]) : 0.0f;
    }
    if (warp == 1) {
        ptx::tmem_alloc(tmem_slot, 128);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------ TMA producer
        if (ptx::elect_one()) {
            const uint32_t tx = (p.n_a + (PACKED ? 0 : 1)) * TILE_BYTES;
            uint32_t issued = 0;
            for (uint32_t kb = 0; kb < KB; ++kb, ++issued) {
                const uint32_t s = kb % STAGES;
                if (kb >= STAGES && !ptx::mbar_wait(&empty[s], ((kb / STAGES) & 1u) ^ 1u)) { atomicExch(s_error, 1u); break; }
                uint8_t* st = tiles + s * stage_bytes;
                ptx::mbar_arrive_expect_tx(&full_a[s], tx);
                const int32_t kx = (int32_t)((kb0 + kb) * BK);
                ptx::tma_load_2d(st, &maps.a[z][0], &full_a[s], kx, (int32_t)m0);
                if (p.n_a == 2) ptx::tma_load_2d(st + TILE_BYTES, &maps.a[z][1], &full_a[s], kx, (int32_t)m0);
                if (!PACKED) ptx::tma_load_2d(st + p.n_a * TILE_BYTES, &maps.b[z], &full_a[s], kx, (int32_t)n0);
            }
            if (*s_error) {
                // leave no copy in flight: wait (bounded) for every stage this thread filled last
                const uint32_t first = issued > STAGES ? issued - STAGES : 0;
                for (uint32_t kb = first; kb < issued; ++kb) ptx::mbar_wait(&full_a[kb % STAGES], (kb / STAGES) & 1u);
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------- MMA issuer
        if (ptx::elect_one()) {
            const uint32_t idesc = ptx::idesc_f16(p.a_fmt, p.b_fmt, BM, BN);
            bool ok = true;
            for (uint32_t kb = 0; kb < KB && ok; ++kb) {
                const uint32_t s = kb % STAGES, ph = (kb / STAGES) & 1u;
                ok = ptx::mbar_wait(&full_a[s], ph);
                if (ok && PACKED) ok = ptx::mbar_wait(&full_b[s], ph);
                if (!ok) { atomicExch(s_error, 2u); break; }
                ptx::tc_fence_after_sync();
                const uint32_t a_addr = ptx::smem_u32(tiles + s * stage_bytes);
                const uint32_t b_addr = a_addr + p.n_a * TILE_BYTES;
#pragma unroll
                for (uint32_t k4 = 0; k4 < BK / 16; ++k4) {
                    const uint64_t db = ptx::smem_desc_sw128(b_addr + k4 * 32);
                    ptx::mma_f16_ss(tmem_base, ptx::smem_desc_sw128(a_addr + k4 * 32), db, idesc, (kb | k4) != 0);
                    if (p.n_a == 2)
                        ptx::mma_f16_ss(tmem_base, ptx::smem_desc_sw128(a_addr + TILE_BYTES + k4 * 32), db, idesc, 1u);
                }
                ptx::mma_commit(&empty[s]);
            }
            ptx::mma_commit(tmem_full);  // also fires on the error path so the epilogue does not wait in vain
        }
    } else {
        // ------------------------------------- weight expansion, then epilogue
        const int r = threadIdx.x - 64;  // tile row of W (0..127) now, output row later
        if (PACKED) {
            const uint32_t n = n0 + r;
            const uint32_t* wrow = pr.bits + ((size_t)n * p.K >> 5);
            for (uint32_t kb = 0; kb < KB; ++kb) {
                const uint32_t s = kb % STAGES;
                if (kb >= STAGES && !ptx::mbar_wait(&empty[s], ((kb / STAGES) & 1u) ^ 1u)) { atomicExch(s_error, 3u); break; }
                uint32_t w0 = 0, w1 = 0;
                if (n < p.N) { w0 = wrow[kb * 2]; w1 = wrow[kb * 2 + 1]; }
                uint8_t* dst = tiles + s * stage_bytes + p.n_a * TILE_BYTES + r * 128;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const uint32_t byte = ((j < 4 ? w0 : w1) >> (8 * (j & 3))) & 0xFFu;
                    *reinterpret_cast<uint4*>(dst + ((j ^ (r & 7)) << 4)) = lut[byte];
                }
                ptx::fence_proxy_async_smem();  // generic-proxy stores -> visible to the MMA's async reads
                ptx::mbar_arrive(&full_b[s]);
            }
        }
        // epilogue: this warp may only touch TMEM lanes 32*(warp%4) .. +31
        const uint32_t quarter = warp & 3;
        const uint32_t row_in_tile = quarter * 32 + lane;
        const uint32_t m = m0 + row_in_tile;
        const bool waited = ptx::mbar_wait(tmem_full, 0);
        if (!waited) atomicExch(s_error, 4u);
        ptx::tc_fence_after_sync();
        if (waited && *s_error == 0) {
            const uint32_t taddr = tmem_base + ((quarter * 32) << 16);
            // the pipeline stages are dead once the accumulator is complete: their space stages the stores
            epilogue<EPI>(p, pr, taddr, m, n0, s_scale, s_bias, lane, blockIdx.x, 0, BN / 32,
                          reinterpret_cast<float*>(tiles + (warp - 2) * STAGE_BYTES));
        }
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, 128);
    }
    if (threadIdx.x == 0 && *s_error) {
        if (atomicCAS(p.status, ULLIS_DEV_OK, ULLIS_DEV_WAIT_TIMEOUT) == ULLIS_DEV_OK) p.status[1] = *s_error;
    }
}

}  // namespace tc
}  // namespace ullis
