// Weight-stationary variant of the tensor-core GEMM for packed +/-1 weights
// with a short inner dimension (K <= 512), the shape of every packed linear of
// the Heron path (D -> D, D -> F, D -> V with D = d_model).
//
// A CTA owns ONE 128-row tile of W for its whole life: the bits are expanded
// once into shared memory (K/64 swizzled 128x64 FP16 tiles, up to 128 KiB) and
// the CTA then walks down the M dimension, one 128-row activation tile after
// another.  Per output tile only the activations move (TMA, a deep ring of
// 16 KiB stages), the MMAs of tile i+1 run while the epilogue warps drain the
// accumulator of tile i (two 128-column TMEM buffers), and nothing is rebuilt
// per k-block.  CTAs that share an activation tile (the other column tiles and,
// for Q/K/V, nothing else) walk M in the same order, so the tile is read from
// HBM once and from L2 afterwards.
//
// Warp roles: warp 0 TMA producer, warp 1 TMEM owner + MMA issuer, warps 2-9
// epilogue (two warps per TMEM lane quarter, half of the columns each).  Every wait is bounded and gives up early once
// another role has recorded an error.
#pragma once
#include "tc_gemm.cuh"

namespace ullis {
namespace tc {

constexpr uint32_t WS_MAX_KB = 8;          // K <= 512
constexpr uint32_t WS_MAX_STAGES = 8;
constexpr uint32_t WS_SMEM_LIMIT = 227 * 1024;
constexpr int WS_THREADS = 320;            // TMA warp, MMA warp, eight epilogue warps (two per TMEM lane quarter)
constexpr uint32_t WS_EPI_GROUPS = 2;      // epilogue warp groups, each takes half of the tile's columns

struct WsShape {
    uint32_t stages;   // activation ring depth
    uint32_t smem;     // dynamic shared memory bytes
};

// ring depth that fits beside the resident weight tile
inline WsShape ws_shape(uint32_t K, uint32_t n_a, bool staged_stores, bool resident_w = true) {
    const uint32_t kb = K / BK;
    const uint32_t fixed = 1024 /*alignment slack*/ + (resident_w ? kb * TILE_BYTES : 0) + 2 * BN * 4 + 256 +
                           (staged_stores ? 8 * STAGE_BYTES : 0);
    if (!resident_w) n_a += 1;   // the weight tile travels with the activations
    uint32_t stages = (WS_SMEM_LIMIT - fixed) / (n_a * TILE_BYTES);
    if (stages > WS_MAX_STAGES) stages = WS_MAX_STAGES;
    return WsShape{stages, fixed + stages * n_a * TILE_BYTES};
}

// bounded wait that also gives up when another role of the CTA has failed
__device__ __forceinline__ bool ws_wait(uint64_t* bar, uint32_t parity, volatile uint32_t* s_error) {
    for (uint32_t spin = 0; spin < (1u << 24); ++spin) {
        if (ptx::mbar_try_wait(bar, parity)) return true;
        if (spin > 64) {
            __nanosleep(spin > 4096 ? 256 : 32);
            if ((spin & 1023u) == 0 && *s_error) return false;
        }
    }
    return false;
}

// RESIDENT_W = false: dense 16-bit weights of any K, fetched by TMA into the same
// ring stage as the activations (nothing stays resident); same roles, same
// double-buffered accumulator.
template <int EPI, bool RESIDENT_W = true>
__global__ void __launch_bounds__(WS_THREADS, 1)
gemm_ws_kernel(const __grid_constant__ GemmMaps maps, const GemmParams p, const uint32_t pairs) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t KB = p.K / BK;
    const uint32_t STAGES = p.stages;
    const uint32_t stage_bytes = (p.n_a + (RESIDENT_W ? 0u : 1u)) * TILE_BYTES;
    uint8_t* w_tiles = smem;                               // [KB] resident weight tiles
    uint8_t* a_ring = smem + (RESIDENT_W ? KB * TILE_BYTES : 0u);   // [STAGES] activation (+ weight) stages
    uint4* lut = reinterpret_cast<uint4*>(a_ring);         // only until the weights are expanded
    float* s_scale = reinterpret_cast<float*>(a_ring + STAGES * stage_bytes);
    float* s_bias = s_scale + BN;
    uint64_t* bars = reinterpret_cast<uint64_t*>(s_bias + BN);
    uint64_t* full = bars;                                 // [STAGES] TMA bytes landed
    uint64_t* empty = bars + WS_MAX_STAGES;                // [STAGES] MMAs that read the stage are done
    uint64_t* tmem_full = bars + 2 * WS_MAX_STAGES;        // [2] accumulator complete
    uint64_t* tmem_empty = tmem_full + 2;                  // [2] accumulator drained
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
    uint32_t* s_error = tmem_slot + 1;
    float* stage_base = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(bars) + 256);   // STORE / RESIDUAL only

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // work split: pair = (problem, column tile), fixed per CTA; the CTAs of a pair interleave over the row tiles
    const uint32_t pair = blockIdx.x % pairs, member = blockIdx.x / pairs;
    const uint32_t members = (gridDim.x - pair + pairs - 1) / pairs;
    const uint32_t n_tiles = (p.N + BN - 1) / BN;
    const uint32_t z = pair / n_tiles, n_tile = pair % n_tiles;
    const uint32_t n0 = n_tile * BN;
    const uint32_t m_tiles = (p.M + BM - 1) / BM;
    const uint32_t my_tiles = member < m_tiles ? (m_tiles - member + members - 1) / members : 0;
    const GemmProblem& pr = p.prob[z];

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < STAGES; ++s) {
            ptx::mbar_init(&full[s], 1);
            ptx::mbar_init(&empty[s], 1);
        }
        for (uint32_t b = 0; b < 2; ++b) {
            ptx::mbar_init(&tmem_full[b], 1);
            ptx::mbar_init(&tmem_empty[b], 128 * WS_EPI_GROUPS);
        }
        *s_error = 0;
        ptx::fence_mbar_init();
        ptx::tma_prefetch_desc(&maps.a[z][0]);
        if (p.n_a == 2) ptx::tma_prefetch_desc(&maps.a[z][1]);
        if (!RESIDENT_W) ptx::tma_prefetch_desc(&maps.b[z]);
    }
    // 8 weight bits -> 8 FP16 values (+1.0 = 0x3C00, -1.0 = 0xBC00), bit i -> element i
    for (int b = threadIdx.x; RESIDENT_W && b < 256; b += WS_THREADS) {
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t lo = (b >> (2 * j)) & 1u, hi = (b >> (2 * j + 1)) & 1u;
            w[j] = (lo ? 0x3C00u : 0xBC00u) | ((hi ? 0x3C00u : 0xBC00u) << 16);
        }
        lut[b] = make_uint4(w[0], w[1], w[2], w[3]);
    }
    if (threadIdx.x < BN) {
        const uint32_t n = n0 + threadIdx.x;
        s_scale[threadIdx.x] = (pr.scale && n < p.N) ? h2f_bits(pr.scale[n]) : 1.0f;
        s_bias[threadIdx.x] = (pr.bias && n < p.N) ? h2f_bits(pr.bias[n]) : 0.0f;
    }
    if (warp == 1) {
        ptx::tmem_alloc(tmem_slot, 256);
        ptx::tmem_relinquish();
    }
    __syncthreads();
    // expand this CTA's weight tile once: row r of k-block kb -> 128 bytes, 16-byte chunk j at j ^ (r % 8)
    for (uint32_t item = threadIdx.x; RESIDENT_W && item < KB * BN; item += WS_THREADS) {
        const uint32_t r = item % BN, kb = item / BN;
        const uint32_t n = n0 + r;
        uint32_t w0 = 0, w1 = 0;
        if (n < p.N) {
            const uint32_t* wrow = pr.bits + ((size_t)n * p.K >> 5);
            w0 = wrow[kb * 2];
            w1 = wrow[kb * 2 + 1];
        }
        uint8_t* dst = w_tiles + kb * TILE_BYTES + r * 128;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const uint32_t byte = ((j < 4 ? w0 : w1) >> (8 * (j & 3))) & 0xFFu;
            *reinterpret_cast<uint4*>(dst + ((j ^ (r & 7)) << 4)) = lut[byte];
        }
    }
    ptx::fence_proxy_async_smem();  // generic-proxy stores -> visible to the MMA's async reads
    ptx::tc_fence_before_sync();
    __syncthreads();                // also: the table is dead, the ring may be filled
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------ TMA producer
        if (ptx::elect_one()) {
            uint32_t it = 0;
            bool ok = true;
            for (uint32_t t = 0; t < my_tiles && ok; ++t) {
                const uint32_t m0 = (member + t * members) * BM;
                for (uint32_t kb = 0; kb < KB; ++kb, ++it) {
                    const uint32_t s = it % STAGES;
                    if (it >= STAGES && !ws_wait(&empty[s], ((it / STAGES) & 1u) ^ 1u, s_error)) {
                        atomicCAS(s_error, 0u, 1u);
                        ok = false;
                        break;
                    }
                    uint8_t* st = a_ring + s * stage_bytes;
                    ptx::mbar_arrive_expect_tx(&full[s], stage_bytes);
                    ptx::tma_load_2d(st, &maps.a[z][0], &full[s], (int32_t)(kb * BK), (int32_t)m0);
                    if (p.n_a == 2)
                        ptx::tma_load_2d(st + TILE_BYTES, &maps.a[z][1], &full[s], (int32_t)(kb * BK), (int32_t)m0);
                    if (!RESIDENT_W)
                        ptx::tma_load_2d(st + p.n_a * TILE_BYTES, &maps.b[z], &full[s], (int32_t)(kb * BK), (int32_t)n0);
                }
            }
            if (!ok) {
                // leave no copy in flight: wait (bounded) for every stage this thread filled last
                const uint32_t first = it > STAGES ? it - STAGES : 0;
                for (uint32_t k = first; k < it; ++k) ptx::mbar_wait(&full[k % STAGES], (k / STAGES) & 1u);
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------- MMA issuer
        if (ptx::elect_one()) {
            const uint32_t idesc = ptx::idesc_f16(p.a_fmt, p.b_fmt, BM, BN);
            const uint32_t w_addr = ptx::smem_u32(w_tiles);
            uint32_t it = 0;
            bool ok = true;
            for (uint32_t t = 0; t < my_tiles && ok; ++t) {
                const uint32_t buf = t & 1u;
                if (t >= 2 && !ws_wait(&tmem_empty[buf], ((t >> 1) & 1u) ^ 1u, s_error)) {
                    atomicCAS(s_error, 0u, 2u);
                    break;
                }
                ptx::tc_fence_after_sync();
                const uint32_t acc = tmem_base + buf * BN;
                for (uint32_t kb = 0; kb < KB; ++kb, ++it) {
                    const uint32_t s = it % STAGES;
                    if (!ws_wait(&full[s], (it / STAGES) & 1u, s_error)) {
                        atomicCAS(s_error, 0u, 3u);
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after_sync();
                    const uint32_t a_addr = ptx::smem_u32(a_ring + s * stage_bytes);
                    const uint32_t b_addr = RESIDENT_W ? w_addr + kb * TILE_BYTES : a_addr + p.n_a * TILE_BYTES;
#pragma unroll
                    for (uint32_t k4 = 0; k4 < BK / 16; ++k4) {
                        const uint64_t db = ptx::smem_desc_sw128(b_addr + k4 * 32);
                        ptx::mma_f16_ss(acc, ptx::smem_desc_sw128(a_addr + k4 * 32), db, idesc, (kb | k4) != 0);
                        if (p.n_a == 2)
                            ptx::mma_f16_ss(acc, ptx::smem_desc_sw128(a_addr + TILE_BYTES + k4 * 32), db, idesc, 1u);
                    }
                    ptx::mma_commit(&empty[s]);
                }
                ptx::mma_commit(&tmem_full[buf]);  // also on the error path: the epilogue does not wait in vain
            }
        }
    } else {
        // ---------------------------------------------------------- epilogue
        // this warp may only touch TMEM lanes 32*(warp%4) .. +31; warps 2-5 take the
        // left half of the tile's columns, warps 6-9 the right half
        const uint32_t quarter = warp & 3;
        const uint32_t group = (uint32_t)(warp - 2) >> 2;
        const uint32_t chunks = (BN / 32) / WS_EPI_GROUPS;
        const uint32_t row_in_tile = quarter * 32 + lane;
        for (uint32_t t = 0; t < my_tiles; ++t) {
            const uint32_t buf = t & 1u;
            const uint32_t m = (member + t * members) * BM + row_in_tile;
            // the accumulator loads below are warp-collective: decide for the whole warp
            if (!__all_sync(0xffffffffu, ws_wait(&tmem_full[buf], (t >> 1) & 1u, s_error))) {
                atomicCAS(s_error, 0u, 4u);
                break;
            }
            ptx::tc_fence_after_sync();
            if (__any_sync(0xffffffffu, *reinterpret_cast<volatile uint32_t*>(s_error) != 0u)) break;
            const uint32_t taddr = tmem_base + buf * BN + ((quarter * 32) << 16);
            epilogue<EPI>(p, pr, taddr, m, n0, s_scale, s_bias, lane, n_tile * WS_EPI_GROUPS + group, group * chunks,
                          (group + 1) * chunks, stage_base + (warp - 2) * (STAGE_BYTES / 4));
            ptx::tc_fence_before_sync();
            ptx::mbar_arrive(&tmem_empty[buf]);
        }
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, 256);
    }
    if (threadIdx.x == 0 && *s_error) {
        if (atomicCAS(p.status, ULLIS_DEV_OK, ULLIS_DEV_WAIT_TIMEOUT) == ULLIS_DEV_OK) p.status[1] = 16u + *s_error;
    }
}

}  // namespace tc
}  // namespace ullis
