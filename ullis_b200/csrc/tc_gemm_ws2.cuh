// CTA-pair form of the weight-stationary GEMM (tc_gemm_ws.cuh) for packed +/-1 weights with K <= 512.
//
// Two CTAs of a cluster of two share one 256 x 256 output tile per step (tcgen05.mma.cta_group::2,
// M = 256, N = 256): CTA r of the pair keeps the 128 weight rows n0 + 128 r .. + 127 expanded in its
// shared memory for its whole life and streams the 128 activation rows m0 + 128 r .. + 127 of every row
// tile through its own TMA ring; the even CTA issues the MMAs, which read A and half of B from each
// CTA's shared memory, and each CTA finds the 128 x 256 accumulator of its rows in its own TMEM.  An
// activation byte fetched from L2 now feeds 256 output columns instead of 128, which is what the
// single-CTA form runs short of.
//
// Barriers (same offsets in both CTAs): full[s] of the EVEN CTA counts the ring bytes of both CTAs
// (loads without multicast whose completion is signalled to the even CTA); empty[s] and tmem_full[b] of
// both CTAs are arrived by the even CTA's commits; tmem_empty[b] of the even CTA collects one arrival
// per epilogue warp of both CTAs.  Every wait is bounded; a cluster barrier before the TMEM release
// keeps either CTA's shared memory and barriers alive until the other is done with them.
#pragma once
#include "tc_gemm_ws.cuh"

namespace ullis {
namespace tc {

constexpr uint32_t WS2_BN = 256;           // output columns per pair
constexpr uint32_t WS2_BM = 256;           // output rows per pair and step
constexpr uint32_t WS2_EPI_WARPS = 16;     // four per TMEM lane quarter, 64 of the 256 columns each
constexpr int WS2_THREADS = 64 + 32 * (int)WS2_EPI_WARPS;   // TMA warp, MMA warp, epilogue warps

constexpr uint32_t WS2_STAGE16_BYTES = 32 * 64;   // per epilogue warp: 32 rows x 32 16-bit outputs (EPI_RELU2)

// bytes of store-staging buffer per epilogue warp
inline uint32_t ws2_staging(int epi) {
    return (epi == EPI_STORE || epi == EPI_RESIDUAL) ? (uint32_t)STAGE_BYTES : epi == EPI_RELU2 ? WS2_STAGE16_BYTES : 0u;
}

inline WsShape ws2_shape(uint32_t K, uint32_t n_a, int epi, bool resident_w = true) {
    const uint32_t kb = K / BK;
    const uint32_t fixed = 1024 /*alignment slack*/ + (resident_w ? kb * TILE_BYTES : 0) + 2 * WS2_BN * 2 + 256 +
                           WS2_EPI_WARPS * ws2_staging(epi);
    if (!resident_w) n_a += 1;   // this CTA's half of the weight tile travels with its activations
    uint32_t stages = (WS_SMEM_LIMIT - fixed) / (n_a * TILE_BYTES);
    if (stages > WS_MAX_STAGES) stages = WS_MAX_STAGES;
    return WsShape{stages, fixed + stages * n_a * TILE_BYTES};
}

// RESIDENT_W = false: dense 16-bit weights of any K; each CTA fetches the 128 weight rows of its half of the
// pair's 256 columns by TMA into the same ring stage as its activations (nothing stays resident).
template <int EPI, bool RESIDENT_W = true>
__global__ void __launch_bounds__(WS2_THREADS, 1)
gemm_ws2_kernel(const __grid_constant__ GemmMaps maps, const GemmParams p, const uint32_t pairs) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t KB = p.K / BK;
    const uint32_t STAGES = p.stages;
    const uint32_t stage_bytes = (p.n_a + (RESIDENT_W ? 0u : 1u)) * TILE_BYTES;
    uint8_t* w_tiles = smem;                               // [KB] this CTA's 128 weight rows
    uint8_t* a_ring = smem + (RESIDENT_W ? KB * TILE_BYTES : 0u);   // [STAGES] this CTA's 128 activation (+ weight) rows
    uint4* lut = reinterpret_cast<uint4*>(a_ring);         // only until the weights are expanded
    __half* s_scale = reinterpret_cast<__half*>(a_ring + STAGES * stage_bytes);   // [256] all columns of the pair
    __half* s_bias = s_scale + WS2_BN;
    uint64_t* bars = reinterpret_cast<uint64_t*>(s_bias + WS2_BN);
    uint64_t* full = bars;                                 // [STAGES] even CTA: ring bytes of both CTAs landed
    uint64_t* empty = bars + WS_MAX_STAGES;                // [STAGES] MMAs that read the stage are done
    uint64_t* tmem_full = bars + 2 * WS_MAX_STAGES;        // [2] accumulator complete
    uint64_t* tmem_empty = tmem_full + 2;                  // [2] even CTA: accumulator drained in both CTAs
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
    uint32_t* s_error = tmem_slot + 1;
    float* stage_base = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(bars) + 256);   // STORE / RESIDUAL / RELU2 only

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = ptx::cluster_ctarank();
    // work split: a pair of CTAs owns one (problem, 256-column tile); the pairs that own the same one
    // interleave over the 256-row tiles
    const uint32_t cluster = blockIdx.x >> 1, clusters = gridDim.x >> 1;
    const uint32_t owner = cluster % pairs, member = cluster / pairs;
    const uint32_t members = (clusters - owner + pairs - 1) / pairs;
    const uint32_t n_tiles = (p.N + WS2_BN - 1) / WS2_BN;
    const uint32_t z = owner / n_tiles, n_tile = owner % n_tiles;
    const uint32_t n0 = n_tile * WS2_BN;
    const uint32_t m_tiles = (p.M + WS2_BM - 1) / WS2_BM;
    const uint32_t my_tiles = member < m_tiles ? (m_tiles - member + members - 1) / members : 0;
    const GemmProblem& pr = p.prob[z];

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < STAGES; ++s) {
            ptx::mbar_init(&full[s], 1);
            ptx::mbar_init(&empty[s], 1);
        }
        for (uint32_t b = 0; b < 2; ++b) {
            ptx::mbar_init(&tmem_full[b], 1);
            ptx::mbar_init(&tmem_empty[b], 2 * WS2_EPI_WARPS);
        }
        *s_error = 0;
        ptx::fence_mbar_init();
        ptx::tma_prefetch_desc(&maps.a[z][0]);
        if (p.n_a == 2) ptx::tma_prefetch_desc(&maps.a[z][1]);
        if (!RESIDENT_W) ptx::tma_prefetch_desc(&maps.b[z]);
    }
    // 8 weight bits -> 8 FP16 values (+1.0 = 0x3C00, -1.0 = 0xBC00), bit i -> element i
    for (int b = threadIdx.x; RESIDENT_W && b < 256; b += WS2_THREADS) {
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t lo = (b >> (2 * j)) & 1u, hi = (b >> (2 * j + 1)) & 1u;
            w[j] = (lo ? 0x3C00u : 0xBC00u) | ((hi ? 0x3C00u : 0xBC00u) << 16);
        }
        lut[b] = make_uint4(w[0], w[1], w[2], w[3]);
    }
    if (threadIdx.x < WS2_BN) {   // FP16 as stored: 1 and 0 stand for a missing scale / bias
        const uint32_t n = n0 + threadIdx.x;
        s_scale[threadIdx.x] = (pr.scale && n < p.N) ? __ushort_as_half(pr.scale[n]) : __ushort_as_half(0x3C00);
        s_bias[threadIdx.x] = (pr.bias && n < p.N) ? __ushort_as_half(pr.bias[n]) : __ushort_as_half(0);
    }
    if (warp == 1) {
        ptx::tmem_alloc_pair(tmem_slot, 512);
        ptx::tmem_relinquish_pair();
    }
    __syncthreads();
    // expand this CTA's 128 weight rows once: row r of k-block kb -> 128 bytes, 16-byte chunk j at j ^ (r % 8)
    for (uint32_t item = threadIdx.x; RESIDENT_W && item < KB * BN; item += WS2_THREADS) {
        const uint32_t r = item % BN, kb = item / BN;
        const uint32_t n = n0 + rank * BN + r;
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
    __syncthreads();                // the table is dead, the ring may be filled
    ptx::cluster_sync_all();        // both CTAs: barriers initialised, weights expanded, TMEM allocated
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------ TMA producer (both CTAs, own rows)
        if (ptx::elect_one()) {
            const uint32_t full_even = ptx::cluster_map(full, 0);
            uint32_t it = 0;
            bool ok = true;
            for (uint32_t t = 0; t < my_tiles && ok; ++t) {
                const uint32_t m0 = (member + t * members) * WS2_BM + rank * BM;
                for (uint32_t kb = 0; kb < KB; ++kb, ++it) {
                    const uint32_t s = it % STAGES;
                    if (it >= STAGES && !ws_wait(&empty[s], ((it / STAGES) & 1u) ^ 1u, s_error)) {
                        atomicCAS(s_error, 0u, 1u);
                        ok = false;
                        break;
                    }
                    uint8_t* st = a_ring + s * stage_bytes;
                    if (rank == 0) ptx::mbar_arrive_expect_tx(&full[s], 2 * stage_bytes);
                    ptx::tma_load_2d_pair(st, &maps.a[z][0], full_even + 8 * s, (int32_t)(kb * BK), (int32_t)m0);
                    if (p.n_a == 2)
                        ptx::tma_load_2d_pair(st + TILE_BYTES, &maps.a[z][1], full_even + 8 * s, (int32_t)(kb * BK),
                                              (int32_t)m0);
                    if (!RESIDENT_W)
                        ptx::tma_load_2d_pair(st + p.n_a * TILE_BYTES, &maps.b[z], full_even + 8 * s, (int32_t)(kb * BK),
                                              (int32_t)(n0 + rank * BN));
                }
            }
            if (!ok && rank == 0) {
                // leave no copy in flight: wait (bounded) for every stage this thread filled last (both CTAs'
                // bytes of a stage are counted on these barriers)
                const uint32_t first = it > STAGES ? it - STAGES : 0;
                for (uint32_t k = first; k < it; ++k) ptx::mbar_wait(&full[k % STAGES], (k / STAGES) & 1u);
            }
            if (!ok && rank == 1) {
                // The odd CTA's copies complete on the even CTA's barriers, which it cannot poll.  A copy it
                // issued goes into a stage the MMAs had released and lands within microseconds; the wait that
                // failed just before took about a second.  Give the last ones far longer than they need
                // before this CTA may leave (the cluster barrier below comes after).
                for (int i = 0; i < 64; ++i) __nanosleep(1000);
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------- MMA issuer (even CTA only)
        if (rank == 0 && ptx::elect_one()) {
            const uint32_t idesc = ptx::idesc_f16(p.a_fmt, p.b_fmt, WS2_BM, WS2_BN);
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
                const uint32_t acc = tmem_base + buf * WS2_BN;
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
                        ptx::mma_f16_ss_pair(acc, ptx::smem_desc_sw128(a_addr + k4 * 32), db, idesc, (kb | k4) != 0);
                        if (p.n_a == 2)
                            ptx::mma_f16_ss_pair(acc, ptx::smem_desc_sw128(a_addr + TILE_BYTES + k4 * 32), db, idesc, 1u);
                    }
                    ptx::mma_commit_pair(&empty[s]);
                }
                ptx::mma_commit_pair(&tmem_full[buf]);  // also on the error path: the epilogues do not wait in vain
            }
        }
    } else {
        // ---------------------------------------------------------- epilogue (both CTAs, own rows)
        // this warp may only touch TMEM lanes 32*(warp%4) .. +31; the four warps of a lane quarter take
        // 64 of the pair's 256 columns each (for the CE epilogue that is one (max, sum exp) partial, the
        // granularity of the single-CTA form, so a row's loss does not depend on which kernel the batch selects)
        const uint32_t quarter = warp & 3;
        const uint32_t group = (uint32_t)(warp - 2) >> 2;
        const uint32_t row_in_tile = quarter * 32 + lane;
        const uint32_t drained_even = ptx::cluster_map(tmem_empty, 0);
        // EPI_RESIDUAL reads the f32 rows it updates: ask L2 for this lane's 256 bytes of the next tile while the
        // current one is drained, so that the read does not pay the HBM latency inside the epilogue (packed weights
        // only: with dense weights the ring already keeps the memory system busy and the prefetch costs time)
        auto prefetch_rows = [&](uint32_t t) {
            const uint32_t mp = (member + t * members) * WS2_BM + rank * BM + row_in_tile;
            if (EPI == EPI_RESIDUAL && RESIDENT_W && t < my_tiles && mp < p.M && n0 + group * 64 < p.N) {
                const float* q = static_cast<const float*>(pr.out) + (size_t)mp * p.N + n0 + group * 64;
                asm volatile("prefetch.global.L2 [%0];" ::"l"(q));
                asm volatile("prefetch.global.L2 [%0];" ::"l"(q + 32));
            }
        };
        prefetch_rows(0);
        for (uint32_t t = 0; t < my_tiles; ++t) {
            const uint32_t buf = t & 1u;
            const uint32_t m = (member + t * members) * WS2_BM + rank * BM + row_in_tile;
            prefetch_rows(t + 1);
            // the accumulator loads below are warp-collective: decide for the whole warp
            if (!__all_sync(0xffffffffu, ws_wait(&tmem_full[buf], (t >> 1) & 1u, s_error))) {
                atomicCAS(s_error, 0u, 4u);
                break;
            }
            ptx::tc_fence_after_sync();
            if (__any_sync(0xffffffffu, *reinterpret_cast<volatile uint32_t*>(s_error) != 0u)) break;
            const uint32_t taddr = tmem_base + buf * WS2_BN + group * 64 + ((quarter * 32) << 16);
            epilogue<EPI, __half, EPI == EPI_RELU2>(
                p, pr, taddr, m, n0 + group * 64, s_scale + group * 64, s_bias + group * 64, lane, n_tile * 4 + group, 0, 2,
                stage_base + (warp - 2) * ((EPI == EPI_RELU2 ? WS2_STAGE16_BYTES : (uint32_t)STAGE_BYTES) / 4));
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive_cluster(drained_even + 8 * buf);
        }
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::cluster_sync_all();        // neither CTA leaves while the other may still read its tiles or ring its barriers
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc_pair(tmem_base, 512);
    }
    if (threadIdx.x == 0 && *s_error) {
        if (atomicCAS(p.status, ULLIS_DEV_OK, ULLIS_DEV_WAIT_TIMEOUT) == ULLIS_DEV_OK) p.status[1] = 32u + *s_error;
    }
}

}  // namespace tc
}  // namespace ullis
