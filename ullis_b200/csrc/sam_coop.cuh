// Warp-cooperative second half of the O(T log T) suffix-automaton match: the
// preorder numbering of the suffix-link tree ("tour") and the replay of time
// over a max tree ("pass 2"), for ONE stream per warp with the working set in
// shared memory.  Pass 1 (the automaton itself) is an inherently serial
// pointer chase and stays one-thread-per-stream in sam.cu; these two phases
// parallelise over states / steps, so a warp does them in far fewer issued
// instructions and without global-memory round trips.
//
//  tour   (whole CTA, 128 threads) Euler tour of the link tree as a linked
//         list of 2n events (enter v, leave v); the rank of every event
//         (number of stamped states entered before it) by in-place pointer
//         jumping over packed (successor, partial sum) words - log2(2n)
//         rounds, all lanes busy.
//  pass 2 (warp 0) 32 steps per round, one step per lane: each lane answers its
//         range maximum from a 16-ary max tree holding the stamps of earlier
//         rounds, takes the stamps of earlier lanes of the same round by
//         shuffles, then all lanes insert their own stamp (one shared-memory
//         atomicMax per tree level).
//
// 16-bit state ids only (2T+2 <= 65535); the caller falls back to the
// one-thread-per-stream routine for longer streams or when the block does not
// fit shared memory.
#pragma once
#include "sam_core.cuh"

namespace ullis {
namespace sam {

constexpr int COOP_THREADS = 128;

struct CoopLayout {
    uint32_t ev, kid, parent, clone_bits, vbits, total;
    __host__ __device__ explicit CoopLayout(uint32_t T) {
        const uint32_t cap = node_capacity(T), wps = (T + 31) / 32;
        uint32_t off = 0;
        const uint32_t ev_bytes = cap * 2 * 4, tree_bytes = tree_entries(T) * 4;
        ev = off;         off += ev_bytes > tree_bytes ? ev_bytes : tree_bytes;   // events, later the max tree
        kid = off;        off += cap * 4;                                        // child pairs, later {lo,hi}
        parent = off;     off += (cap * 2 + 15) & ~15u;
        clone_bits = off; off += (((cap + 31) / 32) * 4 + 15) & ~15u;
        vbits = off;      off += (wps * 4 + 15) & ~15u;
        total = off;
    }
};

#if defined(__CUDACC__)
// max of the entries of one 16-entry group whose index (first + e) lies in [l, r)
__device__ __forceinline__ uint32_t group_max(const uint32_t* g, uint32_t first, uint32_t l, uint32_t r) {
    const uint4* q = reinterpret_cast<const uint4*>(g);
    const uint4 a = q[0], b = q[1], c = q[2], d = q[3];
    const uint32_t val[16] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w, c.x, c.y, c.z, c.w, d.x, d.y, d.z, d.w};
    uint32_t m = 0;
#pragma unroll
    for (uint32_t e = 0; e < 16; ++e)
        if (first + e - l < r - l) m = max(m, val[e]);
    return m;
}

// One CTA of COOP_THREADS threads; `B` is the stream's global scratch block
// after euler_pass1.  Every thread of the CTA must call this.
__device__ __forceinline__ void coop_tour_pass2(uint8_t* smem, const EulerBlock<uint16_t>& B, const uint32_t* vw,
                                                uint32_t* out, uint32_t T) {
    constexpr uint32_t NIL = 0xFFFFu, END = 0xFFFFu;
    const int tid = threadIdx.x, lane = tid & 31;
    const CoopLayout L(T);
    uint32_t* ev = reinterpret_cast<uint32_t*>(smem + L.ev);
    uint32_t* kid = reinterpret_cast<uint32_t*>(smem + L.kid);
    uint16_t* parent = reinterpret_cast<uint16_t*>(smem + L.parent);
    uint32_t* cbits = reinterpret_cast<uint32_t*>(smem + L.clone_bits);
    uint32_t* vbits = reinterpret_cast<uint32_t*>(smem + L.vbits);
    const uint32_t n = B.meta[0], wps = (T + 31) / 32;
    const uint32_t cap = node_capacity(T);

    // ---- stage: suffix links, clone bitmap, v bits.  The smallest / largest
    // child id of every state are collected with one atomicMin / atomicMax
    // each (a binary alphabet gives a state at most two link children); the
    // second array borrows the upper half of the event area for a moment.
    uint32_t* kid_min = kid;
    uint32_t* kid_max = ev + cap;
    const uint2* nodes = reinterpret_cast<const uint2*>(B.N);
    for (uint32_t v = tid; v < n; v += COOP_THREADS) {
        parent[v] = (uint16_t)(nodes[v].y & 0xFFFFu);  // Node = {t0, t1 | fail, maxlen}
        kid_min[v] = 0xFFFFFFFFu;
        kid_max[v] = 0u;
    }
    for (uint32_t w = tid; w < (n + 31) / 32; w += COOP_THREADS) cbits[w] = B.clone_bits[w];
    for (uint32_t w = tid; w < wps; w += COOP_THREADS) vbits[w] = vw[w];
    __syncthreads();
    for (uint32_t v = 1 + tid; v < n; v += COOP_THREADS) {
        const uint32_t p = parent[v];
        atomicMin(&kid_min[p], v);
        atomicMax(&kid_max[p], v);
    }
    __syncthreads();
    for (uint32_t v = tid; v < n; v += COOP_THREADS) {
        const uint32_t a = kid_min[v], b = kid_max[v];
        kid[v] = a == 0xFFFFFFFFu ? 0xFFFFFFFFu : (a | ((a == b ? NIL : b) << 16));
    }
    __syncthreads();

    // ---- Euler tour as a list: event 2v = enter v, 2v+1 = leave v; word = successor | weight << 16
    for (uint32_t v = tid; v < n; v += COOP_THREADS) {
        const uint32_t k = kid[v], a = k & 0xFFFFu;
        const uint32_t stamped = (v != 0 && !((cbits[v >> 5] >> (v & 31)) & 1u)) ? 1u : 0u;
        ev[2 * v] = (a != NIL ? 2 * a : 2 * v + 1) | (stamped << 16);
        uint32_t succ = END;
        if (v != 0) {
            const uint32_t p = parent[v], kp = kid[p];
            succ = ((kp & 0xFFFFu) == v && (kp >> 16) != NIL) ? 2 * (kp >> 16) : 2 * p + 1;
        }
        ev[2 * v + 1] = succ;
    }
    __syncthreads();
    // pointer jumping, in place: a word is read and written as a whole, so a
    // reader always sees a consistent (successor, sum over [e, successor)) pair
    uint32_t rounds = 1;
    while ((1u << rounds) < 2 * n) ++rounds;
    for (uint32_t it = 0; it <= rounds; ++it) {
        int any = 0;
        // eight independent elements per thread and step: the two dependent
        // shared-memory loads of one element overlap with those of the others
        for (uint32_t e0 = tid; e0 < 2 * n; e0 += COOP_THREADS * 8) {
            uint32_t w[8], w2[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const uint32_t e = e0 + COOP_THREADS * u;
                w[u] = e < 2 * n ? ev[e] : END;
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) w2[u] = (w[u] & 0xFFFFu) != END ? ev[w[u] & 0xFFFFu] : 0u;
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                if ((w[u] & 0xFFFFu) != END) {
                    ev[e0 + COOP_THREADS * u] = (w2[u] & 0xFFFFu) | ((w[u] & 0xFFFF0000u) + (w2[u] & 0xFFFF0000u));
                    any = 1;
                }
            }
        }
        if (!__syncthreads_or(any)) break;
    }
    // rank range of state v: stamped states entered before enter(v) / before leave(v)
    const uint32_t total = ev[0] >> 16;
    uint32_t* lh = kid;  // child pairs are dead; same element size
    for (uint32_t v = tid; v < n; v += COOP_THREADS) {
        const uint32_t lo = total - (ev[2 * v] >> 16), hi = total - (ev[2 * v + 1] >> 16);
        lh[v] = lo | (hi << 16);
    }
    __syncthreads();

    // ---- pass 2: 16-ary max tree (level 0 = ranks, level k+1 = maxima of groups of 16)
    uint32_t* tree = ev;  // events are dead
    const uint32_t entries = tree_entries(T);
    for (uint32_t k = tid; k < entries; k += COOP_THREADS) tree[k] = 0;
    __syncthreads();
    if (tid >= 32) return;
    const uint32_t size0 = (T + 15u) & ~15u;
    // the query states / new states of a round come from global memory: fetch one round ahead
    uint32_t v_next = (uint32_t)lane < T ? B.vq[lane] : NIL, j_next = (uint32_t)lane < T ? B.jid[lane] : 0u;
    for (uint32_t t0 = 0; t0 < T; t0 += 32) {
        const uint32_t t = t0 + lane;
        const bool live = t < T;
        const uint32_t v = v_next, j = j_next;
        if (t + 32 < T) { v_next = B.vq[t + 32]; j_next = B.jid[t + 32]; }
        uint32_t lo = 0, hi = 0, my_rank = 0xFFFFFFFFu, m = 0;
        if (live) {
            my_rank = lh[j] & 0xFFFFu;
            if (v != NIL) {
                const uint32_t r = lh[v];
                lo = r & 0xFFFFu;
                hi = r >> 16;
                // whole 16-entry groups are loaded with 128-bit loads and masked in
                // registers: no data-dependent trip counts, no dependent loads
                uint32_t l = lo, rr = hi, base = 0, size = size0;
                while (l < rr) {
                    const uint32_t lg = l >> 4, rg = (rr - 1u) >> 4;
                    m = max(m, group_max(tree + base + (lg << 4), lg << 4, l, rr));
                    if (rg != lg) m = max(m, group_max(tree + base + (rg << 4), rg << 4, l, rr));
                    if (rg <= lg + 1u) break;      // no whole group in between
                    l = lg + 1u; rr = rg;          // the groups in between, one level up
                    base += size;
                    size = ((size >> 4) + 15u) & ~15u;
                }
            }
        }
        // stamps of earlier steps of this round: the highest earlier lane whose rank is in range
        uint32_t hits = 0;
        const uint32_t width = hi - lo;
#pragma unroll
        for (int i = 0; i < 31; ++i) {
            const uint32_t r_i = __shfl_sync(0xffffffffu, my_rank, i);
            hits |= (r_i - lo < width ? 1u : 0u) << i;   // lanes past T carry rank 0xFFFFFFFF: never in range
        }
        hits &= (1u << lane) - 1u;
        if (hits) m = t0 + (31 - __clz(hits)) + 1;       // newer than anything in the tree
        uint32_t bit = 0;
        if (live && v != NIL && m) bit = (vbits[m >> 5] >> (m & 31)) & 1u;
        const uint32_t word = __ballot_sync(0xffffffffu, bit != 0);
        if (lane == 0) out[t0 >> 5] = word;
        __syncwarp();
        if (live) {
            uint32_t pos = my_rank, base = 0, size = size0;
            for (;;) {
                atomicMax(&tree[base + pos], t + 1);
                if (size <= 16u) break;
                base += size;
                size = ((size >> 4) + 15u) & ~15u;
                pos >>= 4;
            }
        }
        __syncwarp();
    }
}
#endif

}  // namespace sam
}  // namespace ullis
