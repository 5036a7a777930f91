// Warp-cooperative second half of the O(T log T) suffix-automaton match: the
// preorder numbering of the suffix-link tree ("tour") and the replay of time
// over a max tree ("pass 2"), for ONE stream per warp with the working set in
// shared memory.  Pass 1 (the automaton itself) is an inherently serial
// pointer chase and stays one-thread-per-stream in sam.cu; these two phases
// parallelise over states / steps, so a warp does them in far fewer issued
// instructions and without global-memory round trips.
//
//  tour   Euler tour of the link tree as a linked list of 2n events
//         (enter v, leave v); the rank of every event (number of stamped
//         states entered before it) by in-place pointer jumping over packed
//         (successor, partial sum) words - log2(2n) rounds, all lanes busy.
//  pass 2 32 steps per round, one step per lane: each lane answers its range
//         maximum from a binary max tree holding the stamps of earlier rounds,
//         takes the stamps of earlier lanes of the same round by shuffles,
//         then all lanes insert their own stamp (shared-memory atomicMax).
//
// 16-bit state ids only (2T+2 <= 65535); the caller falls back to the
// one-thread-per-stream routine for longer streams or when the block does not
// fit shared memory.
#pragma once
#include "sam_core.cuh"

namespace ullis {
namespace sam {

struct CoopLayout {
    uint32_t ev, kid, parent, clone_bits, vbits, total;
    __host__ __device__ explicit CoopLayout(uint32_t T) {
        const uint32_t cap = node_capacity(T), wps = (T + 31) / 32;
        uint32_t off = 0;
        const uint32_t ev_bytes = cap * 2 * 4, tree_bytes = 2 * pow2_at_least(T) * 4;
        ev = off;         off += ev_bytes > tree_bytes ? ev_bytes : tree_bytes;   // events, later the max tree
        kid = off;        off += cap * 4;                                        // child pairs, later {lo,hi}
        parent = off;     off += (cap * 2 + 15) & ~15u;
        clone_bits = off; off += (((cap + 31) / 32) * 4 + 15) & ~15u;
        vbits = off;      off += (wps * 4 + 15) & ~15u;
        total = off;
    }
};

#if defined(__CUDACC__)
// One warp; `B` is the stream's global scratch block after euler_pass1.
// Returns false if an invariant failed (more than two children of a state).
__device__ __forceinline__ bool coop_tour_pass2(uint8_t* smem, const EulerBlock<uint16_t>& B, const uint32_t* vw,
                                                uint32_t* out, uint32_t T) {
    constexpr uint32_t NIL = 0xFFFFu, END = 0xFFFFu;
    const int lane = threadIdx.x & 31;
    const CoopLayout L(T);
    uint32_t* ev = reinterpret_cast<uint32_t*>(smem + L.ev);
    uint32_t* kid = reinterpret_cast<uint32_t*>(smem + L.kid);
    uint16_t* parent = reinterpret_cast<uint16_t*>(smem + L.parent);
    uint32_t* cbits = reinterpret_cast<uint32_t*>(smem + L.clone_bits);
    uint32_t* vbits = reinterpret_cast<uint32_t*>(smem + L.vbits);
    const uint32_t n = B.meta[0], wps = (T + 31) / 32;
    bool ok = true;

    // ---- stage: suffix links, clone bitmap, v bits
    const uint2* nodes = reinterpret_cast<const uint2*>(B.N);
    for (uint32_t v = lane; v < n; v += 32) {
        parent[v] = (uint16_t)(nodes[v].y & 0xFFFFu);  // Node = {t0, t1 | fail, maxlen}
        kid[v] = 0xFFFFFFFFu;
    }
    for (uint32_t w = lane; w < (n + 31) / 32; w += 32) cbits[w] = B.clone_bits[w];
    for (uint32_t w = lane; w < wps; w += 32) vbits[w] = vw[w];
    __syncwarp();

    // ---- children pairs (a binary alphabet gives a state at most two link children)
    for (uint32_t v = 1 + lane; v < n; v += 32) {
        const uint32_t p = parent[v];
        uint32_t old = kid[p];
        for (;;) {
            uint32_t want;
            if ((old & 0xFFFFu) == NIL) want = (old & 0xFFFF0000u) | v;
            else if ((old >> 16) == NIL) want = (old & 0xFFFFu) | (v << 16);
            else { ok = false; break; }
            const uint32_t seen = atomicCAS(&kid[p], old, want);
            if (seen == old) break;
            old = seen;
        }
    }
    __syncwarp();

    // ---- Euler tour as a list: event 2v = enter v, 2v+1 = leave v; word = successor | weight << 16
    for (uint32_t v = lane; v < n; v += 32) {
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
    __syncwarp();
    // pointer jumping, in place: a word is read and written as a whole, so a
    // reader always sees a consistent (successor, sum over [e, successor)) pair
    uint32_t rounds = 1;
    while ((1u << rounds) < 2 * n) ++rounds;
    for (uint32_t it = 0; it <= rounds; ++it) {
        bool any = false;
        for (uint32_t e = lane; e < 2 * n; e += 32) {
            const uint32_t w = ev[e], s = w & 0xFFFFu;
            if (s != END) {
                const uint32_t w2 = ev[s];
                ev[e] = (w2 & 0xFFFFu) | ((w & 0xFFFF0000u) + (w2 & 0xFFFF0000u));
                any = true;
            }
        }
        if (!__any_sync(0xffffffffu, any)) break;
        __syncwarp();
    }
    __syncwarp();
    // rank range of state v: stamped states entered before enter(v) / before leave(v)
    const uint32_t total = ev[0] >> 16;
    uint32_t* lh = kid;  // child pairs are dead; same element size
    for (uint32_t v = lane; v < n; v += 32) {
        const uint32_t lo = total - (ev[2 * v] >> 16), hi = total - (ev[2 * v + 1] >> 16);
        lh[v] = lo | (hi << 16);
    }
    __syncwarp();

    // ---- pass 2
    const uint32_t Lp = pow2_at_least(T);
    uint32_t* tree = ev;  // events are dead
    for (uint32_t k = lane; k < 2 * Lp; k += 32) tree[k] = 0;
    __syncwarp();
    for (uint32_t t0 = 0; t0 < T; t0 += 32) {
        const uint32_t t = t0 + lane;
        const bool live = t < T;
        uint32_t v = NIL, lo = 0, hi = 0, my_rank = 0, m = 0;
        if (live) {
            v = B.vq[t];
            my_rank = lh[B.jid[t]] & 0xFFFFu;
            if (v != NIL) {
                const uint32_t r = lh[v];
                lo = r & 0xFFFFu;
                hi = r >> 16;
                uint32_t l = lo + Lp, rr = hi + Lp;
                while (l < rr) {
                    if (l & 1u) m = max(m, tree[l++]);
                    if (rr & 1u) m = max(m, tree[--rr]);
                    l >>= 1; rr >>= 1;
                }
            }
        }
        // stamps of earlier steps of this round
#pragma unroll 8
        for (int i = 0; i < 31; ++i) {
            const uint32_t r_i = __shfl_sync(0xffffffffu, my_rank, i);
            if (i < lane && t0 + i < T && r_i >= lo && r_i < hi) m = t0 + i + 1;  // increasing i: the last hit is the max
        }
        uint32_t bit = 0;
        if (live && v != NIL && m) bit = (vbits[m >> 5] >> (m & 31)) & 1u;
        const uint32_t word = __ballot_sync(0xffffffffu, bit != 0);
        if (lane == 0) out[t0 >> 5] = word;
        __syncwarp();
        if (live)
            for (uint32_t p = my_rank + Lp; p >= 1; p >>= 1) atomicMax(&tree[p], t + 1);
        __syncwarp();
    }
    return __all_sync(0xffffffffu, ok);
}
#endif

}  // namespace sam
}  // namespace ullis
