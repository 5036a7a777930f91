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
//  pass 2 (whole CTA) 128 steps per round, one step per thread: each thread
//         answers its range maximum from a 16-ary max tree holding the stamps
//         of earlier rounds, takes the stamps of earlier steps of the same round
//         from the round's published ranks (shuffles inside the warp, broadcast
//         loads for earlier warps), then all threads insert their own stamp (one
//         shared-memory atomicMax per tree level).
//
// 16-bit state ids only (2T+2 <= 65535); the caller falls back to the
// one-thread-per-stream routine for longer streams or when the block does not
// fit shared memory.
#pragma once
#include "sam_core.cuh"

namespace ullis {
namespace sam {

constexpr int COOP_THREADS = 128;

// Optional phase timestamps for a profiling build (defined by the includer); nothing by default.
#ifndef ULLIS_COOP_MARK
#define ULLIS_COOP_MARK_BEGIN()
#define ULLIS_COOP_MARK(i)
#endif

struct CoopLayout {
    uint32_t ev, kid, parent, clone_bits, vbits, round_rank, total;
    __host__ __device__ explicit CoopLayout(uint32_t T) {
        const uint32_t cap = node_capacity(T), wps = (T + 31) / 32;
        uint32_t off = 0;
        const uint32_t ev_bytes = cap * 2 * 4, tree_bytes = tree_entries(T) * 4;
        ev = off;         off += ev_bytes > tree_bytes ? ev_bytes : tree_bytes;   // events, later the max tree
        kid = off;        off += (cap * 4 + 15) & ~15u;                          // child pairs, later {lo,hi}
        parent = off;     off += (cap * 2 + 15) & ~15u;
        clone_bits = off; off += (((cap + 31) / 32) * 4 + 15) & ~15u;
        vbits = off;      off += (wps * 4 + 15) & ~15u;
        round_rank = off; off += COOP_THREADS * 4;                                // ranks of the steps of one pass-2 round
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

// about one event index in eight, spread by a multiplicative hash; event 0 always
__device__ __forceinline__ bool is_splitter(uint32_t e) { return e == 0u || ((e * 0x9E3779B1u) >> 29) == 0u; }

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
    uint32_t* round_rank = reinterpret_cast<uint32_t*>(smem + L.round_rank);
    const uint32_t n = B.meta[0], wps = (T + 31) / 32;
    const uint32_t cap = node_capacity(T);
    ULLIS_COOP_MARK_BEGIN();

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
    if (tid == 0) round_rank[0] = 0;   // doubles as the splitter counter of the list ranking
    __syncthreads();
    ULLIS_COOP_MARK(0);
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

    ULLIS_COOP_MARK(1);
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
    ULLIS_COOP_MARK(2);
    // List ranking in two levels.  About one event in eight is a splitter
    // (chosen by a hash of the event index, so that no shape of the tree lines
    // up with it; event 0, the head of the list, always is).  Level 1: the
    // thread that owns a splitter walks its sublist up to the next splitter and
    // leaves in every element (weight of the sublist before it, its splitter);
    // the splitter gets (weight of the whole sublist, next splitter).  Level 2:
    // pointer jumping over the splitters only, in place - a word is read and
    // written as a whole, so a reader always sees a consistent (successor, sum
    // over [s, successor)) pair.  O(events) work instead of O(events log events).
    uint16_t* splitters = reinterpret_cast<uint16_t*>(kid);   // child pairs are dead
    uint32_t* n_splitters = round_rank;                          // free until pass 2
    for (uint32_t e = tid; e < 2 * n; e += COOP_THREADS)
        if (is_splitter(e)) splitters[atomicAdd(n_splitters, 1u)] = (uint16_t)e;
    __syncthreads();
    {
        // one hop per thread and iteration; a thread that reaches the end of a
        // sublist takes its next splitter in the same iteration, so the lanes of
        // a warp stay busy however the sublist lengths fall
        const uint32_t count = *n_splitters;
        uint32_t k = tid, head = 0, cur = 0, before = 0;
        bool busy = k < count;
        if (busy) head = cur = splitters[k];
        for (uint32_t hops = 0; busy && hops < 2 * n; ++hops) {   // all sublists together are no longer than the list
            const uint32_t w = ev[cur];
            const uint32_t nxt = w & 0xFFFFu;
            if (cur != head) ev[cur] = (before << 16) | head;
            before += w >> 16;
            if (nxt == END || is_splitter(nxt)) {
                ev[head] = (before << 16) | nxt;
                k += COOP_THREADS;
                busy = k < count;
                if (busy) head = cur = splitters[k];
                before = 0;
            } else {
                cur = nxt;
            }
        }
    }
    __syncthreads();
    ULLIS_COOP_MARK(3);
    const uint32_t ns = *n_splitters;
    uint32_t rounds = 1;
    while ((1u << rounds) < ns) ++rounds;
    for (uint32_t it = 0; it <= rounds; ++it) {
        int any = 0;
        for (uint32_t k = tid; k < ns; k += COOP_THREADS) {
            const uint32_t sp = splitters[k];
            const uint32_t w = ev[sp];
            if ((w & 0xFFFFu) != END) {
                const uint32_t w2 = ev[w & 0xFFFFu];
                ev[sp] = (w2 & 0xFFFFu) | ((w & 0xFFFF0000u) + (w2 & 0xFFFF0000u));
                any = 1;
            }
        }
        if (!__syncthreads_or(any)) break;
    }
    ULLIS_COOP_MARK(4);
    // weight of [e, end of list): the splitter's, less what lies before e in its sublist
    auto weight_from = [&](uint32_t e) {
        const uint32_t w = ev[e];
        return is_splitter(e) ? (w >> 16) : (ev[w & 0xFFFFu] >> 16) - (w >> 16);
    };
    // rank range of state v: stamped states entered before enter(v) / before leave(v)
    const uint32_t total = ev[0] >> 16;
    uint32_t* lh = kid;  // the splitter list is dead; same element size as the child pairs
    for (uint32_t v = tid; v < n; v += COOP_THREADS) {
        const uint32_t lo = total - weight_from(2 * v), hi = total - weight_from(2 * v + 1);
        lh[v] = lo | (hi << 16);
    }
    __syncthreads();

    // ---- pass 2: 16-ary max tree (level 0 = ranks, level k+1 = maxima of groups of 16)
    uint32_t* tree = ev;  // events are dead
    const uint32_t entries = tree_entries(T);
    for (uint32_t k = tid; k < entries; k += COOP_THREADS) tree[k] = 0;
    __syncthreads();
    ULLIS_COOP_MARK(5);
    // One round = COOP_THREADS consecutive steps, one per thread.  A step may be
    // answered by a stamp of an earlier step of the same round; those are not in
    // the tree yet, so the ranks of the round are published in shared memory
    // (`round_rank`) and searched newest first: the
    // own warp's earlier lanes by shuffles, the earlier warps' by broadcast loads.
    const uint32_t size0 = (T + 15u) & ~15u;
    const int warp = tid >> 5;
    uint32_t v_next = (uint32_t)tid < T ? B.vq[tid] : NIL, j_next = (uint32_t)tid < T ? B.jid[tid] : 0u;
    for (uint32_t t0 = 0; t0 < T; t0 += COOP_THREADS) {
        const uint32_t t = t0 + tid;
        const bool live = t < T;
        const uint32_t v = v_next, j = j_next;
        if (t + COOP_THREADS < T) { v_next = B.vq[t + COOP_THREADS]; j_next = B.jid[t + COOP_THREADS]; }
        uint32_t lo = 0, hi = 0, my_rank = 0xFFFFFFFFu, m = 0;
        if (live) {
            my_rank = lh[j] & 0xFFFFu;
            if (v != NIL) {
                const uint32_t r = lh[v];
                lo = r & 0xFFFFu;
                hi = r >> 16;
            }
        }
        round_rank[tid] = my_rank;
        if (lo < hi) {
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
        __syncthreads();   // ranks of the round published; every tree read of the round done
        // earlier lanes of the own warp: the highest one whose rank is in range
        uint32_t hits = 0;
        const uint32_t width = hi - lo;
#pragma unroll
        for (int i = 0; i < 31; ++i) {
            const uint32_t r_i = __shfl_sync(0xffffffffu, my_rank, i);
            hits |= (r_i - lo < width ? 1u : 0u) << i;   // lanes past T carry rank 0xFFFFFFFF: never in range
        }
        hits &= (1u << lane) - 1u;
        if (hits) {
            m = t0 + warp * 32 + (31 - __clz(hits)) + 1;   // newer than anything in the tree
        } else if (width != 0 && warp != 0) {
            // earlier warps of the round, newest group of four first
            for (int e = warp * 32 - 4; e >= 0; e -= 4) {
                const uint4 r4 = *reinterpret_cast<const uint4*>(round_rank + e);
                const uint32_t f = (r4.x - lo < width ? 1u : 0u) | (r4.y - lo < width ? 2u : 0u) |
                                   (r4.z - lo < width ? 4u : 0u) | (r4.w - lo < width ? 8u : 0u);
                if (f) { m = t0 + e + (31 - __clz(f)) + 1; break; }
            }
        }
        uint32_t bit = 0;
        if (live && v != NIL && m) bit = (vbits[m >> 5] >> (m & 31)) & 1u;
        const uint32_t word = __ballot_sync(0xffffffffu, bit != 0);
        if (lane == 0 && t0 + warp * 32 < T) out[(t0 >> 5) + warp] = word;
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
        __syncthreads();   // the round's stamps are in the tree; round_rank may be overwritten
    }
    ULLIS_COOP_MARK(6);
}
#endif

}  // namespace sam
}  // namespace ullis
