// Warp-cooperative second half of the O(T log T) suffix-automaton match: the
// preorder numbering of the suffix-link tree ("tour") and the replay of time
// over a max tree ("pass 2"), for ONE stream per warp with the working set in
// shared memory.  Pass 1 (the automaton itself) is an inherently serial
// pointer chase and stays one-thread-per-stream in sam.cu; these two phases
// parallelise over states / steps, so a warp does them in far fewer issued
// instructions and without global-memory round trips.
//
//  tour   (whole CTA, 256 to 1024 threads) Euler tour of the link tree as a linked
//         list of 2n events (enter v, leave v); the rank of every event
//         (number of stamped states entered before it) by two-level list
//         ranking: serial walks of short sublists between hashed splitters,
//         then pointer jumping over the splitters only.
//  pass 2 (whole CTA) the stamp of every rank is known up front (a state is
//         stamped once, when created), so a step with a narrow rank range scans
//         that array directly, all steps in parallel.  Steps with wide ranges
//         use a 16-ary max tree whose upper levels are replayed in rounds of one step per thread
//         (one shared-memory atomicMax per level and step); a stream
//         without wide ranges skips the replay.
//
// 16-bit state ids only (2T+2 <= 65535); the caller falls back to the
// one-thread-per-stream routine for longer streams or when the block does not
// fit shared memory.
#pragma once
#include "sam_core.cuh"

namespace ullis {
namespace sam {

constexpr int COOP_MAX_THREADS = 1024;   // the kernel runs with 256, 512 or 1024 threads per stream

// Optional phase timestamps for a profiling build (defined by the includer); nothing by default.
#ifndef ULLIS_COOP_MARK
#define ULLIS_COOP_MARK_BEGIN()
#define ULLIS_COOP_MARK(i)
#endif

struct CoopLayout {
    uint32_t ev, kid, clone_bits, vbits, round_rank, wide, ctrl, total;
    __host__ __device__ explicit CoopLayout(uint32_t T) {
        const uint32_t cap = node_capacity(T), wps = (T + 31) / 32;
        uint32_t off = 0;
        const uint32_t ev_bytes = cap * 2 * 4, tree_bytes = tree_entries(T) * 4;
        ev = off;         off += ev_bytes > tree_bytes ? ev_bytes : tree_bytes;   // events, later the max tree
        kid = off;        off += (cap * 4 + 15) & ~15u;                          // child pairs, later {lo,hi}
        clone_bits = off; off += (((cap + 31) / 32) * 4 + 15) & ~15u;
        vbits = off;      off += (wps * 4 + 15) & ~15u;
        round_rank = off; off += COOP_MAX_THREADS * 4;                                // ranks of the steps of one pass-2 round
        wide = off;       off += (wps * 4 + 15) & ~15u;                           // steps whose rank range is wide
        ctrl = off;       off += 16;                                              // [0] = end of the last round with a wide range
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

// the same over the entries that are <= t (level 0 holds every stamp from the start)
__device__ __forceinline__ uint32_t group_max_le(const uint32_t* g, uint32_t first, uint32_t l, uint32_t r, uint32_t t) {
    const uint4* q = reinterpret_cast<const uint4*>(g);
    const uint4 a = q[0], b = q[1], c = q[2], d = q[3];
    const uint32_t val[16] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w, c.x, c.y, c.z, c.w, d.x, d.y, d.z, d.w};
    uint32_t m = 0;
#pragma unroll
    for (uint32_t e = 0; e < 16; ++e)
        if (first + e - l < r - l && val[e] <= t) m = max(m, val[e]);
    return m;
}

// List-ranking splitters: exactly one event index in every block of eight, at
// a hashed position inside the block so that no shape of the tree lines up with
// them; event 0 (the head of the list) always is one.
__device__ __forceinline__ uint32_t splitter_of_block(uint32_t k) {
    return k == 0u ? 0u : (k << 3) + ((k * 0x9E3779B1u) >> 29);
}
// `blocks` = number of whole blocks of the list; a trailing partial block has no splitter
__device__ __forceinline__ bool is_splitter(uint32_t e, uint32_t blocks) {
    return e == 0u || ((e >> 3) < blocks && splitter_of_block(e >> 3) == e);
}
constexpr uint32_t LAST_OF_SUBLIST = 0x80000000u;   // flag in an event word: the successor is a splitter or the end

// One CTA of NT threads; `B` is the stream's global scratch block
// after euler_pass1.  Every thread of the CTA must call this.
// CLIMB: pass 1 left the walk's (w_t, h_t) instead of v_t (sam_core.cuh): the climb to v_t happens here, every step
// by itself, while the query states are copied into shared memory.  ORIG (the split form): (w_t, h_t) lie in vq /
// head and the clones are the states with an `orig` entry.  CLIMB without ORIG (the interleaved form with the
// deferred climb): (w_t, h_t) lie packed in `rec` and the clones are the states whose id is no jid[t].
template <int NT, bool CLIMB = false, bool ORIG = false>
__device__ __forceinline__ void coop_tour_pass2(uint8_t* smem, const EulerBlock<uint16_t>& B, const uint32_t* vw,
                                                uint32_t* out, uint32_t T) {
    constexpr uint32_t NIL = 0xFFFFu, END = 0xFFFFu;
    const int tid = threadIdx.x, lane = tid & 31;
    const CoopLayout L(T);
    uint32_t* ev = reinterpret_cast<uint32_t*>(smem + L.ev);
    uint32_t* kid = reinterpret_cast<uint32_t*>(smem + L.kid);
    uint32_t* cbits = reinterpret_cast<uint32_t*>(smem + L.clone_bits);
    uint32_t* vbits = reinterpret_cast<uint32_t*>(smem + L.vbits);
    uint32_t* round_rank = reinterpret_cast<uint32_t*>(smem + L.round_rank);
    // the deferred-climb form of pass 1: clone flags per step and their prefix counts (2 * wps <= 1024 words)
    uint32_t* step_words = round_rank;
    uint32_t* step_prefix = round_rank + ((T + 31) / 32);
    auto step_state = [&](uint32_t i) {
        return 1u + i + step_prefix[i >> 5] + (uint32_t)__popc(step_words[i >> 5] & ((1u << (i & 31u)) - 1u));
    };
    const uint32_t n = B.meta[0], wps = (T + 31) / 32;
    const uint32_t cap = node_capacity(T);
    const uint32_t blocks = (2 * n) >> 3;       // whole blocks of eight events: one list-ranking splitter each
    const uint32_t ns = blocks ? blocks : 1u;   // event 0 is a splitter in any case
    ULLIS_COOP_MARK_BEGIN();

    // ---- stage: suffix links, clone bitmap, v bits.  The smallest / largest
    // child id of every state are collected with one atomicMin / atomicMax
    // each (a binary alphabet gives a state at most two link children); the
    // second array borrows the upper half of the event area for a moment.
    uint32_t* kid_min = kid;
    uint32_t* kid_max = ev + cap;
    for (uint32_t v = tid; v < n; v += NT) {
        kid_min[v] = 0xFFFFFFFFu;
        kid_max[v] = 0u;
    }
    if (ORIG) {   // a clone is a state with an `orig` entry (the split extend keeps no bitmap)
        for (uint32_t v = tid; v < ((n + 31u) & ~31u); v += NT) {
            const uint32_t word = __ballot_sync(0xffffffffu, v < n && B.next[v] != NIL);
            if (lane == 0) cbits[v >> 5] = word;
        }
    } else if (CLIMB) {
        // Pass 1 kept one bit per step ("this step made a clone").  Ids are handed out in order, so the state of
        // step i is 1 + i + (clones before step i): a prefix count over the flag words (kept, with the words, in
        // the buffer the pass-2 rounds use much later); the clones are the states no step created.
        for (uint32_t w = tid; w < wps; w += NT) step_words[w] = B.clone_bits[w];
        for (uint32_t w = tid; w < (n + 31) / 32; w += NT) cbits[w] = 0u;
        __syncthreads();
        if (tid < 32) {
            uint32_t carry = 0;
            for (uint32_t base = 0; base < wps; base += 32) {
                const uint32_t c = base + lane < wps ? __popc(step_words[base + lane]) : 0u;
                uint32_t incl = c;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const uint32_t up = __shfl_up_sync(0xffffffffu, incl, o);
                    if (lane >= o) incl += up;
                }
                if (base + lane < wps) step_prefix[base + lane] = carry + incl - c;
                carry += __shfl_sync(0xffffffffu, incl, 31);
            }
        }
        __syncthreads();
        for (uint32_t i = tid; i < T; i += NT) {
            const uint32_t j = step_state(i);
            atomicOr(&cbits[j >> 5], 1u << (j & 31));
        }
        __syncthreads();
        for (uint32_t w = tid; w < (n + 31) / 32; w += NT) cbits[w] = ~cbits[w];
    } else {
        for (uint32_t w = tid; w < (n + 31) / 32; w += NT) cbits[w] = B.clone_bits[w];
    }
    for (uint32_t w = tid; w < wps; w += NT) vbits[w] = vw[w];
    // the query states and new-state ids are needed much later: ask for them now, 128 bytes per thread
    for (uint32_t i = tid * 64u; i < T; i += NT * 64u) {
        if (CLIMB && !ORIG) asm volatile("prefetch.global.L2 [%0];" ::"l"(B.rec + i));
        else asm volatile("prefetch.global.L2 [%0];" ::"l"(B.vq + i));
        if (!(CLIMB && !ORIG)) asm volatile("prefetch.global.L2 [%0];" ::"l"(B.jid + i));
    }
    uint32_t* replay_end = reinterpret_cast<uint32_t*>(smem + L.ctrl);
    if (tid == 0) *replay_end = 0;
    __syncthreads();
    // global loads go out eight at a time, so that their latencies overlap
    const uint32_t* link_words = reinterpret_cast<const uint32_t*>(B.N) + 1;   // Node = {t0, t1 | fail, maxlen}
    for (uint32_t v0 = tid; v0 < n; v0 += NT * 8) {
        uint32_t p[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const uint32_t v = v0 + NT * u;
            p[u] = v < n ? link_words[2 * v] & 0xFFFFu : NIL;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const uint32_t v = v0 + NT * u;
            if (v < n && v != 0) {
                atomicMin(&kid_min[p[u]], v);
                atomicMax(&kid_max[p[u]], v);
            }
        }
    }
    __syncthreads();
    ULLIS_COOP_MARK(0);
    for (uint32_t v = tid; v < n; v += NT) {
        const uint32_t a = kid_min[v], b = kid_max[v];
        kid[v] = a == 0xFFFFFFFFu ? 0xFFFFFFFFu : (a | ((a == b ? NIL : b) << 16));
    }
    __syncthreads();

    ULLIS_COOP_MARK(1);
    // ---- Euler tour as a list: event 2v = enter v, 2v+1 = leave v; word = successor | weight << 16
    // (the suffix links come from global memory again, eight loads at a time: keeping
    // them in shared memory would cost the fourth resident CTA per SM)
    for (uint32_t v0 = tid; v0 < n; v0 += NT * 8) {
        uint32_t par[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const uint32_t v = v0 + NT * u;
            par[u] = v < n ? link_words[2 * v] & 0xFFFFu : NIL;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const uint32_t v = v0 + NT * u;
            if (v >= n) continue;
            const uint32_t k = kid[v], a = k & 0xFFFFu;
            const uint32_t stamped = (v != 0 && !((cbits[v >> 5] >> (v & 31)) & 1u)) ? 1u : 0u;
            const uint32_t first = a != NIL ? 2 * a : 2 * v + 1;
            ev[2 * v] = first | (stamped << 16) | (is_splitter(first, blocks) ? LAST_OF_SUBLIST : 0u);
            uint32_t succ = END;
            if (v != 0) {
                const uint32_t p = par[u], kp = kid[p];
                succ = ((kp & 0xFFFFu) == v && (kp >> 16) != NIL) ? 2 * (kp >> 16) : 2 * p + 1;
            }
            ev[2 * v + 1] = succ | (succ == END || is_splitter(succ, blocks) ? LAST_OF_SUBLIST : 0u);
        }
    }
    __syncthreads();
    ULLIS_COOP_MARK(2);
    // List ranking in two levels.  One event in eight is a splitter.  Level 1: the
    // thread that owns a splitter walks its sublist up to the next splitter and
    // leaves in every element (weight of the sublist before it, its splitter);
    // the splitter gets (weight of the whole sublist, next splitter).  Level 2:
    // pointer jumping over the splitters only, in place - a word is read and
    // written as a whole, so a reader always sees a consistent (successor, sum
    // over [s, successor)) pair.  O(events) work instead of O(events log events).
    ULLIS_COOP_MARK(8);
    {
        // One hop per chain and iteration, two independent chains per thread (their
        // shared-memory latencies overlap).  A chain that reaches the end of a
        // sublist takes the splitter of its next block in the same iteration, so
        // the lanes of a warp stay busy however the sublist lengths fall.
        struct Chain {
            uint32_t k, head, cur, before;
            bool busy;
        } c[2];
        auto next_block = [&](Chain& ch) {
            ch.busy = ch.k < ns;
            ch.head = ch.cur = splitter_of_block(ch.k);
            ch.before = 0;
        };
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            c[u].k = tid + NT * u;
            c[u].head = c[u].cur = c[u].before = 0;
            next_block(c[u]);
        }
        for (uint32_t hops = 0; (c[0].busy || c[1].busy) && hops < 2 * n; ++hops) {   // no sublist is longer than the list
            uint32_t w[2];
#pragma unroll
            for (int u = 0; u < 2; ++u) w[u] = c[u].busy ? ev[c[u].cur] : 0u;
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                if (!c[u].busy) continue;
                if (c[u].cur != c[u].head) ev[c[u].cur] = (c[u].before << 16) | c[u].head;
                c[u].before += (w[u] >> 16) & 1u;
                if (w[u] & LAST_OF_SUBLIST) {
                    ev[c[u].head] = (c[u].before << 16) | (w[u] & 0xFFFFu);
                    c[u].k += NT * 2;
                    next_block(c[u]);
                } else {
                    c[u].cur = w[u] & 0xFFFFu;
                }
            }
        }
    }
    __syncthreads();
    ULLIS_COOP_MARK(3);
    uint32_t rounds = 1;
    while ((1u << rounds) < ns) ++rounds;
    for (uint32_t it = 0; it <= rounds; ++it) {
        int any = 0;
        // eight independent splitters per thread and step: their dependent loads overlap
        for (uint32_t k0 = tid; k0 < ns; k0 += NT * 8) {
            uint32_t sp[8], w[8], w2[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const uint32_t k = k0 + NT * u;
                sp[u] = k < ns ? splitter_of_block(k) : 0xFFFFFFFFu;
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) w[u] = sp[u] != 0xFFFFFFFFu ? ev[sp[u]] : END;
#pragma unroll
            for (int u = 0; u < 8; ++u) w2[u] = (w[u] & 0xFFFFu) != END ? ev[w[u] & 0xFFFFu] : 0u;
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                if ((w[u] & 0xFFFFu) != END) {
                    ev[sp[u]] = (w2[u] & 0xFFFFu) | ((w[u] & 0xFFFF0000u) + (w2[u] & 0xFFFF0000u));
                    any = 1;
                }
            }
        }
        if (!__syncthreads_or(any)) break;
    }
    ULLIS_COOP_MARK(4);
    // weight of [e, end of list): the splitter's, less what lies before e in its sublist
    auto weight_from = [&](uint32_t e) {
        const uint32_t w = ev[e];
        return is_splitter(e, blocks) ? (w >> 16) : (ev[w & 0xFFFFu] >> 16) - (w >> 16);
    };
    // rank range of state v: stamped states entered before enter(v) / before leave(v)
    const uint32_t total = ev[0] >> 16;
    uint32_t* lh = kid;  // the splitter list is dead; same element size as the child pairs
    for (uint32_t v = tid; v < n; v += NT) {
        const uint32_t lo = total - weight_from(2 * v), hi = total - weight_from(2 * v + 1);
        lh[v] = lo | (hi << 16);
    }
    __syncthreads();
    // The events are dead.  The front of their space becomes the max tree, the part
    // behind it takes the query states and the new states of every step.
    uint16_t* vq_s = reinterpret_cast<uint16_t*>(ev + ((tree_entries(T) + 3u) & ~3u));
    uint16_t* jid_s = vq_s + T;
    for (uint32_t i0 = tid; i0 < T; i0 += NT * 8) {
        uint16_t a[8], b[8], hq[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const uint32_t i = i0 + NT * u;
            if (CLIMB && !ORIG) {
                const uint32_t r = i < T ? B.rec[i] : NIL;
                a[u] = (uint16_t)(r & 0xFFFFu);
                hq[u] = (uint16_t)(r >> 16);
            } else {
                a[u] = i < T ? B.vq[i] : (uint16_t)NIL;
                if (CLIMB) hq[u] = (i < T && a[u] != NIL) ? B.head[i] : (uint16_t)0;
            }
            if (CLIMB && !ORIG) b[u] = i < T ? (uint16_t)step_state(i) : (uint16_t)0;
            else b[u] = i < T ? B.jid[i] : (uint16_t)0;
        }
        if (CLIMB) {
#pragma unroll
            for (int u = 0; u < 8; ++u) a[u] = (uint16_t)euler_climb_words(B.N, a[u], hq[u], b[u]);
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const uint32_t i = i0 + NT * u;
            if (i < T) { vq_s[i] = a[u]; jid_s[i] = b[u]; }
        }
    }

    // ---- pass 2.  Every stamped state is stamped exactly once, by the step that
    // creates it, so level 0 of the max tree is a fixed array: stamp[rank of j_i]
    // = i + 1.  The answer of step t is the largest stamp <= t with a rank in
    // [lo, hi) of v_t.
    //   narrow ranges (at most NARROW ranks; almost all of them on typical
    //     streams) are scanned directly in that array, all steps in parallel;
    //   wide ranges go through the upper tree levels (maxima of groups of 16),
    //     which do depend on time: they are replayed in rounds of NT
    //     steps, and only if the stream has a wide range at all.
    constexpr uint32_t NARROW = 16;
    uint32_t* tree = ev;  // events are dead
    uint32_t* wide = reinterpret_cast<uint32_t*>(smem + L.wide);   // bit t: step t has a wide range
    const uint32_t entries = tree_entries(T);
    const uint32_t size0 = (T + 15u) & ~15u;
    const int warp = tid >> 5;
    for (uint32_t k = tid; k < entries; k += NT) tree[k] = 0;
    __syncthreads();
    for (uint32_t i = tid; i < T; i += NT) tree[lh[jid_s[i]] & 0xFFFFu] = i + 1u;
    __syncthreads();
    ULLIS_COOP_MARK(5);
    for (uint32_t t0 = 0; t0 < T; t0 += NT) {
        const uint32_t t = t0 + tid;
        uint32_t m = 0;
        bool is_wide = false;
        if (t < T) {
            const uint32_t v = vq_s[t];
            if (v != NIL) {
                const uint32_t r = lh[v];
                const uint32_t lo = r & 0xFFFFu, hi = r >> 16;
                if (hi - lo <= NARROW) {
                    for (uint32_t k = lo; k < hi; ++k) {
                        const uint32_t stamp = tree[k];
                        if (stamp <= t) m = max(m, stamp);
                    }
                } else {
                    is_wide = true;
                }
            }
        }
        const uint32_t bit = m ? (vbits[m >> 5] >> (m & 31)) & 1u : 0u;
        const uint32_t word = __ballot_sync(0xffffffffu, bit != 0);
        const uint32_t wide_word = __ballot_sync(0xffffffffu, is_wide);
        if (lane == 0 && t0 + warp * 32 < T) {
            out[(t0 >> 5) + warp] = word;
            wide[(t0 >> 5) + warp] = wide_word;
            if (wide_word) atomicMax(replay_end, t0 + NT);
        }
    }
    __syncthreads();
    ULLIS_COOP_MARK(6);
    const uint32_t t_end = min(T, *replay_end);   // nothing after the last wide range needs the upper levels
    if (t_end == 0) return;

    // Replay for the wide ranges.  Whole groups of a range are answered by the
    // upper levels, which hold the stamps of earlier rounds; the partial groups
    // at both ends by level 0 with the `<= t` filter; stamps of earlier steps of
    // the same round by the round's published ranks, newest first.
    for (uint32_t t0 = 0; t0 < t_end; t0 += NT) {
        const uint32_t t = t0 + tid;
        const bool live = t < T;
        const uint32_t my_rank = live ? lh[jid_s[t]] & 0xFFFFu : 0xFFFFFFFFu;
        round_rank[tid] = my_rank;
        const bool is_wide = live && ((wide[t >> 5] >> (t & 31)) & 1u);
        uint32_t lo = 0, hi = 0, m = 0;
        if (is_wide) {
            const uint32_t r = lh[vq_s[t]];
            lo = r & 0xFFFFu;
            hi = r >> 16;
            const uint32_t lg = lo >> 4, rg = (hi - 1u) >> 4;    // hi - lo > 16: at least two groups
            m = max(group_max_le(tree + (lg << 4), lg << 4, lo, hi, t), group_max_le(tree + (rg << 4), rg << 4, lo, hi, t));
            uint32_t l = lg + 1u, rr = rg, base = size0, size = ((size0 >> 4) + 15u) & ~15u;
            while (l < rr) {                                       // the whole groups in between, one level up
                const uint32_t lg2 = l >> 4, rg2 = (rr - 1u) >> 4;
                m = max(m, group_max(tree + base + (lg2 << 4), lg2 << 4, l, rr));
                if (rg2 != lg2) m = max(m, group_max(tree + base + (rg2 << 4), rg2 << 4, l, rr));
                if (rg2 <= lg2 + 1u) break;
                l = lg2 + 1u; rr = rg2;
                base += size;
                size = ((size >> 4) + 15u) & ~15u;
            }
        }
        __syncthreads();   // ranks of the round published; every tree read of the round done
        if (is_wide) {
            const uint32_t width = hi - lo;
            for (int e = (tid - 1) & ~3; e >= 0 && tid != 0; e -= 4) {
                const uint4 r4 = *reinterpret_cast<const uint4*>(round_rank + e);
                uint32_t f = (r4.x - lo < width ? 1u : 0u) | (r4.y - lo < width ? 2u : 0u) |
                             (r4.z - lo < width ? 4u : 0u) | (r4.w - lo < width ? 8u : 0u);
                if (e + 4 > tid) f &= (1u << (tid - e)) - 1u;     // only steps before this one
                if (f) { m = t0 + e + (31 - __clz(f)) + 1; break; }  // newer than anything in the tree
            }
            if (m && ((vbits[m >> 5] >> (m & 31)) & 1u)) atomicOr(&out[t >> 5], 1u << (t & 31));
        }
        if (live && size0 > 16u) {
            uint32_t pos = my_rank >> 4, base = size0, size = ((size0 >> 4) + 15u) & ~15u;
            for (;;) {
                atomicMax(&tree[base + pos], t + 1);
                if (size <= 16u) break;
                base += size;
                size = ((size >> 4) + 15u) & ~15u;
                pos >>= 4;
            }
        }
        __syncthreads();   // the round's stamps are in the upper levels; round_rank may be overwritten
    }
    ULLIS_COOP_MARK(7);
}
#endif

}  // namespace sam
}  // namespace ullis
