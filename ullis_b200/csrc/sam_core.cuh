// 1-bit ROSA suffix-automaton match for ONE (sequence, channel) stream.
//
// Semantics: idx[t] for t = 0..T-1 equals T successive calls of the
// reference's RosaSam::push(q[t], k[t], v[t]) (src/rosa.rs:100-176), i.e.
// rosa_qkv_ref (src/rosa.rs:180-193).  Two implementations live here:
//
//  * run_eager  - statement-by-statement form of push(), including the loop
//    that stamps `last = i` along the whole suffix-link chain of the newest
//    state (src/rosa.rs:168-173).  That loop is O(chain length) per step and
//    O(T^2) per stream on constant / periodic bit streams.
//
//  * run_euler  - same results in O(T log T) regardless of the input:
//      pass 1  builds the automaton and tracks the query state exactly as
//              push() does, but never touches `last`; it records the state
//              v_t each query would read `last` from, and the state j_i that
//              step i creates.  (v_t does not depend on any `last` value:
//              every non-root state is stamped in the step that creates it,
//              so the reference's `last < 0` skip only ever removes the root.)
//      tour    `last[v]` at query time t is the largest i < t whose new state
//              j_i lies in the suffix-link subtree of v.  The link tree only
//              grows by new leaves and by clones subdividing an edge, so
//              ancestor relations between existing states never change and
//              the FINAL tree can be used for every t.  A preorder walk gives
//              each state the half-open rank range [lo, hi) of the stamped
//              (non-clone, non-root) states below it.
//      pass 2  replays time: a max segment tree over ranks holds i+1 for
//              every j_i with i < t; the query is a range max over [lo, hi)
//              of v_t, the answer indexes the v history.
//
// The code is plain C++ over caller-provided memory so that the same source
// runs inside the CUDA kernels and in a host-compiled test harness.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define SAM_HD __host__ __device__ __forceinline__
#else
#define SAM_HD inline
#endif

namespace ullis {
namespace sam {

template <typename Ix>
struct Nil;
template <>
struct Nil<uint16_t> {
    static constexpr uint32_t value = 0xFFFFu;
};
template <>
struct Nil<uint32_t> {
    static constexpr uint32_t value = 0xFFFFFFFFu;
};

// One automaton state; a visit is a single 4*sizeof(Ix)-byte access.
template <typename Ix>
struct alignas(4 * sizeof(Ix)) Node {
    Ix t0, t1, fail, maxlen;
};

SAM_HD uint32_t node_capacity(uint32_t T) { return 2u * T + 2u; }
SAM_HD uint32_t pow2_at_least(uint32_t n) {
    uint32_t p = 1;
    while (p < n) p <<= 1;
    return p;
}
SAM_HD size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// Entries of the 16-ary max tree over T ranks: level sizes T', T'/16, ... down
// to one group (T' = T rounded up to a multiple of 16 per level).
SAM_HD uint32_t tree_entries(uint32_t T) {
    uint32_t total = 0, n = T;
    for (;;) {
        n = (n + 15u) & ~15u;
        total += n;
        if (n <= 16u) break;
        n >>= 4;
    }
    return total;
}

// Byte layout of one stream's scratch block for run_euler.
template <typename Ix>
struct EulerLayout {
    size_t nodes, vq, jid, head, next, lh, clone_bits, meta, total;
    SAM_HD explicit EulerLayout(uint32_t T) {
        const size_t cap = node_capacity(T);
        size_t off = 0;
        nodes = off; off = align_up(off + cap * sizeof(Node<Ix>), 16);
        vq = off;    off = align_up(off + (size_t)T * sizeof(Ix), 16);
        jid = off;   off = align_up(off + (size_t)T * sizeof(Ix), 16);
        // head/next (children lists of the suffix-link tree) are dead once the
        // tour is done; the max tree of pass 2 (about 1.07 T entries <= 2*cap)
        // reuses their space.
        head = off;  off = align_up(off + cap * sizeof(Ix), 16);
        next = off;  off = align_up(off + cap * sizeof(Ix), 16);
        lh = off;    off = align_up(off + cap * 2 * sizeof(Ix), 16);   // {lo, hi} rank range per state
        clone_bits = off; off = align_up(off + ((cap + 31) / 32) * 4, 16);
        meta = off;  off += 16;   // [0] = number of states after pass 1
        total = align_up(off, 128);
    }
};

// Byte layout of one stream's scratch block for run_eager.
template <typename Ix>
struct EagerLayout {
    size_t nodes, last, total;
    SAM_HD explicit EagerLayout(uint32_t T) {
        const size_t cap = node_capacity(T);
        size_t off = 0;
        nodes = off; off = align_up(off + cap * sizeof(Node<Ix>), 16);
        last = off;  off = align_up(off + cap * sizeof(Ix), 16);
        total = align_up(off, 128);
    }
};

SAM_HD uint32_t stream_bit(const uint32_t* words, uint32_t t) { return (words[t >> 5] >> (t & 31)) & 1u; }

// Work counters (optional instrumentation; pass nullptr to skip).
struct Counters {
    unsigned long long node_visits;   // automaton state reads in pass 1 / eager
    unsigned long long chain_steps;   // eager: iterations of the last-stamping loop
};

// ------------------------------------------------------------------ shared step
//
// Query + extend of one time step, without any `last` bookkeeping.
// Returns the state the reference would read `last` from (NIL if none), and
// reports the state created for this step through *j_out / the clone through
// *b_out (NIL when no clone was made).
template <typename Ix>
struct Walker {
    static constexpr uint32_t NIL = Nil<Ix>::value;
    Node<Ix>* N;
    uint32_t u, g, w;
    int32_t h;
    uint32_t gmax;  // maxlen of g
    uint32_t gfail; // suffix link of g, valid while g_fresh
    bool g_fresh;   // g was created by the previous extend: no children yet, every field known

    SAM_HD void init(Node<Ix>* nodes) {
        N = nodes;
        Node<Ix> root;
        root.t0 = (Ix)NIL; root.t1 = (Ix)NIL; root.fail = (Ix)NIL; root.maxlen = 0;
        N[0] = root;
        u = 1; g = 0; w = 0; h = 0; gmax = 0; gfail = NIL; g_fresh = true;   // the root has no children yet either
    }

    // src/rosa.rs:104-128 (query half of push)
    SAM_HD uint32_t query(uint32_t qb, unsigned long long* visits) {
        uint32_t p = w;
        int32_t x = h;
        uint32_t c = NIL;
        while (p != NIL) {
            Node<Ix> n = N[p];
            if (visits) ++*visits;
            c = qb ? n.t1 : n.t0;
            if (c != NIL) break;
            if (x > (int32_t)n.maxlen) x = (int32_t)n.maxlen;
            p = n.fail;
        }
        uint32_t v;
        if (p == NIL) {
            p = 0; x = 0; v = NIL;
        } else {
            p = c; x += 1;
            v = p;
            Node<Ix> nv = N[v];
            if (visits) ++*visits;
            while (nv.fail != NIL) {
                Node<Ix> nf = N[nv.fail];
                if (visits) ++*visits;
                if ((int32_t)nf.maxlen >= x) { v = nv.fail; nv = nf; } else break;
            }
            if (nv.maxlen == 0) v = NIL;  // only the root has maxlen 0; its fail is NIL
        }
        w = p; h = x;
        return v;
    }

    // src/rosa.rs:139-167 (extend half of push). The new state's `last`
    // handling is left to the caller.
    SAM_HD void extend(uint32_t kb, uint32_t* j_out, uint32_t* b_out, uint32_t* d_out,
                       unsigned long long* visits) {
        const uint32_t j = u++;
        Node<Ix> nj;
        nj.t0 = (Ix)NIL; nj.t1 = (Ix)NIL; nj.fail = 0; nj.maxlen = (Ix)(gmax + 1);
        uint32_t p = g, d = NIL, b = NIL;
        Node<Ix> n;
        n.t0 = n.t1 = n.fail = (Ix)NIL; n.maxlen = 0;
        if (g_fresh) {
            // the first state of the walk has no children: its visit is known without a load
            if (kb) N[p].t1 = (Ix)j; else N[p].t0 = (Ix)j;
            p = gfail;
        }
        while (p != NIL) {
            n = N[p];
            if (visits) ++*visits;
            d = kb ? n.t1 : n.t0;
            if (d != NIL) break;
            if (kb) N[p].t1 = (Ix)j; else N[p].t0 = (Ix)j;
            p = n.fail;
        }
        if (p == NIL) {
            nj.fail = 0;
            d = NIL;
        } else {
            Node<Ix> nd = N[d];
            if (visits) ++*visits;
            if ((uint32_t)n.maxlen + 1u == (uint32_t)nd.maxlen) {
                nj.fail = (Ix)d;
                d = NIL;  // no clone
            } else {
                b = u++;
                Node<Ix> nb = nd;            // the clone copies every field of d
                nb.maxlen = (Ix)(n.maxlen + 1u);
                N[b] = nb;
                N[d].fail = (Ix)b;
                nj.fail = (Ix)b;
                while (p != NIL) {
                    Node<Ix> n2 = N[p];
                    if (visits) ++*visits;
                    if ((kb ? n2.t1 : n2.t0) != d) break;
                    if (kb) N[p].t1 = (Ix)b; else N[p].t0 = (Ix)b;
                    p = n2.fail;
                }
            }
        }
        N[j] = nj;
        g = j;
        gmax = gmax + 1;
        gfail = nj.fail;
        g_fresh = true;
        *j_out = j; *b_out = b; *d_out = d;
    }
};

// ------------------------------------------------------------------ eager

// One RosaSam::push (src/rosa.rs:100-176) on a stream whose automaton lives in
// `wk` / `last` (last stores last+1, 0 = never): step number i, bits q and k;
// `vhist` is the stream's v history as bit words and must already hold bit i
// (the reference appends v_t before it queries, src/rosa.rs:102).  Returns idx.
template <typename Ix>
SAM_HD uint32_t eager_step(Walker<Ix>& wk, Ix* last, const uint32_t* vhist, uint32_t i, uint32_t qb, uint32_t kb,
                           Counters* cnt) {
    constexpr uint32_t NIL = Nil<Ix>::value;
    unsigned long long* visits = cnt ? &cnt->node_visits : nullptr;
    const uint32_t v = wk.query(qb, visits);
    uint32_t bit = 0;
    if (v != NIL) {
        const uint32_t pos = last[v];  // == last + 1 >= 1 for any non-root state
        bit = stream_bit(vhist, pos);
    }
    uint32_t j, b, d;
    wk.extend(kb, &j, &b, &d, visits);
    if (b != NIL) last[b] = last[d];
    last[j] = 0;
    // src/rosa.rs:168-173: stamp the whole suffix-link chain of j
    uint32_t c = j;
    while (c != NIL && (uint32_t)last[c] < i + 1u) {
        last[c] = (Ix)(i + 1u);
        c = wk.N[c].fail;
        if (cnt) ++cnt->chain_steps;
    }
    return bit;
}

// What a Walker carries from one step to the next, for automata that outlive a
// kernel (incremental generation): 32 bytes per stream.
struct WalkerState {
    uint32_t u, g, w, gmax, gfail;
    int32_t h;
    uint32_t steps;   // pushes so far
    uint32_t pad;
};
template <typename Ix>
SAM_HD void save_walker(const Walker<Ix>& wk, uint32_t steps, WalkerState* st) {
    st->u = wk.u; st->g = wk.g; st->w = wk.w; st->gmax = wk.gmax; st->gfail = wk.gfail; st->h = wk.h;
    st->steps = steps; st->pad = 0;
}
template <typename Ix>
SAM_HD uint32_t load_walker(Walker<Ix>& wk, Node<Ix>* nodes, const WalkerState* st) {
    wk.N = nodes;
    wk.u = st->u; wk.g = st->g; wk.w = st->w; wk.gmax = st->gmax; wk.gfail = st->gfail; wk.h = st->h;
    wk.g_fresh = true;   // g is the root or the state of the last step: no children either way
    return st->steps;
}

// ------------------------------------------------------------------ incremental pushes, chain kept as an array
//
// src/rosa.rs:168-173 stamps `last = i` on every state of the suffix-link chain of the step's new state j_i; the
// loop never stops early (every older stamp is < i), so it costs the length of the chain, which is the length of
// the key's current run on a biased stream.  Following the links is a chain of dependent loads.  The chain need
// not be followed: its states are the states of all suffixes of the keys so far, and a suffix of keys[0..i] is
// a suffix of keys[0..i-1] followed by k_i.  So
//
//     chain(j_i) = dedupe( child(c, k_i) for c in chain(j_{i-1}) ) ++ [root]
//
// with the children read after step i's extend (which gave every state of the old chain a child on k_i: j_i
// itself below the state the extend's walk stopped at, the old child or its clone from there on; equal children
// are neighbours because a state's strings are contiguous in length).  With chain(j_{i-1}) kept as an array the
// new chain is a map over independent loads, a compaction, and the stamps: one warp per stream does 32 entries
// per round, in place (the compacted position of an entry is never ahead of the entry).  The `last` array holds
// exactly what the reference's holds after every step.
//
// A stream whose key bits have all been equal so far needs no automaton yet.  After t pushes with key c it is a
// chain: states 0..t, state m = c^m, child(m, c) = m+1, link(m) = m-1, maxlen(m) = m, every `last` = t, and the
// query state is (w, w) with w = length of the current run of q == c (not counting step 0, whose query finds an
// empty automaton).  So a push costs O(1), idx = (t >= 1 and q == c) ? v : 0 (the same closed form as
// run_constant_k), and the automaton is written out only when a key bit differs for the first time.
//
// Lanes: inside a CUDA kernel all 32 lanes of a warp call gen_push together with equal arguments; on the host
// one caller stands for a warp of one lane.
namespace lanes {
#if defined(__CUDA_ARCH__)
SAM_HD uint32_t count() { return 32u; }
SAM_HD uint32_t id() { return threadIdx.x & 31u; }
SAM_HD uint32_t ballot(bool p) { return __ballot_sync(0xFFFFFFFFu, p); }
SAM_HD uint32_t from_below(uint32_t v) { return __shfl_up_sync(0xFFFFFFFFu, v, 1); }
SAM_HD uint32_t from_last(uint32_t v) { return __shfl_sync(0xFFFFFFFFu, v, 31); }
SAM_HD void sync() { __syncwarp(); }
#else
SAM_HD uint32_t count() { return 1u; }
SAM_HD uint32_t id() { return 0u; }
SAM_HD uint32_t ballot(bool p) { return p ? 1u : 0u; }
SAM_HD uint32_t from_below(uint32_t v) { return v; }
SAM_HD uint32_t from_last(uint32_t v) { return v; }
SAM_HD void sync() {}
#endif
SAM_HD uint32_t popc(uint32_t m) {
#if defined(__CUDA_ARCH__)
    return (uint32_t)__popc(m);
#else
    uint32_t n = 0;
    for (; m; m &= m - 1u) ++n;
    return n;
#endif
}
}  // namespace lanes

// Byte layout of one stream's block for incremental pushes: the eager layout plus the chain array.
template <typename Ix>
struct GenLayout {
    size_t nodes, last, path, total;
    SAM_HD explicit GenLayout(uint32_t T) {
        const size_t cap = node_capacity(T);
        size_t off = 0;
        nodes = off; off = align_up(off + cap * sizeof(Node<Ix>), 16);
        last = off;  off = align_up(off + cap * sizeof(Ix), 16);
        path = off;  off = align_up(off + ((size_t)T + 2) * sizeof(Ix), 16);   // chain(j_i) has at most i + 2 states
        total = align_up(off, 128);
    }
};

// chain(j_{i-1}) in path[0..len) -> chain(j_i), every state of it stamped; returns the new length.
template <typename Ix>
SAM_HD uint32_t chain_advance(const Node<Ix>* N, Ix* last, Ix* path, uint32_t len, uint32_t kb, uint32_t stamp) {
    constexpr uint32_t NIL = Nil<Ix>::value;
    const uint32_t W = lanes::count(), lane = lanes::id();
    uint32_t cnt = 0, carry = NIL;
    uint32_t t = NIL;
    if (lane < len) {
        const Node<Ix> n = N[path[lane]];
        t = kb ? n.t1 : n.t0;
    }
    for (uint32_t base = 0; base < len; base += W) {
        // the next round's loads are issued before this round's stores (which land at or below base + lane)
        uint32_t t_next = NIL;
        if (base + W + lane < len) {
            const Node<Ix> n = N[path[base + W + lane]];
            t_next = kb ? n.t1 : n.t0;
        }
        uint32_t below = lanes::from_below(t);
        if (lane == 0) below = carry;
        const bool keep = base + lane < len && t != below;
        const uint32_t mask = lanes::ballot(keep);
        if (keep) {
            path[cnt + lanes::popc(mask & ((1u << lane) - 1u))] = (Ix)t;
            last[t] = (Ix)stamp;
        }
        cnt += lanes::popc(mask);
        carry = lanes::from_last(t);   // only read while a further round follows: then lane W-1 held an entry
        t = t_next;
    }
    if (lane == 0) {
        path[cnt] = 0;        // the root ends every chain and is stamped too (src/rosa.rs:168-173 walks up to it)
        last[0] = (Ix)stamp;
    }
    return cnt + 1u;
}

// One RosaSam::push (src/rosa.rs:100-176) of an automaton that outlives the call.  `st` is the caller's copy of the
// stream's WalkerState (every lane holds one; lane 0's is the one to store back).  WalkerState::pad: bit 0 = the
// automaton has been written (see lazy_push: while every key bit so far was equal a push is O(1) and nothing is
// written), bits 1.. = length of the chain array.  `vhist` must already hold bit `steps`.  Returns idx on lane 0.
template <typename Ix>
SAM_HD uint32_t gen_push(Node<Ix>* nodes, Ix* last, Ix* path, const uint32_t* vhist, WalkerState* st, uint32_t qb,
                         uint32_t kb) {
    constexpr uint32_t NIL = Nil<Ix>::value;
    const uint32_t W = lanes::count(), lane = lanes::id();
    const uint32_t t = st->steps;
    uint32_t len = st->pad >> 1;
    if ((st->pad & 1u) == 0) {
        const uint32_t c = t == 0 ? kb : st->g;
        if (kb == c) {
            const uint32_t run = (t >= 1 && qb == c) ? st->w + 1u : 0u;
            st->w = run;
            st->g = c;
            st->steps = t + 1u;
            return run ? stream_bit(vhist, t) : 0u;   // last[v] + 1 = t for every state: the current v bit
        }
        // first differing key bit: write the automaton of t pushes of c (a chain of t + 1 states) and its chain array
        for (uint32_t m = lane; m <= t; m += W) {
            Node<Ix> n;
            n.t0 = (Ix)((m < t && c == 0) ? m + 1u : NIL);
            n.t1 = (Ix)((m < t && c == 1) ? m + 1u : NIL);
            n.fail = (Ix)(m ? m - 1u : NIL);
            n.maxlen = (Ix)m;
            nodes[m] = n;
            last[m] = (Ix)t;   // stored as last + 1 (0 = never); the root too
            path[m] = (Ix)(t - m);
        }
        len = t + 1u;
        const uint32_t run = st->w;
        st->u = t + 1u; st->g = t; st->gmax = t; st->gfail = t ? t - 1u : NIL;
        st->w = run; st->h = (int32_t)run;
        lanes::sync();
    }
    Walker<Ix> wk;
    const uint32_t i = load_walker(wk, nodes, st);
    uint32_t bit = 0;
    if (lane == 0) {
        const uint32_t v = wk.query(qb, nullptr);
        if (v != NIL) bit = stream_bit(vhist, last[v]);   // stored last + 1 >= 1 for any non-root state
        uint32_t j, b, d;
        wk.extend(kb, &j, &b, &d, nullptr);
        // the reference's last[b] = last[d] and last[j] = -1 are both overwritten by the stamps of this very step
    }
    lanes::sync();
    len = chain_advance<Ix>(nodes, last, path, len, kb, i + 1u);
    lanes::sync();
    save_walker(wk, i + 1u, st);
    st->pad = 1u | (len << 1);
    return bit;
}

// scratch: EagerLayout<Ix>(T).total bytes.  qw/kw/vw: this stream's bits, bit t
// at word t/32, bit t%32.  out: idx bits in the same layout (whole words are
// written, tail bits zero).
template <typename Ix>
SAM_HD void run_eager(uint8_t* scratch, const uint32_t* qw, const uint32_t* kw, const uint32_t* vw,
                      uint32_t* out, uint32_t T, Counters* cnt) {
    EagerLayout<Ix> L(T);
    Node<Ix>* N = reinterpret_cast<Node<Ix>*>(scratch + L.nodes);
    Ix* last = reinterpret_cast<Ix*>(scratch + L.last);  // stores last+1, 0 = never
    Walker<Ix> wk;
    wk.init(N);
    last[0] = 0;
    uint32_t acc = 0;
    for (uint32_t i = 0; i < T; ++i) {
        const uint32_t bit = eager_step<Ix>(wk, last, vw, i, stream_bit(qw, i), stream_bit(kw, i), cnt);
        acc |= bit << (i & 31);
        if ((i & 31) == 31 || i + 1 == T) { out[i >> 5] = acc; acc = 0; }
    }
}

// ------------------------------------------------------------------ euler

template <typename Ix>
struct Pair {
    Ix a, b;
};

template <typename Ix>
struct EulerBlock {
    Node<Ix>* N;
    Ix *vq, *jid, *head, *next;
    Pair<Ix>* lh;    // rank range [a, b) of the stamped states below each state
    uint32_t* rec;   // 16-bit ids only, same memory as lh: w_t | h_t << 16 of the pass 1 that leaves the climb for later
    uint32_t* clone_bits;
    uint32_t* meta;
    SAM_HD EulerBlock(uint8_t* scratch, uint32_t T) {
        EulerLayout<Ix> L(T);
        N = reinterpret_cast<Node<Ix>*>(scratch + L.nodes);
        vq = reinterpret_cast<Ix*>(scratch + L.vq);
        jid = reinterpret_cast<Ix*>(scratch + L.jid);
        head = reinterpret_cast<Ix*>(scratch + L.head);
        next = reinterpret_cast<Ix*>(scratch + L.next);
        lh = reinterpret_cast<Pair<Ix>*>(scratch + L.lh);
        rec = reinterpret_cast<uint32_t*>(scratch + L.lh);
        clone_bits = reinterpret_cast<uint32_t*>(scratch + L.clone_bits);
        meta = reinterpret_cast<uint32_t*>(scratch + L.meta);
    }
};

// pass 1: automaton + query states; returns the number of states created
template <typename Ix>
SAM_HD uint32_t euler_pass1(EulerBlock<Ix>& B, const uint32_t* qw, const uint32_t* kw, uint32_t T, Counters* cnt) {
    constexpr uint32_t NIL = Nil<Ix>::value;
    unsigned long long* visits = cnt ? &cnt->node_visits : nullptr;
    const uint32_t cap = node_capacity(T);
    for (uint32_t wd = 0; wd < (cap + 31) / 32; ++wd) B.clone_bits[wd] = 0;
    Walker<Ix> wk;
    wk.init(B.N);
    uint32_t qword = 0, kword = 0;
    for (uint32_t i = 0; i < T; ++i) {
        if ((i & 31) == 0) { qword = qw[i >> 5]; kword = kw[i >> 5]; }
        const uint32_t qb = (qword >> (i & 31)) & 1u, kb = (kword >> (i & 31)) & 1u;
        B.vq[i] = (Ix)wk.query(qb, visits);
        uint32_t j, b, d;
        wk.extend(kb, &j, &b, &d, visits);
        B.jid[i] = (Ix)j;
        if (b != NIL) B.clone_bits[b >> 5] |= 1u << (b & 31);
    }
    B.meta[0] = wk.u;
    return wk.u;
}

// euler_pass1 for 16-bit state ids with every state handled as two 32-bit words
// (x = t0 | t1 << 16, y = fail | maxlen << 16 - the bytes of Node<uint16_t>): one 8-byte load
// per visit, children picked with a shift by 16 * bit, child and link updates as 16-bit
// stores.  The state the extend starts from is always the one the previous step created
// (no children yet, link and length known), so it is never loaded.  Same results as
// euler_pass1<uint16_t>, fewer instructions per step.
struct NodeWords {
    uint32_t x, y;
};
SAM_HD NodeWords load_words(const Node<uint16_t>* N, uint32_t id) {
    const unsigned long long w = *reinterpret_cast<const unsigned long long*>(N + id);
    NodeWords n;
    n.x = (uint32_t)w;
    n.y = (uint32_t)(w >> 32);
    return n;
}
// The child of a state's first word on bit b, as one byte-permute: the selector is worked out once per step
// (CHILD_LO / CHILD_HI) and every visit of the step's walks picks with it.
constexpr uint32_t CHILD_LO = 0x4410u, CHILD_HI = 0x4432u;   // bytes {0, 1} or {2, 3} of the word, zero above
SAM_HD uint32_t child_selector(uint32_t bit) { return CHILD_LO + bit * (CHILD_HI - CHILD_LO); }
SAM_HD uint32_t pick_child(uint32_t x, uint32_t selector) {
#if defined(__CUDA_ARCH__)
    return __byte_perm(x, 0u, selector);
#else
    return selector == CHILD_HI ? x >> 16 : x & 0xFFFFu;
#endif
}
SAM_HD void store_words(Node<uint16_t>* N, uint32_t id, uint32_t x, uint32_t y) {
    *reinterpret_cast<unsigned long long*>(N + id) = (unsigned long long)x | ((unsigned long long)y << 32);
}

// DEFER_CLIMB: the walk up the links to the state whose `last` the step reads (src/rosa.rs:120-128) does not feed
// the next step, so it need not sit in this serial loop: the step then only records where the walk ended, as one
// word w_t | h_t << 16 in `rec` (NIL for a miss), and euler_climb_words finds v_t later, every step by itself, with
// the links read as of step t (a link that points to a state younger than jid[t] is followed on to the first older
// one).  This form keeps neither a clone bitmap over the states (a read-modify-write of global memory in seven
// steps out of ten on biased streams) nor the jid array: it leaves one bit per STEP, "this step made a clone", in
// the words of clone_bits (word t / 32, bit t % 32).  Ids are handed out in order, one per step plus one per
// clone, so jid[t] = 1 + t + (clones of the steps before t), and the clones are the states whose id is no jid[t];
// the tour works both out by itself.  Every store taken out of this loop shortens the serial chain.
// RELOAD_W (with DEFER_CLIMB only): the words of the state the next query starts from are not carried along and
// patched whenever the extend stores into that state ("mirrored"); they are loaded once per step, after the last
// store of the extend that can touch an existing state and before the step's remaining bookkeeping, which hides
// the load.  With the climb gone nothing else in the step needs those words, so the query's hit path has no load
// at all and four compare-and-patch sites leave the loop.
template <bool DEFER_CLIMB = false, bool RELOAD_W = false>
SAM_HD uint32_t euler_pass1_words(EulerBlock<uint16_t>& B, const uint32_t* qw, const uint32_t* kw, uint32_t T) {
    static_assert(DEFER_CLIMB || !RELOAD_W, "the climb inside the loop needs the words of the state it starts from");
    constexpr uint32_t NIL = 0xFFFFu;
    Node<uint16_t>* N = B.N;
    uint16_t* half = reinterpret_cast<uint16_t*>(N);   // field f of state s at half[4 * s + f]
    if (!DEFER_CLIMB) {
        const uint32_t cap = node_capacity(T);
        for (uint32_t wd = 0; wd < (cap + 31) / 32; ++wd) B.clone_bits[wd] = 0;
    }
    store_words(N, 0, 0xFFFFFFFFu, NIL);   // root: no children, no link, length 0
    uint32_t u = 1, g = 0, gmax = 0, gfail = NIL;   // extend side
    uint32_t w = 0, h = 0;                          // query side
    // The words of state w travel in registers from one step to the next: a hit loads them anyway (the query
    // ends in that state), and the few stores the extend makes to an existing state are applied to the copy.
    NodeWords nw;
    nw.x = 0xFFFFFFFFu; nw.y = NIL;
    // So do the words of state gfail, where the next extend starts: it is the state the extend read last (a
    // solid child), the clone it just wrote, or the root it just gave a child - never a load.
    NodeWords ne;
    ne.x = 0xFFFFFFFFu; ne.y = NIL;
    uint32_t qword = 0, kword = 0;
    uint32_t cloned = 0;   // DEFER_CLIMB: bit (i % 32) = step i made a clone; one word per 32 steps goes to clone_bits
    for (uint32_t i = 0; i < T; ++i) {
        if ((i & 31u) == 0) {
            qword = qw[i >> 5]; kword = kw[i >> 5];
            if (DEFER_CLIMB && i) { B.clone_bits[(i >> 5) - 1u] = cloned; cloned = 0; }
        }
        const uint32_t qsel = child_selector(qword & 1u), kb = kword & 1u, ks = kb << 4, ksel = child_selector(kb);
        qword >>= 1; kword >>= 1;
        const uint32_t e0 = gfail;
        // ---- query (src/rosa.rs:104-128)
        bool hit;
        {
            uint32_t p = w, x = h, c, v = NIL;
            NodeWords n = nw;
            for (;;) {
                c = pick_child(n.x, qsel);
                if (c != NIL) break;
                const uint32_t ml = n.y >> 16;
                if (x > ml) x = ml;
                p = n.y & 0xFFFFu;
                if (p == NIL) break;
                n = load_words(N, p);
            }
            hit = c != NIL;
            if (!hit) {
                w = 0; h = 0;
            } else {
                x += 1;
                v = c;
                NodeWords nv;
                nv.x = 0; nv.y = 0;
                if (!RELOAD_W) {
                    nv = load_words(N, v);
                    nw = nv;                      // the state the next query starts from
                }
                if (DEFER_CLIMB) {
                    v = c | (x << 16);            // the record of this step: the climb happens later
                } else {
                    for (;;) {
                        const uint32_t f = nv.y & 0xFFFFu;
                        if (f == NIL) break;
                        const NodeWords nf = load_words(N, f);
                        if ((nf.y >> 16) < x) break;
                        v = f; nv = nf;
                    }
                    if ((nv.y >> 16) == 0) v = NIL;   // only the root has length 0
                }
                w = c; h = x;
            }
            if (DEFER_CLIMB) B.rec[i] = v;   // NIL (0xFFFF) for a miss
            else B.vq[i] = (uint16_t)v;
        }
        // ---- extend (src/rosa.rs:139-167); every store to an existing state is mirrored into nw when it is state w
        {
            const uint32_t j = u++;
            const uint32_t child_mask = ~(0xFFFFu << ks);
            half[4 * g + kb] = (uint16_t)j;   // g has no children yet
            if (!RELOAD_W && g == w) nw.x = (nw.x & child_mask) | (j << ks);
            uint32_t p = e0, d = NIL, jfail = 0, pml = 0;
            NodeWords n = ne;                  // e0 == NIL (first step only): the root's words, for the case below
            while (p != NIL) {
                d = pick_child(n.x, ksel);
                pml = n.y >> 16;
                if (d != NIL) break;
                half[4 * p + kb] = (uint16_t)j;
                if (!RELOAD_W && p == w) nw.x = (nw.x & child_mask) | (j << ks);
                const uint32_t up = n.y & 0xFFFFu;
                if (up == NIL) break;           // p is the root and has its new child: keep its words in n
                p = up;
                n = load_words(N, p);
            }
            if (d != NIL) {
                const NodeWords nd = load_words(N, d);
                if (pml + 1u == (nd.y >> 16)) {
                    jfail = d;
                    ne = nd;
                } else {
                    const uint32_t b = u++;
                    ne.x = nd.x;                // the clone copies every field of d
                    ne.y = (nd.y & 0xFFFFu) | ((pml + 1u) << 16);
                    store_words(N, b, ne.x, ne.y);
                    half[4 * d + 2] = (uint16_t)b;
                    if (!RELOAD_W && d == w) nw.y = (nw.y & 0xFFFF0000u) | b;
                    jfail = b;
                    if (DEFER_CLIMB) cloned |= 1u << (i & 31u);
                    else B.clone_bits[b >> 5] |= 1u << (b & 31);
                    // p still has d as its child (that is where the walk stopped): redirect it, then go on up
                    for (;;) {
                        half[4 * p + kb] = (uint16_t)b;
                        if (!RELOAD_W && p == w) nw.x = (nw.x & child_mask) | (b << ks);
                        p = n.y & 0xFFFFu;
                        if (p == NIL) break;
                        n = load_words(N, p);
                        if (pick_child(n.x, ksel) != d) break;
                    }
                }
            } else {
                // the walk ran out at the root (or started there): the link of j is the root, whose words are n
                // with the child it was just given
                jfail = 0;
                ne.x = (n.x & child_mask) | (j << ks);
                ne.y = n.y;
            }
            // every store into an existing state has been issued: the state the next query starts from (the root
            // after a miss) is read now, and the rest of the step runs while the load is under way
            if (RELOAD_W) nw = load_words(N, w);
            gmax += 1;
            store_words(N, j, 0xFFFFFFFFu, jfail | (gmax << 16));
            g = j; gfail = jfail;
            if (!DEFER_CLIMB) B.jid[i] = (uint16_t)j;   // otherwise j_i = 1 + i + (clones of the steps before i)
        }
        if (!RELOAD_W && !hit) nw = load_words(N, 0);   // a miss sends the query back to the root
    }
    if (DEFER_CLIMB && T) B.clone_bits[(T - 1u) >> 5] = cloned;
    B.meta[0] = u;
    return u;
}

// ------------------------------------------------------------------ pass 1 in three parts
//
// euler_pass1_words interleaves two serial chains that do not need each other step by step: the extend
// never looks at the query, and the query only needs the automaton as it was after the extends of the
// EARLIER steps.  The state ids say when a state was made (ids are handed out in order; step t creates
// state jid[t], a clone right after it), so that older automaton can be read off the FINAL one:
//   * a state exists at query time t iff its id is below lim = jid[t];
//   * every store of the extend writes the id of a state made in that very step, so a child or link field
//     holds either what it held at time t or the id of a younger state.  A younger child id is taken back
//     through `orig` (a clone replaces the state it copies in the transitions it takes over, orig[clone] =
//     that state; a state that is no clone replaces "no child", orig = NIL) until it is older than lim;
//     a younger link is followed upwards until it is older than lim (the link tree only grows by leaves and
//     by clones that subdivide an edge, so the nearest older ancestor is the link of time t);
//   * lengths never change.
// So the pass is split into
//   extend (serial, one thread per stream): the whole automaton of the keys, jid, orig;
//   walk   (serial, one thread per stream): the query state (w_t, h_t) of src/rosa.rs:104-119 for every step
//          against that automaton read "as of time t" - one dependent load per step on a hit;
//   climb  (independent per step, so it runs in parallel with the tour): the state v_t of
//          src/rosa.rs:120-128 from (w_t, h_t), again with links as of time t.
// Each chain is a fraction of the interleaved one, and the climb leaves the serial part altogether.
// Scratch: h_t in the `head` array and orig in the `next` array of the block (both unused until the tour
// of the one-thread form, which the split form does not use: its tour runs in shared memory).  The caller
// fills orig with NIL beforehand; the extend only writes the entries of the clones, and those entries are
// also what tells the tour which states are clones (no stamp of their own).
SAM_HD void euler_extend_words(EulerBlock<uint16_t>& B, const uint32_t* kw, uint32_t T) {
    constexpr uint32_t NIL = 0xFFFFu;
    Node<uint16_t>* N = B.N;
    uint16_t* half = reinterpret_cast<uint16_t*>(N);   // field f of state s at half[4 * s + f]
    uint16_t* orig = B.next;               // the caller has filled it with NIL (0xFFFF): only clones get an entry
    store_words(N, 0, 0xFFFFFFFFu, NIL);   // root: no children, no link, length 0
    uint32_t u = 1, g = 0, gmax = 0, gfail = NIL;
    NodeWords ne;                           // the words of state gfail, where the next extend starts (never loaded)
    ne.x = 0xFFFFFFFFu; ne.y = NIL;
    uint32_t kword = 0;
    for (uint32_t i = 0; i < T; ++i) {
        if ((i & 31u) == 0) kword = kw[i >> 5];
        const uint32_t kb = kword & 1u, ks = kb << 4;
        kword >>= 1;
        const uint32_t j = u++;
        const uint32_t child_mask = ~(0xFFFFu << ks);
        half[4 * g + kb] = (uint16_t)j;   // g has no children yet
        uint32_t p = gfail, d = NIL, jfail = 0, pml = 0;
        NodeWords n = ne;                  // gfail == NIL (first step only): the root's words, for the case below
        while (p != NIL) {
            d = (n.x >> ks) & 0xFFFFu;
            pml = n.y >> 16;
            if (d != NIL) break;
            half[4 * p + kb] = (uint16_t)j;
            const uint32_t up = n.y & 0xFFFFu;
            if (up == NIL) break;           // p is the root and has its new child: keep its words in n
            p = up;
            n = load_words(N, p);
        }
        if (d != NIL) {
            const NodeWords nd = load_words(N, d);
            if (pml + 1u == (nd.y >> 16)) {
                jfail = d;
                ne = nd;
            } else {
                const uint32_t b = u++;
                ne.x = nd.x;                // the clone copies every field of d
                ne.y = (nd.y & 0xFFFFu) | ((pml + 1u) << 16);
                store_words(N, b, ne.x, ne.y);
                orig[b] = (uint16_t)d;      // also what marks b as a clone for the tour
                half[4 * d + 2] = (uint16_t)b;
                jfail = b;
                for (;;) {                  // p still has d as its child: redirect it, then go on up
                    half[4 * p + kb] = (uint16_t)b;
                    p = n.y & 0xFFFFu;
                    if (p == NIL) break;
                    n = load_words(N, p);
                    if (((n.x >> ks) & 0xFFFFu) != d) break;
                }
            }
        } else {
            jfail = 0;                      // the walk ran out at the root, whose words are n with its new child
            ne.x = (n.x & child_mask) | (j << ks);
            ne.y = n.y;
        }
        gmax += 1;
        store_words(N, j, 0xFFFFFFFFu, jfail | (gmax << 16));
        g = j; gfail = jfail;
        B.jid[i] = (uint16_t)j;
    }
    B.meta[0] = u;
}

// child `c` (a raw field of the final automaton) as it was when only states below `lim` existed
SAM_HD uint32_t child_as_of(const uint16_t* orig, uint32_t c, uint32_t lim) {
    while (c != 0xFFFFu && c >= lim) c = orig[c];
    return c;
}
// the same for a suffix link: the nearest ancestor below `lim`
SAM_HD uint32_t link_as_of(const Node<uint16_t>* N, uint32_t f, uint32_t lim) {
    while (f != 0xFFFFu && f >= lim) f = load_words(N, f).y & 0xFFFFu;
    return f;
}

// The query walk of steps [t0, t1) from the state (w, h) held before step t0; writes (w_t, h_t) of a hit to
// vq / head and NIL to vq for a miss, and returns the state after its last step through w / h.
// UNTIL_SAME: the records of these steps already hold a walk from a GUESSED start state; this walk, from the
// true one, stops at the first step whose state equals the recorded one - from there on the two walks are the
// same walk (the next state is a function of the state, the bit and the step alone) - and returns that step
// (t1 if the walks never met).  Without it the return value is t1.
template <bool UNTIL_SAME>
SAM_HD uint32_t euler_walk_words(EulerBlock<uint16_t>& B, const uint32_t* qw, uint32_t t0, uint32_t t1, uint32_t& w,
                                 uint32_t& h) {
    constexpr uint32_t NIL = 0xFFFFu;
    const Node<uint16_t>* N = B.N;
    const uint16_t* orig = B.next;
    uint16_t* hq = B.head;
    NodeWords nw = load_words(N, w);
    uint32_t qword = t0 < t1 ? qw[t0 >> 5] >> (t0 & 31u) : 0u;
    for (uint32_t i = t0; i < t1; ++i) {
        if ((i & 31u) == 0) qword = qw[i >> 5];
        const uint32_t qs = (qword & 1u) << 4;
        qword >>= 1;
        const uint32_t lim = B.jid[i];
        uint32_t x = h, c;
        NodeWords n = nw;
        for (;;) {
            c = child_as_of(orig, (n.x >> qs) & 0xFFFFu, lim);
            if (c != NIL) break;
            const uint32_t ml = n.y >> 16;
            if (x > ml) x = ml;
            const uint32_t p = link_as_of(N, n.y & 0xFFFFu, lim);
            if (p == NIL) break;
            n = load_words(N, p);
        }
        if (c == NIL) {
            w = 0; h = 0;
            if (UNTIL_SAME && B.vq[i] == NIL) return i;
            B.vq[i] = (uint16_t)NIL;
            nw = load_words(N, 0);
        } else {
            w = c; h = x + 1u;
            if (UNTIL_SAME && B.vq[i] == c && hq[i] == h) return i;
            B.vq[i] = (uint16_t)c;
            hq[i] = (uint16_t)h;
            nw = load_words(N, c);
        }
    }
    return t1;
}

// The whole walk in `chunks` pieces, the way a group of lanes runs it: every piece first walks from the guessed
// state "no match" (the true one for piece 0), all pieces at once; then piece after piece is redone from the true
// end state of the piece before it until it meets its guessed walk - after a few steps on streams whose matches
// are short, after the whole piece at worst.  `piece` = steps per piece (a multiple of 32 keeps whole bit words).
SAM_HD void euler_walk_chunked(EulerBlock<uint16_t>& B, const uint32_t* qw, uint32_t T, uint32_t piece) {
    const uint32_t chunks = (T + piece - 1) / piece;
    uint32_t w = 0, h = 0;              // true state at the end of the piece before the current one
    for (uint32_t c = 0; c < chunks; ++c) {   // on the device: all pieces at once, one lane each
        uint32_t gw = 0, gh = 0;
        const uint32_t t0 = c * piece, t1 = t0 + piece < T ? t0 + piece : T;
        euler_walk_words<false>(B, qw, t0, t1, gw, gh);
        if (c == 0) { w = gw; h = gh; }
    }
    for (uint32_t c = 1; c < chunks; ++c) {
        const uint32_t t0 = c * piece, t1 = t0 + piece < T ? t0 + piece : T;
        // the guessed walk's end state: its last record
        uint32_t ew = B.vq[t1 - 1] == 0xFFFFu ? 0u : B.vq[t1 - 1], eh = B.vq[t1 - 1] == 0xFFFFu ? 0u : B.head[t1 - 1];
        uint32_t tw = w, th = h;
        const uint32_t met = euler_walk_words<true>(B, qw, t0, t1, tw, th);
        if (met < t1) { w = ew; h = eh; } else { w = tw; h = th; }
    }
}

// The state step t reads `last` from (src/rosa.rs:120-128), from the walk's (w_t, h_t): up the links as of
// time t while the link's strings are still long enough; only the root has length 0 and is skipped.
SAM_HD uint32_t euler_climb_words(const Node<uint16_t>* N, uint32_t w, uint32_t h, uint32_t lim) {
    constexpr uint32_t NIL = 0xFFFFu;
    if (w == NIL) return NIL;
    uint32_t v = w;
    NodeWords nv = load_words(N, v);
    for (;;) {
        const uint32_t f = link_as_of(N, nv.y & 0xFFFFu, lim);
        if (f == NIL) break;
        const NodeWords nf = load_words(N, f);
        if ((nf.y >> 16) < h) break;
        v = f; nv = nf;
    }
    return (nv.y >> 16) == 0 ? NIL : v;
}

// Interleaved pass 1 without the climb, then the climb of every step (what rosa_pass1_kernel with the deferred
// climb and the tour kernel compute together).
SAM_HD uint32_t euler_pass1_deferred(EulerBlock<uint16_t>& B, const uint32_t* qw, const uint32_t* kw, uint32_t T) {
    const uint32_t n = euler_pass1_words<true, true>(B, qw, kw, T);
    for (uint32_t t = 0, clones = 0; t < T; ++t) {   // the new-state ids from the per-step clone flags
        B.jid[t] = (uint16_t)(1u + t + clones);
        clones += (B.clone_bits[t >> 5] >> (t & 31u)) & 1u;
    }
    for (uint32_t t = 0; t < T; ++t) {
        const uint32_t r = B.rec[t];
        B.vq[t] = (uint16_t)euler_climb_words(B.N, r & 0xFFFFu, r >> 16, B.jid[t]);
    }
    // clones = the states that no step created as its new state
    const uint32_t cap = node_capacity(T);
    for (uint32_t wd = 0; wd < (cap + 31) / 32; ++wd) B.clone_bits[wd] = 0xFFFFFFFFu;
    for (uint32_t t = 0; t < T; ++t) B.clone_bits[B.jid[t] >> 5] &= ~(1u << (B.jid[t] & 31));
    return n;
}

// The three parts one after the other (what the split kernels compute together): same vq / jid / states as
// euler_pass1_words.
// orig <- NIL for every state (before the extend), clone bitmap <- "has an orig" (after it): the pieces the
// kernels do with a fill of the scratch blocks and inside the tour kernel.
SAM_HD void split_fill_orig(EulerBlock<uint16_t>& B, uint32_t T) {
    for (uint32_t v = 0; v < node_capacity(T); ++v) B.next[v] = (uint16_t)0xFFFFu;
}
SAM_HD void split_clone_bits(EulerBlock<uint16_t>& B, uint32_t T) {
    const uint32_t cap = node_capacity(T);
    for (uint32_t wd = 0; wd < (cap + 31) / 32; ++wd) B.clone_bits[wd] = 0;
    for (uint32_t v = 0; v < B.meta[0]; ++v)
        if (B.next[v] != 0xFFFFu) B.clone_bits[v >> 5] |= 1u << (v & 31);
}

SAM_HD uint32_t euler_pass1_split(EulerBlock<uint16_t>& B, const uint32_t* qw, const uint32_t* kw, uint32_t T) {
    split_fill_orig(B, T);
    euler_extend_words(B, kw, T);
    split_clone_bits(B, T);
    uint32_t w = 0, h = 0;
    euler_walk_words<false>(B, qw, 0, T, w, h);
    for (uint32_t t = 0; t < T; ++t)
        B.vq[t] = (uint16_t)euler_climb_words(B.N, B.vq[t], B.head[t], B.jid[t]);
    return B.meta[0];
}

// The same with the walk in pieces of `piece` steps (euler_walk_chunked).
SAM_HD uint32_t euler_pass1_split_chunked(EulerBlock<uint16_t>& B, const uint32_t* qw, const uint32_t* kw, uint32_t T,
                                          uint32_t piece) {
    split_fill_orig(B, T);
    euler_extend_words(B, kw, T);
    split_clone_bits(B, T);
    euler_walk_chunked(B, qw, T, piece);
    for (uint32_t t = 0; t < T; ++t)
        B.vq[t] = (uint16_t)euler_climb_words(B.N, B.vq[t], B.head[t], B.jid[t]);
    return B.meta[0];
}

// tour: children lists, then a preorder walk; every state gets the half-open
// rank range of the stamped (non-clone, non-root) states in its subtree
template <typename Ix>
SAM_HD void euler_tour(EulerBlock<Ix>& B, uint32_t n) {
    constexpr uint32_t NIL = Nil<Ix>::value;
    for (uint32_t v = 0; v < n; ++v) B.head[v] = (Ix)NIL;
    for (uint32_t v = 1; v < n; ++v) {
        const uint32_t f = B.N[v].fail;
        B.next[v] = B.head[f];
        B.head[f] = (Ix)v;
    }
    uint32_t r = 0, v = 0;
    bool entering = true;
    for (;;) {
        if (entering) {
            B.lh[v].a = (Ix)r;
            if (v != 0 && !((B.clone_bits[v >> 5] >> (v & 31)) & 1u)) ++r;
            const uint32_t c = B.head[v];
            if (c != NIL) { v = c; continue; }
            entering = false;
        }
        B.lh[v].b = (Ix)r;
        if (v == 0) break;
        const uint32_t s = B.next[v];
        if (s != NIL) { v = s; entering = true; } else { v = B.N[v].fail; }
    }
}

// pass 2: replay time over a 16-ary max tree keyed by preorder rank. Level 0
// holds i+1 at the rank of j_i once i < t (0 = not yet); level k+1 holds the
// maximum of each group of 16 entries of level k. Stamps only grow with time,
// so an insert is one plain store per level.
template <typename Ix>
SAM_HD void euler_pass2(EulerBlock<Ix>& B, const uint32_t* vw, uint32_t* out, uint32_t T) {
    constexpr uint32_t NIL = Nil<Ix>::value;
    Ix* tree = B.head;  // head/next are dead now, contiguous and large enough
    const uint32_t entries = tree_entries(T);
    for (uint32_t k = 0; k < entries; ++k) tree[k] = 0;
    uint32_t acc = 0;
    for (uint32_t t = 0; t < T; ++t) {
        const uint32_t v = B.vq[t];
        uint32_t bit = 0;
        if (v != NIL) {
            const Pair<Ix> range = B.lh[v];
            uint32_t l = range.a, r = range.b, m = 0, base = 0, size = (T + 15u) & ~15u;
            while (l < r) {
                const uint32_t lg = l >> 4, rg = (r - 1u) >> 4;
                if (lg == rg) {
                    for (uint32_t e = l; e < r; ++e) { const uint32_t s = tree[base + e]; m = s > m ? s : m; }
                    break;
                }
                uint32_t l2 = lg, r2 = rg + 1u;
                if (l & 15u) {
                    for (uint32_t e = l; e < ((lg + 1u) << 4); ++e) { const uint32_t s = tree[base + e]; m = s > m ? s : m; }
                    l2 = lg + 1u;
                }
                if (r & 15u) {
                    for (uint32_t e = rg << 4; e < r; ++e) { const uint32_t s = tree[base + e]; m = s > m ? s : m; }
                    r2 = rg;
                }
                base += size;
                size = ((size >> 4) + 15u) & ~15u;
                l = l2; r = r2;
            }
            // m = last + 1 >= 1: every state that exists at time t has a stamped
            // descendant (itself, or the state whose creation cloned it).
            bit = m ? stream_bit(vw, m) : 0u;
        }
        acc |= bit << (t & 31);
        if ((t & 31) == 31 || t + 1 == T) { out[t >> 5] = acc; acc = 0; }
        uint32_t pos = B.lh[B.jid[t]].a, base = 0, size = (T + 15u) & ~15u;
        for (;;) {
            tree[base + pos] = (Ix)(t + 1u);
            if (size <= 16u) break;
            base += size;
            size = ((size >> 4) + 15u) & ~15u;
            pos >>= 4;
        }
    }
}

// ------------------------------------------------------------ constant k
//
// If every k bit of a stream equals c, the automaton is the chain
// root -> c -> cc -> ... with no clone, every chain state is stamped at every
// step, and the query state either advances along the chain (q_t == c) or
// falls off it to "no match" (q_t != c).  T pushes of the reference then give
//     idx_t = v_t  if t >= 1 and q_t == c,   else 0
// (at t = 0 the automaton is still empty).  Checked exhaustively against the
// step-by-step form in the host harness.
SAM_HD bool k_is_constant(const uint32_t* kw, uint32_t T, uint32_t* c_out) {
    if (T == 0) return false;
    const uint32_t c = kw[0] & 1u, full = c ? 0xFFFFFFFFu : 0u, wps = (T + 31) >> 5;
    const uint32_t tail = (T & 31u) ? ((1u << (T & 31u)) - 1u) : 0xFFFFFFFFu;
    for (uint32_t w = 0; w + 1 < wps; ++w)
        if (kw[w] != full) return false;
    if ((kw[wps - 1] & tail) != (full & tail)) return false;
    *c_out = c;
    return true;
}

SAM_HD void run_constant_k(const uint32_t* qw, const uint32_t* vw, uint32_t* out, uint32_t T, uint32_t c) {
    const uint32_t wps = (T + 31) >> 5;
    const uint32_t tail = (T & 31u) ? ((1u << (T & 31u)) - 1u) : 0xFFFFFFFFu;
    for (uint32_t w = 0; w < wps; ++w) {
        uint32_t word = (c ? qw[w] : ~qw[w]) & vw[w];
        if (w == 0) word &= ~1u;
        if (w + 1 == wps) word &= tail;
        out[w] = word;
    }
}

// ---- constant v.  idx_t is a bit of the v history, so a stream whose v bits
// are all 0 has idx = 0 everywhere.  A stream whose v bits are all 1 has
// idx_t = 1 exactly when the query of step t finds a state to read `last` from
// (that state was stamped when it was created, so its `last` is valid).  The
// query walks up the suffix links until a state has a q_t-child and fails only
// if even the root has none - the root has a c-child as soon as c has occurred
// among the keys - so idx_t = 1 iff q_t occurs in k_0 .. k_{t-1}: no automaton
// at all.  With f the first step whose key differs from k_0 (f = T if none):
// idx_t = (q_t == k_0) for 1 <= t <= f, idx_t = 1 for t > f, idx_0 = 0.
SAM_HD void run_constant_v_one(const uint32_t* qw, const uint32_t* kw, uint32_t* out, uint32_t T) {
    const uint32_t wps = (T + 31) >> 5;
    const uint32_t tail = (T & 31u) ? ((1u << (T & 31u)) - 1u) : 0xFFFFFFFFu;
    const uint32_t c0 = kw[0] & 1u, full = c0 ? 0xFFFFFFFFu : 0u;
    uint32_t f = T;
    for (uint32_t w = 0; w < wps && f == T; ++w) {
        uint32_t diff = kw[w] ^ full;
        if (w + 1 == wps) diff &= tail;
        if (diff) {
            uint32_t b = 0;
            while (!((diff >> b) & 1u)) ++b;
            f = w * 32u + b;
        }
    }
    for (uint32_t w = 0; w < wps; ++w) {
        const uint32_t same = c0 ? qw[w] : ~qw[w];   // q_t == k_0
        // bits of this word at steps > f
        uint32_t after;
        if (f >= w * 32u + 31u) after = 0u;
        else if (f < w * 32u) after = 0xFFFFFFFFu;
        else after = ~((2u << (f - w * 32u)) - 1u);
        uint32_t word = (same & ~after) | after;
        if (w == 0) word &= ~1u;
        if (w + 1 == wps) word &= tail;
        out[w] = word;
    }
}

// Constant q (every query bit equals c).  The query string is c^(t+1), so only
// the runs of c among the keys matter.  With M the longest run of c in
// k_0 .. k_{t-1}, the automaton holds c^m alone in its own state for m < M and
// c^M in a state Z whose shortest string is c^M; the walk reaches Z as soon as
// the run record and the match length (both grow by at most one per step) have
// met, and re-enters it through Z's suffix link whenever Z has no c-child.  The
// state the reference reads is therefore Z, and last[Z] is the end of the most
// recent run of length M:
//   idx_t = v[p + 1],  p = max{ e < t : (length of the run of c ending at e) >= M },
//   idx_t = 0 while no key equals c.
// One O(T) scan, no automaton.  Checked like the other closed forms: every key
// sequence up to T = 18 and long random / periodic ones against the eager form.
SAM_HD void run_constant_q(uint32_t c, const uint32_t* kw, const uint32_t* vw, uint32_t* out, uint32_t T) {
    uint32_t run = 0, best = 0, pv = 0;   // pv = v[p + 1] for the current record position p
    for (uint32_t base = 0; base < T; base += 32u) {
        const uint32_t w = base >> 5;
        const uint32_t n = T - base < 32u ? T - base : 32u;
        const uint32_t kword = kw[w];
        const uint32_t same = c ? kword : ~kword;   // bit i: k_{base+i} == c
        uint32_t acc = 0;
        if (n == 32u && same == 0xFFFFFFFFu && (run == best || best - run > 32u)) {
            // 32 steps inside one run of c, taken at once: either every step sets a record (the run is the
            // longest so far: step base + i answers with v[base + i], the first one with the old pv) or none does
            if (run == best) {
                acc = (vw[w] & ~1u) | (best ? pv : 0u);
                run += 32u;
                best = run;
                pv = base + 32u < T ? stream_bit(vw, base + 32u) : 0u;
            } else {
                acc = pv ? 0xFFFFFFFFu : 0u;
                run += 32u;
            }
        } else if (n == 32u && same == 0u) {   // 32 steps without c: no record, the run ends
            acc = (best && pv) ? 0xFFFFFFFFu : 0u;
            run = 0;
        } else {
            for (uint32_t i = 0; i < n; ++i) {
                const uint32_t t = base + i;
                if (best) acc |= pv << i;
                if ((same >> i) & 1u) {
                    if (++run >= best) {
                        best = run;
                        pv = t + 1 < T ? stream_bit(vw, t + 1) : 0u;
                    }
                } else {
                    run = 0;
                }
            }
        }
        out[w] = acc;
    }
}

template <typename Ix>
SAM_HD bool run_euler(uint8_t* scratch, const uint32_t* qw, const uint32_t* kw, const uint32_t* vw,
                      uint32_t* out, uint32_t T, Counters* cnt) {
    EulerBlock<Ix> B(scratch, T);
    const uint32_t n = euler_pass1<Ix>(B, qw, kw, T, cnt);
    if (n > node_capacity(T)) return false;  // cannot happen: an automaton over T symbols has at most 2T states
    euler_tour<Ix>(B, n);
    euler_pass2<Ix>(B, vw, out, T);
    return true;
}

}  // namespace sam
}  // namespace ullis
