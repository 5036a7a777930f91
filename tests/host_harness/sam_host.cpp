// Host-compiled harness around the device SAM routines (sam_core.cuh), used
// only by the CPU test-suite to check the kernel's index arithmetic against
// the oracle without a GPU.  It is not part of the shipped library.
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "../../ullis_b200/csrc/sam_core.cuh"

using namespace ullis::sam;

template <typename Ix>
static int run_batch(int algo, const uint32_t* qw, const uint32_t* kw, const uint32_t* vw, size_t n_streams,
                     uint32_t T, uint32_t* out, unsigned long long* visits, unsigned long long* chain) {
    const size_t wps = (T + 31) / 32;
    const size_t bytes = algo == 0 ? EagerLayout<Ix>(T).total : algo == 6 ? GenLayout<Ix>(T).total : EulerLayout<Ix>(T).total;
    std::vector<uint8_t> scratch(bytes + 64);
    uint8_t* base = scratch.data();
    base += (64 - reinterpret_cast<uintptr_t>(base) % 64) % 64;
    Counters cnt{0, 0};
    for (size_t s = 0; s < n_streams; ++s) {
        std::memset(base, 0xA5, bytes);  // the routines must not rely on zeroed scratch
        uint32_t c = 0;
        if (algo == 2 && k_is_constant(kw + s * wps, T, &c)) {
            run_constant_k(qw + s * wps, vw + s * wps, out + s * wps, T, c);
            continue;
        }
        if (algo == 2 && k_is_constant(vw + s * wps, T, &c)) {   // the same test on the v words: constant v
            if (c == 0) {
                for (size_t w = 0; w < wps; ++w) out[s * wps + w] = 0;
            } else {
                run_constant_v_one(qw + s * wps, kw + s * wps, out + s * wps, T);
            }
            continue;
        }
        if (algo == 2 && k_is_constant(qw + s * wps, T, &c)) {   // constant q
            run_constant_q(c, kw + s * wps, vw + s * wps, out + s * wps, T);
            continue;
        }
        if (algo == 4) {   // pass 1 on packed state words (16-bit state ids only)
            if (sizeof(Ix) != 2) return 3;
            EulerBlock<uint16_t> B(base, T);
            const uint32_t n = euler_pass1_words(B, qw + s * wps, kw + s * wps, T);
            if (n > node_capacity(T)) return 2;
            euler_tour<uint16_t>(B, n);
            euler_pass2<uint16_t>(B, vw + s * wps, out + s * wps, T);
            continue;
        }
        if (algo == 5) {   // pass 1 split into extend / walk / climb against the final automaton (16-bit state ids only)
            if (sizeof(Ix) != 2) return 3;
            EulerBlock<uint16_t> B(base, T);
            const uint32_t n = euler_pass1_split(B, qw + s * wps, kw + s * wps, T);
            if (n > node_capacity(T)) return 2;
            euler_tour<uint16_t>(B, n);
            euler_pass2<uint16_t>(B, vw + s * wps, out + s * wps, T);
            continue;
        }
        if (algo == 6) {   // incremental pushes of an automaton that is kept between calls (what generation does)
            GenLayout<Ix> L(T);
            WalkerState st;
            st.u = 1; st.g = 0; st.w = 0; st.gmax = 0; st.gfail = 0; st.h = 0; st.steps = 0; st.pad = 0;
            for (uint32_t w = 0; w < wps; ++w) out[s * wps + w] = 0;
            for (uint32_t i = 0; i < T; ++i) {
                const uint32_t bit = gen_push<Ix>(reinterpret_cast<Node<Ix>*>(base + L.nodes), reinterpret_cast<Ix*>(base + L.last),
                                                  reinterpret_cast<Ix*>(base + L.path), vw + s * wps, &st,
                                                  stream_bit(qw + s * wps, i), stream_bit(kw + s * wps, i));
                out[s * wps + (i >> 5)] |= bit << (i & 31);
            }
            continue;
        }
        if (algo == 7) {   // interleaved pass 1 with the climb taken out of the serial loop (16-bit state ids only)
            if (sizeof(Ix) != 2) return 3;
            EulerBlock<uint16_t> B(base, T);
            const uint32_t n = euler_pass1_deferred(B, qw + s * wps, kw + s * wps, T);
            if (n > node_capacity(T)) return 2;
            euler_tour<uint16_t>(B, n);
            euler_pass2<uint16_t>(B, vw + s * wps, out + s * wps, T);
            continue;
        }
        if (algo >= 100) {   // the split form with the query walk in pieces of (algo - 100) steps
            if (sizeof(Ix) != 2) return 3;
            EulerBlock<uint16_t> B(base, T);
            const uint32_t n = euler_pass1_split_chunked(B, qw + s * wps, kw + s * wps, T, (uint32_t)(algo - 100));
            if (n > node_capacity(T)) return 2;
            euler_tour<uint16_t>(B, n);
            euler_pass2<uint16_t>(B, vw + s * wps, out + s * wps, T);
            continue;
        }
        if (algo == 0)
            run_eager<Ix>(base, qw + s * wps, kw + s * wps, vw + s * wps, out + s * wps, T, &cnt);
        else if (!run_euler<Ix>(base, qw + s * wps, kw + s * wps, vw + s * wps, out + s * wps, T, &cnt))
            return 2;  // an internal invariant of the automaton failed
    }
    if (visits) *visits = cnt.node_visits;
    if (chain) *chain = cnt.chain_steps;
    return 0;
}

extern "C" int sam_host_batch(int algo, int ix_bits, const uint32_t* qw, const uint32_t* kw, const uint32_t* vw,
                              size_t n_streams, uint32_t T, uint32_t* out, unsigned long long* visits,
                              unsigned long long* chain) {
    if (ix_bits == 16) {
        if (node_capacity(T) > 0xFFFFu) return 1;
        return run_batch<uint16_t>(algo, qw, kw, vw, n_streams, T, out, visits, chain);
    }
    return run_batch<uint32_t>(algo, qw, kw, vw, n_streams, T, out, visits, chain);
}

extern "C" size_t sam_host_scratch_bytes(int algo, int ix_bits, uint32_t T) {
    if (ix_bits == 16) return algo == 0 ? EagerLayout<uint16_t>(T).total : EulerLayout<uint16_t>(T).total;
    return algo == 0 ? EagerLayout<uint32_t>(T).total : EulerLayout<uint32_t>(T).total;
}
