// ROSA 1-bit suffix-automaton match on the GPU: one thread per (sequence,
// channel) stream, automaton state in a per-stream block of global scratch
// (compact 16-bit state ids whenever 2T+2 <= 65535), bit streams read and idx
// bits written as stream-major 32-step words.  The per-stream algorithm lives
// in sam_core.cuh; results equal T pushes of the reference's RosaSam
// (src/rosa.rs:100-176) for every stream.
//
// Streams with constant k bits are finished by a closed form first; the rest
// are processed in waves sized to the scratch budget, so any batch works; all
// waves are enqueued back to back on the runtime stream.
#include <algorithm>

#include "kernels.hpp"
#include "sam_coop.cuh"
#include "sam_core.cuh"

namespace ullis {
namespace k {

namespace {

// Streams that need no automaton are settled here with a few word operations
// (sam_core.cuh, "constant k", "constant v" and "constant q"): k bits all equal, v bits all 0
// (idx = 0), v bits all 1 (idx_t = "q_t has occurred among the earlier keys") and q bits all
// equal (a scan over the key runs, in a kernel of its own).
// Every other stream id is appended to `list` for the automaton kernels.
// Eight lanes share a stream: each takes every eighth word of its three bit streams (a group reads 32
// consecutive bytes per request), the group combines by shuffle, and the closed forms - all of them word by
// word - are written the same way.  One thread per stream spent its time in 3 x 64 dependent strided loads.
constexpr int CLASSIFY_LANES = 8;
__global__ void __launch_bounds__(128)
rosa_classify_kernel(const uint32_t* __restrict__ q_sw, const uint32_t* __restrict__ k_sw,
                     const uint32_t* __restrict__ v_sw, uint32_t* __restrict__ idx_sw, size_t streams, uint32_t T,
                     size_t wps, uint32_t* __restrict__ list, uint32_t* __restrict__ count,
                     uint32_t* __restrict__ cq_list, uint32_t* __restrict__ cq_count) {
    constexpr uint32_t G = CLASSIFY_LANES;
    const size_t s = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) / G;
    if (s >= streams) return;   // a whole group
    const uint32_t sub = threadIdx.x % G, lane = threadIdx.x & 31u;
    const uint32_t group = ((1u << G) - 1u) << (lane & ~(G - 1u));
    const uint32_t* qw = q_sw + s * wps;
    const uint32_t* kw = k_sw + s * wps;
    const uint32_t* vw = v_sw + s * wps;
    uint32_t* out = idx_sw + s * wps;
    const uint32_t last = (uint32_t)wps - 1u;
    const uint32_t tail = (T & 31u) ? ((1u << (T & 31u)) - 1u) : 0xFFFFFFFFu;
    // AND and OR of the three streams over steps 0 .. T-1 (the bits past T in the last word count for neither)
    uint32_t all[3] = {0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu}, any[3] = {0u, 0u, 0u};
    for (uint32_t w = sub; w <= last; w += G) {
        const uint32_t m = w == last ? tail : 0xFFFFFFFFu;
        const uint32_t x[3] = {kw[w], vw[w], qw[w]};
#pragma unroll
        for (int a = 0; a < 3; ++a) {
            all[a] &= x[a] | ~m;
            any[a] |= x[a] & m;
        }
    }
#pragma unroll
    for (int a = 0; a < 3; ++a) {
#pragma unroll
        for (uint32_t o = 1; o < G; o <<= 1) {
            all[a] &= __shfl_xor_sync(group, all[a], o);
            any[a] |= __shfl_xor_sync(group, any[a], o);
        }
    }
    auto constant = [&](int a, uint32_t* c) {
        if (all[a] == 0xFFFFFFFFu) { *c = 1u; return true; }
        if (any[a] == 0u) { *c = 0u; return true; }
        return false;
    };
    uint32_t c = 0;
    if (constant(0, &c)) {
        // sam::run_constant_k, a word per lane
        for (uint32_t w = sub; w <= last; w += G) {
            uint32_t word = (c ? qw[w] : ~qw[w]) & vw[w];
            if (w == 0) word &= ~1u;
            if (w == last) word &= tail;
            out[w] = word;
        }
    } else if (constant(1, &c)) {
        if (c == 0) {
            for (uint32_t w = sub; w <= last; w += G) out[w] = 0u;
        } else {
            // sam::run_constant_v_one: f = the first step whose key differs from k_0 (it exists: k is not constant)
            const uint32_t c0 = kw[0] & 1u, full = c0 ? 0xFFFFFFFFu : 0u;
            uint32_t f = T;
            for (uint32_t w = sub; w <= last && f == T; w += G) {
                uint32_t diff = kw[w] ^ full;
                if (w == last) diff &= tail;
                if (diff) f = w * 32u + (uint32_t)__ffs((int)diff) - 1u;
            }
#pragma unroll
            for (uint32_t o = 1; o < G; o <<= 1) f = min(f, __shfl_xor_sync(group, f, o));
            for (uint32_t w = sub; w <= last; w += G) {
                const uint32_t same = c0 ? qw[w] : ~qw[w];   // q_t == k_0
                uint32_t after;                               // bits of this word at steps > f
                if (f >= w * 32u + 31u) after = 0u;
                else if (f < w * 32u) after = 0xFFFFFFFFu;
                else after = ~((2u << (f - w * 32u)) - 1u);
                uint32_t word = (same & ~after) | after;
                if (w == 0) word &= ~1u;
                if (w == last) word &= tail;
                out[w] = word;
            }
        }
    } else if (sub == 0) {
        if (constant(2, &c)) cq_list[atomicAdd(cq_count, 1u)] = (uint32_t)s;   // constant q: a long scan, its own kernel
        else list[atomicAdd(count, 1u)] = (uint32_t)s;
    }
}

// The constant-q streams listed by rosa_classify_kernel, one per thread: every thread of a warp runs the
// same scan (inside rosa_classify_kernel a warp would pay for it beside each of the shorter closed forms).
__global__ void __launch_bounds__(128)
rosa_constq_kernel(const uint32_t* __restrict__ q_sw, const uint32_t* __restrict__ k_sw, const uint32_t* __restrict__ v_sw,
                   uint32_t* __restrict__ idx_sw, uint32_t T, size_t wps, const uint32_t* __restrict__ cq_list,
                   const uint32_t* __restrict__ cq_count) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= *cq_count) return;
    const size_t s = cq_list[i];
    sam::run_constant_q(q_sw[s * wps] & 1u, k_sw + s * wps, v_sw + s * wps, idx_sw + s * wps, T);
}

// Only `lanes` threads of each warp carry a stream (the others exit at once).
// A warp-level load completes when its slowest lane does, and a stream's
// accesses are pointer chases into its own state block, so fewer streams per
// warp (and more warps) shortens every dependent step.  Work item i of this
// launch is stream list[first + i]; its state block is block i of `scratch`.
template <typename Ix, int ALGO>
__global__ void __launch_bounds__(128)
rosa_sam_kernel(uint8_t* __restrict__ scratch, size_t scratch_stride, const uint32_t* __restrict__ q_sw,
                const uint32_t* __restrict__ k_sw, const uint32_t* __restrict__ v_sw,
                uint32_t* __restrict__ idx_sw, const uint32_t* __restrict__ list,
                const uint32_t* __restrict__ count, size_t first, size_t wave, uint32_t T, size_t wps, int lanes,
                uint32_t* __restrict__ status) {
    const int lane = threadIdx.x & 31;
    const int spread = 32 / lanes;
    if (lane % spread != 0) return;
    const size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const size_t item = warp * lanes + lane / spread;
    // the grid is rounded up to whole CTAs: an item past the wave has no state block (it belongs to the next wave)
    if (item >= wave || first + item >= *count) return;
    const size_t s = list[first + item];
    uint8_t* block = scratch + item * scratch_stride;
    const uint32_t* qw = q_sw + s * wps;
    const uint32_t* kw = k_sw + s * wps;
    const uint32_t* vw = v_sw + s * wps;
    uint32_t* out = idx_sw + s * wps;
    if (ALGO == ULLIS_CUDA_SAM_EAGER)
        sam::run_eager<Ix>(block, qw, kw, vw, out, T, nullptr);
    else if (!sam::run_euler<Ix>(block, qw, kw, vw, out, T, nullptr)) {
        if (atomicCAS(status, ULLIS_DEV_OK, ULLIS_DEV_SAM_CAPACITY) == ULLIS_DEV_OK) status[1] = (uint32_t)s;
    }
}

// streams of the wave [first, first + wave) that reached the automaton
__device__ __forceinline__ uint32_t wave_items(uint32_t total, size_t first, size_t wave) {
    if (first >= total) return 0u;
    const size_t left = total - first;
    return (uint32_t)(left < wave ? left : wave);
}

// Two-kernel form of the O(T log T) schedule for streams whose tour / pass 2
// working set fits shared memory: pass 1 one thread per stream (below), then
// one warp per stream for the parallel phases (sam_coop.cuh).
// WORDS: 0 = field-wise state layout, 1 = packed words, 2 = packed words with the climb left to the tour kernel,
// 3 = the same without the register copy of the query state's words (one load per step instead of the patches)
// (a kernel each, so that the form that runs gets the registers to itself)
// (16 CTAs per SM = 32 registers: with 40 registers the same loop ran 4 % slower at 64 sequences and 40 % slower at 8)
template <int WORDS>
__global__ void __launch_bounds__(128, 16)
rosa_pass1_kernel(uint8_t* __restrict__ scratch, size_t scratch_stride, const uint32_t* __restrict__ q_sw,
                  const uint32_t* __restrict__ k_sw, const uint32_t* __restrict__ list,
                  const uint32_t* __restrict__ count, size_t first, size_t wave, uint32_t T, size_t wps, int lanes,
                  uint32_t dense_count, uint32_t sparse_count, uint32_t* __restrict__ hint) {
    // how many streams reached the automaton, for the host's choice of kernel the next time round (see rosa_sam)
    if (hint && blockIdx.x == 0 && threadIdx.x == 0) *hint = *count;
    // lanes == 0: choose from the number of streams that are left, which only the device knows -
    // many streams: four per warp (fewer issued instructions); fewer: two, then one per warp (more
    // warps to hide the pointer-chase latency).  The grid is sized for one per warp.
    if (lanes == 0) lanes = *count > dense_count ? 4 : *count > sparse_count ? 2 : 1;
    const int lane = threadIdx.x & 31;
    const int spread = 32 / lanes;
    if (lane % spread != 0) return;
    const size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const size_t item = warp * lanes + lane / spread;
    // the grid is sized for one stream per warp and rounded up to whole CTAs: with several streams per warp an
    // item can lie past the wave, where it has no state block (it belongs to the next wave)
    if (item >= wave || first + item >= *count) return;
    const size_t s = list[first + item];
    sam::EulerBlock<uint16_t> B(scratch + item * scratch_stride, T);
    if (WORDS == 3) sam::euler_pass1_words<true, true>(B, q_sw + s * wps, k_sw + s * wps, T);
    else if (WORDS == 2) sam::euler_pass1_words<true, false>(B, q_sw + s * wps, k_sw + s * wps, T);
    else if (WORDS == 1) sam::euler_pass1_words<false>(B, q_sw + s * wps, k_sw + s * wps, T);
    else sam::euler_pass1<uint16_t>(B, q_sw + s * wps, k_sw + s * wps, T, nullptr);
}

// The same serial pass with the state array of the stream in shared memory, for calls with so few streams that
// every one of them gets its own one-warp CTA at once (six per SM at T = 2048): lane 0 runs the loop - a state
// visit is then a shared-memory access instead of a trip through L1, whose lines the step's own stores keep
// displacing - and the whole warp copies the states out for the tour kernel.  The grid covers every stream of
// the wave, so any number of them is handled (in rounds of resident CTAs); the host launches this form only
// when it expects one round.
__global__ void __launch_bounds__(32)
rosa_pass1_smem_kernel(uint8_t* __restrict__ scratch, size_t scratch_stride, const uint32_t* __restrict__ q_sw,
                       const uint32_t* __restrict__ k_sw, const uint32_t* __restrict__ list,
                       const uint32_t* __restrict__ count, size_t first, size_t wave, uint32_t T, size_t wps,
                       uint32_t* __restrict__ hint) {
    extern __shared__ __align__(16) uint8_t pass1_states[];
    if (hint && blockIdx.x == 0 && threadIdx.x == 0) *hint = *count;
    const size_t item = blockIdx.x;
    if (item >= wave_items(*count, first, wave)) return;
    const size_t s = list[first + item];
    sam::EulerBlock<uint16_t> B(scratch + item * scratch_stride, T);
    if (threadIdx.x == 0) {
        sam::EulerBlock<uint16_t> S = B;
        S.N = reinterpret_cast<sam::Node<uint16_t>*>(pass1_states);
        sam::euler_pass1_words<true, true>(S, q_sw + s * wps, k_sw + s * wps, T);
    }
    __syncwarp();
    const uint32_t n = B.meta[0];   // written by lane 0 just now
    const uint4* src = reinterpret_cast<const uint4*>(pass1_states);
    uint4* dst = reinterpret_cast<uint4*>(B.N);
    for (uint32_t i = threadIdx.x; i < (n + 1u) / 2u; i += 32u) dst[i] = src[i];
}

// Pass 1 in three parts (sam_core.cuh, "pass 1 in three parts"): the extend chain and the query walk as two
// kernels with one thread per stream each, the climb inside the tour kernel.  Work items and state blocks as in
// rosa_pass1_kernel.
__device__ __forceinline__ bool split_item(const uint32_t* __restrict__ count, size_t first, size_t wave, int lanes,
                                           uint32_t dense_count, uint32_t sparse_count, size_t* item_out) {
    if (lanes == 0) lanes = *count > dense_count ? 4 : *count > sparse_count ? 2 : 1;
    const int lane = threadIdx.x & 31;
    const int spread = 32 / lanes;
    if (lane % spread != 0) return false;
    const size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const size_t item = warp * lanes + lane / spread;
    if (item >= wave || first + item >= *count) return false;
    *item_out = item;
    return true;
}

__global__ void __launch_bounds__(128, 16)
rosa_extend_kernel(uint8_t* __restrict__ scratch, size_t scratch_stride, const uint32_t* __restrict__ k_sw,
                   const uint32_t* __restrict__ list, const uint32_t* __restrict__ count, size_t first, size_t wave,
                   uint32_t T, size_t wps, int lanes, uint32_t dense_count, uint32_t sparse_count) {
    // All lanes of the group that belongs to a stream first fill the stream's `orig` array with NIL (16-byte
    // stores, the lanes side by side); then one lane of the group runs the chain and the others leave.
    if (lanes == 0) lanes = *count > dense_count ? 4 : *count > sparse_count ? 2 : 1;
    const int lane = threadIdx.x & 31, spread = 32 / lanes;
    const size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const size_t item = warp * lanes + lane / spread;
    const bool live = item < wave && first + item < *count;
    if (live) {
        sam::EulerBlock<uint16_t> B(scratch + item * scratch_stride, T);
        uint4* o = reinterpret_cast<uint4*>(B.next);                       // 16-byte aligned by the layout
        const uint32_t vecs = (sam::node_capacity(T) * 2u + 15u) / 16u;    // the array's room is a multiple of 16 bytes
        for (uint32_t k = lane % spread; k < vecs; k += spread) o[k] = make_uint4(~0u, ~0u, ~0u, ~0u);
    }
    __syncwarp();
    if (!live || lane % spread != 0) return;
    const size_t s = list[first + item];
    sam::EulerBlock<uint16_t> B(scratch + item * scratch_stride, T);
    sam::euler_extend_words(B, k_sw + s * wps, T);
}

__global__ void __launch_bounds__(128, 16)
rosa_walk_kernel(uint8_t* __restrict__ scratch, size_t scratch_stride, const uint32_t* __restrict__ q_sw,
                 const uint32_t* __restrict__ list, const uint32_t* __restrict__ count, size_t first, size_t wave,
                 uint32_t T, size_t wps, int lanes, uint32_t dense_count, uint32_t sparse_count) {
    size_t item;
    if (!split_item(count, first, wave, lanes, dense_count, sparse_count, &item)) return;
    const size_t s = list[first + item];
    sam::EulerBlock<uint16_t> B(scratch + item * scratch_stride, T);
    uint32_t w = 0, h = 0;
    sam::euler_walk_words<false>(B, q_sw + s * wps, 0, T, w, h);
}

// The query walk with eight lanes per stream (sam_core.cuh euler_walk_chunked): each lane first walks an eighth of
// the steps from the guessed state "no match", all at once; then the pieces are put right one after the other,
// each from the true end state of the piece before it, which takes a few steps where matches are short.  Four
// streams per warp.  A lane only ever reads the records it wrote itself.
__global__ void __launch_bounds__(128, 16)
rosa_walk_chunked_kernel(uint8_t* __restrict__ scratch, size_t scratch_stride, const uint32_t* __restrict__ q_sw,
                         const uint32_t* __restrict__ list, const uint32_t* __restrict__ count, size_t first, size_t wave,
                         uint32_t T, size_t wps) {
    const int lane = threadIdx.x & 31, group = lane >> 3, c = lane & 7;
    const size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const size_t item = warp * 4 + group;
    if (item >= wave || first + item >= *count) return;   // the eight lanes of a group leave together
    const size_t s = list[first + item];
    sam::EulerBlock<uint16_t> B(scratch + item * scratch_stride, T);
    const uint32_t* qw = q_sw + s * wps;
    const uint32_t piece = (((T + 7u) >> 3) + 31u) & ~31u;
    const uint32_t t0 = min((uint32_t)c * piece, T), t1 = min(t0 + piece, T);
    uint32_t w = 0, h = 0;
    sam::euler_walk_words<false>(B, qw, t0, t1, w, h);
    const unsigned mask = 0xFFu << (8 * group);
    for (int k = 1; k < 8; ++k) {
        const uint32_t pw = __shfl_sync(mask, w, (lane & ~7) + k - 1), ph = __shfl_sync(mask, h, (lane & ~7) + k - 1);
        if (c != k) continue;
        if (t0 >= t1) {           // an empty piece hands the state on
            w = pw; h = ph;
        } else {
            uint32_t tw = pw, th = ph;
            if (sam::euler_walk_words<true>(B, qw, t0, t1, tw, th) == t1) { w = tw; h = th; }   // never met: its own end state
        }
    }
}

template <int NT, int MODE = 0>   // 0: pass 1 left v_t; 1: split form (climb here, clones from orig); 2: deferred climb
__global__ void __launch_bounds__(NT)
rosa_coop_kernel(uint8_t* __restrict__ scratch, size_t scratch_stride, const uint32_t* __restrict__ v_sw,
                 uint32_t* __restrict__ idx_sw, const uint32_t* __restrict__ list, const uint32_t* __restrict__ count,
                 size_t first, uint32_t T, size_t wps, uint32_t* __restrict__ status) {
    extern __shared__ __align__(16) uint8_t coop_smem[];
    const size_t item = blockIdx.x;
    if (first + item >= *count) return;
    const size_t s = list[first + item];
    sam::EulerBlock<uint16_t> B(scratch + item * scratch_stride, T);
    if (B.meta[0] > sam::node_capacity(T)) {  // cannot happen: at most 2T states
        if (threadIdx.x == 0 && atomicCAS(status, ULLIS_DEV_OK, ULLIS_DEV_SAM_CAPACITY) == ULLIS_DEV_OK)
            status[1] = (uint32_t)s;
        return;
    }
    sam::coop_tour_pass2<NT, MODE != 0, MODE == 1>(coop_smem, B, v_sw + s * wps, idx_sw + s * wps, T);
}

// EAGER keeps the reference's schedule for every stream (no shortcut): list = all streams
__global__ void rosa_list_all_kernel(uint32_t* __restrict__ list, uint32_t* __restrict__ count, size_t streams) {
    const size_t s = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (s < streams) list[s] = (uint32_t)s;
    if (s == 0) *count = (uint32_t)streams;
}

template <typename Ix>
size_t stride_for(int algo, size_t T) {
    return algo == ULLIS_CUDA_SAM_EAGER ? sam::EagerLayout<Ix>((uint32_t)T).total
                                        : sam::EulerLayout<Ix>((uint32_t)T).total;
}

}  // namespace

size_t rosa_sam_scratch_bytes_per_stream(int algo, size_t time) {
    const bool narrow = sam::node_capacity((uint32_t)time) <= 0xFFFFu;
    return narrow ? stride_for<uint16_t>(algo, time) : stride_for<uint32_t>(algo, time);
}

void rosa_sam(ullis_cuda_runtime* rt, const uint32_t* q_sw, const uint32_t* k_sw, const uint32_t* v_sw,
              uint32_t* idx_sw, size_t streams, size_t time, int site) {
    if (streams == 0 || time == 0) return;
    if (time > 0x3FFFFFFFu) fail(ULLIS_CUDA_ERR_SHAPE, "ROSA time does not fit 32-bit state ids");
    const int algo = rt->sam_algo;
    const bool narrow = sam::node_capacity((uint32_t)time) <= 0xFFFFu;
    const size_t stride = rosa_sam_scratch_bytes_per_stream(algo, time);
    const size_t wps = (time + 31) / 32;
    // wave size: all streams at once when the scratch buffer already holds them;
    // otherwise bounded scratch (12 GiB unless ULLIS_CUDA_SAM_BUDGET_MB says otherwise, or what fits in free memory).
    // The memory query is a blocking driver call, so it is kept off the steady state.
    size_t wave = streams;
    if (rt->sam_scratch.bytes() < streams * stride) {
        size_t free_b = 0, total_b = 0;
        ULLIS_CUDA_CHECK(cudaMemGetInfo(&free_b, &total_b));
        size_t budget = rt->sam_budget_bytes;
        const size_t avail = free_b + rt->sam_scratch.bytes();  // what the scratch buffer could grow to
        if (avail < budget + ((size_t)2 << 30)) budget = avail > ((size_t)4 << 30) ? avail - ((size_t)2 << 30) : avail / 2;
        wave = budget / stride;
        if (wave == 0) fail(ULLIS_CUDA_ERR_NOMEM, "not enough device memory for one suffix-automaton state block");
        if (wave > streams) wave = streams;
    }
    uint8_t* scratch = static_cast<uint8_t*>(rt->sam_scratch.ensure(wave * stride));
    if (streams > 0xFFFFFFFFull) fail(ULLIS_CUDA_ERR_SHAPE, "too many ROSA streams");
    uint32_t* list = rt->sam_list.as<uint32_t>(2 * streams + 2);
    rt->sam_last_streams = streams;
    if (!rt->parent) rt->lanes_last = 1;   // a forward that splits its batch raises this after its last layer
    uint32_t* count = list + streams;
    uint32_t* cq_count = count + 1;           // the constant-q streams, settled by a kernel of their own
    uint32_t* cq_list = count + 2;
    const unsigned cgrid = (unsigned)((streams + 127) / 128);
    // The number of streams left for the automaton is only known on the device;
    // each wave is sized for the worst case and surplus threads exit at once.
    const sam::CoopLayout coop((uint32_t)time);
    const bool use_coop = algo == ULLIS_CUDA_SAM_EULER && narrow && rt->sam_coop && coop.total <= 226 * 1024 &&
                          2 * sam::node_capacity((uint32_t)time) < 0xFFFFu;
    // The constant-q kernel runs on the side stream from the fork below until `stream` has waited for side_join.
    // Whichever way this function leaves in between (a launch error throws), the wait is issued: the next call
    // clears the counters and lists that kernel still reads.
    struct SideJoin {
        ullis_cuda_runtime* rt;
        bool forked = false;
        ~SideJoin() {
            if (forked) cudaStreamWaitEvent(rt->stream, rt->side_join, 0);
        }
    } side{rt};
    if (algo == ULLIS_CUDA_SAM_EAGER) {
        rosa_list_all_kernel<<<cgrid, 128, 0, rt->stream>>>(list, count, streams);
        rt->launched("rosa_list_all");
    } else {
        rt->zero(count, 8);   // both counters
        const unsigned classify_grid = (unsigned)((streams * CLASSIFY_LANES + 127) / 128);
        rosa_classify_kernel<<<classify_grid, 128, 0, rt->stream>>>(q_sw, k_sw, v_sw, idx_sw, streams, (uint32_t)time, wps, list,
                                                             count, cq_list, cq_count);
        rt->launched("rosa_classify");
        // The constant-q scan is a long serial loop for a few thousand threads; it depends on nothing but the
        // classification and writes idx words no other kernel of this call touches, so it runs on the side stream
        // beside the automaton pass (which is bound by latency and leaves most issue slots free).
        if (rt->sam_side) {
            if (!rt->side_stream) {
                ULLIS_CUDA_CHECK(cudaStreamCreateWithFlags(&rt->side_stream, cudaStreamNonBlocking));
                ULLIS_CUDA_CHECK(cudaEventCreateWithFlags(&rt->side_fork, cudaEventDisableTiming));
                ULLIS_CUDA_CHECK(cudaEventCreateWithFlags(&rt->side_join, cudaEventDisableTiming));
            }
            ULLIS_CUDA_CHECK(cudaEventRecord(rt->side_fork, rt->stream));
            ULLIS_CUDA_CHECK(cudaStreamWaitEvent(rt->side_stream, rt->side_fork, 0));
            // side_join must be recorded behind whatever reached the side stream, also when a step below throws
            struct Recorder {
                ullis_cuda_runtime* rt;
                SideJoin* side;
                ~Recorder() {
                    if (cudaEventRecord(rt->side_join, rt->side_stream) == cudaSuccess) side->forked = true;
                }
            };
            Recorder recorder{rt, &side};
            if (rt->kernel_timing) rt->side_begin();
            rosa_constq_kernel<<<cgrid, 128, 0, rt->side_stream>>>(q_sw, k_sw, v_sw, idx_sw, (uint32_t)time, wps, cq_list,
                                                                   cq_count);
            const cudaError_t e = cudaGetLastError();
            if (e != cudaSuccess) fail(ULLIS_CUDA_ERR_CUDA, std::string("launch of rosa_constq: ") + cudaGetErrorString(e));
            ++rt->launches;
            if (rt->kernel_timing) rt->side_end("rosa_constq");
        } else {
            rosa_constq_kernel<<<cgrid, 128, 0, rt->stream>>>(q_sw, k_sw, v_sw, idx_sw, (uint32_t)time, wps, cq_list, cq_count);
            rt->launched("rosa_constq");
        }
    }
    if (use_coop && !rt->sam_coop_ready) {
#define ULLIS_COOP_SMEM(NT, MODE) \
    ULLIS_CUDA_CHECK(cudaFuncSetAttribute(rosa_coop_kernel<NT, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024))
        ULLIS_COOP_SMEM(256, 0); ULLIS_COOP_SMEM(512, 0); ULLIS_COOP_SMEM(1024, 0);
        ULLIS_COOP_SMEM(256, 1); ULLIS_COOP_SMEM(512, 1); ULLIS_COOP_SMEM(1024, 1);
        ULLIS_COOP_SMEM(256, 2); ULLIS_COOP_SMEM(512, 2); ULLIS_COOP_SMEM(1024, 2);
#undef ULLIS_COOP_SMEM
        rt->sam_coop_ready = true;
    }
    for (size_t s0 = 0; s0 < streams; s0 += wave) {
        const size_t n = streams - s0 < wave ? streams - s0 : wave;
        const int lanes = rt->sam_lanes;
        const size_t warps = (n + lanes - 1) / lanes;
        const unsigned grid = (unsigned)((warps * 32 + 127) / 128);
        if (use_coop) {
            // sam_lanes_fixed: the caller pinned the streams per warp; otherwise the kernel picks 2 or 4
            const int pass1_lanes = rt->sam_lanes_fixed ? lanes : 0;
            const size_t pass1_warps = rt->sam_lanes_fixed ? warps : n;
            const unsigned p1_grid = (unsigned)((pass1_warps * 32 + 127) / 128);
            const uint32_t dense = 96u * (uint32_t)rt->sm_count, sparse = rt->sam_sparse_per_sm * (uint32_t)rt->sm_count;
            const bool split = rt->sam_split && rt->sam_words;
            const bool defer = !split && rt->sam_words && rt->sam_defer_climb;
            const int coop_mode = split ? 1 : defer ? 2 : 0;
            if (split) {
                rosa_extend_kernel<<<p1_grid, 128, 0, rt->stream>>>(scratch, stride, k_sw, list, count, s0, n,
                                                                   (uint32_t)time, wps, pass1_lanes, dense, sparse);
                rt->launched("rosa_extend");
                if (rt->sam_walk_chunked) {
                    rosa_walk_chunked_kernel<<<(unsigned)(((n + 3) / 4 * 32 + 127) / 128), 128, 0, rt->stream>>>(
                        scratch, stride, q_sw, list, count, s0, n, (uint32_t)time, wps);
                } else {
                    rosa_walk_kernel<<<p1_grid, 128, 0, rt->stream>>>(scratch, stride, q_sw, list, count, s0, n,
                                                                     (uint32_t)time, wps, pass1_lanes, dense, sparse);
                }
                rt->launched("rosa_walk");
            } else {
                // Few streams: the state arrays in shared memory, one one-warp CTA per stream, all resident at once.
                // How many streams reach the automaton is known on the device only, so the choice goes by what the
                // same call site (`site`: the model's layer) saw the last time its kernel ran - the kernels leave
                // that number in pinned host memory - and only when it was well inside one round of resident CTAs.
                // Either kernel is correct for any number of streams; a wrong guess costs time, not results.
                const size_t state_bytes = (size_t)sam::node_capacity((uint32_t)time) * sizeof(sam::Node<uint16_t>);
                uint32_t* hint = rt->sam_hint_slot(site);
                bool in_smem = false;
                if (defer && rt->sam_reload_w && rt->sam_smem_waves > 0 && hint && wave == streams &&
                    state_bytes <= 226 * 1024) {
                    const size_t per_sm = std::min<size_t>(32, (227 * 1024) / (state_bytes + 1024));
                    const size_t resident = per_sm * (size_t)rt->sm_count * (size_t)rt->sam_smem_waves;
                    const uint32_t expected = *static_cast<volatile uint32_t*>(hint);
                    in_smem = rt->sam_smem_waves >= 1000 || (expected != 0xFFFFFFFFu && (size_t)expected + expected / 8 <= resident);
                }
                if (in_smem) {
                    if (!rt->sam_smem_ready) {   // the attribute belongs to the function, not to this runtime: always the same value
                        ULLIS_CUDA_CHECK(cudaFuncSetAttribute(rosa_pass1_smem_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                              226 * 1024));
                        rt->sam_smem_ready = true;
                    }
                    rosa_pass1_smem_kernel<<<(unsigned)n, 32, state_bytes, rt->stream>>>(scratch, stride, q_sw, k_sw, list, count,
                                                                                        s0, n, (uint32_t)time, wps, hint);
                    rt->launched("rosa_pass1_smem");
                } else {
#define ULLIS_PASS1(W) \
    rosa_pass1_kernel<W><<<p1_grid, 128, 0, rt->stream>>>(scratch, stride, q_sw, k_sw, list, count, s0, n, (uint32_t)time, \
                                                          wps, pass1_lanes, dense, sparse, hint)
                if (!rt->sam_words) ULLIS_PASS1(0);
                else if (defer && rt->sam_reload_w) ULLIS_PASS1(3);
                else if (defer) ULLIS_PASS1(2);
                else ULLIS_PASS1(1);
#undef ULLIS_PASS1
                rt->launched("rosa_pass1");
                }
            }
            // threads per stream: the fewer CTAs shared memory lets an SM hold, the more threads each one gets
            const unsigned coop_per_sm = (unsigned)((227u * 1024u) / (coop.total + 1024u));
            const int coop_threads = rt->sam_coop_threads ? rt->sam_coop_threads : coop_per_sm >= 3 ? 256 : coop_per_sm == 2 ? 512 : 1024;
#define ULLIS_COOP_LAUNCH_MODE(NT, MODE)                                                                                 \
    rosa_coop_kernel<NT, MODE><<<(unsigned)n, NT, coop.total, rt->stream>>>(scratch, stride, v_sw, idx_sw, list, count, s0, \
                                                                            (uint32_t)time, wps, rt->dev_status)
#define ULLIS_COOP_LAUNCH(NT)                                 \
    do {                                                      \
        if (coop_mode == 1) ULLIS_COOP_LAUNCH_MODE(NT, 1);    \
        else if (coop_mode == 2) ULLIS_COOP_LAUNCH_MODE(NT, 2); \
        else ULLIS_COOP_LAUNCH_MODE(NT, 0);                   \
    } while (0)
            if (coop_threads == 256) ULLIS_COOP_LAUNCH(256);
            else if (coop_threads == 512) ULLIS_COOP_LAUNCH(512);
            else ULLIS_COOP_LAUNCH(1024);
#undef ULLIS_COOP_LAUNCH_MODE
#undef ULLIS_COOP_LAUNCH
            rt->launched("rosa_coop");
            continue;
        }
#define ULLIS_SAM_LAUNCH(IX, ALGO)                                                                              \
    rosa_sam_kernel<IX, ALGO><<<grid, 128, 0, rt->stream>>>(scratch, stride, q_sw, k_sw, v_sw, idx_sw, list, count, s0, \
                                                           n, (uint32_t)time, wps, lanes, rt->dev_status)
        if (narrow) {
            if (algo == ULLIS_CUDA_SAM_EAGER) ULLIS_SAM_LAUNCH(uint16_t, ULLIS_CUDA_SAM_EAGER);
            else ULLIS_SAM_LAUNCH(uint16_t, ULLIS_CUDA_SAM_EULER);
        } else {
            if (algo == ULLIS_CUDA_SAM_EAGER) ULLIS_SAM_LAUNCH(uint32_t, ULLIS_CUDA_SAM_EAGER);
            else ULLIS_SAM_LAUNCH(uint32_t, ULLIS_CUDA_SAM_EULER);
        }
#undef ULLIS_SAM_LAUNCH
        rt->launched("rosa_sam");
    }
    // `side` goes out of scope here: `stream` waits for the side kernel, idx is complete on `stream` from then on
}

}  // namespace k
}  // namespace ullis
