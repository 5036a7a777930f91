#include "model.hpp"

#include <algorithm>
#include <cstring>

#include "kernels.hpp"
#include "linear_tc.hpp"
#include "safetensors.hpp"

using namespace ullis;

namespace {

constexpr size_t MAX_CONTEXT_LEN = 32768;  // reference src/config.rs:6
constexpr size_t MIN_VOCAB = 260;          // reference src/tokenizer.rs:34 (4 specials + 256 bytes)

const TensorView& need(const SafeTensors& st, const std::string& name, const char* dtype, size_t elements,
                       const char* what) {
    auto it = st.tensors.find(name);
    if (it == st.tensors.end()) fail(ULLIS_CUDA_ERR_CHECKPOINT, "checkpoint tensor " + name);
    if (it->second.dtype != dtype)
        fail(ULLIS_CUDA_ERR_CHECKPOINT, std::string("expected ") + dtype + " tensor, got " + it->second.dtype +
                                            " (" + name + ")");
    if (it->second.elements() != elements) fail(ULLIS_CUDA_ERR_CHECKPOINT, std::string(what) + " (" + name + ")");
    return it->second;
}

struct ArenaPlan {
    struct Item { const uint8_t* src; size_t bytes, offset; };
    std::vector<Item> items;
    size_t total = 0;
    size_t add(const uint8_t* src, size_t bytes) {
        size_t off = total;
        items.push_back({src, bytes, off});
        total = (total + bytes + 255) / 256 * 256;
        return off;
    }
};

}  // namespace

ullis_cuda_model::~ullis_cuda_model() {
    if (rt)
        for (ullis_cuda_runtime* c : rt->children) cudaStreamSynchronize(c->stream);   // shares may still use the buffers
    for (auto& s : spans) {
        cudaEventDestroy(s.start);
        cudaEventDestroy(s.stop);
    }
}

// reference: from_safetensors_bytes (src/model.rs:3470-3553), require_v2
// (2426-2431), TrainConfig::validate (src/config.rs:151-190, without the
// host-memory admission, which is the trainer's policy for its own process),
// validate_checkpoint_shapes (4402-4456), heron_from_checkpoint (4258-4309).
void ullis_cuda_model::load(const uint8_t* bytes, size_t len) {
    if (len && bytes[0] == '{')
        fail(ULLIS_CUDA_ERR_CHECKPOINT, "JSON v2 checkpoints are not supported by the cuda backend; use checkpoint.safetensors");
    SafeTensors st = parse_safetensors(bytes, len);
    if (!st.has_metadata) fail(ULLIS_CUDA_ERR_CHECKPOINT, "safetensors checkpoint is missing metadata");
    uint64_t version = 0;
    {
        auto it = st.metadata.find("format_version");
        if (it != st.metadata.end()) {
            char* endp = nullptr;
            version = strtoull(it->second.c_str(), &endp, 10);
            if (endp == it->second.c_str() || *endp) version = 0;
        }
    }
    if (version != 2)
        fail(ULLIS_CUDA_ERR_CHECKPOINT,
             "Hyena checkpoints (v1) are intentionally unloadable after the RWKV-8 cut (got format_version " +
                 std::to_string(version) + ")");
    auto cit = st.metadata.find("config");
    if (cit == st.metadata.end()) fail(ULLIS_CUDA_ERR_CHECKPOINT, "safetensors checkpoint is missing config");
    Json cfg = parse_json(cit->second.data(), cit->second.size());
    if (cfg.kind != Json::Object) fail(ULLIS_CUDA_ERR_CHECKPOINT, "parse safetensors checkpoint config");
    if (const Json* arch = cfg.get("architecture"))
        if (arch->kind != Json::String || arch->text != "heron")
            fail(ULLIS_CUDA_ERR_CHECKPOINT, "the cuda backend implements the heron architecture only");
    bool ok_d, ok_l, ok_v, ok_c, ok_b;
    d = cfg.u64("d_model", 0, &ok_d);
    layers = cfg.u64("n_layers", 0, &ok_l);
    vocab = cfg.u64("vocab_size", 0, &ok_v);
    context_len = cfg.u64("context_len", 0, &ok_c);
    batch_size = cfg.u64("batch_size", 0, &ok_b);
    if (!(ok_d && ok_l && ok_v && ok_c && ok_b)) fail(ULLIS_CUDA_ERR_CHECKPOINT, "parse safetensors checkpoint config");
    ffn = cfg.u64("dim_ffn", 0);
    if (ffn == 0) ffn = d * 4;  // src/config.rs:135-141
    if (d == 0 || layers == 0) fail(ULLIS_CUDA_ERR_CHECKPOINT, "d_model and n_layers must be non-zero");
    if (vocab < MIN_VOCAB) fail(ULLIS_CUDA_ERR_CHECKPOINT, "vocab_size must be at least " + std::to_string(MIN_VOCAB));
    if (context_len == 0 || context_len > MAX_CONTEXT_LEN)
        fail(ULLIS_CUDA_ERR_CHECKPOINT, "context_len must be in 1..=" + std::to_string(MAX_CONTEXT_LEN));
    if (batch_size == 0) fail(ULLIS_CUDA_ERR_CHECKPOINT, "batch_size must be positive");
    if (cfg.u64("rosa_bits", 1) != 1) fail(ULLIS_CUDA_ERR_CHECKPOINT, "rosa_bits must be 1 in Ullis 0.10");
    if (cfg.u64("head_size", 16) != 16) fail(ULLIS_CUDA_ERR_CHECKPOINT, "head_size must be 16");
    if (d > (1u << 20) || vocab > (1u << 24) || ffn > (1u << 22) || layers > 4096)
        fail(ULLIS_CUDA_ERR_CHECKPOINT, "model size overflow");

    size_t n_blocks = 0;
    while (st.tensors.count("blocks." + std::to_string(n_blocks) + ".ln2.weight")) ++n_blocks;
    if (n_blocks != layers || st.tensors.count("hybrid_blocks.0.ln_a.weight"))
        fail(ULLIS_CUDA_ERR_CHECKPOINT, "heron checkpoint must store exactly n_layers Heron blocks");

    ArenaPlan plan;
    struct Fix { const void** slot; size_t offset; };
    std::vector<Fix> fixes;
    auto put = [&](const void** slot, const TensorView& v) { fixes.push_back({slot, plan.add(v.data, v.bytes)}); };
    auto f16 = [&](const void** slot, const std::string& name, size_t n, const char* what) {
        put(slot, need(st, name, "F16", n, what));
    };
    auto ln = [&](LayerNormWeights& w, const std::string& prefix) {
        f16((const void**)&w.weight, prefix + ".weight", d, "checkpoint LayerNorm shape mismatch");
        f16((const void**)&w.bias, prefix + ".bias", d, "checkpoint LayerNorm shape mismatch");
    };
    // bias: 1 required, 0 forbidden, -1 optional (head: absent loads as zeros)
    std::vector<uint8_t> zero_bias;
    auto packed = [&](PackedWeights& w, const std::string& prefix, size_t out, size_t in, int bias) {
        w.out = out;
        w.in = in;
        put((const void**)&w.bits, need(st, prefix + ".bits", "U32", (out * in + 31) / 32,
                                        "checkpoint packed-linear shape mismatch"));
        f16((const void**)&w.scale, prefix + ".scale", out, "checkpoint packed-linear shape mismatch");
        const bool has = st.tensors.count(prefix + ".bias") != 0;
        if ((bias == 1 && !has) || (bias == 0 && has))
            fail(ULLIS_CUDA_ERR_CHECKPOINT, "checkpoint packed-linear bias mismatch (" + prefix + ")");
        if (has) {
            f16((const void**)&w.bias, prefix + ".bias", out, "checkpoint packed-linear bias mismatch");
        } else if (bias == -1) {
            zero_bias.assign(out * 2, 0);
            fixes.push_back({(const void**)&w.bias, plan.add(zero_bias.data(), zero_bias.size())});
        }
    };

    blocks.assign(layers, LayerWeights{});
    f16((const void**)&embedding, "embedding", vocab * d, "checkpoint embedding shape does not match its configuration");
    ln(ln_out, "ln_out");
    packed(head, "head", vocab, d, -1);
    for (size_t i = 0; i < layers; ++i) {
        const std::string pre = "blocks." + std::to_string(i);
        LayerWeights& L = blocks[i];
        const bool has_ln0 = st.tensors.count(pre + ".ln0.weight") != 0;
        if (has_ln0 != (i == 0)) fail(ULLIS_CUDA_ERR_CHECKPOINT, "ln0 must be present only on Heron layer 0");
        if (has_ln0) ln(L.ln0, pre + ".ln0");
        ln(L.ln2, pre + ".ln2");
        ln(L.ln3, pre + ".ln3");
        f16((const void**)&L.x_q, pre + ".rosa.x_q", d, "checkpoint x_q length mismatch");
        f16((const void**)&L.x_k, pre + ".rosa.x_k", d, "checkpoint x_k length mismatch");
        f16((const void**)&L.x_v, pre + ".rosa.x_v", d, "checkpoint x_v length mismatch");
        f16((const void**)&L.e, pre + ".rosa.e", d, "checkpoint e length mismatch");
        packed(L.q, pre + ".rosa.q", d, d, 1);
        packed(L.k, pre + ".rosa.k", d, d, 1);
        packed(L.v, pre + ".rosa.v", d, d, 1);
        packed(L.o, pre + ".rosa.o", d, d, 1);
        f16((const void**)&L.ffn_x_k, pre + ".ffn.x_k", d, "checkpoint cmix.x_k length mismatch");
        packed(L.key, pre + ".ffn.key", ffn, d, 0);
        f16((const void**)&L.value, pre + ".ffn.value", ffn * d, "checkpoint cmix.value length mismatch");
    }

    rt->bind();
    uint8_t* base = static_cast<uint8_t*>(arena.ensure(plan.total ? plan.total : 256));
    for (const auto& it : plan.items) rt->h2d(base + it.offset, it.src, it.bytes);
    rt->sync();  // sources (file bytes, zero_bias) may go away after return
    for (const auto& f : fixes) *f.slot = base + f.offset;
}

void ullis_cuda_model::check_shape(size_t batch, size_t time) const {
    // reference src/model.rs:2649-2656
    if (batch == 0 || batch > batch_size || time == 0 || time > context_len)
        fail(ULLIS_CUDA_ERR_SHAPE, "token shape or context length is invalid");
}

void ullis_cuda_model::upload_tokens(const uint32_t* tokens, const uint32_t* lab, size_t batch, size_t time) {
    check_shape(batch, time);
    if (!tokens) fail(ULLIS_CUDA_ERR_ARG, "tokens is null");
    if (lanes_open) join_lanes();   // a forward that failed half way left its shares unjoined: they still read the old ids
    const size_t rows = batch * time;
    for (size_t r = 0; r < rows; ++r)
        if (tokens[r] >= vocab) fail(ULLIS_CUDA_ERR_TOKEN, "token id exceeds vocabulary");
    rt->bind();
    rt->h2d(ids.as<uint32_t>(rows), tokens, rows * 4);
    if (lab) rt->h2d(labels.as<uint32_t>(rows), lab, rows * 4);
    cur_batch = batch;
    cur_time = time;
    have_result = false;
    have_pair = false;
}

void ullis_cuda_model::begin(int phase, ullis_cuda_runtime* on) {
    if (!profile) return;
    if (spans_used == spans.size()) {
        Span s{phase, nullptr, nullptr};
        ULLIS_CUDA_CHECK(cudaEventCreate(&s.start));
        ULLIS_CUDA_CHECK(cudaEventCreate(&s.stop));
        spans.push_back(s);
    }
    spans[spans_used].phase = phase;
    ULLIS_CUDA_CHECK(cudaEventRecord(spans[spans_used].start, (on ? on : rt)->stream));
}

void ullis_cuda_model::end(ullis_cuda_runtime* on) {
    if (!profile) return;
    ULLIS_CUDA_CHECK(cudaEventRecord(spans[spans_used].stop, (on ? on : rt)->stream));
    ++spans_used;
}

void ullis_cuda_model::phase_ms(float ms[6]) {
    for (int i = 0; i < 6; ++i) ms[i] = 0.0f;
    rt->sync();
    for (size_t i = 0; i < spans_used; ++i) {
        float t = 0.0f;
        ULLIS_CUDA_CHECK(cudaEventElapsedTime(&t, spans[i].start, spans[i].stop));
        ms[spans[i].phase] += t;
    }
}

void ullis_cuda_model::save_tap(int layer, int which, const void* src, size_t bytes) {
    if (!taps_enabled) return;
    const size_t slot = which == ULLIS_CUDA_TAP_HIDDEN ? layers * 8 : (size_t)layer * 8 + (size_t)which;
    void* dst = tap_bufs[slot].ensure(bytes);
    ULLIS_CUDA_CHECK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, rt->stream));
}

void ullis_cuda_model::save_tap_bits(int layer, int which, const uint32_t* sw, size_t batch, size_t time) {
    if (!taps_enabled) return;
    const size_t slot = (size_t)layer * 8 + (size_t)which;
    uint8_t* dst = tap_bufs[slot].as<uint8_t>(batch * time * d);
    k::rosa_emit(rt, sw, nullptr, dst, nullptr, batch, time, d);
}

void ullis_cuda_model::tap(int layer, int which, void* out, size_t bytes) {
    if (which < 0 || which > ULLIS_CUDA_TAP_HIDDEN) fail(ULLIS_CUDA_ERR_ARG, "unknown tap");
    if (which != ULLIS_CUDA_TAP_HIDDEN && (layer < 0 || (size_t)layer >= layers))
        fail(ULLIS_CUDA_ERR_ARG, "tap layer out of range");
    if (tap_bufs.empty()) fail(ULLIS_CUDA_ERR_ARG, "taps were not enabled for the last forward");
    const size_t slot = which == ULLIS_CUDA_TAP_HIDDEN ? layers * 8 : (size_t)layer * 8 + (size_t)which;
    const bool is_u8 = which >= ULLIS_CUDA_TAP_Q_BITS && which <= ULLIS_CUDA_TAP_IDX;
    const size_t want = tap_rows * d * (is_u8 ? 1 : 4);
    if (!tap_bufs[slot].get() || want == 0) fail(ULLIS_CUDA_ERR_ARG, "taps were not enabled for the last forward");
    if (bytes != want) fail(ULLIS_CUDA_ERR_SHAPE, "tap size mismatch: expected " + std::to_string(want) + " bytes");
    rt->bind();
    rt->d2h(out, tap_bufs[slot].get(), bytes);
    rt->sync();
}

// UllisHeron::hidden (src/model.rs:2644-2683) with HeronBlock::forward
// (2224-2241), RwkvRosaQkv1Bit::forward (1284-1318), RwkvCMixX070::forward
// (987-1001).  The residual stream `x` stays on the device for the whole pass.
//
// Sequences are independent, so the batch is cut into up to `rt->lanes` shares of whole sequences and
// every share runs the pass on a stream of its own: the suffix-automaton kernels are serial chains that
// leave most of an SM's issue slots and all of its tensor pipes idle, and with several shares in flight
// one share's automata run beside another's GEMMs.  Every kernel treats rows (and streams) independently,
// so a sequence gets the same result whichever share carries it.
void ullis_cuda_model::enqueue_hidden(size_t batch, size_t time, bool join) {
    check_shape(batch, time);
    if (batch != cur_batch || time != cur_time) fail(ULLIS_CUDA_ERR_SHAPE, "upload_tokens was not called for this shape");
    rt->bind();
    if (rt->kernel_timing) rt->mark("(between steps)");   // idle time and copies since the last kernel are not the embed kernel's
    const size_t rows = batch * time, n = rows * d;
    const bool exact = rt->mode == ULLIS_CUDA_MODE_EXACT;
    const size_t wps = (time + 31) / 32, sw_words = batch * d * wps;
    x.as<float>(n);
    a.as<float>(n);
    q_sw.as<uint32_t>(sw_words);
    k_sw.as<uint32_t>(sw_words);
    v_sw.as<uint32_t>(sw_words);
    idx_sw.as<uint32_t>(sw_words);
    if (taps_enabled) {
        if (tap_bufs.size() != layers * 8 + 1) tap_bufs = std::vector<DeviceBuffer>(layers * 8 + 1);
        tap_rows = rows;
    }
    if (train_tape && tape_after.size() != layers) {
        tape_after = std::vector<DeviceBuffer>(layers);
        tape_idx = std::vector<DeviceBuffer>(layers);
    }
    spans_used = 0;
    rt->clear_status();

    // shares: one unless every stage runs on the tensor-core kernels (the CUDA-core fall-backs share scratch
    // buffers of the model) and nothing wants the whole batch's intermediates in one place
    size_t n_lanes = 1;
    if (!exact && !taps_enabled && !train_tape && rt->lanes > 1 && batch > 1 &&
        tc::takes_model(rt, time, time, d, ffn, vocab))
        n_lanes = std::min<size_t>((size_t)rt->lanes, batch);
    if (n_lanes == 1) {   // the fall-back buffers, whole batch
        b.as<float>(n);
        c.as<float>(n);
        dd.as<float>(n);
        wide.as<float>(rows * std::max(ffn, d));
    }
    lanes.clear();
    for (size_t i = 0; i < n_lanes; ++i) {
        const size_t lo = i * batch / n_lanes, hi = (i + 1) * batch / n_lanes;
        lanes.push_back(Lane{i == 0 ? rt : rt->child(i - 1), lo, hi - lo});
    }
    if (n_lanes > 1) {
        if (!rt->lane_event) ULLIS_CUDA_CHECK(cudaEventCreateWithFlags(&rt->lane_event, cudaEventDisableTiming));
        ULLIS_CUDA_CHECK(cudaEventRecord(rt->lane_event, rt->stream));   // ids are in place, the status words clear
        for (size_t i = 1; i < n_lanes; ++i) {
            ULLIS_CUDA_CHECK(cudaStreamWaitEvent(lanes[i].rt->stream, rt->lane_event, 0));
            if (lanes[i].rt->kernel_timing) lanes[i].rt->mark("(between steps)");
        }
    }
    lanes_open = n_lanes > 1;

    float* X = x.as<float>(n);
    for (const Lane& ln : lanes) {
        const size_t r0 = ln.seq0 * time, nr = ln.nseq * time;
        begin(PH_EMBED_LN, ln.rt);
        k::embed(ln.rt, ids.as<uint32_t>(rows) + r0, embedding, X + r0 * d, nr, d, vocab);
        end(ln.rt);
    }
    for (size_t l = 0; l < layers; ++l)
        for (const Lane& ln : lanes) enqueue_layer(ln, l, time);
    float* A = a.as<float>(n);
    for (const Lane& ln : lanes) {
        const size_t r0 = ln.seq0 * time, nr = ln.nseq * time;
        begin(PH_HEAD_CE, ln.rt);
        k::layer_norm(ln.rt, X + r0 * d, ln_out.weight, ln_out.bias, A + r0 * d, nr, d, exact);
        end(ln.rt);
    }
    save_tap(0, ULLIS_CUDA_TAP_HIDDEN, A, n * 4);
    rt->lanes_last = n_lanes;
    if (join) join_lanes();
}

void ullis_cuda_model::join_lanes() {
    if (!lanes_open) return;
    for (size_t i = 1; i < lanes.size(); ++i) {
        ULLIS_CUDA_CHECK(cudaEventRecord(lanes[i].rt->lane_event, lanes[i].rt->stream));
        ULLIS_CUDA_CHECK(cudaStreamWaitEvent(rt->stream, lanes[i].rt->lane_event, 0));
    }
    lanes_open = false;
    if (rt->kernel_timing) rt->mark("(join)");   // waiting for the other shares is no kernel's time
}

// One HeronBlock (src/model.rs:2224-2241) over the sequences of one share, on that share's stream.
void ullis_cuda_model::enqueue_layer(const Lane& ln, size_t l, size_t time) {
    ullis_cuda_runtime* r = ln.rt;
    const LayerWeights& L = blocks[l];
    const bool exact = r->mode == ULLIS_CUDA_MODE_EXACT;
    const size_t batch = ln.nseq, rows = batch * time, n = rows * d, r0 = ln.seq0 * time;
    const size_t wps = (time + 31) / 32, sw_words = batch * d * wps, s0 = ln.seq0 * d * wps;
    float* X = static_cast<float*>(x.get()) + r0 * d;
    float* A = static_cast<float*>(a.get()) + r0 * d;
    uint32_t* QS = static_cast<uint32_t*>(q_sw.get()) + s0;
    uint32_t* KS = static_cast<uint32_t*>(k_sw.get()) + s0;
    uint32_t* VS = static_cast<uint32_t*>(v_sw.get()) + s0;
    uint32_t* IS = static_cast<uint32_t*>(idx_sw.get()) + s0;
    // the CUDA-core fall-backs below are only reached with a single share (r0 == 0, whole batch)
    float* Bq = static_cast<float*>(b.get());
    float* Bk = static_cast<float*>(c.get());
    float* Bv = static_cast<float*>(dd.get());
    float* W = static_cast<float*>(wide.get());
    const bool one = lanes.size() == 1;

    begin(PH_EMBED_LN, r);
    if (l == 0) {  // ln0 REPLACES x on layer 0 (src/model.rs:2225-2229)
        k::layer_norm(r, X, L.ln0.weight, L.ln0.bias, A, rows, d, exact);
        ULLIS_CUDA_CHECK(cudaMemcpyAsync(X, A, n * 4, cudaMemcpyDeviceToDevice, r->stream));
    }
    save_tap((int)l, ULLIS_CUDA_TAP_BLOCK_IN, X, n * 4);
    end(r);

    begin(PH_QKV, r);
    // ln3 belongs to the Q/K/V stage: the tensor-core path folds it into its operand kernel (output left in A)
    if (!tc::rosa_qkv_bits(r, A, L, QS, KS, VS, batch, time, d, X, A)) {
        k::layer_norm(r, X, L.ln3.weight, L.ln3.bias, A, rows, d, exact);
        if (!one) fail(ULLIS_CUDA_ERR_ARG, "internal: a split forward reached a fall-back kernel");
        k::shift_mix(r, A, L.x_q, L.x_k, L.x_v, Bq, Bk, Bv, rows, time, d);
        k::binary_linear_exact(r, Bq, L.q.bits, L.q.scale, L.q.bias, W, rows, d, d, false);
        k::sign_pack_streams(r, W, QS, batch, time, d);
        k::binary_linear_exact(r, Bk, L.k.bits, L.k.scale, L.k.bias, W, rows, d, d, false);
        k::sign_pack_streams(r, W, KS, batch, time, d);
        k::binary_linear_exact(r, Bv, L.v.bits, L.v.scale, L.v.bias, W, rows, d, d, false);
        k::sign_pack_streams(r, W, VS, batch, time, d);
    }
    save_tap((int)l, ULLIS_CUDA_TAP_LN3_OUT, A, n * 4);
    save_tap_bits((int)l, ULLIS_CUDA_TAP_Q_BITS, QS, batch, time);
    save_tap_bits((int)l, ULLIS_CUDA_TAP_K_BITS, KS, batch, time);
    save_tap_bits((int)l, ULLIS_CUDA_TAP_V_BITS, VS, batch, time);
    end(r);

    begin(PH_SAM, r);
    k::rosa_sam(r, QS, KS, VS, IS, batch * d, time, (int)l);
    save_tap_bits((int)l, ULLIS_CUDA_TAP_IDX, IS, batch, time);
    if (train_tape)
        ULLIS_CUDA_CHECK(cudaMemcpyAsync(tape_idx[l].as<uint32_t>(sw_words), IS, sw_words * 4,
                                         cudaMemcpyDeviceToDevice, r->stream));
    end(r);

    begin(PH_O, r);
    if (!tc::rosa_out_residual(r, IS, L, X, batch, time, d)) {
        if (!one) fail(ULLIS_CUDA_ERR_ARG, "internal: a split forward reached a fall-back kernel");
        k::rosa_emit(r, IS, L.e, nullptr, A, batch, time, d);
        k::binary_linear_exact(r, A, L.o.bits, L.o.scale, L.o.bias, X, rows, d, d, true);  // x += rosa out
    }
    save_tap((int)l, ULLIS_CUDA_TAP_AFTER_ROSA, X, n * 4);
    if (train_tape)
        ULLIS_CUDA_CHECK(cudaMemcpyAsync(tape_after[l].as<float>(n), X, n * 4, cudaMemcpyDeviceToDevice,
                                         r->stream));
    end(r);

    begin(PH_CMIX, r);
    if (!tc::cmix_residual(r, L, X, batch, time, d, ffn)) {
        if (!one) fail(ULLIS_CUDA_ERR_ARG, "internal: a split forward reached a fall-back kernel");
        k::layer_norm(r, X, L.ln2.weight, L.ln2.bias, A, rows, d, exact);
        k::shift_mix(r, A, L.ffn_x_k, nullptr, nullptr, Bq, nullptr, nullptr, rows, time, d);
        k::binary_linear_exact(r, Bq, L.key.bits, L.key.scale, nullptr, W, rows, d, ffn, false);
        k::relu2(r, W, W, rows * ffn);
        k::fp16_linear_exact(r, W, L.value, X, rows, ffn, d, true);  // x += cmix out
    }
    save_tap((int)l, ULLIS_CUDA_TAP_BLOCK_OUT, X, n * 4);
    end(r);
}

// CE forward of apply_head_ce (src/model.rs:3205-3228, 3253-3257).
void ullis_cuda_model::enqueue_forward_ce(uint32_t ignore_id, size_t batch, size_t time) {
    enqueue_hidden(batch, time, /*join=*/false);
    const size_t rows = batch * time;
    if (!labels.get() || labels.bytes() < rows * 4) fail(ULLIS_CUDA_ERR_ARG, "labels were not uploaded");
    float* A = a.as<float>(rows * d);
    float* RL = row_loss.as<float>(rows);
    uint8_t* res = static_cast<uint8_t*>(result.ensure(32));   // {f64 sum, u64 count} then the same as two f64
    const uint32_t* lab = labels.as<uint32_t>(rows);
    for (const Lane& ln : lanes) {
        // a share is made of whole sequences, so the valid-row rule (row % time, labels[row + 1]) reads the same
        // with the share's own row numbering
        const size_t r0 = ln.seq0 * time, nr = ln.nseq * time;
        begin(PH_HEAD_CE, ln.rt);
        if (!tc::head_ce(ln.rt, A + r0 * d, head, lab + r0, ignore_id, nr, time, d, vocab, RL + r0)) {
            if (lanes.size() != 1) fail(ULLIS_CUDA_ERR_ARG, "internal: a split forward reached a fall-back kernel");
            const size_t chunk = std::max<size_t>(1, std::min<size_t>(rows, ((size_t)256 << 20) / (vocab * 4)));
            float* LG = logits.as<float>(chunk * vocab);
            for (size_t c0 = 0; c0 < rows; c0 += chunk) {
                const size_t nc = std::min(chunk, rows - c0);
                k::binary_linear_exact(rt, A + c0 * d, head.bits, head.scale, head.bias, LG, nc, d, vocab, false);
                k::ce_rows_from_logits(rt, LG, lab, ignore_id, c0, nc, rows, time, vocab, RL);
            }
        }
        end(ln.rt);
    }
    join_lanes();
    begin(PH_HEAD_CE);
    k::ce_reduce(rt, RL, lab, ignore_id, rows, time, reinterpret_cast<double*>(res),
                 reinterpret_cast<unsigned long long*>(res + 8), reinterpret_cast<double*>(res + 16));
    end();
    have_result = true;
    have_pair = true;
}

void ullis_cuda_model::read_loss(float* mean_loss, double* loss_sum, uint64_t* n_valid, float* rl, size_t rows) {
    if (!have_result) fail(ULLIS_CUDA_ERR_ARG, "no forward_ce result to read");
    rt->bind();
    struct { double sum; unsigned long long n; } host;
    rt->d2h(&host, result.get(), 16);
    if (rl) {
        if (rows != cur_batch * cur_time) fail(ULLIS_CUDA_ERR_SHAPE, "row_loss length mismatch");
        rt->d2h(rl, row_loss.get(), rows * 4);
    }
    rt->check_status();  // synchronises
    if (loss_sum) *loss_sum = host.sum;
    if (n_valid) *n_valid = host.n;
    if (mean_loss) *mean_loss = host.n == 0 ? 0.0f : (float)(host.sum / (double)host.n);
}

// The data-parallel form of read_loss: the {loss_sum, n_valid} pair of the last forward is summed over the
// ranks where it lies (one all-reduce on the runtime stream) and read back once - mean = sum / count over
// all ranks, the reference's single-process mean (src/model.rs:3253-3257).
void ullis_cuda_model::read_loss_global(float* mean_loss, double* loss_sum, uint64_t* n_valid) {
    if (!have_result || !have_pair) fail(ULLIS_CUDA_ERR_ARG, "no forward_ce result to read");
    rt->bind();
    double* pair = reinterpret_cast<double*>(static_cast<uint8_t*>(result.get()) + 16);
    dp_allreduce_device(rt, pair, 2);
    have_pair = false;   // the pair now holds the global sums: a second call would add them up again
    double host[2];
    rt->d2h(host, pair, 16);
    rt->check_status();  // synchronises
    const uint64_t n = (uint64_t)(host[1] + 0.5);
    if (loss_sum) *loss_sum = host[0];
    if (n_valid) *n_valid = n;
    if (mean_loss) *mean_loss = n == 0 ? 0.0f : (float)(host[0] / (double)n);
}

// UllisHeron::logits (src/model.rs:2685-2688)
void ullis_cuda_model::enqueue_logits(size_t batch, size_t time, float* host_logits) {
    enqueue_hidden(batch, time);
    const size_t rows = batch * time;
    float* A = a.as<float>(rows * d);
    const size_t chunk = std::max<size_t>(1, std::min<size_t>(rows, ((size_t)256 << 20) / (vocab * 4)));
    float* LG = logits.as<float>(chunk * vocab);
    for (size_t r0 = 0; r0 < rows; r0 += chunk) {
        const size_t nr = std::min(chunk, rows - r0);
        if (!tc::binary_linear(rt, A + r0 * d, head.bits, head.scale, head.bias, LG, nr, d, vocab))
            k::binary_linear_exact(rt, A + r0 * d, head.bits, head.scale, head.bias, LG, nr, d, vocab, false);
        rt->d2h(host_logits + r0 * vocab, LG, nr * vocab * 4);
        rt->sync();  // LG is reused by the next chunk
    }
    rt->check_status();
}
