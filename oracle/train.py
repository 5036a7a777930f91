"""CPU restatement of one Heron training step in rosa_grad=stop_grad_bits mode
(reference src/model.rs:2827-3020 train_step_on).  TEST INFRASTRUCTURE ONLY:
imported by tests/ and by the CPU-baseline leg of bench.py, never by the CUDA
product path.

The forward and the loss come from the C oracle (exact restatement).  The
gradients are numpy float32 matrix products: the reference accumulates them
row by row in f32 (src/model.rs:745-796, 440-456), so the two agree to f32
rounding of a reordered sum, not bit for bit.  The optimiser steps
(src/precision.rs:106-134) are restated exactly, element by element.
"""
from __future__ import annotations

import numpy as np

from . import oracle as O

BINARYCONNECT_INIT_ABS = 0.01   # src/model.rs:550
HEAD_BIAS_LR_MULT = 8.0         # src/model.rs:97
LAYER_NORM_EPS = 1e-5           # src/model.rs:22


def clipped_sgd(bits, residual, gradient, lr):
    """Fp16Storage::apply_clipped_sgd (src/precision.rs:106-113), vectorised:
    every element is independent.  Returns (bits, residual)."""
    cur = O.fp16_to_f32(bits)
    g = np.clip(np.asarray(gradient, np.float32), np.float32(-1.0), np.float32(1.0))
    update = np.float32(lr) * g
    desired = (cur - update) + np.asarray(residual, np.float32)
    new_bits = O.fp16_from_f32(desired)
    return new_bits, (desired - O.fp16_to_f32(new_bits)).astype(np.float32)


def binaryconnect_sgd(bits, residual, gradient, lr):
    """Fp16Storage::apply_binaryconnect_sgd (src/precision.rs:124-134):
    elements whose gradient is zero or not finite are left alone."""
    bits = np.asarray(bits, np.uint16)
    residual = np.asarray(residual, np.float32)
    gradient = np.asarray(gradient, np.float32)
    cur = O.fp16_to_f32(bits)
    live = np.isfinite(gradient) & (gradient != 0)
    g = np.clip(np.where(live, gradient, 0), np.float32(-1.0), np.float32(1.0)).astype(np.float32)
    update = np.float32(lr) * g
    desired = np.clip((cur - update) + residual, np.float32(-1.0), np.float32(1.0)).astype(np.float32)
    nb = O.fp16_from_f32(desired)
    nr = (desired - O.fp16_to_f32(nb)).astype(np.float32)
    return np.where(live, nb, bits).astype(np.uint16), np.where(live, nr, residual).astype(np.float32)


def unpack_signs(bits, out_features, in_features):
    """+1 / -1 matrix [out, in] of a packed linear (bit o*in+i, LSB first;
    src/model.rs:724-742)."""
    b = np.unpackbits(np.ascontiguousarray(bits, np.uint32).view(np.uint8), bitorder="little")
    b = b[:out_features * in_features].reshape(out_features, in_features)
    return (b.astype(np.float32) * 2 - 1).astype(np.float32)


def pack_signs(latent_bits, n):
    """rebinarize (src/model.rs:878-884): bit = latent >= 0 (so -0.0 packs as plus)."""
    plus = O.fp16_to_f32(latent_bits) >= 0
    pad = (-n) % 32
    bits = np.packbits(np.concatenate([plus.astype(np.uint8), np.zeros(pad, np.uint8)]), bitorder="little")
    return bits.view(np.uint32).copy()


def layer_norm_backward(x, gy, w_bits, rows, channels):
    """LayerNorm::backward (src/model.rs:270-315)."""
    x = np.asarray(x, np.float32).reshape(rows, channels)
    gy = np.asarray(gy, np.float32).reshape(rows, channels)
    w = O.fp16_to_f32(w_bits)
    n = np.float32(channels)
    mean = x.sum(1, dtype=np.float32, keepdims=True) / n
    var = ((x - mean) * (x - mean)).sum(1, dtype=np.float32, keepdims=True) / n
    inv = (np.float32(1.0) / np.sqrt(var + np.float32(LAYER_NORM_EPS))).astype(np.float32)
    xhat = (x - mean) * inv
    dxhat = gy * w
    s1 = dxhat.sum(1, dtype=np.float32, keepdims=True)
    s2 = (dxhat * xhat).sum(1, dtype=np.float32, keepdims=True)
    gx = (inv / n) * (n * dxhat - s1 - xhat * s2)
    return gx.astype(np.float32).ravel(), (gy * xhat).sum(0, dtype=np.float32), gy.sum(0, dtype=np.float32)


def packed_backward_ste(x, gy, bits, scale_bits, rows, in_features, out_features):
    """PackedBinaryLinear::backward_ste (src/model.rs:745-796).
    Returns g_w [out, in], g_x [rows, in], g_scale [out], g_bias [out]."""
    x = np.asarray(x, np.float32).reshape(rows, in_features)
    gy = np.asarray(gy, np.float32).reshape(rows, out_features)
    s = unpack_signs(bits, out_features, in_features)
    scale = O.fp16_to_f32(scale_bits)
    gs = gy * scale
    g_w = gs.T @ x
    g_x = gs @ s
    g_scale = (gy * (x @ s.T)).sum(0, dtype=np.float32)
    return g_w.astype(np.float32), g_x.astype(np.float32), g_scale, gy.sum(0, dtype=np.float32)


def lerp_shift_backward(xx, mix_bits, g_shifted, batch, time, channels):
    """lerp_shift_backward (src/model.rs:1206-1240): returns (g_x, g_mix)."""
    xx = np.asarray(xx, np.float32).reshape(batch, time, channels)
    g = np.asarray(g_shifted, np.float32).reshape(batch, time, channels)
    mix = O.fp16_to_f32(mix_bits)
    g_mix = (g * xx).sum((0, 1), dtype=np.float32)
    g_xx = g * mix
    g_x = g - g_xx
    g_x[:, :-1, :] += g_xx[:, 1:, :]
    return g_x.astype(np.float32).ravel(), g_mix


class HeronTrainer:
    """Model + optimiser carry.  `m` is the HeronOracle whose tensors are
    updated in place, so m.forward_ce after a step sees the new weights."""

    def __init__(self, data: bytes):
        self.m = O.HeronOracle(data)
        t = self.m.t
        if "head.bias" not in t:
            t["head.bias"] = np.zeros(self.m.vocab, np.uint16)   # src/model.rs:4237-4246
        self.latent, self.residual = {}, {}
        for prefix in self.packed_names():
            bits = t[prefix + ".bits"]
            n = self._weights(prefix)
            if prefix + ".latent" in t:   # carry of a resumed run (src/model.rs:3461-3466, 3818-3827)
                self.latent[prefix] = t[prefix + ".latent"].copy()
            else:                         # src/model.rs:640-649
                sign = unpack_signs(bits, 1, n).ravel()
                self.latent[prefix] = O.fp16_from_f32(np.float32(BINARYCONNECT_INIT_ABS) * sign)
            self.residual[prefix + ".latent"] = self._res(prefix + ".latent", n)
        for name in self.fp16_names():
            self.residual[name] = self._res(name, t[name].size)

    def _weights(self, prefix):
        m = self.m
        if prefix == "head":
            return m.vocab * m.d
        if prefix.endswith(".ffn.key"):
            return m.ffn * m.d
        return m.d * m.d

    def _res(self, name, n):
        r = self.m.t.get(name + ".residual")
        return np.zeros(n, np.float32) if r is None else r.astype(np.float32).copy()

    def packed_names(self):
        names = ["head"]
        for l in range(self.m.layers):
            names += [f"blocks.{l}.rosa.o", f"blocks.{l}.ffn.key"]
        return names

    def fp16_names(self):
        """FP16 tensors a stop_grad_bits step updates (q/k/v, their mixes and ln3 are frozen)."""
        names = ["embedding", "ln_out.weight", "ln_out.bias", "head.scale", "head.bias"]
        for l in range(self.m.layers):
            p = f"blocks.{l}"
            if l == 0:
                names += [p + ".ln0.weight", p + ".ln0.bias"]
            names += [p + ".ln2.weight", p + ".ln2.bias", p + ".rosa.e", p + ".rosa.o.scale", p + ".rosa.o.bias",
                      p + ".ffn.x_k", p + ".ffn.key.scale", p + ".ffn.value"]
        return names

    def _sgd(self, name, gradient, lr):
        t = self.m.t
        t[name], self.residual[name] = clipped_sgd(t[name], self.residual[name], gradient, lr)

    def _flip(self, prefix, g_w, lr, ste_scale):
        """flip_after_gradients (src/model.rs:838-876): latent step, re-pack, count changed bits."""
        t = self.m.t
        g = (np.asarray(g_w, np.float32).ravel() * np.float32(ste_scale)).astype(np.float32)
        self.latent[prefix], self.residual[prefix + ".latent"] = binaryconnect_sgd(
            self.latent[prefix], self.residual[prefix + ".latent"], g, lr)
        before = t[prefix + ".bits"]
        after = pack_signs(self.latent[prefix], self._weights(prefix))
        t[prefix + ".bits"] = after
        return int(np.unpackbits((before ^ after).view(np.uint8)).sum())

    def train_step(self, tokens, labels, ignore_id, batch, time, lr):
        m, t = self.m, self.m.t
        d, ffn, vocab = m.d, m.ffn, m.vocab
        rows = batch * time
        lr = float(lr)
        if not np.isfinite(lr) or lr <= 0 or time < 2:
            raise ValueError("train step requires a positive learning rate and time >= 2")
        tokens = np.ascontiguousarray(tokens, np.uint32)
        labels = np.ascontiguousarray(labels, np.uint32)
        taps = {}
        mean, n_valid, row_loss, logits = m.forward_ce(tokens, labels, ignore_id, batch, time, taps, want_logits=True)
        hidden = taps["hidden"].reshape(rows, d)
        pre_ln_out = taps[f"{m.layers - 1}.block_out"]

        # ---- head (src/model.rs:3204-3257)
        logits = logits.reshape(rows, vocab)
        loss_scale = np.float32(0.0 if n_valid == 0 else 1.0 / (time - 1))
        r = np.arange(rows)
        valid = (r % time + 1 < time)
        nxt = np.minimum(r + 1, rows - 1)
        valid &= labels[nxt] != np.uint32(ignore_id)
        mx = logits.max(1, keepdims=True)
        ex = np.exp(logits - mx, dtype=np.float32)
        p = ex / ex.sum(1, dtype=np.float32, keepdims=True)
        onehot = np.zeros_like(p)
        onehot[r[valid], labels[nxt[valid]]] = 1
        gy = np.where(valid[:, None], loss_scale * (p - onehot), np.float32(0)).astype(np.float32)
        g_w, g_x, g_scale, g_bias = packed_backward_ste(hidden, gy, t["head.bits"], t["head.scale"], rows, d, vocab)
        ste = float(time - 1)
        flips_head = self._flip("head", g_w, lr, ste)
        self._sgd("head.scale", g_scale, lr)
        self._sgd("head.bias", g_bias, lr * HEAD_BIAS_LR_MULT)

        # ---- ln_out
        g_x, gw, gb = layer_norm_backward(pre_ln_out, g_x, t["ln_out.weight"], rows, d)
        self._sgd("ln_out.weight", gw, lr)
        self._sgd("ln_out.bias", gb, lr)

        flips_cmix = flips_o = 0
        for l in reversed(range(m.layers)):
            pre = f"blocks.{l}"
            # ---- CMix (src/model.rs:1138-1177)
            ln2_out = taps[f"{l}.ln2_out"]
            xx = O.time_shift_delta(ln2_out, batch, time, d)
            shifted = (ln2_out + xx * np.tile(O.fp16_to_f32(t[pre + ".ffn.x_k"]), rows)).astype(np.float32)
            key = O.binary_linear(shifted, t[pre + ".ffn.key.bits"], t[pre + ".ffn.key.scale"], None, rows, d, ffn)
            key = key.reshape(rows, ffn)
            relu2 = np.maximum(key, 0) ** 2
            gy2 = g_x.reshape(rows, d)
            wv = O.fp16_to_f32(t[pre + ".ffn.value"]).reshape(d, ffn)
            g_relu2 = gy2 @ wv
            g_value = gy2.T @ relu2
            self._sgd(pre + ".ffn.value", g_value.ravel(), lr)
            g_key = np.where(key > 0, 2 * key * g_relu2, np.float32(0)).astype(np.float32)
            g_wk, g_shifted, g_ks, _ = packed_backward_ste(shifted, g_key, t[pre + ".ffn.key.bits"],
                                                           t[pre + ".ffn.key.scale"], rows, d, ffn)
            flips_cmix += self._flip(pre + ".ffn.key", g_wk, lr, ste)
            self._sgd(pre + ".ffn.key.scale", g_ks, lr)
            g_ln2_out, g_mix = lerp_shift_backward(xx, t[pre + ".ffn.x_k"], g_shifted, batch, time, d)
            self._sgd(pre + ".ffn.x_k", g_mix, lr)
            g_in, gw, gb = layer_norm_backward(taps[f"{l}.after_rosa"], g_ln2_out, t[pre + ".ln2.weight"], rows, d)
            self._sgd(pre + ".ln2.weight", gw, lr)
            self._sgd(pre + ".ln2.bias", gb, lr)
            g_x = (g_x + g_in).astype(np.float32)

            # ---- ROSA, gradients stop at the q/k/v bits (src/model.rs:1494-1521, 1608-1634)
            y = taps[f"{l}.y"]
            g_wo, g_y, g_os, g_ob = packed_backward_ste(y, g_x, t[pre + ".rosa.o.bits"], t[pre + ".rosa.o.scale"],
                                                        rows, d, d)
            flips_o += self._flip(pre + ".rosa.o", g_wo, lr, ste)
            self._sgd(pre + ".rosa.o.scale", g_os, lr)
            self._sgd(pre + ".rosa.o.bias", g_ob, lr)
            sign = taps[f"{l}.idx"].reshape(rows, d).astype(np.float32) * 2 - 1
            self._sgd(pre + ".rosa.e", (g_y * sign).sum(0, dtype=np.float32), lr)
        # ---- ln0 of layer 0 and the embedding rows (src/model.rs:2972-2990)
        return self._finish(tokens, g_x, mean, n_valid, flips_head, flips_cmix, flips_o, batch, time, lr)

    def _finish(self, tokens, g_x, mean, n_valid, flips_head, flips_cmix, flips_o, batch, time, lr):
        m, t = self.m, self.m.t
        d, rows = m.d, batch * time
        ln0_in = O.embed(tokens, t["embedding"], d, m.vocab)
        g_x, gw, gb = layer_norm_backward(ln0_in, g_x, t["blocks.0.ln0.weight"], rows, d)
        self._sgd("blocks.0.ln0.weight", gw, lr)
        self._sgd("blocks.0.ln0.bias", gb, lr)
        # one clipped step per ROW, in row order: a token that occurs twice is stepped twice
        emb = t["embedding"].reshape(m.vocab, d)
        res = self.residual["embedding"].reshape(m.vocab, d)
        g = g_x.reshape(rows, d)
        for row, tok in enumerate(tokens):
            emb[tok], res[tok] = clipped_sgd(emb[tok], res[tok], g[row], lr)
        t["embedding"] = emb.reshape(-1)
        self.residual["embedding"] = res.reshape(-1)
        return {"loss": mean, "n_valid": n_valid, "flips_head": flips_head, "flips_cmix": flips_cmix,
                "flips_rosa_o": flips_o, "embed_grad": g_x}

    def install_head_unigram_prior(self, labels, ignore_id):
        """install_head_unigram_prior + shrink_head_kaiming_scale (src/model.rs:3034-3110)."""
        m, t = self.m, self.m.t
        vocab = m.vocab
        bias = O.fp16_to_f32(t["head.bias"])
        rms = lambda bits: float(np.sqrt((O.fp16_to_f32(bits) ** 2).sum(dtype=np.float32) / np.float32(bits.size)))
        if float(np.abs(bias).sum(dtype=np.float32) / np.float32(vocab)) > 0.05:   # HEAD_BIAS_PRIOR_ABS_EPS
            return {"applied": False, "n_targets": 0, "bias_rms": rms(t["head.bias"]), "scale_rms": rms(t["head.scale"]),
                    "shrunk_kaiming_scale": False}
        labels = np.asarray(labels, np.uint32)
        keep = labels[(labels != np.uint32(ignore_id)) & (labels < vocab)]
        if keep.size == 0:
            raise ValueError("head unigram prior needs at least one supervised label")
        counts = np.bincount(keep, minlength=vocab).astype(np.float32)
        logs = (np.log1p(counts, dtype=np.float32) - np.log(np.float32(keep.size) + np.float32(vocab), dtype=np.float32))
        log_sum = np.float32(0)
        for v in logs.astype(np.float32):      # sequential f32 sum, as the reference
            log_sum = np.float32(log_sum + v)
        t["head.bias"] = O.fp16_from_f32((logs - log_sum / np.float32(vocab)).astype(np.float32))
        self.residual["head.bias"][:] = 0      # Fp16Storage::set clears the carry (src/precision.rs:208-211)
        scale = O.fp16_to_f32(t["head.scale"])
        mean = np.float32(0)
        for v in scale:
            mean = np.float32(mean + v)
        mean = mean / np.float32(vocab)
        kaiming = np.float32(1.0) / np.sqrt(np.float32(m.d))
        shrunk = bool(kaiming * np.float32(0.5) < mean < kaiming * np.float32(2.0))
        if shrunk:
            t["head.scale"] = O.fp16_from_f32((scale * np.float32(0.25)).astype(np.float32))   # HEAD_KAIMING_SCALE_SHRINK
            self.residual["head.scale"][:] = 0
        return {"applied": True, "n_targets": int(keep.size), "bias_rms": rms(t["head.bias"]),
                "scale_rms": rms(t["head.scale"]), "shrunk_kaiming_scale": shrunk}
