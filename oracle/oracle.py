"""ctypes binding of the CPU oracle (oracle/ullis_oracle.c) plus the Heron
forward orchestration.  TEST INFRASTRUCTURE ONLY: imported by tests/, by the
smoke check and by the CPU-baseline / reference legs of bench.py; never by the
CUDA product path.

Orchestration follows the reference's forward-only route
(src/model.rs:2644-2688 hidden/logits, 2224-2241 HeronBlock::forward) and the
CE forward inside apply_head_ce (src/model.rs:3205-3228, 3253-3257).
"""
from __future__ import annotations

import ctypes as C
import json
import os
import struct

import numpy as np

from . import build as _build

_LIB = None


def lib() -> C.CDLL:
    global _LIB
    if _LIB is None:
        path = _build.OUT
        if not os.path.exists(path):
            path = _build.build()
        _LIB = C.CDLL(path)
        _LIB.uo_fp16_from_f32.restype = C.c_uint16
        _LIB.uo_fp16_from_f32.argtypes = [C.c_float]
        _LIB.uo_fp16_to_f32.restype = C.c_float
        _LIB.uo_fp16_to_f32.argtypes = [C.c_uint16]
        _LIB.uo_sam_new.restype = C.c_void_p
        _LIB.uo_sam_new.argtypes = [C.c_size_t]
        _LIB.uo_sam_push.restype = C.c_uint8
        _LIB.uo_sam_push.argtypes = [C.c_void_p, C.c_uint8, C.c_uint8, C.c_uint8]
        _LIB.uo_sam_reset.argtypes = [C.c_void_p]
        _LIB.uo_sam_free.argtypes = [C.c_void_p]
        _LIB.uo_sam_walk_steps.restype = C.c_uint64
        _LIB.uo_sam_walk_steps.argtypes = [C.c_void_p]
    return _LIB


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _u16(a):
    return np.ascontiguousarray(a, dtype=np.uint16)


def _u32(a):
    return np.ascontiguousarray(a, dtype=np.uint32)


def _u8(a):
    return np.ascontiguousarray(a, dtype=np.uint8)


def set_threads(n: int) -> None:
    lib().uo_set_threads(C.c_int(int(n)))


def max_threads() -> int:
    return int(lib().uo_max_threads())


# ------------------------------------------------------------------ fp16

def fp16_from_f32(x) -> np.ndarray:
    x = _f32(x)
    out = np.empty(x.shape, np.uint16)
    lib().uo_fp16_from_f32_n(_p(x), _p(out), C.c_size_t(x.size))
    return out


def fp16_to_f32(h) -> np.ndarray:
    h = _u16(h)
    out = np.empty(h.shape, np.float32)
    lib().uo_fp16_to_f32_n(_p(h), _p(out), C.c_size_t(h.size))
    return out


# ------------------------------------------------------------------- ops

def layer_norm(x, w_bits, b_bits, rows, channels) -> np.ndarray:
    x = _f32(x)
    y = np.empty(rows * channels, np.float32)
    rc = lib().uo_layer_norm(_p(x), _p(_u16(w_bits)), _p(_u16(b_bits)), _p(y),
                             C.c_size_t(rows), C.c_size_t(channels))
    if rc:
        raise ValueError("LayerNorm input shape mismatch")
    return y


def time_shift_delta(x, batch, time, channels) -> np.ndarray:
    x = _f32(x)
    xx = np.empty_like(x)
    if lib().uo_time_shift_delta(_p(x), _p(xx), C.c_size_t(batch), C.c_size_t(time), C.c_size_t(channels)):
        raise ValueError("time-shift input shape mismatch")
    return xx


def binary_linear(x, bits, scale_bits, bias_bits, rows, in_features, out_features, scalar=False) -> np.ndarray:
    x = _f32(x)
    bits = _u32(bits)
    if x.size != rows * in_features or bits.size != (in_features * out_features + 31) // 32:
        raise ValueError("packed linear input shape mismatch")
    y = np.empty(rows * out_features, np.float32)
    fn = lib().uo_binary_linear_scalar if scalar else lib().uo_binary_linear
    bias = None if bias_bits is None else _u16(bias_bits)
    fn(_p(x), _p(bits), _p(_u16(scale_bits)), _p(bias), _p(y),
       C.c_size_t(rows), C.c_size_t(in_features), C.c_size_t(out_features))
    return y


def fp16_linear(x, w_bits, rows, in_features, out_features, scalar=False) -> np.ndarray:
    x = _f32(x)
    w_bits = _u16(w_bits)
    if x.size != rows * in_features or w_bits.size != in_features * out_features:
        raise ValueError("FP16 linear input shape mismatch")
    y = np.empty(rows * out_features, np.float32)
    fn = lib().uo_fp16_linear_scalar if scalar else lib().uo_fp16_linear
    fn(_p(x), _p(w_bits), _p(y), C.c_size_t(rows), C.c_size_t(in_features), C.c_size_t(out_features))
    return y


def bits_from_activation(x) -> np.ndarray:
    x = _f32(x)
    out = np.empty(x.size, np.uint8)
    lib().uo_bits_from_activation(_p(x), _p(out), C.c_size_t(x.size))
    return out


def pack_bitplane(bits) -> np.ndarray:
    bits = _u8(bits)
    if bits.size and bits.max() > 1:
        raise ValueError("pack_bitplane bits must be 0 or 1")
    words = np.empty((bits.size + 31) // 32, np.uint32)
    lib().uo_pack_bitplane(_p(bits), _p(words), C.c_size_t(bits.size))
    return words


def sign_pack_bits(x) -> np.ndarray:
    x = _f32(x)
    words = np.empty((x.size + 31) // 32, np.uint32)
    lib().uo_sign_pack_bits(_p(x), _p(words), C.c_size_t(x.size))
    return words


class RosaSam:
    """src/rosa.rs:15-177 RosaSam (with_max_time / push / reset)."""

    def __init__(self, max_time: int):
        self._h = lib().uo_sam_new(C.c_size_t(max_time))

    def push(self, q: int, k: int, v: int) -> int:
        return int(lib().uo_sam_push(self._h, q, k, v))

    def reset(self) -> None:
        lib().uo_sam_reset(self._h)

    def walk_steps(self) -> int:
        return int(lib().uo_sam_walk_steps(self._h))

    def __del__(self):
        if getattr(self, "_h", None):
            lib().uo_sam_free(self._h)
            self._h = None


def rosa_qkv_ref(q, k, v) -> np.ndarray:
    q, k, v = _u8(q), _u8(k), _u8(v)
    if not (q.size == k.size == v.size):
        raise ValueError("rosa_qkv_ref requires q, k, v of equal length")
    idx = np.empty(q.size, np.uint8)
    if lib().uo_rosa_qkv_ref(_p(q), _p(k), _p(v), C.c_size_t(q.size), _p(idx)):
        raise ValueError("rosa_qkv_ref bits must be 0 or 1")
    return idx


def rosa(bits) -> np.ndarray:
    bits = _u8(bits)
    y = np.empty(bits.size, np.int32)
    if lib().uo_rosa(_p(bits), C.c_size_t(bits.size), _p(y)):
        raise ValueError("rosa bits must be 0 or 1")
    return y


def rosa_qkv_batch(q, k, v, batch, time, channels) -> np.ndarray:
    q, k, v = _u8(q), _u8(k), _u8(v)
    n = batch * time * channels
    if q.size != n or k.size != n or v.size != n:
        raise ValueError("rosa_qkv_batch requires q, k, v of length batch*time*channels")
    idx = np.empty(n, np.uint8)
    if lib().uo_rosa_qkv_batch(_p(q), _p(k), _p(v), C.c_size_t(batch), C.c_size_t(time),
                               C.c_size_t(channels), _p(idx)):
        raise ValueError("rosa_qkv_batch dimensions must be non-zero and bits 0/1")
    return idx


def rosa_qkv_batch_packed(q_bits, k_bits, v_bits, batch, time, channels, return_walks=False):
    q_bits, k_bits, v_bits = _u32(q_bits), _u32(k_bits), _u32(v_bits)
    n = batch * time * channels
    words = (n + 31) // 32
    if q_bits.size != words or k_bits.size != words or v_bits.size != words:
        raise ValueError("rosa_qkv_batch_packed word count mismatch")
    idx = np.empty(n, np.uint8)
    walks = C.c_uint64(0)
    if lib().uo_rosa_qkv_batch_packed(_p(q_bits), _p(k_bits), _p(v_bits), C.c_size_t(batch),
                                      C.c_size_t(time), C.c_size_t(channels), _p(idx), C.byref(walks)):
        raise ValueError("rosa_qkv_batch_packed dimensions must be non-zero")
    return (idx, int(walks.value)) if return_walks else idx


def rosa_qkv_streams(qw, kw, vw, n_streams, time, return_walks=False):
    """Stream-major packed driver: arrays are [n_streams, ceil(time/32)] u32."""
    qw, kw, vw = _u32(qw), _u32(kw), _u32(vw)
    wps = (time + 31) // 32
    if qw.size != n_streams * wps or kw.size != qw.size or vw.size != qw.size:
        raise ValueError("rosa_qkv_streams word count mismatch")
    out = np.empty(n_streams * wps, np.uint32)
    walks = C.c_uint64(0)
    lib().uo_rosa_qkv_streams(_p(qw), _p(kw), _p(vw), C.c_size_t(n_streams), C.c_size_t(time),
                              C.c_size_t(wps), _p(out), C.byref(walks))
    out = out.reshape(n_streams, wps)
    return (out, int(walks.value)) if return_walks else out


def rosa_qkv_out_batched(idx, e_bits, batch, time, channels) -> np.ndarray:
    idx = _u8(idx)
    e_bits = _u16(e_bits)
    if idx.size != batch * time * channels or e_bits.size != channels:
        raise ValueError("rosa_qkv_out_batched shape mismatch")
    out = np.empty(idx.size, np.float32)
    lib().uo_rosa_qkv_out_batched(_p(idx), _p(e_bits), _p(out), C.c_size_t(batch), C.c_size_t(time),
                                  C.c_size_t(channels))
    return out


def rosa_block_forward(x, p: dict, batch, time, channels, taps: bool = False):
    """p holds x_q,x_k,x_v,e (u16) and q/k/v/o dicts with bits,scale,bias."""
    x = _f32(x)
    n = batch * time * channels
    out = np.empty(n, np.float32)
    t = {}
    if taps:
        for name in ("q", "k", "v", "y"):
            t[name] = np.empty(n, np.float32)
        for name in ("q_bits", "k_bits", "v_bits", "idx"):
            t[name] = np.empty(n, np.uint8)
    walks = C.c_uint64(0)
    g = lambda name: _p(t[name]) if taps else None
    arrs = [_u16(p["x_q"]), _u16(p["x_k"]), _u16(p["x_v"])]
    lin = []
    for m in ("q", "k", "v"):
        lin += [_u32(p[m]["bits"]), _u16(p[m]["scale"]), _u16(p[m]["bias"])]
    e = _u16(p["e"])
    o = [_u32(p["o"]["bits"]), _u16(p["o"]["scale"]), _u16(p["o"]["bias"])]
    lib().uo_rosa_block_forward(
        _p(x), *[_p(a) for a in arrs], *[_p(a) for a in lin], _p(e), *[_p(a) for a in o],
        C.c_size_t(batch), C.c_size_t(time), C.c_size_t(channels),
        g("q"), g("k"), g("v"), g("q_bits"), g("k_bits"), g("v_bits"), g("idx"), g("y"), _p(out),
        C.byref(walks))
    t["walk_steps"] = int(walks.value)
    return (out, t) if taps else out


def cmix_forward(x, mix, key_bits, key_scale, value_bits, batch, time, d_model, dim_ffn, tap=False):
    x = _f32(x)
    rows = batch * time
    out = np.empty(rows * d_model, np.float32)
    relu2 = np.empty(rows * dim_ffn, np.float32) if tap else None
    lib().uo_cmix_forward(_p(x), _p(_u16(mix)), _p(_u32(key_bits)), _p(_u16(key_scale)), _p(_u16(value_bits)),
                          C.c_size_t(batch), C.c_size_t(time), C.c_size_t(d_model), C.c_size_t(dim_ffn),
                          _p(relu2), _p(out))
    return (out, relu2) if tap else out


def embed(ids, embedding_bits, d_model, vocab) -> np.ndarray:
    ids = _u32(ids)
    x = np.empty(ids.size * d_model, np.float32)
    if lib().uo_embed(_p(ids), _p(_u16(embedding_bits)), _p(x), C.c_size_t(ids.size), C.c_size_t(d_model),
                      C.c_size_t(vocab)):
        raise ValueError("token id exceeds vocabulary")
    return x


CE_NO_IGNORE = 0xFFFFFFFF  # src/model.rs:24


def head_ce(hidden, head_bits, head_scale, head_bias, targets, ignore_id, rows, time, d_model, vocab,
            want_logits=False):
    hidden = _f32(hidden)
    targets = _u32(targets)
    row_loss = np.empty(rows, np.float32)
    mean = C.c_float(0)
    n_valid = C.c_uint64(0)
    logits = np.empty(rows * vocab, np.float32) if want_logits else None
    bias = None if head_bias is None else _u16(head_bias)
    rc = lib().uo_head_ce(_p(hidden), _p(_u32(head_bits)), _p(_u16(head_scale)), _p(bias), _p(targets),
                          C.c_uint32(ignore_id), C.c_size_t(rows), C.c_size_t(time), C.c_size_t(d_model),
                          C.c_size_t(vocab), _p(row_loss), C.byref(mean), C.byref(n_valid), _p(logits))
    if rc:
        raise ValueError("target id exceeds vocabulary")
    return float(mean.value), int(n_valid.value), row_loss, logits


# --------------------------------------------------------------- model

def read_safetensors(data: bytes):
    """Minimal reader of the container (8-byte LE header length, JSON header,
    raw little-endian tensor data) used to load v2 checkpoints into numpy."""
    (hlen,) = struct.unpack("<Q", data[:8])
    header = json.loads(data[8:8 + hlen])
    meta = header.pop("__metadata__", None)
    base = 8 + hlen
    dt = {"F16": np.uint16, "U32": np.uint32, "F32": np.float32}
    tensors = {}
    for name, info in header.items():
        b, e = info["data_offsets"]
        tensors[name] = np.frombuffer(data[base + b:base + e], dtype=dt[info["dtype"]]).copy()
    return tensors, meta


class HeronOracle:
    """CPU Heron model over a v2 checkpoint (tensor names of
    src/model.rs:3428-3441 and 3900-3932)."""

    def __init__(self, data: bytes):
        self.t, meta = read_safetensors(data)
        if not meta or meta.get("format_version") != "2":
            raise ValueError("Hyena checkpoints (v1) are intentionally unloadable")
        self.cfg = json.loads(meta["config"])
        self.d = self.cfg["d_model"]
        self.vocab = self.cfg["vocab_size"]
        self.ffn = self.cfg.get("dim_ffn", 0) or 4 * self.d
        self.layers = self.cfg["n_layers"]

    def _packed(self, prefix):
        t = self.t
        return {"bits": t[prefix + ".bits"], "scale": t[prefix + ".scale"], "bias": t.get(prefix + ".bias")}

    def hidden(self, ids, batch, time, taps=None):
        """src/model.rs:2644-2683.  taps: optional dict filled with per-layer
        arrays keyed '<layer>.<name>'."""
        t, d = self.t, self.d
        rows = batch * time
        ids = np.ascontiguousarray(ids, np.uint32)
        if batch == 0 or time == 0 or ids.size != rows or batch > self.cfg["batch_size"] \
                or time > self.cfg["context_len"]:
            raise ValueError("token shape or context length is invalid")
        x = embed(ids, t["embedding"], d, self.vocab)
        for l in range(self.layers):
            pre = f"blocks.{l}"
            if l == 0:
                x = layer_norm(x, t[pre + ".ln0.weight"], t[pre + ".ln0.bias"], rows, d)
            if taps is not None:
                taps[f"{l}.block_in"] = x.copy()
            rosa_in = layer_norm(x, t[pre + ".ln3.weight"], t[pre + ".ln3.bias"], rows, d)
            rp = {"x_q": t[pre + ".rosa.x_q"], "x_k": t[pre + ".rosa.x_k"], "x_v": t[pre + ".rosa.x_v"],
                  "e": t[pre + ".rosa.e"]}
            for m in "qkvo":
                rp[m] = self._packed(f"{pre}.rosa.{m}")
            if taps is not None:
                rosa_out, rt = rosa_block_forward(rosa_in, rp, batch, time, d, taps=True)
                taps[f"{l}.ln3_out"] = rosa_in
                for k_, v_ in rt.items():
                    taps[f"{l}.{k_}"] = v_
                taps[f"{l}.rosa_out"] = rosa_out
            else:
                rosa_out = rosa_block_forward(rosa_in, rp, batch, time, d)
            x = x + rosa_out  # f32 elementwise add, src/model.rs:2232-2234
            if taps is not None:
                taps[f"{l}.after_rosa"] = x.copy()
            ffn_in = layer_norm(x, t[pre + ".ln2.weight"], t[pre + ".ln2.bias"], rows, d)
            ffn_out = cmix_forward(ffn_in, t[pre + ".ffn.x_k"], t[pre + ".ffn.key.bits"],
                                   t[pre + ".ffn.key.scale"], t[pre + ".ffn.value"], batch, time, d, self.ffn)
            if taps is not None:
                taps[f"{l}.ln2_out"] = ffn_in
                taps[f"{l}.cmix_out"] = ffn_out
            x = x + ffn_out
            if taps is not None:
                taps[f"{l}.block_out"] = x.copy()
        return layer_norm(x, t["ln_out.weight"], t["ln_out.bias"], rows, d)

    def _head_bias(self):
        b = self.t.get("head.bias")  # absent => zero bias, src/model.rs:4237-4246
        return b if b is not None else np.zeros(self.vocab, np.uint16)

    def logits(self, ids, batch, time):
        h = self.hidden(ids, batch, time)
        return binary_linear(h, self.t["head.bits"], self.t["head.scale"], self._head_bias(),
                             batch * time, self.d, self.vocab)

    def forward_ce(self, ids, labels, ignore_id, batch, time, taps=None, want_logits=False):
        h = self.hidden(ids, batch, time, taps)
        mean, n_valid, row_loss, logits = head_ce(h, self.t["head.bits"], self.t["head.scale"],
                                                  self._head_bias(), labels, ignore_id, batch * time, time,
                                                  self.d, self.vocab, want_logits)
        if taps is not None:
            taps["hidden"] = h
        return mean, n_valid, row_loss, logits

    # ---- incremental generation (src/model.rs:2433-2454, 2691-2753)
    def generate_state(self):
        """Empty automata (one per layer and channel), no time-shift history."""
        T = self.cfg["context_len"]
        return {"time": 0,
                "layers": [{"sams": [RosaSam(T) for _ in range(self.d)], "rosa_x_prev": None, "cmix_x_prev": None}
                           for _ in range(self.layers)]}

    @staticmethod
    def _shift_one(x, prev):
        """time_shift_one, src/model.rs:214-228."""
        return -x if prev is None else (prev - x).astype(np.float32)

    def generate_step(self, state, token: int) -> np.ndarray:
        """One token -> last-token logits [vocab]; HeronBlock::forward_one src/model.rs:2243-2262,
        ROSA forward_one 1320-1352, CMix forward_one 1003-1016."""
        t, d = self.t, self.d
        if token >= self.vocab:
            raise ValueError("token id exceeds vocabulary")
        if state["time"] >= self.cfg["context_len"]:
            raise ValueError(f"generate exceeded context_len ({self.cfg['context_len']})")
        x = embed(np.array([token], np.uint32), t["embedding"], d, self.vocab)
        for l, layer in enumerate(state["layers"]):
            pre = f"blocks.{l}"
            if l == 0:
                x = layer_norm(x, t[pre + ".ln0.weight"], t[pre + ".ln0.bias"], 1, d)
            rosa_in = layer_norm(x, t[pre + ".ln3.weight"], t[pre + ".ln3.bias"], 1, d)
            xx = self._shift_one(rosa_in, layer["rosa_x_prev"])
            acts = []
            for m in "qkv":
                mix = fp16_to_f32(t[f"{pre}.rosa.x_{m}"])
                inp = (rosa_in + (xx * mix).astype(np.float32)).astype(np.float32)  # multiply, then add
                w = self._packed(f"{pre}.rosa.{m}")
                acts.append(binary_linear(inp, w["bits"], w["scale"], w["bias"], 1, d, d))
            e = fp16_to_f32(t[pre + ".rosa.e"])
            y = np.empty(d, np.float32)
            for c, sam in enumerate(layer["sams"]):
                idx = sam.push(int(acts[0][c] > 0), int(acts[1][c] > 0), int(acts[2][c] > 0))
                y[c] = np.float32(2.0 * idx - 1.0) * e[c]
            o = self._packed(f"{pre}.rosa.o")
            rosa_out = binary_linear(y, o["bits"], o["scale"], o["bias"], 1, d, d)
            layer["rosa_x_prev"] = rosa_in
            x = (x + rosa_out).astype(np.float32)
            ffn_in = layer_norm(x, t[pre + ".ln2.weight"], t[pre + ".ln2.bias"], 1, d)
            xx = self._shift_one(ffn_in, layer["cmix_x_prev"])
            shifted = (ffn_in + (xx * fp16_to_f32(t[pre + ".ffn.x_k"])).astype(np.float32)).astype(np.float32)
            key = binary_linear(shifted, t[pre + ".ffn.key.bits"], t[pre + ".ffn.key.scale"], None, 1, d, self.ffn)
            pos = np.maximum(key, np.float32(0.0))
            relu2 = (pos * pos).astype(np.float32)
            ffn_out = fp16_linear(relu2, t[pre + ".ffn.value"], 1, self.ffn, d)
            layer["cmix_x_prev"] = ffn_in
            x = (x + ffn_out).astype(np.float32)
        hidden = layer_norm(x, t["ln_out.weight"], t["ln_out.bias"], 1, d)
        state["time"] += 1
        return binary_linear(hidden, t["head.bits"], t["head.scale"], self._head_bias(), 1, d, self.vocab)
