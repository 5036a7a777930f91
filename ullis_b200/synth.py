"""Seeded synthetic weights and inputs for the Heron forward path.

No dataset is involved: every tensor and token stream is drawn from one PRNG
(splitmix64 as in the reference's src/model.rs:134-140) with one sub-seed per
tensor name, and weights are written as a v2 `checkpoint.safetensors` so the
CUDA backend and the CPU oracle load the same bytes through their own loaders.

Distributions follow the benchmark configurations: packed +/-1 weight bits
Bernoulli(0.5); FP16 row scales U[0.005, 0.02]; biases N(0, 0.01); embeddings,
LayerNorm weight and bias, and ROSA `e` N(0, 0.02); time-shift mixes U[0, 1);
CMix value Kaiming-uniform +/- 1/sqrt(dim_ffn) (src/model.rs:473-488).
`ln_gain_one=True` is the secondary variant with LayerNorm weight 1 + N(0, 0.02).
"""
from __future__ import annotations

import json

import numpy as np

from . import checkpoint as ckpt

_GOLDEN = np.uint64(0x9E3779B97F4A7C15)
_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)


def splitmix64_stream(seed: int, n: int) -> np.ndarray:
    """First n outputs of splitmix64 started from `seed` (state += golden, mix)."""
    with np.errstate(over="ignore"):
        state = np.uint64(seed & 0xFFFFFFFFFFFFFFFF) + _GOLDEN * np.arange(1, n + 1, dtype=np.uint64)
        z = state
        z = (z ^ (z >> np.uint64(30))) * _M1
        z = (z ^ (z >> np.uint64(27))) * _M2
        return z ^ (z >> np.uint64(31))


def _fnv1a64(name: str) -> int:
    h = 0xCBF29CE484222325
    for b in name.encode():
        h = ((h ^ b) * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    return h


def sub_seed(seed: int, name: str) -> int:
    return (_fnv1a64(name) ^ (seed * 0x9E3779B97F4A7C15)) & 0xFFFFFFFFFFFFFFFF


def uniform(seed: int, n: int) -> np.ndarray:
    """u = (w >> 11) / 2^53 in [0, 1), float64."""
    return (splitmix64_stream(seed, n) >> np.uint64(11)).astype(np.float64) / float(1 << 53)


def normal(seed: int, n: int) -> np.ndarray:
    """Box-Muller on consecutive uniform pairs, float64."""
    m = (n + 1) // 2
    u = uniform(seed, 2 * m)
    u1 = 1.0 - u[0::2]  # (0, 1]
    u2 = u[1::2]
    r = np.sqrt(-2.0 * np.log(u1))
    z = np.empty(2 * m)
    z[0::2] = r * np.cos(2 * np.pi * u2)
    z[1::2] = r * np.sin(2 * np.pi * u2)
    return z[:n]


def bernoulli_words(seed: int, n_bits: int) -> np.ndarray:
    """Bernoulli(0.5) bits packed LSB-first, 32 per u32 word; tail bits zero."""
    words = (n_bits + 31) // 32
    w = (splitmix64_stream(seed, words) >> np.uint64(32)).astype(np.uint32)
    tail = n_bits % 32
    if tail:
        w[-1] &= np.uint32((1 << tail) - 1)
    return w


def f16_bits(x) -> np.ndarray:
    """IEEE binary16 bit patterns, round to nearest even (numpy's float16 cast
    implements the same rounding as the reference's Fp16::from_f32)."""
    return np.asarray(x, np.float32).astype(np.float16).view(np.uint16)


def train_config(d_model: int, n_layers: int, vocab: int, context_len: int, batch_size: int, dim_ffn: int,
                 seed: int = 7, memory_budget_bytes: int = 4 << 30) -> dict:
    """JSON body of the reference's TrainConfig (src/config.rs:77-100)."""
    return {
        "architecture": "heron", "d_model": d_model, "n_layers": n_layers, "vocab_size": vocab,
        "context_len": context_len, "batch_size": batch_size, "dim_ffn": dim_ffn, "rosa_bits": 1,
        "rosa_grad": "stop_grad_bits", "head_size": 16, "tmix_lora_rank": 16, "seed": seed,
        "memory_budget_bytes": memory_budget_bytes,
    }


CONFIGS = {
    # name: (d_model, n_layers, vocab, context_len, dim_ffn)
    "tiny": (64, 2, 512, 64, 128),
    "small": (256, 6, 8192, 512, 1024),      # reference default, CPU-runnable
    "default": (512, 12, 8192, 2048, 2048),  # train_config.json shape
}


def heron_tensors(cfg: dict, seed: int = 7, ln_gain_one: bool = False, head_bias: bool = True) -> dict:
    """All forward tensors of a Heron checkpoint, keyed by the v2 tensor names
    (src/model.rs:3428-3441, 3900-3932), as flat numpy arrays (u16 = FP16 bits)."""
    d, v, layers = cfg["d_model"], cfg["vocab_size"], cfg["n_layers"]
    f = cfg["dim_ffn"] or 4 * d
    t: dict[str, np.ndarray] = {}

    def n02(name, n):
        return f16_bits(0.02 * normal(sub_seed(seed, name), n))

    def ln(prefix):
        w = 0.02 * normal(sub_seed(seed, prefix + ".weight"), d)
        t[prefix + ".weight"] = f16_bits(1.0 + w if ln_gain_one else w)
        t[prefix + ".bias"] = n02(prefix + ".bias", d)

    def packed(prefix, out, inn, bias):
        t[prefix + ".bits"] = bernoulli_words(sub_seed(seed, prefix + ".bits"), out * inn)
        t[prefix + ".scale"] = f16_bits(0.005 + 0.015 * uniform(sub_seed(seed, prefix + ".scale"), out))
        if bias:
            t[prefix + ".bias"] = f16_bits(0.01 * normal(sub_seed(seed, prefix + ".bias"), out))

    t["embedding"] = n02("embedding", v * d)
    ln("ln_out")
    packed("head", v, d, head_bias)
    for i in range(layers):
        pre = f"blocks.{i}"
        if i == 0:
            ln(pre + ".ln0")
        ln(pre + ".ln2")
        ln(pre + ".ln3")
        for m in ("x_q", "x_k", "x_v"):
            t[f"{pre}.rosa.{m}"] = f16_bits(uniform(sub_seed(seed, f"{pre}.rosa.{m}"), d))
        t[f"{pre}.rosa.e"] = n02(f"{pre}.rosa.e", d)
        for m in "qkvo":
            packed(f"{pre}.rosa.{m}", d, d, True)
        t[f"{pre}.ffn.x_k"] = f16_bits(uniform(sub_seed(seed, f"{pre}.ffn.x_k"), d))
        packed(f"{pre}.ffn.key", f, d, False)
        bound = 1.0 / np.sqrt(float(f))
        t[f"{pre}.ffn.value"] = f16_bits((2.0 * uniform(sub_seed(seed, f"{pre}.ffn.value"), d * f) - 1.0) * bound)
    return t


def heron_checkpoint(name_or_shape="small", batch_size: int = 1, seed: int = 7, ln_gain_one: bool = False,
                     head_bias: bool = True, context_len: int | None = None) -> bytes:
    """Bytes of a v2 checkpoint.safetensors for one of CONFIGS (or a
    (d_model, n_layers, vocab, context_len, dim_ffn) tuple)."""
    shape = CONFIGS[name_or_shape] if isinstance(name_or_shape, str) else tuple(name_or_shape)
    d, layers, vocab, ctx, f = shape
    if context_len is not None:
        ctx = context_len
    cfg = train_config(d, layers, vocab, ctx, batch_size, f, seed, memory_budget_bytes=64 << 30)
    tensors = heron_tensors(cfg, seed, ln_gain_one, head_bias)
    return ckpt.to_safetensors_bytes(tensors, cfg, step=0)


def uniform_tokens(seed: int, n: int, vocab: int) -> np.ndarray:
    return (uniform(sub_seed(seed, "tokens.uniform"), n) * vocab).astype(np.uint32)


def zipf_tokens(seed: int, n: int, vocab: int, exponent: float = 1.1) -> np.ndarray:
    """ids = rank-1 with p(rank) ~ rank^-exponent over ranks 1..vocab
    (float64 inverse-CDF table)."""
    p = np.arange(1, vocab + 1, dtype=np.float64) ** (-exponent)
    cdf = np.cumsum(p / p.sum())
    u = uniform(sub_seed(seed, "tokens.zipf"), n)
    return np.minimum(np.searchsorted(cdf, u, side="right"), vocab - 1).astype(np.uint32)


# ------------------------------------------------ standalone op inputs

def packed_linear_case(seed: int, rows: int, inn: int, out: int, bias: bool = True):
    """Microbenchmark operands: FP16 N(0,1) activations (returned as the f32
    widening of their FP16 values), Bernoulli(0.5) bits, scale U[0.005,0.02],
    bias N(0,0.01)."""
    x = f16_bits(normal(sub_seed(seed, "pl.x"), rows * inn)).view(np.float16).astype(np.float32)
    bits = bernoulli_words(sub_seed(seed, "pl.bits"), out * inn)
    scale = f16_bits(0.005 + 0.015 * uniform(sub_seed(seed, "pl.scale"), out))
    b = f16_bits(0.01 * normal(sub_seed(seed, "pl.bias"), out)) if bias else None
    return x, bits, scale, b


def rosa_bits_iid(seed: int, batch: int, time: int, channels: int):
    """Variant (a): i.i.d. Bernoulli(0.5) q/k/v bit planes packed over [B,T,C]."""
    n = batch * time * channels
    return tuple(bernoulli_words(sub_seed(seed, f"rosa.iid.{m}"), n) for m in "qkv")


def rosa_bits_periodic(seed: int, batch: int, time: int, channels: int, pmin: int = 16, pmax: int = 256,
                       flip: float = 0.10):
    """Variant (b): per (b,c) stream a random period P in [pmin,pmax] and a
    random P-bit base pattern repeated to T; q and k share the base pattern
    with independent `flip` noise, v has its own periodic pattern with noise.
    Returns packed [B,T,C] bit planes."""
    streams = batch * channels
    period = pmin + (uniform(sub_seed(seed, "rosa.per.P"), streams) * (pmax - pmin + 1)).astype(np.int64)
    tt = np.arange(time, dtype=np.int64)[None, :]                      # [1,T]
    phase = tt % period[:, None]                                       # [S,T]
    out = []
    base_qk = (splitmix64_stream(sub_seed(seed, "rosa.per.base.qk"), streams * pmax) & np.uint64(1)) \
        .astype(np.uint8).reshape(streams, pmax)
    base_v = (splitmix64_stream(sub_seed(seed, "rosa.per.base.v"), streams * pmax) & np.uint64(1)) \
        .astype(np.uint8).reshape(streams, pmax)
    for m, base in (("q", base_qk), ("k", base_qk), ("v", base_v)):
        bits = np.take_along_axis(base, phase, axis=1)                 # [S,T]
        noise = uniform(sub_seed(seed, f"rosa.per.flip.{m}"), streams * time).reshape(streams, time) < flip
        bits = bits ^ noise.astype(np.uint8)
        # [S=B*C, T] -> [B,T,C]
        btc = bits.reshape(batch, channels, time).transpose(0, 2, 1).reshape(-1)
        out.append(np.packbits(btc, bitorder="little").view(np.uint32) if btc.size % 32 == 0
                   else _pack_tail(btc))
    return tuple(out)


def _pack_tail(bits: np.ndarray) -> np.ndarray:
    pad = (-bits.size) % 32
    return np.packbits(np.concatenate([bits, np.zeros(pad, np.uint8)]), bitorder="little").view(np.uint32)


def config_json(cfg: dict) -> str:
    return json.dumps(cfg, separators=(",", ":"))
