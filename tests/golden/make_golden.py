"""Regenerates the committed golden fixtures from the CPU oracle.

The reference crate is Rust and cannot be built or imported here, so these
vectors come from the C restatement in oracle/ (itself pinned to the
reference's own known-answer tests, see tests/test_oracle_golden.py).  They
freeze its outputs on seeded inputs so that a change in either the oracle or
the CUDA path shows up as a diff against a committed file.

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import oracle as O  # noqa: E402
from ullis_b200 import synth  # noqa: E402


def sam_streams():
    rng = np.random.default_rng(20240607)
    T, n = 300, 12
    out = {}
    for kind in ("iid", "biased", "periodic"):
        if kind == "iid":
            q, k, v = (rng.integers(0, 2, (n, T), dtype=np.uint8) for _ in range(3))
        elif kind == "biased":
            pr = rng.choice([0.01, 0.99], (n, 1))
            q, k = ((rng.random((n, T)) < pr).astype(np.uint8) for _ in range(2))
            v = rng.integers(0, 2, (n, T), dtype=np.uint8)
        else:
            P = rng.integers(3, 40, n)
            base = rng.integers(0, 2, (n, 40), dtype=np.uint8)
            b = np.take_along_axis(base, np.arange(T)[None, :] % P[:, None], 1)
            q = (b ^ (rng.random((n, T)) < 0.1)).astype(np.uint8)
            k = (b ^ (rng.random((n, T)) < 0.1)).astype(np.uint8)
            v = rng.integers(0, 2, (n, T), dtype=np.uint8)
        idx = np.stack([O.rosa_qkv_ref(q[s], k[s], v[s]) for s in range(n)])
        for name, a in (("q", q), ("k", k), ("v", v), ("idx", idx)):
            out[f"{kind}_{name}"] = np.packbits(a, axis=1)
    out["T"] = np.array(T)
    np.savez_compressed(os.path.join(HERE, "sam_streams.npz"), **out)


def heron_tiny():
    out = {}
    for variant, gain in (("literal", False), ("gain1", True)):
        data = synth.heron_checkpoint("tiny", batch_size=2, seed=7, ln_gain_one=gain)
        m = O.HeronOracle(data)
        B, T = 2, 64
        tokens = synth.uniform_tokens(11, B * T, m.vocab)
        labels = tokens.copy()
        labels[5] = 3
        taps = {}
        mean, n_valid, row_loss, logits = m.forward_ce(tokens, labels, 3, B, T, taps=taps, want_logits=True)
        out[f"{variant}_tokens"] = tokens
        out[f"{variant}_labels"] = labels
        out[f"{variant}_mean"] = np.float32(mean)
        out[f"{variant}_n_valid"] = np.int64(n_valid)
        out[f"{variant}_row_loss"] = row_loss
        out[f"{variant}_hidden"] = taps["hidden"]
        out[f"{variant}_logits_row0"] = logits[:m.vocab]
        for l in range(m.layers):
            out[f"{variant}_idx{l}"] = np.packbits(taps[f"{l}.idx"])
            out[f"{variant}_qbits{l}"] = np.packbits(taps[f"{l}.q_bits"])
            out[f"{variant}_block_out{l}"] = taps[f"{l}.block_out"]
    np.savez_compressed(os.path.join(HERE, "heron_tiny.npz"), **out)


if __name__ == "__main__":
    O.set_threads(1)
    sam_streams()
    heron_tiny()
    for f in ("sam_streams.npz", "heron_tiny.npz"):
        print(f, os.path.getsize(os.path.join(HERE, f)), "bytes")
