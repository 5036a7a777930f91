"""v2 checkpoint.safetensors writer / validator and the seeded generators."""
import json

import numpy as np
import pytest

from ullis_b200 import checkpoint as ckpt
from ullis_b200 import synth


def test_checkpoint_round_trip_and_third_party_reader(tmp_path):
    data = synth.heron_checkpoint("tiny")
    tensors, cfg, step, ema = ckpt.from_safetensors_bytes(data)
    assert cfg["d_model"] == 64 and cfg["n_layers"] == 2 and step == 0 and ema is None
    again = ckpt.to_safetensors_bytes(tensors, cfg, step)
    assert again == data
    # the same bytes through the safetensors package (the container the reference uses)
    from safetensors import safe_open
    p = tmp_path / "checkpoint.safetensors"
    p.write_bytes(data)
    with safe_open(str(p), "np") as f:
        meta = f.metadata()
        assert meta["format_version"] == "2" and json.loads(meta["config"])["vocab_size"] == 512
        assert set(f.keys()) == set(tensors)
        e = f.get_tensor("blocks.0.rosa.e")
        assert e.dtype == np.float16 and np.array_equal(e.view(np.uint16), tensors["blocks.0.rosa.e"])
        assert np.array_equal(f.get_tensor("head.bits"), tensors["head.bits"])


def test_tensor_names_and_shapes_follow_the_reference():
    cfg = synth.train_config(64, 2, 512, 64, 1, 128)
    t = synth.heron_tensors(cfg)
    assert "blocks.0.ln0.weight" in t and "blocks.1.ln0.weight" not in t
    assert "blocks.0.ffn.key.bias" not in t          # CMix key has no bias
    assert t["blocks.1.rosa.q.bits"].size == 64 * 64 // 32 and t["blocks.1.ffn.value"].size == 64 * 128
    assert t["head.bits"].dtype == np.uint32 and t["head.bias"].size == 512
    ckpt.validate_shapes(t, cfg)


def test_v1_and_malformed_checkpoints_are_rejected():
    cfg = synth.train_config(64, 2, 512, 64, 1, 128)
    t = synth.heron_tensors(cfg)
    with pytest.raises(ValueError, match="intentionally unloadable"):
        ckpt.from_safetensors_bytes(ckpt.to_safetensors_bytes(t, cfg, format_version=1))
    with pytest.raises(ValueError):
        ckpt.from_safetensors_bytes(b"\x00\x01")
    bad = dict(t)
    bad["blocks.1.rosa.q.scale"] = bad["blocks.1.rosa.q.scale"][:-1]
    with pytest.raises(ValueError, match="packed-linear shape mismatch"):
        ckpt.from_safetensors_bytes(ckpt.to_safetensors_bytes(bad, cfg))
    bad = dict(t)
    del bad["blocks.1.ln2.weight"]
    with pytest.raises(ValueError, match="exactly n_layers"):
        ckpt.from_safetensors_bytes(ckpt.to_safetensors_bytes(bad, cfg))
    bad = dict(t)
    bad["blocks.0.ffn.key.bias"] = np.zeros(128, np.uint16)
    with pytest.raises(ValueError, match="bias mismatch"):
        ckpt.from_safetensors_bytes(ckpt.to_safetensors_bytes(bad, cfg))


def test_head_without_bias_is_accepted():
    data = synth.heron_checkpoint("tiny", head_bias=False)
    tensors, _, _, _ = ckpt.from_safetensors_bytes(data)
    assert "head.bias" not in tensors


def test_generators_are_deterministic_and_distributed_as_stated():
    a = synth.heron_checkpoint("tiny", seed=7)
    assert a == synth.heron_checkpoint("tiny", seed=7) and a != synth.heron_checkpoint("tiny", seed=8)
    cfg = synth.train_config(256, 1, 8192, 512, 1, 1024)
    t = synth.heron_tensors(cfg)
    scale = t["head.scale"].view(np.float16).astype(np.float32)
    assert 0.0049 <= scale.min() and scale.max() <= 0.0201
    emb = t["embedding"].view(np.float16).astype(np.float32)
    assert abs(emb.std() - 0.02) < 5e-4 and abs(emb.mean()) < 1e-4
    bits = np.unpackbits(t["head.bits"].view(np.uint8))
    assert abs(bits.mean() - 0.5) < 2e-3
    val = t["blocks.0.ffn.value"].view(np.float16).astype(np.float32)
    assert np.abs(val).max() <= 1 / np.sqrt(1024) + 1e-4
    z = synth.zipf_tokens(11, 50000, 8192)
    assert z.max() < 8192 and (z == 0).mean() > 0.05 and np.array_equal(z, synth.zipf_tokens(11, 50000, 8192))
    u = synth.uniform_tokens(11, 4096, 8192)
    assert u.max() < 8192 and len(np.unique(u)) > 2500
    # splitmix64 known answers (state 0: first outputs of the published generator)
    s = synth.splitmix64_stream(0, 3)
    assert [int(x) for x in s] == [0xE220A8397B1DCDAF, 0x6E789E6AA1B965F4, 0x06C45D188009454F]


def test_rosa_bit_generators_shapes():
    q, k, v = synth.rosa_bits_iid(3, 2, 64, 32)
    assert q.size == 2 * 64 * 32 // 32 and not np.array_equal(q, k)
    q, k, v = synth.rosa_bits_periodic(3, 2, 512, 32)
    qb = np.unpackbits(q.view(np.uint8), bitorder="little").reshape(2, 512, 32)
    kb = np.unpackbits(k.view(np.uint8), bitorder="little").reshape(2, 512, 32)
    agree = (qb == kb).mean()
    assert 0.75 < agree < 0.90  # same base pattern, independent 10 % flips: 0.82 expected
