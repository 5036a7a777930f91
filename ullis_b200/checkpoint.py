"""v2 `checkpoint.safetensors` writer/validator for Heron checkpoints.

Format as written by the reference's ModelCheckpoint::to_safetensors_bytes
(src/model.rs:3426-3468): every tensor is flat 1-D (`U32` packed sign bits,
`F16` parameters, `F32` train carry), metadata strings `format_version` = "2",
`config` = JSON TrainConfig, `step`, optional `loss_ema`.  The container is
the safetensors layout: u64 LE header length, JSON header (space padded to 8
bytes), then the raw little-endian tensor bytes in header order.

The CUDA backend parses these files with its own C++ loader; this module is
the host-side mirror used to write synthetic checkpoints and to validate
shapes the way validate_checkpoint_shapes does (src/model.rs:4402-4456).
"""
from __future__ import annotations

import json
import struct

import numpy as np

CHECKPOINT_FORMAT_VERSION = 2  # src/model.rs:21

_DTYPES = {np.dtype(np.uint32): "U32", np.dtype(np.uint16): "F16", np.dtype(np.float32): "F32"}
_NP = {"U32": np.uint32, "F16": np.uint16, "F32": np.float32}


def to_safetensors_bytes(tensors: dict, config: dict, step: int = 0, loss_ema: float | None = None,
                         format_version: int = CHECKPOINT_FORMAT_VERSION) -> bytes:
    meta = {"format_version": str(format_version), "config": json.dumps(config, separators=(",", ":")),
            "step": str(step)}
    if loss_ema is not None:
        meta["loss_ema"] = repr(float(loss_ema))
    # the safetensors serializer orders by descending dtype alignment, then name
    names = sorted(tensors, key=lambda n: (-np.asarray(tensors[n]).dtype.itemsize, n))
    header = {"__metadata__": meta}
    blobs = []
    offset = 0
    for name in names:
        a = np.ascontiguousarray(tensors[name]).reshape(-1)
        dt = _DTYPES[a.dtype]
        raw = a.astype(a.dtype.newbyteorder("<"), copy=False).tobytes()
        header[name] = {"dtype": dt, "shape": [int(a.size)], "data_offsets": [offset, offset + len(raw)]}
        blobs.append(raw)
        offset += len(raw)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((-len(hj)) % 8)
    return struct.pack("<Q", len(hj)) + hj + b"".join(blobs)


def from_safetensors_bytes(data: bytes):
    """Returns (tensors, config, step, loss_ema); raises ValueError with the
    reference's messages for the failure classes it distinguishes
    (src/model.rs:3470-3553, 2420-2431)."""
    if len(data) < 8:
        raise ValueError("parse safetensors checkpoint header")
    (hlen,) = struct.unpack("<Q", data[:8])
    if hlen > len(data) - 8:
        raise ValueError("parse safetensors checkpoint header")
    try:
        header = json.loads(data[8:8 + hlen])
    except Exception as exc:  # noqa: BLE001
        raise ValueError("parse safetensors checkpoint header") from exc
    meta = header.pop("__metadata__", None)
    if meta is None:
        raise ValueError("safetensors checkpoint is missing metadata")
    try:
        version = int(meta.get("format_version", "0"))
    except ValueError:
        version = 0
    if version != CHECKPOINT_FORMAT_VERSION:
        raise ValueError("Hyena checkpoints (v1) are intentionally unloadable after the RWKV-8 cut "
                         f"(got format_version {version})")
    if "config" not in meta:
        raise ValueError("safetensors checkpoint is missing config")
    config = json.loads(meta["config"])
    base = 8 + hlen
    tensors = {}
    for name, info in header.items():
        b, e = info["data_offsets"]
        if info["dtype"] not in _NP or e > len(data) - base or b > e:
            raise ValueError(f"checkpoint tensor {name}")
        tensors[name] = np.frombuffer(data[base + b:base + e], dtype=_NP[info["dtype"]]).copy()
    step = int(meta.get("step", "0")) if meta.get("step", "0").isdigit() else 0
    loss_ema = float(meta["loss_ema"]) if "loss_ema" in meta else None
    validate_shapes(tensors, config)
    return tensors, config, step, loss_ema


def resolved_dim_ffn(config: dict) -> int:  # src/config.rs:135-141
    return config.get("dim_ffn", 0) or 4 * config["d_model"]


def _need(tensors, name, dtype, size, what):
    a = tensors.get(name)
    if a is None:
        raise ValueError(f"checkpoint tensor {name}")
    if a.dtype != dtype:
        raise ValueError(f"expected {'U32' if dtype == np.uint32 else 'F16'} tensor, got {a.dtype}")
    if a.size != size:
        raise ValueError(what)


def validate_shapes(tensors: dict, config: dict) -> None:
    """validate_checkpoint_shapes for the Heron architecture."""
    d, v, layers = config["d_model"], config["vocab_size"], config["n_layers"]
    f = resolved_dim_ffn(config)
    if config.get("architecture", "heron") != "heron":
        raise ValueError("only the heron architecture is supported by the cuda backend")
    _need(tensors, "embedding", np.uint16, v * d, "checkpoint embedding shape does not match its configuration")

    def ln(prefix):
        _need(tensors, prefix + ".weight", np.uint16, d, "checkpoint LayerNorm shape mismatch")
        _need(tensors, prefix + ".bias", np.uint16, d, "checkpoint LayerNorm shape mismatch")

    def packed(prefix, out, inn, bias):
        _need(tensors, prefix + ".bits", np.uint32, (out * inn + 31) // 32, "checkpoint packed-linear shape mismatch")
        _need(tensors, prefix + ".scale", np.uint16, out, "checkpoint packed-linear shape mismatch")
        has = prefix + ".bias" in tensors
        if bias is True and not has or bias is False and has:
            raise ValueError("checkpoint packed-linear bias mismatch")
        if has:
            _need(tensors, prefix + ".bias", np.uint16, out, "checkpoint packed-linear bias mismatch")

    ln("ln_out")
    packed("head", v, d, None)  # head bias optional: absent loads as zeros (src/model.rs:4237-4246)
    n_blocks = 0
    while f"blocks.{n_blocks}.ln2.weight" in tensors:
        n_blocks += 1
    if n_blocks != layers:
        raise ValueError("heron checkpoint must store exactly n_layers Heron blocks")
    for i in range(layers):
        pre = f"blocks.{i}"
        has_ln0 = pre + ".ln0.weight" in tensors
        if has_ln0 != (i == 0):
            raise ValueError("ln0 must be present only on Heron layer 0")
        if has_ln0:
            ln(pre + ".ln0")
        ln(pre + ".ln2")
        ln(pre + ".ln3")
        for m in ("x_q", "x_k", "x_v", "e"):
            _need(tensors, f"{pre}.rosa.{m}", np.uint16, d, f"checkpoint {m} length mismatch")
        for m in "qkvo":
            packed(f"{pre}.rosa.{m}", d, d, True)
        _need(tensors, f"{pre}.ffn.x_k", np.uint16, d, "checkpoint cmix.x_k length mismatch")
        packed(f"{pre}.ffn.key", f, d, False)
        _need(tensors, f"{pre}.ffn.value", np.uint16, f * d, "checkpoint cmix.value length mismatch")
