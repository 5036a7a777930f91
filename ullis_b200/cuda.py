"""Host-side mirror of the reference's backend interface for the `cuda`
backend, over the C ABI of libullis_cuda.so (include/ullis_cuda.h).

`CudaRuntime` plays the role `MetalRuntime` plays in the reference
(src/metal.rs:452-457): one object per device whose methods take host arrays
and return host arrays, one synchronous call each, same names and argument
meaning (`layer_norm`, `binary_linear`, `rosa_qkv_1bit_fwd`,
`rosa_block_forward`, `cmix_block_forward`, ...).  `CudaHeron` is the
device-resident whole-model entry point (UllisHeron::hidden / logits and the
CE forward, src/model.rs:2644-2688, 3205-3228).  Failures raise
`UllisCudaError` carrying the ABI status code and message, the way the
reference's methods return `Err(anyhow!(..))`.

There is no CPU fallback: if the shared library is missing, or no CUDA device
is present, construction fails loudly.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libullis_cuda.so")

OK, ERR_SHAPE, ERR_CHECKPOINT, ERR_CUDA, ERR_DEVICE_CHECK, ERR_NCCL, ERR_TIMEOUT, ERR_ARG, ERR_TOKEN, ERR_NOMEM = range(10)
MODE_FAST, MODE_EXACT = 0, 1
SAM_EULER, SAM_EAGER = 0, 1
CE_NO_IGNORE = 0xFFFFFFFF  # reference src/model.rs:24
TAPS = {"block_in": 0, "ln3_out": 1, "q_bits": 2, "k_bits": 3, "v_bits": 4, "idx": 5, "after_rosa": 6,
        "block_out": 7, "hidden": 8}
PHASES = ("embed_ln", "qkv", "sam", "o", "cmix", "head_ce")

# every symbol include/ullis_cuda.h declares
ABI_SYMBOLS = (
    "ullis_cuda_runtime_create", "ullis_cuda_runtime_destroy", "ullis_cuda_last_error",
    "ullis_cuda_runtime_set_mode", "ullis_cuda_runtime_set_sam", "ullis_cuda_runtime_synchronize",
    "ullis_cuda_runtime_stream", "ullis_cuda_runtime_launch_count", "ullis_cuda_runtime_is_sm100",
    "ullis_cuda_runtime_kernel_timing", "ullis_cuda_runtime_kernel_time", "ullis_cuda_runtime_kernel_names",
    "ullis_cuda_model_load_safetensors", "ullis_cuda_model_destroy", "ullis_cuda_model_dims",
    "ullis_cuda_model_forward_ce", "ullis_cuda_model_upload_tokens", "ullis_cuda_model_enqueue_forward_ce",
    "ullis_cuda_model_read_loss", "ullis_cuda_model_logits", "ullis_cuda_model_hidden",
    "ullis_cuda_model_set_taps", "ullis_cuda_model_tap", "ullis_cuda_model_set_profile",
    "ullis_cuda_model_phase_ms", "ullis_cuda_generate_state_create", "ullis_cuda_generate_state_destroy",
    "ullis_cuda_generate_state_reset", "ullis_cuda_generate_state_time", "ullis_cuda_generate_step",
    "ullis_cuda_rosa_pushers_create", "ullis_cuda_rosa_pushers_destroy", "ullis_cuda_rosa_pushers_reset",
    "ullis_cuda_rosa_pushers_push",
    "ullis_cuda_train_state_create", "ullis_cuda_train_state_destroy", "ullis_cuda_model_train_step",
    "ullis_cuda_train_state_read", "ullis_cuda_train_state_install_head_unigram_prior",
    "ullis_cuda_clipped_sgd_fp16", "ullis_cuda_binaryconnect_sgd_fp16", "ullis_cuda_apply_latent_sgd",
    "ullis_cuda_rosa_qkv_1bit_bwd_e", "ullis_cuda_cmix_relu2_backward", "ullis_cuda_layer_norm_backward",
    "ullis_cuda_layer_norm", "ullis_cuda_time_shift_delta",
    "ullis_cuda_binary_linear", "ullis_cuda_fp16_linear", "ullis_cuda_sign_pack_bits", "ullis_cuda_cmix_relu2",
    "ullis_cuda_residual_add", "ullis_cuda_rosa_qkv_1bit_fwd", "ullis_cuda_rosa_block_forward",
    "ullis_cuda_cmix_block_forward", "ullis_cuda_streamed_ce", "ullis_cuda_rosa_sam_static",
    "ullis_cuda_runtime_sam_counts", "ullis_cuda_runtime_wait_selftest", "ullis_cuda_model_read_loss_global", "ullis_cuda_dp_rendezvous",
    "ullis_cuda_dp_unique_id", "ullis_cuda_dp_init",
    "ullis_cuda_dp_allreduce_loss", "ullis_cuda_dp_finalize",
)


class UllisCudaError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"[ullis-cuda {code}] {message}")
        self.code = code
        self.message = message


_LIB = None


def load_library() -> C.CDLL:
    """Loads libullis_cuda.so (never builds, never falls back)."""
    global _LIB
    if _LIB is None:
        if not os.path.exists(LIB_PATH):
            raise UllisCudaError(ERR_ARG, f"{LIB_PATH} is missing: build it with `python -m ullis_b200.build`")
        lib = C.CDLL(LIB_PATH)
        lib.ullis_cuda_last_error.restype = C.c_char_p
        lib.ullis_cuda_last_error.argtypes = [C.c_void_p]
        lib.ullis_cuda_runtime_stream.restype = C.c_void_p
        lib.ullis_cuda_runtime_stream.argtypes = [C.c_void_p]
        lib.ullis_cuda_runtime_launch_count.restype = C.c_uint64
        lib.ullis_cuda_runtime_launch_count.argtypes = [C.c_void_p]
        lib.ullis_cuda_runtime_destroy.restype = None
        lib.ullis_cuda_runtime_destroy.argtypes = [C.c_void_p]
        lib.ullis_cuda_model_destroy.restype = None
        lib.ullis_cuda_model_destroy.argtypes = [C.c_void_p]
        lib.ullis_cuda_generate_state_destroy.restype = None
        lib.ullis_cuda_generate_state_destroy.argtypes = [C.c_void_p]
        lib.ullis_cuda_rosa_pushers_destroy.restype = None
        lib.ullis_cuda_rosa_pushers_destroy.argtypes = [C.c_void_p]
        lib.ullis_cuda_train_state_destroy.restype = None
        lib.ullis_cuda_train_state_destroy.argtypes = [C.c_void_p]
        lib.ullis_cuda_generate_state_time.restype = C.c_size_t
        lib.ullis_cuda_generate_state_time.argtypes = [C.c_void_p]
        _LIB = lib
    return _LIB


class _Handle:
    """A C handle with the handles that borrow it.  Runtime -> model -> state handles must be
    destroyed children first, but a garbage collection that finds the Python objects unreachable
    together runs their finalisers in no particular order (and has cleared weak references by
    then), so each parent handle keeps its children's handles and closes them before itself.
    A child handle does not refer to its parent: no reference cycle is formed."""

    def __init__(self, h, destroy, parent: "_Handle | None" = None):
        self.h, self._destroy, self.children = h, destroy, []
        if parent is not None:
            parent.children[:] = [c for c in parent.children if c.h]   # drop the ones already closed
            parent.children.append(self)

    def close(self):
        for child in self.children:
            child.close()
        self.children = []
        if self.h:
            self._destroy(self.h)
            self.h = None


def _ptr(a):
    return None if a is None else C.c_void_p(a.ctypes.data)


def _arr(a, dtype, name, size=None, allow_none=False):
    if a is None:
        if allow_none:
            return None
        raise UllisCudaError(ERR_ARG, f"{name} is null")
    a = np.ascontiguousarray(a, dtype=dtype).reshape(-1)
    if size is not None and a.size != size:
        raise UllisCudaError(ERR_SHAPE, f"{name} length mismatch: got {a.size}, expected {size}")
    return a


def _z(n):
    return C.c_size_t(int(n))


class CudaRuntime:
    """One per device per process, used from one thread (like MetalRuntime)."""

    def __init__(self, device: int = 0):
        self._lib = load_library()
        h = C.c_void_p()
        rc = self._lib.ullis_cuda_runtime_create(C.c_int32(device), C.byref(h))
        if rc != OK:
            raise UllisCudaError(rc, self._lib.ullis_cuda_last_error(None).decode())
        self._handle = _Handle(h, self._lib.ullis_cuda_runtime_destroy)
        self.device = device

    @property
    def _h(self):
        return self._handle.h

    def close(self):
        if getattr(self, "_handle", None):
            self._handle.close()

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001
            pass

    def _check(self, rc: int):
        if rc != OK:
            raise UllisCudaError(rc, self._lib.ullis_cuda_last_error(self._h).decode())

    # ---- options / introspection
    def set_mode(self, mode: int):
        self._check(self._lib.ullis_cuda_runtime_set_mode(self._h, C.c_int32(mode)))

    def set_sam(self, algo: int):
        self._check(self._lib.ullis_cuda_runtime_set_sam(self._h, C.c_int32(algo)))

    def synchronize(self):
        self._check(self._lib.ullis_cuda_runtime_synchronize(self._h))

    @property
    def stream(self) -> int:
        return int(self._lib.ullis_cuda_runtime_stream(self._h) or 0)

    @property
    def launch_count(self) -> int:
        return int(self._lib.ullis_cuda_runtime_launch_count(self._h))

    def kernel_timing(self, enabled: bool) -> None:
        """Start (or stop) recording an event behind every launch; starting clears earlier records."""
        self._check(self._lib.ullis_cuda_runtime_kernel_timing(self._h, C.c_int32(1 if enabled else 0)))

    def kernel_times(self) -> dict:
        """{kernel name: (total device ms, launches)} since kernel_timing(True)."""
        need = C.c_size_t(0)
        self._check(self._lib.ullis_cuda_runtime_kernel_names(self._h, None, C.c_size_t(0), C.byref(need)))
        buf = C.create_string_buffer(max(int(need.value), 1))
        self._check(self._lib.ullis_cuda_runtime_kernel_names(self._h, buf, C.c_size_t(len(buf)), C.byref(need)))
        out = {}
        for name in buf.value.decode().split():
            ms, n = C.c_float(0), C.c_uint32(0)
            self._check(self._lib.ullis_cuda_runtime_kernel_time(self._h, name.encode(), C.byref(ms), C.byref(n)))
            out[name] = (float(ms.value), int(n.value))
        return out

    @property
    def is_sm100(self) -> bool:
        return bool(self._lib.ullis_cuda_runtime_is_sm100(self._h))

    # ---- op level (names and argument meaning of MetalRuntime's methods)
    def layer_norm(self, x, weight_bits, bias_bits, rows: int, channels: int) -> np.ndarray:
        x = _arr(x, np.float32, "x", rows * channels)
        w = _arr(weight_bits, np.uint16, "weight", channels)
        b = _arr(bias_bits, np.uint16, "bias", channels)
        y = np.empty(rows * channels, np.float32)
        self._check(self._lib.ullis_cuda_layer_norm(self._h, _ptr(x), _ptr(w), _ptr(b), _ptr(y), _z(rows), _z(channels)))
        return y

    def time_shift_delta(self, x, rows: int, time: int, channels: int) -> np.ndarray:
        x = _arr(x, np.float32, "x", rows * channels)
        xx = np.empty(rows * channels, np.float32)
        self._check(self._lib.ullis_cuda_time_shift_delta(self._h, _ptr(x), _ptr(xx), _z(rows), _z(time), _z(channels)))
        return xx

    def binary_linear(self, x, bits, scale_bits, bias_bits, rows: int, in_features: int, out_features: int):
        x = _arr(x, np.float32, "x", rows * in_features)
        bits = _arr(bits, np.uint32, "bits", (in_features * out_features + 31) // 32)
        s = _arr(scale_bits, np.uint16, "scale", out_features)
        b = _arr(bias_bits, np.uint16, "bias", out_features, allow_none=True)
        y = np.empty(rows * out_features, np.float32)
        self._check(self._lib.ullis_cuda_binary_linear(self._h, _ptr(x), _ptr(bits), _ptr(s), _ptr(b), _ptr(y),
                                                       _z(rows), _z(in_features), _z(out_features)))
        return y

    def fp16_linear(self, x, weight_bits, rows: int, in_features: int, out_features: int) -> np.ndarray:
        x = _arr(x, np.float32, "x", rows * in_features)
        w = _arr(weight_bits, np.uint16, "weight", in_features * out_features)
        y = np.empty(rows * out_features, np.float32)
        self._check(self._lib.ullis_cuda_fp16_linear(self._h, _ptr(x), _ptr(w), _ptr(y), _z(rows), _z(in_features),
                                                     _z(out_features)))
        return y

    def sign_pack_bits(self, x) -> np.ndarray:
        x = _arr(x, np.float32, "x")
        bits = np.zeros((x.size + 31) // 32, np.uint32)
        self._check(self._lib.ullis_cuda_sign_pack_bits(self._h, _ptr(x), _ptr(bits), _z(x.size)))
        return bits

    def cmix_relu2(self, x) -> np.ndarray:
        x = _arr(x, np.float32, "x")
        y = np.empty(x.size, np.float32)
        self._check(self._lib.ullis_cuda_cmix_relu2(self._h, _ptr(x), _ptr(y), _z(x.size)))
        return y

    def _sgd(self, fn, parameters, residual, gradient, learning_rate, *extra):
        w = _arr(parameters, np.uint16, "parameters")
        r = _arr(residual, np.float32, "residual", w.size)
        g = _arr(gradient, np.float32, "gradient", w.size)
        nw, nr = np.empty(w.size, np.uint16), np.empty(w.size, np.float32)
        self._check(fn(self._h, _ptr(w), _ptr(r), _ptr(g), C.c_float(learning_rate), *extra, _z(w.size), _ptr(nw),
                       _ptr(nr)))
        return nw, nr

    def clipped_sgd_fp16(self, parameters, residual, gradient, learning_rate: float):
        """MetalRuntime::clipped_sgd_fp16 (src/metal.rs:3053) -> (next FP16 bits, next carry)."""
        return self._sgd(self._lib.ullis_cuda_clipped_sgd_fp16, parameters, residual, gradient, learning_rate)

    def binaryconnect_sgd_fp16(self, parameters, residual, gradient, learning_rate: float):
        """MetalRuntime::binaryconnect_sgd_fp16 (src/metal.rs:3069)."""
        return self._sgd(self._lib.ullis_cuda_binaryconnect_sgd_fp16, parameters, residual, gradient, learning_rate)

    def apply_latent_sgd(self, latent, residual, gradient, learning_rate: float, ste_scale: float):
        """MetalRuntime::apply_latent_sgd (src/metal.rs:3006) -> (next latent, next carry, next sign bits)."""
        w = _arr(latent, np.uint16, "latent")
        r = _arr(residual, np.float32, "residual", w.size)
        g = _arr(gradient, np.float32, "gradient", w.size)
        nw, nr = np.empty(w.size, np.uint16), np.empty(w.size, np.float32)
        bits = np.empty((w.size + 31) // 32, np.uint32)
        self._check(self._lib.ullis_cuda_apply_latent_sgd(self._h, _ptr(w), _ptr(r), _ptr(g), C.c_float(learning_rate),
                                                          C.c_float(ste_scale), _z(w.size), _ptr(nw), _ptr(nr),
                                                          _ptr(bits)))
        return nw, nr, bits

    def rosa_qkv_1bit_bwd_e(self, output_gradient, idx, batch: int, time: int, channels: int) -> np.ndarray:
        """MetalRuntime::rosa_qkv_1bit_bwd_e (src/metal.rs:1258): g_e [channels]."""
        n = batch * time * channels
        gy = _arr(output_gradient, np.float32, "output_gradient", n)
        ix = _arr(idx, np.uint8, "idx", n)
        out = np.empty(channels, np.float32)
        self._check(self._lib.ullis_cuda_rosa_qkv_1bit_bwd_e(self._h, _ptr(gy), _ptr(ix), _z(batch), _z(time),
                                                             _z(channels), _ptr(out)))
        return out

    def cmix_relu2_backward(self, input, output_gradient) -> np.ndarray:  # noqa: A002
        """MetalRuntime::cmix_relu2_backward (src/metal.rs:1546)."""
        x = _arr(input, np.float32, "input")
        g = _arr(output_gradient, np.float32, "output_gradient", x.size)
        out = np.empty(x.size, np.float32)
        self._check(self._lib.ullis_cuda_cmix_relu2_backward(self._h, _ptr(x), _ptr(g), _ptr(out), _z(x.size)))
        return out

    def layer_norm_backward(self, input, output_gradient, weight_bits, rows: int, channels: int):  # noqa: A002
        """MetalRuntime::layer_norm_backward (src/metal.rs:1628) -> (gx, gw, gb); weight as FP16 bits."""
        x = _arr(input, np.float32, "input", rows * channels)
        g = _arr(output_gradient, np.float32, "output_gradient", rows * channels)
        w = _arr(weight_bits, np.uint16, "weight", channels)
        gx, gw, gb = np.empty(x.size, np.float32), np.empty(channels, np.float32), np.empty(channels, np.float32)
        self._check(self._lib.ullis_cuda_layer_norm_backward(self._h, _ptr(x), _ptr(g), _ptr(w), _z(rows), _z(channels),
                                                             _ptr(gx), _ptr(gw), _ptr(gb)))
        return gx, gw, gb

    def residual_add(self, residual, update) -> np.ndarray:
        a = _arr(residual, np.float32, "residual")
        b = _arr(update, np.float32, "update", a.size)
        out = np.empty(a.size, np.float32)
        self._check(self._lib.ullis_cuda_residual_add(self._h, _ptr(a), _ptr(b), _ptr(out), _z(a.size)))
        return out

    def rosa_qkv_1bit_fwd(self, q_bits, k_bits, v_bits, e_bits, batch: int, time: int, channels: int,
                          want_out: bool = True):
        """Returns (idx u8 [B,T,C], out f32 [B,T,C]) like RosaQkvForward{idx,out}
        (src/metal.rs:253-256); out is None with want_out=False (the ABI's nullable output)."""
        n = batch * time * channels
        words = (n + 31) // 32
        q = _arr(q_bits, np.uint32, "q_bits", words)
        k = _arr(k_bits, np.uint32, "k_bits", words)
        v = _arr(v_bits, np.uint32, "v_bits", words)
        e = _arr(e_bits, np.uint16, "e", channels)
        idx = np.empty(n, np.uint8)
        out = np.empty(n, np.float32) if want_out else None
        self._check(self._lib.ullis_cuda_rosa_qkv_1bit_fwd(self._h, _ptr(q), _ptr(k), _ptr(v), _ptr(e), _ptr(idx),
                                                           _ptr(out), _z(batch), _z(time), _z(channels)))
        return idx, out

    def rosa_block_forward(self, x, p: dict, batch: int, time: int, channels: int) -> dict:
        """p: x_q, x_k, x_v, e (FP16 bits) and q/k/v/o dicts of bits, scale, bias.
        Returns q_plane, k_plane, v_plane (packed [B,T,C] sign planes), idx, y, out."""
        d = channels
        n = batch * time * d
        x = _arr(x, np.float32, "x", n)
        args = [_arr(p[m], np.uint16, m, d) for m in ("x_q", "x_k", "x_v")]
        lin = []
        for m in ("q", "k", "v"):
            lin += [_arr(p[m]["bits"], np.uint32, m + ".bits", (d * d + 31) // 32),
                    _arr(p[m]["scale"], np.uint16, m + ".scale", d), _arr(p[m]["bias"], np.uint16, m + ".bias", d)]
        e = _arr(p["e"], np.uint16, "e", d)
        o = [_arr(p["o"]["bits"], np.uint32, "o.bits", (d * d + 31) // 32),
             _arr(p["o"]["scale"], np.uint16, "o.scale", d), _arr(p["o"]["bias"], np.uint16, "o.bias", d)]
        words = (n + 31) // 32
        r = {"q_plane": np.empty(words, np.uint32), "k_plane": np.empty(words, np.uint32),
             "v_plane": np.empty(words, np.uint32), "idx": np.empty(n, np.uint8),
             "y": np.empty(n, np.float32), "out": np.empty(n, np.float32)}
        self._check(self._lib.ullis_cuda_rosa_block_forward(
            self._h, _ptr(x), *[_ptr(a) for a in args], *[_ptr(a) for a in lin], _ptr(e), *[_ptr(a) for a in o],
            _z(batch), _z(time), _z(d), _ptr(r["q_plane"]), _ptr(r["k_plane"]), _ptr(r["v_plane"]), _ptr(r["idx"]),
            _ptr(r["y"]), _ptr(r["out"])))
        return r

    def cmix_block_forward(self, x, mix_bits, key_bits, key_scale_bits, value_bits, batch: int, time: int,
                           d_model: int, dim_ffn: int) -> np.ndarray:
        n = batch * time * d_model
        x = _arr(x, np.float32, "x", n)
        mix = _arr(mix_bits, np.uint16, "mix", d_model)
        kb = _arr(key_bits, np.uint32, "key_bits", (d_model * dim_ffn + 31) // 32)
        ks = _arr(key_scale_bits, np.uint16, "key_scale", dim_ffn)
        val = _arr(value_bits, np.uint16, "value", d_model * dim_ffn)
        out = np.empty(n, np.float32)
        self._check(self._lib.ullis_cuda_cmix_block_forward(self._h, _ptr(x), _ptr(mix), _ptr(kb), _ptr(ks),
                                                            _ptr(val), _z(batch), _z(time), _z(d_model),
                                                            _z(dim_ffn), _ptr(out)))
        return out

    def streamed_ce(self, hidden, bits, scale_bits, bias_bits, labels, ignore_id: int, rows: int, time: int,
                    channels: int, vocab: int):
        """Returns (mean_loss, n_valid, row_loss)."""
        h = _arr(hidden, np.float32, "hidden", rows * channels)
        bits = _arr(bits, np.uint32, "bits", (vocab * channels + 31) // 32)
        s = _arr(scale_bits, np.uint16, "scale", vocab)
        b = _arr(bias_bits, np.uint16, "bias", vocab, allow_none=True)
        lab = _arr(labels, np.uint32, "labels", rows)
        row_loss = np.empty(rows, np.float32)
        mean = C.c_float(0)
        n_valid = C.c_uint64(0)
        self._check(self._lib.ullis_cuda_streamed_ce(self._h, _ptr(h), _ptr(bits), _ptr(s), _ptr(b), _ptr(lab),
                                                     C.c_uint32(ignore_id), _z(rows), _z(time), _z(channels),
                                                     _z(vocab), _ptr(row_loss), C.byref(mean), C.byref(n_valid)))
        return float(mean.value), int(n_valid.value), row_loss

    # ---- data parallel
    @staticmethod
    def dp_unique_id() -> bytes:
        buf = (C.c_uint8 * 128)()
        rc = load_library().ullis_cuda_dp_unique_id(buf)
        if rc != OK:
            raise UllisCudaError(rc, "ncclGetUniqueId failed")
        return bytes(buf)

    @staticmethod
    def dp_rendezvous(directory: str, tag: str, rank: int, world: int, timeout_s: float = 60.0) -> None:
        """Host-side rendezvous with a deadline (ullis_cuda_dp_rendezvous): raises ERR_TIMEOUT when a rank
        has not announced itself in `directory` in time.  Call it before dp_init."""
        lib = load_library()
        rc = lib.ullis_cuda_dp_rendezvous(directory.encode(), tag.encode(), C.c_int32(rank), C.c_int32(world),
                                          C.c_uint32(int(timeout_s * 1000)))
        if rc != OK:
            raise UllisCudaError(rc, lib.ullis_cuda_last_error(None).decode())

    def wait_selftest(self, polls: int = 2000) -> None:
        """Makes a bounded device wait run out (ullis_cuda_runtime_wait_selftest): always raises, ERR_TIMEOUT
        when the error path works."""
        self._check(self._lib.ullis_cuda_runtime_wait_selftest(self._h, C.c_uint32(polls)))

    def sam_counts(self) -> dict:
        """Streams of the last suffix-automaton call: total, through the automaton, through the constant-q form."""
        t, a, q = C.c_uint64(0), C.c_uint64(0), C.c_uint64(0)
        self._check(self._lib.ullis_cuda_runtime_sam_counts(self._h, C.byref(t), C.byref(a), C.byref(q)))
        return {"total": int(t.value), "automaton": int(a.value), "constant_q": int(q.value)}

    def dp_init(self, rank: int, world: int, unique_id: bytes):
        buf = (C.c_uint8 * 128).from_buffer_copy(unique_id)
        self._check(self._lib.ullis_cuda_dp_init(self._h, C.c_int32(rank), C.c_int32(world), buf))

    def dp_allreduce_loss(self, loss_sum: float, n_valid: int):
        s = C.c_double(loss_sum)
        n = C.c_uint64(n_valid)
        self._check(self._lib.ullis_cuda_dp_allreduce_loss(self._h, C.byref(s), C.byref(n)))
        return float(s.value), int(n.value)

    def dp_finalize(self):
        self._check(self._lib.ullis_cuda_dp_finalize(self._h))


SAM_STATIC_BYTES = 64 << 20


def rosa_sam_static(device: int, cuda_stream: int, q_sw_ptr: int, k_sw_ptr: int, v_sw_ptr: int, idx_sw_ptr: int,
                    streams: int, time: int) -> None:
    """Allocation-free suffix-automaton match over caller-owned DEVICE buffers
    (raw addresses) using the library's built-in 64 MiB state array; see
    ullis_cuda_rosa_sam_static in include/ullis_cuda.h.  Raises on refusal."""
    lib = load_library()
    rc = lib.ullis_cuda_rosa_sam_static(C.c_int32(device), C.c_void_p(cuda_stream or None), C.c_void_p(q_sw_ptr),
                                        C.c_void_p(k_sw_ptr), C.c_void_p(v_sw_ptr), C.c_void_p(idx_sw_ptr),
                                        _z(streams), _z(time))
    if rc != OK:
        raise UllisCudaError(rc, lib.ullis_cuda_last_error(None).decode())


class CudaHeron:
    """Device-resident Heron model loaded from v2 checkpoint.safetensors bytes."""

    def __init__(self, runtime: CudaRuntime, checkpoint_bytes: bytes):
        self.rt = runtime
        self._lib = runtime._lib
        buf = np.frombuffer(checkpoint_bytes, dtype=np.uint8)
        h = C.c_void_p()
        runtime._check(self._lib.ullis_cuda_model_load_safetensors(runtime._h, _ptr(buf), _z(buf.size), C.byref(h)))
        self._handle = _Handle(h, self._lib.ullis_cuda_model_destroy, runtime._handle)
        dims = (C.c_size_t * 6)()
        self._lib.ullis_cuda_model_dims(self._h, dims)
        self.d_model, self.n_layers, self.vocab_size, self.context_len, self.batch_size, self.dim_ffn = \
            [int(v) for v in dims]

    @property
    def _h(self):
        return self._handle.h

    def close(self):
        if getattr(self, "_handle", None):
            self._handle.close()

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001
            pass

    def forward_ce(self, tokens, labels, ignore_id: int, batch: int, time: int, want_row_loss: bool = False):
        """Returns (mean_loss, loss_sum, n_valid[, row_loss])."""
        t = _arr(tokens, np.uint32, "tokens", batch * time)
        lab = _arr(labels, np.uint32, "labels", batch * time)
        mean, s, n = C.c_float(0), C.c_double(0), C.c_uint64(0)
        rl = np.empty(batch * time, np.float32) if want_row_loss else None
        self.rt._check(self._lib.ullis_cuda_model_forward_ce(self._h, _ptr(t), _ptr(lab), C.c_uint32(ignore_id),
                                                             _z(batch), _z(time), C.byref(mean), C.byref(s),
                                                             C.byref(n), _ptr(rl)))
        out = (float(mean.value), float(s.value), int(n.value))
        return out + (rl,) if want_row_loss else out

    def upload_tokens(self, tokens, labels, batch: int, time: int):
        t = _arr(tokens, np.uint32, "tokens", batch * time)
        lab = _arr(labels, np.uint32, "labels", batch * time, allow_none=True)
        self.rt._check(self._lib.ullis_cuda_model_upload_tokens(self._h, _ptr(t), _ptr(lab), _z(batch), _z(time)))

    def enqueue_forward_ce(self, ignore_id: int, batch: int, time: int):
        self.rt._check(self._lib.ullis_cuda_model_enqueue_forward_ce(self._h, C.c_uint32(ignore_id), _z(batch),
                                                                     _z(time)))

    def read_loss(self, rows: int = 0, want_row_loss: bool = False):
        mean, s, n = C.c_float(0), C.c_double(0), C.c_uint64(0)
        rl = np.empty(rows, np.float32) if want_row_loss else None
        self.rt._check(self._lib.ullis_cuda_model_read_loss(self._h, C.byref(mean), C.byref(s), C.byref(n),
                                                            _ptr(rl), _z(rows)))
        out = (float(mean.value), float(s.value), int(n.value))
        return out + (rl,) if want_row_loss else out

    def read_loss_global(self):
        """read_loss summed over the ranks of the runtime's data-parallel group, on the device."""
        mean, loss_sum, n_valid = C.c_float(0), C.c_double(0), C.c_uint64(0)
        self.rt._check(self._lib.ullis_cuda_model_read_loss_global(self._h, C.byref(mean), C.byref(loss_sum),
                                                                    C.byref(n_valid)))
        return float(mean.value), float(loss_sum.value), int(n_valid.value)

    def logits(self, tokens, batch: int, time: int) -> np.ndarray:
        t = _arr(tokens, np.uint32, "tokens", batch * time)
        out = np.empty(batch * time * self.vocab_size, np.float32)
        self.rt._check(self._lib.ullis_cuda_model_logits(self._h, _ptr(t), _z(batch), _z(time), _ptr(out)))
        return out

    def hidden(self, tokens, batch: int, time: int) -> np.ndarray:
        t = _arr(tokens, np.uint32, "tokens", batch * time)
        out = np.empty(batch * time * self.d_model, np.float32)
        self.rt._check(self._lib.ullis_cuda_model_hidden(self._h, _ptr(t), _z(batch), _z(time), _ptr(out)))
        return out

    def generate_state(self, batch: int = 1) -> "CudaGenerateState":
        """UllisHeron::generate_state (src/model.rs:2691-2715) for `batch` independent sequences."""
        return CudaGenerateState(self, batch)

    def generate_step(self, state: "CudaGenerateState", tokens) -> np.ndarray:
        """UllisHeron::generate_step (src/model.rs:2717-2753): logits [batch, vocab] of the new tokens."""
        return state.step(tokens)

    def train_state(self, checkpoint: bytes | None = None) -> "CudaTrainState":
        """Optimiser carry for this model (latents, f32 residuals); `checkpoint` restores a resumed run's."""
        return CudaTrainState(self, checkpoint)

    def set_taps(self, enabled: bool):
        self.rt._check(self._lib.ullis_cuda_model_set_taps(self._h, C.c_int32(1 if enabled else 0)))

    def tap(self, layer: int, which: str, rows: int) -> np.ndarray:
        code = TAPS[which]
        dtype = np.uint8 if 2 <= code <= 5 else np.float32
        out = np.empty(rows * self.d_model, dtype)
        self.rt._check(self._lib.ullis_cuda_model_tap(self._h, C.c_int32(layer), C.c_int32(code), _ptr(out),
                                                      _z(out.nbytes)))
        return out

    def set_profile(self, enabled: bool):
        self.rt._check(self._lib.ullis_cuda_model_set_profile(self._h, C.c_int32(1 if enabled else 0)))

    def phase_ms(self) -> dict:
        ms = (C.c_float * 6)()
        self.rt._check(self._lib.ullis_cuda_model_phase_ms(self._h, ms))
        return {name: float(ms[i]) for i, name in enumerate(PHASES)}


class CudaGenerateState:
    """HeronGenerateState (src/model.rs:2433-2454) on the device: one automaton per
    (sequence, layer, channel) and the time-shift inputs; borrowed model."""

    def __init__(self, model: CudaHeron, batch: int = 1):
        self.model, self.batch = model, int(batch)
        self._lib = model._lib
        h = C.c_void_p()
        model.rt._check(self._lib.ullis_cuda_generate_state_create(model._h, _z(batch), C.byref(h)))
        self._handle = _Handle(h, self._lib.ullis_cuda_generate_state_destroy, model._handle)

    @property
    def _h(self):
        return self._handle.h

    @property
    def time(self) -> int:
        return int(self._lib.ullis_cuda_generate_state_time(self._h))

    def reset(self) -> None:
        self.model.rt._check(self._lib.ullis_cuda_generate_state_reset(self._h))

    def step(self, tokens) -> np.ndarray:
        t = _arr(np.atleast_1d(tokens), np.uint32, "tokens", self.batch)
        out = np.empty((self.batch, self.model.vocab_size), np.float32)
        self.model.rt._check(self._lib.ullis_cuda_generate_step(self._h, _ptr(t), _ptr(out)))
        return out

    def close(self):
        if getattr(self, "_handle", None):
            self._handle.close()

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001
            pass


class CudaRosaPushers:
    """`streams` RosaSam automata (src/rosa.rs:55-176) on the device; push() is RosaSam::push for every stream,
    once per row of q / k / v ([steps, streams] of 0 / 1), and returns idx in the same shape."""

    def __init__(self, rt: CudaRuntime, streams: int, capacity: int):
        self.rt, self.streams, self.capacity = rt, int(streams), int(capacity)
        self._lib = rt._lib
        h = C.c_void_p()
        rt._check(self._lib.ullis_cuda_rosa_pushers_create(rt._h, _z(streams), _z(capacity), C.byref(h)))
        self._handle = _Handle(h, self._lib.ullis_cuda_rosa_pushers_destroy, rt._handle)

    def reset(self) -> None:
        self.rt._check(self._lib.ullis_cuda_rosa_pushers_reset(self._handle.h))

    def push(self, q, k, v) -> np.ndarray:
        q = np.ascontiguousarray(np.atleast_2d(q), np.uint8)
        steps = q.shape[0]
        q, k, v = (_arr(np.atleast_2d(a), np.uint8, n, steps * self.streams) for a, n in ((q, "q"), (k, "k"), (v, "v")))
        idx = np.empty((steps, self.streams), np.uint8)
        self.rt._check(self._lib.ullis_cuda_rosa_pushers_push(self._handle.h, _ptr(q), _ptr(k), _ptr(v), _z(steps), _ptr(idx)))
        return idx

    def close(self):
        if getattr(self, "_handle", None):
            self._handle.close()

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001
            pass


class _TrainResult(C.Structure):
    _fields_ = [("mean_loss", C.c_float), ("n_valid", C.c_uint64), ("flips_head", C.c_uint64),
                ("flips_cmix", C.c_uint64), ("flips_rosa_o", C.c_uint64)]


class _UnigramInstall(C.Structure):
    _fields_ = [("applied", C.c_int32), ("n_targets", C.c_uint64), ("bias_rms", C.c_float), ("scale_rms", C.c_float),
                ("shrunk_kaiming_scale", C.c_int32)]


class CudaTrainState:
    """Weights, BinaryConnect latents and f32 carry of a model being trained on the device
    (UllisHeron::train_step_with_labels, src/model.rs:2773-2785, in stop_grad_bits mode).
    The model is borrowed and modified: its forward / generate calls see the stepped weights."""

    def __init__(self, model: CudaHeron, checkpoint: bytes | None = None):
        self.model = model
        self._lib = model._lib
        h = C.c_void_p()
        buf = None if checkpoint is None else (C.c_uint8 * len(checkpoint)).from_buffer_copy(checkpoint)
        model.rt._check(self._lib.ullis_cuda_train_state_create(model._h, buf, _z(0 if checkpoint is None else
                                                                                  len(checkpoint)), C.byref(h)))
        self._handle = _Handle(h, self._lib.ullis_cuda_train_state_destroy, model._handle)

    @property
    def _h(self):
        return self._handle.h

    def train_step(self, tokens, labels, ignore_id: int, batch: int, time: int, learning_rate: float) -> dict:
        t = _arr(tokens, np.uint32, "tokens", batch * time)
        lab = _arr(labels, np.uint32, "labels", batch * time)
        res = _TrainResult()
        self.model.rt._check(self._lib.ullis_cuda_model_train_step(
            self._h, _ptr(t), _ptr(lab), C.c_uint32(ignore_id), _z(batch), _z(time), C.c_float(learning_rate),
            C.byref(res)))
        return {"loss": float(res.mean_loss), "n_valid": int(res.n_valid), "flips_head": int(res.flips_head),
                "flips_cmix": int(res.flips_cmix), "flips_rosa_o": int(res.flips_rosa_o)}

    def install_head_unigram_prior(self, labels, ignore_id: int) -> dict:
        """UllisHeron::install_head_unigram_prior (src/model.rs:3034-3085) -> HeadUnigramInstall fields."""
        lab = _arr(labels, np.uint32, "labels")
        res = _UnigramInstall()
        self.model.rt._check(self._lib.ullis_cuda_train_state_install_head_unigram_prior(
            self._h, _ptr(lab), _z(lab.size), C.c_uint32(ignore_id), C.byref(res)))
        return {"applied": bool(res.applied), "n_targets": int(res.n_targets), "bias_rms": float(res.bias_rms),
                "scale_rms": float(res.scale_rms), "shrunk_kaiming_scale": bool(res.shrunk_kaiming_scale)}

    def read(self, name: str, dtype, count: int) -> np.ndarray:
        """Tensor of the trained model or of its carry by checkpoint name (u16 = FP16 bits)."""
        out = np.empty(count, dtype)
        self.model.rt._check(self._lib.ullis_cuda_train_state_read(self._h, name.encode(), _ptr(out),
                                                                   _z(out.nbytes)))
        return out

    def close(self):
        if getattr(self, "_handle", None):
            self._handle.close()

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001
            pass
