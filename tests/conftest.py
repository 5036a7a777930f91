import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); deselected by -m 'not gpu'")


def _cuda_device_present() -> bool:
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:  # noqa: BLE001
        return False


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as O
    O.lib()
    O.set_threads(min(16, O.max_threads()))
    return O


@pytest.fixture(scope="session")
def sam_host(tmp_path_factory):
    """Host-compiled build of the device suffix-automaton routines."""
    import ctypes as C
    out = str(tmp_path_factory.mktemp("sam_host") / "libsam_host.so")
    src = os.path.join(ROOT, "tests", "host_harness", "sam_host.cpp")
    subprocess.run(["g++", "-O2", "-std=c++17", "-fPIC", "-shared", src, "-o", out], check=True)
    lib = C.CDLL(out)

    def run(algo, ix_bits, qw, kw, vw, n_streams, T):
        wps = (T + 31) // 32
        qw, kw, vw = [np.ascontiguousarray(a, np.uint32).reshape(-1) for a in (qw, kw, vw)]
        assert qw.size == n_streams * wps
        out_w = np.zeros(n_streams * wps, np.uint32)
        rc = lib.sam_host_batch(C.c_int(algo), C.c_int(ix_bits), C.c_void_p(qw.ctypes.data),
                                C.c_void_p(kw.ctypes.data), C.c_void_p(vw.ctypes.data), C.c_size_t(n_streams),
                                C.c_uint32(T), C.c_void_p(out_w.ctypes.data), None, None)
        assert rc == 0
        return out_w.reshape(n_streams, wps)

    return run


@pytest.fixture(scope="session")
def cuda_rt():
    """CUDA runtime over the C ABI; GPU tests fail (not skip) without the library."""
    from ullis_b200 import cuda
    if not _cuda_device_present():
        pytest.skip("no CUDA device")
    rt = cuda.CudaRuntime(0)
    yield rt
    rt.close()


def pack_streams(bits: np.ndarray) -> np.ndarray:
    """[n, T] 0/1 -> [n, ceil(T/32)] u32, bit t at word t/32, bit t%32."""
    n, T = bits.shape
    pad = (-T) % 32
    b = np.concatenate([bits.astype(np.uint8), np.zeros((n, pad), np.uint8)], 1)
    return np.packbits(b, axis=1, bitorder="little").view(np.uint32).reshape(n, -1).copy()


def pack_plane(bits: np.ndarray) -> np.ndarray:
    """flat 0/1 -> LSB-first u32 words (reference pack_bitplane)."""
    bits = np.asarray(bits, np.uint8).reshape(-1)
    pad = (-bits.size) % 32
    return np.packbits(np.concatenate([bits, np.zeros(pad, np.uint8)]), bitorder="little").view(np.uint32).copy()


def unpack_plane(words: np.ndarray, n: int) -> np.ndarray:
    return np.unpackbits(np.ascontiguousarray(words, np.uint32).view(np.uint8), bitorder="little")[:n]
