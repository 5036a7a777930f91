"""The allocation-free suffix-automaton entry point
(ullis_cuda_rosa_sam_static) against the regular, pool-backed one and against
the CPU oracle.

It exists for callers that may not allocate device memory while they run - a
process working inside a fixed device-memory budget, a latency-critical thread
that cannot afford cudaMalloc's device-wide synchronisation, a plugin in a
process whose own pool already holds the whole GPU.  They pass their own device
buffers; the automaton state sits in a 64 MiB array built into the library.

The file name makes pytest collect it last, so a failure here cannot hide the
result of any other test in a run that stops at the first failure.  It calls
the entry point twice in a row with different shapes: the array keeps the
previous call's contents, and the second result must not depend on them.
"""
import numpy as np
import pytest

from conftest import pack_plane, pack_streams
from ullis_b200 import cuda

pytestmark = pytest.mark.gpu


def _case(rng, n, T, biased):
    if biased:
        pr = rng.choice([0.02, 0.5, 0.98], (n, 1))
        q, k = ((rng.random((n, T)) < pr).astype(np.uint8) for _ in range(2))
    else:
        q, k = (rng.integers(0, 2, (n, T), dtype=np.uint8) for _ in range(2))
    v = rng.integers(0, 2, (n, T), dtype=np.uint8)
    return q, k, v


def _run_static(q, k, v):
    import torch
    n, T = q.shape
    dev = [torch.from_numpy(pack_streams(a).view(np.int32)).cuda() for a in (q, k, v)]
    out = torch.full_like(dev[0], -1)
    torch.cuda.synchronize()
    cuda.rosa_sam_static(0, 0, dev[0].data_ptr(), dev[1].data_ptr(), dev[2].data_ptr(), out.data_ptr(), n, T)
    words = out.cpu().numpy().view(np.uint32)
    bits = np.unpackbits(words.view(np.uint8).reshape(n, -1), axis=1, bitorder="little")[:, :T]
    return bits


def _run_pooled(cuda_rt, q, k, v):
    n, T = q.shape
    planes = [pack_plane(a.T.reshape(-1)) for a in (q, k, v)]  # streams as channels of one sequence
    idx, _ = cuda_rt.rosa_qkv_1bit_fwd(*planes, np.full(n, 0x3C00, np.uint16), 1, T, n)
    return idx.reshape(T, n).T


def _run_oracle(oracle, q, k, v):
    n, T = q.shape
    words = oracle.rosa_qkv_streams(*(pack_streams(a) for a in (q, k, v)), n, T)
    return np.unpackbits(words.view(np.uint8).reshape(n, -1), axis=1, bitorder="little")[:, :T]


def test_static_scratch_entry_matches_pooled_entry_twice_in_a_row(cuda_rt, oracle):
    rng = np.random.default_rng(99)
    for n, T, biased in [(200, 300, False), (50, 64, True), (902, 2048, True)]:
        q, k, v = _case(rng, n, T, biased)
        got = _run_static(q, k, v)
        ref = _run_pooled(cuda_rt, q, k, v)
        assert np.array_equal(got, ref), (n, T)   # integer result: bit-exact
        assert np.array_equal(got, _run_oracle(oracle, q, k, v)), (n, T)   # and equal to the reference's pushes


def test_static_scratch_entry_refuses_what_does_not_fit(cuda_rt):
    import torch
    buf = torch.zeros(1024, dtype=torch.int32, device="cuda")
    p = buf.data_ptr()
    with pytest.raises(cuda.UllisCudaError) as e:   # 903 streams at T=2048 exceed 64 MiB
        cuda.rosa_sam_static(0, 0, p, p, p, p, 903, 2048)
    assert e.value.code == cuda.ERR_NOMEM and "built-in array holds" in e.value.message
    with pytest.raises(cuda.UllisCudaError) as e:
        cuda.rosa_sam_static(0, 0, p, p, p, p, 0, 16)
    assert e.value.code == cuda.ERR_SHAPE
    with pytest.raises(cuda.UllisCudaError) as e:
        cuda.rosa_sam_static(0, 0, 0, p, p, p, 1, 16)
    assert e.value.code == cuda.ERR_ARG
