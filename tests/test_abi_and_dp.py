"""CPU-side checks of the boundary: the shared library loads without a GPU
and exports every symbol the header declares; no-device behaviour; the
data-parallel sharding and loss reduction with world_size-2 gloo ranks."""
import ctypes as C
import os
import re
import subprocess
import sys

import numpy as np
import pytest

from ullis_b200 import cuda, dp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    text = open(os.path.join(ROOT, "include", "ullis_cuda.h")).read()
    return re.findall(r"ULLIS_CUDA_API\s+[\w\s\*]+?\b(ullis_cuda_\w+)\(", text)


def test_library_exports_every_declared_symbol():
    lib = cuda.load_library()
    names = header_symbols()
    assert len(names) >= 35 and set(names) == set(cuda.ABI_SYMBOLS)
    for name in names:
        assert getattr(lib, name) is not None


def test_no_device_means_error_not_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    with pytest.raises(cuda.UllisCudaError) as e:
        cuda.CudaRuntime(0)
    assert e.value.code == cuda.ERR_CUDA and "requires a CUDA device" in e.value.message
    lib = cuda.load_library()
    assert lib.ullis_cuda_layer_norm(None, None, None, None, None, C.c_size_t(1), C.c_size_t(1)) == cuda.ERR_ARG


def test_product_sources_do_not_reference_the_oracle():
    for base, _, files in os.walk(os.path.join(ROOT, "ullis_b200")):
        for f in files:
            if f.endswith((".py", ".cu", ".cpp", ".hpp", ".cuh")):
                text = open(os.path.join(base, f)).read()
                assert not re.search(r"import oracle|from oracle|from \.\.? *oracle|libullis_oracle|\buo_\w+\(|oracle/",
                                     text), f


def test_shard_range_covers_every_sequence_once():
    for n in (0, 1, 7, 64, 65):
        for world in (1, 2, 3, 4, 8):
            spans = [dp.shard_range(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        dp.shard_range(4, 2, 2)


def test_global_mean_is_sum_over_sum():
    assert dp.global_mean([(10.0, 4), (2.0, 1)]) == 12.0 / 5
    assert dp.global_mean([(0.0, 0)]) == 0.0


_WORKER = r"""
import os, sys
sys.path.insert(0, {root!r})
import numpy as np, torch.distributed as dist
from ullis_b200 import dp, synth
from oracle import oracle as O
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo", rank=rank, world_size=world)
data = synth.heron_checkpoint("tiny", batch_size=4)
m = O.HeronOracle(data)
B, T = 3, 32
tokens = synth.uniform_tokens(5, B * T, 512)
labels = tokens.copy(); labels[7] = 3; labels[40] = 3
tok, lab, nb = dp.shard_tokens(tokens, labels, T, rank, world)
if nb:
    mean, n_valid, row_loss, _ = m.forward_ce(tok, lab, 3, nb, T)
    part = (float(row_loss.astype(np.float64).sum()), n_valid)
else:
    part = (0.0, 0)
total, n, mean_all = dp.reduce_loss_torch(*part)
if rank == 0:
    full_mean, full_n, full_rl, _ = m.forward_ce(tokens, labels, 3, B, T)
    assert n == full_n, (n, full_n)
    assert abs(mean_all - float(full_rl.astype(np.float64).sum()) / full_n) < 1e-9
    assert abs(mean_all - full_mean) < 1e-5
    print("DP_OK", n, mean_all)
dist.destroy_process_group()
"""


def test_two_rank_gloo_sharding_matches_single_process(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(_WORKER.format(root=ROOT))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29517", WORLD_SIZE="2", OMP_NUM_THREADS="2")
    procs = [subprocess.Popen([sys.executable, str(script)], env=dict(env, RANK=str(r)), stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=300)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), outs
    assert "DP_OK" in outs[0]


def test_parent_handles_close_their_children_first():
    """Runtime -> model -> state handles borrow one another in the C library, and a
    garbage collection that finds the Python objects unreachable together finalises
    them in no particular order: closing a parent destroys its children first, once each."""
    from ullis_b200 import cuda
    calls = []
    rt = cuda._Handle(1, lambda h: calls.append(("runtime", h)))
    model = cuda._Handle(2, lambda h: calls.append(("model", h)), rt)
    train = cuda._Handle(3, lambda h: calls.append(("train", h)), model)
    gen = cuda._Handle(4, lambda h: calls.append(("generate", h)), model)
    gone = cuda._Handle(5, lambda h: calls.append(("generate", h)), model)
    gone.close()                     # a state that was dropped earlier
    assert calls == [("generate", 5)]
    rt.close()                       # the runtime's finaliser happened to run first
    assert calls[1:] == [("train", 3), ("generate", 4), ("model", 2), ("runtime", 1)]
    for h in (train, gen, model, rt):   # the others' finalisers then find nothing left to do
        h.close()
    assert len(calls) == 5 and rt.h is None and model.h is None
    # closed children are dropped from the parent's list when the next one registers
    rt2 = cuda._Handle(1, lambda h: None)
    for i in range(50):
        cuda._Handle(10 + i, lambda h: None, rt2).close()
    assert len(rt2.children) <= 1


def test_rendezvous_gives_up_when_a_rank_never_joins(tmp_path):
    """The failure is made on the host: rank 1 simply never announces itself.  Rank 0 must get
    ERR_TIMEOUT from the rendezvous - before any NCCL or CUDA call - instead of waiting in the bootstrap."""
    import threading
    import time
    t0 = time.perf_counter()
    with pytest.raises(cuda.UllisCudaError) as e:
        cuda.CudaRuntime.dp_rendezvous(str(tmp_path), "lonely", 0, 2, timeout_s=0.3)
    assert e.value.code == cuda.ERR_TIMEOUT and "rank 1 of 2 never arrived" in e.value.message
    assert 0.25 <= time.perf_counter() - t0 < 5.0
    # both ranks present (the second one late, but inside the deadline): both calls return
    errors = []

    def rank(r, delay):
        try:
            time.sleep(delay)
            cuda.CudaRuntime.dp_rendezvous(str(tmp_path), "pair", r, 2, timeout_s=10.0)
        except Exception as exc:  # noqa: BLE001
            errors.append(exc)

    threads = [threading.Thread(target=rank, args=(0, 0.0)), threading.Thread(target=rank, args=(1, 0.2))]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors
    with pytest.raises(cuda.UllisCudaError) as e:      # arguments are checked
        cuda.CudaRuntime.dp_rendezvous(str(tmp_path), "x", 2, 2)
    assert e.value.code == cuda.ERR_ARG
