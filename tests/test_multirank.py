"""Data-parallel sharding: two ranks each hold half of a batch; after the sum all-reduces
(batch-norm statistics inside the passes, then gradient / Hv / loss) every rank must hold the
full-batch result.  CPU: gloo + the oracle (host-side sharding logic).  GPU: NCCL + the CUDA
library on 2 GPUs (skipped when fewer are visible)."""
import os
import socket
import subprocess
import sys

import numpy as np
import pytest

import oracle_lib as O

HERE = os.path.dirname(os.path.abspath(__file__))


def free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return str(p)


def run_ranks(backend, world, tmp_path, builder):
    port = free_port()
    outs = [str(tmp_path / ("r%d.npz" % r)) for r in range(world)]
    procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "multirank_worker.py"), backend,
                               str(r), str(world), port, outs[r], builder]) for r in range(world)]
    for p in procs:
        assert p.wait(timeout=600) == 0
    return [np.load(o) for o in outs]


def full_batch_reference(builder):
    import multirank_worker as W
    model, x, y, w, v, ncls = W.make_case(builder)
    st = O.gradient(model, x, y, w, ncls, W.N_GLOBAL)
    hv = O.hv(model, x, w, ncls, W.N_GLOBAL, st, v)
    import ctypes as C
    from fitre_b200 import _structs as S
    info = S.KFAC_INFO()
    O.lib().ora_kfac_storage_indices(C.byref(model), C.byref(info))
    A, G = np.zeros(info.OmegaZSize), np.zeros(info.LambdaGSize)
    env = O.make_env()
    O.lib().ora_kfac_omega_z(C.byref(env), C.byref(model), x, st.z, W.N_GLOBAL, A, C.byref(info))
    O.lib().ora_kfac_lambda_delta(C.byref(env), C.byref(model), st.dx, W.N_GLOBAL, G, C.byref(info))
    return st.loss, st.gradient, hv, A, G


def rel(a, b):
    return np.linalg.norm(a - b) / np.linalg.norm(b)


@pytest.mark.parametrize("builder", ["vgg_small", "lenet_small"])
def test_two_rank_oracle_matches_full_batch(tmp_path, builder):
    loss, g, hv, A, G = full_batch_reference(builder)
    for res in run_ranks("gloo", 2, tmp_path, builder):
        assert abs(float(res["loss"]) - loss) <= 1e-12 * abs(loss)
        assert rel(res["gradient"], g) < 1e-12
        assert rel(res["hv"], hv) < 1e-12
        assert rel(res["A"], A) < 1e-12 and rel(res["G"], G) < 1e-12


@pytest.mark.gpu
@pytest.mark.parametrize("builder", ["vgg_small", "alexnet_small"])
def test_two_gpu_cuda_matches_full_batch(tmp_path, builder):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    loss, g, hv, A, G = full_batch_reference(builder)
    for res in run_ranks("nccl", 2, tmp_path, builder):
        assert abs(float(res["loss"]) - loss) <= 1e-10 * abs(loss)
        assert rel(res["gradient"], g) < 1e-10
        assert rel(res["hv"], hv) < 1e-10
        assert rel(res["A"], A) < 1e-10 and rel(res["G"], G) < 1e-10
