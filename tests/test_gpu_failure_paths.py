"""Failure paths of the C ABI, made on the host: non-finite inputs, a scratch area declared too
small, and the data-parallel plumbing losing a peer (stand-in NCCL library returning errors,
a set-up that never completes, a stream parked in a host function, and the real NCCL with a
peer that never joins).  No case makes a GPU fault, wait or spin; the communicator cases run in
child processes so that a helper thread left inside a library cannot hold up the test run."""
import ctypes as C
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import nets
from fitre_b200 import _structs as S

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def test_non_finite_input_returns_status_and_context_stays_usable():
    import gpu_util as G
    from fitre_b200 import api
    n = 4
    model = nets.vgg_small(n)
    api.finalize(model)
    x, y, w, v, ncls = G.synth(model, n, seed=2)
    bad = x.copy()
    bad[17] = np.nan
    with pytest.raises(api.FitreError) as e:
        G.GpuRun(model, bad, y, w, ncls)
    assert e.value.status == S.ERR_NOT_FINITE
    winf = w.copy()
    winf[3] = np.inf
    with pytest.raises(api.FitreError) as e:
        G.GpuRun(model, x, y, winf, ncls)
    assert e.value.status == S.ERR_NOT_FINITE
    run = G.GpuRun(model, x, y, w, ncls)
    assert np.isfinite(run.loss) and np.all(np.isfinite(run.gradient))


def test_truncated_scratch_returns_workspace_status():
    import gpu_util as G
    from fitre_b200 import api, _lib
    L = _lib.load()
    n = 4
    model = nets.vgg_small(n)
    api.finalize(model)
    x, y, w, v, ncls = G.synth(model, n, seed=2)
    run = G.GpuRun(model, x, y, w, ncls)
    c, ws = run.c, run.ws
    need_g = L.fitre_cnn_gradient_mem_required(C.byref(model))
    need_h = L.fitre_cnn_hv_mem_required(C.byref(model))
    need_k = L.fitre_kfac_mem_required(C.byref(model))
    info = api.computeKFACStorageIndices(model)
    A = G.dev(np.zeros(info.OmegaZSize))
    try:
        c.set_scratch_limit(need_g - 1)
        with pytest.raises(api.FitreError) as e:
            api.computeCNNGradient(c, model, run.data, ws.scratch, ws.z, ws.dx, ws.probs, ws.errors, ws.gradient, 0, n, 0.0)
        assert e.value.status == S.ERR_WORKSPACE
        c.set_scratch_limit(need_g)
        api.computeCNNGradient(c, model, run.data, ws.scratch, ws.z, ws.dx, ws.probs, ws.errors, ws.gradient, 0, n, 0.0)
        c.set_scratch_limit(need_h - 1)
        with pytest.raises(api.FitreError) as e:
            run.hv(v)
        assert e.value.status == S.ERR_WORKSPACE
        c.set_scratch_limit(need_h)
        run.hv(v)
        c.set_scratch_limit(need_k - 1)
        with pytest.raises(api.FitreError) as e:
            api.computeOmegaZ(c, model, run.data, ws.z, n, A, info, ws.dev)
        assert e.value.status == S.ERR_WORKSPACE
    finally:
        c.set_scratch_limit(0)
    api.computeOmegaZ(c, model, run.data, ws.z, n, A, info, G.dev(np.zeros(need_k)))


@pytest.fixture(scope="module")
def fake_nccl(tmp_path_factory):
    out = str(tmp_path_factory.mktemp("fake_nccl") / "libfake_nccl.so")
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    subprocess.check_call(["gcc", "-shared", "-fPIC", "-O1", "-o", out, os.path.join(HERE, "fake_nccl", "fake_nccl.c"),
                           "-I", os.path.join(cuda, "include"), "-L", os.path.join(cuda, "lib64"), "-lcudart"])
    return out


def run_worker(mode, env_extra, timeout=120):
    env = dict(os.environ, **env_extra)
    p = subprocess.Popen([sys.executable, os.path.join(HERE, "comm_failure_worker.py"), mode], env=env,
                         stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    try:
        out, err = p.communicate(timeout=timeout)
    except subprocess.TimeoutExpired:
        p.kill()
        p.communicate()
        pytest.fail("worker %s did not finish in %d s" % (mode, timeout))
    assert p.returncode == 0, err[-2000:]
    return json.loads(out.strip().splitlines()[-1])


def test_comm_setup_that_never_completes_is_bounded(fake_nccl):
    r = run_worker("fake_init_never_returns", {"FITRE_NCCL_LIBRARY": fake_nccl, "FAKE_NCCL_INIT_SLEEP": "600"})
    assert r["status"] == S.ERR_COMM and 1.5 < r["seconds"] < 10
    assert r["world_after"] == 1 and r["single_gpu_status_after"] == 0


def test_comm_async_error_aborts_and_returns_status(fake_nccl):
    r = run_worker("fake_async_error", {"FITRE_NCCL_LIBRARY": fake_nccl, "FAKE_NCCL_STALL_MS": "300",
                                        "FAKE_NCCL_ERROR_AFTER_POLLS": "3"})
    assert r["world"] == 2
    assert r["status"] == S.ERR_COMM and "asynchronous error" in r["text"]
    assert r["status_again"] == S.ERR_COMM
    assert r["aborts"] == 2 and r["destroys"] == 0      # both communicators of the context
    assert r["single_gpu_status_after"] == 0


def test_comm_stalled_collective_hits_the_deadline(fake_nccl):
    r = run_worker("fake_stalled_collective", {"FITRE_NCCL_LIBRARY": fake_nccl, "FAKE_NCCL_STALL_MS": "2500"})
    assert r["status"] == S.ERR_COMM and "did not finish" in r["text"]
    assert 0.9 < r["seconds"] < 2.4
    assert r["aborts"] == 2 and r["single_gpu_status_after"] == 0


def test_real_nccl_peer_never_joins():
    """Rank 0 of a two-rank communicator whose rank 1 never starts: NCCL's own set-up waits for
    the peer; the call must come back with FITRE_ERR_COMM after the configured bound, and the
    context must still serve single-GPU calls."""
    r = run_worker("real_peer_never_joins", {})
    assert r["status"] == S.ERR_COMM and r["seconds"] < 15
    assert r["world_after"] == 1 and r["single_gpu_status_after"] == 0


def test_peer_allreduce_kernel_wait_is_bounded():
    """The library's own small all-reduce waits on flags that other ranks raise in this rank's
    mailbox.  On one GPU: a two-rank mailbox whose second flag nothing raises; the kernel gives up
    after the limit, the call reports FITRE_ERR_COMM, and the context goes on working."""
    import time
    import gpu_util as G
    from fitre_b200 import api
    c = G.ctx()
    t0 = time.time()
    with pytest.raises(api.FitreError) as e:
        c.peer_wait_selftest(300.0)
    assert e.value.status == S.ERR_COMM
    assert 0.25 < time.time() - t0 < 5.0
    n = 4
    model = nets.vgg_small(n)
    api.finalize(model)
    x, y, w, v, ncls = G.synth(model, n, seed=2)
    run = G.GpuRun(model, x, y, w, ncls)
    assert np.isfinite(run.loss)
