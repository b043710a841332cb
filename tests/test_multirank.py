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
    # ranks share the host cores: a few OpenMP threads each, sleeping (not spinning) at barriers
    env = dict(os.environ, OMP_NUM_THREADS="4", OMP_WAIT_POLICY="passive")
    procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "multirank_worker.py"), backend,
                               str(r), str(world), port, outs[r], builder], env=env)
             for r in range(world)]
    # a rank that fails or runs out of time must not leave its peers blocked in a collective:
    # on any failure every rank still running is killed and reaped before the test reports
    codes = []
    try:
        for p in procs:
            codes.append(p.wait(timeout=600))
            if codes[-1] != 0:
                break
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
        for p in procs:
            try:
                p.wait(timeout=30)
            except subprocess.TimeoutExpired:
                pass
    assert codes == [0] * world, "rank exit codes %s" % codes
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


def full_batch_inverses(builder, A, G):
    """Oracle inverses (damping 1e-3 + 1e-2) of every used factor block, in the flat layouts."""
    import ctypes as C
    import multirank_worker as W
    from fitre_b200 import _structs as S
    model = W.make_case(builder)[0]
    info = S.KFAC_INFO()
    O.lib().ora_kfac_storage_indices(C.byref(model), C.byref(info))
    Ai, Gi = np.zeros_like(A), np.zeros_like(G)
    for l in range(model.cLayers + model.lLayers):
        if l < model.cLayers:
            c = model.convLayer[l]
            kb, co = c.inChannels * c.kSize ** 2 + (1 if model.bias else 0), c.outChannels
        else:
            f = model.fcLayer[l - model.cLayers]
            kb, co = f.in_ + (1 if model.bias else 0), f.out
        for size, off, src, dst in ((kb, info.OmegaZOffsets[l], A, Ai), (co, info.LambdaGOffsets[l], G, Gi)):
            out = np.zeros(size * size)
            assert O.lib().ora_kfac_matrix_inverse(np.ascontiguousarray(src[off:off + size * size]), out,
                                                   size, 1e-3, 1e-2) == 0
            dst[off:off + size * size] = out
    return Ai, Gi


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
    Ainv, Ginv = full_batch_inverses(builder, A, G)
    for res in run_ranks("nccl", 2, tmp_path, builder):
        assert abs(float(res["loss"]) - loss) <= 1e-10 * abs(loss)
        assert rel(res["gradient"], g) < 1e-10
        assert rel(res["hv"], hv) < 1e-10
        assert rel(res["A"], A) < 1e-10 and rel(res["G"], G) < 1e-10
        # every rank holds every inverse although each computed only its share
        assert rel(res["Ainv"], Ainv) < 1e-8 and rel(res["Ginv"], Ginv) < 1e-8
        # layer-owned factors (reduced onto one rank per layer, natural gradient all-reduced) give
        # every rank the natural gradient of the replicated form, with inverses and with Cholesky solves
        assert rel(res["ng_owned"], res["ng_rep"]) < 1e-9
        assert rel(res["ng_owned_chol"], res["ng_rep"]) < 1e-8
        # the batch-norm statistics went through the library's own kernel over peer memory
        assert int(res["peer_reduce"]) == 1 and int(res["peer_launches"]) > 0
        # host-buffer entry point with ranks: bit-identical to the device-resident calls
        assert float(res["loss_host"]) == float(res["loss"])
        assert np.array_equal(res["gradient_host"], res["gradient"])
        assert np.array_equal(res["hv_host"], res["hv"])
        # ... and with result buffers shared by the ranks (each copies its share only)
        assert np.array_equal(res["gradient_shared"], res["gradient"])
        assert np.array_equal(res["hv_shared"], res["hv"])
        assert res["loss_shared"] == res["loss_host"]
        # ... and with weights and direction uploaded one chunk per rank and all-gathered
        assert np.array_equal(res["gradient_gathered"], res["gradient"])
        assert np.array_equal(res["hv_gathered"], res["hv"])
        assert res["loss_gathered"] == res["loss_host"]
        # 3xTF32 mode across ranks: stated tolerance 1e-3 against the fp64 full-batch result
        assert rel(res["gradient_x3"], g) < 1e-3 and rel(res["hv_x3"], hv) < 1e-3


def single_rank_loop():
    import multirank_worker as W
    model, trainX, trainY, testX, testY, w, info, tr = W.loop_case(8)
    steps, epochs = O.trust_region_kfac(model, trainX, trainY, testX, testY, w, 10, info, tr, seed=5,
                                        steps_cap=64)
    return W.pack_loop(steps, epochs, w)


def check_loop(res, ref, tol):
    assert res["steps"].shape == ref["steps"].shape and ref["steps"].shape[0] == 14
    # flags, accuracies and radii are exact; likelihoods, models and rho within tolerance
    assert np.array_equal(res["steps"][:, [2, 6, 7, 8]], ref["steps"][:, [2, 6, 7, 8]])
    assert np.allclose(res["steps"][:, [0, 1]], ref["steps"][:, [0, 1]], rtol=tol, atol=0)
    assert np.allclose(res["steps"][:, [3, 4, 5]], ref["steps"][:, [3, 4, 5]], rtol=100 * tol, atol=1e-12)
    assert np.array_equal(res["epochs"][:, [1, 3, 4]], ref["epochs"][:, [1, 3, 4]])
    assert np.allclose(res["epochs"][:, [0, 2]], ref["epochs"][:, [0, 2]], rtol=tol, atol=0)
    assert rel(res["w"], ref["w"]) < 10 * tol


def test_two_rank_oracle_loop_matches_single_rank(tmp_path):
    """Host-side sharding of the outer loop: two ranks with 4 images each reproduce one rank
    with 8 (same shuffle, each rank assembling its slice of every global minibatch)."""
    ref = single_rank_loop()
    for res in run_ranks("gloo", 2, tmp_path, "loop"):
        check_loop(res, ref, 1e-9)


@pytest.mark.gpu
def test_two_gpu_cuda_loop_matches_single_rank_oracle(tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    ref = single_rank_loop()
    for res in run_ranks("nccl", 2, tmp_path, "loop"):
        check_loop(res, ref, 1e-8)
