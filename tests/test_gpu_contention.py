"""Bit-repeatability of the TMA-fed kernels while another stream's kernels share the SMs.

The convolution, weight-gradient and A-factor kernels recycle shared-memory stages that a TMA
unit refills; whether a refill can overtake a warp's last reads of the stage only shows when
warps are delayed, i.e. when kernels of another stream are resident on the same SM.  Here a
second context on its own stream, driven by a second host thread, inverts matrices (a stream of
GEMM, triangular-solve and Cholesky-leaf kernels) while the first context repeats the gradient and
the Hessian-vector product of VGG-11-BN; every repetition must return the bits of the first.
"""
import threading

import numpy as np
import pytest

import nets
import oracle_lib as O

pytestmark = pytest.mark.gpu


def test_gradient_and_hv_bits_repeat_beside_another_streams_kernels():
    import torch
    import gpu_util as G
    from fitre_b200 import api, _lib
    L = _lib.load()
    n = 64
    model = nets.vgg11(n)
    O.finalize(model)
    x, y, w, v, ncls = G.synth(model, n, seed=77)
    run = G.GpuRun(model, x, y, w, ncls)
    ws = run.ws
    vv = G.dev(v)

    side = torch.cuda.Stream()
    other = api.Context(torch.cuda.current_device(), stream=side.cuda_stream)
    m = 1536
    rng = np.random.default_rng(5)
    b = rng.standard_normal((m, 256))
    spd = G.dev((b @ b.T / 256 + np.eye(m)).ravel())
    inv = G.dev(np.zeros(m * m))
    scr = G.dev(np.zeros(L.fitre_kfac_inverse_mem_required(m)))
    stop = threading.Event()
    done = {"calls": 0, "error": None}

    def churn():
        try:
            while not stop.is_set():
                api.computeMatrixInverse(other, spd, inv, m, scr, 1e-3, 0.0)
                done["calls"] += 1
        except Exception as e:  # noqa: BLE001 -- reported by the main thread
            done["error"] = e

    t = threading.Thread(target=churn)
    t.start()
    try:
        first = None
        for rep in range(40):
            api.computeCNNGradient(run.c, model, run.data, ws.scratch, ws.z, ws.dx, ws.probs, ws.errors,
                                   ws.gradient, 0, n, 0.0)
            api.cnnHv(run.c, model, run.data, ws.z, ws.probs, ws.errors, ws.dx, vv, ws.hv, 0, n, ws.dev)
            torch.cuda.current_stream().synchronize()
            cur = (ws.gradient.clone(), ws.hv.clone())
            if first is None:
                first = cur
                continue
            assert torch.equal(cur[0], first[0]), "gradient bits changed at repetition %d" % rep
            assert torch.equal(cur[1], first[1]), "Hessian-vector bits changed at repetition %d" % rep
    finally:
        stop.set()
        t.join()
    assert done["error"] is None, done["error"]
    assert done["calls"] > 0  # the other stream really ran beside the passes
    side.synchronize()
    other.close()
