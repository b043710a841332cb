"""The allocation-free A'A entry point (fitre_syrk_tn_static_scratch) against the existing
G-factor entry point (fitre_kfac_lambda_delta), through the C ABI.

Who needs it: callers that cannot allocate device memory -- a driver that gave all free memory
to its own workspace, code issued between stream-capture calls, threads kept off the
allocator.  The entry point keeps its split-sum slabs in an array built into the library, so
the test calls it twice in a row (the second call finds the first call's leftovers in the
array) and checks both results.  Collected last on purpose: a failure here cannot hide the
other tests in a run that stops at the first failure.
"""
import ctypes as C

import numpy as np
import pytest

import nets
from fitre_b200 import _structs as S

pytestmark = pytest.mark.gpu
TOL = 1e-10


def test_static_scratch_syrk_matches_kfac_g_factors_twice():
    import torch
    import gpu_util as G
    from fitre_b200 import api, _lib
    L = _lib.load()
    n = 6
    model = nets.vgg_small(n)
    api.finalize(model)
    x, y, w, v, ncls = G.synth(model, n, seed=123)
    run = G.GpuRun(model, x, y, w, ncls)
    info = api.computeKFACStorageIndices(model)
    need = L.fitre_kfac_mem_required(C.byref(model))
    scratch = G.dev(np.zeros(need))
    Gref = G.dev(np.zeros(info.LambdaGSize))
    api.computeLambdaDelta(run.c, model, run.ws.dx, n, Gref, info, scratch)
    Gref = Gref.cpu().numpy()
    torch.cuda.synchronize()
    for attempt in range(2):
        for l in range(model.cLayers):
            c = model.convLayer[l]
            rows = n * c.outHeight * c.outWidth
            off = model.zOffsets[l + 1] + (c.batchNormOffset if c.batchNorm else c.activationOffset)
            out = torch.full((c.outChannels * c.outChannels,), float("nan"), dtype=torch.float64,
                             device="cuda")
            a_ptr = run.ws.dx.data_ptr() + 8 * off
            rc = L.fitre_syrk_tn_static_scratch(C.c_void_p(a_ptr), rows, c.outChannels, rows,
                                                float(rows), C.c_void_p(out.data_ptr()), None)
            assert rc == S.OK
            torch.cuda.synchronize()
            g0, g1 = info.LambdaGOffsets[l], info.LambdaGOffsets[l + 1]
            assert G.relmax(out.cpu().numpy(), Gref[g0:g1]) < TOL, (attempt, l)


def test_static_scratch_syrk_rejects_oversize():
    import torch
    from fitre_b200 import _lib
    L = _lib.load()
    a = torch.zeros(16, dtype=torch.float64, device="cuda")
    rc = L.fitre_syrk_tn_static_scratch(C.c_void_p(a.data_ptr()), 4, 1025, 4, 1.0,
                                        C.c_void_p(a.data_ptr()), None)
    assert rc == S.ERR_TOO_LARGE
