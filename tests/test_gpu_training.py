"""GPU parity tests of the training-loop pieces either side of the gradient / Hv path: minibatch
assembly (bit-exact index and byte arithmetic), running batch-norm statistics and the accuracy
modes, the accuracy count, the generalisation sweeps and the FITRE outer loop, each against the
CPU oracle on the same seeded inputs."""
import ctypes as C

import numpy as np
import pytest

import nets
import oracle_lib as O
from fitre_b200 import _structs as S
from fitre_b200 import layout
from test_training_oracle import images, loop_params, small_problem

pytestmark = pytest.mark.gpu
TOL = 1e-10


def full_dataset(G, api, model, trainX, trainY, testX, testY, w, batch):
    c0 = model.convLayer[0]
    feat = c0.inChannels * c0.height * c0.width
    W = G.dev(w)
    return api.make_full_dataset(W, G.dev(trainX), G.dev(trainY),
                                 None if testX is None else G.dev(testX),
                                 None if testY is None else G.dev(testY), 10, feat, batch), W


def test_cuda_prepare_minibatch_bit_exact():
    import torch
    import gpu_util as G
    from fitre_b200 import api
    c = G.ctx()
    rng = np.random.default_rng(21)
    for (ch, h, w_), n_set, n in (((3, 8, 8), 40, 7), ((3, 32, 32), 64, 16), ((3, 16, 16), 9, 9)):
        model = nets.vgg_small(n, hw=h) if h != 32 else nets.vgg11(n)
        api.finalize(model)
        imgs = images(rng, n_set, ch, h, w_)
        setX, setY = imgs.reshape(n_set, -1).ravel(), rng.integers(1, 11, n_set).astype(np.float64)
        perm = rng.permutation(n_set).astype(np.int32)
        data, _ = full_dataset(G, api, model, setX, setY, None, None, np.zeros(model.pSize), n)
        X, Y = G.dev(setX), G.dev(setY)
        idx = torch.tensor(perm, dtype=torch.int32, device="cuda")
        for off, aug in ((0, False), (n_set - n, True), (1 if n_set > n else 0, True)):
            u = rng.random(3 * n) if aug else None
            U = G.dev(u) if aug else None
            api.prepareMinibatch(c, model, data, X, Y, idx, off, n, U)
            torch.cuda.synchronize()
            keep = data._keep[5]
            got = keep[n * ch * h * w_:2 * n * ch * h * w_].cpu().numpy()
            assert data.currentBatch == keep.data_ptr() + 8 * n * ch * h * w_
            want, lab = O.prepare_minibatch(setX, setY, perm, off, n, ch, h, w_, 10, u)
            assert np.array_equal(got, want)
            assert np.array_equal(data._keep[6].cpu().numpy(), lab)
        # contiguous slice without an index vector
        api.prepareMinibatch(c, model, data, X, Y, None, 0, n, None)
        got = data._keep[5][n * ch * h * w_:2 * n * ch * h * w_].cpu().numpy()
        assert np.array_equal(got, O.prepare_minibatch(setX, setY, None, 0, n, ch, h, w_)[0])


@pytest.mark.parametrize("builder,n", [("vgg_small", 6), ("alexnet_small", 8)])
def test_cuda_running_statistics_and_accuracy_modes(builder, n):
    import torch
    import gpu_util as G
    from fitre_b200 import api
    model = getattr(nets, builder)(n)
    O.finalize(model)
    x, y, w, v, ncls = G.synth(model, n, seed=41)
    c = G.ctx()
    ws = api.Workspace(model, ncls)
    data = api.make_dataset(G.dev(w), G.dev(x), G.dev(y), ncls)
    ws.z.zero_()
    api.initBatchNormData(c, model, ws.z)
    zo = np.zeros(model.zSize)
    O.lib().ora_init_batch_norm_data(C.byref(model), zo)
    po, eo = np.zeros(n * ncls), np.zeros(max(model.maxDeltaSize, n * ncls))
    env = O.make_env()
    for _ in range(2):  # two training forwards: the running statistics accumulate
        lo = O.lib().ora_cnn_forward(C.byref(env), C.byref(model), x, y, w, ncls, zo, po, eo, n)
        lg = api.cnnForwardEval(c, model, data, ws.scratch, ws.z, ws.probs, ws.errors, n, 10)
        assert abs(lg - lo) <= TOL * abs(lo)
    z = ws.z.cpu().numpy()
    assert G.relmax(z, zo) < TOL  # the whole state, running statistics included
    for mode in (20, 30):
        env_t = O.make_env(eval_type=mode)
        lo = O.lib().ora_cnn_forward(C.byref(env_t), C.byref(model), x, y, w, ncls, zo, po, eo, n)
        lg = api.cnnForwardEval(c, model, data, ws.scratch, ws.z, ws.probs, ws.errors, n, mode)
        assert abs(lg - lo) <= TOL * abs(lo)
        assert G.relmax(ws.probs.cpu().numpy()[:n * ncls], po) < TOL
        assert G.relmax(ws.z.cpu().numpy(), zo) < TOL
        hits, acc = api.computeAccuracy(c, ws.probs, data._keep[2], n, ncls)
        h = C.c_double()
        acc_o = O.lib().ora_compute_accuracy(C.byref(env_t), po, y, n, ncls, C.byref(h))
        assert hits == h.value and acc == acc_o
    assert abs(api.evaluateCNNModel(c, model, data, ws.scratch, ws.z, ws.probs, ws.errors, 0, n)
               - O.lib().ora_cnn_forward(C.byref(env), C.byref(model), x, y, w, ncls, zo, po, eo, n)) <= TOL * abs(lo)


def test_cuda_accuracy_rule():
    import gpu_util as G
    from fitre_b200 import api
    c = G.ctx()
    probs = np.array([0.1, 0.7, 0.2, 0.4, 0.4, 0.2, 0.0, 0.0, 0.0, 0.2, 0.3, 0.5])
    target = np.array([2., 2., 1., 3.])
    assert api.computeAccuracy(c, G.dev(probs), G.dev(target), 4, 3) == (3.0, 75.0)
    rng = np.random.default_rng(2)
    p = rng.random((1000, 10))
    p /= p.sum(1, keepdims=True)
    t = rng.integers(1, 11, 1000).astype(np.float64)
    hits, acc = api.computeAccuracy(c, G.dev(p.ravel()), G.dev(t), 1000, 10)
    assert hits == float(np.sum(p.argmax(1) + 1 == t)) and acc == hits / 10.


def test_cuda_generalization_errors_vs_oracle():
    import torch
    import gpu_util as G
    from fitre_b200 import api, _lib
    rng = np.random.default_rng(11)
    model, trainX, trainY, testX, testY, w = small_problem(rng)
    c = G.ctx()
    data, _ = full_dataset(G, api, model, trainX, trainY, testX, testY, w, model.batchSize)
    ws = api.Workspace(model, 10)
    need = _lib.load().fitre_generalization_mem_required(C.byref(model))
    scr = api.make_scratch(torch.zeros(need, dtype=torch.float64, device="cuda"))
    # running statistics after one training forward on some batch
    zo = np.zeros(model.zSize)
    O.lib().ora_init_batch_norm_data(C.byref(model), zo)
    xb, yb = O.prepare_minibatch(trainX, trainY, None, 0, 8, 3, 8, 8)
    po, eo = np.zeros(80), np.zeros(max(model.maxDeltaSize, 80))
    env = O.make_env()
    O.lib().ora_cnn_forward(C.byref(env), C.byref(model), xb, yb, w, 10, zo, po, eo, 8)
    ws.z.copy_(G.dev(zo))
    for mode, setX, setY, size, test in ((30, testX, testY, 19, 1), (20, trainX, trainY, 52, 0)):
        lik, acc = C.c_double(), C.c_double()
        O.lib().ora_generalization_errors(C.byref(env), C.byref(model), setX, setY, size, 10, w, 10,
                                          zo, test, C.byref(lik), C.byref(acc))
        lg, ag = api.computeGeneralizationErrors(c, model, data, scr, ws.z, ws.probs, ws.errors, mode)
        assert abs(lg - lik.value) <= TOL * abs(lik.value)
        assert ag == acc.value
    # running statistics are still those of the model's own layout
    cl = model.convLayer[0]
    bo = model.zOffsets[1] + cl.batchNormOffset + cl.runningMeansOffset
    assert np.array_equal(ws.z.cpu().numpy()[bo:bo + 2 * cl.outChannels], zo[bo:bo + 2 * cl.outChannels])


@pytest.mark.parametrize("check_grad,enable_da,inverse_freq,solver",
                         [(1, 1, 1, 0), (0, 0, 1, 0), (1, 1, 3, 0), (1, 1, 1, 1), (1, 0, 3, 1)])
def test_cuda_trust_region_loop_vs_oracle(check_grad, enable_da, inverse_freq, solver):
    import torch
    import gpu_util as G
    from fitre_b200 import api, _lib
    rng = np.random.default_rng(12)
    model, trainX, trainY, testX, testY, w = small_problem(rng)
    c = G.ctx()
    info_o, tr_o = loop_params()
    info_o.checkGrad, info_o.inverseFreq, info_o.stats_decay = check_grad, inverse_freq, 0.81
    wo = w.copy()
    steps_o, epochs_o = O.trust_region_kfac(model, trainX, trainY, testX, testY, wo, 10, info_o, tr_o,
                                            seed=7, enable_da=enable_da, steps_cap=64)
    info_g, tr_g = loop_params()
    info_g.checkGrad, info_g.inverseFreq, info_g.stats_decay = check_grad, inverse_freq, 0.81
    data, W = full_dataset(G, api, model, trainX, trainY, testX, testY, w, model.batchSize)
    need = _lib.load().fitre_trust_region_kfac_mem_required(C.byref(model), C.byref(data), C.byref(info_g))
    scr = api.make_scratch(torch.zeros(need, dtype=torch.float64, device="cuda"))
    c.set_kfac_solver(solver)  # 1: Cholesky factors + triangular solves instead of explicit inverses
    try:
        steps_g, epochs_g = api.subsampledTrustRegionKFAC(c, model, data, info_g, tr_g, scr, seed=7,
                                                          enableDA=enable_da, stepsCap=64)
    finally:
        c.set_kfac_solver(0)
    assert len(steps_g) == len(steps_o) == 12 and tr_g.curIteration == tr_o.curIteration
    close = lambda a, b, t=1e-7: abs(a - b) <= t * max(abs(b), 1e-12)
    for sg, so in zip(steps_g, steps_o):
        assert (sg.usedKfac, sg.reverted) == (so.usedKfac, so.reverted)
        assert close(sg.trainLikelihood, so.trainLikelihood) and close(sg.newTrainLikelihood, so.newTrainLikelihood)
        assert close(sg.modelKfac, so.modelKfac, 1e-6) and close(sg.modelGradient, so.modelGradient, 1e-6)
        assert close(sg.rho, so.rho, 1e-5) and sg.delta == so.delta
        assert sg.newTrainAccuracy == so.newTrainAccuracy
    for eg, eo_ in zip(epochs_g, epochs_o):
        assert eg.miniBatches == eo_.miniBatches == 6
        assert close(eg.testLikelihood, eo_.testLikelihood) and close(eg.trainLikelihood, eo_.trainLikelihood)
        assert eg.testAccuracy == eo_.testAccuracy and eg.trainAccuracy == eo_.trainAccuracy
    assert G.rel(W.cpu().numpy(), wo) < 1e-7
    assert tr_g.delta == tr_o.delta


def test_cuda_running_average_factors_vs_oracle():
    """The speed-up variant's pieces one by one: running averages of inputs / outputs / errors over
    three minibatches and the factors computed from them."""
    import gpu_util as G
    from fitre_b200 import api, _lib
    L = _lib.load()
    n = 6
    for builder, kwargs in (("vgg_small", dict()), ("alexnet_small", dict(bias=True))):
        model = getattr(nets, builder)(n, **kwargs)
        O.finalize(model)
        info = S.KFAC_INFO()
        O.lib().ora_kfac_storage_indices(C.byref(model), C.byref(info))
        info.stats_decay = 0.49
        c0 = model.convLayer[0]
        feat = c0.inChannels * c0.height * c0.width
        dI_o, dZ_o, dL_o = np.zeros(feat * n), np.zeros(model.zztSize), np.zeros(model.zztSize)
        dI, dZ, dL = G.dev(dI_o), G.dev(dZ_o), G.dev(dL_o)
        c = G.ctx()
        for it in range(3):
            x, y, w, v, ncls = G.synth(model, n, seed=60 + it)
            st = O.gradient(model, x, y, w, ncls, n)
            run = G.GpuRun(model, x, y, w, ncls)
            O.lib().ora_kfac_speedup_omega_z(C.byref(info), C.byref(model), x, feat, n, st.z, dI_o, dZ_o, it)
            O.lib().ora_kfac_speedup_lambda_delta(C.byref(info), C.byref(model), n, st.dx, dL_o, it)
            run.data.features = feat
            c.check(L.fitre_kfac_speedup_omega_z(c.h, C.byref(info), C.byref(model), C.byref(run.data), n,
                                                 run.ws.z.data_ptr(), dI.data_ptr(), dZ.data_ptr(), it))
            c.check(L.fitre_kfac_speedup_lambda_delta(c.h, C.byref(info), C.byref(model), n,
                                                      run.ws.dx.data_ptr(), dL.data_ptr(), it))
        assert G.relmax(dI.cpu().numpy(), dI_o) < TOL and G.relmax(dZ.cpu().numpy(), dZ_o) < TOL
        assert G.relmax(dL.cpu().numpy(), dL_o) < TOL
        A_o, G_o = np.zeros(info.OmegaZSize), np.zeros(info.LambdaGSize)
        env = O.make_env()
        O.lib().ora_kfac_omega_z_damped(C.byref(env), C.byref(model), dI_o, dZ_o, n, A_o, C.byref(info))
        O.lib().ora_kfac_lambda_delta_damped(C.byref(env), C.byref(model), dL_o, n, G_o, C.byref(info))
        scr = G.dev(np.zeros(L.fitre_kfac_mem_required(C.byref(model))))
        A, Gm = G.dev(np.zeros(info.OmegaZSize)), G.dev(np.zeros(info.LambdaGSize))
        c.check(L.fitre_kfac_omega_z_damped(c.h, C.byref(model), dI.data_ptr(), dZ.data_ptr(), n, A.data_ptr(),
                                            C.byref(info), scr.data_ptr()))
        c.check(L.fitre_kfac_lambda_delta_damped(c.h, C.byref(model), dL.data_ptr(), n, Gm.data_ptr(),
                                                 C.byref(info), scr.data_ptr()))
        assert G.rel(A.cpu().numpy(), A_o) < TOL and G.rel(Gm.cpu().numpy(), G_o) < TOL
        # updateRunningStats on its own
        a, b = np.arange(10.) + 1, np.arange(10.) * 0.5
        A1 = G.dev(a)
        c.check(L.fitre_update_running_stats(c.h, A1.data_ptr(), G.dev(b).data_ptr(), 10, 0.7))
        O.lib().ora_update_running_stats(a, b, 10, 0.7)
        assert np.array_equal(A1.cpu().numpy(), a)
