"""GPU parity tests: the CUDA library (through the C ABI) against the committed golden
fixtures and against the CPU oracle on the same seeded inputs.  Tolerance: 1e-10 relative
(fp64), both norm-wise and max-wise; integer artefacts (arg-max routing) show up as exact
agreement of the routed tensors."""
import ctypes as C
import glob
import json
import os

import numpy as np
import pytest

import nets
import oracle_lib as O
from fitre_b200 import _structs as S

pytestmark = pytest.mark.gpu

TOL = 1e-10
_ALL = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "*.npz")))
GOLDEN = [p for p in _ALL if not os.path.basename(p).startswith("kfac_")]
KFAC_GOLDEN = [p for p in _ALL if os.path.basename(p).startswith("kfac_")]
FLAGS = {"Small Residue": S.CG_CONVERGED, "Negative Curvature": S.CG_NEG_CURVATURE,
         "Hit Boundary": S.CG_HIT_BOUNDARY, "Maximum Iterations": S.CG_MAX_ITERS}


def load_case(path):
    d = np.load(path, allow_pickle=False)
    spec = json.loads(str(d["spec"]))
    model = getattr(nets, spec["builder"])(spec["batch"], **spec["kwargs"])
    return d, spec, model


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[:-4] for p in GOLDEN])
def test_cuda_matches_golden(path):
    import gpu_util as G
    d, spec, model = load_case(path)
    run = G.GpuRun(model, d["batch"], d["labels"], d["weights"], spec["classes"], ref_softmax=0)
    assert abs(run.loss - float(d["loss"])) <= TOL * abs(float(d["loss"]))
    assert G.rel(run.gradient, d["gradient"]) < TOL
    assert G.relmax(run.gradient, d["gradient"]) < TOL
    hv = run.hv(d["vector"])
    assert G.rel(hv, d["hv"]) < TOL
    assert G.relmax(hv, d["hv"]) < TOL


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[:-4] for p in GOLDEN])
def test_cuda_quadratic_model_and_cg_match_golden(path):
    import gpu_util as G
    from fitre_b200 import api
    d, spec, model = load_case(path)
    run = G.GpuRun(model, d["batch"], d["labels"], d["weights"], spec["classes"], ref_softmax=0)
    ws = run.ws
    g = ws.gradient.clone()
    v = G.dev(d["vector"])
    mval = api.computeQuadraticModel(run.c, model, run.data, ws.z, ws.probs, ws.errors, ws.dx, g, v,
                                     float(d["clip_delta"]), 0, run.n, 0.0, ws.dev)
    assert abs(mval - float(d["clip_model"])) <= 1e-9 * abs(float(d["clip_model"]))
    assert G.rel(v.cpu().numpy(), d["clip_vector"]) < 1e-9
    for tag in ("cg", "cgb", "cgw"):
        prm = S.CG_PARAMS()
        prm.delta = float(d[tag + "_delta"])
        prm.tolerance = 1e-30
        prm.maxIterations = 10
        prm.weightDecay = float(d["cgw_weight"]) if tag == "cgw" else 0.0
        p = G.dev(np.zeros(model.pSize))
        api.cgSteihaug(run.c, model, run.data, ws.z, ws.probs, ws.errors, ws.dx, g, p, run.n,
                       ws.dev, prm)
        assert prm.flag == FLAGS[str(d[tag + "_flag"])], tag
        assert prm.iterations == int(d[tag + "_iters"]), tag
        assert G.rel(p.cpu().numpy(), d[tag + "_p"]) < 1e-7, tag
        assert abs(prm.modelValue - float(d[tag + "_model"])) <= 1e-7 * abs(float(d[tag + "_model"])), tag


@pytest.mark.parametrize("path", KFAC_GOLDEN, ids=[os.path.basename(p)[:-4] for p in KFAC_GOLDEN])
def test_cuda_kfac_matches_reference_pytorch_fixtures(path):
    """A and G factors, damped inverses and natural gradient against the fixtures produced by the
    reference's own PyTorch KFAC code (pytorch/kfac/kfac_utils.py, tests/golden/make_kfac_golden.py),
    explicit-inverse and Cholesky form."""
    import gpu_util as G
    from fitre_b200 import api, _lib
    L = _lib.load()
    d, spec, model = load_case(path)
    n, ncls = spec["batch"], spec["classes"]
    run = G.GpuRun(model, d["batch"], d["labels"], d["weights"], ncls, ref_softmax=0)
    assert G.rel(run.gradient, d["gradient"]) < TOL
    ws = run.ws
    # second backward pass on the sampled labels (the fixture fixes them): errors (p - onehot) / N
    probs = ws.probs.cpu().numpy().reshape(n, ncls)
    onehot = np.zeros((n, ncls))
    onehot[np.arange(n), d["sampled_labels"].astype(int) - 1] = 1.0
    md = model.maxDeltaSize + n * ncls
    e1, e2 = G.dev(np.zeros(md)), G.dev(np.zeros(md))
    e1[:n * ncls] = G.dev(((probs - onehot) / n).reshape(-1))
    g2, dx2 = G.dev(np.zeros(model.pSize)), G.dev(np.zeros(model.zSize))
    api.cnnBackward(run.c, model, run.data, ws.dev, ws.z, g2, dx2, e1, e2, 0, n)
    info = api.computeKFACStorageIndices(model)
    info.regLambda, info.dampGamma = float(d["regLambda"]), float(d["dampGamma"])
    scratch = G.dev(np.zeros(max(L.fitre_kfac_factors_and_inverses_mem_required(C.byref(model)),
                                 L.fitre_kfac_natural_gradient_mem_required(C.byref(model)))))
    nl = model.cLayers + model.lLayers
    for solver in (0, 1):
        run.c.set_kfac_solver(solver)
        try:
            A, Gm = G.dev(np.zeros(info.OmegaZSize)), G.dev(np.zeros(info.LambdaGSize))
            Ai, Gi = G.dev(np.zeros(info.OmegaZSize)), G.dev(np.zeros(info.LambdaGSize))
            api.computeFactorsAndInverses(run.c, model, run.data, ws.z, dx2, n, A, Ai, Gm, Gi, info, scratch)
            ng = G.dev(np.zeros(model.pSize))
            api.computeNaturalGradient(run.c, model, info, Ai, Gi, ws.gradient, ng, scratch)
        finally:
            run.c.set_kfac_solver(0)
        A_h, G_h, Ai_h, Gi_h = (t.cpu().numpy() for t in (A, Gm, Ai, Gi))
        for l in range(nl):
            if l < model.cLayers:
                c = model.convLayer[l]
                kb, co = c.inChannels * c.kSize ** 2 + model.bias, c.outChannels
            else:
                f = model.fcLayer[l - model.cLayers]
                kb, co = f.in_ + model.bias, f.out
            a0, g0 = info.OmegaZOffsets[l], info.LambdaGOffsets[l]
            assert G.relmax(A_h[a0:a0 + kb * kb].reshape(kb, kb), d["A%d" % l]) < TOL, l
            assert G.relmax(G_h[g0:g0 + co * co].reshape(co, co), d["G%d" % l]) < TOL, l
            assert G.rel(Gi_h[g0:g0 + co * co].reshape(co, co), d["Ginv%d" % l]) < 1e-9, l
            if solver == 0:
                assert G.rel(Ai_h[a0:a0 + kb * kb].reshape(kb, kb), d["Ainv%d" % l]) < 1e-9, l
        assert G.rel(ng.cpu().numpy(), d["natural_gradient"]) < 1e-9, solver


def test_cuda_softmax_reference_quirks_known_answer():
    """The hand-worked two-sample, three-class case of functions/softmax_loss.cu:24-27,55 (running
    maximum starting at 0, + 1e-10 after normalising) through the CUDA forward pass: an identity
    convolution and a selecting FC layer put the chosen logits in front of the softmax."""
    import gpu_util as G
    from fitre_b200 import api
    model = S.describe_model(
        [dict(cin=1, cout=1, h=2, w=2, k=3, pad=1, bn=False, act=S.CNN_ACT_NONE, pool=None)],
        [(4, 3, S.CNN_ACT_NONE)], 2, False)
    api.finalize(model)
    w = np.zeros(model.pSize)
    w[4] = 1.0                              # centre tap: the convolution copies its input
    for o in range(3):                      # FC weights out x in column-major: logit o = pixel o
        w[model.wOffsets[1] + o * 3 + o] = 1.0
    # [C=1][N=2][W][H] with h fastest; the FC layer reads a sample as (h, w) row-major, so pixel
    # (h, w) = (0, 1) is the second logit and (1, 0) the third
    x = np.array([-1.0, -0.5, -2.5, 9.0, 2.0, -1.0, 0.5, 9.0])
    y = np.array([2.0, 1.0])
    want_p = np.array([0.3482074279837349, 0.0776955792485706, 0.5740969930676946,
                       0.7855970346892759, 0.1752903922400367, 0.03911257337068746])
    want_loss = 1.3981341074423905
    c = G.ctx(1)
    ws = api.Workspace(model, 3)
    data = api.make_dataset(G.dev(w), G.dev(x), G.dev(y), 3)
    loss = api.cnnForward(c, model, data, ws.scratch, ws.z, ws.probs, ws.errors, 0, 2)
    probs, errs = ws.probs.cpu().numpy(), ws.errors.cpu().numpy()
    assert np.abs(probs - want_p).max() < 4e-16
    assert abs(loss - want_loss) < 4e-15
    onehot = np.array([0, 1, 0, 1, 0, 0], dtype=np.float64)
    assert np.abs(errs - (want_p - onehot) / 2).max() < 4e-16
    G.ctx(0)                                # textbook softmax: the + 1e-10 is gone
    api.cnnForward(G.ctx(0), model, data, ws.scratch, ws.z, ws.probs, ws.errors, 0, 2)
    assert np.abs((probs - ws.probs.cpu().numpy()) - 1e-10).max() < 1e-15
    G.ctx(1)


def test_cuda_quadratic_model_damping_term_both_forms():
    """weightDecay != 0: the reference form (Hv + lambda * weights, functions/model_reduction.cu:50-52,
    the default) and the PyTorch twin's (Hv + lambda * v) against the oracle in the same setting."""
    import gpu_util as G
    from fitre_b200 import api
    n, lam, delta = 6, 0.3, 0.7
    model = nets.vgg_small(n)
    O.finalize(model)
    x, y, w, v, ncls = G.synth(model, n, seed=19)
    vals = {}
    for refq in (1, 0):
        env = O.make_env(ref_quadratic=refq)
        st = O.gradient(model, x, y, w, ncls, n, weight_decay=lam, env=env)
        v_o = v.copy()
        m_o = O.lib().ora_quadratic_model(C.byref(env), C.byref(model), x, w, ncls, st.z, st.probs,
                                          st.errors, st.dx, st.gradient, v_o, delta, n, lam)
        run = G.GpuRun(model, x, y, w, ncls, weight_decay=lam)
        run.c.set_reference_quadratic_damping(refq)
        try:
            vd = G.dev(v)
            ws = run.ws
            m_g = api.computeQuadraticModel(run.c, model, run.data, ws.z, ws.probs, ws.errors, ws.dx,
                                            ws.gradient, vd, delta, 0, n, lam, ws.dev)
        finally:
            run.c.set_reference_quadratic_damping(1)
        assert abs(m_g - m_o) <= 1e-10 * abs(m_o), refq
        assert G.rel(vd.cpu().numpy(), v_o) < TOL, refq
        vals[refq] = m_g
    assert vals[0] != vals[1]


CASES = [
    ("test_vgg", dict(), 7),
    ("test_vgg", dict(bn=True, act=S.CNN_ACT_SWISH), 5),
    ("lenet_small", dict(), 9),
    ("lenet_small", dict(act=S.CNN_ACT_RELU, pool=S.MAX_POOL), 9),
    ("lenet_small", dict(act=S.CNN_ACT_SOFTPLUS, bias=False), 3),
    ("alexnet_small", dict(), 8),
    ("alexnet_small", dict(bn=False, bias=True, ch=5, hw=12), 6),
    ("vgg_small", dict(), 6),
    ("vgg_small", dict(act=S.CNN_ACT_RELU, bias=True), 4),
    ("vgg_small", dict(act=S.CNN_ACT_SOFTPLUS, bn=False, hw=16), 3),
    ("lenet", dict(), 16),
    ("lenet", dict(act=S.CNN_ACT_RELU, pool=S.MAX_POOL), 16),
    ("lenet_small", dict(fc_act=S.ACT_LOGISTIC), 7),
    ("lenet_small", dict(fc_act=S.ACT_TANH, act=S.CNN_ACT_SOFTPLUS), 5),
]


@pytest.mark.parametrize("builder,kwargs,n", CASES,
                         ids=["%s-%d" % (c[0], i) for i, c in enumerate(CASES)])
def test_cuda_matches_oracle(builder, kwargs, n):
    """Same seeded inputs through the CUDA path and the oracle, reference-exact softmax;
    compares loss, gradient, Hv and the whole z / dx state (arg-max routing included)."""
    import gpu_util as G
    model = getattr(nets, builder)(n, **kwargs)
    O.finalize(model)
    x, y, w, v, ncls = G.synth(model, n, seed=100 + n)
    st = O.gradient(model, x, y, w, ncls, n, weight_decay=1e-3)
    hv_o = O.hv(model, x, w, ncls, n, st, v)
    run = G.GpuRun(model, x, y, w, ncls, ref_softmax=1, weight_decay=1e-3)
    assert abs(run.loss - st.loss) <= TOL * abs(st.loss)
    assert G.rel(run.gradient, st.gradient) < TOL
    assert G.relmax(run.gradient, st.gradient) < TOL
    hv = run.hv(v)
    assert G.rel(hv, hv_o) < TOL
    assert G.relmax(hv, hv_o) < TOL
    # stored state: everything except the running batch-norm statistics (uninitialised input)
    z = run.ws.z.cpu().numpy()
    dx = run.ws.dx.cpu().numpy()
    mask = np.ones(model.zSize, dtype=bool)
    for l in range(model.cLayers):
        c = model.convLayer[l]
        if c.batchNorm != S.NO_BATCH_NORM:
            b = model.zOffsets[l + 1] + c.batchNormOffset
            mask[b + c.runningMeansOffset:b + c.runningVariancesOffset + c.outChannels] = False
    assert G.relmax(z[mask], st.z[mask]) < TOL
    # dx: compare the slots the backward pass defines
    for l in range(model.cLayers):
        c = model.convLayer[l]
        V = c.convVolumn * n
        b = model.zOffsets[l + 1]
        for off in (0, c.activationOffset) + ((c.batchNormOffset,) if c.batchNorm else ()):
            assert G.relmax(dx[b + off:b + off + V], st.dx[b + off:b + off + V]) < TOL


def test_cuda_midsize_alexnet_and_vgg11_vs_oracle():
    import gpu_util as G
    for model, n in ((nets.alexnet(16), 16), (nets.vgg11(8), 8)):
        O.finalize(model)
        x, y, w, v, ncls = G.synth(model, n, seed=7)
        st = O.gradient(model, x, y, w, ncls, n)
        hv_o = O.hv(model, x, w, ncls, n, st, v)
        run = G.GpuRun(model, x, y, w, ncls)
        assert abs(run.loss - st.loss) <= TOL * abs(st.loss)
        assert G.rel(run.gradient, st.gradient) < TOL
        assert G.rel(run.hv(v), hv_o) < TOL


def test_cuda_kfac_factors_vs_oracle():
    import gpu_util as G
    from fitre_b200 import api, _lib
    # vgg11 at 4 images: factor sizes 576 ... 4608, the shapes the TMA-fed A-factor kernel takes
    for builder, kwargs, n in (("vgg_small", dict(), 6), ("lenet_small", dict(), 5),
                               ("alexnet_small", dict(bias=True), 4), ("vgg11", dict(), 4),
                               ("alexnet", dict(), 2)):  # 5 x 5 taps, K = 1600, through the TMA kernel
        model = getattr(nets, builder)(n, **kwargs)
        O.finalize(model)
        x, y, w, v, ncls = G.synth(model, n, seed=31)
        st = O.gradient(model, x, y, w, ncls, n)
        info = S.KFAC_INFO()
        assert O.lib().ora_kfac_storage_indices(C.byref(model), C.byref(info)) == 0
        A_o = np.zeros(info.OmegaZSize)
        G_o = np.zeros(info.LambdaGSize)
        env = O.make_env()
        O.lib().ora_kfac_omega_z(C.byref(env), C.byref(model), x, st.z, n, A_o, C.byref(info))
        O.lib().ora_kfac_lambda_delta(C.byref(env), C.byref(model), st.dx, n, G_o, C.byref(info))
        run = G.GpuRun(model, x, y, w, ncls)
        info2 = api.computeKFACStorageIndices(model)
        assert list(info2.OmegaZOffsets) == list(info.OmegaZOffsets)
        assert list(info2.LambdaGOffsets) == list(info.LambdaGOffsets)
        need = _lib.load().fitre_kfac_mem_required(C.byref(model))
        scratch = G.dev(np.zeros(need))
        A = G.dev(np.zeros(info.OmegaZSize))
        Gm = G.dev(np.zeros(info.LambdaGSize))
        api.computeOmegaZ(run.c, model, run.data, run.ws.z, n, A, info2, scratch)
        api.computeLambdaDelta(run.c, model, run.ws.dx, n, Gm, info2, scratch)
        A, Gm = A.cpu().numpy(), Gm.cpu().numpy()
        L = model.cLayers + model.lLayers
        for l in range(L):
            # used part of each A block: K' x K' with K' = K + bias
            if l < model.cLayers:
                c = model.convLayer[l]
                kb = c.inChannels * c.kSize ** 2 + (1 if model.bias else 0)
            else:
                kb = model.fcLayer[l - model.cLayers].in_ + (1 if model.bias else 0)
            a0 = info.OmegaZOffsets[l]
            assert G.relmax(A[a0:a0 + kb * kb], A_o[a0:a0 + kb * kb]) < TOL, l
            g0, g1 = info.LambdaGOffsets[l], info.LambdaGOffsets[l + 1]
            assert G.relmax(Gm[g0:g1], G_o[g0:g1]) < TOL, l
        # the gather kernel (TMA off) forms the same factors
        run.c.set_tma(0)
        try:
            A2 = G.dev(np.zeros(info.OmegaZSize))
            api.computeOmegaZ(run.c, model, run.data, run.ws.z, n, A2, info2, scratch)
        finally:
            run.c.set_tma(1)
        assert G.relmax(A2.cpu().numpy(), A) < 1e-13


def test_cuda_host_entry_point():
    import gpu_util as G
    from fitre_b200 import api
    n = 6
    model = nets.vgg_small(n)
    O.finalize(model)
    x, y, w, v, ncls = G.synth(model, n, seed=77)
    st = O.gradient(model, x, y, w, ncls, n)
    hv_o = O.hv(model, x, w, ncls, n, st, v)
    g, hv = np.zeros(model.pSize), np.zeros(model.pSize)
    c = G.ctx(1)
    for _ in range(2):  # second call reuses the context workspace
        loss = api.gradientHvHost(c, model, x, y, w, v, n, ncls, 0.0, g, hv)
        assert abs(loss - st.loss) <= TOL * abs(st.loss)
        assert G.rel(g, st.gradient) < TOL and G.rel(hv, hv_o) < TOL


def test_cuda_rejects_bad_arguments():
    import gpu_util as G
    from fitre_b200 import api
    model = nets.vgg_small(4)
    api.finalize(model)
    x, y, w, v, ncls = G.synth(model, 4, seed=1)
    run = G.GpuRun(model, x, y, w, ncls)
    with pytest.raises(api.FitreError) as e:  # partial batches are outside the path
        api.computeCNNGradient(run.c, model, run.data, run.ws.scratch, run.ws.z, run.ws.dx,
                               run.ws.probs, run.ws.errors, run.ws.gradient, 0, 3, 0.0)
    assert e.value.status == S.ERR_BAD_ARG
    bad = nets.vgg_small(4)
    bad.convLayer[0].stride = 2
    api.finalize(bad)
    with pytest.raises(api.FitreError) as e:
        G.GpuRun(bad, x, y, w, ncls)
    assert e.value.status == S.ERR_UNSUPPORTED


def test_cuda_full_size_properties_vgg11():
    """VGG-11-BN at 512 images (the benchmark shape), where the oracle is too slow:
    Hv is linear and symmetric, and the directional derivative and curvature along the
    gradient direction agree with central differences of the loss."""
    import torch
    import gpu_util as G
    n = 512
    model = nets.vgg11(n)
    O.finalize(model)
    x, y, w, v1, ncls = G.synth(model, n, seed=3234)
    v2 = np.random.default_rng(9).standard_normal(model.pSize)
    run = G.GpuRun(model, x, y, w, ncls, ref_softmax=0)
    h1, h2 = run.hv(v1), run.hv(v2)
    h12 = run.hv(0.3 * v1 - 1.7 * v2)
    assert G.rel(h12, 0.3 * h1 - 1.7 * h2) < 1e-9
    s12, s21 = v1.dot(h2), v2.dot(h1)
    assert abs(s12 - s21) <= 1e-8 * max(abs(s12), abs(s21))
    g, f0 = run.gradient.copy(), run.loss
    d = g / np.linalg.norm(g)          # steepest-ascent direction: g.d = |g| is well scaled
    dHd = d.dot(run.hv(d))
    del run
    torch.cuda.empty_cache()
    h = 1e-4
    rp = G.GpuRun(model, x, y, w + h * d, ncls, ref_softmax=0)
    fp = rp.loss
    del rp
    torch.cuda.empty_cache()
    rm = G.GpuRun(model, x, y, w - h * d, ncls, ref_softmax=0)
    fm = rm.loss
    del rm
    torch.cuda.empty_cache()
    fd_g = (fp - fm) / (2 * h)
    assert abs(fd_g - g.dot(d)) <= 1e-4 * abs(g.dot(d)), (fd_g, g.dot(d))
    # curvature along d from the loss alone (a component-wise difference of gradients is
    # dominated by max-pool arg-max switches at this size and is not a usable check)
    fd_h = (fp - 2 * f0 + fm) / (h * h)
    assert abs(fd_h - dHd) <= 2e-2 * abs(dHd), (fd_h, dHd)


def test_cuda_distribution_errors_and_sampled_backward_vs_oracle():
    """KFAC's second backward pass: labels sampled from the model's distribution (injected
    uniforms), errors, then cnnBackward on them; sampled labels must be identical."""
    import gpu_util as G
    from fitre_b200 import api
    n = 12
    model = nets.vgg_small(n)
    O.finalize(model)
    x, y, w, v, ncls = G.synth(model, n, seed=41)
    u = np.random.default_rng(4238).random(n)
    u[0], u[1] = 0.0, 1.0 - 1e-16  # edges of the inverse CDF
    st = O.gradient(model, x, y, w, ncls, n)
    env = O.make_env()
    t_o, e_o = np.zeros(n), np.zeros(n * ncls)
    O.lib().ora_distribution_errors(C.byref(env), st.probs, u, n, ncls, t_o, e_o)
    g_o, dx_o = np.zeros(model.pSize), np.zeros(model.zSize)
    O.lib().ora_cnn_backward(C.byref(env), C.byref(model), x, w, st.z, g_o, dx_o, e_o, n)
    run = G.GpuRun(model, x, y, w, ncls)
    ws = run.ws
    t_d, e_d = G.dev(np.zeros(n)), G.dev(np.zeros(model.maxDeltaSize + n * ncls))
    e2 = G.dev(np.zeros(model.maxDeltaSize + n * ncls))
    api.computeDistributionErrors(run.c, ws.probs, G.dev(u), t_d, e_d, n, ncls)
    assert np.array_equal(t_d.cpu().numpy(), t_o)
    assert G.relmax(e_d.cpu().numpy()[:n * ncls], e_o) < TOL
    g_d, dx_d = G.dev(np.zeros(model.pSize)), G.dev(np.zeros(model.zSize))
    api.cnnBackward(run.c, model, run.data, ws.dev, ws.z, g_d, dx_d, e_d, e2, 0, n)
    assert G.rel(g_d.cpu().numpy(), g_o) < TOL


def test_cuda_kfac_inverse_and_natural_gradient_vs_oracle():
    """Damped Cholesky inverses of every factor and the natural gradient G^-1 [W|b] A^-1.
    The inverse is compared to the oracle's and by its residual; tolerance 1e-9 (two different
    factorisation orders on matrices with condition number up to ~1e4)."""
    import gpu_util as G
    from fitre_b200 import api, _lib
    L = _lib.load()
    lam, gamma = 1e-3, 1e-2
    for builder, kwargs, n in (("vgg_small", dict(), 6), ("alexnet_small", dict(bias=True, ch=6), 4)):
        model = getattr(nets, builder)(n, **kwargs)
        O.finalize(model)
        x, y, w, v, ncls = G.synth(model, n, seed=55)
        run = G.GpuRun(model, x, y, w, ncls)
        info = api.computeKFACStorageIndices(model)
        need = max(L.fitre_kfac_mem_required(C.byref(model)), L.fitre_kfac_inverse_mem_required(512),
                   L.fitre_kfac_natural_gradient_mem_required(C.byref(model)))
        scratch = G.dev(np.zeros(need))
        A, Gm = G.dev(np.zeros(info.OmegaZSize)), G.dev(np.zeros(info.LambdaGSize))
        api.computeOmegaZ(run.c, model, run.data, run.ws.z, n, A, info, scratch)
        api.computeLambdaDelta(run.c, model, run.ws.dx, n, Gm, info, scratch)
        Ai, Gi = G.dev(np.zeros(info.OmegaZSize)), G.dev(np.zeros(info.LambdaGSize))
        A_h, G_h = A.cpu().numpy(), Gm.cpu().numpy()
        Ai_o, Gi_o = np.zeros(info.OmegaZSize), np.zeros(info.LambdaGSize)
        nl = model.cLayers + model.lLayers
        for l in range(nl):
            if l < model.cLayers:
                c = model.convLayer[l]
                kb, co = c.inChannels * c.kSize ** 2 + (1 if model.bias else 0), c.outChannels
            else:
                f = model.fcLayer[l - model.cLayers]
                kb, co = f.in_ + (1 if model.bias else 0), f.out
            for size, off, src, dst, dst_o, src_h in ((kb, info.OmegaZOffsets[l], A, Ai, Ai_o, A_h),
                                                      (co, info.LambdaGOffsets[l], Gm, Gi, Gi_o, G_h)):
                api.computeMatrixInverse(run.c, src[off:off + size * size], dst[off:off + size * size],
                                         size, scratch, lam, gamma)
                blk = np.ascontiguousarray(src_h[off:off + size * size])
                out = np.zeros(size * size)
                assert O.lib().ora_kfac_matrix_inverse(blk, out, size, lam, gamma) == 0
                dst_o[off:off + size * size] = out
                got = dst[off:off + size * size].cpu().numpy()
                assert G.relmax(got, out) < 1e-9, (builder, l, size)
                M = blk.reshape(size, size) + (lam + gamma) * np.eye(size)
                assert np.abs(M @ got.reshape(size, size) - np.eye(size)).max() < 1e-9
        # the same inverses in one call (several streams)
        info.regLambda, info.dampGamma = lam, gamma
        Ai2, Gi2 = G.dev(np.zeros(info.OmegaZSize)), G.dev(np.zeros(info.LambdaGSize))
        scr2 = G.dev(np.zeros(L.fitre_kfac_invert_factors_mem_required(C.byref(model))))
        api.invertFactors(run.c, model, info, A, Ai2, Gm, Gi2, scr2)
        assert np.array_equal(Ai2.cpu().numpy(), Ai.cpu().numpy())
        assert np.array_equal(Gi2.cpu().numpy(), Gi.cpu().numpy())
        ng = G.dev(np.zeros(model.pSize))
        api.computeNaturalGradient(run.c, model, info, Ai, Gi, run.ws.gradient, ng, scratch)
        ng_o = np.zeros(model.pSize)
        O.lib().ora_natural_gradient(C.byref(model), C.byref(info), Ai_o, Gi_o, run.gradient, ng_o)
        assert G.rel(ng.cpu().numpy(), ng_o) < 1e-8
        # Cholesky-solve form: factors instead of inverses in the A slots, same natural gradient
        run.c.set_kfac_solver(1)
        try:
            Ac, Gi3 = G.dev(np.zeros(info.OmegaZSize)), G.dev(np.zeros(info.LambdaGSize))
            api.invertFactors(run.c, model, info, A, Ac, Gm, Gi3, scr2)
            assert np.array_equal(Gi3.cpu().numpy(), Gi.cpu().numpy())
            ng_c = G.dev(np.zeros(model.pSize))
            api.computeNaturalGradient(run.c, model, info, Ac, Gi3, run.ws.gradient, ng_c, scratch)
        finally:
            run.c.set_kfac_solver(0)
        assert G.rel(ng_c.cpu().numpy(), ng_o) < 1e-8


def test_cuda_cholesky_solve_natural_gradient_large_blocks():
    """The Cholesky-solve form on VGG-11's factor sizes (27 ... 4608: every level of the blocked
    factorisation and of the recursive triangular solves).  Checked three ways: L L' reproduces the
    damped factor; the natural gradient equals LAPACK's solves on the host (1e-9); and it equals
    the explicit-inverse form of the same library (1e-9)."""
    import gpu_util as G
    from fitre_b200 import api, _lib
    L = _lib.load()
    n = 2
    model = nets.vgg11(n)
    O.finalize(model)
    x, y, w, v, ncls = G.synth(model, n, seed=77)
    run = G.GpuRun(model, x, y, w, ncls)
    info = api.computeKFACStorageIndices(model)
    info.regLambda, info.dampGamma = 1e-3, 1e-2
    damp = info.regLambda + info.dampGamma
    scratch = G.dev(np.zeros(max(L.fitre_kfac_mem_required(C.byref(model)),
                                 L.fitre_kfac_invert_factors_mem_required(C.byref(model)),
                                 L.fitre_kfac_natural_gradient_mem_required(C.byref(model)))))
    A, Gm = G.dev(np.zeros(info.OmegaZSize)), G.dev(np.zeros(info.LambdaGSize))
    api.computeOmegaZ(run.c, model, run.data, run.ws.z, n, A, info, scratch)
    api.computeLambdaDelta(run.c, model, run.ws.dx, n, Gm, info, scratch)
    Ai, Gi = G.dev(np.zeros(info.OmegaZSize)), G.dev(np.zeros(info.LambdaGSize))
    api.invertFactors(run.c, model, info, A, Ai, Gm, Gi, scratch)
    ng_inv = G.dev(np.zeros(model.pSize))
    api.computeNaturalGradient(run.c, model, info, Ai, Gi, run.ws.gradient, ng_inv, scratch)
    run.c.set_kfac_solver(1)
    try:
        Ac, Gi2 = G.dev(np.zeros(info.OmegaZSize)), G.dev(np.zeros(info.LambdaGSize))
        api.invertFactors(run.c, model, info, A, Ac, Gm, Gi2, scratch)
        ng = G.dev(np.zeros(model.pSize))
        api.computeNaturalGradient(run.c, model, info, Ac, Gi2, run.ws.gradient, ng, scratch)
        # the same sequence launched kernel by kernel instead of replayed from the captured graph
        run.c.set_graphs(0)
        Ac2, Gi3 = G.dev(np.zeros(info.OmegaZSize)), G.dev(np.zeros(info.LambdaGSize))
        api.invertFactors(run.c, model, info, A, Ac2, Gm, Gi3, scratch)
        ng2 = G.dev(np.zeros(model.pSize))
        api.computeNaturalGradient(run.c, model, info, Ac2, Gi3, run.ws.gradient, ng2, scratch)
        run.c.set_graphs(1)
        assert np.array_equal(Ac2.cpu().numpy(), Ac.cpu().numpy())
        assert np.array_equal(ng2.cpu().numpy(), ng.cpu().numpy())
        # replay (second call with the same buffers) gives the same bits as the capture run
        api.invertFactors(run.c, model, info, A, Ac, Gm, Gi2, scratch)
        api.computeNaturalGradient(run.c, model, info, Ac, Gi2, run.ws.gradient, ng, scratch)
        assert np.array_equal(Ac2.cpu().numpy(), Ac.cpu().numpy())
        assert np.array_equal(ng2.cpu().numpy(), ng.cpu().numpy())
    finally:
        run.c.set_graphs(1)
        run.c.set_kfac_solver(0)
    # factors and factorisations in one overlapped call: the same bits as the separate calls
    fscr = G.dev(np.zeros(L.fitre_kfac_factors_and_inverses_mem_required(C.byref(model))))
    for solver, want in ((0, Ai), (1, Ac)):
        run.c.set_kfac_solver(solver)
        try:
            A3, G3 = G.dev(np.zeros(info.OmegaZSize)), G.dev(np.zeros(info.LambdaGSize))
            Ai3, Gi4 = G.dev(np.zeros(info.OmegaZSize)), G.dev(np.zeros(info.LambdaGSize))
            for _ in range(2):  # capture, then replay
                api.computeFactorsAndInverses(run.c, model, run.data, run.ws.z, run.ws.dx, n, A3, Ai3, G3, Gi4,
                                              info, fscr)
        finally:
            run.c.set_kfac_solver(0)
        assert np.array_equal(A3.cpu().numpy(), A.cpu().numpy())
        assert np.array_equal(G3.cpu().numpy(), Gm.cpu().numpy())
        assert np.array_equal(Ai3.cpu().numpy(), want.cpu().numpy())
        assert np.array_equal(Gi4.cpu().numpy(), Gi.cpu().numpy())
    g_h, ng_h = run.ws.gradient.cpu().numpy(), ng.cpu().numpy()
    for l in range(model.cLayers):
        c = model.convLayer[l]
        K, co = c.inChannels * c.kSize ** 2, c.outChannels
        a0, g0 = info.OmegaZOffsets[l], info.LambdaGOffsets[l]
        Al = A[a0:a0 + K * K].cpu().numpy().reshape(K, K) + damp * np.eye(K)
        Lc = np.tril(Ac[a0:a0 + K * K].cpu().numpy().reshape(K, K).T)  # column-major slot
        assert np.abs(Lc @ Lc.T - Al).max() <= 1e-12 * np.abs(Al).max() * K, l
        Gl = Gm[g0:g0 + co * co].cpu().numpy().reshape(co, co) + damp * np.eye(co)
        Wg = g_h[model.wOffsets[l]:model.wOffsets[l] + K * co].reshape(co, K)  # row o = column o of K x Cout
        ref = np.linalg.solve(Gl, np.linalg.solve(Al, Wg.T).T)
        got = ng_h[model.wOffsets[l]:model.wOffsets[l] + K * co].reshape(co, K)
        assert G.rel(got, ref) < 1e-9, l
    assert G.rel(ng_h, ng_inv.cpu().numpy()) < 1e-9


def test_cuda_two_call_factor_step_same_bits_as_one_call():
    """fitre_kfac_omega_z_begin / fitre_kfac_lambda_delta_finish around the sampled-label backward
    pass (the A side runs underneath it on the library's own streams) against
    fitre_kfac_factors_and_inverses after it: identical factors, inverses and Cholesky factors, on
    the first call (graph capture) and on the replay, and the scratch of the pass in between is
    left alone."""
    import gpu_util as G
    from fitre_b200 import api, _lib
    L = _lib.load()
    for model, n in ((nets.vgg11(2), 2), (nets.vgg_small(6), 6), (nets.alexnet_small(4, bias=True), 4)):
        O.finalize(model)
        x, y, w, v, ncls = G.synth(model, n, seed=91)
        run = G.GpuRun(model, x, y, w, ncls)
        ws = run.ws
        info = api.computeKFACStorageIndices(model)
        info.regLambda, info.dampGamma = 1e-3, 1e-2
        u = G.dev(np.random.default_rng(5).random(n))
        md = model.maxDeltaSize + n * ncls
        fscr = G.dev(np.zeros(L.fitre_kfac_factors_and_inverses_mem_required(C.byref(model))))
        kscr = G.dev(np.zeros(max(L.fitre_kfac_mem_required(C.byref(model)), ws.dev.numel())))

        def sampled_backward():
            t, e1, e2 = G.dev(np.zeros(n)), G.dev(np.zeros(md)), G.dev(np.zeros(md))
            api.computeDistributionErrors(run.c, ws.probs, u, t, e1, n, ncls)
            g2, dx2 = G.dev(np.zeros(model.pSize)), G.dev(np.zeros(model.zSize))
            api.cnnBackward(run.c, model, run.data, kscr, ws.z, g2, dx2, e1, e2, 0, n)
            return g2, dx2

        for solver in (0, 1):
            run.c.set_kfac_solver(solver)
            try:
                g_ref, dx_ref = sampled_backward()
                A1, G1, Ai1, Gi1 = (G.dev(np.zeros(k)) for k in (info.OmegaZSize, info.LambdaGSize) * 2)
                api.computeFactorsAndInverses(run.c, model, run.data, ws.z, dx_ref, n, A1, Ai1, G1, Gi1, info, fscr)
                for _ in range(2):  # capture, then replay
                    A2, G2, Ai2, Gi2 = (G.dev(np.zeros(k)) for k in (info.OmegaZSize, info.LambdaGSize) * 2)
                    api.computeOmegaZBegin(run.c, model, run.data, ws.z, n, A2, Ai2, info, fscr)
                    g2, dx2 = sampled_backward()
                    api.computeLambdaDeltaFinish(run.c, model, dx2, n, G2, Gi2, info, fscr)
                    assert np.array_equal(g2.cpu().numpy(), g_ref.cpu().numpy())
                    assert np.array_equal(dx2.cpu().numpy(), dx_ref.cpu().numpy())
                    for a, b in ((A1, A2), (G1, G2), (Ai1, Ai2), (Gi1, Gi2)):
                        assert np.array_equal(a.cpu().numpy(), b.cpu().numpy()), solver
            finally:
                run.c.set_kfac_solver(0)
        # the finish call without its begin call is refused
        with pytest.raises(api.FitreError) as e:
            api.computeLambdaDeltaFinish(run.c, model, dx_ref, n, G1, Gi1, info, fscr)
        assert e.value.status == S.ERR_BAD_ARG
        del run


def test_cuda_matrix_inverse_blocked_sizes_and_failure():
    """Sizes that exercise the blocked path (several 64-blocks, ragged last block) and the
    not-positive-definite status."""
    import gpu_util as G
    from fitre_b200 import api, _lib
    L = _lib.load()
    c = G.ctx()
    rng = np.random.default_rng(3)
    for n in (1, 64, 65, 128, 200, 333, 1000, 2600):  # 2600: the 128 x 128 GEMM tiles take over
        B = rng.standard_normal((n, n + 8))
        F = B @ B.T / n
        scratch = G.dev(np.zeros(L.fitre_kfac_inverse_mem_required(n)))
        out = G.dev(np.zeros(n * n))
        api.computeMatrixInverse(c, G.dev(F.reshape(-1)), out, n, scratch, 1e-3, 0.1)
        ref = np.linalg.inv(F + 0.101 * np.eye(n))
        assert G.relmax(out.cpu().numpy().reshape(n, n), ref) < 1e-9, n
    # the Cholesky form of a block: L L' reproduces the damped matrix, every size class
    for n in (1, 63, 64, 65, 200, 257, 333, 1000):
        B = rng.standard_normal((n, n + 8))
        F = B @ B.T / n
        out = G.dev(np.zeros(n * n))
        api.computeMatrixFactor(c, G.dev(F.reshape(-1)), out, n, 1e-3, 0.1)
        Lf = np.tril(out.cpu().numpy().reshape(n, n).T)
        ref = F + 0.101 * np.eye(n)
        assert np.abs(Lf @ Lf.T - ref).max() < 1e-12 * np.abs(ref).max() * max(n, 8), n
        assert np.abs(Lf - np.linalg.cholesky(ref)).max() < 1e-10 * np.abs(ref).max(), n
    with pytest.raises(api.FitreError) as e:
        api.computeMatrixFactor(c, G.dev(-np.eye(70).reshape(-1)), G.dev(np.zeros(4900)), 70, 0.0, 0.0)
    assert e.value.status == S.ERR_NOT_CONVERGED
    with pytest.raises(api.FitreError) as e:
        api.computeMatrixInverse(c, G.dev(-np.eye(70).reshape(-1)), G.dev(np.zeros(4900)), 70,
                                 G.dev(np.zeros(L.fitre_kfac_inverse_mem_required(70))), 0.0, 0.0)
    assert e.value.status == S.ERR_NOT_CONVERGED


def test_cuda_reduced_precision_modes_within_stated_tolerance():
    """Opt-in modes: convolution forward / data-gradient / weight-gradient products on the tcgen05
    tensor cores (fp32 accumulation), everything else fp64.  Stated tolerances against the fp64 oracle,
    relative and norm-wise:
      mode 2 (error-compensated 3 x TF32): 1e-3 for loss, gradient and Hessian-vector product;
      mode 1 (one TF32 product): 1e-3 for the loss, 1e-1 for gradient and Hessian-vector
      product (batch norm and the backward sweep amplify the 3e-4 rounding of each product)."""
    import gpu_util as G
    TOL = {2: (1e-3, 1e-3), 1: (1e-3, 1e-1)}
    c = G.ctx()
    try:
        # a net whose layers exercise the expander-free kernel with 64-wide and ragged channel tiles
        # and the tensor-core weight gradient (channels 32 / 64 / 96, average pooling, 5x5 and 3x3)
        wide = S.describe_model(
            [dict(cin=3, cout=32, h=8, w=8, k=3, pad=1, bn=True, act=S.CNN_ACT_SWISH, pool=None),
             dict(cin=32, cout=64, h=8, w=8, k=5, pad=2, bn=True, act=S.CNN_ACT_SWISH, pool=(S.AVG_POOL, 2, 2, 0)),
             dict(cin=64, cout=96, h=4, w=4, k=3, pad=1, bn=True, act=S.CNN_ACT_SOFTPLUS, pool=(S.AVG_POOL, 2, 2, 0))],
            [(96 * 2 * 2, 10, S.CNN_ACT_NONE)], 16, True)
        for model, n in ((nets.vgg_small(6), 6), (nets.alexnet_small(8, ch=8), 8), (nets.vgg11(8), 8), (wide, 16)):
            O.finalize(model)
            x, y, w, v, ncls = G.synth(model, n, seed=17)
            st = O.gradient(model, x, y, w, ncls, n)
            hv_o = O.hv(model, x, w, ncls, n, st, v)
            for mode in (2, 1):
                tol_loss, tol_grad = TOL[mode]
                c.set_precision(mode)
                run = G.GpuRun(model, x, y, w, ncls)
                hv = run.hv(v)
                eg, eh = G.rel(run.gradient, st.gradient), G.rel(hv, hv_o)
                assert abs(run.loss - st.loss) <= tol_loss * abs(st.loss), (mode, run.loss, st.loss)
                assert eg < tol_grad and eh < tol_grad, (mode, eg, eh)
                # the mode really is reduced precision on these nets (not a silent fp64 fallback)
                assert eg > 1e-11, (mode, eg)
                c.set_precision(0)
                del run
    finally:
        c.set_precision(0)


def test_cuda_int8_tensor_core_fp64_mode_within_1e_10():
    """Opt-in mode 3: convolution products from base-128 digit planes on the int8 tensor cores with
    exact int32 digit sums, recombined in fp64.  Stated tolerance against the fp64 oracle: the
    default mode's own 1e-10, norm-wise and max-wise."""
    import gpu_util as G
    wide = S.describe_model(
        [dict(cin=3, cout=64, h=8, w=8, k=3, pad=1, bn=True, act=S.CNN_ACT_SWISH, pool=None),
         dict(cin=64, cout=64, h=8, w=8, k=5, pad=2, bn=True, act=S.CNN_ACT_SWISH, pool=(S.MAX_POOL, 2, 2, 0)),
         dict(cin=64, cout=96, h=4, w=4, k=3, pad=1, bn=True, act=S.CNN_ACT_SOFTPLUS, pool=(S.AVG_POOL, 2, 2, 0))],
        [(96 * 2 * 2, 10, S.CNN_ACT_NONE)], 16, True)
    c = G.ctx()
    try:
        for model, n in ((nets.vgg11(8), 8), (wide, 16)):
            O.finalize(model)
            x, y, w, v, ncls = G.synth(model, n, seed=23)
            st = O.gradient(model, x, y, w, ncls, n)
            hv_o = O.hv(model, x, w, ncls, n, st, v)
            c.set_precision(3)
            run = G.GpuRun(model, x, y, w, ncls)
            hv = run.hv(v)
            c.set_precision(0)
            assert abs(run.loss - st.loss) <= TOL * abs(st.loss)
            eg, eh = G.rel(run.gradient, st.gradient), G.rel(hv, hv_o)
            assert eg < TOL and eh < TOL, (eg, eh)
            assert G.relmax(run.gradient, st.gradient) < TOL and G.relmax(hv, hv_o) < TOL
            # the integer path really ran (the fp64 kernels agree with the oracle to ~1e-14)
            assert eg > 2e-13, eg
            del run
    finally:
        c.set_precision(0)
