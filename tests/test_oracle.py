"""CPU tests that pin the oracle: golden fixtures, the reference's known-answer vectors,
offset tables, index maps and the Taylor derivative test (utilities/cnn_derivative_test.cu)."""
import ctypes as C
import glob
import json
import os

import numpy as np
import pytest

import nets
import oracle_lib as O
from fitre_b200 import _structs as S
from fitre_b200 import layout

_ALL = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "*.npz")))
GOLDEN = [p for p in _ALL if not os.path.basename(p).startswith("kfac_")]
KFAC_GOLDEN = [p for p in _ALL if os.path.basename(p).startswith("kfac_")]
FLAGS = {"Small Residue": S.CG_CONVERGED, "Negative Curvature": S.CG_NEG_CURVATURE,
         "Hit Boundary": S.CG_HIT_BOUNDARY, "Maximum Iterations": S.CG_MAX_ITERS}


def rel(a, b):
    return np.linalg.norm(np.asarray(a) - np.asarray(b)) / max(np.linalg.norm(b), 1e-300)


def load_case(path):
    d = np.load(path, allow_pickle=False)
    spec = json.loads(str(d["spec"]))
    model = getattr(nets, spec["builder"])(spec["batch"], **spec["kwargs"])
    O.finalize(model)
    return d, spec, model


def test_fixtures_present():
    assert len(GOLDEN) >= 7 and len(KFAC_GOLDEN) >= 3


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[:-4] for p in GOLDEN])
def test_gradient_hv_match_golden(path):
    d, spec, model = load_case(path)
    n, ncls = spec["batch"], spec["classes"]
    env = O.make_env(ref_softmax=0)
    st = O.gradient(model, d["batch"], d["labels"], d["weights"], ncls, n, env=env)
    assert abs(st.loss - float(d["loss"])) <= 1e-12 * abs(float(d["loss"]))
    assert rel(st.gradient, d["gradient"]) < 1e-12
    hv = O.hv(model, d["batch"], d["weights"], ncls, n, st, d["vector"], env=env)
    assert rel(hv, d["hv"]) < 1e-12


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[:-4] for p in GOLDEN])
def test_quadratic_model_and_cg_match_golden(path):
    d, spec, model = load_case(path)
    n, ncls = spec["batch"], spec["classes"]
    env = O.make_env(ref_softmax=0)
    st = O.gradient(model, d["batch"], d["labels"], d["weights"], ncls, n, env=env)
    L = O.lib()
    v = d["vector"].copy()
    mval = L.ora_quadratic_model(C.byref(env), C.byref(model), d["batch"], d["weights"], ncls,
                                 st.z, st.probs, st.errors, st.dx, st.gradient, v,
                                 float(d["clip_delta"]), n, 0.0)
    assert abs(mval - float(d["clip_model"])) <= 1e-10 * abs(float(d["clip_model"]))
    assert rel(v, d["clip_vector"]) < 1e-10
    for tag, wd in (("cg", 0.0), ("cgb", 0.0), ("cgw", None)):
        prm = S.CG_PARAMS()
        prm.delta = float(d[tag + "_delta"])
        prm.tolerance = 1e-30
        prm.maxIterations = 10
        prm.weightDecay = float(d["cgw_weight"]) if wd is None else wd
        p = np.zeros(model.pSize)
        L.ora_cg_steihaug(C.byref(env), C.byref(model), d["batch"], d["weights"], ncls, st.z,
                          st.probs, st.errors, st.dx, st.gradient, p, n, C.byref(prm))
        assert prm.flag == FLAGS[str(d[tag + "_flag"])], tag
        assert prm.iterations == int(d[tag + "_iters"]), tag
        assert rel(p, d[tag + "_p"]) < 1e-8, tag
        assert abs(prm.modelValue - float(d[tag + "_model"])) <= 1e-8 * abs(float(d[tag + "_model"])), tag


def test_batch_norm_backward_known_answer():
    # inputs and expected output: pytorch/testing/batchnorm_derivative.py:6-36, my.out:9
    err = np.array([-0.6080235940, 0.0599059907, 0.4858675772, 0.0622500264])
    zout = np.array([0.8759333415, -1.0024917965, 1.0906678043, -0.9641093493])
    var = np.array([0.0003580263])
    expected = np.array([-30.29323517, 1.51922096, 27.07121368, 1.70280053])
    out = np.zeros(4)
    env = O.make_env()
    O.lib().ora_batch_norm_backward(C.byref(env), err, 1, 1, 1, 4, var, zout, 1e-5, out)
    assert np.allclose(out, expected, rtol=0, atol=5e-8)


def test_batch_norm_rop_backward_known_inputs():
    # inputs: pytorch/testing/batchnorm_rop.py:9-20; expected value = the two terms that
    # script derives (its last line adds the unscaled first factor; the terms are what the
    # CUDA code sums, functions/dev_batch_norm.cu:787-960)
    m, eps = 4, 1e-5
    mean, var = np.array([0.8285777243]), np.array([0.0004594150])
    zin = np.array([0.8644751360, 0.8250697742, 0.8099140393, 0.8148519478])
    zout = np.array([1.6568555953, -0.1619104702, -0.8614278725, -0.6335172527])
    rzin = np.array([1.5819700810, 1.0040864902, 0.9148101685, 1.0778613252])
    rzout = np.array([1.3013500693, -4.6440685046, -0.7928236666, 4.1355421018])
    err = np.array([-0.2559813623, 0.1206990214, 0.0599662929, 0.0753160484])
    rerr = np.array([0.4685278021, -0.6415989045, -0.0878175082, 0.2608886103])
    err_in = m * err - err.sum() - zout * err.dot(zout)
    r1 = -(1. / (m * m)) / pow(var[0] + eps, 1.5) * ((zin - mean[0]) * (rzin - rzin.mean())).sum()
    r2 = m * rerr - rerr.sum() - rzout * err.dot(zout) - zout * (rerr.dot(zout) + rzout.dot(err))
    expected = r1 * err_in + r2 / (m * np.sqrt(var[0] + eps))
    rd = rerr.copy()
    env = O.make_env()
    O.lib().ora_rop_batch_norm_backward(C.byref(env), zin, zout, rzin, rzout, err, rd, eps, mean,
                                        var, 1, 1, 1, 4)
    assert np.allclose(rd, expected, rtol=1e-12, atol=1e-12)


def test_lenet_offsets_match_reference_log():
    # pytorch/kfac/cifar_kfac_trust_iteration.txt:12-13 (LeNet with bias, pSize 62006)
    model = nets.lenet(8)
    O.finalize(model)
    expected = [0, 450, 456, 2856, 2872, 50872, 50992, 61072, 61156, 61996, 62006]
    got = []
    for l in range(5):
        got += [model.wOffsets[l], model.bOffsets[l]]
    got.append(model.pSize)
    assert got == expected


def test_vgg11_sizes():
    model = nets.vgg11(2)
    O.finalize(model)
    assert model.pSize == 9222848  # 9.22 M parameters without bias
    model = nets.alexnet(2)
    O.finalize(model)
    assert model.pSize == 1755712


def test_zoffsets_layout_vgg_style():
    model = nets.vgg_small(4)
    O.finalize(model)
    c = model.convLayer[0]
    V = 4 * 8 * 8 * 8
    assert (c.batchNormOffset, c.meansOffset, c.variancesOffset) == (V, V, V + 8)
    assert c.activationOffset == 2 * V + 32 and c.poolOffset == 3 * V + 32
    assert c.outputOffset == c.poolOffset
    assert model.zOffsets[2] == 3 * V + 32 + V // 4
    c1 = model.convLayer[1]
    assert c1.outputOffset == c1.activationOffset  # no pool


def test_im2col_index_map():
    # row r = n*Ho*Wo + wo*Ho + ho, column q = cin*k*k + j*k + i (functions/dev_image.cu:20-49)
    N, Cc, H, W, k, pad = 2, 3, 5, 4, 3, 1
    Ho, Wo = H + 2 * pad - k + 1, W + 2 * pad - k + 1
    M, K = N * Ho * Wo, Cc * k * k
    idx = np.zeros(M * K, dtype=np.int64)
    O.lib().ora_im2col_index(N, Cc, H, W, k, pad, 1, idx)
    idx = idx.reshape(K, M)
    for cin in range(Cc):
        for j in range(k):
            for i in range(k):
                for n in range(N):
                    for wo in range(Wo):
                        for ho in range(Ho):
                            h, w = ho - pad + i, wo - pad + j
                            exp = -1
                            if 0 <= h < H and 0 <= w < W:
                                exp = ((cin * N + n) * W + w) * H + h
                            assert idx[cin * k * k + j * k + i, n * Ho * Wo + wo * Ho + ho] == exp
    x = np.random.default_rng(0).standard_normal(Cc * N * W * H)
    cols = np.zeros(M * K)
    O.lib().ora_im2col(x, N, Cc, H, W, k, pad, 1, cols)
    ref = np.where(idx.reshape(-1) >= 0, x[np.maximum(idx.reshape(-1), 0)], 0.0)
    assert np.array_equal(cols, ref)


def test_max_pool_argmax_tie_rule_and_window():
    # window start (k-1)*stride + ksize - 2*pad and first-maximum-in-column-major-scan
    # (functions/dev_pool.cu:363,374-391); 3/2/1 pooling on a constant plane: every window
    # must pick its first valid element in column-major order.
    N, Cc, H, W = 1, 1, 6, 6
    act = np.zeros(Cc * N * H * W)
    am = np.zeros(3 * 3, dtype=np.int32)
    O.lib().ora_max_pool_argmax(act, N, Cc, H, W, 3, 2, 1, am)
    am = am.reshape(3, 3)  # [wp][hp]
    for l in range(3):
        for k in range(3):
            r0, c0 = max(2 * k - 1, 0), max(2 * l - 1, 0)
            assert am[l, k] == c0 * H + r0


def test_layout_round_trip():
    model = nets.lenet_small(3)
    O.finalize(model)
    rng = np.random.default_rng(5)
    flat = rng.standard_normal(model.pSize)
    assert np.array_equal(layout.params_to_ref(model, layout.params_from_ref(model, flat)), flat)
    x = rng.standard_normal((3, 3, 16, 16))
    assert np.array_equal(layout.batch_from_ref(layout.batch_to_ref(x), 3, 3, 16, 16), x)


@pytest.mark.parametrize("builder,kwargs", [
    ("lenet_small", {}), ("vgg_small", {}), ("alexnet_small", {}),
    ("vgg_small", dict(act=S.CNN_ACT_SOFTPLUS, bias=True)),
    ("lenet_small", dict(fc_act=S.ACT_LOGISTIC)), ("lenet_small", dict(fc_act=S.ACT_TANH)),
])
def test_taylor_derivative(builder, kwargs):
    # utilities/cnn_derivative_test.cu:48-235: first-order remainder O(|d|^2),
    # second-order remainder O(|d|^3) along a random direction.
    n = 4
    model = getattr(nets, builder)(n, **kwargs)
    O.finalize(model)
    rng = np.random.default_rng(11)
    c0 = model.convLayer[0]
    ncls = model.fcLayer[model.lLayers - 1].out
    x = layout.batch_to_ref(rng.standard_normal((n, c0.inChannels, c0.height, c0.width)))
    y = rng.integers(1, ncls + 1, n).astype(np.float64)
    w = layout.he_normal_params(model, rng)
    d0 = rng.standard_normal(model.pSize)
    d0 /= np.linalg.norm(d0)
    env = O.make_env(ref_softmax=0)  # the +1e-10 quirk makes g an inexact gradient
    st = O.gradient(model, x, y, w, ncls, n, env=env)
    hd = O.hv(model, x, w, ncls, n, st, d0, env=env)
    f0, g = st.loss, st.gradient
    e2, e3, hs = [], [], []
    for k in range(6, 12):
        h = 0.5 ** k
        f1 = O.gradient(model, x, y, w + h * d0, ncls, n, env=env).loss
        e2.append(abs(f1 - f0 - h * g.dot(d0)))
        e3.append(abs(f1 - f0 - h * g.dot(d0) - 0.5 * h * h * d0.dot(hd)))
        hs.append(h)
    # halving the step must divide the remainders by 4 and 8 (median over the halvings: a
    # max-pool arg-max can switch inside the largest steps)
    q2 = np.median([e2[i] / e2[i + 1] for i in range(len(e2) - 1)])
    q3 = np.median([e3[i] / e3[i + 1] for i in range(len(e3) - 1)])
    assert 3.6 < q2 < 4.5, (q2, e2)
    assert 6.5 < q3 < 9.5, (q3, e3)


def test_reference_softmax_quirk_is_small_but_present():
    model = nets.test_vgg(5)
    O.finalize(model)
    rng = np.random.default_rng(2)
    x = layout.batch_to_ref(rng.standard_normal((5, 2, 4, 4)))
    y = rng.integers(1, 11, 5).astype(np.float64)
    w = layout.he_normal_params(model, rng)
    a = O.gradient(model, x, y, w, 10, 5, env=O.make_env(ref_softmax=1))
    b = O.gradient(model, x, y, w, 10, 5, env=O.make_env(ref_softmax=0))
    r = rel(a.gradient, b.gradient)
    assert 0 < r < 1e-8
    assert np.all(a.probs >= 1e-10)


def test_kfac_inverse_and_natural_gradient_host():
    """(F + damping)^-1 against numpy, and G^-1 [W|b] A^-1 against a direct numpy statement."""
    import ctypes as C
    rng = np.random.default_rng(8)
    n = 37
    B = rng.standard_normal((n, 2 * n))
    F = B @ B.T / (2 * n)
    inv = np.zeros(n * n)
    assert O.lib().ora_kfac_matrix_inverse(np.ascontiguousarray(F.T).reshape(-1), inv, n, 1e-3, 0.05) == 0
    ref = np.linalg.inv(F + (1e-3 + 0.05) * np.eye(n))
    assert np.allclose(inv.reshape(n, n).T, ref, rtol=1e-10, atol=1e-12)
    bad = -np.eye(n)
    assert O.lib().ora_kfac_matrix_inverse(bad.reshape(-1).copy(), inv, n, 0.0, 0.0) == 1
    model = nets.lenet_small(4)
    O.finalize(model)
    info = S.KFAC_INFO()
    O.lib().ora_kfac_storage_indices(C.byref(model), C.byref(info))
    Ainv = rng.standard_normal(info.OmegaZSize)
    Ginv = rng.standard_normal(info.LambdaGSize)
    g = rng.standard_normal(model.pSize)
    ng = np.zeros(model.pSize)
    O.lib().ora_natural_gradient(C.byref(model), C.byref(info), Ainv, Ginv, g, ng)
    # layer 1 (conv 6->16, 5x5, with bias): W is K x Cout column-major, bias follows
    c = model.convLayer[1]
    K, Co = c.inChannels * 25, c.outChannels
    Wm = g[model.wOffsets[1]:model.wOffsets[1] + K * Co].reshape(Co, K)      # [o][q]
    Wb = np.concatenate([Wm, g[model.bOffsets[1]:model.bOffsets[1] + Co][:, None]], axis=1)
    A = Ainv[info.OmegaZOffsets[1]:info.OmegaZOffsets[1] + (K + 1) ** 2].reshape(K + 1, K + 1).T
    Gm = Ginv[info.LambdaGOffsets[1]:info.LambdaGOffsets[1] + Co * Co].reshape(Co, Co).T
    exp = Gm @ Wb @ A
    assert np.allclose(ng[model.wOffsets[1]:model.wOffsets[1] + K * Co].reshape(Co, K), exp[:, :K])
    assert np.allclose(ng[model.bOffsets[1]:model.bOffsets[1] + Co], exp[:, K])


def kfac_layer_sizes(model, l):
    """(rows of the A block incl. the bias column, rows of the G block) of layer l."""
    if l < model.cLayers:
        c = model.convLayer[l]
        return c.inChannels * c.kSize ** 2 + model.bias, c.outChannels
    f = model.fcLayer[l - model.cLayers]
    return f.in_ + model.bias, f.out


@pytest.mark.parametrize("path", KFAC_GOLDEN, ids=[os.path.basename(p)[:-4] for p in KFAC_GOLDEN])
def test_kfac_factors_inverses_natural_gradient_match_reference_pytorch(path):
    """The fixtures were produced by the reference's own PyTorch KFAC code
    (pytorch/kfac/kfac_utils.py: matmulOmega, matmul3d, matmulLambda, computeMatVec) run on CPU:
    they pin the factor scalings 1/N, 1/(Ho Wo), N Ho Wo and N, the bias column, the damping
    (lambda + gamma) I and the order G^-1 [W|b] A^-1 of the oracle's restatement of
    solvers/kfac_inverses.cu:450-630,759-857 and solvers/kfac_natural_gradient.cu:36-241."""
    d, spec, model = load_case(path)
    n, ncls = spec["batch"], spec["classes"]
    L = O.lib()
    env = O.make_env(ref_softmax=0)
    st = O.gradient(model, d["batch"], d["labels"], d["weights"], ncls, n, env=env)
    assert rel(st.gradient, d["gradient"]) < 1e-12
    # the second backward pass of KFAC is a backward pass on other labels
    st_s = O.gradient(model, d["batch"], d["sampled_labels"], d["weights"], ncls, n, env=env)
    info = S.KFAC_INFO()
    assert L.ora_kfac_storage_indices(C.byref(model), C.byref(info)) == 0
    A, G = np.zeros(info.OmegaZSize), np.zeros(info.LambdaGSize)
    L.ora_kfac_omega_z(C.byref(env), C.byref(model), d["batch"], st.z, n, A, C.byref(info))
    L.ora_kfac_lambda_delta(C.byref(env), C.byref(model), st_s.dx, n, G, C.byref(info))
    lam, gam = float(d["regLambda"]), float(d["dampGamma"])
    Ai, Gi = np.zeros(info.OmegaZSize), np.zeros(info.LambdaGSize)
    for l in range(model.cLayers + model.lLayers):
        kb, co = kfac_layer_sizes(model, l)
        a0, g0 = info.OmegaZOffsets[l], info.LambdaGOffsets[l]
        a, g = A[a0:a0 + kb * kb].reshape(kb, kb), G[g0:g0 + co * co].reshape(co, co)
        assert d["A%d" % l].shape == (kb, kb) and d["G%d" % l].shape == (co, co)
        assert rel(a, d["A%d" % l]) < 1e-12, l       # symmetric: row / column major agree
        assert rel(g, d["G%d" % l]) < 1e-12, l
        ai, gi = np.zeros(kb * kb), np.zeros(co * co)
        assert L.ora_kfac_matrix_inverse(np.ascontiguousarray(a.reshape(-1)), ai, kb, lam, gam) == 0
        assert L.ora_kfac_matrix_inverse(np.ascontiguousarray(g.reshape(-1)), gi, co, lam, gam) == 0
        assert rel(ai.reshape(kb, kb), d["Ainv%d" % l]) < 1e-9, l
        assert rel(gi.reshape(co, co), d["Ginv%d" % l]) < 1e-9, l
        Ai[a0:a0 + kb * kb], Gi[g0:g0 + co * co] = ai, gi
    ng = np.zeros(model.pSize)
    L.ora_natural_gradient(C.byref(model), C.byref(info), Ai, Gi, st.gradient, ng)
    assert rel(ng, d["natural_gradient"]) < 1e-9


def test_softmax_reference_quirks_known_answer():
    """functions/softmax_loss.cu:24-27,55 and :231-245, worked by hand for two samples of three
    classes.  Sample 1 has only negative logits: the running maximum starts at 0, so nothing is
    subtracted and e = exp(z) itself; sample 2 is shifted by its largest logit 2.  Every
    probability then gets + 1e-10; loss = mean of -log p_label; errors = (p - onehot) / N."""
    logits = np.array([-1.0, -2.5, -0.5, 2.0, 0.5, -1.0])      # [classes x N] column-major
    target = np.array([2.0, 1.0])
    want_p = np.array([0.3482074279837349, 0.0776955792485706, 0.5740969930676946,
                       0.7855970346892759, 0.1752903922400367, 0.03911257337068746])
    want_loss = 1.3981341074423905
    # the same by the formula, written out
    e1 = np.exp(np.array([-1.0, -2.5, -0.5]) - 0.0)
    e2 = np.exp(np.array([2.0, 0.5, -1.0]) - 2.0)
    by_formula = np.concatenate([e1 / e1.sum() + 1e-10, e2 / e2.sum() + 1e-10])
    assert np.abs(by_formula - want_p).max() < 1e-15
    assert abs(by_formula.sum() - (2.0 + 6e-10)) < 1e-14        # rows sum to 1 + 3e-10, not 1
    env = O.make_env(ref_softmax=1)
    probs = np.zeros(6)
    loss = O.lib().ora_softmax_loss(C.byref(env), logits, target, 2, 3, probs)
    assert np.abs(probs - want_p).max() < 2e-16
    assert abs(loss - want_loss) < 1e-15
    # textbook softmax (quirks off) differs by exactly the 1e-10 shift
    env0 = O.make_env(ref_softmax=0)
    probs0 = np.zeros(6)
    O.lib().ora_softmax_loss(C.byref(env0), logits, target, 2, 3, probs0)
    assert np.abs((probs - probs0) - 1e-10).max() < 1e-15


def test_quadratic_model_damping_term_reference_and_pytorch_forms():
    """functions/model_reduction.cu:50-52 adds weightDecay * weights to Hv before v'Hv;
    pytorch/peng/utils.py:77 adds weightDecay * v.  Both forms against the formulas written out."""
    n = 5
    model = nets.vgg_small(n)
    O.finalize(model)
    rng = np.random.default_rng(8)
    c0 = model.convLayer[0]
    x = layout.batch_to_ref(rng.standard_normal((n, c0.inChannels, c0.height, c0.width)))
    y = rng.integers(1, 11, n).astype(np.float64)
    w = layout.he_normal_params(model, rng)
    v = rng.standard_normal(model.pSize)
    lam, delta = 0.3, 0.7
    for refq in (1, 0):
        env = O.make_env(ref_quadratic=refq)
        st = O.gradient(model, x, y, w, 10, n, weight_decay=lam, env=env)
        hv = O.hv(model, x, w, 10, n, st, v, env=env) + lam * (w if refq else v)
        vHv, nrm, gv = hv.dot(v), np.linalg.norm(v), st.gradient.dot(v)
        alpha = delta / nrm if vHv < 0 else min(gv / (vHv + 1e-6), delta / (nrm + 1e-16))
        want = 0.5 * vHv * alpha * alpha - gv * alpha
        vv = v.copy()
        got = O.lib().ora_quadratic_model(C.byref(env), C.byref(model), x, w, 10, st.z, st.probs,
                                          st.errors, st.dx, st.gradient, vv, delta, n, lam)
        assert abs(got - want) <= 1e-12 * abs(want)
        assert rel(vv, alpha * v) < 1e-13
