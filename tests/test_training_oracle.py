"""CPU tests of the oracle's training-loop pieces: running batch-norm statistics and the accuracy
modes, the accuracy count, minibatch assembly (index arithmetic checked against a step-by-step
numpy restatement of the reference's kernel sequence), the `.params` text format, and the FITRE
outer loop's bookkeeping."""
import ctypes as C
import os

import numpy as np

import nets
import oracle_lib as O
from fitre_b200 import _structs as S
from fitre_b200 import layout

MEAN = np.array([0.4914, 0.4822, 0.4465])
STD = np.array([0.2470, 0.2435, 0.2616])


def images(rng, n, c=3, h=8, w=8):
    """n images as columns of a features x n matrix, each image [C][W][H] with byte values."""
    return rng.integers(0, 256, (n, c, w, h)).astype(np.float64)


def reference_pipeline(imgs, idx, uniforms):
    """selectColumnMatrix -> reshapeMatrix -> randomCrop -> flipData -> normalizeCIFAR10, one step
    at a time on [C][N][W][H] arrays (solvers/kfac_da.cu:22-89)."""
    n = len(idx)
    sel = imgs[idx]                                   # [N][C][W][H]
    x = np.transpose(sel, (1, 0, 2, 3)).copy()        # [C][N][W][H]
    c_, _, w_, h_ = x.shape
    if uniforms is not None:
        dr = (uniforms[:n] * 100.).astype(np.int64) % 9 - 4
        dc = (uniforms[n:2 * n] * 100.).astype(np.int64) % 9 - 4
        crop = np.zeros_like(x)
        for im in range(n):
            for col in range(w_):
                for row in range(h_):
                    sr, sc = row + dr[im], col + dc[im]
                    if 0 <= sr < h_ and 0 <= sc < w_:
                        crop[:, im, col, row] = x[:, im, sc, sr]
        flip = crop.copy()
        for im in range(n):
            if uniforms[2 * n + im] < 0.5:
                flip[:, im, :, :] = crop[:, im, ::-1, :]
        x = flip
    x = x / 255.
    for ch in range(c_):
        x[ch] = (x[ch] - MEAN[ch]) / STD[ch]
    return x.ravel()


def test_prepare_minibatch_matches_reference_kernel_sequence():
    rng = np.random.default_rng(5)
    imgs = images(rng, 40)
    setX = imgs.reshape(40, -1).ravel()               # features x samples, column per image
    setY = rng.integers(1, 11, 40).astype(np.float64)
    perm = rng.permutation(40).astype(np.int32)
    for n, off, aug in ((7, 3, False), (8, 16, True), (1, 39, True)):
        u = rng.random(3 * n) if aug else None
        got, lab = O.prepare_minibatch(setX, setY, perm, off, n, 3, 8, 8, 10, u)
        want = reference_pipeline(imgs, perm[off:off + n], u)
        assert np.array_equal(got, want)
        assert np.array_equal(lab, setY[perm[off:off + n]])
    # contiguous slice (evaluation sweeps), no index vector
    got, lab = O.prepare_minibatch(setX, setY, None, 5, 6, 3, 8, 8, 10, None)
    assert np.array_equal(got, reference_pipeline(imgs, np.arange(5, 11), None))


def test_crop_shift_and_flip_edge_values():
    """shift = trunc(u*100) % 9 - 4 covers -4..4; u = 0.5 is not flipped (strict <)."""
    rng = np.random.default_rng(6)
    imgs = images(rng, 4)
    setX, setY = imgs.reshape(4, -1).ravel(), np.ones(4)
    u = np.array([0.00, 0.04, 0.08, 0.995,     # row shifts -4, 0, 4, 99 % 9 - 4 = -4
                  0.01, 0.05, 0.13, 0.50,      # col shifts -3, 1, 13 % 9 - 4 = 0, 50 % 9 - 4 = 1
                  0.5, 0.4999, 0.0, 0.9])      # flips: no, yes, yes, no
    got, _ = O.prepare_minibatch(setX, setY, None, 0, 4, 3, 8, 8, 10, u)
    assert np.array_equal(got, reference_pipeline(imgs, np.arange(4), u))


def test_accuracy_rule():
    env = O.make_env()
    probs = np.array([0.1, 0.7, 0.2,      # class 2
                      0.4, 0.4, 0.2,      # tie: first maximum wins -> class 1
                      0.0, 0.0, 0.0,      # nothing exceeds 0 -> class 1
                      0.2, 0.3, 0.5])     # class 3
    target = np.array([2., 2., 1., 3.])
    hits = C.c_double()
    acc = O.lib().ora_compute_accuracy(C.byref(env), probs, target, 4, 3, C.byref(hits))
    assert hits.value == 3.0 and acc == 75.0


def test_running_statistics_and_accuracy_modes():
    n = 6
    model = nets.vgg_small(n)
    O.finalize(model)
    rng = np.random.default_rng(9)
    c0 = model.convLayer[0]
    x = layout.batch_to_ref(rng.standard_normal((n, c0.inChannels, c0.height, c0.width)))
    y = rng.integers(1, 11, n).astype(np.float64)
    w = layout.he_normal_params(model, rng)
    z = np.zeros(model.zSize)
    O.lib().ora_init_batch_norm_data(C.byref(model), z)
    probs, errors = np.zeros(n * 10), np.zeros(max(model.maxDeltaSize, n * 10))
    env = O.make_env()
    O.lib().ora_cnn_forward(C.byref(env), C.byref(model), x, y, w, 10, z, probs, errors, n)
    for l in range(model.cLayers):
        c = model.convLayer[l]
        b = model.zOffsets[l + 1] + c.batchNormOffset
        mean = z[b + c.meansOffset:b + c.meansOffset + c.outChannels]
        var = z[b + c.variancesOffset:b + c.variancesOffset + c.outChannels]
        rm = z[b + c.runningMeansOffset:b + c.runningMeansOffset + c.outChannels]
        rv = z[b + c.runningVariancesOffset:b + c.runningVariancesOffset + c.outChannels]
        assert np.allclose(rm, 0.1 * mean, rtol=1e-14, atol=1e-300)
        assert np.allclose(rv, 0.9 + 0.1 * var, rtol=1e-14)
    # accuracy mode: normalises with the running statistics and leaves them alone
    z2 = z.copy()
    env_t = O.make_env(eval_type=30)
    O.lib().ora_cnn_forward(C.byref(env_t), C.byref(model), x, y, w, 10, z2, probs, errors, n)
    c = model.convLayer[0]
    b = model.zOffsets[1]
    V = c.convVolumn * n
    rows = V // c.outChannels
    conv = z2[b:b + V].reshape(c.outChannels, rows)
    bo = b + c.batchNormOffset
    rm = z2[bo + c.runningMeansOffset:bo + c.runningMeansOffset + c.outChannels]
    rv = z2[bo + c.runningVariancesOffset:bo + c.runningVariancesOffset + c.outChannels]
    want = (conv - rm[:, None]) / np.sqrt(rv[:, None] + 1e-5)
    assert np.allclose(z2[bo:bo + V].reshape(c.outChannels, rows), want, rtol=1e-13, atol=1e-13)
    assert np.array_equal(rm, z[bo + c.runningMeansOffset:bo + c.runningMeansOffset + c.outChannels])


def small_problem(rng, n_train=52, n_test=19, batch=8):
    model = nets.vgg_small(batch)
    O.finalize(model)
    c0 = model.convLayer[0]
    tr = images(rng, n_train, c0.inChannels, c0.height, c0.width)
    te = images(rng, n_test, c0.inChannels, c0.height, c0.width)
    trainX, testX = tr.reshape(n_train, -1).ravel(), te.reshape(n_test, -1).ravel()
    trainY = rng.integers(1, 11, n_train).astype(np.float64)
    testY = rng.integers(1, 11, n_test).astype(np.float64)
    w = layout.he_normal_params(model, rng)
    return model, trainX, trainY, testX, testY, w


def loop_params():
    info = S.KFAC_INFO()
    info.regLambda, info.dampGamma, info.momentum, info.stats_decay = 1e-3, 1e-2, 0.5, 0.0
    info.checkGrad, info.inverseFreq = 1, 1
    tr = S.TRUST_REGION_PARAMS()
    tr.delta, tr.minDelta, tr.maxDelta, tr.maxIters = 0.1, 1e-6, 10.0, 2
    return info, tr


def test_generalization_sweep_bounds():
    """Test sweep covers every image (partial last batch included); train sweep leaves before the
    last batch but still divides by the set size (functions/cnn_accuracy.cu:76-108,138-170)."""
    rng = np.random.default_rng(11)
    model, trainX, trainY, testX, testY, w = small_problem(rng)
    z = np.zeros(model.zSize)
    O.lib().ora_init_batch_norm_data(C.byref(model), z)
    env = O.make_env()
    lik, acc = C.c_double(), C.c_double()
    O.lib().ora_generalization_errors(C.byref(env), C.byref(model), testX, testY, 19, 10, w, 10, z, 1,
                                      C.byref(lik), C.byref(acc))
    # by hand: batches 8, 8, 3 with the running statistics (mean 0, variance 1)
    tot, hits = 0.0, 0.0
    for first, n in ((0, 8), (8, 8), (16, 3)):
        m2 = nets.vgg_small(n)
        O.finalize(m2)
        z2 = np.zeros(m2.zSize)
        O.lib().ora_init_batch_norm_data(C.byref(m2), z2)
        xb, yb = O.prepare_minibatch(testX, testY, None, first, n, 3, 8, 8)
        probs, errors = np.zeros(n * 10), np.zeros(max(m2.maxDeltaSize, n * 10))
        e = O.make_env(eval_type=30)
        tot += n * O.lib().ora_cnn_forward(C.byref(e), C.byref(m2), xb, yb, w, 10, z2, probs, errors, n)
        h = C.c_double()
        O.lib().ora_compute_accuracy(C.byref(e), probs, yb, n, 10, C.byref(h))
        hits += h.value
    assert abs(lik.value - tot / 19) <= 1e-13 * abs(tot / 19)
    assert acc.value == hits * 100. / 19
    # the running statistics survive the partial batch
    c = model.convLayer[0]
    bo = model.zOffsets[1] + c.batchNormOffset
    assert np.all(z[bo + c.runningVariancesOffset:bo + c.runningVariancesOffset + c.outChannels] == 1.0)
    # train sweep: 52 images, batch 8 -> batches at 0..40 (6 batches), 48 left out
    O.lib().ora_generalization_errors(C.byref(env), C.byref(model), trainX, trainY, 52, 10, w, 10, z, 0,
                                      C.byref(lik), C.byref(acc))
    tot = 0.0
    for first in range(0, 48, 8):
        xb, yb = O.prepare_minibatch(trainX, trainY, None, first, 8, 3, 8, 8)
        probs, errors = np.zeros(80), np.zeros(max(model.maxDeltaSize, 80))
        e = O.make_env(eval_type=20)
        tot += 8 * O.lib().ora_cnn_forward(C.byref(e), C.byref(model), xb, yb, w, 10, z.copy(), probs, errors, 8)
    assert abs(lik.value - tot / 52) <= 1e-13 * abs(tot / 52)


def test_outer_loop_bookkeeping():
    rng = np.random.default_rng(12)
    model, trainX, trainY, testX, testY, w = small_problem(rng)
    info, tr = loop_params()
    w0 = w.copy()
    steps, epochs = O.trust_region_kfac(model, trainX, trainY, testX, testY, w, 10, info, tr, seed=7,
                                        steps_cap=64)
    # 52 images, batch 8: offsets 0..40 satisfy offset + 8 < 52 -> 6 minibatches per epoch
    assert [e.miniBatches for e in epochs] == [6, 6] and len(steps) == 12 == tr.curIteration
    assert not np.array_equal(w, w0) and np.all(np.isfinite(w))
    for s in steps:
        assert np.isfinite(s.rho) and 1e-6 <= s.delta <= 10.0
        assert s.usedKfac == (1 if s.modelKfac < s.modelGradient else 0)
        assert s.reverted == (1 if (s.rho < 1e-4 or s.newTrainLikelihood > 10 * s.trainLikelihood) else 0)
        assert s.modelKfac <= 0 or s.modelGradient <= 0 or s.reverted  # a descent model exists
    for e in epochs:
        assert 0 <= e.testAccuracy <= 100 and 0 <= e.trainAccuracy <= 100 and e.testLikelihood > 0
    # same seed, same run; another seed, another shuffle
    w1 = w0.copy()
    info2, tr2 = loop_params()
    steps2, _ = O.trust_region_kfac(model, trainX, trainY, testX, testY, w1, 10, info2, tr2, seed=7,
                                    steps_cap=64)
    assert np.allclose(w, w1, rtol=1e-8, atol=1e-12)  # OpenMP sums are not order-stable
    w2 = w0.copy()
    info3, tr3 = loop_params()
    O.trust_region_kfac(model, trainX, trainY, testX, testY, w2, 10, info3, tr3, seed=8, steps_cap=64)
    assert not np.allclose(w, w2, rtol=1e-4)


def test_vector_files_round_trip(tmp_path):
    from fitre_b200 import api
    rng = np.random.default_rng(3)
    v = rng.standard_normal(257) * 10.0 ** rng.integers(-8, 8, 257)
    p = os.path.join(tmp_path, "w.params")
    api.writeVector(p, v, referenceFormat=0)
    assert np.array_equal(api.readVector(p, 257), v)
    assert api.readVector(p, 100).size == 100 and api.readVector(p, 1000).size == 257
    api.writeVector(p, v, referenceFormat=1)
    lines = open(p).read().split("\n")
    assert lines[0] == "%6.10f" % v[0] and len(lines) == 258
    assert np.allclose(api.readVector(p, 257), v, atol=5.1e-11, rtol=0)


def test_outer_loop_running_average_variant():
    """inverseFreq 3: factors are refreshed on minibatches 0, 3, 6, ...; the run differs from the
    every-minibatch loop after the first minibatch and equals it on the first."""
    rng = np.random.default_rng(12)
    model, trainX, trainY, testX, testY, w = small_problem(rng)
    runs = []
    for freq in (1, 3):
        info, tr = loop_params()
        info.inverseFreq, info.stats_decay = freq, 0.81
        wi = w.copy()
        steps, _ = O.trust_region_kfac(model, trainX, trainY, testX, testY, wi, 10, info, tr, seed=7,
                                       steps_cap=64)
        runs.append((steps, wi))
    (s1, w1), (s3, w3) = runs
    assert len(s1) == len(s3) == 12
    assert abs(s1[0].modelKfac - s3[0].modelKfac) <= 1e-9 * abs(s1[0].modelKfac)
    assert any(abs(a.modelKfac - b.modelKfac) > 1e-6 * abs(a.modelKfac) for a, b in zip(s1[1:], s3[1:]))
    assert np.all(np.isfinite(w3))
