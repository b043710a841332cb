"""Bit-exact GPU checks of the integer work on the path: the im2col gather of the convolution
kernels and the arg-max routing of max pooling.

Every case runs the CUDA library through the C ABI on integer-valued tensors, so that all sums
are sums of integers far below 2^53 and therefore exact in fp64 whatever the summation order:
any difference from the oracle is an indexing difference, and the comparison is
numpy.array_equal, not a tolerance.

  functions/dev_image.cu:20-49        im2col row / column / padding rule
  functions/dev_backprop_convolution.cu:60-97  tap flip and bounds of the data gradient
  functions/dev_pool.cu:363,374-391   pooling window start and first-maximum tie rule
"""
import ctypes as C

import numpy as np
import pytest

import oracle_lib as O
from fitre_b200 import _structs as S

pytestmark = pytest.mark.gpu


def _forward(model, x, y, w, ncls):
    """fitre_cnn_forward on numpy inputs; returns (context, workspace, dataset)."""
    import gpu_util as G
    from fitre_b200 import api
    api.finalize(model)
    c = G.ctx(1)
    ws = api.Workspace(model, ncls)
    data = api.make_dataset(G.dev(w), G.dev(x), G.dev(y), ncls)
    api.cnnForward(c, model, data, ws.scratch, ws.z, ws.probs, ws.errors, 0, model.batchSize)
    return c, ws, data


GATHER_CASES = [
    # cin, hw, k, pad, n, expects the TMA kernel when TMA is on
    (4, 8, 3, 1, 4, True),
    (2, 10, 3, 0, 4, True),
    (2, 8, 3, 2, 3, False),    # Ho = 10 does not divide the 128-row tile: gather kernel
    (2, 8, 5, 2, 4, True),     # 5 x 5 taps: chunks of 2 channels (50 weight rows carried as 52)
    (2, 12, 5, 0, 2, True),
    (4, 16, 5, 1, 2, False),   # Ho = 14
    (3, 7, 3, 1, 5, False),    # odd height and odd K
    (6, 16, 3, 1, 16, True),   # one image per tile row block, several tiles
    (2, 32, 5, 2, 6, True),    # Ho * Wo > 128: tiles of 4 output columns
    (2, 32, 3, 1, 6, True),
    (5, 16, 5, 2, 3, False),   # odd K = 125: 16-byte stride rule of the weight map fails
    (6, 16, 5, 2, 3, True),    # three chunks of two channels
]


@pytest.mark.parametrize("tma", [1, 0], ids=["tma", "gather"])
@pytest.mark.parametrize("cin,hw,k,pad,n,want_tma", GATHER_CASES,
                         ids=["c%d-h%d-k%d-p%d-n%d" % t[:5] for t in GATHER_CASES])
def test_im2col_gather_is_index_exact(cin, hw, k, pad, n, want_tma, tma):
    """The input holds its own flat index + 1 and column q of the weight matrix is the q-th unit
    vector, so output channel q of the convolution IS column q of the im2col matrix: the gathered
    source index + 1, or 0 where the patch lies in the padding."""
    import gpu_util as G
    K = cin * k * k
    Ho = hw + 2 * pad - k + 1
    M = n * Ho * Ho
    model = S.describe_model(
        [dict(cin=cin, cout=K, h=hw, w=hw, k=k, pad=pad, bn=False, act=S.CNN_ACT_NONE, pool=None)],
        [(K * Ho * Ho, 10, S.CNN_ACT_NONE)], n, False)
    O.finalize(model)
    x = np.arange(1, cin * n * hw * hw + 1, dtype=np.float64)
    w = np.zeros(model.pSize)
    w[:K * K] = np.eye(K).reshape(-1)   # K x Cout column-major, Cout = K
    y = np.ones(n)
    c = G.ctx(1)
    c.set_tma(tma)
    try:
        before = c.kernel_launches("conv_tma_kernel")
        _, ws, _ = _forward(model, x, y, w, 10)
        used_tma = c.kernel_launches("conv_tma_kernel") - before
    finally:
        c.set_tma(1)
    assert (used_tma > 0) == bool(tma and want_tma)
    idx = np.zeros(M * K, dtype=np.int64)
    O.lib().ora_im2col_index(n, cin, hw, hw, k, pad, 1, idx)
    want = (idx + 1).astype(np.float64)            # -1 (padding) -> 0
    b = model.zOffsets[1]
    got = ws.z[b:b + K * M].cpu().numpy()
    assert np.array_equal(got, want)


def _integer_net(kind, n):
    relu = S.CNN_ACT_RELU
    if kind == "vgg":      # 3x3 convolutions, 2/2/0 max pooling, TMA shapes
        convs = [dict(cin=4, cout=8, h=16, w=16, k=3, pad=1, bn=False, act=relu, pool=(S.MAX_POOL, 2, 2, 0)),
                 dict(cin=8, cout=16, h=8, w=8, k=3, pad=1, bn=False, act=relu, pool=None),
                 dict(cin=16, cout=72, h=8, w=8, k=3, pad=1, bn=False, act=relu, pool=(S.MAX_POOL, 2, 2, 0))]
        fin = 72 * 4 * 4
    elif kind == "alex":   # 5x5 convolutions, overlapping 3/2/1 max pooling
        convs = [dict(cin=4, cout=8, h=16, w=16, k=5, pad=2, bn=False, act=relu, pool=(S.MAX_POOL, 3, 2, 1)),
                 dict(cin=8, cout=66, h=8, w=8, k=5, pad=2, bn=False, act=relu, pool=(S.MAX_POOL, 3, 2, 1))]
        fin = 66 * 4 * 4
    else:                  # odd planes: the gather kernels; average pooling by 4 is exact too
        convs = [dict(cin=3, cout=5, h=14, w=14, k=3, pad=1, bn=False, act=relu, pool=(S.AVG_POOL, 2, 2, 0)),
                 dict(cin=5, cout=6, h=7, w=7, k=3, pad=1, bn=False, act=S.CNN_ACT_NONE, pool=None)]
        fin = 6 * 7 * 7
    return S.describe_model(convs, [(fin, 10, S.CNN_ACT_NONE)], n, True)


@pytest.mark.parametrize("kind,n", [("vgg", 8), ("vgg", 32), ("alex", 8), ("alex", 16), ("odd", 5)])
def test_integer_net_forward_backward_bit_exact(kind, n):
    """Small integer inputs, weights in {-1, 0, 1} and integer output errors through ReLU + max
    pooling nets: the planes are full of exact ties (zeros after ReLU, repeated small integers),
    so the pooled values, the routed errors (dx), the data gradients and the weight gradients
    equal the oracle's bit for bit only if gather indices, tap flips and the arg-max tie rule
    are the reference's."""
    import gpu_util as G
    from fitre_b200 import api
    model = _integer_net(kind, n)
    O.finalize(model)
    rng = np.random.default_rng(11)
    c0 = model.convLayer[0]
    x = rng.integers(-2, 3, c0.inChannels * n * c0.height * c0.width).astype(np.float64)
    w = rng.integers(-1, 2, model.pSize).astype(np.float64)
    y = rng.integers(1, 11, n).astype(np.float64)
    err = rng.integers(-3, 4, 10 * n).astype(np.float64)
    env = O.make_env()
    z_o, probs_o, e_o = np.zeros(model.zSize), np.zeros(10 * n), np.zeros(max(model.maxDeltaSize, 10 * n))
    O.lib().ora_cnn_forward(C.byref(env), C.byref(model), x, y, w, 10, z_o, probs_o, e_o, n)
    g_o, dx_o = np.zeros(model.pSize), np.zeros(model.zSize)
    O.lib().ora_cnn_backward(C.byref(env), C.byref(model), x, w, z_o, g_o, dx_o, err, n)
    assert np.abs(z_o).max() < 2.0 ** 40 and np.abs(g_o).max() < 2.0 ** 40  # far inside exact range

    c, ws, data = _forward(model, x, y, w, 10)
    z = ws.z.cpu().numpy()
    md = model.maxDeltaSize + 10 * n
    d1, d2 = G.dev(np.zeros(md)), G.dev(np.zeros(md))
    d1[:10 * n] = G.dev(err)
    g, dx = G.dev(np.zeros(model.pSize)), G.dev(np.zeros(model.zSize))
    api.cnnBackward(c, model, data, ws.dev, ws.z, g, dx, d1, d2, 0, n)
    dx = dx.cpu().numpy()
    for l in range(model.cLayers):
        cl = model.convLayer[l]
        V, b = cl.convVolumn * n, model.zOffsets[l + 1]
        assert np.array_equal(z[b:b + V], z_o[b:b + V]), (l, "conv")
        a = b + cl.activationOffset
        assert np.array_equal(z[a:a + V], z_o[a:a + V]), (l, "act")
        if cl.outputOffset != cl.activationOffset:
            p, Pv = b + cl.poolOffset, cl.poolVolumn * n
            assert np.array_equal(z[p:p + Pv], z_o[p:p + Pv]), (l, "pool")
        # errors after pooling backward (arg-max routing) and after the activation derivative
        assert np.array_equal(dx[b:b + V], dx_o[b:b + V]), (l, "dx after pool backward")
        assert np.array_equal(dx[a:a + V], dx_o[a:a + V]), (l, "dx after activation backward")
    assert np.array_equal(g.cpu().numpy(), g_o)


@pytest.mark.parametrize("ks,stride,pad", [(2, 2, 0), (3, 2, 1)])
@pytest.mark.parametrize("plane", ["constant", "stripes"])
def test_max_pool_backward_routes_to_reference_argmax(ks, stride, pad, plane):
    """Tie-laden planes: a constant plane (every window is one big tie) and a plane of repeated
    column values.  The pooled errors must land exactly on the element ora_max_pool_argmax names
    (first maximum of a column-major scan of the window that starts at
    (k_out - 1) * stride + ksize - 2 * pad), errors of overlapping windows summed."""
    import gpu_util as G
    from fitre_b200 import api
    n, ch, hw = 3, 2, 8
    Hp = (hw - ks + 2 * pad) // stride + 1
    model = S.describe_model(
        [dict(cin=ch, cout=ch, h=hw, w=hw, k=3, pad=1, bn=False, act=S.CNN_ACT_NONE,
              pool=(S.MAX_POOL, ks, stride, pad))],
        [(ch * Hp * Hp, 10, S.CNN_ACT_NONE)], n, True)
    O.finalize(model)
    # the convolution copies its input: centre tap of channel c -> c (weights K x Cout, q = cin*9 + j*3 + i)
    w = np.zeros(model.pSize)
    for c_ in range(ch):
        w[c_ * (ch * 9) + c_ * 9 + 4] = 1.0
    fcw = model.wOffsets[1]
    rng = np.random.default_rng(5)
    w[fcw:fcw + 10 * ch * Hp * Hp] = rng.integers(1, 6, 10 * ch * Hp * Hp)
    if plane == "constant":
        x = np.full(ch * n * hw * hw, 2.0)
    else:  # value depends on the column only and repeats with period 2: ties inside every window
        x = np.tile(np.repeat((np.arange(hw) % 2).astype(np.float64), hw), ch * n)
    y = np.ones(n)
    err = rng.integers(-3, 4, 10 * n).astype(np.float64)
    c, ws, data = _forward(model, x, y, w, 10)
    cl = model.convLayer[0]
    V, b = cl.convVolumn * n, model.zOffsets[1]
    act = ws.z[b + cl.activationOffset:b + cl.activationOffset + V].cpu().numpy()
    assert np.array_equal(act, x)
    md = model.maxDeltaSize + 10 * n
    d1, d2 = G.dev(np.zeros(md)), G.dev(np.zeros(md))
    d1[:10 * n] = G.dev(err)
    g, dx = G.dev(np.zeros(model.pSize)), G.dev(np.zeros(model.zSize))
    api.cnnBackward(c, model, data, ws.dev, ws.z, g, dx, d1, d2, 0, n)
    got = dx[b:b + V].cpu().numpy()
    # expected: pooled errors = (FC weights)' * err, flattened (c, h, w) per sample, scattered to the arg-max
    Wfc = w[fcw:fcw + 10 * ch * Hp * Hp].reshape(ch * Hp * Hp, 10).T      # out x in, column-major
    E = err.reshape(n, 10).T                                            # classes x N, column-major
    dpool = (Wfc.T @ E).reshape(ch, Hp, Hp, n)                          # [c][hp][wp][n]
    am = np.zeros(ch * n * Hp * Hp, dtype=np.int32)
    O.lib().ora_max_pool_argmax(x, n, ch, hw, hw, ks, stride, pad, am)
    am = am.reshape(ch, n, Hp, Hp)                                      # [c][n][wp][hp] -> flat index into the tensor
    want = np.zeros(V)
    for c_ in range(ch):
        for i in range(n):
            for wp in range(Hp):
                for hp in range(Hp):
                    want[am[c_, i, wp, hp]] += dpool[c_, hp, wp, i]
    assert np.array_equal(got, want)
