"""Host-side layout helpers: the reference's flat layouts <-> ordinary NCHW arrays.

Layouts (reference file:line in parentheses):
  batch tensor   [C][N][W][H], h fastest                 (functions/dev_image.cu:37-38)
  conv weights   per layer a column-major (k*k*Cin) x Cout matrix, kernel row fastest:
                 flat = o*K + i*k*k + c*k + r            (functions/eval_convolution.cu:115-119,
                                                          pytorch/testing/readWeights.py:3-24)
  FC weights     out x in, column-major                  (functions/eval_gradient.cu:62-66)
  bias           follows the weights of the same layer when the model has biases
                                                         (nn/utils.c:74-105)
  labels         doubles in 1..numClasses                (functions/softmax_loss.cu:73,222)
"""
import numpy as np


def batch_to_ref(x_nchw):
    """[N][C][H][W] -> reference [C][N][W][H] (flat, float64)."""
    x = np.asarray(x_nchw, dtype=np.float64)
    return np.ascontiguousarray(x.transpose(1, 0, 3, 2)).reshape(-1)


def batch_from_ref(flat, n, c, h, w):
    return np.asarray(flat, dtype=np.float64).reshape(c, n, w, h).transpose(1, 0, 3, 2)


def conv_weight_to_ref(w_oihw):
    """torch [O][I][kh][kw] -> flat o*K + i*k*k + c*k + r."""
    w = np.asarray(w_oihw, dtype=np.float64)
    return np.ascontiguousarray(w.transpose(0, 1, 3, 2)).reshape(-1)


def conv_weight_from_ref(flat, o, i, k):
    return np.asarray(flat, dtype=np.float64).reshape(o, i, k, k).transpose(0, 1, 3, 2)


def fc_weight_to_ref(w_out_in):
    return np.asarray(w_out_in, dtype=np.float64).reshape(w_out_in.shape).T.reshape(-1)


def fc_weight_from_ref(flat, out, inp):
    return np.asarray(flat, dtype=np.float64).reshape(inp, out).T


def param_shapes(model):
    """[(kind, shape)] in flat-vector order for a CNN_MODEL (ctypes)."""
    shapes = []
    for l in range(model.cLayers):
        c = model.convLayer[l]
        shapes.append(("conv_w", (c.outChannels, c.inChannels, c.kSize, c.kSize)))
        if model.bias:
            shapes.append(("bias", (c.outChannels,)))
    for l in range(model.lLayers):
        f = model.fcLayer[l]
        shapes.append(("fc_w", (f.out, f.in_)))
        if model.bias:
            shapes.append(("bias", (f.out,)))
    return shapes


def params_to_ref(model, arrays):
    """list of torch-layout arrays (order of param_shapes) -> flat parameter vector."""
    out = []
    for (kind, shape), a in zip(param_shapes(model), arrays):
        a = np.asarray(a, dtype=np.float64)
        assert tuple(a.shape) == tuple(shape), (a.shape, shape)
        if kind == "conv_w":
            out.append(conv_weight_to_ref(a))
        elif kind == "fc_w":
            out.append(fc_weight_to_ref(a))
        else:
            out.append(a.reshape(-1))
    return np.concatenate(out)


def params_from_ref(model, flat):
    flat = np.asarray(flat, dtype=np.float64)
    arrays, off = [], 0
    for kind, shape in param_shapes(model):
        n = int(np.prod(shape))
        chunk = flat[off:off + n]
        off += n
        if kind == "conv_w":
            arrays.append(conv_weight_from_ref(chunk, *shape[:3]))
        elif kind == "fc_w":
            arrays.append(fc_weight_from_ref(chunk, *shape))
        else:
            arrays.append(chunk.copy())
    assert off == flat.size
    return arrays


def he_normal_params(model, rng):
    """He-normal weights (std sqrt(2/fan_in)), zero biases, in the flat reference layout."""
    arrays = []
    for kind, shape in param_shapes(model):
        if kind == "conv_w":
            fan_in = shape[1] * shape[2] * shape[3]
            arrays.append(rng.standard_normal(shape) * np.sqrt(2.0 / fan_in))
        elif kind == "fc_w":
            arrays.append(rng.standard_normal(shape) * np.sqrt(2.0 / shape[1]))
        else:
            arrays.append(np.zeros(shape))
    return params_to_ref(model, arrays)


def shard_batch(flat_ref, n, c, h, w, rank, world):
    """Samples [rank*n/world, (rank+1)*n/world) of a reference-layout batch, same layout."""
    assert n % world == 0
    per = n // world
    x = np.asarray(flat_ref, dtype=np.float64).reshape(c, n, w * h)
    return np.ascontiguousarray(x[:, rank * per:(rank + 1) * per, :]).reshape(-1)
