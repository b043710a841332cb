"""PyTorch (CPU, fp64) statement of the same nets, gradient by autograd and Hessian-vector
product by double backward -- the operator of the reference's PyTorch path
(pytorch/kfac/alexnet_cifar.py:297-324, pytorch/testing/test_vgg.py:108-222).
Test infrastructure: an independent cross-check of the C oracle and the generator of the
committed golden fixtures.
"""
import numpy as np
import torch
import torch.nn.functional as F

from fitre_b200 import _structs as S
from fitre_b200 import layout


def _act(kind, x):
    if kind == S.CNN_ACT_SWISH:
        return x * torch.sigmoid(x)
    if kind == S.CNN_ACT_SOFTPLUS:
        return F.softplus(x)  # threshold 20, as functions/dev_activations.cu:24-39
    if kind == S.CNN_ACT_RELU:
        return F.relu(x)
    if kind in (S.CNN_ACT_NONE, S.ACT_LINEAR):
        return x
    raise ValueError(kind)


def forward(model, params, x):
    """params: list of tensors in layout.param_shapes order; x: [N][C][H][W]."""
    it = iter(params)
    out = x
    for l in range(model.cLayers):
        c, p = model.convLayer[l], model.poolLayer[l]
        w = next(it)
        b = next(it) if model.bias else None
        out = F.conv2d(out, w, b, stride=c.stride, padding=c.padding)
        if c.batchNorm != S.NO_BATCH_NORM:
            out = F.batch_norm(out, None, None, training=True, eps=1e-5)
        out = _act(model.actFuns[l], out)
        if p.type == S.MAX_POOL:
            out = F.max_pool2d(out, p.pSize, p.stride, p.padding)
        elif p.type == S.AVG_POOL:
            out = F.avg_pool2d(out, p.pSize, p.stride, p.padding)
    out = out.reshape(out.shape[0], -1)
    for l in range(model.lLayers):
        f = model.fcLayer[l]
        w = next(it)
        b = next(it) if model.bias else None
        out = F.linear(out, w, b)
        out = _act(f.actFun, out)
    return out


def forward_capture(model, params, x):
    """forward() that also returns, per layer, the tensor the layer reads (conv: [N][C][H][W];
    FC: the previous layer's output, 4-D in front of the first FC layer) and the tensor its
    convolution / matrix product writes (before batch norm and activation) -- what the
    reference's KFAC hooks store as Zis and dxA (pytorch/kfac/kfac_utils.py:30-32)."""
    it = iter(params)
    out = x
    ins, outs = [], []
    for l in range(model.cLayers):
        c, p = model.convLayer[l], model.poolLayer[l]
        w = next(it)
        b = next(it) if model.bias else None
        ins.append(out)
        out = F.conv2d(out, w, b, stride=c.stride, padding=c.padding)
        outs.append(out)
        if c.batchNorm != S.NO_BATCH_NORM:
            out = F.batch_norm(out, None, None, training=True, eps=1e-5)
        out = _act(model.actFuns[l], out)
        if p.type == S.MAX_POOL:
            out = F.max_pool2d(out, p.pSize, p.stride, p.padding)
        elif p.type == S.AVG_POOL:
            out = F.avg_pool2d(out, p.pSize, p.stride, p.padding)
    for l in range(model.lLayers):
        f = model.fcLayer[l]
        w = next(it)
        b = next(it) if model.bias else None
        ins.append(out)
        out = F.linear(out.reshape(out.shape[0], -1), w, b)
        outs.append(out)
        out = _act(f.actFun, out)
    return out, ins, outs


def torch_params(model, flat):
    return [torch.tensor(np.ascontiguousarray(a), dtype=torch.float64, requires_grad=True)
            for a in layout.params_from_ref(model, flat)]


def flat_from_torch(model, tensors):
    return layout.params_to_ref(model, [t.detach().numpy() for t in tensors])


def loss_grad_hv(model, flat_w, batch_ref, labels1, n, vectors=()):
    """Returns loss, flat gradient, [flat Hv for each flat vector]."""
    c0 = model.convLayer[0]
    x = torch.tensor(layout.batch_from_ref(batch_ref, n, c0.inChannels, c0.height, c0.width).copy(),
                     dtype=torch.float64)
    y = torch.tensor(np.asarray(labels1, dtype=np.int64) - 1)
    params = torch_params(model, flat_w)
    logits = forward(model, params, x)
    loss = F.cross_entropy(logits, y)
    grads = torch.autograd.grad(loss, params, create_graph=True)
    g_flat = flat_from_torch(model, grads)
    hvs = []
    for v in vectors:
        vs = [torch.tensor(np.ascontiguousarray(a), dtype=torch.float64)
              for a in layout.params_from_ref(model, v)]
        dotp = sum((g * t).sum() for g, t in zip(grads, vs))
        hv = torch.autograd.grad(dotp, params, retain_graph=True)
        hvs.append(flat_from_torch(model, hv))
    return float(loss.detach()), g_flat, hvs, (params, grads, loss)
