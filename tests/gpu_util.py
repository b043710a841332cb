"""Helpers for the GPU parity tests: run the CUDA library through its C ABI (via
fitre_b200.api) on numpy inputs and hand back numpy outputs."""
import numpy as np

from fitre_b200 import api, layout
from fitre_b200 import _structs as S

_CTX = {}


def ctx(ref_softmax=1):
    import torch
    if "c" not in _CTX:
        _CTX["c"] = api.Context(torch.cuda.current_device())
    _CTX["c"].set_reference_softmax(ref_softmax)
    return _CTX["c"]


def dev(a):
    import torch
    return torch.tensor(np.ascontiguousarray(a), dtype=torch.float64, device="cuda")


def synth(model, n, seed, bias_noise=0.05):
    rng = np.random.default_rng(seed)
    c0 = model.convLayer[0]
    ncls = model.fcLayer[model.lLayers - 1].out
    x = layout.batch_to_ref(rng.standard_normal((n, c0.inChannels, c0.height, c0.width)))
    y = rng.integers(1, ncls + 1, n).astype(np.float64)
    w = layout.he_normal_params(model, rng)
    if model.bias:
        w = w + bias_noise * rng.standard_normal(w.size)
    v = rng.standard_normal(model.pSize)
    return x, y, w, v, ncls


class GpuRun:
    """One gradient evaluation on the GPU; keeps the state for Hessian-vector calls."""

    def __init__(self, model, x, y, w, ncls, ref_softmax=1, weight_decay=0.0):
        api.finalize(model)
        self.c = ctx(ref_softmax)
        self.model, self.n, self.ncls = model, model.batchSize, ncls
        self.ws = api.Workspace(model, ncls)
        self.w, self.x, self.y = dev(w), dev(x), dev(y)
        self.data = api.make_dataset(self.w, self.x, self.y, ncls)
        ws = self.ws
        self.loss = api.computeCNNGradient(self.c, model, self.data, ws.scratch, ws.z, ws.dx,
                                           ws.probs, ws.errors, ws.gradient, 0, self.n,
                                           weight_decay)
        self.gradient = ws.gradient.cpu().numpy()

    def hv(self, v):
        ws = self.ws
        vv = dev(v)
        api.cnnHv(self.c, self.model, self.data, ws.z, ws.probs, ws.errors, ws.dx, vv, ws.hv, 0,
                  self.n, ws.dev)
        return ws.hv.cpu().numpy()


def rel(a, b):
    a, b = np.asarray(a), np.asarray(b)
    return np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-300)


def relmax(a, b):
    a, b = np.asarray(a), np.asarray(b)
    return np.max(np.abs(a - b)) / max(np.max(np.abs(b)), 1e-300)
