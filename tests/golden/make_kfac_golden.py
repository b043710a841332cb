"""Generates the committed KFAC fixtures tests/golden/kfac_*.npz from the reference's own
PyTorch implementation of the factors.

    python tests/golden/make_kfac_golden.py [--reference <path to the reference checkout>]

What comes from the reference itself (imported from pytorch/kfac/kfac_utils.py and run
unchanged on CPU, with the module's tensor type switched from torch.cuda.FloatTensor to
torch.DoubleTensor):
  * KFACUtils.getExpandedForm + matmulOmega (:74-137): A factor of a convolution,
    (1/N) P'P with P = [unfolded input / (Ho Wo), 1];
  * KFACUtils.matmul3d (:189-236): A factor of a fully connected layer, (1/N) [z,1]'[z,1];
  * KFACUtils.matmulLambda (:139-187): G factors, (N Ho Wo) d'd for a convolution and N d'd for
    a fully connected layer, d = gradient of the mean loss on SAMPLED labels with respect to
    the layer's output;
  * KFACUtils.computeMatVec (:278-404): natural gradient G^-1 [W|b] A^-1.
Restated here because it calls an API that current PyTorch no longer has:
  * getPseudoInverse (:35-41, torch.gesv(I, mat)): the solution X of mat X = I, by
    torch.linalg.solve; computeInverses (:44-72) around it damps with (regLambda + gamma) I.
The net's forward pass and the sampled-label gradient come from autograd on the restated net
(tests/torch_ref.py), as in make_golden.py.

Index order: the reference's PyTorch code orders a patch (channel, kernel row, kernel column),
its CUDA code (channel, kernel column, kernel row) (functions/dev_image.cu:20-49); the fixtures
store the factors in the CUDA order, i.e. rows and columns permuted, nothing else changed.
"""
import argparse
import json
import os
import sys

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import nets  # noqa: E402
import oracle_lib as O  # noqa: E402  (only to fill offsets/sizes of the model struct)
import torch_ref as T  # noqa: E402
from fitre_b200 import _structs as S  # noqa: E402
from fitre_b200 import layout  # noqa: E402

CASES = [
    # name, builder, kwargs, batch
    ("kfac_vgg_small_bn_swish", "vgg_small", dict(), 6),
    ("kfac_lenet_small_swish_avg_bias", "lenet_small", dict(), 5),
    ("kfac_alexnet_small_bn_bias", "alexnet_small", dict(bias=True), 4),
]
LAMBDA, GAMMA = 1e-3, 1e-2


def patch_perm(cin, k, bias):
    """perm[q_cuda] = q_torch for q = (c, kernel column j, kernel row i) <- (c, row, column)."""
    perm = []
    for c in range(cin):
        for j in range(k):
            for i in range(k):
                perm.append(c * k * k + i * k + j)
    if bias:
        perm.append(cin * k * k)
    return np.asarray(perm)


def main():
    ap = argparse.ArgumentParser()
    beside = os.path.join(os.path.dirname(ROOT), "reference")
    ap.add_argument("--reference", default=beside)
    args = ap.parse_args()
    sys.dont_write_bytecode = True
    sys.path.insert(0, os.path.join(args.reference, "pytorch", "kfac"))
    import kfac_utils  # reference module
    kfac_utils.TYPE = torch.DoubleTensor

    torch.set_num_threads(4)
    for idx, (name, builder, kwargs, n) in enumerate(CASES):
        model = getattr(nets, builder)(n, **kwargs)
        O.finalize(model)
        rng = np.random.default_rng(4234 + idx)
        c0 = model.convLayer[0]
        ncls = model.fcLayer[model.lLayers - 1].out
        x_ref = layout.batch_to_ref(rng.standard_normal((n, c0.inChannels, c0.height, c0.width)))
        y = rng.integers(1, ncls + 1, n).astype(np.float64)
        y_sampled = rng.integers(1, ncls + 1, n).astype(np.float64)
        w = layout.he_normal_params(model, rng)
        if model.bias:
            w = w + 0.05 * rng.standard_normal(w.size)
        bias = bool(model.bias)
        nl = model.cLayers + model.lLayers
        kinds = ["conv"] * model.cLayers + ["linear"] * model.lLayers

        x = torch.tensor(layout.batch_from_ref(x_ref, n, c0.inChannels, c0.height, c0.width).copy(),
                         dtype=torch.float64)
        params = T.torch_params(model, w)
        logits, ins, outs = T.forward_capture(model, params, x)
        # gradient of the mean loss on the true labels: the vector the natural gradient is taken of
        loss = F.cross_entropy(logits, torch.tensor(y.astype(np.int64) - 1))
        grads = torch.autograd.grad(loss, params, retain_graph=True)
        # second backward pass on the sampled labels: errors at every layer's output
        loss_s = F.cross_entropy(logits, torch.tensor(y_sampled.astype(np.int64) - 1))
        dxs = torch.autograd.grad(loss_s, outs)

        ku = kfac_utils.KFACUtils(3, 1, kinds, n, bias, False, GAMMA, LAMBDA, 0)
        A, G = [], []
        for l in range(nl):
            if l < model.cLayers:
                c = model.convLayer[l]
                ku.kSize, ku.padding = c.kSize, c.padding
                a = ku.matmulOmega(ku.getExpandedForm(ins[l].detach().clone()), None)
            else:
                a = ku.matmul3d(ins[l].detach().clone(), ins[l].dim() == 4, None)
            g = ku.matmulLambda(dxs[l].detach().clone(), None)
            A.append(a)
            G.append(g)
        # computeInverses (:44-72) with getPseudoInverse restated: mat X = I
        ku.ZInv, ku.dInv = [], []
        scale = ku.regLambda + ku.gamma
        for l in range(nl):
            for src, dst in ((A[l], ku.ZInv), (G[l], ku.dInv)):
                mat = src + scale * torch.eye(src.size(0), dtype=torch.float64)
                dst.append(torch.linalg.solve(mat, torch.eye(src.size(0), dtype=torch.float64)))
        ng = ku.computeMatVec([g.detach() for g in grads])

        out = dict(spec=json.dumps(dict(builder=builder, kwargs=kwargs, batch=n, classes=ncls)),
                   batch=x_ref, labels=y, sampled_labels=y_sampled, weights=w,
                   regLambda=LAMBDA, dampGamma=GAMMA,
                   gradient=T.flat_from_torch(model, grads),
                   natural_gradient=T.flat_from_torch(model, ng))
        for l in range(nl):
            a, g = A[l].numpy(), G[l].numpy()
            ai, gi = ku.ZInv[l].numpy(), ku.dInv[l].numpy()
            if l < model.cLayers:
                c = model.convLayer[l]
                p = patch_perm(c.inChannels, c.kSize, bias)
                a, ai = a[np.ix_(p, p)], ai[np.ix_(p, p)]
            out["A%d" % l], out["G%d" % l] = np.ascontiguousarray(a), np.ascontiguousarray(g)
            out["Ainv%d" % l], out["Ginv%d" % l] = np.ascontiguousarray(ai), np.ascontiguousarray(gi)
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, **out)
        print("%-34s layers %d pSize %5d |A0| %.4e |G0| %.4e |ng| %.4e -> %s" % (
            name, nl, model.pSize, np.linalg.norm(out["A0"]), np.linalg.norm(out["G0"]),
            np.linalg.norm(out["natural_gradient"]), os.path.basename(path)))


if __name__ == "__main__":
    main()
