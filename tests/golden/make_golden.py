"""Generates the committed golden fixtures tests/golden/*.npz.

Run once where the reference checkout is available (default: a `reference` directory beside
this repository):

    python tests/golden/make_golden.py [--reference <path to the reference checkout>]

What comes from the reference itself:
  * the flat-vector <-> tensor mapping: pytorch/testing/readWeights.py (get4DMatrix,
    get2DMatrix) is imported and used to unpack weights and vectors;
  * the one-direction trust-region model and Steihaug-CG: pytorch/peng/utils.py
    (hessian_clip, cg_steihaug) is imported and run unchanged on CPU;
  * gradient = autograd.grad(loss, params, create_graph=True) and
    Hv = autograd.grad(grad . v, params), the operator of pytorch/kfac/alexnet_cifar.py:297-324
    and pytorch/testing/test_vgg.py:108-222 (those scripts are hard-wired to CUDA tensors and
    removed PyTorch APIs, so the net is restated in tests/torch_ref.py).
Inputs are seeded synthetic data (N(0,1) images, uniform labels, He-normal weights).
The tests load the fixtures only; nothing here runs on the GPU box.
"""
import argparse
import json
import os
import sys

import numpy as np
import torch

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
    ("testvgg_softplus_bias", "test_vgg", dict(), 10),
    ("testvgg_softplus_bn_bias", "test_vgg", dict(bn=True), 10),
    ("lenet_small_swish_avg", "lenet_small", dict(), 6),
    ("lenet_small_relu_max", "lenet_small", dict(act=S.CNN_ACT_RELU, pool=S.MAX_POOL), 6),
    ("alexnet_small_bn_swish", "alexnet_small", dict(), 8),
    ("vgg_small_bn_swish", "vgg_small", dict(), 6),
    ("vgg_small_bn_relu", "vgg_small", dict(act=S.CNN_ACT_RELU), 6),
]


def unpack_with_reference(readWeights, model, flat):
    """flat parameter vector -> torch-layout arrays using the reference's own reader."""
    arrays, off = [], 0
    for kind, shape in layout.param_shapes(model):
        n = int(np.prod(shape))
        chunk = np.asarray(flat[off:off + n], dtype=np.float64)
        off += n
        if kind == "conv_w":
            arrays.append(readWeights.get4DMatrix(chunk, list(shape)))
        elif kind == "fc_w":
            arrays.append(readWeights.get2DMatrix(chunk, list(shape)))
        else:
            arrays.append(readWeights.get1DMatrix(chunk, list(shape)))
    return arrays


def main():
    ap = argparse.ArgumentParser()
    here = os.path.dirname(os.path.abspath(__file__))
    beside = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(here))), "reference")
    ap.add_argument("--reference", default=beside)
    args = ap.parse_args()
    sys.path.insert(0, os.path.join(args.reference, "pytorch", "testing"))
    sys.path.insert(0, os.path.join(args.reference, "pytorch", "peng"))
    import readWeights  # reference module
    import utils as peng_utils  # reference module (hessian_clip, cg_steihaug)

    torch.set_num_threads(4)
    for idx, (name, builder, kwargs, n) in enumerate(CASES):
        model = getattr(nets, builder)(n, **kwargs)
        O.finalize(model)
        rng = np.random.default_rng(1234 + idx)
        c0 = model.convLayer[0]
        ncls = model.fcLayer[model.lLayers - 1].out
        x = layout.batch_to_ref(rng.standard_normal((n, c0.inChannels, c0.height, c0.width)))
        y = rng.integers(1, ncls + 1, n).astype(np.float64)
        w = layout.he_normal_params(model, rng)
        if model.bias:
            w = w + 0.05 * rng.standard_normal(w.size)
        v = rng.standard_normal(model.pSize)

        # the mapping used by torch_ref must be the reference's mapping
        ref_arrays = unpack_with_reference(readWeights, model, w)
        mine = layout.params_from_ref(model, w)
        for a, b in zip(ref_arrays, mine):
            assert np.array_equal(np.asarray(a), np.asarray(b)), "layout mapping differs from readWeights.py"

        loss, g, hvs, (params, grads, loss_t) = T.loss_grad_hv(model, w, x, y, n, [v])
        out = dict(spec=json.dumps(dict(builder=builder, kwargs=kwargs, batch=n, classes=ncls)),
                   batch=x, labels=y, weights=w, vector=v, loss=loss, gradient=g, hv=hvs[0])

        # one-direction trust-region model (reference: hessian_clip) on direction v, delta = 0.7
        vs = [torch.tensor(np.ascontiguousarray(a)) for a in layout.params_from_ref(model, v)]
        gd = [gr.detach() for gr in grads]
        sv, mval = peng_utils.hessian_clip(grads, gd, params, 0.7, vs, weight=0.0)
        out["clip_delta"] = 0.7
        out["clip_vector"] = layout.params_to_ref(model, [t.detach().numpy() for t in sv])
        out["clip_model"] = mval

        # Steihaug-CG, 10 iterations, radius large enough that no boundary exit occurs
        ps, mobj, iters, flag = peng_utils.cg_steihaug(grads, gd, params, 1e3, weight=0.0,
                                                       max_iters=10, tol=1e-30)
        out["cg_delta"] = 1e3
        out["cg_iters"] = iters
        out["cg_flag"] = flag
        out["cg_p"] = layout.params_to_ref(model, [t.detach().numpy() for t in ps])
        out["cg_model"] = float(mobj)
        # and a small radius that forces the boundary exit
        ps, mobj, iters, flag = peng_utils.cg_steihaug(grads, gd, params, 0.05, weight=0.0,
                                                       max_iters=10, tol=1e-30)
        out["cgb_delta"] = 0.05
        out["cgb_iters"] = iters
        out["cgb_flag"] = flag
        out["cgb_p"] = layout.params_to_ref(model, [t.detach().numpy() for t in ps])
        out["cgb_model"] = float(mobj)

        # damped operator H + 5 I is positive definite here: runs all 10 iterations
        ps, mobj, iters, flag = peng_utils.cg_steihaug(grads, gd, params, 1e3, weight=5.0,
                                                       max_iters=10, tol=1e-30)
        out["cgw_delta"] = 1e3
        out["cgw_weight"] = 5.0
        out["cgw_iters"] = iters
        out["cgw_flag"] = flag
        out["cgw_p"] = layout.params_to_ref(model, [t.detach().numpy() for t in ps])
        out["cgw_model"] = float(mobj)

        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, **out)
        print("%-28s pSize %5d loss %.10f cg %s/%d cgb %s/%d cgw %s/%d -> %s" % (
            name, model.pSize, loss, out["cg_flag"], out["cg_iters"], out["cgb_flag"],
            out["cgb_iters"], out["cgw_flag"], out["cgw_iters"], os.path.basename(path)))


if __name__ == "__main__":
    main()
