"""The reference-facing boundary at link level: struct layouts of include/fitre_b200.h equal the
reference's (fixture measured against the reference's own headers), and
libfitre_reference_shim.so exports every C++ symbol a reference driver object imports for this
path (fixture produced by compiling against the reference's headers).  When the reference tree is
present the fixtures are regenerated and compared, so they cannot go stale unnoticed."""
import ctypes as C
import json
import os
import subprocess
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
GOLD = os.path.join(HERE, "golden")
sys.path.insert(0, GOLD)
# the reference checkout, when it sits beside this repository (absent on GPU machines)
REFERENCE = os.path.join(os.path.dirname(ROOT), "reference")


def shim_path():
    from fitre_b200 import build
    if not os.path.exists(build.SHIM_LIB):
        build.build()
    return build.SHIM_LIB


def exported(lib):
    out = subprocess.check_output(["nm", "-D", "--defined-only", lib], text=True)
    return {l.split()[-1] for l in out.splitlines() if l.split()}


def test_struct_layouts_equal_the_reference():
    import make_reference_layout as L
    want = json.load(open(os.path.join(GOLD, "reference_struct_layout.json")))
    mine = L.run_probe(["fitre_b200.h"], [os.path.join(ROOT, "include")])
    assert mine == want
    if os.path.isdir(REFERENCE):
        cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
        fresh = L.run_probe(["nn/nn_decl.h", "core/structdefs.h", "solvers/params.h"],
                            [REFERENCE, os.path.join(cuda, "include")])
        assert fresh == want


def test_shim_exports_the_reference_symbols():
    want = open(os.path.join(GOLD, "reference_symbols.txt")).read().split()
    assert len(want) == 25
    have = exported(shim_path())
    missing = [s for s in want if s not in have]
    assert not missing, missing


def test_reference_style_caller_links_against_the_shim(tmp_path):
    """A translation unit that declares the functions the way the reference's headers do (same
    typedef'd struct tags) and references them links against the shim without unresolved names."""
    src = tmp_path / "caller.cpp"
    src.write_text('''
typedef double real;
typedef struct cnn CNN_MODEL; typedef struct dev_dataset DEVICE_DATASET;
typedef struct scratch_space SCRATCH_AREA;
typedef enum eval_type { MODEL_TRAIN = 10, MODEL_TRAIN_ACCURACY = 20, MODEL_TEST_ACCURACY = 30 } EVAL_TYPE;
real computeCNNGradient(CNN_MODEL *model, DEVICE_DATASET *data, SCRATCH_AREA *scratch, real *z, real *dx,
   real *probs, real *lossFuncErrors, real *gradient, int offset, int curBatchSize, real weightDecay);
real cnnForward(CNN_MODEL *model, DEVICE_DATASET *data, SCRATCH_AREA *scratch, real *z, real *probs,
   real *errors, int s, int curBatchSize, EVAL_TYPE forTesting);
void cnnHv(CNN_MODEL *model, DEVICE_DATASET *data, real *z, real *probs, real *lossFuncErrors, real *dx,
   real *vector, real *hv, int s, int curBatchSize, real *devPtr, real *hostPtr, real weightDecay);
real computeQuadraticModel(CNN_MODEL *model, DEVICE_DATASET *data, real *z, real *probs,
   real *lossFuncErrors, real *dx, real *gradient, real *vector, real delta, int offset, int curBatchSize,
   real weightDecay, real *devPtr, real *hostPtr, real *pageLckPtr);
void *imports[] = {(void *)&computeCNNGradient, (void *)&cnnForward, (void *)&cnnHv,
                   (void *)&computeQuadraticModel};
int main() { return imports[0] == 0; }
''')
    lib = shim_path()
    d = os.path.dirname(lib)
    exe = tmp_path / "caller"
    subprocess.check_call(["g++", str(src), "-o", str(exe), "-L", d, "-lfitre_reference_shim",
                           "-lfitre_b200", "-Wl,-rpath," + d, "-Wl,--no-undefined"])
    if os.path.isdir(REFERENCE):
        import make_reference_symbols  # noqa: F401  (generator stays importable)


@pytest.mark.gpu
def test_shim_gradient_and_hv_match_the_oracle():
    """Calls through the mangled reference entry points (as a reference driver would)."""
    import torch
    import gpu_util as G
    import nets
    import oracle_lib as O
    from fitre_b200 import api
    lib = C.CDLL(shim_path())
    grad = getattr(lib, "_Z18computeCNNGradientP3cnnP11dev_datasetP13scratch_spacePdS5_S5_S5_S5_iid")
    grad.restype = C.c_double
    grad.argtypes = [C.c_void_p] * 8 + [C.c_int, C.c_int, C.c_double]
    hvf = getattr(lib, "_Z5cnnHvP3cnnP11dev_datasetPdS3_S3_S3_S3_S3_iiS3_S3_d")
    hvf.restype = None
    hvf.argtypes = [C.c_void_p] * 8 + [C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_double]
    n = 6
    model = nets.vgg_small(n)
    O.finalize(model)
    x, y, w, v, ncls = G.synth(model, n, seed=5)
    st = O.gradient(model, x, y, w, ncls, n, weight_decay=1e-3)
    hv_o = O.hv(model, x, w, ncls, n, st, v)
    ws = api.Workspace(model, ncls)
    data = api.make_dataset(G.dev(w), G.dev(x), G.dev(y), ncls)
    V = G.dev(v)
    loss = grad(C.addressof(model), C.addressof(data), C.addressof(ws.scratch), ws.z.data_ptr(),
                ws.dx.data_ptr(), ws.probs.data_ptr(), ws.errors.data_ptr(), ws.gradient.data_ptr(), 0, n, 1e-3)
    assert abs(loss - st.loss) <= 1e-10 * abs(st.loss)
    assert G.rel(ws.gradient.cpu().numpy(), st.gradient) < 1e-10
    hvf(C.addressof(model), C.addressof(data), ws.z.data_ptr(), ws.probs.data_ptr(), ws.errors.data_ptr(),
        ws.dx.data_ptr(), V.data_ptr(), ws.hv.data_ptr(), 0, n, ws.dev.data_ptr(), None, 0.0)
    assert G.rel(ws.hv.cpu().numpy(), hv_o) < 1e-10
