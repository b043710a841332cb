"""Writes tests/golden/reference_symbols.txt: the C++-mangled names of the reference functions on
the hot path and its callers, obtained by compiling a translation unit that includes the
REFERENCE'S OWN HEADERS and takes the address of each function (so the names are what a
reference driver object would import).  Usage: python make_reference_symbols.py <reference root>.
Needs g++, nm and the CUDA headers; the reference tree is only read."""
import os
import subprocess
import sys
import tempfile

HEADERS = ["functions/cnn_gradient.h", "functions/cnn_forward.h", "functions/cnn_backward.h",
           "functions/cnn_hessian_vec.h", "functions/cnn_hv_forward.h", "functions/cnn_hv_backward.h",
           "functions/model_reduction.h", "functions/cnn_eval_model.h", "functions/cnn_accuracy.h",
           "functions/softmax_loss.h", "solvers/kfac_da.h", "utilities/sample_matrix.h",
           "solvers/kfac_utils.h", "solvers/kfac_inverses.h", "solvers/kfac_natural_gradient.h"]
FUNCTIONS = ["computeCNNGradient", "cnnForwardMemRequired", "cnnForward", "cnnBackwardMemRequired",
             "cnnBackward", "cnnHv", "cnnROpForwardMemRequired", "cnnROpForward",
             "cnnROpBackwardMemRequired", "cnnROpBackward", "computeQuadraticModel", "evaluateCNNModel",
             "computeAccuracy", "computeTestGeneralizationErrors", "computeTrainGeneralizationErrors",
             "computeDistributionErrors", "augmentData", "selectColumnMatrix",
             "computeKFACStorageIndices", "computeOmegaZ", "computeLambdaDelta", "computeNaturalGradient",
             "updateRunningStats", "computeSpeedUpOmegaZ", "computeSpeedUpLambdaDelta"]


def main():
    ref = sys.argv[1]
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    with tempfile.TemporaryDirectory() as tmp:
        src, obj = os.path.join(tmp, "caller.cpp"), os.path.join(tmp, "caller.o")
        with open(src, "w") as f:
            for h in HEADERS:
                f.write("#include <%s>\n" % h)
            f.write("void *fitre_reference_imports[] = {\n")
            for fn in FUNCTIONS:
                f.write("    (void *)&%s,\n" % fn)
            f.write("};\n")
        subprocess.check_call(["g++", "-std=c++14", "-fpermissive", "-w", "-c", "-I", ref,
                               "-I", os.path.join(cuda, "include"), src, "-o", obj])
        out = subprocess.check_output(["nm", "-u", obj], text=True)
    syms = sorted(l.split()[-1] for l in out.splitlines() if l.split() and l.split()[-1].startswith("_Z"))
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_symbols.txt")
    with open(dst, "w") as f:
        f.write("\n".join(syms) + "\n")
    print("%d symbols -> %s" % (len(syms), dst))


if __name__ == "__main__":
    main()
