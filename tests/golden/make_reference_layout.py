"""Writes tests/golden/reference_struct_layout.json: sizeof and field offsets of the structs that
cross the boundary, measured by compiling a probe against the REFERENCE'S OWN HEADERS.
Usage: python make_reference_layout.py <reference root>.  The probe source is shared with
tests/test_shim.py, which compiles the same probe against include/fitre_b200.h."""
import json
import os
import subprocess
import sys
import tempfile

# (struct, fields) -- typedef names are the same in the reference and in include/fitre_b200.h
STRUCTS = [
    ("CONV_LAYER", ["inChannels", "outChannels", "kSize", "padding", "stride", "batchNorm", "height", "width",
                    "outHeight", "outWidth", "convVolumn", "activationOffset", "poolOffset", "batchNormOffset",
                    "meansOffset", "variancesOffset", "runningMeansOffset", "runningVariancesOffset",
                    "outputOffset"]),
    ("POOL_LAYER", ["type", "pSize", "stride", "padding", "height", "width", "outHeight", "outWidth"]),
    ("FC_LAYER", ["in", "out", "actFun", "offset"]),
    ("CNN_MODEL", ["convLayer", "actFuns", "poolLayer", "cLayers", "lLayers", "fcLayer", "pSize", "zSize",
                   "maxDeltaSize", "batchSize", "bias", "wOffsets", "bOffsets", "zOffsets", "zztOffsets",
                   "zztSize", "enableBatchNorm"]),
    ("SCRATCH_AREA", ["hostWorkspace", "devWorkspace", "pageLckWorkspace", "nextDevPtr", "nextHostPtr",
                      "nextPageLckPtr"]),
    ("DEVICE_DATASET", ["trainSetX", "trainSetY", "testSetX", "testSetY", "weights", "numClasses",
                        "datasetType", "features", "height", "width", "testSizeX", "testSizeY", "trainSizeX",
                        "trainSizeY", "sampleSize", "sampledTrainX", "sampledTrainY", "currentBatch",
                        "spSamplingMatrix"]),
    ("TRUST_REGION_PARAMS", ["delta", "minDelta", "maxDelta", "eta1", "eta2", "gamma1", "gamma2", "maxProps",
                             "maxMatVecs", "maxEpochs", "maxIters", "hessianType", "alpha", "curIteration", "hs",
                             "lambda"]),
]


def probe_source(includes):
    lines = ["#include <cstddef>", "#include <cstdio>"] + ["#include <%s>" % h for h in includes]
    lines.append("int main() {")
    for s, fields in STRUCTS:
        lines.append('    printf("%s.sizeof %%zu\\n", sizeof(%s));' % (s, s))
        for f in fields:
            lines.append('    printf("%s.%s %%zu\\n", offsetof(%s, %s));' % (s, f, s, f))
    lines += ["    return 0;", "}"]
    return "\n".join(lines) + "\n"


def run_probe(includes, include_dirs):
    with tempfile.TemporaryDirectory() as tmp:
        src, exe = os.path.join(tmp, "probe.cpp"), os.path.join(tmp, "probe")
        open(src, "w").write(probe_source(includes))
        cmd = ["g++", "-std=c++14", "-fpermissive", "-w", src, "-o", exe]
        for d in include_dirs:
            cmd += ["-I", d]
        subprocess.check_call(cmd)
        out = subprocess.check_output([exe], text=True)
    return {k: int(v) for k, v in (l.split() for l in out.splitlines())}


def main():
    ref = sys.argv[1]
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    layout = run_probe(["nn/nn_decl.h", "core/structdefs.h", "solvers/params.h"],
                       [ref, os.path.join(cuda, "include")])
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_struct_layout.json")
    json.dump(layout, open(dst, "w"), indent=0, sort_keys=True)
    print("%d entries -> %s" % (len(layout), dst))


if __name__ == "__main__":
    main()
