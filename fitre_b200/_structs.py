"""ctypes mirrors of the boundary structs declared in include/fitre_b200.h.

Field order and types follow the reference's structs (nn/nn_decl.h:64-155,
core/structdefs.h:25-83) so that a struct filled by a reference driver can be
passed through unchanged.
"""
import ctypes as C

MAX_LAYERS = 20

# enum values (nn/nn_decl.h:13-101)
NO_BATCH_NORM, BATCH_NORM = 0, 10
MODEL_TRAIN = 10
ACT_LOGISTIC, ACT_TANH, ACT_LINEAR = 1, 2, 3
CNN_ACT_NONE, CNN_ACT_SOFTPLUS, CNN_ACT_ELU, CNN_ACT_RELU, CNN_ACT_SWISH = 10, 11, 12, 13, 14
MAX_POOL, AVG_POOL, NO_POOL = 0, 1, 2

# status codes
OK, ERR_BAD_ARG, ERR_UNSUPPORTED, ERR_WORKSPACE, ERR_CUDA, ERR_COMM, ERR_NOT_CONVERGED, ERR_TOO_LARGE, ERR_NOT_FINITE = range(9)

CG_CONVERGED, CG_NEG_CURVATURE, CG_HIT_BOUNDARY, CG_MAX_ITERS = range(4)

real_p = C.POINTER(C.c_double)


class CONV_LAYER(C.Structure):
    _fields_ = [(n, C.c_int) for n in (
        "inChannels", "outChannels", "width", "height", "outWidth", "outHeight",
        "kSize", "stride", "padding",
        "activationOffset", "poolOffset", "batchNormOffset", "outputOffset",
        "batchNorm", "meansOffset", "variancesOffset",
        "runningMeansOffset", "runningVariancesOffset",
        "convVolumn", "activationVolumn", "poolVolumn", "batchNormVolumn")]


class POOL_LAYER(C.Structure):
    _fields_ = [(n, C.c_int) for n in (
        "height", "width", "outHeight", "outWidth", "type", "pSize", "padding", "stride")]


class FC_LAYER(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("in_", "out", "actFun", "batchNorm", "offset")]


class CNN_MODEL(C.Structure):
    _fields_ = [
        ("convLayer", CONV_LAYER * MAX_LAYERS),
        ("actFuns", C.c_int * MAX_LAYERS),
        ("poolLayer", POOL_LAYER * MAX_LAYERS),
        ("cLayers", C.c_int),
        ("lLayers", C.c_int),
        ("fcLayer", FC_LAYER * MAX_LAYERS),
        ("bias", C.c_int), ("pSize", C.c_int), ("zSize", C.c_int), ("batchSize", C.c_int),
        ("maxDeltaSize", C.c_int), ("name", C.c_int), ("enableBatchNorm", C.c_int),
        ("wOffsets", C.c_int * MAX_LAYERS),
        ("bOffsets", C.c_int * MAX_LAYERS),
        ("zOffsets", C.c_int * MAX_LAYERS),
        ("zztSize", C.c_int),
        ("zztOffsets", C.c_int * MAX_LAYERS),
        ("rZOffsets", C.c_int * MAX_LAYERS),
    ]


class SCRATCH_AREA(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in (
        "hostWorkspace", "devWorkspace", "pageLckWorkspace",
        "nextDevPtr", "nextHostPtr", "nextPageLckPtr")]


class SPARSE_DATASET(C.Structure):
    _fields_ = [("rowPtr", C.c_void_p), ("colPtr", C.c_void_p), ("rowCsrPtr", C.c_void_p),
                ("valPtr", C.c_void_p), ("nnz", C.c_int), ("sortedVals", C.c_void_p),
                ("P", C.c_void_p), ("descr", C.c_void_p)]


class DEVICE_DATASET(C.Structure):
    _fields_ = [
        ("trainSetX", C.c_void_p), ("trainSetY", C.c_void_p),
        ("testSetX", C.c_void_p), ("testSetY", C.c_void_p),
        ("weights", C.c_void_p),
        ("numClasses", C.c_int), ("datasetType", C.c_int),
        ("features", C.c_int), ("height", C.c_int), ("width", C.c_int),
        ("testSizeX", C.c_int), ("testSizeY", C.c_int),
        ("trainSizeX", C.c_int), ("trainSizeY", C.c_int),
        ("sampleSize", C.c_int),
        ("sampledTrainX", C.c_void_p), ("sampledTrainY", C.c_void_p),
        ("currentBatch", C.c_void_p),
        ("spSamplingMatrix", SPARSE_DATASET),
    ]


class KFAC_INFO(C.Structure):
    _fields_ = [
        ("OmegaZOffsets", C.c_int * MAX_LAYERS),
        ("LambdaGOffsets", C.c_int * MAX_LAYERS),
        ("OmegaZSize", C.c_int), ("LambdaGSize", C.c_int),
        ("regLambda", C.c_double), ("dampGamma", C.c_double),
        ("stats_decay", C.c_double), ("momentum", C.c_double),
        ("checkGrad", C.c_int), ("inverseFreq", C.c_int),
    ]


class TRUST_REGION_PARAMS(C.Structure):  # solvers/params.h:11-33
    _fields_ = [
        ("delta", C.c_double), ("minDelta", C.c_double), ("maxDelta", C.c_double),
        ("eta1", C.c_double), ("eta2", C.c_double), ("gamma1", C.c_double), ("gamma2", C.c_double),
        ("maxProps", C.c_ulong), ("maxMatVecs", C.c_int), ("maxEpochs", C.c_int),
        ("maxIters", C.c_int), ("hessianType", C.c_int), ("alpha", C.c_double),
        ("curIteration", C.c_int), ("hs", C.c_double), ("lambda_", C.c_double),
    ]


class TR_STEP(C.Structure):
    _fields_ = [
        ("trainLikelihood", C.c_double), ("newTrainLikelihood", C.c_double),
        ("newTrainAccuracy", C.c_double), ("modelKfac", C.c_double), ("modelGradient", C.c_double),
        ("rho", C.c_double), ("delta", C.c_double), ("usedKfac", C.c_int), ("reverted", C.c_int),
    ]


class TR_EPOCH(C.Structure):
    _fields_ = [
        ("testLikelihood", C.c_double), ("testAccuracy", C.c_double),
        ("trainLikelihood", C.c_double), ("trainAccuracy", C.c_double),
        ("seconds", C.c_double), ("miniBatches", C.c_int),
    ]


class CG_PARAMS(C.Structure):
    _fields_ = [
        ("delta", C.c_double), ("tolerance", C.c_double), ("maxIterations", C.c_int),
        ("weightDecay", C.c_double),
        ("iterations", C.c_int), ("flag", C.c_int), ("modelValue", C.c_double),
        ("hvCalls", C.c_int),
    ]


def describe_model(convs, fcs, batch_size, bias):
    """Fill the caller-owned part of a CNN_MODEL.

    convs: list of dicts {cin, cout, h, w, k, pad, stride(=1), bn(bool), act,
           pool: (type, size, stride, pad) or None}
    fcs:   list of (in, out, act)
    The derived fields (offsets, sizes) are filled by a `*_model_finalize` call.
    """
    m = CNN_MODEL()
    m.cLayers, m.lLayers = len(convs), len(fcs)
    m.bias, m.batchSize = int(bool(bias)), int(batch_size)
    any_bn = False
    for i, c in enumerate(convs):
        L = m.convLayer[i]
        L.inChannels, L.outChannels = c["cin"], c["cout"]
        L.height, L.width = c["h"], c["w"]
        L.kSize, L.padding, L.stride = c["k"], c["pad"], c.get("stride", 1)
        L.batchNorm = BATCH_NORM if c.get("bn") else NO_BATCH_NORM
        any_bn = any_bn or bool(c.get("bn"))
        m.actFuns[i] = c["act"]
        P = m.poolLayer[i]
        if c.get("pool"):
            P.type, P.pSize, P.stride, P.padding = c["pool"]
        else:
            P.type, P.pSize, P.stride, P.padding = NO_POOL, 2, 2, 0
    m.enableBatchNorm = int(any_bn)
    for i, (fin, fout, act) in enumerate(fcs):
        F = m.fcLayer[i]
        F.in_, F.out, F.actFun = fin, fout, act
    return m
