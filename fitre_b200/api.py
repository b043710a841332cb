"""Host-side mirror of the reference's operator interface for the CNN gradient /
Hessian-vector path, on top of the C ABI (include/fitre_b200.h).

Function names, argument order and meaning follow the reference:
  computeCNNGradient  functions/cnn_gradient.h:9-12
  cnnForward          functions/cnn_forward.h:11-13
  cnnBackward         functions/cnn_backward.h:13-16
  cnnHv               functions/cnn_hessian_vec.h:9-13
  computeQuadraticModel functions/model_reduction.cu:20-93
Device buffers are torch CUDA tensors of dtype float64 (torch is only the allocator); the
structs are the ctypes mirrors in _structs.py.  Errors raise FitreError(status, text)
instead of the reference's print-and-exit (device/cuda_utils.h:28-92).
"""
import ctypes as C

from . import _lib
from . import _structs as S


class FitreError(RuntimeError):
    def __init__(self, status, text):
        super().__init__("fitre status %d: %s" % (status, text))
        self.status = status


def _ptr(t):
    if t is None:
        return None
    if isinstance(t, int):
        return C.c_void_p(t)
    if hasattr(t, "data_ptr"):
        import torch
        if t.dtype != torch.float64 or not t.is_cuda or not t.is_contiguous():
            raise FitreError(S.ERR_BAD_ARG, "device buffers must be contiguous float64 CUDA tensors")
        return C.c_void_p(t.data_ptr())
    raise TypeError(type(t))


class Context:
    """One per GPU (reference: the global handles of device/handles.h:15-20)."""

    def __init__(self, device=0, stream=None):
        self.lib = _lib.load()
        h = C.c_void_p()
        sp = C.c_void_p(stream) if stream else None
        rc = self.lib.fitre_context_create(C.byref(h), int(device), sp)
        if rc != S.OK:
            raise FitreError(rc, "fitre_context_create failed (is a CUDA device visible?)")
        self.h = h
        self.device = device

    def close(self):
        if getattr(self, "h", None):
            self.lib.fitre_context_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def check(self, rc):
        if rc != S.OK:
            raise FitreError(rc, self.lib.fitre_last_error(self.h).decode())

    @property
    def launches(self):
        return int(self.lib.fitre_launch_count(self.h))

    def set_reference_softmax(self, on):
        self.check(self.lib.fitre_set_reference_softmax(self.h, int(bool(on))))

    def set_reference_quadratic_damping(self, on):
        """1 (default): computeQuadraticModel adds weightDecay * weights to Hv as the C reference
        does (functions/model_reduction.cu:50-52); 0: weightDecay * vector (pytorch/peng/utils.py:77)."""
        self.check(self.lib.fitre_set_reference_quadratic_damping(self.h, int(bool(on))))

    def set_scratch_limit(self, doubles):
        """Doubles available behind the scratch pointers of the following calls (0 = unchecked)."""
        self.check(self.lib.fitre_set_scratch_limit(self.h, int(doubles)))

    def kernel_launches(self, name):
        """Launches issued so far of the kernel called `name` (e.g. "conv_tma_kernel")."""
        return int(self.lib.fitre_kernel_launches(self.h, name.encode()))

    def set_precision(self, precision):
        """0 = fp64 (reference arithmetic); opt-in tcgen05 modes for the convolution products:
        1 = one TF32 product (loss within 1e-3, deep-net gradients only within 1e-1),
        2 = error-compensated 3 x TF32 (gradient and Hv within 1e-3 of fp64)."""
        self.check(self.lib.fitre_set_precision(self.h, int(precision)))

    def set_kfac_solver(self, solver):
        """0 = explicit damped inverses of the A blocks (reference form); 1 = Cholesky factors in
        the same slots, applied by two triangular solves in the natural gradient."""
        self.check(self.lib.fitre_set_kfac_solver(self.h, int(solver)))

    def set_kfac_distribution(self, mode):
        """With ranks: 0 = every rank holds all factors and inverses; 1 = each layer's factors live
        on an owner rank, which also forms that layer's slice of the natural gradient."""
        self.check(self.lib.fitre_set_kfac_distribution(self.h, int(mode)))

    def set_host_results_shared(self, on):
        """gradientHvHost's result buffers are one shared, page-locked segment on every rank:
        each rank copies its share only (see fitre_set_host_results_shared)."""
        self.check(self.lib.fitre_set_host_results_shared(self.h, int(bool(on))))

    def set_host_inputs_replicated(self, on):
        """gradientHvHost's weights and vector hold the same values on every rank: each rank uploads
        one chunk, the chunks are all-gathered on the device (see fitre_set_host_inputs_replicated)."""
        self.check(self.lib.fitre_set_host_inputs_replicated(self.h, int(bool(on))))

    def set_graphs(self, on):
        """CUDA-graph replay of the factor-inverse and natural-gradient launch sequences (default on)."""
        self.check(self.lib.fitre_set_graphs(self.h, int(bool(on))))

    def set_tma(self, on):
        self.check(self.lib.fitre_set_tma(self.h, int(bool(on))))

    def profile_enable(self, on):
        self.check(self.lib.fitre_profile_enable(self.h, int(bool(on))))

    def profile_read(self, kind):
        """(device ms, algorithmic flops, launches) of kernel class `kind` since the last read."""
        ms, fl, n = C.c_double(), C.c_double(), C.c_long()
        self.check(self.lib.fitre_profile_read(self.h, kind, C.byref(ms), C.byref(fl), C.byref(n)))
        return ms.value, fl.value, n.value

    def comm_init_from_torch(self):
        """Create the NCCL communicator over torch.distributed's default group (plumbing:
        the 128-byte unique id is broadcast from rank 0 with the group's own backend)."""
        import torch
        import torch.distributed as dist
        rank, world = dist.get_rank(), dist.get_world_size()
        buf = (C.c_ubyte * 128)()
        if rank == 0:
            rc = self.lib.fitre_comm_unique_id(C.cast(buf, C.c_void_p))
            if rc != S.OK:
                raise FitreError(rc, "fitre_comm_unique_id failed")
        dev = "cuda" if dist.get_backend() == "nccl" else "cpu"
        t = torch.tensor(list(buf), dtype=torch.uint8, device=dev)
        dist.broadcast(t, src=0)
        raw = bytes(t.cpu().tolist())
        idbuf = (C.c_ubyte * 128).from_buffer_copy(raw)
        self.check(self.lib.fitre_comm_init(self.h, C.cast(idbuf, C.c_void_p), rank, world))

    def set_comm_timeout(self, seconds):
        """Bound (seconds) of communicator set-up and of every host wait on a collective."""
        self.check(self.lib.fitre_set_comm_timeout(self.h, float(seconds)))

    @property
    def peer_reduce_enabled(self):
        """True when short vectors are all-reduced by the library's own kernel over peer memory."""
        return bool(self.lib.fitre_peer_reduce_enabled(self.h))

    def peer_wait_selftest(self, wait_ms):
        """Runs the peer all-reduce kernel against a flag nothing raises; raises FitreError(ERR_COMM)."""
        self.check(self.lib.fitre_peer_wait_selftest(self.h, float(wait_ms)))

    def comm_init(self, unique_id_bytes, rank, world):
        """fitre_comm_init with an id obtained from comm_unique_id() on rank 0."""
        idbuf = (C.c_ubyte * 128).from_buffer_copy(bytes(unique_id_bytes))
        self.check(self.lib.fitre_comm_init(self.h, C.cast(idbuf, C.c_void_p), int(rank), int(world)))

    @staticmethod
    def comm_unique_id():
        buf = (C.c_ubyte * 128)()
        rc = _lib.load().fitre_comm_unique_id(C.cast(buf, C.c_void_p))
        if rc != S.OK:
            raise FitreError(rc, "fitre_comm_unique_id failed")
        return bytes(buf)

    @property
    def world(self):
        return int(self.lib.fitre_comm_world(self.h))


def finalize(model):
    rc = _lib.load().fitre_model_finalize(C.byref(model))
    if rc != S.OK:
        raise FitreError(rc, "fitre_model_finalize")
    return model


def readLenetCNN(channels, width, height, batchSize, enableBias, enableBatchNorm,
                 actFun=S.CNN_ACT_SWISH, poolType=S.AVG_POOL):
    m = S.CNN_MODEL()
    rc = _lib.load().fitre_read_lenet_cnn(C.byref(m), channels, width, height, batchSize,
                                          enableBias, enableBatchNorm, actFun, poolType)
    if rc != S.OK:
        raise FitreError(rc, "fitre_read_lenet_cnn")
    return m


def readAlexNetCNN(batchSize, height, width, numClasses, enableBias, enableBatchNorm,
                   actFun=S.CNN_ACT_SWISH):
    m = S.CNN_MODEL()
    rc = _lib.load().fitre_read_alexnet_cnn(C.byref(m), batchSize, height, width, numClasses,
                                            enableBias, enableBatchNorm, actFun)
    if rc != S.OK:
        raise FitreError(rc, "fitre_read_alexnet_cnn")
    return m


def readVGG11(batchSize, height, width, numClasses, inChannels, bias, enableBatchNorm,
              actFun=S.CNN_ACT_SWISH):
    m = S.CNN_MODEL()
    rc = _lib.load().fitre_read_vgg11(C.byref(m), batchSize, height, width, numClasses,
                                      inChannels, bias, enableBatchNorm, actFun)
    if rc != S.OK:
        raise FitreError(rc, "fitre_read_vgg11")
    return m


def readTestVGG(batchSize, height, width, numClasses, inChannels, bias, bn,
                actFun=S.CNN_ACT_SOFTPLUS):
    m = S.CNN_MODEL()
    rc = _lib.load().fitre_read_test_vgg(C.byref(m), batchSize, height, width, numClasses,
                                         inChannels, bias, bn, actFun)
    if rc != S.OK:
        raise FitreError(rc, "fitre_read_test_vgg")
    return m


def make_dataset(weights, currentBatch, sampledTrainY, numClasses):
    d = S.DEVICE_DATASET()
    d.weights = weights.data_ptr()
    d.currentBatch = currentBatch.data_ptr()
    d.sampledTrainY = sampledTrainY.data_ptr()
    d.numClasses = int(numClasses)
    d._keep = (weights, currentBatch, sampledTrainY)
    return d


def make_scratch(dev_tensor):
    s = S.SCRATCH_AREA()
    s.devWorkspace = dev_tensor.data_ptr()
    s.nextDevPtr = dev_tensor.data_ptr()
    s._keep = dev_tensor
    return s


def mem_required(model, which):
    return int(getattr(_lib.load(), "fitre_cnn_%s_mem_required" % which)(C.byref(model)))


def computeCNNGradient(ctx, model, data, scratch, z, dx, probs, lossFuncErrors, gradient,
                       offset, curBatchSize, weightDecay):
    loss = C.c_double()
    ctx.check(ctx.lib.fitre_compute_cnn_gradient(
        ctx.h, C.byref(model), C.byref(data), C.byref(scratch), _ptr(z), _ptr(dx), _ptr(probs),
        _ptr(lossFuncErrors), _ptr(gradient), offset, curBatchSize, float(weightDecay),
        C.byref(loss)))
    return loss.value


def cnnForward(ctx, model, data, scratch, z, probs, errors, s, curBatchSize, evalType=S.MODEL_TRAIN):
    loss = C.c_double()
    ctx.check(ctx.lib.fitre_cnn_forward(ctx.h, C.byref(model), C.byref(data), C.byref(scratch),
                                        _ptr(z), _ptr(probs), _ptr(errors), s, curBatchSize,
                                        evalType, C.byref(loss)))
    return loss.value


def cnnBackward(ctx, model, data, devPtr, z, gradient, dx, delta, delta_new, offset, batchSize,
                hostPtr=None):
    ctx.check(ctx.lib.fitre_cnn_backward(ctx.h, C.byref(model), C.byref(data), _ptr(devPtr),
                                         _ptr(z), _ptr(gradient), _ptr(dx), _ptr(delta),
                                         _ptr(delta_new), offset, batchSize, None))


def cnnHv(ctx, model, data, z, probs, lossFuncErrors, dx, vector, hv, s, curBatchSize, devPtr,
          hostPtr=None, weightDecay=0.0):
    ctx.check(ctx.lib.fitre_cnn_hv(ctx.h, C.byref(model), C.byref(data), _ptr(z), _ptr(probs),
                                   _ptr(lossFuncErrors), _ptr(dx), _ptr(vector), _ptr(hv), s,
                                   curBatchSize, _ptr(devPtr), None, float(weightDecay)))


def computeQuadraticModel(ctx, model, data, z, probs, lossFuncErrors, dx, gradient, vector, delta,
                          offset, curBatchSize, weightDecay, devPtr, hostPtr=None, pageLckPtr=None):
    val = C.c_double()
    ctx.check(ctx.lib.fitre_compute_quadratic_model(
        ctx.h, C.byref(model), C.byref(data), _ptr(z), _ptr(probs), _ptr(lossFuncErrors), _ptr(dx),
        _ptr(gradient), _ptr(vector), float(delta), offset, curBatchSize, float(weightDecay),
        _ptr(devPtr), None, None, C.byref(val)))
    return val.value


def cgSteihaug(ctx, model, data, z, probs, lossFuncErrors, dx, gradient, p, curBatchSize, devPtr,
               params):
    ctx.check(ctx.lib.fitre_cg_steihaug(ctx.h, C.byref(model), C.byref(data), _ptr(z), _ptr(probs),
                                        _ptr(lossFuncErrors), _ptr(dx), _ptr(gradient), _ptr(p),
                                        curBatchSize, _ptr(devPtr), C.byref(params)))
    return params


def computeDistributionErrors(ctx, probs, uniforms, distTarget, distError, rows, num_classes):
    """functions/softmax_loss.cu:104-136 with injected uniforms."""
    ctx.check(ctx.lib.fitre_compute_distribution_errors(ctx.h, _ptr(probs), _ptr(uniforms),
                                                        _ptr(distTarget), _ptr(distError), rows,
                                                        num_classes))


def computeKFACStorageIndices(model):
    info = S.KFAC_INFO()
    rc = _lib.load().fitre_kfac_storage_indices(C.byref(model), C.byref(info))
    if rc != S.OK:
        raise FitreError(rc, "fitre_kfac_storage_indices")
    return info


def computeOmegaZ(ctx, model, data, z, samples, omegaZ, info, devPtr):
    ctx.check(ctx.lib.fitre_kfac_omega_z(ctx.h, C.byref(model), C.byref(data), _ptr(z), samples,
                                         _ptr(omegaZ), C.byref(info), _ptr(devPtr)))


def computeLambdaDelta(ctx, model, dx, samples, lambdaG, info, devPtr):
    ctx.check(ctx.lib.fitre_kfac_lambda_delta(ctx.h, C.byref(model), _ptr(dx), samples,
                                              _ptr(lambdaG), C.byref(info), _ptr(devPtr)))


def computeMatrixInverse(ctx, matrix, inverse, n, devPtr, lam, dampGamma):
    """solvers/kfac_inverses.cu:133-186: inverse = (matrix + (lam + dampGamma) I)^-1."""
    ctx.check(ctx.lib.fitre_kfac_matrix_inverse(ctx.h, _ptr(matrix), _ptr(inverse), n, _ptr(devPtr),
                                                float(lam), float(dampGamma)))


def computeMatrixFactor(ctx, matrix, factor, n, lam, gamma):
    """Packed Cholesky factor of matrix + (lam + gamma) I (the Cholesky form of one A block)."""
    ctx.check(ctx.lib.fitre_kfac_matrix_factor(ctx.h, _ptr(matrix), _ptr(factor), n, lam, gamma))


def computeNaturalGradient(ctx, model, info, omegaZInv, lambdaGInv, gradient, nGradient, devPtr):
    """solvers/kfac_natural_gradient.cu:36-241."""
    ctx.check(ctx.lib.fitre_compute_natural_gradient(ctx.h, C.byref(model), C.byref(info),
                                                     _ptr(omegaZInv), _ptr(lambdaGInv),
                                                     _ptr(gradient), _ptr(nGradient), _ptr(devPtr)))


def gradientHvHost(ctx, model, batch, labels, weights, vector, curBatchSize, numClasses,
                   weightDecay, gradient_out, hv_out):
    """Host-buffer entry point: numpy / pinned torch CPU arrays in and out."""
    def hp(a):
        if hasattr(a, "data_ptr"):
            return C.c_void_p(a.data_ptr())
        return C.c_void_p(a.ctypes.data)
    loss = C.c_double()
    ctx.check(ctx.lib.fitre_gradient_hv_host(ctx.h, C.byref(model), hp(batch), hp(labels),
                                             hp(weights), hp(vector), curBatchSize, numClasses,
                                             float(weightDecay), C.byref(loss), hp(gradient_out),
                                             hp(hv_out)))
    return loss.value


class Workspace:
    """Every device buffer one model needs for gradient + Hessian-vector calls, sized with the
    library's *_mem_required figures (the reference carves the same buffers from one big
    workspace: drivers/cnn_driver.cu:193-209)."""

    def __init__(self, model, num_classes, device="cuda"):
        import torch
        L = _lib.load()
        f64 = dict(dtype=torch.float64, device=device)
        n = model.batchSize
        self.model = model
        self.z = torch.zeros(model.zSize, **f64)
        self.dx = torch.zeros(model.zSize, **f64)
        self.probs = torch.zeros(n * num_classes, **f64)
        self.errors = torch.zeros(n * num_classes, **f64)
        self.gradient = torch.zeros(model.pSize, **f64)
        self.hv = torch.zeros(model.pSize, **f64)
        need = max(L.fitre_cnn_gradient_mem_required(C.byref(model)),
                   L.fitre_cnn_hv_mem_required(C.byref(model)))
        self.extra = 4 * (model.pSize + 32) + 64
        self.dev = torch.zeros(need + self.extra, **f64)
        self.scratch = make_scratch(self.dev)


# ---- training-loop pieces either side of the path -------------------------------------------

def make_full_dataset(weights, trainX, trainY, testX, testY, numClasses, features, batchSize,
                      datasetType=10):
    """DEVICE_DATASET over whole train / test sets (features x samples, column per image, as the
    reference stores them) with the sampled-batch buffers allocSampledDataset would provide."""
    import torch
    d = S.DEVICE_DATASET()
    d.weights = weights.data_ptr()
    d.trainSetX, d.trainSetY = trainX.data_ptr(), trainY.data_ptr()
    d.trainSizeX = d.trainSizeY = int(trainY.numel())
    if testX is not None:
        d.testSetX, d.testSetY = testX.data_ptr(), testY.data_ptr()
        d.testSizeX = d.testSizeY = int(testY.numel())
    d.numClasses, d.features, d.datasetType = int(numClasses), int(features), int(datasetType)
    sx = torch.zeros(2 * batchSize * features, dtype=torch.float64, device=weights.device)
    sy = torch.zeros(batchSize, dtype=torch.float64, device=weights.device)
    d.sampledTrainX, d.sampledTrainY = sx.data_ptr(), sy.data_ptr()
    d.currentBatch = sx.data_ptr()
    d.sampleSize = int(batchSize)
    d._keep = (weights, trainX, trainY, testX, testY, sx, sy)
    return d


def computeFactorsAndInverses(ctx, model, data, z, dx, samples, omegaZ, omegaZInv, lambdaG, lambdaGInv, info,
                              devPtr):
    """computeOmegaZ + computeLambdaDelta of the reference in one call (factors and their damped
    inverses, solvers/kfac_inverses.cu:450-630,759-857), factorisations overlapped with the factor
    products; live state (the batch, z, dx of the sampled-label backward pass)."""
    ctx.check(ctx.lib.fitre_kfac_factors_and_inverses(
        ctx.h, C.byref(model), data.currentBatch, z.data_ptr(), dx.data_ptr(), 0, int(samples),
        omegaZ.data_ptr(), omegaZInv.data_ptr(), lambdaG.data_ptr(), lambdaGInv.data_ptr(), C.byref(info),
        devPtr.data_ptr()))


def computeOmegaZBegin(ctx, model, data, z, samples, omegaZ, omegaZInv, info, devPtr):
    """A factors and their damped factorisations, started on the library's own streams; returns at
    once.  Pair with computeLambdaDeltaFinish; queue the sampled-label backward pass in between."""
    ctx.check(ctx.lib.fitre_kfac_omega_z_begin(
        ctx.h, C.byref(model), data.currentBatch, z.data_ptr(), 0, int(samples), omegaZ.data_ptr(),
        omegaZInv.data_ptr(), C.byref(info), devPtr.data_ptr()))


def computeLambdaDeltaFinish(ctx, model, dx, samples, lambdaG, lambdaGInv, info, devPtr):
    """G factors and inverses, then waits for everything computeOmegaZBegin started."""
    ctx.check(ctx.lib.fitre_kfac_lambda_delta_finish(
        ctx.h, C.byref(model), dx.data_ptr(), 0, int(samples), lambdaG.data_ptr(), lambdaGInv.data_ptr(),
        C.byref(info), devPtr.data_ptr()))


def invertFactors(ctx, model, info, omegaZ, omegaZInv, lambdaG, lambdaGInv, devPtr):
    """All damped factor inverses of one KFAC step (several streams, divided among ranks)."""
    ctx.check(ctx.lib.fitre_kfac_invert_factors(ctx.h, C.byref(model), C.byref(info), omegaZ.data_ptr(),
                                                omegaZInv.data_ptr(), lambdaG.data_ptr(),
                                                lambdaGInv.data_ptr(), devPtr.data_ptr()))


def initBatchNormData(ctx, model, z):
    ctx.check(ctx.lib.fitre_init_batch_norm_data(ctx.h, C.byref(model), z.data_ptr()))


def cnnForwardEval(ctx, model, data, scratch, z, probs, errors, curBatchSize, evalType):
    """cnnForward with an explicit EVAL_TYPE (10 train, 20 / 30 accuracy modes)."""
    loss = C.c_double()
    ctx.check(ctx.lib.fitre_cnn_forward(ctx.h, C.byref(model), C.byref(data), C.byref(scratch),
                                        z.data_ptr(), probs.data_ptr(), errors.data_ptr(), 0,
                                        int(curBatchSize), int(evalType), C.byref(loss)))
    return loss.value


def evaluateCNNModel(ctx, model, data, scratch, z, probs, lossFuncErrors, offset, curBatchSize):
    loss = C.c_double()
    ctx.check(ctx.lib.fitre_evaluate_cnn_model(ctx.h, C.byref(model), C.byref(data), C.byref(scratch),
                                               z.data_ptr(), probs.data_ptr(),
                                               lossFuncErrors.data_ptr(), int(offset),
                                               int(curBatchSize), C.byref(loss)))
    return loss.value


def computeAccuracy(ctx, probs, target, rows, numClasses):
    """Returns (hits, percent)."""
    hits, acc = C.c_double(), C.c_double()
    ctx.check(ctx.lib.fitre_compute_accuracy(ctx.h, probs.data_ptr(), target.data_ptr(), int(rows),
                                             int(numClasses), C.byref(hits), C.byref(acc)))
    return hits.value, acc.value


def prepareMinibatch(ctx, model, data, setX, setY, indices, offset, n, uniforms=None):
    ctx.check(ctx.lib.fitre_prepare_minibatch(
        ctx.h, C.byref(model), C.byref(data), setX.data_ptr(), setY.data_ptr(),
        indices.data_ptr() if indices is not None else None, int(offset), int(n),
        uniforms.data_ptr() if uniforms is not None else None))


def computeGeneralizationErrors(ctx, model, data, scratch, z, probs, errors, evalType):
    """Returns (likelihood, accuracy percent) over the test (30) or train (20) set."""
    lik, acc = C.c_double(), C.c_double()
    ctx.check(ctx.lib.fitre_compute_generalization_errors(
        ctx.h, C.byref(model), C.byref(data), C.byref(scratch), z.data_ptr(), probs.data_ptr(),
        errors.data_ptr(), int(evalType), C.byref(lik), C.byref(acc)))
    return lik.value, acc.value


def subsampledTrustRegionKFAC(ctx, model, data, kfacInfo, trParams, scratch, seed=1, enableDA=1,
                              maxMiniBatches=0, stepsCap=0):
    """Runs the FITRE loop; returns (steps, epochs) as lists of TR_STEP / TR_EPOCH."""
    steps = (S.TR_STEP * max(stepsCap, 1))()
    epochs = (S.TR_EPOCH * max(trParams.maxIters, 1))()
    ctx.check(ctx.lib.fitre_subsampled_trust_region_kfac(
        ctx.h, C.byref(model), C.byref(data), C.byref(kfacInfo), C.byref(trParams), C.byref(scratch),
        int(seed), int(enableDA), int(maxMiniBatches), steps, int(stepsCap), epochs))
    n = min(stepsCap, trParams.curIteration)
    return list(steps[:n]), list(epochs[:trParams.maxIters])


def writeVector(path, host_array, referenceFormat=0):
    import numpy as np
    a = np.ascontiguousarray(host_array, dtype=np.float64)
    rc = _lib.load().fitre_write_vector(str(path).encode(), a.ctypes.data, a.size, int(referenceFormat))
    if rc:
        raise OSError("fitre_write_vector failed for %s" % path)


def readVector(path, n):
    import numpy as np
    a = np.zeros(n)
    got = C.c_long()
    rc = _lib.load().fitre_read_vector(str(path).encode(), a.ctypes.data, n, C.byref(got))
    if rc:
        raise OSError("fitre_read_vector failed for %s" % path)
    return a[:got.value]
