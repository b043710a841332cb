"""ctypes binding of the CPU oracle (oracle/libfitre_oracle.so) for the tests.

Only tests, the smoke check and the benchmark's CPU-baseline leg may use this module.
"""
import ctypes as C
import os
import subprocess

import numpy as np

from fitre_b200 import _structs as S

_HERE = os.path.dirname(os.path.abspath(__file__))
_ORACLE_DIR = os.path.join(os.path.dirname(_HERE), "oracle")
_LIB = None

dp = np.ctypeslib.ndpointer(dtype=np.float64, flags="C_CONTIGUOUS")
ALLREDUCE_FN = C.CFUNCTYPE(None, C.POINTER(C.c_double), C.c_long, C.c_void_p)


class ORA_ENV(C.Structure):
    _fields_ = [("ref_softmax", C.c_int), ("world", C.c_int),
                ("allreduce", ALLREDUCE_FN), ("user", C.c_void_p), ("eval_type", C.c_int),
                ("rank", C.c_int), ("ref_quadratic", C.c_int)]


def lib():
    global _LIB
    if _LIB is None:
        so = os.path.join(_ORACLE_DIR, "libfitre_oracle.so")
        src = os.path.join(_ORACLE_DIR, "fitre_oracle.c")
        if not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
            subprocess.check_call(["make", "-C", _ORACLE_DIR, "libfitre_oracle.so"])
        L = C.CDLL(so)
        MP, EP = C.POINTER(S.CNN_MODEL), C.POINTER(ORA_ENV)
        i, d = C.c_int, C.c_double
        L.ora_set_num_threads.argtypes = [i]
        L.ora_set_num_threads.restype = None
        L.ora_model_finalize.argtypes = [MP]
        L.ora_model_finalize.restype = i
        L.ora_cnn_gradient.argtypes = [EP, MP, dp, dp, dp, i, dp, dp, dp, dp, dp, i, d]
        L.ora_cnn_gradient.restype = d
        L.ora_cnn_forward.argtypes = [EP, MP, dp, dp, dp, i, dp, dp, dp, i]
        L.ora_cnn_forward.restype = d
        L.ora_cnn_hv.argtypes = [EP, MP, dp, dp, i, dp, dp, dp, dp, dp, dp, dp, i]
        L.ora_cnn_hv.restype = None
        L.ora_quadratic_model.argtypes = [EP, MP, dp, dp, i, dp, dp, dp, dp, dp, dp, d, i, d]
        L.ora_quadratic_model.restype = d
        L.ora_cg_steihaug.argtypes = [EP, MP, dp, dp, i, dp, dp, dp, dp, dp, dp, i,
                                      C.POINTER(S.CG_PARAMS)]
        L.ora_cg_steihaug.restype = None
        L.ora_kfac_storage_indices.argtypes = [MP, C.POINTER(S.KFAC_INFO)]
        L.ora_kfac_storage_indices.restype = i
        L.ora_kfac_omega_z.argtypes = [EP, MP, dp, dp, i, dp, C.POINTER(S.KFAC_INFO)]
        L.ora_kfac_lambda_delta.argtypes = [EP, MP, dp, i, dp, C.POINTER(S.KFAC_INFO)]
        L.ora_kfac_matrix_inverse.argtypes = [dp, dp, i, d, d]
        L.ora_kfac_matrix_inverse.restype = i
        L.ora_natural_gradient.argtypes = [MP, C.POINTER(S.KFAC_INFO), dp, dp, dp, dp]
        L.ora_cnn_backward.argtypes = [EP, MP, dp, dp, dp, dp, dp, dp, i]
        L.ora_distribution_errors.argtypes = [EP, dp, dp, i, i, dp, dp]
        L.ora_softmax_loss.argtypes = [EP, dp, dp, i, i, dp]
        L.ora_softmax_loss.restype = d
        L.ora_im2col.argtypes = [dp, i, i, i, i, i, i, i, dp]
        L.ora_im2col_index.argtypes = [i, i, i, i, i, i, i,
                                       np.ctypeslib.ndpointer(dtype=np.int64, flags="C_CONTIGUOUS")]
        L.ora_max_pool_argmax.argtypes = [dp, i, i, i, i, i, i, i,
                                          np.ctypeslib.ndpointer(dtype=np.int32, flags="C_CONTIGUOUS")]
        L.ora_pool_forward.argtypes = [dp, i, i, i, i, i, i, i, i, dp]
        L.ora_batch_norm_forward.argtypes = [EP, dp, i, i, i, i, dp, dp, dp, d]
        L.ora_batch_norm_backward.argtypes = [EP, dp, i, i, i, i, dp, dp, d, dp]
        L.ora_rop_batch_norm_forward.argtypes = [EP, dp, dp, dp, dp, d, i, i, i, i, dp]
        L.ora_rop_batch_norm_backward.argtypes = [EP, dp, dp, dp, dp, dp, dp, d, dp, dp, i, i, i, i]
        L.ora_conv_dgrad.argtypes = [dp, i, i, i, dp, i, i, i, i, i, i, dp]
        L.ora_gemm.argtypes = [i, i, C.c_long, C.c_long, C.c_long, d, dp, C.c_long, dp, C.c_long,
                               d, dp, C.c_long]
        ip = np.ctypeslib.ndpointer(dtype=np.int32, flags="C_CONTIGUOUS")
        L.ora_init_batch_norm_data.argtypes = [MP, dp]
        L.ora_compute_accuracy.argtypes = [EP, dp, dp, i, i, C.POINTER(C.c_double)]
        L.ora_compute_accuracy.restype = d
        L.ora_prepare_minibatch.argtypes = [dp, dp, C.c_void_p, C.c_long, i, i, i, i, i, C.c_void_p,
                                            dp, dp]
        KP = C.POINTER(S.KFAC_INFO)
        L.ora_update_running_stats.argtypes = [dp, dp, C.c_long, d]
        L.ora_kfac_speedup_omega_z.argtypes = [KP, MP, dp, C.c_long, i, dp, dp, dp, i]
        L.ora_kfac_speedup_lambda_delta.argtypes = [KP, MP, i, dp, dp, i]
        L.ora_kfac_omega_z_damped.argtypes = [EP, MP, dp, dp, i, dp, KP]
        L.ora_kfac_lambda_delta_damped.argtypes = [EP, MP, dp, i, dp, KP]
        L.ora_generalization_errors.argtypes = [EP, MP, dp, dp, C.c_long, i, dp, i, dp, i,
                                                C.POINTER(C.c_double), C.POINTER(C.c_double)]
        L.ora_subsampled_trust_region_kfac.argtypes = [
            EP, MP, dp, dp, C.c_long, C.c_void_p, C.c_void_p, C.c_long, i, dp, i,
            C.POINTER(S.KFAC_INFO), C.POINTER(S.TRUST_REGION_PARAMS), C.c_ulonglong, i, i,
            C.POINTER(S.TR_STEP), i, C.POINTER(S.TR_EPOCH)]
        L.ora_subsampled_trust_region_kfac.restype = i
        _LIB = L
    return _LIB


def make_env(ref_softmax=1, world=1, allreduce=None, eval_type=10, rank=0, ref_quadratic=1):
    env = ORA_ENV()
    env.rank = int(rank)
    env.ref_quadratic = int(ref_quadratic)
    env.ref_softmax, env.world = int(ref_softmax), int(world)
    env.eval_type = int(eval_type)
    if allreduce is not None:
        env._cb = ALLREDUCE_FN(allreduce)  # keep alive
        env.allreduce = env._cb
    return env


def finalize(model):
    rc = lib().ora_model_finalize(C.byref(model))
    if rc != 0:
        raise ValueError("ora_model_finalize failed: %d" % rc)
    return model


class OracleState:
    """Buffers of one oracle gradient evaluation (z, dx, probs, errors, gradient)."""

    def __init__(self, model, n, num_classes):
        self.z = np.zeros(model.zSize)
        self.dx = np.zeros(model.zSize)
        self.rz = np.zeros(model.zSize)
        self.probs = np.zeros(n * num_classes)
        self.errors = np.zeros(max(model.maxDeltaSize, n * num_classes))
        self.gradient = np.zeros(model.pSize)
        self.loss = None


def gradient(model, batch, labels, weights, num_classes, n, weight_decay=0.0, env=None):
    env = env or make_env()
    st = OracleState(model, n, num_classes)
    st.loss = lib().ora_cnn_gradient(C.byref(env), C.byref(model), batch, labels, weights,
                                     num_classes, st.z, st.dx, st.probs, st.errors, st.gradient,
                                     n, weight_decay)
    return st


def hv(model, batch, weights, num_classes, n, st, vector, env=None):
    env = env or make_env()
    out = np.zeros(model.pSize)
    lib().ora_cnn_hv(C.byref(env), C.byref(model), batch, weights, num_classes, st.z, st.probs,
                     st.errors, st.dx, np.ascontiguousarray(vector), out, st.rz, n)
    return out


def prepare_minibatch(setX, setY, indices, offset, n, C_, H, W, dataset_type=10, uniforms=None):
    """Oracle minibatch assembly; returns (batch [C][N][W][H] flat, labels)."""
    batch = np.zeros(n * C_ * H * W)
    labels = np.zeros(n)
    idx = None if indices is None else np.ascontiguousarray(indices, dtype=np.int32)
    u = None if uniforms is None else np.ascontiguousarray(uniforms, dtype=np.float64)
    lib().ora_prepare_minibatch(np.ascontiguousarray(setX), np.ascontiguousarray(setY),
                                None if idx is None else idx.ctypes.data, int(offset), int(n), C_, H,
                                W, int(dataset_type), None if u is None else u.ctypes.data, batch,
                                labels)
    return batch, labels


def trust_region_kfac(model, trainX, trainY, testX, testY, weights, num_classes, info, tr, seed=1,
                      enable_da=1, max_mini_batches=0, steps_cap=0, dataset_type=10, env=None):
    """Oracle FITRE loop; updates `weights` in place, returns (steps, epochs)."""
    env = env or make_env()
    steps = (S.TR_STEP * max(steps_cap, 1))()
    epochs = (S.TR_EPOCH * max(tr.maxIters, 1))()
    tX = None if testX is None else np.ascontiguousarray(testX)
    tY = None if testY is None else np.ascontiguousarray(testY)
    rc = lib().ora_subsampled_trust_region_kfac(
        C.byref(env), C.byref(model), np.ascontiguousarray(trainX), np.ascontiguousarray(trainY),
        int(trainY.size), None if tX is None else tX.ctypes.data,
        None if tY is None else tY.ctypes.data, 0 if tY is None else int(tY.size),
        int(dataset_type), weights, int(num_classes), C.byref(info), C.byref(tr), int(seed),
        int(enable_da), int(max_mini_batches), steps, int(steps_cap), epochs)
    if rc:
        raise RuntimeError("oracle loop: a factor was not positive definite")
    n = min(steps_cap, tr.curIteration)
    return list(steps[:n]), list(epochs[:tr.maxIters])
