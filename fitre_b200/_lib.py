"""Loads libfitre_b200.so (built in-tree by fitre_b200.build) and declares its C ABI.

There is no CPU fallback: if the CUDA library is missing the import fails loudly.
"""
import ctypes as C
import os

from . import _structs as S

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libfitre_b200.so")

# every symbol include/fitre_b200.h declares
SYMBOLS = [
    "fitre_context_create", "fitre_context_destroy", "fitre_last_error", "fitre_launch_count",
    "fitre_set_reference_softmax", "fitre_set_reference_quadratic_damping", "fitre_set_scratch_limit", "fitre_kernel_launches", "fitre_set_precision", "fitre_set_kfac_solver", "fitre_set_kfac_distribution", "fitre_get_kfac_solver", "fitre_kfac_matrix_factor", "fitre_set_graphs", "fitre_set_tma", "fitre_profile_enable", "fitre_profile_read",
    "fitre_comm_unique_id", "fitre_comm_init", "fitre_comm_world", "fitre_set_comm_timeout", "fitre_peer_reduce_enabled", "fitre_peer_wait_selftest",
    "fitre_read_lenet_cnn", "fitre_read_alexnet_cnn", "fitre_read_vgg11", "fitre_read_test_vgg",
    "fitre_model_finalize", "fitre_model_validate",
    "fitre_cnn_forward_mem_required", "fitre_cnn_backward_mem_required",
    "fitre_cnn_rop_forward_mem_required", "fitre_cnn_rop_backward_mem_required",
    "fitre_cnn_gradient_mem_required", "fitre_cnn_hv_mem_required",
    "fitre_cnn_forward", "fitre_cnn_backward", "fitre_compute_cnn_gradient",
    "fitre_cnn_rop_forward", "fitre_cnn_rop_backward", "fitre_cnn_hv",
    "fitre_quadratic_model_mem_required", "fitre_compute_quadratic_model", "fitre_cg_steihaug",
    "fitre_compute_distribution_errors", "fitre_kfac_storage_indices", "fitre_kfac_mem_required", "fitre_kfac_omega_z",
    "fitre_kfac_lambda_delta", "fitre_kfac_inverse_mem_required", "fitre_kfac_matrix_inverse",
    "fitre_update_running_stats", "fitre_kfac_speedup_omega_z", "fitre_kfac_speedup_lambda_delta",
    "fitre_kfac_omega_z_damped", "fitre_kfac_lambda_delta_damped",
    "fitre_kfac_invert_factors_mem_required", "fitre_kfac_invert_factors",
    "fitre_kfac_factors_and_inverses_mem_required", "fitre_kfac_factors_and_inverses",
    "fitre_kfac_omega_z_begin", "fitre_kfac_lambda_delta_finish",
    "fitre_kfac_natural_gradient_mem_required", "fitre_compute_natural_gradient",
    "fitre_syrk_tn_static_scratch", "fitre_gradient_hv_host", "fitre_set_host_results_shared", "fitre_set_host_inputs_replicated",
    "fitre_init_batch_norm_data", "fitre_evaluate_cnn_model", "fitre_compute_accuracy",
    "fitre_select_column_matrix", "fitre_prepare_minibatch", "fitre_generalization_mem_required",
    "fitre_compute_generalization_errors", "fitre_trust_region_kfac_mem_required",
    "fitre_subsampled_trust_region_kfac", "fitre_write_vector", "fitre_read_vector",
]

_lib = None


def load():
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            "fitre_b200: %s is missing -- build it with `python -m fitre_b200.build` "
            "(there is no CPU fallback)" % LIB_PATH)
    L = C.CDLL(LIB_PATH)
    vp, i, d, l = C.c_void_p, C.c_int, C.c_double, C.c_long
    MP = C.POINTER(S.CNN_MODEL)
    DP = C.POINTER(S.DEVICE_DATASET)
    SP = C.POINTER(S.SCRATCH_AREA)
    dbl_p = C.POINTER(C.c_double)

    def sig(name, res, *args):
        f = getattr(L, name)
        f.restype = res
        f.argtypes = list(args)

    sig("fitre_context_create", i, C.POINTER(vp), i, vp)
    sig("fitre_context_destroy", i, vp)
    sig("fitre_last_error", C.c_char_p, vp)
    sig("fitre_launch_count", C.c_longlong, vp)
    sig("fitre_set_reference_softmax", i, vp, i)
    sig("fitre_set_reference_quadratic_damping", i, vp, i)
    sig("fitre_kernel_launches", C.c_longlong, vp, C.c_char_p)
    sig("fitre_set_precision", i, vp, i)
    sig("fitre_set_kfac_solver", i, vp, i)
    sig("fitre_set_graphs", i, vp, i)
    sig("fitre_set_host_results_shared", i, vp, i)
    sig("fitre_set_host_inputs_replicated", i, vp, i)
    sig("fitre_set_kfac_distribution", i, vp, i)
    sig("fitre_get_kfac_solver", i, vp)
    sig("fitre_kfac_matrix_factor", i, vp, vp, vp, i, d, d)
    sig("fitre_set_tma", i, vp, i)
    sig("fitre_profile_enable", i, vp, i)
    sig("fitre_profile_read", i, vp, i, dbl_p, dbl_p, C.POINTER(C.c_long))
    sig("fitre_comm_unique_id", i, vp)
    sig("fitre_comm_init", i, vp, vp, i, i)
    sig("fitre_comm_world", i, vp)
    sig("fitre_set_comm_timeout", i, vp, d)
    sig("fitre_peer_reduce_enabled", i, vp)
    sig("fitre_peer_wait_selftest", i, vp, d)
    sig("fitre_read_lenet_cnn", i, MP, i, i, i, i, i, i, i, i)
    sig("fitre_read_alexnet_cnn", i, MP, i, i, i, i, i, i, i)
    sig("fitre_read_vgg11", i, MP, i, i, i, i, i, i, i, i)
    sig("fitre_read_test_vgg", i, MP, i, i, i, i, i, i, i, i)
    sig("fitre_model_finalize", i, MP)
    sig("fitre_model_validate", i, MP)
    for n in ("forward", "backward", "rop_forward", "rop_backward", "gradient", "hv"):
        sig("fitre_cnn_%s_mem_required" % n, l, MP)
    sig("fitre_kfac_mem_required", l, MP)
    sig("fitre_cnn_forward", i, vp, MP, DP, SP, vp, vp, vp, i, i, i, dbl_p)
    sig("fitre_cnn_backward", i, vp, MP, DP, vp, vp, vp, vp, vp, vp, i, i, vp)
    sig("fitre_compute_cnn_gradient", i, vp, MP, DP, SP, vp, vp, vp, vp, vp, i, i, d, dbl_p)
    sig("fitre_cnn_rop_forward", i, vp, MP, DP, SP, vp, vp, vp, i, i, vp, vp)
    sig("fitre_cnn_rop_backward", i, vp, MP, DP, SP, vp, vp, vp, vp, vp, vp, vp, i, i, vp, vp)
    sig("fitre_cnn_hv", i, vp, MP, DP, vp, vp, vp, vp, vp, vp, i, i, vp, vp, d)
    sig("fitre_quadratic_model_mem_required", l, MP)
    sig("fitre_compute_quadratic_model", i, vp, MP, DP, vp, vp, vp, vp, vp, vp, d, i, i, d,
        vp, vp, vp, dbl_p)
    sig("fitre_cg_steihaug", i, vp, MP, DP, vp, vp, vp, vp, vp, vp, i, vp, C.POINTER(S.CG_PARAMS))
    sig("fitre_compute_distribution_errors", i, vp, vp, vp, vp, vp, i, i)
    sig("fitre_kfac_storage_indices", i, MP, C.POINTER(S.KFAC_INFO))
    sig("fitre_kfac_omega_z", i, vp, MP, DP, vp, i, vp, C.POINTER(S.KFAC_INFO), vp)
    sig("fitre_kfac_lambda_delta", i, vp, MP, vp, i, vp, C.POINTER(S.KFAC_INFO), vp)
    sig("fitre_kfac_inverse_mem_required", l, i)
    sig("fitre_kfac_matrix_inverse", i, vp, vp, vp, i, vp, d, d)
    KP = C.POINTER(S.KFAC_INFO)
    sig("fitre_update_running_stats", i, vp, vp, vp, l, d)
    sig("fitre_kfac_speedup_omega_z", i, vp, KP, MP, DP, i, vp, vp, vp, i)
    sig("fitre_kfac_speedup_lambda_delta", i, vp, KP, MP, i, vp, vp, i)
    sig("fitre_kfac_omega_z_damped", i, vp, MP, vp, vp, i, vp, KP, vp)
    sig("fitre_kfac_lambda_delta_damped", i, vp, MP, vp, i, vp, KP, vp)
    sig("fitre_kfac_invert_factors_mem_required", l, MP)
    sig("fitre_kfac_invert_factors", i, vp, MP, C.POINTER(S.KFAC_INFO), vp, vp, vp, vp, vp)
    sig("fitre_kfac_factors_and_inverses_mem_required", l, MP)
    sig("fitre_kfac_factors_and_inverses", i, vp, MP, vp, vp, vp, i, i, vp, vp, vp, vp, C.POINTER(S.KFAC_INFO), vp)
    sig("fitre_kfac_omega_z_begin", i, vp, MP, vp, vp, i, i, vp, vp, C.POINTER(S.KFAC_INFO), vp)
    sig("fitre_kfac_lambda_delta_finish", i, vp, MP, vp, i, i, vp, vp, C.POINTER(S.KFAC_INFO), vp)
    sig("fitre_kfac_natural_gradient_mem_required", l, MP)
    sig("fitre_compute_natural_gradient", i, vp, MP, C.POINTER(S.KFAC_INFO), vp, vp, vp, vp, vp)
    sig("fitre_syrk_tn_static_scratch", i, vp, l, i, l, d, vp, vp)
    sig("fitre_gradient_hv_host", i, vp, MP, vp, vp, vp, vp, i, i, d, dbl_p, vp, vp)
    sig("fitre_init_batch_norm_data", i, vp, MP, vp)
    sig("fitre_evaluate_cnn_model", i, vp, MP, DP, SP, vp, vp, vp, i, i, dbl_p)
    sig("fitre_compute_accuracy", i, vp, vp, vp, i, i, dbl_p, dbl_p)
    sig("fitre_select_column_matrix", i, vp, DP, i, vp, i)
    sig("fitre_prepare_minibatch", i, vp, MP, DP, vp, vp, vp, l, i, vp)
    sig("fitre_generalization_mem_required", l, MP)
    sig("fitre_compute_generalization_errors", i, vp, MP, DP, SP, vp, vp, vp, i, dbl_p, dbl_p)
    sig("fitre_trust_region_kfac_mem_required", l, MP, DP, C.POINTER(S.KFAC_INFO))
    sig("fitre_subsampled_trust_region_kfac", i, vp, MP, DP, C.POINTER(S.KFAC_INFO),
        C.POINTER(S.TRUST_REGION_PARAMS), SP, C.c_ulonglong, i, i, C.POINTER(S.TR_STEP), i,
        C.POINTER(S.TR_EPOCH))
    sig("fitre_write_vector", i, C.c_char_p, vp, l, i)
    sig("fitre_read_vector", i, C.c_char_p, vp, l, C.POINTER(C.c_long))
    _lib = L
    return L
