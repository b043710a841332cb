"""CPU checks of the boundary: the shared library loads without a GPU, exports every symbol
include/fitre_b200.h declares, the ctypes struct mirrors have the C sizes, the builders and
validators (pure host code) behave, and a context cannot be created without a CUDA device."""
import ctypes as C
import os
import re

import pytest

import nets
import oracle_lib as O
from fitre_b200 import _lib, api
from fitre_b200 import _structs as S

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    text = open(os.path.join(ROOT, "include", "fitre_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fitre_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    L = _lib.load()
    syms = header_symbols()
    assert len(syms) >= 30
    missing = [s for s in syms if not hasattr(L, s)]
    assert not missing, missing
    assert sorted(_lib.SYMBOLS) == syms  # the Python binding list tracks the header


def test_struct_sizes_match_c_layout():
    # CONV_LAYER 22 ints, POOL_LAYER 8 ints, FC_LAYER 5 ints (nn/nn_decl.h:64-121)
    assert C.sizeof(S.CONV_LAYER) == 22 * 4
    assert C.sizeof(S.POOL_LAYER) == 8 * 4
    assert C.sizeof(S.FC_LAYER) == 5 * 4
    ints = 20 * 22 + 20 + 20 * 8 + 2 + 20 * 5 + 7 + 3 * 20 + 1 + 2 * 20
    assert C.sizeof(S.CNN_MODEL) == ints * 4
    assert C.sizeof(S.SCRATCH_AREA) == 6 * 8


def test_builders_agree_with_oracle_offsets():
    for mine, theirs in ((api.readVGG11(16, 32, 32, 10, 3, 0, 1), nets.vgg11(16)),
                         (api.readAlexNetCNN(8, 32, 32, 10, 0, 1), nets.alexnet(8)),
                         (api.readLenetCNN(3, 32, 32, 8, 1, 0), nets.lenet(8)),
                         (api.readTestVGG(10, 4, 4, 10, 2, 1, 0), nets.test_vgg(10))):
        O.finalize(theirs)
        assert bytes(mine)[:C.sizeof(S.CNN_MODEL) - 80] is not None
        for f in ("pSize", "zSize", "maxDeltaSize", "cLayers", "lLayers", "zztSize"):
            assert getattr(mine, f) == getattr(theirs, f), f
        assert list(mine.wOffsets) == list(theirs.wOffsets)
        assert list(mine.bOffsets) == list(theirs.bOffsets)
        assert list(mine.zOffsets) == list(theirs.zOffsets)
        for l in range(mine.cLayers):
            for f, _ in S.CONV_LAYER._fields_:
                assert getattr(mine.convLayer[l], f) == getattr(theirs.convLayer[l], f), (l, f)


def test_validate_rejects_unsupported_shapes():
    L = _lib.load()
    m = nets.vgg_small(4)
    api.finalize(m)
    assert L.fitre_model_validate(C.byref(m)) == S.OK
    m2 = nets.vgg_small(4)
    m2.convLayer[1].stride = 2
    api.finalize(m2)
    assert L.fitre_model_validate(C.byref(m2)) in (S.ERR_UNSUPPORTED, S.ERR_BAD_ARG)
    m3 = nets.vgg_small(4)
    m3.poolLayer[0].pSize, m3.poolLayer[0].stride, m3.poolLayer[0].padding = 3, 2, 0
    api.finalize(m3)
    assert L.fitre_model_validate(C.byref(m3)) in (S.ERR_UNSUPPORTED, S.ERR_BAD_ARG)
    m4 = nets.vgg_small(4)
    m4.actFuns[0] = S.CNN_ACT_ELU
    api.finalize(m4)
    assert L.fitre_model_validate(C.byref(m4)) == S.ERR_UNSUPPORTED


def test_mem_required_is_far_below_materialised_im2col():
    m = api.readVGG11(512, 32, 32, 10, 3, 0, 1)
    need = api.mem_required(m, "backward")
    # the reference sizes its scratch for the largest im2col matrix, M*K doubles
    # (functions/cnn_backward.cu:51-74): layer 1 at 512 images is 131072 x 576
    assert 0 < need < 131072 * 576 // 2


def test_no_context_without_cuda_device():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    with pytest.raises(api.FitreError):
        api.Context(0)


def test_no_alloc_entry_point_checks_arguments_on_host():
    L = _lib.load()
    assert L.fitre_syrk_tn_static_scratch(None, 4, 4, 4, 1.0, None, None) == S.ERR_BAD_ARG
