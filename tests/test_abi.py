"""CPU tests of the drop-in boundary: the shared library loads, exports every symbol that
include/mascot.h declares, and fails loudly (no CPU fallback) when no GPU is usable."""
import ctypes as C
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "mascot.h")).read()
    return re.findall(r"^MASCOT_API\s+[\w\s\*]+?\b(mascot_\w+)\s*\(", text, flags=re.M)


def test_header_declares_the_expected_surface():
    names = declared_symbols()
    assert len(names) == len(set(names)) and len(names) >= 32
    for must in ("mascot_create", "mascot_set_ratings", "mascot_train_epoch", "mascot_eval_rmse",
                 "mascot_get_factors", "mascot_get_group_info", "mascot_destroy", "mascot_rmse_host"):
        assert must in names


def test_library_exports_every_declared_symbol(mascot):
    lib = mascot.load()
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} is declared in include/mascot.h but not exported"
    assert set(mascot.EXPORTS) <= set(declared_symbols())


def test_config_defaults_follow_the_reference_cli(mascot):
    cfg = mascot.default_config()
    # main.cu:19-32
    assert cfg.k == 128 and cfg.epoch == 50 and cfg.num_workers == 2048 and cfg.thread_block_size == 128
    assert cfg.user_group_num == 10 and cfg.item_group_num == 10 and cfg.version == 7 and cfg.interval == 1
    assert np.float32(cfg.lambda_) == np.float32(0.015) and np.float32(cfg.learning_rate) == np.float32(0.01)
    assert np.float32(cfg.decay) == np.float32(0.1) and np.float32(cfg.sample_ratio) == np.float32(0.01)
    assert np.float32(cfg.error_threshold) == np.float32(0.001)
    assert cfg.shuffle == 1 and cfg.deterministic == 0
    ver, csz, ssz = C.c_uint32(), C.c_uint32(), C.c_uint32()
    assert mascot.load().mascot_abi_info(C.byref(ver), C.byref(csz), C.byref(ssz)) == 0
    assert (ver.value, csz.value, ssz.value) == (1, C.sizeof(mascot.Config), C.sizeof(mascot.EpochStats))


def test_bad_arguments_are_rejected_without_touching_a_gpu(mascot):
    lib = mascot.load()
    assert lib.mascot_config_default(None) == mascot.ERR_BAD_ARG
    h = C.c_void_p()
    cfg = mascot.default_config(k=96)
    assert lib.mascot_create(C.byref(cfg), C.byref(h)) == mascot.ERR_BAD_ARG
    assert b"k must be 64 or 128" in lib.mascot_last_error(None)
    cfg = mascot.default_config(version=9)
    assert lib.mascot_create(C.byref(cfg), C.byref(h)) == mascot.ERR_BAD_ARG
    assert lib.mascot_create(None, C.byref(h)) == mascot.ERR_BAD_ARG
    assert lib.mascot_destroy(None) == mascot.OK
    assert lib.mascot_status_string(mascot.ERR_NO_DEVICE) == b"no usable CUDA device"


def test_no_cpu_fallback(mascot):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(mascot.MascotError) as e:
        mascot.Engine(mascot.default_config(version=mascot.V_SGD))
    assert e.value.status == mascot.ERR_NO_DEVICE
    with pytest.raises(mascot.MascotError) as e:
        mascot.rmse_host(np.zeros((4, 64), np.float32), np.zeros((4, 64), np.float32),
                         np.zeros(3, mascot.RATING), 64)
    assert e.value.status == mascot.ERR_NO_DEVICE
