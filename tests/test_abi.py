"""CPU checks of the drop-in boundary: the library loads and exports every symbol the
header declares; argument validation answers without a device."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from ferrograd_b200 import build, _lib
    build.build()
    return _lib.load()


def header_functions():
    text = open(os.path.join(ROOT, "include", "ferrograd_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fg_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_functions():
    names = header_functions()
    assert len(names) >= 40
    for must in ("fg_gemm_f32", "fg_gemm_bwd_f32", "fg_softmax_ce_fwd_bwd", "fg_adamw_step", "fg_sgd_step",
                 "fg_eltwise_chain_fwd", "fg_eltwise_chain_bwd", "fg_plan_begin", "fg_allreduce_sum_f32"):
        assert must in names


def test_library_exports_every_declared_symbol(lib):
    from ferrograd_b200 import _lib
    raw = C.CDLL(_lib.LIB_PATH)
    for name in header_functions():
        assert hasattr(raw, name), f"{name} declared in the header but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no Python signature"
    assert set(_lib.SIGNATURES) <= set(header_functions())


def test_version_string(lib):
    assert b"sm_100a" in lib.fg_version()


def test_null_context_is_rejected(lib):
    # No device is touched: a NULL context short-circuits to NotInitialized.
    assert lib.fg_sync(None) == 8
    assert lib.fg_sgd_step(None, None, None, 0, 0.0, 1.0, 1) == 8
    assert lib.fg_gemm_f32(None, 0, 0, 0, 1, 1, 1, None, None, None, None, 0, None) == 8
    assert lib.fg_plan_begin(None) == 8


def test_context_creation_fails_cleanly_without_device(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    h = C.c_void_p()
    code = lib.fg_ctx_create(0, C.byref(h))
    assert code == 3 and not h.value   # FG_ERR_INVALID_DEVICE, no fallback context


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from ferrograd_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(ImportError):
        _lib.load()


def test_noalloc_mse_limit_matches_its_static_scratch():
    # the largest accepted n uses exactly the last of the 4096 static partial sums (65,536 elements each);
    # checked on the header's constant, so that the 1 GiB inputs need not be allocated
    m = re.search(r"#define\s+FG_MSE_NOALLOC_MAX_N\s+(\d+)ull", open(os.path.join(ROOT, "include", "ferrograd_b200.h")).read())
    assert m, "FG_MSE_NOALLOC_MAX_N not found in the header"
    n = int(m.group(1))
    assert (n + 65536 - 1) // 65536 == 4096 and (n + 1 + 65536 - 1) // 65536 == 4097
