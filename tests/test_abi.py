"""CPU tests of the drop-in boundary: the shared library loads without a GPU,
exports every symbol include/qmatmul.h declares, and reports errors as codes."""
import ctypes
import os

import pytest

import lib_b200
from lib_b200 import _capi


def test_library_exports_every_declared_symbol():
    names = _capi.declared_symbols()
    assert len(names) >= 22
    raw = ctypes.CDLL(_capi._LIB_PATH)
    for n in names:
        assert hasattr(raw, n), "libqmatmul.so does not export %s" % n


def test_version_and_error_strings():
    assert lib_b200.lib.qm_version() == 100
    assert b"multiple of the block" in lib_b200.lib.qm_error_string(-1)
    assert b"insufficient" in lib_b200.lib.qm_error_string(-2)
    assert lib_b200.lib.qm_error_string(-12345) is not None


def test_null_arguments_are_errors_not_crashes():
    L = lib_b200.lib
    assert L.qm_init(0, None) == -5
    assert L.qm_destroy(None) == -5
    assert L.qm_sync(None) == -5
    assert L.qm_matvec(None, 0, 0, 0, 1, 0, 0, 0, 0) == -5
    assert L.qm_launch_count(None) == -1


def test_kernel_images_and_descriptions_are_built():
    d = os.path.join(os.path.dirname(_capi._LIB_PATH), "csrc", "build")
    for stem in ("qm_gemv", "qm_dequant", "qm_gemv_q4k"):
        cubin = os.path.join(d, stem + ".sm_100a.cubin")
        assert os.path.getsize(cubin) > 1000
        assert open(cubin, "rb").read(4) == b"\x7fELF"
        assert os.path.exists(os.path.join(d, stem + ".sm_100a.json"))


@pytest.mark.skipif(os.path.exists("/dev/nvidiactl"), reason="only meaningful without a GPU")
def test_no_gpu_means_no_context_and_no_fallback():
    with pytest.raises(lib_b200.QmError) as e:
        lib_b200.Context(0)
    assert e.value.code in (-6, 100, 999, 3)  # no driver library / no device
