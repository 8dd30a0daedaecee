"""The C-ABI library: loads without a GPU, exports every symbol the header declares, and
its argument/config checks answer with the documented codes.  No kernel runs here."""
import ctypes
import os
import re

import pytest

from conftest import ROOT
from flextensor_b200 import backend

HEADER = os.path.join(ROOT, "include", "ftb200.h")


def _declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ftb_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported(native_lib):
    names = _declared_functions()
    assert len(names) >= 12
    for name in names:
        assert hasattr(native_lib, name), "header declares %s but the library does not export it" % name
    # and the Python binding knows each of them
    for name in names:
        assert name in backend.EXPORTED_SYMBOLS, name


def test_version_and_strerror(native_lib):
    assert native_lib.ftb_version() == 100
    assert native_lib.ftb_strerror(0) == b"ok"
    for code in range(-7, 0):
        assert native_lib.ftb_strerror(code) not in (b"ok", b"unknown error")
    assert native_lib.ftb_strerror(-99) == b"unknown error"


def test_config_struct_layout():
    assert ctypes.sizeof(backend.FtbConfig) == 16 * 4
    cfg = backend.FtbConfig.from_dict({"tile_n": 128, "cluster": 2, "stages": 5})
    assert cfg.to_dict()["tile_n"] == 128 and cfg.to_dict()["cluster"] == 2 and cfg.to_dict()["raster"] == 0
    with pytest.raises(KeyError):
        backend.FtbConfig.from_dict({"no_such_knob": 1})


def test_validate(native_lib):
    ok = backend.validate
    assert ok(backend.OP_BGEMM_BF16, None, 2048, 2048, 2048) == 0
    assert ok(backend.OP_BGEMM_BF16, {"cluster": 2, "tile_n": 256, "stages": 6}, 2048, 2048, 2048) == 0
    assert ok(backend.OP_BGEMM_BF16, {"cluster": 2, "tile_n": 256, "stages": 7}, 2048, 2048, 2048) == -3  # smem
    assert ok(backend.OP_BGEMM_BF16, {"cluster": 1, "tile_n": 256, "stages": 5}, 2048, 2048, 2048) == -3
    assert ok(backend.OP_BGEMM_BF16, {"tile_n": 48}, 64, 64, 64) == -3
    assert ok(backend.OP_BGEMM_BF16, {"split_k": 2}, 64, 64, 512) == -3      # split-K needs an fp32 output
    assert ok(backend.OP_GEMM_F32, {"split_k": 2}, 64, 64, 512) == 0
    assert ok(backend.OP_GEMM_F32, {"split_k": 64}, 64, 64, 64) == -3        # more splits than K blocks
    assert ok(backend.OP_GEMM_F32, {"fp32_mode": 1, "cluster": 2}, 512, 512, 512) == -3
    assert ok(backend.OP_GEMM_F32, {"fp32_mode": 2}, 512, 512, 512) == -3
    assert ok(backend.OP_CONV2D, {"cluster": 2}, 512, 64, 576) == 0
    assert ok(backend.OP_CONV2D, {"cluster": 2, "fp32_mode": 1}, 512, 64, 576) == -3
    assert ok(backend.OP_DWCONV2D, {"threads": 100}, 1, 1, 1) == -3
    assert ok(backend.OP_DWCONV2D, {"threads": 128, "tile_h": 7}, 1, 1, 1) == 0
    assert ok(9, None, 1, 1, 1) == -1
    assert ok(backend.OP_GEMM_F32, None, 0, 1, 1) == -1


def test_launchers_refuse_without_device(native_lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    assert native_lib.ftb_device_check() == -6
    # bad arguments are rejected before any device work
    assert native_lib.ftb_gemm_f32(None, None, None, 8, 8, 8, 0, 0, None, None, None) == -1
    buf = ctypes.create_string_buffer(4096)
    p = ctypes.cast(buf, ctypes.c_void_p)
    assert native_lib.ftb_gemm_f32(p, p, p, -1, 8, 8, 0, 0, None, None, None) == -1
    # well-formed call, no sm_100 device: refused, not executed on the CPU
    assert native_lib.ftb_gemm_f32(p, p, p, 16, 16, 16, 0, 0, None, None, None) == -6
    assert native_lib.ftb_launch_count() == 0


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(backend, "_lib", None)
    monkeypatch.setattr(backend, "_LIB_PATH", str(tmp_path / "nothing.so"))
    with pytest.raises(RuntimeError, match="no fallback"):
        backend.lib()


def test_product_does_not_import_the_oracle():
    pkg = os.path.join(ROOT, "flextensor_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert not re.search(r"\boracle\b", text), "%s mentions the oracle" % os.path.join(dirpath, f)
                assert not re.search(r"(^|[\s/\"'])_work/", text)
