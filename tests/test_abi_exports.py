"""The C-ABI library loads and exports every symbol include/beholdd_b200.h declares
(no compute calls: this runs without a GPU)."""
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from exec_beholdd_b200 import build, device

    build.build()
    return device.load_library()


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "beholdd_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(bhd_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_what_the_binding_lists():
    from exec_beholdd_b200 import EXPORTS

    assert declared_symbols() == sorted(EXPORTS)


def test_library_exports_every_declared_symbol(lib):
    for name in declared_symbols():
        assert hasattr(lib, name), name


def test_pure_host_entry_points(lib):
    assert lib.bhd_device_name().decode() == "cuda-b200"
    assert lib.bhd_error_text(0).decode() == "ok"
    assert "shape" in lib.bhd_error_text(-2).decode()
    # Device::supports: crates/beholdd-backend/src/cpu.rs:1357-1366 lists what the CPU decodes.
    for kind in (0, 1, 8, 12, 13, 14):
        assert lib.bhd_supports(kind) == 1
    for kind in (2, 23, 9999):
        assert lib.bhd_supports(kind) == 0


def test_missing_library_fails_loudly(tmp_path):
    from exec_beholdd_b200 import device

    with pytest.raises(ImportError):
        device.load_library(str(tmp_path / "nope.so"))
