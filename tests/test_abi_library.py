"""The C-ABI library loads on a machine without a GPU and exports every symbol the header declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    src = open(os.path.join(ROOT, "include", "forge_b200.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(forge_[a-z0-9_]+)\s*\(", src)))


def test_header_symbols_exported():
    from forge import _abi
    lib = _abi.load_library()
    names = _declared()
    assert len(names) >= 18
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/forge_b200.h but not exported"
    # the Python prototypes cover the same set
    assert sorted(_abi.exported_symbols()) == names


def test_version_and_error_string():
    from forge import _abi
    lib = _abi.load_library()
    assert lib.forge_version() >= 100
    assert isinstance(lib.forge_last_error(), bytes)


def test_argument_validation_needs_no_gpu():
    """Null pointers are rejected before any CUDA call."""
    from forge import _abi
    lib = _abi.load_library()
    rc = lib.forge_pack_int4(None, None, 4, 8, 8, None, None)
    assert rc == 1
    assert b"null" in lib.forge_last_error()
    assert lib.forge_chol_workspace_bytes(2, 128) >= 2 * 2 * 2 * 64 * 64 * 4


def test_no_cpu_fallback_without_cuda():
    import torch
    if torch.cuda.is_available():
        pytest.skip("CUDA present")
    from forge.backend.cuda import kernels
    with pytest.raises(RuntimeError):
        kernels.build_group_meta_packed(torch.zeros(4, 32), 4, True)


def test_product_does_not_import_oracle():
    pkg = os.path.join(ROOT, "4bit-forge_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                txt = open(os.path.join(dirpath, f)).read()
                assert "ref_port" not in txt and "forge_oracle" not in txt, f
