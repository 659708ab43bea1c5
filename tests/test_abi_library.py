"""The C-ABI library loads on a machine without a GPU and exports every symbol the header declares."""
import ctypes
import os
import re
import sys

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


REFERENCE = os.environ.get("FORGE_REFERENCE_ROOT", os.path.join(os.path.dirname(ROOT), "reference"))


@pytest.mark.skipif(not os.path.isdir(os.path.join(REFERENCE, "forge", "utils")), reason="no reference checkout here")
def test_package_coexists_with_the_reference_checkout():
    """The reference driver's imports (quant.py:15-17: `import forge.utils`, `from forge.gptq import GPTQ`) with this
    package AHEAD of the reference on sys.path: forge.gptq / forge.backend come from here, forge.utils from the
    reference.  Run in a child interpreter so that this process's import state does not matter; third-party packages
    the reference's utils import at module level and that are not installed here get empty stand-ins."""
    import subprocess
    import textwrap
    code = textwrap.dedent(f"""
        import sys, types, importlib.machinery
        import transformers  # before the stand-ins: it probes for optional packages with find_spec
        sys.path[:0] = [{os.path.join(ROOT, '4bit-forge_b200')!r}, {REFERENCE!r}]
        for name, attrs in (("accelerate", ("init_empty_weights",)), ("accelerate.utils", ("set_module_tensor_to_device",)),
                            ("huggingface_hub", ("hf_hub_download",)), ("datasets", ("load_dataset",))):
            try:
                __import__(name)
            except Exception:
                m = types.ModuleType(name)
                m.__spec__ = importlib.machinery.ModuleSpec(name, None)
                for a in attrs:
                    setattr(m, a, None)
                sys.modules[name] = m
        import forge.utils
        from forge.gptq import GPTQ
        from forge.backend.cuda import kernels
        import forge, forge.moe
        ours = {os.path.join(ROOT, '4bit-forge_b200', 'forge')!r}
        assert forge.gptq.__file__.startswith(ours), forge.gptq.__file__
        assert forge.utils.__file__.startswith({os.path.join(REFERENCE, 'forge', 'utils')!r}), forge.utils.__file__
        assert hasattr(forge.utils.engine, "dequantize_forge_full") and hasattr(forge.utils.io, "_apply_block_scale_inv_2d")
        assert hasattr(kernels, "gptq_solver") and hasattr(GPTQ, "quantize")
        print("coexist ok")
    """)
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "coexist ok" in r.stdout, r.stderr[-2000:]
