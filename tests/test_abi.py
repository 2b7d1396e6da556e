"""The C ABI without a GPU: the shared library loads, exports every function the header
declares, and the ctypes table covers the same set.  No compute call is made."""
import ctypes
import os
import re

from parallelreverseautodiff_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "prad_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(prad_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_functions():
    names = _declared()
    assert "prad_matmul_backward" in names and "prad_clip_adam" in names
    assert len(names) >= 55


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(_lib.LIB_PATH)
    missing = [n for n in _declared() if not hasattr(lib, n)]
    assert not missing, f"declared in prad_cuda.h but not exported: {missing}"


def test_ctypes_table_matches_header():
    bound = set(_lib.SIGNATURES) | set(_lib.STRING_FUNCS)
    assert bound == set(_declared())


def test_no_device_means_a_status_code_not_a_fallback():
    lib = _lib.load()
    ctx = ctypes.c_void_p()
    st = lib.prad_init(0, ctypes.byref(ctx))
    if st == 0:      # a GPU is present: nothing to check here
        lib.prad_shutdown(ctx)
        return
    assert st in (_lib.ERR_NOT_INITIALIZED, _lib.ERR_UNSUPPORTED)
    assert lib.prad_last_error()
    # a dead context is refused, never dereferenced
    assert lib.prad_sync(None) == _lib.ERR_NOT_INITIALIZED


def test_package_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "parallelreverseautodiff_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                src = open(os.path.join(dirpath, f)).read()
                assert "import oracle" not in src and "from oracle" not in src, f
                assert "prad_oracle" not in src, f


def test_managed_binding_file_is_current_and_complete():
    """integration/PradCuda.cs is generated from the header: it must be up to date and carry one
    [DllImport] for every exported function, and every enum value of the header."""
    import importlib.util
    path = os.path.join(ROOT, "integration", "make_bindings.py")
    spec = importlib.util.spec_from_file_location("make_bindings", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    on_disk = open(os.path.join(ROOT, "integration", "PradCuda.cs")).read()
    assert mod.generate() == on_disk, "run python integration/make_bindings.py"
    for name in _declared():
        assert re.search(r"extern\s+\w+\s+%s\(" % name, on_disk), name
    assert on_disk.count("[DllImport(") == len(_declared())
    for value in ("AmplifiedSigmoid = 6", "ErrTimeout = 8", "Div = 19"):
        assert value in on_disk
