"""The shared library loads without a GPU and exports every symbol the header declares."""
import ctypes
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    names = set()
    for header in (ROOT / "include").glob("*.h"):
        text = re.sub(r"/\*.*?\*/", "", header.read_text(), flags=re.S)
        names.update(re.findall(r"\b(stark_b200_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_library_exports_every_declared_symbol():
    from stark_b200 import _lib, build
    build.build()
    lib = ctypes.CDLL(str(_lib.LIB_PATH))
    names = declared_symbols()
    assert len(names) >= 10
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_abi_version_and_status_names():
    from stark_b200 import _lib
    lib = _lib.load()
    assert lib.stark_b200_abi_version() == _lib.ABI_VERSION
    for code, name in enumerate(_lib.STATUS_NAMES):
        assert lib.stark_b200_status_name(code).decode() == name
    assert lib.stark_b200_status_name(99).decode() == "unknown"


def test_binding_covers_header():
    from stark_b200 import _lib
    lib = _lib.load()
    for n in declared_symbols():
        assert getattr(lib, n).argtypes is not None, f"{n} has no ctypes signature in stark_b200/_lib.py"
