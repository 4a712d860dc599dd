"""CPU-side checks of the boundary: the shared library builds, loads and exports every symbol that
include/manta_b200.h declares; the oracle and the package stay separate."""
import os
import re

from manta_b200 import native

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols(header="manta_b200.h"):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(manta_b200_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from manta_b200 import build

    build.build()
    lib = native.load()
    declared = _declared_symbols()
    assert declared, "no declarations found"
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    assert sorted(native.EXPORTS) == sorted(declared)
    host = _declared_symbols("manta_b200_host.h")
    assert len(host) >= 8
    for name in host:
        assert hasattr(lib, name), f"{name} is declared in the host header but not exported"


def test_header_cites_reference_for_each_entry_point():
    text = open(os.path.join(ROOT, "include", "manta_b200.h")).read()
    assert text.count(".go:") >= 15


def test_package_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "manta_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".cpp")):
                src = open(os.path.join(dirpath, f)).read()
                assert "import oracle" not in src and "from oracle" not in src and "manta_oracle" not in src, f
