"""The C-ABI library loads without a GPU and exports every entry point the header declares."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
LIB = ROOT / "kvskip_b200" / "libkvskip_b200.so"


def declared():
    text = "\n".join(p.read_text() for p in sorted((ROOT / "include").glob("*.h")))
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(kvskip_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_reference_launchers():
    names = declared()
    for n in ("kvskip_launch_decode", "kvskip_launch_vskip1", "kvskip_launch_pv", "kvskip_launch_plan",
              "kvskip_launch_update", "kvskip_launch_read", "kvskip_max_smem_bytes", "kvskip_last_error"):
        assert n in names


def test_library_exports_every_declared_symbol():
    if not LIB.exists():
        from kvskip_b200 import build
        build.build_lib()
    lib = ctypes.CDLL(str(LIB))
    for n in declared():
        assert hasattr(lib, n), f"{n} declared in include/ but not exported"
    assert lib.kvskip_version() >= 100
    lib.kvskip_last_error.restype = ctypes.c_char_p
    assert lib.kvskip_last_error() == b""
    # argument errors are reported without touching a device
    assert lib.kvskip_launch_decode(None, 128, 4, 2, 0, 0, 1, None) == -1
    assert b"null" in lib.kvskip_last_error()
    assert lib.kvskip_max_smem_bytes(128, 2, 1) > 48 * 1024


def test_ctypes_structs_match_header_sizes():
    """Field-by-field mirror in kvskip_b200/cabi.py: sizes as the C compiler lays them out."""
    import subprocess, tempfile
    from kvskip_b200 import cabi
    src = '#include <stdio.h>\n#include "kvskip_b200.h"\nint main(){printf("%zu %zu %zu", sizeof(kvskip_params), sizeof(kvskip_plan_params), sizeof(kvskip_update_params));return 0;}\n'
    with tempfile.TemporaryDirectory() as d:
        c = Path(d) / "s.c"
        c.write_text(src)
        subprocess.run(["/usr/bin/gcc", "-I", str(ROOT / "include"), str(c), "-o", str(Path(d) / "s")], check=True)
        out = subprocess.run([str(Path(d) / "s")], capture_output=True, text=True, check=True).stdout.split()
    assert [int(x) for x in out] == [ctypes.sizeof(cabi.Params), ctypes.sizeof(cabi.PlanParams),
                                     ctypes.sizeof(cabi.UpdateParams)]


def test_front_end_fails_loudly_without_extension(monkeypatch, tmp_path):
    """No CPU fallback: a missing extension is an error, not a slower path."""
    from kvskip_b200 import kvskip as K
    from kvskip_b200 import build
    monkeypatch.setattr(K, "_EXT", None)
    monkeypatch.setattr(build, "EXT", tmp_path / "_kvskip_ext.so")
    monkeypatch.setenv("KVSKIP_NO_BUILD", "1")
    with pytest.raises(RuntimeError):
        K.ext()
