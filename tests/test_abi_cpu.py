"""The C-ABI library: builds, loads, exports every declared symbol, rejects bad arguments.
No kernel is launched here (no GPU needed)."""
import ctypes
import os
import re

import pytest

from conftest import ROOT
from cats_b200 import _build, _lib


def declared_functions():
    src = open(os.path.join(ROOT, "include", "cats_b200.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(cats_[a-z_0-9]+)\s*\(", src)))


def test_library_builds_and_loads():
    path = _build.build()
    assert os.path.exists(path)
    L = _lib.lib()
    assert L.cats_abi_version() == 1


def test_every_declared_symbol_is_exported_and_bound():
    L = _lib.lib()
    names = declared_functions()
    assert len(names) >= 15
    for n in names:
        assert hasattr(L, n), f"{n} declared in include/cats_b200.h but not exported"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes signature"
    assert sorted(_lib.SIGNATURES) == names


def test_workspace_size_is_monotonic_and_covers_lists():
    L = _lib.lib()
    a = L.cats_workspace_bytes(1, 4096, 11008)
    b = L.cats_workspace_bytes(1, 4096, 14336)
    c = L.cats_workspace_bytes(16, 8192, 28672)
    assert 0 < a < b < c
    # two int lists + two fp32 [I, 16] arrays + [16, H] accumulators at least
    assert b >= 2 * 4 * 14336 + 2 * 4 * 16 * 14336 + 4 * 16 * 4096
    assert L.cats_workspace_bytes(1, 0, 14336) == 0


@pytest.mark.parametrize("status,needle", [(-1, "dtype"), (-2, "shape"), (-3, "aligned"),
                                           (-4, "NULL"), (-5, "workspace"), (-7, "mode"),
                                           (-8, "cats_mlp_static")])
def test_status_strings(status, needle):
    assert needle.lower() in _lib.lib().cats_status_string(status).decode().lower()


def test_argument_errors_are_status_codes_not_exits():
    """Bad arguments come back as negative codes before anything is launched (the reference
    prints and exits the process: flash_gemv/csrc/cuda/fuse_gemv_cmp_cuda.cu:2397-2400)."""
    L = _lib.lib()
    buf = ctypes.create_string_buffer(1 << 16)
    p = ctypes.addressof(buf)
    p16 = (p + 15) // 16 * 16
    big = 1 << 30
    # dtype
    assert L.cats_gate(p16, p16, p16, big, 1, 64, 32, 9, 0.1, None, None, None) == -1
    # batch out of range (reference supports {1,2,8,16}; here 1..16)
    assert L.cats_gate(p16, p16, p16, big, 17, 64, 32, 1, 0.1, None, None, None) == -2
    assert L.cats_gate(p16, p16, p16, big, 0, 64, 32, 1, 0.1, None, None, None) == -2
    # H not a whole number of 16-byte vectors
    assert L.cats_gate(p16, p16, p16, big, 1, 68, 32, 1, 0.1, None, None, None) == -2
    assert L.cats_gate(p16, p16, p16, big, 1, 66, 32, 0, 0.1, None, None, None) == -2
    # null / misaligned pointers
    assert L.cats_gate(None, p16, p16, big, 1, 64, 32, 1, 0.1, None, None, None) == -4
    assert L.cats_gate(p16 + 2, p16, p16, big, 1, 64, 32, 1, 0.1, None, None, None) == -3
    # workspace too small
    assert L.cats_gate(p16, p16, p16, 1024, 1, 64, 32, 1, 0.1, None, None, None) == -5
    # modes of the down projection
    assert L.cats_updown(p16, p16, p16, p16, big, 1, 64, 32, 1, p16, 5, None, None, None, 0.0,
                         None) == -7
    assert L.cats_updown(p16, p16, p16, p16, big, 1, 64, 32, 1, p16, 1, p16, None, None, 0.0,
                         None) == -7
    assert L.cats_updown(p16, p16, p16, p16, big, 1, 64, 32, 1, None, 0, None, None, None, 0.0,
                         None) == -4
    with pytest.raises(RuntimeError, match="dtype"):
        _lib.check(-1, "cats_gate")
