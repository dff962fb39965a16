"""The C-ABI library loads here (no GPU) and exports exactly what include/glmflash_b200.h declares."""
import ctypes as C
import os
import re

import pytest

from conftest import ROOT


def declared():
    text = open(os.path.join(ROOT, "include", "glmflash_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(glmflash_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(pkg):
    import __graft_entry__ as entry
    entry.build()
    lib = C.CDLL(pkg.SO_PATH)
    names = declared()
    assert len(names) >= 30
    for n in names:
        assert hasattr(lib, n), f"{n} declared in the header but not exported"
    assert sorted(pkg.SYMBOLS) == names, "python binding and header disagree"


def test_handshakes(pkg):
    L = pkg.lib()
    assert L.glmflash_abi_version() == 1
    assert L.glmflash_config_bytes() == C.sizeof(pkg.Config) == 64
    assert L.glmflash_weights_bytes() == C.sizeof(pkg.Weights) == 72
    import threading
    seen = []
    t = threading.Thread(target=lambda: seen.append(L.glmflash_error()))     # the last error is per thread: a new one has none
    t.start()
    t.join()
    assert seen == [b""]


def test_constructors_reject_bad_config_without_touching_a_gpu(pkg):
    L = pkg.lib()
    h = C.c_void_p()
    cfg = pkg.make_config(hidden=2048, inter=1536, experts=64, slots=5, max_rows=17)     # > 16 rows
    assert L.glmflash_experts_new(C.byref(cfg), C.sizeof(cfg), C.byref(h)) == -1 and not h.value
    assert b"max_rows" in L.glmflash_error()
    cfg = pkg.make_config(hidden=2000)
    assert L.glmflash_grouping_new(C.byref(cfg), C.sizeof(cfg), C.byref(h)) == -1
    assert b"hidden" in L.glmflash_error()
    cfg = pkg.make_config()
    assert L.glmflash_moe_new(C.byref(cfg), C.sizeof(cfg) - 4, C.byref(h)) == -1
    assert b"size mismatch" in L.glmflash_error()


def test_no_cpu_fallback(pkg):
    import torch
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    L = pkg.lib()
    h = C.c_void_p()
    cfg = pkg.make_config()
    assert L.glmflash_experts_new(C.byref(cfg), C.sizeof(cfg), C.byref(h)) == -1
    assert b"no CUDA device" in L.glmflash_error()
    with pytest.raises(pkg.GlmFlashError):
        pkg.ExpertGpu(cfg)


def test_every_entry_point_is_declared_and_has_a_binding_line():
    """The header, the ctypes table and the reference-side binding shown to maintainers name the same entry points."""
    import re
    from conftest import ROOT
    import __graft_entry__ as entry
    pkg = entry.load_package()
    header = open(os.path.join(ROOT, "include", "glmflash_b200.h")).read()
    stub = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    declared = set(re.findall(r"\b(glmflash_[a-z0-9_]+)\s*\(", header))
    assert declared == set(pkg.SYMBOLS), declared ^ set(pkg.SYMBOLS)
    assert not [s for s in pkg.SYMBOLS if "fn " + s + "(" not in stub]
