"""The C-ABI library loads and exports every symbol include/gact_b200.h declares; argument validation that needs
no GPU answers with the documented status codes.  No kernel is launched here."""
import ctypes
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def declared_functions():
    text = (ROOT / "include" / "gact_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"\b(gact_[a-z0-9_]+)\s*\(", text)
    return sorted(set(names))


def test_header_declares_the_expected_entry_points():
    names = declared_functions()
    for must in ("gact_quantize", "gact_dequantize", "gact_minimax", "gact_mask_pack", "gact_mask_unpack", "gact_sq_diffs3",
                 "gact_sensitivity", "gact_calc_precision", "gact_packed_bytes", "gact_mask_words", "gact_error_string", "gact_version",
                 "gact_pipeline_error", "gact_pipeline_error_reset", "gact_pipeline_test_hook", "gact_sq_diffs3_noalloc"):
        assert must in names


def test_library_exports_every_declared_symbol():
    from gact import _native as nv
    lib = ctypes.CDLL(str(nv.LIB_PATH))
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} is declared in include/gact_b200.h but not exported"
    # and the binding covers them all
    for name in declared_functions():
        assert name in nv._SIGNATURES, f"{name} has no ctypes signature in gact/_native.py"


def test_host_only_entry_points():
    from gact import _native as nv
    L = nv.lib
    assert L.gact_version() >= 100
    assert L.gact_packed_bytes(3145728, 2) == 786432                   # config 1: 12 288 groups -> 3 072 row-blocks
    assert L.gact_packed_bytes(102760448, 1) == 12845056 and L.gact_packed_bytes(102760448, 8) == 102760448
    assert L.gact_packed_bytes(1, 4) == 256 and L.gact_packed_bytes(0, 4) == 0
    assert L.gact_packed_bytes(100, 3) == -1 and L.gact_packed_bytes(-5, 2) == -1
    assert L.gact_mask_words(1) == 16 and L.gact_mask_words(512) == 16 and L.gact_mask_words(513) == 32
    assert L.gact_sq_diffs3_scratch_bytes() > 0
    assert L.gact_error_string(0) == b"ok" and b"bits" in L.gact_error_string(1)


def test_argument_validation_without_a_gpu():
    """These return before any CUDA call is made."""
    from gact import _native as nv
    f = nv.lib.gact_quantize
    buf = ctypes.create_string_buffer(4096 + 64)
    p = (ctypes.addressof(buf) + 63) & ~63
    assert f(p, 0, 512, 3, 0, 0, None, 1, p, p, p, None) == 1            # bits
    assert f(p, 9, 512, 2, 0, 0, None, 1, p, p, p, None) == 2            # dtype
    assert f(None, 0, 512, 2, 0, 0, None, 1, p, p, p, None) == 3         # null pointer
    assert f(p + 2, 0, 100, 2, 0, 0, None, 1, p, p, p, None) == 4        # x not aligned to its element size
    assert f(p, 0, 100, 2, 0, 0, None, 1, p + 8, p, p, None) == 4        # packed output not 16-byte aligned
    assert f(p, 0, -1, 2, 0, 0, None, 1, p, p, p, None) == 5             # size
    assert f(p, 0, 512, 2, 0, 7, None, 1, p, p, p, None) == 6            # rng mode
    assert f(p, 0, 512, 2, 0, 3, None, 1, p, p, p, None) == 6            # external noise missing
    assert f(p, 0, 0, 2, 0, 0, None, 1, p, p, p, None) == 0              # empty tensor: nothing to do
    g = nv.lib.gact_dequantize
    assert g(p, p, p, 0, 512, 5, p, None) == 1 and g(p, p, p, 4, 512, 2, p, None) == 2 and g(None, p, p, 0, 512, 2, p, None) == 3
    assert nv.lib.gact_calc_precision(None, None, None, 0, 1.0, None, None) == 0
    assert nv.lib.gact_calc_precision(None, None, None, 5, 1.0, None, None) == 3
    assert nv.lib.gact_sq_diffs3_noalloc(p, p, None, 8, p, p, p, 5000, p, None) == 9      # more segments than it holds
    # the host tables of the allocation-free entry point are checked before anything is launched
    h = nv.lib.gact_sq_diffs3_noalloc
    ptrs = (ctypes.c_uint64 * 3)(p, p, p)
    lens = (ctypes.c_int64 * 3)(4, 2, 2)

    def tables(offs, lens_=lens, ptrs_=ptrs):
        o = (ctypes.c_int64 * 3)(*offs)
        return h(p, p, None, 8, ctypes.addressof(ptrs_), ctypes.addressof(o), ctypes.addressof(lens_), 3, p, None)

    assert tables([1, 5, 7]) == 5                                       # does not start at 0
    assert tables([0, 5, 7]) == 5                                       # a gap
    assert tables([0, 3, 5]) == 5                                       # overlap
    assert tables([0, 4, 6], lens_=(ctypes.c_int64 * 3)(4, 2, 1)) == 5  # lengths do not add up to P
    assert tables([0, 4, 6], ptrs_=(ctypes.c_uint64 * 3)(p, 0, p)) == 3  # a null segment


def test_import_fails_loudly_without_the_library(tmp_path, monkeypatch):
    import importlib.util
    import shutil
    src = ROOT / "gact-icml_b200" / "gact" / "_native.py"
    dst = tmp_path / "_native_copy.py"
    shutil.copy(src, dst)
    spec = importlib.util.spec_from_file_location("_native_copy", dst)
    mod = importlib.util.module_from_spec(spec)
    try:
        spec.loader.exec_module(mod)
    except ImportError as e:
        assert "no fallback" in str(e)
    else:
        raise AssertionError("importing the binding next to no library must raise")


def test_calc_precision_host_twin(golden_dir=None):
    """gact_calc_precision_host (no GPU involved) through the pybind-compatible shim: the recorded outputs of the
    reference's calc_precision.cc, random cases against the oracle, the 1-bit-entries case, and the unreachable budget."""
    import json
    import numpy as np
    import pytest
    import torch
    import oracle
    from gact.cpp_extension.calc_precision import calc_precision
    cases = json.loads((ROOT / "tests" / "golden" / "calc_precision.json").read_text())["cases"]
    for c in cases:
        C = torch.from_numpy(np.array(c["C_bits"], dtype=np.uint32).view(np.float32).copy())
        w = torch.tensor(c["w"], dtype=torch.int64)
        b = torch.full((len(c["w"]),), c["start"], dtype=torch.int32)
        out = calc_precision(b, C, w, c["target"])
        assert out is b and out.tolist() == c["bits"]
    g = torch.Generator().manual_seed(7)
    for L in (1, 2, 17, 300, 2000):
        C = torch.rand(L, generator=g) * torch.tensor(10.0) ** torch.randint(-6, 6, (L,), generator=g)
        C[::7] = C[0]                                              # equal keys: larger index first
        w = torch.randint(1, 1 << 20, (L,), generator=g, dtype=torch.int64)
        start = torch.tensor([32, 8, 4, 2, 1], dtype=torch.int32)[torch.randint(0, 5, (L,), generator=g)]
        for avg in (1.0, 1.5, 3.0, 7.9):
            target = avg * float(w.sum())
            want, st = oracle.calc_precision(start.clone(), C, w, target)
            if st:
                continue
            got = calc_precision(start.clone(), C, w, target)
            assert torch.equal(got, want), (L, avg)
    with pytest.raises(RuntimeError):
        calc_precision(torch.full((4,), 32, dtype=torch.int32), torch.ones(4), torch.full((4,), 256, dtype=torch.int64), 100.0)
    with pytest.raises(RuntimeError):
        calc_precision(torch.full((4,), 32, dtype=torch.int64), torch.ones(4), torch.full((4,), 256, dtype=torch.int64), 1e9)


def test_fastcall_module_forwards_to_the_same_entry_points():
    """gact/_fastcall.so (built by gact-icml_b200/build.py) must answer argument errors exactly as the ctypes route."""
    from gact import _native as nv
    assert nv._fastcall is not None, "gact/_fastcall.so was not built"
    buf = ctypes.create_string_buffer(4096 + 64)
    p = (ctypes.addressof(buf) + 63) & ~63
    cases = [(p, 0, 512, 3, 0, 0, None, 1, p, p, p, None), (p, 9, 512, 2, 0, 0, None, 1, p, p, p, None),
             (None, 0, 512, 2, 0, 0, None, 1, p, p, p, None), (p + 4, 0, 100, 2, 0, 0, None, 1, p, p, p, None),
             (p, 0, -1, 2, 0, 0, None, 1, p, p, p, None), (p, 0, 512, 2, 2**64 - 1, 7, None, 1, p, p, p, None),
             (p, 0, 0, 2, 0, 0, None, 1, p, p, p, None)]
    for c in cases:
        assert nv._fastcall.quantize(*c) == nv.lib.gact_quantize(*c)
    for c in [(p, p, p, 0, 512, 3, p, None), (p, p, p, 7, 512, 2, p, None), (None, p, p, 0, 512, 2, p, None), (p, p, p, 0, 0, 2, p, None)]:
        assert nv._fastcall.dequantize(*c) == nv.lib.gact_dequantize(*c)
