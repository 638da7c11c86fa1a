"""The C-ABI library loads and exports exactly what include/frink_b200.h declares.
No compute call is made here: this runs where there is no GPU."""
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _build():
    from frink_b200 import build
    return build.build()


def header_symbols():
    text = open(os.path.join(ROOT, "include", "frink_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fk_[a-z0-9_]+)\s*\(", text)))


def test_library_builds_and_exports_every_declared_symbol():
    import ctypes
    path = _build()
    assert os.path.exists(path)
    L = ctypes.CDLL(path)
    declared = header_symbols()
    assert len(declared) >= 20
    missing = [s for s in declared if not hasattr(L, s)]
    assert not missing, f"declared in the header but not exported: {missing}"


def test_python_binding_table_matches_the_header():
    from frink_b200 import _lib
    assert sorted(_lib.SYMBOLS) == header_symbols()
    _lib.lib()  # resolves every symbol with its signature


def test_block_geometry_and_status_mapping():
    from frink_b200 import _lib
    L = _lib.lib()
    assert [L.fk_block_bytes(k) for k in (8, 12, 14, 39)] == [34, 144, 210, 17]
    assert [L.fk_block_elems(k) for k in (8, 12, 14, 39)] == [32, 256, 256, 32]
    assert L.fk_block_bytes(2) == -1
    with pytest.raises(_lib.Unsupported):
        _lib.check(_lib.FK_UNSUPPORTED)
    with pytest.raises(_lib.CudaError):
        _lib.check(_lib.FK_LAUNCH)


def test_no_gpu_means_a_loud_error_not_a_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from frink_b200 import _lib, device, gpu
    with pytest.raises(_lib.DriverInit):
        device.context()
    assert gpu.probe() is None


def test_kind_tables_agree():
    from frink_b200 import matvec_kinds, mul_mm
    from oracle import frink_oracle as fo
    # the matvec table has one kind more than the GEMM table: Q5_K has the plain matvec only
    assert [k.name for k in matvec_kinds.KINDS if k.name != "Q5_K"] == [k.name for k in mul_mm.KINDS]
    assert mul_mm.kind_by_name("Q5_K") is None
    for k in matvec_kinds.KINDS:
        assert fo.block_bytes(k.tag) == k.block_bytes and fo.block_elems(k.tag) == k.block_elems
        assert matvec_kinds.kind_by_name(k.fn_name) is k and matvec_kinds.kind_by_name(k.name) is k
    assert matvec_kinds.kind_by_name("q5_k_matvec").tag == 13 and matvec_kinds.kind_by_name("q3_k_matvec") is None
    assert not mul_mm.worth_a_gemm(8) and mul_mm.worth_a_gemm(64)


def test_the_rust_sys_crate_declares_every_entry_point_of_the_header():
    """`bindings/rust/frink-b200-sys/src/lib.rs` is generated from the header (`bindings/rust/gen_sys.py`); a header
    change without a regeneration shows up here."""
    import os
    import re
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    h = re.sub(r"/\*.*?\*/", "", open(os.path.join(root, "include", "frink_b200.h")).read(), flags=re.S)
    declared = set(re.findall(r"\b(fk_\w+)\s*\(", h))
    rs = open(os.path.join(root, "bindings", "rust", "frink-b200-sys", "src", "lib.rs")).read()
    in_rs = set(re.findall(r"pub fn (fk_\w+)\(", rs))
    assert declared == in_rs, (declared - in_rs, in_rs - declared)
    # and the wrapper crate only calls what the -sys crate declares
    used = set()
    wrap = os.path.join(root, "bindings", "rust", "frink-cuda-b200", "src")
    for f in os.listdir(wrap):
        used |= set(re.findall(r"sys::(fk_\w+)", open(os.path.join(wrap, f)).read()))
    assert used and used <= in_rs, used - in_rs
