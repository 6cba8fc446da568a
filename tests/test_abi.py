"""The C-ABI library loads and exports every symbol the headers under include/ declare (no compute call is made)."""
import ctypes
import os
import re

import pytest

import fortis_b200
from fortis_b200 import build as fb

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    fb.build()
    return fortis_b200.load()


def declared_symbols():
    inc = os.path.join(ROOT, "include")
    text = "\n".join(open(os.path.join(inc, f)).read() for f in sorted(os.listdir(inc)) if f.endswith(".h"))
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"^\s*(?:const\s+)?(?:void|int|double|char|long)\s*\*?\s*(\w+)\s*\(", text, flags=re.M)
    names += re.findall(r"^extern\s+int\s+(\w+)\s*;", text, flags=re.M)
    return sorted(set(names))


def test_header_lists_the_reference_surface():
    names = declared_symbols()
    for ref in ("fortis_gather", "fortis_scatter", "mlp_forward", "mlp_forward_batched", "mlp_upload", "mlp_forward_dev",
                "mlp_download", "fortis_pack", "fortis_unpack", "fortis_model_input", "fortis_model_output", "fortis_begin",
                "mgpuStreamCreate", "mgpuStreamDestroy", "mgpuStreamSynchronize", "fortis_alloc", "fortis_free",
                "fortis_gemm", "fortis_conv2d", "fortis_conv3d", "fortis_conv3d_direct", "fortis_conv3d_fft", "fortis_step", "fortis_capturing"):
        assert ref in names


def test_every_declared_symbol_is_exported(lib):
    for name in declared_symbols():
        assert hasattr(lib, name), "libfortis_b200.so does not export %s" % name


def test_configuration_errors_are_reported_not_thrown(lib):
    assert lib.fortis_configure(b"gather", b"{not json") == -1
    assert b"JSON" in lib.fortis_last_error_message()
    assert lib.fortis_configure(b"nonsense", b"{}") == -1
    assert lib.fortis_load_model_mem(ctypes.c_char_p(b"garbage!garbage!"), 16) == -1
    assert b"magic" in lib.fortis_last_error_message()
    blob = fortis_b200.write_blob(fortis_b200.mlp_layers([4, 8, 2], seed=0))
    assert lib.fortis_load_model_mem(ctypes.c_char_p(blob[:40]), 40) == -1          # truncated
    assert b"truncated" in lib.fortis_last_error_message()
    assert lib.fortis_set_option(b"precision", b"int4") == -1
    lib.fortis_reset()


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from fortis_b200 import lib as fl
    monkeypatch.setattr(fl, "_LIB", None)
    monkeypatch.setattr(fl, "HERE", str(tmp_path))
    with pytest.raises(fl.FortisError):
        fl.load()


def test_fortran_interface_module_names_exported_entries():
    """include/fortis_bindc.f90 binds by name: every name= in it must be declared in the C header and exported."""
    text = open(os.path.join(ROOT, "include", "fortis_bindc.f90")).read()
    names = re.findall(r"bind\(C,\s*name='(\w+)'\)", text)
    assert len(names) >= 25 and len(set(names)) == len(names)
    declared = set(declared_symbols())
    L = ctypes.CDLL(fortis_b200.lib_path())
    for n in names:
        assert n in declared, "%s is not declared in include/fortis_b200.h" % n
        assert hasattr(L, n), "libfortis_b200.so does not export %s" % n
    # subroutine / function ... end pairs balance (no Fortran compiler in this image: a structural check only)
    assert len(re.findall(r"^\s*(subroutine|function)\s", text, re.M)) == len(re.findall(r"^\s*end (subroutine|function)", text, re.M))


def test_every_option_key_is_documented_in_a_header():
    """fortis_set_option's keys, read off the source, all appear in the option lists of the headers under include/."""
    src = open(os.path.join(ROOT, "fortis_b200", "csrc", "fortis_api.cu")).read()
    body = src[src.index("int fortis_set_option("):]
    body = body[:body.index("void fortis_reset(")]
    keys = set(re.findall(r'k == "(\w+)"', body))
    assert {"precision", "graph", "checksum", "host_access", "tc_pair"} <= keys
    inc = os.path.join(ROOT, "include")
    docs = "\n".join(open(os.path.join(inc, f)).read() for f in sorted(os.listdir(inc)) if f.endswith(".h"))
    missing = [k for k in sorted(keys) if '"%s"' % k not in docs]
    assert not missing, "option keys without a line in include/*.h: %s" % missing
