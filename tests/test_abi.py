"""The C-ABI library: it loads without a GPU and exports every symbol the header
declares; argument errors come back as status codes (no compute calls here)."""
import ctypes as C
import os
import subprocess

import pytest


def test_library_exports_every_declared_symbol(built_lib):
    from cyb_b200 import qeng
    lib = C.CDLL(built_lib)
    names = qeng.declared_symbols()
    assert len(names) >= 40
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_binding_covers_every_declared_symbol(built_lib):
    from cyb_b200 import qeng
    src = open(qeng.__file__).read()
    unbound = [n for n in qeng.declared_symbols() if '"%s"' % n not in src]
    assert not unbound, unbound


def test_header_is_plain_c():
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run(["/usr/bin/gcc", "-std=c99", "-fsyntax-only", "-x", "c", os.path.join(root, "include", "qeng.h")],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr


def test_no_cpu_fallback_without_a_gpu(built_lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from cyb_b200 import qeng
    with pytest.raises(qeng.QengError):
        qeng.Context(0)


def test_null_arguments_are_status_codes(built_lib):
    lib = C.CDLL(built_lib)
    lib.qeng_create.restype = C.c_int32
    assert lib.qeng_create(0, None) == -1
    lib.qeng_destroy.restype = C.c_int32
    assert lib.qeng_destroy(None) == -1
    assert lib.qeng_version() >= 100


def test_product_does_not_import_the_oracle():
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for dirpath, _, files in os.walk(os.path.join(root, "cyb_b200")):
        for f in files:
            if f.endswith((".py", ".cu", ".h", ".cpp")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.replace("no oracle", ""), os.path.join(dirpath, f)


def test_rust_declarations_name_every_symbol():
    """bindings/qeng.rs (uncompiled: no Rust toolchain here) declares exactly the header's functions."""
    import re
    from cyb_b200 import qeng
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    rs = open(os.path.join(root, "bindings", "qeng.rs")).read()
    declared = sorted(set(re.findall(r"pub fn (qeng_[a-z0-9_]+)\(", rs)))
    assert declared == qeng.declared_symbols()
    # the two plain structs carry the header's fields in the header's order
    hdr = open(qeng.HEADER_PATH).read()
    for struct in ("qeng_options", "qeng_model_cfg"):
        body = re.search(r"typedef struct %s \{(.*?)\} %s;" % (struct, struct), hdr, re.S).group(1)
        body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
        c_fields = re.findall(r"([a-z_0-9]+)\s*[,;]", body)
        r_body = re.search(r"pub struct %s \{(.*?)\}" % struct, rs, re.S).group(1)
        assert re.findall(r"pub ([a-z_0-9]+):", r_body) == c_fields, struct
