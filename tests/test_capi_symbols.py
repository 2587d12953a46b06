"""The C-ABI library loads without a GPU and exports every function include/*.h declares (CPU)."""
import ctypes
import glob
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    names = set()
    for header in glob.glob(os.path.join(ROOT, "include", "*.h")):
        text = open(header).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        text = re.sub(r"//[^\n]*", "", text)
        for m in re.finditer(r"\b((?:b200kv|acl|aclrt|aclnn)\w*)\s*\(", text):
            name = m.group(1)
            pre = text[: m.start()].rstrip()
            # a declaration: preceded by a type token, not by "#define" or an operator
            if pre.endswith(("#define", "(", ",", "=", "return")):
                continue
            names.add(name)
    return sorted(names)


def test_library_loads_and_exports_declared_symbols():
    import b200kv

    lib = ctypes.CDLL(b200kv.LIB_PATH)
    names = declared_functions()
    assert len(names) >= 20, names
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, f"declared in include/*.h but not exported: {missing}"
    assert b200kv.lib.b200kv_abi_version() == 5


def test_host_side_argument_refusals():
    """Validation that needs no device: null and malformed arguments come back as status codes with text."""
    import b200kv

    view = b200kv.PoolView()
    rc = b200kv.lib.b200kv_append(ctypes.byref(view), None, 512, None, 64, None, 1, None, None)
    assert rc == b200kv.ERR_NULLPTR and "null" in b200kv.last_error()
    view.latent, view.rope = 0x1000, 0x2000
    view.latent_row_stride, view.rope_row_stride, view.pool_rows = 513, 64, 128
    rc = b200kv.lib.b200kv_append(ctypes.byref(view), 0x3000, 512, 0x4000, 64, 0x5000, 1, None, None)
    assert rc == b200kv.ERR_INVALID and "multiples of 8" in b200kv.last_error()
    assert b200kv.lib.b200kv_mla_decode(None, None, None) == b200kv.ERR_NULLPTR


def test_ctypes_structures_match_the_header_layout(tmp_path):
    """The binding's ctypes structures and include/b200kv.h describe the same bytes: a C program compiled
    against the header prints each struct's size and the offset of its last field."""
    import subprocess

    import b200kv

    cases = [("b200kv_pool_view", "pool_rows", b200kv.PoolView), ("b200kv_decode_args", "flags", b200kv.DecodeArgs),
             ("b200kv_producer_args", "rstd_out", b200kv.ProducerArgs)]
    lines = "".join(f'  printf("%zu %zu\\n", sizeof({c}), offsetof({c}, {f}));\n' for c, f, _ in cases)
    src = tmp_path / "layout.c"
    src.write_text('#include <stddef.h>\n#include <stdio.h>\n#include "b200kv.h"\nint main(void) {\n' + lines +
                   "  return 0;\n}\n")
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-std=c11", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split("\n")
    for (c_name, field, py), line in zip(cases, out):
        size, last = (int(x) for x in line.split())
        assert ctypes.sizeof(py) == size, c_name
        assert getattr(py, field).offset == last, (c_name, field)
