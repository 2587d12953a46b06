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
    assert b200kv.lib.b200kv_abi_version() == 6


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


def _decode_args_of_fake_pointers(b200kv):
    a = b200kv.DecodeArgs()
    a.pool.latent, a.pool.rope = 0x10000, 0x20000
    a.pool.latent_row_stride, a.pool.rope_row_stride, a.pool.pool_rows = 512, 64, 128
    a.q, a.q_seq_stride, a.q_head_stride = 0x30000, 64 * 576, 576
    a.block_table, a.max_blocks, a.kv_len = 0x40000, 2, 0x50000
    a.batch, a.heads, a.block_size, a.scale = 2, 64, 64, 1.0 / 24.0
    a.out = 0x60000
    return a


def test_decode_refuses_inconsistent_optional_arguments_before_touching_the_device():
    """The refusals of the row list and of the quantised output are host checks: they answer without a GPU
    (the pointers here are never dereferenced)."""
    import b200kv

    a = _decode_args_of_fake_pointers(b200kv)
    a.row_index, a.row_index_stride, a.kv_begin = 0x70000, 512, 0x80000   # a row list excludes a KV range
    assert b200kv.lib.b200kv_mla_decode(ctypes.byref(a), None, None) == b200kv.ERR_INVALID
    assert "row_index" in b200kv.last_error()
    a = _decode_args_of_fake_pointers(b200kv)
    a.row_index, a.row_index_stride = 0x70000, 0                          # ... and needs a stride
    assert b200kv.lib.b200kv_mla_decode(ctypes.byref(a), None, None) == b200kv.ERR_INVALID
    a = _decode_args_of_fake_pointers(b200kv)
    a.out_fp8 = 0x90000                                                    # codes without scales
    assert b200kv.lib.b200kv_mla_decode(ctypes.byref(a), None, None) == b200kv.ERR_INVALID
    assert "out_fp8" in b200kv.last_error()
    a = _decode_args_of_fake_pointers(b200kv)
    a.out, a.out_fp8, a.out_scale = None, 0x90000, 0xa0000                 # quantised output of partials: no
    a.partial_o, a.partial_m, a.partial_l = 0xb0000, 0xc0000, 0xd0000
    assert b200kv.lib.b200kv_mla_decode(ctypes.byref(a), None, None) == b200kv.ERR_INVALID


def test_indexer_refuses_the_tensor_core_variant_where_it_cannot_run():
    import b200kv

    a = b200kv.IndexerArgs()
    a.q, a.q_scale, a.weights, a.heads = 0x1000, 0x2000, 0x3000, 64
    a.key_pool, a.key_stride, a.k_scale, a.pool_rows = 0x4000, 128, 0x5000, 256
    a.block_table, a.max_blocks, a.kv_len = 0x6000, 4, 0x7000
    a.batch, a.block_size, a.max_kv_len, a.k = 2, 16, 64, 8
    a.index_out, a.n_selected_out, a.workspace = 0x8000, 0x9000, 0xa000
    a.workspace_bytes = b200kv.lib.b200kv_indexer_workspace_bytes(2, 64)
    a.variant = b200kv.INDEXER_TCGEN05                                     # blocks of 16 tokens
    assert b200kv.lib.b200kv_indexer_topk(ctypes.byref(a), None, None) == b200kv.ERR_INVALID
    assert "tensor-core" in b200kv.last_error()
    a.variant = 7
    assert b200kv.lib.b200kv_indexer_topk(ctypes.byref(a), None, None) == b200kv.ERR_INVALID


def test_ctypes_structures_match_the_header_layout(tmp_path):
    """The binding's ctypes structures and include/b200kv.h describe the same bytes: a C program compiled
    against the header prints each struct's size and the offset of its last field."""
    import subprocess

    import b200kv

    cases = [("b200kv_pool_view", "pool_rows", b200kv.PoolView), ("b200kv_decode_args", "flags", b200kv.DecodeArgs),
             ("b200kv_decode_args", "row_index_stride", b200kv.DecodeArgs), ("b200kv_decode_args", "out_scale", b200kv.DecodeArgs),
             ("b200kv_indexer_args", "rows_out", b200kv.IndexerArgs), ("b200kv_producer_args", "rstd_out", b200kv.ProducerArgs)]
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
