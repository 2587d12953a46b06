"""The operators outside the KV path: every one the reference resolves by name (src/core/op_table.cpp:47-88)
is exported in both phases with the argument list of its plan-function type, refuses null required
arguments with 161001, plans with no workspace, and launches only with its own executor (CPU)."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# Names as the reference's operator table lists them, minus the two KV-path operators (tested on the GPU)
# and the undeclared workspace helper.
OTHER_OPS = [
    "RmsNorm", "RmsNormDynamicMxQuant", "DynamicMxQuant", "Cast", "Matmul", "QuantMatmulV5", "ApplyRotaryPosEmbV2",
    "Sigmoid", "Mul", "InplaceAdd", "SwiGlu", "ArgMax", "Softplus", "Sqrt", "MoeGatingTopKV2", "MoeInitRoutingV4",
    "GroupedMatmulV5", "SwigluMxQuant", "MoeTokenUnpermute", "GroupedMatmulSwigluQuantV2",
    "GroupedMatmulFinalizeRoutingV3", "MhcPre", "MhcSinkhorn", "MhcPost", "QuantLightningIndexer",
]

SCALARS = {"int64_t": ctypes.c_int64, "double": ctypes.c_double, "float": ctypes.c_float, "bool": ctypes.c_bool,
           "int8_t": ctypes.c_int8, "aclDataType": ctypes.c_int}


def plan_signatures():
    """name -> list of (C type, argument name) parsed from the header, protocol arguments included."""
    text = open(os.path.join(ROOT, "include", "b200kv_aclnn.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    out = {}
    for m in re.finditer(r"aclnnStatus aclnn(\w+)GetWorkspaceSize\((.*?)\);", text, re.S):
        args = []
        for piece in " ".join(m.group(2).split()).split(", "):
            ctype, name = piece.rsplit(" ", 1)
            args.append((ctype, name))
        out[m.group(1)] = args
    return out


class Handles:
    """One of each descriptor kind, created through the library's own constructors."""

    def __init__(self, lib):
        self.lib = lib
        lib.aclCreateTensor.restype = ctypes.c_void_p
        lib.aclCreateTensorList.restype = ctypes.c_void_p
        lib.aclCreateIntArray.restype = ctypes.c_void_p
        lib.aclCreateScalar.restype = ctypes.c_void_p
        dims = (ctypes.c_int64 * 2)(4, 8)
        self.tensor = lib.aclCreateTensor(dims, ctypes.c_uint64(2), 27, None, ctypes.c_int64(0), 2, dims,
                                          ctypes.c_uint64(2), ctypes.c_void_p(0x1000))
        inner = lib.aclCreateTensor(dims, ctypes.c_uint64(2), 27, None, ctypes.c_int64(0), 2, dims,
                                    ctypes.c_uint64(2), ctypes.c_void_p(0x2000))
        arr = (ctypes.c_void_p * 1)(inner)
        self.tensor_list = lib.aclCreateTensorList(arr, ctypes.c_uint64(1))
        vals = (ctypes.c_int64 * 2)(1, 2)
        self.int_array = lib.aclCreateIntArray(vals, ctypes.c_uint64(2))
        one = ctypes.c_float(1.0)
        self.scalar = lib.aclCreateScalar(ctypes.byref(one), 0)
        assert self.tensor and self.tensor_list and self.int_array and self.scalar

    def value_for(self, ctype, null):
        base = ctype.replace("const ", "").strip()
        if base in SCALARS:
            return SCALARS[base](1)
        if base == "char*":
            return ctypes.c_char_p(None if null else b"rint")
        if null:
            return ctypes.c_void_p(None)
        return ctypes.c_void_p({"aclTensor*": self.tensor, "aclTensorList*": self.tensor_list,
                                "aclIntArray*": self.int_array, "aclScalar*": self.scalar}[base])


def test_every_other_operator_plans_and_launches_only_its_own_executor():
    import b200kv

    lib = ctypes.CDLL(b200kv.LIB_PATH)
    sigs = plan_signatures()
    handles = Handles(lib)
    assert len(OTHER_OPS) == 25 and len(set(OTHER_OPS)) == 25
    executors = {}
    for op in OTHER_OPS:
        assert op in sigs, f"aclnn{op}GetWorkspaceSize is not declared in include/b200kv_aclnn.h"
        plan = getattr(lib, f"aclnn{op}GetWorkspaceSize")
        launch = getattr(lib, f"aclnn{op}")
        plan.restype = launch.restype = ctypes.c_int32
        args = sigs[op][:-2]
        assert [n for _, n in sigs[op][-2:]] == ["workspace_size", "executor"]
        ws = ctypes.c_uint64(77)
        exe = ctypes.c_void_p(0x1)
        # every descriptor null: refused, no executor handed out
        rc = plan(*[handles.value_for(t, True) for t, _ in args], ctypes.byref(ws), ctypes.byref(exe))
        assert rc == 161001 and exe.value is None, (op, rc)
        assert f"aclnn{op}" in b200kv.last_error()
        # protocol outputs null: refused
        rc = plan(*[handles.value_for(t, False) for t, _ in args], None, None)
        assert rc == 161001, (op, rc)
        # everything given: a plan without workspace
        rc = plan(*[handles.value_for(t, False) for t, _ in args], ctypes.byref(ws), ctypes.byref(exe))
        assert rc == 0 and exe.value and ws.value == 0, (op, rc, ws.value)
        assert lib.aclSetAclOpExecutorRepeatable(exe) == 0
        executors[op] = (exe, launch)
    # launches: own executor twice (repeatable), somebody else's refused, null refused
    names = list(executors)
    for i, op in enumerate(names):
        exe, launch = executors[op]
        assert launch(None, ctypes.c_uint64(0), exe, None) == 0
        assert launch(None, ctypes.c_uint64(0), exe, None) == 0
        other_exe, _ = executors[names[(i + 1) % len(names)]]
        assert launch(None, ctypes.c_uint64(0), other_exe, None) == 161002, op
        assert "planned for" in b200kv.last_error()
        assert launch(None, ctypes.c_uint64(0), None, None) == 161001
    for exe, _ in executors.values():
        assert lib.aclDestroyAclOpExecutor(exe) == 0


def test_optional_arguments_may_be_null():
    """RmsNorm without rstd output, the gate operator without bias: the plan still succeeds."""
    import b200kv

    lib = ctypes.CDLL(b200kv.LIB_PATH)
    h = Handles(lib)
    t = ctypes.c_void_p(h.tensor)
    ws, exe = ctypes.c_uint64(1), ctypes.c_void_p()
    lib.aclnnRmsNormGetWorkspaceSize.restype = ctypes.c_int32
    rc = lib.aclnnRmsNormGetWorkspaceSize(t, t, ctypes.c_double(1e-6), t, None, ctypes.byref(ws), ctypes.byref(exe))
    assert rc == 0 and exe.value
    # not marked repeatable: the launch consumes it
    lib.aclnnRmsNorm.restype = ctypes.c_int32
    assert lib.aclnnRmsNorm(None, ctypes.c_uint64(0), exe, None) == 0
    # a KV-path executor is not accepted by another operator's launch: covered on the GPU side; here the
    # scatter plan's own null check
    lib.aclnnScatterPaKvCacheGetWorkspaceSize.restype = ctypes.c_int32
    rc = lib.aclnnScatterPaKvCacheGetWorkspaceSize(None, None, None, None, None, None, None, None, None, None, None,
                                                   None, ctypes.byref(ws), ctypes.byref(exe))
    assert rc == 161001
