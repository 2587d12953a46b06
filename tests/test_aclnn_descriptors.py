"""Descriptor getters of the operator ABI (CPU): what aclGetViewShape, aclGetViewStrides and aclGetStorageShape
hand out belongs to the caller, who releases it with delete[]. The reference does exactly that: it wraps each
result in std::unique_ptr<int64_t[]> when it copies a tensor into a list (src/memory/static_arena.cpp:181-188) and
when it checks a matmul's shapes (src/core/matmul_contract.cpp:16-23); its own stand-in allocates them with
new int64_t[] (mock/mock_descriptor.cpp:183-199). A getter that returned the descriptor's internal storage would
make that delete[] corrupt the heap, so the test releases every result through the C++ runtime's operator
delete[] and then uses the descriptor again."""
import ctypes
import ctypes.util

import b200kv


def _delete_array():
    libstdcpp = ctypes.CDLL(ctypes.util.find_library("stdc++") or "libstdc++.so.6")
    fn = libstdcpp._ZdaPv  # operator delete[](void*)
    fn.argtypes = [ctypes.c_void_p]
    fn.restype = None
    return fn


def _get(fn, tensor):
    data = ctypes.POINTER(ctypes.c_int64)()
    count = ctypes.c_uint64(0)
    assert fn(ctypes.c_void_p(tensor), ctypes.byref(data), ctypes.byref(count)) == 0
    values = [data[i] for i in range(count.value)]
    return values, ctypes.cast(data, ctypes.c_void_p).value


def test_shape_getters_return_caller_owned_copies():
    lib = b200kv.lib
    lib.aclCreateTensor.restype = ctypes.c_void_p
    delete_array = _delete_array()
    dims = (ctypes.c_int64 * 4)(86, 128, 1, 512)
    strides = (ctypes.c_int64 * 4)(128 * 512, 512, 512, 1)
    storage = (ctypes.c_int64 * 4)(86, 128, 1, 512)
    tensor = lib.aclCreateTensor(dims, ctypes.c_uint64(4), 27, strides, ctypes.c_int64(0), 2, storage,
                                 ctypes.c_uint64(4), ctypes.c_void_p(0x10000))
    assert tensor
    for _ in range(3):  # the descriptor keeps answering after its earlier answers were deleted
        seen = set()
        for fn, want in ((lib.aclGetViewShape, list(dims)), (lib.aclGetViewStrides, list(strides)),
                         (lib.aclGetStorageShape, list(storage))):
            first, p1 = _get(fn, tensor)
            second, p2 = _get(fn, tensor)
            assert first == want and second == want
            assert p1 != p2, "two calls returned the same storage: not a copy per call"
            seen.update((p1, p2))
            delete_array(p1)
            delete_array(p2)
    assert lib.aclDestroyTensor(ctypes.c_void_p(tensor)) == 0


def test_storage_shape_defaults_to_the_view_shape():
    lib = b200kv.lib
    lib.aclCreateTensor.restype = ctypes.c_void_p
    delete_array = _delete_array()
    dims = (ctypes.c_int64 * 2)(4, 8)
    tensor = lib.aclCreateTensor(dims, ctypes.c_uint64(2), 27, None, ctypes.c_int64(0), 2, None, ctypes.c_uint64(0),
                                 ctypes.c_void_p(0x1000))
    values, ptr = _get(lib.aclGetStorageShape, tensor)
    assert values == [4, 8]
    delete_array(ptr)
    values, ptr = _get(lib.aclGetViewStrides, tensor)
    assert values == [8, 1]  # contiguous row-major strides when none are given
    delete_array(ptr)
    assert lib.aclDestroyTensor(ctypes.c_void_p(tensor)) == 0


def test_getters_refuse_null_arguments():
    lib = b200kv.lib
    data = ctypes.POINTER(ctypes.c_int64)()
    count = ctypes.c_uint64(0)
    for fn in (lib.aclGetViewShape, lib.aclGetViewStrides, lib.aclGetStorageShape):
        assert fn(None, ctypes.byref(data), ctypes.byref(count)) == 161001
