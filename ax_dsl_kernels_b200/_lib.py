"""ctypes binding of libq35b200.so: tensors are bound BY NAME, as the reference's hosts bind kernel IO
(tools/board/axrun.cc:55-110; models/qwen35_2b/whole/src/q35_layer_mc.py:915-916).

There is no fallback: if the shared library is missing or a call fails, an exception is raised.
"""
import ctypes
import json
import os

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libq35b200.so")
MAX_DIMS = 6

# AX engine element codes of the reference's IO tables (tools/manifest/onnx_io.py:21-32)
U8, F32, I32, BF16, F16, E4M3, FP4 = 1, 3, 6, 9, 10, 11, 15
_DTYPE_CODE = {
    torch.uint8: U8, torch.float32: F32, torch.int32: I32, torch.bfloat16: BF16, torch.float16: F16,
    torch.float8_e4m3fn: E4M3, torch.int8: U8,  # int8 KV rows travel as bytes (the AX table has no int8 code)
}
for _n, _c in (("float8_e8m0fnu", U8), ("float4_e2m1fn_x2", U8)):  # scale / packed-FP4 views are raw bytes
    if hasattr(torch, _n):
        _DTYPE_CODE[getattr(torch, _n)] = _c


class Q35Error(RuntimeError):
    def __init__(self, status, text):
        super().__init__(f"q35b200 status {status}: {text}")
        self.status = status


class _IO(ctypes.Structure):
    _fields_ = [("name", ctypes.c_char_p), ("ptr", ctypes.c_void_p), ("bytes", ctypes.c_size_t),
                ("dtype", ctypes.c_int), ("ndim", ctypes.c_int), ("shape", ctypes.c_int64 * MAX_DIMS)]


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise Q35Error(-1, f"{LIB_PATH} is missing: build it with `python -m ax_dsl_kernels_b200.build` "
                               "(there is no CPU or PyTorch fallback)")
        L = ctypes.CDLL(LIB_PATH)
        L.q35_run.argtypes = [ctypes.c_char_p, ctypes.POINTER(_IO), ctypes.c_int, ctypes.c_void_p]
        L.q35_run.restype = ctypes.c_int
        L.q35_workspace_bytes.argtypes = [ctypes.c_char_p, ctypes.POINTER(_IO), ctypes.c_int]
        L.q35_workspace_bytes.restype = ctypes.c_int64
        L.q35_io_table.argtypes = [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_size_t]
        L.q35_io_table.restype = ctypes.c_int
        L.q35_role_count.restype = ctypes.c_int
        L.q35_role_name.argtypes = [ctypes.c_int]
        L.q35_role_name.restype = ctypes.c_char_p
        L.q35_last_error.restype = ctypes.c_char_p
        L.q35_device_status.argtypes = [ctypes.c_void_p]
        L.q35_device_status.restype = ctypes.c_int
        L.q35_version.restype = ctypes.c_int
        L.q35_launch_count.restype = ctypes.c_longlong
        _lib = L
    return _lib


def _table(tensors):
    arr = (_IO * len(tensors))()
    keep = []
    for i, (name, t) in enumerate(tensors.items()):
        if not isinstance(t, torch.Tensor):
            raise TypeError(f"{name}: expected a torch.Tensor, got {type(t).__name__}")
        if not t.is_contiguous():
            raise ValueError(f"{name}: tensor must be contiguous")
        if t.dim() > MAX_DIMS:
            raise ValueError(f"{name}: more than {MAX_DIMS} dims")
        code = _DTYPE_CODE.get(t.dtype)
        if code is None:
            raise TypeError(f"{name}: unsupported dtype {t.dtype}")
        b = name.encode()
        keep.append(b)
        arr[i].name = b
        arr[i].ptr = t.data_ptr()
        arr[i].bytes = t.numel() * t.element_size()
        arr[i].dtype = code
        arr[i].ndim = t.dim()
        for d in range(t.dim()):
            arr[i].shape[d] = t.shape[d]
    return arr, keep


def _check(st):
    if st != 0:
        raise Q35Error(st, lib().q35_last_error().decode())


def workspace_bytes(role, **tensors):
    arr, _keep = _table(tensors)
    n = lib().q35_workspace_bytes(role.encode(), arr, len(tensors))
    if n < 0:
        raise Q35Error(-n, lib().q35_last_error().decode())
    return int(n)


_ws_cache = {}
_need_cache = {}


def _workspace(device, nbytes, stream=0):
    """one growing scratch buffer per (device, stream), owned by the Python host (the library itself never allocates);
    roles running concurrently on different streams must not share scratch"""
    key = (device.type, device.index, stream)
    buf = _ws_cache.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _ws_cache[key] = buf
    return buf


def run(role, stream=None, **tensors):
    """q35_run(role, ...) with the given tensors bound by name; a `workspace` is added when the role needs one."""
    L = lib()
    dev = None
    for t in tensors.values():
        if not t.is_cuda:
            raise ValueError("all tensors must live on the GPU (the library has no CPU path)")
        dev = t.device
    if "workspace" not in tensors:
        # the scratch size depends on shapes and dtypes only: ask the library once per signature
        sig = (role, tuple((n, t.dtype, tuple(t.shape)) for n, t in tensors.items()))
        need = _need_cache.get(sig)
        if need is None:
            need = _need_cache[sig] = workspace_bytes(role, **tensors)
        if stream is None:
            stream = torch.cuda.current_stream(dev).cuda_stream
        if need:
            tensors = dict(tensors, workspace=_workspace(dev, need, stream))
    arr, _keep = _table(tensors)
    if stream is None:
        stream = torch.cuda.current_stream(dev).cuda_stream
    with torch.cuda.device(dev):
        _check(L.q35_run(role.encode(), arr, len(tensors), ctypes.c_void_p(stream)))


def io_table(role):
    L = lib()
    n = L.q35_io_table(role.encode(), None, 0)
    if n < 0:
        raise Q35Error(-n, L.q35_last_error().decode())
    buf = ctypes.create_string_buffer(n + 1)
    L.q35_io_table(role.encode(), buf, n + 1)
    return json.loads(buf.value.decode())


def roles():
    L = lib()
    return [L.q35_role_name(i).decode() for i in range(L.q35_role_count())]


def device_status(stream=None):
    if stream is None:
        stream = torch.cuda.current_stream().cuda_stream
    return lib().q35_device_status(ctypes.c_void_p(stream))
