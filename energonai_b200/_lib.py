"""ctypes binding of libenergon_b200.so (the C-ABI CUDA library).

The argument types of every entry point are derived from the declarations in
include/energon_b200.h, so the header is the single description of the boundary.  There is
no fallback: if the shared library has not been built, loading raises.
"""
import ctypes
import os
import re

_HERE = os.path.dirname(os.path.abspath(__file__))
HEADER = os.path.join(os.path.dirname(_HERE), "include", "energon_b200.h")
LIB_PATH = os.path.join(_HERE, "libenergon_b200.so")

F32, F16, BF16 = 0, 1, 2
ACT_NONE, ACT_RELU, ACT_GELU_TANH, ACT_GELU_ERF = 0, 1, 2, 3
SM_CAUSAL, SM_KEYLEN, SM_ALLROWS = 1, 2, 4

_SCALARS = {"int": ctypes.c_int, "int32_t": ctypes.c_int32, "int64_t": ctypes.c_int64, "size_t": ctypes.c_size_t,
            "float": ctypes.c_float, "long long": ctypes.c_longlong, "double": ctypes.c_double, "unsigned": ctypes.c_uint, "uint64_t": ctypes.c_uint64}


def parse_header(path=HEADER):
    """Returns {name: (restype, [argtypes])} for every EB_API declaration in the header."""
    text = re.sub(r"/\*.*?\*/", "", open(path).read(), flags=re.S)
    decls = {}
    for m in re.finditer(r"EB_API\s+([\w\s\*]+?)\b(eb_\w+)\s*\(([^)]*)\)\s*;", text):
        ret, name, args = m.group(1).strip(), m.group(2), m.group(3).strip()
        restype = ctypes.c_char_p if "*" in ret else _SCALARS[ret]
        argtypes = []
        if args and args != "void":
            for a in args.split(","):
                a = a.strip()
                if "*" in a:
                    argtypes.append(ctypes.c_void_p)
                else:
                    words = a.replace("const", "").split()[:-1]
                    argtypes.append(_SCALARS[" ".join(words)])
        decls[name] = (restype, argtypes)
    return decls


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m energonai_b200.build` "
                               "(there is no CPU or PyTorch fallback)")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (restype, argtypes) in parse_header().items():
            fn = getattr(handle, name)      # AttributeError if the library lacks a declared symbol
            fn.restype, fn.argtypes = restype, argtypes
        _lib = handle
    return _lib


def last_error():
    return lib().eb_last_error().decode()


launch_count = 0     # successful compute calls through the C ABI (each launches exactly one kernel)


def check(rc, what="", launches=1):
    global launch_count
    launch_count += launches
    if rc != 0:
        raise RuntimeError(f"energon_b200 {what} failed ({rc}): {last_error()}")


def dtype_code(torch_dtype):
    import torch
    try:
        return {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}[torch_dtype]
    except KeyError:
        raise RuntimeError(f"unsupported dtype {torch_dtype}") from None


def ptr(t):
    """Device pointer of a tensor (None -> NULL)."""
    return None if t is None else t.data_ptr()


def stream_ptr():
    import torch
    return torch.cuda.current_stream().cuda_stream


def require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("energon_b200 kernels take CUDA tensors only (no CPU path exists)")
