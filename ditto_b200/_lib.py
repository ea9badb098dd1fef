"""ctypes binding of libditto_b200.so (the C ABI declared in include/ditto_b200.h).

There is no CPU fallback: if the shared library is missing this module raises,
and every operator built on it fails with it.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))

OK = 0
ERR_INVALID_ARG = -1
ERR_UNSUPPORTED = -2
ERR_CUDA = -3
ERR_TIMEOUT = -4
ERR_WORKSPACE = -5
ERR_DRIVER = -6

DTYPE_FP16 = 0
DTYPE_BF16 = 1
OP_BMM_SOFTMAX_BMM = 0
OP_GEMM_RELU_GEMM = 1
FLAG_P_VIA_SMEM = 1
FLAG_ONE_TILE = 2
FLAG_TWO_TILES = 4
EPILOGUE_PAIR_MMA = 0x200
EPILOGUE_QUAD_MMA = 0x400
EPILOGUE_WIDE_MMA = 0x800

EXPORTS = (
    "ditto_b200_bmm_softmax_bmm",
    "ditto_b200_gemm_relu_gemm",
    "ditto_b200_gemm_relu_gemm_static_scratch",
    "ditto_b200_multi_head_attention",
    "ditto_b200_ffn",
    "ditto_b200_workspace_bytes",
    "ditto_b200_mlp_cluster_slots",
    "ditto_b200_selftest_umma",
    "ditto_b200_selftest_umma_pair",
    "ditto_b200_selftest_wait_limit",
    "ditto_b200_check_status",
    "ditto_b200_strerror",
    "ditto_b200_last_cuda_error",
    "ditto_b200_version",
)


class DittoError(RuntimeError):
    """A non-zero status from the C ABI."""

    def __init__(self, code, where):
        self.code = code
        lib = load()
        msg = lib.ditto_b200_strerror(code).decode()
        detail = lib.ditto_b200_last_cuda_error().decode() if code in (ERR_CUDA, ERR_DRIVER) else ""
        super().__init__(f"{where}: {msg} (code {code}){' -- ' + detail if detail else ''}")


def library_path():
    return os.environ.get("DITTO_B200_LIB", os.path.join(_HERE, "lib", "libditto_b200.so"))


_lib = None


def load():
    """Load the shared library once and attach argument types."""
    global _lib
    if _lib is not None:
        return _lib
    path = library_path()
    if not os.path.exists(path):
        raise ImportError(
            f"{path} not found: build it with `python -m ditto_b200.build_lib` (needs nvcc); "
            "ditto_b200 has no CPU fallback")
    lib = ctypes.CDLL(path)
    vp, i, f, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_size_t
    lib.ditto_b200_bmm_softmax_bmm.argtypes = [vp, vp, vp, vp, i, i, i, i, i, i, i, f, i, vp, sz, vp, vp]
    lib.ditto_b200_bmm_softmax_bmm.restype = i
    lib.ditto_b200_gemm_relu_gemm.argtypes = [vp, vp, vp, vp, i, i, i, i, i, i, i, i, vp, sz, vp, vp]
    lib.ditto_b200_gemm_relu_gemm.restype = i
    lib.ditto_b200_gemm_relu_gemm_static_scratch.argtypes = [vp, vp, vp, vp, i, i, i, i, i, i, i, i, vp, vp]
    lib.ditto_b200_gemm_relu_gemm_static_scratch.restype = i
    lib.ditto_b200_multi_head_attention.argtypes = [vp, vp, i, i, i, i, i, f, i, vp, vp]
    lib.ditto_b200_multi_head_attention.restype = i
    lib.ditto_b200_ffn.argtypes = [vp, vp, vp, vp, vp, vp, i, i, i, i, i, i, i, i, i, vp, vp]
    lib.ditto_b200_ffn.restype = i
    lib.ditto_b200_workspace_bytes.argtypes = [i, i, i, i, i, i, i]
    lib.ditto_b200_workspace_bytes.restype = sz
    lib.ditto_b200_mlp_cluster_slots.argtypes = [i, i]
    lib.ditto_b200_mlp_cluster_slots.restype = i
    lib.ditto_b200_selftest_umma.argtypes = [vp, vp, vp, i, i, i, i, i, vp, vp]
    lib.ditto_b200_selftest_umma.restype = i
    lib.ditto_b200_selftest_umma_pair.argtypes = [vp, vp, vp, i, i, i, i, vp, vp]
    lib.ditto_b200_selftest_umma_pair.restype = i
    lib.ditto_b200_selftest_wait_limit.argtypes = [i, vp, vp]
    lib.ditto_b200_selftest_wait_limit.restype = i
    lib.ditto_b200_check_status.argtypes = [vp, vp, ctypes.POINTER(ctypes.c_int)]
    lib.ditto_b200_check_status.restype = i
    lib.ditto_b200_strerror.argtypes = [i]
    lib.ditto_b200_strerror.restype = ctypes.c_char_p
    lib.ditto_b200_last_cuda_error.argtypes = []
    lib.ditto_b200_last_cuda_error.restype = ctypes.c_char_p
    lib.ditto_b200_version.argtypes = []
    lib.ditto_b200_version.restype = i
    _lib = lib
    return lib


def check(code, where):
    if code != OK:
        raise DittoError(code, where)
