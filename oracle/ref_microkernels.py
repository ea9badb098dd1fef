"""ctypes face of oracle/_ref/libditto_ref_microkernels.so: the reference's own CPU micro-kernels
(built by oracle/build_ref.py from python/ditto/auto_tensorize/intrinsic.py), and the reference's CPU
chains evaluated tile by tile THROUGH those micro-kernels.

Test infrastructure.  The tile loops here restate what the reference's TE definitions say
(zero-padded 6-row blocks, 16-wide column tiles, reduction in chunks of KI):
  * (A.B).D                   benchmark/chimera/cpu/bmm_bmm_cpu.py:55-116
  * relu(A.B).C               python_test/auto_tensorize/test_hyper_fusion_cpu.py:24-96
  * exp(Q.K).[V | 1] / sum    benchmark/chimera/cpu/bmm_softmax_bmm.py:64-170  (ones column at index N, no epsilon)
They are slow (one ctypes call per 6 x 16 tile) and meant for small shapes: their outputs are the
golden vectors under tests/golden/ that pin the C restatement in chain_oracle.c.
"""
import ctypes

import numpy as np

from . import build_ref

MI, NI = 6, 16
_LIB = None


def available():
    """The library exists (built here or shipped prebuilt) and this host can execute its AVX2 + FMA code."""
    return {"avx2", "fma"} <= build_ref.host_flags() and build_ref.build() is not None


def lib():
    global _LIB
    if _LIB is None:
        path = build_ref.build()
        if path is None:
            raise RuntimeError("reference micro-kernels are not built (no reference tree and no prebuilt library)")
        _LIB = ctypes.CDLL(path)
    return _LIB


def has_exp():
    """The exponential kernels are AVX-512: built only on such a host, and only callable on one."""
    return "avx512f" in build_ref.host_flags() and hasattr(lib(), "ref_exp_6x16_compute_exp")


def _fp(a):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_float))


def _ki_for(K):
    for ki in (128, 64, 32, 16):
        if K % ki == 0:
            return ki
    raise ValueError(f"reduction length {K} is not a multiple of 16")


def gemm(A, B, ki=None):
    """A[M, K] . B[K, N] in fp32 through <prefix>_update on zero-padded 6 x 16 tiles, reduction in chunks of ki."""
    A = np.ascontiguousarray(A, dtype=np.float32)
    B = np.ascontiguousarray(B, dtype=np.float32)
    M, K = A.shape
    K2, N = B.shape
    assert K == K2 and N % NI == 0
    ki = ki or _ki_for(K)
    assert K % ki == 0
    upd = getattr(lib(), f"ref_gemm_k{ki}_update")
    rst = getattr(lib(), f"ref_gemm_k{ki}_reset")
    Mp = -(-M // MI) * MI
    Ap = np.zeros((Mp, K), dtype=np.float32)
    Ap[:M] = A
    C = np.empty((Mp, N), dtype=np.float32)
    esz = 4
    for m0 in range(0, Mp, MI):
        for n0 in range(0, N, NI):
            c_ptr = ctypes.cast(C.ctypes.data + (m0 * N + n0) * esz, ctypes.POINTER(ctypes.c_float))
            rst(c_ptr, N)
            for k0 in range(0, K, ki):
                a_ptr = ctypes.cast(Ap.ctypes.data + (m0 * K + k0) * esz, ctypes.POINTER(ctypes.c_float))
                b_ptr = ctypes.cast(B.ctypes.data + (k0 * N + n0) * esz, ctypes.POINTER(ctypes.c_float))
                upd(c_ptr, a_ptr, b_ptr, K, N, N)
    return C[:M]


def exp(x):
    """Element-wise exp of a [rows, cols] fp32 array (cols % 16 == 0) through the reference's polynomial kernel."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, cols = x.shape
    assert cols % NI == 0
    y = np.empty_like(x)
    k6, k1 = lib().ref_exp_6x16_compute_exp, lib().ref_exp_1x16_compute_exp
    esz = 4
    for r0 in range(0, rows, MI):
        fn = k6 if r0 + MI <= rows else None
        for c0 in range(0, cols, NI):
            if fn is not None:
                fn(ctypes.cast(y.ctypes.data + (r0 * cols + c0) * esz, ctypes.POINTER(ctypes.c_float)),
                   ctypes.cast(x.ctypes.data + (r0 * cols + c0) * esz, ctypes.POINTER(ctypes.c_float)), cols, cols)
            else:
                for r in range(r0, rows):
                    k1(ctypes.cast(y.ctypes.data + (r * cols + c0) * esz, ctypes.POINTER(ctypes.c_float)),
                       ctypes.cast(x.ctypes.data + (r * cols + c0) * esz, ctypes.POINTER(ctypes.c_float)), cols, cols)
    return y


def bmm_bmm(A, B, D, ki1=None, ki2=None):
    return np.stack([gemm(gemm(A[b], B[b], ki1), D[b], ki2) for b in range(A.shape[0])])


def bmm_relu_bmm(A, B, C, ki1=None, ki2=None):
    return np.stack([gemm(np.maximum(gemm(A[b], B[b], ki1), np.float32(0)), C[b], ki2) for b in range(A.shape[0])])


def bmm_softmax_bmm_cpu(Q, K, V, ki1=None, ki2=None):
    """The reference's CPU softmax chain: exp without max subtraction, the row sum taken by a column
    of ones appended to V at index N (padded to a multiple of 16), then one division, no epsilon."""
    batch, L, N = V.shape
    Np = -(-(N + 1) // NI) * NI
    out = []
    for b in range(batch):
        P = exp(gemm(Q[b], K[b], ki1))
        Vp = np.zeros((L, Np), dtype=np.float32)
        Vp[:, :N] = V[b]
        Vp[:, N] = 1.0
        E = gemm(P, Vp, ki2)
        out.append(E[:, :N] / E[:, N:N + 1])
    return np.stack(out)


def linear(x, weight, bias=None, ki=None):
    """The reference's linear op (python/ditto/auto_compute/nn/functional/linear.py:4-41): x [M, in] times
    weight [out, in] transposed, through the GEMM micro-kernel, then the bias add as its own step."""
    y = gemm(x, np.ascontiguousarray(np.asarray(weight, dtype=np.float32).T), ki)
    if bias is not None:
        y = y + np.asarray(bias, dtype=np.float32)[None, :]
    return y.astype(np.float32)


def ffn(x, w1, b1, w2, b2, relu1=True, relu2=True):
    """The reference's feed-forward block (python/ditto/auto_compute/nn/model/transformer.py:21-34):
    activation(w_2(activation(w_1(x)))) with biased [out, in] linears; activation = ReLU as
    if_then_else(v > 0, v, 0) (nn/functional/activation.py:9-26) or, for the variants without it, identity."""
    h = linear(x, w1, b1)
    if relu1:
        h = np.where(h > 0, h, np.float32(0)).astype(np.float32)
    y = linear(h, w2, b2)
    if relu2:
        y = np.where(y > 0, y, np.float32(0)).astype(np.float32)
    return y
