"""Python face of the CPU oracle (test infrastructure only).

Two independent restatements of the reference's chain arithmetic live here:

* the C library built from chain_oracle.c (fast enough for the parity tests), reached through
  ctypes, and
* plain numpy versions (`np_*`) that follow the same reference definitions line by line and are
  used to cross-check the C code on small shapes.

Reference definitions: python/ditto/auto_compute/nn/functional/bmm_chain.py:40-103 (attention
chain), benchmark/chimera/cpu/bmm_bmm_cpu.py:55-116 (plain chain),
python_test/auto_tensorize/test_hyper_fusion_cpu.py:24-96 (ReLU chain).

Parity: pinned at the reference's CPU micro-kernels (ref_microkernels.py, bit for bit), unpinned for
the fp16 / bf16 forms above them - the reference ships no golden vectors and its generated kernels
cannot be built here (TVM is an absent submodule); the header of chain_oracle.c has the details.
"""
import ctypes
import os

import numpy as np

from . import build as _build

FP16, BF16, FP32 = 0, 1, 2
_lib = None


def lib():
    global _lib
    if _lib is None:
        try:
            path = _build.build()              # rebuilds only when chain_oracle.c is newer than the library
        except (OSError, RuntimeError):
            path = _build.LIB
            if not os.path.exists(path):
                raise
        L = ctypes.CDLL(path)
        fp = ctypes.POINTER(ctypes.c_float)
        i, f = ctypes.c_int, ctypes.c_float
        L.oracle_round.argtypes = [fp, fp, ctypes.c_long, i]
        L.oracle_bmm_softmax_bmm_literal.argtypes = [fp, fp, fp, fp, i, i, i, i, i, i]
        L.oracle_bmm_softmax_bmm.argtypes = [fp, fp, fp, fp, i, i, i, i, i, f, i, i]
        L.oracle_gemm_act_gemm.argtypes = [fp, fp, fp, fp, i, i, i, i, i, i, i, i]
        L.oracle_ffn.argtypes = [fp, fp, fp, fp, fp, fp, i, i, i, i, i, i, i, i]
        L.oracle_exp_ref_literal.argtypes = [fp, fp, ctypes.c_long]
        L.oracle_bmm_softmax_bmm_cpu_literal.argtypes = [fp, fp, fp, fp, i, i, i, i, i]
        L.baseline_chain_fp32.argtypes = [fp, fp, fp, fp, i, i, i, i, i, i, f, i]
        L.baseline_chain_fp32.restype = i
        L.oracle_max_threads.restype = i
        _lib = L
    return _lib


def _p(a):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_float))


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _shape(A, B, C):
    batch, M, K = A.shape
    b2, K2, L = B.shape
    b3, L2, N = C.shape
    assert batch == b2 == b3 and K == K2 and L == L2, (A.shape, B.shape, C.shape)
    return batch, M, N, K, L


# ------------------------------------------------------------------ rounding
def round_np(x, in_dtype):
    """Round float32 values to the storage type and back, with numpy / bit arithmetic."""
    x = np.asarray(x, dtype=np.float32)
    if in_dtype == FP16:
        with np.errstate(over="ignore"):
            return x.astype(np.float16).astype(np.float32)
    if in_dtype == BF16:
        u = x.view(np.uint32).astype(np.uint64)
        u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
        out = u.astype(np.uint32).view(np.float32)
        return np.where(np.isnan(x), x, out)
    return x.copy()


def round_c(x, in_dtype):
    x = _f32(x)
    out = np.empty_like(x)
    lib().oracle_round(_p(x), _p(out), x.size, in_dtype)
    return out


# ------------------------------------------------------------------ C oracle
def bmm_softmax_bmm_literal(A, B, C, in_dtype=FP16):
    """exp -> ones-column sum -> divide(+1e-5), all casts as in bmm_chain.py:64-103."""
    A, B, C = _f32(A), _f32(B), _f32(C)
    batch, M, N, K, L = _shape(A, B, C)
    F = np.empty((batch, M, N), np.float32)
    lib().oracle_bmm_softmax_bmm_literal(_p(A), _p(B), _p(C), _p(F), batch, M, N, K, L, in_dtype)
    return F


def exp_ref_literal(x):
    """The reference's CPU exponential (polynomial, clamped), bit for bit: intrinsic.py:1480-1672."""
    x = _f32(x)
    y = np.empty_like(x)
    lib().oracle_exp_ref_literal(_p(x), _p(y), x.size)
    return y


def bmm_softmax_bmm_cpu_literal(A, B, C):
    """The reference's fp32 CPU attention chain (benchmark/chimera/cpu/bmm_softmax_bmm.py:64-170)."""
    A, B, C = _f32(A), _f32(B), _f32(C)
    batch, M, N, K, L = _shape(A, B, C)
    F = np.empty((batch, M, N), dtype=np.float32)
    lib().oracle_bmm_softmax_bmm_cpu_literal(_p(A), _p(B), _p(C), _p(F), batch, M, N, K, L)
    return F


def bmm_softmax_bmm(A, B, C, scale=1.0, in_dtype=FP16, wide=False):
    """softmax(scale * A B) C in max-subtracted form; P rounded to in_dtype; fp32 result."""
    A, B, C = _f32(A), _f32(B), _f32(C)
    batch, M, N, K, L = _shape(A, B, C)
    F = np.empty((batch, M, N), np.float32)
    lib().oracle_bmm_softmax_bmm(_p(A), _p(B), _p(C), _p(F), batch, M, N, K, L, float(scale), in_dtype, int(wide))
    return F


def gemm_act_gemm(A, B, C, act=1, in_dtype=BF16, wide=False):
    """act(A B) C with the intermediate rounded to in_dtype; act 0 = identity, 1 = ReLU; fp32 result."""
    A, B, C = _f32(A), _f32(B), _f32(C)
    batch, M, N, K, L = _shape(A, B, C)
    F = np.empty((batch, M, N), np.float32)
    lib().oracle_gemm_act_gemm(_p(A), _p(B), _p(C), _p(F), batch, M, N, K, L, act, in_dtype, int(wide))
    return F


def ffn(A, B, b1, C, b2, act1=1, act2=1, in_dtype=BF16):
    """act2(round(act1(A B + b1)) C + b2); weights [in, out]; biases [batch, L] / [batch, N] or None."""
    A, B, C = _f32(A), _f32(B), _f32(C)
    batch, M, N, K, L = _shape(A, B, C)
    b1 = None if b1 is None else _f32(b1).reshape(batch, L)
    b2 = None if b2 is None else _f32(b2).reshape(batch, N)
    F = np.empty((batch, M, N), np.float32)
    null = ctypes.POINTER(ctypes.c_float)()
    lib().oracle_ffn(_p(A), _p(B), _p(b1) if b1 is not None else null, _p(C), _p(b2) if b2 is not None else null, _p(F),
                     batch, M, N, K, L, act1, act2, in_dtype)
    return F


def np_ffn(A, B, b1, C, b2, act1=1, act2=1, in_dtype=BF16):
    """numpy / fp64 restatement of ffn() for cross-checking the C code."""
    def act(v, a):
        if a == 1:
            return np.where(v > 0, v, 0.0)
        if a == 2:
            return 0.5 * v * (1.0 + np.tanh(v * 0.7978845608 * (1.0 + 0.044715 * v * v)))
        return v
    A, B, C = (np.asarray(t, np.float64) for t in (A, B, C))
    H = np.einsum("bmk,bkl->bml", A, B).astype(np.float32).astype(np.float64)
    if b1 is not None:
        H = H + np.asarray(b1, np.float64).reshape(A.shape[0], 1, -1)
    H = round_np(act(H, act1).astype(np.float32), in_dtype).astype(np.float64)
    Y = np.einsum("bml,bln->bmn", H, C).astype(np.float32).astype(np.float64)
    if b2 is not None:
        Y = Y + np.asarray(b2, np.float64).reshape(A.shape[0], 1, -1)
    return act(Y, act2).astype(np.float32)


def baseline_chain_fp32(A, B, C, kind, scale=1.0, threads=0):
    """The timed CPU baseline (blocked, multi-threaded fp32); kind 0 softmax, 1 ReLU, 2 identity."""
    A, B, C = _f32(A), _f32(B), _f32(C)
    batch, M, N, K, L = _shape(A, B, C)
    F = np.empty((batch, M, N), np.float32)
    rc = lib().baseline_chain_fp32(_p(A), _p(B), _p(C), _p(F), batch, M, N, K, L, kind, float(scale), threads)
    if rc != 0:
        raise ValueError("baseline_chain_fp32: L and N must be multiples of 16")
    return F


def max_threads():
    return int(lib().oracle_max_threads())


# ------------------------------------------------------------------ numpy restatements
def np_bmm_softmax_bmm_literal(A, B, C, in_dtype=FP16):
    """bmm_chain.py:40-103 line by line, including the padded ones column of C_ext."""
    A, B, C = (np.asarray(t, np.float32) for t in (A, B, C))
    batch, M, N, K, L = _shape(A, B, C)
    NI = 16
    ext_N = 2 ** int(np.ceil(np.log2(N // NI + 1))) * NI
    D = np.einsum("bmk,bkl->bml", A, B, dtype=np.float32)
    with np.errstate(over="ignore"):
        P = round_np(np.exp(D), in_dtype)
    C_ext = np.ones((batch, L, ext_N), np.float32)
    C_ext[:, :, :N] = C
    E = np.einsum("bml,bln->bmn", P, C_ext, dtype=np.float32)
    num = round_np(E[:, :, :N], in_dtype)
    den = round_np(round_np(E[:, :, ext_N - 1 :], in_dtype) + round_np(np.float32(1e-5), in_dtype), in_dtype)
    with np.errstate(invalid="ignore", divide="ignore"):
        return round_np(num / den, in_dtype)


def np_bmm_softmax_bmm(A, B, C, scale=1.0, in_dtype=FP32, wide=True):
    dt = np.float64 if wide else np.float32
    A, B, C = (np.asarray(t, dt) for t in (A, B, C))
    S = np.einsum("bmk,bkl->bml", A, B) * dt(scale)
    S = S - S.max(axis=-1, keepdims=True)
    P = np.exp(S)
    den = P.sum(axis=-1, keepdims=True)
    P = round_np(P.astype(np.float32), in_dtype).astype(dt)
    return (np.einsum("bml,bln->bmn", P, C) / den).astype(np.float32)


def np_gemm_act_gemm(A, B, C, act=1, in_dtype=FP32, wide=True):
    dt = np.float64 if wide else np.float32
    A, B, C = (np.asarray(t, dt) for t in (A, B, C))
    H = np.einsum("bmk,bkl->bml", A, B).astype(np.float32)
    if act == 1:
        H = np.where(H > 0, H, np.float32(0))
    H = round_np(H, in_dtype).astype(dt)
    return np.einsum("bml,bln->bmn", H, C).astype(np.float32)
