"""Chain definitions (the `ditto.auto_compute.nn.functional` ops on the fused-chain path).

Each builder returns the output tensor of a symbolic DAG with the same op names and the same
producer structure as the reference's TE definition, so caller code that walks
`F.op.input_tensors` keeps working.  Shapes follow the reference tuple (batch, M, N, K, L):
query/A [batch, M, K], key/B [batch, K, L], value/C [batch, L, N], result [batch, M, N].
"""
import math

from .... import te


def _dims(A, B, C):
    batch, M, K = A.shape
    _b, _K, L = B.shape
    _b2, _L, N = C.shape
    if not (batch == _b == _b2 and K == _K and L == _L):
        raise ValueError(f"inconsistent chain shapes: {A.shape} x {B.shape} x {C.shape}")
    return batch, M, N, K, L


def _first_gemm(A, B, MI, NI, KI, in_dtype, acc_dtype):
    batch, M, K = A.shape
    L = B.shape[2]
    A_shared = te.compute([batch, M // MI, K // KI, MI, KI], [A], "A_shared", in_dtype,
                          axis_names=["b", "mo", "ko", "mi", "ki"])
    B_shared = te.compute([batch, K // KI, L // NI, KI, NI], [B], "B_shared", in_dtype,
                          axis_names=["b", "ko", "lo", "ki", "li"])
    D_frag = te.compute([batch, M // MI, L // NI, MI, NI], [A_shared, B_shared], "D_frag", acc_dtype, tag="cubic",
                        axis_names=["b", "mo", "lo", "mi", "li"], reduce=[("rko", K // KI), ("rki", KI)])
    return D_frag


def BatchGemmSoftmaxGemmMMA(query, key, value, MI=16, NI=16, KI=16, in_dtype="float16", acc_dtype="float32",
                            scale=1.0):
    """Fused attention chain: F = exp(Q K) [V | 1] normalised by its last column.

    Mirrors python/ditto/auto_compute/nn/functional/bmm_chain.py:5-104: the same asserts on the
    16 x 16 x 16 tiling, the same intermediate ops (A_shared, B_shared, D_frag, exp, C_ext with
    the appended ones column, E_frag, F).  `key` is the reference's pre-transposed [batch, K, L].
    `scale` (default 1 = the reference's semantics) multiplies the logits before the exponential.
    """
    batch, M, N, K, L = _dims(query, key, value)
    assert M % MI == 0, f"M={M}, MI={MI}"
    assert N % NI == 0, f"N={N}, NI={NI}"
    assert K % KI == 0, f"K={K}, KI={KI}"
    assert L % NI == 0, f"L={L}, NI={NI}"
    assert L % KI == 0, f"L={L}, KI={KI}"
    D_frag = _first_gemm(query, key, MI, NI, KI, in_dtype, acc_dtype)
    exp = te.compute(D_frag.shape, [D_frag], "exp", in_dtype, tag="exp",
                     axis_names=["b", "mo", "lo", "mi", "li"], attrs={"scale": float(scale)})
    ext_N = 2 ** math.ceil(math.log2(N // NI + 1)) * NI
    C_ext = te.compute([batch, L // KI, ext_N // NI, KI, NI], [value], "C_ext", in_dtype, tag="pad_ones",
                       axis_names=["b", "lo", "no", "li", "ni"])
    E_frag = te.compute([batch, M // MI, ext_N // NI, MI, NI], [exp, C_ext], "E_frag", acc_dtype, tag="cubic",
                        axis_names=["b", "mo", "no", "mi", "ni"], reduce=[("rlo", L // KI), ("rli", KI)])
    F = te.compute([batch, M, N], [E_frag], "F", in_dtype, tag="normalize", axis_names=["b", "m", "n"])
    return F


def BatchGemmSoftmaxGemm(batch, M, N, K, L, in_dtype="float16", acc_dtype="float32", scale=1.0):
    """Placeholder-creating form used by the reference's benchmarks
    (benchmark/chimera/cuda/bmm_softmax_bmm_cuda.py:69-155): returns ([A, B, C], [F])."""
    A = te.placeholder([batch, M, K], name="A", dtype=in_dtype)
    B = te.placeholder([batch, K, L], name="B", dtype=in_dtype)
    C = te.placeholder([batch, L, N], name="C", dtype=in_dtype)
    F = BatchGemmSoftmaxGemmMMA(A, B, C, in_dtype=in_dtype, acc_dtype=acc_dtype, scale=scale)
    return [A, B, C], [F]


def _gemm_chain(batch, M, N, K, L, in_dtype, acc_dtype, act):
    MI = NI = KI = 16
    for v, nm in ((M, "M"), (N, "N"), (K, "K"), (L, "L")):
        assert v % 16 == 0, f"{nm}={v} must be a multiple of 16"
    A = te.placeholder([batch, M, K], name="A", dtype=in_dtype)
    B = te.placeholder([batch, K, L], name="B", dtype=in_dtype)
    C = te.placeholder([batch, L, N], name="C", dtype=in_dtype)
    D_frag = _first_gemm(A, B, MI, NI, KI, in_dtype, acc_dtype)
    mid = te.compute(D_frag.shape, [D_frag], "relu" if act == "relu" else "cast", in_dtype,
                     tag="relu" if act == "relu" else "identity", axis_names=["b", "mo", "lo", "mi", "li"])
    C_ext = te.compute([batch, L // KI, N // NI, KI, NI], [C], "C_ext", in_dtype,
                       axis_names=["b", "lo", "no", "li", "ni"])
    E_frag = te.compute([batch, M // MI, N // NI, MI, NI], [mid, C_ext], "E_frag", acc_dtype, tag="cubic",
                        axis_names=["b", "mo", "no", "mi", "ni"], reduce=[("rlo", L // KI), ("rli", KI)])
    F = te.compute([batch, M, N], [E_frag], "F", in_dtype, tag="identity", axis_names=["b", "m", "n"])
    return [A, B, C], [F]


def BatchGemmGemm(batch=1, M=512, N=64, K=64, L=512, in_dtype="float16", acc_dtype="float32"):
    """Plain chain F = (A B) C with the intermediate cast to in_dtype
    (benchmark/chimera/cuda/bmm_bmm_cuda.py:69-150)."""
    return _gemm_chain(batch, M, N, K, L, in_dtype, acc_dtype, "identity")


def BatchGemmReluGemm(batch=1, M=512, N=64, K=64, L=512, in_dtype="bfloat16", acc_dtype="float32"):
    """F = relu(A B) C, relu as if_then_else(D > 0, D, 0) cast to in_dtype
    (python_test/auto_tensorize/test_hyper_fusion_cpu.py:24-96, evaluation/cpu/bmm_relu_bmm.py:56-125)."""
    return _gemm_chain(batch, M, N, K, L, in_dtype, acc_dtype, "relu")
