"""CPU tests of the oracle itself: rounding helpers, C vs numpy restatements, the checks the
reference's own tests make, and the committed golden vectors."""
import glob
import os

import numpy as np
import pytest
import torch

from ditto_b200 import workloads as W

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def _rand(seed, shape, lo=-1.0, hi=1.0):
    return np.random.default_rng(seed).uniform(lo, hi, shape).astype(np.float32)


@pytest.mark.parametrize("dt", [0, 1])
def test_rounding_matches_numpy_and_torch(oracle, dt):
    rng = np.random.default_rng(7)
    x = rng.standard_normal(200000).astype(np.float32) * np.float32(10.0) ** rng.integers(-9, 6, 200000).astype(np.float32)
    x = np.concatenate([x, np.float32([0, -0.0, 65504, 65519.9, 65520, 1e-8, 6e-8, 2 ** -24, 2 ** -25, 3 * 2 ** -25])])
    c = oracle.round_c(x, dt)
    assert np.array_equal(c, oracle.round_np(x, dt))
    tdt = torch.float16 if dt == 0 else torch.bfloat16
    t = torch.from_numpy(x).to(tdt).float().numpy()
    assert np.array_equal(c, t)


def test_c_matches_numpy_restatements(oracle):
    A, B, C = _rand(1, (3, 48, 32)), _rand(2, (3, 32, 80)), _rand(3, (3, 80, 48))
    for dt in (0, 1):
        A16, B16, C16 = (oracle.round_np(t, dt) for t in (A, B, C))
        lit_c = oracle.bmm_softmax_bmm_literal(A16, B16, C16, dt)
        lit_np = oracle.np_bmm_softmax_bmm_literal(A16, B16, C16, dt)
        ulp = 2.0 ** (-10 if dt == 0 else -7)
        assert np.abs(lit_c - lit_np).max() <= ulp * np.abs(lit_np).max()  # at most one rounding step apart
        st_c = oracle.bmm_softmax_bmm(A16, B16, C16, 0.7, dt, wide=True)
        st_np = oracle.np_bmm_softmax_bmm(A16, B16, C16, 0.7, dt, wide=True)
        # exp in C vs numpy may differ in the last bit before rounding P to in_dtype
        assert np.abs(st_c - st_np).max() <= 2 * ulp * np.abs(st_np).max()
        for act in (0, 1):
            g_c = oracle.gemm_act_gemm(A16, B16, C16, act, dt, wide=True)
            g_np = oracle.np_gemm_act_gemm(A16, B16, C16, act, dt, wide=True)
            assert np.abs(g_c - g_np).max() <= 1e-5 * np.abs(g_np).max()


def test_fp32_paths_agree_with_fp64(oracle):
    A, B, C = _rand(4, (2, 64, 64)), _rand(5, (2, 64, 128)), _rand(6, (2, 128, 64))
    a = oracle.bmm_softmax_bmm(A, B, C, 1.0, oracle.FP32, wide=False)
    b = oracle.bmm_softmax_bmm(A, B, C, 1.0, oracle.FP32, wide=True)
    np.testing.assert_allclose(a, b, rtol=1e-4, atol=1e-6)
    a = oracle.gemm_act_gemm(A, B, C, 1, oracle.FP32, wide=False)
    b = oracle.gemm_act_gemm(A, B, C, 1, oracle.FP32, wide=True)
    np.testing.assert_allclose(a, b, rtol=1e-4, atol=1e-4)


def test_literal_and_stable_forms_agree(oracle):
    """exp/sum with the ones column and +1e-5 (reference-literal) vs max-subtracted softmax:
    identical up to the epsilon and rounding while nothing overflows (inputs U(-0.5,0.5), K=64)."""
    A, B, C = (oracle.round_np(t, 0) for t in (_rand(7, (2, 64, 64), -0.5, 0.5), _rand(8, (2, 64, 256), -0.5, 0.5),
                                               _rand(9, (2, 256, 64))))
    lit = oracle.bmm_softmax_bmm_literal(A, B, C, 0)
    st = oracle.bmm_softmax_bmm(A, B, C, 1.0, 0, wide=True)
    np.testing.assert_allclose(lit, st, rtol=4e-3, atol=1e-3)


def test_literal_fp16_form_overflows_where_stable_does_not(oracle):
    """With U(-1,1) operands and K = 64 some logits pass ln(65504) ~ 11.09, exp() rounds to inf in
    fp16 and the reference-literal chain yields non-finite rows -- the NaNs the reference's own GPU
    test reports (testing/hyper_fusion/bmm_softmax_bmm_wmma_m16n16k16_fp16fp16fp32.py:612-613).
    The max-subtracted form the kernels implement stays finite on the same inputs."""
    A, B, C = (oracle.round_np(t, 0) for t in (_rand(7, (2, 64, 64)), _rand(8, (2, 64, 256)), _rand(9, (2, 256, 64))))
    lit = oracle.bmm_softmax_bmm_literal(A, B, C, 0)
    st = oracle.bmm_softmax_bmm(A, B, C, 1.0, 0, wide=True)
    assert not np.isfinite(lit).all()
    assert np.isfinite(st).all()
    # rows whose exp row-sum stays inside fp16 range still agree; the others are NaN (inf/inf) or
    # collapse to 0 (finite/inf)
    rowsum = np.exp(np.einsum("bmk,bkl->bml", A, B)).sum(-1)
    ok = rowsum < 3.0e4
    assert ok.any() and not ok.all()
    np.testing.assert_allclose(lit[ok], st[ok], rtol=4e-3, atol=1e-3)


def test_reference_test_llvm_pin(oracle):
    """The one numeric assertion the reference makes on this chain: its fp32 CPU build equals
    torch.bmm -> softmax -> bmm at (12, 512, 64, 64, 512), U(-1, 1), rtol = atol = 0.1
    (testing/hyper_fusion/bmm_softmax_bmm_wmma_m16n16k16_fp16fp16fp32.py:552-587).  The oracle in
    both forms must satisfy it (and does so far inside the tolerance)."""
    A, B, C = _rand(10, (12, 512, 64)), _rand(11, (12, 64, 512)), _rand(12, (12, 512, 64))
    want = torch.bmm(torch.softmax(torch.bmm(torch.from_numpy(A), torch.from_numpy(B)), dim=-1), torch.from_numpy(C)).numpy()
    for got in (oracle.bmm_softmax_bmm_literal(A, B, C, oracle.FP32), oracle.bmm_softmax_bmm(A, B, C, 1.0, oracle.FP32)):
        np.testing.assert_allclose(got, want, rtol=0.1, atol=0.1)
        np.testing.assert_allclose(got, want, rtol=1e-3, atol=1e-4)


def test_reference_micro_kernel_pin(oracle):
    """python_test/auto_tensorize/test_cpu_intrin.py:1013-1096 checks the reference's GEMM
    micro-kernel on all-ones operands against numpy (atol = 1, rtol = 1e-3); the baseline's
    6 x 16 register tile must pass the same check."""
    for (M, K, L, N) in ((6, 64, 16, 16), (12, 256, 64, 32), (7, 64, 48, 16)):
        A, B, C = np.ones((1, M, K), np.float32), np.ones((1, K, L), np.float32), np.ones((1, L, N), np.float32)
        got = oracle.baseline_chain_fp32(A, B, C, 2)
        np.testing.assert_allclose(got, np.full((1, M, N), float(K * L), np.float32), atol=1, rtol=1e-3)


@pytest.mark.parametrize("kind", [0, 1, 2])
def test_baseline_matches_oracle(oracle, kind):
    A, B, C = _rand(13, (3, 100, 64)), _rand(14, (3, 64, 128)), _rand(15, (3, 128, 64))
    got = oracle.baseline_chain_fp32(A, B, C, kind, 0.5)
    if kind == 0:
        want = oracle.bmm_softmax_bmm(A, B, C, 0.5, oracle.FP32, wide=True)
    else:
        want = oracle.gemm_act_gemm(A, B, C, 1 if kind == 1 else 0, oracle.FP32, wide=True)
    np.testing.assert_allclose(got, want, rtol=2e-4, atol=2e-4)


def test_ffn_c_matches_numpy(oracle):
    A, B, C = _rand(20, (2, 40, 64)), _rand(21, (2, 64, 96), -0.2, 0.2), _rand(22, (2, 96, 48), -0.2, 0.2)
    b1, b2 = _rand(23, (2, 96)), _rand(24, (2, 48))
    for a1, a2 in ((1, 1), (2, 0), (0, 2)):
        got = oracle.ffn(A, B, b1, C, b2, a1, a2, oracle.BF16)
        want = oracle.np_ffn(A, B, b1, C, b2, a1, a2, oracle.BF16)
        np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-5)
    # without biases and with ReLU / identity it is the plain chain
    np.testing.assert_allclose(oracle.ffn(A, B, None, C, None, 1, 0, oracle.BF16),
                               oracle.gemm_act_gemm(A, B, C, 1, oracle.BF16, wide=True), rtol=1e-6, atol=1e-6)


def test_cfg1_cpu_case(oracle):
    """Benchmark configuration 1: E = (A B) D in fp32, A[8,512,64] B[8,64,512] D[8,512,64] ~ U(-1,1)."""
    w = W.WORKLOADS["cfg1"]
    A, B, C = W.chain_inputs(w)
    want = np.einsum("bml,bln->bmn", np.einsum("bmk,bkl->bml", A.astype(np.float64), B.astype(np.float64)), C.astype(np.float64))
    got = oracle.gemm_act_gemm(A, B, C, 0, oracle.FP32)
    np.testing.assert_allclose(got, want, rtol=1e-4, atol=1e-3)
    np.testing.assert_allclose(oracle.baseline_chain_fp32(A, B, C, 2), want, rtol=1e-4, atol=1e-3)


def test_golden_vectors(oracle):
    """Committed outputs (tests/golden/*.npz, written by tests/golden/make_golden.py) are
    reproduced bit for bit by today's oracle on the regenerated seeded inputs."""
    from tests.golden import make_golden
    files = [f for f in sorted(glob.glob(os.path.join(GOLDEN, "*.npz")))
             if os.path.splitext(os.path.basename(f))[0] in make_golden.CASES]
    assert files, "no golden vectors committed"
    for path in files:
        case = os.path.splitext(os.path.basename(path))[0]
        stored = np.load(path)
        fresh = make_golden.compute(case, oracle)
        for key in stored.files:
            assert np.array_equal(stored[key], fresh[key]), f"{case}:{key} changed"


# ---------------------------------------------------------------- pins against the reference's own micro-kernels
REF_GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "ref_microkernels.npz")


def _bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def test_reference_microkernel_golden_exp(oracle):
    """oracle_exp_ref_literal reproduces the reference's AVX-512 exponential bit for bit on the committed
    vectors (edge values, +-90, N(0, 8), U(-1, 1)); those vectors were produced by the kernel the reference
    generates (intrinsic.py:1480-1672), see tests/golden/make_ref_golden.py."""
    g = np.load(REF_GOLDEN)
    got = oracle.exp_ref_literal(g["exp_x"])
    assert np.array_equal(_bits(got), _bits(g["exp_y"]))
    # and what that kernel is: exp up to the Cody-Waite sign slip, 4.24e-4 relative per unit of round(x / ln 2)
    x = g["exp_x"].astype(np.float64)
    inside = np.abs(x) < 80
    n = np.floor(g["exp_x"] * np.float32(1.44269504088896341) + np.float32(0.5)).astype(np.float64)   # as the kernel rounds it
    model = np.exp(x) * np.exp(2 * n * -2.12194440e-4)
    assert np.max(np.abs(g["exp_y"][inside] / model[inside] - 1)) < 5e-6


def test_reference_microkernel_golden_chains(oracle):
    """The three CPU chains evaluated through the reference's 6 x 16 GEMM micro-kernel (and its exponential):
    the C restatement equals them bit for bit where it fixes the operation order (the literal softmax chain,
    the timed baseline's register tile), and to 1e-6 relative where the compiler chooses it."""
    g = np.load(REF_GOLDEN)
    i = 0
    while f"c{i}_shape" in g:
        a, b, c = g[f"c{i}_a"], g[f"c{i}_b"], g[f"c{i}_c"]
        assert np.array_equal(_bits(oracle.bmm_softmax_bmm_cpu_literal(a, b, c)), _bits(g[f"c{i}_bmm_softmax_bmm"])), i
        assert np.array_equal(_bits(oracle.baseline_chain_fp32(a, b, c, 2)), _bits(g[f"c{i}_bmm_bmm"])), i
        assert np.array_equal(_bits(oracle.baseline_chain_fp32(a, b, c, 1)), _bits(g[f"c{i}_bmm_relu_bmm"])), i
        for act, key in ((2, "bmm_bmm"), (1, "bmm_relu_bmm")):
            got = oracle.gemm_act_gemm(a, b, c, act=act, in_dtype=oracle.FP32)
            want = g[f"c{i}_{key}"]
            assert np.max(np.abs(got - want)) <= 1e-6 * np.max(np.abs(want)) + 1e-6, (i, key)
        # the stable-softmax oracle the GPU tests use differs from the reference's CPU chain only by the
        # exponential's error (<= 4.24e-4 * |n|, partly cancelling in the quotient) and summation order
        stable = oracle.bmm_softmax_bmm(a, b, c, 1.0, oracle.FP32, wide=True)
        want = g[f"c{i}_bmm_softmax_bmm"]
        assert np.max(np.abs(stable - want)) <= 2e-2 * np.max(np.abs(want)), i
        i += 1
    assert i == 3


def test_reference_microkernel_golden_ffn(oracle):
    """The feed-forward block -- linear + bias -> ReLU -> linear + bias -> ReLU with [out, in] weights
    (nn/model/transformer.py:21-34, nn/functional/linear.py:4-41) -- evaluated through the reference's GEMM
    micro-kernel: the C restatement `oracle_ffn` (fp32, no rounding of the hidden layer) agrees to 1e-6."""
    g = np.load(REF_GOLDEN)
    i = 0
    while f"f{i}_x" in g:
        x, w1, b1, w2, b2 = (g[f"f{i}_{k}"] for k in ("x", "w1", "b1", "w2", "b2"))
        io1, io2 = np.ascontiguousarray(w1.T)[None], np.ascontiguousarray(w2.T)[None]
        for key, a1, a2, bias in (("relu_relu", 1, 1, True), ("relu_identity", 1, 0, True),
                                  ("identity_identity_nobias", 0, 0, False)):
            got = oracle.ffn(x[None], io1, b1[None] if bias else None, io2, b2[None] if bias else None, a1, a2,
                             oracle.FP32)[0]
            want = g[f"f{i}_{key}"]
            assert np.max(np.abs(got - want)) <= 1e-6 * np.max(np.abs(want)) + 1e-6, (i, key)
        i += 1
    assert i == 2


def test_reference_microkernels_live(oracle):
    """Where the reference tree (or the library built from it) is present: fresh seeded inputs through the
    reference's micro-kernels against the restatement, so the pin is not limited to the committed cases."""
    from oracle import ref_microkernels as R
    if not R.available():
        pytest.skip("reference micro-kernel library not built (no reference tree on this machine)")
    rng = np.random.default_rng(2024)
    for (batch, M, N, K, L) in ((1, 13, 16, 32, 32), (2, 30, 48, 128, 64)):
        a = rng.uniform(-1, 1, (batch, M, K)).astype(np.float32)
        b = rng.uniform(-1, 1, (batch, K, L)).astype(np.float32)
        c = rng.uniform(-1, 1, (batch, L, N)).astype(np.float32)
        assert np.array_equal(_bits(oracle.baseline_chain_fp32(a, b, c, 2)), _bits(R.bmm_bmm(a, b, c)))
        assert np.array_equal(_bits(oracle.baseline_chain_fp32(a, b, c, 1)), _bits(R.bmm_relu_bmm(a, b, c)))
        if R.has_exp():
            assert np.array_equal(_bits(oracle.bmm_softmax_bmm_cpu_literal(a, b, c)), _bits(R.bmm_softmax_bmm_cpu(a, b, c)))
    x = rng.standard_normal((14, 32)).astype(np.float32)
    w1, w2 = rng.standard_normal((48, 32)).astype(np.float32) / 6, rng.standard_normal((32, 48)).astype(np.float32) / 7
    b1, b2 = rng.standard_normal(48).astype(np.float32), rng.standard_normal(32).astype(np.float32)
    got = oracle.ffn(x[None], np.ascontiguousarray(w1.T)[None], b1[None], np.ascontiguousarray(w2.T)[None], b2[None], 1, 1,
                     oracle.FP32)[0]
    want = R.ffn(x, w1, b1, w2, b2, True, True)
    assert np.max(np.abs(got - want)) <= 1e-6 * np.max(np.abs(want)) + 1e-6
    if R.has_exp():
        x = rng.normal(0, 20, (24, 64)).astype(np.float32)
        assert np.array_equal(_bits(oracle.exp_ref_literal(x)), _bits(R.exp(x)))
