"""GPU parity tests of the fused bmm -> softmax -> bmm kernel, through the C ABI, against the CPU
oracle on the same seeded inputs.  Tolerances: tests/tolerances.py."""
import os

import numpy as np
import pytest
import torch

from ditto_b200 import _lib, ops
from ditto_b200 import workloads as W
from tests.golden import make_golden
from tests.tolerances import assert_close

pytestmark = pytest.mark.gpu

TDT = {"float16": torch.float16, "bfloat16": torch.bfloat16}
ODT = {"float16": 0, "bfloat16": 1}
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def _dev(a, dtype, cuda):
    return torch.from_numpy(np.ascontiguousarray(a)).to(cuda).to(TDT[dtype])


def _run(cuda, q, k, v, dtype, scale, layout="LK", flags=0):
    """q [b,M,K], k [b,L,K], v [b,L,N] float32 arrays of dtype-rounded values -> float32 result."""
    dq, dv = _dev(q, dtype, cuda), _dev(v, dtype, cuda)
    dk = _dev(k.transpose(0, 2, 1), dtype, cuda) if layout == "KL" else _dev(k, dtype, cuda)
    out = torch.full((q.shape[0], q.shape[1], v.shape[2]), float("nan"), dtype=TDT[dtype], device=cuda)  # poison
    ops.bmm_softmax_bmm(dq, dk, dv, out=out, scale=scale, key_layout=layout, flags=flags)
    assert ops.device_status(cuda) == 0
    return out.float().cpu().numpy()


def _oracle(oracle, q, k, v, dtype, scale):
    return oracle.bmm_softmax_bmm(q, np.ascontiguousarray(k.transpose(0, 2, 1)), v, scale, ODT[dtype], wide=False)


def _case(seed, b, M, L, d, dtype, dist="normal"):
    w = W.Workload("t", "softmax", b, M, d, d, L, dtype, 1.0, dist, seed)
    return W.attention_inputs(w, 0, b)


@pytest.mark.parametrize("b_mn,a_tmem", [(0, 0), (1, 0), (1, 1), (0, 1)])
@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
def test_umma_building_blocks(cuda, b_mn, a_tmem, dtype):
    """One tcgen05 MMA chain per operand form the fused kernels use, against a CPU product."""
    lib = _lib.load()
    status = torch.zeros(1, dtype=torch.int32, device=cuda)
    for N, K in ((64, 64), (128, 64), (64, 128), (128, 128), (256, 256)):
        rng = np.random.default_rng(N * 1000 + K)
        a = W._round(rng.standard_normal((128, K)).astype(np.float32), dtype)
        b = W._round(rng.standard_normal((K, N) if b_mn else (N, K)).astype(np.float32), dtype)
        c = torch.full((128, N), float("nan"), device=cuda)
        da, db = _dev(a, dtype, cuda), _dev(b, dtype, cuda)
        rc = lib.ditto_b200_selftest_umma(da.data_ptr(), db.data_ptr(), c.data_ptr(), N, K, ODT[dtype], b_mn, a_tmem,
                                          status.data_ptr(), None)
        torch.cuda.synchronize()
        assert rc == 0 and int(status.item()) == 0
        want = a.astype(np.float64) @ (b if b_mn else b.T).astype(np.float64)
        np.testing.assert_allclose(c.cpu().numpy(), want, rtol=1e-5, atol=2e-4)


@pytest.mark.parametrize("dtype,d", [("float16", 64), ("float16", 128), ("bfloat16", 64), ("bfloat16", 128)])
@pytest.mark.parametrize("layout", ["LK", "KL"])
@pytest.mark.parametrize("flags", [0, _lib.FLAG_ONE_TILE, _lib.FLAG_TWO_TILES, _lib.FLAG_P_VIA_SMEM,
                                   _lib.FLAG_P_VIA_SMEM | _lib.FLAG_ONE_TILE])
def test_parity_small(cuda, oracle, dtype, d, layout, flags):
    """Every kernel variant (dtype x head dim x key layout x tile count x P staging) on small shapes."""
    for (b, M, L) in ((2, 128, 128), (3, 256, 384), (1, 512, 128)):
        q, k, v = _case(11, b, M, L, d, dtype)
        scale = d ** -0.5
        got = _run(cuda, q, k, v, dtype, scale, layout, flags)
        assert_close(got, _oracle(oracle, q, k, v, dtype, scale), dtype, f"{dtype} d={d} {layout} flags={flags} {(b, M, L)}")


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
def test_reference_semantics_scale_one(cuda, oracle, dtype):
    """scale = 1 with U(-0.5,0.5) operands: the reference's exp / ones-column sum / divide chain
    (bmm_chain.py:64-103) and the kernel's max-subtracted softmax are the same function."""
    q, k, v = _case(12, 4, 256, 256, 64, dtype, dist="uniform_half")
    got = _run(cuda, q, k, v, dtype, 1.0, "KL")
    assert_close(got, _oracle(oracle, q, k, v, dtype, 1.0), dtype, "scale=1 stable")
    lit = oracle.bmm_softmax_bmm_literal(q, np.ascontiguousarray(k.transpose(0, 2, 1)), v, ODT[dtype])
    assert_close(got, lit, dtype, "scale=1 literal")


def test_large_logits_stay_finite(cuda, oracle):
    """Unscaled N(0,1) logits at d = 64 have sigma 8: exp() overflows fp16 in the reference's literal
    form; the online softmax must stay finite and match the stable oracle.  Also exercises the
    running-max rescale of the accumulator, which small logits never trigger."""
    q, k, v = _case(13, 2, 256, 512, 64, "float16")
    got = _run(cuda, q, k, v, "float16", 1.0)
    assert_close(got, _oracle(oracle, q, k, v, "float16", 1.0), "float16", "scale=1 N(0,1)")
    # rows whose maximum keeps growing block after block: forces a rescale at every K/V block
    k2 = k.copy()
    for j in range(4):
        k2[:, j * 128:(j + 1) * 128] *= np.float32(0.25 * (j + 1))
    k2 = W._round(k2, "float16")
    got = _run(cuda, q, k2, v, "float16", 1.0)
    assert_close(got, _oracle(oracle, q, k2, v, "float16", 1.0), "float16", "growing max")


@pytest.mark.parametrize("case", ["attn_fp16_d64", "attn_bf16_d128", "attn_fp16_reference_semantics"])
def test_golden_vectors(cuda, case):
    w = make_golden.workload(case)
    A, B, C = make_golden.inputs(case)   # B in the reference's [K, L] layout
    dq, dk, dv = _dev(A, w.dtype, cuda), _dev(B, w.dtype, cuda), _dev(C, w.dtype, cuda)
    out = ops.bmm_softmax_bmm(dq, dk, dv, scale=w.scale, key_layout="KL")
    assert ops.device_status(cuda) == 0
    stored = np.load(os.path.join(GOLDEN, case + ".npz"))
    for key in stored.files:
        assert_close(out.float().cpu().numpy(), stored[key], w.dtype, f"{case}:{key}")


def test_cfg2_full(cuda, oracle):
    """Benchmark configuration 2 at full size: 12 slices, S = 512, d = 64, fp16, scale 1/8, both key layouts."""
    w = W.WORKLOADS["cfg2"]
    q, k, v = W.attention_inputs(w, 0, w.batch)
    want = _oracle(oracle, q, k, v, w.dtype, w.scale)
    for layout in ("LK", "KL"):
        got = _run(cuda, q, k, v, w.dtype, w.scale, layout)
        mabs, mrel = assert_close(got, want, w.dtype, f"cfg2 {layout}")
        print(f"cfg2 {layout}: max abs {mabs:.3e} max rel {mrel:.3e}")


@pytest.mark.parametrize("name,slices", [("cfg3", (0, 1, 255, 256, 510, 511)), ("cfg5", (0, 127, 128, 511, 512, 1023))])
def test_large_configs_on_sampled_slices(cuda, oracle, name, slices):
    """Configs 3 and 5 at their own size (512 / 1024 slices in one launch): the sampled slices (first, last,
    the shard boundaries of 2 / 8 GPUs) are generated from their seeds and placed at their true index; the
    other slices hold unrelated random data, so a slice mix-up shows.  Compared with the oracle."""
    w = W.WORKLOADS[name]
    tdt = TDT[w.dtype]
    g = torch.Generator(device=cuda).manual_seed(5)
    n = w.batch
    q = torch.empty(n, w.M, w.K, device=cuda, dtype=tdt)
    k = torch.empty(n, w.L, w.K, device=cuda, dtype=tdt)
    v = torch.empty(n, w.L, w.N, device=cuda, dtype=tdt)
    for t in (q, k, v):                       # filled in pieces: no fp32 copy of a 700 MB tensor
        for lo in range(0, n, 64):
            t[lo:lo + 64] = torch.randn(t[lo:lo + 64].shape, device=cuda, generator=g).to(tdt)
    placed = {}
    for s in slices:
        qs, ks, vs = W.attention_slice(w, s)
        q[s], k[s], v[s] = (torch.from_numpy(t).to(cuda).to(tdt) for t in (qs, ks, vs))
        placed[s] = (qs, ks, vs)
    out = ops.bmm_softmax_bmm(q, k, v, scale=w.scale, key_layout="LK")
    assert ops.device_status(cuda) == 0
    for lo in range(0, n, 64):
        assert torch.isfinite(out[lo:lo + 64].float()).all()
    for s, (qs, ks, vs) in placed.items():
        want = _oracle(oracle, qs[None], ks[None], vs[None], w.dtype, w.scale)[0]
        assert_close(out[s].float().cpu().numpy(), want, w.dtype, f"{name} slice {s}")


def test_full_size_properties(cuda):
    """Size-independent properties at config-3 size (512 slices, S = 512, d = 64):
    * softmax rows sum to one: with V = all-ones the output is exactly 1 up to rounding;
    * permuting the K/V rows of a slice leaves the result unchanged;
    * the result is linear in V;
    * repeated launches are bitwise identical."""
    w = W.WORKLOADS["cfg3"]
    g = torch.Generator(device=cuda).manual_seed(9)
    q = torch.randn(w.batch, w.M, w.K, device=cuda, generator=g).half()
    k = torch.randn(w.batch, w.L, w.K, device=cuda, generator=g).half()
    v = torch.randn(w.batch, w.L, w.N, device=cuda, generator=g).half()
    ones = ops.bmm_softmax_bmm(q, k, torch.ones_like(v), scale=w.scale, key_layout="LK")
    assert (ones.float() - 1).abs().max().item() <= 2e-3
    base = ops.bmm_softmax_bmm(q, k, v, scale=w.scale, key_layout="LK")
    again = ops.bmm_softmax_bmm(q, k, v, scale=w.scale, key_layout="LK")
    assert torch.equal(base, again)
    perm = torch.randperm(w.L, device=cuda, generator=g)
    permuted = ops.bmm_softmax_bmm(q, k[:, perm].contiguous(), v[:, perm].contiguous(), scale=w.scale, key_layout="LK")
    assert (permuted.float() - base.float()).abs().max().item() <= 4e-3
    v2 = torch.randn(w.batch, w.L, w.N, device=cuda, generator=g).half()
    lin = ops.bmm_softmax_bmm(q, k, (v + 2 * v2).half(), scale=w.scale, key_layout="LK")
    second = ops.bmm_softmax_bmm(q, k, v2, scale=w.scale, key_layout="LK")
    assert (lin.float() - (base.float() + 2 * second.float())).abs().max().item() <= 1.5e-2
    assert ops.device_status(cuda) == 0


def test_reference_style_entry_point(cuda, oracle):
    """The chain built and launched the way the reference's benchmark does it
    (benchmark/chimera/cuda/bmm_softmax_bmm_cuda.py:158-261): builder -> fusion state ->
    tensorize_cuda -> build -> func(*inputs, *outputs) with caller-allocated, pre-filled outputs."""
    import ditto_b200 as ditto
    from ditto_b200 import auto_compute as ac, auto_tensorize as at, hardware as hw
    batch, M, N, K, L = 12, 512, 64, 64, 512
    ins, outs = ac.nn.functional.BatchGemmSoftmaxGemm(batch, M, N, K, L, "float16", "float32")
    A, B, C = ins
    (F,) = outs
    E_frag = F.op.input_tensors[0]
    exp, C_ext = E_frag.op.input_tensors
    D_frag = exp.op.input_tensors[0]
    b, m, n, mi, ni = E_frag.op.axis
    rlo, rli = E_frag.op.reduce_axis
    fuse_choice = at.fusion_choice(D_frag.op, E_frag.op, [b, m, n, rlo, mi, ni, rli], 3)
    p1 = at.cuda_wmma(M=16, N=16, K=16, in_dtype="float16", out_dtype="float32", scope="shared")
    p2 = at.cuda_wmma(M=16, N=16, K=16, in_dtype="float16", out_dtype="float32", scope="global")
    mi1 = at.match_info(at.intrinsic_match(D_frag, p1, ["InnerMost", "SameRange"])[0], p1)
    mi2 = at.match_info(at.intrinsic_match(E_frag, p2, ["InnerMost", "SameRange"])[0], p2)
    layer = ac.layer([F.op], inputs=[A, B, C])
    state = at.tensorize_hyper_fusion_state(layer, fuse_choice, {D_frag.op: mi1, E_frag.op: mi2})
    sch = at.tensorize_cuda(layer, state, hw.query_hw_param("gpu.cuda.B200"), at.cuda_tensorize_param(ty_size=4, tz_size=2))
    func = ditto.build(sch, layer.schedule_tensors, "cuda")
    rng = np.random.default_rng(3)
    a, bb, c = (W._round(rng.uniform(-0.5, 0.5, t.shape).astype(np.float32), "float16") for t in ins)
    f = torch.from_numpy(rng.uniform(-1, 1, F.shape).astype(np.float32)).to(cuda).half()
    func(_dev(a, "float16", cuda), _dev(bb, "float16", cuda), _dev(c, "float16", cuda), f)
    assert ops.device_status(cuda) == 0
    want = oracle.bmm_softmax_bmm(a, bb, c, 1.0, 0, wide=False)
    assert_close(f.float().cpu().numpy(), want, "float16", "reference-style entry")
    cost = func.time_evaluator(func.entry_name, None, min_repeat_ms=50)(_dev(a, "float16", cuda), _dev(bb, "float16", cuda),
                                                                        _dev(c, "float16", cuda), f).mean
    assert 0 < cost < 1e-2


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
@pytest.mark.parametrize("layout", ["LK", "KL"])
def test_ragged_shapes(cuda, oracle, dtype, layout):
    """Shapes that are multiples of 16 but not of the 128-row tiles, and head dimensions other than
    64 / 128: the rest of the reference's benchmark table (ViT-*/16: 196 -> 208 tokens, ViT-Huge:
    d = 80, Mixer: M != L; benchmark/chimera/cuda/bmm_softmax_bmm_cuda.py:294-308) plus corner cases
    (a single 16-row tile, tails on both M and L, d = 16).  Outputs are poison-filled first."""
    shapes = ((12, 208, 64, 208), (16, 208, 80, 208), (16, 256, 80, 256), (1, 512, 64, 256), (1, 768, 64, 384),
              (2, 16, 16, 16), (3, 144, 48, 272), (2, 400, 112, 144), (1, 1040, 128, 528))
    for (b, M, d, L) in shapes:
        q, k, v = _case(17, b, M, L, d, dtype)
        scale = d ** -0.5
        for flags in (0, _lib.FLAG_ONE_TILE, _lib.FLAG_TWO_TILES):
            got = _run(cuda, q, k, v, dtype, scale, layout, flags)
            assert_close(got, _oracle(oracle, q, k, v, dtype, scale), dtype, f"{dtype} {layout} flags={flags} {(b, M, d, L)}")


def test_many_slices(cuda):
    """More slices than the 65535 of a grid's y / z dimension (e.g. batch x heads of a long batch)."""
    n = 70000
    g = torch.Generator(device=cuda).manual_seed(2)
    q = torch.randn(n, 128, 64, device=cuda, generator=g).half()
    k = torch.randn(n, 128, 64, device=cuda, generator=g).half()
    v = torch.randn(n, 128, 64, device=cuda, generator=g).half()
    out = ops.bmm_softmax_bmm(q, k, v, scale=0.125, key_layout="LK")
    assert ops.device_status(cuda) == 0
    for i in (0, 65535, 65536, n - 1):
        ref = torch.softmax(q[i].float() @ k[i].float().t() * 0.125, -1) @ v[i].float()
        assert (out[i].float() - ref).abs().max().item() <= 2e-3


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_work_loop_many_items(cuda, dtype):
    """Head dims <= 64 with at most 1024 keys run a persistent kernel whose CTAs walk several
    (slice, row block) items each, with Q double-buffered and scores issued across item borders:
    every output row of a launch with ~7 items per CTA is compared with a float32 product, for one
    to five key blocks per item and a ragged tail.  1152 keys take the non-persistent kernel."""
    g = torch.Generator(device=cuda).manual_seed(5)
    for (b, M, L, d) in ((2100, 128, 128, 64), (1050, 256, 256, 64), (700, 384, 640, 64), (530, 208, 400, 48),
                         (300, 512, 1024, 32), (40, 512, 1152, 64)):
        q = (torch.rand(b, M, d, device=cuda, generator=g) - 0.5).to(dtype)
        k = (torch.rand(b, L, d, device=cuda, generator=g) - 0.5).to(dtype)
        v = (torch.rand(b, L, d, device=cuda, generator=g) - 0.5).to(dtype)
        out = torch.full((b, M, d), float("nan"), dtype=dtype, device=cuda)
        ops.bmm_softmax_bmm(q, k, v, out=out, scale=1.0, key_layout="LK")
        assert ops.device_status(cuda) == 0
        ref = torch.softmax(q.float() @ k.float().transpose(1, 2), -1) @ v.float()
        tol = 2e-2 if dtype == torch.float16 else 3e-2
        err = (out.float() - ref).abs()
        bound = tol * ref.abs() + (1e-3 if dtype == torch.float16 else 4e-3)
        assert not torch.isnan(out).any(), (b, M, L, d)
        assert bool((err <= bound).all()), ((b, M, L, d), err.max().item())


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_work_loop_head_dimension_128(cuda, dtype):
    """Head dimensions above 64 run the two-tile (one-tile for M <= 128) kernel inside a work loop: one CTA per
    SM walks the (slice, tile) items, Q is reloaded per item behind the item's last scores, the next item's first
    scores are issued behind the last P V.  Every output row of launches with more items than SMs is compared with
    a float32 product: one key block per item (its only scores are also its last), two, three and many; a
    partial second query tile; a ragged key tail; the reference's transposed-K layout; a narrower value width."""
    g = torch.Generator(device=cuda).manual_seed(7)
    cases = ((330, 128, 128, 128, 128, "LK"), (170, 384, 128, 96, 96, "LK"), (160, 256, 256, 128, 128, "KL"),
             (150, 512, 384, 80, 80, "LK"), (80, 528, 1104, 128, 64, "LK"), (24, 2048, 2048, 128, 128, "LK"))
    for (b, M, L, d, dv, layout) in cases:
        q = (torch.rand(b, M, d, device=cuda, generator=g) - 0.5).to(dtype)
        k = (torch.rand(b, L, d, device=cuda, generator=g) - 0.5).to(dtype)
        v = (torch.rand(b, L, dv, device=cuda, generator=g) - 0.5).to(dtype)
        out = torch.full((b, M, dv), float("nan"), dtype=dtype, device=cuda)
        kk = k.transpose(1, 2).contiguous() if layout == "KL" else k
        ops.bmm_softmax_bmm(q, kk, v, out=out, scale=1.0, key_layout=layout)
        assert ops.device_status(cuda) == 0
        ref = torch.softmax(q.float() @ k.float().transpose(1, 2), -1) @ v.float()
        tol = 2e-2 if dtype == torch.float16 else 3e-2
        err = (out.float() - ref).abs()
        bound = tol * ref.abs() + (1e-3 if dtype == torch.float16 else 4e-3)
        assert not torch.isnan(out).any(), (b, M, L, d, dv, layout)
        assert bool((err <= bound).all()), ((b, M, L, d, dv, layout), err.max().item())
        again = torch.empty_like(out)
        ops.bmm_softmax_bmm(q, kk, v, out=again, scale=1.0, key_layout=layout)
        assert torch.equal(out, again), "runs of the work loop differ"


def test_unsupported_shapes_raise(cuda):
    q = torch.zeros(1, 128, 144, dtype=torch.float16, device=cuda)     # head dimension above 128
    kv = torch.zeros(1, 128, 64, dtype=torch.float16, device=cuda)
    with pytest.raises(_lib.DittoError) as e:
        ops.bmm_softmax_bmm(q, q, q, key_layout="LK")
    assert e.value.code == _lib.ERR_UNSUPPORTED
    with pytest.raises(_lib.DittoError) as e:
        ops.bmm_softmax_bmm(kv[:, :120].contiguous(), kv, kv, key_layout="LK")   # M = 120 is not a multiple of 16
    assert e.value.code == _lib.ERR_INVALID_ARG
    with pytest.raises(ValueError):
        ops.bmm_softmax_bmm(kv, kv[:, :, :32].contiguous(), kv, key_layout="LK")
    with pytest.raises(ValueError):
        ops.bmm_softmax_bmm(kv, kv.transpose(1, 2), kv, key_layout="KL")   # non-contiguous


@pytest.mark.parametrize("b_mn", [0, 1])
@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
def test_umma_pair_building_block(cuda, b_mn, dtype):
    """One cta_group::2 MMA chain (two CTAs, M = 256) against a CPU product: 2-CTA TMEM allocation,
    TMA byte counts reported to the leader's barrier, the split of B between the CTAs and the
    completion signal to both."""
    lib = _lib.load()
    status = torch.zeros(1, dtype=torch.int32, device=cuda)
    for N, K in ((128, 64), (256, 64), (128, 256), (256, 256)):
        rng = np.random.default_rng(N * 1000 + K + 7)
        a = W._round(rng.standard_normal((256, K)).astype(np.float32), dtype)
        b = W._round(rng.standard_normal((K, N) if b_mn else (N, K)).astype(np.float32), dtype)
        c = torch.full((256, N), float("nan"), device=cuda)
        da, db = _dev(a, dtype, cuda), _dev(b, dtype, cuda)
        rc = lib.ditto_b200_selftest_umma_pair(da.data_ptr(), db.data_ptr(), c.data_ptr(), N, K, ODT[dtype], b_mn,
                                               status.data_ptr(), None)
        torch.cuda.synchronize()
        assert rc == 0 and int(status.item()) == 0
        want = a.astype(np.float64) @ (b if b_mn else b.T).astype(np.float64)
        np.testing.assert_allclose(c.cpu().numpy(), want, rtol=1e-5, atol=2e-4)


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
def test_value_width_differs_from_key_width(cuda, oracle, dtype):
    """N != K: the reference's definition takes the width of V / the output (N) and the reduction length of
    Q K^T (K) independently (bmm_chain.py:28-38).  Both layouts of K, ragged rows included."""
    for (batch, M, N, K, L) in ((2, 256, 128, 64, 256), (3, 208, 64, 128, 272), (1, 128, 48, 80, 144),
                                (2, 384, 32, 64, 1040), (1, 512, 112, 16, 512)):
        rng = np.random.default_rng(97)
        q = W._round(rng.standard_normal((batch, M, K)).astype(np.float32), dtype)
        k = W._round(rng.standard_normal((batch, L, K)).astype(np.float32), dtype)
        v = W._round(rng.standard_normal((batch, L, N)).astype(np.float32), dtype)
        want = _oracle(oracle, q, k, v, dtype, K ** -0.5)
        for layout in ("LK", "KL"):
            got = _run(cuda, q, k, v, dtype, K ** -0.5, layout)
            assert got.shape == (batch, M, N)
            assert_close(got, want, dtype, f"{dtype} N != K {(batch, M, N, K, L)} {layout}")
