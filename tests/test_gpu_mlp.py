"""GPU parity tests of the fused GEMM -> activation -> GEMM kernel, through the C ABI, against the
CPU oracle on the same seeded inputs.  Tolerances: tests/tolerances.py (the absolute floor is scaled
by the magnitude of the result, which grows with the hidden size)."""
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


def _inputs(seed, batch, M, N, K, L, dtype):
    rng = np.random.default_rng(seed)
    x = W._round(rng.standard_normal((batch, M, K)).astype(np.float32), dtype)
    w1 = W._round((rng.standard_normal((batch, K, L)) * K ** -0.5).astype(np.float32), dtype)
    w2 = W._round((rng.standard_normal((batch, L, N)) * L ** -0.5).astype(np.float32), dtype)
    return x, w1, w2


def _run(cuda, x, w1, w2, dtype, act, layout="IO", variant="auto", workspace="auto"):
    dx = _dev(x, dtype, cuda)
    if layout == "OI":
        d1, d2 = _dev(w1.transpose(0, 2, 1), dtype, cuda), _dev(w2.transpose(0, 2, 1), dtype, cuda)
    else:
        d1, d2 = _dev(w1, dtype, cuda), _dev(w2, dtype, cuda)
    out = torch.full((x.shape[0], x.shape[1], w2.shape[2]), float("nan"), dtype=TDT[dtype], device=cuda)  # poison
    ops.gemm_relu_gemm(dx, d1, d2, out=out, activation=act, weight_layout=layout, variant=variant, workspace=workspace)
    assert ops.device_status(cuda) == 0
    return out.float().cpu().numpy()


# (batch, M, N, K, L).  Four-CTA kernel: L = 4096 gives eight rounds (every hidden-chunk slot and barrier phase
# wraps several times); row counts that are not multiples of the 128-row block (208 tokens, a 16-row call);
# hidden sizes that are not multiples of four chunks (the last round is partial; with fewer than four chunks
# in all some CTAs own none).
QUAD_SHAPES = ((2, 256, 512, 128, 1024), (1, 512, 1024, 256, 1536), (1, 256, 512, 64, 4096),
               (1, 128, 256, 64, 512), (1, 128, 1024, 192, 512), (3, 384, 768, 960, 2048),
               (2, 208, 768, 768, 1024), (1, 16, 256, 64, 512),
               (1, 256, 512, 128, 768), (2, 128, 256, 64, 128), (1, 384, 1024, 192, 1664))
# CTA-pair kernel (256-row blocks, 256-wide hidden chunks, four chunks a round): one full round; one full and one
# partial round; four rounds (slots and phases wrap); two chunks in all, second CTA of each pair without rows;
# a K that is not a multiple of 64 with 208 rows and three chunks; a single chunk and 16 rows; three
# batch entries with a partial second row block.
PAIR_SHAPES = ((2, 256, 512, 128, 1024), (1, 512, 1024, 256, 1536), (1, 256, 512, 64, 4096),
               (1, 128, 1024, 192, 512), (2, 208, 1024, 80, 768), (1, 16, 512, 64, 256),
               (3, 384, 512, 960, 2048))
# Y widths the 256-wide-chunk kernel covers in both layouts, the pair kernel only with [out, in] weights (K-major W2 tiles)
PAIR_SHAPES_OI = ((1, 256, 768, 128, 1024), (1, 272, 256, 64, 512))


@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
@pytest.mark.parametrize("act", ["relu", "identity"])
@pytest.mark.parametrize("layout", ["IO", "OI"])
@pytest.mark.parametrize("variant", ["quad", "wide", "pair"])
def test_parity_small(cuda, oracle, dtype, act, layout, variant):
    """Every kernel, each forced: four-CTA clusters with single-SM MMAs and 128-wide or 256-wide hidden
    chunks, and eight-CTA clusters of CTA pairs with 2-SM MMAs (no scratch memory here: one cluster per row
    block)."""
    shapes = {"quad": QUAD_SHAPES, "wide": PAIR_SHAPES + PAIR_SHAPES_OI,
              "pair": PAIR_SHAPES + (PAIR_SHAPES_OI if layout == "OI" else ())}[variant]
    for (batch, M, N, K, L) in shapes:
        x, w1, w2 = _inputs(21, batch, M, N, K, L, dtype)
        got = _run(cuda, x, w1, w2, dtype, act, layout, variant, workspace=None)
        want = oracle.gemm_act_gemm(x, w1, w2, 1 if act == "relu" else 0, ODT[dtype], wide=False)
        assert_close(got, want, dtype, f"{dtype} {act} {layout} {variant} {(batch, M, N, K, L)}")


@pytest.mark.parametrize("layout", ["IO", "OI"])
@pytest.mark.parametrize("variant", ["quad", "wide", "pair"])
def test_shared_row_blocks(cuda, oracle, layout, variant):
    """Few row blocks (or a last wave that would leave most of the device idle): some row blocks are shared
    by several clusters, each takes a range of the hidden dimension, and the fp32 partials of Y are combined
    through the caller's scratch memory.  Checked against the oracle, against the run without scratch memory
    (same kernel, one cluster per row block) and for run-to-run identity."""
    lib = _lib.load()
    dtype = "bfloat16"
    split_cases = 0
    for (batch, M, N, K, L) in ((1, 16, 1024, 128, 4096), (1, 256, 1024, 256, 4096), (2, 208, 512, 64, 2048),
                                (1, 2048, 1024, 256, 4096), (1, 4352, 512, 64, 1024)):
        bits = {"pair": _lib.EPILOGUE_PAIR_MMA, "quad": _lib.EPILOGUE_QUAD_MMA, "wide": _lib.EPILOGUE_WIDE_MMA}[variant]
        need = lib.ditto_b200_workspace_bytes(_lib.OP_GEMM_RELU_GEMM | bits, batch, M, N, K, L, _lib.DTYPE_BF16)
        if need == 0:
            continue        # the planner found nothing to gain at this shape on this device
        split_cases += 1
        x, w1, w2 = _inputs(23, batch, M, N, K, L, dtype)
        ws = torch.full((need,), 0xA5, dtype=torch.uint8, device=cuda)   # scratch arrives dirty
        got = _run(cuda, x, w1, w2, dtype, "relu", layout, variant, workspace=ws)
        want = oracle.gemm_act_gemm(x, w1, w2, 1, ODT[dtype], wide=False)
        assert_close(got, want, dtype, f"shared {variant} {layout} {(batch, M, N, K, L)}")
        again = _run(cuda, x, w1, w2, dtype, "relu", layout, variant, workspace=ws)
        assert np.array_equal(got, again), "runs with shared row blocks differ"
        whole = _run(cuda, x, w1, w2, dtype, "relu", layout, variant, workspace=None)
        assert_close(got, whole, dtype, f"shared vs whole {variant} {layout} {(batch, M, N, K, L)}")
        # a workspace that is too small is not an error: the call computes every row block whole
        small = _run(cuda, x, w1, w2, dtype, "relu", layout, variant, workspace=ws[:1024])
        assert np.array_equal(small, whole)
    assert split_cases >= 2, "the planner shared row blocks in fewer cases than expected"


@pytest.mark.parametrize("layout", ["IO", "OI"])
@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
def test_work_loop_many_items(cuda, oracle, dtype, layout):
    """More (batch entry, row block) items than the device holds clusters at once (33 of four CTAs on a B200):
    a cluster walks several items with its rings, slots and barrier phases running on.  Shapes: two hidden
    chunks (two of the four CTAs own none and only write Y), a single chunk, six chunks (partial second
    round) with partial last row blocks in three batch entries and a K that is not a multiple of 64, and
    whole rounds.  Also the general (bias / GELU) form of the loop."""
    lib = _lib.load()
    slots = lib.ditto_b200_mlp_cluster_slots(_lib.DTYPE_BF16, _lib.EPILOGUE_WIDE_MMA)
    assert slots > 0
    for (batch, M, N, K, L) in ((1, 128 * 70, 256, 64, 512), (1, 128 * 40, 768, 128, 256),
                                (3, 128 * 23 + 16, 512, 80, 1536), (2, 4480, 1024, 64, 1024)):
        assert batch * ((M + 127) // 128) > slots, "the shape no longer needs the work loop on this device"
        x, w1, w2 = _inputs(29, batch, M, N, K, L, dtype)
        got = _run(cuda, x, w1, w2, dtype, "relu", layout, "wide", workspace=None)
        want = oracle.gemm_act_gemm(x, w1, w2, 1, ODT[dtype], wide=False)
        assert_close(got, want, dtype, f"work loop {dtype} {layout} {(batch, M, N, K, L)}")
        again = _run(cuda, x, w1, w2, dtype, "relu", layout, "wide", workspace=None)
        assert np.array_equal(got, again), "runs of the work loop differ"
    M, N, K, L = 128 * 40, 256, 64, 768
    x, w1, w2 = _inputs(31, 1, M, N, K, L, dtype)
    rng = np.random.default_rng(32)
    b1 = W._round(rng.standard_normal((1, L)).astype(np.float32) * 0.5, dtype)
    b2 = W._round(rng.standard_normal((1, N)).astype(np.float32) * 0.5, dtype)
    d1, d2 = ((_dev(w1.transpose(0, 2, 1), dtype, cuda), _dev(w2.transpose(0, 2, 1), dtype, cuda)) if layout == "OI"
              else (_dev(w1, dtype, cuda), _dev(w2, dtype, cuda)))
    out = torch.full((1, M, N), float("nan"), dtype=TDT[dtype], device=cuda)
    ops.ffn(_dev(x, dtype, cuda), d1, _dev(b1, dtype, cuda), d2, _dev(b2, dtype, cuda), out=out, act1="gelu", act2="relu",
            weight_layout=layout)
    assert ops.device_status(cuda) == 0
    assert_close(out.float().cpu().numpy(), oracle.ffn(x, w1, b1, w2, b2, 2, 1, ODT[dtype]), dtype, f"work loop ffn {dtype} {layout}")


@pytest.mark.parametrize("layout", ["IO", "OI"])
def test_results_wider_than_1024_columns(cuda, oracle, layout):
    """N above 1024 (any multiple of 256): the result is computed in column groups of at most 1024, one
    launch each -- 2048 = 1024 + 1024, 1280 = 768 + 512, 3072 = 3 x 1024 -- with and without scratch memory for
    shared row blocks, and with biases (the second one is offset per group) in the feed-forward form."""
    dtype = "bfloat16"
    for (batch, M, N, K, L) in ((1, 256, 2048, 64, 512), (2, 208, 1280, 80, 768), (1, 128, 3072, 128, 256),
                                (1, 128 * 36, 1536, 64, 512)):
        x, w1, w2 = _inputs(37, batch, M, N, K, L, dtype)
        want = oracle.gemm_act_gemm(x, w1, w2, 1, ODT[dtype], wide=False)
        for ws in (None, "auto"):
            got = _run(cuda, x, w1, w2, dtype, "relu", layout, "auto", workspace=ws)
            assert_close(got, want, dtype, f"wide N {layout} ws={ws} {(batch, M, N, K, L)}")
    M, N, K, L = 384, 2048, 64, 512
    x, w1, w2 = _inputs(38, 1, M, N, K, L, dtype)
    rng = np.random.default_rng(39)
    b1 = W._round(rng.standard_normal((1, L)).astype(np.float32) * 0.5, dtype)
    b2 = W._round(rng.standard_normal((1, N)).astype(np.float32) * 0.5, dtype)
    d1, d2 = ((_dev(w1.transpose(0, 2, 1), dtype, cuda), _dev(w2.transpose(0, 2, 1), dtype, cuda)) if layout == "OI"
              else (_dev(w1, dtype, cuda), _dev(w2, dtype, cuda)))
    out = torch.full((1, M, N), float("nan"), dtype=TDT[dtype], device=cuda)
    ops.ffn(_dev(x, dtype, cuda), d1, _dev(b1, dtype, cuda), d2, _dev(b2, dtype, cuda), out=out, act1="relu", act2="relu",
            weight_layout=layout)
    assert ops.device_status(cuda) == 0
    assert_close(out.float().cpu().numpy(), oracle.ffn(x, w1, b1, w2, b2, 1, 1, ODT[dtype]), dtype, f"wide N ffn {layout}")


@pytest.mark.parametrize("layout", ["IO", "OI"])
@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
def test_hidden_sizes_with_a_partial_last_chunk(cuda, oracle, dtype, layout):
    """Hidden sizes that are multiples of 64 but not of the 256-wide chunk: the last chunk reaches past L (W1
    columns / W2 rows beyond it are zero-filled on load, the bias is not read there).  64 and 192: a single
    partial chunk; 320, 448, 1088: full chunks and a partial one, in the first or a later round; with and
    without bias / GELU, and inside the work loop (more row blocks than cluster places)."""
    for (batch, M, N, K, L) in ((1, 128, 256, 64, 64), (2, 208, 512, 80, 192), (1, 256, 1024, 128, 320),
                                (1, 384, 256, 64, 448), (1, 128, 512, 64, 1088), (1, 128 * 36, 256, 64, 320)):
        x, w1, w2 = _inputs(41, batch, M, N, K, L, dtype)
        got = _run(cuda, x, w1, w2, dtype, "relu", layout, "auto", workspace=None)
        want = oracle.gemm_act_gemm(x, w1, w2, 1, ODT[dtype], wide=False)
        assert_close(got, want, dtype, f"partial chunk {dtype} {layout} {(batch, M, N, K, L)}")
    for (M, N, K, L, acts) in ((256, 256, 64, 320, ("gelu", "relu")), (128, 512, 128, 192, ("relu", "identity"))):
        x, w1, w2 = _inputs(42, 1, M, N, K, L, dtype)
        rng = np.random.default_rng(43)
        b1 = W._round(rng.standard_normal((1, L)).astype(np.float32) * 0.5, dtype)
        b2 = W._round(rng.standard_normal((1, N)).astype(np.float32) * 0.5, dtype)
        d1, d2 = ((_dev(w1.transpose(0, 2, 1), dtype, cuda), _dev(w2.transpose(0, 2, 1), dtype, cuda)) if layout == "OI"
                  else (_dev(w1, dtype, cuda), _dev(w2, dtype, cuda)))
        out = torch.full((1, M, N), float("nan"), dtype=TDT[dtype], device=cuda)
        # the bias vector sits at the end of an allocation poisoned behind it: a read past L would show
        pad = torch.full((L + 512,), float("nan"), dtype=TDT[dtype], device=cuda)
        pad[:L] = _dev(b1, dtype, cuda).view(-1)
        ops.ffn(_dev(x, dtype, cuda), d1, pad[:L].view(1, L), d2, _dev(b2, dtype, cuda), out=out, act1=acts[0], act2=acts[1],
                weight_layout=layout)
        assert ops.device_status(cuda) == 0
        code = {"identity": 0, "relu": 1, "gelu": 2}
        assert_close(out.float().cpu().numpy(), oracle.ffn(x, w1, b1, w2, b2, code[acts[0]], code[acts[1]], ODT[dtype]), dtype,
                     f"partial chunk ffn {dtype} {layout} {(M, N, K, L)}")


def test_golden_vector(cuda):
    case = "mlp_bf16_relu"
    w = make_golden.workload(case)
    A, B, C = make_golden.inputs(case)
    out = ops.gemm_relu_gemm(_dev(A, w.dtype, cuda), _dev(B, w.dtype, cuda), _dev(C, w.dtype, cuda), activation="relu")
    assert ops.device_status(cuda) == 0
    stored = np.load(os.path.join(GOLDEN, case + ".npz"))
    assert_close(out.float().cpu().numpy(), stored["chain_fp32"], w.dtype, case)


def test_cfg4_sampled_row_blocks(cuda, oracle):
    """Benchmark configuration 4 at full size (X[16384,1024], W1[1024,4096], W2[4096,1024], bf16): seeded
    row blocks (first, last and the shard boundaries of 2/4/8 GPUs) are placed at their index, the
    rest of X is unrelated random data, and those blocks are compared with the oracle."""
    w = W.WORKLOADS["cfg4"]
    w1, w2 = W.mlp_weights(w)
    g = torch.Generator(device=cuda).manual_seed(3)
    x = torch.randn(w.M, w.K, device=cuda, generator=g).bfloat16()
    blocks = (0, 15, 16, 63, 64, 127)
    rows = {}
    for blk in blocks:
        r = W.mlp_rows(w, blk)
        x[blk * 128:(blk + 1) * 128] = torch.from_numpy(r).to(cuda).bfloat16()
        rows[blk] = r
    out = ops.gemm_relu_gemm(x, _dev(w1, w.dtype, cuda), _dev(w2, w.dtype, cuda), activation="relu")
    assert ops.device_status(cuda) == 0
    assert torch.isfinite(out.float()).all()
    for blk, r in rows.items():
        want = oracle.gemm_act_gemm(r[None], w1[None], w2[None], 1, oracle.BF16, wide=False)[0]
        assert_close(out[blk * 128:(blk + 1) * 128].float().cpu().numpy(), want, w.dtype, f"cfg4 row block {blk}")


def test_full_size_properties(cuda):
    """Size-independent checks at config-4 size: rows are independent (permuting row blocks
    permutes the result), the identity chain is linear in X, ReLU of a non-negative hidden layer
    equals the identity chain, and repeated launches are bitwise identical."""
    w = W.WORKLOADS["cfg4"]
    g = torch.Generator(device=cuda).manual_seed(4)
    x = torch.randn(w.M, w.K, device=cuda, generator=g).bfloat16()
    w1 = (torch.randn(w.K, w.L, device=cuda, generator=g) * w.K ** -0.5).bfloat16()
    w2 = (torch.randn(w.L, w.N, device=cuda, generator=g) * w.L ** -0.5).bfloat16()
    base = ops.gemm_relu_gemm(x, w1, w2, activation="relu")
    assert torch.equal(base, ops.gemm_relu_gemm(x, w1, w2, activation="relu"))
    perm = torch.randperm(w.M // 128, device=cuda, generator=g)
    xp = x.view(-1, 128, w.K)[perm].reshape(w.M, w.K).contiguous()
    # Bit for bit where every row block is computed the same way (no scratch memory: one cluster per row block).
    # With scratch memory the last row blocks may be shared by several clusters, whose fp32 partials are added in a
    # different order than one accumulator adds them: there the permuted result agrees to rounding only.
    whole = ops.gemm_relu_gemm(x, w1, w2, activation="relu", workspace=None)
    assert torch.equal(ops.gemm_relu_gemm(xp, w1, w2, activation="relu", workspace=None),
                       whole.view(-1, 128, w.N)[perm].reshape(w.M, w.N))
    moved = ops.gemm_relu_gemm(xp, w1, w2, activation="relu").float()
    want = base.view(-1, 128, w.N)[perm].reshape(w.M, w.N).float()
    assert (moved - want).abs().max().item() <= 2e-2 * want.abs().max().item()
    lin = ops.gemm_relu_gemm((2 * x).bfloat16(), w1, w2, activation="identity").float()
    one = ops.gemm_relu_gemm(x, w1, w2, activation="identity").float()
    assert (lin - 2 * one).abs().max().item() <= 2e-2 * one.abs().max().item()
    pos = ops.gemm_relu_gemm(x.abs(), w1.abs(), w2, activation="relu")
    assert torch.equal(pos, ops.gemm_relu_gemm(x.abs(), w1.abs(), w2, activation="identity"))
    assert ops.device_status(cuda) == 0


def test_unsupported_shapes_raise(cuda):
    x = torch.zeros(128, 64, dtype=torch.bfloat16, device=cuda)
    w1 = torch.zeros(64, 208, dtype=torch.bfloat16, device=cuda)   # hidden 208 is not a multiple of 64
    w2 = torch.zeros(208, 256, dtype=torch.bfloat16, device=cuda)
    with pytest.raises(_lib.DittoError) as e:
        ops.gemm_relu_gemm(x, w1, w2)
    assert e.value.code == _lib.ERR_UNSUPPORTED


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
@pytest.mark.parametrize("act", ["relu", "identity"])
@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("layout", ["IO", "OI"])
def test_small_n_chains(cuda, oracle, dtype, act, d, layout):
    """N = K in {64, 128}: the reference's own shape family (benchmark/chimera/cuda/bmm_bmm_cuda.py
    shapes table, python_test/auto_tensorize/test_hyper_fusion_cpu.py) -- batched, per-slice weights, as
    [in, out] (the reference's chain operands) and as [out, in] (its linear layers' weights)."""
    for (batch, M, L) in ((2, 128, 128), (3, 256, 384), (8, 512, 512), (2, 208, 272), (1, 516 // 4 * 4 // 16 * 16 + 16, 512)):
        rng = np.random.default_rng(31)
        a = W._round(rng.uniform(-1, 1, (batch, M, d)).astype(np.float32), dtype)
        b = W._round(rng.uniform(-1, 1, (batch, d, L)).astype(np.float32), dtype)
        c = W._round(rng.uniform(-1, 1, (batch, L, d)).astype(np.float32), dtype)
        got = _run(cuda, a, b, c, dtype, act, layout)
        want = oracle.gemm_act_gemm(a, b, c, 1 if act == "relu" else 0, ODT[dtype], wide=False)
        # |result| grows like sqrt(K L) for U(-1,1) operands: scale the absolute floor with it
        assert_close(got, want, dtype, f"{dtype} {act} d={d} {layout} {(batch, M, L)}", scale=float(np.abs(want).max()))


@pytest.mark.parametrize("act", ["relu", "identity"])
@pytest.mark.parametrize("layout", ["IO", "OI"])
def test_small_n_chains_with_different_widths(cuda, oracle, act, layout):
    """N != K, both <= 128: (A B) C with A [M, K], B [K, L], C [L, N] on the attention kernel's chain mode."""
    dtype = "float16"
    for (batch, M, N, K, L) in ((2, 256, 128, 64, 256), (3, 208, 64, 128, 272), (1, 128, 48, 80, 144), (2, 384, 32, 64, 1040)):
        rng = np.random.default_rng(33)
        a = W._round(rng.uniform(-1, 1, (batch, M, K)).astype(np.float32), dtype)
        b = W._round(rng.uniform(-1, 1, (batch, K, L)).astype(np.float32), dtype)
        c = W._round(rng.uniform(-1, 1, (batch, L, N)).astype(np.float32), dtype)
        got = _run(cuda, a, b, c, dtype, act, layout)
        want = oracle.gemm_act_gemm(a, b, c, 1 if act == "relu" else 0, ODT[dtype], wide=False)
        assert_close(got, want, dtype, f"{act} {layout} N != K {(batch, M, N, K, L)}", scale=float(np.abs(want).max()))


def test_small_n_golden_and_cfg1_shape(cuda, oracle):
    case = "chain_fp16_identity"
    w = make_golden.workload(case)
    A, B, C = make_golden.inputs(case)
    out = ops.gemm_relu_gemm(_dev(A, w.dtype, cuda), _dev(B, w.dtype, cuda), _dev(C, w.dtype, cuda), activation="identity")
    assert ops.device_status(cuda) == 0
    stored = np.load(os.path.join(GOLDEN, case + ".npz"))["chain_fp32"]
    assert_close(out.float().cpu().numpy(), stored, w.dtype, case, scale=float(np.abs(stored).max()))
    # benchmark configuration 1's shape (A[8,512,64] B[8,64,512] D[8,512,64], U(-1,1)) in fp16 on the GPU; the
    # fp32 CPU case itself is checked in tests/test_oracle.py
    cfg1 = W.WORKLOADS["cfg1"]
    a, b, c = (W._round(t, "float16") for t in W.chain_inputs(cfg1))
    got = _run(cuda, a, b, c, "float16", "identity", "IO")
    want = oracle.gemm_act_gemm(a, b, c, 0, oracle.FP16, wide=False)
    assert_close(got, want, "float16", "cfg1 shape fp16", scale=float(np.abs(want).max()))


@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
@pytest.mark.parametrize("acts", [("relu", "relu"), ("gelu", "identity"), ("identity", "gelu")])
@pytest.mark.parametrize("layout", ["OI", "IO"])
def test_ffn_with_bias(cuda, oracle, dtype, acts, layout):
    """The reference's feed-forward block: linear (+ bias, [out, in] weights) -> ReLU -> linear -> ReLU
    (nn/model/transformer.py:21-34), plus its GELU (nn/functional/activation.py:29-39)."""
    code = {"identity": 0, "relu": 1, "gelu": 2}
    for (M, N, K, L) in ((128, 256, 64, 512), (256, 1024, 128, 1024)):
        x, w1, w2 = _inputs(51, 1, M, N, K, L, dtype)
        rng = np.random.default_rng(52)
        b1 = W._round(rng.standard_normal((1, L)).astype(np.float32) * 0.5, dtype)
        b2 = W._round(rng.standard_normal((1, N)).astype(np.float32) * 0.5, dtype)
        if layout == "OI":
            d1, d2 = _dev(w1.transpose(0, 2, 1), dtype, cuda), _dev(w2.transpose(0, 2, 1), dtype, cuda)
        else:
            d1, d2 = _dev(w1, dtype, cuda), _dev(w2, dtype, cuda)
        out = torch.full((1, M, N), float("nan"), dtype=TDT[dtype], device=cuda)
        ops.ffn(_dev(x, dtype, cuda), d1, _dev(b1, dtype, cuda), d2, _dev(b2, dtype, cuda), out=out, act1=acts[0],
                act2=acts[1], weight_layout=layout)
        assert ops.device_status(cuda) == 0
        want = oracle.ffn(x, w1, b1, w2, b2, code[acts[0]], code[acts[1]], ODT[dtype])
        assert_close(out.float().cpu().numpy(), want, dtype, f"ffn {dtype} {acts} {layout} {(M, N, K, L)}")
        # no bias, ReLU then identity == the plain chain entry point, bit for bit
        if acts == ("relu", "relu"):
            a = ops.ffn(_dev(x, dtype, cuda), d1, None, d2, None, act1="relu", act2="identity", weight_layout=layout)
            bq = ops.gemm_relu_gemm(_dev(x, dtype, cuda), d1, d2, activation="relu", weight_layout=layout,
                                    workspace=None)   # like ffn: no scratch memory, one cluster per row block
            assert torch.equal(a, bq)
