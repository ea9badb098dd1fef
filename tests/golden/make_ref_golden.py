"""Write ref_microkernels.npz: outputs of the REFERENCE'S OWN CPU micro-kernels on seeded inputs.

    python -m tests.golden.make_ref_golden        (needs the reference tree; run in the development container)

oracle/build_ref.py compiles the 6 x 16 AVX2 GEMM micro-kernel and the AVX-512 exponential that the
reference generates (python/ditto/auto_tensorize/intrinsic.py:274-604, 1480-1672);
oracle/ref_microkernels.py evaluates the reference's three CPU chains tile by tile through them.
The vectors written here are those results, so tests/test_oracle.py can hold the C restatement
(oracle/chain_oracle.c) to the reference's own arithmetic on machines where the reference tree is
absent.  Inputs are stored with the outputs (the cases are small).
"""
import os

import numpy as np

from oracle import ref_microkernels as R

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "ref_microkernels.npz")

# (batch, M, N, K, L): M need not be a multiple of the 6-row tile (the reference pads, bmm_bmm_cpu.py:294)
CHAIN_SHAPES = ((2, 20, 32, 64, 48), (1, 96, 64, 64, 128), (3, 6, 16, 16, 16))
# feed-forward block (rows, d_model, d_ff): linear + bias -> ReLU -> linear + bias -> ReLU, weights [out, in]
FFN_SHAPES = ((20, 32, 64), (96, 64, 128))


def exp_inputs():
    rng = np.random.default_rng(77)
    edge = np.array([0.0, -0.0, 1.0, -1.0, 0.5, -0.5, 88.0, 88.3762626647949, 89.0, 1e4, -87.0, -88.3762626647949,
                     -89.0, -1e4, 0.34657359, 0.3465736, -0.34657359, 1e-8, -1e-8, 0.6931472, 10.0, -10.0], dtype=np.float32)
    edge = np.resize(edge, 32)
    return np.concatenate([edge.reshape(1, 32), rng.uniform(-90, 90, (16, 32)), rng.normal(0, 8, (16, 32)),
                           rng.uniform(-1, 1, (15, 32))]).astype(np.float32)


def chain_inputs(shape, seed):
    batch, M, N, K, L = shape
    rng = np.random.default_rng(seed)
    a = rng.uniform(-1, 1, (batch, M, K)).astype(np.float32)
    b = rng.uniform(-1, 1, (batch, K, L)).astype(np.float32)
    c = rng.uniform(-1, 1, (batch, L, N)).astype(np.float32)
    return a, b, c


def main():
    if not R.available() or not R.has_exp():
        raise SystemExit("the reference micro-kernels could not be built here (reference tree or AVX-512 missing)")
    out = {}
    x = exp_inputs()
    out["exp_x"] = x
    out["exp_y"] = R.exp(x)
    for i, shape in enumerate(CHAIN_SHAPES):
        a, b, c = chain_inputs(shape, 500 + i)
        out[f"c{i}_shape"] = np.array(shape, dtype=np.int32)
        out[f"c{i}_a"], out[f"c{i}_b"], out[f"c{i}_c"] = a, b, c
        out[f"c{i}_bmm_bmm"] = R.bmm_bmm(a, b, c)
        out[f"c{i}_bmm_relu_bmm"] = R.bmm_relu_bmm(a, b, c)
        # unscaled U(-1,1) logits reach +-25 at K = 64: well inside the fp32 range of exp, as in the reference's runs
        out[f"c{i}_bmm_softmax_bmm"] = R.bmm_softmax_bmm_cpu(a, b, c)
        # the same with the reduction split into 16-wide chunks (KI1 = KI2 = 16): identical by construction
        assert np.array_equal(out[f"c{i}_bmm_bmm"], R.bmm_bmm(a, b, c, 16, 16))
    for i, (rows, d_model, d_ff) in enumerate(FFN_SHAPES):
        rng = np.random.default_rng(600 + i)
        x = rng.standard_normal((rows, d_model)).astype(np.float32)
        w1 = (rng.standard_normal((d_ff, d_model)) * d_model ** -0.5).astype(np.float32)
        b1 = (rng.standard_normal(d_ff) * 0.5).astype(np.float32)
        w2 = (rng.standard_normal((d_model, d_ff)) * d_ff ** -0.5).astype(np.float32)
        b2 = (rng.standard_normal(d_model) * 0.5).astype(np.float32)
        out[f"f{i}_x"], out[f"f{i}_w1"], out[f"f{i}_b1"], out[f"f{i}_w2"], out[f"f{i}_b2"] = x, w1, b1, w2, b2
        out[f"f{i}_relu_relu"] = R.ffn(x, w1, b1, w2, b2, True, True)
        out[f"f{i}_relu_identity"] = R.ffn(x, w1, b1, w2, b2, True, False)
        out[f"f{i}_identity_identity_nobias"] = R.ffn(x, w1, None, w2, None, False, False)
    np.savez_compressed(OUT, **out)
    print("wrote", OUT, os.path.getsize(OUT), "bytes")


if __name__ == "__main__":
    main()
