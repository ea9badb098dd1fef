"""Parity tolerances of the GPU kernels against the fp32 CPU oracle.

|gpu - oracle| <= rtol * |oracle| + atol, element-wise.  fp16: the 2e-2 relative bound the task
states, with a 1e-3 absolute floor for outputs near zero.  bf16 (8-bit mantissa, unit round-off
2^-9 on both the probabilities and the output): 3e-2 relative, 4e-3 absolute.
"""
import numpy as np

RTOL = {"float16": 2e-2, "bfloat16": 3e-2}
ATOL = {"float16": 1e-3, "bfloat16": 4e-3}


def assert_close(got, want, dtype, what="", scale=1.0):
    got = np.asarray(got, dtype=np.float32)
    want = np.asarray(want, dtype=np.float32)
    assert got.shape == want.shape, (got.shape, want.shape)
    assert np.isfinite(got).all(), f"{what}: non-finite values in the GPU result"
    err = np.abs(got - want)
    bound = RTOL[dtype] * np.abs(want) + ATOL[dtype] * scale
    worst = np.unravel_index(np.argmax(err - bound), err.shape)
    assert (err <= bound).all(), (
        f"{what}: max abs err {err.max():.3e}, worst at {worst}: got {got[worst]:.6f} want {want[worst]:.6f} "
        f"(rtol {RTOL[dtype]}, atol {ATOL[dtype] * scale})")
    return float(err.max()), float((err / (np.abs(want) + ATOL[dtype] * scale)).max())
