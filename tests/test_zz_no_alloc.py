"""The MLP chain through the entry point that allocates nothing (ditto_b200_gemm_relu_gemm_static_scratch).

Who needs it: a caller that cannot give the library scratch memory because it cannot allocate any -- code
running under stream capture or in a callback where cudaMalloc is off limits, a plugin that is handed input
and output buffers and nothing else, a service whose memory budget was fixed at start-up.  For them the
scratch memory is an array inside the library image (12 MiB per GPU).  This test calls the entry point
through the C ABI exactly as such a caller would -- caller-owned inputs and outputs only -- twice in a row on
shapes where row blocks are shared between clusters (so the scratch array is really used and reused), and
checks the output against the regular entry point run with a workspace the test allocates itself.

The file sorts last on purpose: if this additional entry point ever breaks, a run that stops at the first
failure has already gone through every other test.
"""
import numpy as np
import pytest
import torch

from ditto_b200 import _lib, ops
from ditto_b200 import workloads as W
from tests.tolerances import assert_close

pytestmark = pytest.mark.gpu

STATIC_SCRATCH_BYTES = 12 << 20


def _inputs(seed, batch, M, N, K, L):
    rng = np.random.default_rng(seed)
    x = W._round(rng.standard_normal((batch, M, K)).astype(np.float32), "bfloat16")
    w1 = W._round((rng.standard_normal((batch, K, L)) * K ** -0.5).astype(np.float32), "bfloat16")
    w2 = W._round((rng.standard_normal((batch, L, N)) * L ** -0.5).astype(np.float32), "bfloat16")
    return x, w1, w2


def _call_static(lib, cuda, dx, d1, d2, out, batch, M, N, K, L, relu=1):
    with torch.cuda.device(cuda):
        return lib.ditto_b200_gemm_relu_gemm_static_scratch(
            dx.data_ptr(), d1.data_ptr(), d2.data_ptr(), out.data_ptr(), batch, M, N, K, L, _lib.DTYPE_BF16, 0, relu,
            ops._status_ptr(torch.device(cuda)), torch.cuda.current_stream().cuda_stream)


def test_static_scratch_matches_the_workspace_entry_point(cuda, oracle):
    lib = _lib.load()
    used_scratch = 0
    for (batch, M, N, K, L) in ((1, 256, 1024, 256, 4096), (2, 208, 512, 64, 2048), (1, 16, 256, 128, 1024),
                                (1, 384, 768, 192, 512)):
        need = lib.ditto_b200_workspace_bytes(_lib.OP_GEMM_RELU_GEMM | _lib.EPILOGUE_QUAD_MMA, batch, M, N, K, L,
                                              _lib.DTYPE_BF16)
        assert need <= STATIC_SCRATCH_BYTES
        used_scratch += need > 0
        x, w1, w2 = _inputs(61, batch, M, N, K, L)
        dx, d1, d2 = (torch.from_numpy(t).to(cuda).bfloat16() for t in (x, w1, w2))
        # the regular entry point, same kernel, scratch memory allocated by the caller (this test)
        ws = torch.empty(max(need, 1), dtype=torch.uint8, device=cuda)
        want_gpu = ops.gemm_relu_gemm(dx, d1, d2, activation="relu", variant="quad", workspace=ws)
        assert ops.device_status(cuda) == 0
        want_cpu = oracle.gemm_act_gemm(x, w1, w2, 1, oracle.BF16, wide=False)
        for attempt in range(2):                 # the second call finds the array as the first one left it
            out = torch.full((batch, M, N), float("nan"), dtype=torch.bfloat16, device=cuda)   # poison
            rc = _call_static(lib, cuda, dx, d1, d2, out, batch, M, N, K, L)
            assert rc == _lib.OK, lib.ditto_b200_strerror(rc)
            assert ops.device_status(cuda) == 0
            got = out.float().cpu().numpy()
            assert_close(got, want_gpu.float().cpu().numpy(), "bfloat16", f"static scratch vs workspace, call {attempt}")
            assert torch.equal(out, want_gpu)    # same kernel, same plan: in fact bit for bit
            assert_close(got, want_cpu, "bfloat16", f"static scratch vs oracle, call {attempt}")
    assert used_scratch >= 2, "the shapes above were meant to exercise the scratch array"


def test_static_scratch_rejects_what_does_not_fit(cuda):
    lib = _lib.load()
    for (batch, M, N, K, L) in ((1, 1024, 1024, 64, 4096), (1, 2048, 1024, 64, 4096), (2, 1024, 1024, 64, 4096)):
        need = lib.ditto_b200_workspace_bytes(_lib.OP_GEMM_RELU_GEMM | _lib.EPILOGUE_QUAD_MMA, batch, M, N, K, L,
                                              _lib.DTYPE_BF16)
        x = torch.zeros(batch, M, K, dtype=torch.bfloat16, device=cuda)
        w1 = torch.zeros(batch, K, L, dtype=torch.bfloat16, device=cuda)
        w2 = torch.zeros(batch, L, N, dtype=torch.bfloat16, device=cuda)
        out = torch.full((batch, M, N), 7.0, dtype=torch.bfloat16, device=cuda)
        rc = _call_static(lib, cuda, x, w1, w2, out, batch, M, N, K, L)
        if need > STATIC_SCRATCH_BYTES:
            assert rc == _lib.ERR_WORKSPACE
            assert b"scratch" in lib.ditto_b200_last_cuda_error()
            torch.cuda.synchronize(cuda)
            assert bool((out == 7.0).all())      # nothing was launched
        else:
            assert rc == _lib.OK
            assert ops.device_status(cuda) == 0 and bool((out == 0).all())
    # argument errors are reported like everywhere else
    assert lib.ditto_b200_gemm_relu_gemm_static_scratch(None, None, None, None, 1, 128, 256, 64, 512, 1, 0, 1, None, None) \
        == _lib.ERR_INVALID_ARG
