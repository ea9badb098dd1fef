"""GPU tests of the callers around the kernels: the packed multi-head attention layer and the
GraphEngine (plain and CUDA-graph) that launches compiled layers."""
import numpy as np
import pytest
import torch

import ditto_b200 as ditto
from ditto_b200 import auto_compute as ac, auto_tensorize as at, hardware as hw, ops, runtime
from ditto_b200 import workloads as W
from ditto_b200 import _lib
from tests.tolerances import assert_close

pytestmark = pytest.mark.gpu


def _mha_reference(oracle, qkv, heads, dtype_code, scale):
    """Head split / merge exactly as nn/module/self_attention.py:46-73 does it, then the CPU oracle."""
    batch, M, k3 = qkv.shape
    hidden = k3 // 3
    d = hidden // heads
    q, k, v = qkv[:, :, :hidden], qkv[:, :, hidden:2 * hidden], qkv[:, :, 2 * hidden:]
    fold = lambda t: t.reshape(batch, M, heads, d).transpose(0, 2, 1, 3).reshape(batch * heads, M, d)
    kt = q.reshape(batch, M, heads, d)  # placeholder to keep shapes obvious
    kt = k.reshape(batch, M, heads, d).transpose(0, 2, 3, 1).reshape(batch * heads, d, M)
    o = oracle.bmm_softmax_bmm(fold(q), np.ascontiguousarray(kt), fold(v), scale, dtype_code, wide=False)
    return o.reshape(batch, heads, M, d).transpose(0, 2, 1, 3).reshape(batch, M, hidden)


@pytest.mark.parametrize("dtype,heads,d,M", [("float16", 12, 64, 256), ("bfloat16", 4, 128, 256), ("float16", 3, 64, 256),
                                             ("float16", 16, 80, 208), ("bfloat16", 5, 48, 400)])
def test_packed_multi_head_attention(cuda, oracle, dtype, heads, d, M):
    """Includes ViT-Huge/16 (16 heads of 80, 196 -> 208 tokens): ragged rows and a head dimension that
    is not a tile size, read straight out of the packed tensor."""
    tdt = {"float16": torch.float16, "bfloat16": torch.bfloat16}[dtype]
    batch = 2
    rng = np.random.default_rng(41)
    qkv = W._round((rng.standard_normal((batch, M, 3 * heads * d)) * 0.5).astype(np.float32), dtype)
    dq = torch.from_numpy(qkv).to(cuda).to(tdt)
    out = torch.full((batch, M, heads * d), float("nan"), dtype=tdt, device=cuda)
    ops.multi_head_attention(dq, heads, out=out, scale=1.0)
    assert ops.device_status(cuda) == 0
    want = _mha_reference(oracle, qkv, heads, 0 if dtype == "float16" else 1, 1.0)
    assert_close(out.float().cpu().numpy(), want, dtype, f"mha {dtype} h={heads} d={d}")
    # and against the unfused route: torch views + the batched kernel
    hidden = heads * d
    fold = lambda t: t.reshape(batch, M, heads, d).permute(0, 2, 1, 3).reshape(batch * heads, M, d).contiguous()
    q, k, v = dq[..., :hidden], dq[..., hidden:2 * hidden], dq[..., 2 * hidden:]
    o2 = ops.bmm_softmax_bmm(fold(q), fold(k), fold(v), scale=1.0, key_layout="LK")
    o2 = o2.reshape(batch, heads, M, d).permute(0, 2, 1, 3).reshape(batch, M, hidden)
    assert torch.equal(o2, out)


def _mha_graph():
    mha = ac.nn.module.MultiHeadAttentionMMA(12, 768, in_dtype="float16")
    x = ac.layer_tensor([4, 512, 3 * 768], name="qkv", dtype="float16")
    y = mha(x)
    return ac.graph([x], [y]), x, y


@pytest.mark.parametrize("factory", [runtime.create_graph_engine, runtime.create_cuda_graph_engine])
def test_graph_engine_runs_the_attention_layer(cuda, oracle, factory):
    """The reference's engine protocol: create_graph_engine(graph, built_mods, dev) then
    get_function("init" / "set_inputs" / "compile" / "run" / "timeit" / "get_outputs")
    (benchmark/chimera/cuda/bert_inference.py:114-129)."""
    g, x, y = _mha_graph()
    layer = y.layer
    built = {layer.fingerprint: ditto.build(at.tensorize_cuda(layer, None, hw.query_hw_param("gpu.cuda.B200")),
                                           layer.schedule_tensors, "cuda")}
    engine = factory(g, built, "cuda")
    engine.get_function("init")()
    rng = np.random.default_rng(43)
    qkv = W._round((rng.standard_normal((4, 512, 2304)) * 0.5).astype(np.float32), "float16")
    engine.get_function("set_inputs")(torch.from_numpy(qkv))
    engine.get_function("compile")()
    engine.get_function("run")()
    (out,) = engine.get_function("get_outputs")()
    assert ops.device_status(cuda) == 0
    want = _mha_reference(oracle, qkv, 12, 0, 1.0)
    assert_close(out.float().cpu().numpy(), want, "float16", "graph engine")
    ms = engine.get_function("timeit")(20)
    assert 0 < ms < 5
    with pytest.raises(AttributeError):
        engine.get_function("no_such_function")


def test_expired_wait_is_reported_not_fatal(cuda):
    """The failure path of the device-side waits, exercised without faulting anything: a CTA waits (with the
    bounded wait all kernels share) on a barrier nobody signals; at the limit the wait gives up, the code
    lands in the status word, the kernel ends normally -- and the context keeps working: the next fused
    call on the same device is correct and leaves the status word clean."""
    lib = _lib.load()
    status = torch.zeros(1, dtype=torch.int32, device=cuda)
    with torch.cuda.device(cuda):
        rc = lib.ditto_b200_selftest_wait_limit(0x6A1, status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize(cuda)
    assert int(status.item()) == 0x6A1
    assert lib.ditto_b200_selftest_wait_limit(0, status.data_ptr(), None) == _lib.ERR_INVALID_ARG
    q = (torch.rand(2, 256, 64, device=cuda) - 0.5).half()
    out = ops.bmm_softmax_bmm(q, q, q, scale=1.0, key_layout="LK")
    assert ops.device_status(cuda) == 0
    ref = torch.softmax(q.float() @ q.float().transpose(1, 2), -1) @ q.float()
    assert (out.float() - ref).abs().max().item() < 2e-3
