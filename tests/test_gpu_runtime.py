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
    # the same report through the C ABI's helper: DITTO_ERR_TIMEOUT with the code, and the word is cleared
    import ctypes
    with torch.cuda.device(cuda):
        stream = torch.cuda.current_stream().cuda_stream
        status.zero_()                  # the word keeps the first code it was given until somebody clears it
        assert lib.ditto_b200_selftest_wait_limit(0x6A2, status.data_ptr(), stream) == 0
        code = ctypes.c_int(0)
        assert lib.ditto_b200_check_status(status.data_ptr(), stream, ctypes.byref(code)) == _lib.ERR_TIMEOUT
        assert code.value == 0x6A2 and int(status.item()) == 0
        assert lib.ditto_b200_check_status(status.data_ptr(), stream, None) == _lib.OK
    q = (torch.rand(2, 256, 64, device=cuda) - 0.5).half()
    out = ops.bmm_softmax_bmm(q, q, q, scale=1.0, key_layout="LK")
    assert ops.device_status(cuda) == 0
    ref = torch.softmax(q.float() @ q.float().transpose(1, 2), -1) @ q.float()
    assert (out.float() - ref).abs().max().item() < 2e-3


def _chain_module(kind, b, M, N, K, L):
    """The reference's call sequence from chain definition to built module (bmm_softmax_bmm_cuda.py:158-261)."""
    build = ac.nn.functional.BatchGemmSoftmaxGemm if kind == "softmax" else ac.nn.functional.BatchGemmGemm
    ins, outs = build(b, M, N, K, L, "float16", "float32")
    F = outs[0]
    E_frag = F.op.input_tensors[0]
    mid, _ = E_frag.op.input_tensors
    D_frag = mid.op.input_tensors[0]
    bb, m, n, mi, ni = E_frag.op.axis
    rlo, rli = E_frag.op.reduce_axis
    fc = at.fusion_choice(D_frag.op, E_frag.op, [bb, m, n, rlo, mi, ni, rli], 3)
    p1, p2 = at.cuda_wmma(scope="shared"), at.cuda_wmma(scope="global")
    c1 = at.intrinsic_match(D_frag, p1, ["InnerMost", "SameRange"])[0]
    c2 = at.intrinsic_match(E_frag, p2, ["InnerMost", "SameRange"])[0]
    layer = ac.layer([F.op], inputs=ins)
    st = at.tensorize_hyper_fusion_state(layer, fc, {D_frag.op: at.match_info(c1, p1), E_frag.op: at.match_info(c2, p2)})
    sch = at.tensorize_cuda(layer, st, hw.query_hw_param("gpu.cuda.B200"), at.cuda_tensorize_param())
    return ditto.build(sch, layer.schedule_tensors, "cuda")


def test_repeated_calls_take_the_prepared_path_and_stay_checked(cuda):
    """`func(*inputs, *outputs)` with the same tensor objects as the previous call skips re-validation
    (the reference's benchmark loop, an engine with pre-allocated buffers); results are identical, new
    contents of the same buffers are picked up, and different tensors are validated again."""
    for kind in ("softmax", "identity"):
        b, M, N, K, L = 3, 256, 64, 64, 256
        func = _chain_module(kind, b, M, N, K, L)
        g = torch.Generator(device=cuda).manual_seed(3)
        a = (torch.rand(b, M, K, device=cuda, generator=g) - 0.5).half()
        bm = (torch.rand(b, K, L, device=cuda, generator=g) - 0.5).half()
        c = (torch.rand(b, L, N, device=cuda, generator=g) - 0.5).half()
        f = torch.full((b, M, N), float("nan"), dtype=torch.float16, device=cuda)
        func(a, bm, c, f)
        first = f.clone()
        for _ in range(3):
            f.fill_(float("nan"))
            func(a, bm, c, f)                                  # prepared path
            assert torch.equal(f, first)
        a.mul_(0.5)                                            # same buffers, new contents
        func(a, bm, c, f)
        s = a.float() @ bm.float()
        ref = (torch.softmax(s, -1) if kind == "softmax" else s.half().float()) @ c.float()
        assert (f.float() - ref).abs().max().item() < 2e-2 * ref.abs().max().item() + 1e-3
        assert ops.device_status(cuda) == 0
        with pytest.raises(ValueError):
            func(a[:, :128].contiguous(), bm, c, f)            # other tensors are checked again
        func(a, bm, c, f)                                      # and the module still works afterwards
        assert ops.device_status(cuda) == 0


@pytest.mark.parametrize("factory", [runtime.create_graph_engine, runtime.create_cuda_graph_engine])
def test_model_level_flow_attention_then_feed_forward(cuda, oracle, factory):
    """The whole sequence of benchmark/chimera/cuda/bert_inference.py:68-129 through `import ditto`: model ->
    graph -> chimera.graph_fusion -> extract_tasks_from_graph -> chimera.task_binding ->
    auto_schedule_bound_tasks -> build per key -> create_graph_engine -> compile / run / get_outputs /
    timeit(n).value, on a block of multi-head attention followed by the feed-forward block
    (linear + bias -> ReLU -> linear + bias -> ReLU, weights [out, in]); the output is compared with the
    oracle evaluated layer by layer."""
    import ditto as ref_name                      # the reference's package name resolves to this package
    from ditto import auto_schedule, chimera
    from ditto.auto_compute.nn.model import TransformerBlock
    assert ref_name.runtime is runtime
    batch, M, heads, hidden, d_ff, dtype = 2, 256, 4, 256, 1024, "float16"
    qkv_lt = ac.layer_tensor([batch, M, 3 * hidden], name="qkv", dtype=dtype)
    model = TransformerBlock(hidden, heads, d_ff, dtype=dtype, mma_in_dtype=dtype)
    out_lt = model(qkv_lt)
    graph = ac.graph([qkv_lt], [out_lt])
    assert [l.name for l in graph.all_layers] == ["multi_head_attention_mma_layer", "linear_layer", "relu_layer",
                                                  "linear_layer", "relu_layer"]
    graph = chimera.graph_fusion(graph)
    assert [l.name for l in graph.all_layers] == ["multi_head_attention_mma_layer", "ffn_layer"]
    option = auto_schedule.ScheduleOption("cuda", trials=10, device_name="gpu.cuda.B200", dtype=dtype,
                                          mma_in_dtype=dtype, mma_acc_dtype="float32")
    tasks = auto_schedule.extract_tasks_from_graph(graph)
    bound = chimera.task_binding(tasks)
    assert len(bound["chimera"]) == 2 and not bound["ansor"]
    schedules = auto_schedule.auto_schedule_bound_tasks(bound, option)
    built = {key: ditto.build(sch, args, "cuda") for key, (sch, args) in schedules.items()}
    assert sorted(m.schedule.kind for m in built.values()) == ["ffn", "mha"]
    engine = factory(graph, built, "cuda")
    engine.get_function("init")()
    rng = np.random.default_rng(47)
    qkv = W._round((rng.standard_normal((batch, M, 3 * hidden)) * 0.5).astype(np.float32), dtype)
    w1 = W._round((rng.standard_normal((d_ff, hidden)) * hidden ** -0.5).astype(np.float32), dtype)
    b1 = W._round((rng.standard_normal(d_ff) * 0.5).astype(np.float32), dtype)
    w2 = W._round((rng.standard_normal((hidden, d_ff)) * d_ff ** -0.5).astype(np.float32), dtype)
    b2 = W._round((rng.standard_normal(hidden) * 0.5).astype(np.float32), dtype)
    ffn_layer = graph.all_layers[1]
    for tensor, value in zip(ffn_layer.weights, (w1, b1, w2, b2)):
        engine.get_function("set_weight")(ffn_layer, tensor, torch.from_numpy(value))
    engine.get_function("set_inputs")(torch.from_numpy(qkv))
    engine.get_function("compile")()
    engine.get_function("run")()
    (out,) = engine.get_function("get_outputs")()
    assert ops.device_status(cuda) == 0
    attn = W._round(_mha_reference(oracle, qkv, heads, 0, 1.0), dtype)          # the layer writes fp16
    want = oracle.ffn(attn.reshape(1, batch * M, hidden), np.ascontiguousarray(w1.T)[None], b1[None],
                      np.ascontiguousarray(w2.T)[None], b2[None], 1, 1, 0).reshape(batch, M, hidden)
    assert_close(out.float().cpu().numpy(), want, dtype, "attention + feed-forward through the graph engine",
                 scale=float(np.abs(want).max()))
    cost = engine.get_function("timeit")(20).value
    assert 0 < cost < 5
