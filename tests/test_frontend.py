"""CPU tests of the host-side mirror of the reference's operator API."""
import pytest

import ditto_b200 as ditto
from ditto_b200 import auto_compute as ac
from ditto_b200 import auto_tensorize as at
from ditto_b200 import hardware as hw
from ditto_b200 import te
from ditto_b200 import workloads as W


def _softmax_chain(batch=12, M=512, N=64, K=64, L=512, scale=1.0):
    ins, outs = ac.nn.functional.BatchGemmSoftmaxGemm(batch, M, N, K, L, "float16", "float32", scale=scale)
    return ins, outs[0]


def _state(ins, F):
    E_frag = F.op.input_tensors[0]
    mid, C_ext = E_frag.op.input_tensors
    D_frag = mid.op.input_tensors[0]
    b, m, n, mi, ni = E_frag.op.axis
    rlo, rli = E_frag.op.reduce_axis
    fc = at.fusion_choice(D_frag.op, E_frag.op, [b, m, n, rlo, mi, ni, rli], 3)
    p1, p2 = at.cuda_wmma(scope="shared"), at.cuda_wmma(scope="global")
    c1 = at.intrinsic_match(D_frag, p1, ["InnerMost", "SameRange"])[0]
    c2 = at.intrinsic_match(E_frag, p2, ["InnerMost", "SameRange"])[0]
    layer = ac.layer([F.op], inputs=ins)
    st = at.tensorize_hyper_fusion_state(layer, fc, {D_frag.op: at.match_info(c1, p1), E_frag.op: at.match_info(c2, p2)})
    return layer, st


def test_chain_dag_has_the_reference_structure():
    ins, F = _softmax_chain()
    E_frag = F.op.input_tensors[0]
    exp, C_ext = E_frag.op.input_tensors
    D_frag = exp.op.input_tensors[0]
    A_shared, B_shared = D_frag.op.input_tensors
    assert [t.name for t in (F, E_frag, exp, C_ext, D_frag, A_shared, B_shared)] == \
        ["F", "E_frag", "exp", "C_ext", "D_frag", "A_shared", "B_shared"]
    assert E_frag.shape == (12, 32, 8, 16, 16)       # ext_N = 128: V padded with the ones column
    assert D_frag.shape == (12, 32, 32, 16, 16)
    assert [iv.extent for iv in E_frag.op.reduce_axis] == [32, 16]
    assert F.shape == (12, 512, 64) and F.dtype == "float16"


def test_chain_asserts_multiples_of_16_like_the_reference():
    with pytest.raises(AssertionError):
        _softmax_chain(M=500)
    with pytest.raises(AssertionError):
        ac.nn.functional.BatchGemmReluGemm(1, 128, 64, 72, 128)


def test_layer_argument_order_and_counters():
    ins, F = _softmax_chain()
    layer = ac.layer([F.op], inputs=ins)
    assert layer.schedule_tensors == [*ins, F]
    assert layer.num_inputs == 3
    # 2 * MACs of both contractions, the second one over ext_N = 128 columns like the reference counts it
    assert layer.gflops == pytest.approx(2 * 12 * 512 * 512 * (64 + 128) / 1e9)
    assert layer.data_transfer_amount == 4 * 12 * 512 * 64 * 2
    ins2, F2 = _softmax_chain()
    assert ac.layer([F2.op], inputs=ins2).fingerprint == layer.fingerprint
    ins3, F3 = _softmax_chain(batch=8)
    assert ac.layer([F3.op], inputs=ins3).fingerprint != layer.fingerprint
    with pytest.raises(ValueError):
        ac.layer([F.op], inputs=ins[:2])


def test_serial_fusion_state_and_partition():
    ins, F = _softmax_chain()
    layer, st = _state(ins, F)
    sfs = at.build_serial_fusion_state(layer)
    assert (sfs.first_op.name, sfs.second_op.name) == ("D_frag", "E_frag")
    assert [[o.name for o in g] for g in st.first_op_prologue] == [["A_shared"], ["B_shared"]]
    assert [[o.name for o in g] for g in st.second_op_prologue] == [["C_ext"]]
    assert [o.name for o in st.inter_path] == ["exp"]
    assert [o.name for o in st.epilogue] == ["F"]
    assert st.chain_kind == "softmax"
    fc = at.build_fusion_choice(sfs, hw.query_hw_param("gpu.cuda.B200"), "float16", -1)
    assert fc.attach_pos == 3 and [iv.name for iv in fc.ordered_iters] == ["b", "mo", "no", "rlo", "mi", "ni", "rli"]


def test_relu_and_identity_chains_classify():
    for builder, kind in ((ac.nn.functional.BatchGemmReluGemm, "relu"), (ac.nn.functional.BatchGemmGemm, "identity")):
        ins, outs = builder(1, 256, 128, 128, 512, "bfloat16", "float32")
        layer, st = _state(ins, outs[0])
        assert st.chain_kind == kind
        sch = at.tensorize_cuda(layer, st, hw.query_hw_param("gpu.cuda.B200"), at.cuda_tensorize_param())
        assert (sch.kind, sch.batch, sch.M, sch.N, sch.K, sch.L, sch.dtype) == (kind, 1, 256, 128, 128, 512, "bfloat16")


def test_non_chains_are_rejected():
    A = te.placeholder([1, 64, 64], "A", "float16")
    B = te.placeholder([1, 64, 64], "B", "float16")
    one = te.compute([1, 4, 4, 16, 16], [A, B], "D", "float32", tag="cubic", reduce=[("rk", 4), ("rki", 16)])
    with pytest.raises(at.FusionError):
        at.build_serial_fusion_state(ac.layer([one.op], inputs=[A, B]))
    # first GEMM consumed twice: not a linear chain
    d = te.compute([1, 4, 4, 16, 16], [A, B], "D", "float32", tag="cubic", reduce=[("rk", 4), ("rki", 16)])
    e = te.compute([1, 4, 4, 16, 16], [d, d], "E", "float32", tag="cubic", reduce=[("rl", 4), ("rli", 16)])
    with pytest.raises(at.FusionError):
        at.build_serial_fusion_state(ac.layer([e.op], inputs=[A, B]))


def test_tensorize_and_build_carry_shape_dtype_scale():
    ins, F = _softmax_chain(scale=0.125)
    layer, st = _state(ins, F)
    param = at.cuda_tensorize_param(warp_size=32, ty_size=4, tz_size=2, input_vector_len=4, serial_y=2, serial_z=1,
                                    block_rx=8, warp_rx=4, block_ry=1, warp_ry=4, unroll_steps=512)
    assert param.to_json()["block_rx"] == 8
    sch = at.tensorize_cuda(layer, st, hw.query_hw_param("gpu.cuda.B200"), param)
    assert (sch.kind, sch.scale, sch.dtype) == ("softmax", 0.125, "float16")
    func = ditto.build(sch, layer.schedule_tensors, "cuda")
    assert func.entry_name == "default_function"
    assert func.get_function("default_function") is func
    with pytest.raises(ValueError):
        ditto.build(sch, layer.schedule_tensors, "llvm")
    # fp32 operands have no tensor-core path here
    ins32, outs32 = ac.nn.functional.BatchGemmSoftmaxGemm(2, 128, 64, 64, 128, "float32", "float32")
    layer32, st32 = _state(ins32, outs32[0])
    with pytest.raises(at.FusionError):
        at.tensorize_cuda(layer32, st32, hw.query_hw_param("gpu.cuda.B200"))


def test_hardware_table():
    b200 = hw.query_hw_param("gpu.cuda.B200")
    assert b200.num_groups == 148 and b200.shared_memory_per_group_kb == 227
    assert hw.query_hw_param("gpu.cuda.A100").num_groups == 108
    with pytest.raises(KeyError):
        hw.query_hw_param("gpu.cuda.H100")


def test_multi_head_attention_module_layer():
    mha = ac.nn.module.MultiHeadAttentionMMA(12, 768, in_dtype="float16")
    x = ac.layer_tensor([4, 512, 3 * 768], name="qkv", dtype="float16")
    y = mha(x)
    assert y.shape == (4, 512, 768)
    assert ac.nn.module.is_self_attention_layer(y.layer)
    sfs = at.build_serial_fusion_state(y.layer)
    assert sfs.first_op.shape == (48, 32, 32, 16, 16)
    g = ac.graph([x], [y])
    assert [lay.name for lay in g.all_layers] == ["multi_head_attention_mma_layer"]
    with pytest.raises(RuntimeError):
        mha(ac.layer_tensor([4, 512, 768], dtype="float16"))


def test_workload_table_matches_the_configs():
    w = W.WORKLOADS
    assert w["cfg2"].flops == pytest.approx(0.805e9, rel=1e-3) and w["cfg2"].bytes == pytest.approx(3.146e6, rel=1e-3)
    assert w["cfg3"].flops == pytest.approx(34.36e9, rel=1e-3) and w["cfg3"].bytes == pytest.approx(134.2e6, rel=1e-3)
    assert w["cfg4"].flops == pytest.approx(274.9e9, rel=1e-3) and w["cfg4"].bytes == pytest.approx(83.9e6, rel=1e-3)
    assert w["cfg5"].flops == pytest.approx(2.199e12, rel=1e-3) and w["cfg5"].bytes == pytest.approx(2.147e9, rel=1e-3)
    for world in (1, 2, 4, 8, 3):
        for name in ("cfg3", "cfg4", "cfg5"):
            spans = [w[name].shard(r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == w[name].units
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))


def test_seeded_inputs_do_not_depend_on_the_shard():
    w = W.WORKLOADS["cfg2"]
    q_all, k_all, v_all = W.attention_inputs(w, 0, 4)
    q2, k2, v2 = W.attention_slice(w, 2)
    assert (q_all[2] == q2).all() and (k_all[2] == k2).all() and (v_all[2] == v2).all()
    assert abs(float(q_all.std()) - 1.0) < 0.02
    import numpy as np
    assert (q2.astype(np.float16).astype(np.float32) == q2).all()  # already representable in fp16


def test_self_attention_layer_schedules_without_a_fusion_state():
    mha = ac.nn.module.MultiHeadAttentionMMA(12, 768, in_dtype="float16")
    y = mha(ac.layer_tensor([4, 512, 2304], dtype="float16"))
    sch = at.tensorize_cuda(y.layer, None, hw.query_hw_param("gpu.cuda.B200"))
    assert (sch.kind, sch.batch, sch.M, sch.N, sch.K, sch.L, sch.heads) == ("mha", 4, 512, 768, 64, 512, 12)
    func = ditto.build(sch, y.layer.schedule_tensors, "cuda")
    assert func.entry_name == "default_function"


def test_model_level_flow_binds_and_schedules_attention_layers():
    """The flow of benchmark/chimera/cuda/bert_inference.py:68-112: extract tasks by fingerprint,
    bind them, schedule the bound tasks, build one module per key."""
    from ditto_b200 import auto_schedule, chimera
    mha = ac.nn.module.MultiHeadAttentionMMA(12, 768, in_dtype="float16")
    x = ac.layer_tensor([4, 512, 2304], dtype="float16")
    y1 = mha(x)
    g = ac.graph([x], [y1])
    option = auto_schedule.ScheduleOption("cuda", trials=10, device_name="gpu.cuda.B200", dtype="float16")
    assert option.device.num_groups == 148
    tasks = auto_schedule.extract_tasks_from_graph(g)
    assert list(tasks) == [y1.layer.fingerprint] and len(tasks[y1.layer.fingerprint]) == 1
    bound = chimera.task_binding(tasks)
    assert list(bound["chimera"]) == [y1.layer.fingerprint] and not bound["ansor"]
    schedules = auto_schedule.auto_schedule_bound_tasks(bound, option)
    built = {key: ditto.build(sch, args, "cuda") for key, (sch, args) in schedules.items()}
    assert built[y1.layer.fingerprint].schedule.kind == "mha"
    # a plain fused chain is bound to the same scheduler; an unfusable layer is not
    ins, outs = ac.nn.functional.BatchGemmReluGemm(1, 256, 512, 128, 1024, "bfloat16", "float32")
    chain = ac.layer([outs[0].op], inputs=ins)
    A = te.placeholder([1, 64, 64], "A", "float16")
    single = ac.layer([te.compute([1, 64, 64], [A], "copy", "float16").op], inputs=[A], name="copy_layer")
    bound = chimera.task_binding({"c": [chain], "s": [single]})
    assert list(bound["chimera"]) == ["c"] and list(bound["ansor"]) == ["s"]
    sch, args = auto_schedule.get_tasks_scheduler_builder("chimera")({"c": [chain]}, option)["c"]
    assert sch.kind == "relu" and args == chain.schedule_tensors
    with pytest.raises(NotImplementedError):
        auto_schedule.get_tasks_scheduler_builder("ansor")


def test_reference_package_name_and_module_paths_resolve():
    """`import ditto` and the module paths the reference's callers use name the same module objects."""
    import importlib
    import ditto as ref_name
    import ditto_b200
    for path in ("auto_compute", "auto_compute.nn.functional", "auto_compute.nn.functional.bmm_chain",
                 "auto_compute.nn.functional.activation", "auto_compute.nn.functional.linear",
                 "auto_compute.nn.functional.softmax", "auto_compute.nn.module.self_attention",
                 "auto_compute.nn.module.linear_module", "auto_compute.nn.model.transformer", "auto_tensorize",
                 "auto_schedule", "chimera", "chimera.graph_fusion", "chimera.task_binding", "hardware", "runtime",
                 "runtime.graph_engine"):
        assert importlib.import_module("ditto." + path) is importlib.import_module("ditto_b200." + path), path
    from ditto import auto_compute as ac2, auto_tensorize as at2
    assert ac2 is ac and at2 is at and ref_name.build is ditto_b200.build


def test_library_ops_of_the_path():
    """softmax / ReLU / GELU / linear with the reference's names, argument order and op structure
    (nn/functional/softmax.py:4-35, activation.py:9-39, linear.py:4-41)."""
    F = ac.nn.functional
    x = te.placeholder([4, 8, 16], "x", "float16")
    w = te.placeholder([32, 16], "w", "float16")
    b = te.placeholder([32], "b", "float16")
    y = F.linear(x, w, b, out_dtype="float16")
    assert y.shape == (4, 8, 32) and y.op.tag == "bias_add" and y.op.input_tensors[0].op.tag == "linear"
    assert F.linear(x, w).op.reduce_axis[0].extent == 16
    with pytest.raises(AssertionError):
        F.linear(x, te.placeholder([32, 8], "w", "float16"))
    assert F.ReLU(y).op.name == "ReLU" and F.GELU(y).op.name == "gelu" and F.GELU(y).shape == y.shape
    s = F.softmax(x, dim=1)
    assert s.op.name == "softmax" and s.op.input_tensors[1].op.name == "sum_val"
    assert s.op.input_tensors[1].shape == (4, 16) and s.shape == x.shape
    with pytest.raises(AssertionError):
        F.softmax(x, dim=3)


def test_graph_fusion_builds_the_feed_forward_layer():
    """linear -> ReLU -> linear -> ReLU (nn/model/transformer.py:21-34) becomes one ffn layer; a lone linear + ReLU
    (which the reference would fuse and hand to Ansor) is left alone and bound to "ansor"."""
    from ditto_b200 import auto_schedule, chimera
    from ditto_b200.auto_compute.nn.model import PositionwiseFeedForward
    x = ac.layer_tensor([2, 128, 256], dtype="bfloat16")
    y = PositionwiseFeedForward(256, 1024, dtype="bfloat16", out_dtype="bfloat16")(x)
    g = chimera.graph_fusion(ac.graph([x], [y]))
    (ffn,) = g.all_layers
    assert ffn.name == "ffn_layer" and ffn.ffn_attrs == {"act1": "relu", "act2": "relu", "bias1": True, "bias2": True}
    assert [tuple(t.shape) for t in ffn.weights] == [(1024, 256), (1024,), (256, 1024), (256,)]
    sch = at.tensorize_cuda(ffn, None, hw.query_hw_param("gpu.cuda.B200"))
    assert (sch.kind, sch.batch, sch.M, sch.N, sch.K, sch.L) == ("ffn", 1, 256, 256, 256, 1024)
    assert (sch.act1, sch.act2, sch.bias1, sch.bias2) == ("relu", "relu", True, True)
    assert ffn.gflops == 0 or ffn.gflops > 0          # the property still evaluates on the fused DAG
    # GELU in the middle, no trailing activation, no biases
    m = ac.nn.module
    x2 = ac.layer_tensor([64, 128], dtype="float16")
    l1, l2 = m.Linear(128, 512, dtype="float16", out_dtype="float16"), m.Linear(512, 256, dtype="float16", out_dtype="float16")
    g2 = chimera.graph_fusion(ac.graph([x2], [l2(m.GELU()(l1(x2)))]))
    (f2,) = g2.all_layers
    assert f2.ffn_attrs == {"act1": "gelu", "act2": "identity", "bias1": False, "bias2": False}
    # not a feed-forward pattern
    x3 = ac.layer_tensor([64, 128], dtype="float16")
    y3 = m.ReLU()(m.Linear(128, 512, dtype="float16", out_dtype="float16")(x3))
    g3 = chimera.graph_fusion(ac.graph([x3], [y3]))
    assert [l.name for l in g3.all_layers] == ["linear_layer", "relu_layer"]
    bound = chimera.task_binding(auto_schedule.extract_tasks_from_graph(g3))
    assert not bound["chimera"] and len(bound["ansor"]) == 2
    # mixed dtypes are rejected where the kernel could not run them
    x4 = ac.layer_tensor([64, 128], dtype="float16")
    y4 = PositionwiseFeedForward(128, 512, dtype="float16", out_dtype="float32")(x4)
    (f4,) = chimera.graph_fusion(ac.graph([x4], [y4])).all_layers
    with pytest.raises(at.FusionError):
        at.tensorize_cuda(f4, None, hw.query_hw_param("gpu.cuda.B200"))
