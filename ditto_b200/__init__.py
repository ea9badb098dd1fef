"""ditto_b200: the fused GEMM-chain path of KnowingNothing/Ditto, rebuilt for B200 (sm_100a).

    from ditto_b200 import auto_compute as ac, auto_tensorize as at, hardware as hw, runtime
    ins, outs = ac.nn.functional.BatchGemmSoftmaxGemm(12, 512, 64, 64, 512)
    layer = ac.layer([outs[0].op], inputs=ins)
    sfs = at.build_serial_fusion_state(layer)
    ...
    func = ditto_b200.build(at.tensorize_cuda(layer, state, hw.query_hw_param("gpu.cuda.B200")),
                            layer.schedule_tensors, "cuda")
    func(q, k, v, out)            # torch CUDA tensors, destination passing like the reference

or directly `ditto_b200.ops.bmm_softmax_bmm(q, k, v)` / `ditto_b200.ops.gemm_relu_gemm(x, w1, w2)`.
The arithmetic runs only in libditto_b200.so (hand-written CUDA); there is no CPU fallback.
"""
from . import te
from . import hardware
from . import auto_compute
from . import auto_tensorize
from . import runtime
from . import ops
from . import auto_schedule
from . import chimera
from .runtime import build

__all__ = ["te", "hardware", "auto_compute", "auto_tensorize", "auto_schedule", "chimera", "runtime", "ops", "build"]
