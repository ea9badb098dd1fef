"""Scheduler glue of the model-level flow (`ditto.auto_schedule`): task extraction, options, and the
"chimera" builder that maps fused-chain layers onto the sm_100a kernels.

In the reference this layer drives Ansor for ordinary layers and a tensor-core parameter search for
self-attention layers (python/ditto/auto_schedule/schedulers/dispatch.py:17-161,
chimera_integrate.py:298-556).  Here there is nothing to search -- the kernels have fixed tiles -- so
scheduling a bound task returns the chain schedule directly; layers that are not fused chains have no
scheduler on this path and are reported as such.
"""
from collections import OrderedDict

from .. import auto_tensorize as at
from .. import hardware as hw
from ..auto_compute.nn.module import is_self_attention_layer


class ScheduleOption:
    """Same fields as the reference's ScheduleOption (dispatch.py:17-80); the search-related ones
    (trials, log_file, builder, runner) are recorded and unused."""

    def __init__(self, target, target_host="llvm", trials=100, task_name="", log_file="tmp.log", builder="local",
                 runner="local", scheduler=None, verbose=2, device_name=None, dtype="float32",
                 mma_in_dtype="float16", mma_acc_dtype="float32", mma_MI=16, mma_NI=16, mma_KI=16):
        self.target = target
        self.target_host = target_host
        self.trials = trials
        self.task_name = task_name
        self.log_file = log_file
        self.builder = builder
        self.runner = runner
        self.scheduler = scheduler
        self.verbose = verbose
        self.device = hw.query_hw_param(device_name) if device_name is not None else None
        self.dtype = dtype
        self.mma_in_dtype = mma_in_dtype
        self.mma_acc_dtype = mma_acc_dtype
        self.mma_MI, self.mma_NI, self.mma_KI = mma_MI, mma_NI, mma_KI


def extract_tasks_from_graph(graph):
    """fingerprint -> layers with that fingerprint, in graph order (schedulers/common.py:34-42)."""
    tasks = OrderedDict()
    for layer in graph.all_layers:
        tasks.setdefault(layer.fingerprint, []).append(layer)
    return tasks


def _schedule_layer(layer, option):
    device = option.device or hw.query_hw_param("gpu.cuda.B200")
    if is_self_attention_layer(layer) or layer.name == "ffn_layer":
        return at.tensorize_cuda(layer, None, device)
    sfs = at.build_serial_fusion_state(layer)          # raises FusionError for non-chains
    choice = at.build_fusion_choice(sfs, device, option.mma_in_dtype, -1)
    packed = at.cuda_wmma(option.mma_MI, option.mma_NI, option.mma_KI, option.mma_in_dtype, option.mma_acc_dtype)
    info = {op: at.match_info(at.intrinsic_match(op.output(0), packed, ["InnerMost", "SameRange"])[0], packed)
            for op in (sfs.first_op, sfs.second_op)}
    state = at.tensorize_hyper_fusion_state(layer, choice, info)
    return at.tensorize_cuda(layer, state, device)


def get_tasks_scheduler_builder(name):
    """"chimera" -> function(tasks, option) -> {key: (schedule, args)}; "ansor" does not exist here."""
    if name != "chimera":
        raise NotImplementedError(f"scheduler {name!r} is not part of the fused-chain path (only 'chimera')")

    def build(tasks, option):
        return OrderedDict((key, (_schedule_layer(layers[0], option), layers[0].schedule_tensors))
                           for key, layers in tasks.items())
    return build


def auto_schedule_bound_tasks(bound_tasks, option):
    """{scheduler: {key: [layers]}} -> {key: (schedule, args)} (schedule.py:82-104 in the reference)."""
    schedules = OrderedDict()
    for scheduler, tasks in bound_tasks.items():
        if not tasks:
            continue
        schedules.update(get_tasks_scheduler_builder(scheduler)(tasks, option))
    return schedules


retrieve_schedule_bound_tasks = auto_schedule_bound_tasks   # nothing is tuned, so nothing is stored
