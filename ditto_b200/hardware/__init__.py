"""Hardware parameter tables (`ditto.hardware.query_hw_param`,
python/ditto/hardware/__init__.py:43-54, devices/nvgpu/cuda_param.py:9-80), with a B200 entry."""
from dataclasses import dataclass


@dataclass(frozen=True)
class HardwareParam:
    register_per_processor_kb: float
    shared_memory_per_group_kb: float
    shared_memory_bandwidth_gbs: float
    global_memory_gb: float
    global_memory_bandwidth_gbs: float
    num_processors_per_group: int
    num_groups: int
    fp32_peak_perf_gflops: float
    launch_latency_s: float
    platform: str = "NVGPU"
    # additions for the tcgen05 path
    tensor_peak_fp16_gflops: float = 0.0
    tensor_memory_per_group_kb: float = 0.0
    l2_cache_mb: float = 0.0


_PARAMS = {
    # nominal figures: 148 SMs x 4 sub-partitions, 227 KB usable smem and 256 KB TMEM per SM,
    # 180 GB HBM3e at 7.7 TB/s, 2.25 PFLOP/s dense fp16/bf16, 126 MB L2
    "B200": HardwareParam(64, 227, 148 * 128 * 1.9, 180, 7700, 4, 148, 80e3, 3e-6, "NVGPU", 2.25e6, 256, 126),
    # kept so caller scripts written for the reference's tables still resolve; values as in the
    # reference's cuda_param.py
    "V100": HardwareParam(64, 96, 12080, 16, 750, 4, 80, 14e3, 5e-6),
    "A100": HardwareParam(64, 164, 12080, 40, 1555, 4, 108, 19.5e3, 5e-6),
    "RTX3090": HardwareParam(64, 100, 12080, 24, 936, 4, 82, 35.6e3, 5e-6),
}


def parse_target(target):
    """target ::= device_type.programming_model.architecture, e.g. gpu.cuda.B200"""
    return target.split(".")


def query_hw_param(target):
    dev_type, pmodel, arch = parse_target(target)
    if dev_type != "gpu" or pmodel != "cuda":
        raise KeyError(f"only gpu.cuda.* targets are known, got {target!r}")
    arch = arch.split("-")[0]
    if arch not in _PARAMS:
        raise KeyError(f"unknown architecture {arch!r}; known: {sorted(_PARAMS)}")
    return _PARAMS[arch]
