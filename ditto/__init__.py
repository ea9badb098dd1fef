"""`import ditto` for callers of KnowingNothing/Ditto's fused GEMM-chain path.

The reference's Python package is called `ditto`; its scripts do `from ditto import auto_compute as ac`,
`from ditto import auto_tensorize as at`, `import ditto.runtime` ... (benchmark/chimera/cuda/
bmm_softmax_bmm_cuda.py:1-12, bert_inference.py:5-12).  This package makes those imports resolve to
`ditto_b200`: every module of ditto_b200 is also importable under the reference's module path, e.g.

    ditto.auto_compute.nn.functional.bmm_chain      ditto.auto_compute.nn.module.self_attention
    ditto.auto_compute.nn.model.transformer         ditto.runtime.graph_engine
    ditto.auto_schedule    ditto.auto_tensorize     ditto.chimera.graph_fusion    ditto.hardware

Both names refer to the same module objects (no second copy of any state).  Parts of the reference outside
this path (autograd, dse, conv ops, the model zoo) do not exist here and raise ImportError as usual.
"""
import importlib
import pkgutil
import sys

import ditto_b200 as _impl

_SKIP = ("ditto_b200.build_lib", "ditto_b200.csrc")


def _alias_all():
    names = ["ditto_b200"]
    for info in pkgutil.walk_packages(_impl.__path__, prefix="ditto_b200."):
        if not info.name.startswith(_SKIP):
            names.append(info.name)
    for name in names:
        mod = importlib.import_module(name)
        alias = "ditto" + name[len("ditto_b200"):]
        if alias != "ditto":
            sys.modules.setdefault(alias, mod)


_alias_all()

from ditto_b200 import (auto_compute, auto_schedule, auto_tensorize, chimera, hardware, ops, runtime, te)  # noqa: E402
from ditto_b200 import build  # noqa: E402

__all__ = list(_impl.__all__)
