"""Compile the reference's own CPU micro-kernels into oracle/_ref/libditto_ref_microkernels.so.

Test infrastructure.  The reference's CPU path is TVM-generated code around two hand-written
micro-kernels whose C++/asm text is produced by plain Python string builders:

  * gemm_impl((6, 16, KI), "avx2", "float32", prefix)   python/ditto/auto_tensorize/intrinsic.py:274-604
        <prefix>_update(C, A, B, K, N, c_stride):  C[6 x 16] += A[6 x KI] (row stride K) * B[KI x 16] (row stride N)
        <prefix>_reset(C, stride)
  * exp_impl((MI, NI), "avx512", "float32", prefix)     python/ditto/auto_tensorize/intrinsic.py:1480-1672
        <prefix>compute_exp(dst, src, dst_stride, src_stride): Cephes-style polynomial exp on MI x NI floats

TVM itself is absent, so the builders are imported from the reference tree where it lies with
stand-ins for the few `tvm` names they touch (`clang.create_llvm` just hands the source text back).
The generated text is written under oracle/_ref/ (git-ignored, never committed) and compiled with
g++.  Where the reference tree is not present (any machine but the development container) this
script does nothing and a previously built library keeps being used.
"""
import importlib.util
import os
import subprocess
import sys
import tempfile
import types

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
LIB = os.path.join(OUT_DIR, "libditto_ref_microkernels.so")
GEMM_KI = (16, 32, 64, 128)            # reduction lengths baked into the generated kernels
EXP_SHAPES = ((1, 16), (6, 16), (6, 64))


def reference_root():
    """Where the reference's source tree lies: $DITTO_REFERENCE_ROOT, else a `reference` directory beside
    this repository (the layout of the development container).  A machine without it keeps the prebuilt library."""
    return os.environ.get("DITTO_REFERENCE_ROOT",
                          os.path.normpath(os.path.join(HERE, os.pardir, os.pardir, "reference")))


def host_flags():
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("flags"):
                    return set(line.split(":", 1)[1].split())
    except OSError:
        pass
    return set()


def _stub_tvm():
    """Minimal stand-ins for the tvm modules intrinsic.py imports at module level or inside the builders."""
    captured = {}

    def register_object(_name=None):
        return lambda cls: cls

    def create_llvm(code, output=None, options=None):
        captured["last"] = code
        return code

    class _TempDir:
        def __init__(self):
            self._d = tempfile.mkdtemp(prefix="ditto_ref_")

        def relpath(self, name):
            return os.path.join(self._d, name)

    class _Any:
        """Whatever else the module's annotations and decorators name (tvm.te.tensor_intrin.TensorIntrin ...)."""

        def __getattr__(self, _name):
            return _Any()

        def __call__(self, *a, **k):
            return _Any()

    class _Module(types.ModuleType):
        def __getattr__(self, name):
            if name.startswith("__"):
                raise AttributeError(name)
            return _Any()

    mods = {name: _Module(name) for name in
            ("tvm", "tvm._ffi", "tvm.runtime", "tvm.te", "tvm.contrib", "tvm.contrib.utils", "tvm.contrib.clang")}
    mods["tvm._ffi"].register_object = register_object
    mods["tvm.runtime"].Object = object
    mods["tvm.contrib.utils"].tempdir = _TempDir
    mods["tvm.contrib.clang"].create_llvm = create_llvm
    mods["tvm"]._ffi = mods["tvm._ffi"]
    mods["tvm"].runtime = mods["tvm.runtime"]
    mods["tvm"].te = mods["tvm.te"]
    mods["tvm"].contrib = mods["tvm.contrib"]
    mods["tvm.contrib"].utils = mods["tvm.contrib.utils"]
    mods["tvm.contrib"].clang = mods["tvm.contrib.clang"]
    return mods


def _load_generators():
    path = os.path.join(reference_root(), "python", "ditto", "auto_tensorize", "intrinsic.py")
    if not os.path.exists(path):
        return None
    saved = {k: sys.modules.get(k) for k in list(_stub_tvm().keys()) + ["_ditto_ref_at", "_ditto_ref_at._ffi_api"]}
    try:
        sys.modules.update(_stub_tvm())
        pkg = types.ModuleType("_ditto_ref_at")
        pkg.__path__ = []
        sys.modules["_ditto_ref_at"] = pkg
        sys.modules["_ditto_ref_at._ffi_api"] = types.ModuleType("_ditto_ref_at._ffi_api")
        spec = importlib.util.spec_from_file_location("_ditto_ref_at.intrinsic", path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        return mod
    finally:
        # the stand-ins stay only as long as the builders need them: they are re-installed in build()
        for k, v in saved.items():
            if v is None:
                sys.modules.pop(k, None)
            else:
                sys.modules[k] = v


def _run(cmd):
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError(" ".join(cmd[:3]) + " ... failed on the generated micro-kernels:\n" + r.stdout[-4000:])


def build(force=False, verbose=False):
    """Returns the library path, or None when neither the reference tree nor a built library exists."""
    have_lib = os.path.exists(LIB)
    if have_lib and not force:
        return LIB
    flags = host_flags()
    if not {"avx2", "fma"} <= flags:
        return LIB if have_lib else None
    gen = _load_generators()
    if gen is None:
        return LIB if have_lib else None
    os.makedirs(OUT_DIR, exist_ok=True)
    sources = []
    cwd = os.getcwd()
    stubs = _stub_tvm()
    saved = {k: sys.modules.get(k) for k in stubs}
    sys.modules.update(stubs)
    try:
        os.chdir(OUT_DIR)                      # gemm_impl drops a copy of its text into the working directory
        for ki in GEMM_KI:
            text = gen.gemm_impl((6, 16, ki), "avx2", "float32", f"ref_gemm_k{ki}")
            p = os.path.join(OUT_DIR, f"ref_gemm_k{ki}.cc")
            with open(p, "w") as f:
                f.write(text)
            sources.append(p)
        if "avx512f" in flags:
            for (mi, ni) in EXP_SHAPES:
                text = gen.exp_impl((mi, ni), "avx512", "float32", f"ref_exp_{mi}x{ni}_")
                p = os.path.join(OUT_DIR, f"ref_exp_{mi}x{ni}.cc")
                with open(p, "w") as f:
                    f.write(text)
                sources.append(p)
    finally:
        os.chdir(cwd)
        for k, v in saved.items():
            if v is None:
                sys.modules.pop(k, None)
            else:
                sys.modules[k] = v
    stray = os.path.join(OUT_DIR, "gemm.cc")
    if os.path.exists(stray):
        os.remove(stray)
    isa = ["-mavx2", "-mfma"] + (["-mavx512f"] if "avx512f" in flags else [])
    objects = []
    for src in sources:
        tag = os.path.splitext(os.path.basename(src))[0]
        obj = os.path.join(OUT_DIR, tag + ".o")
        _run(["g++", "-O2", "-fPIC", "-w", "-c"] + isa + ["-o", obj, src])
        if tag.startswith("ref_exp"):
            # every exp unit defines the same two external pointers to its constants: make them unit-local
            _run(["objcopy", "--localize-symbol=_ps_exp_hi_p", "--localize-symbol=_ps_one_p", obj])
        objects.append(obj)
    _run(["g++", "-shared", "-o", LIB] + objects)
    for f in objects + sources:                # only the library stays: the generated text is the reference's
        os.remove(f)
    if verbose:
        print("built", LIB, "from", [os.path.basename(s) for s in sources])
    return LIB


if __name__ == "__main__":
    print(build(force=True, verbose=True))
