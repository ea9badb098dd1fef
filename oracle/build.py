"""Compile the CPU oracle (chain_oracle.c) into oracle/liboracle.so with gcc.

Test infrastructure: only tests/, the smoke check and the benchmark's CPU-baseline leg use it.
AVX2 + FMA is the only ISA extension assumed, so the prebuilt library runs on any x86-64-v3 host.
"""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "chain_oracle.c")
LIB = os.path.join(HERE, "liboracle.so")


def build(force=False):
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= os.path.getmtime(SRC):
        return LIB
    cmd = ["gcc", "-O3", "-mavx2", "-mfma", "-fopenmp", "-fPIC", "-shared", "-fno-strict-aliasing",
           "-o", LIB, SRC, "-lm"]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError("gcc failed on chain_oracle.c:\n" + r.stdout)
    return LIB


if __name__ == "__main__":
    print(build(force=True))
