"""Build the CPU oracle (test infrastructure) into oracle/_build/libk3oracle.so.

Plain g++ with OpenMP; -ffp-contract=off so the only fused multiply-adds are the ones
the source spells out, -mfma so std::fmaf is a single instruction.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_build")
OUT = os.path.join(OUT_DIR, "libk3oracle.so")
SRCS = [os.path.join(HERE, "k3o_ops.cpp")]
DEPS = SRCS + [os.path.join(HERE, "k3o_numerics.h")]


def stale():
    if not os.path.exists(OUT):
        return True
    t = os.path.getmtime(OUT)
    return any(os.path.getmtime(d) > t for d in DEPS)


def build(force=False):
    if not force and not stale():
        return OUT
    os.makedirs(OUT_DIR, exist_ok=True)
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-fopenmp", "-ffp-contract=off",
           "-mavx2", "-mfma", "-fvisibility=hidden", "-o", OUT] + SRCS
    subprocess.check_call(cmd)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
