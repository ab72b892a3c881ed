"""Build tests/native/libk3g_probe.so (test infrastructure: device-side probes the shipped library does not
export).  Plain nvcc for sm_100a; rebuilt when a source or the library's device headers are newer."""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
CSRC = os.path.join(ROOT, "kern-k3_b200", "csrc")
SO = os.path.join(HERE, "libk3g_probe.so")
SOURCES = [os.path.join(HERE, "situ_probe.cu"), os.path.join(HERE, "store_probe.cu")]


def build(force=False):
    deps = SOURCES + [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cuh")]
    if not force and os.path.exists(SO) and all(os.path.getmtime(d) <= os.path.getmtime(SO) for d in deps):
        return SO
    cmd = [os.environ.get("NVCC", "nvcc"), "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo", "-shared",
           "-Xcompiler", "-fPIC,-fvisibility=hidden", "-I", CSRC, "-o", SO] + SOURCES
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("build failed: " + " ".join(cmd))
    return SO


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
