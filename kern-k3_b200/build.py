"""Build the library in-tree.

  lib/libk3g.so        all sm_100a kernels + the C ABI (include/k3g.h)
  lib/cubin/*.cubin    one module per reference module name: the same `extern "C"` entry
                       names and parameter lists as the reference's cubins, so a manifest's
                       `modules` table can point at them

Compilation is plain nvcc for sm_100a only; objects are rebuilt when a source or header is
newer.  Usage: python kern-k3_b200/build.py [--force] [--verbose] [--no-cubins]
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "lib")
OBJ = os.path.join(LIB, "obj")
SO = os.path.join(LIB, "libk3g.so")

NVCC = os.environ.get("NVCC", "nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr"]

SOURCES = ["resnorm.cu", "quant.cu", "router.cu", "moe_route.cu", "collectives.cu", "mla_prep.cu", "kda.cu",
           "peer.cu", "quant_noalloc.cu", "glue_small.cu", "prefill_misc.cu", "weight_prep.cu"]

# reference module name -> (source, defines).  Names follow kernels.toml of the reference.
CUBINS = {
    "k3_residual_v2": ("resnorm.cu", []),
    "k3_residual_v2+LAND_BF16=1": ("resnorm.cu", ["-DLAND_BF16=1"]),
    "k3_residual_nb+LAND_BF16=1": ("resnorm.cu", ["-DLAND_BF16=1", "-DK3G_NB_NO_STATS=1"]),
    "k3_residual_nb_stats": ("resnorm.cu", ["-DLAND_BF16=1"]),
    "k3_residual_push_add2": ("resnorm.cu", ["-DLAND_BF16=1"]),
    "k3_quant_fp8_pair_v2": ("quant.cu", []),
    "k3_moe_prefill_v4+EP_RANKS=4+EP_STRIDED=1+TILE_SHIFT=7+SCATTER_WARPS=16":
        ("moe_route.cu", ["-DEP_RANKS=4", "-DEP_STRIDED=1", "-DTILE_SHIFT=7"]),
    "k3_router_argmax": ("router.cu", []),
    "k3_moe_prefill_v3+EP_STRIDED=1": ("moe_route.cu", ["-DEP_RANKS=4", "-DEP_STRIDED=1"]),
    "k3_collectives": ("collectives.cu", ["-DK3G_NR=4"]),
    "k3_rs_arrive_v2": ("collectives.cu", ["-DK3G_NR=4"]),
    "k3_allgather4_v3": ("collectives.cu", ["-DK3G_NR=4"]),
    "k3_reducescatter_pull_nr4": ("collectives.cu", ["-DK3G_NR=4", "-DK3G_ORDER=6"]),
    "k3_mla_prep_v2+INNER=3072+MLA_FUSED=5184": ("mla_prep.cu", ["-DINNER=3072", "-DMLA_FUSED=5184"]),
    "k3_mla_prep_bf16+INNER=3072+MLA_FUSED=5184": ("mla_prep.cu", ["-DINNER=3072", "-DMLA_FUSED=5184", "-DK3G_MLA_BF16=1"]),
    "k3_residual_push_v3": ("resnorm.cu", ["-DLAND_BF16=1", "-DK3G_PUSH_V3=1"]),
    "k3_land_fused": ("glue_small.cu", []),
    "k3_land": ("glue_small.cu", []),
    "k3_prefill": ("prefill_misc.cu", []),
    "embedding": ("prefill_misc.cu", []),
    "copy_rows": ("prefill_misc.cu", []),
    "k3_weight_prep": ("weight_prep.cu", []),
    "weight_prep": ("weight_prep.cu", []),
    "sigmoid_mul": ("glue_small.cu", []),
    "k3_span_state+HEADS=24": ("glue_small.cu", ["-DHEADS=24"]),
    "k3_mla_v2": ("glue_small.cu", []),
    "k3_span_gather_v3+HEADS=24": ("kda.cu", ["-DHEADS=24"]),
    "k3_kda_out_gate_v3+HEADS=24": ("kda.cu", ["-DHEADS=24"]),
    # entries of the fused call list (patch_manifest.py --fuse); no counterpart module in the reference
    "k3g_fused_residual": ("resnorm.cu", ["-DLAND_BF16=1", "-DK3G_FUSED_ENTRIES=1", "-DK3G_NR=4"]),
    "k3g_fused_situ": ("glue_small.cu", ["-DK3G_FUSED_ENTRIES=1", "-DK3G_NR=4"]),
}


def _headers():
    return [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))] + \
           [os.path.join(HERE, "..", "include", "k3g.h")]


def _newer(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.exists(d) and os.path.getmtime(d) > t for d in deps)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("build failed: " + " ".join(cmd))
    if verbose:
        sys.stdout.write(r.stdout + r.stderr)


def sources():
    return [s for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]


def build(force=False, verbose=False, cubins=True):
    os.makedirs(OBJ, exist_ok=True)
    hdrs = _headers()
    jobs = []
    objs = []
    for s in sources():
        src = os.path.join(CSRC, s)
        obj = os.path.join(OBJ, s.replace(".cu", ".o"))
        objs.append(obj)
        if force or _newer(obj, [src] + hdrs):
            jobs.append([NVCC] + ARCH + COMMON + (["-Xptxas", "-v"] if verbose else []) +
                        ["-Xcompiler", "-fPIC,-fvisibility=hidden", "-I", os.path.join(HERE, "..", "include"),
                         "-c", src, "-o", obj])
    if cubins:
        cdir = os.path.join(LIB, "cubin")
        os.makedirs(cdir, exist_ok=True)
        for name, (s, defs) in CUBINS.items():
            src = os.path.join(CSRC, s)
            if not os.path.exists(src):
                continue
            out = os.path.join(cdir, name + ".cubin")
            if force or _newer(out, [src] + hdrs):
                jobs.append([NVCC, "-cubin", "-arch=sm_100a", "-O3", "-std=c++17", "-lineinfo", "-DK3G_CUBIN_ONLY=1"] +
                            defs + ["-I", os.path.join(HERE, "..", "include"), "-o", out, src])
    with ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as ex:
        list(ex.map(lambda c: _run(c, verbose), jobs))
    if force or jobs or _newer(SO, objs):
        _run([NVCC] + ARCH + ["-shared", "-o", SO] + objs, verbose)
    return SO


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, cubins="--no-cubins" not in sys.argv))
