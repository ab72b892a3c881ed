"""TEST INFRASTRUCTURE — compile the reference's own kernels for sm_100a.

Reads the .cu files where they lie under the reference checkout (never copied into this
repository) and writes one cubin per module into oracle/_ref/, with the defines the
reference's kernels.toml gives each module.  The cubins are the device-side A/B oracle: on a
GPU box tests load them with the CUDA driver API and compare their outputs with the CPU
oracle and with this library's kernels, and tests/golden/make_golden.py records their
outputs as golden vectors.

The reference is device code only (no CPU path), so there is nothing to build for the host.
Usage: python oracle/build_ref.py [reference_root]   (default: K3_REFERENCE_ROOT, else the `reference` directory beside this repository)
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
REF_ROOT = os.environ.get("K3_REFERENCE_ROOT", os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference"))

# module -> (source relative to the reference root, defines, needs the ulonglong4_16a shim)
MODULES = {
    "k3_residual_v2": ("source/k3_residual_v2.cu", [], False),
    "k3_residual_v2+LAND_BF16=1": ("source/k3_residual_v2.cu", ["-DLAND_BF16=1"], False),
    "k3_residual_nb_stats": ("source/k3_residual_nb_stats.cu", ["-DLAND_BF16=1"], False),
    "k3_residual_push_add2": ("source/k3_residual_push_add2.cu", [], False),
    "k3_quant_fp8_pair_v2": ("source/k3_quant_fp8_pair_v2.cu", [], False),
    "k3_moe_prefill_v4+EP_RANKS=4+EP_STRIDED=1+TILE_SHIFT=7+SCATTER_WARPS=16":
        ("source/k3_moe_prefill_v4.cu", ["-DEP_RANKS=4", "-DEP_STRIDED=1", "-DTILE_SHIFT=7", "-DSCATTER_WARPS=16"], True),
    "k3_router_argmax": ("source/k3_router_argmax.cu", [], False),
    "k3_collectives": ("source/k3_collectives.cu", [], False),
    "k3_reducescatter_pull_nr4": ("source/k3_reducescatter_pull_nr4.cu", ["-DNR=4", "-DORDER=6"], False),
    "k3_rs_arrive_v2": ("source/k3_rs_arrive_v2.cu", [], False),
    "k3_allgather4_v3": ("source/k3_allgather4_v3.cu", [], False),
    "k3_mla_prep_v2+INNER=3072+MLA_FUSED=5184": ("source/k3_mla_prep_v2.cu", ["-DINNER=3072", "-DMLA_FUSED=5184"], False),
    "k3_mla_prep_bf16+INNER=3072+MLA_FUSED=5184": ("source/k3_mla_prep_bf16.cu", ["-DINNER=3072", "-DMLA_FUSED=5184"], False),
    "k3_land_fused": ("source/k3_land_fused.cu", [], False),
    "k3_land": ("source/k3_land.cu", [], False),
    "k3_prefill": ("source/k3_prefill.cu", [], False),
    "embedding": ("source/embedding.cu", [], False),
    "copy_rows": ("source/copy_rows.cu", [], False),
    "k3_weight_prep": ("source/k3_weight_prep.cu", [], False),
    "weight_prep": ("source/weight_prep.cu", [], False),
    "k3_residual_push_v3": ("source/k3_residual_push_v3.cu", [], False),
    "sigmoid_mul": ("source/sigmoid_mul.cu", [], False),
    "k3_span_gather_v3+HEADS=24": ("source/k3_span_gather_v3.cu", ["-DHEADS=24"], False),
    "k3_kda_out_gate_v3+HEADS=24": ("source/k3_kda_out_gate_v3.cu", ["-DHEADS=24"], False),
}


def build(ref_root=REF_ROOT, force=False):
    """Returns the list of cubins built or already present; [] when the reference is absent."""
    if not os.path.isdir(ref_root):
        return [os.path.join(OUT, f) for f in sorted(os.listdir(OUT))] if os.path.isdir(OUT) else []
    os.makedirs(OUT, exist_ok=True)
    done = []
    for name, (rel, defs, shim) in MODULES.items():
        src = os.path.join(ref_root, rel)
        out = os.path.join(OUT, name + ".cubin")
        if force or not os.path.exists(out) or os.path.getmtime(src) > os.path.getmtime(out):
            cmd = ["nvcc", "-cubin", "-arch=sm_100a", "-O3"] + defs
            if shim:
                cmd += ["-include", os.path.join(HERE, "ref_shim.h")]
            cmd += ["-o", out, src]
            subprocess.check_call(cmd)
        done.append(out)
    return done


if __name__ == "__main__":
    for p in build(*(sys.argv[1:2]), force="--force" in sys.argv):
        print(p)
