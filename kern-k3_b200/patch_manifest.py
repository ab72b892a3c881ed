"""Repoint a kern-k3 manifest at this library's cubins (what every scripts/gen_*.py of the reference
does for one optimisation: rewrite `modules` and the launches of `ops`, idempotently).

    python kern-k3_b200/patch_manifest.py MANIFEST.json [--out OUT.json] [--keep-grids]

Every launch whose (module, entry) pair this library provides is moved to a new module entry
`b200/<cubin name>` (source = the cubin file, sha256 = its digest); the entry name, the parameter
list and the argument mapping are left untouched, because the kernels take exactly the reference's
parameters.  Launch dims are kept unless this library has a better geometry for the kernel (all
kernels are grid-stride, so the reference's dims stay valid); `--keep-grids` disables the overrides.
Launches of kernels outside the glue path (GEMM, grouped GEMM, FMHA, FlashKDA) are not touched.  Prints a summary; exits non-zero if a provided entry is missing from its cubin.
"""
import argparse
import hashlib
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CUBIN_DIR = os.path.join(HERE, "lib", "cubin")

RES = ["kern_k3_land_add_attnres_rms_nb%d" % k for k in range(1, 9)]
# reference module -> (our cubin, entries of that module we provide with the same parameter list)
PROVIDED = {
    "k3_residual_v2": ("k3_residual_v2", ["kern_k3_attnres_rms", "kern_k3_land_add_attnres_rms", "kern_k3_land_add2"]),
    "k3_residual_v2+LAND_BF16=1": ("k3_residual_v2+LAND_BF16=1", ["kern_k3_attnres_rms", "kern_k3_land_add_attnres_rms", "kern_k3_land_add2"]),
    "k3_residual_nb+LAND_BF16=1": ("k3_residual_nb+LAND_BF16=1", RES),
    "k3_residual_nb_stats": ("k3_residual_nb_stats", RES),
    "k3_residual_push_add2": ("k3_residual_push_add2", ["kern_k3_attnres_rms_push"]),
    "k3_quant_fp8_pair_v2": ("k3_quant_fp8_pair_v2", ["kern_quant_fp8_amax_v2", "kern_quant_fp8_apply_v2"]),
    "k3_moe_prefill_v3+EP_STRIDED=1": ("k3_moe_prefill_v3+EP_STRIDED=1", ["kern_k3_moe_route_count", "kern_k3_moe_finalize", "kern_k3_moe_w_shuffle",
                                                                        "kern_k3_moe_sf_shuffle"]),
    "k3_moe_prefill_v4+EP_RANKS=4+EP_STRIDED=1+TILE_SHIFT=7+SCATTER_WARPS=16":
        ("k3_moe_prefill_v4+EP_RANKS=4+EP_STRIDED=1+TILE_SHIFT=7+SCATTER_WARPS=16",
         ["kern_k3_moe_route_count", "kern_k3_moe_route_tables", "kern_k3_moe_route_scatter", "kern_k3_moe_finalize",
          "kern_k3_moe_w_shuffle", "kern_k3_moe_sf_shuffle"]),
    "k3_router_argmax": ("k3_router_argmax", ["kern_k3_router_topk", "kern_k3_argmax_f32_partial", "kern_k3_argmax_f32_final"]),
    "k3_residual_push_v3": ("k3_residual_push_v3", ["kern_k3_attnres_rms_push"]),
    "k3_land": ("k3_land", ["kern_k3_land_situ", "kern_k3_land", "kern_k3_rms"]),
    "k3_prefill": ("k3_prefill", ["kern_k3_rank_rows", "kern_k3_zero_rows", "kern_k3_fmha_lens"]),
    "embedding": ("embedding", ["kern_embedding_i64_bf16"]),
    "copy_rows": ("copy_rows", ["kern_copy_rows_bf16", "kern_last_row_bf16", "kern_own_rows"]),
    "k3_weight_prep": ("k3_weight_prep", ["kern_fill_bf16", "kern_k3_conv_taps", "kern_k3_scoring", "kern_k3_wsm", "kern_k3_mega_sf_pack", "kern_k3_kvb_aug"]),
    "weight_prep": ("weight_prep", ["kern_weight_p1_bf16_f32", "kern_cast_bf16_f32", "kern_rope_table_bf16", "kern_fill_f32", "kern_fill_i32",
                                    "kern_fill_i64", "kern_fill_u8", "kern_iota_i32"]),
    "k3_collectives": ("k3_collectives", ["kern_k3_flags_init", "kern_k3_epoch_bump"]),
    "k3_rs_arrive_v2": ("k3_rs_arrive_v2", ["kern_k3_rs_arrive1"]),
    "k3_reducescatter_pull_nr4": ("k3_reducescatter_pull_nr4", ["kern_k3_rs_pull"]),
    "k3_allgather4_v3": ("k3_allgather4_v3", ["kern_k3_allgather4_push"]),
    "k3_mla_prep_bf16+INNER=3072+MLA_FUSED=5184": ("k3_mla_prep_bf16+INNER=3072+MLA_FUSED=5184", ["kern_k3_mla_prep_head", "kern_k3_mla_prep_gate"]),
    "k3_mla_prep_v2+INNER=3072+MLA_FUSED=5184": ("k3_mla_prep_v2+INNER=3072+MLA_FUSED=5184", ["kern_k3_mla_prep_head", "kern_k3_mla_prep_gate"]),
    "k3_land_fused": ("k3_land_fused", ["kern_k3_situ_rms_bf16"]),
    "sigmoid_mul": ("sigmoid_mul", ["kern_sigmoid_mul_bf16"]),
    "k3_span_state+HEADS=24": ("k3_span_state+HEADS=24", ["kern_k3_span_state"]),
    "k3_mla_v2": ("k3_mla_v2", ["kern_k3_latent_gather"]),
    "k3_span_gather_v3+HEADS=24": ("k3_span_gather_v3+HEADS=24", ["kern_k3_span_gather"]),
    "k3_kda_out_gate_v3+HEADS=24": ("k3_kda_out_gate_v3+HEADS=24", ["kern_k3_kda_out_gate"]),
}
# kern_k3_moe_quant lives in the quant cubin here
MOVED = {("k3_moe_prefill_v3+EP_STRIDED=1", "kern_k3_moe_quant"): "k3_quant_fp8_pair_v2",
         ("k3_moe_prefill_v4+EP_RANKS=4+EP_STRIDED=1+TILE_SHIFT=7+SCATTER_WARPS=16", "kern_k3_moe_quant"): "k3_quant_fp8_pair_v2"}

# better launch dims for this library's kernels: entry -> (block, grid expression over `tokens`)
T4 = {"ceil_div": ["tokens", 4]}
GRIDS = {
    "kern_k3_router_topk": ([256, 1, 1], [{"ceil_div": [T4, 8]}, 1, 1]),                          # one warp per row, 8 rows per block
    "kern_k3_moe_quant": ([256, 1, 1], [{"ceil_div": [{"mul": [T4, 112]}, 256]}, 1, 1]),          # one 32-group per thread (unchanged)
    "kern_k3_span_gather": ([128, 1, 1], [6, 4, {"ceil_div": ["tokens", 64]}]),                   # 64 rows per block
    "kern_k3_kda_out_gate": ([128, 1, 1], [{"ceil_div": ["tokens", 2]}, 3, 1]),                   # two rows per pass
    "kern_k3_mla_prep_head": ([128, 1, 1], [{"ceil_div": ["tokens", 4]}, 1, 1]),                  # one warp per row
    "kern_k3_situ_rms_bf16": ([128, 1, 1], [{"mul": [{"ceil_div": ["tokens", 8]}, 5]}, 1, 1]),            # one item per 128-thread block, 1 norm : 4 SiTU
    "kern_k3_mla_prep_gate": ([256, 1, 1], [{"ceil_div": [{"mul": ["tokens", 384]}, 256]}, 1, 1]),  # 8 columns per thread, flat
}


def sha256(path):
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 20), b""):
            h.update(chunk)
    return h.hexdigest()


def patch(manifest, cubin_dir=CUBIN_DIR, keep_grids=False):
    """Patches `manifest` (a dict) in place; returns a summary dict."""
    moved, left, missing = [], [], []
    blobs = {}

    def cubin_for(name, entry):
        path = os.path.join(cubin_dir, name + ".cubin")
        if name not in blobs:
            blobs[name] = open(path, "rb").read() if os.path.exists(path) else None
        if blobs[name] is None or entry.encode() + b"\0" not in blobs[name]:
            missing.append((name, entry))
            return None
        return path

    for op_name, op in manifest.get("ops", {}).items():
        for launch in op.get("impl", {}).get("launches", []):
            mod, entry = launch.get("module"), launch.get("entry")
            if mod is None:
                continue
            if mod.startswith("b200/"):
                moved.append((op_name, entry, mod))
                continue
            ours = None
            if (mod, entry) in MOVED:
                ours = MOVED[(mod, entry)]
            elif mod in PROVIDED and entry in PROVIDED[mod][1]:
                ours = PROVIDED[mod][0]
            if ours is None:
                left.append((op_name, entry, mod))
                continue
            path = cubin_for(ours, entry)
            if path is None:
                continue
            key = "b200/" + ours
            manifest["modules"][key] = {"source": os.path.basename(path), "sha256": sha256(path)}
            launch["module"] = key
            if not keep_grids and entry in GRIDS:
                launch["block"], launch["grid"] = GRIDS[entry][0], GRIDS[entry][1]
            moved.append((op_name, entry, key))
    used = {l.get("module") for op in manifest.get("ops", {}).values() for l in op.get("impl", {}).get("launches", [])}
    for name in [m for m in manifest.get("modules", {}) if m not in used and m in PROVIDED]:
        del manifest["modules"][name]          # a module no launch references any more
    return {"moved": moved, "left": left, "missing": missing}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("manifest")
    ap.add_argument("--out")
    ap.add_argument("--cubins", default=CUBIN_DIR)
    ap.add_argument("--keep-grids", action="store_true")
    a = ap.parse_args()
    m = json.load(open(a.manifest))
    s = patch(m, a.cubins, a.keep_grids)
    json.dump(m, open(a.out or a.manifest, "w"), indent=1)
    print("launches moved to b200 cubins: %d; left on reference modules: %d" % (len(s["moved"]), len(s["left"])))
    for op, entry, mod in s["moved"]:
        print("  moved  %-42s %-36s -> %s" % (op, entry, mod))
    for name, entry in s["missing"]:
        print("  MISSING entry %s in %s.cubin" % (entry, name))
    sys.exit(1 if s["missing"] else 0)


if __name__ == "__main__":
    main()
