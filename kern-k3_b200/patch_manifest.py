"""Repoint a kern-k3 manifest at this library's cubins (what every scripts/gen_*.py of the reference
does for one optimisation: rewrite `modules` and the launches of `ops`, idempotently).

    python kern-k3_b200/patch_manifest.py MANIFEST.json [--out OUT.json] [--keep-grids] [--fuse]

Every launch whose (module, entry) pair this library provides is moved to a new module entry
`b200/<cubin name>` (source = the cubin file, sha256 = its digest); the entry name, the parameter
list and the argument mapping are left untouched, because the kernels take exactly the reference's
parameters.  Launch dims are kept unless this library has a better geometry for the kernel (all
kernels are grid-stride, so the reference's dims stay valid); `--keep-grids` disables the overrides.
Launches of kernels outside the glue path (GEMM, grouped GEMM, FMHA, FlashKDA) are not touched.  Prints a summary; exits non-zero if a provided entry is missing from its cubin.

`--fuse` additionally rewrites `programs.prefill.calls` to this library's fused call list, the way the reference adopts
its own optimisations (scripts/gen_push_add2.py, scripts/gen_attn_stats.py: new op records, scratch buffers and a
call-list edit, idempotent).  Per layer, with outputs bit-identical to the unfused list:
  * the producers of the three per-tensor FP8 operands leave the maxima the quantisation needs (rows of `normed_all`,
    rows of `normed`, 4096-element items of `shared_act`), and `quant_fp8_tensor` (amax launch + apply launch) becomes
    `quant_fp8_apply` (the apply launch alone, reading those maxima);
  * `reduce_attn` (arrive + pull reduce-scatter) disappears into `res_mlp`: `rs_land_add_attnres_rms` = the same arrive
    launch, then the landing kernel pulling the four ranks' partial rows itself;
  * `scatter_moe` disappears into `shared_situ` the same way: `rs_situ_rms`.
New scratch buffers: `rowmax_all` (exported, with its peer table `rowmax_all_peer`), `rowmax`, `item_max`.
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


FUSED_RES, FUSED_SITU, QUANT = "b200/k3g_fused_residual", "b200/k3g_fused_situ", "b200/k3_quant_fp8_pair_v2"
B4 = {"ceil_div": ["tokens", 4]}                                   # rows per rank
NB_OPS = ["land_add_attnres_rms_bf16_v2_nb%d" % k for k in range(1, 9)]


def _module(manifest, key, cubin_dir):
    path = os.path.join(cubin_dir, key[len("b200/"):] + ".cubin")
    manifest["modules"][key] = {"source": os.path.basename(path), "sha256": sha256(path)}


def fuse(manifest, cubin_dir=CUBIN_DIR):
    """Rewrites the prefill call list of a manifest already patched by `patch` to the fused list; idempotent.
    Returns {"layers_*": counts, "launches_before": n, "launches_after": n}."""
    ops, bufs, calls = manifest["ops"], manifest["buffers"], manifest["programs"]["prefill"]["calls"]
    launches = lambda: sum(len(ops[c["op"]]["impl"]["launches"]) for c in calls)
    before = launches()
    rows_all = bufs["normed_all"]["shape"][0]
    rows_own = bufs["attn_stats"]["shape"][0] if "attn_stats" in bufs else (rows_all + 3) // 4
    # ---- scratch buffers -------------------------------------------------------------------------------------------
    bufs.setdefault("rowmax_all", {"dtype": "f32", "shape": [rows_all], "kind": "workspace", "export": True})
    bufs.setdefault("rowmax_all_peer", {"dtype": "u64", "shape": [4], "kind": "peer", "of": "rowmax_all", "group": "tp"})
    bufs.setdefault("rowmax", {"dtype": "f32", "shape": [rows_own], "kind": "workspace"})
    bufs.setdefault("item_max", {"dtype": "f32", "shape": [(rows_own * 6144 + 4095) // 4096], "kind": "workspace"})
    bufs.setdefault("attn_stats", {"dtype": "f32", "shape": [rows_own, 8, 2], "kind": "workspace"})
    # ---- op records --------------------------------------------------------------------------------------------------
    if "attnres_rms_push_add2_amax" not in ops:
        op = json.loads(json.dumps(ops["attnres_rms_push_add2"]))
        n = len(op["params"])
        op["params"] += ["out buffer<f32>", "in buffer<u64>"]
        l = op["impl"]["launches"][0]
        l["module"], l["entry"] = FUSED_RES, "kern_k3g_attnres_rms_push_amax"
        l["params"] = l["params"] + ["out buffer<f32>", "in buffer<u64>"]
        l["args"] = l["args"] + [{"param": n}, {"param": n + 1}]
        ops["attnres_rms_push_add2_amax"] = op
    if "quant_fp8_apply" not in ops:
        apply_l = json.loads(json.dumps(ops["quant_fp8_tensor"]["impl"]["launches"][1]))      # kern_quant_fp8_apply_v2(x, y, n, partials, nb, scale)
        apply_l["module"] = QUANT
        apply_l["grid"] = [592, 1, 1]          # every block reduces all partial maxima first: one resident wave, not 2048 blocks
        apply_l["args"] = [{"param": 0}, {"param": 1}, {"param": 5}, {"param": 3}, {"param": 4}, {"param": 2}]
        ops["quant_fp8_apply"] = {"params": ["in buffer<bf16>", "out buffer<u8>", "out buffer<f32>", "in buffer<f32>", "i32", "i32"],
                                  "impl": {"launches": [apply_l]}}
    arrive = json.loads(json.dumps(ops["k3_reducescatter_bf16"]["impl"]["launches"][0]))      # kern_k3_rs_arrive1, 11 kernel parameters
    if "rs_land_add_attnres_rms" not in ops:
        # op parameters: partial, partial_peer, flags, flags_peer, units, slot, prefix, blocks, sw, gamma, prefix2, normed, nb, snapshot, B,
        #                stats, nb_stats, rowmax
        a = json.loads(json.dumps(arrive))
        a["args"] = [{"param": 0}, {"param": 0}, {"param": 1}, {"param": 2}, {"param": 3}, {"i64": 0}, {"param": 4}, {"param": 5}, {"i32": 6},
                     {"rank": "tp"}, {"i32": 4}]
        ops["rs_land_add_attnres_rms"] = {
            "params": ["in buffer<bf16>", "in buffer<u64>", "out buffer<u64>", "in buffer<u64>", "i32", "i32", "in buffer<bf16>", "in buffer<bf16>",
                       "in buffer<f32>", "in buffer<bf16>", "out buffer<bf16>", "out buffer<bf16>", "i32", "i32", "i32", "in buffer<f32>", "i32",
                       "out buffer<f32>"],
            "impl": {"launches": [a, {
                "module": FUSED_RES, "entry": "kern_k3g_rs_land_add_attnres_rms",
                "params": ["in buffer<bf16>", "in buffer<u64>", "i32", "i32", "in buffer<bf16>", "in buffer<bf16>", "in buffer<f32>", "in buffer<bf16>",
                           "out buffer<bf16>", "out buffer<bf16>", "i32", "i32", "i32", "in buffer<f32>", "i32", "out buffer<f32>"],
                "args": [{"param": 0}, {"param": 1}, {"rank": "tp"}, {"i32": 4}] + [{"param": i} for i in range(6, 18)],
                "block": [128, 1, 1], "grid": [B4, 1, 1]}]}}
    if "rs_situ_rms" not in ops:
        # op parameters: sp, act, partial, partial_peer, flags, flags_peer, units, slot, gam, ln, B, L, item_max
        a = json.loads(json.dumps(arrive))
        a["args"] = [{"param": 2}, {"param": 2}, {"param": 3}, {"param": 4}, {"param": 5}, {"i64": 0}, {"param": 6}, {"param": 7}, {"i32": 6},
                     {"rank": "tp"}, {"i32": 4}]
        ops["rs_situ_rms"] = {
            "params": ["in buffer<bf16>", "out buffer<bf16>", "in buffer<bf16>", "in buffer<u64>", "out buffer<u64>", "in buffer<u64>", "i32", "i32",
                       "in buffer<bf16>", "out buffer<bf16>", "i32", "i32", "out buffer<f32>"],
            "impl": {"launches": [a, {
                "module": FUSED_SITU, "entry": "kern_k3g_rs_situ_rms",
                "params": ["in buffer<bf16>", "out buffer<bf16>", "in buffer<bf16>", "in buffer<u64>", "i32", "i32", "in buffer<bf16>",
                           "out buffer<bf16>", "i32", "i32", "i32", "i32", "out buffer<f32>"],
                "args": [{"param": 0}, {"param": 1}, {"param": 2}, {"param": 3}, {"rank": "tp"}, {"i32": 4}, {"param": 8}, {"param": 9}, {"i32": 6144},
                         {"param": 10}, {"i32": 3584}, {"param": 11}, {"param": 12}],
                # two block kinds, interleaved: one per latent row, one per 4096-element activation item (1.5 per row)
                "block": [128, 1, 1], "grid": [{"mul": [{"ceil_div": [{"mul": [B4, 3]}, 2]}, 2]}, 1, 1]}]}}
    for key in (FUSED_RES, FUSED_SITU, QUANT):
        _module(manifest, key, cubin_dir)
    # ---- the call list, layer by layer ---------------------------------------------------------------------------------
    by_layer = {}
    for c in calls:
        if "." in c["label"]:
            layer, what = c["label"].split(".", 1)
            by_layer.setdefault(layer, {})[what] = c
    drop, done = set(), {"layers_qkvg_quant": 0, "layers_res_mlp": 0, "layers_normed_quant": 0, "layers_shared_situ": 0}
    items = {"expr": {"ceil_div": [{"mul": [B4, 6144]}, 4096]}}
    for layer, c in by_layer.items():
        ri, qq = c.get("res_in"), c.get("qkvg_quant")
        if ri is not None and qq is not None and ri["op"] in ("attnres_rms_push_add2", "attnres_rms_push_add2_amax"):
            if ri["op"] == "attnres_rms_push_add2":
                ri["op"] = "attnres_rms_push_add2_amax"
                ri["args"] = ri["args"] + [{"buf": "rowmax_all"}, {"buf": "rowmax_all_peer"}]
            if qq["op"] == "quant_fp8_tensor":
                x, y, scale, _, n = qq["args"]
                qq["op"], qq["args"] = "quant_fp8_apply", [x, y, scale, {"buf": "rowmax_all"}, {"var": "tokens"}, n]
            done["layers_qkvg_quant"] += 1
        ra, rm = c.get("reduce_attn"), c.get("res_mlp")
        if rm is not None and rm["op"] == "rs_land_add_attnres_rms":
            done["layers_res_mlp"] += 1
        elif ra is not None and rm is not None and ra["op"] == "k3_reducescatter_bf16" and rm["op"] in NB_OPS:
            part, own, peer, flags, flags_peer, _count, units, slot, _order = ra["args"]
            la = rm["args"]
            assert la[0] == own, (layer, la[0], own)                  # the landing consumes exactly what the reduce-scatter produced
            stats = la[10:12] if len(la) >= 12 else [{"buf": "attn_stats"}, {"i32": 0}]
            rm["op"] = "rs_land_add_attnres_rms"
            rm["args"] = [part, peer, flags, flags_peer, units, slot] + la[1:10] + stats + [{"buf": "rowmax"}]
            drop.add(id(ra))
            done["layers_res_mlp"] += 1
        nq = c.get("normed_quant")
        if nq is not None and rm is not None and rm["op"] == "rs_land_add_attnres_rms":
            if nq["op"] == "quant_fp8_tensor":
                x, y, scale, _, n = nq["args"]
                nq["op"], nq["args"] = "quant_fp8_apply", [x, y, scale, {"buf": "rowmax"}, {"expr": B4}, n]
            done["layers_normed_quant"] += 1
        sm, ss, sq = c.get("scatter_moe"), c.get("shared_situ"), c.get("shared_act_quant")
        if ss is not None and ss["op"] == "rs_situ_rms":
            done["layers_shared_situ"] += 1
        elif sm is not None and ss is not None and sm["op"] == "k3_reducescatter_bf16" and ss["op"] == "land_situ_rms":
            part, own, peer, flags, flags_peer, _count, units, slot, _order = sm["args"]
            sp, act, lat, gam, ln, B, L = ss["args"]
            assert lat == own, (layer, lat, own)
            ss["op"], ss["args"] = "rs_situ_rms", [sp, act, part, peer, flags, flags_peer, units, slot, gam, ln, B, L, {"buf": "item_max"}]
            drop.add(id(sm))
            done["layers_shared_situ"] += 1
        if sq is not None and ss is not None and ss["op"] == "rs_situ_rms" and sq["op"] == "quant_fp8_tensor":
            x, y, scale, _, n = sq["args"]
            sq["op"], sq["args"] = "quant_fp8_apply", [x, y, scale, {"buf": "item_max"}, items, n]
    manifest["programs"]["prefill"]["calls"] = [c for c in calls if id(c) not in drop]
    calls = manifest["programs"]["prefill"]["calls"]
    for c in calls:                                                    # every call matches its op's parameter count
        assert len(c["args"]) == len(ops[c["op"]]["params"]), (c["label"], c["op"], len(c["args"]), len(ops[c["op"]]["params"]))
    done.update({"launches_before": before, "launches_after": launches(), "calls": len(calls)})
    return done


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("manifest")
    ap.add_argument("--out")
    ap.add_argument("--cubins", default=CUBIN_DIR)
    ap.add_argument("--keep-grids", action="store_true")
    ap.add_argument("--fuse", action="store_true", help="also rewrite programs.prefill.calls to the fused call list")
    a = ap.parse_args()
    m = json.load(open(a.manifest))
    s = patch(m, a.cubins, a.keep_grids)
    if a.fuse and not s["missing"]:
        f = fuse(m, a.cubins)
        print("fused call list: " + ", ".join("%s=%s" % kv for kv in f.items()))
    json.dump(m, open(a.out or a.manifest, "w"), indent=1)
    print("launches moved to b200 cubins: %d; left on reference modules: %d" % (len(s["moved"]), len(s["left"])))
    for op, entry, mod in s["moved"]:
        print("  moved  %-42s %-36s -> %s" % (op, entry, mod))
    for name, entry in s["missing"]:
        print("  MISSING entry %s in %s.cubin" % (entry, name))
    sys.exit(1 if s["missing"] else 0)


if __name__ == "__main__":
    main()
