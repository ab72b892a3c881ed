"""The manifest patcher: launches of kernels this library provides are repointed at its cubins, with
entry names, parameter lists and argument mappings untouched; everything else is left alone."""
import copy
import json
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "kern-k3_b200"))
REF_MANIFEST = os.path.join(os.environ.get("K3_REFERENCE_ROOT", os.path.join(os.path.dirname(ROOT), "reference")), "manifests", "k3-tp4-prefill-16k.json")


@pytest.fixture(scope="module")
def pm():
    if not os.path.isdir(os.path.join(ROOT, "kern-k3_b200", "lib", "cubin")):
        import build
        build.build()
    import patch_manifest
    return patch_manifest


def _mini():
    return {
        "modules": {"k3_router_argmax": {"source": "x", "sha256": "0"}, "k3_moe_prefill_v3+EP_STRIDED=1": {"source": "y", "sha256": "1"},
                    "k3_rs_arrive_v2": {"source": "z", "sha256": "2"}, "gemm": {"source": "g", "sha256": "3"}},
        "ops": {
            "router_topk": {"params": ["in buffer<f32>"], "impl": {"launches": [
                {"module": "k3_router_argmax", "entry": "kern_k3_router_topk", "block": [256, 1, 1], "grid": [{"ceil_div": ["tokens", 4]}, 1, 1]}]}},
            "argmax": {"impl": {"launches": [{"module": "k3_router_argmax", "entry": "kern_k3_decode_only", "block": [1024, 1, 1], "grid": [1, 64, 1]}]}},
            "moe_quant": {"impl": {"launches": [{"module": "k3_moe_prefill_v3+EP_STRIDED=1", "entry": "kern_k3_moe_quant", "block": [256, 1, 1],
                                                 "grid": [7, 1, 1], "args": [{"param": 0}, {"i32": 3584}]}]}},
            "k3_allgather_push": {"impl": {"launches": [{"module": "k3_rs_arrive_v2", "entry": "kern_k3_rs_arrive1", "block": [32, 1, 1], "grid": [1, 1, 1],
                                                         "args": [{"param": 0}, {"rank": "tp"}]}]}},
            "gemm_bf16": {"impl": {"launches": [{"module": "gemm", "entry": "extern:cublas", "block": [1, 1, 1], "grid": [1, 1, 1]}]}},
        },
    }


def test_patch_small_manifest(pm):
    m = _mini()
    before = copy.deepcopy(m)
    s = pm.patch(m)
    assert not s["missing"]
    l = m["ops"]["router_topk"]["impl"]["launches"][0]
    assert l["module"] == "b200/k3_router_argmax" and l["entry"] == "kern_k3_router_topk"
    assert l["grid"] != before["ops"]["router_topk"]["impl"]["launches"][0]["grid"]           # better geometry applied
    assert m["ops"]["argmax"]["impl"]["launches"][0]["module"] == "k3_router_argmax"          # not ours: untouched
    assert "k3_router_argmax" in m["modules"]                                                 # still referenced by argmax
    q = m["ops"]["moe_quant"]["impl"]["launches"][0]
    assert q["module"] == "b200/k3_quant_fp8_pair_v2" and q["args"] == before["ops"]["moe_quant"]["impl"]["launches"][0]["args"]
    assert "k3_moe_prefill_v3+EP_STRIDED=1" not in m["modules"]                               # no launch left on it
    assert m["ops"]["k3_allgather_push"]["impl"]["launches"][0]["args"] == [{"param": 0}, {"rank": "tp"}]
    assert m["ops"]["gemm_bf16"] == before["ops"]["gemm_bf16"]
    sha = m["modules"]["b200/k3_router_argmax"]["sha256"]
    assert len(sha) == 64 and sha == pm.sha256(os.path.join(pm.CUBIN_DIR, "k3_router_argmax.cubin"))
    again = copy.deepcopy(m)
    pm.patch(again)
    assert again == m                                                                         # idempotent
    keep = _mini()
    pm.patch(keep, keep_grids=True)
    assert keep["ops"]["router_topk"]["impl"]["launches"][0]["grid"] == before["ops"]["router_topk"]["impl"]["launches"][0]["grid"]


@pytest.mark.skipif(not os.path.exists(REF_MANIFEST), reason="reference checkout not present")
def test_patch_reference_default_manifest(pm):
    m = json.load(open(REF_MANIFEST))
    calls = m["programs"]["prefill"]["calls"]
    s = pm.patch(m)
    assert not s["missing"]
    moved_ops = {op for op, _, _ in s["moved"]}
    for op in ("attnres_rms_push_add2", "k3_reducescatter_bf16", "k3_allgather4_push", "k3_allgather_push", "quant_fp8_tensor", "router_topk",
               "moe_quant", "moe_route_count", "moe_route_tables", "moe_route_scatter", "moe_finalize", "mla_prep", "span_gather_v2",
               "kda_out_gate_v2", "k3_epoch_bump"):
        assert op in moved_ops, op
    assert any(op.startswith("land_add_attnres_rms_bf16_v2_nb") for op in moved_ops)
    # share of the prefill program's calls that now run on this library's kernels
    n = sum(1 for c in calls if c["op"] in moved_ops)
    assert n > 0.5 * len(calls), (n, len(calls))
    # every launch the prefill program still makes on a reference module is a GEMM, an attention kernel or FlashKDA
    for c in calls:
        for l in m["ops"][c["op"]]["impl"]["launches"]:
            if not str(l.get("module", "")).startswith("b200/"):
                assert str(l.get("entry", l.get("extern", ""))).startswith(("extern:", "bmm_", "fmha", "_Z22_flash_kda", "_Z25_flash_kda")), (c["op"], l["entry"][:60])
    for _, entry, mod in s["moved"]:
        blob = open(os.path.join(pm.CUBIN_DIR, mod[len("b200/"):] + ".cubin"), "rb").read()
        assert entry.encode() + b"\0" in blob


@pytest.mark.skipif(not os.path.exists(REF_MANIFEST), reason="reference checkout not present")
def test_fuse_reference_default_manifest(pm):
    """--fuse on the reference's default manifest: 185 calls and 437 launches fewer (per fused layer: the two
    reduce-scatter calls folded into their consumers, three amax launches dropped), every rewritten call matches its op
    record, the new entries exist in the cubins, nothing but the glue calls moves, and a second run changes nothing."""
    m = json.load(open(REF_MANIFEST))
    ref_calls = copy.deepcopy(m["programs"]["prefill"]["calls"])
    assert not pm.patch(m)["missing"]
    launches_before = sum(len(m["ops"][c["op"]]["impl"]["launches"]) for c in m["programs"]["prefill"]["calls"])
    f = pm.fuse(m)
    calls = m["programs"]["prefill"]["calls"]
    assert f["launches_before"] == launches_before == 3455 and len(ref_calls) == 2923
    assert f["layers_res_mlp"] == 93 and f["layers_shared_situ"] == 92 and f["layers_normed_quant"] == 92 and f["layers_qkvg_quant"] == 68
    assert len(calls) == len(ref_calls) - 93 - 92
    assert f["launches_after"] == launches_before - 2 * 93 - 2 * 92 - 68 + 93 + 92 - 92 - 92 == 3018
    labels = [c["label"] for c in calls]
    assert not any(l.endswith((".reduce_attn", ".scatter_moe")) for l in labels)
    kept = [c for c in ref_calls if not c["label"].endswith((".reduce_attn", ".scatter_moe"))]
    assert labels == [c["label"] for c in kept]                                              # order and everything else untouched
    changed = {"attnres_rms_push_add2_amax", "quant_fp8_apply", "rs_land_add_attnres_rms", "rs_situ_rms"}
    for new, old in zip(calls, kept):
        if new["op"] not in changed:
            assert new == old, new["label"]
        assert len(new["args"]) == len(m["ops"][new["op"]]["params"])
    for op in changed:
        for l in m["ops"][op]["impl"]["launches"]:
            assert l["module"].startswith("b200/") and l["module"] in m["modules"]
            blob = open(os.path.join(pm.CUBIN_DIR, l["module"][len("b200/"):] + ".cubin"), "rb").read()
            assert l["entry"].encode() + b"\0" in blob, l["entry"]
            assert len(l["args"]) == len(l["params"])
    for name in ("rowmax_all", "rowmax_all_peer", "rowmax", "item_max"):
        assert name in m["buffers"]
    assert m["buffers"]["rowmax_all"]["export"] is True and m["buffers"]["rowmax_all_peer"]["of"] == "rowmax_all"
    # the landing keeps its statistics hand-off: layers whose landing read attn_stats still do, with the same count
    for new, old in zip(calls, kept):
        if new["op"] == "rs_land_add_attnres_rms" and len(old["args"]) == 12:
            assert new["args"][15:17] == old["args"][10:12]
    again = copy.deepcopy(m)
    f2 = pm.fuse(again)
    assert again == m and f2["launches_after"] == f["launches_after"]
