"""Seeded inputs of the golden cases, and how each case is run on (a) the reference's own cubins
(oracle/_ref, GPU only), (b) the CPU oracle.  tests/golden/make_golden.py records (a) into
tests/golden/reference_outputs.npz; tests/test_golden.py checks (b) against the record on any
machine; tests/test_reference_ab.py re-runs (a) live on a GPU box and compares it with this library.

Every case names the reference module / entry / launch dims it uses (the default manifest's geometry).  `exact` lists the outputs that must match bit for bit; the others use approximate
device instructions in the reference (rsqrtf, expf, ex2.approx) and are compared at `ulp` bf16 ulps
on at most `frac` of the elements.
"""
import numpy as np

import k3o

MOE = "k3_moe_prefill_v4+EP_RANKS=4+EP_STRIDED=1+TILE_SHIFT=7+SCATTER_WARPS=16"


def _g(seed):
    return np.random.Generator(np.random.Philox(seed))


def _bf(g, shape, mean=0.0, std=1.0):
    return k3o.f32_to_bf16((g.standard_normal(shape, dtype=np.float32) * std + mean).astype(np.float32))


def inputs(name):
    g = _g({"k1b_nb0": 1, "k1b_nb3": 2, "k1a_nb2": 3, "k1c": 4, "moe_quant": 5, "quant_pair": 6, "router": 7, "route": 8, "rs_pull": 9,
            "mla_prep": 10, "span_gather": 11, "out_gate": 12, "push_add2": 13, "situ_rms": 14, "sigmoid_mul": 15,
            "land_situ": 16, "rms": 17, "argmax": 18, "push_first": 19, "copies": 20, "moe_shuffle": 21, "weight_prep": 22}[name])
    H = 7168
    if name in ("k1b_nb0", "k1b_nb3", "k1a_nb2"):
        B = 3
        return dict(partial=_bf(g, (B, H), std=0.5), prefix=_bf(g, (B, H)), blocks=_bf(g, (B, 8, H)),
                    sw=(g.standard_normal(H, dtype=np.float32) * 0.05).astype(np.float32), gamma=_bf(g, (H,), 1.0, 0.02))
    if name == "push_add2":
        B = 3
        return dict(blocks=_bf(g, (B, 8, H)), sw=(g.standard_normal(H, dtype=np.float32) * 0.05).astype(np.float32),
                    sw_mlp=(g.standard_normal(H, dtype=np.float32) * 0.05).astype(np.float32), gamma=_bf(g, (H,), 1.0, 0.02),
                    p1=_bf(g, (B, H), std=0.5), p2=_bf(g, (B, H), std=0.5), prefix2=_bf(g, (B, H)), partial=_bf(g, (B, H), std=0.5))
    if name == "situ_rms":
        return dict(sp=_bf(g, (6, 2 * 6144), std=3.0), lat=_bf(g, (6, 3584)), gam=_bf(g, (3584,), 1.0, 0.02))
    if name == "sigmoid_mul":
        return dict(attn=_bf(g, (9, 3072)), gate=_bf(g, (9, 3072), std=2.0))
    if name == "land_situ":
        return dict(p=(g.standard_normal((5, 2 * 1280), dtype=np.float32) * 3.0).astype(np.float32))
    if name == "rms":
        return dict(x=_bf(g, (6, 3584), std=2.0), gam=_bf(g, (3584,), 1.0, 0.02))
    if name == "argmax":
        x = g.standard_normal((3, 163840), dtype=np.float32)
        x[0, 70000] = 9.0; x[0, 163839] = 9.0                       # tie: the smaller index wins
        x[1, :] = -1.0; x[1, 5] = -0.5
        return dict(x=x)
    if name == "push_first":
        B = 3
        return dict(prefix=_bf(g, (B, H)), blocks=_bf(g, (B, 8, H)), sw=(g.standard_normal(H, dtype=np.float32) * 0.05).astype(np.float32),
                    gamma=_bf(g, (H,), 1.0, 0.02))
    if name == "weight_prep":
        return dict(q=g.standard_normal((256, 4), dtype=np.float32), k=g.standard_normal((256, 4), dtype=np.float32),
                    v=g.standard_normal((256, 4), dtype=np.float32), norm=_bf(g, (512,)), proj=_bf(g, (512,)), b=_bf(g, (24, 64)), fa=_bf(g, (128, 64)),
                    raw=g.integers(0, 256, (2, 256, 8), dtype=np.uint8), wkv=_bf(g, (2 * 256, 512)))
    if name == "moe_shuffle":
        return dict(w=g.integers(0, 256, (3, 128, 48), dtype=np.uint8), sf=g.integers(0, 256, (3, 256, 12), dtype=np.uint8))
    if name == "copies":
        return dict(src=_bf(g, (11, 7168)), table=_bf(g, (40, 7168)), ids=g.integers(0, 40, 9).astype(np.int64),
                    seq=np.array([12345], np.int32))
    if name == "k1c":
        B = 3
        return dict(p1=g.standard_normal((B, H), dtype=np.float32), p2=g.standard_normal((B, H), dtype=np.float32), prefix2=_bf(g, (B, H)))
    if name == "moe_quant":
        x = _bf(g, (8, 3584), std=3.0)
        x[0, :32] = 0
        x[1] = k3o.f32_to_bf16(np.full(3584, 7.0 * 2.0 ** 9, np.float32))
        x[2] = k3o.f32_to_bf16(np.full(3584, 1.0e-38, np.float32))
        return dict(x=x)
    if name == "quant_pair":
        return dict(x=_bf(g, (7168 * 4 + 3,), std=2.0))
    if name == "router":
        return dict(S=g.standard_normal((96, 224), dtype=np.float32), bias=(g.standard_normal(224, dtype=np.float32) * 0.1).astype(np.float32),
                    rs=k3o.f32_to_bf16(np.array([2.5], np.float32)))
    if name == "route":
        T = 700
        ids = np.stack([g.permutation(224)[:16] for _ in range(T)]).astype(np.int32)
        tabs = k3o.moe_route(ids, 1, 56, 4, 1, 128)
        rows = int(tabs["total_padded"][0])
        return dict(ids=ids, fc2=_bf(g, (rows, 256)), wts=g.random((T, 16), dtype=np.float32))
    if name == "rs_pull":
        count = 7168 * 2
        return dict(**{"partial%d" % r: _bf(g, (4 * count,), std=0.125) for r in range(4)})
    if name == "mla_prep":
        B = 9
        slots = np.array([5, 64, -1, 0, 130, 63, 7, -1, 129], np.int64)
        return dict(partial=g.standard_normal((B, 5184), dtype=np.float32), gq=_bf(g, (1536,), 1.0, 0.02), gkv=_bf(g, (512,), 1.0, 0.02),
                    slots=slots, slab=_bf(g, (3 * 64 * 576 * 2,)))
    if name == "span_gather":
        rows, inner = 24, 3072
        return dict(partial=_bf(g, (rows, 4 * inner)), cw=(g.standard_normal((3, 4, inner), dtype=np.float32) * 0.5).astype(np.float32),
                    win=_bf(g, (3, 3, inner)), wsm=g.standard_normal((rows, 256), dtype=np.float32))
    if name == "out_gate":
        rows, inner = 12, 3072
        return dict(attn=_bf(g, (10, inner)), gate=_bf(g, (rows, 4 * inner)), gamma_o=(1 + 0.1 * g.standard_normal(128, dtype=np.float32)).astype(np.float32))
    raise KeyError(name)


NAMES = ["weight_prep", "moe_shuffle", "land_situ", "rms", "argmax", "push_first", "copies", "situ_rms", "sigmoid_mul", "push_add2", "k1b_nb0", "k1b_nb3", "k1a_nb2", "k1c", "moe_quant", "quant_pair", "router", "route", "rs_pull", "mla_prep", "span_gather", "out_gate"]

# outputs that must be bit-identical between the reference cubin and the CPU oracle
EXACT = {
    "land_situ": [], "rms": [], "argmax": ["out"], "push_first": ["blocks"],
    "copies": ["rank_rows", "zero_rows", "lens", "embedding", "last_row"], "moe_shuffle": ["w_plain", "w_gated", "sf_plain", "sf_gated"],
    "weight_prep": ["cw", "sw", "wsm", "sf_pack", "sf_pack_interleaved", "kvb_aug"],
    "situ_rms": [], "sigmoid_mul": [],
    "push_add2": ["hidden", "blocks", "res_mlp_prefix2"],
    "k1b_nb0": ["prefix2"], "k1b_nb3": ["prefix2"], "k1a_nb2": ["blocks"], "k1c": ["hidden"], "moe_quant": ["q", "sf"],
    "quant_pair": ["y", "scale"], "router": [], "route": ["blockcount", "blockoff", "cta_batch", "cta_limit", "num_non_exiting", "total_padded",
                                                           "route_map", "exp2perm", "finalize"],
    "rs_pull": ["dst0", "dst1", "dst2", "dst3"], "mla_prep": ["gate"], "span_gather": ["win", "beta", "flow"], "out_gate": [],
}
# bf16 outputs compared at tolerance: name -> (max ulp, max fraction of differing elements)
TOLERANT = {
    "weight_prep": {"cos": (1, 0.05), "sin": (1, 0.05)},
    "land_situ": {"act": (2, 0.2)}, "rms": {"o": (1, 2e-3)}, "push_first": {"normed_all": (1, 2e-3)},
    "situ_rms": {"act": (2, 0.2), "ln": (1, 2e-3)}, "sigmoid_mul": {"out": (1, 5e-3)},
    "push_add2": {"normed_all": (4, 5e-3), "res_mlp_normed": (4, 5e-3)},   # mixed rows: a cancelling mix amplifies the 1e-7 softmax difference
    "k1b_nb0": {"normed": (1, 2e-3)}, "k1b_nb3": {"normed": (2, 5e-3)}, "k1a_nb2": {"normed": (2, 5e-3)},
    "mla_prep": {"q_norm": (1, 2e-3), "slab": (1, 2e-3)}, "span_gather": {"q": (1, 5e-3), "k": (1, 5e-3), "v": (1, 5e-3)},
    "out_gate": {"gated": (1, 1e-2)},
}


def run_oracle(name, inp):
    """CPU oracle outputs as a dict of numpy arrays (eps and constants as the reference builds them)."""
    if name == "situ_rms":
        act, ln = k3o.situ_rms(inp["sp"], inp["lat"], inp["gam"], 6144, 3584)
        return dict(act=act, ln=ln)
    if name == "land_situ":
        return dict(act=k3o.land_situ(inp["p"], 1280))
    if name == "rms":
        return dict(o=k3o.rms(inp["x"], inp["gam"]))
    if name == "argmax":
        return dict(out=k3o.argmax_f32(inp["x"]))
    if name == "push_first":
        # first layer: nb = 0, snapshot = 1, rank 1 of 4 (manifest op attnres_rms_push_first_v3)
        blocks = inp["blocks"].copy()
        normed = k3o.attnres_rms(inp["prefix"], blocks, inp["sw"], inp["gamma"], 0, 1, 1e-5)
        B, H = normed.shape
        normed_all = np.zeros((4 * B, H), np.uint16)
        normed_all[B:2 * B] = normed
        return dict(blocks=blocks, normed_all=normed_all)
    if name == "weight_prep":
        cos, sin = k3o.rope_table(64, 32, 50000.0)
        return dict(cw=k3o.conv_taps(inp["q"], inp["k"], inp["v"]), sw=k3o.scoring(inp["norm"], inp["proj"]), wsm=k3o.wsm(inp["b"], inp["fa"], 24),
                    sf_pack=k3o.mega_sf_pack(inp["raw"], 0), sf_pack_interleaved=k3o.mega_sf_pack(inp["raw"], 1), kvb_aug=k3o.kvb_aug(inp["wkv"], 2),
                    cos=cos, sin=sin)
    if name == "moe_shuffle":
        return dict(w_plain=k3o.moe_w_shuffle(inp["w"], 0), w_gated=k3o.moe_w_shuffle(inp["w"], 1),
                    sf_plain=k3o.moe_sf_shuffle(inp["sf"], 0), sf_gated=k3o.moe_sf_shuffle(inp["sf"], 1))
    if name == "copies":
        return dict(rank_rows=k3o.rank_rows(inp["src"], 2, 4), zero_rows=k3o.zero_rows(inp["src"], 3, 9), lens=k3o.fmha_lens(inp["seq"], 4096),
                    embedding=k3o.embedding(inp["ids"], inp["table"]), last_row=inp["src"][10].copy())
    if name == "sigmoid_mul":
        return dict(out=k3o.sigmoid_mul(inp["attn"], inp["gate"], 24, 128, 3072, 128))
    if name == "push_add2":
        # res_in (push, nb = 3, snapshot, two partials, rank 1 of 4) followed by res_mlp (nb = 4) fed with its statistics
        blocks = inp["blocks"].copy()
        hidden, normed, stats = k3o.attnres_rms_push(blocks, inp["sw"], inp["gamma"], 3, 1, inp["sw_mlp"], inp["p1"], inp["p2"], inp["prefix2"], 1, 1e-5)
        B, H = hidden.shape
        normed_all = np.zeros((4 * B, H), np.uint16)
        normed_all[B:2 * B] = normed
        p2, n2 = k3o.land_add_attnres_rms_stats(inp["partial"], hidden, blocks, inp["sw_mlp"], inp["gamma"], 4, 0, 1e-5, stats, 3)
        return dict(hidden=hidden, blocks=blocks, normed_all=normed_all, stats=stats, res_mlp_prefix2=p2, res_mlp_normed=n2)
    if name in ("k1b_nb0", "k1b_nb3"):
        nb = 0 if name == "k1b_nb0" else 3
        p2, n = k3o.land_add_attnres_rms(inp["partial"], inp["prefix"], inp["blocks"], inp["sw"], inp["gamma"], nb, 0, 1e-5)
        return dict(prefix2=p2, normed=n)
    if name == "k1a_nb2":
        blocks = inp["blocks"].copy()
        n = k3o.attnres_rms(inp["prefix"], blocks, inp["sw"], inp["gamma"], 2, 1, 1e-5)
        return dict(blocks=blocks, normed=n)
    if name == "k1c":
        return dict(hidden=k3o.land_add2(inp["p1"], inp["p2"], inp["prefix2"], 1))
    if name == "moe_quant":
        q, sf = k3o.moe_quant(inp["x"])
        return dict(q=q, sf=sf)
    if name == "quant_pair":
        y, sc = k3o.quant_fp8_tensor(inp["x"])
        return dict(y=y, scale=sc)
    if name == "router":
        idx, w = k3o.router_topk(inp["S"], inp["bias"], inp["rs"], 16)
        return dict(idx=idx, wts=w)
    if name == "route":
        t = k3o.moe_route(inp["ids"], 1, 56, 4, 1, 128)
        t["finalize"] = k3o.moe_finalize(inp["fc2"], t["exp2perm"], inp["wts"], inp["ids"].shape[0], 256)
        return t
    if name == "rs_pull":
        parts = [inp["partial%d" % r] for r in range(4)]
        return {"dst%d" % r: k3o.rs_pull(parts, r, 6) for r in range(4)}
    if name == "mla_prep":
        slab = inp["slab"].copy()
        q = k3o.mla_prep_head(inp["partial"], inp["gq"], inp["gkv"], inp["slots"], slab, 64 * 576, 64 * 576 * 2, 1e-5)
        return dict(q_norm=q, slab=slab, gate=k3o.mla_prep_gate(inp["partial"], 3072))
    if name == "span_gather":
        q, k, v, win = k3o.span_conv_silu(inp["partial"], 4 * 3072, inp["cw"], inp["win"], 3072, 2, 20)
        beta, flow = k3o.span_beta_flow(inp["wsm"], 24, 2, 20)
        return dict(q=q, k=k, v=v, win=win, beta=beta, flow=flow)
    if name == "out_gate":
        gated, _, _ = k3o.kda_out_gate(inp["attn"], inp["gate"], 4 * 3072, 3 * 3072, inp["gamma_o"], 24, 2, 10, 12, 1e-5)
        return dict(gated=gated)
    raise KeyError(name)
