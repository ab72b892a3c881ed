"""Record the outputs of the reference's own kernels (oracle/_ref/*.cubin, compiled for sm_100a by
oracle/build_ref.py from the reference checkout) on the seeded inputs of tests/golden/cases.py.

Runs on a GPU box:   python tests/golden/make_golden.py [out.npz]
The result is committed as tests/golden/reference_outputs.npz; tests/test_golden.py checks the CPU
oracle against it without a GPU.  `run_reference` is also used live by tests/test_reference_ab.py.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
for p in (os.path.join(ROOT, "oracle"), os.path.join(ROOT, "tests"), HERE):
    if p not in sys.path:
        sys.path.insert(0, p)
import cases  # noqa: E402
import refcubin  # noqa: E402
from refcubin import I64  # noqa: E402


def _up(a, dev):
    import torch
    if a.dtype == np.uint16:
        return torch.from_numpy(a.view(np.int16).copy()).to(dev).view(torch.bfloat16)
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev)


def _bits(t):
    import torch
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


def run_reference(name, inp, dev):
    """Launch the reference's kernels with the manifest's block sizes; returns numpy outputs."""
    import torch
    bf = torch.bfloat16
    z = lambda shape, dt: torch.zeros(shape, dtype=dt, device=dev)
    if name == "land_situ":
        B, n = inp["p"].shape[0], 1280
        act = z((B, n), bf)
        refcubin.run("k3_land", "kern_k3_land_situ", (B, (n + 1023) // 1024), 1024, [_up(inp["p"], dev), act, n, B])
        torch.cuda.synchronize()
        return dict(act=_bits(act))
    if name == "rms":
        B, h = inp["x"].shape
        o = z((B, h), bf)
        refcubin.run("k3_land", "kern_k3_rms", B, 1024, [_up(inp["x"], dev), _up(inp["gam"], dev), o, h, B])
        torch.cuda.synchronize()
        return dict(o=_bits(o))
    if name == "argmax":
        B, n = inp["x"].shape
        pmax, pidx, out = z((B, 64), torch.float32), z((B, 64), torch.int32), z((B,), torch.int64)
        refcubin.run("k3_router_argmax", "kern_k3_argmax_f32_partial", (B, 64), 1024, [_up(inp["x"], dev), pmax, pidx, n])
        refcubin.run("k3_router_argmax", "kern_k3_argmax_f32_final", B, 64, [pmax, pidx, out, 64])
        torch.cuda.synchronize()
        return dict(out=out.cpu().numpy())
    if name == "push_first":
        B, H = inp["prefix"].shape
        blocks = _up(inp["blocks"], dev)
        normed_all = z((4 * B, H), bf)
        others = [z((4 * B, H), bf) for _ in range(3)]
        tab = torch.tensor([others[0].data_ptr(), normed_all.data_ptr(), others[1].data_ptr(), others[2].data_ptr()], dtype=torch.int64, device=dev)
        refcubin.run("k3_residual_push_v3", "kern_k3_attnres_rms_push", B, 128,
                     [_up(inp["prefix"], dev), blocks, _up(inp["sw"], dev), _up(inp["gamma"], dev), normed_all, tab, 0, 1, B, 1, 4])
        torch.cuda.synchronize()
        for o in others:
            assert torch.equal(o, normed_all)
        return dict(blocks=_bits(blocks), normed_all=_bits(normed_all))
    if name == "weight_prep":
        cw = z((3, 4, 256), torch.float32)
        refcubin.run("k3_weight_prep", "kern_k3_conv_taps", 1, 256, [_up(inp["q"], dev), _up(inp["k"], dev), _up(inp["v"], dev), cw, 256])
        sw = z((512,), torch.float32)
        refcubin.run("k3_weight_prep", "kern_k3_scoring", 2, 256, [_up(inp["norm"], dev), _up(inp["proj"], dev), sw, 512])
        wsm = z((256, 64), bf)
        refcubin.run("k3_weight_prep", "kern_k3_wsm", 64, 256, [_up(inp["b"], dev), _up(inp["fa"], dev), wsm, 24, 64])
        raw = _up(inp["raw"], dev)
        packs = []
        for il in (0, 1):
            o = z((2, 2, 256), torch.int32)
            refcubin.run("k3_weight_prep", "kern_k3_mega_sf_pack", 4, 256, [raw, o, 2, 256, 8, il])
            packs.append(o)
        aug = z((2 * 320, 576), bf)
        refcubin.run("k3_weight_prep", "kern_k3_kvb_aug", (2 * 320 * 576 + 255) // 256, 256, [_up(inp["wkv"], dev), aug, 2 * 320 * 576])
        cs = z((64, 64), bf)
        refcubin.run("weight_prep", "kern_rope_table_bf16", 64, 32, [cs, cs.view(-1)[32:], 64, 32, 64, 50000.0])
        torch.cuda.synchronize()
        csb = _bits(cs)
        return dict(cw=cw.cpu().numpy(), sw=sw.cpu().numpy(), wsm=_bits(wsm), sf_pack=packs[0].cpu().numpy(), sf_pack_interleaved=packs[1].cpu().numpy(),
                    kvb_aug=_bits(aug), cos=np.ascontiguousarray(csb[:, :32]), sin=np.ascontiguousarray(csb[:, 32:]))
    if name == "moe_shuffle":
        w, sf = _up(inp["w"], dev), _up(inp["sf"], dev)
        res = {}
        for gated in (0, 1):
            dw, dsf = torch.zeros_like(w), torch.zeros_like(sf)
            e, n, rb = inp["w"].shape
            refcubin.run(cases.MOE, "kern_k3_moe_w_shuffle", (e * n * (rb // 16) + 255) // 256, 256, [w, dw, e, n, rb, gated])
            e, n, kg = inp["sf"].shape
            refcubin.run(cases.MOE, "kern_k3_moe_sf_shuffle", (e * n * kg + 255) // 256, 256, [sf, dsf, e, n, kg, gated])
            torch.cuda.synchronize()
            tag = "gated" if gated else "plain"
            res["w_" + tag], res["sf_" + tag] = dw.cpu().numpy(), dsf.cpu().numpy()
        return res
    if name == "copies":
        src, table = _up(inp["src"], dev), _up(inp["table"], dev)
        rr = z((4, 7168), bf)
        refcubin.run("k3_prefill", "kern_k3_rank_rows", 4, 256, [rr, src, 2, 4, 14336, 11])
        zr = src.clone()
        refcubin.run("k3_prefill", "kern_k3_zero_rows", 1, 1024, [zr, 14336, 3, 9])
        lens = torch.full((8,), -1, dtype=torch.int32, device=dev)
        refcubin.run("k3_prefill", "kern_k3_fmha_lens", 1, 32, [_up(inp["seq"], dev), lens, 4096])
        emb = z((9, 7168), bf)
        refcubin.run("embedding", "kern_embedding_i64_bf16", 9, 256, [_up(inp["ids"], dev), table, emb, 9, 7168])
        last = z((7168,), bf)
        refcubin.run("copy_rows", "kern_last_row_bf16", 1, 1024, [last, src, 7168, 7168, 11])
        torch.cuda.synchronize()
        return dict(rank_rows=_bits(rr), zero_rows=_bits(zr), lens=lens.cpu().numpy(), embedding=_bits(emb), last_row=_bits(last))
    if name == "situ_rms":
        B, n, h = inp["sp"].shape[0], 6144, 3584
        act, ln = z((B, n), bf), z((B, h), bf)
        refcubin.run("k3_land_fused", "kern_k3_situ_rms_bf16", 3 * ((4 * B + 15) // 16), 512,
                     [_up(inp["sp"], dev), act, _up(inp["lat"], dev), _up(inp["gam"], dev), ln, n, B, h, B])
        torch.cuda.synchronize()
        return dict(act=_bits(act), ln=_bits(ln))
    if name == "sigmoid_mul":
        T = inp["attn"].shape[0]
        out = z((T, 3072), bf)
        refcubin.run("sigmoid_mul", "kern_sigmoid_mul_bf16", (T, 2), 256, [out, _up(inp["attn"], dev), _up(inp["gate"], dev), 24, 128, 3072, 128])
        torch.cuda.synchronize()
        return dict(out=_bits(out))
    if name == "push_add2":
        B, H = inp["prefix2"].shape
        blocks, hidden = _up(inp["blocks"], dev), z((B, H), bf)
        normed_all = z((4 * B, H), bf)
        others = [z((4 * B, H), bf) for _ in range(3)]      # the three peers' copies, on this GPU
        tab = torch.tensor([others[0].data_ptr(), normed_all.data_ptr(), others[1].data_ptr(), others[2].data_ptr()], dtype=torch.int64, device=dev)
        stats = z((B, 8, 2), torch.float32)
        refcubin.run("k3_residual_push_add2", "kern_k3_attnres_rms_push", B, 128,
                     [blocks, _up(inp["sw"], dev), _up(inp["gamma"], dev), normed_all, tab, 3, 1, B, 1, 4, _up(inp["sw_mlp"], dev), stats,
                      _up(inp["p1"], dev), _up(inp["p2"], dev), _up(inp["prefix2"], dev), hidden, 1])
        torch.cuda.synchronize()
        for o in others:
            assert torch.equal(o, normed_all)                # every rank's copy received the same slice
        p2, n2 = z((B, H), bf), z((B, H), bf)
        refcubin.run("k3_residual_nb_stats", "kern_k3_land_add_attnres_rms_nb4", B, 128,
                     [_up(inp["partial"], dev), hidden, blocks, _up(inp["sw_mlp"], dev), _up(inp["gamma"], dev), p2, n2, 4, 0, B, stats, 3])
        torch.cuda.synchronize()
        return dict(hidden=_bits(hidden), blocks=_bits(blocks), normed_all=_bits(normed_all), stats=stats.cpu().numpy(),
                    res_mlp_prefix2=_bits(p2), res_mlp_normed=_bits(n2))
    if name in ("k1b_nb0", "k1b_nb3"):
        nb = 0 if name == "k1b_nb0" else 3
        B, H = inp["partial"].shape
        p2, n = z((B, H), bf), z((B, H), bf)
        refcubin.run("k3_residual_v2+LAND_BF16=1", "kern_k3_land_add_attnres_rms", B, 128,
                     [_up(inp["partial"], dev), _up(inp["prefix"], dev), _up(inp["blocks"], dev), _up(inp["sw"], dev), _up(inp["gamma"], dev), p2, n, nb, 0, B])
        torch.cuda.synchronize()
        return dict(prefix2=_bits(p2), normed=_bits(n))
    if name == "k1a_nb2":
        B, H = inp["prefix"].shape
        blocks, n = _up(inp["blocks"], dev), z((B, H), bf)
        refcubin.run("k3_residual_v2", "kern_k3_attnres_rms", B, 128, [_up(inp["prefix"], dev), blocks, _up(inp["sw"], dev), _up(inp["gamma"], dev), n, 2, 1, B])
        torch.cuda.synchronize()
        return dict(blocks=_bits(blocks), normed=_bits(n))
    if name == "k1c":
        B, H = inp["prefix2"].shape
        h = z((B, H), bf)
        refcubin.run("k3_residual_v2", "kern_k3_land_add2", B, 128, [_up(inp["p1"], dev), _up(inp["p2"], dev), _up(inp["prefix2"], dev), h, 1, B])
        torch.cuda.synchronize()
        return dict(hidden=_bits(h))
    if name == "moe_quant":
        rows, cols = inp["x"].shape
        q, sf = z((rows, cols), torch.uint8), z((rows, cols // 32), torch.uint8)
        refcubin.run(cases.MOE, "kern_k3_moe_quant", (rows * cols // 32 + 255) // 256, 256, [_up(inp["x"], dev), q, sf, rows, cols])
        torch.cuda.synchronize()
        return dict(q=q.cpu().numpy(), sf=sf.cpu().numpy())
    if name == "quant_pair":
        n = inp["x"].size
        x, y, part, sc = _up(inp["x"], dev), z((n,), torch.uint8), z((2048,), torch.float32), z((1,), torch.float32)
        refcubin.run("k3_quant_fp8_pair_v2", "kern_quant_fp8_amax_v2", 2048, 256, [x, n, part])
        refcubin.run("k3_quant_fp8_pair_v2", "kern_quant_fp8_apply_v2", 2048, 256, [x, y, n, part, 2048, sc])
        torch.cuda.synchronize()
        return dict(y=y.cpu().numpy(), scale=sc.cpu().numpy())
    if name == "router":
        B = inp["S"].shape[0]
        idx, w = z((B, 16), torch.int32), z((B, 16), torch.float32)
        refcubin.run("k3_router_argmax", "kern_k3_router_topk", B, 256, [_up(inp["S"], dev), _up(inp["bias"], dev), _up(inp["rs"], dev), idx, w, B])
        torch.cuda.synchronize()
        return dict(idx=idx.cpu().numpy(), wts=w.cpu().numpy())
    if name == "route":
        ids = _up(inp["ids"], dev)
        T, E, tile = inp["ids"].shape[0], 56, 128
        blocks = (T + 255) // 256
        nct = (T * 16 + tile - 1) // tile + E
        bc, bo = z((blocks, E), torch.int32), z((blocks, E), torch.int32)
        neg = lambda n: torch.full((n,), -1, dtype=torch.int32, device=dev)
        cb, cl, rm = neg(nct), neg(nct), neg(nct * tile)
        nne, tot = z((1,), torch.int32), z((1,), torch.int32)
        e2p = z((T, 16), torch.int32)
        refcubin.run(cases.MOE, "kern_k3_moe_route_count", blocks, 256, [ids, T, 1, E, bc])
        refcubin.run(cases.MOE, "kern_k3_moe_route_tables", 1, 1024, [bc, blocks, E, tile, bo, cb, cl, nne, tot, rm])
        refcubin.run(cases.MOE, "kern_k3_moe_route_scatter", blocks, 512, [ids, bo, T, 1, E, rm, e2p])
        out = z((T, 256), bf)
        refcubin.run(cases.MOE, "kern_k3_moe_finalize", (T + 1) // 2, 128, [_up(inp["fc2"], dev), e2p, _up(inp["wts"], dev), out, T, 256])
        torch.cuda.synchronize()
        c = lambda t: t.cpu().numpy()
        return dict(blockcount=c(bc), blockoff=c(bo), cta_batch=c(cb), cta_limit=c(cl), num_non_exiting=c(nne), total_padded=c(tot),
                    route_map=c(rm), exp2perm=c(e2p), finalize=_bits(out))
    if name == "rs_pull":
        parts = [_up(inp["partial%d" % r], dev) for r in range(4)]
        tab = torch.tensor([p.data_ptr() for p in parts], dtype=torch.int64, device=dev)
        count = parts[0].numel() // 4
        res = {}
        for r in range(4):
            dst = z((count,), bf)
            refcubin.run("k3_reducescatter_pull_nr4", "kern_k3_rs_pull", 4, 1024, [parts[r], dst, tab, None, None, I64(count), 0, 6, r, 4])
            torch.cuda.synchronize()
            res["dst%d" % r] = _bits(dst)
        return res
    if name == "mla_prep":
        B = inp["partial"].shape[0]
        part, slab = _up(inp["partial"], dev), _up(inp["slab"], dev)
        qn, gate = z((B, 1536), bf), z((B, 3072), bf)
        mod = "k3_mla_prep_v2+INNER=3072+MLA_FUSED=5184"
        refcubin.run(mod, "kern_k3_mla_prep_head", (B + 3) // 4, 512, [part, _up(inp["gq"], dev), _up(inp["gkv"], dev), _up(inp["slots"], dev), slab,
                                                                      I64(64 * 576), I64(64 * 576 * 2), qn, B])
        refcubin.run(mod, "kern_k3_mla_prep_gate", (B + 3) // 4, 384, [part, gate, B])
        torch.cuda.synchronize()
        return dict(q_norm=_bits(qn), slab=_bits(slab), gate=_bits(gate))
    if name == "span_gather":
        inner, at, span = 3072, 2, 20
        rec = 24 * 128 * 128 * 4
        line = torch.zeros(rec + 3 * 3 * inner * 2, dtype=torch.uint8, device=dev)
        line[rec:] = _up(inp["win"], dev).view(torch.uint8).reshape(-1)
        line_index = z((inp["partial"].shape[0],), torch.int32)
        span_at = torch.tensor([at], dtype=torch.int32, device=dev)
        q, k, v = z((span, inner), bf), z((span, inner), bf), z((span, inner), bf)
        beta, flow = z((24, span), bf), z((span, 128), bf)
        refcubin.run("k3_span_gather_v3+HEADS=24", "kern_k3_span_gather", (6, 4, (span + 15) // 16), 128,
                     [_up(inp["partial"], dev), _up(inp["cw"], dev), line, line_index, I64(line.numel()), _up(inp["wsm"], dev), q, k, v, beta, flow, span_at, span])
        torch.cuda.synchronize()
        win = line[rec:].view(bf).reshape(3, 3, inner)
        return dict(q=_bits(q), k=_bits(k), v=_bits(v), win=_bits(win), beta=_bits(beta), flow=_bits(flow))
    if name == "out_gate":
        at, span, rows, inner = 2, 10, 12, 3072
        gated = z((rows, inner), bf)
        span_at = torch.tensor([at], dtype=torch.int32, device=dev)
        refcubin.run("k3_kda_out_gate_v3+HEADS=24", "kern_k3_kda_out_gate", (span, 3), 128,
                     [_up(inp["attn"], dev), _up(inp["gate"], dev), _up(inp["gamma_o"], dev), gated, span_at, span])
        torch.cuda.synchronize()
        return dict(gated=_bits(gated))
    raise KeyError(name)


def main():
    import torch
    out = sys.argv[1] if len(sys.argv) > 1 else os.path.join(HERE, "reference_outputs.npz")
    dev = torch.device("cuda:0")
    rec = {}
    for name in cases.NAMES:
        for k, v in run_reference(name, cases.inputs(name), dev).items():
            rec["%s/%s" % (name, k)] = v
    np.savez_compressed(out, **rec)
    print("wrote %s: %d arrays, %.1f KB" % (out, len(rec), os.path.getsize(out) / 1e3))


if __name__ == "__main__":
    main()
