"""TEST INFRASTRUCTURE — time the reference's own kernels (oracle/_ref, the reference sources
compiled for sm_100a) next to this library's kernels on the same GPU, same shapes, same inputs.

    python oracle/time_reference_kernels.py [out.json]

Shapes are the reference deployment's (16384-token prefill, TP4/EP4: 4096-row shards, 24 KDA heads,
56 local experts).  Reference kernels run with the manifest's grid/block; this library runs through
its C ABI.  CUDA events, 20 launches after 3 warm-ups.  Tensors of one op total more than the L2.
"""
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.join(ROOT, "kern-k3_b200"))
import k3g  # noqa: E402
import refcubin  # noqa: E402
from refcubin import I64  # noqa: E402

MOE = "k3_moe_prefill_v4+EP_RANKS=4+EP_STRIDED=1+TILE_SHIFT=7+SCATTER_WARPS=16"


def time_us(fn, iters=20, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) * 1e3 / iters


def main():
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev); g.manual_seed(1)
    bf = torch.bfloat16
    rnd = lambda *s: torch.randn(s, generator=g, device=dev).to(bf)
    rndf = lambda *s: torch.randn(s, generator=g, device=dev)
    s = k3g.current_stream()
    B, T, H = 4096, 16384, 7168
    rows = []

    def add(name, ref_fn, our_fn, nbytes):
        r, o = time_us(ref_fn), time_us(our_fn)
        rows.append({"op": name, "reference_us": round(r, 2), "k3g_us": round(o, 2), "speedup": round(r / o, 2), "bytes": nbytes,
                     "k3g_gbs": round(nbytes / o / 1e3, 1)})
        print(rows[-1], flush=True)

    partial, prefix, blocks = rnd(T, H), rnd(T, H), rnd(B, 8, H)
    sw, gamma = 0.05 * rndf(H), (1 + 0.02 * rndf(H)).to(bf)
    p2, nrm = torch.empty((T, H), dtype=bf, device=dev), torch.empty((T, H), dtype=bf, device=dev)
    for nb, R in ((0, T), (4, B)):
        add("land_add_attnres_rms bf16 nb=%d, %d rows" % (nb, R),
            lambda: refcubin.run("k3_residual_v2+LAND_BF16=1", "kern_k3_land_add_attnres_rms", R, 128, [partial, prefix, blocks, sw, gamma, p2, nrm, nb, 0, R]),
            lambda: k3g.call("k3g_land_add_attnres_rms", partial, 1, prefix, blocks, sw, gamma, p2, nrm, nb, 0, R, H, 1e-5, s), (8 + 2 * nb) * R * H)
    pf1, pf2 = rndf(B, H), rndf(B, H)
    add("land_add2 f32 two, 4096 rows",
        lambda: refcubin.run("k3_residual_v2", "kern_k3_land_add2", B, 128, [pf1, pf2, prefix, p2, 1, B]),
        lambda: k3g.call("k3g_land_add2", pf1, pf2, 0, prefix, p2, 1, B, H, s), 12 * B * H)
    q8, sf8 = torch.empty((T, H), dtype=torch.uint8, device=dev), torch.empty((T, H // 32), dtype=torch.uint8, device=dev)
    R2 = 2 * T
    add("moe_quant 32768x3584",
        lambda: refcubin.run(MOE, "kern_k3_moe_quant", (R2 * 3584 // 32 + 255) // 256, 256, [partial, q8, sf8, R2, 3584]),
        lambda: k3g.call("k3g_moe_quant", partial, q8, sf8, R2, 3584, 0, s), R2 * 3584 * 3 + R2 * 112)
    part, sc = torch.empty(2048, device=dev), torch.empty(1, device=dev)
    n = T * H

    def ref_quant():
        refcubin.run("k3_quant_fp8_pair_v2", "kern_quant_fp8_amax_v2", 2048, 256, [partial, n, part])
        refcubin.run("k3_quant_fp8_pair_v2", "kern_quant_fp8_apply_v2", 2048, 256, [partial, q8, n, part, 2048, sc])
    add("quant_fp8_tensor 16384x7168 (2 launches)", ref_quant, lambda: k3g.call("k3g_quant_fp8_tensor", partial, q8, sc, part, n, 2048, s), 3 * n)
    S, bias, rs = rndf(T, 224), 0.1 * rndf(224), torch.ones(1, dtype=bf, device=dev)
    idx, wts = torch.empty((T, 16), dtype=torch.int32, device=dev), torch.empty((T, 16), device=dev)
    add("router_topk k=16, 16384 rows",
        lambda: refcubin.run("k3_router_argmax", "kern_k3_router_topk", T, 256, [S, bias, rs, idx, wts, T]),
        lambda: k3g.call("k3g_router_topk", S, bias, rs, idx, wts, T, 224, 16, s), T * 224 * 4 + T * 16 * 8)
    torch.cuda.synchronize()
    E, tile, nblk = 56, 128, T // 256
    nct = T * 16 // tile + E
    bc, bo = torch.zeros((nblk, E), dtype=torch.int32, device=dev), torch.zeros((nblk, E), dtype=torch.int32, device=dev)
    cb, cl = torch.zeros(nct, dtype=torch.int32, device=dev), torch.zeros(nct, dtype=torch.int32, device=dev)
    rm = torch.zeros(nct * tile, dtype=torch.int32, device=dev)
    nne, tot = torch.zeros(1, dtype=torch.int32, device=dev), torch.zeros(1, dtype=torch.int32, device=dev)
    e2p = torch.zeros((T, 16), dtype=torch.int32, device=dev)

    def ref_route():
        refcubin.run(MOE, "kern_k3_moe_route_count", nblk, 256, [idx, T, 1, E, bc])
        refcubin.run(MOE, "kern_k3_moe_route_tables", 1, 1024, [bc, nblk, E, tile, bo, cb, cl, nne, tot, rm])
        refcubin.run(MOE, "kern_k3_moe_route_scatter", nblk, 512, [idx, bo, T, 1, E, rm, e2p])

    def our_route():
        k3g.call("k3g_moe_route_count", idx, T, 1, E, 16, 4, 1, bc, s)
        k3g.call("k3g_moe_route_tables", bc, nblk, E, tile, bo, cb, cl, nne, tot, rm, s)
        k3g.call("k3g_moe_route_scatter", idx, bo, T, 1, E, 16, 4, 1, rm, e2p, s)
    add("route count+tables+scatter (3 launches), T=16384", ref_route, our_route, T * 16 * 4 * 4)
    torch.cuda.synchronize()
    prow = int(tot.item())
    fc2 = rnd(prow, 3584); fout = torch.empty((T, 3584), dtype=bf, device=dev)
    add("moe_finalize 16384x3584, %d permuted rows" % prow,
        lambda: refcubin.run(MOE, "kern_k3_moe_finalize", (T + 1) // 2, 128, [fc2, e2p, wts, fout, T, 3584]),
        lambda: k3g.call("k3g_moe_finalize", fc2, e2p, wts, fout, T, 3584, 16, s), (T * 4 + T) * 3584 * 2)
    del fc2
    mp = rndf(T, 5184); gq, gkv = gamma[:1536].contiguous(), gamma[:512].contiguous()
    slots = torch.arange(T, dtype=torch.int64, device=dev)
    slab = torch.zeros((T // 64) * 64 * 576, dtype=bf, device=dev)
    qn, mg = torch.empty((T, 1536), dtype=bf, device=dev), torch.empty((T, 3072), dtype=bf, device=dev)
    mod = "k3_mla_prep_v2+INNER=3072+MLA_FUSED=5184"

    def ref_mla():
        refcubin.run(mod, "kern_k3_mla_prep_head", T // 4, 512, [mp, gq, gkv, slots, slab, I64(0), I64(64 * 576), qn, T])
        refcubin.run(mod, "kern_k3_mla_prep_gate", T // 4, 384, [mp, mg, T])
    add("mla_prep f32 head+gate, 16384 rows", ref_mla,
        lambda: k3g.call("k3g_mla_prep", mp, 0, gq, gkv, slots, slab, 0, 64 * 576, qn, mg, T, 3072, 1e-5, s), T * (5184 * 4 + 1536 * 2 + 576 * 2 + 3072 * 2))
    del mp
    inner = 3072
    kp = rnd(T, 4 * inner); cw = 0.5 * rndf(3, 4, inner); wsm = rndf(T, 256)
    rec = 24 * 128 * 128 * 4
    line = torch.zeros(rec + 3 * 3 * inner * 2, dtype=torch.uint8, device=dev)
    line_index = torch.zeros(T, dtype=torch.int32, device=dev); span_at = torch.zeros(1, dtype=torch.int32, device=dev)
    oq, ok, ov = (torch.empty((T, inner), dtype=bf, device=dev) for _ in range(3))
    beta, flow = torch.empty((24, T), dtype=bf, device=dev), torch.empty((T, 128), dtype=bf, device=dev)
    win = line[rec:].view(bf)
    add("span_gather conv+SiLU+beta/flow, 16384 rows",
        lambda: refcubin.run("k3_span_gather_v3+HEADS=24", "kern_k3_span_gather", (6, 4, T // 16), 128,
                             [kp, cw, line, line_index, I64(line.numel()), wsm, oq, ok, ov, beta, flow, span_at, T]),
        lambda: k3g.call("k3g_span_gather", kp, 4 * inner, cw, 0, win, wsm, oq, ok, ov, beta, flow, 24, 0, T, 0, s), T * 3 * inner * 4 + T * 256 * 4)
    gated = torch.empty((T, inner), dtype=bf, device=dev); gamma_o = torch.ones(128, device=dev)
    add("kda_out_gate, 16384 rows",
        lambda: refcubin.run("k3_kda_out_gate_v3+HEADS=24", "kern_k3_kda_out_gate", (T, 3), 128, [oq, kp, gamma_o, gated, span_at, T]),
        lambda: k3g.call("k3g_kda_out_gate", oq, kp, 4 * inner, 3 * inner, gamma_o, gated, None, None, 24, 0, T, 1e-5, s), T * inner * 6)
    fm, ag = rnd(T, inner), torch.empty((T, inner), dtype=bf, device=dev)
    add("sigmoid_mul (mla gate), 16384x3072",
        lambda: refcubin.run("sigmoid_mul", "kern_sigmoid_mul_bf16", (T, 2), 256, [ag, fm, oq, 24, 128, inner, 128]),
        lambda: k3g.call("k3g_sigmoid_mul", ag, fm, oq, T, 24, 128, inner, 128, s), T * inner * 6)
    del kp
    SH, LAT = 6144, 3584
    sp, lat, gl = rnd(B, 2 * SH), rnd(B, LAT), gamma[:LAT].contiguous()
    act, ln = torch.empty((B, SH), dtype=bf, device=dev), torch.empty((B, LAT), dtype=bf, device=dev)
    add("situ_rms (SiTU landing + latent RMSNorm), 4096 rows",
        lambda: refcubin.run("k3_land_fused", "kern_k3_situ_rms_bf16", 3 * ((4 * B + 15) // 16), 512,
                             [sp, act, lat, gl, ln, SH, B, LAT, B]),
        lambda: k3g.call("k3g_situ_rms", sp, act, lat, gl, ln, SH, B, LAT, B, s), B * (SH * 6 + LAT * 4))
    del sp, act
    pf, act33 = rndf(B, 2 * 33792), torch.empty((B, 33792), dtype=bf, device=dev)
    add("land_situ f32 (layer 0 dense MLP), 4096 x 33792",
        lambda: refcubin.run("k3_land", "kern_k3_land_situ", (B, 33), 1024, [pf, act33, 33792, B]),
        lambda: k3g.call("k3g_land_situ", pf, act33, 33792, B, s), B * 33792 * 10)
    if len(sys.argv) > 1:
        json.dump(rows, open(sys.argv[1], "w"), indent=1)


if __name__ == "__main__":
    main()
