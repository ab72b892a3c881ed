"""Parity of the router and MoE routing / dispatch / combine kernels with the CPU oracle.
Indices, offsets and tables are compared bit for bit; so are the weights (the sigmoid uses only
IEEE operations on both sides) and the bf16 combine (fixed fma order)."""
import numpy as np
import pytest

import k3o
from util import bf16_bits, normal_bf16, rng, to_dev, to_dev_bf16

pytestmark = pytest.mark.gpu


def _router(k3g, dev, S, bias, rs, topk):
    import torch
    B = S.shape[0]
    idx = torch.full((B, topk), -7, dtype=torch.int32, device=dev)
    wts = torch.zeros((B, topk), dtype=torch.float32, device=dev)
    k3g.call("k3g_router_topk", to_dev(S, dev), to_dev(bias, dev), to_dev_bf16(rs, dev), idx, wts, B, 224, topk, k3g.current_stream())
    torch.cuda.synchronize()
    return idx.cpu().numpy(), wts.cpu().numpy()


@pytest.mark.parametrize("B,topk", [(1, 16), (7, 8), (4096, 16), (16384, 8), (1001, 16)])
def test_router_topk(k3g, dev, B, topk):
    g = rng(B + topk)
    S = g.standard_normal((B, 224), dtype=np.float32)
    bias = (g.standard_normal(224, dtype=np.float32) * 0.1).astype(np.float32)
    rs = k3o.f32_to_bf16(np.array([2.5 if topk == 16 else 1.0], np.float32))
    o_idx, o_w = k3o.router_topk(S, bias, rs, topk)
    g_idx, g_w = _router(k3g, dev, S, bias, rs, topk)
    assert np.array_equal(g_idx, o_idx)
    assert np.array_equal(g_w.view(np.uint32), o_w.view(np.uint32))
    assert np.allclose(g_w.sum(1), float(k3o.bf16_to_f32(rs)[0]), rtol=1e-5)


def test_router_ties_and_extremes(k3g, dev):
    """Equal keys resolve to the smallest expert id; saturated logits stay finite."""
    B = 6
    S = np.zeros((B, 224), np.float32)
    bias = np.zeros(224, np.float32)
    S[1, 100:] = 3.0
    S[2] = 90.0; S[3] = -90.0
    S[4, ::2] = 1e30; S[5, 5] = np.float32(1e-30)
    rs = k3o.f32_to_bf16(np.array([1.0], np.float32))
    o_idx, o_w = k3o.router_topk(S, bias, rs, 8)
    g_idx, g_w = _router(k3g, dev, S, bias, rs, 8)
    assert np.array_equal(g_idx, o_idx) and np.array_equal(g_w.view(np.uint32), o_w.view(np.uint32))
    assert list(g_idx[0]) == list(range(8)) and list(g_idx[1]) == list(range(100, 108))
    assert np.isfinite(g_w).all()


def _route(k3g, dev, ids, rank, E, ep, strided, tile, fused=False):
    import torch
    T, topk = ids.shape
    blocks = (T + 255) // 256
    d_ids = to_dev(ids, dev)
    max_ctas = (T * topk + tile - 1) // tile + E
    bc = torch.zeros((blocks, E), dtype=torch.int32, device=dev); bo = torch.zeros_like(bc)
    cb = torch.full((max_ctas,), -1, dtype=torch.int32, device=dev); cl = torch.full_like(cb, -1)
    nne = torch.zeros(1, dtype=torch.int32, device=dev); tot = torch.zeros(1, dtype=torch.int32, device=dev)
    rm = torch.full((max_ctas * tile,), -1, dtype=torch.int32, device=dev)
    e2p = torch.full((T, topk), -9, dtype=torch.int32, device=dev)
    s = k3g.current_stream()
    k3g.call("k3g_moe_route_count", d_ids, T, rank, E, topk, ep, strided, bc, s)
    if fused:                                                     # tables folded into the scatter launch
        k3g.call("k3g_moe_route_tables_scatter", d_ids, bc, T, rank, E, topk, ep, strided, tile, bo, cb, cl, nne, tot, rm, e2p, s)
    else:
        k3g.call("k3g_moe_route_tables", bc, blocks, E, tile, bo, cb, cl, nne, tot, rm, s)
        k3g.call("k3g_moe_route_scatter", d_ids, bo, T, rank, E, topk, ep, strided, rm, e2p, s)
    torch.cuda.synchronize()
    return dict(blockcount=bc, blockoff=bo, cta_batch=cb, cta_limit=cl, num_non_exiting=nne, total_padded=tot, route_map=rm,
                exp2perm=e2p)


def _ids(g, T, topk, experts=224):
    return np.stack([g.permutation(experts)[:topk] for _ in range(T)]).astype(np.int32)


@pytest.mark.parametrize("T,topk,ep,strided,tile", [(1, 16, 4, 1, 128), (255, 16, 4, 1, 128), (4097, 16, 4, 1, 128), (16384, 16, 4, 1, 128),
                                                   (16384, 8, 1, 0, 1), (3000, 8, 2, 0, 128), (777, 8, 8, 1, 1), (513, 8, 4, 0, 16),
                                                   (16384, 16, 1, 1, 128), (5000, 16, 2, 1, 128), (300, 8, 1, 0, 128)])
def test_route_tables_bit_exact(k3g, dev, T, topk, ep, strided, tile):
    g = rng(T + topk + ep)
    ids = _ids(g, T, topk)
    E = 224 // ep            # 224 / 112 local experts at EP = 1 / 2 take the wide kernels (16-bit counters in dynamic shared memory)
    for rank in sorted({0, ep - 1}):
        o = k3o.moe_route(ids, rank, E, ep, strided, tile)
        d = _route(k3g, dev, ids, rank, E, ep, strided, tile)
        for k in o:
            assert np.array_equal(d[k].cpu().numpy().reshape(o[k].shape), o[k]), (k, rank)
        # permutation properties: every local (t, k) lands on a distinct row holding its token
        e2p, rm = o["exp2perm"], o["route_map"]
        live = e2p >= 0
        assert len(np.unique(e2p[live])) == live.sum()
        assert np.array_equal(rm[e2p[live]], np.nonzero(live)[0])


@pytest.mark.parametrize("T,topk,ep,strided,tile", [(1, 16, 4, 1, 128), (4097, 16, 4, 1, 128), (16384, 16, 4, 1, 128), (16384, 8, 1, 0, 1),
                                                   (3000, 8, 2, 0, 128), (777, 8, 8, 1, 1), (16384, 16, 1, 1, 128), (16384, 8, 8, 0, 128)])
def test_route_tables_folded_into_scatter(k3g, dev, T, topk, ep, strided, tile):
    """count + (tables + scatter in one launch) leaves every table bit-identical to the oracle's three steps."""
    g = rng(T * 5 + topk + ep)
    ids = _ids(g, T, topk)
    E = 224 // ep
    for rank in sorted({0, ep - 1}):
        o = k3o.moe_route(ids, rank, E, ep, strided, tile)
        d = _route(k3g, dev, ids, rank, E, ep, strided, tile, fused=True)
        for k in o:
            assert np.array_equal(d[k].cpu().numpy().reshape(o[k].shape), o[k]), (k, rank)


@pytest.mark.parametrize("fused", [False, True])
@pytest.mark.parametrize("T,topk,ep,strided,tile", [(16384, 8, 8, 1, 128), (16384, 8, 4, 0, 128), (5000, 16, 2, 1, 128), (700, 8, 8, 0, 1),
                                                   (16384, 8, 1, 0, 128)])
def test_route_tables_of_every_owner_at_once(k3g, dev, T, topk, ep, strided, tile, fused):
    """rank = -1 builds the tables of all `ep` owners in one pass, stacked owner-major: owner o's slice, shifted by
    its first row, must be exactly the tables the oracle builds for rank o alone (the reference's per-rank tables)."""
    g = rng(T * 7 + topk + ep + strided)
    ids = _ids(g, T, topk)
    per = 224 // ep
    d = _route(k3g, dev, ids, -1, 224, ep, strided, tile, fused=fused)
    e2p_all, rm_all, bo_all = d["exp2perm"].cpu().numpy(), d["route_map"].cpu().numpy(), d["blockoff"].cpu().numpy()
    owner = ids % ep if strided else ids // per
    total = 0
    for o in range(ep):
        t = k3o.moe_route(ids, o, per, ep, strided, tile)
        base = int(bo_all[0, o * per])
        assert base == total                                       # owners are stacked without gaps
        rows = int(t["total_padded"][0])
        mine = owner == o
        assert np.array_equal(e2p_all[mine] - base, t["exp2perm"][mine])
        assert np.array_equal(rm_all[base:base + rows], t["route_map"][:rows])
        assert np.array_equal(bo_all[:, o * per:(o + 1) * per] - base, t["blockoff"])
        total += rows
    assert int(d["total_padded"].cpu().numpy()[0]) == total


def _dispatch_case(k3g, dev, T, topk, ep, strided, tile, cols, seed):
    """All `ep` ranks emulated on one GPU (the dispatch kernel never waits): rank r dispatches its T / ep tokens into
    the ep owners' buffers; returns what every owner received and the oracle's expert-sorted rows."""
    import torch
    g = rng(seed)
    ids = _ids(g, T, topk)
    per, B = 224 // ep, T // ep
    q = g.integers(0, 256, (T, cols), dtype=np.uint8); sf = g.integers(0, 256, (T, cols // 32), dtype=np.uint8)
    d = _route(k3g, dev, ids, -1, 224, ep, strided, tile, fused=True)
    want = [k3o.moe_route(ids, o, per, ep, strided, tile) for o in range(ep)]
    rows = [int(w["total_padded"][0]) for w in want]
    out_q = [torch.full((max(r, 1), cols), 0xEE, dtype=torch.uint8, device=dev) for r in rows]
    out_sf = [torch.full((max(r, 1), cols // 32), 0xEE, dtype=torch.uint8, device=dev) for r in rows]
    tq = torch.tensor([t.data_ptr() for t in out_q], dtype=torch.int64, device=dev)
    tsf = torch.tensor([t.data_ptr() for t in out_sf], dtype=torch.int64, device=dev)
    d_ids, dq, dsf = to_dev(ids, dev), to_dev(q, dev), to_dev(sf, dev)
    for r in range(ep):
        k3g.call("k3g_permute_dispatch", dq[r * B:(r + 1) * B], dsf[r * B:(r + 1) * B], d_ids, d["exp2perm"], d["blockoff"], B, r * B, topk, cols,
                 224, ep, strided, tq, tsf, k3g.current_stream())
    torch.cuda.synchronize()
    return q, sf, want, rows, out_q, out_sf


@pytest.mark.parametrize("T,topk,ep,strided,tile,cols", [(64, 8, 2, 0, 1, 7168), (1000, 8, 4, 1, 128, 7168), (504, 16, 8, 1, 128, 3584),
                                                        (96, 8, 8, 0, 16, 96), (300, 8, 1, 0, 128, 7168), (8, 8, 8, 1, 128, 7168)])
def test_permute_dispatch_to_owning_ranks(k3g, dev, T, topk, ep, strided, tile, cols):
    """Every owner's buffer holds, on the live rows of its own expert-sorted order, exactly what the oracle's
    permute_gather builds from that owner's route_map; the tile-padding rows are not written."""
    q, sf, want, rows, out_q, out_sf = _dispatch_case(k3g, dev, T, topk, ep, strided, tile, cols, T + ep + cols)
    for o in range(ep):
        if rows[o] == 0:
            continue
        o_q, o_sf = k3o.permute_gather(q, sf, want[o]["route_map"], rows[o])
        live = np.zeros(rows[o], bool)
        live[want[o]["exp2perm"][want[o]["exp2perm"] >= 0]] = True
        got_q, got_sf = out_q[o].cpu().numpy(), out_sf[o].cpu().numpy()
        assert np.array_equal(got_q[live], o_q[live]) and np.array_equal(got_sf[live], o_sf[live]), o
        assert (got_q[~live] == 0xEE).all() and (got_sf[~live] == 0xEE).all()


def test_route_empty_experts_and_duplicates(k3g, dev):
    """All tokens pick the same experts; most local experts receive nothing (zero tiles)."""
    T = 600
    ids = np.tile(np.arange(0, 64, 4, dtype=np.int32), (T, 1))
    o = k3o.moe_route(ids, 0, 56, 4, 1, 128)
    d = _route(k3g, dev, ids, 0, 56, 4, 1, 128)
    for k in o:
        assert np.array_equal(d[k].cpu().numpy().reshape(o[k].shape), o[k]), k


@pytest.mark.parametrize("T,cols,topk,ep", [(5, 3584, 16, 4), (2049, 3584, 16, 4), (300, 7168, 8, 1), (64, 256, 8, 2)])
def test_finalize_and_fused_residual(k3g, dev, T, cols, topk, ep):
    import torch
    g = rng(T + cols)
    ids = _ids(g, T, topk)
    E = min(224 // ep, 64)
    ids = (ids % (E * ep)).astype(np.int32)
    tabs = k3o.moe_route(ids, 0, E, ep, 1, 128)
    rows = int(tabs["total_padded"][0])
    fc2 = normal_bf16(g, (max(rows, 1), cols))
    wts = g.random((T, topk), dtype=np.float32)
    residual = normal_bf16(g, (T, cols))
    o_fin = k3o.moe_finalize(fc2, tabs["exp2perm"], wts, T, cols)
    o_res = k3o.finalize_residual(fc2, tabs["exp2perm"], wts, residual)
    d_fc2, d_e2p, d_w = to_dev_bf16(fc2, dev), to_dev(tabs["exp2perm"], dev), to_dev(wts, dev)
    out = torch.empty((T, cols), dtype=torch.bfloat16, device=dev); out2 = torch.empty_like(out)
    k3g.call("k3g_moe_finalize", d_fc2, d_e2p, d_w, out, T, cols, topk, k3g.current_stream())
    k3g.call("k3g_finalize_residual", d_fc2, d_e2p, d_w, to_dev_bf16(residual, dev), out2, T, cols, topk, k3g.current_stream())
    torch.cuda.synchronize()
    assert np.array_equal(bf16_bits(out), o_fin)
    assert np.array_equal(bf16_bits(out2), o_res)
    # fused == unfused composition (finalize, then the one-partial landing add)
    assert np.array_equal(o_res, k3o.land_add2(o_fin, None, residual, 0))


@pytest.mark.parametrize("T,cols,topk,tile", [(100, 7168, 8, 1), (1000, 7168, 8, 128), (50, 3584, 16, 128), (9, 96, 8, 1)])
def test_permute_gather(k3g, dev, T, cols, topk, tile):
    import torch
    g = rng(T * 3 + cols)
    ids = (_ids(g, T, topk) % 64).astype(np.int32)
    tabs = k3o.moe_route(ids, 0, 64, 1, 0, tile)
    rows = int(tabs["total_padded"][0])
    q = g.integers(0, 256, (T, cols), dtype=np.uint8); sf = g.integers(0, 256, (T, cols // 32), dtype=np.uint8)
    o_q, o_sf = k3o.permute_gather(q, sf, tabs["route_map"], rows)
    out_q = torch.zeros((rows, cols), dtype=torch.uint8, device=dev); out_sf = torch.zeros((rows, cols // 32), dtype=torch.uint8, device=dev)
    k3g.call("k3g_permute_gather", to_dev(q, dev), to_dev(sf, dev), to_dev(tabs["route_map"], dev), rows, cols, out_q, out_sf,
             k3g.current_stream())
    torch.cuda.synchronize()
    assert np.array_equal(out_q.cpu().numpy(), o_q) and np.array_equal(out_sf.cpu().numpy(), o_sf)
    # round trip: scattering the gathered rows back through exp2perm reproduces every token row
    e2p = tabs["exp2perm"]
    assert np.array_equal(o_q[e2p[:, 0]], q)


@pytest.mark.parametrize("experts,n,row_bytes,kg", [(3, 128, 48, 12), (2, 256, 1792, 112), (1, 384, 16, 4), (0, 128, 16, 4)])
@pytest.mark.parametrize("gated", [0, 1])
def test_expert_weight_and_scale_layouts(k3g, dev, experts, n, row_bytes, kg, gated):
    """Load-time rearrangement of expert weights / scale bytes into the grouped GEMM's layouts (byte-exact)."""
    import torch
    g = rng(experts * 13 + n + gated)
    w = g.integers(0, 256, (experts, n, row_bytes), dtype=np.uint8); sf = g.integers(0, 256, (experts, n, kg), dtype=np.uint8)
    dw = torch.zeros((max(experts, 1), n, row_bytes), dtype=torch.uint8, device=dev); dsf = torch.zeros((max(experts, 1), n, kg), dtype=torch.uint8, device=dev)
    s = k3g.current_stream()
    k3g.call("k3g_moe_w_shuffle", to_dev(w, dev) if experts else dw, dw, experts, n, row_bytes, gated, s)
    k3g.call("k3g_moe_sf_shuffle", to_dev(sf, dev) if experts else dsf, dsf, experts, n, kg, gated, s)
    torch.cuda.synchronize()
    if experts:
        assert np.array_equal(dw.cpu().numpy(), k3o.moe_w_shuffle(w, gated))
        assert np.array_equal(dsf.cpu().numpy(), k3o.moe_sf_shuffle(sf, gated))
