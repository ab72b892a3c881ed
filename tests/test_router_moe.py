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


def _route(k3g, dev, ids, rank, E, ep, strided, tile):
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
