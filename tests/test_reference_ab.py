"""GPU A/B: the reference's own kernels (oracle/_ref/*.cubin, built from the reference sources for
sm_100a) against the committed golden record, and against this library's drop-in cubins launched
with the SAME entry names, parameter lists and manifest launch dims."""
import os
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
sys.path.insert(0, os.path.join(HERE, "golden"))
import cases  # noqa: E402
from util import bf16_ulp_diff  # noqa: E402

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(HERE, "golden", "reference_outputs.npz")
REF = os.path.join(ROOT, "oracle", "_ref")
OURS = os.path.join(ROOT, "kern-k3_b200", "lib", "cubin")


def _have_ref():
    return os.path.isdir(REF) and any(f.endswith(".cubin") for f in os.listdir(REF))


@pytest.mark.parametrize("name", cases.NAMES)
def test_reference_kernels_reproduce_the_golden_record(dev, name):
    if not _have_ref():
        pytest.skip("oracle/_ref not built (needs the reference checkout at build time)")
    import make_golden
    golden = np.load(GOLDEN)
    out = make_golden.run_reference(name, cases.inputs(name), dev)
    for k, v in out.items():
        assert np.array_equal(v, golden["%s/%s" % (name, k)]), (name, k)


@pytest.mark.parametrize("name", cases.NAMES)
def test_dropin_cubins_with_reference_launch_dims(dev, name, monkeypatch):
    """Point the reference launcher at THIS library's cubins: same module names, entries, parameters,
    grid and block.  Outputs must agree with the reference's record exactly where the arithmetic is
    IEEE-only and within the documented bf16 tolerance elsewhere."""
    import make_golden
    import refcubin
    k3g_build = os.path.join(ROOT, "kern-k3_b200")
    if not os.path.isdir(OURS):
        sys.path.insert(0, k3g_build)
        import build
        build.build()
    alias = {"k3_rs_arrive_v2": "k3_reducescatter_pull_nr4", "k3_allgather4_v3": "k3_reducescatter_pull_nr4",
             cases.MOE: cases.MOE}
    def ours(module, entry):
        mod = alias.get(module, module)
        if entry == "kern_k3_moe_quant":
            mod = "k3_quant_fp8_pair_v2"
        return refcubin.load_external(os.path.join(OURS, mod + ".cubin"), entry)
    monkeypatch.setattr(refcubin, "function", ours)
    golden = np.load(GOLDEN)
    out = make_golden.run_reference(name, cases.inputs(name), dev)
    for k in cases.EXACT[name]:
        assert np.array_equal(out[k], golden["%s/%s" % (name, k)]), (name, k)
    for k, (ulp, frac) in cases.TOLERANT.get(name, {}).items():
        d = bf16_ulp_diff(out[k], golden["%s/%s" % (name, k)])
        assert d.max() <= ulp and (d > 0).mean() <= frac, (name, k, int(d.max()), float((d > 0).mean()))
    if name == "router":
        # IEEE-only sigmoid here, libdevice expf in the reference: picks may differ only at near-ties of the biased score
        from util import router_picks_differ_only_at_near_ties
        inp = cases.inputs("router")
        differing, _ = router_picks_differ_only_at_near_ties(inp["S"], inp["bias"], out["idx"], golden["router/idx"], ulps=4)
        same = (out["idx"] == golden["router/idx"]).all(axis=1)
        assert differing <= 1 and np.allclose(out["wts"][same], golden["router/wts"][same], rtol=2e-6)


@pytest.mark.parametrize("span,gz", [(40, 32), (5, 8), (2, 4), (100, 7)])
def test_dropin_span_gather_short_span_under_a_wide_grid(dev, span, gz):
    """`span` is a run-time parameter of kern_k3_span_gather, separate from the token count the grid was sized for:
    a span of at most 2 * gridDim.z rows must not let a block that starts at row 1 or 2 read the stored window
    while the row-0 block overwrites it.  The drop-in cubin, launched with such a grid, against the CPU oracle:
    window, beta and flow bit for bit, q / k / v at the approximate-sigmoid tolerance."""
    import torch
    import k3o
    import refcubin
    from refcubin import I64
    from util import bf16_bits, normal_bf16, rng, to_dev, to_dev_bf16
    g = rng(900 + span)
    inner, at, rows = 3072, 1, span + 3
    partial = normal_bf16(g, (rows, 4 * inner)); cw = (g.standard_normal((3, 4, inner), dtype=np.float32) * 0.5).astype(np.float32)
    win = normal_bf16(g, (3, 3, inner)); wsm = g.standard_normal((rows, 256), dtype=np.float32)
    o_q, o_k, o_v, o_win = k3o.span_conv_silu(partial, 4 * inner, cw, win, inner, at, span)
    o_beta, o_flow = k3o.span_beta_flow(wsm, 24, at, span)
    rec = 24 * 128 * 128 * 4
    line = torch.zeros(rec + 3 * 3 * inner * 2, dtype=torch.uint8, device=dev)
    line[rec:] = to_dev_bf16(win, dev).view(torch.uint8).reshape(-1)
    line_index = torch.zeros(rows, dtype=torch.int32, device=dev); span_at = torch.tensor([at], dtype=torch.int32, device=dev)
    bf = torch.bfloat16
    q, k, v = (torch.zeros((span, inner), dtype=bf, device=dev) for _ in range(3))
    beta, flow = torch.zeros((24, span), dtype=bf, device=dev), torch.zeros((span, 128), dtype=bf, device=dev)
    fn = refcubin.load_external(os.path.join(OURS, "k3_span_gather_v3+HEADS=24.cubin"), "kern_k3_span_gather")
    for _ in range(3):                                               # a race would not show on every launch
        line[rec:] = to_dev_bf16(win, dev).view(torch.uint8).reshape(-1)
        refcubin.launch(fn, (6, 4, gz), 128, [to_dev_bf16(partial, dev), to_dev(cw, dev), line, line_index, I64(line.numel()), to_dev(wsm, dev),
                                              q, k, v, beta, flow, span_at, span])
        torch.cuda.synchronize()
        assert np.array_equal(bf16_bits(line[rec:].view(bf).reshape(3, 3, inner)), o_win)
        assert np.array_equal(bf16_bits(beta), o_beta) and np.array_equal(bf16_bits(flow), o_flow)
        for got, want in zip((q, k, v), (o_q, o_k, o_v)):
            d = bf16_ulp_diff(bf16_bits(got), want)
            assert d.max() <= 1 and (d > 0).mean() < 5e-3


def test_router_against_the_reference_kernel_at_16384_rows(k3g, dev):
    """Routing indices at the benchmark's own size, this library (through the C ABI) against the reference's kernel
    run live: the two differ only in the last ulp of the sigmoid (IEEE-only polynomial here, libdevice expf there),
    so rows may differ only where two biased scores are within 4 f32 ulps; the count is printed.  Indices and weights
    are also compared with the CPU oracle (same sigmoid): bit for bit."""
    if not _have_ref():
        pytest.skip("oracle/_ref not built (needs the reference checkout at build time)")
    import torch
    import k3o
    import refcubin
    from util import rng, router_picks_differ_only_at_near_ties, to_dev
    g = rng(16384)
    B = 16384
    S = g.standard_normal((B, 224), dtype=np.float32); bias = (g.standard_normal(224, dtype=np.float32) * 0.1).astype(np.float32)
    rs = k3o.f32_to_bf16(np.array([1.0], np.float32))
    dS, dbias = to_dev(S, dev), to_dev(bias, dev)
    drs = torch.from_numpy(rs.view(np.int16)).to(dev).view(torch.bfloat16)
    ref_idx, ref_w = torch.zeros((B, 16), dtype=torch.int32, device=dev), torch.zeros((B, 16), dtype=torch.float32, device=dev)
    refcubin.run("k3_router_argmax", "kern_k3_router_topk", B, 256, [dS, dbias, drs, ref_idx, ref_w, B])
    idx, w = torch.zeros_like(ref_idx), torch.zeros_like(ref_w)
    k3g.call("k3g_router_topk", dS, dbias, drs, idx, w, B, 224, 16, k3g.current_stream())
    torch.cuda.synchronize()
    idx, w, ref_idx, ref_w = idx.cpu().numpy(), w.cpu().numpy(), ref_idx.cpu().numpy(), ref_w.cpu().numpy()
    o_idx, o_w = k3o.router_topk(S, bias, rs, 16)
    assert np.array_equal(idx, o_idx) and np.array_equal(w.view(np.uint32), o_w.view(np.uint32))
    differing, worst = router_picks_differ_only_at_near_ties(S, bias, idx, ref_idx, ulps=4)
    print("ROUTER_VS_REFERENCE rows=%d differing_rows=%d worst_gap_ulps=%.2f" % (B, differing, worst))
    assert differing <= B // 1000                                   # ~1e-5 per pick expected; 0.1 % of rows is already a bug
    same = (idx == ref_idx).all(axis=1)
    assert np.allclose(w[same], ref_w[same], rtol=2e-6, atol=0)


def test_fused_cubin_entries_equal_the_c_abi(k3g, dev):
    """The entries `patch_manifest.py --fuse` points the fused call list at (modules k3g_fused_residual / k3g_fused_situ,
    built for a tensor-parallel group of 4) launched with the manifest's geometry on four emulated ranks: their outputs
    equal the C-ABI entry points' byte for byte (those are checked against the oracle elsewhere)."""
    import torch
    import refcubin
    from util import normal_bf16, rng, to_dev, to_dev_bf16
    W, B, H, nb = 4, 21, 7168, 4
    g = rng(4242)
    bf = torch.bfloat16
    z = lambda *shape, dt=bf: torch.zeros(shape, dtype=dt, device=dev)
    tab = lambda ts: torch.tensor([t.data_ptr() for t in ts], dtype=torch.int64, device=dev)
    s = k3g.current_stream()
    # ---- push with row maxima (rank 1 of 4) --------------------------------------------------------------------------
    blocks_h = normal_bf16(g, (B, 8, H)); sw = to_dev((g.standard_normal(H, dtype=np.float32) * 0.05).astype(np.float32), dev)
    sw_mlp = to_dev((g.standard_normal(H, dtype=np.float32) * 0.05).astype(np.float32), dev); gamma = to_dev_bf16(normal_bf16(g, (H,), 1.0, 0.02), dev)
    p1, p2, prefix2 = (to_dev_bf16(normal_bf16(g, (B, H), std=0.5), dev) for _ in range(3))
    res = []
    for use_cubin in (False, True):
        blocks = to_dev_bf16(blocks_h, dev)
        alls = [z(W * B, H) for _ in range(W)]; maxes = [z(W * B, dt=torch.float32) for _ in range(W)]
        hidden, stats = z(B, H), z(B, 8, 2, dt=torch.float32)
        if use_cubin:
            fn = refcubin.load_external(os.path.join(OURS, "k3g_fused_residual.cubin"), "kern_k3g_attnres_rms_push_amax")
            refcubin.launch(fn, B, 128, [blocks, sw, gamma, alls[1], tab(alls), nb, 1, B, 1, W, sw_mlp, stats, p1, p2, prefix2, hidden, 1, maxes[1], tab(maxes)])
        else:
            k3g.call("k3g_attnres_rms_push_amax", blocks, sw, gamma, alls[1], tab(alls), nb, 1, B, 1, W, sw_mlp, stats, p1, p2, prefix2, hidden, 1, H,
                     1e-5, maxes[1], tab(maxes), s)
        torch.cuda.synchronize()
        res.append([blocks, hidden, stats] + alls + maxes)
    for a, b in zip(*res):
        assert torch.equal(a.view(torch.uint8), b.view(torch.uint8))
    assert res[0][3].abs().sum() > 0 and res[0][7][B:2 * B].min() > 0          # a peer's copy and the pushed maxima are populated
    # ---- reduce-scatter inside the landing (rank 2 of 4) ---------------------------------------------------------------
    parts = [to_dev_bf16(normal_bf16(g, (W * B, H), std=0.2), dev) for _ in range(W)]
    stats = res[0][2]; blocks = res[0][0]; prefix = res[0][1]
    out = []
    for use_cubin in (False, True):
        pre2, nrm, rowmax = z(B, H), z(B, H), z(B, dt=torch.float32)
        if use_cubin:
            fn = refcubin.load_external(os.path.join(OURS, "k3g_fused_residual.cubin"), "kern_k3g_rs_land_add_attnres_rms")
            refcubin.launch(fn, B, 128, [parts[2], tab(parts), 2, W, prefix, blocks, sw_mlp, gamma, pre2, nrm, nb, 0, B, stats, nb, rowmax])
        else:
            k3g.call("k3g_rs_land_add_attnres_rms", parts[2], tab(parts), 2, W, prefix, blocks, sw_mlp, gamma, pre2, nrm, nb, 0, B, H, 1e-5, stats, nb, rowmax, s)
        torch.cuda.synchronize()
        out.append([pre2, nrm, rowmax])
    for a, b in zip(*out):
        assert torch.equal(a.view(torch.uint8), b.view(torch.uint8))
    assert out[0][1].abs().sum() > 0
    # ---- reduce-scatter inside the latent norm + SiTU landing (rank 3 of 4), manifest grid -----------------------------
    n, h = 6144, 3584
    lat_parts = [to_dev_bf16(normal_bf16(g, (W * B, h), std=0.3), dev) for _ in range(W)]
    sp = to_dev_bf16(normal_bf16(g, (B, 2 * n), std=2.0), dev); gam = to_dev_bf16(normal_bf16(g, (h,), 1.0, 0.02), dev)
    out = []
    for use_cubin in (False, True):
        act, ln, item_max = z(B, n), z(B, h), z((B * n + 4095) // 4096, dt=torch.float32)
        if use_cubin:
            fn = refcubin.load_external(os.path.join(OURS, "k3g_fused_situ.cubin"), "kern_k3g_rs_situ_rms")
            refcubin.launch(fn, ((B * 3 + 1) // 2) * 2, 128, [sp, act, lat_parts[3], tab(lat_parts), 3, W, gam, ln, n, B, h, B, item_max])
        else:
            k3g.call("k3g_rs_situ_rms", sp, act, lat_parts[3], tab(lat_parts), 3, W, gam, ln, n, B, h, B, item_max, s)
        torch.cuda.synchronize()
        out.append([act, ln, item_max])
    for a, b in zip(*out):
        assert torch.equal(a.view(torch.uint8), b.view(torch.uint8))
    assert out[0][0].abs().sum() > 0 and out[0][1].abs().sum() > 0
