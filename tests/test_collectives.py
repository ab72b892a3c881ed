"""Collective kernels on ONE GPU: the data paths at world 1/2/4/8 with the W ranks emulated as W
sets of buffers on the same device (kernels that never wait run one after the other; the epoch is
left at 0 so every poll is satisfied at once), the real flag protocol at world 1, and the bounded
wait: a counter that nothing advances makes the wait expire after ~1 ms and report, with the
context still usable.  Nothing here spins on another launch."""
import numpy as np
import pytest

import k3o
from util import bf16_bits, normal_bf16, rng, to_dev, to_dev_bf16

pytestmark = pytest.mark.gpu


def _table(tensors, dev):
    import torch
    return torch.tensor([t.data_ptr() for t in tensors], dtype=torch.int64, device=dev)


@pytest.mark.parametrize("W,order", [(1, 0), (2, 2), (4, 6), (8, 14), (4, 0), (4, 3), (4, 7), (2, 1), (3, 4), (8, 5)])
@pytest.mark.parametrize("count", [8, 7168 * 5, 7168 * 37 + 8])
def test_rs_pull_matches_ring_chain(k3g, dev, W, order, count):
    import torch
    g = rng(W * 100 + order + count)
    partials = [normal_bf16(g, (W * count,), std=0.5 / W) for _ in range(W)]
    d_part = [to_dev_bf16(p, dev) for p in partials]
    tab = _table(d_part, dev)
    for rank in range(W):
        want = k3o.rs_pull(partials, rank, order)
        dst = torch.zeros(count, dtype=torch.bfloat16, device=dev)
        k3g.call("k3g_rs_pull", d_part[rank], dst, tab, count, order, rank, W, 7, k3g.current_stream())
        torch.cuda.synchronize()
        assert np.array_equal(bf16_bits(dst), want), rank


def test_rs_pull_is_order_sensitive_and_linear(k3g, dev):
    """Properties: the chain order changes bits (so the test above discriminates), and a rank's chunk
    only depends on that chunk of every partial."""
    g = rng(5)
    W, count = 4, 7168 * 8
    partials = [normal_bf16(g, (W * count,)) for _ in range(W)]
    a, b = k3o.rs_pull(partials, 1, 6), k3o.rs_pull(partials, 1, 0)
    assert (a != b).any()
    other = [p.copy() for p in partials]
    for p in other:
        p[:count] = 0
    assert np.array_equal(k3o.rs_pull(other, 1, 6), a)


def _flags(dev, n=16):
    import torch
    return torch.zeros(n, dtype=torch.int64, device=dev)


def test_flag_protocol_world1(k3g, dev):
    import torch
    flags = torch.full((16,), 99, dtype=torch.int64, device=dev)
    tab = _table([flags], dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    s = k3g.current_stream()
    k3g.call("k3g_flags_init", flags, 16, s)
    for replay in range(1, 4):
        k3g.call("k3g_epoch_bump", flags, 896, s)
        for slot in (1, 2, 5):
            k3g.call("k3g_rs_arrive", flags, tab, 896, slot, 1, 1000, status, s)
    torch.cuda.synchronize()
    f = flags.cpu().numpy()
    assert f[0] == 3 * 896 and f[1] == f[2] == f[5] == 3 * 896 and f[3] == 0
    assert not status.cpu().numpy().any()


def test_epoch_bump_folded_into_the_first_barrier(k3g, dev):
    """k3g_epoch_arrive = epoch bump + arrive in one launch: same counters as the two calls."""
    import torch
    flags = _flags(dev)
    tab = _table([flags], dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    s = k3g.current_stream()
    for replay in range(3):
        k3g.call("k3g_epoch_arrive", flags, tab, 896, 1, 1, 1000, status, s)
        k3g.call("k3g_rs_arrive", flags, tab, 896, 2, 1, 1000, status, s)
    torch.cuda.synchronize()
    f = flags.cpu().numpy()
    assert f[0] == f[1] == f[2] == 3 * 896 and not status.cpu().numpy().any()
    # a peer that has not arrived in this epoch makes it expire like k3g_rs_arrive (fresh tables: a slot is used every epoch)
    mine, peer = _flags(dev), _flags(dev)
    tab2 = _table([mine, peer], dev)
    k3g.call("k3g_epoch_arrive", mine, tab2, 896, 3, 2, 1000, status, s)
    torch.cuda.synchronize()
    assert list(status.cpu().numpy()[:3]) == [1, 3, 1] and int(mine[0]) == 896 and int(mine[3]) == 896


def test_bounded_wait_reports_and_returns(k3g, dev):
    """Rank 0 of an emulated world of 2 waits on a peer counter that nothing advances: the wait runs
    out after the 1 ms limit, records {1, slot, peer, observed} and the kernel returns normally."""
    import torch
    mine, peer = _flags(dev), _flags(dev)
    tab = _table([mine, peer], dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    s = k3g.current_stream()
    k3g.call("k3g_epoch_bump", mine, 4, s)
    t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    k3g.call("k3g_rs_arrive", mine, tab, 4, 3, 2, 1000, status, s)
    t1.record()
    torch.cuda.synchronize()
    assert list(status.cpu().numpy()) == [1, 3, 1, 0]
    assert t0.elapsed_time(t1) < 100.0                          # ms: bounded, nowhere near the 2 s default
    assert mine.cpu().numpy()[3] == 4                           # own arrival still published
    # the context is healthy: the same call succeeds once the peer has arrived
    peer[3] = 4
    status.zero_()
    k3g.call("k3g_rs_arrive", mine, tab, 4, 3, 2, 1000, status, s)
    torch.cuda.synchronize()
    assert not status.cpu().numpy().any()
    # without a status pointer the record lands in the library's own status word
    host = np.zeros(4, np.uint32)
    k3g.call("k3g_wait_status", host, 1, s)
    k3g.call("k3g_rs_arrive", mine, tab, 4, 4, 2, 1000, None, s)
    k3g.call("k3g_wait_status", host, 1, s)
    assert list(host) == [1, 4, 1, 0]
    k3g.call("k3g_wait_status", host, 0, s)
    assert not host.any()


def test_wait_compares_full_64_bit_counters(k3g, dev):
    """Counters are never reset, so a long-lived process crosses 2^32 arrivals.  With the epoch just above
    2^32 and the peer's counter just below it, the low 32 bits of the peer (0xfffffffc) exceed those of the
    epoch (4): a 32-bit compare would pass at once.  The wait must expire; once the peer really arrives it passes."""
    import torch
    mine, peer = _flags(dev), _flags(dev)
    tab = _table([mine, peer], dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    s = k3g.current_stream()
    mine[0] = (1 << 32) + 4; mine[3] = (1 << 32)                 # own slot one step behind its epoch
    peer[3] = (1 << 32) - 4
    k3g.call("k3g_rs_arrive", mine, tab, 4, 3, 2, 1000, status, s)
    torch.cuda.synchronize()
    st = status.cpu().numpy().view(np.uint32)
    assert list(st) == [1, 3, 1, 0xfffffffc]
    assert int(mine[3]) == (1 << 32) + 4
    peer[3] = (1 << 32) + 4
    status.zero_()
    k3g.call("k3g_rs_arrive", mine, tab, 4, 4, 2, 1000, status, s)   # slot 4: both sides at zero, epoch far ahead -> expires
    torch.cuda.synchronize()
    assert status.cpu().numpy()[0] == 1
    status.zero_(); mine[4] = (1 << 32); peer[4] = (1 << 32) + 4
    k3g.call("k3g_rs_arrive", mine, tab, 4, 4, 2, 1000, status, s)
    torch.cuda.synchronize()
    assert not status.cpu().numpy().any()


@pytest.mark.parametrize("W", [1, 2, 4, 8])
def test_allgather4_push_emulated(k3g, dev, W):
    import torch
    g = rng(W)
    rows = 37
    sizes = [rows * 3584, rows * 112, rows * 16 * 4, rows * 16 * 4]
    srcs = [[to_dev(g.integers(0, 256, n, dtype=np.uint8), dev) for n in sizes] for _ in range(W)]
    dsts = [[torch.zeros(W * n, dtype=torch.uint8, device=dev) for n in sizes] for _ in range(W)]
    tabs = [_table([dsts[r][i] for r in range(W)], dev) for i in range(4)]
    flags = [_flags(dev) for _ in range(W)]
    ftab = _table(flags, dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    for r in range(W):
        a = []
        for i in range(4):
            a += [srcs[r][i], dsts[r][i], tabs[i], sizes[i]]
        k3g.call("k3g_allgather4_push", *a, flags[r], ftab, 2, r, W, 13, 1000, status, k3g.current_stream())
    torch.cuda.synchronize()
    assert not status.cpu().numpy().any()
    for i in range(4):
        want = torch.cat([srcs[r][i] for r in range(W)])
        for r in range(W):
            assert torch.equal(dsts[r][i], want)
    assert all(int(f[2]) == 13 for f in flags)                  # one arrival per block


@pytest.mark.parametrize("W,H,rows", [(1, 7168, 9), (2, 7168, 33), (4, 7168, 17), (8, 7168, 5), (4, 1024, 64), (2, 2048, 3)])
def test_fused_rs_resnorm_ag_emulated(k3g, dev, W, H, rows):
    """Fused pull reduce-scatter -> residual/RMSNorm/MXFP8 -> push all-gather == the oracle's
    rs_pull followed by resnorm_mxfp8, gathered in rank order on every rank."""
    import torch
    g = rng(W * 7 + H + rows)
    T = W * rows
    partials = [normal_bf16(g, (T * H,), std=0.5 / W) for _ in range(W)]
    residual = [normal_bf16(g, (rows, H)) for _ in range(W)]
    gamma = normal_bf16(g, (H,), mean=1.0, std=0.02)
    want_res, want_q, want_sf = [], [], []
    for r in range(W):
        delta = k3o.rs_pull(partials, r, 2 * (W - 1)).reshape(rows, H)
        o, q, sf, _ = k3o.resnorm_mxfp8(residual[r], delta, gamma, 1e-6, want_normed=False)
        want_res.append(o); want_q.append(q); want_sf.append(sf)
    want_q, want_sf = np.concatenate(want_q), np.concatenate(want_sf)
    d_part = [to_dev_bf16(p, dev) for p in partials]
    ptab = _table(d_part, dev)
    q_all = [torch.zeros((T, H), dtype=torch.uint8, device=dev) for _ in range(W)]
    sf_all = [torch.zeros((T, H // 32), dtype=torch.uint8, device=dev) for _ in range(W)]
    qtab, sftab = _table(q_all, dev), _table(sf_all, dev)
    d_gamma = to_dev_bf16(gamma, dev)
    for r in range(W):
        res_out = torch.zeros((rows, H), dtype=torch.bfloat16, device=dev)
        k3g.call("k3g_rs_resnorm_mxfp8_ag", d_part[r], ptab, to_dev_bf16(residual[r], dev), d_gamma, res_out, q_all[r], qtab, sf_all[r],
                 sftab, rows, H, 1e-6, r, W, 0, 0, 0, k3g.current_stream())
        torch.cuda.synchronize()
        assert np.array_equal(bf16_bits(res_out), want_res[r])
    for r in range(W):
        assert np.array_equal(sf_all[r].cpu().numpy(), want_sf)
        assert np.array_equal(q_all[r].cpu().numpy(), want_q)


def test_fused_kernel_in_row_chunks_equals_one_call(k3g, dev):
    """A shard processed as three row chunks (row_begin / rows / shard_rows) gives the same bytes as
    one call -- what the host-side copy/compute pipeline relies on."""
    import torch
    g = rng(31)
    W, H, rows = 2, 7168, 21
    T = W * rows
    partials = [to_dev_bf16(normal_bf16(g, (T * H,), std=0.25), dev) for _ in range(W)]
    ptab = _table(partials, dev)
    residual = to_dev_bf16(normal_bf16(g, (rows, H)), dev); gamma = to_dev_bf16(normal_bf16(g, (H,), mean=1.0, std=0.02), dev)
    outs = []
    for chunks in ([(0, rows)], [(0, 8), (8, 8), (16, 5)]):
        q_all = [torch.zeros((T, H), dtype=torch.uint8, device=dev) for _ in range(W)]
        sf_all = [torch.zeros((T, H // 32), dtype=torch.uint8, device=dev) for _ in range(W)]
        qtab, sftab = _table(q_all, dev), _table(sf_all, dev)
        res_out = torch.zeros((rows, H), dtype=torch.bfloat16, device=dev)
        for r0, n in chunks:
            k3g.call("k3g_rs_resnorm_mxfp8_ag", partials[1], ptab, residual, gamma, res_out, q_all[1], qtab, sf_all[1], sftab, n, H, 1e-6, 1, W, 0,
                     r0, rows, k3g.current_stream())
        torch.cuda.synchronize()
        outs.append((res_out, q_all[0], q_all[1], sf_all[0], sf_all[1]))
    for a, b in zip(*outs):
        assert torch.equal(a, b)
    assert int(outs[0][1][rows:].max()) > 0 and int(outs[0][1][:rows].max()) == 0     # rank 1's rows landed in its slice only
    s = k3g.current_stream()
    assert k3g.raw("k3g_rs_resnorm_mxfp8_ag", partials[1], ptab, residual, gamma, res_out, q_all[1], qtab, sf_all[1], sftab, 8, H, 1e-6, 1, W, 0, 16, rows, s) == -4


def test_collective_argument_errors(k3g, dev):
    import torch
    x = torch.zeros(64, dtype=torch.bfloat16, device=dev); tab = _table([x], dev); f = _flags(dev)
    s = k3g.current_stream()
    assert k3g.raw("k3g_rs_pull", x, x, tab, 12, 0, 0, 1, 1, s) == -2          # count not a multiple of 8
    assert k3g.raw("k3g_rs_pull", x, x, tab, 16, 0, 2, 2, 1, s) == -4          # rank out of range
    assert k3g.raw("k3g_rs_pull", x, x, None, 16, 0, 0, 1, 1, s) == -1
    assert k3g.raw("k3g_rs_arrive", f, tab, 4, 0, 1, 1000, None, s) == -4      # slot 0 is the epoch
    assert k3g.raw("k3g_rs_resnorm_mxfp8_ag", x, tab, x, x, x, x, tab, x, tab, 1, 7168, 1e-6, 0, 3, 0, 0, 0, s) == -2


def test_glue_step_host_paths_agree(k3g, dev):
    """World-1 glue step three ways -- device-resident step, CUDA-graph replay through pinned host
    buffers, and the row-chunked three-stream pipeline -- all bit-identical to the CPU oracle."""
    import torch
    from k3g.pipeline import TpGlue
    T, H = 96, 7168
    g = rng(91)
    partial, residual = normal_bf16(g, (T, H), std=0.5), normal_bf16(g, (T, H))
    gamma = normal_bf16(g, (H,), mean=1.0, std=0.02)
    want_res, want_q, want_sf, _ = k3o.resnorm_mxfp8(residual, partial, gamma, 1e-6, want_normed=False)
    glue = TpGlue(0, 1, T, H, 1e-6)
    glue.gamma.copy_(to_dev_bf16(gamma, dev))
    hp = to_dev_bf16(partial, "cpu").pin_memory(); hr = to_dev_bf16(residual, "cpu").pin_memory()
    for mode in ("serial", "graph", "pipelined"):
        ho = torch.zeros((T, H), dtype=torch.bfloat16).pin_memory()
        hq = torch.zeros((T, H), dtype=torch.uint8).pin_memory(); hs = torch.zeros((T, H // 32), dtype=torch.uint8).pin_memory()
        if mode == "graph":
            glue.capture()
        if mode == "pipelined":
            glue.step_host_pipelined(hp, hr, ho, hq, hs, chunks=5)
        else:
            glue.step_host(hp, hr, ho, hq, hs)
        torch.cuda.synchronize()
        glue.check_status()
        assert np.array_equal(bf16_bits(ho), want_res), mode
        assert np.array_equal(hq.numpy(), want_q) and np.array_equal(hs.numpy(), want_sf), mode
    glue.close()


@pytest.mark.parametrize("W", [1, 2, 4, 8])
def test_moe_quant_allgather_push_emulated(k3g, dev, W):
    """One launch == k3g_moe_quant followed by k3g_allgather4_push: identical gathered codes, scales and payloads on every
    rank (ranks emulated on one GPU with the epoch at 0, so nothing waits)."""
    import torch
    g = rng(40 + W)
    rows, cols = 19, 3584
    xs = [to_dev_bf16(normal_bf16(g, (rows, cols), std=3.0), dev) for _ in range(W)]
    pay = [[to_dev(g.integers(0, 256, rows * 64, dtype=np.uint8), dev) for _ in range(2)] for _ in range(W)]
    q_all = [torch.zeros((W * rows, cols), dtype=torch.uint8, device=dev) for _ in range(W)]
    sf_all = [torch.zeros((W * rows, cols // 32), dtype=torch.uint8, device=dev) for _ in range(W)]
    d2 = [torch.zeros(W * rows * 64, dtype=torch.uint8, device=dev) for _ in range(W)]
    d3 = [torch.zeros(W * rows * 64, dtype=torch.uint8, device=dev) for _ in range(W)]
    tq, tsf, t2, t3 = _table(q_all, dev), _table(sf_all, dev), _table(d2, dev), _table(d3, dev)
    flags = [_flags(dev) for _ in range(W)]
    ftab = _table(flags, dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    s = k3g.current_stream()
    want_q, want_sf = [], []
    for r in range(W):
        k3g.call("k3g_moe_quant_allgather_push", xs[r], rows, cols, q_all[r], tq, sf_all[r], tsf, pay[r][0], d2[r], t2, rows * 64, pay[r][1], d3[r], t3,
                 rows * 64, flags[r], ftab, 2, r, W, 13, 1000, status, s)
        q, sf = torch.zeros((rows, cols), dtype=torch.uint8, device=dev), torch.zeros((rows, cols // 32), dtype=torch.uint8, device=dev)
        k3g.call("k3g_moe_quant", xs[r], q, sf, rows, cols, 0, s)
        want_q.append(q); want_sf.append(sf)
    torch.cuda.synchronize()
    assert not status.cpu().numpy().any()
    want_q, want_sf = torch.cat(want_q), torch.cat(want_sf)
    for r in range(W):
        assert torch.equal(q_all[r], want_q) and torch.equal(sf_all[r], want_sf)
        assert torch.equal(d2[r], torch.cat([pay[k][0] for k in range(W)])) and torch.equal(d3[r], torch.cat([pay[k][1] for k in range(W)]))
    assert all(int(f[2]) == 13 for f in flags)
