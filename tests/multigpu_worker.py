"""Worker of tests/test_multigpu.py: one rank of a world-W run of the collective kernels over real NVLink peers.

Part 1 (3 replays, everything against the CPU oracle): flag protocol, pull reduce-scatter, the fused
reduce-scatter -> residual/RMSNorm/MXFP8 -> all-gather kernel, the reduce-scatter folded into the residual kernel and
into the latent norm, the four-payload push all-gather with its ticket tail, the residual push with its row maxima,
the epoch-and-barrier launch, the latent quantisation written into every rank's gathered buffers, the whole per-layer
call list (fused list against reference list, byte for byte on every rank), and the dispatch to owning ranks (strided
and blocked expert placement).

Part 2 (soak, K3G_SOAK_REPLAYS replays, default 500): the same protocol round with the inputs CHANGED every replay --
the rows of every shard are rotated by a replay-dependent amount, the all-gather payloads and the dispatched token
rows are xor-ed with a replay-dependent byte -- and every output compared bit for bit on the device against the
(rotated / xor-ed) oracle result.
Nothing synchronises the ranks between replays except the kernels' own arrive / poll barriers, so a stale read, a
store that lands after the barrier or a ticket published early shows up as a mismatch.  All waits are bounded: an
expired wait sets the status word, which fails the run.

Every rank regenerates every rank's seeded inputs, so no data is exchanged besides the IPC handles."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in ("kern-k3_b200", "oracle", "tests"):
    sys.path.insert(0, os.path.join(ROOT, p))
import k3g  # noqa: E402
import k3o  # noqa: E402
from k3g.peer import PeerGroup, collective_units  # noqa: E402
from util import bf16_bits, normal_bf16, rng, to_dev, to_dev_bf16  # noqa: E402

TIMEOUT_US = 5_000_000


class Dispatch:
    """Dispatch to owning ranks across real peers: T tokens, 8 slots, 224 / world experts per rank, strided or blocked
    placement.  check() runs one dispatch round and compares every live row this rank received with the oracle's
    expert-sorted gather on this rank's own route_map; with a key the token rows are xor-ed with it first (so a round
    that delivers an earlier round's bytes is caught), and the comparison stays on the device."""

    def __init__(self, pg, rank, world, dev, s, strided, tag):
        self.rank, self.world, self.dev, self.s, self.strided = rank, world, dev, s, strided
        T, K, cols, tile = 64 * world, 8, 7168, 128
        self.T, self.K, self.cols, self.B, per = T, K, cols, T // world, 224 // world
        g = rng(77 + strided)
        ids = np.stack([g.permutation(224)[:K] for _ in range(T)]).astype(np.int32)
        self.q = g.integers(0, 256, (T, cols), dtype=np.uint8); self.sf = g.integers(0, 256, (T, cols // 32), dtype=np.uint8)
        want = k3o.moe_route(ids, rank, per, world, strided, tile)
        self.rows = int(want["total_padded"][0])
        cap = max(int(k3o.moe_route(ids, o, per, world, strided, tile)["total_padded"][0]) for o in range(world))
        self.b_q, self.b_sf = pg.symmetric("disp_q" + tag, cap * cols), pg.symmetric("disp_sf" + tag, cap * cols // 32)
        self.b_fl = pg.symmetric("disp_flags" + tag, 64)
        self.out_q, self.out_sf = self.b_q.tensor(torch.uint8, (cap, cols)), self.b_sf.tensor(torch.uint8, (cap, cols // 32))
        self.flags = self.b_fl.tensor(torch.int64, (8,))
        self.status = torch.zeros(4, dtype=torch.int32, device=dev)
        k3g.call("k3g_flags_init", self.flags, 8, s)
        blocks, E = (T + 255) // 256, 224
        nct = T * K // tile + E
        i32 = lambda *shape: torch.zeros(shape, dtype=torch.int32, device=dev)
        bc, self.bo, cb, cl, nne, tot, rm, self.e2p = i32(blocks, E), i32(blocks, E), i32(nct), i32(nct), i32(1), i32(1), i32(nct * tile), i32(T, K)
        self.d_ids = to_dev(ids, dev)
        k3g.call("k3g_moe_route_count", self.d_ids, T, -1, E, K, world, strided, bc, s)
        k3g.call("k3g_moe_route_tables_scatter", self.d_ids, bc, T, -1, E, K, world, strided, tile, self.bo, cb, cl, nne, tot, rm, self.e2p, s)
        o_q, o_sf = k3o.permute_gather(self.q, self.sf, want["route_map"], self.rows)
        live = np.zeros(self.rows, bool)
        live[want["exp2perm"][want["exp2perm"] >= 0]] = True
        self.live = to_dev(live, dev)
        self.want_q, self.want_sf = to_dev(o_q, dev), to_dev(o_sf, dev)
        B = self.B
        self.my_q, self.my_sf = to_dev(self.q[rank * B:(rank + 1) * B], dev), to_dev(self.sf[rank * B:(rank + 1) * B], dev)
        self.src_q, self.src_sf = torch.empty_like(self.my_q), torch.empty_like(self.my_sf)
        torch.cuda.synchronize(); dist.barrier()

    def round(self, key):
        """One epoch: fill the receive buffers, barrier, dispatch, barrier; returns a device flag: 1 if anything differs."""
        s = self.s
        torch.bitwise_xor(self.my_q, key, out=self.src_q); torch.bitwise_xor(self.my_sf, key, out=self.src_sf)
        self.out_q.fill_(0xEE); self.out_sf.fill_(0xEE)
        k3g.call("k3g_epoch_bump", self.flags, 4, s)
        k3g.call("k3g_rs_arrive", self.flags, self.b_fl.table, 4, 1, self.world, TIMEOUT_US, self.status, s)      # every rank's buffers are refilled
        k3g.call("k3g_permute_dispatch", self.src_q, self.src_sf, self.d_ids, self.e2p, self.bo, self.B, self.rank * self.B, self.K, self.cols, 224,
                 self.world, self.strided, self.b_q.table, self.b_sf.table, s)
        k3g.call("k3g_rs_arrive", self.flags, self.b_fl.table, 4, 2, self.world, TIMEOUT_US, self.status, s)      # every rank's rows have landed
        got_q, got_sf = self.out_q[:self.rows], self.out_sf[:self.rows]
        lv = self.live[:, None]
        bad = ((got_q != torch.bitwise_xor(self.want_q, key)) & lv).any() | ((got_sf != torch.bitwise_xor(self.want_sf, key)) & lv).any()
        bad = bad | ((got_q != 0xEE) & ~lv).any() | ((got_sf != 0xEE) & ~lv).any()             # padding rows untouched
        return bad.to(torch.int64) + (self.status[0] != 0).to(torch.int64)


def layer_entries_check(pg, rank, world, dev, s):
    """The per-layer entries that store to peers, across real GPUs and against the oracle: the residual push with its
    row maxima (k3g_attnres_rms_push_amax: every rank ends with all ranks' normed rows and maxima), the barrier that
    follows it in the fused call list (k3g_epoch_arrive), and the latent quantisation written straight into every
    rank's gathered buffers with the router payloads and its own barrier tail (k3g_moe_quant_allgather_push)."""
    from test_residual_push import _case
    B, H, nb, LAT = 24, 7168, 3, 3584
    T = world * B
    cases = [_case(700 + r, B) for r in range(world)]
    b_n, b_m, b_f = pg.symmetric("le_normed", T * H * 2), pg.symmetric("le_rowmax", T * 4), pg.symmetric("le_flags", 64)
    normed_all, rowmax_all = b_n.tensor(torch.bfloat16, (T, H)), b_m.tensor(torch.float32, (T,))
    flags = b_f.tensor(torch.int64, (8,))
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    normed_all.zero_(); rowmax_all.fill_(-1.0)
    k3g.call("k3g_flags_init", flags, 8, s)
    g = rng(900 + rank)
    x = normal_bf16(g, (B, LAT), std=2.0)
    pay = [g.integers(0, 256, B * 64, dtype=np.uint8) for _ in range(2)]
    b_q, b_sf = pg.symmetric("le_q", T * LAT), pg.symmetric("le_sf", T * LAT // 32)
    b_p = [pg.symmetric("le_pay%d" % i, T * 64) for i in range(2)]
    q_all, sf_all = b_q.tensor(torch.uint8, (T, LAT)), b_sf.tensor(torch.uint8, (T, LAT // 32))
    pay_all = [b.tensor(torch.uint8, (T * 64,)) for b in b_p]
    q_all.zero_(); sf_all.zero_()
    for t in pay_all:
        t.zero_()
    torch.cuda.synchronize(); dist.barrier()
    d = cases[rank]
    units = 5
    blocks, hidden = to_dev_bf16(d["blocks"], dev), torch.zeros((B, H), dtype=torch.bfloat16, device=dev)
    stats = torch.zeros((B, 8, 2), dtype=torch.float32, device=dev)
    k3g.call("k3g_attnres_rms_push_amax", blocks, to_dev(d["sw"], dev), to_dev_bf16(d["gamma"], dev), normed_all, b_n.table, nb, 1, B, rank, world,
             to_dev(d["sw_mlp"], dev), stats, to_dev_bf16(d["p1"], dev), to_dev_bf16(d["p2"], dev), to_dev_bf16(d["prefix2"], dev), hidden, 1, H, 1e-5,
             rowmax_all, b_m.table, s)
    k3g.call("k3g_epoch_arrive", flags, b_f.table, units, 1, world, TIMEOUT_US, status, s)          # every rank's rows and maxima have landed
    k3g.call("k3g_moe_quant_allgather_push", to_dev_bf16(x, dev), B, LAT, q_all, b_q.table, sf_all, b_sf.table, to_dev(pay[0], dev), pay_all[0],
             b_p[0].table, B * 64, to_dev(pay[1], dev), pay_all[1], b_p[1].table, B * 64, flags, b_f.table, 2, rank, world, units, TIMEOUT_US, status, s)
    torch.cuda.synchronize()
    assert not status.cpu().numpy().any(), status
    want_rows = []
    for r, c in enumerate(cases):
        o_hidden, o_normed, o_stats = k3o.attnres_rms_push(c["blocks"].copy(), c["sw"], c["gamma"], nb, 1, c["sw_mlp"], c["p1"], c["p2"], c["prefix2"], 1, 1e-5)
        want_rows.append(o_normed)
        if r == rank:
            assert np.array_equal(bf16_bits(hidden), o_hidden) and np.array_equal(stats.cpu().numpy().view(np.uint32), o_stats.view(np.uint32))
    want = np.concatenate(want_rows)
    assert np.array_equal(bf16_bits(normed_all), want)
    assert np.array_equal(rowmax_all.cpu().numpy(), (((want & 0x7fff).max(axis=1).astype(np.uint32)) << 16).view(np.float32))
    wq, wsf, wpay = [], [], [[], []]
    for r in range(world):
        gr = rng(900 + r)
        xr = normal_bf16(gr, (B, LAT), std=2.0)
        q, sf = k3o.moe_quant(xr)
        wq.append(q); wsf.append(sf)
        for i in range(2):
            wpay[i].append(gr.integers(0, 256, B * 64, dtype=np.uint8))
    assert np.array_equal(q_all.cpu().numpy(), np.concatenate(wq)) and np.array_equal(sf_all.cpu().numpy(), np.concatenate(wsf))
    for i in range(2):
        assert np.array_equal(pay_all[i].cpu().numpy(), np.concatenate(wpay[i]))
    f = flags.cpu().numpy()
    assert f[0] == units and f[1] == units and f[2] == units
    dist.barrier()


def layer_program_check(rank, world, dev):
    """The whole per-layer call list over real peers: the fused list must leave, on every rank, exactly the bytes the
    reference call list leaves (activations, quantised tensors, routing tables, flag counters), for a KDA and an MLA
    layer, two passes each so that flags and epochs have advanced once."""
    from k3g.layer import LayerGlue
    from test_layer_program import OUTPUTS
    for kind in ("kda", "mla"):
        got = {}
        for fused in (False, True):
            lg = LayerGlue(rank, world, tokens=1024, kind=kind, nb=3, seed=5, fused=fused)
            lg.run()
            lg.run()
            torch.cuda.synchronize()
            lg.check_status()
            extra = ["span_q", "span_k", "span_v", "gated"] if kind == "kda" else ["q_norm", "mla_gate", "attn_gated", "latent_rows"]
            got[fused] = {name: getattr(lg, name).clone() for name in OUTPUTS + extra}
            dist.barrier()
            lg.close()
        bad = [name for name, ref in got[False].items() if not torch.equal(ref.view(torch.uint8), got[True][name].view(torch.uint8))]
        assert not bad, (kind, bad)


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda")
    dist.init_process_group("nccl")
    rows, H = 96, 7168
    T = rows * world
    units = collective_units(T, world)
    pg = PeerGroup(rank, world)
    s = k3g.current_stream()
    partials = [normal_bf16(rng(1000 + r), (T * H,), std=0.5 / world) for r in range(world)]
    residual = [normal_bf16(rng(2000 + r), (rows, H)) for r in range(world)]
    gamma = normal_bf16(rng(3), (H,), mean=1.0, std=0.02)

    b_part = pg.symmetric("partial", T * H * 2)
    b_q = pg.symmetric("q_all", T * H)
    b_sf = pg.symmetric("sf_all", T * H // 32)
    b_flags = pg.symmetric("flags", 64 * 8)
    part = b_part.tensor(torch.bfloat16, (T * H,)); part.copy_(to_dev_bf16(partials[rank], dev))
    q_all = b_q.tensor(torch.uint8, (T, H)); sf_all = b_sf.tensor(torch.uint8, (T, H // 32))
    flags = b_flags.tensor(torch.int64, (64,))
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    k3g.call("k3g_flags_init", flags, 64, s)
    torch.cuda.synchronize(); dist.barrier()

    want_delta = k3o.rs_pull(partials, rank, 2 * (world - 1))
    wq, wsf = [], []
    for r in range(world):
        d = k3o.rs_pull(partials, r, 2 * (world - 1)).reshape(rows, H)
        o, q, sf, _ = k3o.resnorm_mxfp8(residual[r], d, gamma, 1e-6, want_normed=False)
        wq.append(q); wsf.append(sf)
        if r == rank:
            want_res = o
    wq, wsf = np.concatenate(wq), np.concatenate(wsf)
    d_res, d_gamma = to_dev_bf16(residual[rank], dev), to_dev_bf16(gamma, dev)
    sizes = (rows * 3584, rows * 112, rows * 64, rows * 64)
    payload = lambda r, i: rng(50 + r * 4 + i).integers(0, 256, sizes[i], dtype=np.uint8)
    srcs = [to_dev(payload(rank, i), dev) for i in range(4)]
    bufs = [pg.symmetric("ag%d" % i, world * n) for i, n in enumerate(sizes)]
    gathered = [b.tensor(torch.uint8, (world * n,)) for b, n in zip(bufs, sizes)]
    want_gathered = [np.concatenate([payload(r, i) for r in range(world)]) for i in range(4)]

    def push4(src_list):
        a = []
        for t, b in zip(src_list, bufs):
            a += [t, b.ptr, b.table, t.numel()]
        k3g.call("k3g_allgather4_push", *a, flags, b_flags.table, 4, rank, world, units, TIMEOUT_US, status, s)

    for replay in range(3):
        q_all.zero_(); sf_all.zero_()
        torch.cuda.synchronize(); dist.barrier()
        k3g.call("k3g_epoch_bump", flags, units, s)
        # unfused: arrive, pull reduce-scatter
        k3g.call("k3g_rs_arrive", flags, b_flags.table, units, 1, world, TIMEOUT_US, status, s)
        dst = torch.zeros(rows * H, dtype=torch.bfloat16, device=dev)
        k3g.call("k3g_rs_pull", part, dst, b_part.table, rows * H, 2 * (world - 1), rank, world, units, s)
        # fused: arrive (partials ready), fused kernel, arrive (pushes landed)
        k3g.call("k3g_rs_arrive", flags, b_flags.table, units, 2, world, TIMEOUT_US, status, s)
        res_out = torch.zeros((rows, H), dtype=torch.bfloat16, device=dev)
        k3g.call("k3g_rs_resnorm_mxfp8_ag", part, b_part.table, d_res, d_gamma, res_out, q_all,
                 b_q.table, sf_all, b_sf.table, rows, H, 1e-6, rank, world, 0, 0, 0, s)
        k3g.call("k3g_rs_arrive", flags, b_flags.table, units, 3, world, TIMEOUT_US, status, s)
        torch.cuda.synchronize()
        assert not status.cpu().numpy().any(), status
        assert np.array_equal(bf16_bits(dst), want_delta)
        assert np.array_equal(bf16_bits(res_out), want_res)
        assert np.array_equal(sf_all.cpu().numpy(), wsf)
        assert np.array_equal(q_all.cpu().numpy(), wq)
        # the same partials pulled inside the residual kernel (reduce-scatter folded into its consumer), world 1/2/4/8
        if world in (1, 2, 4, 8):
            nb = 3
            blocks_h = normal_bf16(rng(4000 + rank), (rows, 8, H)); sw_h = (rng(5).standard_normal(H, dtype=np.float32) * 0.05).astype(np.float32)
            p2, nrm = torch.zeros((rows, H), dtype=torch.bfloat16, device=dev), torch.zeros((rows, H), dtype=torch.bfloat16, device=dev)
            rowmax = torch.zeros(rows, dtype=torch.float32, device=dev)
            k3g.call("k3g_rs_land_add_attnres_rms", part, b_part.table, rank, world, d_res, to_dev_bf16(blocks_h, dev),
                     to_dev(sw_h, dev), d_gamma, p2, nrm, nb, 0, rows, H, 1e-5, None, 0, rowmax, s)
            torch.cuda.synchronize()
            o_p2, o_n = k3o.land_add_attnres_rms(want_delta.reshape(rows, H), residual[rank], blocks_h, sw_h, gamma, nb, 0, 1e-5)
            assert np.array_equal(bf16_bits(p2), o_p2) and np.array_equal(bf16_bits(nrm), o_n)
            assert np.array_equal(rowmax.cpu().numpy(), (((o_n & 0x7fff).max(axis=1).astype(np.uint32)) << 16).view(np.float32))
            # ... and inside the latent norm: the same buffer seen as [world * 2 rows, 3584]
            L2, h2 = 2 * rows, H // 2
            gam2 = normal_bf16(rng(6), (h2,), mean=1.0, std=0.02)
            sp_h = normal_bf16(rng(7000 + rank), (5, 2 * 256), std=3.0)
            act, ln = torch.zeros((5, 256), dtype=torch.bfloat16, device=dev), torch.zeros((L2, h2), dtype=torch.bfloat16, device=dev)
            k3g.call("k3g_rs_situ_rms", to_dev_bf16(sp_h, dev), act, part, b_part.table, rank, world, to_dev_bf16(gam2, dev), ln, 256, 5, h2, L2, None, s)
            torch.cuda.synchronize()
            o_act, o_ln = k3o.situ_rms(sp_h, want_delta.reshape(L2, h2), gam2, 256, h2)
            assert np.array_equal(bf16_bits(ln), o_ln)
        # push all-gather of four byte streams with its own barrier tail
        push4(srcs)
        torch.cuda.synchronize()
        assert not status.cpu().numpy().any(), status
        for i in range(4):
            assert np.array_equal(gathered[i].cpu().numpy(), want_gathered[i]), i
        dist.barrier()
    f = flags.cpu().numpy()
    assert f[0] == 3 * units and all(f[k] == 3 * units for k in (1, 2, 3, 4))

    if world in (1, 2, 4, 8):
        layer_entries_check(pg, rank, world, dev, s)
        layer_program_check(rank, world, dev)
    dispatchers = [Dispatch(pg, rank, world, dev, s, strided, "_s%d" % strided) for strided in (1, 0)] if world in (1, 2, 4, 8) else []
    for d in dispatchers:
        assert int(d.round(0)) == 0, ("dispatch", d.strided, d.status.cpu().tolist())

    # ---- part 2: soak with inputs that change every replay ------------------------------------------------------------
    replays = int(os.environ.get("K3G_SOAK_REPLAYS", "500"))
    base_part = [to_dev_bf16(partials[r], dev).view(world, rows, H) for r in range(world)]      # every rank's partial, by shard
    base_res = [to_dev_bf16(residual[r], dev) for r in range(world)]
    base_delta = to_dev_bf16(want_delta.reshape(rows, H), dev)
    base_res_out = to_dev_bf16(want_res, dev)
    base_q, base_sf = to_dev(wq, dev).view(world, rows, H), to_dev(wsf, dev).view(world, rows, H // 32)
    base_gathered = [to_dev(w, dev) for w in want_gathered]
    bad = torch.zeros(7, dtype=torch.int64, device=dev)
    res_in = torch.empty((rows, H), dtype=torch.bfloat16, device=dev)
    dst = torch.empty(rows * H, dtype=torch.bfloat16, device=dev); res_out = torch.empty((rows, H), dtype=torch.bfloat16, device=dev)
    soak_src = [torch.empty_like(t) for t in srcs]
    torch.cuda.synchronize(); dist.barrier()
    for replay in range(replays):
        shift = (replay * 7 + 1) % rows
        key = (replay * 37 + 11) & 0xff
        # this replay's inputs: rows of every shard rotated by `shift`; payloads xor `key`.  No host barrier: the peers are
        # held back by the arrive launches alone.
        part.view(world, rows, H).copy_(torch.roll(base_part[rank], shift, dims=1))
        res_in.copy_(torch.roll(base_res[rank], shift, dims=0))
        for t, b in zip(soak_src, srcs):
            torch.bitwise_xor(b, key, out=t)
        q_all.fill_(0x5a); sf_all.fill_(0x5a); dst.zero_(); res_out.zero_()
        for t in gathered:
            t.fill_(0xa5)
        k3g.call("k3g_epoch_bump", flags, units, s)
        k3g.call("k3g_rs_arrive", flags, b_flags.table, units, 1, world, TIMEOUT_US, status, s)
        k3g.call("k3g_rs_pull", part, dst, b_part.table, rows * H, 2 * (world - 1), rank, world, units, s)
        k3g.call("k3g_rs_arrive", flags, b_flags.table, units, 2, world, TIMEOUT_US, status, s)
        k3g.call("k3g_rs_resnorm_mxfp8_ag", part, b_part.table, res_in, d_gamma, res_out, q_all, b_q.table, sf_all, b_sf.table, rows, H, 1e-6,
                 rank, world, 0, 0, 0, s)
        k3g.call("k3g_rs_arrive", flags, b_flags.table, units, 3, world, TIMEOUT_US, status, s)
        push4(soak_src)
        bad[0] += (dst.view(rows, H) != torch.roll(base_delta, shift, dims=0)).any()
        bad[1] += (res_out != torch.roll(base_res_out, shift, dims=0)).any()
        bad[2] += (q_all.view(world, rows, H) != torch.roll(base_q, shift, dims=1)).any()
        bad[3] += (sf_all.view(world, rows, H // 32) != torch.roll(base_sf, shift, dims=1)).any()
        for i in range(4):
            bad[4] += (gathered[i] != torch.bitwise_xor(base_gathered[i], key)).any()
        for d in dispatchers:                                     # the dispatch to owners, both placements, payload xor key
            bad[6] += d.round(key)
        if replay % 100 == 99 or replay == replays - 1:
            torch.cuda.synchronize()
            bad[5] = int(status[0])
            assert not bad.cpu().numpy().any(), ("soak replay %d: mismatching replays [pull, residual, codes, scales, gather4, expired waits, dispatch] = %s, status %s"
                                                 % (replay, bad.cpu().tolist(), status.cpu().tolist()))
    torch.cuda.synchronize(); dist.barrier()
    f = flags.cpu().numpy()
    assert f[0] == (3 + replays) * units and all(f[k] == (3 + replays) * units for k in (1, 2, 3, 4))
    pg.release()
    dist.barrier()
    if rank == 0:
        print("MULTIGPU_OK world=%d soak_replays=%d" % (world, replays))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
