"""Worker of tests/test_multigpu.py: one rank of a world-W run of the collective kernels, checked
against the CPU oracle.  Every rank regenerates every rank's seeded inputs, so no data is exchanged
besides the IPC handles."""
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

    for replay in range(3):
        q_all.zero_(); sf_all.zero_()
        torch.cuda.synchronize(); dist.barrier()
        k3g.call("k3g_epoch_bump", flags, units, s)
        # unfused: arrive, pull reduce-scatter
        k3g.call("k3g_rs_arrive", flags, b_flags.table, units, 1, world, 5_000_000, status, s)
        dst = torch.zeros(rows * H, dtype=torch.bfloat16, device=dev)
        k3g.call("k3g_rs_pull", part, dst, b_part.table, rows * H, 2 * (world - 1), rank, world, units, s)
        # fused: arrive (partials ready), fused kernel, arrive (pushes landed)
        k3g.call("k3g_rs_arrive", flags, b_flags.table, units, 2, world, 5_000_000, status, s)
        res_out = torch.zeros((rows, H), dtype=torch.bfloat16, device=dev)
        k3g.call("k3g_rs_resnorm_mxfp8_ag", part, b_part.table, to_dev_bf16(residual[rank], dev), to_dev_bf16(gamma, dev), res_out, q_all,
                 b_q.table, sf_all, b_sf.table, rows, H, 1e-6, rank, world, 0, 0, 0, s)
        k3g.call("k3g_rs_arrive", flags, b_flags.table, units, 3, world, 5_000_000, status, s)
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
            k3g.call("k3g_rs_land_add_attnres_rms", part, b_part.table, rank, world, to_dev_bf16(residual[rank], dev), to_dev_bf16(blocks_h, dev),
                     to_dev(sw_h, dev), to_dev_bf16(gamma, dev), p2, nrm, nb, 0, rows, H, 1e-5, None, 0, rowmax, s)
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
        srcs = [torch.from_numpy(rng(50 + rank * 4 + i).integers(0, 256, n, dtype=np.uint8)).to(dev) for i, n in enumerate((rows * 3584, rows * 112, rows * 64, rows * 64))]
        if replay == 0:
            bufs = [pg.symmetric("ag%d" % i, world * t.numel()) for i, t in enumerate(srcs)]
        a = []
        for t, b in zip(srcs, bufs):
            a += [t, b.ptr, b.table, t.numel()]
        k3g.call("k3g_allgather4_push", *a, flags, b_flags.table, 4, rank, world, units, 5_000_000, status, s)
        torch.cuda.synchronize()
        assert not status.cpu().numpy().any(), status
        for i, b in enumerate(bufs):
            n = srcs[i].numel()
            got = b.tensor(torch.uint8, (world * n,)).cpu().numpy()
            want = np.concatenate([rng(50 + r * 4 + i).integers(0, 256, n, dtype=np.uint8) for r in range(world)])
            assert np.array_equal(got, want), i
        dist.barrier()
    f = flags.cpu().numpy()
    assert f[0] == 3 * units and all(f[k] == 3 * units for k in (1, 2, 3, 4))
    pg.release()
    dist.barrier()
    if rank == 0:
        print("MULTIGPU_OK world=%d" % world)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
