"""World-2 gloo rank for tests/test_host_cpu.py: the peer-table exchange and the row sharding with a
fake allocator (no CUDA), the sharded oracle pipeline reassembled across ranks, and the expert-parallel
dispatch (who owns which expert, which row a routed token lands on) played through on the host."""
import os
import sys
import time

import numpy as np
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in ("kern-k3_b200", "oracle", "tests"):
    sys.path.insert(0, os.path.join(ROOT, p))
import k3o  # noqa: E402
from k3g.peer import PeerGroup, collective_units, shard_rows  # noqa: E402
from util import normal_bf16, rng  # noqa: E402


class FakeAllocator:
    """Addresses are (rank << 40) | serial; a handle is the address as 64 bytes; opening a handle maps
    it at (1 << 60) | address, so own and opened addresses are distinguishable."""

    def __init__(self, rank):
        self.rank, self.n, self.closed, self.freed = rank, 0, [], []

    def alloc(self, nbytes):
        self.n += 1
        return (self.rank << 40) | (self.n << 12)

    def export(self, ptr):
        return int(ptr).to_bytes(64, "little")

    def open(self, handle):
        return (1 << 60) | int.from_bytes(handle, "little")

    def close(self, ptr):
        self.closed.append(ptr)
        self.last_close = time.monotonic()

    def free(self, ptr):
        self.freed.append(ptr)
        self.first_free = min(getattr(self, "first_free", float("inf")), time.monotonic())

    def upload_table(self, addrs):
        return list(addrs)


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    alloc = FakeAllocator(rank)
    pg = PeerGroup(rank, world, allocator=alloc)
    a = pg.symmetric("partial", 1000)
    b = pg.symmetric("flags", 64)
    for buf in (a, b):
        assert buf.nbytes % 256 == 0 and len(buf.table) == world
        for r in range(world):
            if r == rank:
                assert buf.table[r] == buf.ptr and (buf.ptr >> 40) == rank
            else:
                assert buf.table[r] >> 60 == 1 and ((buf.table[r] & ((1 << 60) - 1)) >> 40) == r
    pg.release()
    assert len(alloc.closed) == 2 * (world - 1) and len(alloc.freed) == 2
    # teardown order across ranks: every rank has unmapped its peers' buffers before any rank frees exported memory
    # (freeing memory a peer still has mapped is undefined with CUDA IPC); the monotonic clock is system-wide
    times = [None] * world
    dist.all_gather_object(times, (alloc.last_close, alloc.first_free))
    assert max(t[0] for t in times) <= min(t[1] for t in times), times

    # sharding: rows in block order, one collective grid width for the whole replay
    T, H = 64, 1024
    rows = shard_rows(T, world)
    assert rows == 32 and shard_rows(16384, 4) == 4096 and shard_rows(5, 4) == 2
    assert collective_units(16384, 4) == 896 and collective_units(16384, 8) == 448 and collective_units(1, 4) == 1
    # each rank reduces and normalises its own shard; gathering the shards over gloo reproduces the
    # single-process result
    partials = [normal_bf16(rng(10 + r), (T * H,), std=0.5 / world) for r in range(world)]
    residual = normal_bf16(rng(20), (T, H)); gamma = normal_bf16(rng(21), (H,), mean=1.0, std=0.02)
    delta = k3o.rs_pull(partials, rank, 2 * (world - 1)).reshape(rows, H)
    _, q, sf, _ = k3o.resnorm_mxfp8(residual[rank * rows:(rank + 1) * rows], delta, gamma, 1e-6, want_normed=False)
    gathered = [None] * world
    dist.all_gather_object(gathered, (q, sf))
    q_all = np.concatenate([x[0] for x in gathered]); sf_all = np.concatenate([x[1] for x in gathered])
    total = sum(k3o.bf16_to_f32(p).astype(np.float64) for p in partials).reshape(T, H)
    full_delta = np.concatenate([k3o.rs_pull(partials, r, 2 * (world - 1)).reshape(rows, H) for r in range(world)])
    assert np.allclose(k3o.bf16_to_f32(full_delta), total, rtol=2e-2, atol=1e-2)
    _, q_ref, sf_ref, _ = k3o.resnorm_mxfp8(residual, full_delta, gamma, 1e-6, want_normed=False)
    assert np.array_equal(q_all, q_ref) and np.array_equal(sf_all, sf_ref)
    # expert-parallel dispatch, EP = world: every rank routes its own tokens, the ids are gathered, every rank builds
    # its OWN tables from the gathered ids (the oracle's per-rank tables), and each (token, slot) is delivered by the
    # rank that holds the token to the rank that owns the expert, at the row the owner's tables assign.  What an owner
    # receives must be exactly the live rows of the oracle's expert-sorted gather on the owner's route_map.
    Tt, K, cols, tile = 96, 8, 64, 16
    B, per = Tt // world, 224 // world
    g = rng(30 + rank)
    my_ids = np.stack([g.permutation(224)[:K] for _ in range(B)]).astype(np.int32)
    my_q = g.integers(0, 256, (B, cols), dtype=np.uint8); my_sf = g.integers(0, 256, (B, cols // 32), dtype=np.uint8)
    everyone = [None] * world
    dist.all_gather_object(everyone, (my_ids, my_q, my_sf))
    ids = np.concatenate([e[0] for e in everyone]); q_all_rows = np.concatenate([e[1] for e in everyone]); sf_all_rows = np.concatenate([e[2] for e in everyone])
    tabs = [k3o.moe_route(ids, o, per, world, 1, tile) for o in range(world)]     # every rank can build every owner's tables
    outbox = [[] for _ in range(world)]
    for b in range(B):
        t = rank * B + b
        for k in range(K):
            o = int(ids[t, k]) % world                                # strided placement: owner = id % EP
            row = int(tabs[o]["exp2perm"][t, k])
            assert row >= 0 and all(int(tabs[x]["exp2perm"][t, k]) == -1 for x in range(world) if x != o)   # exactly one owner
            outbox[o].append((row, my_q[b].copy(), my_sf[b].copy()))
    inbox = [None] * world
    dist.all_gather_object(inbox, outbox)
    rows_mine = int(tabs[rank]["total_padded"][0])
    got_q = np.full((rows_mine, cols), 0xEE, np.uint8); got_sf = np.full((rows_mine, cols // 32), 0xEE, np.uint8)
    seen = np.zeros(rows_mine, bool)
    for sender in range(world):
        for row, qr, sr in inbox[sender][rank]:
            assert not seen[row]                                      # every destination row is written once
            seen[row] = True; got_q[row] = qr; got_sf[row] = sr
    want_q, want_sf = k3o.permute_gather(q_all_rows, sf_all_rows, tabs[rank]["route_map"], rows_mine)
    live = np.zeros(rows_mine, bool)
    live[tabs[rank]["exp2perm"][tabs[rank]["exp2perm"] >= 0]] = True
    assert np.array_equal(seen, live) and np.array_equal(got_q[live], want_q[live]) and np.array_equal(got_sf[live], want_sf[live])
    assert sum(int(t["exp2perm"].__ge__(0).sum()) for t in tabs) == Tt * K          # the owners' live rows partition the routed slots
    dist.barrier()
    print("GLOO_OK rank %d" % rank)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
