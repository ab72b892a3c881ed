"""Host-side program for one tensor-parallel glue step (benchmark configuration 1):

    epoch bump -> arrive (partials ready) -> fused pull reduce-scatter + residual add + RMSNorm +
    MXFP8 + push all-gather -> arrive (pushes landed)

mirroring, call for call, the slice `reduce_attn -> res_mlp -> quant -> gather` of the reference's
`programs.prefill` (xiaguan/kern-k3 manifests/k3-tp4-prefill-16k-l0-bf16.json, calls l1.reduce_attn
.. l1.gather_*), with the collectives done in-kernel over NVLink peer pointers.  All device work
goes through the C ABI; this module only owns buffers and the launch order.
"""
import torch

from . import call, current_stream
from .peer import PeerGroup, collective_units, shard_rows

SLOT_PARTIALS_READY = 1
SLOT_PUSH_LANDED = 2
N_FLAGS = 16
LAUNCHES_PER_STEP = 4


class TpGlue:
    def __init__(self, rank, world, tokens, H=7168, eps=1e-6, timeout_us=2_000_000, group=None):
        self.rank, self.world, self.tokens, self.H, self.eps, self.timeout_us = rank, world, tokens, H, eps, timeout_us
        self.rows = shard_rows(tokens, world)
        assert self.rows * world == tokens, "tokens must divide evenly across ranks"
        self.units = collective_units(tokens, world, H)
        self.pg = PeerGroup(rank, world, group=group)
        T = tokens
        self._b_partial = self.pg.symmetric("partial", T * H * 2)
        self._b_q = self.pg.symmetric("q_all", T * H)
        self._b_sf = self.pg.symmetric("sf_all", T * H // 32)
        self._b_flags = self.pg.symmetric("flags", N_FLAGS * 8)
        self.partial = self._b_partial.tensor(torch.bfloat16, (T, H))
        self.q_all = self._b_q.tensor(torch.uint8, (T, H))
        self.sf_all = self._b_sf.tensor(torch.uint8, (T, H // 32))
        self.flags = self._b_flags.tensor(torch.int64, (N_FLAGS,))
        dev = self.partial.device
        self.residual = torch.zeros((self.rows, H), dtype=torch.bfloat16, device=dev)
        self.residual_out = torch.empty_like(self.residual)
        self.gamma = torch.ones((H,), dtype=torch.bfloat16, device=dev)
        self.status = torch.zeros(4, dtype=torch.int32, device=dev)
        call("k3g_flags_init", self.flags, N_FLAGS, current_stream())
        torch.cuda.synchronize()
        self.kernel_events = None      # set to a list to collect (start, end) events around the fused kernel

    def step(self, grid_hint=0, row_begin=0, rows=None):
        """One glue step on device-resident inputs (self.partial, self.residual, self.gamma); with
        row_begin / rows, one protocol round over that row chunk of every rank's shard."""
        s = current_stream()
        rows = self.rows if rows is None else rows
        call("k3g_epoch_bump", self.flags, self.units, s)
        call("k3g_rs_arrive", self.flags, self._b_flags.table, self.units, SLOT_PARTIALS_READY, self.world, self.timeout_us, self.status, s)
        if self.kernel_events is not None:
            e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
            e0.record()
        call("k3g_rs_resnorm_mxfp8_ag", self.partial, self._b_partial.table, self.residual, self.gamma, self.residual_out, self.q_all,
             self._b_q.table, self.sf_all, self._b_sf.table, rows, self.H, self.eps, self.rank, self.world, grid_hint, row_begin, self.rows, s)
        if self.kernel_events is not None:
            e1.record()
            self.kernel_events.append((e0, e1))
        call("k3g_rs_arrive", self.flags, self._b_flags.table, self.units, SLOT_PUSH_LANDED, self.world, self.timeout_us, self.status, s)

    def capture(self):
        """Capture step() into a CUDA graph (the reference replays its whole program as one graph per
        rank); collective on every rank, because the warm-up step runs the flag protocol."""
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self.step()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        keep, self.kernel_events = self.kernel_events, None
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.step()
        self.kernel_events = keep

    def replay(self):
        self.graph.replay()

    def step_host(self, host_partial, host_residual, host_residual_out, host_q_all, host_sf_all):
        """The same step with HOST (pinned) inputs and outputs: copies in, step, copies out."""
        self.partial.copy_(host_partial, non_blocking=True)
        self.residual.copy_(host_residual, non_blocking=True)
        self.replay() if getattr(self, "graph", None) is not None else self.step()
        host_residual_out.copy_(self.residual_out, non_blocking=True)
        host_q_all.copy_(self.q_all, non_blocking=True)
        host_sf_all.copy_(self.sf_all, non_blocking=True)

    @staticmethod
    def chunk_bounds(rows, chunks, taper=3):
        """Row ranges [r0, r1) of the host pipeline: `chunks` equal parts, the last of them cut again into
        1/2, 1/4, ... (`taper` halvings) of a part.  The link into the device is the bottleneck, so what is left once the
        last copy in has landed -- the last chunk's kernels and its copy out -- is the only part of the pipeline nothing
        overlaps: the smaller the last chunk, the shorter that tail."""
        part = max(1, (rows + chunks - 1) // chunks)
        bounds, r = [], 0
        while rows - r > part:
            bounds.append((r, r + part)); r += part
        left = rows - r
        for _ in range(taper):
            piece = left // 2
            if piece < 1:
                break
            bounds.append((r, r + piece)); r += piece; left -= piece
        if left > 0:
            bounds.append((r, rows))
        return bounds

    def step_host_pipelined(self, host_partial, host_residual, host_residual_out, host_q_all, host_sf_all, chunks=8, taper=3):
        """step_host with the shard cut into row chunks (chunk_bounds: equal parts with a tapered tail) and three
        streams: while chunk c is reduced, normalised and gathered, chunk c + 1 is on its way in and chunk c - 1 on its
        way out, so the host link is busy in both directions at once.  Each chunk is a full protocol round (epoch bump,
        arrive, fused kernel over rows [r0, r1) of every shard, arrive)."""
        if not hasattr(self, "_s_in"):
            self._s_in, self._s_cmp, self._s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
        cur = torch.cuda.current_stream()
        start = torch.cuda.Event(); start.record(cur)
        for st in (self._s_in, self._s_cmp, self._s_out):
            st.wait_event(start)
        R, W = self.rows, self.world
        for r0, r1 in self.chunk_bounds(R, chunks, taper):
            with torch.cuda.stream(self._s_in):
                for q in range(W):
                    self.partial[q * R + r0:q * R + r1].copy_(host_partial[q * R + r0:q * R + r1], non_blocking=True)
                self.residual[r0:r1].copy_(host_residual[r0:r1], non_blocking=True)
                ev_in = torch.cuda.Event(); ev_in.record(self._s_in)
            with torch.cuda.stream(self._s_cmp):
                self._s_cmp.wait_event(ev_in)
                self.step(row_begin=r0, rows=r1 - r0)
                ev_done = torch.cuda.Event(); ev_done.record(self._s_cmp)
            with torch.cuda.stream(self._s_out):
                self._s_out.wait_event(ev_done)
                host_residual_out[r0:r1].copy_(self.residual_out[r0:r1], non_blocking=True)
                for q in range(W):
                    host_q_all[q * R + r0:q * R + r1].copy_(self.q_all[q * R + r0:q * R + r1], non_blocking=True)
                    host_sf_all[q * R + r0:q * R + r1].copy_(self.sf_all[q * R + r0:q * R + r1], non_blocking=True)
        end = torch.cuda.Event(); end.record(self._s_out)
        cur.wait_event(end)

    def h2d_bytes(self):
        return self.tokens * self.H * 2 + self.rows * self.H * 2

    def d2h_bytes(self):
        return self.rows * self.H * 2 + self.tokens * self.H + self.tokens * self.H // 32

    def check_status(self):
        st = self.status.cpu().tolist()
        if st[0] != 0:
            raise RuntimeError("a collective wait expired: slot %d, peer %d, observed counter %d" % (st[1], st[2], st[3]))

    def close(self):
        torch.cuda.synchronize()
        self.pg.release()
