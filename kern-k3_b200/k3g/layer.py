"""The non-GEMM calls of ONE prefill layer, in the reference's order, with the GEMMs left out.

Mirrors `programs.prefill.calls` of the reference for a KDA layer (labels l1.res_in .. l1.shared_act_quant,
xiaguan/kern-k3 manifests/k3-tp4-prefill-16k.json calls 22-53) and for an MLA layer (calls 86-96: the
span block replaced by mla_prep).  Buffers that a GEMM or attention kernel would produce hold seeded
random data.  This is the program the metric "per-layer glue us at 16k tokens" is measured on: the
whole list replayed as one CUDA graph per rank, plus a per-call breakdown from events.

Shapes follow the reference deployment: H = 7168, MoE latent 3584, 224 experts placed round-robin
(strided, xiaguan/kern-k3 source/k3_moe_prefill_v4.cu:100-109) on an expert-parallel group as wide as the
tensor-parallel one -- EP = W, so 224 / 112 / 56 / 28 local experts at W = 1 / 2 / 4 / 8 and each rank routes,
combines and reduce-scatters T * 16 / W expert rows -- 16 slots per token, 96 attention heads split over the
W ranks, rows sharded T / W.  W = 4 is the reference's own deployment (56 local experts).
"""
import torch

from . import call, current_stream
from .peer import PeerGroup, collective_units, shard_rows

H, LATENT, EXPERTS, TOPK, TILE = 7168, 3584, 224, 16, 128
SHARED = 6144
# grid of an apply-only quantisation launch: every block first reduces the producer's partial maxima, so one resident
# wave of four 256-thread blocks per SM beats the reference op's 2048 (measured: 2 us per call at 16k tokens)
APPLY_GRID = 592


class LayerGlue:
    def __init__(self, rank, world, tokens=16384, kind="kda", nb=4, seed=1, timeout_us=2_000_000, group=None, fused=False):
        assert kind in ("kda", "mla")
        self.rank, self.world, self.T, self.kind, self.nb, self.timeout_us = rank, world, tokens, kind, nb, timeout_us
        self.fused = fused
        self.B = shard_rows(tokens, world)
        assert self.B * world == tokens and 96 % world == 0
        self.heads = 96 // world
        self.inner = 128 * self.heads
        self.units = collective_units(tokens, world, H)
        self.pg = PeerGroup(rank, world, group=group)
        dev = torch.device("cuda")
        g = torch.Generator(device=dev); g.manual_seed(seed * 1000 + rank)
        bf = torch.bfloat16
        T, B, inner = self.T, self.B, self.inner
        rnd = lambda *s, std=1.0: (torch.randn(s, generator=g, device=dev) * std).to(bf)
        rndf = lambda *s, std=1.0: torch.randn(s, generator=g, device=dev) * std
        sym = lambda name, nbytes: self.pg.symmetric(name, nbytes)
        # symmetric (exported) buffers
        self.b_flags = sym("coll_flags", 16 * 8); self.flags = self.b_flags.tensor(torch.int64, (16,))
        self.b_normed_all = sym("normed_all", T * H * 2); self.normed_all = self.b_normed_all.tensor(bf, (T, H))
        self.b_attn_part = sym("attn_part", T * H * 2); self.attn_part = self.b_attn_part.tensor(bf, (T, H))
        self.b_moe_partial = sym("moe_partial", T * LATENT * 2); self.moe_partial = self.b_moe_partial.tensor(bf, (T, LATENT))
        self.b_lq = sym("latent_q_all", T * LATENT); self.latent_q_all = self.b_lq.tensor(torch.uint8, (T, LATENT))
        self.b_lsf = sym("latent_sf_all", T * LATENT // 32); self.latent_sf_all = self.b_lsf.tensor(torch.uint8, (T, LATENT // 32))
        self.b_idx = sym("topk_idx_all", T * TOPK * 4); self.idx_all = self.b_idx.tensor(torch.int32, (T, TOPK))
        self.b_w = sym("topk_weight_all", T * TOPK * 4); self.wts_all = self.b_w.tensor(torch.float32, (T, TOPK))
        self.b_rowmax = sym("rowmax_all", T * 4); self.rowmax_all = self.b_rowmax.tensor(torch.float32, (T,))
        self.rowmax = torch.zeros(B, dtype=torch.float32, device=dev)
        self.item_max = torch.zeros((B * SHARED + 4095) // 4096, dtype=torch.float32, device=dev)
        self.attn_part.copy_(rnd(T, H, std=0.5 / world))
        # residual stream
        self.prefix2, self.p1, self.p2 = rnd(B, H), rnd(B, H, std=0.3), rnd(B, H, std=0.3)
        self.blocks = rnd(B, 8, H)
        self.sw, self.sw_mlp = rndf(H, std=0.05), rndf(H, std=0.05)
        self.gamma = (1 + 0.02 * torch.randn(H, generator=g, device=dev)).to(bf)
        self.hidden = torch.empty((B, H), dtype=bf, device=dev)
        self.stats = torch.zeros((B, 8, 2), dtype=torch.float32, device=dev)
        self.attn_own = torch.empty((B, H), dtype=bf, device=dev)
        self.prefix2_next = torch.empty((B, H), dtype=bf, device=dev)
        self.normed = torch.empty((B, H), dtype=bf, device=dev)
        # per-tensor fp8 operands
        self.fp8_big = torch.empty((T, H), dtype=torch.uint8, device=dev)
        self.fp8_small = torch.empty((B, H), dtype=torch.uint8, device=dev)
        self.qpart = torch.zeros(2048, dtype=torch.float32, device=dev); self.qscale = torch.zeros(4, dtype=torch.float32, device=dev)
        self.shared_partial = rnd(B, 2 * SHARED, std=2.0); self.shared_act = torch.empty((B, SHARED), dtype=bf, device=dev)
        self.shared_q = torch.empty((B, SHARED), dtype=torch.uint8, device=dev)
        self.gamma_lat = self.gamma[:LATENT].contiguous(); self.routed_latent_norm = torch.empty((B, LATENT), dtype=bf, device=dev)
        # attention block
        if kind == "kda":
            self.kda_partial = rnd(T, 4 * inner)
            self.cw = rndf(3, 4, inner, std=0.5)
            self.win = torch.zeros((3, 3, inner), dtype=bf, device=dev)
            self.wsm = rndf(T, 256)
            self.span_q, self.span_k, self.span_v = (torch.empty((T, inner), dtype=bf, device=dev) for _ in range(3))
            self.beta = torch.empty((self.heads, T), dtype=bf, device=dev); self.flow = torch.empty((T, 128), dtype=bf, device=dev)
            self.gamma_o = torch.ones(128, device=dev)
            self.gated = torch.empty((T, inner), dtype=bf, device=dev)
            self.state_lines = torch.zeros(self.heads * 128 * 128 * 4 + 3 * 3 * inner * 2, dtype=torch.uint8, device=dev)
            self.state_buf = torch.zeros(self.heads * 128 * 128, dtype=torch.float32, device=dev)
            self.line_index = torch.zeros(T, dtype=torch.int32, device=dev); self.span_at = torch.zeros(1, dtype=torch.int32, device=dev)
        else:
            self.mla_partial = rnd(T, 2112 + inner)
            self.gq, self.gkv = self.gamma[:1536].contiguous(), self.gamma[:512].contiguous()
            self.slots = torch.arange(T, dtype=torch.int64, device=dev)
            self.slab = torch.zeros((T // 64) * 64 * 576, dtype=bf, device=dev)
            self.q_norm = torch.empty((T, 1536), dtype=bf, device=dev); self.mla_gate = torch.empty((T, inner), dtype=bf, device=dev)
            self.block_table = torch.arange(T // 64, dtype=torch.int32, device=dev); self.lens = torch.tensor([T], dtype=torch.int32, device=dev)
            self.latent_rows = torch.empty((T, 576), dtype=bf, device=dev)
            self.fmha_out = rnd(T, inner); self.attn_gated = torch.empty((T, inner), dtype=bf, device=dev)
        # MoE
        self.logits = rndf(B, EXPERTS); self.bias = rndf(EXPERTS, std=0.1); self.rs = torch.ones(1, dtype=bf, device=dev)
        self.idx = torch.empty((B, TOPK), dtype=torch.int32, device=dev); self.wts = torch.empty((B, TOPK), dtype=torch.float32, device=dev)
        self.latent = rnd(B, LATENT)
        self.latent_q = torch.empty((B, LATENT), dtype=torch.uint8, device=dev); self.latent_sf = torch.empty((B, LATENT // 32), dtype=torch.uint8, device=dev)
        self.ep = world                      # expert-parallel group = tensor-parallel group
        self.E = EXPERTS // self.ep
        nblk = (T + 255) // 256
        nct = T * TOPK // TILE + self.E
        i32 = lambda *s: torch.zeros(s, dtype=torch.int32, device=dev)
        self.blockcount, self.blockoff = i32(nblk, self.E), i32(nblk, self.E)
        self.cta_batch, self.cta_limit, self.nne, self.total = i32(nct), i32(nct), i32(1), i32(1)
        self.route_map, self.exp2perm = i32(nct * TILE), i32(T, TOPK)
        self.fc2 = rnd(nct * TILE, LATENT)
        self.routed_latent = torch.empty((B, LATENT), dtype=bf, device=dev)
        self.status = torch.zeros(4, dtype=torch.int32, device=dev)
        call("k3g_flags_init", self.flags, 16, current_stream())
        torch.cuda.synchronize()
        self.graph = None

    # ---- the call list ---------------------------------------------------------------------------
    def calls(self):
        s = current_stream
        W, r, T, B, inner, heads, nb = self.world, self.rank, self.T, self.B, self.inner, self.heads, self.nb
        ft, fl, un, to, st = self.b_flags.table, self.flags, self.units, self.timeout_us, self.status
        ep_rank, EP = r, self.ep
        c = [("coll_epoch", lambda: call("k3g_epoch_bump", fl, un, s())),
             ("res_in (land_add2 + attnres + rms + push)", lambda: call(
                 "k3g_attnres_rms_push", self.blocks, self.sw, self.gamma, self.normed_all, self.b_normed_all.table, nb, 0, B, r, W, self.sw_mlp,
                 self.stats, self.p1, self.p2, self.prefix2, self.hidden, 1, H, 1e-5, s())),
             ("normed_sync (arrive)", lambda: call("k3g_rs_arrive", fl, ft, un, 1, W, to, st, s())),
             ("qkvg_quant (fp8 tensor, T rows)", lambda: call("k3g_quant_fp8_tensor", self.normed_all, self.fp8_big, self.qscale, self.qpart, T * H, 2048, s()))]
        if self.kind == "kda":
            c += [("span_gather (conv4 + SiLU, beta, flow)", lambda: call(
                      "k3g_span_gather", self.kda_partial, 4 * inner, self.cw, 0, self.win, self.wsm, self.span_q, self.span_k, self.span_v, self.beta,
                      self.flow, heads, 0, T, 0, s())),
                  ("span_state_in + span_state_out (2 copies)", lambda: (
                      call("k3g_span_state", self.state_lines, self.line_index, self.state_lines.numel(), self.span_at, self.state_buf, 0, heads, s()),
                      call("k3g_span_state", self.state_lines, self.line_index, self.state_lines.numel(), self.span_at, self.state_buf, 1, heads, s()))),
                  ("span_out_gate", lambda: call("k3g_kda_out_gate", self.span_v, self.kda_partial, 4 * inner, 3 * inner, self.gamma_o, self.gated, None,
                                                 None, heads, 0, T, 1e-5, s()))]
        else:
            c += [("mla_prep (head + gate)", lambda: call("k3g_mla_prep", self.mla_partial, 1, self.gq, self.gkv, self.slots, self.slab, 0, 64 * 576,
                                                          self.q_norm, self.mla_gate, T, inner, 1e-5, s())),
                  ("latent_gather", lambda: call("k3g_latent_gather", self.slab, self.block_table, 64 * 576, self.lens, self.latent_rows, T, s())),
                  ("mla_gate (sigmoid_mul)", lambda: call("k3g_sigmoid_mul", self.attn_gated, self.fmha_out, self.mla_gate, T, heads, 128, inner, 128, s()))]
        c += [("reduce_attn (arrive)", lambda: call("k3g_rs_arrive", fl, ft, un, 2, W, to, st, s())),
              ("reduce_attn (pull RS)", lambda: call("k3g_rs_pull", self.attn_part, self.attn_own, self.b_attn_part.table, B * H, 2 * (W - 1), r, W, un, s())),
              ("res_mlp (land + attnres + rms, stats)", lambda: call(
                  "k3g_land_add_attnres_rms_stats", self.attn_own, 1, self.hidden, self.blocks, self.sw_mlp, self.gamma, self.prefix2_next, self.normed,
                  nb, 0, B, H, 1e-5, self.stats, nb, s())),
              ("normed_quant (fp8 tensor, B rows)", lambda: call("k3g_quant_fp8_tensor", self.normed, self.fp8_small, self.qscale[1:], self.qpart, B * H, 2048, s())),
              ("topk (router)", lambda: call("k3g_router_topk", self.logits, self.bias, self.rs, self.idx, self.wts, B, EXPERTS, TOPK, s())),
              ("moe_quant (MXFP8 latent)", lambda: call("k3g_moe_quant", self.latent, self.latent_q, self.latent_sf, B, LATENT, 0, s())),
              ("gather_small (AG4 push + barrier)", lambda: call(
                  "k3g_allgather4_push", self.latent_q, self.latent_q_all, self.b_lq.table, B * LATENT, self.latent_sf, self.latent_sf_all,
                  self.b_lsf.table, B * LATENT // 32, self.idx, self.idx_all, self.b_idx.table, B * TOPK * 4, self.wts, self.wts_all, self.b_w.table,
                  B * TOPK * 4, fl, ft, 3, r, W, un, to, st, s())),
              ("route_count", lambda: call("k3g_moe_route_count", self.idx_all, T, ep_rank, self.E, TOPK, EP, 1, self.blockcount, s())),
              ("route_tables", lambda: call("k3g_moe_route_tables", self.blockcount, (T + 255) // 256, self.E, TILE, self.blockoff, self.cta_batch,
                                            self.cta_limit, self.nne, self.total, self.route_map, s())),
              ("route_scatter", lambda: call("k3g_moe_route_scatter", self.idx_all, self.blockoff, T, ep_rank, self.E, TOPK, EP, 1, self.route_map,
                                             self.exp2perm, s())),
              ("finalize", lambda: call("k3g_moe_finalize", self.fc2, self.exp2perm, self.wts_all, self.moe_partial, T, LATENT, TOPK, s())),
              ("scatter_moe (arrive)", lambda: call("k3g_rs_arrive", fl, ft, un, 4, W, to, st, s())),
              ("scatter_moe (pull RS)", lambda: call("k3g_rs_pull", self.moe_partial, self.routed_latent, self.b_moe_partial.table, B * LATENT,
                                                     2 * (W - 1), r, W, un, s())),
              ("shared_situ (SiTU landing + latent RMSNorm)", lambda: call("k3g_situ_rms", self.shared_partial, self.shared_act, self.routed_latent,
                                                                           self.gamma_lat, self.routed_latent_norm, SHARED, B, LATENT, B, s())),
              ("shared_act_quant (fp8 tensor)", lambda: call("k3g_quant_fp8_tensor", self.shared_act, self.shared_q, self.qscale[2:], self.qpart, B * SHARED,
                                                             2048, s()))]
        if self.fused:
            # Fusions beyond the reference's call list, all with bit-identical outputs:
            #  - the producers leave the maxima a per-tensor quantisation needs, so the three quantisations run
            #    their apply launch only (one pass over each tensor less);
            #  - the latent MXFP8 quantisation writes straight into every rank's gathered buffers (one launch with the
            #    small all-gather; a thread's 32 codes leave as one 32-byte store per rank, a full sector on the links);
            #  - the attention reduce-scatter is pulled inside the residual kernel that consumes it and the routed-latent
            #    reduce-scatter inside the latent norm, so their HBM / special-function work hides under the NVLink
            #    transfer and the reduce-scattered tensors are never written.
            #  - the epoch bump rides in the first barrier launch and the routing tables are built inside the scatter
            #    launch (two launches fewer, same tables).
            swap = {
                "coll_epoch": None,
                "normed_sync (arrive)": ("normed_sync (epoch + arrive)", lambda: call("k3g_epoch_arrive", fl, ft, un, 1, W, to, st, s())),
                "route_tables": None,
                "route_scatter": ("route_tables + route_scatter (one launch)", lambda: call(
                    "k3g_moe_route_tables_scatter", self.idx_all, self.blockcount, T, ep_rank, self.E, TOPK, EP, 1, TILE, self.blockoff,
                    self.cta_batch, self.cta_limit, self.nne, self.total, self.route_map, self.exp2perm, s())),
                "res_in (land_add2 + attnres + rms + push)": ("res_in (land_add2 + attnres + rms + push, row maxima)", lambda: call(
                    "k3g_attnres_rms_push_amax", self.blocks, self.sw, self.gamma, self.normed_all, self.b_normed_all.table, nb, 0, B, r, W,
                    self.sw_mlp, self.stats, self.p1, self.p2, self.prefix2, self.hidden, 1, H, 1e-5, self.rowmax_all, self.b_rowmax.table, s())),
                "qkvg_quant (fp8 tensor, T rows)": ("qkvg_quant (fp8 apply only, T rows)", lambda: call(
                    "k3g_quant_fp8_apply", self.normed_all, self.fp8_big, self.qscale, self.rowmax_all, T, T * H, APPLY_GRID, s())),
                "reduce_attn (pull RS)": None,
                "res_mlp (land + attnres + rms, stats)": ("reduce_attn + res_mlp (pull RS inside land + attnres + rms, stats, row maxima)", lambda: call(
                    "k3g_rs_land_add_attnres_rms", self.attn_part, self.b_attn_part.table, r, W, self.hidden, self.blocks, self.sw_mlp, self.gamma,
                    self.prefix2_next, self.normed, nb, 0, B, H, 1e-5, self.stats, nb, self.rowmax, s())),
                "normed_quant (fp8 tensor, B rows)": ("normed_quant (fp8 apply only, B rows)", lambda: call(
                    "k3g_quant_fp8_apply", self.normed, self.fp8_small, self.qscale[1:], self.rowmax, B, B * H, APPLY_GRID, s())),
                "moe_quant (MXFP8 latent)": None,
                "gather_small (AG4 push + barrier)": ("moe_quant + gather_small (MXFP8 written straight into every rank's gathered buffers + barrier)",
                                                      lambda: call(
                    "k3g_moe_quant_allgather_push", self.latent, B, LATENT, self.latent_q_all, self.b_lq.table, self.latent_sf_all, self.b_lsf.table,
                    self.idx, self.idx_all, self.b_idx.table, B * TOPK * 4, self.wts, self.wts_all, self.b_w.table, B * TOPK * 4, fl, ft, 3, r, W, un,
                    to, st, s())),
                "scatter_moe (pull RS)": None,
                "shared_situ (SiTU landing + latent RMSNorm)": ("scatter_moe + shared_situ (pull RS inside the latent RMSNorm, SiTU landing, item maxima)",
                                                                lambda: call(
                    "k3g_rs_situ_rms", self.shared_partial, self.shared_act, self.moe_partial, self.b_moe_partial.table, r, W, self.gamma_lat,
                    self.routed_latent_norm, SHARED, B, LATENT, B, self.item_max, s())),
                "shared_act_quant (fp8 tensor)": ("shared_act_quant (fp8 apply only)", lambda: call(
                    "k3g_quant_fp8_apply", self.shared_act, self.shared_q, self.qscale[2:], self.item_max, self.item_max.numel(), B * SHARED, APPLY_GRID,
                    s())),
            }
            c = [swap.get(label, (label, fn)) for label, fn in c if swap.get(label, 0) is not None]
        return c

    def traffic(self):
        """label prefix -> (HBM bytes, NVLink bytes per direction) per rank: the unique bytes a call must move through this
        GPU's HBM and must receive / send over NVLink (0 at world 1); small table kernels have neither."""
        W, T, B, inner, nb = self.world, self.T, self.B, self.inner, self.nb
        EB, ET = B * H * 2, T * H * 2                       # one bf16 pass over the shard / over all rows
        link = lambda nbytes: (W - 1) * nbytes
        small = B * (LATENT + LATENT // 32 + 2 * TOPK * 4)
        t = {
            "coll_epoch": (0, 0), "normed_sync": (0, 0), "reduce_attn (arrive)": (0, 0), "scatter_moe (arrive)": (0, 0),
            "res_in": ((3 + 2 * nb + 2) * EB, link(EB)),
            "qkvg_quant": (3 * ET // 2, 0),
            "span_gather": (T * 3 * inner * 4 + T * 256 * 4, 0), "span_state_in": (0, 0),
            "span_out_gate": (T * inner * 6, 0),
            "mla_prep": (T * ((2112 + inner) * 2 + (1536 + 576 + inner) * 2), 0), "latent_gather": (T * 576 * 4, 0),
            "mla_gate": (T * inner * 6, 0),
            "reduce_attn (pull RS)": (2 * EB, link(EB)),
            "res_mlp": ((4 + nb) * EB, 0),
            "reduce_attn + res_mlp": ((4 + nb) * EB, link(EB)),
            "normed_quant": (3 * EB // 2, 0), "topk": (0, 0),
            "moe_quant (": (B * LATENT * 3 + B * LATENT // 32, 0),
            "gather_small": (2 * small, link(small)),
            "moe_quant + gather_small": (B * LATENT * 3, link(small)),
            "route_count": (0, 0), "route_tables": (0, 0), "route_scatter": (0, 0),
            "finalize": ((T * TOPK // self.ep + T) * LATENT * 2, 0),
            "scatter_moe (pull RS)": (2 * B * LATENT * 2, link(B * LATENT * 2)),
            "shared_situ": (B * (SHARED * 6 + LATENT * 4), 0),
            "scatter_moe + shared_situ": (B * (SHARED * 6 + LATENT * 4), link(B * LATENT * 2)),
            "shared_act_quant": (3 * B * SHARED, 0),
        }
        return t

    def traffic_of(self, label, hbm_gbs=6529.7, link_gbs=770.0):
        """(bytes, bound) of the call: the resource whose roofline time is larger -- "hbm", "nvlink" or "latency"."""
        best = None
        for k, v in self.traffic().items():
            if label.startswith(k) and (best is None or len(k) > len(best[0])):
                best = (k, v)
        if best is None:
            return 0, "latency"
        hbm, lnk = best[1]
        if hbm == 0 and lnk == 0:
            return 0, "latency"
        return (lnk, "nvlink") if lnk / link_gbs > hbm / hbm_gbs else (hbm, "hbm")

    def launches(self):
        """Kernel launches of one pass of the call list (a two-pass quantisation and the pair of state copies are two each)."""
        two = ("(fp8 tensor", "span_state_in + span_state_out")
        return sum(2 if any(k in label for k in two) else 1 for label, _ in self.calls())

    def run(self):
        for _, fn in self.calls():
            fn()

    def run_timed(self):
        """One pass with an event between every call; returns [(label, start_event, end_event)]."""
        out = []
        prev = torch.cuda.Event(enable_timing=True); prev.record()
        for label, fn in self.calls():
            fn()
            e = torch.cuda.Event(enable_timing=True); e.record()
            out.append((label, prev, e))
            prev = e
        return out

    def capture(self):
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self.run()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.run()

    def replay(self):
        self.graph.replay()

    def check_status(self):
        stt = self.status.cpu().tolist()
        if stt[0] != 0:
            raise RuntimeError("a collective wait expired: slot %d, peer %d, observed counter %d" % (stt[1], stt[2], stt[3]))

    def close(self):
        torch.cuda.synchronize()
        self.pg.release()
