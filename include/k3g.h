/* k3g — B200 (sm_100a) kernels for the non-GEMM glue of K3 MoE prefill, C ABI.
 *
 * Drop-in boundary.  The reference project (xiaguan/kern-k3) has no host API: its unit of
 * replacement is a cubin whose `extern "C" __global__` entries a manifest-driven runtime
 * launches with caller-owned device buffers (README.md:32-34).  This library exposes the
 * same operators two ways:
 *   (1) lib/cubin/<module>.cubin — entries with the reference's names and parameter lists;
 *   (2) the functions below — one host launcher per manifest op, taking the op's kernel
 *       parameters in the reference's order, then the deployment constants the reference
 *       fixes at compile time (row width, eps, world size ...), then the CUDA stream.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer owned by the caller unless its name starts with
 *     `host_`; the launchers neither allocate, free nor synchronise and can be captured into a CUDA
 *     graph.  The exceptions are named where they are declared: k3g_wait_status (copies 16 bytes
 *     to the host and synchronises the stream), the k3g_peer_* set-up helpers (allocate / map),
 *     the first k3g_moe_route_scatter call with more than 64 local experts on a device (raises the
 *     kernel's shared-memory limit once) and the first k3g_quant_fp8_tensor_noalloc call on a device;
 *   - bf16 / e4m3 / ue8m0 buffers are passed as void*;
 *   - `stream` is a cudaStream_t (void* 0 = the legacy default stream);
 *   - return value: 0 ok; < 0 argument rejected before any launch (K3G_E*); > 0 cudaError_t.
 */
#ifndef K3G_H
#define K3G_H

#ifdef __cplusplus
extern "C" {
#endif

#define K3G_ENULL (-1)  /* a required pointer is null */
#define K3G_ESHAPE (-2) /* unsupported size (row width, world size, count alignment) */
#define K3G_EALIGN (-3) /* pointer not 16-byte aligned */
#define K3G_ERANGE (-4) /* rank / slot / nb / order out of range */
#define K3G_ELIMIT (-5) /* size beyond a built-in maximum */

/* ---- residual stream --------------------------------------------------------------------- */

/* Fused residual add + RMSNorm + MXFP8 (benchmark configuration 0).  Composition of
 * kern_k3_land_add_attnres_rms with nb = 0 (source/k3_residual_v2.cu:295-345, :224-256) and
 * kern_k3_moe_quant (source/k3_moe_prefill_v4.cu:111-140) in one pass:
 *   residual_out = bf16(residual + delta); normed = bf16(bf16(residual_out * r) * gamma);
 *   q = E4M3 codes of normed, sf = one UE8M0 byte per 32 elements ([rows, H/32]).
 * normed_opt may be null.  H in {1024, 2048, 4096, 7168, 8192}.  grid_hint <= 0: one block per row. */
int k3g_resnorm_mxfp8(const void* residual, const void* delta, const void* gamma, void* residual_out, void* q,
                      void* sf, void* normed_opt, int rows, int H, float eps, int grid_hint, void* stream);

/* kern_k3_attnres_rms, source/k3_residual_v2.cu:260 (op attnres_rms_v2). */
int k3g_attnres_rms(const void* prefix, void* blocks, const void* sw, const void* gamma, void* normed, int nb,
                    int snapshot, int B, int H, float eps, void* stream);

/* kern_k3_land_add_attnres_rms, source/k3_residual_v2.cu:295 (op land_add_attnres_rms_bf16_v2;
 * partial_is_bf16 = the LAND_BF16 build). */
int k3g_land_add_attnres_rms(const void* partial, int partial_is_bf16, const void* prefix, const void* blocks,
                             const void* sw, const void* gamma, void* prefix2, void* normed, int nb, int snapshot,
                             int B, int H, float eps, void* stream);

/* kern_k3_land_add_attnres_rms_nb1..8, source/k3_residual_nb_stats.cu:366-842 (ops
 * land_add_attnres_rms_bf16_v2_nb{1..8}): the same kernel with the statistics hand-off -- stats [B, 8, 2]
 * f32 = (sum x^2, sum x * sw) of the snapshot candidates c < nb_stats, written by k3g_attnres_rms_push. */
int k3g_land_add_attnres_rms_stats(const void* partial, int partial_is_bf16, const void* prefix, const void* blocks,
                                   const void* sw, const void* gamma, void* prefix2, void* normed, int nb, int snapshot,
                                   int B, int H, float eps, const void* stats, int nb_stats, void* stream);

/* kern_k3_attnres_rms_push, source/k3_residual_push_add2.cu:369 (op attnres_rms_push_add2): landing add
 * (hidden = bf16(prefix2 + p1 (+ p2))), optional snapshot, attention-residual mix, RMSNorm, and the normed
 * row pushed into this rank's slice of every rank's normed_all [nranks * B, H] (dst_peer = peer table of
 * normed_all).  stats (may be null) receives (sum x^2, sum x * sw_mlp) per snapshot candidate.  The
 * all-gather's barrier is a separate k3g_rs_arrive.  p1 == NULL selects the first layer's form
 * (kern_k3_attnres_rms_push of source/k3_residual_push_v3.cu:328, op attnres_rms_push_first_v3): the row
 * is prefix2 itself, nothing is added and hidden is not written. */
int k3g_attnres_rms_push(void* blocks, const void* sw, const void* gamma, void* normed_all, const void* dst_peer, int nb,
                         int snapshot, int B, int rank, int nranks, const void* sw_mlp, void* stats, const void* p1,
                         const void* p2, const void* prefix2, void* hidden, int two, int H, float eps, void* stream);

/* Producer-side maxima for a following per-tensor FP8 quantisation (no counterpart in the reference, which
 * always runs the two-pass pair): the same kernels also store max |output| per row (per 4096 elements for
 * SiTU) as non-negative f32, and k3g_quant_fp8_apply consumes them in place of the amax pass.  Outputs of the
 * kernels themselves are unchanged; the quantised result is bit-identical to k3g_quant_fp8_tensor.
 *   k3g_attnres_rms_push_amax: rowmax_all [nranks * B] f32 on every rank (rowmax_peer = u64 peer table),
 *                              index rank * B + b, pushed like the row itself.
 *   k3g_land_add_attnres_rms_stats_amax: rowmax [B] f32.
 *   k3g_situ_rms_amax: item_max [ceil(B * n / 4096)] f32. */
int k3g_attnres_rms_push_amax(void* blocks, const void* sw, const void* gamma, void* normed_all, const void* dst_peer, int nb,
                              int snapshot, int B, int rank, int nranks, const void* sw_mlp, void* stats, const void* p1,
                              const void* p2, const void* prefix2, void* hidden, int two, int H, float eps, void* rowmax_all,
                              const void* rowmax_peer, void* stream);
int k3g_land_add_attnres_rms_stats_amax(const void* partial, int partial_is_bf16, const void* prefix, const void* blocks,
                                        const void* sw, const void* gamma, void* prefix2, void* normed, int nb, int snapshot,
                                        int B, int H, float eps, const void* stats, int nb_stats, void* rowmax, void* stream);
int k3g_situ_rms_amax(const void* sp, void* act, const void* lat, const void* gam, void* ln, int n, int B, int h, int L, void* item_max,
                      void* stream);
int k3g_quant_fp8_apply(const void* x, void* y, void* scale_out, const void* partials, int nparts, int n, int grid, void* stream);

/* Pull reduce-scatter folded into the residual kernel that consumes it (no counterpart in the reference, which runs
 * kern_k3_rs_pull, source/k3_reducescatter_pull_nr4.cu:124, and then kern_k3_land_add_attnres_rms_nbK): partial =
 * this rank's [nranks * B, H] bf16 partial sums, partial_peer = u64 table of every rank's buffer.  Row b lands the
 * ring-order chain of row rank * B + b (k3g_rs_pull with order 2 (nranks - 1)) and continues as
 * k3g_land_add_attnres_rms_stats_amax; outputs are bit-identical to the two calls in sequence, the reduce-scattered
 * tensor is never written.  Bracket with k3g_rs_arrive as for k3g_rs_pull.  H = 7168; nranks 1, 2, 4 or 8; stats
 * and rowmax may be null.  With nranks > 1 every rank's partial buffer must be 32-byte aligned (peer rows are read
 * 32 bytes per access). */
int k3g_rs_land_add_attnres_rms(const void* partial, const void* partial_peer, int rank, int nranks, const void* prefix,
                                const void* blocks, const void* sw, const void* gamma, void* prefix2, void* normed, int nb,
                                int snapshot, int B, int H, float eps, const void* stats, int nb_stats, void* rowmax, void* stream);

/* kern_k3_moe_quant followed by kern_k3_allgather4_push in one launch (no counterpart in the reference): MXFP8 codes and
 * scale bytes of x [rows, cols] bf16 written straight to rows rank * rows .. of every rank's q_all [nranks * rows, cols] /
 * sf_all [nranks * rows, cols / 32] (q_peer / sf_peer = u64 peer tables); payloads s2 -> d2 and s3 -> d3 (n bytes each, the
 * router's indices and weights) gathered as by k3g_allgather4_push; the same barrier tail.  Identical gathered bytes.
 * nranks 1, 2, 4 or 8. */
int k3g_moe_quant_allgather_push(const void* x, int rows, int cols, void* q_all, const void* q_peer, void* sf_all, const void* sf_peer,
                                 const void* s2, void* d2, const void* p2, long long n2, const void* s3, void* d3, const void* p3,
                                 long long n3, void* flags, const void* flags_peer, int slot, int rank, int nranks, int units,
                                 long long timeout_us, void* status, void* stream);

/* The same folding for the routed-latent reduce-scatter and the latent norm of k3g_situ_rms (no counterpart in the
 * reference): partial = this rank's [nranks * L, h] bf16 partial sums, partial_peer = u64 table; ln [L, h] is the norm
 * of the ring-order chain of rows rank * L + r; act / item_max as k3g_situ_rms_amax (item_max may be null).  Outputs
 * bit-identical to k3g_rs_pull followed by k3g_situ_rms.  h <= 4096; nranks 1, 2, 4 or 8. */
int k3g_rs_situ_rms(const void* sp, void* act, const void* partial, const void* partial_peer, int rank, int nranks, const void* gam,
                    void* ln, int n, int B, int h, int L, void* item_max, void* stream);

/* kern_k3_land_add2, source/k3_residual_v2.cu:349 (op land_add2_v2; bf16 partials as in
 * source/k3_land_bf16.cu:96). */
int k3g_land_add2(const void* p1, const void* p2, int partial_is_bf16, const void* prefix2, void* hidden, int two,
                  int B, int H, void* stream);

/* ---- quantisation -------------------------------------------------------------------------- */

/* kern_k3_moe_quant, source/k3_moe_prefill_v4.cu:111 (op moe_quant): MXFP8 of x [rows, cols]. */
int k3g_moe_quant(const void* x, void* q, void* sf, int rows, int cols, int grid_hint, void* stream);

/* kern_quant_fp8_amax_v2 + kern_quant_fp8_apply_v2, source/k3_quant_fp8_pair_v2.cu:42,63
 * (op quant_fp8_tensor): per-tensor E4M3; partials holds `grid` floats. */
int k3g_quant_fp8_tensor(const void* x, void* y, void* scale_out, void* partials, int n, int grid, void* stream);

/* No counterpart in the reference.  k3g_quant_fp8_tensor for hosts that cannot allocate or pass a
 * workspace at call time (a runtime whose memory was all handed out at load, a server that bans
 * cudaMalloc after start-up because it synchronises the device): the block maxima live in a static
 * 8 KB device array inside the library, so grid is limited to 2048 (K3G_ELIMIT beyond), each GPU that
 * loads the library holds the array until exit, calls that overlap on one GPU race on it, and the
 * first call on a device does a one-time host-side address lookup (make it before any stream
 * capture) whose result is kept until the process exits: the device's primary context has to live
 * as long (no cudaDeviceReset between calls).  Results equal k3g_quant_fp8_tensor's for the same grid. */
int k3g_quant_fp8_tensor_noalloc(const void* x, void* y, void* scale_out, int n, int grid, void* stream);

/* ---- router and MoE routing ------------------------------------------------------------------ */

/* kern_k3_router_topk, source/k3_router_argmax.cu:87 (op router_topk).  experts must be 224; topk 8 or
 * 16.  idx/wts are [B, topk] in pick order.  The sigmoid is evaluated with IEEE-only operations. */
int k3g_router_topk(const void* S, const void* bias, const void* rs, void* idx, void* wts, int B, int experts,
                    int topk, void* stream);

/* kern_k3_moe_route_count, source/k3_moe_prefill_v4.cu:142 (op moe_route_count).  E local experts (up to 256: the
 * drop-in kernels cover 64, as the reference's 56; expert-parallel groups of 1 or 2 -- 224 / 112 local experts -- take
 * wider kernels behind the same three calls); placement strided (id % ep_ranks == rank, slot id / ep_ranks) or
 * blocked (source :100-109).  rank = -1 (all three routing calls; no counterpart in the reference) builds the tables
 * of every owner at once: E is then the TOTAL expert count, owner o's experts take slots o * E / ep_ranks ..., so
 * owner o's own tables are these shifted by the constant row blockoff[o * E / ep_ranks] (k3g_permute_dispatch). */
int k3g_moe_route_count(const void* ids, int T, int rank, int E, int topk, int ep_ranks, int strided, void* blockcount,
                        void* stream);

/* kern_k3_moe_route_tables, source/k3_moe_prefill_v4.cu:159 (op moe_route_tables). */
int k3g_moe_route_tables(const void* blockcount, int blocks, int E, int tile, void* blockoff, void* cta_batch,
                         void* cta_limit, void* num_non_exiting, void* total_padded, void* route_map, void* stream);

/* kern_k3_moe_route_scatter, source/k3_moe_prefill_v4.cu:205 (op moe_route_scatter).  With E > 64 the first
 * call on a device raises the wide kernel's dynamic shared-memory limit (a host-side attribute call): make
 * it before any stream capture. */
int k3g_moe_route_scatter(const void* ids, const void* blockoff, int T, int rank, int E, int topk, int ep_ranks,
                          int strided, void* route_map, void* exp2perm, void* stream);

/* k3g_moe_route_tables followed by k3g_moe_route_scatter in ONE launch (no counterpart in the reference, whose
 * tables kernel is a one-block launch of its own, source/k3_moe_prefill_v4.cu:159): each scatter block derives its own
 * row of blockoff from blockcount, block 0 also writes cta_batch / cta_limit / the two scalars / the padding rows.
 * Every output is bit-identical to the two calls.  T > 0. */
int k3g_moe_route_tables_scatter(const void* ids, const void* blockcount, int T, int rank, int E, int topk, int ep_ranks, int strided,
                                 int tile, void* blockoff, void* cta_batch, void* cta_limit, void* num_non_exiting, void* total_padded,
                                 void* route_map, void* exp2perm, void* stream);

/* kern_k3_moe_finalize, source/k3_moe_prefill_v4.cu:254 (op moe_finalize). */
int k3g_moe_finalize(const void* fc2, const void* exp2perm, const void* wts, void* out, int T, int cols, int topk,
                     void* stream);

/* Finalize fused with the one-partial residual add of kern_k3_land_add2 (source/k3_residual_v2.cu:349,
 * two = 0): out = bf16(residual + bf16(sum_k w * fc2[row_k])).  Benchmark configuration 2 combine. */
int k3g_finalize_residual(const void* fc2, const void* exp2perm, const void* wts, const void* residual, void* out, int T,
                          int cols, int topk, void* stream);

/* Dispatch gather (benchmark configuration 2): out row r = row route_map[r] of the MXFP8 token rows
 * (q [*, cols] codes, sf [*, cols/32] scales).  The reference leaves this gather to its grouped GEMM,
 * which reads route_map (source/k3_moe_prefill_v4.cu:36-46). */
int k3g_permute_gather(const void* q, const void* sf, const void* route_map, long long rows, int cols, void* out_q,
                       void* out_sf, void* stream);

/* Dispatch to the owning ranks over NVLink (benchmark configuration 2 at EP > 1; no counterpart in the reference,
 * which all-gathers every token to every rank -- source/k3_allgather4_v3.cu:61 -- and lets its grouped GEMM select).
 * q [B, cols] / sf [B, cols / 32]: the MXFP8 rows of this rank's tokens token_begin .. token_begin + B of the T gathered
 * tokens; ids / exp2perm [T, topk] and blockoff: the gathered expert ids and the all-owner routing tables
 * (k3g_moe_route_* with rank = -1, E = experts).  The row of token t is stored once per slot k into row
 * exp2perm[t, k] - blockoff[owner * experts / ep_ranks] of the owner's out_q / out_sf (out_*_peer: u64 tables of every
 * rank's buffer, own included), owner = ids % ep_ranks (strided) or ids / (experts / ep_ranks).  Destination rows are
 * exactly the live rows of the owner's own expert-sorted order (k3g_permute_gather on its route_map); the tile-padding
 * rows are not written.  The caller guarantees token_begin + B <= T (the tables' token count, which this call does not
 * take).  Plain peer stores, 32 bytes each when q and every rank's out_q are 32-byte aligned and cols % 32 == 0, else 16;
 * follow with k3g_rs_arrive before the owner reads. */
int k3g_permute_dispatch(const void* q, const void* sf, const void* ids, const void* exp2perm, const void* blockoff, int B,
                         long long token_begin, int topk, int cols, int experts, int ep_ranks, int strided, const void* out_q_peer,
                         const void* out_sf_peer, void* stream);

/* ---- collectives over NVLink peer pointers ---------------------------------------------------- */
/* Peer tables (`*_peer`) are device arrays of u64 addresses, one per rank, own rank included, as the
 * reference's runtime provides them (scripts/gen_collectives_p2p.py:77-86).  `flags` is this rank's
 * u64 counter table: flags[0] the epoch, flags[slot >= 1] one counter per collective call site.
 * `status` (device, 4 x u32, may be null) receives {1, slot, peer, observed} when a wait expires. */

/* kern_k3_flags_init, source/k3_collectives.cu:64 (op k3_flags_init). */
int k3g_flags_init(void* flags, int n, void* stream);

/* kern_k3_epoch_bump, source/k3_collectives.cu:74 (op k3_epoch_bump): flags[0] += units. */
int k3g_epoch_bump(void* flags, int units, void* stream);

/* kern_k3_rs_arrive1, source/k3_rs_arrive_v2.cu:41 (ops k3_allgather_push and the first launch of
 * k3_reducescatter_bf16): flags[slot] += units, then wait for every peer's flags[slot] >= flags[0]. */
int k3g_rs_arrive(void* flags, const void* flags_peer, int units, int slot, int nranks, long long timeout_us, void* status,
                  void* stream);

/* k3g_epoch_bump followed by k3g_rs_arrive in one launch (no counterpart in the reference, which always bumps the
 * epoch with its own kern_k3_epoch_bump launch, source/k3_collectives.cu:74): for a replay whose first waiting
 * call is a plain barrier.  Calls of the replay that publish arrivals without waiting (a push kernel's stores) may
 * come before it; nothing that WAITS may. */
int k3g_epoch_arrive(void* flags, const void* flags_peer, int units, int slot, int nranks, long long timeout_us, void* status,
                     void* stream);

/* kern_k3_rs_pull, source/k3_reducescatter_pull_nr4.cu:124 (second launch of k3_reducescatter_bf16).
 * order = 2 * ownpos + descend (source/k3_collectives.cu:222-236); 2 * (nranks - 1) is the ring order. */
int k3g_rs_pull(const void* src, void* dst, const void* src_peer, long long count, int order, int rank, int nranks, int grid,
                void* stream);

/* kern_k3_allgather4_push, source/k3_allgather4_v3.cu:61 (op k3_allgather4_push).  The launch publishes
 * `units` arrivals on its slot, so `units` must be the epoch increment.  The blocks of a push launch count
 * themselves on a per-device ticket word chosen by slot % 64 (the last one publishes the arrivals): at most
 * ONE push launch (this entry, k3g_moe_quant_allgather_push, the drop-in kern_k3_allgather4_push) per slot
 * modulo 64 may be in flight on a device at a time; launches on one stream, or the nodes of one graph chain,
 * satisfy that by construction. */
int k3g_allgather4_push(const void* s0, void* d0, const void* p0, long long n0, const void* s1, void* d1, const void* p1,
                        long long n1, const void* s2, void* d2, const void* p2, long long n2, const void* s3, void* d3,
                        const void* p3, long long n3, void* flags, const void* flags_peer, int slot, int rank, int nranks,
                        int units, long long timeout_us, void* status, void* stream);

/* Fused reduce-scatter -> residual add -> RMSNorm -> MXFP8 -> all-gather (benchmark configuration 1):
 * kern_k3_rs_pull + kern_k3_land_add_attnres_rms (nb = 0) + kern_k3_moe_quant + the all-gather push of
 * kern_k3_attnres_rms_push (source/k3_residual_push_add2.cu:356-360) in one kernel.  Bracket it with
 * k3g_rs_arrive before (partials ready) and after (pushes landed).  Processes rows
 * [row_begin, row_begin + rows) of a shard of shard_rows rows (shard_rows <= 0: shard = rows).  With nranks > 1
 * every rank's partial buffer must be 32-byte aligned (peer rows are read 32 bytes per access; scale bytes leave
 * as 16-byte stores, staged per row in shared memory). */
int k3g_rs_resnorm_mxfp8_ag(const void* partial, const void* partial_peer, const void* residual, const void* gamma,
                            void* residual_out, void* q_all, const void* q_all_peer, void* sf_all, const void* sf_all_peer,
                            int rows, int H, float eps, int rank, int nranks, int grid_hint, int row_begin, int shard_rows,
                            void* stream);

/* Status of the last expired wait of a launch that had no status pointer (host_status: 4 x u32).  Copies
 * the record to the host and SYNCHRONISES `stream`; not capturable. */
int k3g_wait_status(void* host_status, int clear, void* stream);

/* Set-up helpers standing in for the reference's external runtime (allocation + peer mapping with CUDA
 * IPC, one process per GPU).  These allocate / synchronise; handles are 64 bytes. */
int k3g_peer_alloc(long long bytes, void** host_out_dptr);
int k3g_peer_free(void* dptr);
int k3g_peer_export(void* dptr, void* host_handle64);
int k3g_peer_open(const void* host_handle64, void** host_out_dptr);
int k3g_peer_close(void* dptr);
/* Returns the SM count of the current device (> 0); host_cc receives major * 10 + minor. */
int k3g_device_sms(int* host_cc);

/* ---- MLA prep ----------------------------------------------------------------------------------- */

/* kern_k3_mla_prep_head + kern_k3_mla_prep_gate, source/k3_mla_prep_v2.cu:130,91 (op mla_prep; bf16
 * partial as in source/k3_mla_prep_bf16.cu).  mla_gate may be null (head only). */
int k3g_mla_prep(const void* partial, int partial_is_bf16, const void* gamma_q, const void* gamma_kv, const void* slot_mapping,
                 void* slab, long long layer_off, long long page_stride, void* q_norm, void* mla_gate, int B, int inner,
                 float eps, void* stream);

/* Benchmark configuration 3: latent RMSNorm + RoPE on the rope slices of q and k + k_rope broadcast into
 * the packed k buffer.  rope_tab [T, 64] bf16 = cos(32) | sin(32) (table convention of
 * source/weight_prep.cu:34-45); half-split pairing.  No counterpart kernel in the reference. */
int k3g_mla_prep_rope_pack(const void* kv, const void* q, const void* gamma_kv, const void* rope_tab, void* q_out, void* k_out,
                           void* latent_out, int T, int heads, float eps, void* stream);

/* ---- KDA -------------------------------------------------------------------------------------------- */

/* kern_k3_span_gather, source/k3_span_gather_v3.cu:251 (op span_gather_v2), with the window passed
 * directly instead of through the KDA state line. */
int k3g_span_gather(const void* partial, long long row_stride, const void* cw, int taps_bf16, void* win, const void* wsm_partial,
                    void* span_q, void* span_k, void* span_v, void* span_beta, void* span_flow, int heads, int at, int span,
                    int rows_per_block, void* stream);

/* kern_k3_kda_out_gate, source/k3_kda_out_gate_v3.cu:36 (op kda_out_gate_v2), optionally with the
 * MXFP8 epilogue of benchmark configuration 4. */
int k3g_kda_out_gate(const void* attn, const void* gate, long long gate_stride, long long gate_off, const void* gamma_o,
                     void* gated, void* q, void* sf, int heads, int at, int span, float eps, void* stream);

/* kern_k3_moe_w_shuffle / kern_k3_moe_sf_shuffle, source/k3_moe_prefill_v4.cu:304-327 (load time): expert weight
 * rows [experts, n, row_bytes] and their scale bytes [experts, n, kg] rearranged into the layouts the grouped GEMM
 * reads -- rows permuted inside groups of 32 (and gate/up rows interleaved when gated), scales additionally packed
 * into 128 x 4 tiles of 512 bytes.  n % 32 == 0 (weights), n % 128 == 0 and kg % 4 == 0 (scales). */
int k3g_moe_w_shuffle(const void* src, void* dst, int experts, int n, int row_bytes, int gated, void* stream);
int k3g_moe_sf_shuffle(const void* src, void* dst, int experts, int n, int kg, int gated, void* stream);

/* kern_k3_argmax_f32_partial + kern_k3_argmax_f32_final, source/k3_router_argmax.cu:186,225 (op argmax_f32_one):
 * out [B] i64 = index of the largest of n f32 logits per row, ties to the smallest index; pmax / pidx [B, parts]
 * are the caller's scratch for the two stages. */
int k3g_argmax_f32(const void* logits, void* pmax, void* pidx, void* out, int B, int n, int parts, void* stream);

/* ---- load-time derived tables (source/k3_weight_prep.cu, source/weight_prep.cu; run once after load) ----------- */

/* kern_fill_bf16 (k3_weight_prep.cu:32), kern_fill_f32 / _i32 / _i64 / _u8 (weight_prep.cu:47-65): p[i] = value, i < n.
 * kind 0 bf16 (v), 1 f32 (v), 2 i32 (iv), 3 i64 (iv), 4 u8 (iv). */
int k3g_fill(void* p, long long n, int kind, float v, long long iv, void* stream);
/* kern_iota_i32, weight_prep.cu:67: p[i * stride] = start + i * step. */
int k3g_iota_i32(void* p, int n, int start, int step, int stride, void* stream);
/* kern_cast_bf16_f32 / kern_weight_p1_bf16_f32, weight_prep.cu:24-32: out[i] = f32(w[i]) (+ 1 when plus_one). */
int k3g_cast_bf16_f32(const void* w, void* out, int n, int plus_one, void* stream);
/* kern_rope_table_bf16, weight_prep.cu:34: cos / sin [rows][stride], columns j < half: angle = r / base^(j / half). */
int k3g_rope_table(void* cos_t, void* sin_t, int rows, int half, int stride, float base, void* stream);
/* kern_k3_conv_taps, k3_weight_prep.cu:37: cw [3][4][inner] f32 from the q, k, v conv weights [inner][4] f32. */
int k3g_conv_taps(const void* q, const void* k, const void* v, void* cw, int inner, void* stream);
/* kern_k3_scoring, k3_weight_prep.cu:48: sw[j] = f32(norm[j]) * f32(proj[j]). */
int k3g_scoring(const void* norm, const void* proj, void* sw, int n, void* stream);
/* kern_k3_wsm, k3_weight_prep.cu:54: [256, h] block, rows 0..heads = b, rows 96..224 = f_a, others zero. */
int k3g_wsm(const void* b, const void* f_a, void* wsm, int heads, int h, void* stream);
/* kern_k3_mega_sf_pack, k3_weight_prep.cu:71: scale bytes [experts][n][kg] -> i32 [experts][kg / 4][n], rows permuted. */
int k3g_mega_sf_pack(const void* raw, void* out, int experts, int n, int kg, int interleave, void* stream);
/* kern_k3_kvb_aug, k3_weight_prep.cu:81: [heads * 320, 576] expansion weight from kv_b_proj [heads * 256, 512]. */
int k3g_kvb_aug(const void* w_kv_b, void* out, int heads, void* stream);

/* ---- once-per-prefill helpers (byte movement) ---------------------------------------------------------- */

/* kern_k3_rank_rows, source/k3_prefill.cu:28 (op rank_rows): dst[j] = src[min(rank * own + j, rows - 1)], j < own. */
int k3g_rank_rows(void* dst, const void* src, int rank, int own, int row_bytes, int rows, void* stream);
/* kern_k3_zero_rows, source/k3_prefill.cu:42 (op zero_rows): rows [from, to) of buf zeroed. */
int k3g_zero_rows(void* buf, int row_bytes, int from, int to, void* stream);
/* kern_k3_fmha_lens, source/k3_prefill.cu:49 (op fmha_lens): lens[8] = {kv, 0, 0, T, 0, kv, 0, 0}, kv = seq_lens[0]. */
int k3g_fmha_lens(const void* seq_lens, void* lens, int T, void* stream);
/* kern_embedding_i64_bf16, source/embedding.cu:6 (op embedding): out[r] = table[ids[r]], rows of `hidden` bf16. */
int k3g_embedding(const void* ids, const void* table, void* out, int tokens, int hidden, void* stream);
/* kern_copy_rows_bf16, source/copy_rows.cu:23: dst[r, :width] = src[r, :width], strides in elements. */
int k3g_copy_rows(void* dst, const void* src, int dst_stride, int src_stride, int width, int rows, void* stream);
/* kern_last_row_bf16, source/copy_rows.cu:32 (op last_row): dst[0, :width] = src[rows - 1, :width]. */
int k3g_last_row(void* dst, const void* src, int src_stride, int width, int rows, void* stream);
/* kern_own_rows, source/copy_rows.cu:39: dst[j] = src[min(blocks[rank] + j, rows - 1)], j < own. */
int k3g_own_rows(void* dst, const void* src, const void* blocks, int rank, int own, int row_bytes, int rows, void* stream);

/* ---- remaining per-layer glue --------------------------------------------------------------------- */

/* kern_k3_situ_rms_bf16, source/k3_land_fused.cu:123 (op land_situ_rms): shared-expert SiTU landing
 * act [B, n] = bf16((4 tanh(g/4) sigmoid(g)) * 25 tanh(u/25)) from sp [B, 2n] = g | u, and the MoE latent
 * RMSNorm ln [L, h] = bf16(lat * rs) (x) gam, in one launch.  n % 8 == 0, h % 8 == 0, h <= 8192. */
int k3g_situ_rms(const void* sp, void* act, const void* lat, const void* gam, void* ln, int n, int B, int h, int L, void* stream);

/* kern_k3_land_situ, source/k3_land.cu:211 (op land_situ_n33792): act [B, n] = bf16(SiTU(bf16(g), bf16(u))) from
 * the f32 partial p [B, 2n] = g | u (both operands land to bf16 before the activation). */
int k3g_land_situ(const void* p, void* act, int n, int B, void* stream);

/* kern_k3_land, source/k3_land.cu:166: o [B, n] = bf16(p[b * ldc + off + i]). */
int k3g_land(const void* p, void* o, int n, int off, int ldc, int B, void* stream);

/* kern_k3_rms, source/k3_land.cu:107: o [B, h] = bf16(x * rs) (x) gamma, rs = rsqrt(mean(x^2) + 1e-5); the sum in
 * the order of the reference's 1024-thread block.  h % 8 == 0, h <= 8192. */
int k3g_rms(const void* x, const void* gamma, void* o, int h, int B, void* stream);

/* kern_sigmoid_mul_bf16, source/sigmoid_mul.cu:15 (op mla_gate): out = bf16(attn * bf16(sigmoid(gate))),
 * gate(t, h, d) = gate + t * gate_tstride + h * gate_hstride + d. */
int k3g_sigmoid_mul(void* out, const void* attn, const void* gate, int tokens, int heads, int head_dim, int gate_tstride,
                    int gate_hstride, void* stream);

/* kern_k3_span_state, source/k3_span_state.cu:19 (ops span_state_load / span_state_store): copy of the
 * sequence's [heads][128][128] f32 KDA state between its state line and a flat buffer.  The reference fixes
 * heads = 24 when it builds the module; here it is an argument (the drop-in cubin keeps the reference's list). */
int k3g_span_state(void* kda_base, const void* line_index, long long line_bytes, const void* span_at, void* buf, int to_line,
                   int heads, void* stream);

/* kern_k3_latent_gather, source/k3_mla_v2.cu:22 (op latent_gather): cached latent rows [n, 576] laid
 * contiguous from 64-row pages; rows >= lens[0] are zero. */
int k3g_latent_gather(const void* slab, const void* block_table, long long page_stride, const void* lens, void* out, int n,
                      void* stream);

#ifdef __cplusplus
}
#endif
#endif /* K3G_H */
