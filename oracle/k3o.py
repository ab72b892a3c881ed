"""TEST INFRASTRUCTURE — numpy front end of the CPU oracle (oracle/k3o_ops.cpp).

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline / reference arm import
this module.  bf16 tensors travel as numpy uint16 arrays holding the bit patterns.
"""
import ctypes
import os
import sys

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, _HERE)
import build_oracle  # noqa: E402

_lib = None


def lib():
    global _lib
    if _lib is None:
        path = build_oracle.build()
        try:
            _lib = ctypes.CDLL(path)
        except OSError:
            _lib = ctypes.CDLL(build_oracle.build(force=True))
        for name, res in (("k3o_bf16_to_f32", ctypes.c_float), ("k3o_e4m3_decode", ctypes.c_float),
                          ("k3o_rsqrt_rn", ctypes.c_float), ("k3o_det_exp", ctypes.c_float),
                          ("k3o_det_sigmoid", ctypes.c_float), ("k3o_f32_to_bf16", ctypes.c_uint16),
                          ("k3o_e4m3_encode", ctypes.c_uint8)):
            getattr(_lib, name).restype = res
        for name in ("k3o_f32_to_bf16", "k3o_e4m3_encode", "k3o_ue8m0_exp", "k3o_ue8m0_exp_float_formula",
                     "k3o_rsqrt_rn", "k3o_det_exp", "k3o_det_sigmoid"):
            getattr(_lib, name).argtypes = [ctypes.c_float]
        _lib.k3o_bf16_to_f32.argtypes = [ctypes.c_uint16]
        _lib.k3o_e4m3_decode.argtypes = [ctypes.c_uint8]
    return _lib


def _p(a):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"], "oracle arrays must be contiguous"
    return ctypes.c_void_p(a.ctypes.data)


I = ctypes.c_int
LL = ctypes.c_longlong
F = ctypes.c_float


# ---- dtype helpers ---------------------------------------------------------------------------
def f32_to_bf16(x):
    """float32 array -> uint16 bf16 bit patterns, round to nearest even."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    r[nan] = 0x7FFF
    return r


def bf16_to_f32(h):
    return (np.ascontiguousarray(h, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def e4m3_to_f32(c):
    c = np.ascontiguousarray(c, dtype=np.uint8).astype(np.int32)
    s, ex, m = c >> 7, (c >> 3) & 0xF, c & 7
    v = np.where(ex == 0, m * 2.0 ** -9, (1.0 + m / 8.0) * 2.0 ** (ex - 7.0))
    v = np.where((ex == 15) & (m == 7), np.nan, v)
    return np.where(s == 1, -v, v).astype(np.float32)


# ---- ops ---------------------------------------------------------------------------------------
def resnorm_mxfp8(residual, delta, gamma, eps, want_normed=True):
    B, H = residual.shape
    out = np.empty((B, H), np.uint16)
    q = np.empty((B, H), np.uint8)
    sf = np.empty((B, H // 32), np.uint8)
    normed = np.empty((B, H), np.uint16) if want_normed else None
    lib().k3o_resnorm_mxfp8(_p(residual), _p(delta), _p(gamma), _p(out), _p(q), _p(sf), _p(normed), I(B), I(H), F(eps))
    return out, q, sf, normed


def attnres_rms(prefix, blocks, sw, gamma, nb, snapshot, eps):
    B, H = prefix.shape
    normed = np.empty((B, H), np.uint16)
    lib().k3o_attnres_rms(_p(prefix), _p(blocks), _p(sw), _p(gamma), _p(normed), I(nb), I(snapshot), I(B), I(H), F(eps))
    return normed


def land_add_attnres_rms(partial, prefix, blocks, sw, gamma, nb, snapshot, eps):
    B, H = partial.shape
    is_bf16 = int(partial.dtype == np.uint16)
    prefix2 = np.empty((B, H), np.uint16)
    normed = np.empty((B, H), np.uint16)
    lib().k3o_land_add_attnres_rms(_p(partial), I(is_bf16), _p(prefix), _p(blocks), _p(sw), _p(gamma), _p(prefix2),
                                   _p(normed), I(nb), I(snapshot), I(B), I(H), F(eps))
    return prefix2, normed


def land_add_attnres_rms_stats(partial, prefix, blocks, sw, gamma, nb, snapshot, eps, stats, nb_stats):
    B, H = partial.shape
    is_bf16 = int(partial.dtype == np.uint16)
    prefix2 = np.empty((B, H), np.uint16)
    normed = np.empty((B, H), np.uint16)
    lib().k3o_land_add_attnres_rms_stats(_p(partial), I(is_bf16), _p(prefix), _p(blocks), _p(sw), _p(gamma), _p(prefix2),
                                         _p(normed), I(nb), I(snapshot), I(B), I(H), F(eps), _p(stats), I(nb_stats))
    return prefix2, normed


def attnres_rms_push(blocks, sw, gamma, nb, snapshot, sw_mlp, p1, p2, prefix2, two, eps, want_stats=True):
    """Returns (hidden, normed, stats); blocks is updated in place when snapshot is set."""
    B, H = prefix2.shape
    hidden = np.empty((B, H), np.uint16)
    normed = np.empty((B, H), np.uint16)
    stats = np.zeros((B, 8, 2), np.float32) if want_stats else None
    lib().k3o_attnres_rms_push(_p(blocks), _p(sw), _p(gamma), _p(normed), I(nb), I(snapshot), I(B), _p(sw_mlp), _p(stats),
                               _p(p1), _p(p2), _p(prefix2), _p(hidden), I(two), I(H), F(eps))
    return hidden, normed, stats


def land_add2(p1, p2, prefix2, two):
    B, H = prefix2.shape
    is_bf16 = int(p1.dtype == np.uint16)
    hidden = np.empty((B, H), np.uint16)
    lib().k3o_land_add2(_p(p1), _p(p2), I(is_bf16), _p(prefix2), _p(hidden), I(two), I(B), I(H))
    return hidden


def quant_fp8_tensor(x):
    y = np.empty(x.shape, np.uint8)
    scale = np.empty(1, np.float32)
    lib().k3o_quant_fp8_tensor(_p(x), _p(y), _p(scale), LL(x.size))
    return y, scale


def moe_quant(x):
    rows, cols = x.shape
    q = np.empty((rows, cols), np.uint8)
    sf = np.empty((rows, cols // 32), np.uint8)
    lib().k3o_moe_quant(_p(x), _p(q), _p(sf), LL(rows), I(cols))
    return q, sf


def router_topk(S, bias, rs, topk):
    B, E = S.shape
    idx = np.empty((B, topk), np.int32)
    wts = np.empty((B, topk), np.float32)
    lib().k3o_router_topk(_p(S), _p(bias), _p(rs), _p(idx), _p(wts), I(B), I(E), I(topk))
    return idx, wts


def moe_route(ids, rank, E, ep_ranks, strided, tile):
    """route_count + route_tables + route_scatter; returns a dict of all tables."""
    T, topk = ids.shape
    blocks = (T + 255) // 256
    blockcount = np.zeros((blocks, E), np.int32)
    lib().k3o_moe_route_count(_p(ids), I(T), I(rank), I(E), I(topk), I(ep_ranks), I(strided), _p(blockcount))
    max_ctas = (T * topk + tile - 1) // tile + E
    blockoff = np.zeros((blocks, E), np.int32)
    cta_batch = np.full(max_ctas, -1, np.int32)
    cta_limit = np.full(max_ctas, -1, np.int32)
    nne = np.zeros(1, np.int32)
    total = np.zeros(1, np.int32)
    route_map = np.full(max_ctas * tile, -1, np.int32)
    lib().k3o_moe_route_tables(_p(blockcount), I(blocks), I(E), I(tile), _p(blockoff), _p(cta_batch), _p(cta_limit),
                               _p(nne), _p(total), _p(route_map))
    exp2perm = np.empty((T, topk), np.int32)
    lib().k3o_moe_route_scatter(_p(ids), _p(blockoff), I(T), I(rank), I(E), I(topk), I(ep_ranks), I(strided),
                                _p(route_map), _p(exp2perm))
    return dict(blockcount=blockcount, blockoff=blockoff, cta_batch=cta_batch, cta_limit=cta_limit,
                num_non_exiting=nne, total_padded=total, route_map=route_map, exp2perm=exp2perm)


def moe_finalize(fc2, exp2perm, wts, T, cols):
    topk = exp2perm.shape[1]
    out = np.empty((T, cols), np.uint16)
    lib().k3o_moe_finalize(_p(fc2), _p(exp2perm), _p(wts), _p(out), I(T), I(cols), I(topk))
    return out


def finalize_residual(fc2, exp2perm, wts, residual):
    T, cols = residual.shape
    topk = exp2perm.shape[1]
    out = np.empty((T, cols), np.uint16)
    lib().k3o_finalize_residual(_p(fc2), _p(exp2perm), _p(wts), _p(residual), _p(out), I(T), I(cols), I(topk))
    return out


def permute_gather(q, sf, route_map, rows):
    cols = q.shape[1]
    out_q = np.empty((rows, cols), np.uint8)
    out_sf = np.empty((rows, cols // 32), np.uint8)
    lib().k3o_permute_gather(_p(q), _p(sf), _p(route_map), LL(rows), I(cols), _p(out_q), _p(out_sf))
    return out_q, out_sf


def rs_sequence(rank, W, order):
    seq = np.empty(W, np.int32)
    lib().k3o_rs_sequence(I(rank), I(W), I(order), _p(seq))
    return seq


def rs_pull(partials, rank, order):
    """partials: list of W uint16 arrays [W * count]; returns this rank's reduced chunk."""
    W = len(partials)
    count = partials[0].size // W
    arr = (ctypes.c_void_p * W)(*[p.ctypes.data for p in partials])
    dst = np.empty(count, np.uint16)
    lib().k3o_rs_pull(arr, _p(dst), LL(count), I(rank), I(W), I(order))
    return dst


def sim_barrier(W, slots, replays, units, absent_rank=-1, timeout_us=200000):
    status = np.zeros(W, np.int32)
    bad = lib().k3o_sim_barrier(I(W), I(slots), I(replays), I(units), I(absent_rank), I(timeout_us), _p(status))
    return bad, status


def mla_prep_head(partial, gamma_q, gamma_kv, slot_mapping, slab, layer_off, page_stride, eps):
    B, fused = partial.shape
    is_bf16 = int(partial.dtype == np.uint16)
    q_norm = np.empty((B, 1536), np.uint16)
    lib().k3o_mla_prep_head(_p(partial), I(is_bf16), I(fused), _p(gamma_q), _p(gamma_kv), _p(slot_mapping), _p(slab),
                            LL(layer_off), LL(page_stride), _p(q_norm), I(B), F(eps))
    return q_norm


def mla_prep_gate(partial, inner):
    B, fused = partial.shape
    is_bf16 = int(partial.dtype == np.uint16)
    g = np.empty((B, inner), np.uint16)
    lib().k3o_mla_prep_gate(_p(partial), I(is_bf16), I(fused), I(inner), _p(g), I(B))
    return g


def mla_prep_rope_pack(kv, q, gamma_kv, rope_tab, eps, k_out_init=None):
    T, heads = q.shape[0], q.shape[1]
    q_out = np.empty_like(q)
    k_out = np.zeros_like(q) if k_out_init is None else k_out_init.copy()
    latent = np.empty((T, 512), np.uint16)
    lib().k3o_mla_prep_rope_pack(_p(kv), _p(q), _p(gamma_kv), _p(rope_tab), _p(q_out), _p(k_out), _p(latent), I(T),
                                 I(heads), F(eps))
    return q_out, k_out, latent


def span_conv_silu(partial, row_stride, cw, win, inner, at, span):
    taps_bf16 = int(cw.dtype == np.uint16)
    outs = [np.empty((span, inner), np.uint16) for _ in range(3)]
    win = win.copy()
    lib().k3o_span_conv_silu(_p(partial), LL(row_stride), _p(cw), I(taps_bf16), _p(win), _p(outs[0]), _p(outs[1]),
                             _p(outs[2]), I(inner), I(at), I(span))
    return outs[0], outs[1], outs[2], win


def span_beta_flow(wsm_partial, heads, at, span):
    beta = np.empty((heads, span), np.uint16)
    flow = np.empty((span, 128), np.uint16)
    lib().k3o_span_beta_flow(_p(wsm_partial), I(heads), _p(beta), _p(flow), I(at), I(span))
    return beta, flow


def kda_out_gate(attn, gate, gate_stride, gate_off, gamma_o, heads, at, span, rows, eps, quant=False):
    inner = heads * 128
    gated = np.zeros((rows, inner), np.uint16)
    q = np.zeros((rows, inner), np.uint8) if quant else None
    sf = np.zeros((rows, inner // 32), np.uint8) if quant else None
    lib().k3o_kda_out_gate(_p(attn), _p(gate), LL(gate_stride), LL(gate_off), _p(gamma_o), _p(gated), _p(q), _p(sf),
                           I(heads), I(at), I(span), F(eps))
    return gated, q, sf


def situ_rms(sp, lat, gam, n, h):
    B, L = sp.shape[0], lat.shape[0]
    act = np.empty((B, n), np.uint16)
    ln = np.empty((L, h), np.uint16)
    lib().k3o_situ_rms(_p(sp), _p(act), _p(lat), _p(gam), _p(ln), I(n), I(B), I(h), I(L))
    return act, ln


def sigmoid_mul(attn, gate, heads, head_dim, gate_tstride, gate_hstride):
    tokens = attn.shape[0]
    out = np.empty((tokens, heads * head_dim), np.uint16)
    lib().k3o_sigmoid_mul(_p(out), _p(attn), _p(gate), I(tokens), I(heads), I(head_dim), I(gate_tstride), I(gate_hstride))
    return out


# ---- once-per-prefill helpers and f32 landings (byte movement / thin wrappers) ------------------------------
def land_situ(p, n):
    """kern_k3_land_situ (source/k3_land.cu:199-237): both operands land to bf16, then SiTU; p is f32 [B, 2n]."""
    sp = f32_to_bf16(np.ascontiguousarray(p, np.float32))
    h = 8
    return situ_rms(sp, np.zeros((0, h), np.uint16), np.zeros(h, np.uint16), n, h)[0]


def land(p, n, off, ldc):
    """kern_k3_land (source/k3_land.cu:166-188): o[b, i] = bf16(p[b * ldc + off + i])."""
    p = np.ascontiguousarray(p, np.float32).reshape(-1, ldc)
    return f32_to_bf16(np.ascontiguousarray(p[:, off:off + n]))


def rms(x, gamma):
    """kern_k3_rms at block 1024 (source/k3_land.cu:107-160) for h <= 8192: the latent norm of situ_rms."""
    h = x.shape[1]
    return situ_rms(np.zeros((0, 16), np.uint16), x, gamma, 8, h)[1]


def rank_rows(src, rank, own):
    """kern_k3_rank_rows (source/k3_prefill.cu:28-40)."""
    rows = src.shape[0]
    return src[np.minimum(rank * own + np.arange(own), rows - 1)].copy()


def zero_rows(buf, lo, hi):
    """kern_k3_zero_rows (source/k3_prefill.cu:42-47)."""
    out = buf.copy()
    if hi > lo:
        out[lo:hi] = 0
    return out


def fmha_lens(seq_lens, T):
    """kern_k3_fmha_lens (source/k3_prefill.cu:49-60)."""
    kv = int(seq_lens[0])
    return np.array([kv, 0, 0, T, 0, kv, 0, 0], np.int32)


def embedding(ids, table):
    """kern_embedding_i64_bf16 (source/embedding.cu:6-16)."""
    return table[ids].copy()


def own_rows(src, blocks, rank, own):
    """kern_own_rows (source/copy_rows.cu:39-47)."""
    rows = src.shape[0]
    return src[np.minimum(int(blocks[rank]) + np.arange(own), rows - 1)].copy()


def argmax_f32(logits):
    """kern_k3_argmax_f32_partial/_final (source/k3_router_argmax.cu:186-241): the largest value under the monotone
    u32 order of the float's bits (so +NaN patterns order above +inf), ties to the smallest index."""
    b = np.ascontiguousarray(logits, np.float32).view(np.uint32)
    key = np.where(b & np.uint32(0x80000000), ~b, b | np.uint32(0x80000000))
    return np.argmax(key, axis=1).astype(np.int64)


def _shuffled_src_row(r, n, gated):
    u = (r // 32) * 32 + (r % 8) * 4 + (r % 32) // 8
    return np.where(u % 2 == 1, n // 2, 0) + u // 2 if gated else u


def moe_w_shuffle(src, gated):
    """kern_k3_moe_w_shuffle (source/k3_moe_prefill_v4.cu:304-317): src [experts, n, row_bytes] u8."""
    n = src.shape[1]
    return src[:, _shuffled_src_row(np.arange(n), n, gated)].copy()


def moe_sf_shuffle(src, gated):
    """kern_k3_moe_sf_shuffle (source/k3_moe_prefill_v4.cu:319-327): src [experts, n, kg] u8 -> same size, tiled."""
    experts, n, kg = src.shape
    r, c = np.meshgrid(np.arange(n), np.arange(kg), indexing="ij")
    at = ((r // 128) * (kg // 4) + c // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + c % 4
    out = np.zeros((experts, n * kg), np.uint8)
    out[:, at.reshape(-1)] = src[:, _shuffled_src_row(np.arange(n), n, gated)].reshape(experts, -1)
    return out.reshape(experts, n, kg)


# ---- load-time derived tables (source/k3_weight_prep.cu, source/weight_prep.cu) ------------------------------
def rope_table(rows, half, base):
    """kern_rope_table_bf16 (source/weight_prep.cu:34-45): f32 arithmetic as written, landed to bf16 (cos, sin)."""
    j = np.arange(half, dtype=np.float32)
    inv = (np.float32(1.0) / np.power(np.float32(base), (np.float32(2.0) * j) / np.float32(2 * half), dtype=np.float32)).astype(np.float32)
    ang = (np.arange(rows, dtype=np.float32)[:, None] * inv[None, :]).astype(np.float32)
    return f32_to_bf16(np.cos(ang.astype(np.float64)).astype(np.float32)), f32_to_bf16(np.sin(ang.astype(np.float64)).astype(np.float32))


def conv_taps(q, k, v):
    """kern_k3_conv_taps (source/k3_weight_prep.cu:37-46): [inner, 4] x 3 -> [3, 4, inner]."""
    return np.ascontiguousarray(np.stack([q, k, v]).transpose(0, 2, 1))


def scoring(norm, proj):
    """kern_k3_scoring (source/k3_weight_prep.cu:48-52)."""
    return (bf16_to_f32(norm) * bf16_to_f32(proj)).astype(np.float32)


def wsm(b, f_a, heads):
    """kern_k3_wsm (source/k3_weight_prep.cu:54-60)."""
    h = b.shape[1]
    out = np.zeros((256, h), np.uint16)
    out[:heads] = b[:heads]
    out[96:224] = f_a[:128]
    return out


def mega_sf_pack(raw, interleave):
    """kern_k3_mega_sf_pack (source/k3_weight_prep.cu:62-79): raw [experts, n, kg] u8 -> i32 [experts, kg / 4, n]."""
    experts, n, kg = raw.shape
    r = np.arange(n)
    u = (r // 128) * 128 + (r % 4) * 32 + (r % 128) // 4
    src = np.where((u >> 3) & 1 == 1, n // 2, 0) + (u >> 4) * 8 + (u & 7) if interleave else u
    words = np.ascontiguousarray(raw[:, src, :]).view("<u4")            # [experts, n, kg / 4], LSB-first bytes
    return np.ascontiguousarray(words.transpose(0, 2, 1)).view(np.int32)


def kvb_aug(w_kv_b, heads):
    """kern_k3_kvb_aug (source/k3_weight_prep.cu:81-93): [heads * 256, 512] bf16 -> [heads * 320, 576] bf16."""
    w = w_kv_b.reshape(heads, 256, 512)
    out = np.zeros((heads, 320, 576), np.uint16)
    out[:, :128, :512] = w[:, :128]
    out[:, 192:, :512] = w[:, 128:]
    one = f32_to_bf16(np.ones(1, np.float32))[0]
    for d in range(64):
        out[:, 128 + d, 512 + d] = one
    return out.reshape(heads * 320, 576)


def num_threads():
    return int(lib().k3o_num_threads())
