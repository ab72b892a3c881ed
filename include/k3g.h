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
 *     `host_`; nothing here allocates, frees or synchronises; launchers are graph-capturable;
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

#ifdef __cplusplus
}
#endif
#endif /* K3G_H */
