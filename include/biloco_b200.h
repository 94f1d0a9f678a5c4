/* biloco_b200 — C ABI of the B200 (sm_100a) implementation of the fused BiLoCo decode linear
 *
 *     y[M,N] = alpha * FP4(x)[M,K] . FP4(R)[N,K]^T  +  sum_i S_i (x . v_i) u_i          (M <= 32)
 *
 * Plain pointers and sizes only; every pointer is DEVICE memory unless stated otherwise. All functions
 * enqueue work on `stream` and return without synchronising. Return value: 0 on success, a negative
 * BILOCO_ERR_* code otherwise (nothing is enqueued in that case). Nothing here throws or allocates
 * device memory: scratch is caller-owned (see biloco_b200_scratch_bytes).
 *
 * Each entry point names the interface of the reference (jindavid/BiLoCo) that it stands in for.
 */
#ifndef BILOCO_B200_H_
#define BILOCO_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* biloco_stream_t; /* same type as cudaStream_t */

#define BILOCO_OK 0
#define BILOCO_ERR_NULL -1           /* a required pointer is null */
#define BILOCO_ERR_SHAPE -2          /* shape not supported (see each function) */
#define BILOCO_ERR_ALIGN -3          /* a pointer is not aligned as required */
#define BILOCO_ERR_SCRATCH -4        /* scratch too small */
#define BILOCO_ERR_CUDA -5           /* a CUDA runtime / driver call failed */
#define BILOCO_ERR_MODE -6           /* unknown schedule (mode) or quantisation rule */
#define BILOCO_ERR_EPOCH -7          /* epoch must be >= 1 */
#define BILOCO_ERR_LIMIT -8          /* size beyond a stated maximum */
#define BILOCO_ERR_WAIT -9           /* a bounded wait on the device ran out (host-synchronous routines only) */

/* NVFP4 block-scale selection rules of the activation quantiser (biloco/fp4.py:12-18). */
#define BILOCO_RULE_STATIC_6 0
#define BILOCO_RULE_STATIC_4 1
#define BILOCO_RULE_MSE 2            /* "four over six": per block, 6 or 4, smaller squared error */
#define BILOCO_RULE_GIVEN_SCALE 0x100 /* OR-ed to a rule: a_gscale[0] already holds the tensor scale (not recomputed) */

/* Schedules of the fused kernel; numbered like the reference's modes (biloco/kernel.py:18-26,66-76).
 *   2: every CTA that contributes to a tile expands z for a share of the ranks and adds it to its partial sum
 *      (spreads the expansion over all SMs: for larger batches)
 *   4: the CTA that finishes a tile expands z for all ranks; the other contributors publish their partial sums
 *      without waiting for z (shortest dependency chain: for the smallest batches)
 *   5: a tile belongs to a thread-block cluster of c CTAs (c = SMs / tiles, at most 8) that split its k-tiles; the
 *      partial sums go to the finishing CTA through distributed shared memory instead of global memory (M <= 8 and
 *      a tile count that lets tiles * c fill at least two thirds of the SMs; other shapes are refused)
 * In all of them z is computed by all CTAs at entry (rank-sliced) and handed over without a counter: every published z
 * value carries a validity mark in its lowest mantissa bit that flips with each launch completed on the scratch, and the
 * consumers poll the values themselves. */
#define BILOCO_MODE_COUNTER 2
#define BILOCO_MODE_OWNER 4
#define BILOCO_MODE_CLUSTER 5
/*   7: row slabs, for one to four activation rows: N is split only (CTA c owns the ceil8(N / SMs) weight rows c, all of K),
 *      so no partial sum leaves a CTA; the tensor-core tile's 128 rows hold the same weight rows for up to four
 *      consecutive k-tiles, matched by one activation-operand row per k-tile, and the diagonal blocks of the
 *      accumulator are summed in the epilogue. Needs the copy made by biloco_b200_tile_weights_slab as W_tiled,
 *      M <= 4 (three rows run as four; with three or four rows K <= 8192 and at most 16 ranks per z slice, i.e.
 *      R <= 16 * floor(SMs / M)), K % 512 == 0, N <= 128 * SMs, one column group. No counterpart in the reference. */
#define BILOCO_MODE_SLAB 7

/* OR-ed to the mode: Y is fp32 [M,N] instead of bf16 (the unrounded sum). For partial outputs that are reduced across
 * devices before the single bf16 rounding (row-parallel shards). No counterpart in the reference (single GPU). */
#define BILOCO_OUT_FP32 0x400

/* 1 if biloco_b200_fused_linear accepts this problem in this mode on a device with num_sms multiprocessors
 * (0 = the current device), else 0. Host-only. Counterpart: modes_for (biloco/kernel.py:66-76). */
int biloco_b200_mode_supported(int M, int N, int K, int R, int mode, int num_sms);

/* Human-readable text for an error code (host pointer, static storage). */
const char* biloco_b200_error_string(int code);

/* ABI version of this library (bumped when a signature changes). */
int biloco_b200_abi_version(void);

/* Bytes of the block-scale tensor of a [rows, k] NVFP4 operand in the 128x4 atom layout.
 * Replaces: biloco/kernel.py:132-134 (nvfp4_sf_bytes). Host-only arithmetic. */
size_t biloco_b200_sf_bytes(int rows, int k);

/* z[m,i] = S[i] * sum_k sign(V[i,k]) X[m,k], fp32 [M,R].   X bf16 [M,K], V_packed u8 [R,K/8] (bit set = +1,
 * LSB first), S bf16 [R]. K % 8 == 0.
 * Replaces: torch.ops.biloco.binary_z_reference (csrc/bindings.cpp:46, csrc/reference_ops.cu:169-215). */
int biloco_b200_binary_z(const void* X_bf16, const void* V_packed, const void* S_bf16, float* z,
                         int M, int K, int R, biloco_stream_t stream);

/* Y[m,n] = bf16( sum_i z[m,i] sign(U[i,n]) ).   z fp32 [M,R], U_packed u8 [R,N/8], Y bf16 [M,N]. N % 8 == 0.
 * Replaces: torch.ops.biloco.binary_expand_reference (csrc/bindings.cpp:47, csrc/reference_ops.cu:217-252). */
int biloco_b200_binary_expand(const float* z, const void* U_packed, void* Y_bf16,
                              int M, int N, int R, biloco_stream_t stream);

/* U_packed u8 [R, N/8] -> U_col32 int32 [N, ceil(R/32)] (bit b of word w of column n = sign of rank 32w+b).
 * Replaces: biloco/kernel.py:37-47 (pack_u_col32, a host loop in the reference). N % 8 == 0. */
int biloco_b200_pack_u_col32(const void* U_packed, int32_t* U_col32, int N, int R, biloco_stream_t stream);

/* NVFP4 activation quantiser: X bf16 [M,K] -> codes u8 [A_rows, K/2] (rows >= M zeroed), block scales
 * (E4M3, 128x4 atom layout, biloco_b200_sf_bytes(A_rows,K) bytes, fully written), a_gscale fp32 [1]
 * (decode scale of the tensor) and, if w_gscale != NULL, alpha_out[0] = w_gscale[0] * a_gscale[0].
 * If smooth_bf16 != NULL the input is first divided by it per channel (result rounded to bf16) and, if
 * Xs_bf16 != NULL, that smoothed activation is written there (the low-rank term consumes it).
 * One global scale per call over all M rows (biloco/fp4.py:3-4). K % 64 == 0, M <= A_rows <= 128.
 * With BILOCO_RULE_GIVEN_SCALE the scale is an input: ranks that each hold a K-slice of one activation first agree on
 * amax (a one-float max all-reduce) and so quantise exactly as a single device would.
 * Replaces: biloco/fp4.py:30-35 (fake_quantize_fp4 -> fouroversix.quantize_to_fp4) and the x/smooth_scale
 * division of biloco/layer.py:55. */
int biloco_b200_act_quant(const void* X_bf16, const void* smooth_bf16, void* Xs_bf16,
                          void* A_codes, void* A_sf, float* a_gscale, float* alpha_out, const float* w_gscale,
                          int M, int A_rows, int K, int rule, biloco_stream_t stream);

/* The same with the step in front of the linear folded in (the decode-step fusion around the path): if
 * norm_weight_bf16 != NULL, every row is first RMS-normalised, x * rsqrt(mean(x^2) + eps) rounded to bf16, times the bf16
 * weight, rounded to bf16 (then divided by smooth_bf16 if given), and that activation is written to Xn_bf16 [M,K]
 * (required then; it is what the low-rank term and the quantisation consume). w_gscale / alpha_out are arrays of
 * n_alpha (1..16) entries: one decode scale per linear that consumes this activation (q/k/v, gate/up), so the
 * activation is quantised once for all of them.
 * No counterpart in the reference (its layers call fake_quantize_fp4 per linear, biloco/layer.py:60, and the norm
 * lives in the surrounding model). */
int biloco_b200_norm_act_quant(const void* X_bf16, const void* norm_weight_bf16, float eps, const void* smooth_bf16,
                               void* Xn_bf16, void* A_codes, void* A_sf, void* A_rec, float* a_gscale, float* alpha_out,
                               const float* w_gscale, int n_alpha, int M, int A_rows, int K, int rule,
                               biloco_stream_t stream);

/* The same with the gated activation of a SwiGLU block folded in: GU_bf16 is [M, 2K] = [gate | up] (the stacked output
 * of a gate/up launch), the activation is bf16(bf16(silu(gate)) * up) with silu(g) = g / (1 + exp(-g)) in fp32 (the
 * roundings of the separate silu and multiply it replaces), divided by smooth_bf16 if given; it is written to Xa_bf16
 * [M, K] (required) and quantised. No counterpart in the reference (the surrounding model does this in torch). */
int biloco_b200_swiglu_act_quant(const void* GU_bf16, const void* smooth_bf16, void* Xa_bf16, void* A_codes, void* A_sf,
                                 void* A_rec, float* a_gscale, float* alpha_out, const float* w_gscale, int n_alpha, int M,
                                 int A_rows, int K, int rule, biloco_stream_t stream);

/* All-reduce of the K-sharded linears' fp32 partial outputs over peer memory, ONE launch per rank (one process per GPU;
 * plain NVLink stores and loads, no library collective). Every rank creates a receive buffer of
 * biloco_b200_peer_buffer_bytes(world, slot_elems) bytes (biloco_b200_peer_buffer_create: device memory, zeroed, plus
 * its 64-byte inter-process handle), sends the handle to its peers by whatever means the host has (the Python side uses
 * torch.distributed.all_gather_object) and maps theirs (biloco_b200_peer_buffer_open). recv_ptrs_dev: device array of
 * `world` pointers, entry p = rank p's buffer as mapped in this process (entry `rank`: the local one). A call:
 *     out[i] = round( sum over ranks p = 0 .. world-1, in that order, of partial_p[i]  (+ residual[i]) ),  i < count
 * The calls of a group are numbered by a counter the kernel keeps in `status` (so a captured CUDA graph can be
 * replayed); the ranks must issue the group's calls in the same order. Rank r stores {value, call number} words into its
 * slot of every peer's buffer and polls its own buffer for the peers' words: one traversal of the link; every rank forms
 * the same sum bit for bit. count <= slot_elems.
 * out: bf16 (or fp32 with BILOCO_OUT_FP32 in flags); residual_bf16 may be NULL. status: int32 [16] on the device, zeroed
 * once before the first call and then left alone (word 8 is the call counter); word 0 becomes 1 when a poll ran out of
 * its time budget (BILOCO_OPT_WAIT_BUDGET_US; the call's output is then undefined). No counterpart in the reference. */
#define BILOCO_AR_PUSHED 0x1          /* flags of biloco_b200_peer_allreduce: the partial's producer has pushed it already */
size_t biloco_b200_peer_buffer_bytes(int world, int slot_elems);
int biloco_b200_peer_buffer_create(size_t bytes, void** ptr, void* handle64);
int biloco_b200_peer_buffer_open(const void* handle64, void** ptr);
int biloco_b200_peer_buffer_close(void* ptr);
int biloco_b200_peer_buffer_destroy(void* ptr);
int biloco_b200_peer_allreduce(const float* partial, const void* residual_bf16, void* out, void* const* recv_ptrs_dev, int* status,
                               int world, int rank, int count, int slot_elems, int flags, biloco_stream_t stream);

/* biloco_b200_fused_linear_rec whose epilogue also PUSHES its fp32 outputs to the peers of a row-parallel group (schedules
 * 2 / 4 / 5 with BILOCO_OUT_FP32 in `mode`): the thread that stores Y[m, n] also stores {value, call number} into this rank's
 * slot of every peer's receive buffer (recv_ptrs_dev, ar_status, world, rank, slot_elems as for
 * biloco_b200_peer_allreduce; M * N <= slot_elems), so the transfer over NVLink starts tile by tile with the epilogue
 * instead of with a later launch. The all-reduce is completed by biloco_b200_peer_allreduce(..., flags | BILOCO_AR_PUSHED),
 * issued next on the same stream with the same partial (Y) — it only gathers. No counterpart in the reference. */
int biloco_b200_fused_linear_push(const void* W_codes, const void* W_sf, const void* W_tiled, const float* alpha,
                                  const void* A_codes, const void* A_sf, const void* A_rec, const void* X_bf16,
                                  const void* V_packed, const int32_t* U_col32, const void* S_bf16, const void* C_bf16,
                                  void* Y_f32, void* scratch, size_t scratch_bytes, int M, int A_rows, int N, int K, int R,
                                  int mode, int epoch, void* const* recv_ptrs_dev, const int* ar_status, int world, int rank,
                                  int slot_elems, biloco_stream_t stream);

/* Greedy sign peeling on the GPU:  W ~ sum_i S[i] u_i v_i^T + R  with u_i, v_i in {+-1}  (the decomposition that yields
 * the packed low-rank operands). R: fp32 [m][n] on the device, holds W on entry and the residual on return (updated in
 * place). v_init: fp32 [r][n], the random start vector of every atom (only its signs are used; sgn(0) = +1). Atom i:
 * v = sgn(v_init[i]); T times  u = sgn(R v), v = sgn(R^T u);  S[i] = u^T R v / (m n);  R <- R - S[i] u v^T.
 * Outputs: U fp32 [m][r], V fp32 [n][r] (+-1), S fp32 [r]. scratch: biloco_b200_peel_scratch_bytes(m, n, 0) bytes, 16-byte
 * aligned (0 = shape not taken: n % 4 != 0 or n > 14336). The call returns when the work is done (it synchronises the
 * stream: an offline step, not for graph capture); BILOCO_ERR_WAIT if a bounded device-side wait for a row copy ran out. Sums are fp32 in a fixed order (deterministic); one pass over the
 * residual performs a whole alternation and carries the previous atom's update (see csrc/peel.cu).
 * Replaces: binary_peel (biloco/peel.py:14-42), which issues 2 T + 2 library products and an outer-product update per atom. */
size_t biloco_b200_peel_scratch_bytes(int m, int n, int num_sms);
int biloco_b200_binary_peel(float* R, const float* v_init, float* U, float* V, float* S, void* scratch, size_t scratch_bytes,
                            int m, int n, int r, int T, biloco_stream_t stream);

/* The fused decode linear on a RAW activation, one launch (row-slab schedule, M <= 2): the kernel forms the activation
 * the linear sees, quantises it to NVFP4 itself and multiplies -- no quantiser launch in front and no A_codes / A_sf /
 * alpha / X buffers in between. Per row of X_raw (bf16 [M,K]; [M,2K] = [gate | up] with swiglu != 0):
 *     x = X_raw                                                      (norm_weight == NULL, swiglu == 0)
 *     x = bf16(bf16(X_raw * rsqrt(mean(X_raw^2) + eps)) * norm_weight)          (norm_weight: bf16 [K])
 *     x = bf16(bf16(silu(gate)) * up)                                           (swiglu; not together with norm_weight)
 *     x = bf16(x / smooth)                                                      (smooth: bf16 [K], may be NULL)
 * then the tensor scale, block scales and codes of biloco_b200_act_quant for `rule` (BILOCO_RULE_STATIC_6 / _STATIC_4 /
 * _MSE, bit for bit the same as that launch gives), alpha = w_gscale[0] * tensor scale, and
 *     Y[m,n] = bf16( alpha * sum_k A[m,k] W[n,k]  +  sum_i z[m,i] sign(U[i,n])  (+ C[m,n]) ),  z = S .* (x sign(V)^T).
 * W_slab: the copy made by biloco_b200_tile_weights_slab; w_gscale: fp32 [1] on the device (the weights' tensor scale,
 * static like the weights: it is read before the previous kernel of the stream has finished). act_out (may be NULL):
 * fp32 [2] on the device, receives the activation's tensor scale and alpha. flags: BILOCO_OUT_FP32 (Y is fp32) or 0.
 * scratch: as for biloco_b200_fused_linear (biloco_b200_scratch_bytes for the same M, N, K, R), same bounded waits and
 * status words. Shapes: those biloco_b200_slab_info accepts with enough shared memory left for M rows of K bf16.
 * Replaces: the reference layer's activation path in front of its linear -- division by smooth_scale, fake_quantize_fp4
 * (biloco/layer.py:55,60; biloco/fp4.py:30-35) -- together with torch.ops.biloco.biloco_gemm_mode2/4/5
 * (csrc/bindings.cpp:37-43); the reference runs them as separate kernels. */
int biloco_b200_fused_linear_act_supported(int M, int N, int K, int R, int num_sms);      /* 1 / 0; num_sms = 0: current device */
int biloco_b200_fused_linear_act(const void* W_slab, const float* w_gscale, const void* X_raw_bf16,
                                 const void* norm_weight_bf16, float eps, const void* smooth_bf16, int swiglu, int rule,
                                 const void* V_packed, const int32_t* U_col32, const void* S_bf16, const void* C_bf16,
                                 void* Y, float* act_out, void* scratch, size_t scratch_bytes, int M, int N, int K, int R,
                                 int flags, int epoch, biloco_stream_t stream);

/* A_rec (optional, biloco_b200_act_rec_bytes(M, K) bytes, K % 256 == 0, M <= 32): the same codes and block scales once
 * more, laid out per 256-wide k-tile exactly as the fused kernel keeps them in shared memory (the activation tile with
 * the 128-byte swizzle applied, followed by its four scale atoms). biloco_b200_fused_linear_rec then fetches the
 * activation side of a work unit with ONE bulk copy instead of a tiled TMA load plus a bulk copy (two requests per
 * unit instead of three, no tensor map on the path; results are bit-identical, and the measured time is the same).
 * Internal layout of this library (like the unit-contiguous weights); no counterpart in the reference. */
size_t biloco_b200_act_rec_bytes(int M, int K);
int biloco_b200_fused_linear_rec(const void* W_codes, const void* W_sf, const void* W_tiled, const float* alpha,
                                 const void* A_codes, const void* A_sf, const void* A_rec, const void* X_bf16,
                                 const void* V_packed, const int32_t* U_col32, const void* S_bf16, const void* C_bf16,
                                 void* Y_bf16, void* scratch, size_t scratch_bytes, int M, int A_rows, int N, int K,
                                 int R, int mode, int epoch, biloco_stream_t stream);

/* Several linears that read the same activation (q/k/v, gate/up) in ONE launch: n_groups (1..4) column groups stacked
 * along N, group g covering group_rows[g] output columns (host array; every entry a multiple of 128, their sum = N).
 * Every group has its own R ranks (R a multiple of 32): V_packed [n_groups*R, K/8] and S_bf16 [n_groups*R] are the
 * groups' factors stacked in group order, U_col32 [N, R/32] holds for every column the sign words of its own group's
 * ranks, alpha is an array of n_groups decode scales (what biloco_b200_norm_act_quant writes for n_alpha = n_groups).
 * W_codes / W_sf / W_tiled are the groups' weights stacked along N (each group re-laid on its own or all at once: the
 * same bytes), C_bf16 / Y_bf16 are [M, N]. The z stage computes all n_groups*R ranks once; a column tile expands its
 * own group's. Scratch: biloco_b200_scratch_bytes(M, N, K, n_groups * R, num_sms). A_rec may be NULL.
 * Column for column the result equals the separate launches' up to the fp32 summation order of the k split.
 * No counterpart in the reference (one launch per linear, biloco/kernel.py:121-130). */
int biloco_b200_fused_linear_grouped(const void* W_codes, const void* W_sf, const void* W_tiled, const float* alpha,
                                     const void* A_codes, const void* A_sf, const void* A_rec, const void* X_bf16,
                                     const void* V_packed, const int32_t* U_col32, const void* S_bf16, const void* C_bf16,
                                     void* Y_bf16, void* scratch, size_t scratch_bytes, int M, int A_rows, int N, int K,
                                     int R, int n_groups, const int* group_rows, int mode, int epoch,
                                     biloco_stream_t stream);

/* Clusters of `cluster` (2..8) CTAs of the fused kernel for M activation rows that the current device keeps resident at
 * the same time (driver query; 0 if it fails). The cluster schedule needs one per 128-column tile, because every CTA of
 * a launch must be resident at once; biloco_b200_mode_supported(..., num_sms = 0) and the launcher take it into account.
 * No counterpart in the reference. */
int biloco_b200_max_active_clusters(int M, int cluster);

/* One decode step of attention between the stacked q/k/v launch and the output projection, as one launch: qkv_bf16
 * [M, (H + 2*KVH) * D] (q heads, k heads, v heads; D = 64 or 128); optional per-head RMS norm of q and k (bf16 [D] weights,
 * NULL = none); rotary embedding (halves convention) from cos_table / sin_table fp32 [max_len, D/2] at the position
 * pos_dev[0] (int64 in device memory, so that a captured graph can be replayed while it advances); the new key and value
 * are written to k_cache / v_cache bf16 [M, KVH, max_len, D] at that position; out_bf16 [M, H*D] = softmax(q k^T /
 * sqrt(D)) v over positions 0 .. pos, fp32 arithmetic on bf16 inputs. Query head h reads KV head h / (H / KVH).
 * No counterpart in the reference (the surrounding model does this with framework tensor operations). */
int biloco_b200_decode_attention(const void* qkv_bf16, const void* q_norm_bf16, const void* k_norm_bf16, float eps,
                                 const float* cos_table, const float* sin_table, const long long* pos_dev,
                                 void* k_cache_bf16, void* v_cache_bf16, void* out_bf16, int M, int H, int KVH, int D,
                                 int max_len, biloco_stream_t stream);

/* Scratch bytes needed by biloco_b200_fused_linear for this problem on a device
 * with `num_sms` multiprocessors (0 = query the current device). The scratch must be zero-filled once
 * before the first call; it needs no clearing between calls (the reference's BiLoCoGemm owns z/flags/corr/cnt
 * buffers the same way, biloco/kernel.py:98-119). Its first biloco_b200_scratch_head_bytes() bytes hold the
 * status words and counters: zero those again after a call whose status word reported a wait that ran out.
 * Calls that share a scratch must not overlap on the device. Returns 0 for an unsupported shape. Host-only
 * arithmetic unless num_sms == 0. */
size_t biloco_b200_scratch_bytes(int M, int N, int K, int R, int num_sms);

/* Bytes at the start of the scratch that hold status words and counters (what BiLoCoGemm.reset() clears,
 * biloco/kernel.py:115-119). */
size_t biloco_b200_scratch_head_bytes(int M, int N, int K, int R, int num_sms);

/* Work split the fused kernel will use for this problem: out[0] = 128-row tiles, out[1] = 256-wide k-tiles,
 * out[2] = CTAs launched, out[3] = partial-sum slots per tile, out[4] = MMA N (8/16/32), out[5] = pipeline
 * stages. Host-only; for tests and sizing. No counterpart in the reference (its tiling is fixed by CUTLASS
 * template parameters, csrc/biloco_gemm.cu:3017-3020). */
int biloco_b200_schedule_info(int M, int N, int K, int R, int num_sms, int* out6);

/* Bytes of the unit-contiguous copy of an [N, K] NVFP4 weight (codes + block scales, N padded to 128). */
size_t biloco_b200_tiled_bytes(int N, int K);

/* Re-layout W_codes u8 [N,K/2] + W_sf (atom layout) into the order the fused kernel streams them: one contiguous
 * 18 KB record per (128-row tile, 256-wide k-tile) = the 128x128 B block of codes with the shared-memory swizzle
 * already applied, followed by its four 512 B scale atoms. Done once per layer; lets every weight read of the
 * fused kernel be a sequential 18 KB burst instead of 128 strided 128 B pieces.
 * Replaces: the operand re-layouts BiLoCoGemm.__init__ performs in the reference (pack_v_perm / U_rw,
 * biloco/kernel.py:98-102). K % 256 == 0; 16-byte aligned pointers. */
int biloco_b200_tile_weights(const void* W_codes, const void* W_sf, void* W_tiled, int N, int K, biloco_stream_t stream);

/* Row-slab copy of an [N, K] NVFP4 weight for BILOCO_MODE_SLAB: per CTA slab c (rows c Rt .., Rt = ceil8(N / num_sms))
 * and per group of kg = min(128 / Rt, 4) consecutive k-tiles one contiguous record = the codes of the group's units
 * with the shared-memory swizzle applied (row g Rt + r of the tensor-core tile), followed by their block scales
 * (16 bytes per row and unit). The layout depends on N, K and the SM count only (num_sms = 0: the current device).
 * biloco_b200_slab_bytes returns 0 for shapes the schedule does not take. biloco_b200_slab_info: out[0..7] = Rt, kg,
 * k-tiles, records per CTA, CTAs, pipeline stages, shared memory per CTA, most ranks of a z slice (for tests and sizing).
 * Replaces: the operand re-layouts BiLoCoGemm.__init__ performs in the reference (biloco/kernel.py:98-102). */
size_t biloco_b200_slab_bytes(int N, int K, int num_sms);
int biloco_b200_slab_info(int M, int N, int K, int R, int num_sms, int* out8);
int biloco_b200_tile_weights_slab(const void* W_codes, const void* W_sf, void* W_slab, int N, int K, int num_sms,
                                  biloco_stream_t stream);

/* The fused decode linear, one launch:
 *     Y[m,n] = bf16( alpha[0] * sum_k A[m,k] W[n,k]  +  sum_i z[m,i] sign(U[i,n]) ),  z = S .* (X sign(V)^T)
 * W_codes u8 [N,K/2], W_sf E4M3 (atom layout, rows padded to 128), alpha fp32 [1] (device), A_codes u8
 * [A_rows,K/2] (A_rows >= M; rows beyond M are ignored), A_sf E4M3 (atom layout), X bf16 [M,K],
 * V_packed u8 [R,K/8], U_col32 int32 [N, ceil(R/32)], S bf16 [R], Y bf16 [M,N] (row stride N).
 * W_tiled (may be NULL): the copy made by biloco_b200_tile_weights; when given it is streamed instead of
 * W_codes / W_sf (which may then be NULL).
 * R == 0 skips the low-rank term (X, V, U, S may then be NULL). C_bf16 (may be NULL): bf16 [M,N] added
* before the final rounding. `epoch` (>= 1) is the caller's launch count on this scratch; it is recorded in the status
 * words when a wait gives up and has no other effect (the validity mark of the z values follows a launch count that the
 * kernels keep in the scratch itself, so a captured CUDA graph can be replayed).
 * Shapes: 1 <= M <= 32, K % 256 == 0, N % 8 == 0. 16-byte alignment for W_codes, A_codes, W_sf, A_sf, X.
 * Device-side waits are bounded; a wait that ran out leaves a non-zero code in the first int32 of scratch
 * (read it with biloco_b200_read_status) and the call's output is undefined.
 * Replaces: torch.ops.biloco.biloco_gemm_mode2/4/5 (csrc/bindings.cpp:37-43; host launcher
 * csrc/biloco_gemm.cu:2986-3431, dispatchers :3435-3562) and, with R == 0, fp4_gemm / fp4_gemm_n64 /
 * fp4_gemm_n128 / fp4_gemm_residual (csrc/bindings.cpp:22-27, csrc/biloco_gemm.cu:2744-2983). */
int biloco_b200_fused_linear(const void* W_codes, const void* W_sf, const void* W_tiled, const float* alpha,
                             const void* A_codes, const void* A_sf, const void* X_bf16,
                             const void* V_packed, const int32_t* U_col32, const void* S_bf16,
                             const void* C_bf16, void* Y_bf16,
                             void* scratch, size_t scratch_bytes,
                             int M, int A_rows, int N, int K, int R,
                             int mode, int epoch, biloco_stream_t stream);

/* The fused decode linear for callers that cannot allocate device memory.
 *
 * Some hosts of this library have no way to obtain scratch: code running inside another framework's stream-ordered
 * or pooled allocator that must not be re-entered from a callback, inference servers that freeze their memory
 * plan at start-up, plugins loaded into a process whose memory budget is fully handed out. biloco_b200_fused_linear
 * asks such a caller for a scratch buffer it cannot provide. This variant takes none: its scratch is an array built
 * into the library (BILOCO_NOALLOC_SCRATCH_BYTES of device memory on every GPU that loads the library, held until the
 * process exits; with the CUDA runtime's lazy module loading the driver sets the array aside when the library's code is
 * first loaded on a device, which on a GPU whose memory is fully committed can make that first call fail with
 * BILOCO_ERR_CUDA). It calls no cudaMalloc / cudaFree and no allocating library routine; inputs and outputs are still
 * the caller's. Same arithmetic and same results as biloco_b200_fused_linear (arguments as there, minus scratch and
 * epoch), with two restrictions: `mode` is BILOCO_MODE_COUNTER or BILOCO_MODE_OWNER (optionally OR-ed with
 * BILOCO_OUT_FP32); BILOCO_MODE_CLUSTER and BILOCO_MODE_SLAB return BILOCO_ERR_MODE here.
 *   - Limit: problems whose biloco_b200_scratch_bytes(M, N, K, R, 0) exceeds BILOCO_NOALLOC_SCRATCH_BYTES are rejected
 *     with BILOCO_ERR_LIMIT (nothing is enqueued). K = N = 5120 needs 0.8 MB (M <= 8) to 2.8 MB (M = 32).
 *   - The first call on a device looks up the array's device address (a set-up step of a few microseconds): make
 *     that first call outside any stream capture.
 *   - All calls on a device share the one array. It keeps what the previous call left; each call clears, on `stream`,
 *     the words that have to start at zero (a cudaMemsetAsync of up to about 0.3 MB in front of the kernel, which also
 *     means that this launch does not start early under the previous kernel of the stream). Two calls that overlap on the GPU (different streams without ordering)
 *     race on it: keep calls to this entry point ordered.
 * No counterpart in the reference (its scratch tensors are allocated by BiLoCoGemm through PyTorch). */
#define BILOCO_NOALLOC_SCRATCH_BYTES (4 * 1024 * 1024)
int biloco_b200_fused_linear_noalloc(const void* W_codes, const void* W_sf, const void* W_tiled, const float* alpha,
                                     const void* A_codes, const void* A_sf, const void* X_bf16,
                                     const void* V_packed, const int32_t* U_col32, const void* S_bf16,
                                     const void* C_bf16, void* Y_bf16,
                                     int M, int A_rows, int N, int K, int R, int mode, biloco_stream_t stream);

/* Status words (as biloco_b200_read_status) of the built-in scratch of the current device; BILOCO_ERR_CUDA before the
 * first biloco_b200_fused_linear_noalloc call on that device. No counterpart in the reference. */
int biloco_b200_noalloc_status(int32_t* out16, biloco_stream_t stream);

/* Copy the 16 int32 status words at the start of a scratch buffer to host memory `out16` (synchronises
 * `stream`). Word 0: 0 = no device-side wait ran out since the scratch was last zeroed; otherwise the code
 * of the first wait that gave up. Words 1..3: block index, epoch and role of that wait. */
int biloco_b200_read_status(const void* scratch, int32_t* out16, biloco_stream_t stream);

/* Process-wide options. BILOCO_OPT_PDL (default 1): launch the fused kernel with programmatic stream
 * serialization, so that its set-up and its weight prefetch overlap the tail of the previous kernel of the stream
 * (the kernel itself waits for that kernel before it reads activations or touches scratch). 0 = plain launches.
 * The reference launches with a "pdl" flag as well (csrc/biloco_gemm.cu:3421-3429). */
/* Contract that comes with it: the fused kernels read their STATIC operands (W_codes / W_sf / W_tiled, V_packed, U_col32,
 * S) before that wait, so these must be complete before the kernel that precedes the fused launch on the stream begins.
 * The library's own re-layout calls (biloco_b200_tile_weights, biloco_b200_tile_weights_slab, biloco_b200_pack_u_col32)
 * are covered: the first fused launch that follows one of them on the same stream is issued as a plain launch. A caller
 * that writes these operands with a kernel of its own directly in front of a fused launch sets BILOCO_OPT_PDL to 0 for
 * that launch (or puts any other kernel in between). Activations, alpha, C and the scratch are read after the wait. */
#define BILOCO_OPT_PDL 1
/* Pipeline stages the fused kernel keeps in flight. 0 (default): chosen by the library - for M <= 8 with dependent
 * launch on, a ring of 4 stages so that two consecutive launches are resident on an SM at the same time (the second
 * one's first weights are in shared memory before the first has finished); otherwise all the stages that fit.
 * Other values are clamped to [4, what fits]. */
#define BILOCO_OPT_RING 2
/* Where a CTA of the fused kernel allows the next kernel of the stream to start (programmatic dependent launch):
 * -1 (default) chosen by the library, 0 after set-up, 4 after its dependency wait, 3 once its activation row has
 * landed, 1 after its z stage, 2 after its first expansion. Tuning aid. */
#define BILOCO_OPT_TRIGGER 3
/* 1 (default): from 16 activation rows up the expansion of z through the U signs runs on the tensor cores (bf16 sign
 * image x z split into two bf16 parts, fp32 accumulation); 0: on the CUDA cores for every row count. */
#define BILOCO_OPT_LR_TC 4
/* Budget of a device-side wait in microseconds (default 200 000; <= 0 restores the default). A wait that runs out
 * records its code in the status words and the launch returns (row-slab schedule; the other schedules keep 200 ms).
 * Counterpart in the reference: the bounded polls that record codes in Diag[4095] (csrc/biloco_gemm.cu:1149-1151). */
#define BILOCO_OPT_WAIT_BUDGET_US 5
/* Test aid for the failure path: CTA `value` of a row-slab launch computes its z values but does not publish them, so
 * that every consumer's poll runs out of its budget (-1, the default: off). */
#define BILOCO_OPT_SKIP_PUBLISH 6
/* Row-slab schedule: weight records a CTA keeps in flight while it fills its ring ahead of the dependency wait
 * (0, the default: chosen by the library). Tuning aid. */
#define BILOCO_OPT_INFLIGHT 7
/* z stage as a tensor-core launch of its own in front of the fused launch (schedules 2 / 4 / 5): -1 (default) from 16
 * activation rows, 0 never, n > 0 from n rows. */
#define BILOCO_OPT_ZTC 8
int biloco_b200_set_option(int option, int value);

/* Debug aid: while a device buffer is registered here, every fused launch of this process writes 16 uint64
 * %globaltimer stamps per CTA into it (CTA c at words 16c..16c+15: 0 set-up done, 1 z published, 2 z complete seen,
 * 3 expansion done, 4 accumulators ready, 5/6 first/last segment stored, 7 last stage consumed, 8 first z reads
 * landed, 9 z computed, 10 CTA entry, 11 previous kernel complete, 13 CTA exit). bytes >= 128 * CTAs; a larger
 * buffer is used as consecutive slots of 128 * CTAs bytes by consecutive launches, round-robin; NULL turns it off.
 * Counterpart in the reference: the optional Diag tensor (csrc/biloco_gemm.cu:313-317, 446-464). */
int biloco_b200_debug_stamps(void* device_buf, size_t bytes);

/* CUDA-core FP4 GEMM used to cross-check the tensor-core path on the device at full size:
 * D[m,n] = bf16(alpha[0] * sum_k A[m,k] W[n,k] + C[m,n]). Same operand formats as above; K % 16 == 0.
 * Replaces (functionally): torch.ops.biloco.fp4_gemm_residual as used by biloco/kernel.py:137-142. */
int biloco_b200_fp4_gemm_simt(const void* A_codes, const void* A_sf, const void* W_codes, const void* W_sf,
                              const float* alpha, const void* C_bf16, void* D_bf16,
                              int M, int N, int K, biloco_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* BILOCO_B200_H_ */
