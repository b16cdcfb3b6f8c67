/*
 * fluxb200 — C ABI of the B200 (sm_100a) kernels for the Flux DiT block forward path.
 *
 * Every entry point takes raw device pointers, explicit sizes/strides (in ELEMENTS unless a
 * name says bytes), a dtype code and a CUDA stream, launches on that stream without
 * synchronising, and returns 0 or a negative FLUXB_ERR_* code (text via fluxb_last_error()).
 * Outputs are caller-allocated; inputs are borrowed until the stream reaches the launch.
 * Unless stated otherwise the entry points allocate nothing on the device; the only device
 * allocation the library ever makes is one 8-byte status word per device on first use.
 *
 * Each declaration names the function of ai-compiler-study/triton-kernels it stands in for
 * (paths relative to that project's root).
 */
#ifndef FLUXB200_H_
#define FLUXB200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes. */
#define FLUXB_OK 0
#define FLUXB_ERR_BAD_ARG (-1)     /* null pointer, negative size, misaligned pointer/stride */
#define FLUXB_ERR_UNSUPPORTED (-2) /* dtype / shape outside what the kernels implement */
#define FLUXB_ERR_CUDA (-3)        /* a CUDA runtime/driver call failed (launch, encode) */
#define FLUXB_ERR_TIMEOUT (-4)     /* a bounded device-side wait gave up (status word) */

/* Element types of activations.  Tensor-core kernels accept FLUXB_BF16 only. */
#define FLUXB_F32 0
#define FLUXB_BF16 1

/* GEMM epilogues (fluxb_linear). */
#define FLUXB_EPI_NONE 0       /* y = acc + bias */
#define FLUXB_EPI_GELU 1       /* y = gelu_tanh(acc + bias) */
#define FLUXB_EPI_GATE_RESID 2 /* y = resid + gate[batch] * (acc + bias) */

typedef void* fluxb_stream_t; /* a cudaStream_t */

/* Library / device utilities (no counterpart in the reference). */
int fluxb_version(void);
const char* fluxb_last_error(void);
/* Reads and clears the per-device status word written by kernels whose bounded waits gave
 * up.  Synchronises the device.  out[0] = code (0 = none), out[1] = kernel-specific tag. */
int fluxb_device_status_read(int* out2);

/*
 * y[M,N] = x[M,K] · w[N,K]^T (+ bias[N]) with a fused epilogue; bf16 in, fp32 accumulate in
 * TMEM, bf16 out.  Replaces triton_kernels/kernels/linear.py:104-151 (`linear`, kernel
 * `_linear_fwd` :31-101, `gelu` :22-28) and the un-launched triton_kernels/ops/linear.py:5-71.
 *   x: row stride ldx, w: row stride ldw (nn.Linear layout, K contiguous), y: row stride ldy.
 *   Output columns [0, split) go to y, columns [split, N) go to y2 (row stride ldy2, column
 *   c lands at y2[r*ldy2 + c - split]) with epilogue `epi2`; pass split = N, y2 = NULL for a
 *   single output.  split must be a multiple of 256.
 *   FLUXB_EPI_GATE_RESID: y = resid[r*ldr + c] + gate[(r / rows_per_batch) * gate_stride + c]
 *   * (acc + bias); replaces the torch elementwise pair at triton_kernels/modules/blocks.py:123,
 *   166-171 and triton_kernels/ops/modulation.py:29-44.
 *   round_before_act != 0 rounds acc + bias to bf16 before GELU, as `_linear_fwd` does (:92-95).
 *   Pointers must be 16-byte aligned; K, ldx, ldw multiples of 8; N, ldy multiples of 8.
 */
int fluxb_linear(const void* x, const void* w, const void* bias, void* y, int64_t M, int64_t N,
                 int64_t K, int64_t ldx, int64_t ldw, int64_t ldy, int epi, void* y2, int64_t ldy2,
                 int64_t split, int epi2, const void* resid, int64_t ldr, const void* gate,
                 int64_t gate_stride, int64_t rows_per_batch, int round_before_act,
                 fluxb_stream_t stream);

/*
 * Up to four linears that share N, K and the epilogue but have their own operands, outputs
 * and row counts, run as ONE launch (their tiles share the persistent grid).  The double-stream
 * block uses it to run the image-stream and text-stream projections together: alone, the
 * 512-token text GEMMs fill a third of the SMs.  Replaces pairs of calls such as
 * triton_kernels/modules/blocks.py:147+153, 166+170 and the two MLPs at :167-171.
 * Fields have the meaning of the fluxb_linear arguments of the same name.
 */
typedef struct {
  const void* x;
  const void* w;
  const void* bias;
  void* y;
  int64_t M, ldx, ldw, ldy;
  void* y2;
  int64_t ldy2;
  const void* resid;
  int64_t ldr;
  const void* gate;
  int64_t gate_stride, rows_per_batch;
} fluxb_linear_problem;
int fluxb_linear_grouped(const fluxb_linear_problem* problems, int count, int64_t N, int64_t K,
                         int epi, int64_t split, int epi2, int round_before_act,
                         fluxb_stream_t stream);

/*
 * out[b, n] = sum_k silu(vec[b,k]) * w[n,k] + bias[n]  for small b (<= 8): the adaLN
 * modulation projection.  Replaces `Modulation.forward`, triton_kernels/modules/blocks.py:61-67
 * (F.silu + tk.linear with M = batch) and triton_kernels/ops/silu.py:5-13 as its prologue.
 * apply_silu = 0 gives a plain small-M linear.  bf16 storage, fp32 accumulation.  For K a
 * multiple of 1536 silu(vec) is rounded to bf16 before the products (as the reference's bf16
 * SiLU output is) and the products run on the tensor pipe; other K keep silu(vec) in fp32.
 */
int fluxb_modulation_gemv(const void* vec, const void* w, const void* bias, void* out, int64_t B,
                          int64_t N, int64_t K, int apply_silu, fluxb_stream_t stream);

/*
 * fluxb_modulation_gemv over a range of output rows: w, bias and out point at the first row of the
 * range (N rows), out rows of different batch items lie out_stride elements apart (the packed
 * [B, 6C] modulation tensor is filled in two calls).  light != 0 launches 128-thread blocks, at
 * most two per SM, which fit beside a tensor-core kernel holding one block per SM: the half of
 * the projection that is needed only after attention streams its weights during the q|k|v GEMM.
 * No counterpart in the reference (its Modulation is one `linear` call).
 */
int fluxb_modulation_gemv_rows(const void* vec, const void* w, const void* bias, void* out,
                               int64_t B, int64_t N, int64_t K, int64_t out_stride, int apply_silu,
                               int light, fluxb_stream_t stream);

/*
 * Non-causal attention softmax(q k^T * sm_scale) v, bf16, head_dim 64 or 128.
 * Replaces triton_kernels/kernels/attention.py:173-221 (`scaled_dot_product_attention`,
 * kernels `_attn_fwd` :69-170 / `_attn_fwd_inner` :10-46).
 *   q,k,v: [B,H,L,D] addressed through element strides (batch, head, row); last dim contiguous.
 *   o: same addressing with its own strides, so the caller can ask for [B,L,H*D] directly
 *   (the rearrange at triton_kernels/modules/blocks.py:14) or write into a wider buffer.
 *   Any Lq, Lk >= 1 (tails masked).  Strides must be multiples of 8 elements.
 */
int fluxb_attention(const void* q, const void* k, const void* v, void* o, int64_t B, int64_t H,
                    int64_t Lq, int64_t Lk, int64_t D, int64_t q_sb, int64_t q_sh, int64_t q_sl,
                    int64_t k_sb, int64_t k_sh, int64_t k_sl, int64_t v_sb, int64_t v_sh,
                    int64_t v_sl, int64_t o_sb, int64_t o_sh, int64_t o_sl, float sm_scale,
                    fluxb_stream_t stream);

/*
 * y = LayerNorm(x) (no affine, biased variance, eps) * (1 + scale[b]) + shift[b].
 * Replaces triton_kernels/kernels/normalization.py:47-77 (`layer_norm_modulation`, kernel
 * `_layer_norm_modulation_fwd` :8-44) and triton_kernels/ops/modulation.py:5-27.
 *   x: rows x cols, row stride x_ld; y: row stride y_ld; batch index = row / rows_per_batch;
 *   scale/shift: cols contiguous, batch stride mod_stride (chunk views of the packed
 *   modulation tensor are passed without copying).  Statistics in fp32: one pass over rows of
 *   2-24 KB (mean and E[x^2] together; fp32 rows shifted by their first element), mean then
 *   centred variance otherwise.
 */
int fluxb_layer_norm_modulation(const void* x, const void* scale, const void* shift, void* y,
                                int64_t rows, int64_t cols, int64_t rows_per_batch, int64_t x_ld,
                                int64_t y_ld, int64_t mod_stride, float eps, int dtype,
                                fluxb_stream_t stream);

/*
 * y = x * rsqrt(mean(x^2) + eps) * w over the last dim.  Replaces
 * triton_kernels/kernels/normalization.py:142-169 (`_rms_norm.forward`, kernel `_rms_norm_fwd`
 * :80-106).  x is addressed as [n0,n1,n2,cols] with element strides s0,s1,s2 (last dim
 * contiguous) so head-split views need no copy; y is contiguous.  w has dtype `dtype`.
 * rstd (optional, fp32, one per row) is what the reference saves for backward.
 */
int fluxb_rms_norm(const void* x, const void* w, void* y, float* rstd, int64_t n0, int64_t n1,
                   int64_t n2, int64_t cols, int64_t s0, int64_t s1, int64_t s2, float eps,
                   int dtype, fluxb_stream_t stream);

/*
 * RMSNorm backward: dx = rstd*(dy*w) - rstd^3/cols * sum(dy*w*x) * x and dw = sum_rows
 * dy*x*rstd.  Replaces triton_kernels/kernels/normalization.py:171-190 (`_rms_norm.backward`,
 * kernel `_rms_norm_bwd` :109-139).  All tensors contiguous [rows, cols]; dw_partial is
 * caller-provided fp32 scratch of dw_partial_rows x cols that the kernel fills with per-block
 * column sums (the caller reduces it over rows); dw_partial_rows is returned by
 * fluxb_rms_norm_bwd_partial_rows().
 */
int64_t fluxb_rms_norm_bwd_partial_rows(int64_t rows);
int fluxb_rms_norm_bwd(const void* dy, const void* x, const void* w, const float* rstd, void* dx,
                       float* dw_partial, int64_t rows, int64_t cols, int dtype,
                       fluxb_stream_t stream);

/*
 * RMSNorm backward for callers that must not allocate.  (No counterpart in the reference: it
 * allocates freely through torch.)
 *
 * Who needs it: code that runs where device allocation is off limits — inside a serving loop
 * with a frozen memory plan, under a host-side allocator that forbids cudaMalloc after start-up,
 * in a plugin whose host only hands it a stream and finished buffers.  fluxb_rms_norm_bwd asks
 * such a caller for fp32 scratch; this entry point instead keeps the scratch in a fixed 4 MiB
 * array inside the library image (resident on every GPU that loads the library, until exit)
 * and also does the final reduction, so the caller passes only inputs and outputs:
 *   dx [rows, cols] (dtype), dw [cols] fp32.
 * It never calls cudaMalloc / cudaFree or any allocating routine.
 * Limit: ceil(rows / 64) * cols <= fluxb_rms_norm_bwd_static_max_floats() (1 Mi floats);
 * larger problems are rejected with FLUXB_ERR_UNSUPPORTED.
 * The first call on each device looks the array's address up (a one-time host-side query);
 * make that first call outside any stream capture.
 * All calls on a device share the one array: two calls whose kernels may run at the same
 * time (different streams, no ordering between them) race on it.  Calls ordered on one stream
 * are safe, and no call depends on what an earlier one left in the array.
 */
int fluxb_rms_norm_bwd_static_max_floats(void);
int fluxb_rms_norm_bwd_static(const void* dy, const void* x, const void* w, const float* rstd,
                              void* dx, float* dw, int64_t rows, int64_t cols, int dtype,
                              fluxb_stream_t stream);

/*
 * Rotary embedding with a general 2x2 table: out[2i+j] = pe[l,i,j,0]*x[2i] + pe[l,i,j,1]*x[2i+1]
 * for q and k.  Replaces triton_kernels/kernels/positional_embedding.py:55-82 (`apply_rope`,
 * kernel `_rope_fwd` :9-52).  q,k,oq,ok: contiguous [BH, L, D]; pe: fp32 [L, D/2, 2, 2].
 */
int fluxb_rope(const void* q, const void* k, const float* pe, void* oq, void* ok, int64_t BH,
               int64_t L, int64_t D, int dtype, fluxb_stream_t stream);

/*
 * Head-major q/k/v assembly for joint attention, optionally with per-stream QK-RMSNorm and
 * RoPE fused in: for every token row of up to two streams (stream 0 rows first — text before
 * image), splits the packed projection row [3*H*D] into q,k,v, normalises q and k per head
 * (if qscale/kscale given), rotates them with pe (if given) and writes q,k,v as [B,H,L,D] with
 * L = L0 + L1.  Replaces triton_kernels/ops/qkv_concat.py:5-60 and, fused, the rearrange /
 * QKNorm / torch.cat / apply_rope sequence at triton_kernels/modules/blocks.py:113-119,148-162
 * (QKNorm at triton_kernels/modules/normalization.py:19-26).
 *   src_s: [B, L_s, ld_s] with the q|k|v columns first; qscale_s/kscale_s: [D] bf16 or NULL.
 *   pe: fp32 [L, D/2, 2, 2] or NULL.  D must be 128.  bf16 only.
 *   Output addressing: heads_per_group <= 0 means contiguous [B,H,L,D].  Otherwise element
 *   (b, h, l, :) of q, k and v lands at b*o_sb + (h / heads_per_group)*o_sg +
 *   (h % heads_per_group)*o_sh + l*o_sl, which lets a sequence-parallel caller have the rows
 *   written directly in the per-destination-rank layout of its head all-to-all (no counterpart
 *   in the reference, which has no multi-GPU path).
 */
int fluxb_qkv_prep(const void* src0, int64_t L0, int64_t ld0, const void* qscale0,
                   const void* kscale0, const void* src1, int64_t L1, int64_t ld1,
                   const void* qscale1, const void* kscale1, const float* pe, void* q, void* k,
                   void* v, int64_t B, int64_t H, int64_t D, int64_t heads_per_group, int64_t o_sb,
                   int64_t o_sg, int64_t o_sh, int64_t o_sl, float eps, fluxb_stream_t stream);

/*
 * out = (1 + scale) * x + shift with shift/scale taken from the packed modulation tensor
 * mod[B, n_chunks*C]: chunks (0,1) if is_mod1 else (3,4).  Replaces
 * triton_kernels/ops/modulation.py:5-27.  x,out: [B, L, C] contiguous.
 */
int fluxb_modulation_scale_shift(const void* x, const void* mod, void* out, int64_t B, int64_t L,
                                 int64_t C, int64_t mod_row_stride, int is_mod1, int dtype,
                                 fluxb_stream_t stream);

/*
 * out = resid + gate * proj with gate = chunk `gate_chunk` (2 or 5) of the packed modulation
 * tensor.  Replaces triton_kernels/ops/modulation.py:29-44.
 */
int fluxb_modulation_gate_proj(const void* resid, const void* mod, const void* proj, void* out,
                               int64_t B, int64_t L, int64_t C, int64_t mod_row_stride,
                               int gate_chunk, int dtype, fluxb_stream_t stream);

/* out = x * sigmoid(x), flat.  Replaces triton_kernels/ops/silu.py:5-13. */
int fluxb_silu(const void* x, void* out, int64_t n, int dtype, fluxb_stream_t stream);

/*
 * The q|k|v projections of up to four token streams (same weights' shape, different operands
 * and row counts) in one launch, with everything between the projection and attention done in
 * the GEMM epilogue: per-head RMS norm of q and k with the stream's scales, rotation with the
 * stream's rows of pe, head-major layout and stream concatenation.  Replaces, fused, the
 * qkv Linear of triton_kernels/modules/blocks.py:33,47 plus the rearrange / QKNorm / torch.cat /
 * apply_rope sequence at triton_kernels/modules/blocks.py:113-119,148-162.
 *   problems[i]: x [B*L_i, K] (ldx), w [3*H*D, K] (ldw), bias [3*H*D] or NULL, M = B*L_i,
 *                rows_per_batch = L_i (a multiple of 128); the other fields are ignored.
 *   streams[i]:  pe fp32 [L_total, D/2, 2, 2] or NULL; q_scale, k_scale bf16 [D] or both NULL;
 *                row_offset = position of the stream's first token in the joint sequence (a
 *                multiple of 128).
 *   qkv_out: bf16 [3, B, H, L_total, D].  D must be 128.  The projection is rounded to bf16
 *   before the norm, as the reference's bf16 Linear output is.
 *   N2 > 0: w has N2 more rows after the 3*H*D of q|k|v (bias likewise); those columns are an
 *   ordinary output, written to problems[i].y2 (row stride ldy2) with epilogue epi2 (none or
 *   GELU, round_before_act as in fluxb_linear).  This is linear1 of the single-stream block
 *   (triton_kernels/modules/blocks.py:93,108-110): qkv and the MLP's up-projection in one GEMM.
 */
typedef struct {
  const float* pe;
  const void* q_scale;
  const void* k_scale;
  int64_t row_offset;
} fluxb_qkv_stream;
int fluxb_linear_qkv_grouped(const fluxb_linear_problem* problems, const fluxb_qkv_stream* streams, int count,
                             int64_t B, int64_t H, int64_t D, int64_t L_total, int64_t K, void* qkv_out,
                             float eps, int64_t N2, int epi2, int round_before_act, fluxb_stream_t stream);

/*
 * fluxb_linear_qkv_grouped with one output base per head group instead of qkv_out (the
 * sequence-parallel form; no counterpart in the reference, whose blocks know one GPU): heads
 * [g*H/n_groups, (g+1)*H/n_groups) of q land at group_bases[g] + b*o_sb + (h % (H/n_groups))*o_sh
 * + l*o_sl with l = row_offset + row, those of k and v k_off and v_off elements further, written
 * with plain 16-byte stores (the bases may point into other ranks' arenas, as for
 * fluxb_qkv_prep_scatter).  Rows are masked one by one: with B == 1 the stream lengths and row
 * offsets need not be multiples of 128.
 */
int fluxb_linear_qkv_grouped_scatter(const fluxb_linear_problem* problems, const fluxb_qkv_stream* streams,
                                     int count, int64_t B, int64_t H, int64_t D, int64_t L_total, int64_t K,
                                     void* const* group_bases, int n_groups, int64_t k_off, int64_t v_off,
                                     int64_t o_sb, int64_t o_sh, int64_t o_sl, float eps, int64_t N2, int epi2,
                                     int round_before_act, fluxb_stream_t stream);

/* ---------------------------------------------------------------------------------------
 * Sequence-parallel (Ulysses) exchange over peer memory.  The reference has no multi-GPU path,
 * so nothing in this section replaces a reference function; the entry points exist so that the
 * two kernels on either side of the head all-to-all store straight into the consuming GPU's
 * memory (plain global stores over NVLink; peers are never read, and never touched by TMA).
 *
 * An "arena" is a device allocation whose first fluxb_peer_header_bytes() bytes belong to the
 * library (arrival flags written by the peers, this rank's epoch counters); the caller lays
 * out its exchange buffers after the header.  One process per GPU: fluxb_peer_alloc + export
 * on the owner, fluxb_peer_open on every other rank (CUDA IPC), then `arenas[r]` is rank r's
 * arena as addressable from the calling process (its own allocation for r == rank).
 * ------------------------------------------------------------------------------------- */
int fluxb_peer_header_bytes(void);
/* Allocates `bytes` (>= header) of zeroed device memory on the current device.  Setup only. */
int fluxb_peer_alloc(int64_t bytes, void** ptr);
int fluxb_peer_free(void* ptr);
/* Writes the 64-byte IPC handle of an arena from fluxb_peer_alloc. */
int fluxb_peer_export(const void* ptr, void* handle64);
/* Maps another process's arena into this one (peer access enabled lazily). */
int fluxb_peer_open(const void* handle64, void** ptr);
int fluxb_peer_close(void* ptr);
/*
 * Barrier halves, stream-ordered, no host synchronisation, safe to capture in a CUDA graph (the
 * epochs live in the arena).  fluxb_peer_signal: everything enqueued on `stream` before it is
 * complete and visible to the other ranks once they pass the matching wait.  fluxb_peer_wait:
 * returns (on the stream) when every rank has signalled `barrier` as many times as this rank
 * has waited on it.  The wait is bounded (2 s): on expiry the device status word reports
 * FLUXB_ERR_TIMEOUT with site 61 + barrier and the stream continues.  barrier: 0 or 1.
 */
int fluxb_peer_signal(const void* const* arenas, int n_ranks, int rank, int barrier, fluxb_stream_t stream);
int fluxb_peer_wait(const void* const* arenas, int n_ranks, int rank, int barrier, fluxb_stream_t stream);

/*
 * fluxb_qkv_prep with one output base per head group: heads [g*heads_per_group,
 * (g+1)*heads_per_group) of q land at group_bases[g] + b*o_sb + (h % heads_per_group)*o_sh +
 * l*o_sl, those of k and v k_off and v_off elements further.  n_groups*heads_per_group == H,
 * n_groups <= 8.  The bases may point into other ranks' arenas.
 */
int fluxb_qkv_prep_scatter(const void* src0, int64_t L0, int64_t ld0, const void* qscale0,
                           const void* kscale0, const void* src1, int64_t L1, int64_t ld1,
                           const void* qscale1, const void* kscale1, const float* pe,
                           void* const* group_bases, int n_groups, int64_t k_off, int64_t v_off,
                           int64_t B, int64_t H, int64_t D, int64_t heads_per_group, int64_t o_sb,
                           int64_t o_sh, int64_t o_sl, float eps, fluxb_stream_t stream);

/*
 * fluxb_attention with one output base per owner of query rows: row r goes to
 * o_bases[r / rows_per_rank] + b*o_sb + h*o_sh + (r % rows_per_rank)*o_sl.  n_ranks <= 8,
 * n_ranks*rows_per_rank >= Lq.  The bases may point into other ranks' arenas.
 */
int fluxb_attention_scatter(const void* q, const void* k, const void* v, void* const* o_bases,
                            int n_ranks, int64_t rows_per_rank, int64_t B, int64_t H, int64_t Lq,
                            int64_t Lk, int64_t D, int64_t q_sb, int64_t q_sh, int64_t q_sl,
                            int64_t k_sb, int64_t k_sh, int64_t k_sl, int64_t v_sb, int64_t v_sh,
                            int64_t v_sl, int64_t o_sb, int64_t o_sh, int64_t o_sl, float sm_scale,
                            fluxb_stream_t stream);

/*
 * fluxb_attention / fluxb_attention_scatter with the keys cut into k_splits ranges that run as
 * separate CTAs, plus a merge pass (no counterpart in the reference; its kernel
 * triton_kernels/kernels/attention.py:69-170 walks all keys in one program).  For grids that
 * leave most SMs idle in their last wave: 3 heads x 66 query blocks = 198 CTAs on 148 SMs run
 * as two waves, 396 half-length CTAs as three half-waves.  n_ranks == 0: plain form, output o;
 * n_ranks > 0: scatter form, o ignored.  part_o: fp32 scratch of k_splits*B*H*Lq*D elements,
 * part_lse: fp32 scratch of k_splits*B*H*Lq elements (caller-owned, contents undefined
 * afterwards).  k_splits == 1 is the ordinary kernel and needs no scratch.
 */
int fluxb_attention_split(const void* q, const void* k, const void* v, void* o, void* const* o_bases,
                          int n_ranks, int64_t rows_per_rank, int64_t B, int64_t H, int64_t Lq, int64_t Lk,
                          int64_t D, int64_t q_sb, int64_t q_sh, int64_t q_sl, int64_t k_sb, int64_t k_sh,
                          int64_t k_sl, int64_t v_sb, int64_t v_sh, int64_t v_sl, int64_t o_sb, int64_t o_sh,
                          int64_t o_sl, float sm_scale, int k_splits, float* part_o, float* part_lse,
                          fluxb_stream_t stream);

#ifdef __cplusplus
}
#endif

#endif /* FLUXB200_H_ */
