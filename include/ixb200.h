/*
 * ixb200 -- C ABI of the B200 (sm_100a) INT8-X weight path.
 *
 * One shared library, plain pointers and sizes, no framework types.  Every
 * pointer named "device" is a CUDA device pointer on the current device; every
 * call launches on the given stream and returns without synchronising.  All
 * functions return 0 on success and a non-zero IXB_E_* code otherwise;
 * ixb_last_error() then gives a message for the calling thread.
 *
 * The packed tensor layout is exactly the dict produced by the reference's
 * quantiser (ixrun/quantize.py:110-122): two nested bitmaps and three value
 * streams for a row-major [out_f, in_f] int8 code matrix, plus one bf16 scale.
 *
 * Each entry point names the reference interface it stands in for.
 */
#ifndef IXB200_H
#define IXB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define IXB_OK 0
#define IXB_E_ARG 1        /* bad argument (null pointer, shape, alignment) */
#define IXB_E_UNSUPPORTED 2 /* shape outside what the kernels handle */
#define IXB_E_CUDA 3       /* a CUDA runtime call failed */
#define IXB_E_SCRATCH 4    /* scratch/workspace too small */

typedef void *ixb_stream_t; /* cudaStream_t */

/* Device-resident packed tensor (reference: the GPU buffers StreamingLinear
 * registers, ixrun/engine.py:58-66).  Stream base pointers must be 16-byte
 * aligned; lengths are exact (no padding is assumed or read). */
typedef struct ixb_packed {
    const void *b1;       /* int32 words, bit e      = element e is level 1 */
    int64_t b1_words;
    const void *b2;       /* int32 words, bit r      = r-th non-L1 element is level 2 */
    int64_t b2_words;
    const void *l1;       /* int32 words, 3-bit fields, code+3   */
    int64_t l1_words;
    const void *l2;       /* int32 words, 5-bit fields, code+15  */
    int64_t l2_words;
    const void *l3;       /* bytes, code+127 */
    int64_t l3_bytes;
    const void *scale;    /* one bf16 */
    int64_t out_f;
    int64_t in_f;
} ixb_packed;

/* library / device facts */
int ixb_version(void);
const char *ixb_last_error(void);
/* number of kernels this library has launched in this process (all threads) */
int64_t ixb_launch_count(void);

/*
 * Rank prefix tables.  q1[u], q2[u] = number of level-1 / level-2 elements
 * strictly before flat position u*gran, u in [0, n_units).
 *   gran = 1024  replaces precompute_block_offsets (ixrun/triton_kernels.py:180-220)
 *   gran = in_f  replaces compute_row_prefixes(packed)        (ixrun/fused.py:60-65)
 *   gran = chunk replaces compute_row_prefixes(packed, chunk) (ixrun/fused.py:67-78)
 * `ws` is device workspace of at least ixb_prefix_workspace_bytes(N) bytes.
 */
size_t ixb_prefix_workspace_bytes(int64_t n_elements);
int ixb_prefix_tables(const ixb_packed *w, int64_t gran, int64_t n_units,
                      int32_t *q1_device, int32_t *q2_device,
                      void *ws_device, size_t ws_bytes, ixb_stream_t stream);

/*
 * Packed streams -> dense matrix.  blk_q1/blk_q2 are the gran=1024 tables.
 *   out_kind 0: int8 codes      (the integers ixrun/quantize.py:65-72 produced)
 *   out_kind 1: bf16 weights    (replaces _ix_decode_kernel + launcher,
 *                                ixrun/triton_kernels.py:68-177, :224-259, and
 *                                StreamingLinear._decode, ixrun/engine.py:109-133)
 */
int ixb_decode(const ixb_packed *w, const int32_t *blk_q1, const int32_t *blk_q2,
               void *out_device, int out_kind, ixb_stream_t stream);

/*
 * Fused decode + matrix product for m_rows activations (1 <= m_rows <= 8):
 *   y[m][n] = sum_k float(x[m][k]) * float(bf16(code[n][k] * scale))  (+ bias[n])
 * accumulated in fp32; decoded weights never reach device memory.
 * Replaces fused_gemv / _ix_gemv_kernel / _ix_gemv_split_kernel
 * (ixrun/fused.py:84-179, :209-294, :297-347) including the caller-side
 * zeroing and bf16 cast of the split-K path (ixrun/engine.py:145-159).
 *   x       bf16 [m_rows][in_f], row stride in_f
 *   bias    bf16 [out_f] or NULL; added after the sum is rounded to the
 *           output type when y is bf16 (ixrun/engine.py:166-168)
 *   y       bf16 or fp32 [m_rows][out_f]
 *   scratch device memory of ixb_gemv_scratch_bytes() bytes whose first 256
 *           bytes were zero before the first call; the library leaves them
 *           zero again.  One call at a time per scratch buffer.
 * Requires in_f % 32 == 0.
 */
size_t ixb_gemv_scratch_bytes(int64_t out_f, int64_t in_f, int64_t m_rows);
int ixb_gemv(const ixb_packed *w, const int32_t *blk_q1, const int32_t *blk_q2,
             const void *x_device, int64_t m_rows, const void *bias_device,
             void *y_device, int y_is_f32,
             void *scratch_device, size_t scratch_bytes, ixb_stream_t stream);

/*
 * Device-side quantiser and packer for deploy time.  Replaces int8x_quantize
 * (ixrun/quantize.py:41-122: per-tensor scale = max|W|/127 evaluated in bf16,
 * codes = clamp(round_half_even(W/scale), +-127), level split, LSB-first bit
 * packing of ixrun/bitpack.py:13-61); the streams come out bit for bit as the
 * CPU quantiser writes them.  Three steps, because the stream sizes are only
 * known after counting:
 *   1. ixb_quantize_codes (from a bf16 weight) or ixb_count_codes (from int8
 *      codes, e.g. a tensor-parallel slice that keeps the unsharded scale):
 *      writes codes / scale, the B1 bitmap and the gran=1024 rank tables and
 *      returns counts_host[3] = {#L1, #L2, #L3}.  Synchronises the stream.
 *   2. the caller allocates b2 (ceil((n2+n3)/32) words), l1 (ceil(3 n1/32)),
 *      l2 (ceil(5 n2/32)), l3 (n3 bytes)
 *   3. ixb_pack_codes fills them (they are zeroed by the call).
 * `ws`: ixb_pack_workspace_bytes(N) bytes of device workspace.
 */
size_t ixb_pack_workspace_bytes(int64_t n_elements);
int ixb_quantize_codes(const void *w_bf16_device, int64_t n_elements, void *scale_bf16_device,
                       int8_t *codes_device, void *b1_device, int32_t *blk_q1_device, int32_t *blk_q2_device,
                       int64_t *counts_host, void *ws_device, size_t ws_bytes, ixb_stream_t stream);
int ixb_count_codes(const int8_t *codes_device, int64_t n_elements, void *b1_device,
                    int32_t *blk_q1_device, int32_t *blk_q2_device, int64_t *counts_host,
                    void *ws_device, size_t ws_bytes, ixb_stream_t stream);
int ixb_pack_codes(const int8_t *codes_device, const ixb_packed *out, const int32_t *blk_q1_device,
                   const int32_t *blk_q2_device, ixb_stream_t stream);

/* TPAB tile format (ixrun/tpab.py:37-203; GEMV ixrun/tpab_gemv.py:28-143): tiles of tile_r x 64, per tile a bit
 * width 2..6, an fp16 scale and its element offset inside the group of tiles of that width; element L of tile t is
 * the field at bit gbase_bit[b] + (goff[t] + L) * b of `body` (uint32 words, two readable words behind the last),
 * weight bf16(f32(field - (2^(b-1) - 1)) * f32(scale)); outliers replace their weights.  The packed dict of
 * ixrun.tpab.encode_tpab is consumed as it is (bodies concatenated as ixrun.tpab.stage_gpu does).
 * ixb_tpab_decode: -> bf16 [out_f, in_f] (outliers (tile, element, fp16 value) scattered over their weights).
 * ixb_tpab_gemv: batch-1 y = W x, fp32 accumulation, one rounding, bias after it; the outliers as per-row lists
 *   (ol_offs [out_f + 1], columns, fp16 values: what ixrun.tpab_gemv.prepare_gemv_stage builds).  Reproducible (no
 *   floating-point atomics).  scratch: ixb_tpab_gemv_scratch_bytes, any contents. */
typedef struct ixb_tpab {
    const void *body;
    const void *bits;
    const void *scales;
    const void *goff;
    int32_t gbase_bit[8];
    int64_t out_f;
    int64_t in_f;
    int64_t tile_r;
} ixb_tpab;
int ixb_tpab_decode(const ixb_tpab *t, const int32_t *ol_t_device, const int32_t *ol_l_device, const void *ol_val_fp16_device,
                    int64_t n_outliers, void *out_bf16_device, ixb_stream_t stream);
size_t ixb_tpab_gemv_scratch_bytes(int64_t out_f, int64_t in_f, int64_t tile_r);
int ixb_tpab_gemv(const ixb_tpab *t, const void *x_device, const int32_t *ol_offs_device, const int32_t *ol_k_device,
                  const void *ol_v_fp16_device, const void *bias_device, void *y_device, int y_is_f32, void *scratch_device,
                  size_t scratch_bytes, ixb_stream_t stream);

/* Sibling format with one fp16 scale per `group` consecutive elements (ixgs/quantize.py:35-112; decode
 * ixgs/kernels.py:31-102): its five streams are read by ixb_decode unchanged (out_kind 0: int8 codes; the per-tensor
 * scale of the ixb_packed is not used then), and this call turns codes + group scales into the bf16 weights
 * bf16(f32(code) * f32(scale[e / group])). */
int ixb_group_scale(const int8_t *codes_device, const void *group_scales_fp16_device, int64_t n, int64_t group,
                    void *out_bf16_device, ixb_stream_t stream);

/*
 * Resident re-layout "P6".  It has no counterpart in the reference, whose
 * kernels read the (3,5,8) streams directly; it plays the role of the
 * reference's deploy-time derived buffers (ixrun/engine.py:68-97).  The streams
 * stay the interchange / cache-file format; at deploy time the int8 codes they
 * decode to are re-laid out on the GPU, losslessly, so that nothing is
 * addressed by rank:
 *   plane    a 6-bit field per element, blocks of 16 rows x 64 columns (ragged
 *            edges padded), 768 contiguous bytes per block, block b =
 *            row_tile * ceil(in_f / 64) + column_block.  The field is bits 7..2
 *            of the low byte of the bf16 number 1 + code / 32 (codes -16 .. 31),
 *            so the GEMV needs a shift, a mask and ONE fused multiply-add per
 *            pair of weights to obtain bf16(code * scale) -- the reference's
 *            dequantised weight (ixrun/quantize.py:182, ixrun/fused.py:169-170),
 *            rounded once
 *   esc      every other code as a uint32 entry: bf16(code * scale) in the high
 *            half, row in tile, block index mod 64 and column in block below;
 *            blk_off: int32 first entry of every block
 * about 6 + 32 * P(code outside -16 .. 31) bits per weight.  Buffer sizes
 * (B = ixb_p6_blocks): plane (B + 5) * 768 bytes, blk_off (B + 1) * 4 bytes,
 * esc (n_esc + 64) * 4 bytes; plane and esc 16-byte aligned.
 * ixb_p6_build: int8 codes [out_f, in_f] + the bf16 scale -> layout (n_esc =
 *   number of codes outside -16 .. 31; entries beyond n_esc are not written;
 *   ws: (B + 1) * 4 bytes).
 * ixb_p6_decode: layout -> int8 codes / bf16 weights (out_kind as ixb_decode).
 * ixb_p6_gemv: same result definition, bias and argument meaning as ixb_gemv,
 *   1..8 activation rows in one kernel: plane on the tensor cores (mma.sync,
 *   exact bf16 x bf16 products, fp32 accumulation), outliers on the CUDA cores;
 *   partial sums are added in a fixed order (reproducible, no floating-point
 *   atomics).  Scratch: ixb_p6_gemv_scratch_bytes bytes, 16-byte aligned, zero
 *   before the first call; every launch leaves it all zero again, so one buffer
 *   (sized for the largest need) may serve layers of any shape one after the
 *   other, but not two launches that can overlap on the GPU.
 */
typedef struct ixb_p6 {
    const void *plane;
    const void *blk_off;
    const void *esc;
    int64_t n_esc;
    const void *scale;    /* scale_stride 0: one bf16; 1: one bf16 per 16-row tile */
    int64_t out_f;
    int64_t in_f;
    int64_t scale_stride; /* 1: a tensor fused row-wise from several (q|k|v, gate|up), every part a
                             whole number of row tiles with its own per-tensor scale */
} ixb_p6;
int64_t ixb_p6_blocks(int64_t out_f, int64_t in_f);
int ixb_p6_build(const int8_t *codes_device, const void *scale_device, int64_t scale_stride, int64_t out_f, int64_t in_f,
                 void *plane_device,
                 int32_t *blk_off_device, void *esc_device, int64_t n_esc, void *ws_device, size_t ws_bytes,
                 ixb_stream_t stream);
int ixb_p6_decode(const ixb_p6 *t, void *out_device, int out_kind, ixb_stream_t stream);
size_t ixb_p6_gemv_scratch_bytes(int64_t out_f, int64_t in_f, int64_t m_rows);
int ixb_p6_gemv(const ixb_p6 *t, const void *x_device, int64_t m_rows, const void *bias_device,
                void *y_device, int y_is_f32, void *scratch_device, size_t scratch_bytes, ixb_stream_t stream);
/* Small-M GEMM on the resident layout: 1..64 activation rows, y[m][n] as ixb_p6_gemv defines it, in one pass over
 * the tensor's bytes on the tcgen05 tensor cores (accumulator in TMEM); the bf16 weights exist only in shared memory.
 * Takes the place of the reference's decode + dense matmul for 9..64 rows (ixrun/engine.py:171-173; precedent for a
 * fused kernel: ixrun/tpab_gemm.py:34-94).  in_f must be a multiple of 64.  scratch: ixb_p6_gemm_scratch_bytes bytes,
 * 256-byte aligned, any contents (split-K partial sums, added in a fixed order: reproducible). */
size_t ixb_p6_gemm_scratch_bytes(int64_t out_f, int64_t in_f, int64_t m_rows);
int ixb_p6_gemm(const ixb_p6 *t, const void *x_device, int64_t m_rows, const void *bias_device, void *y_device,
                int y_is_f32, void *scratch_device, size_t scratch_bytes, ixb_stream_t stream);
/*
 * Programmatic dependent launch for ixb_p6_gemv (process-wide switch, off by
 * default; returns the previous setting).  No counterpart in the reference,
 * whose per-layer kernels run strictly one after the other.  When on, an
 * ixb_p6_gemv launch may start while the kernel ahead of it in the stream is
 * still finishing: it fetches its first weight blocks and outlier entries, then
 * waits for that kernel to complete before it reads x or writes y or the
 * scratch.  Turn it on only once the layouts it will read are complete (after
 * deployment and a synchronise): a layout still being built by the kernel just
 * ahead in the stream would be read too early.
 */
int ixb_set_pdl(int on);

/*
 * One-shot all-reduce (sum, fp32) over peer memory for the partial outputs of
 * row-parallel packed linears.  No counterpart in the reference, which is
 * single-GPU; it stands where a tensor-parallel ixrun would call its
 * collective after o_proj / down_proj (ixrun/engine.py:135-168 per shard).
 * Every rank owns one buffer of ixb_allreduce_bytes(world, n_max) bytes that
 * all ranks can address (peer pointers, e.g. torch symmetric memory), zeroed
 * and followed by a barrier before the first call.  peer_buffers: host array
 * of `world` device pointers, entry r = rank r's buffer as seen from this
 * rank.  Every rank must make the same sequence of calls with the same n.
 *   x: this rank's n fp32 partial sums (n a multiple of 4, n <= n_max)
 *   y: n sums over the ranks, added in rank order (the same bits on every
 *      rank), + bias (bf16, after rounding for bf16 output), bf16 or fp32
 * One kernel: peer stores of {value, call number} words, a bounded wait for
 * the call number on the local copies (on a time-out the error word behind the
 * epochs becomes non-zero and the result is wrong; the kernel never hangs),
 * local sum.  Graph-capturable;
 * follows ixb_set_pdl.  world in {1, 2, 4, 8}.
 */
size_t ixb_allreduce_bytes(int world, int64_t n_max);
int ixb_allreduce(const void *x_device_f32, int64_t n, void *const *peer_buffers, int rank, int world, int64_t n_max,
                  const void *bias_device, void *y_device, int y_is_f32, ixb_stream_t stream);
/*
 * The same exchange with the senders' half inside the GEMV (no counterpart in
 * the reference; it stands where a tensor-parallel ixrun would run a
 * row-parallel o_proj / down_proj shard followed by its collective,
 * ixrun/engine.py:135-168 per shard):
 * ixb_p6_gemv_push: ixb_p6_gemv of a row-parallel shard whose epilogue stores
 *   every finished output (m_rows * out_f fp32 partial sums, no bias) as a
 *   marked word into this rank's slot of EVERY rank's all-reduce buffer -- plain
 *   peer stores, no local y, no second kernel for the sending side.
 * ixb_allreduce_finish: waits (bounded) for every rank's words of this call in
 *   this rank's own buffer, adds them in rank order, adds the bias, writes y;
 *   n = m_rows * out_f of the push before it.  Every rank calls push, then
 *   finish, in the same order; calls of ixb_allreduce may be mixed in on the
 *   same buffers.
 * ixb_p6_gemv_allreduce: both halves in ONE kernel.  The GEMV pushes as
 *   ixb_p6_gemv_push does; every warp that is done with its blocks then takes a
 *   share of the outputs, waits (bounded) for all ranks' words of this call,
 *   adds them in rank order (+ bias after the bf16 rounding, as ixb_gemv) and
 *   writes y: the sum over the ranks of x @ W.T.  The transfer over NVLink
 *   overlaps the remaining tiles' arithmetic; no second launch.  Needs an even
 *   out_f.  Calls of all three kinds may be mixed on the same buffers.
 * ixb_allreduce_spin_limit: polls after which a wait of these kernels gives up
 *   (0 restores the default of 2^22); returns the previous value.  For tests and
 *   diagnosis: after a wait gave up the error word behind the counters stays set
 *   and later waits give up after 64 polls, until the buffers are zeroed again
 *   (with a barrier between the ranks, as before the first call).
 */
int ixb_p6_gemv_push(const ixb_p6 *t, const void *x_device, int64_t m_rows, void *const *peer_buffers, int rank,
                     int world, int64_t n_max, void *scratch_device, size_t scratch_bytes, ixb_stream_t stream);
int ixb_allreduce_finish(void *const *peer_buffers, int rank, int world, int64_t n, int64_t n_max,
                         const void *bias_device, void *y_device, int y_is_f32, ixb_stream_t stream);
int ixb_p6_gemv_allreduce(const ixb_p6 *t, const void *x_device, int64_t m_rows, void *const *peer_buffers, int rank,
                          int world, int64_t n_max, const void *bias_device, void *y_device, int y_is_f32,
                          void *scratch_device, size_t scratch_bytes, ixb_stream_t stream);
uint32_t ixb_allreduce_spin_limit(uint32_t polls);

/*
 * Per-token glue of a decode step around the packed linears (batch 1, up to a
 * few rows).  The reference leaves this work to HuggingFace eager code and to
 * fla's Triton kernels (ixrun/fla_patch.py:23-72); here each is one launch that
 * can sit in a captured CUDA graph (positions are read from device memory) and
 * takes part in programmatic dependent launch (ixb_set_pdl).  bf16 in and out,
 * fp32 arithmetic, rounded to bf16 where the eager path holds a bf16 tensor.
 * ixb_add_rmsnorm: h[rows, hidden] += delta (may be NULL); xn = bf16(h * rsqrt(
 *   mean(h^2) + eps)) * w -- the residual add and the norm in front of the next
 *   linears (HF LlamaRMSNorm arithmetic).
 * ixb_swiglu: y [rows][cols] = silu(g) * u; g and u may be column slices of a
 *   wider matrix (row pitch in_stride elements).
 * ixb_rope_kv: optional per-head RMSNorm of q and k (weights [head_dim] or
 *   NULL), rotate-half rotary embedding of the first rot_dim dimensions with
 *   the caller's fp32 tables cos / sin [max_seq][rot_dim / 2]; q [rows] (row
 *   stride q_stride elements, heads contiguous) rotated in place, k and v
 *   [rows][hkv][head_dim] (row pitch kv_stride) written into the caches
 *   [max_seq][hkv][head_dim] at
 *   positions pos[0] + row.  head_dim 64, 128 or 256.
 * ixb_attn_decode: one query per head (q [hq][head_dim]) over positions
 *   0 .. pos[0] of the static caches, grouped-query (hq a multiple of hkv),
 *   softmax(scale * q.k) v, the context cut into `splits` ranges that run on
 *   separate CTAs; optional output gate: out *= sigmoid(gate[head * gate_stride
 *   + d]).  scratch: batch * ixb_attn_scratch_bytes.
 *   Batched decode (ixrun/batching.py:88-234 drives B sequences per step): batch_stride > 0 in ixb_rope_kv makes
 *   row r the newest token of sequence r (position pos[r], cache r starts batch_stride elements after cache r - 1);
 *   ixb_attn_decode takes `batch` queries (row pitch q_stride, gate row pitch gate_row_stride), one per sequence.
 * ixb_conv_update: causal depth-wise conv1d step: y_c = silu(sum_j w[c][j] *
 *   input_{t-k+1+j} + bias_c) over the last k inputs of every channel; state
 *   [channels][k - 1] (oldest first) takes x in.
 * ixb_gdn_step: gated delta rule, one recurrent step (the published Gated
 *   DeltaNet recurrence that fla's fused_recurrent_gated_delta_rule computes):
 *   qkv = [q (hk * 128) | k (hk * 128) | v (hv * 128)], q and k L2-normalised
 *   per head, q scaled by 128^-0.5; per value head g = exp(-exp(A_log) *
 *   softplus(a + dt_bias)), beta = sigmoid(b); S <- g S; delta = (v - S^T k)
 *   beta; S <- S + k delta^T; o = S^T q; out = rmsnorm(o) * norm_w * silu(z).
 *   state: fp32 [hv][128][128], updated in place (read once, written once).
 */
int ixb_add_rmsnorm(void *h_device, const void *delta_device, const void *w_device, float eps, void *xn_device,
                    int64_t rows, int64_t hidden, ixb_stream_t stream);
/* ixb_allreduce_finish with the residual add and the RMSNorm that follow a row-parallel linear in the same kernel:
 * h [rows][hidden] (bf16, in/out) += bf16(sum over the ranks' words of this call), xn = rmsnorm(h) * w.  rows <= 8,
 * hidden a multiple of 8 and at most 5120, rows * hidden <= n_max.  No reference counterpart (the reference is
 * single-GPU); the result equals ixb_allreduce_finish into a bf16 vector followed by ixb_add_rmsnorm.  One CTA per row
 * pulls every rank's words through one SM: fewer launches, but slower than the two calls (measured at 2 and 8 ranks). */
int ixb_allreduce_finish_add_rmsnorm(void *const *peer_buffers, int rank, int world, int64_t n_max, void *h_device,
                                     const void *w_device, float eps, void *xn_device, int64_t rows, int64_t hidden,
                                     ixb_stream_t stream);
int ixb_swiglu(const void *g_device, const void *u_device, void *y_device, int64_t rows, int64_t cols, int64_t in_stride,
               ixb_stream_t stream);
int ixb_rope_kv(void *q_device, const void *k_device, const void *v_device, const int32_t *pos_device, void *k_cache_device,
                void *v_cache_device, const void *q_norm_device, const void *k_norm_device, const float *cos_device,
                const float *sin_device, int64_t rows, int64_t hq, int64_t hkv, int64_t head_dim, int64_t rot_dim, float eps,
                int64_t q_stride, int64_t max_seq, int64_t kv_stride, int64_t batch_stride, ixb_stream_t stream);
size_t ixb_attn_scratch_bytes(int64_t hq, int64_t head_dim, int64_t splits);
int ixb_attn_decode(const void *q_device, const void *k_cache_device, const void *v_cache_device, const int32_t *pos_device,
                    const void *gate_device, int64_t gate_stride, void *out_device, void *scratch_device, size_t scratch_bytes,
                    int64_t hq, int64_t hkv, int64_t head_dim, int64_t splits, float scale, int64_t batch, int64_t q_stride,
                    int64_t batch_stride, int64_t gate_row_stride, ixb_stream_t stream);
int ixb_conv_update(const void *x_device, void *state_device, const void *w_device, const void *bias_device, void *y_device,
                    int64_t channels, int64_t k, ixb_stream_t stream);
int ixb_gdn_step(const void *qkv_device, const void *z_device, const void *a_device, const void *b_device,
                 const float *A_log_device, const float *dt_bias_device, const void *norm_w_device, float *state_device,
                 void *out_device, int64_t hk, int64_t hv, float eps, ixb_stream_t stream);
/* ixb_conv_update (kernel size 4, no bias) and ixb_gdn_step in one kernel: qkv_raw is the projection before the conv;
 * conv_state [2][channels][3] (bf16, channels = (2 hk + hv) * 128) keeps the conv's history twice: the step at position
 * pos[0] reads copy pos[0] & 1 and writes the other one, so the caller advances pos[0] by one per step. */
int ixb_gdn_conv_step(const void *qkv_raw_device, void *conv_state_device, const void *conv_w_device,
                      const int32_t *pos_device, const void *z_device, const void *a_device, const void *b_device,
                      const float *A_log_device, const float *dt_bias_device, const void *norm_w_device, float *state_device,
                      void *out_device, int64_t hk, int64_t hv, float eps, ixb_stream_t stream);

/*
 * Fused decode + small-M GEMM on the tensor cores (tcgen05, accumulators in
 * TMEM) for 1 <= m_rows <= 64; intended for 9..64 rows (batched decode, MTP
 * verify), below that ixb_gemv is the better call.  Same result definition and
 * argument meaning as ixb_gemv; products are bf16 x bf16 accumulated in fp32.
 * Replaces, for these row counts, the reference's decode-to-bf16 followed by a
 * dense matmul (ixrun/engine.py:171-173); the only fused decode+GEMM in the
 * reference is the TPAB one (ixrun/tpab_gemm.py:34-94).
 * Requires in_f % 1024 == 0.  If a tensor-core completion wait ever runs out
 * the whole output is set to NaN instead of hanging.
 */
size_t ixb_gemm_scratch_bytes(int64_t out_f, int64_t in_f, int64_t m_rows);
int ixb_gemm(const ixb_packed *w, const int32_t *blk_q1, const int32_t *blk_q2,
             const void *x_device, int64_t m_rows, const void *bias_device,
             void *y_device, int y_is_f32,
             void *scratch_device, size_t scratch_bytes, ixb_stream_t stream);

/*
 * ixb_gemv for callers that cannot hand over scratch memory.  It has no
 * counterpart in the reference.
 *
 * Some hosts may not allocate device memory at the point where they run a
 * layer: a serving process that gave the whole device to its own pool at
 * start-up, a host framework that plans every buffer ahead and rejects later
 * allocations, or a plain C caller that only owns the input and output buffers
 * it was handed.  For them this call takes the same arguments as ixb_gemv minus
 * the scratch: the partial-sum slots and the completion counter live in an
 * array of IXB_STATIC_SCRATCH_BYTES bytes that is part of the library image on
 * every device that loads it (so that much device memory stays taken until the
 * process exits).  The call performs no cudaMalloc/cudaFree and uses no
 * allocating library routine.
 *
 *  - Shapes whose scratch need (ixb_gemv_scratch_bytes) exceeds
 *    IXB_STATIC_SCRATCH_BYTES are rejected with IXB_E_SCRATCH.
 *  - The first call on each device looks up the array's device address with
 *    that device current; make that first call before starting any stream
 *    capture.
 *  - All calls on a device share the one array and each call reuses what the
 *    previous one left (the counter is re-zeroed on the stream before every
 *    launch).  Two calls whose kernels can overlap on the GPU (different
 *    streams, no ordering) race on it: serialise them, or use ixb_gemv with
 *    one scratch buffer per stream.
 */
#define IXB_STATIC_SCRATCH_BYTES (4 * 1024 * 1024)
int ixb_gemv_static(const ixb_packed *w, const int32_t *blk_q1, const int32_t *blk_q2,
                    const void *x_device, int64_t m_rows, const void *bias_device,
                    void *y_device, int y_is_f32, ixb_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* IXB200_H */
