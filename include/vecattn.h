/* vecattn.h -- C ABI of libvecattn.so: the VecAttention prefill path on NVIDIA B200 (sm_100a).
 *
 * Every entry point takes plain pointers and sizes, launches its kernels on the stream it is
 * given, allocates no device memory, performs no host synchronisation and returns an int
 * status (0 = ok, negative = error, see va_status_string).  All tensor pointers are device
 * pointers.  Citations name files of the reference project (anminliu/VecAttention) whose
 * interface each entry point stands in for.
 *
 * Tensor layout: 4-d tensors are (batch, heads, sequence, head_dim) with head_dim = 128, the
 * innermost stride 1 and the other three strides given in elements, so both (B,H,S,D) and
 * transposed (B,S,H,D) storage can be passed without a copy.  Rows must be 16-byte aligned.
 */
#ifndef VECATTN_H_
#define VECATTN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* va_stream_t; /* a cudaStream_t */

enum {
  VA_OK = 0,
  VA_ERR_NULL = -1,      /* a required pointer is NULL */
  VA_ERR_DTYPE = -2,     /* dtype is neither VA_BF16 nor VA_FP16 */
  VA_ERR_SHAPE = -3,     /* unsupported or inconsistent sizes */
  VA_ERR_ALIGN = -4,     /* pointer or stride not 16-byte aligned */
  VA_ERR_CAPACITY = -5,  /* index capacity or workspace too small */
  VA_ERR_CUDA = -6,      /* a CUDA call failed (launch error) */
  VA_ERR_PARAM = -7,     /* parameter combination the reference also rejects */
  VA_ERR_STATIC_SCRATCH = -8 /* va_prefill_static: the problem needs more than VA_STATIC_SCRATCH_BYTES */
};

enum { VA_BF16 = 0, VA_FP16 = 1 };

/* bit set in a device status word by the selection kernel when a row kept more keys than
 * the index capacity (indices beyond the capacity are dropped, the count stays exact) */
enum { VA_STATUS_OVERFLOW = 1,
       /* a kernel gave up waiting on one of its internal barriers (a bug, never expected): its output is invalid */
       VA_STATUS_TIMEOUT = 2 };

typedef struct {
  const void* ptr;
  int64_t stride_b, stride_h, stride_s; /* elements */
} va_tensor4;

typedef struct {
  void* ptr;
  int64_t stride_b, stride_h, stride_s;
} va_tensor4_out;

/* ---- mean pooling of Q -------------------------------------------------------------------
 * Replaces average_vector(q, block_size, use_triton=True), spattn/src/utils.py:340-351 and the
 * Triton kernel bnhd_pool_kernel, spattn/src/utils.py:8-83.  out[b,h,t,:] = mean over the rows
 * of query tile t (a ragged last tile divides by its own row count), summed in fp32 as a
 * balanced binary tree and rounded to the input dtype.  out is (B,H,ceil(S/pq),D) contiguous. */
typedef struct {
  int32_t dtype, batch, heads, seq_len, head_dim, pq;
  va_tensor4 q;
  void* out;
} va_pool_args;
int va_pool_q(const va_pool_args* args, va_stream_t stream);

/* ---- important-vector (key column) selection -------------------------------------------------
 * Replaces fuse_qk_softmax_minp_wo_causal(avg_q_chunk, k, avg_q_chunk_offset, gap, causal,
 * q_pooling_size, k_local_size, wo_initial, group_k_block),
 * spattn/src/kernels/vecattention_kernels.py:59-181, and its two Triton kernels (:206-345).
 *   avg_q      (B,H,nq,D) contiguous pooled queries of one chunk (unscaled; scaled by 1/sqrt(D)
 *              in fp32 and re-rounded inside, as the reference kernel does, :244-245)
 *   k          (B,Hkv,Sk,D), H % Hkv == 0 (the reference requires Hkv == H, :92; Hkv < H behaves
 *              as the reference does on repeat_kv-expanded keys)
 *   tile_offset index of the chunk's first query tile in the whole sequence (:233)
 *   gap / gaps  -ln(threshold): one float, or if gaps != NULL a device array read as
 *              gaps[b * gaps_stride_b + h] (the reference reads gaps[b*H + h], :301-302)
 *   compat_bsq  the reference's Triton program height (64 for every shipped causal config).
 *              Causal only: the first pooled row of every compat_bsq rows of the chunk loses the
 *              key blocks that start inside the tile before its diagonal tile, except the first
 *              (truncating division at :260).  0 = strict rule (all keys before the diagonal tile).
 *   col_count  (B,H,nq) int32 out; col_idx (B,H,nq,capacity) int32 out, every row ascending.
 *              capacity >= Sk can never overflow.  status (optional) receives VA_STATUS_* bits.
 *   workspace  scratch of va_select_workspace_bytes() bytes, 16-byte aligned: one keep bit per
 *              (pooled row, key), written by the estimate kernel and read by the kernel that forms
 *              the index lists (about Sk / 8 bytes per pooled row; the reference's wrapper allocates
 *              a zero-filled (B,H,nq,Sk) int32 buffer and a padded copy of K instead,
 *              vecattention_kernels.py:104-136).
 * Unlike the reference no buffer is zero-filled: entries of col_idx past col_count are not written. */
typedef struct {
  int32_t dtype, batch, heads, kv_heads, nq, sk, head_dim;
  int32_t pq, bk, group_k_block;
  int32_t causal, wo_initial, compat_bsq, tile_offset;
  const void* avg_q;
  va_tensor4 k;
  float gap;
  const float* gaps;
  int64_t gaps_stride_b;
  int32_t* col_count;
  int32_t* col_idx;
  int64_t capacity;
  int32_t* status;
  int32_t chunk_tiles; /* > 0: avg_q spans several prefill chunks of chunk_tiles query tiles each and the
                          compat_bsq rule restarts at every chunk boundary; 0: avg_q is one chunk */
  void* workspace;
  size_t workspace_bytes;
} va_select_args;
int va_select(const va_select_args* args, va_stream_t stream);
/* Bytes of scratch va_select needs for these sizes (batch, heads, kv_heads, nq, sk are read). */
int va_select_workspace_bytes(const va_select_args* args, size_t* bytes);

/* ---- vector-sparse flash attention --------------------------------------------------------------
 * Replaces vllm_flash_attn.sparse_attn_func(q, k, v, q_pooling_size, block_count, block_offset,
 * column_count, column_index, return_softmax_lse=False, causal=...), called at
 * spattn/src/VecAttention.py:110-121 (package vllm-flash-attn 2.7.2.post1, a fork whose source is
 * not in the reference tree).  For query tile t (pq rows): out = softmax(q K_t^T * scale) V_t over
 * K_t = 64-key blocks starting at blk_idx[b,h,t,:blk_count] plus keys col_idx[b,h,t,:col_count]
 * (the two sets must be disjoint).  causal: key <= q_offset + row, applied per element.
 *   q, out     (B,H,Sq,D) rows q_offset .. q_offset+Sq-1 of the sequence;  k, v (B,Hkv,Sk,D)
 *   blk_count  (B,H,nq) int32, blk_idx (B,H,nq,blk_stride) int32 (may be NULL when no blocks)
 *   col_count  (B,H,nq) int32, col_idx (B,H,nq,col_stride) int32
 *   softmax_scale 0 selects 1/sqrt(D).  A tile with no key at all writes zeros.
 *   lse        optional (B,H,Sq) float32 contiguous: natural-log sum of exp(score * scale) over the
 *              row's visible keys (the reference API's return_softmax_lse); -inf for a row without keys.
 *   Indices must satisfy 0 <= idx < Sk.
 *
 * Vision-slice composition in one launch (vision_mode = 1; pq 64, causal, Sq == Sk, q_offset 0).
 * Replaces the three attention calls and the concatenation of the "vecattention" branch of
 * customize_prefill_attention, spattn/src/models/utils.py:97-128: rows [0, vision_begin) get full causal
 * attention, rows [vision_begin, vision_end) the sparse attention of their query tile, rows
 * [vision_end, Sq) full causal attention over all keys.  The tables then describe the query tiles of
 * rows [0, vision_end) only (nq = ceil(vision_end / 64) entries per head, as the selection over those rows
 * produced them); the dense parts need no tables.  0 <= vision_begin <= vision_end <= Sq. */
typedef struct {
  int32_t dtype, batch, heads, kv_heads, sq, sk, head_dim, pq;
  int32_t causal, q_offset;
  va_tensor4 q, k, v;
  va_tensor4_out out;
  const int32_t* blk_count;
  const int32_t* blk_idx;
  int64_t blk_stride;
  const int32_t* col_count;
  const int32_t* col_idx;
  int64_t col_stride;
  float softmax_scale;
  int32_t* status; /* optional device word receiving VA_STATUS_* bits */
  float* lse;      /* optional, see above */
  int32_t vision_mode, vision_begin, vision_end; /* see above; all zero: off */
} va_attn_args;
int va_sparse_attn(const va_attn_args* args, va_stream_t stream);
/* Scratch va_sparse_attn needs besides its outputs: none (bytes = 0); the reference call site makes
 * three transposed copies of q, k and v first (spattn/src/VecAttention.py:110-113). */
int va_sparse_attn_workspace_bytes(const va_attn_args* args, size_t* bytes);

/* ---- dense 64-key block tables -----------------------------------------------------------------
 * Replaces the table construction in VecAttention_prefill, spattn/src/VecAttention.py:62-92:
 * causal -> sink blocks + diagonal blocks per tile, non-causal -> none.
 * blk_count (B,H,nq), blk_idx (B,H,nq,max(1, 2*pq/64)) int32 contiguous. */
int va_block_tables(int32_t batch, int32_t heads, int32_t seq_len, int32_t pq, int32_t causal,
                    int32_t* blk_count, int32_t* blk_idx, va_stream_t stream);

/* ---- the whole operator -----------------------------------------------------------------------
 * Replaces VecAttention_prefill(query_states, key_states, value_states, threshold,
 * q_pooling_size, k_local_size, group_k_block, causal, chunk_size),
 * spattn/src/VecAttention.py:10-123: pooling, selection and sparse attention for every chunk,
 * enqueued on one stream with no host synchronisation.  workspace must hold
 * va_prefill_workspace_bytes() bytes and be 256-byte aligned.
 *
 * Workspace size and chunk_size.  The reference processes chunk_size query rows at a time, which
 * bounds its index buffer (spattn/src/VecAttention.py:94-108).  Here the caller chooses through
 * single_pass_budget: when the selected-column lists of the whole sequence
 * (4 * batch * heads * ceil(Sq/q_pooling_size) * Sk bytes) fit in that many bytes, every stage runs
 * once for all chunks (same results: chunk_size then only positions the reference's causal
 * chunk-boundary effect); otherwise the chunk loop of the reference is used and chunk_size bounds
 * the workspace exactly as it does there.  single_pass_budget = 0 selects
 * VA_SINGLE_PASS_INDEX_BYTES_DEFAULT; 1 forces the chunk loop.  va_prefill_workspace_bytes and
 * va_prefill must be given the same value.  col_count_out (optional, (B,H,ceil(Sq/pq)) int32)
 * receives the per-tile selection counts. */
#define VA_SINGLE_PASS_INDEX_BYTES_DEFAULT (4ull << 30)
typedef struct {
  int32_t dtype, batch, heads, kv_heads, sq, sk, head_dim;
  int32_t pq, bk, group_k_block, causal, chunk_size, compat_bsq;
  va_tensor4 q, k, v;
  va_tensor4_out out;
  float gap;
  const float* gaps;
  int64_t gaps_stride_b;
  void* workspace;
  size_t workspace_bytes;
  int32_t* col_count_out;
  int32_t* status;
  size_t single_pass_budget; /* see above; 0 = VA_SINGLE_PASS_INDEX_BYTES_DEFAULT */
} va_prefill_args;
int va_prefill_workspace_bytes(const va_prefill_args* args, size_t* bytes);
int va_prefill(const va_prefill_args* args, va_stream_t stream);

/* ---- the whole operator, for callers that must not allocate --------------------------------
 * No counterpart in the reference (there every call allocates its temporaries through PyTorch).
 *
 * Who needs it: code that may not call cudaMalloc or a caching allocator at the point where the
 * operator runs -- an inference server whose memory is handed out once at start-up and is owned
 * by another component, a plugin running inside someone else's stream-ordered region, a host
 * thread that is not allowed to touch the allocator's lock.  Such a caller still owns q, k, v and
 * out; what it cannot provide is the scratch va_prefill wants in `workspace`.
 *
 * Same arguments and results as va_prefill; `workspace`, `workspace_bytes` and `single_pass_budget`
 * are ignored.  The scratch is a fixed array of VA_STATIC_SCRATCH_BYTES bytes that is part of the
 * library image: every GPU that loads the library carries it until the process exits.  The whole
 * sequence is processed in one pass if its scratch fits the array, else chunk by chunk as the
 * reference does; only a problem whose per-chunk scratch still exceeds the array is refused with
 * VA_ERR_STATIC_SCRATCH, and then nothing is launched.  (So a problem may be accepted although
 * va_prefill_workspace_bytes reports more than VA_STATIC_SCRATCH_BYTES for it.)  The per-chunk
 * scratch is dominated by 4 * batch * heads * ceil(chunk_size / q_pooling_size) * Sk bytes of index
 * lists, so a smaller chunk_size makes a larger problem fit.  va_prefill_static_fits answers the
 * question on the host without launching anything (1 = accepted, 0 = refused, negative = the
 * arguments are invalid).
 *
 * The function calls no cudaMalloc/cudaFree and no allocating library routine.  Its first call on
 * a device makes the CUDA runtime load the library's device code there, and every call looks up
 * the array's device address (cudaGetSymbolAddress, with the caller's device current: a host-side
 * table lookup once the code is loaded); make the first call on a device before any stream capture
 * begins.
 *
 * All calls on a device share the one array and it keeps whatever the previous call left.  The
 * kernels never read scratch they have not written in the same call, so nothing needs clearing;
 * but two calls whose kernels overlap on the GPU (different streams, no ordering between them)
 * race on it and corrupt each other's results.  Order such calls, or use va_prefill. */
#define VA_STATIC_SCRATCH_BYTES (32u << 20)
int va_prefill_static(const va_prefill_args* args, va_stream_t stream);
int va_prefill_static_fits(const va_prefill_args* args);

/* ---- self-test of the bounded waits -----------------------------------------------------------
 * No counterpart in the reference.  Every wait inside the kernels (on an mbarrier that a copy, an
 * MMA or another warp completes) gives up after a fixed number of polls, reports
 * VA_STATUS_TIMEOUT through the status word and lets the CTA unwind (free its tensor memory,
 * return), so a protocol bug ends a kernel instead of hanging the GPU.  This entry point runs that
 * path on purpose: a one-CTA kernel allocates tensor memory, then one of its threads waits with
 * the kernels' own wait routine, limited to `polls` polls (a few microseconds each), on a barrier
 * that nothing ever completes.  The kernel returns normally; *status (a device int32, required)
 * has VA_STATUS_TIMEOUT OR-ed in.  polls must be in [1, 4096]. */
int va_selftest_wait_timeout(int32_t* status, int32_t polls, va_stream_t stream);

/* ---- RMSNorm + rotary embedding of Q and K, feeding the operator without a layout change -----------
 * Replaces, for a video-DiT attention layer (eval/DiTEvalKit/models/wan/attention.py:108-136), the RMSNorm
 * of the projected Q and K over the hidden dimension (Triton kernel eval/DiTEvalKit/kernels/triton/
 * rmsnorm.py:8-47), the three transposed copies to (B,H,S,D) (:123-128) and the in-place rotary embedding on
 * interleaved element pairs (apply_qk_rope_inplace_cossin_complex, eval/DiTEvalKit/kernels/csrc/ops.h and
 * include/rope/rope_enc_complex.cuh) by one pass over Q and K: the outputs keep the (B,S,H*D) storage, which
 * va_prefill and the other entry points read in place as (B,H,S,D) with strides (H*D*S, D, H*D).
 *   q, k        (B, S, heads*128) / (B, S, kv_heads*128), unit inner stride, row strides in elements
 *   q_out, k_out  same shapes; may be the inputs themselves (in place)
 *   q_weight, k_weight  RMSNorm weights of the hidden size in the tensors' dtype; NULL skips the norm
 *   eps         added to the mean square
 *   cos, sin    (S - rope_skip, 64) float32 tables, or NULL for no rotation; token s >= rope_skip uses row
 *               s - rope_skip, earlier tokens are not rotated
 * y = round16(x * rsqrt(mean(x^2) + eps) * w) in fp32, then per pair (y0, y1) -> round16(y0 cos - y1 sin),
 * round16(y1 cos + y0 sin) in double precision, the reference kernels' arithmetic. */
typedef struct {
  int32_t dtype, batch, seq_len, heads, kv_heads, rope_skip;
  const void* q;
  const void* k;
  int64_t q_row_stride, k_row_stride;
  void* q_out;
  void* k_out;
  int64_t q_out_row_stride, k_out_row_stride;
  const void* q_weight;
  const void* k_weight;
  float eps;
  const float* cos;
  const float* sin;
} va_norm_rope_args;
int va_qk_norm_rope(const va_norm_rope_args* args, va_stream_t stream);

/* The same preparation where the tensors are (B,H,L,128) already and the norm is per head (HunyuanVideo,
 * eval/DiTEvalKit/models/hyvideo/attention.py:187-213): replaces rms_norm_forward on the rows of 128 elements
 * (eval/DiTEvalKit/kernels/csrc/ops.h:52-74, include/norm/narrow_rms_norm.cuh) and
 * apply_qk_rope_inplace_cossin_txtlast (csrc/ops.h:146, include/rope/rope_enc_txtlast.cuh) by one pass.
 *   q, k          (B,H,L,128) / (B,Hkv,L,128), any 16-byte aligned strides; q_out, k_out may be the inputs
 *   q_weight, k_weight  128 elements of the tensors' dtype; NULL skips the norm
 *   cos, sin      (rope_len, 128) float32, per element; NULL for no rotation.  Tokens l < rope_len are rotated
 *                 (the text tokens come last): out[i] = y[i] cos[l,i] + (i even ? -y[i+1] : y[i-1]) sin[l,i], fp32.
 * y = T((x * rsqrt(sum(x^2)/128 + eps)) * w). */
typedef struct {
  int32_t dtype, batch, seq_len, heads, kv_heads, rope_len;
  va_tensor4 q, k;
  va_tensor4_out q_out, k_out;
  const void* q_weight;
  const void* k_weight;
  float eps;
  const float* cos;
  const float* sin;
} va_head_norm_rope_args;
int va_qk_head_norm_rope(const va_head_norm_rope_args* args, va_stream_t stream);

const char* va_status_string(int code);
/* 100 * major + minor of this interface (201: va_attn_args gained the vision_* fields, va_qk_head_norm_rope added). */
int va_version(void);

#ifdef __cplusplus
}
#endif
#endif /* VECATTN_H_ */
