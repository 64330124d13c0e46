// C ABI of libvecattn.so: argument validation, workspace carving and kernel launches.
// No device allocation, no host synchronisation, no C++ exception crosses this boundary.
#include "va_common.cuh"
#include "va_sm100.cuh"

namespace va {
int pool_q(const va_pool_args& a, cudaStream_t stream);
int select(const va_select_args& a, cudaStream_t stream);
size_t select_workspace_bytes(int batch, int heads, int kv_heads, int nq, int sk);
int sparse_attn(const va_attn_args& a, cudaStream_t stream);
int qk_norm_rope(const va_norm_rope_args& a, cudaStream_t stream);
int qk_head_norm_rope(const va_head_norm_rope_args& a, cudaStream_t stream);

// dense-block tables of query tiles [tile_off, tile_off + nqc) written as a contiguous (BH, nqc) slice
__global__ void block_tables_kernel(int bh, int seq_len, int pq, int causal, int tile_off, int nqc,
                                    int32_t* __restrict__ blk_count, int32_t* __restrict__ blk_idx) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= bh * nqc) return;
  const int n = pq / 64;
  const int width = causal ? 2 * n : 1;
  const int t = tile_off + i % nqc;
  const int nq = (seq_len + pq - 1) / pq;
  int32_t* row = blk_idx + (int64_t)i * width;
  if (!causal) {
    blk_count[i] = 0;
    row[0] = 0;
    return;
  }
  int cnt = 2 * n;
  if (t == 0) cnt = (min(seq_len, pq) + 63) / 64;
  else if (t == nq - 1 && seq_len % pq != 0) cnt = n + (seq_len - (seq_len / pq) * pq + 63) / 64;
  blk_count[i] = cnt;
  for (int j = 0; j < n; ++j) {
    row[j] = j * 64;
    row[n + j] = t * pq + j * 64;
  }
}

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
static inline bool strides_ok(int64_t sb, int64_t sh, int64_t ss) { return sb % 8 == 0 && sh % 8 == 0 && ss % 8 == 0; }
template <class TT> static inline int check_tensor(const TT& t) {
  if (!t.ptr) return VA_ERR_NULL;
  if (!aligned16(t.ptr) || !strides_ok(t.stride_b, t.stride_h, t.stride_s)) return VA_ERR_ALIGN;
  return VA_OK;
}
static inline bool bk_ok(int bk) { return bk == 16 || bk == 32 || bk == 64 || bk == 128; }
static inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

struct PrefillPlan {
  int nq_total, nqc_max, blk_width, step;  // step: query rows handled per launch
  int64_t capacity;
  size_t off_avg, off_cnt, off_idx, off_bcnt, off_bidx, off_mask, mask_bytes, total;
};

static inline size_t budget_of(const va_prefill_args& a) {
  return a.single_pass_budget ? a.single_pass_budget : (size_t)VA_SINGLE_PASS_INDEX_BYTES_DEFAULT;
}

static int plan_prefill(const va_prefill_args& a, PrefillPlan& pl, size_t single_pass_budget) {
  if (a.dtype != VA_BF16 && a.dtype != VA_FP16) return VA_ERR_DTYPE;
  if (a.head_dim != kHeadDim || a.batch <= 0 || a.heads <= 0 || a.kv_heads <= 0 || a.sq <= 0 || a.sk <= 0)
    return VA_ERR_SHAPE;
  if (a.heads % a.kv_heads != 0 || a.heads > 65535 || a.batch > 65535) return VA_ERR_SHAPE;
  if (a.pq != 64 && a.pq != 128) return VA_ERR_PARAM;                    // VecAttention.py:44
  if (a.chunk_size <= 0 || a.chunk_size % a.pq != 0) return VA_ERR_PARAM;  // VecAttention.py:43
  if (!bk_ok(a.bk) || a.group_k_block <= 0) return VA_ERR_SHAPE;
  if (a.causal && a.pq % a.bk != 0) return VA_ERR_PARAM;                 // vecattention_kernels.py:129
  if (a.causal && a.sq != a.sk) return VA_ERR_PARAM;
  const size_t bh = (size_t)a.batch * a.heads;
  const int chunk = a.chunk_size < a.sq ? a.chunk_size : a.sq;
  pl.nq_total = (a.sq + a.pq - 1) / a.pq;
  pl.blk_width = a.causal ? 2 * (a.pq / 64) : 1;
  pl.capacity = (a.sk + 3) / 4 * 4;
  // one launch per stage for the whole sequence when its index lists fit the budget
  const bool single = bh * (size_t)pl.nq_total * (size_t)pl.capacity * 4 <= single_pass_budget;
  pl.step = single ? a.sq : chunk;
  pl.nqc_max = (pl.step + a.pq - 1) / a.pq;
  size_t off = 0;
  pl.off_avg = off;  off = align_up(off + bh * pl.nqc_max * kHeadDim * 2, 256);
  pl.off_cnt = off;  off = align_up(off + bh * pl.nqc_max * 4, 256);
  pl.off_bcnt = off; off = align_up(off + bh * pl.nqc_max * 4, 256);
  pl.off_bidx = off; off = align_up(off + bh * pl.nqc_max * pl.blk_width * 4, 256);
  pl.mask_bytes = select_workspace_bytes(a.batch, a.heads, a.kv_heads, pl.nqc_max, a.sk);
  pl.off_mask = off; off = align_up(off + pl.mask_bytes, 256);
  pl.off_idx = off;  off = align_up(off + bh * pl.nqc_max * (size_t)pl.capacity * 4, 256);
  pl.total = off;
  return VA_OK;
}
}  // namespace va

using namespace va;

extern "C" {

int va_version(void) { return 201; }  // 201: va_attn_args gained the vision fields; va_qk_head_norm_rope

const char* va_status_string(int code) {
  switch (code) {
    case VA_OK: return "ok";
    case VA_ERR_NULL: return "a required pointer is NULL";
    case VA_ERR_DTYPE: return "dtype must be VA_BF16 or VA_FP16";
    case VA_ERR_SHAPE: return "unsupported or inconsistent sizes (head_dim must be 128, k_local_size one of 16/32/64/128, heads a multiple of kv_heads)";
    case VA_ERR_ALIGN: return "pointers and strides must be multiples of 16 bytes";
    case VA_ERR_CAPACITY: return "index capacity or workspace too small";
    case VA_ERR_CUDA: return "CUDA launch failed";
    case VA_ERR_STATIC_SCRATCH: return "problem needs more scratch than the built-in VA_STATIC_SCRATCH_BYTES array of va_prefill_static holds (use a smaller chunk_size, or va_prefill with a workspace)";
    case VA_ERR_PARAM: return "parameters rejected (q_pooling_size must be 64 or 128, chunk_size a multiple of it, causal needs q_pooling_size % k_local_size == 0 and Sq == Sk)";
    default: return "unknown status";
  }
}

int va_pool_q(const va_pool_args* a, va_stream_t stream) {
  if (!a || !a->out) return VA_ERR_NULL;
  if (a->dtype != VA_BF16 && a->dtype != VA_FP16) return VA_ERR_DTYPE;
  if (a->head_dim != kHeadDim || a->batch <= 0 || a->heads <= 0 || a->seq_len <= 0 || a->heads > 65535 || a->batch > 65535)
    return VA_ERR_SHAPE;
  if (a->pq != 64 && a->pq != 128) return VA_ERR_PARAM;
  if (int rc = check_tensor(a->q)) return rc;
  if (!aligned16(a->out)) return VA_ERR_ALIGN;
  return pool_q(*a, reinterpret_cast<cudaStream_t>(stream));
}

int va_select(const va_select_args* a, va_stream_t stream) {
  if (!a || !a->avg_q || !a->col_count || !a->col_idx) return VA_ERR_NULL;
  if (a->dtype != VA_BF16 && a->dtype != VA_FP16) return VA_ERR_DTYPE;
  if (a->head_dim != kHeadDim || a->batch <= 0 || a->heads <= 0 || a->kv_heads <= 0 || a->nq <= 0 || a->sk <= 0)
    return VA_ERR_SHAPE;
  if (a->heads % a->kv_heads != 0 || a->kv_heads > 65535 || a->batch > 65535) return VA_ERR_SHAPE;
  if (!bk_ok(a->bk) || a->group_k_block <= 0 || a->pq <= 0) return VA_ERR_SHAPE;
  if ((a->causal || a->wo_initial) && a->pq % a->bk != 0) return VA_ERR_PARAM;
  if (a->capacity <= 0) return VA_ERR_CAPACITY;
  if (a->compat_bsq < 0 || a->tile_offset < 0 || a->chunk_tiles < 0) return VA_ERR_SHAPE;
  if (int rc = check_tensor(a->k)) return rc;
  if (!aligned16(a->avg_q)) return VA_ERR_ALIGN;
  return select(*a, reinterpret_cast<cudaStream_t>(stream));
}

int va_select_workspace_bytes(const va_select_args* a, size_t* bytes) {
  if (!a || !bytes) return VA_ERR_NULL;
  if (a->batch <= 0 || a->heads <= 0 || a->kv_heads <= 0 || a->nq <= 0 || a->sk <= 0 || a->heads % a->kv_heads != 0)
    return VA_ERR_SHAPE;
  *bytes = select_workspace_bytes(a->batch, a->heads, a->kv_heads, a->nq, a->sk);
  return VA_OK;
}

int va_sparse_attn_workspace_bytes(const va_attn_args* a, size_t* bytes) {
  if (!a || !bytes) return VA_ERR_NULL;
  *bytes = 0;
  return VA_OK;
}

int va_sparse_attn(const va_attn_args* a, va_stream_t stream) {
  if (!a || !a->col_count || !a->col_idx) return VA_ERR_NULL;
  if (a->blk_count && !a->blk_idx) return VA_ERR_NULL;
  if (a->dtype != VA_BF16 && a->dtype != VA_FP16) return VA_ERR_DTYPE;
  if (a->head_dim != kHeadDim || a->batch <= 0 || a->heads <= 0 || a->kv_heads <= 0 || a->sq <= 0 || a->sk <= 0)
    return VA_ERR_SHAPE;
  if (a->heads % a->kv_heads != 0 || a->heads > 65535 || a->batch > 65535) return VA_ERR_SHAPE;
  if (a->pq != 64 && a->pq != 128) return VA_ERR_PARAM;
  if (a->q_offset < 0 || a->col_stride <= 0) return VA_ERR_SHAPE;
  if (a->vision_mode) {  // spattn/src/models/utils.py:97: causal only; one sequence for queries and keys
    if (a->pq != 64 || !a->causal || a->sq != a->sk || a->q_offset != 0) return VA_ERR_PARAM;
    if (a->vision_begin < 0 || a->vision_begin > a->vision_end || a->vision_end > a->sq) return VA_ERR_SHAPE;
  }
  if (int rc = check_tensor(a->q)) return rc;
  if (int rc = check_tensor(a->k)) return rc;
  if (int rc = check_tensor(a->v)) return rc;
  if (int rc = check_tensor(a->out)) return rc;
  return sparse_attn(*a, reinterpret_cast<cudaStream_t>(stream));
}

int va_qk_norm_rope(const va_norm_rope_args* a, va_stream_t stream) {
  if (!a || !a->q || !a->k || !a->q_out || !a->k_out) return VA_ERR_NULL;
  if ((a->cos == nullptr) != (a->sin == nullptr)) return VA_ERR_NULL;
  if (a->dtype != VA_BF16 && a->dtype != VA_FP16) return VA_ERR_DTYPE;
  if (a->batch <= 0 || a->seq_len <= 0 || a->heads <= 0 || a->kv_heads <= 0 || a->rope_skip < 0) return VA_ERR_SHAPE;
  if (a->heads > 64 || a->kv_heads > 64) return VA_ERR_SHAPE;  // hidden sizes up to 8192
  if ((int64_t)a->batch * a->seq_len > 0x7fffffff) return VA_ERR_SHAPE;
  const void* ptrs[] = {a->q, a->k, a->q_out, a->k_out, a->q_weight, a->k_weight, a->cos, a->sin};
  for (const void* p : ptrs)
    if (p && !aligned16(p)) return VA_ERR_ALIGN;
  if (a->q_row_stride % 8 || a->k_row_stride % 8 || a->q_out_row_stride % 8 || a->k_out_row_stride % 8) return VA_ERR_ALIGN;
  return qk_norm_rope(*a, reinterpret_cast<cudaStream_t>(stream));
}

int va_qk_head_norm_rope(const va_head_norm_rope_args* a, va_stream_t stream) {
  if (!a || !a->q.ptr || !a->k.ptr || !a->q_out.ptr || !a->k_out.ptr) return VA_ERR_NULL;
  if ((a->cos == nullptr) != (a->sin == nullptr)) return VA_ERR_NULL;
  if (a->dtype != VA_BF16 && a->dtype != VA_FP16) return VA_ERR_DTYPE;
  if (a->batch <= 0 || a->seq_len <= 0 || a->heads <= 0 || a->kv_heads <= 0) return VA_ERR_SHAPE;
  if (a->rope_len < 0 || a->rope_len > a->seq_len) return VA_ERR_SHAPE;
  if (int rc = check_tensor(a->q)) return rc;
  if (int rc = check_tensor(a->k)) return rc;
  if (int rc = check_tensor(a->q_out)) return rc;
  if (int rc = check_tensor(a->k_out)) return rc;
  const void* ptrs[] = {a->q_weight, a->k_weight, a->cos, a->sin};
  for (const void* p : ptrs)
    if (p && !aligned16(p)) return VA_ERR_ALIGN;
  return qk_head_norm_rope(*a, reinterpret_cast<cudaStream_t>(stream));
}

int va_block_tables(int32_t batch, int32_t heads, int32_t seq_len, int32_t pq, int32_t causal, int32_t* blk_count,
                    int32_t* blk_idx, va_stream_t stream) {
  if (!blk_count || !blk_idx) return VA_ERR_NULL;
  if (batch <= 0 || heads <= 0 || seq_len <= 0) return VA_ERR_SHAPE;
  if (pq != 64 && pq != 128) return VA_ERR_PARAM;
  const int nq = (seq_len + pq - 1) / pq;
  const int64_t n = (int64_t)batch * heads * nq;
  if (n > 0x7fffffff) return VA_ERR_SHAPE;
  block_tables_kernel<<<(unsigned)((n + 255) / 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      batch * heads, seq_len, pq, causal, 0, nq, blk_count, blk_idx);
  return cudaGetLastError() == cudaSuccess ? VA_OK : VA_ERR_CUDA;
}

int va_prefill_workspace_bytes(const va_prefill_args* a, size_t* bytes) {
  if (!a || !bytes) return VA_ERR_NULL;
  PrefillPlan pl;
  if (int rc = plan_prefill(*a, pl, budget_of(*a))) return rc;
  *bytes = pl.total;
  return VA_OK;
}

static int run_prefill(const va_prefill_args* a, size_t single_pass_budget, va_stream_t stream_) {
  if (!a || !a->workspace) return VA_ERR_NULL;
  PrefillPlan pl;
  if (int rc = plan_prefill(*a, pl, single_pass_budget)) return rc;
  if (a->workspace_bytes < pl.total) return VA_ERR_CAPACITY;
  if ((reinterpret_cast<uintptr_t>(a->workspace) & 255u) != 0) return VA_ERR_ALIGN;
  if (int rc = check_tensor(a->q)) return rc;
  if (int rc = check_tensor(a->k)) return rc;
  if (int rc = check_tensor(a->v)) return rc;
  if (int rc = check_tensor(a->out)) return rc;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  unsigned char* ws = static_cast<unsigned char*>(a->workspace);
  void* avg = ws + pl.off_avg;
  int32_t* cnt = reinterpret_cast<int32_t*>(ws + pl.off_cnt);
  int32_t* idx = reinterpret_cast<int32_t*>(ws + pl.off_idx);
  int32_t* bcnt = reinterpret_cast<int32_t*>(ws + pl.off_bcnt);
  int32_t* bidx = reinterpret_cast<int32_t*>(ws + pl.off_bidx);
  const int bh = a->batch * a->heads;
  const size_t esz = 2;

  for (int i = 0; i < a->sq; i += pl.step) {  // VecAttention.py:94 (one iteration when the whole sequence fits)
    const int sqc = (a->sq - i) < pl.step ? (a->sq - i) : pl.step;
    const int nqc = (sqc + a->pq - 1) / a->pq;
    va_tensor4 qc = a->q;
    qc.ptr = static_cast<const unsigned char*>(a->q.ptr) + (size_t)i * a->q.stride_s * esz;
    va_tensor4_out oc = a->out;
    oc.ptr = static_cast<unsigned char*>(a->out.ptr) + (size_t)i * a->out.stride_s * esz;

    va_pool_args pa{a->dtype, a->batch, a->heads, sqc, a->head_dim, a->pq, qc, avg};
    if (int rc = pool_q(pa, stream)) return rc;

    va_select_args sa{};
    sa.dtype = a->dtype; sa.batch = a->batch; sa.heads = a->heads; sa.kv_heads = a->kv_heads;
    sa.nq = nqc; sa.sk = a->sk; sa.head_dim = a->head_dim;
    sa.pq = a->pq; sa.bk = a->bk; sa.group_k_block = a->group_k_block;
    sa.causal = a->causal; sa.wo_initial = a->causal;  // VecAttention.py:101
    sa.compat_bsq = a->compat_bsq; sa.tile_offset = i / a->pq;
    sa.avg_q = avg; sa.k = a->k; sa.gap = a->gap; sa.gaps = a->gaps; sa.gaps_stride_b = a->gaps_stride_b;
    sa.col_count = cnt; sa.col_idx = idx; sa.capacity = pl.capacity; sa.status = a->status;
    sa.chunk_tiles = a->chunk_size / a->pq;
    sa.workspace = ws + pl.off_mask; sa.workspace_bytes = pl.mask_bytes;
    if (int rc = select(sa, stream)) return rc;

    block_tables_kernel<<<(bh * nqc + 255) / 256, 256, 0, stream>>>(bh, a->sq, a->pq, a->causal, i / a->pq, nqc, bcnt,
                                                                    bidx);
    if (cudaGetLastError() != cudaSuccess) return VA_ERR_CUDA;

    va_attn_args aa{};
    aa.dtype = a->dtype; aa.batch = a->batch; aa.heads = a->heads; aa.kv_heads = a->kv_heads;
    aa.sq = sqc; aa.head_dim = a->head_dim; aa.pq = a->pq;
    const int64_t kend = (int64_t)i + pl.step;
    aa.sk = a->causal ? (int)(kend < a->sk ? kend : a->sk) : a->sk;  // VecAttention.py:107-108
    aa.causal = a->causal; aa.q_offset = i;
    aa.q = qc; aa.k = a->k; aa.v = a->v; aa.out = oc;
    aa.blk_count = bcnt; aa.blk_idx = bidx; aa.blk_stride = pl.blk_width;
    aa.col_count = cnt; aa.col_idx = idx; aa.col_stride = pl.capacity;
    aa.softmax_scale = 0.f;
    aa.status = a->status;
    if (int rc = sparse_attn(aa, stream)) return rc;

    if (a->col_count_out) {
      if (cudaMemcpy2DAsync(a->col_count_out + i / a->pq, (size_t)pl.nq_total * 4, cnt, (size_t)nqc * 4,
                            (size_t)nqc * 4, bh, cudaMemcpyDeviceToDevice, stream) != cudaSuccess)
        return VA_ERR_CUDA;
    }
  }
  return VA_OK;
}

int va_prefill(const va_prefill_args* a, va_stream_t stream) {
  if (!a) return VA_ERR_NULL;
  return run_prefill(a, budget_of(*a), stream);
}

// ---- the operator for callers that cannot allocate device memory -----------------------------
// The scratch of the prefill (pooled queries, per-tile counts, block tables and the selected-
// column index lists) lives in this fixed array instead of a caller-supplied workspace.  It is
// part of the loaded module, so every GPU that loads the library holds it until the process exits.
static __device__ __align__(256) unsigned char g_static_scratch[VA_STATIC_SCRATCH_BYTES];

// One pass over the whole sequence if that fits the array, else chunk by chunk; VA_ERR_STATIC_SCRATCH
// if even one chunk's scratch exceeds it.  `budget` receives the single-pass budget of the chosen plan.
static int plan_static(const va_prefill_args& a, PrefillPlan& pl, size_t& budget) {
  budget = VA_STATIC_SCRATCH_BYTES;
  if (int rc = plan_prefill(a, pl, budget)) return rc;
  if (pl.total > (size_t)VA_STATIC_SCRATCH_BYTES) {
    budget = 1;  // nothing fits one byte: the chunk loop
    if (int rc = plan_prefill(a, pl, budget)) return rc;
    if (pl.total > (size_t)VA_STATIC_SCRATCH_BYTES) return VA_ERR_STATIC_SCRATCH;
  }
  return VA_OK;
}

int va_prefill_static_fits(const va_prefill_args* a) {
  if (!a) return VA_ERR_NULL;
  PrefillPlan pl;
  size_t budget;
  const int rc = plan_static(*a, pl, budget);
  return rc == VA_OK ? 1 : (rc == VA_ERR_STATIC_SCRATCH ? 0 : rc);
}

int va_prefill_static(const va_prefill_args* a, va_stream_t stream) {
  if (!a) return VA_ERR_NULL;
  PrefillPlan pl;
  size_t budget;
  if (int rc = plan_static(*a, pl, budget)) return rc;
  // In host code `g_static_scratch` names a host-side shadow of the array, not device memory: the
  // device address must be asked for, with the caller's device current.  It is asked for on every
  // call (a host-side lookup once the module is loaded on the device), so nothing stale survives a
  // cudaDeviceReset or a re-created context.
  void* ptr = nullptr;
  if (cudaGetSymbolAddress(&ptr, g_static_scratch) != cudaSuccess || !ptr) return VA_ERR_CUDA;
  va_prefill_args b = *a;
  b.workspace = ptr;
  b.workspace_bytes = VA_STATIC_SCRATCH_BYTES;
  return run_prefill(&b, budget, stream);
}

// ---- self-test of the bounded waits -----------------------------------------------------------
// One CTA: warp 0 allocates tensor memory as the real kernels do; one thread of warp 1 waits, with
// the kernels' own wait routine, on a barrier that nothing completes.  The wait gives up after
// `polls` polls, the status word receives VA_STATUS_TIMEOUT, the CTA meets at its final barrier and
// frees the tensor memory: the unwinding path of the real kernels, run on purpose.
__global__ void __launch_bounds__(64, 1) wait_timeout_kernel(int32_t* status, int polls) {
  __shared__ uint64_t never;
  __shared__ uint32_t tmem_base_s;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    sm100::mbar_init(&never, 1);
    sm100::fence_proxy_async();
  }
  if (warp == 0) {
    sm100::tmem_alloc(&tmem_base_s, 32);
    sm100::tmem_relinquish();
  }
  sm100::tc_fence_before();
  __syncthreads();
  sm100::tc_fence_after();
  bool timed_out = false;
  if (warp == 1 && lane == 0) timed_out = !sm100::mbar_wait(&never, 0, polls);
  if (timed_out) atomicOr(status, VA_STATUS_TIMEOUT);
  sm100::tc_fence_before();
  __syncthreads();
  if (warp == 0) sm100::tmem_dealloc(tmem_base_s, 32);
}

int va_selftest_wait_timeout(int32_t* status, int32_t polls, va_stream_t stream) {
  if (!status) return VA_ERR_NULL;
  if (polls < 1 || polls > 4096) return VA_ERR_SHAPE;
  wait_timeout_kernel<<<1, 64, 0, reinterpret_cast<cudaStream_t>(stream)>>>(status, polls);
  return cudaGetLastError() == cudaSuccess ? VA_OK : VA_ERR_CUDA;
}

}  // extern "C"
