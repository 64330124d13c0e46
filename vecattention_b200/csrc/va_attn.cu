// Vector-sparse flash attention: launch parameters from the C ABI's argument struct, and the choice of the
// kernel by query-tile height (q_pooling_size 64: va_attn64.cu, 128: va_attn128.cu).
#include "va_common.cuh"
#include "va_attn.cuh"

namespace va {

int launch_attn64(const AttnParams& p, int dtype, int batch, cudaStream_t stream);   // va_attn64.cu
int launch_attn128(const AttnParams& p, int dtype, int batch, cudaStream_t stream);  // va_attn128.cu

int sparse_attn(const va_attn_args& a, cudaStream_t stream) {
  AttnParams p;
  p.q = a.q.ptr; p.k = a.k.ptr; p.v = a.v.ptr; p.out = a.out.ptr;
  p.q_sb = a.q.stride_b; p.q_sh = a.q.stride_h; p.q_ss = a.q.stride_s;
  p.k_sb = a.k.stride_b; p.k_sh = a.k.stride_h; p.k_ss = a.k.stride_s;
  p.v_sb = a.v.stride_b; p.v_sh = a.v.stride_h; p.v_ss = a.v.stride_s;
  p.o_sb = a.out.stride_b; p.o_sh = a.out.stride_h; p.o_ss = a.out.stride_s;
  p.blk_count = a.blk_idx ? a.blk_count : nullptr;
  p.blk_idx = a.blk_idx; p.blk_stride = a.blk_stride;
  p.col_count = a.col_count; p.col_idx = a.col_idx; p.col_stride = a.col_stride;
  p.status = a.status;
  p.lse = a.lse;
  p.heads = a.heads; p.rep = a.heads / a.kv_heads; p.sq = a.sq; p.sk = a.sk;
  p.vis_on = a.vision_mode != 0; p.vis_begin = a.vision_begin; p.vis_end = a.vision_end;
  p.nq = ((p.vis_on ? a.vision_end : a.sq) + a.pq - 1) / a.pq;
  p.causal = a.causal; p.q_offset = a.q_offset;
  const float scale = a.softmax_scale > 0.f ? a.softmax_scale : 0.08838834764831845f;
  p.scale_log2 = scale * 1.4426950408889634f;
  return a.pq == 64 ? launch_attn64(p, a.dtype, a.batch, stream) : launch_attn128(p, a.dtype, a.batch, stream);
}

}  // namespace va
