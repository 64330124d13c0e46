// Launch parameters shared by the sparse-attention kernels.
#pragma once

#include <stdint.h>

namespace va {

struct AttnParams {
  const void* q;
  const void* k;
  const void* v;
  void* out;
  int64_t q_sb, q_sh, q_ss, k_sb, k_sh, k_ss, v_sb, v_sh, v_ss, o_sb, o_sh, o_ss;
  const int32_t* blk_count;
  const int32_t* blk_idx;
  int64_t blk_stride;
  const int32_t* col_count;
  const int32_t* col_idx;
  int64_t col_stride;
  int32_t* status;
  float* lse;  // optional (B,H,sq): natural-log sum of exp over the row's keys
  int heads, rep, sq, sk, nq;
  int causal, q_offset;
  float scale_log2;  // softmax_scale * log2(e)
  // Vision-slice composition (64-row kernel only): rows [0, vis_begin) and [vis_end, sq) get full causal attention
  // from tiles that need no tables, rows [vis_begin, vis_end) the sparse attention of their tile; `nq` then counts
  // the table tiles (rows [0, vis_end)) and the grid has the dense tiles behind them.
  int vis_on, vis_begin, vis_end;
};

}  // namespace va
