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
};

}  // namespace va
