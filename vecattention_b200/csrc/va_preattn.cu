// What a video-DiT attention layer does to Q and K between the projections and the operator, in one pass:
// RMSNorm over the hidden dimension, the rotary embedding on interleaved (even, odd) element pairs, and no
// layout change at all, because the operator reads (B, S, H, D) storage in place through strides.
//
// Reference (eval/DiTEvalKit/models/wan/attention.py:108-136): a Triton RMSNorm kernel (read + write),
// three transposed copies to (B, H, S, D) (read + write each) and an in-place rotary kernel (read + write).
// Here every element of Q and K is read once and written once; V is not touched.
//
// One CTA of 256 threads per token row of one tensor (grid.y: 0 = Q, 1 = K).  A thread owns 16-byte pieces
// (8 elements) of the row: sum of squares in fp32 (per thread in element order, then a fixed shuffle tree and a
// fixed sum over the warps), y = round16(x * rstd * w) as the norm kernel stores it
// (eval/DiTEvalKit/kernels/triton/rmsnorm.py:30-47), then out = round16(double(y0) * cos - double(y1) * sin),
// round16(double(y1) * cos + double(y0) * sin) for every pair, in double precision as the rotary kernel
// computes it (eval/DiTEvalKit/kernels/include/rope/rope_enc_complex.cuh:27-45).
#include "va_common.cuh"

namespace va {

namespace {

constexpr int kNormThreads = 256;
constexpr int kMaxPieces = 4;  // 16-byte pieces per thread: hidden sizes up to 256 * 4 * 8 = 8192 elements

template <int DT>
__device__ __forceinline__ typename Elem<DT>::T from_double(double x) {
  if constexpr (DT == VA_BF16) return __double2bfloat16(x);
  else return __double2half(x);
}

template <int DT>
__global__ void __launch_bounds__(kNormThreads) qk_norm_rope_kernel(const va_norm_rope_args a) {
  using T = typename Elem<DT>::T;
  const bool is_k = blockIdx.y == 1;
  const int64_t token = blockIdx.x;                 // b * seq_len + s
  const int s = (int)(token % a.seq_len);
  const int hidden = (is_k ? a.kv_heads : a.heads) * kHeadDim;
  const T* x = static_cast<const T*>(is_k ? a.k : a.q) + token * (is_k ? a.k_row_stride : a.q_row_stride);
  T* y = static_cast<T*>(is_k ? a.k_out : a.q_out) + token * (is_k ? a.k_out_row_stride : a.q_out_row_stride);
  const T* w = static_cast<const T*>(is_k ? a.k_weight : a.q_weight);
  const int pieces = hidden / 8;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  float v[kMaxPieces][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < kMaxPieces; ++i) {
    const int pc = tid + i * kNormThreads;
    if (pc < pieces) {
      const uint4 raw = __ldg(reinterpret_cast<const uint4*>(x + pc * 8));
      const uint32_t ww[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = Elem<DT>::unpack(ww[j]);
        v[i][2 * j] = f.x;
        v[i][2 * j + 1] = f.y;
        ss = fmaf(f.x, f.x, ss);
        ss = fmaf(f.y, f.y, ss);
      }
    }
  }
  __shared__ float part[kNormThreads / 32];
  __shared__ float rstd_s;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if (lane == 0) part[warp] = ss;
  __syncthreads();
  if (tid == 0) {
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < kNormThreads / 32; ++i) tot += part[i];
    rstd_s = 1.0f / sqrtf(tot / (float)hidden + a.eps);
  }
  __syncthreads();
  const float rstd = w ? rstd_s : 1.0f;  // no weight: no normalisation (rotary embedding only)

  const int rs = s - a.rope_skip;  // row of the cos / sin tables; the first rope_skip tokens are not rotated
  const bool rotate = a.cos != nullptr && rs >= 0;
#pragma unroll
  for (int i = 0; i < kMaxPieces; ++i) {
    const int pc = tid + i * kNormThreads;
    if (pc < pieces) {
      float yv[8];
      if (w) {
        const uint4 wr = __ldg(reinterpret_cast<const uint4*>(w + pc * 8));
        const uint32_t ww[4] = {wr.x, wr.y, wr.z, wr.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = Elem<DT>::unpack(ww[j]);
          // x_hat = x * rstd, y = x_hat * w, rounded to the 16-bit type as the norm kernel stores it
          yv[2 * j] = Elem<DT>::to_float(Elem<DT>::from_float(__fmul_rn(__fmul_rn(v[i][2 * j], rstd), f.x)));
          yv[2 * j + 1] = Elem<DT>::to_float(Elem<DT>::from_float(__fmul_rn(__fmul_rn(v[i][2 * j + 1], rstd), f.y)));
        }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) yv[j] = v[i][j];
      }
      uint32_t out[4];
      if (rotate) {
        const int d0 = (pc * 8) % kHeadDim;  // position of the piece inside its head
        const float4 c = __ldg(reinterpret_cast<const float4*>(a.cos + (int64_t)rs * (kHeadDim / 2) + d0 / 2));
        const float4 sn = __ldg(reinterpret_cast<const float4*>(a.sin + (int64_t)rs * (kHeadDim / 2) + d0 / 2));
        const float cc[4] = {c.x, c.y, c.z, c.w}, sv[4] = {sn.x, sn.y, sn.z, sn.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const double e = yv[2 * j], o = yv[2 * j + 1], cj = cc[j], sj = sv[j];
          const T r0 = from_double<DT>(e * cj + (-o) * sj);
          const T r1 = from_double<DT>(o * cj + e * sj);
          out[j] = (uint32_t) * reinterpret_cast<const uint16_t*>(&r0) | ((uint32_t) * reinterpret_cast<const uint16_t*>(&r1) << 16);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) out[j] = Elem<DT>::pack(yv[2 * j], yv[2 * j + 1]);
      }
      *reinterpret_cast<uint4*>(y + pc * 8) = make_uint4(out[0], out[1], out[2], out[3]);
    }
  }
}

}  // namespace

int qk_norm_rope(const va_norm_rope_args& a, cudaStream_t stream) {
  dim3 grid((unsigned)((int64_t)a.batch * a.seq_len), 2, 1);
  if (a.dtype == VA_BF16) qk_norm_rope_kernel<VA_BF16><<<grid, kNormThreads, 0, stream>>>(a);
  else qk_norm_rope_kernel<VA_FP16><<<grid, kNormThreads, 0, stream>>>(a);
  return cudaGetLastError() == cudaSuccess ? VA_OK : VA_ERR_CUDA;
}

}  // namespace va
