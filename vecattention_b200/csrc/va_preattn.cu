// What a video-DiT attention layer does to Q and K between the projections and the operator, in one pass:
// RMSNorm over the hidden dimension, the rotary embedding on interleaved (even, odd) element pairs, and no
// layout change at all, because the operator reads (B, S, H, D) storage in place through strides.
//
// Reference (eval/DiTEvalKit/models/wan/attention.py:108-136): a Triton RMSNorm kernel (read + write),
// three transposed copies to (B, H, S, D) (read + write each) and an in-place rotary kernel (read + write).
// Here every element of Q and K is read once and written once; V is not touched.
//
// A token row of one tensor (grid.y: 0 = Q, 1 = K) is taken by one, two or four warps, whose lanes own 16-byte
// pieces (8 elements) of it: sum of squares in fp32 (per lane in piece order, a fixed shuffle tree, a fixed sum over
// the row's warps), y = round16(x * rstd * w) as the norm kernel stores it
// (eval/DiTEvalKit/kernels/triton/rmsnorm.py:30-47), then out = round16(double(y0) * cos - double(y1) * sin),
// round16(double(y1) * cos + double(y0) * sin) for every pair, in double precision as the rotary kernel
// computes it (eval/DiTEvalKit/kernels/include/rope/rope_enc_complex.cuh:27-45).
// A second kernel serves models whose tensors are (B, H, L, 128) already, with a per-head norm and the text tokens
// last (HunyuanVideo).
#include "va_common.cuh"

namespace va {

namespace {

template <int DT>
__device__ __forceinline__ typename Elem<DT>::T from_double(double x) {
  if constexpr (DT == VA_BF16) return __double2bfloat16(x);
  else return __double2half(x);
}

// ---- the hidden-size form: W warps per token row ------------------------------------------------------------------
// A row is taken by W = ceil(hidden / 1024) warps; a lane keeps its (up to) four 16-byte pieces packed in registers,
// so every warp has its whole share of the row in flight at once, and the W warps add their partial sums through
// shared memory (one block barrier).  Few registers, hence some thirty warps resident per SM: enough outstanding
// memory, which one CTA per row with one piece or two per thread in flight was not (2.4 TB/s).  A CTA holds as many
// whole rows as fit eight warps.
constexpr int NP = 4;  // pieces per lane
template <int DT>
__global__ void __launch_bounds__(256) qk_norm_rope_rows_kernel(const va_norm_rope_args a, int64_t rows, int W, int rows_per_cta) {
  using T = typename Elem<DT>::T;
  __shared__ float part[8];  // [row of the CTA * W + warp of the row]
  const bool is_k = blockIdx.y == 1;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int rsub = warp / W, wsub = warp % W;
  const int64_t token = (int64_t)blockIdx.x * rows_per_cta + rsub;  // b * seq_len + s
  const bool live = token < rows;
  const int s = (int)((live ? token : 0) % a.seq_len);
  const int hidden = (is_k ? a.kv_heads : a.heads) * kHeadDim;
  const T* x = static_cast<const T*>(is_k ? a.k : a.q) + (live ? token : 0) * (is_k ? a.k_row_stride : a.q_row_stride);
  T* y = static_cast<T*>(is_k ? a.k_out : a.q_out) + (live ? token : 0) * (is_k ? a.k_out_row_stride : a.q_out_row_stride);
  const T* w = static_cast<const T*>(is_k ? a.k_weight : a.q_weight);
  const int pieces = live ? hidden / 8 : 0;

  uint4 raw[NP];
#pragma unroll
  for (int i = 0; i < NP; ++i) {
    const int pc = wsub * 32 + lane + 32 * W * i;
    raw[i] = pc < pieces ? __ldg(reinterpret_cast<const uint4*>(x + pc * 8)) : make_uint4(0, 0, 0, 0);
  }
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < NP; ++i) {
    const uint32_t ww[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = Elem<DT>::unpack(ww[j]);
      ss = fmaf(f.x, f.x, ss);
      ss = fmaf(f.y, f.y, ss);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if (W > 1) {
    if (lane == 0) part[rsub * W + wsub] = ss;
    __syncthreads();
    ss = 0.f;
    for (int i = 0; i < W; ++i) ss += part[rsub * W + i];  // the same order in every warp of the row
  }
  const float rstd = w ? 1.0f / sqrtf(ss / (float)hidden + a.eps) : 1.0f;  // no weight: no normalisation

  const int rs = s - a.rope_skip;  // row of the cos / sin tables; the first rope_skip tokens are not rotated
  const bool rotate = a.cos != nullptr && rs >= 0;
#pragma unroll
  for (int i = 0; i < NP; ++i) {
    const int pc = wsub * 32 + lane + 32 * W * i;
    if (pc < pieces) {
      const uint32_t xw[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
      float yv[8];
      if (w) {
        const uint4 wr = __ldg(reinterpret_cast<const uint4*>(w + pc * 8));
        const uint32_t ww[4] = {wr.x, wr.y, wr.z, wr.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = Elem<DT>::unpack(ww[j]), v = Elem<DT>::unpack(xw[j]);
          // x_hat = x * rstd, y = x_hat * w, rounded to the 16-bit type as the norm kernel stores it
          yv[2 * j] = Elem<DT>::to_float(Elem<DT>::from_float(__fmul_rn(__fmul_rn(v.x, rstd), f.x)));
          yv[2 * j + 1] = Elem<DT>::to_float(Elem<DT>::from_float(__fmul_rn(__fmul_rn(v.y, rstd), f.y)));
        }
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 v = Elem<DT>::unpack(xw[j]);
          yv[2 * j] = v.x;
          yv[2 * j + 1] = v.y;
        }
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

template <int DT>
int launch_rows_dt(const va_norm_rope_args& a, cudaStream_t stream) {
  const int64_t rows = (int64_t)a.batch * a.seq_len;
  const int pieces = (a.heads > a.kv_heads ? a.heads : a.kv_heads) * kHeadDim / 8;  // of the wider of the two tensors
  const int W = (pieces + 32 * NP - 1) / (32 * NP);                                 // 1 .. 8 (hidden sizes up to 8192)
  const int per = 8 / W;
  dim3 grid((unsigned)((rows + per - 1) / per), 2, 1);
  qk_norm_rope_rows_kernel<DT><<<grid, 32 * W * per, 0, stream>>>(a, rows, W, per);
  return cudaGetLastError() == cudaSuccess ? VA_OK : VA_ERR_CUDA;
}

// ---- the per-head form (HunyuanVideo): tensors are (B, H, L, 128) already ---------------------------------------
// RMSNorm over the 128 elements of every (batch, head, token) row (eval/DiTEvalKit/kernels/include/norm/
// narrow_rms_norm.cuh:22-73: sixteen threads per row, eight elements each, sum of squares in element order, xor
// shuffles 8-4-2-1, rsqrtf(sum / 128 + eps), y = T((x * r) * w)), then the rotary embedding on interleaved pairs
// in fp32 with per-element tables, out[i] = y[i] cos[i] + (i even ? -y[i+1] : y[i-1]) sin[i]
// (eval/DiTEvalKit/kernels/include/rope/rope_enc_txtlast.cuh:32-76: tokens from rope_len on are left alone).
// The same sixteen-threads-per-row layout here.
template <int DT>
__global__ void __launch_bounds__(256) qk_head_norm_rope_kernel(const va_head_norm_rope_args a, int64_t tokens) {
  using T = typename Elem<DT>::T;
  // Sixteen lanes per token (b, l); they walk the token's heads, Q's then K's, four at a time, so that the token's
  // 1 KB of cos / sin entries is read once and four rows are in flight per lane.
  const int lane16 = threadIdx.x & 15;
  const int64_t token = (int64_t)blockIdx.x * 16 + (threadIdx.x >> 4);
  const bool live = token < tokens;
  const int l = (int)((live ? token : 0) % a.seq_len);
  const int b = (int)((live ? token : 0) / a.seq_len);
  const bool rotate = a.cos != nullptr && l < a.rope_len;
  float cc[8], sn[8];
  if (rotate) {
    const float* cr = a.cos + (int64_t)l * kHeadDim + lane16 * 8;
    const float* sr = a.sin + (int64_t)l * kHeadDim + lane16 * 8;
    const float4 c0 = __ldg(reinterpret_cast<const float4*>(cr)), c1 = __ldg(reinterpret_cast<const float4*>(cr + 4));
    const float4 s0 = __ldg(reinterpret_cast<const float4*>(sr)), s1 = __ldg(reinterpret_cast<const float4*>(sr + 4));
    cc[0] = c0.x; cc[1] = c0.y; cc[2] = c0.z; cc[3] = c0.w; cc[4] = c1.x; cc[5] = c1.y; cc[6] = c1.z; cc[7] = c1.w;
    sn[0] = s0.x; sn[1] = s0.y; sn[2] = s0.z; sn[3] = s0.w; sn[4] = s1.x; sn[5] = s1.y; sn[6] = s1.z; sn[7] = s1.w;
  }
#pragma unroll 1
  for (int which = 0; which < 2; ++which) {  // 0: Q, 1: K
    const va_tensor4& in = which ? a.k : a.q;
    const va_tensor4_out& out = which ? a.k_out : a.q_out;
    const int heads = which ? a.kv_heads : a.heads;
    const T* w = static_cast<const T*>(which ? a.k_weight : a.q_weight);
    const T* xb = static_cast<const T*>(in.ptr) + b * in.stride_b + (int64_t)l * in.stride_s + lane16 * 8;
    T* yb = static_cast<T*>(out.ptr) + b * out.stride_b + (int64_t)l * out.stride_s + lane16 * 8;
    float wv[8];
    if (w) {
      const uint4 wr = __ldg(reinterpret_cast<const uint4*>(w + lane16 * 8));
      const uint32_t ww[4] = {wr.x, wr.y, wr.z, wr.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = Elem<DT>::unpack(ww[j]);
        wv[2 * j] = f.x;
        wv[2 * j + 1] = f.y;
      }
    }
#pragma unroll 1
    for (int h0 = 0; h0 < heads; h0 += 4) {
      uint4 raw[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        raw[u] = (live && h0 + u < heads) ? __ldg(reinterpret_cast<const uint4*>(xb + (int64_t)(h0 + u) * in.stride_h)) : make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const uint32_t xw[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
        float v[8];
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = Elem<DT>::unpack(xw[j]);
          v[2 * j] = f.x;
          v[2 * j + 1] = f.y;
          ss = fmaf(f.x, f.x, ss);
          ss = fmaf(f.y, f.y, ss);
        }
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);  // within the token's sixteen lanes
        if (w) {
          const float rs = rsqrtf(ss / (float)kHeadDim + a.eps);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[j] = Elem<DT>::to_float(Elem<DT>::from_float(__fmul_rn(__fmul_rn(v[j], rs), wv[j])));
        }
        uint32_t o4[4];
        if (rotate) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float e = v[2 * j], od = v[2 * j + 1];
            const float r0 = fmaf(-od, sn[2 * j], __fmul_rn(e, cc[2 * j]));        // x[i] cos[i] + (-x[i+1]) sin[i]
            const float r1 = fmaf(e, sn[2 * j + 1], __fmul_rn(od, cc[2 * j + 1]));  // x[i] cos[i] + x[i-1] sin[i]
            o4[j] = Elem<DT>::pack(r0, r1);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j) o4[j] = Elem<DT>::pack(v[2 * j], v[2 * j + 1]);
        }
        if (live && h0 + u < heads)
          *reinterpret_cast<uint4*>(yb + (int64_t)(h0 + u) * out.stride_h) = make_uint4(o4[0], o4[1], o4[2], o4[3]);
      }
    }
  }
}

}  // namespace

int qk_head_norm_rope(const va_head_norm_rope_args& a, cudaStream_t stream) {
  const int64_t tokens = (int64_t)a.batch * a.seq_len;
  const unsigned grid = (unsigned)((tokens + 15) / 16);
  if (a.dtype == VA_BF16) qk_head_norm_rope_kernel<VA_BF16><<<grid, 256, 0, stream>>>(a, tokens);
  else qk_head_norm_rope_kernel<VA_FP16><<<grid, 256, 0, stream>>>(a, tokens);
  return cudaGetLastError() == cudaSuccess ? VA_OK : VA_ERR_CUDA;
}

int qk_norm_rope(const va_norm_rope_args& a, cudaStream_t stream) {
  return a.dtype == VA_BF16 ? launch_rows_dt<VA_BF16>(a, stream) : launch_rows_dt<VA_FP16>(a, stream);
}

}  // namespace va
