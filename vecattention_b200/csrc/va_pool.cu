// Mean pooling of Q per query tile (HBM-bound: reads Q once, writes one row per tile).
//
// One CTA of 128 threads per (tile, head, batch).  A row is 128 elements = 16 chunks of 16
// bytes; thread t owns chunk (t & 15) of the rows of row group (t >> 4).  The fp32 sum over the
// pq rows is a balanced binary tree: each thread first reduces its pq/8 consecutive rows as a
// tree in registers (an aligned sub-tree), then the 8 group partials are combined as a tree from
// shared memory.  The CPU oracle uses the same association, so both round identically.
#include "va_common.cuh"

namespace va {

template <int DT, int PQ>
__global__ void __launch_bounds__(128) pool_q_kernel(const typename Elem<DT>::T* __restrict__ q,
                                                     int64_t sb, int64_t sh, int64_t ss, int seq_len,
                                                     int nq, typename Elem<DT>::T* __restrict__ out) {
  constexpr int R = PQ / 8;  // rows per thread
  const int tile = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int t = threadIdx.x, c = t & 15, g = t >> 4;
  const int row0 = tile * PQ;
  const int valid = min(PQ, seq_len - row0);
  const typename Elem<DT>::T* base = q + b * sb + h * sh + (int64_t)row0 * ss + c * 8;

  uint4 raw[R];
#pragma unroll
  for (int i = 0; i < R; ++i) {
    int r = g * R + i;
    raw[i] = (r < valid) ? __ldg(reinterpret_cast<const uint4*>(base + (int64_t)r * ss)) : make_uint4(0, 0, 0, 0);
  }
  float acc[R][8];
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const uint32_t w[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 f = Elem<DT>::unpack(w[j]);
      acc[i][2 * j] = f.x;
      acc[i][2 * j + 1] = f.y;
    }
  }
#pragma unroll
  for (int n = R; n > 1; n >>= 1) {
#pragma unroll
    for (int i = 0; i < n / 2; ++i) {
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[i][j] = __fadd_rn(acc[2 * i][j], acc[2 * i + 1][j]);
    }
  }
  __shared__ float part[8][kHeadDim];
#pragma unroll
  for (int j = 0; j < 8; ++j) part[g][c * 8 + j] = acc[0][j];
  __syncthreads();
  const int d = t;  // 128 threads, one output element each
  float p01 = __fadd_rn(part[0][d], part[1][d]);
  float p23 = __fadd_rn(part[2][d], part[3][d]);
  float p45 = __fadd_rn(part[4][d], part[5][d]);
  float p67 = __fadd_rn(part[6][d], part[7][d]);
  float tot = __fadd_rn(__fadd_rn(p01, p23), __fadd_rn(p45, p67));
  float mean = __fdiv_rn(tot, static_cast<float>(valid));
  out[(((int64_t)b * gridDim.y + h) * nq + tile) * kHeadDim + d] = Elem<DT>::from_float(mean);
}

template <int DT>
static int launch_pool(const va_pool_args& a, cudaStream_t stream) {
  using T = typename Elem<DT>::T;
  const int nq = (a.seq_len + a.pq - 1) / a.pq;
  dim3 grid(nq, a.heads, a.batch);
  if (a.pq == 64)
    pool_q_kernel<DT, 64><<<grid, 128, 0, stream>>>(static_cast<const T*>(a.q.ptr), a.q.stride_b, a.q.stride_h,
                                                    a.q.stride_s, a.seq_len, nq, static_cast<T*>(a.out));
  else
    pool_q_kernel<DT, 128><<<grid, 128, 0, stream>>>(static_cast<const T*>(a.q.ptr), a.q.stride_b, a.q.stride_h,
                                                     a.q.stride_s, a.seq_len, nq, static_cast<T*>(a.out));
  return cudaGetLastError() == cudaSuccess ? VA_OK : VA_ERR_CUDA;
}

int pool_q(const va_pool_args& a, cudaStream_t stream) {
  return a.dtype == VA_BF16 ? launch_pool<VA_BF16>(a, stream) : launch_pool<VA_FP16>(a, stream);
}

}  // namespace va
