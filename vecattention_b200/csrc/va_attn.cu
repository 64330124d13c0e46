// Vector-sparse flash attention: one CTA per query tile, keys taken 64 at a time from the tile's
// dense 64-key blocks and then from its selected-column list (row gather).
//
// Each warp owns 16 query rows.  K and V chunks are gathered row by row into swizzled shared
// memory with cp.async (double buffered); S = Q K^T and O += P V run on mma.sync m16n8k16 with
// fp32 accumulators and an online softmax kept in registers (exp2 domain), P rounded to the
// input dtype before the PV product.
#include "va_common.cuh"

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
  int heads, rep, sq, sk, nq;
  int causal, q_offset;
  float scale_log2;  // softmax_scale * log2(e)
};

constexpr int kChunk = 64;  // keys per step

template <int PQ> constexpr size_t attn_smem_bytes() { return (size_t)PQ * 256 + 4 * (size_t)kChunk * 256; }

template <int DT, int PQ>
__global__ void __launch_bounds__(PQ * 2) sparse_attn_kernel(const AttnParams p) {
  using T = typename Elem<DT>::T;
  constexpr int NT = PQ * 2;  // threads: 16 rows per warp
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* q_s = smem;
  unsigned char* kv_s = smem + PQ * 256;  // [stage][K|V][64 rows][256 B]
  __shared__ int s_keys[2][kChunk];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int tile = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int hkv = h / p.rep;
  const int row0 = tile * PQ;
  const int64_t trow = ((int64_t)b * p.heads + h) * p.nq + tile;
  const int nblk = p.blk_count ? __ldg(p.blk_count + trow) : 0;
  const int ncol = __ldg(p.col_count + trow);
  const int32_t* blk = p.blk_idx + trow * p.blk_stride;
  const int32_t* col = p.col_idx + trow * p.col_stride;
  const int nchunks = nblk + (ncol + kChunk - 1) / kChunk;

  const T* qb = static_cast<const T*>(p.q) + b * p.q_sb + h * p.q_sh;
  const T* kb = static_cast<const T*>(p.k) + b * p.k_sb + hkv * p.k_sh;
  const T* vb = static_cast<const T*>(p.v) + b * p.v_sb + hkv * p.v_sh;

  // key index of slot s of chunk c, or -1 (slot unused / key outside the sequence)
  auto key_of = [&](int c, int s) -> int {
    int key;
    if (c < nblk) {
      key = __ldg(blk + c) + s;
    } else {
      const int i = (c - nblk) * kChunk + s;
      key = i < ncol ? __ldg(col + i) : -1;
    }
    return (key >= 0 && key < p.sk) ? key : -1;
  };
  auto load_chunk = [&](int c, int stage) {
    unsigned char* kd = kv_s + (size_t)stage * 2 * kChunk * 256;
    unsigned char* vd = kd + kChunk * 256;
#pragma unroll
    for (int i = 0; i < kChunk * 16 / NT; ++i) {
      const int pce = tid + i * NT;
      const int r = pce >> 4, cc = pce & 15;
      const int key = key_of(c, r);
      const bool ok = key >= 0;
      const int64_t kk = ok ? key : 0;
      cp_async16(smem_u32(kd + swz_off(r, cc)), kb + kk * p.k_ss + cc * 8, ok);
      cp_async16(smem_u32(vd + swz_off(r, cc)), vb + kk * p.v_ss + cc * 8, ok);
      if (cc == 0) s_keys[stage][r] = key;
    }
  };

  // ---- Q tile -> shared ----
  for (int i = tid; i < PQ * 16; i += NT) {
    const int r = i >> 4, c = i & 15;
    const bool ok = row0 + r < p.sq;
    cp_async16(smem_u32(q_s + swz_off(r, c)), qb + (int64_t)(ok ? row0 + r : 0) * p.q_ss + c * 8, ok);
  }
  cp_async_commit();
  if (nchunks > 0) load_chunk(0, 0);
  cp_async_commit();
  cp_async_wait<1>();
  __syncthreads();

  uint32_t qf[8][4];
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {
    const int r = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
    const int c = ks * 2 + (lane >> 4);
    ldmatrix_x4(qf[ks], smem_u32(q_s + swz_off(r, c)));
  }

  float o[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[i][e] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;  // rows lane/4 and lane/4+8 (scaled log2 domain)
  const int qpos0 = p.q_offset + row0 + warp * 16 + (lane >> 2);
  const int qpos1 = qpos0 + 8;

  for (int c = 0; c < nchunks; ++c) {
    const int stage = c & 1;
    if (c + 1 < nchunks) load_chunk(c + 1, stage ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const unsigned char* ks_ = kv_s + (size_t)stage * 2 * kChunk * 256;
    const unsigned char* vs_ = ks_ + kChunk * 256;

    // ---- S = Q K^T (16 x 64 per warp) ----
    float s[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[nt][e] = 0.f;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        uint32_t bf[4];
        const int r = np * 16 + (lane & 7) + (lane >> 4) * 8;
        const int cc = ks * 2 + ((lane >> 3) & 1);
        ldmatrix_x4(bf, smem_u32(ks_ + swz_off(r, cc)));
        mma16816<DT>(s[np * 2], qf[ks], bf[0], bf[1]);
        mma16816<DT>(s[np * 2 + 1], qf[ks], bf[2], bf[3]);
      }
    }
    // ---- mask: unused slots, keys outside the sequence, causal ----
    // a chunk needs the per-element test only if it has an invalid slot or a key beyond the first
    // query position of the tile
    {
      const int* keys = s_keys[stage];
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const int c0 = nt * 8 + (lane & 3) * 2;
        const int ka = keys[c0], kb2 = keys[c0 + 1];
        const bool da = ka < 0, db = kb2 < 0;
        if (da || (p.causal && ka > qpos0)) s[nt][0] = -INFINITY;
        if (db || (p.causal && kb2 > qpos0)) s[nt][1] = -INFINITY;
        if (da || (p.causal && ka > qpos1)) s[nt][2] = -INFINITY;
        if (db || (p.causal && kb2 > qpos1)) s[nt][3] = -INFINITY;
      }
    }
    // ---- online softmax ----
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      mx0 = fmaxf(mx0, fmaxf(s[nt][0], s[nt][1]));
      mx1 = fmaxf(mx1, fmaxf(s[nt][2], s[nt][3]));
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(m0, mx0 * p.scale_log2), mn1 = fmaxf(m1, mx1 * p.scale_log2);
    // a row with no valid key so far keeps m = -inf; use 0 as the reference point to avoid inf-inf
    const float ref0 = mn0 == -INFINITY ? 0.f : mn0, ref1 = mn1 == -INFINITY ? 0.f : mn1;
    const float a0 = exp2f(m0 - ref0), a1 = exp2f(m1 - ref1);
    m0 = mn0;
    m1 = mn1;
    float rs0 = 0.f, rs1 = 0.f;
    uint32_t pf[4][4];  // P as A fragments: 4 k-steps of 16 keys
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      const float p0 = exp2f(fmaf(s[nt][0], p.scale_log2, -ref0));
      const float p1 = exp2f(fmaf(s[nt][1], p.scale_log2, -ref0));
      const float p2 = exp2f(fmaf(s[nt][2], p.scale_log2, -ref1));
      const float p3 = exp2f(fmaf(s[nt][3], p.scale_log2, -ref1));
      rs0 += p0 + p1;
      rs1 += p2 + p3;
      pf[nt >> 1][(nt & 1) * 2] = Elem<DT>::pack(p0, p1);
      pf[nt >> 1][(nt & 1) * 2 + 1] = Elem<DT>::pack(p2, p3);
    }
    l0 = l0 * a0 + rs0;
    l1 = l1 * a1 + rs1;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      o[i][0] *= a0;
      o[i][1] *= a0;
      o[i][2] *= a1;
      o[i][3] *= a1;
    }
    // ---- O += P V ----
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
      for (int dp = 0; dp < 8; ++dp) {  // pairs of n8 tiles along head_dim
        uint32_t bf[4];
        const int r = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        const int cc = dp * 2 + (lane >> 4);
        ldmatrix_x4_trans(bf, smem_u32(vs_ + swz_off(r, cc)));
        mma16816<DT>(o[dp * 2], pf[kk], bf[0], bf[1]);
        mma16816<DT>(o[dp * 2 + 1], pf[kk], bf[2], bf[3]);
      }
    }
    __syncthreads();  // this stage may be overwritten by the load issued in the next iteration
  }
  cp_async_wait<0>();

  // ---- finalise: O / l ----
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float i0 = l0 > 0.f ? 1.f / l0 : 0.f, i1 = l1 > 0.f ? 1.f / l1 : 0.f;
  T* ob = static_cast<T*>(p.out) + b * p.o_sb + h * p.o_sh;
  const int r0 = row0 + warp * 16 + (lane >> 2), r1 = r0 + 8;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int d = i * 8 + (lane & 3) * 2;
    if (r0 < p.sq) *reinterpret_cast<uint32_t*>(ob + (int64_t)r0 * p.o_ss + d) = Elem<DT>::pack(o[i][0] * i0, o[i][1] * i0);
    if (r1 < p.sq) *reinterpret_cast<uint32_t*>(ob + (int64_t)r1 * p.o_ss + d) = Elem<DT>::pack(o[i][2] * i1, o[i][3] * i1);
  }
}

template <int DT, int PQ>
static int launch_attn_pq(const AttnParams& p, int batch, cudaStream_t stream) {
  constexpr size_t smem = attn_smem_bytes<PQ>();
  // per-device attribute; setting it on every launch keeps multi-device processes correct
  if (cudaFuncSetAttribute(sparse_attn_kernel<DT, PQ>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
    return VA_ERR_CUDA;
  dim3 grid(p.nq, p.heads, batch);
  sparse_attn_kernel<DT, PQ><<<grid, PQ * 2, smem, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? VA_OK : VA_ERR_CUDA;
}

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
  p.heads = a.heads; p.rep = a.heads / a.kv_heads; p.sq = a.sq; p.sk = a.sk;
  p.nq = (a.sq + a.pq - 1) / a.pq;
  p.causal = a.causal; p.q_offset = a.q_offset;
  const float scale = a.softmax_scale > 0.f ? a.softmax_scale : 0.08838834764831845f;
  p.scale_log2 = scale * 1.4426950408889634f;
  if (a.dtype == VA_BF16)
    return a.pq == 64 ? launch_attn_pq<VA_BF16, 64>(p, a.batch, stream) : launch_attn_pq<VA_BF16, 128>(p, a.batch, stream);
  return a.pq == 64 ? launch_attn_pq<VA_FP16, 64>(p, a.batch, stream) : launch_attn_pq<VA_FP16, 128>(p, a.batch, stream);
}

}  // namespace va
