// Important-vector selection: pooled-Q . K^T estimate + streaming MinP threshold + compaction.
//
// Work decomposition.  The pooled rows of all query heads that share one KV head form one row
// list (row R -> head hkv*rep + R/nq, tile R%nq); a CTA owns 128 consecutive rows of that list and
// walks the keys of its KV head once, tile by tile, in ascending order.  Because one CTA sees all
// keys of its rows in order, the running (prefix) maximum of a key-block group is a per-thread
// register, every row's index list comes out ascending and deterministic, and no atomics, no
// zero-filled buffers and no second pass are needed.
//
// Per key tile (BN keys): the four warps compute the 128 x BN estimate tile with mma.sync
// (A = scaled pooled Q held in registers, B = the K tile staged in swizzled shared memory by
// cp.async, double buffered) and park it in shared memory; then thread r walks row r of the tile
// block by block (BK keys): block maximum -> running maximum -> keep test -> append.
#include "va_common.cuh"

namespace va {

struct SelectParams {
  const void* avg_q;  // (B,H,nq,D)
  const void* k;
  int64_t k_sb, k_sh, k_ss;
  const float* gaps;
  int64_t gaps_sb;
  float gap;
  int32_t* col_count;
  int32_t* col_idx;
  int64_t capacity;
  int32_t* status;
  int heads, kv_heads, rep, nq, sk;
  int pq, group_k_block;
  int causal, wo_initial, compat_bsq, tile_offset;
};

constexpr int kSelRows = 128;  // pooled rows per CTA

template <int BK> struct SelTile { static constexpr int BN = BK < 64 ? 64 : BK; };

template <int BK> constexpr size_t select_smem_bytes() {
  constexpr int BN = SelTile<BK>::BN;
  return (size_t)kSelRows * 256        // scaled pooled Q
         + 2 * (size_t)BN * 256        // K tile, two stages
         + (size_t)kSelRows * (BN + 1) * 4;  // estimate tile
}

template <int DT, int BK>
__global__ void __launch_bounds__(128) select_kernel(const SelectParams p) {
  using T = typename Elem<DT>::T;
  constexpr int BN = SelTile<BK>::BN;
  constexpr int SS = BN + 1;  // row stride of the estimate tile (floats), odd => conflict-free row walk
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* q_s = smem;
  unsigned char* k_s = smem + kSelRows * 256;
  float* s_s = reinterpret_cast<float*>(smem + kSelRows * 256 + 2 * BN * 256);
  __shared__ int s_khi[4];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int hkv = blockIdx.y, b = blockIdx.z;
  const int nrows = p.rep * p.nq;
  const int row_base = blockIdx.x * kSelRows;

  // ---- per-row state (thread r owns row r of the CTA) ----
  const int R = row_base + tid;
  const bool row_ok = R < nrows;
  const int h = hkv * p.rep + (row_ok ? R / p.nq : 0);
  const int tile = row_ok ? R % p.nq : 0;
  const int lo = p.wo_initial ? p.pq : 0;
  int hi = 0;
  if (row_ok) {
    if (!p.causal) {
      hi = p.sk;
    } else {
      const int64_t g = (int64_t)p.tile_offset + tile;
      int64_t lim = g * p.pq;
      if (p.compat_bsq > 0 && (tile % p.compat_bsq) == 0) {
        int64_t q1 = (g - 1) * p.pq + BK;
        lim = q1 < lim ? q1 : lim;
      }
      lim = lim < p.sk ? lim : p.sk;
      hi = lim > 0 ? (int)lim : 0;
    }
  }
  const float gap = p.gaps ? __ldg(p.gaps + b * p.gaps_sb + h) : p.gap;
  const int64_t out_row = ((int64_t)b * p.heads + h) * p.nq + tile;
  int32_t* idx_out = p.col_idx + out_row * p.capacity;
  int cnt = 0;
  float run_max = -INFINITY;

  // CTA-wide key range [k_lo, k_hi)
  int whi = hi;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) whi = max(whi, __shfl_xor_sync(0xffffffffu, whi, o));
  if (lane == 0) s_khi[warp] = whi;

  // ---- scaled pooled Q -> shared (q~ = round(fp32(q_bar) * fp32(1/sqrt(D)))) ----
  {
    const float scale = 0.08838834764831845f;  // fp32(1/sqrt(128))
    const T* aq = static_cast<const T*>(p.avg_q);
    for (int i = tid; i < kSelRows * 16; i += 128) {
      const int r = i >> 4, c = i & 15;
      const int RR = row_base + r;
      uint4 w = make_uint4(0, 0, 0, 0);
      if (RR < nrows) {
        const int hh = hkv * p.rep + RR / p.nq, tt = RR % p.nq;
        w = __ldg(reinterpret_cast<const uint4*>(aq + (((int64_t)b * p.heads + hh) * p.nq + tt) * kHeadDim + c * 8));
        uint32_t* ww = reinterpret_cast<uint32_t*>(&w);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 f = Elem<DT>::unpack(ww[j]);
          ww[j] = Elem<DT>::pack(__fmul_rn(f.x, scale), __fmul_rn(f.y, scale));
        }
      }
      *reinterpret_cast<uint4*>(q_s + swz_off(r, c)) = w;
    }
  }
  __syncthreads();
  const int k_hi = max(max(s_khi[0], s_khi[1]), max(s_khi[2], s_khi[3]));
  const int t_lo = lo / BN;
  const int t_hi = (k_hi + BN - 1) / BN;  // exclusive

  // ---- A fragments: rows 32*warp .. +31, two m16 tiles, 8 k-steps ----
  uint32_t qf[2][8][4];
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      const int r = warp * 32 + mt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
      const int c = ks * 2 + (lane >> 4);
      ldmatrix_x4(qf[mt][ks], smem_u32(q_s + swz_off(r, c)));
    }

  const T* kbase = static_cast<const T*>(p.k) + b * p.k_sb + hkv * p.k_sh;
  auto load_k_tile = [&](int t, int stage) {
    unsigned char* dst = k_s + stage * BN * 256;
    const int key0 = t * BN;
#pragma unroll
    for (int i = 0; i < BN * 16 / 128; ++i) {
      const int pce = tid + i * 128;
      const int r = pce >> 4, c = pce & 15;
      const int key = key0 + r;
      const bool ok = key < p.sk;
      cp_async16(smem_u32(dst + swz_off(r, c)), kbase + (int64_t)(ok ? key : 0) * p.k_ss + c * 8, ok);
    }
  };

  if (t_lo < t_hi) load_k_tile(t_lo, 0);
  cp_async_commit();

  for (int t = t_lo; t < t_hi; ++t) {
    const int stage = (t - t_lo) & 1;
    if (t + 1 < t_hi) load_k_tile(t + 1, stage ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();  // K tile t visible; previous tile's row walk finished

    const unsigned char* kt = k_s + stage * BN * 256;
#pragma unroll 1
    for (int nc = 0; nc < BN / 64; ++nc) {
      float acc[2][8][4];
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) acc[mt][nt][e] = 0.f;
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
#pragma unroll
        for (int np = 0; np < 4; ++np) {  // pairs of n8 tiles
          uint32_t bf[4];
          const int r = nc * 64 + np * 16 + (lane & 7) + (lane >> 4) * 8;
          const int c = ks * 2 + ((lane >> 3) & 1);
          ldmatrix_x4(bf, smem_u32(kt + swz_off(r, c)));
#pragma unroll
          for (int mt = 0; mt < 2; ++mt) {
            mma16816<DT>(acc[mt][np * 2], qf[mt][ks], bf[0], bf[1]);
            mma16816<DT>(acc[mt][np * 2 + 1], qf[mt][ks], bf[2], bf[3]);
          }
        }
      }
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
          const int r = warp * 32 + mt * 16 + (lane >> 2);
          const int c = nc * 64 + nt * 8 + (lane & 3) * 2;
          s_s[r * SS + c] = acc[mt][nt][0];
          s_s[r * SS + c + 1] = acc[mt][nt][1];
          s_s[(r + 8) * SS + c] = acc[mt][nt][2];
          s_s[(r + 8) * SS + c + 1] = acc[mt][nt][3];
        }
    }
    __syncthreads();  // estimate tile complete

    // ---- row walk: thread tid owns row tid ----
    const float* srow = s_s + tid * SS;
    const int key_t = t * BN;
#pragma unroll 1
    for (int blk = 0; blk < BN / BK; ++blk) {
      const int key0 = key_t + blk * BK;
      if (key0 < lo) continue;
      if (key0 >= k_hi) break;
      if (((key0 / BK) % p.group_k_block) == 0) run_max = -INFINITY;  // a new key-block group starts
      const float* sv = srow + blk * BK;
      float bmax = -INFINITY;
      if (key0 + BK <= p.sk) {
#pragma unroll
        for (int j = 0; j < BK; ++j) bmax = fmaxf(bmax, sv[j]);
      } else {
        for (int j = 0; j < BK; ++j)
          if (key0 + j < p.sk) bmax = fmaxf(bmax, sv[j]);
      }
      run_max = fmaxf(run_max, bmax);
      if (key0 < hi) {
        const int jn = min(BK, hi - key0);
        for (int j = 0; j < jn; ++j) {
          if (__fadd_rn(sv[j], gap) >= run_max) {
            if (cnt < p.capacity) idx_out[cnt] = key0 + j;
            ++cnt;
          }
        }
      }
    }
  }
  cp_async_wait<0>();
  if (row_ok) {
    p.col_count[out_row] = cnt;
    if (cnt > p.capacity && p.status) atomicOr(p.status, VA_STATUS_OVERFLOW);
  }
}

template <int DT, int BK>
static int launch_select_bk(const SelectParams& p, int batch, cudaStream_t stream) {
  constexpr size_t smem = select_smem_bytes<BK>();
  // per-device attribute; setting it on every launch keeps multi-device processes correct
  if (cudaFuncSetAttribute(select_kernel<DT, BK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
    return VA_ERR_CUDA;
  const int nrows = p.rep * p.nq;
  dim3 grid((nrows + kSelRows - 1) / kSelRows, p.kv_heads, batch);
  select_kernel<DT, BK><<<grid, 128, smem, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? VA_OK : VA_ERR_CUDA;
}

template <int DT>
static int launch_select_dt(const SelectParams& p, int bk, int batch, cudaStream_t stream) {
  switch (bk) {
    case 16: return launch_select_bk<DT, 16>(p, batch, stream);
    case 32: return launch_select_bk<DT, 32>(p, batch, stream);
    case 64: return launch_select_bk<DT, 64>(p, batch, stream);
    case 128: return launch_select_bk<DT, 128>(p, batch, stream);
    default: return VA_ERR_SHAPE;
  }
}

int select(const va_select_args& a, cudaStream_t stream) {
  SelectParams p;
  p.avg_q = a.avg_q;
  p.k = a.k.ptr;
  p.k_sb = a.k.stride_b;
  p.k_sh = a.k.stride_h;
  p.k_ss = a.k.stride_s;
  p.gaps = a.gaps;
  p.gaps_sb = a.gaps_stride_b;
  p.gap = a.gap;
  p.col_count = a.col_count;
  p.col_idx = a.col_idx;
  p.capacity = a.capacity;
  p.status = a.status;
  p.heads = a.heads;
  p.kv_heads = a.kv_heads;
  p.rep = a.heads / a.kv_heads;
  p.nq = a.nq;
  p.sk = a.sk;
  p.pq = a.pq;
  p.group_k_block = a.group_k_block;
  p.causal = a.causal;
  p.wo_initial = a.wo_initial;
  p.compat_bsq = a.compat_bsq;
  p.tile_offset = a.tile_offset;
  return a.dtype == VA_BF16 ? launch_select_dt<VA_BF16>(p, a.bk, a.batch, stream)
                            : launch_select_dt<VA_FP16>(p, a.bk, a.batch, stream);
}

}  // namespace va
