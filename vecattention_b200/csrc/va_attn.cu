// Vector-sparse flash attention on tcgen05: one CTA per query tile, keys taken 128 at a time from
// the tile's dense 64-key blocks and then from its selected-column list (row gather).
//
// Warp roles (288 threads, one CTA per SM):
//   warps 0-3  softmax: thread t owns accumulator row t (TMEM lane t).  Per chunk it reads its row
//              of S = Q K^T from tensor memory, keeps the running maximum / sum (exp2 domain, the
//              maximum is raised lazily: only when a chunk exceeds it by more than 2^8), writes
//              P in the input dtype to shared memory and rescales its row of O when the maximum
//              moved.
//   warp  4    MMA issuer (one thread): S_j = Q K_j^T and O += P_j V_j as tcgen05.mma with fp32
//              accumulators in tensor memory; S is double buffered so that S_{j+1} is computed
//              while the softmax of chunk j runs.
//   warps 5-8  gather producers: cp.async 16-byte pieces of the selected K and V rows into a
//              two-stage ring of 128-byte-swizzled operand tiles; copy completion is reported to
//              the stage's mbarrier asynchronously, so the producers never wait for their own loads.
// All hand-offs are mbarriers; every wait is bounded (sm100::mbar_wait) and a timeout sets
// VA_STATUS_TIMEOUT in the status word and unwinds the CTA.
//
// The MMA tile is always 128 rows: with q_pooling_size 64 the upper 64 rows are zero queries.
#include "va_common.cuh"
#include "va_sm100.cuh"
#include "va_attn.cuh"

namespace va {

using namespace sm100;

int launch_attn64(const AttnParams& p, int dtype, int batch, cudaStream_t stream);  // va_attn64.cu

constexpr int kChunk = 128;                // keys per step
constexpr int kTileBytes = 128 * 256;      // one 128-row operand tile (two 16 KB halves)
constexpr int kStages = 2;
constexpr int kAttnThreads = 288;
constexpr size_t kAttnSmem = 1024 + (size_t)kTileBytes * (1 + 2 * kStages + 1);  // Q, K/V ring, P
constexpr float kRescaleThreshold = 8.0f;  // log2 units

struct AttnBarriers {
  uint64_t qfull, kfull[kStages], kempty[kStages], vfull[kStages], vempty[kStages];
  uint64_t sfull[2], sempty[2], pfull, pempty, ofull;
};

template <int DT, int PQ>
__global__ void __launch_bounds__(kAttnThreads, 1) sparse_attn_kernel(const AttnParams p) {
  using T = typename Elem<DT>::T;
  extern __shared__ unsigned char smem_raw[];
  __shared__ AttnBarriers bars;
  __shared__ uint32_t tmem_base_s;
  __shared__ int keys_s[4][kChunk];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // causal tiles grow with their index: the longest are started first, so the grid's tail is made of short ones
  const int tile = p.causal ? (int)(gridDim.x - 1 - blockIdx.x) : (int)blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int hkv = h / p.rep;
  const int row0 = tile * PQ;
  const int64_t trow = ((int64_t)b * p.heads + h) * p.nq + tile;
  const int nblk = p.blk_count ? __ldg(p.blk_count + trow) : 0;
  const int ncol = __ldg(p.col_count + trow);
  const int nslots = nblk * 64 + ncol;
  const int nchunks = (nslots + kChunk - 1) / kChunk;
  T* ob = static_cast<T*>(p.out) + b * p.o_sb + h * p.o_sh;

  if (nchunks == 0) {  // no key at all: the tile's output is zero
    for (int i = tid; i < PQ * 16; i += kAttnThreads) {
      const int r = i >> 4, c = i & 15;
      if (row0 + r < p.sq) *reinterpret_cast<uint4*>(ob + (int64_t)(row0 + r) * p.o_ss + c * 8) = make_uint4(0, 0, 0, 0);
    }
    if (p.lse && tid < PQ && row0 + tid < p.sq) p.lse[((int64_t)b * p.heads + h) * p.sq + row0 + tid] = -INFINITY;
    return;
  }

  unsigned char* smem = smem_raw + ((1024u - (smem_addr(smem_raw) & 1023u)) & 1023u);
  unsigned char* q_s = smem;
  unsigned char* kv_s = smem + kTileBytes;                      // [stage][K|V]
  unsigned char* p_s = smem + kTileBytes * (1 + 2 * kStages);

  if (tid == 0) {
    mbar_init(&bars.qfull, 256);  // per producer thread: one asynchronous copy-completion arrival + one plain arrival
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&bars.kfull[s], 256);
      mbar_init(&bars.vfull[s], 256);
      mbar_init(&bars.kempty[s], 1);
      mbar_init(&bars.vempty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars.sfull[s], 1);
      mbar_init(&bars.sempty[s], 128);
    }
    mbar_init(&bars.pfull, 128);
    mbar_init(&bars.pempty, 1);
    mbar_init(&bars.ofull, 1);
    fence_proxy_async();
  }
  if (warp == 4) {
    tmem_alloc(&tmem_base_s, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  const uint32_t t_s0 = tmem, t_o = tmem + 256;  // S buffers at columns 0 and 128, O at 256

  bool timed_out = false;

  if (warp >= 5) {
    // ======================= gather producers =======================
    const int pt = tid - 160;
    const T* qb = static_cast<const T*>(p.q) + b * p.q_sb + h * p.q_sh;
    const T* kb = static_cast<const T*>(p.k) + b * p.k_sb + hkv * p.k_sh;
    const T* vb = static_cast<const T*>(p.v) + b * p.v_sb + hkv * p.v_sh;
    const int32_t* blk = p.blk_idx + trow * p.blk_stride;
    const int32_t* col = p.col_idx + trow * p.col_stride;
    // Q tile (rows beyond the tile or the sequence are zero)
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int pce = pt + i * 128, r = pce >> 4, c = pce & 15;
      const bool ok = r < PQ && row0 + r < p.sq;
      cp_async16(smem_addr(q_s + tile_off(128, r, c)), qb + (int64_t)(ok ? row0 + r : 0) * p.q_ss + c * 8, ok);
    }
    // completion of this thread's copies is reported to the barrier asynchronously (no wait here);
    // the plain arrive that follows releases the thread's ordinary shared-memory stores
    cp_async_arrive_noinc(&bars.qfull);
    mbar_arrive(&bars.qfull);
    // Index loads are issued one chunk ahead as a batch of independent non-coherent loads, so their
    // latency overlaps the copies of the current chunk instead of preceding them.
    auto load_keys = [&](int j, int (&raw)[16]) {
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const int slot = j * kChunk + (pt >> 4) + 8 * i;
        const int ci = min(max(slot - nblk * 64, 0), max(ncol - 1, 0));
        const int32_t* src = slot < nblk * 64 ? blk + (slot >> 6) : col + ci;
        raw[i] = ldg_nc(src);
      }
    };
    int raw[16];
    load_keys(0, raw);
    for (int j = 0; j < nchunks && !timed_out; ++j) {
      const int s = j % kStages, u = j / kStages;
      int keys[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const int slot = j * kChunk + (pt >> 4) + 8 * i;
        const int key = slot < nblk * 64 ? raw[i] + (slot & 63) : (slot < nslots ? raw[i] : -1);
        keys[i] = (key >= 0 && key < p.sk) ? key : -1;
      }
      if (j + 1 < nchunks) load_keys(j + 1, raw);
      if ((pt & 15) == 0) {
#pragma unroll
        for (int i = 0; i < 16; ++i) keys_s[j & 3][(pt >> 4) + 8 * i] = keys[i];
      }
#pragma unroll
      for (int kv = 0; kv < 2; ++kv) {
        uint64_t* empty = kv ? &bars.vempty[s] : &bars.kempty[s];
        uint64_t* full = kv ? &bars.vfull[s] : &bars.kfull[s];
        if (!mbar_wait(empty, (u & 1) ^ 1)) { timed_out = true; break; }
        unsigned char* dst = kv_s + (size_t)(s * 2 + kv) * kTileBytes;
        const T* base = kv ? vb : kb;
        const int64_t stride = kv ? p.v_ss : p.k_ss;
        const int c = pt & 15;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const int r = (pt >> 4) + 8 * i;
          const bool ok = keys[i] >= 0;
          cp_async16(smem_addr(dst + tile_off(128, r, c)), base + (int64_t)(ok ? keys[i] : 0) * stride + c * 8, ok);
        }
        cp_async_arrive_noinc(full);
        mbar_arrive(full);
      }
    }
    cp_async_commit();
    cp_async_wait<0>();  // nothing of this thread may still be in flight when the CTA retires
  } else if (warp == 4) {
    // ======================= MMA issuer =======================
    if (lane == 0) {
      constexpr uint32_t in16 = DT == VA_BF16 ? 1u : 0u;
      constexpr uint32_t idesc_s = umma_idesc(128, 128, in16, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc(128, 128, in16, 0, 1);
      const uint32_t q_addr = smem_addr(q_s), p_addr = smem_addr(p_s), kv_addr = smem_addr(kv_s);
      auto issue_s = [&](int j) -> bool {
        const int s = j % kStages, u = j / kStages, sb = j & 1, ub = j >> 1;
        if (!mbar_wait(&bars.kfull[s], u & 1)) return false;
        if (!mbar_wait(&bars.sempty[sb], (ub & 1) ^ 1)) return false;
        fence_proxy_async();
        tc_fence_after();
        const uint32_t k_addr = kv_addr + (uint32_t)(s * 2) * kTileBytes;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t off = (uint32_t)(ks >> 2) * (128 * 128) + (uint32_t)(ks & 3) * 32;
          umma(t_s0 + (uint32_t)sb * 128, umma_desc(q_addr + off, 16, 1024), umma_desc(k_addr + off, 16, 1024), idesc_s,
               ks > 0);
        }
        umma_commit(&bars.kempty[s]);
        umma_commit(&bars.sfull[sb]);
        return true;
      };
      auto issue_pv = [&](int j) -> bool {
        const int s = j % kStages, u = j / kStages;
        if (!mbar_wait(&bars.vfull[s], u & 1)) return false;
        if (!mbar_wait(&bars.pfull, j & 1)) return false;
        fence_proxy_async();
        tc_fence_after();
        const uint32_t v_addr = kv_addr + (uint32_t)(s * 2 + 1) * kTileBytes;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t poff = (uint32_t)(ks >> 2) * (128 * 128) + (uint32_t)(ks & 3) * 32;
          umma(t_o, umma_desc(p_addr + poff, 16, 1024), umma_desc(v_addr + (uint32_t)ks * 16 * 128, 128 * 128, 1024),
               idesc_pv, (j > 0 || ks > 0) ? 1u : 0u);
        }
        umma_commit(&bars.vempty[s]);
        umma_commit(&bars.pempty);
        if (j == nchunks - 1) umma_commit(&bars.ofull);
        return true;
      };
      bool ok = mbar_wait(&bars.qfull, 0);
      if (ok) ok = issue_s(0);
      for (int j = 0; j < nchunks && ok; ++j) {
        if (j + 1 < nchunks) ok = issue_s(j + 1);
        if (ok) ok = issue_pv(j);
      }
      timed_out = !ok;
    }
  } else {
    // ======================= softmax / correction / epilogue =======================
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    const int row = tid;
    const int qpos = p.q_offset + row0 + row;
    float m_used = -INFINITY, l = 0.f;
    const float sc = p.scale_log2;
    for (int j = 0; j < nchunks && !timed_out; ++j) {
      const int sb = j & 1, ub = j >> 1;
      const bool masked = p.causal || j == nchunks - 1 || j * kChunk < nblk * 64;
      const int* keys = keys_s[j & 3];
      if (!mbar_wait(&bars.sfull[sb], ub & 1)) { timed_out = true; break; }
      tc_fence_after();
      const uint32_t t_s = t_s0 + (uint32_t)sb * 128 + lane_base;
      // ---- pass 1: row maximum of the chunk ----
      float mx = -INFINITY;
#pragma unroll 1
      for (int qd = 0; qd < 4; ++qd) {
        uint32_t v[32];
        tmem_ld32(t_s + qd * 32, v);
        tmem_wait_ld();
        if (masked) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int key = keys[qd * 32 + i];
            const bool drop = key < 0 || (p.causal && key > qpos);
            mx = fmaxf(mx, drop ? -INFINITY : __uint_as_float(v[i]));
          }
        } else {
          float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
          for (int i = 0; i < 32; ++i) m4[i & 3] = fmaxf(m4[i & 3], __uint_as_float(v[i]));
          mx = fmaxf(mx, fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])));
        }
      }
      const float mx_s = mx * sc;
      const bool grow = mx_s > m_used + kRescaleThreshold || (m_used == -INFINITY && mx_s > -INFINITY);
      const float m_new = grow ? mx_s : m_used;
      const bool rescale = __any_sync(0xffffffffu, grow && j > 0);
      // P buffer free <=> the PV product of the previous chunk has completed, so O is quiescent
      if (!mbar_wait(&bars.pempty, (j & 1) ^ 1)) { timed_out = true; break; }
      if (rescale) {
        tc_fence_after();
        const float alpha = grow ? ex2_approx(m_used - m_new) : 1.f;  // exp2(-inf) = 0 when nothing was accumulated yet
#pragma unroll 1
        for (int qd = 0; qd < 4; ++qd) {
          uint32_t v[32];
          tmem_ld32(t_o + lane_base + qd * 32, v);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
          tmem_st32(t_o + lane_base + qd * 32, v);
        }
        tmem_wait_st();
        l *= alpha;
      }
      m_used = m_new;
      const float mref = m_used == -INFINITY ? 0.f : m_used;
      // ---- pass 2: P = exp2(S * scale - m), row sum, P -> shared memory ----
#pragma unroll 1
      for (int qd = 0; qd < 4; ++qd) {
        uint32_t v[32];
        tmem_ld32(t_s + qd * 32, v);
        tmem_wait_ld();
        uint32_t pk[16];
        float l0 = 0.f, l1 = 0.f;
        if (masked) {  // kept out of the arithmetic loop: a branch per element pair would serialise it
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int key = keys[qd * 32 + i];
            if (key < 0 || (p.causal && key > qpos)) v[i] = 0xff800000u;  // -inf
          }
        }
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float p0 = ex2_approx(fmaf(__uint_as_float(v[i]), sc, -mref));
          const float p1 = ex2_approx(fmaf(__uint_as_float(v[i + 1]), sc, -mref));
          l0 += p0;
          l1 += p1;
          pk[i >> 1] = Elem<DT>::pack(p0, p1);
        }
        l += l0 + l1;
#pragma unroll
        for (int c = 0; c < 4; ++c)
          *reinterpret_cast<uint4*>(p_s + tile_off(128, row, qd * 4 + c)) =
              make_uint4(pk[c * 4], pk[c * 4 + 1], pk[c * 4 + 2], pk[c * 4 + 3]);
      }
      tc_fence_before();
      mbar_arrive(&bars.sempty[sb]);
      fence_proxy_async();
      mbar_arrive(&bars.pfull);
    }
    // ---- epilogue: O / l -> global ----
    if (!timed_out && mbar_wait(&bars.ofull, 0)) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      const bool row_ok = row < PQ && row0 + row < p.sq;
      if (p.lse && row_ok)  // m_used is in the exp2 domain
        p.lse[((int64_t)b * p.heads + h) * p.sq + row0 + row] = l > 0.f ? (m_used + log2f(l)) * 0.6931471805599453f : -INFINITY;
      T* orow = ob + (int64_t)(row0 + (row_ok ? row : 0)) * p.o_ss;
#pragma unroll 1
      for (int qd = 0; qd < 4; ++qd) {
        uint32_t v[32];
        tmem_ld32(t_o + lane_base + qd * 32, v);
        tmem_wait_ld();
        if (row_ok) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint4 w;
            w.x = Elem<DT>::pack(__uint_as_float(v[c * 8 + 0]) * inv, __uint_as_float(v[c * 8 + 1]) * inv);
            w.y = Elem<DT>::pack(__uint_as_float(v[c * 8 + 2]) * inv, __uint_as_float(v[c * 8 + 3]) * inv);
            w.z = Elem<DT>::pack(__uint_as_float(v[c * 8 + 4]) * inv, __uint_as_float(v[c * 8 + 5]) * inv);
            w.w = Elem<DT>::pack(__uint_as_float(v[c * 8 + 6]) * inv, __uint_as_float(v[c * 8 + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + qd * 32 + c * 8) = w;
          }
        }
      }
    } else {
      timed_out = true;
    }
  }
  if (timed_out && p.status) atomicOr(p.status, VA_STATUS_TIMEOUT);
  tc_fence_before();
  __syncthreads();
  if (warp == 4) tmem_dealloc(tmem, 512);
}

template <int DT, int PQ>
static int launch_attn_pq(const AttnParams& p, int batch, cudaStream_t stream) {
  // per-device attribute; setting it on every launch keeps multi-device processes correct
  if (cudaFuncSetAttribute(sparse_attn_kernel<DT, PQ>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kAttnSmem) !=
      cudaSuccess)
    return VA_ERR_CUDA;
  dim3 grid(p.nq, p.heads, batch);
  sparse_attn_kernel<DT, PQ><<<grid, kAttnThreads, kAttnSmem, stream>>>(p);
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
  p.status = a.status;
  p.lse = a.lse;
  p.heads = a.heads; p.rep = a.heads / a.kv_heads; p.sq = a.sq; p.sk = a.sk;
  p.nq = (a.sq + a.pq - 1) / a.pq;
  p.causal = a.causal; p.q_offset = a.q_offset;
  const float scale = a.softmax_scale > 0.f ? a.softmax_scale : 0.08838834764831845f;
  p.scale_log2 = scale * 1.4426950408889634f;
  if (a.pq == 64) return launch_attn64(p, a.dtype, a.batch, stream);
  return a.dtype == VA_BF16 ? launch_attn_pq<VA_BF16, 128>(p, a.batch, stream)
                            : launch_attn_pq<VA_FP16, 128>(p, a.batch, stream);
}

}  // namespace va
