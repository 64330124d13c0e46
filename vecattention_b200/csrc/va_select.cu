// Important-vector selection: pooled-Q . K^T estimate + streaming MinP threshold + compaction,
// with the estimate on tcgen05 tensor cores and the accumulator in tensor memory.
//
// Work decomposition.  The pooled rows of all query heads that share one KV head form one row
// list (row R -> head hkv*rep + R/nq, tile R%nq); a CTA owns 128 consecutive rows of that list and
// walks the keys of its KV head once, 128 keys per tile, in ascending order.  Because one CTA sees
// all keys of its rows in order, the running (prefix) maximum of a key-block group is a per-thread
// register, every row's index list comes out ascending and deterministic, and no atomics, no
// zero-filled buffers and no second pass are needed.
//
// Warp roles (672 threads, one CTA per SM):
//   warps 0-15  row walkers: pooled row r = TMEM lane r is owned by four threads, one per 32-key
//              quarter of the tile (warp w walks quarter w / 4 of the rows of lane quarter w % 4,
//              the only lanes it can reach).  Per tile each pulls its 32 estimates into registers
//              and forms the maxima of its key blocks; the four swap them through shared memory,
//              so all know the running maximum entering every block; each builds the keep mask
//              fp32(s + gap) >= m of its quarter; the counts travel with the next tile's maxima
//              (one meeting per tile), after which each appends its kept keys at its own offset of
//              the row's list.
//              (Blocks of 64 or 128 keys span two or four quarters: their maximum is formed from the
//              quarters' published maxima.)
//   warps 16-19 producers: cp.async the next K tile (128 contiguous key rows) into a 4-stage ring
//              of 128-byte-swizzled operand tiles; completion is reported to the stage's mbarrier.
//   warp  20   MMA issuer (one thread): S_t = Q~ K_t^T, 128 x 128 x 128 as eight tcgen05.mma, into
//              one of two 128-column accumulator buffers in tensor memory.
// All hand-offs are mbarriers with bounded waits; a timeout sets VA_STATUS_TIMEOUT.
#include "va_common.cuh"
#include "va_sm100.cuh"

namespace va {

using namespace sm100;

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
  int causal, wo_initial, compat_bsq, tile_offset, chunk_tiles;
};

namespace {

constexpr int kRows = 128;   // pooled rows per CTA
constexpr int kTile = 128;   // keys per tile
constexpr int kTileBytes = 128 * 256;
constexpr int kStages = 4;
constexpr int kThreads = 672;
constexpr int kWalkerWarps = 16;
constexpr size_t kSmem = 1024 + (size_t)kTileBytes * (1 + kStages);

struct Barriers {
  uint64_t kfull[kStages], kempty[kStages], sfull[2], sempty[2], quad[4];
};

// per-row walking state
struct Row {
  float run_max, gap;
  int cnt, hi;
  int32_t* out;
};

// 4-byte global store executed only where `pred` is true, without a branch
__device__ __forceinline__ void st_global_if(int32_t* ptr, int value, bool pred) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %2, 0;\n\t@p st.global.b32 [%0], %1;\n\t}" ::"l"(ptr), "r"(value), "r"((int)pred)
               : "memory");
}

// three-input maximum (one instruction)
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
// maximum of N estimates (N = 16 or 32) as two chains of three-input maxima
template <int N>
__device__ __forceinline__ float max_of(const uint32_t* v) {
  float a = __uint_as_float(v[0]), b = __uint_as_float(v[1]);
  int i = 2;
#pragma unroll
  for (; i + 3 < N; i += 4) {
    a = fmax3(a, __uint_as_float(v[i]), __uint_as_float(v[i + 1]));
    b = fmax3(b, __uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
  }
  if (i + 1 < N) a = fmax3(a, __uint_as_float(v[i]), __uint_as_float(v[i + 1]));
  return fmaxf(a, b);
}

// Running maximum for the walker of key quarter CQ on a tile that lies wholly inside the walked key
// range: only the blocks up to its own last one are visited (the thread of the last quarter ends
// with the value the next tile starts from and publishes it).  pm = own block maxima, xq = the
// row's published maxima [quarter][block][lane stride 32], gpos = position of the tile's first
// block inside its group of G blocks.
template <int BK, int CQ>
__device__ __forceinline__ void prefix_interior(const float* pm, const float* xq, float& run_max, int gpos, int G, float* rm_own) {
  constexpr int NP = BK < 32 ? 32 / BK : 1;
  constexpr int QPB = BK <= 32 ? 1 : BK / 32;                   // key quarters per block (blocks of 64 or 128 keys span several)
  constexpr int LAST = BK <= 32 ? (CQ + 1) * NP : CQ / QPB + 1;  // blocks up to and including my last
#pragma unroll
  for (int k = 0; k < LAST; ++k) {
    float m;
    bool mine;
    if (BK <= 32) {
      const int q = k / NP, kb = k % NP;
      mine = q == CQ;
      m = mine ? pm[kb] : xq[(q * 2 + kb) * 32];
    } else {  // the block spans QPB quarters
      mine = k == CQ / QPB;
      m = -INFINITY;
#pragma unroll
      for (int i = 0; i < QPB; ++i) {
        const int q = k * QPB + i;
        m = fmaxf(m, q == CQ ? pm[0] : xq[(q * 2) * 32]);
      }
    }
    if (gpos == 0) run_max = -INFINITY;  // a new key-block group starts
    gpos = gpos + 1 == G ? 0 : gpos + 1;
    run_max = fmaxf(run_max, m);
    if (mine) rm_own[BK <= 32 ? k % NP : 0] = run_max;
  }
}

template <int DT, int BK>
__global__ void __launch_bounds__(kThreads, 1) select_kernel(const SelectParams p) {
  using T = typename Elem<DT>::T;
  extern __shared__ unsigned char smem_raw[];
  __shared__ Barriers bars;
  __shared__ uint32_t tmem_base_s;
  __shared__ int s_khi;
  // exchange areas of a row's four threads, double buffered by tile parity (the threads meet once per tile)
  __shared__ float xmax_s[2][4 * 4 * 2 * 32];  // [parity][lane quarter][key quarter][block][lane]: block maxima
  __shared__ float xrm_s[2][4 * 32];         // [parity][lane quarter][lane]: running maximum after the tile, from the thread of the last key quarter
  __shared__ int xcnt_s[2][4 * 4 * 32];      // [parity][lane quarter][key quarter][lane]: kept-key counts

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int hkv = blockIdx.y, b = blockIdx.z;
  const int nrows = p.rep * p.nq;
  // causal rows walk more keys the later their tile: the longest walks are started first
  const int row_base = (p.causal ? (int)(gridDim.x - 1 - blockIdx.x) : (int)blockIdx.x) * kRows;

  // ---- per-row state: walker threads (warps 0-15) own row (warp % 4) * 32 + lane ----
  const bool is_walker = warp < kWalkerWarps;
  const int wrow = (warp & 3) * 32 + lane;
  const int R = row_base + wrow;
  const bool row_ok = is_walker && R < nrows;
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
      const int tile_in_chunk = p.chunk_tiles > 0 ? tile % p.chunk_tiles : tile;
      if (p.compat_bsq > 0 && (tile_in_chunk % p.compat_bsq) == 0) {
        const int64_t q1 = (g - 1) * p.pq + BK;
        lim = q1 < lim ? q1 : lim;
      }
      lim = lim < p.sk ? lim : p.sk;
      hi = lim > 0 ? (int)lim : 0;
    }
  }
  const int64_t out_row = ((int64_t)b * p.heads + h) * p.nq + tile;

  if (tid == 0) s_khi = 0;
  __syncthreads();
  if (warp < 4) {
    int whi = hi;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) whi = max(whi, __shfl_xor_sync(0xffffffffu, whi, o));
    if (lane == 0) atomicMax(&s_khi, whi);
  }
  __syncthreads();
  const int k_hi = s_khi;                       // CTA-wide end of the key walk
  const int t_lo = lo / kTile;
  const int t_hi = (k_hi + kTile - 1) / kTile;  // exclusive
  if (t_lo >= t_hi || k_hi <= lo) {             // nothing selectable for any row of this CTA
    if (row_ok) p.col_count[out_row] = 0;
    return;
  }

  unsigned char* smem = smem_raw + ((1024u - (smem_addr(smem_raw) & 1023u)) & 1023u);
  unsigned char* q_s = smem;
  unsigned char* k_s = smem + kTileBytes;

  // ---- scaled pooled Q -> shared operand tile (q~ = round(fp32(q_bar) * fp32(1/sqrt(D)))) ----
  {
    const float scale = 0.08838834764831845f;  // fp32(1/sqrt(128))
    const T* aq = static_cast<const T*>(p.avg_q);
    for (int i = tid; i < kRows * 16; i += kThreads) {
      const int r = i >> 4, c = i & 15;
      const int RR = row_base + r;
      uint4 w = make_uint4(0, 0, 0, 0);
      if (RR < nrows) {
        const int hh = hkv * p.rep + RR / p.nq, tt = RR % p.nq;
        w = __ldg(reinterpret_cast<const uint4*>(aq + (((int64_t)b * p.heads + hh) * p.nq + tt) * kHeadDim + c * 8));
        uint32_t* ww = reinterpret_cast<uint32_t*>(&w);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = Elem<DT>::unpack(ww[j]);
          ww[j] = Elem<DT>::pack(__fmul_rn(f.x, scale), __fmul_rn(f.y, scale));
        }
      }
      *reinterpret_cast<uint4*>(q_s + tile_off(128, r, c)) = w;
    }
    fence_proxy_async();
  }
  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&bars.kfull[s], 256);  // per producer thread: asynchronous copy-completion arrival + plain arrival
      mbar_init(&bars.kempty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars.sfull[s], 1);
      mbar_init(&bars.sempty[s], kWalkerWarps * 32);
    }
    for (int s = 0; s < 4; ++s) mbar_init(&bars.quad[s], 128);
    fence_proxy_async();
  }
  if (warp == 20) {
    tmem_alloc(&tmem_base_s, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  bool timed_out = false;

  if (warp >= 16 && warp < 20) {
    // ======================= K tile producers =======================
    const int pw = warp - 16, hh = lane >> 4, c = lane & 15;
    const int rbase = 2 * pw + hh;  // this thread copies piece c of rows rbase + 8 i, i = 0..15
    const uint32_t dst_off = tile_off(128, rbase, c);
    const T* kbase = static_cast<const T*>(p.k) + b * p.k_sb + hkv * p.k_sh + c * 8;
    for (int t = t_lo; t < t_hi; ++t) {
      const int n = t - t_lo, s = n % kStages, u = n / kStages;
      if (!mbar_wait(&bars.kempty[s], (u & 1) ^ 1)) { timed_out = true; break; }
      const uint32_t dst = smem_addr(k_s + (size_t)s * kTileBytes) + dst_off;
      const int key0 = t * kTile + rbase;
      if (t * kTile + kTile <= p.sk) {
        const T* src = kbase + (int64_t)key0 * p.k_ss;
#pragma unroll
        for (int i = 0; i < 16; ++i) cp_async16_full(dst + i * 1024, src + (int64_t)(8 * i) * p.k_ss);
      } else {  // last tile: rows past the sequence re-read its last row (finite; the walker ignores them)
#pragma unroll
        for (int i = 0; i < 16; ++i)
          cp_async16_full(dst + i * 1024, kbase + (int64_t)min(key0 + 8 * i, p.sk - 1) * p.k_ss);
      }
      cp_async_arrive_noinc(&bars.kfull[s]);
      mbar_arrive(&bars.kfull[s]);
    }
    cp_async_commit();
    cp_async_wait<0>();  // nothing of this thread may still be in flight when the CTA retires
  } else if (warp == 20) {
    // ======================= MMA issuer =======================
    if (lane == 0) {
      constexpr uint32_t in16 = DT == VA_BF16 ? 1u : 0u;
      constexpr uint32_t idesc = umma_idesc(128, 128, in16, 0, 0);
      const uint32_t q_addr = smem_addr(q_s), kr_addr = smem_addr(k_s);
      uint64_t qd[8];
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) qd[ks] = umma_desc(q_addr + (uint32_t)(ks >> 2) * (128 * 128) + (uint32_t)(ks & 3) * 32, 16, 1024);
      for (int t = t_lo; t < t_hi; ++t) {
        const int n = t - t_lo, s = n % kStages, u = n / kStages, sb = n & 1, ub = n >> 1;
        if (!mbar_wait(&bars.kfull[s], u & 1) || !mbar_wait(&bars.sempty[sb], (ub & 1) ^ 1)) { timed_out = true; break; }
        fence_proxy_async();
        tc_fence_after();
        const uint32_t k_addr = kr_addr + (uint32_t)s * kTileBytes;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma(tmem + (uint32_t)sb * 128, qd[ks],
               umma_desc(k_addr + (uint32_t)(ks >> 2) * (128 * 128) + (uint32_t)(ks & 3) * 32, 16, 1024), idesc, ks > 0);
        umma_commit(&bars.kempty[s]);
        umma_commit(&bars.sfull[sb]);
      }
    }
  } else {
    // ======================= row walkers =======================
    const int qtr = warp & 3, cq = warp >> 2;  // TMEM lane quarter, key quarter of the tile
    const uint32_t lane_base = (uint32_t)(qtr * 32) << 16;
    Row row;
    row.run_max = -INFINITY;
    row.gap = p.gaps ? __ldg(p.gaps + b * p.gaps_sb + h) : p.gap;
    row.cnt = 0;
    row.hi = hi;
    row.out = p.col_idx + out_row * p.capacity;
    int gpos = (lo / BK) % p.group_k_block;  // position of the next walked block inside its key-block group
    const int G = p.group_k_block;
    // one key block: group bookkeeping is uniform over the CTA, the rest is per row
    auto block_begin = [&](int key0) -> bool {
      if (key0 < lo || key0 >= k_hi) return false;
      if (gpos == 0) row.run_max = -INFINITY;  // a new key-block group starts
      gpos = gpos + 1 == G ? 0 : gpos + 1;
      return true;
    };
    {
      constexpr int SB = BK < 32 ? BK : 32;  // keys per published maximum
      constexpr int NP = 32 / SB;            // maxima a thread publishes per tile
      constexpr int NBT = kTile / BK;        // key blocks per tile
      // The four threads of a row meet once per tile: the meeting that publishes a tile's block
      // maxima also carries the previous tile's counts (and the running maximum it ended with), so
      // a tile's kept keys are appended one tile later, after the positions are known.
      uint32_t prev_mask = 0u;  // keep mask of the previous tile, not yet appended
      int prev_key = 0, prev_cnt = 0;
      auto append_prev = [&](int par) {
        int before = 0, total = 0;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int cnt_q = q == cq ? prev_cnt : xcnt_s[par][(qtr * 4 + q) * 32 + lane];
          if (q < cq) before += cnt_q;
          total += cnt_q;
        }
        int pos = row.cnt + before;
        row.cnt += total;
        uint32_t mask = prev_mask;
        if (row.cnt <= p.capacity) {
          // The first four kept keys go out as straight-line predicated stores (no divergence: the
          // lanes of a warp keep different numbers of keys), the rare rest in a loop.
          int32_t* wp = row.out + pos;
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int j = __ffs((int)mask) - 1;
            st_global_if(wp + e, prev_key + j, mask != 0u);
            mask &= mask - 1u;
          }
          wp += 4;
          while (mask) {
            const int j = __ffs((int)mask) - 1;
            mask &= mask - 1u;
            *wp++ = prev_key + j;
          }
        } else {
          while (mask) {
            const int j = __ffs((int)mask) - 1;
            mask &= mask - 1u;
            if (pos < p.capacity) row.out[pos] = prev_key + j;
            ++pos;
          }
        }
      };
      int n_done = 0;
      for (int t = t_lo; t < t_hi; ++t) {
        const int n = t - t_lo, sb = n & 1, ub = n >> 1, par = n & 1;
        if (!mbar_wait(&bars.sfull[sb], ub & 1)) { timed_out = true; break; }
        tc_fence_after();
        const int key_t = t * kTile, key_q = key_t + cq * 32;
        // ---- my 32 estimates -> registers; the accumulator buffer is free again ----
        uint32_t v[32];
        tmem_ld32(tmem + (uint32_t)sb * 128 + lane_base + cq * 32, v);
        tmem_wait_ld();
        tc_fence_before();
        mbar_arrive(&bars.sempty[sb]);
        // ---- maxima of my key blocks (keys past the sequence end never count) ----
        float pm[NP];
        if (key_q + 32 <= p.sk) {
#pragma unroll
          for (int kb = 0; kb < NP; ++kb) pm[kb] = max_of<SB>(v + kb * SB);
        } else {
#pragma unroll
          for (int kb = 0; kb < NP; ++kb) {
            pm[kb] = -INFINITY;
#pragma unroll
            for (int j = 0; j < SB; ++j)
              if (key_q + kb * SB + j < p.sk) pm[kb] = fmaxf(pm[kb], __uint_as_float(v[kb * SB + j]));
          }
        }
#pragma unroll
        for (int kb = 0; kb < NP; ++kb) xmax_s[par][((qtr * 4 + cq) * 2 + kb) * 32 + lane] = pm[kb];
        mbar_arrive(&bars.quad[qtr]);
        if (!mbar_wait(&bars.quad[qtr], par)) { timed_out = true; break; }
        if (n > 0) {  // the previous tile: where it ended and where its keys go
          row.run_max = xrm_s[par ^ 1][qtr * 32 + lane];
          append_prev(par ^ 1);
        }
        // ---- running maximum entering / after every block of the tile, identical in the four threads ----
        // A tile inside the walked key range (all but the first and last of a CTA) needs no range
        // tests and lets each thread stop at its own last block.
        const bool interior = key_t >= lo && key_t + kTile <= k_hi;
        float rm_own[NP];
        bool on_own[NP];
        if (interior) {
          const float* xq = xmax_s[par] + (qtr * 4 * 2) * 32 + lane;
          switch (cq) {
            case 0: prefix_interior<BK, 0>(pm, xq, row.run_max, gpos, G, rm_own); break;
            case 1: prefix_interior<BK, 1>(pm, xq, row.run_max, gpos, G, rm_own); break;
            case 2: prefix_interior<BK, 2>(pm, xq, row.run_max, gpos, G, rm_own); break;
            default: prefix_interior<BK, 3>(pm, xq, row.run_max, gpos, G, rm_own); break;
          }
#pragma unroll
          for (int kb = 0; kb < NP; ++kb) on_own[kb] = true;
          gpos += NBT;
          while (gpos >= G) gpos -= G;
        } else {
#pragma unroll
          for (int k = 0; k < NBT; ++k) {
            float m;
            bool mine;
            if constexpr (BK <= 32) {
              const int q = k / NP, kb = k % NP;  // the quarter that holds block k and its place there
              mine = q == cq;
              m = mine ? pm[kb] : xmax_s[par][((qtr * 4 + q) * 2 + kb) * 32 + lane];
            } else {  // the block spans QPB quarters
              constexpr int QPB = BK / 32;
              mine = k == cq / QPB;
              m = -INFINITY;
#pragma unroll
              for (int i = 0; i < QPB; ++i) {
                const int q = k * QPB + i;
                m = fmaxf(m, q == cq ? pm[0] : xmax_s[par][((qtr * 4 + q) * 2) * 32 + lane]);
              }
            }
            const bool on = block_begin(key_t + k * BK);
            if (on) row.run_max = fmaxf(row.run_max, m);
            if (mine) {
              rm_own[BK <= 32 ? k % NP : 0] = row.run_max;
              on_own[BK <= 32 ? k % NP : 0] = on;
            }
          }
        }
        if (cq == 3) xrm_s[par][qtr * 32 + lane] = row.run_max;  // the value the next tile starts from
        // ---- keep mask of my 32 keys.  fp32(s + gap) >= m  <=>  the difference fp32(s + gap) - m is
        // not negative (a difference of two floats has the exact sign); its sign bit is shifted
        // into the mask, last key first, so key c ends up in bit c.  Two additions on the FMA pipe
        // and one funnel shift per estimate: the integer pipe is the busy one in this kernel. ----
        uint32_t neg = 0u;
#pragma unroll
        for (int c = 31; c >= 0; --c) {
          const float d = __fsub_rn(__fadd_rn(__uint_as_float(v[c]), row.gap), rm_own[c / SB]);
          neg = __funnelshift_l(__float_as_uint(d), neg, 1);
        }
        uint32_t mask = ~neg;
#pragma unroll
        for (int kb = 0; kb < NP; ++kb)
          if (!on_own[kb]) mask &= ~((SB == 32 ? 0xffffffffu : ((1u << SB) - 1u)) << (kb * SB));
        const int room = row.hi - key_q;  // keys at or past the row's limit are cut off
        if (room < 32) mask = room <= 0 ? 0u : (mask & ((1u << room) - 1u));
        prev_mask = mask;
        prev_key = key_q;
        prev_cnt = __popc(mask);
        xcnt_s[par][(qtr * 4 + cq) * 32 + lane] = prev_cnt;
        n_done = n + 1;
      }
      // ---- the last tile's keys: one more meeting for its counts ----
      if (!timed_out && n_done > 0) {
        mbar_arrive(&bars.quad[qtr]);
        if (mbar_wait(&bars.quad[qtr], n_done & 1)) append_prev((n_done - 1) & 1);
        else timed_out = true;
      }
    }
    if (row_ok && !timed_out && cq == 0) {  // the row's count is written by the thread of the first quarter
      p.col_count[out_row] = row.cnt;
      if (row.cnt > p.capacity && p.status) atomicOr(p.status, VA_STATUS_OVERFLOW);
    }
  }
  if (timed_out && p.status) atomicOr(p.status, VA_STATUS_TIMEOUT);
  tc_fence_before();
  __syncthreads();
  if (warp == 20) tmem_dealloc(tmem, 256);
}

template <int DT, int BK>
int launch_bk(const SelectParams& p, int batch, cudaStream_t stream) {
  // per-device attribute; setting it on every launch keeps multi-device processes correct
  if (cudaFuncSetAttribute(select_kernel<DT, BK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmem) != cudaSuccess)
    return VA_ERR_CUDA;
  const int nrows = p.rep * p.nq;
  dim3 grid((nrows + kRows - 1) / kRows, p.kv_heads, batch);
  select_kernel<DT, BK><<<grid, kThreads, kSmem, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? VA_OK : VA_ERR_CUDA;
}

template <int DT>
int launch_dt(const SelectParams& p, int bk, int batch, cudaStream_t stream) {
  switch (bk) {
    case 16: return launch_bk<DT, 16>(p, batch, stream);
    case 32: return launch_bk<DT, 32>(p, batch, stream);
    case 64: return launch_bk<DT, 64>(p, batch, stream);
    case 128: return launch_bk<DT, 128>(p, batch, stream);
    default: return VA_ERR_SHAPE;
  }
}

}  // namespace


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
  p.chunk_tiles = a.chunk_tiles;
  return a.dtype == VA_BF16 ? launch_dt<VA_BF16>(p, a.bk, a.batch, stream) : launch_dt<VA_FP16>(p, a.bk, a.batch, stream);
}

}  // namespace va
