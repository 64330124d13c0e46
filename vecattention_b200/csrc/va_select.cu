// Important-vector selection: pooled-Q . K^T estimate + streaming MinP threshold + compaction,
// with the estimate on tcgen05 tensor cores and the accumulator in tensor memory.
//
// Two kernels.
//
// 1. select_mask_kernel: estimate, running maximum and keep test; its result is one keep BIT per
//    (pooled row, key), written row-major to scratch memory.  The pooled rows of all query heads that
//    share one KV head form one row list (row R -> head hkv*rep + R/nq, tile R%nq); a CTA owns 128
//    consecutive rows of that list and walks the keys of its KV head once, 128 keys per tile, in
//    ascending order, so the running (prefix) maximum of a key-block group is a per-thread register.
//    Warp roles (608 threads, one CTA per SM):
//      warps 0-15  row walkers, by turns: warp w can reach TMEM lane quarter w % 4 (32 pooled rows) and takes
//                 every fourth key tile (tiles n with n % 4 == w / 4, accumulator buffer w / 4), so the four
//                 warps of a scheduler work on four different tiles.  A thread walks its row's whole tile:
//                 it reads the 128 estimates and forms the maxima of the tile's key blocks, receives the
//                 row's running maximum after the previous tile from the warp that walked it (one float
//                 per row through shared memory, an mbarrier per warp pair), forms the running maximum
//                 entering every block and hands the one after its tile on at once; then it reads the
//                 estimates again, builds the 128 keep bits fp32(s + gap) >= m and stores them as one
//                 16-byte piece of the row's mask.  With few row blocks the key range is cut into up to
//                 four segments (one CTA each): a CTA still walks from the first tile for the maxima but
//                 writes keep bits only for its own segment.
//      warp 16    one thread streams K: a TMA tensor-map copy per 128-key tile (two boxes of 128 rows
//                 x 128 bytes, 128-byte swizzle) into a 4-stage ring; rows past the sequence read as zeros.
//      warps 17,18 one thread each issues S_t = Q~ K_t^T for alternate tiles, 128 x 128 x 128 as eight
//                 tcgen05.mma, into one of four 128-column accumulator buffers in tensor memory.
//    All hand-offs are mbarriers with bounded waits; a timeout sets VA_STATUS_TIMEOUT.
//
// 2. select_expand_kernel: one warp per pooled row turns the row's keep bits into its ascending
//    index list (population counts, a warp scan, staging in shared memory, coalesced stores) and
//    writes the row's count.  Lists are deterministic; nothing is zero-filled; no atomics.
#include "va_common.cuh"
#include "va_sm100.cuh"
#include "va_tmap.cuh"

#include <type_traits>

namespace va {

using namespace sm100;

struct SelectParams {
  const void* avg_q;  // (B,H,nq,D)
  const float* gaps;
  int64_t gaps_sb;
  float gap;
  int32_t* col_count;
  int32_t* col_idx;
  int64_t capacity;
  int32_t* status;
  uint32_t* mask;     // keep bits, [(b * kv_heads + hkv) * rows_pad + R][wpad] 32-bit words, bit j of word w = key 32 w + j
  int rows_pad;       // pooled rows per KV head, rounded up to the CTA height
  int wpad;           // words per mask row (whole groups of four key tiles)
  int heads, kv_heads, rep, nq, sk;
  int pq, group_k_block;
  int nseg;           // CTAs per block of 128 rows, each writing the keep bits of one segment of the key range
  int by_length;      // causal, whole row blocks per head: blockIdx.x lists the row blocks of all heads longest walk first
  int tail_from, tail_seg;  // tail_seg > 0: a flat grid; the CTAs from number tail_from on (the last, partial wave of
                            // equally long walks) are cut into tail_seg key segments each
  int causal, wo_initial, compat_bsq, tile_offset, chunk_tiles;
};

namespace {

constexpr int kRows = 128;   // pooled rows per CTA
constexpr int kTile = 128;   // keys per tile
constexpr int kTileBytes = 128 * 256;
constexpr int kStages = 4;   // K ring
constexpr int kSBufs = 4;    // accumulator buffers in tensor memory (4 x 128 columns = all of it)
constexpr int kThreads = 608;  // 16 walker warps, the K producer, two MMA issuers
constexpr int kWalkerWarps = 16;
constexpr size_t kSmem = 1024 + (size_t)kTileBytes * (1 + kStages);

struct Barriers {
  uint64_t kfull[kStages], kempty[kStages], sfull[kSBufs], sempty[kSBufs];
  uint64_t hand[4][4];  // [lane quarter][turn]: that warp has published the rows' running maximum after its tile
};

// End (exclusive) of the keys pooled row `tile` of the chunk may select, spattn/src/kernels/
// vecattention_kernels.py:231-233,260: all keys, or under the causal rule the keys before the row's
// diagonal tile; the first row of every compat_bsq rows of a chunk also loses the key blocks that
// start inside the tile before it, except the first (the reference's truncating division).
__device__ __forceinline__ int row_key_limit(const SelectParams& p, int tile, int bk) {
  if (!p.causal) return p.sk;
  const int64_t g = (int64_t)p.tile_offset + tile;
  int64_t lim = g * p.pq;
  const int tile_in_chunk = p.chunk_tiles > 0 ? tile % p.chunk_tiles : tile;
  if (p.compat_bsq > 0 && (tile_in_chunk % p.compat_bsq) == 0) {
    const int64_t q1 = (g - 1) * p.pq + bk;
    lim = q1 < lim ? q1 : lim;
  }
  lim = lim < p.sk ? lim : p.sk;
  return lim > 0 ? (int)lim : 0;
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

// two fp32 additions in one instruction (round to nearest, no flush: each half is an IEEE add)
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ uint64_t pack2u(uint32_t lo, uint32_t hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
  return r;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t x, uint32_t& lo, uint32_t& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=r"(lo), "=r"(hi) : "l"(x));
}

// ---- the row walkers ------------------------------------------------------------------------------
// Sixteen warps; warp (qtr, turn) = (w % 4, w / 4) owns the pooled rows of TMEM lane quarter qtr (a warp
// reaches only the quarter w % 4) on every fourth key tile, n = turn (mod 4), which lives in accumulator
// buffer `turn`.  A thread handles its row's whole tile: first the maxima of the tile's key blocks
// (independent of earlier tiles), then, once the warp of the previous tile has handed over the rows'
// running maximum, the running maximum entering every block, which it hands on at once, and last the
// keep bits of the 128 keys, read from tensor memory a second time.  The four warps of a quarter sit on one
// scheduler and are in different phases of different tiles, so one's latencies hide behind another's work.
struct WalkShared {
  float rmx[4][4][32];  // [lane quarter][turn][lane]: running maximum after that warp's latest tile
};

// what a walker thread knows about its CTA and its row
struct WalkArgs {
  uint32_t tmem;       // first accumulator buffer
  int t_lo, t_hi;      // key tiles the CTA walks
  int t_keep;          // first tile whose keep bits this CTA writes (earlier tiles only feed the running maximum)
  int lo, k_hi;        // key range the CTA walks
  int sk, hi;          // sequence length; end of this thread's row
  int G;               // key blocks per group
  float gap;
  uint32_t* mrow;      // this thread's mask row
};

// one wait, cheap when the phase is already complete
__device__ __forceinline__ bool wait_fast(uint64_t* bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait(bar, parity);
}

// Keep bits of 32 estimates: fp32(s + gap) >= m  <=>  fp32(s + gap) - m is not negative (the difference of
// two floats has the exact sign).  m_lo applies to estimates 0..15, m_hi to 16..31.  Two packed additions per
// pair of estimates and one funnel shift per estimate that moves the sign bit into a byte of the mask, last key
// first; four independent chains of eight shifts, joined by byte permutes, so key c ends up in bit c.
__device__ __forceinline__ uint32_t keep_bits(const uint32_t (&v)[32], uint64_t gap2, float m_lo, float m_hi) {
  uint32_t neg[4];
#pragma unroll
  for (int q = 3; q >= 0; --q) {
    const float m = q >= 2 ? m_hi : m_lo;
    const uint64_t nm2 = pack2(-m, -m);
    uint32_t x = 0u;
#pragma unroll
    for (int c = q * 8 + 7; c > q * 8; c -= 2) {
      uint32_t d_lo, d_hi;
      unpack2(add2(add2(pack2u(v[c - 1], v[c]), gap2), nm2), d_lo, d_hi);
      x = __funnelshift_l(d_hi, x, 1);
      x = __funnelshift_l(d_lo, x, 1);
    }
    neg[q] = x;  // eight sign bits in the low byte
  }
  const uint32_t lo16 = __byte_perm(neg[0], neg[1], 0x0040), hi16 = __byte_perm(neg[2], neg[3], 0x0040);
  return ~__byte_perm(lo16, hi16, 0x5410);
}

// Walk every fourth key tile of the CTA for the rows of lane quarter `qtr`.  Returns false if a wait ran
// out.  BK = k_local_size; ALIGNED: groups of key blocks begin only where tiles begin.
template <int BK, bool ALIGNED>
__device__ __forceinline__ bool walk_rows(const WalkArgs& a, Barriers& bars, WalkShared& sh, int qtr, int turn, int lane) {
  constexpr int NBT = kTile / BK;  // key blocks per tile
  const uint32_t taddr = a.tmem + ((uint32_t)(qtr * 32) << 16) + (uint32_t)turn * 128;
  const uint64_t gap2 = pack2(a.gap, a.gap);
  uint64_t* const sfull = &bars.sfull[turn];
  uint64_t* const sempty = &bars.sempty[turn];
  uint64_t* const hand_in = &bars.hand[qtr][(turn + 3) & 3];
  uint64_t* const hand_out = &bars.hand[qtr][turn];
  const float* rm_in = &sh.rmx[qtr][(turn + 3) & 3][lane];
  float* rm_out = &sh.rmx[qtr][turn][lane];
  const int ntiles = a.t_hi - a.t_lo;
  const unsigned tpg = ALIGNED ? (unsigned)(((int64_t)a.G * BK) / kTile) : 1u;  // tiles per group of key blocks
  const int t_in_lo = (a.lo + kTile - 1) / kTile;  // first tile wholly at or after lo
  const int t_in_hi = min(a.k_hi, a.sk) / kTile;   // tiles before this one end at or before k_hi

  for (int n = turn; n < ntiles; n += 4) {
    const int t = a.t_lo + n, key_t = t * kTile;
    const uint32_t par = (uint32_t)(n >> 2) & 1u;
    const bool inner = ALIGNED && t >= t_in_lo && t < t_in_hi;  // no range tests, no group start inside the tile
    if (!wait_fast(sfull, par)) return false;
    tc_fence_after();
    // ---- maxima of the tile's key blocks (keys past the sequence end never count) ----
    float pm[NBT];
#pragma unroll
    for (int k = 0; k < NBT; ++k) pm[k] = -INFINITY;
#pragma unroll
    for (int c4 = 0; c4 < 4; ++c4) {
      uint32_t v[32];
      tmem_ld32(taddr + c4 * 32, v);
      tmem_wait_ld();
      if (key_t + c4 * 32 + 32 <= a.sk) {
        if (BK == 16) {
          pm[(2 * c4) % NBT] = max_of<16>(v);
          pm[(2 * c4 + 1) % NBT] = max_of<16>(v + 16);
        } else {
          const int k = (c4 * 32 / BK) % NBT;
          pm[k] = fmaxf(pm[k], max_of<32>(v));
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (key_t + c4 * 32 + j < a.sk) {
            const int k = ((c4 * 32 + j) / BK) % NBT;
            pm[k] = fmaxf(pm[k], __uint_as_float(v[j]));
          }
      }
    }
    // ---- the rows' running maximum after the previous tile, from the warp that walked it ----
    float run = -INFINITY;
    if (n > 0) {
      if (!wait_fast(hand_in, (uint32_t)((n - 1) >> 2) & 1u)) return false;
      run = *rm_in;
    }
    // ---- running maximum entering / after every block; handed on before the keep bits are formed ----
    float rm[NBT];
    uint32_t on_bits = 0xffffffffu;  // bit k: block k lies inside the walked key range
    if (inner) {
      if ((unsigned)t % tpg == 0u) run = -INFINITY;  // a new group of key blocks starts with this tile
#pragma unroll
      for (int k = 0; k < NBT; ++k) {
        run = fmaxf(run, pm[k]);
        rm[k] = run;
      }
    } else {
      int gp = (int)((unsigned)(key_t / BK) % (unsigned)a.G);  // position of the tile's first block inside its group
      on_bits = 0u;
#pragma unroll
      for (int k = 0; k < NBT; ++k) {
        const int key0 = key_t + k * BK;
        if (key0 >= a.lo && key0 < a.k_hi) {
          if (gp == 0) run = -INFINITY;  // a new group of key blocks starts
          run = fmaxf(run, pm[k]);
          on_bits |= 1u << k;
        }
        gp = gp + 1 == a.G ? 0 : gp + 1;
        rm[k] = run;
      }
    }
    *rm_out = run;
    mbar_arrive(hand_out);
    if (t < a.t_keep) {  // another CTA writes this tile's keep bits: only the running maximum was needed
      tc_fence_before();
      mbar_arrive(sempty);
      continue;
    }
    // ---- keep bits of the 128 keys ----
    uint32_t w[4];
#pragma unroll
    for (int c4 = 0; c4 < 4; ++c4) {
      uint32_t v[32];
      tmem_ld32(taddr + c4 * 32, v);
      tmem_wait_ld();
      if (c4 == 3) {  // the accumulator buffer is free again
        tc_fence_before();
        mbar_arrive(sempty);
      }
      const int k_lo = BK == 16 ? 2 * c4 : (c4 * 32 / BK) % NBT, k_hi16 = BK == 16 ? 2 * c4 + 1 : k_lo;
      uint32_t m = keep_bits(v, gap2, rm[k_lo % NBT], rm[k_hi16 % NBT]);
      if (!inner) {
        if (!((on_bits >> (k_lo % NBT)) & 1u)) m &= 0xffff0000u;
        if (!((on_bits >> (k_hi16 % NBT)) & 1u)) m &= 0x0000ffffu;
      }
      const int room = a.hi - (key_t + c4 * 32);  // keys at or past the row's limit are cut off
      if (room < 32) m = room <= 0 ? 0u : (m & ((1u << room) - 1u));
      w[c4] = m;
    }
    *reinterpret_cast<uint4*>(a.mrow + (size_t)t * 4) = make_uint4(w[0], w[1], w[2], w[3]);
  }
  return true;
}

// BK = k_local_size.  ALIGNED: a key-block group (group_k_block * BK keys) is a whole number of
// tiles, so groups begin only where tiles begin and a tile inside the walked key range needs no
// per-block bookkeeping.
template <int DT, int BK, bool ALIGNED>
__global__ void __launch_bounds__(kThreads, 1) select_mask_kernel(const __grid_constant__ CUtensorMap kmap, const SelectParams p) {
  using T = typename Elem<DT>::T;
  extern __shared__ unsigned char smem_raw[];
  __shared__ Barriers bars;
  __shared__ uint32_t tmem_base_s;
  __shared__ int s_khi;
  __shared__ WalkShared wsh;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int hkv = blockIdx.y;
  int b = blockIdx.z;
  const int nrows = p.rep * p.nq;
  // causal rows walk more keys the later their tile: the longest walks are started first
  int bx = p.causal ? (int)(gridDim.x - 1 - blockIdx.x) : (int)blockIdx.x;
  if (p.by_length) {
    // one grid row for all KV heads: CTAs are handed out in blockIdx.x order, so all heads' last 128 tiles come
    // first, then all heads' last but one, ...: a longest-first schedule over the whole launch
    const int blocks_per_head = p.nq / kRows, per_rank = p.rep * p.kv_heads;
    const int rank = (int)blockIdx.x / per_rank, r2 = (int)blockIdx.x % per_rank;
    hkv = r2 % p.kv_heads;
    bx = (r2 / p.kv_heads) * blocks_per_head + (blocks_per_head - 1 - rank);
  }
  int nseg = p.nseg;
  int row_base = (bx / p.nseg) * kRows, seg = bx % p.nseg;
  if (p.tail_seg > 0) {
    // Equally long walks fill whole waves of SMs except for the last CTAs; those are cut into key segments so that
    // the last wave is shorter (a segment's CTA re-walks the maxima of the segments before it, the cheap half).
    const int lin = (int)blockIdx.x, nb = p.rows_pad / kRows;
    int cta = lin;
    seg = 0;
    nseg = 1;
    if (lin >= p.tail_from) {
      const int r = lin - p.tail_from;
      cta = p.tail_from + r / p.tail_seg;
      seg = r % p.tail_seg;
      nseg = p.tail_seg;
    }
    row_base = (cta % nb) * kRows;
    hkv = (cta / nb) % p.kv_heads;
    b = cta / (nb * p.kv_heads);
  }

  // ---- per-row limits: walker threads (warps 0-15) own row (warp % 4) * 32 + lane ----
  const bool is_walker = warp < kWalkerWarps;
  const int wrow = (warp & 3) * 32 + lane;
  const int R = row_base + wrow;
  const bool row_ok = is_walker && R < nrows;
  const int h = hkv * p.rep + (row_ok ? R / p.nq : 0);
  const int lo = p.wo_initial ? p.pq : 0;
  const int hi = row_ok ? row_key_limit(p, R % p.nq, BK) : 0;

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
  int t_hi = (k_hi + kTile - 1) / kTile;  // exclusive
  if (t_lo >= t_hi || k_hi <= lo) return;  // nothing selectable for any row of this CTA (the expansion writes zero counts)
  // With few row blocks the key range is cut into segments, one CTA each: a CTA walks from the first tile (the
  // running maximum is a prefix quantity) but forms keep bits only for its own segment, and stops after it.
  int t_keep = t_lo;
  if (nseg > 1) {
    const int per = (t_hi - t_lo + nseg - 1) / nseg;
    t_keep = t_lo + seg * per;
    if (t_keep >= t_hi) return;
    t_hi = min(t_hi, t_keep + per);
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
      mbar_init(&bars.kfull[s], 1);   // the producer's arrival; the copies complete it by byte count
      mbar_init(&bars.kempty[s], 1);
    }
    for (int s = 0; s < kSBufs; ++s) {
      mbar_init(&bars.sfull[s], 1);
      mbar_init(&bars.sempty[s], 4 * 32);  // the four warps (one per lane quarter) that walk the buffer's tiles
    }
    for (int s = 0; s < 16; ++s) mbar_init(&bars.hand[s >> 2][s & 3], 32);
    fence_proxy_async();
  }
  if (warp == 17) {
    tmem_alloc(&tmem_base_s, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  bool timed_out = false;

  if (warp == 16) {
    // ======================= K tile producer (one thread, TMA) =======================
    if (lane == 0) {
      int issued = 0, s = 0;
      uint32_t epar = 1;  // phase parity of the stage's "empty" barrier
      const uint32_t k_base = smem_addr(k_s);
      for (int t = t_lo; t < t_hi; ++t) {
        if (!wait_fast(&bars.kempty[s], epar)) { timed_out = true; break; }
        mbar_expect_tx(&bars.kfull[s], kTileBytes);
        const uint32_t dst = k_base + (uint32_t)s * kTileBytes;
        tma_load_4d(dst, &kmap, 0, t * kTile, hkv, b, &bars.kfull[s]);                    // elements 0..63 of the 128 rows
        tma_load_4d(dst + kTileBytes / 2, &kmap, 64, t * kTile, hkv, b, &bars.kfull[s]);  // elements 64..127
        issued = t - t_lo + 1;
        if (++s == kStages) { s = 0; epar ^= 1u; }
      }
      if (timed_out) {  // no copy of this CTA may still be in flight when it retires
        for (int n = max(0, issued - kStages); n < issued; ++n) mbar_wait(&bars.kfull[n % kStages], (n / kStages) & 1);
      }
    }
  } else if (warp >= 17) {
    // ======================= MMA issuers =======================
    // Two threads (warps 17 and 18) take alternate tiles: while one is held by the tensor pipe's queue, the
    // other has already passed the barrier waits of the next tile, so the pipe never runs dry between tiles.
    if (lane == 0) {
      constexpr uint32_t in16 = DT == VA_BF16 ? 1u : 0u;
      constexpr uint32_t idesc = umma_idesc(128, 128, in16, 0, 0);
      const uint64_t qd = umma_desc(smem_addr(q_s), 16, 1024), kd0 = umma_desc(smem_addr(k_s), 16, 1024);
      int s = warp - 17, sb = warp - 17;
      uint32_t kpar = 0, spar = 1;  // phase parities of the stage's "full" and the buffer's "empty" barrier
      for (int t = t_lo + (warp - 17); t < t_hi; t += 2) {
        if (!wait_fast(&bars.kfull[s], kpar) || !wait_fast(&bars.sempty[sb], spar)) { timed_out = true; break; }
        tc_fence_after();
        umma_k128_rows128(tmem + (uint32_t)sb * 128, qd, kd0 + (uint64_t)(s * (kTileBytes >> 4)), idesc);
        umma_commit(&bars.kempty[s]);
        umma_commit(&bars.sfull[sb]);
        if ((s += 2) >= kStages) { s -= kStages; kpar ^= 1u; }
        if ((sb += 2) >= kSBufs) { sb -= kSBufs; spar ^= 1u; }
      }
    }
  } else {
    // ======================= row walkers =======================
    WalkArgs a;
    a.tmem = tmem;
    a.t_lo = t_lo;
    a.t_hi = t_hi;
    a.t_keep = t_keep;
    a.lo = lo;
    a.k_hi = k_hi;
    a.sk = p.sk;
    a.hi = hi;
    a.G = p.group_k_block;
    a.gap = p.gaps ? __ldg(p.gaps + b * p.gaps_sb + h) : p.gap;
    a.mrow = p.mask + ((size_t)(b * p.kv_heads + hkv) * p.rows_pad + row_base + wrow) * p.wpad;
    timed_out = !walk_rows<BK, ALIGNED>(a, bars, wsh, warp & 3, warp >> 2, lane);
  }
  if (timed_out && p.status) atomicOr(p.status, VA_STATUS_TIMEOUT);
  tc_fence_before();
  __syncthreads();
  if (warp == 17) tmem_dealloc(tmem, 512);
}

// ---- keep bits -> ascending index lists ---------------------------------------------------------
// One warp per pooled row (b, h, tile).  Per step the lanes take 32 consecutive mask words (1024
// keys), a warp scan of their population counts gives every lane the place of its keys, the keys
// are staged in shared memory and leave as contiguous stores.  The mask kernel has already cleared
// every bit outside the row's key range.
constexpr int kExpandWarps = 8;

template <int BK>
__global__ void __launch_bounds__(kExpandWarps * 32) select_expand_kernel(const SelectParams p, int64_t total_rows) {
  __shared__ int32_t stage_s[kExpandWarps][1024];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t row = (int64_t)blockIdx.x * kExpandWarps + warp;  // = (b * heads + h) * nq + tile
  if (row >= total_rows) return;
  const int tile = (int)(row % p.nq);
  const int64_t bh = row / p.nq;
  const int h = (int)(bh % p.heads), b = (int)(bh / p.heads);
  const int hkv = h / p.rep;
  const int R = (h % p.rep) * p.nq + tile;
  const int lo = p.wo_initial ? p.pq : 0;
  const int hi = row_key_limit(p, tile, BK);
  const uint32_t* mrow = p.mask + ((size_t)(b * p.kv_heads + hkv) * p.rows_pad + R) * p.wpad;
  int32_t* out = p.col_idx + row * p.capacity;
  int32_t* stage = stage_s[warp];
  int64_t cnt = 0;
  if (hi > lo) {
    const int w_lo = lo >> 5, w_hi = (hi + 31) >> 5;
    uint32_t cur = w_lo + lane < w_hi ? __ldg(mrow + w_lo + lane) : 0u;
    for (int w0 = w_lo; w0 < w_hi; w0 += 32) {
      const uint32_t nxt = w0 + 32 + lane < w_hi ? __ldg(mrow + w0 + 32 + lane) : 0u;  // the next step's words, fetched early
      uint32_t word = cur;
      const int c = __popc(word);
      int incl = c;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
      }
      const int total = __shfl_sync(0xffffffffu, incl, 31);
      if (total > 0) {
        int sp = incl - c;
        const int key0 = (w0 + lane) << 5;
        while (word) {
          stage[sp++] = key0 + __ffs((int)word) - 1;
          word &= word - 1u;
        }
        __syncwarp();
        for (int i = lane; i < total; i += 32)
          if (cnt + i < p.capacity) out[cnt + i] = stage[i];
        __syncwarp();
        cnt += total;
      }
      cur = nxt;
    }
  }
  if (lane == 0) {
    p.col_count[row] = (int32_t)cnt;
    if (cnt > p.capacity && p.status) atomicOr(p.status, VA_STATUS_OVERFLOW);
  }
}

template <int DT, int BK>
int launch_bk(const SelectParams& p, const CUtensorMap& kmap, int batch, cudaStream_t stream) {
  const bool aligned = ((int64_t)p.group_k_block * BK) % kTile == 0;
  auto kern = aligned ? select_mask_kernel<DT, BK, true> : select_mask_kernel<DT, BK, false>;
  // per-device attribute; setting it on every launch keeps multi-device processes correct
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmem) != cudaSuccess) return VA_ERR_CUDA;
  dim3 grid(p.rows_pad / kRows * p.nseg, p.kv_heads, batch);
  if (p.by_length) grid = dim3(p.rows_pad / kRows * p.kv_heads, 1, batch);
  if (p.tail_seg > 0) {
    const int ctas = p.rows_pad / kRows * p.kv_heads * batch;
    grid = dim3(p.tail_from + (ctas - p.tail_from) * p.tail_seg, 1, 1);
  }
  kern<<<grid, kThreads, kSmem, stream>>>(kmap, p);
  if (cudaGetLastError() != cudaSuccess) return VA_ERR_CUDA;
  const int64_t total_rows = (int64_t)batch * p.heads * p.nq;
  select_expand_kernel<BK><<<(unsigned)((total_rows + kExpandWarps - 1) / kExpandWarps), kExpandWarps * 32, 0, stream>>>(p, total_rows);
  return cudaGetLastError() == cudaSuccess ? VA_OK : VA_ERR_CUDA;
}

template <int DT>
int launch_dt(const SelectParams& p, const CUtensorMap& kmap, int bk, int batch, cudaStream_t stream) {
  switch (bk) {
    case 16: return launch_bk<DT, 16>(p, kmap, batch, stream);
    case 32: return launch_bk<DT, 32>(p, kmap, batch, stream);
    case 64: return launch_bk<DT, 64>(p, kmap, batch, stream);
    case 128: return launch_bk<DT, 128>(p, kmap, batch, stream);
    default: return VA_ERR_SHAPE;
  }
}

}  // namespace

// mask rows per KV head and words per mask row for a selection of nq pooled rows per head over sk keys
static inline void mask_geometry(int heads, int kv_heads, int nq, int sk, int& rows_pad, int& wpad) {
  const int nrows = (heads / kv_heads) * nq;
  rows_pad = (nrows + kRows - 1) / kRows * kRows;
  const int tiles = (sk + kTile - 1) / kTile;
  wpad = (tiles + 3) / 4 * 16;
}

size_t select_workspace_bytes(int batch, int heads, int kv_heads, int nq, int sk) {
  int rows_pad, wpad;
  mask_geometry(heads, kv_heads, nq, sk, rows_pad, wpad);
  return (size_t)batch * kv_heads * rows_pad * wpad * 4;
}

int select(const va_select_args& a, cudaStream_t stream) {
  SelectParams p;
  p.avg_q = a.avg_q;
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
  mask_geometry(a.heads, a.kv_heads, a.nq, a.sk, p.rows_pad, p.wpad);
  {  // few CTAs: cut the key range so that more SMs take part (each extra segment re-walks the earlier ones' maxima)
    int sms = 148, dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int64_t ctas = (int64_t)(p.rows_pad / kRows) * a.kv_heads * a.batch;
    const int tiles = (a.sk + kTile - 1) / kTile;
    int nseg = (int)(sms / (ctas > 0 ? ctas : 1));
    nseg = nseg < 1 ? 1 : (nseg > 4 ? 4 : nseg);
    if (tiles < 64 * nseg) nseg = 1;  // short walks gain nothing
    p.nseg = nseg;
  }
  p.by_length = (a.causal && p.nseg == 1 && a.nq % kRows == 0) ? 1 : 0;
  p.tail_from = p.tail_seg = 0;
  if (!a.causal && p.nseg == 1) {  // equally long walks: shorten the last, partial wave
    int sms = 148, dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int64_t ctas = (int64_t)(p.rows_pad / kRows) * a.kv_heads * a.batch;
    const int64_t full = ctas / sms * sms, rest = ctas - full;
    if (full > 0 && rest > 0 && rest * 2 <= sms && (a.sk + kTile - 1) / kTile >= 128 && ctas < (1 << 30)) {
      p.tail_from = (int)full;
      p.tail_seg = (int)(sms / rest < 4 ? sms / rest : 4);
    }
  }
  if (!a.workspace) return VA_ERR_NULL;
  if (a.workspace_bytes < select_workspace_bytes(a.batch, a.heads, a.kv_heads, a.nq, a.sk)) return VA_ERR_CAPACITY;
  if ((reinterpret_cast<uintptr_t>(a.workspace) & 15u) != 0) return VA_ERR_ALIGN;
  p.mask = static_cast<uint32_t*>(a.workspace);
  CUtensorMap kmap;
  if (!encode_rows_map(&kmap, a.dtype == VA_BF16, a.k.ptr, a.batch, a.kv_heads, a.sk, a.k.stride_b, a.k.stride_h, a.k.stride_s,
                       kTile))
    return VA_ERR_CUDA;
  return a.dtype == VA_BF16 ? launch_dt<VA_BF16>(p, kmap, a.bk, a.batch, stream) : launch_dt<VA_FP16>(p, kmap, a.bk, a.batch, stream);
}

}  // namespace va
