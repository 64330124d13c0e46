// Vector-sparse flash attention for q_pooling_size 64 on tcgen05 weight-stationary MMAs.
//
// Persistent CTAs, one per SM, each working through query tiles of 64 rows; keys are taken 128 at a time from the tile's dense 64-key
// blocks and then from its selected-column list (row gather).  Both products use
// tcgen05.mma.ws with M = 64, N = 128, whose accumulator occupies all 128 TMEM lanes: row r of
// the 64 x 128 result lives in lane r (columns 0..63 of the result) and lane 64 + r (columns
// 64..127), 64 TMEM columns each.  So every accumulator row is owned by two threads, each holding
// half of it, and all four softmax warps do useful work on a 64-row tile.
//
// Warp roles (448 threads, one CTA per SM):
//   warps 0-3, 10-13  softmax: four threads own a quarter (32 scores) of a row each.  Per chunk a
//              thread pulls its scores from tensor memory into registers (which frees the S buffer at once), forms
//              the row maximum with its three partner threads through shared memory, raises the running
//              maximum lazily (only when a chunk exceeds it by more than 2^8), writes
//              P = exp2(S*scale - m) in the input dtype into a double-buffered operand tile and
//              rescales its part of the row of O in the rare chunks where the maximum moved.
//   warps 4,9  MMA issuers (one thread each): warp 4 issues S_j = Q K_j^T, warp 9 issues O += P_j V_j;
//              S and P are double buffered, so the tensor pipe works on S_{j+1} and
//              O += P_{j-1} V_{j-1} while softmax j runs.
//   warps 5-8  gather producers: cp.async 16-byte pieces of the selected K and V rows into rings of
//              128-byte-swizzled operand tiles (2 K stages, 3 V stages; K runs a chunk ahead of V);
//              copy completion is reported to the stage's mbarrier asynchronously, index loads run
//              further ahead and are exchanged inside the warp with shuffles.
// Every wait is a bounded mbarrier wait; a timeout sets VA_STATUS_TIMEOUT and unwinds the CTA.
#include "va_common.cuh"
#include "va_sm100.cuh"
#include "va_attn.cuh"

namespace va {

using namespace sm100;

namespace {

// Build with -DVA_DEBUG_STAMPS to record clock64() time stamps of one CTA's pipeline events.
#ifdef VA_DEBUG_STAMPS
__device__ long long g_stamps[32 * 16];
#define VA_STAMPT(ev) do { if (blockIdx.x == 7 && threadIdx.x == 160 && it < 16) g_stamps[(ev) * 16 + it] = clock64(); } while (0)
#define VA_STAMP(ev, j) do { if (blockIdx.x == 7) { int sl_ = -1; if (it == 0 && (j) >= nchunks - 8) sl_ = (j) - (nchunks - 8); if (it == 1 && (j) < 8) sl_ = 8 + (j); if (sl_ >= 0 && sl_ < 16) g_stamps[(ev) * 16 + sl_] = clock64(); } } while (0)
#else
#define VA_STAMP(ev, j) do { } while (0)
#define VA_STAMPT(ev) do { } while (0)
#endif

constexpr int kChunk = 128;
constexpr int kKvTile = 128 * 256;  // 128 gathered rows
constexpr int kQTile = 64 * 256;    // 64 query rows / 64 rows of P
constexpr int kKStages = 2;  // K tiles are released as soon as S_j has been computed
constexpr int kVStages = 3;  // V tiles live until O += P_j V_j has completed
constexpr int kThreads = 448;
constexpr size_t kSmem = 1024 + (size_t)kQTile * 3 + (size_t)kKvTile * (kKStages + kVStages);  // Q, P x2, K ring, V ring
constexpr float kRescaleThreshold = 8.0f;                                            // log2 units

struct Barriers {
  uint64_t qfull, kfull[kKStages], kempty[kKStages], vfull[kVStages], vempty[kVStages];
  uint64_t sfull[2], sempty[2], pfull[2], pempty[2], ofull, oempty, qempty, xch[2];
};

// D[tmem] (+)= A[smem] * B[smem], weight-stationary form (M = 64 uses all 128 lanes)
__device__ __forceinline__ void umma_ws(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.ws.cta_group::1.kind::f16.collector::b0::discard [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// What one query tile needs; every role derives the same values from the same table entries.
struct TileInfo {
  int b, h, tile, nblk, ncol, nslots, nchunks;
  int64_t trow;
};
// The table loads of a tile are issued while the previous tile is being processed (`tile_fetch`)
// and only interpreted when the tile starts (`tile_finish`), so no role waits for them.
__device__ __forceinline__ TileInfo tile_fetch(const AttnParams& p, int lin, int num_tiles) {
  TileInfo t;
  t.trow = lin;  // ((b * heads + h) * nq + tile)
  t.nblk = 0;
  t.ncol = 0;
  if (lin < num_tiles) {
    if (p.blk_count) t.nblk = ldg_nc(p.blk_count + lin);
    t.ncol = ldg_nc(p.col_count + lin);
  }
  return t;
}
__device__ __forceinline__ void tile_finish(const AttnParams& p, TileInfo& t) {
  const int lin = (int)t.trow;
  t.tile = lin % p.nq;
  const int bh = lin / p.nq;
  t.h = bh % p.heads;
  t.b = bh / p.heads;
  t.nslots = t.nblk * 64 + t.ncol;
  t.nchunks = (t.nslots + kChunk - 1) / kChunk;
}

// Persistent kernel: CTA c works on query tiles c, c + gridDim.x, ... (tiles of one head are
// neighbours in that order, so the CTAs running at the same time share its K/V through L2).
// All rings and double buffers simply continue across tiles: stage and parity come from running
// chunk counters, so the producers fetch the next tile's keys and the first S of the next tile is
// computed while the current tile's last softmax, PV product and epilogue are still in flight.
template <int DT>
__global__ void __launch_bounds__(kThreads, 1) sparse_attn64_kernel(const AttnParams p, int num_tiles) {
  using T = typename Elem<DT>::T;
  constexpr int PQ = 64;
  extern __shared__ unsigned char smem_raw[];
  __shared__ Barriers bars;
  __shared__ uint32_t tmem_base_s;
  __shared__ int keys_s[8][kChunk];  // ring deep enough that a slot is rewritten long after its last reader
  __shared__ float xch_s[2][256];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  unsigned char* smem = smem_raw + ((1024u - (smem_addr(smem_raw) & 1023u)) & 1023u);
  unsigned char* q_s = smem;
  unsigned char* p_s = smem + kQTile;                     // two buffers
  unsigned char* k_s = smem + 3 * kQTile;                 // K ring
  unsigned char* v_s = k_s + (size_t)kKStages * kKvTile;  // V ring

  if (tid == 0) {
    mbar_init(&bars.qfull, 256);  // per producer thread: one asynchronous copy-completion arrival + one plain arrival
    mbar_init(&bars.qempty, 1);
    for (int s = 0; s < kKStages; ++s) {
      mbar_init(&bars.kfull[s], 256);
      mbar_init(&bars.kempty[s], 1);
    }
    for (int s = 0; s < kVStages; ++s) {
      mbar_init(&bars.vfull[s], 256);
      mbar_init(&bars.vempty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars.sfull[s], 1);
      mbar_init(&bars.sempty[s], 256);
      mbar_init(&bars.pfull[s], 256);
      mbar_init(&bars.pempty[s], 1);
      mbar_init(&bars.xch[s], 128);
    }
    mbar_init(&bars.ofull, 1);
    mbar_init(&bars.oempty, 256);
    fence_proxy_async();
  }
  if (warp == 4) {
    tmem_alloc(&tmem_base_s, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  const uint32_t t_s0 = tmem, t_o = tmem + 128;  // S buffers at columns 0 and 64, O at 128 (64 columns each)

  bool timed_out = false;

  if (warp >= 5 && warp <= 8) {
    // ======================= gather producers =======================
    const int pt = tid - 160;
    // Copy geometry.  A warp covers two key rows per instruction: lanes 0-15 the sixteen 16-byte
    // pieces of row rbase + 8 i, lanes 16-31 those of the next row.  Because the rows of one thread
    // differ by multiples of 8, its swizzled piece position is the same in all of them and the
    // shared-memory destinations are one base address plus i * 1024.
    // Each lane fetches ONE key index per chunk (that of row rbase + 8 * (lane & 15)); the sixteen
    // indices a thread needs are then exchanged with warp shuffles.
    const int pw = warp - 5, hi = lane >> 4, c = lane & 15;
    const int rbase = 2 * pw + hi;
    const uint32_t dst_off = tile_off(128, rbase, c);
    const int my_slot = rbase + 8 * c;
    auto spread = [&](int key, int (&out)[16]) {
      const int kcl = max(key, 0);  // an unused slot copies row 0: its scores are masked and its P is zero
#pragma unroll
      for (int i = 0; i < 16; ++i) out[i] = __shfl_sync(0xffffffffu, kcl, (lane & 16) + i);
    };
    int g = 0;  // chunks produced so far by this CTA
    int it = 0;
    TileInfo tnext = tile_fetch(p, blockIdx.x, num_tiles);
    // first column indices of the next tile (valid when it has no dense blocks), fetched a tile ahead
    auto first_cols = [&](int lin) -> int {
      const int64_t off = (int64_t)(lin < num_tiles ? lin : 0) * p.col_stride;
      return ldg_nc(p.col_idx + off + (my_slot < p.col_stride ? my_slot : 0));
    };
    int raw_first = first_cols(blockIdx.x);
    for (int lin = blockIdx.x; lin < num_tiles && !timed_out; lin += gridDim.x) {
      TileInfo ti = tnext;
      const int raw_pref = raw_first;
      tnext = tile_fetch(p, lin + gridDim.x, num_tiles);
      raw_first = first_cols(lin + gridDim.x);
      VA_STAMPT(12);
      tile_finish(p, ti);
      if (ti.nchunks == 0) continue;
      const int nblk = ti.nblk, ncol = ti.ncol, nslots = ti.nslots, nchunks = ti.nchunks;
      const int hkv = ti.h / p.rep, row0 = ti.tile * PQ;
      const T* qb = static_cast<const T*>(p.q) + ti.b * p.q_sb + ti.h * p.q_sh;
      const T* kb = static_cast<const T*>(p.k) + ti.b * p.k_sb + hkv * p.k_sh;
      const T* vb = static_cast<const T*>(p.v) + ti.b * p.v_sb + hkv * p.v_sh;
      const int32_t* blk = p.blk_idx + ti.trow * p.blk_stride;
      const int32_t* col = p.col_idx + ti.trow * p.col_stride;
      // The raw index load is issued ahead and only interpreted an iteration later, so the in-order
      // warp never stalls on it.
      auto fetch_raw = [&](int j) -> int {
        const int slot = j * kChunk + my_slot;
        const int ci = min(max(slot - nblk * 64, 0), max(ncol - 1, 0));
        return ldg_nc(slot < nblk * 64 ? blk + (slot >> 6) : col + ci);
      };
      auto decode = [&](int j, int raw) -> int {
        const int slot = j * kChunk + my_slot;
        const int key = slot < nblk * 64 ? raw + (slot & 63) : (slot < nslots ? raw : -1);
        return (key >= 0 && key < p.sk) ? key : -1;
      };
      auto copy_tile = [&](unsigned char* tile, const T* base, int64_t stride, const int (&keys)[16], uint64_t* full) {
        const uint32_t dst = smem_addr(tile) + dst_off;
        const T* src = base + c * 8;
#pragma unroll
        for (int i = 0; i < 16; ++i) cp_async16_full(dst + i * 1024, src + (int64_t)keys[i] * stride);
        cp_async_arrive_noinc(full);
        mbar_arrive(full);
      };
      int kcur[16], knext[16];
      const int key0 = decode(0, nblk == 0 ? raw_pref : fetch_raw(0));
      // Q tile first (it is on the critical path of the tile's first S product; rows beyond the
      // sequence are zero), as soon as the previous tile's S products are done with the old one
      if (!mbar_wait(&bars.qempty, (it & 1) ^ 1)) { timed_out = true; break; }
      VA_STAMPT(14);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int pce = pt + i * 128, r = pce >> 4, cc = pce & 15;
        const bool ok = row0 + r < p.sq;
        cp_async16(smem_addr(q_s + tile_off(64, r, cc)), qb + (int64_t)(ok ? row0 + r : 0) * p.q_ss + cc * 8, ok);
      }
      cp_async_arrive_noinc(&bars.qfull);
      mbar_arrive(&bars.qfull);
      VA_STAMPT(15);
      // the next tile's queries are pulled into L2 now, a whole tile ahead of their use
      if (lin + (int)gridDim.x < num_tiles) {
        const int ln = lin + gridDim.x, tn = ln % p.nq, bhn = ln / p.nq;
        const int rn = tn * PQ + (pt >> 1);
        if (rn < p.sq)
          prefetch_l2(static_cast<const T*>(p.q) + (bhn / p.heads) * p.q_sb + (bhn % p.heads) * p.q_sh + (int64_t)rn * p.q_ss +
                      (pt & 1) * 64);
      }
      // K of the tile's first chunk
      {
        const int ks = g % kKStages, ku = g / kKStages;
        keys_s[g & 7][my_slot] = key0;
        spread(key0, kcur);
        if (!mbar_wait(&bars.kempty[ks], (ku & 1) ^ 1)) { timed_out = true; break; }
        VA_STAMPT(13);
        copy_tile(k_s + (size_t)ks * kKvTile, kb, p.k_ss, kcur, &bars.kfull[ks]);
      }
      // raw indices of the next chunks: loaded now, interpreted an iteration later (assigned
      // directly: copying a register whose load is still in flight would stall the warp)
      int raw1 = nchunks > 1 ? fetch_raw(1) : 0;
      int raw2 = nchunks > 2 ? fetch_raw(2) : 0;
      // K runs one chunk ahead of V: K_{j+1} only needs S_{j-1} to be done, while V_j has to wait for
      // the PV product three chunks back.
      for (int j = 0; j < nchunks && !timed_out; ++j) {
        if (pt == 0) VA_STAMP(0, j);
        if (j + 1 < nchunks) {
          const int gn = g + j + 1, ks = gn % kKStages, ku = gn / kKStages;
          const int key = decode(j + 1, raw1);
          raw1 = raw2;
          if (j + 3 < nchunks) raw2 = fetch_raw(j + 3);
          keys_s[gn & 7][my_slot] = key;
          spread(key, knext);
          if (!mbar_wait(&bars.kempty[ks], (ku & 1) ^ 1)) { timed_out = true; break; }
          if (pt == 0) VA_STAMP(1, j);
          copy_tile(k_s + (size_t)ks * kKvTile, kb, p.k_ss, knext, &bars.kfull[ks]);
          if (pt == 0) VA_STAMP(2, j);
        }
        {
          const int gv = g + j, vs = gv % kVStages, vu = gv / kVStages;
          if (!mbar_wait(&bars.vempty[vs], (vu & 1) ^ 1)) { timed_out = true; break; }
          if (pt == 0) VA_STAMP(3, j);
          copy_tile(v_s + (size_t)vs * kKvTile, vb, p.v_ss, kcur, &bars.vfull[vs]);
          if (pt == 0) VA_STAMP(4, j);
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) kcur[i] = knext[i];
      }
      g += nchunks;
      ++it;
    }
    cp_async_commit();
    cp_async_wait<0>();  // nothing of this thread may still be in flight when the CTA retires
  } else if (warp == 4 || warp == 9) {
    // ======================= MMA issuers =======================
    // Two independent issuing threads, so that neither product waits behind the other's barriers:
    // warp 4 issues S_j = Q K_j^T, warp 9 issues O += P_j V_j.
    if (lane == 0) {
      constexpr uint32_t in16 = DT == VA_BF16 ? 1u : 0u;
      bool ok = true;
      int g = 0, it = 0;
      if (warp == 4) {
        constexpr uint32_t idesc_s = umma_idesc(64, 128, in16, 0, 0);
        const uint32_t q_addr = smem_addr(q_s), kr_addr = smem_addr(k_s);
        TileInfo tnext = tile_fetch(p, blockIdx.x, num_tiles);
        for (int lin = blockIdx.x; lin < num_tiles && ok; lin += gridDim.x) {
          TileInfo ti = tnext;
          tnext = tile_fetch(p, lin + gridDim.x, num_tiles);
          tile_finish(p, ti);
          const int nchunks = ti.nchunks;
          if (nchunks == 0) continue;
          ok = mbar_wait(&bars.qfull, it & 1);
          for (int j = 0; j < nchunks && ok; ++j) {
            const int gj = g + j, s = gj % kKStages, u = gj / kKStages, sb = gj & 1, ub = gj >> 1;
            ok = mbar_wait(&bars.kfull[s], u & 1) && mbar_wait(&bars.sempty[sb], (ub & 1) ^ 1);
            if (!ok) break;
            tc_fence_after();
            VA_STAMP(5, j);
            const uint32_t k_addr = kr_addr + (uint32_t)s * kKvTile;
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
              const uint32_t qoff = (uint32_t)(ks >> 2) * (64 * 128) + (uint32_t)(ks & 3) * 32;
              const uint32_t koff = (uint32_t)(ks >> 2) * (128 * 128) + (uint32_t)(ks & 3) * 32;
              umma_ws(t_s0 + (uint32_t)sb * 64, umma_desc(q_addr + qoff, 16, 1024), umma_desc(k_addr + koff, 16, 1024),
                      idesc_s, ks > 0);
            }
            umma_commit(&bars.kempty[s]);
            umma_commit(&bars.sfull[sb]);
            if (j == nchunks - 1) umma_commit(&bars.qempty);  // the Q tile may be replaced
            VA_STAMP(6, j);
          }
          g += nchunks;
          ++it;
        }
      } else {
        constexpr uint32_t idesc_pv = umma_idesc(64, 128, in16, 0, 1);
        const uint32_t p_addr = smem_addr(p_s), vr_addr = smem_addr(v_s);
        TileInfo tnext = tile_fetch(p, blockIdx.x, num_tiles);
        for (int lin = blockIdx.x; lin < num_tiles && ok; lin += gridDim.x) {
          TileInfo ti = tnext;
          tnext = tile_fetch(p, lin + gridDim.x, num_tiles);
          tile_finish(p, ti);
          const int nchunks = ti.nchunks;
          if (nchunks == 0) continue;
          // the first product of a tile overwrites O: the previous tile's epilogue must have read it
          ok = mbar_wait(&bars.oempty, (it & 1) ^ 1);
          for (int j = 0; j < nchunks && ok; ++j) {
            const int gj = g + j, s = gj % kVStages, u = gj / kVStages, pb = gj & 1, upb = gj >> 1;
            ok = mbar_wait(&bars.vfull[s], u & 1) && mbar_wait(&bars.pfull[pb], upb & 1);
            if (!ok) break;
            tc_fence_after();
            VA_STAMP(7, j);
            const uint32_t v_addr = vr_addr + (uint32_t)s * kKvTile;
            const uint32_t pa = p_addr + (uint32_t)pb * kQTile;
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
              const uint32_t poff = (uint32_t)(ks >> 2) * (64 * 128) + (uint32_t)(ks & 3) * 32;
              umma_ws(t_o, umma_desc(pa + poff, 16, 1024), umma_desc(v_addr + (uint32_t)ks * 16 * 128, 128 * 128, 1024),
                      idesc_pv, (j > 0 || ks > 0) ? 1u : 0u);
            }
            umma_commit(&bars.vempty[s]);
            umma_commit(&bars.pempty[pb]);
            if (j == nchunks - 1) umma_commit(&bars.ofull);
          }
          g += nchunks;
          ++it;
        }
      }
      timed_out = !ok;
    }
  } else {
    // ======================= softmax / correction / epilogue =======================
    // Eight warps.  Accumulator row r lives in TMEM lanes r and 64 + r (64 columns each); a warp can
    // only reach the lane quarter (warp % 4), so warps 0-3 take columns 0..31 and warps 10-13 columns
    // 32..63 of their quarter: four threads own a quarter row each and meet through shared memory.
    const int qtr = warp & 3, colh = warp >= 10 ? 1 : 0;
    const uint32_t lane_base = (uint32_t)(qtr * 32) << 16;
    const int tl = qtr * 32 + lane;           // TMEM lane
    const int row = tl & 63, half = tl >> 6;  // query row, which 64-key half of the chunk
    const int grp = qtr & 1;                  // rows 0..31 / 32..63: the four warps that share them
    const int member = half * 2 + colh;
    const float sc = p.scale_log2;
    auto xslot = [&](int buf, int m) -> float& { return xch_s[buf][(grp * 4 + m) * 32 + lane]; };
    int g = 0, it = 0, xc = 0;  // chunks consumed, tiles with work done, exchanges done
    TileInfo tnext = tile_fetch(p, blockIdx.x, num_tiles);
    for (int lin = blockIdx.x; lin < num_tiles && !timed_out; lin += gridDim.x) {
      TileInfo ti = tnext;
      tnext = tile_fetch(p, lin + gridDim.x, num_tiles);
      tile_finish(p, ti);
      const int nblk = ti.nblk, nchunks = ti.nchunks, row0 = ti.tile * PQ;
      T* ob = static_cast<T*>(p.out) + ti.b * p.o_sb + ti.h * p.o_sh;
      const bool row_ok = row0 + row < p.sq;
      T* orow = ob + (int64_t)(row0 + (row_ok ? row : 0)) * p.o_ss + half * 64 + colh * 32;
      if (nchunks == 0) {  // no key at all: the tile's output is zero
        if (row_ok) {
#pragma unroll
          for (int cc = 0; cc < 4; ++cc) *reinterpret_cast<uint4*>(orow + cc * 8) = make_uint4(0, 0, 0, 0);
        }
        continue;
      }
      const int qpos = p.q_offset + row0 + row;
      float m_used = -INFINITY, l = 0.f;
      for (int j = 0; j < nchunks && !timed_out; ++j) {
        const int gj = g + j, sb = gj & 1, ub = gj >> 1;
        const bool masked = p.causal || j == nchunks - 1 || j * kChunk < nblk * 64;
        const int* keys = keys_s[gj & 7] + half * 64 + colh * 32;
        if (!mbar_wait(&bars.sfull[sb], ub & 1)) { timed_out = true; break; }
        tc_fence_after();
        if (tid == 0) VA_STAMP(8, j);
        // ---- this thread's 32 scores -> registers; the S buffer is free again right away ----
        uint32_t v[32];
        tmem_ld32(t_s0 + (uint32_t)sb * 64 + colh * 32 + lane_base, v);
        tmem_wait_ld();
        tc_fence_before();
        mbar_arrive(&bars.sempty[sb]);
        if (masked) {  // kept out of the arithmetic loops: a branch per element would serialise them
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int key = keys[i];
            if (key < 0 || (p.causal && key > qpos)) v[i] = 0xff800000u;  // -inf
          }
        }
        // ---- row maximum: own quarter, then the three others through shared memory ----
        float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int i = 0; i < 32; ++i) m4[i & 3] = fmaxf(m4[i & 3], __uint_as_float(v[i]));
        float mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
        xslot(xc & 1, member) = mx;
        mbar_arrive(&bars.xch[grp]);
        if (!mbar_wait(&bars.xch[grp], xc & 1)) { timed_out = true; break; }
        mx = fmaxf(fmaxf(xslot(xc & 1, 0), xslot(xc & 1, 1)), fmaxf(xslot(xc & 1, 2), xslot(xc & 1, 3)));
        ++xc;
        if (tid == 0) VA_STAMP(9, j);
        const float mx_s = mx * sc;
        const bool grow = mx_s > m_used + kRescaleThreshold || (m_used == -INFINITY && mx_s > -INFINITY);
        const float m_new = grow ? mx_s : m_used;
        const bool rescale = __any_sync(0xffffffffu, grow && j > 0);  // same rows, hence same verdict, in all four warps
        // P buffer free <=> the PV product that read it two chunks ago has completed
        if (!mbar_wait(&bars.pempty[gj & 1], ((gj >> 1) & 1) ^ 1)) { timed_out = true; break; }
        if (rescale) {
          // O must be quiescent: wait for the PV product of the previous chunk
          if (!mbar_wait(&bars.pempty[(gj - 1) & 1], ((gj - 1) >> 1) & 1)) { timed_out = true; break; }
          tc_fence_after();
          const float alpha = grow ? ex2_approx(m_used - m_new) : 1.f;  // 2^-inf = 0 when nothing was accumulated yet
          uint32_t o[32];
          tmem_ld32(t_o + lane_base + colh * 32, o);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st32(t_o + lane_base + colh * 32, o);
          tmem_wait_st();
          l *= alpha;
        }
        if (tid == 0) VA_STAMP(10, j);
        m_used = m_new;
        const float mref = m_used == -INFINITY ? 0.f : m_used;
        // ---- P = exp2(S * scale - m), row sum, P -> shared memory (K-major operand, this thread's 32 keys) ----
        unsigned char* pdst = p_s + (size_t)(gj & 1) * kQTile;
        float l0 = 0.f, l1 = 0.f;
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          uint32_t pk[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float p0 = ex2_approx(fmaf(__uint_as_float(v[cc * 8 + e * 2]), sc, -mref));
            const float p1 = ex2_approx(fmaf(__uint_as_float(v[cc * 8 + e * 2 + 1]), sc, -mref));
            l0 += p0;
            l1 += p1;
            pk[e] = Elem<DT>::pack(p0, p1);
          }
          *reinterpret_cast<uint4*>(pdst + tile_off(64, row, half * 8 + colh * 4 + cc)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        }
        l += l0 + l1;
        tc_fence_before();
        fence_proxy_async();
        mbar_arrive(&bars.pfull[gj & 1]);
        if (tid == 0) VA_STAMP(11, j);
      }
      if (timed_out) break;
      // ---- epilogue: O / l -> global; the row sum is the sum of the four owners' sums ----
      if (!mbar_wait(&bars.ofull, it & 1)) { timed_out = true; break; }
      tc_fence_after();
      uint32_t o[32];
      tmem_ld32(t_o + lane_base + colh * 32, o);
      tmem_wait_ld();
      tc_fence_before();
      mbar_arrive(&bars.oempty);  // O is in registers: the next tile's first PV product may overwrite it
      xslot(xc & 1, member) = l;
      mbar_arrive(&bars.xch[grp]);
      if (!mbar_wait(&bars.xch[grp], xc & 1)) { timed_out = true; break; }
      l = (xslot(xc & 1, 0) + xslot(xc & 1, 1)) + (xslot(xc & 1, 2) + xslot(xc & 1, 3));
      ++xc;
      const float inv = l > 0.f ? 1.f / l : 0.f;
      if (row_ok) {
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          uint4 w;
          w.x = Elem<DT>::pack(__uint_as_float(o[cc * 8 + 0]) * inv, __uint_as_float(o[cc * 8 + 1]) * inv);
          w.y = Elem<DT>::pack(__uint_as_float(o[cc * 8 + 2]) * inv, __uint_as_float(o[cc * 8 + 3]) * inv);
          w.z = Elem<DT>::pack(__uint_as_float(o[cc * 8 + 4]) * inv, __uint_as_float(o[cc * 8 + 5]) * inv);
          w.w = Elem<DT>::pack(__uint_as_float(o[cc * 8 + 6]) * inv, __uint_as_float(o[cc * 8 + 7]) * inv);
          *reinterpret_cast<uint4*>(orow + cc * 8) = w;
        }
      }
      g += nchunks;
      ++it;
    }
  }
  if (timed_out && p.status) atomicOr(p.status, VA_STATUS_TIMEOUT);
  tc_fence_before();
  __syncthreads();
  if (warp == 4) tmem_dealloc(tmem, 256);
}

template <int DT>
int launch(const AttnParams& p, int batch, cudaStream_t stream) {
  // per-device attributes; queried and set on every launch so that multi-device processes stay correct
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
    return VA_ERR_CUDA;
  if (cudaFuncSetAttribute(sparse_attn64_kernel<DT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmem) !=
      cudaSuccess)
    return VA_ERR_CUDA;
  const long long tiles = (long long)p.nq * p.heads * batch;
  if (tiles > 0x7fffffffLL) return VA_ERR_SHAPE;
  const int grid = (int)(tiles < sms ? tiles : sms);  // one persistent CTA per SM
  sparse_attn64_kernel<DT><<<grid, kThreads, kSmem, stream>>>(p, (int)tiles);
  return cudaGetLastError() == cudaSuccess ? VA_OK : VA_ERR_CUDA;
}

}  // namespace

#ifdef VA_DEBUG_STAMPS
extern "C" int va_debug_read_stamps(long long* host_out) {
  return (int)cudaMemcpyFromSymbol(host_out, g_stamps, sizeof(long long) * 32 * 16);
}
#endif

int launch_attn64(const AttnParams& p, int dtype, int batch, cudaStream_t stream) {
  return dtype == VA_BF16 ? launch<VA_BF16>(p, batch, stream) : launch<VA_FP16>(p, batch, stream);
}

}  // namespace va
