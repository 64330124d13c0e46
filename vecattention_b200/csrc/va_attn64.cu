// Vector-sparse flash attention for q_pooling_size 64 on tcgen05 weight-stationary MMAs.
//
// One CTA per query tile of 64 rows; keys are taken 128 at a time from the tile's dense 64-key
// blocks and then from its selected-column list (row gather).  Both products use
// tcgen05.mma.ws with M = 64, N = 128, whose accumulator occupies all 128 TMEM lanes: row r of
// the 64 x 128 result lives in lane r (columns 0..63 of the result) and lane 64 + r (columns
// 64..127), 64 TMEM columns each.  So every accumulator row is owned by two threads, each holding
// half of it, and all four softmax warps do useful work on a 64-row tile.
//
// Warp roles (576 threads, one CTA per SM):
//   warps 0-7  softmax: two groups of four warps (0-3, 4-7) take alternate chunks; inside a group
//              two threads own half a row (64 scores) each.  Per chunk a thread pulls its scores
//              from tensor memory into registers (which frees the S buffer at once), forms the row
//              maximum with its partner thread through shared memory, raises the running maximum
//              lazily (only when a chunk exceeds it by more than 2^8; the value is shared by both
//              groups), writes P = exp2(S*scale - m) in the input dtype into a double-buffered
//              operand tile and rescales its part of the row of O in the rare chunks where the
//              maximum moved.
//   warps 8-11  K gather producers, warps 12-15 V gather producers: cp.async 16-byte pieces of the
//              selected rows into rings of 128-byte-swizzled operand tiles (3 K stages, 2 V
//              stages); copy completion is reported to the stage's mbarrier asynchronously; index
//              loads run two chunks ahead and are exchanged inside the warp through shared memory.
//   warps 16,17  MMA issuers (one thread each): warp 16 issues S_j = Q K_j^T, warp 17 issues
//              O += P_j V_j; S and P are double buffered, so the tensor pipe works on S_{j+1} and
//              O += P_{j-1} V_{j-1} while softmax j runs.
// The producer warpgroups give registers to the softmax warpgroups (setmaxnreg).
// Every wait is a bounded mbarrier wait; a timeout sets VA_STATUS_TIMEOUT and unwinds the CTA.
#include "va_common.cuh"
#include "va_sm100.cuh"
#include "va_attn.cuh"

namespace va {

using namespace sm100;

namespace {

constexpr int kChunk = 128;
constexpr int kKvTile = 128 * 256;  // 128 gathered rows
constexpr int kQTile = 64 * 256;    // 64 query rows / 64 rows of P
constexpr int kKStages = 3;  // K tiles are released as soon as S_j has been computed; the S issuer is the one that waits for data
constexpr int kVStages = 2;  // V tiles live until O += P_j V_j has completed
constexpr int kThreads = 576;
// Registers per thread: the kernel is launched with 96 (the most 18 warps can all have); the two
// producer warpgroups hand 40 each back and the two softmax warpgroups take them:
// 256 * 56 + 256 * 136 + 64 * 96 = 576 * 96.
constexpr int kProducerRegs = 56, kSoftmaxRegs = 136;
// The softmax warps can only take what the producer warps hand back (the CTA's own allocation is the pool); if the
// sum exceeded the launch allocation they would wait for registers nobody releases.
static_assert(256 * kProducerRegs + 256 * kSoftmaxRegs + 64 * 96 <= kThreads * 96, "setmaxnreg pool");
constexpr size_t kSmem = 1024 + (size_t)kQTile * 3 + (size_t)kKvTile * (kKStages + kVStages);  // Q, P x2, K ring, V ring
constexpr float kRescaleThreshold = 8.0f;                                            // log2 units

struct Barriers {
  uint64_t qfull, kfull[kKStages], kempty[kKStages], vfull[kVStages], vempty[kVStages];
  uint64_t sfull[2], sempty[2], pfull[2], pempty[2], ofull, xch[4], dec[2], fin;
};
// Expected arrivals, in the order of the members above (thread i initialises barrier i).  The "full" barriers of
// the gathered tiles count one arrival per producer thread, made by the hardware when the thread's copies have landed.
constexpr int kNumBarriers = sizeof(Barriers) / sizeof(uint64_t);
__device__ __forceinline__ uint32_t barrier_count(int i) {
  constexpr int kq = 0, kf = kq + 1, ke = kf + kKStages, vf = ke + kKStages, ve = vf + kVStages, sf = ve + kVStages;
  constexpr int se = sf + 2, pf = se + 2, pe = pf + 2, of = pe + 2, xc = of + 1, dc = xc + 4, fn = dc + 2;
  static_assert(fn + 1 == kNumBarriers, "barrier table out of step with struct Barriers");
  if (i < ke) return 128;              // qfull, kfull
  if (i < vf) return 1;                // kempty
  if (i < ve) return 128;              // vfull
  if (i < se) return 1;                // vempty, sfull
  if (i < pe) return 128;              // sempty, pfull
  if (i < xc) return 1;                // pempty, ofull
  if (i < dc) return 64;               // xch
  if (i < fn) return 128;              // dec
  return 256;                          // fin
}

// Register hand-over between warpgroups (four consecutive warps, all of which execute it).
template <int N>
__device__ __forceinline__ void reg_alloc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N>
__device__ __forceinline__ void reg_dealloc() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }

// D[tmem] (+)= A[smem] * B[smem], weight-stationary form (M = 64 uses all 128 lanes)
__device__ __forceinline__ void umma_ws(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.ws.cta_group::1.kind::f16.collector::b0::discard [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// VIS: the vision-slice composition (a kernel of its own, so that the ordinary one carries none of its bookkeeping)
template <int DT, bool VIS>
__global__ void __launch_bounds__(kThreads, 1) sparse_attn64_kernel(const AttnParams p) {
  using T = typename Elem<DT>::T;
  constexpr int PQ = 64;
  extern __shared__ unsigned char smem_raw[];
  __shared__ Barriers bars;
  __shared__ uint32_t tmem_base_s;
  __shared__ int keys_s[8][kChunk];  // ring deep enough that a slot is rewritten long after its last reader
  __shared__ __align__(16) int xk_s[8][2][32];  // per producer warp: the lanes' key indices of a chunk, for the exchange
  __shared__ __align__(16) int mask_s[8][4];  // per chunk and K producer warp: does any of its keys need masking?
  __shared__ float xch_s[2][256];   // [group][phase][TMEM lane]: chunk maxima swapped by a row's two owners
  __shared__ float m_row_s[2][64];   // [chunk parity][row]: the rows' shared reference maxima (exp2 domain)
  __shared__ float fin_s[256];       // [group][TMEM lane]: row sums, added in the epilogue

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // causal tiles grow with their index: the longest are started first, so the grid's tail is made of short ones
  const int tile = p.causal ? (int)(gridDim.x - 1 - blockIdx.x) : (int)blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int hkv = h / p.rep;
  // The tile's rows [row0, row_end).  Ordinarily tile t has rows 64 t ... ; in the vision-slice composition the
  // first p.nq tiles are the sparse tiles of rows [0, vis_end), cut to the rows from vis_begin on, and behind
  // them come dense tiles for rows [0, vis_begin) and for rows [vis_end, sq): all 64-key blocks up to the
  // tile's last row, no tables.
  int row0 = tile * PQ, row_end_v = 0;
  bool dense = false;
  if constexpr (VIS) {
    int row_end = min(row0 + PQ, p.sq);
    if (tile < p.nq) {
      row_end = min(row0 + PQ, p.vis_end);
      row0 = max(row0, p.vis_begin);
    } else {
      dense = true;
      const int e = tile - p.nq, n_before = (p.vis_begin + PQ - 1) / PQ;
      if (e < n_before) {
        row0 = e * PQ;
        row_end = min(row0 + PQ, p.vis_begin);
      } else {
        row0 = p.vis_end + (e - n_before) * PQ;
        row_end = min(row0 + PQ, p.sq);
      }
    }
    if (row_end <= row0) return;  // every row of this sparse tile belongs to the dense part before it
    row_end_v = row_end;
  }
  const int row_end = VIS ? row_end_v : p.sq;  // rows of the tile at or past it do not exist (a tile has at most 64)
  const int64_t trow = (VIS && dense) ? 0 : ((int64_t)b * p.heads + h) * p.nq + tile;

  unsigned char* smem = smem_raw + ((1024u - (smem_addr(smem_raw) & 1023u)) & 1023u);
  unsigned char* q_s = smem;
  unsigned char* p_s = smem + kQTile;       // two buffers
  unsigned char* k_s = smem + 3 * kQTile;                          // K ring
  unsigned char* v_s = k_s + (size_t)kKStages * kKvTile;           // V ring

  // The start of a tile is a chain of memory latencies (counts -> indices -> rows -> first product).  What only
  // depends on the tile's position is requested before the counts are known: the Q tile, and the first two chunks'
  // column indices (speculatively: a tile with dense blocks, which come first in slot order, fetches again).
  const int32_t* blk = (VIS && dense) ? nullptr : p.blk_idx + trow * p.blk_stride;  // no table: blocks 0, 64, 128, ...
  const int32_t* col = p.col_idx + trow * p.col_stride;
  int raw_first = 0, raw_second = 0;
  if (warp >= 8 && warp < 16) {
    if (warp < 12) {
      const int pt = tid - 256;
      const T* qb = static_cast<const T*>(p.q) + b * p.q_sb + h * p.q_sh;
#pragma unroll
      for (int i = 0; i < 8; ++i) {  // Q tile: rows beyond the sequence are zero
        const int pce = pt + i * 128, r = pce >> 4, c = pce & 15;
        const bool ok = row0 + r < row_end;
        cp_async16(smem_addr(q_s + tile_off(64, r, c)), qb + (int64_t)(ok ? row0 + r : 0) * p.q_ss + c * 8, ok);
      }
    }
    const int my_slot = 2 * (warp & 3) + (lane >> 4) + 8 * (lane & 15);
    if (!(VIS && dense) && my_slot < p.col_stride) raw_first = ldg_nc(col + my_slot);
    if (!(VIS && dense) && kChunk + my_slot < p.col_stride) raw_second = ldg_nc(col + kChunk + my_slot);
  }
  const int nblk = (VIS && dense) ? (row_end - 1) / 64 + 1 : (p.blk_count ? __ldg(p.blk_count + trow) : 0);
  const int ncol = (VIS && dense) ? 0 : __ldg(p.col_count + trow);
  const int nslots = nblk * 64 + ncol;
  const int nchunks = (nslots + kChunk - 1) / kChunk;
  T* ob = static_cast<T*>(p.out) + b * p.o_sb + h * p.o_sh;

  if (nchunks == 0) {  // no key at all: the tile's output is zero
    for (int i = tid; i < PQ * 16; i += kThreads) {
      const int r = i >> 4, c = i & 15;
      if (row0 + r < row_end) *reinterpret_cast<uint4*>(ob + (int64_t)(row0 + r) * p.o_ss + c * 8) = make_uint4(0, 0, 0, 0);
    }
    if (p.lse && tid < PQ && row0 + tid < row_end) p.lse[((int64_t)b * p.heads + h) * p.sq + row0 + tid] = -INFINITY;
    cp_async_commit();
    cp_async_wait<0>();  // the Q copies requested above must not outlive the CTA
    return;
  }

  auto fetch_raw = [&](int j, int my_slot) -> int {
    const int slot = j * kChunk + my_slot;
    if (VIS && slot < nblk * 64 && blk == nullptr) return (slot >> 6) << 6;  // a dense tile: block i starts at key 64 i
    const int ci = min(max(slot - nblk * 64, 0), max(ncol - 1, 0));
    return ldg_nc(slot < nblk * 64 ? blk + (slot >> 6) : col + ci);
  };
  if (nblk > 0 && warp >= 8 && warp < 16) {
    const int my_slot = 2 * (warp & 3) + (lane >> 4) + 8 * (lane & 15);
    raw_first = fetch_raw(0, my_slot);
    raw_second = nchunks > 1 ? fetch_raw(1, my_slot) : 0;
  }
  if (tid < kNumBarriers) {
    mbar_init(reinterpret_cast<uint64_t*>(&bars) + tid, barrier_count(tid));
    fence_proxy_async();
  }
  if (warp == 16) {
    tmem_alloc(&tmem_base_s, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  const uint32_t t_s0 = tmem, t_o = tmem + 128;  // S buffers at columns 0 and 64, O at 128 (64 columns each)

  bool timed_out = false;

  if (warp >= 8 && warp < 16) {
    // ======================= gather producers (warps 8-11: K and the Q tile, warps 12-15: V) =======================
    reg_dealloc<kProducerRegs>();
    const bool is_v = warp >= 12;
    const int pt = is_v ? tid - 384 : tid - 256;
    const T* kb = static_cast<const T*>(p.k) + b * p.k_sb + hkv * p.k_sh;
    const T* vb = static_cast<const T*>(p.v) + b * p.v_sb + hkv * p.v_sh;
    if (!is_v) cp_async_arrive_noinc(&bars.qfull);  // the Q copies were issued at the top of the kernel
    // Copy geometry.  A warp covers two key rows per instruction: lanes 0-15 the sixteen 16-byte
    // pieces of row rbase + 8 i, lanes 16-31 those of the next row.  Because the rows of one thread
    // differ by multiples of 8, its swizzled piece position is the same in all of them and the
    // shared-memory destinations are one base address plus i * 1024.
    // Each lane fetches ONE key index per chunk (that of row rbase + 8 * (lane & 15)), one chunk
    // ahead; the sixteen indices a thread needs are then exchanged through shared memory.
    const int pw = (pt >> 5), hi = lane >> 4, c = lane & 15;
    const int rbase = 2 * pw + hi;
    const uint32_t dst_off = tile_off(128, rbase, c);
    const int my_slot = rbase + 8 * c;
    auto decode = [&](int j, int raw) -> int {
      const int slot = j * kChunk + my_slot;
      const int key = slot < nblk * 64 ? raw + (slot & 63) : (slot < nslots ? raw : -1);
      return (key >= 0 && key < p.sk) ? key : -1;
    };
    // All sixteen keys of this thread's rows, from the lanes that fetched them: through a small exchange array of
    // the warp (one store and four 16-byte loads per thread instead of sixteen shuffles; two buffers, so the
    // next chunk's stores cannot overtake this chunk's loads).
    int* xk = xk_s[warp - 8][0];
    auto spread = [&](int j, int key, int (&out)[16]) {
      int* buf = xk + (j & 1) * 32;
      buf[lane] = max(key, 0);  // an unused slot copies row 0: its scores are masked and its P is zero
      __syncwarp();
      const int4* src = reinterpret_cast<const int4*>(buf + (lane & 16));
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int4 q4 = src[i];
        out[4 * i] = q4.x; out[4 * i + 1] = q4.y; out[4 * i + 2] = q4.z; out[4 * i + 3] = q4.w;
      }
    };
    auto copy_tile = [&](unsigned char* tile, const T* base, int64_t stride, const int (&keys)[16], uint64_t* full) {
      const uint32_t dst = smem_addr(tile) + dst_off;
      const T* src = base + c * 8;
#pragma unroll
      for (int i = 0; i < 16; ++i) cp_async16_full(dst + i * 1024, src + (int64_t)keys[i] * stride);
      cp_async_arrive_noinc(full);
    };
    // K and V have producer warps of their own, so neither copy waits behind the other's stage:
    // a K stage is free as soon as S has been computed from it, a V stage only after the PV
    // product.  Raw index loads run two chunks ahead and are only interpreted at the top of a
    // later iteration, so the in-order warp never stalls on them.
    {
      int keys[16];
      int raw0 = raw_first, raw1 = raw_second;
      // a tile without dense blocks (every non-causal tile): slot s is entry s of the column list
      const bool plain = nblk == 0;
      int stage = 0;           // ring position of chunk j, and how often the ring has gone round (mod 2)
      uint32_t round = 0;
      for (int j = 0; j < nchunks && !timed_out; ++j) {
        int key;
        if (plain) {
          const int slot = j * kChunk + my_slot;
          key = (slot < ncol && (unsigned)raw0 < (unsigned)p.sk) ? raw0 : -1;
          raw0 = raw1;
          if (j + 2 < nchunks) raw1 = ldg_nc(col + min(slot + 2 * kChunk, ncol - 1));
        } else {
          key = decode(j, raw0);
          raw0 = raw1;
          if (j + 2 < nchunks) raw1 = fetch_raw(j + 2, my_slot);
        }
        if (!is_v) {
          keys_s[j & 7][my_slot] = key;
          // unused slots, and keys that some row of the tile may not see, make the chunk take the masking pass
          const bool flag = key < 0 || (p.causal && key > p.q_offset + row0);
          const int any = __any_sync(0xffffffffu, flag);
          if (lane == 0) mask_s[j & 7][pw] = any;
        }
        spread(j, key, keys);
        if (!is_v) {
          if (!mbar_wait(&bars.kempty[stage], round ^ 1)) { timed_out = true; break; }
          copy_tile(k_s + (size_t)stage * kKvTile, kb, p.k_ss, keys, &bars.kfull[stage]);
          if (++stage == kKStages) { stage = 0; round ^= 1; }
        } else {
          if (!mbar_wait(&bars.vempty[stage], round ^ 1)) { timed_out = true; break; }
          copy_tile(v_s + (size_t)stage * kKvTile, vb, p.v_ss, keys, &bars.vfull[stage]);
          if (++stage == kVStages) { stage = 0; round ^= 1; }
        }
      }
    }
    cp_async_commit();
    cp_async_wait<0>();  // nothing of this thread may still be in flight when the CTA retires
  } else if (warp >= 16) {
    // ======================= MMA issuers =======================
    // Two independent issuing threads, so that neither product waits behind the other's barriers:
    // warp 16 issues S_j = Q K_j^T, warp 17 issues O += P_j V_j.
    if (lane == 0) {
      constexpr uint32_t in16 = DT == VA_BF16 ? 1u : 0u;
      bool ok = true;
      if (warp == 16) {
        constexpr uint32_t idesc_s = umma_idesc(64, 128, in16, 0, 0);
        const uint32_t q_addr = smem_addr(q_s), kr_addr = smem_addr(k_s);
        ok = mbar_wait(&bars.qfull, 0);
        for (int j = 0; j < nchunks && ok; ++j) {
          const int s = j % kKStages, u = j / kKStages, sb = j & 1, ub = j >> 1;
          ok = mbar_wait(&bars.kfull[s], u & 1) && mbar_wait(&bars.sempty[sb], (ub & 1) ^ 1);
          if (!ok) break;
          fence_proxy_async();  // the producers' cp.async writes (generic proxy) -> visible to the MMA's operand reads
          tc_fence_after();
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
        }
      } else {
        constexpr uint32_t idesc_pv = umma_idesc(64, 128, in16, 0, 1);
        const uint32_t p_addr = smem_addr(p_s), vr_addr = smem_addr(v_s);
        for (int j = 0; j < nchunks && ok; ++j) {
          const int s = j % kVStages, u = j / kVStages, pb = j & 1, upb = j >> 1;
          ok = mbar_wait(&bars.vfull[s], u & 1) && mbar_wait(&bars.pfull[pb], upb & 1);
          if (!ok) break;
          fence_proxy_async();
          tc_fence_after();
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
      }
      timed_out = !ok;
    }
  } else {
    // ======================= softmax / correction / epilogue =======================
    // Two groups of four warps work on alternate chunks (group 0 = warps 0-3 the even ones, group 1
    // = warps 4-7 the odd ones), so the latencies of one chunk's softmax (tensor-memory load,
    // maximum exchange, exponentials, shared-memory stores) overlap the other's.  Inside a group,
    // accumulator row r lives in TMEM lanes r and 64 + r (64 columns each; a warp reaches the lane
    // quarter warp % 4): two threads own half a row each and meet through shared memory.
    // The reference maximum of a row is one value shared by both groups (m_row_s): the decision for
    // chunk g starts from the value left by chunk g - 1, so all P tiles and O stay on one scale.
    reg_alloc<kSoftmaxRegs>();
    const int grp = warp >> 2;
    const int qtr = warp & 3;
    const uint32_t lane_base = (uint32_t)(qtr * 32) << 16;
    const int tl = qtr * 32 + lane;           // TMEM lane
    const int row = tl & 63, half = tl >> 6;  // query row, which 64-key half of the chunk
    const int pair = qtr & 1;                 // rows 0..31 / 32..63: the two warps of the group that share them
    const int qpos = p.q_offset + row0 + row;
    float m_seen = -INFINITY, l = 0.f;        // reference this thread's row sum is currently scaled to
    const float sc = p.scale_log2;
    float* xbuf = xch_s[grp];                 // [2 phases][128]
    int xc = 0;
    for (int j = grp; j < nchunks && !timed_out; j += 2) {
      const int sb = grp, ub = j >> 1;
      const int* keys = keys_s[j & 7] + half * 64;
      if (!mbar_wait(&bars.sfull[sb], ub & 1)) { timed_out = true; break; }
      tc_fence_after();
      const int4 mk = *reinterpret_cast<const int4*>(mask_s[j & 7]);
      const bool masked = (mk.x | mk.y | mk.z | mk.w) != 0;
      // ---- this thread's 64 scores -> registers; the S buffer is free again right away ----
      uint32_t v[64];
      {
        uint32_t lo[32], hi[32];
        tmem_ld32(t_s0 + (uint32_t)sb * 64 + lane_base, lo);
        tmem_ld32(t_s0 + (uint32_t)sb * 64 + lane_base + 32, hi);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          v[i] = lo[i];
          v[32 + i] = hi[i];
        }
      }
      tc_fence_before();
      mbar_arrive(&bars.sempty[sb]);
      if (masked) {  // kept out of the arithmetic loops: a branch per element would serialise them
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          const int key = keys[i];
          if (key < 0 || (p.causal && key > qpos)) v[i] = 0xff800000u;  // -inf
        }
      }
      // ---- row maximum of the chunk: own half, then the partner's through shared memory ----
      float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int i = 0; i < 64; ++i) m4[i & 3] = fmaxf(m4[i & 3], __uint_as_float(v[i]));
      float mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
      xbuf[(xc & 1) * 128 + tl] = mx;
      mbar_arrive(&bars.xch[grp * 2 + pair]);
      if (!mbar_wait(&bars.xch[grp * 2 + pair], xc & 1)) { timed_out = true; break; }
      mx = fmaxf(mx, xbuf[(xc & 1) * 128 + (tl ^ 64)]);
      ++xc;
      // ---- the row's reference maximum: continue from what the previous chunk (other group) left ----
      if (j > 0 && !mbar_wait(&bars.dec[grp ^ 1], ((j - 1) >> 1) & 1)) { timed_out = true; break; }
      const float m_prev = j > 0 ? m_row_s[(j - 1) & 1][row] : -INFINITY;
      const float mx_s = mx * sc;
      const bool grow = mx_s > m_prev + kRescaleThreshold || (m_prev == -INFINITY && mx_s > -INFINITY);
      const float m_new = grow ? mx_s : m_prev;
      // Written to the slot of this chunk's parity, never to the one just read: the row's other owner
      // (in another warp) may not have read it yet.  Both owners write the same value.
      m_row_s[j & 1][row] = m_new;
      mbar_arrive(&bars.dec[grp]);
      const bool rescale = __any_sync(0xffffffffu, grow && j > 0);  // same rows, hence the same outcome, in the partner warp
      // P buffer free <=> the PV product that read it two chunks ago has completed
      if (!mbar_wait(&bars.pempty[sb], (ub & 1) ^ 1)) { timed_out = true; break; }
      if (rescale) {
        // O must be quiescent: wait for the PV product of the previous chunk
        if (!mbar_wait(&bars.pempty[sb ^ 1], ((j - 1) >> 1) & 1)) { timed_out = true; break; }
        tc_fence_after();
        const float alpha = grow ? ex2_approx(m_prev - m_new) : 1.f;  // 2^-inf = 0 when nothing was accumulated yet
#pragma unroll 1
        for (int qd = 0; qd < 2; ++qd) {
          uint32_t o[32];
          tmem_ld32(t_o + lane_base + qd * 32, o);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st32(t_o + lane_base + qd * 32, o);
        }
        tmem_wait_st();
      }
      if (m_seen != m_new) {  // bring this thread's row sum to the current scale (also after the other group moved it)
        l *= ex2_approx(m_seen - m_new);
        m_seen = m_new;
      }
      const float mref = m_new == -INFINITY ? 0.f : m_new;
      // ---- P = exp2(S * scale - m), row sum, P -> shared memory (K-major operand, this thread's 64 keys) ----
      unsigned char* pdst = p_s + (size_t)sb * kQTile;
      float l0 = 0.f, l1 = 0.f;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        uint32_t pk[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float p0 = ex2_approx(fmaf(__uint_as_float(v[c * 8 + e * 2]), sc, -mref));
          const float p1 = ex2_approx(fmaf(__uint_as_float(v[c * 8 + e * 2 + 1]), sc, -mref));
          l0 += p0;
          l1 += p1;
          pk[e] = Elem<DT>::pack(p0, p1);
        }
        *reinterpret_cast<uint4*>(pdst + tile_off(64, row, half * 8 + c)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
      }
      l += l0 + l1;
      tc_fence_before();
      fence_proxy_async();
      mbar_arrive(&bars.pfull[sb]);
    }
    // ---- epilogue: O / l -> global.  Every thread first brings its row sum to the final scale
    // (the last chunk's decision), then the four owners of a row add their sums. ----
    int jl = 0;
    if (!timed_out) {
      jl = nchunks - 1;  // the last chunk, decided by group (jl & 1)
      if (!mbar_wait(&bars.dec[jl & 1], (jl >> 1) & 1) || !mbar_wait(&bars.ofull, 0)) timed_out = true;
    }
    if (!timed_out) {
      tc_fence_after();
      const float m_fin = m_row_s[jl & 1][row];
      if (m_seen != m_fin) l *= ex2_approx(m_seen - m_fin);  // l == 0 when m_seen == -inf
      fin_s[grp * 128 + tl] = l;
      mbar_arrive(&bars.fin);
      if (mbar_wait(&bars.fin, 0)) {
        l = (fin_s[tl] + fin_s[tl ^ 64]) + (fin_s[128 + tl] + fin_s[128 + (tl ^ 64)]);
        const float inv = l > 0.f ? 1.f / l : 0.f;
        const bool row_ok = row0 + row < row_end;
        if (p.lse && row_ok && grp == 0 && half == 0)  // one of the row's four owners; m is in the exp2 domain
          p.lse[((int64_t)b * p.heads + h) * p.sq + row0 + row] = l > 0.f ? (m_fin + log2f(l)) * 0.6931471805599453f : -INFINITY;
        // the two groups split the 64 columns of a lane: group 0 writes the lower 32, group 1 the upper
        T* orow = ob + (int64_t)(row0 + (row_ok ? row : 0)) * p.o_ss + half * 64 + grp * 32;
        uint32_t o[32];
        tmem_ld32(t_o + lane_base + grp * 32, o);
        tmem_wait_ld();
        if (row_ok) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint4 w;
            w.x = Elem<DT>::pack(__uint_as_float(o[c * 8 + 0]) * inv, __uint_as_float(o[c * 8 + 1]) * inv);
            w.y = Elem<DT>::pack(__uint_as_float(o[c * 8 + 2]) * inv, __uint_as_float(o[c * 8 + 3]) * inv);
            w.z = Elem<DT>::pack(__uint_as_float(o[c * 8 + 4]) * inv, __uint_as_float(o[c * 8 + 5]) * inv);
            w.w = Elem<DT>::pack(__uint_as_float(o[c * 8 + 6]) * inv, __uint_as_float(o[c * 8 + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + c * 8) = w;
          }
        }
      } else {
        timed_out = true;
      }
    }
  }
  if (timed_out && p.status) atomicOr(p.status, VA_STATUS_TIMEOUT);
  tc_fence_before();
  __syncthreads();
  if (warp == 16) tmem_dealloc(tmem, 256);
}

template <int DT>
int launch(const AttnParams& p, int batch, cudaStream_t stream) {
  // per-device attribute; setting it on every launch keeps multi-device processes correct
  auto kern = p.vis_on ? sparse_attn64_kernel<DT, true> : sparse_attn64_kernel<DT, false>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmem) != cudaSuccess) return VA_ERR_CUDA;
  int tiles = p.nq;
  if (p.vis_on) tiles += (p.vis_begin + 63) / 64 + (p.sq - p.vis_end + 63) / 64;  // the dense tiles before and after
  dim3 grid(tiles, p.heads, batch);
  kern<<<grid, kThreads, kSmem, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? VA_OK : VA_ERR_CUDA;
}

}  // namespace


int launch_attn64(const AttnParams& p, int dtype, int batch, cudaStream_t stream) {
  return dtype == VA_BF16 ? launch<VA_BF16>(p, batch, stream) : launch<VA_FP16>(p, batch, stream);
}

}  // namespace va
