// Persistent paged MLA decode on tcgen05: one CTA per SM walks an equal share of all KV tiles of the batch.
//
// The per-tile machinery is the one of mla_tcgen05.cuh (64 (query, head) columns on the TMEM lanes, 64-token
// tiles, S of tile t+1 issued before P.V of tile t).  What this kernel changes is everything around the tiles,
// which is where a decode step of few rows x many heads spent most of its time:
//
//   * Work is not one CTA per (sequence, head group, split).  The (sequence, head group) pairs are laid end to end
//     in units of KV tiles, the total is cut into gridDim.x equal chunks, and CTA k walks chunk k: a run of
//     *segments*, each a range of tiles of one pair.  The cut is computed in the kernel from the device-side
//     sequence lengths (every CTA scans the same prefix sums), so a captured CUDA graph balances whatever lengths
//     it is replayed on and no host-side work list or split count exists.
//   * TMEM, barriers and the tile ring are set up once per CTA.  Between segments only the query tile is reloaded
//     (after the last S of the previous segment has read it), while the KV loads of the next segment are already
//     in flight and the tensor pipe idles only for the previous segment's accumulator read-out.
//   * A pair that one CTA covers whole is normalised and stored directly.  A pair cut across CTAs leaves
//     unnormalised partials (m, l, O) in a scratch slot per CTA end; the CTA that arrives last at the pair's
//     counter merges them and stores the row, so no second kernel runs.
//   * The producer prefetches the tiles a few steps ahead into L2 (cp.async.bulk.prefetch.tensor), because
//     shared memory holds two tiles next to the 72 KB query and a tile's slots free up only one tile-time before
//     they are needed again: without the prefetch every tile waited for DRAM.
//   * The softmax threads turn scores into probabilities before they wait for the previous P.V to finish.
//
// Scope: one query per sequence, heads a multiple of 64 (the shapes of a request-split tensor-parallel group and
// of a single GPU).  Other geometries and prefill stay on mla_kernel<NCOL>.  All waits are bounded.
//
// Replaces (by behaviour): flashinfer's trtllm-gen MLA decode as called by
// batchgen/attention/mla/trtllm_gen_mla.py:49-93; contract batchgen/attention/mla/paged_decode.py:1-31.
#include "mla_tcgen05.cuh"

namespace bg {
namespace mla {

constexpr int kPersistThreads = 192;
constexpr int kMaxPairsPersist = 2048;      // (sequence, head group) pairs one launch can schedule
constexpr int kPrefetchTiles = 3;           // how far ahead of the shared-memory loads the L2 prefetch runs
constexpr int kMinChunkTiles = 4;           // a CTA's share is at least this many tiles (tiny batches use fewer CTAs)
constexpr int kPPairs = 8;                  // ring of 16 KB slots (two 64-dim chunks of one tile)
constexpr int kPRope = 2;
constexpr int kPQBytes = 9 * 64 * 128;
constexpr int kPSmemTiles = kPQBytes + kPPairs * kPairBytes + kPRope * kChunkBytes + kPBytes;

struct PersistParams {
  const int* block_table;
  int bt_stride;
  const int* seqlens;
  __nv_bfloat16* out;       // [B, H, 512]
  float* part_o;            // [2 * gridDim.x, 64, 512]
  float* part_ml;           // [2 * gridDim.x, 64, 2]
  unsigned int* counters;   // [pairs], zero between launches (the merging CTA resets its counter)
  int* prefix;              // [gridDim.x, kMaxPairsPersist + 1]: every CTA's own copy of the tile prefix sums
  int B;
  int H;
  int groups;               // H / 64
  float scale_log2;
  int* status;
};

struct PersistShared {
  uint64_t q_full;
  uint64_t q_empty;
  uint64_t pair_full[kPPairs];
  uint64_t pair_empty[kPPairs];
  uint64_t rope_full[kPRope];
  uint64_t rope_empty[kPRope];
  uint64_t s_full[2];
  uint64_t p_full;
  uint64_t o_done;
  uint64_t o_free;
  uint32_t tmem_base;
  int abort_flag;
  int merge_flag;
};

__device__ __forceinline__ void tma_prefetch_l2_2d(const CUtensorMap* map, int c0, int c1) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(map), "r"(c0), "r"(c1)
               : "memory");
}

// One segment: tiles [t0, t1) of pair `pair`.
struct Seg {
  int pair, seq, group;
  int t0, t1;
  int tiles_pair;
  bool whole;        // the segment is the whole pair: normalise and store directly
  int slot;          // partial slot of this CTA for a cut pair
};

// Walks the segments of chunk [cb, ce) of the global tile sequence.  Every role of the CTA builds the same walk.
struct SegWalk {
  const int* prefix;
  int P, groups, cb, ce, p, cta;
  bool first;
  __device__ SegWalk(const int* prefix_, int P_, int groups_, int cb_, int ce_, int cta_)
      : prefix(prefix_), P(P_), groups(groups_), cb(cb_), ce(ce_), cta(cta_), first(true) {
    // first pair with prefix[p + 1] > cb
    int lo = 0, hi = P;
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (prefix[mid + 1] > cb) hi = mid; else lo = mid + 1;
    }
    p = lo;
  }
  __device__ bool next(Seg& s) {
    while (p < P && prefix[p + 1] <= max(prefix[p], cb)) ++p;   // empty pairs and pairs that end before the chunk
    if (p >= P || prefix[p] >= ce) return false;
    const int a = prefix[p], b = prefix[p + 1];
    s.pair = p;
    s.seq = p / groups;
    s.group = p - s.seq * groups;
    s.tiles_pair = b - a;
    s.t0 = max(a, cb) - a;
    s.t1 = min(b, ce) - a;
    s.whole = (s.t0 == 0 && s.t1 == s.tiles_pair);
    s.slot = 2 * cta + (first ? 0 : 1);
    first = false;
    ++p;
    return true;
  }
};

// Flat cursor over the tiles of the chunk (producer: shared-memory loads and the L2 prefetch ahead of them).
struct TileCursor {
  SegWalk walk;
  Seg s;
  int t;
  bool valid;
  __device__ TileCursor(const int* prefix, int P, int groups, int cb, int ce, int cta)
      : walk(prefix, P, groups, cb, ce, cta), t(0), valid(false) {
    valid = walk.next(s);
    if (valid) t = s.t0;
  }
  __device__ void advance() {
    if (!valid) return;
    if (++t >= s.t1) {
      valid = walk.next(s);
      if (valid) t = s.t0;
    }
  }
};

__global__ void __launch_bounds__(kPersistThreads, 1)
mla_decode_persist_kernel(const __grid_constant__ CUtensorMap tm_kv, const __grid_constant__ CUtensorMap tm_q,
                          const __grid_constant__ CUtensorMap tm_qpe, PersistParams p) {
  constexpr int NS = 128;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_buf = smem;
  uint8_t* pair_buf = q_buf + kPQBytes;
  uint8_t* rope_buf = pair_buf + kPPairs * kPairBytes;
  uint8_t* p_buf = rope_buf + kPRope * kChunkBytes;
  PersistShared& ss = *reinterpret_cast<PersistShared*>(p_buf + kPBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort_flag = &ss.abort_flag;
  const int P = p.B * p.groups;

  if (threadIdx.x == 0) {
    mbar_init(&ss.q_full, 1);
    mbar_init(&ss.q_empty, 1);
    for (int i = 0; i < kPPairs; ++i) { mbar_init(&ss.pair_full[i], 1); mbar_init(&ss.pair_empty[i], 1); }
    for (int i = 0; i < kPRope; ++i) { mbar_init(&ss.rope_full[i], 1); mbar_init(&ss.rope_empty[i], 1); }
    mbar_init(&ss.s_full[0], 1);
    mbar_init(&ss.s_full[1], 1);
    mbar_init(&ss.p_full, NS);
    mbar_init(&ss.o_done, 1);
    mbar_init(&ss.o_free, NS);
    ss.abort_flag = 0;
    ss.merge_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&ss.tmem_base, kTmemCols);
    tmem_relinquish();
  }
  // ---- tiles per pair, then an exclusive prefix sum (warp 0: a run of entries per lane, shuffle scan of the lane
  // sums).  The array does not fit next to the tiles in shared memory: each CTA keeps its copy in global scratch,
  // written and read by this CTA only.
  int* prefix = p.prefix + (size_t)blockIdx.x * (kMaxPairsPersist + 1);
  for (int i = threadIdx.x; i < P; i += kPersistThreads) {
    const int len = p.seqlens[i / p.groups];
    prefix[i + 1] = (max(len, 0) + kTile - 1) / kTile;
  }
  if (threadIdx.x == 0) prefix[0] = 0;
  __syncthreads();
  if (warp == 0) {
    const int per = (P + 31) / 32;
    const int a = min(P, lane * per), b = min(P, a + per);
    int sum = 0;
    for (int i = a; i < b; ++i) sum += prefix[i + 1];
    int incl = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    int run = incl - sum;
    for (int i = a; i < b; ++i) {
      run += prefix[i + 1];
      prefix[i + 1] = run;
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ss.tmem_base;
  const int total = prefix[P];
  const int n_cta = gridDim.x;
  const int chunk = max((total + n_cta - 1) / n_cta, kMinChunkTiles);
  const int cb = min(total, (int)blockIdx.x * chunk), ce = min(total, cb + chunk);

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (elect_one()) {
      tma_prefetch_desc(&tm_kv);
      TileCursor cur(prefix, P, p.groups, cb, ce, blockIdx.x);
      TileCursor pre(prefix, P, p.groups, cb, ce, blockIdx.x);
      auto prefetch_tile = [&](const TileCursor& c) {
        const int row0 = p.block_table[(size_t)c.s.seq * p.bt_stride + c.t] * kPage;
#pragma unroll
        for (int ch = 0; ch < 9; ++ch) tma_prefetch_l2_2d(&tm_kv, ch * 64, row0);
      };
      for (int i = 0; i < kPrefetchTiles && pre.valid; ++i) {
        prefetch_tile(pre);
        pre.advance();
      }
      bool ok = true;
      uint32_t pit = 0, rit = 0, seg_no = 0;
      int loaded_pair = -1;
      auto load_q = [&](const Seg& s) -> bool {
        if (seg_no > 0 && !mbar_wait(&ss.q_empty, (seg_no - 1) & 1, abort_flag, kTimeoutProducer)) return false;
        mbar_expect_tx(&ss.q_full, kPQBytes);
        const int grow = s.seq * p.H + s.group * 64;
        for (int c = 0; c < 8; ++c) tma_load_2d(q_buf + c * 64 * 128, &tm_q, &ss.q_full, c * 64, grow);
        tma_load_2d(q_buf + 8 * 64 * 128, &tm_qpe, &ss.q_full, 0, grow);
        ++seg_no;
        return true;
      };
      while (ok && cur.valid) {
        const bool seg_start = (cur.s.pair != loaded_pair);
        // first segment: the query goes first; later segments: the tile first, so that KV keeps streaming while the
        // previous segment's last S still reads the query buffer
        if (seg_start && seg_no == 0) {
          if (!load_q(cur.s)) { ok = false; break; }
          loaded_pair = cur.s.pair;
        }
        const int row0 = p.block_table[(size_t)cur.s.seq * p.bt_stride + cur.t] * kPage;
        for (int m = 0; m < 4 && ok; ++m, ++pit) {
          const int slot = pit % kPPairs;
          if (!mbar_wait(&ss.pair_empty[slot], ((pit / kPPairs) & 1) ^ 1, abort_flag, kTimeoutProducer)) { ok = false; break; }
          mbar_expect_tx(&ss.pair_full[slot], kPairBytes);
          uint8_t* dst = pair_buf + slot * kPairBytes;
          tma_load_2d(dst, &tm_kv, &ss.pair_full[slot], (2 * m) * 64, row0);
          tma_load_2d(dst + kChunkBytes, &tm_kv, &ss.pair_full[slot], (2 * m + 1) * 64, row0);
        }
        if (!ok) break;
        const int rslot = rit % kPRope;
        if (!mbar_wait(&ss.rope_empty[rslot], ((rit / kPRope) & 1) ^ 1, abort_flag, kTimeoutProducer)) { ok = false; break; }
        mbar_expect_tx(&ss.rope_full[rslot], kChunkBytes);
        tma_load_2d(rope_buf + rslot * kChunkBytes, &tm_kv, &ss.rope_full[rslot], 8 * 64, row0);
        ++rit;
        if (seg_start && cur.s.pair != loaded_pair) {
          if (!load_q(cur.s)) { ok = false; break; }
          loaded_pair = cur.s.pair;
        }
        if (pre.valid) {
          prefetch_tile(pre);
          pre.advance();
        }
        cur.advance();
      }
      if (ok) {  // drain: every armed slot is released by the MMA role
        const uint32_t np = pit < (uint32_t)kPPairs ? pit : (uint32_t)kPPairs;
        for (uint32_t j = pit - np; j < pit; ++j)
          if (!mbar_wait(&ss.pair_empty[j % kPPairs], (j / kPPairs) & 1, abort_flag, kTimeoutProducer)) break;
        const uint32_t nr = rit < (uint32_t)kPRope ? rit : (uint32_t)kPRope;
        for (uint32_t j = rit - nr; j < rit; ++j)
          if (!mbar_wait(&ss.rope_empty[j % kPRope], (j / kPRope) & 1, abort_flag, kTimeoutProducer)) break;
      } else {
        for (uint32_t i = 0; i < (1u << 16); ++i) __nanosleep(20);  // bounded grace period for copies in flight
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc_s = make_idesc_bf16(kMRows, kTile, 0, 0);
      constexpr uint32_t idesc_pv = make_idesc_bf16(kMRows, 128, 0, 1);
      const uint32_t tm_o = tmem_base + 2 * kTile;
      SegWalk walk(prefix, P, p.groups, cb, ce, blockIdx.x);
      Seg s;
      bool ok = true;
      uint32_t gt = 0;        // tiles issued so far (S side), over all segments
      uint32_t seg_no = 0;
      // S(tile g) = Q . KV^T over 9 chunks into S buffer g & 1; `last` releases the query buffer afterwards
      auto issue_s = [&](uint32_t g, bool last) -> bool {
        const uint32_t tm_s = tmem_base + (g & 1) * kTile;
        for (int m = 0; m < 4; ++m) {
          const uint32_t pit = g * 4 + m;
          const int slot = pit % kPPairs;
          if (!mbar_wait(&ss.pair_full[slot], (pit / kPPairs) & 1, abort_flag, kTimeoutMma)) return false;
          tc_fence_after();
          for (int cc = 0; cc < 2; ++cc) {
            const uint64_t adesc = make_smem_desc_sw128(smem_u32(q_buf + (2 * m + cc) * 64 * 128));
            const uint64_t bdesc = make_smem_desc_sw128(smem_u32(pair_buf + slot * kPairBytes + cc * kChunkBytes));
#pragma unroll
            for (int k = 0; k < 4; ++k)
              mma_f16(tm_s, adesc + 2 * k, bdesc + 2 * k, idesc_s, (m | cc | k) ? 1u : 0u);
          }
        }
        const int rslot = g % kPRope;
        if (!mbar_wait(&ss.rope_full[rslot], (g / kPRope) & 1, abort_flag, kTimeoutMma)) return false;
        tc_fence_after();
        const uint64_t adesc = make_smem_desc_sw128(smem_u32(q_buf + 8 * 64 * 128));
        const uint64_t bdesc = make_smem_desc_sw128(smem_u32(rope_buf + rslot * kChunkBytes));
#pragma unroll
        for (int k = 0; k < 4; ++k) mma_f16(tm_s, adesc + 2 * k, bdesc + 2 * k, idesc_s, 1u);
        tc_commit(&ss.rope_empty[rslot]);
        tc_commit(&ss.s_full[g & 1]);
        if (last) tc_commit(&ss.q_empty);
        return true;
      };
      while (ok && walk.next(s)) {
        const int n_tiles = s.t1 - s.t0;
        if (!mbar_wait(&ss.q_full, seg_no & 1, abort_flag, kTimeoutMma)) { ok = false; break; }
        tc_fence_after();
        const uint32_t g0 = gt;
        if (!issue_s(g0, n_tiles == 1)) { ok = false; break; }
        for (int t = 0; ok && t < n_tiles; ++t) {
          const uint32_t g = g0 + t;
          bool next_issued = true;
          if (t + 1 < n_tiles) {
            next_issued = mbar_test(&ss.rope_full[(g + 1) % kPRope], ((g + 1) / kPRope) & 1);
            if (next_issued && !issue_s(g + 1, t + 2 == n_tiles)) { ok = false; break; }
          }
          if (t == 0 && seg_no > 0) {       // the previous segment's accumulator must have been read out
            if (!mbar_wait(&ss.o_free, (seg_no - 1) & 1, abort_flag, kTimeoutMma)) { ok = false; break; }
          }
          if (!mbar_wait(&ss.p_full, g & 1, abort_flag, kTimeoutMma)) { ok = false; break; }
          tc_fence_after();
          const uint64_t pdesc = make_smem_desc_sw128(smem_u32(p_buf));
          for (int m = 0; m < 4; ++m) {
            const int slot = (g * 4 + m) % kPPairs;
            const uint32_t b_base = smem_u32(pair_buf + slot * kPairBytes);
            const uint32_t d = tm_o + (m & 1) * 128 + ((m >> 1) ? (16u << 16) : 0u);
#pragma unroll
            for (int j = 0; j < kTile / 16; ++j) {
              const uint64_t bdesc = make_desc_mn_sw128(b_base + j * 2048, kChunkBytes, 1024);
              mma_f16(d, pdesc + 2 * j, bdesc, idesc_pv, (t > 0 || j > 0) ? 1u : 0u);
            }
            tc_commit(&ss.pair_empty[slot]);
          }
          tc_commit(&ss.o_done);
          if (!next_issued && !issue_s(g + 1, t + 2 == n_tiles)) { ok = false; break; }
        }
        gt = g0 + n_tiles;
        ++seg_no;
      }
    }
  } else {
    // ------------------------------------------------------------ softmax / correction / epilogue / merge
    const int quad = warp & 3;
    const bool lo = lane < 16;
    const int col = quad * 16 + (lane & 15);
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t tm_o = tmem_base + 2 * kTile + lane_addr;
    const int src_lane = lane & 15;
    const int stid = threadIdx.x - 64;                 // 0 .. 127
    uint8_t* prow = p_buf + (col >> 3) * 1024 + (col & 7) * 128;
    SegWalk walk(prefix, P, p.groups, cb, ce, blockIdx.x);
    Seg s;
    bool ok = true;
    uint32_t gt = 0, seg_no = 0;
    while (ok && walk.next(s)) {
      const int n_tiles = s.t1 - s.t0;
      const int lim = p.seqlens[s.seq];
      float m_run = -INFINITY, l_run = 0.f;
      for (int t = 0; ok && t < n_tiles; ++t) {
        const uint32_t g = gt + t;
        if (softmax_vote_any<NS>(!mbar_wait(&ss.s_full[g & 1], (g >> 1) & 1, abort_flag, kTimeoutEpilogue))) { ok = false; break; }
        tc_fence_after();
        const int tok0 = (s.t0 + t) * kTile;
        uint32_t sv[64];
        tmem_ld<32>(tmem_base + lane_addr + (g & 1) * kTile, sv);
        tmem_ld<32>(tmem_base + lane_addr + (g & 1) * kTile + 32, sv + 32);
        tmem_ld_wait();
        float mt = -INFINITY;
        const int n_ok = lo ? min(max(lim - tok0, 0), kTile) : 0;
#pragma unroll
        for (int j = 0; j < 64; ++j) {
          const float v = (j < n_ok) ? __uint_as_float(sv[j]) * p.scale_log2 : -INFINITY;
          sv[j] = __float_as_uint(v);
          mt = fmaxf(mt, v);
        }
        const bool grow = mt > m_run + 8.f;
        const float m_new = grow ? mt : m_run;
        const float alpha = (grow && m_run != -INFINITY) ? ex2_approx(m_run - m_new) : 1.f;
        // probabilities first (registers only); the wait for the previous P.V comes after
        uint32_t pk[32];
        float lsum = 0.f;
        if (lo) {
          const float neg_m = (m_new == -INFINITY) ? 0.f : -m_new;
#pragma unroll
          for (int q = 0; q < 32; ++q) {
            const float p0 = ex2_approx(__uint_as_float(sv[2 * q]) + neg_m);
            const float p1 = ex2_approx(__uint_as_float(sv[2 * q + 1]) + neg_m);
            const __nv_bfloat162 o = __floats2bfloat162_rn(p0, p1);
            lsum += __low2float(o) + __high2float(o);
            pk[q] = *reinterpret_cast<const uint32_t*>(&o);
          }
        }
        // the previous tile's second GEMM reads P and accumulates into O: both are touched below
        if (t > 0 && softmax_vote_any<NS>(!mbar_wait(&ss.o_done, (g - 1) & 1, abort_flag, kTimeoutEpilogue))) { ok = false; break; }
        tc_fence_after();
        const float alpha_row = __shfl_sync(0xffffffffu, alpha, src_lane);
        if (t > 0 && __any_sync(0xffffffffu, alpha_row != 1.f)) {
#pragma unroll 1
          for (int c = 0; c < 8; ++c) {
            uint32_t ov[32];
            tmem_ld<32>(tm_o + c * 32, ov);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) ov[j] = __float_as_uint(__uint_as_float(ov[j]) * alpha_row);
            tmem_st<32>(tm_o + c * 32, ov);
          }
          tmem_st_wait();
        }
        if (lo) {
#pragma unroll
          for (int c = 0; c < 8; ++c)
            *reinterpret_cast<uint4*>(prow + ((c ^ (col & 7)) << 4)) = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
          l_run = l_run * alpha + lsum;
          m_run = m_new;
        }
        fence_async_smem();
        tc_fence_before();
        mbar_arrive(&ss.p_full);
      }
      if (!ok) break;
      // ---- read the accumulator out
      const uint32_t g_last = gt + n_tiles - 1;
      if (softmax_vote_any<NS>(!mbar_wait(&ss.o_done, g_last & 1, abort_flag, kTimeoutEpilogue))) { ok = false; break; }
      tc_fence_after();
      const float l_row = __shfl_sync(0xffffffffu, l_run, src_lane);
      const float m_row = __shfl_sync(0xffffffffu, m_run, src_lane);
      const int dim0 = lo ? 0 : 256;
      const float inv = l_row > 0.f ? 1.0f / l_row : 0.f;
      __nv_bfloat16* orow = p.out + ((size_t)s.seq * p.H + s.group * 64 + col) * kLatent + dim0;
      float* prow_o = p.part_o + ((size_t)s.slot * 64 + col) * kLatent + dim0;
#pragma unroll 1
      for (int c = 0; c < 8; ++c) {
        uint32_t ov[32];
        tmem_ld<32>(tm_o + c * 32, ov);
        tmem_ld_wait();
        if (c == 7) {                      // the accumulator is in registers: the next segment may overwrite it
          tc_fence_before();
          mbar_arrive(&ss.o_free);
        }
        if (s.whole) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            __align__(16) __nv_bfloat162 o[4];
#pragma unroll
            for (int q = 0; q < 4; ++q)
              o[q] = __floats2bfloat162_rn(__uint_as_float(ov[j + 2 * q]) * inv, __uint_as_float(ov[j + 2 * q + 1]) * inv);
            *reinterpret_cast<uint4*>(orow + c * 32 + j) = *reinterpret_cast<const uint4*>(o);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; j += 4)
            __stcg(reinterpret_cast<uint4*>(prow_o + c * 32 + j), make_uint4(ov[j], ov[j + 1], ov[j + 2], ov[j + 3]));
        }
      }
      if (!s.whole) {
        if (lo) {
          __stcg(p.part_ml + ((size_t)s.slot * 64 + col) * 2 + 0, m_row);
          __stcg(p.part_ml + ((size_t)s.slot * 64 + col) * 2 + 1, l_row);
        }
        // ---- the CTA that arrives last at the pair's counter merges the pair
        __threadfence();
        softmax_bar<NS>();
        const int a_t = prefix[s.pair], b_t = prefix[s.pair + 1];
        const int ka = a_t / chunk, kb = (b_t - 1) / chunk;
        const int n_seg = kb - ka + 1;
        if (stid == 0) {
          const unsigned int prev = atomicAdd(p.counters + s.pair, 1u);
          ss.merge_flag = (prev == (unsigned int)(n_seg - 1)) ? 1 : 0;
          if (ss.merge_flag) p.counters[s.pair] = 0u;        // ready for the next launch
        }
        softmax_bar<NS>();
        if (ss.merge_flag) {
          __threadfence();
          // warp q merges columns 16q .. 16q + 15; a lane owns dims {4 * lane + 128 * i + 0..3}
          for (int cc = 0; cc < 16; ++cc) {
            const int c2 = quad * 16 + cc;
            float mx = -INFINITY;
            for (int k = ka; k <= kb; ++k) {
              const int sl = 2 * k + ((k == ka && a_t > ka * chunk) ? 1 : 0);
              mx = fmaxf(mx, __ldcg(p.part_ml + ((size_t)sl * 64 + c2) * 2));
            }
            float acc[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) acc[j] = 0.f;
            float l = 0.f;
            for (int k = ka; k <= kb; ++k) {
              const int sl = 2 * k + ((k == ka && a_t > ka * chunk) ? 1 : 0);
              const float ms = __ldcg(p.part_ml + ((size_t)sl * 64 + c2) * 2);
              const float ls = __ldcg(p.part_ml + ((size_t)sl * 64 + c2) * 2 + 1);
              const float f = (ms == -INFINITY) ? 0.f : exp2f(ms - mx);
              l = fmaf(ls, f, l);
              if (f != 0.f) {
                const float4* src = reinterpret_cast<const float4*>(p.part_o + ((size_t)sl * 64 + c2) * kLatent);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const float4 v = __ldcg(src + lane + 32 * i);
                  acc[4 * i + 0] = fmaf(v.x, f, acc[4 * i + 0]);
                  acc[4 * i + 1] = fmaf(v.y, f, acc[4 * i + 1]);
                  acc[4 * i + 2] = fmaf(v.z, f, acc[4 * i + 2]);
                  acc[4 * i + 3] = fmaf(v.w, f, acc[4 * i + 3]);
                }
              }
            }
            const float invl = l > 0.f ? 1.0f / l : 0.f;
            __nv_bfloat16* o = p.out + ((size_t)s.seq * p.H + s.group * 64 + c2) * kLatent;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              __align__(8) __nv_bfloat162 w2[2];
              w2[0] = __floats2bfloat162_rn(acc[4 * i] * invl, acc[4 * i + 1] * invl);
              w2[1] = __floats2bfloat162_rn(acc[4 * i + 2] * invl, acc[4 * i + 3] * invl);
              *reinterpret_cast<uint2*>(o + 4 * lane + 128 * i) = *reinterpret_cast<const uint2*>(w2);
            }
          }
        }
        softmax_bar<NS>();        // merge_flag is rewritten by the next cut segment
      }
      gt += n_tiles;
      ++seg_no;
    }
    // ---- sequences without any token (padding rows of a graph bucket): their output rows are zeros
    for (int pr = blockIdx.x; pr < P; pr += n_cta) {
      if (prefix[pr + 1] != prefix[pr]) continue;
      const int seq = pr / p.groups, grp = pr - seq * p.groups;
      uint4* o = reinterpret_cast<uint4*>(p.out + ((size_t)seq * p.H + grp * 64) * kLatent);
      for (int i = stid; i < 64 * kLatent / 8; i += NS) o[i] = make_uint4(0u, 0u, 0u, 0u);
    }
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
  if (threadIdx.x == 0 && ss.abort_flag != 0 && p.status != nullptr) atomicMax(p.status, ss.abort_flag);
}

}  // namespace mla
}  // namespace bg

extern "C" {

// Scratch sizes of bg_mla_decode_persist for a grid of `ctas` CTAs: floats of part_o and part_ml.
void bg_mla_decode_persist_scratch(int ctas, long long* part_o_floats, long long* part_ml_floats) {
  *part_o_floats = 2ll * ctas * 64 * bg::mla::kLatent;
  *part_ml_floats = 2ll * ctas * 64 * 2;
}

// Paged absorbed MLA decode, one query per sequence, heads % 64 == 0.
// q_abs: [B*H, 512] bf16 with row stride `qabs_stride` elements; q_pe: [B*H, 64] bf16 with row stride `qpe_stride`;
// cache: [cache_rows, 576] bf16 (64-token pages); block_table [B, bt_stride]; seqlens [B]; out [B*H, 512] bf16.
// part_o / part_ml: scratch sized by bg_mla_decode_persist_scratch(ctas); counters: B * H / 64 zeroed uint32
// (left zeroed by the kernel); prefix_scratch: ctas * 2049 ints.  ctas: grid size (<= SM count).
int bg_mla_decode_persist(const void* q_abs, long long qabs_stride, const void* q_pe, long long qpe_stride, int B, int H,
                          const void* cache, long long cache_rows, const int* block_table, int bt_stride,
                          const int* seqlens, void* out, float* part_o, float* part_ml, unsigned int* counters,
                          int* prefix_scratch, int ctas, float scale, int* status, cudaStream_t stream) {
  using namespace bg::mla;
  if (B <= 0) return 0;
  if (H <= 0 || H % 64 != 0 || (qpe_stride * 2) % 16 != 0 || qabs_stride < kLatent || (qabs_stride * 2) % 16 != 0 ||
      ctas <= 0)
    return -1;
  const int groups = H / 64;
  if ((long long)B * groups > kMaxPairsPersist) return -3;
  CUtensorMap tkv, tq, tqpe;
  if (make_map(&tkv, cache, cache_rows, kRow, kRow * 2, kPage) != 0) return -10;
  if (make_map(&tq, q_abs, (long long)B * H, kLatent, qabs_stride * 2, 64) != 0) return -11;
  if (make_map(&tqpe, q_pe, (long long)B * H, kRope, qpe_stride * 2, 64) != 0) return -12;
  PersistParams p;
  p.block_table = block_table; p.bt_stride = bt_stride; p.seqlens = seqlens;
  p.out = reinterpret_cast<__nv_bfloat16*>(out); p.part_o = part_o; p.part_ml = part_ml; p.counters = counters; p.prefix = prefix_scratch;
  p.B = B; p.H = H; p.groups = groups; p.scale_log2 = scale * 1.4426950408889634f; p.status = status;
  static bg::DeviceOnce attr_set;
  const size_t smem = kPSmemTiles + sizeof(PersistShared) + 1024;
  if (!bg::ensure_dynamic_smem(mla_decode_persist_kernel, smem, attr_set)) return -13;
  mla_decode_persist_kernel<<<ctas, kPersistThreads, smem, stream>>>(tkv, tq, tqpe, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -14;
}

}  // extern "C"
