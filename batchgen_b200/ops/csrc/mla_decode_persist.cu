// Persistent paged MLA decode on tcgen05: one CTA per SM walks an equal share of all KV tiles of the batch.
//
// The per-tile machinery is the one of mla_tcgen05.cuh (64 (query, head) columns on the TMEM lanes, 64-token
// tiles, S of tile t+1 issued before P.V of tile t).  What this kernel changes is everything around the tiles,
// which is where a decode step of few rows x many heads spent most of its time:
//
//   * Work is not one CTA per (sequence, head group, split).  The sequences are laid end to end in units of KV
//     tiles, the total is cut into gridDim.x / groups equal chunks, and the CTAs k * groups + g (g = head group of
//     64 heads) all walk chunk k: a run of *segments*, each a range of tiles of one sequence.  The CTAs of one chunk
//     sit next to each other and stream the same tiles at the same pace, so every tile comes from DRAM once and from
//     L2 for the other head groups.  The cut is computed in the kernel from the device-side sequence lengths (every
//     CTA scans the same prefix sums), so a captured CUDA graph balances whatever lengths it is replayed on and no
//     host-side work list or split count exists.
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
#define BG_FILE_TAG 7      // kernel-trace ids of this file are (tag << 16) | line
#include "mla_tcgen05.cuh"

namespace bg {
namespace mla {

constexpr int kPersistThreads = 224;        // producer, S issuer, four softmax warps, P.V issuer
constexpr int kMaxPairsPersist = 2048;      // sequences one launch can schedule
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
  float* part_o;            // [2 * gridDim.x] slots of 64 x 512 floats, see the epilogue for the order inside a slot
  float* part_ml;           // [2 * gridDim.x, 64, 2]
  unsigned int* counters;   // [B * groups], zero between launches (the merging CTA resets its counter)
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
  uint64_t s_free[2];
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

// ---- CTA pairs (thread-block cluster of two): the two head-group CTAs of a chunk walk the same KV tiles, so each
// loads half of every tile from global memory and hands its half to the partner through distributed shared memory
// (a plain shared -> shared::cluster bulk copy; no TMA load is multicast).  KV then crosses the L2 -> SM fabric once
// per tile instead of twice.
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(smem_addr), "r"(rank));
  return out;
}
__device__ __forceinline__ void dsmem_copy(uint32_t dst_cluster, uint32_t src_cta, uint32_t bytes, uint32_t mbar_cluster) {
  asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   dst_cluster),
               "r"(src_cta), "r"(bytes), "r"(mbar_cluster)
               : "memory");
}
// commit that arrives on the barrier at the same offset in every CTA of `mask`
__device__ __forceinline__ void tc_commit_mc(uint64_t* bar, uint16_t mask) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
                   smem_u32(bar)),
               "h"(mask)
               : "memory");
}

// 16 TMEM lanes x 32 columns for each half of the warp: thread i < 16 receives columns [c, c + 32) of lane (base + i),
// thread i + 16 receives columns [c + 32, c + 64) of the same lane.  One score row is thus split between two threads.
__device__ __forceinline__ void tmem_ld_16x32bx2_x32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.16x32bx2.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32], 32;"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
        "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
        "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}

// One segment: tiles [t0, t1) of sequence `seq` (the CTA's head group is fixed); pair = seq * groups + group.
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
  int P, groups, group, cb, ce, p, cta;
  bool first;
  __device__ SegWalk(const int* prefix_, int P_, int groups_, int cb_, int ce_, int cta_)
      : prefix(prefix_), P(P_), groups(groups_), group(cta_ % groups_), cb(cb_), ce(ce_), cta(cta_), first(true) {
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
    s.seq = p;
    s.group = group;
    s.pair = p * groups + group;
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

template <bool PAIR>
__global__ void __launch_bounds__(PAIR ? kPersistThreads + 32 : kPersistThreads, 1)
mla_decode_persist_kernel(const __grid_constant__ CUtensorMap tm_kv, const __grid_constant__ CUtensorMap tm_q,
                          const __grid_constant__ CUtensorMap tm_qpe, PersistParams p) {
  bg::pdl_prologue((BG_FILE_TAG << 16) | __LINE__);
  constexpr int NS = 128;
  const uint32_t crank = PAIR ? cluster_ctarank() : 0u;      // PAIR: warp 7 forwards this CTA's half of every tile
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_buf = smem;
  uint8_t* pair_buf = q_buf + kPQBytes;
  uint8_t* rope_buf = pair_buf + kPPairs * kPairBytes;
  uint8_t* p_buf = rope_buf + kPRope * kChunkBytes;
  PersistShared& ss = *reinterpret_cast<PersistShared*>(p_buf + kPBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort_flag = &ss.abort_flag;
  const int P = p.B;                     // the tile sequence runs over sequences; the head group is the CTA's own

  if (threadIdx.x == 0) {
    mbar_init(&ss.q_full, 1);
    mbar_init(&ss.q_empty, 1);
    for (int i = 0; i < kPPairs; ++i) { mbar_init(&ss.pair_full[i], 1); mbar_init(&ss.pair_empty[i], PAIR ? 2 : 1); }
    for (int i = 0; i < kPRope; ++i) { mbar_init(&ss.rope_full[i], 1); mbar_init(&ss.rope_empty[i], 1); }
    mbar_init(&ss.s_full[0], 1);
    mbar_init(&ss.s_full[1], 1);
    mbar_init(&ss.s_free[0], NS);
    mbar_init(&ss.s_free[1], NS);
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
  for (int i = threadIdx.x; i < P; i += blockDim.x) {
    const int len = p.seqlens[i];
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
  if (PAIR) cluster_sync_all();          // the partner's barriers are initialised before anything arrives on them
  const uint32_t tmem_base = ss.tmem_base;
  const int total = prefix[P];
  const int n_cta = gridDim.x;
  const int n_chunks = max(n_cta / p.groups, 1);
  const int chunk = max((total + n_chunks - 1) / n_chunks, kMinChunkTiles);
  const int my_chunk = blockIdx.x / p.groups;
  const int cb = (my_chunk < n_chunks) ? min(total, my_chunk * chunk) : total;
  const int ce = min(total, cb + chunk);

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (elect_one()) {
      tma_prefetch_desc(&tm_kv);
      TileCursor cur(prefix, P, p.groups, cb, ce, blockIdx.x);
      TileCursor pre(prefix, P, p.groups, cb, ce, blockIdx.x);
      // The page of a tile is looked up once, kPrefetchTiles tiles before the tile is loaded: the lookup (a dependent
      // global load) feeds the L2 prefetch at once and waits in a small register queue for the shared-memory load.
      int rq[kPrefetchTiles];
      auto page_row = [&](const TileCursor& c) {
        return p.block_table[(size_t)c.s.seq * p.bt_stride + c.t] * kPage;
      };
      auto prefetch_rows = [&](int row0) {
        if (PAIR) {                          // only what this CTA loads itself
#pragma unroll
          for (int ch = 0; ch < 4; ++ch) tma_prefetch_l2_2d(&tm_kv, (4 * (int)crank + ch) * 64, row0);
          tma_prefetch_l2_2d(&tm_kv, 8 * 64, row0);
        } else {
#pragma unroll
          for (int ch = 0; ch < 9; ++ch) tma_prefetch_l2_2d(&tm_kv, ch * 64, row0);
        }
      };
#pragma unroll
      for (int i = 0; i < kPrefetchTiles; ++i) {
        rq[i] = 0;
        if (pre.valid) {
          rq[i] = page_row(pre);
          prefetch_rows(rq[i]);
          pre.advance();
        }
      }
      bool ok = true;
      uint32_t pit = 0, rit = 0, seg_no = 0;
      int loaded_pair = -1;
      BG_TR(0, 0, 7);
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
        const int row0 = rq[0];
#pragma unroll
        for (int i = 0; i + 1 < kPrefetchTiles; ++i) rq[i] = rq[i + 1];
        const bool more = pre.valid;
        if (more) rq[kPrefetchTiles - 1] = page_row(pre);      // issued now, first used after this tile's loads
        for (int m = 0; m < 4 && ok; ++m, ++pit) {
          const int slot = pit % kPPairs;
          if (!mbar_wait(&ss.pair_empty[slot], ((pit / kPPairs) & 1) ^ 1, abort_flag, kTimeoutProducer)) { ok = false; break; }
          if (m == 0) BG_TR(0, rit, 0);
          mbar_expect_tx(&ss.pair_full[slot], kPairBytes);
          if (!PAIR || (uint32_t)(m >> 1) == crank) {        // PAIR: the other two slots are filled by the partner
            uint8_t* dst = pair_buf + slot * kPairBytes;
            tma_load_2d(dst, &tm_kv, &ss.pair_full[slot], (2 * m) * 64, row0);
            tma_load_2d(dst + kChunkBytes, &tm_kv, &ss.pair_full[slot], (2 * m + 1) * 64, row0);
          }
        }
        if (!ok) break;
        const int rslot = rit % kPRope;
        if (!mbar_wait(&ss.rope_empty[rslot], ((rit / kPRope) & 1) ^ 1, abort_flag, kTimeoutProducer)) { ok = false; break; }
        mbar_expect_tx(&ss.rope_full[rslot], kChunkBytes);
        tma_load_2d(rope_buf + rslot * kChunkBytes, &tm_kv, &ss.rope_full[rslot], 8 * 64, row0);
        BG_TR(0, rit, 1);
        ++rit;
        if (seg_start && cur.s.pair != loaded_pair) {
          if (!load_q(cur.s)) { ok = false; break; }
          loaded_pair = cur.s.pair;
        }
        if (more) {
          prefetch_rows(rq[kPrefetchTiles - 1]);
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
    // ------------------------------------------------------------ S issuer: S(g) = Q . KV(g)^T, as far ahead as the
    // two score buffers and the tile ring allow (the P.V MMAs are issued by their own warp, so a wait for the
    // softmax never holds back the next tile's scores)
    if (elect_one()) {
      constexpr uint32_t idesc_s = make_idesc_bf16(kMRows, kTile, 0, 0);
      SegWalk walk(prefix, P, p.groups, cb, ce, blockIdx.x);
      Seg s;
      bool ok = true;
      uint32_t g = 0;         // tiles issued so far, over all segments
      uint32_t seg_no = 0;
      while (ok && walk.next(s)) {
        const int n_tiles = s.t1 - s.t0;
        if (!mbar_wait(&ss.q_full, seg_no & 1, abort_flag, kTimeoutMma)) { ok = false; break; }
        tc_fence_after();
        for (int t = 0; ok && t < n_tiles; ++t, ++g) {
          BG_TR(1, g, 0);
          if (g >= 2 && !mbar_wait(&ss.s_free[g & 1], ((g >> 1) - 1) & 1, abort_flag, kTimeoutMma)) { ok = false; break; }
          tc_fence_after();
          const uint32_t tm_s = tmem_base + (g & 1) * kTile;
          for (int mi = 0; mi < 4 && ok; ++mi) {
            const int m = PAIR ? (mi + 2 * (int)crank) & 3 : mi;     // PAIR: the half this CTA loaded itself comes first
            const uint32_t pit = g * 4 + m;
            const int slot = pit % kPPairs;
            if (!mbar_wait(&ss.pair_full[slot], (pit / kPPairs) & 1, abort_flag, kTimeoutMma)) { ok = false; break; }
            tc_fence_after();
            for (int cc = 0; cc < 2; ++cc) {
              const uint64_t adesc = make_smem_desc_sw128(smem_u32(q_buf + (2 * m + cc) * 64 * 128));
              const uint64_t bdesc = make_smem_desc_sw128(smem_u32(pair_buf + slot * kPairBytes + cc * kChunkBytes));
#pragma unroll
              for (int k = 0; k < 4; ++k)
                mma_f16(tm_s, adesc + 2 * k, bdesc + 2 * k, idesc_s, (mi | cc | k) ? 1u : 0u);
            }
          }
          if (!ok) break;
          const int rslot = g % kPRope;
          if (!mbar_wait(&ss.rope_full[rslot], (g / kPRope) & 1, abort_flag, kTimeoutMma)) { ok = false; break; }
          BG_TR(1, g, 1);
          tc_fence_after();
          const uint64_t adesc = make_smem_desc_sw128(smem_u32(q_buf + 8 * 64 * 128));
          const uint64_t bdesc = make_smem_desc_sw128(smem_u32(rope_buf + rslot * kChunkBytes));
#pragma unroll
          for (int k = 0; k < 4; ++k) mma_f16(tm_s, adesc + 2 * k, bdesc + 2 * k, idesc_s, 1u);
          tc_commit(&ss.rope_empty[rslot]);
          tc_commit(&ss.s_full[g & 1]);
          if (t + 1 == n_tiles) tc_commit(&ss.q_empty);      // the query buffer may be refilled for the next segment
          BG_TR(1, g, 2);
        }
        ++seg_no;
      }
    }
  } else if (warp == 6) {
    // ------------------------------------------------------------ P.V issuer: O += P(g) . KV(g)[:, 0:512]
    if (elect_one()) {
      constexpr uint32_t idesc_pv = make_idesc_bf16(kMRows, 128, 0, 1);
      const uint32_t tm_o = tmem_base + 2 * kTile;
      SegWalk walk(prefix, P, p.groups, cb, ce, blockIdx.x);
      Seg s;
      bool ok = true;
      uint32_t g = 0, seg_no = 0;
      while (ok && walk.next(s)) {
        const int n_tiles = s.t1 - s.t0;
        for (int t = 0; ok && t < n_tiles; ++t, ++g) {
          if (t == 0 && seg_no > 0) {       // the previous segment's accumulator must have been read out
            if (!mbar_wait(&ss.o_free, (seg_no - 1) & 1, abort_flag, kTimeoutMma)) { ok = false; break; }
          }
          BG_TR(1, g, 3);
          if (!mbar_wait(&ss.p_full, g & 1, abort_flag, kTimeoutMma)) { ok = false; break; }
          BG_TR(1, g, 4);
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
            if (PAIR) tc_commit_mc(&ss.pair_empty[slot], 0x3);   // the slot is free once both CTAs have read it
            else tc_commit(&ss.pair_empty[slot]);
          }
          tc_commit(&ss.o_done);
          BG_TR(1, g, 5);
        }
        ++seg_no;
      }
    }
  } else if (warp == 7) {
    // ------------------------------------------------------------ PAIR: hand this CTA's half of every tile to the partner
    if (PAIR && elect_one()) {
      const uint32_t peer = crank ^ 1u;
      const int n_tiles = ce - cb;
      bool ok = true;
      for (int g = 0; ok && g < n_tiles; ++g) {
        for (int mm = 0; mm < 2 && ok; ++mm) {
          const uint32_t pit = (uint32_t)g * 4 + 2 * crank + mm;
          const int slot = pit % kPPairs;
          if (!mbar_wait(&ss.pair_full[slot], (pit / kPPairs) & 1, abort_flag, kTimeoutMma)) { ok = false; break; }
          const uint32_t src = smem_u32(pair_buf + slot * kPairBytes);
          dsmem_copy(map_to_cta(src, peer), src, kPairBytes, map_to_cta(smem_u32(&ss.pair_full[slot]), peer));
        }
      }
    }
  } else {
    // ------------------------------------------------------------ softmax / correction / epilogue / merge
    const int quad = warp & 3;
    const bool lo = lane < 16;
    const int col = quad * 16 + (lane & 15);
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t tm_o = tmem_base + 2 * kTile + lane_addr;
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
        if (threadIdx.x == 64) BG_TR(2, g, 0);
        if (softmax_vote_any<NS>(!mbar_wait(&ss.s_full[g & 1], (g >> 1) & 1, abort_flag, kTimeoutEpilogue))) { ok = false; break; }
        if (threadIdx.x == 64) BG_TR(2, g, 1);
        tc_fence_after();
        // lanes 0..15 take tokens 0..31 of the tile for their column, lanes 16..31 tokens 32..63 of the same column
        const int tok0 = (s.t0 + t) * kTile + (lo ? 0 : 32);
        uint32_t sv[32];
        tmem_ld_16x32bx2_x32(tmem_base + lane_addr + (g & 1) * kTile, sv);
        tmem_ld_wait();
        tc_fence_before();
        mbar_arrive(&ss.s_free[g & 1]);                  // the scores are in registers: the buffer may take S(g + 2)
        float mt = -INFINITY;
        const int n_ok = min(max(lim - tok0, 0), 32);
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const float v = (j < n_ok) ? __uint_as_float(sv[j]) * p.scale_log2 : -INFINITY;
          sv[j] = __float_as_uint(v);
          mt = fmaxf(mt, v);
        }
        mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, 16));
        const bool grow = mt > m_run + 8.f;
        const float m_new = grow ? mt : m_run;
        const float alpha = (grow && m_run != -INFINITY) ? ex2_approx(m_run - m_new) : 1.f;
        // probabilities first (registers only); the wait for the previous P.V comes after
        uint32_t pk[16];
        float lsum = 0.f;
        {
          const float neg_m = (m_new == -INFINITY) ? 0.f : -m_new;
#pragma unroll
          for (int q = 0; q < 16; ++q) {
            const float p0 = ex2_approx(__uint_as_float(sv[2 * q]) + neg_m);
            const float p1 = ex2_approx(__uint_as_float(sv[2 * q + 1]) + neg_m);
            const __nv_bfloat162 o = __floats2bfloat162_rn(p0, p1);
            lsum += __low2float(o) + __high2float(o);
            pk[q] = *reinterpret_cast<const uint32_t*>(&o);
          }
        }
        if (threadIdx.x == 64) BG_TR(2, g, 2);
        // the previous tile's second GEMM reads P and accumulates into O: both are touched below
        if (t > 0 && softmax_vote_any<NS>(!mbar_wait(&ss.o_done, (g - 1) & 1, abort_flag, kTimeoutEpilogue))) { ok = false; break; }
        tc_fence_after();
        if (threadIdx.x == 64) BG_TR(2, g, 3);
        if (t > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll 1
          for (int c = 0; c < 8; ++c) {
            uint32_t ov[32];
            tmem_ld<32>(tm_o + c * 32, ov);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) ov[j] = __float_as_uint(__uint_as_float(ov[j]) * alpha);
            tmem_st<32>(tm_o + c * 32, ov);
          }
          tmem_st_wait();
        }
        {
          const int c0 = lo ? 0 : 4;               // 16-byte pieces of the 128-byte P row this lane writes
#pragma unroll
          for (int c = 0; c < 4; ++c)
            *reinterpret_cast<uint4*>(prow + (((c0 + c) ^ (col & 7)) << 4)) = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
          l_run = l_run * alpha + lsum;            // per-lane share of the row sum; the two halves are added at the end
          m_run = m_new;
        }
        fence_async_smem();
        tc_fence_before();
        mbar_arrive(&ss.p_full);
        if (threadIdx.x == 64) BG_TR(2, g, 4);
      }
      if (!ok) break;
      if (threadIdx.x == 64) BG_TR(2, gt + n_tiles - 1, 5);
      // ---- read the accumulator out
      const uint32_t g_last = gt + n_tiles - 1;
      if (softmax_vote_any<NS>(!mbar_wait(&ss.o_done, g_last & 1, abort_flag, kTimeoutEpilogue))) { ok = false; break; }
      tc_fence_after();
      const float l_row = l_run + __shfl_xor_sync(0xffffffffu, l_run, 16);
      const float m_row = m_run;
      const int dim0 = lo ? 0 : 256;
      const float inv = l_row > 0.f ? 1.0f / l_row : 0.f;
      __nv_bfloat16* orow = p.out + ((size_t)s.seq * p.H + s.group * 64 + col) * kLatent + dim0;
      // A partial slot is not row-major: the piece (chunk c, 16-byte group q) of all 128 (column, half) rows is one
      // contiguous 2 KB run, so a warp's store (and the merging warp's load) covers 512 contiguous bytes instead of 32
      // rows 2 KB apart.
      const int rr = quad * 32 + lane;
      uint4* pslot = reinterpret_cast<uint4*>(p.part_o) + (size_t)s.slot * (64 * kLatent / 4);
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
          for (int q = 0; q < 8; ++q)
            __stcg(pslot + (c * 8 + q) * 128 + rr, make_uint4(ov[4 * q], ov[4 * q + 1], ov[4 * q + 2], ov[4 * q + 3]));
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
        const int a_t = prefix[s.seq], b_t = prefix[s.seq + 1];
        const int ka = a_t / chunk, kb = (b_t - 1) / chunk;          // chunks that hold tiles of this sequence
        const int n_seg = kb - ka + 1;
        if (stid == 0) {
          const unsigned int prev = atomicAdd(p.counters + s.pair, 1u);
          ss.merge_flag = (prev == (unsigned int)(n_seg - 1)) ? 1 : 0;
          if (ss.merge_flag) p.counters[s.pair] = 0u;        // ready for the next launch
        }
        softmax_bar<NS>();
        if (ss.merge_flag) {
          __threadfence();
          // slot of chunk k's piece of this sequence: the CTA (k, group) wrote it as its first segment unless the
          // sequence starts inside chunk ka
          auto slot_of = [&](int k) { return 2 * (k * p.groups + s.group) + ((k == ka && a_t > ka * chunk) ? 1 : 0); };
          // every thread merges the (column, half) row it owns in the epilogue layout: weights of the pieces first,
          // then the 256 dims in eight chunks of 32; the loads of two pieces are issued together
          float mx = -INFINITY;
#pragma unroll 4
          for (int k = ka; k <= kb; ++k) mx = fmaxf(mx, __ldcg(p.part_ml + ((size_t)slot_of(k) * 64 + col) * 2));
          float l = 0.f;
#pragma unroll 4
          for (int k = ka; k <= kb; ++k) {
            const float ms = __ldcg(p.part_ml + ((size_t)slot_of(k) * 64 + col) * 2);
            const float ls = __ldcg(p.part_ml + ((size_t)slot_of(k) * 64 + col) * 2 + 1);
            l = fmaf(ls, (ms == -INFINITY) ? 0.f : exp2f(ms - mx), l);
          }
          const float invl = l > 0.f ? 1.0f / l : 0.f;
#pragma unroll 1
          for (int c = 0; c < 8; ++c) {
            float acc[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) acc[j] = 0.f;
            for (int k0 = ka; k0 <= kb; k0 += 2) {
              uint4 v[2][8];
              float f[2];
#pragma unroll
              for (int u = 0; u < 2; ++u) {
                const int k = min(k0 + u, kb);
                const int sl = slot_of(k);
                const float ms = __ldcg(p.part_ml + ((size_t)sl * 64 + col) * 2);
                f[u] = (k0 + u > kb || ms == -INFINITY) ? 0.f : exp2f(ms - mx);
                const uint4* src = reinterpret_cast<const uint4*>(p.part_o) + (size_t)sl * (64 * kLatent / 4) + c * 8 * 128 + rr;
#pragma unroll
                for (int q = 0; q < 8; ++q) v[u][q] = __ldcg(src + q * 128);
              }
#pragma unroll
              for (int u = 0; u < 2; ++u) {
                if (f[u] == 0.f) continue;            // an empty piece's partial is undefined
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                  acc[4 * q + 0] = fmaf(__uint_as_float(v[u][q].x), f[u], acc[4 * q + 0]);
                  acc[4 * q + 1] = fmaf(__uint_as_float(v[u][q].y), f[u], acc[4 * q + 1]);
                  acc[4 * q + 2] = fmaf(__uint_as_float(v[u][q].z), f[u], acc[4 * q + 2]);
                  acc[4 * q + 3] = fmaf(__uint_as_float(v[u][q].w), f[u], acc[4 * q + 3]);
                }
              }
            }
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              __align__(16) __nv_bfloat162 o[4];
#pragma unroll
              for (int q = 0; q < 4; ++q) o[q] = __floats2bfloat162_rn(acc[j + 2 * q] * invl, acc[j + 2 * q + 1] * invl);
              *reinterpret_cast<uint4*>(orow + c * 32 + j) = *reinterpret_cast<const uint4*>(o);
            }
          }
        }
        softmax_bar<NS>();        // merge_flag is rewritten by the next cut segment
      }
      if (threadIdx.x == 64) BG_TR(2, gt + n_tiles - 1, 6);
      gt += n_tiles;
      ++seg_no;
    }
    // ---- sequences without any token (padding rows of a graph bucket): their output rows are zeros
    for (int pr = blockIdx.x; pr < P * p.groups; pr += n_cta) {
      const int seq = pr / p.groups, grp = pr - seq * p.groups;
      if (prefix[seq + 1] != prefix[seq]) continue;
      uint4* o = reinterpret_cast<uint4*>(p.out + ((size_t)seq * p.H + grp * 64) * kLatent);
      for (int i = stid; i < 64 * kLatent / 8; i += NS) o[i] = make_uint4(0u, 0u, 0u, 0u);
    }
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (PAIR) cluster_sync_all();          // neither CTA leaves while the partner may still write into or signal it
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
  if (B > kMaxPairsPersist || groups > ctas) return -3;
  CUtensorMap tkv, tq, tqpe;
  if (make_map(&tkv, cache, cache_rows, kRow, kRow * 2, kPage) != 0) return -10;
  if (make_map(&tq, q_abs, (long long)B * H, kLatent, qabs_stride * 2, 64) != 0) return -11;
  if (make_map(&tqpe, q_pe, (long long)B * H, kRope, qpe_stride * 2, 64) != 0) return -12;
  PersistParams p;
  p.block_table = block_table; p.bt_stride = bt_stride; p.seqlens = seqlens;
  p.out = reinterpret_cast<__nv_bfloat16*>(out); p.part_o = part_o; p.part_ml = part_ml; p.counters = counters; p.prefix = prefix_scratch;
  p.B = B; p.H = H; p.groups = groups; p.scale_log2 = scale * 1.4426950408889634f; p.status = status;
  static bg::DeviceOnce attr_set, attr_set_pair;
  const size_t smem = kPSmemTiles + sizeof(PersistShared) + 1024;
  static const bool pair_on = [] {
    const char* e = getenv("BG_MLA_PAIR");
    return e != nullptr && e[0] == '1';
  }();
  if (pair_on && groups == 2 && ctas >= 2) {
    // CTA pairs: both head groups of a chunk in one cluster.  The grid is cut to the number of pairs that can be
    // resident at once (a GPC with an odd number of free SMs cannot host a last pair: a second wave of a persistent
    // kernel would double its time).
    auto kern = mla_decode_persist_kernel<true>;
    if (!bg::ensure_dynamic_smem(kern, smem, attr_set_pair)) return -13;
    static int max_pairs[bg::kMaxDevices] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < bg::kMaxDevices && max_pairs[dev] == 0) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(ctas & ~1);
      cfg.blockDim = dim3(kPersistThreads + 32);
      cfg.dynamicSmemBytes = smem;
      cudaLaunchAttribute at[1];
      at[0].id = cudaLaunchAttributeClusterDimension;
      at[0].val.clusterDim.x = 2;
      at[0].val.clusterDim.y = 1;
      at[0].val.clusterDim.z = 1;
      cfg.attrs = at;
      cfg.numAttrs = 1;
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) n = -1;
      max_pairs[dev] = n;
    }
    const int mp = (dev >= 0 && dev < bg::kMaxDevices) ? max_pairs[dev] : -1;
    if (mp > 0) {
      int grid = ctas & ~1;
      if (grid > 2 * mp) grid = 2 * mp;
      bg::launch_pdl_cluster(kern, dim3(grid), dim3(kPersistThreads + 32), dim3(2, 1, 1), smem, stream, tkv, tq, tqpe, p);
      return cudaGetLastError() == cudaSuccess ? 0 : -14;
    }
  }
  if (!bg::ensure_dynamic_smem(mla_decode_persist_kernel<false>, smem, attr_set)) return -13;
  bg::launch_pdl(mla_decode_persist_kernel<false>, dim3(ctas), dim3(kPersistThreads), smem, stream, tkv, tq, tqpe, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -14;
}

}  // extern "C"

BG_TRACE_SETTER(mla_decode_persist)
