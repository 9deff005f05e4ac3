// Absorbed multi-head latent attention over the paged latent KV cache on tcgen05 tensor cores.
//
// One kernel serves decode (one query per sequence), multi-query prefill chunks (causal) and
// split-KV partials.  The latent cache row is 576 bf16 = 512 (normalised c_kv, also the value) +
// 64 (roped k_pe).  A CTA owns up to 64 (query, head) "columns" of one sequence and walks its KV range
// in 64-token tiles (one page, loaded once by TMA as 9 swizzled 64-dim chunks that feed both GEMMs):
//
//   S[col, tok]   = Q[col, 0:576] . KV[tok, 0:576]          (M = 64 columns, N = 64 tokens; both K-major)
//   O[col, dim]  += P[col, tok] . KV[tok, dim]              (M = 64, N = 128 dims per MMA, B read N-major)
//
// With the columns on the TMEM lanes the softmax needs no cross-thread reduction at all: one thread
// owns one column, reads its 64 scores with tcgen05.ld, keeps the running maximum and sum in registers,
// and writes its probabilities as one swizzled 128-byte row of the A operand of the second GEMM.  The
// accumulator is rescaled (in TMEM, by the thread that owns the row) only when a maximum grew by more
// than 2^8, so most tiles skip it.  An M = 64 accumulator occupies lanes 0..15 of each 32-lane TMEM
// quadrant; O[:, 0:256] uses those and O[:, 256:512] the lanes 16..31 at the same columns.
//
// Pipeline: shared memory holds two to three tiles, so the MMA warp issues S of tile t+1 before the
// second GEMM of tile t whenever that tile has landed; the tensor pipe then works on S(t+1) while the
// softmax warps turn S(t) into P(t), and the loads of tiles t+2.. are already in flight.
//
// Roles (192 threads): warp 0 TMA producer, warp 1 MMA issuer + TMEM owner, warps 2..5 softmax /
// correction / epilogue.  All waits are bounded (see common.cuh).
//
// Replaces (by behaviour): FlashMLA flash_mla_with_kvcache as used by
// batchgen/attention/mla/flashmla_backend.py:1202-1400, the flashinfer trtllm-gen MLA decode the
// reference uses on Blackwell (batchgen/attention/mla/trtllm_gen_mla.py:49-93), contract
// batchgen/attention/mla/paged_decode.py:1-31.
#pragma once
#include "common.cuh"

namespace bg {
namespace mla {

// Optional per-role timestamps of CTA 0 (diagnostic builds only: -DBG_MLA_TRACE).
#ifdef BG_MLA_TRACE
__device__ long long g_mla_trace[3 * 32 * 8];
#define BG_TR(role, t, ev)                                                                   \
  do {                                                                                       \
    if (blockIdx.x == 0 && (t) < 32) g_mla_trace[((role) * 32 + (t)) * 8 + (ev)] = clock64(); \
  } while (0)
#else
#define BG_TR(role, t, ev) do {} while (0)
#endif

constexpr int kLatent = 512;
constexpr int kRope = 64;
constexpr int kRow = kLatent + kRope;     // 576
constexpr int kPage = 64;
constexpr int kTile = 64;                 // KV tokens per tile (= 1 page)
constexpr int kChunkBytes = kTile * 128;  // one 64-dim chunk of a tile: 64 rows x 128 B
constexpr int kPairBytes = 2 * kChunkBytes;

struct Work {
  int q_row;      // first query row (rows are [R, H, *])
  int n_q;        // queries handled (columns = n_q * heads_per_group <= NCOL)
  int seq;        // row of the block table / seqlens
  int ctx_base;   // >= 0: query i sees ctx_base + i + 1 tokens (prefill); < 0: seqlens[seq] (decode)
  int split;      // this CTA's share of the KV tiles
  int n_splits;
  int head_group; // first head = head_group * heads_per_group
  int out_slot;   // partial-output slot (split path)
};

struct Params {
  const Work* work;
  const int* block_table;
  int bt_stride;
  const int* seqlens;
  __nv_bfloat16* out;     // [R, H, 512]
  float* part_o;          // [slots, NCOL, 512]   (split path)
  float* part_ml;         // [slots, NCOL, 2]     (m, l)
  int H;
  int heads_per_group;
  float scale_log2;       // softmax scale * log2(e)
  int* status;
};

constexpr int kMRows = 64;                // MMA M: (query, head) columns per CTA, padded
constexpr int kPBytes = kMRows * kTile * 2;   // P: 64 rows x 128 B, one swizzle atom

template <int NCOL> struct Cfg {
  // shared memory: Q (9 chunks x NCOL rows x 128 B), a ring of 16 KB slots (two 64-dim chunks of one
  // 64-token tile), a ring of 8 KB rope chunks, and P.  Q comes first: the M = 64 descriptor of a Q chunk
  // with fewer than 64 rows reads on into the ring (rows that are never used), not past the allocation.
  static constexpr int kPairs = NCOL == 64 ? 8 : 10;
  static constexpr int kRopeSlots = NCOL == 16 ? 3 : 2;
  static constexpr int kQBytes = 9 * NCOL * 128;
  static constexpr int kSmemTiles = kQBytes + kPairs * kPairBytes + kRopeSlots * kChunkBytes + kPBytes;
};
constexpr int kThreads = 192;
constexpr int kTmemCols = 512;            // S: 2 x 64 columns; O: 256 columns x two lane halves
constexpr int kMaxPairs = 10;
constexpr int kMaxRopeSlots = 3;

struct Shared {
  uint64_t q_full;
  uint64_t pair_full[kMaxPairs];
  uint64_t pair_empty[kMaxPairs];
  uint64_t rope_full[kMaxRopeSlots];
  uint64_t rope_empty[kMaxRopeSlots];
  uint64_t s_full[2];
  uint64_t p_full;
  uint64_t o_done;
  uint32_t tmem_base;
  int abort_flag;
  int limit[64];
};

// no-swizzle K-major descriptor (core matrices of 8 rows x 16 bytes)
__device__ __forceinline__ uint64_t make_desc_nosw(uint32_t addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(lbo >> 4) << 16;
  d |= static_cast<uint64_t>(sbo >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  return d;
}
// MN-major 128B-swizzled descriptor: lbo = distance between 64-element atoms along M,
// sbo = distance between 8-row groups along K.
__device__ __forceinline__ uint64_t make_desc_mn_sw128(uint32_t addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(lbo >> 4) << 16;
  d |= static_cast<uint64_t>(sbo >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}
__host__ __device__ constexpr uint32_t make_idesc_bf16(int M, int N, int a_mn_major, int b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(a_mn_major) << 15) |
         (static_cast<uint32_t>(b_mn_major) << 16) | (static_cast<uint32_t>(N >> 3) << 17) |
         (static_cast<uint32_t>(M >> 4) << 24);
}
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int N> __device__ __forceinline__ void tmem_ld(uint32_t taddr, uint32_t* v);
template <> __device__ __forceinline__ void tmem_ld<16>(uint32_t taddr, uint32_t* v) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}
template <> __device__ __forceinline__ void tmem_ld<32>(uint32_t taddr, uint32_t* v) {
  tmem_ld<16>(taddr, v);
  tmem_ld<16>(taddr + 16, v + 16);
}
template <int N> __device__ __forceinline__ void tmem_st(uint32_t taddr, const uint32_t* v);
template <> __device__ __forceinline__ void tmem_st<16>(uint32_t taddr, const uint32_t* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
      "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
      : "memory");
}
template <> __device__ __forceinline__ void tmem_st<32>(uint32_t taddr, const uint32_t* v) {
  tmem_st<16>(taddr, v);
  tmem_st<16>(taddr + 16, v + 16);
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
template <int N> __device__ __forceinline__ void softmax_bar() {
  asm volatile("bar.sync 1, %0;" ::"n"(N) : "memory");
}
// Barrier over the softmax threads that also ORs a flag, so that a bounded wait that expired in one
// thread makes every thread leave the loop together (no thread is left alone at a barrier).
template <int N> __device__ __forceinline__ bool softmax_vote_any(bool v) {
  uint32_t r;
  asm volatile(
      "{\n"
      ".reg .pred p, q;\n"
      "setp.ne.u32 q, %1, 0;\n"
      "bar.red.or.pred p, 2, %2, q;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(r)
      : "r"(static_cast<uint32_t>(v)), "n"(N)
      : "memory");
  return r != 0;
}
// Non-blocking probe of an mbarrier phase.
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

template <int NCOL>
__global__ void __launch_bounds__(kThreads, 1)
mla_kernel(const __grid_constant__ CUtensorMap tm_kv, const __grid_constant__ CUtensorMap tm_q,
           const __grid_constant__ CUtensorMap tm_qpe, Params p) {
  bg::pdl_prologue((BG_FILE_TAG << 16) | __LINE__);
  using C = Cfg<NCOL>;
  constexpr int NS = 128;                                       // softmax threads
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_buf = smem;                                        // 9 chunks x NCOL rows x 128 B
  uint8_t* pair_buf = q_buf + C::kQBytes;                       // kPairs x 16 KB
  uint8_t* rope_buf = pair_buf + C::kPairs * kPairBytes;        // kRopeSlots x 8 KB
  uint8_t* p_buf = rope_buf + C::kRopeSlots * kChunkBytes;      // P: 64 rows x 128 B, K-major swizzled
  Shared& ss = *reinterpret_cast<Shared*>(p_buf + kPBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort_flag = &ss.abort_flag;
  const Work w = p.work[blockIdx.x];
  const int hpg = p.heads_per_group;

  if (threadIdx.x == 0) {
    mbar_init(&ss.q_full, 1);
    for (int i = 0; i < C::kPairs; ++i) { mbar_init(&ss.pair_full[i], 1); mbar_init(&ss.pair_empty[i], 1); }
    for (int i = 0; i < C::kRopeSlots; ++i) { mbar_init(&ss.rope_full[i], 1); mbar_init(&ss.rope_empty[i], 1); }
    mbar_init(&ss.s_full[0], 1);
    mbar_init(&ss.s_full[1], 1);
    mbar_init(&ss.p_full, NS);
    mbar_init(&ss.o_done, 1);
    ss.abort_flag = 0;
    mbar_fence_init();
  }
  if (threadIdx.x < 64) {
    int lim = 0;
    if (threadIdx.x < NCOL) {
      const int qi = threadIdx.x / hpg;
      if (qi < w.n_q) lim = (w.ctx_base < 0) ? p.seqlens[w.seq] : (w.ctx_base + qi + 1);
    }
    ss.limit[threadIdx.x] = lim;
  }
  if (warp == 1) {
    tmem_alloc(&ss.tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ss.tmem_base;

  int max_limit = 0;
#pragma unroll 1
  for (int j = 0; j < NCOL; ++j) max_limit = max(max_limit, ss.limit[j]);
  const int n_tiles_total = (max_limit + kTile - 1) / kTile;      // = pages in use
  const int tile_begin = (int)(((long long)n_tiles_total * w.split) / w.n_splits);
  const int tile_end = (int)(((long long)n_tiles_total * (w.split + 1)) / w.n_splits);
  const int n_tiles = tile_end - tile_begin;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (elect_one()) {
      tma_prefetch_desc(&tm_kv);
      // Q: rows (q_row + qi) * H + head_group * hpg .. + hpg, 8 latent chunks + 1 rope chunk
      mbar_expect_tx(&ss.q_full, C::kQBytes);
      for (int qi = 0; qi < NCOL / hpg; ++qi) {
        const int grow = (w.q_row + min(qi, w.n_q - 1)) * p.H + w.head_group * hpg;
        for (int c = 0; c < 8; ++c)
          tma_load_2d(q_buf + c * NCOL * 128 + qi * hpg * 128, &tm_q, &ss.q_full, c * 64, grow);
        tma_load_2d(q_buf + 8 * NCOL * 128 + qi * hpg * 128, &tm_qpe, &ss.q_full, 0, grow);
      }
      const int* bt = p.block_table + (size_t)w.seq * p.bt_stride;
      bool ok = true;
      uint32_t pit = 0, rit = 0;
      for (int t = 0; ok && t < n_tiles; ++t) {
        const int row0 = bt[tile_begin + t] * kPage;          // a tile is one page
        for (int m = 0; m < 4 && ok; ++m, ++pit) {
          const int slot = pit % C::kPairs;
          if (!mbar_wait(&ss.pair_empty[slot], ((pit / C::kPairs) & 1) ^ 1, abort_flag, kTimeoutProducer)) { ok = false; break; }
          mbar_expect_tx(&ss.pair_full[slot], kPairBytes);
          uint8_t* dst = pair_buf + slot * kPairBytes;
          tma_load_2d(dst, &tm_kv, &ss.pair_full[slot], (2 * m) * 64, row0);
          tma_load_2d(dst + kChunkBytes, &tm_kv, &ss.pair_full[slot], (2 * m + 1) * 64, row0);
        }
        if (!ok) break;
        const int rslot = rit % C::kRopeSlots;
        if (!mbar_wait(&ss.rope_empty[rslot], ((rit / C::kRopeSlots) & 1) ^ 1, abort_flag, kTimeoutProducer)) { ok = false; break; }
        mbar_expect_tx(&ss.rope_full[rslot], kChunkBytes);
        tma_load_2d(rope_buf + rslot * kChunkBytes, &tm_kv, &ss.rope_full[rslot], 8 * 64, row0);
        BG_TR(0, t, 0);
        ++rit;
      }
      if (ok) {  // drain: every armed slot is released by the MMA role
        const uint32_t np = pit < (uint32_t)C::kPairs ? pit : (uint32_t)C::kPairs;
        for (uint32_t j = pit - np; j < pit; ++j)
          if (!mbar_wait(&ss.pair_empty[j % C::kPairs], (j / C::kPairs) & 1, abort_flag, kTimeoutProducer)) break;
        const uint32_t nr = rit < (uint32_t)C::kRopeSlots ? rit : (uint32_t)C::kRopeSlots;
        for (uint32_t j = rit - nr; j < rit; ++j)
          if (!mbar_wait(&ss.rope_empty[j % C::kRopeSlots], (j / C::kRopeSlots) & 1, abort_flag, kTimeoutProducer)) break;
      } else {
        for (uint32_t i = 0; i < (1u << 16); ++i) __nanosleep(20);  // bounded grace period for copies in flight
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc_s = make_idesc_bf16(kMRows, kTile, 0, 0);     // Q . KV^T: both K-major
      constexpr uint32_t idesc_pv = make_idesc_bf16(kMRows, 128, 0, 1);      // P . V: V read N-major (dims contiguous)
      const uint32_t tm_o = tmem_base + 2 * kTile;
      bool ok = mbar_wait(&ss.q_full, 0, abort_flag, kTimeoutMma);
      // S(t) = Q . KV(t)^T over 9 chunks, into S buffer t & 1
      auto issue_s = [&](int t) -> bool {
        BG_TR(1, t, 0);
        const uint32_t tm_s = tmem_base + (t & 1) * kTile;
        for (int m = 0; m < 4; ++m) {
          const uint32_t pit = (uint32_t)t * 4 + m;
          const int slot = pit % C::kPairs;
          if (!mbar_wait(&ss.pair_full[slot], (pit / C::kPairs) & 1, abort_flag, kTimeoutMma)) return false;
          tc_fence_after();
          for (int cc = 0; cc < 2; ++cc) {
            const uint64_t adesc = make_smem_desc_sw128(smem_u32(q_buf + (2 * m + cc) * NCOL * 128));
            const uint64_t bdesc = make_smem_desc_sw128(smem_u32(pair_buf + slot * kPairBytes + cc * kChunkBytes));
#pragma unroll
            for (int k = 0; k < 4; ++k)
              mma_f16(tm_s, adesc + 2 * k, bdesc + 2 * k, idesc_s, (m | cc | k) ? 1u : 0u);
          }
        }
        const int rslot = t % C::kRopeSlots;
        if (!mbar_wait(&ss.rope_full[rslot], (t / C::kRopeSlots) & 1, abort_flag, kTimeoutMma)) return false;
        BG_TR(1, t, 1);
        tc_fence_after();
        const uint64_t adesc = make_smem_desc_sw128(smem_u32(q_buf + 8 * NCOL * 128));
        const uint64_t bdesc = make_smem_desc_sw128(smem_u32(rope_buf + rslot * kChunkBytes));
#pragma unroll
        for (int k = 0; k < 4; ++k) mma_f16(tm_s, adesc + 2 * k, bdesc + 2 * k, idesc_s, 1u);
        tc_commit(&ss.rope_empty[rslot]);
        tc_commit(&ss.s_full[t & 1]);
        BG_TR(1, t, 2);
        return true;
      };
      if (ok && n_tiles > 0) ok = issue_s(0);
      for (int t = 0; ok && t < n_tiles; ++t) {
        // S of the next tile goes first when that tile has already landed (its rope chunk is the last
        // load of a tile); otherwise the second GEMM of this tile is not held up behind the loads
        bool next_issued = true;
        if (t + 1 < n_tiles) {
          next_issued = mbar_test(&ss.rope_full[(t + 1) % C::kRopeSlots], ((t + 1) / C::kRopeSlots) & 1);
          if (next_issued && !issue_s(t + 1)) { ok = false; break; }
        }
        // ---- O += P . V : four 128-dim blocks; blocks 2, 3 accumulate in the upper lane halves
        BG_TR(1, t, 3);
        if (!mbar_wait(&ss.p_full, t & 1, abort_flag, kTimeoutMma)) { ok = false; break; }
        BG_TR(1, t, 4);
        tc_fence_after();
        const uint64_t pdesc = make_smem_desc_sw128(smem_u32(p_buf));
        for (int m = 0; m < 4; ++m) {
          const int slot = ((uint32_t)t * 4 + m) % C::kPairs;
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
        BG_TR(1, t, 5);
        if (!next_issued && !issue_s(t + 1)) { ok = false; break; }
      }
    }
  } else {
    // ------------------------------------------------------------ softmax / correction / epilogue
    // Lanes 0..15 of warp q own columns 16q .. 16q+15: their S rows and O[:, 0:256].  Lanes 16..31 own
    // O[:, 256:512] of the same columns (TMEM lanes 16..31 of the quadrant) and idle during the softmax.
    const int quad = warp & 3;
    const bool lo = lane < 16;
    const int col = quad * 16 + (lane & 15);
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t tm_o = tmem_base + 2 * kTile + lane_addr;
    const int lim = ss.limit[col];
    const int src_lane = lane & 15;
    float m_run = -INFINITY, l_run = 0.f;          // in scaled (log2) units; valid in lanes 0..15
    uint8_t* prow = p_buf + (col >> 3) * 1024 + (col & 7) * 128;
    bool ok = true;
    for (int t = 0; ok && t < n_tiles; ++t) {
      if (threadIdx.x == 64) BG_TR(2, t, 0);
      if (softmax_vote_any<NS>(!mbar_wait(&ss.s_full[t & 1], (t >> 1) & 1, abort_flag, kTimeoutEpilogue))) { ok = false; break; }
      tc_fence_after();
      if (threadIdx.x == 64) BG_TR(2, t, 1);
      const int tok0 = (tile_begin + t) * kTile;
      uint32_t sv[64];
      tmem_ld<32>(tmem_base + lane_addr + (t & 1) * kTile, sv);
      tmem_ld<32>(tmem_base + lane_addr + (t & 1) * kTile + 32, sv + 32);
      tmem_ld_wait();
      float mt = -INFINITY;
      const int n_ok = lo ? min(max(lim - tok0, 0), kTile) : 0;      // tokens of this tile the column may see
#pragma unroll
      for (int j = 0; j < 64; ++j) {
        const float v = (j < n_ok) ? __uint_as_float(sv[j]) * p.scale_log2 : -INFINITY;
        sv[j] = __float_as_uint(v);
        mt = fmaxf(mt, v);
      }
      // keep the old maximum unless it grew by more than 2^8: probabilities stay below 256 and the
      // accumulator is rescaled rarely
      const bool grow = mt > m_run + 8.f;
      const float m_new = grow ? mt : m_run;
      const float alpha = (grow && m_run != -INFINITY) ? ex2_approx(m_run - m_new) : 1.f;
      if (threadIdx.x == 64) BG_TR(2, t, 2);
      // The previous tile's second GEMM reads P and accumulates into O: both are touched below.
      if (t > 0 && softmax_vote_any<NS>(!mbar_wait(&ss.o_done, (t - 1) & 1, abort_flag, kTimeoutEpilogue))) { ok = false; break; }
      tc_fence_after();
      if (threadIdx.x == 64) BG_TR(2, t, 3);
      const float alpha_row = __shfl_sync(0xffffffffu, alpha, src_lane);     // upper lanes: the factor of their column
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
      if (threadIdx.x == 64) BG_TR(2, t, 4);
      if (lo) {
        // probabilities -> one swizzled 128-byte row of P (the K-major A operand of the second GEMM)
        float lsum = 0.f;
        const float neg_m = (m_new == -INFINITY) ? 0.f : -m_new;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          __align__(16) __nv_bfloat162 o[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float p0 = ex2_approx(__uint_as_float(sv[c * 8 + 2 * q]) + neg_m);
            const float p1 = ex2_approx(__uint_as_float(sv[c * 8 + 2 * q + 1]) + neg_m);
            o[q] = __floats2bfloat162_rn(p0, p1);
            lsum += __low2float(o[q]) + __high2float(o[q]);
          }
          *reinterpret_cast<uint4*>(prow + ((c ^ (col & 7)) << 4)) = *reinterpret_cast<const uint4*>(o);
        }
        l_run = l_run * alpha + lsum;
        m_run = m_new;
      }
      fence_async_smem();
      tc_fence_before();
      mbar_arrive(&ss.p_full);
      if (threadIdx.x == 64) BG_TR(2, t, 5);
    }
    // ---- epilogue
    if (ok && n_tiles > 0)
      ok = !softmax_vote_any<NS>(!mbar_wait(&ss.o_done, (n_tiles - 1) & 1, abort_flag, kTimeoutEpilogue));
    if (ok) {
      tc_fence_after();
      const float l_row = __shfl_sync(0xffffffffu, l_run, src_lane);
      const float m_row = __shfl_sync(0xffffffffu, m_run, src_lane);
      const int qi = col / hpg, hl = col % hpg;
      const bool col_ok = col < NCOL && qi < w.n_q;
      const bool direct = (w.n_splits == 1);
      const int dim0 = lo ? 0 : 256;
      const float inv = l_row > 0.f ? 1.0f / l_row : 0.f;
      __nv_bfloat16* orow = p.out + ((size_t)(w.q_row + qi) * p.H + w.head_group * hpg + hl) * kLatent + dim0;
      float* prow_o = direct ? nullptr : p.part_o + ((size_t)w.out_slot * NCOL + col) * kLatent + dim0;
#pragma unroll 1
      for (int c = 0; c < 8; ++c) {
        uint32_t ov[32];
        if (n_tiles > 0) {
          tmem_ld<32>(tm_o + c * 32, ov);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) ov[j] = 0u;
        }
        if (!col_ok) continue;
        if (direct) {
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
            *reinterpret_cast<uint4*>(prow_o + c * 32 + j) = make_uint4(ov[j], ov[j + 1], ov[j + 2], ov[j + 3]);
        }
      }
      if (!direct && lo && col_ok) {
        p.part_ml[((size_t)w.out_slot * NCOL + col) * 2 + 0] = m_row;
        p.part_ml[((size_t)w.out_slot * NCOL + col) * 2 + 1] = l_row;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
  if (threadIdx.x == 0 && ss.abort_flag != 0 && p.status != nullptr) atomicMax(p.status, ss.abort_flag);
}

// Merge split-KV partials: one block per (work item, column); slot of split s = first_slot[item] + s.  A block's
// loads do not depend on one another (no early exit between them), so the splits' rows stream in together.
static __global__ void __launch_bounds__(128)
mla_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, const int* __restrict__ items,
                 __nv_bfloat16* __restrict__ out, int ncol, int H, int hpg) {
  bg::pdl_prologue((BG_FILE_TAG << 16) | __LINE__);
  // items[i] = {q_row, n_q, head_group, first_slot, n_splits}
  const int* it = items + blockIdx.x * 5;
  const int q_row = it[0], n_q = it[1], hg = it[2], first = it[3], ns = it[4];
  const int j = blockIdx.y;
  const int qi = j / hpg, hl = j % hpg;
  if (qi >= n_q) return;
  const float* ml = part_ml + ((size_t)first * ncol + j) * 2;
  const size_t ml_step = (size_t)ncol * 2, o_step = (size_t)ncol * kLatent;
  float m = -INFINITY;
  for (int s = 0; s < ns; ++s) m = fmaxf(m, ml[s * ml_step]);
  float l = 0.f;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  const float* po = part_o + ((size_t)first * ncol + j) * kLatent + threadIdx.x;
#pragma unroll 4
  for (int s = 0; s < ns; ++s) {
    const float ms = ml[s * ml_step], ls = ml[s * ml_step + 1];
    const float f = (ms == -INFINITY) ? 0.f : exp2f(ms - m);
    l = fmaf(ls, f, l);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float v = po[s * o_step + 128 * q];
      acc[q] = (f == 0.f) ? acc[q] : fmaf(v, f, acc[q]);        // an empty split's partial row is undefined
    }
  }
  const float inv = l > 0.f ? 1.0f / l : 0.f;
  __nv_bfloat16* o = out + ((size_t)(q_row + qi) * H + hg * hpg + hl) * kLatent;
#pragma unroll
  for (int q = 0; q < 4; ++q) o[threadIdx.x + 128 * q] = __float2bfloat16(acc[q] * inv);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}
static int make_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t row_stride_bytes,
                    uint32_t box_rows) {
  EncodeTiledFn enc = get_encode();
  if (enc == nullptr) return -1;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -2;
}

// Sets the kernel's shared-memory limit on the current device (once per device and column variant).  Callers that
// must not run attribute calls later (a stream capture in progress) call this for every variant up front.
template <int NCOL>
static bool prepare_device() {
  static DeviceOnce attr_set;
  return ensure_dynamic_smem(mla_kernel<NCOL>, Cfg<NCOL>::kSmemTiles + sizeof(Shared) + 1024, attr_set);
}

template <int NCOL>
static int launch(const CUtensorMap& kv, const CUtensorMap& q, const CUtensorMap& qpe, const Params& p, int n_work,
                  cudaStream_t stream) {
  auto kern = mla_kernel<NCOL>;
  const size_t smem = Cfg<NCOL>::kSmemTiles + sizeof(Shared) + 1024;
  if (!prepare_device<NCOL>()) return -12;
  bg::launch_pdl(kern, dim3(n_work), dim3(kThreads), smem, stream, kv, q, qpe, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -13;
}

}  // namespace mla
}  // namespace bg

