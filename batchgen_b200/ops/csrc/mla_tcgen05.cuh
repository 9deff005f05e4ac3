// Absorbed multi-head latent attention over the paged latent KV cache on tcgen05 tensor cores.
//
// One kernel serves decode (one query per sequence), multi-query prefill chunks (causal) and
// split-KV partials.  The latent cache row is 576 bf16 = 512 (normalised c_kv, also the value) +
// 64 (roped k_pe).  Because MLA has a single KV head, the natural tensor-core shape puts the KV
// *tokens* on the M axis and the (query, head) pairs on the N axis:
//
//   S^T[tok, col]  = KV[tok, 0:576] . Q[col, 0:576]          (A = KV tile, K-major;  B = Q, K-major)
//   O^T[dim, col] += KV[tok, dim]^T . P^T[tok, col]          (A = same KV tile read MN-major;  B = P^T)
//
// so a 128-token KV tile is loaded once by TMA (9 swizzled 64-dim chunks) and feeds both GEMMs, with
// N = 16 or 32 columns per CTA (e.g. the 16 heads of one tensor-parallel rank, or 32 of 128 heads).
// S^T and the four 128-dim blocks of O^T live in TMEM.  The softmax runs over TMEM lanes (one
// thread per token): column maxima are reduced with warp shuffles + shared memory, probabilities go
// to shared memory as the B operand of the second GEMM, and O^T is rescaled in TMEM only when a
// running maximum moves.
//
// Roles (192 threads): warp 0 TMA producer, warp 1 MMA issuer + TMEM owner, warps 2..5 softmax /
// correction / epilogue (thread = TMEM lane).  All waits are bounded (see common.cuh).
//
// Replaces (by behaviour): FlashMLA flash_mla_with_kvcache as used by
// batchgen/attention/mla/flashmla_backend.py:1202-1400, the flashinfer trtllm-gen MLA decode the
// reference uses on Blackwell (batchgen/attention/mla/trtllm_gen_mla.py:49-93), contract
// batchgen/attention/mla/paged_decode.py:1-31.
#pragma once
#include "common.cuh"

namespace bg {
namespace mla {

constexpr int kLatent = 512;
constexpr int kRope = 64;
constexpr int kRow = kLatent + kRope;     // 576
constexpr int kPage = 64;
constexpr int kTile = 128;                // KV tokens per tile (= 2 pages)
constexpr int kChunkBytes = kTile * 128;  // one 64-dim chunk of a tile: 128 rows x 128 B
constexpr int kPairBytes = 2 * kChunkBytes;
constexpr int kThreads = 192;
constexpr int kRopeSlots = 2;

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

template <int NCOL> struct Cfg {
  static constexpr int kPairs = NCOL == 16 ? 5 : 4;
  static constexpr int kQBytes = 9 * NCOL * 128;
  static constexpr int kPBytes = NCOL * kTile * 2;
  static constexpr int kTmemCols = NCOL == 16 ? 128 : 256;
  static constexpr int kSmemTiles = kPairs * kPairBytes + kRopeSlots * kChunkBytes + kQBytes + kPBytes;
};

struct Shared {
  uint64_t q_full;
  uint64_t pair_full[5];
  uint64_t pair_empty[5];
  uint64_t rope_full[kRopeSlots];
  uint64_t rope_empty[kRopeSlots];
  uint64_t s_full;
  uint64_t p_full;
  uint64_t o_done;
  uint32_t tmem_base;
  int abort_flag;
  int limit[32];
  float red[4][32];
  float alpha_flag;
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
__host__ __device__ constexpr uint32_t make_idesc_bf16(int M, int N, int a_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(a_mn_major) << 15) |
         (static_cast<uint32_t>(N >> 3) << 17) | (static_cast<uint32_t>(M >> 4) << 24);
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
__device__ __forceinline__ void softmax_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
// Barrier over the 128 softmax threads that also ORs a flag, so that a bounded wait that expired in
// one thread makes every thread leave the loop together (no thread is left alone at a barrier).
__device__ __forceinline__ bool softmax_vote_any(bool v) {
  uint32_t r;
  asm volatile(
      "{\n"
      ".reg .pred p, q;\n"
      "setp.ne.u32 q, %1, 0;\n"
      "bar.red.or.pred p, 2, 128, q;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(r)
      : "r"(static_cast<uint32_t>(v))
      : "memory");
  return r != 0;
}

template <int NCOL>
__global__ void __launch_bounds__(kThreads, 1)
mla_kernel(const __grid_constant__ CUtensorMap tm_kv, const __grid_constant__ CUtensorMap tm_q,
           const __grid_constant__ CUtensorMap tm_qpe, Params p) {
  using C = Cfg<NCOL>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* pair_buf = smem;                                     // kPairs x 32 KB
  uint8_t* rope_buf = pair_buf + C::kPairs * kPairBytes;        // 2 x 16 KB
  uint8_t* q_buf = rope_buf + kRopeSlots * kChunkBytes;         // 9 chunks x NCOL rows x 128 B
  uint8_t* p_buf = q_buf + C::kQBytes;                          // P^T, no-swizzle K-major
  Shared& ss = *reinterpret_cast<Shared*>(p_buf + C::kPBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort_flag = &ss.abort_flag;
  const Work w = p.work[blockIdx.x];
  const int hpg = p.heads_per_group;

  if (threadIdx.x == 0) {
    mbar_init(&ss.q_full, 1);
    for (int i = 0; i < C::kPairs; ++i) { mbar_init(&ss.pair_full[i], 1); mbar_init(&ss.pair_empty[i], 1); }
    for (int i = 0; i < kRopeSlots; ++i) { mbar_init(&ss.rope_full[i], 1); mbar_init(&ss.rope_empty[i], 1); }
    mbar_init(&ss.s_full, 1);
    mbar_init(&ss.p_full, 128);
    mbar_init(&ss.o_done, 1);
    ss.abort_flag = 0;
    mbar_fence_init();
  }
  if (threadIdx.x < 32) {
    int lim = 0;
    if (threadIdx.x < NCOL) {
      const int qi = threadIdx.x / hpg;
      if (qi < w.n_q) lim = (w.ctx_base < 0) ? p.seqlens[w.seq] : (w.ctx_base + qi + 1);
    }
    ss.limit[threadIdx.x] = lim;
  }
  if (warp == 1) {
    tmem_alloc(&ss.tmem_base, C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ss.tmem_base;

  int max_limit = 0;
#pragma unroll 1
  for (int j = 0; j < NCOL; ++j) max_limit = max(max_limit, ss.limit[j]);
  const int n_tiles_total = (max_limit + kTile - 1) / kTile;
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
      const int n_pages = (max_limit + kPage - 1) / kPage;
      bool ok = true;
      uint32_t pit = 0, rit = 0;
      for (int t = 0; ok && t < n_tiles; ++t) {
        const int tile = tile_begin + t;
        int page_id[2];
        for (int h = 0; h < 2; ++h) {
          const int pi = tile * 2 + h;
          page_id[h] = bt[pi < n_pages ? pi : 0];   // past-the-end halves re-read a valid page; they are masked
        }
        for (int m = 0; m < 4 && ok; ++m, ++pit) {
          const int slot = pit % C::kPairs;
          if (!mbar_wait(&ss.pair_empty[slot], ((pit / C::kPairs) & 1) ^ 1, abort_flag, kTimeoutProducer)) { ok = false; break; }
          mbar_expect_tx(&ss.pair_full[slot], kPairBytes);
          uint8_t* dst = pair_buf + slot * kPairBytes;
          for (int cc = 0; cc < 2; ++cc)
            for (int h = 0; h < 2; ++h)
              tma_load_2d(dst + cc * kChunkBytes + h * (kPage * 128), &tm_kv, &ss.pair_full[slot], (2 * m + cc) * 64,
                          page_id[h] * kPage);
        }
        if (!ok) break;
        const int rslot = rit % kRopeSlots;
        if (!mbar_wait(&ss.rope_empty[rslot], ((rit / kRopeSlots) & 1) ^ 1, abort_flag, kTimeoutProducer)) { ok = false; break; }
        mbar_expect_tx(&ss.rope_full[rslot], kChunkBytes);
        for (int h = 0; h < 2; ++h)
          tma_load_2d(rope_buf + rslot * kChunkBytes + h * (kPage * 128), &tm_kv, &ss.rope_full[rslot], 8 * 64,
                      page_id[h] * kPage);
        ++rit;
      }
      if (ok) {  // drain: every armed slot is released by the MMA role
        const uint32_t np = pit < (uint32_t)C::kPairs ? pit : (uint32_t)C::kPairs;
        for (uint32_t j = pit - np; j < pit; ++j)
          if (!mbar_wait(&ss.pair_empty[j % C::kPairs], (j / C::kPairs) & 1, abort_flag, kTimeoutProducer)) break;
        const uint32_t nr = rit < (uint32_t)kRopeSlots ? rit : (uint32_t)kRopeSlots;
        for (uint32_t j = rit - nr; j < rit; ++j)
          if (!mbar_wait(&ss.rope_empty[j % kRopeSlots], (j / kRopeSlots) & 1, abort_flag, kTimeoutProducer)) break;
      } else {
        for (uint32_t i = 0; i < (1u << 16); ++i) __nanosleep(20);  // bounded grace period for copies in flight
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, NCOL, 0);
      constexpr uint32_t idesc_pv = make_idesc_bf16(128, NCOL, 1);
      const uint32_t tm_s = tmem_base;
      const uint32_t tm_o = tmem_base + NCOL;
      bool ok = mbar_wait(&ss.q_full, 0, abort_flag, kTimeoutMma);
      uint32_t pit = 0, rit = 0;
      for (int t = 0; ok && t < n_tiles; ++t) {
        const uint32_t pit0 = pit;
        // ---- S^T = KV . Q^T over 9 chunks
        for (int m = 0; m < 4 && ok; ++m, ++pit) {
          const int slot = pit % C::kPairs;
          if (!mbar_wait(&ss.pair_full[slot], (pit / C::kPairs) & 1, abort_flag, kTimeoutMma)) { ok = false; break; }
          tc_fence_after();
          for (int cc = 0; cc < 2; ++cc) {
            const uint64_t adesc = make_smem_desc_sw128(smem_u32(pair_buf + slot * kPairBytes + cc * kChunkBytes));
            const uint64_t bdesc = make_smem_desc_sw128(smem_u32(q_buf + (2 * m + cc) * NCOL * 128));
#pragma unroll
            for (int k = 0; k < 4; ++k)
              mma_f16(tm_s, adesc + 2 * k, bdesc + 2 * k, idesc_s, (m | cc | k) ? 1u : 0u);
          }
        }
        if (!ok) break;
        {
          const int rslot = rit % kRopeSlots;
          if (!mbar_wait(&ss.rope_full[rslot], (rit / kRopeSlots) & 1, abort_flag, kTimeoutMma)) { ok = false; break; }
          tc_fence_after();
          const uint64_t adesc = make_smem_desc_sw128(smem_u32(rope_buf + rslot * kChunkBytes));
          const uint64_t bdesc = make_smem_desc_sw128(smem_u32(q_buf + 8 * NCOL * 128));
#pragma unroll
          for (int k = 0; k < 4; ++k) mma_f16(tm_s, adesc + 2 * k, bdesc + 2 * k, idesc_s, 1u);
          tc_commit(&ss.rope_empty[rslot]);
          tc_commit(&ss.s_full);
          ++rit;
        }
        // ---- O^T += V^T . P^T
        if (!mbar_wait(&ss.p_full, t & 1, abort_flag, kTimeoutMma)) { ok = false; break; }
        tc_fence_after();
        for (int m = 0; m < 4; ++m) {
          const int slot = (pit0 + m) % C::kPairs;
          const uint32_t a_base = smem_u32(pair_buf + slot * kPairBytes);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const uint64_t adesc = make_desc_mn_sw128(a_base + j * 2048, kChunkBytes, 1024);
            const uint64_t bdesc = make_desc_nosw(smem_u32(p_buf + j * (NCOL / 8) * 256), 128, 256);
            mma_f16(tm_o + m * NCOL, adesc, bdesc, idesc_pv, (t > 0 || j > 0) ? 1u : 0u);
          }
          tc_commit(&ss.pair_empty[slot]);
        }
        tc_commit(&ss.o_done);
      }
    }
  } else {
    // ------------------------------------------------------------ softmax / correction / epilogue
    const int sw = warp - 2;                 // 0..3
    const int quad = warp & 3;               // TMEM lane quadrant of this warp
    const int row = quad * 32 + lane;        // token within the tile; later: dim within an O^T block
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t tm_s = tmem_base + lane_addr;
    const uint32_t tm_o = tmem_base + NCOL + lane_addr;
    float m_run[NCOL], l_part[NCOL];
#pragma unroll
    for (int j = 0; j < NCOL; ++j) { m_run[j] = -INFINITY; l_part[j] = 0.f; }
    bool ok = true;
    for (int t = 0; ok && t < n_tiles; ++t) {
      if (softmax_vote_any(!mbar_wait(&ss.s_full, t & 1, abort_flag, kTimeoutEpilogue))) { ok = false; break; }
      tc_fence_after();
      uint32_t sv[NCOL];
      tmem_ld<NCOL>(tm_s, sv);
      tmem_ld_wait();
      const int tok = (tile_begin + t) * kTile + row;
      float s[NCOL], tmax[NCOL];
#pragma unroll
      for (int j = 0; j < NCOL; ++j) {
        s[j] = (tok < ss.limit[j]) ? __uint_as_float(sv[j]) * p.scale_log2 : -INFINITY;
        tmax[j] = warp_max(s[j]);
      }
      if (lane == 0) {
#pragma unroll
        for (int j = 0; j < NCOL; ++j) ss.red[sw][j] = tmax[j];
      }
      softmax_bar();
      bool changed = false;
      float alpha[NCOL];
#pragma unroll
      for (int j = 0; j < NCOL; ++j) {
        const float mt = fmaxf(fmaxf(ss.red[0][j], ss.red[1][j]), fmaxf(ss.red[2][j], ss.red[3][j]));
        const float mn = fmaxf(m_run[j], mt);
        alpha[j] = (mn == -INFINITY) ? 1.f : exp2f(m_run[j] - mn);   // m_run = -inf -> 0 (nothing accumulated yet)
        changed |= (mn > m_run[j]);
        m_run[j] = mn;
      }
      if (changed && t > 0) {
        // running maxima moved: rescale the accumulators (O^T in TMEM, l in registers).  The previous
        // tile's second GEMM has completed: its commit precedes this tile's s_full in issue order.
#pragma unroll 1
        for (int blk = 0; blk < 4; ++blk) {
          uint32_t ov[NCOL];
          tmem_ld<NCOL>(tm_o + blk * NCOL, ov);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < NCOL; ++j) ov[j] = __float_as_uint(__uint_as_float(ov[j]) * alpha[j]);
          tmem_st<NCOL>(tm_o + blk * NCOL, ov);
        }
        tmem_st_wait();
#pragma unroll
        for (int j = 0; j < NCOL; ++j) l_part[j] *= alpha[j];
      }
      // probabilities -> shared memory (B operand, K-major core matrices: [k-step][col/8][k-half][col%8][tok%8])
#pragma unroll
      for (int j = 0; j < NCOL; ++j) {
        const float pj = (s[j] == -INFINITY) ? 0.f : exp2f(s[j] - m_run[j]);
        const __nv_bfloat16 pb = __float2bfloat16(pj);
        l_part[j] += __bfloat162float(pb);
        const uint32_t off = (row >> 4) * ((NCOL / 8) * 256) + (j >> 3) * 256 + ((row >> 3) & 1) * 128 + (j & 7) * 16 +
                             (row & 7) * 2;
        *reinterpret_cast<__nv_bfloat16*>(p_buf + off) = pb;
      }
      fence_async_smem();
      tc_fence_before();
      mbar_arrive(&ss.p_full);
      softmax_bar();   // red[] is reused by the next tile
    }
    // ---- epilogue
    if (ok && n_tiles > 0)
      ok = !softmax_vote_any(!mbar_wait(&ss.o_done, (n_tiles - 1) & 1, abort_flag, kTimeoutEpilogue));
    if (ok) {
      tc_fence_after();
      // total row sums: reduce the per-thread partials over the 128 token lanes
      float l_tot[NCOL];
#pragma unroll
      for (int j = 0; j < NCOL; ++j) l_tot[j] = warp_sum(l_part[j]);
      softmax_bar();
      if (lane == 0) {
#pragma unroll
        for (int j = 0; j < NCOL; ++j) ss.red[sw][j] = l_tot[j];
      }
      softmax_bar();
#pragma unroll
      for (int j = 0; j < NCOL; ++j) l_tot[j] = ss.red[0][j] + ss.red[1][j] + ss.red[2][j] + ss.red[3][j];
      const bool direct = (w.n_splits == 1);
#pragma unroll 1
      for (int blk = 0; blk < 4; ++blk) {
        uint32_t ov[NCOL];
        if (n_tiles > 0) {
          tmem_ld<NCOL>(tm_o + blk * NCOL, ov);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < NCOL; ++j) ov[j] = 0u;
        }
        const int dim = blk * 128 + row;
#pragma unroll
        for (int j = 0; j < NCOL; ++j) {
          const int qi = j / hpg, hl = j % hpg;
          if (qi >= w.n_q) continue;
          const float o = __uint_as_float(ov[j]);
          if (direct) {
            const float inv = l_tot[j] > 0.f ? 1.0f / l_tot[j] : 0.f;
            p.out[((size_t)(w.q_row + qi) * p.H + w.head_group * hpg + hl) * kLatent + dim] = __float2bfloat16(o * inv);
          } else {
            p.part_o[((size_t)w.out_slot * NCOL + j) * kLatent + dim] = o;
          }
        }
      }
      if (!direct && threadIdx.x == 64) {
        for (int j = 0; j < NCOL; ++j) {
          p.part_ml[((size_t)w.out_slot * NCOL + j) * 2 + 0] = m_run[j];
          p.part_ml[((size_t)w.out_slot * NCOL + j) * 2 + 1] = l_tot[j];
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, C::kTmemCols);
  if (threadIdx.x == 0 && ss.abort_flag != 0 && p.status != nullptr) atomicMax(p.status, ss.abort_flag);
}

// Merge split-KV partials: one block per (row, head); slot of split s = first_slot[item] + s.
static __global__ void __launch_bounds__(128)
mla_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, const int* __restrict__ items,
                 __nv_bfloat16* __restrict__ out, int ncol, int H, int hpg) {
  // items[i] = {q_row, n_q, head_group, first_slot, n_splits}
  const int* it = items + blockIdx.x * 5;
  const int q_row = it[0], n_q = it[1], hg = it[2], first = it[3], ns = it[4];
  for (int j = 0; j < ncol; ++j) {
    const int qi = j / hpg, hl = j % hpg;
    if (qi >= n_q) continue;
    float m = -INFINITY;
    for (int s = 0; s < ns; ++s) m = fmaxf(m, part_ml[((size_t)(first + s) * ncol + j) * 2]);
    float l = 0.f;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < ns; ++s) {
      const float ms = part_ml[((size_t)(first + s) * ncol + j) * 2];
      const float ls = part_ml[((size_t)(first + s) * ncol + j) * 2 + 1];
      if (ms == -INFINITY) continue;
      const float f = exp2f(ms - m);
      l += ls * f;
      const float* po = part_o + ((size_t)(first + s) * ncol + j) * kLatent;
#pragma unroll
      for (int q = 0; q < 4; ++q) acc[q] += po[threadIdx.x + 128 * q] * f;
    }
    const float inv = l > 0.f ? 1.0f / l : 0.f;
    __nv_bfloat16* o = out + ((size_t)(q_row + qi) * H + hg * hpg + hl) * kLatent;
#pragma unroll
    for (int q = 0; q < 4; ++q) o[threadIdx.x + 128 * q] = __float2bfloat16(acc[q] * inv);
  }
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

template <int NCOL>
static int launch(const CUtensorMap& kv, const CUtensorMap& q, const CUtensorMap& qpe, const Params& p, int n_work,
                  cudaStream_t stream) {
  static bool attr_set = false;
  auto kern = mla_kernel<NCOL>;
  const size_t smem = Cfg<NCOL>::kSmemTiles + sizeof(Shared) + 1024;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return -12;
    attr_set = true;
  }
  kern<<<n_work, kThreads, smem, stream>>>(kv, q, qpe, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -13;
}

}  // namespace mla
}  // namespace bg

