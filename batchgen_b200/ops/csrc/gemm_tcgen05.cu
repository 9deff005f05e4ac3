// Block-scaled FP8 (e4m3) and bf16 GEMM on the 5th-generation tensor cores: dense and ragged
// grouped (per-expert) forms in one persistent, warp-specialised kernel.
//
//   D[m, n] = sum_kb  sA[m, kb] * sB[n / 128, kb] * ( A[m, kb*128 : +128] . B[n, kb*128 : +128] )
//
// A is the activation [M, K] (1x128 scales), B the weight [N, K] (128x128 scales), both
// K-major, so every operand tile is a TMA box of 128-byte rows in the 128B-swizzled layout that
// tcgen05.mma reads directly.  The tensor core has no fp32 block scaling, so each 128-wide K
// block is multiplied into its own TMEM accumulator (double buffered) and the epilogue warps
// fold it into fp32 registers with the block's scale while the next block is being multiplied.
//
// Roles (320 threads, one CTA per SM, persistent over tiles):
//   warp 0      TMA producer (one elected lane)
//   warp 1      TMEM allocator + tcgen05.mma issuer (one elected lane)
//   warps 2..9  epilogue: warp w owns TMEM lanes 32*(w%4).. and columns 64*((w-2)/4)..
//
// Replaces (by behaviour): DeepGEMM fp8_gemm_nt / m_grouped contiguous as called from
// batchgen/gemm/w8a8_deepgemm.py:126 and batchgen/moe/grouped_fp8_deepgemm_moe.py:45-232, the
// CuTe sm90 blockwise grouped GEMM batchgen_kernels/src/moe/fp8_blockwise/fp8_blockwise_gemm_kernel.cuh:363
// and its fused gate+up+SiLU stage batchgen_kernels/src/moe/fp8_blockwise/fp8_blockwise_s1_kernel.cuh:131.
#define BG_FILE_TAG 5      // kernel-trace ids of this file are (tag << 16) | line
#include "common.cuh"

namespace bg {

constexpr int BM = 128;
constexpr int BN = 128;
constexpr int BK_BYTES = 128;  // one swizzle atom of K per stage
constexpr int kStages = 6;
constexpr int kThreads = 320;
constexpr int kEpiWarps = 8;
constexpr int kTmemCols = 256;  // two 128-column accumulators
constexpr int kMaxGroups = 1024;
constexpr int kEpiStageBytes = 16 * 128;   // per epilogue warp: 16 rows x 64 bf16, staging for peer-bound rows

constexpr int KIND_FP8 = 0;
constexpr int KIND_BF16 = 1;
constexpr int EPI_STORE = 0;
constexpr int EPI_SILU_MUL = 1;  // B rows interleaved (32 gate, 32 up): out = silu(gate) * up
constexpr int EPI_STORE_F32 = 2;  // fp32 output (router logits): D is float*, ldd in floats

struct GemmParams {
  const float* sA;      // [KB, sa_stride] (transposed: scale of row m, block kb at sA[kb*sa_stride+m])
  int sa_stride;
  const float* sB;      // [groups, ceil(Nw/128), KB]
  __nv_bfloat16* D;     // [M, ldd]
  int ldd;
  const int* offsets;   // [groups+1] device row offsets, every segment start 128-aligned; null = dense
  const int* counts;    // [groups] rows really present in each segment (null: offsets[g+1] - offsets[g]); rows
                        // past the count are neither multiplied as whole tiles nor stored
  int groups;
  int M;                // rows of A (dense) / capacity of A (grouped)
  int N;                // rows of B per group (GEMM N)
  int K;                // elements
  int* status;
  // ---- hooks that fuse the GEMM with a collective over peer memory (all optional) -------------
  // all-gather -> GEMM: rows [i*a_ready_rows, (i+1)*a_ready_rows) of A were pushed into this GPU's
  // memory by rank i; they are valid once a_ready[i] >= epoch.  The TMA producer waits per tile.
  const uint32_t* a_ready;
  int a_ready_rows;
  uint32_t epoch;              // compared / published value = epoch + *epoch_base (base lives on the device so
  const uint32_t* epoch_base;  // that a captured CUDA graph advances its epochs from replay to replay)
  int m_rotate;         // dense: row block processed first (tiles rotate, e.g. local rows first / last)
  // GEMM -> reduce-scatter / combine: the epilogue stores each output row into the memory of the
  // rank that owns it.  row_map[row] = (rank, dest row) (rank < 0: drop the row); without a map row m
  // goes to rank m / rs_rows_per_rank, dest row my_rank * rs_rows_per_rank + m % rs_rows_per_rank.
  void* peer_out[8];
  const int2* row_map;
  int rs_rows_per_rank;
  int my_rank, world;
  // completion: when the last CTA finishes, peer_flags[r][done_flag_index + my_rank] = epoch for all r
  uint32_t* peer_flags[8];
  int done_flag_index;
  unsigned int* done_counter;
  // split K (dense GEMMs with too few output tiles to fill the SMs): work item = (tile, split); every split
  // accumulates its range of K blocks, parks the fp32 partial tile in `splitk_ws` and bumps the tile's counter; the
  // split that arrives last sums all partials in split order (one summation order whoever is last), runs the
  // epilogue and clears the counter.
  int splits;
  float* splitk_ws;       // [tiles * splits][64][kEpiWarps * 32]
  int* splitk_cnt;        // [tiles], zero between launches
};

struct SharedStorage {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  int split_last;
  int offs[kMaxGroups + 1];
  int cnt[kMaxGroups];
};

struct Tile {
  int g;      // group (expert)
  int m0;     // first row in A / D
  int m_end;  // one past the last valid row
  int nt;     // n tile
};

// Deterministic tile walk shared by all roles.  Dense: tile -> (nt, mt) with mt fastest.
// Grouped: groups in order, inside a group nt-major with mt fastest.
struct TileWalker {
  const int* offs;
  const int* cnt;
  int groups, n_tiles, M, m_rotate;
  int g, before;  // grouped walk state: current group and number of tiles in earlier groups
  __device__ TileWalker(const int* offs_, const int* cnt_, int groups_, int n_tiles_, int M_, int m_rotate_ = 0)
      : offs(offs_), cnt(cnt_), groups(groups_), n_tiles(n_tiles_), M(M_), m_rotate(m_rotate_), g(0), before(0) {}
  __device__ bool get(int tile, Tile& t) {
    if (offs == nullptr) {
      const int m_tiles = (M + BM - 1) / BM;
      if (tile >= m_tiles * n_tiles) return false;
      t.g = 0;
      t.nt = tile / m_tiles;
      t.m0 = (((tile % m_tiles) + m_rotate) % m_tiles) * BM;
      t.m_end = M;
      return true;
    }
    while (g < groups) {
      const int rows = cnt[g];
      const int m_tiles = (rows + BM - 1) / BM;
      const int here = m_tiles * n_tiles;
      if (tile < before + here) {
        const int local = tile - before;
        t.g = g;
        t.nt = local / m_tiles;
        t.m0 = offs[g] + (local % m_tiles) * BM;
        t.m_end = offs[g] + rows;
        return true;
      }
      before += here;
      ++g;
    }
    return false;
  }
};

template <int KIND, int EPI>
__global__ void __launch_bounds__(kThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, GemmParams p) {
  bg::pdl_prologue((BG_FILE_TAG << 16) | __LINE__);
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // carve: operand stages first (1024-byte aligned), bookkeeping after
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA_tiles = smem;
  uint8_t* sB_tiles = smem + kStages * BM * BK_BYTES;
  SharedStorage& ss = *reinterpret_cast<SharedStorage*>(smem + kStages * (BM + BN) * BK_BYTES);
  uint8_t* epi_stage = smem + kStages * (BM + BN) * BK_BYTES + ((sizeof(SharedStorage) + 15) & ~size_t(15));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t epoch = p.epoch + (p.epoch_base != nullptr ? *p.epoch_base : 0u);
  constexpr int kElemBytes = (KIND == KIND_FP8) ? 1 : 2;
  constexpr int BK = BK_BYTES / kElemBytes;  // elements of K per stage
  const int KB = p.K / BK;
  const int S = p.splits > 1 ? p.splits : 1;     // K splits per output tile
  const int n_tiles = (p.N + BN - 1) / BN;
  const int nblk = (p.N + 127) / 128;
  volatile int* abort_flag = &ss.abort_flag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&ss.full[s], 1);
      mbar_init(&ss.empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&ss.tmem_full[b], 1);
      mbar_init(&ss.tmem_empty[b], kEpiWarps);
    }
    ss.abort_flag = 0;
    mbar_fence_init();
  }
  if (p.offsets != nullptr) {
    for (int i = threadIdx.x; i <= p.groups; i += kThreads) ss.offs[i] = p.offsets[i];
    for (int i = threadIdx.x; i < p.groups; i += kThreads) {
      const int padded = p.offsets[i + 1] - p.offsets[i];
      ss.cnt[i] = p.counts != nullptr ? min(max(p.counts[i], 0), padded) : padded;
    }
  }
  if (warp == 1) {
    tmem_alloc(&ss.tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ss.tmem_base;
  const int* offs = (p.offsets != nullptr) ? ss.offs : nullptr;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (elect_one()) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      TileWalker walk(offs, ss.cnt, p.groups, n_tiles, p.M, p.m_rotate);
      Tile t;
      uint32_t it = 0;
      uint32_t ready_mask = 0;
      bool ok = true;
      for (int item = blockIdx.x; ok && walk.get(item / S, t); item += gridDim.x) {
        const int sp = item % S;
        const int kb0 = sp * KB / S, kb1 = (sp + 1) * KB / S;
        const int brow = t.g * p.N + t.nt * BN;
        if (p.a_ready != nullptr) {
          // rows of this tile were pushed by other ranks: wait (bounded) for their arrival flags
          const int last = min(t.m0 + BM, t.m_end) - 1;
          const int i_lo = p.a_ready_rows > 0 ? t.m0 / p.a_ready_rows : 0;            // rows == 0: wait for every rank
          const int i_hi = p.a_ready_rows > 0 ? last / p.a_ready_rows : p.world - 1;
          for (int i = i_lo; ok && i <= i_hi; ++i) {
            if (ready_mask & (1u << i)) continue;   // flags only grow: a rank seen once stays arrived
            if (wait_flag_ge(p.a_ready + i, epoch, p.status)) {
              ready_mask |= 1u << i;
            } else {
              if (*abort_flag == 0) *abort_flag = kTimeoutPeer;
              if (p.status != nullptr) atomicMax(p.status, (int)kTimeoutPeer);
              ok = false;
            }
          }
          if (!ok) break;
          fence_proxy_async_global();
        }
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (!mbar_wait(&ss.empty[s], ph ^ 1, abort_flag, kTimeoutProducer)) { ok = false; break; }
          mbar_expect_tx(&ss.full[s], (BM + BN) * BK_BYTES);
          tma_load_2d(sA_tiles + s * BM * BK_BYTES, &tmA, &ss.full[s], kb * BK, t.m0);
          tma_load_2d(sB_tiles + s * BN * BK_BYTES, &tmB, &ss.full[s], kb * BK, brow);
        }
      }
      // Drain: do not leave the CTA while bulk copies may still land in its shared memory.
      // Every armed stage is consumed by the MMA role, which releases it through `empty`; wait
      // (bounded) for the last kStages releases.
      if (ok) {
        const uint32_t n = it < (uint32_t)kStages ? it : (uint32_t)kStages;
        for (uint32_t j = it - n; j < it; ++j) {
          const int s = j % kStages;
          const uint32_t ph = (j / kStages) & 1;
          if (!mbar_wait(&ss.empty[s], ph, abort_flag, kTimeoutProducer)) break;
        }
      } else {
        for (int s = 0; s < kStages; ++s) {  // aborted: give in-flight copies a bounded time to land
          for (uint32_t i = 0; i < (1u << 14); ++i) {
            if (mbar_try_wait(&ss.full[s], 0) || mbar_try_wait(&ss.full[s], 1)) break;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc(BM, BN, KIND == KIND_FP8 ? 0 : 1, KIND == KIND_FP8 ? 0 : 1);
      TileWalker walk(offs, ss.cnt, p.groups, n_tiles, p.M, p.m_rotate);
      Tile t;
      uint32_t it = 0;   // smem stage counter
      uint32_t acc = 0;  // accumulator hand-off counter
      bool ok = true;
      for (int item = blockIdx.x; ok && walk.get(item / S, t); item += gridDim.x) {
        const int sp = item % S;
        const int kb0 = sp * KB / S, kb1 = (sp + 1) * KB / S;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          const bool new_acc = (KIND == KIND_FP8) || kb == kb0;
          const int buf = acc & 1;
          if (new_acc) {
            if (!mbar_wait(&ss.tmem_empty[buf], ((acc >> 1) & 1) ^ 1, abort_flag, kTimeoutMma)) { ok = false; break; }
          }
          if (!mbar_wait(&ss.full[s], ph, abort_flag, kTimeoutMma)) { ok = false; break; }
          tc_fence_after();
          const uint32_t d = tmem_base + buf * BN;
          const uint64_t adesc = make_smem_desc_sw128(smem_u32(sA_tiles + s * BM * BK_BYTES));
          const uint64_t bdesc = make_smem_desc_sw128(smem_u32(sB_tiles + s * BN * BK_BYTES));
#pragma unroll
          for (int k = 0; k < 4; ++k) {  // 4 x 32 bytes of K per stage
            const uint32_t accum = (k > 0 || !new_acc) ? 1u : 0u;
            if (KIND == KIND_FP8) mma_f8f6f4(d, adesc + 2 * k, bdesc + 2 * k, idesc, accum);
            else mma_f16(d, adesc + 2 * k, bdesc + 2 * k, idesc, accum);
          }
          tc_commit(&ss.empty[s]);
          const bool last_of_acc = (KIND == KIND_FP8) || kb == kb1 - 1;
          if (last_of_acc) {
            tc_commit(&ss.tmem_full[buf]);
            ++acc;
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue
    const int ew = warp - 2;
    const int quad = warp & 3;        // TMEM lane quadrant this warp may access
    const int half = ew >> 2;         // which 64 columns of the tile
    const int row_in_tile = quad * 32 + lane;
    TileWalker walk(offs, ss.cnt, p.groups, n_tiles, p.M, p.m_rotate);
    Tile t;
    uint32_t acc = 0;
    bool ok = true;
    for (int item = blockIdx.x; ok && walk.get(item / S, t); item += gridDim.x) {
      const int tile = item / S, sp = item % S;
      const int kb0 = sp * KB / S, kb1 = (sp + 1) * KB / S;
      const int groups_of_k = (KIND == KIND_FP8) ? (kb1 - kb0) : 1;
      float r[64];
#pragma unroll
      for (int j = 0; j < 64; ++j) r[j] = 0.f;
      const int row = t.m0 + row_in_tile;
      const bool row_ok = row < t.m_end;
      // scale pointers
      const float* sa_ptr = (KIND == KIND_FP8) ? p.sA + row : nullptr;
      int sb_blk_lo, sb_blk_hi;  // weight scale block for columns [0,32) and [32,64) of this half
      if (EPI == EPI_SILU_MUL) {
        const int I = p.N / 2;
        sb_blk_lo = (t.nt * 64) / 128;
        sb_blk_hi = (I + t.nt * 64) / 128;
      } else {
        sb_blk_lo = sb_blk_hi = t.nt;
      }
      const float* sb_lo = (KIND == KIND_FP8) ? p.sB + (size_t)(t.g * nblk + sb_blk_lo) * KB : nullptr;
      const float* sb_hi = (KIND == KIND_FP8) ? p.sB + (size_t)(t.g * nblk + sb_blk_hi) * KB : nullptr;
      // Activation scales pushed by other ranks (all-gather / dispatch fused into this GEMM) may only be
      // read once the producer has seen the arrival flags, i.e. after this tile's first accumulator
      // hand-off, and with coherent loads; local inputs are prefetched one K block ahead right away.
      const bool remote_a = (p.a_ready != nullptr);
      float sa_next = 1.f, sbl_next = 1.f, sbh_next = 1.f;
      if (KIND == KIND_FP8) {
        sa_ptr += (size_t)kb0 * p.sa_stride;         // this split's first K block
        sb_lo += kb0;
        sb_hi += kb0;
        if (!remote_a) sa_next = row_ok ? __ldg(sa_ptr) : 0.f;
        sbl_next = __ldg(sb_lo);
        sbh_next = __ldg(sb_hi);
      }
      for (int kg = 0; kg < groups_of_k; ++kg, ++acc) {
        float sa = sa_next;
        const float sbl = sbl_next, sbh = sbh_next;
        if (KIND == KIND_FP8 && kg + 1 < groups_of_k) {
          if (!remote_a) sa_next = row_ok ? __ldg(sa_ptr + (size_t)(kg + 1) * p.sa_stride) : 0.f;
          sbl_next = __ldg(sb_lo + kg + 1);
          sbh_next = __ldg(sb_hi + kg + 1);
        }
        const int buf = acc & 1;
        // warp-uniform outcome: the lanes of a warp leave the loop together
        if (!__all_sync(0xffffffffu, mbar_wait(&ss.tmem_full[buf], (acc >> 1) & 1, abort_flag, kTimeoutEpilogue))) {
          ok = false;
          break;
        }
        tc_fence_after();
        if (KIND == KIND_FP8 && remote_a) {
          const volatile float* sv = sa_ptr;
          if (kg == 0) sa = row_ok ? sv[0] : 0.f;
          if (kg + 1 < groups_of_k) sa_next = row_ok ? sv[(size_t)(kg + 1) * p.sa_stride] : 0.f;
        }
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + buf * BN + half * 64;
        uint32_t v0[32], v1[32];
        tmem_ld_32x32(taddr, v0);
        tmem_ld_32x32(taddr + 32, v1);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&ss.tmem_empty[buf]);
        const float s_lo = sa * sbl, s_hi = sa * sbh;
        const float2 s_lo2 = make_float2(s_lo, s_lo), s_hi2 = make_float2(s_hi, s_hi);
#pragma unroll
        for (int j = 0; j < 32; j += 2) {              // packed FMAs (fma.rn.f32x2): half the issue slots
          const float2 a = __ffma2_rn(make_float2(__uint_as_float(v0[j]), __uint_as_float(v0[j + 1])), s_lo2,
                                      make_float2(r[j], r[j + 1]));
          const float2 b = __ffma2_rn(make_float2(__uint_as_float(v1[j]), __uint_as_float(v1[j + 1])), s_hi2,
                                      make_float2(r[32 + j], r[33 + j]));
          r[j] = a.x;
          r[j + 1] = a.y;
          r[32 + j] = b.x;
          r[33 + j] = b.y;
        }
      }
      if (!ok) break;
      if (S > 1) {
        const int et = ew * 32 + lane;                              // 0 .. 255 over the epilogue warps
        constexpr int kEpiThreads = kEpiWarps * 32;
        float* mine = p.splitk_ws + ((size_t)tile * S + sp) * 64 * kEpiThreads + et;
#pragma unroll
        for (int j = 0; j < 64; ++j) __stcg(mine + j * kEpiThreads, r[j]);
        __threadfence();
        asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
        if (et == 0) {
          const int prev = atomicAdd(p.splitk_cnt + tile, 1);
          ss.split_last = (prev == S - 1) ? 1 : 0;
          if (prev == S - 1) p.splitk_cnt[tile] = 0;               // ready for the next launch / graph replay
        }
        asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
        if (ss.split_last == 0) continue;                          // another split finishes this tile
        __threadfence();
        const float* all = p.splitk_ws + (size_t)tile * S * 64 * kEpiThreads + et;
#pragma unroll
        for (int j = 0; j < 64; ++j) r[j] = 0.f;
        for (int q = 0; q < S; ++q) {
#pragma unroll
          for (int j = 0; j < 64; ++j) r[j] += __ldcg(all + ((size_t)q * 64 + j) * kEpiThreads);
        }
      }
      __nv_bfloat16* out_base = p.D;
      size_t out_row = (size_t)row;
      bool store_ok = row_ok;
      if (p.peer_out[0] != nullptr && row_ok) {
        int drank, drow;
        if (p.row_map != nullptr) {
          const int2 rm = p.row_map[row];
          drank = rm.x;
          drow = rm.y;
        } else {
          drank = row / p.rs_rows_per_rank;
          drow = p.my_rank * p.rs_rows_per_rank + row % p.rs_rows_per_rank;
        }
        store_ok = drank >= 0;
        if (store_ok) {
          out_base = reinterpret_cast<__nv_bfloat16*>(p.peer_out[drank]);
          out_row = (size_t)drow;
        }
      }
      if (store_ok) {
        if (EPI == EPI_SILU_MUL) {
          // columns [0,32) of this half = gate, [32,64) = up of output columns nt*64 + half*32 + j
          const int col0 = t.nt * 64 + half * 32;
          const int n_out = p.N / 2;
          __nv_bfloat16* dst = out_base + out_row * p.ldd + col0;
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            if (col0 + j + 8 <= n_out) {
              __align__(16) __nv_bfloat162 o[4];
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const float a = silu(r[j + 2 * q]) * r[32 + j + 2 * q];
                const float b = silu(r[j + 2 * q + 1]) * r[32 + j + 2 * q + 1];
                o[q] = __floats2bfloat162_rn(a, b);
              }
              *reinterpret_cast<uint4*>(dst + j) = *reinterpret_cast<const uint4*>(o);
            } else {
              for (int q = 0; q < 8; ++q)
                if (col0 + j + q < n_out) dst[j + q] = __float2bfloat16(silu(r[j + q]) * r[32 + j + q]);
            }
          }
        } else if (EPI == EPI_STORE_F32) {
          const int col0 = t.nt * BN + half * 64;
          float* dst = reinterpret_cast<float*>(p.D) + out_row * p.ldd + col0;
#pragma unroll
          for (int j = 0; j < 64; j += 4) {
            if (col0 + j + 4 <= p.N) {
              *reinterpret_cast<float4*>(dst + j) = make_float4(r[j], r[j + 1], r[j + 2], r[j + 3]);
            } else {
              for (int q = 0; q < 4; ++q)
                if (col0 + j + q < p.N) dst[j + q] = r[j + q];
            }
          }
        } else if (p.peer_out[0] == nullptr) {
          const int col0 = t.nt * BN + half * 64;
          __nv_bfloat16* dst = out_base + out_row * p.ldd + col0;
#pragma unroll
          for (int j = 0; j < 64; j += 8) {
            if (col0 + j + 8 <= p.N) {
              __align__(16) __nv_bfloat162 o[4];
#pragma unroll
              for (int q = 0; q < 4; ++q) o[q] = __floats2bfloat162_rn(r[j + 2 * q], r[j + 2 * q + 1]);
              *reinterpret_cast<uint4*>(dst + j) = *reinterpret_cast<const uint4*>(o);
            } else {
              for (int q = 0; q < 8; ++q)
                if (col0 + j + q < p.N) dst[j + q] = __float2bfloat16(r[j + q]);
            }
          }
        }
      }
      if (EPI == EPI_STORE && p.peer_out[0] != nullptr) {
        // Rows bound for peer memory leave as whole 128-byte runs: the warp's 32 x 64 block goes through
        // shared memory 16 rows at a time, then 8 lanes write one row's 128 bytes together (a row per
        // thread would cross NVLink as 16-byte fragments).  Chunks are XOR-swizzled against bank conflicts.
        const int col0 = t.nt * BN + half * 64;
        uint8_t* stg = epi_stage + ew * kEpiStageBytes;
        const unsigned long long my_dst =
            store_ok ? reinterpret_cast<unsigned long long>(out_base + out_row * p.ldd + col0) : 0ull;
#pragma unroll
        for (int pass = 0; pass < 2; ++pass) {
          if ((lane >> 4) == pass) {
            const int lr = lane & 15;
#pragma unroll
            for (int c = 0; c < 8; ++c) {
              __align__(16) __nv_bfloat162 o[4];
#pragma unroll
              for (int q = 0; q < 4; ++q) o[q] = __floats2bfloat162_rn(r[c * 8 + 2 * q], r[c * 8 + 2 * q + 1]);
              *reinterpret_cast<uint4*>(stg + lr * 128 + ((c ^ (lr & 7)) << 4)) = *reinterpret_cast<const uint4*>(o);
            }
          }
          __syncwarp();
#pragma unroll
          for (int it = 0; it < 4; ++it) {
            const int lr = it * 4 + (lane >> 3);
            const int c = lane & 7;
            const unsigned long long d = __shfl_sync(0xffffffffu, my_dst, pass * 16 + lr);
            const uint4 v = *reinterpret_cast<const uint4*>(stg + lr * 128 + ((c ^ (lr & 7)) << 4));
            if (d != 0ull && col0 + c * 8 + 8 <= p.N) *(reinterpret_cast<uint4*>(d) + c) = v;
          }
          __syncwarp();
        }
      }
    }
  }

  if (p.done_counter != nullptr) __threadfence_system();   // this thread's peer stores, before the CTA reports
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
  if (threadIdx.x == 0 && ss.abort_flag != 0 && p.status != nullptr) atomicMax(p.status, ss.abort_flag);
  if (threadIdx.x == 0 && p.done_counter != nullptr) {
    // every store of this CTA (ordered before the barrier above) becomes visible system-wide, then
    // the last CTA to get here tells every rank that this rank's outputs are complete
    __threadfence_system();
    const unsigned int prev = atomicAdd(p.done_counter, 1u);
    if (prev == gridDim.x - 1) {
      *p.done_counter = 0u;
      __threadfence_system();
      for (int r = 0; r < p.world; ++r) st_relaxed_sys(p.peer_flags[r] + p.done_flag_index + p.my_rank, epoch);
    }
  }
}

// ------------------------------------------------------------------ host side
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

// 2-D row-major [rows, cols] tensor of `elem_bytes` elements, box = [box_rows, 128 bytes], 128B swizzle.
static int make_map_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, int elem_bytes,
                       uint32_t box_rows) {
  EncodeTiledFn enc = get_encode();
  if (enc == nullptr) return -1;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * (uint64_t)elem_bytes};
  cuuint32_t box[2] = {(cuuint32_t)(128 / elem_bytes), box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapDataType dt = elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUresult r = enc(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -2;
}

static size_t gemm_smem_bytes() {
  return kStages * (BM + BN) * BK_BYTES + ((sizeof(SharedStorage) + 15) & ~size_t(15)) + kEpiWarps * kEpiStageBytes + 1024;
}

// Split-K scratch of the calling thread's current device, installed from the host side (bg_gemm_set_splitk_ws)
// before the first launch: allocating here would not be legal while a stream is being captured.
struct SplitKWorkspace {
  float* ws = nullptr;
  int* cnt = nullptr;
  size_t max_items = 0;     // (tile, split) partials that fit
  int max_tiles = 0;        // counters
};
static SplitKWorkspace g_splitk[kMaxDevices];
static SplitKWorkspace& splitk_workspace() {
  static SplitKWorkspace none;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return none;
  return g_splitk[dev];
}

template <int KIND, int EPI>
static int launch_gemm(const void* A, const void* B, const GemmParams& p, int a_rows, int b_rows, int num_sms,
                       cudaStream_t stream) {
  constexpr int eb = (KIND == KIND_FP8) ? 1 : 2;
  CUtensorMap tmA, tmB;
  if (make_map_2d(&tmA, A, a_rows, p.K, eb, BM) != 0) return -10;
  if (make_map_2d(&tmB, B, b_rows, p.K, eb, BN) != 0) return -11;
  static DeviceOnce attr_set;   // one per template instantiation, tracked per device
  auto kern = gemm_kernel<KIND, EPI>;
  const size_t smem = gemm_smem_bytes();
  if (!ensure_dynamic_smem(kern, smem, attr_set)) return -12;
  int grid = num_sms;
  GemmParams q = p;
  q.splits = 1;
  q.splitk_ws = nullptr;
  q.splitk_cnt = nullptr;
  if (p.offsets == nullptr) {
    const int tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN);
    const int KB = p.K / (BK_BYTES / eb);
    SplitKWorkspace& ws = splitk_workspace();
    // Pick the split count from a cost model in units of one K block of one tile: a work item costs its K blocks
    // plus a fixed part (pipeline fill, accumulator hand-off, epilogue: about 10), the tile's last split pays about
    // 3 per partial it reduces, and items run in waves over the SMs.  Measured anchors: o_proj at 384 rows (168
    // tiles, 128 K blocks) 145 -> 121 us with a split; the shared expert's down projection (168 tiles, 16 K
    // blocks) 25 -> 48 us when it was split, so short K stays whole.
    int S = 1;
    if (ws.ws != nullptr && tiles < 2 * num_sms && tiles <= ws.max_tiles) {
      auto cost = [&](int c) {
        const int waves = (tiles * c + num_sms - 1) / num_sms;
        return (float)waves * ((float)KB / (float)c + 10.0f) + (c > 1 ? 3.0f * (float)c : 0.0f);
      };
      float best = 0.9f * cost(1);                 // a split has to win by a margin
      for (int c = 2; c <= 16; ++c) {
        if (KB / c < 2 || (size_t)tiles * c > ws.max_items) break;
        const float v = cost(c);
        if (v < best) {
          best = v;
          S = c;
        }
      }
    }
    if (S > 1) {
      q.splits = S;
      q.splitk_ws = ws.ws;
      q.splitk_cnt = ws.cnt;
    }
    if (tiles * S < grid) grid = tiles * S;
  }
  if (grid < 1) grid = 1;
  bg::launch_pdl(kern, dim3(grid), dim3(kThreads), smem, stream, tmA, tmB, q);
  return cudaGetLastError() == cudaSuccess ? 0 : -13;
}

}  // namespace bg

extern "C" {

// Collective hooks of the next bg_gemm call on this thread (consumed by that call, then cleared).
struct BgGemmHooks {
  const uint32_t* a_ready; int a_ready_rows; uint32_t epoch; const uint32_t* epoch_base; int m_rotate;
  void* peer_out[8]; const int2* row_map; int rs_rows_per_rank; int my_rank; int world;
  uint32_t* peer_flags[8]; int done_flag_index; unsigned int* done_counter;
};
static thread_local BgGemmHooks g_hooks;
static thread_local bool g_hooks_set = false;
static thread_local const int* g_counts = nullptr;

void bg_gemm_set_hooks(const uint32_t* a_ready, int a_ready_rows, uint32_t epoch, const uint32_t* epoch_base, int m_rotate,
                       void* const* peer_out,
                       const void* row_map, int rs_rows_per_rank, int my_rank, int world, uint32_t* const* peer_flags,
                       int done_flag_index, unsigned int* done_counter) {
  g_hooks.a_ready = a_ready; g_hooks.a_ready_rows = a_ready_rows; g_hooks.epoch = epoch;
  g_hooks.epoch_base = epoch_base; g_hooks.m_rotate = m_rotate;
  for (int i = 0; i < 8; ++i) {
    g_hooks.peer_out[i] = (peer_out != nullptr && i < world) ? peer_out[i] : nullptr;
    g_hooks.peer_flags[i] = (peer_flags != nullptr && i < world) ? peer_flags[i] : nullptr;
  }
  g_hooks.row_map = reinterpret_cast<const int2*>(row_map); g_hooks.rs_rows_per_rank = rs_rows_per_rank;
  g_hooks.my_rank = my_rank; g_hooks.world = world; g_hooks.done_flag_index = done_flag_index;
  g_hooks.done_counter = done_counter;
  g_hooks_set = true;
}

// Scratch for split-K launches on the current device: `ws` holds `max_items` partial tiles of 128 x 128 fp32,
// `counters` holds `max_tiles` zeroed ints.  Null `ws` switches split K off.
int bg_gemm_set_splitk_ws(float* ws, long long max_items, int* counters, int max_tiles) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= bg::kMaxDevices) return -1;
  bg::g_splitk[dev].ws = ws;
  bg::g_splitk[dev].cnt = counters;
  bg::g_splitk[dev].max_items = ws != nullptr ? (size_t)max_items : 0;
  bg::g_splitk[dev].max_tiles = max_tiles;
  return 0;
}

// Real row counts of the next grouped bg_gemm on this thread: counts[g] rows of segment g are present, the
// rest of the (128-aligned) segment is padding that is neither computed as whole tiles nor stored.
void bg_gemm_set_counts(const int* counts) { g_counts = counts; }

// Dense or grouped GEMM.  kind: 0 = e4m3 block scaled, 1 = bf16.  epi: 0 = store, 1 = silu-mul
// (weight rows interleaved in 32-row gate/up blocks; output has N/2 columns).
// offsets == nullptr -> dense [M, K] x [N, K]^T.  Otherwise A holds `groups` row segments
// (128-aligned starts, offsets[groups] <= M) and B is [groups * N, K].
// K must be a multiple of 128 elements (fp8) / 64 (bf16).  Returns 0 on a successful launch.
int bg_gemm(int kind, int epi, const void* A, const float* sA, int sa_stride, const void* B, const float* sB,
            void* D, int ldd, const int* offsets, int groups, int M, int N, int K, int num_sms, int* status,
            cudaStream_t stream) {
  using namespace bg;
  if (M <= 0 || N <= 0) return 0;
  const int bk = kind == KIND_FP8 ? 128 : 64;
  if (K % bk != 0 || groups > kMaxGroups || (epi == EPI_SILU_MUL && (N % 256) != 0)) return -1;
  if (offsets == nullptr) groups = 1;
  GemmParams p;
  p.counts = (offsets != nullptr) ? g_counts : nullptr;
  g_counts = nullptr;
  p.sA = sA; p.sa_stride = sa_stride; p.sB = sB; p.D = reinterpret_cast<__nv_bfloat16*>(D); p.ldd = ldd;
  p.offsets = offsets; p.groups = groups; p.M = M; p.N = N; p.K = K; p.status = status;
  p.a_ready = nullptr; p.a_ready_rows = 1; p.epoch = 0; p.epoch_base = nullptr; p.m_rotate = 0; p.row_map = nullptr; p.rs_rows_per_rank = 1;
  p.my_rank = 0; p.world = 1; p.done_flag_index = 0; p.done_counter = nullptr;
  for (int i = 0; i < 8; ++i) { p.peer_out[i] = nullptr; p.peer_flags[i] = nullptr; }
  if (g_hooks_set) {
    p.a_ready = g_hooks.a_ready; p.a_ready_rows = g_hooks.a_ready_rows;
    p.epoch = g_hooks.epoch; p.epoch_base = g_hooks.epoch_base; p.m_rotate = g_hooks.m_rotate; p.row_map = g_hooks.row_map;
    p.rs_rows_per_rank = g_hooks.rs_rows_per_rank > 0 ? g_hooks.rs_rows_per_rank : 1;
    p.my_rank = g_hooks.my_rank; p.world = g_hooks.world; p.done_flag_index = g_hooks.done_flag_index;
    p.done_counter = g_hooks.done_counter;
    for (int i = 0; i < 8; ++i) { p.peer_out[i] = g_hooks.peer_out[i]; p.peer_flags[i] = g_hooks.peer_flags[i]; }
    g_hooks_set = false;
  }
  // rows bound for peer memory are written in 16-byte pieces: whole pieces and aligned rows only
  if (p.peer_out[0] != nullptr && (epi != EPI_STORE || (N % 8) != 0 || (ldd % 8) != 0)) return -1;
  if (epi == EPI_STORE_F32 && (kind != KIND_BF16 || (ldd % 4) != 0)) return -1;
  const int b_rows = groups * N;
  if (kind == KIND_FP8 && epi == EPI_STORE) return launch_gemm<KIND_FP8, EPI_STORE>(A, B, p, M, b_rows, num_sms, stream);
  if (kind == KIND_FP8 && epi == EPI_SILU_MUL) return launch_gemm<KIND_FP8, EPI_SILU_MUL>(A, B, p, M, b_rows, num_sms, stream);
  if (kind == KIND_BF16 && epi == EPI_STORE) return launch_gemm<KIND_BF16, EPI_STORE>(A, B, p, M, b_rows, num_sms, stream);
  if (kind == KIND_BF16 && epi == EPI_SILU_MUL) return launch_gemm<KIND_BF16, EPI_SILU_MUL>(A, B, p, M, b_rows, num_sms, stream);
  if (kind == KIND_BF16 && epi == EPI_STORE_F32) return launch_gemm<KIND_BF16, EPI_STORE_F32>(A, B, p, M, b_rows, num_sms, stream);
  return -2;
}

}  // extern "C"

BG_TRACE_SETTER(gemm_tcgen05)
