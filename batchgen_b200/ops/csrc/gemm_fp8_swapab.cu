// Block-scaled FP8 GEMM for few rows per weight matrix (decode-sized steps): weights on the tensor-core M side.
//
// A decode step gives every expert a dozen tokens.  With tokens on the MMA's M side (the other two FP8 kernels) a
// 128-row tile is nine tenths padding, and since every 128-deep K block needs its own accumulator (the 1x128 / 128x128
// scales change per K block) the epilogue drags 128 x 256 fp32 values out of TMEM per K block for a dozen useful rows.
// That hand-off, not HBM, set the pace: 0.57 - 0.73 of copy bandwidth measured while streaming expert weights.
//
// Here the roles of the operands are swapped (D^T = W . X^T):
//   * A = a 128-row tile of the weight matrix (MMA M = 128, on the TMEM lanes), B = a tile of 32 tokens (MMA N = 32);
//   * a K block's accumulator is 128 lanes x 32 columns, one tcgen05.ld per epilogue thread; eight of them fit in 256
//     TMEM columns, so the MMA runs up to eight K blocks ahead of the epilogue;
//   * eight 20 KB stages (16 KB of weights, 4 KB of tokens) keep 128 KB of weights in flight per SM;
//   * the weight scale of a K block is one number for the whole tile and the token scales are 32 numbers shared by all
//     threads: both are staged in shared memory once per tile instead of being loaded per row and K block;
//   * experts without tokens cost nothing, experts with more than 32 tokens take several token tiles that sit next to
//     each other in the schedule (their weights come from L2).
// Epilogues: plain store (bf16, transposed back to [token, feature]), SiLU(gate) * up on the tile-interleaved gate/up
// layout, and the row-return form that stores every token's row into its owner rank's buffer over NVLink and raises
// the arrival flags when the last CTA is done.  The A operand may have been pushed by peers (arrival flags waited for).
//
// Roles (192 threads, one CTA per SM, persistent): warp 0 TMA producer, warp 1 MMA issuer + TMEM owner, warps 2..5
// epilogue (one thread per weight row).  All waits are bounded.
//
// Replaces (by behaviour): the reference's swap-AB grouped kernels for decode (batchgen_kernels/src/moe/mxfp4/
// marlin_grouped_mxfp4_v3.cuh:163-198 idea applied to block-scaled FP8) and DeepGEMM's masked m-grouped FP8 GEMM
// (batchgen/models/glm/glm5/moe_deepgemm_masked.py).
#define BG_FILE_TAG 4      // kernel-trace ids of this file are (tag << 16) | line
#include "common.cuh"

namespace bg {
namespace swab {

constexpr int BW = 128;                  // weight rows per tile (MMA M)
constexpr int BT = 32;                   // tokens per tile (MMA N)
constexpr int BKB = 128;                 // bytes of K per stage
constexpr int kStages = 8;
constexpr int kAcc = 8;                  // TMEM accumulators of BT columns
constexpr int kTmemCols = 256;
constexpr int kThreads = 192;
constexpr int kMaxGroups = 1024;
constexpr int kMaxKB = 144;              // K <= 18432
constexpr int EPI_STORE = 0;
constexpr int EPI_SILU_MUL = 1;

struct Params {
  const float* sA;           // token scales, [KB, sa_stride] (scale(m, kb) at kb * sa_stride + m)
  int sa_stride;
  const float* sB;           // weight scales [groups, ceil(N / 128), KB]
  __nv_bfloat16* D;
  int ldd;
  const int* offsets;        // grouped: first token row of every group (null: one group of M rows)
  const int* counts;         // grouped: tokens really present in every group (null: the whole segment)
  int groups, M, N, K;
  int* status;
  const uint32_t* a_ready;   // tokens were pushed by peers: wait for every rank's flag >= epoch
  uint32_t epoch;
  const uint32_t* epoch_base;
  int world;
  void* peer_out[8];         // row return: token row r goes to peer_out[row_map[r].x] at row row_map[r].y
  const int2* row_map;
  uint32_t* peer_flags[8];
  int done_index, my_rank;
  uint32_t done_epoch;
  unsigned int* done_counter;
};

struct Shared {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t tmem_full[kAcc];
  uint64_t tmem_empty[kAcc];
  uint32_t tmem_base;
  int abort_flag;
  int flags_ok;
  int offs[kMaxGroups + 1];
  int cnt[kMaxGroups];
  float st[2][kMaxKB][BT];    // token scales of the current and of the next tile
  float sw[2][2][kMaxKB];     // weight scales of the two tiles (SiLU epilogue: [.][0] gate block, [.][1] up block)
  float xch[2][BT][32];       // SiLU epilogue: the up rows' results, handed to the gate rows' threads
};

struct Tile { int g, n0, m0, m_end; };

// Tiles in the order (group, weight tile, token tile): token tiles of one weight tile are neighbours.
struct Walker {
  const int* offs;
  const int* cnt;
  int groups, n_tiles, M, g, before;
  __device__ Walker(const int* o, const int* c, int gr, int nt, int m) : offs(o), cnt(c), groups(gr), n_tiles(nt), M(m), g(0), before(0) {}
  __device__ bool get(int tile, Tile& t) {
    while (g < groups) {
      const int rows = (offs != nullptr) ? cnt[g] : M;
      const int tt = (rows + BT - 1) / BT;
      const int here = tt * n_tiles;
      if (tile < before + here) {
        const int local = tile - before;
        const int base = (offs != nullptr) ? offs[g] : 0;
        t.g = g; t.n0 = (local / tt) * BW; t.m0 = base + (local % tt) * BT; t.m_end = base + rows;
        return true;
      }
      before += here;
      ++g;
    }
    return false;
  }
};

template <int EPI>
__global__ void __launch_bounds__(kThreads, 1)
gemm_fp8_swapab_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, Params p) {
  bg::pdl_prologue((BG_FILE_TAG << 16) | __LINE__);
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* w_tiles = smem;                                   // kStages x 16 KB
  uint8_t* x_tiles = smem + kStages * BW * BKB;              // kStages x 4 KB
  Shared& ss = *reinterpret_cast<Shared*>(x_tiles + kStages * BT * BKB);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t epoch = p.epoch + (p.epoch_base != nullptr ? *p.epoch_base : 0u);
  const int KB = p.K / BKB;
  const int n_tiles = (p.N + BW - 1) / BW;
  const int nblk = (p.N + 127) / 128;
  volatile int* abort_flag = &ss.abort_flag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&ss.full[s], 1); mbar_init(&ss.empty[s], 1); }
    for (int b = 0; b < kAcc; ++b) { mbar_init(&ss.tmem_full[b], 1); mbar_init(&ss.tmem_empty[b], 4); }
    ss.abort_flag = 0;
    ss.flags_ok = 1;
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
      tma_prefetch_desc(&tmW);
      tma_prefetch_desc(&tmX);
      Walker walk(offs, ss.cnt, p.groups, n_tiles, p.M);
      Tile t;
      uint32_t it = 0;
      bool ok = true, arrived = (p.a_ready == nullptr);
      for (int tile = blockIdx.x; ok && walk.get(tile, t); tile += gridDim.x) {
        if (!arrived) {      // tokens pushed by other ranks: wait (bounded) once for every rank's arrival flag
          for (int i = 0; ok && i < p.world; ++i) {
            if (!wait_flag_ge(p.a_ready + i, epoch, p.status)) {
              if (*abort_flag == 0) *abort_flag = kTimeoutPeer;
              if (p.status != nullptr) atomicMax(p.status, (int)kTimeoutPeer);
              ok = false;
            }
          }
          if (!ok) break;
          fence_proxy_async_global();
          arrived = true;
        }
        const int wrow = t.g * p.N + t.n0;
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const int s = it % kStages;
          if (!mbar_wait(&ss.empty[s], ((it / kStages) & 1) ^ 1, abort_flag, kTimeoutProducer)) { ok = false; break; }
          mbar_expect_tx(&ss.full[s], (BW + BT) * BKB);
          tma_load_2d(w_tiles + s * BW * BKB, &tmW, &ss.full[s], kb * BKB, wrow);
          tma_load_2d(x_tiles + s * BT * BKB, &tmX, &ss.full[s], kb * BKB, t.m0);
        }
      }
      if (ok) {
        const uint32_t n = it < (uint32_t)kStages ? it : (uint32_t)kStages;
        for (uint32_t j = it - n; j < it; ++j)
          if (!mbar_wait(&ss.empty[j % kStages], (j / kStages) & 1, abort_flag, kTimeoutProducer)) break;
      } else {
        for (uint32_t i = 0; i < (1u << 16); ++i) __nanosleep(20);   // bounded grace period for copies in flight
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer: one 128 x 32 accumulator per K block
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc(BW, BT, 0, 0);
      Walker walk(offs, ss.cnt, p.groups, n_tiles, p.M);
      Tile t;
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && walk.get(tile, t); tile += gridDim.x) {
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const int s = it % kStages;
          const int buf = it % kAcc;
          if (!mbar_wait(&ss.tmem_empty[buf], ((it / kAcc) & 1) ^ 1, abort_flag, kTimeoutMma) ||
              !mbar_wait(&ss.full[s], (it / kStages) & 1, abort_flag, kTimeoutMma)) { ok = false; break; }
          tc_fence_after();
          const uint32_t d = tmem_base + buf * BT;
          const uint64_t adesc = make_smem_desc_sw128(smem_u32(w_tiles + s * BW * BKB));
          const uint64_t bdesc = make_smem_desc_sw128(smem_u32(x_tiles + s * BT * BKB));
#pragma unroll
          for (int k = 0; k < 4; ++k) mma_f8f6f4(d, adesc + 2 * k, bdesc + 2 * k, idesc, k > 0 ? 1u : 0u);
          tc_commit(&ss.empty[s]);
          tc_commit(&ss.tmem_full[buf]);
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue: thread = one weight row of the tile
    const int quad = warp & 3;                      // TMEM lane quadrant this warp may access
    const int et = threadIdx.x - 64;                // 0 .. 127
    const int lrow = quad * 32 + lane;              // weight row inside the tile
    const bool remote_a = (p.a_ready != nullptr);
    if (remote_a) {
      // pushed token scales may only be read after the ranks' arrival flags; the producer waits for them too
      if (et == 0) {
        int okf = 1;
        for (int i = 0; i < p.world; ++i)
          if (!wait_flag_ge(p.a_ready + i, epoch, p.status)) okf = 0;
        ss.flags_ok = okf;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
    }
    Walker walk(offs, ss.cnt, p.groups, n_tiles, p.M);
    Tile t;
    uint32_t it = 0;
    bool ok = ss.flags_ok != 0;
    // Scales of a tile are copied into shared memory asynchronously (cp.async) while the previous tile is being folded:
    // the copy of tile i + 1 is issued at the start of tile i and waited for at the start of tile i + 1.  Token scales
    // pushed by peers are read with L1-bypassing loads instead (an L1 line may be stale).
    auto stage = [&](const Tile& tt, int b) {
      for (int i = et; i < KB * BT; i += 128) {
        const int kb = i / BT, j = i - kb * BT;
        const int m = tt.m0 + j;
        const bool in = m < tt.m_end;
        const float* src = p.sA + (size_t)kb * p.sa_stride + (in ? m : tt.m0);
        if (remote_a) {
          ss.st[b][kb][j] = in ? __ldcg(src) : 0.f;
        } else {
          asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(smem_u32(&ss.st[b][kb][j])), "l"(src),
                       "r"(in ? 4 : 0)
                       : "memory");
        }
      }
      int blk0, blk1;
      if (EPI == EPI_SILU_MUL) {
        blk0 = (tt.n0 / 2) / 128;
        blk1 = (p.N / 2 + tt.n0 / 2) / 128;
      } else {
        blk0 = blk1 = tt.n0 / 128;
      }
      const float* s0 = p.sB + (size_t)(tt.g * nblk + min(blk0, nblk - 1)) * KB;
      const float* s1 = p.sB + (size_t)(tt.g * nblk + min(blk1, nblk - 1)) * KB;
      for (int i = et; i < KB; i += 128) {
        asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(&ss.sw[b][0][i])), "l"(s0 + i) : "memory");
        asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(&ss.sw[b][1][i])), "l"(s1 + i) : "memory");
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    };
    int sbuf = 0;
    bool have = ok && walk.get(blockIdx.x, t);
    if (have) stage(t, 0);
    for (int tile = blockIdx.x; ok && have; tile += gridDim.x, sbuf ^= 1) {
      asm volatile("cp.async.wait_all;" ::: "memory");
      asm volatile("bar.sync 1, 128;" ::: "memory");          // this tile's scales are in place; the other buffer is free
      Tile tn;
      const bool have_next = walk.get(tile + gridDim.x, tn);
      if (have_next) stage(tn, sbuf ^ 1);
      const int which = (EPI == EPI_SILU_MUL) ? (quad & 1) : 0;      // odd quadrants hold the up rows
      float r[BT];
#pragma unroll
      for (int j = 0; j < BT; ++j) r[j] = 0.f;
      for (int kb = 0; kb < KB; ++kb, ++it) {
        const int buf = it % kAcc;
        if (!__all_sync(0xffffffffu, mbar_wait(&ss.tmem_full[buf], (it / kAcc) & 1, abort_flag, kTimeoutEpilogue))) {
          ok = false;
          break;
        }
        tc_fence_after();
        uint32_t v[BT];
        tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + buf * BT, v);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&ss.tmem_empty[buf]);         // the accumulator is in registers
        const float sw = ss.sw[sbuf][which][kb];
        const float4* stv = reinterpret_cast<const float4*>(&ss.st[sbuf][kb][0]);
#pragma unroll
        for (int q = 0; q < BT / 4; ++q) {
          const float4 s4 = stv[q];
          r[4 * q + 0] = fmaf(__uint_as_float(v[4 * q + 0]), s4.x * sw, r[4 * q + 0]);
          r[4 * q + 1] = fmaf(__uint_as_float(v[4 * q + 1]), s4.y * sw, r[4 * q + 1]);
          r[4 * q + 2] = fmaf(__uint_as_float(v[4 * q + 2]), s4.z * sw, r[4 * q + 2]);
          r[4 * q + 3] = fmaf(__uint_as_float(v[4 * q + 3]), s4.w * sw, r[4 * q + 3]);
        }
      }
      if (!ok) break;
      const int n_tok = min(BT, t.m_end - t.m0);
      if (EPI == EPI_SILU_MUL) {
        // rows [64b, 64b + 32) of the tile are gate rows of output columns n0/2 + 32b + [0, 32), rows [64b + 32, 64b + 64)
        // the up rows of the same columns: the up threads hand their results over, the gate threads finish
        const int b2 = quad >> 1;
        if (quad & 1) {
#pragma unroll
          for (int j = 0; j < BT; ++j) ss.xch[b2][j][lane] = r[j];
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (!(quad & 1)) {
          const int col = t.n0 / 2 + b2 * 32 + lane;
          if (col < p.N / 2) {
            __nv_bfloat16* dst = p.D + (size_t)t.m0 * p.ldd + col;
#pragma unroll
            for (int j = 0; j < BT; ++j)
              if (j < n_tok) dst[(size_t)j * p.ldd] = __float2bfloat16(silu(r[j]) * ss.xch[b2][j][lane]);
          }
        }
      } else {
        const int col = t.n0 + lrow;
        if (col < p.N) {
          if (p.row_map != nullptr) {
#pragma unroll
            for (int j = 0; j < BT; ++j) {
              if (j >= n_tok) continue;
              const int2 rm = p.row_map[t.m0 + j];
              if (rm.x < 0 || rm.x >= p.world) continue;
              reinterpret_cast<__nv_bfloat16*>(p.peer_out[rm.x])[(size_t)rm.y * p.ldd + col] = __float2bfloat16(r[j]);
            }
          } else {
            __nv_bfloat16* dst = p.D + (size_t)t.m0 * p.ldd + col;
#pragma unroll
            for (int j = 0; j < BT; ++j)
              if (j < n_tok) dst[(size_t)j * p.ldd] = __float2bfloat16(r[j]);
          }
        }
      }
      t = tn;
      have = have_next;
    }
    asm volatile("cp.async.wait_all;" ::: "memory");         // nothing of this thread is left in flight at exit
  }
  if (p.done_counter != nullptr) __threadfence_system();   // this thread's peer stores, before the CTA reports
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
  if (threadIdx.x == 0 && ss.abort_flag != 0 && p.status != nullptr) atomicMax(p.status, ss.abort_flag);
  if (threadIdx.x == 0 && p.done_counter != nullptr) {
    // the last CTA to get here tells every rank that this rank's rows have all been stored
    __threadfence_system();
    const unsigned int prev = atomicAdd(p.done_counter, 1u);
    if (prev == gridDim.x - 1) {
      *p.done_counter = 0u;
      __threadfence_system();
      const uint32_t e = p.done_epoch + (p.epoch_base != nullptr ? *p.epoch_base : 0u);
      for (int r = 0; r < p.world; ++r) st_relaxed_sys(p.peer_flags[r] + p.done_index + p.my_rank, e);
    }
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
static int make_map(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  EncodeTiledFn enc = get_encode();
  if (enc == nullptr) return -1;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols};
  cuuint32_t box[2] = {BKB, box_rows};
  cuuint32_t es[2] = {1, 1};
  return enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, es,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS ? 0 : -2;
}

template <int EPI>
static int launch(const void* X, const void* W, const Params& p, int w_rows, int num_sms, cudaStream_t stream) {
  CUtensorMap tw, tx;
  if (make_map(&tw, W, (uint64_t)w_rows, (uint64_t)p.K, BW) != 0) return -10;
  if (make_map(&tx, X, (uint64_t)p.M, (uint64_t)p.K, BT) != 0) return -11;
  static DeviceOnce attr_set;
  auto kern = gemm_fp8_swapab_kernel<EPI>;
  const size_t smem = kStages * (BW + BT) * BKB + sizeof(Shared) + 1024;
  if (!ensure_dynamic_smem(kern, smem, attr_set)) return -12;
  bg::launch_pdl(kern, dim3(num_sms), dim3(kThreads), smem, stream, tw, tx, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -13;
}

}  // namespace swab
}  // namespace bg

extern "C" {

static int gemm_fp8_swapab_impl(int epi, const void* X, const float* sA, int sa_stride, const void* W, const float* sB,
                                void* D, int ldd, const int* offsets, const int* counts, int groups, int M, int N, int K,
                                int num_sms, bg::swab::Params p, cudaStream_t stream) {
  using namespace bg::swab;
  if (M <= 0 || N <= 0) return 0;
  if (K % 128 != 0 || K / 128 > kMaxKB || N % 128 != 0 || groups > kMaxGroups || (epi == EPI_SILU_MUL && (N % 256) != 0))
    return -1;
  if (p.row_map != nullptr && epi != EPI_STORE) return -1;
  if (offsets == nullptr) groups = 1;
  p.sA = sA; p.sa_stride = sa_stride; p.sB = sB; p.D = reinterpret_cast<__nv_bfloat16*>(D); p.ldd = ldd;
  p.offsets = offsets; p.counts = offsets != nullptr ? counts : nullptr; p.groups = groups; p.M = M; p.N = N; p.K = K;
  if (epi == EPI_SILU_MUL) return launch<EPI_SILU_MUL>(X, W, p, groups * N, num_sms, stream);
  return launch<EPI_STORE>(X, W, p, groups * N, num_sms, stream);
}

static bg::swab::Params swab_plain(const uint32_t* a_ready, uint32_t epoch, const uint32_t* epoch_base, int world,
                                   int* status) {
  bg::swab::Params p;
  p.status = status; p.a_ready = a_ready; p.epoch = epoch; p.epoch_base = epoch_base; p.world = world;
  p.row_map = nullptr; p.done_counter = nullptr; p.done_index = 0; p.my_rank = 0; p.done_epoch = 0;
  for (int i = 0; i < 8; ++i) { p.peer_out[i] = nullptr; p.peer_flags[i] = nullptr; }
  return p;
}

// Same arguments as bg_gemm_fp8_n256: X [M, K] e4m3 tokens with scales sA (kb-major), W [groups * N, K] e4m3 weights
// with scales sB, D [M, N] bf16 (N / 2 columns with the SiLU epilogue).  Meant for few tokens per group.
int bg_gemm_fp8_swapab(int epi, const void* X, const float* sA, int sa_stride, const void* W, const float* sB, void* D,
                       int ldd, const int* offsets, const int* counts, int groups, int M, int N, int K, int num_sms,
                       const uint32_t* a_ready, uint32_t epoch, const uint32_t* epoch_base, int world, int* status,
                       cudaStream_t stream) {
  return gemm_fp8_swapab_impl(epi, X, sA, sa_stride, W, sB, D, ldd, offsets, counts, groups, M, N, K, num_sms,
                              swab_plain(a_ready, epoch, epoch_base, world, status), stream);
}

// Row-return form (see bg_gemm_fp8_n256_return).
int bg_gemm_fp8_swapab_return(const void* X, const float* sA, int sa_stride, const void* W, const float* sB, int ldd,
                              const int* offsets, const int* counts, int groups, int M, int N, int K, int num_sms,
                              void* const* peer_out, const void* row_map, uint32_t* const* peer_flags, int done_index,
                              uint32_t done_epoch, const uint32_t* epoch_base, unsigned int* done_counter, int my_rank,
                              int world, int* status, cudaStream_t stream) {
  if (world < 1 || world > 8 || peer_out == nullptr || row_map == nullptr || peer_flags == nullptr ||
      done_counter == nullptr || offsets == nullptr)
    return -1;
  bg::swab::Params p = swab_plain(nullptr, 0, epoch_base, world, status);
  for (int i = 0; i < world; ++i) { p.peer_out[i] = peer_out[i]; p.peer_flags[i] = peer_flags[i]; }
  p.row_map = reinterpret_cast<const int2*>(row_map);
  p.done_index = done_index; p.done_epoch = done_epoch; p.done_counter = done_counter; p.my_rank = my_rank;
  return gemm_fp8_swapab_impl(bg::swab::EPI_STORE, X, sA, sa_stride, W, sB, peer_out[my_rank], ldd, offsets, counts,
                              groups, M, N, K, num_sms, p, stream);
}

}  // extern "C"

BG_TRACE_SETTER(gemm_fp8_swapab)
