// Block-scaled FP8 GEMM with 128 x 256 output tiles (dense and ragged grouped), for the compute-bound shapes.
//
// Same contract and numerics as the 128 x 128 kernel in gemm_tcgen05.cu (1x128 activation scales, 128x128
// weight scales, each 128-wide K block multiplied into its own TMEM accumulator and folded into fp32
// registers with the block's scales), but a tile is twice as wide:
//   * operand bytes staged per FLOP drop by a quarter (16 KB of A + 32 KB of B per K block for twice the
//     math), which is what bounds the narrower kernel (L2 -> shared memory traffic);
//   * one tcgen05.mma covers N = 256, and the two 256-column accumulators fill TMEM exactly;
//   * sixteen epilogue warps (four per TMEM lane quadrant, 64 columns each) have twice the time per K block
//     to fold an accumulator, so the tensor pipe waits for them less.
// The collective hooks that store rows to peers stay on the narrower kernel (their staging does not fit
// beside four 48 KB stages); the arrival-flag wait on the A operand and the real-row counts are supported.
//
// Roles (576 threads, one CTA per SM, persistent): warp 0 TMA producer, warp 1 MMA issuer + TMEM owner,
// warps 2..17 epilogue.
#define BG_FILE_TAG 3      // kernel-trace ids of this file are (tag << 16) | line
#include "common.cuh"

namespace bg {
namespace g256 {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BKB = 128;                 // bytes of K per stage (one swizzle atom)
constexpr int kStages = 4;
constexpr int kEpiWarps = 16;
constexpr int kThreads = 64 + 32 * kEpiWarps;
constexpr int kTmemCols = 512;
constexpr int kMaxGroups = 1024;
constexpr int EPI_STORE = 0;
constexpr int EPI_SILU_MUL = 1;

struct Params {
  const float* sA;
  int sa_stride;
  const float* sB;       // [groups, ceil(N / 128), KB]
  __nv_bfloat16* D;
  int ldd;
  const int* offsets;
  const int* counts;
  int groups, M, N, K;
  int* status;
  const uint32_t* a_ready;   // rows of A were pushed by peers: wait for every rank's flag >= epoch
  uint32_t epoch;
  const uint32_t* epoch_base;
  int world;
  // row return (EPI_STORE only): row r of D is stored at row row_map[r].y of rank row_map[r].x's buffer instead
  // (x < 0: dropped).  Each thread writes its 128-byte run with 16-byte stores, which suits decode-sized steps
  // (a few MB per launch); the 128 x 128 kernel stages rows through shared memory for the large ones.  When the
  // last CTA is done, flag done_index + my_rank of every rank is set to done_epoch (+ *epoch_base).
  void* peer_out[8];
  const int2* row_map;
  uint32_t* peer_flags[8];
  int done_index, my_rank;
  uint32_t done_epoch;
  unsigned int* done_counter;
};

struct Shared {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  int offs[kMaxGroups + 1];
  int cnt[kMaxGroups];
};

struct Tile { int g, m0, m_end, nt; };

struct Walker {
  const int* offs;
  const int* cnt;
  int groups, n_tiles, M, g, before;
  __device__ Walker(const int* o, const int* c, int gr, int nt, int m) : offs(o), cnt(c), groups(gr), n_tiles(nt), M(m), g(0), before(0) {}
  __device__ bool get(int tile, Tile& t) {
    if (offs == nullptr) {
      const int m_tiles = (M + BM - 1) / BM;
      if (tile >= m_tiles * n_tiles) return false;
      t.g = 0; t.nt = tile / m_tiles; t.m0 = (tile % m_tiles) * BM; t.m_end = M;
      return true;
    }
    while (g < groups) {
      const int rows = cnt[g];
      const int m_tiles = (rows + BM - 1) / BM;
      const int here = m_tiles * n_tiles;
      if (tile < before + here) {
        const int local = tile - before;
        t.g = g; t.nt = local / m_tiles; t.m0 = offs[g] + (local % m_tiles) * BM; t.m_end = offs[g] + rows;
        return true;
      }
      before += here;
      ++g;
    }
    return false;
  }
};

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* v) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}

template <int EPI>
__global__ void __launch_bounds__(kThreads, 1)
gemm_fp8_n256_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, Params p) {
  bg::pdl_prologue((BG_FILE_TAG << 16) | __LINE__);
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* a_tiles = smem;
  uint8_t* b_tiles = smem + kStages * BM * BKB;
  Shared& ss = *reinterpret_cast<Shared*>(b_tiles + kStages * BN * BKB);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t epoch = p.epoch + (p.epoch_base != nullptr ? *p.epoch_base : 0u);
  const int KB = p.K / BKB;
  const int n_tiles = (p.N + BN - 1) / BN;
  const int nblk = (p.N + 127) / 128;
  volatile int* abort_flag = &ss.abort_flag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&ss.full[s], 1); mbar_init(&ss.empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&ss.tmem_full[b], 1); mbar_init(&ss.tmem_empty[b], kEpiWarps); }
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
      Walker walk(offs, ss.cnt, p.groups, n_tiles, p.M);
      Tile t;
      uint32_t it = 0;
      bool ok = true, arrived = (p.a_ready == nullptr);
      for (int tile = blockIdx.x; ok && walk.get(tile, t); tile += gridDim.x) {
        if (!arrived) {      // rows pushed by other ranks: wait (bounded) once for every rank's arrival flag
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
        const int brow = t.g * p.N + t.nt * BN;
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const int s = it % kStages;
          if (!mbar_wait(&ss.empty[s], ((it / kStages) & 1) ^ 1, abort_flag, kTimeoutProducer)) { ok = false; break; }
          mbar_expect_tx(&ss.full[s], (BM + BN) * BKB);
          tma_load_2d(a_tiles + s * BM * BKB, &tmA, &ss.full[s], kb * BKB, t.m0);
          tma_load_2d(b_tiles + s * BN * BKB, &tmB, &ss.full[s], kb * BKB, brow);
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
    // ------------------------------------------------------------ MMA issuer: one accumulator per K block
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc(BM, BN, 0, 0);
      Walker walk(offs, ss.cnt, p.groups, n_tiles, p.M);
      Tile t;
      uint32_t it = 0, acc = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && walk.get(tile, t); tile += gridDim.x) {
        for (int kb = 0; kb < KB; ++kb, ++it, ++acc) {
          const int s = it % kStages;
          const int buf = acc & 1;
          if (!mbar_wait(&ss.tmem_empty[buf], ((acc >> 1) & 1) ^ 1, abort_flag, kTimeoutMma) ||
              !mbar_wait(&ss.full[s], (it / kStages) & 1, abort_flag, kTimeoutMma)) { ok = false; break; }
          tc_fence_after();
          const uint32_t d = tmem_base + buf * BN;
          const uint64_t adesc = make_smem_desc_sw128(smem_u32(a_tiles + s * BM * BKB));
          const uint64_t bdesc = make_smem_desc_sw128(smem_u32(b_tiles + s * BN * BKB));
#pragma unroll
          for (int k = 0; k < 4; ++k) mma_f8f6f4(d, adesc + 2 * k, bdesc + 2 * k, idesc, k > 0 ? 1u : 0u);
          tc_commit(&ss.empty[s]);
          tc_commit(&ss.tmem_full[buf]);
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue: warp = (lane quadrant, 64-column slice)
    const int quad = warp & 3;
    const int slice = (warp - 2) >> 2;            // 0..3
    const int row_in_tile = quad * 32 + lane;
    Walker walk(offs, ss.cnt, p.groups, n_tiles, p.M);
    Tile t;
    uint32_t acc = 0;
    bool ok = true;
    const bool remote_a = (p.a_ready != nullptr);
    for (int tile = blockIdx.x; ok && walk.get(tile, t); tile += gridDim.x) {
      float2 r2[32];                                // 64 fp32 accumulators as pairs: promotion uses packed FMAs
#pragma unroll
      for (int j = 0; j < 32; ++j) r2[j] = make_float2(0.f, 0.f);
      const int row = t.m0 + row_in_tile;
      const bool row_ok = row < t.m_end;
      const float* sa_ptr = p.sA + row;
      const int gslice = t.nt * 4 + slice;          // 64-column slice index along N
      int blk_lo, blk_hi;                           // weight scale block of columns [0,32) and [32,64) of the slice
      if (EPI == EPI_SILU_MUL) {
        blk_lo = (gslice * 32) / 128;
        blk_hi = (p.N / 2 + gslice * 32) / 128;
      } else {
        blk_lo = blk_hi = (gslice * 64) / 128;
      }
      blk_lo = min(blk_lo, nblk - 1);
      blk_hi = min(blk_hi, nblk - 1);
      const float* sb_lo = p.sB + (size_t)(t.g * nblk + blk_lo) * KB;
      const float* sb_hi = p.sB + (size_t)(t.g * nblk + blk_hi) * KB;
      float sa_next = 1.f, sbl_next = __ldg(sb_lo), sbh_next = __ldg(sb_hi);
      if (!remote_a) sa_next = row_ok ? __ldg(sa_ptr) : 0.f;
      for (int kg = 0; kg < KB; ++kg, ++acc) {
        float sa = sa_next;
        const float sbl = sbl_next, sbh = sbh_next;
        if (kg + 1 < KB) {
          if (!remote_a) sa_next = row_ok ? __ldg(sa_ptr + (size_t)(kg + 1) * p.sa_stride) : 0.f;
          sbl_next = __ldg(sb_lo + kg + 1);
          sbh_next = __ldg(sb_hi + kg + 1);
        }
        const int buf = acc & 1;
        if (!__all_sync(0xffffffffu, mbar_wait(&ss.tmem_full[buf], (acc >> 1) & 1, abort_flag, kTimeoutEpilogue))) {
          ok = false;
          break;
        }
        tc_fence_after();
        if (remote_a) {       // pushed scales are only valid once the producer has seen the arrival flags
          const volatile float* sv = sa_ptr;
          if (kg == 0) sa = row_ok ? sv[0] : 0.f;
          if (kg + 1 < KB) sa_next = row_ok ? sv[(size_t)(kg + 1) * p.sa_stride] : 0.f;
        }
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + buf * BN + slice * 64;
        const float s_lo = sa * sbl, s_hi = sa * sbh;
        const float2 s_lo2 = make_float2(s_lo, s_lo), s_hi2 = make_float2(s_hi, s_hi);
        // two 16-column chunks in flight: chunk c + 1 is read from TMEM while chunk c is promoted, and the promotion
        // is 8 packed FMAs (fma.rn.f32x2) per chunk instead of 16 scalar ones
        uint32_t v[2][16];
        tmem_ld16(taddr, v[0]);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          tmem_ld_wait();
          if (c + 1 < 4) tmem_ld16(taddr + (c + 1) * 16, v[(c + 1) & 1]);
          const float2 sc = c < 2 ? s_lo2 : s_hi2;
#pragma unroll
          for (int j = 0; j < 8; ++j)
            r2[c * 8 + j] = __ffma2_rn(make_float2(__uint_as_float(v[c & 1][2 * j]), __uint_as_float(v[c & 1][2 * j + 1])),
                                       sc, r2[c * 8 + j]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&ss.tmem_empty[buf]);
      }
      if (!ok) break;
      if (row_ok) {
        if (EPI == EPI_SILU_MUL) {
          const int col0 = gslice * 32;
          const int n_out = p.N / 2;
          __nv_bfloat16* dst = p.D + (size_t)row * p.ldd + col0;
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            if (col0 + j + 8 <= n_out) {
              __align__(16) __nv_bfloat162 o[4];
#pragma unroll
              for (int q = 0; q < 4; ++q)
                o[q] = __floats2bfloat162_rn(silu(r2[j / 2 + q].x) * r2[16 + j / 2 + q].x,
                                             silu(r2[j / 2 + q].y) * r2[16 + j / 2 + q].y);
              *reinterpret_cast<uint4*>(dst + j) = *reinterpret_cast<const uint4*>(o);
            }
          }
        } else {
          const int col0 = gslice * 64;
          __nv_bfloat16* dst = p.D + (size_t)row * p.ldd + col0;
          if (p.row_map != nullptr) {
            const int2 rm = p.row_map[row];
            if (rm.x < 0 || rm.x >= p.world) continue;
            dst = reinterpret_cast<__nv_bfloat16*>(p.peer_out[rm.x]) + (size_t)rm.y * p.ldd + col0;
          }
#pragma unroll
          for (int j = 0; j < 64; j += 8) {
            if (col0 + j + 8 <= p.N) {
              __align__(16) __nv_bfloat162 o[4];
#pragma unroll
              for (int q = 0; q < 4; ++q) o[q] = __floats2bfloat162_rn(r2[j / 2 + q].x, r2[j / 2 + q].y);
              *reinterpret_cast<uint4*>(dst + j) = *reinterpret_cast<const uint4*>(o);
            } else {
              for (int q = 0; q < 8; ++q)
                if (col0 + j + q < p.N) dst[j + q] = __float2bfloat16((q & 1) ? r2[(j + q) / 2].y : r2[(j + q) / 2].x);
            }
          }
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
static int launch(const void* A, const void* B, const Params& p, int b_rows, int num_sms, cudaStream_t stream) {
  CUtensorMap ta, tb;
  if (make_map(&ta, A, (uint64_t)p.M, (uint64_t)p.K, BM) != 0) return -10;
  if (make_map(&tb, B, (uint64_t)b_rows, (uint64_t)p.K, BN) != 0) return -11;
  static DeviceOnce attr_set;   // one per template instantiation, tracked per device
  auto kern = gemm_fp8_n256_kernel<EPI>;
  const size_t smem = kStages * (BM + BN) * BKB + sizeof(Shared) + 1024;
  if (!ensure_dynamic_smem(kern, smem, attr_set)) return -12;
  const int n_tiles = (p.N + BN - 1) / BN;
  const long long m_tiles = p.offsets != nullptr ? (long long)p.M / BM + p.groups : (p.M + BM - 1) / BM;
  long long grid = m_tiles * n_tiles;
  if (grid > num_sms) grid = num_sms;
  if (grid < 1) grid = 1;
  bg::launch_pdl(kern, dim3((int)grid), dim3(kThreads), smem, stream, ta, tb, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -13;
}

}  // namespace g256
}  // namespace bg

extern "C" {

// Same arguments as bg_gemm for kind 0 (e4m3 block scaled); a_ready / epoch / epoch_base / world describe an A
// operand pushed by peers (null: local), counts the real rows of each grouped segment (null: padded).
static int gemm_fp8_n256_impl(int epi, const void* A, const float* sA, int sa_stride, const void* B, const float* sB,
                              void* D, int ldd, const int* offsets, const int* counts, int groups, int M, int N, int K,
                              int num_sms, bg::g256::Params p, cudaStream_t stream) {
  using namespace bg::g256;
  if (M <= 0 || N <= 0) return 0;
  if (K % 128 != 0 || groups > kMaxGroups || (epi == EPI_SILU_MUL && (N % 256) != 0) || (ldd % 8) != 0) return -1;
  if (p.row_map != nullptr && (epi != EPI_STORE || (N % 8) != 0)) return -1;
  if (offsets == nullptr) groups = 1;
  p.sA = sA; p.sa_stride = sa_stride; p.sB = sB; p.D = reinterpret_cast<__nv_bfloat16*>(D); p.ldd = ldd;
  p.offsets = offsets; p.counts = offsets != nullptr ? counts : nullptr; p.groups = groups; p.M = M; p.N = N; p.K = K;
  if (epi == EPI_SILU_MUL) return launch<EPI_SILU_MUL>(A, B, p, groups * N, num_sms, stream);
  return launch<EPI_STORE>(A, B, p, groups * N, num_sms, stream);
}

static bg::g256::Params plain_params(const uint32_t* a_ready, uint32_t epoch, const uint32_t* epoch_base, int world,
                                     int* status) {
  bg::g256::Params p;
  p.status = status; p.a_ready = a_ready; p.epoch = epoch; p.epoch_base = epoch_base; p.world = world;
  p.row_map = nullptr; p.done_counter = nullptr; p.done_index = 0; p.my_rank = 0; p.done_epoch = 0;
  for (int i = 0; i < 8; ++i) { p.peer_out[i] = nullptr; p.peer_flags[i] = nullptr; }
  return p;
}

int bg_gemm_fp8_n256(int epi, const void* A, const float* sA, int sa_stride, const void* B, const float* sB, void* D,
                     int ldd, const int* offsets, const int* counts, int groups, int M, int N, int K, int num_sms,
                     const uint32_t* a_ready, uint32_t epoch, const uint32_t* epoch_base, int world, int* status,
                     cudaStream_t stream) {
  return gemm_fp8_n256_impl(epi, A, sA, sa_stride, B, sB, D, ldd, offsets, counts, groups, M, N, K, num_sms,
                            plain_params(a_ready, epoch, epoch_base, world, status), stream);
}

// Grouped GEMM whose output rows return to other ranks: row r goes to peer_out[row_map[r].x] at row row_map[r].y
// (row stride ldd elements); afterwards every rank's flag done_index + my_rank is raised to done_epoch.
int bg_gemm_fp8_n256_return(const void* A, const float* sA, int sa_stride, const void* B, const float* sB, int ldd,
                            const int* offsets, const int* counts, int groups, int M, int N, int K, int num_sms,
                            void* const* peer_out, const void* row_map, uint32_t* const* peer_flags, int done_index,
                            uint32_t done_epoch, const uint32_t* epoch_base, unsigned int* done_counter, int my_rank,
                            int world, int* status, cudaStream_t stream) {
  if (world < 1 || world > 8 || peer_out == nullptr || row_map == nullptr || peer_flags == nullptr ||
      done_counter == nullptr || offsets == nullptr)
    return -1;
  bg::g256::Params p = plain_params(nullptr, 0, epoch_base, world, status);
  for (int i = 0; i < world; ++i) { p.peer_out[i] = peer_out[i]; p.peer_flags[i] = peer_flags[i]; }
  p.row_map = reinterpret_cast<const int2*>(row_map);
  p.done_index = done_index; p.done_epoch = done_epoch; p.done_counter = done_counter; p.my_rank = my_rank;
  return gemm_fp8_n256_impl(bg::g256::EPI_STORE, A, sA, sa_stride, B, sB, peer_out[my_rank], ldd, offsets, counts, groups,
                            M, N, K, num_sms, p, stream);
}

}  // extern "C"

BG_TRACE_SETTER(gemm_fp8_n256)
