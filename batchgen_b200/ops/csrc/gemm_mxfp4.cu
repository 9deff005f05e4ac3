// MXFP4-weight GEMM (W4A16): bf16 activations x e2m1 weights with one e8m0 scale per 32 weights,
// dense and ragged grouped (per-expert), on tcgen05 tensor cores.
//
//   D[m, n] = sum_k A[m, k] * ( e2m1(Wq[n, k]) * 2^(Ws[n, k / 32] - 127) )
//
// The packed weights stay 4-bit all the way from HBM into shared memory (decode is bound by weight
// bytes).  Inside the CTA four warps expand each 128 x 64 weight tile to bf16 directly into the
// 128B-swizzled K-major layout that tcgen05.mma reads, so the tensor core runs a plain bf16 MMA with
// fp32 accumulation in TMEM; the scale is a power of two, hence the expansion is exact.
//
// Roles (320 threads, one CTA per SM, persistent over tiles):
//   warp 0      TMA producer: A tile (bf16, swizzled) + packed weight tile (64 B rows, no swizzle)
//   warp 1      TMEM allocator + tcgen05.mma issuer
//   warps 2..5  weight expansion (thread = weight row of the tile), scales prefetched one stage ahead
//   warps 6..9  epilogue (thread = TMEM lane), optional SiLU(gate) * up on interleaved rows
//
// Replaces (by behaviour): the Marlin-tile MXFP4 grouped kernels
// batchgen_kernels/src/moe/mxfp4/marlin_grouped_gemm.cu (v1/v2/v3), the LUT-dequant WGMMA kernels of
// GPT-OSS, and the load-time dequantisers batchgen_kernels/src/moe/mxfp4/mxfp4_dequant*.cu; weight
// layout per batchgen/models/moonshotai/kimi_linear/k3/mxfp4_layout.py:37-38,179-182 (e2m1 pairs,
// low nibble first, e8m0 per 32).
#include <cuda_fp4.h>

#include "common.cuh"

namespace bg {
namespace mx {

constexpr int BM = 128;
constexpr int BN = 128;
constexpr int BK = 64;                    // bf16 elements of K per stage (one 128-byte swizzle atom)
constexpr int kStages = 5;
constexpr int kThreads = 320;
constexpr int kTmemCols = 256;
constexpr int kMaxGroups = 1024;
constexpr int kABytes = BM * BK * 2;      // 16 KB
constexpr int kWBytes = BN * BK * 2;      // 16 KB expanded
constexpr int kQBytes = BN * BK / 2;      // 4 KB packed
constexpr int kStageBytes = kABytes + kWBytes + kQBytes;
constexpr int EPI_STORE = 0;
constexpr int EPI_SILU_MUL = 1;
constexpr int QMODE_MXFP4 = 0;            // e2m1 values, one e8m0 scale per 32
constexpr int QMODE_INT4 = 1;             // offset-binary int4 (value = q - 8), one bf16 scale per 32

struct Params {
  const uint8_t* ws;     // [groups * N, K / 32] e8m0
  __nv_bfloat16* D;      // [M, ldd]
  int ldd;
  const int* offsets;    // [groups + 1], 128-aligned segment starts; null = dense
  int groups, M, N, K;
  int* status;
};

struct Shared {
  uint64_t full[kStages];      // TMA: A + packed weights landed
  uint64_t expanded[kStages];  // 128 arrivals: bf16 weight tile written
  uint64_t empty[kStages];     // MMA done with the stage
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  int offs[kMaxGroups + 1];
};

struct Tile { int g, m0, m_end, nt; };

struct Walker {
  const int* offs;
  int groups, n_tiles, M, g, before;
  __device__ Walker(const int* o, int gr, int nt, int m) : offs(o), groups(gr), n_tiles(nt), M(m), g(0), before(0) {}
  __device__ bool get(int tile, Tile& t) {
    if (offs == nullptr) {
      const int m_tiles = (M + BM - 1) / BM;
      if (tile >= m_tiles * n_tiles) return false;
      t.g = 0; t.nt = tile / m_tiles; t.m0 = (tile % m_tiles) * BM; t.m_end = M;
      return true;
    }
    while (g < groups) {
      const int rows = offs[g + 1] - offs[g];
      const int here = ((rows + BM - 1) / BM) * n_tiles;
      if (tile < before + here) {
        const int local = tile - before, m_tiles = (rows + BM - 1) / BM;
        t.g = g; t.nt = local / m_tiles; t.m0 = offs[g] + (local % m_tiles) * BM; t.m_end = offs[g + 1];
        return true;
      }
      before += here;
      ++g;
    }
    return false;
  }
};

__device__ __forceinline__ float e8m0_to_float(uint32_t e) {
  // 2^(e - 127); e = 0 is 2^-127 (a subnormal float), e = 255 is NaN in the format and never stored
  return e == 0u ? __uint_as_float(0x00400000u) : __uint_as_float(e << 23);
}

template <int EPI, int QMODE>
__global__ void __launch_bounds__(kThreads, 1)
mxfp4_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmQ, Params p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* a_tiles = smem;
  uint8_t* w_tiles = smem + kStages * kABytes;
  uint8_t* q_tiles = w_tiles + kStages * kWBytes;
  Shared& ss = *reinterpret_cast<Shared*>(q_tiles + kStages * kQBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int KB = p.K / BK;
  const int n_tiles = (p.N + BN - 1) / BN;
  volatile int* abort_flag = &ss.abort_flag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&ss.full[s], 1);
      mbar_init(&ss.expanded[s], 128);
      mbar_init(&ss.empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&ss.tmem_full[b], 1);
      mbar_init(&ss.tmem_empty[b], 4);
    }
    ss.abort_flag = 0;
    mbar_fence_init();
  }
  if (p.offsets != nullptr)
    for (int i = threadIdx.x; i <= p.groups; i += kThreads) ss.offs[i] = p.offsets[i];
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
      Walker walk(offs, p.groups, n_tiles, p.M);
      Tile t;
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && walk.get(tile, t); tile += gridDim.x) {
        const int brow = t.g * p.N + t.nt * BN;
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const int s = it % kStages;
          if (!mbar_wait(&ss.empty[s], ((it / kStages) & 1) ^ 1, abort_flag, kTimeoutProducer)) { ok = false; break; }
          mbar_expect_tx(&ss.full[s], kABytes + kQBytes);
          tma_load_2d(a_tiles + s * kABytes, &tmA, &ss.full[s], kb * BK, t.m0);
          tma_load_2d(q_tiles + s * kQBytes, &tmQ, &ss.full[s], kb * (BK / 2), brow);
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
    // ------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc(BM, BN, 1, 1);   // bf16 x bf16 -> fp32
      Walker walk(offs, p.groups, n_tiles, p.M);
      Tile t;
      uint32_t it = 0, acc = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && walk.get(tile, t); tile += gridDim.x, ++acc) {
        const int buf = acc & 1;
        if (!mbar_wait(&ss.tmem_empty[buf], ((acc >> 1) & 1) ^ 1, abort_flag, kTimeoutMma)) { ok = false; break; }
        tc_fence_after();
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (!mbar_wait(&ss.full[s], ph, abort_flag, kTimeoutMma) ||
              !mbar_wait(&ss.expanded[s], ph, abort_flag, kTimeoutMma)) { ok = false; break; }
          tc_fence_after();
          const uint64_t adesc = make_smem_desc_sw128(smem_u32(a_tiles + s * kABytes));
          const uint64_t bdesc = make_smem_desc_sw128(smem_u32(w_tiles + s * kWBytes));
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            mma_f16(tmem_base + buf * BN, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) ? 1u : 0u);
          tc_commit(&ss.empty[s]);
        }
        if (ok) tc_commit(&ss.tmem_full[buf]);
      }
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------ weight expansion: e2m1 -> bf16, swizzled
    const int r = threadIdx.x - 64;          // weight row within the tile
    Walker walk(offs, p.groups, n_tiles, p.M);
    Tile t;
    uint32_t it = 0;
    bool ok = true;
    constexpr int kScaleBytes = QMODE == QMODE_INT4 ? 2 : 1;     // bf16 group scale or e8m0 block scale
    const int sk = (p.K / 32) * kScaleBytes;                     // scale bytes per weight row
    for (int tile = blockIdx.x; ok && walk.get(tile, t); tile += gridDim.x) {
      const int nrow = t.nt * BN + r;
      const bool row_ok = nrow < p.N;
      const uint8_t* srow = p.ws + (size_t)(t.g * p.N + (row_ok ? nrow : 0)) * sk;
      // the two scales of a 64-wide K stage: 2 bytes (e8m0) or 4 bytes (bf16)
      auto load_scales = [&](int kb) -> uint32_t {
        return QMODE == QMODE_INT4 ? *reinterpret_cast<const uint32_t*>(srow + 4 * kb)
                                   : static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(srow + 2 * kb));
      };
      uint32_t sc_next = load_scales(0);
      for (int kb = 0; kb < KB; ++kb, ++it) {
        const uint32_t sc = sc_next;
        if (kb + 1 < KB) sc_next = load_scales(kb + 1);
        const int s = it % kStages;
        if (!mbar_wait(&ss.full[s], (it / kStages) & 1, abort_flag, kTimeoutEpilogue)) { ok = false; break; }
        const uint4* q = reinterpret_cast<const uint4*>(q_tiles + s * kQBytes + r * (BK / 2));
        uint8_t* wrow = w_tiles + s * kWBytes + (r >> 3) * 1024 + (r & 7) * 128;
#pragma unroll
        for (int h = 0; h < 2; ++h) {        // 32 weights per scale
          const uint4 v = q[h];
          float f;
          if (QMODE == QMODE_INT4) f = row_ok ? __uint_as_float(((sc >> (16 * h)) & 0xFFFFu) << 16) : 0.f;   // bf16 -> fp32
          else f = row_ok ? e8m0_to_float((sc >> (8 * h)) & 0xFFu) : 0.f;
          const uint32_t words[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
          for (int c = 0; c < 4; ++c) {      // 8 weights -> one 16-byte chunk
            __align__(16) __nv_bfloat162 o[4];
#pragma unroll
            for (int b = 0; b < 4; ++b) {
              const uint32_t byte = (words[c] >> (8 * b)) & 0xFFu;
              if (QMODE == QMODE_INT4) {     // offset-binary nibbles: value = q - 8
                o[b] = __floats2bfloat162_rn((static_cast<float>(byte & 0xFu) - 8.f) * f,
                                             (static_cast<float>(byte >> 4) - 8.f) * f);
              } else {
                const __half2_raw hr = __nv_cvt_fp4x2_to_halfraw2(static_cast<__nv_fp4x2_storage_t>(byte), __NV_E2M1);
                const float2 ff = __half22float2(*reinterpret_cast<const __half2*>(&hr));
                o[b] = __floats2bfloat162_rn(ff.x * f, ff.y * f);
              }
            }
            const int chunk = h * 4 + c;
            *reinterpret_cast<uint4*>(wrow + ((chunk ^ (r & 7)) << 4)) = *reinterpret_cast<const uint4*>(o);
          }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        mbar_arrive(&ss.expanded[s]);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue
    const int quad = warp & 3;
    const int row_in_tile = quad * 32 + lane;
    Walker walk(offs, p.groups, n_tiles, p.M);
    Tile t;
    uint32_t acc = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && walk.get(tile, t); tile += gridDim.x, ++acc) {
      const int buf = acc & 1;
      if (!__all_sync(0xffffffffu, mbar_wait(&ss.tmem_full[buf], (acc >> 1) & 1, abort_flag, kTimeoutEpilogue))) { ok = false; break; }
      tc_fence_after();
      const int row = t.m0 + row_in_tile;
      const bool row_ok = row < t.m_end;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + buf * BN;
#pragma unroll 1
      for (int h = 0; h < 2; ++h) {          // 64 accumulator columns at a time
        __syncwarp();
        uint32_t v0[32], v1[32];
        tmem_ld_32x32(taddr + h * 64, v0);
        tmem_ld_32x32(taddr + h * 64 + 32, v1);
        tmem_ld_wait();
        if (!row_ok) continue;
        if (EPI == EPI_SILU_MUL) {
          const int n_out = p.N / 2;
          const int col0 = t.nt * 64 + h * 32;
          __nv_bfloat16* dst = p.D + (size_t)row * p.ldd + col0;
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            if (col0 + j + 8 <= n_out) {
              __align__(16) __nv_bfloat162 o[4];
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const float g0 = __uint_as_float(v0[j + 2 * q]), g1 = __uint_as_float(v0[j + 2 * q + 1]);
                o[q] = __floats2bfloat162_rn(silu(g0) * __uint_as_float(v1[j + 2 * q]),
                                             silu(g1) * __uint_as_float(v1[j + 2 * q + 1]));
              }
              *reinterpret_cast<uint4*>(dst + j) = *reinterpret_cast<const uint4*>(o);
            }
          }
        } else {
          const int col0 = t.nt * BN + h * 64;
          __nv_bfloat16* dst = p.D + (size_t)row * p.ldd + col0;
#pragma unroll
          for (int j = 0; j < 64; j += 8) {
            const uint32_t* src = j < 32 ? v0 + j : v1 + (j - 32);
            if (col0 + j + 8 <= p.N) {
              __align__(16) __nv_bfloat162 o[4];
#pragma unroll
              for (int q = 0; q < 4; ++q)
                o[q] = __floats2bfloat162_rn(__uint_as_float(src[2 * q]), __uint_as_float(src[2 * q + 1]));
              *reinterpret_cast<uint4*>(dst + j) = *reinterpret_cast<const uint4*>(o);
            } else {
              for (int q = 0; q < 8; ++q)
                if (col0 + j + q < p.N) dst[j + q] = __float2bfloat16(__uint_as_float(src[q]));
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ss.tmem_empty[buf]);
    }
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
  if (threadIdx.x == 0 && ss.abort_flag != 0 && p.status != nullptr) atomicMax(p.status, ss.abort_flag);
}

// Load-time / debugging expansion of a packed tensor to bf16: one thread per 32-weight block.
__global__ void mxfp4_dequant_kernel(const uint8_t* __restrict__ wq, const uint8_t* __restrict__ ws,
                                     __nv_bfloat16* __restrict__ out, long long n_blocks) {
  const long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= n_blocks) return;
  const float f = e8m0_to_float(ws[b]);
  const uint4 v = *reinterpret_cast<const uint4*>(wq + b * 16);
  const uint32_t words[4] = {v.x, v.y, v.z, v.w};
  __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(out + b * 32);
#pragma unroll
  for (int c = 0; c < 4; ++c)
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const __half2_raw hr = __nv_cvt_fp4x2_to_halfraw2(
          static_cast<__nv_fp4x2_storage_t>((words[c] >> (8 * k)) & 0xFFu), __NV_E2M1);
      const float2 ff = __half22float2(*reinterpret_cast<const __half2*>(&hr));
      o[c * 4 + k] = __floats2bfloat162_rn(ff.x * f, ff.y * f);
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

template <int EPI, int QMODE>
static int launch(const void* A, const void* Wq, const Params& p, int b_rows, int num_sms, cudaStream_t stream) {
  EncodeTiledFn enc = get_encode();
  if (enc == nullptr) return -10;
  CUtensorMap tmA, tmQ;
  {
    cuuint64_t dims[2] = {(cuuint64_t)p.K, (cuuint64_t)p.M};
    cuuint64_t strides[1] = {(cuuint64_t)p.K * 2};
    cuuint32_t box[2] = {BK, BM};
    cuuint32_t es[2] = {1, 1};
    if (enc(&tmA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(A), dims, strides, box, es,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return -11;
  }
  {
    cuuint64_t dims[2] = {(cuuint64_t)p.K / 2, (cuuint64_t)b_rows};
    cuuint64_t strides[1] = {(cuuint64_t)p.K / 2};
    cuuint32_t box[2] = {BK / 2, BN};
    cuuint32_t es[2] = {1, 1};
    if (enc(&tmQ, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(Wq), dims, strides, box, es,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return -12;
  }
  static DeviceOnce attr_set;
  auto kern = mxfp4_gemm_kernel<EPI, QMODE>;
  const size_t smem = kStages * kStageBytes + sizeof(Shared) + 1024;
  if (!ensure_dynamic_smem(kern, smem, attr_set)) return -13;
  const int n_tiles = (p.N + BN - 1) / BN;
  // upper bound on the tile count (grouped: every segment start is 128-aligned, so <= M/128 + groups row tiles)
  const long long m_tiles = p.offsets != nullptr ? (long long)p.M / BM + p.groups : (p.M + BM - 1) / BM;
  long long grid = m_tiles * n_tiles;
  if (grid > num_sms) grid = num_sms;
  if (grid < 1) grid = 1;
  kern<<<(int)grid, kThreads, smem, stream>>>(tmA, tmQ, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -14;
}

}  // namespace mx
}  // namespace bg

extern "C" {

// A: [M, K] bf16 row-major; Wq: [groups * N, K / 2] packed e2m1 (low nibble = even k); Ws: [groups * N, K / 32]
// e8m0; D: [M, ldd] bf16.  offsets == nullptr -> dense.  K % 64 == 0.  epi 1: rows of W interleaved
// (32 gate, 32 up), D gets N / 2 columns.  Returns 0 on a successful launch.
int bg_mxfp4_gemm(int epi, const void* A, const void* Wq, const void* Ws, void* D, int ldd, const int* offsets,
                  int groups, int M, int N, int K, int num_sms, int* status, cudaStream_t stream) {
  using namespace bg::mx;
  if (M <= 0 || N <= 0) return 0;
  if (K % BK != 0 || groups > kMaxGroups || (epi == EPI_SILU_MUL && (N % 128) != 0) || (ldd % 8) != 0) return -1;
  if (offsets == nullptr) groups = 1;
  Params p;
  p.ws = reinterpret_cast<const uint8_t*>(Ws); p.D = reinterpret_cast<__nv_bfloat16*>(D); p.ldd = ldd;
  p.offsets = offsets; p.groups = groups; p.M = M; p.N = N; p.K = K; p.status = status;
  if (epi == EPI_SILU_MUL) return launch<EPI_SILU_MUL, QMODE_MXFP4>(A, Wq, p, groups * N, num_sms, stream);
  return launch<EPI_STORE, QMODE_MXFP4>(A, Wq, p, groups * N, num_sms, stream);
}

// INT4 W4A16 (group size 32): Wq packs two offset-binary nibbles per byte (low nibble = even k, value = q - 8),
// Ws: [groups * N, K / 32] bf16 scales.  Everything else as bg_mxfp4_gemm.
// Replaces (by behaviour): the Marlin / INT4 WGMMA grouped kernels of the Kimi-K2.5 family (W4A16, gs = 32).
int bg_int4_gemm(int epi, const void* A, const void* Wq, const void* Ws, void* D, int ldd, const int* offsets,
                 int groups, int M, int N, int K, int num_sms, int* status, cudaStream_t stream) {
  using namespace bg::mx;
  if (M <= 0 || N <= 0) return 0;
  if (K % BK != 0 || groups > kMaxGroups || (epi == EPI_SILU_MUL && (N % 128) != 0) || (ldd % 8) != 0) return -1;
  if (offsets == nullptr) groups = 1;
  Params p;
  p.ws = reinterpret_cast<const uint8_t*>(Ws); p.D = reinterpret_cast<__nv_bfloat16*>(D); p.ldd = ldd;
  p.offsets = offsets; p.groups = groups; p.M = M; p.N = N; p.K = K; p.status = status;
  if (epi == EPI_SILU_MUL) return launch<EPI_SILU_MUL, QMODE_INT4>(A, Wq, p, groups * N, num_sms, stream);
  return launch<EPI_STORE, QMODE_INT4>(A, Wq, p, groups * N, num_sms, stream);
}

// out[i] = e2m1(wq[i]) * 2^(ws[i / 32] - 127), n elements (multiple of 32).
int bg_mxfp4_dequant(const void* wq, const void* ws, void* out, long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (n % 32 != 0) return -1;
  const long long nb = n / 32;
  bg::mx::mxfp4_dequant_kernel<<<(unsigned)((nb + 255) / 256), 256, 0, stream>>>(
      reinterpret_cast<const uint8_t*>(wq), reinterpret_cast<const uint8_t*>(ws),
      reinterpret_cast<__nv_bfloat16*>(out), nb);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

}  // extern "C"
