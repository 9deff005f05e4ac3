// Per-head batched bf16 GEMM for the MLA absorb steps, on tcgen05 with strided operands:
//
//   D[t, h, n] = sum_k A[t, h, k] * W[h, n, k]
//
// A and D are addressed in place inside [T, H, *] activations (row stride, head stride), so the
// "absorb W_UK into q" step reads q_nope straight out of the q projection [T, H, nope + rope] and writes
// q_abs [T, H, kv_lora], and the "out-absorb W_UV" step reads the latent attention output [T, H, kv_lora]
// and writes [T, H * v] — no transposes or packing copies around a library batched GEMM.
//
// One CTA per (128-row tile, head, N block); K runs through a 4-stage TMA ring in 64-element chunks;
// the accumulator (128 x BN fp32) lives in TMEM.  Roles: warp 0 TMA, warp 1 MMA, warps 2..5 epilogue.
//
// Replaces (by behaviour): batchgen_kernels/src/attention/fused_q_absorb.cu:13, the Triton
// fused_q_absorb.py and dsa/bf16_absorb.py, and the torch.bmm out-absorb of
// batchgen/models/deepseek/deepseekv3/modeling_deepseek_v3.py (W_UV application after FlashMLA).
#define BG_FILE_TAG 6      // kernel-trace ids of this file are (tag << 16) | line
#include "common.cuh"

namespace bg {
namespace hg {

constexpr int BM = 128;
constexpr int BKE = 64;              // bf16 elements per K chunk (one 128-byte swizzle atom)
constexpr int kStages = 4;
constexpr int kThreads = 192;

struct Params {
  __nv_bfloat16* D;
  long long d_row, d_head;           // element strides of D
  int T, N, K, a_head;               // a_head: element offset between heads inside a row of A
};

template <int BN> struct Shared {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t acc_full;
  uint32_t tmem_base;
  int abort_flag;
};

template <int BN>
__global__ void __launch_bounds__(kThreads, 1)
head_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmW, Params p, int* status) {
  bg::pdl_prologue((BG_FILE_TAG << 16) | __LINE__);
  constexpr int kABytes = BM * 128, kWBytes = BN * 128;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* a_tiles = smem;
  uint8_t* w_tiles = smem + kStages * kABytes;
  Shared<BN>& ss = *reinterpret_cast<Shared<BN>*>(w_tiles + kStages * kWBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.x * BM, h = blockIdx.y, n0 = blockIdx.z * BN;
  const int KC = p.K / BKE;
  volatile int* abort_flag = &ss.abort_flag;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&ss.full[s], 1); mbar_init(&ss.empty[s], 1); }
    mbar_init(&ss.acc_full, 1);
    ss.abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&ss.tmem_base, BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ss.tmem_base;

  if (warp == 0) {
    if (elect_one()) {
      bool ok = true;
      for (int kc = 0; kc < KC; ++kc) {
        const int s = kc % kStages;
        if (!mbar_wait(&ss.empty[s], ((kc / kStages) & 1) ^ 1, abort_flag, kTimeoutProducer)) { ok = false; break; }
        mbar_expect_tx(&ss.full[s], kABytes + kWBytes);
        tma_load_2d(a_tiles + s * kABytes, &tmA, &ss.full[s], h * p.a_head + kc * BKE, m0);
        tma_load_2d(w_tiles + s * kWBytes, &tmW, &ss.full[s], kc * BKE, h * p.N + n0);
      }
      if (ok) {   // every armed stage is released by the MMA role before the CTA may exit
        const int n = KC < kStages ? KC : kStages;
        for (int j = KC - n; j < KC; ++j)
          if (!mbar_wait(&ss.empty[j % kStages], (j / kStages) & 1, abort_flag, kTimeoutProducer)) break;
      } else {
        for (uint32_t i = 0; i < (1u << 16); ++i) __nanosleep(20);   // bounded grace period for copies in flight
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc(BM, BN, 1, 1);
      bool ok = true;
      for (int kc = 0; kc < KC && ok; ++kc) {
        const int s = kc % kStages;
        if (!mbar_wait(&ss.full[s], (kc / kStages) & 1, abort_flag, kTimeoutMma)) { ok = false; break; }
        tc_fence_after();
        const uint64_t adesc = make_smem_desc_sw128(smem_u32(a_tiles + s * kABytes));
        const uint64_t bdesc = make_smem_desc_sw128(smem_u32(w_tiles + s * kWBytes));
#pragma unroll
        for (int k = 0; k < BKE / 16; ++k) mma_f16(tmem_base, adesc + 2 * k, bdesc + 2 * k, idesc, (kc | k) ? 1u : 0u);
        tc_commit(&ss.empty[s]);
      }
      if (ok) tc_commit(&ss.acc_full);
    }
  } else {
    const int quad = warp & 3;
    const int row = m0 + quad * 32 + lane;
    const bool ok = __all_sync(0xffffffffu, mbar_wait(&ss.acc_full, 0, abort_flag, kTimeoutEpilogue));
    if (ok) {
      tc_fence_after();
      __nv_bfloat16* drow = p.D + (size_t)row * p.d_row + (size_t)h * p.d_head + n0;
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + c, v);
        tmem_ld_wait();
        if (row < p.T) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            if (n0 + c + j + 8 <= p.N) {
              __align__(16) __nv_bfloat162 o[4];
#pragma unroll
              for (int q = 0; q < 4; ++q)
                o[q] = __floats2bfloat162_rn(__uint_as_float(v[j + 2 * q]), __uint_as_float(v[j + 2 * q + 1]));
              *reinterpret_cast<uint4*>(drow + c + j) = *reinterpret_cast<const uint4*>(o);
            }
          }
        }
        __syncwarp();
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, BN);
  if (threadIdx.x == 0 && ss.abort_flag != 0 && status != nullptr) atomicMax(status, ss.abort_flag);
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
static int make_map(CUtensorMap* m, const void* base, uint64_t cols, uint64_t rows, uint64_t row_stride_elems,
                    uint32_t box_rows) {
  EncodeTiledFn enc = get_encode();
  if (enc == nullptr) return -1;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {row_stride_elems * 2};
  cuuint32_t box[2] = {BKE, box_rows};
  cuuint32_t es[2] = {1, 1};
  return enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, es,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS ? 0 : -2;
}

template <int BN>
static int launch(const CUtensorMap& a, const CUtensorMap& w, const Params& p, int H, int* status, cudaStream_t stream) {
  static DeviceOnce attr_set;
  auto kern = head_gemm_kernel<BN>;
  const size_t smem = kStages * (BM * 128 + BN * 128) + sizeof(Shared<BN>) + 1024;
  if (!ensure_dynamic_smem(kern, smem, attr_set)) return -12;
  dim3 grid((p.T + BM - 1) / BM, H, (p.N + BN - 1) / BN);
  bg::launch_pdl(kern, dim3(grid), dim3(kThreads), smem, stream, a, w, p, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -13;
}

}  // namespace hg
}  // namespace bg

extern "C" {

// A: bf16 rows of `a_row` elements (row stride), head h at element offset h * a_head, K elements used;
// W: [H, N, K] bf16 contiguous; D: element (t, h, n) at t * d_row + h * d_head + n.
// K % 64 == 0, N % 8 == 0, a_head % 8 == 0, a_row % 8 == 0, d_row % 8 == 0, d_head % 8 == 0.
int bg_head_gemm(const void* A, long long a_row, int a_head, long long a_cols, const void* W, void* D, long long d_row,
                 long long d_head, int T, int H, int N, int K, int* status, cudaStream_t stream) {
  using namespace bg::hg;
  if (T <= 0 || H <= 0) return 0;
  if (K % BKE != 0 || N % 8 != 0 || a_head % 8 != 0 || a_row % 8 != 0 || d_row % 8 != 0 || d_head % 8 != 0) return -1;
  CUtensorMap ta, tw;
  const int bn = N >= 256 ? 256 : 128;
  if (make_map(&ta, A, (uint64_t)a_cols, (uint64_t)T, (uint64_t)a_row, BM) != 0) return -10;
  if (make_map(&tw, W, (uint64_t)K, (uint64_t)H * N, (uint64_t)K, bn) != 0) return -11;
  Params p;
  p.D = reinterpret_cast<__nv_bfloat16*>(D); p.d_row = d_row; p.d_head = d_head;
  p.T = T; p.N = N; p.K = K; p.a_head = a_head;
  return bn == 256 ? launch<256>(ta, tw, p, H, status, stream) : launch<128>(ta, tw, p, H, status, stream);
}

}  // extern "C"

BG_TRACE_SETTER(head_gemm)
