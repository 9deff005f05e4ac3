// Varlen causal multi-head attention for MLA prefill in the expanded (non-absorbed) form, on tcgen05.
//
// For long prompts the absorbed form (queries projected into the 576-wide latent space) costs 3.4x the
// FLOPs of plain attention over up-projected keys and values (192-wide keys = 128 nope + 64 rope, 128-wide
// values).  This kernel is the flash-attention forward for that shape:
//
//   S[q, k] = Q[q, 0:192] . K[k, 0:192]          (M = 128 queries, N = 64 keys; both K-major via TMA)
//   O[q, :] += P[q, k] . V[k, 0:128]             (M = 128, N = 128; V read N-major, P written by the softmax
//                                                 threads as a swizzled K-major tile)
//
// One CTA = one (128-query tile, head).  Query row i of the tile sees the first kv0 + i keys of its
// sequence's key range, which covers causal masking, cached context (kv0 > 1 for the first query) and the
// boundary to the next sequence in the packed batch with a single comparison.  A thread owns a query row
// (TMEM lane), so the online softmax needs no cross-thread reduction; the accumulator is rescaled only when
// the running maximum grew by more than 2^8.  K/V tiles flow through a 3-stage TMA ring; S of tile t+1 is
// issued before P.V of tile t.
//
// Roles (192 threads): warp 0 TMA producer, warp 1 MMA issuer + TMEM owner, warps 2..5 softmax / epilogue.
// All waits are bounded (common.cuh).
//
// Replaces (by behaviour): FA2/FA3 varlen prefill as dispatched by batchgen/attention/varlen_dispatch.py and
// prefill_attn_w8a16_prepacked (batchgen/models/deepseek/deepseekv3/wrappers.py:251-303).
#include "common.cuh"

namespace bg {
namespace mha {

constexpr int kDqk = 192, kDv = 128;
constexpr int kKvRow = 256;                      // per head in the kv_b projection output: 128 key-nope dims | 128 value dims
constexpr int BM = 128, BN = 64;
constexpr int kStages = 3;
constexpr int kThreads = 192;
constexpr int kQBytes = 3 * BM * 128;            // 48 KB
constexpr int kKBytes = 3 * BN * 128;            // 24 KB
constexpr int kVBytes = 2 * BN * 128;            // 16 KB
constexpr int kPBytes = BM * 128;                // 16 KB
constexpr int kTmemCols = 256;                   // S: 2 x 64, O: 128

struct Work {
  int q_row0;    // first query row of the tile (rows of Q / out)
  int n_q;       // queries in the tile (<= 128)
  int k_row0;    // first key row of the sequence (rows of K / V)
  int kv0;       // keys visible to query 0 of the tile (>= 1)
};

struct Shared {
  uint64_t q_full;
  uint64_t kv_full[kStages];
  uint64_t kv_empty[kStages];
  uint64_t s_full[2];
  uint64_t p_full;
  uint64_t o_done;
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ uint64_t desc_mn_sw128(uint32_t addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(lbo >> 4) << 16;
  d |= static_cast<uint64_t>(sbo >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}
__host__ __device__ constexpr uint32_t idesc_bf16(int M, int N, int b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(b_mn_major) << 16) |
         (static_cast<uint32_t>(N >> 3) << 17) | (static_cast<uint32_t>(M >> 4) << 24);
}
__device__ __forceinline__ bool mbar_probe(uint64_t* bar, uint32_t parity) {
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
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ bool vote_any_128(bool v) {      // barrier over the 128 softmax threads, OR of a flag
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
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* v) {
  tmem_ld_32x32(taddr, *reinterpret_cast<uint32_t(*)[32]>(v));
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, "
      "%25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
      "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]),
      "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]),
      "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
      : "memory");
}

__global__ void __launch_bounds__(kThreads, 1)
mha_prefill_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_kv,
                   const __grid_constant__ CUtensorMap tm_kpe, const Work* __restrict__ work,
                   __nv_bfloat16* __restrict__ out, int H, float scale_log2, int* status) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_buf = smem;
  uint8_t* k_buf = q_buf + kQBytes;
  uint8_t* v_buf = k_buf + kStages * kKBytes;
  uint8_t* p_buf = v_buf + kStages * kVBytes;
  Shared& ss = *reinterpret_cast<Shared*>(p_buf + kPBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort_flag = &ss.abort_flag;
  const Work w = work[blockIdx.x];
  const int h = blockIdx.y;
  const int n_tiles = (w.kv0 + w.n_q - 1 + BN - 1) / BN;

  if (threadIdx.x == 0) {
    mbar_init(&ss.q_full, 1);
    for (int s = 0; s < kStages; ++s) { mbar_init(&ss.kv_full[s], 1); mbar_init(&ss.kv_empty[s], 1); }
    mbar_init(&ss.s_full[0], 1);
    mbar_init(&ss.s_full[1], 1);
    mbar_init(&ss.p_full, 128);
    mbar_init(&ss.o_done, 1);
    ss.abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&ss.tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ss.tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (elect_one()) {
      mbar_expect_tx(&ss.q_full, kQBytes);
      for (int c = 0; c < 3; ++c) tma_load_2d(q_buf + c * BM * 128, &tm_q, &ss.q_full, h * kDqk + c * 64, w.q_row0);
      bool ok = true;
      for (int t = 0; t < n_tiles; ++t) {
        const int s = t % kStages;
        if (!mbar_wait(&ss.kv_empty[s], ((t / kStages) & 1) ^ 1, abort_flag, kTimeoutProducer)) { ok = false; break; }
        mbar_expect_tx(&ss.kv_full[s], kKBytes + kVBytes);
        const int krow = w.k_row0 + t * BN;
        // keys: 128 "nope" dims of this head out of the kv_b projection + the 64 roped dims shared by all heads
        for (int c = 0; c < 2; ++c) tma_load_2d(k_buf + s * kKBytes + c * BN * 128, &tm_kv, &ss.kv_full[s], h * kKvRow + c * 64, krow);
        tma_load_2d(k_buf + s * kKBytes + 2 * BN * 128, &tm_kpe, &ss.kv_full[s], 0, krow);
        for (int c = 0; c < 2; ++c) tma_load_2d(v_buf + s * kVBytes + c * BN * 128, &tm_kv, &ss.kv_full[s], h * kKvRow + 128 + c * 64, krow);
      }
      if (ok) {
        const int n = n_tiles < kStages ? n_tiles : kStages;
        for (int j = n_tiles - n; j < n_tiles; ++j)
          if (!mbar_wait(&ss.kv_empty[j % kStages], (j / kStages) & 1, abort_flag, kTimeoutProducer)) break;
      } else {
        for (uint32_t i = 0; i < (1u << 16); ++i) __nanosleep(20);   // bounded grace period for copies in flight
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc_s = idesc_bf16(BM, BN, 0);
      constexpr uint32_t idesc_pv = idesc_bf16(BM, kDv, 1);
      const uint32_t tm_o = tmem_base + 2 * BN;
      bool ok = mbar_wait(&ss.q_full, 0, abort_flag, kTimeoutMma);
      auto issue_s = [&](int t) -> bool {
        const int s = t % kStages;
        if (!mbar_wait(&ss.kv_full[s], (t / kStages) & 1, abort_flag, kTimeoutMma)) return false;
        tc_fence_after();
        const uint32_t tm_s = tmem_base + (t & 1) * BN;
        for (int c = 0; c < 3; ++c) {
          const uint64_t adesc = make_smem_desc_sw128(smem_u32(q_buf + c * BM * 128));
          const uint64_t bdesc = make_smem_desc_sw128(smem_u32(k_buf + s * kKBytes + c * BN * 128));
#pragma unroll
          for (int k = 0; k < 4; ++k) mma_f16(tm_s, adesc + 2 * k, bdesc + 2 * k, idesc_s, (c | k) ? 1u : 0u);
        }
        tc_commit(&ss.s_full[t & 1]);
        return true;
      };
      if (ok && n_tiles > 0) ok = issue_s(0);
      for (int t = 0; ok && t < n_tiles; ++t) {
        bool next_issued = true;
        if (t + 1 < n_tiles) {
          next_issued = mbar_probe(&ss.kv_full[(t + 1) % kStages], ((t + 1) / kStages) & 1);
          if (next_issued && !issue_s(t + 1)) { ok = false; break; }
        }
        if (!mbar_wait(&ss.p_full, t & 1, abort_flag, kTimeoutMma)) { ok = false; break; }
        tc_fence_after();
        const int s = t % kStages;
        const uint64_t pdesc = make_smem_desc_sw128(smem_u32(p_buf));
        const uint32_t v_base = smem_u32(v_buf + s * kVBytes);
#pragma unroll
        for (int j = 0; j < BN / 16; ++j)
          mma_f16(tm_o, pdesc + 2 * j, desc_mn_sw128(v_base + j * 2048, BN * 128, 1024), idesc_pv, (t > 0 || j > 0) ? 1u : 0u);
        tc_commit(&ss.kv_empty[s]);
        tc_commit(&ss.o_done);
        if (!next_issued && !issue_s(t + 1)) { ok = false; break; }
      }
    }
  } else {
    // ------------------------------------------------------------ softmax / correction / epilogue: thread = query row
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t tm_o = tmem_base + 2 * BN + lane_addr;
    const int visible = (r < w.n_q) ? (w.kv0 + r) : 0;       // keys this row may see
    float m_run = -INFINITY, l_run = 0.f;
    uint8_t* prow = p_buf + (r >> 3) * 1024 + (r & 7) * 128;
    bool ok = true;
    for (int t = 0; ok && t < n_tiles; ++t) {
      if (vote_any_128(!mbar_wait(&ss.s_full[t & 1], (t >> 1) & 1, abort_flag, kTimeoutEpilogue))) { ok = false; break; }
      tc_fence_after();
      uint32_t sv[64];
      tmem_ld32(tmem_base + lane_addr + (t & 1) * BN, sv);
      tmem_ld32(tmem_base + lane_addr + (t & 1) * BN + 32, sv + 32);
      tmem_ld_wait();
      const int n_ok = min(max(visible - t * BN, 0), BN);
      float mt = -INFINITY;
#pragma unroll
      for (int j = 0; j < 64; ++j) {
        const float v = (j < n_ok) ? __uint_as_float(sv[j]) * scale_log2 : -INFINITY;
        sv[j] = __float_as_uint(v);
        mt = fmaxf(mt, v);
      }
      const bool grow = mt > m_run + 8.f;
      const float m_new = grow ? mt : m_run;
      const float alpha = (grow && m_run != -INFINITY) ? ex2(m_run - m_new) : 1.f;
      if (t > 0 && vote_any_128(!mbar_wait(&ss.o_done, (t - 1) & 1, abort_flag, kTimeoutEpilogue))) { ok = false; break; }
      tc_fence_after();
      if (t > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t ov[32];
          tmem_ld32(tm_o + c * 32, ov);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) ov[j] = __float_as_uint(__uint_as_float(ov[j]) * alpha);
          tmem_st32(tm_o + c * 32, ov);
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      }
      float lsum = 0.f;
      const float neg_m = (m_new == -INFINITY) ? 0.f : -m_new;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        __align__(16) __nv_bfloat162 o[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float p0 = ex2(__uint_as_float(sv[c * 8 + 2 * q]) + neg_m);
          const float p1 = ex2(__uint_as_float(sv[c * 8 + 2 * q + 1]) + neg_m);
          o[q] = __floats2bfloat162_rn(p0, p1);
          lsum += __low2float(o[q]) + __high2float(o[q]);
        }
        *reinterpret_cast<uint4*>(prow + ((c ^ (r & 7)) << 4)) = *reinterpret_cast<const uint4*>(o);
      }
      l_run = l_run * alpha + lsum;
      m_run = m_new;
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      tc_fence_before();
      mbar_arrive(&ss.p_full);
    }
    if (ok && n_tiles > 0) ok = !vote_any_128(!mbar_wait(&ss.o_done, (n_tiles - 1) & 1, abort_flag, kTimeoutEpilogue));
    if (ok) {
      tc_fence_after();
      const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
      __nv_bfloat16* orow = out + ((size_t)(w.q_row0 + r) * H + h) * kDv;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t ov[32];
        tmem_ld32(tm_o + c * 32, ov);
        tmem_ld_wait();
        if (r < w.n_q) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            __align__(16) __nv_bfloat162 o[4];
#pragma unroll
            for (int q = 0; q < 4; ++q)
              o[q] = __floats2bfloat162_rn(__uint_as_float(ov[j + 2 * q]) * inv, __uint_as_float(ov[j + 2 * q + 1]) * inv);
            *reinterpret_cast<uint4*>(orow + c * 32 + j) = *reinterpret_cast<const uint4*>(o);
          }
        }
        __syncwarp();
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
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
static int make_map(CUtensorMap* m, const void* base, uint64_t cols, uint64_t rows, uint64_t row_stride,
                    uint32_t box_rows) {
  EncodeTiledFn enc = get_encode();
  if (enc == nullptr) return -1;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {row_stride * 2};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t es[2] = {1, 1};
  return enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, es,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS ? 0 : -2;
}

}  // namespace mha
}  // namespace bg

extern "C" {

// q [Tq, H, 192] (nope | roped pe), kv [Tk, H, 256] (key nope | value: the kv_b projection of the latent rows),
// kpe [Tk, kpe_stride] (roped shared key part in the first 64 columns), out [Tq, H, 128]: bf16.
// work: n_work x 4 ints (q_row0, n_q, k_row0, kv0), one CTA per work item and head.
int bg_mha_prefill(const void* q, const void* kv, const void* kpe, long long kpe_stride, void* out, const int* work,
                   int n_work, int Tq, int Tk, int H, float scale, int* status, cudaStream_t stream) {
  using namespace bg::mha;
  if (n_work <= 0 || H <= 0) return 0;
  if (kpe_stride % 8 != 0) return -1;
  CUtensorMap tq, tk, tv;
  if (make_map(&tq, q, (uint64_t)H * kDqk, (uint64_t)Tq, (uint64_t)H * kDqk, BM) != 0) return -10;
  if (make_map(&tk, kv, (uint64_t)H * kKvRow, (uint64_t)Tk, (uint64_t)H * kKvRow, BN) != 0) return -11;
  if (make_map(&tv, kpe, 64, (uint64_t)Tk, (uint64_t)kpe_stride, BN) != 0) return -12;
  static bg::DeviceOnce attr_set;
  const size_t smem = kQBytes + kStages * (kKBytes + kVBytes) + kPBytes + sizeof(Shared) + 1024;
  if (!bg::ensure_dynamic_smem(mha_prefill_kernel, smem, attr_set)) return -13;
  dim3 grid(n_work, H);
  mha_prefill_kernel<<<grid, kThreads, smem, stream>>>(tq, tk, tv, reinterpret_cast<const Work*>(work),
                                                       reinterpret_cast<__nv_bfloat16*>(out), H,
                                                       scale * 1.4426950408889634f, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -14;
}

}  // extern "C"
