// DSA (sparse-attention indexer) kernels.
//
//   index_k_write    LayerNorm -> RoPE on the first `rope` dims -> e4m3 quantisation (scale = max(amax,1e-4)/448,
//                    applied as a reciprocal multiply) -> paged store of the 128-wide index key + its fp32 scale
//   indexer_scores   score[b, t] = ks[t] * sum_h gate[b, h] * relu(q[b, h, :] . k[t, :]) over the paged FP8 index
//                    keys, on tcgen05: keys on the M axis (128 per tile, one 128-byte swizzled row each, loaded
//                    by TMA), the 32 index heads on the N axis, fp32 accumulators in TMEM; the head reduction is
//                    in-thread because a thread owns one key's row of the accumulator
//   topk_select      exact top-k (k <= 2048) of each row's scores by 8-bit radix select on an order-preserving
//                    integer key; rows no longer than k return all positions
//   gather_rows      copy the selected latent rows of every sequence into a dense per-sequence buffer that the
//                    paged MLA kernel then reads as ordinary pages
//
// Replaces (by behaviour): batchgen_kernels/src/attention/fused_indexer_k_norm_rope_write_fp8.cu:174,
// fused_indexer_k_write_fp8.cu:46, deep_gemm.fp8_paged_mqa_logits as called from
// batchgen_kernels/attention/dsa/paged_mqa_scorer.py:345, batchgen_kernels/src/attention/dsa_fast_topk.cu:201,
// batchgen_kernels/attention/dsa/fused_paged_gather.py; oracle batchgen/models/glm/glm5/model.py:610-700.
#include "common.cuh"

namespace bg {
namespace dsa {

constexpr int kD = 128;      // index head dim
constexpr int kPage = 64;
constexpr int kTileKeys = 128;

// One warp per token; lane l owns dims 4l..4l+3.
__global__ void __launch_bounds__(128)
index_k_write_kernel(const __nv_bfloat16* __restrict__ k, int ldk, const __nv_bfloat16* __restrict__ ln_w,
                     const __nv_bfloat16* __restrict__ ln_b, const int* __restrict__ positions,
                     const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rope, int interleaved,
                     const long long* __restrict__ slots, uint8_t* __restrict__ cache_k, float* __restrict__ cache_s,
                     int T, float eps) {
  const int t = blockIdx.x * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (t >= T) return;
  const long long slot = slots[t];
  float x[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) x[i] = __bfloat162float(k[(size_t)t * ldk + lane * 4 + i]);
  float mean = warp_sum(x[0] + x[1] + x[2] + x[3]) * (1.0f / kD);
  float var = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) var += (x[i] - mean) * (x[i] - mean);
  var = warp_sum(var) * (1.0f / kD);
  const float rstd = rsqrtf(var + eps);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int d = lane * 4 + i;
    x[i] = (x[i] - mean) * rstd * __bfloat162float(ln_w[d]) + (ln_b != nullptr ? __bfloat162float(ln_b[d]) : 0.f);
    x[i] = __bfloat162float(__float2bfloat16(x[i]));       // the unfused path rounds the norm output to bf16
  }
  const int half = rope / 2;
  const int pos = positions[t];
  if (interleaved) {
    if (lane * 4 < rope) {
#pragma unroll
      for (int p = 0; p < 2; ++p) {
        const int i = (lane * 4) / 2 + p;
        const float c = cos_t[(size_t)pos * half + i], s = sin_t[(size_t)pos * half + i];
        const float a = x[2 * p], b = x[2 * p + 1];
        x[2 * p] = a * c - b * s;
        x[2 * p + 1] = b * c + a * s;
      }
    }
  } else {
    // pairs (d, d + half): partner lane holds the other element
    const int lanes_half = half / 4;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int d = lane * 4 + i;
      const float other = __shfl_xor_sync(0xffffffffu, x[i], lanes_half);
      if (d < rope) {
        const int j = d % half;
        const float c = cos_t[(size_t)pos * half + j], s = sin_t[(size_t)pos * half + j];
        x[i] = (d < half) ? x[i] * c - other * s : x[i] * c + other * s;
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) x[i] = __bfloat162float(__float2bfloat16(x[i]));
  float amax = fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3])));
  amax = warp_max(amax);
  const float sc = fmaxf(amax, 1e-4f) * (1.0f / 448.0f);
  const float inv = 1.0f / sc;
  if (slot < 0) return;
  __align__(4) uint16_t q[2] = {to_e4m3x2(x[0] * inv, x[1] * inv), to_e4m3x2(x[2] * inv, x[3] * inv)};
  *reinterpret_cast<uint32_t*>(cache_k + (size_t)slot * kD + lane * 4) = *reinterpret_cast<const uint32_t*>(q);
  if (lane == 0) cache_s[slot] = sc;
}

// ---------------------------------------------------------------------------------------------
// Indexer scores on tcgen05.  One CTA per (row b, chunk of key tiles).  Threads: warp 0 = TMA producer,
// warp 1 = MMA issuer + TMEM owner, warps 2..5 = epilogue (thread = key).
constexpr int kScoreThreads = 192;
constexpr int kScoreStages = 8;      // 8 x 16 KB key tiles in flight
constexpr int kHeads = 32;

struct ScoreShared {
  uint64_t full[kScoreStages];
  uint64_t empty[kScoreStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  float gate[kHeads];
};

struct ScoreParams {
  const uint8_t* q8;          // [B, 32, 128] e4m3 (per-head scale folded into gate)
  const float* gate;          // [B, 32]
  const float* key_scale;     // [pages * 64]
  const int* block_table;
  int bt_stride;
  const int* lengths;         // [B] number of keys to score
  float* scores;              // [B, ld_scores]
  long long ld_scores;
  int tiles_per_cta;
  int* status;
};

__global__ void __launch_bounds__(kScoreThreads, 1)
indexer_scores_kernel(const __grid_constant__ CUtensorMap tm_keys, ScoreParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* key_buf = smem;                                   // stages x 128 keys x 128 B
  uint8_t* q_buf = key_buf + kScoreStages * kTileKeys * kD;  // 32 heads x 128 B, swizzled like a TMA tile
  ScoreShared& ss = *reinterpret_cast<ScoreShared*>(q_buf + kHeads * kD);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.y;
  const int len = p.lengths[b];
  const int n_tiles_total = (len + kTileKeys - 1) / kTileKeys;
  const int tile0 = blockIdx.x * p.tiles_per_cta;
  const int n_tiles = max(0, min(p.tiles_per_cta, n_tiles_total - tile0));
  volatile int* abort_flag = &ss.abort_flag;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kScoreStages; ++s) { mbar_init(&ss.full[s], 1); mbar_init(&ss.empty[s], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&ss.acc_full[i], 1); mbar_init(&ss.acc_empty[i], 4); }
    ss.abort_flag = 0;
    mbar_fence_init();
  }
  if (threadIdx.x < kHeads) ss.gate[threadIdx.x] = p.gate[(size_t)b * kHeads + threadIdx.x];
  // Q^T into shared memory in the 128-byte swizzled K-major layout (16-byte chunk index XOR row%8)
  for (int i = threadIdx.x; i < kHeads * 8; i += kScoreThreads) {
    const int h = i / 8, c = i % 8;
    const uint4 v = *reinterpret_cast<const uint4*>(p.q8 + ((size_t)b * kHeads + h) * kD + c * 16);
    *reinterpret_cast<uint4*>(q_buf + (h / 8) * 1024 + (h % 8) * 128 + ((c ^ (h % 8)) * 16)) = v;
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  if (warp == 1) {
    tmem_alloc(&ss.tmem_base, 64);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ss.tmem_base;
  const int* bt = p.block_table + (size_t)b * p.bt_stride;
  const int n_pages = (len + kPage - 1) / kPage;

  if (warp == 0) {
    if (elect_one()) {
      bool ok = true;
      for (int t = 0; ok && t < n_tiles; ++t) {
        const int s = t % kScoreStages;
        if (!mbar_wait(&ss.empty[s], ((t / kScoreStages) & 1) ^ 1, abort_flag, kTimeoutProducer)) { ok = false; break; }
        mbar_expect_tx(&ss.full[s], kTileKeys * kD);
        for (int h = 0; h < 2; ++h) {
          const int pi = (tile0 + t) * 2 + h;
          const int page = bt[pi < n_pages ? pi : 0];
          tma_load_2d(key_buf + s * kTileKeys * kD + h * kPage * kD, &tm_keys, &ss.full[s], 0, page * kPage);
        }
      }
      if (ok) {
        const int n = n_tiles < kScoreStages ? n_tiles : kScoreStages;
        for (int j = n_tiles - n; j < n_tiles; ++j)
          if (!mbar_wait(&ss.empty[j % kScoreStages], (j / kScoreStages) & 1, abort_flag, kTimeoutProducer)) break;
      } else {
        for (uint32_t i = 0; i < (1u << 16); ++i) __nanosleep(20);
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc(128, kHeads, 0, 0);
      const uint64_t bdesc = make_smem_desc_sw128(smem_u32(q_buf));
      bool ok = true;
      for (int t = 0; ok && t < n_tiles; ++t) {
        const int s = t % kScoreStages, buf = t & 1;
        if (!mbar_wait(&ss.acc_empty[buf], ((t >> 1) & 1) ^ 1, abort_flag, kTimeoutMma)) { ok = false; break; }
        if (!mbar_wait(&ss.full[s], (t / kScoreStages) & 1, abort_flag, kTimeoutMma)) { ok = false; break; }
        tc_fence_after();
        const uint64_t adesc = make_smem_desc_sw128(smem_u32(key_buf + s * kTileKeys * kD));
#pragma unroll
        for (int k = 0; k < 4; ++k) mma_f8f6f4(tmem_base + buf * kHeads, adesc + 2 * k, bdesc + 2 * k, idesc, k ? 1u : 0u);
        tc_commit(&ss.empty[s]);
        tc_commit(&ss.acc_full[buf]);
      }
    }
  } else {
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    bool ok = true;
    for (int t = 0; ok && t < n_tiles; ++t) {
      const int buf = t & 1;
      if (!__all_sync(0xffffffffu, mbar_wait(&ss.acc_full[buf], (t >> 1) & 1, abort_flag, kTimeoutEpilogue))) { ok = false; break; }
      tc_fence_after();
      uint32_t v[32];
      tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + buf * kHeads, v);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ss.acc_empty[buf]);
      float acc = 0.f;
#pragma unroll
      for (int h = 0; h < kHeads; ++h) acc = fmaf(ss.gate[h], fmaxf(__uint_as_float(v[h]), 0.f), acc);
      const int key = (tile0 + t) * kTileKeys + row;
      if (key < len) {
        const int page = bt[key / kPage];
        p.scores[(size_t)b * p.ld_scores + key] = acc * p.key_scale[(size_t)page * kPage + key % kPage];
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, 64);
  if (threadIdx.x == 0 && ss.abort_flag != 0 && p.status != nullptr) atomicMax(p.status, ss.abort_flag);
}

// ---------------------------------------------------------------------------------------------
// Exact top-k by radix select.  One CTA of 1024 threads per row.
__device__ __forceinline__ uint32_t order_key(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);     // larger float -> larger unsigned
}

__global__ void __launch_bounds__(1024)
topk_select_kernel(const float* __restrict__ scores, long long ld, const int* __restrict__ lengths, int k,
                   int* __restrict__ out_idx, int ld_out, int* __restrict__ out_len) {
  __shared__ int hist[256];
  __shared__ uint32_t prefix_s;
  __shared__ int need_s, cnt_gt, cnt_eq;
  const int b = blockIdx.x;
  const int len = lengths[b];
  const float* s = scores + (size_t)b * ld;
  int* out = out_idx + (size_t)b * ld_out;
  if (len <= k) {
    for (int i = threadIdx.x; i < len; i += blockDim.x) out[i] = i;
    if (threadIdx.x == 0) out_len[b] = len < 0 ? 0 : len;
    return;
  }
  if (threadIdx.x == 0) { prefix_s = 0u; need_s = k; }
  __syncthreads();
  // four passes, most significant byte first: find the k-th largest key exactly
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    const uint32_t prefix = prefix_s;
    const uint32_t mask = pass == 0 ? 0u : (0xFFFFFFFFu << (shift + 8));
    for (int i = threadIdx.x; i < len; i += blockDim.x) {
      const uint32_t key = order_key(s[i]);
      if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 0xFF], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int need = need_s, bin = 255;
      for (; bin > 0; --bin) {
        if (hist[bin] >= need) break;
        need -= hist[bin];
      }
      need_s = need;
      prefix_s = prefix | (static_cast<uint32_t>(bin) << shift);
    }
    __syncthreads();
  }
  const uint32_t thr = prefix_s;        // key of the k-th largest element
  const int need_eq = need_s;           // how many elements equal to it belong to the top k
  if (threadIdx.x == 0) { cnt_gt = 0; cnt_eq = 0; }
  __syncthreads();
  const int n_gt = k - need_eq;
  for (int i = threadIdx.x; i < len; i += blockDim.x) {
    const uint32_t key = order_key(s[i]);
    if (key > thr) {
      out[atomicAdd(&cnt_gt, 1)] = i;
    } else if (key == thr) {
      const int e = atomicAdd(&cnt_eq, 1);
      if (e < need_eq) out[n_gt + e] = i;
    }
  }
  if (threadIdx.x == 0) out_len[b] = k;
}

// One block per (sequence, selected row): copy a latent row into the dense buffer.  Rows between the selection's
// length and the end of its last 64-row tile are zero-filled (the attention kernel multiplies them by a zero
// probability, so they must be finite); rows past that tile are never read and stay untouched, so the caller does
// not have to clear the buffer.
__global__ void __launch_bounds__(64)
gather_rows_kernel(const uint4* __restrict__ cache, const int* __restrict__ block_table, int bt_stride,
                   const int* __restrict__ sel_idx, int ld_sel, const int* __restrict__ sel_len, uint4* __restrict__ out,
                   int row_vec, int page, int max_sel) {
  const int b = blockIdx.y, j = blockIdx.x;
  const int n = sel_len[b];
  if (j >= n) {
    if (j < (n + page - 1) / page * page) {
      uint4* z = out + ((size_t)b * max_sel + j) * row_vec;
      for (int i = threadIdx.x; i < row_vec; i += blockDim.x) z[i] = make_uint4(0u, 0u, 0u, 0u);
    }
    return;
  }
  const int pos = sel_idx[(size_t)b * ld_sel + j];
  const size_t slot = (size_t)block_table[(size_t)b * bt_stride + pos / page] * page + pos % page;
  const uint4* src = cache + slot * row_vec;
  uint4* dst = out + ((size_t)b * max_sel + j) * row_vec;
  for (int i = threadIdx.x; i < row_vec; i += blockDim.x) dst[i] = src[i];
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

}  // namespace dsa

namespace dsa {

// Indexer queries: RoPE on the leading `rope` dims of every head, per-head e4m3 quantisation, and the per-head
// scale folded into the head gate (gate_out = gate_in * gate_mul * scale).  q [T, 32, 128] bf16 with row stride
// ldq; one warp per (token, head), lane l owns dims 4l..4l+3.
__global__ void __launch_bounds__(256)
index_q_prepare_kernel(const __nv_bfloat16* __restrict__ q, long long ldq, const int* __restrict__ positions,
                       const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rope, int interleaved,
                       const float* __restrict__ gate_in, float gate_mul, uint8_t* __restrict__ q8,
                       float* __restrict__ gate_out, int heads) {
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31;
  const int pos = positions[t];
  const int half = rope / 2;
  for (int h = threadIdx.x >> 5; h < heads; h += blockDim.x >> 5) {
    const __nv_bfloat16* src = q + (size_t)t * ldq + (size_t)h * kD + lane * 4;
    float x[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) x[i] = __bfloat162float(src[i]);
    if (interleaved) {
      if (lane * 4 < rope) {
#pragma unroll
        for (int p = 0; p < 2; ++p) {
          const int i = (lane * 4) / 2 + p;
          const float c = cos_t[(size_t)pos * half + i], s = sin_t[(size_t)pos * half + i];
          const float a = x[2 * p], b = x[2 * p + 1];
          x[2 * p] = a * c - b * s;
          x[2 * p + 1] = b * c + a * s;
        }
      }
    } else {
      const int lanes_half = half / 4;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int d = lane * 4 + i;
        const float other = __shfl_xor_sync(0xffffffffu, x[i], lanes_half);
        if (d < rope) {
          const int j = d % half;
          const float c = cos_t[(size_t)pos * half + j], s = sin_t[(size_t)pos * half + j];
          x[i] = (d < half) ? x[i] * c - other * s : x[i] * c + other * s;
        }
      }
    }
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      x[i] = __bfloat162float(__float2bfloat16(x[i]));      // the unfused path rounds the rotated query to bf16
      amax = fmaxf(amax, fabsf(x[i]));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float sc = fmaxf(amax, 1e-4f) / 448.0f;
    const float inv = 1.0f / sc;
    __nv_fp8x4_e4m3 packed(make_float4(x[0] * inv, x[1] * inv, x[2] * inv, x[3] * inv));
    *reinterpret_cast<__nv_fp8x4_e4m3*>(q8 + ((size_t)t * heads + h) * kD + lane * 4) = packed;
    if (lane == 0) gate_out[(size_t)t * heads + h] = gate_in[(size_t)t * heads + h] * gate_mul * sc;
  }
}

}  // namespace dsa

}  // namespace bg

extern "C" {

int bg_index_k_write(const void* k, int ldk, const void* ln_w, const void* ln_b, const int* positions,
                     const float* cos_t, const float* sin_t, int rope, int interleaved, const long long* slots,
                     void* cache_k, float* cache_s, int T, float eps, cudaStream_t stream) {
  using namespace bg::dsa;
  if (T <= 0) return 0;
  if (rope % 8 != 0 || rope > kD) return -1;
  index_k_write_kernel<<<(T + 3) / 4, 128, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(k), ldk, reinterpret_cast<const __nv_bfloat16*>(ln_w),
      reinterpret_cast<const __nv_bfloat16*>(ln_b), positions, cos_t, sin_t, rope, interleaved, slots,
      reinterpret_cast<uint8_t*>(cache_k), cache_s, T, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// q [T, heads(32), 128] bf16 (row stride ldq elements) -> q8 [T, heads, 128] e4m3 and gate_out [T, heads] fp32.
int bg_index_q_prepare(const void* q, long long ldq, const int* positions, const float* cos_t, const float* sin_t,
                       int rope, int interleaved, const float* gate_in, float gate_mul, void* q8, float* gate_out,
                       int T, int heads, cudaStream_t stream) {
  using namespace bg::dsa;
  if (T <= 0) return 0;
  if (rope % 8 != 0 || rope > kD || heads <= 0) return -1;
  index_q_prepare_kernel<<<T, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(q), ldq, positions, cos_t, sin_t,
                                                rope, interleaved, gate_in, gate_mul,
                                                reinterpret_cast<uint8_t*>(q8), gate_out, heads);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// q8: [B, 32, 128] e4m3; gate: [B, 32] fp32 (already multiplied by the per-head q scale);
// keys: [n_pages*64, 128] e4m3; key_scale: [n_pages*64]; scores: [B, ld_scores] fp32.
int bg_indexer_scores(const void* q8, const float* gate, const void* keys, long long key_rows, const float* key_scale,
                      const int* block_table, int bt_stride, const int* lengths, float* scores, long long ld_scores,
                      int B, int max_len, int num_sms, int* status, cudaStream_t stream) {
  using namespace bg::dsa;
  if (B <= 0 || max_len <= 0) return 0;
  EncodeTiledFn enc = get_encode();
  if (enc == nullptr) return -10;
  CUtensorMap tm;
  cuuint64_t dims[2] = {(cuuint64_t)kD, (cuuint64_t)key_rows};
  cuuint64_t strides[1] = {(cuuint64_t)kD};
  cuuint32_t box[2] = {(cuuint32_t)kD, (cuuint32_t)kPage};
  cuuint32_t estr[2] = {1, 1};
  if (enc(&tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(keys), dims, strides, box, estr,
          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return -11;
  const int tiles = (max_len + kTileKeys - 1) / kTileKeys;
  int chunks = (2 * num_sms + B - 1) / B;                      // enough CTAs to fill the machine twice over
  if (chunks > tiles) chunks = tiles;
  if (chunks < 1) chunks = 1;
  const int tiles_per_cta = (tiles + chunks - 1) / chunks;
  chunks = (tiles + tiles_per_cta - 1) / tiles_per_cta;
  ScoreParams p;
  p.q8 = reinterpret_cast<const uint8_t*>(q8); p.gate = gate; p.key_scale = key_scale; p.block_table = block_table;
  p.bt_stride = bt_stride; p.lengths = lengths; p.scores = scores; p.ld_scores = ld_scores;
  p.tiles_per_cta = tiles_per_cta; p.status = status;
  const size_t smem = kScoreStages * kTileKeys * kD + kHeads * kD + sizeof(ScoreShared) + 1024;
  static bg::DeviceOnce attr;
  if (!bg::ensure_dynamic_smem(indexer_scores_kernel, smem, attr)) return -12;
  indexer_scores_kernel<<<dim3(chunks, B), kScoreThreads, smem, stream>>>(tm, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -13;
}

int bg_topk_select(const float* scores, long long ld, const int* lengths, int k, int* out_idx, int ld_out, int* out_len,
                   int B, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (k <= 0 || k > ld_out) return -1;
  bg::dsa::topk_select_kernel<<<B, 1024, 0, stream>>>(scores, ld, lengths, k, out_idx, ld_out, out_len);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int bg_gather_rows(const void* cache, const int* block_table, int bt_stride, const int* sel_idx, int ld_sel,
                   const int* sel_len, void* out, int row_bytes, int page, int max_sel, int B, cudaStream_t stream) {
  if (B <= 0 || max_sel <= 0) return 0;
  if (row_bytes % 16 != 0) return -1;
  bg::dsa::gather_rows_kernel<<<dim3(max_sel, B), 64, 0, stream>>>(
      reinterpret_cast<const uint4*>(cache), block_table, bt_stride, sel_idx, ld_sel, sel_len,
      reinterpret_cast<uint4*>(out), row_bytes / 16, page, max_sel);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

}  // extern "C"
