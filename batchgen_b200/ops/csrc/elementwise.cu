// Memory-bound fused elementwise kernels: (residual add +) RMSNorm (+ per-token 1x128 e4m3
// quantisation), activation quantisation with optional SiLU*up, and the MLA latent-KV producer
// (RMSNorm of c_kv + RoPE of k_pe + paged cache write).
//
// Quantisation contract: scale = max(amax, 1e-4) / 448 (optionally rounded up to a power of two),
// q = x * (1 / scale) rounded to nearest e4m3, saturating.  The fused norm+quant kernel rounds
// the normalised value to bf16 first, so its bytes equal those of the unfused pair
// (the reference keeps the same contract: batchgen_kernels/src/attention/csrc/add_rmsnorm_fp8_quant.cu:243).
// Scales are written in [KB, stride] layout (scale of row t, block kb at s[kb * stride + t]),
// the layout the GEMM epilogue reads with coalesced loads.
//
// Replaces (by behaviour): batchgen_kernels/src/attention/csrc/rmsnorm.cu:88-254,
// add_rmsnorm_fp8_quant.cu:243, batchgen_kernels/src/moe/fp8_blockwise/fp8_blockwise_ops.cu:39-445,
// batchgen_kernels/src/attention/fused_kv_norm_rope_cache.cu:14, batchgen_kernels/triton/fp8_quantize.py.
#define BG_FILE_TAG 1      // kernel-trace ids of this file are (tag << 16) | line
#include "common.cuh"

namespace bg {

constexpr int kNormThreads = 256;

__device__ __forceinline__ float block_sum_256(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < (blockDim.x >> 5)) ? red[lane] : 0.f;
  t = warp_sum(t);
  __syncthreads();
  return t;
}

__device__ __forceinline__ float quant_scale(float amax, int pow2) {
  float s = fmaxf(amax, 1e-4f) * (1.0f / 448.0f);
  if (pow2) s = exp2f(ceilf(log2f(s)));
  return s;
}

// One block per row.  Each thread owns vectors of 8 consecutive elements; 16 consecutive threads
// cover one 128-wide quantisation block, so the block amax is a 16-lane shuffle reduction.
template <bool ADD, bool QUANT>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ residual,
               const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ out, uint8_t* __restrict__ out_q,
               float* __restrict__ out_s, int s_stride, int H, int ldx, int ldo, float eps, int pow2) {
  bg::pdl_prologue((BG_FILE_TAG << 16) | __LINE__);
  extern __shared__ float row[];  // H floats
  __shared__ float red[32];
  const int t = blockIdx.x;
  const __nv_bfloat16* xr = x + (size_t)t * ldx;
  __nv_bfloat16* rr = ADD ? residual + (size_t)t * H : nullptr;
  float ss = 0.f;
  for (int v = threadIdx.x; v < H / 8; v += kNormThreads) {
    uint4 raw = *reinterpret_cast<const uint4*>(xr + v * 8);
    const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&raw);
    float f[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 a = __bfloat1622float2(xp[i]);
      f[2 * i] = a.x;
      f[2 * i + 1] = a.y;
    }
    if (ADD) {
      uint4 rraw = *reinterpret_cast<const uint4*>(rr + v * 8);
      const __nv_bfloat162* rp = reinterpret_cast<const __nv_bfloat162*>(&rraw);
      __align__(16) __nv_bfloat162 o[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float2 a = __bfloat1622float2(rp[i]);
        o[i] = __floats2bfloat162_rn(f[2 * i] + a.x, f[2 * i + 1] + a.y);
        float2 b = __bfloat1622float2(o[i]);  // the sum as stored (bf16) is what gets normalised
        f[2 * i] = b.x;
        f[2 * i + 1] = b.y;
      }
      *reinterpret_cast<uint4*>(rr + v * 8) = *reinterpret_cast<const uint4*>(o);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      row[v * 8 + i] = f[i];
      ss += f[i] * f[i];
    }
  }
  const float total = block_sum_256(ss, red);
  const float rstd = rsqrtf(total / (float)H + eps);
  for (int v = threadIdx.x; v < H / 8; v += kNormThreads) {
    uint4 wraw = *reinterpret_cast<const uint4*>(w + v * 8);
    const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&wraw);
    __align__(16) __nv_bfloat162 o[4];
    float y[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 ww = __bfloat1622float2(wp[i]);
      o[i] = __floats2bfloat162_rn(row[v * 8 + 2 * i] * rstd * ww.x, row[v * 8 + 2 * i + 1] * rstd * ww.y);
      float2 b = __bfloat1622float2(o[i]);
      y[2 * i] = b.x;
      y[2 * i + 1] = b.y;
    }
    if (out != nullptr) *reinterpret_cast<uint4*>(out + (size_t)t * ldo + v * 8) = *reinterpret_cast<const uint4*>(o);
    if (QUANT) {
      float amax = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(y[i]));
#pragma unroll
      for (int o2 = 8; o2 > 0; o2 >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o2));
      const float s = quant_scale(amax, pow2);
      const float inv = 1.0f / s;
      __align__(8) uint16_t q[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) q[i] = to_e4m3x2(y[2 * i] * inv, y[2 * i + 1] * inv);
      *reinterpret_cast<uint2*>(out_q + (size_t)t * H + v * 8) = *reinterpret_cast<const uint2*>(q);
      if ((threadIdx.x & 15) == 0) out_s[(size_t)(v / 16) * s_stride + t] = s;
    }
  }
}

// Activation quantisation.  MODE 0: x [T, K].  MODE 1: x [T, 2K] = gate | up -> quantise silu(gate)*up.
// One warp per (row, group of 128-blocks): 16 lanes per 128-block, two blocks per warp pass.
template <int MODE>
__global__ void __launch_bounds__(256)
act_quant_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q, float* __restrict__ s, int s_stride,
                 int T, int K, int ldx, int pow2, const int* __restrict__ valid_rows,
                 const int* __restrict__ row_src) {
  bg::pdl_prologue((BG_FILE_TAG << 16) | __LINE__);
  const int t = blockIdx.x;
  if (valid_rows != nullptr && t >= *valid_rows) return;
  if (row_src != nullptr && row_src[t] < 0) return;      // padding row of an expert segment: nothing reads it
  const __nv_bfloat16* xr = x + (size_t)t * ldx;
  for (int v = threadIdx.x; v < K / 8; v += blockDim.x) {
    uint4 raw = *reinterpret_cast<const uint4*>(xr + v * 8);
    const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&raw);
    float f[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 a = __bfloat1622float2(xp[i]);
      f[2 * i] = a.x;
      f[2 * i + 1] = a.y;
    }
    if (MODE == 1) {
      uint4 uraw = *reinterpret_cast<const uint4*>(xr + K + v * 8);
      const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&uraw);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float2 u = __bfloat1622float2(up[i]);
        // round the activation to bf16 first: same bytes as silu_mul (bf16) followed by act_quant
        f[2 * i] = __bfloat162float(__float2bfloat16(silu(f[2 * i]) * u.x));
        f[2 * i + 1] = __bfloat162float(__float2bfloat16(silu(f[2 * i + 1]) * u.y));
      }
    }
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(f[i]));
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float sc = quant_scale(amax, pow2);
    const float inv = 1.0f / sc;
    __align__(8) uint16_t o4[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) o4[i] = to_e4m3x2(f[2 * i] * inv, f[2 * i + 1] * inv);
    *reinterpret_cast<uint2*>(q + (size_t)t * K + v * 8) = *reinterpret_cast<const uint2*>(o4);
    if ((threadIdx.x & 15) == 0) s[(size_t)(v / 16) * s_stride + t] = sc;
  }
}

// MLA latent-KV producer.  One block (128 threads) per token:
//   cache[slot, 0:kv_lora]        = rmsnorm(kv_a[t, 0:kv_lora]) * w
//   cache[slot, kv_lora:+rope]    = rope(kv_a[t, kv_lora:], position[t])
// slot < 0 writes nothing.  cos/sin are fp32 tables [max_pos, rope/2].
__global__ void __launch_bounds__(128)
mla_kv_write_kernel(const __nv_bfloat16* __restrict__ kv_a, int ld, const __nv_bfloat16* __restrict__ w,
                    const int* __restrict__ positions, const float* __restrict__ cos_t,
                    const float* __restrict__ sin_t, const long long* __restrict__ slots,
                    __nv_bfloat16* __restrict__ cache, int kv_lora, int rope, float eps, int interleaved) {
  bg::pdl_prologue((BG_FILE_TAG << 16) | __LINE__);
  __shared__ float red[32];
  const int t = blockIdx.x;
  const long long slot = slots[t];
  const __nv_bfloat16* src = kv_a + (size_t)t * ld;
  float ss = 0.f;
  for (int i = threadIdx.x; i < kv_lora; i += blockDim.x) {
    const float v = __bfloat162float(src[i]);
    ss += v * v;
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
  for (int i = 0; i < (blockDim.x >> 5); ++i) tot += red[i];
  if (slot < 0) return;
  const float rstd = rsqrtf(tot / (float)kv_lora + eps);
  __nv_bfloat16* dst = cache + (size_t)slot * (kv_lora + rope);
  for (int i = threadIdx.x; i < kv_lora; i += blockDim.x)
    dst[i] = __float2bfloat16(__bfloat162float(src[i]) * rstd * __bfloat162float(w[i]));
  const int half = rope / 2;
  const int pos = positions[t];
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const float c = cos_t[(size_t)pos * half + i], s = sin_t[(size_t)pos * half + i];
    const int i0 = interleaved ? 2 * i : i, i1 = interleaved ? 2 * i + 1 : i + half;
    const float a = __bfloat162float(src[kv_lora + i0]), b = __bfloat162float(src[kv_lora + i1]);
    dst[kv_lora + i0] = __float2bfloat16(a * c - b * s);
    dst[kv_lora + i1] = __float2bfloat16(b * c + a * s);
  }
}

// In-place RoPE on the trailing `rope` dims of every head of q [T, H, D].
__global__ void rope_q_kernel(__nv_bfloat16* __restrict__ q, int H, int D, int rope, const int* __restrict__ positions,
                              const float* __restrict__ cos_t, const float* __restrict__ sin_t, int interleaved,
                              long long ld_t) {
  bg::pdl_prologue((BG_FILE_TAG << 16) | __LINE__);
  const int t = blockIdx.x;
  const int half = rope / 2;
  const int pos = positions[t];
  for (int idx = threadIdx.x; idx < H * half; idx += blockDim.x) {
    const int h = idx / half, i = idx % half;
    __nv_bfloat16* p = q + (size_t)t * ld_t + (size_t)h * D + (D - rope);
    const float c = cos_t[(size_t)pos * half + i], s = sin_t[(size_t)pos * half + i];
    const int i0 = interleaved ? 2 * i : i, i1 = interleaved ? 2 * i + 1 : i + half;
    const float a = __bfloat162float(p[i0]), b = __bfloat162float(p[i1]);
    p[i0] = __float2bfloat16(a * c - b * s);
    p[i1] = __float2bfloat16(b * c + a * s);
  }
}

}  // namespace bg

extern "C" {

// y = rmsnorm(x (+ residual)) * w; residual (if given) is updated in place with the sum.
// out (bf16, may be null), out_q/out_s (e4m3 + scales, may be null).  H % 128 == 0 when quantising,
// H % 8 == 0 always.
int bg_rmsnorm(const void* x, void* residual, const void* w, void* out, void* out_q, float* out_s, int s_stride,
               int T, int H, int ldx, int ldo, float eps, int pow2, cudaStream_t stream) {
  using namespace bg;
  if (T <= 0) return 0;
  if (H % 8 != 0 || (out_q != nullptr && H % 128 != 0)) return -1;
  const size_t smem = (size_t)H * sizeof(float);
  auto X = reinterpret_cast<const __nv_bfloat16*>(x);
  auto R = reinterpret_cast<__nv_bfloat16*>(residual);
  auto W = reinterpret_cast<const __nv_bfloat16*>(w);
  auto O = reinterpret_cast<__nv_bfloat16*>(out);
  auto Q = reinterpret_cast<uint8_t*>(out_q);
#define BG_LAUNCH(ADD, QNT)                                                                                      \
  bg::launch_pdl(rmsnorm_kernel<ADD, QNT>, dim3(T), dim3(kNormThreads), smem, stream, X, R, W, O, Q, out_s, s_stride, H, ldx, ldo, eps, pow2)
  if (residual != nullptr && out_q != nullptr) BG_LAUNCH(true, true);
  else if (residual != nullptr) BG_LAUNCH(true, false);
  else if (out_q != nullptr) BG_LAUNCH(false, true);
  else BG_LAUNCH(false, false);
#undef BG_LAUNCH
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// mode 0: quantise x [T, K] (row stride ldx); mode 1: quantise silu(x[:, :K]) * x[:, K:2K].
// valid_rows (device int, may be null) limits the rows that are processed.
int bg_act_quant(int mode, const void* x, void* q, float* s, int s_stride, int T, int K, int ldx, int pow2,
                 const int* valid_rows, const int* row_src, cudaStream_t stream) {
  using namespace bg;
  if (T <= 0) return 0;
  if (K % 128 != 0) return -1;
  const int threads = K / 8 >= 256 ? 256 : ((K / 8 + 31) / 32) * 32;
  auto X = reinterpret_cast<const __nv_bfloat16*>(x);
  auto Q = reinterpret_cast<uint8_t*>(q);
  if (mode == 0) bg::launch_pdl(act_quant_kernel<0>, dim3(T), dim3(threads), 0, stream, X, Q, s, s_stride, T, K, ldx, pow2, valid_rows, row_src);
  else bg::launch_pdl(act_quant_kernel<1>, dim3(T), dim3(threads), 0, stream, X, Q, s, s_stride, T, K, ldx, pow2, valid_rows, row_src);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int bg_mla_kv_write(const void* kv_a, int ld, const void* w, const int* positions, const float* cos_t,
                    const float* sin_t, const long long* slots, void* cache, int T, int kv_lora, int rope, float eps,
                    int interleaved, cudaStream_t stream) {
  using namespace bg;
  if (T <= 0) return 0;
  bg::launch_pdl(mla_kv_write_kernel, dim3(T), dim3(128), 0, stream, reinterpret_cast<const __nv_bfloat16*>(kv_a), ld,
                                             reinterpret_cast<const __nv_bfloat16*>(w), positions, cos_t, sin_t, slots,
                                             reinterpret_cast<__nv_bfloat16*>(cache), kv_lora, rope, eps, interleaved);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int bg_rope_q(void* q, int T, int H, int D, int rope, const int* positions, const float* cos_t, const float* sin_t,
              int interleaved, long long ld_t, cudaStream_t stream) {
  using namespace bg;
  if (T <= 0) return 0;
  bg::launch_pdl(rope_q_kernel, dim3(T), dim3(256), 0, stream, reinterpret_cast<__nv_bfloat16*>(q), H, D, rope, positions, cos_t, sin_t,
                                       interleaved, ld_t);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

}  // extern "C"

BG_TRACE_SETTER(elementwise)
