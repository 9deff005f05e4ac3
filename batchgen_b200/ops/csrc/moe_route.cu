// MoE routing kernels for the single-GPU path and the NCCL baseline path:
//   router_topk      sigmoid (+bias) group-limited top-k / softmax top-k, one warp per token
//   moe_count        per-local-expert counts -> 128-aligned segment offsets
//   moe_scatter      (token, k) pairs -> grouped row positions
//   moe_gather_quant gather token rows into the expert-grouped buffer fused with e4m3 quantisation
//   moe_combine      out[t] = sum_k w[t,k] * y[pos[t,k]] (+ shared-expert output), fixed k order
//
// Replaces (by behaviour): batchgen_kernels/src/moe/routing/gate_sigmoid_topk.cu:72,304,
// gate_topk_softmax.cu:44, mgn/moe_fused_gate.cu:84, routing/dispatch_count_gather.cu:32-239,
// dispatch_scatter_3d.cu:152-345, routing/reduce_weighted_scatter.cu:27 and
// dispatch_scatter_3d.cu:366-661 (ordered reduce: the k order here is fixed, so results are
// bit-reproducible run to run).
#define BG_FILE_TAG 2      // kernel-trace ids of this file are (tag << 16) | line
#include "common.cuh"

namespace bg {

constexpr int kMaxExperts = 1024;
constexpr int kMaxTopK = 16;

// One warp per token.  E <= 1024, K <= 16, n_group <= 32.
__global__ void __launch_bounds__(128)
router_topk_kernel(const float* __restrict__ logits, const float* __restrict__ bias, int* __restrict__ idx_out,
                   float* __restrict__ w_out, int T, int E, int K, int n_group, int topk_group, int norm, float scale,
                   int softmax_mode, const int* __restrict__ num_valid) {
  bg::pdl_prologue((BG_FILE_TAG << 16) | __LINE__);
  __shared__ float choice_s[4][kMaxExperts];
  __shared__ float score_s[4][kMaxExperts];
  __shared__ float group_s[4][32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 4 + warp;
  if (t >= T) return;
  float* choice = choice_s[warp];
  float* score = score_s[warp];
  if (num_valid != nullptr && t >= *num_valid) {  // padding row: deterministic filler
    for (int k = lane; k < K; k += 32) {
      idx_out[(size_t)t * K + k] = -1;
      w_out[(size_t)t * K + k] = 0.f;
    }
    return;
  }
  const float* lrow = logits + (size_t)t * E;
  // scoring modes: 0 sigmoid, 1 softmax over the selected logits, 2 softmax over every expert, 3 sqrt(softplus)
  float rmax = -INFINITY, rinv = 0.f;
  if (softmax_mode == 2) {
    for (int e = lane; e < E; e += 32) rmax = fmaxf(rmax, lrow[e]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) rmax = fmaxf(rmax, __shfl_xor_sync(0xffffffffu, rmax, o));
    float rsum = 0.f;
    for (int e = lane; e < E; e += 32) rsum += expf(lrow[e] - rmax);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) rsum += __shfl_xor_sync(0xffffffffu, rsum, o);
    rinv = 1.0f / rsum;
  }
  for (int e = lane; e < E; e += 32) {
    const float l = lrow[e];
    if (softmax_mode == 1) {
      score[e] = l;
      choice[e] = l;
    } else {
      float s;
      if (softmax_mode == 0) s = 1.0f / (1.0f + expf(-l));
      else if (softmax_mode == 2) s = expf(l - rmax) * rinv;
      else s = sqrtf(l > 20.f ? l : log1pf(expf(l)));
      score[e] = s;
      choice[e] = bias != nullptr ? s + bias[e] : s;
    }
  }
  __syncwarp();
  if (n_group > 1) {
    const int gs = E / n_group;
    if (lane < n_group) {
      float m1 = -INFINITY, m2 = -INFINITY;
      for (int i = 0; i < gs; ++i) {
        const float v = choice[lane * gs + i];
        if (v > m1) { m2 = m1; m1 = v; } else if (v > m2) { m2 = v; }
      }
      group_s[warp][lane] = softmax_mode == 2 ? m1 : m1 + m2;   // softmax_all ranks a group by its best expert
    }
    __syncwarp();
    // keep the topk_group best groups (ties -> lower index); lane g decides for group g
    if (lane < n_group) {
      const float mine = group_s[warp][lane];
      int better = 0;
      for (int g = 0; g < n_group; ++g) {
        const float o = group_s[warp][g];
        better += (o > mine) || (o == mine && g < lane);
      }
      if (better >= topk_group) {
        for (int i = 0; i < gs; ++i) choice[lane * gs + i] = -INFINITY;
      }
    }
    __syncwarp();
  }
  float wsum = 0.f;
  float my_w = 0.f;
  int my_i = -1;
  float sel_max = -INFINITY;
  for (int k = 0; k < K; ++k) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float v = choice[e];
      if (v > best) { best = v; bi = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (bi == 0x7fffffff) bi = 0;
    if (k == 0) sel_max = best;
    float wv = score[bi];
    if (softmax_mode == 1) wv = expf(wv - sel_max);
    wsum += wv;
    if (lane == k) { my_w = wv; my_i = bi; }
    __syncwarp();
    if (lane == 0) choice[bi] = -INFINITY;
    __syncwarp();
  }
  if (lane < K) {
    float wv = my_w;
    if (softmax_mode == 1) wv = wv / wsum;
    else if (norm && K > 1) wv = wv / (wsum + 1e-20f);
    idx_out[(size_t)t * K + lane] = my_i;
    w_out[(size_t)t * K + lane] = wv * scale;
  }
}

// Single block: counts of pairs routed to local experts [lo, hi) -> offsets with every segment
// start aligned to `align` rows; cursor[] zeroed for the scatter pass; total rows in offsets[El].
__global__ void __launch_bounds__(1024)
moe_count_kernel(const int* __restrict__ topk_idx, int n_pairs, int lo, int hi, int align, int* __restrict__ offsets,
                 int* __restrict__ cursor, const int* __restrict__ num_valid, int K) {
  bg::pdl_prologue((BG_FILE_TAG << 16) | __LINE__);
  __shared__ int cnt[kMaxExperts];
  const int El = hi - lo;
  for (int e = threadIdx.x; e < El; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  const int limit = (num_valid != nullptr) ? min(n_pairs, *num_valid * K) : n_pairs;
  for (int i = threadIdx.x; i < limit; i += blockDim.x) {
    const int e = topk_idx[i];
    if (e >= lo && e < hi) atomicAdd(&cnt[e - lo], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < El; ++e) {
      offsets[e] = run;
      run += ((cnt[e] + align - 1) / align) * align;
    }
    offsets[El] = run;
  }
  for (int e = threadIdx.x; e < El; e += blockDim.x) cursor[e] = 0;
}

__global__ void moe_scatter_kernel(const int* __restrict__ topk_idx, int n_pairs, int K, int lo, int hi,
                                   const int* __restrict__ offsets, int* __restrict__ cursor, int* __restrict__ pos,
                                   int* __restrict__ src_row, const int* __restrict__ num_valid) {
  bg::pdl_prologue((BG_FILE_TAG << 16) | __LINE__);
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_pairs) return;
  const int limit = (num_valid != nullptr) ? *num_valid * K : n_pairs;
  const int e = (i < limit) ? topk_idx[i] : -1;
  if (e >= lo && e < hi) {
    const int r = offsets[e - lo] + atomicAdd(&cursor[e - lo], 1);
    pos[i] = r;
    src_row[r] = i / K;
  } else {
    pos[i] = -1;
  }
}

// One block per grouped row: gather hidden[src_row[r]] (bf16) and quantise to e4m3 with 1x128
// scales.  Padding rows (src < 0) become zeros with scale 0 so they produce exact zeros, or are left
// untouched when `zero_padding` is 0 (the grouped GEMM is then given the real row counts).
__global__ void __launch_bounds__(256)
moe_gather_quant_kernel(const __nv_bfloat16* __restrict__ hidden, int ldh, const int* __restrict__ src_row,
                        const int* __restrict__ total_rows, uint8_t* __restrict__ q, float* __restrict__ s,
                        int s_stride, int K, int pow2, int zero_padding) {
  bg::pdl_prologue((BG_FILE_TAG << 16) | __LINE__);
  const int r = blockIdx.x;
  if (r >= *total_rows) return;
  const int src = src_row[r];
  if (src < 0 && !zero_padding) return;
  for (int v = threadIdx.x; v < K / 8; v += blockDim.x) {
    float f[8];
    if (src >= 0) {
      uint4 raw = *reinterpret_cast<const uint4*>(hidden + (size_t)src * ldh + v * 8);
      const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float2 a = __bfloat1622float2(xp[i]);
        f[2 * i] = a.x;
        f[2 * i + 1] = a.y;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = 0.f;
    }
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(f[i]));
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    float sc = fmaxf(amax, 1e-4f) * (1.0f / 448.0f);
    if (pow2) sc = exp2f(ceilf(log2f(sc)));
    const float inv = 1.0f / sc;
    __align__(8) uint16_t o4[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) o4[i] = to_e4m3x2(f[2 * i] * inv, f[2 * i + 1] * inv);
    *reinterpret_cast<uint2*>(q + (size_t)r * K + v * 8) = *reinterpret_cast<const uint2*>(o4);
    if ((threadIdx.x & 15) == 0) s[(size_t)(v / 16) * s_stride + r] = (src >= 0) ? sc : 0.f;
  }
}

// out[t] = (extra[t] if given) + sum_k w[t,k] * y[pos[t,k]], k ascending.  Grid (token, 2,048-column chunk): a
// thread owns 8 columns and has the top-k rows' loads in flight together, so a 48-token decode step still fills
// the SMs instead of walking each row serially in 48 blocks.
__global__ void __launch_bounds__(256)
moe_combine_kernel(const __nv_bfloat16* __restrict__ y, int ldy, const int* __restrict__ pos,
                   const float* __restrict__ w, const __nv_bfloat16* __restrict__ extra, int lde,
                   __nv_bfloat16* __restrict__ out, int ldo, int K, int H, int out_fp32) {
  bg::pdl_prologue((BG_FILE_TAG << 16) | __LINE__);
  const int t = blockIdx.x;
  __shared__ int p_s[kMaxTopK];
  __shared__ float w_s[kMaxTopK];
  if (threadIdx.x < K) {
    p_s[threadIdx.x] = pos[(size_t)t * K + threadIdx.x];
    w_s[threadIdx.x] = w[(size_t)t * K + threadIdx.x];
  }
  __syncthreads();
  const int v = blockIdx.y * blockDim.x + threadIdx.x;
  if (v < H / 8) {
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    for (int k0 = 0; k0 < K; k0 += 8) {
      uint4 raw[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int k = k0 + j;
        const int p = k < K ? p_s[k] : -1;
        raw[j] = p >= 0 ? *reinterpret_cast<const uint4*>(y + (size_t)p * ldy + v * 8) : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int k = k0 + j;
        if (k >= K || p_s[k] < 0) continue;
        const float wk = w_s[k];
        const __nv_bfloat162* yp = reinterpret_cast<const __nv_bfloat162*>(&raw[j]);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float2 a = __bfloat1622float2(yp[i]);
          acc[2 * i] = fmaf(wk, a.x, acc[2 * i]);
          acc[2 * i + 1] = fmaf(wk, a.y, acc[2 * i + 1]);
        }
      }
    }
    if (extra != nullptr) {
      uint4 raw = *reinterpret_cast<const uint4*>(extra + (size_t)t * lde + v * 8);
      const __nv_bfloat162* ep = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float2 a = __bfloat1622float2(ep[i]);
        acc[2 * i] += a.x;
        acc[2 * i + 1] += a.y;
      }
    }
    if (out_fp32) {
      float* o = reinterpret_cast<float*>(out) + (size_t)t * ldo + v * 8;
      *reinterpret_cast<float4*>(o) = make_float4(acc[0], acc[1], acc[2], acc[3]);
      *reinterpret_cast<float4*>(o + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
    } else {
      __align__(16) __nv_bfloat162 o[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) o[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
      *reinterpret_cast<uint4*>(out + (size_t)t * ldo + v * 8) = *reinterpret_cast<const uint4*>(o);
    }
  }
}

}  // namespace bg

extern "C" {

int bg_router_topk(const float* logits, const float* bias, int* idx, float* w, int T, int E, int K, int n_group,
                   int topk_group, int norm, float scale, int softmax_mode, const int* num_valid,
                   cudaStream_t stream) {
  using namespace bg;
  if (T <= 0) return 0;
  if (E > kMaxExperts || K > kMaxTopK || n_group > 32 || (n_group > 1 && E % n_group != 0)) return -1;
  bg::launch_pdl(router_topk_kernel, dim3((T + 3) / 4), dim3(128), 0, stream, logits, bias, idx, w, T, E, K, n_group, topk_group, norm, scale,
                                                      softmax_mode, num_valid);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// Builds offsets [El+1], pos [T*K], src_row [cap] (pre-filled with -1 here) for experts [lo, hi).
int bg_moe_permute(const int* topk_idx, int T, int K, int lo, int hi, int align, int* offsets, int* cursor, int* pos,
                   int* src_row, int cap, const int* num_valid, cudaStream_t stream) {
  using namespace bg;
  if (hi - lo > kMaxExperts) return -1;
  if (cudaMemsetAsync(src_row, 0xFF, (size_t)cap * sizeof(int), stream) != cudaSuccess) return -3;
  const int n_pairs = T * K;
  bg::launch_pdl(moe_count_kernel, dim3(1), dim3(1024), 0, stream, topk_idx, n_pairs, lo, hi, align, offsets, cursor, num_valid, K);
  if (n_pairs > 0)
    bg::launch_pdl(moe_scatter_kernel, dim3((n_pairs + 255) / 256), dim3(256), 0, stream, topk_idx, n_pairs, K, lo, hi, offsets, cursor, pos,
                                                                 src_row, num_valid);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int bg_moe_gather_quant(const void* hidden, int ldh, const int* src_row, const int* total_rows, void* q, float* s,
                        int s_stride, int cap, int K, int pow2, int zero_padding, cudaStream_t stream) {
  using namespace bg;
  if (cap <= 0) return 0;
  if (K % 128 != 0) return -1;
  bg::launch_pdl(moe_gather_quant_kernel, dim3(cap), dim3(256), 0, stream, reinterpret_cast<const __nv_bfloat16*>(hidden), ldh, src_row,
                                                   total_rows, reinterpret_cast<uint8_t*>(q), s, s_stride, K, pow2, zero_padding);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int bg_moe_combine(const void* y, int ldy, const int* pos, const float* w, const void* extra, int lde, void* out,
                   int ldo, int T, int K, int H, int out_fp32, cudaStream_t stream) {
  using namespace bg;
  if (T <= 0) return 0;
  if (K > kMaxTopK || H % 8 != 0) return -1;
  bg::launch_pdl(moe_combine_kernel, dim3(T, (H / 8 + 255) / 256), dim3(256), 0, stream, reinterpret_cast<const __nv_bfloat16*>(y), ldy, pos, w,
                                            reinterpret_cast<const __nv_bfloat16*>(extra), lde,
                                            reinterpret_cast<__nv_bfloat16*>(out), ldo, K, H, out_fp32);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

}  // extern "C"

BG_TRACE_SETTER(moe_route)
