// Grouped-query attention decode over a paged K/V cache, with sliding window and attention sinks.
//
// Cache row layout (one token): [K of Hkv heads | V of Hkv heads], each head D bf16 (D = 64 or 128), pages of
// `page` tokens (<= 64 per tile step).  One CTA handles one (sequence, KV head, split): the G = Hq / Hkv query
// heads that share the KV head are processed together, so every K/V byte is read once per CTA.  Decode is
// bound by those bytes, so the math runs on the CUDA cores: thread-per-token dot products for the scores,
// warp reductions for the per-head tile maxima, thread-per-dimension accumulation for P.V with the running
// (max, sum) rescaling of flash decoding.  Sequence lengths are read on the device (graph-capturable).
//
//   window > 0: only the last `window` positions are visible (pages wholly outside are skipped);
//   sinks != nullptr: exp(sink[h] - max) joins the softmax denominator of head h (no value).
//
// Replaces (by behaviour): the precompiled GQA decode extension the reference loads for GPT-OSS and its
// contract batchgen/attention/gqa/reference.py:13-141 (paged cache, sinks, sliding window).
#include "common.cuh"

namespace bg {
namespace gqa {

constexpr int kTile = 64;       // tokens per step
constexpr int kThreads = 128;
constexpr int kMaxG = 16;

template <int D>
__global__ void __launch_bounds__(kThreads)
gqa_decode_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ cache,
                  const int* __restrict__ block_table, int bt_stride, const int* __restrict__ seqlens,
                  const float* __restrict__ sinks, __nv_bfloat16* __restrict__ out, float* __restrict__ part_o,
                  float* __restrict__ part_ml, int Hq, int Hkv, int page, int window, float scale_log2, int n_splits) {
  const int b = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int G = Hq / Hkv;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int row = 2 * Hkv * D;                    // elements per cached token
  __shared__ float q_s[kMaxG][D];
  __shared__ float s_s[kTile][kMaxG + 1];
  __shared__ float m_s[kMaxG], a_s[kMaxG], l_s[kMaxG];
  __shared__ float acc_s[kMaxG][D];               // second half's partial when D == 64

  for (int i = tid; i < G * D; i += kThreads)
    q_s[i / D][i % D] = __bfloat162float(q[((size_t)b * Hq + kvh * G + i / D) * D + i % D]) * scale_log2;
  if (tid < G) { m_s[tid] = -INFINITY; l_s[tid] = 0.f; }
  const int L = seqlens[b];
  const int first = (window > 0 && L > window) ? (L - window) : 0;     // first visible position
  const int t_lo = first / kTile, t_hi = (L + kTile - 1) / kTile;     // tiles [t_lo, t_hi)
  const int n_t = max(t_hi - t_lo, 0);
  const int my_lo = t_lo + (int)(((long long)n_t * split) / n_splits);
  const int my_hi = t_lo + (int)(((long long)n_t * (split + 1)) / n_splits);
  // P.V mapping: D == 128 -> thread = dim over all 64 tokens; D == 64 -> thread = (token half, dim)
  constexpr int kHalves = kThreads / D;           // 1 or 2
  const int d = tid % D, thalf = tid / D;
  float acc[kMaxG];
#pragma unroll
  for (int g = 0; g < kMaxG; ++g) acc[g] = 0.f;
  __syncthreads();
  const int* bt = block_table + (size_t)b * bt_stride;
  const int tok_t = tid % kTile, ghalf = tid / kTile;      // score mapping: thread = (token, half of the heads)
  const int g0 = ghalf * ((G + 1) / 2), g1 = min(G, g0 + (G + 1) / 2);

  for (int t = my_lo; t < my_hi; ++t) {
    // ---- scores of this tile: s[tok][g] = q_g . k_tok (log2 domain), -inf outside [first, L)
    {
      const int pos = t * kTile + tok_t;
      const bool ok = pos >= first && pos < L;
      float s[kMaxG / 2 + 1];
#pragma unroll
      for (int i = 0; i < kMaxG / 2 + 1; ++i) s[i] = 0.f;
      if (ok) {
        const __nv_bfloat16* kr = cache + ((size_t)bt[pos / page] * page + pos % page) * row + kvh * D;
#pragma unroll 2
        for (int c = 0; c < D; c += 8) {
          const uint4 raw = *reinterpret_cast<const uint4*>(kr + c);
          const __nv_bfloat162* kp = reinterpret_cast<const __nv_bfloat162*>(&raw);
          float kf[8];
#pragma unroll
          for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(kp[i]); kf[2 * i] = f.x; kf[2 * i + 1] = f.y; }
          for (int g = g0; g < g1; ++g) {
            float a = s[g - g0];
#pragma unroll
            for (int i = 0; i < 8; ++i) a = fmaf(q_s[g][c + i], kf[i], a);
            s[g - g0] = a;
          }
        }
      }
      for (int g = g0; g < g1; ++g) s_s[tok_t][g] = ok ? s[g - g0] : -INFINITY;
    }
    __syncthreads();
    // ---- per-head tile maximum (warp w takes heads w, w + 4, ..), running max / rescale factors
    for (int g = warp; g < G; g += kThreads / 32) {
      float v = fmaxf(s_s[lane][g], s_s[lane + 32][g]);
      v = warp_max(v);
      if (lane == 0) {
        const float mo = m_s[g], mn = fmaxf(mo, v);
        a_s[g] = (mn == -INFINITY) ? 1.f : exp2f(mo - mn);
        m_s[g] = mn;
      }
    }
    __syncthreads();
    // ---- probabilities in place, row sums
    for (int g = g0; g < g1; ++g) {
      const float mn = m_s[g];
      const float sv = s_s[tok_t][g];
      s_s[tok_t][g] = (sv == -INFINITY) ? 0.f : exp2f(sv - mn);
    }
    __syncthreads();
    for (int g = warp; g < G; g += kThreads / 32) {
      float v = warp_sum(s_s[lane][g] + s_s[lane + 32][g]);
      if (lane == 0) l_s[g] = l_s[g] * a_s[g] + v;
    }
    // ---- O = O * alpha + P . V
    {
#pragma unroll
      for (int g = 0; g < kMaxG; ++g)
        if (g < G) acc[g] *= a_s[g];
      const int tok_a = thalf * (kTile / kHalves), tok_b = tok_a + kTile / kHalves;
      for (int tk = tok_a; tk < tok_b; ++tk) {
        const int pos = t * kTile + tk;
        if (pos >= L) break;
        if (pos < first) continue;
        const float v = __bfloat162float(cache[((size_t)bt[pos / page] * page + pos % page) * row + (Hkv + kvh) * D + d]);
#pragma unroll
        for (int g = 0; g < kMaxG; ++g)
          if (g < G) acc[g] = fmaf(s_s[tk][g], v, acc[g]);
      }
    }
    __syncthreads();
  }
  // ---- combine the two token halves (D == 64), then write
  if (kHalves == 2) {
    if (thalf == 1)
      for (int g = 0; g < G; ++g) acc_s[g][d] = acc[g];
    __syncthreads();
    if (thalf == 0)
      for (int g = 0; g < G; ++g) acc[g] += acc_s[g][d];
  }
  if (thalf == 0) {
    for (int g = 0; g < G; ++g) {
      const int h = kvh * G + g;
      if (n_splits == 1) {
        float l = l_s[g];
        if (sinks != nullptr && m_s[g] != -INFINITY) l += exp2f(sinks[h] * 1.4426950408889634f - m_s[g]);
        out[((size_t)b * Hq + h) * D + d] = __float2bfloat16(l > 0.f ? acc[g] / l : 0.f);
      } else {
        part_o[(((size_t)b * Hq + h) * n_splits + split) * D + d] = acc[g];
      }
    }
    if (n_splits > 1 && tid < G) {
      const int h = kvh * G + tid;
      part_ml[(((size_t)b * Hq + h) * n_splits + split) * 2] = m_s[tid];
      part_ml[(((size_t)b * Hq + h) * n_splits + split) * 2 + 1] = l_s[tid];
    }
  }
}

// one block per (sequence, head): merge split partials, add the sink to the denominator
__global__ void gqa_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                 const float* __restrict__ sinks, __nv_bfloat16* __restrict__ out, int Hq, int D,
                                 int n_splits) {
  const int bh = blockIdx.x, h = bh % Hq;
  float m = -INFINITY;
  for (int s = 0; s < n_splits; ++s) m = fmaxf(m, part_ml[((size_t)bh * n_splits + s) * 2]);
  float l = 0.f;
  for (int s = 0; s < n_splits; ++s) {
    const float ms = part_ml[((size_t)bh * n_splits + s) * 2];
    if (ms != -INFINITY) l += part_ml[((size_t)bh * n_splits + s) * 2 + 1] * exp2f(ms - m);
  }
  if (sinks != nullptr && m != -INFINITY) l += exp2f(sinks[h] * 1.4426950408889634f - m);
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float a = 0.f;
    for (int s = 0; s < n_splits; ++s) {
      const float ms = part_ml[((size_t)bh * n_splits + s) * 2];
      if (ms != -INFINITY) a += part_o[((size_t)bh * n_splits + s) * D + d] * exp2f(ms - m);
    }
    out[(size_t)bh * D + d] = __float2bfloat16(l > 0.f ? a / l : 0.f);
  }
}

}  // namespace gqa
}  // namespace bg

extern "C" {

// q [B, Hq, D] bf16 contiguous; cache [pages * page, 2 * Hkv * D] bf16; block_table [B, bt_stride] int32;
// seqlens [B] int32 (tokens visible to the query, including the one just written); sinks [Hq] fp32 or null;
// part_o [B * Hq * n_splits * D] / part_ml [B * Hq * n_splits * 2] fp32 scratch when n_splits > 1.
int bg_gqa_decode(const void* q, const void* cache, const int* block_table, int bt_stride, const int* seqlens,
                  const float* sinks, void* out, float* part_o, float* part_ml, int B, int Hq, int Hkv, int D, int page,
                  int window, float scale, int n_splits, cudaStream_t stream) {
  using namespace bg::gqa;
  if (B <= 0) return 0;
  if ((D != 64 && D != 128) || Hkv <= 0 || Hq % Hkv != 0 || Hq / Hkv > kMaxG || page <= 0 || kTile % page != 0 && page % kTile != 0 ||
      n_splits < 1 || (n_splits > 1 && (part_o == nullptr || part_ml == nullptr)))
    return -1;
  dim3 grid(B, Hkv, n_splits);
  const float sl2 = scale * 1.4426950408889634f;
  auto Q = reinterpret_cast<const __nv_bfloat16*>(q);
  auto C = reinterpret_cast<const __nv_bfloat16*>(cache);
  auto O = reinterpret_cast<__nv_bfloat16*>(out);
  if (D == 64)
    gqa_decode_kernel<64><<<grid, kThreads, 0, stream>>>(Q, C, block_table, bt_stride, seqlens, sinks, O, part_o, part_ml,
                                                         Hq, Hkv, page, window, sl2, n_splits);
  else
    gqa_decode_kernel<128><<<grid, kThreads, 0, stream>>>(Q, C, block_table, bt_stride, seqlens, sinks, O, part_o, part_ml,
                                                          Hq, Hkv, page, window, sl2, n_splits);
  if (n_splits > 1) gqa_merge_kernel<<<B * Hq, 64, 0, stream>>>(part_o, part_ml, sinks, O, Hq, D, n_splits);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

}  // extern "C"
