// CPU decode attention over KV that lives in host memory: grouped-query attention for one new token per
// sequence, bf16 K/V, fp32 accumulation, AVX2 + FMA inner loops, parallel over (sequence, kv head) with
// std::thread.  It lets a row whose KV sits in the host tier take a decode step without first being
// loaded back to the GPU ("hetero attention").
//
// q:   [B, Hq, D]  fp32          out: [B, Hq, D] fp32
// k,v: per sequence a list of page pointers; a page holds `page_size` tokens of [Hkv, D] bf16
// Reference parity: core/Hetero_Attn/CPU_Kernels/grouped_query_attention_cpu_avx2_omp.cpp (bf16 GQA decode,
// AVX2 + OpenMP), core/Hetero_Attn/CPU_Kernels/cpu_kernels.h:50-56.
#include <immintrin.h>
#include <stdint.h>

#include <algorithm>
#include <cmath>
#include <cstring>
#include <thread>
#include <vector>

namespace bgcore {

static inline float bf16_to_f32(uint16_t v) {
  uint32_t u = static_cast<uint32_t>(v) << 16;
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}

#if defined(__AVX2__) && defined(__FMA__)
static inline __m256 load_bf16x8(const uint16_t* p) {
  __m128i raw = _mm_loadu_si128(reinterpret_cast<const __m128i*>(p));
  return _mm256_castsi256_ps(_mm256_slli_epi32(_mm256_cvtepu16_epi32(raw), 16));
}
static inline float hsum(__m256 v) {
  __m128 lo = _mm256_castps256_ps128(v), hi = _mm256_extractf128_ps(v, 1);
  lo = _mm_add_ps(lo, hi);
  lo = _mm_hadd_ps(lo, lo);
  lo = _mm_hadd_ps(lo, lo);
  return _mm_cvtss_f32(lo);
}
#endif

static float dot_bf16(const float* q, const uint16_t* k, int D) {
#if defined(__AVX2__) && defined(__FMA__)
  __m256 acc = _mm256_setzero_ps();
  int d = 0;
  for (; d + 8 <= D; d += 8) acc = _mm256_fmadd_ps(_mm256_loadu_ps(q + d), load_bf16x8(k + d), acc);
  float s = hsum(acc);
  for (; d < D; ++d) s += q[d] * bf16_to_f32(k[d]);
  return s;
#else
  float s = 0.f;
  for (int d = 0; d < D; ++d) s += q[d] * bf16_to_f32(k[d]);
  return s;
#endif
}

static void axpy_bf16(float a, const uint16_t* v, float* out, int D) {
#if defined(__AVX2__) && defined(__FMA__)
  __m256 av = _mm256_set1_ps(a);
  int d = 0;
  for (; d + 8 <= D; d += 8)
    _mm256_storeu_ps(out + d, _mm256_fmadd_ps(av, load_bf16x8(v + d), _mm256_loadu_ps(out + d)));
  for (; d < D; ++d) out[d] += a * bf16_to_f32(v[d]);
#else
  for (int d = 0; d < D; ++d) out[d] += a * bf16_to_f32(v[d]);
#endif
}

// One (sequence, kv head): all query heads of the group share the K/V stream.
static void gqa_one(const float* q, float* out, const uint16_t* const* k_pages, const uint16_t* const* v_pages,
                    int len, int page_size, int Hq, int Hkv, int D, int kvh, float scale, int window) {
  const int group = Hq / Hkv;
  const int start = (window > 0 && len > window) ? len - window : 0;
  std::vector<float> m(group, -INFINITY), l(group, 0.f);
  for (int g = 0; g < group; ++g) std::fill(out + (kvh * group + g) * D, out + (kvh * group + g + 1) * D, 0.f);
  for (int t = start; t < len; ++t) {
    const uint16_t* kp = k_pages[t / page_size] + ((size_t)(t % page_size) * Hkv + kvh) * D;
    const uint16_t* vp = v_pages[t / page_size] + ((size_t)(t % page_size) * Hkv + kvh) * D;
    for (int g = 0; g < group; ++g) {
      const int h = kvh * group + g;
      const float s = dot_bf16(q + h * D, kp, D) * scale;
      float* o = out + h * D;
      if (s > m[g]) {                       // new running maximum: rescale what is accumulated
        const float a = std::exp(m[g] - s);
        for (int d = 0; d < D; ++d) o[d] *= a;
        l[g] = l[g] * a + 1.f;
        m[g] = s;
        axpy_bf16(1.f, vp, o, D);
      } else {
        const float p = std::exp(s - m[g]);
        l[g] += p;
        axpy_bf16(p, vp, o, D);
      }
    }
  }
  for (int g = 0; g < group; ++g) {
    float* o = out + (kvh * group + g) * D;
    const float inv = l[g] > 0.f ? 1.f / l[g] : 0.f;
    for (int d = 0; d < D; ++d) o[d] *= inv;
  }
}

}  // namespace bgcore

extern "C" {

// k_pages / v_pages: [B * max_pages] page pointers (row b starts at b * max_pages).  lens: [B].
int bgc_cpu_gqa_decode(const float* q, float* out, const void* const* k_pages, const void* const* v_pages,
                       const int* lens, int B, int max_pages, int page_size, int Hq, int Hkv, int D, float scale,
                       int window, int num_threads) {
  if (Hkv <= 0 || Hq % Hkv != 0) return -1;
  const int jobs = B * Hkv;
  const int nt = std::max(1, std::min(num_threads, jobs));
  std::vector<std::thread> th;
  for (int t = 0; t < nt; ++t) {
    th.emplace_back([=] {
      for (int j = t; j < jobs; j += nt) {
        const int b = j / Hkv, kvh = j % Hkv;
        bgcore::gqa_one(q + (size_t)b * Hq * D, out + (size_t)b * Hq * D,
                        reinterpret_cast<const uint16_t* const*>(k_pages) + (size_t)b * max_pages,
                        reinterpret_cast<const uint16_t* const*>(v_pages) + (size_t)b * max_pages, lens[b], page_size,
                        Hq, Hkv, D, kvh, scale, window);
      }
    });
  }
  for (auto& x : th) x.join();
  return 0;
}

}  // extern "C"
