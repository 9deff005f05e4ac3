// Token sampling: one block per row.  Greedy rows (temperature <= 0) take an arg-max fast path.
// Sampled rows apply temperature, then top-k, then the top-p nucleus *of the distribution renormalised
// over the top-k survivors* (the two filters are sequential, as in batchgen/sampling.py:417-461), and
// draw from what is left with a caller-provided uniform number.  The kept set is found without
// sorting: a token with probability p is kept iff fewer than k tokens are more probable and the mass of
// the more probable tokens is at most top_p * Z_k (Z_k = mass of the top-k set), which is monotone in
// p, so each cut is a binary search over probability with one pass over the row per step.  With both
// filters active a first search finds the top-k cut and one more pass takes Z_k.  The draw walks the
// kept tokens in vocabulary order.  Rows with a non-finite maximum bump a device counter instead of
// raising.
//
// Replaces (by behaviour): the torch-op sampler batchgen/sampling.py:296-530 (per-row
// temperature/top-p/top-k tensors, greedy split, on-device bad-row counter).
#define BG_FILE_TAG 9      // kernel-trace ids of this file are (tag << 16) | line
#include "common.cuh"

namespace bg {

constexpr int kSampThreads = 1024;

template <typename T> __device__ __forceinline__ float ld_logit(const T* p, int i);
template <> __device__ __forceinline__ float ld_logit<float>(const float* p, int i) { return p[i]; }
template <> __device__ __forceinline__ float ld_logit<__nv_bfloat16>(const __nv_bfloat16* p, int i) {
  return __bfloat162float(p[i]);
}

__device__ __forceinline__ float block_reduce_sum(float v, float* red) {
  v = warp_sum(v);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = (threadIdx.x < 32) ? red[threadIdx.x] : 0.f;
  if (threadIdx.x < 32) t = warp_sum(t);
  if (threadIdx.x == 0) red[32] = t;
  __syncthreads();
  t = red[32];
  __syncthreads();
  return t;
}

template <typename T>
__global__ void __launch_bounds__(kSampThreads)
sample_kernel(const T* __restrict__ logits, long long ld, int V, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ uniform,
              int* __restrict__ out, int* __restrict__ bad_rows) {
  bg::pdl_prologue((BG_FILE_TAG << 16) | __LINE__);
  __shared__ float red[33];
  __shared__ float redv[32];
  __shared__ int redi[32];
  __shared__ float scan[kSampThreads];
  __shared__ int result;
  const int row = blockIdx.x;
  const T* l = logits + (size_t)row * ld;
  const int tid = threadIdx.x;
  // contiguous chunk per thread so that the final walk is in vocabulary order
  const int per = (V + kSampThreads - 1) / kSampThreads;
  const int lo = min(V, tid * per), hi = min(V, lo + per);

  // ---- arg-max (also the softmax max)
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = lo; i < hi; ++i) {
    const float v = ld_logit(l, i);
    if (v > best) { best = v; bi = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  if ((tid & 31) == 0) { redv[tid >> 5] = best; redi[tid >> 5] = bi; }
  __syncthreads();
  if (tid < 32) {
    best = redv[tid];
    bi = redi[tid];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (tid == 0) { redv[0] = best; redi[0] = bi; }
  }
  __syncthreads();
  const float gmax = redv[0];
  const int garg = redi[0];
  __syncthreads();
  const float temp = temperature != nullptr ? temperature[row] : 0.f;
  if (!(gmax > -INFINITY) || !(gmax < INFINITY)) {
    if (tid == 0) {
      if (bad_rows != nullptr) atomicAdd(bad_rows, 1);
      out[row] = garg == 0x7fffffff ? 0 : garg;
    }
    return;
  }
  if (temp <= 0.f) {
    if (tid == 0) out[row] = garg;
    return;
  }
  const float inv_t = 1.0f / fmaxf(temp, 1e-6f);
  // ---- normaliser
  float z = 0.f;
  for (int i = lo; i < hi; ++i) z += __expf((ld_logit(l, i) - gmax) * inv_t);
  z = block_reduce_sum(z, red);
  const float inv_z = 1.0f / z;
  const int k = (top_k != nullptr && top_k[row] > 0) ? top_k[row] : V;
  const float pp = top_p != nullptr ? top_p[row] : 1.0f;
  // ---- Z_k: mass of the top-k set (only needed when the nucleus is taken inside a real top-k cut)
  float zk = 1.0f;
  if (k < V && pp < 1.0f) {
    float lo_t = 0.f, hi_t = 1.0f;  // invariant: {p > hi_t} has fewer than k members
    for (int it = 0; it < 26; ++it) {
      const float mid = 0.5f * (lo_t + hi_t);
      float cnt = 0.f;
      for (int i = lo; i < hi; ++i) {
        const float p = __expf((ld_logit(l, i) - gmax) * inv_t) * inv_z;
        if (p > mid) cnt += 1.f;
      }
      cnt = block_reduce_sum(cnt, red);
      if (cnt < (float)k) hi_t = mid; else lo_t = mid;
    }
    float mass = 0.f;
    for (int i = lo; i < hi; ++i) {
      const float p = __expf((ld_logit(l, i) - gmax) * inv_t) * inv_z;
      if (p > lo_t) mass += p;
    }
    zk = block_reduce_sum(mass, red);
  }
  const float mass_cap = pp * zk;
  // ---- cut: smallest tau such that {p > tau} has count < k and mass <= top_p * Z_k  -> keep p > cut
  float cut = 0.f;
  if (k < V || pp < 1.0f) {
    float lo_t = 0.f, hi_t = 1.0f;  // invariant: tau = hi_t satisfies the constraints (p_max <= 1)
    for (int it = 0; it < 26; ++it) {
      const float mid = 0.5f * (lo_t + hi_t);
      float mass = 0.f, cnt = 0.f;
      for (int i = lo; i < hi; ++i) {
        const float p = __expf((ld_logit(l, i) - gmax) * inv_t) * inv_z;
        if (p > mid) { mass += p; cnt += 1.f; }
      }
      mass = block_reduce_sum(mass, red);
      cnt = block_reduce_sum(cnt, red);
      if (cnt < (float)k && (pp >= 1.0f || mass <= mass_cap)) hi_t = mid; else lo_t = mid;
    }
    cut = lo_t;  // tokens with p > lo_t: the first token violating the constraint sits just below
  }
  // ---- draw in vocabulary order
  float mine = 0.f;
  for (int i = lo; i < hi; ++i) {
    const float p = __expf((ld_logit(l, i) - gmax) * inv_t) * inv_z;
    if (p > cut || i == garg) mine += p;
  }
  scan[tid] = mine;
  __syncthreads();
  for (int off = 1; off < kSampThreads; off <<= 1) {
    float v = (tid >= off) ? scan[tid - off] : 0.f;
    __syncthreads();
    scan[tid] += v;
    __syncthreads();
  }
  const float total = scan[kSampThreads - 1];
  const float target = uniform[row] * total;
  if (tid == 0) result = garg;
  __syncthreads();
  const float before = scan[tid] - mine;
  if (mine > 0.f && target >= before && target < scan[tid]) {
    float run = before;
    int pick = -1;
    for (int i = lo; i < hi; ++i) {
      const float p = __expf((ld_logit(l, i) - gmax) * inv_t) * inv_z;
      if (p > cut || i == garg) {
        run += p;
        pick = i;
        if (run > target) break;
      }
    }
    if (pick >= 0) result = pick;
  }
  __syncthreads();
  if (tid == 0) out[row] = result;
}

}  // namespace bg

extern "C" {

// logits: [T, ld] of fp32 (dtype 0) or bf16 (dtype 1).  temperature/top_k/top_p/uniform may be null
// (=> greedy).  out: int32 [T].
int bg_sample(int dtype, const void* logits, long long ld, int T, int V, const float* temperature, const int* top_k,
              const float* top_p, const float* uniform, int* out, int* bad_rows, cudaStream_t stream) {
  using namespace bg;
  if (T <= 0) return 0;
  if (temperature != nullptr && uniform == nullptr) return -1;
  if (dtype == 0)
    bg::launch_pdl(sample_kernel<float>, dim3(T), dim3(kSampThreads), 0, stream, reinterpret_cast<const float*>(logits), ld, V, temperature,
                                                          top_k, top_p, uniform, out, bad_rows);
  else
    bg::launch_pdl(sample_kernel<__nv_bfloat16>, dim3(T), dim3(kSampThreads), 0, stream, reinterpret_cast<const __nv_bfloat16*>(logits), ld,
                                                                  V, temperature, top_k, top_p, uniform, out, bad_rows);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

}  // extern "C"

BG_TRACE_SETTER(sampling)
