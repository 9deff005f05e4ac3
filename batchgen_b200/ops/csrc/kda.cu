// Kimi Delta Attention (gated delta-rule linear attention), prefill and decode in one kernel.
//
// Per head the layer keeps a state S [D keys x D values] (fp32) and the last three raw inputs of every
// q/k/v channel (the window of the width-4 causal depthwise convolution).  For each token, in order:
//
//   q, k, v  = silu(conv4(raw q, k, v))                   q, k then L2-normalised, q times `scale`
//   a        = exp(-exp(A_log[h]) * softplus(f + dt_bias))  per key channel (decay in (0, 1])
//   S        = diag(a) S
//   u        = sigmoid(beta) * (v - S^T k)
//   S        = S + k u^T
//   o        = S^T q
//   out      = o * rsqrt(mean(o^2) + eps) * w_norm * sigmoid(z)
//
// One CTA handles one (sequence, head); two threads share value column j of S in registers (D / 2 rows each),
// so S^T k, S^T q and the rank-one update need one exchange of two partial sums per token besides the two
// block-wide sums (the q/k norms and the output norm).  S^T q is taken from the decayed state in the same pass as
// S^T k (o = S'^T q + u * (k . q)), so the state is swept twice per token, not three times.  Decode is the
// one-token case and is bound by reading and writing the state (2 * D * D * 4 bytes per head and row).
//
// Replaces (by behaviour): the fused KDA decode kernel, the causal conv1d forward/update kernels and the
// chunked / recurrent delta-rule library calls of the reference (attention/kda_fused_decode.cu:147,429,707;
// conv1d/causal_conv1d.cu:446,679; batchgen/models/moonshotai/kimi_linear/serving_modules.py:579-722,1074,1202).
#include "common.cuh"

namespace bg {
namespace kda {

struct Params {
  const __nv_bfloat16* qkv;  // [T, >= 3*H*D]: raw q | k | v blocks of H*D each, row stride qkv_stride
  const __nv_bfloat16* f;    // [T, H*D] decay-gate pre-activation
  const __nv_bfloat16* beta; // [T, H]
  const __nv_bfloat16* z;    // [T, H*D] output gate
  int qkv_stride, f_stride, beta_stride, z_stride;
  const float* conv_w;       // [3*H*D, 4], tap 3 multiplies the current token
  const float* conv_b;       // [3*H*D] or null
  const float* A_log;        // [H]
  const float* dt_bias;      // [H*D]
  const float* norm_w;       // [D]
  float* conv_state;         // [slots, 3*H*D, 3] oldest first
  float* rec_state;          // [slots, H, D, D]
  const int* cu_seqlens;     // [nseq + 1] or null (one token per sequence: decode)
  const int* slots;          // [nseq]; < 0 skips the sequence
  const int* has_initial;    // [nseq] or null (null: always continue from the slot)
  __nv_bfloat16* out;        // [T, H*D] contiguous
  int H;
  float scale, eps;
};

__device__ __forceinline__ float silu(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float sigmoid(float x) { return 1.f / (1.f + __expf(-x)); }
__device__ __forceinline__ float softplus(float x) { return x > 20.f ? x : log1pf(__expf(x)); }

template <int D>
__global__ void __launch_bounds__(2 * D, 2) kda_seq_kernel(const Params p) {
  constexpr int R = D / 2;                 // state rows per thread: two threads share a value column
  constexpr int kWarpsHalf = D / 32;
  const int h = blockIdx.x, seq = blockIdx.y, tid = threadIdx.x;
  const int half = tid / D, j = tid % D, warp = tid >> 5, lane = tid & 31;
  const int slot = p.slots[seq];
  if (slot < 0) return;
  const int t0 = p.cu_seqlens ? p.cu_seqlens[seq] : seq;
  const int t1 = p.cu_seqlens ? p.cu_seqlens[seq + 1] : seq + 1;
  if (t1 <= t0) return;
  const int H = p.H, HD = H * D, c = h * D + j;
  const bool init = p.has_initial == nullptr || p.has_initial[seq] != 0;

  __shared__ __align__(16) float sq[2][D], sk[2][D], sa[2][D], sv[2][D];
  __shared__ float red[2][kWarpsHalf][3], red_o[kWarpsHalf];
  __shared__ float2 part[2][D];

  float S[R];
  float* Sg = p.rec_state + (((size_t)slot * H + h) * D + half * R) * D + j;
  if (init) {
#pragma unroll
    for (int i = 0; i < R; ++i) S[i] = Sg[(size_t)i * D];
  } else {
#pragma unroll
    for (int i = 0; i < R; ++i) S[i] = 0.f;
  }
  // half 0 runs the q and k channels of column j, half 1 the v channel and the decay gate
  const int n_ch = half == 0 ? 2 : 1;
  const int ch0 = half == 0 ? 0 : 2;
  float win[2][3], tap[2][4], bias[2];
#pragma unroll
  for (int s = 0; s < 2; ++s) {
    if (s < n_ch) {
      const size_t ch = (size_t)(ch0 + s) * HD + c;
      const float* cs = p.conv_state + ((size_t)slot * 3 * HD + ch) * 3;
#pragma unroll
      for (int i = 0; i < 3; ++i) win[s][i] = init ? cs[i] : 0.f;
      const float4 w4 = *reinterpret_cast<const float4*>(p.conv_w + ch * 4);
      tap[s][0] = w4.x; tap[s][1] = w4.y; tap[s][2] = w4.z; tap[s][3] = w4.w;
      bias[s] = p.conv_b ? p.conv_b[ch] : 0.f;
    } else {
#pragma unroll
      for (int i = 0; i < 3; ++i) win[s][i] = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) tap[s][i] = 0.f;
      bias[s] = 0.f;
    }
  }
  const float neg_a = -__expf(p.A_log[h]);
  const float dtb = p.dt_bias[c];
  const float nw = p.norm_w[j];

  // x[0..1]: raw conv inputs of this thread's channels; g: z (half 0) or f (half 1); bv: beta of the head
  auto load = [&](int t, float (&x)[2], float& g, float& bv) {
    const __nv_bfloat16* r = p.qkv + (size_t)t * p.qkv_stride + (size_t)ch0 * HD + c;
    x[0] = __bfloat162float(r[0]);
    x[1] = half == 0 ? __bfloat162float(r[HD]) : 0.f;
    g = half == 0 ? __bfloat162float(p.z[(size_t)t * p.z_stride + c]) : __bfloat162float(p.f[(size_t)t * p.f_stride + c]);
    bv = __bfloat162float(p.beta[(size_t)t * p.beta_stride + h]);
  };
  float nx[2], ng, nb;
  load(t0, nx, ng, nb);

  for (int t = t0; t < t1; ++t) {
    const int par = (t - t0) & 1;
    const float x[2] = {nx[0], nx[1]};
    const float g = ng, bv = nb;
    if (t + 1 < t1) load(t + 1, nx, ng, nb);              // next token's inputs fly during this token's math
    float y[2];
#pragma unroll
    for (int s = 0; s < 2; ++s) {
      y[s] = silu(bias[s] + tap[s][0] * win[s][0] + tap[s][1] * win[s][1] + tap[s][2] * win[s][2] + tap[s][3] * x[s]);
      win[s][0] = win[s][1]; win[s][1] = win[s][2]; win[s][2] = x[s];
    }
    if (half == 0) {
      sq[par][j] = y[0]; sk[par][j] = y[1];
      const float r0 = warp_sum(y[0] * y[0]), r1 = warp_sum(y[1] * y[1]), r2 = warp_sum(y[0] * y[1]);
      if (lane == 0) { red[par][warp][0] = r0; red[par][warp][1] = r1; red[par][warp][2] = r2; }
    } else {
      sv[par][j] = y[0];
      sa[par][j] = __expf(neg_a * softplus(g + dtb));
    }
    __syncthreads();
    float qq = 0.f, kk = 0.f, qk = 0.f;
#pragma unroll
    for (int w = 0; w < kWarpsHalf; ++w) { qq += red[par][w][0]; kk += red[par][w][1]; qk += red[par][w][2]; }
    const float rq = rsqrtf(qq + 1e-6f) * p.scale, rk = rsqrtf(kk + 1e-6f);
    // pass 1: decay, S'^T k and S'^T q over this thread's rows (raw k, q; the scalar norms scale the sums)
    float ak = 0.f, aq = 0.f;
    const float* pa = &sa[par][half * R];
    const float* pk = &sk[par][half * R];
    const float* pq = &sq[par][half * R];
#pragma unroll
    for (int i = 0; i < R; i += 4) {
      const float4 a4 = *reinterpret_cast<const float4*>(pa + i);
      const float4 k4 = *reinterpret_cast<const float4*>(pk + i);
      const float4 q4 = *reinterpret_cast<const float4*>(pq + i);
      S[i] *= a4.x;     ak = fmaf(S[i], k4.x, ak);     aq = fmaf(S[i], q4.x, aq);
      S[i + 1] *= a4.y; ak = fmaf(S[i + 1], k4.y, ak); aq = fmaf(S[i + 1], q4.y, aq);
      S[i + 2] *= a4.z; ak = fmaf(S[i + 2], k4.z, ak); aq = fmaf(S[i + 2], q4.z, aq);
      S[i + 3] *= a4.w; ak = fmaf(S[i + 3], k4.w, ak); aq = fmaf(S[i + 3], q4.w, aq);
    }
    part[half][j] = make_float2(ak, aq);
    __syncthreads();
    const float2 p0 = part[0][j], p1 = part[1][j];
    const float u = sigmoid(bv) * (sv[par][j] - (p0.x + p1.x) * rk);
    const float o = (p0.y + p1.y) * rq + u * (qk * rq * rk);
    const float uk = u * rk;
    // pass 2: rank-one update
#pragma unroll
    for (int i = 0; i < R; i += 4) {
      const float4 k4 = *reinterpret_cast<const float4*>(pk + i);
      S[i] = fmaf(k4.x, uk, S[i]);
      S[i + 1] = fmaf(k4.y, uk, S[i + 1]);
      S[i + 2] = fmaf(k4.z, uk, S[i + 2]);
      S[i + 3] = fmaf(k4.w, uk, S[i + 3]);
    }
    if (half == 0) {
      const float ro = warp_sum(o * o);
      if (lane == 0) red_o[warp] = ro;
    }
    __syncthreads();
    if (half == 0) {
      float oo = 0.f;
#pragma unroll
      for (int w = 0; w < kWarpsHalf; ++w) oo += red_o[w];
      p.out[(size_t)t * HD + c] = __float2bfloat16(o * rsqrtf(oo / D + p.eps) * nw * sigmoid(g));
    }
  }
#pragma unroll
  for (int i = 0; i < R; ++i) Sg[(size_t)i * D] = S[i];
#pragma unroll
  for (int s = 0; s < 2; ++s) {
    if (s < n_ch) {
      float* cs = p.conv_state + ((size_t)slot * 3 * HD + (size_t)(ch0 + s) * HD + c) * 3;
#pragma unroll
      for (int i = 0; i < 3; ++i) cs[i] = win[s][i];
    }
  }
}

}  // namespace kda
}  // namespace bg

extern "C" {

// See bg::kda::Params for the layouts.  D = 64 or 128; nseq sequences, H heads (this rank's).
int bg_kda_forward(const void* qkv, int qkv_stride, const void* f, int f_stride, const void* beta, int beta_stride,
                   const void* z, int z_stride, const float* conv_w, const float* conv_b, const float* A_log,
                   const float* dt_bias, const float* norm_w, float* conv_state, float* rec_state,
                   const int* cu_seqlens, const int* slots, const int* has_initial, void* out, int nseq, int H, int D,
                   float scale, float eps, cudaStream_t stream) {
  using namespace bg::kda;
  if (nseq <= 0) return 0;
  if ((D != 64 && D != 128) || H <= 0) return -1;
  Params p;
  p.qkv = reinterpret_cast<const __nv_bfloat16*>(qkv);
  p.f = reinterpret_cast<const __nv_bfloat16*>(f);
  p.beta = reinterpret_cast<const __nv_bfloat16*>(beta);
  p.z = reinterpret_cast<const __nv_bfloat16*>(z);
  p.qkv_stride = qkv_stride; p.f_stride = f_stride; p.beta_stride = beta_stride; p.z_stride = z_stride;
  p.conv_w = conv_w; p.conv_b = conv_b; p.A_log = A_log; p.dt_bias = dt_bias; p.norm_w = norm_w;
  p.conv_state = conv_state; p.rec_state = rec_state;
  p.cu_seqlens = cu_seqlens; p.slots = slots; p.has_initial = has_initial;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.H = H; p.scale = scale; p.eps = eps;
  dim3 grid(H, nseq);
  if (D == 128) kda_seq_kernel<128><<<grid, 256, 0, stream>>>(p);
  else kda_seq_kernel<64><<<grid, 128, 0, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

}  // extern "C"
