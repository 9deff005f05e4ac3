// Kernels that move data between GPUs themselves (plain peer loads/stores over NVLink into a
// symmetric heap) fused with the compute around the collective.  No NCCL call; TMA is used on local memory only.
//
//   sp_norm_quant_push     owner side of GEMM->reduce-scatter: sum the partial rows every rank pushed,
//                          add the residual, RMSNorm, quantise to e4m3 and push the quantised rows into
//                          every rank's all-gather buffer (the all-gather of the *next* GEMM's input)
//   ep_count_push          per-expert counts of this rank's routed tokens, pushed to every rank
//   ep_layout              segment layout of every rank's receive buffer from the gathered counts
//   ep_dispatch_send       quantise each local token once, store it straight into the receive buffer of
//                          each expert-owner rank at its expert-grouped row (+ return address)
//   wait_flags             stream-ordered bounded wait on arrival flags
//   barrier_all            flag barrier over all ranks (setup / teardown only)
//
// Synchronisation is by monotonically increasing epochs in flag words of the symmetric heap:
// a producer finishes its stores, issues a system-scope fence and release-stores the epoch into the
// consumer's flag; consumers acquire-load until flag >= epoch, for a bounded number of polls, after
// which they raise the status word and carry on (the host sees the error; the GPU never hangs).
//
// Replaces (by behaviour): NCCL all_gather / reduce_scatter / all_reduce around the MoE and
// tensor-parallel GEMMs (batchgen/models/glm/glm5/model.py:2428-2508,
// batchgen/models/deepseek/deepseekv3/modeling_deepseek_v3.py:3137,3173,
// batchgen/moe/fused_moe_mxfp4_resident.py:1020-1095) and the DeepEP low-latency dispatch/combine
// wrapper batchgen/moe/deepep_ll.py:240-400.
#define BG_FILE_TAG 10      // kernel-trace ids of this file are (tag << 16) | line
#include <cooperative_groups.h>

#include "../../ops/csrc/common.cuh"

namespace bg {
namespace comm {

constexpr int kMaxWorld = 8;
constexpr int kMaxExperts = 1024;

struct Peers {
  void* p[kMaxWorld];
};

// Epochs are passed as (offset, base pointer): the effective value is offset + *base.  The base lives in
// device memory and is bumped by bump_epoch_kernel at the end of every step, so a captured CUDA graph
// publishes and expects fresh epochs on every replay without any host involvement.
struct Epoch {
  uint32_t off;
  const uint32_t* base;
  __device__ __forceinline__ uint32_t get() const { return off + (base != nullptr ? *base : 0u); }
};

// One store that NVSwitch delivers to the same offset of every rank's mapping (multicast address of a symmetric
// region; NVLS).  Bits are stored as they are.
struct Multicast {
  void* ag_q = nullptr;
  void* ag_s = nullptr;
  void* cnt = nullptr;
};
inline Multicast& multicast() {
  static Multicast per_device[bg::kMaxDevices];
  static Multicast none;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= bg::kMaxDevices) return none;
  return per_device[dev];
}

__device__ __forceinline__ void multimem_st_b64(void* mc_addr, uint2 v) {
  asm volatile("multimem.st.relaxed.sys.global.v2.f32 [%0], {%1, %2};" ::"l"(mc_addr), "f"(__uint_as_float(v.x)),
               "f"(__uint_as_float(v.y))
               : "memory");
}
__device__ __forceinline__ void multimem_st_b32(void* mc_addr, uint32_t v) {
  asm volatile("multimem.st.relaxed.sys.global.f32 [%0], %1;" ::"l"(mc_addr), "f"(__uint_as_float(v)) : "memory");
}

__device__ __forceinline__ void signal_all(const Peers& flags, int index, int world, uint32_t epoch) {
  // callers have fenced (system scope) after the data stores; the flag stores themselves need no fence each
  for (int r = 0; r < world; ++r) st_relaxed_sys(reinterpret_cast<uint32_t*>(flags.p[r]) + index, epoch);
}

// Last-CTA-out signalling: every CTA fences its stores; the last one raises the flags.
__device__ __forceinline__ void cta_done_signal(unsigned int* counter, const Peers& flags, int index, int world,
                                                uint32_t epoch) {
  __threadfence_system();   // every thread: its own peer stores first
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const unsigned int prev = atomicAdd(counter, 1u);
    if (prev == gridDim.x * gridDim.y * gridDim.z - 1) {
      *counter = 0u;
      __threadfence_system();
      signal_all(flags, index, world, epoch);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// One cluster of gridDim.y blocks per owned row, each block a contiguous range of 128-column groups; the row's sum
// of squares is combined over the cluster through distributed shared memory (a decode step has few rows: one block
// per row left most SMs idle and made every thread walk several vectors and eight peers serially).
// partials: [n_src, rows, H] bf16 in this rank's memory (n_src = world when
// fed by GEMM->reduce-scatter, 1 when the input is a local tensor).  residual [rows, H] in/out.
// Outputs: y (bf16, local, optional), local e4m3 + scales (optional), and the pushed copy into every
// rank's gather buffer at row (my_rank * rows + r): ag_q [T, H] e4m3, ag_s [KB, ag_s_stride] fp32.
__global__ void __launch_bounds__(256)
sp_norm_quant_push_kernel(const __nv_bfloat16* __restrict__ partials, int n_src, const uint32_t* __restrict__ src_ready,
                          Epoch wait_epoch_e, __nv_bfloat16* __restrict__ residual,
                          const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                          uint8_t* __restrict__ loc_q, float* __restrict__ loc_s, int loc_s_stride, Peers ag_q,
                          Peers ag_s, int ag_s_stride, int push, int rows, int H, float eps, int my_rank, int world,
                          Peers flags, int ready_index, Epoch epoch_e, unsigned int* counter, int* status,
                          int has_residual, uint8_t* __restrict__ mc_q, float* __restrict__ mc_s) {
  bg::pdl_prologue((BG_FILE_TAG << 16) | __LINE__);
  const uint32_t wait_epoch = wait_epoch_e.get();
  const uint32_t epoch = epoch_e.get();
  extern __shared__ float rowbuf[];
  __shared__ float red[32];
  __shared__ float part_ss;
  __shared__ int wait_ok;
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  const int r = blockIdx.x;
  const int parts = gridDim.y;
  const int groups_pp = (H / 128 + parts - 1) / parts;            // 128-column groups per block
  const int v_lo = blockIdx.y * groups_pp * 16;
  const int v_hi = min(H / 8, v_lo + groups_pp * 16);
  if (src_ready != nullptr) {
    if (threadIdx.x == 0) {
      int ok = 1;
      for (int s = 0; s < n_src; ++s)
        if (!wait_flag_ge(src_ready + s, wait_epoch, status)) ok = 0;
      if (!ok && status != nullptr) atomicMax(status, (int)kTimeoutPeer);
      wait_ok = ok;
    }
    __syncthreads();
  }
  float ss = 0.f;
  for (int v = v_lo + threadIdx.x; v < v_hi; v += blockDim.x) {
    float f[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = 0.f;
    for (int s = 0; s < n_src; ++s) {   // fixed source order: bit-reproducible sum
      uint4 raw = *reinterpret_cast<const uint4*>(partials + ((size_t)s * rows + r) * H + v * 8);
      const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float2 a = __bfloat1622float2(xp[i]);
        f[2 * i] += a.x;
        f[2 * i + 1] += a.y;
      }
    }
    if (has_residual) {
      uint4 rraw = *reinterpret_cast<const uint4*>(residual + (size_t)r * H + v * 8);
      const __nv_bfloat162* rp = reinterpret_cast<const __nv_bfloat162*>(&rraw);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float2 a = __bfloat1622float2(rp[i]);
        f[2 * i] += a.x;
        f[2 * i + 1] += a.y;
      }
    }
    __align__(16) __nv_bfloat162 o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      o[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
      float2 b = __bfloat1622float2(o[i]);
      f[2 * i] = b.x;
      f[2 * i + 1] = b.y;
    }
    *reinterpret_cast<uint4*>(residual + (size_t)r * H + v * 8) = *reinterpret_cast<const uint4*>(o);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      rowbuf[(v - v_lo) * 8 + i] = f[i];
      ss += f[i] * f[i];
    }
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int i = 0; i < (blockDim.x >> 5); ++i) t += red[i];
    part_ss = t;
  }
  cluster.sync();                                                  // every block's partial sum is published
  float tot = 0.f;
  for (int q = 0; q < parts; ++q) tot += *cluster.map_shared_rank(&part_ss, q);   // fixed order: reproducible
  cluster.sync();                                                  // nobody leaves while its sum may still be read
  const float rstd = rsqrtf(tot / (float)H + eps);
  const int grow = my_rank * rows + r;
  for (int v = v_lo + threadIdx.x; v < v_hi; v += blockDim.x) {
    uint4 wraw = *reinterpret_cast<const uint4*>(w + v * 8);
    const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&wraw);
    __align__(16) __nv_bfloat162 o[4];
    float yv[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 ww = __bfloat1622float2(wp[i]);
      o[i] = __floats2bfloat162_rn(rowbuf[(v - v_lo) * 8 + 2 * i] * rstd * ww.x,
                                   rowbuf[(v - v_lo) * 8 + 2 * i + 1] * rstd * ww.y);
      float2 b = __bfloat1622float2(o[i]);
      yv[2 * i] = b.x;
      yv[2 * i + 1] = b.y;
    }
    if (y != nullptr) *reinterpret_cast<uint4*>(y + (size_t)r * H + v * 8) = *reinterpret_cast<const uint4*>(o);
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(yv[i]));
#pragma unroll
    for (int o2 = 8; o2 > 0; o2 >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o2));
    const float sc = fmaxf(amax, 1e-4f) * (1.0f / 448.0f);
    const float inv = 1.0f / sc;
    __align__(8) uint16_t q[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) q[i] = to_e4m3x2(yv[2 * i] * inv, yv[2 * i + 1] * inv);
    const uint2 qv = *reinterpret_cast<const uint2*>(q);
    if (loc_q != nullptr) {
      *reinterpret_cast<uint2*>(loc_q + (size_t)r * H + v * 8) = qv;
      if ((threadIdx.x & 15) == 0) loc_s[(size_t)(v / 16) * loc_s_stride + r] = sc;
    }
    if (push && mc_q != nullptr) {
      // NVLS: one multicast store reaches every rank's gather buffer (this rank's own copy included)
      multimem_st_b64(mc_q + (size_t)grow * H + v * 8, qv);
      if ((threadIdx.x & 15) == 0) multimem_st_b32(mc_s + (size_t)(v / 16) * ag_s_stride + grow, __float_as_uint(sc));
    } else if (push) {
      for (int d = 0; d < world; ++d) {   // own copy first, then peers in ring order
        const int dst = (my_rank + d) % world;
        *reinterpret_cast<uint2*>(reinterpret_cast<uint8_t*>(ag_q.p[dst]) + (size_t)grow * H + v * 8) = qv;
        if ((threadIdx.x & 15) == 0)
          reinterpret_cast<float*>(ag_s.p[dst])[(size_t)(v / 16) * ag_s_stride + grow] = sc;
      }
    }
  }
  if (push) cta_done_signal(counter, flags, ready_index + my_rank, world, epoch);
}

// ---------------------------------------------------------------------------------------------
// Expert-parallel dispatch, step 1: counts of this rank's (token, k) pairs per global expert, pushed to
// every rank's count matrix cnt[src = my_rank][E]; also clears this rank's return-address table.
__global__ void __launch_bounds__(1024)
ep_count_push_kernel(const int* __restrict__ topk_idx, int n_pairs, int E, Peers cnt, int my_rank, int world, Peers flags,
                     int ready_index, Epoch epoch_e, int2* __restrict__ row_info, int row_cap, int* __restrict__ mc_cnt) {
  bg::pdl_prologue((BG_FILE_TAG << 16) | __LINE__);
  const uint32_t epoch = epoch_e.get();
  __shared__ int c[kMaxExperts];
  for (int e = threadIdx.x; e < E; e += blockDim.x) c[e] = 0;
  for (int i = threadIdx.x; i < row_cap; i += blockDim.x) row_info[i] = make_int2(-1, -1);
  __syncthreads();
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
    const int e = topk_idx[i];
    if (e >= 0 && e < E) atomicAdd(&c[e], 1);
  }
  __syncthreads();
  if (mc_cnt != nullptr) {               // NVLS: one multicast store per count instead of one per rank
    for (int e = threadIdx.x; e < E; e += blockDim.x)
      multimem_st_b32(mc_cnt + (size_t)my_rank * E + e, (uint32_t)c[e]);
  } else {
    for (int d = 0; d < world; ++d) {
      int* dst = reinterpret_cast<int*>(cnt.p[(my_rank + d) % world]) + (size_t)my_rank * E;
      for (int e = threadIdx.x; e < E; e += blockDim.x) dst[e] = c[e];
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    signal_all(flags, ready_index + my_rank, world, epoch);
  }
}

// Step 2 (one block): wait for every rank's counts, then derive
//   row_base[e]   first row, in the receive buffer of e's owner, for this rank's tokens of expert e
//   offsets[El+1] segment offsets (128-aligned) of this rank's own receive buffer
//   offsets[El+1 .. 2El+1)  real row count of each local expert's segment
//   cursor[e] = 0
__global__ void __launch_bounds__(1024)
ep_layout_kernel(const int* __restrict__ cnt, const uint32_t* __restrict__ cnt_ready, Epoch epoch_e, int E, int world,
                 int my_rank, int align, int* __restrict__ row_base, int* __restrict__ offsets,
                 int* __restrict__ cursor, int* __restrict__ total_rows, int* status) {
  bg::pdl_prologue((BG_FILE_TAG << 16) | __LINE__);
  __shared__ int tot[kMaxExperts];
  __shared__ int mine[kMaxExperts];
  __shared__ int seg[kMaxExperts];
  __shared__ int ok_s;
  const uint32_t epoch = epoch_e.get();
  if (threadIdx.x == 0) {
    int ok = 1;
    for (int s = 0; s < world; ++s)
      if (!wait_flag_ge(cnt_ready + s, epoch, status)) ok = 0;
    if (!ok && status != nullptr) atomicMax(status, (int)kTimeoutPeer);
    ok_s = ok;
  }
  __syncthreads();
  const int El = E / world;
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int t = 0, before = 0;
    for (int s = 0; s < world; ++s) {
      const int v = cnt[(size_t)s * E + e];
      if (s < my_rank) before += v;
      t += v;
    }
    tot[e] = t;
    mine[e] = before;
    cursor[e] = 0;
  }
  __syncthreads();
  if (threadIdx.x < world) {   // one thread per destination rank: serial scan over its El experts
    const int d = threadIdx.x;
    int run = 0;
    for (int j = 0; j < El; ++j) {
      const int e = d * El + j;
      seg[e] = run;
      if (d == my_rank) {
        offsets[j] = run;
        offsets[El + 1 + j] = tot[e];      // rows really present in the segment (the rest is alignment padding)
      }
      run += ((tot[e] + align - 1) / align) * align;
    }
    if (d == my_rank) {
      offsets[El] = run;
      *total_rows = run;
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) row_base[e] = seg[e] + mine[e];
}

// Step 3: one block per local token.  Quantise the token once (1x128 e4m3), then store it into the
// receive buffer of every routed expert's owner at its expert-grouped row, with its scales and the
// return address (owner rank, token * K + k) for the combine.
__global__ void __launch_bounds__(256)
ep_dispatch_send_kernel(const __nv_bfloat16* __restrict__ hidden, int ldh, const int* __restrict__ topk_idx, int K,
                        int E, int H, const int* __restrict__ row_base, int* __restrict__ cursor, Peers recv_q,
                        Peers recv_s, int recv_s_stride, Peers recv_info, int recv_cap, int* __restrict__ sent_row,
                        int my_rank, int world, Peers flags, int ready_index, Epoch epoch_e, unsigned int* counter,
                        int* status) {
  bg::pdl_prologue((BG_FILE_TAG << 16) | __LINE__);
  const uint32_t epoch = epoch_e.get();
  __shared__ int dest_rank[16], dest_row[16];
  const int t = blockIdx.x;
  const int El = E / world;
  if (threadIdx.x < K) {
    const int e = topk_idx[(size_t)t * K + threadIdx.x];
    int dr = -1, row = -1;
    if (e >= 0 && e < E) {
      dr = e / El;
      row = row_base[e] + atomicAdd(&cursor[e], 1);
      if (row >= recv_cap) {
        if (status != nullptr) atomicMax(status, (int)kOverflow);
        dr = -1;
      }
    }
    dest_rank[threadIdx.x] = dr;
    dest_row[threadIdx.x] = row;
    sent_row[(size_t)t * K + threadIdx.x] = row;
    if (dr >= 0) reinterpret_cast<int2*>(recv_info.p[dr])[row] = make_int2(my_rank, t * K + threadIdx.x);
  }
  __syncthreads();
  for (int v = threadIdx.x; v < H / 8; v += blockDim.x) {
    uint4 raw = *reinterpret_cast<const uint4*>(hidden + (size_t)t * ldh + v * 8);
    const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&raw);
    float f[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 a = __bfloat1622float2(xp[i]);
      f[2 * i] = a.x;
      f[2 * i + 1] = a.y;
    }
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(f[i]));
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float sc = fmaxf(amax, 1e-4f) * (1.0f / 448.0f);
    const float inv = 1.0f / sc;
    __align__(8) uint16_t q[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) q[i] = to_e4m3x2(f[2 * i] * inv, f[2 * i + 1] * inv);
    const uint2 qv = *reinterpret_cast<const uint2*>(q);
    for (int k = 0; k < K; ++k) {
      const int dr = dest_rank[k];
      if (dr < 0) continue;
      const int row = dest_row[k];
      *reinterpret_cast<uint2*>(reinterpret_cast<uint8_t*>(recv_q.p[dr]) + (size_t)row * H + v * 8) = qv;
      if ((threadIdx.x & 15) == 0)
        reinterpret_cast<float*>(recv_s.p[dr])[(size_t)(v / 16) * recv_s_stride + row] = sc;
    }
  }
  cta_done_signal(counter, flags, ready_index + my_rank, world, epoch);
}

__global__ void wait_flags_kernel(const uint32_t* flags, int n, Epoch epoch_e, int* status, uint64_t budget_ns) {
  bg::pdl_prologue((BG_FILE_TAG << 16) | __LINE__);
  const uint32_t epoch = epoch_e.get();
  if (threadIdx.x < n) {
    if (!wait_flag_ge(flags + threadIdx.x, epoch, status, budget_ns) && status != nullptr)
      atomicMax(status, (int)kTimeoutPeer);
  }
}

// All-to-all of equal slices over peer memory.  A slice is `n_chunks` chunks of `chunk_vec` 16-byte vectors; chunk b
// bound for rank d is read at src + d * src_d + b * src_b and stored into rank d's receive buffer at
// my_rank * dst_r + b * dst_b (all in vectors), so either side of the exchange can be laid out [rank, chunk] or
// [chunk, rank] and no transposing copy is needed around it.  When the last CTA is done every rank's flag
// (index + my_rank) is raised.  grid = (blocks per slice, world); blockIdx.y walks the destinations in ring order
// starting with this rank.
__global__ void __launch_bounds__(256)
a2a_push_kernel(const uint4* __restrict__ src, Peers dst, size_t n_chunks, size_t chunk_vec, size_t src_d, size_t src_b,
                size_t dst_r, size_t dst_b, int my_rank, int world, Peers flags, int ready_index, Epoch epoch_e,
                unsigned int* counter) {
  bg::pdl_prologue((BG_FILE_TAG << 16) | __LINE__);
  const uint32_t epoch = epoch_e.get();
  const int d = (my_rank + blockIdx.y) % world;
  const uint4* s = src + (size_t)d * src_d;
  uint4* o = reinterpret_cast<uint4*>(dst.p[d]) + (size_t)my_rank * dst_r;
  const size_t total = n_chunks * chunk_vec;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t b = i / chunk_vec, within = i - b * chunk_vec;
    o[b * dst_b + within] = s[b * src_b + within];
  }
  // last-CTA-out over the whole 2-D grid
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const unsigned int prev = atomicAdd(counter, 1u);
    if (prev == gridDim.x * gridDim.y - 1) {
      *counter = 0u;
      __threadfence_system();
      signal_all(flags, ready_index + my_rank, world, epoch);
    }
  }
}

// Streamed-expert fan-out: the rank that brought a weight frame onto its GPU (host -> device copy into its ring
// slot) writes the frame into the same slot of every member of the replica group, so the frame crosses PCIe once
// per group and NVLink once per member.  members: bit r set = rank r receives a copy.  With a multicast address
// of the slot (NVLS) one store per 16 bytes reaches every rank; without it the kernel stores to each member in turn.
// The last CTA raises flag (index + my_rank) on every member: the frame is complete in its slot.
__global__ void __launch_bounds__(256)
fanout_push_kernel(const uint4* __restrict__ src, Peers dst, size_t n_vec, unsigned int members, uint4* __restrict__ mc_dst,
                   int my_rank, int world, Peers flags, int ready_index, Epoch epoch_e, unsigned int* counter) {
  bg::pdl_prologue((BG_FILE_TAG << 16) | __LINE__);
  const uint32_t epoch = epoch_e.get();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += (size_t)gridDim.x * blockDim.x) {
    const uint4 v = src[i];
    if (mc_dst != nullptr) {
      asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_dst + i),
                   "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)),
                   "f"(__uint_as_float(v.w))
                   : "memory");
    } else {
      for (int d = 1; d < world; ++d) {            // ring order, the owner's own slot already holds the frame
        const int r = (my_rank + d) % world;
        if (members & (1u << r)) reinterpret_cast<uint4*>(dst.p[r])[i] = v;
      }
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const unsigned int prev = atomicAdd(counter, 1u);
    if (prev == gridDim.x - 1) {
      *counter = 0u;
      __threadfence_system();
      for (int r = 0; r < world; ++r)
        if (members & (1u << r)) st_relaxed_sys(reinterpret_cast<uint32_t*>(flags.p[r]) + ready_index + my_rank, epoch);
    }
  }
}

__global__ void bump_epoch_kernel(uint32_t* base, uint32_t n) {
  bg::pdl_prologue((BG_FILE_TAG << 16) | __LINE__);
  if (threadIdx.x == 0) *base += n;
}

__global__ void signal_kernel(Peers flags, int index, int world, Epoch epoch_e) {
  bg::pdl_prologue((BG_FILE_TAG << 16) | __LINE__);
  const uint32_t epoch = epoch_e.get();
  if (threadIdx.x == 0) {
    __threadfence_system();
    signal_all(flags, index, world, epoch);
  }
}

}  // namespace comm
}  // namespace bg

extern "C" {

using bg::comm::Peers;

static Peers to_peers(void* const* arr, int world) {
  Peers p;
  for (int i = 0; i < bg::comm::kMaxWorld; ++i) p.p[i] = (arr != nullptr && i < world) ? arr[i] : nullptr;
  return p;
}

// Multicast (NVLS) addresses of the broadcast regions of the symmetric heap on the calling thread's device; null
// = not installed: the kernels then store to each peer in turn.
int bg_comm_set_multicast(void* ag_q, void* ag_s, void* cnt) {
  bg::comm::Multicast& m = bg::comm::multicast();
  m.ag_q = ag_q;
  m.ag_s = ag_s;
  m.cnt = cnt;
  return 0;
}

int bg_sp_norm_quant_push(const void* partials, int n_src, const uint32_t* src_ready, uint32_t wait_epoch,
                          const uint32_t* epoch_base,
                          void* residual, int has_residual, const void* w, void* y, void* loc_q, float* loc_s,
                          int loc_s_stride, void* const* ag_q, void* const* ag_s, int ag_s_stride, int push, int rows,
                          int H, float eps, int my_rank, int world, void* const* flags, int ready_index, uint32_t epoch,
                          unsigned int* counter, int* status, cudaStream_t stream) {
  using namespace bg::comm;
  if (rows <= 0) return 0;
  if (H % 128 != 0 || world > kMaxWorld) return -1;
  // few rows (decode): four blocks per row in one cluster; many rows (prefill): one block per row as before
  const int groups = H / 128;
  int parts = 1;
  if (rows <= 1024) parts = groups % 4 == 0 ? 4 : (groups % 2 == 0 ? 2 : 1);
  bg::launch_pdl_cluster(sp_norm_quant_push_kernel, dim3(rows, parts), dim3(256), dim3(1, parts, 1),
                         (size_t)H * sizeof(float), stream, 
      reinterpret_cast<const __nv_bfloat16*>(partials), n_src, src_ready, Epoch{wait_epoch, epoch_base},
      reinterpret_cast<__nv_bfloat16*>(residual), reinterpret_cast<const __nv_bfloat16*>(w),
      reinterpret_cast<__nv_bfloat16*>(y), reinterpret_cast<uint8_t*>(loc_q), loc_s, loc_s_stride, to_peers(ag_q, world),
      to_peers(ag_s, world), ag_s_stride, push, rows, H, eps, my_rank, world, to_peers(flags, world), ready_index,
      Epoch{epoch, epoch_base}, counter, status, has_residual, reinterpret_cast<uint8_t*>(multicast().ag_q),
      reinterpret_cast<float*>(multicast().ag_s));
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int bg_ep_count_push(const int* topk_idx, int n_pairs, int E, void* const* cnt, int my_rank, int world,
                     void* const* flags, int ready_index, uint32_t epoch, const uint32_t* epoch_base, void* row_info,
                     int row_cap, cudaStream_t stream) {
  using namespace bg::comm;
  if (E > kMaxExperts || world > kMaxWorld) return -1;
  bg::launch_pdl(ep_count_push_kernel, dim3(1), dim3(1024), 0, stream, topk_idx, n_pairs, E, to_peers(cnt, world), my_rank, world,
                                               to_peers(flags, world), ready_index, Epoch{epoch, epoch_base},
                                               reinterpret_cast<int2*>(row_info), row_cap,
                                               reinterpret_cast<int*>(multicast().cnt));
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int bg_ep_layout(const int* cnt, const uint32_t* cnt_ready, uint32_t epoch, const uint32_t* epoch_base, int E, int world,
                 int my_rank, int align,
                 int* row_base, int* offsets, int* cursor, int* total_rows, int* status, cudaStream_t stream) {
  using namespace bg::comm;
  if (E > kMaxExperts || E % world != 0) return -1;
  bg::launch_pdl(ep_layout_kernel, dim3(1), dim3(1024), 0, stream, cnt, cnt_ready, Epoch{epoch, epoch_base}, E, world, my_rank, align, row_base,
                                           offsets, cursor,
                                           total_rows, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int bg_ep_dispatch_send(const void* hidden, int ldh, const int* topk_idx, int T, int K, int E, int H,
                        const int* row_base, int* cursor, void* const* recv_q, void* const* recv_s, int recv_s_stride,
                        void* const* recv_info, int recv_cap, int* sent_row, int my_rank, int world, void* const* flags,
                        int ready_index, uint32_t epoch, const uint32_t* epoch_base, unsigned int* counter, int* status,
                        cudaStream_t stream) {
  using namespace bg::comm;
  if (K > 16 || H % 128 != 0) return -1;
  if (T <= 0) {  // nothing to send, but peers still wait for this rank's flag
    bg::launch_pdl(signal_kernel, dim3(1), dim3(32), 0, stream, to_peers(flags, world), ready_index + my_rank, world, Epoch{epoch, epoch_base});
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
  }
  bg::launch_pdl(ep_dispatch_send_kernel, dim3(T), dim3(256), 0, stream, reinterpret_cast<const __nv_bfloat16*>(hidden), ldh, topk_idx, K, E, H,
                                                 row_base, cursor, to_peers(recv_q, world), to_peers(recv_s, world),
                                                 recv_s_stride, to_peers(recv_info, world), recv_cap, sent_row, my_rank,
                                                 world, to_peers(flags, world), ready_index, Epoch{epoch, epoch_base}, counter,
                                                 status);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// Fan a frame of `bytes` (multiple of 16) out from `src` (this rank's slot) to dst[r] for every rank r in `members`;
// mc_dst: multicast address of the slot or null.
int bg_fanout_push(const void* src, void* const* dst, unsigned long long bytes, unsigned int members, void* mc_dst,
                   int my_rank, int world, void* const* flags, int ready_index, uint32_t epoch,
                   const uint32_t* epoch_base, unsigned int* counter, int num_sms, cudaStream_t stream) {
  if (bytes == 0) return 0;
  if (bytes % 16 != 0 || world < 1 || world > 8) return -1;
  const size_t vec = bytes / 16;
  int bx = (int)((vec + 255) / 256);
  if (bx > 2 * num_sms) bx = 2 * num_sms;
  bg::launch_pdl(bg::comm::fanout_push_kernel, dim3(bx), dim3(256), 0, stream, reinterpret_cast<const uint4*>(src),
                 to_peers(dst, world), vec, members, reinterpret_cast<uint4*>(mc_dst), my_rank, world,
                 to_peers(flags, world), ready_index, bg::comm::Epoch{epoch, epoch_base}, counter);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// Chunked form (see a2a_push_kernel): sizes and strides in bytes, multiples of 16.
int bg_a2a_push_chunks(const void* src, void* const* dst, unsigned long long n_chunks, unsigned long long chunk_bytes,
                       unsigned long long src_d, unsigned long long src_b, unsigned long long dst_r,
                       unsigned long long dst_b, int my_rank, int world, void* const* flags, int ready_index,
                       uint32_t epoch, const uint32_t* epoch_base, unsigned int* counter, cudaStream_t stream) {
  if (n_chunks == 0 || chunk_bytes == 0) return 0;
  if ((chunk_bytes | src_d | src_b | dst_r | dst_b) % 16 != 0 || world < 1 || world > 8) return -1;
  const size_t vec = n_chunks * (chunk_bytes / 16);
  int bx = (int)((vec + 255) / 256);
  if (bx > 64) bx = 64;
  dim3 grid(bx, world);
  bg::launch_pdl(bg::comm::a2a_push_kernel, dim3(grid), dim3(256), 0, stream, reinterpret_cast<const uint4*>(src), to_peers(dst, world), n_chunks,
                                                      chunk_bytes / 16, src_d / 16, src_b / 16, dst_r / 16, dst_b / 16,
                                                      my_rank, world, to_peers(flags, world), ready_index,
                                                      bg::comm::Epoch{epoch, epoch_base}, counter);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// src: [world, slice_bytes] (slice_bytes a multiple of 16); dst[r]: rank r's receive buffer [world, slice_bytes].
int bg_a2a_push(const void* src, void* const* dst, unsigned long long slice_bytes, int my_rank, int world,
                void* const* flags, int ready_index, uint32_t epoch, const uint32_t* epoch_base, unsigned int* counter,
                cudaStream_t stream) {
  return bg_a2a_push_chunks(src, dst, 1, slice_bytes, slice_bytes, 0, slice_bytes, 0, my_rank, world, flags, ready_index,
                            epoch, epoch_base, counter, stream);
}

int bg_wait_flags(const uint32_t* flags, int n, uint32_t epoch, const uint32_t* epoch_base, int* status,
                  cudaStream_t stream) {
  bg::launch_pdl(bg::comm::wait_flags_kernel, dim3(1), dim3(32), 0, stream, flags, n, bg::comm::Epoch{epoch, epoch_base}, status,
                                                    bg::kFlagBudgetNs);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// Same wait with an explicit budget in milliseconds (failure-detection tests make a wait run out on a flag
// that nothing raises and read the status word; the context stays usable).
int bg_wait_flags_budget(const uint32_t* flags, int n, uint32_t epoch, const uint32_t* epoch_base, int budget_ms,
                         int* status, cudaStream_t stream) {
  if (n < 0 || n > 32 || budget_ms < 0) return -1;
  bg::launch_pdl(bg::comm::wait_flags_kernel, dim3(1), dim3(32), 0, stream, flags, n, bg::comm::Epoch{epoch, epoch_base}, status,
                                                    (uint64_t)budget_ms * 1000000ull);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int bg_signal(void* const* flags, int index, int world, uint32_t epoch, const uint32_t* epoch_base, cudaStream_t stream) {
  bg::launch_pdl(bg::comm::signal_kernel, dim3(1), dim3(32), 0, stream, to_peers(flags, world), index, world, bg::comm::Epoch{epoch, epoch_base});
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int bg_bump_epoch(uint32_t* base, uint32_t n, cudaStream_t stream) {
  bg::launch_pdl(bg::comm::bump_epoch_kernel, dim3(1), dim3(32), 0, stream, base, n);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

}  // extern "C"

BG_TRACE_SETTER(fused_comm)
