// Shared device helpers for the sm_100a kernels: mbarrier, TMA, tcgen05 (TMEM) wrappers.
//
// Every wait in here is bounded: a spin that exceeds its iteration budget raises the CTA's
// abort flag and returns false, so that a broken pipeline ends with an error status in global
// memory instead of a hung GPU.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace bg {

constexpr uint64_t kWaitBudgetNs = 30ull * 1000000000ull;   // intra-CTA pipeline waits (wall time)
constexpr uint64_t kFlagBudgetNs = 10ull * 1000000000ull;   // waits on a flag that a peer GPU raises

enum Status : int {
  kOk = 0,
  kTimeoutProducer = 1,
  kTimeoutMma = 2,
  kTimeoutEpilogue = 3,
  kTimeoutPeer = 4,
  kBadArgument = 5,
  kOverflow = 6,
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n"
      ".reg .pred P;\n"
      "elect.sync _|P, 0xffffffff;\n"
      "selp.u32 %0, 1, 0, P;\n"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait.  Returns false (and raises *abort_flag) when the budget runs out or another role
// already aborted.  The budget is wall time (kWaitBudgetNs), checked every 64K polls: a role inside a
// CTA may legitimately sit here for as long as its producer waits for a peer GPU (kFlagBudgetNs, which is
// shorter), so the limit must not depend on how fast the poll loop spins.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          int why) {
  uint64_t t0 = 0;
  for (uint32_t i = 0;; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 255u) == 255u) {
      if (*abort_flag) return false;
      if ((i & 0xFFFFu) == 0xFFFFu) {
        const uint64_t t = global_timer_ns();
        if (t0 == 0) t0 = t;
        else if (t - t0 > kWaitBudgetNs) break;
      }
    }
  }
  if (*abort_flag == 0) *abort_flag = why;
  return false;
}

// ---------------------------------------------------------------- TMA (plain per-CTA tile loads only)
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0,
                                            int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0,
                                            int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// ---------------------------------------------------------------- tcgen05 / TMEM
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_holder, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_holder)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// Arrive on an mbarrier once all tcgen05.mma issued so far by this thread have completed.
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// Shared-memory matrix descriptor for a K-major operand tile whose rows are exactly one
// 128-byte swizzle atom wide (rows * 128 B, 8-row groups 1024 B apart), as written by a TMA
// load with CU_TENSOR_MAP_SWIZZLE_128B.
__device__ __forceinline__ uint64_t make_smem_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);  // start address, 16-byte units
  d |= static_cast<uint64_t>(0) << 16;                      // leading byte offset (unused here)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;              // stride byte offset between 8-row groups
  d |= static_cast<uint64_t>(1) << 46;                      // descriptor version (sm_100)
  d |= static_cast<uint64_t>(2) << 61;                      // layout: 128-byte swizzle
  return d;
}

// Instruction descriptor: fp32 accumulate, both operands K-major, M x N tile.
// a_fmt/b_fmt: kind::f8f6f4 -> 0 = e4m3; kind::f16 -> 1 = bf16.
__host__ __device__ constexpr uint32_t make_idesc(int M, int N, int a_fmt, int b_fmt) {
  return (1u << 4) | (static_cast<uint32_t>(a_fmt) << 7) | (static_cast<uint32_t>(b_fmt) << 10) |
         (static_cast<uint32_t>(N >> 3) << 17) | (static_cast<uint32_t>(M >> 4) << 24);
}

__device__ __forceinline__ void mma_f8f6f4(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// 32 lanes x 32 columns of fp32: thread i of the warp receives lane (base+i), columns c..c+31.
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
        "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
        "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---------------------------------------------------------------- cross-GPU flags (peer memory over NVLink)
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Strong relaxed store: after one __threadfence_system() a run of these publishes to every peer without
// paying a release fence per store.
__device__ __forceinline__ void st_relaxed_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Wait until *flag >= value (flags are monotonically increasing epochs).  Bounded by wall time
// (kFlagBudgetNs: ranks can be seconds apart after loading weights or capturing graphs); and once any
// kernel has raised the status word (a peer is late or gone) later waits give up at once, so a
// broken step drains in milliseconds instead of one timeout per kernel.
__device__ __forceinline__ bool wait_flag_ge(const uint32_t* flag, uint32_t value, const int* status = nullptr,
                                             uint64_t budget_ns = kFlagBudgetNs) {
  uint64_t t0 = 0;
  for (uint32_t i = 0;; ++i) {
    if (static_cast<int32_t>(ld_acquire_sys(flag) - value) >= 0) return true;
    if ((i & 63u) == 0u) {
      if (status != nullptr && *reinterpret_cast<const volatile int*>(status) != 0) return false;
      if ((i & 1023u) == 0u) {
        const uint64_t t = global_timer_ns();
        if (t0 == 0) t0 = t;
        else if (t - t0 > budget_ns) return false;
      }
    }
    __nanosleep(200);
  }
}
__device__ __forceinline__ void fence_proxy_async_global() { asm volatile("fence.proxy.async.global;" ::: "memory"); }

// ---------------------------------------------------------------- host: per-device kernel attributes
// The dynamic shared-memory limit of a kernel is a per-device (per-context) attribute, so "already set" is
// tracked per device: a process that drives several GPUs sets it once on each.
constexpr int kMaxDevices = 64;
struct DeviceOnce {
  bool done[kMaxDevices] = {};
};
template <typename Kernel>
inline bool ensure_dynamic_smem(Kernel kernel, size_t bytes, DeviceOnce& once) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return false;
  const bool tracked = dev >= 0 && dev < kMaxDevices;
  if (tracked && once.done[dev]) return true;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes) != cudaSuccess)
    return false;
  if (tracked) once.done[dev] = true;
  return true;
}

// ---------------------------------------------------------------- programmatic dependent launch
// Every kernel starts with pdl_prologue(): it lets the next kernel of the stream begin launching (its blocks take
// free SMs and run their own prologue) and then waits until the kernels it depends on have completed and their
// writes are visible.  Without the launch attribute both instructions do nothing.  launch_pdl() sets the attribute,
// so the gap between two kernels of a captured step shrinks from a full launch to the dependency hand-over.
//
// Kernel trace: when a trace buffer is installed (bg_trace_set_<file>, one per translation unit), thread 0 of block
// 0 of every kernel appends (global timer, id) on entry; consecutive entries give each kernel's period inside a
// captured step (duration + the gap to the next kernel), which events around a graph replay cannot show.
#ifndef BG_FILE_TAG
#define BG_FILE_TAG 0
#endif
struct TraceBuf {
  unsigned int n, cap;
  unsigned long long rec[2];      // cap pairs of (time in ns, id) follow
};
static __device__ TraceBuf* g_trace = nullptr;
__device__ __forceinline__ void pdl_prologue(unsigned int id = 0) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) {
    TraceBuf* tb = g_trace;
    if (tb != nullptr) {
      const unsigned int i = atomicAdd(&tb->n, 1u);
      if (i < tb->cap) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        tb->rec[2 * i] = t;
        tb->rec[2 * i + 1] = id;
      }
    }
  }
}
#define BG_TRACE_SETTER(name)                                                                       \
  extern "C" int bg_trace_set_##name(void* p) {                                                     \
    return cudaMemcpyToSymbol(bg::g_trace, &p, sizeof(p)) == cudaSuccess ? 0 : -1;                  \
  }
inline bool pdl_enabled() {
  static const bool on = [] {
    const char* e = getenv("BG_PDL");
    return e != nullptr && e[0] == '1';
  }();
  return on;
}
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Same, with a thread-block cluster of (cx, cy, 1) CTAs.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, dim3 cluster, size_t smem,
                                      cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = cluster.x;
  attr[1].val.clusterDim.y = cluster.y;
  attr[1].val.clusterDim.z = cluster.z;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// ---------------------------------------------------------------- misc math
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float silu(float x) { return x / (1.0f + __expf(-x)); }

// Saturating fp32 -> e4m3 (round to nearest even), one byte.
__device__ __forceinline__ uint8_t to_e4m3(float x) {
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3));
}
__device__ __forceinline__ uint16_t to_e4m3x2(float lo, float hi) {
  return static_cast<uint16_t>(__nv_cvt_float2_to_fp8x2(make_float2(lo, hi), __NV_SATFINITE, __NV_E4M3));
}

}  // namespace bg
