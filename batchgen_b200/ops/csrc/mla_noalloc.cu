// Split-KV MLA decode that allocates nothing: see bg_noalloc.h for who needs it and for its limits.
#include "bg_noalloc.h"
#include "mla_tcgen05.cuh"

namespace bg {
namespace mla {

constexpr int kNoallocMaxWork = BG_NOALLOC_MAX_WORK;
constexpr int kNoallocNcolMax = 32;

struct NoallocScratch {
  float part_o[kNoallocMaxWork][kNoallocNcolMax][kLatent];   // unnormalised partial outputs
  float part_ml[kNoallocMaxWork][kNoallocNcolMax][2];        // running max and row sum of each partial
  Work work[kNoallocMaxWork];                                // one descriptor per CTA
  int items[kNoallocMaxWork][5];                             // merge list
};

// The scratch itself.  In host code this name is only a stand-in for the symbol: the address that
// kernels may use comes from cudaGetSymbolAddress (below), once per device.
static __device__ __align__(256) unsigned char g_noalloc_scratch[sizeof(NoallocScratch)];

static void* g_scratch_dev_ptr[64] = {nullptr};

// Fills the work and merge lists for a decode batch: item (b, g) owns slots (b*groups + g)*splits ...
// It also resets the (running max, row sum) pair of every partial this call owns to (-inf, 0), the value the merge
// skips: the array keeps the previous call's partials, and a CTA that gives up on a bounded wait writes nothing, so
// without the reset the merge would fold stale numbers into a plausible-looking result.
static __global__ void noalloc_fill_lists(NoallocScratch* s, int B, int groups, int splits, int ncol) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const int n_work = B * groups * splits;
  if (i < n_work) {
    float* ml = &s->part_ml[0][0][0] + (size_t)i * ncol * 2;     // pitch of this launch's column variant
    for (int c = 0; c < ncol; ++c) {
      ml[2 * c] = -INFINITY;
      ml[2 * c + 1] = 0.f;
    }
    const int item = i / splits;
    Work w;
    w.q_row = item / groups;
    w.n_q = 1;
    w.seq = item / groups;
    w.ctx_base = -1;
    w.split = i % splits;
    w.n_splits = splits;
    w.head_group = item % groups;
    w.out_slot = i;
    s->work[i] = w;
  }
  if (i < B * groups) {
    s->items[i][0] = i / groups;
    s->items[i][1] = 1;
    s->items[i][2] = i % groups;
    s->items[i][3] = i * splits;
    s->items[i][4] = splits;
  }
}

}  // namespace mla
}  // namespace bg

extern "C" {

const char* bg_noalloc_strerror(int code) {
  switch (code) {
    case 0: return "ok";
    case BG_NOALLOC_E_TOO_LARGE:
      return "batch * head groups * splits exceeds BG_NOALLOC_MAX_WORK (256): the built-in scratch is too small";
    case BG_NOALLOC_E_BAD_SHAPE:
      return "unsupported shape: heads must be a multiple of 8, num_splits >= 2, q_pe row stride a multiple of 8";
    case BG_NOALLOC_E_SETUP: return "could not resolve the scratch symbol or set the kernel attribute on this device";
    default: return "kernel launch failed";
  }
}

int bg_mla_decode_split_noalloc(const void* q_abs, const void* q_pe, long long qpe_stride, int B, int H,
                                const void* cache, long long cache_rows, const int* block_table, int bt_stride,
                                const int* seqlens, void* out, int num_splits, float scale, int* status,
                                cudaStream_t stream) {
  using namespace bg::mla;
  if (B <= 0) return 0;
  if (H <= 0 || H % 8 != 0 || num_splits < 2 || (qpe_stride * 2) % 16 != 0) return BG_NOALLOC_E_BAD_SHAPE;
  const int hpg = (H % 32 == 0) ? 32 : (H % 16 == 0 ? 16 : 8);
  const int ncol = (hpg == 32) ? 32 : 16;
  const int groups = H / hpg;
  const long long n_work = (long long)B * groups * num_splits;
  if (n_work > kNoallocMaxWork) return BG_NOALLOC_E_TOO_LARGE;

  // ---- once per device: the device address of the scratch array
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return BG_NOALLOC_E_SETUP;
  if (g_scratch_dev_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_noalloc_scratch) != cudaSuccess || ptr == nullptr) return BG_NOALLOC_E_SETUP;
    // both column variants get their shared-memory limit now, so that no later call on this device (which may run
    // inside a stream capture) has an attribute to set or a module to load
    if (!prepare_device<16>() || !prepare_device<32>()) return BG_NOALLOC_E_SETUP;
    g_scratch_dev_ptr[dev] = ptr;
  }
  NoallocScratch* s = reinterpret_cast<NoallocScratch*>(g_scratch_dev_ptr[dev]);

  CUtensorMap tkv, tq, tqpe;
  if (make_map(&tkv, cache, cache_rows, kRow, kRow * 2, kPage) != 0) return BG_NOALLOC_E_SETUP;
  if (make_map(&tq, q_abs, (long long)B * H, kLatent, kLatent * 2, hpg) != 0) return BG_NOALLOC_E_SETUP;
  if (make_map(&tqpe, q_pe, (long long)B * H, kRope, qpe_stride * 2, hpg) != 0) return BG_NOALLOC_E_SETUP;

  noalloc_fill_lists<<<((int)n_work + 127) / 128, 128, 0, stream>>>(s, B, groups, num_splits, ncol);
  if (cudaGetLastError() != cudaSuccess) return -2;

  Params p;
  p.work = s->work;
  p.block_table = block_table; p.bt_stride = bt_stride; p.seqlens = seqlens;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  // both partial arrays are declared with 32 columns; a 16-column launch uses the same base with its own pitch
  p.part_o = &s->part_o[0][0][0];
  p.part_ml = &s->part_ml[0][0][0];
  p.H = H; p.heads_per_group = hpg; p.scale_log2 = scale * 1.4426950408889634f; p.status = status;
  int rc = (ncol == 16) ? launch<16>(tkv, tq, tqpe, p, (int)n_work, stream) : launch<32>(tkv, tq, tqpe, p, (int)n_work, stream);
  if (rc == -12) return BG_NOALLOC_E_SETUP;
  if (rc != 0) return rc;
  mla_merge_kernel<<<dim3(B * groups, ncol), 128, 0, stream>>>(p.part_o, p.part_ml, &s->items[0][0], p.out, ncol, H, hpg);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

}  // extern "C"
