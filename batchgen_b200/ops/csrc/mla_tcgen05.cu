// C entry points of the tcgen05 paged-MLA kernels (kernel bodies: mla_tcgen05.cuh).
#define BG_FILE_TAG 8      // kernel-trace ids of this file are (tag << 16) | line
#include "mla_tcgen05.cuh"

extern "C" {

// Paged absorbed MLA.  q_abs: [R*H, 512] bf16 contiguous; q_pe: [R*H, 64] bf16 with row stride
// `qpe_stride` elements; cache: [n_pages*64, 576] bf16; work: device array of bg::mla::Work
// (8 ints each); ncol: 16, 32 or 64 = n_q * heads_per_group columns per CTA.  Split partials go to
// part_o / part_ml and are merged by bg_mla_merge.
// q_abs rows may be wider than the 512 latent columns (``qabs_stride`` elements between (row, head) entries, a
// multiple of 8): the latent and rope parts of a query can then be two views of one [rows, heads, 576] buffer.
int bg_mla_attention_strided(const void* q_abs, long long qabs_stride, const void* q_pe, long long qpe_stride,
                             long long q_rows, const void* cache, long long cache_rows, const int* work, int n_work,
                             const int* block_table, int bt_stride, const int* seqlens, void* out, float* part_o,
                             float* part_ml, int H, int heads_per_group, int ncol, float scale, int* status,
                             cudaStream_t stream) {
  using namespace bg::mla;
  if (n_work <= 0) return 0;
  if ((ncol != 16 && ncol != 32 && ncol != 64) || heads_per_group <= 0 || ncol % heads_per_group != 0 || heads_per_group % 8 != 0 ||
      H % heads_per_group != 0 || (qpe_stride * 2) % 16 != 0 || qabs_stride < kLatent || (qabs_stride * 2) % 16 != 0)
    return -1;
  CUtensorMap tkv, tq, tqpe;
  if (make_map(&tkv, cache, cache_rows, kRow, kRow * 2, kPage) != 0) return -10;
  if (make_map(&tq, q_abs, q_rows, kLatent, qabs_stride * 2, heads_per_group) != 0) return -11;
  if (make_map(&tqpe, q_pe, q_rows, kRope, qpe_stride * 2, heads_per_group) != 0) return -12;
  Params p;
  p.work = reinterpret_cast<const Work*>(work);
  p.block_table = block_table; p.bt_stride = bt_stride; p.seqlens = seqlens;
  p.out = reinterpret_cast<__nv_bfloat16*>(out); p.part_o = part_o; p.part_ml = part_ml;
  p.H = H; p.heads_per_group = heads_per_group; p.scale_log2 = scale * 1.4426950408889634f; p.status = status;
  if (ncol == 16) return launch<16>(tkv, tq, tqpe, p, n_work, stream);
  if (ncol == 32) return launch<32>(tkv, tq, tqpe, p, n_work, stream);
  return launch<64>(tkv, tq, tqpe, p, n_work, stream);
}

int bg_mla_attention(const void* q_abs, const void* q_pe, long long qpe_stride, long long q_rows, const void* cache,
                     long long cache_rows, const int* work, int n_work, const int* block_table, int bt_stride,
                     const int* seqlens, void* out, float* part_o, float* part_ml, int H, int heads_per_group,
                     int ncol, float scale, int* status, cudaStream_t stream) {
  return bg_mla_attention_strided(q_abs, bg::mla::kLatent, q_pe, qpe_stride, q_rows, cache, cache_rows, work, n_work,
                                  block_table, bt_stride, seqlens, out, part_o, part_ml, H, heads_per_group, ncol, scale,
                                  status, stream);
}

int bg_mla_merge(const float* part_o, const float* part_ml, const int* items, int n_items, void* out, int ncol, int H,
                 int heads_per_group, cudaStream_t stream) {
  using namespace bg::mla;
  if (n_items <= 0) return 0;
  mla_merge_kernel<<<dim3(n_items, ncol), 128, 0, stream>>>(part_o, part_ml, items, reinterpret_cast<__nv_bfloat16*>(out), ncol, H,
                                                heads_per_group);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

}  // extern "C"

BG_TRACE_SETTER(mla_tcgen05)
