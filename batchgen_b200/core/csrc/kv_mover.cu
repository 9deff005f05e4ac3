// KV page movers: gather / scatter pages between pinned host memory and the device page pool.
//
// A copy request is a list of (source pointer, destination pointer) pairs, one per page fragment, plus
// the fragment size.  Two engines serve it, both on a private non-blocking stream so that transfers
// overlap compute:
//   * the copy-engine path: one cudaMemcpyAsync per fragment (best for a few large fragments);
//   * the kernel path: page_copy_kernel, one CTA per fragment moving 16 bytes per thread per step
//     through unified virtual addressing — pinned host pointers are valid device pointers, so one
//     launch moves hundreds of small fragments (the per-layer rows of decode appends) either way.
// submit() returns a task id; done()/wait() poll or block on the task's event (KVAsyncTask in the
// reference).  Pointer tables are staged in a pinned ring owned by the mover and every ring entry owns its
// dependency event, so submit allocates nothing and creates nothing after construction.  The kernel path
// moves 16 bytes per thread and therefore needs 16-byte aligned fragments; a request with a misaligned
// pointer takes the copy-engine path instead.  The first CUDA error of a request is returned as a negative
// task id (-100 - cudaError) and nothing is recorded for it.
//
// Reference parity: core/KV_Storage/uva_copy_kernel.cu:53-73, core/HtoD_Engine/HtoD_Engine_Kernels.cu:4,
// core/HtoD_Engine/HtoD_Engine.cu:1784-1830 (batched page copy), core/DtoH_Engine/DtoH_Engine.h:42-71,
// core/KV_Storage/host_paged_kv_worker_view.h:386-1400 (async load / offload / append with futures).
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>
#include <vector>

namespace bgcore {

__global__ void __launch_bounds__(256)
page_copy_kernel(const void* const* __restrict__ src, void* const* __restrict__ dst, size_t bytes) {
  const uint4* s = reinterpret_cast<const uint4*>(src[blockIdx.x]);
  uint4* d = reinterpret_cast<uint4*>(dst[blockIdx.x]);
  const size_t n16 = bytes / 16;
  for (size_t i = threadIdx.x; i < n16; i += blockDim.x) d[i] = s[i];
  const size_t tail = n16 * 16;
  const char* sc = reinterpret_cast<const char*>(src[blockIdx.x]);
  char* dc = reinterpret_cast<char*>(dst[blockIdx.x]);
  for (size_t i = tail + threadIdx.x; i < bytes; i += blockDim.x) dc[i] = sc[i];
}

class KVMover {
 public:
  KVMover(int device, int max_fragments, int ring = 8) : device_(device), cap_(max_fragments), ring_(ring) {
    ok_ = cudaSetDevice(device) == cudaSuccess &&
          cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking) == cudaSuccess &&
          cudaHostAlloc(&tables_, sizeof(void*) * 2 * (size_t)cap_ * ring_, cudaHostAllocMapped) == cudaSuccess;
    events_.resize(ring_, nullptr);
    deps_.resize(ring_, nullptr);
    for (int i = 0; ok_ && i < ring_; ++i)
      ok_ = cudaEventCreateWithFlags(&events_[i], cudaEventDisableTiming) == cudaSuccess &&
            cudaEventCreateWithFlags(&deps_[i], cudaEventDisableTiming) == cudaSuccess;
    busy_.assign(ring_, 0);
  }
  ~KVMover() {
    if (stream_) cudaStreamSynchronize(stream_);
    for (auto e : events_)
      if (e) cudaEventDestroy(e);
    for (auto e : deps_)
      if (e) cudaEventDestroy(e);
    if (tables_) cudaFreeHost(tables_);
    if (stream_) cudaStreamDestroy(stream_);
  }
  bool ok() const { return ok_; }

  // Returns a task id >= 0, -1 if the request is too large.  With every ring entry still in flight the call waits
  // for the oldest transfer (counted in ring_waits) and reuses its entry; -2 if that wait fails.
  long submit(const void* const* src, void* const* dst, int n, size_t bytes, int use_kernel, void* after_stream) {
    if (!ok_ || n > cap_) return -1;
    std::lock_guard<std::mutex> lk(mu_);
    int slot = -1;
    for (int i = 0; i < ring_; ++i) {
      int c = (next_ + i) % ring_;
      if (busy_[c] && cudaEventQuery(events_[c]) != cudaErrorNotReady) busy_[c] = 0;
      if (!busy_[c]) { slot = c; break; }
    }
    if (slot < 0) {                  // every entry in flight: the oldest one (transfers run in order) is reused
      slot = next_;
      if (cudaEventSynchronize(events_[slot]) != cudaSuccess) return -2;
      busy_[slot] = 0;
      ring_waits_ += 1;
    }
    next_ = (slot + 1) % ring_;
    cudaError_t err = cudaSetDevice(device_);
    auto note = [&err](cudaError_t e) { if (err == cudaSuccess && e != cudaSuccess) err = e; };
    if (after_stream != nullptr) {   // order the transfer after work already queued on a compute stream
      note(cudaEventRecord(deps_[slot], reinterpret_cast<cudaStream_t>(after_stream)));
      note(cudaStreamWaitEvent(stream_, deps_[slot], 0));
    }
    if (use_kernel) {                // 16 bytes per thread: every fragment must start on a 16-byte boundary
      uintptr_t any = 0;
      for (int i = 0; i < n; ++i) any |= reinterpret_cast<uintptr_t>(src[i]) | reinterpret_cast<uintptr_t>(dst[i]);
      if (any % 16 != 0) {
        use_kernel = 0;
        fallbacks_ += 1;
      }
    }
    if (use_kernel) {
      void** ts = tables_ + (size_t)slot * 2 * cap_;
      void** td = ts + cap_;
      for (int i = 0; i < n; ++i) {
        ts[i] = const_cast<void*>(src[i]);
        td[i] = dst[i];
      }
      void **ds = nullptr, **dd = nullptr;
      note(cudaHostGetDevicePointer(reinterpret_cast<void**>(&ds), ts, 0));
      note(cudaHostGetDevicePointer(reinterpret_cast<void**>(&dd), td, 0));
      if (n > 0 && err == cudaSuccess) {
        page_copy_kernel<<<n, 256, 0, stream_>>>(ds, dd, bytes);
        note(cudaGetLastError());
      }
    } else {
      for (int i = 0; i < n && err == cudaSuccess; ++i)
        note(cudaMemcpyAsync(dst[i], src[i], bytes, cudaMemcpyDefault, stream_));
    }
    if (err == cudaSuccess) note(cudaEventRecord(events_[slot], stream_));
    if (err != cudaSuccess) return -100 - (long)err;     // nothing handed out for a request that was not queued
    busy_[slot] = 1;
    bytes_moved_ += (uint64_t)n * bytes;
    tasks_ += 1;
    return (long)slot;
  }
  int done(long task) {
    if (task < 0 || task >= ring_) return -1;
    return cudaEventQuery(events_[task]) != cudaErrorNotReady ? 1 : 0;
  }
  int wait(long task) {
    if (task < 0 || task >= ring_) return -1;
    return cudaEventSynchronize(events_[task]) == cudaSuccess ? 0 : -2;
  }
  // Make a compute stream wait for a transfer (host->device loads before attention reads the pages).
  int stream_wait(long task, void* stream) {
    if (task < 0 || task >= ring_) return -1;
    return cudaStreamWaitEvent(reinterpret_cast<cudaStream_t>(stream), events_[task], 0) == cudaSuccess ? 0 : -2;
  }
  uint64_t bytes_moved() const { return bytes_moved_; }
  uint64_t tasks() const { return tasks_; }
  uint64_t misaligned_fallbacks() const { return fallbacks_; }

 private:
  int device_, cap_, ring_;
  bool ok_ = false;
  cudaStream_t stream_ = nullptr;
  void** tables_ = nullptr;
  std::vector<cudaEvent_t> events_;   // completion of the task in each ring entry
  std::vector<cudaEvent_t> deps_;     // dependency on a compute stream, one per ring entry
  std::vector<char> busy_;
  int next_ = 0;
  std::mutex mu_;
  uint64_t bytes_moved_ = 0, tasks_ = 0, fallbacks_ = 0, ring_waits_ = 0;
};

}  // namespace bgcore

extern "C" {

void* bgc_mover_create(int device, int max_fragments, int ring) {
  auto* m = new bgcore::KVMover(device, max_fragments, ring);
  if (!m->ok()) {
    delete m;
    return nullptr;
  }
  return m;
}
void bgc_mover_destroy(void* m) { delete static_cast<bgcore::KVMover*>(m); }
long bgc_mover_submit(void* m, const void* const* src, void* const* dst, int n, size_t bytes, int use_kernel,
                      void* after_stream) {
  return static_cast<bgcore::KVMover*>(m)->submit(src, dst, n, bytes, use_kernel, after_stream);
}
int bgc_mover_done(void* m, long task) { return static_cast<bgcore::KVMover*>(m)->done(task); }
int bgc_mover_wait(void* m, long task) { return static_cast<bgcore::KVMover*>(m)->wait(task); }
int bgc_mover_stream_wait(void* m, long task, void* stream) {
  return static_cast<bgcore::KVMover*>(m)->stream_wait(task, stream);
}
unsigned long long bgc_mover_bytes(void* m) { return static_cast<bgcore::KVMover*>(m)->bytes_moved(); }
unsigned long long bgc_mover_misaligned(void* m) { return static_cast<bgcore::KVMover*>(m)->misaligned_fallbacks(); }
int bgc_pin_host(void* p, size_t bytes) { return cudaHostRegister(p, bytes, cudaHostRegisterDefault) == cudaSuccess ? 0 : -1; }
int bgc_unpin_host(void* p) { return cudaHostUnregister(p) == cudaSuccess ? 0 : -1; }

}  // extern "C"
