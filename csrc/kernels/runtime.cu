// Host-side runtime shared by the kernel launchers: tensor-map encoding through
// the driver entry point, the per-device status word that bounded waits write
// to, and cached device properties.
#include "sm100_common.cuh"

#include <cudaTypedefs.h>
#include <atomic>
#include <cstdlib>
#include <mutex>
#include <stdio.h>

namespace rbh {

namespace {
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;
std::once_flag g_encode_once;

constexpr int kMaxDevices = 16;
int* g_status[kMaxDevices] = {nullptr};
int g_sm_count[kMaxDevices] = {0};
std::mutex g_mu;

void load_encode() {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
  if (e == cudaSuccess && qres == cudaDriverEntryPointSuccess) g_encode = (EncodeTiledFn)fn;
}
}  // namespace

int encode_tensor_map(CUtensorMap* out, int dtype, int rank, void* base, const uint64_t* dims,
                      const uint64_t* strides_bytes, const uint32_t* box, int swizzle_128b) {
  return encode_tensor_map_strided(out, dtype, rank, base, dims, strides_bytes, box, nullptr, swizzle_128b);
}

int encode_tensor_map_strided(CUtensorMap* out, int dtype, int rank, void* base, const uint64_t* dims,
                              const uint64_t* strides_bytes, const uint32_t* box, const uint32_t* elem_strides,
                              int swizzle_128b) {
  std::call_once(g_encode_once, load_encode);
  if (!g_encode) return -1;
  // The driver entry point needs a current context on the calling thread.  Threads that have
  // only been handed a device index (autograd worker threads) get the primary context bound by
  // their first runtime call; make sure that has happened.
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    cudaFree(0);
    ctx_bound = true;
  }
  CUtensorMapDataType dt = dtype == DT_F32    ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                           : dtype == DT_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                             : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  cuuint64_t gdims[5];
  cuuint64_t gstrides[5];
  cuuint32_t gbox[5];
  cuuint32_t estr[5];
  for (int i = 0; i < rank; ++i) {
    gdims[i] = dims[i];
    gbox[i] = box[i];
    estr[i] = elem_strides ? elem_strides[i] : 1;
    if (i > 0) gstrides[i - 1] = strides_bytes[i];
  }
  CUresult r = g_encode(out, dt, (cuuint32_t)rank, base, gdims, gstrides, gbox, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE,
                        swizzle_128b ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

int* device_status_word() {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_status[dev]) {
    int* p = nullptr;
    if (cudaMalloc(&p, 256) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, 256);
    g_status[dev] = p;
  }
  return g_status[dev];
}

int read_and_clear_status() {
  int* p = device_status_word();
  if (!p) return -1;
  int v = 0;
  cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost);
  if (v != 0) cudaMemset(p, 0, sizeof(int));
  return v;
}

int* next_sched_slot() {
  static std::atomic<unsigned> counter{0};
  static int* g_sched[kMaxDevices] = {nullptr};
  constexpr int kSlots = 256;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= kMaxDevices) return nullptr;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_sched[dev]) {
      int* p = nullptr;
      if (cudaMalloc(&p, kSlots * 2 * sizeof(int)) != cudaSuccess) return nullptr;
      cudaMemset(p, 0, kSlots * 2 * sizeof(int));
      g_sched[dev] = p;
    }
  }
  return g_sched[dev] + 2 * (counter.fetch_add(1) % kSlots);
}

bool dynamic_tiles() {
  static const bool on = [] {
    const char* e = std::getenv("RB_GEMM_DYNAMIC");
    return !(e && e[0] == '0');
  }();
  return on;
}

int sm_count() {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= kMaxDevices) return 148;
  if (!g_sm_count[dev]) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    g_sm_count[dev] = n > 0 ? n : 148;
  }
  return g_sm_count[dev];
}

}  // namespace rbh

extern "C" {
// Reads the device status word (synchronises the device) and clears it.
// 0 = no kernel reported a timed-out wait or a bounds violation.
int rb_read_status() { return rbh::read_and_clear_status(); }
int rb_sm_count() { return rbh::sm_count(); }
// Make sure the status word exists (call once per device before graph capture).
int rb_init_device() { return (rbh::device_status_word() && rbh::next_sched_slot()) ? 0 : -1; }
}
