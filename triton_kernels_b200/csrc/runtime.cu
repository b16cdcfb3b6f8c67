// Host-side runtime shared by the kernel families: error text, the per-device status word,
// SM count, and tensor-map encoding through a driver entry point resolved at run time (so the
// shared library loads, and its symbols can be listed, on a machine without a driver).
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <mutex>

#include "common.cuh"

namespace fluxb {

static thread_local char g_err[512] = "";

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

static constexpr int kMaxDevices = 64;
static std::mutex g_mu;
static DeviceStatus* g_status[kMaxDevices] = {};
static int g_sms[kMaxDevices] = {};

DeviceStatus* device_status_ptr() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_status[dev] == nullptr) {
    DeviceStatus* p = nullptr;
    if (cudaMalloc(&p, sizeof(DeviceStatus)) != cudaSuccess) return nullptr;
    if (cudaMemset(p, 0, sizeof(DeviceStatus)) != cudaSuccess) return nullptr;
    g_status[dev] = p;
  }
  return g_status[dev];
}

int sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_sms[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    g_sms[dev] = n;
  }
  return g_sms[dev];
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  std::lock_guard<std::mutex> lk(g_mu);
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

int encode_tmap_bf16(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                     const uint64_t* strides_bytes, const uint32_t* box) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return set_error(FLUXB_ERR_CUDA, "cuTensorMapEncodeTiled entry point unavailable");
  cuuint64_t d[5];
  cuuint64_t s[5];
  cuuint32_t b[5];
  cuuint32_t e[5];
  for (int i = 0; i < rank; ++i) {
    d[i] = dims[i];
    b[i] = box[i];
    e[i] = 1;
    if (i > 0) s[i - 1] = strides_bytes[i - 1];
  }
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(base), d, s, b, e,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_error(FLUXB_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return FLUXB_OK;
}

}  // namespace fluxb

extern "C" int fluxb_version(void) { return 101; }  // 101: peer-exchange entry points

extern "C" const char* fluxb_last_error(void) { return fluxb::g_err; }

extern "C" int fluxb_device_status_read(int* out2) {
  using namespace fluxb;
  if (out2 == nullptr) return set_error(FLUXB_ERR_BAD_ARG, "device_status_read: null pointer");
  DeviceStatus* p = device_status_ptr();
  if (p == nullptr) return set_error(FLUXB_ERR_CUDA, "device_status_read: no status word on this device");
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return set_error(FLUXB_ERR_CUDA, "device_status_read: %s", cudaGetErrorString(e));
  DeviceStatus h;
  e = cudaMemcpy(&h, p, sizeof(h), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return set_error(FLUXB_ERR_CUDA, "device_status_read: %s", cudaGetErrorString(e));
  out2[0] = h.code;
  out2[1] = h.where;
  if (h.code != 0) cudaMemset(p, 0, sizeof(DeviceStatus));
  return FLUXB_OK;
}
