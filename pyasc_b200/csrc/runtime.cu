// Device / stream / memory / event wrappers of libasc_cuda and the shared host helpers.
// CUDA bodies behind the wrapper names the reference's runtime binding already calls
// (python/asc/lib/runtime/rt_wrapper.cpp:23-244).
#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <thread>
#include <vector>

#include <cudaTypedefs.h>

#include "../../include/asc_cuda.h"
#include "host_common.h"

namespace aschost {

static thread_local char g_last_error[512] = {0};
std::atomic<uint64_t> g_launch_count{0};

int32_t record_cuda_error(cudaError_t e, const char* what) {
  snprintf(g_last_error, sizeof(g_last_error), "%s: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e));
  cudaGetLastError();  // clear the sticky-less error state so later calls report their own failures
  return ASC_ERR_CUDA;
}

int32_t record_driver_error(int code, const char* what) {
  snprintf(g_last_error, sizeof(g_last_error), "%s: driver error %d", what, code);
  return ASC_ERR_CUDA;
}

static constexpr int kMaxDevices = 64;
static uint32_t* g_status_ptr[kMaxDevices] = {nullptr};
static std::atomic<int> g_sm_count[kMaxDevices];
static std::mutex g_mutex;
static std::vector<cudaStream_t> g_streams[kMaxDevices];

__device__ uint32_t g_device_status = 0;

int32_t device_status_word(uint32_t** out) {
  int dev = 0;
  ASC_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return ASC_ERR_INVALID_ARG;
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_status_ptr[dev] == nullptr) {
    void* p = nullptr;
    ASC_CUDA_TRY(cudaGetSymbolAddress(&p, g_device_status));
    g_status_ptr[dev] = static_cast<uint32_t*>(p);
  }
  *out = g_status_ptr[dev];
  return ASC_OK;
}

int32_t sm_count(int* out) {
  int dev = 0;
  ASC_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return ASC_ERR_INVALID_ARG;
  int cached = g_sm_count[dev].load(std::memory_order_acquire);
  if (cached == 0) {
    int n = 0;
    ASC_CUDA_TRY(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev));
    g_sm_count[dev].store(n, std::memory_order_release);
    cached = n;
  }
  *out = cached;
  return ASC_OK;
}

static cudaMemPool_t g_scratch_pool[kMaxDevices] = {nullptr};

int32_t scratch_alloc(void** out, size_t bytes, cudaStream_t stream) {
  int dev = 0;
  ASC_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return ASC_ERR_INVALID_ARG;
  cudaMemPool_t pool = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (g_scratch_pool[dev] == nullptr) {
      cudaMemPoolProps props = {};
      props.allocType = cudaMemAllocationTypePinned;
      props.handleTypes = cudaMemHandleTypeNone;
      props.location.type = cudaMemLocationTypeDevice;
      props.location.id = dev;
      ASC_CUDA_TRY(cudaMemPoolCreate(&pool, &props));
      uint64_t keep = ~0ull;      // freed blocks stay in the pool
      ASC_CUDA_TRY(cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep));
      g_scratch_pool[dev] = pool;
    }
    pool = g_scratch_pool[dev];
  }
  ASC_CUDA_TRY(cudaMallocFromPoolAsync(out, bytes, pool, stream));
  return ASC_OK;
}

int32_t scratch_free(void* ptr, cudaStream_t stream) {
  ASC_CUDA_TRY(cudaFreeAsync(ptr, stream));
  return ASC_OK;
}

static std::atomic<PFN_cuTensorMapEncodeTiled_v12000> g_encode{nullptr};

int32_t encode_tmap(CUtensorMap* out, CUtensorMapDataType dtype, uint32_t rank, const void* base,
                    const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                    CUtensorMapSwizzle swizzle, CUtensorMapL2promotion promo) {
  PFN_cuTensorMapEncodeTiled_v12000 encode = g_encode.load(std::memory_order_acquire);
  if (encode == nullptr) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    ASC_CUDA_TRY(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
    if (fn == nullptr || qres != cudaDriverEntryPointSuccess) return record_driver_error(-1, "cuTensorMapEncodeTiled lookup");
    encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
    g_encode.store(encode, std::memory_order_release);
  }
  cuuint64_t gdims[5];
  cuuint64_t gstrides[4];
  cuuint32_t gbox[5];
  cuuint32_t estr[5];
  for (uint32_t i = 0; i < rank; ++i) {
    gdims[i] = dims[i];
    gbox[i] = box[i];
    estr[i] = 1;
    if (i + 1 < rank) gstrides[i] = strides_bytes[i];
  }
  CUresult r = encode(out, dtype, rank, const_cast<void*>(base), gdims, gstrides, gbox, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return record_driver_error(static_cast<int>(r), "cuTensorMapEncodeTiled");
  return ASC_OK;
}

}  // namespace aschost

using namespace aschost;

extern "C" {

int32_t GetSocVersionWrapper(char* ver, uint32_t maxLen) {
  if (ver == nullptr || maxLen == 0) return ASC_ERR_INVALID_ARG;
  int dev = 0;
  ASC_CUDA_TRY(cudaGetDevice(&dev));
  cudaDeviceProp prop;
  ASC_CUDA_TRY(cudaGetDeviceProperties(&prop, dev));
  snprintf(ver, maxLen, "%s", prop.name);
  return ASC_OK;
}

int32_t GetDeviceCountWrapper(int32_t* cnt) {
  if (cnt == nullptr) return ASC_ERR_INVALID_ARG;
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess) {
    *cnt = 0;
    return record_cuda_error(e, "cudaGetDeviceCount");
  }
  *cnt = n;
  return ASC_OK;
}

int32_t GetDeviceInfoWrapper(uint32_t deviceId, int32_t /*moduleType*/, int32_t infoType, int64_t* val) {
  if (val == nullptr) return ASC_ERR_INVALID_ARG;
  int v = 0;
  const int dev = static_cast<int>(deviceId);
  switch (infoType) {
    case 0:
      ASC_CUDA_TRY(cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev));
      *val = v;
      return ASC_OK;
    case 1: {
      cudaDeviceProp prop;
      ASC_CUDA_TRY(cudaGetDeviceProperties(&prop, dev));
      *val = static_cast<int64_t>(prop.totalGlobalMem);
      return ASC_OK;
    }
    case 2:
      ASC_CUDA_TRY(cudaDeviceGetAttribute(&v, cudaDevAttrL2CacheSize, dev));
      *val = v;
      return ASC_OK;
    case 3:
      ASC_CUDA_TRY(cudaDeviceGetAttribute(&v, cudaDevAttrClockRate, dev));
      *val = v;
      return ASC_OK;
    case 4: {
      int major = 0, minor = 0;
      ASC_CUDA_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
      ASC_CUDA_TRY(cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev));
      *val = major * 10 + minor;
      return ASC_OK;
    }
    default:
      return ASC_ERR_INVALID_ARG;
  }
}

int32_t DeviceResetWrapper(int32_t devId) {
  if (devId < 0 || devId >= kMaxDevices) return ASC_ERR_INVALID_ARG;
  std::vector<cudaStream_t> streams;
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    streams.swap(g_streams[devId]);
  }
  if (streams.empty()) return ASC_OK;
  int prev = 0;
  ASC_CUDA_TRY(cudaGetDevice(&prev));
  ASC_CUDA_TRY(cudaSetDevice(devId));
  for (cudaStream_t s : streams) cudaStreamDestroy(s);
  ASC_CUDA_TRY(cudaSetDevice(prev));
  return ASC_OK;
}

int32_t SetDeviceWrapper(int32_t devId) {
  if (devId < 0) return ASC_ERR_INVALID_ARG;
  ASC_CUDA_TRY(cudaSetDevice(devId));
  return ASC_OK;
}

int32_t StreamCreateWrapper(void** stm, int32_t priority) {
  if (stm == nullptr) return ASC_ERR_INVALID_ARG;
  cudaStream_t s = nullptr;
  ASC_CUDA_TRY(cudaStreamCreateWithPriority(&s, cudaStreamNonBlocking, priority));
  int dev = 0;
  ASC_CUDA_TRY(cudaGetDevice(&dev));
  if (dev >= 0 && dev < kMaxDevices) {
    std::lock_guard<std::mutex> lock(g_mutex);
    g_streams[dev].push_back(s);
  }
  *stm = s;
  return ASC_OK;
}

int32_t StreamDestroyWrapper(void* stm) {
  if (stm == nullptr) return ASC_OK;
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    for (auto& vec : g_streams) {
      for (size_t i = 0; i < vec.size(); ++i) {
        if (vec[i] == stm) {
          vec.erase(vec.begin() + i);
          break;
        }
      }
    }
  }
  ASC_CUDA_TRY(cudaStreamDestroy(static_cast<cudaStream_t>(stm)));
  return ASC_OK;
}

int32_t MallocWrapper(void** devPtr, uint64_t size, int32_t /*type*/, uint16_t /*moduleId*/) {
  if (devPtr == nullptr || size == 0) return ASC_ERR_INVALID_ARG;
  ASC_CUDA_TRY(cudaMalloc(devPtr, size));
  return ASC_OK;
}

static bool to_cuda_kind(int32_t kind, cudaMemcpyKind* out) {
  switch (kind) {
    case 0: *out = cudaMemcpyHostToHost; return true;
    case 1: *out = cudaMemcpyHostToDevice; return true;
    case 2: *out = cudaMemcpyDeviceToHost; return true;
    case 3: *out = cudaMemcpyDeviceToDevice; return true;
    default: return false;
  }
}

int32_t MemcpyWrapper(void* dst, uint64_t destMax, const void* src, uint64_t cnt, int32_t kind) {
  cudaMemcpyKind k;
  if (dst == nullptr || src == nullptr || cnt > destMax || !to_cuda_kind(kind, &k)) return ASC_ERR_INVALID_ARG;
  if (cnt == 0) return ASC_OK;
  ASC_CUDA_TRY(cudaMemcpy(dst, src, cnt, k));
  return ASC_OK;
}

int32_t MemcpyAsyncWrapper(void* dst, uint64_t destMax, const void* src, uint64_t cnt, int32_t kind, void* stm) {
  cudaMemcpyKind k;
  if (dst == nullptr || src == nullptr || cnt > destMax || !to_cuda_kind(kind, &k)) return ASC_ERR_INVALID_ARG;
  if (cnt == 0) return ASC_OK;
  ASC_CUDA_TRY(cudaMemcpyAsync(dst, src, cnt, k, static_cast<cudaStream_t>(stm)));
  return ASC_OK;
}

int32_t StreamSynchronizeWithTimeoutWrapper(void* stm, int32_t timeout) {
  if (timeout <= 0) return StreamSynchronizeWrapper(stm);
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout);
  for (;;) {
    cudaError_t e = cudaStreamQuery(static_cast<cudaStream_t>(stm));
    if (e == cudaSuccess) return ASC_OK;
    if (e != cudaErrorNotReady) return record_cuda_error(e, "cudaStreamQuery");
    if (std::chrono::steady_clock::now() > deadline) return ASC_ERR_DEVICE_TIMEOUT;
    std::this_thread::sleep_for(std::chrono::microseconds(50));
  }
}

int32_t StreamSynchronizeWrapper(void* stm) {
  ASC_CUDA_TRY(cudaStreamSynchronize(static_cast<cudaStream_t>(stm)));
  return ASC_OK;
}

int32_t FreeWrapper(void* devPtr) {
  if (devPtr == nullptr) return ASC_OK;
  ASC_CUDA_TRY(cudaFree(devPtr));
  return ASC_OK;
}

int32_t DeviceSynchronizeWrapper(void) {
  ASC_CUDA_TRY(cudaDeviceSynchronize());
  return ASC_OK;
}

int32_t HostMallocWrapper(void** hostPtr, uint64_t size) {
  if (hostPtr == nullptr || size == 0) return ASC_ERR_INVALID_ARG;
  ASC_CUDA_TRY(cudaHostAlloc(hostPtr, size, cudaHostAllocDefault));
  return ASC_OK;
}

int32_t HostFreeWrapper(void* hostPtr) {
  if (hostPtr == nullptr) return ASC_OK;
  ASC_CUDA_TRY(cudaFreeHost(hostPtr));
  return ASC_OK;
}

int32_t HostRegisterWrapper(void* hostPtr, uint64_t size) {
  if (hostPtr == nullptr || size == 0) return ASC_ERR_INVALID_ARG;
  ASC_CUDA_TRY(cudaHostRegister(hostPtr, size, cudaHostRegisterDefault));
  return ASC_OK;
}

int32_t HostUnregisterWrapper(void* hostPtr) {
  if (hostPtr == nullptr) return ASC_OK;
  ASC_CUDA_TRY(cudaHostUnregister(hostPtr));
  return ASC_OK;
}

int32_t asc_cuda_event_create(void** ev) {
  if (ev == nullptr) return ASC_ERR_INVALID_ARG;
  cudaEvent_t e = nullptr;
  ASC_CUDA_TRY(cudaEventCreate(&e));
  *ev = e;
  return ASC_OK;
}

int32_t asc_cuda_event_record(void* ev, void* stream) {
  if (ev == nullptr) return ASC_ERR_INVALID_ARG;
  ASC_CUDA_TRY(cudaEventRecord(static_cast<cudaEvent_t>(ev), static_cast<cudaStream_t>(stream)));
  return ASC_OK;
}

int32_t StreamWaitEventWrapper(void* stm, void* ev) {
  if (ev == nullptr) return ASC_ERR_INVALID_ARG;
  ASC_CUDA_TRY(cudaStreamWaitEvent(static_cast<cudaStream_t>(stm), static_cast<cudaEvent_t>(ev), 0));
  return ASC_OK;
}

int32_t asc_cuda_event_create_notiming(void** ev) {
  if (ev == nullptr) return ASC_ERR_INVALID_ARG;
  cudaEvent_t e = nullptr;
  ASC_CUDA_TRY(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
  *ev = e;
  return ASC_OK;
}

int32_t asc_cuda_event_synchronize(void* ev) {
  if (ev == nullptr) return ASC_ERR_INVALID_ARG;
  ASC_CUDA_TRY(cudaEventSynchronize(static_cast<cudaEvent_t>(ev)));
  return ASC_OK;
}

int32_t asc_cuda_event_elapsed_ms(void* start, void* stop, float* ms) {
  if (start == nullptr || stop == nullptr || ms == nullptr) return ASC_ERR_INVALID_ARG;
  ASC_CUDA_TRY(cudaEventElapsedTime(ms, static_cast<cudaEvent_t>(start), static_cast<cudaEvent_t>(stop)));
  return ASC_OK;
}

int32_t asc_cuda_event_destroy(void* ev) {
  if (ev == nullptr) return ASC_OK;
  ASC_CUDA_TRY(cudaEventDestroy(static_cast<cudaEvent_t>(ev)));
  return ASC_OK;
}

int32_t asc_cuda_status_string(int32_t code, char* buf, uint32_t n) {
  if (buf == nullptr || n == 0) return ASC_ERR_INVALID_ARG;
  const char* s = "unknown status";
  switch (code) {
    case ASC_OK: s = "ok"; break;
    case ASC_ERR_INVALID_ARG: s = "invalid argument"; break;
    case ASC_ERR_MISALIGNED: s = "misaligned pointer or leading dimension"; break;
    case ASC_ERR_UNSUPPORTED: s = "unsupported shape or dtype"; break;
    case ASC_ERR_CUDA: s = "CUDA call failed"; break;
    case ASC_ERR_DEVICE_TIMEOUT: s = "bounded device-side wait ran out"; break;
    case ASC_ERR_TOO_LARGE: s = "size beyond the documented maximum"; break;
    case ASC_ERR_NO_DEVICE: s = "no usable CUDA device"; break;
    default: break;
  }
  snprintf(buf, n, "%s", s);
  return ASC_OK;
}

int32_t asc_cuda_last_cuda_error(char* buf, uint32_t n) {
  if (buf == nullptr || n == 0) return ASC_ERR_INVALID_ARG;
  snprintf(buf, n, "%s", g_last_error);
  return ASC_OK;
}

int32_t asc_cuda_check_device_status(void* stream, uint32_t* dev_code) {
  if (dev_code == nullptr) return ASC_ERR_INVALID_ARG;
  uint32_t* word = nullptr;
  int32_t rc = device_status_word(&word);
  if (rc != ASC_OK) return rc;
  ASC_CUDA_TRY(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  uint32_t v = 0;
  ASC_CUDA_TRY(cudaMemcpy(&v, word, sizeof(v), cudaMemcpyDeviceToHost));
  *dev_code = v;
  if (v != 0) {
    ASC_CUDA_TRY(cudaMemset(word, 0, sizeof(v)));
    return ASC_ERR_DEVICE_TIMEOUT;
  }
  return ASC_OK;
}

int32_t asc_cuda_launch_count(uint64_t* count) {
  if (count == nullptr) return ASC_ERR_INVALID_ARG;
  *count = g_launch_count.load();
  return ASC_OK;
}

}  // extern "C"
