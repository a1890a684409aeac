// Host-side plumbing shared by all entry points: error strings, CUDA error
// mapping, tensor-map encoding through the driver entry point, device status.
#include "common.cuh"

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <utility>

#include "../../include/ossm_b200.h"

namespace ossm_b200 {

static thread_local char tls_error[512] = "";

void set_last_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(tls_error, sizeof(tls_error), fmt, ap);
  va_end(ap);
}

int check_cuda(cudaError_t err, const char* what) {
  if (err == cudaSuccess) return kOk;
  set_last_error("%s: %s", what, cudaGetErrorString(err));
  return kErrCuda;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(p);
    }
  });
  return fn;
}

static bool encode_2d(CUtensorMap* map, CUtensorMapDataType dt, uint32_t esize, const void* base, uint64_t cols,
                      uint64_t rows, uint64_t pitch_bytes, uint32_t box_cols, uint32_t box_rows,
                      CUtensorMapSwizzle swz) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return false;
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0) return false;
  if ((pitch_bytes & 15u) != 0 || pitch_bytes >= (1ull << 40)) return false;
  if (cols == 0 || rows == 0 || cols > 0xffffffffull || rows > 0xffffffffull) return false;
  if (box_cols > 256 || box_rows > 256 || ((uint64_t)box_cols * esize) % 16 != 0) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {pitch_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMap tmp;
  CUresult r = fn(&tmp, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  memcpy(map, &tmp, sizeof(tmp));
  return true;
}

bool make_tensor_map_2d_f32(CUtensorMap* map, const void* base, uint64_t cols, uint64_t rows, uint64_t pitch_bytes,
                            uint32_t box_cols, uint32_t box_rows) {
  return encode_2d(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, base, cols, rows, pitch_bytes, box_cols, box_rows,
                   CU_TENSOR_MAP_SWIZZLE_NONE);
}

bool make_tensor_map_2d_f32_sw128(CUtensorMap* map, const void* base, uint64_t cols, uint64_t rows,
                                  uint64_t pitch_bytes, uint32_t box_cols, uint32_t box_rows) {
  if (box_cols * 4 != 128) return false;
  return encode_2d(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, base, cols, rows, pitch_bytes, box_cols, box_rows,
                   CU_TENSOR_MAP_SWIZZLE_128B);
}

bool make_tensor_map_2d_f32_sw64(CUtensorMap* map, const void* base, uint64_t cols, uint64_t rows,
                                 uint64_t pitch_bytes, uint32_t box_cols, uint32_t box_rows) {
  if (box_cols * 4 != 64) return false;
  return encode_2d(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, base, cols, rows, pitch_bytes, box_cols, box_rows,
                   CU_TENSOR_MAP_SWIZZLE_64B);
}

bool make_tensor_map_3d_f32(CUtensorMap* map, const void* base, const uint64_t dims[3], const uint64_t strides_bytes[2],
                            const uint32_t box[3]) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return false;
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0 || (box[0] * 4) % 16 != 0) return false;
  cuuint64_t d[3], st[2];
  cuuint32_t bx[3], es[3] = {1, 1, 1};
  for (int i = 0; i < 3; ++i) {
    if (dims[i] == 0 || dims[i] > 0xffffffffull || box[i] == 0 || box[i] > 256) return false;
    d[i] = dims[i];
    bx[i] = box[i];
  }
  for (int i = 0; i < 2; ++i) {
    if ((strides_bytes[i] & 15u) != 0 || strides_bytes[i] >= (1ull << 40)) return false;
    st[i] = strides_bytes[i];
  }
  CUtensorMap tmp;
  CUresult r = fn(&tmp, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(base), d, st, bx, es,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  memcpy(map, &tmp, sizeof(tmp));
  return true;
}

bool make_tensor_map_4d_f32_sw128(CUtensorMap* map, const void* base, const uint64_t dims[4],
                                  const uint64_t strides_bytes[3], const uint32_t box[4], bool atom32) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return false;
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0 || box[0] * 4 != 128) return false;
  cuuint64_t d[4], st[3];
  cuuint32_t bx[4], es[4] = {1, 1, 1, 1};
  for (int i = 0; i < 4; ++i) {
    if (dims[i] == 0 || dims[i] > 0xffffffffull || box[i] == 0 || box[i] > 256) return false;
    d[i] = dims[i];
    bx[i] = box[i];
  }
  for (int i = 0; i < 3; ++i) {
    if ((strides_bytes[i] & 15u) != 0 || strides_bytes[i] >= (1ull << 40)) return false;
    st[i] = strides_bytes[i];
  }
  CUtensorMap tmp;
  CUresult r = fn(&tmp, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<void*>(base), d, st, bx, es,
                  CU_TENSOR_MAP_INTERLEAVE_NONE,
                  atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  memcpy(map, &tmp, sizeof(tmp));
  return true;
}

bool make_tensor_map_2d_b16(CUtensorMap* map, const void* base, uint64_t cols, uint64_t rows, uint64_t pitch_bytes,
                            uint32_t box_cols, uint32_t box_rows, bool swizzle128) {
  return encode_2d(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, base, cols, rows, pitch_bytes, box_cols, box_rows,
                   swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE);
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

int ensure_dynamic_smem(const void* kernel, size_t bytes) {
  static std::mutex mu;
  static std::map<std::pair<const void*, int>, size_t> granted;
  int dev = 0;
  if (int rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice")) return rc;
  std::lock_guard<std::mutex> lock(mu);
  size_t& have = granted[std::make_pair(kernel, dev)];
  if (bytes <= have) return kOk;
  if (int rc = check_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes),
                          "cudaFuncSetAttribute(max dynamic smem)"))
    return rc;
  have = bytes;
  return kOk;
}

}  // namespace ossm_b200

namespace ossm_b200 {
OSSM_B200_STATUS_ACCESSOR(status_common)

// A CTA of one thread waits on an mbarrier that nothing ever completes, with a short limit: the
// wait must give up, record kStatusTmaTimeout and let the kernel return.
__global__ void wait_timeout_selftest_kernel(unsigned long long limit_ns, int* gave_up) {
  __shared__ uint64_t bar;
  mbar_init(&bar, 1);
  fence_barrier_init();
  const bool ok = mbar_wait(&bar, 0, limit_ns);
  *gave_up = ok ? 0 : 1;
}
}  // namespace ossm_b200

extern "C" {

const char* ossm_b200_last_error(void) { return ossm_b200::tls_error; }

int ossm_b200_selftest_wait_timeout(uint64_t limit_ns, int* gave_up_dev, cudaStream_t stream) {
  using namespace ossm_b200;
  if (gave_up_dev == nullptr || limit_ns == 0 || limit_ns > 100000000ull) {
    set_last_error("selftest_wait_timeout: need a device int and a limit of 1 ns .. 100 ms");
    return kErrInvalidArgument;
  }
  wait_timeout_selftest_kernel<<<1, 1, 0, stream>>>(limit_ns, gave_up_dev);
  return check_cuda(cudaGetLastError(), "wait_timeout_selftest_kernel launch");
}

int ossm_b200_version(void) { return 1; }

int ossm_b200_device_status(int* status, int clear) {
  using namespace ossm_b200;
  if (status == nullptr) {
    set_last_error("device_status: null output pointer");
    return kErrInvalidArgument;
  }
  // first non-zero word wins; every word is cleared when asked
  int (*const words[])(int*, int) = {status_common, status_lti, status_linoss_generic, status_sdlinoss,
                                     status_selective_scan, status_layer, status_mixer};
  int first = 0;
  for (auto fn : words) {
    int v = 0;
    if (int rc = fn(&v, clear)) return rc;
    if (first == 0) first = v;
  }
  *status = first;
  return kOk;
}

}  // extern "C"
