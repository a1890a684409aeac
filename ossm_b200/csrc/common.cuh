// Shared device/host helpers for the ossm_b200 scan kernels (sm_100a only).
//
//  * mbarrier + TMA (cp.async.bulk.tensor) wrappers in inline PTX.  Every wait
//    is bounded in time (%globaltimer, kWaitLimitNs): a waiter that runs out
//    records an error in a device status word and the kernel returns, so a lost
//    copy can never hang the GPU.
//  * host-side tensor-map construction through the driver entry point (the
//    library does not link libcuda).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstring>

namespace ossm_b200 {

// ---- error plumbing (host) -------------------------------------------------
enum : int {
  kOk = 0,
  kErrInvalidArgument = -1,
  kErrCuda = -2,
  kErrUnsupported = -3,
  kErrWorkspace = -4,
};

void set_last_error(const char* fmt, ...);
int check_cuda(cudaError_t err, const char* what);

// Device status word: 0 = fine, otherwise the code of the first bounded wait
// that gave up (kStatus*).  Read with ossm_b200_device_status().
enum : int { kStatusTmaTimeout = 1, kStatusMmaTimeout = 2 };
// Every translation unit has its own word (no relocatable device code); each one
// exposes it through an accessor made by OSSM_B200_STATUS_ACCESSOR, and
// ossm_b200_device_status() combines them.
#ifdef __CUDACC__
static __device__ int g_device_status = 0;
#define OSSM_B200_STATUS_ACCESSOR(fn)                                                                   \
  int fn(int* status, int clear) {                                                                      \
    int v = 0;                                                                                          \
    if (int rc = check_cuda(cudaMemcpyFromSymbol(&v, g_device_status, sizeof(int)), "device_status read")) \
      return rc;                                                                                        \
    *status = v;                                                                                        \
    if (clear && v != 0) {                                                                              \
      int z = 0;                                                                                        \
      return check_cuda(cudaMemcpyToSymbol(g_device_status, &z, sizeof(int)), "device_status clear");  \
    }                                                                                                   \
    return kOk;                                                                                         \
  }
#endif
int status_common(int* status, int clear);
int status_lti(int* status, int clear);
int status_linoss_generic(int* status, int clear);
int status_sdlinoss(int* status, int clear);
int status_selective_scan(int* status, int clear);
int status_layer(int* status, int clear);
int status_mixer(int* status, int clear);

// ---- tensor maps (host) ----------------------------------------------------
// 2-D fp32 view [rows, cols] with row pitch `pitch_bytes`; box = box_cols x box_rows.
// Returns false (and leaves `map` untouched) when the view violates a TMA rule
// (16-byte base / pitch alignment, extent limits) so the caller can take the
// plain-load kernel instead.
bool make_tensor_map_2d_f32(CUtensorMap* map, const void* base, uint64_t cols, uint64_t rows,
                            uint64_t pitch_bytes, uint32_t box_cols, uint32_t box_rows);
// Same with the 128-byte shared-memory swizzle (box_cols * 4 must be 128): the layout the tensor-core
// matrix descriptors of the projection kernels expect.
bool make_tensor_map_2d_f32_sw128(CUtensorMap* map, const void* base, uint64_t cols, uint64_t rows,
                                  uint64_t pitch_bytes, uint32_t box_cols, uint32_t box_rows);
// Same with the 64-byte swizzle (box_cols * 4 must be 64).
bool make_tensor_map_2d_f32_sw64(CUtensorMap* map, const void* base, uint64_t cols, uint64_t rows,
                                 uint64_t pitch_bytes, uint32_t box_cols, uint32_t box_rows);
// Rank-4 float32 map with a 128-byte swizzle span.  dims / box are innermost first; strides_bytes are the byte
// strides of dimensions 1..3 (dimension 0 is dense).  box[0] * 4 must be 128.  atom32 selects the variant
// that swizzles 32-byte chunks (CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B), the only layout the tensor cores
// accept for 32-bit operands whose M / N index is the contiguous one.
// Rank-3 tiled map of float32 data without swizzle: dims / box innermost first, strides in bytes of dimensions 1 and 2.
bool make_tensor_map_3d_f32(CUtensorMap* map, const void* base, const uint64_t dims[3], const uint64_t strides_bytes[2],
                            const uint32_t box[3]);
bool make_tensor_map_4d_f32_sw128(CUtensorMap* map, const void* base, const uint64_t dims[4],
                                  const uint64_t strides_bytes[3], const uint32_t box[4], bool atom32);
// Same for 16-bit elements (bf16 payloads are moved as raw 16-bit words).
bool make_tensor_map_2d_b16(CUtensorMap* map, const void* base, uint64_t cols, uint64_t rows,
                            uint64_t pitch_bytes, uint32_t box_cols, uint32_t box_rows,
                            bool swizzle128);

int sm_count();
// Raises a kernel's dynamic shared-memory limit to `bytes`; remembered per (kernel, device) so the
// attribute call is made only when a launch needs more than any earlier one.
int ensure_dynamic_smem(const void* kernel, size_t bytes);

// ---- device helpers --------------------------------------------------------
#ifdef __CUDACC__
constexpr uint64_t kWaitLimitNs = 2000000000ull;  // longest time any wait may take (wall clock of the GPU)

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait.  Returns false once `limit_ns` of GPU wall-clock time have passed without the
// phase completing (the caller must bail out); the clock is read every 32 failed polls, each of
// which may itself block for a hardware-defined slice.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint64_t limit_ns = kWaitLimitNs,
                                          int code = kStatusTmaTimeout) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  for (uint32_t polls = 1;; ++polls) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((polls & 31u) == 0 && globaltimer_ns() - t0 > limit_ns) break;
  }
  atomicCAS(&g_device_status, 0, code);
  return false;
}

// 2-D tiled TMA load global -> shared, completion on `bar` (non-multicast).
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int32_t x,
                                            int32_t y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}

// 3-D tiled TMA load global -> shared, completion on `bar` (non-multicast).
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, uint64_t* bar, int32_t c0, int32_t c1,
                                            int32_t c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

// 4-D tiled TMA load global -> shared, completion on `bar` (non-multicast).
__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* map, uint64_t* bar, int32_t c0, int32_t c1,
                                            int32_t c2, int32_t c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// Plain arrival (release at CTA scope) on an mbarrier whose expected count is a number of threads.
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// 2-D tiled TMA store shared -> global as part of the thread's current bulk group.  The part of the
// box outside the tensor is not written.  x (the inner coordinate) times the element size must be a
// multiple of 16 bytes, and neither coordinate may be negative.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* src, int32_t x, int32_t y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(src)), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Returns once every committed bulk store of this thread has finished READING its shared-memory source.
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// Returns once every committed bulk store of this thread has completed.
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ float2 ld_nc_f2(const float2* p) {
  float2 v;
  asm volatile("ld.global.nc.L1::no_allocate.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "l"(p));
  return v;
}

__device__ __forceinline__ float4 ld_nc_f4(const float4* p) {
  float4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ void st_cs_f2(float2* p, float2 v) {
  asm volatile("st.global.cs.v2.f32 [%0], {%1, %2};" ::"l"(p), "f"(v.x), "f"(v.y) : "memory");
}

__device__ __forceinline__ void st_cs_f4(float4* p, float4 v) {
  asm volatile("st.global.cs.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
               : "memory");
}
#endif  // __CUDACC__

}  // namespace ossm_b200
