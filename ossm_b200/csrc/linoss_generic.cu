// Generic LinOSS scan: per-channel COMPLEX 2x2 transition applied to a complex
// 2-vector, forcing given per step:  s_t = M s_{t-1} + b_t,  b_seq [L,B,P,2].
//
// Replaces ossm::linoss_scan (src/ossm/csrc/linoss_scan.cpp:115-146,
// linoss_scan_cuda.cu:34-153) and the Python-loop backward of _LinossScanFn
// (src/ossm/models/linoss.py:83-151).  This is the compatibility entry point
// (the LinOSS layers themselves use the real-coefficient oscillator scan in
// lti_scan.cu, which moves half the bytes); it keeps the reference's contract
// of materialised states: forward writes [L,B,P,2], backward reads them back.
//
// One thread per series, serial in time.  The staged kernels (any 16-byte aligned
// operands) give a CTA 64 series and let TMA bring tiles of 32 time steps x 1 KiB
// into a ring of shared-memory stages, several tiles ahead of the arithmetic: the
// loads in flight, not the number of resident warps, hide the HBM latency, and
// 8192 series already occupy 128 SMs.  Stores are 16 bytes per lane, 1 KiB
// contiguous per step and CTA.  The plain kernels (register double-buffer of
// kBatch steps) remain for operands a tensor map cannot describe.  Matrix
// gradients are per-series partial sums reduced over the batch by a second,
// fixed-order kernel (deterministic, no atomics).
#include "common.cuh"

#include "../../include/ossm_b200.h"

namespace ossm_b200 {
OSSM_B200_STATUS_ACCESSOR(status_linoss_generic)
namespace lgen {

constexpr int kBatch = 8;
constexpr int kThreads = 128;

struct Cx {
  float re, im;
};
__device__ __forceinline__ Cx cmul(Cx a, Cx b) { return {a.re * b.re - a.im * b.im, a.re * b.im + a.im * b.re}; }
__device__ __forceinline__ Cx cadd(Cx a, Cx b) { return {a.re + b.re, a.im + b.im}; }
__device__ __forceinline__ Cx cconj(Cx a) { return {a.re, -a.im}; }
__device__ __forceinline__ Cx cfma(Cx a, Cx b, Cx c) {  // a*b + c
  return {fmaf(a.re, b.re, fmaf(-a.im, b.im, c.re)), fmaf(a.re, b.im, fmaf(a.im, b.re, c.im))};
}

__global__ void __launch_bounds__(kThreads)
linoss_forward_kernel(const float2* __restrict__ m11, const float2* __restrict__ m12, const float2* __restrict__ m21,
                      const float2* __restrict__ m22, const float4* __restrict__ b_seq, float4* __restrict__ out,
                      long long L, long long N, long long P) {
  const long long n = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= N) return;
  const long long ch = n % P;
  const Cx a11{m11[ch].x, m11[ch].y}, a12{m12[ch].x, m12[ch].y};
  const Cx a21{m21[ch].x, m21[ch].y}, a22{m22[ch].x, m22[ch].y};
  Cx s0{0.f, 0.f}, s1{0.f, 0.f};
  float4 cur[kBatch], nxt[kBatch];
  auto load = [&](float4* dst, long long t0) {
#pragma unroll
    for (int r = 0; r < kBatch; ++r) {
      const long long t = t0 + r;
      dst[r] = t < L ? ld_nc_f4(b_seq + t * N + n) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  };
  load(cur, 0);
  for (long long t0 = 0; t0 < L; t0 += kBatch) {
    load(nxt, t0 + kBatch);
#pragma unroll
    for (int r = 0; r < kBatch; ++r) {
      const long long t = t0 + r;
      const Cx b0{cur[r].x, cur[r].y}, b1{cur[r].z, cur[r].w};
      const Cx n0 = cfma(a12, s1, cfma(a11, s0, b0));
      const Cx n1 = cfma(a22, s1, cfma(a21, s0, b1));
      s0 = n0;
      s1 = n1;
      if (t < L) out[t * N + n] = make_float4(s0.re, s0.im, s1.re, s1.im);
    }
#pragma unroll
    for (int r = 0; r < kBatch; ++r) cur[r] = nxt[r];
  }
}

// partials: [8][N] = Re/Im of the four sums  sum_t G_i * conj(p_j)  of this series
__global__ void __launch_bounds__(kThreads)
linoss_backward_kernel(const float2* __restrict__ m11, const float2* __restrict__ m12,
                       const float2* __restrict__ m21, const float2* __restrict__ m22,
                       const float4* __restrict__ states, const float4* __restrict__ grad_out,
                       float4* __restrict__ grad_b, float* __restrict__ partials, long long L, long long N,
                       long long P) {
  const long long n = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= N) return;
  const long long ch = n % P;
  // adjoint transition M^H (linoss.py:109-112, 140-141)
  const Cx c11 = cconj({m11[ch].x, m11[ch].y}), c12 = cconj({m12[ch].x, m12[ch].y});
  const Cx c21 = cconj({m21[ch].x, m21[ch].y}), c22 = cconj({m22[ch].x, m22[ch].y});
  Cx l0{0.f, 0.f}, l1{0.f, 0.f};
  Cx d11{0.f, 0.f}, d12{0.f, 0.f}, d21{0.f, 0.f}, d22{0.f, 0.f};
  float4 gcur[kBatch], gnxt[kBatch], pcur[kBatch], pnxt[kBatch];
  // batch covering times t0 .. t0-kBatch+1 (descending); previous state of t is states[t-1]
  auto load = [&](float4* gd, float4* pd, long long t0) {
#pragma unroll
    for (int r = 0; r < kBatch; ++r) {
      const long long t = t0 - r;
      gd[r] = t >= 0 ? ld_nc_f4(grad_out + t * N + n) : make_float4(0.f, 0.f, 0.f, 0.f);
      pd[r] = t >= 1 ? ld_nc_f4(states + (t - 1) * N + n) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  };
  load(gcur, pcur, L - 1);
  for (long long t0 = L - 1; t0 >= 0; t0 -= kBatch) {
    load(gnxt, pnxt, t0 - kBatch);
#pragma unroll
    for (int r = 0; r < kBatch; ++r) {
      const long long t = t0 - r;
      if (t < 0) break;
      const Cx g0 = cadd(l0, {gcur[r].x, gcur[r].y});
      const Cx g1 = cadd(l1, {gcur[r].z, gcur[r].w});
      grad_b[t * N + n] = make_float4(g0.re, g0.im, g1.re, g1.im);
      const Cx q0 = cconj({pcur[r].x, pcur[r].y}), q1 = cconj({pcur[r].z, pcur[r].w});
      d11 = cfma(g0, q0, d11);
      d12 = cfma(g0, q1, d12);
      d21 = cfma(g1, q0, d21);
      d22 = cfma(g1, q1, d22);
      l0 = cfma(g1, c21, cmul(g0, c11));
      l1 = cfma(g1, c22, cmul(g0, c12));
    }
#pragma unroll
    for (int r = 0; r < kBatch; ++r) { gcur[r] = gnxt[r]; pcur[r] = pnxt[r]; }
  }
  partials[0 * N + n] = d11.re; partials[1 * N + n] = d11.im;
  partials[2 * N + n] = d12.re; partials[3 * N + n] = d12.im;
  partials[4 * N + n] = d21.re; partials[5 * N + n] = d21.im;
  partials[6 * N + n] = d22.re; partials[7 * N + n] = d22.im;
}


// ---- TMA-staged kernels ----------------------------------------------------------------------
constexpr int kSeries = 64;                         // threads = series per CTA (a box row of 256 floats)
constexpr int kRows = 32;                           // time steps per tile
constexpr int kTileBytes = kRows * kSeries * 16;    // 32 KiB

// Shared memory: barriers (1 KiB) | ring of tiles.
__global__ void __launch_bounds__(kSeries)
linoss_forward_staged_kernel(const __grid_constant__ CUtensorMap tm_b, const float2* __restrict__ m11,
                             const float2* __restrict__ m12, const float2* __restrict__ m21,
                             const float2* __restrict__ m22, float4* __restrict__ out, long long L, long long N,
                             long long P, int ring) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw);
  unsigned char* ring_base = smem_raw + 1024;
  const long long col0 = (long long)blockIdx.x * kSeries;
  const long long n = col0 + threadIdx.x;
  const bool valid = n < N;
  const long long ch = valid ? n % P : 0;
  const Cx a11{m11[ch].x, m11[ch].y}, a12{m12[ch].x, m12[ch].y};
  const Cx a21{m21[ch].x, m21[ch].y}, a22{m22[ch].x, m22[ch].y};
  const long long ntiles = (L + kRows - 1) / kRows;
  if (threadIdx.x == 0) {
    prefetch_tensormap(&tm_b);
    for (int s = 0; s < ring; ++s) mbar_init(&bars[s], 1);
    fence_barrier_init();
    fence_proxy_async();
    const int pre = (int)(ntiles < ring ? ntiles : ring);
    for (int s = 0; s < pre; ++s) {
      mbar_expect_tx(&bars[s], kTileBytes);
      tma_load_2d(ring_base + (size_t)s * kTileBytes, &tm_b, &bars[s], (int32_t)(col0 * 4), s * kRows);
    }
  }
  __syncthreads();
  Cx s0{0.f, 0.f}, s1{0.f, 0.f};
  int slot = 0;
  uint32_t parity = 0;
  float4* dst = out + n;
  for (long long tile = 0; tile < ntiles; ++tile) {
    if (!mbar_wait(&bars[slot], parity)) return;
    const float4* rows = reinterpret_cast<const float4*>(ring_base + (size_t)slot * kTileBytes) + threadIdx.x;
    const long long t0 = tile * kRows;
    const int live = (L - t0) < kRows ? (int)(L - t0) : kRows;
#pragma unroll 8
    for (int r = 0; r < kRows; ++r) {
      const float4 b = rows[r * kSeries];
      const Cx n0 = cfma(a12, s1, cfma(a11, s0, {b.x, b.y}));
      const Cx n1 = cfma(a22, s1, cfma(a21, s0, {b.z, b.w}));
      s0 = n0;
      s1 = n1;
      if (valid && r < live) st_cs_f4(dst + (t0 + r) * N, make_float4(s0.re, s0.im, s1.re, s1.im));
    }
    __syncthreads();   // every thread is done with this stage
    if (threadIdx.x == 0 && tile + ring < ntiles) {
      fence_proxy_async();
      mbar_expect_tx(&bars[slot], kTileBytes);
      tma_load_2d(ring_base + (size_t)slot * kTileBytes, &tm_b, &bars[slot], (int32_t)(col0 * 4),
                  (int32_t)((tile + ring) * kRows));
    }
    if (++slot == ring) { slot = 0; parity ^= 1; }
  }
}

// Stage = grad_out rows [t0, t0+32) followed by the states rows [t0-1, t0+31): the state BEFORE step t is row t-1
// (the row before the first one is read as zeros by TMA).  Tiles are walked from the last to the first.
__global__ void __launch_bounds__(kSeries)
linoss_backward_staged_kernel(const __grid_constant__ CUtensorMap tm_g, const __grid_constant__ CUtensorMap tm_s,
                              const float2* __restrict__ m11, const float2* __restrict__ m12,
                              const float2* __restrict__ m21, const float2* __restrict__ m22,
                              float4* __restrict__ grad_b, float* __restrict__ partials, long long L, long long N,
                              long long P, int ring) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw);
  unsigned char* ring_base = smem_raw + 1024;
  constexpr uint32_t kPair = 2 * kTileBytes;
  const long long col0 = (long long)blockIdx.x * kSeries;
  const long long n = col0 + threadIdx.x;
  const bool valid = n < N;
  const long long ch = valid ? n % P : 0;
  // adjoint transition M^H (linoss.py:109-112, 140-141)
  const Cx c11 = cconj({m11[ch].x, m11[ch].y}), c12 = cconj({m12[ch].x, m12[ch].y});
  const Cx c21 = cconj({m21[ch].x, m21[ch].y}), c22 = cconj({m22[ch].x, m22[ch].y});
  const long long ntiles = (L + kRows - 1) / kRows;
  auto issue = [&](int s, long long tile) {
    unsigned char* dst = ring_base + (size_t)s * kPair;
    mbar_expect_tx(&bars[s], kPair);
    tma_load_2d(dst, &tm_g, &bars[s], (int32_t)(col0 * 4), (int32_t)(tile * kRows));
    tma_load_2d(dst + kTileBytes, &tm_s, &bars[s], (int32_t)(col0 * 4), (int32_t)(tile * kRows) - 1);
  };
  if (threadIdx.x == 0) {
    prefetch_tensormap(&tm_g);
    prefetch_tensormap(&tm_s);
    for (int s = 0; s < ring; ++s) mbar_init(&bars[s], 1);
    fence_barrier_init();
    fence_proxy_async();
    const int pre = (int)(ntiles < ring ? ntiles : ring);
    for (int s = 0; s < pre; ++s) issue(s, ntiles - 1 - s);
  }
  __syncthreads();
  Cx l0{0.f, 0.f}, l1{0.f, 0.f};
  Cx d11{0.f, 0.f}, d12{0.f, 0.f}, d21{0.f, 0.f}, d22{0.f, 0.f};
  int slot = 0;
  uint32_t parity = 0;
  float4* dst = grad_b + n;
  for (long long it = 0; it < ntiles; ++it) {
    const long long tile = ntiles - 1 - it;
    if (!mbar_wait(&bars[slot], parity)) return;
    const float4* gr = reinterpret_cast<const float4*>(ring_base + (size_t)slot * kPair) + threadIdx.x;
    const float4* pr = reinterpret_cast<const float4*>(ring_base + (size_t)slot * kPair + kTileBytes) + threadIdx.x;
    const long long t0 = tile * kRows;
    const int live = (L - t0) < kRows ? (int)(L - t0) : kRows;
#pragma unroll 8
    for (int r = kRows - 1; r >= 0; --r) {
      // rows past the end hold a zero gradient (and the adjoint is still zero there): they change nothing
      const float4 g = gr[r * kSeries], q = pr[r * kSeries];
      const Cx g0 = cadd(l0, {g.x, g.y});
      const Cx g1 = cadd(l1, {g.z, g.w});
      if (valid && r < live) st_cs_f4(dst + (t0 + r) * N, make_float4(g0.re, g0.im, g1.re, g1.im));
      const Cx q0 = cconj({q.x, q.y}), q1 = cconj({q.z, q.w});
      d11 = cfma(g0, q0, d11);
      d12 = cfma(g0, q1, d12);
      d21 = cfma(g1, q0, d21);
      d22 = cfma(g1, q1, d22);
      l0 = cfma(g1, c21, cmul(g0, c11));
      l1 = cfma(g1, c22, cmul(g0, c12));
    }
    __syncthreads();
    if (threadIdx.x == 0 && it + ring < ntiles) {
      fence_proxy_async();
      issue(slot, tile - ring);
    }
    if (++slot == ring) { slot = 0; parity ^= 1; }
  }
  if (valid) {
    partials[0 * N + n] = d11.re; partials[1 * N + n] = d11.im;
    partials[2 * N + n] = d12.re; partials[3 * N + n] = d12.im;
    partials[4 * N + n] = d21.re; partials[5 * N + n] = d21.im;
    partials[6 * N + n] = d22.re; partials[7 * N + n] = d22.im;
  }
}

// Tensor map over a [L, N] array of float4 seen as [L rows][4 N floats]; boxes of 64 series x 32 steps.
static bool staged_map(CUtensorMap* tm, const void* base, long long L, long long N) {
  if (N * 4 > 0x7fffffffLL || L > 0x7fffffffLL - kRows) return false;
  return make_tensor_map_2d_f32(tm, base, (uint64_t)N * 4, (uint64_t)L, (uint64_t)N * 16, kSeries * 4, kRows);
}

// grad_m: [P][2][2] complex64 (interleaved) -- batch sums in double, fixed order:
// thread (cx, gy) sums series b = gy, gy+kGroups, ... of channel cx; thread (cx, 0)
// then adds the group sums in group order.
constexpr int kGradCh = 32;
constexpr int kGroups = 8;
__global__ void __launch_bounds__(kGradCh * kGroups)
linoss_matrix_grad_kernel(const float* __restrict__ partials, float2* __restrict__ grad_m, long long B,
                          long long P) {
  __shared__ double red[8][kGroups][kGradCh];
  const int cx = threadIdx.x % kGradCh, gy = threadIdx.x / kGradCh;
  const long long ch = (long long)blockIdx.x * kGradCh + cx;
  const long long N = B * P;
  double s[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) s[i] = 0.0;
  if (ch < P) {
#pragma unroll 2
    for (long long b = gy; b < B; b += kGroups) {
#pragma unroll
      for (int i = 0; i < 8; ++i) s[i] += (double)partials[(long long)i * N + b * P + ch];
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) red[i][gy][cx] = s[i];
  __syncthreads();
  if (gy != 0 || ch >= P) return;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    double t = red[i][0][cx];
    for (int k = 1; k < kGroups; ++k) t += red[i][k][cx];
    s[i] = t;
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) grad_m[ch * 4 + i] = make_float2((float)s[2 * i], (float)s[2 * i + 1]);
}

}  // namespace lgen
}  // namespace ossm_b200

extern "C" {

using namespace ossm_b200;

size_t ossm_b200_linoss_scan_backward_workspace_bytes(int64_t L, int64_t B, int64_t P) {
  if (L <= 0 || B <= 0 || P <= 0) return 0;
  return (size_t)8 * (size_t)B * (size_t)P * sizeof(float);
}

static int linoss_check(const char* fn, const void* m11, const void* m12, const void* m21, const void* m22,
                        int64_t L, int64_t B, int64_t P) {
  if (L < 0 || B < 0 || P < 0) { set_last_error("%s: negative extent", fn); return kErrInvalidArgument; }
  if (!m11 || !m12 || !m21 || !m22) { set_last_error("%s: null coefficient pointer", fn); return kErrInvalidArgument; }
  if ((B * P + lgen::kThreads - 1) / lgen::kThreads > 0x7fffffffLL) {
    set_last_error("%s: B*P too large", fn);
    return kErrInvalidArgument;
  }
  return kOk;
}

int ossm_b200_linoss_scan_forward(const void* m11, const void* m12, const void* m21, const void* m22,
                                  const void* b_seq, void* out, int64_t L, int64_t B, int64_t P,
                                  cudaStream_t stream) {
  if (int rc = linoss_check("linoss_scan_forward", m11, m12, m21, m22, L, B, P)) return rc;
  if (L == 0 || B == 0 || P == 0) return kOk;
  if (!b_seq || !out || (reinterpret_cast<uintptr_t>(b_seq) & 15u) || (reinterpret_cast<uintptr_t>(out) & 15u)) {
    set_last_error("linoss_scan_forward: null or misaligned b_seq/out (16-byte alignment required)");
    return kErrInvalidArgument;
  }
  const long long N = B * P;
  {
    CUtensorMap tm;
    memset(&tm, 0, sizeof(tm));
    if (lgen::staged_map(&tm, b_seq, L, N)) {
      const int ring = 4;
      const size_t smem = 1024 + (size_t)ring * lgen::kTileBytes;
      if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(lgen::linoss_forward_staged_kernel), smem)) return rc;
      const unsigned ctas = (unsigned)((N + lgen::kSeries - 1) / lgen::kSeries);
      lgen::linoss_forward_staged_kernel<<<ctas, lgen::kSeries, smem, stream>>>(
          tm, static_cast<const float2*>(m11), static_cast<const float2*>(m12), static_cast<const float2*>(m21),
          static_cast<const float2*>(m22), static_cast<float4*>(out), L, N, P, ring);
      return check_cuda(cudaGetLastError(), "linoss_forward_staged_kernel launch");
    }
  }
  const unsigned grid = (unsigned)((N + lgen::kThreads - 1) / lgen::kThreads);
  lgen::linoss_forward_kernel<<<grid, lgen::kThreads, 0, stream>>>(
      static_cast<const float2*>(m11), static_cast<const float2*>(m12), static_cast<const float2*>(m21),
      static_cast<const float2*>(m22), static_cast<const float4*>(b_seq), static_cast<float4*>(out), L, N, P);
  return check_cuda(cudaGetLastError(), "linoss_forward_kernel launch");
}

int ossm_b200_linoss_scan_backward(const void* m11, const void* m12, const void* m21, const void* m22,
                                   const void* states, const void* grad_out, void* grad_b, void* grad_m,
                                   void* workspace, size_t workspace_bytes, int64_t L, int64_t B, int64_t P,
                                   cudaStream_t stream) {
  if (int rc = linoss_check("linoss_scan_backward", m11, m12, m21, m22, L, B, P)) return rc;
  if (P == 0) return kOk;
  if (!grad_m) { set_last_error("linoss_scan_backward: null grad_m"); return kErrInvalidArgument; }
  if (L == 0 || B == 0) return check_cuda(cudaMemsetAsync(grad_m, 0, (size_t)P * 4 * 8, stream), "linoss memset");
  if (!states || !grad_out || !grad_b || (reinterpret_cast<uintptr_t>(states) & 15u) ||
      (reinterpret_cast<uintptr_t>(grad_out) & 15u) || (reinterpret_cast<uintptr_t>(grad_b) & 15u)) {
    set_last_error("linoss_scan_backward: null or misaligned states/grad_out/grad_b");
    return kErrInvalidArgument;
  }
  if (!workspace || workspace_bytes < ossm_b200_linoss_scan_backward_workspace_bytes(L, B, P)) {
    set_last_error("linoss_scan_backward: workspace too small");
    return kErrWorkspace;
  }
  const long long N = B * P;
  CUtensorMap tg, ts;
  memset(&tg, 0, sizeof(tg));
  memset(&ts, 0, sizeof(ts));
  if (lgen::staged_map(&tg, grad_out, L, N) && lgen::staged_map(&ts, states, L, N)) {
    const int ring = 3;
    const size_t smem = 1024 + (size_t)ring * 2 * lgen::kTileBytes;
    if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(lgen::linoss_backward_staged_kernel), smem)) return rc;
    const unsigned ctas = (unsigned)((N + lgen::kSeries - 1) / lgen::kSeries);
    lgen::linoss_backward_staged_kernel<<<ctas, lgen::kSeries, smem, stream>>>(
        tg, ts, static_cast<const float2*>(m11), static_cast<const float2*>(m12), static_cast<const float2*>(m21),
        static_cast<const float2*>(m22), static_cast<float4*>(grad_b), static_cast<float*>(workspace), L, N, P, ring);
    if (int rc = check_cuda(cudaGetLastError(), "linoss_backward_staged_kernel launch")) return rc;
  } else {
    const unsigned grid = (unsigned)((N + lgen::kThreads - 1) / lgen::kThreads);
    lgen::linoss_backward_kernel<<<grid, lgen::kThreads, 0, stream>>>(
        static_cast<const float2*>(m11), static_cast<const float2*>(m12), static_cast<const float2*>(m21),
        static_cast<const float2*>(m22), static_cast<const float4*>(states), static_cast<const float4*>(grad_out),
        static_cast<float4*>(grad_b), static_cast<float*>(workspace), L, N, P);
    if (int rc = check_cuda(cudaGetLastError(), "linoss_backward_kernel launch")) return rc;
  }
  const unsigned g2 = (unsigned)((P + lgen::kGradCh - 1) / lgen::kGradCh);
  lgen::linoss_matrix_grad_kernel<<<g2, lgen::kGradCh * lgen::kGroups, 0, stream>>>(static_cast<const float*>(workspace),
                                                          static_cast<float2*>(grad_m), B, P);
  return check_cuda(cudaGetLastError(), "linoss_matrix_grad_kernel launch");
}

}  // extern "C"
