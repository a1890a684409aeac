// Mamba selective scan, forward and backward, for sm_100a.
//
//   h_t[n] = exp(dt_t * A[d,n]) * h_{t-1}[n] + dt_t * B_t[n] * u_t
//   y_t    = sum_n C_t[n] * h_t[n]  (+ Dskip[d] * u_t)
//   out_t  = y_t * silu(z_t)                       (gate optional)
//
// Replaces the reference's wrapper + vendored kernels
// (src/ossm/csrc/selective_scan_cuda.cu:253-393, csrc/mamba/selective_scan_fwd_kernel.cuh,
// selective_scan_bwd_kernel.cuh) and its CPU kernels (selective_scan_cpu.cpp:78-360).
//
// Layout: u, dt, z, out [B, D, L] (time contiguous); A [D, N] fp32; B, C given
// time-contiguous as [B, N, L]; u/z/out/B/C in fp32 or bf16, dt and all state
// arithmetic in fp32.
//
// Decomposition.  A warp scans one (batch, channel) lane over a chunk of
// T = 32 * kItems steps: each thread owns kItems consecutive steps (one or two
// 16-byte loads per operand, fully coalesced across the warp), composes them
// locally, and a warp-shuffle scan over the 32 per-thread (decay, state) pairs
// plus the carry from the previous chunk gives every step its true state.  The
// N state dimensions are a serial loop inside the thread, so y_t, du_t and
// ddt_t are plain per-thread sums.  A CTA is kWarps warps x kCI channels of
// ONE batch element marching through the chunks together: the B_t/C_t tile of a
// chunk (N x T, converted to fp32) is staged in shared memory once and reused by
// all kWarps*kCI channels, and in the backward pass dB_t/dC_t are summed over
// those channels in shared memory before a single atomic add per (n, t).
//
// Backward walks the chunks right-to-left: it re-runs the forward scan of a
// chunk from the chunk-entry state saved by the forward pass, runs the adjoint
// recurrence  lam_t = a_t * (gy_t*C_t + lam_{t+1})  as a reverse warp scan, and
// forms all six gradients from registers.  Nothing of size L*N is ever stored.
#include "common.cuh"

#include <cuda_bf16.h>

#include "../../include/ossm_b200.h"

namespace ossm_b200 {
namespace sscan {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kCI = 8;                      // channels per warp
constexpr int kChannelsPerCta = kWarps * kCI;
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float sigmoidf(float x) { return 1.0f / (1.0f + ex2(-x * kLog2e)); }

template <typename IO>
__device__ __forceinline__ float io_load(const IO* p);
template <>
__device__ __forceinline__ float io_load<float>(const float* p) { return __ldg(p); }
template <>
__device__ __forceinline__ float io_load<__nv_bfloat16>(const __nv_bfloat16* p) {
  return __bfloat162float(*p);
}
template <typename IO>
__device__ __forceinline__ void io_store(IO* p, float v);
template <>
__device__ __forceinline__ void io_store<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void io_store<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// kItems consecutive elements of a row, zero past `limit` (elements left in the row).
template <typename IO, int kItems>
__device__ __forceinline__ void load_items(const IO* row, long long t0, long long L, bool vec_ok, float (&v)[kItems]) {
  if (vec_ok && t0 + kItems <= L) {
    if constexpr (sizeof(IO) == 4 && kItems % 4 == 0) {
#pragma unroll
      for (int q = 0; q < kItems / 4; ++q) {
        const float4 x = *reinterpret_cast<const float4*>(row + t0 + 4 * q);
        v[4 * q] = x.x; v[4 * q + 1] = x.y; v[4 * q + 2] = x.z; v[4 * q + 3] = x.w;
      }
      return;
    } else if constexpr (sizeof(IO) == 2 && kItems % 8 == 0) {
#pragma unroll
      for (int q = 0; q < kItems / 8; ++q) {
        const uint4 x = *reinterpret_cast<const uint4*>(row + t0 + 8 * q);
        const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          v[8 * q + 2 * i] = __uint_as_float(w[i] << 16);
          v[8 * q + 2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
      }
      return;
    }
  }
#pragma unroll
  for (int j = 0; j < kItems; ++j) v[j] = (t0 + j < L) ? io_load<IO>(row + t0 + j) : 0.0f;
}

template <typename IO, int kItems>
__device__ __forceinline__ void store_items(IO* row, long long t0, long long L, bool vec_ok, const float (&v)[kItems]) {
  if (vec_ok && t0 + kItems <= L) {
    if constexpr (sizeof(IO) == 4 && kItems % 4 == 0) {
#pragma unroll
      for (int q = 0; q < kItems / 4; ++q)
        *reinterpret_cast<float4*>(row + t0 + 4 * q) = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
      return;
    } else if constexpr (sizeof(IO) == 2 && kItems % 8 == 0) {
#pragma unroll
      for (int q = 0; q < kItems / 8; ++q) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const __nv_bfloat162 h = __floats2bfloat162_rn(v[8 * q + 2 * i], v[8 * q + 2 * i + 1]);
          w[i] = *reinterpret_cast<const uint32_t*>(&h);
        }
        *reinterpret_cast<uint4*>(row + t0 + 8 * q) = make_uint4(w[0], w[1], w[2], w[3]);
      }
      return;
    }
  }
#pragma unroll
  for (int j = 0; j < kItems; ++j)
    if (t0 + j < L) io_store<IO>(row + t0 + j, v[j]);
}

// Stages the [N][T] fp32 tile of a [B, N, L] operand for chunk starting at t_base.
template <typename IO>
__device__ __forceinline__ void stage_tile(float* dst, const IO* src_b, int N, int T, long long t_base, long long L) {
  const int total = N * T;
  for (int idx = threadIdx.x; idx < total; idx += kThreads) {
    const int n = idx / T, t = idx - n * T;
    const long long tt = t_base + t;
    dst[idx] = tt < L ? io_load<IO>(src_b + (long long)n * L + tt) : 0.0f;
  }
}

// Inclusive warp scan of affine maps x -> P*x + H (lane order = time order),
// returned as the EXCLUSIVE prefix (the map applied before this lane) and the
// total over the warp.
__device__ __forceinline__ void warp_scan_affine(float P, float H, int lane, float& Pex, float& Hex, float& Ptot,
                                                 float& Htot) {
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const float Pp = __shfl_up_sync(0xffffffffu, P, off);
    const float Hp = __shfl_up_sync(0xffffffffu, H, off);
    if (lane >= off) {
      H = fmaf(P, Hp, H);
      P = P * Pp;
    }
  }
  Ptot = __shfl_sync(0xffffffffu, P, 31);
  Htot = __shfl_sync(0xffffffffu, H, 31);
  Pex = __shfl_up_sync(0xffffffffu, P, 1);
  Hex = __shfl_up_sync(0xffffffffu, H, 1);
  if (lane == 0) { Pex = 1.0f; Hex = 0.0f; }
}

// Same in reverse time order: suffix maps (lane 31 is applied first).
__device__ __forceinline__ void warp_scan_affine_rev(float P, float H, int lane, float& Pex, float& Hex,
                                                     float& Ptot, float& Htot) {
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const float Pp = __shfl_down_sync(0xffffffffu, P, off);
    const float Hp = __shfl_down_sync(0xffffffffu, H, off);
    if (lane + off < 32) {
      H = fmaf(P, Hp, H);
      P = P * Pp;
    }
  }
  Ptot = __shfl_sync(0xffffffffu, P, 0);
  Htot = __shfl_sync(0xffffffffu, H, 0);
  Pex = __shfl_down_sync(0xffffffffu, P, 1);
  Hex = __shfl_down_sync(0xffffffffu, H, 1);
  if (lane == 31) { Pex = 1.0f; Hex = 0.0f; }
}

struct Params {
  const void* u;
  const float* dt;
  const float* A;
  const void* Bm;   // [B, N, L]
  const void* Cm;   // [B, N, L]
  const void* z;    // nullable
  const float* Dskip;  // nullable, [D]
  void* out;
  float* chunk_states;  // [B, D, nchunks, N], state entering each chunk (nullable in forward)
  // backward only
  const void* dout;
  void* du;
  float* ddt;
  void* dz;
  float* dB;  // [B, N, L] fp32, zero-initialised by the host entry
  float* dC;
  float* dA_part;  // [B, D, N]
  float* dD_part;  // [B, D] (nullable)
  long long B, D, L, N;
  bool vec_ok;
};

// Shared memory (floats): Bs[N*T] | Cs[N*T] | carry[kWarps*kCI*N]
template <typename IO, int kItems>
__global__ void __launch_bounds__(kThreads) sscan_forward_kernel(Params p) {
  constexpr int T = 32 * kItems;
  extern __shared__ __align__(16) float smem[];
  const int N = (int)p.N;
  float* Bs = smem;
  float* Cs = Bs + N * T;
  float* carry = Cs + N * T;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long b = blockIdx.y;
  const long long d0 = (long long)blockIdx.x * kChannelsPerCta + warp * kCI;
  const long long nchunks = (p.L + T - 1) / T;
  const IO* Bm_b = static_cast<const IO*>(p.Bm) + b * p.N * p.L;
  const IO* Cm_b = static_cast<const IO*>(p.Cm) + b * p.N * p.L;

  for (int i = threadIdx.x; i < kWarps * kCI * N; i += kThreads) carry[i] = 0.0f;

  for (long long c = 0; c < nchunks; ++c) {
    const long long t_base = c * T;
    __syncthreads();  // everyone is done with the previous tiles (and carry init)
    stage_tile<IO>(Bs, Bm_b, N, T, t_base, p.L);
    stage_tile<IO>(Cs, Cm_b, N, T, t_base, p.L);
    __syncthreads();
    const long long t0 = t_base + (long long)lane * kItems;
#pragma unroll 1
    for (int ci = 0; ci < kCI; ++ci) {
      const long long d = d0 + ci;
      if (d >= p.D) break;  // warp-uniform
      const long long row = (b * p.D + d) * p.L;
      float u[kItems], dt[kItems], y[kItems];
      load_items<IO, kItems>(static_cast<const IO*>(p.u) + row, t0, p.L, p.vec_ok, u);
      load_items<float, kItems>(p.dt + row, t0, p.L, p.vec_ok, dt);
      float dtu[kItems];
#pragma unroll
      for (int j = 0; j < kItems; ++j) { dtu[j] = dt[j] * u[j]; y[j] = 0.0f; }
      float* cw = carry + (warp * kCI + ci) * N;
      float* cs_out = p.chunk_states ? p.chunk_states + ((b * p.D + d) * nchunks + c) * p.N : nullptr;
#pragma unroll 1
      for (int n = 0; n < N; ++n) {
        const float A2 = __ldg(p.A + d * p.N + n) * kLog2e;
        const float* Bn = Bs + n * T + lane * kItems;
        const float* Cn = Cs + n * T + lane * kItems;
        float hloc[kItems], cp[kItems];
        float P = 1.0f, H = 0.0f;
#pragma unroll
        for (int j = 0; j < kItems; ++j) {
          const float a = ex2(dt[j] * A2);
          H = fmaf(a, H, dtu[j] * Bn[j]);
          P *= a;
          hloc[j] = H;
          cp[j] = P;
        }
        const float h_in = cw[n];  // read before the scan: its shuffles order this read before lane 0's update
        float Pex, Hex, Ptot, Htot;
        warp_scan_affine(P, H, lane, Pex, Hex, Ptot, Htot);
        const float hstart = fmaf(Pex, h_in, Hex);
#pragma unroll
        for (int j = 0; j < kItems; ++j) y[j] = fmaf(fmaf(cp[j], hstart, hloc[j]), Cn[j], y[j]);
        if (lane == 0) {
          if (cs_out) cs_out[n] = h_in;
          cw[n] = fmaf(Ptot, h_in, Htot);
        }
      }
      if (p.Dskip) {
        const float ds = __ldg(p.Dskip + d);
#pragma unroll
        for (int j = 0; j < kItems; ++j) y[j] = fmaf(ds, u[j], y[j]);
      }
      if (p.z) {
        float zz[kItems];
        load_items<IO, kItems>(static_cast<const IO*>(p.z) + row, t0, p.L, p.vec_ok, zz);
#pragma unroll
        for (int j = 0; j < kItems; ++j) y[j] *= zz[j] * sigmoidf(zz[j]);
      }
      store_items<IO, kItems>(static_cast<IO*>(p.out) + row, t0, p.L, p.vec_ok, y);
      __syncwarp();  // cw[] written by lane 0 is read by all lanes in the next chunk
    }
  }
}

// Shared memory (floats):
//   Bs[N*T] | Cs[N*T] | dBs[N*T] | dCs[N*T] | red[2][kWarps][T] | lam[kWarps*kCI*N] | dAacc[kWarps*kCI*N]
//   | dDacc[kWarps*kCI]
template <typename IO, int kItems>
__global__ void __launch_bounds__(kThreads) sscan_backward_kernel(Params p) {
  constexpr int T = 32 * kItems;
  extern __shared__ __align__(16) float smem[];
  const int N = (int)p.N;
  float* Bs = smem;
  float* Cs = Bs + N * T;
  float* dBs = Cs + N * T;
  float* dCs = dBs + N * T;
  float* red = dCs + N * T;                 // [2][kWarps][T]
  float* lam = red + 2 * kWarps * T;        // adjoint carried from the later chunk
  float* dAacc = lam + kWarps * kCI * N;
  float* dDacc = dAacc + kWarps * kCI * N;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long b = blockIdx.y;
  const long long d0 = (long long)blockIdx.x * kChannelsPerCta + warp * kCI;
  const long long nchunks = (p.L + T - 1) / T;
  const IO* Bm_b = static_cast<const IO*>(p.Bm) + b * p.N * p.L;
  const IO* Cm_b = static_cast<const IO*>(p.Cm) + b * p.N * p.L;
  // number of channel iterations in which at least one warp of this CTA is active
  const long long ch_left = p.D - (long long)blockIdx.x * kChannelsPerCta;

  for (int i = threadIdx.x; i < kWarps * kCI * N; i += kThreads) { lam[i] = 0.0f; dAacc[i] = 0.0f; }
  for (int i = threadIdx.x; i < kWarps * kCI; i += kThreads) dDacc[i] = 0.0f;

  for (long long c = nchunks - 1; c >= 0; --c) {
    const long long t_base = c * T;
    __syncthreads();
    stage_tile<IO>(Bs, Bm_b, N, T, t_base, p.L);
    stage_tile<IO>(Cs, Cm_b, N, T, t_base, p.L);
    for (int i = threadIdx.x; i < 2 * N * T; i += kThreads) dBs[i] = 0.0f;  // dBs and dCs are adjacent
    __syncthreads();
    const long long t0 = t_base + (long long)lane * kItems;
#pragma unroll 1
    for (int ci = 0; ci < kCI; ++ci) {
      if ((long long)ci >= ch_left) break;                   // CTA-uniform: no channel left in any warp
      const long long d = d0 + ci;
      const bool active = d < p.D;                            // warp-uniform
      const long long row = active ? (b * p.D + d) * p.L : 0;
      const long long tl = active ? p.L : 0;                  // inactive warps load nothing, contribute zeros
      float u[kItems], dt[kItems], gy[kItems], dtu[kItems];
      float dus[kItems], ddts[kItems], y[kItems];
      load_items<IO, kItems>(static_cast<const IO*>(p.u) + row, t0, tl, p.vec_ok, u);
      load_items<float, kItems>(p.dt + row, t0, tl, p.vec_ok, dt);
      load_items<IO, kItems>(static_cast<const IO*>(p.dout) + row, t0, tl, p.vec_ok, gy);
      float zz[kItems], dout_raw[kItems];
      if (p.z) {
        load_items<IO, kItems>(static_cast<const IO*>(p.z) + row, t0, tl, p.vec_ok, zz);
#pragma unroll
        for (int j = 0; j < kItems; ++j) { dout_raw[j] = gy[j]; gy[j] *= zz[j] * sigmoidf(zz[j]); }
      }
#pragma unroll
      for (int j = 0; j < kItems; ++j) { dtu[j] = dt[j] * u[j]; dus[j] = 0.f; ddts[j] = 0.f; y[j] = 0.f; }
      const int slot = (warp * kCI + ci) * N;
      const float* cs_in = active ? p.chunk_states + ((b * p.D + d) * nchunks + c) * p.N : nullptr;
#pragma unroll 1
      for (int n = 0; n < N; ++n) {
        const float An = active ? __ldg(p.A + d * p.N + n) : 0.0f;
        const float A2 = An * kLog2e;
        const float* Bn = Bs + n * T + lane * kItems;
        const float* Cn = Cs + n * T + lane * kItems;
        float a[kItems], hloc[kItems], cp[kItems], Bv[kItems], Cv[kItems];
        float P = 1.0f, H = 0.0f;
#pragma unroll
        for (int j = 0; j < kItems; ++j) {
          Bv[j] = Bn[j];
          Cv[j] = Cn[j];
          a[j] = ex2(dt[j] * A2);
          H = fmaf(a[j], H, dtu[j] * Bv[j]);
          P *= a[j];
          hloc[j] = H;
          cp[j] = P;
        }
        float Pex, Hex, Ptot, Htot;
        warp_scan_affine(P, H, lane, Pex, Hex, Ptot, Htot);
        const float h_in = active ? __ldg(cs_in + n) : 0.0f;
        const float hstart = fmaf(Pex, h_in, Hex);
        // adjoint: lam_t = a_t * (gy_t*C_t + lam_{t+1}), right to left
        float lloc[kItems], cq[kItems];
        float Q = 1.0f, R = 0.0f;
#pragma unroll
        for (int j = kItems - 1; j >= 0; --j) {
          R = a[j] * fmaf(gy[j], Cv[j], R);
          Q *= a[j];
          lloc[j] = R;
          cq[j] = Q;
        }
        const float lam_in = lam[slot + n];                // lam entering the chunk from the right
        float Qex, Rex, Qtot, Rtot;
        warp_scan_affine_rev(Q, R, lane, Qex, Rex, Qtot, Rtot);
        const float lstart = fmaf(Qex, lam_in, Rex);       // lam_{t+1} for this lane's last item
        float dA_t = 0.0f;
        float dBv[kItems], dCv[kItems];
#pragma unroll
        for (int j = kItems - 1; j >= 0; --j) {
          const float h = fmaf(cp[j], hstart, hloc[j]);
          const float hprev = j > 0 ? fmaf(cp[j - 1], hstart, hloc[j - 1]) : hstart;
          const float lam_next = j < kItems - 1 ? fmaf(cq[j + 1], lstart, lloc[j + 1]) : lstart;
          const float G = fmaf(gy[j], Cv[j], lam_next);
          const float q = (G * a[j]) * hprev;              // G * a_t * h_{t-1}
          y[j] = fmaf(h, Cv[j], y[j]);
          dCv[j] = gy[j] * h;
          dBv[j] = G * dtu[j];
          dus[j] = fmaf(G, Bv[j], dus[j]);
          dA_t = fmaf(q, dt[j], dA_t);
          ddts[j] = fmaf(q, An, ddts[j]);
        }
        // carries for the next (earlier) chunk and per-channel dA
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) dA_t += __shfl_xor_sync(0xffffffffu, dA_t, off);
        if (lane == 0) {
          lam[slot + n] = fmaf(Qtot, lam_in, Rtot);
          dAacc[slot + n] += dA_t;
        }
        // dB_t[n], dC_t[n]: sum over the kWarps channels processed in this iteration
        // (single staging buffer, guarded by the two barriers below)
        float* redB = red + warp * T + lane * kItems;
        float* redC = red + kWarps * T + warp * T + lane * kItems;
#pragma unroll
        for (int j = 0; j < kItems; ++j) { redB[j] = dBv[j]; redC[j] = dCv[j]; }
        __syncthreads();
        for (int i = threadIdx.x; i < 2 * T; i += kThreads) {
          const int which = i / T, t = i - which * T;
          const float* src = red + which * kWarps * T + t;
          float s = 0.0f;
#pragma unroll
          for (int w = 0; w < kWarps; ++w) s += src[w * T];
          float* acc = (which ? dCs : dBs) + n * T + t;
          *acc += s;
        }
        __syncthreads();
      }
      if (active) {
        // du_t = dt_t * sum_n G*B (+ gy*Dskip) ; ddt_t = sum_n q*A + u_t * sum_n G*B
        float ds = 0.0f, dD_t = 0.0f;
        if (p.Dskip) ds = __ldg(p.Dskip + d);
        float duv[kItems], ddv[kItems];
#pragma unroll
        for (int j = 0; j < kItems; ++j) {
          duv[j] = fmaf(dt[j], dus[j], gy[j] * ds);
          ddv[j] = fmaf(u[j], dus[j], ddts[j]);
          dD_t = fmaf(gy[j], u[j], dD_t);
        }
        store_items<IO, kItems>(static_cast<IO*>(p.du) + row, t0, p.L, p.vec_ok, duv);
        store_items<float, kItems>(p.ddt + row, t0, p.L, p.vec_ok, ddv);
        if (p.z) {
          float dzv[kItems];
#pragma unroll
          for (int j = 0; j < kItems; ++j) {
            const float sg = sigmoidf(zz[j]);
            const float yy = fmaf(ds, u[j], y[j]);
            dzv[j] = dout_raw[j] * yy * (sg * (1.0f + zz[j] * (1.0f - sg)));
          }
          store_items<IO, kItems>(static_cast<IO*>(p.dz) + row, t0, p.L, p.vec_ok, dzv);
        }
        if (p.dD_part) {
#pragma unroll
          for (int off = 16; off > 0; off >>= 1) dD_t += __shfl_xor_sync(0xffffffffu, dD_t, off);
          if (lane == 0) dDacc[warp * kCI + ci] += dD_t;
        }
      }
      __syncwarp();
    }
    // flush this chunk's dB/dC sums (over this CTA's channels) to global
    __syncthreads();
    for (int i = threadIdx.x; i < N * T; i += kThreads) {
      const int n = i / T, t = i - n * T;
      const long long tt = t_base + t;
      if (tt < p.L) {
        atomicAdd(p.dB + (b * p.N + n) * p.L + tt, dBs[i]);
        atomicAdd(p.dC + (b * p.N + n) * p.L + tt, dCs[i]);
      }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < kWarps * kCI * N; i += kThreads) {
    const int wc = i / N, n = i - wc * N;
    const long long d = (long long)blockIdx.x * kChannelsPerCta + wc;
    if (d < p.D) p.dA_part[(b * p.D + d) * p.N + n] = dAacc[i];
  }
  if (p.dD_part) {
    for (int i = threadIdx.x; i < kWarps * kCI; i += kThreads) {
      const long long d = (long long)blockIdx.x * kChannelsPerCta + i;
      if (d < p.D) p.dD_part[b * p.D + d] = dDacc[i];
    }
  }
}

// dA[d,n] = sum_b dA_part[b,d,n] ; dD[d] = sum_b dD_part[b,d]  (fixed order, double)
__global__ void sscan_reduce_batch_kernel(const float* __restrict__ part, float* __restrict__ out, long long B,
                                          long long M) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= M) return;
  double s = 0.0;
  for (long long b = 0; b < B; ++b) s += (double)part[b * M + i];
  out[i] = (float)s;
}

static int items_for(long long N) {
  if (N <= 16) return 8;
  if (N <= 32) return 4;
  if (N <= 64) return 2;
  return 1;
}

template <typename K>
static int set_smem(K kernel, size_t bytes) {
  return check_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes),
                    "cudaFuncSetAttribute(max dynamic smem)");
}

template <typename IO, int kItems>
static int launch_fwd(const Params& p, cudaStream_t stream) {
  const int T = 32 * kItems;
  const size_t smem = sizeof(float) * (2 * (size_t)p.N * T + (size_t)kWarps * kCI * p.N);
  if (smem > 200 * 1024) { set_last_error("selective_scan_forward: d_state too large"); return kErrUnsupported; }
  if (int rc = set_smem(sscan_forward_kernel<IO, kItems>, smem)) return rc;
  dim3 grid((unsigned)((p.D + kChannelsPerCta - 1) / kChannelsPerCta), (unsigned)p.B);
  sscan_forward_kernel<IO, kItems><<<grid, kThreads, smem, stream>>>(p);
  return check_cuda(cudaGetLastError(), "sscan_forward_kernel launch");
}

template <typename IO, int kItems>
static int launch_bwd(const Params& p, cudaStream_t stream) {
  const int T = 32 * kItems;
  const size_t smem = sizeof(float) * (4 * (size_t)p.N * T + 2 * (size_t)kWarps * T +
                                       2 * (size_t)kWarps * kCI * p.N + kWarps * kCI);
  if (smem > 200 * 1024) { set_last_error("selective_scan_backward: d_state too large"); return kErrUnsupported; }
  if (int rc = set_smem(sscan_backward_kernel<IO, kItems>, smem)) return rc;
  dim3 grid((unsigned)((p.D + kChannelsPerCta - 1) / kChannelsPerCta), (unsigned)p.B);
  sscan_backward_kernel<IO, kItems><<<grid, kThreads, smem, stream>>>(p);
  return check_cuda(cudaGetLastError(), "sscan_backward_kernel launch");
}

template <typename IO>
static int dispatch_items(bool backward, const Params& p, cudaStream_t stream) {
  switch (items_for(p.N)) {
    case 8: return backward ? launch_bwd<IO, 8>(p, stream) : launch_fwd<IO, 8>(p, stream);
    case 4: return backward ? launch_bwd<IO, 4>(p, stream) : launch_fwd<IO, 4>(p, stream);
    case 2: return backward ? launch_bwd<IO, 2>(p, stream) : launch_fwd<IO, 2>(p, stream);
    default: return backward ? launch_bwd<IO, 1>(p, stream) : launch_fwd<IO, 1>(p, stream);
  }
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace sscan
}  // namespace ossm_b200

extern "C" {

using namespace ossm_b200;

int ossm_b200_selective_scan_chunk(int64_t N) { return 32 * sscan::items_for(N); }

size_t ossm_b200_selective_scan_state_bytes(int64_t B, int64_t D, int64_t L, int64_t N) {
  if (B <= 0 || D <= 0 || L <= 0 || N <= 0) return 0;
  const int64_t T = 32 * sscan::items_for(N);
  return (size_t)B * D * ((L + T - 1) / T) * N * sizeof(float);
}

size_t ossm_b200_selective_scan_backward_workspace_bytes(int64_t B, int64_t D, int64_t L, int64_t N) {
  if (B <= 0 || D <= 0 || L <= 0 || N <= 0) return 0;
  return (size_t)B * D * (N + 1) * sizeof(float);
}

static int sscan_check(const char* fn, const void* u, const float* dt, const float* A, const void* Bm,
                       const void* Cm, int64_t B, int64_t D, int64_t L, int64_t N, int io_dtype) {
  if (B < 0 || D < 0 || L < 0 || N < 0) { set_last_error("%s: negative extent", fn); return kErrInvalidArgument; }
  if (io_dtype != OSSM_B200_DTYPE_F32 && io_dtype != OSSM_B200_DTYPE_BF16) {
    set_last_error("%s: unknown io dtype %d", fn, io_dtype);
    return kErrInvalidArgument;
  }
  if (N > 128) { set_last_error("%s: d_state > 128 is not supported", fn); return kErrUnsupported; }
  if (B > 65535) { set_last_error("%s: batch > 65535 is not supported", fn); return kErrUnsupported; }
  if (B == 0 || D == 0 || L == 0 || N == 0) return kOk;
  if (!u || !dt || !A || !Bm || !Cm) { set_last_error("%s: null input pointer", fn); return kErrInvalidArgument; }
  return kOk;
}

int ossm_b200_selective_scan_forward(const void* u, const float* dt, const float* A, const void* Bm, const void* Cm,
                                     const void* z, const float* Dskip, void* out, float* chunk_states, int64_t B,
                                     int64_t D, int64_t L, int64_t N, int io_dtype, cudaStream_t stream) {
  if (int rc = sscan_check("selective_scan_forward", u, dt, A, Bm, Cm, B, D, L, N, io_dtype)) return rc;
  if (B == 0 || D == 0 || L == 0) return kOk;
  if (!out) { set_last_error("selective_scan_forward: null out"); return kErrInvalidArgument; }
  if (N == 0) {
    set_last_error("selective_scan_forward: d_state must be positive");
    return kErrInvalidArgument;
  }
  sscan::Params p{};
  p.u = u; p.dt = dt; p.A = A; p.Bm = Bm; p.Cm = Cm; p.z = z; p.Dskip = Dskip; p.out = out;
  p.chunk_states = chunk_states;
  p.B = B; p.D = D; p.L = L; p.N = N;
  const int es = io_dtype == OSSM_B200_DTYPE_F32 ? 4 : 2;
  p.vec_ok = sscan::aligned16(u) && sscan::aligned16(dt) && sscan::aligned16(out) && (!z || sscan::aligned16(z)) &&
             (L * es) % 16 == 0 && (L * 4) % 16 == 0;
  return io_dtype == OSSM_B200_DTYPE_F32 ? sscan::dispatch_items<float>(false, p, stream)
                                         : sscan::dispatch_items<__nv_bfloat16>(false, p, stream);
}

int ossm_b200_selective_scan_backward(const void* u, const float* dt, const float* A, const void* Bm,
                                      const void* Cm, const void* z, const float* Dskip, const void* dout,
                                      const float* chunk_states, void* du, float* ddt, float* dA, float* dB,
                                      float* dC, void* dz, float* dD, void* workspace, size_t workspace_bytes,
                                      int64_t B, int64_t D, int64_t L, int64_t N, int io_dtype,
                                      cudaStream_t stream) {
  if (int rc = sscan_check("selective_scan_backward", u, dt, A, Bm, Cm, B, D, L, N, io_dtype)) return rc;
  if (D == 0 || N == 0) return kOk;
  if (!dA) { set_last_error("selective_scan_backward: null dA"); return kErrInvalidArgument; }
  if (int rc = check_cuda(cudaMemsetAsync(dA, 0, (size_t)D * N * sizeof(float), stream), "memset dA")) return rc;
  if (dD) if (int rc = check_cuda(cudaMemsetAsync(dD, 0, (size_t)D * sizeof(float), stream), "memset dD")) return rc;
  if (B == 0 || L == 0) return kOk;
  if (!dout || !chunk_states || !du || !ddt || !dB || !dC || (z && !dz) || (Dskip && !dD)) {
    set_last_error("selective_scan_backward: null pointer among dout/chunk_states/du/ddt/dB/dC/dz/dD");
    return kErrInvalidArgument;
  }
  if (!workspace || workspace_bytes < ossm_b200_selective_scan_backward_workspace_bytes(B, D, L, N)) {
    set_last_error("selective_scan_backward: workspace too small");
    return kErrWorkspace;
  }
  const size_t bc_bytes = (size_t)B * N * L * sizeof(float);
  if (int rc = check_cuda(cudaMemsetAsync(dB, 0, bc_bytes, stream), "memset dB")) return rc;
  if (int rc = check_cuda(cudaMemsetAsync(dC, 0, bc_bytes, stream), "memset dC")) return rc;
  sscan::Params p{};
  p.u = u; p.dt = dt; p.A = A; p.Bm = Bm; p.Cm = Cm; p.z = z; p.Dskip = Dskip;
  p.chunk_states = const_cast<float*>(chunk_states);
  p.dout = dout; p.du = du; p.ddt = ddt; p.dz = dz; p.dB = dB; p.dC = dC;
  p.dA_part = static_cast<float*>(workspace);
  p.dD_part = Dskip ? p.dA_part + (size_t)B * D * N : nullptr;
  p.B = B; p.D = D; p.L = L; p.N = N;
  const int es = io_dtype == OSSM_B200_DTYPE_F32 ? 4 : 2;
  p.vec_ok = sscan::aligned16(u) && sscan::aligned16(dt) && sscan::aligned16(dout) && sscan::aligned16(du) &&
             sscan::aligned16(ddt) && (!z || (sscan::aligned16(z) && sscan::aligned16(dz))) &&
             (L * es) % 16 == 0 && (L * 4) % 16 == 0;
  int rc = io_dtype == OSSM_B200_DTYPE_F32 ? sscan::dispatch_items<float>(true, p, stream)
                                           : sscan::dispatch_items<__nv_bfloat16>(true, p, stream);
  if (rc) return rc;
  const long long M = D * N;
  sscan::sscan_reduce_batch_kernel<<<(unsigned)((M + 255) / 256), 256, 0, stream>>>(p.dA_part, dA, B, M);
  if (int rc2 = check_cuda(cudaGetLastError(), "sscan_reduce_batch_kernel launch")) return rc2;
  if (p.dD_part) {
    sscan::sscan_reduce_batch_kernel<<<(unsigned)((D + 255) / 256), 256, 0, stream>>>(p.dD_part, dD, B, D);
    if (int rc2 = check_cuda(cudaGetLastError(), "sscan_reduce_batch_kernel launch")) return rc2;
  }
  return kOk;
}

}  // extern "C"
