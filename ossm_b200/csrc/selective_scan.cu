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
OSSM_B200_STATUS_ACCESSOR(status_selective_scan)
namespace sscan {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kCI = 8;                      // channels per warp
constexpr float kLog2e = 1.4426950408889634f;
constexpr int kMaxState = 256;              // the reference kernels' MAX_DSTATE (csrc/mamba/selective_scan_common.h:41)
constexpr int kStateTile = 64;              // backward: states per pass over a chunk when d_state is larger

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float sigmoidf(float x) { return 1.0f / (1.0f + ex2(-x * kLog2e)); }

__device__ __forceinline__ float lg2(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Step size used by the scan from the raw one: raw + bias, through softplus when asked (identity above
// 20, as in the vendored Mamba kernel, selective_scan_fwd_kernel.cuh:123-161).  Small arguments use
// log1p(e) = e - e^2/2 so that tiny steps keep their relative accuracy.
__device__ __forceinline__ float step_transform(float raw, float bias, bool softplus) {
  float x = raw + bias;
  if (softplus && x <= 20.0f) {
    const float e = ex2(x * kLog2e);
    x = e < 1e-4f ? e * fmaf(-0.5f, e, 1.0f) : 0.6931471805599453f * lg2(1.0f + e);
  }
  return x;
}
// d(step)/d(raw) expressed through the transformed step: sigmoid(x) = 1 - exp(-softplus(x)).
__device__ __forceinline__ float step_transform_grad(float dt, bool softplus) {
  if (!softplus) return 1.0f;
  return dt < 1e-3f ? dt * fmaf(-0.5f, dt, 1.0f) : 1.0f - ex2(-dt * kLog2e);
}


// Pair arithmetic on (state 2p, state 2p+1): packed f32x2 instructions (measured 13 %
// faster in the backward than the scalar forms, which remain selectable for comparison).
#ifndef OSSM_SSCAN_PACKED
#define OSSM_SSCAN_PACKED 1
#endif
__device__ __forceinline__ float2 p2fma(float2 a, float2 b, float2 c) {
#if OSSM_SSCAN_PACKED
  return __ffma2_rn(a, b, c);
#else
  return make_float2(fmaf(a.x, b.x, c.x), fmaf(a.y, b.y, c.y));
#endif
}
__device__ __forceinline__ float2 p2mul(float2 a, float2 b) {
#if OSSM_SSCAN_PACKED
  return __fmul2_rn(a, b);
#else
  return make_float2(a.x * b.x, a.y * b.y);
#endif
}
__device__ __forceinline__ float2 p2add(float2 a, float2 b) {
#if OSSM_SSCAN_PACKED
  return __fadd2_rn(a, b);
#else
  return make_float2(a.x + b.x, a.y + b.y);
#endif
}

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

// ---------------------------------------------------------------------------
// Shared-memory tiles.  States are processed two at a time (n = 2p, 2p+1) so that
// every per-(step, state) operation is one packed f32x2 instruction on a
// (state 2p, state 2p+1) register pair.  A tile holds, per state pair, the T
// steps of a chunk as float2 (one value per state); a thread's kItems steps are
// spread over kItems/2 float4 slots laid out [pair][slot][lane][4] so that the 32
// lanes of a warp read 512 contiguous bytes per 16-byte access (no bank
// conflicts).  An odd last state is padded with a zero partner.
// ---------------------------------------------------------------------------
template <int kItems>
__device__ __forceinline__ int tile_index(int pair, int t_local, int s) {
  if constexpr (kItems >= 2) {
    const int lane = t_local / kItems, j = t_local % kItems;
    return ((pair * (kItems / 2) + (j >> 1)) * 32 + lane) * 4 + (j & 1) * 2 + s;
  } else {
    return (pair * 32 + t_local) * 2 + s;
  }
}

template <int kItems>
__device__ __forceinline__ void lds_pairs(const float* tile, int pair, int lane, float2 (&v)[kItems]) {
  if constexpr (kItems >= 2) {
#pragma unroll
    for (int q = 0; q < kItems / 2; ++q) {
      const float4 x = reinterpret_cast<const float4*>(tile)[(pair * (kItems / 2) + q) * 32 + lane];
      v[2 * q] = make_float2(x.x, x.y);
      v[2 * q + 1] = make_float2(x.z, x.w);
    }
  } else {
    v[0] = reinterpret_cast<const float2*>(tile)[pair * 32 + lane];
  }
}

template <int kItems>
__device__ __forceinline__ void sts_pairs(float* tile, int pair, int lane, const float2 (&v)[kItems]) {
  if constexpr (kItems >= 2) {
#pragma unroll
    for (int q = 0; q < kItems / 2; ++q)
      reinterpret_cast<float4*>(tile)[(pair * (kItems / 2) + q) * 32 + lane] =
          make_float4(v[2 * q].x, v[2 * q].y, v[2 * q + 1].x, v[2 * q + 1].y);
  } else {
    reinterpret_cast<float2*>(tile)[pair * 32 + lane] = v[0];
  }
}

// Stages the chunk tile of a [B, N, L] operand (converted to fp32) for the chunk
// starting at t_base; global reads are coalesced along time.
// `src_b` points at the first of the N rows to stage (a tile of the states when they are processed in tiles).
template <typename IO, int kItems>
__device__ __forceinline__ void stage_tile(float* dst, const IO* src_b, int N, long long t_base, long long L) {
  constexpr int T = 32 * kItems;
  const int rows = 2 * ((N + 1) / 2);
  for (int idx = threadIdx.x; idx < rows * T; idx += kThreads) {
    const int n = idx / T, t = idx - n * T;
    const long long tt = t_base + t;
    const float v = (n < N && tt < L) ? io_load<IO>(src_b + (long long)n * L + tt) : 0.0f;
    dst[tile_index<kItems>(n >> 1, t, n & 1)] = v;
  }
}

__device__ __forceinline__ float2 shfl_up2(float2 v, int off) {
  return make_float2(__shfl_up_sync(0xffffffffu, v.x, off), __shfl_up_sync(0xffffffffu, v.y, off));
}
__device__ __forceinline__ float2 shfl_down2(float2 v, int off) {
  return make_float2(__shfl_down_sync(0xffffffffu, v.x, off), __shfl_down_sync(0xffffffffu, v.y, off));
}
__device__ __forceinline__ float2 shfl2(float2 v, int src) {
  return make_float2(__shfl_sync(0xffffffffu, v.x, src), __shfl_sync(0xffffffffu, v.y, src));
}

// Warp scan of affine maps x -> P*x + H in time order (lane 0 first), two states
// at once.  Returns the EXCLUSIVE prefix map of each lane and the map of the
// whole warp.
__device__ __forceinline__ void warp_scan_affine(float2 P, float2 H, int lane, float2& Pex, float2& Hex,
                                                 float2& Ptot, float2& Htot) {
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const float2 Pp = shfl_up2(P, off);
    const float2 Hp = shfl_up2(H, off);
    if (lane >= off) {
      H = p2fma(P, Hp, H);
      P = p2mul(P, Pp);
    }
  }
  Ptot = shfl2(P, 31);
  Htot = shfl2(H, 31);
  Pex = shfl_up2(P, 1);
  Hex = shfl_up2(H, 1);
  if (lane == 0) { Pex = make_float2(1.f, 1.f); Hex = make_float2(0.f, 0.f); }
}

// Same in reverse time order (lane 31 is applied first).
__device__ __forceinline__ void warp_scan_affine_rev(float2 P, float2 H, int lane, float2& Pex, float2& Hex,
                                                     float2& Ptot, float2& Htot) {
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const float2 Pp = shfl_down2(P, off);
    const float2 Hp = shfl_down2(H, off);
    if (lane + off < 32) {
      H = p2fma(P, Hp, H);
      P = p2mul(P, Pp);
    }
  }
  Ptot = shfl2(P, 0);
  Htot = shfl2(H, 0);
  Pex = shfl_down2(P, 1);
  Hex = shfl_down2(H, 1);
  if (lane == 31) { Pex = make_float2(1.f, 1.f); Hex = make_float2(0.f, 0.f); }
}

// Forward (P,H: lane 0 first) and reverse (Q,R: lane 31 first) scans in the same
// five rounds, so their shuffle latencies overlap.
__device__ __forceinline__ void warp_scan_dual(float2 P, float2 H, float2 Q, float2 R, int lane, float2& Pex,
                                               float2& Hex, float2& Qex, float2& Rex, float2& Qtot,
                                               float2& Rtot) {
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const float2 Pp = shfl_up2(P, off), Hp = shfl_up2(H, off);
    const float2 Qp = shfl_down2(Q, off), Rp = shfl_down2(R, off);
    if (lane >= off) {
      H = p2fma(P, Hp, H);
      P = p2mul(P, Pp);
    }
    if (lane + off < 32) {
      R = p2fma(Q, Rp, R);
      Q = p2mul(Q, Qp);
    }
  }
  Qtot = shfl2(Q, 0);
  Rtot = shfl2(R, 0);
  Pex = shfl_up2(P, 1);
  Hex = shfl_up2(H, 1);
  Qex = shfl_down2(Q, 1);
  Rex = shfl_down2(R, 1);
  if (lane == 0) { Pex = make_float2(1.f, 1.f); Hex = make_float2(0.f, 0.f); }
  if (lane == 31) { Qex = make_float2(1.f, 1.f); Rex = make_float2(0.f, 0.f); }
}

__device__ __forceinline__ float2 splat(float v) { return make_float2(v, v); }

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
  const float* delta_bias;  // [D] (nullable): dt = raw + delta_bias[d]
  int delta_softplus;       // dt = softplus(raw + bias)
  float* dbias_part;        // [B, D] (nullable), backward only
  long long B, D, L, N;
  long long nstates;   // saved states per lane = ceil(L / state_interval)
  int state_interval;  // steps between saved states (= the backward's chunk)
  int cpw;             // channels per warp (<= kCI); smaller for small problems so the grid fills the GPU
  int state_tile;      // backward: states processed per pass over a chunk (even; >= N means a single pass)
  bool vec_ok;
  bool bc_vec_ok;      // B / C rows may be read with 16-byte loads
  int split_flush_parts;   // split backward: threads per item of the dB / dC sums (0 = all the CTA has)
  bool bc_step_major;      // split kernels: B / C are given [B, L, N] (a step's N values contiguous), not [B, N, L]
  long long bc_pitch;      // ... with this many elements between the rows of consecutive steps (>= N)
};

// (A[d,2p], A[d,2p+1]) * log2(e); a missing odd partner gets 0 (decay 1, no forcing).
__device__ __forceinline__ float2 load_A_pair(const float* A, long long d, int N, int pair, bool active) {
  if (!active) return make_float2(0.f, 0.f);
  const int n0 = 2 * pair;
  const float a0 = __ldg(A + d * N + n0);
  const float a1 = n0 + 1 < N ? __ldg(A + d * N + n0 + 1) : 0.0f;
  return make_float2(a0, a1);
}

// Shared memory (floats): Bs[NP*T*2] | Cs[NP*T*2] | carry[kWarps*kCI*NP*2]   (NP = ceil(N/2))
template <typename IO, int kItems>
__global__ void __launch_bounds__(kThreads) sscan_forward_kernel(Params p) {
  constexpr int T = 32 * kItems;
  extern __shared__ __align__(16) float smem[];
  const int N = (int)p.N;
  const int NP = (N + 1) / 2;
  float* Bs = smem;
  float* Cs = Bs + NP * T * 2;
  float2* carry = reinterpret_cast<float2*>(Cs + NP * T * 2);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long b = blockIdx.y;
  const long long d0 = (long long)blockIdx.x * (kWarps * p.cpw) + warp * p.cpw;
  const long long nchunks = (p.L + T - 1) / T;
  const IO* Bm_b = static_cast<const IO*>(p.Bm) + b * p.N * p.L;
  const IO* Cm_b = static_cast<const IO*>(p.Cm) + b * p.N * p.L;

  for (int i = threadIdx.x; i < kWarps * kCI * NP; i += kThreads) carry[i] = make_float2(0.f, 0.f);

  for (long long c = 0; c < nchunks; ++c) {
    const long long t_base = c * T;
    __syncthreads();  // everyone is done with the previous tiles (and carry init)
    stage_tile<IO, kItems>(Bs, Bm_b, N, t_base, p.L);
    stage_tile<IO, kItems>(Cs, Cm_b, N, t_base, p.L);
    __syncthreads();
    const long long t0 = t_base + (long long)lane * kItems;
#pragma unroll 1
    for (int ci = 0; ci < p.cpw; ++ci) {
      const long long d = d0 + ci;
      if (d >= p.D) break;  // warp-uniform
      const long long row = (b * p.D + d) * p.L;
      float u[kItems], dt[kItems];
      float2 y2[kItems], dtu2[kItems];
      load_items<IO, kItems>(static_cast<const IO*>(p.u) + row, t0, p.L, p.vec_ok, u);
      load_items<float, kItems>(p.dt + row, t0, p.L, p.vec_ok, dt);
      if (p.delta_bias || p.delta_softplus) {   // steps past the end of the sequence stay zero (no-ops)
        const float bias = p.delta_bias ? __ldg(p.delta_bias + d) : 0.0f;
#pragma unroll
        for (int j = 0; j < kItems; ++j) dt[j] = (t0 + j < p.L) ? step_transform(dt[j], bias, p.delta_softplus != 0) : 0.0f;
      }
#pragma unroll
      for (int j = 0; j < kItems; ++j) { dtu2[j] = splat(dt[j] * u[j]); y2[j] = make_float2(0.f, 0.f); }
      float2* cw = carry + (warp * kCI + ci) * NP;
      // States are saved every p.state_interval steps (the backward's chunk): the
      // lanes whose first step starts such an interval write the state entering it.
      const int lanes_per_save = p.state_interval / kItems;
      const bool saver = p.chunk_states != nullptr && (lane % lanes_per_save) == 0 && t0 < p.L;
      float* cs_out = saver ? p.chunk_states + ((b * p.D + d) * p.nstates + t0 / p.state_interval) * p.N : nullptr;
#pragma unroll 1
      for (int pr = 0; pr < NP; ++pr) {
        const float2 Ap = load_A_pair(p.A, d, N, pr, true);
        const float2 A2 = make_float2(Ap.x * kLog2e, Ap.y * kLog2e);
        float2 Bv[kItems], Cv[kItems];
        lds_pairs<kItems>(Bs, pr, lane, Bv);
        lds_pairs<kItems>(Cs, pr, lane, Cv);
        float2 hloc[kItems], cp[kItems];
        float2 P = make_float2(1.f, 1.f), H = make_float2(0.f, 0.f);
#pragma unroll
        for (int j = 0; j < kItems; ++j) {
          const float2 x = p2mul(splat(dt[j]), A2);
          const float2 a = make_float2(ex2(x.x), ex2(x.y));
          H = p2fma(a, H, p2mul(dtu2[j], Bv[j]));
          P = p2mul(P, a);
          hloc[j] = H;
          cp[j] = P;
        }
        const float2 h_in = cw[pr];  // read before the scan: its shuffles order this read before lane 0's update
        float2 Pex, Hex, Ptot, Htot;
        warp_scan_affine(P, H, lane, Pex, Hex, Ptot, Htot);
        const float2 hstart = p2fma(Pex, h_in, Hex);
#pragma unroll
        for (int j = 0; j < kItems; ++j) y2[j] = p2fma(p2fma(cp[j], hstart, hloc[j]), Cv[j], y2[j]);
        if (cs_out) {
          cs_out[2 * pr] = hstart.x;
          if (2 * pr + 1 < N) cs_out[2 * pr + 1] = hstart.y;
        }
        if (lane == 0) cw[pr] = p2fma(Ptot, h_in, Htot);
      }
      float y[kItems];
#pragma unroll
      for (int j = 0; j < kItems; ++j) y[j] = y2[j].x + y2[j].y;
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

// Shared memory (floats), NP = ceil(N/2); the states are processed in tiles of NT = p.state_tile states
// (NPt = NT/2 pairs, tile = NPt*T*2; one tile covers all states when N <= 64):
//   Bs | Cs (one tile each) | acc[kWarps][2 (dB,dC)][tile] | lam[kWarps*cpw*NP*2] | dAacc[kWarps*cpw*NP*2]
//   | dDacc[kWarps*cpw] | dBiasacc[kWarps*cpw] | part[kWarps*cpw][3][kItems][32][2] (only with several tiles)
// Every warp owns a private dB/dC accumulator tile, so the warps of a CTA run
// independently between the three barriers of a pass (tile staging, flush).  With several state tiles
// a chunk is walked once per tile; the per-step sums over the states (y, du, ddt) of every channel wait
// in `part` between the passes and the per-channel outputs are written by the last one.
template <typename IO, int kItems>
__global__ void __launch_bounds__(kThreads) sscan_backward_kernel(Params p) {
  constexpr int T = 32 * kItems;
  extern __shared__ __align__(16) float smem[];
  const int N = (int)p.N;
  const int NP = (N + 1) / 2;
  const int NT = p.state_tile < 2 * NP ? p.state_tile : 2 * NP;     // states per tile (even)
  const int ntiles = (2 * NP + NT - 1) / NT;
  const int tile = (NT / 2) * T * 2;
  const int cpw = p.cpw;
  float* Bs = smem;
  float* Cs = Bs + tile;
  float* acc = Cs + tile;
  float2* lam = reinterpret_cast<float2*>(acc + kWarps * 2 * tile);   // adjoint carried from the later chunk
  float2* dAacc = lam + kWarps * cpw * NP;
  float* dDacc = reinterpret_cast<float*>(dAacc + kWarps * cpw * NP);
  float* dBiasacc = dDacc + kWarps * cpw;
  float2* part = reinterpret_cast<float2*>(dBiasacc + kWarps * cpw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long b = blockIdx.y;
  const long long d0 = (long long)blockIdx.x * (kWarps * cpw) + warp * cpw;
  const long long nchunks = (p.L + T - 1) / T;
  const IO* Bm_b = static_cast<const IO*>(p.Bm) + b * p.N * p.L;
  const IO* Cm_b = static_cast<const IO*>(p.Cm) + b * p.N * p.L;
  float* accB = acc + warp * 2 * tile;
  float* accC = accB + tile;

  for (int i = threadIdx.x; i < kWarps * cpw * NP; i += kThreads) {
    lam[i] = make_float2(0.f, 0.f);
    dAacc[i] = make_float2(0.f, 0.f);
  }
  for (int i = threadIdx.x; i < kWarps * cpw; i += kThreads) { dDacc[i] = 0.0f; dBiasacc[i] = 0.0f; }

  for (long long c = nchunks - 1; c >= 0; --c) {
    const long long t_base = c * T;
    const long long t0 = t_base + (long long)lane * kItems;
#pragma unroll 1
    for (int st = 0; st < ntiles; ++st) {
    const int n0 = st * NT;                                   // first state of this tile
    const int ncur = (N - n0) < NT ? (N - n0) : NT;           // states in this tile
    const int npcur = (ncur + 1) / 2;
    const int pr0 = n0 / 2;
    const bool first_tile = st == 0, last_tile = st == ntiles - 1;
    __syncthreads();  // previous flush finished
    stage_tile<IO, kItems>(Bs, Bm_b + (long long)n0 * p.L, ncur, t_base, p.L);
    stage_tile<IO, kItems>(Cs, Cm_b + (long long)n0 * p.L, ncur, t_base, p.L);
    for (int i = threadIdx.x; i < kWarps * 2 * tile; i += kThreads) acc[i] = 0.0f;
    __syncthreads();

    // operands of the first channel; those of channel ci+1 are fetched while ci is processed
    float u[kItems], dt[kItems], go[kItems], zz[kItems];
    auto fetch = [&](int ci, float (&fu)[kItems], float (&fdt)[kItems], float (&fgo)[kItems], float (&fz)[kItems]) {
      const long long d = d0 + ci;
      const bool ok = ci < cpw && d < p.D;
      const long long row = ok ? (b * p.D + d) * p.L : 0;
      const long long tl = ok ? p.L : 0;
      load_items<IO, kItems>(static_cast<const IO*>(p.u) + row, t0, tl, p.vec_ok, fu);
      load_items<float, kItems>(p.dt + row, t0, tl, p.vec_ok, fdt);
      if (p.delta_bias || p.delta_softplus) {
        const float bias = (ok && p.delta_bias) ? __ldg(p.delta_bias + d) : 0.0f;
#pragma unroll
        for (int j = 0; j < kItems; ++j) fdt[j] = (t0 + j < tl) ? step_transform(fdt[j], bias, p.delta_softplus != 0) : 0.0f;
      }
      load_items<IO, kItems>(static_cast<const IO*>(p.dout) + row, t0, tl, p.vec_ok, fgo);
      if (p.z) load_items<IO, kItems>(static_cast<const IO*>(p.z) + row, t0, tl, p.vec_ok, fz);
    };
    fetch(0, u, dt, go, zz);
#pragma unroll 1
    for (int ci = 0; ci < cpw; ++ci) {
      const long long d = d0 + ci;
      if (d >= p.D) break;                                    // warp-uniform; no CTA barrier inside this loop
      const long long row = (b * p.D + d) * p.L;
      float nu[kItems], ndt[kItems], ngo[kItems], nz[kItems];
      fetch(ci + 1, nu, ndt, ngo, nz);
      float gy[kItems];
      float2 dtu2[kItems], dus2[kItems], ddts2[kItems], y2[kItems];
      float2* mypart = part + (size_t)((warp * cpw + ci) * 3) * kItems * 32 + lane;
#pragma unroll
      for (int j = 0; j < kItems; ++j) {
        gy[j] = p.z ? go[j] * (zz[j] * sigmoidf(zz[j])) : go[j];
        dtu2[j] = splat(dt[j] * u[j]);
        if (first_tile) {
          dus2[j] = make_float2(0.f, 0.f);
          ddts2[j] = make_float2(0.f, 0.f);
          y2[j] = make_float2(0.f, 0.f);
        } else {
          dus2[j] = mypart[(0 * kItems + j) * 32];
          ddts2[j] = mypart[(1 * kItems + j) * 32];
          y2[j] = mypart[(2 * kItems + j) * 32];
        }
      }
      const int slot = (warp * cpw + ci) * NP;
      const float* cs_in = p.chunk_states + ((b * p.D + d) * p.nstates + c * (T / p.state_interval)) * p.N;
#pragma unroll 1
      for (int pr = 0; pr < npcur; ++pr) {
        const int gp = pr0 + pr;                              // pair index among all states
        const float2 Ap = load_A_pair(p.A, d, N, gp, true);
        const float2 A2 = make_float2(Ap.x * kLog2e, Ap.y * kLog2e);
        float2 a[kItems], Bv[kItems], Cv[kItems];
        lds_pairs<kItems>(Bs, pr, lane, Bv);
        lds_pairs<kItems>(Cs, pr, lane, Cv);
        // summaries of this thread's steps: forward map (P,H), adjoint map (Q,R)
        //   lam_t = a_t * (gy_t*C_t + lam_{t+1})
        float2 P = make_float2(1.f, 1.f), H = make_float2(0.f, 0.f);
#pragma unroll
        for (int j = 0; j < kItems; ++j) {
          const float2 x = p2mul(splat(dt[j]), A2);
          a[j] = make_float2(ex2(x.x), ex2(x.y));
          H = p2fma(a[j], H, p2mul(dtu2[j], Bv[j]));
          P = p2mul(P, a[j]);
        }
        float2 Q = make_float2(1.f, 1.f), R = make_float2(0.f, 0.f);
#pragma unroll
        for (int j = kItems - 1; j >= 0; --j) {
          R = p2mul(a[j], p2fma(splat(gy[j]), Cv[j], R));
          Q = p2mul(Q, a[j]);
        }
        float2 h_in;
        h_in.x = __ldg(cs_in + 2 * gp);
        h_in.y = (2 * gp + 1 < N) ? __ldg(cs_in + 2 * gp + 1) : 0.0f;
        const float2 lam_in = lam[slot + gp];              // adjoint entering the chunk from the right
        float2 Pex, Hex, Qex, Rex, Qtot, Rtot;
        warp_scan_dual(P, H, Q, R, lane, Pex, Hex, Qex, Rex, Qtot, Rtot);
        float2 h = p2fma(Pex, h_in, Hex);             // state entering this thread's steps
        float2 lnext = p2fma(Qex, lam_in, Rex);       // lam_{t+1} of this thread's last step
        // true states left to right (kept), then the adjoint right to left
        float2 hprev[kItems], dCv[kItems], dBv[kItems];
        lds_pairs<kItems>(accC, pr, lane, dCv);
        lds_pairs<kItems>(accB, pr, lane, dBv);
#pragma unroll
        for (int j = 0; j < kItems; ++j) {
          hprev[j] = h;
          h = p2fma(a[j], h, p2mul(dtu2[j], Bv[j]));
          y2[j] = p2fma(h, Cv[j], y2[j]);
          dCv[j] = p2fma(splat(gy[j]), h, dCv[j]);
        }
        float2 dA2 = make_float2(0.f, 0.f);
#pragma unroll
        for (int j = kItems - 1; j >= 0; --j) {
          const float2 G = p2fma(splat(gy[j]), Cv[j], lnext);
          lnext = p2mul(G, a[j]);                     // lam_t
          const float2 q = p2mul(lnext, hprev[j]);    // G * a_t * h_{t-1}
          dBv[j] = p2fma(G, dtu2[j], dBv[j]);
          dus2[j] = p2fma(G, Bv[j], dus2[j]);
          dA2 = p2fma(q, splat(dt[j]), dA2);
          ddts2[j] = p2fma(q, Ap, ddts2[j]);
        }
        sts_pairs<kItems>(accC, pr, lane, dCv);
        sts_pairs<kItems>(accB, pr, lane, dBv);
        // carry for the next (earlier) chunk and per-channel dA
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
          dA2.x += __shfl_xor_sync(0xffffffffu, dA2.x, off);
          dA2.y += __shfl_xor_sync(0xffffffffu, dA2.y, off);
        }
        if (lane == 0) {
          lam[slot + gp] = p2fma(Qtot, lam_in, Rtot);
          dAacc[slot + gp] = p2add(dAacc[slot + gp], dA2);
        }
      }
      if (!last_tile) {
        // sums over the states seen so far wait for the remaining tiles
#pragma unroll
        for (int j = 0; j < kItems; ++j) {
          mypart[(0 * kItems + j) * 32] = dus2[j];
          mypart[(1 * kItems + j) * 32] = ddts2[j];
          mypart[(2 * kItems + j) * 32] = y2[j];
        }
      } else {
      // du_t = dt_t * sum_n G*B (+ gy*Dskip) ; ddt_t = sum_n q*A + u_t * sum_n G*B
      float ds = 0.0f, dD_t = 0.0f;
      if (p.Dskip) ds = __ldg(p.Dskip + d);
      float duv[kItems], ddv[kItems];
#pragma unroll
      for (int j = 0; j < kItems; ++j) {
        const float gb = dus2[j].x + dus2[j].y;
        duv[j] = fmaf(dt[j], gb, gy[j] * ds);
        ddv[j] = fmaf(u[j], gb, ddts2[j].x + ddts2[j].y);
        dD_t = fmaf(gy[j], u[j], dD_t);
      }
      float dbias_t = 0.0f;
      if (p.delta_bias || p.delta_softplus) {   // gradient with respect to the raw step
#pragma unroll
        for (int j = 0; j < kItems; ++j) {
          ddv[j] = (t0 + j < p.L) ? ddv[j] * step_transform_grad(dt[j], p.delta_softplus != 0) : 0.0f;
          dbias_t += ddv[j];
        }
      }
      store_items<IO, kItems>(static_cast<IO*>(p.du) + row, t0, p.L, p.vec_ok, duv);
      store_items<float, kItems>(p.ddt + row, t0, p.L, p.vec_ok, ddv);
      if (p.z) {
        float dzv[kItems];
#pragma unroll
        for (int j = 0; j < kItems; ++j) {
          const float sg = sigmoidf(zz[j]);
          const float yy = fmaf(ds, u[j], y2[j].x + y2[j].y);
          dzv[j] = go[j] * yy * (sg * (1.0f + zz[j] * (1.0f - sg)));
        }
        store_items<IO, kItems>(static_cast<IO*>(p.dz) + row, t0, p.L, p.vec_ok, dzv);
      }
      if (p.dD_part) {
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) dD_t += __shfl_xor_sync(0xffffffffu, dD_t, off);
        if (lane == 0) dDacc[warp * cpw + ci] += dD_t;
      }
      if (p.dbias_part) {
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) dbias_t += __shfl_xor_sync(0xffffffffu, dbias_t, off);
        if (lane == 0) dBiasacc[warp * cpw + ci] += dbias_t;
      }
      }
#pragma unroll
      for (int j = 0; j < kItems; ++j) { u[j] = nu[j]; dt[j] = ndt[j]; go[j] = ngo[j]; zz[j] = nz[j]; }
      __syncwarp();
    }
    // sum the warps' private tiles and flush this pass's dB/dC rows to global
    __syncthreads();
    for (int i = threadIdx.x; i < ncur * T; i += kThreads) {
      const int n = i / T, t = i - n * T;
      const long long tt = t_base + t;
      if (tt < p.L) {
        const int ti = tile_index<kItems>(n >> 1, t, n & 1);
        float sb = 0.0f, sc = 0.0f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
          sb += acc[w * 2 * tile + ti];
          sc += acc[w * 2 * tile + tile + ti];
        }
        atomicAdd(p.dB + (b * p.N + n0 + n) * p.L + tt, sb);
        atomicAdd(p.dC + (b * p.N + n0 + n) * p.L + tt, sc);
      }
    }
    }  // state tiles
  }
  __syncthreads();
  for (int i = threadIdx.x; i < kWarps * cpw * N; i += kThreads) {
    const int wc = i / N, n = i - wc * N;
    const int w = wc / cpw, ci = wc - w * cpw;
    const long long d = (long long)blockIdx.x * (kWarps * cpw) + w * cpw + ci;
    if (d < p.D) {
      const float2 v = dAacc[wc * NP + (n >> 1)];
      p.dA_part[(b * p.D + d) * p.N + n] = (n & 1) ? v.y : v.x;
    }
  }
  if (p.dD_part) {
    for (int i = threadIdx.x; i < kWarps * cpw; i += kThreads) {
      const int w = i / cpw, ci = i - w * cpw;
      const long long d = (long long)blockIdx.x * (kWarps * cpw) + w * cpw + ci;
      if (d < p.D) p.dD_part[b * p.D + d] = dDacc[i];
    }
  }
  if (p.dbias_part) {
    for (int i = threadIdx.x; i < kWarps * cpw; i += kThreads) {
      const int w = i / cpw, ci = i - w * cpw;
      const long long d = (long long)blockIdx.x * (kWarps * cpw) + w * cpw + ci;
      if (d < p.D) p.dbias_part[b * p.D + d] = dBiasacc[i];
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

// Steps per thread.  The backward keeps more per-step values in registers and a
// private accumulator tile per warp in shared memory, so it works on shorter
// chunks than the forward; the forward saves the states the backward needs at
// the backward's chunk interval.
static int items_bwd(long long N) {
  if (N <= 16) return 4;
  if (N <= 32) return 2;
  return 1;
}
static int items_fwd(long long N) {
  if (N <= 16) return 8;
  if (N <= 32) return 4;
  if (N <= 64) return 2;
  return 1;
}

template <typename K>
static int set_smem(K kernel, size_t bytes) {
  return ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), bytes);
}

template <typename IO, int kItems>
static int launch_fwd(const Params& p, cudaStream_t stream) {
  const int T = 32 * kItems;
  const size_t np2 = 2 * (size_t)((p.N + 1) / 2);
  const size_t smem = sizeof(float) * (2 * np2 * T + (size_t)kWarps * kCI * np2);
  if (smem > 200 * 1024) { set_last_error("selective_scan_forward: d_state too large"); return kErrUnsupported; }
  if (int rc = set_smem(sscan_forward_kernel<IO, kItems>, smem)) return rc;
  dim3 grid((unsigned)((p.D + kWarps * p.cpw - 1) / (kWarps * p.cpw)), (unsigned)p.B);
  sscan_forward_kernel<IO, kItems><<<grid, kThreads, smem, stream>>>(p);
  return check_cuda(cudaGetLastError(), "sscan_forward_kernel launch");
}

template <typename IO, int kItems>
static int launch_bwd(const Params& p, cudaStream_t stream) {
  const int T = 32 * kItems;
  const size_t np2 = 2 * (size_t)((p.N + 1) / 2);
  const size_t nt = (size_t)p.state_tile < np2 ? (size_t)p.state_tile : np2;    // states per tile
  const size_t ntiles = (np2 + nt - 1) / nt;
  const size_t smem = sizeof(float) * ((2 + 2 * (size_t)kWarps) * nt * T + 2 * (size_t)kWarps * p.cpw * np2 +
                                       2 * kWarps * p.cpw +
                                       (ntiles > 1 ? (size_t)kWarps * p.cpw * 3 * kItems * 32 * 2 : 0));
  if (smem > 220 * 1024) { set_last_error("selective_scan_backward: d_state too large"); return kErrUnsupported; }
  if (int rc = set_smem(sscan_backward_kernel<IO, kItems>, smem)) return rc;
  dim3 grid((unsigned)((p.D + kWarps * p.cpw - 1) / (kWarps * p.cpw)), (unsigned)p.B);
  sscan_backward_kernel<IO, kItems><<<grid, kThreads, smem, stream>>>(p);
  return check_cuda(cudaGetLastError(), "sscan_backward_kernel launch");
}

template <typename IO>
static int dispatch_items(bool backward, const Params& p, cudaStream_t stream) {
  if (backward) {
    switch (items_bwd(p.N)) {
      case 4: return launch_bwd<IO, 4>(p, stream);
      case 2: return launch_bwd<IO, 2>(p, stream);
      default: return launch_bwd<IO, 1>(p, stream);
    }
  }
  switch (items_fwd(p.N)) {
    case 8: return launch_fwd<IO, 8>(p, stream);
    case 4: return launch_fwd<IO, 4>(p, stream);
    case 2: return launch_fwd<IO, 2>(p, stream);
    default: return launch_fwd<IO, 1>(p, stream);
  }
}

}  // namespace sscan
}  // namespace ossm_b200

#include "selective_scan_serial.cuh"

namespace ossm_b200 {
namespace sscan {
#include "selective_scan_split.cuh"
}  // namespace sscan
}  // namespace ossm_b200

namespace ossm_b200 {
namespace sscan {

// Serial-in-time kernels (selective_scan_serial.cuh) are used for the state sizes they are built for.
static int g_use_serial = 1;
static bool serial_ok(long long N) { return g_use_serial && N == 16; }
// Steps between the states the forward saves for the backward.
static int state_interval_for(long long N) {
  if (serial_ok(N)) return kSerialInterval;
  if (g_use_serial && split_bwd_ok(N)) return kSplitChunk;
  return 32 * items_bwd(N);
}

// Channels per warp: the most that still gives one CTA per SM.
static int pick_cpw(long long B, long long D) {
  int cpw = kCI;
  while (cpw > 1 && B * ((D + kWarps * cpw - 1) / (kWarps * cpw)) < (long long)sm_count()) cpw >>= 1;
  return cpw;
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace sscan
}  // namespace ossm_b200

extern "C" {

using namespace ossm_b200;

int ossm_b200_selective_scan_chunk(int64_t N) { return sscan::state_interval_for(N); }

int ossm_b200_selective_scan_set_tuning(const char* key, int value) {
  if (key != nullptr && !strcmp(key, "serial")) { sscan::g_use_serial = value != 0; return kOk; }
  if (key != nullptr && !strcmp(key, "split_bwd_wide_from") && value > 0) { sscan::g_split_bwd_wide_from = value; return kOk; }
  if (key != nullptr && !strcmp(key, "split_flush_parts") && value >= 0) { sscan::g_split_flush_parts = value; return kOk; }
  if (key != nullptr && !strcmp(key, "bwd_split") && (value == 2 || value == 4)) { sscan::g_bwd_split = value; return kOk; }
  set_last_error("selective_scan_set_tuning: unknown key %s", key ? key : "(null)");
  return kErrInvalidArgument;
}

size_t ossm_b200_selective_scan_state_bytes(int64_t B, int64_t D, int64_t L, int64_t N) {
  if (B <= 0 || D <= 0 || L <= 0 || N <= 0) return 0;
  const int64_t T = sscan::state_interval_for(N);
  return (size_t)B * D * ((L + T - 1) / T) * N * sizeof(float);
}

size_t ossm_b200_selective_scan_backward_workspace_bytes(int64_t B, int64_t D, int64_t L, int64_t N) {
  if (B <= 0 || D <= 0 || L <= 0 || N <= 0) return 0;
  return (size_t)B * D * (N + 2) * sizeof(float);   // batch partials of dA, dD and d(delta_bias)
}

static int sscan_check(const char* fn, const void* u, const float* dt, const float* A, const void* Bm,
                       const void* Cm, int64_t B, int64_t D, int64_t L, int64_t N, int io_dtype) {
  if (B < 0 || D < 0 || L < 0 || N < 0) { set_last_error("%s: negative extent", fn); return kErrInvalidArgument; }
  if (io_dtype != OSSM_B200_DTYPE_F32 && io_dtype != OSSM_B200_DTYPE_BF16) {
    set_last_error("%s: unknown io dtype %d", fn, io_dtype);
    return kErrInvalidArgument;
  }
  if (N > sscan::kMaxState) {
    set_last_error("%s: d_state > %d is not supported", fn, sscan::kMaxState);
    return kErrUnsupported;
  }
  if (B > 65535) { set_last_error("%s: batch > 65535 is not supported", fn); return kErrUnsupported; }
  if (B == 0 || D == 0 || L == 0 || N == 0) return kOk;
  if (!u || !dt || !A || !Bm || !Cm) { set_last_error("%s: null input pointer", fn); return kErrInvalidArgument; }
  return kOk;
}

static int selective_scan_forward_impl(bool step_major, int64_t bc_pitch, const void* u, const float* dt, const float* A, const void* Bm,
                                       const void* Cm, const void* z, const float* Dskip, const float* delta_bias,
                                       int delta_softplus, void* out, float* chunk_states, int64_t B, int64_t D,
                                       int64_t L, int64_t N, int io_dtype, cudaStream_t stream) {
  if (int rc = sscan_check("selective_scan_forward", u, dt, A, Bm, Cm, B, D, L, N, io_dtype)) return rc;
  if (step_major && !(sscan::g_use_serial && (sscan::split_ok(N) || sscan::serial_ok(N)))) {
    set_last_error("selective_scan_forward: B / C in [B, L, N] order are taken for d_state 16, 32, 64, 128, 256 only "
                   "(ossm_b200_selective_scan_step_major_bc)");
    return kErrInvalidArgument;
  }
  if (step_major && bc_pitch < N) {
    set_last_error("selective_scan: bc_pitch must be at least N");
    return kErrInvalidArgument;
  }
  if (B == 0 || D == 0 || L == 0) return kOk;
  if (!out) { set_last_error("selective_scan_forward: null out"); return kErrInvalidArgument; }
  if (N == 0) {
    set_last_error("selective_scan_forward: d_state must be positive");
    return kErrInvalidArgument;
  }
  sscan::Params p{};
  p.u = u; p.dt = dt; p.A = A; p.Bm = Bm; p.Cm = Cm; p.z = z; p.Dskip = Dskip; p.out = out;
  p.delta_bias = delta_bias; p.delta_softplus = delta_softplus != 0;
  p.chunk_states = chunk_states;
  p.B = B; p.D = D; p.L = L; p.N = N;
  p.state_interval = sscan::state_interval_for(N);
  p.nstates = (L + p.state_interval - 1) / p.state_interval;
  p.cpw = sscan::pick_cpw(B, D);
  const int es = io_dtype == OSSM_B200_DTYPE_F32 ? 4 : 2;
  p.vec_ok = sscan::aligned16(u) && sscan::aligned16(dt) && sscan::aligned16(out) && (!z || sscan::aligned16(z)) &&
             (L * es) % 16 == 0 && (L * 4) % 16 == 0;
  if (sscan::serial_ok(N)) {
    if (!sscan::aligned16(chunk_states)) {
      set_last_error("selective_scan_forward: chunk_states must be 16-byte aligned");
      return kErrInvalidArgument;
    }
    // the B/C tiles are also read with 16-byte loads
    p.bc_step_major = step_major;
    p.bc_pitch = bc_pitch;
    p.bc_vec_ok = sscan::aligned16(Bm) && sscan::aligned16(Cm) && (bc_pitch * es) % 16 == 0;
    if (!step_major) p.vec_ok = p.vec_ok && sscan::aligned16(Bm) && sscan::aligned16(Cm);
    return io_dtype == OSSM_B200_DTYPE_F32 ? sscan::launch_fwd_serial<float>(p, stream)
                                           : sscan::launch_fwd_serial<__nv_bfloat16>(p, stream);
  }
  if (sscan::g_use_serial && sscan::split_ok(N)) {
    if (!sscan::aligned16(chunk_states)) {
      set_last_error("selective_scan_forward: chunk_states must be 16-byte aligned");
      return kErrInvalidArgument;
    }
    p.bc_step_major = step_major;
    p.bc_pitch = bc_pitch;
    p.bc_vec_ok = sscan::aligned16(Bm) && sscan::aligned16(Cm) && ((step_major ? bc_pitch : L) * es) % 16 == 0;
    return io_dtype == OSSM_B200_DTYPE_F32 ? sscan::launch_fwd_split<float>(p, stream)
                                           : sscan::launch_fwd_split<__nv_bfloat16>(p, stream);
  }
  return io_dtype == OSSM_B200_DTYPE_F32 ? sscan::dispatch_items<float>(false, p, stream)
                                         : sscan::dispatch_items<__nv_bfloat16>(false, p, stream);
}

int ossm_b200_selective_scan_forward(const void* u, const float* dt, const float* A, const void* Bm, const void* Cm,
                                     const void* z, const float* Dskip, const float* delta_bias, int delta_softplus,
                                     void* out, float* chunk_states, int64_t B, int64_t D, int64_t L, int64_t N,
                                     int io_dtype, cudaStream_t stream) {
  return selective_scan_forward_impl(false, 0, u, dt, A, Bm, Cm, z, Dskip, delta_bias, delta_softplus, out, chunk_states,
                                     B, D, L, N, io_dtype, stream);
}

int ossm_b200_selective_scan_forward_step_major_bc(const void* u, const float* dt, const float* A, const void* Bm,
                                                   const void* Cm, const void* z, const float* Dskip,
                                                   const float* delta_bias, int delta_softplus, void* out,
                                                   float* chunk_states, int64_t B, int64_t D, int64_t L, int64_t N,
                                                   int64_t bc_pitch, int io_dtype, cudaStream_t stream) {
  return selective_scan_forward_impl(true, bc_pitch, u, dt, A, Bm, Cm, z, Dskip, delta_bias, delta_softplus, out, chunk_states,
                                     B, D, L, N, io_dtype, stream);
}

int ossm_b200_selective_scan_step_major_bc(int64_t N) {
  return (sscan::g_use_serial && (sscan::split_ok(N) || sscan::serial_ok(N))) ? 1 : 0;
}

static int selective_scan_backward_impl(bool step_major, int64_t bc_pitch, const void* u, const float* dt, const float* A, const void* Bm,
                                        const void* Cm, const void* z, const float* Dskip, const float* delta_bias,
                                        int delta_softplus, const void* dout, const float* chunk_states, void* du,
                                        float* ddt, float* dA, float* dB, float* dC, void* dz, float* dD,
                                        float* ddelta_bias, void* workspace, size_t workspace_bytes, int64_t B,
                                        int64_t D, int64_t L, int64_t N, int io_dtype, cudaStream_t stream) {
  if (int rc = sscan_check("selective_scan_backward", u, dt, A, Bm, Cm, B, D, L, N, io_dtype)) return rc;
  if (step_major && !(sscan::g_use_serial && (sscan::split_bwd_ok(N) || sscan::serial_ok(N)))) {
    set_last_error("selective_scan_backward: B / C in [B, L, N] order are taken for d_state 16, 32, 64, 128, 256 only "
                   "(ossm_b200_selective_scan_step_major_bc)");
    return kErrInvalidArgument;
  }
  if (step_major && bc_pitch < N) {
    set_last_error("selective_scan: bc_pitch must be at least N");
    return kErrInvalidArgument;
  }
  if (D == 0 || N == 0) return kOk;
  if (!dA) { set_last_error("selective_scan_backward: null dA"); return kErrInvalidArgument; }
  if (int rc = check_cuda(cudaMemsetAsync(dA, 0, (size_t)D * N * sizeof(float), stream), "memset dA")) return rc;
  if (dD) if (int rc = check_cuda(cudaMemsetAsync(dD, 0, (size_t)D * sizeof(float), stream), "memset dD")) return rc;
  if (ddelta_bias)
    if (int rc = check_cuda(cudaMemsetAsync(ddelta_bias, 0, (size_t)D * sizeof(float), stream), "memset ddelta_bias"))
      return rc;
  if (B == 0 || L == 0) return kOk;
  if (!dout || !chunk_states || !du || !ddt || !dB || !dC || (z && !dz) || (Dskip && !dD) ||
      (delta_bias && !ddelta_bias)) {
    set_last_error("selective_scan_backward: null pointer among dout/chunk_states/du/ddt/dB/dC/dz/dD/ddelta_bias");
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
  p.dbias_part = delta_bias ? p.dA_part + (size_t)B * D * (N + 1) : nullptr;
  p.delta_bias = delta_bias; p.delta_softplus = delta_softplus != 0;
  p.B = B; p.D = D; p.L = L; p.N = N;
  p.state_interval = sscan::state_interval_for(N);
  p.nstates = (L + p.state_interval - 1) / p.state_interval;
  p.cpw = sscan::pick_cpw(B, D);
  p.state_tile = sscan::kStateTile;
  if (N > sscan::kStateTile && p.cpw > 2) p.cpw = 2;   // bounds the per-channel carries in shared memory
  const int es = io_dtype == OSSM_B200_DTYPE_F32 ? 4 : 2;
  p.vec_ok = sscan::aligned16(u) && sscan::aligned16(dt) && sscan::aligned16(dout) && sscan::aligned16(du) &&
             sscan::aligned16(ddt) && (!z || (sscan::aligned16(z) && sscan::aligned16(dz))) &&
             (L * es) % 16 == 0 && (L * 4) % 16 == 0;
  int rc;
  if (sscan::serial_ok(N)) {
    if (!sscan::aligned16(chunk_states)) {
      set_last_error("selective_scan_backward: chunk_states must be 16-byte aligned");
      return kErrInvalidArgument;
    }
    // B/C tiles, dB and dC are also accessed with 16-byte operations
    p.bc_step_major = step_major;
    p.bc_pitch = bc_pitch;
    p.bc_vec_ok = sscan::aligned16(Bm) && sscan::aligned16(Cm) && (bc_pitch * es) % 16 == 0;
    p.vec_ok = p.vec_ok && (step_major || (sscan::aligned16(Bm) && sscan::aligned16(Cm))) && sscan::aligned16(dB) &&
               sscan::aligned16(dC);
    rc = io_dtype == OSSM_B200_DTYPE_F32 ? sscan::launch_bwd_serial<float>(p, stream)
                                         : sscan::launch_bwd_serial<__nv_bfloat16>(p, stream);
  } else if (sscan::g_use_serial && sscan::split_bwd_ok(N)) {
    if (!sscan::aligned16(chunk_states)) {
      set_last_error("selective_scan_backward: chunk_states must be 16-byte aligned");
      return kErrInvalidArgument;
    }
    p.bc_step_major = step_major;
    p.bc_pitch = bc_pitch;
    // dB / dC ([B, N, L] in both cases) take 16-byte atomics along t; B / C rows 16-byte loads along t or along n
    p.bc_vec_ok = sscan::aligned16(Bm) && sscan::aligned16(Cm) && sscan::aligned16(dB) && sscan::aligned16(dC) &&
                  ((step_major ? bc_pitch : L) * es) % 16 == 0 && (L * 4) % 16 == 0;
    rc = io_dtype == OSSM_B200_DTYPE_F32 ? sscan::launch_bwd_split<float>(p, stream)
                                         : sscan::launch_bwd_split<__nv_bfloat16>(p, stream);
  } else {
    rc = io_dtype == OSSM_B200_DTYPE_F32 ? sscan::dispatch_items<float>(true, p, stream)
                                         : sscan::dispatch_items<__nv_bfloat16>(true, p, stream);
  }
  if (rc) return rc;
  const long long M = D * N;
  sscan::sscan_reduce_batch_kernel<<<(unsigned)((M + 255) / 256), 256, 0, stream>>>(p.dA_part, dA, B, M);
  if (int rc2 = check_cuda(cudaGetLastError(), "sscan_reduce_batch_kernel launch")) return rc2;
  if (p.dD_part) {
    sscan::sscan_reduce_batch_kernel<<<(unsigned)((D + 255) / 256), 256, 0, stream>>>(p.dD_part, dD, B, D);
    if (int rc2 = check_cuda(cudaGetLastError(), "sscan_reduce_batch_kernel launch")) return rc2;
  }
  if (p.dbias_part) {
    sscan::sscan_reduce_batch_kernel<<<(unsigned)((D + 255) / 256), 256, 0, stream>>>(p.dbias_part, ddelta_bias, B, D);
    if (int rc2 = check_cuda(cudaGetLastError(), "sscan_reduce_batch_kernel launch")) return rc2;
  }
  return kOk;
}

int ossm_b200_selective_scan_backward(const void* u, const float* dt, const float* A, const void* Bm,
                                      const void* Cm, const void* z, const float* Dskip, const float* delta_bias,
                                      int delta_softplus, const void* dout, const float* chunk_states, void* du,
                                      float* ddt, float* dA, float* dB, float* dC, void* dz, float* dD,
                                      float* ddelta_bias, void* workspace, size_t workspace_bytes, int64_t B,
                                      int64_t D, int64_t L, int64_t N, int io_dtype, cudaStream_t stream) {
  return selective_scan_backward_impl(false, 0, u, dt, A, Bm, Cm, z, Dskip, delta_bias, delta_softplus, dout, chunk_states,
                                      du, ddt, dA, dB, dC, dz, dD, ddelta_bias, workspace, workspace_bytes, B, D, L, N,
                                      io_dtype, stream);
}

int ossm_b200_selective_scan_backward_step_major_bc(const void* u, const float* dt, const float* A, const void* Bm,
                                                    const void* Cm, const void* z, const float* Dskip,
                                                    const float* delta_bias, int delta_softplus, const void* dout,
                                                    const float* chunk_states, void* du, float* ddt, float* dA,
                                                    float* dB, float* dC, void* dz, float* dD, float* ddelta_bias,
                                                    void* workspace, size_t workspace_bytes, int64_t B, int64_t D,
                                                    int64_t L, int64_t N, int64_t bc_pitch, int io_dtype,
                                                    cudaStream_t stream) {
  return selective_scan_backward_impl(true, bc_pitch, u, dt, A, Bm, Cm, z, Dskip, delta_bias, delta_softplus, dout, chunk_states,
                                      du, ddt, dA, dB, dC, dz, dD, ddelta_bias, workspace, workspace_bytes, B, D, L, N,
                                      io_dtype, stream);
}

}  // extern "C"
