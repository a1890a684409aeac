// D-LinOSS (imex1 / imex2 / im / ex) and LinOSS (IM / IMEX) scans, forward and
// backward, for sm_100a.
//
// The recurrence is linear and time-invariant per channel: a real 2x2
// transition M[p] and real forcing scales F[p] act on a complex 2-state,
//     s_t = M s_{t-1} + F * bu_t ,   x_t = (s_t)_1 ,
// so the real and imaginary parts are two independent real recurrences that
// share M.  Replaces the reference kernels dlinoss_{imex1,imex2,im,ex}_cuda.cu
// (forward + backward) and the LinOSS layer recurrence (linoss.py:244-315) with
// its Python-loop backward (linoss.py:83-151).
//
// Data layout: time-major [L, B, P] complex64 with P contiguous, viewed as a
// 2-D matrix [L rows, N = B*P columns] of 8-byte elements.
//
// Work decomposition: one warp owns 32 adjacent columns (a 256-byte row
// segment) for the whole sequence; each lane runs one series serially in time,
// which keeps the fp32 evaluation order of a sequential scan.  What makes this
// bandwidth- rather than latency-bound is the staging: a per-warp ring of
// shared-memory stages is filled by TMA (one 2-D box of kChunk rows x 256 B per
// stage, completion on an mbarrier), so the time loop only ever touches shared
// memory and registers while several stages of HBM reads are in flight.
// Outputs leave through 256-byte (x) / 512-byte (full states) coalesced warp
// stores.
//
// Backward: the forward pass saves the state at every kChunk-th step
// ("carries", 16 B per series per chunk).  The backward warp walks the chunks
// in reverse; for each chunk it re-runs the forward recurrence from the saved
// carry (keeping the kChunk previous states in registers) and then runs the
// adjoint recurrence right-to-left, producing grad_bu and per-series partial
// sums for the coefficient gradients.  A second tiny kernel reduces the
// partials over the batch in a fixed order and applies the chain rule to
// (A, G, step), so results are run-to-run deterministic (no atomics).
#include "common.cuh"

#include "../../include/ossm_b200.h"

namespace ossm_b200 {
OSSM_B200_STATUS_ACCESSOR(status_lti)
namespace lti {

constexpr int kChunk = 32;          // rows per stage == carry interval
constexpr int kCols = 32;           // columns (series) per warp
constexpr int kStageBytes = kChunk * kCols * 8;
constexpr int kNumAcc = 6;          // per-series partial sums written by backward

enum Variant : int {
  kImex1 = OSSM_B200_VARIANT_IMEX1,
  kImex2 = OSSM_B200_VARIANT_IMEX2,
  kIm = OSSM_B200_VARIANT_IM,
  kEx = OSSM_B200_VARIANT_EX,
  kLinossIm = OSSM_B200_VARIANT_LINOSS_IM,
  kLinossImex = OSSM_B200_VARIANT_LINOSS_IMEX,
  kDiag = OSSM_B200_VARIANT_DIAG,   // x_t = lambda * x_{t-1} + b_t, complex lambda = (a, g) per channel
};

// Coefficients as (v, v) pairs: the real and imaginary parts of a state evolve
// under the same real coefficients, so every update is one packed f32x2
// instruction (fma.rn.f32x2 on sm_100) on an (re, im) register pair.
struct Coef {
  float2 m11, m12, m21, m22, f1, f2;
};

__device__ __forceinline__ float2 bcast(float v) { return make_float2(v, v); }

// Coefficient formulas: dlinoss_imex1_cuda.cu:30-38, dlinoss_imex2_cuda.cu:32-35,
// dlinoss_im_cuda.cu:31-37, dlinoss_ex_cuda.cu:30-33, linoss.py:244-258 + 295-300.
// IEEE division (this file is built without fast-math).
template <int V>
__device__ __forceinline__ Coef make_coef(float al, float ga, float si) {
  float m11, m12, m21, m22, f1, f2;
  if constexpr (V == kImex1) {
    const float inv = 1.0f / (1.0f + si * ga);
    const float s2i = si * si * inv;
    m11 = inv; m12 = -al * s2i; m21 = inv; m22 = 1.0f + m12; f1 = s2i; f2 = s2i;
  } else if constexpr (V == kImex2) {
    const float s2 = si * si;
    m11 = 1.0f - si * ga; m12 = -si * al; m21 = si - s2 * ga; m22 = 1.0f - s2 * al;
    f1 = si; f2 = s2;
  } else if constexpr (V == kIm) {
    const float s2 = si * si;
    const float inv = 1.0f / (1.0f + si * ga + s2 * al);
    const float si_inv = si * inv;
    m11 = inv; m12 = -al * si_inv; m21 = si_inv; m22 = (1.0f + si * ga) * inv;
    f1 = si_inv; f2 = s2 * inv;
  } else if constexpr (V == kEx) {
    m11 = 1.0f - si * ga; m12 = -si * al; m21 = si; m22 = 1.0f; f1 = si; f2 = 0.0f;
  } else if constexpr (V == kLinossIm) {
    const float s2a = si * si * al;
    const float schur = 1.0f / (1.0f + s2a);
    m11 = 1.0f - s2a * schur; m12 = -si * al * schur; m21 = si * schur; m22 = schur;
    f1 = m11 * si; f2 = m21 * si;
  } else if constexpr (V == kLinossImex) {
    m11 = 1.0f; m12 = -si * al; m21 = si; m22 = 1.0f - si * si * al; f1 = si; f2 = si * si;
  } else {  // kDiag: (m11, m12) = (Re lambda, Im lambda), the other entries are unused
    m11 = al; m12 = ga; m21 = 0.0f; m22 = 0.0f; f1 = 1.0f; f2 = 0.0f;
  }
  Coef c;
  c.m11 = bcast(m11); c.m12 = bcast(m12); c.m21 = bcast(m21); c.m22 = bcast(m22);
  c.f1 = bcast(f1); c.f2 = bcast(f2);
  return c;
}

// One forward step on an (re, im) pair.  imex1 keeps the reference's
// "w' = ... ; x' = w' + x" form (dlinoss_imex1_cuda.cu:53-57), whose transition
// has determinant exactly `inv`; the other variants use the plain 2x2 form.
template <int V>
__device__ __forceinline__ void fwd_step(const Coef& c, float2& s0, float2& s1, float2 b) {
  if constexpr (V == kDiag) {
    // complex multiply-add on the (re, im) pair: x' = lambda * x + b  (lru_scan.cpp:11-66, s5_scan.cpp)
    const float2 rot = make_float2(-s1.y, s1.x);
    s1 = __ffma2_rn(s1, c.m11, __ffma2_rn(rot, c.m12, b));
    return;
  }
  const float2 n0 = __ffma2_rn(s1, c.m12, __ffma2_rn(s0, c.m11, __fmul2_rn(b, c.f1)));
  if constexpr (V == kImex1) {
    s1 = __fadd2_rn(n0, s1);
  } else {
    s1 = __ffma2_rn(s1, c.m22, __ffma2_rn(s0, c.m21, __fmul2_rn(b, c.f2)));
  }
  s0 = n0;
}

struct FwdParams {
  const float* a;
  const float* g;
  const float* step;
  const float2* bu;      // [L, N]
  float2* x;             // [L, N] or null
  float4* states;        // [L, N] of (s0.re, s0.im, s1.re, s1.im) or null
  float4* carries;       // [nchunks-1, N] or null
  long long L, N, P;
  int ring;              // stages per warp
  // time segments (grid.y): segment s covers chunks [s*seg_chunks, (s+1)*seg_chunks)
  long long seg_chunks;  // chunks per segment (>= nchunks when the sequence is not split)
  const float4* seg_init;  // [S, N] state entering each segment, or null (zero)
  float4* seg_end;         // [S, N] state leaving each segment (summary pass), or null
};

// Shared memory per warp: ring * kStageBytes, preceded (per CTA) by the barriers.
// kOut: 1 = write x, 2 = write full states, 3 = both.
// kW: warps per CTA when known at compile time (0 = read from the launch); a constant makes every
// shared-memory offset of the unrolled time loop an immediate.
template <int V, bool kTma, int kOut, int kW = 0>
__global__ void __launch_bounds__(128) lti_forward_kernel(const __grid_constant__ CUtensorMap tm_bu, FwdParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const int warp = threadIdx.x >> 5;
  const int warps = kW > 0 ? kW : (int)(blockDim.x >> 5);
  const int cta_cols = warps * kCols;                      // columns of one shared stage
  const long long cta_col0 = (long long)blockIdx.x * cta_cols;
  const long long n = cta_col0 + threadIdx.x;              // this lane's series
  const bool valid = n < p.N;
  if (!kTma && cta_col0 + (long long)warp * kCols >= p.N) return;
  const long long ch = valid ? (n % p.P) : 0;
  const Coef c = make_coef<V>(p.a[ch], p.g ? p.g[ch] : 0.0f, p.step ? p.step[ch] : 0.0f);

  const long long nchunks = (p.L + kChunk - 1) / kChunk;
  const long long k0 = (long long)blockIdx.y * p.seg_chunks;            // this CTA's time segment
  const long long k1 = (k0 + p.seg_chunks) < nchunks ? (k0 + p.seg_chunks) : nchunks;
  float2 s0 = make_float2(0.f, 0.f), s1 = make_float2(0.f, 0.f);
  if (p.seg_init && valid) {
    const float4 v = p.seg_init[(long long)blockIdx.y * p.N + n];
    s0 = make_float2(v.x, v.y);
    s1 = make_float2(v.z, v.w);
  }
  float2* xp = (kOut & 1) ? p.x + k0 * kChunk * p.N + n : nullptr;
  float4* sp = (kOut & 2) ? p.states + k0 * kChunk * p.N + n : nullptr;

  if constexpr (kTma) {
    // All warps of the CTA consume the same stage (one TMA box of kChunk rows x
    // cta_cols columns, i.e. rows of warps*256 contiguous bytes) and meet at a
    // CTA barrier once per chunk before the slot is refilled.  No warp leaves
    // early: warps past the last column see zero-filled tiles and store nothing.
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw);
    unsigned char* ring_base = smem_raw + 1024;
    const uint32_t stage_bytes = (uint32_t)warps * kStageBytes;
    if (threadIdx.x == 0) {
      prefetch_tensormap(&tm_bu);
      for (int s = 0; s < p.ring; ++s) mbar_init(&bars[s], 1);
      fence_barrier_init();
      fence_proxy_async();
      const int pre = (int)((k1 - k0) < p.ring ? (k1 - k0) : p.ring);
      for (int s = 0; s < pre; ++s) {
        mbar_expect_tx(&bars[s], stage_bytes);
        tma_load_2d(ring_base + (size_t)s * stage_bytes, &tm_bu, &bars[s], (int32_t)(cta_col0 * 2),
                    (int32_t)((k0 + s) * kChunk));
      }
    }
    __syncthreads();
    int slot = 0;
    uint32_t parity = 0;
    for (long long k = k0; k < k1; ++k) {
      if (!mbar_wait(&bars[slot], parity)) return;
      const float2* stage = reinterpret_cast<const float2*>(ring_base + (size_t)slot * stage_bytes) + threadIdx.x;
      const int rows = (int)((p.L - k * kChunk) < kChunk ? (p.L - k * kChunk) : kChunk);
      if (rows == kChunk) {
        // full chunk: straight-line code, no per-row predicates
#pragma unroll
        for (int r = 0; r < kChunk; ++r) {
          fwd_step<V>(c, s0, s1, stage[r * cta_cols]);
          if (valid) {
            if constexpr (kOut & 1) st_cs_f2(xp, s1);
            if constexpr (kOut & 2) st_cs_f4(sp, make_float4(s0.x, s0.y, s1.x, s1.y));
          }
          if constexpr (kOut & 1) xp += p.N;
          if constexpr (kOut & 2) sp += p.N;
        }
      } else {
        for (int r = 0; r < rows; ++r) {
          fwd_step<V>(c, s0, s1, stage[r * cta_cols]);
          if (valid) {
            if constexpr (kOut & 1) st_cs_f2(xp, s1);
            if constexpr (kOut & 2) st_cs_f4(sp, make_float4(s0.x, s0.y, s1.x, s1.y));
          }
          if constexpr (kOut & 1) xp += p.N;
          if constexpr (kOut & 2) sp += p.N;
        }
      }
      if (p.carries && valid && k + 1 < nchunks) p.carries[k * p.N + n] = make_float4(s0.x, s0.y, s1.x, s1.y);
      __syncthreads();  // every warp is done reading this slot
      if (threadIdx.x == 0 && k + p.ring < k1) {
        fence_proxy_async();
        mbar_expect_tx(&bars[slot], stage_bytes);
        tma_load_2d(ring_base + (size_t)slot * stage_bytes, &tm_bu, &bars[slot], (int32_t)(cta_col0 * 2),
                    (int32_t)((k + p.ring) * kChunk));
      }
      if (++slot == p.ring) { slot = 0; parity ^= 1; }
    }
    if (p.seg_end && valid) p.seg_end[(long long)blockIdx.y * p.N + n] = make_float4(s0.x, s0.y, s1.x, s1.y);
  } else {
    // Plain-load path for views TMA cannot describe (odd N, unaligned base):
    // register double-buffering of kBatch rows.
    constexpr int kBatch = 8;
    float2 cur[kBatch], nxt[kBatch];
    auto load = [&](float2* dst, long long t0) {
#pragma unroll
      for (int r = 0; r < kBatch; ++r) {
        const long long t = t0 + r;
        dst[r] = (valid && t < p.L) ? ld_nc_f2(p.bu + t * p.N + n) : make_float2(0.f, 0.f);
      }
    };
    load(cur, 0);
    for (long long t0 = 0; t0 < p.L; t0 += kBatch) {
      load(nxt, t0 + kBatch);
#pragma unroll
      for (int r = 0; r < kBatch; ++r) {
        const long long t = t0 + r;
        if (t < p.L) fwd_step<V>(c, s0, s1, cur[r]);     // the state after the last real step leaves through seg_end
        if (valid && t < p.L) {
          const long long off = t * p.N;
          if constexpr (kOut & 1) xp[off] = s1;
          if constexpr (kOut & 2) sp[off] = make_float4(s0.x, s0.y, s1.x, s1.y);
          if (p.carries && ((t + 1) % kChunk) == 0 && (t + 1) < p.L)
            p.carries[((t + 1) / kChunk - 1) * p.N + n] = make_float4(s0.x, s0.y, s1.x, s1.y);
        }
      }
#pragma unroll
      for (int r = 0; r < kBatch; ++r) cur[r] = nxt[r];
    }
    if (p.seg_end && valid) p.seg_end[n] = make_float4(s0.x, s0.y, s1.x, s1.y);
  }
}

// ---------------------------------------------------------------------------
// backward
// ---------------------------------------------------------------------------
struct BwdParams {
  const float* a;
  const float* g;
  const float* step;
  const float2* bu;        // [L, N]
  const float2* grad_x;    // [L, N]
  const float4* carry_src; // state at the end of row (c*carry_mul + carry_off), see below
  long long carry_mul, carry_off;
  float2* grad_bu;         // [L, N]
  float* partials;         // [kNumAcc, S*N] (segment-major inside each accumulator)
  long long L, N, P;
  int ring;
  long long seg_chunks;       // chunks per time segment (grid.y segments)
  const float4* lam_init;     // [S, N] adjoint entering each segment from the right, or null (zero)
  const float4* state_in;     // [N] state entering the first chunk (a time slice of a longer sequence), or null (zero)
  float4* lam_end;            // [S, N] adjoint leaving each segment on the left, or null
};

// Kahan-compensated add of a chunk-local sum into a running total.
__device__ __forceinline__ void kahan_add(float& sum, float& comp, float v) {
  const float y = v - comp;
  const float t = sum + y;
  comp = (t - sum) - y;
  sum = t;
}

// One adjoint step (dlinoss_imex1_cuda.cu:129-158 / dlinoss_im_cuda.cu:131-158).
// (l0, l1): adjoint of the state after this step; gx: upstream gradient on x_t;
// (p0, p1): state before the step; b: bu_t.  Updates the chunk-local pair
// accumulators `loc` (re and im products are kept apart and summed later) and
// returns grad_bu_t.
template <int V>
__device__ __forceinline__ float2 bwd_step(const Coef& c, float2& l0, float2& l1, float2 gx, float2 p0, float2 p1,
                                           float2 b, float2 (&loc)[kNumAcc]) {
  const float2 g1 = __fadd2_rn(l1, gx);
  if constexpr (V == kDiag) {
    // G = g_t + lam ; dlambda += G * conj(x_{t-1}) ; lam <- G * conj(lambda) ; grad_b = G   (lru.py:69-78)
    const float2 rot = make_float2(g1.y, -g1.x);
    loc[0] = __ffma2_rn(g1, p1, loc[0]);     // Re: Gr*pr + Gi*pi
    loc[1] = __ffma2_rn(rot, p1, loc[1]);    // Im: Gi*pr - Gr*pi
    l1 = __ffma2_rn(rot, c.m12, __fmul2_rn(g1, c.m11));
    return g1;
  }
  if constexpr (V == kImex1) {
    const float2 gt = __fadd2_rn(l0, g1);
    loc[0] = __ffma2_rn(gt, p0, loc[0]);
    loc[1] = __ffma2_rn(gt, p1, loc[1]);
    loc[2] = __ffma2_rn(gt, b, loc[2]);
    l0 = __fmul2_rn(gt, c.m11);
    l1 = __ffma2_rn(gt, c.m12, g1);
    return __fmul2_rn(gt, c.f1);
  } else {
    const float2 g0 = l0;
    loc[0] = __ffma2_rn(g0, p0, loc[0]);
    loc[1] = __ffma2_rn(g0, p1, loc[1]);
    loc[2] = __ffma2_rn(g1, p0, loc[2]);
    loc[3] = __ffma2_rn(g1, p1, loc[3]);
    loc[4] = __ffma2_rn(g0, b, loc[4]);
    loc[5] = __ffma2_rn(g1, b, loc[5]);
    l0 = __ffma2_rn(g1, c.m21, __fmul2_rn(g0, c.m11));
    l1 = __ffma2_rn(g1, c.m22, __fmul2_rn(g0, c.m12));
    return __ffma2_rn(g1, c.f2, __fmul2_rn(g0, c.f1));
  }
}

// Per-series partial sums (real inner products over time):
//   generic variants: acc = { <g0,p0>, <g0,p1>, <g1,p0>, <g1,p1>, <g0,bu>, <g1,bu> }
//   imex1           : acc = { <gt,p0>, <gt,p1>, <gt,bu>, 0, 0, 0 }  with gt = g0 + g1
// (g0,g1) = adjoint after adding the upstream gradient, (p0,p1) = previous state.
template <int V, bool kTma, int kW = 0>
__global__ void __launch_bounds__(128, 1)
lti_backward_kernel(const __grid_constant__ CUtensorMap tm_bu, const __grid_constant__ CUtensorMap tm_gx,
                    BwdParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const int warp = threadIdx.x >> 5;
  const int warps = kW > 0 ? kW : (int)(blockDim.x >> 5);
  const int cta_cols = warps * kCols;
  const long long cta_col0 = (long long)blockIdx.x * cta_cols;
  const long long n = cta_col0 + threadIdx.x;
  const bool valid = n < p.N;
  if (!kTma && cta_col0 + (long long)warp * kCols >= p.N) return;
  const long long ch = valid ? (n % p.P) : 0;
  const Coef c = make_coef<V>(p.a[ch], p.g ? p.g[ch] : 0.0f, p.step ? p.step[ch] : 0.0f);
  const long long nchunks = (p.L + kChunk - 1) / kChunk;

  float acc[kNumAcc], comp[kNumAcc];
#pragma unroll
  for (int i = 0; i < kNumAcc; ++i) { acc[i] = 0.f; comp[i] = 0.f; }
  const long long k0 = (long long)blockIdx.y * p.seg_chunks;            // this CTA's time segment [k0, k1)
  const long long k1 = (k0 + p.seg_chunks) < nchunks ? (k0 + p.seg_chunks) : nchunks;
  const long long nseg = k1 - k0;
  float2 l0 = make_float2(0.f, 0.f), l1 = make_float2(0.f, 0.f);  // adjoint carried to earlier times
  if (p.lam_init && valid) {
    const float4 v = p.lam_init[(long long)blockIdx.y * p.N + n];
    l0 = make_float2(v.x, v.y);
    l1 = make_float2(v.z, v.w);
  }

  auto load_carry = [&](long long chunk) -> float4 {
    if (!valid) return make_float4(0.f, 0.f, 0.f, 0.f);
    if (chunk <= 0) return p.state_in ? ld_nc_f4(p.state_in + n) : make_float4(0.f, 0.f, 0.f, 0.f);
    return ld_nc_f4(p.carry_src + (chunk * p.carry_mul + p.carry_off) * p.N + n);
  };

  // Stage = bu tile followed by grad_x tile, shared by all warps of the CTA
  // (rows of warps*256 contiguous bytes per TMA box).
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw);
  unsigned char* ring_base = smem_raw + 1024;
  const uint32_t tile_bytes = (uint32_t)warps * kStageBytes;
  const uint32_t pair_bytes = 2 * tile_bytes;
  if constexpr (kTma) {
    if (threadIdx.x == 0) {
      prefetch_tensormap(&tm_bu);
      prefetch_tensormap(&tm_gx);
      for (int s = 0; s < p.ring; ++s) mbar_init(&bars[s], 1);
      fence_barrier_init();
      fence_proxy_async();
      const int pre = (int)(nseg < p.ring ? nseg : p.ring);
      for (int s = 0; s < pre; ++s) {
        const int32_t row = (int32_t)((k1 - 1 - s) * kChunk);
        unsigned char* dst = ring_base + (size_t)s * pair_bytes;
        mbar_expect_tx(&bars[s], pair_bytes);
        tma_load_2d(dst, &tm_bu, &bars[s], (int32_t)(cta_col0 * 2), row);
        tma_load_2d(dst + tile_bytes, &tm_gx, &bars[s], (int32_t)(cta_col0 * 2), row);
      }
    }
    __syncthreads();
  }

  int slot = 0;
  uint32_t parity = 0;
  float4 carry = load_carry(k1 - 1);
  for (long long k = 0; k < nseg; ++k) {
    const long long chunk = k1 - 1 - k;
    const long long t0 = chunk * kChunk;
    const float4 carry_next = load_carry(chunk - 1);  // prefetch for the next iteration
    const int rows = (int)((p.L - t0) < kChunk ? (p.L - t0) : kChunk);

    float2 p0[kChunk], p1[kChunk];
    float2 s0 = make_float2(carry.x, carry.y), s1 = make_float2(carry.z, carry.w);
    float2 loc[kNumAcc];
#pragma unroll
    for (int i = 0; i < kNumAcc; ++i) loc[i] = make_float2(0.f, 0.f);
    float2* gbp = p.grad_bu + (t0 + kChunk - 1) * p.N + n;  // walks backwards

    if constexpr (kTma) {
      if (!mbar_wait(&bars[slot], parity)) return;
      const float2* sbu = reinterpret_cast<const float2*>(ring_base + (size_t)slot * pair_bytes) + threadIdx.x;
      const float2* sgx = reinterpret_cast<const float2*>(ring_base + (size_t)slot * pair_bytes + tile_bytes) + threadIdx.x;
      // forward re-scan of the chunk, remembering the state *before* each step
      // (rows past the end of the sequence hold zeros: harmless to step through)
#pragma unroll
      for (int r = 0; r < kChunk; ++r) {
        p0[r] = s0; p1[r] = s1;
        fwd_step<V>(c, s0, s1, sbu[r * cta_cols]);
      }
      // adjoint recurrence, right to left
      if (rows == kChunk) {
#pragma unroll
        for (int r = kChunk - 1; r >= 0; --r) {
          const float2 gb = bwd_step<V>(c, l0, l1, sgx[r * cta_cols], p0[r], p1[r], sbu[r * cta_cols], loc);
          if (valid) st_cs_f2(gbp, gb);
          gbp -= p.N;
        }
      } else {
#pragma unroll
        for (int r = kChunk - 1; r >= 0; --r) {
          if (r < rows) {  // warp-uniform
            const float2 gb = bwd_step<V>(c, l0, l1, sgx[r * cta_cols], p0[r], p1[r], sbu[r * cta_cols], loc);
            if (valid) st_cs_f2(gbp, gb);
          }
          gbp -= p.N;
        }
      }
    } else {
      float2 rbu[kChunk], rgx[kChunk];
#pragma unroll
      for (int r = 0; r < kChunk; ++r) {
        const long long t = t0 + r;
        const bool ok = valid && t < p.L;
        rbu[r] = ok ? ld_nc_f2(p.bu + t * p.N + n) : make_float2(0.f, 0.f);
        rgx[r] = ok ? ld_nc_f2(p.grad_x + t * p.N + n) : make_float2(0.f, 0.f);
      }
#pragma unroll
      for (int r = 0; r < kChunk; ++r) {
        p0[r] = s0; p1[r] = s1;
        fwd_step<V>(c, s0, s1, rbu[r]);
      }
#pragma unroll
      for (int r = kChunk - 1; r >= 0; --r) {
        if (r < rows) {
          const float2 gb = bwd_step<V>(c, l0, l1, rgx[r], p0[r], p1[r], rbu[r], loc);
          if (valid) *gbp = gb;
        }
        gbp -= p.N;
      }
    }
#pragma unroll
    for (int i = 0; i < kNumAcc; ++i) kahan_add(acc[i], comp[i], loc[i].x + loc[i].y);

    if constexpr (kTma) {
      __syncthreads();  // every warp is done reading this slot
      if (threadIdx.x == 0 && k + p.ring < nseg) {
        const int32_t row = (int32_t)((chunk - p.ring) * kChunk);
        unsigned char* dst = ring_base + (size_t)slot * pair_bytes;
        fence_proxy_async();
        mbar_expect_tx(&bars[slot], pair_bytes);
        tma_load_2d(dst, &tm_bu, &bars[slot], (int32_t)(cta_col0 * 2), row);
        tma_load_2d(dst + tile_bytes, &tm_gx, &bars[slot], (int32_t)(cta_col0 * 2), row);
      }
      if (++slot == p.ring) { slot = 0; parity ^= 1; }
    }
    carry = carry_next;
  }
  if (valid) {
    const long long SN = (long long)gridDim.y * p.N;
#pragma unroll
    for (int i = 0; i < kNumAcc; ++i) p.partials[(long long)i * SN + (long long)blockIdx.y * p.N + n] = acc[i];
    if (p.lam_end) p.lam_end[(long long)blockIdx.y * p.N + n] = make_float4(l0.x, l0.y, l1.x, l1.y);
  }
}

// Adjoint summary of a time segment: runs lam <- M^T (lam + e2 * g_t) right to left
// over the segment from lam = 0 and writes lam at the segment's left end.  Reads
// grad_x only (8 B/elem).  Same staging as the other kernels.
template <int V>
__global__ void __launch_bounds__(128)
lti_adjoint_summary_kernel(const __grid_constant__ CUtensorMap tm_gx, BwdParams p, float4* seg_out) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const int warps = blockDim.x >> 5;
  const int cta_cols = warps * kCols;
  const long long cta_col0 = (long long)blockIdx.x * cta_cols;
  const long long n = cta_col0 + threadIdx.x;
  const bool valid = n < p.N;
  const long long ch = valid ? (n % p.P) : 0;
  const Coef c = make_coef<V>(p.a[ch], p.g ? p.g[ch] : 0.0f, p.step ? p.step[ch] : 0.0f);
  const long long nchunks = (p.L + kChunk - 1) / kChunk;
  const long long k0 = (long long)blockIdx.y * p.seg_chunks;
  const long long k1 = (k0 + p.seg_chunks) < nchunks ? (k0 + p.seg_chunks) : nchunks;
  const long long nseg = k1 - k0;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw);
  unsigned char* ring_base = smem_raw + 1024;
  const uint32_t stage_bytes = (uint32_t)warps * kStageBytes;
  if (threadIdx.x == 0) {
    prefetch_tensormap(&tm_gx);
    for (int s = 0; s < p.ring; ++s) mbar_init(&bars[s], 1);
    fence_barrier_init();
    fence_proxy_async();
    const int pre = (int)(nseg < p.ring ? nseg : p.ring);
    for (int s = 0; s < pre; ++s) {
      mbar_expect_tx(&bars[s], stage_bytes);
      tma_load_2d(ring_base + (size_t)s * stage_bytes, &tm_gx, &bars[s], (int32_t)(cta_col0 * 2),
                  (int32_t)((k1 - 1 - s) * kChunk));
    }
  }
  __syncthreads();
  float2 l0 = make_float2(0.f, 0.f), l1 = make_float2(0.f, 0.f);
  int slot = 0;
  uint32_t parity = 0;
  for (long long k = 0; k < nseg; ++k) {
    const long long chunk = k1 - 1 - k;
    if (!mbar_wait(&bars[slot], parity)) return;
    const float2* sgx = reinterpret_cast<const float2*>(ring_base + (size_t)slot * stage_bytes) + threadIdx.x;
    // rows past the end of the sequence hold zeros and leave lam = 0 unchanged
#pragma unroll
    for (int r = kChunk - 1; r >= 0; --r) {
      const float2 g1 = __fadd2_rn(l1, sgx[r * cta_cols]);
      if constexpr (V == kImex1) {
        const float2 gt = __fadd2_rn(l0, g1);
        l0 = __fmul2_rn(gt, c.m11);
        l1 = __ffma2_rn(gt, c.m12, g1);
      } else {
        const float2 g0 = l0;
        l0 = __ffma2_rn(g1, c.m21, __fmul2_rn(g0, c.m11));
        l1 = __ffma2_rn(g1, c.m22, __fmul2_rn(g0, c.m12));
      }
    }
    __syncthreads();
    if (threadIdx.x == 0 && k + p.ring < nseg) {
      fence_proxy_async();
      mbar_expect_tx(&bars[slot], stage_bytes);
      tma_load_2d(ring_base + (size_t)slot * stage_bytes, &tm_gx, &bars[slot], (int32_t)(cta_col0 * 2),
                  (int32_t)((chunk - p.ring) * kChunk));
    }
    if (++slot == p.ring) { slot = 0; parity ^= 1; }
  }
  if (valid) seg_out[(long long)blockIdx.y * p.N + n] = make_float4(l0.x, l0.y, l1.x, l1.y);
}

// Stitches the segment summaries together: with T = M^len (the transition over a
// whole segment, by repeated squaring in double precision) the state entering
// segment s+1 is  c_{s+1} = T c_s + e_s  (forward, kAdjoint = false; e_s = state
// leaving segment s when started from zero), and the adjoint entering segment s
// from the right is  lam_s = (M^T)^len_{s+1} lam_{s+1} + r_{s+1}  (kAdjoint = true).
// One thread per series.
template <int V, bool kAdjoint>
__global__ void lti_segment_combine_kernel(const float* __restrict__ a, const float* __restrict__ g,
                                           const float* __restrict__ step, const float4* __restrict__ summary,
                                           float4* __restrict__ init, long long L, long long N, long long P,
                                           long long seg_chunks, int S) {
  const long long n = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= N) return;
  const long long ch = n % P;
  const Coef c = make_coef<V>(a[ch], g ? g[ch] : 0.0f, step ? step[ch] : 0.0f);
  // the map one step applies to the state (imex1: x' = w' + x makes the second row (m11, 1 + m12))
  double m11 = c.m11.x, m12 = c.m12.x, m21, m22;
  if constexpr (V == kImex1) { m21 = m11; m22 = 1.0 + m12; } else { m21 = c.m21.x; m22 = c.m22.x; }
  if (kAdjoint) { const double t = m12; m12 = m21; m21 = t; }
  auto power = [&](long long e, double (&T)[4]) {
    double b0 = m11, b1 = m12, b2 = m21, b3 = m22;
    T[0] = 1.0; T[1] = 0.0; T[2] = 0.0; T[3] = 1.0;
    while (e > 0) {
      if (e & 1) {
        const double t0 = T[0] * b0 + T[1] * b2, t1 = T[0] * b1 + T[1] * b3;
        const double t2 = T[2] * b0 + T[3] * b2, t3 = T[2] * b1 + T[3] * b3;
        T[0] = t0; T[1] = t1; T[2] = t2; T[3] = t3;
      }
      const double q0 = b0 * b0 + b1 * b2, q1 = b0 * b1 + b1 * b3;
      const double q2 = b2 * b0 + b3 * b2, q3 = b2 * b1 + b3 * b3;
      b0 = q0; b1 = q1; b2 = q2; b3 = q3;
      e >>= 1;
    }
  };
  const long long full = seg_chunks * kChunk;
  double T[4];
  power(full, T);
  double v[4] = {0.0, 0.0, 0.0, 0.0};   // (s0.re, s0.im, s1.re, s1.im)
  if (!kAdjoint) {
    init[n] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s + 1 < S; ++s) {
      const float4 e = summary[(long long)s * N + n];
      const double n0r = T[0] * v[0] + T[1] * v[2] + e.x, n0i = T[0] * v[1] + T[1] * v[3] + e.y;
      const double n1r = T[2] * v[0] + T[3] * v[2] + e.z, n1i = T[2] * v[1] + T[3] * v[3] + e.w;
      v[0] = n0r; v[1] = n0i; v[2] = n1r; v[3] = n1i;
      init[(long long)(s + 1) * N + n] = make_float4((float)v[0], (float)v[1], (float)v[2], (float)v[3]);
    }
  } else {
    init[(long long)(S - 1) * N + n] = make_float4(0.f, 0.f, 0.f, 0.f);
    const long long last = L - (long long)(S - 1) * full;   // steps in the rightmost segment
    double Tl[4];
    power(last, Tl);
    for (int s = S - 2; s >= 0; --s) {
      const double* U = (s == S - 2) ? Tl : T;              // transition over segment s+1
      const float4 e = summary[(long long)(s + 1) * N + n];
      const double n0r = U[0] * v[0] + U[1] * v[2] + e.x, n0i = U[0] * v[1] + U[1] * v[3] + e.y;
      const double n1r = U[2] * v[0] + U[3] * v[2] + e.z, n1i = U[2] * v[1] + U[3] * v[3] + e.w;
      v[0] = n0r; v[1] = n0i; v[2] = n1r; v[3] = n1i;
      init[(long long)s * N + n] = make_float4((float)v[0], (float)v[1], (float)v[2], (float)v[3]);
    }
  }
}

// Fixed-order batch reduction of the per-series partials + chain rule to
// (A, G, step) in double precision.  A block covers kPgCh channels with
// kPgGroups batch groups: thread (cx, gy) sums the series b = gy, gy+kPgGroups,
// ... of channel cx, then thread (cx, 0) adds the group sums in group order, so
// the result does not depend on scheduling.
// Chain rules: dlinoss_imex1_cuda.cu:160-172, dlinoss_im_cuda.cu:160-187,
// dlinoss_imex2_cuda.cu:146-196, dlinoss_ex_cuda.cu:135-160; LinOSS by
// differentiating linoss.py:244-258 / 295-300.
constexpr int kPgCh = 32;
constexpr int kPgGroups = 16;

template <int V>
__global__ void __launch_bounds__(kPgCh * kPgGroups)
lti_param_grad_kernel(const float* __restrict__ a, const float* __restrict__ g, const float* __restrict__ step,
                      const float* __restrict__ partials, float* __restrict__ grad_a, float* __restrict__ grad_g,
                      float* __restrict__ grad_step, long long B, long long P) {
  __shared__ double red[kNumAcc][kPgGroups][kPgCh];
  const int cx = threadIdx.x % kPgCh;
  const int gy = threadIdx.x / kPgCh;
  const long long pch = (long long)blockIdx.x * kPgCh + cx;
  const long long N = B * P;
  constexpr int kUsed = (V == kImex1) ? 3 : (V == kDiag ? 2 : kNumAcc);  // sums actually accumulated
  double s[kNumAcc];
#pragma unroll
  for (int i = 0; i < kNumAcc; ++i) s[i] = 0.0;
  if (pch < P) {
#pragma unroll 4
    for (long long b = gy; b < B; b += kPgGroups) {
#pragma unroll
      for (int i = 0; i < kUsed; ++i) s[i] += (double)partials[(long long)i * N + b * P + pch];
    }
  }
#pragma unroll
  for (int i = 0; i < kUsed; ++i) red[i][gy][cx] = s[i];
  __syncthreads();
  if (gy != 0 || pch >= P) return;
#pragma unroll
  for (int i = 0; i < kUsed; ++i) {
    double t = red[i][0][cx];
    for (int k = 1; k < kPgGroups; ++k) t += red[i][k][cx];
    s[i] = t;
  }
  const double al = a[pch], ga = g ? g[pch] : 0.0, si = step ? step[pch] : 0.0;
  double da = 0.0, dg = 0.0, ds = 0.0;
  if constexpr (V == kDiag) {
    da = s[0];   // Re sum G conj(x_{t-1})
    dg = s[1];   // Im
  } else if constexpr (V == kImex1) {
    // s = { <gt,p0>, <gt,p1>, <gt,bu> }
    const double inv = 1.0 / (1.0 + si * ga);
    const double s2i = si * si * inv;
    const double d_s2i = s[2] - al * s[1];
    da = -s2i * s[1];
    const double d_inv = s[0] + si * si * d_s2i;
    ds = 2.0 * si * inv * d_s2i - ga * inv * inv * d_inv;
    dg = -si * inv * inv * d_inv;
  } else {
    const double d11 = s[0], d12 = s[1], d21 = s[2], d22 = s[3], df1 = s[4], df2 = s[5];
    if constexpr (V == kImex2) {
      da = -si * d12 - si * si * d22;
      dg = -si * d11 - si * si * d21;
      ds = -ga * d11 - al * d12 + (1.0 - 2.0 * si * ga) * d21 - 2.0 * si * al * d22 + df1 + 2.0 * si * df2;
    } else if constexpr (V == kIm) {
      const double inv = 1.0 / (1.0 + si * ga + si * si * al);
      const double d_inv = d11 - al * si * d12 + si * d21 + (1.0 + si * ga) * d22 + si * df1 + si * si * df2;
      const double d_den = -inv * inv * d_inv;
      da = -si * inv * d12 + si * si * d_den;
      dg = si * inv * d22 + si * d_den;
      ds = -al * inv * d12 + inv * d21 + ga * inv * d22 + inv * df1 + 2.0 * si * inv * df2 +
           (ga + 2.0 * si * al) * d_den;
    } else if constexpr (V == kEx) {
      da = -si * d12;
      dg = -si * d11;
      ds = -ga * d11 - al * d12 + d21 + df1;
    } else if constexpr (V == kLinossIm) {
      const double schur = 1.0 / (1.0 + si * si * al);
      const double m11 = 1.0 - si * si * al * schur, m21 = si * schur;
      const double t11 = d11 + si * df1, t21 = d21 + si * df2;
      const double d_sch = -si * si * al * t11 - si * al * d12 + si * t21 + d22;
      da = -si * si * schur * t11 - si * schur * d12 - schur * schur * si * si * d_sch;
      ds = m11 * df1 + m21 * df2 - 2.0 * si * al * schur * t11 - al * schur * d12 + schur * t21 -
           schur * schur * 2.0 * si * al * d_sch;
    } else {  // kLinossImex
      da = -si * d12 - si * si * d22;
      ds = -al * d12 + d21 - 2.0 * si * al * d22 + df1 + 2.0 * si * df2;
    }
  }
  grad_a[pch] = (float)da;
  if (grad_g) grad_g[pch] = (float)dg;
  if (grad_step) grad_step[pch] = (float)ds;
}

#include "lti_scan_twolevel.cuh"

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
struct Tuning {
  int fwd_ring = 2;
  int fwd_warps = 4;
  int bwd_ring = 2;
  int bwd_warps = 4;
  int force_plain = 0;
  int segments = 0;   // 0 = automatic
  int twolevel = 1;   // 1 = two-level kernels for long sequences of few series, 0 = never
  int tl_fwd_ring = 0;   // stages of the two-level kernels, 0 = by CTA count (measured best)
  int tl_bwd_ring = 0;
};
static Tuning g_tuning;

// Long sequences of few series take the two-level kernels (lti_scan_twolevel.cuh): enough series for
// 96 CTAs of 16 columns, too few for the wide kernels to fill the GPU, and at least four tiles of time.
// The upper bound also keeps the backward's partial sums (6 * 8 * N floats) inside the built-in
// scratch of the allocation-free entry, so that entry and the workspace entry always take the same path.
static bool use_twolevel(int variant, long long L, long long N) {
  if (!g_tuning.twolevel || g_tuning.segments > 0 || g_tuning.force_plain || variant == kDiag) return false;
  return N >= 1536 && N <= 8192 && L >= 4 * kTlRows;
}

template <typename K>
static int set_smem(K kernel, size_t bytes) {
  return ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), bytes);
}

// Number of time segments.  A sequence is split only when the series alone cannot
// occupy the GPU (few column tiles) and it is long enough; each segment then costs
// one extra read of its input for the summary pass.
template <int V>
static int pick_segments_for(long long L, long long N, int warps);

static int pick_segments(long long L, long long N, int warps) {
  if (g_tuning.segments > 0) {
    const long long nchunks = (L + kChunk - 1) / kChunk;
    return (int)(g_tuning.segments < nchunks ? g_tuning.segments : nchunks);
  }
  const long long tiles = (N + (long long)kCols * warps - 1) / ((long long)kCols * warps);
  if (tiles >= 96) return 1;
  const long long nchunks = (L + kChunk - 1) / kChunk;
  long long S = sm_count() / tiles;
  if (S > 16) S = 16;
  if (S > nchunks / 16) S = nchunks / 16;   // at least 512 steps per segment
  return S < 2 ? 1 : (int)S;
}

// The stitching kernel assumes a real transition shared by the real and imaginary parts;
// the complex diagonal scan is therefore never split.
template <int V>
static int pick_segments_for(long long L, long long N, int warps) {
  return V == kDiag ? 1 : pick_segments(L, N, warps);
}

static size_t twolevel_backward_ws_bytes(long long N) { return (size_t)kNumAcc * kTlSub * N * sizeof(float); }
static size_t forward_ws_bytes(int S, long long N) { return S > 1 ? (size_t)2 * S * N * sizeof(float4) : 0; }
static size_t backward_ws_bytes(int S, long long N) {
  return (size_t)kNumAcc * S * N * sizeof(float) + (S > 1 ? (size_t)2 * S * N * sizeof(float4) : 0);
}

template <int V, int kOut>
static int launch_forward_out(const FwdParams& p, cudaStream_t stream, void* workspace, size_t ws_bytes) {
  CUtensorMap tm;
  memset(&tm, 0, sizeof(tm));
  const int tw = g_tuning.fwd_warps;
  const bool tma = !g_tuning.force_plain &&
                   make_tensor_map_2d_f32(&tm, p.bu, (uint64_t)p.N * 2, (uint64_t)p.L, (uint64_t)p.N * 8,
                                          kCols * 2 * tw, kChunk);
  const int warps = tma ? tw : 4;
  const long long tiles = (p.N + kCols - 1) / kCols;
  const long long grid = (tiles + warps - 1) / warps;
  if (grid > 0x7fffffffLL) {
    set_last_error("lti_scan_forward: B*P too large");
    return kErrInvalidArgument;
  }
  const long long nchunks = (p.L + kChunk - 1) / kChunk;
  FwdParams q = p;
  q.seg_chunks = nchunks;
  // a time slice of a longer sequence (state handed in / out by the caller) runs as one segment
  const bool slice = p.seg_init != nullptr || p.seg_end != nullptr;
  if (tma && !slice && use_twolevel(V, p.L, p.N)) {
    CUtensorMap tm2;
    memset(&tm2, 0, sizeof(tm2));
    if (make_tensor_map_2d_f32(&tm2, p.bu, (uint64_t)p.N * 2, (uint64_t)p.L, (uint64_t)p.N * 8, kTlCols * 2,
                               kTlRows)) {
      const unsigned ctas = (unsigned)((p.N + kTlCols - 1) / kTlCols);
      // one CTA per SM wants a deep ring of its own; with several waves the co-resident CTAs overlap instead
      q.ring = g_tuning.tl_fwd_ring > 0 ? g_tuning.tl_fwd_ring : ((int)ctas <= sm_count() ? 3 : 4);
      const size_t smem = 4096 + (size_t)q.ring * kTlTileBytes;
      if (int rc = set_smem(lti_forward_twolevel_kernel<V, kOut>, smem)) return rc;
      lti_forward_twolevel_kernel<V, kOut><<<ctas, kTlThreads, smem, stream>>>(tm2, q);
      return check_cuda(cudaGetLastError(), "lti_forward_twolevel_kernel launch");
    }
  }
  if (tma) {
    q.ring = g_tuning.fwd_ring;
    const size_t smem = 1024 + (size_t)warps * q.ring * kStageBytes;
    int S = slice ? 1 : pick_segments_for<V>(p.L, p.N, warps);
    if (workspace == nullptr || ws_bytes < forward_ws_bytes(S, p.N)) S = 1;
    if (S > 1) {
      // pass 1: per-segment end states from zero; pass 2: stitch; pass 3: the scan proper
      float4* seg_end = static_cast<float4*>(workspace);
      float4* seg_init = seg_end + (size_t)S * p.N;
      q.seg_chunks = (nchunks + S - 1) / S;
      S = (int)((nchunks + q.seg_chunks - 1) / q.seg_chunks);
      FwdParams sum = q;
      sum.x = nullptr; sum.states = nullptr; sum.carries = nullptr; sum.seg_end = seg_end;
      if (int rc = set_smem(lti_forward_kernel<V, true, 0>, smem)) return rc;
      lti_forward_kernel<V, true, 0><<<dim3((unsigned)grid, S), warps * 32, smem, stream>>>(tm, sum);
      if (int rc = check_cuda(cudaGetLastError(), "lti_forward_kernel (summary) launch")) return rc;
      lti_segment_combine_kernel<V, false><<<(unsigned)((p.N + 127) / 128), 128, 0, stream>>>(
          p.a, p.g, p.step, seg_end, seg_init, p.L, p.N, p.P, q.seg_chunks, S);
      if (int rc = check_cuda(cudaGetLastError(), "lti_segment_combine_kernel launch")) return rc;
      q.seg_init = seg_init;
    }
    if (warps == 4) {
      if (int rc = set_smem(lti_forward_kernel<V, true, kOut, 4>, smem)) return rc;
      lti_forward_kernel<V, true, kOut, 4><<<dim3((unsigned)grid, S), warps * 32, smem, stream>>>(tm, q);
    } else {
      if (int rc = set_smem(lti_forward_kernel<V, true, kOut>, smem)) return rc;
      lti_forward_kernel<V, true, kOut><<<dim3((unsigned)grid, S), warps * 32, smem, stream>>>(tm, q);
    }
  } else {
    q.ring = 0;
    lti_forward_kernel<V, false, kOut><<<(unsigned)grid, warps * 32, 0, stream>>>(tm, q);
  }
  return check_cuda(cudaGetLastError(), "lti_forward_kernel launch");
}

template <int V>
static int launch_forward(const FwdParams& p, cudaStream_t stream, void* workspace, size_t ws_bytes) {
  if (p.x && p.states) return launch_forward_out<V, 3>(p, stream, workspace, ws_bytes);
  if (p.states) return launch_forward_out<V, 2>(p, stream, workspace, ws_bytes);
  return launch_forward_out<V, 1>(p, stream, workspace, ws_bytes);
}

template <int V>
static int launch_backward(const BwdParams& p, float* grad_a, float* grad_g, float* grad_step, long long B,
                           cudaStream_t stream, size_t ws_bytes) {
  CUtensorMap tm_bu, tm_gx;
  memset(&tm_bu, 0, sizeof(tm_bu));
  memset(&tm_gx, 0, sizeof(tm_gx));
  const int tw = g_tuning.bwd_warps;
  const bool tma = !g_tuning.force_plain &&
                   make_tensor_map_2d_f32(&tm_bu, p.bu, (uint64_t)p.N * 2, (uint64_t)p.L, (uint64_t)p.N * 8,
                                          kCols * 2 * tw, kChunk) &&
                   make_tensor_map_2d_f32(&tm_gx, p.grad_x, (uint64_t)p.N * 2, (uint64_t)p.L, (uint64_t)p.N * 8,
                                          kCols * 2 * tw, kChunk);
  const int warps = tma ? tw : 2;
  const long long tiles = (p.N + kCols - 1) / kCols;
  const long long grid = (tiles + warps - 1) / warps;
  if (grid > 0x7fffffffLL) {
    set_last_error("lti_scan_backward: B*P too large");
    return kErrInvalidArgument;
  }
  const long long nchunks = (p.L + kChunk - 1) / kChunk;
  BwdParams q = p;
  q.seg_chunks = nchunks;
  const bool slice = p.lam_init != nullptr || p.lam_end != nullptr || p.state_in != nullptr;
  int S = 1;
  if (tma && !slice && use_twolevel(V, p.L, p.N) && ws_bytes >= twolevel_backward_ws_bytes(p.N)) {
    CUtensorMap tb, tg;
    memset(&tb, 0, sizeof(tb));
    memset(&tg, 0, sizeof(tg));
    if (make_tensor_map_2d_f32(&tb, p.bu, (uint64_t)p.N * 2, (uint64_t)p.L, (uint64_t)p.N * 8, kTlCols * 2, kTlRows) &&
        make_tensor_map_2d_f32(&tg, p.grad_x, (uint64_t)p.N * 2, (uint64_t)p.L, (uint64_t)p.N * 8, kTlCols * 2,
                               kTlRows)) {
      const unsigned ctas = (unsigned)((p.N + kTlCols - 1) / kTlCols);
      // a single stage lets two CTAs share an SM (68 KiB each), which wins once there are several waves
      q.ring = g_tuning.tl_bwd_ring > 0 ? g_tuning.tl_bwd_ring : ((int)ctas <= sm_count() ? 2 : 1);
      const size_t smem = 4096 + (size_t)q.ring * 2 * kTlTileBytes;
      if (int rc = set_smem(lti_backward_twolevel_kernel<V>, smem)) return rc;
      lti_backward_twolevel_kernel<V><<<ctas, kTlThreads, smem, stream>>>(tb, tg, q);
      if (int rc = check_cuda(cudaGetLastError(), "lti_backward_twolevel_kernel launch")) return rc;
      const unsigned blocks = (unsigned)((p.P + kPgCh - 1) / kPgCh);
      // the sub-chunk positions of a series are summed like extra batch entries
      lti_param_grad_kernel<V><<<blocks, kPgCh * kPgGroups, 0, stream>>>(p.a, p.g, p.step, p.partials, grad_a, grad_g,
                                                                       grad_step, B * kTlSub, p.P);
      return check_cuda(cudaGetLastError(), "lti_param_grad_kernel launch");
    }
  }
  if (tma) {
    q.ring = g_tuning.bwd_ring;
    S = slice ? 1 : pick_segments_for<V>(p.L, p.N, warps);
    if (ws_bytes < backward_ws_bytes(S, p.N)) S = 1;
    if (S > 1) {
      q.seg_chunks = (nchunks + S - 1) / S;
      S = (int)((nchunks + q.seg_chunks - 1) / q.seg_chunks);
      float4* seg_sum = reinterpret_cast<float4*>(p.partials + (size_t)kNumAcc * S * p.N);
      float4* seg_init = seg_sum + (size_t)S * p.N;
      const size_t smem1 = 1024 + (size_t)warps * q.ring * kStageBytes;
      if (int rc = set_smem(lti_adjoint_summary_kernel<V>, smem1)) return rc;
      lti_adjoint_summary_kernel<V><<<dim3((unsigned)grid, S), warps * 32, smem1, stream>>>(tm_gx, q, seg_sum);
      if (int rc = check_cuda(cudaGetLastError(), "lti_adjoint_summary_kernel launch")) return rc;
      lti_segment_combine_kernel<V, true><<<(unsigned)((p.N + 127) / 128), 128, 0, stream>>>(
          p.a, p.g, p.step, seg_sum, seg_init, p.L, p.N, p.P, q.seg_chunks, S);
      if (int rc = check_cuda(cudaGetLastError(), "lti_segment_combine_kernel launch")) return rc;
      q.lam_init = seg_init;
    }
    const size_t smem = 1024 + (size_t)warps * q.ring * 2 * kStageBytes;
    if (warps == 4) {
      if (int rc = set_smem(lti_backward_kernel<V, true, 4>, smem)) return rc;
      lti_backward_kernel<V, true, 4><<<dim3((unsigned)grid, S), warps * 32, smem, stream>>>(tm_bu, tm_gx, q);
    } else {
      if (int rc = set_smem(lti_backward_kernel<V, true>, smem)) return rc;
      lti_backward_kernel<V, true><<<dim3((unsigned)grid, S), warps * 32, smem, stream>>>(tm_bu, tm_gx, q);
    }
  } else {
    q.ring = 0;
    lti_backward_kernel<V, false><<<(unsigned)grid, warps * 32, 0, stream>>>(tm_bu, tm_gx, q);
  }
  if (int rc = check_cuda(cudaGetLastError(), "lti_backward_kernel launch")) return rc;
  const int threads = kPgCh * kPgGroups;
  const unsigned blocks = (unsigned)((p.P + kPgCh - 1) / kPgCh);
  // the segments of a series are summed like extra batch entries
  lti_param_grad_kernel<V><<<blocks, threads, 0, stream>>>(p.a, p.g, p.step, p.partials, grad_a, grad_g, grad_step,
                                                           B * S, p.P);
  return check_cuda(cudaGetLastError(), "lti_param_grad_kernel launch");
}

static bool variant_ok(int v) { return v >= kImex1 && v <= kDiag; }
static bool needs_g(int v) { return v <= kEx || v == kDiag; }
static bool needs_step(int v) { return v != kDiag; }

#define OSSM_DISPATCH_VARIANT(v, CALL)                  \
  switch (v) {                                          \
    case kImex1: { constexpr int V = kImex1; return CALL; }       \
    case kImex2: { constexpr int V = kImex2; return CALL; }       \
    case kIm: { constexpr int V = kIm; return CALL; }             \
    case kEx: { constexpr int V = kEx; return CALL; }             \
    case kLinossIm: { constexpr int V = kLinossIm; return CALL; } \
    case kDiag: { constexpr int V = kDiag; return CALL; }         \
    default: { constexpr int V = kLinossImex; return CALL; }      \
  }

static int forward_dispatch(int variant, const FwdParams& p, cudaStream_t stream, void* ws, size_t ws_bytes) {
  OSSM_DISPATCH_VARIANT(variant, launch_forward<V>(p, stream, ws, ws_bytes));
}

static int backward_dispatch(int variant, const BwdParams& p, float* ga, float* gg, float* gs, long long B,
                             cudaStream_t stream, size_t ws_bytes) {
  OSSM_DISPATCH_VARIANT(variant, launch_backward<V>(p, ga, gg, gs, B, stream, ws_bytes));
}

}  // namespace lti
}  // namespace ossm_b200

extern "C" {

using namespace ossm_b200;
using namespace ossm_b200::lti;

int ossm_b200_lti_chunk(void) { return kChunk; }

int ossm_b200_lti_set_tuning(const char* key, int value) {
  if (key == nullptr) return kErrInvalidArgument;
  if (!strcmp(key, "fwd_ring") && value >= 1 && value <= 24) { g_tuning.fwd_ring = value; return kOk; }
  if (!strcmp(key, "fwd_warps") && value >= 1 && value <= 4) { g_tuning.fwd_warps = value; return kOk; }
  if (!strcmp(key, "bwd_ring") && value >= 1 && value <= 12) { g_tuning.bwd_ring = value; return kOk; }
  if (!strcmp(key, "bwd_warps") && value >= 1 && value <= 4) { g_tuning.bwd_warps = value; return kOk; }
  if (!strcmp(key, "force_plain")) { g_tuning.force_plain = value != 0; return kOk; }
  if (!strcmp(key, "segments") && value >= 0 && value <= 64) { g_tuning.segments = value; return kOk; }
  if (!strcmp(key, "twolevel")) { g_tuning.twolevel = value != 0; return kOk; }
  if (!strcmp(key, "tl_fwd_ring") && value >= 0 && value <= 6) { g_tuning.tl_fwd_ring = value; return kOk; }
  if (!strcmp(key, "tl_bwd_ring") && value >= 0 && value <= 3) { g_tuning.tl_bwd_ring = value; return kOk; }
  set_last_error("lti_set_tuning: unknown key or value out of range: %s=%d", key, value);
  return kErrInvalidArgument;
}

size_t ossm_b200_lti_carry_bytes(int64_t L, int64_t B, int64_t P) {
  if (L <= 0 || B <= 0 || P <= 0) return 0;
  const int64_t nchunks = (L + kChunk - 1) / kChunk;
  return (size_t)(nchunks - 1) * (size_t)B * (size_t)P * 16;
}

size_t ossm_b200_lti_backward_workspace_bytes(int64_t L, int64_t B, int64_t P) {
  if (L <= 0 || B <= 0 || P <= 0) return 0;
  const int S = g_tuning.segments > 0 ? 64 : pick_segments(L, B * P, g_tuning.bwd_warps);
  const size_t seg = backward_ws_bytes(S, B * P);
  const size_t two = use_twolevel(kImex1, L, B * P) ? twolevel_backward_ws_bytes(B * P) : 0;
  return seg > two ? seg : two;
}

size_t ossm_b200_lti_forward_workspace_bytes(int64_t L, int64_t B, int64_t P) {
  if (L <= 0 || B <= 0 || P <= 0) return 0;
  if (use_twolevel(kImex1, L, B * P)) return 0;   // the two-level forward needs no scratch
  const int S = g_tuning.segments > 0 ? 64 : pick_segments(L, B * P, g_tuning.fwd_warps);
  return forward_ws_bytes(S, B * P);
}

static int check_common(const char* fn, int variant, const void* a, const void* g, const void* step, int64_t L,
                        int64_t B, int64_t P) {
  if (!variant_ok(variant)) { set_last_error("%s: unknown variant %d", fn, variant); return kErrInvalidArgument; }
  if (L < 0 || B < 0 || P < 0) { set_last_error("%s: negative extent", fn); return kErrInvalidArgument; }
  if (a == nullptr || (needs_step(variant) && step == nullptr) || (needs_g(variant) && g == nullptr)) {
    set_last_error("%s: null coefficient pointer", fn);
    return kErrInvalidArgument;
  }
  if (L > 0x7fffffffLL - kChunk) { set_last_error("%s: L too large", fn); return kErrInvalidArgument; }
  return kOk;
}

int ossm_b200_lti_scan_forward_ws(int variant, const float* a, const float* g, const float* step, const void* bu,
                                  void* x, void* states, void* carries, void* workspace, size_t workspace_bytes,
                                  int64_t L, int64_t B, int64_t P, cudaStream_t stream) {
  if (int rc = check_common("lti_scan_forward", variant, a, g, step, L, B, P)) return rc;
  if (L == 0 || B == 0 || P == 0) return kOk;
  if (bu == nullptr || (x == nullptr && states == nullptr)) {
    set_last_error("lti_scan_forward: null bu or no output buffer");
    return kErrInvalidArgument;
  }
  if ((reinterpret_cast<uintptr_t>(bu) & 7u) || (reinterpret_cast<uintptr_t>(x) & 7u) ||
      (reinterpret_cast<uintptr_t>(states) & 15u) || (reinterpret_cast<uintptr_t>(carries) & 15u) ||
      (reinterpret_cast<uintptr_t>(workspace) & 15u)) {
    set_last_error("lti_scan_forward: misaligned buffer (bu/x need 8 B, states/carries/workspace 16 B)");
    return kErrInvalidArgument;
  }
  FwdParams p;
  p.a = a; p.g = needs_g(variant) ? g : nullptr; p.step = needs_step(variant) ? step : nullptr;
  p.bu = static_cast<const float2*>(bu);
  p.x = static_cast<float2*>(x);
  p.states = static_cast<float4*>(states);
  p.carries = static_cast<float4*>(carries);
  p.L = L; p.N = B * P; p.P = P; p.ring = 0;
  p.seg_chunks = 0; p.seg_init = nullptr; p.seg_end = nullptr;
  return forward_dispatch(variant, p, stream, workspace, workspace_bytes);
}

int ossm_b200_lti_scan_forward_slice(int variant, const float* a, const float* g, const float* step, const void* bu,
                                     void* x, void* carries, const void* state_in, void* state_out, int64_t L,
                                     int64_t B, int64_t P, cudaStream_t stream) {
  if (int rc = check_common("lti_scan_forward_slice", variant, a, g, step, L, B, P)) return rc;
  if (variant == kDiag) { set_last_error("lti_scan_forward_slice: not available for the diagonal variant"); return kErrUnsupported; }
  if (B == 0 || P == 0) return kOk;
  if (L == 0) {
    if (state_out == nullptr) return kOk;
    if (state_in) return check_cuda(cudaMemcpyAsync(state_out, state_in, (size_t)B * P * 16, cudaMemcpyDeviceToDevice, stream), "state copy");
    return check_cuda(cudaMemsetAsync(state_out, 0, (size_t)B * P * 16, stream), "state clear");
  }
  if (bu == nullptr || x == nullptr) { set_last_error("lti_scan_forward_slice: null bu or x"); return kErrInvalidArgument; }
  if ((reinterpret_cast<uintptr_t>(bu) & 7u) || (reinterpret_cast<uintptr_t>(x) & 7u) ||
      (reinterpret_cast<uintptr_t>(carries) & 15u) || (reinterpret_cast<uintptr_t>(state_in) & 15u) ||
      (reinterpret_cast<uintptr_t>(state_out) & 15u)) {
    set_last_error("lti_scan_forward_slice: misaligned buffer (bu/x need 8 B, carries/states 16 B)");
    return kErrInvalidArgument;
  }
  FwdParams p;
  p.a = a; p.g = needs_g(variant) ? g : nullptr; p.step = step;
  p.bu = static_cast<const float2*>(bu);
  p.x = static_cast<float2*>(x);
  p.states = nullptr;
  p.carries = static_cast<float4*>(carries);
  p.L = L; p.N = B * P; p.P = P; p.ring = 0; p.seg_chunks = 0;
  p.seg_init = static_cast<const float4*>(state_in);
  p.seg_end = static_cast<float4*>(state_out);
  return forward_dispatch(variant, p, stream, nullptr, 0);
}

int ossm_b200_lti_scan_forward(int variant, const float* a, const float* g, const float* step, const void* bu,
                               void* x, void* states, void* carries, int64_t L, int64_t B, int64_t P,
                               cudaStream_t stream) {
  // without scratch the sequence is never split into time segments
  return ossm_b200_lti_scan_forward_ws(variant, a, g, step, bu, x, states, carries, nullptr, 0, L, B, P, stream);
}

static int backward_common(const char* fn, int variant, const float* a, const float* g, const float* step,
                           const void* bu, const void* carry_src, long long mul, long long off, const void* grad_x,
                           void* grad_bu, float* grad_a, float* grad_g, float* grad_step, void* workspace,
                           size_t workspace_bytes, int64_t L, int64_t B, int64_t P, cudaStream_t stream,
                           const void* state_in = nullptr, const void* adjoint_in = nullptr,
                           void* adjoint_out = nullptr) {
  if (int rc = check_common(fn, variant, a, g, step, L, B, P)) return rc;
  if (grad_a == nullptr || (needs_step(variant) && grad_step == nullptr) || (needs_g(variant) && grad_g == nullptr)) {
    set_last_error("%s: null coefficient-gradient pointer", fn);
    return kErrInvalidArgument;
  }
  if (P == 0) return kOk;
  if (L == 0 || B == 0) {
    if (int rc = check_cuda(cudaMemsetAsync(grad_a, 0, P * sizeof(float), stream), fn)) return rc;
    if (grad_g) if (int rc = check_cuda(cudaMemsetAsync(grad_g, 0, P * sizeof(float), stream), fn)) return rc;
    if (grad_step == nullptr) return kOk;
    return check_cuda(cudaMemsetAsync(grad_step, 0, P * sizeof(float), stream), fn);
  }
  if (bu == nullptr || grad_x == nullptr || grad_bu == nullptr) {
    set_last_error("%s: null bu / grad_x / grad_bu", fn);
    return kErrInvalidArgument;
  }
  const int64_t nchunks = (L + kChunk - 1) / kChunk;
  if (nchunks > 1 && carry_src == nullptr) {
    set_last_error("%s: carries/states required when L > %d", fn, kChunk);
    return kErrInvalidArgument;
  }
  if ((reinterpret_cast<uintptr_t>(bu) & 7u) || (reinterpret_cast<uintptr_t>(grad_x) & 7u) ||
      (reinterpret_cast<uintptr_t>(grad_bu) & 7u) || (reinterpret_cast<uintptr_t>(carry_src) & 15u) ||
      (reinterpret_cast<uintptr_t>(workspace) & 15u)) {
    set_last_error("%s: misaligned buffer", fn);
    return kErrInvalidArgument;
  }
  if (workspace == nullptr || workspace_bytes < backward_ws_bytes(1, B * P)) {
    set_last_error("%s: workspace too small (%zu < %zu bytes)", fn, workspace_bytes, backward_ws_bytes(1, B * P));
    return kErrWorkspace;
  }
  BwdParams p;
  p.a = a; p.g = needs_g(variant) ? g : nullptr; p.step = needs_step(variant) ? step : nullptr;
  p.bu = static_cast<const float2*>(bu);
  p.grad_x = static_cast<const float2*>(grad_x);
  p.carry_src = static_cast<const float4*>(carry_src);
  p.carry_mul = mul; p.carry_off = off;
  p.grad_bu = static_cast<float2*>(grad_bu);
  p.partials = static_cast<float*>(workspace);
  p.L = L; p.N = B * P; p.P = P; p.ring = 0;
  p.seg_chunks = 0;
  p.lam_init = static_cast<const float4*>(adjoint_in);
  p.state_in = static_cast<const float4*>(state_in);
  p.lam_end = static_cast<float4*>(adjoint_out);
  return backward_dispatch(variant, p, grad_a, needs_g(variant) ? grad_g : nullptr,
                           needs_step(variant) ? grad_step : nullptr, B, stream,
                           workspace_bytes);
}

int ossm_b200_lti_scan_backward(int variant, const float* a, const float* g, const float* step, const void* bu,
                                const void* carries, const void* grad_x, void* grad_bu, float* grad_a,
                                float* grad_g, float* grad_step, void* workspace, size_t workspace_bytes, int64_t L,
                                int64_t B, int64_t P, cudaStream_t stream) {
  // carries row r = state after step (r+1)*kChunk - 1 = carry-in of chunk r+1
  return backward_common("lti_scan_backward", variant, a, g, step, bu, carries, 1, -1, grad_x, grad_bu, grad_a,
                         grad_g, grad_step, workspace, workspace_bytes, L, B, P, stream);
}

int ossm_b200_lti_scan_backward_slice(int variant, const float* a, const float* g, const float* step, const void* bu,
                                      const void* carries, const void* state_in, const void* grad_x,
                                      const void* adjoint_in, void* adjoint_out, void* grad_bu, float* grad_a,
                                      float* grad_g, float* grad_step, void* workspace, size_t workspace_bytes,
                                      int64_t L, int64_t B, int64_t P, cudaStream_t stream) {
  if (variant == kDiag) { set_last_error("lti_scan_backward_slice: not available for the diagonal variant"); return kErrUnsupported; }
  if ((reinterpret_cast<uintptr_t>(state_in) & 15u) || (reinterpret_cast<uintptr_t>(adjoint_in) & 15u) ||
      (reinterpret_cast<uintptr_t>(adjoint_out) & 15u)) {
    set_last_error("lti_scan_backward_slice: state / adjoint buffers need 16-byte alignment");
    return kErrInvalidArgument;
  }
  if (L == 0 && B > 0 && P > 0 && adjoint_out != nullptr) {
    // an empty slice passes the adjoint through
    if (adjoint_in) {
      if (int rc = check_cuda(cudaMemcpyAsync(adjoint_out, adjoint_in, (size_t)B * P * 16, cudaMemcpyDeviceToDevice, stream), "adjoint copy")) return rc;
    } else if (int rc = check_cuda(cudaMemsetAsync(adjoint_out, 0, (size_t)B * P * 16, stream), "adjoint clear")) {
      return rc;
    }
  }
  return backward_common("lti_scan_backward_slice", variant, a, g, step, bu, carries, 1, -1, grad_x, grad_bu, grad_a,
                         grad_g, grad_step, workspace, workspace_bytes, L, B, P, stream, state_in, adjoint_in,
                         adjoint_out);
}

// ---------------------------------------------------------------------------
// Backward without any allocation by the caller or by this library.
//
// Some hosts of this code cannot hand out scratch memory at call time: a plugin
// running inside an inference server or a real-time control loop that forbids
// device allocation after start-up, or a binding written in a language whose
// runtime owns no CUDA allocator (a cgo / JNI stub that only forwards pointers it
// was given).  For them the per-series partial sums of the backward live in a
// fixed array inside the library image instead of a caller-supplied workspace.
// The array is part of every context that loads the library (kStaticSeries * 6
// floats = 1.5 MiB per GPU, held until the process exits).
// ---------------------------------------------------------------------------
namespace ossm_b200 {
namespace lti {
constexpr long long kStaticSeries = 65536;  // largest B*P the allocation-free entry point accepts
static __device__ __align__(256) float g_static_partials[kNumAcc * kStaticSeries];

// The array's name is only a host-side handle; the kernels need its device
// address, which differs per device.  Looked up once per device, with that device
// current, and cached.
static int static_partials_ptr(float** out) {
  static float* cached[64] = {nullptr};
  int dev = -1;
  if (int rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice")) return rc;
  if (dev < 0 || dev >= 64) {
    set_last_error("lti_scan_backward_static: device ordinal %d out of range", dev);
    return kErrUnsupported;
  }
  if (cached[dev] == nullptr) {
    void* ptr = nullptr;
    if (int rc = check_cuda(cudaGetSymbolAddress(&ptr, g_static_partials), "cudaGetSymbolAddress(static scratch)"))
      return rc;
    cached[dev] = static_cast<float*>(ptr);
  }
  *out = cached[dev];
  return kOk;
}
}  // namespace lti
}  // namespace ossm_b200

size_t ossm_b200_lti_scan_backward_static_max_series(void) { return (size_t)ossm_b200::lti::kStaticSeries; }

int ossm_b200_lti_scan_backward_static(int variant, const float* a, const float* g, const float* step,
                                       const void* bu, const void* carries, const void* grad_x, void* grad_bu,
                                       float* grad_a, float* grad_g, float* grad_step, int64_t L, int64_t B,
                                       int64_t P, cudaStream_t stream) {
  if (B > 0 && P > 0 && (B > kStaticSeries || P > kStaticSeries || B * P > kStaticSeries)) {
    set_last_error("lti_scan_backward_static: B*P = %lld series exceed the built-in scratch (%lld); use "
                   "lti_scan_backward with a caller workspace",
                   (long long)(B * P), (long long)kStaticSeries);
    return kErrWorkspace;
  }
  float* scratch = nullptr;
  if (int rc = static_partials_ptr(&scratch)) return rc;
  return backward_common("lti_scan_backward_static", variant, a, g, step, bu, carries, 1, -1, grad_x, grad_bu,
                         grad_a, grad_g, grad_step, scratch, sizeof(float) * kNumAcc * kStaticSeries, L, B, P,
                         stream);
}

int ossm_b200_lti_scan_backward_states(int variant, const float* a, const float* g, const float* step,
                                       const void* bu, const void* states, const void* grad_x, void* grad_bu,
                                       float* grad_a, float* grad_g, float* grad_step, void* workspace,
                                       size_t workspace_bytes, int64_t L, int64_t B, int64_t P,
                                       cudaStream_t stream) {
  // full trajectory given: the carry-in of chunk c is states row c*kChunk - 1
  return backward_common("lti_scan_backward_states", variant, a, g, step, bu, states, kChunk, -1, grad_x, grad_bu,
                         grad_a, grad_g, grad_step, workspace, workspace_bytes, L, B, P, stream);
}

}  // extern "C"
