// Causal depthwise conv1d + bias + SiLU of the Mamba mixer, forward and backward (sm_100a).
//
// The mixer (src/ossm/models/mambarec.py:143-151) takes x = in_proj(inputs)[..., :D] of shape [B, L, D],
// transposes it to [B, D, L], pads K-1 zeros on the left, runs nn.Conv1d(groups = D) and nn.SiLU, and
// transposes back for x_proj: five passes over [B, D, L].  The result is needed in BOTH layouts -- time
// contiguous [B, D, L] for the selective scan, channel contiguous [B, L, D] for the x_proj GEMM -- so one
// kernel reads x once (through a shared-memory tile that also does the transpose) and writes both.
//
//   pre[b,d,t] = bias[d] + sum_k w[d,k] * x[b, t - (K-1) + k, d]        (zero for negative time)
//   out        = pre * sigmoid(pre)
//
// HBM-bound elementwise work: 4 B read + 8 B written per element forward; backward reads x and the two
// upstream gradients (one per layout) and writes grad_x.  The weight and bias gradients are sums over
// (batch, time): reduced over the CTA in shared memory, then one atomic add per (channel, tap) and CTA.
#include "common.cuh"

#include "../../include/ossm_b200.h"

namespace ossm_b200 {
OSSM_B200_STATUS_ACCESSOR(status_mixer)
namespace mixer {

constexpr int kTileT = 64;      // time steps per CTA
constexpr int kTileD = 32;      // channels per CTA
constexpr int kMaxTaps = 4;     // kernel sizes 1..4 (Mamba's d_conv default is 4)
constexpr int kRowsY = 8;       // threadIdx.y extent

struct ConvParams {
  const float* x;        // [B, L, D] with row pitch ldx floats
  const float* w;        // [D, K]
  const float* bias;     // [D] or null
  float* out_bdl;        // [B, D, L] or null
  float* out_bld;        // [B, L, D] or null
  // backward
  const float* g_bdl;    // [B, D, L] or null
  const float* g_bld;    // [B, L, D] or null
  float* grad_x;         // [B, L, D]
  float* grad_w;         // [D, K], zero on entry
  float* grad_bias;      // [D] or null, zero on entry
  long long B, L, D, ldx;
  int taps;
};

// Scalar kernels: any shape and alignment (odd channel counts, sequence lengths that are not multiples of 4).
// K = number of taps (compile time: the tap loops unroll and the halo is a constant).  Index arithmetic is kept in
// 32 bits inside a tile and in running pointers across rows; they are bound by instruction issue, not by HBM,
// which is why aligned shapes take the vector kernels below.
template <int K>
__global__ void __launch_bounds__(kTileD * kRowsY) conv_silu_forward_kernel(ConvParams p) {
  constexpr int halo = K - 1;
  __shared__ float xin[kTileT + halo][kTileD + 1];
  __shared__ float yout[kTileT][kTileD + 1];
  const int tx = threadIdx.x, ty = threadIdx.y;
  const long long b = blockIdx.z;
  const int d0 = blockIdx.y * kTileD;
  const long long t0 = (long long)blockIdx.x * kTileT;
  const int d = d0 + tx;
  const bool dok = d < (int)p.D;
  const int rows_left = (int)((p.L - t0) < (kTileT) ? (p.L - t0) : kTileT);      // real time steps in this tile
  {
    const float* src = p.x + (b * p.L + t0 - halo + ty) * p.ldx + d;
    const long long step = (long long)kRowsY * p.ldx;
#pragma unroll
    for (int r = ty; r < kTileT + halo; r += kRowsY, src += step) {
      const bool ok = dok && (t0 + r >= halo) && (r - halo < rows_left);
      xin[r][tx] = ok ? __ldg(src) : 0.0f;
    }
  }
  float w[K];
#pragma unroll
  for (int k = 0; k < K; ++k) w[k] = dok ? __ldg(p.w + d * K + k) : 0.0f;
  const float bias = (p.bias && dok) ? __ldg(p.bias + d) : 0.0f;
  __syncthreads();
  {
    float* dst = p.out_bld ? p.out_bld + (b * p.L + t0 + ty) * p.D + d : nullptr;
    const long long step = (long long)kRowsY * p.D;
#pragma unroll
    for (int r = ty; r < kTileT; r += kRowsY) {
      float pre = bias;
#pragma unroll
      for (int k = 0; k < K; ++k) pre = fmaf(w[k], xin[r + k][tx], pre);
      const float y = __fdividef(pre, 1.0f + __expf(-pre));
      yout[r][tx] = y;
      if (dst) {
        if (dok && r < rows_left) *dst = y;
        dst += step;
      }
    }
  }
  if (p.out_bdl == nullptr) return;
  __syncthreads();
  // transposed store: consecutive threads write consecutive time steps of one channel
  const int lin = ty * kTileD + tx;
#pragma unroll
  for (int i = lin; i < kTileT * kTileD; i += kTileD * kRowsY) {
    const int dd = i / kTileT, tt = i % kTileT;
    if (d0 + dd < (int)p.D && tt < rows_left) p.out_bdl[(b * p.D + d0 + dd) * p.L + t0 + tt] = yout[tt][dd];
  }
}

template <int K>
__global__ void __launch_bounds__(kTileD * kRowsY) conv_silu_backward_kernel(ConvParams p) {
  constexpr int halo = K - 1;
  __shared__ float xin[kTileT + 2 * halo][kTileD + 1];     // x for t0-halo .. t0+T+halo
  __shared__ float dpre[kTileT + halo][kTileD + 1];        // d(pre) for t0 .. t0+T+halo
  __shared__ float red[kRowsY][K + 1][kTileD];
  const int tx = threadIdx.x, ty = threadIdx.y;
  const long long b = blockIdx.z;
  const int d0 = blockIdx.y * kTileD;
  const long long t0 = (long long)blockIdx.x * kTileT;
  const int d = d0 + tx;
  const bool dok = d < (int)p.D;
  const long long left = p.L - t0;                          // time steps from t0 to the end of the sequence
  const int rows_ext = (int)(left < kTileT + halo ? left : kTileT + halo);    // real steps among tile + right halo
  {
    const float* src = p.x + (b * p.L + t0 - halo + ty) * p.ldx + d;
    const long long step = (long long)kRowsY * p.ldx;
#pragma unroll
    for (int r = ty; r < kTileT + 2 * halo; r += kRowsY, src += step) {
      const bool ok = dok && (t0 + r >= halo) && (r - halo < left);
      xin[r][tx] = ok ? __ldg(src) : 0.0f;
    }
  }
  // upstream gradient of the time-contiguous output, transposed through dpre as staging
  if (p.g_bdl) {
    const int lin = ty * kTileD + tx;
    for (int i = lin; i < (kTileT + halo) * kTileD; i += kTileD * kRowsY) {
      const int dd = i / (kTileT + halo), tt = i % (kTileT + halo);
      dpre[tt][dd] = (d0 + dd < (int)p.D && tt < rows_ext) ? __ldg(p.g_bdl + (b * p.D + d0 + dd) * p.L + t0 + tt) : 0.0f;
    }
  }
  float w[K];
#pragma unroll
  for (int k = 0; k < K; ++k) w[k] = dok ? __ldg(p.w + d * K + k) : 0.0f;
  const float bias = (p.bias && dok) ? __ldg(p.bias + d) : 0.0f;
  __syncthreads();
  float acc_w[K], acc_b = 0.f;
#pragma unroll
  for (int k = 0; k < K; ++k) acc_w[k] = 0.f;
  {
    const float* g2 = p.g_bld ? p.g_bld + (b * p.L + t0 + ty) * p.D + d : nullptr;
    const long long step = (long long)kRowsY * p.D;
#pragma unroll
    for (int r = ty; r < kTileT + halo; r += kRowsY) {
      const bool live = dok && r < rows_ext;
      float g = p.g_bdl ? dpre[r][tx] : 0.0f;
      if (g2) {
        if (live) g += __ldg(g2);
        g2 += step;
      }
      float pre = bias;
#pragma unroll
      for (int k = 0; k < K; ++k) pre = fmaf(w[k], xin[r + k][tx], pre);   // x index of output t0 + r is r + k
      const float sg = __fdividef(1.0f, 1.0f + __expf(-pre));
      const float dp = live ? g * (sg * fmaf(pre, 1.0f - sg, 1.0f)) : 0.0f;
      dpre[r][tx] = dp;
      if (r < kTileT) {       // the halo rows belong to the next tile's sums
        acc_b += dp;
#pragma unroll
        for (int k = 0; k < K; ++k) acc_w[k] = fmaf(dp, xin[r + k][tx], acc_w[k]);
      }
    }
  }
  __syncthreads();
  {
    // grad_x[t] = sum_k w[k] * dpre[t + halo - k]
    float* dst = p.grad_x + (b * p.L + t0 + ty) * p.D + d;
    const long long step = (long long)kRowsY * p.D;
#pragma unroll
    for (int r = ty; r < kTileT; r += kRowsY, dst += step) {
      float gx = 0.0f;
#pragma unroll
      for (int k = 0; k < K; ++k) gx = fmaf(w[k], dpre[r + halo - k][tx], gx);
      if (dok && r < left) *dst = gx;
    }
  }
#pragma unroll
  for (int k = 0; k < K; ++k) red[ty][k][tx] = acc_w[k];
  red[ty][K][tx] = acc_b;
  __syncthreads();
  if (ty == 0 && dok) {
#pragma unroll
    for (int k = 0; k <= K; ++k) {
      float s = 0.0f;
#pragma unroll
      for (int j = 0; j < kRowsY; ++j) s += red[j][k][tx];
      if (k < K) atomicAdd(p.grad_w + d * K + k, s);
      else if (p.grad_bias) atomicAdd(p.grad_bias + d, s);
    }
  }
}


// ---------------------------------------------------------------------------------------------
// Vector kernels: the path of every shape the mixer produces (even channel count and pitch, 8-byte aligned
// rows; sequence length a multiple of 4 where the time-contiguous layout is read or written).  A thread owns
// two channel pairs (float2 at channels 2*lane and 64 + 2*lane of a 128-channel block) and walks 16 time
// steps with the taps in registers, so a warp's global accesses are 256 contiguous bytes and the per-element
// index arithmetic of the scalar kernels is shared by 64 elements.  Shared memory is used for the transpose
// only: rows of 130 floats make both the float2 row writes and the 4-times-by-8-channels transposed reads
// conflict-free ((2*(4*tq + i) + c8) mod 32 is a bijection of (tq, c8)), and the time-contiguous layout moves
// as float4, four lanes per 64-byte run of one channel.
constexpr int kVT = 64;          // time steps per tile
constexpr int kVD = 128;         // channels per CTA
constexpr int kVWarps = 4;
constexpr int kVSteps = kVT / kVWarps;
constexpr int kVPitch = 130;

__device__ __forceinline__ float2 ldg2(const float* p) { return __ldg(reinterpret_cast<const float2*>(p)); }

template <int K>
__global__ void __launch_bounds__(32 * kVWarps, 5) conv_silu_forward_vec_kernel(ConvParams p) {
  constexpr int halo = K - 1;
  __shared__ __align__(16) float tile[kVT][kVPitch];
  const int lane = threadIdx.x, w = threadIdx.y;
  const long long b = blockIdx.z;
  const int d0 = blockIdx.y * kVD;
  const long long t0 = (long long)blockIdx.x * kVT;
  const long long ts = t0 + w * kVSteps;
  const int D = (int)p.D;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int c = 64 * h + 2 * lane;
    const bool ok = d0 + c < D;
    float2 wt[K];
#pragma unroll
    for (int k = 0; k < K; ++k)
      wt[k] = ok ? make_float2(__ldg(p.w + (d0 + c) * K + k), __ldg(p.w + (d0 + c + 1) * K + k)) : make_float2(0.f, 0.f);
    const float2 bias = (ok && p.bias) ? ldg2(p.bias + d0 + c) : make_float2(0.f, 0.f);
    float2 xv[kVSteps + halo];
    {
      const float* src = p.x + (b * p.L + ts - halo) * p.ldx + d0 + c;
#pragma unroll
      for (int j = 0; j < kVSteps + halo; ++j, src += p.ldx) {
        const long long t = ts - halo + j;
        xv[j] = (ok && t >= 0 && t < p.L) ? ldg2(src) : make_float2(0.f, 0.f);
      }
    }
    float* dst = p.out_bld ? p.out_bld + (b * p.L + ts) * p.D + d0 + c : nullptr;
#pragma unroll
    for (int i = 0; i < kVSteps; ++i) {
      float2 pre = bias;
#pragma unroll
      for (int k = 0; k < K; ++k) {
        pre.x = fmaf(wt[k].x, xv[i + k].x, pre.x);
        pre.y = fmaf(wt[k].y, xv[i + k].y, pre.y);
      }
      float2 y;
      y.x = __fdividef(pre.x, 1.0f + __expf(-pre.x));
      y.y = __fdividef(pre.y, 1.0f + __expf(-pre.y));
      *reinterpret_cast<float2*>(&tile[w * kVSteps + i][c]) = y;
      if (dst) {
        if (ok && ts + i < p.L) *reinterpret_cast<float2*>(dst) = y;
        dst += p.D;
      }
    }
  }
  if (p.out_bdl == nullptr) return;
  __syncthreads();
  const int tq = lane & 3, c8 = lane >> 2;
#pragma unroll 4
  for (int it = w; it < (kVD / 8) * (kVT / 16); it += kVWarps) {
    const int cc = (it >> 2) * 8 + c8, tt = (it & 3) * 16 + tq * 4;
    const float4 v = make_float4(tile[tt][cc], tile[tt + 1][cc], tile[tt + 2][cc], tile[tt + 3][cc]);
    if (d0 + cc < D && t0 + tt < p.L)
      *reinterpret_cast<float4*>(p.out_bdl + (b * p.D + d0 + cc) * p.L + t0 + tt) = v;
  }
}

// One CTA walks `tiles_per_cta` consecutive time tiles of one (batch entry, block of 64 channels: one float2 per
// thread, which keeps the kernel near 128 registers) and keeps the weight and bias sums in registers across them:
// one shared-memory reduction and one atomic add per (channel, tap) at the end.
constexpr int kVDB = 64;
constexpr int kVPitchB = kVDB + 2;
template <int K>
__global__ void __launch_bounds__(32 * kVWarps, 4) conv_silu_backward_vec_kernel(ConvParams p, int tiles_per_cta) {
  constexpr int halo = K - 1;
  constexpr int kRows = kVT + halo;
  static_assert(kRows * kVPitchB >= kVWarps * (K + 1) * kVDB, "reduction reuses the tile");
  __shared__ __align__(16) float tile[kRows][kVPitchB];     // upstream gradient of the time-contiguous output
  const int lane = threadIdx.x, w = threadIdx.y;
  const long long b = blockIdx.z;
  const int d0 = blockIdx.y * kVDB;
  const int D = (int)p.D;
  const int tq = lane & 3, c8 = lane >> 2;
  const int c = 2 * lane;
  const bool ok = d0 + c < D;
  float2 wt[K], accw[K];
#pragma unroll
  for (int k = 0; k < K; ++k) {
    wt[k] = ok ? make_float2(__ldg(p.w + (d0 + c) * K + k), __ldg(p.w + (d0 + c + 1) * K + k)) : make_float2(0.f, 0.f);
    accw[k] = make_float2(0.f, 0.f);
  }
  const float2 bias = (ok && p.bias) ? ldg2(p.bias + d0 + c) : make_float2(0.f, 0.f);
  float2 accb = make_float2(0.f, 0.f);
  for (int ti = 0; ti < tiles_per_cta; ++ti) {
    const long long t0 = ((long long)blockIdx.x * tiles_per_cta + ti) * kVT;
    if (t0 >= p.L) break;
    if (p.g_bdl) {
      if (ti) __syncthreads();        // the previous tile has been consumed
#pragma unroll 4
      for (int it = w; it < (kVDB / 8) * (kVT / 16); it += kVWarps) {
        const int cc = (it >> 2) * 8 + c8, tt = (it & 3) * 16 + tq * 4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (d0 + cc < D && t0 + tt < p.L)
          v = __ldg(reinterpret_cast<const float4*>(p.g_bdl + (b * p.D + d0 + cc) * p.L + t0 + tt));
        tile[tt][cc] = v.x; tile[tt + 1][cc] = v.y; tile[tt + 2][cc] = v.z; tile[tt + 3][cc] = v.w;
      }
      for (int i = w * 32 + lane; i < halo * kVDB; i += 32 * kVWarps) {     // the K-1 steps after the tile
        const int r = kVT + i / kVDB, cc = i % kVDB;
        tile[r][cc] = (d0 + cc < D && t0 + r < p.L) ? __ldg(p.g_bdl + (b * p.D + d0 + cc) * p.L + t0 + r) : 0.0f;
      }
      __syncthreads();
    }
    const long long ts = t0 + w * kVSteps;
    float2 xv[kVSteps + 2 * halo];
    {
      const float* src = p.x + (b * p.L + ts - halo) * p.ldx + d0 + c;
#pragma unroll
      for (int j = 0; j < kVSteps + 2 * halo; ++j, src += p.ldx) {
        const long long t = ts - halo + j;
        xv[j] = (ok && t >= 0 && t < p.L) ? ldg2(src) : make_float2(0.f, 0.f);
      }
    }
    float2 gv[kVSteps + halo];
    {
      const float* src = p.g_bld ? p.g_bld + (b * p.L + ts) * p.D + d0 + c : nullptr;
#pragma unroll
      for (int j = 0; j < kVSteps + halo; ++j)
        gv[j] = (src && ok && ts + j < p.L) ? ldg2(src + (long long)j * p.D) : make_float2(0.f, 0.f);
    }
    float2 dp[kVSteps + halo];
    float* dst = p.grad_x + (b * p.L + ts) * p.D + d0 + c;
#pragma unroll
    for (int j = 0; j < kVSteps + halo; ++j) {
      float2 g = gv[j];
      if (p.g_bdl) {
        const float2 s = *reinterpret_cast<const float2*>(&tile[w * kVSteps + j][c]);
        g.x += s.x; g.y += s.y;
      }
      float2 pre = bias;
#pragma unroll
      for (int k = 0; k < K; ++k) {
        pre.x = fmaf(wt[k].x, xv[j + k].x, pre.x);
        pre.y = fmaf(wt[k].y, xv[j + k].y, pre.y);
      }
      const float sx = __fdividef(1.0f, 1.0f + __expf(-pre.x)), sy = __fdividef(1.0f, 1.0f + __expf(-pre.y));
      const bool live = ok && ts + j < p.L;
      dp[j].x = live ? g.x * (sx * fmaf(pre.x, 1.0f - sx, 1.0f)) : 0.0f;
      dp[j].y = live ? g.y * (sy * fmaf(pre.y, 1.0f - sy, 1.0f)) : 0.0f;
      if (j < kVSteps) {          // the steps after the warp's own belong to the next warp's sums
        accb.x += dp[j].x; accb.y += dp[j].y;
#pragma unroll
        for (int k = 0; k < K; ++k) {
          accw[k].x = fmaf(dp[j].x, xv[j + k].x, accw[k].x);
          accw[k].y = fmaf(dp[j].y, xv[j + k].y, accw[k].y);
        }
      }
      if (j >= halo) {            // grad_x[ts + j - halo] = sum_k w[k] * dpre[ts + j - k]
        float2 gx = make_float2(0.f, 0.f);
#pragma unroll
        for (int k = 0; k < K; ++k) {
          gx.x = fmaf(wt[k].x, dp[j - k].x, gx.x);
          gx.y = fmaf(wt[k].y, dp[j - k].y, gx.y);
        }
        if (ok && ts + j - halo < p.L) *reinterpret_cast<float2*>(dst) = gx;
        dst += p.D;
      }
    }
  }
  __syncthreads();
  float* red = &tile[0][0];            // [warp][K + 1][kVDB]
#pragma unroll
  for (int k = 0; k < K; ++k) *reinterpret_cast<float2*>(red + (w * (K + 1) + k) * kVDB + c) = accw[k];
  *reinterpret_cast<float2*>(red + (w * (K + 1) + K) * kVDB + c) = accb;
  __syncthreads();
  const int cr = w * 32 + lane;
  if (cr < kVDB && d0 + cr < D) {
#pragma unroll
    for (int k = 0; k <= K; ++k) {
      float s = 0.0f;
#pragma unroll
      for (int j = 0; j < kVWarps; ++j) s += red[(j * (K + 1) + k) * kVDB + cr];
      if (k < K) atomicAdd(p.grad_w + (d0 + cr) * K + k, s);
      else if (p.grad_bias) atomicAdd(p.grad_bias + d0 + cr, s);
    }
  }
}


// ---------------------------------------------------------------------------------------------
// Staged forward: the same arithmetic as the vector kernel, but x arrives through TMA.  A CTA owns 64 channels of
// one batch entry and walks consecutive time tiles; a rank-3 tensor map (channels, time, batch) delivers each tile
// with its K-1 rows of history -- the rows before the start of the sequence come back as zeros, which is the causal
// padding -- into a ring of stages, several tiles ahead of the arithmetic, so that the loads in flight do not depend
// on registers or on how many warps are resident.
constexpr int kSC = 64;                 // channels per CTA = one 256-byte box row
constexpr int kSPitch = kSC + 2;        // transpose tile pitch (see the vector kernels)
constexpr int kSMaxRing = 6;

template <int K>
__global__ void __launch_bounds__(32 * kVWarps)
conv_silu_forward_staged_kernel(const __grid_constant__ CUtensorMap tm_x, ConvParams p, int tiles_per_cta, int ring) {
  constexpr int halo = K - 1;
  constexpr int kStageBytes = (kVT + halo) * kSC * 4;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw);
  unsigned char* ring_base = smem_raw + 1024;
  float (*turn)[kSPitch] = reinterpret_cast<float (*)[kSPitch]>(ring_base + (size_t)ring * kStageBytes);
  const int lane = threadIdx.x, w = threadIdx.y;
  const bool leader = lane == 0 && w == 0;
  const int b = blockIdx.z;
  const int d0 = blockIdx.y * kSC;
  const int D = (int)p.D;
  const long long tiles_all = (p.L + kVT - 1) / kVT;
  const long long tile0 = (long long)blockIdx.x * tiles_per_cta;
  const int ntiles = (int)(tiles_all - tile0 < tiles_per_cta ? tiles_all - tile0 : tiles_per_cta);
  if (leader) {
    prefetch_tensormap(&tm_x);
    for (int s = 0; s < ring; ++s) mbar_init(&bars[s], 1);
    fence_barrier_init();
    fence_proxy_async();
    for (int s = 0; s < ring && s < ntiles; ++s) {
      mbar_expect_tx(&bars[s], kStageBytes);
      tma_load_3d(ring_base + (size_t)s * kStageBytes, &tm_x, &bars[s], d0, (int32_t)((tile0 + s) * kVT) - halo, b);
    }
  }
  const int c = 2 * lane;
  const bool ok = d0 + c < D;
  float2 wt[K];
#pragma unroll
  for (int k = 0; k < K; ++k)
    wt[k] = ok ? make_float2(__ldg(p.w + (d0 + c) * K + k), __ldg(p.w + (d0 + c + 1) * K + k)) : make_float2(0.f, 0.f);
  const float2 bias = (ok && p.bias) ? ldg2(p.bias + d0 + c) : make_float2(0.f, 0.f);
  const int tq = lane & 3, c8 = lane >> 2;
  __syncthreads();
  int slot = 0;
  uint32_t parity = 0;
  for (int i = 0; i < ntiles; ++i) {
    const long long t0 = (tile0 + i) * kVT;
    const long long ts = t0 + w * kVSteps;
    if (!mbar_wait(&bars[slot], parity)) return;
    const float2* rows = reinterpret_cast<const float2*>(ring_base + (size_t)slot * kStageBytes) +
                         (size_t)(w * kVSteps) * (kSC / 2) + lane;      // row r holds time t0 - halo + r
    float2 xv[kVSteps + halo];
#pragma unroll
    for (int j = 0; j < kVSteps + halo; ++j) xv[j] = rows[j * (kSC / 2)];
    float* dst = p.out_bld ? p.out_bld + ((long long)b * p.L + ts) * p.D + d0 + c : nullptr;
#pragma unroll
    for (int s = 0; s < kVSteps; ++s) {
      float2 pre = bias;
#pragma unroll
      for (int k = 0; k < K; ++k) {
        pre.x = fmaf(wt[k].x, xv[s + k].x, pre.x);
        pre.y = fmaf(wt[k].y, xv[s + k].y, pre.y);
      }
      float2 y;
      y.x = __fdividef(pre.x, 1.0f + __expf(-pre.x));
      y.y = __fdividef(pre.y, 1.0f + __expf(-pre.y));
      if (p.out_bdl) *reinterpret_cast<float2*>(&turn[w * kVSteps + s][c]) = y;
      if (dst) {
        if (ok && ts + s < p.L) *reinterpret_cast<float2*>(dst) = y;
        dst += p.D;
      }
    }
    __syncthreads();          // the stage has been read; the turn tile is complete
    if (leader && i + ring < ntiles) {
      fence_proxy_async();
      mbar_expect_tx(&bars[slot], kStageBytes);
      tma_load_3d(ring_base + (size_t)slot * kStageBytes, &tm_x, &bars[slot], d0,
                  (int32_t)((tile0 + i + ring) * kVT) - halo, b);
    }
    if (p.out_bdl) {
#pragma unroll 4
      for (int it = w; it < (kSC / 8) * (kVT / 16); it += kVWarps) {
        const int cc = (it >> 2) * 8 + c8, tt = (it & 3) * 16 + tq * 4;
        const float4 v = make_float4(turn[tt][cc], turn[tt + 1][cc], turn[tt + 2][cc], turn[tt + 3][cc]);
        if (d0 + cc < D && t0 + tt < p.L)
          *reinterpret_cast<float4*>(p.out_bdl + ((long long)b * p.D + d0 + cc) * p.L + t0 + tt) = v;
      }
      __syncthreads();        // the turn tile may be overwritten
    }
    if (++slot == ring) { slot = 0; parity ^= 1; }
  }
}

// Tensor map (channels, time, batch) over x [B, L, D] with row pitch ldx; boxes of 64 channels x `rows` steps.
static bool staged_x_map(CUtensorMap* tm, const float* x, long long B, long long L, long long D, long long ldx,
                         uint32_t rows) {
  if ((ldx & 3) != 0 || rows > 256) return false;
  const uint64_t dims[3] = {(uint64_t)D, (uint64_t)L, (uint64_t)B};
  const uint64_t strides[2] = {(uint64_t)ldx * 4, (uint64_t)L * (uint64_t)ldx * 4};
  const uint32_t box[3] = {(uint32_t)kSC, rows, 1};
  return make_tensor_map_3d_f32(tm, x, dims, strides, box);
}

// Staged backward.  Stage = x rows [t0-(K-1), t0+64+(K-1)) | grad_bld rows [t0, t0+64+(K-1)) (both channel
// contiguous, 256 B per row) | grad_bdl as [64 channels][68 steps] (time contiguous; a thread reads its channels'
// steps with 16-byte loads).  Nothing is transposed by hand and nothing waits on a register load; the weight and
// bias sums stay in registers across the tiles a CTA walks.
template <int K>
__global__ void __launch_bounds__(32 * kVWarps)
conv_silu_backward_staged_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_g2,
                                 const __grid_constant__ CUtensorMap tm_g1, ConvParams p, int tiles_per_cta, int ring) {
  constexpr int halo = K - 1;
  constexpr int kXBytes = (kVT + 2 * halo) * kSC * 4;
  constexpr int kG2Bytes = (kVT + halo) * kSC * 4;
  constexpr int kG1Pitch = kVT + 4;                         // steps per channel row of the time-contiguous tile
  constexpr int kG1Bytes = kSC * kG1Pitch * 4;
  constexpr int kStageBytes = kXBytes + kG2Bytes + kG1Bytes;
  static_assert(kXBytes % 128 == 0 && kG2Bytes % 128 == 0 && kG1Bytes % 128 == 0, "TMA destinations stay 128-byte aligned");
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw);
  unsigned char* ring_base = smem_raw + 1024;
  const int lane = threadIdx.x, w = threadIdx.y;
  const bool leader = lane == 0 && w == 0;
  const int b = blockIdx.z;
  const int d0 = blockIdx.y * kSC;
  const int D = (int)p.D;
  const long long tiles_all = (p.L + kVT - 1) / kVT;
  const long long tile0 = (long long)blockIdx.x * tiles_per_cta;
  const int ntiles = (int)(tiles_all - tile0 < tiles_per_cta ? tiles_all - tile0 : tiles_per_cta);
  const uint32_t tx_bytes = kXBytes + (p.g_bld ? kG2Bytes : 0) + (p.g_bdl ? kG1Bytes : 0);
  auto issue = [&](int s, long long tile) {
    unsigned char* st = ring_base + (size_t)s * kStageBytes;
    const int32_t t0 = (int32_t)(tile * kVT);
    mbar_expect_tx(&bars[s], tx_bytes);
    tma_load_3d(st, &tm_x, &bars[s], d0, t0 - halo, b);
    if (p.g_bld) tma_load_3d(st + kXBytes, &tm_g2, &bars[s], d0, t0, b);
    if (p.g_bdl) tma_load_3d(st + kXBytes + kG2Bytes, &tm_g1, &bars[s], t0, d0, b);
  };
  if (leader) {
    prefetch_tensormap(&tm_x);
    if (p.g_bld) prefetch_tensormap(&tm_g2);
    if (p.g_bdl) prefetch_tensormap(&tm_g1);
    for (int s = 0; s < ring; ++s) mbar_init(&bars[s], 1);
    fence_barrier_init();
    fence_proxy_async();
    for (int s = 0; s < ring && s < ntiles; ++s) issue(s, tile0 + s);
  }
  const int c = 2 * lane;
  const bool ok = d0 + c < D;
  float2 wt[K], accw[K];
#pragma unroll
  for (int k = 0; k < K; ++k) {
    wt[k] = ok ? make_float2(__ldg(p.w + (d0 + c) * K + k), __ldg(p.w + (d0 + c + 1) * K + k)) : make_float2(0.f, 0.f);
    accw[k] = make_float2(0.f, 0.f);
  }
  const float2 bias = (ok && p.bias) ? ldg2(p.bias + d0 + c) : make_float2(0.f, 0.f);
  float2 accb = make_float2(0.f, 0.f);
  __syncthreads();
  int slot = 0;
  uint32_t parity = 0;
  for (int i = 0; i < ntiles; ++i) {
    const long long t0 = (tile0 + i) * kVT;
    const long long ts = t0 + w * kVSteps;
    if (!mbar_wait(&bars[slot], parity)) return;
    const unsigned char* st = ring_base + (size_t)slot * kStageBytes;
    const float2* xr = reinterpret_cast<const float2*>(st) + (size_t)(w * kVSteps) * (kSC / 2) + lane;   // time ts - halo + j
    const float2* g2r = reinterpret_cast<const float2*>(st + kXBytes) + (size_t)(w * kVSteps) * (kSC / 2) + lane;
    const float* g1a = reinterpret_cast<const float*>(st + kXBytes + kG2Bytes) + (size_t)c * kG1Pitch + w * kVSteps;
    float2 xv[kVSteps + 2 * halo];
#pragma unroll
    for (int j = 0; j < kVSteps + 2 * halo; ++j) xv[j] = xr[j * (kSC / 2)];
    float2 gv[kVSteps + 4];
#pragma unroll
    for (int j = 0; j < kVSteps + 4; ++j) gv[j] = make_float2(0.f, 0.f);
    if (p.g_bld) {
#pragma unroll
      for (int j = 0; j < kVSteps + halo; ++j) gv[j] = g2r[j * (kSC / 2)];
    }
    if (p.g_bdl) {
#pragma unroll
      for (int j = 0; j < kVSteps + 4; j += 4) {
        if (j < kVSteps + halo) {
          const float4 a = *reinterpret_cast<const float4*>(g1a + j);
          const float4 bq = *reinterpret_cast<const float4*>(g1a + kG1Pitch + j);
          gv[j].x += a.x; gv[j + 1].x += a.y; gv[j + 2].x += a.z; gv[j + 3].x += a.w;
          gv[j].y += bq.x; gv[j + 1].y += bq.y; gv[j + 2].y += bq.z; gv[j + 3].y += bq.w;
        }
      }
    }
    float2 dp[kVSteps + halo];
    float* dst = p.grad_x + ((long long)b * p.L + ts) * p.D + d0 + c;
#pragma unroll
    for (int j = 0; j < kVSteps + halo; ++j) {
      float2 pre = bias;
#pragma unroll
      for (int k = 0; k < K; ++k) {
        pre.x = fmaf(wt[k].x, xv[j + k].x, pre.x);
        pre.y = fmaf(wt[k].y, xv[j + k].y, pre.y);
      }
      const float sx = __fdividef(1.0f, 1.0f + __expf(-pre.x)), sy = __fdividef(1.0f, 1.0f + __expf(-pre.y));
      const bool live = ok && ts + j < p.L;
      dp[j].x = live ? gv[j].x * (sx * fmaf(pre.x, 1.0f - sx, 1.0f)) : 0.0f;
      dp[j].y = live ? gv[j].y * (sy * fmaf(pre.y, 1.0f - sy, 1.0f)) : 0.0f;
      if (j < kVSteps) {          // the steps after the warp's own belong to the next warp's sums
        accb.x += dp[j].x; accb.y += dp[j].y;
#pragma unroll
        for (int k = 0; k < K; ++k) {
          accw[k].x = fmaf(dp[j].x, xv[j + k].x, accw[k].x);
          accw[k].y = fmaf(dp[j].y, xv[j + k].y, accw[k].y);
        }
      }
      if (j >= halo) {            // grad_x[ts + j - halo] = sum_k w[k] * dpre[ts + j - k]
        float2 gx = make_float2(0.f, 0.f);
#pragma unroll
        for (int k = 0; k < K; ++k) {
          gx.x = fmaf(wt[k].x, dp[j - k].x, gx.x);
          gx.y = fmaf(wt[k].y, dp[j - k].y, gx.y);
        }
        if (ok && ts + j - halo < p.L) *reinterpret_cast<float2*>(dst) = gx;
        dst += p.D;
      }
    }
    __syncthreads();          // the stage has been read
    if (leader && i + ring < ntiles) {
      fence_proxy_async();
      issue(slot, tile0 + i + ring);
    }
    if (++slot == ring) { slot = 0; parity ^= 1; }
  }
  // sums over the CTA's warps, one atomic per (channel, tap)
  float* red = reinterpret_cast<float*>(ring_base);            // [warp][K + 1][kSC]; every stage has been consumed
#pragma unroll
  for (int k = 0; k < K; ++k) *reinterpret_cast<float2*>(red + (w * (K + 1) + k) * kSC + c) = accw[k];
  *reinterpret_cast<float2*>(red + (w * (K + 1) + K) * kSC + c) = accb;
  __syncthreads();
  const int cr = w * 32 + lane;
  if (cr < kSC && d0 + cr < D) {
#pragma unroll
    for (int k = 0; k <= K; ++k) {
      float s = 0.0f;
#pragma unroll
      for (int j = 0; j < kVWarps; ++j) s += red[(j * (K + 1) + k) * kSC + cr];
      if (k < K) atomicAdd(p.grad_w + (d0 + cr) * K + k, s);
      else if (p.grad_bias) atomicAdd(p.grad_bias + d0 + cr, s);
    }
  }
}

// Tensor map (time, channels, batch) over a time-contiguous [B, D, L] array; boxes of 68 steps x 64 channels.
static bool staged_bdl_map(CUtensorMap* tm, const float* g, long long B, long long L, long long D) {
  if ((L & 3) != 0) return false;
  const uint64_t dims[3] = {(uint64_t)L, (uint64_t)D, (uint64_t)B};
  const uint64_t strides[2] = {(uint64_t)L * 4, (uint64_t)D * (uint64_t)L * 4};
  const uint32_t box[3] = {(uint32_t)(kVT + 4), (uint32_t)kSC, 1};
  return make_tensor_map_3d_f32(tm, g, dims, strides, box);
}

static inline bool aligned(const void* ptr, uintptr_t a) { return (reinterpret_cast<uintptr_t>(ptr) & (a - 1)) == 0; }

static bool forward_vec_ok(const ConvParams& p) {
  return (p.D % 2 == 0) && (p.ldx % 2 == 0) && aligned(p.x, 8) && aligned(p.bias, 8) && aligned(p.out_bld, 8) &&
         (!p.out_bdl || (p.L % 4 == 0 && aligned(p.out_bdl, 16)));
}
static bool backward_vec_ok(const ConvParams& p) {
  return (p.D % 2 == 0) && (p.ldx % 2 == 0) && aligned(p.x, 8) && aligned(p.bias, 8) && aligned(p.g_bld, 8) &&
         aligned(p.grad_x, 8) && (!p.g_bdl || (p.L % 4 == 0 && aligned(p.g_bdl, 16)));
}

template <int K>
static void launch_forward(const ConvParams& p, cudaStream_t stream) {
  CUtensorMap tm;
  memset(&tm, 0, sizeof(tm));
  if (forward_vec_ok(p) && p.L >= 4 * kVT && staged_x_map(&tm, p.x, p.B, p.L, p.D, p.ldx, kVT + K - 1)) {
    const int ring = 3;
    const size_t smem = 1024 + (size_t)ring * (kVT + K - 1) * kSC * 4 + (size_t)kVT * kSPitch * 4;
    if (ensure_dynamic_smem(reinterpret_cast<const void*>(conv_silu_forward_staged_kernel<K>), smem) == kOk) {
      // a CTA walks up to 16 consecutive time tiles; fewer when that would leave SMs without work
      const long long tiles_t = (p.L + kVT - 1) / kVT, dblocks = (p.D + kSC - 1) / kSC;
      long long per_cta = tiles_t * dblocks * p.B / (8LL * sm_count());
      per_cta = per_cta < 1 ? 1 : (per_cta > 16 ? 16 : per_cta);
      dim3 grid((unsigned)((tiles_t + per_cta - 1) / per_cta), (unsigned)dblocks, (unsigned)p.B);
      conv_silu_forward_staged_kernel<K><<<grid, dim3(32, kVWarps), smem, stream>>>(tm, p, (int)per_cta, ring);
      return;
    }
  }
  if (forward_vec_ok(p)) {
    dim3 grid((unsigned)((p.L + kVT - 1) / kVT), (unsigned)((p.D + kVD - 1) / kVD), (unsigned)p.B);
    conv_silu_forward_vec_kernel<K><<<grid, dim3(32, kVWarps), 0, stream>>>(p);
  } else {
    dim3 grid((unsigned)((p.L + kTileT - 1) / kTileT), (unsigned)((p.D + kTileD - 1) / kTileD), (unsigned)p.B);
    conv_silu_forward_kernel<K><<<grid, dim3(kTileD, kRowsY), 0, stream>>>(p);
  }
}
template <int K>
static void launch_backward(const ConvParams& p, cudaStream_t stream) {
  CUtensorMap tx, t2, t1;
  memset(&tx, 0, sizeof(tx));
  memset(&t2, 0, sizeof(t2));
  memset(&t1, 0, sizeof(t1));
  if (backward_vec_ok(p) && p.L >= 4 * kVT && staged_x_map(&tx, p.x, p.B, p.L, p.D, p.ldx, kVT + 2 * (K - 1)) &&
      (!p.g_bld || staged_x_map(&t2, p.g_bld, p.B, p.L, p.D, p.D, kVT + K - 1)) &&
      (!p.g_bdl || staged_bdl_map(&t1, p.g_bdl, p.B, p.L, p.D))) {
    const int ring = 2;
    const size_t stage = (size_t)(kVT + 2 * (K - 1)) * kSC * 4 + (size_t)(kVT + K - 1) * kSC * 4 + (size_t)kSC * (kVT + 4) * 4;
    const size_t smem = 1024 + ring * stage;
    if (ensure_dynamic_smem(reinterpret_cast<const void*>(conv_silu_backward_staged_kernel<K>), smem) == kOk) {
      const long long tiles_t = (p.L + kVT - 1) / kVT, dblocks = (p.D + kSC - 1) / kSC;
      long long per_cta = tiles_t * dblocks * p.B / (8LL * sm_count());
      per_cta = per_cta < 1 ? 1 : (per_cta > 16 ? 16 : per_cta);
      dim3 grid((unsigned)((tiles_t + per_cta - 1) / per_cta), (unsigned)dblocks, (unsigned)p.B);
      conv_silu_backward_staged_kernel<K><<<grid, dim3(32, kVWarps), smem, stream>>>(tx, t2, t1, p, (int)per_cta, ring);
      return;
    }
  }
  if (backward_vec_ok(p)) {
    // enough CTAs for a few waves, as few partial sums (atomics) as that allows
    const long long tiles_t = (p.L + kVT - 1) / kVT, dblocks = (p.D + kVDB - 1) / kVDB;
    long long per_cta = tiles_t * dblocks * p.B / 8192;
    per_cta = per_cta < 1 ? 1 : (per_cta > tiles_t ? tiles_t : per_cta);
    dim3 grid((unsigned)((tiles_t + per_cta - 1) / per_cta), (unsigned)dblocks, (unsigned)p.B);
    conv_silu_backward_vec_kernel<K><<<grid, dim3(32, kVWarps), 0, stream>>>(p, (int)per_cta);
  } else {
    dim3 grid((unsigned)((p.L + kTileT - 1) / kTileT), (unsigned)((p.D + kTileD - 1) / kTileD), (unsigned)p.B);
    conv_silu_backward_kernel<K><<<grid, dim3(kTileD, kRowsY), 0, stream>>>(p);
  }
}

static int check(const char* fn, const ConvParams& p) {
  if (p.B < 0 || p.L < 0 || p.D < 0) { set_last_error("%s: negative extent", fn); return kErrInvalidArgument; }
  if (p.taps < 1 || p.taps > kMaxTaps) { set_last_error("%s: kernel size must be 1..%d", fn, kMaxTaps); return kErrUnsupported; }
  if (p.B > 65535 || (p.D + kTileD - 1) / kTileD > 65535) { set_last_error("%s: batch or channel count too large", fn); return kErrUnsupported; }
  if (p.ldx < p.D) { set_last_error("%s: row pitch smaller than the channel count", fn); return kErrInvalidArgument; }
  return kOk;
}

}  // namespace mixer
}  // namespace ossm_b200

extern "C" {

using namespace ossm_b200;

int ossm_b200_conv1d_silu_forward(const float* x, int64_t ldx, const float* weight, const float* bias, float* out_bdl,
                                  float* out_bld, int64_t B, int64_t L, int64_t D, int taps, cudaStream_t stream) {
  mixer::ConvParams p{};
  p.x = x; p.w = weight; p.bias = bias; p.out_bdl = out_bdl; p.out_bld = out_bld;
  p.B = B; p.L = L; p.D = D; p.ldx = ldx; p.taps = taps;
  if (int rc = mixer::check("conv1d_silu_forward", p)) return rc;
  if (B == 0 || L == 0 || D == 0) return kOk;
  if (!x || !weight || (!out_bdl && !out_bld)) { set_last_error("conv1d_silu_forward: null pointer"); return kErrInvalidArgument; }
  switch (taps) {
    case 1: mixer::launch_forward<1>(p, stream); break;
    case 2: mixer::launch_forward<2>(p, stream); break;
    case 3: mixer::launch_forward<3>(p, stream); break;
    default: mixer::launch_forward<4>(p, stream); break;
  }
  return check_cuda(cudaGetLastError(), "conv_silu_forward_kernel launch");
}

int ossm_b200_conv1d_silu_backward(const float* x, int64_t ldx, const float* weight, const float* bias,
                                   const float* grad_bdl, const float* grad_bld, float* grad_x, float* grad_weight,
                                   float* grad_bias, int64_t B, int64_t L, int64_t D, int taps, cudaStream_t stream) {
  mixer::ConvParams p{};
  p.x = x; p.w = weight; p.bias = bias; p.g_bdl = grad_bdl; p.g_bld = grad_bld;
  p.grad_x = grad_x; p.grad_w = grad_weight; p.grad_bias = grad_bias;
  p.B = B; p.L = L; p.D = D; p.ldx = ldx; p.taps = taps;
  if (int rc = mixer::check("conv1d_silu_backward", p)) return rc;
  if (D == 0) return kOk;
  if (!grad_weight || (bias && !grad_bias)) { set_last_error("conv1d_silu_backward: null gradient pointer"); return kErrInvalidArgument; }
  if (int rc = check_cuda(cudaMemsetAsync(grad_weight, 0, (size_t)D * taps * sizeof(float), stream), "memset grad_weight")) return rc;
  if (grad_bias)
    if (int rc = check_cuda(cudaMemsetAsync(grad_bias, 0, (size_t)D * sizeof(float), stream), "memset grad_bias")) return rc;
  if (B == 0 || L == 0) return kOk;
  if (!x || !weight || !grad_x || (!grad_bdl && !grad_bld)) { set_last_error("conv1d_silu_backward: null pointer"); return kErrInvalidArgument; }
  switch (taps) {
    case 1: mixer::launch_backward<1>(p, stream); break;
    case 2: mixer::launch_backward<2>(p, stream); break;
    case 3: mixer::launch_backward<3>(p, stream); break;
    default: mixer::launch_backward<4>(p, stream); break;
  }
  return check_cuda(cudaGetLastError(), "conv_silu_backward_kernel launch");
}

}  // extern "C"
