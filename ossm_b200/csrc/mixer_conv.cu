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

__device__ __forceinline__ float sigmoidf_(float v) { return 1.0f / (1.0f + __expf(-v)); }

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

__global__ void __launch_bounds__(kTileD * kRowsY) conv_silu_forward_kernel(ConvParams p) {
  __shared__ float xin[kTileT + kMaxTaps - 1][kTileD + 1];
  __shared__ float yout[kTileT][kTileD + 1];
  const int tx = threadIdx.x, ty = threadIdx.y;
  const long long b = blockIdx.z;
  const long long d0 = (long long)blockIdx.y * kTileD, t0 = (long long)blockIdx.x * kTileT;
  const int halo = p.taps - 1;
  const long long d = d0 + tx;
  const float* xb = p.x + b * p.L * p.ldx;
  for (int r = ty; r < kTileT + halo; r += kRowsY) {
    const long long t = t0 - halo + r;
    xin[r][tx] = (d < p.D && t >= 0 && t < p.L) ? __ldg(xb + t * p.ldx + d) : 0.0f;
  }
  float w[kMaxTaps];
#pragma unroll
  for (int k = 0; k < kMaxTaps; ++k) w[k] = (k < p.taps && d < p.D) ? __ldg(p.w + d * p.taps + k) : 0.0f;
  const float bias = (p.bias && d < p.D) ? __ldg(p.bias + d) : 0.0f;
  __syncthreads();
  for (int r = ty; r < kTileT; r += kRowsY) {
    float pre = bias;
#pragma unroll
    for (int k = 0; k < kMaxTaps; ++k)
      if (k < p.taps) pre = fmaf(w[k], xin[r + k][tx], pre);
    const float y = pre * sigmoidf_(pre);
    yout[r][tx] = y;
    const long long t = t0 + r;
    if (p.out_bld && d < p.D && t < p.L) p.out_bld[(b * p.L + t) * p.D + d] = y;
  }
  if (p.out_bdl == nullptr) return;
  __syncthreads();
  // transposed store: consecutive threads write consecutive time steps of one channel
  for (int i = ty * kTileD + tx; i < kTileT * kTileD; i += kTileD * kRowsY) {
    const int dd = i / kTileT, tt = i % kTileT;
    const long long dch = d0 + dd, t = t0 + tt;
    if (dch < p.D && t < p.L) p.out_bdl[(b * p.D + dch) * p.L + t] = yout[tt][dd];
  }
}

__global__ void __launch_bounds__(kTileD * kRowsY) conv_silu_backward_kernel(ConvParams p) {
  __shared__ float xin[kTileT + 2 * (kMaxTaps - 1)][kTileD + 1];    // x for t0-halo .. t0+T+halo
  __shared__ float dpre[kTileT + kMaxTaps - 1][kTileD + 1];         // d(pre) for t0 .. t0+T+halo
  __shared__ float red[kRowsY][kMaxTaps + 1][kTileD];
  const int tx = threadIdx.x, ty = threadIdx.y;
  const long long b = blockIdx.z;
  const long long d0 = (long long)blockIdx.y * kTileD, t0 = (long long)blockIdx.x * kTileT;
  const int halo = p.taps - 1;
  const long long d = d0 + tx;
  const float* xb = p.x + b * p.L * p.ldx;
  for (int r = ty; r < kTileT + 2 * halo; r += kRowsY) {
    const long long t = t0 - halo + r;
    xin[r][tx] = (d < p.D && t >= 0 && t < p.L) ? __ldg(xb + t * p.ldx + d) : 0.0f;
  }
  // upstream gradient of the time-contiguous output, transposed through dpre as staging
  if (p.g_bdl) {
    for (int i = ty * kTileD + tx; i < (kTileT + halo) * kTileD; i += kTileD * kRowsY) {
      const int dd = i / (kTileT + halo), tt = i % (kTileT + halo);
      const long long dch = d0 + dd, t = t0 + tt;
      dpre[tt][dd] = (dch < p.D && t < p.L) ? __ldg(p.g_bdl + (b * p.D + dch) * p.L + t) : 0.0f;
    }
  }
  float w[kMaxTaps];
#pragma unroll
  for (int k = 0; k < kMaxTaps; ++k) w[k] = (k < p.taps && d < p.D) ? __ldg(p.w + d * p.taps + k) : 0.0f;
  const float bias = (p.bias && d < p.D) ? __ldg(p.bias + d) : 0.0f;
  __syncthreads();
  float acc_w[kMaxTaps] = {0.f, 0.f, 0.f, 0.f}, acc_b = 0.f;
  for (int r = ty; r < kTileT + halo; r += kRowsY) {
    const long long t = t0 + r;
    float g = p.g_bdl ? dpre[r][tx] : 0.0f;
    if (p.g_bld && d < p.D && t < p.L) g += __ldg(p.g_bld + (b * p.L + t) * p.D + d);
    float pre = bias;
#pragma unroll
    for (int k = 0; k < kMaxTaps; ++k)
      if (k < p.taps) pre = fmaf(w[k], xin[r + k][tx], pre);     // x index of output t = t0 + r is r + k (offset halo cancels)
    const float sg = sigmoidf_(pre);
    const float dp = (t < p.L) ? g * (sg * (1.0f + pre * (1.0f - sg))) : 0.0f;
    dpre[r][tx] = dp;
    if (r < kTileT) {       // the halo rows belong to the next tile's sums
      acc_b += dp;
#pragma unroll
      for (int k = 0; k < kMaxTaps; ++k)
        if (k < p.taps) acc_w[k] = fmaf(dp, xin[r + k][tx], acc_w[k]);
    }
  }
  __syncthreads();
  // grad_x[t] = sum_k w[k] * dpre[t + halo - k]
  for (int r = ty; r < kTileT; r += kRowsY) {
    const long long t = t0 + r;
    float gx = 0.0f;
#pragma unroll
    for (int k = 0; k < kMaxTaps; ++k)
      if (k < p.taps) gx = fmaf(w[k], dpre[r + halo - k][tx], gx);
    if (d < p.D && t < p.L) p.grad_x[(b * p.L + t) * p.D + d] = gx;
  }
#pragma unroll
  for (int k = 0; k < kMaxTaps; ++k) red[ty][k][tx] = acc_w[k];
  red[ty][kMaxTaps][tx] = acc_b;
  __syncthreads();
  if (ty == 0 && d < p.D) {
    for (int k = 0; k <= kMaxTaps; ++k) {
      float s = 0.0f;
      for (int j = 0; j < kRowsY; ++j) s += red[j][k][tx];
      if (k < p.taps) atomicAdd(p.grad_w + d * p.taps + k, s);
      else if (k == kMaxTaps && p.grad_bias) atomicAdd(p.grad_bias + d, s);
    }
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
  dim3 grid((unsigned)((L + mixer::kTileT - 1) / mixer::kTileT), (unsigned)((D + mixer::kTileD - 1) / mixer::kTileD), (unsigned)B);
  mixer::conv_silu_forward_kernel<<<grid, dim3(mixer::kTileD, mixer::kRowsY), 0, stream>>>(p);
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
  dim3 grid((unsigned)((L + mixer::kTileT - 1) / mixer::kTileT), (unsigned)((D + mixer::kTileD - 1) / mixer::kTileD), (unsigned)B);
  mixer::conv_silu_backward_kernel<<<grid, dim3(mixer::kTileD, mixer::kRowsY), 0, stream>>>(p);
  return check_cuda(cudaGetLastError(), "conv_silu_backward_kernel launch");
}

}  // extern "C"
