// Mamba selective scan, serial-in-time kernels for the common state sizes (sm_100a).
//
// The time-parallel kernels of selective_scan.cu spend most of their instructions
// in warp shuffles (an affine-map scan per state pair per chunk).  For d_state = 16
// the whole state of a channel fits in registers, so here one lane owns one
// (batch, channel) series and walks the sequence serially, exactly like the
// reference CPU loop (selective_scan_cpu.cpp:118-152): per step and state one
// ex2, one multiply for the decay argument, one for the forcing and two FMAs
// (packed two states at a time as f32x2), no shuffles and no scan.  What bounds
// the kernel is the special-function unit (one ex2 per step and state); HBM
// traffic is far below the roofline.
//
// A CTA is one warp covering 64 channels of ONE batch element (two channels per lane,
// so that every B_t / C_t value fetched from shared memory feeds two series), and the
// B_t / C_t values of a step are the same for every lane: tiles of kStage steps are
// transposed into shared memory as [step][B | C] once per CTA, kept in the I/O type
// (bf16 halves the shared-memory traffic, which otherwise limits the kernel before
// the special-function unit does) and read back with broadcast 16-byte loads.  u, dt, z and out move through per-lane 16-byte vector accesses
// along the (contiguous) time axis, one group of 8 steps at a time, prefetched one
// group ahead.
//
// The forward also saves the state entering every kSerialInterval-step window
// (float32 [B, D, ceil(L/interval), N]): the backward recomputes inside a window only.
#include "common.cuh"

#include <cuda_bf16.h>

#include "../../include/ossm_b200.h"

namespace ossm_b200 {
namespace sscan {

constexpr int kSerialLanes = 32;      // threads per CTA (one warp)
constexpr int kSerialCh = 2;          // channels per lane: lane l owns channels base + l and base + 32 + l
constexpr int kSerialSpan = kSerialLanes * kSerialCh;   // channels per CTA
constexpr int kSerialInterval = 8;    // steps per group == steps between saved states
constexpr int kStage = 32;            // steps per B/C shared-memory tile

// Moves the [N, kStage] slabs of B and C starting at step t_base into a tile laid out
// [step][B_0..B_{N-1} | C_0..C_{N-1}] in the I/O element type, in two steps: issue() starts
// asynchronous 16-byte copies (cp.async) of the raw rows into a staging buffer, finish() --
// called by the same thread after the copies have landed -- transposes its own items.  No
// registers are held in between.  Work item i covers row r = i % 2N (B rows, then C rows) and
// the kVec consecutive steps of chunk i / 2N.
template <typename IO, int N, int kThreads>
struct TileLoader {
  static constexpr int kVec = 16 / (int)sizeof(IO);
  static constexpr int kItemsTotal = 2 * N * kStage / kVec;
  static constexpr int kPerThread = (kItemsTotal + kThreads - 1) / kThreads;

  static __device__ __forceinline__ void issue(uint4* raw, const IO* B_b, const IO* C_b, long long t_base,
                                               long long L, bool vec_ok) {
#pragma unroll
    for (int q = 0; q < kPerThread; ++q) {
      const int i = threadIdx.x + q * kThreads;
      if (i >= kItemsTotal) continue;
      const int r = i % (2 * N), c = i / (2 * N);
      const long long t = t_base + (long long)c * kVec;
      const IO* row = (r < N ? B_b + (long long)r * L : C_b + (long long)(r - N) * L);
      if (vec_ok && t + kVec <= L) {
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(raw + i)), "l"(row + t) : "memory");
      } else {
        IO tmp[kVec];
#pragma unroll
        for (int j = 0; j < kVec; ++j) tmp[j] = (t + j < L) ? row[t + j] : IO(0.0f);
        raw[i] = *reinterpret_cast<const uint4*>(tmp);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  }

  static __device__ __forceinline__ void finish(const uint4* raw, IO* tile) {
    asm volatile("cp.async.wait_group 0;" ::: "memory");
#pragma unroll
    for (int q = 0; q < kPerThread; ++q) {
      const int i = threadIdx.x + q * kThreads;
      if (i >= kItemsTotal) continue;
      const int r = i % (2 * N), c = i / (2 * N);
      IO* o = tile + (c * kVec) * (2 * N) + r;
      const uint4 v = raw[i];
      const IO* e = reinterpret_cast<const IO*>(&v);
#pragma unroll
      for (int j = 0; j < kVec; ++j) o[j * 2 * N] = e[j];
    }
  }
};

// (state 2q, state 2q+1) pairs of B and C of one step from the tile, as fp32.
template <typename IO, int N>
__device__ __forceinline__ void load_bc_step(const IO* step, float2 (&Bp)[N / 2], float2 (&Cp)[N / 2]) {
  if constexpr (sizeof(IO) == 4) {
    const float4* v = reinterpret_cast<const float4*>(step);
#pragma unroll
    for (int q = 0; q < N / 4; ++q) {
      const float4 b = v[q], c = v[N / 4 + q];
      Bp[2 * q] = make_float2(b.x, b.y); Bp[2 * q + 1] = make_float2(b.z, b.w);
      Cp[2 * q] = make_float2(c.x, c.y); Cp[2 * q + 1] = make_float2(c.z, c.w);
    }
  } else {
    // a 32-bit word holds the bf16 of states 2q (low half) and 2q+1 (high half)
    const uint4* v = reinterpret_cast<const uint4*>(step);
#pragma unroll
    for (int q = 0; q < N / 8; ++q) {
      const uint4 b = v[q], c = v[N / 8 + q];
      const uint32_t bw[4] = {b.x, b.y, b.z, b.w}, cw[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        Bp[4 * q + k] = make_float2(__uint_as_float(bw[k] << 16), __uint_as_float(bw[k] & 0xffff0000u));
        Cp[4 * q + k] = make_float2(__uint_as_float(cw[k] << 16), __uint_as_float(cw[k] & 0xffff0000u));
      }
    }
  }
}

// Per-lane input groups (G steps of u, dt, z of each of the lane's channels) are prefetched one
// group ahead with cp.async into a [buffer][16-byte vector][lane] slab of shared memory: no
// registers are tied up and the compiler cannot sink the loads towards their use.
template <typename IO, int kThreads>
struct GroupStream {
  static constexpr int G = kSerialInterval;
  static constexpr int kVecIO = G * (int)sizeof(IO) / 16;   // 16-byte vectors of u (and of z)
  static constexpr int kVecs = 2 * kVecIO + 2;               // per channel: u | dt (two vectors) | z
  uint4* slab;                                               // [2][kSerialCh * kVecs][kThreads]

  __device__ __forceinline__ uint4* slot(int buf, int ch, int v) const {
    return slab + ((buf * kSerialCh + ch) * kVecs + v) * kThreads + threadIdx.x;
  }

  template <typename T>
  __device__ __forceinline__ void issue_row(int buf, int ch, int v0, const T* row, long long t0, long long L,
                                            bool vec_ok) const {
    constexpr int kPer = 16 / (int)sizeof(T);
    constexpr int kNum = G / kPer;
    if (vec_ok && t0 + G <= L) {
#pragma unroll
      for (int v = 0; v < kNum; ++v)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(slot(buf, ch, v0 + v))),
                     "l"(row + t0 + v * kPer) : "memory");
    } else {
#pragma unroll
      for (int v = 0; v < kNum; ++v) {
        T tmp[kPer];
#pragma unroll
        for (int j = 0; j < kPer; ++j) tmp[j] = (t0 + v * kPer + j < L) ? row[t0 + v * kPer + j] : T(0.0f);
        *slot(buf, ch, v0 + v) = *reinterpret_cast<const uint4*>(tmp);
      }
    }
  }

  // rows of channel ch start at u + off[ch] etc.
  __device__ __forceinline__ void issue(int buf, const IO* u, const float* dt, const IO* z, const long long (&off)[kSerialCh],
                                        long long t0, long long L, bool vec_ok) const {
    if (t0 < L) {
#pragma unroll
      for (int ch = 0; ch < kSerialCh; ++ch) {
        issue_row<IO>(buf, ch, 0, u + off[ch], t0, L, vec_ok);
        issue_row<float>(buf, ch, kVecIO, dt + off[ch], t0, L, vec_ok);
        if (z) issue_row<IO>(buf, ch, kVecIO + 2, z + off[ch], t0, L, vec_ok);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  }

  template <typename T>
  __device__ __forceinline__ void read(int buf, int ch, int v0, float (&out)[G]) const {
    constexpr int kPer = 16 / (int)sizeof(T);
#pragma unroll
    for (int v = 0; v < G / kPer; ++v) {
      const uint4 r = *slot(buf, ch, v0 + v);
      const uint32_t w[4] = {r.x, r.y, r.z, r.w};
      if constexpr (sizeof(T) == 4) {
#pragma unroll
        for (int j = 0; j < 4; ++j) out[v * 4 + j] = __uint_as_float(w[j]);
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          out[v * 8 + 2 * j] = __uint_as_float(w[j] << 16);
          out[v * 8 + 2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
        }
      }
    }
  }
};

template <typename IO, int N>
__global__ void __launch_bounds__(kSerialLanes) sscan_forward_serial_kernel(Params p) {
  constexpr int NP = N / 2;
  constexpr int G = kSerialInterval;
  constexpr int kGroupsPerStage = kStage / G;
  constexpr int CH = kSerialCh;
  using Loader = TileLoader<IO, N, kSerialLanes>;
  using Stream = GroupStream<IO, kSerialLanes>;
  __shared__ __align__(16) IO tile[2][kStage * 2 * N];
  __shared__ uint4 raw[Loader::kItemsTotal];
  __shared__ uint4 slab[2 * CH * Stream::kVecs * kSerialLanes];
  const long long b = blockIdx.y;
  const IO* Bm_b = static_cast<const IO*>(p.Bm) + b * N * p.L;
  const IO* Cm_b = static_cast<const IO*>(p.Cm) + b * N * p.L;
  const IO* u_all = static_cast<const IO*>(p.u);
  const IO* z_all = static_cast<const IO*>(p.z);
  Stream stream{slab};

  long long dch[CH], off[CH];
  bool active[CH];
  float2 A2[CH][NP], h[CH][NP];
  float dskip[CH];
  float* cs_out[CH];
#pragma unroll
  for (int ch = 0; ch < CH; ++ch) {
    dch[ch] = (long long)blockIdx.x * kSerialSpan + ch * kSerialLanes + threadIdx.x;
    active[ch] = dch[ch] < p.D;
    const long long d = active[ch] ? dch[ch] : 0;    // idle lanes shadow channel 0 and store nothing
    off[ch] = (b * p.D + d) * p.L;
#pragma unroll
    for (int q = 0; q < NP; ++q) {
      A2[ch][q] = make_float2(__ldg(p.A + d * N + 2 * q) * kLog2e, __ldg(p.A + d * N + 2 * q + 1) * kLog2e);
      h[ch][q] = make_float2(0.f, 0.f);
    }
    dskip[ch] = p.Dskip ? __ldg(p.Dskip + d) : 0.0f;
    cs_out[ch] = (p.chunk_states && active[ch]) ? p.chunk_states + (b * p.D + d) * p.nstates * N : nullptr;
  }

  const long long nstages = (p.L + kStage - 1) / kStage;
  Loader::issue(raw, Bm_b, Cm_b, 0, p.L, p.vec_ok);
  stream.issue(0, u_all, p.dt, z_all, off, 0, p.L, p.vec_ok);
  Loader::finish(raw, tile[0]);   // waits for everything issued so far
  __syncwarp();

  for (long long s = 0; s < nstages; ++s) {
    const int buf = (int)(s & 1);
#pragma unroll 1
    for (int g = 0; g < kGroupsPerStage; ++g) {
      const long long t0 = s * kStage + (long long)g * G;
      if (t0 >= p.L) break;
      const int gb = g & 1;   // kGroupsPerStage is even: the parity of the global group index
      stream.issue(gb ^ 1, u_all, p.dt, z_all, off, t0 + G, p.L, p.vec_ok);
      if (g == 0 && s + 1 < nstages) {
        // next stage's B/C rows (each thread transposes only what it copied itself); issued after
        // the group prefetch so that waiting for this group's data does not wait for them
        Loader::issue(raw, Bm_b, Cm_b, (s + 1) * kStage, p.L, p.vec_ok);
        asm volatile("cp.async.wait_group 2;" ::: "memory");
      } else {
        asm volatile("cp.async.wait_group 1;" ::: "memory");   // everything but the prefetch just issued has landed
      }
      float u_c[CH][G], dt_c[CH][G], z_c[CH][G], y[CH][G];
#pragma unroll
      for (int ch = 0; ch < CH; ++ch) {
        stream.template read<IO>(gb, ch, 0, u_c[ch]);
        stream.template read<float>(gb, ch, Stream::kVecIO, dt_c[ch]);
        if (z_all) stream.template read<IO>(gb, ch, Stream::kVecIO + 2, z_c[ch]);
        if (cs_out[ch]) {   // state entering this window
          float4* o = reinterpret_cast<float4*>(cs_out[ch] + (t0 / G) * N);
#pragma unroll
          for (int q = 0; q < NP / 2; ++q)
            o[q] = make_float4(h[ch][2 * q].x, h[ch][2 * q].y, h[ch][2 * q + 1].x, h[ch][2 * q + 1].y);
        }
      }
      const IO* steps = tile[buf] + g * G * 2 * N;
#pragma unroll
      for (int j = 0; j < G; ++j) {
        float2 Bp[NP], Cp[NP];
        load_bc_step<IO, N>(steps + j * 2 * N, Bp, Cp);
#pragma unroll
        for (int ch = 0; ch < CH; ++ch) {
          const float2 dtv = splat(dt_c[ch][j]);
          const float2 dtu = splat(dt_c[ch][j] * u_c[ch][j]);
          float2 acc0 = make_float2(0.f, 0.f), acc1 = make_float2(0.f, 0.f);
#pragma unroll
          for (int q = 0; q < NP; q += 2) {
            const float2 x0 = p2mul(dtv, A2[ch][q]), x1 = p2mul(dtv, A2[ch][q + 1]);
            const float2 a0 = make_float2(ex2(x0.x), ex2(x0.y)), a1 = make_float2(ex2(x1.x), ex2(x1.y));
            h[ch][q] = p2fma(a0, h[ch][q], p2mul(dtu, Bp[q]));
            h[ch][q + 1] = p2fma(a1, h[ch][q + 1], p2mul(dtu, Bp[q + 1]));
            acc0 = p2fma(Cp[q], h[ch][q], acc0);
            acc1 = p2fma(Cp[q + 1], h[ch][q + 1], acc1);
          }
          const float2 acc = p2add(acc0, acc1);
          float yv = fmaf(dskip[ch], u_c[ch][j], acc.x + acc.y);
          if (z_all) {
            const float zv = z_c[ch][j];
            yv *= __fdividef(zv, 1.0f + ex2(-zv * kLog2e));
          }
          y[ch][j] = yv;
        }
      }
#pragma unroll
      for (int ch = 0; ch < CH; ++ch)
        if (active[ch]) store_items<IO, G>(static_cast<IO*>(p.out) + off[ch], t0, p.L, p.vec_ok, y[ch]);
    }
    if (s + 1 < nstages) Loader::finish(raw, tile[buf ^ 1]);
    __syncwarp();
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}

template <typename IO>
static int launch_fwd_serial(const Params& p, cudaStream_t stream) {
  dim3 grid((unsigned)((p.D + kSerialSpan - 1) / kSerialSpan), (unsigned)p.B);
  sscan_forward_serial_kernel<IO, 16><<<grid, kSerialLanes, 0, stream>>>(p);
  return check_cuda(cudaGetLastError(), "sscan_forward_serial_kernel launch");
}

}  // namespace sscan
}  // namespace ossm_b200
