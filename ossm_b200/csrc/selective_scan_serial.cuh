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
// (float32 [B, ceil(L/interval), D, N], channels contiguous so that a warp's states of one
// window are one 2 KB block): the backward recomputes inside a window only.
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
// the kVec consecutive steps of chunk i / 2N.  With B and C given step-major ([B, L, N], `pitch`
// elements between the rows of consecutive steps: ossm's own argument order) item i is the i-th
// 16-byte piece of the tile itself -- step i / (2N / kVec), B then C, kVec consecutive states --
// and finish() only converts.
template <typename IO, int N, int kThreads>
struct TileLoader {
  static constexpr int kVec = 16 / (int)sizeof(IO);
  static constexpr int kItemsTotal = 2 * N * kStage / kVec;
  static constexpr int kPerThread = (kItemsTotal + kThreads - 1) / kThreads;

  static __device__ __forceinline__ void issue(uint4* raw, const IO* B_b, const IO* C_b, long long t_base,
                                               long long L, bool vec_ok, bool step_major = false,
                                               long long pitch = 0) {
    if (step_major) {
      constexpr int kPieces = N / kVec;     // pieces of a step's B (or C) row
#pragma unroll
      for (int q = 0; q < kPerThread; ++q) {
        const int i = threadIdx.x + q * kThreads;
        if (i >= kItemsTotal) continue;
        const int st = i / (2 * kPieces), wc = (i / kPieces) & 1, g = i % kPieces;
        const long long t = t_base + st;
        const IO* src = (wc ? C_b : B_b) + t * pitch + g * kVec;
        if (vec_ok && t < L) {
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(raw + i)), "l"(src) : "memory");
        } else {
          IO tmp[kVec];
#pragma unroll
          for (int j = 0; j < kVec; ++j) tmp[j] = (t < L) ? src[j] : IO(0.0f);
          raw[i] = *reinterpret_cast<const uint4*>(tmp);
        }
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
      return;
    }
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

  // TT: element type of the tile, the I/O type or float (converted here, once per CTA, instead of at every use)
  template <typename TT>
  static __device__ __forceinline__ void finish(const uint4* raw, TT* tile, bool step_major = false) {
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    if (step_major) {
#pragma unroll
      for (int q = 0; q < kPerThread; ++q) {
        const int i = threadIdx.x + q * kThreads;
        if (i >= kItemsTotal) continue;
        const uint4 v = raw[i];
        const IO* e = reinterpret_cast<const IO*>(&v);
        TT* o = tile + i * kVec;
#pragma unroll
        for (int j = 0; j < kVec; ++j) o[j] = static_cast<TT>(e[j]);
      }
      return;
    }
#pragma unroll
    for (int q = 0; q < kPerThread; ++q) {
      const int i = threadIdx.x + q * kThreads;
      if (i >= kItemsTotal) continue;
      const int r = i % (2 * N), c = i / (2 * N);
      TT* o = tile + (c * kVec) * (2 * N) + r;
      const uint4 v = raw[i];
      const IO* e = reinterpret_cast<const IO*>(&v);
#pragma unroll
      for (int j = 0; j < kVec; ++j) o[j * 2 * N] = static_cast<TT>(e[j]);
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

// kStep: the given dt is a raw step to be biased / passed through softplus (a template parameter so that the
// plain case keeps its register allocation)
// kStepMajor: B and C are given [B, L, N] (a template parameter for the same reason)
template <typename IO, int N, bool kStep, bool kStepMajor>
__global__ void __launch_bounds__(kSerialLanes) sscan_forward_serial_kernel(Params p) {
  constexpr int NP = N / 2;
  constexpr int G = kSerialInterval;
  constexpr int kGroupsPerStage = kStage / G;
  constexpr int CH = kSerialCh;
  using Loader = TileLoader<IO, N, kSerialLanes>;
  using Stream = GroupStream<IO, kSerialLanes>;
  __shared__ __align__(16) float tile[2][kStage * 2 * N];   // fp32: no unpacking in the time loop
  __shared__ uint4 raw[Loader::kItemsTotal];
  __shared__ uint4 slab[2 * CH * Stream::kVecs * kSerialLanes];
  // outputs of one stage, [channel of the CTA][16-byte vector of the stage's steps]: written by the owning lane per
  // group, stored at the end of the stage with consecutive lanes covering consecutive bytes of a row
  constexpr int kOutVecs = kStage * (int)sizeof(IO) / 16;   // per channel and stage (4 or 8)
  static_assert(kOutVecs == 4 || kOutVecs == 8, "swizzle below");
  __shared__ uint4 ostage[kSerialSpan * kOutVecs];
  const long long b = blockIdx.y;
  const long long bc_batch = kStepMajor ? p.L * p.bc_pitch : N * p.L;   // elements per batch entry of B, C
  const IO* Bm_b = static_cast<const IO*>(p.Bm) + b * bc_batch;
  const IO* Cm_b = static_cast<const IO*>(p.Cm) + b * bc_batch;
  const bool tile_vec = kStepMajor ? p.bc_vec_ok : p.vec_ok;
  const IO* u_all = static_cast<const IO*>(p.u);
  const IO* z_all = static_cast<const IO*>(p.z);
  Stream stream{slab};

  long long dch[CH], off[CH];
  bool active[CH];
  float2 A2[CH][NP], h[CH][NP];
  float dskip[CH], dbias[CH];
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
    dbias[ch] = (kStep && p.delta_bias) ? __ldg(p.delta_bias + d) : 0.0f;
    // saved states are laid out [B, window, D, N]: the 32 channels of a warp store 2 KB contiguous per window
    cs_out[ch] = (p.chunk_states && active[ch]) ? p.chunk_states + (b * p.nstates * p.D + d) * N : nullptr;
  }

  const long long nstages = (p.L + kStage - 1) / kStage;
  Loader::issue(raw, Bm_b, Cm_b, 0, p.L, tile_vec, kStepMajor, p.bc_pitch);
  stream.issue(0, u_all, p.dt, z_all, off, 0, p.L, p.vec_ok);
  Loader::finish(raw, tile[0], kStepMajor);   // waits for everything issued so far
  __syncwarp();

  for (long long s = 0; s < nstages; ++s) {
    const int buf = (int)(s & 1);
    const bool staged = p.vec_ok && (s + 1) * kStage <= p.L;   // whole stage inside the sequence, rows 16-byte aligned
#pragma unroll 1
    for (int g = 0; g < kGroupsPerStage; ++g) {
      const long long t0 = s * kStage + (long long)g * G;
      if (t0 >= p.L) break;
      const int gb = g & 1;   // kGroupsPerStage is even: the parity of the global group index
      stream.issue(gb ^ 1, u_all, p.dt, z_all, off, t0 + G, p.L, p.vec_ok);
      if (g == 0 && s + 1 < nstages) {
        // next stage's B/C rows (each thread transposes only what it copied itself); issued after
        // the group prefetch so that waiting for this group's data does not wait for them
        Loader::issue(raw, Bm_b, Cm_b, (s + 1) * kStage, p.L, tile_vec, kStepMajor, p.bc_pitch);
        asm volatile("cp.async.wait_group 2;" ::: "memory");
      } else {
        asm volatile("cp.async.wait_group 1;" ::: "memory");   // everything but the prefetch just issued has landed
      }
      float u_c[CH][G], dt_c[CH][G], z_c[CH][G], y[CH][G];
#pragma unroll
      for (int ch = 0; ch < CH; ++ch) {
        stream.template read<IO>(gb, ch, 0, u_c[ch]);
        stream.template read<float>(gb, ch, Stream::kVecIO, dt_c[ch]);
        if constexpr (kStep) {   // steps past the end of the sequence stay zero (no-ops)
#pragma unroll
          for (int j = 0; j < G; ++j)
            dt_c[ch][j] = (t0 + j < p.L) ? step_transform(dt_c[ch][j], dbias[ch], p.delta_softplus != 0) : 0.0f;
        }
        if (z_all) stream.template read<IO>(gb, ch, Stream::kVecIO + 2, z_c[ch]);
        if (cs_out[ch]) {   // state entering this window
          float4* o = reinterpret_cast<float4*>(cs_out[ch] + (t0 / G) * p.D * N);
#pragma unroll
          for (int q = 0; q < NP / 2; ++q)
            o[q] = make_float4(h[ch][2 * q].x, h[ch][2 * q].y, h[ch][2 * q + 1].x, h[ch][2 * q + 1].y);
        }
      }
      const float* steps = tile[buf] + g * G * 2 * N;
#pragma unroll
      for (int j = 0; j < G; ++j) {
        float2 Bp[NP], Cp[NP];
        load_bc_step<float, N>(steps + j * 2 * N, Bp, Cp);
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
      if (staged) {
        constexpr int kV = Stream::kVecIO;   // vectors per group
#pragma unroll
        for (int ch = 0; ch < CH; ++ch) {
          // vector v of channel chn sits at chn * kOutVecs + (v ^ swizzle(chn)): 8 lanes hit 8 different bank groups
          const int chn = ch * kSerialLanes + threadIdx.x;
          const int sw = kOutVecs == 4 ? ((chn >> 1) & 3) : (chn & 7);
          uint4* ob = ostage + chn * kOutVecs;
          if constexpr (sizeof(IO) == 4) {
            ob[(g * kV) ^ sw] = make_uint4(__float_as_uint(y[ch][0]), __float_as_uint(y[ch][1]),
                                           __float_as_uint(y[ch][2]), __float_as_uint(y[ch][3]));
            ob[(g * kV + 1) ^ sw] = make_uint4(__float_as_uint(y[ch][4]), __float_as_uint(y[ch][5]),
                                               __float_as_uint(y[ch][6]), __float_as_uint(y[ch][7]));
          } else {
            uint32_t wv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const __nv_bfloat162 hv = __floats2bfloat162_rn(y[ch][2 * i], y[ch][2 * i + 1]);
              wv[i] = *reinterpret_cast<const uint32_t*>(&hv);
            }
            ob[(g * kV) ^ sw] = make_uint4(wv[0], wv[1], wv[2], wv[3]);
          }
        }
      } else {
#pragma unroll
        for (int ch = 0; ch < CH; ++ch)
          if (active[ch]) store_items<IO, G>(static_cast<IO*>(p.out) + off[ch], t0, p.L, p.vec_ok, y[ch]);
      }
    }
    if (staged) {
      __syncwarp();
      // kOutVecs consecutive lanes write one channel's stage (kStage elements, contiguous in memory)
#pragma unroll
      for (int it = 0; it < kSerialSpan * kOutVecs / kSerialLanes; ++it) {
        const int i = it * kSerialLanes + threadIdx.x;
        const int chn = i / kOutVecs, v = i % kOutVecs;
        const long long dd = (long long)blockIdx.x * kSerialSpan + chn;
        if (dd < p.D) {
          IO* dst = static_cast<IO*>(p.out) + (b * p.D + dd) * p.L + s * kStage;
          const int sw = kOutVecs == 4 ? ((chn >> 1) & 3) : (chn & 7);
          reinterpret_cast<uint4*>(dst)[v] = ostage[chn * kOutVecs + (v ^ sw)];
        }
      }
      __syncwarp();
    }
    if (s + 1 < nstages) Loader::finish(raw, tile[buf ^ 1], kStepMajor);
    __syncwarp();
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}

// ---------------------------------------------------------------------------
// backward
// ---------------------------------------------------------------------------
// Lane groups: the kSplit lanes l, l + CW, l + 2 CW ... of a warp (CW = 32 / kSplit channels
// per warp) own consecutive groups of NH = N / kSplit states of channel (warp base + l % CW),
// so a thread keeps, for one window of kSerialInterval steps, the decays a_t[n] and the states
// h_{t-1}[n] of its NH states in registers.  Windows are walked right to left.  Per window:
// re-run the forward recurrence from the state saved by the forward pass, then the adjoint
//     g_t = C_t * gy_t + a_{t+1} g_{t+1}
// right to left, forming du, ddt, dz (sums over the N states: shuffles between the lanes of a
// channel), dA, dD (register accumulators over the whole sequence) and the per-step
// dB_t[n] = g_t dt_t u_t, dC_t[n] = gy_t h_t, which are sums over channels: within a warp
// through a padded shared-memory transpose (lane c of a group ends up with value c of that
// group summed over the CW channels; this needs 2 NH = CW, i.e. N = 16), across the CTA's
// warps through a per-window partial tile, and across CTAs with one 16-byte vector atomic
// per (n, 4 steps).
constexpr int kBwdWarps = 4;
constexpr int kBwdThreads = kBwdWarps * 32;
constexpr float kLn2 = 0.6931471805599453f;

__device__ __forceinline__ void red_add_v4(float* addr, float4 v) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
               : "memory");
}

template <typename IO, int N, int kSplit>
struct BwdSmem {
  static constexpr int G = kSerialInterval;
  static constexpr int CW = 32 / kSplit;               // channels per warp
  static constexpr int NH = N / kSplit;                // states per thread
  static constexpr int kVecIO = G * (int)sizeof(IO) / 16;
  static constexpr int kChVecs = 3 * kVecIO + 2;       // u | dt dt | z | dout
  static constexpr int kSnapVecs = NH / 4;             // 16-byte vectors of a lane's saved state
  static constexpr int kPad = 2 * NH + 4;              // floats per lane in the transpose buffer (2 NH used):
                                                       // 20 and 12 keep the 16-byte stores of 8 lanes on distinct banks
  IO tile[2][kStage * 2 * N];                          // B | C per step, two stages
  uint4 raw[TileLoader<IO, N, kBwdThreads>::kItemsTotal];
  uint4 slab[2][kBwdWarps][kChVecs][CW];               // per-channel operands of a window, two windows
  uint4 snap[2][kBwdWarps][kSnapVecs][32];             // saved state of each lane's NH states
  float xpose[kBwdWarps][32 * kPad + kSplit * CW];     // per-warp transpose buffer (group g shifted by g*CW banks)
  float part[2][kBwdWarps][G][32];                     // per-warp channel sums of dB / dC of a window
};

template <typename IO, int N, int kSplit, bool kStep, bool kStepMajor>
__global__ void __launch_bounds__(kBwdThreads, kSplit == 2 ? 2 : 3) sscan_backward_serial_kernel(Params p) {
  using Smem = BwdSmem<IO, N, kSplit>;
  constexpr int G = kSerialInterval;
  constexpr int CW = Smem::CW;
  constexpr int NH = Smem::NH;        // states per thread
  constexpr int NQ = NH / 2;          // state pairs per thread
  constexpr int kSpan = kBwdWarps * CW;   // channels per CTA
  constexpr int kWinPerStage = kStage / G;
  constexpr int kVecIO = Smem::kVecIO;
  constexpr int kPad = Smem::kPad;
  static_assert(2 * NH == CW, "the channel reduction maps one value to one lane of a group");
  using Loader = TileLoader<IO, N, kBwdThreads>;
  extern __shared__ __align__(16) unsigned char bwd_smem_raw[];
  Smem& sm = *reinterpret_cast<Smem*>(bwd_smem_raw);
  auto& tile = sm.tile;
  auto& raw = sm.raw;
  auto& slab = sm.slab;
  auto& snap = sm.snap;
  auto& xpose = sm.xpose;
  auto& part = sm.part;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int grp = lane / CW, c = lane % CW;
  const long long b = blockIdx.y;
  const long long dch = (long long)blockIdx.x * kSpan + warp * CW + c;
  const bool active = dch < p.D;
  const long long d = active ? dch : 0;          // idle lanes shadow channel 0 and store nothing
  const long long row = (b * p.D + d) * p.L;
  const IO* u_row = static_cast<const IO*>(p.u) + row;
  const float* dt_row = p.dt + row;
  const IO* z_row = p.z ? static_cast<const IO*>(p.z) + row : nullptr;
  const IO* go_row = static_cast<const IO*>(p.dout) + row;
  const long long bc_batch = kStepMajor ? p.L * p.bc_pitch : N * p.L;   // elements per batch entry of B, C
  const IO* Bm_b = static_cast<const IO*>(p.Bm) + b * bc_batch;
  const IO* Cm_b = static_cast<const IO*>(p.Cm) + b * bc_batch;
  const bool tile_vec = kStepMajor ? p.bc_vec_ok : p.vec_ok;
  const float* snaps = p.chunk_states + (b * p.nstates * p.D + d) * N + grp * NH;   // [B, window, D, N]

  float2 A2[NQ], ag[NQ], dAacc[NQ];
#pragma unroll
  for (int q = 0; q < NQ; ++q) {
    const int n = grp * NH + 2 * q;
    A2[q] = make_float2(__ldg(p.A + d * N + n) * kLog2e, __ldg(p.A + d * N + n + 1) * kLog2e);
    ag[q] = make_float2(0.f, 0.f);
    dAacc[q] = make_float2(0.f, 0.f);
  }
  const float dskip = p.Dskip ? __ldg(p.Dskip + d) : 0.0f;
  const float dbias = (kStep && p.delta_bias) ? __ldg(p.delta_bias + d) : 0.0f;
  constexpr bool raw_step = kStep;   // the given dt is a raw step to be biased / passed through softplus
  float dDacc = 0.0f, dBiasAcc = 0.0f;

  const long long nwin = (p.L + G - 1) / G;
  const long long nstages = (p.L + kStage - 1) / kStage;

  // 16-byte vectors of one row segment -> slab (lanes of group 0 only) ----------------------------
  auto issue_vecs = [&](uint4* dst0, const void* rowp, int elem_bytes, long long t0, int nvec) {
    // dst0 + v * CW is this channel's v-th vector
    const char* src = static_cast<const char*>(rowp) + t0 * elem_bytes;
    if (p.vec_ok && t0 + G <= p.L) {
      for (int v = 0; v < nvec; ++v)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst0 + v * CW)), "l"(src + 16 * v)
                     : "memory");
    } else {
      const int per = 16 / elem_bytes;
      for (int v = 0; v < nvec; ++v) {
        uint4 tmp = make_uint4(0u, 0u, 0u, 0u);
        char* tb = reinterpret_cast<char*>(&tmp);
        for (int j = 0; j < per; ++j)
          if (t0 + v * per + j < p.L)
            for (int k = 0; k < elem_bytes; ++k) tb[j * elem_bytes + k] = src[(v * per + j) * elem_bytes + k];
        dst0[v * CW] = tmp;
      }
    }
  };
  auto issue_window = [&](int buf, long long w) {
    if (w >= 0) {
      const long long t0 = w * G;
      if (grp == 0) {
        uint4* base = &slab[buf][warp][0][c];
        issue_vecs(base, u_row, (int)sizeof(IO), t0, kVecIO);
        issue_vecs(base + kVecIO * CW, dt_row, 4, t0, 2);
        if (z_row) issue_vecs(base + (kVecIO + 2) * CW, z_row, (int)sizeof(IO), t0, kVecIO);
        issue_vecs(base + (2 * kVecIO + 2) * CW, go_row, (int)sizeof(IO), t0, kVecIO);
      }
      const float* sp = snaps + w * p.D * N;
#pragma unroll
      for (int v = 0; v < Smem::kSnapVecs; ++v)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(&snap[buf][warp][v][lane])),
                     "l"(sp + 4 * v) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  auto read_vecs = [&](const uint4* src0, int elem_bytes, float (&out)[G]) {
    if (elem_bytes == 4) {
#pragma unroll
      for (int v = 0; v < 2; ++v) {
        const uint4 r = src0[v * CW];
        out[4 * v] = __uint_as_float(r.x); out[4 * v + 1] = __uint_as_float(r.y);
        out[4 * v + 2] = __uint_as_float(r.z); out[4 * v + 3] = __uint_as_float(r.w);
      }
    } else {
      const uint4 r = src0[0];
      const uint32_t wv[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        out[2 * j] = __uint_as_float(wv[j] << 16);
        out[2 * j + 1] = __uint_as_float(wv[j] & 0xffff0000u);
      }
    }
  };
  // (state pairs of this lane's group) of B and C of one tile step
  auto load_bc_part = [&](const IO* step, float2 (&Bp)[NQ], float2 (&Cp)[NQ]) {
    if constexpr (sizeof(IO) == 4) {
      const float2* bv = reinterpret_cast<const float2*>(step + grp * NH);
      const float2* cv = reinterpret_cast<const float2*>(step + N + grp * NH);
      if constexpr (NQ % 2 == 0) {
#pragma unroll
        for (int q = 0; q < NQ; q += 2) {
          const float4 x = *reinterpret_cast<const float4*>(bv + q), y = *reinterpret_cast<const float4*>(cv + q);
          Bp[q] = make_float2(x.x, x.y); Bp[q + 1] = make_float2(x.z, x.w);
          Cp[q] = make_float2(y.x, y.y); Cp[q + 1] = make_float2(y.z, y.w);
        }
      } else {
#pragma unroll
        for (int q = 0; q < NQ; ++q) { Bp[q] = bv[q]; Cp[q] = cv[q]; }
      }
    } else {
      uint32_t bw[NQ], cw[NQ];   // a 32-bit word holds the bf16 of states 2q (low half) and 2q+1 (high half)
      if constexpr (NQ == 4) {
        const uint4 x = *reinterpret_cast<const uint4*>(step + grp * NH);
        const uint4 y = *reinterpret_cast<const uint4*>(step + N + grp * NH);
        bw[0] = x.x; bw[1] = x.y; bw[2] = x.z; bw[3] = x.w;
        cw[0] = y.x; cw[1] = y.y; cw[2] = y.z; cw[3] = y.w;
      } else {
        const uint2 x = *reinterpret_cast<const uint2*>(step + grp * NH);
        const uint2 y = *reinterpret_cast<const uint2*>(step + N + grp * NH);
        bw[0] = x.x; bw[1] = x.y;
        cw[0] = y.x; cw[1] = y.y;
      }
#pragma unroll
      for (int q = 0; q < NQ; ++q) {
        Bp[q] = make_float2(__uint_as_float(bw[q] << 16), __uint_as_float(bw[q] & 0xffff0000u));
        Cp[q] = make_float2(__uint_as_float(cw[q] << 16), __uint_as_float(cw[q] & 0xffff0000u));
      }
    }
  };
  // sum over the kSplit lanes of a channel
  auto channel_sum = [&](float v) {
#pragma unroll
    for (int m = CW; m < 32; m <<= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
    return v;
  };

  // prologue: last stage's tiles and the last window's operands
  Loader::issue(raw, Bm_b, Cm_b, (nstages - 1) * kStage, p.L, tile_vec, kStepMajor, p.bc_pitch);
  issue_window((int)((nwin - 1) & 1), nwin - 1);
  Loader::finish(raw, tile[(nstages - 1) & 1], kStepMajor);
  __syncthreads();

  for (long long w = nwin - 1; w >= 0; --w) {
    const long long t0 = w * G;
    const long long s = w / kWinPerStage;
    const int tb = (int)(s & 1), wb = (int)(w & 1);
    const int tl = (int)(w % kWinPerStage) * G;          // first step of the window inside the tile
    const bool stage_head = (w % kWinPerStage) == kWinPerStage - 1 || w == nwin - 1;   // first window of a stage we process
    issue_window(wb ^ 1, w - 1);
    if (stage_head && s > 0) {
      Loader::issue(raw, Bm_b, Cm_b, (s - 1) * kStage, p.L, tile_vec, kStepMajor, p.bc_pitch);
      asm volatile("cp.async.wait_group 2;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    }
    __syncwarp();   // group 0's copies are read by every lane of the channel

    float u_c[G], dt_c[G], z_c[G], go_c[G];
    {
      const uint4* base = &slab[wb][warp][0][c];
      read_vecs(base, (int)sizeof(IO), u_c);
      read_vecs(base + kVecIO * CW, 4, dt_c);
      if constexpr (raw_step) {   // steps past the end of the sequence stay zero (no-ops)
#pragma unroll
        for (int j = 0; j < G; ++j) dt_c[j] = (t0 + j < p.L) ? step_transform(dt_c[j], dbias, p.delta_softplus != 0) : 0.0f;
      }
      if (z_row) read_vecs(base + (kVecIO + 2) * CW, (int)sizeof(IO), z_c);
      read_vecs(base + (2 * kVecIO + 2) * CW, (int)sizeof(IO), go_c);
      if (!active) {   // a shadow lane must not add to the sums over channels
#pragma unroll
        for (int j = 0; j < G; ++j) go_c[j] = 0.0f;
      }
    }
    float2 h[NQ];
#pragma unroll
    for (int v = 0; v < Smem::kSnapVecs; ++v) {
      const uint4 sv = snap[wb][warp][v][lane];
      h[2 * v] = make_float2(__uint_as_float(sv.x), __uint_as_float(sv.y));
      h[2 * v + 1] = make_float2(__uint_as_float(sv.z), __uint_as_float(sv.w));
    }
    const IO* steps = tile[tb] + tl * 2 * N;

    // forward re-run of the window
    float2 a[G][NQ], hw[G][NQ];
    float yv[G];
#pragma unroll
    for (int j = 0; j < G; ++j) {
      float2 Bp[NQ], Cp[NQ];
      load_bc_part(steps + j * 2 * N, Bp, Cp);
      const float2 dtv = splat(dt_c[j]);
      const float2 dtu = splat(dt_c[j] * u_c[j]);
      float2 acc = make_float2(0.f, 0.f);
#pragma unroll
      for (int q = 0; q < NQ; ++q) {
        const float2 x = p2mul(dtv, A2[q]);
        a[j][q] = make_float2(ex2(x.x), ex2(x.y));
        hw[j][q] = h[q];
        h[q] = p2fma(a[j][q], h[q], p2mul(dtu, Bp[q]));
        acc = p2fma(Cp[q], h[q], acc);
      }
      yv[j] = acc.x + acc.y;
    }
    if (z_row) {
#pragma unroll
      for (int j = 0; j < G; ++j) yv[j] = fmaf(dskip, u_c[j], channel_sum(yv[j]));
    }

    // adjoint, right to left
    float du_v[G], ddt_v[G], dz_v[G];
    float* xp = xpose[warp];
#pragma unroll
    for (int j = G - 1; j >= 0; --j) {
      float2 Bp[NQ], Cp[NQ];
      load_bc_part(steps + j * 2 * N, Bp, Cp);
      float gy = go_c[j];
      if (z_row) {
        const float zv = z_c[j];
        const float sg = __fdividef(1.0f, 1.0f + ex2(-zv * kLog2e));
        gy = go_c[j] * zv * sg;
        dz_v[j] = go_c[j] * yv[j] * (sg * fmaf(zv, 1.0f - sg, 1.0f));
      }
      const float2 gy2 = splat(gy), dtv = splat(dt_c[j]), dtu = splat(dt_c[j] * u_c[j]);
      float2 gb = make_float2(0.f, 0.f), dd = make_float2(0.f, 0.f);
      float2 dBv[NQ], dCv[NQ];
#pragma unroll
      for (int q = 0; q < NQ; ++q) {
        const float2 h_after = (j == G - 1) ? h[q] : hw[(j + 1) % G][q];
        const float2 g = p2fma(Cp[q], gy2, ag[q]);
        dCv[q] = p2mul(gy2, h_after);
        const float2 t1 = p2mul(p2mul(g, hw[j][q]), a[j][q]);   // g * a_t * h_{t-1}
        dd = p2fma(t1, A2[q], dd);
        dAacc[q] = p2fma(t1, dtv, dAacc[q]);
        gb = p2fma(g, Bp[q], gb);
        dBv[q] = p2mul(g, dtu);
        ag[q] = p2mul(a[j][q], g);
      }
      const float sgb = channel_sum(gb.x + gb.y);
      const float sdd = channel_sum((dd.x + dd.y) * kLn2);      // A2 carries log2(e)
      du_v[j] = fmaf(dt_c[j], sgb, gy * dskip);
      ddt_v[j] = fmaf(u_c[j], sgb, sdd);
      if constexpr (raw_step) {   // gradient with respect to the raw step
        ddt_v[j] = (t0 + j < p.L) ? ddt_v[j] * step_transform_grad(dt_c[j], p.delta_softplus != 0) : 0.0f;
        dBiasAcc += ddt_v[j];
      }
      dDacc = fmaf(gy, u_c[j], dDacc);
      // sum dB, dC over the CW channels of this warp: lane (grp, c) ends with value c of its group
      float2* xo = reinterpret_cast<float2*>(xp + lane * kPad + grp * CW);
      if constexpr (NQ % 2 == 0) {
#pragma unroll
        for (int q = 0; q < NQ; q += 2) {
          *reinterpret_cast<float4*>(xo + q) = make_float4(dBv[q].x, dBv[q].y, dBv[q + 1].x, dBv[q + 1].y);
          *reinterpret_cast<float4*>(xo + NQ + q) = make_float4(dCv[q].x, dCv[q].y, dCv[q + 1].x, dCv[q + 1].y);
        }
      } else {
#pragma unroll
        for (int q = 0; q < NQ; ++q) { xo[q] = dBv[q]; xo[NQ + q] = dCv[q]; }
      }
      __syncwarp();
      float sum = 0.0f;
      const float* xi = xp + (grp * CW) * kPad + grp * CW + c;
#pragma unroll
      for (int k = 0; k < CW; ++k) sum += xi[k * kPad];
      part[wb][warp][j][lane] = sum;
      __syncwarp();
    }

    // per-channel outputs, spread over the lanes of the channel: du | ddt | dz.  (Staging them in shared memory
    // for row-contiguous stores, as the forward does with its output, cost more in barriers than it saved.)
    if (active) {
      if (grp == 0) store_items<IO, G>(static_cast<IO*>(p.du) + row, t0, p.L, p.vec_ok, du_v);
      if (grp == 1) store_items<float, G>(p.ddt + row, t0, p.L, p.vec_ok, ddt_v);
      if (z_row && grp == (kSplit > 2 ? 2 : 0))
        store_items<IO, G>(static_cast<IO*>(p.dz) + row, t0, p.L, p.vec_ok, dz_v);
    }
    if (stage_head && s > 0) Loader::finish(raw, tile[tb ^ 1], kStepMajor);
    __syncthreads();   // partials of this window and (at a stage head) the next tile are visible
    if (threadIdx.x < 64) {
      // value id l = (grp, c): c < NH -> dB[grp*NH + c], else dC[grp*NH + c - NH]; four steps per thread
      const int l = threadIdx.x & 31, jg = threadIdx.x >> 5;
      float4 sum4 = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int wq = 0; wq < kBwdWarps; ++wq) {
        sum4.x += part[wb][wq][4 * jg][l];
        sum4.y += part[wb][wq][4 * jg + 1][l];
        sum4.z += part[wb][wq][4 * jg + 2][l];
        sum4.w += part[wb][wq][4 * jg + 3][l];
      }
      const int lc = l % CW, n = (l / CW) * NH + (lc % NH);
      float* dst = ((lc >= NH) ? p.dC : p.dB) + (b * N + n) * p.L + t0 + 4 * jg;
      if (p.vec_ok && t0 + G <= p.L) {
        red_add_v4(dst, sum4);
      } else {
        const float vals[4] = {sum4.x, sum4.y, sum4.z, sum4.w};
        for (int k = 0; k < 4; ++k)
          if (t0 + 4 * jg + k < p.L) atomicAdd(dst + k, vals[k]);
      }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  if (active) {
#pragma unroll
    for (int q = 0; q < NQ; ++q) {
      const int n = grp * NH + 2 * q;
      p.dA_part[(b * p.D + d) * N + n] = dAacc[q].x;
      p.dA_part[(b * p.D + d) * N + n + 1] = dAacc[q].y;
    }
    if (p.dD_part && grp == 0) p.dD_part[b * p.D + d] = dDacc;
    if (p.dbias_part && grp == 0) p.dbias_part[b * p.D + d] = dBiasAcc;
  }
}

template <typename IO>
static int launch_fwd_serial(const Params& p, cudaStream_t stream) {
  dim3 grid((unsigned)((p.D + kSerialSpan - 1) / kSerialSpan), (unsigned)p.B);
  const bool step = p.delta_bias || p.delta_softplus;
  if (p.bc_step_major) {
    if (step) sscan_forward_serial_kernel<IO, 16, true, true><<<grid, kSerialLanes, 0, stream>>>(p);
    else sscan_forward_serial_kernel<IO, 16, false, true><<<grid, kSerialLanes, 0, stream>>>(p);
  } else {
    if (step) sscan_forward_serial_kernel<IO, 16, true, false><<<grid, kSerialLanes, 0, stream>>>(p);
    else sscan_forward_serial_kernel<IO, 16, false, false><<<grid, kSerialLanes, 0, stream>>>(p);
  }
  return check_cuda(cudaGetLastError(), "sscan_forward_serial_kernel launch");
}

}  // namespace sscan
}  // namespace ossm_b200

namespace ossm_b200 {
namespace sscan {
static int g_bwd_split = 2;   // lanes per channel in the serial backward (2 or 4; 2 measured 8 % faster)

template <typename IO, int kSplit>
static int launch_bwd_serial_split(const Params& p, cudaStream_t stream) {
  constexpr int kSpan = kBwdWarps * (32 / kSplit);
  dim3 grid((unsigned)((p.D + kSpan - 1) / kSpan), (unsigned)p.B);
  const size_t smem = sizeof(BwdSmem<IO, 16, kSplit>);
  const bool step = p.delta_bias || p.delta_softplus;
  auto kernel = p.bc_step_major ? (step ? sscan_backward_serial_kernel<IO, 16, kSplit, true, true>
                                        : sscan_backward_serial_kernel<IO, 16, kSplit, false, true>)
                                : (step ? sscan_backward_serial_kernel<IO, 16, kSplit, true, false>
                                        : sscan_backward_serial_kernel<IO, 16, kSplit, false, false>);
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), smem)) return rc;
  kernel<<<grid, kBwdThreads, smem, stream>>>(p);
  return check_cuda(cudaGetLastError(), "sscan_backward_serial_kernel launch");
}

template <typename IO>
static int launch_bwd_serial(const Params& p, cudaStream_t stream) {
  return g_bwd_split == 2 ? launch_bwd_serial_split<IO, 2>(p, stream) : launch_bwd_serial_split<IO, 4>(p, stream);
}
}  // namespace sscan
}  // namespace ossm_b200
