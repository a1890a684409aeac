// Mamba selective scan, forward, serial in time with the states of a channel split over lanes
// (included by selective_scan.cu inside namespace ossm_b200::sscan, after selective_scan_serial.cuh).
//
// State sizes 32, 64, 128, 256 (ossm's shipped Mamba4Rec configuration uses 256, configs/model/mambarec.yaml).
// The time-parallel forward of selective_scan.cu pays a warp scan of affine maps per state pair and chunk; for
// large states that is ten times the arithmetic of the recurrence itself.  Here a group of S = N/8 lanes owns one
// channel, every lane keeps 8 of its states in registers and walks the sequence like the reference CPU loop
// (selective_scan_cpu.cpp:118-152): per step and state one ex2, a multiply for the decay argument and two FMAs
// (packed two states at a time).  The only exchange is the sum of the S partial outputs y_t = sum_n C_t[n] h_t[n],
// done for eight steps at a time after the recurrence of those steps (shuffles off the dependent path).
//
// A CTA is 8 warps = 256 / S channels of one batch element; B_t / C_t tiles of 4096 / N steps are transposed into
// shared memory as float32 [step][B | C][half][lane][4] and read back with 16-byte loads (neighbouring lanes 16 bytes
// apart); a 16-bit I/O type keeps the tile in that type from 128 states on ([step][B | C][state], a lane's eight
// states one 16-byte read, twice the steps per tile).  u, dt arrive as one 8-step vector per row and group; the lane that ends up with a step's output after the
// exchange gates and stores it (staging u, dt, z one group ahead with asynchronous copies, as the backward does per
// chunk, was measured 5-10 % slower here: three resident CTAs already cover that latency).  The state entering
// every p.state_interval steps is saved in the layout the time-parallel backward reads ([B, D, L / interval, N]).

constexpr int kSplitWarps = 8;
constexpr int kSplitThreads = kSplitWarps * 32;
constexpr int kSplitStates = 8;                 // states per lane
constexpr int kSplitGroup = 8;                  // steps per register group
constexpr int kSplitTileFloats = 8192;          // floats per B|C tile: 4096 / N steps of 2 N values (32 KiB; 64 KiB is no faster)

// One 16-byte vector of a row, elements t .. t + 16 / elem_bytes - 1, into shared memory: an asynchronous copy where
// the row is 16-byte aligned and the vector lies inside it, else element by element with zeros past the end.
__device__ __forceinline__ void stage_vec(uint4* dst, const void* rowp, int elem_bytes, long long t, long long L,
                                          bool vec_ok) {
  const char* src = static_cast<const char*>(rowp) + t * elem_bytes;
  const int per = 16 / elem_bytes;
  if (vec_ok && t + per <= L) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
  } else {
    uint4 tmp = make_uint4(0u, 0u, 0u, 0u);
    char* tb = reinterpret_cast<char*>(&tmp);
    for (int j = 0; j < per; ++j)
      if (t + j < L)
        for (int k = 0; k < elem_bytes; ++k) tb[j * elem_bytes + k] = src[j * elem_bytes + k];
    *dst = tmp;
  }
}
// eight consecutive elements of a staged row (two vectors of float32, one of a 16-bit type) as floats
template <typename T>
__device__ __forceinline__ void read_staged8(const uint4* src, float (&out)[8]) {
  if constexpr (sizeof(T) == 4) {
#pragma unroll
    for (int v = 0; v < 2; ++v) {
      const uint4 r = src[v];
      out[4 * v] = __uint_as_float(r.x); out[4 * v + 1] = __uint_as_float(r.y);
      out[4 * v + 2] = __uint_as_float(r.z); out[4 * v + 3] = __uint_as_float(r.w);
    }
  } else {
    const uint4 r = src[0];
    const uint32_t wv[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      out[2 * j] = __uint_as_float(wv[j] << 16);
      out[2 * j + 1] = __uint_as_float(wv[j] & 0xffff0000u);
    }
  }
}
// element j of a staged row
template <typename T>
__device__ __forceinline__ float read_staged1(const uint4* src, int j) {
  if constexpr (sizeof(T) == 4) return reinterpret_cast<const float*>(src)[j];
  else return __uint_as_float((uint32_t) reinterpret_cast<const unsigned short*>(src)[j] << 16);
}

// Sums the eight per-step values v[0..7] over the S lanes of a channel (S = 4 .. 32, a power of two).  Each of the
// first rounds halves the values a lane carries (the lane with the mask bit clear keeps the lower half and hands the
// upper half over), so the exchange costs 4 + 2 + 1 (+ 1 per further round) shuffles instead of 8 per round.  On
// return v[0] is the total of step `sub >> (lgS - 3)` (S >= 8; lanes that agree in those bits hold the same total),
// resp. v[0], v[1] the totals of steps 2 sub, 2 sub + 1 (S = 4).
__device__ __forceinline__ void group_reduce_scatter8(float (&v)[8], int S, int lane) {
  int m = S >> 1;
  {
    const bool hi = (lane & m) != 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float send = hi ? v[i] : v[i + 4], keep = hi ? v[i + 4] : v[i];
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, m);
    }
    m >>= 1;
  }
  {
    const bool hi = (lane & m) != 0;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const float send = hi ? v[i] : v[i + 2], keep = hi ? v[i + 2] : v[i];
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, m);
    }
    m >>= 1;
  }
  if (m == 0) return;
  {
    const bool hi = (lane & m) != 0;
    const float send = hi ? v[0] : v[1], keep = hi ? v[1] : v[0];
    v[0] = keep + __shfl_xor_sync(0xffffffffu, send, m);
    m >>= 1;
  }
  for (; m > 0; m >>= 1) v[0] += __shfl_xor_sync(0xffffffffu, v[0], m);
}
// a += x as two packed additions
__device__ __forceinline__ void add4(float4& a, const float4& x) {
  const float2 lo = p2add(make_float2(a.x, a.y), make_float2(x.x, x.y));
  const float2 hi = p2add(make_float2(a.z, a.w), make_float2(x.z, x.w));
  a = make_float4(lo.x, lo.y, hi.x, hi.y);
}
// The steps of a window whose totals a lane holds after group_reduce_scatter8, and whether it is the lane that
// stores them (the first of the lanes holding the same total).
__device__ __forceinline__ void group_owned_steps(int S, int sub, int& first, int& count, bool& owner) {
  if (S >= 8) {
    const int lg = 31 - __clz(S);
    first = sub >> (lg - 3); count = 1; owner = (sub & ((S >> 3) - 1)) == 0;
  } else {
    first = 2 * sub; count = 2; owner = true;
  }
}

// kMinCtas: resident CTAs per SM the register allocation leaves room for -- 4 (64 registers) is faster from 64 states
// on, 3 (80 registers) at 32 states, where a warp carries eight channels and the per-group work per lane is largest.
// kKeep16: a 16-bit I/O type keeps its tile in that type (half the shared-memory reads, eight unpacking instructions
// per step): faster from 128 states on (N=256: 15.8 against 18.1 ms), slower below.
template <typename IO, bool kStep, int kMinCtas, bool kKeep16>
__global__ void __launch_bounds__(kSplitThreads, kMinCtas) sscan_forward_split_kernel(Params p) {
  extern __shared__ __align__(16) float split_tile[];            // [steps][2 N]
  constexpr int G = kSplitGroup;
  const int N = (int)p.N;
  const int S = N / kSplitStates;                                // lanes per channel
  // the tile keeps the I/O type: float32 as [step][B|C][half][lane][4], a 16-bit type as [step][B|C][state] (a lane's
  // eight states are one 16-byte read) with twice the steps in the same 32 KiB
  constexpr bool kTile16 = sizeof(IO) == 2 && kKeep16;
  constexpr int kTileElems = kTile16 ? 2 * kSplitTileFloats : kSplitTileFloats;
  IO* tile16 = reinterpret_cast<IO*>(split_tile);
  const int tile_steps = kTileElems / (2 * N);                   // 16 .. 256, a multiple of 8
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane % S;                                      // which 8 states of the channel
  const int per_warp = 32 / S;
  const long long b = blockIdx.y;
  const long long dch = (long long)blockIdx.x * (kSplitWarps * per_warp) + warp * per_warp + lane / S;
  const bool active = dch < p.D;
  const long long d = active ? dch : 0;                          // idle groups shadow channel 0 and store nothing
  const long long row = (b * p.D + d) * p.L;
  const IO* u_row = static_cast<const IO*>(p.u) + row;
  const float* dt_row = p.dt + row;
  const IO* z_row = p.z ? static_cast<const IO*>(p.z) + row : nullptr;
  IO* out_row = static_cast<IO*>(p.out) + row;
  const long long bc_batch = p.bc_step_major ? p.L * p.bc_pitch : p.N * p.L;   // elements per batch entry of B, C
  const IO* Bm_b = static_cast<const IO*>(p.Bm) + b * bc_batch;
  const IO* Cm_b = static_cast<const IO*>(p.Cm) + b * bc_batch;

  float2 A2[kSplitStates / 2], h[kSplitStates / 2];
#pragma unroll
  for (int q = 0; q < kSplitStates / 2; ++q) {
    const int n = sub * kSplitStates + 2 * q;
    A2[q] = make_float2(__ldg(p.A + d * N + n) * kLog2e, __ldg(p.A + d * N + n + 1) * kLog2e);
    h[q] = make_float2(0.f, 0.f);
  }
  const float dskip = p.Dskip ? __ldg(p.Dskip + d) : 0.0f;
  const float dbias = (kStep && p.delta_bias) ? __ldg(p.delta_bias + d) : 0.0f;
  float* snaps = p.chunk_states ? p.chunk_states + (b * p.D + d) * p.nstates * p.N + sub * kSplitStates : nullptr;

  int own_first, own_count;
  bool own_lane;
  group_owned_steps(S, sub, own_first, own_count, own_lane);
  const int save_every = p.state_interval / G;                   // groups between saved states (the interval is a multiple of 8)
  int until_save = 0;
  for (long long t_tile = 0; t_tile < p.L; t_tile += tile_steps) {
    __syncthreads();                       // the previous tile has been consumed
    // rows of B then C, one 16-byte vector of consecutive steps per item, transposed into [step][value]
    // (fetching the next tile into registers during the steps of this one was measured: no faster)
    constexpr int kVec = 16 / (int)sizeof(IO);
    if (p.bc_step_major) {
      // B, C given [B, L, N] (rows p.bc_pitch elements apart): a step's N values are contiguous, 16-byte pieces go
      // straight to their place in the tile
      const int lgP = 31 - __clz(N) - (kVec == 8 ? 3 : 2);       // log2 of the pieces per row
#pragma unroll 4
      for (int i = threadIdx.x; i < kTileElems / kVec; i += kSplitThreads) {
        const int g = i & ((1 << lgP) - 1), wc = (i >> lgP) & 1, st = i >> (lgP + 1);
        const long long t = t_tile + st;
        uint4 raw = make_uint4(0u, 0u, 0u, 0u);
        if (t < p.L) {
          const IO* src = (wc ? Cm_b : Bm_b) + t * p.bc_pitch + g * kVec;
          if (p.bc_vec_ok) {
            raw = *reinterpret_cast<const uint4*>(src);
          } else {
            IO* e = reinterpret_cast<IO*>(&raw);
#pragma unroll
            for (int j = 0; j < kVec; ++j) e[j] = src[j];
          }
        }
        float* dstp = split_tile + (size_t)st * 2 * N + wc * N;
        if constexpr (kTile16) {               // states 8g .. 8g+7 as they are
          *reinterpret_cast<uint4*>(tile16 + (size_t)st * 2 * N + wc * N + g * 8) = raw;
        } else if constexpr (kVec == 4) {      // states 4g .. 4g+3: lane g >> 1, half g & 1
          *reinterpret_cast<uint4*>(dstp + ((((g & 1) * S) + (g >> 1)) << 2)) = raw;
        } else {                               // states 8g .. 8g+7: lane g, both halves, as float32
          const uint32_t wv[4] = {raw.x, raw.y, raw.z, raw.w};
          *reinterpret_cast<float4*>(dstp + (g << 2)) =
              make_float4(__uint_as_float(wv[0] << 16), __uint_as_float(wv[0] & 0xffff0000u),
                          __uint_as_float(wv[1] << 16), __uint_as_float(wv[1] & 0xffff0000u));
          *reinterpret_cast<float4*>(dstp + ((S + g) << 2)) =
              make_float4(__uint_as_float(wv[2] << 16), __uint_as_float(wv[2] & 0xffff0000u),
                          __uint_as_float(wv[3] << 16), __uint_as_float(wv[3] & 0xffff0000u));
        }
      }
    } else if constexpr (kTile16) {
      for (int i = threadIdx.x; i < 2 * N * (tile_steps / kVec); i += kSplitThreads) {
        const int r = i & (2 * N - 1), cv = i >> (32 - __clz(N));      // N is a power of two
        const long long t = t_tile + (long long)kVec * cv;
        const IO* src = (r < N ? Bm_b + (long long)r * p.L : Cm_b + (long long)(r - N) * p.L);
        uint4 raw;
        IO* e = reinterpret_cast<IO*>(&raw);
        if (p.bc_vec_ok && t + kVec <= p.L) {
          raw = *reinterpret_cast<const uint4*>(src + t);
        } else {
#pragma unroll
          for (int j = 0; j < kVec; ++j) e[j] = (t + j < p.L) ? src[t + j] : IO(0.0f);
        }
#pragma unroll
        for (int j = 0; j < kVec; ++j) tile16[(kVec * cv + j) * 2 * N + r] = e[j];
      }
    } else
    for (int i = threadIdx.x; i < 2 * N * (tile_steps / kVec); i += kSplitThreads) {
      const int r = i & (2 * N - 1), cv = i >> (32 - __clz(N));      // N is a power of two
      const long long t = t_tile + (long long)kVec * cv;
      const IO* src = (r < N ? Bm_b + (long long)r * p.L : Cm_b + (long long)(r - N) * p.L);
      float v[kVec];
      load_items<IO, kVec>(src, t, p.L, p.bc_vec_ok, v);
      // state n = 8 * sub + 4 * half + e lives at ((half * S + sub) * 4 + e): a lane's two 16-byte reads of a step
      // are then 16 bytes apart from its neighbours' (read straight as [sub][8] they are 32 bytes apart and
      // conflict two ways: 41 % of the kernel's shared-memory wavefronts in the profile)
      const int rr = r < N ? r : r - N;
      const int pos = (r < N ? 0 : N) + ((((rr & 7) >> 2) * S + (rr >> 3)) << 2) + (rr & 3);
#pragma unroll
      for (int j = 0; j < kVec; ++j) split_tile[(kVec * cv + j) * 2 * N + pos] = v[j];
    }
    __syncthreads();
    const int groups = tile_steps / G;
    for (int gi = 0; gi < groups; ++gi) {
      const long long t0 = t_tile + (long long)gi * G;
      if (t0 >= p.L) break;                // block-uniform
      if (until_save == 0) {               // a counter instead of 64-bit divisions of t0 in the step loop
        until_save = save_every;
        if (snaps && active) {
          *reinterpret_cast<float4*>(snaps) = make_float4(h[0].x, h[0].y, h[1].x, h[1].y);
          *reinterpret_cast<float4*>(snaps + 4) = make_float4(h[2].x, h[2].y, h[3].x, h[3].y);
          snaps += p.N;
        }
      }
      --until_save;
      float u_c[G], dt_c[G];
      load_items<IO, G>(u_row, t0, p.L, p.vec_ok, u_c);
      if constexpr (kStep) {
        // the step transform once per step, not once per lane: lane `sub` of the channel transforms step sub (and
        // sub + 4 where the channel has four lanes), then every lane collects the eight values.  Steps past the end
        // of the sequence stay zero (no-ops).
        const long long ta = t0 + (sub & 7), tb = ta + 4;
        const float va = ta < p.L ? step_transform(__ldg(dt_row + ta), dbias, p.delta_softplus != 0) : 0.0f;
        const float vb = (S == 4 && tb < p.L) ? step_transform(__ldg(dt_row + tb), dbias, p.delta_softplus != 0) : 0.0f;
        const int base = lane & ~(S - 1);
#pragma unroll
        for (int j = 0; j < G; ++j)
          dt_c[j] = __shfl_sync(0xffffffffu, (S == 4 && j >= 4) ? vb : va, base + (S == 4 ? (j & 3) : j));
      } else {
        load_items<float, G>(dt_row, t0, p.L, p.vec_ok, dt_c);
      }
      // gate values of the steps this lane will finish: requested here so that the latency passes during the recurrence
      float z_m[2] = {0.0f, 0.0f};
      if (z_row && own_lane) {
#pragma unroll
        for (int e = 0; e < 2; ++e)
          if (e < own_count && t0 + own_first + e < p.L) z_m[e] = io_load<IO>(z_row + t0 + own_first + e);
      }
      float y[G];
      const float* steps = split_tile + (size_t)(gi * G) * 2 * N + sub * 4;
      const IO* steps16 = tile16 + (size_t)(gi * G) * 2 * N + sub * 8;
#pragma unroll
      for (int j = 0; j < G; ++j) {
        float2 Bp[4], Cp[4];
        if constexpr (kTile16) {
          const uint4 x = *reinterpret_cast<const uint4*>(steps16 + j * 2 * N);
          const uint4 y = *reinterpret_cast<const uint4*>(steps16 + j * 2 * N + N);
          const uint32_t bw[4] = {x.x, x.y, x.z, x.w}, cw[4] = {y.x, y.y, y.z, y.w};
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            Bp[q] = make_float2(__uint_as_float(bw[q] << 16), __uint_as_float(bw[q] & 0xffff0000u));
            Cp[q] = make_float2(__uint_as_float(cw[q] << 16), __uint_as_float(cw[q] & 0xffff0000u));
          }
        } else {
          const float4 b0 = *reinterpret_cast<const float4*>(steps + j * 2 * N);
          const float4 b1 = *reinterpret_cast<const float4*>(steps + j * 2 * N + 4 * S);
          const float4 c0 = *reinterpret_cast<const float4*>(steps + j * 2 * N + N);
          const float4 c1 = *reinterpret_cast<const float4*>(steps + j * 2 * N + N + 4 * S);
          Bp[0] = make_float2(b0.x, b0.y); Bp[1] = make_float2(b0.z, b0.w); Bp[2] = make_float2(b1.x, b1.y); Bp[3] = make_float2(b1.z, b1.w);
          Cp[0] = make_float2(c0.x, c0.y); Cp[1] = make_float2(c0.z, c0.w); Cp[2] = make_float2(c1.x, c1.y); Cp[3] = make_float2(c1.z, c1.w);
        }
        const float2 dtv = splat(dt_c[j]);
        const float2 dtu = splat(dt_c[j] * u_c[j]);
        float2 acc = make_float2(0.f, 0.f);
#pragma unroll
        for (int q = 0; q < kSplitStates / 2; ++q) {
          const float2 x = p2mul(dtv, A2[q]);
          const float2 a = make_float2(ex2(x.x), ex2(x.y));
          h[q] = p2fma(a, h[q], p2mul(dtu, Bp[q]));
          acc = p2fma(Cp[q], h[q], acc);
        }
        y[j] = acc.x + acc.y;
      }
      // sum over the lanes of the channel, eight steps at a time; the totals end up spread over the lanes, each of
      // which finishes and stores its own step (the owners of a window store 8 consecutive elements in one instruction)
      group_reduce_scatter8(y, S, lane);
      if (own_lane && active) {
        for (int e = 0; e < own_count; ++e) {
          const long long t = t0 + own_first + e;
          if (t < p.L) {
            float yy = fmaf(dskip, io_load<IO>(u_row + t), e == 0 ? y[0] : y[1]);
            if (z_row) {
              const float zz = e == 0 ? z_m[0] : z_m[1];
              yy *= zz * sigmoidf(zz);
            }
            io_store<IO>(out_row + t, yy);
          }
        }
      }
    }
  }
}

static bool split_ok(long long N) { return N == 32 || N == 64 || N == 128 || N == 256; }
static bool split_bwd_ok(long long N) { return split_ok(N); }

static int g_split_fwd_four_ctas_from = 64;   // state sizes from which the forward is built for four CTAs per SM (measured)
static int g_split_fwd_keep16_from = 128;     // state sizes from which a 16-bit I/O type keeps its tile in that type (measured)

template <typename IO>
static int launch_fwd_split(const Params& p, cudaStream_t stream) {
  const int per_cta = kSplitWarps * (32 / (int)(p.N / kSplitStates));
  dim3 grid((unsigned)((p.D + per_cta - 1) / per_cta), (unsigned)p.B);
  const size_t smem = kSplitTileFloats * sizeof(float);
  const bool step = p.delta_bias || p.delta_softplus;
  auto launch = [&](auto kernel) -> int {
    if (int rc = set_smem(kernel, smem)) return rc;
    kernel<<<grid, kSplitThreads, smem, stream>>>(p);
    return kOk;
  };
  int rc;
  if (sizeof(IO) == 2 && p.N >= g_split_fwd_keep16_from)
    rc = step ? launch(sscan_forward_split_kernel<IO, true, 4, true>) : launch(sscan_forward_split_kernel<IO, false, 4, true>);
  else if (p.N >= g_split_fwd_four_ctas_from)
    rc = step ? launch(sscan_forward_split_kernel<IO, true, 4, false>) : launch(sscan_forward_split_kernel<IO, false, 4, false>);
  else
    rc = step ? launch(sscan_forward_split_kernel<IO, true, 3, false>) : launch(sscan_forward_split_kernel<IO, false, 3, false>);
  if (rc) return rc;
  return check_cuda(cudaGetLastError(), "sscan_forward_split_kernel launch");
}

// ---------------------------------------------------------------------------------------------
// Backward for the same state sizes, same ownership (a group of S = N/8 lanes per channel, 8 states per lane).
//
// The forward saves the state entering every chunk of 32 steps.  Per chunk, right to left:
//   pass A   the recurrence from the saved state through the chunk's first three windows of 8 steps, keeping the state
//            that enters each window in shared memory (one more ex2 per step and state instead of four times the
//            saved states in HBM);
//   pass B   windows right to left: re-run of the window with the decays a_t[n] and the states h_{t-1}[n] kept in
//            registers, then the adjoint  g_t = C_t gy_t + a_{t+1} g_{t+1}  forming du, ddt, dz (sums over the states:
//            one exchange between the lanes of a channel per window, eight steps at a time), dA, dD (register
//            accumulators over the whole sequence) and dB_t[n] = g_t dt_t u_t, dC_t[n] = gy_t h_t (sums over the
//            channels): every lane stores its 16 values of a step into its warp's private slice of a half-window
//            buffer (conflict-free, no atomics); after every four steps the CTA sums the slices -- over its warps
//            and the 32 / S channels of each, with 16-byte loads, every thread a share of the rows -- and adds the
//            result to global memory with 16-byte vector atomics per (n, 4 steps).  Two half-window buffers
//            alternate, so one barrier per half window is enough.
// u, dt, z, dout of a chunk are copied into shared memory asynchronously one chunk ahead by the lanes of the channel, so
// that no global-load latency sits inside the window loops.
// Shared memory: B|C chunk tile in the I/O type [32][2N] | partial sums float [2][warps][4 steps][16][32] |
// window-entry states [3][8][threads] | chunk operands [2][channels][8 + 3 * (4 or 8) + 1 vectors].
constexpr int kSplitChunk = 32;
constexpr int kSplitWindows = kSplitChunk / kSplitGroup;

// kBwdWarps: 8 (one CTA per SM) where a warp holds a single channel and the B|C tile is the larger cost, else 4 (two
// CTAs per SM, whose barriers and phases overlap).
template <typename IO, bool kStep, int kBwdWarps>
__global__ void __launch_bounds__(kBwdWarps * 32, 8 / kBwdWarps) sscan_backward_split_kernel(Params p) {
  constexpr int kSplitBwdWarps = kBwdWarps;
  constexpr int kSplitBwdThreads = kBwdWarps * 32;
  constexpr int G = kSplitGroup;
  constexpr int NQ = kSplitStates / 2;
  extern __shared__ __align__(16) unsigned char split_smem[];
  const int N = (int)p.N;
  const int S = N / kSplitStates;
  IO* bc = reinterpret_cast<IO*>(split_smem);
  constexpr int kPartFloats = kSplitBwdWarps * 4 * 16 * 32;     // one half-window buffer
  float* part = reinterpret_cast<float*>(split_smem + (size_t)kSplitChunk * 2 * N * sizeof(IO));   // two of them
  float* wstate = part + 2 * kPartFloats;
  // dt | u | z | dout of a chunk of 32 steps, per channel, copied asynchronously one chunk ahead by the lanes of the
  // channel (an odd pitch in vectors keeps the channels of a warp on distinct banks)
  constexpr int kVIO = kSplitChunk * (int)sizeof(IO) / 16;      // vectors of u, z or dout per chunk: 4 or 8
  constexpr int kWIO = G * (int)sizeof(IO) / 16;                // ... per window: 1 or 2
  constexpr int kCV = 8 + 3 * kVIO, kCS = kCV + 1;
  uint4* cslab = reinterpret_cast<uint4*>(wstate + (kSplitWindows - 1) * kSplitStates * kSplitBwdThreads);   // [2][channels][kCS]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int lgN = 31 - __clz(N), lgS = lgN - 3;                 // N is a power of two
  const int sub = lane & (S - 1);
  const int per_warp = 32 >> lgS;
  const long long b = blockIdx.y;
  const long long dch = (long long)blockIdx.x * (kSplitBwdWarps * per_warp) + warp * per_warp + (lane >> lgS);
  const bool active = dch < p.D;
  const long long d = active ? dch : 0;                  // idle groups shadow channel 0 with a zero upstream gradient
  const long long row = (b * p.D + d) * p.L;
  const IO* u_row = static_cast<const IO*>(p.u) + row;
  const float* dt_row = p.dt + row;
  const IO* z_row = p.z ? static_cast<const IO*>(p.z) + row : nullptr;
  const IO* go_row = static_cast<const IO*>(p.dout) + row;
  const long long bc_batch = p.bc_step_major ? p.L * p.bc_pitch : p.N * p.L;   // elements per batch entry of B, C
  const IO* Bm_b = static_cast<const IO*>(p.Bm) + b * bc_batch;
  const IO* Cm_b = static_cast<const IO*>(p.Cm) + b * bc_batch;
  const float* snaps = p.chunk_states + (b * p.D + d) * p.nstates * p.N + sub * kSplitStates;

  float2 A2[NQ], ag[NQ], dAacc[NQ];
#pragma unroll
  for (int q = 0; q < NQ; ++q) {
    const int n = sub * kSplitStates + 2 * q;
    A2[q] = make_float2(__ldg(p.A + d * N + n) * kLog2e, __ldg(p.A + d * N + n + 1) * kLog2e);
    ag[q] = make_float2(0.f, 0.f);
    dAacc[q] = make_float2(0.f, 0.f);
  }
  const float dskip = p.Dskip ? __ldg(p.Dskip + d) : 0.0f;
  const float dbias = (kStep && p.delta_bias) ? __ldg(p.delta_bias + d) : 0.0f;
  float dDacc = 0.0f, dBiasAcc = 0.0f;
  int own_first, own_count;
  bool own_lane;
  group_owned_steps(S, sub, own_first, own_count, own_lane);
  const int ch_cta = warp * per_warp + (lane >> lgS);
  const int nch = kSplitBwdWarps * per_warp;
  auto issue_chunk = [&](long long cn) {
    if (cn >= 0) {
      const long long tn = cn * kSplitChunk;
      uint4* dst = cslab + ((size_t)(cn & 1) * nch + ch_cta) * kCS;
      for (int v = sub; v < kCV; v += S) {
        if (v < 8) {
          stage_vec(dst + v, dt_row, 4, tn + 4 * v, p.L, p.vec_ok);
        } else {
          const int k = (v - 8) / kVIO, vv = (v - 8) - k * kVIO;
          const IO* rowp = k == 0 ? u_row : (k == 1 ? z_row : go_row);
          if (rowp) stage_vec(dst + v, rowp, (int)sizeof(IO), tn + vv * (16 / (int)sizeof(IO)), p.L, p.vec_ok);
        }
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  // (state pairs of this lane) of B and C of one step of the tile
  // A float32 tile is laid out [step][B|C][half][lane][4] as in the forward (a lane's two 16-byte reads 16 bytes from
  // its neighbours'); a 16-bit tile keeps [step][B|C][state], where a lane's eight states are one 16-byte read.
  constexpr bool kPermuted = sizeof(IO) == 4;
  const int bc_lane = kPermuted ? sub * 4 : sub * kSplitStates;   // this lane's offset inside a step's B (or C) values
  auto load_bc8 = [&](const IO* stepp, float2 (&Bp)[NQ], float2 (&Cp)[NQ]) {
    if constexpr (sizeof(IO) == 4) {
      const float4 x0 = *reinterpret_cast<const float4*>(stepp), x1 = *reinterpret_cast<const float4*>(stepp + 4 * S);
      const float4 y0 = *reinterpret_cast<const float4*>(stepp + N), y1 = *reinterpret_cast<const float4*>(stepp + N + 4 * S);
      Bp[0] = make_float2(x0.x, x0.y); Bp[1] = make_float2(x0.z, x0.w); Bp[2] = make_float2(x1.x, x1.y); Bp[3] = make_float2(x1.z, x1.w);
      Cp[0] = make_float2(y0.x, y0.y); Cp[1] = make_float2(y0.z, y0.w); Cp[2] = make_float2(y1.x, y1.y); Cp[3] = make_float2(y1.z, y1.w);
    } else {
      const uint4 x = *reinterpret_cast<const uint4*>(stepp), y = *reinterpret_cast<const uint4*>(stepp + N);
      const uint32_t bw[4] = {x.x, x.y, x.z, x.w}, cw[4] = {y.x, y.y, y.z, y.w};
#pragma unroll
      for (int q = 0; q < NQ; ++q) {
        Bp[q] = make_float2(__uint_as_float(bw[q] << 16), __uint_as_float(bw[q] & 0xffff0000u));
        Cp[q] = make_float2(__uint_as_float(cw[q] << 16), __uint_as_float(cw[q] & 0xffff0000u));
      }
    }
  };
  // sums of one half window (steps 4*hq .. 4*hq+3 of the window at t0, buffer hq) over the CTA's channels, added to
  // dB / dC.  An item is (value v of 16, four consecutive lanes of a channel): a thread reads it with 16-byte loads from
  // its share of the (warp, channel-of-the-warp) rows, for the four steps, and issues one vector atomic per lane of the
  // four.  The rows are divided over `nparts` threads per item so that every thread of the CTA has work; the channel
  // index is rotated by v so that the loads of a quarter-warp fall into distinct banks.
  const int flush_items = 4 * S, lgI = lgS + 2;
  const int flush_rows = kSplitBwdWarps * per_warp;
  int nparts = kSplitBwdThreads >> lgI;
  if (p.split_flush_parts > 0 && p.split_flush_parts < nparts) nparts = p.split_flush_parts;
  const int rows_per_part = flush_rows / nparts;
  auto flush_half = [&](int hq, long long t0) {
    const int part_id = threadIdx.x >> lgI;
    if (part_id >= nparts) return;
    const int i = threadIdx.x & (flush_items - 1);
    const int v = i >> (lgS - 2), s4 = i & ((S >> 2) - 1);
    const float* pb = part + hq * kPartFloats + v * 32 + 4 * s4;
    float4 a0 = make_float4(0.f, 0.f, 0.f, 0.f), a1 = a0, a2 = a0, a3 = a0;
    const int r0 = part_id * rows_per_part;
#pragma unroll 4
    for (int rr = r0; rr < r0 + rows_per_part; ++rr) {
      const int w = rr >> (5 - lgS), cw = (rr ^ v) & (per_warp - 1);
      const float4* src = reinterpret_cast<const float4*>(pb + (size_t)(w * 4 * 16) * 32 + cw * S);
      const float4 x0 = src[0], x1 = src[16 * 32 / 4], x2 = src[2 * 16 * 32 / 4], x3 = src[3 * 16 * 32 / 4];
      add4(a0, x0); add4(a1, x1); add4(a2, x2); add4(a3, x3);
    }
    const int k = v & 7;
    float* base = ((v >> 3) ? p.dC : p.dB) + (b * N + (4 * s4) * kSplitStates + k) * p.L + t0 + 4 * hq;
    const float4 o[4] = {make_float4(a0.x, a1.x, a2.x, a3.x), make_float4(a0.y, a1.y, a2.y, a3.y),
                         make_float4(a0.z, a1.z, a2.z, a3.z), make_float4(a0.w, a1.w, a2.w, a3.w)};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float* dst = base + (long long)e * kSplitStates * p.L;     // state (4 s4 + e) * 8 + k
      if (p.bc_vec_ok && t0 + G <= p.L) {
        red_add_v4(dst, o[e]);
      } else {
        const float vals[4] = {o[e].x, o[e].y, o[e].z, o[e].w};
        for (int kk = 0; kk < 4; ++kk)
          if (t0 + 4 * hq + kk < p.L) atomicAdd(dst + kk, vals[kk]);
      }
    }
  };
  const long long nchunks = (p.L + kSplitChunk - 1) / kSplitChunk;
  issue_chunk(nchunks - 1);
  for (long long c = nchunks - 1; c >= 0; --c) {
    const long long t_c = c * kSplitChunk;
    __syncthreads();                       // the previous chunk's tile and the operand buffer of chunk c + 1 have been consumed
    issue_chunk(c - 1);
    // the state entering the chunk (in flight during the tile load)
    float2 h0[NQ];
    {
      const float* sp = snaps + c * p.N;
      const float4 s0 = *reinterpret_cast<const float4*>(sp), s1 = *reinterpret_cast<const float4*>(sp + 4);
      h0[0] = make_float2(s0.x, s0.y); h0[1] = make_float2(s0.z, s0.w);
      h0[2] = make_float2(s1.x, s1.y); h0[3] = make_float2(s1.z, s1.w);
    }
    {
      // rows of B then C, one 16-byte vector of consecutive steps per item, transposed into [step][value]; four
      // loads in flight per thread before the first store
      constexpr int kVec = 16 / (int)sizeof(IO);
      const int total = 2 * N * (kSplitChunk / kVec);
      if (p.bc_step_major) {
        // B, C given [B, L, N] (rows p.bc_pitch elements apart): a step's N values are contiguous, 16-byte pieces
        // go straight to their place in the tile
        const int lgP = lgN - (kVec == 8 ? 3 : 2);               // log2 of the pieces per row
        for (int i0 = threadIdx.x; i0 < total; i0 += 4 * kSplitBwdThreads) {
          uint4 v[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int i = i0 + k * kSplitBwdThreads;
            v[k] = make_uint4(0u, 0u, 0u, 0u);
            const int g = i & ((1 << lgP) - 1), wc = (i >> lgP) & 1, st = i >> (lgP + 1);
            const long long t = t_c + st;
            if (i < total && t < p.L) {
              const IO* src = (wc ? Cm_b : Bm_b) + t * p.bc_pitch + g * kVec;
              if (p.bc_vec_ok) {
                v[k] = *reinterpret_cast<const uint4*>(src);
              } else {
                IO* e = reinterpret_cast<IO*>(&v[k]);
#pragma unroll
                for (int j = 0; j < kVec; ++j) e[j] = src[j];
              }
            }
          }
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int i = i0 + k * kSplitBwdThreads;
            if (i < total) {
              const int g = i & ((1 << lgP) - 1), wc = (i >> lgP) & 1, st = i >> (lgP + 1);
              const int pos = wc * N + (kPermuted ? ((((g & 1) * S) + (g >> 1)) << 2) : g * kVec);
              *reinterpret_cast<uint4*>(bc + (size_t)st * 2 * N + pos) = v[k];
            }
          }
        }
      } else
      for (int i0 = threadIdx.x; i0 < total; i0 += 4 * kSplitBwdThreads) {
        uint4 v[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int i = i0 + k * kSplitBwdThreads;
          v[k] = make_uint4(0u, 0u, 0u, 0u);
          if (i < total) {
            const int r = i & (2 * N - 1), cv = i >> (lgN + 1);
            const long long t = t_c + (long long)kVec * cv;
            const IO* src = (r < N ? Bm_b + (long long)r * p.L : Cm_b + (long long)(r - N) * p.L);
            if (p.bc_vec_ok && t + kVec <= p.L) {
              v[k] = *reinterpret_cast<const uint4*>(src + t);
            } else {
              IO* e = reinterpret_cast<IO*>(&v[k]);
#pragma unroll
              for (int j = 0; j < kVec; ++j) e[j] = (t + j < p.L) ? src[t + j] : IO(0.0f);
            }
          }
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int i = i0 + k * kSplitBwdThreads;
          if (i < total) {
            const int r = i & (2 * N - 1), cv = i >> (lgN + 1);
            const IO* e = reinterpret_cast<const IO*>(&v[k]);
            int pos = r;
            if constexpr (kPermuted) {
              const int rr = r & (N - 1);
              pos = (r & N) + ((((rr & 7) >> 2) * S + (rr >> 3)) << 2) + (rr & 3);
            }
#pragma unroll
            for (int j = 0; j < kVec; ++j) bc[(kVec * cv + j) * 2 * N + pos] = e[j];
          }
        }
      }
    }
    asm volatile("cp.async.wait_group 1;" ::: "memory");   // this chunk's operands have landed
    uint4* cs = cslab + ((size_t)(c & 1) * nch + ch_cta) * kCS;
    if constexpr (kStep) {
      // the step transform once per step of the chunk, in place, shared by the lanes of the channel and by both
      // passes; steps past the end of the sequence were staged as zeros and stay zero (no-ops)
      __syncwarp();
      float* dts = reinterpret_cast<float*>(cs);
      for (int j = sub; j < kSplitChunk; j += S)
        if (t_c + j < p.L) dts[j] = step_transform(dts[j], dbias, p.delta_softplus != 0);
    }
    __syncthreads();
    // ---- pass A: states entering windows 1 .. 3
    {
      float2 h[NQ];
#pragma unroll
      for (int q = 0; q < NQ; ++q) h[q] = h0[q];
#pragma unroll 1
      for (int w = 0; w + 1 < kSplitWindows; ++w) {
        const long long t0 = t_c + (long long)w * G;
        if (t0 + G >= p.L) break;            // no later window inside the sequence (block-uniform)
        float u_c[G], dt_c[G];
        read_staged8<float>(cs + 2 * w, dt_c);
        read_staged8<IO>(cs + 8 + kWIO * w, u_c);
#pragma unroll
        for (int j = 0; j < G; ++j) {
          float2 Bp[NQ], Cp[NQ];
          load_bc8(bc + (size_t)(w * G + j) * 2 * N + bc_lane, Bp, Cp);
          const float2 dtv = splat(dt_c[j]), dtu = splat(dt_c[j] * u_c[j]);
#pragma unroll
          for (int q = 0; q < NQ; ++q) {
            const float2 x = p2mul(dtv, A2[q]);
            h[q] = p2fma(make_float2(ex2(x.x), ex2(x.y)), h[q], p2mul(dtu, Bp[q]));
          }
        }
#pragma unroll
        for (int q = 0; q < NQ; ++q) {
          wstate[((w * kSplitStates) + 2 * q) * kSplitBwdThreads + threadIdx.x] = h[q].x;
          wstate[((w * kSplitStates) + 2 * q + 1) * kSplitBwdThreads + threadIdx.x] = h[q].y;
        }
      }
    }
    // ---- pass B: windows right to left
#pragma unroll 1
    for (int w = kSplitWindows - 1; w >= 0; --w) {
      const long long t0 = t_c + (long long)w * G;
      if (t0 >= p.L) continue;               // block-uniform
      float u_c[G], dt_c[G], z_c[G], go_c[G];
      read_staged8<float>(cs + 2 * w, dt_c);
      read_staged8<IO>(cs + 8 + kWIO * w, u_c);
      if (z_row) read_staged8<IO>(cs + 8 + kVIO + kWIO * w, z_c);
      read_staged8<IO>(cs + 8 + 2 * kVIO + kWIO * w, go_c);
      if (!active) {
#pragma unroll
        for (int j = 0; j < G; ++j) go_c[j] = 0.0f;
      }
      float2 h[NQ];
      if (w == 0) {
#pragma unroll
        for (int q = 0; q < NQ; ++q) h[q] = h0[q];
      } else {
#pragma unroll
        for (int q = 0; q < NQ; ++q)
          h[q] = make_float2(wstate[(((w - 1) * kSplitStates) + 2 * q) * kSplitBwdThreads + threadIdx.x],
                             wstate[(((w - 1) * kSplitStates) + 2 * q + 1) * kSplitBwdThreads + threadIdx.x]);
      }
      const IO* steps = bc + (size_t)(w * G) * 2 * N + bc_lane;
      // re-run of the window
      float2 a[G][NQ], hw[G][NQ];
      float yv[G];
#pragma unroll
      for (int j = 0; j < G; ++j) {
        float2 Bp[NQ], Cp[NQ];
        load_bc8(steps + (size_t)j * 2 * N, Bp, Cp);
        const float2 dtv = splat(dt_c[j]), dtu = splat(dt_c[j] * u_c[j]);
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
      // adjoint, right to left (the partial outputs yv are summed over the lanes after it, with du and ddt)
      float du_v[G], ddt_v[G];
#pragma unroll
      for (int j = G - 1; j >= 0; --j) {
        float2 Bp[NQ], Cp[NQ];
        load_bc8(steps + (size_t)j * 2 * N, Bp, Cp);
        float gy = go_c[j];
        if (z_row) {
          const float zv = z_c[j];
          gy = go_c[j] * zv * __fdividef(1.0f, 1.0f + ex2(-zv * kLog2e));
        }
        const float2 gy2 = splat(gy), dtv = splat(dt_c[j]), dtu = splat(dt_c[j] * u_c[j]);
        float2 gb = make_float2(0.f, 0.f), dd = make_float2(0.f, 0.f);
        float* pp = part + (j >> 2) * kPartFloats + (size_t)((warp * 4 + (j & 3)) * 16) * 32 + lane;   // [half][warp][step][value][lane]
#pragma unroll
        for (int q = 0; q < NQ; ++q) {
          const float2 h_after = (j == G - 1) ? h[q] : hw[(j + 1) % G][q];
          const float2 g = p2fma(Cp[q], gy2, ag[q]);
          const float2 dCv = p2mul(gy2, h_after);
          const float2 t1 = p2mul(p2mul(g, hw[j][q]), a[j][q]);   // g * a_t * h_{t-1}
          dd = p2fma(t1, A2[q], dd);
          dAacc[q] = p2fma(t1, dtv, dAacc[q]);
          gb = p2fma(g, Bp[q], gb);
          const float2 dBv = p2mul(g, dtu);
          ag[q] = p2mul(a[j][q], g);
          pp[(2 * q) * 32] = dBv.x;
          pp[(2 * q + 1) * 32] = dBv.y;
          pp[(8 + 2 * q) * 32] = dCv.x;
          pp[(8 + 2 * q + 1) * 32] = dCv.y;
        }
        du_v[j] = gb.x + gb.y;
        ddt_v[j] = (dd.x + dd.y) * kLn2;                          // A2 carries log2(e)
        dDacc = fmaf(gy, u_c[j], dDacc);
        if ((j & 3) == 0) {
          // the half window is complete in every warp's slice of buffer j >> 2; the other buffer, which the next four
          // steps fill, was summed before this barrier, and this one is next written after the following barrier
          __syncthreads();
          flush_half(j >> 2, t0);
        }
      }
      // sums over the states: the totals of the window's steps end up spread over the lanes of the channel, and the
      // lane holding a step finishes du, ddt, dz of that step from the step's scalars and stores them
      group_reduce_scatter8(du_v, S, lane);
      group_reduce_scatter8(ddt_v, S, lane);
      if (z_row) group_reduce_scatter8(yv, S, lane);
      if (own_lane && active) {
        for (int e = 0; e < own_count; ++e) {
          const long long t = t0 + own_first + e;
          if (t >= p.L) break;
          const float sgb = e == 0 ? du_v[0] : du_v[1], sdd = e == 0 ? ddt_v[0] : ddt_v[1];
          const int jc = w * G + own_first + e;          // step inside the chunk
          const float u_m = read_staged1<IO>(cs + 8, jc), go_m = read_staged1<IO>(cs + 8 + 2 * kVIO, jc);
          const float dt_m = read_staged1<float>(cs, jc);         // already transformed
          float gy = go_m;
          if (z_row) {
            const float zv = read_staged1<IO>(cs + 8 + kVIO, jc);
            const float sg = __fdividef(1.0f, 1.0f + ex2(-zv * kLog2e));
            const float y_m = fmaf(dskip, u_m, e == 0 ? yv[0] : yv[1]);
            gy = go_m * zv * sg;
            io_store<IO>(static_cast<IO*>(p.dz) + row + t, go_m * y_m * (sg * fmaf(zv, 1.0f - sg, 1.0f)));
          }
          io_store<IO>(static_cast<IO*>(p.du) + row + t, fmaf(dt_m, sgb, gy * dskip));
          float ddt_m = fmaf(u_m, sgb, sdd);
          if constexpr (kStep) {     // gradient with respect to the raw step
            ddt_m *= step_transform_grad(dt_m, p.delta_softplus != 0);
            dBiasAcc += ddt_m;
          }
          p.ddt[row + t] = ddt_m;
        }
      }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  if (p.dbias_part) {                      // the steps of a channel were finished by different lanes
    for (int m = 1; m < S; m <<= 1) dBiasAcc += __shfl_xor_sync(0xffffffffu, dBiasAcc, m);
  }
  if (active) {
#pragma unroll
    for (int q = 0; q < NQ; ++q) {
      const int n = sub * kSplitStates + 2 * q;
      p.dA_part[(b * p.D + d) * N + n] = dAacc[q].x;
      p.dA_part[(b * p.D + d) * N + n + 1] = dAacc[q].y;
    }
    if (p.dD_part && sub == 0) p.dD_part[b * p.D + d] = dDacc;
    if (p.dbias_part && sub == 0) p.dbias_part[b * p.D + d] = dBiasAcc;
  }
}

template <typename IO, int kSplitBwdWarps>
static int launch_bwd_split_w(const Params& p, cudaStream_t stream) {
  constexpr int kSplitBwdThreads = kSplitBwdWarps * 32;
  const int per_cta = kSplitBwdWarps * (32 / (int)(p.N / kSplitStates));
  dim3 grid((unsigned)((p.D + per_cta - 1) / per_cta), (unsigned)p.B);
  const size_t smem = (size_t)kSplitChunk * 2 * p.N * sizeof(IO) + (size_t)2 * kSplitBwdWarps * 4 * 16 * 32 * sizeof(float) +
                      (size_t)(kSplitWindows - 1) * kSplitStates * kSplitBwdThreads * sizeof(float) +
                      2 * (size_t)per_cta * (8 + 3 * (kSplitChunk * sizeof(IO) / 16) + 1) * 16;
  if (p.delta_bias || p.delta_softplus) {
    if (int rc = set_smem(sscan_backward_split_kernel<IO, true, kSplitBwdWarps>, smem)) return rc;
    sscan_backward_split_kernel<IO, true, kSplitBwdWarps><<<grid, kSplitBwdThreads, smem, stream>>>(p);
  } else {
    if (int rc = set_smem(sscan_backward_split_kernel<IO, false, kSplitBwdWarps>, smem)) return rc;
    sscan_backward_split_kernel<IO, false, kSplitBwdWarps><<<grid, kSplitBwdThreads, smem, stream>>>(p);
  }
  return check_cuda(cudaGetLastError(), "sscan_backward_split_kernel launch");
}

static int g_split_bwd_wide_from = 128;     // state sizes from which the backward uses 8-warp CTAs (measured)
static int g_split_flush_parts = 0;         // threads sharing the rows of one flush item; 0 = measured default by state size

template <typename IO>
static int launch_bwd_split(const Params& p, cudaStream_t stream) {
  Params q = p;
  // fewer threads per item mean fewer vector atomics: 32 states ran fastest with 4, 64 / 128 with 2, 256 with 1
  q.split_flush_parts = g_split_flush_parts > 0 ? g_split_flush_parts : (q.N <= 32 ? 4 : (q.N <= 128 ? 2 : 1));
  return q.N >= g_split_bwd_wide_from ? launch_bwd_split_w<IO, 8>(q, stream) : launch_bwd_split_w<IO, 4>(q, stream);
}
