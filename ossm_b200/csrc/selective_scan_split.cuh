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
// shared memory as float32 [step][B_0..B_{N-1} | C_0..C_{N-1}] and read back with 16-byte loads (the lanes of a
// channel read consecutive 32-byte pieces).  u, dt, z arrive as one 8-step vector per row and group, the output leaves
// the same way from the group's first lane.  The state entering every p.state_interval steps is saved in the
// layout the time-parallel backward reads ([B, D, L / interval, N]).

constexpr int kSplitWarps = 8;
constexpr int kSplitThreads = kSplitWarps * 32;
constexpr int kSplitStates = 8;                 // states per lane
constexpr int kSplitGroup = 8;                  // steps per register group
constexpr int kSplitTileFloats = 8192;          // floats per B|C tile: 4096 / N steps of 2 N values (32 KiB; 64 KiB is no faster)

template <typename IO, bool kStep>
__global__ void __launch_bounds__(kSplitThreads) sscan_forward_split_kernel(Params p) {
  extern __shared__ __align__(16) float split_tile[];            // [steps][2 N]
  constexpr int G = kSplitGroup;
  const int N = (int)p.N;
  const int S = N / kSplitStates;                                // lanes per channel
  const int tile_steps = kSplitTileFloats / (2 * N);             // 16 .. 128, a multiple of 8
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
  const IO* Bm_b = static_cast<const IO*>(p.Bm) + b * p.N * p.L;
  const IO* Cm_b = static_cast<const IO*>(p.Cm) + b * p.N * p.L;

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

  for (long long t_tile = 0; t_tile < p.L; t_tile += tile_steps) {
    __syncthreads();                       // the previous tile has been consumed
    // rows of B then C, one 16-byte vector of consecutive steps per item, transposed into [step][value]
    // (fetching the next tile into registers during the steps of this one was measured: no faster)
    constexpr int kVec = 16 / (int)sizeof(IO);
    for (int i = threadIdx.x; i < 2 * N * (tile_steps / kVec); i += kSplitThreads) {
      const int r = i % (2 * N), cv = i / (2 * N);
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
      if (snaps && (t0 % p.state_interval) == 0 && active) {
        float* dst = snaps + (t0 / p.state_interval) * p.N;
        *reinterpret_cast<float4*>(dst) = make_float4(h[0].x, h[0].y, h[1].x, h[1].y);
        *reinterpret_cast<float4*>(dst + 4) = make_float4(h[2].x, h[2].y, h[3].x, h[3].y);
      }
      float u_c[G], dt_c[G];
      load_items<IO, G>(u_row, t0, p.L, p.vec_ok, u_c);
      load_items<float, G>(dt_row, t0, p.L, p.vec_ok, dt_c);
      if constexpr (kStep) {               // steps past the end of the sequence stay zero (no-ops)
#pragma unroll
        for (int j = 0; j < G; ++j) dt_c[j] = (t0 + j < p.L) ? step_transform(dt_c[j], dbias, p.delta_softplus != 0) : 0.0f;
      }
      float y[G];
      const float* steps = split_tile + (size_t)(gi * G) * 2 * N + sub * 4;
#pragma unroll
      for (int j = 0; j < G; ++j) {
        const float4 b0 = *reinterpret_cast<const float4*>(steps + j * 2 * N);
        const float4 b1 = *reinterpret_cast<const float4*>(steps + j * 2 * N + 4 * S);
        const float4 c0 = *reinterpret_cast<const float4*>(steps + j * 2 * N + N);
        const float4 c1 = *reinterpret_cast<const float4*>(steps + j * 2 * N + N + 4 * S);
        const float2 Bp[4] = {make_float2(b0.x, b0.y), make_float2(b0.z, b0.w), make_float2(b1.x, b1.y), make_float2(b1.z, b1.w)};
        const float2 Cp[4] = {make_float2(c0.x, c0.y), make_float2(c0.z, c0.w), make_float2(c1.x, c1.y), make_float2(c1.z, c1.w)};
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
      // sum over the lanes of the channel, eight steps at a time
      for (int m = 1; m < S; m <<= 1) {
#pragma unroll
        for (int j = 0; j < G; ++j) y[j] += __shfl_xor_sync(0xffffffffu, y[j], m);
      }
      if (sub == 0 && active) {
#pragma unroll
        for (int j = 0; j < G; ++j) y[j] = fmaf(dskip, u_c[j], y[j]);
        if (z_row) {
          float zz[G];
          load_items<IO, G>(z_row, t0, p.L, p.vec_ok, zz);
#pragma unroll
          for (int j = 0; j < G; ++j) y[j] *= zz[j] * sigmoidf(zz[j]);
        }
        store_items<IO, G>(out_row, t0, p.L, p.vec_ok, y);
      }
    }
  }
}

static bool split_ok(long long N) { return N == 32 || N == 64 || N == 128 || N == 256; }
static bool split_bwd_ok(long long N) { return split_ok(N); }

template <typename IO>
static int launch_fwd_split(const Params& p, cudaStream_t stream) {
  const int per_cta = kSplitWarps * (32 / (int)(p.N / kSplitStates));
  dim3 grid((unsigned)((p.D + per_cta - 1) / per_cta), (unsigned)p.B);
  const size_t smem = kSplitTileFloats * sizeof(float);
  if (p.delta_bias || p.delta_softplus) {
    if (int rc = set_smem(sscan_forward_split_kernel<IO, true>, smem)) return rc;
    sscan_forward_split_kernel<IO, true><<<grid, kSplitThreads, smem, stream>>>(p);
  } else {
    if (int rc = set_smem(sscan_forward_split_kernel<IO, false>, smem)) return rc;
    sscan_forward_split_kernel<IO, false><<<grid, kSplitThreads, smem, stream>>>(p);
  }
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
//            buffer (conflict-free, no atomics); after every four steps the CTA sums the slices -- over its 8 warps
//            and the 32 / S channels of each -- and adds the result to global memory with one 16-byte vector atomic
//            per (n, 4 steps).
// Shared memory: B|C chunk tile in the I/O type [32][2N] | partial sums float [8 warps][4 steps][16][32] |
// window-entry states [3][8][256].
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
  float* part = reinterpret_cast<float*>(split_smem + (size_t)kSplitChunk * 2 * N * sizeof(IO));
  float* wstate = part + kSplitBwdWarps * 4 * 16 * 32;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane % S;
  const int per_warp = 32 / S;
  const long long b = blockIdx.y;
  const long long dch = (long long)blockIdx.x * (kSplitBwdWarps * per_warp) + warp * per_warp + lane / S;
  const bool active = dch < p.D;
  const long long d = active ? dch : 0;                  // idle groups shadow channel 0 with a zero upstream gradient
  const long long row = (b * p.D + d) * p.L;
  const IO* u_row = static_cast<const IO*>(p.u) + row;
  const float* dt_row = p.dt + row;
  const IO* z_row = p.z ? static_cast<const IO*>(p.z) + row : nullptr;
  const IO* go_row = static_cast<const IO*>(p.dout) + row;
  const IO* Bm_b = static_cast<const IO*>(p.Bm) + b * p.N * p.L;
  const IO* Cm_b = static_cast<const IO*>(p.Cm) + b * p.N * p.L;
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

  // (state pairs of this lane) of B and C of one step of the tile
  auto load_bc8 = [&](const IO* stepp, float2 (&Bp)[NQ], float2 (&Cp)[NQ]) {
    if constexpr (sizeof(IO) == 4) {
      const float4 x0 = *reinterpret_cast<const float4*>(stepp), x1 = *reinterpret_cast<const float4*>(stepp + 4);
      const float4 y0 = *reinterpret_cast<const float4*>(stepp + N), y1 = *reinterpret_cast<const float4*>(stepp + N + 4);
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
  // sums of one half window (steps 4*hq .. 4*hq+3 of the window at t0) over the CTA's channels, added to dB / dC
  auto flush_half = [&](int hq, long long t0) {
    const int per_warp_ch = 32 / S;
    for (int i = threadIdx.x; i < 2 * N; i += kSplitBwdThreads) {
      const int is_c = i / N, r = i - is_c * N;
      const int k = r / S, sb = r - k * S;
      const int v = is_c * 8 + k;
      float4 s4 = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int w = 0; w < kSplitBwdWarps; ++w) {
        for (int cw = 0; cw < per_warp_ch; ++cw) {
          const float* src = part + (size_t)((w * 4) * 16 + v) * 32 + cw * S + sb;
          s4.x += src[0]; s4.y += src[16 * 32]; s4.z += src[2 * 16 * 32]; s4.w += src[3 * 16 * 32];
        }
      }
      const int n = sb * kSplitStates + k;
      float* dst = (is_c ? p.dC : p.dB) + (b * N + n) * p.L + t0 + 4 * hq;
      if (p.bc_vec_ok && t0 + G <= p.L) {
        red_add_v4(dst, s4);
      } else {
        const float vals[4] = {s4.x, s4.y, s4.z, s4.w};
        for (int kk = 0; kk < 4; ++kk)
          if (t0 + 4 * hq + kk < p.L) atomicAdd(dst + kk, vals[kk]);
      }
    }
  };
  const long long nchunks = (p.L + kSplitChunk - 1) / kSplitChunk;
  for (long long c = nchunks - 1; c >= 0; --c) {
    const long long t_c = c * kSplitChunk;
    __syncthreads();                       // the previous chunk's tile has been consumed
    {
      constexpr int kVec = 16 / (int)sizeof(IO);
      for (int i = threadIdx.x; i < 2 * N * (kSplitChunk / kVec); i += kSplitBwdThreads) {
        const int r = i % (2 * N), cv = i / (2 * N);
        const long long t = t_c + (long long)kVec * cv;
        const IO* src = (r < N ? Bm_b + (long long)r * p.L : Cm_b + (long long)(r - N) * p.L);
        IO v[kVec];
        if (p.bc_vec_ok && t + kVec <= p.L) {
          *reinterpret_cast<uint4*>(v) = *reinterpret_cast<const uint4*>(src + t);
        } else {
#pragma unroll
          for (int j = 0; j < kVec; ++j) v[j] = (t + j < p.L) ? src[t + j] : IO(0.0f);
        }
#pragma unroll
        for (int j = 0; j < kVec; ++j) bc[(kVec * cv + j) * 2 * N + r] = v[j];
      }
    }
    __syncthreads();
    // the state entering the chunk
    float2 h0[NQ];
    {
      const float* sp = snaps + c * p.N;
      const float4 s0 = *reinterpret_cast<const float4*>(sp), s1 = *reinterpret_cast<const float4*>(sp + 4);
      h0[0] = make_float2(s0.x, s0.y); h0[1] = make_float2(s0.z, s0.w);
      h0[2] = make_float2(s1.x, s1.y); h0[3] = make_float2(s1.z, s1.w);
    }
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
        load_items<IO, G>(u_row, t0, p.L, p.vec_ok, u_c);
        load_items<float, G>(dt_row, t0, p.L, p.vec_ok, dt_c);
        if constexpr (kStep) {
#pragma unroll
          for (int j = 0; j < G; ++j) dt_c[j] = (t0 + j < p.L) ? step_transform(dt_c[j], dbias, p.delta_softplus != 0) : 0.0f;
        }
#pragma unroll
        for (int j = 0; j < G; ++j) {
          float2 Bp[NQ], Cp[NQ];
          load_bc8(bc + (size_t)(w * G + j) * 2 * N + sub * kSplitStates, Bp, Cp);
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
      load_items<IO, G>(u_row, t0, p.L, p.vec_ok, u_c);
      load_items<float, G>(dt_row, t0, p.L, p.vec_ok, dt_c);
      if constexpr (kStep) {
#pragma unroll
        for (int j = 0; j < G; ++j) dt_c[j] = (t0 + j < p.L) ? step_transform(dt_c[j], dbias, p.delta_softplus != 0) : 0.0f;
      }
      if (z_row) load_items<IO, G>(z_row, t0, p.L, p.vec_ok, z_c);
      load_items<IO, G>(go_row, t0, p.L, p.vec_ok, go_c);
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
      const IO* steps = bc + (size_t)(w * G) * 2 * N + sub * kSplitStates;
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
      if (z_row) {
        for (int m = 1; m < S; m <<= 1) {          // eight independent exchanges per round
#pragma unroll
          for (int j = 0; j < G; ++j) yv[j] += __shfl_xor_sync(0xffffffffu, yv[j], m);
        }
#pragma unroll
        for (int j = 0; j < G; ++j) yv[j] = fmaf(dskip, u_c[j], yv[j]);
      }
      // adjoint, right to left
      float du_v[G], ddt_v[G], dz_v[G], gyd_v[G];
#pragma unroll
      for (int j = G - 1; j >= 0; --j) {
        float2 Bp[NQ], Cp[NQ];
        load_bc8(steps + (size_t)j * 2 * N, Bp, Cp);
        float gy = go_c[j];
        dz_v[j] = 0.0f;
        if (z_row) {
          const float zv = z_c[j];
          const float sg = __fdividef(1.0f, 1.0f + ex2(-zv * kLog2e));
          gy = go_c[j] * zv * sg;
          dz_v[j] = go_c[j] * yv[j] * (sg * fmaf(zv, 1.0f - sg, 1.0f));
        }
        const float2 gy2 = splat(gy), dtv = splat(dt_c[j]), dtu = splat(dt_c[j] * u_c[j]);
        float2 gb = make_float2(0.f, 0.f), dd = make_float2(0.f, 0.f);
        float* pp = part + (size_t)((warp * 4 + (j & 3)) * 16) * 32 + lane;   // [warp][step of the half][value][lane]
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
        gyd_v[j] = gy * dskip;
        dDacc = fmaf(gy, u_c[j], dDacc);
        if ((j & 3) == 0) {         // a half window is complete in every warp's slice
          __syncthreads();
          flush_half(j >> 2, t0);
          __syncthreads();
        }
      }
      for (int m = 1; m < S; m <<= 1) {            // sixteen independent exchanges per round
#pragma unroll
        for (int j = 0; j < G; ++j) {
          du_v[j] += __shfl_xor_sync(0xffffffffu, du_v[j], m);
          ddt_v[j] += __shfl_xor_sync(0xffffffffu, ddt_v[j], m);
        }
      }
#pragma unroll
      for (int j = 0; j < G; ++j) {
        const float sgb = du_v[j];
        const float sdd = ddt_v[j];
        du_v[j] = fmaf(dt_c[j], sgb, gyd_v[j]);
        ddt_v[j] = fmaf(u_c[j], sgb, sdd);
        if constexpr (kStep) {     // gradient with respect to the raw step
          ddt_v[j] = (t0 + j < p.L) ? ddt_v[j] * step_transform_grad(dt_c[j], p.delta_softplus != 0) : 0.0f;
          dBiasAcc += ddt_v[j];
        }
      }
      if (sub == 0 && active) {
        store_items<IO, G>(static_cast<IO*>(p.du) + row, t0, p.L, p.vec_ok, du_v);
        store_items<float, G>(p.ddt + row, t0, p.L, p.vec_ok, ddt_v);
        if (z_row) store_items<IO, G>(static_cast<IO*>(p.dz) + row, t0, p.L, p.vec_ok, dz_v);
      }
    }
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
  const size_t smem = (size_t)kSplitChunk * 2 * p.N * sizeof(IO) + (size_t)kSplitBwdWarps * 4 * 16 * 32 * sizeof(float) +
                      (size_t)(kSplitWindows - 1) * kSplitStates * kSplitBwdThreads * sizeof(float);
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

template <typename IO>
static int launch_bwd_split(const Params& p, cudaStream_t stream) {
  return p.N >= g_split_bwd_wide_from ? launch_bwd_split_w<IO, 8>(p, stream) : launch_bwd_split_w<IO, 4>(p, stream);
}
