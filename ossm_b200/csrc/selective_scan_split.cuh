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
#pragma unroll
      for (int j = 0; j < kVec; ++j) split_tile[(kVec * cv + j) * 2 * N + r] = v[j];
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
      const float* steps = split_tile + (size_t)(gi * G) * 2 * N + sub * kSplitStates;
#pragma unroll
      for (int j = 0; j < G; ++j) {
        const float4 b0 = *reinterpret_cast<const float4*>(steps + j * 2 * N);
        const float4 b1 = *reinterpret_cast<const float4*>(steps + j * 2 * N + 4);
        const float4 c0 = *reinterpret_cast<const float4*>(steps + j * 2 * N + N);
        const float4 c1 = *reinterpret_cast<const float4*>(steps + j * 2 * N + N + 4);
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
