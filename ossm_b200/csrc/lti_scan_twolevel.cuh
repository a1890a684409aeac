// Two-level variants of the oscillator scan kernels for long sequences of FEW series
// (included by lti_scan.cu inside namespace ossm_b200::lti).
//
// With N = B*P series the one-lane-per-series kernels expose N/128 CTAs; a shard such as
// B = 8, P = 256 (2048 series, L = 131072) would fill 16 of 148 SMs.  Here a CTA owns only
// kTlCols = 16 adjacent series, stages a tile of kTlRows = 256 time steps of them in shared
// memory (one TMA box of 256 rows x 128 B) and its 128 threads split the tile in time: thread
// (col, sub) owns the kChunk = 32 steps of sub-chunk `sub` of series `col`.
//
//   pass 1   every thread scans its sub-chunk from a ZERO state and publishes the end state e_sub
//   combine  entry states by the inter-chunk prefix  c_{j+1} = T c_j + e_j,  T = M^32 per channel,
//            evaluated by every thread in double precision (the chain across sub-chunks and
//            tiles therefore carries no float32 rounding of its own)
//   pass 2   every thread re-scans the SAME shared-memory rows from its true entry state and
//            stores x (and / or the full states); the state after each sub-chunk is also the
//            carry the backward needs
//
// so the data crosses HBM once in each direction (16 B/elem forward, 24 B/elem backward), as in
// the wide kernels, with 8x the CTAs.  The backward does the same with the adjoint recurrence
// running right to left: pass A = adjoint summary of the sub-chunk from zero, combine with
// (M^T)^32, then the state recompute from the saved carry and the full adjoint sweep.
//
// The reference runs one thread per series for any shape (dlinoss_imex1_cuda.cu:189-197).

constexpr int kTlCols = 16;                       // series per CTA
constexpr int kTlSub = 8;                         // sub-chunks per tile
constexpr int kTlThreads = kTlCols * kTlSub;      // 128
constexpr int kTlRows = kTlSub * kChunk;          // 256 time steps per tile
constexpr int kTlTileBytes = kTlRows * kTlCols * 8;   // 32 KiB

// 2x2 real transition of one step in plain matrix form, and its kChunk-th power (double).
struct Mat2d {
  double m11, m12, m21, m22;
};

template <int V>
__device__ __forceinline__ Mat2d step_matrix(const Coef& c) {
  Mat2d m;
  m.m11 = c.m11.x; m.m12 = c.m12.x;
  if constexpr (V == kImex1) { m.m21 = m.m11; m.m22 = 1.0 + m.m12; }   // x' = w' + x
  else { m.m21 = c.m21.x; m.m22 = c.m22.x; }
  return m;
}

__device__ __forceinline__ Mat2d chunk_power(Mat2d b) {
  // kChunk = 32 = 2^5
#pragma unroll
  for (int i = 0; i < 5; ++i) {
    Mat2d q;
    q.m11 = b.m11 * b.m11 + b.m12 * b.m21;
    q.m12 = b.m11 * b.m12 + b.m12 * b.m22;
    q.m21 = b.m21 * b.m11 + b.m22 * b.m21;
    q.m22 = b.m21 * b.m12 + b.m22 * b.m22;
    b = q;
  }
  return b;
}

// State / adjoint pair in double: (v0.re, v0.im, v1.re, v1.im).
struct Vec2c {
  double r0, i0, r1, i1;
};

__device__ __forceinline__ Vec2c affine(const Mat2d& t, const Vec2c& v, const float4& e) {
  Vec2c n;
  n.r0 = t.m11 * v.r0 + t.m12 * v.r1 + (double)e.x;
  n.i0 = t.m11 * v.i0 + t.m12 * v.i1 + (double)e.y;
  n.r1 = t.m21 * v.r0 + t.m22 * v.r1 + (double)e.z;
  n.i1 = t.m21 * v.i0 + t.m22 * v.i1 + (double)e.w;
  return n;
}

// Shared memory: barriers (1 KiB) | ebuf float4[kTlSub][kTlCols] (2 KiB) | ring of stages.
template <int V, int kOut>
__global__ void __launch_bounds__(kTlThreads)
lti_forward_twolevel_kernel(const __grid_constant__ CUtensorMap tm_bu, FwdParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw);
  float4* ebuf = reinterpret_cast<float4*>(smem_raw + 1024);
  unsigned char* ring_base = smem_raw + 4096;
  const int col = threadIdx.x % kTlCols, sub = threadIdx.x / kTlCols;
  const long long cta_col0 = (long long)blockIdx.x * kTlCols;
  const long long n = cta_col0 + col;
  const bool valid = n < p.N;
  const long long ch = valid ? (n % p.P) : 0;
  const Coef c = make_coef<V>(p.a[ch], p.g ? p.g[ch] : 0.0f, p.step ? p.step[ch] : 0.0f);
  const Mat2d T = chunk_power(step_matrix<V>(c));
  const long long nchunks = (p.L + kChunk - 1) / kChunk;
  const long long ntiles = (p.L + kTlRows - 1) / kTlRows;

  if (threadIdx.x == 0) {
    prefetch_tensormap(&tm_bu);
    for (int s = 0; s < p.ring; ++s) mbar_init(&bars[s], 1);
    fence_barrier_init();
    fence_proxy_async();
    const int pre = (int)(ntiles < p.ring ? ntiles : p.ring);
    for (int s = 0; s < pre; ++s) {
      mbar_expect_tx(&bars[s], kTlTileBytes);
      tma_load_2d(ring_base + (size_t)s * kTlTileBytes, &tm_bu, &bars[s], (int32_t)(cta_col0 * 2),
                  (int32_t)(s * kTlRows));
    }
  }
  __syncthreads();

  Vec2c carry = {0.0, 0.0, 0.0, 0.0};     // state entering the tile (same in every thread of a column)
  int slot = 0;
  uint32_t parity = 0;
  for (long long tile = 0; tile < ntiles; ++tile) {
    if (!mbar_wait(&bars[slot], parity)) return;
    const float2* rows = reinterpret_cast<const float2*>(ring_base + (size_t)slot * kTlTileBytes) +
                         (size_t)sub * kChunk * kTlCols + col;
    // pass 1: end state of the sub-chunk from zero (rows past the end of the sequence hold zeros)
    float2 s0 = make_float2(0.f, 0.f), s1 = make_float2(0.f, 0.f);
#pragma unroll
    for (int r = 0; r < kChunk; ++r) fwd_step<V>(c, s0, s1, rows[r * kTlCols]);
    ebuf[sub * kTlCols + col] = make_float4(s0.x, s0.y, s1.x, s1.y);
    __syncthreads();
    // inter-chunk prefix in double; every thread walks all sub-chunks, so all leave with the tile's exit state
    Vec2c cur = carry, mine = carry;
#pragma unroll
    for (int j = 0; j < kTlSub; ++j) {
      if (j == sub) mine = cur;
      cur = affine(T, cur, ebuf[j * kTlCols + col]);
    }
    carry = cur;
    // pass 2: the same rows again, now from the true entry state
    s0 = make_float2((float)mine.r0, (float)mine.i0);
    s1 = make_float2((float)mine.r1, (float)mine.i1);
    const long long k = tile * kTlSub + sub;            // chunk index of this sub-chunk
    const long long t0 = k * kChunk;
    float2* xp = (kOut & 1) ? p.x + t0 * p.N + n : nullptr;
    float4* sp = (kOut & 2) ? p.states + t0 * p.N + n : nullptr;
    if (t0 + kChunk <= p.L) {
#pragma unroll
      for (int r = 0; r < kChunk; ++r) {
        fwd_step<V>(c, s0, s1, rows[r * kTlCols]);
        if (valid) {
          if constexpr (kOut & 1) st_cs_f2(xp, s1);
          if constexpr (kOut & 2) st_cs_f4(sp, make_float4(s0.x, s0.y, s1.x, s1.y));
        }
        if constexpr (kOut & 1) xp += p.N;
        if constexpr (kOut & 2) sp += p.N;
      }
      if (p.carries && valid && k + 1 < nchunks) p.carries[k * p.N + n] = make_float4(s0.x, s0.y, s1.x, s1.y);
    } else if (t0 < p.L) {
      const int rows_left = (int)(p.L - t0);
      for (int r = 0; r < rows_left; ++r) {
        fwd_step<V>(c, s0, s1, rows[r * kTlCols]);
        if (valid) {
          if constexpr (kOut & 1) st_cs_f2(xp, s1);
          if constexpr (kOut & 2) st_cs_f4(sp, make_float4(s0.x, s0.y, s1.x, s1.y));
        }
        if constexpr (kOut & 1) xp += p.N;
        if constexpr (kOut & 2) sp += p.N;
      }
    }
    __syncthreads();   // every thread is done with this stage and with ebuf
    if (threadIdx.x == 0 && tile + p.ring < ntiles) {
      fence_proxy_async();
      mbar_expect_tx(&bars[slot], kTlTileBytes);
      tma_load_2d(ring_base + (size_t)slot * kTlTileBytes, &tm_bu, &bars[slot], (int32_t)(cta_col0 * 2),
                  (int32_t)((tile + p.ring) * kTlRows));
    }
    if (++slot == p.ring) { slot = 0; parity ^= 1; }
  }
}

// Backward.  Stage = bu tile followed by grad_x tile (64 KiB).  Per-thread partial sums go to
// partials[i][sub][n]: the sub-chunk positions of a series are summed like extra batch entries.
template <int V>
__global__ void __launch_bounds__(kTlThreads, 1)
lti_backward_twolevel_kernel(const __grid_constant__ CUtensorMap tm_bu, const __grid_constant__ CUtensorMap tm_gx,
                             BwdParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw);
  float4* rbuf = reinterpret_cast<float4*>(smem_raw + 1024);
  unsigned char* ring_base = smem_raw + 4096;
  constexpr uint32_t kPair = 2 * kTlTileBytes;
  const int col = threadIdx.x % kTlCols, sub = threadIdx.x / kTlCols;
  const long long cta_col0 = (long long)blockIdx.x * kTlCols;
  const long long n = cta_col0 + col;
  const bool valid = n < p.N;
  const long long ch = valid ? (n % p.P) : 0;
  const Coef c = make_coef<V>(p.a[ch], p.g ? p.g[ch] : 0.0f, p.step ? p.step[ch] : 0.0f);
  Mat2d Tt = chunk_power(step_matrix<V>(c));
  { const double t = Tt.m12; Tt.m12 = Tt.m21; Tt.m21 = t; }     // adjoint: (M^T)^32
  const long long ntiles = (p.L + kTlRows - 1) / kTlRows;

  if (threadIdx.x == 0) {
    prefetch_tensormap(&tm_bu);
    prefetch_tensormap(&tm_gx);
    for (int s = 0; s < p.ring; ++s) mbar_init(&bars[s], 1);
    fence_barrier_init();
    fence_proxy_async();
    const int pre = (int)(ntiles < p.ring ? ntiles : p.ring);
    for (int s = 0; s < pre; ++s) {
      const int32_t row = (int32_t)((ntiles - 1 - s) * kTlRows);
      unsigned char* dst = ring_base + (size_t)s * kPair;
      mbar_expect_tx(&bars[s], kPair);
      tma_load_2d(dst, &tm_bu, &bars[s], (int32_t)(cta_col0 * 2), row);
      tma_load_2d(dst + kTlTileBytes, &tm_gx, &bars[s], (int32_t)(cta_col0 * 2), row);
    }
  }
  __syncthreads();

  float acc[kNumAcc], comp[kNumAcc];
#pragma unroll
  for (int i = 0; i < kNumAcc; ++i) { acc[i] = 0.f; comp[i] = 0.f; }
  Vec2c lam_carry = {0.0, 0.0, 0.0, 0.0};   // adjoint entering the tile from the right
  int slot = 0;
  uint32_t parity = 0;
  for (long long it = 0; it < ntiles; ++it) {
    const long long tile = ntiles - 1 - it;
    const long long k = tile * kTlSub + sub;              // chunk index of this sub-chunk
    const long long t0 = k * kChunk;
    // state entering the sub-chunk, saved by the forward (issued early, used after the combine)
    float4 carry = make_float4(0.f, 0.f, 0.f, 0.f);
    if (k > 0 && valid && t0 < p.L) carry = ld_nc_f4(p.carry_src + (k * p.carry_mul + p.carry_off) * p.N + n);
    if (!mbar_wait(&bars[slot], parity)) return;
    const float2* sbu = reinterpret_cast<const float2*>(ring_base + (size_t)slot * kPair) +
                        (size_t)sub * kChunk * kTlCols + col;
    const float2* sgx = reinterpret_cast<const float2*>(ring_base + (size_t)slot * kPair + kTlTileBytes) +
                        (size_t)sub * kChunk * kTlCols + col;
    // pass A: adjoint summary of the sub-chunk from zero (zero rows past the end leave zero unchanged)
    float2 l0 = make_float2(0.f, 0.f), l1 = make_float2(0.f, 0.f);
#pragma unroll
    for (int r = kChunk - 1; r >= 0; --r) {
      const float2 g1 = __fadd2_rn(l1, sgx[r * kTlCols]);
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
    rbuf[sub * kTlCols + col] = make_float4(l0.x, l0.y, l1.x, l1.y);
    __syncthreads();
    Vec2c cur = lam_carry, mine = lam_carry;
#pragma unroll
    for (int j = kTlSub - 1; j >= 0; --j) {
      if (j == sub) mine = cur;
      cur = affine(Tt, cur, rbuf[j * kTlCols + col]);
    }
    lam_carry = cur;
    l0 = make_float2((float)mine.r0, (float)mine.i0);
    l1 = make_float2((float)mine.r1, (float)mine.i1);

    // state recompute of the sub-chunk, remembering the state before each step
    float2 p0[kChunk], p1[kChunk];
    float2 s0 = make_float2(carry.x, carry.y), s1 = make_float2(carry.z, carry.w);
#pragma unroll
    for (int r = 0; r < kChunk; ++r) {
      p0[r] = s0; p1[r] = s1;
      fwd_step<V>(c, s0, s1, sbu[r * kTlCols]);
    }
    float2 loc[kNumAcc];
#pragma unroll
    for (int i = 0; i < kNumAcc; ++i) loc[i] = make_float2(0.f, 0.f);
    float2* gbp = p.grad_bu + (t0 + kChunk - 1) * p.N + n;   // walks backwards
    const int rows = (p.L - t0) >= kChunk ? kChunk : (p.L > t0 ? (int)(p.L - t0) : 0);
    if (rows == kChunk) {
#pragma unroll
      for (int r = kChunk - 1; r >= 0; --r) {
        const float2 gb = bwd_step<V>(c, l0, l1, sgx[r * kTlCols], p0[r], p1[r], sbu[r * kTlCols], loc);
        if (valid) st_cs_f2(gbp, gb);
        gbp -= p.N;
      }
    } else {
#pragma unroll
      for (int r = kChunk - 1; r >= 0; --r) {
        if (r < rows) {
          const float2 gb = bwd_step<V>(c, l0, l1, sgx[r * kTlCols], p0[r], p1[r], sbu[r * kTlCols], loc);
          if (valid) st_cs_f2(gbp, gb);
        }
        gbp -= p.N;
      }
    }
#pragma unroll
    for (int i = 0; i < kNumAcc; ++i) kahan_add(acc[i], comp[i], loc[i].x + loc[i].y);

    __syncthreads();   // every thread is done with this stage and with rbuf
    if (threadIdx.x == 0 && it + p.ring < ntiles) {
      const int32_t row = (int32_t)((tile - p.ring) * kTlRows);
      unsigned char* dst = ring_base + (size_t)slot * kPair;
      fence_proxy_async();
      mbar_expect_tx(&bars[slot], kPair);
      tma_load_2d(dst, &tm_bu, &bars[slot], (int32_t)(cta_col0 * 2), row);
      tma_load_2d(dst + kTlTileBytes, &tm_gx, &bars[slot], (int32_t)(cta_col0 * 2), row);
    }
    if (++slot == p.ring) { slot = 0; parity ^= 1; }
  }
  if (valid) {
    const long long SN = (long long)kTlSub * p.N;
#pragma unroll
    for (int i = 0; i < kNumAcc; ++i) p.partials[(long long)i * SN + (long long)sub * p.N + n] = acc[i];
  }
}
