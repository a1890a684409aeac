// Projections of the D-LinOSS layer on the 5th-generation tensor cores (tcgen05, sm_100a).
//
// The layer body (src/ossm/models/dlinoss.py:217-247) wraps the scan in two pairs of real GEMMs,
//     bu = u B_re^T + i u B_im^T            (prologue)      y = Re(C x) + D u       (epilogue)
// plus permutes between the batch-major activations [B, L, H] and the time-major scan operands
// [L, B, P] complex64.  Both are instances of
//     out[dest(m), n] = sum_k A[m, k] * W[n, k]  (+ diag[n] * aux[dest(m), n])
// with A an activation matrix (rows = (b, l) or (l, b) pairs, K contiguous), W a small weight
// matrix (K contiguous) and dest(m) the row permutation between the two orders, so the permute
// copies and the real / imaginary split of the reference disappear into the GEMM's addressing:
//   prologue   A = u [B*L, H],    W = (B_re | B_im) interleaved [2P, H],  out = bu viewed [L*B, 2P]
//   epilogue   A = x [L*B, 2P],   W = (C_re | -C_im) interleaved [H, 2P], out = y [B*L, H], aux = u, diag = D
// and their transposes in the backward pass (grad_x from grad_y, grad_u from grad_bu).
//
// Accuracy: the parity bound of the layer is 1e-5, which plain TF32 (10-bit mantissa) misses by two
// orders of magnitude.  Every float32 operand is therefore split into two TF32 numbers,
//     v = hi + lo,   hi = v with the 13 low mantissa bits cleared,   lo = v - hi  (exact),
// and the product is accumulated as  hi*hi + hi*lo + lo*hi  in the float32 accumulator (the dropped
// lo*lo term is below 2^-22 relative).  The weights are split once by split_tf32_kernel; the
// activations are split inside the GEMM by four "splitter" warps between the TMA load and the MMA.
//
// Kernel structure (persistent CTAs, one per SM, each walking 128 x BN output tiles; K in slices of 16 floats = 64 B
// through a ring of 4 stages that runs on across tiles; two accumulators alternate in tensor memory):
//   warp 0       producer: one lane issues the TMA loads (SWIZZLE_64B) of A, W_hi, W_lo per slice
//   warp 1       allocates tensor memory; one lane issues 6 tcgen05.mma per slice (2 K-steps of 8 x 3 operand
//                combinations), commits the stage back to the producer and, per tile, the accumulator to the epilogue
//   warps 2..5   splitters: rewrite the A slice in place as hi and write lo beside it
//   warps 6..9   epilogue: tcgen05.ld the finished accumulator (lane = output row), add diag*aux, store, hand the
//                accumulator back -- while the other warps already work on the next tile
// Stages are handed over with mbarriers; every wait is bounded in time and a wait that gives up sets
// the device status word and lets the CTA run to its normal end (tensor memory is always released).
// No cluster launch and no multicast: the same kernel runs unchanged under several ranks per node.
#include "common.cuh"

#include "../../include/ossm_b200.h"

namespace ossm_b200 {
OSSM_B200_STATUS_ACCESSOR(status_layer)
namespace layer {

constexpr int kBM = 128;            // output rows per CTA = TMEM lanes
constexpr int kBK = 16;             // weight-gradient kernel: K rows (time steps) per slice; a four-deep ring fits
constexpr int kPK = 16;             // projection kernel: floats per K slice = one 64-byte swizzle row; the smaller
                                    // slice buys a four-deep ring (TMA -> split -> MMA needs the depth, the MMAs of
                                    // one slice take less time than its load and split)
constexpr int kThreads = 320;       // producer warp, MMA warp, four splitter warps, four epilogue warps
constexpr int kATile = kBM * kPK * 4;   // 8 KiB

enum RowMap : int { kRowIdentity = 0, kRowBatchToTime = 1, kRowTimeToBatch = 2 };

// SMs the persistent kernels leave free (a caller that runs a collective beside them sets this: a CTA of these
// kernels fills an SM's shared memory, so a library kernel launched meanwhile would otherwise wait for the whole grid).
static int g_reserve_sms = 0;
static int sm_budget() {
  const int n = sm_count() - g_reserve_sms;
  return n < 1 ? 1 : n;
}

struct GemmParams {
  float* out;            // [rows_out, ldo]
  const float* aux;      // nullable, same indexing as out
  const float* diag;     // nullable, [N]
  long long M, N, K;
  long long ldo;         // floats between output rows
  long long col_block;   // output columns per plane (N when the output is one matrix)
  long long plane_stride;  // floats between planes: column n goes to plane n / col_block, column n % col_block
  long long batch, length;   // for the row maps: M = batch * length
  int row_map;
  int stages;
  long long tiles_m, tiles_n;   // output tiles of 128 x BN
};

__device__ __forceinline__ long long dest_row(const GemmParams& p, long long m) {
  if (p.row_map == kRowBatchToTime) {           // m = b * L + l  ->  l * B + b
    const long long b = m / p.length, l = m - b * p.length;
    return l * p.batch + b;
  }
  if (p.row_map == kRowTimeToBatch) {           // m = l * B + b  ->  b * L + l
    const long long l = m / p.batch, b = m - l * p.batch;
    return b * p.length + l;
  }
  return m;
}

// ---- tcgen05 wrappers ------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem]^T, TF32 inputs, float32 accumulate, issued by one thread.
__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on `bar` once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
// 32 consecutive accumulator columns of this thread's lane.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 64 bytes (16 floats), stored with the
// 64-byte swizzle (what TMA writes with CU_TENSOR_MAP_SWIZZLE_64B): groups of 8 rows are 512 B apart
// (stride byte offset), the leading byte offset is unused for this layout (1), descriptor version 1
// (sm_100), layout type 4 = SWIZZLE_64B.  `addr` must lie in a 512-byte aligned tile; advancing it by
// 32 B selects the next K step of 8 TF32 values inside the swizzle row.
__device__ __forceinline__ uint64_t smem_desc_k_sw64(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3ffffu) >> 4);          // start address, bits [0,14)
  d |= (uint64_t)1 << 16;                           // leading byte offset (16-byte units), bits [16,30)
  d |= (uint64_t)(512 >> 4) << 32;                  // stride byte offset, bits [32,46)
  d |= (uint64_t)1 << 46;                           // descriptor version, bits [46,48)
  d |= (uint64_t)4 << 61;                           // layout type, bits [61,64)
  return d;
}

// Instruction descriptor: float32 accumulator (bits [4,6) = 1), TF32 A and B (bits [7,10), [10,13) = 2),
// both operands K-major (bits 15, 16 = 0), N >> 3 in bits [17,23), M >> 4 in bits [24,29).
__host__ __device__ constexpr uint32_t instr_desc_tf32(int m, int n) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

constexpr int kTurnPitch = 36;      // floats per row of an epilogue turn buffer: 16-byte accesses of 8 lanes hit 32 banks

// Shared memory: [0,1024) barriers + TMEM address | stages x (A_hi 8K | A_lo 8K | W_hi BN*64 | W_lo BN*64)
template <int BN>
struct Smem {
  static constexpr int kWTile = BN * kPK * 4;
  static constexpr int kStage = 2 * kATile + 2 * kWTile;
  // barriers | stages | four epilogue turn buffers | alignment slack
  static constexpr size_t bytes(int stages) { return 1024 + (size_t)stages * kStage + 4 * 32 * kTurnPitch * 4 + 1024; }
};

constexpr int kMaxStages = 6;

// Persistent CTA (one per SM): output tiles blockIdx.x, blockIdx.x + gridDim.x, ... in an order that puts the
// column blocks of one row block on neighbouring SMs at the same time (the second reads its activations from L2).
// The ring of K slices runs on across tile boundaries, and two accumulators alternate in tensor memory, so the
// loads and MMAs of tile i+1 overlap the epilogue of tile i.
template <int BN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tf32x3_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_whi,
                   const __grid_constant__ CUtensorMap tm_wlo, GemmParams p) {
  extern __shared__ unsigned char smem_dyn[];
  // swizzled tiles need 1024-byte alignment
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem);            // [stages] TMA landed
  uint64_t* split = full + kMaxStages;                           // [stages] A split into hi / lo
  uint64_t* empty = split + kMaxStages;                          // [stages] MMAs of the stage finished
  uint64_t* acc_full = empty + kMaxStages;                       // [2] accumulator complete
  uint64_t* acc_empty = acc_full + 2;                            // [2] accumulator read out by the epilogue
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  unsigned char* stage0 = smem + 1024;
  using S = Smem<BN>;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nslices = (int)((p.K + kPK - 1) / kPK);
  const int stages = p.stages;
  const long long ntiles = p.tiles_m * p.tiles_n;

  if (threadIdx.x == 0) {
    prefetch_tensormap(&tm_a);
    prefetch_tensormap(&tm_whi);
    prefetch_tensormap(&tm_wlo);
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&split[s], 128);
      mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], 128);
    }
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 1) tmem_alloc(tmem_slot, 2 * BN);   // two accumulators of BN float32 columns x 128 lanes
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---- producer
    if (lane == 0) {
      long long g = 0;                              // slices issued so far, over all tiles of this CTA
      bool ok = true;
      for (long long tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
        const int32_t m0 = (int32_t)((tile / p.tiles_n) * kBM), n0 = (int32_t)((tile % p.tiles_n) * BN);
        for (int s = 0; s < nslices; ++s, ++g) {
          const int b = (int)(g % stages);
          if (g >= stages && !mbar_wait(&empty[b], (uint32_t)((g / stages) - 1) & 1u, kWaitLimitNs, kStatusMmaTimeout)) {
            ok = false;
            break;
          }
          unsigned char* st = stage0 + (size_t)b * S::kStage;
          mbar_expect_tx(&full[b], kATile + 2 * S::kWTile);
          tma_load_2d(st, &tm_a, &full[b], s * kPK, m0);
          tma_load_2d(st + 2 * kATile, &tm_whi, &full[b], s * kPK, n0);
          tma_load_2d(st + 2 * kATile + S::kWTile, &tm_wlo, &full[b], s * kPK, n0);
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = instr_desc_tf32(kBM, BN);
      long long g = 0, it = 0;
      bool ok = true;
      for (long long tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x, ++it) {
        const int buf = (int)(it & 1);
        if (it >= 2) ok = mbar_wait(&acc_empty[buf], (uint32_t)((it >> 1) - 1) & 1u);
        if (!ok) break;
        tc_fence_after();
        const uint32_t tmem_acc = tmem_base + (uint32_t)(buf * BN);
        for (int s = 0; s < nslices; ++s, ++g) {
          const int b = (int)(g % stages);
          const uint32_t ph = (uint32_t)(g / stages) & 1u;
          ok = mbar_wait(&full[b], ph) && mbar_wait(&split[b], ph);
          if (!ok) break;
          tc_fence_after();
          const uint32_t st = smem_u32(stage0 + (size_t)b * S::kStage);
          const uint32_t a_hi = st, a_lo = st + kATile, w_hi = st + 2 * kATile, w_lo = w_hi + S::kWTile;
#pragma unroll
          for (int k = 0; k < kPK / 8; ++k) {
            const uint32_t off = k * 32;     // 8 TF32 values = 32 bytes along the swizzle row
            umma_tf32(tmem_acc, smem_desc_k_sw64(a_hi + off), smem_desc_k_sw64(w_hi + off), idesc, (s | k) != 0);
            umma_tf32(tmem_acc, smem_desc_k_sw64(a_hi + off), smem_desc_k_sw64(w_lo + off), idesc, 1);
            umma_tf32(tmem_acc, smem_desc_k_sw64(a_lo + off), smem_desc_k_sw64(w_hi + off), idesc, 1);
          }
          umma_commit(&empty[b]);            // the stage may be refilled once these MMAs have read it
        }
        if (ok) umma_commit(&acc_full[buf]);  // everything issued so far: this tile's accumulator is final
      }
    }
  } else if (warp < 6) {
    // ---- splitters: hi in place, lo beside it (same swizzled positions, so the layout is irrelevant here)
    const int t = threadIdx.x - 64;        // 0..127
    long long g = 0;
    bool ok = true;
    for (long long tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
      for (int s = 0; s < nslices; ++s, ++g) {
        const int b = (int)(g % stages);
        ok = mbar_wait(&full[b], (uint32_t)(g / stages) & 1u);
        if (!ok) break;
        float4* hi = reinterpret_cast<float4*>(stage0 + (size_t)b * S::kStage);
        float4* lo = reinterpret_cast<float4*>(stage0 + (size_t)b * S::kStage + kATile);
#pragma unroll
        for (int i = 0; i < kATile / 16 / 128; ++i) {     // 4 vectors of 16 bytes per thread
          const float4 v = hi[i * 128 + t];
          float4 h, l;
          h.x = __uint_as_float(__float_as_uint(v.x) & 0xffffe000u); l.x = v.x - h.x;
          h.y = __uint_as_float(__float_as_uint(v.y) & 0xffffe000u); l.y = v.y - h.y;
          h.z = __uint_as_float(__float_as_uint(v.z) & 0xffffe000u); l.z = v.z - h.z;
          h.w = __uint_as_float(__float_as_uint(v.w) & 0xffffe000u); l.w = v.w - h.w;
          lo[i * 128 + t] = l;                 // hi stays as loaded: the tensor core ignores the 13 low bits
        }
        fence_proxy_async();                 // generic-proxy writes become visible to the tensor core
        mbar_arrive(&split[b]);
      }
    }
  } else {
    // ---- epilogue: lane quarter (warp % 4) of the accumulator, 32 columns at a time.  tcgen05.ld gives every
    // lane 32 consecutive columns of ITS row; stored like that, one instruction would touch 32 rows with 16 bytes
    // each.  The chunk is turned through a padded shared-memory buffer instead, so that eight lanes write one
    // 128-byte line of a row (and read aux the same way): four full lines per store instruction.
    const int q = warp & 3;
    const bool vec = ((p.ldo & 3) == 0) && ((p.plane_stride & 3) == 0) && ((p.col_block & 31) == 0) &&
                     ((reinterpret_cast<uintptr_t>(p.out) & 15u) == 0) &&
                     (!p.aux || (reinterpret_cast<uintptr_t>(p.aux) & 15u) == 0);
    float* turn = reinterpret_cast<float*>(stage0 + (size_t)stages * S::kStage) + q * (32 * kTurnPitch);
    const int sub = lane >> 3, col4 = (lane & 7) * 4;       // read-out: row 4*i + sub, columns col4 .. col4+3
    long long it = 0;
    for (long long tile = blockIdx.x; tile < ntiles; tile += gridDim.x, ++it) {
      const int buf = (int)(it & 1);
      if (!mbar_wait(&acc_full[buf], (uint32_t)(it >> 1) & 1u, kWaitLimitNs, kStatusMmaTimeout)) break;
      tc_fence_after();
      const long long m0 = (tile / p.tiles_n) * kBM, n0 = (tile % p.tiles_n) * BN;
      const uint32_t tmem_acc = tmem_base + (uint32_t)(buf * BN);
      const long long m = m0 + q * 32 + lane;
      const bool row_ok = m < p.M;
      const long long drow = row_ok ? dest_row(p, m) : -1;     // -1: row beyond M
      // destination rows of the eight rows this lane stores in the turned layout
      long long drow_t[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) drow_t[i] = __shfl_sync(0xffffffffu, drow, 4 * i + sub);
      // aux (the D*u term of the output projection) is fetched one chunk ahead: its latency would otherwise be paid
      // eight times per tile and make the epilogue, not the MMAs, the pace of the kernel
      float4 aux_next[8];
      auto fetch_aux = [&](long long n, float4 (&dst)[8]) {
        const bool in = p.aux && vec && n + 32 <= p.N;
        const long long off = in ? (n / p.col_block) * p.plane_stride + (n % p.col_block) + col4 : 0;
#pragma unroll
        for (int i = 0; i < 8; ++i)
          dst[i] = (in && drow_t[i] >= 0) ? __ldg(reinterpret_cast<const float4*>(p.aux + drow_t[i] * p.ldo + off))
                                          : make_float4(0.f, 0.f, 0.f, 0.f);
      };
      if (p.aux) fetch_aux(n0, aux_next);
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        float v[32];
        float4 aux_cur[8];
        if (p.aux) {
#pragma unroll
          for (int i = 0; i < 8; ++i) aux_cur[i] = aux_next[i];
          if (c0 + 32 < BN) fetch_aux(n0 + c0 + 32, aux_next);
        }
        __syncwarp();
        tmem_ld32(tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, v);   // whole warp takes part
        const long long n = n0 + c0;
        if (n >= p.N) continue;
        if (vec && n + 32 <= p.N) {
          // 32 columns of one plane (col_block is a multiple of 32 here)
          const long long off = (n / p.col_block) * p.plane_stride + (n % p.col_block) + col4;
#pragma unroll
          for (int j = 0; j < 32; j += 4)
            *reinterpret_cast<float4*>(turn + lane * kTurnPitch + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
          __syncwarp();
          float4 d = make_float4(0.f, 0.f, 0.f, 0.f);
          if (p.aux) d = *reinterpret_cast<const float4*>(p.diag + n + col4);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            float4 o = *reinterpret_cast<const float4*>(turn + (4 * i + sub) * kTurnPitch + col4);
            if (drow_t[i] < 0) continue;
            if (p.aux) {
              const float4 a = aux_cur[i];
              o.x = fmaf(d.x, a.x, o.x); o.y = fmaf(d.y, a.y, o.y); o.z = fmaf(d.z, a.z, o.z); o.w = fmaf(d.w, a.w, o.w);
            }
            *reinterpret_cast<float4*>(p.out + drow_t[i] * p.ldo + off) = o;
          }
        } else if (row_ok) {
          float* out_row = p.out + drow * p.ldo;
          const float* aux_row = p.aux ? p.aux + drow * p.ldo : nullptr;
          for (int j = 0; j < 32 && n + j < p.N; ++j) {
            const long long off = ((n + j) / p.col_block) * p.plane_stride + ((n + j) % p.col_block);
            float o = v[j];
            if (aux_row) o = fmaf(p.diag[n + j], aux_row[off], o);
            out_row[off] = o;
          }
        }
      }
      tc_fence_before();
      mbar_arrive(&acc_empty[buf]);          // this thread's reads of the accumulator are complete
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * BN);
  }
}

// ---------------------------------------------------------------------------------------------
// Weight gradients:  out[m, n] = sum over all (b, l) rows of  X[row_x(b,l), m] * Y[row_y(b,l), n]
// (grad_B from grad_bu and u, grad_C from grad_y and x: dlinoss.py:217-247 differentiated).  The
// contraction runs over the ROWS of both activation matrices, which may be stored in different row
// orders (batch-major b*L + l or time-major l*B + b): a K slice is 16 consecutive time steps of one
// batch entry, fetched from either order by a rank-4 tensor map (32 columns, time, column block, batch)
// whose box {32, 16, tile/32, 1} lands in shared memory as column blocks of [16 rows x 128 B] -- the
// canonical MN-major operand layout of the tensor core: leading byte offset = 2048 B between column
// blocks, K rows 128 B apart in groups of 4 (512 B, the stride byte offset).  For 32-bit operands in this
// orientation the hardware takes one swizzle only, 32-byte chunks within the 128-byte row
// (CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B on the TMA side, layout type 1 in the matrix descriptor).  Both operands are activations, so both are split into hi / lo
// halves by the splitter warps.  The M x N output is small and K = B*L is huge: the K slices are divided
// over gridDim.z CTAs per output tile, each writes its partial tile, and the caller sums the partials in a
// fixed order (deterministic, no atomics).
constexpr int kWgThreads = 64 + 256;      // producer warp, MMA warp, eight splitter warps (four of them also epilogue)

__device__ __forceinline__ uint64_t smem_desc_mn_sw128(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3ffffu) >> 4);          // start address
  d |= (uint64_t)((kBK * 128) >> 4) << 16;          // leading byte offset: next block of 32 M/N elements
  d |= (uint64_t)(512 >> 4) << 32;                  // stride byte offset: next group of 4 K rows
  d |= (uint64_t)1 << 46;                           // descriptor version
  d |= (uint64_t)1 << 61;                           // 128-byte swizzle span with 32-byte chunks
  return d;
}
// as instr_desc_tf32 with both operands MN-major (bits 15 and 16)
__host__ __device__ constexpr uint32_t instr_desc_tf32_mn(int m, int n) {
  return instr_desc_tf32(m, n) | (1u << 15) | (1u << 16);
}

struct WgradParams {
  float* partial;          // [splits, M, N]
  long long M, N;
  long long batch, length;
  int slices_per_batch;    // ceil(length / 32)
  int stages;
};

// MT = output row tiles of 128 per CTA (1 or 2): with two, the Y slice -- the wider operand -- is fetched and split once
// for twice the MMAs, and the two accumulators fill tensor memory (there is no epilogue to overlap: a CTA reads its
// accumulators out once, at the end of its K range).
template <int BN, int MT>
__global__ void __launch_bounds__(kWgThreads, 1)
wgrad_tf32x3_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_y, WgradParams p) {
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem);
  uint64_t* split = full + kMaxStages;
  uint64_t* empty = split + kMaxStages;
  uint64_t* acc_done = empty + kMaxStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_done + 1);
  unsigned char* stage0 = smem + 1024;
  constexpr int kXTile = MT * kBM * kBK * 4;   // 8 KiB per row tile: 4 column blocks of [16 rows][32 floats] each
  constexpr int kYTile = BN * kBK * 4;
  constexpr int kStage = 2 * kXTile + 2 * kYTile;   // X_hi | X_lo | Y_hi | Y_lo
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long m0 = (long long)blockIdx.x * (MT * kBM);
  const long long n0 = (long long)blockIdx.y * BN;
  const long long total = p.batch * p.slices_per_batch;
  const long long per = (total + gridDim.z - 1) / gridDim.z;
  const long long s_begin = (long long)blockIdx.z * per;
  const long long s_end = s_begin + per < total ? s_begin + per : total;
  const int nslices = s_end > s_begin ? (int)(s_end - s_begin) : 0;
  const int stages = p.stages;

  if (threadIdx.x == 0) {
    prefetch_tensormap(&tm_x);
    prefetch_tensormap(&tm_y);
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&split[s], 256);
      mbar_init(&empty[s], 1);
    }
    mbar_init(acc_done, 1);
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 1) tmem_alloc(tmem_slot, MT * BN);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_acc = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      for (int s = 0; s < nslices; ++s) {
        const int b = s % stages;
        if (s >= stages && !mbar_wait(&empty[b], ((s / stages) - 1) & 1, kWaitLimitNs, kStatusMmaTimeout)) break;
        const long long g = s_begin + s;
        const int bi = (int)(g / p.slices_per_batch);
        const int l0 = (int)(g - (long long)bi * p.slices_per_batch) * kBK;
        unsigned char* st = stage0 + (size_t)b * kStage;
        mbar_expect_tx(&full[b], kXTile + kYTile);
        tma_load_4d(st, &tm_x, &full[b], 0, l0, (int32_t)(m0 / 32), bi);
        tma_load_4d(st + 2 * kXTile, &tm_y, &full[b], 0, l0, (int32_t)(n0 / 32), bi);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = instr_desc_tf32_mn(kBM, BN);
      for (int s = 0; s < nslices; ++s) {
        const int b = s % stages;
        const uint32_t ph = (s / stages) & 1;
        if (!(mbar_wait(&full[b], ph) && mbar_wait(&split[b], ph))) break;
        tc_fence_after();
        const uint32_t st = smem_u32(stage0 + (size_t)b * kStage);
        const uint32_t x_hi = st, x_lo = st + kXTile, y_hi = st + 2 * kXTile, y_lo = y_hi + kYTile;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          const uint32_t xo = mt * (kBM * kBK * 4);     // the row tile's four column blocks
          const uint32_t acc = tmem_acc + (uint32_t)(mt * BN);
#pragma unroll
          for (int k = 0; k < kBK / 8; ++k) {
            const uint32_t off = k * 1024;     // 8 K rows = two swizzle groups inside every column block
            umma_tf32(acc, smem_desc_mn_sw128(x_hi + xo + off), smem_desc_mn_sw128(y_hi + off), idesc, (s | k) != 0);
            umma_tf32(acc, smem_desc_mn_sw128(x_hi + xo + off), smem_desc_mn_sw128(y_lo + off), idesc, 1);
            umma_tf32(acc, smem_desc_mn_sw128(x_lo + xo + off), smem_desc_mn_sw128(y_hi + off), idesc, 1);
          }
        }
        umma_commit(&empty[b]);
      }
      umma_commit(acc_done);
    }
  } else {
    const int t = threadIdx.x - 64;        // 0..255
    bool ok = true;
    for (int s = 0; s < nslices; ++s) {
      const int b = s % stages;
      ok = mbar_wait(&full[b], (s / stages) & 1);
      if (!ok) break;
      unsigned char* st = stage0 + (size_t)b * kStage;
      auto split_tile = [&](float4* hi, float4* lo, int vecs) {
        for (int i = t; i < vecs; i += 256) {
          const float4 v = hi[i];
          float4 h, l;
          h.x = __uint_as_float(__float_as_uint(v.x) & 0xffffe000u); l.x = v.x - h.x;
          h.y = __uint_as_float(__float_as_uint(v.y) & 0xffffe000u); l.y = v.y - h.y;
          h.z = __uint_as_float(__float_as_uint(v.z) & 0xffffe000u); l.z = v.z - h.z;
          h.w = __uint_as_float(__float_as_uint(v.w) & 0xffffe000u); l.w = v.w - h.w;
          lo[i] = l;                           // hi stays as loaded: the tensor core ignores the 13 low bits
        }
      };
      split_tile(reinterpret_cast<float4*>(st), reinterpret_cast<float4*>(st + kXTile), kXTile / 16);
      split_tile(reinterpret_cast<float4*>(st + 2 * kXTile), reinterpret_cast<float4*>(st + 2 * kXTile + kYTile), kYTile / 16);
      fence_proxy_async();
      mbar_arrive(&split[b]);
    }
    if (warp < 6) {    // warps 2..5: one accumulator lane quarter each
      if (ok && nslices > 0) ok = mbar_wait(acc_done, 0, kWaitLimitNs, kStatusMmaTimeout);
      if (ok) {
        tc_fence_after();
        const int q = warp & 3;
#pragma unroll 1
        for (int mt = 0; mt < MT; ++mt) {
        const long long m = m0 + mt * kBM + q * 32 + lane;
        float* row = p.partial + ((long long)blockIdx.z * p.M + (m < p.M ? m : 0)) * p.N;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          float v[32];
          __syncwarp();
          if (nslices > 0) {
            tmem_ld32(tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)(mt * BN + c0), v);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = 0.0f;      // a split without slices contributes zeros
          }
          const long long n = n0 + c0;
          if (m >= p.M || n >= p.N) continue;
          if (n + 32 <= p.N && (p.N & 3) == 0) {
#pragma unroll
            for (int j = 0; j < 32; j += 4)
              *reinterpret_cast<float4*>(row + n + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
          } else {
            for (int j = 0; j < 32 && n + j < p.N; ++j) row[n + j] = v[j];
          }
        }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_acc, MT * BN);
  }
}

// hi / lo TF32 split of a weight matrix (done once per call of the layer, a few hundred KB).
__global__ void split_tf32_kernel(const float* __restrict__ w, float* __restrict__ hi, float* __restrict__ lo,
                                  long long n) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float v = w[i];
  const float h = __uint_as_float(__float_as_uint(v) & 0xffffe000u);
  hi[i] = h;
  lo[i] = v - h;
}


// grad_D[n] = sum over rows of X[m, n] * Y[m, n] (dlinoss.py:247 differentiated: y = ... + u * D).  Both matrices are
// read once with 16-byte loads; a CTA covers a row range and writes one partial row, which the caller adds up in a
// fixed order.  HBM-bound: 8 B per element.
constexpr int kDotThreads = 256;
__global__ void __launch_bounds__(kDotThreads)
colwise_dot_kernel(const float* __restrict__ X, const float* __restrict__ Y, float* __restrict__ partial,
                   long long rows, long long cols, long long rows_per_cta) {
  __shared__ float4 red[kDotThreads];
  const int vec_cols = (int)(cols >> 2);                    // float4 columns (cols is a multiple of 4)
  const int lanes_c = vec_cols < kDotThreads ? vec_cols : kDotThreads;   // threads along the columns
  const int lanes_r = kDotThreads / lanes_c;                // rows in flight per pass
  const int tc = threadIdx.x % lanes_c, tr = threadIdx.x / lanes_c;
  const long long r0 = (long long)blockIdx.x * rows_per_cta;
  const long long r1 = r0 + rows_per_cta < rows ? r0 + rows_per_cta : rows;
  for (int cb = 0; cb < vec_cols; cb += lanes_c) {          // uniform trip count: the loop holds barriers
    const int c = cb + tc;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (tr < lanes_r && c < vec_cols) {
      const float4* x = reinterpret_cast<const float4*>(X) + c;
      const float4* y = reinterpret_cast<const float4*>(Y) + c;
#pragma unroll 4
      for (long long r = r0 + tr; r < r1; r += lanes_r) {
        const float4 a = ld_nc_f4(x + r * vec_cols), b = ld_nc_f4(y + r * vec_cols);
        acc.x = fmaf(a.x, b.x, acc.x); acc.y = fmaf(a.y, b.y, acc.y);
        acc.z = fmaf(a.z, b.z, acc.z); acc.w = fmaf(a.w, b.w, acc.w);
      }
    }
    red[threadIdx.x] = acc;
    __syncthreads();
    if (tr == 0 && c < vec_cols) {
      for (int j = 1; j < lanes_r; ++j) {
        const float4 o = red[j * lanes_c + tc];
        acc.x += o.x; acc.y += o.y; acc.z += o.z; acc.w += o.w;
      }
      reinterpret_cast<float4*>(partial + (long long)blockIdx.x * cols)[c] = acc;
    }
    __syncthreads();
  }
}

static int colwise_dot_ctas(long long rows) {
  long long n = 4LL * sm_count();
  if (n > rows) n = rows;
  return n < 1 ? 1 : (int)n;
}

template <int BN>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& th, const CUtensorMap& tl, GemmParams p,
                       cudaStream_t stream) {
  using S = Smem<BN>;
  int stages = kMaxStages;
  while (stages > 1 && S::bytes(stages) > 220 * 1024) --stages;
  p.stages = stages;
  p.tiles_m = (p.M + kBM - 1) / kBM;
  p.tiles_n = (p.N + BN - 1) / BN;
  const size_t smem = S::bytes(stages);
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(gemm_tf32x3_kernel<BN>), smem)) return rc;
  const long long ntiles = p.tiles_m * p.tiles_n;
  const unsigned grid = (unsigned)(ntiles < (long long)sm_budget() ? ntiles : (long long)sm_budget());
  gemm_tf32x3_kernel<BN><<<grid, kThreads, smem, stream>>>(ta, th, tl, p);
  return check_cuda(cudaGetLastError(), "gemm_tf32x3_kernel launch");
}

// K slices are divided over enough CTAs to fill the GPU once.
static int wgrad_row_tiles(long long M) { return M > kBM ? 2 : 1; }

static int wgrad_splits(long long M, long long N, long long batch, long long length) {
  const int BN = N > 128 ? 256 : (N > 64 ? 128 : 64);
  const long long bm = (long long)kBM * wgrad_row_tiles(M);
  const long long tiles = ((M + bm - 1) / bm) * ((N + BN - 1) / BN);
  const long long total = batch * ((length + kBK - 1) / kBK);
  long long splits = (sm_budget() + tiles - 1) / tiles;
  if (splits * tiles > sm_budget() && splits > 1) --splits;     // never more CTAs than the budget
  if (splits > total) splits = total;
  if (splits > 512) splits = 512;
  return splits < 1 ? 1 : (int)splits;
}

template <int BN, int MT>
static int launch_wgrad(const CUtensorMap& tx, const CUtensorMap& ty, WgradParams p, int splits, cudaStream_t stream) {
  constexpr size_t stage = 2 * (size_t)MT * kBM * kBK * 4 + 2 * (size_t)BN * kBK * 4;
  int stages = kMaxStages;
  while (stages > 1 && 2048 + stages * stage > 220 * 1024) --stages;
  p.stages = stages;
  const size_t smem = 2048 + stages * stage;
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(wgrad_tf32x3_kernel<BN, MT>), smem)) return rc;
  dim3 grid((unsigned)((p.M + MT * kBM - 1) / (MT * kBM)), (unsigned)((p.N + BN - 1) / BN), (unsigned)splits);
  wgrad_tf32x3_kernel<BN, MT><<<grid, kWgThreads, smem, stream>>>(tx, ty, p);
  return check_cuda(cudaGetLastError(), "wgrad_tf32x3_kernel launch");
}

}  // namespace layer
}  // namespace ossm_b200

extern "C" {

using namespace ossm_b200;

int ossm_b200_split_tf32(const float* w, float* w_hi, float* w_lo, int64_t count, cudaStream_t stream) {
  if (count < 0) { set_last_error("split_tf32: negative count"); return kErrInvalidArgument; }
  if (count == 0) return kOk;
  if (!w || !w_hi || !w_lo) { set_last_error("split_tf32: null pointer"); return kErrInvalidArgument; }
  layer::split_tf32_kernel<<<(unsigned)((count + 255) / 256), 256, 0, stream>>>(w, w_hi, w_lo, count);
  return check_cuda(cudaGetLastError(), "split_tf32_kernel launch");
}

size_t ossm_b200_wgrad_tf32x3_workspace_bytes(int64_t M, int64_t N, int64_t batch, int64_t length) {
  if (M <= 0 || N <= 0 || batch <= 0 || length <= 0) return 0;
  return (size_t)layer::wgrad_splits(M, N, batch, length) * (size_t)M * (size_t)N * sizeof(float);
}

int ossm_b200_layer_set_tuning(const char* key, int value) {
  if (key != nullptr && !strcmp(key, "reserve_sms") && value >= 0 && value <= 64) {
    layer::g_reserve_sms = value;
    return kOk;
  }
  set_last_error("layer_set_tuning: unknown key or value out of range");
  return kErrInvalidArgument;
}

int ossm_b200_wgrad_tf32x3(const float* X, int x_time_major, const float* Y, int y_time_major, float* partial,
                           size_t partial_bytes, int* splits_out, int64_t M, int64_t N, int64_t batch, int64_t length,
                           cudaStream_t stream) {
  if (M <= 0 || N <= 0 || batch <= 0 || length <= 0) { set_last_error("wgrad_tf32x3: extents must be positive"); return kErrInvalidArgument; }
  if (!X || !Y || !partial || !splits_out) { set_last_error("wgrad_tf32x3: null pointer"); return kErrInvalidArgument; }
  if ((M % 32) != 0 || (N % 32) != 0) {
    set_last_error("wgrad_tf32x3: M and N must be multiples of 32 (column blocks of the operand tiles)");
    return kErrUnsupported;
  }
  const int splits = layer::wgrad_splits(M, N, batch, length);
  if (partial_bytes < (size_t)splits * M * N * sizeof(float)) { set_last_error("wgrad_tf32x3: workspace too small"); return kErrWorkspace; }
  const int BN = N > 128 ? 256 : (N > 64 ? 128 : 64);
  auto make = [&](CUtensorMap* tm, const float* base, long long C, bool time_major, uint32_t tile) {
    // dims innermost first: 32 columns of a block, time, column block, batch
    const uint64_t dims[4] = {32, (uint64_t)length, (uint64_t)(C / 32), (uint64_t)batch};
    const uint64_t row = (uint64_t)C * 4;
    const uint64_t strides[3] = {time_major ? row * (uint64_t)batch : row, 128,
                                 time_major ? row : row * (uint64_t)length};
    const uint32_t box[4] = {32, (uint32_t)layer::kBK, tile / 32, 1};
    return make_tensor_map_4d_f32_sw128(tm, base, dims, strides, box, true);
  };
  CUtensorMap tx, ty;
  const int MT = layer::wgrad_row_tiles(M);
  if (!make(&tx, X, M, x_time_major != 0, (uint32_t)(MT * layer::kBM)) || !make(&ty, Y, N, y_time_major != 0, (uint32_t)BN)) {
    set_last_error("wgrad_tf32x3: operands must be 16-byte aligned dense matrices");
    return kErrUnsupported;
  }
  layer::WgradParams p{};
  p.partial = partial; p.M = M; p.N = N; p.batch = batch; p.length = length;
  p.slices_per_batch = (int)((length + layer::kBK - 1) / layer::kBK);
  *splits_out = splits;
  if (MT == 2) {
    if (BN == 256) return layer::launch_wgrad<256, 2>(tx, ty, p, splits, stream);
    if (BN == 128) return layer::launch_wgrad<128, 2>(tx, ty, p, splits, stream);
    return layer::launch_wgrad<64, 2>(tx, ty, p, splits, stream);
  }
  if (BN == 256) return layer::launch_wgrad<256, 1>(tx, ty, p, splits, stream);
  if (BN == 128) return layer::launch_wgrad<128, 1>(tx, ty, p, splits, stream);
  return layer::launch_wgrad<64, 1>(tx, ty, p, splits, stream);
}

int ossm_b200_gemm_tf32x3(const float* A, const float* W_hi, const float* W_lo, float* out, const float* aux,
                          const float* diag, int64_t M, int64_t N, int64_t K, int64_t ldo, int64_t col_block,
                          int64_t plane_stride, int row_map, int64_t batch, int64_t length, cudaStream_t stream) {
  if (M < 0 || N < 0 || K < 0) { set_last_error("gemm_tf32x3: negative extent"); return kErrInvalidArgument; }
  if (M == 0 || N == 0) return kOk;
  if (!A || !W_hi || !W_lo || !out || (aux != nullptr) != (diag != nullptr)) {
    set_last_error("gemm_tf32x3: null pointer (aux and diag come together)");
    return kErrInvalidArgument;
  }
  if (K == 0 || (K & 3) != 0) { set_last_error("gemm_tf32x3: K must be a positive multiple of 4"); return kErrUnsupported; }
  if (row_map < layer::kRowIdentity || row_map > layer::kRowTimeToBatch ||
      (row_map != layer::kRowIdentity && (batch <= 0 || length <= 0 || batch * length != M))) {
    set_last_error("gemm_tf32x3: bad row map (batch * length must equal M)");
    return kErrInvalidArgument;
  }
  if (col_block <= 0 || col_block > N) { col_block = N; plane_stride = 0; }
  if (ldo < col_block) { set_last_error("gemm_tf32x3: output pitch smaller than the column block"); return kErrInvalidArgument; }
  if (M > 0x7fffffffLL - layer::kBM || N > 0x7fffffffLL - 256) { set_last_error("gemm_tf32x3: extent too large"); return kErrInvalidArgument; }
  const int BN = N > 128 ? 256 : (N > 64 ? 128 : 64);
  CUtensorMap ta, th, tl;
  if (!make_tensor_map_2d_f32_sw64(&ta, A, (uint64_t)K, (uint64_t)M, (uint64_t)K * 4, layer::kPK, layer::kBM) ||
      !make_tensor_map_2d_f32_sw64(&th, W_hi, (uint64_t)K, (uint64_t)N, (uint64_t)K * 4, layer::kPK, BN) ||
      !make_tensor_map_2d_f32_sw64(&tl, W_lo, (uint64_t)K, (uint64_t)N, (uint64_t)K * 4, layer::kPK, BN)) {
    set_last_error("gemm_tf32x3: operands must be 16-byte aligned, dense row-major matrices");
    return kErrUnsupported;
  }
  layer::GemmParams p{};
  p.out = out; p.aux = aux; p.diag = diag;
  p.col_block = col_block; p.plane_stride = plane_stride;
  p.M = M; p.N = N; p.K = K; p.ldo = ldo; p.batch = batch; p.length = length; p.row_map = row_map;
  if (BN == 256) return layer::launch_gemm<256>(ta, th, tl, p, stream);
  if (BN == 128) return layer::launch_gemm<128>(ta, th, tl, p, stream);
  return layer::launch_gemm<64>(ta, th, tl, p, stream);
}

int ossm_b200_colwise_dot_partials(int64_t rows) { return rows > 0 ? layer::colwise_dot_ctas(rows) : 0; }

int ossm_b200_colwise_dot(const float* X, const float* Y, float* partial, int64_t rows, int64_t cols,
                          cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) { set_last_error("colwise_dot: extents must be positive"); return kErrInvalidArgument; }
  if (!X || !Y || !partial) { set_last_error("colwise_dot: null pointer"); return kErrInvalidArgument; }
  if ((cols & 3) != 0 || ((reinterpret_cast<uintptr_t>(X) | reinterpret_cast<uintptr_t>(Y) | reinterpret_cast<uintptr_t>(partial)) & 15u) != 0) {
    set_last_error("colwise_dot: the column count must be a multiple of 4 and the matrices 16-byte aligned");
    return kErrUnsupported;
  }
  const int ctas = layer::colwise_dot_ctas(rows);
  const long long per = (rows + ctas - 1) / ctas;
  layer::colwise_dot_kernel<<<ctas, layer::kDotThreads, 0, stream>>>(X, Y, partial, rows, cols, per);
  return check_cuda(cudaGetLastError(), "colwise_dot_kernel launch");
}

}  // extern "C"
