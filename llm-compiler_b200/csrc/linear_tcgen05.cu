// serve.linear on the 5th-generation tensor cores: tcgen05.mma with the accumulator in tensor
// memory (TMEM), operands staged in shared memory by TMA.
//
// y[M,N] = x[M,K] W[N,K]^T, both operands K-major bf16. One CTA computes a 128 x bn tile over
// one K slice (bn: a runtime multiple of 16 up to the template's BN accumulator columns of
// TMEM, fp32). Roles inside the CTA of 4 warps:
//   warp 0, one elected lane  TMA producer: per k-block one A_ROWS x 64 box of x and one bn x 64
//                             box of W (128-byte swizzled rows) into a ring of stages,
//                             completion on the stage's `full` mbarrier. W does not depend on
//                             the kernel before this one: when the caller says weights are
//                             constants, the first ring of W boxes is requested BEFORE the
//                             dependency wait (their bytes are announced on the barrier without
//                             arriving), the x boxes after it;
//   warp 1, one elected lane  MMA issuer: per stage four tcgen05.mma (M 128, N bn, K 16) whose
//                             shared-memory descriptors walk the 64-wide swizzled tile in 32-byte
//                             steps; tcgen05.commit arrives on the stage's `empty` mbarrier when
//                             the tensor core is done reading it, and on `accum` after the last
//                             k-block;
//   all 4 warps               epilogue: tcgen05.ld of the warp's 32 TMEM lanes (= 32 output
//                             rows) x 32 columns at a time; bias / residual / SwiGLU with the
//                             reference's bf16 rounding points, or fp32 split-K partials.
// Decode-size M (A_ROWS 64): the x box has 64 rows and the MMA, which always spans 128, reads on
// into the W tile behind it; accumulator lanes 64..127 then hold junk that nobody reads.
// Every mbarrier wait is bounded; a wait that gives up sets B200_STATUS_WAIT_TIMEOUT, the CTA
// still frees its TMEM columns and returns. No cluster launch, no load shared between CTAs:
// each CTA fetches its own tiles; with BN 128 at prefill sizes a second CTA resident on the SM
// overlaps its main loop with this one's epilogue (2 x 96 KB of stages, 2 x 128 TMEM columns).
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "common.cuh"
#include "tcgen05.cuh"
#include "tensor_map.cuh"

namespace b200 {
namespace {

constexpr int kBM = 128;
constexpr int kBK = 64;
constexpr int kThreads = 128;

constexpr int kEpiloguePartial = 100;  // internal: fp32 split-K partials, no rounding
// internal: the K slices of a tile are the CTAs of one thread-block cluster (cluster extent =
// splits along grid z); they add their fp32 accumulators through distributed shared memory and
// write r(r(x W^T) + residual) themselves: no partials in global memory, no reduce kernel
constexpr int kEpilogueClusterResidual = 101;

struct Tcgen05Params {
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual;
  __nv_bfloat16* out;
  float* partials;  // [splits, m, n] fp32 when epilogue == kEpiloguePartial
  int32_t* status;
  int m, k, n, epilogue, splits;
  int bn;  // columns per tile: a multiple of 16, at most the kernel's BN
  int prefetch_weights;  // W tiles may be fetched before the predecessor kernel has finished
  // Grid x walks the M tiles (and y the N tiles) instead of the other way round: CTAs are placed
  // in x-fastest order, so the few M tiles of one N tile then run side by side and the second
  // finds the W tile in L2. With N fastest and a W larger than L2 (a 7B gate|up projection at
  // 256 rows: 271 MB, two M tiles) every M tile streamed W from HBM again.
  int m_fastest = 0;
  // With prefetch_weights: the W tiles behind the first ring are requested into L2 before the
  // dependency wait as well, so that the ring's later rounds cost an L2 hit, not an HBM access.
  int prefetch_l2 = 0;
  uint32_t wait_limit = 4000000u;  // polls of a bounded wait
  int drop_loads = 0;              // debug: the producer issues nothing (every wait runs out)
  // RMSNorm folded into the projection (norm_input != nullptr): the A operand is the
  // un-normalised x, the norm weight is already multiplied into W's columns, and the epilogue
  // scales row r of the accumulator by rsqrt(mean(x_r^2) + eps) before bias / SwiGLU.
  const __nv_bfloat16* norm_input = nullptr;
  int64_t norm_row_stride = 0;
  float norm_eps = 0.0f;
  // Partial-sum producer only: the CTAs of the first N tile also leave sum(x_r^2) over their K
  // slice in row_squares[split, m], for the consumer that applies the folded RMSNorm.
  float* row_squares = nullptr;
  // Cluster split-K only: sum(y_r^2) of the stored (rounded) output rows over the units this
  // CTA owns, squares_out[(N tile * splits + K slice), m]: the row sums of squares that a folded
  // RMSNorm behind this projection needs, left for it in slices that it adds in a fixed order.
  float* squares_out = nullptr;
  // Folded RMSNorm whose producer left such slices (norm_squares[norm_slices, m]): the two idle
  // warps add them instead of squaring every x box.
  const float* norm_squares = nullptr;
  int norm_slices = 0;
};

// silu for the fused SwiGLU epilogue: x / (1 + 2^(-x log2 e)) on the special-function unit
// (ex2.approx, rcp.approx: a few ulp of fp32, far below the bf16 rounding that follows). An
// IEEE expf + division costs ~160 cycles per element on the epilogue's lone warps, which made
// the epilogue of the gate|up projection longer than its main loop.
__device__ __forceinline__ float silu_f32(float x) {
  return __fdividef(x, 1.0f + exp2f(-1.4426950408889634f * x));
}

// Bias onto 32 accumulator columns (16-byte loads where all 32 columns exist and are aligned).
__device__ __forceinline__ void add_bias(const Tcgen05Params& p, int col0, int n_end, float (&v)[32]) {
  const bool whole = col0 + 32 <= n_end;
  if (p.bias != nullptr) {
    if (whole && (reinterpret_cast<uintptr_t>(p.bias + col0) & 15u) == 0) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint4 b = __ldg(reinterpret_cast<const uint4*>(p.bias + col0) + i);
        v[8 * i] += bf16_lo(b.x); v[8 * i + 1] += bf16_hi(b.x);
        v[8 * i + 2] += bf16_lo(b.y); v[8 * i + 3] += bf16_hi(b.y);
        v[8 * i + 4] += bf16_lo(b.z); v[8 * i + 5] += bf16_hi(b.z);
        v[8 * i + 6] += bf16_lo(b.w); v[8 * i + 7] += bf16_hi(b.w);
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (col0 + i < n_end) v[i] += __bfloat162float(p.bias[col0 + i]);
    }
  }
}

// r(r(x W^T + b) + residual) for 32 columns of one output row.
__device__ __forceinline__ void add_residual(const Tcgen05Params& p, int epilogue, int row, int col0,
                                             int n_end, float (&v)[32]) {
  const bool whole = col0 + 32 <= n_end;
  const int64_t o = static_cast<int64_t>(row) * p.n + col0;
  if (epilogue == B200_EPILOGUE_RESIDUAL) {  // r(r(x W^T + b) + residual)
#pragma unroll
    for (int i = 0; i < 32; i += 2) round_bf16_pair(v[i], v[i + 1]);
    if (whole && (reinterpret_cast<uintptr_t>(p.residual + o) & 15u) == 0) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint4 r = *(reinterpret_cast<const uint4*>(p.residual + o) + i);
        v[8 * i] = __fadd_rn(v[8 * i], bf16_lo(r.x)); v[8 * i + 1] = __fadd_rn(v[8 * i + 1], bf16_hi(r.x));
        v[8 * i + 2] = __fadd_rn(v[8 * i + 2], bf16_lo(r.y)); v[8 * i + 3] = __fadd_rn(v[8 * i + 3], bf16_hi(r.y));
        v[8 * i + 4] = __fadd_rn(v[8 * i + 4], bf16_lo(r.z)); v[8 * i + 5] = __fadd_rn(v[8 * i + 5], bf16_hi(r.z));
        v[8 * i + 6] = __fadd_rn(v[8 * i + 6], bf16_lo(r.w)); v[8 * i + 7] = __fadd_rn(v[8 * i + 7], bf16_hi(r.w));
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (col0 + i < n_end) v[i] = __fadd_rn(v[i], __bfloat162float(p.residual[o + i]));
    }
  }  // (without a residual the store below is the one rounding)
}

// y_j = r(silu(r(gate_j))) * r(up_j) for the 16 (gate, up) column pairs of a 32-column chunk;
// the caller's store rounds the product. The roundings go through the conversion unit, which
// the exponentials and reciprocals of silu also queue for, so they are taken in pairs.
__device__ __forceinline__ void swiglu_of_chunk(float (&v)[32], float (&y)[16]) {
#pragma unroll
  for (int j = 0; j < 16; j += 2) {
    round_bf16_pair(v[2 * j], v[2 * j + 1]);
    round_bf16_pair(v[2 * j + 2], v[2 * j + 3]);
    float g0 = silu_f32(v[2 * j]), g1 = silu_f32(v[2 * j + 2]);
    round_bf16_pair(g0, g1);
    y[j] = g0 * v[2 * j + 1];
    y[j + 1] = g1 * v[2 * j + 3];
  }
}

// The bf16 epilogue of 32 accumulator columns of one output row: bias, then SwiGLU (columns
// 2j / 2j+1 are gate_j / up_j) or the residual, with the reference's bf16 rounding points.
// EPI >= 0: the epilogue is known at compile time (the decode chain's instantiations carry
// only their own); -1: taken from the parameters.
template <int EPI = -1>
__device__ __forceinline__ void store_chunk(const Tcgen05Params& p, int row, int col0, int n_end,
                                            float (&v)[32]) {
  const int epilogue = EPI >= 0 ? EPI : p.epilogue;
  const int out_cols = epilogue == B200_EPILOGUE_SWIGLU ? p.n / 2 : p.n;
  const bool whole = col0 + 32 <= n_end;  // all 32 columns exist: 16-byte accesses where aligned
  add_bias(p, col0, n_end, v);
  if (epilogue == B200_EPILOGUE_SWIGLU) {
    // columns 2j / 2j+1 are gate_j / up_j
    __nv_bfloat16* dst = p.out + static_cast<int64_t>(row) * out_cols + col0 / 2;
    float y[16];
    swiglu_of_chunk(v, y);
    if (col0 + 32 <= n_end && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
#pragma unroll
      for (int i = 0; i < 2; ++i)
        reinterpret_cast<uint4*>(dst)[i] =
            make_uint4(pack_bf16x2(y[8 * i], y[8 * i + 1]), pack_bf16x2(y[8 * i + 2], y[8 * i + 3]),
                       pack_bf16x2(y[8 * i + 4], y[8 * i + 5]), pack_bf16x2(y[8 * i + 6], y[8 * i + 7]));
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j)
        if (col0 + 2 * j + 1 < n_end) dst[j] = __float2bfloat16_rn(y[j]);
    }
    return;
  }
  const int64_t o = static_cast<int64_t>(row) * p.n + col0;
  add_residual(p, epilogue, row, col0, n_end, v);
  __nv_bfloat16* dst = p.out + o;
  if (whole && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
#pragma unroll
    for (int i = 0; i < 4; ++i)
      reinterpret_cast<uint4*>(dst)[i] =
          make_uint4(pack_bf16x2(v[8 * i], v[8 * i + 1]), pack_bf16x2(v[8 * i + 2], v[8 * i + 3]),
                     pack_bf16x2(v[8 * i + 4], v[8 * i + 5]), pack_bf16x2(v[8 * i + 6], v[8 * i + 7]));
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (col0 + i < n_end) dst[i] = __float2bfloat16_rn(v[i]);
  }
}

// A_ROWS: rows of the x box a stage holds. With at most 64 activation rows (decode) the box
// is 64 rows and the MMA, which always spans 128 rows, reads on into the W tile behind it:
// accumulator lanes 64..127 then hold junk that the epilogue never touches (rows >= M).
// FORM: which of the four jobs this instantiation does (a compile-time choice: a decode-size
// launch pays for every instruction it carries, in registers and in first-touch instruction
// fetches; two extra branches in the producer / MMA loops once cost 7 % of a decode step).
constexpr int kFormPlain = 0;    // bias / residual / SwiGLU epilogue
constexpr int kFormPartial = 1;  // fp32 split-K partials (+ row sums of squares of x)
constexpr int kFormCluster = 2;  // split-K over a thread-block cluster, residual inside
constexpr int kFormNorm = 3;     // folded RMSNorm, bias, no other epilogue (an LM head)
constexpr int kFormNormSwiglu = 4;  // folded RMSNorm + SwiGLU (a gate|up projection)

template <int BN, int STAGES, int A_ROWS, int FORM>
__global__ void __launch_bounds__(kThreads)
linear_tcgen05_kernel(const Tcgen05Params p, const __grid_constant__ CUtensorMap a_map,
                      const __grid_constant__ CUtensorMap b_map) {
  constexpr bool kCluster = FORM == kFormCluster, kPartial = FORM == kFormPartial;
  constexpr bool kNorm = FORM == kFormNorm || FORM == kFormNormSwiglu;
  constexpr int kEpilogue = FORM == kFormNormSwiglu ? B200_EPILOGUE_SWIGLU : FORM == kFormNorm ? B200_EPILOGUE_NONE : -1;
  constexpr int kABytes = A_ROWS * 128;
  // TMEM is allocated in powers of two of at least 32 columns
  constexpr int kTmemColumns = BN <= 32 ? 32 : BN <= 64 ? 64 : BN <= 128 ? 128 : BN <= 256 ? 256 : 512;
  constexpr int kBBytes = BN * 128;
  constexpr int kStageBytes = kABytes + kBBytes;
  const int bn = p.bn;
  const uint32_t idesc = instruction_descriptor(kBM, bn);
  const uint32_t stage_tx_bytes = static_cast<uint32_t>(kABytes + bn * 128);

  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ __align__(8) uint64_t full_bar[STAGES];
  __shared__ __align__(8) uint64_t empty_bar[STAGES];
  __shared__ __align__(8) uint64_t accum_bar;
  __shared__ __align__(8) uint64_t reduce_bar;  // cluster split-K: all slices of my units have landed
  __shared__ uint32_t tmem_base_slot;
  __shared__ int failed;
  __shared__ float row_scale[kBM];  // folded RMSNorm: rsqrt(mean(x_r^2) + eps) per tile row

  TraceScope trace(1);
  grid_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile_n = p.m_fastest ? blockIdx.y : blockIdx.x, tile_m = p.m_fastest ? blockIdx.x : blockIdx.y;
  const int split = blockIdx.z;
  const int kb_total = (p.k + kBK - 1) / kBK;
  const int kb_per = (kb_total + p.splits - 1) / p.splits;
  const int kb_first = split * kb_per;
  const int nkb = max(0, min(kb_first + kb_per, kb_total) - kb_first);
  const uint32_t smem_base = smem_u32(smem);
  // warps 2 and 3 square the rows of x as they pass through shared memory
  const bool squares = (kNorm && p.norm_squares == nullptr) ||
                       (kPartial && p.row_squares != nullptr && tile_n == 0);

  if (threadIdx.x == 0) {
    failed = 0;
#pragma unroll
    for (int s = 0; s < STAGES; ++s) {
      mbarrier_init(smem_u32(&full_bar[s]), 1);
      // a stage is free once the tensor core has read it and, with a folded RMSNorm, once
      // warps 2 and 3 have squared its rows of x as well
      mbarrier_init(smem_u32(&empty_bar[s]), squares ? 3 : 1);
    }
    mbarrier_init(smem_u32(&accum_bar), 1);
    mbarrier_init(smem_u32(&reduce_bar), 1);
    fence_mbarrier_init();
  }
  if (warp == 1) {  // one warp allocates the accumulator columns and later frees them
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&tmem_base_slot)), "r"(static_cast<uint32_t>(kTmemColumns))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_slot;
  // Cluster split-K: the other CTAs of the cluster will signal reduce_bar; none may do so
  // before it is initialised, hence one cluster barrier here, in the prologue that overlaps
  // the predecessor kernel. Then this CTA announces the bytes it is going to receive.
  const int reduce_owned = kCluster
      ? (A_ROWS * (bn / 4) + p.splits - 1) / p.splits : 0;  // 16-byte units this CTA sums
  if (kCluster) {
    cluster_sync();
    if (threadIdx.x == 0)
      mbarrier_arrive_expect_tx(smem_u32(&reduce_bar), static_cast<uint32_t>(p.splits * reduce_owned * 16));
  }

  if (warp == 0 && lane == 0 && !p.drop_loads) {
    // ---- TMA producer ----
    // The first ring of W tiles does not depend on the kernel before this one: fetch it
    // before waiting for that kernel (the transaction bytes are announced without arriving,
    // so a stage cannot complete before its x box has been requested as well).
    const int early = p.prefetch_weights ? min(nkb, STAGES) : 0;
    auto k_of = [&](int kb) { return (kb_first + kb) * kBK; };  // element offset of the kb-th k-block
    for (int kb = 0; kb < early; ++kb) {
      const uint32_t bar = smem_u32(&full_bar[kb]);
      mbarrier_expect_tx(bar, static_cast<uint32_t>(bn * 128));
      tma_load_2d(smem_base + kb * kStageBytes + kABytes, &b_map, bar, k_of(kb), tile_n * bn);
    }
    if (p.prefetch_l2)
      for (int kb = early; kb < nkb; ++kb) tma_prefetch_l2_2d(&b_map, k_of(kb), tile_n * bn);
    grid_dependency_wait();
    trace.mark(0);
    for (int kb = 0; kb < nkb; ++kb) {
      const int s = kb % STAGES;
      if (kb >= STAGES &&
          !mbarrier_wait_bounded(smem_u32(&empty_bar[s]), ((kb / STAGES) - 1) & 1, p.wait_limit)) {
        failed = 1;
        break;
      }
      const uint32_t bar = smem_u32(&full_bar[s]);
      const uint32_t a_dst = smem_base + s * kStageBytes;
      if (kb < early) {
        mbarrier_arrive_expect_tx(bar, static_cast<uint32_t>(kABytes));
        tma_load_2d(a_dst, &a_map, bar, k_of(kb), tile_m * kBM);
      } else {
        mbarrier_arrive_expect_tx(bar, stage_tx_bytes);
        tma_load_2d(a_dst, &a_map, bar, k_of(kb), tile_m * kBM);
        tma_load_2d(a_dst + kABytes, &b_map, bar, k_of(kb), tile_n * bn);
      }
    }
  } else if (warp == 1 && lane == 0) {
    // The MMA issuer waits too (a K slice without k-blocks has no TMA copy to order it after
    // the producer's wait). The other threads only ever act on what these three hand them
    // through mbarriers, and stay out of the way of the kernels still running on the SM.
    grid_dependency_wait();
  }
  if ((kNorm || kPartial) && warp >= 2 && squares) {
    // Folded RMSNorm (A_ROWS == 64): warps 2 and 3 have nothing else to do until the accumulator
    // is complete. Every k-block's 64 x 64 box of x passes through shared memory for the tensor
    // core anyway; thread t of the two warps squares row t of each box as it lands (128 bytes,
    // eight 16-byte reads that start at chunk t & 7 so that a quarter-warp never shares a bank;
    // the swizzle only permutes chunks within the row, which a sum does not care about; columns
    // beyond K are zero-filled by the copy). One fixed summation order per row, no extra global
    // traffic, and the row factors are ready when the last k-block is.
    // (A_ROWS == 128: the same 64 threads take rows t and t + 64 of every box)
    constexpr int kRowsEach = A_ROWS / 64;
    const int r = (warp - 2) * 32 + lane;
    float ss[kRowsEach];
#pragma unroll
    for (int h = 0; h < kRowsEach; ++h) ss[h] = 0.0f;
    bool fine = true;
    for (int kb = 0; kb < nkb && fine; ++kb) {
      const int s = kb % STAGES;
      fine = __all_sync(0xffffffffu, mbarrier_wait_bounded(smem_u32(&full_bar[s]), (kb / STAGES) & 1, p.wait_limit));
      if (fine) {
#pragma unroll
        for (int h = 0; h < kRowsEach; ++h) {
          const uint32_t row_addr = smem_base + s * kStageBytes + (r + 64 * h) * 128;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            uint4 raw;
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(raw.x), "=r"(raw.y), "=r"(raw.z), "=r"(raw.w)
                         : "r"(row_addr + (((j + r) & 7) << 4)));
            ss[h] = fmaf(bf16_lo(raw.x), bf16_lo(raw.x), ss[h]); ss[h] = fmaf(bf16_hi(raw.x), bf16_hi(raw.x), ss[h]);
            ss[h] = fmaf(bf16_lo(raw.y), bf16_lo(raw.y), ss[h]); ss[h] = fmaf(bf16_hi(raw.y), bf16_hi(raw.y), ss[h]);
            ss[h] = fmaf(bf16_lo(raw.z), bf16_lo(raw.z), ss[h]); ss[h] = fmaf(bf16_hi(raw.z), bf16_hi(raw.z), ss[h]);
            ss[h] = fmaf(bf16_lo(raw.w), bf16_lo(raw.w), ss[h]); ss[h] = fmaf(bf16_hi(raw.w), bf16_hi(raw.w), ss[h]);
          }
        }
      }
      __syncwarp();
      if (lane == 0)
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&empty_bar[s])) : "memory");
    }
    if (!fine) failed = 1;
#pragma unroll
    for (int h = 0; h < kRowsEach; ++h) {
      const int row = r + 64 * h;
      if (kNorm)
        row_scale[row] = rsqrtf(ss[h] / static_cast<float>(p.k) + p.norm_eps);
      else if (tile_m * kBM + row < p.m)
        p.row_squares[static_cast<int64_t>(split) * p.m + tile_m * kBM + row] = fine ? ss[h] : 0.0f;
    }
  }
  if (kNorm && warp >= 2 && p.norm_squares != nullptr) {
    // Folded RMSNorm, row sums of squares left by the kernel that produced x: thread t of warps
    // 2 and 3 adds the slices of row t (and of row t + 64 of a 128-row tile) in slice order (L2
    // reads, sixteen in flight) while the main loop runs. The slices are that kernel's output:
    // wait for it first.
    if (lane == 0) grid_dependency_wait();
    __syncwarp();
#pragma unroll 1
    for (int row = (warp - 2) * 32 + lane; row < A_ROWS; row += 64) {
      const int global_row = tile_m * kBM + row;
      float ss = 0.0f;
      if (global_row < p.m) {
        const float* src = p.norm_squares + global_row;
        int slice = 0;
#pragma unroll 1
        for (; slice + 16 <= p.norm_slices; slice += 16) {
          float t[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) t[i] = __ldcg(src + static_cast<int64_t>(slice + i) * p.m);
#pragma unroll
          for (int i = 0; i < 16; ++i) ss += t[i];
        }
#pragma unroll 1
        for (; slice < p.norm_slices; ++slice) ss += __ldcg(src + static_cast<int64_t>(slice) * p.m);
      }
      row_scale[row] = rsqrtf(ss / static_cast<float>(p.k) + p.norm_eps);
    }
  }
  if (warp == 1 && lane == 0) {
    // ---- MMA issuer ----
    for (int kb = 0; kb < nkb; ++kb) {
      const int s = kb % STAGES;
      if (!mbarrier_wait_bounded(smem_u32(&full_bar[s]), (kb / STAGES) & 1, p.wait_limit)) {
        failed = 1;
        break;
      }

      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t a_addr = smem_base + s * kStageBytes;
      const uint32_t b_addr = a_addr + kABytes;
#pragma unroll
      for (int j = 0; j < kBK / 16; ++j)
        umma_bf16(tmem_base, smem_descriptor(a_addr + j * 32), smem_descriptor(b_addr + j * 32),
                  idesc, (kb > 0 || j > 0) ? 1u : 0u);
      umma_commit(smem_u32(&empty_bar[s]));  // the stage is free once these MMAs have read it
    }
    umma_commit(smem_u32(&accum_bar));  // the accumulator is complete once all MMAs retired
  }
  __syncwarp();

  // ---- epilogue: all four warps, warp w reads TMEM lanes 32w .. 32w+31 = output rows ----
  bool ok = mbarrier_wait_bounded(smem_u32(&accum_bar), 0, p.wait_limit);
  trace.mark_middle();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  if (kNorm) __syncthreads();  // the row scales of warps 2 and 3
  ok = ok && failed == 0;
  if constexpr (kCluster) {
    // ---- split-K over a thread-block cluster: reduce through distributed shared memory ----
    // The tile's 4-column units (A_ROWS x bn / 4 of them) are dealt round-robin to the CTAs of
    // the cluster (one per K slice): unit i belongs to CTA i % splits, as its local unit
    // i / splits. Behind the stage ring every CTA has a send region [owner][local unit] and a
    // receive region [slice][local unit] of 16-byte units. The CTA sorts its fp32 accumulator
    // into the send region (plain shared-memory stores), then one thread per owner ships that
    // owner's chunk with ONE bulk copy through distributed shared memory, which completes on
    // the owner's reduce_bar. An owner that has received all slices adds them in slice order
    // from its own shared memory, rounds, adds the residual, rounds and stores. The cluster
    // barrier around the sums only keeps every CTA resident until the copies that read its
    // send region have landed. A CTA whose waits gave up still ships (zeros) and arrives.
    // (The code is kept small on purpose -- one division per thread, rolled loops: a kernel this
    // short pays for every instruction-cache line it touches for the first time.)
    const int rows = min(A_ROWS, p.m - tile_m * kBM);
    const int unit_shift = 31 - __clz(bn / 4);  // bn is 32, 64 or 128 here: 8, 16 or 32 units a row
    const int owned = reduce_owned;
    const uint32_t chunk_bytes = static_cast<uint32_t>(owned * 16);
    const int rank = cluster_cta_rank();
    const int n_end = min(p.n, (tile_n + 1) * bn);
    const uint32_t send_base = smem_base + STAGES * kStageBytes + 9216;
    const uint32_t recv_base = send_base + p.splits * chunk_bytes;
    if (warp * 32 < A_ROWS) {
      const int r = warp * 32 + lane;
      int owner = (r << unit_shift) % p.splits, local = (r << unit_shift) / p.splits;
#pragma unroll 1
      for (int c0 = 0; c0 < bn; c0 += 32) {
        float v[32];
        tmem_load_32x32(tmem_base + (static_cast<uint32_t>(warp * 32) << 16) + c0, v);
        if (!ok || nkb == 0) {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0.0f;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {  // consecutive units go to consecutive owners
          asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(
                           send_base + owner * chunk_bytes + local * 16),
                       "f"(v[4 * u]), "f"(v[4 * u + 1]), "f"(v[4 * u + 2]), "f"(v[4 * u + 3]) : "memory");
          if (++owner == p.splits) {
            owner = 0;
            ++local;
          }
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the copies below read these stores
    }
    __syncthreads();
    trace.stamp(2);
    if (threadIdx.x < p.splits) {
      const int owner = threadIdx.x;
      uint32_t remote_dst, remote_bar;
      asm volatile("mapa.shared::cluster.u32 %0, %1, %2;"
                   : "=r"(remote_dst) : "r"(recv_base + rank * chunk_bytes), "r"(owner));
      asm volatile("mapa.shared::cluster.u32 %0, %1, %2;"
                   : "=r"(remote_bar) : "r"(smem_u32(&reduce_bar)), "r"(owner));
      asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                   ::"r"(remote_dst), "r"(send_base + owner * chunk_bytes), "r"(chunk_bytes), "r"(remote_bar)
                   : "memory");
    }
    // the residual of this thread's first unit travels while the slices do
    const int first_item = threadIdx.x * p.splits + rank;
    const int first_row = first_item >> unit_shift, first_col = tile_n * bn + (first_item & ((bn / 4) - 1)) * 4;
    const bool first_valid = threadIdx.x < owned && first_row < rows && first_col < n_end;
    const int64_t first_offset = static_cast<int64_t>(tile_m * kBM + first_row) * p.n + first_col;
    uint2 res = first_valid ? *reinterpret_cast<const uint2*>(p.residual + first_offset) : make_uint2(0u, 0u);
    const bool landed = mbarrier_wait_bounded(smem_u32(&reduce_bar), 0, p.wait_limit);
    trace.stamp(4);
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
#pragma unroll 1
    for (int local = threadIdx.x; local < owned && landed; local += kThreads) {
      const int item = local * p.splits + rank;
      const int r = item >> unit_shift, col = tile_n * bn + (item & ((bn / 4) - 1)) * 4;
      if (r >= rows || col >= n_end) {
        if (p.squares_out != nullptr)
          asm volatile("st.shared.f32 [%0], %1;" ::"r"(recv_base + local * 16), "f"(0.0f) : "memory");
        continue;
      }
      const int64_t o = static_cast<int64_t>(tile_m * kBM + r) * p.n + col;  // n % 4 == 0
      if (local != threadIdx.x) res = *reinterpret_cast<const uint2*>(p.residual + o);
      float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      float4 t[8];
#pragma unroll
      for (int s0 = 0; s0 < 8; ++s0) {
        const uint32_t addr = recv_base + (s0 < p.splits ? s0 : 0) * chunk_bytes + local * 16;
        asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                     : "=f"(t[s0].x), "=f"(t[s0].y), "=f"(t[s0].z), "=f"(t[s0].w) : "r"(addr) : "memory");
      }
#pragma unroll
      for (int s0 = 0; s0 < 8; ++s0)
        if (s0 < p.splits) { acc.x += t[s0].x; acc.y += t[s0].y; acc.z += t[s0].z; acc.w += t[s0].w; }
      round_bf16_pair(acc.x, acc.y);
      round_bf16_pair(acc.z, acc.w);
      acc.x = __fadd_rn(acc.x, bf16_lo(res.x)); acc.y = __fadd_rn(acc.y, bf16_hi(res.x));
      acc.z = __fadd_rn(acc.z, bf16_lo(res.y)); acc.w = __fadd_rn(acc.w, bf16_hi(res.y));
      *reinterpret_cast<uint2*>(p.out + o) = make_uint2(pack_bf16x2(acc.x, acc.y), pack_bf16x2(acc.z, acc.w));
      if (p.squares_out != nullptr) {
        // the squares of what was stored; slice 0's copy of this unit, read by this thread alone, is free
        round_bf16_pair(acc.x, acc.y);
        round_bf16_pair(acc.z, acc.w);
        const float sq = fmaf(acc.x, acc.x, fmaf(acc.y, acc.y, fmaf(acc.z, acc.z, acc.w * acc.w)));
        asm volatile("st.shared.f32 [%0], %1;" ::"r"(recv_base + local * 16), "f"(sq) : "memory");
      }
    }
    if (p.squares_out != nullptr) {
      // one thread per row adds the units of its row that this CTA owns, in unit order
      __syncthreads();
      const int r = threadIdx.x, units_per_row = bn / 4, first = r * units_per_row;
      if (r < rows && landed) {
        float ss = 0.0f;
#pragma unroll 1
        for (int i = first + (rank - first % p.splits + p.splits) % p.splits; i < first + units_per_row; i += p.splits) {
          float sq;
          asm volatile("ld.shared.f32 %0, [%1];" : "=f"(sq) : "r"(recv_base + (i / p.splits) * 16) : "memory");
          ss += sq;
        }
        p.squares_out[static_cast<int64_t>(tile_n * p.splits + rank) * p.m + tile_m * kBM + r] = ss;
      }
    }
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    ok = ok && __syncthreads_and(landed);
    trace.stamp(6);
    if (!ok && threadIdx.x == 0 && p.status != nullptr) atomicOr(p.status, B200_STATUS_WAIT_TIMEOUT);
  } else if (ok) {
    const int row = tile_m * kBM + warp * 32 + lane;
    const float scale = kNorm ? row_scale[(warp * 32 + lane) % kBM] : 1.0f;
    const int n_end = min(p.n, (tile_n + 1) * bn);  // columns of this tile
#pragma unroll 1
    for (int c0 = 0; c0 < bn; c0 += 32) {
      const int col0 = tile_n * bn + c0;
      if (col0 >= n_end) break;  // warp-uniform: tcgen05.ld is a warp-wide instruction
      float v[32];
      tmem_load_32x32(tmem_base + (static_cast<uint32_t>(warp * 32) << 16) + c0, v);
      if (row >= p.m) continue;
      if (nkb == 0) {  // a K slice without k blocks contributes zeros, not stale TMEM
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = 0.0f;
      }
      if (kNorm) {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] *= scale;
      }
      if (kPartial) {
        float* dst = p.partials + (static_cast<int64_t>(split) * p.m + row) * p.n + col0;
        if (col0 + 32 <= n_end && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
#pragma unroll
          for (int i = 0; i < 8; ++i)
            reinterpret_cast<float4*>(dst)[i] =
                make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (col0 + i < n_end) dst[i] = v[i];
        }
        continue;
      }
      store_chunk<kEpilogue>(p, row, col0, n_end, v);
    }
  } else if (threadIdx.x == 0 && p.status != nullptr) {
    atomicOr(p.status, B200_STATUS_WAIT_TIMEOUT);
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;"
                 ::"r"(tmem_base), "r"(static_cast<uint32_t>(kTmemColumns)) : "memory");
  trace.mark(1);
}

// Prefill-size M: a persistent kernel, one CTA per SM walking 128 x bn output tiles (bn up to
// 256), with two accumulators in tensor memory so that the epilogue of one tile runs under the
// main loop of the next. With K = 896 (14 k-blocks) the epilogue of a 128 x 256 tile is about a
// third of its main loop; unhidden it capped these GEMMs near 0.45 of the tensor peak.
// Roles: warps 0-3 epilogue (warp w reads TMEM lanes 32 w ..), warp 4 (one lane) TMA producer,
// warp 5 (one lane) MMA issuer and owner of the 512 TMEM columns. The stage ring runs on across
// tile boundaries: the producer is already fetching the next tile while the last k-blocks of
// the current one are multiplied. Tiles are taken round-robin with N fastest, so the CTAs that
// run at the same time share their rows of x and the (small) W in L2.
constexpr int kPersistentStages = 4;
constexpr int kPersistentThreads = 192;
constexpr int kPersistentBN = 256;

__global__ void __launch_bounds__(kPersistentThreads, 1)
linear_tcgen05_persistent_kernel(const Tcgen05Params p, const __grid_constant__ CUtensorMap a_map,
                                 const __grid_constant__ CUtensorMap b_map) {
  constexpr int STAGES = kPersistentStages;
  constexpr int kABytes = kBM * 128;
  constexpr int kStageBytes = kABytes + kPersistentBN * 128;
  const int bn = p.bn;
  const uint32_t idesc = instruction_descriptor(kBM, bn);
  const uint32_t stage_tx_bytes = static_cast<uint32_t>(kABytes + bn * 128);

  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ __align__(8) uint64_t full_bar[STAGES], empty_bar[STAGES];
  __shared__ __align__(8) uint64_t acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int failed;

  TraceScope trace(9);
  grid_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nkb = (p.k + kBK - 1) / kBK;
  const int tiles_n = (p.n + bn - 1) / bn;
  const int tiles = tiles_n * ((p.m + kBM - 1) / kBM);
  const uint32_t smem_base = smem_u32(smem);

  if (threadIdx.x == 0) {
    failed = 0;
#pragma unroll
    for (int s = 0; s < STAGES; ++s) {
      mbarrier_init(smem_u32(&full_bar[s]), 1);
      mbarrier_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbarrier_init(smem_u32(&acc_full[a]), 1);
      mbarrier_init(smem_u32(&acc_empty[a]), 4);  // one arrival per epilogue warp
    }
    fence_mbarrier_init();
  }
  if (warp == 5) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&tmem_base_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_slot;

  if (warp == 4 && lane == 0 && !p.drop_loads) {
    // ---- TMA producer ----
    grid_dependency_wait();
    int round = 0;  // k-blocks issued so far, over all tiles
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < tiles; tile += gridDim.x) {
      const int tile_n = tile % tiles_n, tile_m = tile / tiles_n;
      for (int kb = 0; kb < nkb; ++kb, ++round) {
        const int s = round % STAGES;
        if (round >= STAGES &&
            !mbarrier_wait_bounded(smem_u32(&empty_bar[s]), ((round / STAGES) - 1) & 1, p.wait_limit)) {
          ok = false;
          break;
        }
        const uint32_t bar = smem_u32(&full_bar[s]);
        const uint32_t a_dst = smem_base + s * kStageBytes;
        mbarrier_arrive_expect_tx(bar, stage_tx_bytes);
        tma_load_2d(a_dst, &a_map, bar, kb * kBK, tile_m * kBM);
        tma_load_2d(a_dst + kABytes, &b_map, bar, kb * kBK, tile_n * bn);
      }
    }
    if (!ok) failed = 1;
  } else if (warp == 5 && lane == 0) {
    // ---- MMA issuer ----
    grid_dependency_wait();
    int round = 0, local = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < tiles; tile += gridDim.x, ++local) {
      const int acc = local & 1;
      // the epilogue must have read this accumulator's previous tile
      if (local >= 2 && !mbarrier_wait_bounded(smem_u32(&acc_empty[acc]), ((local >> 1) - 1) & 1, p.wait_limit)) {
        ok = false;
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t d_tmem = tmem_base + acc * kPersistentBN;
      for (int kb = 0; kb < nkb; ++kb, ++round) {
        const int s = round % STAGES;
        if (!mbarrier_wait_bounded(smem_u32(&full_bar[s]), (round / STAGES) & 1, p.wait_limit)) {
          ok = false;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a_addr = smem_base + s * kStageBytes;
        const uint32_t b_addr = a_addr + kABytes;
#pragma unroll
        for (int j = 0; j < kBK / 16; ++j)
          umma_bf16(d_tmem, smem_descriptor(a_addr + j * 32), smem_descriptor(b_addr + j * 32), idesc,
                    (kb > 0 || j > 0) ? 1u : 0u);
        umma_commit(smem_u32(&empty_bar[s]));  // the stage is free once these MMAs have read it
      }
      if (ok) umma_commit(smem_u32(&acc_full[acc]));  // the tile's accumulator is complete
    }
    if (!ok) failed = 1;
  } else if (warp < 4) {
    // ---- epilogue: warp w owns TMEM lanes 32 w .. 32 w + 31 = 32 output rows of the tile ----
    grid_dependency_wait();  // the residual was written by an earlier kernel
    int local = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++local) {
      const int acc = local & 1;
      const int tile_n = tile % tiles_n, tile_m = tile / tiles_n;
      // (the wait's outcome is made warp-uniform: tcgen05.ld is a warp-wide instruction)
      ok = ok && __all_sync(0xffffffffu, mbarrier_wait_bounded(smem_u32(&acc_full[acc]), (local >> 1) & 1, p.wait_limit));
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int row = tile_m * kBM + warp * 32 + lane;
      const int n_end = min(p.n, (tile_n + 1) * bn);
      const uint32_t t_addr = tmem_base + acc * kPersistentBN + (static_cast<uint32_t>(warp * 32) << 16);
      // The outputs go through a 4 KB staging tile per warp, 64 output columns at a time: each lane packs its row's 128 bytes into shared memory (16-byte units
      // XOR-swizzled by row), then the warp stores four whole 128-byte row segments per
      // instruction instead of 32 scattered 16-byte pieces.
      const bool swiglu = p.epilogue == B200_EPILOGUE_SWIGLU;
      const int out_cols = swiglu ? p.n / 2 : p.n;
      const bool staged = out_cols % 8 == 0 && (reinterpret_cast<uintptr_t>(p.out) & 15u) == 0;
      const int span = swiglu ? 128 : 64;  // accumulator columns that make 64 output columns
      const uint32_t stage_tile = smem_base + STAGES * kStageBytes + warp * 4096;
      const int row0 = tile_m * kBM + warp * 32;
#pragma unroll 1
      for (int c0 = 0; c0 < bn;) {
        const int col0 = tile_n * bn + c0;
        if (col0 >= n_end) break;  // warp-uniform
        if (staged && c0 + span <= bn && col0 + span <= n_end) {
          uint4 packed[8];
          if (swiglu) {
#pragma unroll
            for (int quarter = 0; quarter < 4; ++quarter) {
              float v[32], y[16];
              tmem_load_32x32(t_addr + c0 + quarter * 32, v);
              if (row < p.m) add_bias(p, col0 + quarter * 32, n_end, v);
              swiglu_of_chunk(v, y);
#pragma unroll
              for (int i = 0; i < 2; ++i)
                packed[quarter * 2 + i] =
                    make_uint4(pack_bf16x2(y[8 * i], y[8 * i + 1]), pack_bf16x2(y[8 * i + 2], y[8 * i + 3]),
                               pack_bf16x2(y[8 * i + 4], y[8 * i + 5]), pack_bf16x2(y[8 * i + 6], y[8 * i + 7]));
            }
          } else {
#pragma unroll
            for (int half = 0; half < 2; ++half) {
              float v[32];
              tmem_load_32x32(t_addr + c0 + half * 32, v);
              if (row < p.m) {
                add_bias(p, col0 + half * 32, n_end, v);
                add_residual(p, p.epilogue, row, col0 + half * 32, n_end, v);
              }
#pragma unroll
              for (int i = 0; i < 4; ++i)
                packed[half * 4 + i] =
                    make_uint4(pack_bf16x2(v[8 * i], v[8 * i + 1]), pack_bf16x2(v[8 * i + 2], v[8 * i + 3]),
                               pack_bf16x2(v[8 * i + 4], v[8 * i + 5]), pack_bf16x2(v[8 * i + 6], v[8 * i + 7]));
            }
          }
          __syncwarp();  // the previous round's reads of the staging tile are done
#pragma unroll
          for (int u = 0; u < 8; ++u)
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(
                             stage_tile + lane * 128 + ((u ^ (lane & 7)) << 4)),
                         "r"(packed[u].x), "r"(packed[u].y), "r"(packed[u].z), "r"(packed[u].w) : "memory");
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int r = i * 4 + (lane >> 3), u = lane & 7;
            uint4 value;
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(value.x), "=r"(value.y), "=r"(value.z), "=r"(value.w)
                         : "r"(stage_tile + r * 128 + ((u ^ (r & 7)) << 4)));
            if (row0 + r < p.m)
              *reinterpret_cast<uint4*>(p.out + static_cast<int64_t>(row0 + r) * out_cols +
                                        (swiglu ? col0 / 2 : col0) + u * 8) = value;
          }
          c0 += span;
        } else {
          float v[32];
          tmem_load_32x32(t_addr + c0, v);
          if (row < p.m) store_chunk(p, row, col0, n_end, v);
          c0 += 32;
        }
      }
      // the accumulator may be overwritten by the tile after next
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0)
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&acc_empty[acc])) : "memory");
    }
    if (!ok) failed = 1;
  }
  __syncwarp();
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (failed && threadIdx.x == 0 && p.status != nullptr) atomicOr(p.status, B200_STATUS_WAIT_TIMEOUT);
  if (warp == 5)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u)
                 : "memory");
  trace.mark(1);
}

int launch_persistent(const Tcgen05Params& p, const CUtensorMap& a_map, const CUtensorMap& b_map,
                      cudaStream_t stream) {
  // the stage ring, 4 KB of store staging per epilogue warp, alignment slack
  constexpr int smem = kPersistentStages * (kBM + kPersistentBN) * 128 + 4 * 4096 + 1024;
  static_assert(smem <= 227 * 1024, "stage ring exceeds shared memory");
  auto kernel = linear_tcgen05_persistent_kernel;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
    return B200_ERR_LAUNCH;
  if (p.bn <= 0 || p.bn > kPersistentBN || p.bn % 16 != 0) return B200_ERR_BAD_ARGUMENT;
  const int64_t tiles = ceil_div(p.n, p.bn) * ceil_div(p.m, kBM);
  dim3 grid(static_cast<unsigned>(tiles < kNumSMs ? tiles : kNumSMs));
  if (launch_chained(kernel, grid, dim3(kPersistentThreads), smem, stream, p, a_map, b_map) != cudaSuccess)
    return B200_ERR_LAUNCH;
  return launch_status();
}

struct PartialPlan {
  int bn, splits;
};

// Decode-size GEMMs with rings just deep enough for their K slice: the CTAs of the next kernel
// of the chain then fit on the SM beside them and run their set-up (and first weight fetches)
// early. B200_GEMM_RINGS=deep keeps the deep rings.
bool small_rings() {
  static const bool value = [] {
    const char* text = getenv("B200_GEMM_RINGS");
    return text == nullptr || strcmp(text, "deep") != 0;
  }();
  return value;
}

template <int BN, int STAGES, int A_ROWS, int FORM>
int launch(const Tcgen05Params& p, const CUtensorMap& a_map, const CUtensorMap& b_map,
           cudaStream_t stream) {
  // the instantiation must be the one the parameters describe
  if ((FORM == kFormCluster) != (p.epilogue == kEpilogueClusterResidual) ||
      (FORM == kFormPartial) != (p.epilogue == kEpiloguePartial) ||
      (FORM == kFormNorm || FORM == kFormNormSwiglu) != (p.norm_input != nullptr) ||
      (FORM == kFormNormSwiglu && p.epilogue != B200_EPILOGUE_SWIGLU) ||
      (FORM == kFormNorm && p.epilogue != B200_EPILOGUE_NONE))
    return B200_ERR_BAD_ARGUMENT;
  // slack: the last stage's 64-row x box is followed by up to 8 KB that the 128-row MMA reads past
  constexpr int ring = STAGES * (A_ROWS + BN) * 128 + 9216;
  static_assert(ring <= 227 * 1024, "stage ring exceeds shared memory");
  if (p.bn <= 0 || p.bn > BN || p.bn % 16 != 0) return B200_ERR_BAD_ARGUMENT;
  // cluster split-K: behind the ring, room for every slice's copy of the units this CTA owns
  int smem = ring;
  if (p.epilogue == kEpilogueClusterResidual) {
    const int owned = (A_ROWS * p.bn / 4 + p.splits - 1) / p.splits;
    if (owned > 4 * kThreads) return B200_ERR_UNSUPPORTED;
    smem += 2 * p.splits * owned * 16;  // a send and a receive region
    if (smem > 227 * 1024) return B200_ERR_UNSUPPORTED;
  }
  auto kernel = linear_tcgen05_kernel<BN, STAGES, A_ROWS, FORM>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
    return B200_ERR_LAUNCH;
  const int64_t tiles_n = ceil_div(p.n, p.bn), tiles_m = ceil_div(p.m, kBM);
  Tcgen05Params q = p;
  static const bool n_fastest_always = [] {  // B200_TILE_ORDER=n: the comparison run
    const char* text = getenv("B200_TILE_ORDER");
    return text != nullptr && strcmp(text, "n") == 0;
  }();
  // a decode-size launch whose W (at most 64 MB, with L2 to spare) is a constant
  static const bool l2_prefetch_off = [] {  // B200_WEIGHT_L2_PREFETCH=0: the comparison run
    const char* text = getenv("B200_WEIGHT_L2_PREFETCH");
    return text != nullptr && strcmp(text, "0") == 0;
  }();
  q.prefetch_l2 = !l2_prefetch_off && p.prefetch_weights && A_ROWS == 64 &&
                          static_cast<int64_t>(p.n) * p.k * 2 <= (64ll << 20) ? 1 : 0;
  q.m_fastest = !n_fastest_always && tiles_m >= 2 && tiles_m <= 16 && tiles_n <= 65535 &&
                        static_cast<int64_t>(p.n) * p.k * 2 > (64ll << 20) ? 1 : 0;
  dim3 grid(static_cast<unsigned>(q.m_fastest ? tiles_m : tiles_n),
            static_cast<unsigned>(q.m_fastest ? tiles_n : tiles_m), static_cast<unsigned>(p.splits));
  // the K slices of a tile are one thread-block cluster when they reduce among themselves
  const unsigned cluster_z = p.epilogue == kEpilogueClusterResidual ? static_cast<unsigned>(p.splits) : 1u;
  if (launch_chained_cluster_xz(kernel, grid, dim3(kThreads), smem, stream, 1u, cluster_z, q, a_map,
                                b_map) != cudaSuccess)
    return B200_ERR_LAUNCH;
  return launch_status();
}

// serve.linear proper: with or without the folded RMSNorm
template <int BN, int STAGES, int A_ROWS>
int launch_linear(const Tcgen05Params& p, const CUtensorMap& a_map, const CUtensorMap& b_map,
                  cudaStream_t stream) {
  if (p.norm_input == nullptr) return launch<BN, STAGES, A_ROWS, kFormPlain>(p, a_map, b_map, stream);
  return p.epilogue == B200_EPILOGUE_SWIGLU ? launch<BN, STAGES, A_ROWS, kFormNormSwiglu>(p, a_map, b_map, stream)
                                            : launch<BN, STAGES, A_ROWS, kFormNorm>(p, a_map, b_map, stream);
}

// How many clusters of `splits` CTAs of this kernel configuration the GPU holds at once (0 if the
// configuration cannot run). A cluster needs all its CTAs on one GPC, so the answer is not
// simply SMs / splits: 28 clusters of 5 one-CTA-per-SM blocks, for instance, do not fit.
template <int BN, int STAGES, int A_ROWS>
int resident_clusters(int bn, int splits) {
  const int owned = (A_ROWS * bn / 4 + splits - 1) / splits;
  const int smem = STAGES * (A_ROWS + BN) * 128 + 9216 + 2 * splits * owned * 16;
  if (owned > 4 * kThreads || smem > 227 * 1024) return 0;
  auto kernel = linear_tcgen05_kernel<BN, STAGES, A_ROWS, kFormCluster>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(1, 1, static_cast<unsigned>(splits));
  config.blockDim = dim3(kThreads);
  config.dynamicSmemBytes = smem;
  cudaLaunchAttribute attribute;
  attribute.id = cudaLaunchAttributeClusterDimension;
  attribute.val.clusterDim.x = 1;
  attribute.val.clusterDim.y = 1;
  attribute.val.clusterDim.z = static_cast<unsigned>(splits);
  config.attrs = &attribute;
  config.numAttrs = 1;
  int clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &config) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  return clusters;
}

// The kernel configuration the cluster split-K launcher uses for a tile width and slice length
// (rings short enough to leave room for the send and receive regions of the reduction).
enum class ClusterConfig { k32x3, k32x8, k64x4, k64x6, k128x4, k32x6r128, k64x4r128 };
ClusterConfig cluster_config(int a_rows, int bn, int64_t slice_blocks) {
  if (a_rows == 64) {
    if (bn <= 32) return small_rings() && slice_blocks <= 4 ? ClusterConfig::k32x3 : ClusterConfig::k32x8;
    if (bn <= 64) return small_rings() ? ClusterConfig::k64x4 : ClusterConfig::k64x6;
    return ClusterConfig::k128x4;
  }
  return bn <= 32 ? ClusterConfig::k32x6r128 : ClusterConfig::k64x4r128;
}
int resident_clusters_of(ClusterConfig config, int bn, int splits) {
  static int cache[7][129][9];  // 0 = not asked yet, else the answer + 1 (per device 0's shape)
  int& slot = cache[static_cast<int>(config)][bn][splits];
  if (slot == 0) {
    int value = 0;
    switch (config) {
      case ClusterConfig::k32x3: value = resident_clusters<32, 3, 64>(bn, splits); break;
      case ClusterConfig::k32x8: value = resident_clusters<32, 8, 64>(bn, splits); break;
      case ClusterConfig::k64x4: value = resident_clusters<64, 4, 64>(bn, splits); break;
      case ClusterConfig::k64x6: value = resident_clusters<64, 6, 64>(bn, splits); break;
      case ClusterConfig::k128x4: value = resident_clusters<128, 4, 64>(bn, splits); break;
      case ClusterConfig::k32x6r128: value = resident_clusters<32, 6, 128>(bn, splits); break;
      case ClusterConfig::k64x4r128: value = resident_clusters<64, 4, 128>(bn, splits); break;
    }
    slot = value + 1;
  }
  return slot - 1;
}

// Plan of the cluster split-K projection (M <= 128): N tile width and K slices (= cluster size,
// at most the portable 8) with about one CTA per SM. The cost of a candidate is what one CTA
// streams (k-blocks of its slice x stage bytes) plus a per-slice charge for the reduction.
PartialPlan plan_cluster(int64_t m, int64_t k, int64_t n) {
  static const char* forced = getenv("B200_SPLITK_PLAN");  // "bn,splits[,k]": experiments only
  if (forced != nullptr) {
    int bn = 0, splits = 0;
    long long only_k = 0;
    const int fields = sscanf(forced, "%d,%d,%lld", &bn, &splits, &only_k);
    if (fields >= 2 && (bn == 32 || bn == 64 || bn == 128) && splits >= 1 && splits <= 8 &&
        (fields < 3 || only_k == k))
      return PartialPlan{bn, splits};
  }
  const int64_t kb = ceil_div(k, kBK);
  PartialPlan best{64, 1};
  double best_cost = 1e300;
  const int64_t rows = m <= 64 ? 64 : 128;
  for (int bn : {32, 64, 128}) {
    if (rows * bn > 64 * 128) break;  // two copies of the fp32 tile must fit behind the ring
    const int64_t tiles = ceil_div(n, bn) * ceil_div(m, kBM);
    for (int64_t splits = 1; splits <= 8 && splits <= kb; ++splits) {
      if (tiles * splits > kNumSMs) break;
      // (the last slices may come out empty, e.g. 14 k-blocks over 8 slices of 2: such a CTA
      // ships zeros; 8 slices of at most 2 k-blocks measured faster than 4 slices of 4)
      const int64_t per = ceil_div(kb, splits);
      if (ceil_div(rows * bn / 4, splits) > 4 * kThreads) continue;  // units one CTA can own
      // every cluster resident at once: a second wave would double the time
      if (splits > 1 && resident_clusters_of(cluster_config(static_cast<int>(rows), bn, per), bn,
                                             static_cast<int>(splits)) < tiles)
        continue;
      // a thread that owns a second unit pays a second residual round trip after the barrier
      const int64_t rounds = ceil_div(ceil_div(rows * bn / 4, splits), kThreads);
      const double cost = static_cast<double>(per) * (64 + bn) + 6.0 * splits + 300.0 * (rounds - 1) +
                          (tiles * splits < 64 ? 1e6 : 0.0);  // far too few CTAs to stream at speed
      if (cost < best_cost) {
        best_cost = cost;
        best = PartialPlan{bn, static_cast<int>(splits)};
      }
    }
  }
  return best;
}

// Split-K plan of the partial-sum producer: N tile width and K slices chosen to put about
// one CTA on each of the 148 SMs at the least traffic (activation re-reads per N tile +
// fp32 partials written and read back per K slice).
PartialPlan plan_partial(int64_t m, int64_t k, int64_t n) {
  static const char* forced = getenv("B200_PARTIAL_PLAN");  // "bn,splits": experiments only
  if (forced != nullptr) {
    int bn = 0, splits = 0;
    if (sscanf(forced, "%d,%d", &bn, &splits) == 2 && (bn == 32 || bn == 64 || bn == 128) &&
        splits >= 1 && splits <= ceil_div(k, kBK))
      return PartialPlan{bn, splits};
  }
  const int64_t kb = ceil_div(k, kBK);
  PartialPlan best{128, 1};
  double best_cost = 1e300;
  for (int bn : {32, 64, 128}) {
    const int64_t tiles = ceil_div(n, bn);
    // A small weight matrix (the q|k|v projection of a 0.5B model: 2 MB) is fetched in a
    // couple of microseconds by a hundred CTAs; more K slices only add partials for the
    // consumer to sum (36 tiles x 3 slices measured 0.7 % of the decode step faster than x 4).
    const int64_t target = n * k * 2 <= (4ll << 20) ? kNumSMs * 3 / 4 : kNumSMs;
    int64_t splits = (target + tiles / 2) / tiles;
    if (splits < 1) splits = 1;
    if (splits > kb) splits = kb;
    const int64_t per = ceil_div(kb, splits);
    splits = ceil_div(kb, per);
    const double ctas = static_cast<double>(tiles * splits);
    const double bytes = static_cast<double>(tiles) * m * k * 2 + 2.0 * splits * m * n * 4;
    const double fill = ctas >= target ? 1.0 : ctas / target;
    const double cost = bytes / fill;
    if (cost < best_cost) {
      best_cost = cost;
      best = PartialPlan{bn, static_cast<int>(splits)};
    }
  }
  return best;
}

}  // namespace

// Called by b200_linear. Returns B200_ERR_UNSUPPORTED when this path does not apply (a
// tensor map cannot describe the operands, or a decode-size M with too few N tiles to fill
// the GPU without split-K), in which case the caller uses the warp-level kernel.
int linear_tcgen05(const void* input, const void* weight, const void* bias, const void* residual,
                   void* output, int64_t m, int64_t k, int64_t n, int64_t input_row_stride,
                   int epilogue, int32_t* status, cudaStream_t stream, bool fold_norm,
                   double norm_eps, const float* norm_squares, int norm_slices) {
  if (ceil_div(m, kBM) > 65535) return B200_ERR_UNSUPPORTED;
  if (fold_norm && m > 128) return B200_ERR_UNSUPPORTED;  // the idle-warp scheme: one or two rows a thread
  int bn;
  bool persistent = false;
  if (m > 64) {
    bn = n % 256 == 0 || n > 1024 ? 256 : 128;
    // A few M tiles (65 .. 1023 rows: large decode batches, short prefills) stream W rather than
    // reuse it: the widest tile that still gives about three quarters of the SMs a CTA, else the
    // narrowest (a 3584-column projection at 256 rows: 112 CTAs of 64 columns instead of 28 of 256).
    if (m < 1024) {
      const int64_t tiles_m = ceil_div(m, kBM);
      bn = 64;
      for (int candidate : {256, 128}) {
        if (ceil_div(n, candidate) * tiles_m >= kNumSMs * 3 / 4) {
          bn = candidate;
          break;
        }
      }
    }
    // From a few tiles per SM on, the persistent kernel (B200_LINEAR_PERSISTENT=0 keeps one tile
    // per CTA, for comparison). Its tile width is the multiple of 16 up to 256 that wastes the
    // fewest columns of the last N tile (896 -> 224, 1152 -> 192); 256 if that pads N by at most 1.5 %.
    const char* persistent_text = getenv("B200_LINEAR_PERSISTENT");
    if (m >= 1024 && (persistent_text == nullptr || strcmp(persistent_text, "0") != 0)) {
      persistent = true;
      int64_t least = -1;
      for (int candidate = 256; candidate >= 128; candidate -= 16) {
        const int64_t waste = ceil_div(n, candidate) * candidate - n;
        if (waste * 64 <= n) {  // the widest tile that pads N by at most 1.5 %
          bn = candidate;
          break;
        }
        if (least < 0 || waste < least) {
          least = waste;
          bn = candidate;
        }
      }
    }
  } else {
    // Weight streaming with one deep-pipelined CTA per SM: the N tile is the width (a
    // multiple of 16, at most 256) whose tile count fills whole waves of 148 CTAs best;
    // fewer than ~120 tiles would leave SMs idle and is left to the split-K kernel.
    // (a folded-norm call has no other kernel to fall back to: it runs here whatever the fill)
    if (!fold_norm && ceil_div(n, 16) < kNumSMs - 28) return B200_ERR_UNSUPPORTED;
    double best = -1.0;
    bn = 0;
    for (int candidate = 256; candidate >= 16; candidate -= 16) {
      const int64_t tiles = ceil_div(n, candidate);
      const int64_t waves = ceil_div(tiles, kNumSMs);
      const double fill = static_cast<double>(tiles) / static_cast<double>(waves * kNumSMs);
      // wider tiles re-read the activations less often: prefer them on (near) ties
      const double score = fill + 0.0002 * candidate;
      if (score > best) {
        best = score;
        bn = candidate;
      }
    }
    if (best < 0.8 && !fold_norm) return B200_ERR_UNSUPPORTED;
    // A folded-norm projection at decode sizes (gate|up: 17 MB of weights) is a chain of
    // latencies, not a stream: 64-column tiles with short rings put two or three CTAs on an SM,
    // whose ring round trips and two-warp SwiGLU epilogues overlap. Measured on the Qwen2-0.5B
    // step: 1.389 ms with 152 x 64 columns against 1.449 ms with 122 x 80 (one CTA per SM).
    if (fold_norm && small_rings()) {
      const int64_t tiles64 = ceil_div(n, 64);
      if (tiles64 >= kNumSMs - 28 && tiles64 <= 3 * kNumSMs) bn = 64;
    }
    if (fold_norm) {  // B200_FOLD_BN: tile width of the folded-norm projection (experiments only)
      static const int forced = [] {
        const char* text = getenv("B200_FOLD_BN");
        const int value = text != nullptr ? atoi(text) : 0;
        return value >= 16 && value <= 256 && value % 16 == 0 ? value : 0;
      }();
      if (forced != 0) bn = forced;
    }
    // Many waves of tiles (an LM head): 192-column tiles with a 3-stage ring leave room for two
    // CTAs per SM, so one CTA's ramp and epilogue hide under the other's streaming; measured
    // 60.2 us against 71.2 - 78.3 us for one 208 ... 256-column CTA per SM at N = 151936.
    if (ceil_div(n, 192) >= 4 * kNumSMs) bn = 192;
  }
  CUtensorMap a_map, b_map;
  if (!make_bf16_matrix_map(&a_map, input, m, k, input_row_stride, m <= 64 ? 64 : kBM) ||
      !make_bf16_matrix_map(&b_map, weight, n, k, k, bn))
    return B200_ERR_UNSUPPORTED;
  Tcgen05Params p;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.residual = static_cast<const __nv_bfloat16*>(residual);
  p.out = static_cast<__nv_bfloat16*>(output);
  p.partials = nullptr;
  p.status = status;
  p.m = static_cast<int>(m);
  p.k = static_cast<int>(k);
  p.n = static_cast<int>(n);
  p.epilogue = epilogue;
  p.splits = 1;
  p.bn = bn;
  p.prefetch_weights = (launch_mode() & B200_LAUNCH_CONSTANT_WEIGHTS) != 0 ? 1 : 0;
  p.wait_limit = wait_limit();
  p.drop_loads = drop_loads();
  if (fold_norm) {
    p.norm_input = static_cast<const __nv_bfloat16*>(input);
    p.norm_row_stride = input_row_stride;
    p.norm_eps = static_cast<float>(norm_eps);
    p.norm_squares = norm_slices > 0 ? norm_squares : nullptr;
    p.norm_slices = norm_slices;
  }
  if (m <= 64) {
    if (bn == 192 && ceil_div(n, 192) >= 4 * kNumSMs) return launch_linear<192, 3, 64>(p, a_map, b_map, stream);
    if (bn > 128) return launch_linear<256, 5, 64>(p, a_map, b_map, stream);
    if (bn > 64)
      return small_rings() && fold_norm ? launch_linear<128, 4, 64>(p, a_map, b_map, stream)
                                        : launch_linear<128, 8, 64>(p, a_map, b_map, stream);
    // narrow tiles of a folded-norm projection: short rings, three CTAs per SM
    // (4-stage rings measured best: 3 stages -4 %, 6 stages -2 %, 12 stages -17 % of the decode step)
    if (small_rings() && fold_norm)
      return bn > 32 ? launch_linear<64, 4, 64>(p, a_map, b_map, stream) : launch_linear<32, 4, 64>(p, a_map, b_map, stream);
    return launch_linear<64, 12, 64>(p, a_map, b_map, stream);
  }
  if (persistent) return launch_persistent(p, a_map, b_map, stream);
  if (bn == 256) return launch_linear<256, 4, 128>(p, a_map, b_map, stream);
  if (bn == 128) return launch_linear<128, 3, 128>(p, a_map, b_map, stream);
  return launch_linear<64, 4, 128>(p, a_map, b_map, stream);
}

int linear_partial_splits(int64_t m, int64_t k, int64_t n) { return plan_partial(m, k, n).splits; }

int linear_partial_tcgen05(const void* input, const void* weight, float* partials,
                           float* row_squares, int64_t m, int64_t k, int64_t n,
                           int64_t input_row_stride, int splits, int32_t* status,
                           cudaStream_t stream) {
  if (row_squares != nullptr && m > 128) return B200_ERR_UNSUPPORTED;
  const PartialPlan plan = plan_partial(m, k, n);
  const int a_rows = m <= 64 ? 64 : 128;
  CUtensorMap a_map, b_map;
  if (!make_bf16_matrix_map(&a_map, input, m, k, input_row_stride, a_rows) ||
      !make_bf16_matrix_map(&b_map, weight, n, k, k, plan.bn))
    return B200_ERR_UNSUPPORTED;
  Tcgen05Params p;
  p.bias = nullptr;
  p.residual = nullptr;
  p.out = nullptr;
  p.partials = partials;
  p.status = status;
  p.m = static_cast<int>(m);
  p.k = static_cast<int>(k);
  p.n = static_cast<int>(n);
  p.epilogue = kEpiloguePartial;
  p.splits = splits;
  p.row_squares = row_squares;
  p.bn = plan.bn;
  p.prefetch_weights = (launch_mode() & B200_LAUNCH_CONSTANT_WEIGHTS) != 0 ? 1 : 0;
  p.wait_limit = wait_limit();
  p.drop_loads = drop_loads();
  if (a_rows == 64) {
    // A K slice of many k-blocks is a long weight stream: it wants about 2 us x 44 GB/s of
    // loads in flight per SM, twice what the 96 KB rings of the short slices hold.
    const bool long_slice = ceil_div(ceil_div(k, kBK), splits) >= 24;
    if (plan.bn == 32)
      return small_rings() && ceil_div(ceil_div(k, kBK), splits) <= 4 ? launch<32, 4, 64, kFormPartial>(p, a_map, b_map, stream)
                                                                      : launch<32, 8, 64, kFormPartial>(p, a_map, b_map, stream);
    if (plan.bn == 64)
      return long_slice ? launch<64, 12, 64, kFormPartial>(p, a_map, b_map, stream) : launch<64, 6, 64, kFormPartial>(p, a_map, b_map, stream);
    return long_slice ? launch<128, 8, 64, kFormPartial>(p, a_map, b_map, stream) : launch<128, 4, 64, kFormPartial>(p, a_map, b_map, stream);
  }
  if (plan.bn == 32) return launch<32, 6, 128, kFormPartial>(p, a_map, b_map, stream);
  if (plan.bn == 64) return launch<64, 4, 128, kFormPartial>(p, a_map, b_map, stream);
  return launch<128, 3, 128, kFormPartial>(p, a_map, b_map, stream);
}

int linear_splitk_residual_tcgen05(const void* input, const void* weight, const void* residual,
                                   void* output, int64_t m, int64_t k, int64_t n,
                                   int64_t input_row_stride, int32_t* status, cudaStream_t stream,
                                   float* squares_out) {
  const PartialPlan plan = plan_cluster(m, k, n);
  const int a_rows = m <= 64 ? 64 : 128;
  // enough N x M tiles to fill the GPU without cutting K: the plain kernel with the residual epilogue
  if (plan.splits <= 1)
    return linear_tcgen05(input, weight, nullptr, residual, output, m, k, n, input_row_stride,
                          B200_EPILOGUE_RESIDUAL, status, stream, false, 0.0, nullptr, 0);
  CUtensorMap a_map, b_map;
  if (!make_bf16_matrix_map(&a_map, input, m, k, input_row_stride, a_rows) ||
      !make_bf16_matrix_map(&b_map, weight, n, k, k, plan.bn))
    return B200_ERR_UNSUPPORTED;
  Tcgen05Params p;
  p.bias = nullptr;
  p.residual = static_cast<const __nv_bfloat16*>(residual);
  p.out = static_cast<__nv_bfloat16*>(output);
  p.partials = nullptr;
  p.status = status;
  p.m = static_cast<int>(m);
  p.k = static_cast<int>(k);
  p.n = static_cast<int>(n);
  p.epilogue = kEpilogueClusterResidual;
  p.squares_out = squares_out;
  p.splits = plan.splits;
  p.bn = plan.bn;
  p.prefetch_weights = (launch_mode() & B200_LAUNCH_CONSTANT_WEIGHTS) != 0 ? 1 : 0;
  p.wait_limit = wait_limit();
  p.drop_loads = drop_loads();
  // (rings short enough to leave room for the send and receive regions of the reduction)
  switch (cluster_config(a_rows, plan.bn, ceil_div(ceil_div(k, kBK), plan.splits))) {
    case ClusterConfig::k32x3: return launch<32, 3, 64, kFormCluster>(p, a_map, b_map, stream);
    case ClusterConfig::k32x8: return launch<32, 8, 64, kFormCluster>(p, a_map, b_map, stream);
    case ClusterConfig::k64x4: return launch<64, 4, 64, kFormCluster>(p, a_map, b_map, stream);
    case ClusterConfig::k64x6: return launch<64, 6, 64, kFormCluster>(p, a_map, b_map, stream);
    case ClusterConfig::k128x4: return launch<128, 4, 64, kFormCluster>(p, a_map, b_map, stream);
    case ClusterConfig::k32x6r128: return launch<32, 6, 128, kFormCluster>(p, a_map, b_map, stream);
    case ClusterConfig::k64x4r128: return launch<64, 4, 128, kFormCluster>(p, a_map, b_map, stream);
  }
  return B200_ERR_UNSUPPORTED;
}

// Slices of row sums of squares that the cluster split-K projection leaves (N tiles x K slices);
// 0 when the shape runs without a cluster (then nothing is written).
int64_t linear_splitk_slices(int64_t m, int64_t k, int64_t n) {
  const PartialPlan plan = plan_cluster(m, k, n);
  return plan.splits <= 1 ? 0 : ceil_div(n, static_cast<int64_t>(plan.bn)) * plan.splits;
}

}  // namespace b200

using namespace b200;

extern "C" int64_t b200_linear_splitk_slices(int64_t m, int64_t k, int64_t n) {
  if (m <= 0 || m > 256 || k <= 0 || n <= 0) return 0;
  return linear_splitk_slices(m, k, n);
}

extern "C" int b200_linear_splitk_residual(const void* input, const void* weight,
                                           const void* residual, void* output,
                                           void* row_squares_out, int64_t m, int64_t k, int64_t n,
                                           int64_t input_row_stride, int32_t* status, void* stream) {
  if (!input || !weight || !residual || !output || m <= 0 || k <= 0 || n <= 0 ||
      input_row_stride < k)
    return B200_ERR_BAD_ARGUMENT;
  if (m > 256) return B200_ERR_TOO_LARGE;
  if (k % 8 != 0 || input_row_stride % 8 != 0 || n % 4 != 0) return B200_ERR_UNSUPPORTED;
  if (!aligned16(input) || !aligned16(weight) || !aligned16(residual) || !aligned16(output))
    return B200_ERR_ALIGNMENT;
  return linear_splitk_residual_tcgen05(input, weight, residual, output, m, k, n, input_row_stride,
                                        status, static_cast<cudaStream_t>(stream),
                                        static_cast<float*>(row_squares_out));
}

extern "C" int b200_linear_rms_input(const void* input, const void* folded_weight, const void* bias,
                                     void* output, const void* row_squares, int64_t row_square_slices,
                                     int64_t m, int64_t k, int64_t n, int64_t input_row_stride,
                                     double epsilon, int epilogue, int32_t* status, void* stream) {
  if (!input || !folded_weight || !output || m <= 0 || k <= 0 || n <= 0 || input_row_stride < k ||
      !(epsilon >= 0.0) || row_square_slices < 0 || row_square_slices > 65535 ||
      (row_square_slices > 0 && !row_squares))
    return B200_ERR_BAD_ARGUMENT;
  if (epilogue != B200_EPILOGUE_NONE && epilogue != B200_EPILOGUE_SWIGLU) return B200_ERR_BAD_ARGUMENT;
  if (epilogue == B200_EPILOGUE_SWIGLU && n % 2 != 0) return B200_ERR_BAD_ARGUMENT;
  if (m > 128) return B200_ERR_TOO_LARGE;
  if (k % 8 != 0 || input_row_stride % 8 != 0) return B200_ERR_UNSUPPORTED;
  if (!aligned16(input) || !aligned16(folded_weight)) return B200_ERR_ALIGNMENT;
  return linear_tcgen05(input, folded_weight, bias, nullptr, output, m, k, n, input_row_stride,
                        epilogue, status, static_cast<cudaStream_t>(stream), true, epsilon,
                        static_cast<const float*>(row_squares), static_cast<int>(row_square_slices));
}

extern "C" int64_t b200_linear_partial_splits(int64_t m, int64_t k, int64_t n) {
  if (m <= 0 || k <= 0 || n <= 0) return 0;
  return linear_partial_splits(m, k, n);
}

extern "C" int b200_linear_partial(const void* input, const void* weight, void* partials,
                                   void* row_squares, int64_t m, int64_t k, int64_t n,
                                   int64_t input_row_stride, int64_t splits, int32_t* status,
                                   void* stream) {
  if (!input || !weight || !partials || m <= 0 || k <= 0 || n <= 0 || input_row_stride < k ||
      splits <= 0)
    return B200_ERR_BAD_ARGUMENT;
  if (m > 128 || splits > ceil_div(k, kBK) || splits > 65535) return B200_ERR_TOO_LARGE;
  if (k % 8 != 0 || input_row_stride % 8 != 0 || n % 4 != 0) return B200_ERR_UNSUPPORTED;
  if (!aligned16(input) || !aligned16(weight) || !aligned16(partials)) return B200_ERR_ALIGNMENT;
  if (row_squares != nullptr && m > 128) return B200_ERR_TOO_LARGE;
  return linear_partial_tcgen05(input, weight, static_cast<float*>(partials),
                                static_cast<float*>(row_squares), m, k, n, input_row_stride,
                                static_cast<int>(splits), status, static_cast<cudaStream_t>(stream));
}
