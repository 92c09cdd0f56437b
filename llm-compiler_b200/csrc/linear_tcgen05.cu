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

struct Tcgen05Params {
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual;
  __nv_bfloat16* out;
  float* partials;  // [splits, m, n] fp32 when epilogue == kEpiloguePartial
  int32_t* status;
  int m, k, n, epilogue, splits;
  int bn;  // columns per tile: a multiple of 16, at most the kernel's BN
  int prefetch_weights;  // W tiles may be fetched before the predecessor kernel has finished
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
__device__ __forceinline__ void add_residual(const Tcgen05Params& p, int row, int col0, int n_end,
                                             float (&v)[32]) {
  const bool whole = col0 + 32 <= n_end;
  const int64_t o = static_cast<int64_t>(row) * p.n + col0;
  if (p.epilogue == B200_EPILOGUE_RESIDUAL) {  // r(r(x W^T + b) + residual)
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
__device__ __forceinline__ void store_chunk(const Tcgen05Params& p, int row, int col0, int n_end,
                                            float (&v)[32]) {
  const int out_cols = p.epilogue == B200_EPILOGUE_SWIGLU ? p.n / 2 : p.n;
  const bool whole = col0 + 32 <= n_end;  // all 32 columns exist: 16-byte accesses where aligned
  add_bias(p, col0, n_end, v);
  if (p.epilogue == B200_EPILOGUE_SWIGLU) {
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
  add_residual(p, row, col0, n_end, v);
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
template <int BN, int STAGES, int A_ROWS>
__global__ void __launch_bounds__(kThreads)
linear_tcgen05_kernel(const Tcgen05Params p, const __grid_constant__ CUtensorMap a_map,
                      const __grid_constant__ CUtensorMap b_map) {
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
  __shared__ uint32_t tmem_base_slot;
  __shared__ int failed;

  TraceScope trace(1);
  grid_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile_n = blockIdx.x, tile_m = blockIdx.y, split = blockIdx.z;
  const int kb_total = (p.k + kBK - 1) / kBK;
  const int kb_per = (kb_total + p.splits - 1) / p.splits;
  const int kb_first = split * kb_per;
  const int nkb = max(0, min(kb_first + kb_per, kb_total) - kb_first);
  const uint32_t smem_base = smem_u32(smem);

  if (threadIdx.x == 0) {
    failed = 0;
#pragma unroll
    for (int s = 0; s < STAGES; ++s) {
      mbarrier_init(smem_u32(&full_bar[s]), 1);
      mbarrier_init(smem_u32(&empty_bar[s]), 1);
    }
    mbarrier_init(smem_u32(&accum_bar), 1);
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

  if (warp == 0 && lane == 0) {
    // ---- TMA producer ----
    // The first ring of W tiles does not depend on the kernel before this one: fetch it
    // before waiting for that kernel (the transaction bytes are announced without arriving,
    // so a stage cannot complete before its x box has been requested as well).
    const int early = p.prefetch_weights ? min(nkb, STAGES) : 0;
    for (int kb = 0; kb < early; ++kb) {
      const uint32_t bar = smem_u32(&full_bar[kb]);
      mbarrier_expect_tx(bar, static_cast<uint32_t>(bn * 128));
      tma_load_2d(smem_base + kb * kStageBytes + kABytes, &b_map, bar, (kb_first + kb) * kBK,
                  tile_n * bn);
    }
    grid_dependency_wait();
    trace.mark(0);
    for (int kb = 0; kb < nkb; ++kb) {
      const int s = kb % STAGES;
      if (kb >= STAGES &&
          !mbarrier_wait_bounded(smem_u32(&empty_bar[s]), ((kb / STAGES) - 1) & 1)) {
        failed = 1;
        break;
      }
      const uint32_t bar = smem_u32(&full_bar[s]);
      const uint32_t a_dst = smem_base + s * kStageBytes;
      if (kb < early) {
        mbarrier_arrive_expect_tx(bar, static_cast<uint32_t>(kABytes));
        tma_load_2d(a_dst, &a_map, bar, (kb_first + kb) * kBK, tile_m * kBM);
      } else {
        mbarrier_arrive_expect_tx(bar, stage_tx_bytes);
        tma_load_2d(a_dst, &a_map, bar, (kb_first + kb) * kBK, tile_m * kBM);
        tma_load_2d(a_dst + kABytes, &b_map, bar, (kb_first + kb) * kBK, tile_n * bn);
      }
    }
  } else if (warp == 1 && lane == 0) {
    // The MMA issuer waits too (a K slice without k-blocks has no TMA copy to order it after
    // the producer's wait). The other threads only ever act on what these three hand them
    // through mbarriers, and stay out of the way of the kernels still running on the SM.
    grid_dependency_wait();
  }
  if (warp == 1 && lane == 0) {
    // ---- MMA issuer ----
    for (int kb = 0; kb < nkb; ++kb) {
      const int s = kb % STAGES;
      if (!mbarrier_wait_bounded(smem_u32(&full_bar[s]), (kb / STAGES) & 1)) {
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
  bool ok = mbarrier_wait_bounded(smem_u32(&accum_bar), 0);
  trace.mark_middle();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  ok = ok && failed == 0;
  if (ok) {
    const int row = tile_m * kBM + warp * 32 + lane;
#pragma unroll 1
    const int n_end = min(p.n, (tile_n + 1) * bn);  // columns of this tile
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
      if (p.epilogue == kEpiloguePartial) {
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
      store_chunk(p, row, col0, n_end, v);
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

  if (warp == 4 && lane == 0) {
    // ---- TMA producer ----
    grid_dependency_wait();
    int round = 0;  // k-blocks issued so far, over all tiles
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < tiles; tile += gridDim.x) {
      const int tile_n = tile % tiles_n, tile_m = tile / tiles_n;
      for (int kb = 0; kb < nkb; ++kb, ++round) {
        const int s = round % STAGES;
        if (round >= STAGES &&
            !mbarrier_wait_bounded(smem_u32(&empty_bar[s]), ((round / STAGES) - 1) & 1)) {
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
      if (local >= 2 && !mbarrier_wait_bounded(smem_u32(&acc_empty[acc]), ((local >> 1) - 1) & 1)) {
        ok = false;
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t d_tmem = tmem_base + acc * kPersistentBN;
      for (int kb = 0; kb < nkb; ++kb, ++round) {
        const int s = round % STAGES;
        if (!mbarrier_wait_bounded(smem_u32(&full_bar[s]), (round / STAGES) & 1)) {
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
      ok = ok && __all_sync(0xffffffffu, mbarrier_wait_bounded(smem_u32(&acc_full[acc]), (local >> 1) & 1));
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
                add_residual(p, row, col0 + half * 32, n_end, v);
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

template <int BN, int STAGES, int A_ROWS>
int launch(const Tcgen05Params& p, const CUtensorMap& a_map, const CUtensorMap& b_map,
           cudaStream_t stream) {
  // slack: the last stage's 64-row x box is followed by up to 8 KB that the 128-row MMA reads past
  constexpr int smem = STAGES * (A_ROWS + BN) * 128 + 9216;
  static_assert(smem <= 227 * 1024, "stage ring exceeds shared memory");
  auto kernel = linear_tcgen05_kernel<BN, STAGES, A_ROWS>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
    return B200_ERR_LAUNCH;
  if (p.bn <= 0 || p.bn > BN || p.bn % 16 != 0) return B200_ERR_BAD_ARGUMENT;
  dim3 grid(static_cast<unsigned>(ceil_div(p.n, p.bn)), static_cast<unsigned>(ceil_div(p.m, kBM)),
            static_cast<unsigned>(p.splits));
  if (launch_chained(kernel, grid, dim3(kThreads), smem, stream, p, a_map, b_map) != cudaSuccess)
    return B200_ERR_LAUNCH;
  return launch_status();
}

// Split-K plan of the partial-sum producer: N tile width and K slices chosen to put about
// one CTA on each of the 148 SMs at the least traffic (activation re-reads per N tile +
// fp32 partials written and read back per K slice).
struct PartialPlan {
  int bn, splits;
};

PartialPlan plan_partial(int64_t m, int64_t k, int64_t n) {
  const int64_t kb = ceil_div(k, kBK);
  PartialPlan best{128, 1};
  double best_cost = 1e300;
  for (int bn : {32, 64, 128}) {
    const int64_t tiles = ceil_div(n, bn);
    int64_t splits = (kNumSMs + tiles / 2) / tiles;
    if (splits < 1) splits = 1;
    if (splits > kb) splits = kb;
    const int64_t per = ceil_div(kb, splits);
    splits = ceil_div(kb, per);
    const double ctas = static_cast<double>(tiles * splits);
    const double bytes = static_cast<double>(tiles) * m * k * 2 + 2.0 * splits * m * n * 4;
    const double fill = ctas >= kNumSMs ? 1.0 : ctas / kNumSMs;
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
                   int epilogue, int32_t* status, cudaStream_t stream) {
  if (ceil_div(m, kBM) > 65535) return B200_ERR_UNSUPPORTED;
  int bn;
  bool persistent = false;
  if (m > 64) {
    bn = n % 256 == 0 || n > 1024 ? 256 : 128;
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
    if (ceil_div(n, 16) < kNumSMs - 28) return B200_ERR_UNSUPPORTED;
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
    if (best < 0.8) return B200_ERR_UNSUPPORTED;
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
  if (m <= 64) {
    if (bn == 192 && ceil_div(n, 192) >= 4 * kNumSMs) return launch<192, 3, 64>(p, a_map, b_map, stream);
    if (bn > 128) return launch<256, 5, 64>(p, a_map, b_map, stream);
    if (bn > 64) return launch<128, 8, 64>(p, a_map, b_map, stream);
    return launch<64, 12, 64>(p, a_map, b_map, stream);
  }
  if (persistent) return launch_persistent(p, a_map, b_map, stream);
  if (bn == 256) return launch<256, 4, 128>(p, a_map, b_map, stream);
  if (bn == 128) return launch<128, 3, 128>(p, a_map, b_map, stream);
  return launch<64, 4, 128>(p, a_map, b_map, stream);
}

int linear_partial_splits(int64_t m, int64_t k, int64_t n) { return plan_partial(m, k, n).splits; }

int linear_partial_tcgen05(const void* input, const void* weight, float* partials, int64_t m,
                           int64_t k, int64_t n, int64_t input_row_stride, int splits,
                           int32_t* status, cudaStream_t stream) {
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
  p.bn = plan.bn;
  p.prefetch_weights = (launch_mode() & B200_LAUNCH_CONSTANT_WEIGHTS) != 0 ? 1 : 0;
  if (a_rows == 64) {
    // A K slice of many k-blocks is a long weight stream: it wants about 2 us x 44 GB/s of
    // loads in flight per SM, twice what the 96 KB rings of the short slices hold.
    const bool long_slice = ceil_div(ceil_div(k, kBK), splits) >= 24;
    if (plan.bn == 32) return launch<32, 8, 64>(p, a_map, b_map, stream);
    if (plan.bn == 64)
      return long_slice ? launch<64, 12, 64>(p, a_map, b_map, stream) : launch<64, 6, 64>(p, a_map, b_map, stream);
    return long_slice ? launch<128, 8, 64>(p, a_map, b_map, stream) : launch<128, 4, 64>(p, a_map, b_map, stream);
  }
  if (plan.bn == 32) return launch<32, 6, 128>(p, a_map, b_map, stream);
  if (plan.bn == 64) return launch<64, 4, 128>(p, a_map, b_map, stream);
  return launch<128, 3, 128>(p, a_map, b_map, stream);
}

}  // namespace b200

using namespace b200;

extern "C" int64_t b200_linear_partial_splits(int64_t m, int64_t k, int64_t n) {
  if (m <= 0 || k <= 0 || n <= 0) return 0;
  return linear_partial_splits(m, k, n);
}

extern "C" int b200_linear_partial(const void* input, const void* weight, void* partials,
                                   int64_t m, int64_t k, int64_t n, int64_t input_row_stride,
                                   int64_t splits, int32_t* status, void* stream) {
  if (!input || !weight || !partials || m <= 0 || k <= 0 || n <= 0 || input_row_stride < k ||
      splits <= 0)
    return B200_ERR_BAD_ARGUMENT;
  if (m > 128 || splits > ceil_div(k, kBK) || splits > 65535) return B200_ERR_TOO_LARGE;
  if (k % 8 != 0 || input_row_stride % 8 != 0 || n % 4 != 0) return B200_ERR_UNSUPPORTED;
  if (!aligned16(input) || !aligned16(weight) || !aligned16(partials)) return B200_ERR_ALIGNMENT;
  return linear_partial_tcgen05(input, weight, static_cast<float*>(partials), m, k, n,
                                input_row_stride, static_cast<int>(splits), status,
                                static_cast<cudaStream_t>(stream));
}
