// GQA decode attention over the physical B x C x Hkv x D KV buffers with per-sequence
// device lengths: split-KV online softmax.
//
// bf16 kernel. Grid (split, kv-head block, batch). A CTA owns one (sequence, KV head,
// split of `split_tokens` tokens) and serves ALL grouped query heads of that KV head
// from one read of K and V: the G query heads are the M rows (padded to 16) of
// warp-level tensor-core tiles, S = Q K^T and O += P V. The CTA's 4 warps take
// interleaved sub-tiles of 32 tokens (16 at head_dim 128); each warp streams its own
// sub-tiles through a private 3-stage ring in shared memory, so the main loop has no
// CTA-wide barrier. The ring is filled by TMA: one elected lane issues one tensor-map box
// copy for K and one for V per stage (128-byte swizzled rows, completion on a per-stage
// mbarrier, every wait bounded); a 16-byte cp.async path with the same layout is kept as
// the variant for buffers a tensor map cannot describe. Loop bounds come from lengths[b]
// on the device, never from the capacity. The softmax keeps the running maximum in the
// raw-score domain (one FFMA + ex2 per probability) and rescales O only when a maximum
// actually moved. Warps merge their (max, sum, O) partials through shared memory; with
// more than one split the CTA parks an fp32 partial in the workspace and the CTA that
// arrives last at the (sequence, head block) counter combines the splits in order.
//
// Algorithmic traffic per call: every valid K and V byte once (2 * len * Hkv * D * 2 B
// per sequence) + Q + O; the split partials add 4*(D+2) bytes per (q head, split).
#include <cuda.h>

#include <algorithm>
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include "common.cuh"
#include "tensor_map.cuh"

namespace b200 {
namespace {

constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;
constexpr int kStages = 3;
constexpr float kLog2e = 1.4426950408889634f;
constexpr int64_t kCounterBytes = 65536;  // fixed region: calls of any shape share a workspace
constexpr int64_t kMaxCounters = kCounterBytes / 4;

struct DecodeParams {
  const __nv_bfloat16* q;
  const __nv_bfloat16* kbuf;
  const __nv_bfloat16* vbuf;
  const int64_t* lengths;
  const void* mask;
  __nv_bfloat16* out;
  float* ws_o;    // [B, Hq, splits, D]
  float* ws_ml;   // [B, Hq, splits, 2]  (max in log2 domain, sum)
  int* counters;  // [B * head blocks], zero between calls; nullptr = separate merge kernel
  int32_t* status;
  int64_t q_batch_stride, q_head_stride, mask_batch_stride;
  int batch, q_heads, kv_heads, groups, capacity, mask_len, split_tokens, num_splits;
  int mask_dtype;  // B200_F32 / B200_BF16
  int compat;      // keep the reference's bf16 rounding of the scores
  int early_kv;    // lengths[] and the KV rows below lengths[b] - 1 are stable: fetch before the wait
  float scale;
  // Fused form (qkv_partials != nullptr): q, and the K/V row of the newest token, are not read
  // from memory but reduced here from the fp32 split-K partials [qkv_splits, B, (Hq + 2 Hkv) D]
  // of the fused q|k|v projection (+ bias, RoPE); the newest row (index lengths[b] - 1) is
  // stored into the KV buffers by the CTA that owns it and joins the softmax from registers.
  const float* qkv_partials = nullptr;
  const __nv_bfloat16* qkv_bias = nullptr;
  const __nv_bfloat16* cosine = nullptr;  // [B, D]
  const __nv_bfloat16* sine = nullptr;
  __nv_bfloat16* kstore = nullptr;  // the KV buffers again, writable
  __nv_bfloat16* vstore = nullptr;
  int qkv_splits = 0;
  // RMSNorm folded into the q|k|v projection (norm_row_squares != nullptr): the partials are
  // products of the un-normalised hidden rows x [B, norm_hidden] with norm-weight-scaled
  // projection weights, norm_row_squares[qkv_splits, B] holds sum(x_b^2) per K slice; the
  // reduced sums are scaled by rsqrt(mean(x_b^2) + norm_eps) before the bias.
  const float* norm_row_squares = nullptr;
  // Fused form: lengths[] may still hold the lengths BEFORE the new token (the caller advances
  // every slot once at the end of the step): the attention length is lengths[b] + length_bias.
  int length_bias = 0;
  // Paged layout (block_table != nullptr): kbuf / vbuf are block pools [blocks, block_size, Hkv,
  // D]; token t of sequence b lives in block block_table[b * table_stride + t / block_size] at
  // row t % block_size. block_size is a multiple of the tokens a warp copies per step, so a copy
  // never straddles two blocks. `capacity` is then table_stride * block_size.
  const int32_t* block_table = nullptr;
  // order != nullptr: grid z = i serves sequence order[i] (a permutation of 0 .. batch-1). CTAs
  // are placed in grid order, so a caller that lists the longest sequences first gets
  // longest-first scheduling when the grid is several waves of CTAs.
  const int32_t* order = nullptr;
  int block_size = 0, table_stride = 0;
  int64_t pool_rows = 0;  // blocks x block_size: the extent of the pools' tensor maps
  uint32_t wait_limit = 4000000u;  // polls of a bounded wait
  int drop_loads = 0;              // debug: no KV copy is issued (every wait runs out)
  int norm_hidden = 0;
  float norm_eps = 0.0f;
};

// No-op hook of stream_segment.
struct NoPrepare {
  __device__ __forceinline__ void operator()() const {}
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float load_mask(const void* mask, int dtype, int64_t index) {
  if (dtype == B200_F32) return static_cast<const float*>(mask)[index];
  if (dtype == B200_F16) return __half2float(static_cast<const __half*>(mask)[index]);
  return __bfloat162float(static_cast<const __nv_bfloat16*>(mask)[index]);
}

// A tile of TOK rows x D bf16 is stored as D/64 panels of [TOK][64] (128-byte rows), the
// 16-byte chunk index XOR-ed with (row & 7): the layout a 128B-swizzled TMA box produces.
template <int TOK>
__device__ __forceinline__ uint32_t tile_offset(int row, int chunk) {
  return static_cast<uint32_t>((chunk >> 3) * (TOK * 128) + row * 128 +
                               (((chunk ^ row) & 7) << 4));
}

// FAST: no mask and fast numerics (the serving engine's case); otherwise mask and the
// compatible rounding are runtime flags.
// Streams tokens [start, end) of one (sequence, KV head) through the CTA: the 4 warps take
// interleaved TOK-token sub-tiles, each through its own ring (stage index and mbarrier parity
// continue from `it_base`, which is per warp and advanced here), and leave their partial
// (max in the log2 domain, sum, O) in their ring regions; ends with a CTA barrier. Returns
// false when a bounded wait gave up.
// `prepare` runs (all threads, may synchronise the CTA) after the dependency wait and before the
// query fragments are read from `qbase` (row stride `q_row_stride` elements; global or shared).
template <int D, int TOK, bool WIDE, bool FAST, bool TMA, typename Prepare = NoPrepare,
          int WARPS = kWarps>
__device__ __forceinline__ bool stream_segment(const DecodeParams& p, const CUtensorMap& kmap,
                                               const CUtensorMap& vmap, unsigned char* smem,
                                               uint32_t bar0, int b, int kvh, int g0, int rows,
                                               int start, int end, int& it_base,
                                               int stable_end = -1, TraceScope* trace = nullptr,
                                               const __nv_bfloat16* qbase = nullptr,
                                               int64_t q_row_stride = 0,
                                               Prepare prepare = Prepare()) {
  constexpr int kChunksPerRow = D / 8;
  constexpr int kTileBytes = TOK * D * 2;  // one of K or V, one stage
  constexpr int kStageBytes = 2 * kTileBytes;
  constexpr int kWarpBytes = kStages * kStageBytes;
  constexpr int kCopiesPerLane = TOK * kChunksPerRow / 32;
  constexpr int kKSteps = D / 16;
  constexpr int kNTiles = D / 8;
  constexpr int kSTiles = TOK / 8;  // score n-tiles per step
  constexpr int kRows = WIDE ? 2 : 1;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int it0 = it_base;

  const uint32_t warp_smem = smem_u32(smem) + warp * kWarpBytes;
  const int64_t token_stride = static_cast<int64_t>(p.kv_heads) * D;
  const __nv_bfloat16* kglob = p.kbuf + (static_cast<int64_t>(b) * p.capacity * p.kv_heads + kvh) * D;
  const __nv_bfloat16* vglob = p.vbuf + (static_cast<int64_t>(b) * p.capacity * p.kv_heads + kvh) * D;
  // first buffer row of the TOK tokens that start at token t0 of this sequence
  auto first_row = [&](int t0) -> int64_t {
    if (p.block_table == nullptr) return static_cast<int64_t>(b) * p.capacity + t0;
    const int block = __ldg(p.block_table + static_cast<int64_t>(b) * p.table_stride + t0 / p.block_size);
    return static_cast<int64_t>(block) * p.block_size + t0 % p.block_size;
  };

  // sub-tile j of this split covers tokens start + j*TOK ...; warp w owns j = w, w+4, ...
  const int n_sub = (end - start + TOK - 1) / TOK;
  const int my_count = n_sub > warp ? (n_sub - warp + WARPS - 1) / WARPS : 0;

  // per-lane constants of the cp.async variant: this lane's rows / chunks inside a sub-tile
  uint32_t lane_soff[TMA ? 1 : kCopiesPerLane];
  int64_t lane_goff[TMA ? 1 : kCopiesPerLane];
  int lane_row[TMA ? 1 : kCopiesPerLane];
  if (!TMA) {
#pragma unroll
    for (int i = 0; i < kCopiesPerLane; ++i) {
      const int id = i * 32 + lane;
      const int r = id / kChunksPerRow, c = id % kChunksPerRow;
      lane_row[i] = r;
      lane_soff[i] = tile_offset<TOK>(r, c);
      lane_goff[i] = r * token_stride + c * 8;
    }
  }

  auto issue_load = [&](int it) {
    const int t0 = start + (it * WARPS + warp) * TOK;
    const uint32_t kdst = warp_smem + ((it0 + it) % kStages) * kStageBytes;
    const uint32_t vdst = kdst + kTileBytes;
    if (TMA) {
      if (lane == 0 && !p.drop_loads) {
        const uint32_t bar = bar0 + ((it0 + it) % kStages) * 8;
        mbarrier_arrive_expect_tx(bar, kStageBytes);
        // (rows past the tensor end are zero-filled; t0 < end <= capacity, so a paged lookup
        // stays inside the sequence's row of the block table)
        const int row = static_cast<int>(first_row(t0));
#pragma unroll
        for (int panel = 0; panel < D / 64; ++panel) {
          tma_load_3d(kdst + panel * (TOK * 128), &kmap, bar, panel * 64, kvh, row);
          tma_load_3d(vdst + panel * (TOK * 128), &vmap, bar, panel * 64, kvh, row);
        }
      }
    } else {
      const int64_t row0 = first_row(t0) - static_cast<int64_t>(b) * p.capacity;  // relative to kglob
      const __nv_bfloat16* ksrc = kglob + row0 * token_stride;
      const __nv_bfloat16* vsrc = vglob + row0 * token_stride;
      if (t0 + TOK <= end) {
#pragma unroll
        for (int i = 0; i < kCopiesPerLane; ++i) {
          cp_async16(kdst + lane_soff[i], ksrc + lane_goff[i]);
          cp_async16(vdst + lane_soff[i], vsrc + lane_goff[i]);
        }
      } else {
#pragma unroll
        for (int i = 0; i < kCopiesPerLane; ++i) {
          const bool valid = t0 + lane_row[i] < end;
          cp_async16_zfill(kdst + lane_soff[i], valid ? ksrc + lane_goff[i] : kglob, valid ? 16 : 0);
          cp_async16_zfill(vdst + lane_soff[i], valid ? vsrc + lane_goff[i] : vglob, valid ? 16 : 0);
        }
      }
    }
  };

  // running max: raw-score domain when FAST, log2 domain otherwise (rows r0, r0 + 8)
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.0f, 0.0f};  // this thread's share of the running sum
  float oacc[kNTiles][4];
#pragma unroll
  for (int i = 0; i < kNTiles; ++i)
    oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.0f;

  const float scale_log2 = p.scale * kLog2e;
  const float softmax_scale = FAST ? scale_log2 : 1.0f;
  bool timed_out = false;

  // Pipeline prologue. With stable_end >= 0 (the caller vouches that lengths[] and the KV rows
  // below stable_end are written by no kernel still running) the sub-tiles that end at or
  // below it are requested BEFORE the dependency wait, so the ring is full when the kernel
  // before this one finishes; the query, and any sub-tile that may hold the newest row, come
  // after the wait.
  uint32_t requested = 0;
  if (TMA && stable_end > 0) {
#pragma unroll
    for (int s = 0; s < kStages - 1; ++s)
      if (s < my_count && start + (s * WARPS + warp + 1) * TOK <= stable_end) {
        issue_load(s);
        requested |= 1u << s;
      }
  }
  if (stable_end >= 0) {
    grid_dependency_wait_cta();
    if (trace != nullptr) trace->mark(0);
  }

  // ---- Q fragments straight from global memory (A operand, 16 x D, rows = q heads) ----
  uint32_t qa[kKSteps][4];
  {
    const int r0 = lane >> 2;
    const int col = (lane & 3) * 2;
    prepare();
    if (qbase == nullptr) {
      qbase = p.q + b * p.q_batch_stride + static_cast<int64_t>(kvh * p.groups + g0) * p.q_head_stride;
      q_row_stride = p.q_head_stride;
    }
#pragma unroll
    for (int ks = 0; ks < kKSteps; ++ks) {
      const int c0 = ks * 16 + col;
      qa[ks][0] = r0 < rows ? *reinterpret_cast<const uint32_t*>(qbase + r0 * q_row_stride + c0) : 0u;
      qa[ks][2] = r0 < rows ? *reinterpret_cast<const uint32_t*>(qbase + r0 * q_row_stride + c0 + 8) : 0u;
      if (WIDE) {
        qa[ks][1] = r0 + 8 < rows ? *reinterpret_cast<const uint32_t*>(qbase + (r0 + 8) * q_row_stride + c0) : 0u;
        qa[ks][3] = r0 + 8 < rows ? *reinterpret_cast<const uint32_t*>(qbase + (r0 + 8) * q_row_stride + c0 + 8) : 0u;
      } else {
        qa[ks][1] = 0u;
        qa[ks][3] = 0u;
      }
    }
  }

#pragma unroll
  for (int s = 0; s < kStages - 1; ++s) {
    if (s < my_count && !(requested & (1u << s))) issue_load(s);
    if (!TMA) cp_async_commit();
  }

  for (int it = 0; it < my_count; ++it) {
    if (TMA) {
      if (!mbarrier_wait_bounded(bar0 + ((it0 + it) % kStages) * 8, ((it0 + it) / kStages) & 1, p.wait_limit)) {
        timed_out = true;
        break;
      }
    } else {
      cp_async_wait<kStages - 2>();
    }
    __syncwarp();  // every lane is done reading the stage that is refilled next
    if (it + kStages - 1 < my_count) issue_load(it + kStages - 1);
    if (!TMA) cp_async_commit();

    const int t0 = start + (it * WARPS + warp) * TOK;
    const uint32_t ksm = warp_smem + ((it0 + it) % kStages) * kStageBytes;
    const uint32_t vsm = ksm + kTileBytes;
    const bool partial = t0 + TOK > end;

    if (TMA && partial) {
      // a box copy brings whole rows: rows past `end` hold whatever the buffer holds, and a
      // non-finite V there would poison 0 * V. Zero them (K is masked by score instead).
      for (int id = lane; id < TOK * kChunksPerRow; id += 32) {
        const int r = id / kChunksPerRow, c = id % kChunksPerRow;
        if (t0 + r >= end)
          *reinterpret_cast<uint4*>(smem + (vsm - smem_u32(smem)) + tile_offset<TOK>(r, c)) =
              make_uint4(0, 0, 0, 0);
      }
      __syncwarp();
    }

    // ---- S = Q K^T : 16 x TOK ----
    float sacc[kSTiles][4];
#pragma unroll
    for (int i = 0; i < kSTiles; ++i) sacc[i][0] = sacc[i][1] = sacc[i][2] = sacc[i][3] = 0.0f;
    {
      const int mat = lane >> 3;
      const int krow = ((mat >> 1) << 3) + (lane & 7);
#pragma unroll
      for (int ks = 0; ks < kKSteps; ++ks) {
#pragma unroll
        for (int np = 0; np < kSTiles / 2; ++np) {
          uint32_t kb[4];
          ldmatrix_x4(kb, ksm + tile_offset<TOK>(np * 16 + krow, ks * 2 + (mat & 1)));
          mma_bf16_16816(sacc[np * 2], qa[ks], kb[0], kb[1]);
          mma_bf16_16816(sacc[np * 2 + 1], qa[ks], kb[2], kb[3]);
        }
      }
    }

    // ---- scores -> softmax domain, tail masking ----
    if (!FAST) {
#pragma unroll
      for (int nt = 0; nt < kSTiles; ++nt) {
#pragma unroll
        for (int e = 0; e < 2 * kRows; ++e) {
          const int token = t0 + nt * 8 + (lane & 3) * 2 + (e & 1);
          float s;
          if (p.compat)  // reference order: r(q k^T) -> r(. * scale) -> fp32 (+ mask)
            s = round_bf16(round_bf16(sacc[nt][e]) * p.scale) * kLog2e;
          else
            s = sacc[nt][e] * scale_log2;
          if (token < end) {
            if (p.mask != nullptr)
              s += load_mask(p.mask, p.mask_dtype, b * p.mask_batch_stride + token) * kLog2e;
          } else {
            s = -INFINITY;
          }
          sacc[nt][e] = s;
        }
      }
    } else if (partial) {
#pragma unroll
      for (int nt = 0; nt < kSTiles; ++nt) {
#pragma unroll
        for (int e = 0; e < 2 * kRows; ++e) {
          const int token = t0 + nt * 8 + (lane & 3) * 2 + (e & 1);
          if (token >= end) sacc[nt][e] = -INFINITY;
        }
      }
    }

    // ---- online softmax ----
    float m_new[2], m_safe[2];
    bool moved = false;
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
      float mx = -INFINITY;
#pragma unroll
      for (int nt = 0; nt < kSTiles; ++nt)
        mx = fmaxf(mx, fmaxf(sacc[nt][2 * r], sacc[nt][2 * r + 1]));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      m_new[r] = fmaxf(m_run[r], mx);
      m_safe[r] = m_new[r] == -INFINITY ? 0.0f : m_new[r];
      moved = moved || m_new[r] != m_run[r];
    }
    if (__any_sync(0xffffffffu, moved)) {
      float alpha[2] = {1.0f, 1.0f};
#pragma unroll
      for (int r = 0; r < kRows; ++r) {
        alpha[r] = fast_exp2((m_run[r] - m_safe[r]) * softmax_scale);  // exp2(-inf) = 0 at first
        m_run[r] = m_new[r];
        l_run[r] *= alpha[r];
      }
#pragma unroll
      for (int i = 0; i < kNTiles; ++i) {
        oacc[i][0] *= alpha[0];
        oacc[i][1] *= alpha[0];
        if (WIDE) {
          oacc[i][2] *= alpha[1];
          oacc[i][3] *= alpha[1];
        }
      }
    }
    uint32_t pa[kSTiles][2];  // [n-tile][row half] packed bf16 probabilities
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
      const float bias = -m_safe[r] * softmax_scale;
      float sum = 0.0f;
#pragma unroll
      for (int nt = 0; nt < kSTiles; ++nt) {
        const float p0 = fast_exp2(fmaf(sacc[nt][2 * r], softmax_scale, bias));
        const float p1 = fast_exp2(fmaf(sacc[nt][2 * r + 1], softmax_scale, bias));
        sum += p0 + p1;
        pa[nt][r] = pack_bf16x2(p0, p1);
      }
      l_run[r] += sum;
    }

    // ---- O += P V : (16 x TOK) x (TOK x D) ----
    {
      const int mat = lane >> 3;
      const int vrow = ((mat & 1) << 3) + (lane & 7);
#pragma unroll
      for (int kk = 0; kk < TOK / 16; ++kk) {
        uint32_t a[4];
        a[0] = pa[kk * 2][0];
        a[1] = WIDE ? pa[kk * 2][1] : 0u;
        a[2] = pa[kk * 2 + 1][0];
        a[3] = WIDE ? pa[kk * 2 + 1][1] : 0u;
#pragma unroll
        for (int np = 0; np < kNTiles / 2; ++np) {
          uint32_t vb[4];
          ldmatrix_x4_trans(vb, vsm + tile_offset<TOK>(kk * 16 + vrow, np * 2 + (mat >> 1)));
          mma_bf16_16816(oacc[np * 2], a, vb[0], vb[1]);
          mma_bf16_16816(oacc[np * 2 + 1], a, vb[2], vb[3]);
        }
      }
    }
  }
  if (TMA) {
    if (timed_out) {
      if (lane == 0 && p.status != nullptr) atomicOr(p.status, B200_STATUS_WAIT_TIMEOUT);
      // give the copies still in flight a bounded chance to land before the CTA retires
      for (int it = 0; it < my_count && it < kStages && !p.drop_loads; ++it)
        mbarrier_wait_bounded(bar0 + ((it0 + it) % kStages) * 8, 0, min(p.wait_limit, 100000u));
    }
  } else {
    cp_async_wait<0>();
  }
  __syncwarp();

  // quad-reduce the row sums; bring the maxima to the log2 domain
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    if (FAST) m_run[r] *= scale_log2;  // -inf stays -inf (scale > 0)
  }

  // ---- merge the 4 warps through shared memory (each warp reuses its own ring) ----
  float* my_o = reinterpret_cast<float*>(smem + warp * kWarpBytes);  // [16][D]
  float* my_ml = my_o + 16 * D;                                       // [16][2]
  {
    const int r0 = lane >> 2;
    const int col = (lane & 3) * 2;
#pragma unroll
    for (int nt = 0; nt < kNTiles; ++nt) {
      *reinterpret_cast<float2*>(my_o + r0 * D + nt * 8 + col) = make_float2(oacc[nt][0], oacc[nt][1]);
      if (WIDE)
        *reinterpret_cast<float2*>(my_o + (r0 + 8) * D + nt * 8 + col) =
            make_float2(oacc[nt][2], oacc[nt][3]);
    }
    if ((lane & 3) == 0) {
      my_ml[r0 * 2] = m_run[0];
      my_ml[r0 * 2 + 1] = l_run[0];
      if (WIDE) {
        my_ml[(r0 + 8) * 2] = m_run[1];
        my_ml[(r0 + 8) * 2 + 1] = l_run[1];
      }
    }
  }
  it_base = it0 + my_count;
  return __syncthreads_and(!timed_out) != 0;  // the same answer in every thread of the CTA
}

// CLUSTER: the splits of one (sequence, head block) form a thread-block cluster (gridDim.x ==
// cluster size <= 8) and are combined through distributed shared memory by the cluster's
// first CTA; otherwise through the fp32 scratch in global memory by whichever CTA arrives last.
template <int D, int TOK, bool WIDE, bool FAST, bool TMA, bool CLUSTER, int WARPS, bool FUSED>
__global__ void __launch_bounds__(WARPS * 32)
decode_attention_kernel(const DecodeParams p, const __grid_constant__ CUtensorMap kmap,
                        const __grid_constant__ CUtensorMap vmap) {
  constexpr int kWarpBytes = kStages * 2 * TOK * D * 2;
  constexpr int kStagingBytes = kWarpBytes / 2;  // merged partial of this CTA, in warp 0's ring
  static_assert(kStagingBytes >= 16 * D * 4 + 128 && kWarpBytes - kStagingBytes >= 16 * D * 4 + 128,
                "ring region too small to hold the partials");

  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ __align__(8) uint64_t full_bar[WARPS][kStages];
  __shared__ int merge_flag;
  // fused form only: the rotated query rows of this head block, the newest token's K and V row
  // (bf16 values held as floats) and its scores against the query rows (log2 domain)
  __shared__ __align__(16) __nv_bfloat16 q_stage[16 * D];
  __shared__ float new_k[D], new_v[D], new_score[16];

  const int split = blockIdx.x;
  const int head_block = blockIdx.y;  // kv head * blocks-per-kv-head + 16-row block
  const int b = p.order != nullptr ? __ldg(p.order + blockIdx.z) : static_cast<int>(blockIdx.z);
  if (b < 0 || b >= p.batch) return;  // (not a permutation: every CTA of that z leaves alike)
  const int row_blocks = (p.groups + 15) / 16;
  const int kvh = head_block / row_blocks;
  const int g0 = (head_block % row_blocks) * 16;  // first group row of this CTA
  const int rows = min(16, p.groups - g0);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  TraceScope trace(4);
  grid_launch_dependents();
  if (!p.early_kv) {
    grid_dependency_wait();  // lengths, q and the newest KV row come from kernels before this one
    trace.mark(0);
  }
  int64_t len = p.lengths[b] + p.length_bias;
  if (len > p.mask_len) {
    if (threadIdx.x == 0 && split == 0 && head_block == 0 && p.status != nullptr)
      atomicOr(p.status, B200_STATUS_LENGTH_OVER_MASK);
    len = p.mask_len;
  }
  if (len < 0) len = 0;
  const int n_tokens = static_cast<int>(len);
  const int start = split * p.split_tokens;
  if (!CLUSTER && start >= n_tokens && split > 0) return;  // (a cluster member must stay for the barriers)
  constexpr bool fused = FUSED;  // (the launcher picks the instantiation by p.qkv_partials)
  // fused: the newest row is not streamed from the buffer (its owner is writing it right now)
  const int streamed = fused ? max(n_tokens - 1, 0) : n_tokens;
  const int end = max(start, min(start + p.split_tokens, streamed));
  const bool owner = fused && n_tokens >= 1 && p.lengths[b] + p.length_bias <= p.mask_len &&
                     n_tokens - 1 >= start && n_tokens - 1 < start + p.split_tokens;
  if (fused && n_tokens < 1 && threadIdx.x == 0 && split == 0 && head_block == 0 && p.status != nullptr)
    atomicOr(p.status, B200_STATUS_BAD_POSITION);  // no row for the new token

  // Reduces the q|k|v partials of this CTA's rows (sum over K slices in order, + bias, rounded to
  // bf16 like the projection's own output), rotates q and k, leaves q in q_stage; the owner of
  // the newest token also stores its K / V row (first head block only) and keeps it in new_k/v.
  auto prepare_fused = [&]() {
    float row_scale = 1.0f;
    if (p.norm_row_squares != nullptr)
      row_scale = rsqrtf(sum_slices(p.norm_row_squares + b, p.batch, p.qkv_splits) /
                         static_cast<float>(p.norm_hidden) + p.norm_eps);
    const int half = D / 2;
    const int width = (p.q_heads + 2 * p.kv_heads) * D;
    const int64_t slice = static_cast<int64_t>(p.batch) * width;
    const float* prow = p.qkv_partials + static_cast<int64_t>(b) * width;
    const __nv_bfloat16* cos_row = p.cosine + static_cast<int64_t>(b) * D;
    const __nv_bfloat16* sin_row = p.sine + static_cast<int64_t>(b) * D;
    const int q_items = rows * half;
    const int items = q_items + (owner ? 2 * half : 0);
    for (int item = threadIdx.x; item < items; item += (WARPS * 32)) {
      int column, d;
      bool rotate = true;
      if (item < q_items) {
        d = item % half;
        column = (kvh * p.groups + g0 + item / half) * D;
      } else if (item < q_items + half) {
        d = item - q_items;
        column = (p.q_heads + kvh) * D;
      } else {
        d = item - q_items - half;
        column = (p.q_heads + p.kv_heads + kvh) * D;
        rotate = false;
      }
      const float clo = __bfloat162float(cos_row[d]), chi = __bfloat162float(cos_row[d + half]);
      const float slo = __bfloat162float(sin_row[d]), shi = __bfloat162float(sin_row[d + half]);
      const float bias_lo = p.qkv_bias != nullptr ? __bfloat162float(p.qkv_bias[column + d]) : 0.0f;
      const float bias_hi = p.qkv_bias != nullptr ? __bfloat162float(p.qkv_bias[column + d + half]) : 0.0f;
      float lo = sum_slices(prow + column + d, slice, p.qkv_splits) * row_scale;
      float hi = sum_slices(prow + column + d + half, slice, p.qkv_splits) * row_scale;
      if (p.qkv_bias != nullptr) {
        lo += bias_lo;
        hi += bias_hi;
      }
      lo = round_bf16(lo);
      hi = round_bf16(hi);
      float ylo = lo, yhi = hi;
      if (rotate) {
        ylo = round_bf16(__fadd_rn(round_bf16(__fmul_rn(lo, clo)), round_bf16(__fmul_rn(-hi, slo))));
        yhi = round_bf16(__fadd_rn(round_bf16(__fmul_rn(hi, chi)), round_bf16(__fmul_rn(lo, shi))));
      }
      if (item < q_items) {
        q_stage[(item / half) * D + d] = __float2bfloat16_rn(ylo);
        q_stage[(item / half) * D + d + half] = __float2bfloat16_rn(yhi);
      } else {
        float* keep = rotate ? new_k : new_v;
        keep[d] = ylo;
        keep[d + half] = yhi;
        if (g0 == 0) {
          // the row of the newest token: contiguous slot b, or through the block table
          int64_t row = static_cast<int64_t>(b) * p.capacity + (n_tokens - 1);
          if (p.block_table != nullptr) {
            const int t = n_tokens - 1;
            const int block = __ldg(p.block_table + static_cast<int64_t>(b) * p.table_stride + t / p.block_size);
            row = static_cast<int64_t>(block) * p.block_size + t % p.block_size;
            if (block < 0 || row >= p.pool_rows) {  // no block assigned: nothing is written
              if (d == 0 && p.status != nullptr) atomicOr(p.status, B200_STATUS_KV_OVERFLOW);
              continue;
            }
          }
          __nv_bfloat16* dst = (rotate ? p.kstore : p.vstore) + (row * p.kv_heads + kvh) * D;
          dst[d] = __float2bfloat16_rn(ylo);
          dst[d + half] = __float2bfloat16_rn(yhi);
        }
      }
    }
    __syncthreads();
  };

  const uint32_t bar0 = smem_u32(&full_bar[warp][0]);
  if (TMA) {
    if (lane == 0) {
#pragma unroll
      for (int s = 0; s < kStages; ++s) mbarrier_init(bar0 + s * 8, 1);
      fence_mbarrier_init();
    }
    __syncwarp();
  }
  int it_base = 0;
  const int stable_end = p.early_kv ? max(n_tokens - 1, 0) : -1;
  if constexpr (FUSED)
    stream_segment<D, TOK, WIDE, FAST, TMA, decltype(prepare_fused), WARPS>(
        p, kmap, vmap, smem, bar0, b, kvh, g0, rows, start, end, it_base, stable_end, &trace, q_stage,
        static_cast<int64_t>(D), prepare_fused);
  else
    stream_segment<D, TOK, WIDE, FAST, TMA, NoPrepare, WARPS>(
        p, kmap, vmap, smem, bar0, b, kvh, g0, rows, start, end, it_base, stable_end, &trace);
  trace.mark_middle();
  if (owner) {
    // the newest token as one more partial: max = its score (log2 domain), sum = 1, O = its V row
    for (int row = warp; row < rows; row += WARPS) {
      float dot = 0.0f;
      for (int c = lane; c < D; c += 32) dot = fmaf(__bfloat162float(q_stage[row * D + c]), new_k[c], dot);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
      if (lane == 0) new_score[row] = dot * p.scale * kLog2e;
    }
    __syncthreads();
  }

  for (int idx = threadIdx.x; idx < rows * D; idx += (WARPS * 32)) {
    const int row = idx / D;
    const int col = idx % D;
    float mw[WARPS], m_all = -INFINITY;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
      mw[w] = reinterpret_cast<const float*>(smem + w * kWarpBytes)[16 * D + row * 2];
      m_all = fmaxf(m_all, mw[w]);
    }
    if (owner) m_all = fmaxf(m_all, new_score[row]);
    float l_all = 0.0f, o_all = 0.0f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
      const float* wo = reinterpret_cast<const float*>(smem + w * kWarpBytes);
      const float wgt = mw[w] == -INFINITY ? 0.0f : fast_exp2(mw[w] - m_all);
      l_all += wo[16 * D + row * 2 + 1] * wgt;
      o_all += wo[row * D + col] * wgt;
    }
    if (owner) {
      const float wgt = fast_exp2(new_score[row] - m_all);
      l_all += wgt;
      o_all += new_v[col] * wgt;
    }
    const int hq = kvh * p.groups + g0 + row;
    if (p.num_splits == 1) {
      p.out[(static_cast<int64_t>(b) * p.q_heads + hq) * D + col] =
          __float2bfloat16_rn(o_all / l_all);  // 0/0 = NaN for an empty sequence, as the oracle
    } else if (CLUSTER) {
      float* staging = reinterpret_cast<float*>(smem + kStagingBytes);
      staging[idx] = o_all;
      if (col == 0) {
        staging[16 * D + row * 2] = m_all;
        staging[16 * D + row * 2 + 1] = l_all;
      }
    } else {
      const int64_t slot = (static_cast<int64_t>(b) * p.q_heads + hq) * p.num_splits + split;
      p.ws_o[slot * D + col] = o_all;
      if (col == 0) {
        p.ws_ml[slot * 2] = m_all;
        p.ws_ml[slot * 2 + 1] = l_all;
      }
    }
  }
  trace.mark(1);
  if (p.num_splits == 1) return;
  if (CLUSTER) {
    // every CTA of the cluster has published its partial; the first one combines them in split
    // order, the others stay until it has read them
    cluster_sync();
    if (split == 0) {
      const uint32_t staging = smem_u32(smem + kStagingBytes);
      for (int idx = threadIdx.x; idx < rows * D; idx += (WARPS * 32)) {
        const int row = idx / D;
        const int col = idx % D;
        float m_all = -INFINITY;
        for (int s = 0; s < p.num_splits; ++s)
          m_all = fmaxf(m_all, load_cluster_f32(staging + (16 * D + row * 2) * 4, s));
        float l_all = 0.0f, o_all = 0.0f;
        for (int s = 0; s < p.num_splits; ++s) {
          const float m = load_cluster_f32(staging + (16 * D + row * 2) * 4, s);
          const float wgt = m == -INFINITY ? 0.0f : fast_exp2(m - m_all);
          l_all += load_cluster_f32(staging + (16 * D + row * 2 + 1) * 4, s) * wgt;
          o_all += load_cluster_f32(staging + idx * 4, s) * wgt;
        }
        const int hq = kvh * p.groups + g0 + row;
        p.out[(static_cast<int64_t>(b) * p.q_heads + hq) * D + col] =
            __float2bfloat16_rn(o_all / l_all);
      }
    }
    cluster_sync();
    return;
  }
  if (p.counters == nullptr) return;

  // ---- the CTA that arrives last for this (sequence, head block) combines the splits ----
  int used = (n_tokens + p.split_tokens - 1) / p.split_tokens;
  if (used < 1) used = 1;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    int* counter = p.counters + b * gridDim.y + head_block;
    const int arrived = atomicAdd(counter, 1);
    merge_flag = arrived == used - 1;
    if (merge_flag) *counter = 0;  // ready for the next call on this workspace
  }
  __syncthreads();
  if (!merge_flag) return;
  __threadfence();
  for (int idx = threadIdx.x; idx < rows * D; idx += (WARPS * 32)) {
    const int row = idx / D;
    const int col = idx % D;
    const int hq = kvh * p.groups + g0 + row;
    const int64_t base = (static_cast<int64_t>(b) * p.q_heads + hq) * p.num_splits;
    float m_all = -INFINITY;
    for (int s = 0; s < used; ++s) m_all = fmaxf(m_all, __ldcg(p.ws_ml + (base + s) * 2));
    float l_all = 0.0f, o_all = 0.0f;
    int s = 0;
    for (; s + 4 <= used; s += 4) {  // four independent loads in flight per round
      float m4[4], l4[4], o4[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        m4[j] = __ldcg(p.ws_ml + (base + s + j) * 2);
        l4[j] = __ldcg(p.ws_ml + (base + s + j) * 2 + 1);
        o4[j] = __ldcg(p.ws_o + (base + s + j) * D + col);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float wgt = m4[j] == -INFINITY ? 0.0f : fast_exp2(m4[j] - m_all);
        l_all += l4[j] * wgt;
        o_all += o4[j] * wgt;
      }
    }
    for (; s < used; ++s) {
      const float m = __ldcg(p.ws_ml + (base + s) * 2);
      const float wgt = m == -INFINITY ? 0.0f : fast_exp2(m - m_all);
      l_all += __ldcg(p.ws_ml + (base + s) * 2 + 1) * wgt;
      o_all += __ldcg(p.ws_o + (base + s) * D + col) * wgt;
    }
    p.out[(static_cast<int64_t>(b) * p.q_heads + hq) * D + col] = __float2bfloat16_rn(o_all / l_all);
  }
}

// ---- Flat schedule ---------------------------------------------------------------------
// Work items are (sequence, head block, chunk of 4 x TOK tokens); item counts come from
// lengths[] on the device. The grid is 2 x 148 CTAs (two per SM) and CTA c owns the contiguous
// item range [c * ipc, (c + 1) * ipc): every SM streams the same number of tokens whatever the
// lengths are. A range may cover the end of one (sequence, head block) pair and the start of
// the next ones; a pair cut by range boundaries is finished by the CTA that arrives last at
// its counter, which merges the parts in order.
constexpr int kMaxFlatBatch = 2048;

template <int D, int TOK, bool WIDE, bool FAST, bool TMA>
__global__ void __launch_bounds__(kThreads)
decode_attention_flat_kernel(const DecodeParams p, const __grid_constant__ CUtensorMap kmap,
                             const __grid_constant__ CUtensorMap vmap) {
  constexpr int kChunk = kWarps * TOK;
  constexpr int kWarpBytes = kStages * 2 * TOK * D * 2;

  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ __align__(8) uint64_t full_bar[kWarps][kStages];
  __shared__ int prefix[kMaxFlatBatch + 1];  // chunks of the sequences before b
  __shared__ int warp_totals[kWarps];
  __shared__ int merge_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int row_blocks = (p.groups + 15) / 16;
  const int head_blocks = p.kv_heads * row_blocks;
  const int rows_per_block = min(16, p.groups);

  auto clamped_length = [&](int b) {
    int64_t len = p.lengths[b];
    if (len > p.mask_len) {
      if (blockIdx.x == 0 && p.status != nullptr) atomicOr(p.status, B200_STATUS_LENGTH_OVER_MASK);
      len = p.mask_len;
    }
    return static_cast<int>(len < 0 ? 0 : len);
  };
  auto chunks_of = [&](int b) { return max(1, (clamped_length(b) + kChunk - 1) / kChunk); };

  grid_launch_dependents();
  grid_dependency_wait();  // lengths, q and the newest KV row come from kernels before this one
  // ---- chunk counts and their exclusive prefix sums (every CTA builds the same table) ----
  {
    const int per_thread = (p.batch + kThreads - 1) / kThreads;
    const int first = threadIdx.x * per_thread;
    int local = 0;
    for (int i = 0; i < per_thread; ++i)
      if (first + i < p.batch) local += chunks_of(first + i);
    int scan = local;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, scan, o);
      if (lane >= o) scan += t;
    }
    if (lane == 31) warp_totals[warp] = scan;
    __syncthreads();
    int running = scan - local;
    for (int w = 0; w < warp; ++w) running += warp_totals[w];
    for (int i = 0; i < per_thread; ++i)
      if (first + i < p.batch) {
        prefix[first + i] = running;
        running += chunks_of(first + i);
      }
    if (threadIdx.x == kThreads - 1) prefix[p.batch] = running;
    __syncthreads();
  }
  const int total = head_blocks * prefix[p.batch];
  const int ipc = max(1, (total + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x));
  const int lo = blockIdx.x * ipc;
  const int hi = min(lo + ipc, total);
  if (lo >= total) return;

  const uint32_t bar0 = smem_u32(&full_bar[warp][0]);
  if (TMA) {
    if (lane == 0) {
#pragma unroll
      for (int s = 0; s < kStages; ++s) mbarrier_init(bar0 + s * 8, 1);
      fence_mbarrier_init();
    }
    __syncwarp();
  }

  int b;
  {
    int below = 0, above = p.batch;  // largest b with head_blocks * prefix[b] <= lo
    while (above - below > 1) {
      const int mid = (below + above) >> 1;
      if (head_blocks * prefix[mid] <= lo) below = mid; else above = mid;
    }
    b = below;
  }
  int it_base = 0;
  int g = lo;
  while (g < hi) {
    const int n_b = prefix[b + 1] - prefix[b];
    const int within = g - head_blocks * prefix[b];
    const int hb = within / n_b;
    const int c0 = within % n_b;
    const int pair_begin = g - c0;
    const int pair_end = pair_begin + n_b;
    const int seg_end = min(hi, pair_end);
    const int c1 = c0 + (seg_end - g);
    const int n_tokens = clamped_length(b);
    const int start = min(c0 * kChunk, n_tokens);
    const int end = min(c1 * kChunk, n_tokens);
    const int first_cta = pair_begin / ipc;
    const int parts = (pair_end - 1) / ipc - first_cta + 1;
    const int part = static_cast<int>(blockIdx.x) - first_cta;
    const int kvh = hb / row_blocks;
    const int g0 = (hb % row_blocks) * 16;
    const int rows = min(16, p.groups - g0);
    const int pair = b * head_blocks + hb;

    const bool ok = stream_segment<D, TOK, WIDE, FAST, TMA>(p, kmap, vmap, smem, bar0, b, kvh, g0,
                                                            rows, start, end, it_base);
    const bool fits = part < p.num_splits;  // the host bound on parts per pair
    if ((!ok || !fits) && threadIdx.x == 0 && p.status != nullptr)
      atomicOr(p.status, B200_STATUS_WAIT_TIMEOUT);

    for (int idx = threadIdx.x; idx < rows * D; idx += kThreads) {
      const int row = idx / D;
      const int col = idx % D;
      float mw[kWarps], m_all = -INFINITY;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) {
        mw[w] = reinterpret_cast<const float*>(smem + w * kWarpBytes)[16 * D + row * 2];
        m_all = fmaxf(m_all, mw[w]);
      }
      float l_all = 0.0f, o_all = 0.0f;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) {
        const float* wo = reinterpret_cast<const float*>(smem + w * kWarpBytes);
        const float wgt = mw[w] == -INFINITY ? 0.0f : fast_exp2(mw[w] - m_all);
        l_all += wo[16 * D + row * 2 + 1] * wgt;
        o_all += wo[row * D + col] * wgt;
      }
      const int hq = kvh * p.groups + g0 + row;
      if (parts == 1) {
        p.out[(static_cast<int64_t>(b) * p.q_heads + hq) * D + col] =
            __float2bfloat16_rn(o_all / l_all);  // 0/0 = NaN for an empty sequence, as the oracle
      } else if (fits) {
        const int64_t slot =
            (static_cast<int64_t>(pair) * p.num_splits + part) * rows_per_block + row;
        p.ws_o[slot * D + col] = o_all;
        if (col == 0) {
          p.ws_ml[slot * 2] = m_all;
          p.ws_ml[slot * 2 + 1] = l_all;
        }
      }
    }
    if (parts > 1) {
      __threadfence();
      __syncthreads();
      if (threadIdx.x == 0) {
        int* counter = p.counters + pair;
        const int arrived = atomicAdd(counter, 1);
        merge_flag = arrived == parts - 1;
        if (merge_flag) *counter = 0;  // ready for the next call on this workspace
      }
      __syncthreads();
      if (merge_flag) {
        __threadfence();
        const int used = min(parts, p.num_splits);
        for (int idx = threadIdx.x; idx < rows * D; idx += kThreads) {
          const int row = idx / D;
          const int col = idx % D;
          const int64_t base = static_cast<int64_t>(pair) * p.num_splits * rows_per_block + row;
          float m_all = -INFINITY;
          for (int s = 0; s < used; ++s)
            m_all = fmaxf(m_all, __ldcg(p.ws_ml + (base + s * rows_per_block) * 2));
          float l_all = 0.0f, o_all = 0.0f;
          int s = 0;
          for (; s + 4 <= used; s += 4) {  // four independent loads in flight per round
            float m4[4], l4[4], o4[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int64_t slot = base + (s + j) * rows_per_block;
              m4[j] = __ldcg(p.ws_ml + slot * 2);
              l4[j] = __ldcg(p.ws_ml + slot * 2 + 1);
              o4[j] = __ldcg(p.ws_o + slot * D + col);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float wgt = m4[j] == -INFINITY ? 0.0f : fast_exp2(m4[j] - m_all);
              l_all += l4[j] * wgt;
              o_all += o4[j] * wgt;
            }
          }
          for (; s < used; ++s) {
            const int64_t slot = base + s * rows_per_block;
            const float m = __ldcg(p.ws_ml + slot * 2);
            const float wgt = m == -INFINITY ? 0.0f : fast_exp2(m - m_all);
            l_all += __ldcg(p.ws_ml + slot * 2 + 1) * wgt;
            o_all += __ldcg(p.ws_o + slot * D + col) * wgt;
          }
          const int hq = kvh * p.groups + g0 + row;
          p.out[(static_cast<int64_t>(b) * p.q_heads + hq) * D + col] =
              __float2bfloat16_rn(o_all / l_all);
        }
      }
    }
    if (!ok) return;
    __syncthreads();  // the ring regions held the partials: free them for the next segment
    if (TMA) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    g = seg_end;
    if (g >= head_blocks * prefix[b + 1]) ++b;
  }
}

// Combines the per-split partials of one (sequence, q head) when the in-kernel merge is
// not available (more head blocks than counters). blockDim.x == D.
__global__ void decode_merge_kernel(const float* __restrict__ ws_o, const float* __restrict__ ws_ml,
                                    const int64_t* __restrict__ lengths,
                                    __nv_bfloat16* __restrict__ out, int q_heads, int head_dim,
                                    int num_splits, int split_tokens, int mask_len) {
  const int bh = blockIdx.x;
  const int b = bh / q_heads;
  int64_t len = lengths[b];
  if (len > mask_len) len = mask_len;
  if (len < 0) len = 0;
  int used = static_cast<int>((len + split_tokens - 1) / split_tokens);
  if (used < 1) used = 1;
  if (used > num_splits) used = num_splits;
  const float* ml = ws_ml + static_cast<int64_t>(bh) * num_splits * 2;
  const float* o = ws_o + static_cast<int64_t>(bh) * num_splits * head_dim;
  float m_all = -INFINITY;
  for (int s = 0; s < used; ++s) m_all = fmaxf(m_all, ml[s * 2]);
  float l_all = 0.0f, o_all = 0.0f;
  for (int s = 0; s < used; ++s) {
    const float m = ml[s * 2];
    const float wgt = m == -INFINITY ? 0.0f : fast_exp2(m - m_all);
    l_all += ml[s * 2 + 1] * wgt;
    o_all += o[s * head_dim + threadIdx.x] * wgt;
  }
  out[static_cast<int64_t>(bh) * head_dim + threadIdx.x] = __float2bfloat16_rn(o_all / l_all);
}

// ---- fp32 path (CUDA cores, IEEE fp32 dots): small graphs in full precision ----------
// One CTA per (sequence, q head); thread t walks tokens t, t+blockDim, ... with its own
// online-softmax state, then the CTA merges. Matches the oracle to fp32 round-off.
// The generic kernel: fp32, fp16, and the head sizes the tensor-core kernels do not take
// (16, 32, 256). One CTA of 64 threads per (sequence, query head), thread t owning tokens
// t, t + 64, ...; all arithmetic in fp32 on the CUDA cores, one rounding on the way out (and,
// in the compatible mode of a 16-bit type, the reference's two roundings of the scores).
template <int D, typename T>
__global__ void decode_attention_generic_kernel(const T* __restrict__ q, const T* __restrict__ kbuf,
                                                const T* __restrict__ vbuf,
                                                const int64_t* __restrict__ lengths,
                                                const void* __restrict__ mask, T* __restrict__ out,
                                                int q_heads, int kv_heads, int groups, int capacity,
                                                int mask_len, int64_t q_batch_stride,
                                                int64_t q_head_stride, int64_t mask_batch_stride,
                                                int mask_dtype, float scale, bool compat,
                                                int32_t* status) {
  constexpr int kT = D > 128 ? 32 : 64;  // (the merge buffer of 64 threads x 256 columns would not fit)
  const int hq = blockIdx.x;
  const int b = blockIdx.y;
  const int kvh = hq / groups;
  int64_t len = lengths[b];
  if (len > mask_len) {
    if (threadIdx.x == 0 && hq == 0 && status != nullptr)
      atomicOr(status, B200_STATUS_LENGTH_OVER_MASK);
    len = mask_len;
  }
  if (len < 0) len = 0;
  __shared__ float sq[D];
  __shared__ float sm[kT], sl[kT];
  __shared__ float so[kT][D + 1];
  for (int d = threadIdx.x; d < D; d += kT)
    sq[d] = Elem<T>::load(q + b * q_batch_stride + hq * q_head_stride + d);
  __syncthreads();
  float m = -INFINITY, l = 0.0f, acc[D];
#pragma unroll
  for (int d = 0; d < D; ++d) acc[d] = 0.0f;
  for (int t = threadIdx.x; t < len; t += kT) {
    const T* krow = kbuf + ((static_cast<int64_t>(b) * capacity + t) * kv_heads + kvh) * D;
    const T* vrow = vbuf + ((static_cast<int64_t>(b) * capacity + t) * kv_heads + kvh) * D;
    float s = 0.0f;
#pragma unroll
    for (int d = 0; d < D; ++d) s = fmaf(sq[d], Elem<T>::load(krow + d), s);
    s = compat ? Elem<T>::round(Elem<T>::round(s) * scale) : s * scale;
    if (mask != nullptr) s += load_mask(mask, mask_dtype, b * mask_batch_stride + t);
    const float m_new = fmaxf(m, s);
    const float m_safe = m_new == -INFINITY ? 0.0f : m_new;
    const float alpha = expf(m - m_safe);
    const float pr = expf(s - m_safe);
    l = l * alpha + pr;
#pragma unroll
    for (int d = 0; d < D; ++d) acc[d] = acc[d] * alpha + pr * Elem<T>::load(vrow + d);
    m = m_new;
  }
  sm[threadIdx.x] = m;
  sl[threadIdx.x] = l;
#pragma unroll
  for (int d = 0; d < D; ++d) so[threadIdx.x][d] = acc[d];
  __syncthreads();
  for (int d = threadIdx.x; d < D; d += kT) {
    float m_all = -INFINITY;
    for (int t = 0; t < kT; ++t) m_all = fmaxf(m_all, sm[t]);
    float l_all = 0.0f, o_all = 0.0f;
    for (int t = 0; t < kT; ++t) {
      const float wgt = sm[t] == -INFINITY ? 0.0f : expf(sm[t] - m_all);
      l_all += sl[t] * wgt;
      o_all += so[t][d] * wgt;
    }
    Elem<T>::store(out + (static_cast<int64_t>(b) * q_heads + hq) * D + d, o_all / l_all);
  }
}

template <int D>
constexpr int tokens_per_step() {
  return D <= 64 ? 32 : 16;
}

// 128B-swizzled box of TOK tokens x 64 elements of one KV head out of the B x C x Hkv x D buffer,
// seen as a 3-D tensor (D, Hkv, B*C).
bool make_kv_tensor_map(CUtensorMap* map, const void* buffer, int64_t batch, int64_t capacity,
                        int64_t kv_heads, int64_t head_dim, int tokens_per_box) {
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(head_dim), static_cast<cuuint64_t>(kv_heads),
                              static_cast<cuuint64_t>(batch * capacity)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(head_dim * 2),
                                 static_cast<cuuint64_t>(kv_heads * head_dim * 2)};
  const cuuint32_t box[3] = {64, 1, static_cast<cuuint32_t>(tokens_per_box)};
  const cuuint32_t element_strides[3] = {1, 1, 1};
  if (batch * capacity >= (int64_t(1) << 31)) return false;
  EncodeTiledFn encode = tensor_map_encoder();
  if (encode == nullptr) return false;
  const CUresult result = encode(
      map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(buffer), dims, strides, box,
      element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return result == CUDA_SUCCESS;
}

bool use_tma_loads() {
  const char* value = getenv("B200_DECODE_ATTENTION_LOADS");
  return value == nullptr || strcmp(value, "cp.async") != 0;
}

// Two splits of a pair on two 4-warp CTAs that share an SM, or the same tokens on one 8-warp
// CTA that merges in its own shared memory: the second form halves the cross-CTA merging (a
// two-split plan needs none at all) and measured 24.0 against 27.8 us at batch 64 x 4096. It is
// used whenever the plan has an even number of splits (B200_DECODE_ATTENTION_WARPS=4 keeps
// 4-warp CTAs).
bool wide_cta_enabled() {
  const char* value = getenv("B200_DECODE_ATTENTION_WARPS");
  return value == nullptr || strcmp(value, "4") != 0;
}

// Head_dim 64, TMA, fast mode: the token range of an 8-warp CTA can be served by 16 warps on
// 16-token sub-tiles (the same 196 KB of rings). The fused form does so: its prologue (q|k|v
// reduction, RoPE, KV store) and its merge are spread over 512 threads, and the decode step of
// 64 sequences x 4096 tokens measured 1.289 against 1.302 ms, 32 sequences 1.056 against 1.069.
// The plain form keeps 8 warps (alone, 64 x 4096: 24.4 against 24.8 us; ragged 64 x 4096: 17.8
// against 19.5). B200_DECODE_ATTENTION_WARPS=16 / 8 forces either for both forms.
bool sixteen_warps(bool fused) {
  const char* value = getenv("B200_DECODE_ATTENTION_WARPS");
  if (value != nullptr && strcmp(value, "16") == 0) return true;
  if (value != nullptr && strcmp(value, "8") == 0) return false;
  return fused;
}

// The splits of a pair merge through distributed shared memory when they fit one portable
// cluster and the whole grid is resident at once: that is the latency-bound regime the cluster
// merge is for. Larger grids measured slower as clusters (batch 256 x 4096: 86 vs 60 us),
// because a cluster member whose split is empty has to stay for the barriers instead of leaving
// its slot to the next CTA. B200_DECODE_ATTENTION_MERGE=global always keeps the scratch in
// global memory.
struct GridPlan {
  int warps;         // 4 or 8 per CTA
  int splits;        // CTAs per (sequence, head block)
  int split_tokens;  // tokens per CTA
  bool cluster;      // the splits of a pair form a thread-block cluster
};

GridPlan plan_grid(int64_t splits, int64_t split_tokens, int64_t batch, int64_t head_blocks) {
  GridPlan plan = {kWarps, static_cast<int>(splits), static_cast<int>(split_tokens), false};
  if (splits % 2 == 0 && wide_cta_enabled()) {
    plan.warps = 2 * kWarps;
    plan.splits = static_cast<int>(splits / 2);
    plan.split_tokens = static_cast<int>(2 * split_tokens);
  }
  const char* merge = getenv("B200_DECODE_ATTENTION_MERGE");
  const bool global_only = merge != nullptr && strcmp(merge, "global") == 0;
  const int64_t resident = plan.warps == kWarps ? 2 * kNumSMs : kNumSMs;  // CTAs at once
  plan.cluster = !global_only && plan.splits >= 2 && plan.splits <= 8 &&
                 plan.splits * batch * head_blocks <= resident;
  return plan;
}

template <int D, bool WIDE, bool FAST, bool TMA, int WARPS, bool FUSED, int TOK = tokens_per_step<D>()>
int launch_grid(const DecodeParams& p, const CUtensorMap& kmap, const CUtensorMap& vmap,
                bool cluster, cudaStream_t stream) {
  constexpr int smem = WARPS * kStages * 2 * TOK * D * 2;
  const int row_blocks = (p.groups + 15) / 16;
  dim3 grid(p.num_splits, p.kv_heads * row_blocks, p.batch);
  auto kernel = cluster ? decode_attention_kernel<D, TOK, WIDE, FAST, TMA, true, WARPS, FUSED>
                        : decode_attention_kernel<D, TOK, WIDE, FAST, TMA, false, WARPS, FUSED>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
    return B200_ERR_LAUNCH;
  if (launch_chained_cluster(kernel, grid, dim3(WARPS * 32), smem, stream,
                             cluster ? static_cast<unsigned>(p.num_splits) : 1u, p, kmap,
                             vmap) != cudaSuccess)
    return B200_ERR_LAUNCH;
  return cudaGetLastError() == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}

template <int D, bool WIDE, bool FAST, bool TMA, bool FUSED = false>
int launch_variant(const DecodeParams& p, const CUtensorMap& kmap, const CUtensorMap& vmap,
                   cudaStream_t stream) {
  const int row_blocks = (p.groups + 15) / 16;
  const GridPlan plan = plan_grid(p.num_splits, p.split_tokens, p.batch, p.kv_heads * row_blocks);
  DecodeParams q = p;
  q.num_splits = plan.splits;
  q.split_tokens = plan.split_tokens;
  if (q.ws_o != nullptr)  // the scratch was sized for at least this many splits
    q.ws_ml = q.ws_o + static_cast<int64_t>(p.batch) * p.q_heads * plan.splits * D;
  if (plan.warps == kWarps)
    return launch_grid<D, WIDE, FAST, TMA, kWarps, FUSED>(q, kmap, vmap, plan.cluster, stream);
  if constexpr (D == 64 && TMA && FAST) {
    if (sixteen_warps(FUSED))  // (the caller built the tensor maps with 16-token boxes)
      return launch_grid<D, WIDE, FAST, TMA, 4 * kWarps, FUSED, 16>(q, kmap, vmap, plan.cluster, stream);
  }
  return launch_grid<D, WIDE, FAST, TMA, 2 * kWarps, FUSED>(q, kmap, vmap, plan.cluster, stream);
}

template <int D, bool WIDE, bool FAST, bool TMA>
int launch_flat_variant(const DecodeParams& p, const CUtensorMap& kmap, const CUtensorMap& vmap,
                        int grid, cudaStream_t stream) {
  constexpr int TOK = tokens_per_step<D>();
  constexpr int smem = kWarps * kStages * 2 * TOK * D * 2;
  auto kernel = decode_attention_flat_kernel<D, TOK, WIDE, FAST, TMA>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
    return B200_ERR_LAUNCH;
  if (launch_chained(kernel, dim3(grid), dim3(kThreads), smem, stream, p, kmap, vmap) != cudaSuccess)
    return B200_ERR_LAUNCH;
  return cudaGetLastError() == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}

// flat_grid > 0 selects the flat schedule with that many CTAs.
template <int D>
int launch_bf16(const DecodeParams& p, cudaStream_t stream, int flat_grid = 0) {
  const bool fast = p.mask == nullptr && !p.compat && p.scale > 0.0f;
  const bool wide = p.groups > 8;
  CUtensorMap kmap, vmap;
  memset(&kmap, 0, sizeof(kmap));
  memset(&vmap, 0, sizeof(vmap));
  bool tma = use_tma_loads();
  int box_tokens = tokens_per_step<D>();
  if (D == 64 && tma && fast && flat_grid == 0 && sixteen_warps(p.qkv_partials != nullptr) &&
      plan_grid(p.num_splits, p.split_tokens, p.batch, p.kv_heads * ((p.groups + 15) / 16)).warps == 2 * kWarps)
    box_tokens = 16;
  if (tma)
    tma = p.block_table != nullptr
              ? make_kv_tensor_map(&kmap, p.kbuf, 1, p.pool_rows, p.kv_heads, D, box_tokens) &&
                    make_kv_tensor_map(&vmap, p.vbuf, 1, p.pool_rows, p.kv_heads, D, box_tokens)
              : make_kv_tensor_map(&kmap, p.kbuf, p.batch, p.capacity, p.kv_heads, D, box_tokens) &&
                    make_kv_tensor_map(&vmap, p.vbuf, p.batch, p.capacity, p.kv_heads, D, box_tokens);
  int code;
  if (p.qkv_partials != nullptr) {
    // the fused form (q|k|v reduction, RoPE and KV store in front of the streaming) is its own
    // instantiation, so that neither form carries the other's code; it is always the fast one
    if (!fast || flat_grid > 0) return B200_ERR_UNSUPPORTED;
    if (tma) code = wide ? launch_variant<D, true, true, true, true>(p, kmap, vmap, stream)
                         : launch_variant<D, false, true, true, true>(p, kmap, vmap, stream);
    else code = wide ? launch_variant<D, true, true, false, true>(p, kmap, vmap, stream)
                     : launch_variant<D, false, true, false, true>(p, kmap, vmap, stream);
  } else {
#define B200_DISPATCH(W, F, T)                                                        \
  code = flat_grid > 0 ? launch_flat_variant<D, W, F, T>(p, kmap, vmap, flat_grid, stream) \
                       : launch_variant<D, W, F, T>(p, kmap, vmap, stream)
  if (tma) {
    if (wide) { if (fast) B200_DISPATCH(true, true, true); else B200_DISPATCH(true, false, true); }
    else { if (fast) B200_DISPATCH(false, true, true); else B200_DISPATCH(false, false, true); }
  } else {
    if (wide) { if (fast) B200_DISPATCH(true, true, false); else B200_DISPATCH(true, false, false); }
    else { if (fast) B200_DISPATCH(false, true, false); else B200_DISPATCH(false, false, false); }
  }
#undef B200_DISPATCH
  }
  if (code != B200_OK) return code;
  const GridPlan plan = plan_grid(p.num_splits, p.split_tokens, p.batch,
                                  p.kv_heads * ((p.groups + 15) / 16));
  if (flat_grid == 0 && plan.splits > 1 && p.counters == nullptr && !plan.cluster) {
    decode_merge_kernel<<<p.batch * p.q_heads, D, 0, stream>>>(
        p.ws_o, p.ws_o + static_cast<int64_t>(p.batch) * p.q_heads * plan.splits * D, p.lengths,
        p.out, p.q_heads, D, plan.splits, plan.split_tokens, p.mask_len);
  }
  return launch_status();
}

int64_t round_up(int64_t v, int64_t m) { return (v + m - 1) / m * m; }

// Tokens per split when the caller does not choose. A (sequence, head block) unit is served by
// 8-warp CTAs, one per SM (an even number of 4-warp splits is run as half as many 8-warp CTAs):
// - up to 148 units: as many 8-warp CTAs per unit as fit one wave of 148, none shorter than
//   768 tokens, none longer than 8192. Measured at 4580 tokens, 14 / 2 heads x 64 (us, this rule / the rule it
//   replaced, which scored "fill of 296 slots x streaming share"): 16 sequences 12.3 / 17.1,
//   32: 17.7 / 29.5, 48: 21.7 / 36.8, 64: unchanged (one 8-warp CTA per unit);
// - up to 296 units: one 4-warp CTA per unit, two per SM, all resident at once (96 sequences
//   38.0 / 51.7, 128: 48.7 / 63.6);
// - beyond: several waves whatever the split; the earlier scoring stands (splits are multiples
//   of the 128 tokens four warps cover per step and never shorter than 256 tokens).
int64_t default_split_tokens(int64_t batch, int64_t head_blocks, int64_t max_length) {
  const int64_t units = batch * head_blocks;
  if (units <= kNumSMs) {
    int64_t wide = std::min<int64_t>(kNumSMs / std::max<int64_t>(units, 1), std::max<int64_t>(max_length / 768, 1));
    // (nor longer than 8192 tokens: with ragged lengths the longest sequence would set the time;
    // several waves of 2 MB pieces balance, and their fixed cost is small beside 20 us of streaming)
    wide = std::max<int64_t>(wide, ceil_div(max_length, 8192));
    for (; wide >= 1; --wide) {
      const int64_t tokens = round_up(ceil_div(max_length, 2 * wide), 128);
      if (ceil_div(max_length, tokens) == 2 * wide || wide == 1) return tokens;
    }
  }
  if (units <= 2 * kNumSMs) return round_up(max_length, 128);
  const int64_t slots = static_cast<int64_t>(kNumSMs) * 2;
  int64_t best_tokens = round_up(max_length, 128);
  double best_score = -1.0;
  for (int64_t splits = 1; splits <= 64; ++splits) {
    const int64_t tokens = round_up(ceil_div(max_length, splits), 128);
    if (tokens < 256 && splits > 1) break;
    const int64_t real_splits = ceil_div(max_length, tokens);
    const int64_t ctas = units * real_splits;
    const int64_t waves = ceil_div(ctas, slots);
    const double fill = static_cast<double>(ctas) / static_cast<double>(waves * slots);
    const double streaming = static_cast<double>(tokens) / static_cast<double>(tokens + 96);
    const double score = fill * streaming;
    if (score > best_score + 1e-9) {
      best_score = score;
      best_tokens = tokens;
    }
  }
  return best_tokens;
}

int64_t workspace_bytes_for(int64_t batch, int64_t q_heads, int64_t head_dim, int64_t splits) {
  return kCounterBytes + round_up(batch * q_heads * splits * (head_dim + 2) * 4, 256);
}

// The flat schedule: CTAs launched, the most parts one (sequence, head block) pair can be cut
// into whatever the lengths turn out to be, and the scratch that holds those parts.
struct FlatPlan {
  bool usable;
  int grid;
  int max_parts;
  int64_t workspace_bytes;
};

// Opt-in (B200_DECODE_ATTENTION_SCHEDULE=flat): on B200 the fixed grid measured faster at
// every batch x length point tried (28.9 vs 36.0 us at 64 x 4096), because a CTA of the flat
// schedule pays the pipeline ramp and the merge once per segment.
bool flat_schedule_enabled() {
  const char* value = getenv("B200_DECODE_ATTENTION_SCHEDULE");
  return value != nullptr && strcmp(value, "flat") == 0;
}

FlatPlan plan_flat(int64_t batch, int64_t q_heads, int64_t kv_heads, int64_t head_dim,
                   int64_t max_length) {
  FlatPlan plan = {false, 0, 1, 0};
  const int64_t groups = q_heads / kv_heads;
  const int64_t head_blocks = kv_heads * ceil_div(groups, 16);
  const int64_t pairs = batch * head_blocks;
  if (!flat_schedule_enabled() || batch > kMaxFlatBatch || pairs > kMaxCounters) return plan;
  const int64_t chunk = kWarps * (head_dim == 64 ? tokens_per_step<64>() : tokens_per_step<128>());
  const int64_t chunks = std::max<int64_t>(1, ceil_div(max_length, chunk));
  if (pairs * chunks > INT32_MAX) return plan;
  const int64_t grid = std::min<int64_t>(2 * kNumSMs, pairs * chunks);
  // A pair of n chunks among `pairs` pairs meets at most n * grid / (n + pairs - 1) item-range
  // boundaries (every other pair holds at least one chunk), plus one at either end.
  const int64_t cut = chunks * grid / (chunks + pairs - 1) + 2;
  plan.usable = true;
  plan.grid = static_cast<int>(grid);
  plan.max_parts = static_cast<int>(std::min(std::min(chunks, grid), cut));
  const int64_t rows = std::min<int64_t>(16, groups);
  plan.workspace_bytes =
      plan.max_parts <= 1
          ? 0
          : kCounterBytes + round_up(pairs * plan.max_parts * rows * (head_dim + 2) * 4, 256);
  return plan;
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" int64_t b200_decode_attention_workspace_bytes(int64_t batch, int64_t q_heads,
                                                         int64_t kv_heads, int64_t head_dim,
                                                         int64_t max_length,
                                                         int64_t split_tokens) {
  if (batch <= 0 || q_heads <= 0 || kv_heads <= 0 || head_dim <= 0 || max_length <= 0) return 0;
  const int64_t groups = q_heads / kv_heads;
  const int64_t head_blocks = kv_heads * ceil_div(groups, 16);
  if (split_tokens <= 0 && (head_dim == 64 || head_dim == 128)) {
    const FlatPlan plan = plan_flat(batch, q_heads, kv_heads, head_dim, max_length);
    if (plan.usable) return plan.workspace_bytes;
  }
  if (split_tokens <= 0) split_tokens = default_split_tokens(batch, head_blocks, max_length);
  split_tokens = round_up(split_tokens, 32);
  const int64_t splits = ceil_div(max_length, split_tokens);
  if (splits <= 1) return 0;
  return workspace_bytes_for(batch, q_heads, head_dim, splits);
}

static int decode_attention_impl(const void* query, const void* key_buffer,
                                 const void* value_buffer, const int64_t* lengths,
                                 const void* mask, void* output, int64_t batch,
                                 int64_t q_heads, int64_t kv_heads, int64_t head_dim,
                                 int64_t capacity, int64_t mask_len, int64_t q_batch_stride,
                                 int64_t q_head_stride, int64_t mask_batch_stride,
                                 int mask_dtype, double scale, int dtype, int mode,
                                 int64_t split_tokens, int64_t max_length_hint,
                                 void* workspace, int64_t workspace_bytes, int32_t* status,
                                 void* stream, const int32_t* sequence_order) {
  if (!query || !key_buffer || !value_buffer || !lengths || !output || batch < 0 ||
      q_heads <= 0 || kv_heads <= 0 || head_dim <= 0 || capacity <= 0 || mask_len <= 0 ||
      mask_len > capacity || q_heads % kv_heads != 0)
    return B200_ERR_BAD_ARGUMENT;
  if (mask != nullptr && !known_dtype(mask_dtype))
    return B200_ERR_UNSUPPORTED;
  if (batch == 0) return B200_OK;
  if (batch > 65535) return B200_ERR_TOO_LARGE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int groups = static_cast<int>(q_heads / kv_heads);

  if (!known_dtype(dtype)) return B200_ERR_UNSUPPORTED;
  if (dtype != B200_BF16 || (head_dim != 64 && head_dim != 128)) {
    if (sequence_order != nullptr) return B200_ERR_UNSUPPORTED;  // (a service order is the tensor-core kernel's)
    if (head_dim != 16 && head_dim != 32 && head_dim != 64 && head_dim != 128 && head_dim != 256)
      return B200_ERR_UNSUPPORTED;
    dim3 grid(static_cast<unsigned>(q_heads), static_cast<unsigned>(batch));
    const bool compat = mode == B200_MODE_PYTORCH_COMPATIBLE && dtype != B200_F32;
    with_element_type(dtype, [&](auto tag) {
      using T = typename decltype(tag)::type;
      auto run = [&](auto kernel) {
        kernel<<<grid, head_dim > 128 ? 32 : 64, 0, s>>>(
            static_cast<const T*>(query), static_cast<const T*>(key_buffer),
            static_cast<const T*>(value_buffer), lengths, mask, static_cast<T*>(output),
            static_cast<int>(q_heads), static_cast<int>(kv_heads), groups, static_cast<int>(capacity),
            static_cast<int>(mask_len), q_batch_stride, q_head_stride, mask_batch_stride, mask_dtype,
            static_cast<float>(scale), compat, status);
      };
      if (head_dim == 16) run(decode_attention_generic_kernel<16, T>);
      else if (head_dim == 32) run(decode_attention_generic_kernel<32, T>);
      else if (head_dim == 64) run(decode_attention_generic_kernel<64, T>);
      else if (head_dim == 128) run(decode_attention_generic_kernel<128, T>);
      else run(decode_attention_generic_kernel<256, T>);
    });
    return launch_status();
  }
  if (!aligned16(key_buffer) || !aligned16(value_buffer) ||
      (reinterpret_cast<uintptr_t>(query) & 3u) != 0 || q_head_stride % 2 != 0 ||
      q_batch_stride % 2 != 0)
    return B200_ERR_ALIGNMENT;
  if (capacity > INT32_MAX / 2 || batch * capacity > INT32_MAX) return B200_ERR_TOO_LARGE;

  int64_t max_length = max_length_hint > 0 && max_length_hint < mask_len ? max_length_hint : mask_len;
  const int64_t head_blocks = kv_heads * ceil_div(groups, 16);
  FlatPlan flat = {false, 0, 1, 0};
  if (split_tokens <= 0) flat = plan_flat(batch, q_heads, kv_heads, head_dim, max_length);
  if (split_tokens <= 0) split_tokens = default_split_tokens(batch, head_blocks, max_length);
  split_tokens = round_up(split_tokens, 32);
  const int64_t splits = flat.usable ? flat.max_parts : ceil_div(max_length, split_tokens);
  if (splits > 65535 || split_tokens > INT32_MAX) return B200_ERR_TOO_LARGE;

  DecodeParams p;
  p.q = static_cast<const __nv_bfloat16*>(query);
  p.kbuf = static_cast<const __nv_bfloat16*>(key_buffer);
  p.vbuf = static_cast<const __nv_bfloat16*>(value_buffer);
  p.lengths = lengths;
  p.mask = mask;
  p.out = static_cast<__nv_bfloat16*>(output);
  p.status = status;
  p.q_batch_stride = q_batch_stride;
  p.q_head_stride = q_head_stride;
  p.mask_batch_stride = mask_batch_stride;
  p.batch = static_cast<int>(batch);
  p.q_heads = static_cast<int>(q_heads);
  p.kv_heads = static_cast<int>(kv_heads);
  p.groups = groups;
  p.capacity = static_cast<int>(capacity);
  p.mask_len = static_cast<int>(max_length);
  p.split_tokens = static_cast<int>(split_tokens);
  p.num_splits = static_cast<int>(splits);
  p.mask_dtype = mask_dtype;
  p.compat = mode == B200_MODE_PYTORCH_COMPATIBLE ? 1 : 0;
  p.early_kv = (launch_mode() & B200_LAUNCH_STABLE_KV_PREFIX) != 0 ? 1 : 0;
  p.wait_limit = wait_limit();
  p.drop_loads = drop_loads();
  p.scale = static_cast<float>(scale);
  p.ws_o = nullptr;
  p.ws_ml = nullptr;
  p.counters = nullptr;
  p.order = flat.usable ? nullptr : sequence_order;  // (the flat schedule balances by itself)
  if (flat.usable) {
    if (flat.max_parts > 1) {
      if (!workspace || workspace_bytes < flat.workspace_bytes) return B200_ERR_WORKSPACE;
      const int64_t rows = std::min<int64_t>(16, groups);
      p.counters = static_cast<int*>(workspace);
      p.ws_o = reinterpret_cast<float*>(static_cast<char*>(workspace) + kCounterBytes);
      p.ws_ml = p.ws_o + batch * head_blocks * flat.max_parts * rows * head_dim;
    }
    return head_dim == 64 ? launch_bf16<64>(p, s, flat.grid) : launch_bf16<128>(p, s, flat.grid);
  }
  const GridPlan grid_plan = plan_grid(splits, split_tokens, batch, head_blocks);
  if (grid_plan.splits > 1 && !grid_plan.cluster) {  // (a cluster combines its splits in shared memory)
    const int64_t need = workspace_bytes_for(batch, q_heads, head_dim, splits);
    if (!workspace || workspace_bytes < need) return B200_ERR_WORKSPACE;
    if (batch * head_blocks <= kMaxCounters) p.counters = static_cast<int*>(workspace);
    p.ws_o = reinterpret_cast<float*>(static_cast<char*>(workspace) + kCounterBytes);
    p.ws_ml = p.ws_o + batch * q_heads * splits * head_dim;
  }
  return head_dim == 64 ? launch_bf16<64>(p, s) : launch_bf16<128>(p, s);
}

extern "C" int b200_decode_attention(const void* query, const void* key_buffer,
                                     const void* value_buffer, const int64_t* lengths,
                                     const void* mask, void* output, int64_t batch,
                                     int64_t q_heads, int64_t kv_heads, int64_t head_dim,
                                     int64_t capacity, int64_t mask_len, int64_t q_batch_stride,
                                     int64_t q_head_stride, int64_t mask_batch_stride,
                                     int mask_dtype, double scale, int dtype, int mode,
                                     int64_t split_tokens, int64_t max_length_hint,
                                     void* workspace, int64_t workspace_bytes, int32_t* status,
                                     void* stream) {
  return decode_attention_impl(query, key_buffer, value_buffer, lengths, mask, output, batch, q_heads,
                               kv_heads, head_dim, capacity, mask_len, q_batch_stride, q_head_stride,
                               mask_batch_stride, mask_dtype, scale, dtype, mode, split_tokens,
                               max_length_hint, workspace, workspace_bytes, status, stream, nullptr);
}

// The same with a service order: CTA group i of the grid serves sequence sequence_order[i].
extern "C" int b200_decode_attention_ordered(
    const void* query, const void* key_buffer, const void* value_buffer, const int64_t* lengths,
    const void* mask, void* output, const int32_t* sequence_order, int64_t batch, int64_t q_heads,
    int64_t kv_heads, int64_t head_dim, int64_t capacity, int64_t mask_len, int64_t q_batch_stride,
    int64_t q_head_stride, int64_t mask_batch_stride, int mask_dtype, double scale, int dtype,
    int mode, int64_t split_tokens, int64_t max_length_hint, void* workspace,
    int64_t workspace_bytes, int32_t* status, void* stream) {
  if (!sequence_order) return B200_ERR_BAD_ARGUMENT;
  if (dtype != B200_BF16) return B200_ERR_UNSUPPORTED;
  return decode_attention_impl(query, key_buffer, value_buffer, lengths, mask, output, batch, q_heads,
                               kv_heads, head_dim, capacity, mask_len, q_batch_stride, q_head_stride,
                               mask_batch_stride, mask_dtype, scale, dtype, mode, split_tokens,
                               max_length_hint, workspace, workspace_bytes, status, stream,
                               sequence_order);
}

// ---- Paged KV layout ---------------------------------------------------------------------
// The same kernel over block pools and a block table instead of one contiguous buffer per
// sequence. Splits merge through the caller's workspace (the cluster merge and the fused
// q|k|v form are for the contiguous layout).
extern "C" int b200_paged_decode_attention(
    const void* query, const void* key_pool, const void* value_pool, const int32_t* block_table,
    const int64_t* lengths, const void* mask, void* output, int64_t batch, int64_t q_heads,
    int64_t kv_heads, int64_t head_dim, int64_t num_blocks, int64_t block_size,
    int64_t max_blocks_per_sequence, int64_t mask_len, int64_t q_batch_stride, int64_t q_head_stride,
    int64_t mask_batch_stride, int mask_dtype, double scale, int mode, int64_t split_tokens,
    int64_t max_length_hint, void* workspace, int64_t workspace_bytes, int32_t* status, void* stream) {
  const int64_t capacity = max_blocks_per_sequence * block_size;
  if (!query || !key_pool || !value_pool || !block_table || !lengths || !output || batch < 0 ||
      q_heads <= 0 || kv_heads <= 0 || head_dim <= 0 || num_blocks <= 0 || block_size <= 0 ||
      max_blocks_per_sequence <= 0 || mask_len <= 0 || mask_len > capacity || q_heads % kv_heads != 0)
    return B200_ERR_BAD_ARGUMENT;
  if (mask != nullptr && !known_dtype(mask_dtype)) return B200_ERR_UNSUPPORTED;
  if (head_dim != 64 && head_dim != 128) return B200_ERR_UNSUPPORTED;
  if (block_size % 32 != 0) return B200_ERR_UNSUPPORTED;  // a 32-token copy must stay inside one block
  if (batch == 0) return B200_OK;
  if (batch > 65535) return B200_ERR_TOO_LARGE;
  if (!aligned16(key_pool) || !aligned16(value_pool) ||
      (reinterpret_cast<uintptr_t>(query) & 3u) != 0 || q_head_stride % 2 != 0 || q_batch_stride % 2 != 0)
    return B200_ERR_ALIGNMENT;
  if (capacity > INT32_MAX / 2 || num_blocks * block_size > INT32_MAX) return B200_ERR_TOO_LARGE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int groups = static_cast<int>(q_heads / kv_heads);
  int64_t max_length = max_length_hint > 0 && max_length_hint < mask_len ? max_length_hint : mask_len;
  const int64_t head_blocks = kv_heads * ceil_div(groups, 16);
  if (split_tokens <= 0) split_tokens = default_split_tokens(batch, head_blocks, max_length);
  split_tokens = round_up(split_tokens, 32);
  const int64_t splits = ceil_div(max_length, split_tokens);
  if (splits > 65535 || split_tokens > INT32_MAX) return B200_ERR_TOO_LARGE;

  DecodeParams p;
  p.q = static_cast<const __nv_bfloat16*>(query);
  p.kbuf = static_cast<const __nv_bfloat16*>(key_pool);
  p.vbuf = static_cast<const __nv_bfloat16*>(value_pool);
  p.lengths = lengths;
  p.mask = mask;
  p.out = static_cast<__nv_bfloat16*>(output);
  p.status = status;
  p.q_batch_stride = q_batch_stride;
  p.q_head_stride = q_head_stride;
  p.mask_batch_stride = mask_batch_stride;
  p.batch = static_cast<int>(batch);
  p.q_heads = static_cast<int>(q_heads);
  p.kv_heads = static_cast<int>(kv_heads);
  p.groups = groups;
  p.capacity = static_cast<int>(capacity);
  p.mask_len = static_cast<int>(max_length);
  p.split_tokens = static_cast<int>(split_tokens);
  p.num_splits = static_cast<int>(splits);
  p.mask_dtype = mask_dtype;
  p.compat = mode == B200_MODE_PYTORCH_COMPATIBLE ? 1 : 0;
  p.early_kv = 0;
  p.wait_limit = wait_limit();
  p.drop_loads = drop_loads();
  p.scale = static_cast<float>(scale);
  p.ws_o = nullptr;
  p.ws_ml = nullptr;
  p.counters = nullptr;
  p.block_table = block_table;
  p.block_size = static_cast<int>(block_size);
  p.table_stride = static_cast<int>(max_blocks_per_sequence);
  p.pool_rows = num_blocks * block_size;
  const GridPlan grid_plan = plan_grid(splits, split_tokens, batch, head_blocks);
  if (grid_plan.splits > 1) {
    const int64_t need = workspace_bytes_for(batch, q_heads, head_dim, splits);
    if (!workspace || workspace_bytes < need) return B200_ERR_WORKSPACE;
    if (batch * head_blocks <= kMaxCounters) p.counters = static_cast<int*>(workspace);
    p.ws_o = reinterpret_cast<float*>(static_cast<char*>(workspace) + kCounterBytes);
    p.ws_ml = p.ws_o + batch * q_heads * splits * head_dim;
  }
  return head_dim == 64 ? launch_bf16<64>(p, s) : launch_bf16<128>(p, s);
}

// ---- Entry point that allocates nothing ------------------------------------------------
// Same computation as b200_decode_attention, for callers that are not allowed to allocate
// device memory at all: the split-KV scratch (tile counters + fp32 partials) lives in a
// file-scope device array that every GPU loading this library holds until the process exits.
namespace b200 {
namespace {

constexpr int64_t kStaticScratchBytes = 8ll << 20;  // 8 MiB per GPU, the stated maximum
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
// Device addresses of g_static_scratch, one per device. In host code the array's name is
// only a host-side stand-in; the address a kernel may use comes from cudaGetSymbolAddress.
void* g_static_scratch_address[kMaxDevices] = {};

// Set-up, once per device, with that device current. Returns nullptr on failure.
void* static_scratch_for_current_device() {
  int device = -1;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) return nullptr;
  if (g_static_scratch_address[device] == nullptr) {
    void* address = nullptr;
    if (cudaGetSymbolAddress(&address, g_static_scratch) != cudaSuccess) return nullptr;
    g_static_scratch_address[device] = address;
  }
  return g_static_scratch_address[device];
}

}  // namespace
}  // namespace b200

extern "C" int64_t b200_decode_attention_static_scratch_bytes(void) { return kStaticScratchBytes; }

extern "C" int b200_decode_attention_static_scratch(
    const void* query, const void* key_buffer, const void* value_buffer, const int64_t* lengths,
    const void* mask, void* output, int64_t batch, int64_t q_heads, int64_t kv_heads,
    int64_t head_dim, int64_t capacity, int64_t mask_len, int64_t q_batch_stride,
    int64_t q_head_stride, int64_t mask_batch_stride, int mask_dtype, double scale, int dtype,
    int mode, int64_t split_tokens, int64_t max_length_hint, int32_t* status, void* stream) {
  if (!query || !key_buffer || !value_buffer || !lengths || !output || batch < 0 ||
      q_heads <= 0 || kv_heads <= 0 || head_dim <= 0 || capacity <= 0 || mask_len <= 0 ||
      mask_len > capacity || q_heads % kv_heads != 0)
    return B200_ERR_BAD_ARGUMENT;
  if (mask != nullptr && !known_dtype(mask_dtype))
    return B200_ERR_UNSUPPORTED;
  if (dtype != B200_BF16) return B200_ERR_UNSUPPORTED;  // the fp32 kernel needs no scratch
  if (head_dim != 64 && head_dim != 128) return B200_ERR_UNSUPPORTED;
  if (batch == 0) return B200_OK;
  if (batch > 65535) return B200_ERR_TOO_LARGE;
  if (!aligned16(key_buffer) || !aligned16(value_buffer) ||
      (reinterpret_cast<uintptr_t>(query) & 3u) != 0 || q_head_stride % 2 != 0 ||
      q_batch_stride % 2 != 0)
    return B200_ERR_ALIGNMENT;
  if (capacity > INT32_MAX / 2 || batch * capacity > INT32_MAX) return B200_ERR_TOO_LARGE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int groups = static_cast<int>(q_heads / kv_heads);
  {
    // The scratch array used is the current device's copy: operands that live on another GPU
    // would pair this GPU's scratch with that GPU's tensors. Refused before anything is queued.
    int current = -1;
    cudaPointerAttributes attributes;
    if (cudaGetDevice(&current) != cudaSuccess) return B200_ERR_LAUNCH;
    if (cudaPointerGetAttributes(&attributes, output) == cudaSuccess &&
        attributes.type == cudaMemoryTypeDevice && attributes.device != current)
      return B200_ERR_BAD_ARGUMENT;
    (void)cudaGetLastError();
  }

  int64_t max_length = max_length_hint > 0 && max_length_hint < mask_len ? max_length_hint : mask_len;
  const int64_t head_blocks = kv_heads * ceil_div(groups, 16);
  if (split_tokens <= 0) split_tokens = default_split_tokens(batch, head_blocks, max_length);
  split_tokens = round_up(split_tokens, 32);
  const int64_t splits = ceil_div(max_length, split_tokens);
  if (splits > 65535 || split_tokens > INT32_MAX) return B200_ERR_TOO_LARGE;
  // the request must fit the fixed array: counters + partials, or it is refused outright
  if (splits > 1 && (workspace_bytes_for(batch, q_heads, head_dim, splits) > kStaticScratchBytes ||
                     batch * head_blocks > kMaxCounters))
    return B200_ERR_TOO_LARGE;

  DecodeParams p;
  p.q = static_cast<const __nv_bfloat16*>(query);
  p.kbuf = static_cast<const __nv_bfloat16*>(key_buffer);
  p.vbuf = static_cast<const __nv_bfloat16*>(value_buffer);
  p.lengths = lengths;
  p.mask = mask;
  p.out = static_cast<__nv_bfloat16*>(output);
  p.status = status;
  p.q_batch_stride = q_batch_stride;
  p.q_head_stride = q_head_stride;
  p.mask_batch_stride = mask_batch_stride;
  p.batch = static_cast<int>(batch);
  p.q_heads = static_cast<int>(q_heads);
  p.kv_heads = static_cast<int>(kv_heads);
  p.groups = groups;
  p.capacity = static_cast<int>(capacity);
  p.mask_len = static_cast<int>(max_length);
  p.split_tokens = static_cast<int>(split_tokens);
  p.num_splits = static_cast<int>(splits);
  p.mask_dtype = mask_dtype;
  p.compat = mode == B200_MODE_PYTORCH_COMPATIBLE ? 1 : 0;
  p.early_kv = (launch_mode() & B200_LAUNCH_STABLE_KV_PREFIX) != 0 ? 1 : 0;
  p.wait_limit = wait_limit();
  p.drop_loads = drop_loads();
  p.scale = static_cast<float>(scale);
  p.ws_o = nullptr;
  p.ws_ml = nullptr;
  p.counters = nullptr;
  if (splits > 1) {
    void* scratch = static_scratch_for_current_device();
    if (scratch == nullptr) return B200_ERR_LAUNCH;
    // the array keeps whatever the last call left: the counters must start from zero
    if (cudaMemsetAsync(scratch, 0, kCounterBytes, s) != cudaSuccess) return B200_ERR_LAUNCH;
    p.counters = static_cast<int*>(scratch);
    p.ws_o = reinterpret_cast<float*>(static_cast<char*>(scratch) + kCounterBytes);
    p.ws_ml = p.ws_o + batch * q_heads * splits * head_dim;
  }
  return head_dim == 64 ? launch_bf16<64>(p, s) : launch_bf16<128>(p, s);
}

// ---- Fused q|k|v reduction + RoPE + KV store + decode attention ---------------------------
// block_table == nullptr: key_buffer / value_buffer are the contiguous [B, capacity, Hkv, D]
// buffers; else they are block pools [num_blocks, block_size, Hkv, D] and capacity is
// max_blocks_per_sequence * block_size.
static int qkv_decode_attention_impl(
    const void* qkv_partials, int64_t qkv_splits, const void* qkv_bias, const void* cosine,
    const void* sine, void* key_buffer, void* value_buffer, const int64_t* lengths, void* output,
    int64_t batch, int64_t q_heads, int64_t kv_heads, int64_t head_dim, int64_t capacity,
    int64_t mask_len, double scale, int64_t split_tokens, int64_t max_length_hint,
    int64_t length_offset, const void* norm_row_squares, int64_t norm_hidden, double norm_epsilon,
    void* workspace, int64_t workspace_bytes, int32_t* status, void* stream,
    const int32_t* block_table, int64_t num_blocks, int64_t block_size,
    const int32_t* sequence_order) {
  if (norm_row_squares != nullptr && (norm_hidden <= 0 || !(norm_epsilon >= 0.0)))
    return B200_ERR_BAD_ARGUMENT;
  if (length_offset < 0 || length_offset > 1) return B200_ERR_BAD_ARGUMENT;
  if (!qkv_partials || !cosine || !sine || !key_buffer || !value_buffer || !lengths || !output ||
      qkv_splits <= 0 || batch < 0 || q_heads <= 0 || kv_heads <= 0 || head_dim <= 0 ||
      capacity <= 0 || mask_len <= 0 || mask_len > capacity || q_heads % kv_heads != 0 ||
      !(scale > 0.0))
    return B200_ERR_BAD_ARGUMENT;
  if (head_dim != 64 && head_dim != 128) return B200_ERR_UNSUPPORTED;
  if (batch == 0) return B200_OK;
  if (batch > 65535) return B200_ERR_TOO_LARGE;
  if (!aligned16(key_buffer) || !aligned16(value_buffer) || !aligned16(qkv_partials))
    return B200_ERR_ALIGNMENT;
  if (capacity > INT32_MAX / 2 ||
      (block_table == nullptr ? batch * capacity : num_blocks * block_size) > INT32_MAX)
    return B200_ERR_TOO_LARGE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int groups = static_cast<int>(q_heads / kv_heads);
  int64_t max_length = max_length_hint > 0 && max_length_hint < mask_len ? max_length_hint : mask_len;
  const int64_t head_blocks = kv_heads * ceil_div(groups, 16);
  if (split_tokens <= 0) split_tokens = default_split_tokens(batch, head_blocks, max_length);
  split_tokens = round_up(split_tokens, 32);
  const int64_t splits = ceil_div(max_length, split_tokens);
  if (splits > 65535 || split_tokens > INT32_MAX) return B200_ERR_TOO_LARGE;

  DecodeParams p;
  p.q = nullptr;
  p.kbuf = static_cast<const __nv_bfloat16*>(key_buffer);
  p.vbuf = static_cast<const __nv_bfloat16*>(value_buffer);
  p.lengths = lengths;
  p.mask = nullptr;
  p.out = static_cast<__nv_bfloat16*>(output);
  p.status = status;
  p.q_batch_stride = p.q_head_stride = p.mask_batch_stride = 0;
  p.batch = static_cast<int>(batch);
  p.q_heads = static_cast<int>(q_heads);
  p.kv_heads = static_cast<int>(kv_heads);
  p.groups = groups;
  p.capacity = static_cast<int>(capacity);
  p.mask_len = static_cast<int>(max_length);
  p.split_tokens = static_cast<int>(split_tokens);
  p.num_splits = static_cast<int>(splits);
  p.mask_dtype = B200_F32;
  p.compat = 0;
  p.early_kv = (launch_mode() & B200_LAUNCH_STABLE_KV_PREFIX) != 0 ? 1 : 0;
  p.wait_limit = wait_limit();
  p.drop_loads = drop_loads();
  p.scale = static_cast<float>(scale);
  p.ws_o = nullptr;
  p.ws_ml = nullptr;
  p.counters = nullptr;
  p.qkv_partials = static_cast<const float*>(qkv_partials);
  p.qkv_bias = static_cast<const __nv_bfloat16*>(qkv_bias);
  p.cosine = static_cast<const __nv_bfloat16*>(cosine);
  p.sine = static_cast<const __nv_bfloat16*>(sine);
  p.kstore = static_cast<__nv_bfloat16*>(key_buffer);
  p.vstore = static_cast<__nv_bfloat16*>(value_buffer);
  p.qkv_splits = static_cast<int>(qkv_splits);
  p.norm_row_squares = static_cast<const float*>(norm_row_squares);
  p.length_bias = static_cast<int>(length_offset);
  p.norm_hidden = static_cast<int>(norm_hidden);
  p.norm_eps = static_cast<float>(norm_epsilon);
  if (block_table != nullptr) {
    p.block_table = block_table;
    p.block_size = static_cast<int>(block_size);
    p.table_stride = static_cast<int>(capacity / block_size);
    p.pool_rows = num_blocks * block_size;
  }
  p.order = sequence_order;
  const GridPlan grid_plan = plan_grid(splits, split_tokens, batch, head_blocks);
  if (grid_plan.splits > 1 && !grid_plan.cluster) {
    const int64_t need = workspace_bytes_for(batch, q_heads, head_dim, splits);
    if (!workspace || workspace_bytes < need) return B200_ERR_WORKSPACE;
    if (batch * head_blocks <= kMaxCounters) p.counters = static_cast<int*>(workspace);
    p.ws_o = reinterpret_cast<float*>(static_cast<char*>(workspace) + kCounterBytes);
    p.ws_ml = p.ws_o + batch * q_heads * splits * head_dim;
  }
  return head_dim == 64 ? launch_bf16<64>(p, s) : launch_bf16<128>(p, s);
}

extern "C" int b200_qkv_decode_attention(
    const void* qkv_partials, int64_t qkv_splits, const void* qkv_bias, const void* cosine,
    const void* sine, void* key_buffer, void* value_buffer, const int64_t* lengths, void* output,
    int64_t batch, int64_t q_heads, int64_t kv_heads, int64_t head_dim, int64_t capacity,
    int64_t mask_len, double scale, int64_t split_tokens, int64_t max_length_hint,
    int64_t length_offset, const void* norm_row_squares, int64_t norm_hidden, double norm_epsilon,
    const int32_t* sequence_order, void* workspace, int64_t workspace_bytes, int32_t* status,
    void* stream) {
  return qkv_decode_attention_impl(qkv_partials, qkv_splits, qkv_bias, cosine, sine, key_buffer,
                                   value_buffer, lengths, output, batch, q_heads, kv_heads, head_dim,
                                   capacity, mask_len, scale, split_tokens, max_length_hint,
                                   length_offset, norm_row_squares, norm_hidden, norm_epsilon,
                                   workspace, workspace_bytes, status, stream, nullptr, 0, 0,
                                   sequence_order);
}

extern "C" int b200_paged_qkv_decode_attention(
    const void* qkv_partials, int64_t qkv_splits, const void* qkv_bias, const void* cosine,
    const void* sine, void* key_pool, void* value_pool, const int32_t* block_table,
    const int64_t* lengths, void* output, int64_t batch, int64_t q_heads, int64_t kv_heads,
    int64_t head_dim, int64_t num_blocks, int64_t block_size, int64_t max_blocks_per_sequence,
    int64_t mask_len, double scale, int64_t split_tokens, int64_t max_length_hint,
    int64_t length_offset, const void* norm_row_squares, int64_t norm_hidden, double norm_epsilon,
    const int32_t* sequence_order, void* workspace, int64_t workspace_bytes, int32_t* status,
    void* stream) {
  if (!block_table || num_blocks <= 0 || block_size <= 0 || max_blocks_per_sequence <= 0)
    return B200_ERR_BAD_ARGUMENT;
  if (block_size % 32 != 0) return B200_ERR_UNSUPPORTED;  // a 32-token copy must stay inside one block
  return qkv_decode_attention_impl(qkv_partials, qkv_splits, qkv_bias, cosine, sine, key_pool,
                                   value_pool, lengths, output, batch, q_heads, kv_heads, head_dim,
                                   max_blocks_per_sequence * block_size, mask_len, scale, split_tokens,
                                   max_length_hint, length_offset, norm_row_squares, norm_hidden,
                                   norm_epsilon, workspace, workspace_bytes, status, stream,
                                   block_table, num_blocks, block_size, sequence_order);
}
