// serve.prefill_attention (causal-proved, bf16, fast mode) on the 5th-generation tensor cores:
// a pair of 128-row query tiles per CTA, one CTA per SM, the output accumulated in tensor memory.
//
// Two softmax groups of eight warps each own one query tile of the pair and share every K / V
// tile the CTA fetches (causal: nothing beyond a tile's diagonal is touched). Per group and
// 128-key tile:
//   S = Q K^T     tcgen05.mma M 128 x N 128 into the group's 128 TMEM columns; Q and K tiles
//                 K-major in 128-byte swizzled shared memory (TMA boxes)
//   softmax       two threads per query row (a warp may only read its own quarter of the TMEM
//                 lanes, so warps w and w + 4 share 32 rows and split the keys in halves): the
//                 half row of S is read into registers once, which frees S for the next product
//                 at once; the halves exchange their maxima through shared memory; exp2; bf16
//                 probabilities written as the K-major A operand P
//   O += P V      tcgen05.mma M 128 x N D accumulating in the group's D TMEM columns; V is used
//                 as it lies in memory (an MN-major B operand: no transpose pass)
// The running maximum is lazy: probabilities are taken against a reference maximum that is moved
// (and O and the row sums rescaled, O in tensor memory by the row's own threads) only when a
// tile raises a row's maximum by more than 8 in the log2 domain, so probabilities stay below 2^8
// and most tiles touch O only through the tensor core. The result is O / row sum.
// With the row in registers a group's next S is computed during its current softmax, and the
// tensor core works for one group while the other group's warps are in their exponentials.
// Roles: warps 0-7 and 8-15 softmax groups, warp 16 (one lane) TMA producer (two K buffers, two
// V buffers at D = 64, one at D = 128; K one tile ahead of V), warp 17 (one lane) MMA issuer and
// owner of the 512 TMEM columns (S at 0 and 128, O behind them). Every mbarrier wait is bounded:
// a wait that gives up sets B200_STATUS_WAIT_TIMEOUT, tensor memory is freed and the CTA
// returns. Query blocks are handed out heaviest first across all heads and sequences.
//
// MASKED variant: the reference's own contract, an arbitrary additive fp32 mask B x 1 x T x T
// (`causal: "mask"`, passes/prefill_attention.py:173-180). A pre-pass classifies every 128 x 128
// tile of the mask as all zero, all -inf or mixed (one read of the mask); a CTA then walks only
// the key tiles between the first and the last tile that is not all -inf for its query tiles,
// adds nothing on all-zero tiles, and on the others adds the mask values (fetched while the
// tensor core computes S, carried as bf16 pairs: exact for 0 and -inf) to the scaled scores
// before the running maximum. A causal mask given as data therefore costs what the causal-proved
// kernel costs plus the pre-pass; a row with every key masked yields NaN as in the reference.
#include <stdlib.h>
#include <string.h>

#include "common.cuh"
#include "tcgen05.cuh"
#include "tensor_map.cuh"

namespace b200 {
namespace {

constexpr int kTile = 128;    // query rows per group = keys per step
constexpr int kKStages = 2;  // K tiles are double-buffered
constexpr float kLog2e = 1.4426950408889634f;

struct PrefillTcParams {
  __nv_bfloat16* out;  // [B, T, Hq, D]
  int32_t* status;
  int q_heads, groups, tokens;
  int q_token_dim1, k_token_dim1, v_token_dim1;  // coordinate order of the three tensor maps
  float scale_log2;
  // MASKED: additive fp32 mask with a contiguous last dimension; classes of its 128 x 128 tiles
  const float* mask = nullptr;
  int64_t mask_stride_b = 0, mask_stride_q = 0;
  const uint8_t* tile_class = nullptr;  // [batch or 1][q tiles][k tiles]: 0 zero, 1 -inf, 2 mixed
  int64_t class_stride_b = 0;
  uint32_t wait_limit = 4000000u, spin_limit = 2000000u;  // polls of the bounded waits
  int drop_loads = 0;  // debug: the producer issues nothing (every wait runs out)
};

// Classes of the 128 x 128 tiles of an additive mask. Rows beyond T are ignored, key columns
// beyond T count as -inf (the attention kernel must not let zero-filled keys take part).
__global__ void __launch_bounds__(256)
mask_tile_class_kernel(const float* __restrict__ mask, int64_t stride_b, int64_t stride_q, int tokens,
                       int tiles, uint8_t* __restrict__ classes) {
  const int tk = blockIdx.x, tq = blockIdx.y, b = blockIdx.z;
  const float* base = mask + b * stride_b;
  bool nonzero = false, finite = false;  // something is not 0 / something is not -inf
  for (int item = threadIdx.x; item < 128 * 32; item += 256) {
    const int row = tq * 128 + item / 32, key = tk * 128 + (item % 32) * 4;
    if (row >= tokens) continue;
    const float* src = base + static_cast<int64_t>(row) * stride_q + key;
    if (key + 3 < tokens) {
      const float4 v = __ldg(reinterpret_cast<const float4*>(src));
      nonzero |= v.x != 0.0f || v.y != 0.0f || v.z != 0.0f || v.w != 0.0f;
      finite |= v.x != -INFINITY || v.y != -INFINITY || v.z != -INFINITY || v.w != -INFINITY;
    } else {
      for (int i = 0; i < 4; ++i) {
        const float v = key + i < tokens ? __ldg(src + i) : -INFINITY;
        nonzero |= v != 0.0f;
        finite |= v != -INFINITY;
      }
    }
  }
  const int any_nonzero = __syncthreads_or(nonzero), any_finite = __syncthreads_or(finite);
  if (threadIdx.x == 0)
    classes[(static_cast<int64_t>(b) * tiles + tq) * tiles + tk] = !any_nonzero ? 0 : (!any_finite ? 1 : 2);
}

__device__ __forceinline__ float exp2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void load_box(uint32_t dst, const CUtensorMap* map, uint32_t bar, int d0,
                                         int t0, int head, int batch, int token_dim1) {
  if (token_dim1) tma_load_4d(dst, map, bar, d0, t0, head, batch);
  else tma_load_4d(dst, map, bar, d0, head, t0, batch);
}

constexpr int kGroups = 2;
constexpr int kSoftmaxWarps = 8 * kGroups;  // two warps per 32 query rows
constexpr int kThreads = (kSoftmaxWarps + 2) * 32;  // + TMA warp + MMA warp
constexpr float kRescaleThreshold = 8.0f;  // log2 domain
constexpr uint32_t kSpinLimit = 2000000u;   // polls of an MMA thread before it gives up (about 0.1 s)

// 18 warps: five on one of the four 16 K-register sub-partitions, so at most 96 registers each.
template <int D, bool MASKED>
__global__ void __launch_bounds__(640, 1)
prefill_attention_tcgen05_kernel(const PrefillTcParams p, const __grid_constant__ CUtensorMap q_map,
                                 const __grid_constant__ CUtensorMap k_map,
                                 const __grid_constant__ CUtensorMap v_map) {
  constexpr int G = kGroups;
  constexpr int kVStages = D == 64 ? 2 : 1;               // 227 KB hold one V tile at D = 128
  // With two V buffers V_j has long landed when P_j is written and a softmax warp vouches for it;
  // a single buffer is refilled late, and only the MMA thread should wait for that.
  constexpr bool kSoftmaxChecksV = kVStages > 1;
  constexpr int kPanels = D / 64;                         // 64-wide (128-byte) panels along D
  constexpr uint32_t kPanelBytes = kTile * 128;           // 128 rows x 128 B
  constexpr uint32_t kTileBytes = kPanels * kPanelBytes;  // one of Q, K, V
  constexpr uint32_t kPBytes = kTile * kTile * 2;         // probabilities of one group
  constexpr uint32_t kTmemColumns = 512;
  constexpr int kTmaWarp = kSoftmaxWarps, kMmaWarp = kSoftmaxWarps + 1;

  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ __align__(8) uint64_t q_full, s_full[G], s_free[G], p_full[G], o_done[G];
  __shared__ __align__(8) uint64_t k_full[kKStages], k_empty[kKStages], v_full[kVStages], v_empty[kVStages];
  // Static shared memory must stay below 3 KB: at D = 128 the tiles take 224 of the 227 KB.
  __shared__ __nv_bfloat16 row_max_slot[2][G][2][kTile];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int failed;

  TraceScope trace(8);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Blocks are handed out with z slowest: every (batch, head) gets its heaviest query block (the
  // last: most key tiles) before any gets a lighter one, so the lightest blocks fill the tail.
  const int q_block = static_cast<int>(gridDim.z) - 1 - static_cast<int>(blockIdx.z);
  const int hq = blockIdx.x, b = blockIdx.y;
  const int kvh = hq / p.groups;
  const int q0 = q_block * G * kTile;
  const int all_tiles = (p.tokens + kTile - 1) / kTile;
  // Key tiles are walked from `lo` on; `j` below counts from there (buffer slots and barrier
  // phases follow j, coordinates lo + j). causal: group g (query tile G q_block + g) needs key
  // tiles 0 .. its own. MASKED: from the first to the last tile that is not all -inf for the
  // group's query tile (a group without any such tile still walks one, and yields NaN rows).
  int lo = 0, tiles_0 = min(q_block * G + 1, all_tiles), tiles_1 = min(q_block * G + 2, all_tiles);
  const uint8_t* class_row[G] = {nullptr, nullptr};
  if (MASKED) {
    int first[G], last[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const int q_tile = min(q_block * G + g, all_tiles - 1);  // (a tile past the end mirrors the last)
      class_row[g] = p.tile_class + b * p.class_stride_b + static_cast<int64_t>(q_tile) * all_tiles;
      first[g] = -1;
      last[g] = 0;
      for (int j = 0; j < all_tiles; ++j)
        if (class_row[g][j] != 1) {
          if (first[g] < 0) first[g] = j;
          last[g] = j;
        }
      if (first[g] < 0) first[g] = 0;
    }
    lo = min(first[0], first[1]);
    tiles_0 = last[0] + 1 - lo;
    tiles_1 = last[1] + 1 - lo;
    if (tiles_0 < 1) tiles_0 = 1;
    if (tiles_1 < 1) tiles_1 = 1;
  }
  auto tiles_of = [&](int g) { return g == 0 ? tiles_0 : tiles_1; };
  const int n_tiles = max(tiles_0, tiles_1);

  const uint32_t q_smem = smem_u32(smem);                   // G tiles
  const uint32_t k_smem = q_smem + G * kTileBytes;          // two buffers
  const uint32_t v_smem = k_smem + kKStages * kTileBytes;   // one or two buffers
  const uint32_t p_smem = v_smem + kVStages * kTileBytes;   // G x [2 panels][128 rows][128 B]

  if (threadIdx.x == 0) {
    failed = 0;
    mbarrier_init(smem_u32(&q_full), 1);
    for (int g = 0; g < G; ++g) {
      mbarrier_init(smem_u32(&s_full[g]), 1);
      mbarrier_init(smem_u32(&s_free[g]), 8);  // one arrival per softmax warp of the group
      mbarrier_init(smem_u32(&p_full[g]), 8);
      mbarrier_init(smem_u32(&o_done[g]), 1);
    }
    for (int s = 0; s < kKStages; ++s) {
      mbarrier_init(smem_u32(&k_full[s]), 1);
      mbarrier_init(smem_u32(&k_empty[s]), 1);
    }
    for (int s = 0; s < kVStages; ++s) {
      mbarrier_init(smem_u32(&v_full[s]), 1);
      mbarrier_init(smem_u32(&v_empty[s]), 1);
    }
    fence_mbarrier_init();
  }
  if (warp == kMmaWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&tmem_base_slot)), "r"(kTmemColumns) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_slot;
  auto s_column = [&](int g) { return tmem_base + g * kTile; };
  auto o_column = [&](int g) { return tmem_base + G * kTile + g * D; };

  if (warp == kTmaWarp && lane == 0 && !p.drop_loads) {
    // ---- TMA producer ----
    mbarrier_arrive_expect_tx(smem_u32(&q_full), G * kTileBytes);
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
      for (int panel = 0; panel < kPanels; ++panel)
        load_box(q_smem + g * kTileBytes + panel * kPanelBytes, &q_map, smem_u32(&q_full), panel * 64,
                 q0 + g * kTile, hq, b, p.q_token_dim1);
    // K runs one tile ahead of V: K_{j+1} is wanted early in the softmax of tile j (for the next
    // S), V_j only at its end, and a single V buffer is not free before the previous P V is done.
    auto load_k = [&](int j) {
      const int s = j % kKStages, use = j / kKStages;
      if (use > 0 && !mbarrier_wait_bounded(smem_u32(&k_empty[s]), (use - 1) & 1, p.wait_limit)) return false;
      mbarrier_arrive_expect_tx(smem_u32(&k_full[s]), kTileBytes);
#pragma unroll
      for (int panel = 0; panel < kPanels; ++panel)
        load_box(k_smem + s * kTileBytes + panel * kPanelBytes, &k_map, smem_u32(&k_full[s]),
                 panel * 64, (lo + j) * kTile, kvh, b, p.k_token_dim1);
      return true;
    };
    bool ok = load_k(0);
    for (int j = 0; ok && j < n_tiles; ++j) {
      if (j + 1 < n_tiles) ok = load_k(j + 1);
      if (!ok) break;
      const int vs = j % kVStages, v_use = j / kVStages;
      ok = v_use == 0 || mbarrier_wait_bounded(smem_u32(&v_empty[vs]), (v_use - 1) & 1, p.wait_limit);
      if (!ok) break;
      mbarrier_arrive_expect_tx(smem_u32(&v_full[vs]), kTileBytes);
#pragma unroll
      for (int panel = 0; panel < kPanels; ++panel)
        load_box(v_smem + vs * kTileBytes + panel * kPanelBytes, &v_map, smem_u32(&v_full[vs]),
                 panel * 64, (lo + j) * kTile, kvh, b, p.v_token_dim1);
    }
    if (!ok) failed = 1;
  } else if (warp == kMmaWarp && lane == 0) {
    // ---- MMA issuer ----
    // A poll that follows a tcgen05.commit of the same thread takes a few hundred cycles, so this
    // thread polls as little as it can: that a K or V tile has landed is checked by a softmax
    // warp before it reports S read or P written.
    constexpr uint32_t idesc_s = instruction_descriptor(kTile, kTile);
    constexpr uint32_t idesc_o = instruction_descriptor(kTile, D, true);  // V: MN-major B operand
    const uint64_t q_desc = smem_descriptor(q_smem), k_desc = smem_descriptor(k_smem);
    const uint64_t p_desc = smem_descriptor(p_smem);
    const uint64_t v_desc = smem_descriptor_mn_major(v_smem, kPanelBytes);
    auto issue_s = [&](int g, int j) {  // S_g = Q_g K_j^T, K = D
      const uint64_t a = descriptor_advance(q_desc, g * kTileBytes);
      const uint64_t bd = descriptor_advance(k_desc, (j % kKStages) * kTileBytes);
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const uint32_t offset = (ks / 4) * kPanelBytes + (ks % 4) * 32;
        umma_bf16(s_column(g), descriptor_advance(a, offset), descriptor_advance(bd, offset), idesc_s,
                  ks > 0 ? 1u : 0u);
      }
      umma_commit(smem_u32(&s_full[g]));
    };
    auto issue_o = [&](int g, int j) {  // O_g (+)= P_g V_j, K = 128 keys
      const uint64_t a = descriptor_advance(p_desc, g * kPBytes);
      const uint64_t bd = descriptor_advance(v_desc, (j % kVStages) * kTileBytes);
#pragma unroll
      for (int ks = 0; ks < kTile / 16; ++ks) {
        const uint32_t p_offset = (ks / 4) * kPanelBytes + (ks % 4) * 32;
        umma_bf16(o_column(g), descriptor_advance(a, p_offset), descriptor_advance(bd, ks * 2048),
                  idesc_o, (j > 0 || ks > 0) ? 1u : 0u);
      }
      umma_commit(smem_u32(&o_done[g]));
    };
    bool ok = mbarrier_spin_bounded(smem_u32(&q_full), 0, p.spin_limit) &&
              mbarrier_spin_bounded(smem_u32(&k_full[0]), 0, p.spin_limit);
    if (ok) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
      for (int g = 0; g < G; ++g) issue_s(g, 0);  // every group has key tile 0
      umma_commit(smem_u32(&k_empty[0]));
    }
    for (int j = 0; ok && j < n_tiles; ++j) {
      // S of the next key tile as soon as a group holds its current row of S in registers (its
      // report also says that K_{j+1} has landed) ...
      const bool more = j + 1 < n_tiles;
#pragma unroll
      for (int g = 0; g < G; ++g) {
        if (ok && more && j + 1 < tiles_of(g)) {
          ok = mbarrier_spin_bounded(smem_u32(&s_free[g]), j & 1, p.spin_limit);
          if (ok) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            issue_s(g, j + 1);
          }
        }
      }
      if (ok && more) umma_commit(smem_u32(&k_empty[(j + 1) % kKStages]));  // K_{j+1}: all S issued
      // ... and O += P V once the group has written its probabilities (and has seen V_j land)
      bool v_landed = kSoftmaxChecksV;
#pragma unroll
      for (int g = 0; g < G; ++g) {
        if (ok && j < tiles_of(g)) {
          ok = mbarrier_spin_bounded(smem_u32(&p_full[g]), j & 1, p.spin_limit) &&
               (v_landed ||
                mbarrier_spin_bounded(smem_u32(&v_full[j % kVStages]), (j / kVStages) & 1, p.spin_limit));
          v_landed = true;
          if (ok) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            issue_o(g, j);
          }
        }
      }
      if (ok) umma_commit(smem_u32(&v_empty[j % kVStages]));  // V_j is free once its last reader retires
    }
    if (!ok) failed = 1;
  } else if (warp < kSoftmaxWarps) {
    // ---- softmax + epilogue: two threads per query row, each with one half of the keys ----
    // Warp w of a group may read the TMEM lanes 32 (w % 4) ..: warps w and w + 4 share 32 query
    // rows and split the 128 key columns (and, where O is touched, its D columns) in halves.
    const int g = warp >> 3, half = (warp >> 2) & 1;
    const int row = ((warp & 3) << 5) | lane;
    const int q_tile = q_block * G + g;
    const int my_tiles = tiles_of(g);
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t s_taddr = s_column(g) + lane_base + half * 64;
    const uint32_t o_taddr = o_column(g) + lane_base + half * (D / 2);
    const uint32_t p_row = p_smem + g * kPBytes + half * kPanelBytes + row * 128;  // panel = 64 keys
    const uint32_t swizzle = row & 7;
    const int key0 = half * 64;               // first key column of this thread inside a tile
    const uint32_t group_barrier = 1 + g;     // named barrier of the group's 256 threads
    float m_ref = -INFINITY, l_run = 0.0f;
    bool ok = true;
    for (int j = 0; j < my_tiles; ++j) {
      // A wait that gives up ends this warp's work, but the warp keeps meeting the group at the
      // named barrier once per tile. (Every wait's outcome is made warp-uniform: the
      // tensor-memory accesses are warp-collective.)
      // MASKED: a tile of class "zero" takes the same path as the causal-proved kernel (raw scores,
      // the scale folded into the exponent). For a "mixed" tile this thread's 64 mask values (two
      // 128-byte lines of its mask row) are requested into L2 while the tensor core computes S,
      // read once S is in registers, and the scores move to the log2 domain with the mask added.
      // Nothing of the mask is held in registers across the wait: the kernel sits at its
      // register cap, and the zero tiles are the common case.
      bool mixed = false;  // uniform over the group
      const float* mask_src = nullptr;
      bool mask_whole = false;  // all 64 values exist: 16-byte loads
      if (MASKED) {
        mixed = class_row[g][lo + j] != 0;
        if (mixed) {
          const int q_abs = q0 + g * kTile + row, key_abs = (lo + j) * kTile + key0;
          mask_src = p.mask + b * p.mask_stride_b + static_cast<int64_t>(min(q_abs, p.tokens - 1)) * p.mask_stride_q + key_abs;
          mask_whole = q_abs < p.tokens && key_abs + 64 <= p.tokens;
          if (mask_whole) {
            asm volatile("prefetch.global.L2 [%0];" ::"l"(mask_src));
            asm volatile("prefetch.global.L2 [%0];" ::"l"(mask_src + 32));
          }
        }
      }
      const float to_log2 = MASKED && mixed ? 1.0f : p.scale_log2;
      ok = ok && __all_sync(0xffffffffu, mbarrier_wait_ready_first(smem_u32(&s_full[g]), j & 1, p.wait_limit));
      uint32_t s0[32], s1[32];  // this thread's half of the row of S
      __nv_bfloat16 half_max = __float2bfloat16_rn(0.0f);
      if (ok) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (MASKED && mixed) {
          // scores to the log2 domain, mask added, one half at a time
          const int q_abs = q0 + g * kTile + row, key_abs = (lo + j) * kTile + key0;
          // (the tensor-memory wait is warp-collective: it stays outside the per-thread branches)
          auto add_mask = [&](uint32_t (&s)[32], int first) {
            float4 m[8];
            if (mask_whole) {
#pragma unroll
              for (int c = 0; c < 8; ++c) m[c] = __ldg(reinterpret_cast<const float4*>(mask_src + first) + c);
            } else {  // a ragged edge: rows past T add nothing, keys past T are masked out
              auto value = [&](int i) {
                return q_abs >= p.tokens ? 0.0f
                       : (key_abs + first + i < p.tokens ? __ldg(mask_src + first + i) : -INFINITY);
              };
#pragma unroll
              for (int c = 0; c < 8; ++c)
                m[c] = make_float4(value(4 * c), value(4 * c + 1), value(4 * c + 2), value(4 * c + 3));
            }
            tmem_load_wait(s);
#pragma unroll
            for (int c = 0; c < 8; ++c) {
              s[4 * c] = __float_as_uint(fmaf(__uint_as_float(s[4 * c]), p.scale_log2, m[c].x * kLog2e));
              s[4 * c + 1] = __float_as_uint(fmaf(__uint_as_float(s[4 * c + 1]), p.scale_log2, m[c].y * kLog2e));
              s[4 * c + 2] = __float_as_uint(fmaf(__uint_as_float(s[4 * c + 2]), p.scale_log2, m[c].z * kLog2e));
              s[4 * c + 3] = __float_as_uint(fmaf(__uint_as_float(s[4 * c + 3]), p.scale_log2, m[c].w * kLog2e));
            }
          };
          tmem_load_32x32_issue(s_taddr, s0);
          add_mask(s0, 0);
          tmem_load_32x32_issue(s_taddr + 32, s1);
          add_mask(s1, 32);
        } else {
          tmem_load_32x32_issue(s_taddr, s0);
          tmem_load_32x32_issue(s_taddr + 32, s1);
          tmem_load_wait(s0);
          tmem_load_wait(s1);
        }
        // S is free for the product with the next key tile
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) {
          // the group's first warp vouches for K_{j+1}: the MMA thread then needs one poll, not two
          bool landed = true;
          if ((warp & 7) == 0 && j + 1 < my_tiles)
            landed = mbarrier_wait_ready_first(smem_u32(&k_full[(j + 1) % kKStages]), ((j + 1) / kKStages) & 1,
                                               p.wait_limit);
          if (landed)
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&s_free[g])) : "memory");
          else
            failed = 1;
        }
        if (!MASKED && j == q_tile) {  // diagonal tile: keys beyond the row's own position are masked
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            if (key0 + i > row) s0[i] = 0xff800000u;
            if (key0 + i + 32 > row) s1[i] = 0xff800000u;
          }
        }
        float max0 = -INFINITY, max1 = -INFINITY, max2 = -INFINITY, max3 = -INFINITY;
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          max0 = fmaxf(max0, __uint_as_float(s0[i]));
          max1 = fmaxf(max1, __uint_as_float(s0[i + 1]));
          max2 = fmaxf(max2, __uint_as_float(s1[i]));
          max3 = fmaxf(max3, __uint_as_float(s1[i + 1]));
        }
        half_max = __float2bfloat16_rn(fmaxf(fmaxf(max0, max1), fmaxf(max2, max3)));
      }
      // The two halves of a row exchange their maxima (two slots: a thread may be one tile ahead),
      // rounded to bf16 on both sides so that both take the same reference: it only has to be
      // near the maximum, not equal to it.
      row_max_slot[j & 1][g][half][row] = half_max;
      asm volatile("bar.sync %0, 256;" ::"r"(group_barrier) : "memory");
      // (the scores of a mixed tile are in the log2 domain already)
      const float m_tile = fmaxf(__bfloat162float(half_max),
                                 __bfloat162float(row_max_slot[j & 1][g][half ^ 1][row])) * to_log2;
      if (ok && j == 0) m_ref = m_tile;  // O is still empty: the first product overwrites it
      if (ok && j > 0) {
        const bool raise = __any_sync(0xffffffffu, m_tile > m_ref + kRescaleThreshold);
        // P and O are in use until the group's previous product has completed
        ok = __all_sync(0xffffffffu, mbarrier_wait_ready_first(smem_u32(&o_done[g]), (j - 1) & 1, p.wait_limit));
        if (ok && raise) {  // warp-uniform: move the reference maximum of the warp's rows
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const float m_new = fmaxf(m_ref, m_tile);
          // (a row that has seen only -inf so far holds O = 0 and sum 0: any factor keeps them)
          const float factor = m_ref == -INFINITY ? 0.0f : exp2_fast(m_ref - m_new);
          l_run *= factor;
          m_ref = m_new;
#pragma unroll
          for (int c0 = 0; c0 < D / 2; c0 += 32) {  // this thread's half of the row of O
            float v[32];
            tmem_load_32x32(o_taddr + c0, v);
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] *= factor;
            tmem_store_32x32(o_taddr + c0, v);
          }
          tmem_store_wait();
        }
      }
      if (!ok) continue;
      // (a reference of -inf, every key so far masked, must not turn -inf - -inf into NaN)
      const float neg_ref = MASKED && m_ref == -INFINITY ? 0.0f : -m_ref;
      float sum0 = 0.0f, sum1 = 0.0f;
      auto emit = [&](const uint32_t (&s)[32], int c0) {  // 32 probabilities: exp2, sum, bf16, store
        uint32_t packed[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float p0 = exp2_fast(fmaf(__uint_as_float(s[i]), to_log2, neg_ref));
          const float p1 = exp2_fast(fmaf(__uint_as_float(s[i + 1]), to_log2, neg_ref));
          sum0 += p0;
          sum1 += p1;
          packed[i / 2] = pack_bf16x2(p0, p1);
        }
        // K-major A operand: row = query, 16-byte chunks of the 128-byte row XOR-swizzled by row % 8
#pragma unroll
        for (int chunk = 0; chunk < 4; ++chunk) {
          const uint32_t logical = c0 / 8 + chunk;
          const uint32_t address = p_row + ((logical ^ swizzle) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(address),
                       "r"(packed[chunk * 4]), "r"(packed[chunk * 4 + 1]),
                       "r"(packed[chunk * 4 + 2]), "r"(packed[chunk * 4 + 3]) : "memory");
        }
      };
      emit(s0, 0);
      emit(s1, 32);
      l_run += sum0 + sum1;
      // generic-proxy writes of P must be visible to the tensor core (async proxy)
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) {
        bool landed = true;  // likewise for V_j
        if (kSoftmaxChecksV && (warp & 7) == 0)
          landed = mbarrier_wait_ready_first(smem_u32(&v_full[j % kVStages]), (j / kVStages) & 1, p.wait_limit);
        if (landed)
          asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&p_full[g])) : "memory");
        else
          failed = 1;
      }
    }
    if (ok && my_tiles > 0)
      ok = __all_sync(0xffffffffu, mbarrier_wait_ready_first(smem_u32(&o_done[g]), (my_tiles - 1) & 1, p.wait_limit));
    // The row sum is the sum of the two halves (both took the same reference maximum); they meet
    // in the first K buffer, which nothing reads any more once the last product has completed
    // (on the failure path the sums are not used).
    float* row_sum_slot = reinterpret_cast<float*>(smem + G * kTileBytes) + g * 2 * kTile;
    row_sum_slot[half * kTile + row] = l_run;
    asm volatile("bar.sync %0, 256;" ::"r"(group_barrier) : "memory");
    const int q_row = q0 + g * kTile + row;
    if (!ok) {
      failed = 1;
    } else {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const float inv = 1.0f / (l_run + row_sum_slot[(half ^ 1) * kTile + row]);
      __nv_bfloat16* dst = p.out + ((static_cast<int64_t>(b) * p.tokens + q_row) * p.q_heads + hq) * D +
                           half * (D / 2);
#pragma unroll
      for (int c0 = 0; c0 < D / 2; c0 += 32) {
        float v[32];
        tmem_load_32x32(o_taddr + c0, v);  // warp-collective: rows past the end load too
        if (q_row < p.tokens) {
#pragma unroll
          for (int i = 0; i < 32; i += 8)
            *reinterpret_cast<uint4*>(dst + c0 + i) = make_uint4(
                pack_bf16x2(v[i] * inv, v[i + 1] * inv), pack_bf16x2(v[i + 2] * inv, v[i + 3] * inv),
                pack_bf16x2(v[i + 4] * inv, v[i + 5] * inv), pack_bf16x2(v[i + 6] * inv, v[i + 7] * inv));
        }
      }
    }
  }
  __syncwarp();
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (failed && threadIdx.x == 0 && p.status != nullptr) atomicOr(p.status, B200_STATUS_WAIT_TIMEOUT);
  if (warp == kMmaWarp)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemColumns)
                 : "memory");
  trace.mark(1);
}

}  // namespace

// Bytes of tile classes the masked variant needs in the caller's workspace.
int64_t prefill_attention_tcgen05_workspace_bytes(int64_t batch, int64_t tokens) {
  const int64_t tiles = ceil_div(tokens, static_cast<int64_t>(kTile));
  return (batch * tiles * tiles + 255) / 256 * 256;
}

// Called by b200_prefill_attention for bf16 calls in the fast mode: causal-proved (mask ==
// nullptr), or with an additive fp32 mask whose last dimension is contiguous (mask_strides in
// elements; a batch stride of 0 is one mask for every sequence), in which case `workspace` must
// hold prefill_attention_tcgen05_workspace_bytes(batch, tokens). Returns B200_ERR_UNSUPPORTED
// when this path does not apply (head_dim, strides that no tensor map can describe, a mask
// layout without 16-byte rows, B200_PREFILL_ATTENTION_PATH=mma.sync): the caller then uses the
// warp-level kernel.
int prefill_attention_tcgen05(const void* query, const void* key, const void* value, void* output,
                              int64_t batch, int64_t q_heads, int64_t kv_heads, int64_t tokens,
                              int64_t head_dim, const int64_t query_strides[4],
                              const int64_t key_strides[4], const int64_t value_strides[4],
                              double scale, int32_t* status, cudaStream_t stream, const void* mask,
                              const int64_t* mask_strides, void* workspace, int64_t workspace_bytes) {
  if ((launch_mode() & B200_LAUNCH_PREFILL_WARP_LEVEL) != 0) return B200_ERR_UNSUPPORTED;
  const char* path = getenv("B200_PREFILL_ATTENTION_PATH");
  if (path != nullptr && strcmp(path, "mma.sync") == 0) return B200_ERR_UNSUPPORTED;
  if (head_dim != 64 && head_dim != 128) return B200_ERR_UNSUPPORTED;
  if (!(scale > 0.0) || tokens < 1) return B200_ERR_UNSUPPORTED;
  const int64_t q_blocks = ceil_div(tokens, static_cast<int64_t>(kTile) * kGroups);
  if (q_blocks > 65535 || batch > 65535) return B200_ERR_UNSUPPORTED;
  const int64_t tiles = ceil_div(tokens, static_cast<int64_t>(kTile));
  if (mask != nullptr) {
    if (mask_strides == nullptr || mask_strides[3] != 1 || mask_strides[0] % 4 != 0 ||
        mask_strides[2] % 4 != 0 || !aligned16(mask) || tiles > 65535)
      return B200_ERR_UNSUPPORTED;
    if (workspace == nullptr || workspace_bytes < prefill_attention_tcgen05_workspace_bytes(batch, tokens))
      return B200_ERR_WORKSPACE;
  }
  CUtensorMap q_map, k_map, v_map;
  bool q_dim1, k_dim1, v_dim1;
  if (!make_bf16_bhtd_map(&q_map, query, batch, q_heads, tokens, head_dim, query_strides[0],
                          query_strides[1], query_strides[2], kTile, &q_dim1) ||
      !make_bf16_bhtd_map(&k_map, key, batch, kv_heads, tokens, head_dim, key_strides[0],
                          key_strides[1], key_strides[2], kTile, &k_dim1) ||
      !make_bf16_bhtd_map(&v_map, value, batch, kv_heads, tokens, head_dim, value_strides[0],
                          value_strides[1], value_strides[2], kTile, &v_dim1))
    return B200_ERR_UNSUPPORTED;
  PrefillTcParams p;
  p.out = static_cast<__nv_bfloat16*>(output);
  p.status = status;
  p.q_heads = static_cast<int>(q_heads);
  p.groups = static_cast<int>(q_heads / kv_heads);
  p.tokens = static_cast<int>(tokens);
  p.q_token_dim1 = q_dim1 ? 1 : 0;
  p.k_token_dim1 = k_dim1 ? 1 : 0;
  p.v_token_dim1 = v_dim1 ? 1 : 0;
  p.scale_log2 = static_cast<float>(scale) * kLog2e;
  p.wait_limit = wait_limit();
  p.spin_limit = p.wait_limit < kSpinLimit ? p.wait_limit : kSpinLimit;
  p.drop_loads = drop_loads();
  if (mask != nullptr) {
    const int64_t distinct = mask_strides[0] == 0 ? 1 : batch;  // one mask for all: classified once
    p.mask = static_cast<const float*>(mask);
    p.mask_stride_b = mask_strides[0];
    p.mask_stride_q = mask_strides[2];
    p.tile_class = static_cast<const uint8_t*>(workspace);
    p.class_stride_b = mask_strides[0] == 0 ? 0 : tiles * tiles;
    mask_tile_class_kernel<<<dim3(static_cast<unsigned>(tiles), static_cast<unsigned>(tiles),
                                  static_cast<unsigned>(distinct)), 256, 0, stream>>>(
        p.mask, p.mask_stride_b, p.mask_stride_q, p.tokens, static_cast<int>(tiles),
        static_cast<uint8_t*>(workspace));
  }
  dim3 grid(static_cast<unsigned>(q_heads), static_cast<unsigned>(batch), static_cast<unsigned>(q_blocks));
  const int tile_bytes = static_cast<int>(head_dim) * kTile * 2;
  const int v_stages = head_dim == 64 ? 2 : 1;
  // the pair of Q tiles, two K tiles, one or two V tiles, the pair of probability tiles
  const int smem = tile_bytes * (kGroups + kKStages + v_stages) + kGroups * kTile * kTile * 2;
  auto launch = [&](auto kernel) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
      return false;
    kernel<<<grid, kThreads, smem, stream>>>(p, q_map, k_map, v_map);
    return true;
  };
  bool launched;
  if (mask != nullptr)
    launched = head_dim == 64 ? launch(prefill_attention_tcgen05_kernel<64, true>)
                              : launch(prefill_attention_tcgen05_kernel<128, true>);
  else
    launched = head_dim == 64 ? launch(prefill_attention_tcgen05_kernel<64, false>)
                              : launch(prefill_attention_tcgen05_kernel<128, false>);
  if (!launched) return B200_ERR_LAUNCH;
  return launch_status();
}

}  // namespace b200
