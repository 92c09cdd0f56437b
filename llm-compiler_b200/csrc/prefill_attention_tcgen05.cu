// serve.prefill_attention (causal-proved, bf16, fast mode) on the 5th-generation tensor cores.
//
// One CTA owns 128 query rows of one (batch, query head) and walks the key tiles 0 .. its own
// (causal: nothing beyond the diagonal tile is touched). Per 128-key tile:
//   S = Q K^T     tcgen05.mma, M 128 x N 128, K = D in steps of 16; Q and K tiles K-major in
//                 128-byte swizzled shared memory (TMA boxes), S in 128 TMEM columns (fp32)
//   softmax       four warps, one query row per thread = one TMEM lane: two passes of
//                 tcgen05.ld over the row (max, then exp2 and sum), probabilities rounded to bf16
//                 and written as the K-major A operand of the next product
//   O_j = P V     tcgen05.mma, M 128 x N D, K = 128 keys; V is used as it lies in memory (keys x
//                 D, an MN-major B operand: no transpose pass); O_j in D TMEM columns
//   O = O a + O_j in registers (a = exp2(old max - new max)): tensor memory is never rescaled
// Roles: warps 0-3 softmax + epilogue, warp 4 (one lane) TMA producer (two K buffers, one V),
// warp 5 (one lane) MMA issuer and owner of the TMEM allocation. Once P_j is written the MMA
// thread issues S of tile j + 1 and then P_j V_j: the softmax warps take the row maxima of tile
// j + 1 while O_j is computed, fold O_j, and only then overwrite P.
// Every mbarrier wait is bounded: a wait that gives up sets B200_STATUS_WAIT_TIMEOUT, TMEM is
// freed and the CTA returns. Heavier CTAs (later query tiles) are scheduled first.
#include <stdlib.h>
#include <string.h>

#include "common.cuh"
#include "tcgen05.cuh"
#include "tensor_map.cuh"

namespace b200 {
namespace {

constexpr int kTile = 128;     // query rows per CTA = keys per step
constexpr int kThreadsOneGroup = 192;  // 4 softmax warps + TMA warp + MMA warp
constexpr int kKStages = 2;  // K tiles are double-buffered, V has one buffer (see the kernel)
constexpr float kLog2e = 1.4426950408889634f;

struct PrefillTcParams {
  __nv_bfloat16* out;  // [B, T, Hq, D]
  int32_t* status;
  int q_heads, groups, tokens;
  int q_token_dim1, k_token_dim1, v_token_dim1;  // coordinate order of the three tensor maps
  float scale_log2;
};

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

// G query tiles of 128 rows per CTA. G = 2 (D = 64): two softmax groups of four warps work half
// a period apart, so the tensor core computes one group's products while the other group is in
// its softmax, and both share every K / V tile the CTA fetches. G = 1 (D = 128): one group.
// Threads: 4 G softmax warps (warp % 4 = the TMEM lane quarter it may read), then the TMA warp
// and the MMA warp. G = 2 runs one CTA per SM (ten warps, at most three on one of the four
// 16 K-register sub-partitions: up to 170 registers per thread); G = 1 at D = 64 fits two CTAs
// per SM, which needs at most 128 registers per thread.
template <int D, int G>
__global__ void __launch_bounds__(G == 2 ? 384 : (D == 64 ? 256 : kThreadsOneGroup),
                                  (G == 1 && D == 64) ? 2 : 1)
prefill_attention_tcgen05_kernel(const PrefillTcParams p, const __grid_constant__ CUtensorMap q_map,
                                 const __grid_constant__ CUtensorMap k_map,
                                 const __grid_constant__ CUtensorMap v_map) {
  constexpr int kPanels = D / 64;                         // 64-wide (128-byte) panels along D
  constexpr uint32_t kPanelBytes = kTile * 128;           // 128 rows x 128 B
  constexpr uint32_t kTileBytes = kPanels * kPanelBytes;  // one of Q, K, V
  constexpr uint32_t kPBytes = kTile * kTile * 2;         // probabilities of one group
  constexpr uint32_t kTmemColumns = G * (kTile + D) <= 256 ? 256 : 512;  // S and O_j per group
  constexpr int kTmaWarp = 4 * G, kMmaWarp = 4 * G + 1;

  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ __align__(8) uint64_t q_full, s_full[G], p_full[G], o_full[G];
  __shared__ __align__(8) uint64_t k_full[kKStages], k_empty[kKStages], v_full, v_empty;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int failed;

  TraceScope trace(7);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_block = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);  // heavy first
  const int hq = blockIdx.y, b = blockIdx.z;
  const int kvh = hq / p.groups;
  const int q0 = q_block * G * kTile;
  const int all_tiles = (p.tokens + kTile - 1) / kTile;
  // causal: group g (query tile G q_block + g) needs key tiles 0 .. its own
  int tiles_of[G];
#pragma unroll
  for (int g = 0; g < G; ++g) tiles_of[g] = min(q_block * G + g + 1, all_tiles);
  const int n_tiles = tiles_of[G - 1];

  const uint32_t q_smem = smem_u32(smem);                   // G tiles
  const uint32_t k_smem = q_smem + G * kTileBytes;          // two buffers
  const uint32_t v_smem = k_smem + kKStages * kTileBytes;   // one buffer (wanted a softmax later than K)
  const uint32_t p_smem = v_smem + kTileBytes;              // G x [2 panels][128 rows][128 B]

  if (threadIdx.x == 0) {
    failed = 0;
    mbarrier_init(smem_u32(&q_full), 1);
    for (int g = 0; g < G; ++g) {
      mbarrier_init(smem_u32(&s_full[g]), 1);
      mbarrier_init(smem_u32(&p_full[g]), 4);  // one arrival per softmax warp
      mbarrier_init(smem_u32(&o_full[g]), 1);
    }
    for (int s = 0; s < kKStages; ++s) {
      mbarrier_init(smem_u32(&k_full[s]), 1);
      mbarrier_init(smem_u32(&k_empty[s]), 1);
    }
    mbarrier_init(smem_u32(&v_full), 1);
    mbarrier_init(smem_u32(&v_empty), 1);
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

  if (warp == kTmaWarp && lane == 0) {
    // ---- TMA producer ----
    mbarrier_arrive_expect_tx(smem_u32(&q_full), G * kTileBytes);
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
      for (int panel = 0; panel < kPanels; ++panel)
        load_box(q_smem + g * kTileBytes + panel * kPanelBytes, &q_map, smem_u32(&q_full), panel * 64,
                 q0 + g * kTile, hq, b, p.q_token_dim1);
    for (int j = 0; j < n_tiles; ++j) {
      const int s = j & 1;
      if (j >= kKStages && !mbarrier_wait_bounded(smem_u32(&k_empty[s]), ((j >> 1) - 1) & 1)) {
        failed = 1;
        break;
      }
      mbarrier_arrive_expect_tx(smem_u32(&k_full[s]), kTileBytes);
#pragma unroll
      for (int panel = 0; panel < kPanels; ++panel)
        load_box(k_smem + s * kTileBytes + panel * kPanelBytes, &k_map, smem_u32(&k_full[s]),
                 panel * 64, j * kTile, kvh, b, p.k_token_dim1);
      if (j >= 1 && !mbarrier_wait_bounded(smem_u32(&v_empty), (j - 1) & 1)) {
        failed = 1;
        break;
      }
      mbarrier_arrive_expect_tx(smem_u32(&v_full), kTileBytes);
#pragma unroll
      for (int panel = 0; panel < kPanels; ++panel)
        load_box(v_smem + panel * kPanelBytes, &v_map, smem_u32(&v_full), panel * 64, j * kTile, kvh,
                 b, p.v_token_dim1);
    }
  } else if (warp == kMmaWarp && lane == 0) {
    // ---- MMA issuer ----
    constexpr uint32_t idesc_s = instruction_descriptor(kTile, kTile);
    constexpr uint32_t idesc_o = instruction_descriptor(kTile, D, true);  // V: MN-major B operand
    auto issue_s = [&](int g, int j) {  // S_g = Q_g K_j^T, K = D
      const uint32_t q_tile = q_smem + g * kTileBytes, k_tile = k_smem + (j & 1) * kTileBytes;
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const uint32_t offset = (ks / 4) * kPanelBytes + (ks % 4) * 32;
        umma_bf16(s_column(g), smem_descriptor(q_tile + offset), smem_descriptor(k_tile + offset),
                  idesc_s, ks > 0 ? 1u : 0u);
      }
      umma_commit(smem_u32(&s_full[g]));
    };
    auto issue_o = [&](int g) {  // O_j of group g = P_g V_j, K = 128 keys
      const uint32_t p_tile = p_smem + g * kPBytes;
#pragma unroll
      for (int ks = 0; ks < kTile / 16; ++ks) {
        const uint32_t p_offset = (ks / 4) * kPanelBytes + (ks % 4) * 32;
        umma_bf16(o_column(g), smem_descriptor(p_tile + p_offset),
                  smem_descriptor_mn_major(v_smem + ks * 2048, kPanelBytes), idesc_o, ks > 0 ? 1u : 0u);
      }
      umma_commit(smem_u32(&o_full[g]));
    };
    bool ok = mbarrier_spin_bounded(smem_u32(&q_full), 0) &&
              mbarrier_spin_bounded(smem_u32(&k_full[0]), 0);
    if (ok) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
      for (int g = 0; g < G; ++g) issue_s(g, 0);  // every group has key tile 0
      umma_commit(smem_u32(&k_empty[0]));  // K_0 is free once these have been computed
    }
    for (int j = 0; ok && j < n_tiles; ++j) {
      // Per group, once its softmax has written P_j (which also says that its S_j and its
      // O_{j-1} have been read): first S of the next key tile, so that the group can take the
      // row maxima of that tile while the tensor core computes O_j = P_j V_j behind it.
      const bool more = j + 1 < n_tiles;
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const bool has_tile = j < tiles_of[g];
        if (has_tile && !mbarrier_spin_bounded(smem_u32(&p_full[g]), j & 1)) {
          ok = false;
          break;
        }
        if (more && j + 1 < tiles_of[g]) {
          if (!mbarrier_spin_bounded(smem_u32(&k_full[(j + 1) & 1]), ((j + 1) >> 1) & 1)) {
            ok = false;
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          issue_s(g, j + 1);
        }
        if (more && g == G - 1) umma_commit(smem_u32(&k_empty[(j + 1) & 1]));  // K_{j+1}: all S issued
        if (has_tile) {
          if (!mbarrier_spin_bounded(smem_u32(&v_full), j & 1)) {
            ok = false;
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          issue_o(g);  // P_g is free again when o_full[g] fires
        }
        if (g == G - 1) umma_commit(smem_u32(&v_empty));  // V_j is free once its last reader retires
      }
    }
    if (!ok) failed = 1;
  } else if (warp < 4 * G) {
    // ---- softmax + epilogue: thread = query row = TMEM lane of its group ----
    const int g = warp >> 2;
    const int row = threadIdx.x & 127;
    const int q_tile = q_block * G + g;
    const int my_tiles = tiles_of[g];
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t s_taddr = s_column(g) + lane_base, o_taddr = o_column(g) + lane_base;
    const uint32_t p_tile = p_smem + g * kPBytes;
    float m_run = -INFINITY, l_run = 0.0f;
    float o[D];
#pragma unroll
    for (int i = 0; i < D; ++i) o[i] = 0.0f;
    bool ok = true;
    float alpha_pending = 0.0f;  // factor of the O_j that is still in tensor memory
    auto fold = [&](int j) {     // o = o * alpha_j + O_j
      if (!mbarrier_wait_ready_first(smem_u32(&o_full[g]), j & 1)) return false;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
      for (int c0 = 0; c0 < D; c0 += 32) {
        float v[32];
        tmem_load_32x32(o_taddr + c0, v);
#pragma unroll
        for (int i = 0; i < 32; ++i) o[c0 + i] = fmaf(o[c0 + i], alpha_pending, v[i]);
      }
      return true;
    };
    for (int j = 0; j < my_tiles; ++j) {
      if (!mbarrier_wait_ready_first(smem_u32(&s_full[g]), j & 1)) {
        ok = false;
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const bool diagonal = j == q_tile;  // keys beyond the row's own position are masked
      float row_max = -INFINITY;
#pragma unroll 1
      for (int c0 = 0; c0 < kTile; c0 += 32) {
        float s[32];
        tmem_load_32x32(s_taddr + c0, s);
        if (diagonal) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (c0 + i <= row) row_max = fmaxf(row_max, s[i]);
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) row_max = fmaxf(row_max, s[i]);
        }
      }
      const float m_new = fmaxf(m_run, row_max * p.scale_log2);  // key 0 is never masked
      const float alpha = exp2_fast(m_run - m_new);              // exp2(-inf) = 0 at the first tile
      // O_{j-1} ran on the tensor core during the pass above; P is free once it is complete
      if (j > 0 && !fold(j - 1)) {
        ok = false;
        break;
      }
      alpha_pending = alpha;
      float sum = 0.0f;
#pragma unroll 1
      for (int c0 = 0; c0 < kTile; c0 += 32) {
        float s[32];
        tmem_load_32x32(s_taddr + c0, s);
        uint32_t packed[16];
        if (diagonal) {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float p0 = exp2_fast(fmaf(s[i], p.scale_log2, -m_new));
            float p1 = exp2_fast(fmaf(s[i + 1], p.scale_log2, -m_new));
            if (c0 + i > row) p0 = 0.0f;
            if (c0 + i + 1 > row) p1 = 0.0f;
            sum += p0 + p1;
            packed[i / 2] = pack_bf16x2(p0, p1);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float p0 = exp2_fast(fmaf(s[i], p.scale_log2, -m_new));
            const float p1 = exp2_fast(fmaf(s[i + 1], p.scale_log2, -m_new));
            sum += p0 + p1;
            packed[i / 2] = pack_bf16x2(p0, p1);
          }
        }
        // K-major A operand: panel = 64 keys, row = query, 16-byte chunks XOR-swizzled by row % 8
        const uint32_t panel = p_tile + (c0 / 64) * kPanelBytes + row * 128;
#pragma unroll
        for (int chunk = 0; chunk < 4; ++chunk) {
          const int logical = (c0 % 64) / 8 + chunk;
          const uint32_t address = panel + ((logical ^ (row & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(address),
                       "r"(packed[chunk * 4]), "r"(packed[chunk * 4 + 1]),
                       "r"(packed[chunk * 4 + 2]), "r"(packed[chunk * 4 + 3]) : "memory");
        }
      }
      l_run = l_run * alpha + sum;
      m_run = m_new;
      // generic-proxy writes of P must be visible to the tensor core (async proxy)
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0)
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&p_full[g])) : "memory");
    }
    if (ok && my_tiles > 0) ok = fold(my_tiles - 1);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    const int q_row = q0 + g * kTile + row;
    if (!ok) {
      failed = 1;
    } else if (q_row < p.tokens) {
      const float inv = 1.0f / l_run;
      __nv_bfloat16* dst = p.out + ((static_cast<int64_t>(b) * p.tokens + q_row) * p.q_heads + hq) * D;
#pragma unroll
      for (int i = 0; i < D; i += 8)
        *reinterpret_cast<uint4*>(dst + i) =
            make_uint4(pack_bf16x2(o[i] * inv, o[i + 1] * inv), pack_bf16x2(o[i + 2] * inv, o[i + 3] * inv),
                       pack_bf16x2(o[i + 4] * inv, o[i + 5] * inv), pack_bf16x2(o[i + 6] * inv, o[i + 7] * inv));
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

// Called by b200_prefill_attention for causal-proved bf16 calls in the fast mode. Returns
// B200_ERR_UNSUPPORTED when this path does not apply (head_dim, strides that no tensor map can
// describe, B200_PREFILL_ATTENTION_PATH=mma.sync): the caller then uses the warp-level kernel.
int prefill_attention_tcgen05(const void* query, const void* key, const void* value, void* output,
                              int64_t batch, int64_t q_heads, int64_t kv_heads, int64_t tokens,
                              int64_t head_dim, const int64_t query_strides[4],
                              const int64_t key_strides[4], const int64_t value_strides[4],
                              double scale, int32_t* status, cudaStream_t stream) {
  if ((launch_mode() & B200_LAUNCH_PREFILL_WARP_LEVEL) != 0) return B200_ERR_UNSUPPORTED;
  const char* path = getenv("B200_PREFILL_ATTENTION_PATH");
  if (path != nullptr && strcmp(path, "mma.sync") == 0) return B200_ERR_UNSUPPORTED;
  if (head_dim != 64 && head_dim != 128) return B200_ERR_UNSUPPORTED;
  if (!(scale > 0.0) || tokens < 1) return B200_ERR_UNSUPPORTED;
  // One query tile per CTA (two CTAs per SM at D = 64) unless B200_PREFILL_QUERY_TILES=2 asks for
  // two tiles per CTA at D = 64: measured equal within 3 % either way from 1024 to 16384 tokens.
  int query_tiles = 1;
  const char* tiles_text = getenv("B200_PREFILL_QUERY_TILES");
  if (tiles_text != nullptr && strcmp(tiles_text, "2") == 0 && head_dim == 64) query_tiles = 2;
  const int64_t q_blocks = ceil_div(tokens, static_cast<int64_t>(kTile) * query_tiles);
  if (q_blocks > 65535 || q_heads > 65535 || batch > 65535) return B200_ERR_UNSUPPORTED;
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
  dim3 grid(static_cast<unsigned>(q_blocks), static_cast<unsigned>(q_heads),
            static_cast<unsigned>(batch));
  // G query tiles + two K tiles + one V tile + G tiles of probabilities
  const int tile_bytes = static_cast<int>(head_dim) * kTile * 2;
  const int smem = tile_bytes * (query_tiles + kKStages + 1) + query_tiles * kTile * kTile * 2;
  const int threads = (4 * query_tiles + 2) * 32;
  auto launch = [&](auto kernel) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
      return false;
    // two single-group CTAs per SM need the largest shared-memory carve-out
    cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                         cudaSharedmemCarveoutMaxShared);
    kernel<<<grid, threads, smem, stream>>>(p, q_map, k_map, v_map);
    return true;
  };
  bool launched;
  if (head_dim == 64)
    launched = query_tiles == 2 ? launch(prefill_attention_tcgen05_kernel<64, 2>)
                                : launch(prefill_attention_tcgen05_kernel<64, 1>);
  else
    launched = launch(prefill_attention_tcgen05_kernel<128, 1>);
  if (!launched) return B200_ERR_LAUNCH;
  return launch_status();
}

}  // namespace b200
