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
// warp 5 (one lane) MMA issuer and owner of the TMEM allocation. The MMA thread issues S of tile
// j + 1 right behind P V of tile j, so the tensor core works while the softmax warps fold O_j.
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
constexpr int kThreads = 192;  // 4 softmax warps + TMA warp + MMA warp
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

// Launch bounds: at D = 64 two CTAs share an SM, which needs at most 128 registers per thread
// (the register file is split over four sub-partitions of 16 K registers; two of a CTA's six
// warps land on the same one). Declaring 256 threads x 2 CTAs makes the compiler keep to that.
template <int D>
__global__ void __launch_bounds__(D == 64 ? 256 : kThreads, D == 64 ? 2 : 1)
prefill_attention_tcgen05_kernel(const PrefillTcParams p, const __grid_constant__ CUtensorMap q_map,
                                 const __grid_constant__ CUtensorMap k_map,
                                 const __grid_constant__ CUtensorMap v_map) {
  constexpr int kPanels = D / 64;                   // 64-wide (128-byte) panels along D
  constexpr uint32_t kPanelBytes = kTile * 128;     // 128 rows x 128 B
  constexpr uint32_t kTileBytes = kPanels * kPanelBytes;  // one of Q, K, V
  constexpr uint32_t kTmemColumns = 256;            // S: 128, O_j: D
  constexpr uint32_t kSColumn = 0, kOColumn = 128;

  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ __align__(8) uint64_t q_full, s_full, p_full, o_full;
  __shared__ __align__(8) uint64_t k_full[kKStages], k_empty[kKStages], v_full, v_empty;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int failed;

  TraceScope trace(7);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_tile = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);  // heavy first
  const int hq = blockIdx.y, b = blockIdx.z;
  const int kvh = hq / p.groups;
  const int q0 = q_tile * kTile;
  const int n_tiles = q_tile + 1;  // causal: key tiles 0 .. the diagonal one

  const uint32_t q_smem = smem_u32(smem);
  // K_{j+1} is wanted the moment P V_j has been issued, V_{j+1} only a softmax later: two K
  // buffers and one V buffer keep the CTA below half of the shared memory at D = 64, so that
  // two CTAs share an SM and fill each other's softmax gaps on the tensor core.
  const uint32_t k_smem = q_smem + kTileBytes;
  const uint32_t v_smem = k_smem + kKStages * kTileBytes;
  const uint32_t p_smem = v_smem + kTileBytes;  // [2 panels][128 rows][128 B]

  if (threadIdx.x == 0) {
    failed = 0;
    mbarrier_init(smem_u32(&q_full), 1);
    mbarrier_init(smem_u32(&s_full), 1);
    mbarrier_init(smem_u32(&p_full), 4);  // one arrival per softmax warp
    mbarrier_init(smem_u32(&o_full), 1);
    for (int s = 0; s < kKStages; ++s) {
      mbarrier_init(smem_u32(&k_full[s]), 1);
      mbarrier_init(smem_u32(&k_empty[s]), 1);
    }
    mbarrier_init(smem_u32(&v_full), 1);
    mbarrier_init(smem_u32(&v_empty), 1);
    fence_mbarrier_init();
  }
  if (warp == 5) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&tmem_base_slot)), "r"(kTmemColumns) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_slot;

  if (warp == 4 && lane == 0) {
    // ---- TMA producer ----
    mbarrier_arrive_expect_tx(smem_u32(&q_full), kTileBytes);
#pragma unroll
    for (int panel = 0; panel < kPanels; ++panel)
      load_box(q_smem + panel * kPanelBytes, &q_map, smem_u32(&q_full), panel * 64, q0, hq, b,
               p.q_token_dim1);
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
  } else if (warp == 5 && lane == 0) {
    // ---- MMA issuer ----
    constexpr uint32_t idesc_s = instruction_descriptor(kTile, kTile);
    constexpr uint32_t idesc_o = instruction_descriptor(kTile, D, true);  // V: MN-major B operand
    auto issue_s = [&](int j) {  // S = Q K_j^T, K = D
      const uint32_t k_tile = k_smem + (j & 1) * kTileBytes;
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const uint32_t offset = (ks / 4) * kPanelBytes + (ks % 4) * 32;
        umma_bf16(tmem_base + kSColumn, smem_descriptor(q_smem + offset),
                  smem_descriptor(k_tile + offset), idesc_s, ks > 0 ? 1u : 0u);
      }
      umma_commit(smem_u32(&s_full));
      umma_commit(smem_u32(&k_empty[j & 1]));  // K_j is free once S_j has been computed
    };
    bool ok = mbarrier_wait_bounded(smem_u32(&q_full), 0) &&
              mbarrier_wait_bounded(smem_u32(&k_full[0]), 0);
    if (ok) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      issue_s(0);
    }
    for (int j = 0; ok && j < n_tiles; ++j) {
      // O_j = P V_j once the softmax warps have written P (which also says S and O_{j-1} are read)
      if (!mbarrier_wait_bounded(smem_u32(&p_full), j & 1) ||
          !mbarrier_wait_bounded(smem_u32(&v_full), j & 1)) {
        ok = false;
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t v_tile = v_smem;
#pragma unroll
      for (int ks = 0; ks < kTile / 16; ++ks) {
        const uint32_t p_offset = (ks / 4) * kPanelBytes + (ks % 4) * 32;
        umma_bf16(tmem_base + kOColumn, smem_descriptor(p_smem + p_offset),
                  smem_descriptor_mn_major(v_tile + ks * 2048, kPanelBytes), idesc_o,
                  ks > 0 ? 1u : 0u);
      }
      umma_commit(smem_u32(&o_full));
      umma_commit(smem_u32(&v_empty));  // V_j is free once these MMAs retire
      if (j + 1 < n_tiles) {
        if (!mbarrier_wait_bounded(smem_u32(&k_full[(j + 1) & 1]), ((j + 1) >> 1) & 1)) {
          ok = false;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        issue_s(j + 1);  // its commit also covers P V_j: P is free when s_full fires
      }
    }
    if (!ok) failed = 1;
  } else if (warp < 4) {
    // ---- softmax + epilogue: thread = query row = TMEM lane ----
    const int row = threadIdx.x;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
    float m_run = -INFINITY, l_run = 0.0f;
    float o[D];
#pragma unroll
    for (int i = 0; i < D; ++i) o[i] = 0.0f;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      if (!mbarrier_wait_bounded(smem_u32(&s_full), j & 1)) {
        ok = false;
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const bool diagonal = j == q_tile;  // keys beyond the row's own position are masked
      float row_max = -INFINITY;
#pragma unroll 1
      for (int c0 = 0; c0 < kTile; c0 += 32) {
        float s[32];
        tmem_load_32x32(lane_base + kSColumn + c0, s);
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
      float sum = 0.0f;
#pragma unroll 1
      for (int c0 = 0; c0 < kTile; c0 += 32) {
        float s[32];
        tmem_load_32x32(lane_base + kSColumn + c0, s);
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
        const uint32_t panel = p_smem + (c0 / 64) * kPanelBytes + row * 128;
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
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&p_full)) : "memory");
      if (!mbarrier_wait_bounded(smem_u32(&o_full), j & 1)) {
        ok = false;
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
      for (int c0 = 0; c0 < D; c0 += 32) {
        float v[32];
        tmem_load_32x32(lane_base + kOColumn + c0, v);
#pragma unroll
        for (int i = 0; i < 32; ++i) o[c0 + i] = fmaf(o[c0 + i], alpha, v[i]);
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    if (!ok) {
      failed = 1;
    } else if (q0 + row < p.tokens) {
      const float inv = 1.0f / l_run;
      __nv_bfloat16* dst = p.out + ((static_cast<int64_t>(b) * p.tokens + q0 + row) * p.q_heads + hq) * D;
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
  if (warp == 5)
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
  const int64_t q_tiles = ceil_div(tokens, kTile);
  if (q_tiles > 65535 || q_heads > 65535 || batch > 65535) return B200_ERR_UNSUPPORTED;
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
  dim3 grid(static_cast<unsigned>(q_tiles), static_cast<unsigned>(q_heads),
            static_cast<unsigned>(batch));
  // Q + two K tiles + one V tile + P
  const int smem = static_cast<int>(head_dim) * kTile * 2 * (2 + kKStages) + kTile * kTile * 2;
  if (head_dim == 64) {
    auto kernel = prefill_attention_tcgen05_kernel<64>;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
      return B200_ERR_LAUNCH;
    // two CTAs per SM need the largest shared-memory carve-out
    cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                         cudaSharedmemCarveoutMaxShared);
    kernel<<<grid, kThreads, smem, stream>>>(p, q_map, k_map, v_map);
  } else {
    auto kernel = prefill_attention_tcgen05_kernel<128>;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
      return B200_ERR_LAUNCH;
    kernel<<<grid, kThreads, smem, stream>>>(p, q_map, k_map, v_map);
  }
  return launch_status();
}

}  // namespace b200
