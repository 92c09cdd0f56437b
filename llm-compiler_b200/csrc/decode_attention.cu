// GQA decode attention over the physical B x C x Hkv x D KV buffers with per-sequence
// device lengths: split-KV online softmax.
//
// bf16 kernel. Grid (split, kv-head block, batch). A CTA owns one (sequence, KV head,
// split of `split_tokens` tokens) and serves ALL grouped query heads of that KV head
// from one read of K and V: the G query heads are the M rows (padded to 16) of
// warp-level tensor-core tiles, S = Q K^T and O += P V. The CTA's 4 warps take
// interleaved 16-token sub-tiles; each warp streams its own sub-tiles through a
// private multi-stage cp.async ring (16-byte copies, XOR-swizzled rows), so the main
// loop has no CTA-wide barrier. Loop bounds come from lengths[b] on the device, never
// from the capacity. Warps merge their (max, sum, O) partials through shared memory;
// with more than one split the CTA writes an fp32 partial and a small merge kernel
// combines the splits.
//
// Algorithmic traffic per call: every valid K and V byte once (2 * len * Hkv * D * 2 B
// per sequence) + Q + O; the split partials add 4*(D+2) bytes per (q head, split).
#include <math.h>

#include "common.cuh"

namespace b200 {
namespace {

constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;
constexpr int kSubTokens = 16;  // tokens per warp step (two n=8 MMA tiles)
constexpr float kLog2e = 1.4426950408889634f;

struct DecodeParams {
  const __nv_bfloat16* q;
  const __nv_bfloat16* kbuf;
  const __nv_bfloat16* vbuf;
  const int64_t* lengths;
  const void* mask;
  __nv_bfloat16* out;
  float* ws_o;   // [B, Hq, splits, D]
  float* ws_ml;  // [B, Hq, splits, 2]  (max in log2 domain, sum)
  int32_t* status;
  int64_t q_batch_stride, q_head_stride, mask_batch_stride;
  int batch, q_heads, kv_heads, groups, capacity, mask_len, split_tokens, num_splits;
  int mask_dtype;  // B200_F32 / B200_BF16
  int compat;      // keep the reference's bf16 rounding of the scores
  float scale;
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float load_mask(const void* mask, int dtype, int64_t index) {
  if (dtype == B200_F32) return static_cast<const float*>(mask)[index];
  return __bfloat162float(static_cast<const __nv_bfloat16*>(mask)[index]);
}

template <int D>
__device__ __forceinline__ uint32_t tile_offset(int row, int chunk) {
  // rows of D bf16; 16-byte chunks XOR-swizzled inside each 128-byte segment
  return static_cast<uint32_t>(row * (D * 2) + (((chunk & ~7) | ((chunk ^ row) & 7)) << 4));
}

template <int D, int STAGES, bool WIDE>  // WIDE: groups > 8, rows 8..15 of the tile are live
__global__ void __launch_bounds__(kThreads)
decode_attention_kernel(const DecodeParams p) {
  constexpr int kChunksPerRow = D / 8;
  constexpr int kTileBytes = kSubTokens * D * 2;    // one of K or V, one stage
  constexpr int kStageBytes = 2 * kTileBytes;
  constexpr int kWarpBytes = STAGES * kStageBytes;
  constexpr int kCopiesPerLane = kSubTokens * kChunksPerRow / 32;
  constexpr int kKSteps = D / 16;
  constexpr int kNTiles = D / 8;

  extern __shared__ __align__(1024) unsigned char smem[];

  const int split = blockIdx.x;
  const int head_block = blockIdx.y;  // kv head * blocks-per-kv-head + 16-row block
  const int b = blockIdx.z;
  const int row_blocks = (p.groups + 15) / 16;
  const int kvh = head_block / row_blocks;
  const int g0 = (head_block % row_blocks) * 16;  // first group row of this CTA
  const int rows = min(16, p.groups - g0);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  int64_t len = p.lengths[b];
  if (len > p.mask_len) {
    if (threadIdx.x == 0 && split == 0 && head_block == 0 && p.status != nullptr)
      atomicOr(p.status, B200_STATUS_LENGTH_OVER_MASK);
    len = p.mask_len;
  }
  if (len < 0) len = 0;
  const int n_tokens = static_cast<int>(len);
  const int start = split * p.split_tokens;
  if (start >= n_tokens && split > 0) return;
  const int end = min(start + p.split_tokens, n_tokens);

  // ---- Q fragments straight from global memory (A operand, 16 x D, rows = q heads) ----
  uint32_t qa[kKSteps][4];
  {
    const int r0 = lane >> 2;
    const int col = (lane & 3) * 2;
    const __nv_bfloat16* qbase =
        p.q + b * p.q_batch_stride + static_cast<int64_t>(kvh * p.groups + g0) * p.q_head_stride;
#pragma unroll
    for (int ks = 0; ks < kKSteps; ++ks) {
      const int c0 = ks * 16 + col;
      qa[ks][0] = r0 < rows ? *reinterpret_cast<const uint32_t*>(qbase + r0 * p.q_head_stride + c0) : 0u;
      qa[ks][2] = r0 < rows ? *reinterpret_cast<const uint32_t*>(qbase + r0 * p.q_head_stride + c0 + 8) : 0u;
      if (WIDE) {
        qa[ks][1] = r0 + 8 < rows ? *reinterpret_cast<const uint32_t*>(qbase + (r0 + 8) * p.q_head_stride + c0) : 0u;
        qa[ks][3] = r0 + 8 < rows ? *reinterpret_cast<const uint32_t*>(qbase + (r0 + 8) * p.q_head_stride + c0 + 8) : 0u;
      } else {
        qa[ks][1] = 0u;
        qa[ks][3] = 0u;
      }
    }
  }

  const uint32_t warp_smem = smem_u32(smem) + warp * kWarpBytes;
  const __nv_bfloat16* kglob = p.kbuf + (static_cast<int64_t>(b) * p.capacity * p.kv_heads + kvh) * D;
  const __nv_bfloat16* vglob = p.vbuf + (static_cast<int64_t>(b) * p.capacity * p.kv_heads + kvh) * D;
  const int64_t token_stride = static_cast<int64_t>(p.kv_heads) * D;

  // sub-tile j of this split covers tokens start + j*16 ...; warp w owns j = w, w+4, ...
  const int n_sub = (end - start + kSubTokens - 1) / kSubTokens;
  const int my_count = n_sub > warp ? (n_sub - warp + kWarps - 1) / kWarps : 0;

  auto issue_load = [&](int it) {
    const int t0 = start + (it * kWarps + warp) * kSubTokens;
    const uint32_t kdst = warp_smem + (it % STAGES) * kStageBytes;
    const uint32_t vdst = kdst + kTileBytes;
#pragma unroll
    for (int i = 0; i < kCopiesPerLane; ++i) {
      const int id = i * 32 + lane;
      const int r = id / kChunksPerRow;
      const int c = id % kChunksPerRow;
      const int token = t0 + r;
      const bool valid = token < end;
      const int64_t goff = valid ? token * token_stride + c * 8 : 0;
      const uint32_t soff = tile_offset<D>(r, c);
      cp_async16_zfill(kdst + soff, kglob + goff, valid ? 16 : 0);
      cp_async16_zfill(vdst + soff, vglob + goff, valid ? 16 : 0);
    }
  };

  float m_run[2] = {-INFINITY, -INFINITY};  // running max, log2 domain (rows r0, r0+8)
  float l_run[2] = {0.0f, 0.0f};            // this thread's share of the running sum
  float oacc[kNTiles][4];
#pragma unroll
  for (int i = 0; i < kNTiles; ++i)
    oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.0f;

  const float scale_log2 = p.scale * kLog2e;

#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < my_count) issue_load(s);
    cp_async_commit();
  }

  for (int it = 0; it < my_count; ++it) {
    cp_async_wait<STAGES - 2>();
    __syncwarp();
    if (it + STAGES - 1 < my_count) issue_load(it + STAGES - 1);
    cp_async_commit();

    const int t0 = start + (it * kWarps + warp) * kSubTokens;
    const uint32_t ksm = warp_smem + (it % STAGES) * kStageBytes;
    const uint32_t vsm = ksm + kTileBytes;

    // ---- S = Q K^T : 16 x 16 ----
    float sacc[2][4];
#pragma unroll
    for (int i = 0; i < 2; ++i) sacc[i][0] = sacc[i][1] = sacc[i][2] = sacc[i][3] = 0.0f;
    {
      const int mat = lane >> 3;
      const int krow = ((mat >> 1) << 3) + (lane & 7);
#pragma unroll
      for (int ks = 0; ks < kKSteps; ++ks) {
        uint32_t kb[4];
        ldmatrix_x4(kb, ksm + tile_offset<D>(krow, ks * 2 + (mat & 1)));
        mma_bf16_16816(sacc[0], qa[ks], kb[0], kb[1]);
        mma_bf16_16816(sacc[1], qa[ks], kb[2], kb[3]);
      }
    }

    // ---- scale, mask, online softmax (log2 domain) ----
    float row_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        if (!WIDE && e >= 2) continue;
        const int token = t0 + nt * 8 + (lane & 3) * 2 + (e & 1);
        float s;
        if (p.compat) {
          // reference order: r(q k^T) -> r(. * scale) -> fp32 (+ mask)
          s = round_bf16(round_bf16(sacc[nt][e]) * p.scale) * kLog2e;
        } else {
          s = sacc[nt][e] * scale_log2;
        }
        if (token < end) {
          if (p.mask != nullptr)
            s += load_mask(p.mask, p.mask_dtype, b * p.mask_batch_stride + token) * kLog2e;
        } else {
          s = -INFINITY;
        }
        sacc[nt][e] = s;
        row_max[e >> 1] = fmaxf(row_max[e >> 1], s);
      }
    }
    uint32_t pa[4];
    float alpha[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      if (!WIDE && r == 1) {
        alpha[1] = 1.0f;
        continue;
      }
      float mx = row_max[r];
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m_run[r], mx);
      const float m_safe = m_new == -INFINITY ? 0.0f : m_new;
      alpha[r] = fast_exp2(m_run[r] - m_safe);  // exp2(-inf) = 0 on the first tile
      m_run[r] = m_new;
      float sum = 0.0f;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        const float p0 = fast_exp2(sacc[nt][2 * r] - m_safe);
        const float p1 = fast_exp2(sacc[nt][2 * r + 1] - m_safe);
        sum += p0 + p1;
        pa[nt * 2 + r] = pack_bf16x2(p0, p1);
      }
      l_run[r] = l_run[r] * alpha[r] + sum;
    }
    if (!WIDE) {
      pa[1] = 0u;
      pa[3] = 0u;
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

    // ---- O += P V : (16 x 16) x (16 x D) ----
    {
      const int mat = lane >> 3;
      const int vrow = ((mat & 1) << 3) + (lane & 7);
#pragma unroll
      for (int np = 0; np < kNTiles / 2; ++np) {
        uint32_t vb[4];
        ldmatrix_x4_trans(vb, vsm + tile_offset<D>(vrow, np * 2 + (mat >> 1)));
        mma_bf16_16816(oacc[np * 2], pa, vb[0], vb[1]);
        mma_bf16_16816(oacc[np * 2 + 1], pa, vb[2], vb[3]);
      }
    }
  }
  cp_async_wait<0>();
  __syncwarp();

  // quad-reduce the row sums
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }

  // ---- merge the 4 warps through shared memory (each warp reuses its own ring) ----
  float* my_o = reinterpret_cast<float*>(smem + warp * kWarpBytes);  // [16][D]
  float* my_ml = my_o + 16 * D;                                       // [16][2]
  {
    const int r0 = lane >> 2;
    const int col = (lane & 3) * 2;
#pragma unroll
    for (int nt = 0; nt < kNTiles; ++nt) {
      my_o[r0 * D + nt * 8 + col] = oacc[nt][0];
      my_o[r0 * D + nt * 8 + col + 1] = oacc[nt][1];
      if (WIDE) {
        my_o[(r0 + 8) * D + nt * 8 + col] = oacc[nt][2];
        my_o[(r0 + 8) * D + nt * 8 + col + 1] = oacc[nt][3];
      }
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
  __syncthreads();

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
    if (p.num_splits == 1) {
      p.out[(static_cast<int64_t>(b) * p.q_heads + hq) * D + col] =
          __float2bfloat16_rn(o_all / l_all);  // 0/0 = NaN for an empty sequence, as the oracle
    } else {
      const int64_t slot = (static_cast<int64_t>(b) * p.q_heads + hq) * p.num_splits + split;
      p.ws_o[slot * D + col] = o_all;
      if (col == 0) {
        p.ws_ml[slot * 2] = m_all;
        p.ws_ml[slot * 2 + 1] = l_all;
      }
    }
  }
}

// Combines the per-split partials of one (sequence, q head). blockDim.x == D.
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
template <int D>
__global__ void decode_attention_f32_kernel(const float* __restrict__ q,
                                            const float* __restrict__ kbuf,
                                            const float* __restrict__ vbuf,
                                            const int64_t* __restrict__ lengths,
                                            const void* __restrict__ mask, float* __restrict__ out,
                                            int q_heads, int kv_heads, int groups, int capacity,
                                            int mask_len, int64_t q_batch_stride,
                                            int64_t q_head_stride, int64_t mask_batch_stride,
                                            int mask_dtype, float scale, int32_t* status) {
  constexpr int kT = 64;
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
    sq[d] = q[b * q_batch_stride + hq * q_head_stride + d];
  __syncthreads();
  float m = -INFINITY, l = 0.0f, acc[D];
#pragma unroll
  for (int d = 0; d < D; ++d) acc[d] = 0.0f;
  for (int t = threadIdx.x; t < len; t += kT) {
    const float* krow = kbuf + ((static_cast<int64_t>(b) * capacity + t) * kv_heads + kvh) * D;
    const float* vrow = vbuf + ((static_cast<int64_t>(b) * capacity + t) * kv_heads + kvh) * D;
    float s = 0.0f;
#pragma unroll
    for (int d = 0; d < D; ++d) s = fmaf(sq[d], krow[d], s);
    s *= scale;
    if (mask != nullptr) s += load_mask(mask, mask_dtype, b * mask_batch_stride + t);
    const float m_new = fmaxf(m, s);
    const float m_safe = m_new == -INFINITY ? 0.0f : m_new;
    const float alpha = expf(m - m_safe);
    const float pr = expf(s - m_safe);
    l = l * alpha + pr;
#pragma unroll
    for (int d = 0; d < D; ++d) acc[d] = acc[d] * alpha + pr * vrow[d];
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
    out[(static_cast<int64_t>(b) * q_heads + hq) * D + d] = o_all / l_all;
  }
}

template <int D>
constexpr int stages_for() {
  return D <= 64 ? 4 : 3;
}

template <int D>
int smem_bytes_for() {
  return kWarps * stages_for<D>() * 2 * kSubTokens * D * 2;
}

template <int D>
int launch_bf16(const DecodeParams& p, cudaStream_t stream) {
  constexpr int STAGES = stages_for<D>();
  const int smem = smem_bytes_for<D>();
  const int row_blocks = (p.groups + 15) / 16;
  dim3 grid(p.num_splits, p.kv_heads * row_blocks, p.batch);
  cudaError_t err;
  if (p.groups > 8) {
    auto kernel = decode_attention_kernel<D, STAGES, true>;
    err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (err != cudaSuccess) return B200_ERR_LAUNCH;
    kernel<<<grid, kThreads, smem, stream>>>(p);
  } else {
    auto kernel = decode_attention_kernel<D, STAGES, false>;
    err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (err != cudaSuccess) return B200_ERR_LAUNCH;
    kernel<<<grid, kThreads, smem, stream>>>(p);
  }
  if (cudaGetLastError() != cudaSuccess) return B200_ERR_LAUNCH;
  if (p.num_splits > 1) {
    decode_merge_kernel<<<p.batch * p.q_heads, D, 0, stream>>>(
        p.ws_o, p.ws_ml, p.lengths, p.out, p.q_heads, D, p.num_splits, p.split_tokens,
        p.mask_len);
  }
  return launch_status();
}

int64_t round_up(int64_t v, int64_t m) { return (v + m - 1) / m * m; }

// Tokens per split when the caller does not choose: enough CTAs for ~4 waves of
// 148 SMs x 3 resident CTAs, never below 256 tokens (a warp then still pipelines
// 4 sub-tiles), rounded to the 64 tokens the 4 warps cover per step.
int64_t default_split_tokens(int64_t batch, int64_t head_blocks, int64_t max_length) {
  const int64_t target_ctas = static_cast<int64_t>(kNumSMs) * 3 * 4;
  const int64_t units = batch * head_blocks;
  int64_t splits = units > 0 ? target_ctas / units : 1;
  if (splits < 1) splits = 1;
  int64_t tokens = round_up(ceil_div(max_length, splits), 64);
  if (tokens < 256) tokens = 256;
  return tokens;
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
  if (split_tokens <= 0) split_tokens = default_split_tokens(batch, head_blocks, max_length);
  const int64_t splits = ceil_div(max_length, split_tokens);
  if (splits <= 1) return 0;
  return round_up(batch * q_heads * splits * (head_dim + 2) * 4, 256);
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
  if (!query || !key_buffer || !value_buffer || !lengths || !output || batch < 0 ||
      q_heads <= 0 || kv_heads <= 0 || head_dim <= 0 || capacity <= 0 || mask_len <= 0 ||
      mask_len > capacity || q_heads % kv_heads != 0)
    return B200_ERR_BAD_ARGUMENT;
  if (mask != nullptr && mask_dtype != B200_F32 && mask_dtype != B200_BF16)
    return B200_ERR_UNSUPPORTED;
  if (batch == 0) return B200_OK;
  if (batch > 65535) return B200_ERR_TOO_LARGE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int groups = static_cast<int>(q_heads / kv_heads);

  if (dtype == B200_F32) {
    dim3 grid(static_cast<unsigned>(q_heads), static_cast<unsigned>(batch));
#define B200_LAUNCH_F32(DIM)                                                                   \
  decode_attention_f32_kernel<DIM><<<grid, 64, 0, s>>>(                                        \
      static_cast<const float*>(query), static_cast<const float*>(key_buffer),                \
      static_cast<const float*>(value_buffer), lengths, mask, static_cast<float*>(output),    \
      static_cast<int>(q_heads), static_cast<int>(kv_heads), groups,                          \
      static_cast<int>(capacity), static_cast<int>(mask_len), q_batch_stride, q_head_stride,  \
      mask_batch_stride, mask_dtype, static_cast<float>(scale), status)
    if (head_dim == 64) B200_LAUNCH_F32(64);
    else if (head_dim == 16) B200_LAUNCH_F32(16);
    else if (head_dim == 32) B200_LAUNCH_F32(32);
    else if (head_dim == 128) B200_LAUNCH_F32(128);
    else return B200_ERR_UNSUPPORTED;
#undef B200_LAUNCH_F32
    return launch_status();
  }
  if (dtype != B200_BF16) return B200_ERR_UNSUPPORTED;
  if (head_dim != 64 && head_dim != 128) return B200_ERR_UNSUPPORTED;
  if (!aligned16(key_buffer) || !aligned16(value_buffer) ||
      (reinterpret_cast<uintptr_t>(query) & 3u) != 0 || q_head_stride % 2 != 0 ||
      q_batch_stride % 2 != 0)
    return B200_ERR_ALIGNMENT;

  int64_t max_length = max_length_hint > 0 && max_length_hint < mask_len ? max_length_hint : mask_len;
  const int64_t head_blocks = kv_heads * ceil_div(groups, 16);
  if (split_tokens <= 0) split_tokens = default_split_tokens(batch, head_blocks, max_length);
  split_tokens = round_up(split_tokens, 16);
  // lengths above the hint are still honoured: the grid covers mask_len when no hint is given
  const int64_t splits = ceil_div(max_length, split_tokens);
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
  p.mask_len = static_cast<int>(max_length < mask_len ? max_length : mask_len);
  p.split_tokens = static_cast<int>(split_tokens);
  p.num_splits = static_cast<int>(splits);
  p.mask_dtype = mask_dtype;
  p.compat = mode == B200_MODE_PYTORCH_COMPATIBLE ? 1 : 0;
  p.scale = static_cast<float>(scale);
  p.ws_o = nullptr;
  p.ws_ml = nullptr;
  if (splits > 1) {
    const int64_t need = round_up(batch * q_heads * splits * (head_dim + 2) * 4, 256);
    if (!workspace || workspace_bytes < need) return B200_ERR_WORKSPACE;
    p.ws_o = static_cast<float*>(workspace);
    p.ws_ml = p.ws_o + batch * q_heads * splits * head_dim;
  }
  return head_dim == 64 ? launch_bf16<64>(p, s) : launch_bf16<128>(p, s);
}
