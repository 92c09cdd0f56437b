// serve.prefill_attention: T-token GQA attention with an arbitrary additive
// B x 1 x T x T mask, or with proven causality (fully masked key tiles are skipped and
// the mask is not read).
//
// bf16 kernel (warp-level tensor cores): a CTA of 4 warps owns 64 query rows of one
// (sequence, q head); each warp keeps 16 rows of Q as A fragments and streams 64-key
// K/V tiles through a cp.async ring of XOR-swizzled rows; S = Q K^T and O += P V are
// m16n8k16 tiles with an fp32 online softmax in the log2 domain. The output is written
// token-major (B x T x Hq x D) so that the transpose + reshape that follows in the
// graph is a view.
//
// fp32 kernel: CUDA cores with IEEE fp32 dots for small full-precision graphs.
#include <math.h>

#include "common.cuh"

namespace b200 {
namespace {

constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;
constexpr int kBM = 64;  // query rows per CTA
constexpr int kBN = 64;  // keys per tile
constexpr float kLog2e = 1.4426950408889634f;

struct PrefillParams {
  const __nv_bfloat16* q;
  const __nv_bfloat16* k;
  const __nv_bfloat16* v;
  const void* mask;
  __nv_bfloat16* out;
  int64_t qs[3], ks[3], vs[3];  // batch, head, token strides (elements)
  int64_t ms[4];                // mask strides: batch, head, query, key
  int batch, q_heads, kv_heads, groups, tokens;
  int mask_dtype, causal, compat;
  float scale;
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

template <int D>
__device__ __forceinline__ uint32_t tile_offset(int row, int chunk) {
  return static_cast<uint32_t>(row * (D * 2) + (((chunk & ~7) | ((chunk ^ row) & 7)) << 4));
}

template <int D, int STAGES>
__global__ void __launch_bounds__(kThreads) prefill_attention_kernel(const PrefillParams p) {
  constexpr int kChunksPerRow = D / 8;
  constexpr int kTileBytes = kBN * D * 2;
  constexpr int kQBytes = kBM * D * 2;
  constexpr int kStageBytes = 2 * kTileBytes;
  constexpr int kCopies = kBN * kChunksPerRow / kThreads;
  constexpr int kKSteps = D / 16;
  constexpr int kNTiles = D / 8;

  extern __shared__ __align__(1024) unsigned char smem[];
  const uint32_t q_sm = smem_u32(smem);
  const uint32_t kv_sm = q_sm + kQBytes;

  const int q0 = blockIdx.x * kBM;
  const int hq = blockIdx.y;
  const int b = blockIdx.z;
  const int kvh = hq / p.groups;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int T = p.tokens;

  const __nv_bfloat16* qg = p.q + b * p.qs[0] + hq * p.qs[1];
  const __nv_bfloat16* kg = p.k + b * p.ks[0] + kvh * p.ks[1];
  const __nv_bfloat16* vg = p.v + b * p.vs[0] + kvh * p.vs[1];

  const int key_end = p.causal ? min(T, q0 + kBM) : T;
  const int n_tiles = (key_end + kBN - 1) / kBN;

  auto issue_kv = [&](int tile) {
    const uint32_t kdst = kv_sm + (tile % STAGES) * kStageBytes;
    const uint32_t vdst = kdst + kTileBytes;
    const int t0 = tile * kBN;
#pragma unroll
    for (int i = 0; i < kCopies; ++i) {
      const int id = i * kThreads + threadIdx.x;
      const int r = id / kChunksPerRow, c = id % kChunksPerRow;
      const int token = t0 + r;
      const bool valid = token < T;
      const uint32_t soff = tile_offset<D>(r, c);
      cp_async16_zfill(kdst + soff, valid ? kg + token * p.ks[2] + c * 8 : kg, valid ? 16 : 0);
      cp_async16_zfill(vdst + soff, valid ? vg + token * p.vs[2] + c * 8 : vg, valid ? 16 : 0);
    }
  };

  // Q tile rides in the first commit group
#pragma unroll
  for (int i = 0; i < kBM * kChunksPerRow / kThreads; ++i) {
    const int id = i * kThreads + threadIdx.x;
    const int r = id / kChunksPerRow, c = id % kChunksPerRow;
    const int token = q0 + r;
    const bool valid = token < T;
    cp_async16_zfill(q_sm + tile_offset<D>(r, c), valid ? qg + token * p.qs[2] + c * 8 : qg,
                     valid ? 16 : 0);
  }
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < n_tiles) issue_kv(s);
    cp_async_commit();
  }

  uint32_t qa[kKSteps][4];
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.0f, 0.0f};
  float oacc[kNTiles][4];
#pragma unroll
  for (int i = 0; i < kNTiles; ++i) oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.0f;

  const float scale_log2 = p.scale * kLog2e;
  const int mat = lane >> 3;
  const int row_lo = q0 + warp * 16 + (lane >> 2);  // this thread's query rows: row_lo, row_lo + 8

  for (int tile = 0; tile < n_tiles; ++tile) {
    cp_async_wait<STAGES - 2>();
    __syncthreads();
    if (tile + STAGES - 1 < n_tiles) issue_kv(tile + STAGES - 1);
    cp_async_commit();

    if (tile == 0) {
#pragma unroll
      for (int ks = 0; ks < kKSteps; ++ks) {
        const int r = warp * 16 + ((mat & 1) << 3) + (lane & 7);
        ldmatrix_x4(qa[ks], q_sm + tile_offset<D>(r, ks * 2 + (mat >> 1)));
      }
    }
    const int k0 = tile * kBN;
    // a warp whose 16 rows all precede this key tile has nothing to do under causality
    const bool warp_active = !p.causal || k0 <= q0 + warp * 16 + 15;
    if (!warp_active) continue;

    const uint32_t ksm = kv_sm + (tile % STAGES) * kStageBytes;
    const uint32_t vsm = ksm + kTileBytes;

    float sacc[kBN / 8][4];
#pragma unroll
    for (int i = 0; i < kBN / 8; ++i) sacc[i][0] = sacc[i][1] = sacc[i][2] = sacc[i][3] = 0.0f;
#pragma unroll
    for (int ks = 0; ks < kKSteps; ++ks) {
#pragma unroll
      for (int np = 0; np < kBN / 16; ++np) {
        uint32_t kb[4];
        const int r = np * 16 + ((mat >> 1) << 3) + (lane & 7);
        ldmatrix_x4(kb, ksm + tile_offset<D>(r, ks * 2 + (mat & 1)));
        mma_bf16_16816(sacc[np * 2], qa[ks], kb[0], kb[1]);
        mma_bf16_16816(sacc[np * 2 + 1], qa[ks], kb[2], kb[3]);
      }
    }

    float row_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < kBN / 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int qrow = row_lo + ((e >> 1) << 3);
        const int key = k0 + nt * 8 + (lane & 3) * 2 + (e & 1);
        float s;
        if (p.compat)
          s = round_bf16(round_bf16(sacc[nt][e]) * p.scale) * kLog2e;
        else
          s = sacc[nt][e] * scale_log2;
        const bool visible = key < T && qrow < T && (!p.causal || key <= qrow);
        if (visible) {
          if (p.mask != nullptr)
            s += load_mask(p.mask, p.mask_dtype,
                           b * p.ms[0] + static_cast<int64_t>(qrow) * p.ms[2] +
                               static_cast<int64_t>(key) * p.ms[3]) *
                 kLog2e;
        } else {
          s = -INFINITY;
        }
        sacc[nt][e] = s;
        row_max[e >> 1] = fmaxf(row_max[e >> 1], s);
      }
    }
    float alpha[2], m_safe[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      float mx = row_max[r];
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m_run[r], mx);
      m_safe[r] = m_new == -INFINITY ? 0.0f : m_new;
      alpha[r] = fast_exp2(m_run[r] - m_safe[r]);
      m_run[r] = m_new;
      l_run[r] *= alpha[r];
    }
#pragma unroll
    for (int i = 0; i < kNTiles; ++i) {
      oacc[i][0] *= alpha[0];
      oacc[i][1] *= alpha[0];
      oacc[i][2] *= alpha[1];
      oacc[i][3] *= alpha[1];
    }
#pragma unroll
    for (int kk = 0; kk < kBN / 16; ++kk) {
      uint32_t pa[4];
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int nt = kk * 2 + half;
        const float p0 = fast_exp2(sacc[nt][0] - m_safe[0]);
        const float p1 = fast_exp2(sacc[nt][1] - m_safe[0]);
        const float p2 = fast_exp2(sacc[nt][2] - m_safe[1]);
        const float p3 = fast_exp2(sacc[nt][3] - m_safe[1]);
        l_run[0] += p0 + p1;
        l_run[1] += p2 + p3;
        pa[half * 2] = pack_bf16x2(p0, p1);
        pa[half * 2 + 1] = pack_bf16x2(p2, p3);
      }
#pragma unroll
      for (int np = 0; np < kNTiles / 2; ++np) {
        uint32_t vb[4];
        const int r = kk * 16 + ((mat & 1) << 3) + (lane & 7);
        ldmatrix_x4_trans(vb, vsm + tile_offset<D>(r, np * 2 + (mat >> 1)));
        mma_bf16_16816(oacc[np * 2], pa, vb[0], vb[1]);
        mma_bf16_16816(oacc[np * 2 + 1], pa, vb[2], vb[3]);
      }
    }
  }
  cp_async_wait<0>();

#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int qrow = row_lo + r * 8;
    if (qrow >= T) continue;
    const float inv = 1.0f / l_run[r];  // all-masked row: 0 * inf = NaN, as the oracle
    __nv_bfloat16* orow = p.out + ((static_cast<int64_t>(b) * T + qrow) * p.q_heads + hq) * D;
#pragma unroll
    for (int nt = 0; nt < kNTiles; ++nt) {
      const int col = nt * 8 + (lane & 3) * 2;
      *reinterpret_cast<uint32_t*>(orow + col) =
          pack_bf16x2(oacc[nt][r * 2] * inv, oacc[nt][r * 2 + 1] * inv);
    }
  }
}

// ---- generic path (fp32, fp16, head sizes 16 / 32 / 256): one CTA per (query token, q head,
// sequence), fp32 arithmetic on the CUDA cores, one rounding on the way out (and, in the
// compatible mode of a 16-bit type, the reference's two roundings of the scores) ----------
template <int D, typename T>
__global__ void prefill_attention_generic_kernel(const T* __restrict__ q, const T* __restrict__ k,
                                                 const T* __restrict__ v,
                                                 const void* __restrict__ mask, T* __restrict__ out,
                                                 int q_heads, int groups, int tokens, int64_t qs0,
                                                 int64_t qs1, int64_t qs2, int64_t ks0, int64_t ks1,
                                                 int64_t ks2, int64_t vs0, int64_t vs1, int64_t vs2,
                                                 int64_t ms0, int64_t ms2, int64_t ms3,
                                                 int mask_dtype, int causal, float scale,
                                                 bool compat) {
  constexpr int kT = D > 128 ? 32 : 64;  // (the merge buffer of 64 threads x 256 columns would not fit)
  const int qt = blockIdx.x, hq = blockIdx.y, b = blockIdx.z;
  const int kvh = hq / groups;
  __shared__ float sq[D];
  __shared__ float sm[kT], sl[kT];
  __shared__ float so[kT][D + 1];
  for (int d = threadIdx.x; d < D; d += kT) sq[d] = Elem<T>::load(q + b * qs0 + hq * qs1 + qt * qs2 + d);
  __syncthreads();
  float m = -INFINITY, l = 0.0f, acc[D];
#pragma unroll
  for (int d = 0; d < D; ++d) acc[d] = 0.0f;
  const int key_end = causal ? qt + 1 : tokens;
  for (int t = threadIdx.x; t < key_end; t += kT) {
    const T* krow = k + b * ks0 + kvh * ks1 + t * ks2;
    const T* vrow = v + b * vs0 + kvh * vs1 + t * vs2;
    float s = 0.0f;
#pragma unroll
    for (int d = 0; d < D; ++d) s = fmaf(sq[d], Elem<T>::load(krow + d), s);
    s = compat ? Elem<T>::round(Elem<T>::round(s) * scale) : s * scale;
    if (mask != nullptr)
      s += load_mask(mask, mask_dtype, b * ms0 + static_cast<int64_t>(qt) * ms2 + t * ms3);
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
    Elem<T>::store(out + ((static_cast<int64_t>(b) * tokens + qt) * q_heads + hq) * D + d, o_all / l_all);
  }
}

template <int D, int STAGES>
int launch_bf16(const PrefillParams& p, cudaStream_t stream) {
  constexpr int smem = kBM * D * 2 + STAGES * 2 * kBN * D * 2;
  auto kernel = prefill_attention_kernel<D, STAGES>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
    return B200_ERR_LAUNCH;
  dim3 grid((p.tokens + kBM - 1) / kBM, p.q_heads, p.batch);
  kernel<<<grid, kThreads, smem, stream>>>(p);
  return launch_status();
}

}  // namespace
}  // namespace b200

namespace b200 {
// prefill_attention_tcgen05.cu
int prefill_attention_tcgen05(const void* query, const void* key, const void* value, void* output,
                              int64_t batch, int64_t q_heads, int64_t kv_heads, int64_t tokens,
                              int64_t head_dim, const int64_t query_strides[4],
                              const int64_t key_strides[4], const int64_t value_strides[4],
                              double scale, int32_t* status, cudaStream_t stream, const void* mask,
                              const int64_t* mask_strides, void* workspace, int64_t workspace_bytes);
int64_t prefill_attention_tcgen05_workspace_bytes(int64_t batch, int64_t tokens);
}  // namespace b200

using namespace b200;

extern "C" int64_t b200_prefill_attention_workspace_bytes(int64_t batch, int64_t tokens) {
  if (batch <= 0 || tokens <= 0) return 0;
  return prefill_attention_tcgen05_workspace_bytes(batch, tokens);
}

extern "C" int b200_prefill_attention(const void* query, const void* key, const void* value,
                                      const void* mask, void* output, int64_t batch,
                                      int64_t q_heads, int64_t kv_heads, int64_t tokens,
                                      int64_t head_dim, const int64_t query_strides[4],
                                      const int64_t key_strides[4],
                                      const int64_t value_strides[4],
                                      const int64_t mask_strides[4], int mask_dtype, double scale,
                                      int causal, int dtype, int mode, void* workspace,
                                      int64_t workspace_bytes, int32_t* status, void* stream) {
  if (!query || !key || !value || !output || !query_strides || !key_strides || !value_strides ||
      batch < 0 || q_heads <= 0 || kv_heads <= 0 || tokens < 0 || head_dim <= 0 ||
      q_heads % kv_heads != 0)
    return B200_ERR_BAD_ARGUMENT;
  if (mask == nullptr && !causal) return B200_ERR_BAD_ARGUMENT;
  if (mask != nullptr && (!mask_strides || (!known_dtype(mask_dtype))))
    return B200_ERR_BAD_ARGUMENT;
  if (query_strides[3] != 1 || key_strides[3] != 1 || value_strides[3] != 1)
    return B200_ERR_UNSUPPORTED;
  if (batch == 0 || tokens == 0) return B200_OK;
  if (batch > 65535 || q_heads > 65535 || tokens > INT32_MAX) return B200_ERR_TOO_LARGE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int groups = static_cast<int>(q_heads / kv_heads);
  const int64_t zero4[4] = {0, 0, 0, 0};
  const int64_t* ms = mask != nullptr ? mask_strides : zero4;

  if (!known_dtype(dtype)) return B200_ERR_UNSUPPORTED;
  if (dtype != B200_BF16 || (head_dim != 64 && head_dim != 128)) {
    if (head_dim != 16 && head_dim != 32 && head_dim != 64 && head_dim != 128 && head_dim != 256)
      return B200_ERR_UNSUPPORTED;
    if (tokens > 65535 * 64) return B200_ERR_TOO_LARGE;
    dim3 grid(static_cast<unsigned>(tokens), static_cast<unsigned>(q_heads),
              static_cast<unsigned>(batch));
    const bool compat = mode == B200_MODE_PYTORCH_COMPATIBLE && dtype != B200_F32;
    with_element_type(dtype, [&](auto tag) {
      using T = typename decltype(tag)::type;
      auto run = [&](auto kernel) {
        kernel<<<grid, head_dim > 128 ? 32 : 64, 0, s>>>(
            static_cast<const T*>(query), static_cast<const T*>(key), static_cast<const T*>(value),
            mask, static_cast<T*>(output), static_cast<int>(q_heads), groups,
            static_cast<int>(tokens), query_strides[0], query_strides[1], query_strides[2],
            key_strides[0], key_strides[1], key_strides[2], value_strides[0], value_strides[1],
            value_strides[2], ms[0], ms[2], ms[3], mask_dtype, causal, static_cast<float>(scale),
            compat);
      };
      if (head_dim == 16) run(prefill_attention_generic_kernel<16, T>);
      else if (head_dim == 32) run(prefill_attention_generic_kernel<32, T>);
      else if (head_dim == 64) run(prefill_attention_generic_kernel<64, T>);
      else if (head_dim == 128) run(prefill_attention_generic_kernel<128, T>);
      else run(prefill_attention_generic_kernel<256, T>);
    });
    return launch_status();
  }
  if (!aligned16(query) || !aligned16(key) || !aligned16(value) ||
      (reinterpret_cast<uintptr_t>(output) & 3u) != 0)
    return B200_ERR_ALIGNMENT;
  for (int i = 0; i < 3; ++i)
    if (query_strides[i] % 8 != 0 || key_strides[i] % 8 != 0 || value_strides[i] % 8 != 0)
      return B200_ERR_ALIGNMENT;

  if (mode == B200_MODE_FAST && ((mask == nullptr && causal) ||
                                 (mask != nullptr && !causal && mask_dtype == B200_F32 && workspace != nullptr))) {
    // the tensor-core kernel: causal-proved, or the additive-mask contract with its tile pre-pass
    const int code = prefill_attention_tcgen05(query, key, value, output, batch, q_heads, kv_heads,
                                               tokens, head_dim, query_strides, key_strides,
                                               value_strides, scale, status, s, mask, mask_strides,
                                               workspace, workspace_bytes);
    if (code != B200_ERR_UNSUPPORTED) return code;
  }

  PrefillParams p;
  p.q = static_cast<const __nv_bfloat16*>(query);
  p.k = static_cast<const __nv_bfloat16*>(key);
  p.v = static_cast<const __nv_bfloat16*>(value);
  p.mask = mask;
  p.out = static_cast<__nv_bfloat16*>(output);
  for (int i = 0; i < 3; ++i) {
    p.qs[i] = query_strides[i];
    p.ks[i] = key_strides[i];
    p.vs[i] = value_strides[i];
  }
  for (int i = 0; i < 4; ++i) p.ms[i] = ms[i];
  p.batch = static_cast<int>(batch);
  p.q_heads = static_cast<int>(q_heads);
  p.kv_heads = static_cast<int>(kv_heads);
  p.groups = groups;
  p.tokens = static_cast<int>(tokens);
  p.mask_dtype = mask_dtype;
  p.causal = causal ? 1 : 0;
  p.compat = mode == B200_MODE_PYTORCH_COMPATIBLE ? 1 : 0;
  p.scale = static_cast<float>(scale);
  return head_dim == 64 ? launch_bf16<64, 3>(p, s) : launch_bf16<128, 2>(p, s);
}
