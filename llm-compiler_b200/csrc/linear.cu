// serve.linear: y[M,N] = x[M,K] W[N,K]^T (+ bias) with fp32 accumulation and fused
// epilogues (residual add, SwiGLU over row-interleaved gate/up weights).
//
// bf16: warp-level tensor-core tiles (m16n8k16) fed by a multi-stage cp.async ring of
// 128-byte XOR-swizzled rows. Both operands are K-major, so A (activations) and B
// (weights) are read with plain ldmatrix. Decode-sized M streams every weight byte
// exactly once; when the tile grid is smaller than ~2 waves of the 148 SMs the K range
// is split across CTAs (grid.z): each CTA parks its fp32 partial in the workspace and the
// CTA that arrives last at the tile's counter adds the partials in split order
// (deterministic) and runs the epilogue. Counters are left at zero for the next call.
//
// fp32: CUDA-core tiled GEMM with IEEE fp32 FMAs (small full-precision graphs).
#include <stdlib.h>
#include <string.h>

#include "common.cuh"

namespace b200 {
namespace {

constexpr int kBK = 64;  // bf16 K extent of a stage: 128-byte rows

struct LinearParams {
  const __nv_bfloat16* x;
  const __nv_bfloat16* w;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual;
  __nv_bfloat16* out;
  float* partials;
  int* counters;
  int64_t x_row_stride;
  int m, k, n, splits, epilogue;
};

__device__ __forceinline__ float silu_f32(float x) {
  return __fdiv_rn(x, __fadd_rn(1.0f, expf(-x)));
}

// Writes the pair of adjacent columns (n, n+1) of row m.
__device__ __forceinline__ void epilogue_pair(const LinearParams& p, int m, int n, float v0,
                                              float v1) {
  if (m >= p.m || n >= p.n) return;
  const bool has1 = n + 1 < p.n;
  if (p.bias != nullptr) {
    v0 += __bfloat162float(p.bias[n]);
    if (has1) v1 += __bfloat162float(p.bias[n + 1]);
  }
  if (p.epilogue == B200_EPILOGUE_SWIGLU) {
    // column 2j is gate_j, column 2j+1 is up_j
    const float g = round_bf16(silu_f32(round_bf16(v0)));
    const float u = round_bf16(v1);
    p.out[static_cast<int64_t>(m) * (p.n / 2) + n / 2] = __float2bfloat16_rn(g * u);
    return;
  }
  v0 = round_bf16(v0);
  v1 = round_bf16(v1);
  const int64_t o = static_cast<int64_t>(m) * p.n + n;
  if (p.epilogue == B200_EPILOGUE_RESIDUAL) {
    v0 = __fadd_rn(v0, __bfloat162float(p.residual[o]));
    if (has1) v1 = __fadd_rn(v1, __bfloat162float(p.residual[o + 1]));
  }
  if (has1 && (o & 1) == 0) {
    *reinterpret_cast<uint32_t*>(p.out + o) = pack_bf16x2(v0, v1);
  } else {
    p.out[o] = __float2bfloat16_rn(v0);
    if (has1) p.out[o + 1] = __float2bfloat16_rn(v1);
  }
}

template <int BM, int BN, int WM, int WN, int STAGES>
__global__ void __launch_bounds__(WM* WN * 32) linear_bf16_kernel(const LinearParams p) {
  constexpr int kThreads = WM * WN * 32;
  constexpr int WTM = BM / WM, WTN = BN / WN;
  constexpr int MT = WTM / 16, NT = WTN / 8;
  static_assert(WTM % 16 == 0 && WTN % 16 == 0, "warp tile must be a multiple of 16 x 16");
  constexpr int kABytes = BM * 128, kBBytes = BN * 128, kStageBytes = kABytes + kBBytes;
  constexpr int kAcc = MT * NT * 4;

  extern __shared__ __align__(1024) unsigned char smem[];
  const uint32_t smem_base = smem_u32(smem);

  const int tile_n = blockIdx.x, tile_m = blockIdx.y, split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int warp_m = warp / WN, warp_n = warp % WN;

  const int kb_total = (p.k + kBK - 1) / kBK;
  const int kb_per = (kb_total + p.splits - 1) / p.splits;
  const int kb0 = split * kb_per;
  const int nkb = max(0, min(kb0 + kb_per, kb_total) - kb0);

  auto issue_load = [&](int stage, int kb) {
    const uint32_t a_dst = smem_base + stage * kStageBytes;
    const uint32_t b_dst = a_dst + kABytes;
    const int k0 = kb * kBK;
#pragma unroll
    for (int i = 0; i < (BM * 8 + kThreads - 1) / kThreads; ++i) {
      const int id = i * kThreads + threadIdx.x;
      if (BM * 8 % kThreads != 0 && id >= BM * 8) break;
      const int r = id >> 3, c = id & 7;
      const int m = tile_m * BM + r;
      const bool valid = m < p.m && k0 + c * 8 < p.k;
      const __nv_bfloat16* src = valid ? p.x + static_cast<int64_t>(m) * p.x_row_stride + k0 + c * 8 : p.x;
      cp_async16_zfill(a_dst + r * 128 + (swizzle128(r, c) << 4), src, valid ? 16 : 0);
    }
#pragma unroll
    for (int i = 0; i < (BN * 8 + kThreads - 1) / kThreads; ++i) {
      const int id = i * kThreads + threadIdx.x;
      if (BN * 8 % kThreads != 0 && id >= BN * 8) break;
      const int r = id >> 3, c = id & 7;
      const int n = tile_n * BN + r;
      const bool valid = n < p.n && k0 + c * 8 < p.k;
      const __nv_bfloat16* src = valid ? p.w + static_cast<int64_t>(n) * p.k + k0 + c * 8 : p.w;
      cp_async16_zfill(b_dst + r * 128 + (swizzle128(r, c) << 4), src, valid ? 16 : 0);
    }
  };

  float acc[MT][NT][4];
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int j = 0; j < NT; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.0f;

#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < nkb) issue_load(s, kb0 + s);
    cp_async_commit();
  }

  const int mat = lane >> 3;
  for (int i = 0; i < nkb; ++i) {
    cp_async_wait<STAGES - 2>();
    __syncthreads();
    if (i + STAGES - 1 < nkb) issue_load((i + STAGES - 1) % STAGES, kb0 + i + STAGES - 1);
    cp_async_commit();

    const uint32_t a_sm = smem_base + (i % STAGES) * kStageBytes;
    const uint32_t b_sm = a_sm + kABytes;
#pragma unroll
    for (int ks = 0; ks < kBK / 16; ++ks) {
      uint32_t af[MT][4];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const int r = warp_m * WTM + mt * 16 + ((mat & 1) << 3) + (lane & 7);
        ldmatrix_x4(af[mt], a_sm + r * 128 + (swizzle128(r, ks * 2 + (mat >> 1)) << 4));
      }
#pragma unroll
      for (int np = 0; np < NT / 2; ++np) {
        uint32_t bf[4];
        const int r = warp_n * WTN + np * 16 + ((mat >> 1) << 3) + (lane & 7);
        ldmatrix_x4(bf, b_sm + r * 128 + (swizzle128(r, ks * 2 + (mat & 1)) << 4));
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          mma_bf16_16816(acc[mt][np * 2], af[mt], bf[0], bf[1]);
          mma_bf16_16816(acc[mt][np * 2 + 1], af[mt], bf[2], bf[3]);
        }
      }
    }
  }
  cp_async_wait<0>();

  if (p.splits > 1) {
    const int tile = tile_m * gridDim.x + tile_n;
    float* mine = p.partials + (static_cast<int64_t>(tile) * p.splits + split) * (kAcc * kThreads);
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e)
          mine[((mt * NT + nt) * 4 + e) * kThreads + threadIdx.x] = acc[mt][nt][e];
    __threadfence();
    __syncthreads();
    __shared__ int is_last;
    if (threadIdx.x == 0) {
      const int arrived = atomicAdd(p.counters + tile, 1);
      is_last = arrived == p.splits - 1;
      if (is_last) p.counters[tile] = 0;  // ready for the next call on this workspace
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    const float* all = p.partials + static_cast<int64_t>(tile) * p.splits * (kAcc * kThreads);
    // split-major, with all kAcc loads of a split in flight together: the sum order is fixed
    // (split 0, 1, ...), the latency of a round is paid once per split, not once per element
    float* flat = &acc[0][0][0];
    for (int s = 0; s < p.splits; ++s) {
      float part[kAcc];
#pragma unroll
      for (int i = 0; i < kAcc; ++i)
        part[i] = __ldcg(all + (static_cast<int64_t>(s) * kAcc + i) * kThreads + threadIdx.x);
#pragma unroll
      for (int i = 0; i < kAcc; ++i) flat[i] = s == 0 ? part[i] : flat[i] + part[i];
    }
  }

#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    const int m0 = tile_m * BM + warp_m * WTM + mt * 16 + (lane >> 2);
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const int n0 = tile_n * BN + warp_n * WTN + nt * 8 + (lane & 3) * 2;
      epilogue_pair(p, m0, n0, acc[mt][nt][0], acc[mt][nt][1]);
      epilogue_pair(p, m0 + 8, n0, acc[mt][nt][2], acc[mt][nt][3]);
    }
  }
}

// ------------------------------------------------------- generic: fp32, fp16 ----
// fp32 arithmetic on the CUDA cores for the element types the tensor-core kernels do not
// take; a 16-bit type is rounded where the reference's kernels round theirs (the result,
// the sum in front of a residual add, gate / up / silu(gate) of a SwiGLU).
template <typename T>
struct LinearParamsGeneric {
  const T* x;
  const T* w;
  const T* bias;
  const T* residual;
  T* out;
  int64_t x_row_stride;
  int m, k, n, epilogue;
};

template <typename T>
__global__ void __launch_bounds__(256) linear_generic_kernel(const LinearParamsGeneric<T> p) {
  constexpr int BM = 64, BN = 64, BKF = 16;
  __shared__ float As[BKF][BM + 1];
  __shared__ float Bs[BKF][BN + 1];
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  const int m_base = blockIdx.y * BM, n_base = blockIdx.x * BN;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
  for (int k0 = 0; k0 < p.k; k0 += BKF) {
    for (int id = threadIdx.x; id < BM * BKF; id += 256) {
      const int r = id / BKF, c = id % BKF;
      const int m = m_base + r, kk = k0 + c;
      As[c][r] = (m < p.m && kk < p.k) ? Elem<T>::load(p.x + static_cast<int64_t>(m) * p.x_row_stride + kk) : 0.0f;
      const int n = n_base + r;
      Bs[c][r] = (n < p.n && kk < p.k) ? Elem<T>::load(p.w + static_cast<int64_t>(n) * p.k + kk) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BKF; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m_base + ty * 4 + i;
    if (m >= p.m) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n_base + tx * 4 + j;
      if (n >= p.n) continue;
      float v = acc[i][j];
      if (p.bias != nullptr) v += Elem<T>::load(p.bias + n);
      if (p.epilogue == B200_EPILOGUE_SWIGLU) {
        // gate in even columns, up in odd columns: pair them inside the thread
        if ((j & 1) == 0) {
          float u = acc[i][j + 1];
          if (p.bias != nullptr) u += Elem<T>::load(p.bias + n + 1);
          const float gate = Elem<T>::round(silu_f32(Elem<T>::round(v)));
          Elem<T>::store(p.out + static_cast<int64_t>(m) * (p.n / 2) + n / 2, gate * Elem<T>::round(u));
        }
        continue;
      }
      const int64_t o = static_cast<int64_t>(m) * p.n + n;
      if (p.epilogue == B200_EPILOGUE_RESIDUAL)
        v = __fadd_rn(Elem<T>::round(v), Elem<T>::load(p.residual + o));
      Elem<T>::store(p.out + o, v);
    }
  }
}

struct TilePlan {
  int bm, bn, threads, splits, tiles_m, tiles_n;
  int64_t partial_floats_per_tile_split;
};

TilePlan plan_bf16(int64_t m, int64_t k, int64_t n) {
  TilePlan t;
  if (m <= 16) {
    t.bm = 16; t.bn = 64; t.threads = 128;
  } else if (m <= 32) {
    t.bm = 32; t.bn = 64; t.threads = 128;
  } else if (m <= 64) {
    t.bm = 64; t.bn = 64; t.threads = 128;
  } else {
    t.bm = 128; t.bn = 128; t.threads = 256;
  }
  t.tiles_m = static_cast<int>(ceil_div(m, t.bm));
  t.tiles_n = static_cast<int>(ceil_div(n, t.bn));
  const int64_t tiles = static_cast<int64_t>(t.tiles_m) * t.tiles_n;
  const int64_t kb = ceil_div(k, kBK);
  int64_t splits = 1;
  const int64_t target = 2 * kNumSMs;
  if (tiles < target) {
    splits = ceil_div(target, tiles);
    if (splits > 8) splits = 8;
    if (splits > kb) splits = kb;
    // no empty splits: every split gets at least one k block
    const int64_t per = ceil_div(kb, splits);
    splits = ceil_div(kb, per);
  }
  t.splits = static_cast<int>(splits);
  t.partial_floats_per_tile_split = static_cast<int64_t>(t.bm) * t.bn;
  return t;
}

// The tile counters sit in a fixed-size region at the start of the workspace, so that calls
// with different tile grids can share one workspace: the region is only ever touched as
// counters (and left at zero), never as partial sums. Split-K is used for < 2 * 148 tiles.
constexpr int64_t kCounterBytes = 4096;
int64_t counters_bytes(const TilePlan& t) {
  (void)t;
  return kCounterBytes;
}
static_assert(2 * kNumSMs * 4 <= kCounterBytes, "counter region too small");

template <int BM, int BN, int WM, int WN, int STAGES>
int launch_tile(const LinearParams& p, const TilePlan& t, cudaStream_t stream) {
  constexpr int smem = STAGES * (BM + BN) * 128;
  auto kernel = linear_bf16_kernel<BM, BN, WM, WN, STAGES>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
    return B200_ERR_LAUNCH;
  dim3 grid(t.tiles_n, t.tiles_m, t.splits);
  kernel<<<grid, WM * WN * 32, smem, stream>>>(p);
  return launch_status();
}

}  // namespace
}  // namespace b200

namespace b200 {
int linear_tcgen05(const void* input, const void* weight, const void* bias, const void* residual,
                   void* output, int64_t m, int64_t k, int64_t n, int64_t input_row_stride,
                   int epilogue, int32_t* status, cudaStream_t stream, bool fold_norm = false,
                   double norm_eps = 0.0, const float* norm_squares = nullptr, int norm_slices = 0);
}

using namespace b200;

// The tcgen05 path takes every problem it can fill the GPU with (it declines decode-size M
// with few N tiles, which need split-K); B200_LINEAR_PATH=mma.sync or the launch-mode flag
// B200_LAUNCH_LINEAR_WARP_LEVEL (what a dispatch plan sets) force the warp-level kernel.
static bool use_tcgen05(int64_t m) {
  (void)m;
  if ((launch_mode() & B200_LAUNCH_LINEAR_WARP_LEVEL) != 0) return false;
  const char* value = getenv("B200_LINEAR_PATH");
  return value == nullptr || strcmp(value, "mma.sync") != 0;
}

extern "C" int64_t b200_linear_workspace_bytes(int64_t m, int64_t k, int64_t n, int dtype,
                                               int epilogue) {
  (void)epilogue;
  if (dtype != B200_BF16 || m <= 0 || k <= 0 || n <= 0) return 0;
  const TilePlan t = plan_bf16(m, k, n);
  if (t.splits <= 1) return 0;
  return counters_bytes(t) + static_cast<int64_t>(t.tiles_m) * t.tiles_n * t.splits *
                                 t.partial_floats_per_tile_split * 4;
}

extern "C" int b200_linear(const void* input, const void* weight, const void* bias,
                           const void* residual, void* output, int64_t m, int64_t k, int64_t n,
                           int64_t input_row_stride, int dtype, int epilogue, void* workspace,
                           int64_t workspace_bytes, int32_t* status, void* stream) {
  if (!input || !weight || !output || m < 0 || k <= 0 || n <= 0 || input_row_stride < k)
    return B200_ERR_BAD_ARGUMENT;
  if (epilogue != B200_EPILOGUE_NONE && epilogue != B200_EPILOGUE_RESIDUAL &&
      epilogue != B200_EPILOGUE_SWIGLU)
    return B200_ERR_BAD_ARGUMENT;
  if (epilogue == B200_EPILOGUE_RESIDUAL && !residual) return B200_ERR_BAD_ARGUMENT;
  if (epilogue == B200_EPILOGUE_SWIGLU && n % 2 != 0) return B200_ERR_BAD_ARGUMENT;
  if (m == 0) return B200_OK;
  if (m > INT32_MAX || k > INT32_MAX || n > INT32_MAX) return B200_ERR_TOO_LARGE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);

  if (dtype == B200_F32 || dtype == B200_F16) {
    dim3 grid(static_cast<unsigned>(ceil_div(n, 64)), static_cast<unsigned>(ceil_div(m, 64)));
    if (grid.y > 65535) return B200_ERR_TOO_LARGE;
    with_element_type(dtype, [&](auto tag) {
      using T = typename decltype(tag)::type;
      LinearParamsGeneric<T> p;
      p.x = static_cast<const T*>(input);
      p.w = static_cast<const T*>(weight);
      p.bias = static_cast<const T*>(bias);
      p.residual = static_cast<const T*>(residual);
      p.out = static_cast<T*>(output);
      p.x_row_stride = input_row_stride;
      p.m = static_cast<int>(m);
      p.k = static_cast<int>(k);
      p.n = static_cast<int>(n);
      p.epilogue = epilogue;
      linear_generic_kernel<T><<<grid, 256, 0, s>>>(p);
    });
    return launch_status();
  }
  if (dtype != B200_BF16) return B200_ERR_UNSUPPORTED;
  if (k % 8 != 0 || input_row_stride % 8 != 0) return B200_ERR_UNSUPPORTED;
  if (!aligned16(input) || !aligned16(weight)) return B200_ERR_ALIGNMENT;

  if (use_tcgen05(m)) {
    const int code = linear_tcgen05(input, weight, bias, residual, output, m, k, n,
                                    input_row_stride, epilogue, status, s);
    if (code != B200_ERR_UNSUPPORTED) return code;
  }
  const TilePlan t = plan_bf16(m, k, n);
  if (t.tiles_m > 65535) return B200_ERR_TOO_LARGE;
  LinearParams p;
  p.x = static_cast<const __nv_bfloat16*>(input);
  p.w = static_cast<const __nv_bfloat16*>(weight);
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.residual = static_cast<const __nv_bfloat16*>(residual);
  p.out = static_cast<__nv_bfloat16*>(output);
  p.x_row_stride = input_row_stride;
  p.m = static_cast<int>(m);
  p.k = static_cast<int>(k);
  p.n = static_cast<int>(n);
  p.splits = t.splits;
  p.epilogue = epilogue;
  p.partials = nullptr;
  p.counters = nullptr;
  if (t.splits > 1) {
    const int64_t need = b200_linear_workspace_bytes(m, k, n, dtype, epilogue);
    if (!workspace || workspace_bytes < need) return B200_ERR_WORKSPACE;
    p.counters = static_cast<int*>(workspace);
    p.partials = reinterpret_cast<float*>(static_cast<char*>(workspace) + counters_bytes(t));
  }
  if (t.bm == 16) return launch_tile<16, 64, 1, 4, 4>(p, t, s);
  if (t.bm == 32) return launch_tile<32, 64, 1, 4, 4>(p, t, s);
  if (t.bm == 64) return launch_tile<64, 64, 1, 4, 4>(p, t, s);
  return launch_tile<128, 128, 2, 4, 3>(p, t, s);
}
