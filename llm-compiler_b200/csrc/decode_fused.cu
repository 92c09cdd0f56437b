// Consumers of the split-K partial sums in the decode step: the reduction over the K slices
// happens while the next operator loads its input, so no CTA ever waits for another and the
// sum order is fixed (slice 0, 1, ...).
//
//   reduce_residual_rms_norm   y = r(sum_s partial[s]) (the linear's bf16 result)
//                              x' = r(y + residual)    (the residual add of the layer)
//                              h  = RMSNorm(x') * w    (the norm that follows), x' and h written
//   reduce_rope_kv_store       qkv = r(sum_s partial[s] + bias); q -> RoPE -> query_out;
//                              k -> RoPE -> K buffer at positions[b]; v -> V buffer
//
// Rounding points are those of the separate reference ops (linear -> add -> rms_norm, and
// linear -> rope -> kv.store), so the fusion changes launch counts, not numerics.
#include "common.cuh"

namespace b200 {
namespace {

constexpr int kNormThreads = 1024;  // one element per thread at hidden <= 1024
constexpr int kMaxPerThread = 4;    // hidden <= 4096 kept in registers

__global__ void __launch_bounds__(kNormThreads)
reduce_residual_rms_norm_kernel(const float* __restrict__ partials, int splits,
                                const __nv_bfloat16* __restrict__ residual,
                                const __nv_bfloat16* __restrict__ weight,
                                __nv_bfloat16* __restrict__ x_out, __nv_bfloat16* __restrict__ h_out,
                                int rows, int hidden, float epsilon, int compat,
                                int early_weight) {
  TraceScope trace(2);
  grid_launch_dependents();
  // the norm weight is a model parameter: when the caller says parameters are constants it is
  // read before the dependency wait, off the critical path
  float w[kMaxPerThread];
  if (early_weight && h_out != nullptr) {
#pragma unroll
    for (int i = 0; i < kMaxPerThread; ++i) {
      const int c = threadIdx.x + i * blockDim.x;
      w[i] = c < hidden ? __bfloat162float(weight[c]) : 0.0f;
    }
  }
  grid_dependency_wait_cta();
  trace.mark(0);
  const int row = blockIdx.x;
  const int64_t slice = static_cast<int64_t>(rows) * hidden;
  const float* prow = partials + static_cast<int64_t>(row) * hidden;
  float x[kMaxPerThread];
  float r[kMaxPerThread];
  float sum = 0.0f;
#pragma unroll
  for (int i = 0; i < kMaxPerThread; ++i) {  // the residual loads fly with the partial loads
    const int c = threadIdx.x + i * blockDim.x;
    r[i] = residual != nullptr && c < hidden
               ? __bfloat162float(residual[static_cast<int64_t>(row) * hidden + c]) : 0.0f;
  }
  if (!(early_weight && h_out != nullptr) && h_out != nullptr) {
#pragma unroll
    for (int i = 0; i < kMaxPerThread; ++i) {
      const int c = threadIdx.x + i * blockDim.x;
      w[i] = c < hidden ? __bfloat162float(weight[c]) : 0.0f;
    }
  }
#pragma unroll
  for (int i = 0; i < kMaxPerThread; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    x[i] = 0.0f;
    if (c < hidden) {
      float v = round_bf16(sum_slices(prow + c, slice, splits));
      if (residual != nullptr) v = round_bf16(__fadd_rn(v, r[i]));
      x[i] = v;
      x_out[static_cast<int64_t>(row) * hidden + c] = __float2bfloat16_rn(v);
      sum = fmaf(v, v, sum);
    }
  }
  if (h_out == nullptr) {
    trace.mark(1);
    return;
  }
  __shared__ float partial_sum[kNormThreads / 32];
  __shared__ float total;
  sum = warp_sum(sum);
  if ((threadIdx.x & 31) == 0) partial_sum[threadIdx.x >> 5] = sum;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x >> 5) ? partial_sum[threadIdx.x] : 0.0f;
    v = warp_sum(v);
    if (threadIdx.x == 0) total = v;
  }
  __syncthreads();
  const float inv_rms = compat ? __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(total, static_cast<float>(hidden)), epsilon)))
                               : rsqrtf(total / static_cast<float>(hidden) + epsilon);
#pragma unroll
  for (int i = 0; i < kMaxPerThread; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    if (c < hidden) {
      const float n = round_bf16(__fmul_rn(x[i], inv_rms));
      h_out[static_cast<int64_t>(row) * hidden + c] = __float2bfloat16_rn(__fmul_rn(w[i], n));
    }
  }
  trace.mark(1);
}

// One thread handles one (sequence, head, rotation pair d / d + D/2).
__global__ void reduce_rope_kv_store_kernel(const float* __restrict__ partials, int splits,
                                            const __nv_bfloat16* __restrict__ bias,
                                            const __nv_bfloat16* __restrict__ cosine,
                                            const __nv_bfloat16* __restrict__ sine,
                                            __nv_bfloat16* __restrict__ q_out,
                                            __nv_bfloat16* __restrict__ kbuf,
                                            __nv_bfloat16* __restrict__ vbuf,
                                            const int64_t* __restrict__ positions, int batch,
                                            int q_heads, int kv_heads, int dim, int capacity,
                                            int32_t* status) {
  TraceScope trace(3);
  grid_launch_dependents();
  grid_dependency_wait_cta();
  trace.mark(0);
  const int half = dim / 2;
  const int heads = q_heads + 2 * kv_heads;
  const int width = heads * dim;  // columns of the fused q|k|v projection
  const int64_t slice = static_cast<int64_t>(batch) * width;
  const int total = batch * heads * half;
  for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += gridDim.x * blockDim.x) {
    const int d = idx % half;
    const int hh = (idx / half) % heads;
    const int b = idx / (half * heads);
    const int col_lo = hh * dim + d, col_hi = col_lo + half;
    const float* prow = partials + static_cast<int64_t>(b) * width;
    // every operand is requested before the first one is used: one memory latency, not four
    const int64_t pos = positions[b];
    const float bias_lo = bias != nullptr ? __bfloat162float(bias[col_lo]) : 0.0f;
    const float bias_hi = bias != nullptr ? __bfloat162float(bias[col_hi]) : 0.0f;
    const float clo = __bfloat162float(cosine[static_cast<int64_t>(b) * dim + d]);
    const float chi = __bfloat162float(cosine[static_cast<int64_t>(b) * dim + d + half]);
    const float slo = __bfloat162float(sine[static_cast<int64_t>(b) * dim + d]);
    const float shi = __bfloat162float(sine[static_cast<int64_t>(b) * dim + d + half]);
    float lo = sum_slices(prow + col_lo, slice, splits);
    float hi = sum_slices(prow + col_hi, slice, splits);
    if (bias != nullptr) {
      lo += bias_lo;
      hi += bias_hi;
    }
    lo = round_bf16(lo);  // the linear's bf16 output
    hi = round_bf16(hi);
    const bool in_range = pos >= 0 && pos < capacity;
    if (hh >= q_heads && !in_range) {
      if (status != nullptr && d == 0 && hh == q_heads)
        atomicOr(status, pos < 0 ? B200_STATUS_BAD_POSITION : B200_STATUS_KV_OVERFLOW);
      continue;
    }
    if (hh >= q_heads + kv_heads) {  // value head: stored as is
      const int h = hh - q_heads - kv_heads;
      __nv_bfloat16* dst = vbuf + ((static_cast<int64_t>(b) * capacity + pos) * kv_heads + h) * dim;
      dst[d] = __float2bfloat16_rn(lo);
      dst[d + half] = __float2bfloat16_rn(hi);
      continue;
    }
    const float ylo = round_bf16(__fadd_rn(round_bf16(__fmul_rn(lo, clo)), round_bf16(__fmul_rn(-hi, slo))));
    const float yhi = round_bf16(__fadd_rn(round_bf16(__fmul_rn(hi, chi)), round_bf16(__fmul_rn(lo, shi))));
    __nv_bfloat16* dst = hh < q_heads
        ? q_out + (static_cast<int64_t>(b) * q_heads + hh) * dim
        : kbuf + ((static_cast<int64_t>(b) * capacity + pos) * kv_heads + (hh - q_heads)) * dim;
    dst[d] = __float2bfloat16_rn(ylo);
    dst[d + half] = __float2bfloat16_rn(yhi);
  }
  trace.mark(1);
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" int b200_reduce_residual_rms_norm(const void* partials, int64_t splits,
                                             const void* residual, const void* norm_weight,
                                             void* x_out, void* h_out, int64_t rows,
                                             int64_t hidden, double epsilon, int mode,
                                             void* stream) {
  if (!partials || !x_out || splits <= 0 || rows < 0 || hidden <= 0 || (h_out && !norm_weight))
    return B200_ERR_BAD_ARGUMENT;
  if (hidden > kNormThreads * kMaxPerThread) return B200_ERR_TOO_LARGE;
  if (rows == 0) return B200_OK;
  int threads = static_cast<int>((hidden + 31) / 32 * 32);
  if (threads > kNormThreads) threads = kNormThreads;
  const cudaError_t launched = launch_chained(
      reduce_residual_rms_norm_kernel, dim3(static_cast<unsigned>(rows)), dim3(threads), 0,
      static_cast<cudaStream_t>(stream), static_cast<const float*>(partials), static_cast<int>(splits),
      static_cast<const __nv_bfloat16*>(residual), static_cast<const __nv_bfloat16*>(norm_weight),
      static_cast<__nv_bfloat16*>(x_out), static_cast<__nv_bfloat16*>(h_out),
      static_cast<int>(rows), static_cast<int>(hidden), static_cast<float>(epsilon),
      mode == B200_MODE_PYTORCH_COMPATIBLE ? 1 : 0,
      (launch_mode() & B200_LAUNCH_CONSTANT_WEIGHTS) != 0 ? 1 : 0);
  return launched == cudaSuccess ? launch_status() : B200_ERR_LAUNCH;
}

extern "C" int b200_reduce_rope_kv_store(const void* partials, int64_t splits, const void* bias,
                                         const void* cosine, const void* sine, void* query_out,
                                         void* key_buffer, void* value_buffer,
                                         const int64_t* positions, int64_t batch, int64_t q_heads,
                                         int64_t kv_heads, int64_t head_dim, int64_t capacity,
                                         int32_t* status, void* stream) {
  if (!partials || !cosine || !sine || !query_out || !key_buffer || !value_buffer || !positions ||
      splits <= 0 || batch < 0 || q_heads <= 0 || kv_heads <= 0 || head_dim <= 0 ||
      head_dim % 2 != 0 || capacity <= 0)
    return B200_ERR_BAD_ARGUMENT;
  const int64_t total = batch * (q_heads + 2 * kv_heads) * (head_dim / 2);
  if (total == 0) return B200_OK;
  if (total > INT32_MAX) return B200_ERR_TOO_LARGE;
  const int threads = 256;
  int64_t blocks = ceil_div(total, threads);
  if (blocks > kNumSMs * 8) blocks = kNumSMs * 8;
  const cudaError_t launched = launch_chained(
      reduce_rope_kv_store_kernel, dim3(static_cast<unsigned>(blocks)), dim3(threads), 0,
      static_cast<cudaStream_t>(stream), static_cast<const float*>(partials), static_cast<int>(splits),
      static_cast<const __nv_bfloat16*>(bias), static_cast<const __nv_bfloat16*>(cosine),
      static_cast<const __nv_bfloat16*>(sine), static_cast<__nv_bfloat16*>(query_out),
      static_cast<__nv_bfloat16*>(key_buffer), static_cast<__nv_bfloat16*>(value_buffer),
      positions, static_cast<int>(batch), static_cast<int>(q_heads), static_cast<int>(kv_heads),
      static_cast<int>(head_dim), static_cast<int>(capacity), status);
  return launched == cudaSuccess ? launch_status() : B200_ERR_LAUNCH;
}
