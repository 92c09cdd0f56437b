// RMSNorm over the last dimension, one launch, each row read once.
//
// FAST mode: one CTA per row, 16-byte loads kept in registers, tree reduction, rsqrtf.
// PYTORCH_COMPATIBLE mode: one warp per row reproducing, operation for operation, what
// the reference's CPU executor computes for
//     variance = x.float().pow(2).mean(-1); n = x.float() * rsqrt(variance + eps)
// i.e. PyTorch's CPU float sum: 8 vector lanes x 4 interleaved accumulators (32 running
// sums = the 32 lanes of a warp, lane t owning elements t, t+32, ...), cascaded in
// blocks of 2^p terms over up to 4 levels, the 4 accumulators folded in order, the
// 8 lanes folded sequentially; then a true division by the row length, an IEEE sqrt
// and an IEEE reciprocal. Every step uses explicit round-to-nearest intrinsics so the
// compiler cannot contract or reassociate.
#include "common.cuh"

namespace b200 {
namespace {

template <typename T>
__device__ __forceinline__ float finish_element(float x, float inv_rms, float w,
                                                bool round_before_weight) {
  if (round_before_weight) {
    const float n = Elem<T>::round(__fmul_rn(x, inv_rms));
    return Elem<T>::round(__fmul_rn(w, n));
  }
  return Elem<T>::round(__fmul_rn(__fmul_rn(x, inv_rms), w));
}

// Two elements of a vector store: the inner rounding of both with one conversion instruction,
// the outer rounding left to the store (rounding twice to the same format changes nothing).
template <typename T>
__device__ __forceinline__ void finish_pair(float x0, float x1, float inv_rms, float w0, float w1,
                                            bool round_before_weight, float& y0, float& y1) {
  float n0 = __fmul_rn(x0, inv_rms), n1 = __fmul_rn(x1, inv_rms);
  if (round_before_weight) Elem<T>::round_pair(n0, n1);
  y0 = round_before_weight ? __fmul_rn(w0, n0) : __fmul_rn(n0, w0);
  y1 = round_before_weight ? __fmul_rn(w1, n1) : __fmul_rn(n1, w1);
}

// ---------------------------------------------------------------- fast mode ----
constexpr int kMaxCached = 4;  // 16-byte chunks a thread keeps in registers

template <typename T, bool kVector>
__global__ void rms_norm_fast_kernel(const T* __restrict__ input, const T* __restrict__ weight,
                                     T* __restrict__ output, int64_t hidden, int64_t row_stride,
                                     float epsilon, bool round_before_weight) {
  constexpr int per = kVector ? Elem<T>::kPerVec : 1;
  const T* row = input + blockIdx.x * row_stride;
  T* out = output + blockIdx.x * hidden;
  const int64_t chunks = hidden / per;

  float cache[kMaxCached][per];
  float sum = 0.0f;
#pragma unroll
  for (int i = 0; i < kMaxCached; ++i) {
    const int64_t c = threadIdx.x + static_cast<int64_t>(i) * blockDim.x;
    if (c < chunks) {
      if (kVector) {
        Vec16<T> v;
        v.load(row + c * per);
#pragma unroll
        for (int j = 0; j < per; ++j) {
          cache[i][j] = v.v[j];
          sum = fmaf(v.v[j], v.v[j], sum);
        }
      } else {
        cache[i][0] = Elem<T>::load(row + c);
        sum = fmaf(cache[i][0], cache[i][0], sum);
      }
    }
  }
  for (int64_t c = threadIdx.x + static_cast<int64_t>(kMaxCached) * blockDim.x; c < chunks;
       c += blockDim.x) {
#pragma unroll
    for (int j = 0; j < per; ++j) {
      const float x = Elem<T>::load(row + c * per + j);
      sum = fmaf(x, x, sum);
    }
  }

  __shared__ float partial[32];
  __shared__ float total;
  sum = warp_sum(sum);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) partial[warp] = sum;
  __syncthreads();
  if (warp == 0) {
    const int warps = (blockDim.x + 31) >> 5;
    float v = lane < warps ? partial[lane] : 0.0f;
    v = warp_sum(v);
    if (lane == 0) total = v;
  }
  __syncthreads();
  const float inv_rms = rsqrtf(total / static_cast<float>(hidden) + epsilon);

#pragma unroll
  for (int i = 0; i < kMaxCached; ++i) {
    const int64_t c = threadIdx.x + static_cast<int64_t>(i) * blockDim.x;
    if (c < chunks) {
      if (kVector) {
        Vec16<T> w, y;
        w.load(weight + c * per);
#pragma unroll
        for (int j = 0; j < per; j += 2)
          finish_pair<T>(cache[i][j], cache[i][j + 1], inv_rms, w.v[j], w.v[j + 1], round_before_weight,
                         y.v[j], y.v[j + 1]);
        y.store(out + c * per);
      } else {
        Elem<T>::store(out + c, finish_element<T>(cache[i][0], inv_rms,
                                                  Elem<T>::load(weight + c),
                                                  round_before_weight));
      }
    }
  }
  for (int64_t c = threadIdx.x + static_cast<int64_t>(kMaxCached) * blockDim.x; c < chunks;
       c += blockDim.x) {
#pragma unroll
    for (int j = 0; j < per; ++j) {
      const int64_t e = c * per + j;
      Elem<T>::store(out + e, finish_element<T>(Elem<T>::load(row + e), inv_rms,
                                                Elem<T>::load(weight + e),
                                                round_before_weight));
    }
  }
}

// Many rows of a short hidden size (a prefill's tokens): one warp per row, eight rows per CTA,
// the row held in registers between the two passes (up to kMaxCached 16-byte chunks per lane),
// no shared memory and no block barrier. One CTA of 128 threads per row leaves most of the
// memory system idle at hidden 896 (23 us for 16384 rows against 9 us of traffic).
constexpr int kRowsPerBlock = 8;

template <typename T>
__global__ void __launch_bounds__(kRowsPerBlock * 32)
rms_norm_rows_kernel(const T* __restrict__ input, const T* __restrict__ weight, T* __restrict__ output,
                     int64_t rows, int64_t hidden, int64_t row_stride, float epsilon,
                     bool round_before_weight) {
  constexpr int per = Elem<T>::kPerVec;
  const int lane = threadIdx.x & 31;
  const int64_t r = static_cast<int64_t>(blockIdx.x) * kRowsPerBlock + (threadIdx.x >> 5);
  if (r >= rows) return;
  const T* row = input + r * row_stride;
  T* out = output + r * hidden;
  const int chunks = static_cast<int>(hidden / per);  // at most 32 * kMaxCached

  float cache[kMaxCached][per];
  float sum = 0.0f;
#pragma unroll
  for (int i = 0; i < kMaxCached; ++i) {
    const int c = lane + i * 32;
    if (c < chunks) {
      Vec16<T> v;
      v.load(row + c * per);
#pragma unroll
      for (int j = 0; j < per; ++j) {
        cache[i][j] = v.v[j];
        sum = fmaf(v.v[j], v.v[j], sum);
      }
    }
  }
  sum = warp_sum(sum);
  const float inv_rms = rsqrtf(sum / static_cast<float>(hidden) + epsilon);
#pragma unroll
  for (int i = 0; i < kMaxCached; ++i) {
    const int c = lane + i * 32;
    if (c < chunks) {
      Vec16<T> w, y;
      w.load(weight + c * per);
#pragma unroll
      for (int j = 0; j < per; j += 2)
        finish_pair<T>(cache[i][j], cache[i][j + 1], inv_rms, w.v[j], w.v[j + 1], round_before_weight,
                       y.v[j], y.v[j + 1]);
      y.store(out + c * per);
    }
  }
}

// ------------------------------------------------------ pytorch_compatible mode ----
__host__ __device__ inline int ceil_log2_i64(int64_t x) {
  int r = 0;
  while ((int64_t(1) << r) < x) ++r;
  return r;
}

constexpr int kWarpsPerBlock = 4;

template <typename T>
__global__ void rms_norm_compat_kernel(const T* __restrict__ input, const T* __restrict__ weight,
                                       T* __restrict__ output, int64_t rows, int64_t hidden,
                                       int64_t row_stride, float epsilon,
                                       bool round_before_weight) {
  const int lane = threadIdx.x & 31;
  const int64_t row_index = blockIdx.x * static_cast<int64_t>(kWarpsPerBlock) + (threadIdx.x >> 5);
  if (row_index >= rows) return;  // whole warp leaves together
  const T* row = input + row_index * row_stride;
  T* out = output + row_index * hidden;

  constexpr int kLanes = 8;    // float lanes of the CPU vector the reference sums with
  constexpr int kIlp = 4;      // interleaved vector accumulators
  constexpr int kLevels = 4;   // cascade depth
  const int64_t vec_count = hidden / kLanes;
  const int64_t groups = vec_count / kIlp;  // terms each of the 32 running sums receives
  const int level_power = max(4, ceil_log2_i64(groups) / kLevels);
  const int64_t level_step = int64_t(1) << level_power;
  const int64_t level_mask = level_step - 1;

  float acc[kLevels] = {0.0f, 0.0f, 0.0f, 0.0f};
  int64_t i = 0;
  while (i + level_step <= groups) {
    for (int64_t j = 0; j < level_step; ++j, ++i) {
      const float x = Elem<T>::load(row + i * 32 + lane);
      acc[0] = __fadd_rn(acc[0], __fmul_rn(x, x));
    }
#pragma unroll
    for (int j = 1; j < kLevels; ++j) {
      acc[j] = __fadd_rn(acc[j], acc[j - 1]);
      acc[j - 1] = 0.0f;
      const int64_t mask = level_mask << (j * level_power);
      if ((i & mask) != 0) break;
    }
  }
  for (; i < groups; ++i) {
    const float x = Elem<T>::load(row + i * 32 + lane);
    acc[0] = __fadd_rn(acc[0], __fmul_rn(x, x));
  }
#pragma unroll
  for (int j = 1; j < kLevels; ++j) acc[0] = __fadd_rn(acc[0], acc[j]);
  float part = acc[0];

  // vectors left over after the groups of four go to accumulator 0 (lanes 0..7)
  for (int64_t v = groups * kIlp; v < vec_count; ++v) {
    if (lane < kLanes) {
      const float x = Elem<T>::load(row + v * kLanes + lane);
      part = __fadd_rn(part, __fmul_rn(x, x));
    }
  }
  // accumulator 0 += accumulator 1, 2, 3, in that order
#pragma unroll
  for (int k = 1; k < kIlp; ++k) {
    const float other = __shfl_sync(0xffffffffu, part, (lane & 7) + k * kLanes);
    if (lane < kLanes) part = __fadd_rn(part, other);
  }
  // scalar tail first, then the 8 lane sums one after the other
  float total = 0.0f;
  for (int64_t e = vec_count * kLanes; e < hidden; ++e) {
    const float x = Elem<T>::load(row + e);
    total = __fadd_rn(total, __fmul_rn(x, x));
  }
#pragma unroll
  for (int k = 0; k < kLanes; ++k)
    total = __fadd_rn(total, __shfl_sync(0xffffffffu, part, k));

  const float variance = __fdiv_rn(total, static_cast<float>(hidden));
  const float inv_rms = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(variance, epsilon)));
  for (int64_t e = lane; e < hidden; e += 32)
    Elem<T>::store(out + e, finish_element<T>(Elem<T>::load(row + e), inv_rms,
                                              Elem<T>::load(weight + e), round_before_weight));
}

template <typename T>
int rms_norm_typed(const void* input, const void* weight, void* output, int64_t rows,
                   int64_t hidden, int64_t row_stride, float epsilon, bool rbw, int mode,
                   cudaStream_t stream) {
  const T* x = static_cast<const T*>(input);
  const T* w = static_cast<const T*>(weight);
  T* y = static_cast<T*>(output);
  if (mode == B200_MODE_PYTORCH_COMPATIBLE) {
    const int grid = static_cast<int>(ceil_div(rows, kWarpsPerBlock));
    rms_norm_compat_kernel<T><<<grid, kWarpsPerBlock * 32, 0, stream>>>(x, w, y, rows, hidden,
                                                                        row_stride, epsilon, rbw);
    return launch_status();
  }
  constexpr int per = Elem<T>::kPerVec;
  const bool vec = hidden % per == 0 && aligned16(input) && aligned16(weight) &&
                   aligned16(output) && (row_stride * static_cast<int64_t>(sizeof(T))) % 16 == 0;
  const int64_t chunks = vec ? hidden / per : hidden;
  int threads = static_cast<int>(((chunks + 31) / 32) * 32);
  if (threads > 1024) threads = 1024;
  if (threads < 32) threads = 32;
  if (vec && chunks <= 32 * kMaxCached && rows >= 4 * kNumSMs * kRowsPerBlock) {
    const int grid = static_cast<int>(ceil_div(rows, kRowsPerBlock));
    rms_norm_rows_kernel<T><<<grid, kRowsPerBlock * 32, 0, stream>>>(x, w, y, rows, hidden, row_stride,
                                                                   epsilon, rbw);
    return launch_status();
  }
  if (vec)
    rms_norm_fast_kernel<T, true><<<static_cast<int>(rows), threads, 0, stream>>>(
        x, w, y, hidden, row_stride, epsilon, rbw);
  else
    rms_norm_fast_kernel<T, false><<<static_cast<int>(rows), threads, 0, stream>>>(
        x, w, y, hidden, row_stride, epsilon, rbw);
  return launch_status();
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" int b200_rms_norm(const void* input, const void* weight, void* output, int64_t rows,
                             int64_t hidden, int64_t input_row_stride, double epsilon,
                             int round_before_weight, int in_dtype, int weight_dtype,
                             int out_dtype, int mode, void* stream) {
  if (!input || !weight || !output || rows < 0 || hidden <= 0 || input_row_stride < hidden)
    return B200_ERR_BAD_ARGUMENT;
  if (mode != B200_MODE_FAST && mode != B200_MODE_PYTORCH_COMPATIBLE)
    return B200_ERR_BAD_ARGUMENT;
  if (in_dtype != weight_dtype || in_dtype != out_dtype) return B200_ERR_UNSUPPORTED;
  // from 32768 elements on, the CPU sum the compatible mode mirrors splits one row across
  // threads and its order is no longer the one reproduced here
  if (mode == B200_MODE_PYTORCH_COMPATIBLE && hidden >= 32768) return B200_ERR_UNSUPPORTED;
  if (rows == 0) return B200_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const float eps = static_cast<float>(epsilon);
  int code = B200_ERR_UNSUPPORTED;
  with_element_type(in_dtype, [&](auto tag) {
    using T = typename decltype(tag)::type;
    code = rms_norm_typed<T>(input, weight, output, rows, hidden, input_row_stride, eps,
                             round_before_weight != 0, mode, s);
  });
  return code;
}
