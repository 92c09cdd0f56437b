// Bandwidth-bound single-launch kernels: KV store, RoPE (plain and fused with the KV
// store), RoPE table, embedding gather, SwiGLU, residual add, strided copy, length
// advance and greedy argmax. All of them move each byte once with 16-byte accesses;
// none needs scratch memory.
#include "common.cuh"

namespace b200 {
namespace {

constexpr int kThreads = 256;

inline int grid_for(int64_t items, int threads = kThreads) {
  int64_t blocks = ceil_div(items, threads);
  // grid-stride loops: cap the grid at a few waves of the 148 SMs
  int64_t cap = static_cast<int64_t>(kNumSMs) * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return static_cast<int>(blocks);
}

struct Strides4 {
  int64_t s[4];
};
struct Strides3 {
  int64_t s[3];
};

// ------------------------------------------------------------------ KV store ----
// One thread moves one 16-byte chunk of K and the matching chunk of V. Consecutive
// threads write consecutive destination chunks (destination rows are contiguous over
// (head, dim) for one token).
template <typename T, bool kVector>
__global__ void kv_store_kernel(T* __restrict__ kbuf, T* __restrict__ vbuf,
                                const T* __restrict__ key, const T* __restrict__ value,
                                const int64_t* __restrict__ positions, int64_t batch,
                                int64_t capacity, int64_t heads, int64_t tokens, int64_t dim,
                                Strides4 ks, Strides4 vs, int32_t* status) {
  constexpr int per = kVector ? Elem<T>::kPerVec : 1;
  const int64_t chunks = dim / per;
  const int64_t total = batch * tokens * heads * chunks;
  for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t c = idx % chunks;
    int64_t r = idx / chunks;
    const int64_t h = r % heads;
    r /= heads;
    const int64_t t = r % tokens;
    const int64_t b = r / tokens;
    const int64_t pos = positions[b];
    const int64_t dst_token = pos + t;
    if (pos < 0) {
      if (status != nullptr && c == 0 && h == 0 && t == 0) atomicOr(status, B200_STATUS_BAD_POSITION);
      continue;
    }
    if (dst_token >= capacity) {
      if (status != nullptr && c == 0 && h == 0) atomicOr(status, B200_STATUS_KV_OVERFLOW);
      continue;
    }
    const int64_t dst = ((b * capacity + dst_token) * heads + h) * dim + c * per;
    const int64_t ksrc = b * ks.s[0] + h * ks.s[1] + t * ks.s[2] + c * per * ks.s[3];
    const int64_t vsrc = b * vs.s[0] + h * vs.s[1] + t * vs.s[2] + c * per * vs.s[3];
    if (kVector) {
      const uint4 kk = *reinterpret_cast<const uint4*>(key + ksrc);
      const uint4 vv = *reinterpret_cast<const uint4*>(value + vsrc);
      *reinterpret_cast<uint4*>(kbuf + dst) = kk;
      *reinterpret_cast<uint4*>(vbuf + dst) = vv;
    } else {
      kbuf[dst] = key[ksrc];
      vbuf[dst] = value[vsrc];
    }
  }
}

bool strides_vectorizable(const void* base, const int64_t* strides, int rank, int64_t dim,
                          int per, size_t elt) {
  if (strides[rank - 1] != 1 || dim % per != 0 || !aligned16(base)) return false;
  for (int i = 0; i < rank - 1; ++i)
    if ((strides[i] * static_cast<int64_t>(elt)) % 16 != 0) return false;
  return true;
}

template <typename T>
int kv_store_typed(void* kbuf, void* vbuf, const void* key, const void* value,
                   const int64_t* positions, int64_t batch, int64_t capacity, int64_t heads,
                   int64_t tokens, int64_t dim, const int64_t* ks, const int64_t* vs,
                   int32_t* status, cudaStream_t stream) {
  Strides4 k4, v4;
  for (int i = 0; i < 4; ++i) {
    k4.s[i] = ks[i];
    v4.s[i] = vs[i];
  }
  constexpr int per = Elem<T>::kPerVec;
  const bool vec = strides_vectorizable(key, ks, 4, dim, per, sizeof(T)) &&
                   strides_vectorizable(value, vs, 4, dim, per, sizeof(T)) && aligned16(kbuf) &&
                   aligned16(vbuf);
  const int64_t total = batch * tokens * heads * (vec ? dim / per : dim);
  if (total == 0) return B200_OK;
  const int grid = grid_for(total);
  if (vec) {
    kv_store_kernel<T, true><<<grid, kThreads, 0, stream>>>(
        static_cast<T*>(kbuf), static_cast<T*>(vbuf), static_cast<const T*>(key),
        static_cast<const T*>(value), positions, batch, capacity, heads, tokens, dim, k4, v4,
        status);
  } else {
    kv_store_kernel<T, false><<<grid, kThreads, 0, stream>>>(
        static_cast<T*>(kbuf), static_cast<T*>(vbuf), static_cast<const T*>(key),
        static_cast<const T*>(value), positions, batch, capacity, heads, tokens, dim, k4, v4,
        status);
  }
  return launch_status();
}

// ----------------------------------------------------------------------- RoPE ----
// y_lo = r(r(x_lo*cos_lo) + r(-x_hi*sin_lo)),  y_hi = r(r(x_hi*cos_hi) + r(x_lo*sin_hi)).
// Products and the sum are separate IEEE operations (no FMA contraction) so that fp32
// tensors match an eager mul/mul/add bit for bit.
template <typename T>
__device__ __forceinline__ void rope_pair(float xlo, float xhi, float clo, float chi, float slo,
                                          float shi, float& ylo, float& yhi) {
  // Roundings are taken two per conversion instruction; the sums are rounded by the store
  // (every caller stores y as T, and rounding twice to the same format changes nothing).
  float a = __fmul_rn(xlo, clo), b = __fmul_rn(-xhi, slo);
  float c = __fmul_rn(xhi, chi), d = __fmul_rn(xlo, shi);
  Elem<T>::round_pair(a, b);
  Elem<T>::round_pair(c, d);
  ylo = __fadd_rn(a, b);
  yhi = __fadd_rn(c, d);
}

// IDX: the type the flat index is taken apart in. 64-bit divisions cost dozens of instructions
// each and there are four per element group; every case whose element count fits 31 bits uses int.
template <typename T, bool kVector, typename IDX>
__global__ void rope_kernel(const T* __restrict__ q, const T* __restrict__ k,
                            const T* __restrict__ cosine, const T* __restrict__ sine,
                            T* __restrict__ q_out, T* __restrict__ k_out, int64_t batch,
                            int64_t q_heads, int64_t kv_heads, int64_t tokens, int64_t dim,
                            Strides4 qs, Strides4 ks, Strides3 cs, Strides3 ss) {
  constexpr int per = kVector ? Elem<T>::kPerVec : 1;
  const int64_t half = dim / 2;
  const IDX chunks = static_cast<IDX>(half / per);
  const IDX heads = static_cast<IDX>(q_heads + kv_heads);
  const IDX total = static_cast<IDX>(batch * heads * tokens * chunks);
  const IDX token_count = static_cast<IDX>(tokens);
  for (IDX idx = static_cast<IDX>(blockIdx.x) * static_cast<IDX>(blockDim.x) + static_cast<IDX>(threadIdx.x);
       idx < total; idx += static_cast<IDX>(gridDim.x) * static_cast<IDX>(blockDim.x)) {
    // chunk fastest, then head, then token: a warp reads neighbouring heads of one token, which
    // lie side by side in a fused q|k|v projection output, and reuses the token's cos / sin
    const int64_t c = idx % chunks;
    IDX r = idx / chunks;
    const int64_t hh = r % heads;
    r /= heads;
    const int64_t t = r % token_count;
    const int64_t b = r / token_count;
    const bool is_q = hh < q_heads;
    const int64_t h = is_q ? hh : hh - q_heads;
    const T* src = is_q ? q + b * qs.s[0] + h * qs.s[1] + t * qs.s[2]
                        : k + b * ks.s[0] + h * ks.s[1] + t * ks.s[2];
    const int64_t last = is_q ? qs.s[3] : ks.s[3];
    T* dst = is_q ? q_out + ((b * q_heads + h) * tokens + t) * dim
                  : k_out + ((b * kv_heads + h) * tokens + t) * dim;
    const T* cp = cosine + b * cs.s[0] + t * cs.s[1];
    const T* sp = sine + b * ss.s[0] + t * ss.s[1];
    const int64_t d0 = c * per;
    if (kVector) {
      Vec16<T> xlo, xhi, clo, chi, slo, shi, ylo, yhi;
      xlo.load(src + d0);
      xhi.load(src + half + d0);
      clo.load(cp + d0);
      chi.load(cp + half + d0);
      slo.load(sp + d0);
      shi.load(sp + half + d0);
#pragma unroll
      for (int i = 0; i < per; ++i)
        rope_pair<T>(xlo.v[i], xhi.v[i], clo.v[i], chi.v[i], slo.v[i], shi.v[i], ylo.v[i],
                     yhi.v[i]);
      ylo.store(dst + d0);
      yhi.store(dst + half + d0);
    } else {
      float ylo, yhi;
      rope_pair<T>(Elem<T>::load(src + d0 * last), Elem<T>::load(src + (half + d0) * last),
                   Elem<T>::load(cp + d0 * cs.s[2]), Elem<T>::load(cp + (half + d0) * cs.s[2]),
                   Elem<T>::load(sp + d0 * ss.s[2]), Elem<T>::load(sp + (half + d0) * ss.s[2]),
                   ylo, yhi);
      Elem<T>::store(dst + d0, ylo);
      Elem<T>::store(dst + half + d0, yhi);
    }
  }
}

template <typename T>
int rope_typed(const void* q, const void* k, const void* cosine, const void* sine, void* q_out,
               void* k_out, int64_t batch, int64_t q_heads, int64_t kv_heads, int64_t tokens,
               int64_t dim, const int64_t* qs, const int64_t* ks, const int64_t* cs,
               const int64_t* ss, cudaStream_t stream) {
  Strides4 q4, k4;
  Strides3 c3, s3;
  for (int i = 0; i < 4; ++i) {
    q4.s[i] = qs[i];
    k4.s[i] = ks[i];
  }
  for (int i = 0; i < 3; ++i) {
    c3.s[i] = cs[i];
    s3.s[i] = ss[i];
  }
  constexpr int per = Elem<T>::kPerVec;
  const int64_t half = dim / 2;
  const bool vec = half % per == 0 && strides_vectorizable(q, qs, 4, dim, per, sizeof(T)) &&
                   strides_vectorizable(k, ks, 4, dim, per, sizeof(T)) &&
                   strides_vectorizable(cosine, cs, 3, dim, per, sizeof(T)) &&
                   strides_vectorizable(sine, ss, 3, dim, per, sizeof(T)) && aligned16(q_out) &&
                   aligned16(k_out);
  const int64_t total = batch * (q_heads + kv_heads) * tokens * (vec ? half / per : half);
  if (total == 0) return B200_OK;
  const int grid = grid_for(total);
  auto launch = [&](auto kernel) {
    kernel<<<grid, kThreads, 0, stream>>>(
        static_cast<const T*>(q), static_cast<const T*>(k), static_cast<const T*>(cosine),
        static_cast<const T*>(sine), static_cast<T*>(q_out), static_cast<T*>(k_out), batch,
        q_heads, kv_heads, tokens, dim, q4, k4, c3, s3);
  };
  // the grid-stride loop adds up to grid * threads beyond `total`: keep that inside 31 bits too
  const bool narrow = total + static_cast<int64_t>(grid) * kThreads < (int64_t(1) << 31);
  if (vec) {
    if (narrow) launch(rope_kernel<T, true, int>);
    else launch(rope_kernel<T, true, int64_t>);
  } else {
    if (narrow) launch(rope_kernel<T, false, int>);
    else launch(rope_kernel<T, false, int64_t>);
  }
  return launch_status();
}

// Decode fusion: one launch rotates q, rotates k into the K buffer and copies v into
// the V buffer at positions[b]. Vector path only (D/2 a multiple of the vector width).
template <typename T>
__global__ void rope_kv_store_kernel(const T* __restrict__ q, const T* __restrict__ k,
                                     const T* __restrict__ v, const T* __restrict__ cosine,
                                     const T* __restrict__ sine, T* __restrict__ q_out,
                                     T* __restrict__ kbuf, T* __restrict__ vbuf,
                                     const int64_t* __restrict__ positions, int64_t batch,
                                     int64_t q_heads, int64_t kv_heads, int64_t dim,
                                     int64_t capacity, int64_t qb, int64_t qh, int64_t kb,
                                     int64_t kh, int64_t vb, int64_t vh, int64_t cb,
                                     int32_t* status) {
  constexpr int per = Elem<T>::kPerVec;
  const int64_t half = dim / 2;
  const int64_t chunks = half / per;
  const int64_t heads = q_heads + 2 * kv_heads;
  const int64_t total = batch * heads * chunks;
  for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t c = idx % chunks;
    int64_t r = idx / chunks;
    const int64_t hh = r % heads;
    const int64_t b = r / heads;
    const int64_t d0 = c * per;
    const int64_t pos = positions[b];
    const bool in_range = pos >= 0 && pos < capacity;
    if (hh >= q_heads && !in_range) {
      if (status != nullptr && c == 0 && hh == q_heads)
        atomicOr(status, pos < 0 ? B200_STATUS_BAD_POSITION : B200_STATUS_KV_OVERFLOW);
      continue;
    }
    if (hh >= q_heads + kv_heads) {  // value head: plain copy of two chunks
      const int64_t h = hh - q_heads - kv_heads;
      const T* src = v + b * vb + h * vh;
      T* dst = vbuf + ((b * capacity + pos) * kv_heads + h) * dim;
      *reinterpret_cast<uint4*>(dst + d0) = *reinterpret_cast<const uint4*>(src + d0);
      *reinterpret_cast<uint4*>(dst + half + d0) =
          *reinterpret_cast<const uint4*>(src + half + d0);
      continue;
    }
    const bool is_q = hh < q_heads;
    const int64_t h = is_q ? hh : hh - q_heads;
    const T* src = is_q ? q + b * qb + h * qh : k + b * kb + h * kh;
    T* dst = is_q ? q_out + (b * q_heads + h) * dim
                  : kbuf + ((b * capacity + pos) * kv_heads + h) * dim;
    const T* cp = cosine + b * cb;
    const T* sp = sine + b * cb;
    Vec16<T> xlo, xhi, clo, chi, slo, shi, ylo, yhi;
    xlo.load(src + d0);
    xhi.load(src + half + d0);
    clo.load(cp + d0);
    chi.load(cp + half + d0);
    slo.load(sp + d0);
    shi.load(sp + half + d0);
#pragma unroll
    for (int i = 0; i < per; ++i)
      rope_pair<T>(xlo.v[i], xhi.v[i], clo.v[i], chi.v[i], slo.v[i], shi.v[i], ylo.v[i],
                   yhi.v[i]);
    ylo.store(dst + d0);
    yhi.store(dst + half + d0);
  }
}

// ------------------------------------------------------------------ RoPE table ----
template <typename T>
__global__ void rope_table_kernel(const int64_t* __restrict__ position_ids,
                                  const float* __restrict__ inv_freq, T* __restrict__ cosine,
                                  T* __restrict__ sine, int64_t rows, int64_t half) {
  const int64_t total = rows * half;
  for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t i = idx % half;
    const int64_t row = idx / half;
    const float f = __fmul_rn(static_cast<float>(position_ids[row]), inv_freq[i]);
    // double-precision evaluation, rounded once to fp32: the correctly rounded value a
    // <= 1 ulp float libm is centred on
    const float c = static_cast<float>(cos(static_cast<double>(f)));
    const float s = static_cast<float>(sin(static_cast<double>(f)));
    T* crow = cosine + row * 2 * half;
    T* srow = sine + row * 2 * half;
    Elem<T>::store(crow + i, c);
    Elem<T>::store(crow + half + i, c);
    Elem<T>::store(srow + i, s);
    Elem<T>::store(srow + half + i, s);
  }
}

// ------------------------------------------------------------------- embedding ----
template <typename T, bool kVector>
__global__ void embedding_kernel(const T* __restrict__ table, const int64_t* __restrict__ ids,
                                 T* __restrict__ out, int64_t rows, int64_t hidden,
                                 int64_t vocab, int32_t* status) {
  constexpr int per = kVector ? Elem<T>::kPerVec : 1;
  const int64_t chunks = hidden / per;
  const int64_t total = rows * chunks;
  for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t c = idx % chunks;
    const int64_t row = idx / chunks;
    const int64_t id = ids[row];
    const bool ok = id >= 0 && id < vocab;
    if (!ok && c == 0 && status != nullptr) atomicOr(status, B200_STATUS_BAD_TOKEN_ID);
    if (kVector) {
      uint4 v = make_uint4(0, 0, 0, 0);
      if (ok) v = *reinterpret_cast<const uint4*>(table + id * hidden + c * per);
      *reinterpret_cast<uint4*>(out + row * hidden + c * per) = v;
    } else {
      out[row * hidden + c] = ok ? table[id * hidden + c] : T(0);
    }
  }
}

// -------------------------------------------------------- SwiGLU / add / copy ----
__device__ __forceinline__ float silu_f32(float x) {
  return __fdiv_rn(x, __fadd_rn(1.0f, expf(-x)));
}

template <typename T, bool kVector>
__global__ void swiglu_kernel(const T* __restrict__ gate, const T* __restrict__ up,
                              T* __restrict__ out, int64_t count) {
  constexpr int per = kVector ? Elem<T>::kPerVec : 1;
  const int64_t total = count / per;
  for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    if (kVector) {
      Vec16<T> g, u, o;
      g.load(gate + idx * per);
      u.load(up + idx * per);
#pragma unroll
      for (int i = 0; i < per; ++i)
        o.v[i] = Elem<T>::round(__fmul_rn(Elem<T>::round(silu_f32(g.v[i])), u.v[i]));
      o.store(out + idx * per);
    } else {
      const float g = Elem<T>::round(silu_f32(Elem<T>::load(gate + idx)));
      Elem<T>::store(out + idx, __fmul_rn(g, Elem<T>::load(up + idx)));
    }
  }
}

template <typename T, bool kVector>
__global__ void add_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out,
                           int64_t count) {
  constexpr int per = kVector ? Elem<T>::kPerVec : 1;
  const int64_t total = count / per;
  for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    if (kVector) {
      Vec16<T> x, y, o;
      x.load(a + idx * per);
      y.load(b + idx * per);
#pragma unroll
      for (int i = 0; i < per; ++i) o.v[i] = __fadd_rn(x.v[i], y.v[i]);
      o.store(out + idx * per);
    } else {
      Elem<T>::store(out + idx, __fadd_rn(Elem<T>::load(a + idx), Elem<T>::load(b + idx)));
    }
  }
}

template <typename TIn, typename TOut>
__global__ void copy4d_kernel(const TIn* __restrict__ in, TOut* __restrict__ out, int64_t n0,
                              int64_t n1, int64_t n2, int64_t n3, Strides4 st) {
  const int64_t total = n0 * n1 * n2 * n3;
  for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t i3 = idx % n3;
    int64_t r = idx / n3;
    const int64_t i2 = r % n2;
    r /= n2;
    const int64_t i1 = r % n1;
    const int64_t i0 = r / n1;
    const float v = Elem<TIn>::load(in + i0 * st.s[0] + i1 * st.s[1] + i2 * st.s[2] + i3 * st.s[3]);
    Elem<TOut>::store(out + idx, v);
  }
}

// ------------------------------------------------------------ lengths / argmax ----
__global__ void advance_lengths_kernel(int64_t* lengths, int64_t count, int64_t delta,
                                       int64_t capacity, int32_t* status) {
  const int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (idx >= count) return;
  int64_t v = lengths[idx] + delta;
  if (v > capacity) {
    v = capacity;
    if (status != nullptr) atomicOr(status, B200_STATUS_KV_OVERFLOW);
  }
  lengths[idx] = v;
}

// ------------------------------------------------------------ mask classifier ----
// flag[0] stays 1 only if every entry of the additive B x 1 x T x T mask is exactly 0 on and
// below the diagonal and -inf above it (the mask make_qwen2_prefill_inputs builds,
// qwen2.py:552-572). Grid-stride over B * T * T entries; a CTA that finds a violation clears
// the flag once. The caller sets flag[0] = 1 before the launch (b200_classify_causal_mask does).
// ------------------------------------------------------------ paged KV store ----
// pool[block_table[b, (pos + t) / bs] * bs + (pos + t) % bs, h, :] = x[b, h, t, :]: the positional
// write of serve.kv.store through a block table. One thread moves one 16-byte chunk of K and of V.
template <typename T>
__global__ void paged_kv_store_kernel(T* __restrict__ kpool, T* __restrict__ vpool,
                                      const int32_t* __restrict__ table, const T* __restrict__ key,
                                      const T* __restrict__ value, const int64_t* __restrict__ positions,
                                      int64_t batch, int64_t heads, int64_t tokens, int64_t dim,
                                      int64_t block_size, int64_t table_stride, int64_t num_blocks,
                                      Strides4 ks, Strides4 vs, int32_t* status) {
  constexpr int per = Elem<T>::kPerVec;
  const int64_t chunks = dim / per;
  const int64_t total = batch * tokens * heads * chunks;
  for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t c = idx % chunks, h = (idx / chunks) % heads;
    const int64_t t = (idx / (chunks * heads)) % tokens, b = idx / (chunks * heads * tokens);
    const int64_t pos = positions[b] + t;
    if (pos < 0 || pos >= table_stride * block_size) {
      if (status != nullptr) atomicOr(status, pos < 0 ? B200_STATUS_BAD_POSITION : B200_STATUS_KV_OVERFLOW);
      continue;
    }
    const int64_t block = table[b * table_stride + pos / block_size];
    if (block < 0 || block >= num_blocks) {  // a table entry nobody assigned
      if (status != nullptr) atomicOr(status, B200_STATUS_BAD_POSITION);
      continue;
    }
    const int64_t dst = ((block * block_size + pos % block_size) * heads + h) * dim + c * per;
    Vec16<T> kv, vv;
    kv.load(key + b * ks.s[0] + h * ks.s[1] + t * ks.s[2] + c * per);
    vv.load(value + b * vs.s[0] + h * vs.s[1] + t * vs.s[2] + c * per);
    kv.store(kpool + dst);
    vv.store(vpool + dst);
  }
}

// ------------------------------------------------------------ weight preparation ----
// out[r, c] = round(weight[r, c] * scale[c]): a norm weight folded into the columns of the
// projection that follows the norm. One-time, at load.
template <typename T>
__global__ void scale_columns_kernel(const T* __restrict__ weight, const T* __restrict__ scale,
                                     T* __restrict__ out, int64_t total, int64_t columns) {
  for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x)
    Elem<T>::store(out + idx, Elem<T>::load(weight + idx) * Elem<T>::load(scale + idx % columns));
}

__global__ void set_flag_kernel(int32_t* flag) { *flag = 1; }

template <typename T>
__global__ void classify_causal_mask_kernel(const T* __restrict__ mask, int64_t batch,
                                            int64_t tokens, int64_t stride_b, int64_t stride_q,
                                            int64_t stride_k, int32_t* flag) {
  const int64_t total = batch * tokens * tokens;
  bool ok = true;
  for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t k = idx % tokens;
    const int64_t q = (idx / tokens) % tokens;
    const int64_t b = idx / (tokens * tokens);
    const float v = Elem<T>::load(mask + b * stride_b + q * stride_q + k * stride_k);
    ok = ok && (k <= q ? v == 0.0f : (v == -INFINITY));
  }
  if (__syncthreads_or(!ok) && threadIdx.x == 0) atomicAnd(flag, 0);
}

constexpr int kArgmaxThreads = 1024;

template <typename T>
__global__ void argmax_kernel(const T* __restrict__ logits, int64_t* __restrict__ ids,
                              int64_t vocab, int64_t row_stride, bool vector_ok) {
  constexpr int per = Elem<T>::kPerVec;
  const T* row = logits + blockIdx.x * row_stride;
  float best = -INFINITY;
  int64_t best_idx = INT64_MAX;
  if (vector_ok) {
    const int64_t chunks = vocab / per;
    for (int64_t c = threadIdx.x; c < chunks; c += blockDim.x) {
      Vec16<T> x;
      x.load(row + c * per);
#pragma unroll
      for (int i = 0; i < per; ++i) {
        // strictly greater keeps the lowest index inside one thread's ascending scan
        if (x.v[i] > best || best_idx == INT64_MAX) {
          best = x.v[i];
          best_idx = c * per + i;
        }
      }
    }
    for (int64_t i = chunks * per + threadIdx.x; i < vocab; i += blockDim.x) {
      const float v = Elem<T>::load(row + i);
      if (v > best || best_idx == INT64_MAX) {
        best = v;
        best_idx = i;
      }
    }
  } else {
    for (int64_t i = threadIdx.x; i < vocab; i += blockDim.x) {
      const float v = Elem<T>::load(row + i);
      if (v > best || best_idx == INT64_MAX) {
        best = v;
        best_idx = i;
      }
    }
  }
  // warp then block reduction on (value, index): larger value wins, lower index on ties
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int64_t oi = __shfl_xor_sync(0xffffffffu, best_idx, o);
    if (ov > best || (ov == best && oi < best_idx)) {
      best = ov;
      best_idx = oi;
    }
  }
  __shared__ float s_val[32];
  __shared__ int64_t s_idx[32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) {
    s_val[warp] = best;
    s_idx[warp] = best_idx;
  }
  __syncthreads();
  if (warp == 0) {
    const int warps = blockDim.x >> 5;
    best = lane < warps ? s_val[lane] : -INFINITY;
    best_idx = lane < warps ? s_idx[lane] : INT64_MAX;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int64_t oi = __shfl_xor_sync(0xffffffffu, best_idx, o);
      if (ov > best || (ov == best && oi < best_idx)) {
        best = ov;
        best_idx = oi;
      }
    }
    if (lane == 0) ids[blockIdx.x] = best_idx == INT64_MAX ? 0 : best_idx;
  }
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

int b200_kv_store(void* key_buffer, void* value_buffer, const void* key, const void* value,
                  const int64_t* positions, int64_t batch, int64_t capacity, int64_t kv_heads,
                  int64_t tokens, int64_t head_dim, const int64_t key_strides[4],
                  const int64_t value_strides[4], int dtype, int32_t* status, void* stream) {
  if (!key_buffer || !value_buffer || !key || !value || !positions || !key_strides ||
      !value_strides || batch < 0 || capacity <= 0 || kv_heads <= 0 || tokens < 0 ||
      head_dim <= 0)
    return B200_ERR_BAD_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int code = B200_ERR_UNSUPPORTED;
  with_element_type(dtype, [&](auto tag) {
    using T = typename decltype(tag)::type;
    code = kv_store_typed<T>(key_buffer, value_buffer, key, value, positions, batch, capacity,
                             kv_heads, tokens, head_dim, key_strides, value_strides, status, s);
  });
  return code;
}

int b200_rope(const void* query, const void* key, const void* cosine, const void* sine,
              void* query_out, void* key_out, int64_t batch, int64_t q_heads, int64_t kv_heads,
              int64_t tokens, int64_t head_dim, const int64_t query_strides[4],
              const int64_t key_strides[4], const int64_t cos_strides[3],
              const int64_t sin_strides[3], int dtype, void* stream) {
  if (!query || !key || !cosine || !sine || !query_out || !key_out || !query_strides ||
      !key_strides || !cos_strides || !sin_strides || batch < 0 || q_heads <= 0 ||
      kv_heads <= 0 || tokens < 0 || head_dim <= 0)
    return B200_ERR_BAD_ARGUMENT;
  if (head_dim % 2 != 0) return B200_ERR_UNSUPPORTED;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int code = B200_ERR_UNSUPPORTED;
  with_element_type(dtype, [&](auto tag) {
    using T = typename decltype(tag)::type;
    code = rope_typed<T>(query, key, cosine, sine, query_out, key_out, batch, q_heads, kv_heads,
                         tokens, head_dim, query_strides, key_strides, cos_strides, sin_strides, s);
  });
  return code;
}

int b200_rope_kv_store(const void* query, const void* key, const void* value, const void* cosine,
                       const void* sine, void* query_out, void* key_buffer, void* value_buffer,
                       const int64_t* positions, int64_t batch, int64_t q_heads, int64_t kv_heads,
                       int64_t head_dim, int64_t capacity, int64_t q_batch_stride,
                       int64_t q_head_stride, int64_t k_batch_stride, int64_t k_head_stride,
                       int64_t v_batch_stride, int64_t v_head_stride, int64_t cos_batch_stride,
                       int dtype, int32_t* status, void* stream) {
  if (!query || !key || !value || !cosine || !sine || !query_out || !key_buffer ||
      !value_buffer || !positions || batch < 0 || q_heads <= 0 || kv_heads <= 0 ||
      head_dim <= 0 || capacity <= 0)
    return B200_ERR_BAD_ARGUMENT;
  if (!known_dtype(dtype)) return B200_ERR_UNSUPPORTED;
  const size_t elt = dtype_bytes(dtype);
  const int per = 16 / static_cast<int>(elt);
  if (head_dim % 2 != 0 || (head_dim / 2) % per != 0) return B200_ERR_UNSUPPORTED;
  const void* ptrs[] = {query, key, value, cosine, sine, query_out, key_buffer, value_buffer};
  for (const void* p : ptrs)
    if (!aligned16(p)) return B200_ERR_ALIGNMENT;
  const int64_t strides[] = {q_batch_stride, q_head_stride, k_batch_stride, k_head_stride,
                             v_batch_stride, v_head_stride, cos_batch_stride};
  for (int64_t st : strides)
    if ((st * static_cast<int64_t>(elt)) % 16 != 0) return B200_ERR_ALIGNMENT;
  const int64_t total = batch * (q_heads + 2 * kv_heads) * (head_dim / 2 / per);
  if (total == 0) return B200_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int grid = grid_for(total);
  with_element_type(dtype, [&](auto tag) {
    using T = typename decltype(tag)::type;
    rope_kv_store_kernel<T><<<grid, kThreads, 0, s>>>(
        static_cast<const T*>(query), static_cast<const T*>(key), static_cast<const T*>(value),
        static_cast<const T*>(cosine), static_cast<const T*>(sine), static_cast<T*>(query_out),
        static_cast<T*>(key_buffer), static_cast<T*>(value_buffer), positions, batch, q_heads,
        kv_heads, head_dim, capacity, q_batch_stride, q_head_stride, k_batch_stride,
        k_head_stride, v_batch_stride, v_head_stride, cos_batch_stride, status);
  });
  return launch_status();
}

int b200_rope_table(const int64_t* position_ids, const float* inv_freq, void* cosine, void* sine,
                    int64_t rows, int64_t half_dim, int out_dtype, void* stream) {
  if (!position_ids || !inv_freq || !cosine || !sine || rows < 0 || half_dim <= 0)
    return B200_ERR_BAD_ARGUMENT;
  if (rows == 0) return B200_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int grid = grid_for(rows * half_dim);
  const bool known = with_element_type(out_dtype, [&](auto tag) {
    using T = typename decltype(tag)::type;
    rope_table_kernel<T><<<grid, kThreads, 0, s>>>(position_ids, inv_freq, static_cast<T*>(cosine),
                                                   static_cast<T*>(sine), rows, half_dim);
  });
  return known ? launch_status() : B200_ERR_UNSUPPORTED;
}

int b200_embedding(const void* table, const int64_t* ids, void* output, int64_t rows,
                   int64_t hidden, int64_t vocab, int dtype, int32_t* status, void* stream) {
  if (!table || !ids || !output || rows < 0 || hidden <= 0 || vocab <= 0)
    return B200_ERR_BAD_ARGUMENT;
  if (!known_dtype(dtype)) return B200_ERR_UNSUPPORTED;
  if (rows == 0) return B200_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int per = 16 / static_cast<int>(dtype_bytes(dtype));
  const bool vec = hidden % per == 0 && aligned16(table) && aligned16(output);
  const int grid = grid_for(rows * (vec ? hidden / per : hidden));
  with_element_type(dtype, [&](auto tag) {
    using T = typename decltype(tag)::type;
    if (vec)
      embedding_kernel<T, true><<<grid, kThreads, 0, s>>>(
          static_cast<const T*>(table), ids, static_cast<T*>(output), rows, hidden, vocab, status);
    else
      embedding_kernel<T, false><<<grid, kThreads, 0, s>>>(
          static_cast<const T*>(table), ids, static_cast<T*>(output), rows, hidden, vocab, status);
  });
  return launch_status();
}

int b200_swiglu(const void* gate, const void* up, void* output, int64_t count, int dtype,
                void* stream) {
  if (!gate || !up || !output || count < 0) return B200_ERR_BAD_ARGUMENT;
  if (!known_dtype(dtype)) return B200_ERR_UNSUPPORTED;
  if (count == 0) return B200_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int per = 16 / static_cast<int>(dtype_bytes(dtype));
  const bool vec = count % per == 0 && aligned16(gate) && aligned16(up) && aligned16(output);
  const int grid = grid_for(vec ? count / per : count);
  with_element_type(dtype, [&](auto tag) {
    using T = typename decltype(tag)::type;
    if (vec)
      swiglu_kernel<T, true><<<grid, kThreads, 0, s>>>(static_cast<const T*>(gate),
                                                       static_cast<const T*>(up),
                                                       static_cast<T*>(output), count);
    else
      swiglu_kernel<T, false><<<grid, kThreads, 0, s>>>(static_cast<const T*>(gate),
                                                        static_cast<const T*>(up),
                                                        static_cast<T*>(output), count);
  });
  return launch_status();
}

int b200_add(const void* a, const void* b, void* output, int64_t count, int dtype, void* stream) {
  if (!a || !b || !output || count < 0) return B200_ERR_BAD_ARGUMENT;
  if (!known_dtype(dtype)) return B200_ERR_UNSUPPORTED;
  if (count == 0) return B200_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int per = 16 / static_cast<int>(dtype_bytes(dtype));
  const bool vec = count % per == 0 && aligned16(a) && aligned16(b) && aligned16(output);
  const int grid = grid_for(vec ? count / per : count);
  with_element_type(dtype, [&](auto tag) {
    using T = typename decltype(tag)::type;
    if (vec)
      add_kernel<T, true><<<grid, kThreads, 0, s>>>(static_cast<const T*>(a),
                                                    static_cast<const T*>(b),
                                                    static_cast<T*>(output), count);
    else
      add_kernel<T, false><<<grid, kThreads, 0, s>>>(static_cast<const T*>(a),
                                                     static_cast<const T*>(b),
                                                     static_cast<T*>(output), count);
  });
  return launch_status();
}

int b200_copy_4d(const void* input, void* output, const int64_t sizes[4],
                 const int64_t input_strides[4], int in_dtype, int out_dtype, void* stream) {
  if (!input || !output || !sizes || !input_strides) return B200_ERR_BAD_ARGUMENT;
  int64_t total = 1;
  Strides4 st;
  for (int i = 0; i < 4; ++i) {
    if (sizes[i] < 0) return B200_ERR_BAD_ARGUMENT;
    total *= sizes[i];
    st.s[i] = input_strides[i];
  }
  if (total == 0) return B200_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int grid = grid_for(total);
  if (!known_dtype(in_dtype) || !known_dtype(out_dtype)) return B200_ERR_UNSUPPORTED;
  with_element_type(in_dtype, [&](auto in_tag) {
    using TIn = typename decltype(in_tag)::type;
    with_element_type(out_dtype, [&](auto out_tag) {
      using TOut = typename decltype(out_tag)::type;
      copy4d_kernel<TIn, TOut><<<grid, kThreads, 0, s>>>(static_cast<const TIn*>(input),
                                                          static_cast<TOut*>(output), sizes[0],
                                                          sizes[1], sizes[2], sizes[3], st);
    });
  });
  return launch_status();
}

int b200_advance_lengths(int64_t* lengths, int64_t slots, int64_t batch, int64_t delta,
                         int64_t capacity, int32_t* status, void* stream) {
  if (!lengths || slots < 0 || batch < 0 || delta <= 0 || capacity <= 0)
    return B200_ERR_BAD_ARGUMENT;
  const int64_t count = slots * batch;
  if (count == 0) return B200_OK;
  advance_lengths_kernel<<<static_cast<int>(ceil_div(count, kThreads)), kThreads, 0,
                           static_cast<cudaStream_t>(stream)>>>(lengths, count, delta, capacity,
                                                                status);
  return launch_status();
}

int b200_paged_kv_store(void* key_pool, void* value_pool, const int32_t* block_table, const void* key,
                        const void* value, const int64_t* positions, int64_t batch, int64_t heads,
                        int64_t tokens, int64_t head_dim, int64_t num_blocks, int64_t block_size,
                        int64_t max_blocks_per_sequence, const int64_t key_strides[4],
                        const int64_t value_strides[4], int dtype, int32_t* status, void* stream) {
  if (!key_pool || !value_pool || !block_table || !key || !value || !positions || !key_strides ||
      !value_strides || batch < 0 || heads <= 0 || tokens < 0 || head_dim <= 0 || num_blocks <= 0 ||
      block_size <= 0 || max_blocks_per_sequence <= 0)
    return B200_ERR_BAD_ARGUMENT;
  if (key_strides[3] != 1 || value_strides[3] != 1) return B200_ERR_UNSUPPORTED;
  if (batch == 0 || tokens == 0) return B200_OK;
  const size_t elt = dtype_bytes(dtype);
  const int per = static_cast<int>(16 / elt);
  if (!known_dtype(dtype)) return B200_ERR_UNSUPPORTED;
  if (head_dim % per != 0 || !aligned16(key_pool) || !aligned16(value_pool) || !aligned16(key) ||
      !aligned16(value))
    return B200_ERR_ALIGNMENT;
  for (int i = 0; i < 3; ++i)
    if (key_strides[i] % per != 0 || value_strides[i] % per != 0) return B200_ERR_ALIGNMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  Strides4 ks, vs;
  for (int i = 0; i < 4; ++i) {
    ks.s[i] = key_strides[i];
    vs.s[i] = value_strides[i];
  }
  const int64_t total = batch * tokens * heads * (head_dim / per);
  with_element_type(dtype, [&](auto tag) {
    using T = typename decltype(tag)::type;
    paged_kv_store_kernel<T><<<grid_for(total), kThreads, 0, s>>>(
        static_cast<T*>(key_pool), static_cast<T*>(value_pool), block_table,
        static_cast<const T*>(key), static_cast<const T*>(value), positions, batch, heads, tokens,
        head_dim, block_size, max_blocks_per_sequence, num_blocks, ks, vs, status);
  });
  return launch_status();
}

int b200_scale_columns(const void* weight, const void* scale, void* output, int64_t rows,
                       int64_t columns, int dtype, void* stream) {
  if (!weight || !scale || !output || rows < 0 || columns <= 0) return B200_ERR_BAD_ARGUMENT;
  if (rows == 0) return B200_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t total = rows * columns;
  const bool known = with_element_type(dtype, [&](auto tag) {
    using T = typename decltype(tag)::type;
    scale_columns_kernel<T><<<grid_for(total), kThreads, 0, s>>>(
        static_cast<const T*>(weight), static_cast<const T*>(scale), static_cast<T*>(output), total,
        columns);
  });
  return known ? launch_status() : B200_ERR_UNSUPPORTED;
}

int b200_classify_causal_mask(const void* mask, int64_t batch, int64_t tokens,
                              const int64_t strides[4], int dtype, int32_t* flag, void* stream) {
  if (!mask || !strides || !flag || batch <= 0 || tokens <= 0) return B200_ERR_BAD_ARGUMENT;
  if (!known_dtype(dtype)) return B200_ERR_UNSUPPORTED;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // a batch-broadcast mask (stride 0) is checked once
  const int64_t distinct = strides[0] == 0 ? 1 : batch;
  const int64_t total = distinct * tokens * tokens;
  const int grid = static_cast<int>(std::min<int64_t>(ceil_div(total, kThreads), 16 * kNumSMs));
  set_flag_kernel<<<1, 1, 0, s>>>(flag);
  with_element_type(dtype, [&](auto tag) {
    using T = typename decltype(tag)::type;
    classify_causal_mask_kernel<T><<<grid, kThreads, 0, s>>>(
        static_cast<const T*>(mask), distinct, tokens, strides[0], strides[2], strides[3], flag);
  });
  return launch_status();
}

int b200_argmax(const void* logits, int64_t* ids, int64_t rows, int64_t vocab,
                int64_t row_stride, int dtype, void* stream) {
  if (!logits || !ids || rows < 0 || vocab <= 0 || row_stride < vocab)
    return B200_ERR_BAD_ARGUMENT;
  if (rows == 0) return B200_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const size_t elt = dtype_bytes(dtype);
  const bool vec = aligned16(logits) && (row_stride * static_cast<int64_t>(elt)) % 16 == 0;
  const bool known = with_element_type(dtype, [&](auto tag) {
    using T = typename decltype(tag)::type;
    argmax_kernel<T><<<static_cast<int>(rows), kArgmaxThreads, 0, s>>>(
        static_cast<const T*>(logits), ids, vocab, row_stride, vec);
  });
  return known ? launch_status() : B200_ERR_UNSUPPORTED;
}

}  // extern "C"
