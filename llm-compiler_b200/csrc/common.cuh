// Shared device helpers for the sm_100a KernelIR backend.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "b200_serve.h"

namespace b200 {

constexpr int kNumSMs = 148;  // B200: 2 dies x 74 SMs; grids are sized in multiples of this

inline int launch_status() {
  return cudaGetLastError() == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}

// Sum over the K slices of one element in slice order. All loads of a round of up to 16 slices
// are issued before the first add (absent slices add +0.0f, which changes nothing): a thread
// pays one memory latency per 16 slices. A rolled loop over the slices would stall at every add
// and serialise the latencies (measured: 0.45 us per extra slice in the decode consumers).
__device__ __forceinline__ float sum_slices(const float* first, int64_t slice, int splits) {
  float acc = 0.0f;
  for (int s = 0; s < splits; s += 16) {
    float t[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) t[j] = s + j < splits ? __ldcg(first + (s + j) * slice) : 0.0f;
#pragma unroll
    for (int j = 0; j < 16; ++j) acc += t[j];
  }
  return acc;
}

// ---- Programmatic dependent launch -------------------------------------------------------
// With B200_LAUNCH_PROGRAMMATIC set (b200_set_launch_mode) the kernels of the decode chain are
// launched with programmatic stream serialisation: a kernel may become resident while its
// predecessor in the stream still runs. Every such kernel signals its own dependents at its
// top and executes grid_dependency_wait() before its first access to memory that another
// kernel writes, and before its first write; only set-up (mbarriers, tensor memory) and, with
// B200_LAUNCH_CONSTANT_WEIGHTS, loads of weight operands come before the wait. Completion is
// transitive: the wait returns once the predecessor has finished, and the predecessor could
// not finish before its own wait did.
int launch_mode();  // defined in api.cu
unsigned wait_limit();  // polls a bounded in-kernel wait makes before it gives up (b200_debug_set_waits)
int drop_loads();       // debug: producers issue no copies, so that every bounded wait runs out

__device__ __forceinline__ void grid_dependency_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
// The same for a whole CTA: one thread waits for the prerequisite grids (whose writes are then
// visible to this grid), the others sleep in the CTA barrier and take no issue slots from the
// kernels still running on the SM. Every thread of the CTA must call it.
__device__ __forceinline__ void grid_dependency_wait_cta() {
  if (threadIdx.x == 0) grid_dependency_wait();
  __syncthreads();
}
__device__ __forceinline__ void grid_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// Thread-block cluster helpers: a barrier over all threads of the cluster (release / acquire,
// so shared-memory writes before it are visible to the other CTAs after it) and a load from
// the shared memory of the cluster's CTA `rank` at the offset of a local address.
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n"
               "barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
__device__ __forceinline__ float load_cluster_f32(uint32_t local_smem_addr, int rank) {
  uint32_t remote;
  float value;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_smem_addr), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(value) : "r"(remote) : "memory");
  return value;
}

__device__ __forceinline__ float4 load_cluster_f32x4(uint32_t local_smem_addr, int rank) {
  uint32_t remote;
  float4 value;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_smem_addr), "r"(rank));
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(value.x), "=f"(value.y), "=f"(value.z), "=f"(value.w)
               : "r"(remote)
               : "memory");
  return value;
}
__device__ __forceinline__ int cluster_cta_rank() {
  uint32_t rank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  return static_cast<int>(rank);
}

// Launches `kernel`; under B200_LAUNCH_PROGRAMMATIC with the programmatic attribute. Only for
// kernels that execute grid_dependency_wait(). A cluster extent > 1 makes that many consecutive
// CTAs along x (or z) a thread-block cluster.
template <typename... Params, typename... Args>
inline cudaError_t launch_chained_cluster_xz(void (*kernel)(Params...), dim3 grid, dim3 block,
                                             size_t smem, cudaStream_t stream, unsigned cluster_x,
                                             unsigned cluster_z, Args&&... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[2];
  unsigned count = 0;
  if ((launch_mode() & B200_LAUNCH_PROGRAMMATIC) != 0) {
    attribute[count].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[count].val.programmaticStreamSerializationAllowed = 1;
    ++count;
  }
  if (cluster_x > 1 || cluster_z > 1) {
    attribute[count].id = cudaLaunchAttributeClusterDimension;
    attribute[count].val.clusterDim.x = cluster_x;
    attribute[count].val.clusterDim.y = 1;
    attribute[count].val.clusterDim.z = cluster_z;
    ++count;
  }
  config.attrs = count > 0 ? attribute : nullptr;
  config.numAttrs = count;
  return cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);
}
template <typename... Params, typename... Args>
inline cudaError_t launch_chained_cluster(void (*kernel)(Params...), dim3 grid, dim3 block,
                                          size_t smem, cudaStream_t stream, unsigned cluster_x,
                                          Args&&... args) {
  return launch_chained_cluster_xz(kernel, grid, block, smem, stream, cluster_x, 1u,
                                   static_cast<Args&&>(args)...);
}
template <typename... Params, typename... Args>
inline cudaError_t launch_chained(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem,
                                  cudaStream_t stream, Args&&... args) {
  return launch_chained_cluster(kernel, grid, block, smem, stream, 1u, static_cast<Args&&>(args)...);
}

// ---- Timeline trace (only in builds with -DB200_TRACE) -----------------------------------
// Thread 0 of every block of a traced kernel records {kernel id, block, SM, globaltimer and
// SM clock at the top, after the dependency wait, at the end} into a caller-provided device
// buffer (b200_trace_attach): word 0 is the next free record, records of 8 words follow.
#ifdef B200_TRACE
static __constant__ unsigned long long* c_trace_buffer;
void register_trace_setter(void (*setter)(unsigned long long*));  // api.cu
static void set_trace_buffer_of_this_file(unsigned long long* buffer) {
  cudaMemcpyToSymbol(c_trace_buffer, &buffer, sizeof(buffer));
}
namespace {
struct TraceRegistrar {
  TraceRegistrar() { register_trace_setter(&set_trace_buffer_of_this_file); }
} g_trace_registrar;
}  // namespace
constexpr unsigned kTraceRecords = 65536;
__device__ __forceinline__ unsigned long long trace_globaltimer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)::"memory");
  return t;
}
struct TraceScope {
  unsigned long long* record;
  __device__ __forceinline__ TraceScope(int kernel_id) : record(nullptr) {
    const unsigned block = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
    if (threadIdx.x != 0 || c_trace_buffer == nullptr) return;
    const unsigned long long slot = atomicAdd(c_trace_buffer, 1ull) % kTraceRecords;
    record = c_trace_buffer + 1 + slot * 8;
    unsigned smid;
    asm volatile("mov.u32 %0, %smid;" : "=r"(smid));
    record[0] = static_cast<unsigned long long>(kernel_id) | (static_cast<unsigned long long>(block) << 16) |
                (static_cast<unsigned long long>(smid) << 48);
    record[1] = trace_globaltimer();
    record[2] = clock64();
    record[3] = record[5] = record[7] = 0;
  }
  __device__ __forceinline__ void mark(int which) {  // 0: after the wait, 1: end
    if (record == nullptr) return;
    record[3 + 2 * which] = trace_globaltimer();
    record[4 + 2 * which] = clock64();
  }
  __device__ __forceinline__ void mark_middle() {  // one more globaltimer sample
    if (record != nullptr) record[7] = trace_globaltimer();
  }
  // extra globaltimer samples in the words that otherwise hold SM clocks (2, 4, 6)
  __device__ __forceinline__ void stamp(int word) {
    if (record != nullptr) record[word] = trace_globaltimer();
  }
};
// Fine-grained samples from block 0 of a kernel: up to 62 SM-clock values per row of 64
// words (word 0: kernel id, word 1: top of the kernel), rows behind the records, the row
// counter in the word before them. Any one thread of block 0 may own a row.
constexpr unsigned kTraceSampleRows = 512;
struct TraceSamples {
  unsigned long long* row;
  __device__ __forceinline__ TraceSamples(int kernel_id, bool owner) : row(nullptr) {
    if (!owner || c_trace_buffer == nullptr || blockIdx.x + blockIdx.y + blockIdx.z != 0) return;
    unsigned long long* area = c_trace_buffer + 1 + 8ull * kTraceRecords;
    const unsigned long long r = atomicAdd(area, 1ull) % kTraceSampleRows;
    row = area + 1 + r * 64;
    row[0] = static_cast<unsigned long long>(kernel_id) | (static_cast<unsigned long long>(gridDim.x) << 16);
    row[1] = trace_globaltimer();
    for (int i = 2; i < 64; ++i) row[i] = 0;
  }
  __device__ __forceinline__ void sample(int i) {
    if (row != nullptr && i >= 0 && i < 62) row[2 + i] = clock64();  // cheap: SM cycles
  }
};
#else
struct TraceScope {
  __device__ __forceinline__ TraceScope(int) {}
  __device__ __forceinline__ void mark(int) {}
  __device__ __forceinline__ void mark_middle() {}
  __device__ __forceinline__ void stamp(int) {}
};
struct TraceSamples {
  __device__ __forceinline__ TraceSamples(int, bool) {}
  __device__ __forceinline__ void sample(int) {}
};
#endif

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

__host__ __device__ inline size_t dtype_bytes(int dtype) { return dtype == B200_F32 ? 4 : 2; }

// ---- bf16 <-> fp32, always round-to-nearest-even (PyTorch's .to(bfloat16)) ----
__device__ __forceinline__ float bf16_to_f32(uint16_t bits) {
  return __uint_as_float(static_cast<uint32_t>(bits) << 16);
}
__device__ __forceinline__ uint16_t f32_to_bf16_bits(float value) {
  return __bfloat16_as_ushort(__float2bfloat16_rn(value));
}
__device__ __forceinline__ float round_bf16(float value) {
  return __bfloat162float(__float2bfloat16_rn(value));
}
// One packed conversion (round to nearest even, both halves): two single conversions would
// each take a slot of the quarter-rate conversion unit that the exponentials also need.
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t packed;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(packed) : "f"(hi), "f"(lo));
  return packed;
}
__device__ __forceinline__ float bf16_lo(uint32_t packed) { return __uint_as_float(packed << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t packed) {
  return __uint_as_float(packed & 0xffff0000u);
}
// Two values rounded to bf16 with one conversion instruction instead of two.
__device__ __forceinline__ void round_bf16_pair(float& a, float& b) {
  const uint32_t packed = pack_bf16x2(a, b);
  a = bf16_lo(packed);
  b = bf16_hi(packed);
}

// Element traits so that one kernel body serves f32 and bf16 tensors.
template <typename T>
struct Elem;
template <>
struct Elem<float> {
  static constexpr int kPerVec = 4;  // elements per 16-byte vector
  __device__ static float load(const float* p) { return *p; }
  __device__ static void store(float* p, float v) { *p = v; }
  __device__ static float round(float v) { return v; }
  __device__ static void round_pair(float&, float&) {}
};
template <>
struct Elem<__nv_bfloat16> {
  static constexpr int kPerVec = 8;
  __device__ static float load(const __nv_bfloat16* p) { return __bfloat162float(*p); }
  __device__ static void store(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
  __device__ static float round(float v) { return round_bf16(v); }
  __device__ static void round_pair(float& a, float& b) { round_bf16_pair(a, b); }  // one conversion
};
template <>
struct Elem<__half> {  // fp16 tensors run on the generic (non-tensor-core) kernels only
  static constexpr int kPerVec = 8;
  __device__ static float load(const __half* p) { return __half2float(*p); }
  __device__ static void store(__half* p, float v) { *p = __float2half_rn(v); }
  __device__ static float round(float v) { return __half2float(__float2half_rn(v)); }
  __device__ static void round_pair(float& a, float& b) {
    const float2 r = __half22float2(__floats2half2_rn(a, b));
    a = r.x;
    b = r.y;
  }
};

// Calls f(TypeTag<T>{}) with the element type of a dtype code; false for an unknown code.
template <typename T>
struct TypeTag { using type = T; };
template <typename F>
inline bool with_element_type(int dtype, F&& f) {
  switch (dtype) {
    case B200_F32: f(TypeTag<float>{}); return true;
    case B200_BF16: f(TypeTag<__nv_bfloat16>{}); return true;
    case B200_F16: f(TypeTag<__half>{}); return true;
    default: return false;
  }
}
inline bool known_dtype(int dtype) { return dtype == B200_F32 || dtype == B200_BF16 || dtype == B200_F16; }

// 16-byte vector of elements, unpacked to floats and back.
template <typename T>
struct Vec16;
template <>
struct Vec16<float> {
  float v[4];
  __device__ void load(const float* p) {
    float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  }
  __device__ void store(float* p) const {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
};
template <>
struct Vec16<__nv_bfloat16> {
  float v[8];
  __device__ void load(const __nv_bfloat16* p) {
    uint4 t = *reinterpret_cast<const uint4*>(p);
    v[0] = bf16_lo(t.x); v[1] = bf16_hi(t.x); v[2] = bf16_lo(t.y); v[3] = bf16_hi(t.y);
    v[4] = bf16_lo(t.z); v[5] = bf16_hi(t.z); v[6] = bf16_lo(t.w); v[7] = bf16_hi(t.w);
  }
  __device__ void store(__nv_bfloat16* p) const {
    uint4 t;
    t.x = pack_bf16x2(v[0], v[1]); t.y = pack_bf16x2(v[2], v[3]);
    t.z = pack_bf16x2(v[4], v[5]); t.w = pack_bf16x2(v[6], v[7]);
    *reinterpret_cast<uint4*>(p) = t;
  }
};

template <>
struct Vec16<__half> {
  float v[8];
  __device__ void load(const __half* p) {
    const uint4 t = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      v[2 * i] = f.x;
      v[2 * i + 1] = f.y;
    }
  }
  __device__ void store(__half* p) const {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
      w[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
  }
};

// ---- warp / block reductions -------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// ---- async copies (global -> shared, 16 bytes, L1 bypass) ---------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void cp_async16(uint32_t smem_addr, const void* gptr) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_addr), "l"(gptr));
}
// Copies src_bytes (0 or 16) and zero-fills the rest: out-of-range rows become zeros.
__device__ __forceinline__ void cp_async16_zfill(uint32_t smem_addr, const void* gptr,
                                                 int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_addr), "l"(gptr),
               "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

// ---- warp-level tensor-core primitives (bf16 in, fp32 accumulate) --------------
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t smem_addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t smem_addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_addr));
}
// D(16x8, f32) += A(16x16, bf16, row) * B(16x8, bf16, col)
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                               uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// ---- TMA (tensor-map bulk copies) and mbarriers ----------------------------------
__device__ __forceinline__ void mbarrier_init(uint32_t bar, uint32_t arrive_count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%1], %0;\n" ::"r"(arrive_count), "r"(bar) : "memory");
}
__device__ __forceinline__ void fence_mbarrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
}
__device__ __forceinline__ void mbarrier_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%1], %0;\n" ::"r"(bytes), "r"(bar)
               : "memory");
}
// Adds `bytes` to the transaction count of the current phase without arriving.
__device__ __forceinline__ void mbarrier_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%1], %0;\n" ::"r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ bool mbarrier_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred P1;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 P1, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, P1;\n\t}"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done != 0;
}
// Bounded wait: gives up after `limit` polls (each poll may itself block for a
// hardware-defined slice) instead of spinning forever; the caller records the failure.
__device__ __forceinline__ bool mbarrier_wait_bounded(uint32_t bar, uint32_t parity,
                                                      uint32_t limit = 4000000u) {
  for (uint32_t i = 0; i < limit; ++i)
    if (mbarrier_try_wait(bar, parity)) return true;
  return false;
}
// A try_wait that succeeds at once still takes about 200 cycles, a test_wait a fraction of
// that: where the phase has usually completed already, test first and suspend only if not.
__device__ __forceinline__ bool mbarrier_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred P1;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 P1, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, P1;\n\t}"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done != 0;
}
__device__ __forceinline__ bool mbarrier_wait_ready_first(uint32_t bar, uint32_t parity,
                                                          uint32_t limit = 4000000u) {
  if (mbarrier_test_wait(bar, parity)) return true;
  return mbarrier_wait_bounded(bar, parity, limit);
}
// Same bound, polling with the non-suspending test: for a wait whose latency matters more
// than the issue slots one spinning thread takes.
__device__ __forceinline__ bool mbarrier_spin_bounded(uint32_t bar, uint32_t parity,
                                                      uint32_t limit = 40000000u) {
  for (uint32_t i = 0; i < limit; ++i) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred P1;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 P1, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, P1;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}
// One 3-D box of a tiled tensor map into shared memory; completion is signalled on `bar`.
// Every CTA fetches its own tiles: no load is shared between the CTAs of a cluster.
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const void* tensor_map, uint32_t bar,
                                            int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5}], [%2];\n" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(tensor_map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const void* tensor_map, uint32_t bar,
                                            int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5, %6}], [%2];\n" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(tensor_map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* tensor_map, uint32_t bar,
                                            int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4}], [%2];\n" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(tensor_map)), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}

// The box a tma_load_2d at these coordinates would copy, requested into L2 only: no shared
// memory, no barrier, nothing to wait for.
__device__ __forceinline__ void tma_prefetch_l2_2d(const void* tensor_map, int c0, int c1) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];\n" ::"l"(
                   reinterpret_cast<uint64_t>(tensor_map)),
               "r"(c0), "r"(c1)
               : "memory");
}

// Shared-memory tiles whose rows are 128 bytes (64 bf16) are stored with the 16-byte
// chunk index XOR-ed by (row & 7): ldmatrix reads of 8 consecutive rows at one logical
// chunk then touch 8 different bank groups.
__device__ __forceinline__ int swizzle128(int row, int chunk) { return chunk ^ (row & 7); }

}  // namespace b200
