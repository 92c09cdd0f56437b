/*
 * b200_serve.h -- C ABI of the sm_100a KernelIR backend (libb200serve.so).
 *
 * Every entry point replaces one kernel wrapper (or one PyTorch fallback op) of
 * StatefulLLM-Compiler's GPU executor; the reference symbol each one stands in
 * for is cited as  <file>:<lines>  relative to the reference project root
 * (src/stateful_llm_compiler/...).
 *
 * Conventions
 *  - All pointers are DEVICE pointers unless the name ends in _host.
 *  - Dimensions and strides are int64; strides are in ELEMENTS.
 *  - `stream` is a cudaStream_t passed as void* (NULL = legacy default stream).
 *  - The library never allocates, frees or synchronises: the caller owns every
 *    buffer, workspaces included. Calls are therefore legal inside CUDA graph
 *    capture (the one exception is documented on the entry point itself).
 *  - Return value: 0 on success, a negative B200_ERR_* code when the request is
 *    rejected on the host (nothing was launched).
 *  - Errors that only the device can see (a KV position past the capacity, a
 *    token id outside the vocabulary, a length above the mask length) never
 *    trap: the kernel skips / clamps the access and ORs a B200_STATUS_* bit into
 *    the caller's int32 status word, which the host reads at a step boundary.
 */
#ifndef B200_SERVE_H_
#define B200_SERVE_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* element types */
#define B200_F32 0
#define B200_BF16 1
#define B200_F16 2 /* generic (non-tensor-core) kernels only; the reference's kernels accept it:
                      backends/triton_linear.py:100-105 */

/* numerical modes: lowering.py:24-37 (_NUMERICAL_LOWERINGS) */
#define B200_MODE_FAST 0
#define B200_MODE_PYTORCH_COMPATIBLE 1

/* host-side rejections */
#define B200_OK 0
#define B200_ERR_BAD_ARGUMENT (-1)  /* null pointer, negative size, bad enum          */
#define B200_ERR_UNSUPPORTED (-2)   /* dtype / head_dim / stride the kernels do not do */
#define B200_ERR_ALIGNMENT (-3)     /* a pointer or stride breaks the 16-byte rule      */
#define B200_ERR_WORKSPACE (-4)     /* workspace missing or too small                  */
#define B200_ERR_LAUNCH (-5)        /* cudaLaunch / cudaGetLastError reported an error */
#define B200_ERR_TOO_LARGE (-6)     /* beyond a documented fixed maximum               */

/* device-side status bits (OR-ed into *status) */
#define B200_STATUS_KV_OVERFLOW 1       /* position + tokens > capacity: write skipped    */
#define B200_STATUS_LENGTH_OVER_MASK 2  /* lengths[b] > mask length: clamped              */
#define B200_STATUS_BAD_TOKEN_ID 4      /* embedding id outside [0, vocab): row zeroed    */
#define B200_STATUS_BAD_POSITION 8      /* negative KV position: write skipped            */
#define B200_STATUS_WAIT_TIMEOUT 16     /* a bounded in-kernel wait gave up: result invalid */

/* launch-mode flags (b200_set_launch_mode) */
#define B200_LAUNCH_PROGRAMMATIC 1      /* decode-chain kernels use programmatic dependent launch */
#define B200_LAUNCH_CONSTANT_WEIGHTS 2  /* weight operands are written by no kernel in flight  */
#define B200_LAUNCH_STABLE_KV_PREFIX 4  /* lengths[] and KV rows < lengths[b] - 1 likewise       */
#define B200_LAUNCH_LINEAR_WARP_LEVEL 8    /* b200_linear: warp-level kernel, not tcgen05       */
#define B200_LAUNCH_PREFILL_WARP_LEVEL 16  /* b200_prefill_attention: warp-level kernel         */

/* Launch mode of the CALLING THREAD for the decode-chain kernels (linear on tcgen05 incl. the
 * partial-sum, folded-norm and cluster split-K forms, the two reduce_* consumers, decode
 * attention; every other kernel, advance_lengths / embedding / rope table among them, is always
 * launched fully serialised, which is what makes lengths[] stable before the attention's wait).
 * Thread-local: two engines driven from two threads do not see each other's promises; launches
 * captured into a CUDA graph keep the mode they were captured with. No counterpart in the
 * reference, whose Triton launches are always
 * fully serialised (ReferenceExecutor.run, execution.py:530-575, runs one operation after another).
 * B200_LAUNCH_PROGRAMMATIC: each of those kernels may become resident before its predecessor
 * in the stream has finished and waits on the device (griddepcontrol.wait) before touching
 * any tensor; results are unchanged. B200_LAUNCH_CONSTANT_WEIGHTS additionally lets a linear
 * kernel fetch its `weight` tiles before that wait: only valid while no kernel that writes a
 * weight tensor is in flight on the device. B200_LAUNCH_STABLE_KV_PREFIX lets decode attention
 * read lengths[] and request the KV rows below lengths[b] - 1 before the wait: valid when the
 * only KV row written since the previous synchronisation point is the newest one (row
 * lengths[b] - 1, stored by the kernel just before attention), as in a decode step whose
 * lengths were advanced at the end of the step before. The two *_WARP_LEVEL flags pick the
 * kernel variant a profile-guided dispatch plan chose (the reference resolves its plan to a
 * backend per call, cost_model.py:220-245). Returns the previous flags, or
 * B200_ERR_BAD_ARGUMENT for unknown bits. Default 0. */
int b200_set_launch_mode(int flags);
int b200_get_launch_mode(void);

/* Debug control of the bounded in-kernel waits (no counterpart in the reference, whose kernels
 * have no waits to bound). Every mbarrier wait of the TMA / tcgen05 kernels gives up after
 * `poll_limit` polls (default 4,000,000), sets B200_STATUS_WAIT_TIMEOUT, frees its tensor memory
 * and returns. drop_loads != 0 makes the copy-issuing threads of those kernels issue nothing, so
 * that with a small limit every wait runs out at once with no copy in flight: how the tests
 * exercise the give-up paths without faulting or hanging the GPU. Process-wide; returns the
 * previous limit (or B200_ERR_BAD_ARGUMENT). Restore (4000000, 0) afterwards. */
int64_t b200_debug_set_waits(int64_t poll_limit, int drop_loads);

/* Version / build probe. Returns 100 * major + minor of this ABI. */
int b200_abi_version(void);
/* Human-readable message for a B200_ERR_* code (static storage). */
const char* b200_error_string(int code);

/* ---- KV store --------------------------------------------------------------
 * buf[b, positions[b] + t, h, :] = x[b, h, t, :] for K and V in one launch.
 * Replaces triton_kv_store (backends/triton_kv.py:71-129); oracle native_kv_store
 * (execution.py:1242-1280). key/value are B x Hkv x T x D with arbitrary element
 * strides (they arrive as view+transpose); buffers are contiguous B x C x Hkv x D.
 * Bit-exact copy. */
int b200_kv_store(void* key_buffer, void* value_buffer, const void* key, const void* value,
                  const int64_t* positions, int64_t batch, int64_t capacity, int64_t kv_heads,
                  int64_t tokens, int64_t head_dim, const int64_t key_strides[4],
                  const int64_t value_strides[4], int dtype, int32_t* status, void* stream);

/* ---- RoPE --------------------------------------------------------------------
 * Dual-output Qwen2 half rotation, y = r(r(x*cos) + r(rot(x)*sin)).
 * Replaces triton_rope (backends/triton_rope.py:299-390); oracle
 * ReferenceExecutor._serve_rope (execution.py:741-767). q: B x Hq x T x D, k: B x Hkv x T x D
 * (strided, last dim contiguous), cos/sin: B x T x D. Outputs are contiguous
 * B x H x T x D. Same rounding points in both numerical modes. */
int b200_rope(const void* query, const void* key, const void* cosine, const void* sine,
              void* query_out, void* key_out, int64_t batch, int64_t q_heads, int64_t kv_heads,
              int64_t tokens, int64_t head_dim, const int64_t query_strides[4],
              const int64_t key_strides[4], const int64_t cos_strides[3],
              const int64_t sin_strides[3], int dtype, void* stream);

/* Decode fusion of serve.rope + serve.kv.store (T == 1): rotates q into query_out
 * (B x Hq x D contiguous), rotates k and writes it with v straight into the KV
 * buffers at positions[b]. Same arithmetic as b200_rope followed by b200_kv_store
 * (passes/kv_bufferize.py:175-200 orders them rope -> length -> store). */
int b200_rope_kv_store(const void* query, const void* key, const void* value, const void* cosine,
                       const void* sine, void* query_out, void* key_buffer, void* value_buffer,
                       const int64_t* positions, int64_t batch, int64_t q_heads, int64_t kv_heads,
                       int64_t head_dim, int64_t capacity, int64_t q_batch_stride,
                       int64_t q_head_stride, int64_t k_batch_stride, int64_t k_head_stride,
                       int64_t v_batch_stride, int64_t v_head_stride, int64_t cos_batch_stride,
                       int dtype, int32_t* status, void* stream);

/* cos/sin table from position ids: f = float(pos) * inv_freq, e = cat(f, f),
 * cos = r(cos(e)), sin = r(sin(e)). Replaces the unlowered aten.to/unsqueeze/mul/cat/
 * cos/sin chain of Qwen2RotaryEmbedding.forward (qwen2.py:136-149). rows = B*T,
 * outputs rows x (2*half_dim). */
int b200_rope_table(const int64_t* position_ids, const float* inv_freq, void* cosine, void* sine,
                    int64_t rows, int64_t half_dim, int out_dtype, void* stream);

/* ---- RMSNorm -----------------------------------------------------------------
 * Replaces triton_rms_norm (backends/triton_rmsnorm.py:205-443) and the
 * kernel.cuda.rms_norm composite (backends/triton_executor.py:149-157); oracle
 * ReferenceExecutor._serve_rms_norm (execution.py:674-692).
 * round_before_weight != 0: y = r(w * r(x * rsqrt(mean(x^2) + eps)));
 * otherwise y = r(x * rsqrt(..) * float(w)).
 * mode FAST sums x^2 in a tree; mode PYTORCH_COMPATIBLE reproduces the summation
 * order of the CPU executor's float sum (8 vector lanes x 4 interleaved
 * accumulators, cascaded) with IEEE sqrt and divide, so the result is bit-identical
 * to the reference's CPU executor. */
int b200_rms_norm(const void* input, const void* weight, void* output, int64_t rows,
                  int64_t hidden, int64_t input_row_stride, double epsilon,
                  int round_before_weight, int in_dtype, int weight_dtype, int out_dtype,
                  int mode, void* stream);

/* ---- Decode attention --------------------------------------------------------
 * One-token GQA attention over the physical B x C x Hkv x D buffers with
 * per-sequence device lengths; split-KV online softmax.
 * Replaces triton_decode_attention (backends/triton_attention.py:134-210); oracle
 * PreallocatedKVCacheState.decode_attention (execution.py:281-327).
 *  query   B x Hq x 1 x D, strides (q_batch_stride, q_head_stride), last dim contiguous
 *  mask    B x 1 x 1 x mask_len additive, dtype mask_dtype, or NULL for "all zero"
 *  output  B x Hq x D contiguous (viewed by the caller as B x Hq x 1 x D)
 *  split_tokens  tokens per split (0 = library default); max_length_hint: an upper
 *                bound on lengths[] known to the host (0 = mask_len / capacity).
 * bf16 with head_dim 64 / 128 runs the tensor-core kernel; fp32, fp16 and head_dim 16 / 32 /
 * 256 (any dtype) a generic one without scratch.
 * Workspace: b200_decode_attention_workspace_bytes(...) bytes, 256-byte aligned. */
int64_t b200_decode_attention_workspace_bytes(int64_t batch, int64_t q_heads, int64_t kv_heads,
                                              int64_t head_dim, int64_t max_length,
                                              int64_t split_tokens);
int b200_decode_attention(const void* query, const void* key_buffer, const void* value_buffer,
                          const int64_t* lengths, const void* mask, void* output, int64_t batch,
                          int64_t q_heads, int64_t kv_heads, int64_t head_dim, int64_t capacity,
                          int64_t mask_len, int64_t q_batch_stride, int64_t q_head_stride,
                          int64_t mask_batch_stride, int mask_dtype, double scale, int dtype,
                          int mode, int64_t split_tokens, int64_t max_length_hint,
                          void* workspace, int64_t workspace_bytes, int32_t* status,
                          void* stream);
/* The same with a service order (bf16): the i-th group of CTAs serves sequence sequence_order[i]
 * (int32 [batch], a permutation of 0 .. batch-1; an entry outside that range skips its group).
 * CTAs are placed in grid order, so listing the longest sequences first gives longest-first
 * scheduling when the (sequence, KV head) pairs outnumber the CTAs the GPU holds at once; the
 * result does not depend on the order. No counterpart in the reference. */
int b200_decode_attention_ordered(const void* query, const void* key_buffer, const void* value_buffer,
                                  const int64_t* lengths, const void* mask, void* output,
                                  const int32_t* sequence_order, int64_t batch, int64_t q_heads,
                                  int64_t kv_heads, int64_t head_dim, int64_t capacity,
                                  int64_t mask_len, int64_t q_batch_stride, int64_t q_head_stride,
                                  int64_t mask_batch_stride, int mask_dtype, double scale, int dtype,
                                  int mode, int64_t split_tokens, int64_t max_length_hint,
                                  void* workspace, int64_t workspace_bytes, int32_t* status,
                                  void* stream);

/* Decode attention for callers that must not allocate device memory (no counterpart in
 * the reference, whose wrappers allocate with torch.empty on every call). Some hosts of
 * this library cannot call cudaMalloc at all: code running inside a CUDA-graph capture or a
 * real-time serving loop with a frozen memory budget, plugins handed a fixed arena by their
 * framework, and runtimes whose allocator is owned by another component. For them the
 * split-KV scratch (tile counters and fp32 partials) is a fixed 8 MiB array that lives in
 * the library itself, on every GPU that loads it, until the process exits
 * (b200_decode_attention_static_scratch_bytes() returns that size). The caller still passes
 * the inputs and the output; arguments are those of b200_decode_attention without the
 * workspace pair. bf16 only (the fp32 kernel needs no scratch).
 *  - A request whose partials do not fit the array (roughly batch * q_heads * splits *
 *    (head_dim + 2) * 4 bytes + 64 KiB > 8 MiB) is refused with B200_ERR_TOO_LARGE; nothing
 *    is launched and nothing is allocated. A larger split_tokens lowers the need.
 *  - The first call on each device looks the array's device address up; make that first
 *    call outside any stream capture.
 *  - All calls on one GPU share the array, which keeps the previous call's contents (the
 *    counter region is cleared at the start of every call): two calls that overlap on the
 *    GPU, on different streams, race. Issue them on one stream or order them with events. */
int64_t b200_decode_attention_static_scratch_bytes(void);
int b200_decode_attention_static_scratch(
    const void* query, const void* key_buffer, const void* value_buffer, const int64_t* lengths,
    const void* mask, void* output, int64_t batch, int64_t q_heads, int64_t kv_heads,
    int64_t head_dim, int64_t capacity, int64_t mask_len, int64_t q_batch_stride,
    int64_t q_head_stride, int64_t mask_batch_stride, int mask_dtype, double scale, int dtype,
    int mode, int64_t split_tokens, int64_t max_length_hint, int32_t* status, void* stream);

/* ---- Paged KV layout -------------------------------------------------------------
 * The layout the reference lists as future work (README.md:295, docs/kv-bufferization.md:319-323;
 * `layout` of KVStateType, ir.py:87, and BufferizeKVCachePass(layout=...), passes/kv_bufferize.py:41-42,
 * are where it would plug in): per layer slot a pool of blocks [num_blocks, block_size, Hkv, D] for
 * K and one for V, and an int32 block table [B, max_blocks_per_sequence] that maps token t of
 * sequence b to row t % block_size of block table[b, t / block_size]. Sequences no longer need
 * contiguous slots sized for the longest context (512 x 8256-token Qwen2-7B slots are 242 GB;
 * the same sequences at their real lengths fit one GPU). Same arithmetic as the contiguous
 * entry points, results equal to them on the same logical KV:
 *   b200_paged_kv_store         serve.kv.store through the block table (bit-exact copy); a
 *                               position beyond the table's reach sets B200_STATUS_KV_OVERFLOW, a
 *                               table entry outside [0, num_blocks) B200_STATUS_BAD_POSITION
 *   b200_paged_decode_attention serve.decode_attention over the pools: one TMA box per 32-token
 *                               step, addressed through the table (block_size % 32 == 0); bf16,
 *                               head_dim 64 / 128; workspace as b200_decode_attention_workspace_bytes
 *                               with max_length = max_blocks_per_sequence * block_size
 *   b200_paged_qkv_decode_attention  b200_qkv_decode_attention (below) on this layout: the new
 *                               token's K / V row is written to the block the table names for
 *                               position lengths[b] - 1; no block there sets B200_STATUS_KV_OVERFLOW
 *                               and writes nothing */
int b200_paged_kv_store(void* key_pool, void* value_pool, const int32_t* block_table, const void* key,
                        const void* value, const int64_t* positions, int64_t batch, int64_t heads,
                        int64_t tokens, int64_t head_dim, int64_t num_blocks, int64_t block_size,
                        int64_t max_blocks_per_sequence, const int64_t key_strides[4],
                        const int64_t value_strides[4], int dtype, int32_t* status, void* stream);
int b200_paged_decode_attention(
    const void* query, const void* key_pool, const void* value_pool, const int32_t* block_table,
    const int64_t* lengths, const void* mask, void* output, int64_t batch, int64_t q_heads,
    int64_t kv_heads, int64_t head_dim, int64_t num_blocks, int64_t block_size,
    int64_t max_blocks_per_sequence, int64_t mask_len, int64_t q_batch_stride, int64_t q_head_stride,
    int64_t mask_batch_stride, int mask_dtype, double scale, int mode, int64_t split_tokens,
    int64_t max_length_hint, void* workspace, int64_t workspace_bytes, int32_t* status, void* stream);
int b200_paged_qkv_decode_attention(
    const void* qkv_partials, int64_t qkv_splits, const void* qkv_bias, const void* cosine,
    const void* sine, void* key_pool, void* value_pool, const int32_t* block_table,
    const int64_t* lengths, void* output, int64_t batch, int64_t q_heads, int64_t kv_heads,
    int64_t head_dim, int64_t num_blocks, int64_t block_size, int64_t max_blocks_per_sequence,
    int64_t mask_len, double scale, int64_t split_tokens, int64_t max_length_hint,
    int64_t length_offset, const void* norm_row_squares, int64_t norm_hidden, double norm_epsilon,
    const int32_t* sequence_order, void* workspace, int64_t workspace_bytes, int32_t* status,
    void* stream);

/* ---- Prefill attention -------------------------------------------------------
 * T-token GQA attention with an arbitrary additive B x 1 x T x T mask, or with
 * proven causality (causal != 0: mask may be NULL and fully masked tiles are skipped).
 * Replaces triton_prefill_attention (backends/triton_prefill_attention.py:152-232);
 * oracle ReferenceExecutor._serve_prefill_attention (execution.py:707-739).
 * q: B x Hq x T x D, k/v: B x Hkv x T x D strided (last dim contiguous);
 * output memory is B x T x Hq x D contiguous (the caller views it as B x Hq x T x D).
 * bf16 calls in the fast mode run on tcgen05 (S and O tiles in tensor memory, operands by
 * TMA): causal-proved ones, and masked ones (the reference's `causal: "mask"` contract,
 * passes/prefill_attention.py:173-180) when the mask is fp32 with a contiguous last dimension
 * and a workspace of b200_prefill_attention_workspace_bytes(batch, tokens) is given; a pre-pass
 * then classifies the mask's 128 x 128 tiles (all zero / all -inf / mixed) so that tiles that
 * are all -inf at either end of a row block are never touched and all-zero tiles read no mask.
 * Other masked calls and the pytorch_compatible mode use the warp-level kernel; fp32, fp16 and
 * head_dim 16 / 32 / 256 (any dtype) a generic CUDA-core kernel (workspace may be NULL). status (may be NULL) receives B200_STATUS_WAIT_TIMEOUT. */
int64_t b200_prefill_attention_workspace_bytes(int64_t batch, int64_t tokens);
int b200_prefill_attention(const void* query, const void* key, const void* value,
                           const void* mask, void* output, int64_t batch, int64_t q_heads,
                           int64_t kv_heads, int64_t tokens, int64_t head_dim,
                           const int64_t query_strides[4], const int64_t key_strides[4],
                           const int64_t value_strides[4], const int64_t mask_strides[4],
                           int mask_dtype, double scale, int causal, int dtype, int mode,
                           void* workspace, int64_t workspace_bytes, int32_t* status,
                           void* stream);

/* ---- Linear ------------------------------------------------------------------
 * y[M,N] = x[M,K] * W[N,K]^T (+ bias[N]) with fp32 accumulation and an optional
 * fused epilogue. Replaces triton_linear (backends/triton_linear.py:87-148) and the
 * kernel.cublas.linear call (backends/triton_executor.py:159-176); oracle F.linear
 * (execution.py:694-705).
 * epilogue: 0 none; 1 residual add, y = r(r(acc + bias) + residual) (the unlowered
 * aten.add.Tensor that follows o_proj / down_proj, qwen2.py:299-304); 2 SwiGLU over
 * row-interleaved gate/up weights: W holds n rows (gate_j, up_j alternating), the output is
 * [M, n/2] and y[m,j] = r(r(silu(r(gate_j))) * r(up_j)) (qwen2.py:262-264).
 * bf16 problems run on tcgen05 tensor cores (TMEM accumulator, TMA-fed stage ring): 64-row
 * activation boxes and a tile width chosen at run time at decode sizes, 128 x 64..256 tiles
 * beyond, a persistent two-accumulator kernel from 1024 rows on. Decode-size calls with too
 * few N tiles to fill the GPU and operands no tensor map can describe run on the warp-level
 * kernel with deterministic split-K, fp32 and fp16 on a generic CUDA-core kernel. Workspace (split-K partial sums + tile counters):
 * b200_linear_workspace_bytes. `status` receives B200_STATUS_WAIT_TIMEOUT if a bounded
 * in-kernel wait gives up. */
#define B200_EPILOGUE_NONE 0
#define B200_EPILOGUE_RESIDUAL 1
#define B200_EPILOGUE_SWIGLU 2
int64_t b200_linear_workspace_bytes(int64_t m, int64_t k, int64_t n, int dtype, int epilogue);
int b200_linear(const void* input, const void* weight, const void* bias, const void* residual,
                void* output, int64_t m, int64_t k, int64_t n, int64_t input_row_stride,
                int dtype, int epilogue, void* workspace, int64_t workspace_bytes,
                int32_t* status, void* stream);

/* ---- Decode-step chain: split-K partial sums reduced by the operator that follows ----------
 * At decode sizes (M <= 128 rows) the projections are weight streaming: the GEMM is cut into
 * N tiles x K slices so that every SM pulls weights, each CTA writes its fp32 partial tile,
 * and the reduction over the K slices happens while the NEXT operator of the layer loads its
 * input (fixed slice order: deterministic). These entry points stand for the op sequences of
 * one decoder layer of the reference graph (qwen2.py:152-304 after the passes):
 *   b200_linear_partial            serve.linear without its epilogue: partials[s, m, n] (fp32),
 *                                  s < b200_linear_partial_splits(m, k, n); with row_squares
 *                                  (fp32 [splits, m], M <= 128; may be NULL) also the sum of
 *                                  squares of every input row over each K slice, for a consumer
 *                                  that applies an RMSNorm folded into this projection
 *   b200_reduce_residual_rms_norm  (o_proj | down_proj result) -> aten.add (residual) ->
 *                                  serve.rms_norm of the next block: x_out = r(r(sum) + residual),
 *                                  h_out = r(w * r(x_out * rsqrt(mean(x_out^2) + eps)));
 *                                  residual and h_out / norm_weight may be NULL
 *   b200_reduce_rope_kv_store      (q|k|v projection result + bias) -> serve.rope -> serve.kv.length
 *                                  -> serve.kv.store: rotated q to query_out (B x Hq x D), rotated
 *                                  k and v into the KV buffers at positions[b]
 * bf16 only; partial buffers are caller-owned, 16-byte aligned, n a multiple of 4. */
int64_t b200_linear_partial_splits(int64_t m, int64_t k, int64_t n);
int b200_linear_partial(const void* input, const void* weight, void* partials,
                        void* row_squares, int64_t m, int64_t k, int64_t n,
                        int64_t input_row_stride, int64_t splits, int32_t* status, void* stream);
int b200_reduce_residual_rms_norm(const void* partials, int64_t splits, const void* residual,
                                  const void* norm_weight, void* x_out, void* h_out, int64_t rows,
                                  int64_t hidden, double epsilon, int mode, void* stream);
int b200_reduce_rope_kv_store(const void* partials, int64_t splits, const void* bias,
                              const void* cosine, const void* sine, void* query_out,
                              void* key_buffer, void* value_buffer, const int64_t* positions,
                              int64_t batch, int64_t q_heads, int64_t kv_heads, int64_t head_dim,
                              int64_t capacity, int32_t* status, void* stream);

/* b200_reduce_rope_kv_store followed by b200_decode_attention in ONE launch, for the decode
 * step: the op sequence (q|k|v projection result + bias) -> serve.rope -> serve.kv.length ->
 * serve.kv.store -> serve.decode_attention of one decoder layer (passes/kv_bufferize.py:175-200
 * orders them so; oracle execution.py:741-767, 1242-1280, 286-333). The new token sits at row
 * lengths[b] - 1: lengths[] are the attention lengths, already counting it. Every CTA reduces
 * the query rows it needs from the partials; the CTA whose KV range holds row lengths[b] - 1
 * also reduces that token's K and V, stores them into the buffers and lets them join the
 * softmax from registers, so no CTA reads a row another one is writing. No mask (causal
 * decode), fast numerical mode, bf16, head_dim 64 or 128. cosine / sine: B x D. Workspace as
 * for b200_decode_attention. lengths[b] < 1 sets B200_STATUS_BAD_POSITION (nothing stored).
 * length_offset 1: lengths[] still hold the lengths before the new token (serve.kv.advance of
 * every slot is deferred to one launch at the end of the step); the kernel adds 1 itself.
 * sequence_order: NULL, or the service order of b200_decode_attention_ordered. */
int b200_qkv_decode_attention(const void* qkv_partials, int64_t qkv_splits, const void* qkv_bias,
                              const void* cosine, const void* sine, void* key_buffer,
                              void* value_buffer, const int64_t* lengths, void* output,
                              int64_t batch, int64_t q_heads, int64_t kv_heads, int64_t head_dim,
                              int64_t capacity, int64_t mask_len, double scale,
                              int64_t split_tokens, int64_t max_length_hint, int64_t length_offset,
                              const void* norm_row_squares, int64_t norm_hidden, double norm_epsilon,
                              const int32_t* sequence_order, void* workspace, int64_t workspace_bytes,
                              int32_t* status, void* stream);

/* ---- Decode-step chain, five launches per layer (fast mode, bf16, M <= 128 rows) ---------
 * The serve.rms_norm in front of a projection (qwen2.py:152-304: input_layernorm -> q|k|v,
 * post_attention_layernorm -> gate|up) is folded into that projection instead of being a launch
 * of its own: y = rsqrt(mean(x^2) + eps) * (x (W * w_norm)^T), with the norm weight multiplied
 * into W's columns once at load time (b200_scale_columns) and the per-row factor applied to the
 * fp32 accumulator. The bf16 roundings of the normalised activations (execution.py:686-691) are
 * skipped: allowed in the fast mode only, inside its 2e-2 tolerance. The o / down projections,
 * whose results feed a residual add (aten.add, qwen2.py:299-304), reduce their K slices among
 * the CTAs of a thread-block cluster through distributed shared memory and add the residual
 * themselves: no partials in global memory, no reduce launch.
 *   b200_scale_columns           out[n, k] = r(weight[n, k] * scale[k])   (weight preparation)
 *   b200_linear_rms_input        serve.rms_norm + serve.linear (+ bias, + SwiGLU epilogue) on the
 *                                un-normalised input and the column-scaled weight
 *   b200_linear_splitk_residual  serve.linear + aten.add: output = r(r(x W^T) + residual);
 *                                n a multiple of 4, M <= 256. With row_squares_out (fp32
 *                                [b200_linear_splitk_slices(m, k, n), m], NULL to skip) it also
 *                                leaves sum(output_r^2) in slices, for a folded RMSNorm behind it;
 *                                a slice count of 0 means this shape writes none.
 * b200_linear_rms_input with row_squares (fp32 [row_square_slices, m], as left by
 * b200_linear_splitk_residual for the same rows) adds those slices instead of squaring x itself.
 * b200_qkv_decode_attention takes the same fold for the q|k|v projection: with
 * norm_row_squares (fp32 [qkv_splits, B], what b200_linear_partial left: sum of squares of the
 * un-normalised rows of width norm_hidden per K slice) it scales the reduced sums by
 * rsqrt(mean(x_b^2) + norm_epsilon) before the bias; NULL keeps plain sums. */
int b200_scale_columns(const void* weight, const void* scale, void* output, int64_t rows,
                       int64_t columns, int dtype, void* stream);
int b200_linear_rms_input(const void* input, const void* folded_weight, const void* bias,
                          void* output, const void* row_squares, int64_t row_square_slices,
                          int64_t m, int64_t k, int64_t n, int64_t input_row_stride,
                          double epsilon, int epilogue, int32_t* status, void* stream);
int64_t b200_linear_splitk_slices(int64_t m, int64_t k, int64_t n);
int b200_linear_splitk_residual(const void* input, const void* weight, const void* residual,
                                void* output, void* row_squares_out, int64_t m, int64_t k,
                                int64_t n, int64_t input_row_stride, int32_t* status, void* stream);

/* ---- Ops the reference leaves to PyTorch eager (execution.py:500-528) ---------- */
/* aten.embedding.default: out[r,:] = table[ids[r],:]. */
int b200_embedding(const void* table, const int64_t* ids, void* output, int64_t rows,
                   int64_t hidden, int64_t vocab, int dtype, int32_t* status, void* stream);
/* aten.silu.default + aten.mul.Tensor: out = r(r(silu(gate)) * up) (qwen2.py:262-264). */
int b200_swiglu(const void* gate, const void* up, void* output, int64_t count, int dtype,
                void* stream);
/* aten.add.Tensor on same-shape contiguous tensors: out = r(a + b) (qwen2.py:299-304). */
int b200_add(const void* a, const void* b, void* output, int64_t count, int dtype, void* stream);
/* aten.contiguous.default / aten.to.dtype on a strided 4-D tensor: dense copy with
 * optional f32 <-> bf16 conversion. */
int b200_copy_4d(const void* input, void* output, const int64_t sizes[4],
                 const int64_t input_strides[4], int in_dtype, int out_dtype, void* stream);

/* ---- Runtime KV helpers --------------------------------------------------------
 * runtime.kv.advance (execution.py:421-443): lengths[b] += delta, in place so that
 * replayed CUDA graphs see fixed addresses; a length that would pass `capacity` is
 * clamped and B200_STATUS_KV_OVERFLOW is raised instead of the reference's device
 * assert (execution.py:1283-1293). `slots` length vectors of `batch` entries,
 * contiguous (slots x batch). */
int b200_advance_lengths(int64_t* lengths, int64_t slots, int64_t batch, int64_t delta,
                         int64_t capacity, int32_t* status, void* stream);
/* Run-time proof of causality for serve.prefill_attention. The reference op carries
 * `causal: "mask"` and an arbitrary additive B x 1 x T x T mask
 * (passes/prefill_attention.py:173-180) and names a proved `causal=true` as its follow-up
 * (docs/prefill-attention.md:43-45). flag[0] becomes 1 if every entry is exactly 0 on and
 * below the diagonal and -inf above it (the mask make_qwen2_prefill_inputs builds,
 * qwen2.py:552-572), else 0; the host reads it once per mask tensor and then calls
 * b200_prefill_attention with causal = 1, which reads no mask. strides are element strides
 * of the 4-D mask (a batch stride of 0 means one mask for all sequences). */
int b200_classify_causal_mask(const void* mask, int64_t batch, int64_t tokens,
                              const int64_t strides[4], int dtype, int32_t* flag, void* stream);
/* Greedy sampling: ids[r] = argmax(logits[r, :]) (lowest index wins ties), the step
 * the reference's callers do with torch.argmax (benchmarks/validate_qwen2_checkpoint.py:365-396). */
int b200_argmax(const void* logits, int64_t* ids, int64_t rows, int64_t vocab,
                int64_t row_stride, int dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200_SERVE_H_ */
