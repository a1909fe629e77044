/*
 * b200_ttperf.h — C ABI of the B200 (sm_100a) implementation of tt-perf's dense-matmul hot path.
 *
 * tt-perf's C++ executors (autograd/dynamic, autograd/static, autograd/traced) do all their
 * arithmetic through the TTNN op library: `ttnn::matmul`, `ttnn::linear`, element-wise ops,
 * row reductions, `ttnn::softmax`, `ttnn::embedding`, plus `ttnn::all_gather` for the sharded
 * matmul. This header declares the plain-C entry points those ops forward to; the C++ header
 * shim under include/ttnn/ and the ctypes binding in the Python package are both written on
 * top of exactly these functions. Each declaration cites the reference interface it stands
 * in for (paths are relative to the tt-perf tree).
 *
 * Conventions
 *  - every function returns a b200_status code (0 = success); b200_last_error() gives the text
 *    of the calling thread's last failure. No function throws, aborts or prints.
 *  - pointers named `d_*`, A, B, C, x, y ... are DEVICE pointers unless the comment says host.
 *  - `stream` is a cudaStream_t passed as void* (NULL = the context's own stream). Calls are
 *    asynchronous and in order on that stream, like ops on a TTNN command queue.
 *  - matrices are row-major with an explicit leading dimension in ELEMENTS; bf16 is the
 *    16-bit brain float stored as uint16_t bit patterns.
 *  - there is no CPU fallback: with no usable sm_100 device every compute call fails with
 *    B200_ERR_CUDA.
 */
#ifndef B200_TTPERF_H
#define B200_TTPERF_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_TTPERF_ABI_VERSION 2

typedef enum b200_status {
    B200_OK = 0,
    B200_ERR_INVALID_ARG = 1,    /* null pointer, negative size, bad enum, misaligned operand */
    B200_ERR_CUDA = 2,           /* a CUDA runtime/driver call failed (text in b200_last_error) */
    B200_ERR_UNSUPPORTED = 3,    /* valid request this build cannot serve */
    B200_ERR_DEVICE_TIMEOUT = 4, /* a kernel's bounded wait ran out; results of that launch are invalid */
    B200_ERR_NOMEM = 5,          /* device arena / workspace exhausted */
    B200_ERR_COMM = 6            /* collective layer (NCCL) failure */
} b200_status;

typedef enum b200_dtype { B200_BF16 = 0, B200_F32 = 1, B200_U32 = 2, B200_FP8_E4M3 = 3 } b200_dtype;

/* Fused activations of ttnn::linear / ttnn::matmul (static/nn.hpp:145-146, bench/metal/bench_fusion.cpp:119). */
typedef enum b200_activation { B200_ACT_NONE = 0, B200_ACT_RELU = 1, B200_ACT_GELU = 2 } b200_activation;

/* MathFidelity of WormholeComputeKernelConfig (verify/verify_fidelity.cpp:50-55). On tcgen05 the
 * accumulator is always fp32; the knob selects the precision of split-K partial sums and of the
 * epilogue math: HIFI4/HIFI3 fp32 partials + exact erf GELU; HIFI2 bf16-rounded partials; LOFI
 * bf16-rounded partials + tanh-approximated GELU. */
typedef enum b200_fidelity { B200_LOFI = 0, B200_HIFI2 = 1, B200_HIFI3 = 2, B200_HIFI4 = 3 } b200_fidelity;

typedef enum b200_gemm_algo {
    B200_GEMM_AUTO = 0,    /* tcgen05 when operands meet the TMA alignment rules, else SIMT */
    B200_GEMM_TCGEN05 = 1, /* TMA + tcgen05.mma + TMEM; fails with INVALID_ARG on misaligned operands */
    B200_GEMM_SIMT = 2     /* CUDA-core tiled kernel: any alignment, any leading dimension */
} b200_gemm_algo;

typedef struct b200_ctx b200_ctx; /* one per (process, GPU): device ordinal, stream, scratch, status word */

/* ---- context / device (MeshDevice::create_unit_mesh, autograd/common.hpp:31-37; Finish / Synchronize,
 *      examples/train_mlp.cpp:129, bench/autograd/bench_mlp.cpp:119) ---------------------------------- */
int b200_ctx_create(int device_ordinal, b200_ctx** out_ctx);
int b200_ctx_destroy(b200_ctx* ctx);
int b200_ctx_device(const b200_ctx* ctx, int* out_device_ordinal);
int b200_ctx_sm_count(const b200_ctx* ctx, int* out_sm_count);
/* The context's own stream (a cudaStream_t), the one calls with stream = NULL run on: lets the host program order its
 * own work — e.g. a collective of its communication library that serves as a barrier between ranks — after the
 * kernels queued here without a host synchronisation. */
int b200_ctx_stream(const b200_ctx* ctx, void** out_stream);
/* Blocks until all work queued on `stream` has finished, then reports a kernel wait that timed out
 * since the last call as B200_ERR_DEVICE_TIMEOUT (and clears it). */
int b200_synchronize(b200_ctx* ctx, void* stream);
/* Exercises that error path without a fault or a hang: queues a one-CTA kernel that waits, with the same bounded wait
 * the GEMM and attention kernels use but with `limit_ns` (1 us .. 100 ms) as its limit, on a barrier nothing ever
 * arrives at; when the limit runs out it raises the status word and returns. The next b200_synchronize therefore
 * reports B200_ERR_DEVICE_TIMEOUT, clears the context's status block, and the context is usable again. */
int b200_selftest_wait_timeout(b200_ctx* ctx, uint64_t limit_ns, void* stream);
/* Device-side timing as the reference's benchmarks do around Finish() (bench/metal/matmul_sweep.cpp:44-79), but with
 * CUDA events on the stream: start records an event, stop records a second one, waits for it and returns the elapsed
 * milliseconds between the two (and releases the timer). */
int b200_timer_start(b200_ctx* ctx, void* stream, void** out_timer);
int b200_timer_stop(b200_ctx* ctx, void* stream, void* timer, float* out_ms);
const char* b200_last_error(void);
int b200_abi_version(void);

/* ---- device memory (Tensor::to_device / .cpu() / .deallocate(), traced/nn.hpp:46-47, common.hpp:53) - */
int b200_malloc(b200_ctx* ctx, size_t bytes, void** out_dptr);
int b200_free(b200_ctx* ctx, void* dptr);
int b200_memcpy_h2d(b200_ctx* ctx, void* d_dst, const void* h_src, size_t bytes, void* stream);
int b200_memcpy_d2h(b200_ctx* ctx, void* h_dst, const void* d_src, size_t bytes, void* stream);
int b200_memset(b200_ctx* ctx, void* d_dst, int byte_value, size_t bytes, void* stream);
/* Device-to-device copy on the stream; either side may be a peer GPU's buffer opened with b200_ipc_open_handle (the
 * copy engine then moves the bytes over NVLink), which is how a rank pushes a row block to its peers. */
int b200_memcpy_d2d(b200_ctx* ctx, void* d_dst, const void* d_src, size_t bytes, void* stream);

/* ---- pooled tensor memory and trace record / replay (TraceContext, autograd/traced/trace.hpp:21-88:
 *      begin_trace_capture / end_trace_capture / execute_trace / release_trace; raw use in
 *      bench/autograd/bench_transformer_train.cpp:91-110) -------------------------------------------------
 * b200_pool_alloc / b200_pool_free: cached device blocks for op results (`out = ttnn::add(a, b)` allocates on every
 * call); blocks go back to the driver only when the context is destroyed.
 * b200_trace_begin starts recording the work queued on the CONTEXT stream (pass stream = NULL to the ops) into a
 * CUDA graph; b200_trace_end instantiates it; b200_trace_execute replays it (blocking != 0 waits for completion);
 * b200_trace_release destroys it. Blocks allocated while recording belong to the trace until it is released, so a
 * replay never writes into memory handed to someone else. Ops that would synchronise (b200_synchronize,
 * b200_memcpy_d2h on the context stream) or grow the context scratch fail with B200_ERR_UNSUPPORTED while
 * recording: run the step once untraced first, as the reference's benchmarks do (bench_mlp.cpp:99-102). */
int b200_pool_alloc(b200_ctx* ctx, size_t bytes, void** out_dptr);
int b200_pool_free(b200_ctx* ctx, void* dptr);
int b200_pool_stats(b200_ctx* ctx, size_t* reserved_bytes, size_t* in_use_bytes);
int b200_trace_begin(b200_ctx* ctx, uint32_t* out_trace_id);
int b200_trace_end(b200_ctx* ctx, uint32_t trace_id);
int b200_trace_execute(b200_ctx* ctx, uint32_t trace_id, int blocking);
/* Replays a trace on the caller's stream instead of the context's: the caller orders it against its own work with its
 * own events (a data-parallel step interleaves segments of the backward pass with NCCL all-reduces on another stream
 * this way). Replays of traces that share buffers must still be ordered by the caller. */
int b200_trace_execute_on(b200_ctx* ctx, uint32_t trace_id, void* stream);
int b200_trace_release(b200_ctx* ctx, uint32_t trace_id);

/* ---- dense matmul: ttnn::matmul(a, b, transpose_a, transpose_b, ..., activation, compute_kernel_config)
 *      (dynamic/ops.hpp:21-46, static/ops.hpp:21-45, traced/ops.hpp:26-36) and
 *      ttnn::linear(x, w, bias, ta, tb, ..., "relu") (static/nn.hpp:145-146) --------------------------
 *
 *   C[b] = act( mask( alpha * op(A[b]) . op(B[b]) + bias ) )          b = 0 .. batch-1
 *
 *   op(A) is M x K: A is stored [M, K] (transpose_a = 0) or [K, M] (transpose_a = 1), leading dim lda.
 *   op(B) is K x N: B is stored [K, N] (transpose_b = 0) or [N, K] (transpose_b = 1), leading dim ldb.
 *   stride_a / stride_b / stride_c: elements between consecutive batch entries; 0 broadcasts an
 *   operand over the batch (rank-2 weight against [B,S,D] activations, traced/transformer.hpp:198).
 *   bias: optional [N] row vector broadcast over rows ([1,N] bias add, traced/nn.hpp:73).
 *   causal_mask: entries with column > row are replaced by mask_value before the activation
 *   (the -1e9 upper-triangular mask of traced/nn.hpp:158-168, fused with the 1/sqrt(dh) scale = alpha).
 *   Inputs bf16, accumulation fp32, output bf16 or fp32 (fp32_dest_acc_en / K-split partial sums).
 */
typedef struct b200_gemm_desc {
    int32_t transpose_a;
    int32_t transpose_b;
    int64_t M, N, K;
    int64_t batch; /* >= 1 */
    const void* A;
    int64_t lda;
    int64_t stride_a;
    const void* B;
    int64_t ldb;
    int64_t stride_b;
    void* C;
    int64_t ldc;
    int64_t stride_c;
    int32_t c_dtype;    /* B200_BF16 or B200_F32 */
    const void* bias;   /* NULL or [N] */
    int32_t bias_dtype; /* B200_BF16 or B200_F32 */
    int32_t activation; /* b200_activation */
    float alpha;
    int32_t causal_mask;
    float mask_value;
    int32_t fidelity; /* b200_fidelity */
    int32_t algo;     /* b200_gemm_algo */
    int32_t split_k;  /* 0 = choose; 1 = never split; n > 1 = split K into n slices (fp32 scratch + reduce) */
    int32_t ab_dtype; /* B200_BF16 (default) or B200_FP8_E4M3: A and B hold 8-bit e4m3 values (one byte per element,
                       * lda / ldb / strides in elements, multiples of 16). The tensor cores then run at twice the bf16
                       * rate (tcgen05 kind::f8f6f4, fp32 accumulation). 8-bit operands cannot be read transposed:
                       * transpose_a must be 0 and transpose_b 1 (the Linear forward form x . W^T). `alpha` carries the
                       * de-quantisation factor 1 / (scale_a * scale_b). This is the reduced-fidelity matmul of the
                       * reference's fidelity study (verify/verify_fidelity.cpp:50-67, 151-208: LoFi trades mantissa
                       * bits of the operands for speed) in B200 terms. */
} b200_gemm_desc;

/* Fills a descriptor with defaults: no transposes, batch 1, alpha 1, bf16 operands and output, HIFI4, AUTO. */
void b200_gemm_desc_init(b200_gemm_desc* desc);
/* K-sliced products (split_k != 1), attention backward, column reductions and LayerNorm backward keep intermediate
 * sums in ONE scratch block, ticket-counter set and staging area per context. Calls that use them on different
 * streams are serialised by the library (the later stream waits for an event recorded on the earlier one), so they
 * are safe but do not overlap; give concurrent streams their own contexts when that matters. When a call needs more
 * scratch than the context holds, the block is reallocated: a device-wide synchronisation plus cudaFree / cudaMalloc
 * (b200_gemm_scratch_bytes tells how much a product needs; run the largest shape once up front). While recorded
 * traces exist the outgrown block stays mapped until the last trace is released, since replays write to the address
 * they recorded. */
int b200_gemm(b200_ctx* ctx, const b200_gemm_desc* desc, void* stream);
/* The same product with A, B and C in HOST memory (pinned memory gives full PCIe speed) — the path a reference program
 * takes from Tensor::from_vector / to_device through ttnn::matmul to .cpu() (bench/metal/matmul_tensor_parallel.cpp:
 * 56-93), as one pipelined call: B is uploaded once, A in `panels` row panels (0 = default 8), each panel's GEMM starts
 * when its rows have landed and its rows of C are downloaded while the next panel computes. Batch 1. Blocks until C is
 * complete in host memory. Device staging buffers are kept in the context and grown on demand. */
int b200_matmul_host(b200_ctx* ctx, const b200_gemm_desc* desc_with_host_pointers, int panels);
/* Bytes of context scratch the split-K path of this descriptor will use (0 when it does not split). */
int b200_gemm_scratch_bytes(b200_ctx* ctx, const b200_gemm_desc* desc, size_t* out_bytes);

/* Which kernel serves a product, and how. The reference sweeps TTNN's program configurations per shape
 * (bench/metal/matmul_sweep.cpp:85-117 core grids, bench/autograd/bench_shape_sweep.cpp:57-121); here the library
 * plans by itself (b200_gemm), the plan can be read (b200_gemm_plan_query, b200_gemm_plan_describe: the kernel's
 * name and tiling as text, e.g. for a benchmark report) and a sweep can run any other plan (b200_gemm_planned).
 *   kernel    B200_GEMM_KERNEL_SIMT          CUDA-core kernel, any alignment
 *             B200_GEMM_KERNEL_TCGEN05       one CTA per 128 x block_n tile (block_n in {64, 128, 192, 256})
 *             B200_GEMM_KERNEL_TCGEN05_PAIR  two CTAs (cta_group::2) per 256 x 256 tile; needs 16-byte aligned rows of C
 *   k_slices  K is cut into this many slices (0 and 1 = no cut); the single-CTA kernel sums them in a second
 *             launch, the pair kernel inside the same launch
 *   group_m   row-tiles per column sweep of the tile order (0 = default) */
typedef enum b200_gemm_kernel {
    B200_GEMM_KERNEL_SIMT = 0, B200_GEMM_KERNEL_TCGEN05 = 1, B200_GEMM_KERNEL_TCGEN05_PAIR = 2
} b200_gemm_kernel;
typedef struct b200_gemm_plan {
    int32_t kernel;
    int32_t block_n;
    int32_t k_slices;
    int32_t group_m;
} b200_gemm_plan;
int b200_gemm_plan_query(b200_ctx* ctx, const b200_gemm_desc* desc, b200_gemm_plan* out_plan);
int b200_gemm_plan_describe(const b200_gemm_desc* desc, const b200_gemm_plan* plan, char* buf, size_t buf_bytes);
int b200_gemm_planned(b200_ctx* ctx, const b200_gemm_desc* desc, const b200_gemm_plan* plan, void* stream);

/* ---- fused attention (traced/nn.hpp:164-192 TracedCausalAttention; transformer_train.hpp:54-70
 * SharedAttentionBuffers::attention_forward / attention_backward; py/nn.py:229-253) ----
 * O = softmax(scale * Q K^T + mask) V per (batch, head), computed tile by tile on the tensor cores without writing the
 * [S, S] score or probability matrices to memory: the forward keeps a running row maximum and row sum and emits, next
 * to O, the row log-sum-exp `lse` (natural log, of the scaled and masked scores); the backward recomputes the
 * probabilities from Q, K and lse. With causal != 0 key j is visible to query i only when j <= i (the reference adds
 * -1e9 above the diagonal, traced/nn.hpp:158-161; here those terms are exactly zero).
 *   operand: bf16, element (b, h, s, d) at ptr[b*stride_b + h*stride_h + s*stride_s + d]; strides in elements and
 *            multiples of 8, ptr 16-byte aligned. [B,H,S,64] tensors and the un-permuted [B,S,H*64] output of a
 *            projection (stride_h = 64, stride_s = row length) are both expressible, so no head split/merge copy is needed.
 *   head_dim must be 64 (B200_ERR_UNSUPPORTED otherwise: compose b200_gemm + b200_softmax instead).
 *   lse      fp32 [B, H, S]
 * b200_attention_backward: given dO it writes dQ, dK, dV (bf16, any operand layout). It uses B*H*S*64 + 2*B*H*S' floats
 * of context scratch (S' = S rounded up to 128): fp32 dQ accumulators, summed with TMA reductions over the key tiles,
 * and the per-query terms of the pass (lse and the row sums of dO * O, pre-scaled and padded).
 * The _hp forms carry one more bf16 tensor between the passes, o_lo = bf16(O - bf16(O)): what the rounding of O to bf16
 * drops. The backward pass needs the row term rowsum(dO * O); with O known only to bf16 that term is off by up to 2^-9
 * of |dO| |O|, equally for every key of the row, and dQ = dS K (dK = dS^T Q) multiplies that common error with whatever
 * the keys (queries) have in common — visible in dQ and dK when attention is nearly uniform or nearly one-hot. With
 * o_lo the row term has fp32 accuracy for 2 more bytes per output element. o_lo = NULL gives the plain forms. */
typedef struct b200_attn_operand {
    void* ptr;
    int64_t stride_b, stride_h, stride_s;
} b200_attn_operand;
int b200_attention_forward(b200_ctx* ctx, const b200_attn_operand* q, const b200_attn_operand* k, const b200_attn_operand* v,
                           const b200_attn_operand* o, float* lse, int64_t B, int64_t H, int64_t S, int head_dim,
                           float scale, int causal, void* stream);
int b200_attention_backward(b200_ctx* ctx, const b200_attn_operand* q, const b200_attn_operand* k,
                            const b200_attn_operand* v, const b200_attn_operand* o, const b200_attn_operand* d_o,
                            const float* lse, const b200_attn_operand* d_q, const b200_attn_operand* d_k,
                            const b200_attn_operand* d_v, int64_t B, int64_t H, int64_t S, int head_dim, float scale,
                            int causal, void* stream);
int b200_attention_forward_hp(b200_ctx* ctx, const b200_attn_operand* q, const b200_attn_operand* k, const b200_attn_operand* v,
                              const b200_attn_operand* o, const b200_attn_operand* o_lo, float* lse, int64_t B, int64_t H,
                              int64_t S, int head_dim, float scale, int causal, void* stream);
int b200_attention_backward_hp(b200_ctx* ctx, const b200_attn_operand* q, const b200_attn_operand* k,
                               const b200_attn_operand* v, const b200_attn_operand* o, const b200_attn_operand* o_lo,
                               const b200_attn_operand* d_o, const float* lse, const b200_attn_operand* d_q,
                               const b200_attn_operand* d_k, const b200_attn_operand* d_v, int64_t B, int64_t H, int64_t S,
                               int head_dim, float scale, int causal, void* stream);

/* The backward pass with options. flags = 0 is b200_attention_backward_hp. B200_ATTN_DETERMINISTIC: every key tile
 * stores its contribution to dQ into a slab of its own instead of adding it to one accumulator with atomic reductions,
 * and the final kernel sums the slabs in key order: two runs on the same inputs give the same bits (the default sums in
 * whatever order the key tiles arrive). It needs ceil(S / 128) times the scratch of the accumulator (B*H*S*64 floats per
 * key tile) and is the slower of the two. */
#define B200_ATTN_DETERMINISTIC 1u
int b200_attention_backward_opts(b200_ctx* ctx, const b200_attn_operand* q, const b200_attn_operand* k,
                                 const b200_attn_operand* v, const b200_attn_operand* o, const b200_attn_operand* o_lo,
                                 const b200_attn_operand* d_o, const float* lse, const b200_attn_operand* d_q,
                                 const b200_attn_operand* d_k, const b200_attn_operand* d_v, int64_t B, int64_t H, int64_t S,
                                 int head_dim, float scale, int causal, unsigned flags, void* stream);

/* ---- row softmax family (traced/ops.hpp:77-81 softmax, :102-106 softmax_backward; py/engine.py:352-384) ----
 * [rows, cols] bf16 matrices, leading dimensions in elements.
 * b200_softmax: y = softmax(alpha * x) along each row. causal_period P > 0 additionally hides, in row r, the
 *   columns > r % P — the [B,H,S,S] score tensor flattened to [B*H*S, S] with P = S gets the upper-triangular
 *   -1e9 mask of traced/nn.hpp:158-168 and the 1/sqrt(dh) scale (alpha) in the same pass.
 * b200_softmax_backward: dx = alpha * y * (dy - sum_row(dy * y)).
 * b200_log_softmax / _backward: y = log softmax(x); dx = dy - exp(y) * sum_row(dy) (py/engine.py:368-381). */
int b200_softmax(b200_ctx* ctx, const void* x, int64_t ldx, void* y, int64_t ldy, int64_t rows, int64_t cols, float alpha,
                 int64_t causal_period, void* stream);
int b200_softmax_backward(b200_ctx* ctx, const void* dy, int64_t lddy, const void* y, int64_t ldy, void* dx, int64_t lddx,
                          int64_t rows, int64_t cols, float alpha, void* stream);
int b200_log_softmax(b200_ctx* ctx, const void* x, int64_t ldx, void* y, int64_t ldy, int64_t rows, int64_t cols,
                     void* stream);
int b200_log_softmax_backward(b200_ctx* ctx, const void* dy, int64_t lddy, const void* log_y, int64_t ldy, void* dx,
                              int64_t lddx, int64_t rows, int64_t cols, void* stream);

/* ---- fused cross-entropy (CrossEntropyLoss, py/nn.py:149-222; last_token_cross_entropy, py/experiment.py:50-118) -
 * One pass over bf16 logits [rows, classes]: per-row loss -log softmax(x)[label] and, when d_logits is not NULL,
 * d_logits = (softmax(x) - onehot(label)) * grad_scale (grad_scale = 1/rows for the mean reduction). Labels are
 * uint32 class ids on the device (no one-hot tensor is built). loss_sum (device fp32 scalar, optional) receives
 * grad_scale * sum of row losses, i.e. the mean loss for grad_scale = 1/rows; row_loss (device fp32 [rows], optional)
 * receives the unscaled per-row losses. */
int b200_cross_entropy(b200_ctx* ctx, const void* logits, int64_t ld, const uint32_t* labels, int64_t rows, int64_t classes,
                       float grad_scale, float* loss_sum, float* row_loss, void* d_logits, int64_t ldd, void* stream);

/* ---- LayerNorm (TracedLayerNorm forward ~10 TTNN ops / backward ~14, traced/nn.hpp:226-269) ----------------
 * Forward: y = (x - mean) * rstd * gamma + beta over the last dim (biased variance, eps inside the sqrt); mean and
 * rstd (device fp32 [rows], optional) are saved for the backward pass.
 * Backward: dx (bf16, optional) and fp32 dgamma / dbeta [cols] (optional; overwritten, not accumulated). */
int b200_layernorm_forward(b200_ctx* ctx, const void* x, int64_t ldx, const void* gamma, const void* beta, void* y,
                           int64_t ldy, float* mean, float* rstd, int64_t rows, int64_t cols, float eps, void* stream);
int b200_layernorm_backward(b200_ctx* ctx, const void* dy, int64_t lddy, const void* x, int64_t ldx, const void* gamma,
                            const float* mean, const float* rstd, void* dx, int64_t lddx, float* dgamma_f32,
                            float* dbeta_f32, int64_t rows, int64_t cols, void* stream);
/* The same with the residual connection folded in, so that no separate element-wise add runs
 * (transformer_train.hpp:201,212,228,250,256 add the residual in a pass of its own):
 * b200_add_layernorm_forward: sum_out = x + residual (bf16), y = LayerNorm(sum_out); mean / rstd are those of sum_out.
 * b200_layernorm_backward_add: dx = LayerNorm'(dy) + upstream, the gradient that reaches the same tensor along the
 *   residual path. Both accept every shape the plain calls accept. */
int b200_add_layernorm_forward(b200_ctx* ctx, const void* x, int64_t ldx, const void* residual, int64_t ldres, void* sum_out,
                               int64_t ldsum, const void* gamma, const void* beta, void* y, int64_t ldy, float* mean,
                               float* rstd, int64_t rows, int64_t cols, float eps, void* stream);
int b200_layernorm_backward_add(b200_ctx* ctx, const void* dy, int64_t lddy, const void* x, int64_t ldx, const void* gamma,
                                const float* mean, const float* rstd, const void* upstream, int64_t ldup, void* dx,
                                int64_t lddx, float* dgamma_f32, float* dbeta_f32, int64_t rows, int64_t cols, void* stream);
/* The general form: upstream may be NULL; dx_colsum_bf16 (optional, [cols] bf16) receives the column sums of the dx
 * that is written. dx is the gradient of a residual stream, i.e. the dY of the Linear layer that feeds that stream
 * (attention output projection, FC2), so these sums ARE that layer's bias gradient (db = sum_batch dy, static/nn.hpp:
 * 84-86) and no separate reduction over dx has to run. */
int b200_layernorm_backward_full(b200_ctx* ctx, const void* dy, int64_t lddy, const void* x, int64_t ldx, const void* gamma,
                                 const float* mean, const float* rstd, const void* upstream, int64_t ldup, void* dx,
                                 int64_t lddx, float* dgamma_f32, float* dbeta_f32, void* dx_colsum_bf16, int64_t rows,
                                 int64_t cols, void* stream);

/* ---- element-wise ops on bf16 buffers ------------------------------------------------------------------------
 * Unary (ttnn::neg / relu / gtz / gelu / rsqrt ..., traced/ops.hpp:54-61; tensor (+,*) float forms, traced/ops.hpp:38-52). */
typedef enum b200_unary_op {
    B200_U_NEG = 0, B200_U_RELU = 1, B200_U_GTZ = 2, B200_U_GELU = 3, B200_U_RSQRT = 4, B200_U_EXP = 5, B200_U_LOG = 6,
    B200_U_TANH = 7, B200_U_SQRT = 8, B200_U_ADD_SCALAR = 9, B200_U_MUL_SCALAR = 10, B200_U_RSUB_SCALAR = 11,
    B200_U_COPY = 12, B200_U_RECIP = 13, B200_U_SQUARE = 14
} b200_unary_op;
int b200_unary(b200_ctx* ctx, int op, const void* x, void* y, int64_t n, float scalar, void* stream);

/* Binary with numpy-style broadcasting (ttnn::add / subtract / multiply with [1,N], [1,1,S,S], [B,S,1] operands,
 * dynamic/ops.hpp:50-134). Shapes are rank 4 (pad with leading 1s); each dim must match or be 1. RELU_BW and GELU_BW
 * take (dy, x): dy * (x > 0) (the gtz mask multiply, traced/ops.hpp:55-57) and ttnn::gelu_bw(dy, x, "none")
 * (traced/ops.hpp:96-99). */
typedef enum b200_binary_op {
    B200_B_ADD = 0, B200_B_SUB = 1, B200_B_MUL = 2, B200_B_DIV = 3, B200_B_RELU_BW = 4, B200_B_GELU_BW = 5, B200_B_MAX = 6
} b200_binary_op;
int b200_binary(b200_ctx* ctx, int op, const void* a, const int64_t a_shape[4], const void* b, const int64_t b_shape[4],
                void* out, void* stream);

/* Reduction of the middle dim of a contiguous bf16 [outer, R, inner] view (ttnn::sum / mean / max(t, dim, keepdim),
 * traced/ops.hpp:63-73; bias gradient = column sum over the batch, traced/nn.hpp:81). Output [outer, inner] bf16.
 * inner > 1 uses outer*inner fp32 words of context scratch. */
typedef enum b200_reduce_op { B200_R_SUM = 0, B200_R_MEAN = 1, B200_R_MAX = 2 } b200_reduce_op;
int b200_reduce(b200_ctx* ctx, int op, const void* x, int64_t outer, int64_t R, int64_t inner, void* y, void* stream);

/* dx = dy * GELU'(x_pre) over a contiguous bf16 [rows, cols] tensor (ttnn::gelu_bw(dy, x, "none"), traced/ops.hpp:96-99)
 * and, when dx_colsum is not NULL, the column sums of the stored dx (bf16 [cols]) from the same pass: dx is the dY of the
 * Linear layer in front of the GELU and its column sums are that layer's bias gradient (traced/nn.hpp:81). The result
 * equals b200_binary(GELU_BW) followed by b200_reduce(SUM) bit for bit in dx; the sums are taken over the rounded dx in
 * fp32 and rounded once. Uses at most 256 fp32 words of context scratch per column. */
int b200_gelu_backward(b200_ctx* ctx, const void* dy, const void* x_pre, void* dx, void* dx_colsum, int64_t rows,
                       int64_t cols, void* stream);

/* 8-bit operands for b200_gemm with ab_dtype = B200_FP8_E4M3.
 * b200_absmax: out_f32[0] = max |x| over n bf16 elements (device scalar, overwritten).
 * b200_quantize_fp8: y[i] = e4m3(x[i] * scale), saturating at +-448; a caller picks scale = 448 / absmax. */
int b200_absmax(b200_ctx* ctx, const void* x_bf16, int64_t n, float* out_f32, void* stream);
int b200_quantize_fp8(b200_ctx* ctx, const void* x_bf16, int64_t n, float scale, void* y_fp8, void* stream);
/* y[c * ldy + r] = e4m3(x[r * ldx + c] * scale) for a [rows, cols] bf16 matrix: the transposed 8-bit copy that the
 * dX (NN) and dW (TN) products of a Linear need, because 8-bit operands are read K-major only. */
int b200_quantize_fp8_transposed(b200_ctx* ctx, const void* x_bf16, int64_t rows, int64_t cols, int64_t ldx, float scale,
                                 void* y_fp8, int64_t ldy, void* stream);
/* Creation and conversion (ttnn::zeros / ones / full / full_like, traced/nn.hpp:30-52). `value` is converted to dtype. */
int b200_fill(b200_ctx* ctx, void* dst, int64_t n, int dtype, float value, void* stream);
int b200_cast(b200_ctx* ctx, const void* src, int src_dtype, void* dst, int dst_dtype, int64_t n, void* stream);

/* Layout: out = permute(x, perm) for a contiguous rank-4 16-bit tensor (ttnn::transpose(t, 1, 2) for the head
 * split/merge, transformer_train.hpp:167-177; ttnn::transpose(weight), dynamic/nn.hpp:25). */
int b200_permute(b200_ctx* ctx, const void* x, const int64_t in_shape[4], const int32_t perm[4], void* y, void* stream);
/* ttnn::triu(t, diagonal) on the last two dims of [batch, rows, cols] (traced/nn.hpp:160). */
int b200_triu(b200_ctx* ctx, const void* x, void* y, int64_t batch, int64_t rows, int64_t cols, int diagonal, void* stream);

/* ---- embedding (TracedEmbedding, traced/nn.hpp:303-321: ttnn::embedding / ttnn::embedding_bw) ----------------
 * forward: out[i, :] = table[ids[i], :]; backward: d_table (fp32 [vocab, dim], overwritten) += dy rows by id. */
int b200_embedding_forward(b200_ctx* ctx, const uint32_t* ids, int64_t n_ids, const void* table, int64_t vocab, int64_t dim,
                           void* out, void* stream);
int b200_embedding_backward(b200_ctx* ctx, const uint32_t* ids, int64_t n_ids, const void* dy, int64_t vocab, int64_t dim,
                            float* d_table_f32, void* stream);

/* ---- optimisers ------------------------------------------------------------------------------------------------
 * Multi-tensor updates: `count` tensors given as HOST arrays of device pointers and element counts.
 * SGD  p <- p - lr * g (traced/ops.hpp:132-134, dynamic/optim.hpp:21-27, py/optim.py:13-22).
 * Adam with bias correction and eps added after the square root (py/optim.py:49-87); m and v are fp32 (the
 * reference keeps them in bf16 tensors, which loses precision); `step` counts from 1. Parameters and gradients are
 * bf16 or fp32 (one dtype for all tensors of a call). shadow_bf16 (optional table, entries may be NULL): bf16 copies of
 * fp32 master parameters, rewritten in the same pass so the next matmul reads up-to-date bf16 weights. */
int b200_sgd_step(b200_ctx* ctx, int64_t count, void* const* params, const void* const* grads, void* const* shadow_bf16,
                  const int64_t* sizes, int p_dtype, int g_dtype, float lr, void* stream);
int b200_adam_step(b200_ctx* ctx, int64_t count, void* const* params, const void* const* grads, float* const* m,
                   float* const* v, void* const* shadow_bf16, const int64_t* sizes, int p_dtype, int g_dtype, float lr,
                   float beta1, float beta2, float eps, int64_t step, void* stream);
/* The same update with the step number in DEVICE memory, for steps that are recorded into a trace and replayed
 * (TraceContext, autograd/traced/trace.hpp:21-88): the arguments of a recorded kernel are frozen, so a host-side step
 * count would apply the bias correction of the recording step on every replay. d_state16 is a 16-byte device buffer
 * the caller zero-fills once ({int64 step; float 1/(1-beta1^step); float 1/(1-beta2^step)}); with advance != 0 a
 * one-thread kernel increments the step and refreshes the two factors before the update reads them. Several calls of
 * one optimiser step (parameter groups of different dtypes) share one state: advance on the first call only. */
int b200_adam_step_device(b200_ctx* ctx, int64_t count, void* const* params, const void* const* grads, float* const* m,
                          float* const* v, void* const* shadow_bf16, const int64_t* sizes, int p_dtype, int g_dtype, float lr,
                          float beta1, float beta2, float eps, void* d_state16, int advance, void* stream);

/* ---- sharded matmul over the GPUs of one node, one process per GPU ---------------------------------------------
 * (benchmark_tensor_parallel_matmul, bench/metal/matmul_tensor_parallel.cpp:54-123: replicate A, shard B on dim 1,
 *  ttnn::matmul then ttnn::all_gather(c, 1); scripts/matmul_2dev_distributed.py:33-109.)
 * The collective is fused into the GEMM epilogue: finished tiles are stored by TMA directly into peer GPUs' memory.
 * Peer buffers are exchanged as CUDA IPC handles (64 opaque bytes) by the host program.
 * Stores to a peer are complete for that peer only after this rank's stream has finished AND the ranks have
 * synchronised (barrier or any collective issued by the host program). */
int b200_ipc_get_handle(b200_ctx* ctx, void* dptr, void* out_handle64);
int b200_ipc_open_handle(b200_ctx* ctx, const void* handle64, void** out_dptr);
int b200_ipc_close_handle(b200_ctx* ctx, void* dptr);
/* Several GPUs driven by one process (MeshDevice with MeshShape(1, g), bench/metal/matmul_tensor_parallel.cpp:158-164):
 * b200_enable_peer_access lets two contexts' GPUs address each other's memory; b200_peer_copy_2d copies a
 * [rows x width_bytes] block between them on dst_ctx's stream after the work already queued on src_ctx's stream —
 * the unfused form of ttnn::all_gather(t, dim) when the caller issues matmul and gather as two separate ops. */
int b200_enable_peer_access(b200_ctx* a, b200_ctx* b);
int b200_peer_copy_2d(b200_ctx* dst_ctx, void* dst, size_t dst_pitch_bytes, b200_ctx* src_ctx, const void* src,
                      size_t src_pitch_bytes, size_t width_bytes, size_t rows);
/* Puts `waiter`'s stream behind everything queued so far on `producer`'s stream (an event, no host wait): after it,
 * work queued on waiter sees what producer's kernels stored into waiter's memory. Between processes the same ordering
 * is b200_comm_barrier. */
int b200_ctx_wait_ctx(b200_ctx* waiter, b200_ctx* producer);
/* A barrier between one-process-per-GPU ranks that is a kernel on this rank's stream and nothing else: no library
 * call, no host wait, about one NVLink round trip. peer_flags[p] = rank p's flag array (n_ranks 32-bit words, zero at the
 * start, peer-mapped: b200_ipc_*), peer_flags[my_rank] the local one; local_epoch = one 32-bit word of this rank's own
 * memory, zero at the start. Every call adds one to the epoch ON THE DEVICE (a recorded trace advances on every
 * replay), stores it with release semantics into word my_rank of every rank's array and waits, with acquire loads and
 * the bounded-wait rule of every kernel here, until its own array shows that epoch in every word. All ranks must call
 * it the same number of times. What was stored into this rank's memory by a peer's kernels queued before the peer's
 * call is visible to what this rank queues after its own. A wait that runs out raises the status word
 * (b200_synchronize then returns B200_ERR_DEVICE_TIMEOUT): a peer that left is found out, not waited for forever.
 * Ranks emulated on ONE GPU must not use it (kernels that wait for each other need GPUs of their own). */
int b200_peer_barrier(b200_ctx* ctx, void* const* peer_flags, int n_ranks, int my_rank, void* local_epoch, void* stream);
/* N-split (column parallel) + all-gather. desc describes the LOCAL product C[:, my_rank*N : (my_rank+1)*N] =
 * op(A) . op(B_shard) with N = shard width; desc->C is ignored; desc->ldc = leading dimension of the full gathered C
 * (>= N * n_ranks). peer_c[p] = base of the full C on rank p (peer_c[my_rank] = the local one). Every rank ends up
 * with the whole C, like ttnn::all_gather(c_sharded, 1). Needs the tcgen05 alignment rules, batch 1, split_k off. */
int b200_gemm_allgather(b200_ctx* ctx, const b200_gemm_desc* desc, void* const* peer_c, int n_ranks, int my_rank,
                        void* stream);
/* K-split (row parallel) + reduce-scatter, step 1: desc describes the LOCAL partial product over this rank's K range
 * (full M x N). The fp32 partial tiles of row block j (M / n_ranks rows) are stored into slot `my_rank` of rank j's
 * staging buffer peer_slots[j], laid out [n_ranks][M / n_ranks][N] in desc->c_dtype: B200_F32, or B200_BF16 to halve
 * the bytes on the links (each partial sum is then rounded once before the fp32 summation: the HiFi2 trade of
 * verify/verify_fidelity.cpp:50-55 applied to the exchange). M / n_ranks must be a multiple of 128.
 * Step 2, after the ranks have synchronised: b200_reduce_slices sums a rank's n_slices slices ([n_slices][batch][M][N]
 * fp32, M = rows of the block; b200_reduce_slices_typed also takes bf16 slices), applies desc's alpha / bias /
 * activation and writes desc->C (bf16 or fp32). */
int b200_gemm_reduce_scatter_partials(b200_ctx* ctx, const b200_gemm_desc* desc, void* const* peer_slots, int n_ranks,
                                      int my_rank, void* stream);
int b200_reduce_slices(b200_ctx* ctx, const float* slices, int n_slices, const b200_gemm_desc* desc, void* stream);
int b200_reduce_slices_typed(b200_ctx* ctx, const void* slices, int slices_dtype, int n_slices, const b200_gemm_desc* desc,
                             void* stream);
/* The kernel and tile width the two fused calls above use for `desc` (reduce_scatter = 0: b200_gemm_allgather, 1:
 * b200_gemm_reduce_scatter_partials), in the terms of b200_gemm_plan; b200_gemm_plan_describe turns it into text. */
int b200_gemm_dist_plan_query(b200_ctx* ctx, const b200_gemm_desc* desc, int n_ranks, int reduce_scatter,
                              b200_gemm_plan* out_plan);

/* ---- rank-to-rank plumbing of the sharded matmul (the fabric set-up and collective calls of the reference's mesh
 *      programs: tt::tt_fabric::SetFabricConfig + open_mesh_device, bench/metal/matmul_tensor_parallel.cpp:155-166;
 *      ttnn::all_gather, :91-93) ---------------------------------------------------------------------------------
 * One communicator per (process, GPU), over NCCL, which is bound at run time: without libnccl.so.2 these calls fail
 * with B200_ERR_COMM and everything else still works. The 128-byte id is made by one rank (b200_comm_unique_id) and
 * shipped to the others by the host program (a file, a socket, its launcher's store); b200_comm_create is collective.
 *   b200_comm_barrier        stream-ordered: completes on a rank's stream only when every rank's stream has reached it,
 *                            so work queued after it sees all peers' earlier stores; nothing blocks the host
 *   b200_comm_exchange_host  every rank contributes bytes_per_rank host bytes and receives all ranks' blobs in rank
 *                            order (how the CUDA IPC handles of peer buffers travel); blocks until done
 *   b200_comm_allreduce      in place on a device buffer of `count` elements (data-parallel gradient averaging)
 *   b200_comm_allgather      device bytes, rank r's block lands at d_recv + r * bytes_per_rank
 * stream = NULL means the context's stream, as everywhere. */
typedef struct b200_comm b200_comm;
typedef enum b200_comm_op { B200_COMM_SUM = 0, B200_COMM_AVG = 1, B200_COMM_MAX = 2 } b200_comm_op;
int b200_comm_unique_id(void* out_id128);
int b200_comm_create(b200_ctx* ctx, const void* id128, int n_ranks, int rank, b200_comm** out_comm);
int b200_comm_destroy(b200_comm* comm);
int b200_comm_size(const b200_comm* comm, int* out_n_ranks, int* out_rank);
int b200_comm_barrier(b200_comm* comm, void* stream);
int b200_comm_exchange_host(b200_comm* comm, const void* h_send, void* h_recv, size_t bytes_per_rank);
int b200_comm_allreduce(b200_comm* comm, void* d_buf, int64_t count, int dtype, int op, void* stream);
int b200_comm_allgather(b200_comm* comm, const void* d_send, void* d_recv, size_t bytes_per_rank, void* stream);

/* ---- NVLink multicast buffers (NVSwitch replicates one store into every rank's copy) ------------------------------
 * b200_mc_alloc is collective over `comm`: every rank allocates `bytes` of device memory, all are bound to one
 * multicast object, and each rank gets two addresses for it: *out_local_ptr, its own copy (ordinary loads, stores,
 * copies and kernels), and *out_multicast_ptr, which only b200_gemm_allgather_mc may write: a store there lands at the
 * same offset of every rank's copy. Fails with B200_ERR_UNSUPPORTED when a rank's GPU or driver has no multicast
 * (b200_mc_supported tells in advance); callers then use b200_gemm_allgather with unicast peer pointers.
 * b200_mc_free is collective too and must be called by every rank before any of them exits: it drains the device,
 * meets the other ranks, and only then unbinds and releases the memory. A rank that disappears while its memory is
 * still bound can fault its peers' NVLink traffic. */
typedef struct b200_mc b200_mc;
int b200_mc_supported(b200_ctx* ctx, int* out_supported);
int b200_mc_alloc(b200_comm* comm, size_t bytes, b200_mc** out_mc, void** out_local_ptr, void** out_multicast_ptr);
int b200_mc_free(b200_mc* mc);
/* Copies `bytes` from this GPU's memory to a multicast address (multimem.st, 16 bytes per thread): the block arrives
 * at the same offset of every rank's copy — an all-gather of row blocks in which each rank sends its block once.
 * Addresses and size are multiples of 16 bytes. Visible to a peer after this rank's stream and a rank barrier. */
int b200_mc_broadcast(b200_ctx* ctx, void* mc_dst, const void* d_src, size_t bytes, void* stream);
/* b200_gemm_allgather with ONE destination: the multicast address of the full C (from b200_mc_alloc). The epilogue
 * stages each finished box in shared memory and the warp writes it with multimem.st, 16 bytes per lane: one store per
 * box instead of one per rank, so a rank's egress is its own slice once ((g-1)/g * |C| / g bytes per peer link set
 * instead of (g-1) * |C| / g). With use_multimem = 0 the same code path issues ordinary 16-byte stores to `mc_c` (any
 * device pointer): what single-GPU tests run. Same operand rules as b200_gemm_allgather; bf16 or fp32 C. */
int b200_gemm_allgather_mc(b200_ctx* ctx, const b200_gemm_desc* desc, void* mc_c, int n_ranks, int my_rank, int use_multimem,
                           void* stream);

/* ---- split-K matmul without device allocation (no counterpart in the reference: TTNN owns its device
 *      memory, so the question never arises there) ----------------------------------------------------
 * Same arguments and result as b200_gemm on the tcgen05 path, for hosts that must not allocate device
 * memory at call time: executors that gave all of HBM to their own arena, loops with a latency bound
 * (cudaMalloc / cudaFree synchronise the device), processes whose device memory is capped below what a growing
 * scratch block would need. The fp32 partial
 * sums of the K slices live in a fixed 32 MiB array inside the library image (held by every GPU that
 * loads the library until the process exits) instead of context scratch; the call performs no
 * cudaMalloc, cudaFree or other allocating routine and needs no b200_ctx.
 *   device    ordinal of the GPU that owns A, B, C and `stream`
 *   stream    required (non-NULL) cudaStream_t
 *   split_k   0 = same choice as b200_gemm, lowered until the partial sums fit; n > 1 = exactly n slices
 * Fails with B200_ERR_INVALID_ARG when k_slices * batch * M * N * 4 bytes exceed 32 MiB, or when the
 * operands do not meet the TMA alignment rules (there is no SIMT path here).
 * All calls on a device share the array: calls whose kernels may overlap on the GPU (different streams
 * or threads) race on it — keep them on one stream. The first call on each device looks up the array's
 * device address, and the first call that uses a kernel variant (tile width x operand layouts) on a device
 * configures that kernel: make one call of every shape class you will use before any stream capture starts.
 * A bounded wait that runs out inside these kernels is recorded in a status word inside the library image;
 * b200_synchronize does not see it, b200_static_scratch_status does: it waits for `stream`, returns
 * B200_ERR_DEVICE_TIMEOUT (and *out_status != 0) when a wait ran out since the last call, and clears the word.
 * It allocates nothing either. */
int b200_gemm_static_scratch(int device, const b200_gemm_desc* desc, void* stream);
int b200_static_scratch_status(int device, void* stream, int* out_status);

#ifdef __cplusplus
} /* extern "C" */
#endif
#endif /* B200_TTPERF_H */
