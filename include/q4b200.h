/*
 * q4b200 — C ABI of the B200 (sm_100a) GPTQ int4 dequant-matmul kernels.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream handle; nothing here
 * knows about torch.  The caller owns all memory and must have made the device that owns the
 * pointers current on the calling thread.  Every function that launches work returns 0 on
 * success or a negative Q4_E_* code; q4_last_error_string() then gives a human-readable
 * reason (thread-local).  Launches are asynchronous on `stream`.
 *
 * Threads: q4_gemv, q4_gemm_*, q4_recons_* and q4_layer_* may be called from several threads at
 * once as long as calls that share a workspace are ordered on one stream.  The q4_*_set_variant
 * and q4_*_set_trace switches are process-wide and unsynchronised: set them while no other thread
 * is inside the library (they exist for tests and measurements).
 *
 * Tensor conventions (GPTQ v2, as stored by Autograd4bitQuantLinear, autograd_4bit.py:176-189):
 *   qweight int32 [K/8, N]   nibble j of word (r, n) is level q of row k = 8r + j, column n
 *   qzeros  int32 [G, N/8]   nibble n%8 of word (g, n/8) is the stored zero point z (kernel adds 1)
 *   scales  T     [G, N]
 *   g_idx   int32 [K]        group of row k
 *   W[k, n] = scales[g,n]*q - scales[g,n]*(z+1),  g = g_idx[k]
 * All matrices are dense row-major.
 */
#ifndef Q4B200_H_
#define Q4B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define Q4_VERSION 100

/* element types of scales / outputs */
#define Q4_F16 0
#define Q4_F32 1

/* status codes */
#define Q4_OK            0
#define Q4_E_BADARG     -1   /* null pointer, non-positive size, unknown enum */
#define Q4_E_SHAPE      -2   /* size not supported by the kernel (divisibility) */
#define Q4_E_ALIGN      -3   /* pointer not 16-byte aligned */
#define Q4_E_WORKSPACE  -4   /* workspace missing or too small */
#define Q4_E_CUDA       -5   /* a CUDA runtime / driver call failed */
#define Q4_E_DEVICE     -6   /* device is not sm_100 */

/* q4_gemv flags */
#define Q4_GEMV_ACCUMULATE 1u  /* y += x*W instead of y = x*W (the reference kernels add into `mul`) */
#define Q4_GEMV_ACT_ORDER  2u  /* take the group of every row from g_idx (else k / groupsize)      */
#define Q4_GEMV_V1         4u  /* v1 layer: scales fp16 [N]; `qzeros` points at fp16 zeros [N];
                                  W = scales[n]*q - zeros[n]; G, groupsize and g_idx are ignored;
                                  K must be a multiple of 128 (Q4_E_SHAPE otherwise), as for the
                                  reference's v1 kernel */

typedef void* q4_stream_t;     /* a cudaStream_t */

int q4_version(void);
const char* q4_last_error_string(void);

/* Reconstruct the dense weight  W [K, N]  from a 4-bit v2 layer.
 * Replaces quant_cuda.vecquant4recons_v2 (quant_cuda.cpp:137-148,
 * quant_cuda_kernel.cu:1127-1183).  `dtype` is the type of `scales` and `out` (Q4_F16: three
 * fp16 roundings, bit-exact with the reference; Q4_F32: one fused multiply-subtract).
 * Needs N % 8 == 0, K % 8 == 0. */
int q4_recons_v2(const int32_t* qweight, void* out, const void* scales, const int32_t* qzeros,
                 const int32_t* g_idx, int K, int N, int G, int dtype, q4_stream_t stream);

/* v1 layer: W[k,n] = scales[n]*q - zeros[n], per-column float scale and zero.
 * Replaces quant_cuda.vecquant4recons_v1 (quant_cuda.cpp:125-135, quant_cuda_kernel.cu:1076-1125). */
int q4_recons_v1(const int32_t* qweight, void* out, const void* scales, const void* zeros,
                 int K, int N, int dtype, q4_stream_t stream);

/* 2-bit v2 layer: qweight int32 [K/16, N], qzeros int32 [G, N/16], zero point = field + 1.
 * Replaces quant_cuda.vecquant2recons_v2 (quant_cuda.cpp:150-161, quant_cuda_kernel.cu:1185-1241).
 * Needs N % 16 == 0, K % 16 == 0. */
int q2_recons_v2(const int32_t* qweight, void* out, const void* scales, const int32_t* qzeros,
                 const int32_t* g_idx, int K, int N, int G, int dtype, q4_stream_t stream);

/* Decode product  y [M, N] (+)= x [M, K] * W,  1 <= M <= 16, without materialising W.
 * Replaces quant_cuda.vecquant4matmul / vecquant4matmul_faster / vecquant4matmul_old_faster /
 * vecquant4matmul_v1_faster / vecquant4matmul_g (quant_cuda.cpp:35-48,95-108,110-123,163-174,
 * 189-202; kernels quant_cuda_kernel.cu:475-536,910-975,978-1041,1243-1302,1488-1567).
 *   x fp16 [M, K]; scales fp16 [G, N]; y of type y_dtype (Q4_F16 or Q4_F32); bias fp16 [N] or NULL.
 *   Without Q4_GEMV_ACT_ORDER the group of row k is k / groupsize and g_idx may be NULL.
 *   Needs K % 32 == 0, N % 32 == 0, groupsize % 32 == 0.
 * `workspace` is caller-provided device scratch of at least q4_gemv_workspace_bytes(M, K, N)
 * bytes that must be zero when first used and is left zero-filled where it has to be (its first
 * 128 KiB: arrival counters, the status word and the slots through which CTAs exchange the sums of a
 * column tile they share); calls that share a workspace must be ordered on one stream.  Summation
 * order is fixed, so results are reproducible run to run.
 * One-row products (M = 1, groups of 128, K a multiple of 256) run on int8 tensor-core MMAs: x is
 * converted to 16-bit block fixed point per group of 128 rows (x_int = rn(x * 2^(14-E)) with 2^E <=
 * max |x| of the group < 2^(E+1)), products and sums are exact integers, and the only rounding
 * is that of x: none for elements within a factor 16 of their group's largest, at most 2^(E-15)
 * absolute for smaller ones (measured 2e-5 relative Frobenius error against the exact product,
 * under the 1e-4 of the fp16-MMA kernels). */
size_t q4_gemv_workspace_bytes(int M, int K, int N);
int q4_gemv(const void* x, const int32_t* qweight, void* y, const void* scales,
            const int32_t* qzeros, const int32_t* g_idx, const void* bias,
            int M, int K, int N, int G, int groupsize, int y_dtype, unsigned flags,
            void* workspace, size_t workspace_bytes, q4_stream_t stream);

/* A layer handle for the per-token call (no counterpart in the reference): a host that calls
 * q4_gemv through a foreign-function interface once per layer and token pays for marshalling its 17
 * arguments every time.  q4_layer_create records the layer's tensors and geometry once (v2 layout,
 * sequential groups, no bias); q4_layer_gemv is q4_gemv(x, <layer>, y, M, ..., Q4_F16, flags 0, ...)
 * with the arguments that change from call to call.  The handle owns no device memory and keeps no
 * reference to the tensors: destroy it before they are freed or moved.  Handles are immutable and
 * may be used from any thread. */
typedef struct q4_layer q4_layer_t;
int q4_layer_create(q4_layer_t** out, const int32_t* qweight, const void* scales, const int32_t* qzeros,
                    int K, int N, int G, int groupsize);
int q4_layer_gemv(const q4_layer_t* layer, const void* x, void* y, int M,
                  void* workspace, size_t workspace_bytes, q4_stream_t stream);
void q4_layer_destroy(q4_layer_t* layer);
/* Tells `layer` which layer the caller will run after it (NULL: none).  A decode step walks the same
 * layers in the same order token after token; with the successor known, the one-row kernel of `layer`
 * asks for the successor's packed weights to be brought into L2 while it computes, so that HBM streams
 * the next layer during this one instead of idling through its tail and the next launch's start.
 * A hint only: results never depend on it, a wrong successor costs bandwidth, not correctness.  The
 * successor's qweight address is copied into `layer`: clear the link (set it to NULL) before that
 * memory is freed.  No counterpart in the reference. */
int q4_layer_set_next(q4_layer_t* layer, const q4_layer_t* next);

/* The same product as q4_gemv for callers that cannot allocate device memory (no counterpart in the
 * reference; added for hosts such as a serving process that handed all of HBM to its own pools, a
 * plugin that may not call the allocator of the process it lives in, or a latency path on which the
 * device-synchronising cudaMalloc is not acceptable).  The scratch is a 2.125 MiB device array built
 * into the library (q4_gemv_static_max_bytes()), present on every GPU that loads the library until
 * the process exits; the call allocates nothing and frees nothing.  That size serves every shape
 * with sequential groups; shapes whose q4_gemv_workspace_bytes() exceeds it (16-row products over
 * roughly 17k-19k columns) are refused with Q4_E_WORKSPACE.
 * The first call on each device looks up the device address of the array; make that first call
 * outside any stream capture.  All calls on a device share the one array, so calls that can overlap
 * on the GPU (different streams without ordering) race; keep them on one stream or order them with
 * events.  The head of the array is cleared on the stream before every launch. */
size_t q4_gemv_static_max_bytes(void);
int q4_gemv_static(const void* x, const int32_t* qweight, void* y, const void* scales,
                   const int32_t* qzeros, const int32_t* g_idx, const void* bias,
                   int M, int K, int N, int G, int groupsize, int y_dtype, unsigned flags,
                   q4_stream_t stream);

/* Large-M products straight from the packed layer (W is never written to global memory):
 *   q4_gemm_fwd:  y  [M, N] = x  [M, K] * W (+ bias)      q4_gemm_bwd:  dx [M, K] = dy [M, N] * W^T
 * Together they replace the reference's reconstruct + torch.matmul composition,
 * matmul_utils_4bit._matmul4bit_v2_recons (matmul_utils_4bit.py:114-127), i.e. the forward and
 * backward of AutogradMatmul4bitCuda (autograd_4bit.py:32-54).  x, dy, y, dx, scales, bias fp16;
 * fp32 accumulation in tensor memory; the dequantised operand is bit-identical to q4_recons_v2.
 * The group of every row is read from g_idx (act-order safe).  Needs K % 128 == 0, N % 128 == 0;
 * any M >= 1.  The forward keeps per-group scale tables for 128 columns in shared memory and
 * returns Q4_E_SHAPE when G is too large for that (about 250 groups).
 * LoRA term, fused as one more pipeline stage of the same kernel (lora_r = 0 switches it off):
 *   forward   y  += U * lora_b^T   U      fp16 [M, 64] = (alpha/r) * x  * lora_A^T, columns >= r zero; lora_b fp16 [N, r]
 *   backward  dx += V * lora_a     lora_v fp16 [M, 64] = (alpha/r) * dy * lora_B,   columns >= r zero; lora_a fp16 [r, K]
 * which is the `lora_B(lora_A(x)) * scaling` of Linear4bitLt.forward (models.py:61-66) and its
 * gradient with respect to x.  1 <= lora_r <= 64. */
int q4_gemm_fwd(const void* x, const int32_t* qweight, void* y, const void* scales, const int32_t* qzeros,
                const int32_t* g_idx, const void* bias, const void* lora_u, const void* lora_b, int lora_r,
                int M, int K, int N, int G, void* workspace, size_t workspace_bytes, q4_stream_t stream);
int q4_gemm_bwd(const void* dy, const int32_t* qweight, void* dx, const void* scales, const int32_t* qzeros,
                const int32_t* g_idx, const void* lora_v, const void* lora_a, int lora_r,
                int M, int K, int N, int G, void* workspace, size_t workspace_bytes, q4_stream_t stream);

/* The fused [gate | up] projection of a LLaMA MLP with its SwiGLU product in the GEMM epilogue: qweight, scales,
 * qzeros describe a [K, N = 2 I] layer whose first I columns are gate_proj and whose last I are up_proj (as
 * make_fused_mlp concatenates them, model_attn_mlp_patch.py:165-247 of the reference, which then computes
 * act_fn(gate) * up on the [M, 2 I] product, :229-232); out [M, I] fp16 = half(silu(half(x W_gate + b))) *
 * half(x W_up + b), the roundings of q4_gemm_fwd followed by q4_swiglu_fwd without the [M, 2 I] tensor ever
 * reaching memory.  N % 256 == 0; bias [N] or NULL; workspace as for q4_gemm_fwd; `zero_terms` (the [G, N] table of
 * q4_zero_term_table, or NULL) and `sequential_groupsize` as for q4_gemm_fwd_residual. */
int q4_gemm_fwd_swiglu(const void* x, const int32_t* qweight, void* out, const void* scales, const int32_t* qzeros,
                       const void* zero_terms, const int32_t* g_idx, const void* bias, int M, int K, int N, int G,
                       int sequential_groupsize, void* workspace, size_t workspace_bytes, q4_stream_t stream);

/* The backward with the layer's zero terms kept by the caller: q4_zero_term_table fills out [G, N] fp16 with
 * rn(scale * (zero + 1)) of every group and column (what q4_gemm_bwd otherwise derives into its workspace with
 * a small kernel ahead of every call - the table depends on the frozen layer only), q4_gemm_bwd_table is
 * q4_gemm_bwd reading that table.  A training step calls the backward of every layer once per step, so a host
 * that keeps the tables (2 G N bytes per layer, 1.6 % of the packed weights) saves that kernel per call.  No
 * reference counterpart. */
int q4_zero_term_table(const void* scales, const int32_t* qzeros, void* out, int G, int N, q4_stream_t stream);
int q4_gemm_bwd_table(const void* dy, const int32_t* qweight, void* dx, const void* scales, const int32_t* qzeros,
                      const void* zero_terms, const int32_t* g_idx, const void* lora_v, const void* lora_a, int lora_r,
                      int M, int K, int N, int G, void* workspace, size_t workspace_bytes, q4_stream_t stream);
/* The forward with the same table: scales and zero terms are then read from global memory (L2) per dequant task,
 * as the backward reads them, instead of from shared-memory tables of all groups x the CTA's 128 columns, and the
 * shared memory the tables would take (512 bytes per group: 43 KiB at K = 11008) goes to pipeline stages.  Worth
 * it on layers with many groups; same arguments and results as q4_gemm_fwd otherwise. */
int q4_gemm_fwd_table(const void* x, const int32_t* qweight, void* y, const void* scales, const int32_t* qzeros,
                      const void* zero_terms, const int32_t* g_idx, const void* bias, const void* lora_u, const void* lora_b,
                      int lora_r, int M, int K, int N, int G, void* workspace, size_t workspace_bytes, q4_stream_t stream);
/* The forward with the skip path of a decoder layer in its epilogue: y = half(half(x W + bias) + residual),
 * residual fp16 [M, N] (the two roundings of the product followed by the fp16 add that LlamaDecoderLayer.forward
 * runs after o_proj and down_proj).  `zero_terms` as for q4_gemm_fwd_table, or NULL; `residual` may be NULL.
 * `sequential_groupsize` (with a table only; 0 = no promise): the caller's word that g_idx[k] == k / groupsize for a
 * groupsize that is a power of two - the kernel then does not read g_idx at all, fetches a dequant task's scales
 * and zero terms one task ahead with its packed words and builds no shared-memory tables (a wrong promise gives
 * wrong products, nothing worse). */
int q4_gemm_fwd_residual(const void* x, const int32_t* qweight, void* y, const void* scales, const int32_t* qzeros,
                         const void* zero_terms, const int32_t* g_idx, const void* bias, const void* residual,
                         const void* lora_u, const void* lora_b, int lora_r, int M, int K, int N, int G,
                         int sequential_groupsize, void* workspace, size_t workspace_bytes, q4_stream_t stream);
/* Optional scratch for the two calls above (no reference counterpart: the reference's scratch is
 * the dense fp16 copy of W it reconstructs).  `workspace` may be NULL; with at least
 * q4_gemm_workspace_bytes(K, N, G) bytes of device memory, 16-byte aligned, whose first 64 KiB are
 * zero before the first call (the kernels leave them zero), the CTA-pair kernel
 *   - may deal all output tiles x contraction stages to the SM pairs as one sequence of equal runs
 *     instead of whole tiles, when whole tiles would leave pairs idle (fp32 partial sums of a tile
 *     that two or more pairs share meet in the workspace and are added in a fixed order: results do
 *     not depend on timing), and
 *   - in the backward reads rn(s*(z+1)) from a [G, N] table a small kernel fills first.
 * One workspace serves calls that are ordered on one stream; calls that may overlap need one each. */
size_t q4_gemm_workspace_bytes(int K, int N, int G);

/* The element-wise work of a decoder layer around the quantised linears, one kernel each way (fp16 in and
 * out, fp32 inside).  The reference leaves these to the stock modules (a handful of framework kernels each:
 * its finetune step runs transformers' LlamaRMSNorm, LlamaMLP and apply_rotary_pos_emb, finetune.py:150-175
 * through gradient_checkpointing.py:19-65); there is no counterpart in its extension.
 *   q4_rmsnorm_fwd   y = weight * half(x * rsqrt(mean(x^2) + eps)) per row of H (H % 8 == 0, H <= 8192);
 *                    rstd [rows] fp32 receives the reciprocal root (may be NULL)
 *   q4_rmsnorm_bwd   dx for a frozen weight: rstd * (g - xh * mean(g * xh)), g = dy * weight, xh = x * rstd
 *   q4_swiglu_fwd    out [rows, I] = half(silu(gate)) * up; gate and up are rows of `pitch` halves (two
 *                    tensors, or the halves of one fused gate_up output)
 *   q4_swiglu_bwd    dgate, dup (rows of `dpitch` halves) from dout, gate, up
 *   q4_rope          rotary embedding of in [tokens, heads, D] (token pitch `in_pitch` halves) with cos / sin
 *                    [table_rows, D] (row = token % table_rows: the tables of one sequence serve a whole batch)
 *                    into out [tokens, heads, D]; `backward` != 0 applies the transpose */
int q4_rmsnorm_fwd(const void* x, const void* weight, void* y, float* rstd, int rows, int H, float eps, q4_stream_t stream);
int q4_rmsnorm_bwd(const void* dy, const void* x, const void* weight, const float* rstd, void* dx, int rows, int H,
                   q4_stream_t stream);
int q4_swiglu_fwd(const void* gate, const void* up, void* out, int rows, int I, int pitch, q4_stream_t stream);
int q4_swiglu_bwd(const void* dout, const void* gate, const void* up, void* dgate, void* dup, int rows, int I, int pitch,
                  int dpitch, q4_stream_t stream);
int q4_rope(const void* in, const void* cos, const void* sin, void* out, int tokens, int heads, int D, int in_pitch,
            int table_rows, int backward, q4_stream_t stream);

/* The rank-r products of a LoRA adapter around q4_gemm_fwd / q4_gemm_bwd (Linear4bitLt.forward,
 * models.py:58-66, runs them as two nn.Linear calls and leaves the gradients to autograd; no single
 * reference function corresponds).
 *   q4_lora_project   out [M, 64] fp16 = scale * x [M, C] * w^T with w fp16 [r, C] (1 <= r <= 64, C % 32 == 0),
 *                     columns r..63 written as zeros: the `lora_u` / `lora_v` operand of the GEMM entry points
 *                     (forward: x and lora_A; backward: dy and lora_B^T)
 *   q4_lora_grads     d_a [r, K] fp32 = v[:, :r]^T x and d_b [N, r] fp32 = dy^T u[:, :r] in one launch
 *                     (v, u fp16 [M, 64] as produced above; x fp16 [M, K]; dy fp16 [M, N]; K, N % 32 == 0);
 *                     either output may be NULL, its operands are then not read */
int q4_lora_project(const void* x, const void* w, void* out, int M, int C, int r, float scale, q4_stream_t stream);
int q4_lora_grads(const void* v, const void* x, float* d_a, int K, const void* dy, const void* u, float* d_b, int N,
                  int M, int r, q4_stream_t stream);

/* One optimiser step over flat fp32 buffers of n elements (every trainable LoRA factor a view of `param`,
 * every gradient a view of `grad`): torch.optim.AdamW's update with torch.amp.GradScaler's loss-scale
 * handling, which is what the reference's trainer runs (finetune.py:150-170: optim="adamw_torch", fp16=True).
 * `state` is four device floats: steps taken, loss scale, steps since the scale changed, non-finite flag
 * (zero before the first call except for the scale).  Three launches on `stream`: (1) state[3] = 1 if any
 * gradient is non-finite; (2) unless it is, param/exp_avg/exp_avg_sq advance by one AdamW step on
 * grad / (state[1] * grad_div)  (grad_div: the number of ranks whose gradients were summed into `grad`);
 * (3) a skipped step multiplies the scale by `backoff`, `growth_interval` clean steps in a row multiply it by
 * `growth` (growth_interval 0: the scale is static), the step count advances and the flag is cleared.
 * `half_shadow` (n halves, or NULL) receives the updated parameters rounded to fp16, which is what the LoRA kernels
 * of the next step read (a skipped step leaves it as it was).  Nothing returns to the host, so the call can be
 * captured in a CUDA graph. */
int q4_adamw_flat(float* param, const float* grad, float* exp_avg, float* exp_avg_sq, size_t n, float lr, float beta1,
                  float beta2, float eps, float weight_decay, float grad_div, float* state, float growth, float backoff,
                  int growth_interval, void* half_shadow, q4_stream_t stream);

/* Copies the device status word to *out (synchronises the device): 0, or 0xDEAD0001 if a bounded
 * wait inside a q4_gemm_* kernel expired (its output is then invalid). */
int q4_device_status(unsigned* out);
/* The same for the decode kernels, which keep their status word with the workspace they were given
 * (its head's last word) instead of in a device global: synchronises the device and copies the word
 * of `workspace` to *out - 0, or 0xDEAD0001 if a bounded wait inside a q4_gemv kernel that used
 * this workspace expired.  The output of that call is invalid and arrival counters in the head may
 * be left non-zero: clear the first 128 KiB of the workspace (which also clears the word) before it
 * is used again (128 KiB from the library version that exchanges shared column tiles through it).
 * No counterpart in the reference, whose kernels wait on nothing. */
int q4_gemv_status(const void* workspace, size_t workspace_bytes, unsigned* out);
/* The status word of the built-in scratch of q4_gemv_static on the current device; a non-zero word
 * is cleared once it has been reported (q4_gemv_static itself re-zeroes the counters before every
 * launch but leaves the word for this call to find). */
int q4_gemv_static_status(unsigned* out);

/* Profiling aid: when `device_buffer` is non-NULL, every CTA of the sequential-group decode kernel
 * writes SM cycle counters at fixed points of its life into 64 uint64 slots (buffer of at least
 * 64 * 8 * number-of-SMs bytes).  NULL switches the trace off (the default). */
int q4_gemv_set_trace(void* device_buffer);
/* Same for the fused GEMM kernels: 256 uint64 slots per CTA (buffer of 256 * 8 * number-of-CTAs bytes). */
int q4_gemm_set_trace(void* device_buffer);
/* Which fused GEMM kernel q4_gemm_fwd / q4_gemm_bwd launch (process-wide; no reference counterpart):
 * 0 = choose per shape (the default: with the number of output columns a multiple of 256, the CTA-pair kernel
 * with 256- or 512-row tiles, whichever its estimate favours, or - forward only, when the caller keeps the
 * zero-term table and promises sequential groups of 64 rows or more - the kernel that holds the dequantised
 * weights in tensor memory, where 256-row tiles would be chosen, where its tiles fit one round, and up to 1024
 * rows; the single-CTA kernel otherwise), 1 = always the single-CTA kernel, 2 / 3 = always the CTA-pair kernel
 * with 256- / 512-row tiles, 4 = always the weights-in-tensor-memory kernel (calls a forced kernel cannot serve
 * fail with Q4_E_SHAPE), 5 = as 0 without the weights-in-tensor-memory kernel.  For tests and measurements. */
int q4_gemm_set_variant(int variant);
/* Forms of the sequential-group decode kernels, for tests and measurements (process-wide; no
 * reference counterpart).  `variant` is a sum of:
 *   bits 0-1  products of 2..8 rows: how the kernel gets x - 0 = choose per shape (the default: every CTA
 *             re-lays the whole of x out once when it has more than one column tile's worth of units and x
 *             fits its shared memory; else every 4 KiB unit brings its own slice), 1 = always per unit,
 *             2 = per CTA wherever it fits
 *   4         deal an even share of all units to every CTA even where whole column tiles per CTA would
 *             end sooner (column tiles that straddle CTAs then meet in the workspace)
 *   8         one-row products: the two-CTAs-per-SM form of the kernel (fewer warps per CTA, so that the next
 *             decode launch of the stream is resident beside this one) instead of one CTA per SM
 *   16        one-row products on the kernel that serves 2..8 rows (fp16 MMA, x re-laid per unit) instead
 *             of the warp-specialised int8-MMA kernel
 *   64        one-row products: no L2 prefetch of the CTA's share of the layer (nor of the next layer)
 * Values outside these combinations are refused with Q4_E_BADARG. */
int q4_gemv_set_variant(int variant);

#ifdef __cplusplus
}
#endif
#endif /* Q4B200_H_ */
