/* arke_b200 — C ABI of the B200 (sm_100a) kernels behind Arke's backend / runner interfaces.
 *
 * Conventions for every entry point
 *   - plain device pointers and sizes; the caller owns every buffer (inputs, outputs, workspaces);
 *   - nothing here allocates, frees or synchronises: work is enqueued on `stream` (a cudaStream_t
 *     passed as void*, NULL = legacy default stream) of the calling thread's current device;
 *   - returns ARKE_OK (0) or a negative ARKE_ERR_* code; arke_b200_last_error() returns the
 *     message of the calling thread's last failure;
 *   - row strides (`ld*`) are in elements;
 *   - kernels with device-side waits bound every wait; if one expires the kernel records a
 *     non-zero code in a per-device status word that arke_b200_kernel_status() reads back.
 *
 * The reference (blueyi/arke) is pure Python and has no FFI of its own; each entry point below
 * replaces the kernel that Arke's code-generating backends would have produced for the op, and
 * is reached from Python through ArkeBackend.run (arke/backend/protocol.py:94-137) /
 * BaselineRunner.get_fn (benchmarks/baselines/base.py:18-114).
 */
#ifndef ARKE_B200_H
#define ARKE_B200_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define ARKE_B200_API __attribute__((visibility("default")))
#else
#define ARKE_B200_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* element types */
enum { ARKE_BF16 = 0, ARKE_F16 = 1, ARKE_F32 = 2, ARKE_I8 = 3, ARKE_E4M3 = 4, ARKE_I32 = 5, ARKE_I64 = 6 };
/* quantised output kinds of quantize_per_token */
enum { ARKE_QUANT_INT8 = 0, ARKE_QUANT_E4M3 = 1 };
/* layout of the GEMM weight operand */
enum { ARKE_W_KN = 0 /* W[K,N], N contiguous */, ARKE_W_NK = 1 /* W[N,K], K contiguous */ };

/* status codes */
enum {
  ARKE_OK = 0,
  ARKE_ERR_ARG = -1,       /* null pointer / bad enum value            */
  ARKE_ERR_DTYPE = -2,     /* unsupported element type                 */
  ARKE_ERR_SHAPE = -3,     /* unsupported shape or stride              */
  ARKE_ERR_ALIGN = -4,     /* pointer or stride not aligned as needed  */
  ARKE_ERR_CUDA = -5,      /* a CUDA runtime / driver call failed      */
  ARKE_ERR_WORKSPACE = -6, /* workspace too small                      */
  ARKE_ERR_DEVICE = -7,    /* device is not sm_100                     */
  ARKE_ERR_KERNEL = -8     /* a kernel reported an expired wait        */
};

/* Library version string, e.g. "arke_b200 0.1 (sm_100a)". */
ARKE_B200_API const char* arke_b200_version(void);
/* Message of the calling thread's most recent failing call ("" if none). */
ARKE_B200_API const char* arke_b200_last_error(void);
/* Reads and clears the current device's kernel status word (synchronises `stream`).
 * 0 = nothing to report; otherwise the first code a kernel recorded: 1..5 = a bounded wait expired
 * (TMA producer, MMA issuer, epilogue, softmax, correction), 6 = arke_b200_fused_linear_ce over
 * the whole vocabulary met a label outside [0, V) (that row's loss is NaN), 7 = a library built
 * with -DARKE_B200_CHECKED computed a global index outside its extent (the access was skipped). */
ARKE_B200_API int arke_b200_kernel_status(void* stream);

/* Failure-path self-test: launches one CTA that waits on a barrier nothing completes, with a
 * limit of `limit_cycles` SM cycles (<= 2e9); the wait expires, the kernel records a non-zero code
 * in the status word exactly like the production kernels and returns normally (no trap, the
 * context stays usable).  arke_b200_kernel_status() then returns that code.  No reference
 * counterpart. */
ARKE_B200_API int arke_b200_selftest_wait_timeout(int64_t limit_cycles, void* stream);

/* Checked build (nvcc -DARKE_B200_CHECKED, `python -m arke_b200.build --flag=-DARKE_B200_CHECKED
 * --out ...`): every kernel re-derives, right before a global access, that the element index it
 * computed lies inside the tensor and otherwise records status code 7 and skips the access.  It
 * stands in for an address sanitizer where none can run.  This self-test evaluates the check on an
 * index one past an extent without touching memory: after it arke_b200_kernel_status() returns
 * 7.  ARKE_ERR_ARG in a default build.  No reference counterpart. */
ARKE_B200_API int arke_b200_selftest_bounds_check(void* stream);

/* Per-thread tuning options for the calls this thread makes afterwards (value 0 restores the
 * library's own choice).  They are what the backend maps the agent loop's strategy decisions to
 * (`lower(graph, strategy=...)`, arke/backend/llvm_backend.py:238-262, arke/ir/strategy.py:368-396):
 *   "gemm_tile_m"   128 = one-CTA 128 x 256 tiles, 256 = CTA-pair 256 x 256 tiles (cta_group::2);
 *                   applies to quant_gemm, matmul and fused_linear_ce
 *   "gemm_band_mb"  MB of the A operand kept L2-resident per band of output tiles (default 32)
 *   "gemm_static_sched" 1 = the CTA pairs of a GEMM take their tiles round robin; 0 = default:
 *                   from a device counter, so that the tiles in flight are always neighbours in
 *                   the tile order and pairs that share an operand tile through the L2 use it
 *                   at the same time
 *   "gemm_no_pdl"   1 = launch the GEMM kernels without programmatic stream serialization (their
 *                   set-up then no longer overlaps the tail of the previous kernel); 0 = default
 *   "gemm_no_split" 1 = the last, partly filled wave of a CTA-pair GEMM keeps whole 256 x 256
 *                   tiles; 0 = default: those tiles are cut into 2 or 4 narrower units along N
 *                   so that they spread over more CTA pairs
 * Results do not depend on them.  get_option returns -1 for an unknown name. */
ARKE_B200_API int arke_b200_set_option(const char* name, int64_t value);
ARKE_B200_API int64_t arke_b200_get_option(const char* name);

/* Per-token (per-row) symmetric quantisation.
 * Replaces the kernels generated for `quantize_per_token`
 * (arke/ir/ops/reference_impls.py:215-218; arke/backend/triton_templates/quantize.py.j2:16-101).
 *   x [M,N] bf16/f16/f32, row stride ldx.  q [M,N] int8 or e4m3 bytes, row stride ldq.
 *   formula 0: scale = amax/127 (int8) or amax/448 (e4m3); q = rint(x/scale) with a correctly
 *              rounded fp32 quotient, half-to-even, clamp [-128,127]; all-zero rows give q = 0.
 *   formula 1: int8 only, the benchmark driver's golden (benchmarks/bench_l1.py:443-448):
 *              q = round(h(h(x/amax)*127)), h = round to the input dtype; scale out = amax. */
ARKE_B200_API int arke_b200_quantize_per_token(const void* x, int x_dtype, int64_t M, int64_t N, int64_t ldx,
                                 void* q, int64_t ldq, float* scale, int out_kind, int formula,
                                 void* stream);

/* Per-channel dequantisation  Y[i,j] = (X[i,j] - zero_point[j]) * scale[j]  in fp32
 * (`dequantize_per_channel`, arke/ir/ops/reference_impls.py:220-224; schema catalog.py:468-479).
 *   x [M,N] int8; scale [N] fp32; zero_point [N] fp32 or NULL (= 0); y [M,N] f32 / bf16 / f16.
 * (Inside the W8A8 path this scaling is fused into the GEMM epilogue; this entry point serves the
 * stand-alone catalog op.) */
ARKE_B200_API int arke_b200_dequantize_per_channel(const void* x, int64_t M, int64_t N, int64_t ldx, const float* scale,
                                     const float* zero_point, void* y, int y_dtype, int64_t ldy,
                                     void* stream);

/* RMSNorm with optional residual add and optional fused per-token quantisation of the result:
 *   h = x (+ residual);  y = T(h / sqrt(mean(h^2) + eps) * w)
 * (`rmsnorm`, arke/ir/ops/reference_impls.py:85-90; `rmsnorm_residual`, the function after
 * ref_gelu_and_mul in the same file; schemas arke/ir/ops/catalog.py:229-239,414-424).
 *   x, residual (may be NULL) [M,N], w [N]: one dtype (bf16/f16/f32).  y [M,N] same dtype or NULL.
 *   q [M,N] int8 / e4m3 bytes + scale [M] (out_kind as in quantize_per_token) or NULL: the
 *   quantisation of the rounded y, exactly what quantize_per_token would produce from it. */
ARKE_B200_API int arke_b200_rmsnorm(const void* x, const void* residual, const void* w, int dtype, int64_t M,
                      int64_t N, int64_t ldx, int64_t ldr, float eps, void* y, int64_t ldy, void* q,
                      int64_t ldq, float* scale, int out_kind, void* stream);

/* Rotary position embedding, rotate-half form (`rope`, arke/ir/ops/reference_impls.py:197-206;
 * schema arke/ir/ops/catalog.py:425-435):
 *   y[..., :D/2] = x1*cos - x2*sin,   y[..., D/2:] = x2*cos + x1*sin
 *   x, y contiguous [B,H,S,D]; cos, sin contiguous [S,D/2]; one dtype for all (bf16 / f16 / f32).
 * Every product and sum is rounded to that dtype, like the interpreter's eager evaluation, so the
 * result is bit-identical to it.  D must be even. */
ARKE_B200_API int arke_b200_rope(const void* x, const void* cos, const void* sin, void* y, int dtype,
                   int64_t B, int64_t H, int64_t S, int64_t D, void* stream);

/* The step between a packed QKV projection and attention in one pass: qkv [B*S, ld] holds, per
 * token, Hq query heads, then Hkv key heads, then Hkv value heads of D values each; Q and K heads
 * get `rope` at position s, V is copied, and all three are written in the [B,H,S,D] layout that
 * `grouped_query_attention` reads (arke/ir/ops/reference_impls.py:236-244).  This is the fused
 * form of the QKV-projection -> rope -> attention slot the reference's fusion harness reserves
 * (benchmarks/bench_l2.py:1135-1191 runs it unfused and without rope).
 *   q [B,Hq,S,D], k, v [B,Hkv,S,D] contiguous; cos, sin [S,D/2]; one dtype for all. */
ARKE_B200_API int arke_b200_qkv_rope_split(const void* qkv, int64_t ld, const void* cos, const void* sin,
                             void* q, void* k, void* v, int dtype, int64_t B, int64_t S,
                             int64_t Hq, int64_t Hkv, int64_t D, void* stream);

/* Device self-test of the quantisation kernels' fast quotient: for every finite 16-bit input
 * value x and every 16-bit row maximum amax >= |x| in [2^-60, 2^60] (rows outside that range
 * take the division path) it compares the quantised code obtained from the three-instruction
 * corrected quotient x / RN(amax / d) (d = 127 for int8, 448 for e4m3) with the code obtained
 * from the IEEE division the reference performs.  counters[0] = mismatching pairs (must be 0), counters[1] = pairs
 * checked; `counters` is device memory for two 64-bit integers.  No reference counterpart. */
ARKE_B200_API int arke_b200_selftest_quant_division(int x_dtype, int out_kind, unsigned long long* counters,
                                      void* stream);

/* Packed SwiGLU: Y = silu(X[:, :N]) * X[:, N:]  (arke/ir/ops/reference_impls.py:167-171;
 * arke/backend/triton_templates/gated_activation.py.j2:21-92), optionally fused with per-row
 * e4m3 re-quantisation of Y (scale = amax|Y| / 448).
 *   x [M,2N] bf16/f16/f32.  y [M,N] same dtype as x, or NULL.  yq [M,N] e4m3 bytes + scale [M],
 *   or NULL.  At least one of y / yq must be given. */
ARKE_B200_API int arke_b200_silu_and_mul(const void* x, int x_dtype, int64_t M, int64_t N, int64_t ldx, void* y,
                           int64_t ldy, void* yq, int64_t ldq, float* scale, void* stream);

/* Quantised GEMM with per-row x per-channel dequantisation:
 *   acc[i,j] = sum_k A[i,k] * W[k,j]   (int8 x int8 -> int32 exact, or e4m3 x e4m3 -> fp32)
 *   Y[i,j]   = out_dtype((float(acc) * sa[i]) * sw[j])
 * Composition of quantize_per_token, matmul and dequantize_per_channel
 * (arke/ir/ops/reference_impls.py:118-119, 215-224; arke/ir/ops/catalog.py:70-80,458-479).
 *   a [M,K] K-contiguous (row stride lda); w per w_layout (row stride ldw);
 *   sa [M], sw [N] fp32 (either may be NULL = 1.0);
 *   y [M,N] bf16/f16/f32 (NULL to skip), acc_out [M,N] int32 or fp32 raw accumulators (NULL to skip).
 *   ab_dtype: ARKE_I8 or ARKE_E4M3. */
ARKE_B200_API int arke_b200_quant_gemm(const void* a, int64_t lda, const void* w, int64_t ldw, int w_layout,
                         int ab_dtype, const float* sa, const float* sw, int64_t M, int64_t N,
                         int64_t K, void* y, int y_dtype, int64_t ldy, void* acc_out,
                         int64_t ldacc, void* stream);

/* Dense GEMM  C[M,N] = A[M,K] * B  with fp32 accumulation (the `matmul` op,
 * arke/ir/ops/reference_impls.py:118-119).  a, b, c: bf16, f16 or f32 (same dtype); f32 operands
 * are multiplied as TF32 (10-bit significand) on the tensor cores, which stays inside the
 * reference's 1e-2 comparison rule (arke/agent/tools.py:510-517).  b per w_layout. */
ARKE_B200_API int arke_b200_matmul(const void* a, int64_t lda, const void* b, int64_t ldb, int w_layout,
                     int dtype, int64_t M, int64_t N, int64_t K, void* c, int64_t ldc,
                     void* stream);

/* C[M,N] = A^T B with A given as [K,M] (M contiguous, row stride lda) — the operand layout of a
 * weight-gradient GEMM (dW = G^T X).  16-bit operands (bf16 / f16), fp32 accumulate; B layout as in
 * arke_b200_matmul; c_dtype bf16 / f16 / f32.  The tensor core reads A as an "MN-major" shared-memory
 * operand, so no transposed copy of A is made. */
ARKE_B200_API int arke_b200_matmul_tn(const void* a, int64_t lda, const void* b, int64_t ldb, int w_layout,
                        int dtype, int64_t M, int64_t N, int64_t K, void* c, int c_dtype, int64_t ldc,
                        void* stream);

/* Causal / non-causal grouped-query flash-attention forward
 * (arke/ir/ops/reference_impls.py:236-244; arke/backend/triton_templates/flash_attention.py.j2).
 *   q [B,Hq,S,D], k,v [B,Hkv,Skv,D] contiguous bf16/f16, D = 128 or 64, Hq % Hkv == 0.
 *   o [B,Hq,S,D] same dtype; lse [B,Hq,S] fp32 natural-log logsumexp of the scaled, masked
 *   scores (may be NULL).  softmax_scale <= 0 selects 1/sqrt(D).  With causal != 0 query i sees
 *   keys j <= i (top-left aligned, as F.scaled_dot_product_attention(is_causal=True)). */
ARKE_B200_API int arke_b200_gqa_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int dtype,
                      int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int64_t Skv, int64_t D,
                      int causal, float softmax_scale, void* stream);

/* Fused linear + cross-entropy without materialising logits
 * (arke/ir/ops/reference_impls.py:211-213): logits = X * W^T in fp32 from 16-bit inputs,
 * loss_i = logsumexp(logits_i) - logits_i[label_i], 0 for label_i == ignore_index.
 *   x [M,D], w [V,D] bf16/f16, labels [M] int64.
 *   loss_tok [M] fp32 (may be NULL), mean_loss [1] fp32 = sum / count(non-ignored) (may be NULL).
 *   partials [M,3] fp32 (may be NULL): per-row (max, sum exp(l - max), target logit or 0) over
 *   this call's vocabulary slice, for combining vocabulary shards; `vocab_offset` is the global
 *   index of w's first row (labels are global indices).
 *   A call with vocab_offset == 0 and partials == NULL covers the whole vocabulary for certain:
 *   a non-ignored label outside [0, V) (the reference's F.cross_entropy raises for it) then gives
 *   that row a NaN loss and records code 6 in the kernel status word.  Slice calls cannot tell a
 *   corrupt label from one that another slice holds and treat it as "not in this slice".
 *   workspace: at least arke_b200_fused_linear_ce_workspace(M, V, D) bytes of device memory. */
ARKE_B200_API size_t arke_b200_fused_linear_ce_workspace(int64_t M, int64_t V, int64_t D);
ARKE_B200_API int arke_b200_fused_linear_ce(const void* x, const void* w, const int64_t* labels, int dtype,
                              int64_t M, int64_t V, int64_t D, int64_t vocab_offset,
                              int64_t ignore_index, float* loss_tok, float* mean_loss,
                              float* partials, void* workspace, size_t workspace_bytes,
                              void* stream);

/* fused_linear_ce for hosts that cannot hand over a workspace.  No counterpart in the reference.
 * Same computation and arguments as arke_b200_fused_linear_ce, but the scratch memory is an 8 MiB
 * array built into the library (resident on every GPU that loads it until the process exits)
 * instead of a caller-allocated workspace: meant for callers whose device memory is entirely
 * owned by their own pool, or that must not trigger an allocation (and the device-wide stall it
 * can bring) where this op runs.  The call allocates and frees nothing.
 *   Limit: arke_b200_fused_linear_ce_workspace(M, V, D) must be <= 8 MiB (8388608 bytes), e.g.
 *   M <= 1024 tokens at V = 128256, or M <= 8192 at V <= 32000; larger problems are rejected with
 *   ARKE_ERR_WORKSPACE.
 *   The first call on each device resolves the array's device address: make it before any
 *   stream capture.  All calls share the array; calls that overlap on the GPU race on it, so
 *   order them on one stream (or with events). */
ARKE_B200_API int arke_b200_fused_linear_ce_static(const void* x, const void* w, const int64_t* labels, int dtype,
                                     int64_t M, int64_t V, int64_t D, int64_t vocab_offset,
                                     int64_t ignore_index, float* loss_tok, float* mean_loss,
                                     float* partials, void* stream);

/* Combines G vocabulary-shard partials [G,M,3] (layout above) into per-token loss and mean. */
ARKE_B200_API int arke_b200_ce_combine(const float* partials, int64_t G, int64_t M, const int64_t* labels,
                         int64_t ignore_index, float* loss_tok, float* mean_loss, void* stream);

/* Backward of fused linear + cross-entropy: gradients of the MEAN loss w.r.t. x and w.
 * The reference implements the forward only (arke/ir/ops/reference_impls.py:211-213); its operator
 * documentation promises a logits gradient (docs/benchmark/benchmark-ops.md:582-593) that none of
 * its backends produces.  Definition: with p = softmax(x w^T) per row and n = number of rows whose
 * label != ignore_index,
 *   G[i,j] = p[i,j] - [j == labels[i] - vocab_offset]                (rows with ignored label: 0)
 *   dx = (g / n) G w   [M,D],      dw = (g / n) G^T x   [V,D]        (fp32 accumulate)
 *   g = grad * (grad_dev ? *grad_dev : 1): `grad_dev` is an optional fp32 device scalar (the
 *   upstream gradient of a training step), so that no host read of it is needed.
 *   dx is written as `dx_dtype`: the operands' dtype, or ARKE_F32 (what a vocabulary-sharded
 *   caller sums over ranks without a 16-bit rounding per rank); dw has the operands' dtype.
 *   lse [M] fp32: natural-log logsumexp of each row's logits over the WHOLE vocabulary, as the
 *   forward's partials give it (max + log(sumexp)); with a vocabulary slice (vocab_offset, V rows
 *   of w) dx is this slice's contribution and the caller sums the slices' dx.
 *   dx / dw may be NULL (skipped).  workspace: arke_b200_fused_linear_ce_backward_workspace(M, V)
 *   bytes, 256-byte aligned (holds G, 16-bit and unscaled, [M, V rounded up to 8]). */
ARKE_B200_API size_t arke_b200_fused_linear_ce_backward_workspace(int64_t M, int64_t V);
ARKE_B200_API int arke_b200_fused_linear_ce_backward(const void* x, const void* w, const int64_t* labels,
                                       const float* lse, int dtype, int64_t M, int64_t V, int64_t D,
                                       int64_t vocab_offset, int64_t ignore_index, float grad,
                                       const float* grad_dev, void* dx, int dx_dtype, void* dw,
                                       void* workspace, size_t workspace_bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* ARKE_B200_H */
