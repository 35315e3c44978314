/*
 * hawk_b200 -- C ABI of the B200 (sm_100a) kernels for Hawk's data-parallel hot path.
 *
 * The reference (fattorib/hawk-pytorch) has no FFI: its seam is three Python names
 * imported into hawk/hawk.py:12-14 (Conv1D, fused_cross_entropy, fused_linear_scan) plus
 * the eager decode step in Hawk.forward.  Each entry point below names the reference code
 * it stands in for.  The Python side of the boundary (hawk_b200.ops) binds these with
 * ctypes and keeps the reference's call signatures.
 *
 * Conventions
 *   - plain pointers and sizes only; every pointer is a DEVICE pointer unless said otherwise;
 *   - nothing here allocates, frees or synchronises: outputs and scratch ("workspace") are
 *     passed in by the caller, sized by the *_workspace_bytes helpers;
 *   - `stream` is a cudaStream_t passed as void*; work is enqueued on it and the call returns;
 *   - return value: HAWK_OK (0) or a negative hawk_status; hawk_strerror() gives the text;
 *     arguments are validated on the host before anything is launched;
 *   - tensors are row-major with the channel (last) dimension contiguous.  `dtype` selects the
 *     storage type of activations (HAWK_F32 or HAWK_BF16); arithmetic is always fp32;
 *     Lambda, conv weights/bias and all parameter gradients are fp32.
 */
#ifndef HAWK_B200_H_
#define HAWK_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define HAWK_B200_ABI_VERSION 4

typedef enum hawk_dtype { HAWK_F32 = 0, HAWK_BF16 = 1 } hawk_dtype;

typedef enum hawk_status {
  HAWK_OK = 0,
  HAWK_ERR_NULL = -1,        /* a required pointer is NULL */
  HAWK_ERR_SHAPE = -2,       /* a dimension is out of range or not a supported multiple */
  HAWK_ERR_DTYPE = -3,       /* unknown dtype enum */
  HAWK_ERR_ALIGN = -4,       /* a pointer or stride breaks the stated alignment */
  HAWK_ERR_WORKSPACE = -5,   /* workspace missing or too small */
  HAWK_ERR_LAUNCH = -6,      /* the CUDA runtime refused a launch (cudaGetLastError) */
  HAWK_ERR_UNSUPPORTED = -7, /* valid request this build does not implement */
  HAWK_ERR_DEVICE = -8,      /* wrong device / driver entry point unavailable */
  HAWK_ERR_TOO_LARGE = -9    /* size exceeds the built-in scratch of a *_noalloc entry point */
} hawk_status;

/* ABI version of the loaded library (HAWK_B200_ABI_VERSION at build time). */
int hawk_version(void);
/* Static, NUL-terminated description of a hawk_status. */
const char* hawk_strerror(int status);

/* ------------------------------------------------------------------------------------------
 * RG-LRU scan.  Replaces hawk/scan_fused.py:319-360 (sequential_scan_forward + the Triton
 * kernel :34-109) and :363-424 (sequential_scan_backward + kernel :112-317, including the
 * batch sum of the Lambda gradient at :424).
 *
 *   i = sigmoid(gx), r = sigmoid(ga), a = exp(-8 r softplus(lam)),
 *   h_t = a_t h_{t-1} + x_t i_t sqrt(1 - a_t^2),   h_{-1} = h0 (zero when h0 == NULL).
 *
 * x, gx, ga, h, go, dx, dgx, dga: [B,T,D] contiguous, `dtype`;  lam, dlam: [D] fp32.
 * D must be a multiple of 64 (as the reference asserts, scan_fused.py:333); T >= 1.
 * h0 / dh0: optional [B,D] fp32 (no counterpart in the reference, whose initial state is
 * fixed at zero, scan_fused.py:77-79); pass NULL for the reference behaviour.
 * gate_bias / dgate_bias: optional [2,D] fp32, row 0 for gx and row 1 for ga.  With gate_bias the
 * gates are sigmoid(gx + gate_bias[0]) and sigmoid(ga + gate_bias[1]): the bias add of the
 * reference's block-diagonal gate projections (BlockDiagonalLinear, hawk/external.py:171-233, the add at
 * :230; called at hawk/hawk.py:181-182) done inside the scan.  The sum is kept in fp32 (the reference
 * rounds gate + bias to bf16 under autocast before its scan, hawk/scan_fused.py:428).  The
 * caller then passes the bias-free projections as gx, ga.  dgate_bias receives the sums of dgx and
 * dga over batch and time (what autograd's bias gradient computes), in fp32, in a fixed order.
 * Pass NULL for the reference's scan signature.
 * The backward reads the forward OUTPUT h (as stored) for h_{t-1}, like the reference.
 * Workspace (backward only): 16-byte aligned; B*D*4 bytes, three times that when dgate_bias is
 * given; hawk_scan_bwd_workspace_bytes(B, D) returns the larger figure.
 * ---------------------------------------------------------------------------------------- */
int hawk_scan_fwd(const void* x, const void* gx, const void* ga, const float* lam, const float* h0,
                  const float* gate_bias, void* h, int B, int T, int D, int dtype, void* stream);
size_t hawk_scan_bwd_workspace_bytes(int B, int D);
int hawk_scan_bwd(const void* x, const void* gx, const void* ga, const float* lam, const float* h0,
                  const float* gate_bias, const void* h, const void* go, void* dx, void* dgx, void* dga,
                  float* dlam, float* dh0, float* dgate_bias, void* workspace, size_t workspace_bytes,
                  int B, int T, int D, int dtype, void* stream);

/* The scan with the recurrent block's epilogue fused in: out = gelu(y) * h (Hawk.epilogue,
 * hawk/hawk.py:134-135, called at :201; exact erf GELU as torch.nn.functional.gelu).  Replaces the scan
 * plus the separate pointwise pass over [B,T,D] that the reference runs after it, in both directions.
 * y is the other half of the block's input projection (hawk/hawk.py:164-166), read in place: element
 * (b,t,d) at y + b*y_batch_stride + t*y_row_stride + d (strides in ELEMENTS, multiples of 16 bytes, base
 * 16-byte aligned).  Forward writes h (needed by the backward, and the decode state) and out, both
 * [B,T,D] contiguous; out is formed from h as stored.  Backward takes dout = d loss / d out and writes
 * dx, dgx, dga ([B,T,D] contiguous) and dy with its own strides (so it can land in the y half of the
 * projection's gradient); h_t is recomputed from the stored h_{t-1}.  Initial state is zero.
 * gate_bias / dgate_bias, lam / dlam and the workspace are as for hawk_scan_fwd / hawk_scan_bwd. */
int hawk_scan_gelu_fwd(const void* x, const void* gx, const void* ga, const float* lam,
                       const float* gate_bias, const void* y, int64_t y_batch_stride, int64_t y_row_stride,
                       void* h, void* out, int B, int T, int D, int dtype, void* stream);
int hawk_scan_gelu_bwd(const void* x, const void* gx, const void* ga, const float* lam,
                       const float* gate_bias, const void* h, const void* y, int64_t y_batch_stride,
                       int64_t y_row_stride, const void* dout, void* dx, void* dgx, void* dga, void* dy,
                       int64_t dy_batch_stride, int64_t dy_row_stride, float* dlam, float* dgate_bias,
                       void* workspace, size_t workspace_bytes, int B, int T, int D, int dtype, void* stream);

/* Time-split scans: the same results as hawk_scan_fwd / hawk_scan_gelu_fwd and hawk_scan_bwd /
 * hawk_scan_gelu_bwd for launches with few (sequence, channel group) pairs -- one long sequence, a narrow
 * model -- where a whole-sequence scan leaves most SMs idle (the reference walks T in one warp per channel
 * block whatever the shape, hawk/scan_fused.py:83).  Every sequence is cut into nsub sub-sequences of
 * T / nsub rows (T % nsub == 0, nsub <= 64); a first pass reduces each to its affine state map, a small
 * kernel composes the maps along the sequence, and the ordinary kernels then run over all B * nsub
 * sub-sequences at once.  Inputs are read twice; results agree with the whole-sequence entry points to
 * fp32 rounding of the carried state.
 * hawk_scan_split_chunks: the nsub this library would use for a shape and pass (HAWK_SCAN_PASS_*; 1: call
 * the whole-sequence entry point).  y == NULL (and out / dy == NULL) selects the plain scan, otherwise the fused gelu(y) * h
 * epilogue; y / dy views need batch stride == T * row stride (else HAWK_ERR_UNSUPPORTED).  go is d loss /
 * d h for the plain scan and d loss / d out for the fused one.  Workspace: 16-byte aligned,
 * hawk_scan_split_workspace_bytes(B, nsub, D) bytes, no initialisation needed. */
#define HAWK_SCAN_PASS_FWD 0      /* plain forward */
#define HAWK_SCAN_PASS_FWD_GELU 1 /* forward with the gelu(y) * h epilogue */
#define HAWK_SCAN_PASS_BWD 2      /* either backward */
int hawk_scan_split_chunks(int B, int T, int D, int pass);
size_t hawk_scan_split_workspace_bytes(int B, int nsub, int D);
int hawk_scan_fwd_split(const void* x, const void* gx, const void* ga, const float* lam, const float* h0,
                        const float* gate_bias, const void* y, int64_t y_batch_stride, int64_t y_row_stride,
                        void* h, void* out, int nsub, void* workspace, size_t workspace_bytes, int B, int T,
                        int D, int dtype, void* stream);
int hawk_scan_bwd_split(const void* x, const void* gx, const void* ga, const float* lam, const float* h0,
                        const float* gate_bias, const void* h, const void* y, int64_t y_batch_stride,
                        int64_t y_row_stride, const void* go, void* dx, void* dgx, void* dga, void* dy,
                        int64_t dy_batch_stride, int64_t dy_row_stride, float* dlam, float* dh0,
                        float* dgate_bias, int nsub, void* workspace, size_t workspace_bytes, int B, int T,
                        int D, int dtype, void* stream);

/* hawk_scan_bwd for hosts that cannot allocate device memory (no counterpart in the reference, which
 * allocates its scratch with torch.empty on every call, hawk/scan_fused.py:378).  Same arguments and
 * results as hawk_scan_bwd without gate biases, but no workspace: the [B,D] fp32 scratch is a fixed 1 MiB array inside the
 * library (per GPU, kept until exit), so B * D <= 262144 or HAWK_ERR_TOO_LARGE.  Calls nothing that
 * allocates.  The first call on each device looks the array's device address up (make it outside a
 * stream capture).  All calls on a device share the array: calls overlapping on the GPU race. */
int hawk_scan_bwd_noalloc(const void* x, const void* gx, const void* ga, const float* lam,
                          const float* h0, const void* h, const void* go, void* dx, void* dgx, void* dga,
                          float* dlam, float* dh0, int B, int T, int D, int dtype, void* stream);

/* ------------------------------------------------------------------------------------------
 * Causal depthwise temporal convolution, width W in [1,4].  Replaces Conv1D.forward
 * (hawk/external.py:49-98) and the autograd backward of its eager ops.
 *
 *   y[b,t,d] = bias[d] + sum_{k<W} w[W-1-k, d] * x[b,t-k,d],   x[b,t<0] = 0.
 *
 * x: element (b,t,d) at x + b*x_batch_stride + t*x_row_stride + d (strides in ELEMENTS), so
 * the strided half of the [B,T,2R] projection (hawk/hawk.py:164-166) is read in place.
 * y, go: [B,T,D] contiguous.  dx is written with its own strides.  w: [W,D], bias: [D], fp32.
 * D must be a multiple of 8; every base pointer 16-byte aligned; strides multiples of 8.
 * Backward workspace: hawk_conv1d_bwd_workspace_bytes(B, T, D, W).
 * ---------------------------------------------------------------------------------------- */
int hawk_conv1d_fwd(const void* x, int64_t x_batch_stride, int64_t x_row_stride, const float* w,
                    const float* bias, void* y, int B, int T, int D, int W, int in_dtype,
                    int out_dtype, void* stream);
size_t hawk_conv1d_bwd_workspace_bytes(int B, int T, int D, int W);
int hawk_conv1d_bwd(const void* go, const void* x, int64_t x_batch_stride, int64_t x_row_stride,
                    const float* w, void* dx, int64_t dx_batch_stride, int64_t dx_row_stride,
                    float* dw, float* dbias, void* workspace, size_t workspace_bytes, int B, int T,
                    int D, int W, int go_dtype, int x_dtype, void* stream);

/* ------------------------------------------------------------------------------------------
 * Cached single-token decode step of one Hawk block, any batch size.  Replaces the eager
 * path hawk/hawk.py:168-179 (conv over [conv_state | x]) + hawk/cache.py:37-43 (roll), and
 * hawk/hawk.py:137-151,193-198 (inference_prologue, h = a*state + x~, cache update).
 *
 * conv step : x_new [B,D] (row stride x_row_stride elements), conv_state [B,W-1,D] contiguous,
 *             oldest row first, updated IN PLACE; y [B,D] contiguous.
 * rglru step: x, gx, ga [B,D] contiguous `dtype`; state [B,D] `state_dtype`, updated IN PLACE
 *             with h; h_out [B,D] `dtype` (may be NULL).
 * ---------------------------------------------------------------------------------------- */
int hawk_decode_conv_step(const void* x_new, int64_t x_row_stride, void* conv_state, const float* w,
                          const float* bias, void* y, int B, int D, int W, int dtype,
                          int state_dtype, void* stream);
int hawk_decode_rglru_step(const void* x, const void* gx, const void* ga, const float* lam,
                           void* state, void* h_out, int B, int D, int dtype, int state_dtype,
                           void* stream);
/* The same cached token for the whole recurrent branch in one launch: conv step (+ cache roll), both
 * block-diagonal gate projections with their biases (hawk/external.py:224-233 at hawk/hawk.py:181-182),
 * RG-LRU step (state in place) and out = gelu(y) * h (hawk/hawk.py:134-135,199).  xy [B, >= 2R] rows of
 * [x_b | y] (`dtype`, row stride in elements); conv_state [B,W-1,R] and state [B,R] (`state_dtype`);
 * wx, wa [R/block_width, block_width, block_width] (`weight_dtype`), bx, ba, lam, conv_w [W,R], conv_b
 * fp32; out [B,R] `dtype`.  block_width <= 128, W <= 4. */
int hawk_decode_block_step(const void* xy, int64_t xy_row_stride, void* conv_state, const float* conv_w,
                           const float* conv_b, const void* wx, const void* wa, const float* bx, const float* ba,
                           const float* lam, void* state, void* out, int B, int R, int block_width, int W,
                           int dtype, int state_dtype, int weight_dtype, void* stream);

/* ------------------------------------------------------------------------------------------
 * Fused linear + cross-entropy.  Replaces CrossEntropyLoopedFused.forward
 * (hawk/fused_cross_entropy.py:13-64): mean cross-entropy of act @ weight^T against labels, and
 * BOTH gradients, in one call (the reference also computes them in its forward, :47-61; its
 * backward only scales them, :66-73).
 *
 * weight [V,H], act [N,H]: contiguous, `dtype` (HAWK_F32 or HAWK_BF16); labels [N] int64 in [0,V).
 * loss: one fp32; dweight [V,H] and dact [N,H]: fp32, already scaled by 1/N.
 * Arithmetic is what the reference does under bf16 autocast: bf16 operands, fp32 accumulation,
 * logits rounded to bf16, softmax in fp32, dprobs rounded to bf16 before the gradient GEMMs.
 * H must be a multiple of 8.  Workspace: hawk_linear_ce_workspace_bytes(N, H, V), 256-byte aligned
 * (bf16 copies of fp32 operands, the [N,V] bf16 logits/dprobs buffer, row statistics; no transposed
 * copies: the gradient GEMMs read their row-contracted operands as MN-major tiles).
 * status: one int32 in device memory, zeroed by the caller once; a kernel whose bounded wait on an
 * mbarrier ran out sets it to 1 (the results of that call are then invalid) instead of hanging, and the
 * call then also overwrites `loss` with NaN, so a caller that never reads the status word still sees it.
 * Labels must lie in [0, V) (the reference's gather would raise otherwise, fused_cross_entropy.py:37-39;
 * it has no ignore_index): a label outside the range makes `loss` non-finite (NaN or inf).
 * ---------------------------------------------------------------------------------------- */
size_t hawk_linear_ce_workspace_bytes(int64_t N, int64_t H, int64_t V);
int hawk_linear_ce_fwd_bwd(const void* weight, const void* act, const int64_t* labels, float* loss,
                           float* dweight, float* dact, void* workspace, size_t workspace_bytes,
                           int64_t N, int64_t H, int64_t V, int dtype, int* status, void* stream);

/* ------------------------------------------------------------------------------------------
 * Both block-diagonal gate projections of the recurrent block, one pass per direction.  Replaces the two
 * BlockDiagonalLinear.forward calls (hawk/external.py:224-233, called at hawk/hawk.py:181-182: einsum ->
 * two bmm launches that each re-read the conv output) and the four GEMMs of their backward.  The biases
 * (external.py:230) are not added here: pass them to the scan as gate_bias.
 *
 *   forward : gx[m, n*bw + j] = sum_i xc[m, n*bw + i] * wx[n][i][j]   (ga likewise with wa)
 *   backward: dxc[m, n*bw + i] += sum_j dgx[m, n*bw + j] * wx[n][i][j] + dga[..] * wa[n][i][j]  (IN PLACE: dxc
 *             arrives holding the scan's input gradient), dwx[n][i][j] = sum_m xc[m, n*bw+i] * dgx[m, n*bw+j]
 *             (dwa likewise), summed in a fixed order.
 *
 * xc, gx, ga, dgx, dga, dxc: [M, R] contiguous bf16 (M = batch * time); wx, wa: [R/bw, bw, bw] in `w_dtype`;
 * dwx, dwa: the same shape in fp32.  bw must divide 128 (>= 8) and R be a multiple of 128.  tcgen05 GEMMs
 * with bf16 operands and fp32 accumulation: the arithmetic of the reference's einsum under autocast.
 * hawk_gates_pack_weights converts both weights once per step into the operand layouts of the kernels
 * (`packed`, hawk_gates_packed_bytes(R, bw) bytes, 16-byte aligned), used by forward and backward.
 * Backward workspace: hawk_gates_bwd_workspace_bytes(M, R, bw), 16-byte aligned.  status: as for
 * hawk_linear_ce_fwd_bwd.
 * ---------------------------------------------------------------------------------------- */
size_t hawk_gates_packed_bytes(int R, int bw);
size_t hawk_gates_bwd_workspace_bytes(int64_t M, int R, int bw);
int hawk_gates_pack_weights(const void* wx, const void* wa, int w_dtype, void* packed, int R, int bw,
                            void* stream);
int hawk_gates_fwd(const void* xc, const void* packed, void* gx, void* ga, int64_t M, int R, int bw,
                   int* status, void* stream);
int hawk_gates_bwd(const void* xc, const void* dgx, const void* dga, const void* packed, void* dxc, float* dwx,
                   float* dwa, void* workspace, size_t workspace_bytes, int64_t M, int R, int bw, int* status,
                   void* stream);

/* Shows that a device-side wait of the tcgen05 kernels gives up instead of hanging (no counterpart in
 * the reference): launches one 128 x 128 tile of the gate-projection kernel inside `scratch` (>= 262144
 * bytes, 256-byte aligned) with its TMA producer switched off and a wait budget of `budget_cycles` clock
 * cycles (1e3 .. 1e8).  The kernel must return by itself and set *status to 1. */
int hawk_debug_wait_timeout(void* scratch, size_t scratch_bytes, long long budget_cycles, int* status,
                            void* stream);

/* ------------------------------------------------------------------------------------------
 * Glue of the block around the GEMMs, one HBM pass each (reference: eager torch ops).
 *
 * gelu_mul: out[m,j] = gelu(a[m,j]) * b[m,j], exact (erf) GELU.  Replaces `F.gelu(gate) * up`
 *   (hawk/hawk.py:82-86) and `F.gelu(y) * h` (hawk/hawk.py:134-135).  a, b, out and the gradients are
 *   [M,J] with unit column stride and their own row pitch in ELEMENTS, so the two halves of a
 *   projection output are read in place and both gradients can land in the halves of one buffer.
 *   J and every pitch multiples of 8; pointers 16-byte aligned; one `dtype` for all tensors.
 * rms_norm: y = x * rsqrt(mean_j x^2 + eps) * w, statistics in fp32 (hawk/hawk.py:47-58); x, dx in
 *   `x_dtype`, y, dy in `y_dtype` (bf16 y from fp32 x is what autocast makes of the next Linear's
 *   input); w, dw, rstd [M] fp32.  H multiple of 4 (backward: H <= 4096).  Backward workspace:
 *   hawk_rms_norm_bwd_workspace_bytes(H).
 * ---------------------------------------------------------------------------------------- */
int hawk_gelu_mul_fwd(const void* a, int64_t lda, const void* b, int64_t ldb, void* out, int64_t ldo,
                      int64_t M, int J, int dtype, void* stream);
int hawk_gelu_mul_bwd(const void* dout, int64_t ldd, const void* a, int64_t lda, const void* b, int64_t ldb,
                      void* da, int64_t ldda, void* db, int64_t lddb, int64_t M, int J, int dtype,
                      void* stream);
int hawk_rms_norm_fwd(const void* x, const float* w, void* y, float* rstd, int64_t M, int H, float eps,
                      int x_dtype, int y_dtype, void* stream);
size_t hawk_rms_norm_bwd_workspace_bytes(int H);
int hawk_rms_norm_bwd(const void* dy, const void* x, const float* w, const float* rstd, void* dx, float* dw,
                      void* workspace, size_t workspace_bytes, int64_t M, int H, int x_dtype, int y_dtype,
                      void* stream);

/* The residual add that precedes every norm of the block (hawk/hawk.py:229,234 followed by :227,232,284)
 * fused into the norm: x_out = x + delta (x_dtype; delta in y_dtype), y = rms_norm(x_out).  Backward:
 * dx = gres + (norm backward of dy), with gres the gradient reaching x_out from everything after it
 * (x_dtype, may be NULL); ddelta (y_dtype, may be NULL) receives the same values for the delta branch. */
int hawk_add_rms_norm_fwd(const void* x, const void* delta, void* x_out, const float* w, void* y, float* rstd,
                          int64_t M, int H, float eps, int x_dtype, int y_dtype, void* stream);
int hawk_add_rms_norm_bwd(const void* dy, const void* x_sum, const float* w, const float* rstd, const void* gres,
                          void* dx, void* ddelta, float* dw, void* workspace, size_t workspace_bytes, int64_t M,
                          int H, int x_dtype, int y_dtype, void* stream);

/* fp32 -> bf16 (round to nearest even) of n contiguous elements: the weight cast that CUDA autocast runs
 * before every bf16 GEMM of an fp32 parameter (torch's type-converting copy, reached from F.linear in
 * hawk/hawk.py:75-86,110-116 under torch.autocast), as one vectorised pass.  src, dst 16-byte aligned. */
int hawk_cast_f32_bf16(const float* src, void* dst, int64_t n, void* stream);

/* One AdamW step (decoupled weight decay, torch.optim.AdamW's update rule with bias correction for
 * step number `step` >= 1) on n contiguous fp32 elements, in place in p, m (first moment) and v (second
 * moment); g is the gradient.  p_bf16 (may be NULL) receives the bf16 rounding of the updated p, so the
 * next forward needs no cast pass.  No counterpart in the reference, which stops at loss.backward()
 * (README.md:36) and leaves the optimiser to the user; this is the update torch.optim.AdamW would make. */
int hawk_adamw_step(float* p, const float* g, float* m, float* v, void* p_bf16, int64_t n, float lr, float beta1,
                    float beta2, float eps, float weight_decay, int64_t step, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* HAWK_B200_H_ */
