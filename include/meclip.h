/*
 * meclip.h - C ABI of libmeclip_sm100.so: the CLIP / LiT contrastive-loss path
 * (forward sums + loss, recompute backward, L2-normalise and its Jacobian) as
 * hand-written sm_100a kernels.
 *
 * Conventions
 *  - Plain C types only.  Every pointer is a DEVICE pointer unless it says host.
 *  - The library never allocates or frees device memory: the caller owns every
 *    buffer, including the workspace (size from meclip_grad_workspace_bytes).
 *  - Every call is asynchronous on `stream` (a cudaStream_t passed as void*),
 *    and may be made from any host thread (PyTorch runs backward on its autograd
 *    thread); calls from several threads are serialised where they share state.
 *    meclip_grad may also use two library-owned side streams, forked from and
 *    joined back into `stream`, so that independent kernels of one backward overlap
 *    (set MECLIP_SERIAL=1 to keep everything on `stream`).
 *  - Return value: MECLIP_OK or an error code; meclip_last_error() gives text.
 *    Nothing here calls exit/abort or throws.
 *  - Matrices are row-major with a leading dimension in ELEMENTS (ld >= D).
 *    Operand matrices of the tile kernels are bf16; their D must be a multiple of 8
 *    and base pointers / row pitches 16-byte aligned (TMA requirements).  The two
 *    row kernels (meclip_normalize_fwd / _bwd) take and give any D, pitch, alignment
 *    and fp32 / bf16 / fp16, and produce such operands by zero padding.
 *  - `status` is a device int the kernels set non-zero when a bounded wait inside
 *    a kernel ran out (MECLIP_ETIMEOUT); read it with meclip_read_status().  The bound
 *    is 2 s of wall time per wait (environment MECLIP_WAIT_LIMIT_MS changes it, e.g. for
 *    a GPU that is time-sliced between processes).
 *
 * Reference = b0nce/MemoryEfficientCLIP (clip_loss.py, lit_loss.py).
 */
#ifndef MECLIP_H
#define MECLIP_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum meclip_status {
    MECLIP_OK = 0,
    MECLIP_EINVAL = 1,       /* null / misaligned pointer, bad size, bad enum */
    MECLIP_ENOSPC = 2,       /* workspace too small */
    MECLIP_ECUDA = 3,        /* a CUDA runtime / driver call failed */
    MECLIP_ETIMEOUT = 4,     /* a bounded in-kernel wait expired (from status word) */
    MECLIP_EUNSUPPORTED = 5  /* not an sm_100 device, or driver lacks TMA entry point */
};

enum meclip_kind { MECLIP_CLIP = 0, MECLIP_LIT = 1, MECLIP_SIGLIP = 2 /* internal to the siglip entry points */ };
enum meclip_dtype { MECLIP_BF16 = 0, MECLIP_F32 = 1, MECLIP_F16 = 2 /* row kernels only */ };

/* How a gradient output buffer is written. */
enum meclip_out_mode {
    MECLIP_STORE_BF16 = 0,  /* out = value, bf16 */
    MECLIP_STORE_F32 = 1,   /* out = value, fp32 */
    MECLIP_ACCUM_F32 = 2    /* out += value, fp32 (ring steps, caller zeroes first) */
};

int meclip_version(void);
const char* meclip_status_string(int code);
/* Copies the calling thread's process-wide last error text (host buffer). */
int meclip_last_error(char* buf, size_t buf_len);
/* Synchronises `stream`, copies *status to the host and maps non-zero to MECLIP_ETIMEOUT. */
int meclip_read_status(const int* status, void* stream);

/*
 * Scalars that live on the device.  The entry points below take the temperature (softmax losses) or the
 * logit scale and bias (sigmoid loss) as host floats, as the reference does (clip_loss.py:181).  A trainer that
 * LEARNS them holds them in device memory; reading them back for every step would stall the host.  This call
 * binds device addresses for the NEXT tile-pass or loss-finalisation call made by the same host thread
 * (meclip_sum_exp, meclip_loss_finalize, meclip_loss_forward, meclip_grad, meclip_grad_t, meclip_grad_static,
 * meclip_loss_backward, meclip_lit_fused_forward, meclip_lit_fused_backward, meclip_siglip_sum,
 * meclip_siglip_grad, meclip_step_forward, meclip_step_backward); that call consumes the binding whether it succeeds or not and ignores its float
 * temperature / scale / bias arguments in favour of the bound values:
 *   temperature_or_scale  fp32 device scalar: T for CLIP / LiT, t for the sigmoid loss
 *   logit_bias            fp32 device scalar or NULL (sigmoid loss only; NULL keeps the float argument)
 *   grad_scale_rule       how a backward completes its grad_scale argument, which the caller then forms for
 *                         T = 1: 0 as given, 1 divided by T (grad_scale = 1/B), 2 divided by sqrt(T)
 *                         (Stable variants, 1/sqrt(B)), 3 multiplied by t (sigmoid loss, 1/B)
 * The scalars are read by the kernels when they run, so the memory must stay valid until then.  The
 * binding is per host thread; nothing is shared between threads.  The reference has no counterpart (its
 * temperature is a Python float and gets no gradient, clip_loss.py:256).
 */
enum meclip_grad_scale_rule {
    MECLIP_GSCALE_FIXED = 0, MECLIP_GSCALE_OVER_T = 1, MECLIP_GSCALE_OVER_SQRT_T = 2, MECLIP_GSCALE_TIMES_T = 3
};
int meclip_bind_device_scalars(const float* temperature_or_scale, const float* logit_bias, int grad_scale_rule);

/*
 * Peer memory for the ring on one NVLink box (one process per GPU).  A rank exports a handle for a device
 * buffer it owns; the other ranks of the node open it and fetch the visiting shard from it with
 * meclip_copy_async, a plain device-to-device cudaMemcpyAsync that runs on the copy engines: no SM is
 * taken from the persistent tile kernels while a shard is in flight, and no kernel of this library ever
 * reads another GPU's memory (a shard always lands in local memory first).
 *   meclip_ipc_export  handle_out: MECLIP_IPC_HANDLE_BYTES host bytes naming the ALLOCATION that contains ptr
 *                      (as cudaMalloc made it), offset_out: ptr's byte offset inside it
 *   meclip_ipc_open    maps that allocation into the calling process (current device, peer access enabled
 *                      on demand) and returns its base; a handle can be opened once per process
 *   meclip_ipc_close   unmaps it
 *   meclip_copy_async  cudaMemcpyAsync(dst, src, bytes, device-to-device) on `stream`
 * Ordering between processes (when a buffer may be read, when it may be overwritten) is the caller's:
 * the ring host uses its collectives for that.  The reference has no counterpart (it is single-GPU).
 */
#define MECLIP_IPC_HANDLE_BYTES 64
int meclip_ipc_export(const void* ptr, void* handle_out, uint64_t* offset_out);
int meclip_ipc_open(const void* handle, void** base_out);
int meclip_ipc_close(void* base);
int meclip_copy_async(void* dst, const void* src, size_t bytes, void* stream);

/*
 * Test hook: one tiny kernel (one CTA, no tile loads, no tensor memory) that waits on a barrier nobody
 * arrives on, with the same bounded-wait routine the tile kernels use and a limit of limit_ns nanoseconds
 * (at most 100 ms).  The wait runs out, the kernel sets *status non-zero and ends normally, so that
 * meclip_read_status() reports MECLIP_ETIMEOUT while the context stays usable: the way to exercise the
 * time-out reporting without disturbing a real kernel.  Has no counterpart in the reference.
 */
int meclip_debug_wait_probe(uint64_t limit_ns, int* status, void* stream);

/*
 * Test hook: override the backward's blocking (rows of the coefficient matrix formed per
 * block, a multiple of 128, and the byte limit of one panel) so that small problems run
 * the multi-panel / multi-row-block code paths; 0, 0 restores the defaults (16384 rows,
 * 512 MiB).  Affects meclip_grad_workspace_bytes too.  Has no counterpart in the reference.
 */
int meclip_debug_set_blocking(int64_t row_block, int64_t panel_bytes);

/*
 * Test hook: in-kernel trace.  device_words points to n_words zeroed 64-bit words on the
 * device; while set, CTA 0 of every tile kernel appends {tag, tile, nanosecond timer}
 * records from word 2 on (the producer, the MMA issuer and the epilogue each fill their
 * own third; unused records stay zero).  Tags: 1/2 loads of a tile
 * begin/end, 10/11/12 MMA tile begin / first operands arrived / last MMA issued,
 * 20/21/22 epilogue begin / accumulator released / end.  NULL switches it off.
 * Has no counterpart in the reference.
 */
int meclip_debug_set_trace(void* device_words, size_t n_words);

/* Number of kernels this library has launched in this process (all threads). */
long long meclip_launch_count(void);

/*
 * Per-kernel timing with CUDA events on the launch stream.  Between begin and end
 * every launch is bracketed by an event pair; end synchronises on them and sums
 * milliseconds, launches and useful FLOPs per tag: 0 sums pass, 1 coefficient
 * panel, 2 dX contraction, 3 dY contraction, and for the HBM-bound passes, whose
 * third figure is algorithmic BYTES (read + written) instead of FLOPs: 4 loss
 * finalisation, 5 normalise / convert forward, 6 normalise Jacobian / convert
 * backward, 7 operand transposes, 8 fp32 accumulation (ring).  n_tags <= 9.
 * Meant for benchmarks; the events serialise nothing but add launch overhead.
 * Has no counterpart in the reference.
 */
int meclip_profile_begin(void);
int meclip_profile_end(double* ms_by_tag, long long* launches_by_tag, double* flops_by_tag, int n_tags);

/*
 * dst[i] += src[i] over n fp32 values (n a multiple of 4, 16-byte aligned).  Used by the
 * ring backward: the owner of a text shard adds the partial gradients the other ranks
 * send it.  Has no counterpart in the reference (which is single-GPU).
 */
int meclip_accumulate_f32(float* dst, const float* src, int64_t n, void* stream);
/*
 * dst[i] += src[i] + src[src_stride + i] + ... + src[(n_src - 1) * src_stride + i], added in that order: the
 * n_src partial gradients that arrived in one backward (one buffer per ring step, src_stride floats apart), in one
 * pass over dst.  Same alignment rules; src_stride a multiple of 4 and >= n.  No counterpart in the reference.
 */
int meclip_accumulate_many_f32(float* dst, const float* src, int n_src, int64_t src_stride, int64_t n, void* stream);

/*
 * x_hat = x / max(||x||_2, 1e-12) per row, written as bf16, plus inv_norm[i] =
 * 1/max(||x_i||, 1e-12).  With normalize == 0 only the dtype conversion to bf16
 * is done (inv_norm may be NULL).  x may be fp32, bf16 or fp16, with ANY d >= 1, pitch
 * and alignment; x_hat gets round_up(d, 8) columns (the extra ones zero, ldh at least
 * that), which is the operand form the tile kernels need.  Replaces F.normalize(dim=1)
 * at clip_loss.py:266-268 / lit_loss.py:257-259 and the fp32 -> bf16 staging.
 */
int meclip_normalize_fwd(const void* x, int x_dtype, int64_t rows, int64_t d, int64_t ldx, int normalize,
                         void* x_hat_bf16, int64_t ldh, float* inv_norm, void* stream);

/*
 * Jacobian of the row normalisation: dx = (g - x_hat * (x_hat . g)) * inv_norm.
 * Replaces the autograd node PyTorch records for F.normalize
 * (clip_loss.py:266-268).  g (fp32 or bf16) and x_hat have round_up(d, 8) columns;
 * dx takes dx_dtype (fp32, bf16 or fp16), any pitch >= d and any alignment.
 * inv_norm == NULL: plain conversion dx = g (x_hat may then be NULL too).
 */
int meclip_normalize_bwd(const void* g, int g_dtype, int64_t ldg, const void* x_hat_bf16, int64_t ldh,
                         const float* inv_norm, int64_t rows, int64_t d, void* dx, int dx_dtype, int64_t lddx,
                         void* stream);

/*
 * Forward tile pass over one rows x cols block of the similarity matrix
 * S = X Y^T (X: rows x d, Y: cols x d, both bf16, L2-normalised):
 *   E_ij = exp(S_ij/T - 1/T);  row_sum[i] += sum_j E_ij;  col_sum[j] += sum_i E_ij
 *   diag_s[i] = S_ij for the column j with row_off + i == col_off + j, if in range.
 * The sums ACCUMULATE (fp32 atomics): zero them before the first block.
 * col_sum may be NULL (LiT).  Out-of-range rows/columns of edge tiles are
 * masked, so any rows/cols >= 1 is exact.  row_off / col_off are the global
 * indices of X row 0 and Y row 0 (0 on one GPU; shard offsets in the ring).
 * tile_counter: optional device word that must be ZERO when the kernel starts; with
 * it the CTAs fetch tiles dynamically (better balance when other kernels, e.g. NCCL
 * transfers, share the GPU); NULL deals the tiles round-robin.
 * Replaces clip_sum_exp_kernel (clip_loss.py:9-64), lit_sum_exp_kernel
 * (lit_loss.py:9-62) and the diagonal einsum (clip_loss.py:206).
 */
int meclip_sum_exp(int kind, const void* x_bf16, const void* y_bf16, int64_t rows, int64_t cols, int64_t d,
                   int64_t ldx, int64_t ldy, float temperature, int64_t row_off, int64_t col_off, float* row_sum,
                   float* col_sum, float* diag_s, unsigned int* tile_counter, int* status, void* stream);

/*
 * meclip_sum_exp with sums that are bit-identical from run to run.  The plain entry point adds its per-tile
 * partial sums with fp32 atomics (as the reference does, clip_loss.py:63-64), so the last bits of row_sum, col_sum,
 * the loss and - through the bf16 rounding of single coefficients - the gradients depend on the order in which
 * tiles finish.  Here every partial is stored in a slot of its own (two per column tile for the rows, one per 128
 * rows for the columns) and a second kernel adds the slots in a fixed order onto row_sum / col_sum; together with
 * the backward, which has no atomics, a whole step is then reproducible bit for bit.  Costs the per-tile hand-in
 * of the column partials and one pass over the slots (33.5 MB each at 32768 x 32768).
 * workspace: meclip_sum_exp_det_workspace_bytes(rows, cols) bytes, 256-byte aligned; cleared by the call.
 */
size_t meclip_sum_exp_det_workspace_bytes(int64_t rows, int64_t cols);
int meclip_sum_exp_det(int kind, const void* x_bf16, const void* y_bf16, int64_t rows, int64_t cols, int64_t d,
                       int64_t ldx, int64_t ldy, float temperature, int64_t row_off, int64_t col_off, float* row_sum,
                       float* col_sum, float* diag_s, unsigned int* tile_counter, void* workspace,
                       size_t workspace_bytes, int* status, void* stream);

/*
 * loss_out (+)= scale * sum_i [ w*(log row_sum[i] + log col_sum[i]) - (diag_s[i] - 1)/T ],
 * w = 1/2 and both logs for CLIP; w = 1 and only the row log for LiT.
 * scale = 1/B gives the mean.  Deterministic single-block reduction.
 * Replaces the loss epilogue at clip_loss.py:206-211 / lit_loss.py:199-203.
 */
int meclip_loss_finalize(int kind, const float* row_sum, const float* col_sum, const float* diag_s, int64_t n,
                         float temperature, float scale, int accumulate, float* loss_out, void* stream);

/* Workspace for meclip_grad on a rows x cols block (bytes; 256-byte aligned base expected). */
size_t meclip_grad_workspace_bytes(int64_t rows, int64_t cols, int64_t d);

/*
 * Backward over one rows x cols block.  Recomputes E from X, Y and the saved
 * sums, forms the coefficient matrix
 *   CLIP: G_ij = g * (E_ij/row_sum[i] + E_ij/col_sum[j]) / 2,   LiT: G_ij = g * E_ij/row_sum[i]
 *   G_ii -= g   (the "-Y/(B T)" initialisation of clip_loss.py:235-236 folded in)
 * with g = grad_scale * (*grad_out), panel by panel in bf16, and contracts it:
 *   dX (rows x d) = G Y,     dY (cols x d) = G^T X   (dY is ignored for LiT).
 * Either output may be NULL (a frozen tower): its contraction is skipped.
 * grad_scale is 1/(B*T) (clip_loss.py:182) or 1/sqrt(B*T) for the Stable
 * variants (clip_loss.py:299); B is the GLOBAL batch.  grad_out is a device
 * scalar (no host sync, unlike clip_loss.py:252).  Deterministic: no atomics.
 * Replaces clip_grad_kernel (clip_loss.py:67-156), lit_grad_kernel
 * (lit_loss.py:65-148) and the gradient glue at clip_loss.py:235-254.
 */
int meclip_grad(int kind, const void* x_bf16, const void* y_bf16, int64_t rows, int64_t cols, int64_t d, int64_t ldx,
                int64_t ldy, float temperature, int64_t row_off, int64_t col_off, const float* row_sum,
                const float* col_sum, const float* grad_out, float grad_scale, void* dx, int dx_mode, int64_t lddx,
                void* dy, int dy_mode, int64_t lddy, void* workspace, size_t workspace_bytes, int* status,
                void* stream);

/*
 * fp32 operands multiplied as tf32 (tcgen05 kind::tf32), for callers whose inputs are fp32 and who want the
 * similarities S = X Y^T formed the way the reference's tl.dot forms them on fp32 inputs (clip_loss.py:53, :113)
 * instead of from bf16-rounded operands: 10 mantissa bits per operand instead of 8, at half the tensor rate and
 * twice the operand bytes for the two passes that form S (forward sums, coefficient pass).  The two gradient
 * contractions keep bf16 operands (G is a bf16 panel either way).
 *   meclip_operand_f32   out[r, :] = x[r, :] * inv_norm[r] (inv_norm NULL: x itself), rounded to nearest tf32 and
 *                        stored as fp32 with round_up(d, 8) columns, zeros in the pad: the fp32 operand next to
 *                        the bf16 one of meclip_normalize_fwd.  The tensor cores drop the low 13 mantissa bits of
 *                        what they read, so operands that are not pre-rounded like this are truncated.
 *   meclip_sum_exp_tf32  meclip_sum_exp on fp32 operands (d % 8 == 0, 16-byte aligned, pitches multiples of 4)
 *   meclip_grad_tf32     meclip_grad whose coefficient pass reads x_f32 / y_f32 (pitches ldxf / ldyf); the
 *                        contractions read x_bf16 / y_bf16 as before.  Same workspace.
 * Always the CTA-pair kernel (cta_group::2), 32 elements per K step.
 */
int meclip_operand_f32(const float* x, int64_t rows, int64_t d, int64_t ldx, const float* inv_norm, float* out,
                       int64_t ldo, void* stream);
int meclip_sum_exp_tf32(int kind, const float* x_f32, const float* y_f32, int64_t rows, int64_t cols, int64_t d,
                        int64_t ldx, int64_t ldy, float temperature, int64_t row_off, int64_t col_off, float* row_sum,
                        float* col_sum, float* diag_s, unsigned int* tile_counter, int* status, void* stream);
int meclip_grad_tf32(int kind, const void* x_bf16, const void* y_bf16, const float* x_f32, int64_t ldxf,
                     const float* y_f32, int64_t ldyf, int64_t rows, int64_t cols, int64_t d, int64_t ldx, int64_t ldy,
                     float temperature, int64_t row_off, int64_t col_off, const float* row_sum, const float* col_sum,
                     const float* grad_out, float grad_scale, void* dx, int dx_mode, int64_t lddx, void* dy, int dy_mode,
                     int64_t lddy, void* workspace, size_t workspace_bytes, int* status, void* stream);

/*
 * meclip_grad that also accumulates sum_g_s[0] += sum_ij G_ij S_ij and sum_g_s[1] += sum_ij G_ij
 * over the block (fp32 device
 * two-element array {sum G S, sum G}, zeroed by the caller, fp32 atomics).  With g = grad_scale * (*grad_out) the matrix G
 * satisfies sum_ij G_ij S_ij = g * B * dL/d(1/T), so for the plain scaling (grad_scale = 1/(B T))
 * the temperature gradient is  grad_out * dL/dT = -(1/T) * sum_g_s.  The reference treats the
 * temperature as a constant (backward returns None for it, clip_loss.py:256); this is the
 * learnable-temperature extension.
 */
int meclip_grad_t(int kind, const void* x_bf16, const void* y_bf16, int64_t rows, int64_t cols, int64_t d, int64_t ldx,
                  int64_t ldy, float temperature, int64_t row_off, int64_t col_off, const float* row_sum,
                  const float* col_sum, const float* grad_out, float grad_scale, void* dx, int dx_mode, int64_t lddx,
                  void* dy, int dy_mode, int64_t lddy, float* sum_g_s, void* workspace, size_t workspace_bytes,
                  int* status, void* stream);

/*
 * LiT with the backward's contraction done in the forward.  The LiT coefficients separate,
 * G_ij = g E_ij / r_i - g [i == j], so dX = g (diag(1/r) E Y - Y): one pass that forms E panel by panel
 * and contracts it with [Y | 1] yields U = [E Y | r | 0...] and the whole step costs 4 B^2 D FLOPs
 * instead of the reference's 6 B^2 D (sum kernel lit_loss.py:9-62 + recomputing gradient kernel
 * lit_loss.py:65-148); the backward proper is a row kernel.
 *   meclip_lit_extend          y[i][d] = 1, y[i][d+1..d+7] = 0 in a bf16 matrix with ld >= d + 8
 *   meclip_lit_fused_forward   u [rows x (d+8)] fp32 (=|+=) E [Y_ext]; block offsets as in meclip_grad;
 *                              workspace of meclip_grad_workspace_bytes(rows, cols, d + 8)
 *   meclip_lit_fused_stats     row_sum[i] = u[i][d], diag_s[i] = <x_i, y_i> (feeds meclip_loss_finalize)
 *   meclip_lit_fused_backward  dx[i][0..d) = g (u[i][:] / row_sum[i] - y[i][:]), g = grad_scale * (*grad_out)
 * Used by the single-GPU LiT modules when the first input needs a gradient and the temperature is a
 * constant; the two-pass entry points above remain for everything else.
 */
int meclip_lit_extend(void* y_bf16, int64_t rows, int64_t d, int64_t ldy, void* stream);
int meclip_lit_fused_forward(const void* x_bf16, const void* y_ext_bf16, int64_t rows, int64_t cols, int64_t d, int64_t ldx,
                             int64_t ldy, float temperature, int64_t row_off, int64_t col_off, float* u, int u_mode,
                             int64_t ldu, void* workspace, size_t workspace_bytes, int* status, void* stream);
int meclip_lit_fused_stats(const void* x_bf16, int64_t ldx, const void* y_ext_bf16, int64_t ldy, const float* u, int64_t ldu,
                           int64_t rows, int64_t d, float* row_sum, float* diag_s, void* stream);
int meclip_lit_fused_backward(const float* u, int64_t ldu, const void* y_ext_bf16, int64_t ldy, const float* row_sum,
                              const float* grad_out, float grad_scale, int64_t rows, int64_t d, void* dx, int dx_dtype,
                              int64_t lddx, void* stream);

/*
 * Sigmoid (SigLIP) pairwise loss on the same tile engine; the reference has no such loss.
 *   a_ij = logit_scale * S_ij + logit_bias,   loss = (1/B) sum_ij softplus(-z_ij a_ij),  z_ii = 1, z_ij = -1
 * meclip_siglip_sum:   row_sum[i] += sum_j softplus(-z_ij a_ij) / ln2 over the block (fp32 atomics, zero first),
 *                      diag_s[i] = S_ii where the diagonal crosses the block (as meclip_sum_exp).
 * meclip_siglip_loss_finalize:  loss_out (+)= scale * ln2 * sum_i row_sum[i]  (diag_s, logit_scale and
 *                      logit_bias are accepted for symmetry and not used).
 * meclip_siglip_grad:  G_ij = g (sigmoid(a_ij) - [i == j]),  g = grad_scale * (*grad_out),  grad_scale = t / B;
 *                      dX = G Y, dY = G^T X (either may be NULL); sums (optional, two zeroed floats) receives
 *                      {sum G S, sum G}:  grad_out * dL/dt = sums[0] / t,  grad_out * dL/db = sums[1] / t.
 * Workspace as for meclip_grad (meclip_grad_workspace_bytes).
 */
int meclip_siglip_sum(const void* x_bf16, const void* y_bf16, int64_t rows, int64_t cols, int64_t d, int64_t ldx,
                      int64_t ldy, float logit_scale, float logit_bias, int64_t row_off, int64_t col_off, float* row_sum,
                      float* diag_s, unsigned int* tile_counter, int* status, void* stream);
int meclip_siglip_loss_finalize(const float* row_sum, const float* diag_s, int64_t n, float logit_scale, float logit_bias,
                                float scale, int accumulate, float* loss_out, void* stream);
int meclip_siglip_grad(const void* x_bf16, const void* y_bf16, int64_t rows, int64_t cols, int64_t d, int64_t ldx,
                       int64_t ldy, float logit_scale, float logit_bias, int64_t row_off, int64_t col_off,
                       const float* grad_out, float grad_scale, void* dx, int dx_mode, int64_t lddx, void* dy,
                       int dy_mode, int64_t lddy, float* sums, void* workspace, size_t workspace_bytes, int* status,
                       void* stream);

/*
 * meclip_grad for callers that have no device memory to give: the coefficient panel
 * goes to a 32 MiB (+ 4 KiB of tile counters) scratch array that is part of the
 * library image, so this entry point takes no workspace, never calls cudaMalloc /
 * cudaFree or any other allocating routine, and keeps all its launches on `stream`.  It is meant for hosts that bind the loss as a fixed
 * (inputs, outputs) plugin with no hook for scratch buffers, and for processes whose
 * device memory is already handed out in full to another allocator, where a fresh
 * allocation would fail or stall the device.
 *   - Limit: rows <= 4096 and cols <= 4096 (any d).  Larger blocks return
 *     MECLIP_ENOSPC; use meclip_grad with a workspace for those.
 *   - The scratch stays allocated on every GPU that loads the library, until exit.
 *   - The first call on each device looks up the scratch address (a one-time host-side
 *     set-up with that device current); make that first call before any stream capture.
 *   - All calls on a device share the one array and it keeps the previous call's
 *     contents.  The call clears the tile counters, the only part that must start at
 *     zero; the panel is overwritten before it is read.  Two calls that overlap on
 *     the GPU - different streams, or different host threads on different streams -
 *     race on it: keep them on one stream or order them with events.
 * Arguments and results are those of meclip_grad without workspace/workspace_bytes.
 * This entry point has no counterpart in the reference.
 */
int meclip_grad_static(int kind, const void* x_bf16, const void* y_bf16, int64_t rows, int64_t cols, int64_t d,
                       int64_t ldx, int64_t ldy, float temperature, int64_t row_off, int64_t col_off,
                       const float* row_sum, const float* col_sum, const float* grad_out, float grad_scale, void* dx,
                       int dx_mode, int64_t lddx, void* dy, int dy_mode, int64_t lddy, int* status, void* stream);

/*
 * One-call forward for a whole batch on one GPU: zeroes the sums, runs
 * meclip_sum_exp with offsets 0 and meclip_loss_finalize with scale 1/B.
 * Mirrors MemoryEfficient{CLIP,LiT}LossNormed.forward (clip_loss.py:160-213,
 * lit_loss.py:152-205): X = first argument of apply(), Y = second.
 * row_sum, col_sum (NULL for LiT), diag_s: B floats each, kept for backward.
 * tile_counter: optional device word (cleared by this call), see meclip_sum_exp.
 */
int meclip_loss_forward(int kind, const void* x_bf16, const void* y_bf16, int64_t batch, int64_t d, int64_t ldx,
                        int64_t ldy, float temperature, float* row_sum, float* col_sum, float* diag_s, float* loss_out,
                        unsigned int* tile_counter, int* status, void* stream);

/*
 * One-call backward for a whole batch on one GPU (offsets 0, square block).
 * Mirrors MemoryEfficient{CLIP,LiT}LossNormed.backward (clip_loss.py:215-256,
 * lit_loss.py:207-247); grad_scale selects plain or Stable scaling.
 */
int meclip_loss_backward(int kind, const void* x_bf16, const void* y_bf16, int64_t batch, int64_t d, int64_t ldx,
                         int64_t ldy, float temperature, const float* row_sum, const float* col_sum,
                         const float* grad_out, float grad_scale, void* dx, int dx_mode, int64_t lddx, void* dy,
                         int dy_mode, int64_t lddy, void* workspace, size_t workspace_bytes, int* status, void* stream);

/*
 * A whole training step of the module in two calls, for SMALL batches (up to a few thousand rows), where
 * the step is bound by the host: the general entry points above cost about a dozen library calls, as many
 * small allocations and 17 launches per step, against 0.06 ms of device work at B = 4096, D = 512.
 *   meclip_step_forward   x, y: the module's inputs as they are (fp32 / bf16 / fp16, both the same dtype, any d
 *                         and pitch); normalize != 0 does F.normalize(dim=1) inside (clip_loss.py:266-268).
 *                         Four launches: both inputs -> bf16 operands (one kernel), ONE clear of
 *                         row sums | column sums | diagonal | tile counter, the tile pass, the loss.
 *                         `saved` (meclip_step_saved_bytes, 256-byte aligned) receives everything the backward
 *                         needs: operands, inverse norms, sums.  Replaces clip_loss.py:160-213 + 265-271.
 *   meclip_step_backward  coefficient panel, the two contractions (one stream, no transposed operand copies:
 *                         at these sizes every extra launch costs more than it saves) and the Jacobian of the
 *                         normalisation for both gradients in one kernel; dx / dy get out_dtype (either may be
 *                         NULL).  `workspace`: meclip_step_workspace_bytes.  Replaces clip_loss.py:215-256 and the
 *                         autograd node of F.normalize.
 * Same arithmetic and kernels as the general path; results agree with it to the last bits of the bf16
 * coefficient rounding.  A device-resident temperature is bound as for the other calls.
 */
size_t meclip_step_saved_bytes(int64_t batch, int64_t d);
size_t meclip_step_workspace_bytes(int64_t batch, int64_t d);
int meclip_step_forward(int kind, const void* x, const void* y, int in_dtype, int64_t batch, int64_t d, int64_t ldx,
                        int64_t ldy, int normalize, float temperature, void* saved, size_t saved_bytes, float* loss_out,
                        int* status, void* stream);
int meclip_step_backward(int kind, const void* saved, size_t saved_bytes, int64_t batch, int64_t d, int normalize,
                         float temperature, const float* grad_out, float grad_scale, void* dx, void* dy, int out_dtype,
                         int64_t lddx, int64_t lddy, void* workspace, size_t workspace_bytes, int* status, void* stream);

/*
 * The ring over peer memory for a C caller: one process per GPU of one NVLink box, rank p keeps rows
 * [p*rows, (p+1)*rows) of both arguments.  These two calls queue the whole choreography of one rank (what
 * memoryefficientclip_b200/ring.py does from Python): at ring step s the tile kernels work on shard
 * (rank + s) mod nranks of the second argument while the copy engines fetch the shard of step s + 1 from its
 * owner into one of two local receive buffers (cudaMemcpyAsync on copy_stream, ordered against the kernels on
 * compute_stream with events; no kernel reads a peer's memory and no NCCL kernel is involved, since the
 * persistent tile kernels hold every SM).  The reference has no counterpart (it is single-GPU); a planned
 * signature over an NCCL communicator was dropped for that reason.
 *
 *   meclip_ring_desc   rank, nranks (>= 1); rows per rank; d (multiple of 8), ldx, ldy as for meclip_sum_exp;
 *                      shards[p]: rank p's bf16 shard of the second argument (rows x ldy, contiguous), readable
 *                      from this device: the own one local, the others mapped with meclip_ipc_open;
 *                      recv[0..1]: two local buffers of rows*ldy bf16 (recv[0] may be NULL when nranks <= 2,
 *                      both when nranks == 1); compute_stream, copy_stream: two different streams.
 *   meclip_ring_sum_exp  the forward sums.  Clears and fills row_sum [rows] (complete: all columns), diag_s
 *                      [rows] and, for MECLIP_CLIP, col_part [nranks*rows]: this rank's partial column sums of
 *                      every shard, to be reduce-scattered by the caller (sum over ranks of col_part[p*rows..] =
 *                      rank p's column sums).  tile_counters: nranks device words (cleared by the call).
 *                      Then meclip_loss_finalize(kind, row_sum, col_sum, diag_s, rows, T, 1/(rows*nranks), ...)
 *                      gives this rank's share of the global loss (sum the shares over the ranks).
 *   meclip_ring_grad   the backward.  col_sum_all [nranks*rows]: all column sums (all-gathered by the caller;
 *                      NULL for MECLIP_LIT).  dx_acc [rows x lddx] fp32: cleared, then the complete gradient of
 *                      the first argument's rows.  MECLIP_CLIP only: dy_own [rows x d] fp32 contiguous receives
 *                      the own-shard part of the second argument's gradient; the part computed at step s >= 1
 *                      belongs to rank (rank+s) mod nranks and is copied (copy engines) to
 *                      inbox[that rank] + (s-1)*rows*d floats, from part[s & 1] (two local fp32 buffers of
 *                      rows*d).  inbox[p]: rank p's inbox of (nranks-1)*rows*d floats as seen from this device.
 *                      When EVERY rank's copy_stream has drained (the caller's barrier or collective), the
 *                      owner finishes with meclip_accumulate_many_f32(dy_own, own inbox, nranks-1, rows*d,
 *                      rows*d, stream): partials added in ring-step order, deterministic.
 *                      workspace: meclip_grad_workspace_bytes(rows, rows, d).
 * Ordering between the processes is the caller's: every shard must be in place before the first copy of a
 * call can run (make copy_stream wait for your barrier or collective), a shard or inbox may be overwritten
 * only when all ranks' copies of the previous call have drained.  One ring call at a time per device is
 * queued (the events are shared); a device-resident temperature is bound as for the other calls and
 * applies to every step of the call.
 */
typedef struct meclip_ring_desc {
    int rank, nranks;
    int64_t rows, d, ldx, ldy;
    const void* const* shards;
    void* recv[2];
    void* compute_stream;
    void* copy_stream;
} meclip_ring_desc;
int meclip_ring_sum_exp(const meclip_ring_desc* ring, int kind, const void* x_bf16, float temperature, float* row_sum,
                        float* col_part, float* diag_s, unsigned int* tile_counters, int* status);
int meclip_ring_grad(const meclip_ring_desc* ring, int kind, const void* x_bf16, float temperature, const float* row_sum,
                     const float* col_sum_all, const float* grad_out, float grad_scale, float* dx_acc, int64_t lddx,
                     float* dy_own, float* part0, float* part1, void* const* inbox, void* workspace,
                     size_t workspace_bytes, int* status);

/*
 * Test hook: C (m x n, fp32, ldc) = A * B^T-style contraction through the same
 * tcgen05 mainloop the loss kernels use.  a_mn_major == 0: A is m x k row-major
 * (K contiguous); 1: A is stored k x m row-major (M contiguous).  Same for B
 * with n.  Has no counterpart in the reference; used by the GPU unit tests.
 */
int meclip_debug_gemm(const void* a_bf16, int64_t lda, int a_mn_major, const void* b_bf16, int64_t ldb, int b_mn_major,
                      int64_t m, int64_t n, int64_t k, int tile_n, float* c, int64_t ldc, const float* c_in,
                      int* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MECLIP_H */
