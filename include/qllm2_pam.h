/*
 * qllm2_pam.h -- C ABI of libqllm2_pam_b200.so: the Phase-Associative-Memory (PAM) hot path
 * of QLLM (reference project gowrav-vishwakarma/qllm2, directory v11/) as hand-written CUDA
 * for NVIDIA B200 (sm_100a).
 *
 * The reference has no FFI layer: its operator surface for this path is a set of Python
 * functions operating on torch tensors.  Each entry point below names the reference function
 * (file:line inside that project) whose arithmetic it replaces.  A maintainer binds these with
 * ctypes (tensor.data_ptr(), torch.cuda.current_stream().cuda_stream).
 *
 * Conventions
 *   - every pointer is a DEVICE pointer owned by the caller; nothing is allocated or freed here
 *   - complex numbers are split-real: innermost axis of length 2, re at 0, im at 1
 *     (v11/complex_ops.py:4-11)
 *   - every function returns 0 on success, a QPAM_E* code otherwise; it never throws/aborts.
 *     qpam_last_error() returns a thread-local, human-readable message for the last failure.
 *   - work is enqueued on `stream` (a cudaStream_t passed as void*); calls are asynchronous.
 *   - functions are re-entrant for distinct streams and distinct output/workspace buffers.
 */
#ifndef QLLM2_PAM_H
#define QLLM2_PAM_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define QPAM_OK 0
#define QPAM_EINVAL 1      /* bad argument (shape, dtype, null pointer, alignment) */
#define QPAM_EWORKSPACE 2  /* workspace too small */
#define QPAM_ECUDA 3       /* a CUDA runtime call failed; see qpam_last_error() */
#define QPAM_EUNSUPPORTED 4

#define QPAM_F32 0
#define QPAM_BF16 1

#define QPAM_MAX_STATES 4  /* K, number of superposed states */

/* ------------------------------------------------------------------------------------------
 * Chunked dual-form scan (training / prefill).
 *
 * Replaces V11PAMLayer._forward_chunked_head (v11/model.py:378-417), _dual_form_block
 * (:354-376), fused_decay_matrix (v11/triton_kernels.py:522-528,570-573), and for K>1
 * _fused_chunk_step / _forward_multistate_fused (v11/model.py:657-781);
 * flash_pam_chunked_head (v11/flash_pam.py:56-152) computes the same function.
 *
 *   S^k_t = (gamma^k_t + gamma_eps) S^k_{t-1} + v_t (x) conj(k_t)
 *   y_t   = sum_k coef_{k,t} * S^k_t (q_t * q_scale)
 *
 * Token tensors q,k,v,y,dy,dq,dk,dv: [B,H,T,d,2] contiguous, dtype io_dtype.
 * Packed ragged mode (cu_seqlens != NULL): B must be 1, T is the packed total, the layout is
 * [H,T,d,2]; cu_seqlens is int32[S+1] on the device, the state restarts at each boundary.
 * Without cu_seqlens there are S = B sequences of T tokens each.
 * gamma: fp32 [K,B,H,T].  coef: fp32 [K,B,H,T,2] or NULL (== 1).
 * s0 / s_final / ds_final / ds0: fp32 [K,S,H,d,d,2] (state[i][j]: i value channel, j key
 * channel, v11/model.py:939-947) or NULL.
 * d in {16,32,64}; 1 <= K <= QPAM_MAX_STATES.  `chunk` is accepted for interface
 * compatibility only: the result of the scan does not depend on the chunk length and the
 * kernels use their own tile (64 tokens in the fp32-math kernels, 128 in the tensor-core ones).
 * cu_seqlens is checked on the device: see qpam_device_status, code 301.
 * ------------------------------------------------------------------------------------------ */
typedef struct {
  const void* q;
  const void* k;
  const void* v;
  const float* gamma;
  const float* coef;
  const float* s0;
  const int32_t* cu_seqlens;
  void* y;
  float* s_final;
  void* workspace;        /* >= qpam_scan_workspace_bytes(args, ..); 256-byte aligned */
  size_t workspace_bytes;
  int32_t B, H, T, d, K, S;
  int32_t chunk;
  int32_t io_dtype;       /* QPAM_F32 | QPAM_BF16 */
  float q_scale;          /* d^-0.5 in the reference (v11/model.py:381) */
  float gamma_eps;        /* 1e-6 in the reference (v11/model.py:396) */
} qpam_scan_args;

/* Bytes of workspace: forward only (with_backward = 0) or forward + backward (1). */
size_t qpam_scan_workspace_bytes(const qpam_scan_args* args, int32_t with_backward);

/* Forward.  Leaves the per-chunk carried states in `workspace`; a following
 * qpam_scan_bwd with the SAME workspace contents may pass states_valid=1 to reuse them. */
int qpam_scan_fwd(const qpam_scan_args* args, void* stream);

/* qpam_scan_fwd with y written token-major, [B,T,H,d,2] (packed mode: [T_total,H,d,2]): the head merge
 * that precedes the output projection (v11/model.py:835-836) without a transpose pass.  Forward only;
 * available where the tensor-core kernels run (bf16, d = 64), QPAM_EUNSUPPORTED otherwise. */
int qpam_scan_fwd_tokens(const qpam_scan_args* args, void* stream);

/* Forward scan with no workspace argument, for hosts that are not allowed to allocate device
 * memory: a server whose memory pool took the whole GPU at start-up, a sandboxed plugin, or a
 * latency-critical loop where cudaMalloc (which may synchronise the device) is forbidden.  The
 * workspace lives in a QPAM_STATIC_SCRATCH_BYTES array inside the library image; every GPU that
 * loads the library holds that much memory until the process exits.  `workspace` and
 * `workspace_bytes` of `args` are ignored; all other fields mean what they mean for
 * qpam_scan_fwd and the results are identical.  Shapes whose forward workspace
 * (qpam_scan_workspace_bytes(args, 0)) exceeds the array are refused with QPAM_EWORKSPACE.
 * The first call on each device looks up the array's device address (device must be current;
 * make that first call before any stream capture).  No cudaMalloc/cudaFree is issued.  All calls
 * share the one array: it keeps the previous call's contents (every byte that is read is
 * written first, so nothing needs clearing) and two calls that overlap on the GPU -- different
 * streams or processes' threads -- race on it.  The backward pass is not offered in this form.
 * This entry point has no counterpart in the reference. */
#define QPAM_STATIC_SCRATCH_BYTES (32u << 20)
int qpam_scan_fwd_static(const qpam_scan_args* args, void* stream);

/* Backward of qpam_scan_fwd w.r.t. q, k, v, gamma (and coef when coef != NULL).
 * Replaces torch autograd through the functions above, including _FusedDecayMatrixFn.backward
 * (v11/triton_kernels.py:447-480).  Exact for gamma + gamma_eps <= 1.
 * dgamma fp32 [K,B,H,T]; dcoef fp32 [K,B,H,T,2] or NULL; ds_final (gradient reaching
 * s_final) and ds0 (gradient w.r.t. s0, output) may be NULL. */
int qpam_scan_bwd(const qpam_scan_args* args, const void* dy, void* dq, void* dk, void* dv,
                  float* dgamma, float* dcoef, const float* ds_final, float* ds0,
                  int32_t states_valid, void* stream);

/* qpam_scan_bwd for one state with dq, dk, dv ADDED to the values the buffers already hold (dgamma, ds0 are
 * written as usual).  The K phase-routed states of a layer (v11/model.py:657-781) are K scans over the same
 * q, k, v whose gradients sum (autograd does that sum in the reference): the first state's backward writes, the
 * others accumulate, with the additions done by the copy engine (TMA reduce).  Offered where the tensor-core
 * kernels run (bf16, d = 64, K = 1 per call, no coef); QPAM_EUNSUPPORTED otherwise. */
int qpam_scan_bwd_accumulate(const qpam_scan_args* args, const void* dy, void* dq, void* dk, void* dv,
                             float* dgamma, const float* ds_final, float* ds0, int32_t states_valid, void* stream);

/* K = 2..4 phase-routed states for TRAINING (tensor-core path: bf16, d = 64; QPAM_EUNSUPPORTED otherwise): the per-state
 * outputs ys [K,B,H,T,d,2] (args->y and args->coef are ignored; the caller forms y = sum_k c_k ys_k, v11/model.py:766-781)
 * and s_final [K,S,H,d,d,2].  The chunk sums of all states come from one pass over k and v
 * (the reference's fused step shares the same products, v11/model.py:657-737); the workspace (sized with
 * qpam_scan_workspace_bytes(args, 1)) keeps every state's chunk states for qpam_scan_bwd_state. */
int qpam_scan_fwd_states(const qpam_scan_args* args, void* ys, void* stream);

/* Backward of state `state` of a qpam_scan_fwd_states call (same args, same workspace): dy is the gradient of that state's
 * output, dgamma [B,H,T] / ds_final / ds0 are that state's arrays; accumulate != 0 adds dq, dk, dv to what the buffers
 * hold (the states share q, k, v: call state 0 with accumulate = 0, the others with 1). */
int qpam_scan_bwd_state(const qpam_scan_args* args, int32_t state, const void* dy, void* dq, void* dk, void* dv,
                        float* dgamma, const float* ds_final, float* ds0, int32_t accumulate, void* stream);

/* ------------------------------------------------------------------------------------------
 * O(1) recurrent decode step over a pool of per-sequence state slots.
 *
 * Replaces V11PAMLayer._recur_step_additive (v11/model.py:927-965) and the K-state loop of
 * _recurrent (:874-906):  S <- gamma S + v (x) conj(k);  y = sum_k coef_k S^k q
 * (note: gamma is used as is, without gamma_eps, exactly as the reference's recurrent path).
 *
 * state_pool: [n_slots, L, K, H, d, d, 2] (state_dtype); the step updates, in place, layer
 * `layer` of the slots named by slot_ids[n].  q (already scaled by d^-0.5), k, v, y: [n,H,d,2]
 * io_dtype.  gamma fp32 [K,n,H]; coef fp32 [K,n,H,2] or NULL.
 * ------------------------------------------------------------------------------------------ */
int qpam_decode_step(void* state_pool, int32_t state_dtype, int64_t n_slots, int32_t L, int32_t layer,
                     const int32_t* slot_ids, const void* q, const void* k, const void* v,
                     const float* gamma, const float* coef, void* y, int32_t n, int32_t H, int32_t d,
                     int32_t K, int32_t io_dtype, void* stream);

/* Copy final prefill states [K,S,H,d,d,2] fp32 into pool slots (sequence s -> slot_ids[s]). */
int qpam_pool_store(void* state_pool, int32_t state_dtype, int64_t n_slots, int32_t L, int32_t layer,
                    const int32_t* slot_ids, const float* states, int32_t S, int32_t H, int32_t d,
                    int32_t K, void* stream);

/* ------------------------------------------------------------------------------------------
 * Fused tied complex LM head + cross-entropy.
 *
 * Replaces _FusedLinearCE.forward/backward and fused_linear_cross_entropy
 * (v11/fused_ce.py:26-94), linear_ce_per_token (:97-115), linear_ce_stats (:118-141) and the
 * tied head of V11LM (v11/model.py:1136-1139,1175-1190):
 *     logits = [lm_r | lm_i] @ [E_r | E_i]^T = h @ w^T,   h [N,F], w [V,F], F = 2*dim.
 * The [N,V] logits are never written to memory.
 *
 * Vocabulary-parallel use: w holds rows [v_offset, v_offset+V) of the full matrix; targets are
 * GLOBAL ids.  qpam_ce_partial writes per-row (max, sum exp(z-max), target logit or 0,
 * argmax value, argmax index) for the local shard; the caller combines shards (all-gather or
 * all-reduce), then qpam_ce_finalize turns combined stats into lse/loss, and qpam_ce_bwd
 * produces local dW and a partial dH that the caller all-reduces.
 * ------------------------------------------------------------------------------------------ */
typedef struct {
  const void* h;          /* [N,F] io_dtype */
  const void* w;          /* [V,F] io_dtype */
  const int64_t* targets; /* [N] global ids; == ignore_index => row ignored */
  const float* mask;      /* [N] or NULL */
  int64_t N, V, v_offset;
  int32_t F;
  int32_t io_dtype;
  int64_t ignore_index;
  void* workspace;        /* >= qpam_ce_workspace_bytes(args, with_backward) */
  size_t workspace_bytes;
} qpam_ce_args;

size_t qpam_ce_workspace_bytes(const qpam_ce_args* args, int32_t with_backward);

/* Per-row shard statistics, each fp32/int64 [N]:
 * row_max, row_sumexp (relative to row_max), row_tgt (target logit if the shard owns the
 * target column, else 0), row_argmax (global column of the largest logit; lowest index wins
 * ties). */
int qpam_ce_partial(const qpam_ce_args* args, float* row_max, float* row_sumexp, float* row_tgt,
                    int64_t* row_argmax, void* stream);

/* From combined stats: lse[N] = max + log(sumexp); per_token[N] = (lse - tgt) or 0 when ignored;
 * loss_sum[0] = sum per_token*mask; denom[0] = valid count or mask sum, clamped to >= 1;
 * correct[0] = sum token_mask * [argmax == target] and tokens[0] = sum token_mask, with
 * token_mask = mask if given else [target != ignore_index] (linear_ce_stats).
 * Any output may be NULL except lse. */
int qpam_ce_finalize(const qpam_ce_args* args, const float* row_max, const float* row_sumexp,
                     const float* row_tgt, const int64_t* row_argmax, float* lse, float* per_token,
                     float* loss_sum, float* denom, float* correct, float* tokens, void* stream);

/* Gradients: dh [N,F], dw [V,F] (io_dtype) of  grad_scale[0] * loss_sum / denom[0]
 * given lse from qpam_ce_finalize.  grad_scale and denom are device scalars. */
int qpam_ce_bwd(const qpam_ce_args* args, const float* lse, const float* grad_scale,
                const float* denom, void* dh, void* dw, void* stream);

/* Same as qpam_ce_bwd; in addition `dh_ready_stream` (a CUDA stream of the caller, may be NULL) is made to wait
 * until dh is complete, while the products for dw are still running on `stream`.  The vocabulary-parallel
 * form enqueues its all-reduce of dh (v11/fused_ce.py:80 computes the same grad_H on one device) on that
 * stream, so the exchange over NVLink overlaps the dw GEMM.  The caller joins the two streams afterwards. */
int qpam_ce_bwd_overlap(const qpam_ce_args* args, const float* lse, const float* grad_scale,
                        const float* denom, void* dh, void* dw, void* stream, void* dh_ready_stream);

/* Decode head: argmax_v (h @ w^T)[n, v] -> ids[N] (int64) and the winning logit (fp32). */
int qpam_head_argmax(const qpam_ce_args* args, int64_t* ids, float* best, void* stream);

/* Sampling decode head: logits[n, v] = (h @ w^T)[n, v] as bf16 rows of `ld` elements (ld >= V, a multiple of 8;
 * `logits` 16-byte aligned) -- the tied-head product that V11LM.generate forms before its sampling block
 * (v11/model.py:1218-1221), on the tensor-core GEMM of the cross-entropy (bf16 h and w with 16-byte aligned rows
 * only: QPAM_EUNSUPPORTED otherwise).  targets / mask / workspace of `args` are not used. */
int qpam_head_logits(const qpam_ce_args* args, void* logits, int64_t ld, void* stream);

/* Token sampling on the device, one row of logits per sequence: the sampling block of V11LM.generate
 * (v11/model.py:1221-1244) -- logits / temperature, repetition penalty over the tokens already in the sequence
 * (x > 0 ? x / penalty : x * penalty), top-k (values below the k-th largest dropped, ties kept), top-p (in
 * descending order a token is dropped when the probability mass before it is >= top_p; tokens that tie with the
 * threshold are all kept), then one draw from the softmax of what is left -- as ONE kernel, without a sort and
 * without a host round trip.  The draw is the inverse CDF in vocabulary order of uniforms[row] in [0,1), which
 * the caller supplies (the reference draws with torch.multinomial: same distribution, different stream of random
 * numbers).  top_k == 0 and top_p == 0 (or >= 1) switch the filters off, repetition_penalty == 1 the penalty.
 *   logits      [n, V] (row stride ld_logits), fp32 or bf16
 *   history     optional int64 [n_hist_rows, ld_hist]: token ids of every sequence so far; row r of the logits
 *               uses history row slot_ids[r] (or r when slot_ids is NULL; a slot outside [0, n_hist_rows) marks a
 *               padded row, which draws nothing and returns id 0); hist_len optional int32 [n_hist_rows]
 *               (NULL: all hist_cols entries count); append != 0 stores the drawn id at history[row][hist_len]
 *               and increments hist_len
 *   next_ids    int64 [n];  stats optional float [n,4] = (max, kept mass, kept count, mass after top-k)
 *   workspace   qpam_sample_workspace_bytes(n, V) bytes (0 while a row fits in shared memory, V <= ~56k) */
size_t qpam_sample_workspace_bytes(int32_t n, int32_t V);
int qpam_sample_logits(const void* logits, int32_t io_dtype, int32_t n, int32_t V, int64_t ld_logits,
                       float temperature, int32_t top_k, float top_p, float repetition_penalty,
                       const int32_t* slot_ids, int64_t* history, int32_t n_hist_rows, int32_t hist_cols,
                       int64_t ld_hist, int32_t* hist_len, int32_t append, const float* uniforms,
                       int64_t* next_ids, float* stats, void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------------------------
 * Fused element-wise complex operators of a V11 block (interleaved [..., C, 2] rows, N rows).
 * They replace the reference's fused operators and their autograd functions:
 *   qpam_cnorm_*     fused_complex_norm   v11/triton_kernels.py:48-80, 209-263, 489-494
 *   qpam_modact_*    fused_mod_swish (beta != NULL) / fused_mod_relu (beta == NULL)
 *                                          v11/triton_kernels.py:82-137, 266-361, 497-508
 *   qpam_cgu_gate_*  fused_cgu_gate        v11/triton_kernels.py:139-166, 364-417, 511-519
 *   qpam_pam_prep_*  the head split, rotary rotation and protect-gate scaling of
 *                    PhaseAssociativeLayer._project / _gamma_and_vprime (v11/model.py:271-350)
 * Parameters (scale, bias, beta, rope, omp) are fp32.  Parameter gradients come back as P partial
 * rows [P, C] that the caller sums over P.  C must be a multiple of 4; rows must be 16-byte
 * aligned.  ld_* are row strides in scalars, so gate/up (and their gradients) may be column
 * blocks of one wider matrix.
 * ------------------------------------------------------------------------------------------ */
/* out = z/(|z|+1e-8) * (|z|/rms) * scale, |z| = sqrt(re^2+im^2+1e-8), rms = sqrt(mean|z|^2 + eps).
 * dtypes: f32->f32, f32->bf16, bf16->bf16.  D <= 3072. */
int qpam_cnorm_fwd(const void* z, int32_t z_dtype, const float* scale, void* out, int32_t out_dtype,
                   int64_t N, int32_t D, float eps, void* stream);
/* P (a multiple of 4) partial rows of d(scale); dz has z's dtype, dout out's. */
int qpam_cnorm_bwd(const void* z, int32_t z_dtype, const float* scale, const void* dout,
                   int32_t out_dtype, void* dz, float* dscale_partials, int32_t P, int64_t N,
                   int32_t D, float eps, void* stream);
int qpam_modact_fwd(const void* z, int32_t dtype, const float* bias, const float* beta, void* out,
                    int64_t N, int32_t C, void* stream);
/* 1 <= P <= min(N, 65535) partial rows of d(bias) and (modSwish) d(beta). */
int qpam_modact_bwd(const void* z, int32_t dtype, const float* bias, const float* beta,
                    const void* dout, void* dz, float* dbias_partials, float* dbeta_partials,
                    int32_t P, int64_t N, int32_t C, void* stream);
/* out = gate/(|gate|+1e-8) * up * sigmoid(|gate|)  (complex product), out dense [N, C, 2]. */
int qpam_cgu_gate_fwd(const void* gate, int64_t ld_gate, const void* up, int64_t ld_up, int32_t dtype,
                      void* out, int64_t N, int32_t C, void* stream);
int qpam_cgu_gate_bwd(const void* gate, int64_t ld_gate, const void* up, int64_t ld_up,
                      const void* dout, int32_t dtype, void* dgate, int64_t ld_dgate, void* dup,
                      int64_t ld_dup, int64_t N, int32_t C, void* stream);
/* qkv [B,T,3,H,d,2] -> q,k,v [B,H,T,d,2]:  q,k *= rope[pos] (rope fp32 [rope_len,d,2] = cos,sin;
 * NULL = no rotation), v *= omp[b,t,h] (fp32 [B,T,H]; NULL = 1).  pos = positions[b,t] (int64,
 * clamped to the table) or offset + t when positions is NULL.  d a power of two in [4,128]. */
int qpam_pam_prep_fwd(const void* qkv, int32_t dtype, const float* rope, int64_t rope_len,
                      const int64_t* positions, int64_t offset, const float* omp, void* q, void* k,
                      void* v, int32_t B, int32_t T, int32_t H, int32_t d, void* stream);
/* dqkv [B,T,3,H,d,2] and, when omp is given, domp [B,T,H] (fp32). */
int qpam_pam_prep_bwd(const void* qkv, int32_t dtype, const float* rope, int64_t rope_len,
                      const int64_t* positions, int64_t offset, const float* omp, const void* dq,
                      const void* dk, const void* dv, void* dqkv, float* domp, int32_t B, int32_t T,
                      int32_t H, int32_t d, void* stream);

/* ------------------------------------------------------------------------------------------
 * Forward-only block fusions for inference (prefill and the per-token decode step driven by
 * V11LM.generate, v11/model.py:1206-1245), where nothing is kept for a backward pass.
 * ------------------------------------------------------------------------------------------ */
/* gate_up [N, ld]: columns [0,2C) = gate, [2C,4C) = up (interleaved complex), one projection output.
 * out [N,C,2] = gate/(|gate|+1e-8) * act(up) * sigmoid(|gate|), act = modSwish (beta != NULL) or
 * modReLU (ComplexGatedUnit.forward, v11/complex_ops.py:175-220). */
int qpam_act_gate_packed_fwd(const void* gate_up, int64_t ld, int32_t dtype, const float* bias,
                             const float* beta, void* out, int64_t N, int32_t C, void* stream);
/* z [N,D,2] += res_scale[0] * delta (delta NULL: unchanged; res_scale NULL: 1), then
 * xn = ComplexNorm(z; norm_scale) (xn NULL: skipped) and mag [N,D] = |xn| (NULL: skipped).
 * The residual add and the pre-norm of V11Block.forward (v11/model.py block forward). */
int qpam_residual_cnorm_fwd(void* z, const void* delta, const float* res_scale, const float* norm_scale,
                            void* xn, void* mag, int32_t dtype, int64_t N, int32_t D, float eps,
                            void* stream);
/* Input stage of the PAM layer from projection outputs (row strides ld_* in scalars):
 *   qkv   [B*T, ld_qkv]  first 3*H*d*2 columns = (q|k|v, head, channel, re/im)
 *   dt    [B*T, ld_dt]   H decay logits            (dt_proj output incl. its bias)
 *   pg    [B*T, ld_pg]   H protect-gate logits     (NULL: no protect gate)
 *   phase [B*T, ld_phase] H*K routing phases, (h,k) order (NULL: 0)
 *   score [B*T, ld_score] H*K routing scores       (NULL: uniform weights 1)
 * Outputs: q (times q_scale), k rotated by rope[pos]; v' = (1-p) v, all [B,H,T,d,2];
 *   gamma [K,B,H,T] fp32 = base (1-p) + p, base = exp(-softplus(dt + dt_bias[h] + state_dt_offset[k]))
 *   (gamma_floor applied to base); coef [K,B,H,T,2] fp32 = K softmax_k(score) e^{i phase} (NULL when K == 1).
 * (PhaseAssociativeLayer._project, _gamma_and_vprime and the phase routing, v11/model.py:271-350, 630-655.) */
typedef struct qpam_front_args {
  const void *qkv, *dt, *pg, *phase, *score;
  int64_t ld_qkv, ld_dt, ld_pg, ld_phase, ld_score;
  const float* dt_bias;          /* [H] */
  const float* state_dt_offset;  /* [K] or NULL */
  const float* rope;             /* [rope_len, d, 2] (cos, sin) or NULL */
  const int64_t* positions;      /* [B*T] or NULL: offset + t */
  int64_t rope_len, offset;
  void *q, *k, *v;
  float* gamma;
  float* coef;
  float gamma_floor, q_scale;
  int32_t B, T, H, d, K, io_dtype;
} qpam_front_args;
int qpam_pam_front_fwd(const qpam_front_args* args, void* stream);

/* Residual with a learnable scalar (V11Block.forward: x + mixed * cgu_scale, x + pam_out * pam_scale):
 * out[i] = x[i] + scale[0] * delta[i] over n scalars (n a multiple of 4; x/out and delta may differ in
 * dtype).  Backward: ddelta = scale[0] * dout, dscale = sum of the P partials, d(x) = dout. */
int qpam_scaled_residual_fwd(const void* x, int32_t x_dtype, const void* delta, int32_t d_dtype,
                             const float* scale, void* out, int64_t n, void* stream);
int qpam_scaled_residual_bwd(const void* dout, int32_t x_dtype, const void* delta, int32_t d_dtype,
                             const float* scale, void* ddelta, float* dscale_partials, int32_t P,
                             int64_t n, void* stream);
/* Real block form of a complex weight (ComplexLinear.forward, v11/complex_ops.py): w [2*out, 2*in] with
 * rows (o,re) = (Wr, -Wi) and (o,im) = (Wi, Wr) over interleaved (j,re),(j,im) columns, so that one real GEMM
 * on interleaved activations is the complex product.  Backward folds dw into dWr, dWi. */
int qpam_block_weight_fwd(const void* wr, const void* wi, int32_t w_dtype, void* w, int32_t out_dtype,
                          int32_t out_dim, int32_t in_dim, void* stream);
int qpam_block_weight_bwd(const void* dw, int32_t out_dtype, void* dwr, void* dwi, int32_t w_dtype,
                          int32_t out_dim, int32_t in_dim, void* stream);

/* Gate arithmetic of the PAM layer from the outputs of its small Linears, all fp32 (v11/model.py:308-350,
 * 630-655, 685-720): dt, pg [B,T,H]; phase, score [B,T,H,K]; pg / phase / score / state_dt_offset may be NULL.
 *   gamma[k,b,h,t] = base'_k (1-p) + p,  base_k = exp(-softplus(dt + dt_bias[h] + state_dt_offset[k])),
 *   base' = gamma_floor + (1-gamma_floor) base,  p = sigmoid(pg);  omp[b,t,h] = 1-p;
 *   coef[k,b,h,t] = K softmax_k(score) e^{i phase_k}   (coef NULL: not produced).
 * Backward: d(dt), d(pg), d(phase), d(score) and P rows of partial sums of d(x_k) [P,H,K], whose sum over P
 * and K is d(dt_bias) and over P and H is d(state_dt_offset). */
int qpam_pam_gates_fwd(const float* dt, const float* pg, const float* phase, const float* score,
                       const float* dt_bias, const float* state_dt_offset, float gamma_floor,
                       float* gamma, float* omp, float* coef, int32_t B, int32_t T, int32_t H, int32_t K,
                       void* stream);
int qpam_pam_gates_bwd(const float* dt, const float* pg, const float* phase, const float* score,
                       const float* dt_bias, const float* state_dt_offset, float gamma_floor,
                       const float* dgamma, const float* domp, const float* dcoef, float* ddt, float* dpg,
                       float* dphase, float* dscore, float* dx_partials, int32_t P, int32_t B, int32_t T,
                       int32_t H, int32_t K, void* stream);

/* mag[i] = sqrt(re_i^2 + im_i^2 + 1e-8) over n complex values (n a multiple of 4), the input of the
 * magnitude-driven gate and routing Linears (v11/model.py:330-349, 640-655); backward dz = dmag z / |z|. */
int qpam_cmagnitude_fwd(const void* z, int32_t dtype, void* mag, int64_t n, void* stream);
int qpam_cmagnitude_bwd(const void* z, const void* dmag, int32_t dtype, void* dz, int64_t n, void* stream);

/* Read-out of K phase-routed states (v11/model.py:766-781: the sum over states weighted by
 * alpha_k e^{i phi_k}):  y[r,:] = sum_k coef[k,r] * yk[k][r,:] over R rows of d complex channels;
 * yk / dyk are HOST arrays of K device pointers, coef / dcoef fp32 [K,R,2].
 * Backward: dyk[k] = conj(coef[k]) dy,  dcoef[k,r] = sum_j dy[r,j] conj(yk[k][r,j]). */
int qpam_state_combine_fwd(const void* const* yk, const float* coef, void* y, int32_t dtype, int32_t K,
                           int64_t R, int32_t d, void* stream);
/* Forward only, inputs [B,H,T,d,2], output token-major [B,T,H,d,2]: the head merge before o_proj
 * (v11/model.py:835-836) folded into the read-out. */
int qpam_state_combine_tokens_fwd(const void* const* yk, const float* coef, void* y, int32_t dtype,
                                  int32_t K, int32_t B, int32_t H, int32_t T, int32_t d, void* stream);
int qpam_state_combine_tokens_bwd(const void* const* yk, const float* coef, const void* dy, void* const* dyk,
                                  float* dcoef, int32_t dtype, int32_t K, int32_t B, int32_t H, int32_t T,
                                  int32_t d, void* stream);   /* dy token-major, dyk [B,H,T,d,2] */
int qpam_state_combine_bwd(const void* const* yk, const float* coef, const void* dy, void* const* dyk,
                           float* dcoef, int32_t dtype, int32_t K, int64_t R, int32_t d, void* stream);

/* ------------------------------------------------------------------------------------------
 * Launch accounting and per-kernel timing.  The reference times whole calls with
 * time.perf_counter around torch.cuda.synchronize (v11/bench_flash_pam.py:73-84); these entry
 * points give the per-kernel split of the same calls.
 *   qpam_launch_count  kernels launched by this library in this process so far
 *   qpam_profile_begin records a base event on `stream` and starts recording one event behind
 *                      every kernel this library launches (all calls must use that stream)
 *   qpam_profile_end   stops recording, waits for the last event and writes one line per kernel
 *                      "name launches total_ms\n" into buf; the time of a kernel is the gap
 *                      between its event and the previous one on the stream
 * ------------------------------------------------------------------------------------------ */
long long qpam_launch_count(void);
int qpam_profile_begin(void* stream);
int qpam_profile_end(char* buf, size_t buf_bytes);

/* Status word written by the kernels: 0 = ok.  Non-zero values:
 *   2xx  a bounded on-device wait (mbarrier) gave up: the outputs of that launch are invalid, and every
 *        tensor-core scan launch that starts while the word is set returns without touching its outputs;
 *   301  a packed-mode scan was given a cu_seqlens descriptor that does not start at 0, decreases, or ends
 *        beyond T: no kernel of that call read or wrote through it, its outputs are untouched.
 * Synchronises the device.  clear != 0 resets the word.  Callers should read it at a point where they
 * synchronise anyway (once per optimizer step, once per decode step).  (No counterpart in the reference.) */
int qpam_device_status(int32_t* status, int32_t clear);

/* Diagnostic: launches one thread that waits on an mbarrier nobody arrives at and gives up after limit_ns
 * (0 < limit_ns <= 1e8), leaving 299 in the status word -- the give-up path of every bounded wait in this
 * library, exercised without hanging or faulting anything.  (No counterpart in the reference.) */
int qpam_selftest_wait_expiry(int64_t limit_ns, void* stream);

const char* qpam_last_error(void);
/* "qllm2_pam_b200 <version> sm_100a" */
const char* qpam_version(void);

#ifdef __cplusplus
}
#endif
#endif /* QLLM2_PAM_H */
