/*
 * mbema.h -- C ABI of libmbema.so: B200 (sm_100a) kernels for MathBrain's Per-Slot-EMA hot path.
 *
 * The reference (Mr-Skeleton-Max/MathBrain) has no FFI: its hot path is a set of Python operators
 * backed by Triton kernels.  Each entry point below names the reference operator it stands in for
 * (path within the reference tree : line).  The Python package mathbrain_b200 binds these symbols
 * with ctypes and re-exports them under the reference's operator names.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless stated otherwise; all tensors are dense, row-major,
 *     innermost dimension contiguous, in the shapes written beside each argument;
 *   - the caller owns every buffer, including `workspace` (size from the matching *_workspace_bytes);
 *     the library allocates nothing and keeps no mutable global state, so calls on different streams
 *     may run concurrently as long as their buffers differ (one exception: mbema_query_scan_static, whose
 *     scratch is a device array inside the library; see there);
 *   - STATUS WORD of the tensor-core entry points (mbema_flash_fwd / _bwd / _rows in MBEMA_MODE_TC_BF16,
 *     mbema_decode_attend_tc): the int32 at the start of `workspace` (the workspace must be 256-byte aligned).
 *     The kernels only ever OR into it and the library never clears it: zero it once, keep passing the same
 *     buffer, and read it at a synchronisation point of your choice.  Non-zero means a bounded wait inside a
 *     kernel gave up (bit 0; bits 8.. name the wait): the outputs of that call and of every later call that
 *     still sees the non-zero word are undefined (their CTAs skip their work).  Zero it again to go on;
 *   - `stream` is a cudaStream_t passed as void*; work is only enqueued, no entry point synchronises;
 *   - the return value is 0 on success, otherwise an MBEMA_ERR_* code (see mbema_strerror); argument
 *     errors are detected before anything is launched;
 *   - dtype codes: MBEMA_F32 = 0, MBEMA_BF16 = 1.
 *
 * State convention (mathbrain/data.py:128-140, tests/test_gold_standard.py:196-221):
 *   the memory state of slot k seen at chunk step t is
 *       M_0[k] = c_base[k],   M_{t+1}[k] = rho * (M_t[k] + [x_t == key_k]).
 */
#ifndef MBEMA_H_
#define MBEMA_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MBEMA_VERSION 200

#define MBEMA_F32 0
#define MBEMA_BF16 1

/* time-tile length of the slot-state snapshots (rows of one attention tile) */
#define MBEMA_TILE_T 128

/* flags */
#define MBEMA_FLAG_SILU 1          /* gate = SiLU(pre); otherwise the gate is linear (use_silu=False)      */
#define MBEMA_FLAG_LISTED_ONLY 2   /* softmax over listed slots only (what the reference's Triton kernel  */
                                   /* computes, mathbrain/triton_flash_ema.py:214-230); default: all       */
                                   /* V_total slots, unlisted ones with score 0 and value 0, as            */
                                   /* mathbrain/flash_ema_attention.py:76-79                               */
#define MBEMA_FLAG_CBASE_EXTRA_DECAY 4 /* M_0 = rho * c_base (mathbrain/triton_flash_ema.py:48-50,185)     */
#define MBEMA_FLAG_FP32_BACKWARD 8     /* MBEMA_MODE_TC_BF16 only: run the backward with the fp32 kernels      */
#define MBEMA_FLAG_INDEX_READY 16      /* mbema_tile_states only: `workspace` still holds the token order that       */
                                       /* mbema_query_scan (or an earlier mbema_tile_states) left there for the SAME  */
                                       /* x, B and T: the sort is skipped, only the links to the listed keys are      */
                                       /* rebuilt (the model calls the scan and the snapshots on the same chunk,      */
                                       /* mathbrain/model.py:157 and :180)                                            */
/* Test hook of the tensor-core forward and backward: one hand-off between the kernel's warps is withheld and the bounded
 * waits give up after a few polls, so the kernel must end through its give-up path (status word set, products in flight
 * drained, TMEM released, outputs undefined).
 * It exists so that this path can be exercised without hanging or faulting a GPU; never set it otherwise. */
#define MBEMA_FLAG_TEST_WITHHOLD_ARRIVE (1 << 30)

/* compute modes of the attention kernels */
#define MBEMA_MODE_FP32 0          /* fp32 arithmetic on the CUDA cores                                    */
#define MBEMA_MODE_TC_BF16 1       /* gate product on tcgen05 tensor cores, bf16 operands, fp32 accumulate */

/* error codes */
#define MBEMA_OK 0
#define MBEMA_ERR_NULL 1
#define MBEMA_ERR_SHAPE 2
#define MBEMA_ERR_UNSUPPORTED 3
#define MBEMA_ERR_WORKSPACE 4
#define MBEMA_ERR_CUDA 5
#define MBEMA_ERR_DTYPE 6
#define MBEMA_ERR_ALIGN 7
#define MBEMA_ERR_STATIC_LIMIT 8

int mbema_version(void);
const char* mbema_strerror(int code);
/* last CUDA runtime error text seen by this thread inside the library (host pointer, never NULL) */
const char* mbema_last_cuda_error(void);

/* ------------------------------------------------------------------------------------------------
 * Query-side per-slot EMA scan.
 * Replaces compute_query_ema_history (mathbrain/triton_ema_query.py:120-169; kernel :11-64).
 *   C_seq[b,t,:] = state of token x[b,t] just before step t; seeded, for every listed key, from
 *   c_init (state seen at step 0); a listed key that occurs more than once in c_init_keys takes the
 *   FIRST entry; key < 0 is ignored.  doc_ids (optional) reset a token's state when the document id
 *   differs from the one at its previous occurrence (:50-57).
 *   x [B,T] i64   rhos [N] f32   c_init [B,K,N] f32 or NULL   c_init_keys [B,K] i64 or NULL
 *   doc_ids [B,T] i32 or NULL    C_seq [B,T,N] f32 (out)
 *   limits: 1 <= T <= 8192, 1 <= N <= 128, tokens in [0, 2^31).
 * ---------------------------------------------------------------------------------------------- */
size_t mbema_query_scan_workspace_bytes(int64_t B, int64_t T);
int mbema_query_scan(const int64_t* x, const float* rhos, const float* c_init, const int64_t* c_init_keys,
                     const int32_t* doc_ids, float* C_seq, int64_t B, int64_t T, int64_t N, int64_t K,
                     int flags, void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Query-side scan for callers that cannot allocate device memory (no counterpart in the reference).
 * Some hosts hand a library nothing but input and output buffers: a serving loop with a fixed memory budget
 * where cudaMalloc (and the device-wide synchronisation it implies) is off limits, or a plugin boundary that
 * offers no allocator at all.  This variant of mbema_query_scan takes no workspace: its index scratch is a fixed
 * array inside the library's device image (about 0.5 MB, resident on every GPU that loads the library until the
 * process exits).  It performs no cudaMalloc / cudaFree and calls no allocating library routine.
 *   limits: B * T <= 32768 tokens and B <= 1024, otherwise MBEMA_ERR_STATIC_LIMIT; all other arguments, limits
 *           and results as mbema_query_scan.
 *   The first call on each device looks up the array's device address (cudaGetSymbolAddress) with that device
 *   current; make that first call outside of any stream capture.
 *   All calls share the one array and it keeps the previous call's contents (nothing in it needs to start at
 *   zero: every entry that is read is written earlier in the same call).  Two calls that overlap on the GPU,
 *   e.g. on different streams, race on it: serialise them.
 * ---------------------------------------------------------------------------------------------- */
int mbema_query_scan_static(const int64_t* x, const float* rhos, const float* c_init, const int64_t* c_init_keys,
                            const int32_t* doc_ids, float* C_seq, int64_t B, int64_t T, int64_t N, int64_t K,
                            int flags, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Slot-state snapshots at the start of every MBEMA_TILE_T-step time tile, plus what the attention
 * kernels need to rebuild the state inside a tile.
 * Replaces precompute_boundaries (mathbrain/triton_flash_ema.py:81-113; kernel :29-78).
 *   unique [B,K] i64 (-1 = not a slot)   c_base [B,K,N] f32 or NULL (zeros)
 *   out: tile_state [B, nT, K, N] f32 with nT = ceil(T / MBEMA_TILE_T), immediately followed in the same buffer
 *                   by the same values in 16 bits [B, nT, K, N] (6 bytes per element in total): fp16 of
 *                   state / 64, saturated (operand of the fp16 gate product)
 *        tok_state  [B, T, N]     f32  state of x[b,t]'s own slot just before step t (0 if unlisted)
 *        kcount     [2B]          i32  [0,B): number of valid (>= 0) entries of unique[b,:];
 *                                       [B,2B): sample indices by decreasing count (launch order of the attention CTAs)
 *   flags: MBEMA_FLAG_CBASE_EXTRA_DECAY.
 * ---------------------------------------------------------------------------------------------- */
size_t mbema_tile_states_workspace_bytes(int64_t B, int64_t T);
int mbema_tile_states(const int64_t* x, const int64_t* unique, const float* rhos, const float* c_base,
                      float* tile_state, float* tok_state, int32_t* kcount, int64_t B, int64_t T, int64_t N,
                      int64_t K, int flags, void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Query gate + LayerNorm, forward and backward.
 * Replaces FusedGatingFunction (mathbrain/triton_fused_gating.py:122-177; kernels :12-57, :61-119).
 *   Y = LayerNorm_eps(x_q * gate(p_pre + bias)) * ln_w + ln_b,  gate = SiLU or identity.
 *   x_q, p_pre [rows, D] (dtype codes)   bias, ln_w, ln_b [D] f32   Y [rows, D] (y_dtype)
 *   mu, rstd [rows] f32 (saved for the backward).   D % 4 == 0, D <= 1024.
 * backward: dY [rows,D] -> dx_q, dp_pre [rows,D] f32;  dbias, dln_w, dln_b [D] f32.
 * ---------------------------------------------------------------------------------------------- */
int mbema_qgate_fwd(const void* x_q, int x_dtype, const void* p_pre, int p_dtype, const float* bias,
                    const float* ln_w, const float* ln_b, float eps, void* Y, int y_dtype, float* mu,
                    float* rstd, int64_t rows, int64_t D, int flags, void* stream);
size_t mbema_qgate_bwd_workspace_bytes(int64_t rows, int64_t D);
int mbema_qgate_bwd(const void* dY, int dy_dtype, const void* x_q, int x_dtype, const void* p_pre, int p_dtype,
                    const float* bias, const float* ln_w, const float* mu, const float* rstd, float* dx_q,
                    float* dp_pre, float* dbias, float* dln_w, float* dln_b, int64_t rows, int64_t D, int flags,
                    void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Flash-EMA gated cross-attention over the listed slots, forward.
 * Replaces FlashEMAFunction.forward / flash_ema_forward / _flash_ema_fwd
 * (mathbrain/triton_flash_ema.py:571-582, :529-568, :121-241); semantics of
 * mathbrain/flash_ema_attention.py:46-82.
 *   Q [B,H,T,hd] (q_dtype)   x [B,T] i64   E_k, E_v [B,K,H*hd] (e_dtype)   W_pe [N,H*hd] f32
 *   rhos [N] f32   unique [B,K] i64   tile_state, tok_state, kcount from mbema_tile_states
 *   seq_lens [B] i32 or NULL: steps >= seq_lens[b] are skipped (O, LSE and dQ are written as zeros there)
 *   out: O [B,H,T,hd] f32, LSE [B,H,T] f32 (log of the softmax normaliser, saved for the backward)
 *   limits: hd == 64; MBEMA_MODE_TC_BF16 needs N in {64, 128}, an even H and a slot list that fits shared memory
 *   (otherwise MBEMA_ERR_UNSUPPORTED; the backward falls back to the fp32 kernels by itself); FP32: N <= 128.
 * ---------------------------------------------------------------------------------------------- */
/* 1 if MBEMA_MODE_TC_BF16 can run the forward for (H heads of 64, N channels, K listed slots), else 0.  The reference
 * chooses between its kernels by itself (mathbrain/model.py:78: `if HAS_TRITON and Q_t.is_cuda`); a caller that wants the
 * same behaviour asks here and passes MBEMA_MODE_FP32 otherwise. */
int mbema_flash_tc_supported(int64_t H, int64_t N, int64_t K);
size_t mbema_flash_fwd_workspace_bytes(int64_t B, int64_t H, int64_t T, int64_t hd, int64_t N, int64_t K, int mode);
int mbema_flash_fwd(const void* Q, int q_dtype, const int64_t* x, const void* E_k, const void* E_v, int e_dtype,
                    const float* W_pe, const float* rhos, const int64_t* unique, const float* tile_state,
                    const float* tok_state, const int32_t* kcount, const int32_t* seq_lens, float* O, float* LSE,
                    int64_t B, int64_t H, int64_t T, int64_t hd, int64_t N, int64_t K, int64_t V_total, int flags,
                    int mode, void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Flash-EMA backward: recomputes state, gate and probabilities tile by tile.
 * Replaces FlashEMAFunction.backward / _flash_ema_bwd_dq_de / _flash_ema_bwd_dw
 * (mathbrain/triton_flash_ema.py:585-650, :250-355, :359-469).
 *   dO [B,H,T,hd] (do_dtype), O and LSE from the forward.
 *   out (all f32, fully overwritten): dQ [B,H,T,hd], dE_k, dE_v [B,K,H*hd], dW_pe [N,H*hd].
 * ---------------------------------------------------------------------------------------------- */
size_t mbema_flash_bwd_workspace_bytes(int64_t B, int64_t H, int64_t T, int64_t hd, int64_t N, int64_t K, int mode);
int mbema_flash_bwd(const void* Q, int q_dtype, const int64_t* x, const void* E_k, const void* E_v, int e_dtype,
                    const float* W_pe, const float* rhos, const int64_t* unique, const float* tile_state,
                    const float* tok_state, const int32_t* kcount, const int32_t* seq_lens, const float* O,
                    const float* LSE, const void* dO, int do_dtype, float* dQ, float* dE_k, float* dE_v,
                    float* dW_pe, int64_t B, int64_t H, int64_t T, int64_t hd, int64_t N, int64_t K,
                    int64_t V_total, int flags, int mode, void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------------------------------
 * The same attention with slot-embedding rows SHARED between samples: E_k, E_v are [e_rows, H*hd] tables and
 * e_row_index [B,K] i32 names the row slot (b, k) reads (for instance one row per token that is listed anywhere in
 * the batch, so that a token's projection is computed once per layer instead of once per sample); dE_k, dE_v are
 * [e_rows, H*hd] f32 and receive the sum over all slots that share a row.  Everything else as mbema_flash_fwd / _bwd.
 * The reference always materialises [B,K,H*hd] (mathbrain/model.py:63-68): this is an extension, the first "next"
 * step around the path.  Entries of e_row_index at padded slots (unique < 0) are not read.
 * ---------------------------------------------------------------------------------------------- */
int mbema_flash_fwd_rows(const void* Q, int q_dtype, const int64_t* x, const void* E_k, const void* E_v, int e_dtype,
                         const int32_t* e_row_index, int64_t e_rows, const float* W_pe, const float* rhos,
                         const int64_t* unique, const float* tile_state, const float* tok_state,
                         const int32_t* kcount, const int32_t* seq_lens, float* O, float* LSE, int64_t B, int64_t H,
                         int64_t T, int64_t hd, int64_t N, int64_t K, int64_t V_total, int flags, int mode,
                         void* workspace, size_t workspace_bytes, void* stream);
int mbema_flash_bwd_rows(const void* Q, int q_dtype, const int64_t* x, const void* E_k, const void* E_v, int e_dtype,
                         const int32_t* e_row_index, int64_t e_rows, const float* W_pe, const float* rhos,
                         const int64_t* unique, const float* tile_state, const float* tok_state,
                         const int32_t* kcount, const int32_t* seq_lens, const float* O, const float* LSE,
                         const void* dO, int do_dtype, float* dQ, float* dE_k, float* dE_v, float* dW_pe, int64_t B,
                         int64_t H, int64_t T, int64_t hd, int64_t N, int64_t K, int64_t V_total, int flags, int mode,
                         void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Slot-gradient scatter: out[slots[r], :] += dE_a[r, :] + dE_b[r, :] for every row r with 0 <= slots[r] < V.
 * Stands in for autograd's backward of F.embedding(safe_unique, E_slots) in mathbrain/model.py:63-64 (the sum, per
 * token, of the gradients of all listed slots that hold it), taking the attention backward's dE_k and dE_v of one
 * layer in one pass.  out is ACCUMULATED (zero it once per step, then call per layer); rows with slots[r] < 0 are
 * skipped.   dE_a, dE_b [R, D] (dtype code; dE_b may be NULL)   slots [R] i64   out [V, D] f32.   D % 8 == 0.
 * Reductions into out are atomic, so the summation order (and the last bits of the result) can differ between runs.
 * ---------------------------------------------------------------------------------------------- */
int mbema_slot_grad_scatter(const void* dE_a, const void* dE_b, int dtype, const int64_t* slots, float* out, int64_t R,
                            int64_t D, int64_t V, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Gather + LayerNorm over distinct slot tokens: out[u, :] = LayerNorm(E[tokens[u], :]) * ln_w + ln_b.
 * Stands in for F.embedding(safe_unique, E_slots) followed by ln_kv (mathbrain/model.py:63-65), computed once per
 * DISTINCT token of the batch (rows for mbema_flash_fwd_rows after the caller's k_proj / v_proj) instead of once per
 * sample and slot.   E [V, D] (dtype code)   tokens [U] i64 (entries outside [0, V) give zero rows)
 * ln_w, ln_b [D] f32   out [U, D] (out dtype code)   mu, rstd [U] f32 (saved for the backward).  D % 4 == 0, D <= 1024.
 * Backward: dY [U, D] -> dE[tokens[u], :] += dx (ACCUMULATED into the [V, D] f32 table: zero it once per step),
 * dln_w, dln_b [D] f32 (ACCUMULATED as well; fp32 atomics, so the last bits depend on the order).
 * ---------------------------------------------------------------------------------------------- */
int mbema_slot_ln_fwd(const void* E, int e_dtype, const int64_t* tokens, const float* ln_w, const float* ln_b, float eps,
                      void* out, int out_dtype, float* mu, float* rstd, int64_t U, int64_t D, int64_t V, void* stream);
int mbema_slot_ln_bwd(const void* dY, int dy_dtype, const void* E, int e_dtype, const int64_t* tokens, const float* ln_w,
                      const float* mu, const float* rstd, float* dE, float* dln_w, float* dln_b, int64_t U, int64_t D,
                      int64_t V, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Chunk-start state of listed slots from RESIDENT per-document state (the layout of the decode entry points below):
 *   c_base[b, k, :] = state[b, v, :] * rho^(t0[b] - last_t[b, v])   for v = slots[b, k] with last_t >= 0, else 0.
 * Stands in for the per-chunk state lookup of the reference's dataset (mathbrain/data.py:128-140), which reads
 * states.bin in a Python loop.   state [B,V,N] f32, last_t [B,V] i32 (-1 = never), slots [B,K] i64 (< 0: zero row),
 * t0 [B] i32 (step of the chunk's first token), rhos [N] f32 -> c_base [B,K,N] f32.
 * ---------------------------------------------------------------------------------------------- */
int mbema_slot_state_gather(const float* state, const int32_t* last_t, const int64_t* slots, const int32_t* t0,
                            const float* rhos, float* c_base, int64_t B, int64_t K, int64_t V, int64_t N, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Softmax cross-entropy over a chunk of logits rows, forward and backward in one launch, IN PLACE:
 *   loss_rows[r] = logsumexp(logits[r, 0:V]) - logits[r, targets[r]]
 *   logits[r, c] <- (softmax(logits[r, 0:V])[c] - [c == targets[r]]) * scale     (columns [V, ld) <- 0)
 * The building block of a chunked tied lm_head + masked cross-entropy (mathbrain/model.py:185-186,
 * train.py:320-323: the reference materialises [B*T, V] logits): GEMM per chunk of valid rows, this kernel, two GEMMs.
 *   logits [R, ld] (dtype code; ld >= V, ld % 8 == 0: every row 16-byte aligned)   targets [R] i64 (outside [0, V):
 *   the row's loss and gradient are zero)   loss_rows [R] f32.
 * ---------------------------------------------------------------------------------------------- */
int mbema_ce_rows(void* logits, int dtype, const int64_t* targets, float scale, float* loss_rows, int64_t R, int64_t V,
                  int64_t ld, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Streaming decode with resident per-sequence slot state.  The reference has no decode loop; one step is one
 * iteration of the loop body of mathbrain/flash_ema_attention.py:46-82 (attention over the slots, then the
 * "+1" of the current token) plus the query-side read of mathbrain/triton_ema_query.py:36-64.
 *   state [B,V,N] f32: value of every slot right after its last update; last_t [B,V] i32: step of that update
 *   (-1 = never); active [B,Kcap] i32 + n_active [B] i32: the slots seen so far.  All caller-owned, resident.
 * mbema_decode_attend: O[b,h,:] = softmax over all V_total slots of q.K/sqrt(hd) times V with
 *   K = E_k * gate(M W_pe), V = E_v * gate(M W_pe), M[v] = state[v] * rho^(t_now - last_t[v]); call it BEFORE
 *   mbema_decode_update of the same step.   q [B,H,64], E_k/E_v [V,H*64] (shared by all sequences), O [B,H,64] f32.
 * mbema_decode_update: C_q[b,:] = M[tok[b]] (query-side state, 0 if never seen), then state[tok] = C_q + 1,
 *   last_t[tok] = t_now, and tok joins the active list.  *overflow is set to 1 if a list is full, 2 if a token
 *   is outside [0, V).
 * ---------------------------------------------------------------------------------------------- */
int mbema_decode_attend(const void* q, int q_dtype, const void* E_k, const void* E_v, int e_dtype, const float* W_pe,
                        const float* rhos, const float* state, const int32_t* last_t, const int32_t* active,
                        const int32_t* n_active, float* O, int64_t B, int64_t H, int64_t hd, int64_t V, int64_t N,
                        int64_t Kcap, int64_t t_now, int64_t V_total, int flags, const int32_t* t_now_dev,
                        void* stream);
/* Tensor-core variant of mbema_decode_attend (16-bit operands, fp32 accumulation; N = 64, hd = 64, H even, E_k/E_v
 * stored as bf16): one walk over the seen slots in 128-slot tiles (tcgen05 gate product, online softmax per CTA, the
 * P.V column sums by a second tcgen05 product), per-CTA partials in the workspace, then a merge kernel that writes O
 * with the softmax over all V_total slots.  Same arguments plus a workspace of
 * mbema_decode_attend_tc_workspace_bytes(B, H, Kcap) bytes; O is written by the call.
 * The int32 at the start of the workspace is the status word described under Conventions. */
size_t mbema_decode_attend_tc_workspace_bytes(int64_t B, int64_t H, int64_t Kcap);
int mbema_decode_attend_tc(const void* q, int q_dtype, const void* E_k, const void* E_v, int e_dtype,
                           const float* W_pe, const float* rhos, const float* state, const int32_t* last_t,
                           const int32_t* active, const int32_t* n_active, float* O, int64_t B, int64_t H, int64_t hd,
                           int64_t V, int64_t N, int64_t Kcap, int64_t t_now, int64_t V_total, int flags,
                           const int32_t* t_now_dev, void* workspace, size_t workspace_bytes, void* stream);
int mbema_decode_update(const int64_t* tok, const float* rhos, float* state, int32_t* last_t, int32_t* active,
                        int32_t* n_active, float* C_q, int32_t* overflow, int64_t B, int64_t V, int64_t N,
                        int64_t Kcap, int64_t t_now, const int32_t* t_now_dev, void* stream);
/* t_now_dev (all three calls above): NULL, or a device int32 holding the step number, which then replaces t_now;
 * with it a whole step (attends, update, mbema_decode_advance) can be captured in a CUDA graph and replayed.
 * mbema_decode_advance adds one to it, ordered on the stream. */
int mbema_decode_advance(int32_t* t_now_dev, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MBEMA_H_ */
