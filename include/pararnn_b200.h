/*
 * pararnn_b200 — C ABI of the B200 (sm_100a) backend for ParaRNN's parallel
 * training hot path: fused Newton + chained linear scan forward, and the
 * reverse-time adjoint scan fused with the packed cell VJP.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless stated otherwise;
 *   - tensors are contiguous, row-major, channel-last:
 *       wx      (B, T, G*d)   gate pre-activations W_x(x)+b, gate-major inside a row
 *       states  (B, T, S, d)  S = 1 (GRU, NLRU) or 4 (sLSTM slots c, n, m, h)
 *   - `dtype` selects the I/O element type of wx / states / h0 / recurrent
 *     parameters / gradients: PRB_F32 or PRB_BF16.  All arithmetic and every
 *     intermediate trajectory is fp32;
 *   - recurrent parameters arrive already clamped (the reference clamps outside
 *     its kernels) ;
 *   - calls enqueue work on `stream` and return without synchronising.  The
 *     return value is 0 or a negative PRB_ERR_* code for argument / launch
 *     errors.  Device-side conditions (a bounded wait that ran out) are
 *     reported in prb_stats.status, which the caller reads after it has
 *     synchronised the stream;
 *   - scratch memory is provided by the caller: ask prb_*_workspace_bytes()
 *     and pass a buffer of at least that size (256-byte aligned).
 *
 * "Reference" citations are file:line in bugkira/pararnn-torch v0.17.5.
 */
#ifndef PARARNN_B200_H
#define PARARNN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* prb_stream_t; /* cudaStream_t */

enum { PRB_F32 = 0, PRB_BF16 = 1 };
enum { PRB_CELL_GRU_DIAG = 0, PRB_CELL_NLRU = 1, PRB_CELL_SLSTM_DIAG = 2, PRB_CELL_GRU_HEAD = 3,
       PRB_CELL_TITANS = 4, PRB_CELL_LSTM = 5, PRB_CELL_CFC = 6 };
enum {
    PRB_OK = 0,
    PRB_ERR_BAD_ARG = -1,     /* null pointer, non-positive size, unknown enum */
    PRB_ERR_WORKSPACE = -2,   /* workspace missing, misaligned or too small */
    PRB_ERR_UNSUPPORTED = -3, /* shape outside what the kernels cover */
    PRB_ERR_LAUNCH = -4,      /* CUDA reported a launch error */
    PRB_ERR_TOO_LARGE = -5,   /* fixed-capacity entry point: size beyond its limit */
    PRB_STATUS_CHAIN_TIMEOUT = 1 /* prb_stats.status: a bounded device wait ran out */
};
#define PRB_MAX_ITERS 16

/* Device-resident statistics block (80 bytes).  max|F| values are stored as the
 * IEEE-754 bit pattern of a non-negative float (NaN sorts highest).
 * Replaces the host-side residual evaluation of the reference,
 * solvers/newton/__init__.py:582-636 (_fill_stats). */
typedef struct prb_stats {
    uint32_t hist_bits[PRB_MAX_ITERS]; /* max|F(H^k)| before Newton pass k */
    uint32_t final_bits;               /* max|F(H^K)| of the returned trajectory */
    int32_t status;                    /* 0 or PRB_STATUS_CHAIN_TIMEOUT */
    int32_t reserved[2];
} prb_stats;

const char* prb_version(void);
const char* prb_error_string(int code);

/* Test and profiling hook, no counterpart in the reference: process-wide switches that force a
 * kernel family or a wait limit so that small test shapes reach code that normally serves large
 * ones.  Not thread-safe; call it while no other call of this library is in progress.  Every
 * option's default is what production calls use.
 *   PRB_OPT_KERNEL_FAMILY  -1 choose by shape (default), 0 look-back kernels, 2 pipelined kernels
 *   PRB_OPT_PICARD_FUSED    1 (default) / 0: all Picard passes in one sweep when the shape allows
 *   PRB_OPT_NEWTON_FUSED    1 (default) / 0: all Newton iterations in one sweep when it allows
 *   PRB_OPT_SPIN_LIMIT      polls after which a look-back wait gives up and reports
 *                           PRB_STATUS_CHAIN_TIMEOUT; <= 0 restores the default */
enum { PRB_OPT_KERNEL_FAMILY = 0, PRB_OPT_PICARD_FUSED = 1, PRB_OPT_NEWTON_FUSED = 2, PRB_OPT_SPIN_LIMIT = 3 };
int prb_debug_set(int option, long long value);

/* Scratch sizes.  `n_heads` is ignored by the diagonal cells. */
size_t prb_newton_workspace_bytes(int cell, int dtype, int B, int T, int d, int n_heads,
                                  int max_iters, int picard_iters);
size_t prb_bwd_workspace_bytes(int cell, int dtype, int B, int T, int d, int n_heads);

/* ---- forward: fused Newton + scan ------------------------------------------------ */

/* ParaGRU mix='diag'.  Replaces pararnn::newton_gru_fused,
 * kernels/custom_ops.py:146-188 -> kernels/newton_gru.py:332-495.
 * wx (B,T,3d) gates (z,r,n); a_z,a_r,a_n (d); h0 (B,d) or NULL; out (B,T,d). */
int prb_newton_gru_fused(const void* wx, const void* a_z, const void* a_r, const void* a_n,
                         const void* h0, void* out, int B, int T, int d, int dtype, int max_iters,
                         float omega, int want_residual, void* workspace, size_t workspace_bytes,
                         prb_stats* stats, prb_stream_t stream);

/* ParaNLRU.  Replaces pararnn::newton_nlru_fused, kernels/custom_ops.py:191-227 ->
 * kernels/newton_nlru.py:320-475.  wx (B,T,2d) gates (a,c); u (d). */
int prb_newton_nlru_fused(const void* wx, const void* u, const void* h0, void* out, int B, int T,
                          int d, int dtype, int max_iters, float omega, int want_residual,
                          void* workspace, size_t workspace_bytes, prb_stats* stats,
                          prb_stream_t stream);

/* ParaTitans (scalar-diagonal memory cell).  Replaces pararnn::newton_titans_fused,
 * kernels/custom_ops.py:269-308 -> kernels/newton_titans.py.  wx (B,T,5d) gates
 * (alpha_pre, theta_pre, k, v, n_pre); u, r (d) clamped; h0 (B,d) or NULL; out (B,T,d). */
int prb_newton_titans_fused(const void* wx, const void* u, const void* r, const void* h0, void* out, int B,
                            int T, int d, int dtype, int max_iters, float omega, int want_residual,
                            void* workspace, size_t workspace_bytes, prb_stats* stats, prb_stream_t stream);

/* ParaCfC (closed-form continuous-time cell with irregular time steps, gate_mix='input').  Replaces
 * pararnn::newton_cfc_fused, kernels/custom_ops.py:230-266 -> kernels/newton_cfc.py.  wx (B,T,4d) is
 * the cell's project_wx(x): gates (f_pre, c_x, dt, b) with dt the clamped time step broadcast over the
 * channels (cells/para_cfc.py:150-157); u (d) clamped; h0 (B,d) or NULL; out (B,T,d). */
int prb_newton_cfc_fused(const void* wx, const void* u, const void* h0, void* out, int B, int T, int d,
                         int dtype, int max_iters, float omega, int want_residual, void* workspace,
                         size_t workspace_bytes, prb_stats* stats, prb_stream_t stream);

/* ParaLSTM (CIFG peephole LSTM, diagonal recurrence, 2x2 block Jacobian per channel).  Replaces
 * pararnn::newton_lstm_fused, kernels/custom_ops.py:437-483 -> kernels/newton_lstm.py and
 * kernels/scan_lstm_block.py.  wx (B,T,3d) gates (f,z,o); a_f,a_z,a_o,c_f,c_o (d) clamped;
 * h0 (B,2,d) slots (c,h) or NULL; out (B,T,2,d).  prb_bwd_lstm replaces reverse_scan_block2
 * (solvers/scan.py:150-164) + lstm_recurrence_vjp (kernels/vjp_lstm.py): g_wx (B,T,3d), g_params
 * fp32 (5,d) in the order (a_f,a_z,a_o,c_f,c_o), g_h0 fp32 (B,2,d) or NULL.  `backward` selects
 * which of the two workspace layouts prb_lstm_workspace_bytes sizes. */
size_t prb_lstm_workspace_bytes(int B, int T, int d, int max_iters, int backward);
int prb_newton_lstm_fused(const void* wx, const void* a_f, const void* a_z, const void* a_o, const void* c_f,
                          const void* c_o, const void* h0, void* out, int B, int T, int d, int dtype,
                          int max_iters, float omega, int want_residual, void* workspace,
                          size_t workspace_bytes, prb_stats* stats, prb_stream_t stream);
int prb_bwd_lstm(const void* states, const void* wx, const void* a_f, const void* a_z, const void* a_o,
                 const void* c_f, const void* c_o, const void* h0, const void* grad_states, void* g_wx,
                 float* g_params, float* g_h0, int B, int T, int d, int dtype, void* workspace,
                 size_t workspace_bytes, prb_stats* stats, prb_stream_t stream);

/* ParaSLSTM mix='diag', including the frozen-gate Picard warm start.  Replaces
 * pararnn::newton_slstm_fused, kernels/custom_ops.py:486-540 ->
 * kernels/newton_slstm.py:2696-2939, and solvers/slstm_picard.py:158-181
 * (slstm_picard_init).  wx (B,T,4d) gates (i,f,z,o); r (4,d); h0 (B,4,d) or NULL;
 * states_guess (B,T,4,d) or NULL (when given it replaces the Picard warm start and
 * is not modified); out (B,T,4,d). */
int prb_newton_slstm_fused(const void* wx, const void* r, const void* h0, const void* states_guess,
                           void* out, int B, int T, int d, int dtype, int max_iters,
                           int picard_iters, float omega, float eps, int want_residual,
                           void* workspace, size_t workspace_bytes, prb_stats* stats,
                           prb_stream_t stream);

/* ParaGRU mix='head' (per-head dense recurrence, d_head in {8,16,32,64}).  Replaces
 * pararnn::newton_gru_head_fused, kernels/custom_ops.py:311-386 ->
 * kernels/newton_gru_head.py:96-195,460-567.  wx (B,T,3d) gate-major then head;
 * a_z,a_r,a_n (H,dh,dh) with y = h A; h0 (B,d) or NULL; out (B,T,d). */
size_t prb_gru_head_workspace_bytes(int B, int T, int d, int n_heads, int max_iters);
int prb_newton_gru_head_fused(const void* wx, const void* a_z, const void* a_r, const void* a_n,
                              const void* h0, void* out, int B, int T, int d, int n_heads, int dtype,
                              int max_iters, float omega, int want_residual, void* workspace,
                              size_t workspace_bytes, prb_stats* stats, prb_stream_t stream);

/* Reverse walk with the factorised J^T and the gate part of the packed VJP.  Replaces
 * pararnn::reverse_gru_head_factor (kernels/custom_ops.py:389-434,
 * kernels/newton_gru_head.py:198-258,570-652), gru_head_t0_vjp (:261-297) and the g_wx part of
 * gru_head_recurrence_vjp (kernels/vjp_gru.py:656-810).  g_wx (B,T,3d) I/O dtype;
 * g_a (3,H,dh,dh) fp32 = grad of (A_z, A_r, A_n), the outer-product sums
 * sum h_prev^T g_z, sum h_prev^T g_r, sum (h_prev r)^T g_n accumulated in the same sweep
 * (no clip mask applied); g_h0 (B,d) fp32 or NULL; mu_out (B,T,d) fp32 or NULL receives the
 * adjoint mu_t = J_{t+1}^T mu_{t+1} + g_t itself, the return value of the reference's op. */
int prb_bwd_gru_head(const void* states, const void* wx, const void* a_z, const void* a_r,
                     const void* a_n, const void* h0, const void* grad_states, void* g_wx, float* g_a,
                     float* g_h0, float* mu_out, int B, int T, int d, int n_heads, int dtype, void* workspace,
                     size_t workspace_bytes, prb_stats* stats, prb_stream_t stream);

/* ---- backward: eq. 2.6 reverse scan fused with the packed VJP ------------------- */

/* Replaces reverse_scan_diag + gru_recurrence_vjp / nlru_recurrence_vjp,
 * solvers/scan.py:126-148, kernels/vjp_gru.py:813-872, kernels/vjp_nlru.py:111-150,
 * and _t0_state_vjp, solvers/newton/dispatch.py:406-441.
 * states, grad_states (B,T,d); g_wx (B,T,G*d) in the I/O dtype;
 * g_params fp32 (NP,d) summed over batch and time (clip mask NOT applied);
 * g_h0 fp32 (B,d) or NULL. */
int prb_bwd_gru(const void* states, const void* wx, const void* a_z, const void* a_r,
                const void* a_n, const void* h0, const void* grad_states, void* g_wx,
                float* g_params, float* g_h0, int B, int T, int d, int dtype, void* workspace,
                size_t workspace_bytes, prb_stats* stats, prb_stream_t stream);
int prb_bwd_nlru(const void* states, const void* wx, const void* u, const void* h0,
                 const void* grad_states, void* g_wx, float* g_params, float* g_h0, int B, int T,
                 int d, int dtype, void* workspace, size_t workspace_bytes, prb_stats* stats,
                 prb_stream_t stream);

/* ParaTitans: reverse_scan_diag (solvers/scan.py:126-148) + the VJP the reference takes by autograd
 * through the cell step (solvers/vjp.py:77-98), in closed form.  g_wx (B,T,5d); g_params fp32
 * (2,d) = grad of (u, r); g_h0 fp32 (B,d) or NULL. */
int prb_bwd_titans(const void* states, const void* wx, const void* u, const void* r, const void* h0,
                   const void* grad_states, void* g_wx, float* g_params, float* g_h0, int B, int T, int d,
                   int dtype, void* workspace, size_t workspace_bytes, prb_stats* stats,
                   prb_stream_t stream);

/* ParaCfC: reverse_scan_diag (solvers/scan.py:126-148) + cfc_recurrence_vjp
 * (kernels/vjp_cfc.py:102-167).  g_wx (B,T,4d) = grads of (f_pre, c_x, dt, b); g_params fp32 (1,d) =
 * grad of u; g_h0 fp32 (B,d) or NULL. */
int prb_bwd_cfc(const void* states, const void* wx, const void* u, const void* h0, const void* grad_states,
                void* g_wx, float* g_params, float* g_h0, int B, int T, int d, int dtype, void* workspace,
                size_t workspace_bytes, prb_stats* stats, prb_stream_t stream);

/* Replaces reverse_scan_block4 + slstm_recurrence_vjp, solvers/scan.py:166-178,
 * kernels/vjp_slstm.py:234-293.  states, grad_states (B,T,4,d); g_wx (B,T,4d);
 * g_params fp32 (4,d); g_h0 fp32 (B,4,d) or NULL. */
int prb_bwd_slstm(const void* states, const void* wx, const void* r, const void* h0,
                  const void* grad_states, void* g_wx, float* g_params, float* g_h0, int B, int T,
                  int d, int dtype, float eps, void* workspace, size_t workspace_bytes,
                  prb_stats* stats, prb_stream_t stream);

/* The reverse scan + VJP of any scalar-diagonal cell (cell = PRB_CELL_GRU_DIAG, _NLRU, _TITANS, _CFC;
 * p0..p2 = its recurrent vectors in the order of the per-cell entry points, unused ones NULL) with one
 * more output: g_bias fp32 (G*d) or NULL = the per-gate sums of g_wx over batch and time, i.e. the
 * gradient of the bias of the input projection (solvers/vjp.py:109-120 computes it as a separate
 * reduction over g_wx).  Everything else as prb_bwd_gru / _nlru / _titans / _cfc. */
int prb_bwd_diag_ex(int cell, const void* states, const void* wx, const void* p0, const void* p1,
                    const void* p2, const void* h0, const void* grad_states, void* g_wx, float* g_params,
                    float* g_bias, float* g_h0, int B, int T, int d, int dtype, void* workspace,
                    size_t workspace_bytes, prb_stats* stats, prb_stream_t stream);

/* prb_bwd_slstm for a layer: the same reverse scan and VJP with two things a layer around the op
 * otherwise does in separate passes over (B,T,4d) arrays.  grad_slot in 0..3: `grad` is (B,T,d), the
 * cotangent of that state slot alone (a layer that outputs the hidden slot h = 3 receives exactly
 * this; the reference materialises the zero-filled (B,T,4,d) array, layers/para_rnn.py:279-283 through
 * select_backward); grad_slot = -1: `grad` is (B,T,4,d) as in prb_bwd_slstm.  The
 * pipelined kernel has the compact form for the hidden slot (3); other slots run on the look-back kernels.  g_bias fp32 (4,d) or
 * NULL: the per-gate sums of g_wx over batch and time, i.e. the gradient of the bias of W_x
 * (solvers/vjp.py:109-120 computes it as g_wx.sum over (B,T)). */
int prb_bwd_slstm_ex(const void* states, const void* wx, const void* r, const void* h0,
                     const void* grad, int grad_slot, void* g_wx, float* g_params, float* g_bias,
                     float* g_h0, int B, int T, int d, int dtype, float eps, void* workspace,
                     size_t workspace_bytes, prb_stats* stats, prb_stream_t stream);

/* ---- residual gate ------------------------------------------------------------------- */

/* max|f(H_{t-1},x_t) - H_t| into stats->final_bits.  Replaces the eager
 * evaluation in solvers/newton/__init__.py:602-606.  params: GRU (3,d) packed
 * a_z,a_r,a_n; NLRU and CfC (1,d); Titans (2,d) = u,r; sLSTM (4,d); all in the I/O dtype. */
int prb_residual(int cell, const void* wx, const void* params, const void* h0, const void* states,
                 int B, int T, int d, int dtype, float eps, void* workspace, size_t workspace_bytes,
                 prb_stats* stats, prb_stream_t stream);

/* ---- pass-level entry points ---------------------------------------------------------
 * One scan pass over a (shard of a) sequence with explicit boundary data, used by the
 * time-sharded multi-GPU driver and for per-kernel timing.  They replace the per-rank
 * pieces of the reference's context-parallel scan, solvers/seq_parallel.py:126-342
 * (local scan, carry, prefix apply), generalised from the scalar monoid to all cells.
 * Parameters, halos and carries here are fp32; `halo` is the state preceding step 0 of
 * the shard, `carry_in` the scan carry entering step 0 (NULL = zeros).
 * mode: 0 = apply, fp32 work trajectory out; 1 = apply, last pass, output in the I/O
 * dtype; 2 = aggregate only: nothing but the shard's aggregate map is written.
 * Time segments (sLSTM passes): with n_seg > 1 the shard's time axis is cut into n_seg pieces of
 * seg_len steps ((n_seg-1)*seg_len < T <= n_seg*seg_len) that are swept by different thread
 * blocks at the same time, which is what fills the GPU when there are fewer (batch row, channel
 * block) chains than SMs.  carry_in then is (n_seg, B, NS, d) (the carry entering each segment,
 * from prb_segment_carries), agg_out (n_seg, B, NV, d); tail_out / head_out stay (B, NS, d) and
 * are written by the segment that ends the scan.  prb_plan_segments proposes n_seg / seg_len for
 * a shape (1 / T when segments would not help or the kernels that support them cannot run).
 * The workspace (prb_pass_workspace_bytes) holds the chain scratch of one pass.
 * prb_stats is NOT cleared by these calls: hist_bits[hist_slot] / final_bits are
 * max-accumulated, so the caller zeroes the block once per solve. */
size_t prb_pass_workspace_bytes(int cell, int B, int T, int d);

int prb_diag_guess(int cell, const void* wx, const float* params, const float* h0, float* out, int B,
                   int T, int d, int dtype, prb_stream_t stream);

/* scalar-diagonal Newton pass: carry = delta (B,d); aggregate (B,2,d) = (a, b) */
int prb_diag_newton_pass(int cell, const void* wx, const float* params, const float* hin,
                         const float* halo, const float* carry_in, void* hout, float* tail_out,
                         float* agg_out, int mode, int B, int T, int d, int dtype, float omega,
                         void* workspace, size_t workspace_bytes, prb_stats* stats, int hist_slot,
                         prb_stream_t stream);

/* reverse pass: carry = nu entering the shard's last step (B,d); head_out = nu leaving
 * its first step (grad_h0 on the first shard); g_params = this shard's partial sums */
int prb_diag_bwd_pass(int cell, const void* states, const void* wx, const float* params,
                      const float* halo, const float* carry_in, const void* grad_states, void* g_wx,
                      float* g_params, float* head_out, float* agg_out, int mode, int B, int T, int d,
                      int dtype, void* workspace, size_t workspace_bytes, prb_stats* stats,
                      prb_stream_t stream);

/* All n_passes frozen-gate passes of the sLSTM warm start (the zero-hidden pass first) in one
 * sweep over the sequence: pass p follows pass p-1 a few steps behind, hidden states never leave
 * the chip.  Replaces slstm_picard_init, solvers/slstm_picard.py:158-181 (P+1 separate scans
 * there).  h_halo (B,d), carry_in (B,3,d) = (c,n,m) preceding step 0 or NULL; writes the full
 * state (B,T,4,d) fp32 of the last pass.  PRB_ERR_UNSUPPORTED when n_passes > 6 or the arrays do
 * not meet the 16-byte stride rule of the bulk tensor loads (use prb_slstm_picard_pass then). */
int prb_slstm_picard_sweep(const void* wx, const float* r, const float* h_halo, const float* carry_in,
                           float* state_out, float* tail_out, int n_passes, int B, int T, int d,
                           int dtype, float eps, void* workspace, size_t workspace_bytes,
                           prb_stats* stats, prb_stream_t stream);

/* All n_iters Newton iterations of a whole sequence in one sweep (iteration k+1 follows iteration
 * k a few steps behind; intermediate iterates never leave the chip), with the residual of the
 * result when want_residual is set.  Replaces the K passes of _newton_slstm_fused_impl,
 * kernels/newton_slstm.py:2696-2939, and the eager residual of _fill_stats,
 * solvers/newton/__init__.py:582-636.  sin (B,T,4,d) fp32 warm start, halo (B,4,d) state preceding
 * step 0 or NULL, sout (B,T,4,d) in the I/O dtype; stats->hist_bits[k] = max|F(H^k)|.
 * PRB_ERR_UNSUPPORTED when n_iters > 4 or the arrays do not meet the 16-byte stride rule of the
 * bulk tensor loads (use prb_slstm_newton_pass then). */
int prb_slstm_newton_sweep(const void* wx, const float* r, const float* sin, const float* halo, void* sout,
                           int n_iters, int want_residual, int B, int T, int d, int dtype, float omega,
                           float eps, void* workspace, size_t workspace_bytes, prb_stats* stats,
                           prb_stream_t stream);

/* sLSTM frozen-gate pass: h_prev (B,T,d) hidden trajectory of the previous pass or NULL
 * (zero-hidden pass); h_halo (B,d); carry (B,3,d) = (c,n,m); aggregate (B,4,d) = (a,b,N,C);
 * writes h_out (B,T,d) or, when state_out is given, the full state (B,T,4,d) */
int prb_slstm_picard_pass(const void* wx, const float* r, const float* h_prev, const float* h_halo,
                          const float* carry_in, float* h_out, float* state_out, float* tail_out,
                          float* agg_out, int mode, int n_seg, int seg_len, int B, int T, int d, int dtype,
                          float eps, void* workspace, size_t workspace_bytes, prb_stats* stats,
                          prb_stream_t stream);

/* sLSTM Newton pass: halo, carry (B,4,d); aggregate (B,20,d) = 4x4 row-major M, then v */
int prb_slstm_newton_pass(const void* wx, const float* r, const float* sin, const float* halo,
                          const float* carry_in, void* sout, float* tail_out, float* agg_out, int mode,
                          int n_seg, int seg_len, int B, int T, int d, int dtype, float omega, float eps,
                          void* workspace, size_t workspace_bytes, prb_stats* stats, int hist_slot,
                          prb_stream_t stream);

int prb_slstm_bwd_pass(const void* states, const void* wx, const float* r, const float* halo,
                       const float* carry_in, const void* grad_states, void* g_wx, float* g_params,
                       float* head_out, float* agg_out, int mode, int n_seg, int seg_len, int B, int T,
                       int d, int dtype, float eps, void* workspace, size_t workspace_bytes,
                       prb_stats* stats, prb_stream_t stream);

/* Carry entering `rank` from the all-gathered per-rank slots (world, B, NV, d): the first
 * rank in scan order (rank 0, or world-1 when reverse != 0) stores the exact carry leaving it
 * in its first NS rows, every other rank its aggregate map.  monoid: 0 scalar affine
 * (NV 2, NS 1), 1 4x4 affine (NV 20, NS 4), 2 sLSTM frozen-gate (NV 4, NS 3).  Replaces the
 * serial fold of solvers/seq_parallel.py:185-191. */
int prb_fold_carries(int monoid, const float* gathered, int rank, int world, int reverse,
                     float* carry_out, int B, int d, prb_stream_t stream);

/* Segment plan for the pass-level sLSTM entry points (see "Time segments" above). */
int prb_plan_segments(int cell, int dtype, int B, int T, int d, int* n_seg, int* seg_len);

/* Map of a whole shard from its segment maps agg (n_seg, B, NV, d), composed in scan order
 * (time order, or backwards when reverse != 0) into slot (B, NV, d): what a rank that does not
 * know its entering carry puts into the all-gather.  Same role as the local scan of
 * solvers/seq_parallel.py:175-183, one level down. */
int prb_fold_segments(int monoid, const float* agg, int n_seg, int reverse, float* slot, int B, int d,
                      prb_stream_t stream);

/* Carries entering every segment, given the carry entering the shard (carry0 (B, NS, d), NULL =
 * zeros): carries (n_seg + 1, B, NS, d); carries[j] enters segment j (at its last step when
 * reverse != 0), carries[n_seg] leaves the shard. */
int prb_segment_carries(int monoid, const float* agg, int n_seg, int reverse, const float* carry0,
                        float* carries, int B, int d, prb_stream_t stream);

/* prb_fold_carries and prb_segment_carries in ONE launch, for a rank that is not the first in scan
 * order.  gathered (world, B, slot_rows, d) fp32: every rank's slot holds its map (or, for the first
 * rank, its outgoing state) in the first rows and whatever rides along after them (slot_rows >= NV).
 * carry_out (B,NS,d): the carry entering the rank.  carries (n_seg+1, B, NS, d) or NULL: the carries
 * entering the rank's segments and the one leaving it, through the segment maps agg (n_seg,B,NV,d).
 * h_end (B,d) or NULL, frozen-gate monoid only: sigmoid(zo) c / (n + eps) with zo = row NV of the
 * previous rank's slot, i.e. the hidden value at the previous rank's last step
 * (cells/para_slstm.py:347-446, the h output of the state the carry holds). */
int prb_shard_carries(int monoid, const float* gathered, int slot_rows, int rank, int world, int reverse,
                      const float* agg, int n_seg, float* carry_out, float* carries, float eps, float* h_end,
                      int B, int d, prb_stream_t stream);

/* residual of a shard with an fp32 halo; states fp32 (states_f32 != 0) or I/O dtype */
int prb_residual_pass(int cell, const void* wx, const float* params, const float* halo,
                      const void* states, int states_f32, int B, int T, int d, int dtype, float eps,
                      prb_stats* stats, prb_stream_t stream);

/* ---- T = 1 decode ----------------------------------------------------------------------
 * One recurrent step of a whole batch in one launch (the serving path: .eval(), T = 1).  Replaces
 * decode_step, kernels/decode.py:119-216 and its three step kernels (:294-475); W_x(x) stays a
 * library GEMM on the caller's side.  state (B, S, d) or, with block_table (B,) int32 slot ids,
 * a pool (C, S, d); wx (B, G*d); params_raw: the UNCLAMPED recurrent vectors (GRU (3,d), NLRU
 * (1,d), CfC (1,d), Titans (2,d), sLSTM (4,d)) in the I/O dtype, clamped to [-cap, cap] in the kernel (cap < 0: no
 * clamp), so a captured CUDA graph needs no extra kernel; out has the shape of state and may BE
 * state (in-place update of the pool rows named by block_table).  Allocates nothing, takes no
 * workspace, never synchronises: it can be captured in a CUDA graph. */
int prb_decode_step(int cell, const void* state, const void* wx, const void* params_raw, float cap,
                    const int* block_table, void* out, int B, int d, int dtype, float eps,
                    prb_stream_t stream);

/* ---- entry point that allocates nothing ------------------------------------------------
 * No counterpart in the reference (its ops allocate scratch through PyTorch on every call).
 *
 * prb_bwd_nlru_static is prb_bwd_nlru without the workspace argument: its scratch (chain
 * flags, tile aggregates, fp32 copies of u and h0, per-tile parameter partials) lives in a
 * fixed array of PRB_STATIC_SCRATCH_BYTES inside the library.  It is meant for callers that
 * must not, or cannot, obtain device memory at the point of the call: code running inside a
 * region where the allocator is off limits (a real-time or interrupt-like service loop, a
 * host callback, a plugin whose host owns all device memory and hands out none), or a
 * process whose memory budget was fixed at start-up.  The function and everything it calls
 * use no cudaMalloc / cudaFree and no allocating library routine; the caller still passes
 * every input and output buffer, including the prb_stats block.
 *
 * Limits and rules
 *   - the problem must satisfy prb_bwd_workspace_bytes(PRB_CELL_NLRU, ...) <=
 *     PRB_STATIC_SCRATCH_BYTES (8 MiB); larger shapes return PRB_ERR_TOO_LARGE and launch
 *     nothing;
 *   - every GPU that loads the library holds the 8 MiB until the process exits;
 *   - the first call on each device looks up the array's device address (with that device
 *     current) and remembers it; make that first call outside any stream capture;
 *   - all calls on a device share the one array and it keeps whatever the last call left in
 *     it: the call re-clears what has to start at zero, but two calls whose GPU work can
 *     overlap (different streams, or two host threads) race on it.  Serialise them. */
#define PRB_STATIC_SCRATCH_BYTES (8u << 20)
size_t prb_static_scratch_bytes(void);
int prb_bwd_nlru_static(const void* states, const void* wx, const void* u, const void* h0,
                        const void* grad_states, void* g_wx, float* g_params, float* g_h0, int B,
                        int T, int d, int dtype, prb_stats* stats, prb_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* PARARNN_B200_H */
