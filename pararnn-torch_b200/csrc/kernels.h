// Internal launcher interface between the C ABI (capi.cu) and the kernel files.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>

#include "common.cuh"

namespace prb {

// SM count of the current device (queried once per device).
int sm_count();

// Process-wide switches set through prb_debug_set (tests and profiling only); the defaults are
// what every normal call uses.
struct Options {
    int kernel_family = -1;            // -1 choose by shape, 0 look-back kernels, 2 pipelined kernels
    bool picard_fused = true;          // all Picard passes in one sweep when the shape allows
    bool newton_fused = true;          // all Newton iterations in one sweep when the shape allows
    unsigned spin_limit = kSpinLimit;  // poll limit of the look-back waits
};
Options& options();

enum Cell : int { kCellGruDiag = 0, kCellNlru = 1, kCellSlstmDiag = 2, kCellGruHead = 3, kCellTitans = 4,
                  kCellLstm = 5, kCellCfc = 6 };
// gates and recurrent parameter vectors per channel of the scalar-diagonal cells
inline bool is_diag_cell(int cell) {
    return cell == kCellGruDiag || cell == kCellNlru || cell == kCellTitans || cell == kCellCfc;
}
inline int diag_cell_params(int cell) { return cell == kCellGruDiag ? 3 : (cell == kCellTitans ? 2 : 1); }
inline int diag_cell_gates(int cell) {
    return cell == kCellGruDiag ? 3 : (cell == kCellNlru ? 2 : (cell == kCellTitans ? 5 : 4));
}
enum DType : int { kF32 = 0, kBF16 = 1 };

// ---- scalar-diagonal cells ------------------------------------------------
struct DiagFwdArgs {
    const void* wx;         // (B,T,G*d) I/O dtype
    const float* par;       // clamped recurrent vectors, fp32 [NP][d]
    const float* halo;      // (B,d) fp32 state preceding step 0 (h0), may be null = zeros
    const float* carry_in;  // (B,d) fp32 delta entering step 0, may be null = zeros
    const float* hin;       // (B,T,d) fp32 input trajectory (unused by the first pass)
    void* hout;             // (B,T,d) fp32 work trajectory, or I/O dtype on the last pass
    float* tail_out;        // (B,d) delta leaving the last step, may be null
    float* agg_out;         // (B,2,d) shard aggregate (aggregate-only sweep)
    unsigned* resid_bits;   // max|F| of the input trajectory (atomicMax target)
    unsigned* final_bits;   // last pass only: max|F| of the output trajectory, may be null
    int B, T, d;
    float omega;
    Chain chain;
};

struct DiagBwdArgs {
    const void* wx;           // (B,T,G*d)
    const void* states;       // (B,T,d) converged trajectory, I/O dtype
    const void* grad_states;  // (B,T,d) I/O dtype
    const float* par;
    const float* halo;      // (B,d) state preceding step 0
    const float* carry_in;  // (B,d) nu entering the last step (from the next shard), may be null
    void* g_wx;             // (B,T,G*d) I/O dtype
    float* gp_partial;      // (B*n_tt, NP, d) per-tile parameter partial sums
    float* gb_partial;      // (same rows, G, d) per-gate sums of g_wx (bias gradient), or null
    float* g_h0;            // (B,d) nu leaving step 0 (= grad_h0 on the first shard), may be null
    float* agg_out;         // (B,2,d)
    float* mu_out;          // optional (B,T,d) fp32
    int B, T, d;
    Chain chain;
};

int diag_tile_steps();
cudaError_t launch_diag_newton(int cell, int dtype, const DiagFwdArgs& a, bool first, bool last,
                               cudaStream_t s);
cudaError_t launch_diag_newton_agg(int cell, int dtype, const DiagFwdArgs& a, cudaStream_t s);
// pipelined persistent family (diag_pipe.cu): one CTA per chain, TMA-fed
cudaError_t launch_diag_newton_pipe(int cell, int dtype, const DiagFwdArgs& a, bool first, bool last,
                                    cudaStream_t s);
// all K Newton iterations (1..4) from the App. A guess, and the residual of the result, in one sweep
cudaError_t launch_diag_newton_fused(int cell, int dtype, const DiagFwdArgs& a, int K, cudaStream_t s);
cudaError_t launch_diag_bwd_pipe(int cell, int dtype, const DiagBwdArgs& a, cudaStream_t s);
cudaError_t launch_diag_guess(int cell, int dtype, bool out_f32, const void* wx, const float* par,
                              const float* h0, void* out, int B, int T, int d, cudaStream_t s);
cudaError_t launch_diag_residual(int cell, int dtype, bool st_f32, const void* wx, const float* par,
                                 const float* halo, const void* st, int B, int T, int d,
                                 unsigned* dst, cudaStream_t s);
cudaError_t launch_diag_bwd(int cell, int dtype, const DiagBwdArgs& a, bool agg_only, cudaStream_t s);
cudaError_t launch_reduce_partials(const float* part, int rows, int np_d, float* out, cudaStream_t s);

// ---- ParaSLSTM mix='diag' ----------------------------------------------------
struct SlstmPicardArgs {
    const void* wx;        // (B,T,4d) I/O dtype, gate order (i,f,z,o)
    const float* r;        // (4,d) fp32 clamped
    const float* h_prev;   // (B,T,d) fp32 hidden trajectory of the previous pass; null = zero-hidden pass
    const float* h_halo;   // (B,d) hidden state preceding step 0 for h_prev; null = zeros
    const float* carry_in; // (c,n,m) entering step 0, slot stride d; null = zeros
    float* h_out;          // (B,T,d) fp32 hidden only (not the last Picard pass)
    float* state_out;      // (B,T,4,d) fp32 full state (last Picard pass), slots (c,n,m,h)
    float* tail_out;       // (B,3,d) (c,n,m) leaving the last step, may be null
    float* agg_out;        // (B,4,d) shard aggregate (a,b,N,C)
    int halo_stride;       // batch stride (floats) of h_halo
    int carry_stride;      // batch stride (floats) of carry_in, slots (c,n,m) d apart
    int B, T, d;
    float eps;
    // time segments: CTA (chain, seg) owns steps [seg*seg_len, min(T, (seg+1)*seg_len)); carry_in
    // and agg_out then have a leading n_seg dimension.  n_seg <= 1 means one segment of T steps.
    int n_seg, seg_len;
    Chain chain;
};

struct SlstmNewtonArgs {
    const void* wx;
    const float* r;
    const float* sin;       // (B,T,4,d) fp32 input trajectory
    const float* halo;      // (B,4,d) state preceding step 0; null = zeros
    const float* carry_in;  // (B,4,d) delta entering step 0; null = zeros
    void* sout;             // (B,T,4,d) fp32, or I/O dtype on the last pass
    float* tail_out;        // (B,4,d)
    float* agg_out;         // (B,20,d)
    unsigned* resid_bits;
    unsigned* final_bits;   // last pass only: max|F| of the output trajectory, may be null
    int halo_stride;        // batch stride (floats) of halo
    int B, T, d;
    float omega, eps;
    // time segments: CTA (chain, seg) owns steps [seg*seg_len, min(T, (seg+1)*seg_len)); carry_in
    // and agg_out then have a leading n_seg dimension.  n_seg <= 1 means one segment of T steps.
    int n_seg, seg_len;
    Chain chain;
};

struct SlstmBwdArgs {
    const void* wx;
    const void* states;       // (B,T,4,d) I/O dtype
    const void* grad_states;  // (B,T,4,d) I/O dtype
    const float* r;
    const float* halo;      // (B,4,d)
    const float* carry_in;  // (B,4,d) nu entering the last step
    void* g_wx;             // (B,T,4d)
    float* gp_partial;      // (B*n_tt,4,d)
    float* gb_partial;      // same rows as gp_partial: per-gate sums of g_wx (bias gradient), or null
    float* g_h0;            // (B,4,d)
    float* agg_out;         // (B,20,d)
    // -1: grad_states is (B,T,4,d).  0..3: grad_states is (B,T,d), the cotangent of that state slot
    // alone (the other slots have none) -- what a layer that outputs the hidden slot receives.
    int g_slot = -1;
    int halo_stride;
    int B, T, d;
    float eps;
    // time segments: CTA (chain, seg) owns steps [seg*seg_len, min(T, (seg+1)*seg_len)); carry_in
    // and agg_out then have a leading n_seg dimension.  n_seg <= 1 means one segment of T steps.
    int n_seg, seg_len;
    Chain chain;
};

int slstm_tile_steps();
int slstm_picard_tile_steps();
cudaError_t launch_slstm_picard(int dtype, const SlstmPicardArgs& a, bool agg_only, cudaStream_t s);
cudaError_t launch_slstm_newton(int dtype, const SlstmNewtonArgs& a, bool last, bool agg_only,
                                cudaStream_t s);
cudaError_t launch_slstm_residual(int dtype, bool st_f32, const void* wx, const float* r,
                                  const float* halo, int halo_stride, const void* st, int B, int T,
                                  int d, float eps, unsigned* dst, cudaStream_t s);
cudaError_t launch_slstm_bwd(int dtype, const SlstmBwdArgs& a, bool agg_only, cudaStream_t s);

// true when TMA tile loads can address the (B,T,G*d) / (B,T,S,d) arrays of this shape and dtype
bool tma_addressable(int dtype, int B, int T, int d);
// all Newton iterations in one sweep (slstm_newton_fused.cu)
int slstm_newton_fused_max_iters();
cudaError_t launch_slstm_newton_fused(int dtype, const SlstmNewtonArgs& a, int n_iters, cudaStream_t s);
// all Picard passes of the warm start in one sweep (slstm_picard_fused.cu)
int slstm_picard_fused_max_passes();
cudaError_t launch_slstm_picard_fused(int dtype, const SlstmPicardArgs& a, int n_pass, cudaStream_t s);

// warp-pipelined variants (slstm_pipe.cu)
cudaError_t launch_slstm_newton_pipe(int dtype, const SlstmNewtonArgs& a, bool last, cudaStream_t s);
cudaError_t launch_slstm_picard_pipe(int dtype, const SlstmPicardArgs& a, cudaStream_t s);
cudaError_t launch_slstm_bwd_pipe(int dtype, const SlstmBwdArgs& a, cudaStream_t s);

// aggregate-only sweeps with one CTA per chain (slstm_agg.cu); any shape
cudaError_t launch_slstm_newton_agg_seg(int dtype, const SlstmNewtonArgs& a, cudaStream_t s);
cudaError_t launch_slstm_picard_agg_seg(int dtype, const SlstmPicardArgs& a, cudaStream_t s);
cudaError_t launch_slstm_bwd_agg_seg(int dtype, const SlstmBwdArgs& a, cudaStream_t s);


// ---- ParaGRU mix='head' (gru_head_kernels.cu) --------------------------------------------
cudaError_t launch_gru_head_fwd(int dtype, const void* wx, const float* A, const float* h0,
                                const float* hin, void* hout, bool out_io, int n_newton, bool resid,
                                unsigned* hist_bits, unsigned* final_bits, int B, int T, int d, int H,
                                float omega, cudaStream_t s);
cudaError_t launch_gru_head_bwd(int dtype, const void* wx, const void* states, const void* grad_states,
                                const float* A, const float* h0, void* g_wx, float* gA_part, float* g_h0,
                                float* mu_out, int B, int T, int d, int H, cudaStream_t s);

// ---- ParaLSTM (lstm_kernels.cu): state (B,T,2,d) slots (c,h), gates (f,z,o), 5 parameter vectors
struct LstmFwdArgs {
    const void* wx;       // (B,T,3d) I/O dtype
    const float* par;     // (5,d) fp32 clamped: a_f, a_z, a_o, c_f, c_o
    const float* halo;    // (B,2,d) fp32 initial state or null
    const float* sin;     // (B,T,2,d) fp32 input trajectory (unused by the first pass)
    void* sout;           // (B,T,2,d) fp32 work trajectory, or I/O dtype on the last pass
    unsigned* resid_bits;
    unsigned* final_bits;
    int B, T, d;
    float omega;
    Chain chain;
};
struct LstmBwdArgs {
    const void* wx;
    const void* states;       // (B,T,2,d) I/O dtype
    const void* grad_states;  // (B,T,2,d) I/O dtype
    const float* par;
    const float* halo;
    void* g_wx;               // (B,T,3d)
    float* gp_partial;        // (B*n_tt,5,d)
    float* g_h0;              // (B,2,d) or null
    int B, T, d;
    Chain chain;
};
int lstm_tile_steps();
cudaError_t launch_lstm_newton(int dtype, const LstmFwdArgs& a, bool first, bool last, cudaStream_t s);
cudaError_t launch_lstm_guess(int dtype, const void* wx, const float* par, const float* h0, void* out, int B,
                              int T, int d, cudaStream_t s);
cudaError_t launch_lstm_residual(int dtype, const void* wx, const float* par, const float* h0, const void* st,
                                 int B, int T, int d, unsigned* dst, cudaStream_t s);
cudaError_t launch_lstm_bwd(int dtype, const LstmBwdArgs& a, cudaStream_t s);
// pipelined persistent family (lstm_pipe.cu): all K <= 4 iterations from the guess in one sweep, and the
// reverse sweep with one parameter-partial row per batch row
cudaError_t launch_lstm_newton_fused(int dtype, const LstmFwdArgs& a, int K, cudaStream_t s);
cudaError_t launch_lstm_bwd_pipe(int dtype, const LstmBwdArgs& a, cudaStream_t s);

// ---- T = 1 decode (decode.cu) ------------------------------------------------------------------
cudaError_t launch_decode_step(int cell, int dtype, const void* state, const void* wx, const void* par,
                               const int* block_table, void* out, int B, int d, float cap, float eps,
                               cudaStream_t s);

}  // namespace prb
