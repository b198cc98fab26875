// T = 1 decode: one launch for the recurrent step of a whole batch (gates + state mix).
//
// The serving-side counterpart of the training kernels: W_x(x) stays a library GEMM, this kernel
// is the rest of cell.step.  Each thread owns one channel of one batch row: it loads the previous
// state (from row b, or from pool row block_table[b]), the gate pre-activations and the RAW
// recurrent parameters, clamps them in-kernel (so that a captured CUDA graph needs no clamp
// kernel and no allocation), evaluates the step and writes the next state (to `out`, which may
// be the state pool itself).  Pure HBM-bound elementwise work: (S + G) reads + S writes per
// channel.  Reference behaviour restated: kernels/decode.py:119-216 (dispatch, out= and
// block_table rules), :294-475 (the three step kernels), cells/para_gru.py:375-383,
// cells/para_nlru.py:149-168, cells/para_slstm.py:347-400.
#include "common.cuh"
#include "diag_cell.cuh"
#include "kernels.h"
#include "slstm_cell.cuh"

namespace prb {

namespace {

__device__ __forceinline__ float clamp_cap(float v, float cap) {
    return cap < 0.f ? v : fminf(fmaxf(v, -cap), cap);
}

template <int CELL, typename TIO>
__global__ void decode_diag_kernel(const TIO* state, const TIO* wx, const TIO* par, const int* bt, TIO* out,
                                   int B, int d, float cap) {
    using C = DiagCell<CELL>;
    const int ch = blockIdx.x * blockDim.x + threadIdx.x, b = blockIdx.y;
    if (ch >= d) return;
    const size_t row = bt ? (size_t)bt[b] : (size_t)b;
    float g[C::G], p[C::NP];
#pragma unroll
    for (int q = 0; q < C::G; ++q) g[q] = ld_f(wx + ((size_t)b * C::G + q) * d + ch);
#pragma unroll
    for (int q = 0; q < C::NP; ++q) p[q] = clamp_cap(ld_f(par + (size_t)q * d + ch), cap);
    const float h = ld_f(state + row * d + ch);
    st_f(out + row * d + ch, C::step(h, g, p));
}

template <typename TIO>
__global__ void decode_slstm_kernel(const TIO* state, const TIO* wx, const TIO* par, const int* bt, TIO* out,
                                    int B, int d, float cap, float eps) {
    const int ch = blockIdx.x * blockDim.x + threadIdx.x, b = blockIdx.y;
    if (ch >= d) return;
    const size_t row = bt ? (size_t)bt[b] : (size_t)b;
    float prev[4], w[4], r[4], pred[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        prev[q] = ld_f(state + (row * 4 + q) * d + ch);
        w[q] = ld_f(wx + ((size_t)b * 4 + q) * d + ch);
        r[q] = clamp_cap(ld_f(par + (size_t)q * d + ch), cap);
    }
    slstm_predict(prev, w, r, eps, pred);
#pragma unroll
    for (int q = 0; q < 4; ++q) st_f(out + (row * 4 + q) * d + ch, pred[q]);
}

template <typename TIO>
cudaError_t launch_t(int cell, const void* state, const void* wx, const void* par, const int* bt, void* out,
                     int B, int d, float cap, float eps, cudaStream_t s) {
    const int threads = 128;
    const dim3 grid((d + threads - 1) / threads, B);
    const TIO* st = reinterpret_cast<const TIO*>(state);
    const TIO* w = reinterpret_cast<const TIO*>(wx);
    const TIO* p = reinterpret_cast<const TIO*>(par);
    TIO* o = reinterpret_cast<TIO*>(out);
    if (cell == kCellGruDiag)
        decode_diag_kernel<kCellGruDiag, TIO><<<grid, threads, 0, s>>>(st, w, p, bt, o, B, d, cap);
    else if (cell == kCellNlru)
        decode_diag_kernel<kCellNlru, TIO><<<grid, threads, 0, s>>>(st, w, p, bt, o, B, d, cap);
    else if (cell == kCellTitans)
        decode_diag_kernel<kCellTitans, TIO><<<grid, threads, 0, s>>>(st, w, p, bt, o, B, d, cap);
    else if (cell == kCellCfc)
        decode_diag_kernel<kCellCfc, TIO><<<grid, threads, 0, s>>>(st, w, p, bt, o, B, d, cap);
    else if (cell == kCellSlstmDiag)
        decode_slstm_kernel<TIO><<<grid, threads, 0, s>>>(st, w, p, bt, o, B, d, cap, eps);
    else
        return cudaErrorNotSupported;
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_decode_step(int cell, int dtype, const void* state, const void* wx, const void* par,
                               const int* block_table, void* out, int B, int d, float cap, float eps,
                               cudaStream_t s) {
    return dtype == kF32 ? launch_t<float>(cell, state, wx, par, block_table, out, B, d, cap, eps, s)
                         : launch_t<__nv_bfloat16>(cell, state, wx, par, block_table, out, B, d, cap, eps, s);
}

}  // namespace prb
