// ParaLSTM (CIFG peephole LSTM with diagonal recurrence; state slots (c, h), gates (f, z, o),
// parameters (a_f, a_z, a_o, c_f, c_o)): fused Newton pass with the 2x2 block Jacobian, residual
// gate, and the fused reverse-time adjoint scan with the packed VJP.  Look-back family (any
// shape): a pass is cut into chains (batch row x 32 channels) and time tiles of W*L steps; a
// thread linearises its L steps and composes their 2x2 affine map, tile_exchange (common.cuh)
// delivers the carry entering its sub-tile, and the thread applies it.
//
// Reference behaviour restated (paths relative to the reference project):
//   cells/para_lstm.py:154-232             step and 2x2 block Jacobian (eq. 3.1b / 3.2b)
//   solvers/newton/__init__.py:467-549,925-940   Newton loop, App.-A initial guess
//   solvers/scan.py:150-164                eq. 2.6 reverse scan with 2x2 blocks
//   kernels/vjp_lstm.py                    packed VJP (lstm_recurrence_vjp)
//   kernels/newton_lstm.py, kernels/scan_lstm_block.py   the fused op this replaces
#include "common.cuh"
#include "kernels.h"
#include "lstm_cell.cuh"

namespace prb {

namespace {

constexpr int kLL = 4, kLW = 8;

// ------------------------------------------------------------------ Newton pass
template <typename TIO, int L, int W, bool FIRST, bool LAST>
__global__ void __launch_bounds__(W * 32) lstm_newton_kernel(LstmFwdArgs a) {
    __shared__ float smem[(W * 6 + 2) * kLanes];
    __shared__ unsigned s_ticket;
    __shared__ unsigned s_red[W];
    const unsigned ticket = take_ticket(a.chain.ticket, &s_ticket);
    const int tt = ticket / a.chain.n_chains;
    const int chain = ticket % a.chain.n_chains;
    const int d = a.d;
    const int ncb = (d + kLanes - 1) / kLanes;
    const int b = chain / ncb, cb = chain % ncb;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ch = cb * kLanes + lane;
    const bool ch_ok = ch < d;
    const int chl = ch_ok ? ch : d - 1;
    const int t0 = tt * (W * L) + warp * L;

    float p[5];
#pragma unroll
    for (int q = 0; q < 5; ++q) p[q] = __ldg(a.par + (size_t)q * d + chl);
    const TIO* wx = reinterpret_cast<const TIO*>(a.wx) + (size_t)b * a.T * 3 * d + chl;
    const float h0c = a.halo ? __ldg(a.halo + ((size_t)b * 2 + 0) * d + chl) : 0.f;
    const float h0h = a.halo ? __ldg(a.halo + ((size_t)b * 2 + 1) * d + chl) : 0.f;

    float w[L][3], st[L + 1][2];
#pragma unroll
    for (int i = 0; i < L; ++i) {
        const int t = min(t0 + i, a.T - 1);
#pragma unroll
        for (int q = 0; q < 3; ++q) w[i][q] = ld_f(wx + ((size_t)t * 3 + q) * d);
    }
    if (FIRST) {
        // App.-A guess on the fly: H^0_t = f(0, x_t), the initial state only at t = 0
        if (t0 == 0) {
            st[0][0] = h0c;
            st[0][1] = h0h;
        } else {
            const int t = min(t0 - 1, a.T - 1);
            float g[3];
#pragma unroll
            for (int q = 0; q < 3; ++q) g[q] = ld_f(wx + ((size_t)t * 3 + q) * d);
            LstmActs ac;
            lstm_step(t == 0 ? h0c : 0.f, t == 0 ? h0h : 0.f, g, p, ac);
            st[0][0] = ac.cn;
            st[0][1] = ac.hn;
        }
#pragma unroll
        for (int i = 0; i < L; ++i) {
            LstmActs ac;
            lstm_step(t0 + i == 0 ? h0c : 0.f, t0 + i == 0 ? h0h : 0.f, w[i], p, ac);
            st[i + 1][0] = ac.cn;
            st[i + 1][1] = ac.hn;
        }
    } else {
        const float* sin = a.sin + (size_t)b * a.T * 2 * d + chl;
#pragma unroll
        for (int i = 0; i < L; ++i) {
            const int t = min(t0 + i, a.T - 1);
            st[i + 1][0] = __ldg(sin + ((size_t)t * 2 + 0) * d);
            st[i + 1][1] = __ldg(sin + ((size_t)t * 2 + 1) * d);
        }
        if (t0 == 0) {
            st[0][0] = h0c;
            st[0][1] = h0h;
        } else {
            const int t = min(t0 - 1, a.T - 1);
            st[0][0] = __ldg(sin + ((size_t)t * 2 + 0) * d);
            st[0][1] = __ldg(sin + ((size_t)t * 2 + 1) * d);
        }
    }

    float J[L][4], F[L][2];
    float mp[6] = {1.f, 0.f, 0.f, 1.f, 0.f, 0.f};
    unsigned rmax = 0u;
#pragma unroll
    for (int i = 0; i < L; ++i) {
        LstmActs ac;
        lstm_step(st[i][0], st[i][1], w[i], p, ac);
        lstm_jac(ac, st[i][0], p, J[i]);
        F[i][0] = ac.cn - st[i + 1][0];
        F[i][1] = ac.hn - st[i + 1][1];
        if (t0 + i >= a.T) {  // identity step beyond the end of the sequence
            J[i][0] = 1.f; J[i][1] = 0.f; J[i][2] = 0.f; J[i][3] = 1.f;
            F[i][0] = F[i][1] = 0.f;
        } else if (ch_ok) {
            rmax = max(rmax, max(absbits(F[i][0]), absbits(F[i][1])));
        }
        const float step_map[6] = {J[i][0], J[i][1], J[i][2], J[i][3], F[i][0], F[i][1]};
        Affine2::compose(mp, step_map);
    }
    float boundary[2] = {0.f, 0.f};
    float carry[2], tile_end[2];
    tile_exchange<Affine2, W>(a.chain, chain, tt, mp, boundary, carry, smem, tile_end);

    float dc = carry[0], dh = carry[1];
    float pc = fmaf(a.omega, dc, st[0][0]), ph = fmaf(a.omega, dh, st[0][1]);  // updated previous state
    unsigned fmax = 0u;
    const bool want_final = LAST && a.final_bits != nullptr;
#pragma unroll
    for (int i = 0; i < L; ++i) {
        const int t = t0 + i;
        const float nc = fmaf(J[i][0], dc, fmaf(J[i][1], dh, F[i][0]));
        const float nh = fmaf(J[i][2], dc, fmaf(J[i][3], dh, F[i][1]));
        dc = nc;
        dh = nh;
        if (t < a.T && ch_ok) {
            const float oc = fmaf(a.omega, dc, st[i + 1][0]), oh = fmaf(a.omega, dh, st[i + 1][1]);
            if (want_final) {
                LstmActs ac;
                lstm_step(pc, ph, w[i], p, ac);
                fmax = max(fmax, max(absbits(ac.cn - oc), absbits(ac.hn - oh)));
                pc = oc;
                ph = oh;
            }
            if (LAST) {
                TIO* o = reinterpret_cast<TIO*>(a.sout) + ((size_t)b * a.T + t) * 2 * d + ch;
                st_f(o, oc);
                st_f(o + d, oh);
            } else {
                float* o = reinterpret_cast<float*>(a.sout) + ((size_t)b * a.T + t) * 2 * d + ch;
                o[0] = oc;
                o[d] = oh;
            }
        }
    }
    block_residual_max(rmax, a.resid_bits, s_red);
    if (want_final) {
        __syncthreads();
        block_residual_max(fmax, a.final_bits, s_red);
    }
}

// Initial guess alone (K = 0) and the residual of a stored trajectory.
template <typename TIO, typename TST, bool GUESS>
__global__ void __launch_bounds__(256) lstm_pointwise_kernel(const TIO* wx, const float* par, const float* h0,
                                                              TST* st, int B, int T, int d, unsigned* dst) {
    __shared__ unsigned s_red[8];
    unsigned rmax = 0u;
    const size_t n = (size_t)B * T * d;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n;
         idx += (size_t)gridDim.x * blockDim.x) {
        const int ch = idx % d;
        const size_t bt = idx / d;
        const int t = bt % T, b = bt / T;
        float p[5], g[3];
#pragma unroll
        for (int q = 0; q < 5; ++q) p[q] = __ldg(par + (size_t)q * d + ch);
#pragma unroll
        for (int q = 0; q < 3; ++q) g[q] = ld_f(wx + (bt * 3 + q) * d + ch);
        float c = 0.f, h = 0.f;
        if (t == 0) {
            c = h0 ? __ldg(h0 + ((size_t)b * 2 + 0) * d + ch) : 0.f;
            h = h0 ? __ldg(h0 + ((size_t)b * 2 + 1) * d + ch) : 0.f;
        } else if (!GUESS) {
            c = ld_f(st + ((bt - 1) * 2 + 0) * d + ch);
            h = ld_f(st + ((bt - 1) * 2 + 1) * d + ch);
        }
        LstmActs ac;
        lstm_step(c, h, g, p, ac);
        if (GUESS) {
            st_f(st + (bt * 2 + 0) * d + ch, ac.cn);
            st_f(st + (bt * 2 + 1) * d + ch, ac.hn);
        } else {
            rmax = max(rmax, max(absbits(ac.cn - ld_f(st + (bt * 2 + 0) * d + ch)),
                                 absbits(ac.hn - ld_f(st + (bt * 2 + 1) * d + ch))));
        }
    }
    if (!GUESS) block_residual_max(rmax, dst, s_red);
}

// ------------------------------------------------------------------ backward
// nu_{t-1} = J_t^T (nu_t + g_t), nu_{T-1} = 0, mu_t = nu_t + g_t, grad_h0 = nu_{-1}; tiles are
// walked from the end of the sequence, within a thread steps run from high t to low t.
template <typename TIO, int L, int W>
__global__ void __launch_bounds__(W * 32) lstm_bwd_kernel(LstmBwdArgs a) {
    __shared__ float smem[(W * 6 + 2) * kLanes];
    __shared__ unsigned s_ticket;
    const unsigned ticket = take_ticket(a.chain.ticket, &s_ticket);
    const int tt = ticket / a.chain.n_chains;
    const int chain = ticket % a.chain.n_chains;
    const int d = a.d;
    const int ncb = (d + kLanes - 1) / kLanes;
    const int b = chain / ncb, cb = chain % ncb;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ch = cb * kLanes + lane;
    const bool ch_ok = ch < d;
    const int chl = ch_ok ? ch : d - 1;
    const int tile_t = a.chain.n_tt - 1 - tt;
    const int t_hi = tile_t * (W * L) + (W - 1 - warp) * L + (L - 1);

    float p[5];
#pragma unroll
    for (int q = 0; q < 5; ++q) p[q] = __ldg(a.par + (size_t)q * d + chl);
    const TIO* wx = reinterpret_cast<const TIO*>(a.wx) + (size_t)b * a.T * 3 * d + chl;
    const TIO* sp = reinterpret_cast<const TIO*>(a.states) + (size_t)b * a.T * 2 * d + chl;
    const TIO* gs = reinterpret_cast<const TIO*>(a.grad_states) + (size_t)b * a.T * 2 * d + chl;

    LstmActs act[L];
    float J[L][4], g[L][2], prev[L][2];
    float mp[6] = {1.f, 0.f, 0.f, 1.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < L; ++i) {
        const int t = t_hi - i;
        const bool ok = t < a.T;
        const int tc = min(t, a.T - 1);
        float w[3];
#pragma unroll
        for (int q = 0; q < 3; ++q) w[q] = ld_f(wx + ((size_t)tc * 3 + q) * d);
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            prev[i][q] = (tc == 0) ? (a.halo ? __ldg(a.halo + ((size_t)b * 2 + q) * d + chl) : 0.f)
                                   : ld_f(sp + ((size_t)(tc - 1) * 2 + q) * d);
            g[i][q] = ok ? ld_f(gs + ((size_t)tc * 2 + q) * d) : 0.f;
        }
        lstm_step(prev[i][0], prev[i][1], w, p, act[i]);
        lstm_jac(act[i], prev[i][0], p, J[i]);
        if (!ok) {
            J[i][0] = 1.f; J[i][1] = 0.f; J[i][2] = 0.f; J[i][3] = 1.f;
        }
        // map of one reverse step: nu -> J^T (nu + g)
        const float step_map[6] = {J[i][0], J[i][2], J[i][1], J[i][3],
                                   fmaf(J[i][0], g[i][0], J[i][2] * g[i][1]),
                                   fmaf(J[i][1], g[i][0], J[i][3] * g[i][1])};
        Affine2::compose(mp, step_map);
    }
    float boundary[2] = {0.f, 0.f};
    float carry[2], tile_end[2];
    tile_exchange<Affine2, W>(a.chain, chain, tt, mp, boundary, carry, smem, tile_end);

    float nc = carry[0], nh = carry[1];
    float gp[5] = {0.f, 0.f, 0.f, 0.f, 0.f};
    TIO* gwx = reinterpret_cast<TIO*>(a.g_wx) + (size_t)b * a.T * 3 * d + ch;
#pragma unroll
    for (int i = 0; i < L; ++i) {
        const int t = t_hi - i;
        if (t < a.T) {
            const LstmActs& s = act[i];
            const float mc = nc + g[i][0], mh = nh + g[i][1];
            const float d_opre = mh * s.hact * s.o * (1.f - s.o);
            const float d_cn = fmaf(mh, s.o * (1.f - s.hact * s.hact), fmaf(d_opre, p[4], mc));
            const float d_fpre = d_cn * (prev[i][0] - s.z) * s.f * (1.f - s.f);
            const float d_zpre = d_cn * (1.f - s.f) * (1.f - s.z * s.z);
            if (ch_ok) {
                TIO* o = gwx + (size_t)t * 3 * d;
                st_f(o, d_fpre);
                st_f(o + d, d_zpre);
                st_f(o + 2 * (size_t)d, d_opre);
            }
            gp[0] = fmaf(d_fpre, prev[i][1], gp[0]);
            gp[1] = fmaf(d_zpre, prev[i][1], gp[1]);
            gp[2] = fmaf(d_opre, prev[i][1], gp[2]);
            gp[3] = fmaf(d_fpre, prev[i][0], gp[3]);
            gp[4] = fmaf(d_opre, s.cn, gp[4]);
            nc = fmaf(J[i][0], mc, J[i][2] * mh);
            nh = fmaf(J[i][1], mc, J[i][3] * mh);
        }
    }
    if (ch_ok && warp == 0 && tt == a.chain.n_tt - 1 && a.g_h0) {
        a.g_h0[((size_t)b * 2 + 0) * d + ch] = tile_end[0];
        a.g_h0[((size_t)b * 2 + 1) * d + ch] = tile_end[1];
    }
    __syncthreads();
    float* s_gp = smem;  // W * 5 * 32 floats fit in the (W * 6 + 2) * 32 of the exchange
#pragma unroll
    for (int q = 0; q < 5; ++q) s_gp[(warp * 5 + q) * kLanes + lane] = gp[q];
    __syncthreads();
    if (warp == 0 && ch_ok) {
#pragma unroll
        for (int q = 0; q < 5; ++q) {
            float s = 0.f;
#pragma unroll
            for (int w2 = 0; w2 < W; ++w2) s += s_gp[(w2 * 5 + q) * kLanes + lane];
            a.gp_partial[(((size_t)b * a.chain.n_tt + tile_t) * 5 + q) * d + ch] = s;
        }
    }
}

template <typename TIO>
cudaError_t launch_fwd_t(const LstmFwdArgs& a, bool first, bool last, cudaStream_t s) {
    const unsigned grid = (unsigned)(a.chain.n_chains * a.chain.n_tt);
    const dim3 blk(kLW * 32);
    if (first && last)
        lstm_newton_kernel<TIO, kLL, kLW, true, true><<<grid, blk, 0, s>>>(a);
    else if (first)
        lstm_newton_kernel<TIO, kLL, kLW, true, false><<<grid, blk, 0, s>>>(a);
    else if (last)
        lstm_newton_kernel<TIO, kLL, kLW, false, true><<<grid, blk, 0, s>>>(a);
    else
        lstm_newton_kernel<TIO, kLL, kLW, false, false><<<grid, blk, 0, s>>>(a);
    return cudaGetLastError();
}

}  // namespace

int lstm_tile_steps() { return kLL * kLW; }

cudaError_t launch_lstm_newton(int dtype, const LstmFwdArgs& a, bool first, bool last, cudaStream_t s) {
    return dtype == kF32 ? launch_fwd_t<float>(a, first, last, s) : launch_fwd_t<__nv_bfloat16>(a, first, last, s);
}

cudaError_t launch_lstm_guess(int dtype, const void* wx, const float* par, const float* h0, void* out, int B,
                              int T, int d, cudaStream_t s) {
    const size_t n = (size_t)B * T * d;
    const int blocks = (int)min((size_t)sm_count() * 16, (n + 255) / 256);
    if (dtype == kF32)
        lstm_pointwise_kernel<float, float, true><<<blocks, 256, 0, s>>>((const float*)wx, par, h0, (float*)out,
                                                                         B, T, d, nullptr);
    else
        lstm_pointwise_kernel<__nv_bfloat16, __nv_bfloat16, true><<<blocks, 256, 0, s>>>(
            (const __nv_bfloat16*)wx, par, h0, (__nv_bfloat16*)out, B, T, d, nullptr);
    return cudaGetLastError();
}

cudaError_t launch_lstm_residual(int dtype, const void* wx, const float* par, const float* h0, const void* st,
                                 int B, int T, int d, unsigned* dst, cudaStream_t s) {
    const size_t n = (size_t)B * T * d;
    const int blocks = (int)min((size_t)sm_count() * 16, (n + 255) / 256);
    if (dtype == kF32)
        lstm_pointwise_kernel<float, float, false><<<blocks, 256, 0, s>>>((const float*)wx, par, h0,
                                                                          (float*)const_cast<void*>(st), B, T, d, dst);
    else
        lstm_pointwise_kernel<__nv_bfloat16, __nv_bfloat16, false><<<blocks, 256, 0, s>>>(
            (const __nv_bfloat16*)wx, par, h0, (__nv_bfloat16*)const_cast<void*>(st), B, T, d, dst);
    return cudaGetLastError();
}

cudaError_t launch_lstm_bwd(int dtype, const LstmBwdArgs& a, cudaStream_t s) {
    const unsigned grid = (unsigned)(a.chain.n_chains * a.chain.n_tt);
    const dim3 blk(kLW * 32);
    if (dtype == kF32)
        lstm_bwd_kernel<float, kLL, kLW><<<grid, blk, 0, s>>>(a);
    else
        lstm_bwd_kernel<__nv_bfloat16, kLL, kLW><<<grid, blk, 0, s>>>(a);
    return cudaGetLastError();
}

}  // namespace prb
