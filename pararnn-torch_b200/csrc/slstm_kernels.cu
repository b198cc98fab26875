// ParaSLSTM mix='diag' (state slots c, n, m, h; gates i, f, z, o): frozen-gate
// Picard pass, fused Newton pass with the structured 4x4 Jacobian, residual
// gate, and the fused reverse-time adjoint scan with the packed VJP.
//
// Reference behaviour restated here (paths relative to the reference project):
//   cells/para_slstm.py:347-446            step and 4x4 Jacobian (12 non-zeros)
//   solvers/slstm_picard.py:51-181          frozen-gate scan and Picard passes
//   solvers/newton/__init__.py:467-549      Newton loop
//   solvers/scan.py:166-178                 eq. 2.6 reverse scan with J^T
//   kernels/vjp_slstm.py:170-231            packed VJP
#include <math_constants.h>

#include "common.cuh"
#include "kernels.h"
#include "slstm_cell.cuh"

namespace prb {

// ------------------------------------------------------------------ Picard
template <typename TIO, int L, int W, bool AGG>
__global__ void __launch_bounds__(W * 32) slstm_picard_kernel(SlstmPicardArgs a) {
    using M = PicardMonoid;
    using MC = MapCarry<PicardMonoid>;
    __shared__ float smem[(W * 4 + 4) * kLanes];
    __shared__ unsigned s_ticket;
    const unsigned ticket = take_ticket(a.chain.ticket, &s_ticket);
    const int tt = ticket / a.chain.n_chains;
    const int chain = ticket % a.chain.n_chains;
    const int ncb = (a.d + kLanes - 1) / kLanes;
    const int b = chain / ncb, cb = chain % ncb;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ch = cb * kLanes + lane;
    const bool ch_ok = ch < a.d;
    const int chl = ch_ok ? ch : a.d - 1;
    const int t0 = tt * (W * L) + warp * L;
    const int d = a.d;

    const TIO* wx = reinterpret_cast<const TIO*>(a.wx) + (size_t)b * a.T * 4 * d + chl;
    float r4[4] = {0.f, 0.f, 0.f, 0.f};
    float hp[L];
    if (a.h_prev) {
#pragma unroll
        for (int q = 0; q < 4; ++q) r4[q] = __ldg(a.r + (size_t)q * d + chl);
        const float* hpv = a.h_prev + (size_t)b * a.T * d + chl;
#pragma unroll
        for (int i = 0; i < L; ++i) {
            const int t = t0 + i;
            hp[i] = (t == 0) ? (a.h_halo ? __ldg(a.h_halo + (size_t)b * a.halo_stride + chl) : 0.f)
                             : __ldg(hpv + (size_t)min(t - 1, a.T - 1) * d);
        }
    } else {
#pragma unroll
        for (int i = 0; i < L; ++i) hp[i] = 0.f;
    }
    float zi[L], zf[L], zz[L], zo[L];
#pragma unroll
    for (int i = 0; i < L; ++i) {
        const int t = min(t0 + i, a.T - 1);
        const TIO* w = wx + (size_t)t * 4 * d;
        zi[i] = fmaf(r4[0], hp[i], ld_f(w));
        zf[i] = fmaf(r4[1], hp[i], ld_f(w + d));
        zz[i] = tanh_f(fmaf(r4[2], hp[i], ld_f(w + 2 * (size_t)d)));
        zo[i] = fmaf(r4[3], hp[i], ld_f(w + 3 * (size_t)d));
    }
    // sub-tile summary
    float mp[4] = {0.f, -CUDART_INF_F, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < L; ++i) {
        if (t0 + i < a.T) {
            const float b1a = mp[1] + zf[i];
            const float e = exp_f(-fabsf(b1a - zi[i]));
            const bool left = b1a >= zi[i];
            const float s1 = left ? 1.f : e, s2 = left ? e : 1.f;
            mp[0] += zf[i];
            mp[1] = left ? b1a : zi[i];
            mp[2] = fmaf(mp[2], s1, s2);
            mp[3] = fmaf(mp[3], s1, s2 * zz[i]);
        }
    }
    if (AGG) {
        float boundary[4] = {0.f, -CUDART_INF_F, 0.f, 0.f};
        float carry[4], tile_end[4];
        tile_exchange<MC, W>(a.chain, chain, tt, mp, boundary, carry, smem, tile_end);
        if (ch_ok && warp == 0 && tt == a.chain.n_tt - 1) {
#pragma unroll
            for (int q = 0; q < 4; ++q) a.agg_out[((size_t)b * 4 + q) * d + ch] = tile_end[q];
        }
        return;
    }
    float boundary[3] = {0.f, 0.f, 0.f};
    if (a.carry_in) {
#pragma unroll
        for (int q = 0; q < 3; ++q) boundary[q] = __ldg(a.carry_in + (size_t)b * a.carry_stride + (size_t)q * d + chl);
    }
    float carry[3], tile_end[3];
    tile_exchange<M, W>(a.chain, chain, tt, mp, boundary, carry, smem, tile_end);
    float c = carry[0], n = carry[1], m = carry[2];
#pragma unroll
    for (int i = 0; i < L; ++i) {
        const int t = t0 + i;
        if (t < a.T) {
            const float left = zf[i] + m;
            const float e = exp_f(-fabsf(left - zi[i]));
            const bool lw = left >= zi[i];
            const float ft = lw ? 1.f : e, it = lw ? e : 1.f;
            // a tie gives ft = it = exp(0) = 1 in the reference; here e = 1 as well
            m = lw ? left : zi[i];
            n = fmaf(ft, n, it);
            c = fmaf(ft, c, it * zz[i]);
            const float h = sigmoid_f(zo[i]) * (c * rcp_f(n + a.eps));
            if (ch_ok) {
                if (a.state_out) {
                    float* o = a.state_out + ((size_t)b * a.T + t) * 4 * d + ch;
                    o[0] = c;
                    o[d] = n;
                    o[2 * (size_t)d] = m;
                    o[3 * (size_t)d] = h;
                } else {
                    a.h_out[((size_t)b * a.T + t) * d + ch] = h;
                }
            }
        }
    }
    if (a.tail_out && ch_ok && warp == 0 && tt == a.chain.n_tt - 1) {
#pragma unroll
        for (int q = 0; q < 3; ++q) a.tail_out[((size_t)b * 3 + q) * d + ch] = tile_end[q];
    }
}

// ------------------------------------------------------------------ Newton
template <typename TIO, int L, int W, bool LAST, bool AGG>
__global__ void __launch_bounds__(W * 32) slstm_newton_kernel(SlstmNewtonArgs a) {
    __shared__ float smem[(W * 20 + 20) * kLanes];
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

    float r4[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) r4[q] = __ldg(a.r + (size_t)q * d + chl);
    const TIO* wx = reinterpret_cast<const TIO*>(a.wx) + (size_t)b * a.T * 4 * d + chl;
    const float* sin = a.sin + (size_t)b * a.T * 4 * d + chl;

    float w[L][4], st[L + 1][4];
#pragma unroll
    for (int i = 0; i < L; ++i) {
        const int t = min(t0 + i, a.T - 1);
#pragma unroll
        for (int q = 0; q < 4; ++q) w[i][q] = ld_f(wx + ((size_t)t * 4 + q) * d);
#pragma unroll
        for (int q = 0; q < 4; ++q) st[i + 1][q] = __ldg(sin + ((size_t)t * 4 + q) * d);
    }
    if (t0 == 0) {
#pragma unroll
        for (int q = 0; q < 4; ++q)
            st[0][q] = a.halo ? __ldg(a.halo + (size_t)b * a.halo_stride + (size_t)q * d + chl) : 0.f;
    } else {
        const int t = min(t0 - 1, a.T - 1);
#pragma unroll
        for (int q = 0; q < 4; ++q) st[0][q] = __ldg(sin + ((size_t)t * 4 + q) * d);
    }

    SlstmLin lin[L];
    float F[L][4];
    float mp[20];
    unsigned rmax = 0u;
#pragma unroll
    for (int i = 0; i < L; ++i) {
        slstm_linearize(st[i], w[i], r4, a.eps, lin[i]);
        const bool ok = t0 + i < a.T;
        float fc = lin[i].pc - st[i + 1][0], fn = lin[i].pn - st[i + 1][1];
        float fm = lin[i].pm - st[i + 1][2], fh = lin[i].ph - st[i + 1][3];
        if (!ok) {
            // identity step beyond the end of the sequence
            lin[i].f = 1.f; lin[i].jcm = 0.f; lin[i].jch = 0.f; lin[i].jnm = 0.f; lin[i].jnh = 0.f;
            lin[i].alpha = 1.f; lin[i].dm = 0.f; lin[i].ia = 0.f; lin[i].ib = 0.f; lin[i].ie = 1.f;
            fc = fn = fm = fh = 0.f;
        } else if (ch_ok) {
            rmax = max(rmax, max(max(absbits(fc), absbits(fn)), max(absbits(fm), absbits(fh))));
        }
        F[i][0] = fc;
        F[i][1] = fn;
        F[i][2] = fm;
        F[i][3] = fh - lin[i].ia * fc - lin[i].ib * fn;
        if (i == 0) {
#pragma unroll
            for (int k = 0; k < 20; ++k) mp[k] = 0.f;
            mp[0] = 1.f; mp[5] = 1.f; mp[10] = 1.f; mp[15] = 1.f;
        }
        // columns k = 0..3 of M and the offset column v (k = 4)
#pragma unroll
        for (int k = 0; k < 5; ++k) {
            const bool off = (k == 4);
            float xc = off ? mp[16] : mp[0 * 4 + k], xn = off ? mp[17] : mp[1 * 4 + k];
            float xm = off ? mp[18] : mp[2 * 4 + k], xh = off ? mp[19] : mp[3 * 4 + k];
            slstm_apply(lin[i], off ? F[i][0] : 0.f, off ? F[i][1] : 0.f, off ? F[i][2] : 0.f,
                        off ? F[i][3] : 0.f, xc, xn, xm, xh);
            if (off) {
                mp[16] = xc; mp[17] = xn; mp[18] = xm; mp[19] = xh;
            } else {
                mp[0 * 4 + k] = xc; mp[1 * 4 + k] = xn; mp[2 * 4 + k] = xm; mp[3 * 4 + k] = xh;
            }
        }
    }
    if (AGG) {
        using MC = MapCarry<Affine4>;
        float boundary[20];
#pragma unroll
        for (int k = 0; k < 20; ++k) boundary[k] = 0.f;
        boundary[0] = boundary[5] = boundary[10] = boundary[15] = 1.f;
        float carry[20], tile_end[20];
        tile_exchange<MC, W>(a.chain, chain, tt, mp, boundary, carry, smem, tile_end);
        if (ch_ok && warp == 0 && tt == a.chain.n_tt - 1) {
#pragma unroll
            for (int k = 0; k < 20; ++k) a.agg_out[((size_t)b * 20 + k) * d + ch] = tile_end[k];
        }
        return;
    }
    float boundary[4] = {0.f, 0.f, 0.f, 0.f};
    if (a.carry_in) {
#pragma unroll
        for (int q = 0; q < 4; ++q) boundary[q] = __ldg(a.carry_in + ((size_t)b * 4 + q) * d + chl);
    }
    float carry[4], tile_end[4];
    tile_exchange<Affine4, W>(a.chain, chain, tt, mp, boundary, carry, smem, tile_end);

    float xc = carry[0], xn = carry[1], xm = carry[2], xh = carry[3];
    // On the last pass the residual of the RETURNED trajectory is evaluated here, on the fp32
    // values before they are rounded to the I/O dtype: F(H^K)_t = f(H^K_{t-1}, x_t) - H^K_t,
    // where H^K at the step before this sub-tile is the old state plus omega times the carry.
    float pn4[4] = {fmaf(a.omega, xc, st[0][0]), fmaf(a.omega, xn, st[0][1]),
                    fmaf(a.omega, xm, st[0][2]), fmaf(a.omega, xh, st[0][3])};
    unsigned fmax = 0u;
    const bool want_final = LAST && a.final_bits != nullptr;
#pragma unroll
    for (int i = 0; i < L; ++i) {
        const int t = t0 + i;
        slstm_apply(lin[i], F[i][0], F[i][1], F[i][2], F[i][3], xc, xn, xm, xh);
        if (t < a.T && ch_ok) {
            const float o0 = fmaf(a.omega, xc, st[i + 1][0]), o1 = fmaf(a.omega, xn, st[i + 1][1]);
            const float o2 = fmaf(a.omega, xm, st[i + 1][2]), o3 = fmaf(a.omega, xh, st[i + 1][3]);
            if (want_final) {
                float pred[4];
                slstm_predict(pn4, w[i], r4, a.eps, pred);
                fmax = max(fmax, max(max(absbits(pred[0] - o0), absbits(pred[1] - o1)),
                                     max(absbits(pred[2] - o2), absbits(pred[3] - o3))));
                pn4[0] = o0; pn4[1] = o1; pn4[2] = o2; pn4[3] = o3;
            }
            if (LAST) {
                TIO* o = reinterpret_cast<TIO*>(a.sout) + ((size_t)b * a.T + t) * 4 * d + ch;
                st_f(o, o0);
                st_f(o + d, o1);
                st_f(o + 2 * (size_t)d, o2);
                st_f(o + 3 * (size_t)d, o3);
            } else {
                float* o = reinterpret_cast<float*>(a.sout) + ((size_t)b * a.T + t) * 4 * d + ch;
                o[0] = o0;
                o[d] = o1;
                o[2 * (size_t)d] = o2;
                o[3 * (size_t)d] = o3;
            }
        }
    }
    if (a.tail_out && ch_ok && warp == 0 && tt == a.chain.n_tt - 1) {
#pragma unroll
        for (int q = 0; q < 4; ++q) a.tail_out[((size_t)b * 4 + q) * d + ch] = tile_end[q];
    }
    block_residual_max(rmax, a.resid_bits, s_red);
    if (want_final) {
        __syncthreads();
        block_residual_max(fmax, a.final_bits, s_red);
    }
}

// ------------------------------------------------------------------ residual
template <typename TIO, typename TST, int L>
__global__ void __launch_bounds__(256) slstm_residual_kernel(const TIO* wx, const float* r,
                                                              const float* halo, int halo_stride,
                                                              const TST* st, int B, int T, int d,
                                                              float eps, unsigned* dst) {
    __shared__ unsigned s_red[8];
    const int ncb = (d + kLanes - 1) / kLanes;
    const int ntt = (T + 8 * L - 1) / (8 * L);
    const int tt = blockIdx.x % ntt;
    const int chain = blockIdx.x / ntt;
    const int b = chain / ncb, cb = chain % ncb;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ch = cb * kLanes + lane;
    unsigned rmax = 0u;
    const int t0 = tt * 8 * L + warp * L;
    if (ch < d && t0 < T) {
        float r4[4], prev[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) r4[q] = __ldg(r + (size_t)q * d + ch);
        const TST* s = st + (size_t)b * T * 4 * d + ch;
        const TIO* w = wx + (size_t)b * T * 4 * d + ch;
#pragma unroll
        for (int q = 0; q < 4; ++q)
            prev[q] = (t0 == 0) ? (halo ? __ldg(halo + (size_t)b * halo_stride + (size_t)q * d + ch) : 0.f)
                                : ld_f(s + ((size_t)(t0 - 1) * 4 + q) * d);
        for (int i = 0; i < L && t0 + i < T; ++i) {
            const int t = t0 + i;
            float g[4], cur[4], pred[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) g[q] = ld_f(w + ((size_t)t * 4 + q) * d);
#pragma unroll
            for (int q = 0; q < 4; ++q) cur[q] = ld_f(s + ((size_t)t * 4 + q) * d);
            slstm_predict(prev, g, r4, eps, pred);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                rmax = max(rmax, absbits(pred[q] - cur[q]));
                prev[q] = cur[q];
            }
        }
    }
    block_residual_max(rmax, dst, s_red);
}

// ------------------------------------------------------------------ backward
//
// nu_{t-1} = J_t^T (nu_t + g_t), nu_{T-1} = 0, mu_t = nu_t + g_t, grad_h0 = nu_{-1}.
template <typename TIO, int L, int W, bool AGG>
__global__ void __launch_bounds__(W * 32) slstm_bwd_kernel(SlstmBwdArgs a) {
    __shared__ float smem[(W * 20 + 20) * kLanes];
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

    float r4[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) r4[q] = __ldg(a.r + (size_t)q * d + chl);
    const TIO* wx = reinterpret_cast<const TIO*>(a.wx) + (size_t)b * a.T * 4 * d + chl;
    const TIO* sp = reinterpret_cast<const TIO*>(a.states) + (size_t)b * a.T * 4 * d + chl;
    const TIO* gs = reinterpret_cast<const TIO*>(a.grad_states) + (size_t)b * a.T * (a.g_slot < 0 ? 4 : 1) * d + chl;

    SlstmAct act[L];
    float g[L][4];
    float mp[20];
#pragma unroll
    for (int i = 0; i < L; ++i) {
        const int t = t_hi - i;
        const bool ok = t < a.T;
        const int tc = min(t, a.T - 1);
        float w[4], prev[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) w[q] = ld_f(wx + ((size_t)tc * 4 + q) * d);
#pragma unroll
        for (int q = 0; q < 4; ++q)
            prev[q] = (tc == 0)
                          ? (a.halo ? __ldg(a.halo + (size_t)b * a.halo_stride + (size_t)q * d + chl) : 0.f)
                          : ld_f(sp + ((size_t)(tc - 1) * 4 + q) * d);
#pragma unroll
        for (int q = 0; q < 4; ++q) g[i][q] = (ok && a.g_slot < 0) ? ld_f(gs + ((size_t)tc * 4 + q) * d) : 0.f;
        if (ok && a.g_slot >= 0) {
            const float v = ld_f(gs + (size_t)tc * d);
#pragma unroll
            for (int q = 0; q < 4; ++q) g[i][q] = (q == a.g_slot) ? v : 0.f;
        }
        SlstmLin lin;
        slstm_linearize(prev, w, r4, a.eps, lin);
        // activations needed by the VJP in the apply phase
        {
            act[i].i = lin.it;
            act[i].f = lin.f;
            act[i].z = lin.z;
            act[i].o = lin.og;
            act[i].c = prev[0];
            act[i].n = prev[1];
            act[i].invD = lin.invD;
            act[i].alpha = lin.alpha;
            act[i].hp = prev[3];
        }
        if (!ok) {
            lin.f = 1.f; lin.jcm = 0.f; lin.jch = 0.f; lin.jnm = 0.f; lin.jnh = 0.f;
            lin.alpha = 1.f; lin.dm = 0.f; lin.ia = 0.f; lin.ib = 0.f; lin.ie = 1.f;
        }
        if (i == 0) {
#pragma unroll
            for (int k = 0; k < 20; ++k) mp[k] = 0.f;
            mp[0] = 1.f; mp[5] = 1.f; mp[10] = 1.f; mp[15] = 1.f;
        }
#pragma unroll
        for (int k = 0; k < 5; ++k) {
            const bool off = (k == 4);
            float xc = off ? mp[16] + g[i][0] : mp[0 * 4 + k], xn = off ? mp[17] + g[i][1] : mp[1 * 4 + k];
            float xm = off ? mp[18] + g[i][2] : mp[2 * 4 + k], xh = off ? mp[19] + g[i][3] : mp[3 * 4 + k];
            slstm_apply_t(lin, xc, xn, xm, xh);
            if (off) {
                mp[16] = xc; mp[17] = xn; mp[18] = xm; mp[19] = xh;
            } else {
                mp[0 * 4 + k] = xc; mp[1 * 4 + k] = xn; mp[2 * 4 + k] = xm; mp[3 * 4 + k] = xh;
            }
        }
    }
    if (AGG) {
        using MC = MapCarry<Affine4>;
        float boundary[20];
#pragma unroll
        for (int k = 0; k < 20; ++k) boundary[k] = 0.f;
        boundary[0] = boundary[5] = boundary[10] = boundary[15] = 1.f;
        float carry[20], tile_end[20];
        tile_exchange<MC, W>(a.chain, chain, tt, mp, boundary, carry, smem, tile_end);
        if (ch_ok && warp == 0 && tt == a.chain.n_tt - 1) {
#pragma unroll
            for (int k = 0; k < 20; ++k) a.agg_out[((size_t)b * 20 + k) * d + ch] = tile_end[k];
        }
        return;
    }
    float boundary[4] = {0.f, 0.f, 0.f, 0.f};
    if (a.carry_in) {
#pragma unroll
        for (int q = 0; q < 4; ++q) boundary[q] = __ldg(a.carry_in + ((size_t)b * 4 + q) * d + chl);
    }
    float carry[4], tile_end[4];
    tile_exchange<Affine4, W>(a.chain, chain, tt, mp, boundary, carry, smem, tile_end);

    float nc = carry[0], nn = carry[1], nm = carry[2], nh = carry[3];
    float gr[4] = {0.f, 0.f, 0.f, 0.f}, gb[4] = {0.f, 0.f, 0.f, 0.f};
    TIO* gwx = reinterpret_cast<TIO*>(a.g_wx) + (size_t)b * a.T * 4 * d + ch;
#pragma unroll
    for (int i = 0; i < L; ++i) {
        const int t = t_hi - i;
        if (t < a.T) {
            const SlstmAct& s = act[i];
            const float mc = nc + g[i][0], mn_ = nn + g[i][1], mm = nm + g[i][2], mh = nh + g[i][3];
            const float cn = fmaf(s.f, s.c, s.i * s.z);
            const float u = cn * s.invD;
            const float d_o = mh * u;
            const float d_cn = fmaf(mh, s.o * s.invD, mc);
            const float d_nn = fmaf(mh, -(s.o * u) * s.invD, mn_);
            const float d_f = fmaf(d_cn, s.c, d_nn * s.n);
            const float d_i = fmaf(d_cn, s.z, d_nn);
            const float d_z = d_cn * s.i;
            const float d_zo = d_o * s.o * (1.f - s.o);
            const float d_zz = d_z * (1.f - s.z * s.z);
            const float d_mn = mm - d_i * s.i - d_f * s.f;
            const float d_zi = fmaf(d_i, s.i, d_mn * (1.f - s.alpha));
            const float d_zf = fmaf(d_f, s.f, d_mn * s.alpha);
            if (ch_ok) {
                TIO* o = gwx + (size_t)t * 4 * d;
                st_f(o, d_zi);
                st_f(o + d, d_zf);
                st_f(o + 2 * (size_t)d, d_zz);
                st_f(o + 3 * (size_t)d, d_zo);
            }
            gr[0] = fmaf(d_zi, s.hp, gr[0]);
            gr[1] = fmaf(d_zf, s.hp, gr[1]);
            gr[2] = fmaf(d_zz, s.hp, gr[2]);
            gr[3] = fmaf(d_zo, s.hp, gr[3]);
            gb[0] += d_zi;
            gb[1] += d_zf;
            gb[2] += d_zz;
            gb[3] += d_zo;
            nc = d_cn * s.f;
            nn = d_nn * s.f;
            nm = d_zf;
            nh = fmaf(r4[0], d_zi, fmaf(r4[1], d_zf, fmaf(r4[2], d_zz, r4[3] * d_zo)));
        }
    }
    if (ch_ok && warp == 0 && tt == a.chain.n_tt - 1 && a.g_h0) {
#pragma unroll
        for (int q = 0; q < 4; ++q) a.g_h0[((size_t)b * 4 + q) * d + ch] = tile_end[q];
    }
    __syncthreads();
    float* s_gp = smem;
#pragma unroll
    for (int p = 0; p < 4; ++p) s_gp[(warp * 4 + p) * kLanes + lane] = gr[p];
    __syncthreads();
    if (warp == 0 && ch_ok) {
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            float s = 0.f;
#pragma unroll
            for (int w2 = 0; w2 < W; ++w2) s += s_gp[(w2 * 4 + p) * kLanes + lane];
            a.gp_partial[(((size_t)b * a.chain.n_tt + tile_t) * 4 + p) * d + ch] = s;
        }
    }
    if (a.gb_partial) {  // same fixed-order reduction for the bias terms
        __syncthreads();
#pragma unroll
        for (int p = 0; p < 4; ++p) s_gp[(warp * 4 + p) * kLanes + lane] = gb[p];
        __syncthreads();
        if (warp == 0 && ch_ok) {
#pragma unroll
            for (int p = 0; p < 4; ++p) {
                float s = 0.f;
#pragma unroll
                for (int w2 = 0; w2 < W; ++w2) s += s_gp[(w2 * 4 + p) * kLanes + lane];
                a.gb_partial[(((size_t)b * a.chain.n_tt + tile_t) * 4 + p) * d + ch] = s;
            }
        }
    }
}

// ------------------------------------------------------------------ launchers
constexpr int kPicL = 8, kPicW = 8;
constexpr int kNewL = 4, kNewW = 8;
int slstm_picard_tile_steps() { return kPicL * kPicW; }
int slstm_tile_steps() { return kNewL * kNewW; }

cudaError_t launch_slstm_picard(int dtype, const SlstmPicardArgs& a, bool agg_only, cudaStream_t s) {
    const unsigned grid = (unsigned)(a.chain.n_chains * a.chain.n_tt);
    const dim3 blk(kPicW * 32);
    if (dtype == kF32) {
        if (agg_only)
            slstm_picard_kernel<float, kPicL, kPicW, true><<<grid, blk, 0, s>>>(a);
        else
            slstm_picard_kernel<float, kPicL, kPicW, false><<<grid, blk, 0, s>>>(a);
    } else {
        if (agg_only)
            slstm_picard_kernel<__nv_bfloat16, kPicL, kPicW, true><<<grid, blk, 0, s>>>(a);
        else
            slstm_picard_kernel<__nv_bfloat16, kPicL, kPicW, false><<<grid, blk, 0, s>>>(a);
    }
    return cudaGetLastError();
}

cudaError_t launch_slstm_newton(int dtype, const SlstmNewtonArgs& a, bool last, bool agg_only,
                                cudaStream_t s) {
    const unsigned grid = (unsigned)(a.chain.n_chains * a.chain.n_tt);
    const dim3 blk(kNewW * 32);
#define PRB_NEWTON(TIO)                                                               \
    if (agg_only)                                                                     \
        slstm_newton_kernel<TIO, kNewL, kNewW, false, true><<<grid, blk, 0, s>>>(a);   \
    else if (last)                                                                    \
        slstm_newton_kernel<TIO, kNewL, kNewW, true, false><<<grid, blk, 0, s>>>(a);   \
    else                                                                              \
        slstm_newton_kernel<TIO, kNewL, kNewW, false, false><<<grid, blk, 0, s>>>(a);
    if (dtype == kF32) {
        PRB_NEWTON(float)
    } else {
        PRB_NEWTON(__nv_bfloat16)
    }
#undef PRB_NEWTON
    return cudaGetLastError();
}

cudaError_t launch_slstm_residual(int dtype, bool st_f32, const void* wx, const float* r,
                                  const float* halo, int halo_stride, const void* st, int B, int T,
                                  int d, float eps, unsigned* dst, cudaStream_t s) {
    constexpr int L = 4;
    const int ncb = (d + kLanes - 1) / kLanes;
    const int ntt = (T + 8 * L - 1) / (8 * L);
    const unsigned grid = (unsigned)(B * ncb * ntt);
    if (dtype == kF32)
        slstm_residual_kernel<float, float, L><<<grid, 256, 0, s>>>(
            (const float*)wx, r, halo, halo_stride, (const float*)st, B, T, d, eps, dst);
    else if (st_f32)
        slstm_residual_kernel<__nv_bfloat16, float, L><<<grid, 256, 0, s>>>(
            (const __nv_bfloat16*)wx, r, halo, halo_stride, (const float*)st, B, T, d, eps, dst);
    else
        slstm_residual_kernel<__nv_bfloat16, __nv_bfloat16, L><<<grid, 256, 0, s>>>(
            (const __nv_bfloat16*)wx, r, halo, halo_stride, (const __nv_bfloat16*)st, B, T, d, eps, dst);
    return cudaGetLastError();
}

cudaError_t launch_slstm_bwd(int dtype, const SlstmBwdArgs& a, bool agg_only, cudaStream_t s) {
    const unsigned grid = (unsigned)(a.chain.n_chains * a.chain.n_tt);
    const dim3 blk(kNewW * 32);
    if (dtype == kF32) {
        if (agg_only)
            slstm_bwd_kernel<float, kNewL, kNewW, true><<<grid, blk, 0, s>>>(a);
        else
            slstm_bwd_kernel<float, kNewL, kNewW, false><<<grid, blk, 0, s>>>(a);
    } else {
        if (agg_only)
            slstm_bwd_kernel<__nv_bfloat16, kNewL, kNewW, true><<<grid, blk, 0, s>>>(a);
        else
            slstm_bwd_kernel<__nv_bfloat16, kNewL, kNewW, false><<<grid, blk, 0, s>>>(a);
    }
    return cudaGetLastError();
}

}  // namespace prb
