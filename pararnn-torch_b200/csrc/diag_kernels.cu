// Scalar-diagonal cells (ParaGRU mix='diag', ParaNLRU): fused Newton pass
// (gate math + diagonal Jacobian + residual + chained linear scan + update),
// initial guess, residual gate, and the fused reverse-time adjoint scan with
// the packed VJP.
//
// Reference behaviour restated here (paths relative to the reference project):
//   cells/para_gru.py:418-467, cells/para_nlru.py:149-168      step + diagonal J
//   solvers/newton/__init__.py:467-549                          Newton loop
//   solvers/scan.py:126-148, solvers/newton/dispatch.py:406-441 eq. 2.6 reverse scan
//   kernels/vjp_gru.py:107-138, kernels/vjp_nlru.py:88-108      packed VJP
#include "common.cuh"
#include "diag_cell.cuh"
#include "kernels.h"

namespace prb {

// ------------------------------------------------------------------ forward
//
// Tile = (W warps x L steps) x 32 channels; lane = channel, warp = sub-tile.
template <int CELL, typename TIO, int L, int W, bool FIRST, bool LAST>
__global__ void __launch_bounds__(W * 32) diag_newton_kernel(DiagFwdArgs a) {
    using C = DiagCell<CELL>;
    constexpr int G = C::G;
    __shared__ float smem[(W * 2 + 2) * kLanes];
    __shared__ unsigned s_ticket;
    __shared__ unsigned s_red[W];

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

    float par[C::NP];
#pragma unroll
    for (int p = 0; p < C::NP; ++p) par[p] = __ldg(a.par + (size_t)p * a.d + chl);

    const TIO* wx = reinterpret_cast<const TIO*>(a.wx) + (size_t)b * a.T * G * a.d + chl;
    float g[L][G];
#pragma unroll
    for (int i = 0; i < L; ++i) {
        const int t = min(t0 + i, a.T - 1);
#pragma unroll
        for (int q = 0; q < G; ++q) g[i][q] = ld_f(wx + ((size_t)t * G + q) * a.d);
    }
    // old trajectory: hold[i+1] = H^k_{t0+i}, hold[0] = H^k_{t0-1}
    float hold[L + 1];
    const float h_init = a.halo ? __ldg(a.halo + (size_t)b * a.d + chl) : 0.f;
    if (FIRST) {
        // App. A guess evaluated on the fly: H^0_t = f(0, x_t), h0 only at t = 0.
        if (t0 == 0) {
            hold[0] = h_init;
        } else {
            float gp[G];
#pragma unroll
            for (int q = 0; q < G; ++q) gp[q] = ld_f(wx + ((size_t)min(t0 - 1, a.T - 1) * G + q) * a.d);
            hold[0] = C::step(t0 - 1 == 0 ? h_init : 0.f, gp, par);
        }
#pragma unroll
        for (int i = 0; i < L; ++i) hold[i + 1] = C::step(t0 + i == 0 ? h_init : 0.f, g[i], par);
    } else {
        const float* hin = a.hin + (size_t)b * a.T * a.d + chl;
        hold[0] = (t0 == 0) ? h_init : __ldg(hin + (size_t)min(t0 - 1, a.T - 1) * a.d);
#pragma unroll
        for (int i = 0; i < L; ++i) hold[i + 1] = __ldg(hin + (size_t)min(t0 + i, a.T - 1) * a.d);
    }

    // local linearisation and in-thread scan: delta_t = P_t * delta_in + D_t
    float P[L], D[L];
    unsigned rmax = 0u;
    {
        float pp = 1.f, dd = 0.f;
#pragma unroll
        for (int i = 0; i < L; ++i) {
            float f, j;
            typename C::Acts acts;
            C::eval(hold[i], g[i], par, f, j, acts);
            float F = f - hold[i + 1];
            const bool ok = (t0 + i < a.T);
            if (!ok) {
                j = 1.f;
                F = 0.f;
            }
            if (ok && ch_ok) rmax = max(rmax, absbits(F));
            dd = fmaf(j, dd, F);
            pp = j * pp;
            P[i] = pp;
            D[i] = dd;
        }
    }
    float my_map[2] = {P[L - 1], D[L - 1]};
    float boundary[1] = {a.carry_in ? __ldg(a.carry_in + (size_t)b * a.d + chl) : 0.f};
    float carry[1], tile_end[1];
    tile_exchange<Affine1, W>(a.chain, chain, tt, my_map, boundary, carry, smem, tile_end);

    unsigned fmax = 0u;
    const bool want_final = LAST && a.final_bits != nullptr;
    if (ch_ok) {
        if (LAST) {
            // the residual of the returned trajectory is evaluated on the fp32 values before
            // rounding; the new state preceding this sub-tile is old state + omega * carry
            TIO* out = reinterpret_cast<TIO*>(a.hout) + (size_t)b * a.T * a.d + ch;
            float prev_new = fmaf(a.omega, carry[0], hold[0]);
#pragma unroll
            for (int i = 0; i < L; ++i)
                if (t0 + i < a.T) {
                    const float nv = fmaf(a.omega, fmaf(P[i], carry[0], D[i]), hold[i + 1]);
                    if (want_final) {
                        fmax = max(fmax, absbits(C::step(prev_new, g[i], par) - nv));
                        prev_new = nv;
                    }
                    st_f(out + (size_t)(t0 + i) * a.d, nv);
                }
        } else {
            float* out = reinterpret_cast<float*>(a.hout) + (size_t)b * a.T * a.d + ch;
#pragma unroll
            for (int i = 0; i < L; ++i)
                if (t0 + i < a.T)
                    out[(size_t)(t0 + i) * a.d] = fmaf(a.omega, fmaf(P[i], carry[0], D[i]), hold[i + 1]);
        }
        if (a.tail_out && warp == 0 && tt == a.chain.n_tt - 1)
            a.tail_out[(size_t)b * a.d + ch] = tile_end[0];
    }
    block_residual_max(rmax, a.resid_bits, s_red);
    if (want_final) {
        __syncthreads();
        block_residual_max(fmax, a.final_bits, s_red);
    }
}

// Aggregate-only sweep over a time shard: same linearisation, but the chain
// carries maps, nothing is written except the shard aggregate (a, b) per channel.
template <int CELL, typename TIO, int L, int W>
__global__ void __launch_bounds__(W * 32) diag_newton_agg_kernel(DiagFwdArgs a) {
    using C = DiagCell<CELL>;
    constexpr int G = C::G;
    using MC = MapCarry<Affine1>;
    __shared__ float smem[(W * 2 + 2) * kLanes];
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
    float par[C::NP];
#pragma unroll
    for (int p = 0; p < C::NP; ++p) par[p] = __ldg(a.par + (size_t)p * a.d + chl);
    const TIO* wx = reinterpret_cast<const TIO*>(a.wx) + (size_t)b * a.T * G * a.d + chl;
    const float* hin = a.hin + (size_t)b * a.T * a.d + chl;
    const float h_init = a.halo ? __ldg(a.halo + (size_t)b * a.d + chl) : 0.f;
    float hp = (t0 == 0) ? h_init : __ldg(hin + (size_t)min(t0 - 1, a.T - 1) * a.d);
    float pp = 1.f, dd = 0.f;
#pragma unroll
    for (int i = 0; i < L; ++i) {
        const int t = min(t0 + i, a.T - 1);
        float g[G];
#pragma unroll
        for (int q = 0; q < G; ++q) g[q] = ld_f(wx + ((size_t)t * G + q) * a.d);
        const float cur = __ldg(hin + (size_t)t * a.d);
        float f, j;
        typename C::Acts acts;
        C::eval(hp, g, par, f, j, acts);
        float F = f - cur;
        if (t0 + i >= a.T) {
            j = 1.f;
            F = 0.f;
        }
        dd = fmaf(j, dd, F);
        pp = j * pp;
        hp = cur;
    }
    float my_map[2] = {pp, dd};
    float boundary[2] = {1.f, 0.f};
    float carry[2], tile_end[2];
    tile_exchange<MC, W>(a.chain, chain, tt, my_map, boundary, carry, smem, tile_end);
    if (ch_ok && warp == 0 && tt == a.chain.n_tt - 1) {
        a.agg_out[((size_t)b * 2 + 0) * a.d + ch] = tile_end[0];
        a.agg_out[((size_t)b * 2 + 1) * a.d + ch] = tile_end[1];
    }
}

// Initial guess H^0_t = f(0, x_t), h0 only at t = 0 (fp32 work trajectory).
template <int CELL, typename TIO, typename TOUT>
__global__ void diag_guess_kernel(const TIO* wx, const float* par, const float* h0, TOUT* out, int B,
                                  int T, int d) {
    using C = DiagCell<CELL>;
    constexpr int G = C::G;
    const size_t n = (size_t)B * T * d;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n;
         idx += (size_t)gridDim.x * blockDim.x) {
        const int ch = idx % d;
        const size_t bt = idx / d;
        const int t = bt % T;
        const int b = bt / T;
        float g[G], p[C::NP];
#pragma unroll
        for (int q = 0; q < G; ++q) g[q] = ld_f(wx + (bt * G + q) * d + ch);
#pragma unroll
        for (int q = 0; q < C::NP; ++q) p[q] = __ldg(par + (size_t)q * d + ch);
        const float hp = (t == 0 && h0) ? __ldg(h0 + (size_t)b * d + ch) : 0.f;
        st_f(out + idx, C::step(hp, g, p));
    }
}

// Residual gate: max |f(H_{t-1}, x_t) - H_t| over the whole trajectory.
template <int CELL, typename TIO, typename TST, int L>
__global__ void __launch_bounds__(256) diag_residual_kernel(const TIO* wx, const float* par,
                                                             const float* halo, const TST* st, int B,
                                                             int T, int d, unsigned* dst) {
    using C = DiagCell<CELL>;
    constexpr int G = C::G;
    __shared__ unsigned s_red[8];
    const int ncb = (d + kLanes - 1) / kLanes;
    const int ntt = (T + 8 * L - 1) / (8 * L);
    const int tt = blockIdx.x % ntt;
    const int chain = blockIdx.x / ntt;
    const int b = chain / ncb, cb = chain % ncb;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ch = cb * kLanes + lane;
    unsigned rmax = 0u;
    if (ch < d) {
        float p[C::NP];
#pragma unroll
        for (int q = 0; q < C::NP; ++q) p[q] = __ldg(par + (size_t)q * d + ch);
        const int t0 = tt * 8 * L + warp * L;
        const TST* s = st + (size_t)b * T * d + ch;
        const TIO* w = wx + (size_t)b * T * G * d + ch;
        float hp = 0.f;
        if (t0 < T) hp = (t0 == 0) ? (halo ? __ldg(halo + (size_t)b * d + ch) : 0.f) : ld_f(s + (size_t)(t0 - 1) * d);
        for (int i = 0; i < L && t0 + i < T; ++i) {
            const int t = t0 + i;
            float g[G];
#pragma unroll
            for (int q = 0; q < G; ++q) g[q] = ld_f(w + ((size_t)t * G + q) * d);
            const float cur = ld_f(s + (size_t)t * d);
            rmax = max(rmax, absbits(C::step(hp, g, p) - cur));
            hp = cur;
        }
    }
    block_residual_max(rmax, dst, s_red);
}

// ------------------------------------------------------------------ backward
//
// nu_{t-1} = j_t (nu_t + g_t), nu_{T-1} = 0; mu_t = nu_t + g_t is the adjoint the
// packed VJP consumes; grad_h0 = nu_{-1}.  Tiles are walked from the end of the
// sequence; within a thread steps run from high t to low t.
template <int CELL, typename TIO, int L, int W>
__global__ void __launch_bounds__(W * 32) diag_bwd_kernel(DiagBwdArgs a) {
    using C = DiagCell<CELL>;
    constexpr int G = C::G, NP = C::NP;
    __shared__ float smem[(W * 2 + 2) * kLanes + W * NP * kLanes];
    __shared__ unsigned s_ticket;
    const unsigned ticket = take_ticket(a.chain.ticket, &s_ticket);
    const int tt = ticket / a.chain.n_chains;  // 0 = last time tile
    const int chain = ticket % a.chain.n_chains;
    const int ncb = (a.d + kLanes - 1) / kLanes;
    const int b = chain / ncb, cb = chain % ncb;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ch = cb * kLanes + lane;
    const bool ch_ok = ch < a.d;
    const int chl = ch_ok ? ch : a.d - 1;
    const int tile_t = a.chain.n_tt - 1 - tt;
    // warp 0 owns the highest steps of the tile (scan direction = decreasing t)
    const int t_hi = tile_t * (W * L) + (W - 1 - warp) * L + (L - 1);

    float par[NP];
#pragma unroll
    for (int p = 0; p < NP; ++p) par[p] = __ldg(a.par + (size_t)p * a.d + chl);
    const TIO* wx = reinterpret_cast<const TIO*>(a.wx) + (size_t)b * a.T * G * a.d + chl;
    const TIO* st = reinterpret_cast<const TIO*>(a.states) + (size_t)b * a.T * a.d + chl;
    const TIO* gs = reinterpret_cast<const TIO*>(a.grad_states) + (size_t)b * a.T * a.d + chl;
    const float h_init = a.halo ? __ldg(a.halo + (size_t)b * a.d + chl) : 0.f;

    // i = 0 is the highest step of the sub-tile
    float hp[L], gg[L], P[L], D[L];
    typename C::Acts acts[L];
    {
        float pp = 1.f, dd = 0.f;
#pragma unroll
        for (int i = 0; i < L; ++i) {
            const int t = t_hi - i;
            const bool ok = t < a.T;
            const int tc = min(t, a.T - 1);
            float g[G];
#pragma unroll
            for (int q = 0; q < G; ++q) g[q] = ld_f(wx + ((size_t)tc * G + q) * a.d);
            hp[i] = (tc == 0) ? h_init : ld_f(st + (size_t)(tc - 1) * a.d);
            gg[i] = ok ? ld_f(gs + (size_t)tc * a.d) : 0.f;
            float f, j;
            C::eval(hp[i], g, par, f, j, acts[i]);
            if (!ok) j = 1.f;
            // before consuming step t: nu_t = P*nu_top + D
            P[i] = pp;
            D[i] = dd + gg[i];  // mu_t = P*nu_top + D[i]
            dd = j * (dd + gg[i]);
            pp = j * pp;
        }
        float my_map[2] = {pp, dd};
        float boundary[1] = {a.carry_in ? __ldg(a.carry_in + (size_t)b * a.d + chl) : 0.f};
        float carry[1], tile_end[1];
        tile_exchange<Affine1, W>(a.chain, chain, tt, my_map, boundary, carry, smem, tile_end);
        float gp_acc[NP], gb_acc[G];
#pragma unroll
        for (int p = 0; p < NP; ++p) gp_acc[p] = 0.f;
#pragma unroll
        for (int q = 0; q < G; ++q) gb_acc[q] = 0.f;
        const bool want_bias = a.gb_partial != nullptr;
        TIO* gwx = reinterpret_cast<TIO*>(a.g_wx) + (size_t)b * a.T * G * a.d + ch;
#pragma unroll
        for (int i = 0; i < L; ++i) {
            const int t = t_hi - i;
            if (t < a.T) {
                const float mu = fmaf(P[i], carry[0], D[i]);
                float gw[G], gp[NP];
                C::vjp(hp[i], acts[i], par, mu, gw, gp);
                if (ch_ok) {
#pragma unroll
                    for (int q = 0; q < G; ++q) st_f(gwx + ((size_t)t * G + q) * a.d, gw[q]);
                    if (a.mu_out) a.mu_out[((size_t)b * a.T + t) * a.d + ch] = mu;
                }
#pragma unroll
                for (int p = 0; p < NP; ++p) gp_acc[p] += gp[p];
                if (want_bias) {
#pragma unroll
                    for (int q = 0; q < G; ++q) gb_acc[q] += gw[q];
                }
            }
        }
        if (ch_ok && warp == 0 && tt == a.chain.n_tt - 1 && a.g_h0)
            a.g_h0[(size_t)b * a.d + ch] = tile_end[0];
        // deterministic per-tile parameter partials: fixed-order sum over the W warps
        float* s_gp = smem + (W * 2 + 2) * kLanes;
        __syncthreads();
#pragma unroll
        for (int p = 0; p < NP; ++p) s_gp[(warp * NP + p) * kLanes + lane] = gp_acc[p];
        __syncthreads();
        if (warp == 0 && ch_ok) {
#pragma unroll
            for (int p = 0; p < NP; ++p) {
                float s = 0.f;
#pragma unroll
                for (int w = 0; w < W; ++w) s += s_gp[(w * NP + p) * kLanes + lane];
                a.gp_partial[(((size_t)b * a.chain.n_tt + tile_t) * NP + p) * a.d + ch] = s;
            }
        }
        if (want_bias) {  // the same fixed-order reduction for the bias terms, one gate at a time
#pragma unroll
            for (int q = 0; q < G; ++q) {
                __syncthreads();
                s_gp[warp * kLanes + lane] = gb_acc[q];
                __syncthreads();
                if (warp == 0 && ch_ok) {
                    float s = 0.f;
#pragma unroll
                    for (int w = 0; w < W; ++w) s += s_gp[w * kLanes + lane];
                    a.gb_partial[(((size_t)b * a.chain.n_tt + tile_t) * G + q) * a.d + ch] = s;
                }
            }
        }
    }
}

// Aggregate-only reverse sweep over a time shard (carry = map).
template <int CELL, typename TIO, int L, int W>
__global__ void __launch_bounds__(W * 32) diag_bwd_agg_kernel(DiagBwdArgs a) {
    using C = DiagCell<CELL>;
    constexpr int G = C::G;
    using MC = MapCarry<Affine1>;
    __shared__ float smem[(W * 2 + 2) * kLanes];
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
    const int tile_t = a.chain.n_tt - 1 - tt;
    const int t_hi = tile_t * (W * L) + (W - 1 - warp) * L + (L - 1);
    float par[C::NP];
#pragma unroll
    for (int p = 0; p < C::NP; ++p) par[p] = __ldg(a.par + (size_t)p * a.d + chl);
    const TIO* wx = reinterpret_cast<const TIO*>(a.wx) + (size_t)b * a.T * G * a.d + chl;
    const TIO* st = reinterpret_cast<const TIO*>(a.states) + (size_t)b * a.T * a.d + chl;
    const TIO* gs = reinterpret_cast<const TIO*>(a.grad_states) + (size_t)b * a.T * a.d + chl;
    const float h_init = a.halo ? __ldg(a.halo + (size_t)b * a.d + chl) : 0.f;
    float pp = 1.f, dd = 0.f;
#pragma unroll
    for (int i = 0; i < L; ++i) {
        const int t = t_hi - i;
        const bool ok = t < a.T;
        const int tc = min(t, a.T - 1);
        float g[G];
#pragma unroll
        for (int q = 0; q < G; ++q) g[q] = ld_f(wx + ((size_t)tc * G + q) * a.d);
        const float hp = (tc == 0) ? h_init : ld_f(st + (size_t)(tc - 1) * a.d);
        const float gg = ok ? ld_f(gs + (size_t)tc * a.d) : 0.f;
        float f, j;
        typename C::Acts acts;
        C::eval(hp, g, par, f, j, acts);
        if (!ok) j = 1.f;
        dd = j * (dd + gg);
        pp = j * pp;
    }
    float my_map[2] = {pp, dd};
    float boundary[2] = {1.f, 0.f};
    float carry[2], tile_end[2];
    tile_exchange<MC, W>(a.chain, chain, tt, my_map, boundary, carry, smem, tile_end);
    if (ch_ok && warp == 0 && tt == a.chain.n_tt - 1) {
        a.agg_out[((size_t)b * 2 + 0) * a.d + ch] = tile_end[0];
        a.agg_out[((size_t)b * 2 + 1) * a.d + ch] = tile_end[1];
    }
}

// Fixed-order sum of per-tile parameter partials: out[p][ch] = sum_{rows} part[row][p][ch].
__global__ void reduce_partials_kernel(const float* part, int rows, int np_d, float* out) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= np_d) return;
    float s = 0.f;
    for (int r = 0; r < rows; ++r) s += __ldg(part + (size_t)r * np_d + i);
    out[i] = s;
}

// ------------------------------------------------------------------ launchers

constexpr int kDiagL = 8, kDiagW = 8;
int diag_tile_steps() { return kDiagL * kDiagW; }

template <int CELL, typename TIO>
static cudaError_t launch_fwd(const DiagFwdArgs& a, bool first, bool last, cudaStream_t s) {
    const unsigned grid = (unsigned)(a.chain.n_chains * a.chain.n_tt);
    const dim3 blk(kDiagW * 32);
    if (first && last)
        diag_newton_kernel<CELL, TIO, kDiagL, kDiagW, true, true><<<grid, blk, 0, s>>>(a);
    else if (first)
        diag_newton_kernel<CELL, TIO, kDiagL, kDiagW, true, false><<<grid, blk, 0, s>>>(a);
    else if (last)
        diag_newton_kernel<CELL, TIO, kDiagL, kDiagW, false, true><<<grid, blk, 0, s>>>(a);
    else
        diag_newton_kernel<CELL, TIO, kDiagL, kDiagW, false, false><<<grid, blk, 0, s>>>(a);
    return cudaGetLastError();
}

cudaError_t launch_diag_newton(int cell, int dtype, const DiagFwdArgs& a, bool first, bool last,
                               cudaStream_t s) {
    if (cell == kCellGruDiag) {
        return dtype == kF32 ? launch_fwd<kCellGruDiag, float>(a, first, last, s)
                             : launch_fwd<kCellGruDiag, __nv_bfloat16>(a, first, last, s);
    }
    if (cell == kCellTitans) {
        return dtype == kF32 ? launch_fwd<kCellTitans, float>(a, first, last, s)
                             : launch_fwd<kCellTitans, __nv_bfloat16>(a, first, last, s);
    }
    if (cell == kCellCfc) {
        return dtype == kF32 ? launch_fwd<kCellCfc, float>(a, first, last, s)
                             : launch_fwd<kCellCfc, __nv_bfloat16>(a, first, last, s);
    }
    return dtype == kF32 ? launch_fwd<kCellNlru, float>(a, first, last, s)
                         : launch_fwd<kCellNlru, __nv_bfloat16>(a, first, last, s);
}

cudaError_t launch_diag_newton_agg(int cell, int dtype, const DiagFwdArgs& a, cudaStream_t s) {
    const unsigned grid = (unsigned)(a.chain.n_chains * a.chain.n_tt);
    const dim3 blk(kDiagW * 32);
    if (cell == kCellGruDiag) {
        if (dtype == kF32)
            diag_newton_agg_kernel<kCellGruDiag, float, kDiagL, kDiagW><<<grid, blk, 0, s>>>(a);
        else
            diag_newton_agg_kernel<kCellGruDiag, __nv_bfloat16, kDiagL, kDiagW><<<grid, blk, 0, s>>>(a);
    } else if (cell == kCellTitans) {
        if (dtype == kF32)
            diag_newton_agg_kernel<kCellTitans, float, kDiagL, kDiagW><<<grid, blk, 0, s>>>(a);
        else
            diag_newton_agg_kernel<kCellTitans, __nv_bfloat16, kDiagL, kDiagW><<<grid, blk, 0, s>>>(a);
    } else if (cell == kCellCfc) {
        if (dtype == kF32)
            diag_newton_agg_kernel<kCellCfc, float, kDiagL, kDiagW><<<grid, blk, 0, s>>>(a);
        else
            diag_newton_agg_kernel<kCellCfc, __nv_bfloat16, kDiagL, kDiagW><<<grid, blk, 0, s>>>(a);
    } else {
        if (dtype == kF32)
            diag_newton_agg_kernel<kCellNlru, float, kDiagL, kDiagW><<<grid, blk, 0, s>>>(a);
        else
            diag_newton_agg_kernel<kCellNlru, __nv_bfloat16, kDiagL, kDiagW><<<grid, blk, 0, s>>>(a);
    }
    return cudaGetLastError();
}

template <int CELL, typename TIO, typename TOUT>
static void launch_guess_t(const void* wx, const float* par, const float* h0, void* out, int B, int T,
                           int d, cudaStream_t s) {
    const size_t n = (size_t)B * T * d;
    const int blocks = (int)min((size_t)sm_count() * 16, (n + 255) / 256);
    diag_guess_kernel<CELL, TIO, TOUT><<<blocks, 256, 0, s>>>(
        reinterpret_cast<const TIO*>(wx), par, h0, reinterpret_cast<TOUT*>(out), B, T, d);
}

cudaError_t launch_diag_guess(int cell, int dtype, bool out_f32, const void* wx, const float* par,
                              const float* h0, void* out, int B, int T, int d, cudaStream_t s) {
#define PRB_GUESS(CELL)                                                                       \
    if (dtype == kF32)                                                                        \
        launch_guess_t<CELL, float, float>(wx, par, h0, out, B, T, d, s);                      \
    else if (out_f32)                                                                         \
        launch_guess_t<CELL, __nv_bfloat16, float>(wx, par, h0, out, B, T, d, s);              \
    else                                                                                      \
        launch_guess_t<CELL, __nv_bfloat16, __nv_bfloat16>(wx, par, h0, out, B, T, d, s);
    if (cell == kCellGruDiag) {
        PRB_GUESS(kCellGruDiag)
    } else if (cell == kCellTitans) {
        PRB_GUESS(kCellTitans)
    } else if (cell == kCellCfc) {
        PRB_GUESS(kCellCfc)
    } else {
        PRB_GUESS(kCellNlru)
    }
#undef PRB_GUESS
    return cudaGetLastError();
}

cudaError_t launch_diag_residual(int cell, int dtype, bool st_f32, const void* wx, const float* par,
                                 const float* halo, const void* st, int B, int T, int d,
                                 unsigned* dst, cudaStream_t s) {
    constexpr int L = 8;
    const int ncb = (d + kLanes - 1) / kLanes;
    const int ntt = (T + 8 * L - 1) / (8 * L);
    const unsigned grid = (unsigned)(B * ncb * ntt);
#define PRB_RES(CELL)                                                                            \
    if (dtype == kF32)                                                                           \
        diag_residual_kernel<CELL, float, float, L><<<grid, 256, 0, s>>>(                         \
            (const float*)wx, par, halo, (const float*)st, B, T, d, dst);                        \
    else if (st_f32)                                                                             \
        diag_residual_kernel<CELL, __nv_bfloat16, float, L><<<grid, 256, 0, s>>>(                 \
            (const __nv_bfloat16*)wx, par, halo, (const float*)st, B, T, d, dst);                \
    else                                                                                         \
        diag_residual_kernel<CELL, __nv_bfloat16, __nv_bfloat16, L><<<grid, 256, 0, s>>>(         \
            (const __nv_bfloat16*)wx, par, halo, (const __nv_bfloat16*)st, B, T, d, dst);
    if (cell == kCellGruDiag) {
        PRB_RES(kCellGruDiag)
    } else if (cell == kCellTitans) {
        PRB_RES(kCellTitans)
    } else if (cell == kCellCfc) {
        PRB_RES(kCellCfc)
    } else {
        PRB_RES(kCellNlru)
    }
#undef PRB_RES
    return cudaGetLastError();
}

cudaError_t launch_diag_bwd(int cell, int dtype, const DiagBwdArgs& a, bool agg_only, cudaStream_t s) {
    const unsigned grid = (unsigned)(a.chain.n_chains * a.chain.n_tt);
    const dim3 blk(kDiagW * 32);
#define PRB_BWD(CELL, TIO)                                                       \
    if (agg_only)                                                                \
        diag_bwd_agg_kernel<CELL, TIO, kDiagL, kDiagW><<<grid, blk, 0, s>>>(a);   \
    else                                                                         \
        diag_bwd_kernel<CELL, TIO, kDiagL, kDiagW><<<grid, blk, 0, s>>>(a);
    if (cell == kCellGruDiag) {
        if (dtype == kF32) {
            PRB_BWD(kCellGruDiag, float)
        } else {
            PRB_BWD(kCellGruDiag, __nv_bfloat16)
        }
    } else if (cell == kCellTitans) {
        if (dtype == kF32) {
            PRB_BWD(kCellTitans, float)
        } else {
            PRB_BWD(kCellTitans, __nv_bfloat16)
        }
    } else if (cell == kCellCfc) {
        if (dtype == kF32) {
            PRB_BWD(kCellCfc, float)
        } else {
            PRB_BWD(kCellCfc, __nv_bfloat16)
        }
    } else {
        if (dtype == kF32) {
            PRB_BWD(kCellNlru, float)
        } else {
            PRB_BWD(kCellNlru, __nv_bfloat16)
        }
    }
#undef PRB_BWD
    return cudaGetLastError();
}

cudaError_t launch_reduce_partials(const float* part, int rows, int np_d, float* out, cudaStream_t s) {
    reduce_partials_kernel<<<(np_d + 127) / 128, 128, 0, s>>>(part, rows, np_d, out);
    return cudaGetLastError();
}

}  // namespace prb
