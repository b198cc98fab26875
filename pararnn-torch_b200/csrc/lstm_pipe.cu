// ParaLSTM (state slots (c, h), 2x2 block Jacobian per channel): pipelined persistent kernels.
//
// Same ownership and input ring as the scalar-diagonal family (diag_pipe.cu): one CTA owns one
// chain (batch row x 32 channels, lane = channel) for the whole time axis and walks it in rounds
// of W*L steps; a producer warp streams the rounds into a shared-memory ring with TMA tile loads
// (full / empty mbarriers).  Each compute warp owns L consecutive steps of a round, linearises them
// and composes their 2x2 affine map (6 floats), which does not depend on the scan carry.  The W
// maps of a round meet in double-buffered shared memory behind ONE named barrier; every warp folds
// all of them itself (W dependent 2x2 applications on a 2-vector), which gives it the carry entering
// its own sub-tile and the one entering the next round, bit-identical in every warp.
//
// Forward: all K <= 4 Newton iterations from the App. A guess, and the residual of the result, in
// ONE sweep: the iterates of a warp's steps stay in registers, the state before the sub-tile moves
// with the delta carry the fold delivers.  wx is read once and H written once.
// Backward: eq. 2.6 reverse scan with J^T fused with the packed VJP; per-CTA parameter partials.
//
// Per-step math: lstm_cell.cuh.  Reference behaviour restated: kernels/newton_lstm.py,
// kernels/scan_lstm_block.py (the fused op), solvers/scan.py:150-164 (reverse 2x2 scan),
// kernels/vjp_lstm.py (packed VJP).
#include "common.cuh"
#include "kernels.h"
#include "lstm_cell.cuh"
#include "tma.cuh"

#include <type_traits>

namespace prb {

namespace {

constexpr uint32_t kLstmPipeWaitLimit = 1u << 24;
constexpr int kLstmFusedMaxK = 4;

__device__ __forceinline__ void lp_mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void lp_named_sync(int id, int count) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}
constexpr int lp_round128(int x) { return (x + 127) / 128 * 128; }

// Fold the W sub-tile maps of a round (scan order = warp order) into the running carry; returns in
// `mine` the carry entering sub-tile `warp`.  Every warp runs the same FMAs in the same order.
template <int W>
__device__ __forceinline__ void fold_round2(const float* maps, int warp, int lane, float (&carry)[2],
                                            float (&mine)[2]) {
    mine[0] = carry[0];
    mine[1] = carry[1];
#pragma unroll
    for (int v = 0; v < W; ++v) {
        if (v == warp) {
            mine[0] = carry[0];
            mine[1] = carry[1];
        }
        float m[6];
#pragma unroll
        for (int q = 0; q < 6; ++q) m[q] = maps[(v * 6 + q) * kLanes + lane];
        Affine2::apply(m, carry);
    }
}

// ------------------------------------------------------------------ forward
template <typename TIO, int L, int W, int NSTAGE>
struct LstmPipeFwdSmem {
    static constexpr int LT = W * L;
    static constexpr int WX_TX = (LT + 1) * 3 * kLanes * (int)sizeof(TIO);  // box starts one step early
    static constexpr int STAGE = lp_round128(WX_TX);
    static constexpr int MAP_OFF = NSTAGE * STAGE;
    static constexpr int MAP_BYTES = 2 * W * 6 * kLanes * 4;  // [parity][W][6][32]
    static constexpr int BAR_OFF = MAP_OFF + MAP_BYTES;
    static constexpr int RED_OFF = BAR_OFF + 2 * NSTAGE * 8;
    static constexpr int TOTAL = RED_OFF + (W + 1) * 4 + 64;
};

template <typename TIO, int L, int W, int NSTAGE>
__global__ void __launch_bounds__((W + 1) * 32, W > 8 ? 1 : 2)
lstm_newton_fused_kernel(const __grid_constant__ CUtensorMap tm_wx, LstmFwdArgs a, int K) {
    using S = LstmPipeFwdSmem<TIO, L, W, NSTAGE>;
    constexpr int LT = S::LT;
    extern __shared__ __align__(128) unsigned char smem[];
    float* s_map = reinterpret_cast<float*>(smem + S::MAP_OFF);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + S::BAR_OFF);
    uint64_t* empty = full + NSTAGE;
    unsigned* s_red = reinterpret_cast<unsigned*>(smem + S::RED_OFF);

    const int d = a.d;
    const int ncb = (d + kLanes - 1) / kLanes;
    const int chain = blockIdx.x;
    const int b = chain / ncb, cb = chain % ncb;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ch = cb * kLanes + lane;
    const bool ch_ok = ch < d;
    const int chl = ch_ok ? ch : d - 1;
    const int n_rounds = (a.T + LT - 1) / LT;
    const int row0 = b * a.T;

    if (threadIdx.x == 0) {
        tma_prefetch_desc(&tm_wx);
        for (int s = 0; s < NSTAGE; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], W);
        }
        mbar_fence_init();
    }
    __syncthreads();

    unsigned rmax[kLstmFusedMaxK] = {0u, 0u, 0u, 0u};
    unsigned fmax = 0u;
    bool timed_out = false;

    if (warp == W) {
        if (lane == 0) {
            for (int r = 0; r < n_rounds; ++r) {
                const int s = r % NSTAGE;
                if (r >= NSTAGE && !mbar_wait_bounded(&empty[s], ((r / NSTAGE) - 1) & 1,
                                                      timed_out ? kWaitLimitAfterTimeout : kLstmPipeWaitLimit))
                    timed_out = true;
                mbar_expect_tx(&full[s], S::WX_TX);
                tma_load_3d(smem + s * S::STAGE, &tm_wx, &full[s], cb * kLanes, 0, row0 + r * LT - 1);
            }
            if (timed_out) drain_ring(full, NSTAGE, n_rounds, kDrainLimit);
        }
    } else {
        float p[5];
#pragma unroll
        for (int q = 0; q < 5; ++q) p[q] = __ldg(a.par + (size_t)q * d + chl);
        const float h0c = a.halo ? __ldg(a.halo + ((size_t)b * 2 + 0) * d + chl) : 0.f;
        const float h0h = a.halo ? __ldg(a.halo + ((size_t)b * 2 + 1) * d + chl) : 0.f;
        const bool want_final = a.final_bits != nullptr;
        float carry[kLstmFusedMaxK][2] = {{0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}};
        int parity = 0;  // the two map buffers alternate from barrier to barrier

        for (int r = 0; r < n_rounds; ++r) {
            const int s = r % NSTAGE;
            if (!mbar_wait_bounded(&full[s], (r / NSTAGE) & 1, timed_out ? kWaitLimitAfterTimeout : kLstmPipeWaitLimit))
                timed_out = true;
            const TIO* t_wx = reinterpret_cast<const TIO*>(smem + s * S::STAGE);
            const int t0 = r * LT + warp * L;

            // Rounds that lie fully inside the sequence take a variant without range checks.
            auto round_body = [&](auto full_c) {
                constexpr bool FULL = decltype(full_c)::value;
                // row k of the box is time step r*LT - 1 + k
                float w[L][3], st[L + 1][2];
    #pragma unroll
                for (int i = 0; i < L; ++i)
    #pragma unroll
                    for (int q = 0; q < 3; ++q) w[i][q] = (float)t_wx[((warp * L + i + 1) * 3 + q) * kLanes + lane];
                // App. A guess: H^0_t = f(0, x_t), the initial state only at t = 0
                if (t0 == 0) {
                    st[0][0] = h0c;
                    st[0][1] = h0h;
                } else {
                    float g[3];
    #pragma unroll
                    for (int q = 0; q < 3; ++q) g[q] = (float)t_wx[((warp * L) * 3 + q) * kLanes + lane];
                    LstmActs ac;
                    lstm_step(t0 - 1 == 0 ? h0c : 0.f, t0 - 1 == 0 ? h0h : 0.f, g, p, ac);
                    st[0][0] = ac.cn;
                    st[0][1] = ac.hn;
                }
                __syncwarp();
                if (lane == 0) lp_mbar_arrive(&empty[s]);
    #pragma unroll
                for (int i = 0; i < L; ++i) {
                    LstmActs ac;
                    lstm_step(t0 + i == 0 ? h0c : 0.f, t0 + i == 0 ? h0h : 0.f, w[i], p, ac);
                    st[i + 1][0] = ac.cn;
                    st[i + 1][1] = ac.hn;
                }

    #pragma unroll
                for (int k = 0; k < kLstmFusedMaxK; ++k) {
                    if (k < K) {
                        // st[0..L] is iterate k of steps t0-1 .. t0+L-1 (the guess for k = 0)
                        float J[L][4], F[L][2];
                        float mp[6] = {1.f, 0.f, 0.f, 1.f, 0.f, 0.f};
    #pragma unroll
                        for (int i = 0; i < L; ++i) {
                            LstmActs ac;
                            lstm_step(st[i][0], st[i][1], w[i], p, ac);
                            lstm_jac(ac, st[i][0], p, J[i]);
                            F[i][0] = ac.cn - st[i + 1][0];
                            F[i][1] = ac.hn - st[i + 1][1];
                            if (!FULL && t0 + i >= a.T) {  // identity step beyond the end of the sequence
                                J[i][0] = 1.f; J[i][1] = 0.f; J[i][2] = 0.f; J[i][3] = 1.f;
                                F[i][0] = F[i][1] = 0.f;
                            } else if (ch_ok) {
                                rmax[k] = max(rmax[k], max(absbits(F[i][0]), absbits(F[i][1])));
                            }
                            const float step_map[6] = {J[i][0], J[i][1], J[i][2], J[i][3], F[i][0], F[i][1]};
                            Affine2::compose(mp, step_map);
                        }
                        float* maps = s_map + parity * (W * 6 * kLanes);
                        parity ^= 1;
    #pragma unroll
                        for (int q = 0; q < 6; ++q) maps[(warp * 6 + q) * kLanes + lane] = mp[q];
                        lp_named_sync(1, W * 32);
                        float dl[2];
                        fold_round2<W>(maps, warp, lane, carry[k], dl);
                        st[0][0] = fmaf(a.omega, dl[0], st[0][0]);
                        st[0][1] = fmaf(a.omega, dl[1], st[0][1]);
    #pragma unroll
                        for (int i = 0; i < L; ++i) {
                            const float nc = fmaf(J[i][0], dl[0], fmaf(J[i][1], dl[1], F[i][0]));
                            const float nh = fmaf(J[i][2], dl[0], fmaf(J[i][3], dl[1], F[i][1]));
                            dl[0] = nc;
                            dl[1] = nh;
                            st[i + 1][0] = fmaf(a.omega, nc, st[i + 1][0]);
                            st[i + 1][1] = fmaf(a.omega, nh, st[i + 1][1]);
                        }
                    }
                }

                if (ch_ok) {
                    TIO* o = reinterpret_cast<TIO*>(a.sout) + ((size_t)b * a.T + t0) * 2 * d + ch;
    #pragma unroll
                    for (int i = 0; i < L; ++i) {
                        if (FULL || t0 + i < a.T) {
                            if (want_final) {
                                LstmActs ac;
                                lstm_step(st[i][0], st[i][1], w[i], p, ac);
                                fmax = max(fmax, max(absbits(ac.cn - st[i + 1][0]), absbits(ac.hn - st[i + 1][1])));
                            }
                            st_f(o + (size_t)i * 2 * d, st[i + 1][0]);
                            st_f(o + (size_t)i * 2 * d + d, st[i + 1][1]);
                        }
                    }
                }
            };
            if (t0 + L <= a.T)
                round_body(std::true_type{});
            else
                round_body(std::false_type{});
        }
    }
    if (timed_out) atomicExch(a.chain.status, (int)kErrChainTimeout);
#pragma unroll
    for (int k = 0; k < kLstmFusedMaxK; ++k) {
        if (k < K) {
            __syncthreads();
            block_residual_max(rmax[k], a.resid_bits + k, s_red);
        }
    }
    if (a.final_bits != nullptr) {
        __syncthreads();
        block_residual_max(fmax, a.final_bits, s_red);
    }
}

// ------------------------------------------------------------------ backward
template <typename TIO, int L, int W, int NSTAGE>
struct LstmPipeBwdSmem {
    static constexpr int LT = W * L;
    static constexpr int WX_TX = LT * 3 * kLanes * (int)sizeof(TIO);
    static constexpr int ST_TX = (LT + 1) * 2 * kLanes * (int)sizeof(TIO);  // starts one step early
    static constexpr int G_TX = LT * 2 * kLanes * (int)sizeof(TIO);
    static constexpr int WX_BYTES = lp_round128(WX_TX);
    static constexpr int ST_BYTES = lp_round128(ST_TX);
    static constexpr int G_BYTES = lp_round128(G_TX);
    static constexpr int STAGE = WX_BYTES + ST_BYTES + G_BYTES;
    static constexpr int MAP_OFF = NSTAGE * STAGE;
    static constexpr int MAP_BYTES = 2 * W * 6 * kLanes * 4;
    static constexpr int GP_OFF = MAP_OFF + MAP_BYTES;
    static constexpr int GP_BYTES = W * 5 * kLanes * 4;
    static constexpr int BAR_OFF = GP_OFF + GP_BYTES;
    static constexpr int TOTAL = BAR_OFF + 2 * NSTAGE * 8 + 64;
};

// Rounds run from the end of the sequence; warp 0 owns the highest steps of a round.  The map of a
// reverse step is nu -> J^T (nu + g); nu_{T-1} = 0, grad_h0 = nu_{-1}.
template <typename TIO, int L, int W, int NSTAGE>
__global__ void __launch_bounds__((W + 1) * 32, W > 8 ? 1 : 2)
lstm_bwd_pipe_kernel(const __grid_constant__ CUtensorMap tm_wx, const __grid_constant__ CUtensorMap tm_st,
                     const __grid_constant__ CUtensorMap tm_g, LstmBwdArgs a) {
    using S = LstmPipeBwdSmem<TIO, L, W, NSTAGE>;
    constexpr int LT = S::LT;
    extern __shared__ __align__(128) unsigned char smem[];
    float* s_map = reinterpret_cast<float*>(smem + S::MAP_OFF);
    float* s_gp = reinterpret_cast<float*>(smem + S::GP_OFF);  // [W][5][32]
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + S::BAR_OFF);
    uint64_t* empty = full + NSTAGE;

    const int d = a.d;
    const int ncb = (d + kLanes - 1) / kLanes;
    const int chain = blockIdx.x;
    const int b = chain / ncb, cb = chain % ncb;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ch = cb * kLanes + lane;
    const bool ch_ok = ch < d;
    const int chl = ch_ok ? ch : d - 1;
    const int n_rounds = (a.T + LT - 1) / LT;
    const int row0 = b * a.T;

    if (threadIdx.x == 0) {
        tma_prefetch_desc(&tm_wx);
        tma_prefetch_desc(&tm_st);
        tma_prefetch_desc(&tm_g);
        for (int s = 0; s < NSTAGE; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], W);
        }
        mbar_fence_init();
    }
    __syncthreads();
    bool timed_out = false;
    float gp[5] = {0.f, 0.f, 0.f, 0.f, 0.f};

    if (warp == W) {
        if (lane == 0) {
            for (int r = 0; r < n_rounds; ++r) {
                const int s = r % NSTAGE;
                const int tile_t = n_rounds - 1 - r;
                if (r >= NSTAGE && !mbar_wait_bounded(&empty[s], ((r / NSTAGE) - 1) & 1,
                                                      timed_out ? kWaitLimitAfterTimeout : kLstmPipeWaitLimit))
                    timed_out = true;
                unsigned char* base = smem + s * S::STAGE;
                mbar_expect_tx(&full[s], S::WX_TX + S::ST_TX + S::G_TX);
                tma_load_3d(base, &tm_wx, &full[s], cb * kLanes, 0, row0 + tile_t * LT);
                tma_load_3d(base + S::WX_BYTES, &tm_st, &full[s], cb * kLanes, 0, row0 + tile_t * LT - 1);
                tma_load_3d(base + S::WX_BYTES + S::ST_BYTES, &tm_g, &full[s], cb * kLanes, 0, row0 + tile_t * LT);
            }
            if (timed_out) drain_ring(full, NSTAGE, n_rounds, kDrainLimit);
        }
    } else {
        float p[5];
#pragma unroll
        for (int q = 0; q < 5; ++q) p[q] = __ldg(a.par + (size_t)q * d + chl);
        const float h0c = a.halo ? __ldg(a.halo + ((size_t)b * 2 + 0) * d + chl) : 0.f;
        const float h0h = a.halo ? __ldg(a.halo + ((size_t)b * 2 + 1) * d + chl) : 0.f;
        float carry[2] = {0.f, 0.f};
        TIO* gwx = reinterpret_cast<TIO*>(a.g_wx) + (size_t)b * a.T * 3 * d + ch;

        for (int r = 0; r < n_rounds; ++r) {
            const int s = r % NSTAGE;
            const int tile_t = n_rounds - 1 - r;
            if (!mbar_wait_bounded(&full[s], (r / NSTAGE) & 1, timed_out ? kWaitLimitAfterTimeout : kLstmPipeWaitLimit))
                timed_out = true;
            const TIO* t_wx = reinterpret_cast<const TIO*>(smem + s * S::STAGE);
            const TIO* t_st = reinterpret_cast<const TIO*>(smem + s * S::STAGE + S::WX_BYTES);
            const TIO* t_g = reinterpret_cast<const TIO*>(smem + s * S::STAGE + S::WX_BYTES + S::ST_BYTES);
            // i = 0 is the highest step of the sub-tile
            const int k_hi = (W - 1 - warp) * L + (L - 1);  // position inside the round
            const int t_hi = tile_t * LT + k_hi;

            auto round_body = [&](auto full_c) {
                constexpr bool FULL = decltype(full_c)::value;
                LstmActs act[L];
                float J[L][4], g[L][2], prev[L][2];
                float mp[6] = {1.f, 0.f, 0.f, 1.f, 0.f, 0.f};
    #pragma unroll
                for (int i = 0; i < L; ++i) {
                    const int k = k_hi - i;
                    const int t = t_hi - i;
                    float w[3];
    #pragma unroll
                    for (int q = 0; q < 3; ++q) w[q] = (float)t_wx[(k * 3 + q) * kLanes + lane];
                    // row k of the state box is step t - 1
                    prev[i][0] = (t == 0) ? h0c : (float)t_st[(k * 2 + 0) * kLanes + lane];
                    prev[i][1] = (t == 0) ? h0h : (float)t_st[(k * 2 + 1) * kLanes + lane];
                    const bool ok = FULL || t < a.T;
                    g[i][0] = ok ? (float)t_g[(k * 2 + 0) * kLanes + lane] : 0.f;
                    g[i][1] = ok ? (float)t_g[(k * 2 + 1) * kLanes + lane] : 0.f;
                    lstm_step(prev[i][0], prev[i][1], w, p, act[i]);
                    lstm_jac(act[i], prev[i][0], p, J[i]);
                    if (!ok) {
                        J[i][0] = 1.f; J[i][1] = 0.f; J[i][2] = 0.f; J[i][3] = 1.f;
                    }
                    const float step_map[6] = {J[i][0], J[i][2], J[i][1], J[i][3],
                                               fmaf(J[i][0], g[i][0], J[i][2] * g[i][1]),
                                               fmaf(J[i][1], g[i][0], J[i][3] * g[i][1])};
                    Affine2::compose(mp, step_map);
                }
                __syncwarp();
                if (lane == 0) lp_mbar_arrive(&empty[s]);

                float* maps = s_map + (r & 1) * (W * 6 * kLanes);
    #pragma unroll
                for (int q = 0; q < 6; ++q) maps[(warp * 6 + q) * kLanes + lane] = mp[q];
                lp_named_sync(1, W * 32);
                float nu[2];
                fold_round2<W>(maps, warp, lane, carry, nu);

                float nc = nu[0], nh = nu[1];
    #pragma unroll
                for (int i = 0; i < L; ++i) {
                    const int t = t_hi - i;
                    if (FULL || t < a.T) {
                        const LstmActs& sa = act[i];
                        const float mc = nc + g[i][0], mh = nh + g[i][1];
                        const float d_opre = mh * sa.hact * sa.o * (1.f - sa.o);
                        const float d_cn = fmaf(mh, sa.o * (1.f - sa.hact * sa.hact), fmaf(d_opre, p[4], mc));
                        const float d_fpre = d_cn * (prev[i][0] - sa.z) * sa.f * (1.f - sa.f);
                        const float d_zpre = d_cn * (1.f - sa.f) * (1.f - sa.z * sa.z);
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
                        gp[4] = fmaf(d_opre, sa.cn, gp[4]);
                        nc = fmaf(J[i][0], mc, J[i][2] * mh);
                        nh = fmaf(J[i][1], mc, J[i][3] * mh);
                    }
                }
                if (r == n_rounds - 1 && warp == 0 && ch_ok && a.g_h0) {
                    a.g_h0[((size_t)b * 2 + 0) * d + ch] = carry[0];
                    a.g_h0[((size_t)b * 2 + 1) * d + ch] = carry[1];
                }
            };
            if (t_hi < a.T)
                round_body(std::true_type{});
            else
                round_body(std::false_type{});
        }
#pragma unroll
        for (int q = 0; q < 5; ++q) s_gp[(warp * 5 + q) * kLanes + lane] = gp[q];
    }
    if (timed_out) atomicExch(a.chain.status, (int)kErrChainTimeout);
    __syncthreads();
    if (warp == 0 && ch_ok) {
#pragma unroll
        for (int q = 0; q < 5; ++q) {
            float sum = 0.f;
#pragma unroll
            for (int w2 = 0; w2 < W; ++w2) sum += s_gp[(w2 * 5 + q) * kLanes + lane];
            a.gp_partial[((size_t)b * 5 + q) * d + ch] = sum;
        }
    }
}

// With few chains (up to 1.5 per SM) every chain gets 16 compute warps per CTA; with many chains
// two 8-warp CTAs share an SM.
inline bool lstm_wide_cta(int B, int d) { return 2 * B * ((d + kLanes - 1) / kLanes) <= 3 * sm_count(); }

template <typename TIO, int NSTAGE, int L, int W>
cudaError_t launch_fused_w(const LstmFwdArgs& a, int K, cudaStream_t s) {
    using S = LstmPipeFwdSmem<TIO, L, W, NSTAGE>;
    CUtensorMap tm_wx;
    const uint64_t rows = (uint64_t)a.B * a.T;
    if (!make_tile_map(&tm_wx, a.wx, sizeof(TIO), rows, 3, a.d, S::LT + 1)) return cudaErrorNotSupported;
    const int grid = a.B * ((a.d + kLanes - 1) / kLanes);
    auto k = lstm_newton_fused_kernel<TIO, L, W, NSTAGE>;
    cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
    k<<<grid, (W + 1) * 32, S::TOTAL, s>>>(tm_wx, a, K);
    return cudaGetLastError();
}

template <typename TIO, int NSTAGE, int L, int W>
cudaError_t launch_bwd_w(const LstmBwdArgs& a, cudaStream_t s) {
    using S = LstmPipeBwdSmem<TIO, L, W, NSTAGE>;
    CUtensorMap tm_wx, tm_st, tm_g;
    const uint64_t rows = (uint64_t)a.B * a.T;
    if (!make_tile_map(&tm_wx, a.wx, sizeof(TIO), rows, 3, a.d, S::LT) ||
        !make_tile_map(&tm_st, a.states, sizeof(TIO), rows, 2, a.d, S::LT + 1) ||
        !make_tile_map(&tm_g, a.grad_states, sizeof(TIO), rows, 2, a.d, S::LT))
        return cudaErrorNotSupported;
    const int grid = a.B * ((a.d + kLanes - 1) / kLanes);
    auto k = lstm_bwd_pipe_kernel<TIO, L, W, NSTAGE>;
    cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
    k<<<grid, (W + 1) * 32, S::TOTAL, s>>>(tm_wx, tm_st, tm_g, a);
    return cudaGetLastError();
}

constexpr int kLPL = 4;  // steps per warp and round: J, F and the iterates of L steps live in registers

}  // namespace

// all K Newton iterations (1..4) from the App. A guess, and the residual of the result, in one sweep;
// a.resid_bits points at the first of K history slots, a.sout is the result in the I/O dtype
cudaError_t launch_lstm_newton_fused(int dtype, const LstmFwdArgs& a, int K, cudaStream_t s) {
    if (K < 1 || K > kLstmFusedMaxK) return cudaErrorNotSupported;
    const bool wide = lstm_wide_cta(a.B, a.d);
    if (dtype == kF32)
        return wide ? launch_fused_w<float, 2, kLPL, 16>(a, K, s) : launch_fused_w<float, 2, kLPL, 8>(a, K, s);
    return wide ? launch_fused_w<__nv_bfloat16, 3, kLPL, 16>(a, K, s)
                : launch_fused_w<__nv_bfloat16, 3, kLPL, 8>(a, K, s);
}

// a.gp_partial receives one row per batch row: (B, 5, d)
cudaError_t launch_lstm_bwd_pipe(int dtype, const LstmBwdArgs& a, cudaStream_t s) {
    const bool wide = lstm_wide_cta(a.B, a.d);
    if (dtype == kF32)
        return wide ? launch_bwd_w<float, 2, kLPL, 16>(a, s) : launch_bwd_w<float, 2, kLPL, 8>(a, s);
    return wide ? launch_bwd_w<__nv_bfloat16, 3, kLPL, 16>(a, s) : launch_bwd_w<__nv_bfloat16, 3, kLPL, 8>(a, s);
}

}  // namespace prb
