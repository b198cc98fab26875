// Scalar-diagonal cells (ParaGRU mix='diag', ParaNLRU, ParaTitans, ParaCfC): warp-pipelined persistent kernels.
//
// One CTA owns one chain (batch row x 32 channels, lane = channel) for the whole time axis and
// walks it in rounds of W*L steps.  A producer warp streams the inputs of the coming rounds into
// a shared-memory ring with TMA tile loads (full / empty mbarriers).  Each of the W compute
// warps owns L consecutive steps of a round: it evaluates the gates, the diagonal Jacobian and
// the residual of its steps and composes them into the prefix maps (P_i, D_i) of its sub-tile,
// none of which depends on the scan carry.  The W sub-tile maps (P_L, D_L) of a round meet in
// shared memory (double-buffered, ONE named barrier of the compute warps per round); every warp
// folds all W of them itself (W dependent FMAs on one float per channel), which yields both the
// carry entering its own sub-tile and the carry entering the next round, so no second barrier
// and no warp-to-warp hand-over chain is needed.  It then writes its L results P_i * c + D_i.
//
// Same math as the look-back kernels of diag_kernels.cu (diag_cell.cuh); used when the arrays
// meet TMA's alignment rules and there are enough chains to occupy the GPU.
#include "common.cuh"
#include "diag_cell.cuh"
#include "kernels.h"
#include "tma.cuh"

#include <type_traits>

namespace prb {

namespace {

constexpr uint32_t kDiagPipeWaitLimit = 1u << 24;

__device__ __forceinline__ void dp_mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void dp_named_sync(int id, int count) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}
// Fold the W sub-tile maps of a round (time order = warp order) into the running carry; returns
// the carry entering sub-tile `warp`.  Every compute warp runs the same sequence of FMAs, so all
// of them hold bit-identical carries.
template <int W>
__device__ __forceinline__ float fold_round(const float* maps, int warp, int lane, float& carry) {
    float mine = carry;
#pragma unroll
    for (int v = 0; v < W; ++v) {
        if (v == warp) mine = carry;
        const float2 m = reinterpret_cast<const float2*>(maps)[v * kLanes + lane];  // (P, D) of sub-tile v
        carry = fmaf(m.x, carry, m.y);
    }
    return mine;
}
constexpr int round128(int x) { return (x + 127) / 128 * 128; }

// ------------------------------------------------------------------ forward
template <int G, typename TIO, int L, int W, int NSTAGE>
struct DiagPipeFwdSmem {
    static constexpr int LT = W * L;
    static constexpr int WX_TX = (LT + 1) * G * kLanes * (int)sizeof(TIO);  // box starts one step early
    static constexpr int H_TX = (LT + 1) * kLanes * 4;
    static constexpr int WX_BYTES = round128(WX_TX);
    static constexpr int H_BYTES = round128(H_TX);
    static constexpr int STAGE = WX_BYTES + H_BYTES;
    static constexpr int MAP_OFF = NSTAGE * STAGE;
    static constexpr int MAP_BYTES = 2 * W * 2 * kLanes * 4;  // [parity][W][P, D][32]
    static constexpr int BAR_OFF = MAP_OFF + MAP_BYTES;
    static constexpr int RED_OFF = BAR_OFF + 2 * NSTAGE * 8;
    static constexpr int TOTAL = RED_OFF + (W + 1) * 4 + 64;
};

template <int CELL, typename TIO, int L, int W, int NSTAGE, bool FIRST, bool LAST>
__global__ void __launch_bounds__((W + 1) * 32, W * L > 64 ? 1 : 2)
diag_newton_pipe_kernel(const __grid_constant__ CUtensorMap tm_wx, const __grid_constant__ CUtensorMap tm_h,
                        DiagFwdArgs a) {
    using C = DiagCell<CELL>;
    constexpr int G = C::G;
    using S = DiagPipeFwdSmem<G, TIO, L, W, NSTAGE>;
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
        if (!FIRST) tma_prefetch_desc(&tm_h);
        for (int s = 0; s < NSTAGE; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], W);
        }
        mbar_fence_init();
    }
    __syncthreads();

    unsigned rmax = 0u, fmax = 0u;
    bool timed_out = false;

    if (warp == W) {
        // ---------------- producer warp: one lane streams the rounds into the ring
        if (lane == 0) {
            for (int r = 0; r < n_rounds; ++r) {
                const int s = r % NSTAGE;
                if (r >= NSTAGE && !mbar_wait_bounded(&empty[s], ((r / NSTAGE) - 1) & 1, timed_out ? kWaitLimitAfterTimeout : kDiagPipeWaitLimit))
                    timed_out = true;
                unsigned char* base = smem + s * S::STAGE;
                mbar_expect_tx(&full[s], FIRST ? S::WX_TX : S::WX_TX + S::H_TX);
                tma_load_3d(base, &tm_wx, &full[s], cb * kLanes, 0, row0 + r * LT - 1);
                if (!FIRST) tma_load_3d(base + S::WX_BYTES, &tm_h, &full[s], cb * kLanes, 0, row0 + r * LT - 1);
            }
            if (timed_out) drain_ring(full, NSTAGE, n_rounds, kDrainLimit);
        }
    } else {
        // ---------------- compute warps
        float par[C::NP];
#pragma unroll
        for (int p = 0; p < C::NP; ++p) par[p] = __ldg(a.par + (size_t)p * d + chl);
        const float h_init = a.halo ? __ldg(a.halo + (size_t)b * d + chl) : 0.f;
        const bool want_final = LAST && a.final_bits != nullptr;
        float carry = a.carry_in ? __ldg(a.carry_in + (size_t)b * d + chl) : 0.f;

        for (int r = 0; r < n_rounds; ++r) {
            const int s = r % NSTAGE;
            if (!mbar_wait_bounded(&full[s], (r / NSTAGE) & 1, timed_out ? kWaitLimitAfterTimeout : kDiagPipeWaitLimit)) timed_out = true;
            const TIO* t_wx = reinterpret_cast<const TIO*>(smem + s * S::STAGE);
            const float* t_h = reinterpret_cast<const float*>(smem + s * S::STAGE + S::WX_BYTES);
            const int t0 = r * LT + warp * L;

            // Rounds that lie fully inside the sequence take a variant without range checks.
            auto round_body = [&](auto full_c) {
                constexpr bool FULL = decltype(full_c)::value;
                // row k of the boxes is time step r*LT - 1 + k
                float g[L][G], hold[L + 1];
    #pragma unroll
                for (int i = 0; i < L; ++i)
    #pragma unroll
                    for (int q = 0; q < G; ++q) g[i][q] = (float)t_wx[((warp * L + i + 1) * G + q) * kLanes + lane];
                if (FIRST) {
                    // App. A guess evaluated on the fly: H^0_t = f(0, x_t), h0 only at t = 0
                    if (t0 == 0) {
                        hold[0] = h_init;
                    } else {
                        float gp[G];
    #pragma unroll
                        for (int q = 0; q < G; ++q) gp[q] = (float)t_wx[((warp * L) * G + q) * kLanes + lane];
                        hold[0] = C::step(t0 - 1 == 0 ? h_init : 0.f, gp, par);
                    }
                } else {
                    hold[0] = (t0 == 0) ? h_init : t_h[(warp * L) * kLanes + lane];
    #pragma unroll
                    for (int i = 0; i < L; ++i) hold[i + 1] = t_h[(warp * L + i + 1) * kLanes + lane];
                }
                // this warp is done with the stage: let the producer refill it
                __syncwarp();
                if (lane == 0) dp_mbar_arrive(&empty[s]);

                if (FIRST) {
    #pragma unroll
                    for (int i = 0; i < L; ++i) hold[i + 1] = C::step(t0 + i == 0 ? h_init : 0.f, g[i], par);
                }

                // ---- carry-independent part: delta_{t0+i} = P_i * delta_in + D_i
                float P[L], D[L];
                {
                    float pp = 1.f, dd = 0.f;
    #pragma unroll
                    for (int i = 0; i < L; ++i) {
                        float f, j;
                        typename C::Acts acts;
                        C::eval(hold[i], g[i], par, f, j, acts);
                        float F = f - hold[i + 1];
                        const bool ok = FULL || t0 + i < a.T;
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

                // ---- the sub-tile maps of the round meet in shared memory
                float* maps = s_map + (r & 1) * (W * 2 * kLanes);
                reinterpret_cast<float2*>(maps)[warp * kLanes + lane] = make_float2(P[L - 1], D[L - 1]);
                dp_named_sync(1, W * 32);
                const float c = fold_round<W>(maps, warp, lane, carry);

                // ---- results
                if (ch_ok) {
                    float prev_new = fmaf(a.omega, c, hold[0]);
                    const size_t o_base = ((size_t)b * a.T + t0) * d + ch;
    #pragma unroll
                    for (int i = 0; i < L; ++i) {
                        const int t = t0 + i;
                        if (FULL || t < a.T) {
                            const float nv = fmaf(a.omega, fmaf(P[i], c, D[i]), hold[i + 1]);
                            if (LAST) {
                                if (want_final) {
                                    fmax = max(fmax, absbits(C::step(prev_new, g[i], par) - nv));
                                    prev_new = nv;
                                }
                                st_f(reinterpret_cast<TIO*>(a.hout) + o_base + (size_t)i * d, nv);
                            } else {
                                reinterpret_cast<float*>(a.hout)[o_base + (size_t)i * d] = nv;
                            }
                        }
                    }
                    if (r == n_rounds - 1 && warp == 0 && a.tail_out) a.tail_out[(size_t)b * d + ch] = carry;
                }
            };
            if (t0 + L <= a.T)
                round_body(std::true_type{});
            else
                round_body(std::false_type{});
        }
    }
    if (timed_out) atomicExch(a.chain.status, (int)kErrChainTimeout);
    __syncthreads();
    block_residual_max(rmax, a.resid_bits, s_red);
    if (LAST && a.final_bits != nullptr) {
        __syncthreads();
        block_residual_max(fmax, a.final_bits, s_red);
    }
}

// ------------------------------------------------------------------ forward, all iterations in one sweep
// The K Newton iterations of a solve (and the residual of the result) in ONE walk over the time
// axis.  Iteration k+1 at step t needs iterate k at steps t-1 and t only; inside a round every warp
// holds the iterates of its own L steps in registers, and the state just before its sub-tile moves
// with the same delta carry the fold gives it (H_{t0-1} += omega * delta_{t0-1}).  So the passes
// follow each other round by round: K times (evaluate, compose, one named barrier, fold, update in
// registers), then the result is written once.  Reads wx once, writes H once; no work trajectory.
// Same arithmetic, in the same order, as K launches of diag_newton_pipe_kernel.
constexpr int kDiagFusedMaxK = 4;

template <int CELL, typename TIO, int L, int W, int NSTAGE>
__global__ void __launch_bounds__((W + 1) * 32, W * L > 64 ? 1 : 2)
diag_newton_fused_kernel(const __grid_constant__ CUtensorMap tm_wx, DiagFwdArgs a, int K) {
    using C = DiagCell<CELL>;
    constexpr int G = C::G;
    using S = DiagPipeFwdSmem<G, TIO, L, W, NSTAGE>;
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

    unsigned rmax[kDiagFusedMaxK] = {0u, 0u, 0u, 0u};
    unsigned fmax = 0u;
    bool timed_out = false;

    if (warp == W) {
        if (lane == 0) {
            for (int r = 0; r < n_rounds; ++r) {
                const int s = r % NSTAGE;
                if (r >= NSTAGE && !mbar_wait_bounded(&empty[s], ((r / NSTAGE) - 1) & 1, timed_out ? kWaitLimitAfterTimeout : kDiagPipeWaitLimit))
                    timed_out = true;
                mbar_expect_tx(&full[s], S::WX_TX);
                tma_load_3d(smem + s * S::STAGE, &tm_wx, &full[s], cb * kLanes, 0, row0 + r * LT - 1);
            }
            if (timed_out) drain_ring(full, NSTAGE, n_rounds, kDrainLimit);
        }
    } else {
        float par[C::NP];
#pragma unroll
        for (int p = 0; p < C::NP; ++p) par[p] = __ldg(a.par + (size_t)p * d + chl);
        const float h_init = a.halo ? __ldg(a.halo + (size_t)b * d + chl) : 0.f;
        const bool want_final = a.final_bits != nullptr;
        float carry[kDiagFusedMaxK] = {0.f, 0.f, 0.f, 0.f};
        int parity = 0;  // the two map buffers alternate from barrier to barrier

        for (int r = 0; r < n_rounds; ++r) {
            const int s = r % NSTAGE;
            if (!mbar_wait_bounded(&full[s], (r / NSTAGE) & 1, timed_out ? kWaitLimitAfterTimeout : kDiagPipeWaitLimit)) timed_out = true;
            const TIO* t_wx = reinterpret_cast<const TIO*>(smem + s * S::STAGE);
            const int t0 = r * LT + warp * L;

            auto round_body = [&](auto full_c) {
                constexpr bool FULL = decltype(full_c)::value;
                // row k of the box is time step r*LT - 1 + k
                float g[L][G], hold[L + 1];
    #pragma unroll
                for (int i = 0; i < L; ++i)
    #pragma unroll
                    for (int q = 0; q < G; ++q) g[i][q] = (float)t_wx[((warp * L + i + 1) * G + q) * kLanes + lane];
                // App. A guess: H^0_t = f(0, x_t), h0 only at t = 0
                if (t0 == 0) {
                    hold[0] = h_init;
                } else {
                    float gp[G];
    #pragma unroll
                    for (int q = 0; q < G; ++q) gp[q] = (float)t_wx[((warp * L) * G + q) * kLanes + lane];
                    hold[0] = C::step(t0 - 1 == 0 ? h_init : 0.f, gp, par);
                }
                __syncwarp();
                if (lane == 0) dp_mbar_arrive(&empty[s]);
    #pragma unroll
                for (int i = 0; i < L; ++i) hold[i + 1] = C::step(t0 + i == 0 ? h_init : 0.f, g[i], par);

    #pragma unroll
                for (int k = 0; k < kDiagFusedMaxK; ++k) {
                    if (k < K) {
                        // hold[0..L] is iterate k of steps t0-1 .. t0+L-1 (the guess for k = 0)
                        float P[L], D[L];
                        float pp = 1.f, dd = 0.f;
    #pragma unroll
                        for (int i = 0; i < L; ++i) {
                            float f, j;
                            typename C::Acts acts;
                            C::eval(hold[i], g[i], par, f, j, acts);
                            float F = f - hold[i + 1];
                            const bool ok = FULL || t0 + i < a.T;
                            if (!ok) {
                                j = 1.f;
                                F = 0.f;
                            }
                            if (ok && ch_ok) rmax[k] = max(rmax[k], absbits(F));
                            dd = fmaf(j, dd, F);
                            pp = j * pp;
                            P[i] = pp;
                            D[i] = dd;
                        }
                        float* maps = s_map + parity * (W * 2 * kLanes);
                        parity ^= 1;
                        reinterpret_cast<float2*>(maps)[warp * kLanes + lane] = make_float2(P[L - 1], D[L - 1]);
                        dp_named_sync(1, W * 32);
                        const float c = fold_round<W>(maps, warp, lane, carry[k]);
                        hold[0] = fmaf(a.omega, c, hold[0]);
    #pragma unroll
                        for (int i = 0; i < L; ++i) hold[i + 1] = fmaf(a.omega, fmaf(P[i], c, D[i]), hold[i + 1]);
                    }
                }

                if (ch_ok) {
                    const size_t o_base = ((size_t)b * a.T + t0) * d + ch;
    #pragma unroll
                    for (int i = 0; i < L; ++i) {
                        if (FULL || t0 + i < a.T) {
                            if (want_final) fmax = max(fmax, absbits(C::step(hold[i], g[i], par) - hold[i + 1]));
                            st_f(reinterpret_cast<TIO*>(a.hout) + o_base + (size_t)i * d, hold[i + 1]);
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
    for (int k = 0; k < kDiagFusedMaxK; ++k) {
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
template <int G, typename TIO, int L, int W, int NSTAGE>
struct DiagPipeBwdSmem {
    static constexpr int LT = W * L;
    static constexpr int WX_TX = LT * G * kLanes * (int)sizeof(TIO);
    static constexpr int ST_TX = (LT + 1) * kLanes * (int)sizeof(TIO);  // starts one step early
    static constexpr int G_TX = LT * kLanes * (int)sizeof(TIO);
    static constexpr int WX_BYTES = round128(WX_TX);
    static constexpr int ST_BYTES = round128(ST_TX);
    static constexpr int G_BYTES = round128(G_TX);
    static constexpr int STAGE = WX_BYTES + ST_BYTES + G_BYTES;
    static constexpr int MAP_OFF = NSTAGE * STAGE;
    static constexpr int MAP_BYTES = 2 * W * 2 * kLanes * 4;
    static constexpr int GP_OFF = MAP_OFF + MAP_BYTES;
    static constexpr int GP_BYTES = W * 3 * kLanes * 4;
    static constexpr int BAR_OFF = GP_OFF + GP_BYTES;
    static constexpr int TOTAL = BAR_OFF + 2 * NSTAGE * 8 + 64;
};

// nu_{t-1} = j_t (nu_t + g_t), nu_{T-1} = 0; mu_t = nu_t + g_t feeds the packed VJP.  Rounds run
// from the end of the sequence; warp 0 owns the highest steps of a round and the baton (nu)
// moves towards lower steps.  Parameter gradients are accumulated per thread over the whole
// sweep and summed over the warps in a fixed order: one partial row per chain.
template <int CELL, typename TIO, int L, int W, int NSTAGE>
__global__ void __launch_bounds__((W + 1) * 32, W * L > 64 ? 1 : 2)
diag_bwd_pipe_kernel(const __grid_constant__ CUtensorMap tm_wx, const __grid_constant__ CUtensorMap tm_st,
                     const __grid_constant__ CUtensorMap tm_g, DiagBwdArgs a) {
    using C = DiagCell<CELL>;
    constexpr int G = C::G, NP = C::NP;
    using S = DiagPipeBwdSmem<G, TIO, L, W, NSTAGE>;
    constexpr int LT = S::LT;
    extern __shared__ __align__(128) unsigned char smem[];
    float* s_map = reinterpret_cast<float*>(smem + S::MAP_OFF);
    float* s_gp = reinterpret_cast<float*>(smem + S::GP_OFF);  // [W][NP][32]
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
    float gp_acc[NP], gb_acc[G];
#pragma unroll
    for (int p = 0; p < NP; ++p) gp_acc[p] = 0.f;
#pragma unroll
    for (int q = 0; q < G; ++q) gb_acc[q] = 0.f;
    const bool want_bias = a.gb_partial != nullptr;

    if (warp == W) {
        if (lane == 0) {
            for (int r = 0; r < n_rounds; ++r) {
                const int s = r % NSTAGE;
                const int tile_t = n_rounds - 1 - r;
                if (r >= NSTAGE && !mbar_wait_bounded(&empty[s], ((r / NSTAGE) - 1) & 1, timed_out ? kWaitLimitAfterTimeout : kDiagPipeWaitLimit))
                    timed_out = true;
                unsigned char* base = smem + s * S::STAGE;
                mbar_expect_tx(&full[s], S::WX_TX + S::ST_TX + S::G_TX);
                tma_load_3d(base, &tm_wx, &full[s], cb * kLanes, 0, row0 + tile_t * LT);
                tma_load_3d(base + S::WX_BYTES, &tm_st, &full[s], cb * kLanes, 0, row0 + tile_t * LT - 1);
                tma_load_3d(base + S::WX_BYTES + S::ST_BYTES, &tm_g, &full[s], cb * kLanes, 0,
                            row0 + tile_t * LT);
            }
            if (timed_out) drain_ring(full, NSTAGE, n_rounds, kDrainLimit);
        }
    } else {
        float par[NP];
#pragma unroll
        for (int p = 0; p < NP; ++p) par[p] = __ldg(a.par + (size_t)p * d + chl);
        const float h_init = a.halo ? __ldg(a.halo + (size_t)b * d + chl) : 0.f;
        float carry = a.carry_in ? __ldg(a.carry_in + (size_t)b * d + chl) : 0.f;
        TIO* gwx = reinterpret_cast<TIO*>(a.g_wx) + (size_t)b * a.T * G * d + ch;

        for (int r = 0; r < n_rounds; ++r) {
            const int s = r % NSTAGE;
            const int tile_t = n_rounds - 1 - r;
            if (!mbar_wait_bounded(&full[s], (r / NSTAGE) & 1, timed_out ? kWaitLimitAfterTimeout : kDiagPipeWaitLimit)) timed_out = true;
            const TIO* t_wx = reinterpret_cast<const TIO*>(smem + s * S::STAGE);
            const TIO* t_st = reinterpret_cast<const TIO*>(smem + s * S::STAGE + S::WX_BYTES);
            const TIO* t_g = reinterpret_cast<const TIO*>(smem + s * S::STAGE + S::WX_BYTES + S::ST_BYTES);
            // i = 0 is the highest step of the sub-tile
            const int k_hi = (W - 1 - warp) * L + (L - 1);  // position inside the round
            const int t_hi = tile_t * LT + k_hi;

            // Rounds that lie fully inside the sequence take a variant without range checks.
            auto round_body = [&](auto full_c) {
                constexpr bool FULL = decltype(full_c)::value;
                float g[L][G], hp[L], gg[L];
    #pragma unroll
                for (int i = 0; i < L; ++i) {
                    const int k = k_hi - i;
    #pragma unroll
                    for (int q = 0; q < G; ++q) g[i][q] = (float)t_wx[(k * G + q) * kLanes + lane];
                    hp[i] = (t_hi - i == 0) ? h_init : (float)t_st[k * kLanes + lane];  // row k = step t-1
                    gg[i] = (FULL || t_hi - i < a.T) ? (float)t_g[k * kLanes + lane] : 0.f;
                }
                __syncwarp();
                if (lane == 0) dp_mbar_arrive(&empty[s]);

                // ---- carry-independent part: mu_{t_hi-i} = P_i * nu_top + D_i
                float P[L], D[L];
                typename C::Acts acts[L];
                float pp = 1.f, dd = 0.f;
    #pragma unroll
                for (int i = 0; i < L; ++i) {
                    float f, j;
                    C::eval(hp[i], g[i], par, f, j, acts[i]);
                    if (!FULL && t_hi - i >= a.T) j = 1.f;
                    P[i] = pp;
                    D[i] = dd + gg[i];
                    dd = j * (dd + gg[i]);
                    pp = j * pp;
                }

                // ---- the sub-tile maps of the round meet in shared memory
                float* maps = s_map + (r & 1) * (W * 2 * kLanes);
                reinterpret_cast<float2*>(maps)[warp * kLanes + lane] = make_float2(pp, dd);
                dp_named_sync(1, W * 32);
                const float c = fold_round<W>(maps, warp, lane, carry);

                // ---- packed VJP
                TIO* gw_hi = gwx + (size_t)t_hi * G * d;
    #pragma unroll
                for (int i = 0; i < L; ++i) {
                    const int t = t_hi - i;
                    if (FULL || t < a.T) {
                        const float mu = fmaf(P[i], c, D[i]);
                        float gw[G], gp[NP];
                        C::vjp(hp[i], acts[i], par, mu, gw, gp);
                        if (ch_ok) {
    #pragma unroll
                            for (int q = 0; q < G; ++q) st_f(gw_hi + ((ptrdiff_t)q - (ptrdiff_t)i * G) * d, gw[q]);
                            if (a.mu_out) a.mu_out[((size_t)b * a.T + t) * d + ch] = mu;
                        }
    #pragma unroll
                        for (int p = 0; p < NP; ++p) gp_acc[p] += gp[p];
                        if (want_bias) {
    #pragma unroll
                            for (int q = 0; q < G; ++q) gb_acc[q] += gw[q];
                        }
                    }
                }
                if (r == n_rounds - 1 && warp == 0 && ch_ok && a.g_h0) a.g_h0[(size_t)b * d + ch] = carry;
            };
            if (t_hi < a.T)
                round_body(std::true_type{});
            else
                round_body(std::false_type{});
        }
#pragma unroll
        for (int p = 0; p < NP; ++p) s_gp[(warp * NP + p) * kLanes + lane] = gp_acc[p];
    }
    if (timed_out) atomicExch(a.chain.status, (int)kErrChainTimeout);
    __syncthreads();
    if (warp == 0 && ch_ok) {
#pragma unroll
        for (int p = 0; p < NP; ++p) {
            float sum = 0.f;
#pragma unroll
            for (int w = 0; w < W; ++w) sum += s_gp[(w * NP + p) * kLanes + lane];
            a.gp_partial[((size_t)b * NP + p) * d + ch] = sum;
        }
    }
    if (want_bias) {  // per-gate sums of g_wx (bias gradient): same fixed-order reduction, one gate at a time
#pragma unroll
        for (int q = 0; q < G; ++q) {
            __syncthreads();
            if (warp < W) s_gp[warp * kLanes + lane] = gb_acc[q];
            __syncthreads();
            if (warp == 0 && ch_ok) {
                float sum = 0.f;
#pragma unroll
                for (int w = 0; w < W; ++w) sum += s_gp[w * kLanes + lane];
                a.gb_partial[((size_t)b * G + q) * d + ch] = sum;
            }
        }
    }
}

// ------------------------------------------------------------------ launchers
template <int CELL, typename TIO, int NSTAGE, int L, int W>
cudaError_t launch_fwd_w(const DiagFwdArgs& a, bool first, bool last, cudaStream_t s) {
    constexpr int G = DiagCell<CELL>::G;
    constexpr int kDPW = W, kDPL = L;
    using S = DiagPipeFwdSmem<G, TIO, kDPL, kDPW, NSTAGE>;
    CUtensorMap tm_wx, tm_h;
    const uint64_t rows = (uint64_t)a.B * a.T;
    if (!make_tile_map(&tm_wx, a.wx, sizeof(TIO), rows, G, a.d, S::LT + 1)) return cudaErrorNotSupported;
    if (first)
        tm_h = tm_wx;
    else if (!make_tile_map(&tm_h, a.hin, 4, rows, 1, a.d, S::LT + 1))
        return cudaErrorNotSupported;
    const int grid = a.B * ((a.d + kLanes - 1) / kLanes);
    const int threads = (kDPW + 1) * 32;
#define PRB_DIAG_FWD(F, LA)                                                                      \
    {                                                                                            \
        auto k = diag_newton_pipe_kernel<CELL, TIO, kDPL, kDPW, NSTAGE, F, LA>;                  \
        cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);          \
        k<<<grid, threads, S::TOTAL, s>>>(tm_wx, tm_h, a);                                       \
    }
    if (first && last) PRB_DIAG_FWD(true, true)
    else if (first) PRB_DIAG_FWD(true, false)
    else if (last) PRB_DIAG_FWD(false, true)
    else PRB_DIAG_FWD(false, false)
#undef PRB_DIAG_FWD
    return cudaGetLastError();
}

template <int CELL, typename TIO, int NSTAGE, int L, int W>
cudaError_t launch_fused_w(const DiagFwdArgs& a, int K, cudaStream_t s) {
    constexpr int G = DiagCell<CELL>::G;
    using S = DiagPipeFwdSmem<G, TIO, L, W, NSTAGE>;
    CUtensorMap tm_wx;
    const uint64_t rows = (uint64_t)a.B * a.T;
    if (!make_tile_map(&tm_wx, a.wx, sizeof(TIO), rows, G, a.d, S::LT + 1)) return cudaErrorNotSupported;
    const int grid = a.B * ((a.d + kLanes - 1) / kLanes);
    auto k = diag_newton_fused_kernel<CELL, TIO, L, W, NSTAGE>;
    cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
    k<<<grid, (W + 1) * 32, S::TOTAL, s>>>(tm_wx, a, K);
    return cudaGetLastError();
}

// With few chains (up to 1.5 per SM) every chain gets 16 compute warps per CTA; with many chains
// two 8-warp CTAs share an SM.
inline bool wide_cta(int B, int d) { return 2 * B * ((d + kLanes - 1) / kLanes) <= 3 * sm_count(); }

template <int CELL, typename TIO, int NSTAGE>
cudaError_t launch_fwd_t(const DiagFwdArgs& a, bool first, bool last, cudaStream_t s) {
    using Wide = DiagPipeFwdSmem<DiagCell<CELL>::G, TIO, 8, 16, NSTAGE>;
    if constexpr (Wide::TOTAL > 227 * 1024) {
        return launch_fwd_w<CELL, TIO, NSTAGE, 8, 8>(a, first, last, s);
    } else {
        if (!wide_cta(a.B, a.d)) return launch_fwd_w<CELL, TIO, NSTAGE, 8, 8>(a, first, last, s);
        return launch_fwd_w<CELL, TIO, NSTAGE, 8, 16>(a, first, last, s);
    }
}

template <int CELL, typename TIO, int NSTAGE>
cudaError_t launch_fused_t(const DiagFwdArgs& a, int K, cudaStream_t s) {
    using Wide = DiagPipeFwdSmem<DiagCell<CELL>::G, TIO, 8, 16, NSTAGE>;
    if constexpr (Wide::TOTAL > 227 * 1024) {
        return launch_fused_w<CELL, TIO, NSTAGE, 8, 8>(a, K, s);
    } else {
        if (!wide_cta(a.B, a.d)) return launch_fused_w<CELL, TIO, NSTAGE, 8, 8>(a, K, s);
        return launch_fused_w<CELL, TIO, NSTAGE, 8, 16>(a, K, s);
    }
}

template <int CELL, typename TIO, int NSTAGE, int L, int W>
cudaError_t launch_bwd_w(const DiagBwdArgs& a, cudaStream_t s) {
    constexpr int G = DiagCell<CELL>::G;
    constexpr int kDPW = W, kDPL = L;
    using S = DiagPipeBwdSmem<G, TIO, kDPL, kDPW, NSTAGE>;
    CUtensorMap tm_wx, tm_st, tm_g;
    const uint64_t rows = (uint64_t)a.B * a.T;
    if (!make_tile_map(&tm_wx, a.wx, sizeof(TIO), rows, G, a.d, S::LT) ||
        !make_tile_map(&tm_st, a.states, sizeof(TIO), rows, 1, a.d, S::LT + 1) ||
        !make_tile_map(&tm_g, a.grad_states, sizeof(TIO), rows, 1, a.d, S::LT))
        return cudaErrorNotSupported;
    const int grid = a.B * ((a.d + kLanes - 1) / kLanes);
    auto k = diag_bwd_pipe_kernel<CELL, TIO, kDPL, kDPW, NSTAGE>;
    cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
    k<<<grid, (kDPW + 1) * 32, S::TOTAL, s>>>(tm_wx, tm_st, tm_g, a);
    return cudaGetLastError();
}

constexpr int kMaxDynSmem = 227 * 1024;

template <int CELL, typename TIO, int NSTAGE>
cudaError_t launch_bwd_t(const DiagBwdArgs& a, cudaStream_t s) {
    // the 16-warp ring of a cell with many gates may not fit shared memory (Titans, fp32)
    using Wide = DiagPipeBwdSmem<DiagCell<CELL>::G, TIO, 8, 16, NSTAGE>;
    if constexpr (Wide::TOTAL > kMaxDynSmem) {
        return launch_bwd_w<CELL, TIO, NSTAGE, 8, 8>(a, s);
    } else {
        if (!wide_cta(a.B, a.d)) return launch_bwd_w<CELL, TIO, NSTAGE, 8, 8>(a, s);
        return launch_bwd_w<CELL, TIO, NSTAGE, 8, 16>(a, s);
    }
}

}  // namespace

cudaError_t launch_diag_newton_pipe(int cell, int dtype, const DiagFwdArgs& a, bool first, bool last,
                                    cudaStream_t s) {
    if (cell == kCellGruDiag)
        return dtype == kF32 ? launch_fwd_t<kCellGruDiag, float, 2>(a, first, last, s)
                             : launch_fwd_t<kCellGruDiag, __nv_bfloat16, 3>(a, first, last, s);
    if (cell == kCellTitans)
        return dtype == kF32 ? launch_fwd_t<kCellTitans, float, 2>(a, first, last, s)
                             : launch_fwd_t<kCellTitans, __nv_bfloat16, 3>(a, first, last, s);
    if (cell == kCellCfc)
        return dtype == kF32 ? launch_fwd_t<kCellCfc, float, 2>(a, first, last, s)
                             : launch_fwd_t<kCellCfc, __nv_bfloat16, 3>(a, first, last, s);
    return dtype == kF32 ? launch_fwd_t<kCellNlru, float, 2>(a, first, last, s)
                         : launch_fwd_t<kCellNlru, __nv_bfloat16, 3>(a, first, last, s);
}

// all K iterations (1 <= K <= 4) from the App. A guess in one sweep; a.resid_bits points at the first
// of K history slots, a.hout is the result in the I/O dtype, a.hin / a.carry_in are not used
cudaError_t launch_diag_newton_fused(int cell, int dtype, const DiagFwdArgs& a, int K, cudaStream_t s) {
    if (K < 1 || K > kDiagFusedMaxK || a.carry_in) return cudaErrorNotSupported;
    if (cell == kCellGruDiag)
        return dtype == kF32 ? launch_fused_t<kCellGruDiag, float, 2>(a, K, s)
                             : launch_fused_t<kCellGruDiag, __nv_bfloat16, 3>(a, K, s);
    if (cell == kCellTitans)
        return dtype == kF32 ? launch_fused_t<kCellTitans, float, 2>(a, K, s)
                             : launch_fused_t<kCellTitans, __nv_bfloat16, 3>(a, K, s);
    if (cell == kCellCfc)
        return dtype == kF32 ? launch_fused_t<kCellCfc, float, 2>(a, K, s)
                             : launch_fused_t<kCellCfc, __nv_bfloat16, 3>(a, K, s);
    return dtype == kF32 ? launch_fused_t<kCellNlru, float, 2>(a, K, s)
                         : launch_fused_t<kCellNlru, __nv_bfloat16, 3>(a, K, s);
}

cudaError_t launch_diag_bwd_pipe(int cell, int dtype, const DiagBwdArgs& a, cudaStream_t s) {
    if (cell == kCellGruDiag)
        return dtype == kF32 ? launch_bwd_t<kCellGruDiag, float, 2>(a, s)
                             : launch_bwd_t<kCellGruDiag, __nv_bfloat16, 3>(a, s);
    if (cell == kCellTitans)
        return dtype == kF32 ? launch_bwd_t<kCellTitans, float, 2>(a, s)
                             : launch_bwd_t<kCellTitans, __nv_bfloat16, 3>(a, s);
    if (cell == kCellCfc)
        return dtype == kF32 ? launch_bwd_t<kCellCfc, float, 2>(a, s)
                             : launch_bwd_t<kCellCfc, __nv_bfloat16, 3>(a, s);
    return dtype == kF32 ? launch_bwd_t<kCellNlru, float, 2>(a, s)
                         : launch_bwd_t<kCellNlru, __nv_bfloat16, 3>(a, s);
}

}  // namespace prb
