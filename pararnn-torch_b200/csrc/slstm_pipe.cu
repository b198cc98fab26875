// ParaSLSTM mix='diag', warp-pipelined persistent kernels (the fast path on a full GPU).
//
// One CTA owns one chain (batch row x 32 channels, lane = channel) and walks the time axis in
// rounds of W*L steps.  A dedicated producer warp streams the inputs of the coming rounds into a
// shared-memory ring with TMA tile loads (full / empty mbarriers).  The W compute warps own L
// consecutive steps of every round each.  A warp first does everything that does not depend on
// the scan carry (gates, Jacobian entries, residual) for its L steps, then waits for the carry of
// the warp before it (named barrier), runs the L-step recurrence on the carry VECTOR, hands the
// carry to the next warp, and only then writes its results.  The carry therefore travels through
// the warps like a baton; no affine maps are composed and the arithmetic per step is the
// sequential algorithm's, while the expensive carry-independent part runs W-way in parallel.
//
// Same math as slstm_kernels.cu (slstm_cell.cuh); reference behaviour
// restated there.
#include "common.cuh"
#include "kernels.h"
#include "slstm_cell.cuh"
#include "tma.cuh"

#include <type_traits>

namespace prb {

constexpr uint32_t kPipeWaitLimit = 1u << 24;

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void named_sync(int id, int count) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}
__device__ __forceinline__ void named_arrive(int id, int count) {
    asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(count) : "memory");
}

// ------------------------------------------------------------------ Newton
template <typename TIO, int L, int W, int NSTAGE>
struct PipeNewtonSmem {
    static constexpr int LT = W * L;
    static constexpr int WX_BYTES = LT * 4 * kLanes * (int)sizeof(TIO);
    static constexpr int ST_BYTES = (LT + 1) * 4 * kLanes * 4;
    static constexpr int STAGE = WX_BYTES + ST_BYTES;
    static constexpr int SLOT_OFF = NSTAGE * STAGE;
    static constexpr int SLOT_BYTES = W * 4 * kLanes * 4;
    static constexpr int BAR_OFF = SLOT_OFF + SLOT_BYTES;
    static constexpr int RED_OFF = BAR_OFF + 2 * NSTAGE * 8;
    static constexpr int TOTAL = RED_OFF + (W + 1) * 4 + 64;
};

template <typename TIO, int L, int W, int NSTAGE, bool LAST>
__global__ void __launch_bounds__((W + 1) * 32, 2)
slstm_newton_pipe_kernel(const __grid_constant__ CUtensorMap tm_wx,
                         const __grid_constant__ CUtensorMap tm_st, SlstmNewtonArgs a) {
    using S = PipeNewtonSmem<TIO, L, W, NSTAGE>;
    constexpr int LT = S::LT;
    extern __shared__ __align__(128) unsigned char smem[];
    float* s_slot = reinterpret_cast<float*>(smem + S::SLOT_OFF);  // [W][4][32] carry entering warp w
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
    const SegRange sg = seg_range(a.T, a.n_seg, a.seg_len);
    const int n_rounds = (sg.hi - sg.lo + LT - 1) / LT;
    const int row0 = b * a.T + sg.lo;

    if (threadIdx.x == 0) {
        tma_prefetch_desc(&tm_wx);
        tma_prefetch_desc(&tm_st);
        for (int s = 0; s < NSTAGE; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], W);
        }
        mbar_fence_init();
    }
    if (warp == 0) {
#pragma unroll
        for (int q = 0; q < 4; ++q)
            s_slot[(0 * 4 + q) * kLanes + lane] =
                a.carry_in ? __ldg(a.carry_in + (((size_t)sg.seg * a.B + b) * 4 + q) * d + chl) : 0.f;
    }
    __syncthreads();

    unsigned rmax = 0u, fmax = 0u;
    bool timed_out = false;

    if (warp == W) {
        // ---------------- producer warp: one lane streams the rounds into the ring
        if (lane == 0) {
            for (int r = 0; r < n_rounds; ++r) {
                const int s = r % NSTAGE;
                if (r >= NSTAGE && !mbar_wait_bounded_sleepy(&empty[s], ((r / NSTAGE) - 1) & 1, timed_out ? kWaitLimitAfterTimeout : kPipeWaitLimit))
                    timed_out = true;
                unsigned char* base = smem + s * S::STAGE;
                mbar_expect_tx(&full[s], S::STAGE);
                tma_load_3d(base, &tm_wx, &full[s], cb * kLanes, 0, row0 + r * LT);
                tma_load_3d(base + S::WX_BYTES, &tm_st, &full[s], cb * kLanes, 0, row0 + r * LT - 1);
            }
            if (timed_out) drain_ring(full, NSTAGE, n_rounds, kDrainLimit);
        }
    } else {
        // ---------------- compute warps
        float r4[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) r4[q] = __ldg(a.r + (size_t)q * d + chl);
        const bool want_final = LAST && a.final_bits != nullptr;
        const int next = (warp + 1) % W;
        float* slot_in = s_slot + warp * 4 * kLanes + lane;
        float* slot_out = s_slot + next * 4 * kLanes + lane;

        for (int r = 0; r < n_rounds; ++r) {
            const int s = r % NSTAGE;
            // after a time-out the warp keeps walking (the named-barrier hand-over needs every
            // warp) but its waits give up after a few polls: the result is void, status says so
            if (!mbar_wait_bounded_sleepy(&full[s], (r / NSTAGE) & 1, timed_out ? kWaitLimitAfterTimeout : kPipeWaitLimit)) timed_out = true;
            const TIO* t_wx = reinterpret_cast<const TIO*>(smem + s * S::STAGE);
            const float* t_st = reinterpret_cast<const float*>(smem + s * S::STAGE + S::WX_BYTES);
            const int t0 = sg.lo + r * LT + warp * L;

            // Rounds that lie fully inside the sequence take a variant without range checks.
            auto round_body = [&](auto full_c) {
                constexpr bool FULL = decltype(full_c)::value;
                float w[L][4], st[L + 1][4];
    #pragma unroll
                for (int i = 0; i < L; ++i) {
    #pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        w[i][q] = (float)t_wx[((warp * L + i) * 4 + q) * kLanes + lane];
                        st[i + 1][q] = t_st[((warp * L + i + 1) * 4 + q) * kLanes + lane];
                    }
                }
                if (t0 == 0) {
    #pragma unroll
                    for (int q = 0; q < 4; ++q)
                        st[0][q] = a.halo ? __ldg(a.halo + (size_t)b * a.halo_stride + (size_t)q * d + chl) : 0.f;
                } else {
    #pragma unroll
                    for (int q = 0; q < 4; ++q) st[0][q] = t_st[((warp * L) * 4 + q) * kLanes + lane];
                }
                // this warp is done with the stage: let the producer refill it
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[s]);

                // ---- carry-independent part
                SlstmLin lin[L];
                float F[L][4];
    #pragma unroll
                for (int i = 0; i < L; ++i) {
                    slstm_linearize(st[i], w[i], r4, a.eps, lin[i]);
                    const bool ok = FULL || t0 + i < sg.hi;
                    float fc = lin[i].pc - st[i + 1][0], fn = lin[i].pn - st[i + 1][1];
                    float fm = lin[i].pm - st[i + 1][2], fh = lin[i].ph - st[i + 1][3];
                    if (!ok) {
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
                }

                // ---- the baton: carry from the previous warp (previous round's last warp for warp 0)
                if (!(r == 0 && warp == 0)) named_sync(1 + warp, 64);
                float xc = slot_in[0], xn = slot_in[kLanes], xm = slot_in[2 * kLanes], xh = slot_in[3 * kLanes];
                const float c0 = xc, c1 = xn, c2 = xm, c3 = xh;
                float dl[L][4];
    #pragma unroll
                for (int i = 0; i < L; ++i) {
                    slstm_apply(lin[i], F[i][0], F[i][1], F[i][2], F[i][3], xc, xn, xm, xh);
                    dl[i][0] = xc; dl[i][1] = xn; dl[i][2] = xm; dl[i][3] = xh;
                }
                slot_out[0] = xc;
                slot_out[kLanes] = xn;
                slot_out[2 * kLanes] = xm;
                slot_out[3 * kLanes] = xh;
                if (!(r == n_rounds - 1 && warp == W - 1)) named_arrive(1 + next, 64);

                // ---- results
                const size_t o_base = ((size_t)b * a.T + t0) * 4 * d + ch;
                float pn4[4] = {fmaf(a.omega, c0, st[0][0]), fmaf(a.omega, c1, st[0][1]),
                                fmaf(a.omega, c2, st[0][2]), fmaf(a.omega, c3, st[0][3])};
    #pragma unroll
                for (int i = 0; i < L; ++i) {
                    const int t = t0 + i;
                    if ((FULL || t < sg.hi) && ch_ok) {
                        const float o0 = fmaf(a.omega, dl[i][0], st[i + 1][0]);
                        const float o1 = fmaf(a.omega, dl[i][1], st[i + 1][1]);
                        const float o2 = fmaf(a.omega, dl[i][2], st[i + 1][2]);
                        const float o3 = fmaf(a.omega, dl[i][3], st[i + 1][3]);
                        if (want_final) {
                            float pred[4];
                            slstm_predict(pn4, w[i], r4, a.eps, pred);
                            fmax = max(fmax, max(max(absbits(pred[0] - o0), absbits(pred[1] - o1)),
                                                 max(absbits(pred[2] - o2), absbits(pred[3] - o3))));
                            pn4[0] = o0; pn4[1] = o1; pn4[2] = o2; pn4[3] = o3;
                        }
                        if (LAST) {
                            TIO* o = reinterpret_cast<TIO*>(a.sout) + o_base + (size_t)i * 4 * d;
                            st_f(o, o0);
                            st_f(o + d, o1);
                            st_f(o + 2 * (size_t)d, o2);
                            st_f(o + 3 * (size_t)d, o3);
                        } else {
                            float* o = reinterpret_cast<float*>(a.sout) + o_base + (size_t)i * 4 * d;
                            o[0] = o0;
                            o[d] = o1;
                            o[2 * (size_t)d] = o2;
                            o[3 * (size_t)d] = o3;
                        }
                    }
                }
                if (r == n_rounds - 1 && warp == W - 1 && a.tail_out && ch_ok && sg.hi == a.T) {
                    a.tail_out[((size_t)b * 4 + 0) * d + ch] = xc;
                    a.tail_out[((size_t)b * 4 + 1) * d + ch] = xn;
                    a.tail_out[((size_t)b * 4 + 2) * d + ch] = xm;
                    a.tail_out[((size_t)b * 4 + 3) * d + ch] = xh;
                }
            };
            if (t0 + L <= sg.hi)
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

// ------------------------------------------------------------------ backward
// HID: the cotangent arrives for one state slot only, as a (B,T,d) array
template <typename TIO, int L, int W, int NSTAGE, bool HID = false>
struct PipeBwdSmem {
    static constexpr int LT = W * L;
    static constexpr int WX_BYTES = LT * 4 * kLanes * (int)sizeof(TIO);
    static constexpr int ST_BYTES = ((LT + 1) * 4 * kLanes * (int)sizeof(TIO) + 127) / 128 * 128;
    static constexpr int G_BYTES = HID ? (LT * kLanes * (int)sizeof(TIO) + 127) / 128 * 128 : WX_BYTES;
    static constexpr int G_TX = HID ? LT * kLanes * (int)sizeof(TIO) : WX_BYTES;
    static constexpr int STAGE = WX_BYTES + ST_BYTES + G_BYTES;
    static constexpr int SLOT_OFF = NSTAGE * STAGE;
    static constexpr int SLOT_BYTES = (W + 1) * 4 * kLanes * 4;  // W carry slots + reduction scratch
    static constexpr int BAR_OFF = SLOT_OFF + SLOT_BYTES + W * 4 * kLanes * 4;
    static constexpr int TOTAL = BAR_OFF + 2 * NSTAGE * 8 + 64;
};

// Rounds run from the end of the sequence; warp 0 owns the highest steps of a round and the
// baton (nu, the adjoint propagated from later steps) moves towards lower steps.
// nu_{t-1} = J_t^T (nu_t + g_t) is evaluated through the packed-VJP quantities:
// (d_cn f, d_nn f, d_zf, sum_g r_g d_zg).
// SLOT = -1: the cotangent is the full (B,T,4,d) array; SLOT = 0..3: it is (B,T,d), of that slot alone
// (a compile-time slot, so the three absent terms cost nothing).
template <typename TIO, int L, int W, int NSTAGE, int SLOT, bool BIAS>
__global__ void __launch_bounds__(W * 32, 2)
slstm_bwd_pipe_kernel(const __grid_constant__ CUtensorMap tm_wx, const __grid_constant__ CUtensorMap tm_st,
                      const __grid_constant__ CUtensorMap tm_g, SlstmBwdArgs a) {
    constexpr bool HID = SLOT >= 0;
    using S = PipeBwdSmem<TIO, L, W, NSTAGE, HID>;
    constexpr int LT = S::LT;
    extern __shared__ __align__(128) unsigned char smem[];
    float* s_slot = reinterpret_cast<float*>(smem + S::SLOT_OFF);
    float* s_gp = s_slot + (W + 1) * 4 * kLanes;  // [W][4][32]
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
    const SegRange sg = seg_range(a.T, a.n_seg, a.seg_len);
    const int n_rounds = (sg.hi - sg.lo + LT - 1) / LT;
    const int row0 = b * a.T + sg.lo;

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
    if (warp == 0) {
#pragma unroll
        for (int q = 0; q < 4; ++q)
            s_slot[q * kLanes + lane] =
                a.carry_in ? __ldg(a.carry_in + (((size_t)sg.seg * a.B + b) * 4 + q) * d + chl) : 0.f;
    }
    __syncthreads();
    bool timed_out = false;
    float gr[4] = {0.f, 0.f, 0.f, 0.f}, gb[4] = {0.f, 0.f, 0.f, 0.f};

    // No dedicated producer warp: lane 0 of warp 0 keeps the TMA ring full.  At the start of round r
    // it refills the stage of round r-1, which every warp has copied to registers by then.
    auto issue = [&](int r) {
        const int s = r % NSTAGE;
        const int tile_t = n_rounds - 1 - r;
        unsigned char* base = smem + s * S::STAGE;
        mbar_expect_tx(&full[s], S::WX_BYTES + (LT + 1) * 4 * kLanes * (int)sizeof(TIO) + S::G_TX);
        tma_load_3d(base, &tm_wx, &full[s], cb * kLanes, 0, row0 + tile_t * LT);
        tma_load_3d(base + S::WX_BYTES, &tm_st, &full[s], cb * kLanes, 0, row0 + tile_t * LT - 1);
        tma_load_3d(base + S::WX_BYTES + S::ST_BYTES, &tm_g, &full[s], cb * kLanes, 0, row0 + tile_t * LT);
    };
    if (threadIdx.x == 0)
        for (int r = 0; r < NSTAGE && r < n_rounds; ++r) issue(r);
    {
        float r4[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) r4[q] = __ldg(a.r + (size_t)q * d + chl);
        const int next = (warp + 1) % W;
        float* slot_in = s_slot + warp * 4 * kLanes + lane;
        float* slot_out = s_slot + next * 4 * kLanes + lane;
        TIO* gwx = reinterpret_cast<TIO*>(a.g_wx) + (size_t)b * a.T * 4 * d + ch;

        for (int r = 0; r < n_rounds; ++r) {
            const int s = r % NSTAGE;
            const int tile_t = n_rounds - 1 - r;
            if (threadIdx.x == 0 && r >= 1 && r - 1 + NSTAGE < n_rounds) {
                if (!mbar_wait_bounded(&empty[(r - 1) % NSTAGE], ((r - 1) / NSTAGE) & 1, timed_out ? kWaitLimitAfterTimeout : kPipeWaitLimit))
                    timed_out = true;
                issue(r - 1 + NSTAGE);
            }
            __syncwarp();
            // after a time-out the warp keeps walking (the named-barrier hand-over needs every
            // warp) but its waits give up after a few polls: the result is void, status says so
            if (!mbar_wait_bounded(&full[s], (r / NSTAGE) & 1, timed_out ? kWaitLimitAfterTimeout : kPipeWaitLimit)) timed_out = true;
            const TIO* t_wx = reinterpret_cast<const TIO*>(smem + s * S::STAGE);
            const TIO* t_st = reinterpret_cast<const TIO*>(smem + s * S::STAGE + S::WX_BYTES);
            const TIO* t_g = reinterpret_cast<const TIO*>(smem + s * S::STAGE + S::WX_BYTES + S::ST_BYTES);
            const int row_hi = (W - 1 - warp) * L + (L - 1);
            const int t_hi = sg.lo + tile_t * LT + row_hi;

            // Rounds that lie fully inside the sequence take a variant without range checks.
            auto round_body = [&](auto full_c) {
                constexpr bool FULL = decltype(full_c)::value;
                SlstmAct act[L];
                float g[L][4];
    #pragma unroll
                for (int i = 0; i < L; ++i) {
                    const int row = row_hi - i;
                    const int t = t_hi - i;
                    float w[4], prev[4];
    #pragma unroll
                    for (int q = 0; q < 4; ++q) w[q] = (float)t_wx[(row * 4 + q) * kLanes + lane];
                    if (i == L - 1 && t == 0) {
    #pragma unroll
                        for (int q = 0; q < 4; ++q)
                            prev[q] = a.halo ? __ldg(a.halo + (size_t)b * a.halo_stride + (size_t)q * d + chl) : 0.f;
                    } else {
    #pragma unroll
                        for (int q = 0; q < 4; ++q) prev[q] = (float)t_st[(row * 4 + q) * kLanes + lane];
                    }
                    if (HID) {
                        const float v = (float)t_g[row * kLanes + lane];
    #pragma unroll
                        for (int q = 0; q < 4; ++q) g[i][q] = (q == SLOT) ? v : 0.f;
                    } else {
    #pragma unroll
                        for (int q = 0; q < 4; ++q) g[i][q] = (float)t_g[(row * 4 + q) * kLanes + lane];
                    }
                    slstm_acts(prev, w, r4, a.eps, act[i]);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[s]);

                if (!(r == 0 && warp == 0)) named_sync(1 + warp, 64);
                float nc = slot_in[0], nn = slot_in[kLanes], nm = slot_in[2 * kLanes], nh = slot_in[3 * kLanes];
                float dz[L][4];
    #pragma unroll
                for (int i = 0; i < L; ++i) {
                    const int t = t_hi - i;
                    if (FULL || t < sg.hi) {
                        const SlstmAct& sa = act[i];
                        const float mc = nc + g[i][0], mn_ = nn + g[i][1], mm = nm + g[i][2], mh = nh + g[i][3];
                        const float cn = fmaf(sa.f, sa.c, sa.i * sa.z);
                        const float u = cn * sa.invD;
                        const float d_o = mh * u;
                        const float d_cn = fmaf(mh, sa.o * sa.invD, mc);
                        const float d_nn = fmaf(mh, -(sa.o * u) * sa.invD, mn_);
                        const float d_f = fmaf(d_cn, sa.c, d_nn * sa.n);
                        const float d_i = fmaf(d_cn, sa.z, d_nn);
                        const float d_z = d_cn * sa.i;
                        const float d_zo = d_o * sa.o * (1.f - sa.o);
                        const float d_zz = d_z * (1.f - sa.z * sa.z);
                        const float d_mn = mm - d_i * sa.i - d_f * sa.f;
                        const float d_zi = fmaf(d_i, sa.i, d_mn * (1.f - sa.alpha));
                        const float d_zf = fmaf(d_f, sa.f, d_mn * sa.alpha);
                        dz[i][0] = d_zi; dz[i][1] = d_zf; dz[i][2] = d_zz; dz[i][3] = d_zo;
                        nc = d_cn * sa.f;
                        nn = d_nn * sa.f;
                        nm = d_zf;
                        nh = fmaf(r4[0], d_zi, fmaf(r4[1], d_zf, fmaf(r4[2], d_zz, r4[3] * d_zo)));
                    } else {
                        dz[i][0] = dz[i][1] = dz[i][2] = dz[i][3] = 0.f;
                    }
                }
                slot_out[0] = nc;
                slot_out[kLanes] = nn;
                slot_out[2 * kLanes] = nm;
                slot_out[3 * kLanes] = nh;
                if (!(r == n_rounds - 1 && warp == W - 1)) named_arrive(1 + next, 64);

                TIO* gw_hi = gwx + (size_t)t_hi * 4 * d;
    #pragma unroll
                for (int i = 0; i < L; ++i) {
                    const int t = t_hi - i;
                    if (FULL || t < sg.hi) {
                        if (ch_ok) {
                            TIO* o = gw_hi - (size_t)i * 4 * d;
                            st_f(o, dz[i][0]);
                            st_f(o + d, dz[i][1]);
                            st_f(o + 2 * (size_t)d, dz[i][2]);
                            st_f(o + 3 * (size_t)d, dz[i][3]);
                        }
    #pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            gr[q] = fmaf(dz[i][q], act[i].hp, gr[q]);
                            if (BIAS) gb[q] += dz[i][q];
                        }
                    }
                }
                if (r == n_rounds - 1 && warp == W - 1 && a.g_h0 && ch_ok && sg.lo == 0) {
                    a.g_h0[((size_t)b * 4 + 0) * d + ch] = nc;
                    a.g_h0[((size_t)b * 4 + 1) * d + ch] = nn;
                    a.g_h0[((size_t)b * 4 + 2) * d + ch] = nm;
                    a.g_h0[((size_t)b * 4 + 3) * d + ch] = nh;
                }
            };
            if (t_hi < sg.hi)
                round_body(std::true_type{});
            else
                round_body(std::false_type{});
        }
#pragma unroll
        for (int p = 0; p < 4; ++p) s_gp[(warp * 4 + p) * kLanes + lane] = gr[p];
    }
    if (timed_out) atomicExch(a.chain.status, (int)kErrChainTimeout);
    if (threadIdx.x == 0 && timed_out) drain_ring(full, NSTAGE, n_rounds, kDrainLimit);
    __syncthreads();
    if (warp == 0 && ch_ok) {
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            float sum = 0.f;
#pragma unroll
            for (int w2 = 0; w2 < W; ++w2) sum += s_gp[(w2 * 4 + p) * kLanes + lane];
            a.gp_partial[(((size_t)sg.seg * a.B + b) * 4 + p) * d + ch] = sum;
        }
    }
    if (BIAS) {  // per-gate sums of g_wx (bias gradient), same fixed-order reduction
        __syncthreads();
#pragma unroll
        for (int p = 0; p < 4; ++p) s_gp[(warp * 4 + p) * kLanes + lane] = gb[p];
        __syncthreads();
        if (warp == 0 && ch_ok) {
#pragma unroll
            for (int p = 0; p < 4; ++p) {
                float sum = 0.f;
#pragma unroll
                for (int w2 = 0; w2 < W; ++w2) sum += s_gp[(w2 * 4 + p) * kLanes + lane];
                a.gb_partial[(((size_t)sg.seg * a.B + b) * 4 + p) * d + ch] = sum;
            }
        }
    }
}

// ------------------------------------------------------------------ Picard (frozen gates)
template <typename TIO, int L, int W, int NSTAGE>
struct PipePicardSmem {
    static constexpr int LT = W * L;
    static constexpr int WX_BYTES = LT * 4 * kLanes * (int)sizeof(TIO);
    static constexpr int H_BYTES = ((LT + 1) * kLanes * 4 + 127) / 128 * 128;
    static constexpr int STAGE = WX_BYTES + H_BYTES;
    static constexpr int SLOT_OFF = NSTAGE * STAGE;
    static constexpr int SLOT_BYTES = W * 3 * kLanes * 4;
    static constexpr int BAR_OFF = (SLOT_OFF + SLOT_BYTES + 7) / 8 * 8;
    static constexpr int TOTAL = BAR_OFF + (2 * NSTAGE + W) * 8 + 64;
};

// The baton is the true state, passed in two parts: m as soon as the max-plus recurrence of the
// warp's steps is done (named barrier), (c, n) after the multiply-add recurrences (mbarrier), so
// that the next warp's m recurrence overlaps this warp's exponentials.
// The baton is the true state (c, n, m).  Inside a warp's L steps the max-plus recurrence of m
// runs first (two dependent ops per step), then the L exponentials are independent of each
// other, then the two multiply-add recurrences of n and c run.
template <typename TIO, int L, int W, int NSTAGE, bool HAS_H>
__global__ void __launch_bounds__((W + 1) * 32, 2)
slstm_picard_pipe_kernel(const __grid_constant__ CUtensorMap tm_wx,
                         const __grid_constant__ CUtensorMap tm_h, SlstmPicardArgs a) {
    using S = PipePicardSmem<TIO, L, W, NSTAGE>;
    constexpr int LT = S::LT;
    extern __shared__ __align__(128) unsigned char smem[];
    float* s_slot = reinterpret_cast<float*>(smem + S::SLOT_OFF);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + S::BAR_OFF);
    uint64_t* empty = full + NSTAGE;
    uint64_t* cnbar = empty + NSTAGE;  // [W]: (c, n) entering warp w is ready

    const int d = a.d;
    const int ncb = (d + kLanes - 1) / kLanes;
    const int chain = blockIdx.x;
    const int b = chain / ncb, cb = chain % ncb;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ch = cb * kLanes + lane;
    const bool ch_ok = ch < d;
    const int chl = ch_ok ? ch : d - 1;
    const SegRange sg = seg_range(a.T, a.n_seg, a.seg_len);
    const int n_rounds = (sg.hi - sg.lo + LT - 1) / LT;
    const int row0 = b * a.T + sg.lo;

    if (threadIdx.x == 0) {
        tma_prefetch_desc(&tm_wx);
        if (HAS_H) tma_prefetch_desc(&tm_h);
        for (int s = 0; s < NSTAGE; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], W);
        }
        for (int w2 = 0; w2 < W; ++w2) mbar_init(&cnbar[w2], 1);
        mbar_fence_init();
    }
    if (warp == 0) {
#pragma unroll
        for (int q = 0; q < 3; ++q)
            s_slot[q * kLanes + lane] =
                a.carry_in ? __ldg(a.carry_in + ((size_t)sg.seg * a.B + b) * a.carry_stride + (size_t)q * d + chl)
                           : 0.f;
    }
    __syncthreads();
    bool timed_out = false;

    if (warp == W) {
        if (lane == 0) {
            for (int r = 0; r < n_rounds; ++r) {
                const int s = r % NSTAGE;
                if (r >= NSTAGE && !mbar_wait_bounded_sleepy(&empty[s], ((r / NSTAGE) - 1) & 1, timed_out ? kWaitLimitAfterTimeout : kPipeWaitLimit))
                    timed_out = true;
                unsigned char* base = smem + s * S::STAGE;
                mbar_expect_tx(&full[s], S::WX_BYTES + (HAS_H ? (LT + 1) * kLanes * 4 : 0));
                tma_load_3d(base, &tm_wx, &full[s], cb * kLanes, 0, row0 + r * LT);
                if (HAS_H) tma_load_3d(base + S::WX_BYTES, &tm_h, &full[s], cb * kLanes, 0, row0 + r * LT - 1);
            }
            if (timed_out) drain_ring(full, NSTAGE, n_rounds, kDrainLimit);
        }
    } else {
        float r4[4] = {0.f, 0.f, 0.f, 0.f};
        if (HAS_H) {
#pragma unroll
            for (int q = 0; q < 4; ++q) r4[q] = __ldg(a.r + (size_t)q * d + chl);
        }
        const int next = (warp + 1) % W;
        float* slot_in = s_slot + warp * 3 * kLanes + lane;
        float* slot_out = s_slot + next * 3 * kLanes + lane;

        for (int r = 0; r < n_rounds; ++r) {
            const int s = r % NSTAGE;
            if (!mbar_wait_bounded_sleepy(&full[s], (r / NSTAGE) & 1, timed_out ? kWaitLimitAfterTimeout : kPipeWaitLimit)) timed_out = true;
            const TIO* t_wx = reinterpret_cast<const TIO*>(smem + s * S::STAGE);
            const float* t_h = reinterpret_cast<const float*>(smem + s * S::STAGE + S::WX_BYTES);
            const int t0 = sg.lo + r * LT + warp * L;

            // Rounds that lie fully inside the sequence take a variant without range checks.
            auto round_body = [&](auto full_c) {
                constexpr bool FULL = decltype(full_c)::value;
                float zi[L], zf[L], zz[L], og[L];
    #pragma unroll
                for (int i = 0; i < L; ++i) {
                    float hp = 0.f;
                    if (HAS_H) {
                        hp = (i == 0 && t0 == 0) ? (a.h_halo ? __ldg(a.h_halo + (size_t)b * a.halo_stride + chl) : 0.f)
                                           : t_h[(warp * L + i) * kLanes + lane];
                    }
                    const int row = warp * L + i;
                    zi[i] = fmaf(r4[0], hp, (float)t_wx[(row * 4 + 0) * kLanes + lane]);
                    zf[i] = fmaf(r4[1], hp, (float)t_wx[(row * 4 + 1) * kLanes + lane]);
                    zz[i] = fmaf(r4[2], hp, (float)t_wx[(row * 4 + 2) * kLanes + lane]);
                    og[i] = fmaf(r4[3], hp, (float)t_wx[(row * 4 + 3) * kLanes + lane]);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[s]);
    #pragma unroll
                for (int i = 0; i < L; ++i) {
                    zz[i] = tanh_f(zz[i]);
                    og[i] = 1.0f + ex2_approx(-1.4426950216293335f * og[i]);  // 1 / sigmoid
                }

                if (!(r == 0 && warp == 0)) named_sync(1 + warp, 64);
                float m = slot_in[2 * kLanes];
                float dlt[L], ms[L];
    #pragma unroll
                for (int i = 0; i < L; ++i) {
                    if (FULL || t0 + i < sg.hi) {
                        const float left = zf[i] + m;
                        dlt[i] = left - zi[i];
                        m = fmaxf(left, zi[i]);
                    } else {
                        dlt[i] = 0.f;
                    }
                    ms[i] = m;
                }
                slot_out[2 * kLanes] = m;
                if (!(r == n_rounds - 1 && warp == W - 1)) named_arrive(1 + next, 64);
                float e[L];
    #pragma unroll
                for (int i = 0; i < L; ++i) e[i] = exp_f(-fabsf(dlt[i]));
                // (c, n) from the previous warp: its r-th hand-over for warps > 0, the last warp's
                // (r-1)-th for warp 0
                if (!(r == 0 && warp == 0)) {
                    const uint32_t par = (warp == 0 ? r - 1 : r) & 1;
                    if (!mbar_wait_bounded_sleepy(&cnbar[warp], par, timed_out ? kWaitLimitAfterTimeout : kPipeWaitLimit)) timed_out = true;
                }
                float c = slot_in[0], n = slot_in[kLanes];
                float cs[L], ns[L];
    #pragma unroll
                for (int i = 0; i < L; ++i) {
                    if (FULL || t0 + i < sg.hi) {
                        const bool lw = dlt[i] >= 0.f;
                        const float ft = lw ? 1.f : e[i], it = lw ? e[i] : 1.f;
                        n = fmaf(ft, n, it);
                        c = fmaf(ft, c, it * zz[i]);
                    }
                    cs[i] = c;
                    ns[i] = n;
                }
                slot_out[0] = c;
                slot_out[kLanes] = n;
                __syncwarp();
                if (lane == 0 && !(r == n_rounds - 1 && warp == W - 1)) mbar_arrive(&cnbar[next]);

                const size_t o_base = ((size_t)b * a.T + t0) * d;

    #pragma unroll
                for (int i = 0; i < L; ++i) {
                    const int t = t0 + i;
                    if ((FULL || t < sg.hi) && ch_ok) {
                        const float h = cs[i] * rcp_f(og[i] * (ns[i] + a.eps));
                        if (a.state_out) {
                            float* o = a.state_out + o_base * 4 + ch + (size_t)i * 4 * d;
                            o[0] = cs[i];
                            o[d] = ns[i];
                            o[2 * (size_t)d] = ms[i];
                            o[3 * (size_t)d] = h;
                        } else {
                            a.h_out[o_base + ch + (size_t)i * d] = h;
                        }
                    }
                }
                if (r == n_rounds - 1 && warp == W - 1 && a.tail_out && ch_ok && sg.hi == a.T) {
                    a.tail_out[((size_t)b * 3 + 0) * d + ch] = c;
                    a.tail_out[((size_t)b * 3 + 1) * d + ch] = n;
                    a.tail_out[((size_t)b * 3 + 2) * d + ch] = m;
                }
            };
            if (t0 + L <= sg.hi)
                round_body(std::true_type{});
            else
                round_body(std::false_type{});
        }
    }
    if (timed_out) atomicExch(a.chain.status, (int)kErrChainTimeout);
}

// ------------------------------------------------------------------ launchers
constexpr int kQL = 4, kQW = 8;

template <typename TIO, int NSTAGE>
static cudaError_t launch_newton_pipe_t(const SlstmNewtonArgs& a, bool last, cudaStream_t s) {
    using S = PipeNewtonSmem<TIO, kQL, kQW, NSTAGE>;
    CUtensorMap tm_wx, tm_st;
    const uint64_t rows = (uint64_t)a.B * a.T;
    if (!make_tile_map(&tm_wx, a.wx, sizeof(TIO), rows, 4, a.d, S::LT) ||
        !make_tile_map(&tm_st, a.sin, 4, rows, 4, a.d, S::LT + 1))
        return cudaErrorNotSupported;
    const dim3 grid(a.B * ((a.d + kLanes - 1) / kLanes), a.n_seg > 1 ? a.n_seg : 1);
    if (last) {
        auto k = slstm_newton_pipe_kernel<TIO, kQL, kQW, NSTAGE, true>;
        cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
        k<<<grid, (kQW + 1) * 32, S::TOTAL, s>>>(tm_wx, tm_st, a);
    } else {
        auto k = slstm_newton_pipe_kernel<TIO, kQL, kQW, NSTAGE, false>;
        cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
        k<<<grid, (kQW + 1) * 32, S::TOTAL, s>>>(tm_wx, tm_st, a);
    }
    return cudaGetLastError();
}

template <typename TIO, int NSTAGE>
static cudaError_t launch_bwd_pipe_t(const SlstmBwdArgs& a, cudaStream_t s) {
    using S = PipeBwdSmem<TIO, kQL, kQW, NSTAGE, false>;
    using SH = PipeBwdSmem<TIO, kQL, kQW, NSTAGE, true>;
    CUtensorMap tm_wx, tm_st, tm_g;
    const uint64_t rows = (uint64_t)a.B * a.T;
    // the compact cotangent is built for the hidden slot (3) only; other slots: not supported here
    if (a.g_slot >= 0 && a.g_slot != 3) return cudaErrorNotSupported;
    const bool hid = a.g_slot == 3;
    if (!make_tile_map(&tm_wx, a.wx, sizeof(TIO), rows, 4, a.d, S::LT) ||
        !make_tile_map(&tm_st, a.states, sizeof(TIO), rows, 4, a.d, S::LT + 1) ||
        !make_tile_map(&tm_g, a.grad_states, sizeof(TIO), rows, hid ? 1 : 4, a.d, S::LT))
        return cudaErrorNotSupported;
    const dim3 grid(a.B * ((a.d + kLanes - 1) / kLanes), a.n_seg > 1 ? a.n_seg : 1);
    auto go = [&](auto k, int smem) {
        cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        k<<<grid, kQW * 32, smem, s>>>(tm_wx, tm_st, tm_g, a);
    };
    const bool bias = a.gb_partial != nullptr;
    if (hid && bias)
        go(slstm_bwd_pipe_kernel<TIO, kQL, kQW, NSTAGE, 3, true>, SH::TOTAL);
    else if (hid)
        go(slstm_bwd_pipe_kernel<TIO, kQL, kQW, NSTAGE, 3, false>, SH::TOTAL);
    else if (bias)
        go(slstm_bwd_pipe_kernel<TIO, kQL, kQW, NSTAGE, -1, true>, S::TOTAL);
    else
        go(slstm_bwd_pipe_kernel<TIO, kQL, kQW, NSTAGE, -1, false>, S::TOTAL);
    return cudaGetLastError();
}

// gp_partial receives one row per batch row: (B, 4, d)
cudaError_t launch_slstm_bwd_pipe(int dtype, const SlstmBwdArgs& a, cudaStream_t s) {
    return dtype == kF32 ? launch_bwd_pipe_t<float, 2>(a, s) : launch_bwd_pipe_t<__nv_bfloat16, 3>(a, s);
}

template <typename TIO, int NSTAGE>
static cudaError_t launch_picard_pipe_t(const SlstmPicardArgs& a, cudaStream_t s) {
    constexpr int L = 8, W = 8;
    using S = PipePicardSmem<TIO, L, W, NSTAGE>;
    CUtensorMap tm_wx, tm_h;
    const uint64_t rows = (uint64_t)a.B * a.T;
    if (!make_tile_map(&tm_wx, a.wx, sizeof(TIO), rows, 4, a.d, S::LT)) return cudaErrorNotSupported;
    const dim3 grid(a.B * ((a.d + kLanes - 1) / kLanes), a.n_seg > 1 ? a.n_seg : 1);
    if (a.h_prev) {
        if (!make_tile_map(&tm_h, a.h_prev, 4, rows, 1, a.d, S::LT + 1)) return cudaErrorNotSupported;
        auto k = slstm_picard_pipe_kernel<TIO, L, W, NSTAGE, true>;
        cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
        k<<<grid, (W + 1) * 32, S::TOTAL, s>>>(tm_wx, tm_h, a);
    } else {
        auto k = slstm_picard_pipe_kernel<TIO, L, W, NSTAGE, false>;
        cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
        k<<<grid, (W + 1) * 32, S::TOTAL, s>>>(tm_wx, tm_wx, a);
    }
    return cudaGetLastError();
}

cudaError_t launch_slstm_picard_pipe(int dtype, const SlstmPicardArgs& a, cudaStream_t s) {
    return dtype == kF32 ? launch_picard_pipe_t<float, 2>(a, s) : launch_picard_pipe_t<__nv_bfloat16, 3>(a, s);
}

cudaError_t launch_slstm_newton_pipe(int dtype, const SlstmNewtonArgs& a, bool last, cudaStream_t s) {
    return dtype == kF32 ? launch_newton_pipe_t<float, 2>(a, last, s)
                         : launch_newton_pipe_t<__nv_bfloat16, 3>(a, last, s);
}

}  // namespace prb
