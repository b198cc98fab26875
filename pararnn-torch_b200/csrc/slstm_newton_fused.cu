// ParaSLSTM mix='diag': all K Newton iterations (and the residual of the returned trajectory) in
// ONE sweep over the sequence.
//
// Iteration k+1 at step t linearises around the iterate k at steps t-1 and t, which exist as soon
// as the scan of iteration k has passed step t.  So, as in slstm_picard_fused.cu, the iterations
// follow each other through the sequence as a wavefront over the warps of a CTA: one CTA owns one
// chain (batch row x 32 channels) and walks it in rounds of W*L steps fed by a TMA ring; a warp
// loads the gate pre-activations and the warm-start state of its L steps once per round, keeps
// the state in registers and, for k = 0..K-1, linearises, waits for iteration k's carry (delta at
// the step before its sub-tile) from the previous warp, runs its L steps of
// delta_t = J_t delta_{t-1} + F_t, hands the carry on and updates its state in place; the state
// preceding the sub-tile is updated with the incoming carry itself.  Only the last iterate is
// written, in the I/O dtype, after its residual has been evaluated on the fp32 values.
//
// Same per-step math as slstm_newton_pipe_kernel (slstm_cell.cuh; reference behaviour restated in
// slstm_kernels.cu: kernels/newton_slstm.py:2696-2939, cells/para_slstm.py:347-446).
#include "common.cuh"
#include "kernels.h"
#include "slstm_cell.cuh"
#include "tma.cuh"

#include <type_traits>

namespace prb {

namespace {

constexpr uint32_t kNfWaitLimit = 1u << 24;
constexpr int kNfMaxIters = 4;

__device__ __forceinline__ void nf_mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

template <typename TIO, int L, int W, int NSTAGE>
struct NewtonFusedSmem {
    static constexpr int LT = W * L;
    static constexpr int WX_BYTES = (LT * 4 * kLanes * (int)sizeof(TIO) + 127) / 128 * 128;
    static constexpr int WX_TX = LT * 4 * kLanes * (int)sizeof(TIO);
    static constexpr int ST_TX = (LT + 1) * 4 * kLanes * 4;
    static constexpr int ST_BYTES = (ST_TX + 127) / 128 * 128;
    static constexpr int STAGE = WX_BYTES + ST_BYTES;
    static constexpr int SLOT_OFF = NSTAGE * STAGE;
    static constexpr int SLOT_BYTES = kNfMaxIters * W * 4 * kLanes * 4;  // [iter][warp][4][32]
    static constexpr int BAR_OFF = SLOT_OFF + SLOT_BYTES;
    static constexpr int N_BARS = 2 * NSTAGE + kNfMaxIters * W;
    static constexpr int RED_OFF = BAR_OFF + N_BARS * 8;
    static constexpr int TOTAL = RED_OFF + (W + 1) * 4 + 64;
};

template <typename TIO, int L, int W, int NSTAGE>
__global__ void __launch_bounds__(W * 32, W > 8 ? 1 : 2)
slstm_newton_fused_kernel(const __grid_constant__ CUtensorMap tm_wx, const __grid_constant__ CUtensorMap tm_st,
                          SlstmNewtonArgs a, int n_iters) {
    using S = NewtonFusedSmem<TIO, L, W, NSTAGE>;
    constexpr int LT = S::LT;
    extern __shared__ __align__(128) unsigned char smem[];
    float* s_slot = reinterpret_cast<float*>(smem + S::SLOT_OFF);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + S::BAR_OFF);
    uint64_t* empty = full + NSTAGE;
    uint64_t* baton = empty + NSTAGE;  // [iter][warp]: the carry entering the warp is ready
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
        tma_prefetch_desc(&tm_st);
        for (int s = 0; s < NSTAGE; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], W);
        }
        for (int k = 0; k < kNfMaxIters * W; ++k) mbar_init(&baton[k], 1);
        mbar_fence_init();
    }
    if (warp == 0) {
        // delta entering step 0 is zero in every iteration
        for (int k = 0; k < n_iters; ++k)
#pragma unroll
            for (int q = 0; q < 4; ++q) s_slot[((k * W + 0) * 4 + q) * kLanes + lane] = 0.f;
    }
    __syncthreads();

    unsigned rm[kNfMaxIters] = {0u, 0u, 0u, 0u};
    unsigned fmax = 0u;
    bool timed_out = false;

    // No dedicated producer warp (it would cost an eighth of the register file): lane 0 of warp 0
    // keeps the TMA ring full.  At the start of round r it refills the stage of round r-1, which
    // every warp has copied to registers long before (the warps are at most half a round apart).
    auto issue = [&](int r) {
        const int s = r % NSTAGE;
        unsigned char* base = smem + s * S::STAGE;
        mbar_expect_tx(&full[s], S::WX_TX + S::ST_TX);
        tma_load_3d(base, &tm_wx, &full[s], cb * kLanes, 0, row0 + r * LT);
        tma_load_3d(base + S::WX_BYTES, &tm_st, &full[s], cb * kLanes, 0, row0 + r * LT - 1);
    };
    if (threadIdx.x == 0)
        for (int r = 0; r < NSTAGE && r < n_rounds; ++r) issue(r);
    {
        float r4[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) r4[q] = __ldg(a.r + (size_t)q * d + chl);
        const bool want_final = a.final_bits != nullptr;
        const int next = (warp + 1) % W;

        for (int r = 0; r < n_rounds; ++r) {
            const int s = r % NSTAGE;
            if (threadIdx.x == 0 && r >= 1 && r - 1 + NSTAGE < n_rounds) {
                if (!mbar_wait_bounded(&empty[(r - 1) % NSTAGE], ((r - 1) / NSTAGE) & 1, timed_out ? kWaitLimitAfterTimeout : kNfWaitLimit))
                    timed_out = true;
                issue(r - 1 + NSTAGE);
            }
            __syncwarp();
            if (!mbar_wait_bounded(&full[s], (r / NSTAGE) & 1, timed_out ? kWaitLimitAfterTimeout : kNfWaitLimit)) timed_out = true;
            const TIO* t_wx = reinterpret_cast<const TIO*>(smem + s * S::STAGE);
            const float* t_st = reinterpret_cast<const float*>(smem + s * S::STAGE + S::WX_BYTES);
            const int t0 = r * LT + warp * L;
            const bool first = (r == 0 && warp == 0);
            const bool last = (r == n_rounds - 1 && warp == W - 1);
            const uint32_t par = (warp == 0 ? r - 1 : r) & 1;

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
            __syncwarp();
            if (lane == 0) nf_mbar_arrive(&empty[s]);

            auto round_body = [&](auto full_c) {
                constexpr bool FULL = decltype(full_c)::value;
                for (int k = 0; k < n_iters; ++k) {
                    float* slot_in = s_slot + ((k * W + warp) * 4) * kLanes + lane;
                    float* slot_out = s_slot + ((k * W + next) * 4) * kLanes + lane;
                    // ---- carry-independent part
                    SlstmLin lin[L];
                    float F[L][4];
                    unsigned rmax = 0u;
#pragma unroll
                    for (int i = 0; i < L; ++i) {
                        slstm_linearize(st[i], w[i], r4, a.eps, lin[i]);
                        const bool ok = FULL || t0 + i < a.T;
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
#pragma unroll
                    for (int kk = 0; kk < kNfMaxIters; ++kk) rm[kk] = (kk == k) ? max(rm[kk], rmax) : rm[kk];

                    // ---- the baton of iteration k
                    if (!first && !mbar_wait_bounded(&baton[k * W + warp], par, timed_out ? kWaitLimitAfterTimeout : kNfWaitLimit)) timed_out = true;
                    float xc = slot_in[0], xn = slot_in[kLanes], xm = slot_in[2 * kLanes], xh = slot_in[3 * kLanes];
                    // the state preceding the sub-tile moves by the incoming carry
                    st[0][0] = fmaf(a.omega, xc, st[0][0]);
                    st[0][1] = fmaf(a.omega, xn, st[0][1]);
                    st[0][2] = fmaf(a.omega, xm, st[0][2]);
                    st[0][3] = fmaf(a.omega, xh, st[0][3]);
#pragma unroll
                    for (int i = 0; i < L; ++i) {
                        slstm_apply(lin[i], F[i][0], F[i][1], F[i][2], F[i][3], xc, xn, xm, xh);
                        st[i + 1][0] = fmaf(a.omega, xc, st[i + 1][0]);
                        st[i + 1][1] = fmaf(a.omega, xn, st[i + 1][1]);
                        st[i + 1][2] = fmaf(a.omega, xm, st[i + 1][2]);
                        st[i + 1][3] = fmaf(a.omega, xh, st[i + 1][3]);
                    }
                    slot_out[0] = xc;
                    slot_out[kLanes] = xn;
                    slot_out[2 * kLanes] = xm;
                    slot_out[3 * kLanes] = xh;
                    __syncwarp();
                    if (lane == 0 && !last) nf_mbar_arrive(&baton[k * W + next]);
                    if (last && k == n_iters - 1 && a.tail_out && ch_ok) {
                        a.tail_out[((size_t)b * 4 + 0) * d + ch] = xc;
                        a.tail_out[((size_t)b * 4 + 1) * d + ch] = xn;
                        a.tail_out[((size_t)b * 4 + 2) * d + ch] = xm;
                        a.tail_out[((size_t)b * 4 + 3) * d + ch] = xh;
                    }
                }
                // ---- the last iterate: residual on the fp32 values, then the I/O-dtype store
                if (ch_ok) {
                    TIO* o = reinterpret_cast<TIO*>(a.sout) + ((size_t)b * a.T + t0) * 4 * d + ch;
#pragma unroll
                    for (int i = 0; i < L; ++i) {
                        if (FULL || t0 + i < a.T) {
                            if (want_final) {
                                float pred[4];
                                slstm_predict(st[i], w[i], r4, a.eps, pred);
                                fmax = max(fmax, max(max(absbits(pred[0] - st[i + 1][0]), absbits(pred[1] - st[i + 1][1])),
                                                     max(absbits(pred[2] - st[i + 1][2]), absbits(pred[3] - st[i + 1][3]))));
                            }
                            TIO* oi = o + (size_t)i * 4 * d;
                            st_f(oi, st[i + 1][0]);
                            st_f(oi + d, st[i + 1][1]);
                            st_f(oi + 2 * (size_t)d, st[i + 1][2]);
                            st_f(oi + 3 * (size_t)d, st[i + 1][3]);
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
    if (threadIdx.x == 0 && timed_out) drain_ring(full, NSTAGE, n_rounds, kDrainLimit);
    for (int k = 0; k < n_iters; ++k) {
        __syncthreads();
        unsigned v = 0u;
#pragma unroll
        for (int kk = 0; kk < kNfMaxIters; ++kk) v = (kk == k) ? rm[kk] : v;
        block_residual_max(v, a.resid_bits + k, s_red);
    }
    if (a.final_bits != nullptr) {
        __syncthreads();
        block_residual_max(fmax, a.final_bits, s_red);
    }
}

template <typename TIO, int NSTAGE, int L, int W>
cudaError_t launch_lw(const SlstmNewtonArgs& a, int n_iters, cudaStream_t s) {
    using S = NewtonFusedSmem<TIO, L, W, NSTAGE>;
    CUtensorMap tm_wx, tm_st;
    const uint64_t rows = (uint64_t)a.B * a.T;
    if (!make_tile_map(&tm_wx, a.wx, sizeof(TIO), rows, 4, a.d, S::LT) ||
        !make_tile_map(&tm_st, a.sin, 4, rows, 4, a.d, S::LT + 1))
        return cudaErrorNotSupported;
    const int grid = a.B * ((a.d + kLanes - 1) / kLanes);
    auto k = slstm_newton_fused_kernel<TIO, L, W, NSTAGE>;
    cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
    k<<<grid, W * 32, S::TOTAL, s>>>(tm_wx, tm_st, a, n_iters);
    return cudaGetLastError();
}

// 8 warps x 4 steps, two CTAs per SM (128 registers per thread) when there are more chains than
// SMs; with fewer chains a CTA has an SM to itself and a single chain's walk is bound by latency,
// so 16 warps put twice as many warps on a round of twice the steps.
template <typename TIO, int NSTAGE>
cudaError_t launch_t(const SlstmNewtonArgs& a, int n_iters, cudaStream_t s) {
    const int chains = a.B * ((a.d + kLanes - 1) / kLanes);
    return chains > sm_count() ? launch_lw<TIO, NSTAGE, 4, 8>(a, n_iters, s) : launch_lw<TIO, NSTAGE, 4, 16>(a, n_iters, s);
}

}  // namespace

int slstm_newton_fused_max_iters() { return kNfMaxIters; }

// K = n_iters Newton iterations in one launch: reads a.sin (fp32 warm start), writes a.sout in the
// I/O dtype, max|F(H^k)| of iterate k to a.resid_bits[k], the residual of the result to
// a.final_bits.  a.carry_in must be null (whole sequences only).
cudaError_t launch_slstm_newton_fused(int dtype, const SlstmNewtonArgs& a, int n_iters, cudaStream_t s) {
    if (n_iters < 1 || n_iters > kNfMaxIters || a.carry_in) return cudaErrorNotSupported;
    return dtype == kF32 ? launch_t<float, 2>(a, n_iters, s) : launch_t<__nv_bfloat16, 3>(a, n_iters, s);
}

}  // namespace prb
