// ParaSLSTM mix='diag': all frozen-gate Picard passes of the warm start in ONE sweep.
//
// Pass p at step t needs the hidden state of pass p-1 at step t-1 only, so the passes can follow
// each other through the sequence a few steps apart instead of one full sweep apart.  One CTA
// owns one chain (batch row x 32 channels) and walks it in rounds of W*L steps fed by a TMA ring,
// exactly like the per-pass kernel of slstm_pipe.cu.  A warp reads the gate pre-activations of
// its L steps from shared memory ONCE per round, keeps them in registers and runs pass 0, 1, ...
// on them back to back; the hidden states a pass produces stay in registers for the next pass.
// Across warps every pass has its own baton (mbarriers + a slot per warp): the state (c, n, m)
// at the end of the previous warp's steps and, for the next pass, that warp's last hidden value.
// The passes therefore move through the warps as a wavefront: while warp w runs pass p on its
// steps, warp w+1 runs pass p-1 on the following ones.  Nothing but the final state is written:
// HBM traffic is `wx` read once plus the fp32 state written once, instead of one read of `wx` and
// one round trip of the hidden trajectory per pass.
//
// Same per-step math, in the same order, as slstm_picard_pipe_kernel (reference behaviour
// restated there and in slstm_kernels.cu: solvers/slstm_picard.py:51-181).
#include "common.cuh"
#include "kernels.h"
#include "slstm_cell.cuh"
#include "tma.cuh"

#include <type_traits>

namespace prb {

namespace {

constexpr uint32_t kFusedWaitLimit = 1u << 24;
constexpr int kFusedMaxPass = 6;

// Gate pre-activations of one step as the warp keeps them between passes: fp32 inputs as they
// are, bf16 inputs two to a register (the upper half of an fp32 word IS the bf16 value).
template <typename TIO>
struct GateRegs;
template <>
struct GateRegs<float> {
    float v[4];
    __device__ __forceinline__ void load(const float* t, int stride) {
#pragma unroll
        for (int q = 0; q < 4; ++q) v[q] = t[q * stride];
    }
    __device__ __forceinline__ float get(int q) const { return v[q]; }
    __device__ __forceinline__ void pin() {}
};
template <>
struct GateRegs<__nv_bfloat16> {
    uint32_t p[2];
    __device__ __forceinline__ void load(const __nv_bfloat16* t, int stride) {
        const unsigned short* u = reinterpret_cast<const unsigned short*>(t);
        p[0] = (uint32_t)u[0] | ((uint32_t)u[stride] << 16);
        p[1] = (uint32_t)u[2 * stride] | ((uint32_t)u[3 * stride] << 16);
    }
    __device__ __forceinline__ float get(int q) const {
        const uint32_t w = p[q >> 1];
        return __uint_as_float((q & 1) ? (w & 0xffff0000u) : (w << 16));
    }
    // keeps the compiler from unpacking once outside the loop over the passes, which would hold
    // the four fp32 values in registers after all
    __device__ __forceinline__ void pin() {
        asm volatile("" : "+r"(p[0]), "+r"(p[1]));
    }
};

__device__ __forceinline__ void fp_mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

template <typename TIO, int L, int W, int NSTAGE>
struct FusedPicardSmem {
    static constexpr int LT = W * L;
    static constexpr int STAGE = LT * 4 * kLanes * (int)sizeof(TIO);
    static constexpr int SLOT_OFF = NSTAGE * STAGE;
    static constexpr int SLOT_BYTES = kFusedMaxPass * W * 4 * kLanes * 4;  // [pass][warp][c,n,m,h][32]
    static constexpr int BAR_OFF = SLOT_OFF + SLOT_BYTES;
    static constexpr int N_BARS = 2 * NSTAGE + 2 * kFusedMaxPass * W;
    static constexpr int TOTAL = BAR_OFF + N_BARS * 8 + 64;
};

template <typename TIO, int L, int W, int NSTAGE>
__global__ void __launch_bounds__(W * 32, W > 8 ? 1 : 2)
slstm_picard_fused_kernel(const __grid_constant__ CUtensorMap tm_wx, SlstmPicardArgs a, int n_pass) {
    using S = FusedPicardSmem<TIO, L, W, NSTAGE>;
    constexpr int LT = S::LT;
    extern __shared__ __align__(128) unsigned char smem[];
    float* s_slot = reinterpret_cast<float*>(smem + S::SLOT_OFF);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + S::BAR_OFF);
    uint64_t* empty = full + NSTAGE;
    uint64_t* mbar_m = empty + NSTAGE;               // [pass][warp]: m entering the warp is ready
    uint64_t* mbar_cn = mbar_m + kFusedMaxPass * W;  // [pass][warp]: (c, n, h_last) are ready

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
        for (int k = 0; k < 2 * kFusedMaxPass * W; ++k) mbar_init(&mbar_m[k], 1);
        mbar_fence_init();
    }
    const float h_halo = a.h_halo ? __ldg(a.h_halo + (size_t)b * a.halo_stride + chl) : 0.f;
    if (warp == 0) {
        // every pass starts from the same state (c, n, m) preceding step 0
        for (int g = 0; g < n_pass; ++g) {
#pragma unroll
            for (int q = 0; q < 3; ++q)
                s_slot[((g * W + 0) * 4 + q) * kLanes + lane] =
                    a.carry_in ? __ldg(a.carry_in + (size_t)b * a.carry_stride + (size_t)q * d + chl) : 0.f;
            s_slot[((g * W + 0) * 4 + 3) * kLanes + lane] = h_halo;
        }
    }
    __syncthreads();
    bool timed_out = false;

    // No dedicated producer warp (it would cost an eighth of the register file): lane 0 of warp 0
    // keeps the TMA ring full.  At the start of round r it refills the stage of round r-1, which
    // every warp has copied to registers long before (the warps are at most half a round apart).
    auto issue = [&](int r) {
        const int s = r % NSTAGE;
        mbar_expect_tx(&full[s], S::STAGE);
        tma_load_3d(smem + s * S::STAGE, &tm_wx, &full[s], cb * kLanes, 0, row0 + r * LT);
    };
    if (threadIdx.x == 0)
        for (int r = 0; r < NSTAGE && r < n_rounds; ++r) issue(r);
    {
        float r4[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) r4[q] = __ldg(a.r + (size_t)q * d + chl);
        const int next = (warp + 1) % W;

        for (int r = 0; r < n_rounds; ++r) {
            const int s = r % NSTAGE;
            if (threadIdx.x == 0 && r >= 1 && r - 1 + NSTAGE < n_rounds) {
                if (!mbar_wait_bounded(&empty[(r - 1) % NSTAGE], ((r - 1) / NSTAGE) & 1, timed_out ? kWaitLimitAfterTimeout : kFusedWaitLimit))
                    timed_out = true;
                issue(r - 1 + NSTAGE);
            }
            __syncwarp();
            if (!mbar_wait_bounded(&full[s], (r / NSTAGE) & 1, timed_out ? kWaitLimitAfterTimeout : kFusedWaitLimit)) timed_out = true;
            const TIO* t_wx = reinterpret_cast<const TIO*>(smem + s * S::STAGE);
            const int t0 = r * LT + warp * L;
            const bool first = (r == 0 && warp == 0);
            const bool last = (r == n_rounds - 1 && warp == W - 1);
            const uint32_t par = (warp == 0 ? r - 1 : r) & 1;

            // gate pre-activations of this warp's steps: read once, used by every pass
            GateRegs<TIO> wxr[L];
#pragma unroll
            for (int i = 0; i < L; ++i) wxr[i].load(t_wx + ((warp * L + i) * 4) * kLanes + lane, kLanes);
            __syncwarp();
            if (lane == 0) fp_mbar_arrive(&empty[s]);

            auto round_body = [&](auto full_c) {
                constexpr bool FULL = decltype(full_c)::value;
                float hp[L];  // hidden state of the previous pass at step t-1, for each of the L steps
#pragma unroll
                for (int i = 0; i < L; ++i) hp[i] = 0.f;
                for (int g = 0; g < n_pass; ++g) {
                    float* slot_in = s_slot + ((g * W + warp) * 4) * kLanes + lane;
                    float* slot_out = s_slot + ((g * W + next) * 4) * kLanes + lane;
                    float zi[L], zf[L], zz[L], og[L];
                    // two steps per packed instruction
#pragma unroll
                    for (int i = 0; i < L; i += 2) {
                        wxr[i].pin();
                        wxr[i + 1].pin();
                        const float2 hp2 = make_float2(hp[i], hp[i + 1]);
                        const float2 vi = __ffma2_rn(splat2(r4[0]), hp2, make_float2(wxr[i].get(0), wxr[i + 1].get(0)));
                        const float2 vf = __ffma2_rn(splat2(r4[1]), hp2, make_float2(wxr[i].get(1), wxr[i + 1].get(1)));
                        const float2 vz = tanh_f2(
                            __ffma2_rn(splat2(r4[2]), hp2, make_float2(wxr[i].get(2), wxr[i + 1].get(2))));
                        const float2 vo = __ffma2_rn(splat2(r4[3]), hp2, make_float2(wxr[i].get(3), wxr[i + 1].get(3)));
                        const float2 go = __fadd2_rn(splat2(1.0f), ex2_2(__fmul2_rn(splat2(-1.4426950216293335f), vo)));
                        zi[i] = vi.x; zi[i + 1] = vi.y;
                        zf[i] = vf.x; zf[i + 1] = vf.y;
                        zz[i] = vz.x; zz[i + 1] = vz.y;
                        og[i] = go.x; og[i + 1] = go.y;
                    }
                    // ---- m: max-plus recurrence
                    if (!first && !mbar_wait_bounded(&mbar_m[g * W + warp], par, timed_out ? kWaitLimitAfterTimeout : kFusedWaitLimit))
                        timed_out = true;
                    float m = slot_in[2 * kLanes];
                    float dlt[L], ms[L];
#pragma unroll
                    for (int i = 0; i < L; ++i) {
                        if (FULL || t0 + i < a.T) {
                            const float left = zf[i] + m;
                            dlt[i] = left - zi[i];
                            m = fmaxf(left, zi[i]);
                        } else {
                            dlt[i] = 0.f;
                        }
                        ms[i] = m;
                    }
                    slot_out[2 * kLanes] = m;
                    __syncwarp();
                    if (lane == 0 && !last) fp_mbar_arrive(&mbar_m[g * W + next]);
                    float e[L];
#pragma unroll
                    for (int i = 0; i < L; i += 2) {
                        const float2 ev = exp_f2(make_float2(-fabsf(dlt[i]), -fabsf(dlt[i + 1])));
                        e[i] = ev.x;
                        e[i + 1] = ev.y;
                    }
                    // ---- (c, n): multiply-add recurrences
                    if (!first && !mbar_wait_bounded(&mbar_cn[g * W + warp], par, timed_out ? kWaitLimitAfterTimeout : kFusedWaitLimit))
                        timed_out = true;
                    float c = slot_in[0], n = slot_in[kLanes];
                    const float h_before = slot_in[3 * kLanes];  // this pass's h at step t0-1
                    float cs[L], ns[L];
#pragma unroll
                    for (int i = 0; i < L; ++i) {
                        if (FULL || t0 + i < a.T) {
                            const bool lw = dlt[i] >= 0.f;
                            const float ft = lw ? 1.f : e[i], it = lw ? e[i] : 1.f;
                            n = fmaf(ft, n, it);
                            c = fmaf(ft, c, it * zz[i]);
                        }
                        cs[i] = c;
                        ns[i] = n;
                    }
                    float h[L];
#pragma unroll
                    for (int i = 0; i < L; i += 2) {
                        const float2 den = __fmul2_rn(make_float2(og[i], og[i + 1]),
                                                      __fadd2_rn(make_float2(ns[i], ns[i + 1]), splat2(a.eps)));
                        const float2 hv = __fmul2_rn(make_float2(cs[i], cs[i + 1]), rcp_2(den));
                        h[i] = hv.x;
                        h[i + 1] = hv.y;
                    }
                    slot_out[0] = c;
                    slot_out[kLanes] = n;
                    slot_out[3 * kLanes] = h[L - 1];
                    __syncwarp();
                    if (lane == 0 && !last) fp_mbar_arrive(&mbar_cn[g * W + next]);

                    if (g == n_pass - 1) {
                        if (ch_ok) {
                            float* o = a.state_out + ((size_t)b * a.T + t0) * 4 * d + ch;
#pragma unroll
                            for (int i = 0; i < L; ++i) {
                                if (FULL || t0 + i < a.T) {
                                    float* oi = o + (size_t)i * 4 * d;
                                    oi[0] = cs[i];
                                    oi[d] = ns[i];
                                    oi[2 * (size_t)d] = ms[i];
                                    oi[3 * (size_t)d] = h[i];
                                }
                            }
                            if (last && a.tail_out) {
                                a.tail_out[((size_t)b * 3 + 0) * d + ch] = c;
                                a.tail_out[((size_t)b * 3 + 1) * d + ch] = n;
                                a.tail_out[((size_t)b * 3 + 2) * d + ch] = m;
                            }
                        }
                    } else {
                        // the next pass sees this pass's hidden state one step earlier
#pragma unroll
                        for (int i = L - 1; i > 0; --i) hp[i] = h[i - 1];
                        hp[0] = (t0 == 0) ? h_halo : h_before;
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
}

template <typename TIO, int NSTAGE, int L, int W>
cudaError_t launch_lw(const SlstmPicardArgs& a, int n_pass, cudaStream_t s) {
    using S = FusedPicardSmem<TIO, L, W, NSTAGE>;
    CUtensorMap tm_wx;
    const uint64_t rows = (uint64_t)a.B * a.T;
    if (!make_tile_map(&tm_wx, a.wx, sizeof(TIO), rows, 4, a.d, S::LT)) return cudaErrorNotSupported;
    const int grid = a.B * ((a.d + kLanes - 1) / kLanes);
    auto k = slstm_picard_fused_kernel<TIO, L, W, NSTAGE>;
    cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
    k<<<grid, W * 32, S::TOTAL, s>>>(tm_wx, a, n_pass);
    return cudaGetLastError();
}

// 8 warps x 8 steps, two CTAs per SM (128 registers per thread) when there are more chains than
// SMs; with fewer chains a CTA has an SM to itself and a single chain's walk is bound by latency,
// so 16 warps x 4 steps put twice as many warps on the same round.
template <typename TIO, int NSTAGE>
cudaError_t launch_t(const SlstmPicardArgs& a, int n_pass, cudaStream_t s) {
    const int chains = a.B * ((a.d + kLanes - 1) / kLanes);
    return chains > sm_count() ? launch_lw<TIO, NSTAGE, 8, 8>(a, n_pass, s) : launch_lw<TIO, NSTAGE, 8, 16>(a, n_pass, s);
}

}  // namespace

int slstm_picard_fused_max_passes() { return kFusedMaxPass; }

// All `n_pass` Picard passes (zero-hidden pass first) of one chain set in one launch; writes
// a.state_out only.  cudaErrorNotSupported when n_pass is out of range or TMA cannot address wx.
cudaError_t launch_slstm_picard_fused(int dtype, const SlstmPicardArgs& a, int n_pass, cudaStream_t s) {
    if (n_pass < 1 || n_pass > kFusedMaxPass || !a.state_out) return cudaErrorNotSupported;
    return dtype == kF32 ? launch_t<float, 2>(a, n_pass, s) : launch_t<__nv_bfloat16, 3>(a, n_pass, s);
}

}  // namespace prb
