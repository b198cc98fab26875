// ParaSLSTM mix='diag', persistent-chain kernels.
//
// One CTA owns one chain (batch row x 32 channels) and walks the whole time axis in rounds of
// W*L steps.  The carry of the scan never leaves the CTA, so there are no inter-CTA waits at
// all; the inputs of round r+NSTAGE are fetched by TMA (cp.async.bulk.tensor tile loads into a
// shared-memory ring, completion on mbarriers) while round r is computed.  Inside a round the
// W warps split the steps: every thread linearises its L steps and composes their map, the maps
// meet in shared memory (one __syncthreads per round), and each warp folds the maps of the
// warps before it into the carry that entered the round.
//
// Used when there are enough chains to fill the GPU and the arrays meet TMA's alignment rules;
// otherwise the look-back kernels of slstm_kernels.cu run.  Same math as those kernels
// (slstm_cell.cuh), same reference behaviour restated (see slstm_kernels.cu).
#include "common.cuh"
#include "kernels.h"
#include "slstm_cell.cuh"
#include "tma.cuh"

namespace prb {

constexpr uint32_t kTmaWaitLimit = 1u << 24;

// ------------------------------------------------------------------ host: tensor maps
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

bool make_tile_map(CUtensorMap* out, const void* base, int elem_bytes, uint64_t rows, uint32_t mid,
                   uint64_t inner, uint32_t box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn || !base) return false;
    if (reinterpret_cast<uintptr_t>(base) & 15u) return false;
    if ((inner * elem_bytes) & 15u) return false;
    if (box_rows > 256 || mid > 256) return false;
    const CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                   : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    cuuint64_t dims[3] = {inner, mid, rows};
    cuuint64_t strides[2] = {inner * elem_bytes, inner * elem_bytes * mid};
    cuuint32_t box[3] = {32, mid, box_rows};
    cuuint32_t estr[3] = {1, 1, 1};
    return fn(out, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// ------------------------------------------------------------------ Newton
template <typename TIO, int L, int W, int NSTAGE>
struct NewtonSmem {
    static constexpr int LT = W * L;
    static constexpr int WX_BYTES = LT * 4 * kLanes * (int)sizeof(TIO);
    static constexpr int ST_BYTES = (LT + 1) * 4 * kLanes * 4;
    static constexpr int STAGE = WX_BYTES + ST_BYTES;
    static constexpr int MAPS_OFF = NSTAGE * STAGE;
    static constexpr int MAPS_BYTES = 2 * W * 20 * kLanes * 4;
    static constexpr int CARRY_OFF = MAPS_OFF + MAPS_BYTES;
    static constexpr int CARRY_BYTES = 2 * 4 * kLanes * 4;
    static constexpr int BAR_OFF = CARRY_OFF + CARRY_BYTES;
    static constexpr int RED_OFF = BAR_OFF + NSTAGE * 8;
    static constexpr int TOTAL = RED_OFF + W * 4 + 64;
};

template <typename TIO, int L, int W, int NSTAGE, bool LAST>
__global__ void __launch_bounds__(W * 32, 2)
slstm_newton_persist_kernel(const __grid_constant__ CUtensorMap tm_wx,
                            const __grid_constant__ CUtensorMap tm_st, SlstmNewtonArgs a) {
    using S = NewtonSmem<TIO, L, W, NSTAGE>;
    constexpr int LT = S::LT;
    extern __shared__ __align__(128) unsigned char smem[];
    float* s_maps = reinterpret_cast<float*>(smem + S::MAPS_OFF);
    float* s_carry = reinterpret_cast<float*>(smem + S::CARRY_OFF);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::BAR_OFF);
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

    auto issue = [&](int r) {
        const int s = r % NSTAGE;
        unsigned char* base = smem + s * S::STAGE;
        mbar_expect_tx(&bars[s], S::STAGE);
        tma_load_3d(base, &tm_wx, &bars[s], cb * kLanes, 0, row0 + r * LT);
        tma_load_3d(base + S::WX_BYTES, &tm_st, &bars[s], cb * kLanes, 0, row0 + r * LT - 1);
    };

    if (threadIdx.x == 0) {
        tma_prefetch_desc(&tm_wx);
        tma_prefetch_desc(&tm_st);
        for (int s = 0; s < NSTAGE; ++s) mbar_init(&bars[s], 1);
        mbar_fence_init();
    }
    if (warp == 0) {
#pragma unroll
        for (int q = 0; q < 4; ++q)
            s_carry[q * kLanes + lane] = a.carry_in ? __ldg(a.carry_in + ((size_t)b * 4 + q) * d + chl) : 0.f;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int r = 0; r < NSTAGE && r < n_rounds; ++r) issue(r);
    }

    float r4[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) r4[q] = __ldg(a.r + (size_t)q * d + chl);

    unsigned rmax = 0u, fmax = 0u;
    const bool want_final = LAST && a.final_bits != nullptr;
    bool timed_out = false;

    for (int r = 0; r < n_rounds; ++r) {
        const int s = r % NSTAGE;
        if (!mbar_wait_bounded(&bars[s], (r / NSTAGE) & 1, kTmaWaitLimit)) timed_out = true;
        const TIO* t_wx = reinterpret_cast<const TIO*>(smem + s * S::STAGE);
        const float* t_st = reinterpret_cast<const float*>(smem + s * S::STAGE + S::WX_BYTES);
        const int t0 = r * LT + warp * L;

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

        SlstmLin lin[L];
        float F[L][4];
        float mp[20];
#pragma unroll
        for (int i = 0; i < L; ++i) {
            slstm_linearize(st[i], w[i], r4, a.eps, lin[i]);
            const bool ok = t0 + i < a.T;
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
            if (i == 0) {
#pragma unroll
                for (int k = 0; k < 20; ++k) mp[k] = 0.f;
                mp[0] = 1.f; mp[5] = 1.f; mp[10] = 1.f; mp[15] = 1.f;
            }
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
        float* maps = s_maps + (r & 1) * (W * 20 * kLanes);
        if (warp < W - 1) {
#pragma unroll
            for (int k = 0; k < 20; ++k) maps[(warp * 20 + k) * kLanes + lane] = mp[k];
        }
        // all reads of stage s are done; the barrier also publishes the maps
        const int bad = __syncthreads_or(timed_out ? 1 : 0);
        if (bad) {
            if (threadIdx.x == 0) atomicExch(a.chain.status, (int)kErrChainTimeout);
            return;
        }
        if (threadIdx.x == 0 && r + NSTAGE < n_rounds) {
            fence_proxy_async();
            issue(r + NSTAGE);
        }
        // carry entering this warp's sub-tile
        const float* cin = s_carry + (r & 1) * (4 * kLanes);
        float cv[4] = {cin[lane], cin[kLanes + lane], cin[2 * kLanes + lane], cin[3 * kLanes + lane]};
#pragma unroll
        for (int w2 = 0; w2 < W - 1; ++w2) {
            if (w2 < warp) {
                float m[20];
#pragma unroll
                for (int k = 0; k < 20; ++k) m[k] = maps[(w2 * 20 + k) * kLanes + lane];
                Affine4::apply(m, cv);
            }
        }
        float xc = cv[0], xn = cv[1], xm = cv[2], xh = cv[3];
        float pn4[4] = {fmaf(a.omega, xc, st[0][0]), fmaf(a.omega, xn, st[0][1]),
                        fmaf(a.omega, xm, st[0][2]), fmaf(a.omega, xh, st[0][3])};
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
        if (warp == W - 1) {
            // (xc..xh) is now the carry leaving the round (identity steps beyond T keep it)
            float* cout = s_carry + ((r + 1) & 1) * (4 * kLanes);
            cout[lane] = xc;
            cout[kLanes + lane] = xn;
            cout[2 * kLanes + lane] = xm;
            cout[3 * kLanes + lane] = xh;
            if (r == n_rounds - 1 && a.tail_out && ch_ok) {
                a.tail_out[((size_t)b * 4 + 0) * d + ch] = xc;
                a.tail_out[((size_t)b * 4 + 1) * d + ch] = xn;
                a.tail_out[((size_t)b * 4 + 2) * d + ch] = xm;
                a.tail_out[((size_t)b * 4 + 3) * d + ch] = xh;
            }
        }
    }
    __syncthreads();
    block_residual_max(rmax, a.resid_bits, s_red);
    if (want_final) {
        __syncthreads();
        block_residual_max(fmax, a.final_bits, s_red);
    }
}


// ------------------------------------------------------------------ Picard
template <typename TIO, int L, int W, int NSTAGE>
struct PicardSmem {
    static constexpr int LT = W * L;
    static constexpr int WX_BYTES = LT * 4 * kLanes * (int)sizeof(TIO);
    static constexpr int H_BYTES = ((LT + 1) * kLanes * 4 + 127) / 128 * 128;
    static constexpr int STAGE = WX_BYTES + H_BYTES;
    static constexpr int MAPS_OFF = NSTAGE * STAGE;
    static constexpr int MAPS_BYTES = 2 * W * 4 * kLanes * 4;
    static constexpr int CARRY_OFF = MAPS_OFF + MAPS_BYTES;
    static constexpr int CARRY_BYTES = 2 * 3 * kLanes * 4;
    static constexpr int BAR_OFF = CARRY_OFF + CARRY_BYTES;
    static constexpr int TOTAL = BAR_OFF + NSTAGE * 8 + 64;
};

// HAS_H: a previous hidden trajectory exists (every pass but the zero-hidden one).
template <typename TIO, int L, int W, int NSTAGE, bool HAS_H>
__global__ void __launch_bounds__(W * 32, 2)
slstm_picard_persist_kernel(const __grid_constant__ CUtensorMap tm_wx,
                            const __grid_constant__ CUtensorMap tm_h, SlstmPicardArgs a) {
    using S = PicardSmem<TIO, L, W, NSTAGE>;
    using M = PicardMonoid;
    constexpr int LT = S::LT;
    extern __shared__ __align__(128) unsigned char smem[];
    float* s_maps = reinterpret_cast<float*>(smem + S::MAPS_OFF);
    float* s_carry = reinterpret_cast<float*>(smem + S::CARRY_OFF);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::BAR_OFF);

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

    auto issue = [&](int r) {
        const int s = r % NSTAGE;
        unsigned char* base = smem + s * S::STAGE;
        mbar_expect_tx(&bars[s], S::WX_BYTES + (HAS_H ? (LT + 1) * kLanes * 4 : 0));
        tma_load_3d(base, &tm_wx, &bars[s], cb * kLanes, 0, row0 + r * LT);
        if (HAS_H) tma_load_3d(base + S::WX_BYTES, &tm_h, &bars[s], cb * kLanes, 0, row0 + r * LT - 1);
    };

    if (threadIdx.x == 0) {
        tma_prefetch_desc(&tm_wx);
        if (HAS_H) tma_prefetch_desc(&tm_h);
        for (int s = 0; s < NSTAGE; ++s) mbar_init(&bars[s], 1);
        mbar_fence_init();
    }
    if (warp == 0) {
#pragma unroll
        for (int q = 0; q < 3; ++q)
            s_carry[q * kLanes + lane] =
                a.carry_in ? __ldg(a.carry_in + (size_t)b * a.carry_stride + (size_t)q * d + chl) : 0.f;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int r = 0; r < NSTAGE && r < n_rounds; ++r) issue(r);
    }
    float r4[4] = {0.f, 0.f, 0.f, 0.f};
    if (HAS_H) {
#pragma unroll
        for (int q = 0; q < 4; ++q) r4[q] = __ldg(a.r + (size_t)q * d + chl);
    }
    bool timed_out = false;

    for (int r = 0; r < n_rounds; ++r) {
        const int s = r % NSTAGE;
        if (!mbar_wait_bounded(&bars[s], (r / NSTAGE) & 1, kTmaWaitLimit)) timed_out = true;
        const TIO* t_wx = reinterpret_cast<const TIO*>(smem + s * S::STAGE);
        const float* t_h = reinterpret_cast<const float*>(smem + s * S::STAGE + S::WX_BYTES);
        const int t0 = r * LT + warp * L;

        float zi[L], zf[L], zz[L], zo[L];
#pragma unroll
        for (int i = 0; i < L; ++i) {
            float hp = 0.f;
            if (HAS_H) {
                hp = (t0 + i == 0) ? (a.h_halo ? __ldg(a.h_halo + (size_t)b * a.halo_stride + chl) : 0.f)
                                   : t_h[(warp * L + i) * kLanes + lane];
            }
            const int row = warp * L + i;
            zi[i] = fmaf(r4[0], hp, (float)t_wx[(row * 4 + 0) * kLanes + lane]);
            zf[i] = fmaf(r4[1], hp, (float)t_wx[(row * 4 + 1) * kLanes + lane]);
            zz[i] = tanh_f(fmaf(r4[2], hp, (float)t_wx[(row * 4 + 2) * kLanes + lane]));
            zo[i] = fmaf(r4[3], hp, (float)t_wx[(row * 4 + 3) * kLanes + lane]);
        }
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
        float* maps = s_maps + (r & 1) * (W * 4 * kLanes);
        if (warp < W - 1) {
#pragma unroll
            for (int k = 0; k < 4; ++k) maps[(warp * 4 + k) * kLanes + lane] = mp[k];
        }
        const int bad = __syncthreads_or(timed_out ? 1 : 0);
        if (bad) {
            if (threadIdx.x == 0) atomicExch(a.chain.status, (int)kErrChainTimeout);
            return;
        }
        if (threadIdx.x == 0 && r + NSTAGE < n_rounds) {
            fence_proxy_async();
            issue(r + NSTAGE);
        }
        const float* cin = s_carry + (r & 1) * (3 * kLanes);
        float cv[3] = {cin[lane], cin[kLanes + lane], cin[2 * kLanes + lane]};
#pragma unroll
        for (int w2 = 0; w2 < W - 1; ++w2) {
            if (w2 < warp) {
                float m[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) m[k] = maps[(w2 * 4 + k) * kLanes + lane];
                M::apply(m, cv);
            }
        }
        float c = cv[0], n = cv[1], m = cv[2];
#pragma unroll
        for (int i = 0; i < L; ++i) {
            const int t = t0 + i;
            if (t < a.T) {
                const float left = zf[i] + m;
                const float e = exp_f(-fabsf(left - zi[i]));
                const bool lw = left >= zi[i];
                const float ft = lw ? 1.f : e, it = lw ? e : 1.f;
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
        if (warp == W - 1) {
            float* cout = s_carry + ((r + 1) & 1) * (3 * kLanes);
            cout[lane] = c;
            cout[kLanes + lane] = n;
            cout[2 * kLanes + lane] = m;
            if (r == n_rounds - 1 && a.tail_out && ch_ok) {
                a.tail_out[((size_t)b * 3 + 0) * d + ch] = c;
                a.tail_out[((size_t)b * 3 + 1) * d + ch] = n;
                a.tail_out[((size_t)b * 3 + 2) * d + ch] = m;
            }
        }
    }
}

// ------------------------------------------------------------------ backward
template <typename TIO, int L, int W, int NSTAGE>
struct BwdSmem {
    static constexpr int LT = W * L;
    static constexpr int WX_BYTES = LT * 4 * kLanes * (int)sizeof(TIO);
    static constexpr int ST_BYTES = ((LT + 1) * 4 * kLanes * (int)sizeof(TIO) + 127) / 128 * 128;
    static constexpr int G_BYTES = WX_BYTES;
    static constexpr int STAGE = WX_BYTES + ST_BYTES + G_BYTES;
    static constexpr int MAPS_OFF = NSTAGE * STAGE;
    static constexpr int MAPS_BYTES = 2 * W * 20 * kLanes * 4;
    static constexpr int CARRY_OFF = MAPS_OFF + MAPS_BYTES;
    static constexpr int CARRY_BYTES = 2 * 4 * kLanes * 4;
    static constexpr int BAR_OFF = CARRY_OFF + CARRY_BYTES;
    static constexpr int TOTAL = BAR_OFF + NSTAGE * 8 + 64;
};

// Rounds run from the end of the sequence to its start; warp 0 owns the highest steps of a
// round.  nu_{t-1} = J_t^T (nu_t + g_t); the carry is nu.
template <typename TIO, int L, int W, int NSTAGE>
__global__ void __launch_bounds__(W * 32, 2)
slstm_bwd_persist_kernel(const __grid_constant__ CUtensorMap tm_wx, const __grid_constant__ CUtensorMap tm_st,
                         const __grid_constant__ CUtensorMap tm_g, SlstmBwdArgs a) {
    using S = BwdSmem<TIO, L, W, NSTAGE>;
    constexpr int LT = S::LT;
    extern __shared__ __align__(128) unsigned char smem[];
    float* s_maps = reinterpret_cast<float*>(smem + S::MAPS_OFF);
    float* s_carry = reinterpret_cast<float*>(smem + S::CARRY_OFF);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::BAR_OFF);

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

    auto issue = [&](int r) {
        const int s = r % NSTAGE;
        const int tile_t = n_rounds - 1 - r;
        unsigned char* base = smem + s * S::STAGE;
        mbar_expect_tx(&bars[s], S::WX_BYTES + (LT + 1) * 4 * kLanes * (int)sizeof(TIO) + S::G_BYTES);
        tma_load_3d(base, &tm_wx, &bars[s], cb * kLanes, 0, row0 + tile_t * LT);
        tma_load_3d(base + S::WX_BYTES, &tm_st, &bars[s], cb * kLanes, 0, row0 + tile_t * LT - 1);
        tma_load_3d(base + S::WX_BYTES + S::ST_BYTES, &tm_g, &bars[s], cb * kLanes, 0, row0 + tile_t * LT);
    };

    if (threadIdx.x == 0) {
        tma_prefetch_desc(&tm_wx);
        tma_prefetch_desc(&tm_st);
        tma_prefetch_desc(&tm_g);
        for (int s = 0; s < NSTAGE; ++s) mbar_init(&bars[s], 1);
        mbar_fence_init();
    }
    if (warp == 0) {
#pragma unroll
        for (int q = 0; q < 4; ++q)
            s_carry[q * kLanes + lane] = a.carry_in ? __ldg(a.carry_in + ((size_t)b * 4 + q) * d + chl) : 0.f;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int r = 0; r < NSTAGE && r < n_rounds; ++r) issue(r);
    }
    float r4[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) r4[q] = __ldg(a.r + (size_t)q * d + chl);
    float gr[4] = {0.f, 0.f, 0.f, 0.f};
    bool timed_out = false;
    TIO* gwx = reinterpret_cast<TIO*>(a.g_wx) + (size_t)b * a.T * 4 * d + ch;

    for (int r = 0; r < n_rounds; ++r) {
        const int s = r % NSTAGE;
        const int tile_t = n_rounds - 1 - r;
        if (!mbar_wait_bounded(&bars[s], (r / NSTAGE) & 1, kTmaWaitLimit)) timed_out = true;
        const TIO* t_wx = reinterpret_cast<const TIO*>(smem + s * S::STAGE);
        const TIO* t_st = reinterpret_cast<const TIO*>(smem + s * S::STAGE + S::WX_BYTES);
        const TIO* t_g = reinterpret_cast<const TIO*>(smem + s * S::STAGE + S::WX_BYTES + S::ST_BYTES);
        const int row_hi = (W - 1 - warp) * L + (L - 1);  // row inside the tile of this thread's top step
        const int t_hi = tile_t * LT + row_hi;

        SlstmAct act[L];
        float g[L][4];
        float mp[20];
#pragma unroll
        for (int i = 0; i < L; ++i) {
            const int row = row_hi - i;
            const int t = t_hi - i;
            const bool ok = t < a.T;
            float w[4], prev[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) w[q] = (float)t_wx[(row * 4 + q) * kLanes + lane];
            if (t == 0) {
#pragma unroll
                for (int q = 0; q < 4; ++q)
                    prev[q] = a.halo ? __ldg(a.halo + (size_t)b * a.halo_stride + (size_t)q * d + chl) : 0.f;
            } else {
#pragma unroll
                for (int q = 0; q < 4; ++q) prev[q] = (float)t_st[(row * 4 + q) * kLanes + lane];
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) g[i][q] = ok ? (float)t_g[(row * 4 + q) * kLanes + lane] : 0.f;
            SlstmLin lin;
            slstm_linearize(prev, w, r4, a.eps, lin);
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
        float* maps = s_maps + (r & 1) * (W * 20 * kLanes);
        if (warp < W - 1) {
#pragma unroll
            for (int k = 0; k < 20; ++k) maps[(warp * 20 + k) * kLanes + lane] = mp[k];
        }
        const int bad = __syncthreads_or(timed_out ? 1 : 0);
        if (bad) {
            if (threadIdx.x == 0) atomicExch(a.chain.status, (int)kErrChainTimeout);
            return;
        }
        if (threadIdx.x == 0 && r + NSTAGE < n_rounds) {
            fence_proxy_async();
            issue(r + NSTAGE);
        }
        const float* cin = s_carry + (r & 1) * (4 * kLanes);
        float cv[4] = {cin[lane], cin[kLanes + lane], cin[2 * kLanes + lane], cin[3 * kLanes + lane]};
#pragma unroll
        for (int w2 = 0; w2 < W - 1; ++w2) {
            if (w2 < warp) {
                float m[20];
#pragma unroll
                for (int k = 0; k < 20; ++k) m[k] = maps[(w2 * 20 + k) * kLanes + lane];
                Affine4::apply(m, cv);
            }
        }
        float nc = cv[0], nn = cv[1], nm = cv[2], nh = cv[3];
#pragma unroll
        for (int i = 0; i < L; ++i) {
            const int t = t_hi - i;
            if (t < a.T) {
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
                if (ch_ok) {
                    TIO* o = gwx + (size_t)t * 4 * d;
                    st_f(o, d_zi);
                    st_f(o + d, d_zf);
                    st_f(o + 2 * (size_t)d, d_zz);
                    st_f(o + 3 * (size_t)d, d_zo);
                }
                gr[0] = fmaf(d_zi, sa.hp, gr[0]);
                gr[1] = fmaf(d_zf, sa.hp, gr[1]);
                gr[2] = fmaf(d_zz, sa.hp, gr[2]);
                gr[3] = fmaf(d_zo, sa.hp, gr[3]);
                nc = d_cn * sa.f;
                nn = d_nn * sa.f;
                nm = d_zf;
                nh = fmaf(r4[0], d_zi, fmaf(r4[1], d_zf, fmaf(r4[2], d_zz, r4[3] * d_zo)));
            }
        }
        if (warp == W - 1) {
            float* cout = s_carry + ((r + 1) & 1) * (4 * kLanes);
            cout[lane] = nc;
            cout[kLanes + lane] = nn;
            cout[2 * kLanes + lane] = nm;
            cout[3 * kLanes + lane] = nh;
            if (r == n_rounds - 1 && a.g_h0 && ch_ok) {
                a.g_h0[((size_t)b * 4 + 0) * d + ch] = nc;
                a.g_h0[((size_t)b * 4 + 1) * d + ch] = nn;
                a.g_h0[((size_t)b * 4 + 2) * d + ch] = nm;
                a.g_h0[((size_t)b * 4 + 3) * d + ch] = nh;
            }
        }
    }
    // one parameter partial per chain: fixed-order sum over the W warps
    __syncthreads();
    float* s_gp = s_maps;
#pragma unroll
    for (int p = 0; p < 4; ++p) s_gp[(warp * 4 + p) * kLanes + lane] = gr[p];
    __syncthreads();
    if (warp == 0 && ch_ok) {
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            float sum = 0.f;
#pragma unroll
            for (int w2 = 0; w2 < W; ++w2) sum += s_gp[(w2 * 4 + p) * kLanes + lane];
            a.gp_partial[((size_t)b * 4 + p) * d + ch] = sum;
        }
    }
}

// ------------------------------------------------------------------ launchers
constexpr int kPL = 4, kPW = 8;

bool slstm_persist_ok(int dtype, int B, int T, int d) {
    const int elem = dtype == kF32 ? 4 : 2;
    if ((d * elem) & 15) return false;                       // TMA stride rule for wx / states
    if ((long long)B * T > 0x7fffff00LL) return false;       // row coordinate is a 32-bit int
    return encode_fn() != nullptr;
}

template <typename TIO, int NSTAGE>
static cudaError_t launch_newton_t(const SlstmNewtonArgs& a, bool last, cudaStream_t s) {
    using S = NewtonSmem<TIO, kPL, kPW, NSTAGE>;
    CUtensorMap tm_wx, tm_st;
    const uint64_t rows = (uint64_t)a.B * a.T;
    if (!make_tile_map(&tm_wx, a.wx, sizeof(TIO), rows, 4, a.d, S::LT) ||
        !make_tile_map(&tm_st, a.sin, 4, rows, 4, a.d, S::LT + 1))
        return cudaErrorNotSupported;
    const int grid = a.B * ((a.d + kLanes - 1) / kLanes);
    if (last) {
        auto k = slstm_newton_persist_kernel<TIO, kPL, kPW, NSTAGE, true>;
        cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
        k<<<grid, kPW * 32, S::TOTAL, s>>>(tm_wx, tm_st, a);
    } else {
        auto k = slstm_newton_persist_kernel<TIO, kPL, kPW, NSTAGE, false>;
        cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
        k<<<grid, kPW * 32, S::TOTAL, s>>>(tm_wx, tm_st, a);
    }
    return cudaGetLastError();
}

template <typename TIO, int NSTAGE>
static cudaError_t launch_picard_t(const SlstmPicardArgs& a, cudaStream_t s) {
    constexpr int L = 8, W = 8;
    using S = PicardSmem<TIO, L, W, NSTAGE>;
    CUtensorMap tm_wx, tm_h;
    const uint64_t rows = (uint64_t)a.B * a.T;
    if (!make_tile_map(&tm_wx, a.wx, sizeof(TIO), rows, 4, a.d, S::LT)) return cudaErrorNotSupported;
    const int grid = a.B * ((a.d + kLanes - 1) / kLanes);
    if (a.h_prev) {
        if (!make_tile_map(&tm_h, a.h_prev, 4, rows, 1, a.d, S::LT + 1)) return cudaErrorNotSupported;
        auto k = slstm_picard_persist_kernel<TIO, L, W, NSTAGE, true>;
        cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
        k<<<grid, W * 32, S::TOTAL, s>>>(tm_wx, tm_h, a);
    } else {
        auto k = slstm_picard_persist_kernel<TIO, L, W, NSTAGE, false>;
        cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
        k<<<grid, W * 32, S::TOTAL, s>>>(tm_wx, tm_wx, a);
    }
    return cudaGetLastError();
}

cudaError_t launch_slstm_picard_persist(int dtype, const SlstmPicardArgs& a, cudaStream_t s) {
    return dtype == kF32 ? launch_picard_t<float, 2>(a, s) : launch_picard_t<__nv_bfloat16, 3>(a, s);
}

template <typename TIO, int NSTAGE>
static cudaError_t launch_bwd_t(const SlstmBwdArgs& a, cudaStream_t s) {
    using S = BwdSmem<TIO, kPL, kPW, NSTAGE>;
    CUtensorMap tm_wx, tm_st, tm_g;
    const uint64_t rows = (uint64_t)a.B * a.T;
    if (!make_tile_map(&tm_wx, a.wx, sizeof(TIO), rows, 4, a.d, S::LT) ||
        !make_tile_map(&tm_st, a.states, sizeof(TIO), rows, 4, a.d, S::LT + 1) ||
        !make_tile_map(&tm_g, a.grad_states, sizeof(TIO), rows, 4, a.d, S::LT))
        return cudaErrorNotSupported;
    const int grid = a.B * ((a.d + kLanes - 1) / kLanes);
    auto k = slstm_bwd_persist_kernel<TIO, kPL, kPW, NSTAGE>;
    cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
    k<<<grid, kPW * 32, S::TOTAL, s>>>(tm_wx, tm_st, tm_g, a);
    return cudaGetLastError();
}

// gp_partial receives one row per batch row: (B, 4, d)
cudaError_t launch_slstm_bwd_persist(int dtype, const SlstmBwdArgs& a, cudaStream_t s) {
    return dtype == kF32 ? launch_bwd_t<float, 2>(a, s) : launch_bwd_t<__nv_bfloat16, 2>(a, s);
}

cudaError_t launch_slstm_newton_persist(int dtype, const SlstmNewtonArgs& a, bool last, cudaStream_t s) {
    return dtype == kF32 ? launch_newton_t<float, 2>(a, last, s)
                         : launch_newton_t<__nv_bfloat16, 2>(a, last, s);
}

}  // namespace prb
