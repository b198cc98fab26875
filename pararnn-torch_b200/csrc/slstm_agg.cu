// ParaSLSTM mix='diag': aggregate-only sweeps for time-sharded runs.
//
// A rank that does not know the carry entering its shard first needs the affine map of the
// WHOLE shard.  Nothing is written but that map, so the sweep has no serial dependency at all:
// one CTA per chain (batch row x 32 channels), each of its W warps walks its own contiguous
// eighth of the shard, composing the per-step maps into one running map in registers.  Every warp
// feeds itself: its lane 0 streams chunks of U steps into a warp-private shared-memory ring with
// TMA tile loads (one mbarrier per stage), several chunks ahead; warps never synchronise with each
// other until the W maps are composed once at the end.
//
// Same per-step math as the other sLSTM kernels (slstm_cell.cuh).
#include "common.cuh"
#include "kernels.h"
#include "slstm_cell.cuh"
#include "tma.cuh"

#include <type_traits>

namespace prb {

constexpr int kAggW = 8;
constexpr uint32_t kAggWaitLimit = 1u << 24;

// compose the W warp maps (time order = warp order) and write the result
template <class M>
__device__ __forceinline__ void finish_agg(float* smem, const float (&mp)[M::NV], int warp, int lane,
                                           float* agg_out, int b, int d, int ch, bool ch_ok) {
#pragma unroll
    for (int k = 0; k < M::NV; ++k) smem[(warp * M::NV + k) * kLanes + lane] = mp[k];
    __syncthreads();
    if (warp == 0) {
        float acc[M::NV];
#pragma unroll
        for (int k = 0; k < M::NV; ++k) acc[k] = mp[k];
        for (int w2 = 1; w2 < kAggW; ++w2) {
            float m[M::NV];
#pragma unroll
            for (int k = 0; k < M::NV; ++k) m[k] = smem[(w2 * M::NV + k) * kLanes + lane];
            M::compose(acc, m);
        }
        if (ch_ok) {
#pragma unroll
            for (int k = 0; k < M::NV; ++k) agg_out[((size_t)b * M::NV + k) * d + ch] = acc[k];
        }
    }
}

// the warp's share of the CTA's time segment [t_lo, t_hi)
__device__ __forceinline__ void seg_bounds(int t_lo, int t_hi, int warp, int& lo, int& hi) {
    const int seg = (t_hi - t_lo + kAggW - 1) / kAggW;
    lo = min(t_hi, t_lo + warp * seg);
    hi = min(t_hi, lo + seg);
}

// Warp-private TMA ring: NST stages of STAGE_BYTES each, one mbarrier per stage.
template <int NST>
struct WarpRing {
    unsigned char* base;
    uint64_t* bars;
    int stage_bytes;
    __device__ __forceinline__ void init(unsigned char* b, uint64_t* br, int sb, int lane) {
        base = b;
        bars = br;
        stage_bytes = sb;
        if (lane == 0) {
            for (int s = 0; s < NST; ++s) mbar_init(&bars[s], 1);
            mbar_fence_init();
        }
        __syncwarp();
    }
    __device__ __forceinline__ unsigned char* stage(int k) const { return base + (k % NST) * stage_bytes; }
    __device__ __forceinline__ bool wait(int k, bool timed_out) const {
        return mbar_wait_bounded(&bars[k % NST], (k / NST) & 1,
                                 timed_out ? kWaitLimitAfterTimeout : kAggWaitLimit);
    }
};

// ------------------------------------------------------------------ Newton
template <typename TIO, int U, int NST>
struct AggNewtonSmem {
    static constexpr int WX = U * 4 * kLanes * (int)sizeof(TIO);
    static constexpr int ST = U * 4 * kLanes * 4;
    static constexpr int STAGE = WX + ST;
    static constexpr int RING = NST * STAGE;
    static constexpr int MAPS_OFF = kAggW * RING;
    static constexpr int BAR_OFF = MAPS_OFF + kAggW * 20 * kLanes * 4;
    static constexpr int TOTAL = BAR_OFF + kAggW * NST * 8 + 64;
};

template <typename TIO, int U, int NST>
__global__ void __launch_bounds__(kAggW * 32, 2)
slstm_newton_agg_seg_kernel(const __grid_constant__ CUtensorMap tm_wx, const __grid_constant__ CUtensorMap tm_st,
                            SlstmNewtonArgs a) {
    using S = AggNewtonSmem<TIO, U, NST>;
    extern __shared__ __align__(128) unsigned char smem[];
    const int d = a.d;
    const int ncb = (d + kLanes - 1) / kLanes;
    const int b = blockIdx.x / ncb, cb = blockIdx.x % ncb;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ch = cb * kLanes + lane;
    const bool ch_ok = ch < d;
    const int chl = ch_ok ? ch : d - 1;
    const SegRange sg = seg_range(a.T, a.n_seg, a.seg_len);
    int lo, hi;
    seg_bounds(sg.lo, sg.hi, warp, lo, hi);
    WarpRing<NST> ring;
    ring.init(smem + warp * S::RING, reinterpret_cast<uint64_t*>(smem + S::BAR_OFF) + warp * NST, S::STAGE, lane);
    const int n_chunks = (hi - lo + U - 1) / U;
    const int row0 = b * a.T;
    auto issue = [&](int k) {
        unsigned char* st = ring.stage(k);
        mbar_expect_tx(&ring.bars[k % NST], S::STAGE);
        tma_load_3d(st, &tm_wx, &ring.bars[k % NST], cb * kLanes, 0, row0 + lo + k * U);
        tma_load_3d(st + S::WX, &tm_st, &ring.bars[k % NST], cb * kLanes, 0, row0 + lo + k * U);
    };
    if (lane == 0)
        for (int k = 0; k < NST && k < n_chunks; ++k) issue(k);
    float r4[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) r4[q] = __ldg(a.r + (size_t)q * d + chl);
    const float* sin = a.sin + (size_t)b * a.T * 4 * d + chl;
    float mp[20];
#pragma unroll
    for (int k = 0; k < 20; ++k) mp[k] = 0.f;
    mp[0] = mp[5] = mp[10] = mp[15] = 1.f;
    float prev[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        if (lo == 0)
            prev[q] = a.halo ? __ldg(a.halo + (size_t)b * a.halo_stride + (size_t)q * d + chl) : 0.f;
        else if (lo < a.T)
            prev[q] = __ldg(sin + ((size_t)(lo - 1) * 4 + q) * d);
        else
            prev[q] = 0.f;
    }
    bool timed_out = false;
    for (int k = 0; k < n_chunks; ++k) {
        if (!ring.wait(k, timed_out)) timed_out = true;
        const TIO* t_wx = reinterpret_cast<const TIO*>(ring.stage(k));
        const float* t_st = reinterpret_cast<const float*>(ring.stage(k) + S::WX);
        // chunks that lie fully inside the warp's range take a variant without range checks
        auto chunk_body = [&](auto full_c) {
            constexpr bool FULL = decltype(full_c)::value;
    #pragma unroll
            for (int i = 0; i < U; ++i) {
                if (FULL || lo + k * U + i < hi) {
                    float w[4], cur[4];
    #pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        w[q] = (float)t_wx[(i * 4 + q) * kLanes + lane];
                        cur[q] = t_st[(i * 4 + q) * kLanes + lane];
                    }
                    SlstmLin lin;
                    slstm_linearize(prev, w, r4, a.eps, lin);
                    const float fc = lin.pc - cur[0], fn = lin.pn - cur[1];
                    const float fm = lin.pm - cur[2], fh = lin.ph - cur[3];
                    const float fh2 = fh - lin.ia * fc - lin.ib * fn;
                    // the four matrix columns two at a time on packed FMAs, then the offset column
    #pragma unroll
                    for (int c2 = 0; c2 < 4; c2 += 2) {
                        float2 xc = make_float2(mp[0 * 4 + c2], mp[0 * 4 + c2 + 1]);
                        float2 xn = make_float2(mp[1 * 4 + c2], mp[1 * 4 + c2 + 1]);
                        float2 xm = make_float2(mp[2 * 4 + c2], mp[2 * 4 + c2 + 1]);
                        float2 xh = make_float2(mp[3 * 4 + c2], mp[3 * 4 + c2 + 1]);
                        slstm_apply_cols2(lin, xc, xn, xm, xh);
                        mp[0 * 4 + c2] = xc.x; mp[0 * 4 + c2 + 1] = xc.y;
                        mp[1 * 4 + c2] = xn.x; mp[1 * 4 + c2 + 1] = xn.y;
                        mp[2 * 4 + c2] = xm.x; mp[2 * 4 + c2 + 1] = xm.y;
                        mp[3 * 4 + c2] = xh.x; mp[3 * 4 + c2 + 1] = xh.y;
                    }
                    slstm_apply(lin, fc, fn, fm, fh2, mp[16], mp[17], mp[18], mp[19]);
    #pragma unroll
                    for (int q = 0; q < 4; ++q) prev[q] = cur[q];
                }
            }
        };
        if (lo + (k + 1) * U <= hi)
            chunk_body(std::true_type{});
        else
            chunk_body(std::false_type{});
        __syncwarp();
        if (lane == 0 && k + NST < n_chunks) {
            fence_proxy_async();
            issue(k + NST);
        }
    }
    if (timed_out) atomicExch(a.chain.status, (int)kErrChainTimeout);
    if (lane == 0 && timed_out) drain_ring(ring.bars, NST, n_chunks, kDrainLimit);
    finish_agg<Affine4>(reinterpret_cast<float*>(smem + S::MAPS_OFF), mp, warp, lane,
                        a.agg_out + (size_t)sg.seg * a.B * 20 * d, b, d, ch, ch_ok);
}

// ------------------------------------------------------------------ Picard
template <typename TIO, int U, int NST>
struct AggPicardSmem {
    static constexpr int WX = U * 4 * kLanes * (int)sizeof(TIO);
    static constexpr int HB = U * kLanes * 4;
    static constexpr int STAGE = WX + HB;
    static constexpr int RING = NST * STAGE;
    static constexpr int MAPS_OFF = kAggW * RING;
    static constexpr int BAR_OFF = MAPS_OFF + kAggW * 4 * kLanes * 4;
    static constexpr int TOTAL = BAR_OFF + kAggW * NST * 8 + 64;
};

template <typename TIO, int U, int NST, bool HAS_H>
__global__ void __launch_bounds__(kAggW * 32, 2)
slstm_picard_agg_seg_kernel(const __grid_constant__ CUtensorMap tm_wx, const __grid_constant__ CUtensorMap tm_h,
                            SlstmPicardArgs a) {
    using S = AggPicardSmem<TIO, U, NST>;
    extern __shared__ __align__(128) unsigned char smem[];
    const int d = a.d;
    const int ncb = (d + kLanes - 1) / kLanes;
    const int b = blockIdx.x / ncb, cb = blockIdx.x % ncb;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ch = cb * kLanes + lane;
    const bool ch_ok = ch < d;
    const int chl = ch_ok ? ch : d - 1;
    const SegRange sg = seg_range(a.T, a.n_seg, a.seg_len);
    int lo, hi;
    seg_bounds(sg.lo, sg.hi, warp, lo, hi);
    WarpRing<NST> ring;
    ring.init(smem + warp * S::RING, reinterpret_cast<uint64_t*>(smem + S::BAR_OFF) + warp * NST, S::STAGE, lane);
    const int n_chunks = (hi - lo + U - 1) / U;
    const int row0 = b * a.T;
    auto issue = [&](int k) {
        unsigned char* st = ring.stage(k);
        mbar_expect_tx(&ring.bars[k % NST], S::WX + (HAS_H ? S::HB : 0));
        tma_load_3d(st, &tm_wx, &ring.bars[k % NST], cb * kLanes, 0, row0 + lo + k * U);
        // hidden state of the PREVIOUS step: rows shifted by one
        if (HAS_H) tma_load_3d(st + S::WX, &tm_h, &ring.bars[k % NST], cb * kLanes, 0, row0 + lo + k * U - 1);
    };
    if (lane == 0)
        for (int k = 0; k < NST && k < n_chunks; ++k) issue(k);
    float r4[4] = {0.f, 0.f, 0.f, 0.f};
    if (HAS_H) {
#pragma unroll
        for (int q = 0; q < 4; ++q) r4[q] = __ldg(a.r + (size_t)q * d + chl);
    }
    float mp[4] = {0.f, -CUDART_INF_F, 0.f, 0.f};
    bool timed_out = false;
    for (int k = 0; k < n_chunks; ++k) {
        if (!ring.wait(k, timed_out)) timed_out = true;
        const TIO* t_wx = reinterpret_cast<const TIO*>(ring.stage(k));
        const float* t_h = reinterpret_cast<const float*>(ring.stage(k) + S::WX);
        // chunks that lie fully inside the warp's range take a variant without range checks
        auto chunk_body = [&](auto full_c) {
            constexpr bool FULL = decltype(full_c)::value;
    #pragma unroll
            for (int i = 0; i < U; ++i) {
                const int t = lo + k * U + i;
                if (FULL || t < hi) {
                    float hp = 0.f;
                    if (HAS_H)
                        hp = (t == 0) ? (a.h_halo ? __ldg(a.h_halo + (size_t)b * a.halo_stride + chl) : 0.f)
                                      : t_h[i * kLanes + lane];
                    const float zi = fmaf(r4[0], hp, (float)t_wx[(i * 4 + 0) * kLanes + lane]);
                    const float zf = fmaf(r4[1], hp, (float)t_wx[(i * 4 + 1) * kLanes + lane]);
                    const float zz = tanh_f(fmaf(r4[2], hp, (float)t_wx[(i * 4 + 2) * kLanes + lane]));
                    const float b1a = mp[1] + zf;
                    const float e = exp_f(-fabsf(b1a - zi));
                    const bool left = b1a >= zi;
                    const float s1 = left ? 1.f : e, s2 = left ? e : 1.f;
                    mp[0] += zf;
                    mp[1] = left ? b1a : zi;
                    mp[2] = fmaf(mp[2], s1, s2);
                    mp[3] = fmaf(mp[3], s1, s2 * zz);
                }
            }
        };
        if (lo + (k + 1) * U <= hi)
            chunk_body(std::true_type{});
        else
            chunk_body(std::false_type{});
        __syncwarp();
        if (lane == 0 && k + NST < n_chunks) {
            fence_proxy_async();
            issue(k + NST);
        }
    }
    if (timed_out) atomicExch(a.chain.status, (int)kErrChainTimeout);
    if (lane == 0 && timed_out) drain_ring(ring.bars, NST, n_chunks, kDrainLimit);
    finish_agg<PicardMonoid>(reinterpret_cast<float*>(smem + S::MAPS_OFF), mp, warp, lane,
                             a.agg_out + (size_t)sg.seg * a.B * 4 * d, b, d, ch, ch_ok);
}

// ------------------------------------------------------------------ backward
// Reverse direction: warp 0 owns the LAST eighth of the shard; map of a step is
// nu -> J_t^T (nu + g_t).  Chunk k of a warp covers steps [hi - (k+1)U, hi - kU).
template <typename TIO, int U, int NST>
struct AggBwdSmem {
    static constexpr int WX = U * 4 * kLanes * (int)sizeof(TIO);
    static constexpr int STAGE = 3 * WX;
    static constexpr int RING = NST * STAGE;
    static constexpr int MAPS_OFF = kAggW * RING;
    static constexpr int BAR_OFF = MAPS_OFF + kAggW * 20 * kLanes * 4;
    static constexpr int TOTAL = BAR_OFF + kAggW * NST * 8 + 64;
};

template <typename TIO, int U, int NST>
__global__ void __launch_bounds__(kAggW * 32, 2)
slstm_bwd_agg_seg_kernel(const __grid_constant__ CUtensorMap tm_wx, const __grid_constant__ CUtensorMap tm_st,
                         const __grid_constant__ CUtensorMap tm_g, SlstmBwdArgs a) {
    using S = AggBwdSmem<TIO, U, NST>;
    extern __shared__ __align__(128) unsigned char smem[];
    const int d = a.d;
    const int ncb = (d + kLanes - 1) / kLanes;
    const int b = blockIdx.x / ncb, cb = blockIdx.x % ncb;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ch = cb * kLanes + lane;
    const bool ch_ok = ch < d;
    const int chl = ch_ok ? ch : d - 1;
    const SegRange sg = seg_range(a.T, a.n_seg, a.seg_len);
    int lo, hi;
    seg_bounds(sg.lo, sg.hi, kAggW - 1 - warp, lo, hi);
    WarpRing<NST> ring;
    ring.init(smem + warp * S::RING, reinterpret_cast<uint64_t*>(smem + S::BAR_OFF) + warp * NST, S::STAGE, lane);
    const int n_chunks = (hi - lo + U - 1) / U;
    const int row0 = b * a.T;
    auto issue = [&](int k) {
        unsigned char* st = ring.stage(k);
        const int t_first = hi - (k + 1) * U;  // may be below lo (or negative): masked later
        mbar_expect_tx(&ring.bars[k % NST], S::STAGE);
        tma_load_3d(st, &tm_wx, &ring.bars[k % NST], cb * kLanes, 0, row0 + t_first);
        tma_load_3d(st + S::WX, &tm_st, &ring.bars[k % NST], cb * kLanes, 0, row0 + t_first - 1);
        tma_load_3d(st + 2 * S::WX, &tm_g, &ring.bars[k % NST], cb * kLanes, 0, row0 + t_first);
    };
    if (lane == 0)
        for (int k = 0; k < NST && k < n_chunks; ++k) issue(k);
    float r4[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) r4[q] = __ldg(a.r + (size_t)q * d + chl);
    float mp[20];
#pragma unroll
    for (int k = 0; k < 20; ++k) mp[k] = 0.f;
    mp[0] = mp[5] = mp[10] = mp[15] = 1.f;
    bool timed_out = false;
    for (int k = 0; k < n_chunks; ++k) {
        if (!ring.wait(k, timed_out)) timed_out = true;
        const TIO* t_wx = reinterpret_cast<const TIO*>(ring.stage(k));
        const TIO* t_st = reinterpret_cast<const TIO*>(ring.stage(k) + S::WX);
        const TIO* t_g = reinterpret_cast<const TIO*>(ring.stage(k) + 2 * S::WX);
        const int t_first = hi - (k + 1) * U;
#pragma unroll
        for (int i = U - 1; i >= 0; --i) {
            const int t = t_first + i;
            if (t >= lo) {
                float w[4], prev[4], g[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    w[q] = (float)t_wx[(i * 4 + q) * kLanes + lane];
                    g[q] = (float)t_g[(i * 4 + q) * kLanes + lane];
                    prev[q] = (t == 0) ? (a.halo ? __ldg(a.halo + (size_t)b * a.halo_stride + (size_t)q * d + chl) : 0.f)
                                       : (float)t_st[(i * 4 + q) * kLanes + lane];
                }
                SlstmLin lin;
                slstm_linearize(prev, w, r4, a.eps, lin);
#pragma unroll
                for (int c2 = 0; c2 < 4; c2 += 2) {
                    float2 xc = make_float2(mp[0 * 4 + c2], mp[0 * 4 + c2 + 1]);
                    float2 xn = make_float2(mp[1 * 4 + c2], mp[1 * 4 + c2 + 1]);
                    float2 xm = make_float2(mp[2 * 4 + c2], mp[2 * 4 + c2 + 1]);
                    float2 xh = make_float2(mp[3 * 4 + c2], mp[3 * 4 + c2 + 1]);
                    slstm_apply_t_cols2(lin, xc, xn, xm, xh);
                    mp[0 * 4 + c2] = xc.x; mp[0 * 4 + c2 + 1] = xc.y;
                    mp[1 * 4 + c2] = xn.x; mp[1 * 4 + c2 + 1] = xn.y;
                    mp[2 * 4 + c2] = xm.x; mp[2 * 4 + c2 + 1] = xm.y;
                    mp[3 * 4 + c2] = xh.x; mp[3 * 4 + c2 + 1] = xh.y;
                }
                {
                    float xc = mp[16] + g[0], xn = mp[17] + g[1], xm = mp[18] + g[2], xh = mp[19] + g[3];
                    slstm_apply_t(lin, xc, xn, xm, xh);
                    mp[16] = xc; mp[17] = xn; mp[18] = xm; mp[19] = xh;
                }
            }
        }
        __syncwarp();
        if (lane == 0 && k + NST < n_chunks) {
            fence_proxy_async();
            issue(k + NST);
        }
    }
    if (timed_out) atomicExch(a.chain.status, (int)kErrChainTimeout);
    if (lane == 0 && timed_out) drain_ring(ring.bars, NST, n_chunks, kDrainLimit);
    finish_agg<Affine4>(reinterpret_cast<float*>(smem + S::MAPS_OFF), mp, warp, lane,
                        a.agg_out + (size_t)sg.seg * a.B * 20 * d, b, d, ch, ch_ok);
}

// ------------------------------------------------------------------ launchers
template <typename TIO>
static cudaError_t agg_newton_t(const SlstmNewtonArgs& a, cudaStream_t s) {
    constexpr int U = 4, NST = sizeof(TIO) == 2 ? 3 : 2;  // two CTAs per SM
    using S = AggNewtonSmem<TIO, U, NST>;
    CUtensorMap tm_wx, tm_st;
    const uint64_t rows = (uint64_t)a.B * a.T;
    if (!make_tile_map(&tm_wx, a.wx, sizeof(TIO), rows, 4, a.d, U) ||
        !make_tile_map(&tm_st, a.sin, 4, rows, 4, a.d, U))
        return cudaErrorNotSupported;
    auto k = slstm_newton_agg_seg_kernel<TIO, U, NST>;
    cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
    k<<<dim3(a.B * ((a.d + kLanes - 1) / kLanes), a.n_seg > 1 ? a.n_seg : 1), kAggW * 32, S::TOTAL, s>>>(tm_wx, tm_st, a);
    return cudaGetLastError();
}
cudaError_t launch_slstm_newton_agg_seg(int dtype, const SlstmNewtonArgs& a, cudaStream_t s) {
    return dtype == kF32 ? agg_newton_t<float>(a, s) : agg_newton_t<__nv_bfloat16>(a, s);
}

template <typename TIO>
static cudaError_t agg_picard_t(const SlstmPicardArgs& a, cudaStream_t s) {
    constexpr int U = 8, NST = sizeof(TIO) == 2 ? 4 : 2;
    using S = AggPicardSmem<TIO, U, NST>;
    CUtensorMap tm_wx, tm_h;
    const uint64_t rows = (uint64_t)a.B * a.T;
    if (!make_tile_map(&tm_wx, a.wx, sizeof(TIO), rows, 4, a.d, U)) return cudaErrorNotSupported;
    const dim3 grid(a.B * ((a.d + kLanes - 1) / kLanes), a.n_seg > 1 ? a.n_seg : 1);
    if (a.h_prev) {
        if (!make_tile_map(&tm_h, a.h_prev, 4, rows, 1, a.d, U)) return cudaErrorNotSupported;
        auto k = slstm_picard_agg_seg_kernel<TIO, U, NST, true>;
        cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
        k<<<grid, kAggW * 32, S::TOTAL, s>>>(tm_wx, tm_h, a);
    } else {
        auto k = slstm_picard_agg_seg_kernel<TIO, U, NST, false>;
        cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
        k<<<grid, kAggW * 32, S::TOTAL, s>>>(tm_wx, tm_wx, a);
    }
    return cudaGetLastError();
}
cudaError_t launch_slstm_picard_agg_seg(int dtype, const SlstmPicardArgs& a, cudaStream_t s) {
    return dtype == kF32 ? agg_picard_t<float>(a, s) : agg_picard_t<__nv_bfloat16>(a, s);
}

template <typename TIO>
static cudaError_t agg_bwd_t(const SlstmBwdArgs& a, cudaStream_t s) {
    constexpr int U = 4, NST = sizeof(TIO) == 2 ? 3 : 2;
    using S = AggBwdSmem<TIO, U, NST>;
    CUtensorMap tm_wx, tm_st, tm_g;
    const uint64_t rows = (uint64_t)a.B * a.T;
    if (!make_tile_map(&tm_wx, a.wx, sizeof(TIO), rows, 4, a.d, U) ||
        !make_tile_map(&tm_st, a.states, sizeof(TIO), rows, 4, a.d, U) ||
        !make_tile_map(&tm_g, a.grad_states, sizeof(TIO), rows, 4, a.d, U))
        return cudaErrorNotSupported;
    auto k = slstm_bwd_agg_seg_kernel<TIO, U, NST>;
    cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
    k<<<dim3(a.B * ((a.d + kLanes - 1) / kLanes), a.n_seg > 1 ? a.n_seg : 1), kAggW * 32, S::TOTAL, s>>>(tm_wx, tm_st, tm_g, a);
    return cudaGetLastError();
}
cudaError_t launch_slstm_bwd_agg_seg(int dtype, const SlstmBwdArgs& a, cudaStream_t s) {
    return dtype == kF32 ? agg_bwd_t<float>(a, s) : agg_bwd_t<__nv_bfloat16>(a, s);
}

}  // namespace prb
