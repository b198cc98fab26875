// Shared device helpers: I/O dtype conversion, gate math, the NaN-propagating
// residual max, and the single-pass chained scan protocol used by every
// time-scan kernel in this library.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

namespace prb {

constexpr int kLanes = 32;         // channels per CTA tile (one per lane)
constexpr int kMaxIters = 16;      // residual_history capacity
constexpr unsigned kStA = 1u;      // tile aggregate published
constexpr unsigned kStP = 2u;      // tile inclusive carry published
constexpr int kLookbackDepth = 12; // max aggregates folded in one look-back
constexpr unsigned kSpinLimit = 1u << 22;

enum Status : int {
    kOk = 0,
    kErrBadArg = -1,
    kErrWorkspace = -2,
    kErrUnsupported = -3,
    kErrLaunch = -4,
    kErrTooLarge = -5,
    kErrChainTimeout = 1,  // device side: a bounded look-back wait ran out
};

// Device-resident statistics block written by the forward kernels.
struct DeviceStats {
    unsigned hist_bits[kMaxIters];  // max|F(H^k)| as IEEE bits (NaN sorts highest)
    unsigned final_bits;            // max|F(H^K)|
    int status;                     // 0 or kErrChainTimeout
    int reserved[2];
};

// Time segment of a CTA: blockIdx.y selects one of n_seg contiguous pieces of the time axis.
struct SegRange {
    int seg, lo, hi;
};
__device__ __forceinline__ SegRange seg_range(int T, int n_seg, int seg_len) {
    SegRange s;
    if (n_seg <= 1) {
        s.seg = 0;
        s.lo = 0;
        s.hi = T;
    } else {
        s.seg = blockIdx.y;
        s.lo = min(T, s.seg * seg_len);
        s.hi = min(T, s.lo + seg_len);
    }
    return s;
}

// ---------------------------------------------------------------- I/O dtype
template <typename T>
__device__ __forceinline__ float ld_f(const T* p);
template <>
__device__ __forceinline__ float ld_f<float>(const float* p) {
    return __ldg(p);
}
template <>
__device__ __forceinline__ float ld_f<__nv_bfloat16>(const __nv_bfloat16* p) {
    return __bfloat162float(__ldg(p));
}
template <typename T>
__device__ __forceinline__ void st_f(T* p, float v);
template <>
__device__ __forceinline__ void st_f<float>(float* p, float v) {
    *p = v;
}
template <>
__device__ __forceinline__ void st_f<__nv_bfloat16>(__nv_bfloat16* p, float v) {
    *p = __float2bfloat16_rn(v);
}

// ---------------------------------------------------------------- math
// exp, reciprocal, sigmoid and tanh built on the SFU approximations (ex2.approx, rcp.approx,
// each accurate to about 1-2 ulp) with the argument reduction of exp carried in two floats, so
// that the result stays within ~3e-7 relative of the correctly rounded value at a third of the
// instruction count of the libm versions.  NaN propagates; arguments below -88 give 0.
__device__ __forceinline__ float ex2_approx(float x) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ float rcp_f(float x) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ float exp_f(float x) {
    x = x < -88.f ? -88.f : x;  // a select, not fmaxf: NaN must survive
    const float kL2E = 1.4426950216293335f;      // float(log2 e)
    const float kL2E_LO = 1.9259629911e-8f;      // log2 e - float(log2 e)
    const float hi = x * kL2E;
    float lo = fmaf(x, kL2E, -hi);
    lo = fmaf(x, kL2E_LO, lo);
    const float r = ex2_approx(hi);
    return fmaf(r, lo * 0.6931471805599453f, r);
}
// In sigmoid and tanh the exponential's argument error is damped by the function's own
// derivative (|x| (1 - tanh^2 x) <= 0.45), so the plain ex2(x * log2 e) is accurate enough there:
// absolute error stays below ~2e-7.  ex2(-inf) = 0 and NaN propagates, no clamp needed.
__device__ __forceinline__ float sigmoid_f(float x) {
    return rcp_f(1.0f + ex2_approx(-1.4426950216293335f * x));
}
__device__ __forceinline__ float tanh_f(float x) {
    return fmaf(-2.0f, rcp_f(ex2_approx(2.885390043258667f * x) + 1.0f), 1.0f);
}
// ---- packed fp32 (fma.rn.f32x2 family, sm_100): two independent time steps per instruction for
// the add / multiply / fma part of the math; the SFU ops stay one per lane.  Each lane computes
// exactly what the scalar function above computes (same operations, same rounding).
__device__ __forceinline__ float2 splat2(float x) { return make_float2(x, x); }
__device__ __forceinline__ float2 ex2_2(float2 v) { return make_float2(ex2_approx(v.x), ex2_approx(v.y)); }
__device__ __forceinline__ float2 rcp_2(float2 v) { return make_float2(rcp_f(v.x), rcp_f(v.y)); }
__device__ __forceinline__ float2 tanh_f2(float2 x) {
    const float2 t = ex2_2(__fmul2_rn(x, splat2(2.885390043258667f)));
    return __ffma2_rn(splat2(-2.0f), rcp_2(__fadd2_rn(t, splat2(1.0f))), splat2(1.0f));
}
__device__ __forceinline__ float2 exp_f2(float2 x) {
    x.x = x.x < -88.f ? -88.f : x.x;
    x.y = x.y < -88.f ? -88.f : x.y;
    const float kL2E = 1.4426950216293335f, kL2E_LO = 1.9259629911e-8f;
    const float2 hi = __fmul2_rn(x, splat2(kL2E));
    const float2 nhi = __fmul2_rn(x, splat2(-kL2E));  // = -hi exactly
    float2 lo = __ffma2_rn(x, splat2(kL2E), nhi);
    lo = __ffma2_rn(x, splat2(kL2E_LO), lo);
    const float2 r = ex2_2(hi);
    return __ffma2_rn(r, __fmul2_rn(lo, splat2(0.6931471805599453f)), r);
}
__device__ __forceinline__ unsigned absbits(float v) { return __float_as_uint(v) & 0x7fffffffu; }

// Block-wide max of |F| bit patterns, then one atomicMax into global memory.
// Comparing the bit patterns as integers orders finite < inf < NaN, so a NaN
// residual wins the maximum exactly like torch.amax.
__device__ __forceinline__ void block_residual_max(unsigned v, unsigned* dst, unsigned* smem_red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = max(v, __shfl_xor_sync(0xffffffffu, v, o));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    if (lane == 0) smem_red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        v = lane < nw ? smem_red[lane] : 0u;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v = max(v, __shfl_xor_sync(0xffffffffu, v, o));
        if (lane == 0 && v != 0u) atomicMax(dst, v);
    }
}

// ---------------------------------------------------------------- chained scan
//
// A scan pass covers `n_chains` independent chains (batch row x block of 32
// channels); each chain is cut into `n_tt` time tiles processed by one CTA each.
// CTAs take a ticket from an atomic counter; tickets are time-major, so every
// predecessor of a tile has started before the tile itself and waiting on it
// cannot deadlock.  A tile publishes its aggregate map (state A) as soon as it
// is known and its inclusive carry (state P) once its own carry-in is known.
// A waiting tile walks back to the nearest P, then folds the aggregates in
// between (decoupled look-back).  Every spin is bounded; on time-out the
// kernel records kErrChainTimeout and carries on with a zero carry so that the
// launch always terminates.
struct Chain {
    unsigned* flags;   // [n_chains * n_tt]
    float* agg;        // [n_chains * n_tt][NV][32]
    float* inc;        // [n_chains * n_tt][NS][32]
    unsigned* ticket;  // one counter, zero at launch
    int* status;       // device status word
    unsigned epoch;    // distinguishes passes that share the flag array
    unsigned spin_limit;  // polls after which a look-back wait gives up
    int n_chains;
    int n_tt;
};

__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_u32(unsigned* p, unsigned v) {
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Returns the ticket of this CTA (broadcast through shared memory).
__device__ __forceinline__ unsigned take_ticket(unsigned* counter, unsigned* smem_slot) {
    if (threadIdx.x == 0) *smem_slot = atomicAdd(counter, 1u);
    __syncthreads();
    unsigned t = *smem_slot;
    __syncthreads();
    return t;
}

template <int N>
__device__ __forceinline__ void chain_publish(const Chain& c, float* base, size_t tile, int lane,
                                              const float (&v)[N], unsigned state) {
    float* p = base + tile * (size_t)(N * kLanes) + lane;
#pragma unroll
    for (int i = 0; i < N; ++i) __stcg(p + i * kLanes, v[i]);
    __threadfence();
    __syncwarp();
    if (lane == 0) st_release_u32(c.flags + tile, (c.epoch << 2) | state);
}

// Monoid concept used below:
//   static constexpr int NV, NS;
//   static void compose(float (&acc)[NV], const float (&next)[NV]);   acc = next o acc
//   static void apply(const float (&map)[NV], float (&vec)[NS]);      vec = map(vec)
//
// Called by warp 0 only (all lanes converged).  `tile0` is the flat index of the
// chain's first tile; `tt` counts tiles in scan direction.  On return `vec`
// holds the carry entering tile `tt` for this lane's channel.
template <class M>
__device__ __forceinline__ void chain_lookback(const Chain& c, size_t tile0, int tt, int lane,
                                               float (&vec)[M::NS]) {
    int k = tt - 1;
    unsigned spins = 0;
    bool ok = true;
    while (true) {
        unsigned f = ld_acquire_u32(c.flags + tile0 + k);
        unsigned st = ((f >> 2) == c.epoch) ? (f & 3u) : 0u;
        if (st == kStP) break;
        if (st == kStA && k > 0 && (tt - 1 - k) < kLookbackDepth) {
            --k;
            continue;
        }
        if (++spins > c.spin_limit) {
            ok = false;
            break;
        }
        __nanosleep(40);
    }
    if (!ok) {
        if (lane == 0) atomicExch(c.status, (int)kErrChainTimeout);
#pragma unroll
        for (int i = 0; i < M::NS; ++i) vec[i] = 0.f;
        return;
    }
    {
        const float* p = c.inc + (tile0 + k) * (size_t)(M::NS * kLanes) + lane;
#pragma unroll
        for (int i = 0; i < M::NS; ++i) vec[i] = __ldcg(p + i * kLanes);
    }
    for (int j = k + 1; j < tt; ++j) {
        float m[M::NV];
        const float* p = c.agg + (tile0 + j) * (size_t)(M::NV * kLanes) + lane;
#pragma unroll
        for (int i = 0; i < M::NV; ++i) m[i] = __ldcg(p + i * kLanes);
        M::apply(m, vec);
    }
}

// Middle phase of a tile: combine the W per-warp sub-tile maps, exchange with
// the neighbouring tiles, and hand every thread the carry entering its own
// sub-tile.  `smem` needs (W*NV + NS) * 32 floats.  `boundary` is the carry
// entering the chain's first tile.  Returns (in `tile_end`, warp 0 only) the
// inclusive carry leaving this tile.
template <class M, int W>
__device__ __forceinline__ void tile_exchange(const Chain& c, int chain_idx, int tt,
                                              const float (&my_map)[M::NV],
                                              const float (&boundary)[M::NS],
                                              float (&carry)[M::NS], float* smem,
                                              float (&tile_end)[M::NS]) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* s_map = smem;                        // [W][NV][32]
    float* s_vec = smem + W * M::NV * kLanes;   // [NS][32]
#pragma unroll
    for (int i = 0; i < M::NV; ++i) s_map[(warp * M::NV + i) * kLanes + lane] = my_map[i];
    __syncthreads();
    if (warp == 0) {
        float acc[M::NV];
#pragma unroll
        for (int i = 0; i < M::NV; ++i) acc[i] = my_map[i];
#pragma unroll
        for (int w = 1; w < W; ++w) {
            float m[M::NV];
#pragma unroll
            for (int i = 0; i < M::NV; ++i) m[i] = s_map[(w * M::NV + i) * kLanes + lane];
            M::compose(acc, m);
#pragma unroll
            for (int i = 0; i < M::NV; ++i) s_map[(w * M::NV + i) * kLanes + lane] = acc[i];
        }
        const size_t tile0 = (size_t)chain_idx * c.n_tt;
        float vec[M::NS];
        if (tt == 0) {
#pragma unroll
            for (int i = 0; i < M::NS; ++i) vec[i] = boundary[i];
        } else {
            if (tt + 1 < c.n_tt) chain_publish<M::NV>(c, c.agg, tile0 + tt, lane, acc, kStA);
            chain_lookback<M>(c, tile0, tt, lane, vec);
        }
#pragma unroll
        for (int i = 0; i < M::NS; ++i) {
            s_vec[i * kLanes + lane] = vec[i];
            tile_end[i] = vec[i];
        }
        M::apply(acc, tile_end);
        if (tt + 1 < c.n_tt) chain_publish<M::NS>(c, c.inc, tile0 + tt, lane, tile_end, kStP);
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < M::NS; ++i) carry[i] = s_vec[i * kLanes + lane];
    if (warp > 0) {
        float m[M::NV];
#pragma unroll
        for (int i = 0; i < M::NV; ++i) m[i] = s_map[((warp - 1) * M::NV + i) * kLanes + lane];
        M::apply(m, carry);
    }
}

// Scalar affine monoid x -> a*x + b  (diagonal-Jacobian cells).
struct Affine1 {
    static constexpr int NV = 2, NS = 1;
    __device__ static __forceinline__ void compose(float (&acc)[2], const float (&nx)[2]) {
        acc[1] = fmaf(nx[0], acc[1], nx[1]);
        acc[0] = nx[0] * acc[0];
    }
    __device__ static __forceinline__ void apply(const float (&m)[2], float (&v)[1]) {
        v[0] = fmaf(m[0], v[0], m[1]);
    }
};

// 2x2 affine monoid x -> M x + v, M row-major in [0,4), v in [4,6) (ParaLSTM, state (c, h)).
struct Affine2 {
    static constexpr int NV = 6, NS = 2;
    __device__ static __forceinline__ void compose(float (&acc)[6], const float (&nx)[6]) {
        const float m00 = fmaf(nx[0], acc[0], nx[1] * acc[2]), m01 = fmaf(nx[0], acc[1], nx[1] * acc[3]);
        const float m10 = fmaf(nx[2], acc[0], nx[3] * acc[2]), m11 = fmaf(nx[2], acc[1], nx[3] * acc[3]);
        const float v0 = fmaf(nx[0], acc[4], fmaf(nx[1], acc[5], nx[4]));
        const float v1 = fmaf(nx[2], acc[4], fmaf(nx[3], acc[5], nx[5]));
        acc[0] = m00; acc[1] = m01; acc[2] = m10; acc[3] = m11; acc[4] = v0; acc[5] = v1;
    }
    __device__ static __forceinline__ void apply(const float (&m)[6], float (&v)[2]) {
        const float a = fmaf(m[0], v[0], fmaf(m[1], v[1], m[4]));
        const float b = fmaf(m[2], v[0], fmaf(m[3], v[1], m[5]));
        v[0] = a;
        v[1] = b;
    }
};

// 4x4 affine monoid x -> M x + v, M row-major in [0,16), v in [16,20).
struct Affine4 {
    static constexpr int NV = 20, NS = 4;
    __device__ static __forceinline__ void compose(float (&acc)[20], const float (&nx)[20]) {
        float r[20];
#pragma unroll
        for (int o = 0; o < 4; ++o) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                float s = nx[o * 4 + 0] * acc[0 * 4 + i];
                s = fmaf(nx[o * 4 + 1], acc[1 * 4 + i], s);
                s = fmaf(nx[o * 4 + 2], acc[2 * 4 + i], s);
                s = fmaf(nx[o * 4 + 3], acc[3 * 4 + i], s);
                r[o * 4 + i] = s;
            }
            float s = nx[16 + o];
            s = fmaf(nx[o * 4 + 0], acc[16 + 0], s);
            s = fmaf(nx[o * 4 + 1], acc[16 + 1], s);
            s = fmaf(nx[o * 4 + 2], acc[16 + 2], s);
            s = fmaf(nx[o * 4 + 3], acc[16 + 3], s);
            r[16 + o] = s;
        }
#pragma unroll
        for (int i = 0; i < 20; ++i) acc[i] = r[i];
    }
    __device__ static __forceinline__ void apply(const float (&m)[20], float (&v)[4]) {
        float r[4];
#pragma unroll
        for (int o = 0; o < 4; ++o) {
            float s = m[16 + o];
            s = fmaf(m[o * 4 + 0], v[0], s);
            s = fmaf(m[o * 4 + 1], v[1], s);
            s = fmaf(m[o * 4 + 2], v[2], s);
            s = fmaf(m[o * 4 + 3], v[3], s);
            r[o] = s;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) v[i] = r[i];
    }
};

// Summary monoid of the sLSTM frozen-gate (Picard) recurrence.
// Frozen-gate recurrence on (c, n, m):  m' = max(zf + m, zi),
// n' = exp(zf + m - m') n + exp(zi - m'),  c' likewise with tanh(zz).
// A run of steps is summarised by (a, b, N, C):
//   m_out = max(a + m_in, b)
//   n_out = exp(a + m_in - m_out) n_in + exp(b - m_out) N      (c likewise with C)
// with a = sum zf, b = max_s (zi_s + sum_{r>s} zf_r) and N, C normalised to b.
struct PicardMonoid {
    static constexpr int NV = 4, NS = 3;  // map (a,b,N,C); vec (c,n,m)
    __device__ static __forceinline__ void compose(float (&acc)[4], const float (&nx)[4]) {
        const float b1a = acc[1] + nx[0];
        const float b = fmaxf(b1a, nx[1]);
        const float s1 = (b1a > -CUDART_INF_F) ? exp_f(b1a - b) : 0.f;
        const float s2 = (nx[1] > -CUDART_INF_F) ? exp_f(nx[1] - b) : 0.f;
        acc[0] += nx[0];
        acc[1] = b;
        acc[2] = acc[2] * s1 + nx[2] * s2;
        acc[3] = acc[3] * s1 + nx[3] * s2;
    }
    __device__ static __forceinline__ void apply(const float (&m)[4], float (&v)[3]) {
        const float am = m[0] + v[2];
        const float mo = fmaxf(am, m[1]);
        const float s1 = exp_f(am - mo);
        const float s2 = (m[1] > -CUDART_INF_F) ? exp_f(m[1] - mo) : 0.f;
        v[0] = v[0] * s1 + m[3] * s2;
        v[1] = v[1] * s1 + m[2] * s2;
        v[2] = mo;
    }
};

// A chain whose carry is itself a map: used to obtain the aggregate of a whole
// time shard (the carry entering the shard is not known yet).
template <class M>
struct MapCarry {
    static constexpr int NV = M::NV, NS = M::NV;
    __device__ static __forceinline__ void compose(float (&acc)[NV], const float (&nx)[NV]) {
        M::compose(acc, nx);
    }
    __device__ static __forceinline__ void apply(const float (&m)[NV], float (&v)[NV]) {
        M::compose(v, m);
    }
};

}  // namespace prb
