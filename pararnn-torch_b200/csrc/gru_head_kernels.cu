// ParaGRU mix='head': per-head dense recurrence (row-vector convention y = h A, A (d_in, d_out)).
//
//   z = sigmoid(h A_z + z_x),  r = sigmoid(h A_r + r_x),  n = tanh((h*r) A_n + n_x),
//   f = h + z (n - h)
//   J d   = (1-z) d + (n-h) z' (d A_z) + z n' ((r d + h r' (d A_r)) A_n)
//   J^T m = (1-z) m + A_z (z'(n-h) m) + r g + A_r (r' h g),   g = A_n (n' z m)
//
// Reference restated: cells/para_gru.py:385-412 and :468-479 (step, dense J),
// kernels/gru_head_factor.py:31-112 (factorised J d and J^T m),
// kernels/vjp_gru.py:141-221 (packed VJP), kernels/newton_gru_head.py:460-652 (the
// reference's sequential-in-time Newton and reverse walks).
//
// Forward kernel: one CTA per (batch row, head).  The K Newton iterations run as a skewed
// software pipeline over ONE sweep of the time axis: stage s handles time step tick - s, so at
// every tick all stages work in parallel (stage s+1 linearises around the trajectory stage s
// produced one tick earlier).  A stage is a group of 64 threads; thread o keeps column o of
// A_z, A_r, A_n in registers, the vectors being multiplied are broadcast from shared memory.
// An optional last stage evaluates the residual of the final trajectory.  No intermediate
// trajectory touches HBM.
#include "common.cuh"
#include "kernels.h"

namespace prb {

constexpr int kHG = 64;  // threads per stage group

// Raw loads for the prefetch rings: the conversion to float happens where the value is used, so
// that nothing waits on the load at the point where it is issued.
__device__ __forceinline__ float raw_f(float v) { return v; }
__device__ __forceinline__ float raw_f(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T>
__device__ __forceinline__ T raw_zero();
template <>
__device__ __forceinline__ float raw_zero<float>() { return 0.f; }
template <>
__device__ __forceinline__ __nv_bfloat16 raw_zero<__nv_bfloat16>() { return __ushort_as_bfloat16(0); }

__device__ __forceinline__ void stage_bar(int id) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(kHG) : "memory");
}

// Dot products of broadcast vectors (shared memory) with register-resident columns.  The
// products run on packed fp32 FMAs (fma.rn.f32x2: two lanes per instruction, sm_100), pairing
// consecutive elements; every product keeps two packed accumulators, i.e. four partial sums,
// because with one warp per scheduler the latency of a dependent FMA chain, not the issue rate,
// sets the pace.
__device__ __forceinline__ float hsum2(float2 a, float2 b) { return (a.x + a.y) + (b.x + b.y); }

template <int DH>
__device__ __forceinline__ void dot2x2(const float* va, const float* vb, const float (&c0)[DH],
                                       const float (&c1)[DH], float& a0, float& a1, float& b0, float& b1) {
    float2 pa0[2] = {{0.f, 0.f}, {0.f, 0.f}}, pa1[2] = {{0.f, 0.f}, {0.f, 0.f}};
    float2 pb0[2] = {{0.f, 0.f}, {0.f, 0.f}}, pb1[2] = {{0.f, 0.f}, {0.f, 0.f}};
#pragma unroll
    for (int i = 0; i < DH; i += 4) {
        const float4 x = *reinterpret_cast<const float4*>(va + i);
        const float4 y = *reinterpret_cast<const float4*>(vb + i);
        const float2 xs[2] = {{x.x, x.y}, {x.z, x.w}}, ys[2] = {{y.x, y.y}, {y.z, y.w}};
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const float2 k0 = make_float2(c0[i + 2 * k], c0[i + 2 * k + 1]);
            const float2 k1 = make_float2(c1[i + 2 * k], c1[i + 2 * k + 1]);
            pa0[k] = __ffma2_rn(xs[k], k0, pa0[k]);
            pa1[k] = __ffma2_rn(xs[k], k1, pa1[k]);
            pb0[k] = __ffma2_rn(ys[k], k0, pb0[k]);
            pb1[k] = __ffma2_rn(ys[k], k1, pb1[k]);
        }
    }
    a0 = hsum2(pa0[0], pa0[1]);
    a1 = hsum2(pa1[0], pa1[1]);
    b0 = hsum2(pb0[0], pb0[1]);
    b1 = hsum2(pb1[0], pb1[1]);
}
template <int DH>
__device__ __forceinline__ void dot2x1(const float* va, const float* vb, const float (&c)[DH], float& a,
                                       float& b) {
    float2 pa[2] = {{0.f, 0.f}, {0.f, 0.f}}, pb[2] = {{0.f, 0.f}, {0.f, 0.f}};
#pragma unroll
    for (int i = 0; i < DH; i += 4) {
        const float4 x = *reinterpret_cast<const float4*>(va + i);
        const float4 y = *reinterpret_cast<const float4*>(vb + i);
        const float2 xs[2] = {{x.x, x.y}, {x.z, x.w}}, ys[2] = {{y.x, y.y}, {y.z, y.w}};
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const float2 kk = make_float2(c[i + 2 * k], c[i + 2 * k + 1]);
            pa[k] = __ffma2_rn(xs[k], kk, pa[k]);
            pb[k] = __ffma2_rn(ys[k], kk, pb[k]);
        }
    }
    a = hsum2(pa[0], pa[1]);
    b = hsum2(pb[0], pb[1]);
}
// two products with two different row sets (reverse kernel)
template <int DH>
__device__ __forceinline__ void dot1x1x2(const float* va, const float* vb, const float (&c0)[DH],
                                         const float (&c1)[DH], float& a, float& b) {
    float2 pa[2] = {{0.f, 0.f}, {0.f, 0.f}}, pb[2] = {{0.f, 0.f}, {0.f, 0.f}};
#pragma unroll
    for (int i = 0; i < DH; i += 4) {
        const float4 x = *reinterpret_cast<const float4*>(va + i);
        const float4 y = *reinterpret_cast<const float4*>(vb + i);
        const float2 xs[2] = {{x.x, x.y}, {x.z, x.w}}, ys[2] = {{y.x, y.y}, {y.z, y.w}};
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            pa[k] = __ffma2_rn(xs[k], make_float2(c0[i + 2 * k], c0[i + 2 * k + 1]), pa[k]);
            pb[k] = __ffma2_rn(ys[k], make_float2(c1[i + 2 * k], c1[i + 2 * k + 1]), pb[k]);
        }
    }
    a = hsum2(pa[0], pa[1]);
    b = hsum2(pb[0], pb[1]);
}
// one broadcast vector against two / one register-resident columns
template <int DH>
__device__ __forceinline__ void dot1x2(const float* va, const float (&c0)[DH], const float (&c1)[DH],
                                       float& a0, float& a1) {
    float2 p0[2] = {{0.f, 0.f}, {0.f, 0.f}}, p1[2] = {{0.f, 0.f}, {0.f, 0.f}};
#pragma unroll
    for (int i = 0; i < DH; i += 4) {
        const float4 x = *reinterpret_cast<const float4*>(va + i);
        const float2 xs[2] = {{x.x, x.y}, {x.z, x.w}};
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            p0[k] = __ffma2_rn(xs[k], make_float2(c0[i + 2 * k], c0[i + 2 * k + 1]), p0[k]);
            p1[k] = __ffma2_rn(xs[k], make_float2(c1[i + 2 * k], c1[i + 2 * k + 1]), p1[k]);
        }
    }
    a0 = hsum2(p0[0], p0[1]);
    a1 = hsum2(p1[0], p1[1]);
}
template <int DH>
__device__ __forceinline__ float dot1x1(const float* va, const float (&c)[DH]) {
    float2 p[2] = {{0.f, 0.f}, {0.f, 0.f}};
#pragma unroll
    for (int i = 0; i < DH; i += 4) {
        const float4 x = *reinterpret_cast<const float4*>(va + i);
        p[0] = __ffma2_rn(make_float2(x.x, x.y), make_float2(c[i], c[i + 1]), p[0]);
        p[1] = __ffma2_rn(make_float2(x.z, x.w), make_float2(c[i + 2], c[i + 3]), p[1]);
    }
    return hsum2(p[0], p[1]);
}

struct HeadFwdArgs {
    const void* wx;      // (B,T,3d) I/O dtype
    const float* A;      // (3,H,dh,dh) fp32, order A_z, A_r, A_n
    const float* h0;     // (B,d) fp32 or null
    const float* hin;    // (B,T,d) fp32 input trajectory, null = App. A guess computed in place
    void* hout;          // (B,T,d): fp32 work trajectory or I/O dtype (out_io)
    unsigned* hist_bits; // n_newton slots
    unsigned* final_bits;
    int out_io, n_newton, resid;
    int B, T, d, H;
    float omega;
};

template <typename TIO, int DH>
__global__ void __launch_bounds__(256, 1) gru_head_newton_kernel(HeadFwdArgs a) {
    constexpr int MAXS = 4;
    __shared__ __align__(16) float s_vec[MAXS][2][kHG];    // hp, delta of each stage
    __shared__ __align__(16) float s_vec2[MAXS][2][kHG];   // u, du of each stage
    __shared__ float s_traj[MAXS + 1][2][kHG];             // trajectory entering each stage
    __shared__ unsigned s_red[8];
    const int stage = threadIdx.x / kHG, o = threadIdx.x % kHG;
    const int nstg = a.n_newton + (a.resid ? 1 : 0);
    const int b = blockIdx.x / a.H, head = blockIdx.x % a.H;
    const bool act = o < DH;
    const bool is_resid = a.resid && stage == a.n_newton;
    const int oc = act ? o : 0;

    float az[DH], ar[DH], an[DH];
    {
        const size_t hs = (size_t)DH * DH;
        const float* Az = a.A + ((size_t)0 * a.H + head) * hs;
        const float* Ar = a.A + ((size_t)1 * a.H + head) * hs;
        const float* An = a.A + ((size_t)2 * a.H + head) * hs;
#pragma unroll
        for (int i = 0; i < DH; ++i) {
            az[i] = __ldg(Az + (size_t)i * DH + oc);
            ar[i] = __ldg(Ar + (size_t)i * DH + oc);
            an[i] = __ldg(An + (size_t)i * DH + oc);
        }
    }
    const TIO* wx = reinterpret_cast<const TIO*>(a.wx) + (size_t)b * a.T * 3 * a.d + head * DH + oc;
    const float* hin = a.hin ? a.hin + (size_t)b * a.T * a.d + head * DH + oc : nullptr;
    const float h_init = a.h0 ? __ldg(a.h0 + (size_t)b * a.d + head * DH + oc) : 0.f;

    float hp = h_init, dl = 0.f;
    unsigned rmax = 0u;
    s_vec[stage][0][o] = act ? hp : 0.f;
    s_vec[stage][1][o] = 0.f;
    s_vec2[stage][0][o] = 0.f;
    s_vec2[stage][1][o] = 0.f;

    // With no input trajectory, stage 0 linearises around the App. A guess f(0, x_t) (h0 only
    // at t = 0), which needs no matrix product except at t = 0 with a non-zero h0.
    float guess0 = 0.f;
    if (!a.hin && a.h0 && stage == 0) {
        __syncthreads();
        float pz, pr, d0, d1;
        dot2x2<DH>(s_vec[0][0], s_vec[0][1], az, ar, pz, pr, d0, d1);
        const float z = sigmoid_f(pz + ld_f(wx)), r = sigmoid_f(pr + ld_f(wx + a.d));
        s_vec2[0][0][o] = act ? hp * r : 0.f;
        stage_bar(1);
        float pn, d2;
        dot2x1<DH>(s_vec2[0][0], s_vec2[0][1], an, pn, d2);
        const float n = tanh_f(pn + ld_f(wx + 2 * (size_t)a.d));
        guess0 = hp + z * (n - hp);
    } else if (!a.hin && a.h0) {
        __syncthreads();
    }

    const int n_ticks = a.T + nstg - 1;
    // inputs are fetched PF ticks ahead into a small register ring, so that no global-memory
    // latency sits on the tick-to-tick critical path
    constexpr int PF = 4;
    TIO b_zx[PF], b_rx[PF], b_nx[PF];
    float b_hin[PF];
    auto fetch = [&](int tick, int slot) {
        const int t = tick - stage;
        b_zx[slot] = b_rx[slot] = b_nx[slot] = raw_zero<TIO>();
        b_hin[slot] = 0.f;
        if (stage < nstg && t >= 0 && t < a.T) {
            b_zx[slot] = __ldg(wx + (size_t)t * 3 * a.d);
            b_rx[slot] = __ldg(wx + (size_t)t * 3 * a.d + a.d);
            b_nx[slot] = __ldg(wx + (size_t)t * 3 * a.d + 2 * (size_t)a.d);
            if (stage == 0 && hin) b_hin[slot] = __ldg(hin + (size_t)t * a.d);
        }
    };
#pragma unroll
    for (int j = 0; j < PF; ++j) fetch(j, j);
    for (int tick0 = 0; tick0 < n_ticks; tick0 += PF) {
#pragma unroll
        for (int j = 0; j < PF; ++j) {
            const int tick = tick0 + j;
            if (tick >= n_ticks) break;
            __syncthreads();
            const int t = tick - stage;
            const bool on = stage < nstg && t >= 0 && t < a.T;
            const float zx = raw_f(b_zx[j]), rx = raw_f(b_rx[j]), nx = raw_f(b_nx[j]);
            float cur = 0.f;
            if (on) {
                if (stage == 0) {
                    if (hin) {
                        cur = b_hin[j];
                    } else if (t == 0 && a.h0) {
                        cur = guess0;
                    } else {
                        cur = sigmoid_f(zx) * tanh_f(nx);  // f(0, x): z * n
                    }
                } else {
                    cur = s_traj[stage][(tick + 1) & 1][o];
                }
            }
            fetch(tick + PF, j);
            if (stage < nstg) {
                float pz, pr, dz, dr;
                dot2x2<DH>(s_vec[stage][0], s_vec[stage][1], az, ar, pz, pr, dz, dr);
                const float z = sigmoid_f(pz + zx), r = sigmoid_f(pr + rx);
                const float rp = r * (1.f - r);
                s_vec2[stage][0][o] = act ? hp * r : 0.f;
                s_vec2[stage][1][o] = act ? fmaf(r, dl, hp * rp * dr) : 0.f;
                stage_bar(1 + stage);
                float pn, dn;
                dot2x1<DH>(s_vec2[stage][0], s_vec2[stage][1], an, pn, dn);
                if (on) {
                    const float n = tanh_f(pn + nx);
                    const float f = fmaf(z, n - hp, hp);
                    const float F = f - cur;
                    if (act) rmax = max(rmax, absbits(F));
                    if (!is_resid) {
                        const float jd = (1.f - z) * dl + (n - hp) * z * (1.f - z) * dz + z * (1.f - n * n) * dn;
                        dl = jd + F;
                        const float nv = fmaf(a.omega, dl, cur);
                        s_traj[stage + 1][tick & 1][o] = nv;
                        if (stage == a.n_newton - 1 && act) {
                            const size_t idx = ((size_t)b * a.T + t) * a.d + head * DH + o;
                            if (a.out_io)
                                st_f(reinterpret_cast<TIO*>(a.hout) + idx, nv);
                            else
                                reinterpret_cast<float*>(a.hout)[idx] = nv;
                        }
                    }
                    hp = cur;
                }
                s_vec[stage][0][o] = act ? hp : 0.f;
                s_vec[stage][1][o] = act ? dl : 0.f;
            }
        }
    }
    // per-stage maxima: stage s < n_newton -> hist_bits[s]; residual stage -> final_bits
    for (int s = 0; s < nstg; ++s) {
        __syncthreads();
        unsigned v = (stage == s) ? rmax : 0u;
        unsigned* dst = (a.resid && s == a.n_newton) ? a.final_bits : a.hist_bits + s;
        block_residual_max(v, dst, s_red);
    }
}

// ------------------------------------------------------------------ backward
struct HeadBwdArgs {
    const void* wx;           // (B,T,3d)
    const void* states;       // (B,T,d) I/O dtype
    const void* grad_states;  // (B,T,d) I/O dtype
    const float* A;           // (3,H,dh,dh)
    const float* h0;          // (B,d) fp32 or null
    void* g_wx;               // (B,T,3d) I/O dtype
    float* gA_part;           // (B,3,H,dh,dh) fp32: this batch row's share of grad A
    float* g_h0;              // (B,d) fp32 or null
    float* mu_out;            // (B,T,d) fp32 or null: mu_t = nu_t + g_t, the adjoint of eq. 2.6
    int B, T, d, H;
};

// Three groups of 64 threads per (batch row, head), skewed by one tick each:
//   group 0 recomputes the gates of step t (columns of A in registers),
//   group 1 walks the adjoint backwards, nu_{t-1} = J_t^T (nu_t + g_t) (rows of A in registers),
//   group 2 accumulates the outer products of the packed VJP,
//           grad A_z += h_prev^T d_z, grad A_r += h_prev^T d_r, grad A_n += (h_prev r)^T d_n,
//           thread o keeping column o of all three in registers for the whole sweep.
template <typename TIO, int DH>
__global__ void __launch_bounds__(192, 1) gru_head_bwd_kernel(HeadBwdArgs a) {
    __shared__ __align__(16) float s_h[3][kHG];       // h_prev of the last three steps (ring)
    __shared__ __align__(16) float s_u[3][kHG];       // h_prev * r, same ring
    __shared__ float s_gate[2][4][kHG];               // z, r, n, h_prev handed to the adjoint group
    __shared__ __align__(16) float s_w[2][kHG];       // w_z, w_n
    __shared__ __align__(16) float s_v3[kHG];         // r' h g
    __shared__ float s_d[2][3][kHG];                  // d_z, d_r, d_n handed to the outer-product group
    const int grp = threadIdx.x / kHG, o = threadIdx.x % kHG;
    const int b = blockIdx.x / a.H, head = blockIdx.x % a.H;
    const bool act = o < DH;
    const int oc = act ? o : 0;
    const size_t hs = (size_t)DH * DH;
    const float* Az = a.A + ((size_t)0 * a.H + head) * hs;
    const float* Ar = a.A + ((size_t)1 * a.H + head) * hs;
    const float* An = a.A + ((size_t)2 * a.H + head) * hs;
    float m0[DH], m1[DH], m2[DH];
#pragma unroll
    for (int i = 0; i < DH; ++i) {
        if (grp == 0) {         // columns: m[i] = A[i][o]
            m0[i] = __ldg(Az + (size_t)i * DH + oc);
            m1[i] = __ldg(Ar + (size_t)i * DH + oc);
            m2[i] = __ldg(An + (size_t)i * DH + oc);
        } else if (grp == 1) {  // rows: m[k] = A[o][k]
            m0[i] = __ldg(Az + (size_t)oc * DH + i);
            m1[i] = __ldg(Ar + (size_t)oc * DH + i);
            m2[i] = __ldg(An + (size_t)oc * DH + i);
        } else {                // accumulators of grad A[i][o]
            m0[i] = 0.f; m1[i] = 0.f; m2[i] = 0.f;
        }
    }
    const size_t base = (size_t)b * a.T * a.d + head * DH + oc;
    const TIO* wx = reinterpret_cast<const TIO*>(a.wx) + (size_t)b * a.T * 3 * a.d + head * DH + oc;
    const TIO* st = reinterpret_cast<const TIO*>(a.states) + base;
    const TIO* gs = reinterpret_cast<const TIO*>(a.grad_states) + base;
    TIO* gwx = reinterpret_cast<TIO*>(a.g_wx) + (size_t)b * a.T * 3 * a.d + head * DH + oc;
    const float h_init = a.h0 ? __ldg(a.h0 + (size_t)b * a.d + head * DH + oc) : 0.f;
    if (grp == 0) {
#pragma unroll
        for (int j = 0; j < 3; ++j) { s_h[j][o] = 0.f; s_u[j][o] = 0.f; }
        s_w[0][o] = 0.f; s_w[1][o] = 0.f; s_v3[o] = 0.f;
    }
    float nu = 0.f;
    __syncthreads();
    // tick k: group 0 handles step T-1-k, group 1 step T-k, group 2 step T+1-k.
    // Global inputs are fetched PF ticks ahead into a register ring.
    constexpr int PF = 4;
    TIO b0[PF], b1[PF], b2[PF], b3[PF];
    auto fetch = [&](int k, int slot) {
        b0[slot] = b1[slot] = b2[slot] = b3[slot] = raw_zero<TIO>();
        if (grp == 0) {
            const int t = a.T - 1 - k;
            if (t >= 0 && k >= 0) {
                if (t > 0) b0[slot] = __ldg(st + (size_t)(t - 1) * a.d);
                b1[slot] = __ldg(wx + (size_t)t * 3 * a.d);
                b2[slot] = __ldg(wx + (size_t)t * 3 * a.d + a.d);
                b3[slot] = __ldg(wx + (size_t)t * 3 * a.d + 2 * (size_t)a.d);
            }
        } else if (grp == 1) {
            const int t = a.T - k;
            if (t >= 0 && t < a.T) b0[slot] = __ldg(gs + (size_t)t * a.d);
        }
    };
#pragma unroll
    for (int j = 0; j < PF; ++j) fetch(j, j);
    int ring = 0;  // k % 3
    for (int k0 = 0; k0 <= a.T + 1; k0 += PF) {
#pragma unroll
        for (int j = 0; j < PF; ++j) {
            const int k = k0 + j;
            if (k > a.T + 1) break;
            if (grp == 0) {
                const int t = a.T - 1 - k;
                const float hpv = (t == 0) ? h_init : raw_f(b0[j]);
                const float zx = raw_f(b1[j]), rx = raw_f(b2[j]), nx = raw_f(b3[j]);
                fetch(k + PF, j);
                if (t >= 0) {
                    s_h[ring][o] = act ? hpv : 0.f;
                    stage_bar(1);
                    float pz, pr;
                    dot1x2<DH>(s_h[ring], m0, m1, pz, pr);
                    const float z = sigmoid_f(pz + zx);
                    const float r = sigmoid_f(pr + rx);
                    s_u[ring][o] = act ? hpv * r : 0.f;
                    stage_bar(1);
                    const float n = tanh_f(dot1x1<DH>(s_u[ring], m2) + nx);
                    s_gate[k & 1][0][o] = z;
                    s_gate[k & 1][1][o] = r;
                    s_gate[k & 1][2][o] = n;
                    s_gate[k & 1][3][o] = hpv;
                }
            } else if (grp == 1) {
                const int t = a.T - k;
                const float gv = raw_f(b0[j]);
                fetch(k + PF, j);
                if (t >= 0 && t < a.T) {
                    const float z = s_gate[(k + 1) & 1][0][o], r = s_gate[(k + 1) & 1][1][o];
                    const float n = s_gate[(k + 1) & 1][2][o], hpv = s_gate[(k + 1) & 1][3][o];
                    const float mu = nu + gv;
                    const float w_z = z * (1.f - z) * (n - hpv) * mu;
                    const float w_n = (1.f - n * n) * z * mu;
                    s_w[0][o] = act ? w_z : 0.f;
                    s_w[1][o] = act ? w_n : 0.f;
                    stage_bar(2);
                    float t2, g;
                    dot1x1x2<DH>(s_w[0], s_w[1], m0, m2, t2, g);
                    const float v3 = r * (1.f - r) * hpv * g;
                    s_v3[o] = act ? v3 : 0.f;
                    stage_bar(2);
                    const float t4 = dot1x1<DH>(s_v3, m1);
                    if (act) {
                        if (a.mu_out) a.mu_out[base + (size_t)t * a.d] = mu;
                        st_f(gwx + (size_t)t * 3 * a.d, w_z);
                        st_f(gwx + (size_t)t * 3 * a.d + a.d, v3);
                        st_f(gwx + (size_t)t * 3 * a.d + 2 * (size_t)a.d, w_n);
                    }
                    s_d[k & 1][0][o] = w_z;
                    s_d[k & 1][1][o] = v3;
                    s_d[k & 1][2][o] = w_n;
                    nu = (1.f - z) * mu + t2 + r * g + t4;
                }
            } else {
                const int t = a.T + 1 - k;
                if (t >= 0 && t < a.T) {
                    const float dz = s_d[(k + 1) & 1][0][o], dr = s_d[(k + 1) & 1][1][o];
                    const float dn = s_d[(k + 1) & 1][2][o];
                    const int slot = ring == 2 ? 0 : ring + 1;  // (k - 2) % 3
                    const float2 dz2 = make_float2(dz, dz), dr2 = make_float2(dr, dr), dn2 = make_float2(dn, dn);
#pragma unroll
                    for (int i = 0; i < DH; i += 4) {
                        const float4 x = *reinterpret_cast<const float4*>(&s_h[slot][i]);
                        const float4 y = *reinterpret_cast<const float4*>(&s_u[slot][i]);
                        const float2 xs[2] = {{x.x, x.y}, {x.z, x.w}}, ys[2] = {{y.x, y.y}, {y.z, y.w}};
#pragma unroll
                        for (int q = 0; q < 2; ++q) {
                            const int j = i + 2 * q;
                            const float2 r0 = __ffma2_rn(xs[q], dz2, make_float2(m0[j], m0[j + 1]));
                            const float2 r1 = __ffma2_rn(xs[q], dr2, make_float2(m1[j], m1[j + 1]));
                            const float2 r2 = __ffma2_rn(ys[q], dn2, make_float2(m2[j], m2[j + 1]));
                            m0[j] = r0.x; m0[j + 1] = r0.y;
                            m1[j] = r1.x; m1[j + 1] = r1.y;
                            m2[j] = r2.x; m2[j + 1] = r2.y;
                        }
                    }
                }
            }
            ring = ring == 2 ? 0 : ring + 1;
            __syncthreads();
        }
    }
    if (grp == 1 && act && a.g_h0) a.g_h0[(size_t)b * a.d + head * DH + o] = nu;
    if (grp == 2 && act) {
        float* dst = a.gA_part + (((size_t)b * 3) * a.H + head) * hs + o;
        const size_t gs3 = (size_t)a.H * hs;
#pragma unroll
        for (int i = 0; i < DH; ++i) {
            dst[(size_t)i * DH] = m0[i];
            dst[gs3 + (size_t)i * DH] = m1[i];
            dst[2 * gs3 + (size_t)i * DH] = m2[i];
        }
    }
}

// ------------------------------------------------------------------ launchers
template <typename TIO>
static cudaError_t launch_head_fwd_t(const HeadFwdArgs& a, int dh, cudaStream_t s) {
    const int grid = a.B * a.H;
    const int threads = kHG * (a.n_newton + (a.resid ? 1 : 0));
    switch (dh) {
        case 8: gru_head_newton_kernel<TIO, 8><<<grid, threads, 0, s>>>(a); break;
        case 16: gru_head_newton_kernel<TIO, 16><<<grid, threads, 0, s>>>(a); break;
        case 32: gru_head_newton_kernel<TIO, 32><<<grid, threads, 0, s>>>(a); break;
        case 64: gru_head_newton_kernel<TIO, 64><<<grid, threads, 0, s>>>(a); break;
        default: return cudaErrorNotSupported;
    }
    return cudaGetLastError();
}

cudaError_t launch_gru_head_fwd(int dtype, const void* wx, const float* A, const float* h0,
                                const float* hin, void* hout, bool out_io, int n_newton, bool resid,
                                unsigned* hist_bits, unsigned* final_bits, int B, int T, int d, int H,
                                float omega, cudaStream_t s) {
    HeadFwdArgs a{wx, A, h0, hin, hout, hist_bits, final_bits, out_io ? 1 : 0, n_newton, resid ? 1 : 0,
                  B, T, d, H, omega};
    if (n_newton + (resid ? 1 : 0) < 1 || n_newton + (resid ? 1 : 0) > 4) return cudaErrorInvalidValue;
    return dtype == kF32 ? launch_head_fwd_t<float>(a, d / H, s) : launch_head_fwd_t<__nv_bfloat16>(a, d / H, s);
}

template <typename TIO>
static cudaError_t launch_head_bwd_t(const HeadBwdArgs& a, int dh, cudaStream_t s) {
    const int grid = a.B * a.H;
    switch (dh) {
        case 8: gru_head_bwd_kernel<TIO, 8><<<grid, 192, 0, s>>>(a); break;
        case 16: gru_head_bwd_kernel<TIO, 16><<<grid, 192, 0, s>>>(a); break;
        case 32: gru_head_bwd_kernel<TIO, 32><<<grid, 192, 0, s>>>(a); break;
        case 64: gru_head_bwd_kernel<TIO, 64><<<grid, 192, 0, s>>>(a); break;
        default: return cudaErrorNotSupported;
    }
    return cudaGetLastError();
}

cudaError_t launch_gru_head_bwd(int dtype, const void* wx, const void* states, const void* grad_states,
                                const float* A, const float* h0, void* g_wx, float* gA_part, float* g_h0,
                                float* mu_out, int B, int T, int d, int H, cudaStream_t s) {
    HeadBwdArgs a{wx, states, grad_states, A, h0, g_wx, gA_part, g_h0, mu_out, B, T, d, H};
    return dtype == kF32 ? launch_head_bwd_t<float>(a, d / H, s) : launch_head_bwd_t<__nv_bfloat16>(a, d / H, s);
}

}  // namespace prb
