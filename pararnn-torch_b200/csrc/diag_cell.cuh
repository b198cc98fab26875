// Per-step math of the scalar-diagonal cells (ParaGRU mix='diag', ParaNLRU, ParaTitans, ParaCfC), shared by
// the look-back kernels (diag_kernels.cu) and the pipelined persistent kernels (diag_pipe.cu).
//
// Reference behaviour restated: cells/para_gru.py:418-467, cells/para_nlru.py:149-168,
// cells/para_titans.py:170-216, cells/para_cfc.py:162-231 (step and diagonal Jacobian),
// kernels/vjp_gru.py:107-138, kernels/vjp_nlru.py:88-108, kernels/vjp_cfc.py:26-100 (packed VJP; the Titans VJP is the closed form of what the reference
// obtains from autograd through ``step``, solvers/vjp.py:77-98).
#pragma once
#include "common.cuh"
#include "kernels.h"

namespace prb {

template <int CELL>
struct DiagCell;

template <>
struct DiagCell<kCellGruDiag> {
    static constexpr int G = 3, NP = 3;
    struct Acts {
        float z, r, n;
    };
    __device__ static __forceinline__ void eval(float h, const float (&g)[3], const float (&p)[3],
                                                float& f, float& j, Acts& a) {
        a.z = sigmoid_f(fmaf(p[0], h, g[0]));
        a.r = sigmoid_f(fmaf(p[1], h, g[1]));
        a.n = tanh_f(fmaf(p[2], h * a.r, g[2]));
        f = fmaf(a.z, a.n - h, h);
        const float zp = a.z * (1.f - a.z), rp = a.r * (1.f - a.r), np_ = 1.f - a.n * a.n;
        j = (1.f - a.z) + (a.n - h) * zp * p[0] + a.z * np_ * p[2] * (a.r + h * rp * p[1]);
    }
    __device__ static __forceinline__ float step(float h, const float (&g)[3], const float (&p)[3]) {
        const float z = sigmoid_f(fmaf(p[0], h, g[0]));
        const float r = sigmoid_f(fmaf(p[1], h, g[1]));
        const float n = tanh_f(fmaf(p[2], h * r, g[2]));
        return fmaf(z, n - h, h);
    }
    // packed VJP: gate pre-activation grads and the per-step parameter terms
    __device__ static __forceinline__ void vjp(float h, const Acts& a, const float (&p)[3], float mu,
                                               float (&gw)[3], float (&gp)[3]) {
        const float d_z = mu * (a.n - h);
        const float d_n = mu * a.z * (1.f - a.n * a.n);
        const float d_zp = d_z * a.z * (1.f - a.z);
        const float d_rp = (d_n * p[2] * h) * a.r * (1.f - a.r);
        gw[0] = d_zp;
        gw[1] = d_rp;
        gw[2] = d_n;
        gp[0] = d_zp * h;
        gp[1] = d_rp * h;
        gp[2] = d_n * (h * a.r);
    }
};

template <>
struct DiagCell<kCellNlru> {
    static constexpr int G = 2, NP = 1;
    struct Acts {
        float a, n;
    };
    __device__ static __forceinline__ void eval(float h, const float (&g)[2], const float (&p)[1],
                                                float& f, float& j, Acts& a) {
        a.a = sigmoid_f(g[0]);
        a.n = tanh_f(fmaf(p[0], h, g[1]));
        f = fmaf(a.a, h, (1.f - a.a) * a.n);
        j = fmaf((1.f - a.a) * (1.f - a.n * a.n), p[0], a.a);
    }
    __device__ static __forceinline__ float step(float h, const float (&g)[2], const float (&p)[1]) {
        const float a = sigmoid_f(g[0]);
        const float n = tanh_f(fmaf(p[0], h, g[1]));
        return fmaf(a, h, (1.f - a) * n);
    }
    __device__ static __forceinline__ void vjp(float h, const Acts& a, const float (&p)[1], float mu,
                                               float (&gw)[2], float (&gp)[1]) {
        const float d_a = mu * (h - a.n) * a.a * (1.f - a.a);
        const float d_c = mu * (1.f - a.a) * (1.f - a.n * a.n);
        gw[0] = d_a;
        gw[1] = d_c;
        gp[0] = d_c * h;
    }
};

// softplus with the reference's (torch.nn.functional.softplus) overflow guard
__device__ __forceinline__ float softplus_f(float x) {
    return x > 20.f ? x : 0.6931471805599453f * __log2f(1.f + exp_f(x));
}

// ParaTitans: h' = (1 - alpha) h - theta (h k - v) k + u tanh(n_x + r h),
// gates (alpha_pre, theta_pre, k, v, n_x) = W_x(x), parameters (u, r).
template <>
struct DiagCell<kCellTitans> {
    static constexpr int G = 5, NP = 2;
    struct Acts {
        float alpha, theta, sg_theta, k, v, n;
    };
    __device__ static __forceinline__ void eval(float h, const float (&g)[5], const float (&p)[2],
                                                float& f, float& j, Acts& a) {
        a.alpha = sigmoid_f(g[0]);
        a.theta = softplus_f(g[1]);
        a.sg_theta = sigmoid_f(g[1]);  // d softplus / d pre
        a.k = g[2];
        a.v = g[3];
        a.n = tanh_f(fmaf(p[1], h, g[4]));
        const float grad = (h * a.k - a.v) * a.k;
        f = fmaf(p[0], a.n, fmaf(-a.theta, grad, (1.f - a.alpha) * h));
        j = (1.f - a.alpha) - a.theta * a.k * a.k + p[0] * (1.f - a.n * a.n) * p[1];
    }
    __device__ static __forceinline__ float step(float h, const float (&g)[5], const float (&p)[2]) {
        const float alpha = sigmoid_f(g[0]);
        const float theta = softplus_f(g[1]);
        const float n = tanh_f(fmaf(p[1], h, g[4]));
        const float grad = (h * g[2] - g[3]) * g[2];
        return fmaf(p[0], n, fmaf(-theta, grad, (1.f - alpha) * h));
    }
    __device__ static __forceinline__ void vjp(float h, const Acts& a, const float (&p)[2], float mu,
                                               float (&gw)[5], float (&gp)[2]) {
        const float np_ = 1.f - a.n * a.n;
        const float err = h * a.k - a.v;
        gw[0] = -mu * h * a.alpha * (1.f - a.alpha);
        gw[1] = -mu * err * a.k * a.sg_theta;
        gw[2] = -mu * a.theta * (err + h * a.k);
        gw[3] = mu * a.theta * a.k;
        gw[4] = mu * p[0] * np_;
        gp[0] = mu * a.n;
        gp[1] = gw[4] * h;
    }
};

// ParaCfC (gate_mix='input'): a = sigmoid(-(softplus(f) dt + b)), h' = a h + (1 - a) tanh(c + u h),
// gates (f, c, dt, b) = project_wx(x) (dt >= 1e-4 is the clamped time step broadcast over the
// channels, b the input-conditioned time bias), parameter u.
template <>
struct DiagCell<kCellCfc> {
    static constexpr int G = 4, NP = 1;
    struct Acts {
        float a, n, soft, sg_f, dt;
    };
    __device__ static __forceinline__ void eval(float h, const float (&g)[4], const float (&p)[1],
                                                float& f, float& j, Acts& a) {
        a.soft = softplus_f(g[0]);
        a.sg_f = sigmoid_f(g[0]);  // d softplus / d pre
        a.dt = g[2];
        a.a = sigmoid_f(-fmaf(a.soft, g[2], g[3]));
        a.n = tanh_f(fmaf(p[0], h, g[1]));
        f = fmaf(a.a, h, (1.f - a.a) * a.n);
        j = fmaf((1.f - a.a) * (1.f - a.n * a.n), p[0], a.a);
    }
    __device__ static __forceinline__ float step(float h, const float (&g)[4], const float (&p)[1]) {
        const float a = sigmoid_f(-fmaf(softplus_f(g[0]), g[2], g[3]));
        const float n = tanh_f(fmaf(p[0], h, g[1]));
        return fmaf(a, h, (1.f - a) * n);
    }
    __device__ static __forceinline__ void vjp(float h, const Acts& a, const float (&p)[1], float mu,
                                               float (&gw)[4], float (&gp)[1]) {
        const float d_pre = -mu * (h - a.n) * a.a * (1.f - a.a);  // grad of (soft dt + b)
        gw[0] = d_pre * a.dt * a.sg_f;
        gw[1] = mu * (1.f - a.a) * (1.f - a.n * a.n);
        gw[2] = d_pre * a.soft;
        gw[3] = d_pre;
        gp[0] = gw[1] * h;
    }
};

}  // namespace prb
