// Per-step math of ParaSLSTM mix='diag' shared by the scan kernels: prediction, structured
// 4x4 Jacobian (12 non-zeros; the h row is a combination of the c and n rows), and the
// activations the packed VJP needs.  Restates reference cells/para_slstm.py:347-446.
#pragma once
#include "common.cuh"

namespace prb {

struct SlstmLin {
    // structured Jacobian pieces of one step
    float f, jcm, jch, jnm, jnh, alpha, dm, ia, ib, ie;
    float pc, pn, pm, ph;  // prediction f(H_{t-1}, x_t)
    float it, z, og, invD;  // gate activations (used by the reverse kernels)
};

__device__ __forceinline__ void slstm_linearize(const float (&prev)[4], const float (&w)[4],
                                                const float (&r)[4], float eps, SlstmLin& o) {
    const float c = prev[0], n = prev[1], m = prev[2], h = prev[3];
    const float zi = fmaf(r[0], h, w[0]), zf = fmaf(r[1], h, w[1]);
    const float zz = fmaf(r[2], h, w[2]), zo = fmaf(r[3], h, w[3]);
    const float left = zf + m;
    const float mn = fmaxf(left, zi);
    const float alpha = left > zi ? 1.f : (left == zi ? 0.5f : 0.f);
    const float beta = 1.f - alpha;
    // one of the two exponentials is exp(0) = 1 exactly
    const float e_ = exp_f(-fabsf(left - zi));
    const float it = left >= zi ? e_ : 1.f;
    const float ft = left >= zi ? 1.f : e_;
    const float z = tanh_f(zz);
    const float og = sigmoid_f(zo);
    const float nn = fmaf(ft, n, it);
    const float cn = fmaf(ft, c, it * z);
    const float invD = rcp_f(nn + eps);
    const float u = cn * invD;  // c_new / D
    o.it = it;
    o.z = z;
    o.og = og;
    o.invD = invD;
    o.pc = cn;
    o.pn = nn;
    o.pm = mn;
    o.ph = og * u;
    const float dm = fmaf(alpha, r[1], beta * r[0]);
    const float di_dm = -it * alpha, df_dm = ft * beta;
    const float di_dh = it * (r[0] - dm), df_dh = ft * (r[1] - dm);
    const float dz_dh = (1.f - z * z) * r[2];
    o.f = ft;
    o.jcm = fmaf(df_dm, c, di_dm * z);
    o.jch = fmaf(df_dh, c, fmaf(di_dh, z, it * dz_dh));
    o.jnm = fmaf(df_dm, n, di_dm);
    o.jnh = fmaf(df_dh, n, di_dh);
    o.alpha = alpha;
    o.dm = dm;
    o.ia = og * invD;
    o.ib = -o.ph * invD;  // -o c_new / D^2
    o.ie = u * og * (1.f - og) * r[3];
}

__device__ __forceinline__ void slstm_predict(const float (&prev)[4], const float (&w)[4],
                                              const float (&r)[4], float eps, float (&pred)[4]) {
    const float c = prev[0], n = prev[1], m = prev[2], h = prev[3];
    const float zi = fmaf(r[0], h, w[0]), zf = fmaf(r[1], h, w[1]);
    const float zz = fmaf(r[2], h, w[2]), zo = fmaf(r[3], h, w[3]);
    const float left = zf + m;
    const float mn = fmaxf(left, zi);
    // one of the two exponentials is exp(0) = 1 exactly
    const float e_ = exp_f(-fabsf(left - zi));
    const float it = left >= zi ? e_ : 1.f;
    const float ft = left >= zi ? 1.f : e_;
    const float z = tanh_f(zz);
    const float nn = fmaf(ft, n, it);
    const float cn = fmaf(ft, c, it * z);
    pred[0] = cn;
    pred[1] = nn;
    pred[2] = mn;
    pred[3] = sigmoid_f(zo) * (cn * rcp_f(nn + eps));
}

// x <- J x + F  for the state ordering (c, n, m, h); fh2 = Fh - ia*Fc - ib*Fn
__device__ __forceinline__ void slstm_apply(const SlstmLin& l, float fc, float fn, float fm, float fh2,
                                            float& xc, float& xn, float& xm, float& xh) {
    const float nc = fmaf(l.f, xc, fmaf(l.jcm, xm, fmaf(l.jch, xh, fc)));
    const float nn = fmaf(l.f, xn, fmaf(l.jnm, xm, fmaf(l.jnh, xh, fn)));
    const float nm = fmaf(l.alpha, xm, fmaf(l.dm, xh, fm));
    const float nh = fmaf(l.ia, nc, fmaf(l.ib, nn, fmaf(l.ie, xh, fh2)));
    xc = nc;
    xn = nn;
    xm = nm;
    xh = nh;
}

// Two columns of a map at once on packed fp32 FMAs (fma.rn.f32x2): x <- J x for both columns, same
// operations and rounding per column as slstm_apply with a zero offset.
__device__ __forceinline__ void slstm_apply_cols2(const SlstmLin& l, float2& xc, float2& xn, float2& xm,
                                                  float2& xh) {
    const float2 nc = __ffma2_rn(splat2(l.f), xc, __ffma2_rn(splat2(l.jcm), xm, __fmul2_rn(splat2(l.jch), xh)));
    const float2 nn = __ffma2_rn(splat2(l.f), xn, __ffma2_rn(splat2(l.jnm), xm, __fmul2_rn(splat2(l.jnh), xh)));
    const float2 nm = __ffma2_rn(splat2(l.alpha), xm, __fmul2_rn(splat2(l.dm), xh));
    const float2 nh = __ffma2_rn(splat2(l.ia), nc, __ffma2_rn(splat2(l.ib), nn, __fmul2_rn(splat2(l.ie), xh)));
    xc = nc;
    xn = nn;
    xm = nm;
    xh = nh;
}

// y = J^T x for two columns at once (packed counterpart of slstm_apply_t)
__device__ __forceinline__ void slstm_apply_t_cols2(const SlstmLin& l, float2& xc, float2& xn, float2& xm,
                                                    float2& xh) {
    const float2 pc = __ffma2_rn(splat2(l.ia), xh, xc), pn = __ffma2_rn(splat2(l.ib), xh, xn);
    const float2 yc = __fmul2_rn(splat2(l.f), pc), yn = __fmul2_rn(splat2(l.f), pn);
    const float2 ym = __ffma2_rn(splat2(l.jcm), pc, __ffma2_rn(splat2(l.jnm), pn, __fmul2_rn(splat2(l.alpha), xm)));
    const float2 yh = __ffma2_rn(
        splat2(l.jch), pc,
        __ffma2_rn(splat2(l.jnh), pn, __ffma2_rn(splat2(l.dm), xm, __fmul2_rn(splat2(l.ie), xh))));
    xc = yc;
    xn = yn;
    xm = ym;
    xh = yh;
}

// Activations kept between the two phases of the reverse kernel.
struct SlstmAct {
    float i, f, z, o, c, n, invD, alpha, hp;
};

// Gate activations of one step (no Jacobian entries): what the packed VJP consumes.
__device__ __forceinline__ void slstm_acts(const float (&prev)[4], const float (&w)[4],
                                           const float (&r)[4], float eps, SlstmAct& o) {
    const float c = prev[0], n = prev[1], m = prev[2], h = prev[3];
    const float zi = fmaf(r[0], h, w[0]), zf = fmaf(r[1], h, w[1]);
    const float zz = fmaf(r[2], h, w[2]), zo = fmaf(r[3], h, w[3]);
    const float left = zf + m;
    const float e_ = exp_f(-fabsf(left - zi));
    o.i = left >= zi ? e_ : 1.f;
    o.f = left >= zi ? 1.f : e_;
    o.alpha = left > zi ? 1.f : (left == zi ? 0.5f : 0.f);
    o.z = tanh_f(zz);
    o.o = sigmoid_f(zo);
    o.c = c;
    o.n = n;
    o.invD = rcp_f(fmaf(o.f, n, o.i) + eps);
    o.hp = h;
}

// y = J^T x with the structured J (11 FMA)
__device__ __forceinline__ void slstm_apply_t(const SlstmLin& l, float& xc, float& xn, float& xm,
                                              float& xh) {
    const float pc = fmaf(l.ia, xh, xc), pn = fmaf(l.ib, xh, xn);
    const float yc = l.f * pc, yn = l.f * pn;
    const float ym = fmaf(l.jcm, pc, fmaf(l.jnm, pn, l.alpha * xm));
    const float yh = fmaf(l.jch, pc, fmaf(l.jnh, pn, fmaf(l.dm, xm, l.ie * xh)));
    xc = yc;
    xn = yn;
    xm = ym;
    xh = yh;
}

}  // namespace prb
