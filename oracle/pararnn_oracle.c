/*
 * CPU restatement of the reference's eager Newton+scan training path.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the product package may call, link or
 * import this file; it exists so that tests, the smoke entry and the CPU arm
 * of the benchmark have an independent checker for the CUDA kernels.
 *
 * Parity status: pinned.  The functions below are checked against vectors
 * produced by importing the reference (pararnn 0.17.5) and running its own
 * eager path; the fixtures and the script that made them live in
 * tests/golden/.
 *
 * Boundary: the op boundary of the reference's fused custom ops, i.e. the
 * input projection wx = W_x(x) is an input, states / gradients w.r.t. wx and
 * the recurrent parameters are outputs.  Recurrent parameters arrive already
 * clamped (the reference clamps outside its kernels, cells/para_gru.py:226-250,
 * cells/para_slstm.py:202-207, cells/para_nlru.py:124-128).
 *
 * Each function cites the reference file:line it restates (paths relative to
 * the reference project root).
 *
 * Compile with -DREAL=float (parity with the reference's fp32 arithmetic) or
 * -DREAL=double (ground truth for error measurements).
 */
#include <math.h>
#include <stddef.h>
#include <stdlib.h>
#include <string.h>

#ifndef REAL
#define REAL float
#endif
typedef REAL real;

enum { CELL_GRU_DIAG = 0, CELL_NLRU = 1, CELL_SLSTM_DIAG = 2, CELL_GRU_HEAD = 3, CELL_TITANS = 4, CELL_LSTM = 5, CELL_CFC = 6 };

static inline real r_exp(real x) { return sizeof(real) == 4 ? (real)expf((float)x) : (real)exp((double)x); }
static inline real r_tanh(real x) { return sizeof(real) == 4 ? (real)tanhf((float)x) : (real)tanh((double)x); }
static inline real r_sigmoid(real x) { return (real)1 / ((real)1 + r_exp(-x)); }
static inline real r_max(real a, real b) { return a > b ? a : b; }
static inline real r_abs(real a) { return a < 0 ? -a : a; }
/* max that lets NaN win, like torch.amax */
static inline real nanmax(real acc, real v) { return (v != v || v > acc) ? v : acc; }

int oracle_real_bytes(void) { return (int)sizeof(real); }

static int gates_of(int kind) {
    return kind == CELL_NLRU ? 2 : ((kind == CELL_SLSTM_DIAG || kind == CELL_CFC) ? 4 : (kind == CELL_TITANS ? 5 : 3));
}
static int slots_of(int kind) { return kind == CELL_SLSTM_DIAG ? 4 : (kind == CELL_LSTM ? 2 : 1); }

/* ------------------------------------------------------------------ */
/* Scalar-diagonal cells                                               */
/* ------------------------------------------------------------------ */

/* ParaGRU mix='diag' step + diagonal Jacobian.
 * cells/para_gru.py:418-441 (_jac_diag) and :449-467 (_recurrence). */
static inline void gru_diag(real h, real zx, real rx, real nx, real az, real ar, real an,
                            real *f, real *j) {
    real z = r_sigmoid(az * h + zx);
    real r = r_sigmoid(ar * h + rx);
    real n = r_tanh(an * (h * r) + nx);
    *f = h + z * (n - h); /* torch.lerp(h, n, z) */
    if (j) {
        real zp = z * (1 - z), rp = r * (1 - r), np_ = 1 - n * n;
        *j = (1 - z) + (n - h) * zp * az + z * np_ * an * (r + h * rp * ar);
    }
}

/* ParaNLRU step + diagonal Jacobian.  cells/para_nlru.py:149-168. */
static inline void nlru(real h, real ax, real cx, real u, real *f, real *j) {
    real a = r_sigmoid(ax);
    real n = r_tanh(cx + u * h);
    *f = a * h + (1 - a) * n;
    if (j) *j = a + (1 - a) * (1 - n * n) * u;
}

/* ParaTitans step + diagonal Jacobian.  cells/para_titans.py:170-216:
 * gates (alpha_pre, theta_pre, k, v, n_pre) = chunk5(wx), parameters (u, r) clamped outside. */
static inline real r_softplus(real x) {
    if (x > 20) return x; /* torch.nn.functional.softplus threshold */
    return sizeof(real) == 4 ? (real)log1pf(expf((float)x)) : (real)log1p(exp((double)x));
}
static inline void titans(real h, real ap, real tp, real k, real v, real np_, real u, real r, real *f,
                          real *j) {
    real alpha = r_sigmoid(ap), theta = r_softplus(tp);
    real grad = (h * k - v) * k;
    real n = r_tanh(np_ + r * h);
    *f = (1 - alpha) * h - theta * grad + u * n;
    if (j) *j = (1 - alpha) - theta * k * k + u * (1 - n * n) * r;
}

/* ParaCfC (gate_mix='input') step + diagonal Jacobian.  cells/para_cfc.py:162-171, 215-231:
 * gates (f_pre, c_x, dt, b) = chunk4(project_wx(x)), a = sigmoid(-(softplus(f_pre) dt + b)),
 * h' = a h + (1 - a) tanh(c_x + u h), J = a + (1 - a)(1 - n^2) u. */
static inline void cfc(real h, real fp, real cx, real dt, real b, real u, real *f, real *j) {
    real a = r_sigmoid(-(r_softplus(fp) * dt + b));
    real n = r_tanh(cx + u * h);
    *f = a * h + (1 - a) * n;
    if (j) *j = a + (1 - a) * (1 - n * n) * u;
}

/* step (+ Jacobian) of a scalar-diagonal cell at channel ch; wt points at the gates of one step */
static inline void diag_step(int kind, real h, const real *wt, int d, const real *params, int ch, real *f,
                             real *j) {
    if (kind == CELL_GRU_DIAG)
        gru_diag(h, wt[0], wt[d], wt[2 * (size_t)d], params[ch], params[d + ch], params[2 * d + ch], f, j);
    else if (kind == CELL_TITANS)
        titans(h, wt[0], wt[d], wt[2 * (size_t)d], wt[3 * (size_t)d], wt[4 * (size_t)d], params[ch],
               params[d + ch], f, j);
    else if (kind == CELL_CFC)
        cfc(h, wt[0], wt[d], wt[2 * (size_t)d], wt[3 * (size_t)d], params[ch], f, j);
    else
        nlru(h, wt[0], wt[d], params[ch], f, j);
}

/* ------------------------------------------------------------------ */
/* ParaLSTM (CIFG peephole LSTM, state (c, h), 2x2 block Jacobian)     */
/* ------------------------------------------------------------------ */

typedef struct {
    real c_new, h_new, f, z, o, hact;
} lstm_acts;

/* cells/para_lstm.py:202-232 (_recurrence): gates (f, z, o) = chunk3(wx), parameters
 * (a_f, a_z, a_o, c_f, c_o) clamped outside. */
static inline void lstm_step(real c, real h, real fx, real zx, real ox, const real p[5], lstm_acts *a) {
    a->f = r_sigmoid(p[0] * h + p[3] * c + fx);
    a->z = r_tanh(p[1] * h + zx);
    a->c_new = a->f * c + (1 - a->f) * a->z;
    a->o = r_sigmoid(p[2] * h + p[4] * a->c_new + ox);
    a->hact = r_tanh(a->c_new);
    a->h_new = a->o * a->hact;
}

/* cells/para_lstm.py:186-200 (step_with_jacobian, eq. 3.2b): J[out*2+in], slots (c, h). */
static inline void lstm_jac(const lstm_acts *a, real c, const real p[5], real J[4]) {
    real fp = a->f * (1 - a->f), zp = 1 - a->z * a->z, op = a->o * (1 - a->o), hp = 1 - a->hact * a->hact;
    real jcc = a->f + (c - a->z) * fp * p[3];
    real jch = (c - a->z) * fp * p[0] + (1 - a->f) * zp * p[1];
    J[0] = jcc;
    J[1] = jch;
    J[2] = (a->hact * op * p[4] + a->o * hp) * jcc;
    J[3] = a->hact * op * (p[2] + p[4] * jch) + a->o * hp * jch;
}

/* ------------------------------------------------------------------ */
/* ParaSLSTM mix='diag'                                                */
/* ------------------------------------------------------------------ */

typedef struct {
    real c_new, n_new, m_new, h_new;
    real i, f, z, o, denom, alpha, c, n;
} slstm_acts;

/* cells/para_slstm.py:347-384 (_acts_from_pre), slots (c, n, m, h). */
static inline void slstm_acts_from_pre(const real st[4], const real pre[4], real eps, slstm_acts *a) {
    real c = st[0], n = st[1], m = st[2];
    real zi = pre[0], zf = pre[1], zz = pre[2], zo = pre[3];
    real left = zf + m;
    real m_new = r_max(left, zi);
    a->alpha = (left > zi) ? (real)1 : ((left == zi) ? (real)0.5 : (real)0);
    a->i = r_exp(zi - m_new);
    a->f = r_exp(zf + m - m_new);
    a->z = r_tanh(zz);
    a->n_new = a->f * n + a->i;
    a->c_new = a->f * c + a->i * a->z;
    a->o = r_sigmoid(zo);
    a->denom = a->n_new + eps;
    a->h_new = a->o * (a->c_new / a->denom);
    a->m_new = m_new;
    a->c = c;
    a->n = n;
}

/* 4x4 Jacobian, row-major [out][in].  cells/para_slstm.py:399-446. */
static inline void slstm_jac(const slstm_acts *a, const real r[4], real J[16]) {
    real alpha = a->alpha, beta = 1 - alpha;
    real dm_dh = alpha * r[1] + beta * r[0];
    real di_dm = -a->i * alpha, df_dm = a->f * beta;
    real di_dh = a->i * (r[0] - dm_dh), df_dh = a->f * (r[1] - dm_dh);
    real dz_dh = (1 - a->z * a->z) * r[2];
    real do_dh = a->o * (1 - a->o) * r[3];
    real j_cm = df_dm * a->c + di_dm * a->z;
    real j_ch = df_dh * a->c + di_dh * a->z + a->i * dz_dh;
    real j_nm = df_dm * a->n + di_dm;
    real j_nh = df_dh * a->n + di_dh;
    real inv = a->o / a->denom;
    real dn = -a->o * a->c_new / (a->denom * a->denom);
    real du = a->c_new / a->denom;
    J[0] = a->f; J[1] = 0; J[2] = j_cm; J[3] = j_ch;
    J[4] = 0; J[5] = a->f; J[6] = j_nm; J[7] = j_nh;
    J[8] = 0; J[9] = 0; J[10] = alpha; J[11] = dm_dh;
    J[12] = inv * a->f; J[13] = dn * a->f; J[14] = inv * j_cm + dn * j_nm;
    J[15] = inv * j_ch + dn * j_nh + du * do_dh;
}

/* One frozen-gate pass for one (batch row, channel): solvers/slstm_picard.py:51-107.
 * pre is read with stride `ps` per time step for the 4 gates at offsets g*d.
 * If hprev_src != NULL the pass uses pre = wx + R*h_prev (slstm_picard.py:173-181),
 * h_prev[t] = hprev_src[(t-1)*hs] for t>0 and h0 (or 0) at t=0. */
static void slstm_frozen_channel(const real *wx, size_t ps, int d, int T, const real *r4,
                                 const real *hprev_src, size_t hs, const real h0[4], real eps,
                                 real *out /* T x 4, stride os */, size_t os, real *tmp /* 6T */) {
    real *p = tmp, *zi = tmp + T, *zf = tmp + 2 * (size_t)T, *zz = tmp + 3 * (size_t)T,
         *zo = tmp + 4 * (size_t)T, *mm = tmp + 5 * (size_t)T;
    real c0 = h0 ? h0[0] : 0, n0 = h0 ? h0[1] : 0, m0 = h0 ? h0[2] : 0, hh0 = h0 ? h0[3] : 0;
    for (int t = 0; t < T; ++t) {
        real hp = 0;
        if (hprev_src) hp = (t == 0) ? hh0 : hprev_src[(size_t)(t - 1) * hs];
        const real *w = wx + (size_t)t * ps;
        zi[t] = w[0] + (hprev_src ? r4[0] * hp : 0);
        zf[t] = w[(size_t)d] + (hprev_src ? r4[1] * hp : 0);
        zz[t] = w[2 * (size_t)d] + (hprev_src ? r4[2] * hp : 0);
        zo[t] = w[3 * (size_t)d] + (hprev_src ? r4[3] * hp : 0);
    }
    /* p = cumsum(z_f); m = p + max(cummax(z_i - p), m0) */
    real acc = 0, cm = 0;
    for (int t = 0; t < T; ++t) {
        acc += zf[t];
        p[t] = acc;
        real v = zi[t] - acc;
        cm = (t == 0) ? v : r_max(cm, v);
        mm[t] = acc + r_max(cm, m0);
    }
    real n = n0, c = c0, mprev = m0;
    for (int t = 0; t < T; ++t) {
        real it = r_exp(zi[t] - mm[t]);
        real ft = r_exp(zf[t] + mprev - mm[t]);
        real z = r_tanh(zz[t]);
        /* scan_diag(f, res): h_t = f_t h_{t-1} + res_t with the initial state
         * folded into res at t=0 (slstm_picard.py:83-86). */
        if (t == 0) {
            n = ft * n0 + it;
            c = ft * c0 + it * z;
        } else {
            n = ft * n + it;
            c = ft * c + it * z;
        }
        real o = r_sigmoid(zo[t]);
        real h = o * (c / (n + eps));
        real *o4 = out + (size_t)t * os;
        o4[0] = c; o4[(size_t)d] = n; o4[2 * (size_t)d] = mm[t]; o4[3 * (size_t)d] = h;
        mprev = mm[t];
    }
}

/* ------------------------------------------------------------------ */
/* ParaGRU mix='head' helpers (row-vector convention y = h A)          */
/* ------------------------------------------------------------------ */

/* y[o] = sum_i v[i] A[i][o]   (cells/para_gru.py:443-445 _head_mix) */
static void mix(const real *v, const real *A, int dh, real *y) {
    for (int o = 0; o < dh; ++o) y[o] = 0;
    for (int i = 0; i < dh; ++i) {
        real vi = v[i];
        const real *row = A + (size_t)i * dh;
        for (int o = 0; o < dh; ++o) y[o] += vi * row[o];
    }
}
/* y[i] = sum_o A[i][o] v[o]   (kernels/gru_head_factor.py:25-27 _mix_t) */
static void mix_t(const real *v, const real *A, int dh, real *y) {
    for (int i = 0; i < dh; ++i) {
        const real *row = A + (size_t)i * dh;
        real s = 0;
        for (int o = 0; o < dh; ++o) s += row[o] * v[o];
        y[i] = s;
    }
}

/* gates of one head at one step; cells/para_gru.py:468-479 */
static void gru_head_gates(const real *h, const real *zx, const real *rx, const real *nx,
                           const real *Az, const real *Ar, const real *An, int dh, real *z,
                           real *r, real *n, real *tmp) {
    mix(h, Az, dh, z);
    mix(h, Ar, dh, r);
    for (int k = 0; k < dh; ++k) {
        z[k] = r_sigmoid(z[k] + zx[k]);
        r[k] = r_sigmoid(r[k] + rx[k]);
        tmp[k] = h[k] * r[k];
    }
    mix(tmp, An, dh, n);
    for (int k = 0; k < dh; ++k) n[k] = r_tanh(n[k] + nx[k]);
}

/* J v ; kernels/gru_head_factor.py:31-71 */
static void gru_head_jvp(const real *h, const real *z, const real *r, const real *n,
                         const real *Az, const real *Ar, const real *An, int dh, const real *v,
                         real *out, real *t1, real *t2) {
    mix(v, Az, dh, t1); /* v A_z */
    mix(v, Ar, dh, t2); /* v A_r */
    for (int k = 0; k < dh; ++k) {
        real rp = r[k] * (1 - r[k]);
        t2[k] = r[k] * v[k] + h[k] * (rp * t2[k]); /* du_v */
    }
    real *t3 = out; /* reuse */
    mix(t2, An, dh, t3);
    for (int k = 0; k < dh; ++k) {
        real zp = z[k] * (1 - z[k]);
        real np_ = 1 - n[k] * n[k];
        real dz_v = zp * t1[k];
        real dn_v = np_ * t3[k];
        out[k] = (1 - z[k]) * v[k] + (n[k] - h[k]) * dz_v + z[k] * dn_v;
    }
}

/* J^T mu ; kernels/gru_head_factor.py:74-112 */
static void gru_head_jt(const real *h, const real *z, const real *r, const real *n,
                        const real *Az, const real *Ar, const real *An, int dh, const real *mu,
                        real *out, real *t1, real *t2, real *t3) {
    for (int k = 0; k < dh; ++k) {
        real zp = z[k] * (1 - z[k]);
        real np_ = 1 - n[k] * n[k];
        t1[k] = zp * ((n[k] - h[k]) * mu[k]); /* w_z */
        t2[k] = np_ * (z[k] * mu[k]);         /* w_n */
    }
    mix_t(t1, Az, dh, out);  /* t2 term: A_z w_z */
    mix_t(t2, An, dh, t3);   /* g_du */
    for (int k = 0; k < dh; ++k) {
        real rp = r[k] * (1 - r[k]);
        t1[k] = rp * (h[k] * t3[k]);
    }
    mix_t(t1, Ar, dh, t2);
    for (int k = 0; k < dh; ++k) out[k] = (1 - z[k]) * mu[k] + out[k] + r[k] * t3[k] + t2[k];
}

/* ------------------------------------------------------------------ */
/* Sequential unroll (solvers/sequential.py:24-120) on precomputed wx   */
/* ------------------------------------------------------------------ */

void oracle_sequential(int kind, const real *wx, const real *params, const real *h0, int B,
                       int T, int d, int n_heads, real eps, real *out) {
    const int G = gates_of(kind), S = slots_of(kind);
    if (kind == CELL_GRU_HEAD) {
        const int dh = d / n_heads;
        const real *Az = params, *Ar = params + (size_t)n_heads * dh * dh,
                   *An = params + 2 * (size_t)n_heads * dh * dh;
#pragma omp parallel for collapse(2) schedule(static)
        for (int b = 0; b < B; ++b)
            for (int hd = 0; hd < n_heads; ++hd) {
                real *buf = (real *)malloc(sizeof(real) * 5 * dh);
                real *h = buf, *z = buf + dh, *r = buf + 2 * dh, *n = buf + 3 * dh, *tmp = buf + 4 * dh;
                for (int k = 0; k < dh; ++k) h[k] = h0 ? h0[(size_t)b * d + hd * dh + k] : 0;
                for (int t = 0; t < T; ++t) {
                    const real *w = wx + ((size_t)b * T + t) * 3 * d + hd * dh;
                    gru_head_gates(h, w, w + d, w + 2 * d, Az + (size_t)hd * dh * dh,
                                   Ar + (size_t)hd * dh * dh, An + (size_t)hd * dh * dh, dh, z, r, n, tmp);
                    real *o = out + ((size_t)b * T + t) * d + hd * dh;
                    for (int k = 0; k < dh; ++k) {
                        h[k] = h[k] + z[k] * (n[k] - h[k]);
                        o[k] = h[k];
                    }
                }
                free(buf);
            }
        return;
    }
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < B; ++b)
        for (int ch = 0; ch < d; ++ch) {
            const real *w = wx + (size_t)b * T * G * d + ch;
            real *o = out + (size_t)b * T * S * d + ch;
            if (kind == CELL_SLSTM_DIAG) {
                real st[4] = {0, 0, 0, 0};
                if (h0) for (int s = 0; s < 4; ++s) st[s] = h0[((size_t)b * 4 + s) * d + ch];
                real r4[4] = {params[ch], params[d + ch], params[2 * d + ch], params[3 * d + ch]};
                for (int t = 0; t < T; ++t) {
                    const real *wt = w + (size_t)t * 4 * d;
                    real pre[4];
                    for (int g = 0; g < 4; ++g) pre[g] = wt[(size_t)g * d] + r4[g] * st[3];
                    slstm_acts a;
                    slstm_acts_from_pre(st, pre, eps, &a);
                    st[0] = a.c_new; st[1] = a.n_new; st[2] = a.m_new; st[3] = a.h_new;
                    for (int s = 0; s < 4; ++s) o[((size_t)t * 4 + s) * d] = st[s];
                }
            } else if (kind == CELL_LSTM) {
                real p5[5];
                for (int k = 0; k < 5; ++k) p5[k] = params[(size_t)k * d + ch];
                real c = h0 ? h0[((size_t)b * 2 + 0) * d + ch] : 0, h = h0 ? h0[((size_t)b * 2 + 1) * d + ch] : 0;
                for (int t = 0; t < T; ++t) {
                    const real *wt = w + (size_t)t * 3 * d;
                    lstm_acts a;
                    lstm_step(c, h, wt[0], wt[d], wt[2 * (size_t)d], p5, &a);
                    c = a.c_new;
                    h = a.h_new;
                    o[((size_t)t * 2 + 0) * d] = c;
                    o[((size_t)t * 2 + 1) * d] = h;
                }
            } else {
                real h = h0 ? h0[(size_t)b * d + ch] : 0;
                for (int t = 0; t < T; ++t) {
                    const real *wt = w + (size_t)t * G * d;
                    real f;
                    diag_step(kind, h, wt, d, params, ch, &f, NULL);
                    h = f;
                    o[(size_t)t * d] = h;
                }
            }
        }
}

/* ------------------------------------------------------------------ */
/* Eager Newton (solvers/newton/__init__.py:467-549)                   */
/* ------------------------------------------------------------------ */

/* One Newton linearisation + scan + update over the whole batch.
 * Returns max|F| of the INPUT trajectory (reference: residual = pred - states,
 * __init__.py:525-529).  When apply==0 only the residual is evaluated
 * (_fill_stats, __init__.py:602-606).
 * delta_t = J_t delta_{t-1} + F_t with delta_{-1}=0 (solvers/scan.py:3-4),
 * states += omega*delta (__init__.py:537-540). */
static real newton_pass(int kind, const real *wx, const real *params, const real *h0, int B, int T,
                        int d, int n_heads, real omega, real eps, real *states, int apply) {
    const int G = gates_of(kind);
    real gmax = 0;
    if (kind == CELL_GRU_HEAD) {
        const int dh = d / n_heads;
        const size_t asz = (size_t)n_heads * dh * dh;
#pragma omp parallel
        {
            real lmax = 0;
            real *buf = (real *)malloc(sizeof(real) * 9 * dh);
            real *hp = buf, *z = buf + dh, *r = buf + 2 * dh, *n = buf + 3 * dh, *tmp = buf + 4 * dh,
                 *dl = buf + 5 * dh, *dn_ = buf + 6 * dh, *t1 = buf + 7 * dh, *t2 = buf + 8 * dh;
#pragma omp for collapse(2) schedule(static)
            for (int b = 0; b < B; ++b)
                for (int hd = 0; hd < n_heads; ++hd) {
                    const real *Az = params + (size_t)hd * dh * dh, *Ar = Az + asz, *An = Ar + asz;
                    for (int k = 0; k < dh; ++k) {
                        hp[k] = h0 ? h0[(size_t)b * d + hd * dh + k] : 0;
                        dl[k] = 0;
                    }
                    for (int t = 0; t < T; ++t) {
                        const real *w = wx + ((size_t)b * T + t) * 3 * d + hd * dh;
                        real *st = states + ((size_t)b * T + t) * d + hd * dh;
                        gru_head_gates(hp, w, w + d, w + 2 * d, Az, Ar, An, dh, z, r, n, tmp);
                        if (apply) gru_head_jvp(hp, z, r, n, Az, Ar, An, dh, dl, dn_, t1, t2);
                        for (int k = 0; k < dh; ++k) {
                            real pred = hp[k] + z[k] * (n[k] - hp[k]);
                            real F = pred - st[k];
                            lmax = nanmax(lmax, r_abs(F));
                            hp[k] = st[k]; /* old trajectory value feeds the next step */
                            if (apply) {
                                dl[k] = dn_[k] + F;
                                st[k] = st[k] + omega * dl[k];
                            }
                        }
                    }
                }
            free(buf);
#pragma omp critical
            gmax = nanmax(gmax, lmax);
        }
        return gmax;
    }
#pragma omp parallel
    {
        real lmax = 0;
#pragma omp for collapse(2) schedule(static)
        for (int b = 0; b < B; ++b)
            for (int ch = 0; ch < d; ++ch) {
                const real *w = wx + (size_t)b * T * G * d + ch;
                if (kind == CELL_SLSTM_DIAG) {
                    real *s = states + (size_t)b * T * 4 * d + ch;
                    real r4[4] = {params[ch], params[d + ch], params[2 * d + ch], params[3 * d + ch]};
                    real prev[4] = {0, 0, 0, 0}, dl[4] = {0, 0, 0, 0};
                    if (h0) for (int k = 0; k < 4; ++k) prev[k] = h0[((size_t)b * 4 + k) * d + ch];
                    for (int t = 0; t < T; ++t) {
                        const real *wt = w + (size_t)t * 4 * d;
                        real pre[4], J[16], cur[4], F[4], nd[4];
                        for (int g = 0; g < 4; ++g) pre[g] = wt[(size_t)g * d] + r4[g] * prev[3];
                        slstm_acts a;
                        slstm_acts_from_pre(prev, pre, eps, &a);
                        real pred[4] = {a.c_new, a.n_new, a.m_new, a.h_new};
                        for (int k = 0; k < 4; ++k) {
                            cur[k] = s[((size_t)t * 4 + k) * d];
                            F[k] = pred[k] - cur[k];
                            lmax = nanmax(lmax, r_abs(F[k]));
                        }
                        if (apply) {
                            slstm_jac(&a, r4, J);
                            for (int o = 0; o < 4; ++o) {
                                real acc = 0;
                                for (int i = 0; i < 4; ++i) acc += J[o * 4 + i] * dl[i];
                                nd[o] = acc + F[o];
                            }
                            for (int k = 0; k < 4; ++k) {
                                dl[k] = nd[k];
                                s[((size_t)t * 4 + k) * d] = cur[k] + omega * dl[k];
                            }
                        }
                        for (int k = 0; k < 4; ++k) prev[k] = cur[k];
                    }
                } else if (kind == CELL_LSTM) {
                    real *s = states + (size_t)b * T * 2 * d + ch;
                    real p5[5];
                    for (int k = 0; k < 5; ++k) p5[k] = params[(size_t)k * d + ch];
                    real pc = h0 ? h0[((size_t)b * 2 + 0) * d + ch] : 0, ph = h0 ? h0[((size_t)b * 2 + 1) * d + ch] : 0;
                    real dc = 0, dh = 0;
                    for (int t = 0; t < T; ++t) {
                        const real *wt = w + (size_t)t * 3 * d;
                        lstm_acts a;
                        lstm_step(pc, ph, wt[0], wt[d], wt[2 * (size_t)d], p5, &a);
                        real cc = s[((size_t)t * 2 + 0) * d], ch_ = s[((size_t)t * 2 + 1) * d];
                        real Fc = a.c_new - cc, Fh = a.h_new - ch_;
                        lmax = nanmax(lmax, r_abs(Fc));
                        lmax = nanmax(lmax, r_abs(Fh));
                        if (apply) {
                            real J[4];
                            lstm_jac(&a, pc, p5, J);
                            real nc = J[0] * dc + J[1] * dh + Fc, nh = J[2] * dc + J[3] * dh + Fh;
                            dc = nc;
                            dh = nh;
                            s[((size_t)t * 2 + 0) * d] = cc + omega * dc;
                            s[((size_t)t * 2 + 1) * d] = ch_ + omega * dh;
                        }
                        pc = cc;
                        ph = ch_;
                    }
                } else {
                    real *s = states + (size_t)b * T * d + ch;
                    real prev = h0 ? h0[(size_t)b * d + ch] : 0, dl = 0;
                    for (int t = 0; t < T; ++t) {
                        const real *wt = w + (size_t)t * G * d;
                        real f, j;
                        diag_step(kind, prev, wt, d, params, ch, &f, &j);
                        real cur = s[(size_t)t * d];
                        real F = f - cur;
                        lmax = nanmax(lmax, r_abs(F));
                        if (apply) {
                            dl = j * dl + F;
                            s[(size_t)t * d] = cur + omega * dl;
                        }
                        prev = cur;
                    }
                }
            }
#pragma omp critical
        gmax = nanmax(gmax, lmax);
    }
    return gmax;
}

/* Initial guess.  GRU / NLRU: App. A guess f(0, x_t) with h0 only at t=0
 * (__init__.py:484-493, 925-940).  sLSTM: zero-hidden frozen-gate scan followed
 * by `picard` frozen-gate passes (solvers/newton/picard.py:161-186,
 * solvers/slstm_picard.py:158-181). */
static void newton_guess(int kind, const real *wx, const real *params, const real *h0, int B, int T,
                         int d, int n_heads, int picard, real eps, real *states) {
    const int G = gates_of(kind);
    if (kind == CELL_GRU_HEAD) {
        const int dh = d / n_heads;
        const size_t asz = (size_t)n_heads * dh * dh;
#pragma omp parallel for collapse(2) schedule(static)
        for (int b = 0; b < B; ++b)
            for (int hd = 0; hd < n_heads; ++hd) {
                real *buf = (real *)malloc(sizeof(real) * 5 * dh);
                real *hp = buf, *z = buf + dh, *r = buf + 2 * dh, *n = buf + 3 * dh, *tmp = buf + 4 * dh;
                const real *Az = params + (size_t)hd * dh * dh, *Ar = Az + asz, *An = Ar + asz;
                for (int t = 0; t < T; ++t) {
                    for (int k = 0; k < dh; ++k)
                        hp[k] = (t == 0 && h0) ? h0[(size_t)b * d + hd * dh + k] : 0;
                    const real *w = wx + ((size_t)b * T + t) * 3 * d + hd * dh;
                    gru_head_gates(hp, w, w + d, w + 2 * d, Az, Ar, An, dh, z, r, n, tmp);
                    real *st = states + ((size_t)b * T + t) * d + hd * dh;
                    for (int k = 0; k < dh; ++k) st[k] = hp[k] + z[k] * (n[k] - hp[k]);
                }
                free(buf);
            }
        return;
    }
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < B; ++b)
        for (int ch = 0; ch < d; ++ch) {
            const real *w = wx + (size_t)b * T * G * d + ch;
            if (kind == CELL_SLSTM_DIAG) {
                real *s = states + (size_t)b * T * 4 * d + ch;
                real r4[4] = {params[ch], params[d + ch], params[2 * d + ch], params[3 * d + ch]};
                real h04[4];
                if (h0) for (int k = 0; k < 4; ++k) h04[k] = h0[((size_t)b * 4 + k) * d + ch];
                real *tmp = (real *)malloc(sizeof(real) * (6 * (size_t)T + 4 * (size_t)T));
                real *alt = tmp + 6 * (size_t)T; /* T x 4 compact copy of the previous pass */
                slstm_frozen_channel(w, (size_t)4 * d, d, T, r4, NULL, 0, h0 ? h04 : NULL, eps, s,
                                     (size_t)4 * d, tmp);
                for (int p = 0; p < picard; ++p) {
                    for (int t = 0; t < T; ++t) alt[t] = s[((size_t)t * 4 + 3) * d];
                    slstm_frozen_channel(w, (size_t)4 * d, d, T, r4, alt, 1, h0 ? h04 : NULL, eps, s,
                                         (size_t)4 * d, tmp);
                }
                free(tmp);
            } else if (kind == CELL_LSTM) {
                real *s = states + (size_t)b * T * 2 * d + ch;
                real p5[5];
                for (int k = 0; k < 5; ++k) p5[k] = params[(size_t)k * d + ch];
                for (int t = 0; t < T; ++t) {
                    const real *wt = w + (size_t)t * 3 * d;
                    real c = (t == 0 && h0) ? h0[((size_t)b * 2 + 0) * d + ch] : 0;
                    real h = (t == 0 && h0) ? h0[((size_t)b * 2 + 1) * d + ch] : 0;
                    lstm_acts a;
                    lstm_step(c, h, wt[0], wt[d], wt[2 * (size_t)d], p5, &a);
                    s[((size_t)t * 2 + 0) * d] = a.c_new;
                    s[((size_t)t * 2 + 1) * d] = a.h_new;
                }
            } else {
                real *s = states + (size_t)b * T * d + ch;
                for (int t = 0; t < T; ++t) {
                    const real *wt = w + (size_t)t * G * d;
                    real hp = (t == 0 && h0) ? h0[(size_t)b * d + ch] : 0, f;
                    diag_step(kind, hp, wt, d, params, ch, &f, NULL);
                    s[(size_t)t * d] = f;
                }
            }
        }
}

/* Initial guess only (exposed so that tests can check the Picard warm start). */
void oracle_guess(int kind, const real *wx, const real *params, const real *h0, int B, int T, int d,
                  int n_heads, int picard, real eps, real *states) {
    newton_guess(kind, wx, params, h0, B, T, d, n_heads, picard, eps, states);
}

/* Final residual max|F(H)| (solvers/newton/__init__.py:602-606). */
real oracle_residual(int kind, const real *wx, const real *params, const real *h0, int B, int T,
                     int d, int n_heads, real eps, const real *states) {
    return newton_pass(kind, wx, params, h0, B, T, d, n_heads, 1, eps, (real *)states, 0);
}

/* Full eager solve.  early_atol < 0 disables the early stop (fixed K, the
 * behaviour of the reference's fused path, __init__.py:426-441).  history has
 * room for max_iters entries; *iters_out = number of residual evaluations in the
 * loop; returns the final max|F(H_K)| as _fill_stats reports it. */
real oracle_newton(int kind, const real *wx, const real *params, const real *h0, int B, int T, int d,
                   int n_heads, int max_iters, int picard, real omega, real eps, real early_atol,
                   real *states, real *history, int *iters_out) {
    newton_guess(kind, wx, params, h0, B, T, d, n_heads, picard, eps, states);
    int iters = 0;
    const size_t nel = (size_t)B * T * slots_of(kind) * d;
    real *backup = NULL;
    if (early_atol >= 0) backup = (real *)malloc(sizeof(real) * nel);
    for (int it = 0; it < max_iters; ++it) {
        if (backup) memcpy(backup, states, sizeof(real) * nel);
        real res = newton_pass(kind, wx, params, h0, B, T, d, n_heads, omega, eps, states, 1);
        history[it] = res;
        iters = it + 1;
        if (early_atol >= 0 && res < early_atol) {
            /* the reference stops BEFORE applying the update (__init__.py:526-533) */
            memcpy(states, backup, sizeof(real) * nel);
            break;
        }
    }
    if (backup) free(backup);
    if (early_atol < 0) iters = max_iters;
    *iters_out = iters;
    return newton_pass(kind, wx, params, h0, B, T, d, n_heads, 1, eps, states, 0);
}

/* ------------------------------------------------------------------ */
/* Backward: eq. 2.6 reverse scan + packed VJP                          */
/* ------------------------------------------------------------------ */

/* mu_t = J_{t+1}^T mu_{t+1} + g_t (solvers/scan.py:126-178), grad_h0 = J_0^T mu_0
 * (solvers/newton/dispatch.py:406-441), then the closed-form cell VJP at
 * (h_prev detached, wx) with cotangent mu:
 *   GRU diag  kernels/vjp_gru.py:107-138
 *   NLRU      kernels/vjp_nlru.py:88-108
 *   sLSTM     kernels/vjp_slstm.py:170-231
 *   GRU head  kernels/vjp_gru.py:141-221
 * Outputs: g_wx (B,T,G*d); g_params summed over (B,T) in the same packing as
 * params; g_h0 (B,S,d); mu_out optional (B,T,S,d). */
void oracle_backward(int kind, const real *states, const real *wx, const real *params,
                     const real *h0, const real *grad_states, int B, int T, int d, int n_heads,
                     real eps, real *g_wx, real *g_params, real *g_h0, real *mu_out) {
    const int G = gates_of(kind);
    if (kind == CELL_GRU_HEAD) {
        const int dh = d / n_heads;
        const size_t asz = (size_t)n_heads * dh * dh;
        memset(g_params, 0, sizeof(real) * 3 * asz);
#pragma omp parallel for schedule(static)
        for (int hd = 0; hd < n_heads; ++hd) {
            const real *Az = params + (size_t)hd * dh * dh, *Ar = Az + asz, *An = Ar + asz;
            real *gAz = g_params + (size_t)hd * dh * dh, *gAr = gAz + asz, *gAn = gAr + asz;
            real *buf = (real *)malloc(sizeof(real) * 12 * dh);
            real *hp = buf, *z = buf + dh, *r = buf + 2 * dh, *n = buf + 3 * dh, *tmp = buf + 4 * dh,
                 *mu = buf + 5 * dh, *jt = buf + 6 * dh, *t1 = buf + 7 * dh, *t2 = buf + 8 * dh,
                 *t3 = buf + 9 * dh, *dnp = buf + 10 * dh, *du = buf + 11 * dh;
            for (int b = 0; b < B; ++b) {
                for (int k = 0; k < dh; ++k) mu[k] = 0;
                for (int t = T - 1; t >= 0; --t) {
                    const real *g = grad_states + ((size_t)b * T + t) * d + hd * dh;
                    /* mu_t = (J_{t+1}^T mu_{t+1}) + g_t ; jt holds the first term */
                    for (int k = 0; k < dh; ++k) mu[k] = (t == T - 1 ? 0 : jt[k]) + g[k];
                    if (mu_out)
                        for (int k = 0; k < dh; ++k) mu_out[((size_t)b * T + t) * d + hd * dh + k] = mu[k];
                    for (int k = 0; k < dh; ++k)
                        hp[k] = t > 0 ? states[((size_t)b * T + t - 1) * d + hd * dh + k]
                                      : (h0 ? h0[(size_t)b * d + hd * dh + k] : 0);
                    const real *w = wx + ((size_t)b * T + t) * 3 * d + hd * dh;
                    gru_head_gates(hp, w, w + d, w + 2 * d, Az, Ar, An, dh, z, r, n, tmp);
                    /* VJP */
                    real *gw = g_wx + ((size_t)b * T + t) * 3 * d + hd * dh;
                    for (int k = 0; k < dh; ++k) {
                        real dz = mu[k] * (n[k] - hp[k]);
                        dnp[k] = mu[k] * z[k] * (1 - n[k] * n[k]);
                        gw[k] = dz * z[k] * (1 - z[k]);
                        gw[2 * (size_t)d + k] = dnp[k];
                    }
                    mix_t(dnp, An, dh, du); /* d_u = d_npre A_n^T */
                    for (int k = 0; k < dh; ++k) gw[d + k] = du[k] * hp[k] * r[k] * (1 - r[k]);
                    for (int i = 0; i < dh; ++i)
                        for (int o = 0; o < dh; ++o) {
                            gAz[(size_t)i * dh + o] += hp[i] * gw[o];
                            gAr[(size_t)i * dh + o] += hp[i] * gw[d + o];
                            gAn[(size_t)i * dh + o] += hp[i] * r[i] * dnp[o];
                        }
                    gru_head_jt(hp, z, r, n, Az, Ar, An, dh, mu, jt, t1, t2, t3);
                }
                if (g_h0) for (int k = 0; k < dh; ++k) g_h0[(size_t)b * d + hd * dh + k] = jt[k];
            }
            free(buf);
        }
        return;
    }
    const int NP = (kind == CELL_GRU_DIAG) ? 3 : ((kind == CELL_NLRU || kind == CELL_CFC) ? 1 : (kind == CELL_TITANS ? 2 : (kind == CELL_LSTM ? 5 : 4)));
#pragma omp parallel for schedule(static)
    for (int ch = 0; ch < d; ++ch) {
        real gp[5] = {0, 0, 0, 0, 0};
        for (int b = 0; b < B; ++b) {
            const real *w = wx + (size_t)b * T * G * d + ch;
            real *gw = g_wx + (size_t)b * T * G * d + ch;
            if (kind == CELL_SLSTM_DIAG) {
                const real *s = states + (size_t)b * T * 4 * d + ch;
                const real *g = grad_states + (size_t)b * T * 4 * d + ch;
                real r4[4] = {params[ch], params[d + ch], params[2 * d + ch], params[3 * d + ch]};
                real jt[4] = {0, 0, 0, 0};
                for (int t = T - 1; t >= 0; --t) {
                    real mu[4], prev[4], pre[4];
                    for (int k = 0; k < 4; ++k) {
                        mu[k] = (t == T - 1 ? 0 : jt[k]) + g[((size_t)t * 4 + k) * d];
                        prev[k] = t > 0 ? s[((size_t)(t - 1) * 4 + k) * d]
                                        : (h0 ? h0[((size_t)b * 4 + k) * d + ch] : 0);
                        if (mu_out) mu_out[((size_t)b * T + t) * 4 * d + (size_t)k * d + ch] = mu[k];
                    }
                    const real *wt = w + (size_t)t * 4 * d;
                    for (int q = 0; q < 4; ++q) pre[q] = wt[(size_t)q * d] + r4[q] * prev[3];
                    slstm_acts a;
                    slstm_acts_from_pre(prev, pre, eps, &a);
                    real J[16];
                    slstm_jac(&a, r4, J);
                    real d_o = mu[3] * (a.c_new / a.denom);
                    real d_cn = mu[0] + mu[3] * (a.o / a.denom);
                    real d_nn = mu[1] + mu[3] * (-a.o * a.c_new / (a.denom * a.denom));
                    real d_f = d_cn * a.c + d_nn * a.n;
                    real d_i = d_cn * a.z + d_nn;
                    real d_z = d_cn * a.i;
                    real d_zo = d_o * a.o * (1 - a.o);
                    real d_zz = d_z * (1 - a.z * a.z);
                    real d_mn = mu[2] - d_i * a.i - d_f * a.f;
                    real d_zi = d_i * a.i + d_mn * (1 - a.alpha);
                    real d_zf = d_f * a.f + d_mn * a.alpha;
                    real *gwt = gw + (size_t)t * 4 * d;
                    gwt[0] = d_zi; gwt[(size_t)d] = d_zf; gwt[2 * (size_t)d] = d_zz; gwt[3 * (size_t)d] = d_zo;
                    gp[0] += d_zi * prev[3]; gp[1] += d_zf * prev[3];
                    gp[2] += d_zz * prev[3]; gp[3] += d_zo * prev[3];
                    for (int i = 0; i < 4; ++i) {
                        real acc = 0;
                        for (int o = 0; o < 4; ++o) acc += J[o * 4 + i] * mu[o];
                        jt[i] = acc;
                    }
                }
                if (g_h0) for (int k = 0; k < 4; ++k) g_h0[((size_t)b * 4 + k) * d + ch] = jt[k];
            } else if (kind == CELL_LSTM) {
                /* eq. 2.6 with 2x2 blocks (solvers/scan.py:150-164) + the packed VJP of
                 * kernels/vjp_lstm.py (lstm_recurrence_vjp_eager) */
                const real *s = states + (size_t)b * T * 2 * d + ch;
                const real *g = grad_states + (size_t)b * T * 2 * d + ch;
                real p5[5];
                for (int k = 0; k < 5; ++k) p5[k] = params[(size_t)k * d + ch];
                real jc = 0, jh = 0;
                for (int t = T - 1; t >= 0; --t) {
                    real mc = (t == T - 1 ? 0 : jc) + g[((size_t)t * 2 + 0) * d];
                    real mh = (t == T - 1 ? 0 : jh) + g[((size_t)t * 2 + 1) * d];
                    if (mu_out) {
                        mu_out[((size_t)b * T + t) * 2 * d + ch] = mc;
                        mu_out[((size_t)b * T + t) * 2 * d + d + ch] = mh;
                    }
                    real pc = t > 0 ? s[((size_t)(t - 1) * 2 + 0) * d] : (h0 ? h0[((size_t)b * 2 + 0) * d + ch] : 0);
                    real ph = t > 0 ? s[((size_t)(t - 1) * 2 + 1) * d] : (h0 ? h0[((size_t)b * 2 + 1) * d + ch] : 0);
                    const real *wt = w + (size_t)t * 3 * d;
                    lstm_acts a;
                    lstm_step(pc, ph, wt[0], wt[d], wt[2 * (size_t)d], p5, &a);
                    real J[4];
                    lstm_jac(&a, pc, p5, J);
                    real d_opre = mh * a.hact * a.o * (1 - a.o);
                    real d_cn = mc + mh * a.o * (1 - a.hact * a.hact) + d_opre * p5[4];
                    real d_fpre = d_cn * (pc - a.z) * a.f * (1 - a.f);
                    real d_zpre = d_cn * (1 - a.f) * (1 - a.z * a.z);
                    real *gwt = gw + (size_t)t * 3 * d;
                    gwt[0] = d_fpre; gwt[d] = d_zpre; gwt[2 * (size_t)d] = d_opre;
                    gp[0] += d_fpre * ph; gp[1] += d_zpre * ph; gp[2] += d_opre * ph;
                    gp[3] += d_fpre * pc; gp[4] += d_opre * a.c_new;
                    jc = J[0] * mc + J[2] * mh;
                    jh = J[1] * mc + J[3] * mh;
                }
                if (g_h0) {
                    g_h0[((size_t)b * 2 + 0) * d + ch] = jc;
                    g_h0[((size_t)b * 2 + 1) * d + ch] = jh;
                }
            } else {
                const real *s = states + (size_t)b * T * d + ch;
                const real *g = grad_states + (size_t)b * T * d + ch;
                real jt = 0;
                for (int t = T - 1; t >= 0; --t) {
                    real mu = (t == T - 1 ? 0 : jt) + g[(size_t)t * d];
                    if (mu_out) mu_out[((size_t)b * T + t) * d + ch] = mu;
                    real hp = t > 0 ? s[(size_t)(t - 1) * d] : (h0 ? h0[(size_t)b * d + ch] : 0);
                    const real *wt = w + (size_t)t * G * d;
                    real *gwt = gw + (size_t)t * G * d;
                    real f, j;
                    if (kind == CELL_GRU_DIAG) {
                        real az = params[ch], ar = params[d + ch], an = params[2 * d + ch];
                        gru_diag(hp, wt[0], wt[d], wt[2 * (size_t)d], az, ar, an, &f, &j);
                        real z = r_sigmoid(az * hp + wt[0]);
                        real r = r_sigmoid(ar * hp + wt[d]);
                        real n = r_tanh(an * (hp * r) + wt[2 * (size_t)d]);
                        real d_z = mu * (n - hp);
                        real d_npre = mu * z * (1 - n * n);
                        real d_zpre = d_z * z * (1 - z);
                        real d_rpre = (d_npre * an * hp) * r * (1 - r);
                        gwt[0] = d_zpre; gwt[d] = d_rpre; gwt[2 * (size_t)d] = d_npre;
                        gp[0] += d_zpre * hp; gp[1] += d_rpre * hp; gp[2] += d_npre * (hp * r);
                    } else if (kind == CELL_TITANS) {
                        /* closed form of the autograd VJP the reference takes through step
                         * (solvers/vjp.py:77-98) */
                        real u = params[ch], r = params[d + ch];
                        real k = wt[2 * (size_t)d], v = wt[3 * (size_t)d];
                        titans(hp, wt[0], wt[d], k, v, wt[4 * (size_t)d], u, r, &f, &j);
                        real alpha = r_sigmoid(wt[0]), theta = r_softplus(wt[d]);
                        real n = r_tanh(wt[4 * (size_t)d] + r * hp);
                        real err = hp * k - v;
                        gwt[0] = -mu * hp * alpha * (1 - alpha);
                        gwt[d] = -mu * err * k * r_sigmoid(wt[d]);
                        gwt[2 * (size_t)d] = -mu * theta * (err + hp * k);
                        gwt[3 * (size_t)d] = mu * theta * k;
                        gwt[4 * (size_t)d] = mu * u * (1 - n * n);
                        gp[0] += mu * n;
                        gp[1] += gwt[4 * (size_t)d] * hp;
                    } else if (kind == CELL_CFC) {
                        /* kernels/vjp_cfc.py:102-128 (cfc_recurrence_vjp_eager) */
                        real u = params[ch];
                        real fp = wt[0], dt = wt[2 * (size_t)d], bb = wt[3 * (size_t)d];
                        cfc(hp, fp, wt[d], dt, bb, u, &f, &j);
                        real soft = r_softplus(fp);
                        real a = r_sigmoid(-(soft * dt + bb));
                        real n = r_tanh(wt[d] + u * hp);
                        real d_h_da = mu * (hp - n), a1a = a * (1 - a);
                        real d_npre = mu * (1 - a) * (1 - n * n);
                        gwt[0] = d_h_da * a1a * (-dt) * r_sigmoid(fp);
                        gwt[d] = d_npre;
                        gwt[2 * (size_t)d] = d_h_da * a1a * (-soft);
                        gwt[3 * (size_t)d] = d_h_da * a1a * (-1);
                        gp[0] += d_npre * hp;
                    } else {
                        real u = params[ch];
                        nlru(hp, wt[0], wt[d], u, &f, &j);
                        real a = r_sigmoid(wt[0]);
                        real n = r_tanh(wt[d] + u * hp);
                        real d_a = mu * (hp - n) * a * (1 - a);
                        real d_c = mu * (1 - a) * (1 - n * n);
                        gwt[0] = d_a; gwt[d] = d_c;
                        gp[0] += d_c * hp;
                    }
                    jt = j * mu;
                }
                if (g_h0) g_h0[(size_t)b * d + ch] = jt;
            }
        }
        for (int p = 0; p < NP; ++p) g_params[(size_t)p * d + ch] = gp[p];
    }
}

/* ------------------------------------------------------------------ */
/* Time-shard helpers for the multi-rank tests                          */
/* ------------------------------------------------------------------ */

/* Contiguous time shards, remainder on the last rank
 * (solvers/seq_parallel.py:126-138 time_shard_bounds). */
void oracle_time_shard_bounds(int T, int world, int rank, int *start, int *end) {
    int base = T / world;
    *start = rank * base;
    *end = (rank == world - 1) ? T : (rank + 1) * base;
}
