// Per-step math of ParaLSTM (CIFG peephole LSTM with diagonal recurrence; state slots (c, h), gates
// (f, z, o), parameters (a_f, a_z, a_o, c_f, c_o)), shared by the look-back kernels
// (lstm_kernels.cu) and the pipelined persistent kernels (lstm_pipe.cu).
// Reference behaviour restated: cells/para_lstm.py:154-232 (step and 2x2 block Jacobian).
#pragma once
#include "common.cuh"

namespace prb {

struct LstmActs {
    float f, z, o, hact, cn, hn;
};

__device__ __forceinline__ void lstm_step(float c, float h, const float (&g)[3], const float (&p)[5],
                                          LstmActs& a) {
    a.f = sigmoid_f(fmaf(p[0], h, fmaf(p[3], c, g[0])));
    a.z = tanh_f(fmaf(p[1], h, g[1]));
    a.cn = fmaf(a.f, c - a.z, a.z);  // f c + (1 - f) z
    a.o = sigmoid_f(fmaf(p[2], h, fmaf(p[4], a.cn, g[2])));
    a.hact = tanh_f(a.cn);
    a.hn = a.o * a.hact;
}

// J[out*2 + in] over slots (c, h)
__device__ __forceinline__ void lstm_jac(const LstmActs& a, float c, const float (&p)[5], float (&J)[4]) {
    const float fp = a.f * (1.f - a.f), zp = 1.f - a.z * a.z, op = a.o * (1.f - a.o), hp = 1.f - a.hact * a.hact;
    const float jcc = fmaf((c - a.z) * fp, p[3], a.f);
    const float jch = fmaf((c - a.z) * fp, p[0], (1.f - a.f) * zp * p[1]);
    const float pk = fmaf(a.hact * op, p[4], a.o * hp);
    J[0] = jcc;
    J[1] = jch;
    J[2] = pk * jcc;
    J[3] = fmaf(a.hact * op, p[2], pk * jch);
}

}  // namespace prb
