"""CPU stand-in for the per-rank scan kernels (ParaGRU mix='diag' and ParaSLSTM mix='diag'), used
to test the time-sharded driver's collective choreography with gloo ranks and no GPU.  Plain
PyTorch loops over time, float64 inside.  Test code: the product path never imports it."""

import torch

from pararnn_b200.seq_shard import NS, NV


def _affine_apply(m, v):
    """m (B, n*n + n, d) row-major matrix then offset; v (B, n, d)."""
    n = v.shape[1]
    M = m[:, : n * n].reshape(m.shape[0], n, n, -1)
    return torch.einsum("boid,bid->bod", M, v) + m[:, n * n:]


def _picard_apply(m, v):
    """m (B, 4, d) = (a, b, N, C); v (B, 3, d) = (c, n, m)."""
    a, b, N, C = m[:, 0], m[:, 1], m[:, 2], m[:, 3]
    am = a + v[:, 2]
    mo = torch.maximum(am, b)
    s1 = torch.exp(am - mo)
    s2 = torch.where(torch.isinf(b), torch.zeros_like(b), torch.exp(b - mo))
    return torch.stack([v[:, 0] * s1 + C * s2, v[:, 1] * s1 + N * s2, mo], dim=1)


class CpuShardOps:
    def __init__(self, kind, wx, rec, eps, omega):
        assert kind in ("gru_diag", "slstm_diag")
        self.kind, self.wx, self.omega, self.eps = kind, wx.double(), float(omega), float(eps)
        self.B, self.T = wx.shape[:2]
        self.d = wx.shape[2] // (3 if kind == "gru_diag" else 4)
        self.dev = wx.device
        self.slots, self.monoid = (1, "affine1") if kind == "gru_diag" else (4, "affine4")
        self.n_seg = 1
        self.par = [p.double() for p in rec] if kind == "gru_diag" else rec[0].double()
        self.bits = torch.zeros(20, dtype=torch.int32)

    def new_traj(self):
        shape = (self.B, self.T, self.d) if self.slots == 1 else (self.B, self.T, 4, self.d)
        return torch.empty(shape, dtype=torch.float64)

    new_out = new_traj

    def stats_bits(self):
        return self.bits

    def _zeros(self, *shape):
        return torch.zeros(*shape, dtype=torch.float64)

    def _bump(self, slot, value):
        as_bits = torch.tensor(float(value), dtype=torch.float32).view(torch.int32)
        self.bits[slot] = torch.maximum(self.bits[slot], as_bits)

    def fold(self, monoid, gathered, rank, world, reverse):
        first, step = (world - 1, -1) if reverse else (0, 1)
        vec = gathered[first][:, : NS[monoid]].double().clone()
        q = first + step
        while q != rank:
            m = gathered[q].double()
            vec = _picard_apply(m, vec) if monoid == "picard" else _affine_apply(m[:, : NV[monoid]], vec)
            q += step
        return vec

    # ------------------------------------------------------------------ GRU diag
    def _eval(self, h, t):
        az, ar, an = self.par
        zx, rx, nx = self.wx[:, t].chunk(3, dim=-1)
        z = torch.sigmoid(az * h + zx)
        r = torch.sigmoid(ar * h + rx)
        n = torch.tanh(an * (h * r) + nx)
        f = h + z * (n - h)
        j = (1 - z) + (n - h) * z * (1 - z) * az + z * (1 - n * n) * an * (r + h * r * (1 - r) * ar)
        return f, j, (z, r, n)

    def diag_guess(self, h0):
        out = self.new_traj()
        for t in range(self.T):
            hp = h0.double() if (t == 0 and h0 is not None) else self._zeros(self.B, self.d)
            out[:, t] = self._eval(hp, t)[0]
        return out

    # ------------------------------------------------------------------ sLSTM diag
    def _slstm(self, prev, t, jac=True):
        """prev (B, 4, d) -> prediction (B, 4, d), J (B, 4, 4, d) [out, in], activations."""
        c, n, m, h = prev[:, 0], prev[:, 1], prev[:, 2], prev[:, 3]
        R = self.par
        wi, wf, wz, wo = self.wx[:, t].chunk(4, dim=-1)
        zi, zf, zz, zo = wi + R[0] * h, wf + R[1] * h, wz + R[2] * h, wo + R[3] * h
        left = zf + m
        mn = torch.maximum(left, zi)
        alpha = (left > zi).double() + 0.5 * (left == zi).double()
        beta = 1 - alpha
        i, f = torch.exp(zi - mn), torch.exp(left - mn)
        z, o = torch.tanh(zz), torch.sigmoid(zo)
        nn, cn = f * n + i, f * c + i * z
        D = nn + self.eps
        hn = o * cn / D
        pred = torch.stack([cn, nn, mn, hn], dim=1)
        acts = dict(i=i, f=f, z=z, o=o, c=c, n=n, D=D, cn=cn, alpha=alpha, beta=beta, h=h)
        if not jac:
            return pred, None, acts
        dm = alpha * R[1] + beta * R[0]
        i_m, f_m = -i * alpha, f * beta
        i_h, f_h = i * (R[0] - dm), f * (R[1] - dm)
        z_h, o_h = (1 - z * z) * R[2], o * (1 - o) * R[3]
        J = self._zeros(self.B, 4, 4, self.d)
        J[:, 0, 0], J[:, 0, 2], J[:, 0, 3] = f, f_m * c + i_m * z, f_h * c + i_h * z + i * z_h
        J[:, 1, 1], J[:, 1, 2], J[:, 1, 3] = f, f_m * n + i_m, f_h * n + i_h
        J[:, 2, 2], J[:, 2, 3] = alpha, dm
        ia, ib = o / D, -o * cn / (D * D)
        J[:, 3] = ia[:, None] * J[:, 0] + ib[:, None] * J[:, 1]
        J[:, 3, 3] = J[:, 3, 3] + cn / D * o_h
        return pred, J, acts

    def picard_pass(self, h_prev, h_halo, carry, mode, h_out, state_out):
        R = self.par
        a = self._zeros(self.B, self.d)
        b = torch.full((self.B, self.d), -float("inf"), dtype=torch.float64)
        N, C = self._zeros(self.B, self.d), self._zeros(self.B, self.d)
        st = self._zeros(self.B, 3, self.d) if carry is None else carry.double().clone()
        c, n, m = st[:, 0], st[:, 1], st[:, 2]
        for t in range(self.T):
            if h_prev is None:
                hp = self._zeros(self.B, self.d)
            elif t == 0:
                hp = self._zeros(self.B, self.d) if h_halo is None else h_halo.double()
            else:
                hp = h_prev[:, t - 1].double()
            wi, wf, wz, wo = self.wx[:, t].chunk(4, dim=-1)
            zi, zf, zz, zo = wi + R[0] * hp, wf + R[1] * hp, torch.tanh(wz + R[2] * hp), wo + R[3] * hp
            if mode == 2:
                b1a = b + zf
                bn = torch.maximum(b1a, zi)
                s1 = torch.where(torch.isinf(b1a), torch.zeros_like(b1a), torch.exp(b1a - bn))
                s2 = torch.exp(zi - bn)
                a, b, N, C = a + zf, bn, N * s1 + s2, C * s1 + s2 * zz
                continue
            mn = torch.maximum(zf + m, zi)
            f, i = torch.exp(zf + m - mn), torch.exp(zi - mn)
            n, c, m = f * n + i, f * c + i * zz, mn
            h = torch.sigmoid(zo) * c / (n + self.eps)
            if state_out is not None:
                state_out[:, t] = torch.stack([c, n, m, h], dim=1)
            else:
                h_out[:, t] = h
        if mode == 2:
            return torch.stack([a, b, N, C], dim=1)[None]
        return torch.stack([c, n, m], dim=1)

    # ------------------------------------------------------------------ passes of both cells
    def _lin(self, prev, t):
        """(prediction, J as (B, n, n, d)) with n = slots."""
        if self.slots == 1:
            f, j, _ = self._eval(prev[:, 0], t)
            return f[:, None], j[:, None, None]
        pred, J, _ = self._slstm(prev, t)
        return pred, J

    def _state(self, traj, t):
        return traj[:, t].double().reshape(self.B, self.slots, self.d)

    def newton_pass(self, traj, halo, carry, mode, out, hist_slot):
        n = self.slots
        eye = torch.eye(n, dtype=torch.float64)[None, :, :, None].expand(self.B, n, n, self.d)
        M, v = eye.clone(), self._zeros(self.B, n, self.d)
        delta = self._zeros(self.B, n, self.d) if carry is None else carry.double().reshape(self.B, n, self.d)
        halo_s = self._zeros(self.B, n, self.d) if halo is None else halo.double().reshape(self.B, n, self.d)
        prev_new = None
        for t in range(self.T):
            prev = self._state(traj, t - 1) if t > 0 else halo_s
            pred, J = self._lin(prev, t)
            F = pred - self._state(traj, t)
            if mode == 2:
                M = torch.einsum("bokd,bkid->boid", J, M)
                v = torch.einsum("boid,bid->bod", J, v) + F
                continue
            self._bump(hist_slot, F.abs().max())
            if mode == 1:
                pn = (prev + self.omega * delta) if t == 0 else prev_new
            delta = torch.einsum("boid,bid->bod", J, delta) + F
            new = self._state(traj, t) + self.omega * delta
            out[:, t] = new.reshape(out[:, t].shape)
            if mode == 1:
                stored = out[:, t].double().reshape(self.B, n, self.d)
                self._bump(16, (self._lin(pn, t)[0] - stored).abs().max())
                prev_new = stored
        if mode == 2:
            return torch.cat([M.reshape(self.B, n * n, self.d), v], dim=1)[None]
        return delta.clone()

    def bwd_pass(self, states, grad_states, halo, carry, mode):
        n = self.slots
        eye = torch.eye(n, dtype=torch.float64)[None, :, :, None].expand(self.B, n, n, self.d)
        M, v = eye.clone(), self._zeros(self.B, n, self.d)
        nu = self._zeros(self.B, n, self.d) if carry is None else carry.double().reshape(self.B, n, self.d)
        halo_s = self._zeros(self.B, n, self.d) if halo is None else halo.double().reshape(self.B, n, self.d)
        g_wx = torch.empty_like(self.wx)
        gp = self._zeros(3 if n == 1 else 4, self.d)
        for t in range(self.T - 1, -1, -1):
            prev = self._state(states, t - 1) if t > 0 else halo_s
            _, J = self._lin(prev, t)
            g = grad_states[:, t].double().reshape(self.B, n, self.d)
            Jt = J.transpose(1, 2)
            if mode == 2:
                # nu -> J^T (nu + g)
                v = torch.einsum("boid,bid->bod", Jt, v + g)
                M = torch.einsum("bokd,bkid->boid", Jt, M)
                continue
            mu = nu + g
            if n == 1:
                az, ar, an = self.par
                hp = prev[:, 0]
                _, _, (z, r, nn_) = self._eval(hp, t)
                m1 = mu[:, 0]
                d_n = m1 * z * (1 - nn_ * nn_)
                d_z = m1 * (nn_ - hp) * z * (1 - z)
                d_r = d_n * an * hp * r * (1 - r)
                g_wx[:, t] = torch.cat([d_z, d_r, d_n], dim=-1)
                gp[0] += (d_z * hp).sum(0)
                gp[1] += (d_r * hp).sum(0)
                gp[2] += (d_n * hp * r).sum(0)
            else:
                _, _, A = self._slstm(prev, t, jac=False)
                mc, mn_, mm, mh = mu[:, 0], mu[:, 1], mu[:, 2], mu[:, 3]
                d_o = mh * A["cn"] / A["D"]
                d_c = mc + mh * A["o"] / A["D"]
                d_n = mn_ - mh * A["o"] * A["cn"] / (A["D"] * A["D"])
                d_f = d_c * A["c"] + d_n * A["n"]
                d_i = d_c * A["z"] + d_n
                d_z = d_c * A["i"]
                d_zo = d_o * A["o"] * (1 - A["o"])
                d_zz = d_z * (1 - A["z"] * A["z"])
                d_m = mm - d_i * A["i"] - d_f * A["f"]
                d_zi = d_i * A["i"] + d_m * A["beta"]
                d_zf = d_f * A["f"] + d_m * A["alpha"]
                g_wx[:, t] = torch.cat([d_zi, d_zf, d_zz, d_zo], dim=-1)
                for q, dz in enumerate((d_zi, d_zf, d_zz, d_zo)):
                    gp[q] += (dz * A["h"]).sum(0)
            nu = torch.einsum("boid,bid->bod", Jt, mu)
        if mode == 2:
            return torch.cat([M.reshape(self.B, n * n, self.d), v], dim=1)[None]
        return g_wx, gp, nu.clone()
