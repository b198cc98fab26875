"""CPU stand-in for the per-rank scan kernels (ParaGRU mix='diag' only), used to test the
time-sharded driver's collective choreography with gloo ranks and no GPU.  Test code: the
product path never imports it."""

import torch

from pararnn_b200.seq_shard import NS, NV


class CpuShardOps:
    def __init__(self, kind, wx, rec, eps, omega):
        assert kind == "gru_diag"
        self.kind, self.wx, self.omega = kind, wx.float(), float(omega)
        self.B, self.T = wx.shape[:2]
        self.d = wx.shape[2] // 3
        self.dev = wx.device
        self.slots, self.monoid = 1, "affine1"
        self.par = [p.float() for p in rec]
        self.bits = torch.zeros(20, dtype=torch.int32)

    def new_traj(self):
        return torch.empty(self.B, self.T, self.d)

    def new_out(self):
        return torch.empty(self.B, self.T, self.d)

    def stats_bits(self):
        return self.bits

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
            hp = h0 if (t == 0 and h0 is not None) else torch.zeros(self.B, self.d)
            out[:, t] = self._eval(hp, t)[0]
        return out

    def fold(self, monoid, gathered, rank, world, reverse):
        first, step = (world - 1, -1) if reverse else (0, 1)
        vec = gathered[first][:, :1].clone()
        q = first + step
        while q != rank:
            vec = gathered[q][:, 0:1] * vec + gathered[q][:, 1:2]
            q += step
        return vec

    def _bump(self, slot, value):
        as_bits = torch.tensor(float(value)).view(torch.int32)
        self.bits[slot] = torch.maximum(self.bits[slot], as_bits)

    def newton_pass(self, traj, halo, carry, mode, out, hist_slot):
        a = torch.ones(self.B, self.d)
        b = torch.zeros(self.B, self.d)
        delta = torch.zeros(self.B, self.d) if carry is None else carry[:, 0]
        prev_new = None
        for t in range(self.T):
            hp = traj[:, t - 1] if t > 0 else (halo if halo is not None else torch.zeros(self.B, self.d))
            f, j, _ = self._eval(hp, t)
            F = f - traj[:, t]
            if mode == 2:
                a, b = j * a, j * b + F
                continue
            self._bump(hist_slot, F.abs().max())
            if mode == 1:
                pn = (hp + self.omega * delta) if t == 0 else prev_new
            delta = j * delta + F
            out[:, t] = traj[:, t] + self.omega * delta
            if mode == 1:
                self._bump(16, (self._eval(pn, t)[0] - out[:, t]).abs().max())
                prev_new = out[:, t].clone()
        if mode == 2:
            return torch.stack([a, b], dim=1)
        return delta[:, None].clone()

    def bwd_pass(self, states, grad_states, halo, carry, mode):
        az, ar, an = self.par
        nu = torch.zeros(self.B, self.d) if carry is None else carry[:, 0]
        a = torch.ones(self.B, self.d)
        b = torch.zeros(self.B, self.d)
        g_wx = torch.empty_like(self.wx)
        gp = torch.zeros(3, self.d)
        for t in range(self.T - 1, -1, -1):
            hp = states[:, t - 1] if t > 0 else (halo if halo is not None else torch.zeros(self.B, self.d))
            _, j, (z, r, n) = self._eval(hp, t)
            g = grad_states[:, t]
            if mode == 2:
                a, b = j * a, j * (b + g)
                continue
            mu = nu + g
            d_n = mu * z * (1 - n * n)
            d_z = mu * (n - hp) * z * (1 - z)
            d_r = d_n * an * hp * r * (1 - r)
            g_wx[:, t] = torch.cat([d_z, d_r, d_n], dim=-1)
            gp[0] += (d_z * hp).sum(0)
            gp[1] += (d_r * hp).sum(0)
            gp[2] += (d_n * hp * r).sum(0)
            nu = j * mu
        if mode == 2:
            return torch.stack([a, b], dim=1)
        return g_wx, gp, nu[:, None].clone()
