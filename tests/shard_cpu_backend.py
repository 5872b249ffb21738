"""CPU stand-in for the shard stage calls (test infrastructure).

Implements, with torch ops in float64, exactly the contract of the
``fastmax_b200_shard_*`` entry points that ``fastmax_b200.sharded`` drives, with one
chunk per shard: raw moment totals ``sum phi(y) (x) [z | e]`` with
``phi(x) = [x(x)x | x | 1]``, read-outs against the sum of other shards' totals,
and the shard's own block in score form.  It lets the exchange logic (which
totals go where, scan direction, ownership of the max-norm row) run on gloo
ranks without a GPU.
"""
import torch


def _phi(x):
    d = x.shape[-1]
    quad = (x.unsqueeze(-1) * x.unsqueeze(-2)).flatten(-2)
    return torch.cat([quad, x, torch.ones_like(x[..., :1])], -1)      # (h, n, d*d+d+1)


class TorchShardBackend:
    def __init__(self, normalize, a0, a1, a2, lim, p, mask=True):
        # mask False: s_base / (kv_states, r_base) hold the totals of ALL shards and nothing is local
        self.mask = mask
        self.normalize, self.a0, self.a1, self.lim, self.p = normalize, a0, a1, lim, p
        self.a2 = a2 if p == 2 else 0.0

    # ---- statistics: (bits of max ||x||^2 as float32) << 32 | (0xFFFFFFFF - global row)
    def rowmax(self, q, k, row_offset):
        words = []
        for x in (q, k):
            n2 = (x.float() ** 2).sum(-1)
            val, idx = n2.max(dim=1)
            bits = val.float().view(torch.int32).to(torch.int64) & 0xFFFFFFFF
            words.append((bits << 32) | (0xFFFFFFFF - (idx + row_offset)))
        return torch.cat(words)

    def _scales(self, stats, h):
        if stats is None:
            return torch.ones(h, dtype=torch.float64), torch.ones(h, dtype=torch.float64), None, None
        n2 = (stats >> 32).to(torch.int32).view(torch.float32).double()
        rows = 0xFFFFFFFF - (stats & 0xFFFFFFFF)
        return self.lim / n2[:h].sqrt(), self.lim / n2[h:].sqrt(), n2, rows

    def _coef(self, stats, h):
        cq, ck, _, _ = self._scales(stats, h)
        c = (cq * ck)[:, None, None]
        return self.a0, self.a1 * c, self.a2 * c * c

    def kv_state(self, k, v):
        vt = torch.cat([v, torch.ones_like(v[..., :1])], -1)
        total = torch.einsum("hnf,hnc->hfc", _phi(k.double()), vt.double())
        return torch.zeros_like(total), total

    def forward(self, q, k, v, stats, kv_states, s_base):
        h, n, d = q.shape
        if s_base is not None:
            if kv_states is None:
                kv_states = s_base.clone()
            else:
                kv_states.copy_(s_base)
        A0, A1, A2 = self._coef(stats, h)
        qd, kd = q.double(), k.double()
        vt = torch.cat([v, torch.ones_like(v[..., :1])], -1).double()
        s = qd @ kd.transpose(1, 2)
        tri = torch.tril(torch.ones(n, n, dtype=torch.float64)) if self.mask else torch.zeros(n, n, dtype=torch.float64)
        f = (A0 + A1 * s + A2 * s * s) * tri
        w = torch.cat([A2.expand(h, 1, 1).repeat(1, 1, d * d), A1.expand(h, 1, 1).repeat(1, 1, d),
                       torch.full((h, 1, 1), A0, dtype=torch.float64)], -1)
        num = f @ vt + torch.einsum("hnf,hfc->hnc", _phi(qd) * w, kv_states)
        den = num[..., d]
        return (num[..., :d] / den[..., None]).to(q.dtype), den.float()

    def qg_state(self, q, out, den, go):
        delta = (go.double() * out.double()).sum(-1)
        ut = torch.cat([go.double() / den.double()[..., None], (-delta / den.double())[..., None]], -1)
        total = torch.einsum("hnf,hnc->hfc", _phi(q.double()), ut)
        return delta.float(), torch.zeros_like(total), total

    @staticmethod
    def _split(state, d):
        return state[:, :d * d].reshape(-1, d, d, d + 1), state[:, d * d:d * d + d], state[:, d * d + d]

    def backward(self, q, k, v, out, den, stats, go, delta, kv_states, qg_states, r_base):
        h, n, d = q.shape
        if r_base is not None:
            if qg_states is None:
                qg_states = r_base.clone()
            else:
                qg_states.copy_(r_base)
        A0, A1, A2 = self._coef(stats, h)
        qd, kd = q.double(), k.double()
        vt = torch.cat([v, torch.ones_like(v[..., :1])], -1).double()
        ut = torch.cat([go.double() / den.double()[..., None], (-delta.double() / den.double())[..., None]], -1)
        tri = torch.tril(torch.ones(n, n, dtype=torch.float64)) if self.mask else torch.zeros(n, n, dtype=torch.float64)
        s = qd @ kd.transpose(1, 2)
        e = (A1 + 2 * A2 * s) * (ut @ vt.transpose(1, 2)) * tri
        pf = (A0 + A1 * s + A2 * s * s) * tri
        S2, S1, _ = self._split(kv_states, d)
        R2, R1, R0 = self._split(qg_states, d)
        gq = e @ kd + A1 * torch.einsum("hac,hic->hia", S1, ut) \
            + 2 * A2 * torch.einsum("habc,hib,hic->hia", S2, qd, ut)
        gk = e.transpose(1, 2) @ qd + A1 * torch.einsum("hac,hjc->hja", R1, vt) \
            + 2 * A2 * torch.einsum("habc,hjb,hjc->hja", R2, kd, vt)
        gv = pf.transpose(1, 2) @ ut[..., :d] + A0 * R0[:, None, :d] \
            + A1 * torch.einsum("hac,hja->hjc", R1, kd)[..., :d] \
            + A2 * torch.einsum("habc,hja,hjb->hjc", R2, kd, kd)[..., :d]
        dots = torch.cat([(gq * qd).sum((1, 2)), (gk * kd).sum((1, 2))]).float()
        return gq.to(q.dtype), gk.to(k.dtype), gv.to(v.dtype), dots

    def norm_fixup(self, q, k, stats, dots, row_offset, gq, gk):
        h = q.shape[0]
        _, _, n2, rows = self._scales(stats, h)
        for x, g, off in ((q, gq, 0), (k, gk, h)):
            for i in range(h):
                r = int(rows[off + i]) - row_offset
                if 0 <= r < x.shape[1]:
                    g[i, r] -= (dots[off + i].double() / n2[off + i]).to(g.dtype) * x[i, r]
