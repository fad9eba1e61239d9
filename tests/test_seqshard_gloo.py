"""Sequence-sharding protocol on CPU ranks (gloo, world sizes 2 and 3): halo
planning and exchange, the MAX/SUM reductions, shard geometry.  The per-rank
stage arithmetic is supplied by the CPU oracle here (the product's stages are
CUDA only and are tested against the same oracle in the GPU tests); what this
file checks is that the distributed protocol reproduces the single-process
result."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_halo_plan_covers_every_window():
    from fly_b200.seqshard import halo_range, plan_halo, shard_bounds
    for n_total, world, w in [(100, 2, 16), (1000, 4, 256), (50, 3, 64), (64, 8, 5), (7, 3, 4)]:
        bounds = shard_bounds(n_total, world)
        assert bounds[0] == 0 and bounds[-1] == n_total
        for rank in range(world):
            lo, hi = bounds[rank], bounds[rank + 1]
            klo, khi = halo_range(lo, hi, w, n_total)
            sends, recvs = plan_halo(bounds, w, rank)
            have = set(range(lo, hi))
            for peer, a, b in recvs:
                assert bounds[peer] <= a < b <= bounds[peer + 1]
                have |= set(range(a, b))
            if hi > lo:
                assert have >= set(range(klo, khi))
            # what I send to a peer is exactly what the peer plans to receive from me
            for peer, a, b in sends:
                assert (rank, a, b) in plan_halo(bounds, w, peer)[1]


class OracleEngine:
    """CPU stand-in for the three stage calls, with the same shard geometry."""

    def __init__(self, q_local, k_ext, v_ext, W, w, tau, eps, key_lengths, lo, klo, n_total, n_own):
        from oracle import sblocal_oracle as so
        self.so = so
        self.q = q_local.permute(0, 2, 1, 3)
        self.k = k_ext.permute(0, 2, 1, 3)
        self.v = v_ext.permute(0, 2, 1, 3)
        self.W, self.w, self.eps = W, w, eps
        self.tau = tau or q_local.shape[-1] ** -0.5
        B = q_local.shape[0]
        self.lengths = key_lengths if key_lengths is not None else torch.full((B,), n_total)
        self.lo, self.klo, self.n_own = lo, klo, n_own

    def key_logscale(self):
        own = self.k[:, :, self.lo - self.klo:self.lo - self.klo + self.n_own]
        return self.so.key_log_features(own, self.W, self.tau).amax(dim=(-1, -2))

    def _phik(self, beta):
        kd = self.so.key_log_features(self.k, self.W, self.tau)
        m = kd.shape[-1]
        phik = torch.exp(kd - beta[..., None, None]) + self.eps / m ** 0.5
        pos = self.klo + torch.arange(self.k.shape[2])
        return phik.masked_fill((pos.view(1, 1, -1, 1) >= self.lengths.view(-1, 1, 1, 1)), 0.0)

    def key_summary(self, beta, out=None):
        a, b = self.lo - self.klo, self.lo - self.klo + self.n_own
        phik = self._phik(beta)[:, :, a:b]
        kv, ksum = torch.einsum('bhsm,bhsd->bhmd', phik, self.v[:, :, a:b]), phik.sum(-2)
        if out is not None:
            out[0].copy_(kv)
            out[1].copy_(ksum)
            return out
        return kv, ksum

    def band_forward(self, beta, kv, ksum):
        so = self.so
        phik = self._phik(beta)
        qp, qls = so.query_features(self.q, self.W, self.tau, self.eps)
        pls = qls + beta[..., None, None]
        T, S, w = self.q.shape[2], self.k.shape[2], self.w
        gi = (self.lo + torch.arange(T)).view(1, 1, T, 1)
        gk = (self.klo + torch.arange(S)).view(1, 1, 1, S)
        win = (gk >= gi - w // 2) & (gk <= gi - w // 2 + w - 1) & (gk < self.lengths.view(-1, 1, 1, 1))
        qk = self.tau * torch.einsum('bhte,bhse->bhts', self.q, self.k)
        dp = torch.einsum('bhtm,bhsm->bhts', qp, phik) * win
        lse = torch.logsumexp(qk.masked_fill(~win, -1e24 * self.tau), -1, keepdim=True)
        Z = torch.einsum('bhtm,bhm->bht', qp, ksum).unsqueeze(-1)
        lrn = torch.log((Z - dp.sum(-1, keepdim=True)).clamp_min(1e-24)) + pls
        n = torch.logaddexp(lse, lrn)
        ps = torch.exp(pls - n)
        dots = torch.exp(qk - n) * win - dp * ps
        out = torch.einsum('bhts,bhsd->bhtd', dots, self.v) + torch.einsum('bhtm,bhmd->bhtd', qp, kv) * ps
        return out.permute(0, 2, 1, 3)


def _free_port():
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]


def _worker(rank, world, port, case, ret):
    sys.path.insert(0, ROOT)
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    dist.init_process_group('gloo', rank=rank, world_size=world)
    try:
        from fly_b200.seqshard import sblocal_forward_seqshard, shard_bounds
        from oracle import sblocal_oracle as so
        B, N, H, E, D, w, r, eps, ragged = case
        torch.manual_seed(1234)
        q, k, v = torch.randn(B, N, H, E) / E ** 0.25, torch.randn(B, N, H, E) / E ** 0.25, torch.randn(B, N, H, D)
        W = so.gaussian_orthogonal_random_matrix(r, E)
        lengths = torch.randint(N // 3, N, (B,)) if ragged else None
        bounds = shard_bounds(N, world)
        lo, hi = bounds[rank], bounds[rank + 1]
        out = sblocal_forward_seqshard(q[:, lo:hi], k[:, lo:hi], v[:, lo:hi], W, w, N, None, eps, lengths,
                                       engine_cls=OracleEngine)
        ref, _ = so.sblocal_forward(q, k, v, W, w, None, eps, lengths)
        ret[rank] = so.rel_err(out, ref[:, lo:hi]) if hi > lo else 0.0
        # the same with the own rows written straight into caller-owned extended buffers (no copy of the shard)
        from fly_b200.seqshard import HaloBuffers
        hb = HaloBuffers(B, N, H, E, D, w, q.dtype, q.device)
        hb.k_local.copy_(k[:, lo:hi])
        hb.v_local.copy_(v[:, lo:hi])
        out2 = sblocal_forward_seqshard(q[:, lo:hi], hb.k_local, hb.v_local, W, w, N, None, eps, lengths,
                                        engine_cls=OracleEngine, halo_buffers=hb)
        if hi > lo:
            ret[rank] = max(ret[rank], so.rel_err(out2, ref[:, lo:hi]))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize('world', [2, 3])
@pytest.mark.parametrize('case', [
    (2, 96, 2, 16, 8, 16, 8, 0.0, False),      # halo from direct neighbours only
    (1, 40, 1, 8, 8, 64, 4, 0.0, False),       # window wider than a shard: halo spans several ranks
    (2, 75, 2, 16, 16, 9, 8, 1e-4, True),      # odd window, eps, ragged key lengths, uneven shards
])
def test_protocol_matches_single_process(world, case):
    port = _free_port()
    ret = mp.get_context('spawn').Manager().dict()
    mp.spawn(_worker, args=(world, port, case, ret), nprocs=world, join=True)
    assert len(ret) == world
    # fp32 bound used throughout (max|diff| / max|ref| <= 1e-4): the sharded sums associate differently from the
    # single-process ones, which alone moves the result by a few 1e-5
    for rank in range(world):
        assert ret[rank] <= 1e-4, f'rank {rank}: rel err {ret[rank]}'
