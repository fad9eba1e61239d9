"""Sequence-sharded SBLocal forward: one long sequence split along N over the
ranks of a torch.distributed group (one process per GPU, NCCL over NVLink).

The reference has no sequence parallelism; the decomposition is exact because
the only couplings between tokens are (i) the band, served by a halo of
w//2 keys before and w-1-w//2 keys after the shard, and (ii) three global
reductions: the key log-scale beta (max), phi(K)^T V and sum phi(K) (sums),
cf. src/models/attention/sblocal_attention.py:87-97 and
src/models/attention/feature_maps_sb.py:78.

Protocol per forward (rank g owns rows [lo, hi) of q, k, v, out):
  1. sbl_key_logscale over the own rows (queued first: the device runs it while the host posts step 2);
  2. halo exchange: every rank sends the K/V rows other ranks' windows reach into (point-to-point, into the
     receivers' own memory), with the all-reduce MAX of the (B,H) log-scales travelling beside it;
  3. sbl_key_summary over own rows (+phi(K) of the halo rows kept in the
     workspace)                                -> all-reduce SUM of (B,H,m,D+1) floats;
  4. sbl_band_forward over the local queries, reading local memory only.
No kernel ever touches another GPU's memory.
"""
import torch
import torch.distributed as dist


def shard_bounds(n_total, world):
    """Contiguous, near-equal shards: rank g owns [b[g], b[g+1])."""
    return [n_total * g // world for g in range(world + 1)]


def halo_range(lo, hi, w, n_total):
    """Global key rows [klo, khi) the queries [lo, hi) can see."""
    return max(0, lo - w // 2), min(n_total, hi - 1 - w // 2 + w)


def plan_halo(bounds, w, rank):
    """Returns (sends, recvs): lists of (peer, global_lo, global_hi) row ranges
    this rank must send to / receive from each peer."""
    world = len(bounds) - 1
    n_total = bounds[-1]
    lo, hi = bounds[rank], bounds[rank + 1]
    klo, khi = halo_range(lo, hi, w, n_total)
    recvs, sends = [], []
    for peer in range(world):
        if peer == rank:
            continue
        plo, phi = bounds[peer], bounds[peer + 1]
        a, b = max(klo, plo), min(khi, phi)          # rows of the peer inside my halo
        if a < b and hi > lo:
            recvs.append((peer, a, b))
        pklo, pkhi = halo_range(plo, phi, w, n_total)
        a, b = max(pklo, lo), min(pkhi, hi)          # my rows inside the peer's halo
        if a < b and phi > plo:
            sends.append((peer, a, b))
    return sends, recvs


class HaloBuffers:
    """K/V storage of one rank that already has room for the halo rows on both sides.

    A caller that writes its shard of K and V straight into `k_local` / `v_local` (views of the extended buffers)
    and passes this object to `sblocal_forward_seqshard` saves the copy of the own rows into the extended buffers
    that the forward otherwise makes on every call (two reads and two writes of the whole shard)."""

    def __init__(self, B, n_total, H, E, D, local_context, dtype, device, group=None):
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        self.bounds = shard_bounds(n_total, world)
        self.lo, self.hi = self.bounds[rank], self.bounds[rank + 1]
        self.klo, self.khi = halo_range(self.lo, self.hi, int(local_context), n_total)
        self.k_ext = torch.empty(B, self.khi - self.klo, H, E, dtype=dtype, device=device)
        self.v_ext = torch.empty(B, self.khi - self.klo, H, D, dtype=dtype, device=device)
        self.k_local = self.k_ext[:, self.lo - self.klo:self.hi - self.klo]
        self.v_local = self.v_ext[:, self.lo - self.klo:self.hi - self.klo]

    def holds(self, k_local, v_local):
        return (k_local.data_ptr() == self.k_local.data_ptr() and v_local.data_ptr() == self.v_local.data_ptr()
                and k_local.shape == self.k_local.shape and v_local.shape == self.v_local.shape
                and k_local.stride() == self.k_local.stride() and v_local.stride() == self.v_local.stride())


class HaloExchange:
    """Window-halo exchange in two steps, so that work which needs only the own rows can be queued in between.

    prepare(): the extended K/V buffers with the own rows in place (the caller's `HaloBuffers`, or fresh ones the
    own rows are copied into); start(): posts the point-to-point transfers (the landing buffers are this rank's own
    memory); finish(): waits for them and places the received rows."""

    def __init__(self, k_local, v_local, bounds, w, group=None, buffers=None):
        self.buffers = buffers
        self.rank = dist.get_rank(group)
        self.group = group
        self.lo, self.hi = bounds[self.rank], bounds[self.rank + 1]
        n_total = bounds[-1]
        self.klo, self.khi = halo_range(self.lo, self.hi, w, n_total)
        self.sends, self.recvs = plan_halo(bounds, w, self.rank)
        self.k_local, self.v_local = k_local, v_local
        self.k_ext = self.v_ext = None
        self._reqs, self._landing, self._keep = [], [], []

    def prepare(self):
        k_local, v_local, lo, hi, klo, khi = self.k_local, self.v_local, self.lo, self.hi, self.klo, self.khi
        B, _, H, E = k_local.shape
        D = v_local.shape[-1]
        if self.buffers is not None:
            # the own rows already sit in the middle of the caller's extended buffers
            self.k_ext, self.v_ext = self.buffers.k_ext, self.buffers.v_ext
        else:
            self.k_ext = k_local.new_empty(B, khi - klo, H, E)
            self.v_ext = v_local.new_empty(B, khi - klo, H, D)
            self.k_ext[:, lo - klo:hi - klo] = k_local
            self.v_ext[:, lo - klo:hi - klo] = v_local
        return self

    def start(self):
        if self.k_ext is None:
            self.prepare()
        k_local, v_local, lo, klo = self.k_local, self.v_local, self.lo, self.klo
        B, _, H, E = k_local.shape
        D = v_local.shape[-1]
        ops_ = []
        for peer, a, b in self.sends:
            ks = k_local[:, a - lo:b - lo].contiguous()
            vs = v_local[:, a - lo:b - lo].contiguous()
            self._keep += [ks, vs]
            ops_ += [dist.P2POp(dist.isend, ks, _global_rank(peer, self.group), self.group),
                     dist.P2POp(dist.isend, vs, _global_rank(peer, self.group), self.group)]
        for peer, a, b in self.recvs:
            # the rows land in place where the slice of the extended buffer is contiguous (B = 1), else in a
            # buffer of their own that finish() copies from
            kr, vr = self.k_ext[:, a - klo:b - klo], self.v_ext[:, a - klo:b - klo]
            if not (kr.is_contiguous() and vr.is_contiguous()):
                kr = k_local.new_empty(B, b - a, H, E)
                vr = v_local.new_empty(B, b - a, H, D)
                self._landing.append((a, b, kr, vr))
            ops_ += [dist.P2POp(dist.irecv, kr, _global_rank(peer, self.group), self.group),
                     dist.P2POp(dist.irecv, vr, _global_rank(peer, self.group), self.group)]
        if ops_:
            self._reqs = dist.batch_isend_irecv(ops_)
        return self

    def finish(self):
        for req in self._reqs:
            req.wait()
        for a, b, kr, vr in self._landing:
            self.k_ext[:, a - self.klo:b - self.klo] = kr
            self.v_ext[:, a - self.klo:b - self.klo] = vr
        self._reqs, self._keep = [], []
        return self.k_ext, self.v_ext, self.klo


def exchange_halo(k_local, v_local, bounds, w, group=None):
    """Returns (k_ext, v_ext, klo): the local K/V rows extended by the halo
    rows received from the neighbours, and the global position of row 0."""
    return HaloExchange(k_local, v_local, bounds, w, group).start().finish()


def _global_rank(group_rank, group):
    return group_rank if group is None else dist.get_global_rank(group, group_rank)


class CudaEngine:
    """The three stage calls of the C ABI on this rank's shard."""

    def __init__(self, q_local, k_ext, v_ext, W, w, tau, eps, key_lengths, lo, klo, n_total, n_own):
        from . import ops
        self.prob = ops.Problem(q_local, k_ext, v_ext, W, w, tau, eps, key_lengths,
                                q_pos0=lo, k_pos0=klo, S_total=n_total,
                                sum_range=(lo - klo, lo - klo + n_own))
        self.ws = self.prob.workspace()

    def key_logscale(self):
        return self.prob.key_logscale(workspace=self.ws)

    def key_summary(self, beta, out=None):
        return self.prob.key_summary(beta, workspace=self.ws, out=out)

    def band_forward(self, beta, kv, ksum):
        return self.prob.band_forward(beta, kv, ksum, workspace=self.ws)


def sblocal_forward_seqshard(q_local, k_local, v_local, W, local_context, n_total, softmax_temp=None,
                             softmax_eps=0.0, key_lengths=None, group=None, engine_cls=CudaEngine, timings=None,
                             halo_buffers=None):
    """SBLocal forward of this rank's shard of one long sequence.

    q_local/k_local/v_local: (B, n_local, H, E|D), rows
    shard_bounds(n_total, world)[rank] ... [rank+1] of the full sequence.
    key_lengths: global (B,) key lengths or None.  Returns out (B, n_local, H, D).
    timings: an empty list to be filled with (stage name, CUDA event) pairs recorded on the current stream
    after each stage (CUDA ranks only).
    halo_buffers: a `HaloBuffers` whose k_local / v_local views ARE k_local / v_local: the own rows are then used
    where they are instead of being copied next to the halo rows.
    """
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    bounds = shard_bounds(n_total, world)
    lo, hi = bounds[rank], bounds[rank + 1]
    if q_local.shape[1] != hi - lo or k_local.shape[1] != hi - lo or v_local.shape[1] != hi - lo:
        raise ValueError(f'rank {rank} must hold rows [{lo},{hi}) of the sequence: got {q_local.shape[1]} rows')
    # The key log-scale reads the own rows only: the halo rows fly while it runs, and its MAX all-reduce travels
    # with them.  The summary and the band stage need the halo rows / the reduced summary.
    mark = (lambda name: None) if timings is None else (lambda name: timings.append((name, _event())))
    mark('start')
    if halo_buffers is not None and not (halo_buffers.bounds == bounds and halo_buffers.holds(k_local, v_local)):
        raise ValueError('halo_buffers must be the HaloBuffers object whose k_local / v_local views are passed in')
    # The log-scale pass is queued first: the device works on it while the host sets up the transfers.
    halo = HaloExchange(k_local, v_local, bounds, int(local_context), group, halo_buffers).prepare()
    eng = engine_cls(q_local, halo.k_ext, halo.v_ext, W, int(local_context), softmax_temp, softmax_eps, key_lengths,
                     lo, halo.klo, n_total, hi - lo)
    beta = eng.key_logscale()
    mark('logscale')
    halo.start()
    beta_work = dist.all_reduce(beta, op=dist.ReduceOp.MAX, group=group, async_op=True)
    halo.finish()
    beta_work.wait()
    mark('halo+max')
    # kv and ksum are two views of one buffer: one collective for both, no packing copies
    B, H, D, m = q_local.shape[0], q_local.shape[2], v_local.shape[-1], 2 * W.shape[0]
    packed = torch.empty(B * H * m * (D + 1), device=q_local.device, dtype=torch.float32)
    views = (packed[:B * H * m * D].view(B, H, m, D), packed[B * H * m * D:].view(B, H, m))
    kv, ksum = eng.key_summary(beta, out=views)
    mark('summary')
    dist.all_reduce(packed, op=dist.ReduceOp.SUM, group=group)
    mark('allreduce')
    out = eng.band_forward(beta, kv, ksum)
    mark('band')
    return out


def _event():
    ev = torch.cuda.Event(enable_timing=True)
    ev.record()
    return ev
