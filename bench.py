"""Benchmark of the SBLocal attention forward on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

One "step" is one forward of the attention layer over one batch of synthetic
inputs.  Default workload: bf16, B=2, H=16, N=16384, d=64, window 256, m=256
(the configuration the roofline target is quoted on).  With N>1 GPUs (launched
by torch.distributed.run, one rank per GPU) every rank runs that batch on its
own (batch x head) units -- the path has no collective -- so the global batch
is N times larger (weak scaling).  Rank 0 prints ONE JSON line.  The same line
carries, under "extra":
  cfg1      the fp32 N=3136 configuration (second shape of the metric), 1 GPU only;
  cfg3/cfg5 the bf16 B4 H12 N4096 d64 and B1 H8 N131072 d128 w512 m512 configurations, 1 GPU only;
  strong    N>1: the FIXED default batch split into contiguous (batch, head) ranges, 32/N units per rank
            (eager launches, and the same steps replayed from one CUDA graph);
  seqshard  N>1: the long sequence (B1 H8 N131072 d128 w512 m512) sharded along N: halo exchange + two all-reduces.

`--impl reference` times the reference's CPU forward on a bounded sample of the
same workload: the reference module itself where its source tree can be
imported (with the restated window functions), else the oracle port of it.
`--workload t2t_vit_t14_b64` times the whole T2T-ViT-t-14 forward (batch 64)
and its two attention stages alone.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (dtype, B, H, N, d, w, m, seed)
    'sblocal_bf16_B2_H16_N16384_d64_w256_m256': ('bf16', 2, 16, 16384, 64, 256, 256, 2),
    'sblocal_fp32_B8_H1_N3136_d64_w256_m256': ('f32', 8, 1, 3136, 64, 256, 256, 0),
    'sblocal_bf16_B4_H12_N4096_d64_w256_m256': ('bf16', 4, 12, 4096, 64, 256, 256, 1),
    'sblocal_bf16_B1_H8_N131072_d128_w512_m512': ('bf16', 1, 8, 131072, 128, 512, 512, 3),
    # a quarter of the default batch: small enough for a multi-pass ncu capture
    'sblocal_bf16_B2_H4_N16384_d64_w256_m256': ('bf16', 2, 4, 16384, 64, 256, 256, 2),
    # the long sequence at the d = 64 head shape
    'sblocal_bf16_B1_H8_N131072_d64_w256_m256': ('bf16', 1, 8, 131072, 64, 256, 256, 3),
    # one head of the long-sequence configuration: small enough for a multi-pass ncu capture
    'sblocal_bf16_B1_H1_N131072_d128_w512_m512': ('bf16', 1, 1, 131072, 128, 512, 512, 3),
}
DEFAULT_WORKLOAD = 'sblocal_bf16_B2_H16_N16384_d64_w256_m256'
CFG1_WORKLOAD = 'sblocal_fp32_B8_H1_N3136_d64_w256_m256'
SEQSHARD_WORKLOAD = 'sblocal_bf16_B1_H8_N131072_d128_w512_m512'
T2T_WORKLOAD = 't2t_vit_t14_b64'
METRIC = 'sblocal_attn_fwd_tokens_per_s'


def load_peaks():
    path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(path):
        with open(path) as fh:
            pk = json.load(fh)
        return dict(hbm_gbs=pk['hbm_gbs'], bf16_tflops=pk['bf16_tflops'],
                    bf16_tflops_sustained=pk.get('bf16_tflops_sustained'), source='measured')
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source='fallback')


def load_band_traffic(B, H, N, d, w, m):
    """DRAM bytes of one band-kernel launch, from the ncu capture recorded in profiles/band_kernel_dram.json
    (a smaller batch of the same shape), scaled by the (batch x head) count: traffic grows in proportion to it."""
    path = os.path.join(ROOT, 'profiles', 'band_kernel_dram.json')
    if not os.path.exists(path):
        return None
    with open(path) as fh:
        records = json.load(fh)['records']
    for rec in records:
        if (rec['N'], rec['d'], rec['w'], rec['m']) == (N, d, w, m):
            return rec['dram_bytes_per_launch'] * (B * H) / rec['units']
    return None


def flops_per_token_head(d, D, w, m):
    """Algorithmic FLOPs of the whole forward per (token, head): two r x d
    projections, phi(K)^T V, phi(Q) KV, phi(Q).sum phi(K), band QK^T, band
    phi(Q)phi(K)^T, band A V."""
    return 2 * (m * d + 2 * m * D + m + w * d + w * m + w * D)


def band_flops_per_token_head(d, D, w, m):
    """Share of the above done by the band kernel: the query projection,
    phi(Q) KV, phi(Q).ksum and the three banded products."""
    return 2 * (m * d // 2 + m * D + m + w * d + w * m + w * D)


def make_inputs(spec, device, seed_offset=0):
    dtype, B, H, N, d, w, m, seed = spec
    g = torch.Generator(device='cpu').manual_seed(seed + 1000 * seed_offset)
    tdt = torch.bfloat16 if dtype == 'bf16' else torch.float32
    scale = d ** 0.25
    mk = lambda: (torch.randn(B, N, H, d, generator=g) / scale).to(tdt)
    q, k, v = mk(), mk(), mk()
    torch.manual_seed(seed)
    from fly_b200.projection_utils import gaussian_orthogonal_random_matrix
    W = gaussian_orthogonal_random_matrix(m // 2, d)
    return q, k, v, W


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed
    region runs."""
    FIELDS = ('clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,'
              'clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,'
              'clocks_event_reasons.sw_power_cap')

    def __init__(self, index):
        self.index = index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ['nvidia-smi', '-i', str(self.index), f'--query-gpu={self.FIELDS}',
                 '--format=csv,noheader,nounits', '-lms', '50'],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append(line.strip())

    def stop(self):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=['nvidia-smi unavailable'])
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], None, set()
        names = ['hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap']
        for row in self.rows:
            parts = [x.strip() for x in row.split(',')]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                smax = float(parts[1])
            except ValueError:
                continue
            for nm, val in zip(names, parts[3:7]):
                if val.lower().startswith('active'):
                    reasons.add(nm)
        sm.sort()
        return dict(sm_mhz=(sm[len(sm) // 2] if sm else None), sm_max_mhz=smax, reasons=sorted(reasons),
                    samples=len(sm))


def time_cpu_forward(spec, units, warmup, steps):
    """Times the reference's CPU forward on `units` (batch, head) units at full N, fp32, all host threads.
    Returns (seconds per forward, kind, output of the last forward, its inputs)."""
    from oracle import ref_bridge
    from oracle import sblocal_oracle as so
    dtype, B, H, N, d, w, m, seed = spec
    torch.set_num_threads(os.cpu_count() or 1)
    q, k, v, W = make_inputs((dtype, units, 1, N, d, w, m, seed), 'cpu')
    q, k, v = q.float(), k.float(), v.float()
    if ref_bridge.reference_available():
        kind = 'reference'
        run = lambda: ref_bridge.reference_forward(q, k, v, W, w)[0]
    else:
        kind = 'port'
        run = lambda: so.sblocal_forward(q, k, v, W, w, row_chunk=1024)[0]
    times, out = [], None
    with torch.no_grad():
        for i in range(warmup + steps):
            t0 = time.perf_counter()
            out = run()
            if i >= warmup:
                times.append(time.perf_counter() - t0)
    return sum(times) / len(times), kind, out, (q, k, v, W)


def cpu_sample_text(units, spec, kind):
    dtype, B, H, N = spec[:4]
    what = ('the reference module (window functions restated on CPU)' if kind == 'reference'
            else 'the oracle port of the reference forward (the reference tree is not on this machine)')
    return f'{units} of {B * H} (batch,head) units at full N={N}, fp32, {what}, scaled to whole-batch tokens/s'


def run_reference(args, spec, rank):
    """CPU arm, rank 0 only: a bounded sample of the workload on the host cores."""
    if rank != 0:
        return
    dtype, B, H, N, d, w, m, seed = spec
    cores = os.cpu_count() or 1
    units = max(1, min(B * H, args.cpu_units))
    t, kind, _, _ = time_cpu_forward(spec, units, args.warmup_cpu, args.steps_cpu)
    value = units * N / t / H          # tokens/s of the full workload = token-heads/s divided by H
    line = dict(metric=METRIC, value=value, unit='tokens/s', impl='reference', n_gpus=args.gpus,
                steps=args.steps_cpu, warmup=args.warmup_cpu, ms_per_step=t * 1e3, higher_is_better=True,
                scaling='weak', vs_baseline=None, dtype='f32', data='synthetic',
                config=dict(workload=args.workload, B_per_gpu=B, global_batch=B, H=H, N=N, d=d, window=w,
                            features=m),
                cpu_baseline=dict(value=value, unit='tokens/s', cores=cores, kind=kind,
                                  sample=cpu_sample_text(units, spec, kind)),
                e2e=dict(value=value, unit='tokens/s', h2d_bytes_per_step=0, d2h_bytes_per_step=0))
    emit(json.dumps(line))


def timed_blocks(run_step, steps, reps, barrier, flush=None):
    """`reps` timed blocks of `steps` steps each, every block bracketed by barrier + synchronize; CUDA events
    on the current stream.  Returns the per-block milliseconds."""
    out = []
    for _ in range(reps):
        barrier()
        if flush is None:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                run_step()
            e1.record()
            barrier()
            out.append(e0.elapsed_time(e1))
        else:
            pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                     for _ in range(steps)]
            for a_, b_ in pairs:
                flush.zero_()
                a_.record()
                run_step()
                b_.record()
            barrier()
            out.append(sum(a_.elapsed_time(b_) for a_, b_ in pairs))
    return out


def max_over_ranks(values, dev, world):
    import torch.distributed as dist
    t = torch.tensor(values, device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(x) for x in t.tolist()]


def min_over_ranks(value, dev, world):
    return -max_over_ranks([-value], dev, world)[0]


def extra_cfg1(dev, steps):
    """The fp32 N = 3136 shape of the metric (generic fp32-math kernels), L2 flushed between steps."""
    from fly_b200 import ops
    spec = WORKLOADS[CFG1_WORKLOAD]
    dtype, B, H, N, d, w, m, seed = spec
    q, k, v, W = (t.to(dev) for t in make_inputs(spec, 'cpu'))
    prob = ops.Problem(q, k, v, W, w)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for _ in range(3):
        prob.forward()
    ms = timed_blocks(prob.forward, steps, 3, lambda: torch.cuda.synchronize(dev), flush)
    ms_step = statistics.median(ms) / steps
    flops = flops_per_token_head(d, d, w, m) * B * H * N
    return dict(workload=CFG1_WORKLOAD, dtype='f32', ms_per_step=ms_step, tokens_per_s=B * N / (ms_step * 1e-3),
                tflops=flops / (ms_step * 1e-3) / 1e12, kernels='generic SIMT fp32 math',
                l2='256 MB buffer rewritten between timed steps')


def extra_tensor_config(dev, name, steps, peak_tf):
    """Another bf16 configuration of the metric through the tensor-core kernels (inputs larger than L2, or the
    256 MB flush between steps): time per forward and its fraction of the tensor roofline."""
    from fly_b200 import ops
    spec = WORKLOADS[name]
    dtype, B, H, N, d, w, m, seed = spec
    q, k, v, W = (t.to(dev) for t in make_inputs(spec, 'cpu'))
    prob = ops.Problem(q, k, v, W, w)
    step_bytes = 4 * B * H * N * d * 2
    flush = None if step_bytes > 192e6 else torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for _ in range(3):
        prob.forward()
    ms = timed_blocks(prob.forward, steps, 3, lambda: torch.cuda.synchronize(dev), flush)
    prob.check_status()
    ms_step = statistics.median(ms) / steps
    tf = flops_per_token_head(d, d, w, m) * B * H * N / (ms_step * 1e-3) / 1e12
    return dict(workload=name, dtype='bf16', ms_per_step=ms_step, tokens_per_s=B * N / (ms_step * 1e-3), tflops=tf,
                roofline_frac=tf / peak_tf,
                kernels='tcgen05+TMA bf16' if prob.status_offset is not None else 'generic SIMT fp32 math',
                l2='inputs exceed L2' if flush is None else '256 MB buffer rewritten between timed steps')


def extra_strong(dev, rank, world, spec, steps, barrier):
    """Strong scaling of the default batch: its B*H (batch, head) units are split into `world` contiguous
    ranges, one per rank, no collective; tokens/s = B*N / (slowest rank's time per forward)."""
    from fly_b200 import ops
    dtype, B, H, N, d, w, m, seed = spec
    units = B * H
    if units % world != 0:
        return dict(skipped=f'{units} units do not split evenly over {world} ranks')
    per = units // world
    u0 = rank * per
    b0, h0 = divmod(u0, H)
    q, k, v, W = make_inputs(spec, 'cpu')
    if per >= H:                      # whole batches per rank
        nb = per // H
        sl = lambda t: t[b0:b0 + nb]
    else:                             # a range of heads of one batch entry (strided views, passed as strides)
        sl = lambda t: t[b0:b0 + 1, :, h0:h0 + per]
    qd, kd, vd = q.to(dev), k.to(dev), v.to(dev)
    prob = ops.Problem(sl(qd), sl(kd), sl(vd), W.to(dev), w)
    for _ in range(5):
        prob.forward()
    ms = timed_blocks(prob.forward, steps, 5, barrier)
    ms = max_over_ranks(ms, dev, world)
    prob.check_status()
    ms_step = statistics.median(ms) / steps
    # The same `steps` forwards replayed from one CUDA graph: at 8 ranks a forward is ~60 us of kernels behind
    # five launches, so the host's launch cost shows; the graph takes it out of the timed region.
    g, why = None, ''
    try:
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            prob.forward()                      # the scratch buffer of this stream exists before the capture
        torch.cuda.synchronize(dev)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            for _ in range(steps):
                prob.forward()
        g.replay()
        torch.cuda.synchronize(dev)
    except Exception as e:                      # the eager figure above stands on its own
        g, why = None, f'{type(e).__name__}: {e}'[:200]
    # every rank times the replay or none does (the timing ends in a collective)
    if min_over_ranks(1.0 if g is not None else 0.0, dev, world) > 0.5:
        gms = max_over_ranks(timed_blocks(g.replay, 1, 5, barrier), dev, world)
        prob.check_status()
        gstep = statistics.median(gms) / steps
        graph = dict(ms_per_step=gstep, tokens_per_s=B * N / (gstep * 1e-3))
    else:
        graph = dict(unavailable=why or 'capture failed on another rank')
    return dict(workload=DEFAULT_WORKLOAD, units_per_rank=per, ms_per_step=ms_step,
                tokens_per_s=B * N / (ms_step * 1e-3), scaling='strong', cuda_graph_replay=graph,
                note='fixed global batch; inputs of a rank (%.0f MB) %s the 126 MB L2'
                     % (4 * per * N * d * 2 / 1e6, 'exceed' if 4 * per * N * d * 2 > 126e6 else 'fit in'))


def extra_seqshard(dev, rank, world, steps, barrier):
    """One long sequence sharded along N over the ranks: halo exchange (point to point), MAX all-reduce of the
    key log-scale, SUM all-reduce of [KV | sum phi(K)], then the band stage on local memory."""
    import torch.distributed as dist
    from fly_b200 import ops
    from fly_b200.seqshard import sblocal_forward_seqshard, shard_bounds
    spec = WORKLOADS[SEQSHARD_WORKLOAD]
    dtype, B, H, N, d, w, m, seed = spec
    q, k, v, W = make_inputs(spec, 'cpu')
    bounds = shard_bounds(N, world)
    lo, hi = bounds[rank], bounds[rank + 1]
    # K and V of the shard live in caller-owned buffers that already have room for the halo rows, so the forward
    # does not copy the shard next to them
    from fly_b200.seqshard import HaloBuffers
    hb = HaloBuffers(B, N, H, d, d, w, q.dtype, dev)
    hb.k_local.copy_(k[:, lo:hi])
    hb.v_local.copy_(v[:, lo:hi])
    ql, kl, vl, Wd = q[:, lo:hi].to(dev), hb.k_local, hb.v_local, W.to(dev)
    run = lambda timings=None: sblocal_forward_seqshard(ql, kl, vl, Wd, w, N, timings=timings, halo_buffers=hb)
    for _ in range(3):
        out = run()
    ms = timed_blocks(run, steps, 3, barrier)
    stages = []
    run(stages)
    torch.cuda.synchronize(dev)
    stage_ms = {name: stages[i - 1][1].elapsed_time(ev) for i, (name, ev) in enumerate(stages) if i > 0}
    vals = max_over_ranks(ms + [stage_ms['halo+max'], stage_ms['allreduce'], stage_ms['band'],
                                stage_ms['logscale'], stage_ms['summary']], dev, world)
    ms_step = statistics.median(vals[:3]) / steps
    # parity of the sharded result against the same sequence run on one GPU (rank 0 holds both)
    gathered = [torch.empty(B, bounds[r + 1] - bounds[r], H, d, device=dev, dtype=out.dtype) for r in range(world)]
    dist.all_gather(gathered, out.contiguous())
    rel = None
    if rank == 0:
        single = ops.Problem(q.to(dev), k.to(dev), v.to(dev), Wd, w)
        ref = single.forward().float()
        single.check_status()
        got = torch.cat(gathered, dim=1).float()
        rel = float((got - ref).abs().max() / ref.abs().max())
    halo_ms, ar_ms, band_ms, ls_ms, sum_ms = vals[3:]
    return dict(workload=SEQSHARD_WORKLOAD, ms_per_step=ms_step, tokens_per_s=B * N / (ms_step * 1e-3),
                rel_err_vs_single_gpu=rel, halo_ms=halo_ms, allreduce_ms=ar_ms,
                stage_ms=dict(logscale=ls_ms, halo_and_max_allreduce=halo_ms, summary=sum_ms, sum_allreduce=ar_ms,
                              band=band_ms),
                buffers='K/V shard written in place into halo-extended buffers (HaloBuffers): no per-call copy',
                not_overlapped='the SUM all-reduce (every band tile needs the reduced summary) and what is left of '
                               'the halo wait after the key log-scale pass, which runs while the halo rows fly',
                note='the long-sequence configuration (d=128, w=512, m=512) through the tensor-core kernels')


def run_t2t(args, dev):
    """Whole T2T-ViT-t-14 forward (random-init, fp32 images) with SBLocal attention in both token stages, and the
    two attention stages alone; inputs come from pinned host memory and logits return to the host every step."""
    from fly_b200 import ops, t2t_vit
    batch = 64
    torch.manual_seed(0)
    model = t2t_vit.t2t_vit_t_14(t2t_vit.sblocal_factory(256, 256), t2t_vit.sblocal_factory(256, 256)).eval()
    layers = [model.patch_embed.attention1.attn.attention_layer, model.patch_embed.attention2.attn.attention_layer]
    for layer in layers:
        layer.feature_map.new_feature_map('cpu')
    model = model.to(dev)
    img_h = torch.randn(batch, 3, 224, 224).pin_memory()
    logits_h = torch.empty(batch, 1000).pin_memory()

    def step():
        with torch.no_grad():
            logits_h.copy_(model(img_h.to(dev, non_blocking=True)), non_blocking=True)

    out = {}
    for name, cdt in (('fp32_attention', None), ('bf16_attention', torch.bfloat16)):
        for layer in layers:
            layer.compute_dtype = cdt
        for _ in range(max(3, args.warmup)):
            step()
        ms = timed_blocks(step, args.steps, 3, lambda: torch.cuda.synchronize(dev))
        whole = statistics.median(ms) / args.steps
        # the two attention calls alone, on inputs of the shapes and temperatures the model feeds them
        attn_ms = 0.0
        for N, tau in ((3136, 147 ** -0.5), (784, 576 ** -0.5)):
            g = torch.Generator().manual_seed(N)
            q, k, v = ((torch.randn(batch, N, 1, 64, generator=g) / 64 ** 0.25).to(dev) for _ in range(3))
            if cdt is not None:
                q, k, v = q.to(cdt), k.to(cdt), v.to(cdt)
            prob = ops.Problem(q, k, v, layers[0].feature_map.projection_matrix, 256, tau)
            for _ in range(3):
                prob.forward()
            a_ms = timed_blocks(prob.forward, args.steps, 3, lambda: torch.cuda.synchronize(dev))
            attn_ms += statistics.median(a_ms) / args.steps
        out[name] = dict(ms_per_step=whole, images_per_s=batch / (whole * 1e-3), attention_only_ms=attn_ms)
    line = dict(metric='t2t_vit_t14_fwd_images_per_s', value=out['fp32_attention']['images_per_s'], unit='images/s',
                n_gpus=1, steps=args.steps, warmup=max(3, args.warmup),
                ms_per_step=out['fp32_attention']['ms_per_step'], higher_is_better=True, scaling='weak',
                vs_baseline=None, dtype='f32', data='synthetic',
                config=dict(workload=T2T_WORKLOAD, batch=batch, image='3x224x224 fp32 N(0,1)', weights='random init',
                            attention='SBLocal w=256 m=256 in both T2T stages (N=3136, N=784, d=64)',
                            backbone='14 dense blocks, width 384, torch scaled_dot_product_attention'),
                e2e=dict(value=out['fp32_attention']['images_per_s'], unit='images/s',
                         h2d_bytes_per_step=img_h.numel() * 4, d2h_bytes_per_step=logits_h.numel() * 4),
                variants=out)
    emit(json.dumps(line))


_RESULT_FD = None


def emit(text):
    """Writes the result line to the process's original stdout."""
    if _RESULT_FD is None:
        print(text, flush=True)
    else:
        os.write(_RESULT_FD, (text + '\n').encode())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=50)
    ap.add_argument('--warmup', type=int, default=5)
    ap.add_argument('--reps', type=int, default=5, help='timed blocks of --steps steps; the median block is reported')
    ap.add_argument('--workload', default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS) + [T2T_WORKLOAD])
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--cpu-units', type=int, default=4, help='(batch,head) units in the CPU sample')
    ap.add_argument('--steps-cpu', type=int, default=2)
    ap.add_argument('--warmup-cpu', type=int, default=1)
    ap.add_argument('--no-cpu-baseline', action='store_true')
    ap.add_argument('--no-extras', action='store_true', help='skip the cfg1 / strong / seqshard side measurements')
    ap.add_argument('--profile', action='store_true',
                    help='run only warm-up and the timed forwards (for ncu captures); prints no JSON line')
    args = ap.parse_args()
    # stdout carries the one result line: whatever libraries write to file descriptor 1 on the way (NCCL prints
    # its version there) is sent to stderr instead
    global _RESULT_FD
    sys.stdout.flush()
    _RESULT_FD = os.dup(1)
    os.dup2(2, 1)
    rank = int(os.environ.get('RANK', '0'))
    local_rank = int(os.environ.get('LOCAL_RANK', '0'))
    world = int(os.environ.get('WORLD_SIZE', '1'))

    if args.impl == 'reference':
        spec = WORKLOADS[DEFAULT_WORKLOAD if args.workload == T2T_WORKLOAD else args.workload]
        run_reference(args, spec, rank)
        return

    if not torch.cuda.is_available():
        raise SystemExit('bench.py needs a CUDA device: the SBLocal path has no CPU fallback')
    import torch.distributed as dist
    from fly_b200 import _cabi, ops
    from fly_b200.sblocal_attention import SBLocalAttention
    _cabi.load()
    torch.cuda.set_device(local_rank)
    dev = torch.device('cuda', local_rank)
    if args.workload == T2T_WORKLOAD:
        if rank == 0:
            run_t2t(args, dev)
        return
    if world > 1:
        # the collectives of the side measurements are small and latency-bound; keep them on plain rings
        os.environ.setdefault('NCCL_NVLS_ENABLE', '0')
        dist.init_process_group('nccl', device_id=dev)
    args.warmup = max(args.warmup, 3)
    spec = WORKLOADS[args.workload]

    dtype, B, H, N, d, w, m, seed = spec
    q_h, k_h, v_h, W = make_inputs(spec, 'cpu', seed_offset=rank)
    q_h, k_h, v_h = q_h.pin_memory(), k_h.pin_memory(), v_h.pin_memory()
    q, k, v = q_h.to(dev), k_h.to(dev), v_h.to(dev)
    Wd = W.to(dev)
    prob = ops.Problem(q, k, v, Wd, w)
    tensor_path = prob.status_offset is not None

    def barrier():
        if world > 1:
            dist.barrier(device_ids=[local_rank])
        torch.cuda.synchronize(dev)

    # ---- device-resident timing: `value` --------------------------------
    # Inputs + phi(K) workspace of one step exceed the 126 MB L2 for the large workloads; for the small ones a
    # 256 MB buffer is rewritten between timed steps (outside the timed events) so that no step starts L2-warm.
    elem_bytes = 2 if dtype == 'bf16' else 4
    step_bytes = 4 * B * H * N * d * elem_bytes
    flush = None if step_bytes > 192e6 else torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for _ in range(args.warmup):
        prob.forward()
    sampler = ClockSampler(local_rank)
    barrier()
    if rank == 0:
        sampler.start()
    reps = 1 if args.profile else max(1, args.reps)
    block_ms = timed_blocks(prob.forward, args.steps, reps, barrier, flush)
    if rank == 0 and not args.profile:
        # nvidia-smi cannot sample faster than the timed region is long (tens of milliseconds): keep the same
        # step running for 0.6 s more (untimed, results discarded) so that the samples show the clocks under
        # this load rather than the idle clocks around it
        t_end = time.time() + 0.6
        while time.time() < t_end:
            for _ in range(20):
                prob.forward()
            torch.cuda.synchronize(dev)
    clocks = sampler.stop() if rank == 0 else None
    if clocks is not None:
        clocks['sampled_over'] = 'timed blocks + 0.6 s untimed repeat of the same step, nvidia-smi every 50 ms'
    if args.profile:
        prob.check_status()
        emit(f'profile run: {block_ms[0] / args.steps:.4f} ms per forward (not a benchmark value)')
        return

    # ---- per-stage timing on the launch stream (roofline of the band kernel) ----
    beta = prob.key_logscale()
    kv, ksum = prob.key_summary(beta)
    prob.band_forward(beta, kv, ksum)
    torch.cuda.synchronize(dev)
    nb = max(5, min(args.steps, 20))
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(nb)]
    stage_ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(nb)]
    for (a, b), se in zip(evs, stage_ev):
        se[0].record()
        prob.key_logscale()
        se[1].record()
        prob.key_summary(beta)          # also evicts the band kernel's inputs from L2 between repeats
        se[2].record()
        a.record()
        prob.band_forward(beta, kv, ksum)
        b.record()
    torch.cuda.synchronize(dev)
    band_ms = sum(a.elapsed_time(b) for a, b in evs) / nb
    logscale_ms = sum(se[0].elapsed_time(se[1]) for se in stage_ev) / nb
    summary_ms = sum(se[1].elapsed_time(se[2]) for se in stage_ev) / nb

    # ---- end to end through the module: host buffers in, host buffer out ----
    layer = SBLocalAttention(w, d, m).to(dev).eval()
    layer.feature_map.new_feature_map(dev)
    layer.feature_map.projection_matrix.copy_(Wd)
    e2e_steps = max(3, min(args.steps, 10))
    # Three streams, two buffer sets: the host->device copy of step i+1 and the device->host copy of
    # step i-1 overlap the kernels of step i (PCIe is full duplex).  Every step still copies its own
    # q, k, v from pinned host memory and its own output back to pinned host memory.
    s_in, s_cmp, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    dev_in = [[torch.empty_like(x, device=dev) for x in (q_h, k_h, v_h)] for _ in range(2)]
    out_hs = [torch.empty(B, N, H, d, dtype=q_h.dtype).pin_memory() for _ in range(2)]
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_cmp = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]

    def e2e_run(n):
        for i in range(n):
            bset = i & 1
            with torch.cuda.stream(s_in):
                if i >= 2:
                    s_in.wait_event(ev_cmp[bset])        # kernels of step i-2 are done with this input set
                for dst, src in zip(dev_in[bset], (q_h, k_h, v_h)):
                    dst.copy_(src, non_blocking=True)
                ev_in[bset].record(s_in)
            with torch.cuda.stream(s_cmp):
                s_cmp.wait_event(ev_in[bset])
                with torch.no_grad():
                    o, _ = layer(*dev_in[bset])
                ev_cmp[bset].record(s_cmp)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_cmp[bset])
                if i >= 2:
                    s_out.wait_event(ev_out[bset])       # (same stream, kept for clarity) host buffer reuse
                o.record_stream(s_out)
                out_hs[bset].copy_(o, non_blocking=True)
                ev_out[bset].record(s_out)
        for st_ in (s_in, s_cmp, s_out):
            torch.cuda.current_stream(dev).wait_stream(st_)

    e2e_run(3)
    e2e_reps = []
    for _ in range(3):                                   # host-link bandwidth is noisy: median of 3 repeats
        barrier()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        for st_ in (s_in, s_cmp, s_out):
            st_.wait_stream(torch.cuda.current_stream(dev))
        e2e_run(e2e_steps)
        s1.record()
        barrier()
        e2e_reps.append(s0.elapsed_time(s1))
    e2e_ms = sorted(e2e_reps)[1]

    vals = max_over_ranks(block_ms + [e2e_ms, band_ms], dev, world)
    block_ms, e2e_ms, band_ms = vals[:reps], vals[reps], vals[reps + 1]
    prob.check_status()     # raises if any kernel gave up on a bounded wait
    ms = statistics.median(block_ms)

    # ---- side measurements (all ranks take part in the distributed ones) ----
    extra = {}
    if not args.no_extras and args.workload == DEFAULT_WORKLOAD:
        side_steps = max(3, min(args.steps, 10))
        if world == 1:
            if rank == 0:
                extra['cfg1'] = extra_cfg1(dev, side_steps)
                peak_tf = load_peaks()['bf16_tflops']
                extra['cfg3'] = extra_tensor_config(dev, 'sblocal_bf16_B4_H12_N4096_d64_w256_m256', side_steps, peak_tf)
                extra['cfg5'] = extra_tensor_config(dev, 'sblocal_bf16_B1_H8_N131072_d128_w512_m512', side_steps,
                                                    peak_tf)
        else:
            extra['strong'] = extra_strong(dev, rank, world, spec, side_steps, barrier)
            extra['seqshard'] = extra_seqshard(dev, rank, world, side_steps, barrier)

    if rank == 0:
        peaks = load_peaks()
        tokens_per_step = world * B * N
        ms_per_step = ms / args.steps
        value = tokens_per_step / (ms_per_step * 1e-3)
        e2e_value = tokens_per_step / (e2e_ms / e2e_steps * 1e-3)
        th = B * H * N
        band_flops = band_flops_per_token_head(d, d, w, m) * th
        fwd_flops = flops_per_token_head(d, d, w, m) * th
        elem = 2 if dtype == 'bf16' else 4
        peak_tf = peaks['bf16_tflops']
        achieved = band_flops / (band_ms * 1e-3) / 1e12
        launches_per_step = 5 if tensor_path else 8
        band_traffic = load_band_traffic(B, H, N, d, w, m) if tensor_path else None
        line = dict(
            metric=METRIC, value=value, unit='tokens/s', n_gpus=world, steps=args.steps, warmup=args.warmup,
            ms_per_step=ms_per_step, higher_is_better=True, scaling='weak', vs_baseline=None,
            dtype='bf16' if dtype == 'bf16' else 'f32', data='synthetic',
            config=dict(workload=args.workload, B_per_gpu=B, global_batch=world * B, H=H, N=N, d=d, window=w,
                        features=m, sharding='batch x head, no collective',
                        l2=('inputs of one step (%.0f MB) exceed the 126 MB L2' % (4 * th * d * elem / 1e6)
                            if flush is None else
                            'L2 flushed (256 MB buffer rewritten) between timed steps; inputs of one step are %.0f MB'
                            % (4 * th * d * elem / 1e6)),
                        kernels='tcgen05+TMA bf16' if tensor_path else 'generic SIMT fp32 math'),
            timed_blocks=dict(count=reps, steps_each=args.steps, ms_per_step_median=ms_per_step,
                              ms_per_step_min=min(block_ms) / args.steps, ms_per_step_max=max(block_ms) / args.steps),
            clocks=clocks,
            e2e=dict(value=e2e_value, unit='tokens/s', h2d_bytes_per_step=3 * th * d * elem,
                     d2h_bytes_per_step=th * d * elem, steps=e2e_steps,
                     pipeline='3 streams, 2 buffer sets: copies of neighbouring steps overlap the kernels'),
            gpu_launches=launches_per_step * args.steps,
            roofline=dict(bound='tensor', kernel='band', achieved=achieved, peak=peak_tf, unit='TFLOP/s',
                          frac=achieved / peak_tf, traffic=band_traffic, peak_source=peaks['source'],
                          kernel_ms=band_ms),
            stage_ms=dict(key_logscale=logscale_ms, key_summary=summary_ms, band_forward=band_ms),
            roofline_forward=dict(bound='tensor', achieved=fwd_flops / (ms_per_step * 1e-3) / 1e12, peak=peak_tf,
                                  unit='TFLOP/s', frac=fwd_flops / (ms_per_step * 1e-3) / 1e12 / peak_tf,
                                  hbm_gbs=4 * th * d * elem / (ms_per_step * 1e-3) / 1e9,
                                  hbm_peak_gbs=peaks['hbm_gbs']),
        )
        if extra:
            line['extra'] = extra
        if not tensor_path:
            # The generic path computes in fp32 on the FMA pipe: its ceiling is the FP32 peak, not the tensor peak.
            # Measured here with an fp32 (TF32 off) cuBLAS GEMM, 8192^3, best of 5.
            tf32 = torch.backends.cuda.matmul.allow_tf32
            torch.backends.cuda.matmul.allow_tf32 = False
            ga = torch.randn(8192, 8192, device=dev)
            gb = torch.randn(8192, 8192, device=dev)
            best = float('inf')
            for _ in range(6):
                g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                g0.record()
                torch.matmul(ga, gb)
                g1.record()
                torch.cuda.synchronize(dev)
                best = min(best, g0.elapsed_time(g1))
            torch.backends.cuda.matmul.allow_tf32 = tf32
            del ga, gb
            fp32_peak = 2 * 8192 ** 3 / (best * 1e-3) / 1e12
            line['roofline']['fp32_peak_tflops'] = fp32_peak
            line['roofline']['frac_of_fp32_peak'] = achieved / fp32_peak
            line['roofline_forward']['frac_of_fp32_peak'] = line['roofline_forward']['achieved'] / fp32_peak
        if world == 1 and not args.no_cpu_baseline:
            from oracle import sblocal_oracle as so
            cores = os.cpu_count() or 1
            units = max(1, min(B * H, args.cpu_units))
            cpu_t, kind, ref_out, (cq, ck, cv, cW) = time_cpu_forward(spec, units, 1, 1)
            line['cpu_baseline'] = dict(value=units * N / cpu_t / H, unit='tokens/s', cores=cores, kind=kind,
                                        sample=cpu_sample_text(units, spec, kind))
            # the same sample through the CUDA path, as a live parity figure
            dq, dk, dv = (x.to(dev).to(q.dtype) for x in (cq, ck, cv))
            got = ops.sblocal_forward(dq, dk, dv, cW.to(dev), w).float().cpu()
            line['parity_vs_cpu_sample'] = so.rel_err(got, ref_out)
        emit(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == '__main__':
    main()
