"""Case table shared by the golden-vector generator and the tests that read
the vectors.  Inputs are regenerated from numpy's legacy RandomState (stable
across numpy versions and machines); only the projection W (drawn through
torch's QR) and the reference outputs are stored in the .npz files."""
import numpy as np

# name: dict(B,H,T,S,E,D,w,nb,tau,eps,ragged,seed,scale,weights,bf16)
#   nb      nb_features handed to the constructor (m = 2*(nb//2))
#   tau     softmax_temp (None -> 1/sqrt(E))
#   ragged  draw key lengths in [S//4, S) like the reference test does
#   scale   'unit' -> N(0,1) inputs (reference test), 'd4' -> N(0,1)/E^0.25 (benchmark inputs)
#   weights also store the three dense attention matrices (need_weights path)
#   bf16    inputs are rounded to bf16 before the fp32 reference runs
CASES = {}


def _add(name, **kw):
    base = dict(B=2, H=2, T=47, S=39, E=21, D=17, w=4, nb=26, tau=None, eps=0.0, ragged=True,
                seed=0, scale='unit', weights=False, bf16=False)
    base.update(kw)
    CASES[name] = base


_seed = 100
# The reference test's own grid (tests/models/attention/test_sblocal_attention.py:24-27),
# on a smaller batch.
for _w in (3, 4, 28, 33):
    for _nb in (73, 26):
        for _tau in (None, 1.0, 0.235):
            _seed += 1
            _add(f'reftest_w{_w}_nb{_nb}_tau{_tau}', B=3, H=2, w=_w, nb=_nb, tau=_tau, seed=_seed,
                 weights=(_w in (4, 33) and _nb == 26))
# LRA-style configuration (configs/experiment/lra/*/sblocal.yaml: eps=1e-4, w 32..128, m 16..64)
_add('lra_eps_w32_nb32', B=2, H=2, T=200, S=200, E=32, D=32, w=32, nb=32, eps=1e-4, seed=201)
_add('lra_eps_w128_nb64_ragged', B=3, H=2, T=300, S=300, E=64, D=64, w=128, nb=64, eps=1e-4, seed=202)
# T != S without a mask, window wider than the sequence, single-row sequence
_add('t_ne_s_nomask', T=70, S=50, E=16, D=24, w=16, nb=32, ragged=False, seed=203)
_add('window_wider_than_seq', T=40, S=40, E=32, D=32, w=128, nb=64, ragged=False, seed=204, scale='d4')
_add('single_token', B=1, H=1, T=1, S=1, E=8, D=8, w=4, nb=8, ragged=False, seed=205)
_add('default_nb_features', B=1, H=2, T=96, S=96, E=16, D=16, w=8, nb=None, ragged=False, seed=206)
# Benchmark-shaped heads: (d,w,m) = (64,256,256) and (128,512,512); T2T stage temperatures
_add('bench_d64_w256_m256', B=1, H=2, T=640, S=640, E=64, D=64, w=256, nb=256, ragged=False, seed=301, scale='d4')
_add('t2t_stage1_tau', B=2, H=1, T=448, S=448, E=64, D=64, w=256, nb=256, tau=147 ** -0.5, ragged=False, seed=302, scale='d4')
_add('t2t_stage2_tau', B=2, H=1, T=392, S=392, E=64, D=64, w=256, nb=256, tau=576 ** -0.5, ragged=False, seed=303, scale='d4')
_add('bench_d128_w512_m512', B=1, H=1, T=1100, S=1100, E=128, D=128, w=512, nb=512, ragged=False, seed=304, scale='d4')
_add('bench_d64_ragged', B=3, H=1, T=520, S=520, E=64, D=64, w=256, nb=256, ragged=True, seed=305, scale='d4')
# bf16-rounded inputs (the bf16 path is compared with the fp32 reference on the same rounded inputs)
_add('bf16_d64_w256_m256', B=1, H=3, T=700, S=700, E=64, D=64, w=256, nb=256, ragged=False, seed=401, scale='d4', bf16=True)
_add('bf16_d128_w512_m512', B=1, H=1, T=1100, S=1100, E=128, D=128, w=512, nb=512, ragged=False, seed=402, scale='d4', bf16=True)
_add('bf16_d64_ragged', B=2, H=2, T=520, S=520, E=64, D=64, w=256, nb=256, ragged=True, seed=403, scale='d4', bf16=True)


def bf16_round(a):
    """Round-to-nearest-even fp32 -> bf16 -> fp32, in numpy."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    r = ((u >> 16) & 1) + np.uint32(0x7FFF)
    return ((u + r) & np.uint32(0xFFFF0000)).view(np.float32)


def make_inputs(case):
    """Returns q (B,T,H,E), k (B,S,H,E), v (B,S,H,D) as fp32 numpy arrays and
    key lengths (B,) int64 or None."""
    c = case
    rs = np.random.RandomState(c['seed'])
    q = rs.standard_normal((c['B'], c['T'], c['H'], c['E'])).astype(np.float32)
    k = rs.standard_normal((c['B'], c['S'], c['H'], c['E'])).astype(np.float32)
    v = rs.standard_normal((c['B'], c['S'], c['H'], c['D'])).astype(np.float32)
    if c['scale'] == 'd4':
        q /= np.float32(c['E'] ** 0.25)
        k /= np.float32(c['E'] ** 0.25)
        v /= np.float32(c['E'] ** 0.25)
    lengths = None
    if c['ragged']:
        lengths = rs.randint(c['S'] // 4, c['S'], size=(c['B'],)).astype(np.int64)
    if c['bf16']:
        q, k, v = bf16_round(q), bf16_round(k), bf16_round(v)
    return q, k, v, lengths
