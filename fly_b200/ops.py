"""Functional layer over the C ABI: builds `SblParams` from torch tensors and
launches on the current CUDA stream.  PyTorch is used only for device memory
and streams; all arithmetic happens in libsblocal_b200.so.
"""
import collections
import ctypes
import math
import threading

import torch

from . import _cabi

_DTYPES = {torch.float32: _cabi.SBL_DTYPE_F32, torch.bfloat16: _cabi.SBL_DTYPE_BF16}
_ws_lock = threading.Lock()
_workspaces = {}


class _StatusWatch:
    """Device status words of earlier forwards, looked at without ever blocking the host.

    The tensor-core kernels leave three int32 words in the workspace (a bounded wait that ran out; an exponential
    that left the fp32 range; a row whose low-rank estimate swamped its exact part).  `post` queues an asynchronous copy of them into pinned host memory behind a
    forward; `poll` inspects the copies that have already landed and raises for the first bad one.  A module
    calls `poll` at the start of every forward, so a bad result is reported by the next call at the latest
    (or by `Problem.check_status`, which synchronises)."""

    def __init__(self):
        self._lock = threading.Lock()
        self._pending = collections.deque()
        self._free = []

    def post(self, workspace, offset, device):
        with self._lock:
            host = self._free.pop() if self._free else torch.empty(3, dtype=torch.int32).pin_memory()
        words = workspace[offset:offset + 12].view(torch.int32)
        host.copy_(words, non_blocking=True)
        event = torch.cuda.Event()
        event.record(torch.cuda.current_stream(device))
        with self._lock:
            self._pending.append((event, host))

    def poll(self):
        while True:
            with self._lock:
                if not self._pending or not self._pending[0][0].query():
                    return
                _, host = self._pending.popleft()
                wait_site, out_of_range, imprecise = host.tolist()
                self._free.append(host)
            if wait_site:
                raise _cabi.SblError(_cabi.SBL_ERR_DEVICE_STATUS,
                                     f'an earlier forward gave up on a bounded wait inside a kernel (wait site '
                                     f'{wait_site}); its output is invalid')
            if out_of_range:
                raise _cabi.SblError(_cabi.SBL_ERR_DEVICE_STATUS,
                                     'an earlier forward met logits beyond the range of the bf16 tensor-core kernels '
                                     '(an exponential left the fp32 range); its output is invalid -- use fp32 inputs '
                                     'or Problem(..., generic=True)')
            if imprecise:
                raise _cabi.SblError(_cabi.SBL_ERR_DEVICE_STATUS,
                                     'an earlier forward met query rows whose in-window low-rank estimate is more than '
                                     '16 times their exact softmax mass (logits 3-4 times the unit scale): the bf16 '
                                     'tensor-core kernels lose accuracy there -- use fp32 inputs or '
                                     'Problem(..., generic=True)')


status_watch = _StatusWatch()


class Problem:
    """One SBLocal problem: parameter block plus the tensors it borrows (kept
    alive for as long as the block is used)."""

    def __init__(self, query, key, value, W, local_context, softmax_temp=None, softmax_eps=0.0,
                 key_lengths=None, out=None, q_pos0=0, k_pos0=0, S_total=None, sum_range=None, generic=False):
        if not (query.is_cuda and key.is_cuda and value.is_cuda):
            raise ValueError('sblocal_b200 runs on CUDA tensors only (there is no CPU path)')
        if query.dim() != 4 or key.dim() != 4 or value.dim() != 4:
            raise ValueError('query/key/value must be (B,T,H,E), (B,S,H,E), (B,S,H,D)')
        if query.dtype not in _DTYPES:
            raise TypeError(f'dtype {query.dtype} is not supported (float32 and bfloat16 are)')
        if key.dtype != query.dtype or value.dtype != query.dtype:
            raise TypeError('query, key and value must share one dtype')
        B, T, H, E = query.shape
        Bk, S, Hk, Ek = key.shape
        Bv, Sv, Hv, D = value.shape
        if (Bk, Hk, Ek) != (B, H, E) or (Bv, Sv, Hv) != (B, S, H):
            raise ValueError(f'shape mismatch: query {tuple(query.shape)}, key {tuple(key.shape)}, '
                             f'value {tuple(value.shape)}')
        if W.dim() != 2 or W.shape[1] != E:
            raise ValueError(f'projection must be (r, {E}), got {tuple(W.shape)}')
        dev = query.device
        # feature axis must be contiguous; the other axes are passed as strides
        query = query if query.stride(-1) == 1 else query.contiguous()
        key = key if key.stride(-1) == 1 else key.contiguous()
        value = value if value.stride(-1) == 1 else value.contiguous()
        W32 = W.detach().to(device=dev, dtype=torch.float32).contiguous()
        if out is None:
            out = torch.empty(B, T, H, D, device=dev, dtype=query.dtype)
        elif out.shape != (B, T, H, D) or out.dtype != query.dtype or out.stride(-1) != 1:
            raise ValueError('out must be (B,T,H,D) in the input dtype with a contiguous last axis')
        if key_lengths is not None:
            key_lengths = key_lengths.to(device=dev, dtype=torch.int64).contiguous()
            if key_lengths.shape != (B,):
                raise ValueError(f'key lengths must have shape ({B},)')
        tau = float(softmax_temp) if softmax_temp else 1.0 / math.sqrt(E)
        p = _cabi.SblParams()
        p.dtype = _DTYPES[query.dtype]
        p.B, p.H, p.T, p.S, p.E, p.D = B, H, T, S, E, D
        p.r, p.w = W.shape[0], int(local_context)
        p.softmax_temp, p.softmax_eps = tau, float(softmax_eps)
        p.q, p.q_stride_b, p.q_stride_t, p.q_stride_h = (query.data_ptr(), query.stride(0), query.stride(1),
                                                         query.stride(2))
        p.k, p.k_stride_b, p.k_stride_s, p.k_stride_h = key.data_ptr(), key.stride(0), key.stride(1), key.stride(2)
        p.v, p.v_stride_b, p.v_stride_s, p.v_stride_h = (value.data_ptr(), value.stride(0), value.stride(1),
                                                         value.stride(2))
        p.out, p.o_stride_b, p.o_stride_t, p.o_stride_h = out.data_ptr(), out.stride(0), out.stride(1), out.stride(2)
        p.W = W32.data_ptr()
        p.key_lengths = key_lengths.data_ptr() if key_lengths is not None else None
        p.q_pos0, p.k_pos0 = int(q_pos0), int(k_pos0)
        p.S_total = int(S_total) if S_total is not None else S
        p.sum_lo, p.sum_hi = sum_range if sum_range is not None else (0, S)
        p.flags = _cabi.SBL_FLAG_GENERIC_PATH if generic else 0
        self.params = p
        self.device = dev
        self.out = out
        self.m = 2 * W.shape[0]
        self.shape = (B, H, T, S, E, D)
        self._keep = (query, key, value, W32, key_lengths, out)
        lib = _cabi.load()
        nbytes = ctypes.c_size_t(0)
        _cabi.check(lib.sbl_workspace_bytes(ctypes.byref(p), ctypes.byref(nbytes)))
        self.workspace_bytes = nbytes.value
        off = ctypes.c_size_t(0)
        self.status_offset = off.value if lib.sbl_status_words(ctypes.byref(p), ctypes.byref(off)) == 0 else None

    def workspace(self):
        """Grow-only scratch buffer per (device, stream)."""
        stream = torch.cuda.current_stream(self.device)
        key = (self.device.index, stream.cuda_stream)
        with _ws_lock:
            buf = _workspaces.get(key)
            if buf is None or buf.numel() < self.workspace_bytes:
                buf = torch.empty(max(self.workspace_bytes, 1 << 20), dtype=torch.uint8, device=self.device)
                _workspaces[key] = buf
        return buf

    def _call(self, fn, *extra, workspace=None):
        ws = workspace if workspace is not None else self.workspace()
        with torch.cuda.device(self.device):
            stream = torch.cuda.current_stream(self.device).cuda_stream
            rc = fn(ctypes.byref(self.params), ws.data_ptr(), ws.numel(), *extra, stream)
        _cabi.check(rc)
        return ws

    # -- entry points -----------------------------------------------------
    def forward(self, workspace=None, watch=False):
        """watch: queue a non-blocking copy of the kernels' status words (see `status_watch`)."""
        ws = self._call(_cabi.load().sbl_forward, workspace=workspace)
        if watch and self.status_offset is not None:
            with torch.cuda.device(self.device):
                status_watch.post(ws, self.status_offset, self.device)
        return self.out

    def check_status(self, workspace=None):
        """Synchronises the stream; raises if a kernel gave up on a bounded wait."""
        self._call(_cabi.load().sbl_check_status, workspace=workspace)

    def key_logscale(self, workspace=None):
        B, H = self.shape[:2]
        beta = torch.empty(B, H, device=self.device, dtype=torch.float32)
        self._call(_cabi.load().sbl_key_logscale, beta.data_ptr(), workspace=workspace)
        return beta

    def key_summary(self, beta, workspace=None, out=None):
        """out: optional (kv, ksum) pair of contiguous fp32 tensors (B,H,m,D) and (B,H,m) to write into (a caller
        that all-reduces both can make them two views of one buffer)."""
        B, H, _, _, _, D = self.shape
        if out is None:
            kv = torch.empty(B, H, self.m, D, device=self.device, dtype=torch.float32)
            ksum = torch.empty(B, H, self.m, device=self.device, dtype=torch.float32)
        else:
            kv, ksum = out
            if (tuple(kv.shape) != (B, H, self.m, D) or tuple(ksum.shape) != (B, H, self.m)
                    or kv.dtype != torch.float32 or ksum.dtype != torch.float32
                    or not kv.is_contiguous() or not ksum.is_contiguous() or kv.device != self.device):
                raise ValueError('out must be contiguous fp32 (B,H,m,D) and (B,H,m) tensors on the problem device')
        beta = beta.contiguous()
        self._call(_cabi.load().sbl_key_summary, beta.data_ptr(), kv.data_ptr(), ksum.data_ptr(),
                   workspace=workspace)
        return kv, ksum

    def band_forward(self, beta, kv, ksum, workspace=None):
        beta, kv, ksum = beta.contiguous(), kv.contiguous(), ksum.contiguous()
        self._call(_cabi.load().sbl_band_forward, beta.data_ptr(), kv.data_ptr(), ksum.data_ptr(),
                   workspace=workspace)
        return self.out

    def attention_weights(self, unnormalized=False, workspace=None):
        """Dense (B,H,T,S) attention matrix (and, with `unnormalized`, the two
        unnormalised matrices) of the forward just run on this workspace; the
        problem must have been created with generic=True."""
        B, H, T, S = self.shape[:4]
        mk = lambda: torch.empty(B, H, T, S, device=self.device, dtype=torch.float32)
        attn = mk()
        un, lr = (mk(), mk()) if unnormalized else (None, None)
        self._call(_cabi.load().sbl_attention_weights, attn.data_ptr(), un.data_ptr() if unnormalized else None,
                   lr.data_ptr() if unnormalized else None, workspace=workspace)
        return (attn, un, lr) if unnormalized else attn

    def query_features(self):
        B, H, T = self.shape[:3]
        qp = torch.empty(B, H, T, self.m, device=self.device, dtype=torch.float32)
        ls = torch.empty(B, H, T, device=self.device, dtype=torch.float32)
        self._call(_cabi.load().sbl_query_features, qp.data_ptr(), ls.data_ptr())
        return qp, ls

    def key_features(self):
        B, H, _, S = self.shape[:4]
        kp = torch.empty(B, H, S, self.m, device=self.device, dtype=torch.float32)
        ls = torch.empty(B, H, device=self.device, dtype=torch.float32)
        self._call(_cabi.load().sbl_key_features, kp.data_ptr(), ls.data_ptr())
        return kp, ls


def sblocal_forward(query, key, value, W, local_context, softmax_temp=None, softmax_eps=0.0,
                    key_lengths=None, out=None, watch=False):
    """out (B,T,H,D) = SBLocal attention of query (B,T,H,E), key (B,S,H,E),
    value (B,S,H,D) with projection W (r,E); one call of `sbl_forward`."""
    return Problem(query, key, value, W, local_context, softmax_temp, softmax_eps, key_lengths,
                   out).forward(watch=watch)
