"""Host-side mirror of the reference's operator interface.

``flash_attention_v2_cutlass(q, k, v, is_causal=False, softmax_scale=1)`` has the
name, positional order, defaults and return type (a one-element list) of the
reference extension's only export (include/attention_api.h:10-11,
csrc/attention_api.cpp:6-10, csrc/flash_attention.cu:639-668).  torch supplies
device memory and the current stream; the work is done by libfa8_b200.so through
its C ABI.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch

from . import _lib

_status_words = {}


def _check_input(x: torch.Tensor, name: str) -> None:
    # CHECK_INPUT of include/attention_api.cuh:12-18 (TORCH_CHECK -> RuntimeError)
    if not x.device.type == "cuda":
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if not x.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")


def status_word(device: torch.device) -> torch.Tensor:
    """The int32 device word kernels on `device` report an expired wait into."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _status_words:
        _status_words[idx] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
    return _status_words[idx]


def check_status(device: Optional[torch.device] = None, word: Optional[torch.Tensor] = None) -> None:
    """Synchronises the current stream of `device` and raises RuntimeError if a kernel
    launched through this module reported an expired wait (or the stream is in error).
    Stands where the reference has cudaDeviceSynchronize + CUDA_ERROR_CHECK
    (csrc/flash_attention.cu:663-665), but raises instead of exiting the process."""
    lib = _lib.load()
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    word = status_word(device) if word is None else word
    code = ctypes.c_int32(0)
    with torch.cuda.device(word.device):
        stream = torch.cuda.current_stream(word.device).cuda_stream
        rc = lib.fa8_check_status(word.data_ptr(), stream, ctypes.byref(code))
    if rc != _lib.FA8_OK:
        word.zero_()
        raise RuntimeError(_lib.error_message(rc) + f" (device code 0x{code.value:x})")


def flash_attention_v2_cutlass(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                               is_causal: bool = False, softmax_scale: float = 1.0, *,
                               v_layout: str = "transposed", o_scale: float = 1.0,
                               out: Optional[torch.Tensor] = None,
                               return_lse: bool = False,
                               descale_q: Optional[torch.Tensor] = None,
                               descale_k: Optional[torch.Tensor] = None,
                               descale_v: Optional[torch.Tensor] = None,
                               _status: Optional[torch.Tensor] = None) -> List[torch.Tensor]:
    """FP8 attention forward.

    q, k: float8_e4m3fn (or, all three, float8_e5m2: the reference's FP8_SWITCH,
          csrc/flash_attention.cu:631) [batch, heads, seqlen, head_dim], CUDA, contiguous.  k and v may have
          fewer heads (a divisor of q's): grouped-query attention, query head h reading K/V
          head h // (heads // heads_kv); their sequence length may differ from q's (the causal
          mask stays top-left aligned: key index <= query index).
    v:    float8_e4m3fn, transposed [batch, heads, head_dim, seqlen] as the reference
          requires (test.py:71), or [batch, heads, seqlen, head_dim] with
          v_layout="natural".
    Returns [O] with O fp16 [batch, heads, seqlen, head_dim] (the reference returns
    e4m3, csrc/flash_attention.cu:656).  The kernel is enqueued on the current
    stream; nothing synchronises (the reference blocks, :663-665) - call
    check_status() to synchronise and surface device-side errors.
    descale_q/k/v: optional one-element fp32 CUDA tensors (as returned by quantize_e4m3);
    the kernel folds them into the softmax scale and into O without a host round trip.
    return_lse=True appends the fp32 [batch, heads, seqlen] log-sum-exp of the scaled
    scores (the reference reserves softmax_lse_ptr for it, csrc/flash.h:56, unused).
    """
    lib = _lib.load()
    _check_input(q, "q")
    _check_input(k, "k")
    _check_input(v, "v")
    if q.dtype not in (torch.float8_e4m3fn, torch.float8_e5m2):
        raise RuntimeError(f"q must be float8_e4m3fn (or float8_e5m2), got {q.dtype}")
    for name, t in (("q", q), ("k", k), ("v", v)):
        if t.dtype != q.dtype:
            raise RuntimeError(f"{name} must be {q.dtype} like q (float8_e4m3fn or float8_e5m2), got {t.dtype}")
        if t.dim() != 4:
            raise RuntimeError(f"{name} must have 4 dimensions [batch, heads, seqlen, head_dim]")
        if t.device != q.device:
            raise RuntimeError("q, k and v must be on the same device")
    B, H, S, D = q.shape
    Hk, Sk = k.shape[1], k.shape[2]
    if tuple(k.shape) != (B, Hk, Sk, D) or Hk < 1 or H % Hk != 0:
        raise RuntimeError(f"k must be [batch, heads_kv, seqlen, head_dim] with heads_kv dividing {H}; "
                           f"q is {tuple(q.shape)}, k is {tuple(k.shape)}")
    if v_layout == "transposed":
        want_v, layout = (B, Hk, D, Sk), _lib.FA8_V_TRANSPOSED
    elif v_layout == "natural":
        want_v, layout = (B, Hk, Sk, D), _lib.FA8_V_NATURAL
    else:
        raise RuntimeError("v_layout must be 'transposed' or 'natural'")
    if tuple(v.shape) != want_v:
        raise RuntimeError(f"v must be {want_v} for v_layout='{v_layout}', got {tuple(v.shape)}")
    if out is None:
        out = torch.empty((B, H, S, D), dtype=torch.float16, device=q.device)
    else:
        _check_input(out, "out")
        if out.dtype != torch.float16 or tuple(out.shape) != (B, H, S, D) or out.device != q.device:
            raise RuntimeError("out must be a float16 CUDA tensor shaped like q")
    # one float per tensor, or one per (batch, head): [B*H] for Q, [B*heads_kv] for K and V
    given = [(n, t, full) for n, t, full in (("descale_q", descale_q, B * H), ("descale_k", descale_k, B * Hk),
                                             ("descale_v", descale_v, B * Hk)) if t is not None]
    per_head = any(t.numel() > 1 for _, t, _ in given)
    for name, t, full in given:
        if t.dtype != torch.float32 or t.device != q.device or not t.is_contiguous() or \
                t.numel() != (full if per_head else 1):
            raise RuntimeError(f"{name} must be a contiguous float32 tensor on q's device with one element, or "
                               f"(all three alike) one per (batch, head): {full}")
    lse = torch.empty((B, H, S), dtype=torch.float32, device=q.device) if return_lse else None
    p = _lib.Fa8FwdParams(
        q=q.data_ptr(), k=k.data_ptr(), v=v.data_ptr(), o=out.data_ptr(),
        batch=B, heads=H, seqlen=S, head_dim=D, softmax_scale=float(softmax_scale),
        is_causal=int(bool(is_causal)), v_layout=layout, o_scale=float(o_scale),
        status_word=(_status if _status is not None else status_word(q.device)).data_ptr(),
        softmax_lse=(lse.data_ptr() if lse is not None else None), heads_kv=Hk,
        descale_q=(descale_q.data_ptr() if descale_q is not None else None),
        descale_k=(descale_k.data_ptr() if descale_k is not None else None),
        descale_v=(descale_v.data_ptr() if descale_v is not None else None),
        fp8_format=(_lib.FA8_FP8_E5M2 if q.dtype == torch.float8_e5m2 else _lib.FA8_FP8_E4M3),
        seqlen_k=Sk, descale_per_head=int(per_head))
    with torch.cuda.device(q.device):
        rc = lib.fa8_fwd(ctypes.byref(p), torch.cuda.current_stream(q.device).cuda_stream)
    if rc != _lib.FA8_OK:
        # FA8_ERR_DEVICE_TIMEOUT here means an EARLIER launch on this device failed (the library
        # learns of it through a host-visible flag); it has cleared the status words and did not
        # enqueue this call.  The reference would have exited the process at that launch
        # (include/attention_api.cuh:20-29).
        raise RuntimeError(_lib.error_message(rc))
    return [out, lse] if return_lse else [out]


def quantize_e4m3(x: torch.Tensor, per_head: bool = False):
    """Amax quantisation of a contiguous fp16 / bf16 CUDA tensor: returns (x8, descale) with
    x8 = e4m3(x * 448 / max|x|) shaped like x and x ~= descale * x8.  Per tensor, descale is a
    one-element fp32 tensor; with per_head=True x is [batch, heads, ...] and every (batch,
    head) slice gets its own scale: descale is [batch*heads].  Stream-ordered, two HBM-bound
    kernels; stands where the reference's callers cast with torch (test.py:20-22, 68-70)."""
    lib = _lib.load()
    _check_input(x, "x")
    if x.dtype not in (torch.float16, torch.bfloat16):
        raise RuntimeError(f"x must be float16 or bfloat16, got {x.dtype}")
    dt = _lib.FA8_DTYPE_BF16 if x.dtype == torch.bfloat16 else _lib.FA8_DTYPE_FP16
    if per_head and x.dim() < 3:
        raise RuntimeError("per_head needs a [batch, heads, ...] tensor")
    x8 = torch.empty(x.shape, dtype=torch.float8_e4m3fn, device=x.device)
    n_seg = x.shape[0] * x.shape[1] if per_head else 1
    scal = torch.empty(2 * n_seg, dtype=torch.float32, device=x.device)       # [amax..., descale...]
    with torch.cuda.device(x.device):
        stream = torch.cuda.current_stream(x.device).cuda_stream
        if per_head:
            rc = lib.fa8_quantize_e4m3_segments(x.data_ptr(), dt, x8.data_ptr(), x.numel() // n_seg, n_seg,
                                                scal.data_ptr(), scal.data_ptr() + 4 * n_seg, stream)
        else:
            rc = lib.fa8_quantize_e4m3(x.data_ptr(), dt, x8.data_ptr(), x.numel(), scal.data_ptr(),
                                       scal.data_ptr() + 4, stream)
    if rc != _lib.FA8_OK:
        raise RuntimeError(_lib.error_message(rc))
    return x8, scal[n_seg:]


class HostRunner:
    """End-to-end call with HOST tensors: pinned host -> device copies, the kernel and the
    device -> host copy of O.  The (batch, head) slices are independent, so the call is cut
    into `chunks` groups of slices and pipelined over three streams: the upload of group
    g+1, the kernel of group g and the download of group g-1 overlap, which uses both
    directions of the host link at once.  The last two groups are cut again into pieces that
    shrink by the factor `taper` (see _groups), so that little is left to compute and download
    when the last upload lands.  The call returns after O has landed in pinned host
    memory: a tensor of its own for every call (torch's pinned-memory cache makes that cheap
    once an earlier result has been released), or the caller's `out=` (fp16, shaped like q;
    pinned if the download is to overlap).  Device buffers are allocated once per shape and
    reused.  Each runner has its own device status word."""

    def __init__(self, device: Optional[torch.device] = None, chunks: int = 6, timing: bool = False, taper: float = 2.0 / 3.0):
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
        self.chunks = max(1, int(chunks))
        self.taper = min(max(0.0, float(taper)), 0.9)
        # timing=True brackets every copy group and kernel with CUDA events and leaves the busy
        # time of each stage of the last call in `last_timing` (milliseconds, summed over groups)
        self.timing = bool(timing)
        self.last_timing = None
        self._key = None
        self._streams = None
        self._status = torch.zeros(1, dtype=torch.int32, device=self.device)

    def _ensure(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor):
        key = (tuple(q.shape), tuple(k.shape), tuple(v.shape), q.dtype)
        if key == self._key:
            return
        B, H, S, D = q.shape
        dev = self.device
        self.dq = torch.empty(q.shape, dtype=q.dtype, device=dev)
        self.dk = torch.empty(k.shape, dtype=k.dtype, device=dev)
        self.dv = torch.empty(v.shape, dtype=v.dtype, device=dev)
        self.do = torch.empty((B, H, S, D), dtype=torch.float16, device=dev)
        if self._streams is None:
            self._streams = tuple(torch.cuda.Stream(device=dev) for _ in range(3))
        self._key = key

    @staticmethod
    def _groups(n: int, parts: int, taper: float = 0.0):
        """[lo, hi) ranges of n slices: `parts` equal groups; with taper > 0 the last two of
        them are cut again into pieces that shrink by that factor (each piece is 1 - taper of
        what is left, at least two slices).  The upload stream is busy from start to end; what
        the call adds to it is the kernel and the download of whatever has not been downloaded
        when the last upload lands.  A download takes about two thirds of the time of the same
        slices' upload, so pieces shrinking by two thirds keep the download stream from
        falling behind while they get small."""
        parts = min(parts, n)
        cuts = [n * g // parts for g in range(parts + 1)]
        if taper <= 0.0 or parts < 2:
            return [(a, b) for a, b in zip(cuts[:-1], cuts[1:])]
        head, lo, hi = cuts[:-2], cuts[-3], cuts[-1]
        tail = []
        while lo < hi:
            tail.append(lo)
            lo += min(hi - lo, max(2, round((hi - lo) * (1.0 - taper))))
        cuts = head[:-1] + tail + [hi]
        return [(a, b) for a, b in zip(cuts[:-1], cuts[1:])]

    def __call__(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, is_causal: bool = False,
                 softmax_scale: float = 1.0, **kw) -> List[torch.Tensor]:
        for name, t in (("q", q), ("k", k), ("v", v)):
            if t.device.type != "cpu":
                raise RuntimeError(f"{name} must be a host tensor")
            if t.dim() != 4 or not t.is_contiguous():
                raise RuntimeError(f"{name} must be a contiguous 4-dimensional tensor")
        self._ensure(q, k, v)
        host_out = kw.pop("out", None)
        if host_out is None:
            host_out = torch.empty(self.do.shape, dtype=torch.float16, pin_memory=True)
        elif (host_out.device.type != "cpu" or host_out.dtype != torch.float16 or not host_out.is_contiguous()
              or tuple(host_out.shape) != tuple(self.do.shape)):
            raise RuntimeError("out must be a contiguous float16 host tensor shaped like q")
        B, H, Hk = q.shape[0], q.shape[1], k.shape[1]
        per_head = any(kw.get(n) is not None and kw[n].numel() > 1 for n in ("descale_q", "descale_k", "descale_v"))
        # A group is a contiguous range of every tensor: a range of the flattened (batch, head)
        # axis when K and V have one head per query head, a range of batch entries otherwise.
        # Row log-sum-exps and per-head descales are indexed by slice: one group then.
        flat = (H == Hk)
        if kw.get("return_lse") or per_head:
            groups = [(0, B * H if flat else B)]
        else:
            groups = self._groups(B * H if flat else B, self.chunks, self.taper)
        if flat:
            hq, hk, hv, dq, dk, dv, do, ho = (t.view(1, B * t.shape[1], t.shape[2], t.shape[3])
                                              for t in (q, k, v, self.dq, self.dk, self.dv, self.do, host_out))
            cut = lambda t, a, b: t[:, a:b]
        else:
            hq, hk, hv, dq, dk, dv, do, ho = q, k, v, self.dq, self.dk, self.dv, self.do, host_out
            cut = lambda t, a, b: t[a:b]
        s_in, s_run, s_out = self._streams
        start = torch.cuda.Event()
        start.record(torch.cuda.current_stream(self.device))
        for st in self._streams:
            st.wait_event(start)
        extra = []
        marks = {"h2d": [], "kernel": [], "d2h": []}

        def mark(stage, stream):
            if self.timing:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record(stream)
                marks[stage].append(ev)

        for (a, b) in groups:
            with torch.cuda.stream(s_in):
                mark("h2d", s_in)
                cut(dq, a, b).copy_(cut(hq, a, b), non_blocking=True)
                cut(dk, a, b).copy_(cut(hk, a, b), non_blocking=True)
                cut(dv, a, b).copy_(cut(hv, a, b), non_blocking=True)
                mark("h2d", s_in)
                up = torch.cuda.Event()
                up.record(s_in)
            with torch.cuda.stream(s_run):
                s_run.wait_event(up)
                mark("kernel", s_run)
                if len(groups) == 1:      # whole tensors in their own shape (lse and per-head descales follow it)
                    extra = flash_attention_v2_cutlass(self.dq, self.dk, self.dv, is_causal, softmax_scale,
                                                       out=self.do, _status=self._status, **kw)[1:]
                else:
                    flash_attention_v2_cutlass(cut(dq, a, b), cut(dk, a, b), cut(dv, a, b), is_causal, softmax_scale,
                                               out=cut(do, a, b), _status=self._status, **kw)
                mark("kernel", s_run)
                ran = torch.cuda.Event()
                ran.record(s_run)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ran)
                mark("d2h", s_out)
                cut(ho, a, b).copy_(cut(do, a, b), non_blocking=True)
                mark("d2h", s_out)
        s_out.synchronize()
        if self.timing:
            self.last_timing = {st: sum(ev[i].elapsed_time(ev[i + 1]) for i in range(0, len(ev), 2))
                                for st, ev in marks.items()}
        check_status(self.device, word=self._status)
        return [host_out] + [t.cpu() for t in extra]

    def bytes_per_call(self, q: torch.Tensor, v: torch.Tensor, k: Optional[torch.Tensor] = None):
        h2d = q.numel() + (q.numel() if k is None else k.numel()) + v.numel()
        d2h = 2 * q.numel()
        return h2d, d2h
