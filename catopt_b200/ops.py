"""Functional wrappers: torch CUDA tensors in, one C-ABI call each.

torch is used for device memory and streams only; every arithmetic step runs in
``libcatopt_b200.so``.  Scratch buffers are torch allocations cached per
(device, purpose) and grown on demand, so steady-state calls allocate nothing
and can be captured in a CUDA graph after a warm-up call.  The cache is keyed by
the current stream as well, so concurrent streams never share a buffer; calls on
one stream do, which stream order makes safe.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from ._lib import B200Error, check, dtype_code, require_cuda, require_device, stream_ptr

_scratch: dict[tuple, torch.Tensor] = {}
_status_words: dict[int, torch.Tensor] = {}


def _scratch_buf(purpose: str, nbytes: int, device: torch.device) -> torch.Tensor | None:
    """A cached uint8 scratch buffer of at least ``nbytes`` (``None`` for 0), one per
    (purpose, device, current stream): calls on different streams never share one."""
    if nbytes <= 0:
        return None
    key = (purpose, device.index, torch.cuda.current_stream(device).cuda_stream)
    buf = _scratch.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(nbytes, dtype=torch.uint8, device=device)
        _scratch[key] = buf
    return buf


def device_status(device: torch.device) -> torch.Tensor:
    """The per-device int32 word kernels write CB2_WAIT_TIMEOUT into."""
    w = _status_words.get(device.index)
    if w is None:
        w = torch.zeros(1, dtype=torch.int32, device=device)
        _status_words[device.index] = w
    return w


def check_device_status(device: torch.device | None = None) -> None:
    """Synchronise and raise if a kernel recorded a bounded-wait timeout."""
    device = device or torch.device("cuda", torch.cuda.current_device())
    w = _status_words.get(device.index)
    if w is None:
        return
    code = int(w.item())
    if code != 0:
        w.zero_()
        site = f", wait at source line {code >> 8} of the kernel" if code >> 8 else ""
        raise B200Error(f"device status: {_lib.status_str(code & 0xff)} (status {code & 0xff}{site})")


def wait_for_flag(flag: torch.Tensor, budget_us: int = 1000) -> None:
    """Order the current stream behind a device flag with a bound: ``cb2_wait_for_flag``
    polls ``flag`` (int32, one element) until it is non-zero or ``budget_us`` microseconds
    have passed; an expired wait leaves ``CB2_WAIT_TIMEOUT`` in the device status word
    (``check_device_status`` raises it) and the stream carries on."""
    require_cuda(flag)
    if flag.dtype != torch.int32 or flag.numel() != 1:
        raise B200Error("wait_for_flag takes one int32 flag")
    rc = _lib.load().cb2_wait_for_flag(flag.data_ptr(), int(budget_us), device_status(flag.device).data_ptr(),
                                       stream_ptr())
    check(rc, "cb2_wait_for_flag")


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


# --------------------------------------------------------------------------- verify
def verify_reduce(ref: torch.Tensor, out: torch.Tensor, n_seg: int = 1,
                  result: torch.Tensor | None = None) -> torch.Tensor:
    """Per-segment ``[max|ref-out|, max|ref|, nan_in_diff, nan_in_ref]``.

    ``ref``/``out`` hold ``n_seg`` equally sized comparisons back to back.
    Returns a float32 CUDA tensor ``[n_seg, 4]`` (no host synchronisation).
    """
    require_cuda(ref, out, result)
    if ref.shape != out.shape or ref.dtype != out.dtype:
        raise B200Error("verify_reduce needs identical shape and dtype on both sides")
    numel = ref.numel()
    if n_seg <= 0 or numel == 0 or numel % n_seg:
        raise B200Error(f"cannot split {numel} elements into {n_seg} equal segments")
    if result is None:
        result = torch.empty(n_seg, 4, dtype=torch.float32, device=ref.device)
    elif result.shape != (n_seg, 4) or result.dtype != torch.float32:
        raise B200Error("result must be float32 [n_seg, 4]")
    rc = _lib.load().cb2_verify_reduce(ref.data_ptr(), out.data_ptr(), numel // n_seg, n_seg,
                                       dtype_code(ref.dtype), result.data_ptr(), stream_ptr())
    check(rc, "cb2_verify_reduce")
    return result


# --------------------------------------------------------------------------- chain
def linear_split_weight(w: torch.Tensor) -> torch.Tensor | None:
    """The TF32 hi/lo split of an fp32 weight ``[out, in]`` as one ``[2, out, in]`` tensor, for
    ``linear_f32(..., w_split=...)``: a module whose weight never changes splits it once instead
    of on every call.  ``None`` when the tensor-core path cannot take the shape."""
    require_cuda(w)
    if w.dtype != torch.float32 or w.dim() != 2:
        raise B200Error("linear_split_weight takes a float32 matrix")
    lib = _lib.load()
    if lib.cb2_linear_f32_split_bytes(w.shape[1], w.shape[0]) == 0:
        return None
    out = torch.empty(2, *w.shape, dtype=torch.float32, device=w.device)
    check(lib.cb2_linear_f32_split_weight(w.data_ptr(), out.data_ptr(), w.shape[1], w.shape[0], stream_ptr()),
          "cb2_linear_f32_split_weight")
    return out


def linear_f32(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None,
               out: torch.Tensor | None = None, w_split: torch.Tensor | None = None) -> torch.Tensor:
    """``x @ w.T (+ bias)`` for fp32 ``x[..., in]``, ``w[out, in]``; ``w_split``
    (``linear_split_weight(w)``) spares the per-call split on the tensor-core path."""
    require_cuda(x, w, bias, out, w_split)
    if x.dtype != torch.float32 or w.dtype != torch.float32:
        raise B200Error("linear_f32 takes float32 tensors")
    if w.dim() != 2 or x.shape[-1] != w.shape[1]:
        raise B200Error(f"linear_f32 shape mismatch: x {tuple(x.shape)}, w {tuple(w.shape)}")
    rows = x.numel() // x.shape[-1]
    n_in, n_out = w.shape[1], w.shape[0]
    if out is None:
        out = torch.empty(*x.shape[:-1], n_out, dtype=torch.float32, device=x.device)
    lib = _lib.load()
    status = device_status(x.device)
    if w_split is not None and rows >= 256:
        if tuple(w_split.shape) != (2, n_out, n_in) or w_split.dtype != torch.float32:
            raise B200Error("w_split must be linear_split_weight(w)")
        rc = lib.cb2_linear_f32_presplit(x.data_ptr(), w_split.data_ptr(), _ptr(bias), out.data_ptr(), rows, n_in,
                                         n_out, status.data_ptr(), stream_ptr())
        check(rc, "cb2_linear_f32_presplit")
        return out
    need = lib.cb2_linear_f32_scratch_bytes(rows, n_in, n_out)
    scratch = _scratch_buf("linear", need, x.device)
    rc = lib.cb2_linear_f32(x.data_ptr(), w.data_ptr(), _ptr(bias), out.data_ptr(), rows, n_in,
                            n_out, _ptr(scratch), need, status.data_ptr(), stream_ptr())
    check(rc, "cb2_linear_f32")
    return out


def matmul_f32(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """``a @ b`` for two dense fp32 matrices."""
    require_cuda(a, b)
    if a.dtype != torch.float32 or b.dtype != torch.float32 or a.dim() != 2 or b.dim() != 2:
        raise B200Error("matmul_f32 takes two float32 matrices")
    if a.shape[1] != b.shape[0]:
        raise B200Error(f"matmul_f32 shape mismatch: {tuple(a.shape)} @ {tuple(b.shape)}")
    c = torch.empty(a.shape[0], b.shape[1], dtype=torch.float32, device=a.device)
    rc = _lib.load().cb2_matmul_f32(a.data_ptr(), b.data_ptr(), c.data_ptr(), a.shape[0],
                                    b.shape[1], a.shape[1], stream_ptr())
    check(rc, "cb2_matmul_f32")
    return c


def chain_fold_f32(weights: list[torch.Tensor]) -> torch.Tensor:
    """``W[k-1] @ (... @ (W[1] @ W[0]))`` for nn.Linear-layout fp32 weights."""
    if not weights:
        raise B200Error("chain_fold_f32 needs at least one weight")
    require_cuda(*weights)
    k = len(weights)
    dims = [weights[0].shape[1]]
    for w in weights:
        if w.dtype != torch.float32 or w.dim() != 2 or w.shape[1] != dims[-1]:
            raise B200Error("chain_fold_f32: weights must be float32 [out_i, in_i] and chain")
        dims.append(w.shape[0])
    lib = _lib.load()
    dims_c = (C.c_int * (k + 1))(*dims)
    ptrs = (C.c_void_p * k)(*[w.data_ptr() for w in weights])
    need = lib.cb2_chain_fold_f32_scratch_bytes(dims_c, k)
    scratch = _scratch_buf("fold", need, weights[0].device)
    out = torch.empty(dims[-1], dims[0], dtype=torch.float32, device=weights[0].device)
    rc = lib.cb2_chain_fold_f32(ptrs, dims_c, k, out.data_ptr(), _ptr(scratch), need, stream_ptr())
    check(rc, "cb2_chain_fold_f32")
    return out


# --------------------------------------------------------------------------- decayed
def decayed_chunk_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, gamma: torch.Tensor,
                      chunk: int, scale: float = 1.0, out: torch.Tensor | None = None,
                      one_pass: bool = False) -> torch.Tensor:
    """Decayed causal linear attention ``[B,H,T,d]`` with per-head ``gamma[H]`` (fp32).

    ``one_pass``: on the tensor-core path, withhold the scratch that lets a call with few
    heads run a head's segments in parallel from precomputed start states.  That form
    rounds the carried state at other points than the one-pass walk (same function, other
    last bits), so a caller that cuts one problem into calls of different sizes and wants
    every head's bits independent of the cut asks for the one-pass form."""
    require_cuda(q, k, v, gamma, out)
    if q.dim() != 4 or q.shape != k.shape or v.shape[:3] != q.shape[:3]:
        raise B200Error("decayed_chunk_fwd takes q,k [B,H,T,dk] and v [B,H,T,dv]")
    if not (q.dtype == k.dtype == v.dtype):
        raise B200Error("q, k, v must share one dtype")
    B, H, T, dk = q.shape
    dv = v.shape[-1]
    if gamma.dtype != torch.float32 or gamma.numel() != H:
        raise B200Error("gamma must be float32 with one rate per head")
    if T % chunk:
        raise B200Error(f"T={T} is not a multiple of chunk={chunk}")
    if out is None:
        out = torch.empty_like(v)
    code = dtype_code(q.dtype)
    lib = _lib.load()
    need = lib.cb2_decayed_chunk_scratch_bytes(B, H, T, dk, dv, chunk, code)
    if one_pass and lib.cb2_decayed_chunk_on_tensor_cores(B, H, T, dk, dv, chunk, code):
        need = 0
    scratch = _scratch_buf("decayed", need, q.device)
    status = device_status(q.device)
    rc = lib.cb2_decayed_chunk_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                                   gamma.data_ptr(), B, H, T, dk, dv, chunk, float(scale), code,
                                   _ptr(scratch), need, status.data_ptr(), stream_ptr())
    check(rc, "cb2_decayed_chunk_fwd")
    return out


# --------------------------------------------------------------------------- om causal
def om_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float | None = None,
           out: torch.Tensor | None = None, causal: bool = False) -> torch.Tensor:
    """Softmax attention, unmasked by default (``om_causal_fwd`` with the mask as an argument)."""
    return om_causal_fwd(q, k, v, scale, out, causal)


def om_causal_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float | None = None,
                  out: torch.Tensor | None = None, causal: bool = True) -> torch.Tensor:
    """Softmax attention ``[B,H,Tq,dk] x [B,H,Tk,dk] x [B,H,Tk,dv]``; with ``causal``
    key j is hidden from query t when j > t.  ``scale`` defaults to ``1/sqrt(dk)``."""
    require_cuda(q, k, v, out)
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise B200Error("om_causal_fwd takes rank-4 q, k, v")
    B, H, Tq, dk = q.shape
    if k.shape[:2] != (B, H) or k.shape[3] != dk or v.shape[:3] != k.shape[:3]:
        raise B200Error("om_causal_fwd: q [B,H,Tq,dk], k [B,H,Tk,dk], v [B,H,Tk,dv]")
    if not (q.dtype == k.dtype == v.dtype):
        raise B200Error("q, k, v must share one dtype")
    Tk, dv = k.shape[2], v.shape[3]
    sc = float(scale) if scale is not None else 1.0 / float(dk) ** 0.5
    if not causal and Tq <= 8 and Tk >= 1024 and dk % 8 == 0 and dv % 4 == 0:
        # a handful of query rows against a long key range, all keys visible: the streaming
        # step's decode kernel (with the causal mask such rows see at most 8 keys)
        res = om_apply_state(om_step_qk(None, q, k, v, sc, False, 0)).to(q.dtype)
        if out is None:
            return res
        out.copy_(res)
        return out
    if out is None:
        out = torch.empty(B, H, Tq, dv, dtype=q.dtype, device=q.device)
    rc = _lib.load().cb2_om_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                                B, H, Tq, Tk, dk, dv, sc, 1 if causal else 0, dtype_code(q.dtype),
                                device_status(q.device).data_ptr(), stream_ptr())
    check(rc, "cb2_om_fwd")
    return out


def attn_bias(mask: torch.Tensor) -> torch.Tensor:
    """An attention mask in additive fp32 form, the reference's ``attnbias`` coercion
    (catopt_carriers/om.py:1036-1050): a floating mask is the bias, a bool keep-mask is
    0 where True and -inf where False."""
    if mask.dtype == torch.bool:
        return torch.zeros(mask.shape, dtype=torch.float32, device=mask.device).masked_fill_(~mask, float("-inf"))
    return mask.float()


def om_bias_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, bias: torch.Tensor, scale: float | None = None,
                out: torch.Tensor | None = None, causal: bool = False) -> torch.Tensor:
    """Softmax attention with an explicit mask: ``softmax(scale * q k^T + bias) v`` —
    the carrier ``om_apply(om_elem(add(scores, attnbias(m)), v))`` of the reference's
    masked sdpa law (om.py:1313-1362).  ``bias`` is fp32 (see :func:`attn_bias` for bool
    masks) and broadcasts to ``[B,H,Tq,Tk]``; broadcast axes are not materialised."""
    require_cuda(q, k, v, out)
    require_device(bias)
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise B200Error("om_bias_fwd takes rank-4 q, k, v")
    B, H, Tq, dk = q.shape
    if k.shape[:2] != (B, H) or k.shape[3] != dk or v.shape[:3] != k.shape[:3]:
        raise B200Error("om_bias_fwd: q [B,H,Tq,dk], k [B,H,Tk,dk], v [B,H,Tk,dv]")
    if not (q.dtype == k.dtype == v.dtype):
        raise B200Error("q, k, v must share one dtype")
    Tk, dv = k.shape[2], v.shape[3]
    b4 = _bias4(bias, B, H, Tq, Tk)
    sc = float(scale) if scale is not None else 1.0 / float(dk) ** 0.5
    if not causal and Tq <= 8 and Tk >= 1024 and dk % 8 == 0 and dv % 4 == 0:
        # a handful of query rows against a long key range: the streaming step's decode kernel
        res = om_apply_state(om_step_qk(None, q, k, v, sc, False, 0, bias=bias)).to(q.dtype)
        if out is None:
            return res
        out.copy_(res)
        return out
    if out is None:
        out = torch.empty(B, H, Tq, dv, dtype=q.dtype, device=q.device)
    rc = _lib.load().cb2_om_bias_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), b4.data_ptr(),
                                     b4.stride(0), b4.stride(1), b4.stride(2), B, H, Tq, Tk, dk, dv, sc,
                                     1 if causal else 0, dtype_code(q.dtype),
                                     device_status(q.device).data_ptr(), stream_ptr())
    check(rc, "cb2_om_bias_fwd")
    return out


def om_empty_state(shape: tuple, dv: int, device: torch.device | str) -> tuple:
    """The identity carrier ``(m, l, a) = (-inf, 0, 0)`` for queries of leading shape
    ``shape = (B, H, Tq)`` (``om_empty_state``, catopt_carriers/om_lower.py:871-893);
    fp32: ``m, l [B,H,Tq,1]``, ``a [B,H,Tq,dv]``."""
    m = torch.full((*shape, 1), float("-inf"), dtype=torch.float32, device=device)
    return m, torch.zeros(*shape, 1, dtype=torch.float32, device=device), \
        torch.zeros(*shape, dv, dtype=torch.float32, device=device)


def _bias4(bias: torch.Tensor, B: int, H: int, Tq: int, Tk: int) -> torch.Tensor:
    """``bias`` (fp32, rank <= 4, broadcastable) as a ``[B,H,Tq,Tk]`` view with contiguous keys; the
    other broadcast axes keep stride 0."""
    if bias.dtype != torch.float32 or bias.dim() > 4:
        raise B200Error("bias must be float32 of rank <= 4")
    bb = bias.reshape(1) if bias.dim() == 0 else bias
    if bb.shape[-1] == 1 and Tk > 1:
        bb = bb.expand(*bb.shape[:-1], Tk)            # one value for every key of a row
    if Tk > 1 and bb.stride(-1) != 1:
        bb = bb.contiguous()                          # the kernel reads a row's keys contiguously
    try:
        b4 = torch.broadcast_to(bb, (B, H, Tq, Tk))
    except RuntimeError as e:
        raise B200Error(f"bias of shape {tuple(bias.shape)} does not broadcast to {(B, H, Tq, Tk)}") from e
    if any(st < 0 for st in b4.stride()):
        raise B200Error("bias with negative strides")
    return b4


def om_step_qk(state: tuple | None, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float = 1.0,
               causal: bool = False, key_offset: int = 0, bias: torch.Tensor | None = None) -> tuple:
    """``state (+) om_elem(scale * q @ k^T, v)``: fold one block of keys/values into
    the running carrier (``om_step_qk``, om_lower.py:911-922; the reference takes
    unscaled, unmasked scores — ``scale`` and the causal mask with its key offset
    are the arguments its carrier terms spell around the product).  ``q [B,H,Tq,dk]``,
    ``k [B,H,Tk,dk]``, ``v [B,H,Tk,dv]``; returns a new fp32 ``(m, l, a)``.
    With ``causal`` key j of this block is hidden from query row t when
    ``key_offset + j > t``: ``key_offset`` = keys folded in before this block minus
    the sequence position of query row 0 (negative in a decode step whose queries
    are the newest positions).  ``bias``: fp32 additive mask over THIS block's keys,
    broadcastable to ``[B,H,Tq,Tk]`` (``cb2_om_bias_step``)."""
    require_cuda(q, k, v)
    require_device(bias)
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise B200Error("om_step_qk takes rank-4 q, k, v")
    B, H, Tq, dk = q.shape
    if k.shape[:2] != (B, H) or k.shape[3] != dk or v.shape[:3] != k.shape[:3] or not (q.dtype == k.dtype == v.dtype):
        raise B200Error("om_step_qk: q [B,H,Tq,dk], k [B,H,Tk,dk], v [B,H,Tk,dv] of one dtype")
    Tk, dv = k.shape[2], v.shape[3]
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    m_out, l_out, a_out = (torch.empty(B, H, Tq, 1, dtype=torch.float32, device=q.device),
                           torch.empty(B, H, Tq, 1, dtype=torch.float32, device=q.device),
                           torch.empty(B, H, Tq, dv, dtype=torch.float32, device=q.device))
    if state is not None:
        m_in, l_in, a_in = (t.to(torch.float32).contiguous() for t in state)
        require_cuda(m_in, l_in, a_in)
        if m_in.shape != m_out.shape or l_in.shape != l_out.shape or a_in.shape != a_out.shape:
            raise B200Error("om_step_qk: state shapes do not match q and v")
        ptrs = (m_in.data_ptr(), l_in.data_ptr(), a_in.data_ptr())
    else:
        ptrs = (None, None, None)
    lib = _lib.load()
    need = lib.cb2_om_step_scratch_bytes(B, H, Tq, Tk, dv)
    scratch = _scratch_buf("om_step", need, q.device)
    if bias is not None:
        b4 = _bias4(bias, B, H, Tq, Tk)
        rc = lib.cb2_om_bias_step(q.data_ptr(), k.data_ptr(), v.data_ptr(), b4.data_ptr(), b4.stride(0), b4.stride(1),
                                  b4.stride(2), *ptrs, m_out.data_ptr(), l_out.data_ptr(), a_out.data_ptr(), B, H,
                                  Tq, Tk, dk, dv, float(scale), 1 if causal else 0, int(key_offset),
                                  dtype_code(q.dtype), _ptr(scratch), need, device_status(q.device).data_ptr(),
                                  stream_ptr())
        check(rc, "cb2_om_bias_step")
        return m_out, l_out, a_out
    rc = lib.cb2_om_step(q.data_ptr(), k.data_ptr(), v.data_ptr(), *ptrs, m_out.data_ptr(),
                         l_out.data_ptr(), a_out.data_ptr(), B, H, Tq, Tk, dk, dv, float(scale),
                         1 if causal else 0, int(key_offset), dtype_code(q.dtype), _ptr(scratch), need,
                         device_status(q.device).data_ptr(), stream_ptr())
    check(rc, "cb2_om_step")
    return m_out, l_out, a_out


def om_apply_state(state: tuple) -> torch.Tensor:
    """The ``om_apply`` readout ``a / l`` (unclamped: a row that saw no key is NaN),
    ``om_apply_state`` (om_lower.py:925-927)."""
    return state[2] / state[1]


# --------------------------------------------------------------------------- scan
def diag_scan_fwd(a: torch.Tensor, x: torch.Tensor, b: torch.Tensor, c: torch.Tensor,
                  h0: torch.Tensor | None = None, want_state: bool = False,
                  out: torch.Tensor | None = None):
    """``h_t = a_t*h_{t-1} + b*x_t``, ``y_t = sum_n c*h_t``.

    ``a`` is ``[B,T,D,N]`` or ``[B,T,D]`` (shared over n); ``x`` ``[B,T,D]``;
    ``b``, ``c`` ``[D,N]``; ``h0`` float32 ``[B,D,N]`` or ``None``.
    Returns ``y`` or ``(y, h_T)`` when ``want_state``.
    """
    require_cuda(a, x, b, c, h0, out)
    if x.dim() != 3 or b.dim() != 2 or b.shape != c.shape:
        raise B200Error("diag_scan_fwd takes x [B,T,D] and b,c [D,N]")
    B, T, D = x.shape
    N = b.shape[1]
    if b.shape[0] != D:
        raise B200Error("b,c must be [D,N]")
    bcast = a.dim() == 3
    if tuple(a.shape) != ((B, T, D) if bcast else (B, T, D, N)):
        raise B200Error(f"a has shape {tuple(a.shape)}; expected [B,T,D,N] or [B,T,D]")
    if not (a.dtype == x.dtype == b.dtype == c.dtype):
        raise B200Error("a, x, b, c must share one dtype")
    if h0 is not None and (h0.dtype != torch.float32 or tuple(h0.shape) != (B, D, N)):
        raise B200Error("h0 must be float32 [B,D,N]")
    y = out if out is not None else torch.empty_like(x)
    status = device_status(x.device)
    lib = _lib.load()
    code = dtype_code(x.dtype)
    n_seg = 1 if bcast else _scan_parallel_segments(B, T, D, N)
    if n_seg > 1:
        # few (batch, channel-block) units: the sequence is cut into segments that run side by
        # side, each from a start state computed up front (one extra pass over a and x)
        starts = torch.empty(B, n_seg, D, N, dtype=torch.float32, device=x.device)
        need = lib.cb2_diag_scan_seg_scratch_bytes(B, D, N, n_seg)
        scratch = _scratch_buf("scan_seg", need, x.device)
        rc = lib.cb2_diag_scan_seg_starts(a.data_ptr(), x.data_ptr(), b.data_ptr(), _ptr(h0), starts.data_ptr(),
                                          B, T, D, N, n_seg, code, _ptr(scratch), need, stream_ptr())
        check(rc, "cb2_diag_scan_seg_starts")
        ends = torch.empty(B, n_seg, D, N, dtype=torch.float32, device=x.device) if want_state else None
        rc = lib.cb2_diag_scan_fwd(a.data_ptr(), x.data_ptr(), b.data_ptr(), c.data_ptr(), starts.data_ptr(),
                                   y.data_ptr(), _ptr(ends), B * n_seg, T // n_seg, D, N, 0, code,
                                   status.data_ptr(), stream_ptr())
        check(rc, "cb2_diag_scan_fwd")
        return (y, ends[:, -1].contiguous()) if want_state else y
    hT = torch.empty(B, D, N, dtype=torch.float32, device=x.device) if want_state else None
    rc = lib.cb2_diag_scan_fwd(a.data_ptr(), x.data_ptr(), b.data_ptr(), c.data_ptr(),
                               _ptr(h0), y.data_ptr(), _ptr(hT), B, T, D, N, int(bcast),
                               code, status.data_ptr(), stream_ptr())
    check(rc, "cb2_diag_scan_fwd")
    return (y, hT) if want_state else y


def _scan_parallel_segments(B: int, T: int, D: int, N: int) -> int:
    """Segments for a scan whose one-pass form (one CTA per batch entry and 32 channels)
    would keep fewer than half of the 148 SMs busy: the largest power of two that brings
    the CTA count to about two per SM, divides T and leaves 256 steps or more per segment;
    1 = one pass.  (Measured, bf16 N=16 T=4096: 32 units 154 -> 72 us, 64 units 154 -> 116 us.)"""
    units = B * ((D + 31) // 32)
    if units * 2 > 148 or N % 4 or T < 1024:
        return 1
    n = 1
    while units * n * 2 <= 296 and T % (n * 2) == 0 and T // (n * 2) >= 256:
        n *= 2
    return n


def diag_compose_apply(a_seq: torch.Tensor, b_seq: torch.Tensor, h: torch.Tensor) -> torch.Tensor | None:
    """Apply the composed diagonal map of ``n`` leaves to ``h``.

    ``a_seq``/``b_seq`` are ``[n, *state]`` in PRODUCT order (latest step first),
    the order the reference's ``fused_diag_levels`` (scan_fused.py:100-120)
    takes; the result is its value ``a_root*h + b_root``.  One pass of
    ``cb2_diag_compose_apply`` over the leaves in stored order (no flip, no copy
    when the stacks already have the full state shape).  Returns ``None`` when
    the kernel cannot take the case (dtype other than float32/bfloat16) so the
    caller can keep its own reduction.
    """
    require_device(a_seq, b_seq, h)
    state_shape = torch.broadcast_shapes(a_seq.shape[1:], b_seq.shape[1:], h.shape)
    n, S = a_seq.shape[0], 1
    for sdim in state_shape:
        S *= sdim
    dt = a_seq.dtype
    if dt not in (torch.float32, torch.bfloat16) or b_seq.dtype != dt or n == 0 or S == 0 or b_seq.shape[0] != n:
        return None
    a = a_seq.expand(n, *state_shape).reshape(n, S).contiguous()
    b = b_seq.expand(n, *state_shape).reshape(n, S).contiguous()
    hh = h.expand(state_shape).to(dt).reshape(S).contiguous()
    out = torch.empty(S, dtype=dt, device=a.device)
    lib = _lib.load()
    code = dtype_code(dt)
    need = lib.cb2_diag_compose_scratch_bytes(n, S, code)
    scratch = _scratch_buf("compose", need, a.device)
    rc = lib.cb2_diag_compose_apply(a.data_ptr(), b.data_ptr(), hh.data_ptr(), out.data_ptr(), n, S, code,
                                    _ptr(scratch), need, stream_ptr())
    check(rc, "cb2_diag_compose_apply")
    return out.reshape(state_shape)


def diag_prefix_maps(a_seq: torch.Tensor, b_seq: torch.Tensor):
    """All prefix maps of a chronological sequence of diagonal affine steps.

    ``a_seq``/``b_seq`` are ``[T, *state]`` (broadcastable against each other);
    step t is ``h -> a_t*h + b_t``.  Returns ``(Pa, Pb)`` with
    ``h_t = Pa[t]*h_0 + Pb[t]``, i.e. ``Pa[t] = a_t ... a_0`` and ``Pb`` the scan
    of the offsets — what the reference's ``BatchedOmdModule._prefix_scan``
    (catopt_carriers/omd_lower.py:771-824) builds from blocked compose steps.
    One pass of ``cb2_diag_prefix_maps``: both operands read once, both maps written
    once (a small state is made up for by cutting the steps into segments: totals
    first, then every segment from its carry-in); an operand shared by every step is
    read in place (step stride 0).  Returns ``None`` when the kernel
    cannot take the case (dtype other than float32/bfloat16, or no steps) so the
    caller keeps its own scan.
    """
    require_device(a_seq, b_seq)      # any layout: broadcast (expanded) operands are welcome
    state_shape = torch.broadcast_shapes(a_seq.shape[1:], b_seq.shape[1:])
    T, S = a_seq.shape[0], 1
    for sdim in state_shape:
        S *= sdim
    dt = a_seq.dtype
    if dt not in (torch.float32, torch.bfloat16) or b_seq.dtype != dt or T == 0 or S == 0 or b_seq.shape[0] != T:
        return None

    def rows(x: torch.Tensor) -> tuple[torch.Tensor, int]:
        x = x.expand(T, *state_shape)
        if T > 1 and x.stride(0) == 0:          # one row shared by every step
            return x[0].reshape(S).contiguous(), 0
        return x.reshape(T, S).contiguous(), S

    a, a_stride = rows(a_seq)
    b, b_stride = rows(b_seq)
    pa = torch.empty(T, *state_shape, dtype=dt, device=a.device)
    pb = torch.empty(T, *state_shape, dtype=dt, device=a.device)
    lib = _lib.load()
    need = lib.cb2_diag_prefix_maps_scratch_bytes(T, S, dtype_code(dt))
    scratch = _scratch_buf("prefix", need, a.device)
    rc = lib.cb2_diag_prefix_maps(a.data_ptr(), b.data_ptr(), pa.data_ptr(), pb.data_ptr(), T, S, a_stride,
                                  b_stride, dtype_code(dt), _ptr(scratch), need, stream_ptr())
    check(rc, "cb2_diag_prefix_maps")
    return pa, pb


def diag_scan_states(a_seq: torch.Tensor, b_seq: torch.Tensor, h: torch.Tensor) -> torch.Tensor | None:
    """Every state of ``h_t = a_t*h_(t-1) + b_t`` from ``h_(-1) = h``.

    ``a_seq``/``b_seq`` are ``[T, *state]`` in time order (broadcastable against each
    other and ``h``; an operand shared by every step is read in place), the result is
    ``[T, *state]`` — the stacked-map form ``applyd(aff_diag(stack affd_a f_t, stack
    affd_b f_t), h)`` that ``gather_applyd_stack`` (catopt_carriers/xcarrier.py:2252-2275)
    offers for an unrolled scan.  One pass of ``cb2_diag_scan_states``.  ``None`` when the
    kernel cannot take the case (dtype other than float32/bfloat16, no steps)."""
    require_device(a_seq, b_seq, h)
    state_shape = torch.broadcast_shapes(a_seq.shape[1:], b_seq.shape[1:], h.shape)
    T, S = a_seq.shape[0], 1
    for sdim in state_shape:
        S *= sdim
    dt = torch.promote_types(torch.promote_types(a_seq.dtype, b_seq.dtype), h.dtype)
    if dt not in (torch.float32, torch.bfloat16) or T == 0 or S == 0 or b_seq.shape[0] != T:
        return None

    def rows(x: torch.Tensor) -> tuple[torch.Tensor, int]:
        x = x.to(dt).expand(T, *state_shape)
        if T > 1 and x.stride(0) == 0:          # one row shared by every step
            return x[0].reshape(S).contiguous(), 0
        return x.reshape(T, S).contiguous(), S

    a, a_stride = rows(a_seq)
    b, b_stride = rows(b_seq)
    hh = h.to(dt).expand(state_shape).reshape(S).contiguous()
    out = torch.empty(T, *state_shape, dtype=dt, device=a.device)
    lib = _lib.load()
    need = lib.cb2_diag_prefix_maps_scratch_bytes(T, S, dtype_code(dt))
    scratch = _scratch_buf("prefix", need, a.device)
    rc = lib.cb2_diag_scan_states(a.data_ptr(), b.data_ptr(), hh.data_ptr(), out.data_ptr(), T, S, a_stride,
                                  b_stride, dtype_code(dt), _ptr(scratch), need, stream_ptr())
    check(rc, "cb2_diag_scan_states")
    return out


def diag_fold_apply(a_rows: torch.Tensor, b_rows: torch.Tensor, h: torch.Tensor) -> torch.Tensor:
    """Fold ``h <- a_t*h + b_t`` over rows in TIME order and return the last state.

    ``a_rows``/``b_rows`` are ``[n, *state]`` or ``[*state]`` (one row shared by every
    step), broadcastable against ``h``'s shape — the sequence form
    ``applyd(aff_diag(a, b), h)`` that the reference's generated scan kernel folds
    along the step axis (catopt_discovery/genkernel.py:1031-1060).  One pass of
    ``cb2_diag_fold_apply``; a row shared by all steps is read through a zero step
    stride instead of being repeated in memory.
    """
    require_device(h, a_rows, b_rows)
    state_shape = tuple(h.shape)
    S = h.numel()
    dt = h.dtype
    n = None
    for r in (a_rows, b_rows):
        if r.dim() == len(state_shape) + 1:
            n = r.shape[0] if n is None else n
            if r.shape[0] != n:
                raise B200Error("diag_fold_apply: a and b disagree on the number of steps")
    if n is None:
        raise B200Error("diag_fold_apply: neither operand carries a step axis")
    if n == 0 or S == 0:
        raise B200Error("diag_fold_apply: empty fold")

    def rows(r: torch.Tensor) -> tuple[torch.Tensor, int]:
        r = r.to(dt)
        if r.dim() == len(state_shape) + 1:
            return r.expand(n, *state_shape).reshape(n, S).contiguous(), S
        return r.expand(state_shape).reshape(S).contiguous(), 0

    a, a_stride = rows(a_rows)
    b, b_stride = rows(b_rows)
    hh = h.reshape(S).contiguous()
    out = torch.empty(S, dtype=dt, device=h.device)
    lib = _lib.load()
    code = dtype_code(dt)
    need = lib.cb2_diag_compose_scratch_bytes(n, S, code)
    scratch = _scratch_buf("compose", need, h.device)
    rc = lib.cb2_diag_fold_apply(a.data_ptr(), b.data_ptr(), hh.data_ptr(), out.data_ptr(), n, S, a_stride,
                                 b_stride, code, _ptr(scratch), need, stream_ptr())
    check(rc, "cb2_diag_fold_apply")
    return out.reshape(state_shape)


# --------------------------------------------------------------------------- gated contraction
def _gate_index_rule(gate_batch: tuple, batch: tuple) -> tuple[int, int] | None:
    """(div, mod) with gate(b) = (b // div) % mod for a gate whose batch dims are each 1
    or full, when its full dims form one contiguous run; ``None`` otherwise."""
    full = [i for i, (gd, bd) in enumerate(zip(gate_batch, batch)) if gd == bd and bd != 1]
    if not full:
        return 1, 1
    if full != list(range(full[0], full[-1] + 1)):
        return None
    if any(gate_batch[i] != 1 for i in range(len(batch)) if i not in full):
        return None
    div = 1
    for bd in batch[full[-1] + 1:]:
        div *= bd
    mod = 1
    for i in full:
        mod *= batch[i]
    return div, mod


def gated_contract(s: torch.Tensor, g: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """``(s * g) @ v`` in one kernel — the ``om_decayed`` element on materialised scores.

    ``s``: ``[..., T, K]`` scores, ``g``: a gate broadcastable to ``s`` (decay mask,
    causal mask, ...), ``v``: ``[..., K, dv]``.  Semantics of the reference's binding
    ``_om_decayed_torch`` (catopt_carriers/om.py:1053-1057): the product is rounded to
    the tensor dtype, the contraction accumulates in fp32.  A gate shared over leading
    batch dims (``[T,K]``, ``[H,T,K]`` under ``[B,H,T,K]``, ``[B,1,T,K]``) is indexed in
    place; other broadcast patterns are expanded first.
    """
    require_device(s, g, v)
    if s.dim() < 2 or v.dim() < 2 or s.shape[-1] != v.shape[-2]:
        raise B200Error(f"gated_contract shape mismatch: s {tuple(s.shape)}, v {tuple(v.shape)}")
    dt = s.dtype
    if v.dtype != dt or g.dtype != dt:
        dt = torch.promote_types(torch.promote_types(s.dtype, g.dtype), v.dtype)
    code = dtype_code(dt)
    T, K, dv = s.shape[-2], s.shape[-1], v.shape[-1]
    gate_tail = torch.broadcast_shapes(g.shape[-2:] if g.dim() >= 2 else g.shape, (T, K))
    if tuple(gate_tail) != (T, K):
        raise B200Error(f"gate {tuple(g.shape)} does not broadcast to the scores {tuple(s.shape)}")
    g_batch_raw = tuple(g.shape[:-2]) if g.dim() >= 2 else ()
    batch = tuple(torch.broadcast_shapes(s.shape[:-2], v.shape[:-2], g_batch_raw))
    nb = 1
    for bd in batch:
        nb *= bd
    out = torch.empty(*batch, T, dv, dtype=dt, device=s.device)
    if nb * T * dv == 0:
        return out
    if K == 0:
        return out.zero_()
    ss = s.to(dt).expand(*batch, T, K).contiguous()
    vv = v.to(dt).expand(*batch, K, dv).contiguous()
    g_batch = (1,) * (len(batch) - len(g_batch_raw)) + g_batch_raw
    rule = _gate_index_rule(g_batch, batch)
    if rule is None:
        gg = g.to(dt).expand(*batch, T, K).contiguous()
        rule, ng = (1, nb), nb
    else:
        gg = g.to(dt).expand(*g_batch_raw, T, K).contiguous()
        ng = rule[1]
    status = device_status(s.device)
    rc = _lib.load().cb2_gated_contract_fwd(ss.data_ptr(), gg.data_ptr(), vv.data_ptr(), out.data_ptr(), nb, ng,
                                            T, K, dv, rule[0], rule[1], code, status.data_ptr(), stream_ptr())
    check(rc, "cb2_gated_contract_fwd")
    return out
