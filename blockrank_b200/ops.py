"""Torch-facing wrappers over the C ABI: tensors in, tensors out, current stream.

PyTorch is used for device memory, streams and the dense projections only; all
BlockRank-specific compute happens in libblockrank_b200.so.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import torch

from . import _lib

_DT = {torch.bfloat16: _lib.BRK_BF16, torch.float32: _lib.BRK_F32}

# kernels launched through this module since import (each C-ABI call adds what it enqueues)
launch_count = 0


def _count(n: int) -> None:
    global launch_count
    launch_count += n


def _dtype_code(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise ValueError(f"blockrank_b200 supports bfloat16 and float32, got {t.dtype}") from None


def _need_cuda(*ts: torch.Tensor) -> None:
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("blockrank_b200 kernels run on CUDA tensors only (there is no CPU path)")


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _view(t: torch.Tensor) -> _lib.View:
    """(B, heads, S, D) tensor (any strides, innermost contiguous) -> brk_view."""
    if t.dim() != 4 or t.stride(-1) != 1:
        raise ValueError("expected a (B, heads, S, D) tensor with contiguous head_dim")
    return _lib.View(t.data_ptr(), t.stride(0), t.stride(1), t.stride(2))


def spans_from_mask(mask_bmh: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """(B, M, H) bool left-padded block mask (collator output) -> int32 (B, M) start, length."""
    _need_cuda(mask_bmh)
    if mask_bmh.dim() != 3:
        raise ValueError("block mask must be (B, M, H)")
    m8 = mask_bmh.contiguous().view(torch.uint8) if mask_bmh.dtype == torch.bool else (mask_bmh != 0).to(torch.uint8).contiguous()
    B, M, H = m8.shape
    start = torch.empty(B, M, dtype=torch.int32, device=m8.device)
    ln = torch.empty(B, M, dtype=torch.int32, device=m8.device)
    with torch.cuda.device(m8.device):
        _lib.check(_lib.lib().brk_spans_from_mask(m8.data_ptr(), B, M, H, start.data_ptr(), ln.data_ptr(),
                                                  _stream(m8)), "brk_spans_from_mask")
    _count(1)
    return start, ln


# One int32 status word per device, zeroed when created.  Every attention call passes it; the kernels set
# it (first event wins) when a bounded wait gives up or the block spans are malformed, and check_status()
# turns it into an exception at the caller's next synchronisation point.
_status_words = {}


def status_word(device) -> torch.Tensor:
    device = torch.device(device)
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _status_words.get(idx)
    if t is None:
        t = _status_words[idx] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
    return t


def check_status(device=None) -> None:
    """Synchronise the current stream of ``device`` and raise if a kernel reported a problem since the last
    check: BlockRankLibraryError (BRK_E_TIMEOUT) after a device-side wait gave up, ValueError (BRK_E_ARG)
    after malformed block spans.  The word is cleared, so the next call starts clean."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    w = status_word(device)
    with torch.cuda.device(w.device):
        _lib.check(_lib.lib().brk_status_poll(w.data_ptr(), torch.cuda.current_stream(w.device).cuda_stream),
                   "brk_status_poll")


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, blk_start: torch.Tensor, blk_len: torch.Tensor,
              scale: float, max_block_len: int, out: Optional[torch.Tensor] = None, return_lse: bool = False,
              algo: int = _lib.ALGO_AUTO, max_query_len: int = 0, lse: Optional[torch.Tensor] = None):
    """BlockRank attention forward.

    q (B,N,S,D), k/v (B,Nk,S,D) views of any stride (head_dim contiguous);
    blk_start/blk_len int32 (B,M) on the device.  Returns out (B,S,N,D)
    [and lse (B,N,S)].  Padding slots of ``out`` are zero.  ``max_query_len``
    (optional) bounds the last block's length and shrinks the scratch of the
    tensor-core path.  Device-side problems (malformed spans, a wait that gave
    up) surface at the next :func:`check_status`.
    """
    _need_cuda(q, k, v, blk_start, blk_len)
    B, N, S, D = q.shape
    Nk = k.shape[1]
    if k.shape != (B, Nk, S, D) or v.shape != k.shape:
        raise ValueError(f"shape mismatch q{tuple(q.shape)} k{tuple(k.shape)} v{tuple(v.shape)}")
    if k.dtype != q.dtype or v.dtype != q.dtype:
        raise ValueError("q, k, v must share a dtype")
    if blk_start.dtype != torch.int32 or blk_len.dtype != torch.int32 or blk_start.shape != blk_len.shape:
        raise ValueError("blk_start / blk_len must be int32 tensors of the same (B, M) shape")
    M = blk_start.shape[-1]
    if out is None:
        out = torch.empty(B, S, N, D, dtype=q.dtype, device=q.device)
    if lse is None and return_lse:
        lse = torch.empty(B, N, S, dtype=torch.float32, device=q.device)
    p = _lib.AttnParams()
    p.dtype, p.algo = _dtype_code(q), algo
    p.B, p.N, p.Nk, p.D, p.S, p.M = B, N, Nk, D, S, M
    p.max_block_len = int(max_block_len)
    p.max_query_len = int(max_query_len)
    p.scale = float(scale)
    p.q, p.k, p.v = _view(q), _view(k), _view(v)
    p.o = _view(out.permute(0, 2, 1, 3))
    p.lse = lse.data_ptr() if lse is not None else None
    bs, bl = blk_start.contiguous(), blk_len.contiguous()
    p.blk_start, p.blk_len = bs.data_ptr(), bl.data_ptr()
    p.status = status_word(q.device).data_ptr()
    L = _lib.lib()
    with torch.cuda.device(q.device):
        nbytes = L.brk_attn_fwd_workspace_bytes(C.byref(p))
        ws = torch.empty(nbytes, dtype=torch.uint8, device=q.device)
        _lib.check(L.brk_attn_fwd(C.byref(p), ws.data_ptr(), nbytes, _stream(q)), "brk_attn_fwd")
    # span check / reset kernel + main kernel [+ merge of the key-chunked query block on the tensor-core path]
    _count(3 if nbytes > 256 else 2)
    return (out, lse) if (return_lse or lse is not None) else out


def attention_bwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor, d_out: torch.Tensor,
                  lse: torch.Tensor, blk_start: torch.Tensor, blk_len: torch.Tensor, scale: float, max_block_len: int):
    """Gradients of :func:`attention` (what autograd derives from the reference's eager / SDPA paths,
    src/blockrank/blockrank_std_attention.py:96-262, 472-650).

    q (B,N,S,D), k/v (B,Nk,S,D) as given to the forward; out / d_out (B,S,N,D); lse (B,N,S) fp32 from the
    forward.  Returns (dq (B,N,S,D), dk, dv (B,Nk,S,D)) in the input dtype; slots outside every block get zeros.
    """
    _need_cuda(q, k, v, out, d_out, lse, blk_start, blk_len)
    B, N, S, D = q.shape
    Nk = k.shape[1]
    if out.shape != (B, S, N, D) or d_out.shape != out.shape:
        raise ValueError(f"out / d_out must be (B,S,N,D) = {(B, S, N, D)}, got {tuple(out.shape)} / {tuple(d_out.shape)}")
    if lse.shape != (B, N, S) or lse.dtype != torch.float32:
        raise ValueError("lse must be the forward's fp32 (B, N, S) tensor")
    if any(t.dtype != q.dtype for t in (k, v, out, d_out)):
        raise ValueError("q, k, v, out, d_out must share a dtype")
    d_out, lse = d_out.contiguous(), lse.contiguous()  # (autograd may hand over expanded or transposed gradients)
    dq = torch.empty(B, S, N, D, dtype=q.dtype, device=q.device).permute(0, 2, 1, 3)
    dk = torch.empty(B, S, Nk, D, dtype=q.dtype, device=q.device).permute(0, 2, 1, 3)
    dv = torch.empty(B, S, Nk, D, dtype=q.dtype, device=q.device).permute(0, 2, 1, 3)
    p = _lib.AttnBwdParams()
    p.dtype = _dtype_code(q)
    p.B, p.N, p.Nk, p.D, p.S, p.M = B, N, Nk, D, S, blk_start.shape[-1]
    p.max_block_len, p.scale = int(max_block_len), float(scale)
    p.q, p.k, p.v = _view(q), _view(k), _view(v)
    p.o, p.d_o = _view(out.permute(0, 2, 1, 3)), _view(d_out.permute(0, 2, 1, 3))
    p.lse = lse.data_ptr()
    bs, bl = blk_start.contiguous(), blk_len.contiguous()
    p.blk_start, p.blk_len = bs.data_ptr(), bl.data_ptr()
    p.dq, p.dk, p.dv = _view(dq), _view(dk), _view(dv)
    L = _lib.lib()
    with torch.cuda.device(q.device):
        nbytes = L.brk_attn_bwd_workspace_bytes(C.byref(p))
        ws = torch.empty(nbytes, dtype=torch.uint8, device=q.device)
        _lib.check(L.brk_attn_bwd(C.byref(p), ws.data_ptr(), nbytes, _stream(q)), "brk_attn_bwd")
    _count(3)  # dq (+ delta), dk/dv accumulation, conversion of the accumulators
    return dq, dk, dv


def _score_params(q, k, blk_start, blk_len, scale, R, temperature=0.05) -> _lib.ScoreParams:
    B, N, S, D = q.shape
    p = _lib.ScoreParams()
    p.dtype = _dtype_code(q)
    p.B, p.N, p.Nk, p.D, p.S, p.M, p.R = B, N, k.shape[1], D, S, blk_start.shape[-1], R
    p.scale, p.temperature = float(scale), float(temperature)
    p.q, p.k = _view(q), _view(k)
    p.blk_start, p.blk_len = blk_start.data_ptr(), blk_len.data_ptr()
    return p


def doc_scores(q: torch.Tensor, k: torch.Tensor, blk_start: torch.Tensor, blk_len: torch.Tensor, rows: torch.Tensor,
               scale: float, temperature: float = 0.05):
    """Fused score epilogue.

    rows: int32 (B, R) slot indices of the signal rows.  Returns
    (doc_mass (B,N,R,num_docs) fp32, logits (B,num_docs) fp32) where logits is
    the mean over heads and rows divided by ``temperature`` -- what the
    reference's compute_auxiliary_attention_loss(return_logits=True) yields.
    """
    _need_cuda(q, k, blk_start, blk_len, rows)
    if rows.dtype != torch.int32 or rows.dim() != 2:
        raise ValueError("rows must be int32 (B, R)")
    B, N, S, D = q.shape
    R = rows.shape[1]
    bs, bl, rows = blk_start.contiguous(), blk_len.contiguous(), rows.contiguous()
    p = _score_params(q, k, bs, bl, scale, R, temperature)
    nd = p.M - 2
    mass = torch.empty(B, N, R, max(nd, 0), dtype=torch.float32, device=q.device)
    logits = torch.empty(B, max(nd, 0), dtype=torch.float32, device=q.device)
    p.rows, p.doc_mass, p.logits = rows.data_ptr(), mass.data_ptr(), logits.data_ptr()
    L = _lib.lib()
    with torch.cuda.device(q.device):
        nbytes = L.brk_doc_scores_workspace_bytes(C.byref(p))
        ws = torch.empty(max(nbytes, 8), dtype=torch.uint8, device=q.device)
        _lib.check(L.brk_doc_scores(C.byref(p), ws.data_ptr(), nbytes, _stream(q)), "brk_doc_scores")
    _count(1)  # per-document partials; the CTA that completes a prompt also writes its masses and logits
    return mass, logits


def raw_scores(q: torch.Tensor, k: torch.Tensor, blk_start: torch.Tensor, blk_len: torch.Tensor, scale: float,
               num_last: int = 16, grid_h: Optional[int] = None) -> torch.Tensor:
    """Reference-compatible second return value: (B, N, R, S) masked logits of the last R slots.

    R = min(num_last, grid_h): on the reference's (M, H) grid the window never reaches past the last
    block's H slots (src/blockrank/blockrank_std_attention.py:256-262); without a grid (padding-free
    layout) R = min(num_last, S)."""
    _need_cuda(q, k, blk_start, blk_len)
    B, N, S, D = q.shape
    R = min(int(num_last), S if grid_h is None else int(grid_h))
    bs, bl = blk_start.contiguous(), blk_len.contiguous()
    p = _score_params(q, k, bs, bl, scale, R)
    out = torch.empty(B, N, R, S, dtype=q.dtype, device=q.device)
    with torch.cuda.device(q.device):
        _lib.check(_lib.lib().brk_raw_scores(C.byref(p), out.data_ptr(), _stream(q)), "brk_raw_scores")
    _count(1)
    return out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, residual: Optional[torch.Tensor] = None,
            out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """RMSNorm over the last dim.  With ``residual`` given: residual += x (in place), norm of the sum."""
    _need_cuda(x, weight, residual)
    if not x.is_contiguous() or (residual is not None and not residual.is_contiguous()):
        raise ValueError("rmsnorm expects contiguous rows")
    hidden = x.shape[-1]
    rows = x.numel() // hidden
    if out is None:
        out = torch.empty_like(x)
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().brk_rmsnorm(_dtype_code(x), x.data_ptr(), residual.data_ptr() if residual is not None else None,
                                          weight.data_ptr(), out.data_ptr(), rows, hidden, float(eps), _stream(x)),
                   "brk_rmsnorm")
    _count(1)
    return out


def rope_(q: Optional[torch.Tensor], k: Optional[torch.Tensor], pos: torch.Tensor, inv_freq: torch.Tensor) -> None:
    """In-place rotate-half RoPE.  q (T, N, D) and/or k (T, Nk, D) may be strided views with
    contiguous (heads, D); either may be None; pos int32 (T,), inv_freq fp32 (D/2,)."""
    ref = q if q is not None else k
    if ref is None:
        return
    _need_cuda(ref, pos, inv_freq)
    T, _, D = ref.shape
    for t in (q, k):
        if t is not None and (t.shape[0] != T or t.shape[2] != D or t.stride(2) != 1 or t.stride(1) != D):
            raise ValueError("rope_ expects (T, heads, D) views with contiguous heads")
    if pos.dtype != torch.int32 or inv_freq.dtype != torch.float32 or pos.numel() != T or not pos.is_contiguous():
        raise ValueError("pos must be contiguous int32 (T,) and inv_freq float32")
    N = q.shape[1] if q is not None else 0
    Nk = k.shape[1] if k is not None else 0
    with torch.cuda.device(ref.device):
        _lib.check(_lib.lib().brk_rope(_dtype_code(ref), q.data_ptr() if q is not None else None,
                                       q.stride(0) if q is not None else 0, N,
                                       k.data_ptr() if k is not None else None, k.stride(0) if k is not None else 0,
                                       Nk, D, pos.data_ptr(), inv_freq.data_ptr(), T, _stream(ref)),
                   "brk_rope")
    _count(1)


def silu_mul(gate_up: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """(rows, 2*I) [gate | up] -> (rows, I) silu(gate) * up."""
    _need_cuda(gate_up)
    if not gate_up.is_contiguous():
        raise ValueError("silu_mul expects a contiguous (rows, 2*I) tensor")
    inter = gate_up.shape[-1] // 2
    rows = gate_up.numel() // (2 * inter)
    if out is None:
        out = torch.empty(*gate_up.shape[:-1], inter, dtype=gate_up.dtype, device=gate_up.device)
    with torch.cuda.device(gate_up.device):
        _lib.check(_lib.lib().brk_silu_mul(_dtype_code(gate_up), gate_up.data_ptr(), out.data_ptr(), rows, inter,
                                           _stream(gate_up)), "brk_silu_mul")
    _count(1)
    return out
