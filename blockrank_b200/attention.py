"""Drop-in registration of the CUDA BlockRank attention into Hugging Face transformers.

Mirrors the reference's operator interface
(src/blockrank/blockrank_std_attention.py:652-665 ``register_blockrank_attention`` and
src/blockrank/blockrank_triton_kernel_attention.py:938-965
``register_triton_blockrank_attention``): one call installs an attention
function and a mask function under a name containing ``blockrank`` (the
reference scripts switch to the block collator on that substring,
scripts/eval_attn.py:36-38).

Differences that matter to callers:
  * the mask function returns compact block spans (``BlockSpans``: an int32
    ``(2, B, M)`` tensor of start and length per block) instead of the
    ``(B,1,M,H,H)`` additive mask of std:264-309; a ``BlockSpans`` passed as
    ``attention_mask`` is used as it is (padding-free layout);
  * K/V heads are shared inside the kernel (no ``repeat_kv`` copy) and the
    output is written directly as ``(B, S, N, D)``;
  * training: under autograd the attention output and the raw last-rows
    logits are differentiable (``brk_attn_bwd`` and two skinny products),
    which is what the auxiliary-loss trainer needs
    (src/blockrank/trainer.py:51-107, src/blockrank/losses.py:37-93); the
    reference's Triton path has no backward at all (triton:759-761).  The
    fused ``blockrank_doc_scores`` output is inference-only.
"""
from __future__ import annotations

import warnings
from typing import Optional

import torch

from . import _lib, ops

ATTN_NAME = "cuda_blockrank"


class BlockSpans(torch.Tensor):
    """int32 (2, B, M) tensor [starts; lengths] that also carries ``max_block_len``, ``max_query_len`` (0 if
    unknown) and ``grid_h`` (the H of the reference's (M, H) grid it was derived from, None for a padding-free
    layout)."""

    @staticmethod
    def make(start: torch.Tensor, length: torch.Tensor, max_block_len: int, grid_h: Optional[int] = None,
             max_query_len: int = 0) -> "BlockSpans":
        t = torch.stack([start.to(torch.int32), length.to(torch.int32)]).contiguous().as_subclass(BlockSpans)
        t.max_block_len = int(max_block_len)
        t.max_query_len = int(max_query_len)
        t.grid_h = grid_h
        return t


def cuda_blockrank_attention_mask(*args, attention_mask: Optional[torch.Tensor] = None, **kwargs):
    """Mask-interface entry.  Accepts both calling conventions of transformers (with or
    without ``cache_position``; everything but ``attention_mask`` is ignored).

    attention_mask: the (B, M, H) bool/0-1 block mask of the block collator
    (src/blockrank/dataset.py:228), or a :class:`BlockSpans` (padding-free layout; build one with
    ``BlockSpans.make(start, length, max_block_len)``).  A plain int32 tensor is always read as a 0/1
    block mask, whatever its shape.
    """
    if attention_mask is None:
        raise ValueError("cuda_blockrank attention needs the (B, M, H) block attention_mask of the block collator")
    if isinstance(attention_mask, BlockSpans):
        return attention_mask
    if attention_mask.dim() != 3:
        raise ValueError(f"expected a (B, M, H) block mask or BlockSpans, got shape {tuple(attention_mask.shape)}")
    start, length = ops.spans_from_mask(attention_mask)
    return BlockSpans.make(start, length, attention_mask.shape[-1], grid_h=attention_mask.shape[-1])


class _AttentionFn(torch.autograd.Function):
    """BlockRank attention with its backward: forward keeps (q, k, v, out, lse), backward is ``brk_attn_bwd``."""

    @staticmethod
    def forward(ctx, q, k, v, start, length, scale, max_block_len, max_query_len, algo):
        out, lse = ops.attention(q, k, v, start, length, scale, max_block_len, return_lse=True, algo=algo,
                                 max_query_len=max_query_len)
        ctx.save_for_backward(q, k, v, out, lse, start, length)
        ctx.scale, ctx.max_block_len = float(scale), int(max_block_len)
        return out

    @staticmethod
    def backward(ctx, d_out):
        q, k, v, out, lse, start, length = ctx.saved_tensors
        dq, dk, dv = ops.attention_bwd(q, k, v, out, d_out.to(out.dtype), lse, start, length, ctx.scale,
                                       ctx.max_block_len)
        return dq, dk, dv, None, None, None, None, None, None


class _RawScoresFn(torch.autograd.Function):
    """Raw logits of the last R slots, (B,N,R,S) = scale * q[:, :, S-R:] k^T + a constant mask addend
    (std:219-233, 256-262), with the gradient autograd gives the reference: the addend is constant, so
    d raw flows to q and k at every position."""

    @staticmethod
    def forward(ctx, q, k, start, length, scale, num_last, grid_h):
        raw = ops.raw_scores(q, k, start, length, scale, num_last, grid_h=grid_h)
        ctx.save_for_backward(q, k)
        ctx.scale = float(scale)
        return raw

    @staticmethod
    def backward(ctx, d_raw):
        q, k = ctx.saved_tensors
        B, N, S, D = q.shape
        Nk, R = k.shape[1], d_raw.shape[2]
        g = (d_raw.float() * ctx.scale).view(B, Nk, N // Nk, R, S)
        q_last = q[:, :, S - R:].float().reshape(B, Nk, N // Nk, R, D)
        dq = torch.zeros(B, N, S, D, dtype=q.dtype, device=q.device)
        dq[:, :, S - R:] = torch.einsum("bkgrs,bksd->bkgrd", g, k.float()).reshape(B, N, R, D).to(q.dtype)
        dk = torch.einsum("bkgrs,bkgrd->bksd", g, q_last).to(k.dtype)
        return dq, dk, None, None, None, None, None


def _wants_scores(module, kwargs) -> bool:
    # same precedence as std:244-254
    layers = kwargs.get("layers_to_return_scores", None)
    if layers is not None:
        idx = getattr(module, "layer_idx", None)
        return idx is not None and idx in layers
    return bool(kwargs.get("return_last_block_attn_scores", False))


def cuda_blockrank_attention_forward(module, query, key, value, attention_mask, scaling: float,
                                     dropout: float = 0.0, **kwargs):
    """Attention-interface entry; same signature and return convention as
    ``eager_blockrank_attention_forward`` (std:96-105).

    query (B,N,S,D), key/value (B,Nk,S,D) -- the strided views HF produces are
    consumed as they are.  Returns ``(attn_output (B,S,N,D), scores_or_None)``.
    At layers selected by ``layers_to_return_scores`` /
    ``return_last_block_attn_scores`` the second value is the raw logits of the
    last ``num_last_queries`` slots, (B,N,R,S), exactly as the reference
    returns them; with ``blockrank_doc_scores=True`` and ``signal_rows``
    (B,R) slot indices it is instead the fused per-document probability mass
    (B,N,R,num_docs).
    """
    if not isinstance(attention_mask, BlockSpans):
        if attention_mask is None:
            raise ValueError("BlockRank attention requires block spans (got attention_mask=None)")
        attention_mask = cuda_blockrank_attention_mask(attention_mask=attention_mask, **kwargs)
    train = torch.is_grad_enabled() and (query.requires_grad or key.requires_grad or value.requires_grad)
    if dropout and getattr(module, "training", False):
        warnings.warn("cuda_blockrank attention ignores attention dropout")
    spans = attention_mask
    start, length = spans[0], spans[1]
    algo = kwargs.get("blockrank_algo", _lib.ALGO_AUTO)
    if train:
        out = _AttentionFn.apply(query, key, value, start, length, scaling, spans.max_block_len,
                                 getattr(spans, "max_query_len", 0), algo)
    else:
        out = ops.attention(query, key, value, start, length, scaling, spans.max_block_len, algo=algo,
                            max_query_len=getattr(spans, "max_query_len", 0))
    scores = None
    if start.shape[-1] > 1 and _wants_scores(module, kwargs):
        if kwargs.get("blockrank_doc_scores", False):
            if train:
                raise NotImplementedError("blockrank_doc_scores=True is inference-only; train on the raw scores "
                                          "(compute_auxiliary_attention_loss differentiates them)")
            rows = kwargs.get("signal_rows")
            if rows is None:
                raise ValueError("blockrank_doc_scores=True needs signal_rows (B, R) slot indices")
            scores, _ = ops.doc_scores(query, key, start, length, rows.to(device=query.device, dtype=torch.int32),
                                       scaling, kwargs.get("temperature", 0.05))
        elif train:
            scores = _RawScoresFn.apply(query, key, start, length, scaling, kwargs.get("num_last_queries", 16),
                                        getattr(spans, "grid_h", None))
        else:
            scores = ops.raw_scores(query, key, start, length, scaling, kwargs.get("num_last_queries", 16),
                                    grid_h=getattr(spans, "grid_h", None))
    return out, scores


def register_cuda_blockrank_attention(name: str = ATTN_NAME) -> str:
    """Install the CUDA attention and its mask function in the transformers registries.

    Idempotent.  Raises ImportError if libblockrank_b200.so has not been built
    (the reference's Triton registration raises the same way when Triton is
    missing, triton:953-957).  Select it with
    ``model.set_attn_implementation(name)`` or ``attn_implementation=name``.
    """
    if "blockrank" not in name:
        raise ValueError("the implementation name must contain 'blockrank'")
    _lib.lib()  # fail now, not at the first forward
    from transformers import AttentionInterface, AttentionMaskInterface
    AttentionInterface.register(name, cuda_blockrank_attention_forward)
    AttentionMaskInterface.register(name, cuda_blockrank_attention_mask)
    return name
