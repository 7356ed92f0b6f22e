"""Gradients of the CUDA BlockRank attention against autograd over the CPU oracle.

The reference gets these gradients from autograd over its eager / SDPA attention
(src/blockrank/blockrank_std_attention.py:96-262, 472-650) and uses them in the auxiliary-loss
trainer (src/blockrank/trainer.py:51-107, src/blockrank/losses.py:37-93).  The checker here is
``oracle.attention_dense`` in fp64 with ``requires_grad`` inputs on the host; the CUDA side is
called through the C ABI (``brk_attn_fwd`` with lse, then ``brk_attn_bwd``) and through the
registered attention function under autograd.
"""
import pytest
import torch

from oracle import blockrank_oracle as orc

pytestmark = pytest.mark.gpu


def _mask(block_lens, H):
    """(B, M, H) left-padded block mask from per-prompt lists of block lengths."""
    B, M = len(block_lens), len(block_lens[0])
    m = torch.zeros(B, M, H, dtype=torch.bool)
    for b, lens in enumerate(block_lens):
        for j, n in enumerate(lens):
            if n:
                m[b, j, H - n:] = True
    return m


def _dense_attention(q, k, v, mask, scale):
    """Differentiable fp64 attention over the oracle's pair predicate (``orc.allowed_pairs``, the one
    ``orc.attention_dense`` uses); rows in no block see themselves, so that their softmax stays finite
    under autograd, and their output is zeroed.  Returns (B,S,N,D)."""
    B, N, S, D = q.shape
    g = N // k.shape[1]
    valid = mask.reshape(B, S)
    ok = orc.allowed_pairs(mask) | ((~valid)[:, :, None] & torch.eye(S, dtype=torch.bool)[None])
    kx, vx = k.repeat_interleave(g, dim=1), v.repeat_interleave(g, dim=1)
    s = (torch.matmul(q, kx.transpose(-1, -2)) * scale).masked_fill(~ok[:, None], float("-inf"))
    out = torch.matmul(torch.softmax(s, dim=-1), vx).transpose(1, 2)
    return out * valid[:, :, None, None]


def _oracle_grads(q, k, v, mask, scale, d_out):
    """fp64 autograd through the dense masked attention; d_out (B,S,N,D)."""
    q64, k64, v64 = (t.double().clone().requires_grad_(True) for t in (q, k, v))
    out = _dense_attention(q64, k64, v64, mask, scale)
    (out * d_out.double()).sum().backward()
    return out.detach(), q64.grad, k64.grad, v64.grad


def _run_cuda(q, k, v, mask, scale, d_out, dtype):
    from blockrank_b200 import ops
    dev = torch.device("cuda")
    qc, kc, vc = (t.to(dev, dtype) for t in (q, k, v))
    start, ln = ops.spans_from_mask(mask.to(dev))
    H = mask.shape[-1]
    out, lse = ops.attention(qc, kc, vc, start, ln, scale, H, return_lse=True)
    dq, dk, dv = ops.attention_bwd(qc, kc, vc, out, d_out.to(dev, dtype), lse, start, ln, scale, H)
    ops.check_status()
    return out, dq, dk, dv


CASES = [
    # name, block lengths per prompt, H, N, Nk, D
    ("ragged_gqa4_d64", [[5, 7, 3, 8, 4], [8, 0, 6, 2, 7]], 8, 8, 2, 64),
    ("one_block", [[11]], 16, 4, 4, 64),
    ("two_blocks", [[9, 5], [3, 16]], 16, 4, 2, 128),
    ("long_docs_d128", [[40, 70, 33, 64, 20]], 72, 8, 2, 128),
    ("mha_many_docs", [[4] + [6, 9, 2, 7, 5, 8, 3, 9, 1, 6, 4, 7, 9, 2, 5, 8, 6, 3] + [5]], 12, 2, 2, 64),
]


@pytest.mark.parametrize("name,lens,H,N,Nk,D", CASES, ids=[c[0] for c in CASES])
def test_attention_backward_fp32_vs_oracle_autograd(name, lens, H, N, Nk, D):
    g = torch.Generator().manual_seed(11)
    mask = _mask(lens, H)
    B, M, _ = mask.shape
    S = M * H
    q = torch.randn(B, N, S, D, generator=g) * 0.7
    k = torch.randn(B, Nk, S, D, generator=g) * 0.7
    v = torch.randn(B, Nk, S, D, generator=g)
    d_out = torch.randn(B, S, N, D, generator=g)
    scale = D ** -0.5
    ref_out, rq, rk, rv = _oracle_grads(q, k, v, mask, scale, d_out)
    out, dq, dk, dv = _run_cuda(q, k, v, mask, scale, d_out, torch.float32)
    valid = mask.reshape(B, S)
    assert (out.cpu().double() - ref_out)[valid].abs().max() < 1e-4
    for got, ref, what in ((dq, rq, "dq"), (dk, rk, "dk"), (dv, rv, "dv")):
        err = (got.cpu().double() - ref).abs().max().item()
        assert err < 2e-4 * max(1.0, ref.abs().max().item()), (what, err)
    # slots outside every block: exactly zero gradients
    pad = ~valid
    if pad.any():
        assert dq.cpu().permute(0, 2, 1, 3)[pad].abs().max() == 0
        assert dk.cpu().permute(0, 2, 1, 3)[pad].abs().max() == 0
        assert dv.cpu().permute(0, 2, 1, 3)[pad].abs().max() == 0


BF16_CASES = [
    # name, block lengths per prompt, H, N, Nk, D
    ("tc_forward_gqa4_d128", [[64, 160, 97, 160, 48], [64, 33, 160, 128, 40]], 160, 8, 2, 128),
    # many blocks: the last block's keys and block 0's rows are split across CTAs
    ("many_docs_gqa2_d64", [[64] + [96, 70, 96, 13, 96, 80, 96, 96, 55, 96, 96, 31, 96, 90] + [40]], 96, 4, 2, 64),
    ("one_block_d128", [[150]], 152, 2, 1, 128),
]


@pytest.mark.parametrize("name,lens,H,N,Nk,D", BF16_CASES, ids=[c[0] for c in BF16_CASES])
def test_attention_backward_bf16(name, lens, H, N, Nk, D):
    """bf16: backward on warp-level tensor-core MMA; with head_dim 128 and 4 query heads per KV head the forward
    (and its lse) comes from the tcgen05 kernel."""
    g = torch.Generator().manual_seed(5)
    mask = _mask(lens, H)
    B, M, _ = mask.shape
    S = M * H
    rb = lambda t: t.bfloat16().float()
    q, k = rb(torch.randn(B, N, S, D, generator=g) * 0.6), rb(torch.randn(B, Nk, S, D, generator=g) * 0.6)
    v, d_out = rb(torch.randn(B, Nk, S, D, generator=g)), rb(torch.randn(B, S, N, D, generator=g))
    scale = D ** -0.5
    _, rq, rk, rv = _oracle_grads(q, k, v, mask, scale, d_out)
    _, dq, dk, dv = _run_cuda(q, k, v, mask, scale, d_out, torch.bfloat16)
    for got, ref, what in ((dq, rq, "dq"), (dk, rk, "dk"), (dv, rv, "dv")):
        rel = (got.cpu().double() - ref).norm() / ref.norm()
        assert rel < 1e-2, (what, rel.item())     # bf16 operands and outputs, fp32 accumulation
    pad = ~mask.reshape(B, S)
    if pad.any():
        for t in (dq, dk, dv):
            assert t.float().cpu().permute(0, 2, 1, 3)[pad].abs().max() == 0


def test_registered_function_trains_attention_and_raw_scores():
    """The registered attention function under autograd: gradients of a loss over the attention output and
    the raw last-rows scores (what compute_auxiliary_attention_loss consumes) match fp64 autograd."""
    from blockrank_b200.attention import cuda_blockrank_attention_forward, cuda_blockrank_attention_mask
    g = torch.Generator().manual_seed(3)
    lens = [[6, 9, 4, 10, 7], [10, 2, 8, 5, 9]]
    H, N, Nk, D, R = 10, 4, 2, 64, 10
    mask = _mask(lens, H)
    B, M, _ = mask.shape
    S = M * H
    scale = D ** -0.5
    q, k, v = (torch.randn(B, n, S, D, generator=g) * 0.7 for n in (N, Nk, Nk))
    w_out, w_raw = torch.randn(B, S, N, D, generator=g), torch.randn(B, N, R, S, generator=g)
    valid = mask.reshape(B, S)
    w_out = w_out * valid[:, :, None, None]
    w_raw = w_raw * valid[:, None, None, :]          # padded keys carry the mask constant: keep them out of the loss

    dev = torch.device("cuda")
    qc, kc, vc = (t.to(dev).requires_grad_(True) for t in (q, k, v))
    spans = cuda_blockrank_attention_mask(attention_mask=mask.to(dev))

    class Layer:  # stands in for the attention module HF passes
        layer_idx, training = 0, True

    out, raw = cuda_blockrank_attention_forward(Layer(), qc, kc, vc, spans, scale, layers_to_return_scores=[0],
                                                num_last_queries=R)
    assert raw.shape == (B, N, R, S)
    loss = (out * w_out.to(dev)).sum() + (raw * w_raw.to(dev)).sum()
    loss.backward()

    q64, k64, v64 = (t.double().clone().requires_grad_(True) for t in (q, k, v))
    o64 = _dense_attention(q64, k64, v64, mask, scale)
    raw64 = torch.einsum("bkgrd,bksd->bkgrs", (q64[:, :, S - R:] * scale).reshape(B, Nk, N // Nk, R, D), k64).reshape(B, N, R, S)
    ((o64 * w_out.double()).sum() + (raw64 * w_raw.double()).sum()).backward()
    for got, ref, what in ((qc.grad, q64.grad, "dq"), (kc.grad, k64.grad, "dk"), (vc.grad, v64.grad, "dv")):
        err = (got.cpu().double() - ref).abs().max().item()
        assert err < 2e-4 * max(1.0, ref.abs().max().item()), (what, err)


def test_fused_doc_scores_refuse_autograd():
    from blockrank_b200.attention import cuda_blockrank_attention_forward, cuda_blockrank_attention_mask
    mask = _mask([[4, 5, 6]], 8)
    dev = torch.device("cuda")
    q = torch.randn(1, 2, 24, 64, device=dev, requires_grad=True)
    k, v = torch.randn(1, 2, 24, 64, device=dev), torch.randn(1, 2, 24, 64, device=dev)

    class Layer:
        layer_idx, training = 0, True

    with pytest.raises(NotImplementedError):
        cuda_blockrank_attention_forward(Layer(), q, k, v, cuda_blockrank_attention_mask(attention_mask=mask.to(dev)),
                                         0.125, layers_to_return_scores=[0], blockrank_doc_scores=True,
                                         signal_rows=torch.tensor([[22, 23]]))
