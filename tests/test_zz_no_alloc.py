"""brk_doc_scores_static: the score epilogue for callers that cannot obtain device memory.

Collected last on purpose (file name), so a run that stops at the first failure has already run
everything else.  The entry point is called through the C ABI and must reproduce brk_doc_scores
exactly (same kernels, only the scratch location differs) on consecutive calls that share the
library's built-in scratch array.
"""
import ctypes as C

import pytest
import torch

from oracle import blockrank_oracle as orc
from tests import helpers as H_

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    from blockrank_b200 import _lib, ops


def _params(q, k, start, ln, rows, mass, logits, scale, temperature=0.05):
    B, N, S, D = q.shape
    p = _lib.ScoreParams()
    p.dtype = _lib.BRK_BF16 if q.dtype == torch.bfloat16 else _lib.BRK_F32
    p.B, p.N, p.Nk, p.D, p.S, p.M, p.R = B, N, k.shape[1], D, S, start.shape[1], rows.shape[1]
    p.scale, p.temperature = scale, temperature
    p.q = _lib.View(q.data_ptr(), q.stride(0), q.stride(1), q.stride(2))
    p.k = _lib.View(k.data_ptr(), k.stride(0), k.stride(1), k.stride(2))
    p.rows, p.blk_start, p.blk_len = rows.data_ptr(), start.data_ptr(), ln.data_ptr()
    p.doc_mass, p.logits = mass.data_ptr(), logits.data_ptr()
    return p


def _case(B, N, Nk, D, M, H, seed, dt):
    lens = H_.random_lens(B, M, H, seed)
    for b in range(B):
        lens[b][-1] = H
    mask = H_.ragged_mask(B, M, H, lens)
    q, k, _ = H_.qkv(B, N, Nk, M * H, D, seed + 50, dt)
    start, ln = ops.spans_from_mask(mask.cuda())
    S = M * H
    rows = torch.tensor([[S - 2, S - 1]] * B, dtype=torch.int32)
    exact = orc.doc_mass(q, k, mask, D ** -0.5, rows.long())   # the oracle's per-head, per-row document masses
    return H_.to_cuda_view(q), H_.to_cuda_view(k), start, ln, rows.cuda(), exact


def test_static_scratch_entry_matches_workspace_entry_twice():
    L = _lib.lib()
    stream = torch.cuda.current_stream().cuda_stream
    # two calls in a row with different problems: the second must not see the first one's leftovers
    for (B, N, Nk, D, M, H, seed, dt) in [(2, 8, 2, 128, 9, 32, 41, torch.bfloat16),
                                          (1, 4, 2, 64, 5, 48, 42, torch.float32)]:
        q, k, start, ln, rows, exact = _case(B, N, Nk, D, M, H, seed, dt)
        ref_mass, ref_logits = ops.doc_scores(q, k, start, ln, rows, D ** -0.5)
        mass = torch.full_like(ref_mass, float("nan"))
        logits = torch.full_like(ref_logits, float("nan"))
        p = _params(q, k, start, ln, rows, mass, logits, D ** -0.5)
        rc = L.brk_doc_scores_static(C.byref(p), stream)
        assert rc == 0, L.brk_last_error()
        torch.cuda.synchronize()
        assert torch.equal(mass, ref_mass)
        assert torch.equal(logits, ref_logits)
        # and directly against the oracle, not only against the library's other entry point
        assert torch.allclose(mass.cpu().double(), exact, rtol=1e-3, atol=1e-6)
        assert torch.allclose(logits.cpu().double(), exact.mean(dim=(1, 2)) / 0.05, rtol=1e-3, atol=1e-6)


def test_static_scratch_entry_rejects_oversized_problem():
    L = _lib.lib()
    q, k, start, ln, rows, _ = _case(1, 4, 2, 64, 5, 48, 43, torch.float32)
    mass = torch.empty(1, 4, 2, 3, device="cuda")
    logits = torch.empty(1, 3, device="cuda")
    p = _params(q, k, start, ln, rows, mass, logits, 0.125)
    p.B = 4096  # 4096 * 4 * 2 * 3 * 8 bytes is fine; make the document count huge instead
    p.B, p.M = 1, 2 + (4 << 20) // (4 * 2 * 8) + 1
    rc = L.brk_doc_scores_static(C.byref(p), torch.cuda.current_stream().cuda_stream)
    assert rc == -3
    msg = L.brk_last_error().decode()
    assert "scratch" in msg and str(4 << 20) in msg
    torch.cuda.synchronize()
