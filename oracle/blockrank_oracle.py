"""CPU oracle for the BlockRank prefill hot path.  TEST INFRASTRUCTURE ONLY.

This file restates, in plain torch-on-CPU (fp32/fp64) arithmetic, the algorithm
of the reference's *std* BlockRank path so that the CUDA kernels can be checked
against it.  Nothing in the shipped package imports it: only the tests, the
smoke check and the benchmark's CPU-baseline leg do.

Pinning: the reference has no tests or golden vectors of its own, so this
restatement is pinned against outputs of the reference's own code executed on
seeded inputs (tests/golden/*.npz, produced by tests/golden/make_golden.py,
which imports the reference files by path).  tests/test_oracle_golden.py checks
every function below against those fixtures.

Reference locations restated here (paths inside the reference project):
  * src/blockrank/blockrank_std_attention.py:264-309  additive block mask
  * src/blockrank/blockrank_std_attention.py:96-262   eager three-region forward
  * src/blockrank/losses.py:37-78                     per-document score reduction
  * src/blockrank/dataset.py:205-257                  block grid, left padding, positions
  * scripts/eval_attn.py:121-151                      early exit, top-k

Layout vocabulary: a prompt is a grid of M blocks x H slots (block 0 =
instruction, blocks 1..M-2 = documents, block M-1 = query); every block is
left-padded, so the valid slots of a block are its last ``len`` slots.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import torch

MASK_FRACTION = 0.7  # reference uses 0.7 * finfo(dtype).min as the "masked" addend (std:306)


# ----------------------------------------------------------------------------
# metadata
# ----------------------------------------------------------------------------
def block_spans(mask_bmh: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """(B,M,H) bool left-padded mask -> (start, length) int32 (B,M) in sequence-slot units.

    start[b,m] is the index of the first valid slot of block m inside the
    flattened (M*H) sequence.  Mirrors how the reference's mask (std:297-303)
    marks the last ``len`` slots of each block as valid.
    """
    B, M, H = mask_bmh.shape
    ln = mask_bmh.sum(-1).to(torch.int32)
    start = (torch.arange(M, dtype=torch.int32)[None, :] * H + (H - ln)).to(torch.int32)
    return start, ln


def allowed_pairs(mask_bmh: torch.Tensor) -> torch.Tensor:
    """Dense (B, MH, MH) bool: may query slot i attend key slot j?

    Restates the union of the three regions of std:158-237:
      same block and key position <= query position; or
      query in a document block (0 < m < M-1) and key in block 0; or
      query in the last block and key in any earlier block;
    always requiring both slots to be valid tokens.  For M == 1 only the first
    clause applies; for M == 2 block 1 is the query block.
    """
    B, M, H = mask_bmh.shape
    S = M * H
    blk = torch.arange(S) // H
    pos = torch.arange(S) % H
    qb, kb = blk[:, None], blk[None, :]
    same = (qb == kb) & (pos[None, :] <= pos[:, None])
    doc_to_prefix = (qb > 0) & (qb < M - 1) & (kb == 0)
    last_to_all = (qb == M - 1) & (kb < qb)
    struct = same | doc_to_prefix | last_to_all
    valid = mask_bmh.reshape(B, S)
    return struct[None] & valid[:, :, None] & valid[:, None, :]


def additive_block_mask(mask_bmh: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """(B,M,H) bool -> (B,1,M,H,H) additive mask, std:294-309."""
    B, M, H = mask_bmh.shape
    causal = torch.tril(torch.ones(H, H, dtype=torch.bool))
    ok = mask_bmh.view(B, 1, M, 1, H) & causal
    neg = MASK_FRACTION * torch.finfo(dtype).min
    out = torch.full(ok.shape, neg, dtype=dtype)
    out[ok] = 0
    return out


# ----------------------------------------------------------------------------
# attention forward
# ----------------------------------------------------------------------------
def _expand_kv(x: torch.Tensor, groups: int) -> torch.Tensor:
    # GQA: query head n reads KV head n // groups (what repeat_kv materialises, std:135-136)
    return x.repeat_interleave(groups, dim=1)


def attention_dense(q, k, v, mask_bmh, scaling: float, dtype=torch.float64):
    """Ground-truth attention from the pair predicate, high precision, no rounding points.

    q (B,N,S,D), k/v (B,Nk,S,D) any float dtype -> out (B,S,N,D), lse (B,N,S) natural log.
    Rows that are padding get out = 0 and lse = -inf (the reference leaves
    finite garbage there, std:306; only valid rows are comparable).
    """
    B, N, S, D = q.shape
    g = N // k.shape[1]
    qf, kf, vf = q.to(dtype), _expand_kv(k, g).to(dtype), _expand_kv(v, g).to(dtype)
    ok = allowed_pairs(mask_bmh)[:, None]  # (B,1,S,S)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scaling
    s = s.masked_fill(~ok, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - torch.where(torch.isinf(lse), torch.zeros_like(lse), lse)[..., None])
    p = torch.where(ok, p, torch.zeros_like(p))
    out = torch.matmul(p, vf).transpose(1, 2).contiguous()
    return out, lse


def attention_blocked(q, k, v, mask_bmh, scaling: float, emulate: Optional[torch.dtype] = None):
    """Region-by-region forward with the reference's rounding points.

    Follows std:154-237: queries are pre-multiplied by ``scaling`` and rounded
    to the working dtype; logits are rounded to the working dtype before the
    additive mask; softmax runs in fp32 and is rounded back; PV is rounded to
    the working dtype.  ``emulate=None`` works in fp32 throughout.
    Cost is O(live pairs), so it is usable at the standalone-op size.
    Returns out (B,S,N,D) in the working dtype (pad rows zero).
    """
    wd = emulate or torch.float32
    B, N, S, D = q.shape
    M, H = mask_bmh.shape[1:]
    g = N // k.shape[1]

    def rnd(x):
        return x.to(wd).to(torch.float32)

    Q = rnd(q.to(torch.float32) * scaling) if emulate else q.to(torch.float32) * scaling
    K, V = k.to(torch.float32), v.to(torch.float32)
    start, ln = block_spans(mask_bmh)
    out = torch.zeros(B, S, N, D, dtype=torch.float32)
    for b in range(B):
        s0, l0 = int(start[b, 0]), int(ln[b, 0])
        for m in range(M):
            sm, lm = int(start[b, m]), int(ln[b, m])
            if lm == 0:
                continue
            if m == 0 or M == 1:
                ctx: List[Tuple[int, int]] = []
            elif m < M - 1:
                ctx = [(s0, l0)]
            else:
                ctx = [(int(start[b, j]), int(ln[b, j])) for j in range(M - 1)]
            idx = torch.cat([torch.arange(a, a + n) for a, n in ctx] + [torch.arange(sm, sm + lm)])
            nctx = idx.numel() - lm
            qm = Q[b, :, sm:sm + lm]                                 # (N, lm, D)
            kk = _expand_kv(K[b:b + 1, :, idx], g)[0]                # (N, nk, D)
            vv = _expand_kv(V[b:b + 1, :, idx], g)[0]
            s = rnd(torch.matmul(qm, kk.transpose(-1, -2)))
            causal = torch.ones(lm, idx.numel(), dtype=torch.bool)
            causal[:, nctx:] = torch.tril(torch.ones(lm, lm, dtype=torch.bool))
            s = s.masked_fill(~causal, float("-inf"))
            p = rnd(torch.softmax(s, dim=-1))
            out[b, sm:sm + lm] = rnd(torch.matmul(p, vv)).transpose(0, 1)
    return out.to(wd)


# ----------------------------------------------------------------------------
# scores
# ----------------------------------------------------------------------------
def raw_last_scores(q, k, mask_bmh, scaling: float, num_last: int = 16, dtype=None):
    """Pre-softmax logits of the last ``min(num_last, H)`` slots of the query block.

    (B,N,R,M*H) = (q*scaling) k^T + additive mask, std:219-233 and :256-262.
    The mask addend is the finite 0.7*finfo(dtype).min of std:306, combined as
    min(key-valid, query-valid) for earlier blocks and causal+valid inside the
    query block.
    """
    wd = dtype or q.dtype
    B, N, S, D = q.shape
    M, H = mask_bmh.shape[1:]
    R = min(num_last, H)
    g = N // k.shape[1]
    Ql = (q[:, :, S - R:].to(wd) * scaling).to(wd).to(torch.float32)
    Kf = _expand_kv(k, g).to(torch.float32)
    s = torch.matmul(Ql, Kf.transpose(-1, -2)).to(wd)
    ok = allowed_pairs(mask_bmh)[:, None, S - R:, :]  # (B,1,R,S)
    neg = MASK_FRACTION * torch.finfo(wd).min
    add = torch.where(ok, torch.zeros((), dtype=wd), torch.full((), neg, dtype=wd))
    return s + add


def doc_scores_from_raw(raw, labels, mask_bmh, temperature: float = 0.05):
    """Per-document relevance logits from raw last-block scores, losses.py:37-78.

    Signal rows are (b-1, b) with b the first window index whose label > -100;
    softmax over the document-span columns only; per-document sum; mean over
    heads and the two rows; divide by temperature.  Returns (B, M-2).
    """
    B, M, H = mask_bmh.shape
    _, N, R, MH = raw.shape
    win = labels[:, -R:] > -100
    b_idx = win.int().argmax(-1)
    rows = torch.stack([b_idx - 1, b_idx], dim=-1)
    if not bool((rows >= 0).all()):
        raise ValueError("signal row not found inside the returned window")
    sel = raw.gather(2, rows[:, None, :, None].expand(B, N, 2, MH))
    docs = sel[..., H:MH - H]
    p = torch.softmax(docs, dim=-1)
    p = p.reshape(B, N, 2, M - 2, H)
    return p.mean(dim=(1, 2)).sum(-1) / temperature


def doc_mass(q, k, mask_bmh, scaling: float, rows: torch.Tensor, dtype=torch.float64):
    """Closed form of the same reduction, per head and per signal row.

    rows: (B,R) int64 sequence-slot indices of the signal rows (inside the
    query block).  Returns (B,N,R,M-2): for each row the softmax taken over all
    valid document tokens, summed over each document's span.  The mean over
    (N,R) divided by the temperature equals doc_scores_from_raw.
    """
    B, N, S, D = q.shape
    M, H = mask_bmh.shape[1:]
    g = N // k.shape[1]
    R = rows.shape[1]
    qs = torch.gather(q, 2, rows[:, None, :, None].expand(B, N, R, D)).to(dtype) * scaling
    kf = _expand_kv(k, g).to(dtype)
    s = torch.matmul(qs, kf.transpose(-1, -2))                     # (B,N,R,S)
    valid = mask_bmh.reshape(B, 1, 1, S).clone()
    valid[..., :H] = False
    valid[..., S - H:] = False
    s = s.masked_fill(~valid, float("-inf"))
    p = torch.softmax(s, dim=-1)
    return p.reshape(B, N, R, M, H)[:, :, :, 1:M - 1].sum(-1)


def topk_docs(scores: torch.Tensor, k: int = 10) -> torch.Tensor:
    """eval_attn.py:150-151."""
    return torch.topk(scores, k=min(k, scores.shape[-1]), dim=-1).indices


# ----------------------------------------------------------------------------
# collator (block grid + permutation-invariant positions)
# ----------------------------------------------------------------------------
def collate_blocks(prompts: Sequence[Sequence[Sequence[int]]], pad_id: int,
                   pad_to_multiple_of: int = 16, max_block_length: Optional[int] = None,
                   completion_len: int = 1):
    """prompts[b][m] = token ids of block m (the completion already merged into the last block).

    Restates dataset.py:205-257 for left padding: H = min(longest block,
    max_block_length) rounded up to the multiple; every block keeps its first
    H tokens and is left-padded; positions restart per block (documents offset
    by the instruction's valid length, query block by 16384, pads 0); labels
    are -100 except the last ``completion_len`` tokens of the last block.
    """
    B, M = len(prompts), len(prompts[0])
    longest = max(len(blk) for p in prompts for blk in p)
    H = min(longest, max_block_length or int(1e9))
    if pad_to_multiple_of:
        H = -(-H // pad_to_multiple_of) * pad_to_multiple_of
    ids = torch.full((B, M, H), pad_id, dtype=torch.long)
    mask = torch.zeros(B, M, H, dtype=torch.bool)
    for b, p in enumerate(prompts):
        assert len(p) == M
        for m, blk in enumerate(p):
            t = list(blk)[:H]
            if t:
                ids[b, m, H - len(t):] = torch.tensor(t)
                mask[b, m, H - len(t):] = True
    pos = mask.long().cumsum(-1)
    pos[:, 1:-1] += pos[:, 0].max(-1).values[:, None, None]
    pos[:, -1] += 16384
    pos = (pos - 1).clamp_min(0)
    pos[~mask] = 0
    labels = torch.full((B, M, H), -100, dtype=torch.long)
    if completion_len:
        labels[:, -1, H - completion_len:] = ids[:, -1, H - completion_len:]
    return {"input_ids": ids.view(B, M * H), "position_ids": pos.view(B, M * H),
            "attention_mask": mask, "labels": labels.view(B, M * H)}


# ----------------------------------------------------------------------------
# Mistral-architecture prefill with early exit (model-level oracle)
# ----------------------------------------------------------------------------
def rms_norm(x, w, eps):
    v = x.to(torch.float32)
    return w * (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype)


def rope_tables(position_ids, head_dim: int, theta: float):
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    ang = position_ids[..., None].to(torch.float32) * inv
    ang = torch.cat([ang, ang], dim=-1)
    return ang.cos(), ang.sin()


def apply_rope(x, cos, sin):
    """x (B,heads,S,D); rotate-half convention of the HF Llama/Mistral family."""
    d = x.shape[-1] // 2
    rot = torch.cat([-x[..., d:], x[..., :d]], dim=-1)
    return x * cos[:, None] + rot * sin[:, None]


def mistral_prefill_scores(w: dict, cfg: dict, input_ids, position_ids, mask_bmh, labels,
                           score_layer: int, temperature: float = 0.05, num_last: int = 16):
    """Layers 0..score_layer of a Mistral-style decoder with the BlockRank pattern, fp32 on CPU.

    ``w`` maps HF parameter names (model.embed_tokens.weight,
    model.layers.{i}.self_attn.q_proj.weight, ...) to tensors; ``cfg`` holds
    n_heads, n_kv_heads, head_dim, rope_theta, rms_eps.  Mirrors what
    scripts/eval_attn.py:121-151 computes: the scoring layer's raw last-block
    logits -> losses.py reduction.  Returns (doc logits (B,M-2), raw scores,
    hidden state entering the scoring layer).
    """
    B, S = input_ids.shape
    N, Nk, D = cfg["n_heads"], cfg["n_kv_heads"], cfg["head_dim"]
    scaling = D ** -0.5
    h = w["model.embed_tokens.weight"][input_ids]
    cos, sin = rope_tables(position_ids, D, cfg["rope_theta"])
    raw = None
    h_in = None
    for i in range(score_layer + 1):
        p = f"model.layers.{i}."
        if i == score_layer:
            h_in = h
        x = rms_norm(h, w[p + "input_layernorm.weight"], cfg["rms_eps"])
        q = (x @ w[p + "self_attn.q_proj.weight"].T).view(B, S, N, D).transpose(1, 2)
        k = (x @ w[p + "self_attn.k_proj.weight"].T).view(B, S, Nk, D).transpose(1, 2)
        q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
        if i == score_layer:  # only the logits of this layer are needed (V, o_proj and the MLP are not)
            raw = raw_last_scores(q, k, mask_bmh, scaling, num_last)
            break
        v = (x @ w[p + "self_attn.v_proj.weight"].T).view(B, S, Nk, D).transpose(1, 2)
        a = attention_blocked(q, k, v, mask_bmh, scaling).to(h.dtype)
        h = h + a.reshape(B, S, N * D) @ w[p + "self_attn.o_proj.weight"].T
        x = rms_norm(h, w[p + "post_attention_layernorm.weight"], cfg["rms_eps"])
        gate = torch.nn.functional.silu(x @ w[p + "mlp.gate_proj.weight"].T)
        h = h + (gate * (x @ w[p + "mlp.up_proj.weight"].T)) @ w[p + "mlp.down_proj.weight"].T
    return doc_scores_from_raw(raw, labels, mask_bmh, temperature), raw, h_in


# ----------------------------------------------------------------------------
# work counters used by the benchmark's roofline (element-exact, tile independent)
# ----------------------------------------------------------------------------
def live_pairs(block_lengths: Sequence[int]) -> int:
    """Allowed (query,key) pairs of one prompt with valid block lengths [I, L_1.., Q]."""
    M = len(block_lengths)
    I = block_lengths[0]
    tri = lambda n: n * (n + 1) // 2
    if M == 1:
        return tri(I)
    docs = block_lengths[1:-1]
    Q = block_lengths[-1]
    return tri(I) + sum(L * I + tri(L) for L in docs) + Q * (I + sum(docs)) + tri(Q)
