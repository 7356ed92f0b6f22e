"""Block collators: the metadata producers in front of the attention kernels.

``block_icr_collate_fn`` keeps the reference collator's name, arguments and
output contract (src/blockrank/dataset.py:191-276) so a DataLoader built for the
reference works unchanged.  ``packed_block_collate_fn`` emits the padding-free
layout the kernels also accept: tokens of a prompt are contiguous and blocks are
described by spans only.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

QUERY_POSITION_OFFSET = 16384  # dataset.py:255


def _block_lengths(item) -> List[int]:
    """Per-prompt block lengths with the completion merged into the last prompt block (dataset.py:197-203)."""
    bl = [int(x) for x in item["block_lengths"]]
    if len(bl) < 2:
        raise ValueError("block_lengths must hold at least one prompt block and the completion length")
    merged = bl[:-2] + [bl[-2] + bl[-1]]
    if sum(merged) != int(item["input_ids"].shape[0]):
        raise ValueError("Block lengths do not sum to input_ids length")
    return merged


def block_icr_collate_fn(batch: Sequence[dict], tok, pad_to_multiple_of: Optional[int] = 16,
                         max_block_length: Optional[int] = None, always_max_len: bool = False,
                         permutation_invariant_pos: bool = True) -> Dict[str, torch.Tensor]:
    """Left/right-padded (B, M, H) block grid.

    batch items: ``input_ids`` (T,) long, ``block_lengths`` (M+1,) with the
    completion length last, ``answer_ids``.  ``tok`` supplies ``pad_token_id``
    and ``padding_side``.  Returns ``input_ids``/``position_ids``/``labels``
    (B, M*H), ``attention_mask`` (B, M, H) bool, ``num_blocks``, ``answer_ids``.
    """
    pad_id, side = tok.pad_token_id, tok.padding_side
    B = len(batch)
    lens = [_block_lengths(it) for it in batch]
    M = len(lens[0])
    if any(len(l) != M for l in lens):
        raise ValueError("Number of blocks mismatch")
    longest = max(max(l) for l in lens)
    if always_max_len:
        H = max_block_length or longest
    else:
        H = min(longest, max_block_length or int(1e9))
    if pad_to_multiple_of is not None:
        H = -(-H // pad_to_multiple_of) * pad_to_multiple_of

    ids = torch.full((B, M, H), pad_id, dtype=torch.long)
    labels = torch.full((B, M, H), -100, dtype=torch.long)
    for b, (it, bl) in enumerate(zip(batch, lens)):
        src = it["input_ids"].to(torch.long)
        comp = int(it["block_lengths"][-1])
        off = 0
        for m, n in enumerate(bl):
            keep = min(n, H)  # a long block keeps its first H tokens (dataset.py:216)
            dst = slice(H - keep, H) if side == "left" else slice(0, keep)
            ids[b, m, dst] = src[off:off + keep]
            if m == M - 1:
                # only completion tokens that survive truncation are labelled (dataset.py:231-250)
                n_prompt = n - comp
                first = (H - keep) + n_prompt if side == "left" else min(n_prompt, H)
                lab = ids[b, m].clone()
                lab[:max(first, 0)] = -100
                labels[b, m] = lab
            off += n
    mask = ids != pad_id
    labels[~mask] = -100

    if permutation_invariant_pos:
        pos = mask.long().cumsum(-1)
        pos[:, 1:-1] += pos[:, 0].max(-1).values[:, None, None]
        pos[:, -1] += QUERY_POSITION_OFFSET
        pos = (pos - 1).clamp_min(0)
        pos[~mask] = 0
    else:
        flat = mask.view(B, -1)
        pos = ((flat.long().cumsum(-1) * flat) - 1).clamp_min(0).view(B, M, H)

    answers = torch.nn.utils.rnn.pad_sequence([it["answer_ids"] for it in batch], batch_first=True, padding_value=-1)
    return {"input_ids": ids.view(B, M * H), "position_ids": pos.view(B, M * H), "attention_mask": mask,
            "labels": labels.view(B, M * H), "num_blocks": torch.tensor(M, dtype=torch.long),
            "answer_ids": answers}


def packed_block_collate_fn(batch: Sequence[dict], tok=None, max_block_length: Optional[int] = None,
                            pad_token_id: int = 0) -> Dict[str, torch.Tensor]:
    """Padding-free layout: the tokens of each prompt stay contiguous.

    Same items as ``block_icr_collate_fn``.  Returns ``input_ids`` and
    ``position_ids`` (B, S) with S = longest prompt (only the tail of shorter
    prompts is padding), ``block_spans`` int32 (2, B, M) [start; length],
    ``max_block_len``, ``labels`` (B, S) and ``signal_rows`` int32 (B, 2) (the
    slot before the first completion token and that token).  Positions follow
    the same permutation-invariant scheme (dataset.py:252-257).
    """
    pad_id = tok.pad_token_id if tok is not None else pad_token_id
    B = len(batch)
    lens = [_block_lengths(it) for it in batch]
    M = len(lens[0])
    if any(len(l) != M for l in lens):
        raise ValueError("Number of blocks mismatch")
    cap = max_block_length or int(1e9)
    kept = [[min(n, cap) for n in l] for l in lens]
    S = max(sum(k) for k in kept)
    S = -(-S // 8) * 8  # keeps every row 16-byte aligned for any head layout
    ids = torch.full((B, S), pad_id, dtype=torch.long)
    pos = torch.zeros(B, S, dtype=torch.long)
    labels = torch.full((B, S), -100, dtype=torch.long)
    spans = torch.zeros(2, B, M, dtype=torch.int32)
    rows = torch.zeros(B, 2, dtype=torch.int32)
    for b, (it, bl, kp) in enumerate(zip(batch, lens, kept)):
        src = it["input_ids"].to(torch.long)
        comp = int(it["block_lengths"][-1])
        off_src = off_dst = 0
        instr = kp[0] if M > 1 else 0
        for m, (n, k) in enumerate(zip(bl, kp)):
            ids[b, off_dst:off_dst + k] = src[off_src:off_src + k]
            base = 0 if m == 0 else (QUERY_POSITION_OFFSET if m == M - 1 else instr)
            if M == 1:
                base = QUERY_POSITION_OFFSET  # a single block is both first and last (dataset.py:254-255)
            pos[b, off_dst:off_dst + k] = base + torch.arange(k)
            spans[0, b, m], spans[1, b, m] = off_dst, k
            if m == M - 1:
                first = off_dst + (n - comp)
                # the two signal rows must lie inside the (possibly truncated) query block; the reference
                # asserts the same where it looks for the first labelled token (losses.py:43-48)
                if comp < 1 or first - 1 < off_dst or first >= off_dst + k:
                    raise ValueError(
                        f"item {b}: the completion's first token is not inside the kept query block "
                        f"(block length {n}, kept {k}, completion length {comp}): no signal rows")
                labels[b, first:off_dst + k] = ids[b, first:off_dst + k]
                rows[b, 0], rows[b, 1] = first - 1, first
            off_src += n
            off_dst += k
    return {"input_ids": ids, "position_ids": pos, "block_spans": spans,
            "max_block_len": max(max(k) for k in kept), "labels": labels, "signal_rows": rows,
            "num_blocks": torch.tensor(M, dtype=torch.long)}
