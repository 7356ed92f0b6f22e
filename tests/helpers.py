"""Seeded synthetic inputs shared by the CPU and GPU tests (generated on the CPU so that the
oracle and the kernels see identical bits)."""
import torch


def ragged_mask(B, M, H, lens):
    mask = torch.zeros(B, M, H, dtype=torch.bool)
    for b in range(B):
        for m in range(M):
            if lens[b][m]:
                mask[b, m, H - lens[b][m]:] = True
    return mask


def random_lens(B, M, H, seed, full_prob=0.3, min_len=1):
    g = torch.Generator().manual_seed(seed)
    lens = torch.randint(min_len, H + 1, (B, M), generator=g)
    full = torch.rand(B, M, generator=g) < full_prob
    lens[full] = H
    return lens.tolist()


def qkv(B, N, Nk, S, D, seed, dtype, scale=0.5):
    """HF memory layout [B,S,heads,D] viewed as (B,heads,S,D)."""
    g = torch.Generator().manual_seed(seed)
    q = (torch.randn(B, S, N, D, generator=g) * scale).to(dtype).transpose(1, 2)
    k = (torch.randn(B, S, Nk, D, generator=g) * scale).to(dtype).transpose(1, 2)
    v = (torch.randn(B, S, Nk, D, generator=g) * scale).to(dtype).transpose(1, 2)
    return q, k, v


def to_cuda_view(t):
    """Move a (B,heads,S,D) view to the GPU keeping the [B,S,heads,D] memory layout."""
    return t.transpose(1, 2).contiguous().cuda().transpose(1, 2)


def packed_spans(block_lens):
    """[[I, L1.., Q], ...] -> (start, len) int32 (B, M), S (multiple of 8), max block length."""
    B, M = len(block_lens), len(block_lens[0])
    start = torch.zeros(B, M, dtype=torch.int32)
    ln = torch.tensor(block_lens, dtype=torch.int32)
    start[:, 1:] = ln.cumsum(1)[:, :-1]
    S = int(ln.sum(1).max())
    S = -(-S // 8) * 8
    return start, ln, S, int(ln.max())


def packed_to_padded(block_lens_b, H):
    """index map packed slot -> padded slot for one prompt (left-padded blocks of size H)."""
    idx = []
    for m, n in enumerate(block_lens_b):
        idx.extend(range(m * H + H - n, m * H + H))
    return torch.tensor(idx, dtype=torch.long)
