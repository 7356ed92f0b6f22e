"""Op-level timing of the attention kernel and the score epilogue on synthetic tensors.

    python -m blockrank_b200.opbench --docs 100 --prompts 2 --algo tc --iters 20

Geometry per prompt: 64-token instruction + ``docs`` x 160-token documents + 48-token query, 32/8
heads, head_dim 128, bf16, padding-free layout; q, k, v ~ N(0,1)*0.5 from a seed.  The working set
(hundreds of MB) exceeds L2, so no flush is needed between iterations.  Small enough to be captured
under a profiler.  Prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import statistics

import torch

from . import _lib, ops


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--docs", type=int, default=100)
    ap.add_argument("--doc-len", type=int, default=160)
    ap.add_argument("--prompts", type=int, default=2)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--algo", default="tc", choices=["tc", "simt"])
    a = ap.parse_args()
    N, Nk, D = 32, 8, 128
    bl = [64] + [a.doc_len] * a.docs + [48]
    T = sum(bl)
    S = -(-T // 8) * 8
    B = a.prompts
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(2)
    mk = lambda h: (torch.randn(B, S, h, D, generator=g, device=dev) * 0.5).bfloat16().transpose(1, 2)
    q, k, v = mk(N), mk(Nk), mk(Nk)
    ln = torch.tensor([bl] * B, dtype=torch.int32, device=dev)
    start = torch.zeros_like(ln)
    start[:, 1:] = ln.cumsum(1)[:, :-1]
    rows = torch.tensor([[T - 2, T - 1]] * B, dtype=torch.int32, device=dev)
    algo = _lib.ALGO_TC if a.algo == "tc" else _lib.ALGO_SIMT
    out = torch.empty(B, S, N, D, dtype=torch.bfloat16, device=dev)
    scale = D ** -0.5

    def timeit(fn):
        for _ in range(a.warmup):
            fn()
        evs = []
        for _ in range(a.iters):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            evs.append((e0, e1))
        torch.cuda.synchronize()
        return [x.elapsed_time(y) for x, y in evs]

    t_attn = timeit(lambda: ops.attention(q, k, v, start, ln, scale, max(bl), out=out, algo=algo))
    t_score = timeit(lambda: ops.doc_scores(q, k, start, ln, rows, scale))
    tri = lambda x: x * (x + 1) // 2
    I, docs, Q = bl[0], bl[1:-1], bl[-1]
    pairs = tri(I) + sum(L * I + tri(L) for L in docs) + Q * (I + sum(docs)) + tri(Q)
    flops = 4 * D * N * pairs * B
    nbytes = (2 * T * D * (N + 2 * Nk) + 2 * T * D * N) * B
    sbytes = (2 * sum(docs) * Nk * D + 2 * 2 * N * D + 4 * N * 2 * len(docs)) * B
    ms_a, ms_s = statistics.median(t_attn), statistics.median(t_score)
    print(json.dumps({"prompts": B, "tokens_per_prompt": T, "algo": a.algo,
                      "attn_ms_median": ms_a, "attn_ms_min": min(t_attn), "attn_tflops_exact": flops / ms_a / 1e9,
                      "attn_hbm_gbs": nbytes / ms_a / 1e6, "score_ms_median": ms_s, "score_ms_min": min(t_score),
                      "score_hbm_gbs": sbytes / ms_s / 1e6}))


if __name__ == "__main__":
    main()
