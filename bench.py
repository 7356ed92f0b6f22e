#!/usr/bin/env python
"""Benchmark of the BlockRank prefill hot path: ranking prompts/sec on the Mistral-7B architecture.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one pass of the early-exit ranker over one batch of synthetic prompts per GPU:
64-token instruction + 100 documents x 160 tokens + 48-token query (16,112 tokens, padding-free
layout), scoring at layer 20, 8 prompts per GPU (64 prompts over 8 GPUs; per-GPU work is fixed,
so scaling is weak).  Token ids are seeded uniform integers, weights are seeded N(0, 0.02) in
bf16: synthetic stand-ins for the ranking lists and checkpoint the reference evaluates on.

`value` times the ranker with its inputs resident in HBM; `e2e` times the public host-tensor API
(pinned host inputs copied in, logits and top-10 copied out, every step).  `--impl reference`
times the reference algorithm's CPU restatement (oracle/) on the host cores on a bounded sample.
Rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "ranking prompts/sec, Mistral-7B arch prefill to attn layer"
INSTR, DOC_LEN, QUERY = 64, 160, 48
SCORE_LAYER = 20


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p["bf16_tflops_sustained"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def block_lengths(n_docs):
    return [INSTR] + [DOC_LEN] * n_docs + [QUERY]


def make_host_batch(n_prompts, n_docs, seed, pin):
    """Packed prompts as the packed collator lays them out (blockrank_b200/collate.py)."""
    bl = block_lengths(n_docs)
    T = sum(bl)
    S = -(-T // 8) * 8
    g = torch.Generator().manual_seed(seed)
    ids = torch.zeros(n_prompts, S, dtype=torch.long)
    ids[:, :T] = torch.randint(3, 32768, (n_prompts, T), generator=g)
    pos = torch.zeros(n_prompts, S, dtype=torch.long)
    spans = torch.zeros(2, n_prompts, len(bl), dtype=torch.int32)
    off = 0
    for m, n in enumerate(bl):
        base = 0 if m == 0 else (16384 if m == len(bl) - 1 else INSTR)
        pos[:, off:off + n] = base + torch.arange(n)
        spans[0, :, m], spans[1, :, m] = off, n
        off += n
    rows = torch.tensor([[T - 2, T - 1]] * n_prompts, dtype=torch.int32)
    batch = {"input_ids": ids, "position_ids": pos, "block_spans": spans, "signal_rows": rows,
             "max_block_len": max(bl)}
    if pin:
        for k, v in batch.items():
            if torch.is_tensor(v):
                batch[k] = v.pin_memory()
    return batch


# ---- work counters -------------------------------------------------------------------------
def attention_work(bl, N=32, Nk=8, D=128):
    """Element-exact FLOPs / bytes of one attention launch over one prompt, plus the FLOPs of the
    tiles the tcgen05 kernel actually issues (128-row tiles of 128/G tokens x G heads, 64-key tiles,
    QK^T N rounded to 16, PV K-steps of 16)."""
    tri = lambda x: x * (x + 1) // 2
    I, docs, Q = bl[0], bl[1:-1], bl[-1]
    pairs = tri(I) + sum(L * I + tri(L) for L in docs) + Q * (I + sum(docs)) + tri(Q)
    T = sum(bl)
    f_exact = 4 * D * N * pairs
    nbytes = 2 * T * D * (N + 2 * Nk) + 2 * T * D * N + 4 * T * N
    G = N // Nk
    tok = 128 // G
    M = len(bl)
    f_tile = 0
    for m, L in enumerate(bl):
        ctx = 0 if m == 0 else (bl[0] if m < M - 1 else sum(bl[:-1]))
        for t0 in range(0, L, tok):
            own = min(L, t0 + tok)
            for rng in (ctx, own):
                for lo in range(0, rng, 64):
                    nk = min(64, rng - lo)
                    f_tile += 2 * 128 * (-(-nk // 16) * 16) * D + 2 * 128 * D * (-(-nk // 16) * 16)
    return f_exact, nbytes, f_tile * Nk


def score_bytes(bl, N=32, Nk=8, D=128, R=2):
    return 2 * sum(bl[1:-1]) * Nk * D + 2 * R * N * D + 4 * N * R * (len(bl) - 2)


# ---- clocks ------------------------------------------------------------------------------------
class ClockSampler:
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.stop, self.th = index, [], threading.Event(), None

    def _run(self):
        while not self.stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                      "-i", str(self.index)], capture_output=True, text=True, timeout=5).stdout
                parts = [x.strip() for x in out.strip().split(",")]
                if len(parts) >= 6:
                    self.rows.append(parts)
            except Exception:
                pass
            self.stop.wait(0.2)

    def __enter__(self):
        self.th = threading.Thread(target=self._run, daemon=True)
        self.th.start()
        return self

    def __exit__(self, *a):
        self.stop.set()
        self.th.join(timeout=6)

    def summary(self):
        sm = [float(r[0]) for r in self.rows if r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


# ---- reference arm / CPU baseline ----------------------------------------------------------------
def cpu_layer_sample(n_docs, threads):
    """One decoder layer + the scoring-layer tail of ONE prompt with the CPU oracle (fp32)."""
    from oracle import blockrank_oracle as orc
    torch.set_num_threads(threads)
    bl = block_lengths(n_docs)
    H = max(bl)
    M = len(bl)
    mask = torch.zeros(1, M, H, dtype=torch.bool)
    for m, n in enumerate(bl):
        mask[0, m, H - n:] = True
    S = M * H
    g = torch.Generator().manual_seed(4)
    hid, inter, N, Nk, D = 4096, 14336, 32, 8, 128
    w = lambda *s: torch.randn(*s, generator=g) * 0.02
    W = {"q": w(N * D, hid), "k": w(Nk * D, hid), "v": w(Nk * D, hid), "o": w(hid, N * D),
         "g": w(inter, hid), "u": w(inter, hid), "d": w(hid, inter), "ln": torch.ones(hid)}
    h = torch.randn(1, S, hid, generator=g)
    pos = torch.zeros(1, S, dtype=torch.long)
    cos, sin = orc.rope_tables(pos, D, 1e6)
    sig = torch.tensor([[S - 2, S - 1]])

    def one_layer():
        x = orc.rms_norm(h, W["ln"], 1e-5)
        q = (x @ W["q"].T).view(1, S, N, D).transpose(1, 2)
        k = (x @ W["k"].T).view(1, S, Nk, D).transpose(1, 2)
        v = (x @ W["v"].T).view(1, S, Nk, D).transpose(1, 2)
        q, k = orc.apply_rope(q, cos, sin), orc.apply_rope(k, cos, sin)
        a = orc.attention_blocked(q, k, v, mask, D ** -0.5)
        h2 = h + a.reshape(1, S, N * D) @ W["o"].T
        x = orc.rms_norm(h2, W["ln"], 1e-5)
        return h2 + (torch.nn.functional.silu(x @ W["g"].T) * (x @ W["u"].T)) @ W["d"].T

    def score_tail():
        x = orc.rms_norm(h, W["ln"], 1e-5)
        q = (x @ W["q"].T).view(1, S, N, D).transpose(1, 2)
        k = (x @ W["k"].T).view(1, S, Nk, D).transpose(1, 2)
        return orc.doc_mass(orc.apply_rope(q, cos, sin), orc.apply_rope(k, cos, sin), mask, D ** -0.5, sig,
                            dtype=torch.float32)

    return one_layer, score_tail


def time_cpu_sample(n_docs, reps=1):
    threads = os.cpu_count() or 1
    one_layer, score_tail = cpu_layer_sample(n_docs, threads)
    with torch.no_grad():
        t0 = time.perf_counter()
        for _ in range(reps):
            one_layer()
        t_layer = (time.perf_counter() - t0) / reps
        t0 = time.perf_counter()
        score_tail()
        t_score = time.perf_counter() - t0
    per_prompt = SCORE_LAYER * t_layer + t_score
    return per_prompt, t_layer, t_score, threads


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    one_layer, score_tail = cpu_layer_sample(args.docs, threads)
    with torch.no_grad():
        for _ in range(args.warmup):
            one_layer()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            one_layer()
        t_layer = (time.perf_counter() - t0) / max(args.steps, 1)
        t0 = time.perf_counter()
        score_tail()
        t_score = time.perf_counter() - t0
    per_prompt = SCORE_LAYER * t_layer + t_score
    v = 1.0 / per_prompt
    sample = (f"each step = 1 full decoder layer (fp32) of 1 prompt of the workload; prompts/s extrapolated as "
              f"1/({SCORE_LAYER} x layer {t_layer:.3f}s + scoring tail {t_score:.3f}s)")
    line = {"impl": "reference", "metric": METRIC, "value": v, "unit": "prompts/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": t_layer * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(args),
            "cpu_baseline": {"value": v, "unit": "prompts/s", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": v, "unit": "prompts/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def workload_config(args):
    return {"workload": f"Mistral-7B arch (32 layers, hidden 4096, 32/8 heads, head_dim 128, MLP 14336, bf16 random init), "
                        f"{args.prompts} prompts per GPU x ({INSTR}-token instruction + {args.docs} docs x {DOC_LEN} + "
                        f"{QUERY}-token query = {sum(block_lengths(args.docs))} tokens), early exit + scoring at layer {SCORE_LAYER}",
            "prompts_per_gpu": args.prompts, "docs_per_prompt": args.docs, "tokens_per_prompt": sum(block_lengths(args.docs)),
            "layout": "padding-free packed blocks", "partition": "by prompt, one bf16 replica per GPU, NCCL gather of scores",
            "l2": "inputs and activations per step exceed L2 (no flush needed)"}


# ---- our arm ------------------------------------------------------------------------------------------
def run_ours(args):
    import torch.distributed as dist
    from blockrank_b200 import _lib, ops
    from blockrank_b200.parallel import gather_scores
    from blockrank_b200.runner import MistralPrefillRanker, RankerConfig

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the hot path has no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    _lib.check(_lib.lib().brk_device_check(), "brk_device_check")

    cfg = RankerConfig.mistral_7b(SCORE_LAYER)
    rk = MistralPrefillRanker(cfg, dev, torch.bfloat16).init_random(seed=3)
    rk.algo = {"auto": _lib.ALGO_AUTO, "simt": _lib.ALGO_SIMT, "tc": _lib.ALGO_TC}[args.algo]
    P = args.prompts
    host = make_host_batch(P, args.docs, seed=4 + rank, pin=True)
    devb = {k: (v.to(dev) if torch.is_tensor(v) else v) for k, v in host.items()}
    micro = min(args.micro, P)
    all_ids = list(range(rank * P, rank * P + P))

    def step_resident():
        outs = []
        for i in range(0, P, micro):
            sl = slice(i, i + micro)
            lg, _ = rk.score(devb["input_ids"][sl], devb["position_ids"][sl], devb["block_spans"][0, sl],
                             devb["block_spans"][1, sl], host["max_block_len"], devb["signal_rows"][sl])
            outs.append(lg)
        scores = torch.cat(outs)
        return gather_scores(scores, all_ids, world * P) if world > 1 else scores

    def step_e2e():
        outs = []
        for i in range(0, P, micro):
            sl = slice(i, i + micro)
            mb = {"input_ids": host["input_ids"][sl], "position_ids": host["position_ids"][sl],
                  "block_spans": host["block_spans"][:, sl], "signal_rows": host["signal_rows"][sl],
                  "max_block_len": host["max_block_len"]}
            outs.append(rk.rank_host(mb))
        return outs

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    for _ in range(args.warmup):
        step_resident()
    barrier()
    launches0 = ops.launch_count
    rk.events = {"attn": [], "score": []}
    with ClockSampler(local) as clk:
        total_ms = timed(step_resident, args.steps)
    launches = ops.launch_count - launches0
    torch.cuda.synchronize()
    attn_ms = [a.elapsed_time(b) for a, b in rk.events["attn"]]
    score_ms = [a.elapsed_time(b) for a, b in rk.events["score"]]
    rk.events = None

    rk.use_graphs = bool(args.graphs)
    for _ in range(min(args.warmup, 3)):
        step_e2e()
    e2e_ms = timed(step_e2e, args.steps)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    pk = peaks()
    bl = block_lengths(args.docs)
    f_exact, a_bytes, f_tile = attention_work(bl)
    attn_avg_s = statistics.mean(attn_ms) / 1e3
    achieved = f_exact * micro / attn_avg_s / 1e12
    live = f_tile * micro / attn_avg_s / 1e12
    sc_avg_s = statistics.mean(score_ms) / 1e3
    value = world * P * args.steps / (total_ms / 1e3)
    e2e = world * P * args.steps / (e2e_ms / 1e3)
    h2d = sum(v.numel() * v.element_size() for v in host.values() if torch.is_tensor(v))
    d2h = P * args.docs * 4 + P * min(10, args.docs) * 8
    line = {
        "metric": METRIC, "value": value, "unit": "prompts/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": workload_config(args),
        "e2e": {"value": e2e, "unit": "prompts/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "roofline": {"bound": "tensor", "kernel": "attn_tc_kernel" if args.algo != "simt" else "attn_simt_kernel",
                     "achieved": achieved, "peak": pk["bf16_tflops_sustained"], "unit": "TFLOP/s",
                     "frac": achieved / pk["bf16_tflops_sustained"],
                     # dram__bytes_read+write of one ncu capture on 2 prompts of this geometry (profiles/),
                     # 471.2 MB per prompt, scaled to the prompts of one launch (traffic grows with prompts)
                     "traffic": 471.2e6 * micro if args.docs == 100 and args.algo != "simt" else None,
                     "peak_source": pk["source"],
                     "flops_exact_per_launch": f_exact * micro, "launch_ms": attn_avg_s * 1e3,
                     "live_tile_tflops": live, "live_tile_frac": live / pk["bf16_tflops_sustained"],
                     "exact_over_tile": f_exact / f_tile,
                     "hbm_gbs": a_bytes * micro / attn_avg_s / 1e9,
                     "hbm_frac": a_bytes * micro / attn_avg_s / 1e9 / pk["hbm_gbs"],
                     "launches_timed": len(attn_ms)},
        "score_epilogue": {"bound": "hbm", "achieved": score_bytes(bl) * micro / sc_avg_s / 1e9, "peak": pk["hbm_gbs"],
                           "unit": "GB/s", "frac": score_bytes(bl) * micro / sc_avg_s / 1e9 / pk["hbm_gbs"],
                           "launch_ms": sc_avg_s * 1e3, "note": "two launches (per-document partials, per-prompt finalize) timed together"},
        "clocks": clk.summary(),
    }
    if world == 1 and not args.no_cpu_baseline:
        per_prompt, t_layer, t_score, threads = time_cpu_sample(args.docs)
        line["cpu_baseline"] = {
            "value": 1.0 / per_prompt, "unit": "prompts/s", "cores": threads, "kind": "port",
            "sample": f"1 decoder layer (fp32) of 1 prompt = {t_layer:.2f}s, scoring tail {t_score:.2f}s; "
                      f"extrapolated to {SCORE_LAYER} layers + tail"}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--prompts", type=int, default=8, help="prompts per GPU per step")
    ap.add_argument("--docs", type=int, default=100)
    ap.add_argument("--micro", type=int, default=4, help="prompts per forward pass")
    ap.add_argument("--algo", default="auto", choices=["auto", "simt", "tc"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--graphs", action="store_true", help="e2e leg replays one captured CUDA graph per forward pass")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        if args.warmup < 3:
            args.warmup = 3
        run_ours(args)


if __name__ == "__main__":
    main()
