#!/usr/bin/env python
"""Op-level comparison on one GPU: this library's BlockRank attention + score epilogue beside the
reference's own GPU paths, on identical seeded bf16 tensors.

    python opbench.py --config c2|c4 [--impl all|ours|ours_packed|triton_ref|sdpa_ref|eager_ref] [--iters 20]

Configs (per prompt: 64-token instruction + docs x 160 tokens + 48-token query, 32/8 heads,
head_dim 128, bf16, q/k/v ~ N(0,1)*0.5 drawn on the CPU from seed 2):
    c2  4 prompts x 20 documents  (3,312 tokens; padded grid M=22, H=160)
    c4  1 prompt  x 100 documents (16,112 tokens; padded grid M=102, H=160)

Implementations:
    ours         libblockrank_b200 on the reference's left-padded (M, H) grid (same tensors as the reference paths)
    ours_packed  libblockrank_b200 on the padding-free layout (same tokens, pads removed) -- the layout the runner uses
    triton_ref   the reference's Triton kernels, triton_blockrank_attention_forward
                 (src/blockrank/blockrank_triton_kernel_attention.py:798-884)
    sdpa_ref     sdpa_blockrank_attention_forward (src/blockrank/blockrank_std_attention.py:472-650)
    eager_ref    eager_blockrank_attention_forward (std:96-262), the parity oracle, run in bf16 on the GPU

The reference files are loaded unmodified from baseline/_ref (see baseline/install_ref.sh).  For every
implementation: CUDA-event time of the attention call (median, min), element-exact TFLOP/s, and the
largest absolute difference of its output from `ours` on valid rows; for the paths that return raw
scores, the time of the scoring step (reference: raw-score return + compute_auxiliary_attention_loss;
ours: the fused epilogue) and the largest relative difference of the document logits.  The working
set exceeds L2, so no flush is needed between iterations.  One JSON line per implementation.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import traceback

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

N, NK, D = 32, 8, 128
INSTR, DOC_LEN, QUERY = 64, 160, 48
CONFIGS = {"c2": (4, 20), "c4": (1, 100)}


def make_case(prompts, docs):
    """Padded (M, H) grid tensors on the CPU in HF memory layout [B, S, heads, D]."""
    bl = [INSTR] + [DOC_LEN] * docs + [QUERY]
    M, H = len(bl), max(bl)
    S = M * H
    g = torch.Generator().manual_seed(2)
    mk = lambda h: (torch.randn(prompts, S, h, D, generator=g) * 0.5).bfloat16()
    q, k, v = mk(N), mk(NK), mk(NK)
    mask = torch.zeros(prompts, M, H, dtype=torch.bool)
    for m, n in enumerate(bl):
        mask[:, m, H - n:] = True
    return bl, M, H, S, q, k, v, mask


def exact_flops(bl):
    tri = lambda x: x * (x + 1) // 2
    I, docs, Q = bl[0], bl[1:-1], bl[-1]
    pairs = tri(I) + sum(L * I + tri(L) for L in docs) + Q * (I + sum(docs)) + tri(Q)
    return 4 * D * N * pairs


def timeit(fn, iters, warmup=3):
    for _ in range(warmup):
        fn()
    evs = []
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        evs.append((e0, e1))
    torch.cuda.synchronize()
    ts = [a.elapsed_time(b) for a, b in evs]
    return statistics.median(ts), min(ts)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="c4", choices=sorted(CONFIGS))
    ap.add_argument("--impl", default="all")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--prompts", type=int, default=0, help="override the config's prompt count (profiling runs)")
    ap.add_argument("--model", action="store_true",
                    help="model level: a Hugging Face Mistral (7B geometry, layers 0..20, random bf16) run the way "
                         "scripts/eval_attn.py runs it, only the registered attention implementation changes "
                         "(impls: cuda_blockrank, triton_ref, eager_ref, sdpa_ref, runner)")
    ap.add_argument("--backward", action="store_true",
                    help="time forward + backward instead (impls: ours, eager_ref, sdpa_ref; the Triton path has none)")
    a = ap.parse_args()
    from baseline import ref_loader
    from blockrank_b200 import _lib, ops

    prompts, docs = CONFIGS[a.config]
    prompts = a.prompts or prompts
    bl, M, H, S, q_c, k_c, v_c, mask_c = make_case(prompts, docs)
    dev = torch.device("cuda")
    q, k, v = (t.to(dev).transpose(1, 2) for t in (q_c, k_c, v_c))   # (B, heads, S, D) views of [B, S, heads, D]
    mask = mask_c.to(dev)
    valid = mask.reshape(prompts, S)
    scale = D ** -0.5
    flops = exact_flops(bl) * prompts
    labels = torch.full((prompts, S), -100, dtype=torch.long, device=dev)
    labels[:, -1] = 7
    rows = torch.tensor([[S - 2, S - 1]] * prompts, dtype=torch.int32, device=dev)
    impls = ["ours", "ours_packed", "triton_ref", "sdpa_ref", "eager_ref"] if a.impl == "all" else a.impl.split(",")

    start, ln = ops.spans_from_mask(mask)
    base_out = ops.attention(q, k, v, start, ln, scale, H, algo=_lib.ALGO_TC)
    _, base_logits = ops.doc_scores(q, k, start, ln, rows, scale)
    torch.cuda.synchronize()

    def report(name, ms, out=None, logits=None, score_ms=None, note=None):
        line = {"config": a.config, "impl": name, "prompts": prompts, "tokens_per_prompt": sum(bl),
                "attn_ms_median": ms[0], "attn_ms_min": ms[1], "attn_tflops_exact": flops / ms[0] / 1e9}
        if out is not None:
            line["out_max_abs_diff_vs_ours"] = float((out.float() - base_out.float())[valid].abs().max())
        if logits is not None:
            line["logits_max_rel_diff_vs_ours"] = float(((logits.float() - base_logits) / base_logits).abs().max())
            line["top10_equal_ours"] = bool(torch.equal(torch.topk(logits.float(), 10).indices,
                                                        torch.topk(base_logits, 10).indices))
        if score_ms is not None:
            line["score_ms_median"], line["score_ms_min"] = score_ms
        if note:
            line["note"] = note
        print(json.dumps(line), flush=True)

    if a.model:
        return model_bench(a, ops, ref_loader, mask, H, S, prompts, bl)
    if a.backward:
        return backward_bench(a, ops, ref_loader, q, k, v, mask, start, ln, scale, H, S, prompts, bl, flops, valid)

    for name in impls:
        try:
            if name == "ours":
                out = torch.empty(prompts, S, N, D, dtype=torch.bfloat16, device=dev)
                ms = timeit(lambda: ops.attention(q, k, v, start, ln, scale, H, out=out, algo=_lib.ALGO_TC), a.iters)
                sm = timeit(lambda: ops.doc_scores(q, k, start, ln, rows, scale), a.iters)
                report(name, ms, out, base_logits, sm)
            elif name == "ours_packed":
                keep = mask_c.reshape(prompts, S)
                T = int(keep[0].sum())
                Sp = -(-T // 8) * 8
                def pack(t):
                    o = torch.zeros(prompts, Sp, t.shape[2], D, dtype=t.dtype)
                    for b in range(prompts):
                        o[b, :T] = t[b][keep[b]]
                    return o.to(dev).transpose(1, 2)
                qp, kp, vp = pack(q_c), pack(k_c), pack(v_c)
                lnp = torch.tensor([bl] * prompts, dtype=torch.int32, device=dev)
                stp = torch.zeros_like(lnp)
                stp[:, 1:] = lnp.cumsum(1)[:, :-1]
                rp = torch.tensor([[T - 2, T - 1]] * prompts, dtype=torch.int32, device=dev)
                out = torch.empty(prompts, Sp, N, D, dtype=torch.bfloat16, device=dev)
                ms = timeit(lambda: ops.attention(qp, kp, vp, stp, lnp, scale, H, out=out, algo=_lib.ALGO_TC), a.iters)
                sm = timeit(lambda: ops.doc_scores(qp, kp, stp, lnp, rp, scale), a.iters)
                _, lg = ops.doc_scores(qp, kp, stp, lnp, rp, scale)
                full = torch.zeros_like(base_out)
                full[valid] = out[:, :T].reshape(-1, N, D)
                report(name, ms, full, lg, sm)
            else:
                if not ref_loader.available():
                    raise RuntimeError(ref_loader.why_unavailable())
                std, losses = ref_loader.load("std"), ref_loader.load("losses")
                mod = ref_loader.AttnModule(N // NK)
                add = std.eager_blockrank_attention_mask(prompts, None, S, attention_mask=mask, dtype=torch.bfloat16)
                if name == "triton_ref":
                    fwd = ref_loader.load("triton").triton_blockrank_attention_forward
                elif name == "sdpa_ref":
                    fwd = std.sdpa_blockrank_attention_forward
                else:
                    fwd = std.eager_blockrank_attention_forward
                with torch.no_grad():
                    out, _ = fwd(mod, q, k, v, add, scale)
                    ms = timeit(lambda: fwd(mod, q, k, v, add, scale), a.iters)
                    logits = sm = None
                    if name != "sdpa_ref":   # sdpa returns unscaled raw scores (std:537): not the scoring path
                        def scored():
                            _, raw = fwd(mod, q, k, v, add, scale, return_last_block_attn_scores=True)
                            return losses.compute_auxiliary_attention_loss(raw, labels, mask, None, return_logits=True)
                        logits = scored()
                        t_all = timeit(scored, a.iters)
                        sm = (t_all[0] - ms[0], t_all[1] - ms[1])
                report(name, ms, out, logits, sm,
                       note="score time = (attention with raw-score return + loss-function reduction) - attention alone")
        except Exception as e:  # a reference path that does not compile or run here is reported, not retried
            tb = traceback.format_exc().strip().splitlines()
            print(json.dumps({"config": a.config, "impl": name, "unavailable": f"{type(e).__name__}: {e}"[:400],
                              "where": tb[-3:] if len(tb) >= 3 else tb}), flush=True)
            torch.cuda.synchronize()


def model_bench(a, ops, ref_loader, mask, H, S, prompts, bl):
    """The drop-in at model level: one Hugging Face MistralForCausalLM (7B geometry, layers 0..l* = 20, random bf16
    weights) on the GPU, called as scripts/eval_attn.py:135-151 calls it (lm_head patched to identity, raw scores of
    layer l* through ``layers_to_return_scores``, the reference's loss function as the reduction); only
    ``attn_implementation`` changes between the rows.  ``runner`` is this library's lean early-exit runner loaded
    with the same weights."""
    from transformers import MistralConfig, MistralForCausalLM
    from blockrank_b200 import register_cuda_blockrank_attention
    from blockrank_b200.runner import MistralPrefillRanker, RankerConfig
    dev = torch.device("cuda")
    L = 20
    cfg = MistralConfig(vocab_size=32768, hidden_size=4096, intermediate_size=14336, num_hidden_layers=L + 1,
                        num_attention_heads=N, num_key_value_heads=NK, head_dim=D, rope_theta=1e6, rms_norm_eps=1e-5,
                        sliding_window=None, max_position_embeddings=32768)
    torch.manual_seed(0)
    old = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        with torch.device(dev):
            model = MistralForCausalLM(cfg).eval()
    finally:
        torch.set_default_dtype(old)
    ident = lambda self_, hidden_states, *x, **kw: hidden_states
    model.lm_head.forward = ident.__get__(model.lm_head, type(model.lm_head))
    losses = ref_loader.load("losses") if ref_loader.available() else None
    g = torch.Generator().manual_seed(7)
    valid = mask.reshape(prompts, S)
    ids = torch.randint(3, 32768, (prompts, S), generator=g).to(dev) * valid
    pos = ((valid.long().cumsum(1) - 1).clamp_min(0)) * valid       # running index over the valid slots
    labels = torch.full((prompts, S), -100, dtype=torch.long, device=dev)
    labels[:, -1] = 7
    names = {"cuda_blockrank": None, "triton_ref": "triton_blockrank", "eager_ref": "eager_blockrank",
             "sdpa_ref": "sdpa_blockrank"}
    impls = ["cuda_blockrank", "triton_ref", "eager_ref", "runner"] if a.impl == "all" else a.impl.split(",")
    base = None
    for name in impls:
        try:
            if name == "runner":
                rk = MistralPrefillRanker(RankerConfig.mistral_7b(score_layer=L), dev).load_state_dict(model.state_dict())
                start, ln = ops.spans_from_mask(mask)
                rows = torch.tensor([[S - 2, S - 1]] * prompts, dtype=torch.int32, device=dev)
                run = lambda: rk.score(ids, pos, start, ln, H, rows, max_query_len=bl[-1])[0]
            else:
                if losses is None:  # the reduction of the raw scores is the reference's own function
                    raise RuntimeError(ref_loader.why_unavailable())
                impl = register_cuda_blockrank_attention() if name == "cuda_blockrank" else ref_loader.register(names[name])
                model.set_attn_implementation(impl)

                def run():
                    out = model(input_ids=ids, position_ids=pos, attention_mask=mask, output_attentions=True,
                                layers_to_return_scores=[L])
                    return losses.compute_auxiliary_attention_loss(out.attentions[0], labels, mask, None, return_logits=True)
            logits = run().float()
            ms = timeit(run, a.iters, warmup=2)
            line = {"config": a.config, "impl": name, "mode": "model (21 layers, 7B geometry, bf16)", "prompts": prompts,
                    "tokens_per_prompt": sum(bl), "ms_median": ms[0], "ms_min": ms[1],
                    "prompts_per_s": prompts / ms[0] * 1e3}
            if base is None:
                base = logits
            else:
                line["logits_max_rel_diff_vs_first"] = float(((logits - base) / base).abs().max())
                line["top10_equal_first"] = bool(torch.equal(torch.topk(logits, 10).indices, torch.topk(base, 10).indices))
            print(json.dumps(line), flush=True)
        except Exception as e:
            tb = traceback.format_exc().strip().splitlines()
            print(json.dumps({"config": a.config, "impl": name, "mode": "model", "unavailable": f"{type(e).__name__}: {e}"[:400],
                              "where": tb[-3:]}), flush=True)
            torch.cuda.synchronize()


def backward_bench(a, ops, ref_loader, q, k, v, mask, start, ln, scale, H, S, prompts, bl, flops, valid):
    """Forward + backward of the attention op under autograd: this library (tcgen05 forward, CUDA-core backward)
    beside autograd over the reference's eager and SDPA functions, same tensors, gradients compared."""
    from blockrank_b200.attention import _AttentionFn
    from blockrank_b200 import _lib
    g = torch.Generator(device=q.device).manual_seed(4)
    d_out = (torch.randn(prompts, S, N, D, generator=g, device=q.device) * valid[:, :, None, None]).bfloat16()
    impls = ["ours", "eager_ref", "sdpa_ref"] if a.impl == "all" else a.impl.split(",")
    base = None
    for name in impls:
        try:
            qg, kg, vg = (t.detach().clone().requires_grad_(True) for t in (q, k, v))
            if name == "ours":
                run = lambda: _AttentionFn.apply(qg, kg, vg, start, ln, scale, H, 0, _lib.ALGO_AUTO)
            else:
                if not ref_loader.available():
                    raise RuntimeError(ref_loader.why_unavailable())
                std = ref_loader.load("std")
                mod = ref_loader.AttnModule(N // NK)
                add = std.eager_blockrank_attention_mask(prompts, None, S, attention_mask=mask, dtype=torch.bfloat16)
                fwd = std.sdpa_blockrank_attention_forward if name == "sdpa_ref" else std.eager_blockrank_attention_forward
                run = lambda: fwd(mod, qg, kg, vg, add, scale)[0]

            def step():
                for t in (qg, kg, vg):
                    t.grad = None
                run().backward(d_out)

            with torch.enable_grad():
                ms = timeit(step, a.iters)
                step()
            grads = [t.grad.float() for t in (qg, kg, vg)]
            line = {"config": a.config, "impl": name, "mode": "forward+backward", "prompts": prompts,
                    "tokens_per_prompt": sum(bl), "ms_median": ms[0], "ms_min": ms[1],
                    "tflops_exact_fwd_plus_2.5x": 3.5 * flops / ms[0] / 1e9}
            if base is None:
                base = grads
            else:
                vm = valid[:, None, :, None]
                line["grad_rel_diff_vs_first"] = [float(((x - y) * vm).norm() / (y * vm).norm()) for x, y in zip(grads, base)]
            print(json.dumps(line), flush=True)
        except Exception as e:
            tb = traceback.format_exc().strip().splitlines()
            print(json.dumps({"config": a.config, "impl": name, "mode": "forward+backward",
                              "unavailable": f"{type(e).__name__}: {e}"[:400], "where": tb[-3:]}), flush=True)
            torch.cuda.synchronize()


if __name__ == "__main__":
    with torch.no_grad():
        main()
