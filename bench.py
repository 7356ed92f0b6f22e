#!/usr/bin/env python
"""Benchmark of the BlockRank prefill hot path: ranking prompts/sec on the Mistral-7B architecture.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config c3|c4|c5]

One step = one pass of the early-exit ranker (layers 0..19 in full, scoring at layer 20, bf16) over one
batch of synthetic prompts per GPU, padding-free layout.  Workloads (per-GPU work is fixed, so scaling
over GPUs is weak; prompts are partitioned by rank and the fp32 scores gathered once per step):
    c4 (default)  8 prompts of 64-token instruction + 100 documents x 160 tokens + 48-token query (16,112 tokens)
    c3            8 prompts of 64 + 20 x 160 + 48 tokens (3,312 tokens)
    c5            2 prompts of 64 + 500 documents of 32..256 tokens (seeded) + 48 (~72k tokens), balanced by token count
Token ids are seeded uniform integers, weights are seeded N(0, 0.02) in bf16: synthetic stand-ins for the
ranking lists and checkpoint the reference evaluates on.

`value` times the ranker with its inputs resident in HBM; `e2e` times the public host-tensor API (pinned host
inputs copied in, logits and top-10 copied out, the same gather of scores, every step).  At N=1 the line also
carries `cpu_baseline` -- the reference's own eager BlockRank attention, mask builder and score reduction, run
unmodified inside a Hugging Face Mistral decoder layer on the host cores on a bounded sample -- and `parity`,
which compares that CPU run with the GPU path on the same prompt.  `--impl reference` times the same CPU path
alone.  Rank 0 prints one JSON line.
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
QUERY_POS = 16384  # position of the query block's first token (src/blockrank/dataset.py:252-257)
CONFIGS = {
    "c3": {"prompts": 8, "micro": 8, "docs": 20, "ragged": None},
    "c4": {"prompts": 8, "micro": 4, "docs": 100, "ragged": None},
    "c5": {"prompts": 2, "micro": 1, "docs": 500, "ragged": (32, 256)},
}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p["bf16_tflops_sustained"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def block_lengths(cfg, prompt_index):
    """Block lengths [instruction, documents..., query] of global prompt number ``prompt_index``."""
    if cfg["ragged"] is None:
        return [INSTR] + [DOC_LEN] * cfg["docs"] + [QUERY]
    lo, hi = cfg["ragged"]
    g = torch.Generator().manual_seed(5 + 1000 * prompt_index)
    return [INSTR] + torch.randint(lo, hi + 1, (cfg["docs"],), generator=g).tolist() + [QUERY]


def make_host_batch(bls, seed, pin):
    """Packed prompts as the packed collator lays them out (blockrank_b200/collate.py)."""
    n = len(bls)
    S = -(-max(sum(bl) for bl in bls) // 8) * 8
    M = len(bls[0])
    g = torch.Generator().manual_seed(seed)
    ids = torch.zeros(n, S, dtype=torch.long)
    pos = torch.zeros(n, S, dtype=torch.long)
    spans = torch.zeros(2, n, M, dtype=torch.int32)
    rows = torch.zeros(n, 2, dtype=torch.int32)
    for b, bl in enumerate(bls):
        T = sum(bl)
        ids[b, :T] = torch.randint(3, 32768, (T,), generator=g)
        off = 0
        for m, ln in enumerate(bl):
            base = 0 if m == 0 else (QUERY_POS if m == M - 1 else bl[0])
            pos[b, off:off + ln] = base + torch.arange(ln)
            spans[0, b, m], spans[1, b, m] = off, ln
            off += ln
        rows[b, 0], rows[b, 1] = T - 2, T - 1
    batch = {"input_ids": ids, "position_ids": pos, "block_spans": spans, "signal_rows": rows,
             "max_block_len": max(max(bl) for bl in bls)}
    if pin:
        for k, v in batch.items():
            if torch.is_tensor(v):
                batch[k] = v.pin_memory()
    return batch


# ---- work counters -------------------------------------------------------------------------
def attention_work(bl, S, N=32, Nk=8, D=128):
    """Element-exact FLOPs / bytes of one attention launch over one prompt, plus the FLOPs of the tiles the
    tcgen05 kernel issues: 128-row tiles (128/G tokens x G heads) against 64-key slots paired into 128-key MMA
    tiles; every tile of a row tile but its last is issued at 128 keys, the last at its key count rounded up
    to 16; the query block's context is cut into ceil(S/1024) chunks and tiles pair up inside a chunk."""
    tri = lambda x: x * (x + 1) // 2
    I, docs, Q = bl[0], bl[1:-1], bl[-1]
    pairs = tri(I) + sum(L * I + tri(L) for L in docs) + Q * (I + sum(docs)) + tri(Q)
    T = sum(bl)
    f_exact = 4 * D * N * pairs
    nbytes = 2 * T * D * (N + 2 * Nk) + 2 * T * D * N + 4 * T * N
    tok = 128 // (N // Nk)
    M = len(bl)
    up = lambda x, q: -(-x // q) * q

    def issued(slot_keys):          # key counts of the slots one MMA sequence walks -> keys issued
        tiles = [slot_keys[i:i + 2] for i in range(0, len(slot_keys), 2)]
        return sum(128 for _ in tiles[:-1]) + (len(tiles[-1]) - 1) * 64 + up(tiles[-1][-1], 16) if tiles else 0

    def slots(n):                   # n keys -> key counts of its 64-key slots
        return [min(64, n - lo) for lo in range(0, n, 64)]

    keys = 0
    for m, L in enumerate(bl):
        last = m == M - 1 and M > 1
        ctx = 0 if m == 0 else (I if not last else sum(bl[:-1]))
        for t0 in range(0, L, tok):
            own = slots(min(L, t0 + tok))
            if not last:
                keys += issued(slots(ctx) + own)
                continue
            cs = slots(ctx)
            ns = max(1, min(32, -(-S // 1024)))
            per = -(-len(cs) // ns)
            for c in range(ns):
                part = cs[c * per:(c + 1) * per] + (own if c == ns - 1 else [])
                keys += issued(part)
    f_tile = 4 * 128 * D * keys * Nk
    return f_exact, nbytes, f_tile


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
class ReferenceLayer:
    """One Hugging Face Mistral decoder layer (7B geometry, fp32, host cores) with the reference's own eager
    BlockRank attention and mask builder registered, called the way scripts/eval_attn.py calls the model:
    lm_head patched to identity, raw scores of the layer requested through ``layers_to_return_scores``, reduced
    by the reference's compute_auxiliary_attention_loss(return_logits=True).  The reference files are loaded
    unmodified from baseline/_ref."""

    kind = "reference"

    def __init__(self, threads):
        from baseline import ref_loader
        from transformers import MistralConfig, MistralForCausalLM
        torch.set_num_threads(threads)
        self.losses = ref_loader.load("losses")
        name = ref_loader.register("eager_blockrank")
        cfg = MistralConfig(vocab_size=8, hidden_size=4096, intermediate_size=14336, num_hidden_layers=1,
                            num_attention_heads=32, num_key_value_heads=8, head_dim=128, rope_theta=1e6,
                            rms_norm_eps=1e-5, sliding_window=None, max_position_embeddings=32768,
                            attn_implementation=name)
        torch.manual_seed(3)
        self.model = MistralForCausalLM(cfg).eval()          # HF default init: N(0, 0.02), norms 1
        ident = lambda self_, hidden_states, *a, **kw: hidden_states
        self.model.lm_head.forward = ident.__get__(self.model.lm_head, type(self.model.lm_head))
        self.layer = self.model.model.layers[0]
        self.grabbed = {}
        self.layer.register_forward_hook(lambda mod, args, out: self.grabbed.__setitem__(
            "h", (out[0] if isinstance(out, tuple) else out).detach()))

    def load(self, tensors):
        """tensors: dict of HF names relative to the layer (self_attn.q_proj.weight, ...) -> fp32 host tensors."""
        sd = self.layer.state_dict()
        for k, v in tensors.items():
            sd[k].copy_(v)

    @torch.no_grad()
    def layer_pass(self, h, pos, mask):
        """h (1, M*H, hidden) fp32, pos (1, M*H), mask (1, M, H) bool -> the layer's output hidden states."""
        self.model(inputs_embeds=h, position_ids=pos, attention_mask=mask)
        return self.grabbed["h"]

    @torch.no_grad()
    def scored_pass(self, h, pos, mask, labels):
        out = self.model(inputs_embeds=h, position_ids=pos, attention_mask=mask, output_attentions=True,
                         layers_to_return_scores=[0])
        return self.losses.compute_auxiliary_attention_loss(out.attentions[0], labels, mask, None, return_logits=True)


class PortLayer:
    """Fallback when baseline/_ref is missing: the same layer restated with the CPU oracle (oracle/)."""

    kind = "port"

    def __init__(self, threads):
        from oracle import blockrank_oracle as orc
        torch.set_num_threads(threads)
        self.orc = orc
        g = torch.Generator().manual_seed(3)
        hid, inter, qd, kd = 4096, 14336, 4096, 1024
        w = lambda *s: torch.randn(*s, generator=g) * 0.02
        self.w = {"self_attn.q_proj.weight": w(qd, hid), "self_attn.k_proj.weight": w(kd, hid),
                  "self_attn.v_proj.weight": w(kd, hid), "self_attn.o_proj.weight": w(hid, qd),
                  "mlp.gate_proj.weight": w(inter, hid), "mlp.up_proj.weight": w(inter, hid),
                  "mlp.down_proj.weight": w(hid, inter), "input_layernorm.weight": torch.ones(hid),
                  "post_attention_layernorm.weight": torch.ones(hid)}

    def load(self, tensors):
        for k, v in tensors.items():
            self.w[k] = v.clone()

    def _qk(self, h, pos):
        o, w = self.orc, self.w
        S = h.shape[1]
        x = o.rms_norm(h, w["input_layernorm.weight"], 1e-5)
        cos, sin = o.rope_tables(pos, 128, 1e6)
        q = o.apply_rope((x @ w["self_attn.q_proj.weight"].T).view(1, S, 32, 128).transpose(1, 2), cos, sin)
        k = o.apply_rope((x @ w["self_attn.k_proj.weight"].T).view(1, S, 8, 128).transpose(1, 2), cos, sin)
        return x, q, k

    @torch.no_grad()
    def layer_pass(self, h, pos, mask):
        o, w = self.orc, self.w
        S = h.shape[1]
        x, q, k = self._qk(h, pos)
        v = (x @ w["self_attn.v_proj.weight"].T).view(1, S, 8, 128).transpose(1, 2)
        a = o.attention_blocked(q, k, v, mask, 128 ** -0.5)
        h = h + a.reshape(1, S, 4096) @ w["self_attn.o_proj.weight"].T
        x = o.rms_norm(h, w["post_attention_layernorm.weight"], 1e-5)
        return h + (torch.nn.functional.silu(x @ w["mlp.gate_proj.weight"].T) * (x @ w["mlp.up_proj.weight"].T)) @ \
            w["mlp.down_proj.weight"].T

    @torch.no_grad()
    def scored_pass(self, h, pos, mask, labels):
        self.layer_pass(h, pos, mask)  # the reference runs the scoring layer in full (scripts/eval_attn.py:121-130)
        _, q, k = self._qk(h, pos)
        return self.orc.doc_scores_from_raw(self.orc.raw_last_scores(q, k, mask, 128 ** -0.5), labels, mask)


def make_cpu_layer(threads):
    from baseline import ref_loader
    return ReferenceLayer(threads) if ref_loader.available() else PortLayer(threads)


def padded_grid(bl, pos_packed=None):
    """The reference's left-padded (M, H) grid of one prompt: mask (1, M, H), packed->padded slot index, positions, labels."""
    M, H = len(bl), -(-max(bl) // 16) * 16
    mask = torch.zeros(1, M, H, dtype=torch.bool)
    idx = []
    for m, n in enumerate(bl):
        mask[0, m, H - n:] = True
        idx.extend(range(m * H + H - n, m * H + H))
    idx = torch.tensor(idx, dtype=torch.long)
    pos = torch.zeros(1, M * H, dtype=torch.long)
    if pos_packed is None:
        off = 0
        pk = torch.zeros(sum(bl), dtype=torch.long)
        for m, n in enumerate(bl):
            base = 0 if m == 0 else (QUERY_POS if m == M - 1 else bl[0])
            pk[off:off + n] = base + torch.arange(n)
            off += n
        pos_packed = pk
    pos[0, idx] = pos_packed
    labels = torch.full((1, M * H), -100, dtype=torch.long)
    labels[0, -1] = 7
    return mask, idx, pos, labels


def workload_config(args, cfg, bl0):
    ragged = cfg["ragged"] is not None
    docs = f"{cfg['docs']} docs of {cfg['ragged'][0]}..{cfg['ragged'][1]} tokens (seeded)" if ragged else f"{cfg['docs']} docs x {DOC_LEN}"
    return {"workload": f"{args.config}: Mistral-7B arch (32 layers, hidden 4096, 32/8 heads, head_dim 128, MLP 14336, bf16 random "
                        f"init), {args.prompts} prompts per GPU x ({INSTR}-token instruction + {docs} + {QUERY}-token query"
                        f"{'' if ragged else ' = ' + str(sum(bl0)) + ' tokens'}), early exit + scoring at layer {SCORE_LAYER}",
            "config": args.config, "prompts_per_gpu": args.prompts, "docs_per_prompt": cfg["docs"],
            "tokens_per_prompt": sum(bl0) if not ragged else None, "prompts_per_forward": args.micro,
            "layout": "padding-free packed blocks",
            "partition": "by prompt" + (" (balanced by token count)" if ragged else "") +
                         ", one bf16 replica per GPU, NCCL gather of scores",
            "l2": "inputs and activations per step exceed L2 (no flush needed)"}


def run_reference(args, cfg):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    cpu = make_cpu_layer(threads)
    bl = block_lengths(cfg, 0)
    mask, idx, pos, labels = padded_grid(bl)
    g = torch.Generator().manual_seed(4)
    h = torch.randn(1, mask.shape[1] * mask.shape[2], 4096, generator=g) * 0.02
    for _ in range(args.warmup):
        cpu.layer_pass(h, pos, mask)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu.layer_pass(h, pos, mask)
    t_layer = (time.perf_counter() - t0) / max(args.steps, 1)
    t0 = time.perf_counter()
    cpu.scored_pass(h, pos, mask, labels)
    t_score = time.perf_counter() - t0
    per_prompt = SCORE_LAYER * t_layer + t_score
    v = 1.0 / per_prompt
    sample = (f"each step = 1 decoder layer (fp32, HF Mistral layer + the reference's eager BlockRank attention) of 1 prompt on "
              f"the reference's padded grid; prompts/s extrapolated as 1/({SCORE_LAYER} x layer {t_layer:.3f}s + scoring "
              f"layer with raw scores and score reduction {t_score:.3f}s)")
    line = {"impl": "reference", "metric": METRIC, "value": v, "unit": "prompts/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": t_layer * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(args, cfg, bl),
            "cpu_baseline": {"value": v, "unit": "prompts/s", "cores": threads, "kind": cpu.kind, "sample": sample},
            "e2e": {"value": v, "unit": "prompts/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ---- our arm ------------------------------------------------------------------------------------------
def layer_tensors(rk, i):
    """The runner's fused weights of layer i under the HF names of one decoder layer, fp32 on the host."""
    c = rk.cfg
    qd, kd, inter = c.num_attention_heads * c.head_dim, c.num_key_value_heads * c.head_dim, c.intermediate_size
    L = rk.layers[i]
    f = lambda t: t.float().cpu()
    out = {"input_layernorm.weight": f(L["ln1"])}
    if "wqkv" in L:
        out.update({"self_attn.q_proj.weight": f(L["wqkv"][:qd]), "self_attn.k_proj.weight": f(L["wqkv"][qd:qd + kd]),
                    "self_attn.v_proj.weight": f(L["wqkv"][qd + kd:]), "self_attn.o_proj.weight": f(L["wo"]),
                    "post_attention_layernorm.weight": f(L["ln2"]), "mlp.gate_proj.weight": f(L["wgu"][:inter]),
                    "mlp.up_proj.weight": f(L["wgu"][inter:]), "mlp.down_proj.weight": f(L["wd"])})
    else:   # the scoring layer: only its logits are used, so only q_proj / k_proj exist on the device
        out.update({"self_attn.q_proj.weight": f(L["wq"]), "self_attn.k_proj.weight": f(L["wk"])})
    return out


def cpu_baseline_and_parity(rk, devb, bl, mbl):
    """Rank 0, N=1: the CPU layer on prompt 0 of the timed batch, fed with the GPU path's own activations.
    (1) layer 0: input = the embedding rows the GPU looked up, weights = the GPU's layer-0 weights; its output
        is compared with the GPU's layer-0 output (timed: one plain decoder layer);
    (2) scoring layer: input = the residual stream the GPU produced for layer 20, weights = the GPU's q/k
        projections of layer 20; its document logits are compared with the GPU's (timed: one layer with the raw
        scores returned, plus the score reduction)."""
    from blockrank_b200 import ops
    threads = os.cpu_count() or 1
    cpu = make_cpu_layer(threads)
    T = sum(bl)
    mask, idx, pos_d, labels = padded_grid(bl, devb["position_ids"][0, :T].cpu())
    S = devb["input_ids"].shape[1]
    one = lambda k: devb[k][:1]
    sp0, sp1 = devb["block_spans"][0, :1], devb["block_spans"][1, :1]
    pos32 = one("position_ids").reshape(S).to(torch.int32)
    h = torch.embedding(rk.embed, one("input_ids").reshape(S))
    h_in0 = h.float().cpu()
    rk.decoder_layer(0, h, pos32, 1, S, sp0, sp1, mbl, bl[-1])
    h_out0 = h.float().cpu()
    h20 = rk.hidden_before_score_layer(one("input_ids"), one("position_ids"), sp0, sp1, mbl, bl[-1])
    logits_gpu, _ = rk.score_from_hidden(h20, one("position_ids"), sp0, sp1, one("signal_rows"))
    h20, logits_gpu = h20.float().cpu(), logits_gpu.float().cpu()
    ops.check_status()
    hid = h_in0.shape[1]
    grid = lambda t: torch.zeros(1, mask.shape[1] * mask.shape[2], hid).index_copy_(1, idx, t[:T][None])

    cpu.load(layer_tensors(rk, 0))
    t0 = time.perf_counter()
    ref_out0 = cpu.layer_pass(grid(h_in0), pos_d, mask)
    t_layer = time.perf_counter() - t0
    d0 = (ref_out0[0, idx] - h_out0[:T])
    cpu.load(layer_tensors(rk, SCORE_LAYER))
    t0 = time.perf_counter()
    ref_logits = cpu.scored_pass(grid(h20), pos_d, mask, labels).float()
    t_score = time.perf_counter() - t0
    rel = ((logits_gpu - ref_logits).abs() / ref_logits.abs()).max().item()
    k = min(10, ref_logits.shape[-1])
    srt = ref_logits.sort(-1, descending=True).values
    per_prompt = SCORE_LAYER * t_layer + t_score
    base = {"value": 1.0 / per_prompt, "unit": "prompts/s", "cores": threads, "kind": cpu.kind,
            "sample": f"prompt 0 of the batch on the reference's padded grid, fp32: 1 decoder layer = {t_layer:.2f}s, scoring "
                      f"layer with raw scores + score reduction = {t_score:.2f}s; extrapolated to {SCORE_LAYER} layers + scoring layer"}
    parity = {"checked": "prompt 0: GPU layer-0 output and GPU document logits vs the CPU reference layer fed with the GPU's "
                         "own layer inputs and weights (fp32 on the host)",
              "layer0_max_abs_err": d0.abs().max().item(),
              "layer0_rel_fro_err": (d0.norm() / ref_out0[0, idx].norm()).item(),
              "logits_max_rel_err": rel,
              "top10_equal": bool(torch.equal(torch.topk(logits_gpu, k).indices, torch.topk(ref_logits, k).indices)),
              "ref_min_gap_top11": (srt[:, :k] - srt[:, 1:k + 1]).min().item() if ref_logits.shape[-1] > k else None,
              "logits_max_abs_err": (logits_gpu - ref_logits).abs().max().item()}
    return base, parity


def run_ours(args, cfg):
    import torch.distributed as dist
    from blockrank_b200 import _lib, ops
    from blockrank_b200.parallel import gather_scores, partition_prompts
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

    rcfg = RankerConfig.mistral_7b(SCORE_LAYER)
    rk = MistralPrefillRanker(rcfg, dev, torch.bfloat16).init_random(seed=3)
    rk.algo = {"auto": _lib.ALGO_AUTO, "simt": _lib.ALGO_SIMT, "tc": _lib.ALGO_TC}[args.algo]
    P = args.prompts
    total = world * P
    all_bl = [block_lengths(cfg, p) for p in range(total)]
    costs = [sum(bl) for bl in all_bl] if cfg["ragged"] is not None else None
    my_ids = partition_prompts(total, world, rank, costs)
    max_share = max(len(partition_prompts(total, world, r, costs)) for r in range(world))
    bls = [all_bl[p] for p in my_ids]
    host = make_host_batch(bls, seed=4 + rank, pin=True)
    devb = {k: (v.to(dev) if torch.is_tensor(v) else v) for k, v in host.items()}
    mbl, mql = host["max_block_len"], max(bl[-1] for bl in bls)
    n_local = len(bls)
    micro = max(1, min(args.micro, n_local))
    # every forward is padded to the longest prompt of ITS micro-batch, as a caller batching ragged prompts would do
    # (the collated batch is padded to the longest local prompt)
    s_mb = {i: min(host["input_ids"].shape[1], -(-max(sum(bl) for bl in bls[i:i + micro]) // 8) * 8)
            for i in range(0, n_local, micro)}

    def step_resident():
        outs = []
        for i in range(0, n_local, micro):
            sl = slice(i, i + micro)
            lg, _ = rk.score(devb["input_ids"][sl, :s_mb[i]], devb["position_ids"][sl, :s_mb[i]], devb["block_spans"][0, sl],
                             devb["block_spans"][1, sl], mbl, devb["signal_rows"][sl], mql)
            outs.append(lg)
        scores = torch.cat(outs)
        return gather_scores(scores, my_ids, total, max_share=max_share) if world > 1 else scores

    def step_e2e():
        outs = []
        for i in range(0, n_local, micro):
            sl = slice(i, i + micro)
            mb = {"input_ids": host["input_ids"][sl, :s_mb[i]], "position_ids": host["position_ids"][sl, :s_mb[i]],
                  "block_spans": host["block_spans"][:, sl], "signal_rows": host["signal_rows"][sl],
                  "max_block_len": mbl}
            outs.append(rk.rank_host(mb))
        if world > 1:   # the same collective as the resident step: every rank ends up with all scores
            return gather_scores(torch.cat([lg for lg, _ in outs]).to(dev), my_ids, total, max_share=max_share)
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
    ops.check_status(dev)
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
    ops.check_status(dev)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    pk = peaks()
    work = [attention_work(bl, s_mb[(j // micro) * micro]) for j, bl in enumerate(bls)]
    step_exact, step_bytes, step_tile = (sum(w[i] for w in work) for i in range(3))
    # every timed attention launch covers one micro-batch of one layer: per step, SCORE_LAYER launches per micro-batch
    attn_s_per_step = sum(attn_ms) / 1e3 / args.steps / SCORE_LAYER      # all micro-batches of one layer
    n_micro = -(-n_local // micro)
    achieved = step_exact / attn_s_per_step / 1e12
    live = step_tile / attn_s_per_step / 1e12
    sc_s_per_step = sum(score_ms) / 1e3 / args.steps
    sc_bytes = sum(score_bytes(bl) for bl in bls)
    value = total * args.steps / (total_ms / 1e3)
    e2e = total * args.steps / (e2e_ms / 1e3)
    h2d = sum(v.numel() * v.element_size() for key, v in host.items() if torch.is_tensor(v) and key not in ("input_ids", "position_ids"))
    h2d += sum(2 * 8 * len(bls[i:i + micro]) * s for i, s in s_mb.items())  # int64 ids and positions of each forward
    nd = cfg["docs"]
    d2h = n_local * nd * 4 + n_local * min(10, nd) * 8
    tc = args.algo != "simt"
    line = {
        "metric": METRIC, "value": value, "unit": "prompts/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": workload_config(args, cfg, bls[0]),
        "e2e": {"value": e2e, "unit": "prompts/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "roofline": {"bound": "tensor", "kernel": "attn_tc_kernel" if tc else "attn_simt_kernel",
                     "achieved": achieved, "peak": pk["bf16_tflops_sustained"], "unit": "TFLOP/s",
                     "frac": achieved / pk["bf16_tflops_sustained"],
                     # dram__bytes_read+write per prompt from the ncu capture summarised under profiles/ (2 prompts of the
                     # c4 geometry), scaled to the prompts of one launch: traffic grows in proportion to the prompts
                     "traffic": NCU_TRAFFIC_PER_PROMPT * micro if args.config == "c4" and tc and NCU_TRAFFIC_PER_PROMPT else None,
                     "peak_source": pk["source"],
                     "flops_exact_per_launch": step_exact / n_micro, "launch_ms": attn_s_per_step / n_micro * 1e3,
                     "live_tile_tflops": live, "live_tile_frac": live / pk["bf16_tflops_sustained"],
                     "exact_over_tile": step_exact / step_tile,
                     "hbm_gbs": step_bytes / attn_s_per_step / 1e9,
                     "hbm_frac": step_bytes / attn_s_per_step / 1e9 / pk["hbm_gbs"],
                     "launches_timed": len(attn_ms)},
        "score_epilogue": {"bound": "hbm", "achieved": sc_bytes / sc_s_per_step / 1e9, "peak": pk["hbm_gbs"],
                           "unit": "GB/s", "frac": sc_bytes / sc_s_per_step / 1e9 / pk["hbm_gbs"],
                           "launch_ms": sc_s_per_step / n_micro * 1e3},
        "clocks": clk.summary(),
    }
    if world == 1 and not args.no_cpu_baseline and (cfg["ragged"] is None or args.cpu_baseline):
        line["cpu_baseline"], line["parity"] = cpu_baseline_and_parity(rk, devb, bls[0], mbl)
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# dram__bytes_read.sum + dram__bytes_write.sum of attn_tc_kernel per prompt of the c4 geometry (profiles/)
NCU_TRAFFIC_PER_PROMPT = 388.3e6


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="c4", choices=sorted(CONFIGS))
    ap.add_argument("--prompts", type=int, default=0, help="prompts per GPU per step (default: the config's)")
    ap.add_argument("--micro", type=int, default=0, help="prompts per forward pass (default: the config's)")
    ap.add_argument("--algo", default="auto", choices=["auto", "simt", "tc"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-baseline", action="store_true", help="run the CPU leg for the ragged config too (minutes, tens of GB)")
    ap.add_argument("--graphs", action="store_true", help="e2e leg replays one captured CUDA graph per forward pass")
    args = ap.parse_args()
    cfg = CONFIGS[args.config]
    args.prompts = args.prompts or cfg["prompts"]
    args.micro = args.micro or cfg["micro"]
    if args.impl == "reference":
        run_reference(args, cfg)
    else:
        if args.warmup < 3:
            args.warmup = 3
        with torch.no_grad():
            run_ours(args, cfg)


if __name__ == "__main__":
    main()
