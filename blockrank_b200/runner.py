"""Early-exit Mistral-architecture prefill ranker: what scripts/eval_attn.py does, minus the waste.

The reference scores documents by running the HF model with every layer after
the scoring layer ``l*`` patched to identity (scripts/eval_attn.py:121-130) and
reducing that layer's raw attention logits (src/blockrank/losses.py:37-78).
Layer ``l*`` itself still runs completely there.  This runner computes the same
scores with the minimal work: layers 0..l*-1 in full, and at layer ``l*`` only
the input RMSNorm, ``k_proj`` for every token, ``q_proj`` for the signal rows,
RoPE and the fused score epilogue.

Dense projections are cuBLAS GEMMs through torch.matmul; RMSNorm, RoPE,
SiLU*up, the block-sparse attention and the scorer are this package's CUDA
kernels.  Weights use the HF parameter names, so a real checkpoint's state
dict loads directly.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import torch

from . import ops, _lib


@dataclass
class RankerConfig:
    vocab_size: int = 32768
    hidden_size: int = 4096
    intermediate_size: int = 14336
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    head_dim: int = 128
    rope_theta: float = 1e6
    rms_norm_eps: float = 1e-5
    score_layer: int = 20
    temperature: float = 0.05

    @staticmethod
    def mistral_7b(score_layer: int = 20) -> "RankerConfig":
        return RankerConfig(score_layer=score_layer)

    @staticmethod
    def tiny(score_layer: int = 2) -> "RankerConfig":
        return RankerConfig(vocab_size=32768, hidden_size=256, intermediate_size=688, num_hidden_layers=4,
                            num_attention_heads=4, num_key_value_heads=2, head_dim=64, score_layer=score_layer)


@dataclass
class _CapturedScore:
    graph: "torch.cuda.CUDAGraph"
    static: list   # input buffers the graph reads
    out: tuple     # (logits, doc_mass) the graph writes


class MistralPrefillRanker:
    """Holds the fused weights of layers 0..score_layer on one GPU and ranks prompts."""

    def __init__(self, cfg: RankerConfig, device, dtype=torch.bfloat16):
        if cfg.score_layer >= cfg.num_hidden_layers:
            raise ValueError("score_layer must index an existing layer")
        _lib.lib()  # no CUDA library, no runner
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        self.embed: Optional[torch.Tensor] = None
        self.layers = []  # dicts: ln1, wqkv, wo, ln2, wgu, wd   (scoring layer: ln1, wq, wk)
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, cfg.head_dim, 2, dtype=torch.int64).float() / cfg.head_dim))
        self.inv_freq = inv.to(self.device)
        self.algo = _lib.ALGO_AUTO
        self.events = None  # set to {"attn": [], "score": []} to collect (start, end) CUDA events per launch
        self.use_graphs = False  # rank_host replays one captured CUDA graph per batch geometry instead of launching eagerly
        self._graphs: Dict[tuple, "_CapturedScore"] = {}

    # ---- weights ---------------------------------------------------------------
    def load_state_dict(self, sd: Dict[str, torch.Tensor]) -> "MistralPrefillRanker":
        """Take HF-named tensors (model.embed_tokens.weight, model.layers.{i}.self_attn.q_proj.weight, ...)."""
        c, dev, dt = self.cfg, self.device, self.dtype
        g = lambda name: sd[name].detach().to(device=dev, dtype=dt)
        self.embed = g("model.embed_tokens.weight")
        self.layers = []
        for i in range(c.score_layer + 1):
            p = f"model.layers.{i}."
            L = {"ln1": g(p + "input_layernorm.weight")}
            if i < c.score_layer:
                L["wqkv"] = torch.cat([g(p + "self_attn.q_proj.weight"), g(p + "self_attn.k_proj.weight"),
                                       g(p + "self_attn.v_proj.weight")], 0).contiguous()
                L["wo"] = g(p + "self_attn.o_proj.weight")
                L["ln2"] = g(p + "post_attention_layernorm.weight")
                L["wgu"] = torch.cat([g(p + "mlp.gate_proj.weight"), g(p + "mlp.up_proj.weight")], 0).contiguous()
                L["wd"] = g(p + "mlp.down_proj.weight")
            else:
                L["wq"] = g(p + "self_attn.q_proj.weight")
                L["wk"] = g(p + "self_attn.k_proj.weight")
            self.layers.append(L)
        return self

    def init_random(self, seed: int = 3, std: float = 0.02) -> "MistralPrefillRanker":
        """Random weights N(0, std) drawn on the device (norm weights 1); only layers 0..score_layer exist."""
        c, dev, dt = self.cfg, self.device, self.dtype
        gen = torch.Generator(device=dev).manual_seed(seed)
        rnd = lambda *shape: (torch.randn(*shape, generator=gen, device=dev, dtype=torch.float32) * std).to(dt)
        ones = lambda n: torch.ones(n, device=dev, dtype=dt)
        qd, kd = c.num_attention_heads * c.head_dim, c.num_key_value_heads * c.head_dim
        self.embed = rnd(c.vocab_size, c.hidden_size)
        self.layers = []
        for i in range(c.score_layer + 1):
            L = {"ln1": ones(c.hidden_size)}
            if i < c.score_layer:
                L["wqkv"] = rnd(qd + 2 * kd, c.hidden_size)
                L["wo"] = rnd(c.hidden_size, qd)
                L["ln2"] = ones(c.hidden_size)
                L["wgu"] = rnd(2 * c.intermediate_size, c.hidden_size)
                L["wd"] = rnd(c.hidden_size, c.intermediate_size)
            else:
                L["wq"] = rnd(qd, c.hidden_size)
                L["wk"] = rnd(kd, c.hidden_size)
            self.layers.append(L)
        return self

    # ---- forward ---------------------------------------------------------------
    @torch.no_grad()
    def decoder_layer(self, i, h, pos, B, S, blk_start, blk_len, max_block_len, max_query_len=0):
        """One full decoder layer ``i < score_layer`` applied in place to the residual stream ``h`` (B*S, hidden).

        Both residual additions happen in the epilogue of the GEMM that produces the branch
        (``h.addmm_``: C = C + A·B, added in fp32 before the rounding), so the branch output is never
        written to memory and the RMSNorm that follows reads one tensor instead of two."""
        c = self.cfg
        N, Nk, D = c.num_attention_heads, c.num_key_value_heads, c.head_dim
        qd, kd = N * D, Nk * D
        T = B * S
        L = self.layers[i]
        x = ops.rmsnorm(h, L["ln1"], c.rms_norm_eps)
        qkv = torch.matmul(x, L["wqkv"].t())                         # (T, qd + 2 kd)
        q3 = qkv[:, :qd].view(T, N, D)
        k3 = qkv[:, qd:qd + kd].view(T, Nk, D)
        ops.rope_(q3, k3, pos, self.inv_freq)
        q4 = qkv[:, :qd].view(B, S, N, D).permute(0, 2, 1, 3)
        k4 = qkv[:, qd:qd + kd].view(B, S, Nk, D).permute(0, 2, 1, 3)
        v4 = qkv[:, qd + kd:].view(B, S, Nk, D).permute(0, 2, 1, 3)
        ev = self._tick("attn")
        attn = ops.attention(q4, k4, v4, blk_start, blk_len, D ** -0.5, max_block_len, algo=self.algo,
                             max_query_len=max_query_len)
        self._tock(ev)
        h.addmm_(attn.view(T, qd), L["wo"].t())                      # h += o_proj(attn)
        x = ops.rmsnorm(h, L["ln2"], c.rms_norm_eps)
        act = ops.silu_mul(torch.matmul(x, L["wgu"].t()))
        h.addmm_(act, L["wd"].t())                                   # h += down_proj(act)
        return h

    @torch.no_grad()
    def hidden_before_score_layer(self, input_ids, position_ids, blk_start, blk_len, max_block_len, max_query_len=0):
        """Run layers 0..l*-1; returns the residual stream entering layer l*, shape (B*S, hidden)."""
        B, S = input_ids.shape
        pos = position_ids.reshape(B * S).to(torch.int32)
        h = torch.embedding(self.embed, input_ids.reshape(B * S))
        for i in range(self.cfg.score_layer):
            self.decoder_layer(i, h, pos, B, S, blk_start, blk_len, max_block_len, max_query_len)
        return h

    @torch.no_grad()
    def score(self, input_ids, position_ids, blk_start, blk_len, max_block_len, signal_rows, max_query_len=0):
        """input_ids/position_ids (B, S) on the device, spans int32 (B, M), signal_rows int32 (B, R);
        ``max_query_len`` (optional) bounds the query block's length (smaller attention scratch).

        Returns (logits (B, num_docs) fp32, doc_mass (B, N, R, num_docs) fp32).  Device-side problems
        (malformed spans, a kernel wait that gave up) are raised by ``ops.check_status()``, which
        :meth:`rank_host` calls after copying the scores back.
        """
        h = self.hidden_before_score_layer(input_ids, position_ids, blk_start, blk_len, max_block_len, max_query_len)
        return self.score_from_hidden(h, position_ids, blk_start, blk_len, signal_rows)

    @torch.no_grad()
    def score_from_hidden(self, h, position_ids, blk_start, blk_len, signal_rows):
        """The scoring layer's share of the work, from the residual stream ``h`` (B*S, hidden) entering it:
        input RMSNorm, ``k_proj`` of every token, ``q_proj`` of the signal rows, RoPE, fused score epilogue."""
        c = self.cfg
        B, S = position_ids.shape
        N, Nk, D = c.num_attention_heads, c.num_key_value_heads, c.head_dim
        R = signal_rows.shape[1]
        L = self.layers[c.score_layer]
        x = ops.rmsnorm(h, L["ln1"], c.rms_norm_eps)
        T = B * S
        pos = position_ids.reshape(T).to(torch.int32)
        k = torch.matmul(x, L["wk"].t()).view(T, Nk, D)
        flat_rows = (signal_rows.to(torch.int64) + torch.arange(B, device=x.device)[:, None] * S).reshape(-1)
        q = torch.matmul(x.index_select(0, flat_rows), L["wq"].t()).view(B * R, N, D)
        # RoPE: keys of every token, queries of the signal rows only
        ops.rope_(q, None, pos.index_select(0, flat_rows), self.inv_freq)
        ops.rope_(None, k, pos, self.inv_freq)
        q4 = q.view(B, R, N, D).permute(0, 2, 1, 3)
        k4 = k.view(B, S, Nk, D).permute(0, 2, 1, 3)
        local_rows = torch.arange(R, device=x.device, dtype=torch.int32).expand(B, R).contiguous()
        ev = self._tick("score")
        mass, logits = ops.doc_scores(q4, k4, blk_start, blk_len, local_rows, D ** -0.5, c.temperature)
        self._tock(ev)
        return logits, mass

    # ---- CUDA graphs -----------------------------------------------------------
    @torch.no_grad()
    def score_graphed(self, input_ids, position_ids, blk_start, blk_len, max_block_len, signal_rows, max_query_len=0):
        """Same contract as :meth:`score`, but the whole launch sequence (about 440 kernels for the 7B
        architecture) is captured once per batch geometry ``(B, S, M, R, max_block_len)`` and replayed.

        Inputs are copied into the graph's static buffers; the returned tensors are the graph's static
        outputs and are overwritten by the next call with the same geometry.  The first call for a
        geometry runs eagerly twice (library initialisation, allocator warm-up) before capturing.
        """
        key = (tuple(input_ids.shape), tuple(blk_start.shape), tuple(signal_rows.shape), int(max_block_len),
               int(max_query_len))
        cap = self._graphs.get(key)
        if cap is None:
            if self.events is not None:
                raise RuntimeError("per-launch events cannot be collected while capturing a CUDA graph")
            static = [t.clone() for t in (input_ids, position_ids, blk_start, blk_len, signal_rows)]
            side = torch.cuda.Stream(device=self.device)
            side.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(side):
                for _ in range(2):
                    self.score(static[0], static[1], static[2], static[3], int(max_block_len), static[4], int(max_query_len))
            torch.cuda.current_stream(self.device).wait_stream(side)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                out = self.score(static[0], static[1], static[2], static[3], int(max_block_len), static[4], int(max_query_len))
            cap = self._graphs[key] = _CapturedScore(graph, static, out)
        for dst, src in zip(cap.static, (input_ids, position_ids, blk_start, blk_len, signal_rows)):
            dst.copy_(src, non_blocking=True)
        cap.graph.replay()
        return cap.out

    def _tick(self, kind):
        if self.events is None:
            return None
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self.events[kind].append((a, b))
        a.record()
        return b

    @staticmethod
    def _tock(ev):
        if ev is not None:
            ev.record()

    @torch.no_grad()
    def rank_host(self, batch: dict, k: int = 10):
        """End-to-end call on HOST tensors: ``batch`` holds pinned ``input_ids``/``position_ids`` (B, S) int64,
        ``block_spans`` int32 (2, B, M), ``signal_rows`` int32 (B, R) and ``max_block_len``.  Copies them to the
        device, scores, and returns (logits, top-k document indices) on the host."""
        dev = self.device
        ids = batch["input_ids"].to(dev, non_blocking=True)
        pos = batch["position_ids"].to(dev, non_blocking=True)
        spans = batch["block_spans"].to(dev, non_blocking=True)
        rows = batch["signal_rows"].to(dev, non_blocking=True)
        run = self.score_graphed if self.use_graphs else self.score
        mql = int(batch["block_spans"][1, :, -1].max())  # host tensor: no synchronisation
        logits, _ = run(ids, pos, spans[0], spans[1], int(batch["max_block_len"]), rows, mql)
        top = torch.topk(logits, k=min(k, logits.shape[-1]), dim=-1).indices
        out = logits.cpu(), top.cpu()
        ops.check_status(dev)  # raises if a kernel reported malformed spans or a wait that gave up
        return out

    def weight_bytes(self) -> int:
        n = self.embed.numel() * self.embed.element_size()
        for L in self.layers:
            n += sum(t.numel() * t.element_size() for t in L.values())
        return n
