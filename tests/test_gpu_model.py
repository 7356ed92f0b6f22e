"""GPU tests of the model-level path: runner helper kernels, the Hugging Face registry
drop-in on the tiny Mistral (the tiny CPU-plumbing configuration) and the early-exit runner."""
import os

import numpy as np
import pytest
import torch

from oracle import blockrank_oracle as orc
from tests import helpers as H_

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    from blockrank_b200 import ops, register_cuda_blockrank_attention, signal_rows_from_labels
    from blockrank_b200.runner import MistralPrefillRanker, RankerConfig


def _load(golden_dir, name):
    z = np.load(os.path.join(golden_dir, name + ".npz"))
    return {k: z[k] for k in z.files}


@pytest.mark.parametrize("hidden", [256, 1024, 4096])  # 256: row staged in shared memory; 1024, 4096: register-resident rows
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_rmsnorm(dt, hidden):
    g = torch.Generator().manual_seed(0)
    x = torch.randn(37, hidden, generator=g).to(dt)
    h = torch.randn(37, hidden, generator=g).to(dt)
    w = (1 + 0.1 * torch.randn(hidden, generator=g)).to(dt)
    out = ops.rmsnorm(x.cuda(), w.cuda(), 1e-5).cpu()
    ref = orc.rms_norm(x, w, 1e-5)
    tol = 2e-2 if dt == torch.bfloat16 else 1e-5
    assert (out.float() - ref.float()).abs().max().item() < tol
    hc = h.clone().cuda()
    out2 = ops.rmsnorm(x.cuda(), w.cuda(), 1e-5, residual=hc).cpu()
    summed = (x + h)
    assert (hc.cpu().float() - summed.float()).abs().max().item() < tol
    assert (out2.float() - orc.rms_norm(summed, w, 1e-5).float()).abs().max().item() < 2 * tol


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_rope(dt):
    g = torch.Generator().manual_seed(1)
    T, N, Nk, D = 50, 4, 2, 64
    qkv = torch.randn(T, (N + 2 * Nk) * D, generator=g).to(dt)
    pos = torch.randint(0, 17000, (T,), generator=g)
    inv = 1.0 / (1e6 ** (torch.arange(0, D, 2, dtype=torch.int64).float() / D))
    c = qkv.cuda()
    ops.rope_(c[:, :N * D].view(T, N, D), c[:, N * D:(N + Nk) * D].view(T, Nk, D), pos.int().cuda(), inv.cuda())
    cos, sin = orc.rope_tables(pos[None], D, 1e6)
    qr = orc.apply_rope(qkv[:, :N * D].view(1, T, N, D).transpose(1, 2).float(), cos, sin).transpose(1, 2).reshape(T, -1)
    kr = orc.apply_rope(qkv[:, N * D:(N + Nk) * D].view(1, T, Nk, D).transpose(1, 2).float(), cos, sin).transpose(1, 2).reshape(T, -1)
    # bf16: two roundings of values up to ~4 (ulp 2^-6 there), so the bound is relative to magnitude
    tol = 2e-5 if dt == torch.float32 else None
    got = c.cpu().float()
    for a_, r_ in ((got[:, :N * D], qr), (got[:, N * D:(N + Nk) * D], kr)):
        bound = tol if tol else (2 ** -6) * r_.abs().clamp_min(1.0)
        assert bool(((a_ - r_).abs() <= bound).all())
    assert torch.equal(got[:, (N + Nk) * D:], qkv[:, (N + Nk) * D:].float())  # V untouched


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_silu_mul(dt):
    g = torch.Generator().manual_seed(2)
    gu = torch.randn(33, 2 * 688, generator=g).to(dt)
    out = ops.silu_mul(gu.cuda()).cpu().float()
    ref = torch.nn.functional.silu(gu[:, :688].float()) * gu[:, 688:].float()
    assert (out - ref).abs().max().item() < (3e-2 if dt == torch.bfloat16 else 1e-5)


def _tiny_hf_model():
    from transformers import MistralConfig, MistralForCausalLM
    torch.manual_seed(0)
    cfg = MistralConfig(vocab_size=32768, hidden_size=256, intermediate_size=688, num_hidden_layers=4,
                        num_attention_heads=4, num_key_value_heads=2, head_dim=64, rope_theta=1e6,
                        rms_norm_eps=1e-5, sliding_window=None)
    return MistralForCausalLM(cfg).eval()


def _check_weights(model, fx):
    wsum = float(sum(p.detach().double().abs().sum() for p in model.parameters()))
    if abs(wsum - float(fx["weight_abs_sum"])) > 1e-6 * wsum:
        pytest.skip("seeded HF initialisation differs from the one the fixture was made with")


def test_hf_registry_tiny_mistral_matches_reference(golden_dir):
    """Config 1 through the transformers registries, reference call sequence of scripts/eval_attn.py:
    early exit after layer l*, raw scores out of `attentions`, then the reference reduction."""
    fx = _load(golden_dir, "tiny_mistral")
    model = _tiny_hf_model()
    _check_weights(model, fx)
    name = register_cuda_blockrank_attention()
    assert "blockrank" in name
    model.set_attn_implementation(name)
    model = model.cuda()
    L = int(fx["score_layer"])
    layers = model.model.layers

    def ident(self, hidden_states, *a, **kw):
        return hidden_states

    for i in range(L + 1, len(layers)):
        layers[i].forward = ident.__get__(layers[i], type(layers[i]))
    model.lm_head.forward = ident.__get__(model.lm_head, type(model.lm_head))
    ids = torch.from_numpy(fx["input_ids"]).cuda()
    pos = torch.from_numpy(fx["position_ids"]).cuda()
    mask = torch.from_numpy(fx["mask"]).cuda()
    labels = torch.from_numpy(fx["labels"])
    with torch.no_grad():
        out = model(input_ids=ids, position_ids=pos, attention_mask=mask, output_attentions=True,
                    layers_to_return_scores=[L])
    assert len(out.attentions) == 1
    raw = out.attentions[0].float().cpu()
    ref_raw = torch.from_numpy(fx["raw"])
    assert raw.shape == ref_raw.shape
    live = ref_raw > -1e30
    assert (raw - ref_raw)[live].abs().max().item() < 1e-4
    logits = orc.doc_scores_from_raw(raw, labels, torch.from_numpy(fx["mask"]))
    ref = torch.from_numpy(fx["logits"])
    assert torch.allclose(logits, ref, rtol=1e-4)
    assert torch.equal(orc.topk_docs(logits), orc.topk_docs(ref))
    # fused scorer through the same registry call
    rows = signal_rows_from_labels(labels).cuda()
    with torch.no_grad():
        out2 = model(input_ids=ids, position_ids=pos, attention_mask=mask, output_attentions=True,
                     layers_to_return_scores=[L], blockrank_doc_scores=True, signal_rows=rows)
    mass = out2.attentions[0]
    fused = (mass.mean(dim=(1, 2)) / 0.05).cpu()
    assert torch.allclose(fused, ref, rtol=1e-4)


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_runner_tiny_matches_reference(golden_dir, dt):
    """The lean early-exit runner on the same seeded weights: logits and top-10 vs the reference."""
    fx = _load(golden_dir, "tiny_mistral")
    model = _tiny_hf_model()
    _check_weights(model, fx)
    L = int(fx["score_layer"])
    rk = MistralPrefillRanker(RankerConfig.tiny(score_layer=L), "cuda", dtype=dt).load_state_dict(model.state_dict())
    mask = torch.from_numpy(fx["mask"])
    start, ln = ops.spans_from_mask(mask.cuda())
    rows = signal_rows_from_labels(torch.from_numpy(fx["labels"])).cuda()
    logits, mass = rk.score(torch.from_numpy(fx["input_ids"]).cuda(), torch.from_numpy(fx["position_ids"]).cuda(),
                            start, ln, mask.shape[-1], rows)
    ref = torch.from_numpy(fx["logits"])
    rel = ((logits.cpu() - ref).abs() / ref.abs()).max().item()
    assert rel < (1e-2 if dt == torch.bfloat16 else 1e-4), rel
    if dt == torch.float32:
        assert torch.equal(orc.topk_docs(logits.cpu()), orc.topk_docs(ref))
        h = rk.hidden_before_score_layer(torch.from_numpy(fx["input_ids"]).cuda(),
                                         torch.from_numpy(fx["position_ids"]).cuda(), start, ln, mask.shape[-1])
        hid = h.cpu().view(1, -1, 256)
        vr = mask.reshape(1, -1)
        assert (hid - torch.from_numpy(fx["hidden_in"]))[vr].abs().max().item() < 1e-4


def test_runner_packed_equals_padded():
    """Padding-free prompt layout through the runner gives the same scores as the padded grid."""
    cfg = RankerConfig.tiny(score_layer=2)
    rk = MistralPrefillRanker(cfg, "cuda", dtype=torch.float32).init_random(seed=3)
    blens = [[20, 33, 7, 48, 15, 30], [31, 48, 48, 1, 9, 16]]
    B, M, Hp = 2, 6, 48
    g = torch.Generator().manual_seed(9)
    toks = [[torch.randint(3, 32768, (n,), generator=g).tolist() for n in bl] for bl in blens]
    pad = orc.collate_blocks(toks, pad_id=0, pad_to_multiple_of=16)
    mask = pad["attention_mask"]
    assert mask.shape[-1] == Hp
    start, ln = ops.spans_from_mask(mask.cuda())
    S = M * Hp
    rows = torch.tensor([[S - 2, S - 1]] * B, dtype=torch.int32).cuda()
    lp, _ = rk.score(pad["input_ids"].cuda(), pad["position_ids"].cuda(), start, ln, Hp, rows)
    ps, pl, Sp, mbl = H_.packed_spans(blens)
    ids = torch.zeros(B, Sp, dtype=torch.long)
    pos = torch.zeros(B, Sp, dtype=torch.long)
    prow = torch.zeros(B, 2, dtype=torch.int32)
    for b in range(B):
        idx = H_.packed_to_padded(blens[b], Hp)
        ids[b, :idx.numel()] = pad["input_ids"][b, idx]
        pos[b, :idx.numel()] = pad["position_ids"][b, idx]
        prow[b, 0], prow[b, 1] = idx.numel() - 2, idx.numel() - 1
    lq, _ = rk.score(ids.cuda(), pos.cuda(), ps.cuda(), pl.cuda(), mbl, prow.cuda())
    assert torch.allclose(lp, lq, rtol=1e-4), (lp, lq)


def test_runner_graph_replay_equals_eager():
    """The captured CUDA graph of the scoring pass gives the eager result, also when replayed on new
    inputs of the same geometry (bf16, tensor-core attention: head_dim 128, N/Nk = 4)."""
    cfg = RankerConfig(vocab_size=1024, hidden_size=512, intermediate_size=1024, num_hidden_layers=3,
                       num_attention_heads=4, num_key_value_heads=1, head_dim=128, score_layer=2)
    rk = MistralPrefillRanker(cfg, "cuda", dtype=torch.bfloat16).init_random(seed=5)
    blens = [[24, 40, 33, 64, 17, 20], [16, 64, 50, 9, 31, 12]]
    ps, pl, Sp, mbl = H_.packed_spans(blens)
    B = len(blens)
    g = torch.Generator().manual_seed(11)
    rows = torch.tensor([[sum(bl) - 2, sum(bl) - 1] for bl in blens], dtype=torch.int32).cuda()
    outs = []
    for trial in range(2):
        ids = torch.randint(3, 1024, (B, Sp), generator=g).cuda()
        pos = torch.arange(Sp).expand(B, Sp).contiguous().cuda()
        eager, _ = rk.score(ids, pos, ps.cuda(), pl.cuda(), mbl, rows)
        graphed, _ = rk.score_graphed(ids, pos, ps.cuda(), pl.cuda(), mbl, rows)
        torch.cuda.synchronize()
        assert torch.equal(eager, graphed.clone()), (trial, (eager - graphed).abs().max())
        outs.append(eager.clone())
    assert len(rk._graphs) == 1            # one geometry, one capture
    assert not torch.equal(outs[0], outs[1])  # the replay really saw the new tokens


def test_rank_items_matches_score_topk():
    """metrics.rank_items (collate -> rank_host -> top-k lists) against the same prompts scored directly."""
    from blockrank_b200 import metrics
    from blockrank_b200.collate import packed_block_collate_fn
    cfg = RankerConfig.tiny(score_layer=2)
    rk = MistralPrefillRanker(cfg, "cuda", dtype=torch.float32).init_random(seed=7)
    g = torch.Generator().manual_seed(21)
    items = []
    for _ in range(3):
        bl = [12] + [int(x) for x in torch.randint(5, 30, (12,), generator=g)] + [9]  # instruction, 12 docs, query
        items.append({"input_ids": torch.randint(3, 32768, (sum(bl) + 1,), generator=g),
                      "block_lengths": torch.tensor(bl + [1])})                          # completion = last token
    preds = metrics.rank_items(rk, items, batch_size=2, k=5)
    assert len(preds) == 3 and all(len(p) == 5 for p in preds)
    for i, it in enumerate(items):
        b = packed_block_collate_fn([it])
        logits, _ = rk.score(b["input_ids"].cuda(), b["position_ids"].cuda(), b["block_spans"][0].cuda(),
                             b["block_spans"][1].cuda(), b["max_block_len"], b["signal_rows"].cuda())
        assert preds[i] == torch.topk(logits[0], 5).indices.tolist()
    m = metrics.ranking_metrics(preds, [p[0] for p in preds])
    assert m["accuracy"] == 100.0


def test_hf_registry_training_step_gradients(golden_dir):
    """A training step as the auxiliary-loss trainer makes it (src/blockrank/trainer.py:51-107): LM loss plus the
    InfoNCE loss over the per-document logits of layer l* (src/blockrank/losses.py:37-93), back-propagated through
    the registered CUDA attention.  Parameter gradients are compared with the same model run through a plain
    PyTorch attention over the oracle's pair predicate (autograd does the backward there)."""
    import copy
    from transformers import AttentionInterface, AttentionMaskInterface
    from blockrank_b200.attention import cuda_blockrank_attention_mask
    fx = _load(golden_dir, "tiny_mistral")
    base = _tiny_hf_model().float()
    L = int(fx["score_layer"])
    ids = torch.from_numpy(fx["input_ids"]).cuda()
    pos = torch.from_numpy(fx["position_ids"]).cuda()
    mask_cpu = torch.from_numpy(fx["mask"])
    mask = mask_cpu.cuda()
    labels = torch.from_numpy(fx["labels"]).cuda()
    B, M, Hh = mask.shape
    S = M * Hh
    ok = orc.allowed_pairs(mask_cpu).cuda()                       # (B, S, S)
    valid = mask.reshape(B, S)
    ok_safe = ok | ((~valid)[:, :, None] & torch.eye(S, dtype=torch.bool, device="cuda")[None])
    answers = torch.tensor([[1, 3]] * B).cuda()

    def torch_attention(module, query, key, value, attention_mask, scaling, dropout=0.0, **kw):
        g = query.shape[1] // key.shape[1]
        kx, vx = key.repeat_interleave(g, dim=1), value.repeat_interleave(g, dim=1)
        s = torch.matmul(query, kx.transpose(-1, -2)) * scaling
        out = torch.matmul(torch.softmax(s.masked_fill(~ok_safe[:, None], float("-inf")), dim=-1), vx)
        out = out.transpose(1, 2) * valid[:, :, None, None]
        raw = None
        if kw.get("layers_to_return_scores") and module.layer_idx in kw["layers_to_return_scores"]:
            R = min(16, Hh)
            raw = s[:, :, S - R:] + torch.where(ok[:, None, S - R:], 0.0, 0.7 * torch.finfo(s.dtype).min)
        return out, raw

    AttentionInterface.register("torch_ref_blockrank", torch_attention)
    AttentionMaskInterface.register("torch_ref_blockrank", cuda_blockrank_attention_mask)
    name = register_cuda_blockrank_attention()

    def step(impl):
        model = copy.deepcopy(base)
        model.set_attn_implementation(impl)
        model = model.cuda().train()
        out = model(input_ids=ids, position_ids=pos, attention_mask=mask, labels=labels, output_attentions=True,
                    layers_to_return_scores=[L])
        raw = out.attentions[0].float()
        logits = orc.doc_scores_from_raw(raw, labels, mask)          # (B, docs), differentiable
        pos_mask = torch.zeros_like(logits, dtype=torch.bool).scatter_(1, answers, True)
        aux = -(torch.logsumexp(logits.masked_fill(~pos_mask, float("-inf")), 1) - torch.logsumexp(logits, 1)).mean()
        loss = out.loss + 0.1 * aux
        loss.backward()
        return loss.item(), aux.item(), {n: p.grad.detach().double().cpu() for n, p in model.named_parameters() if p.grad is not None}

    loss_c, aux_c, g_c = step(name)
    loss_t, aux_t, g_t = step("torch_ref_blockrank")
    assert abs(loss_c - loss_t) < 1e-4 * abs(loss_t) and abs(aux_c - aux_t) < 1e-4 * max(1.0, abs(aux_t))
    assert g_c.keys() == g_t.keys() and len(g_c) > 20
    worst = max(((g_c[n] - g_t[n]).norm() / g_t[n].norm().clamp_min(1e-12)).item() for n in g_t)
    assert worst < 1e-3, worst
