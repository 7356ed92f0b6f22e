"""Pin the CPU oracle against fixtures produced by the reference's own code."""
import os

import numpy as np
import pytest
import torch

from oracle import blockrank_oracle as orc

ATTN_CASES = ["attn_fp32_ragged", "attn_bf16_ragged", "attn_fp32_m1", "attn_fp32_m2", "attn_fp32_short_window"]


def load(golden_dir, name):
    z = np.load(os.path.join(golden_dir, name + ".npz"))
    return {k: z[k] for k in z.files}


def valid_rows(mask):
    return torch.from_numpy(mask).reshape(mask.shape[0], -1)


@pytest.mark.parametrize("name", ATTN_CASES)
def test_attention_matches_reference(golden_dir, name):
    fx = load(golden_dir, name)
    q, k, v = (torch.from_numpy(fx[n]) for n in "qkv")
    mask = torch.from_numpy(fx["mask"])
    ref = torch.from_numpy(fx["out"])
    rows = valid_rows(fx["mask"])
    bf16 = str(fx["dtype"]) == "bfloat16"
    dense, _ = orc.attention_dense(q, k, v, mask, float(fx["scaling"]))
    err = (dense.float() - ref)[rows].abs().max().item()
    assert err < (2e-2 if bf16 else 2e-6), err
    blocked = orc.attention_blocked(q, k, v, mask, float(fx["scaling"]),
                                    emulate=torch.bfloat16 if bf16 else None).float()
    err_b = (blocked - ref)[rows].abs().max().item()
    # with the rounding points emulated the bf16 run is reproduced to one output ulp
    assert err_b < (8e-3 if bf16 else 2e-6), err_b
    # the reference's SDPA variant agrees with its eager variant on valid rows
    err_s = (torch.from_numpy(fx["out_sdpa"]) - ref)[rows].abs().max().item()
    assert err_s < (2e-2 if bf16 else 2e-6)
    # pad rows of the oracle are zero by convention
    assert blocked[~rows].abs().max().item() == 0 if (~rows).any() else True


@pytest.mark.parametrize("name", ["attn_fp32_ragged", "attn_fp32_m2", "attn_fp32_short_window"])
def test_additive_mask_matches_reference(golden_dir, name):
    fx = load(golden_dir, name)
    add = orc.additive_block_mask(torch.from_numpy(fx["mask"]), torch.float32)
    assert torch.equal(add, torch.from_numpy(fx["add_mask"]))


@pytest.mark.parametrize("name", ["attn_fp32_ragged", "attn_bf16_ragged", "attn_fp32_m2", "attn_fp32_short_window",
                                  "attn_fp32_h8"])
def test_raw_scores_match_reference(golden_dir, name):
    fx = load(golden_dir, name)
    q, k = torch.from_numpy(fx["q"]), torch.from_numpy(fx["k"])
    dt = torch.bfloat16 if str(fx["dtype"]) == "bfloat16" else torch.float32
    raw = orc.raw_last_scores(q.to(dt), k.to(dt), torch.from_numpy(fx["mask"]), float(fx["scaling"]),
                              int(fx["num_last"])).float()
    ref = torch.from_numpy(fx["raw"])
    assert raw.shape == ref.shape
    live = ref > -1e30
    assert torch.equal(live, raw > -1e30)
    tol = 6e-2 if dt == torch.bfloat16 else 1e-5
    assert (raw - ref)[live].abs().max().item() < tol
    # masked entries carry the reference's finite addend
    assert torch.allclose(raw[~live], ref[~live], rtol=1e-2)


@pytest.mark.parametrize("name", ["attn_fp32_ragged", "attn_bf16_ragged", "attn_fp32_short_window"])
def test_doc_scores_match_reference(golden_dir, name):
    fx = load(golden_dir, name)
    mask = torch.from_numpy(fx["mask"])
    labels = torch.from_numpy(fx["labels"])
    ref = torch.from_numpy(fx["logits"])
    bf16 = str(fx["dtype"]) == "bfloat16"
    raw = torch.from_numpy(fx["raw"])
    got = orc.doc_scores_from_raw(raw, labels, mask)
    assert torch.allclose(got, ref, rtol=2e-2 if bf16 else 1e-5, atol=1e-6)
    # closed form: per-head/per-row document masses
    B, M, H = mask.shape
    S = M * H
    rows = torch.tensor([[S - 2, S - 1]] * B)
    mass = orc.doc_mass(torch.from_numpy(fx["q"]), torch.from_numpy(fx["k"]), mask, float(fx["scaling"]), rows)
    closed = (mass.mean(dim=(1, 2)) / 0.05).float()
    assert torch.allclose(closed, ref, rtol=3e-2 if bf16 else 1e-4, atol=1e-5)
    assert torch.allclose(mass.sum(-1), torch.ones_like(mass.sum(-1)), atol=1e-9)


def test_collate_matches_reference(golden_dir):
    fx = load(golden_dir, "collate")
    for ci in range(3):
        n = int(fx[f"c{ci}_n"])
        cap = int(fx[f"c{ci}_cap"]) or None
        prompts = []
        for b in range(n):
            ids, lens = fx[f"c{ci}_ids{b}"], fx[f"c{ci}_lens{b}"].tolist()
            lens = lens[:-2] + [lens[-2] + lens[-1]]  # completion merged into the last block
            cuts = np.cumsum([0] + lens)
            prompts.append([ids[cuts[i]:cuts[i + 1]].tolist() for i in range(len(lens))])
        got = orc.collate_blocks(prompts, pad_id=0, pad_to_multiple_of=16, max_block_length=cap)
        for key in ("input_ids", "position_ids", "attention_mask"):
            assert np.array_equal(got[key].numpy(), fx[f"c{ci}_{key}"]), (ci, key)
        if cap is None:  # labels of a truncated query block depend on what survives the cut
            assert np.array_equal(got["labels"].numpy(), fx[f"c{ci}_labels"]), ci


def test_block_spans_and_pairs():
    mask = torch.zeros(1, 3, 4, dtype=torch.bool)
    mask[0, 0, 2:] = True
    mask[0, 1, 1:] = True
    mask[0, 2, 3:] = True
    start, ln = orc.block_spans(mask)
    assert start.tolist() == [[2, 5, 11]] and ln.tolist() == [[2, 3, 1]]
    ok = orc.allowed_pairs(mask)[0]
    assert ok.sum().item() == orc.live_pairs([2, 3, 1])
    # the document never sees the query block, the query row sees every valid earlier token
    assert not ok[5:8, 8:].any() and ok[11, [2, 3, 5, 6, 7, 11]].all()


def test_tiny_mistral_matches_reference(golden_dir):
    """The tiny CPU-plumbing configuration end to end: rebuild the seeded HF weights, run the restated decoder."""
    from transformers import MistralConfig, MistralForCausalLM
    fx = load(golden_dir, "tiny_mistral")
    torch.manual_seed(0)
    cfg = MistralConfig(vocab_size=32768, hidden_size=256, intermediate_size=688, num_hidden_layers=4,
                        num_attention_heads=4, num_key_value_heads=2, head_dim=64, rope_theta=1e6,
                        rms_norm_eps=1e-5, sliding_window=None)
    model = MistralForCausalLM(cfg).eval()
    wsum = float(sum(p.double().abs().sum() for p in model.parameters()))
    if abs(wsum - float(fx["weight_abs_sum"])) > 1e-6 * wsum:
        pytest.skip("seeded HF initialisation differs from the one the fixture was made with")
    w = {k: v.detach() for k, v in model.state_dict().items()}
    c = dict(n_heads=4, n_kv_heads=2, head_dim=64, rope_theta=1e6, rms_eps=1e-5)
    logits, raw, h_in = orc.mistral_prefill_scores(
        w, c, torch.from_numpy(fx["input_ids"]), torch.from_numpy(fx["position_ids"]),
        torch.from_numpy(fx["mask"]), torch.from_numpy(fx["labels"]), int(fx["score_layer"]))
    rows = valid_rows(fx["mask"])
    assert (h_in - torch.from_numpy(fx["hidden_in"]))[rows].abs().max().item() < 1e-4
    ref_raw = torch.from_numpy(fx["raw"])
    live = ref_raw > -1e30
    assert (raw - ref_raw)[live].abs().max().item() < 1e-4
    ref = torch.from_numpy(fx["logits"])
    assert torch.allclose(logits, ref, rtol=1e-4)
    assert torch.equal(orc.topk_docs(logits), orc.topk_docs(ref))
