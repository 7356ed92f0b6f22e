"""Generate the golden fixtures in this directory from the reference's own code.

Run where the reference checkout is available (it is NOT needed to run the
tests):

    python tests/golden/make_golden.py --reference /path/to/BlockRank

The reference package cannot be imported as a package (its __init__ pulls in
training-only dependencies), so the three files on the prefill path are loaded
by file path.  transformers >= 5 calls mask functions without
``cache_position``; the shim below supplies it.  Every fixture stores its
inputs, so the tests never have to regenerate random numbers.
"""
import argparse
import importlib.util
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _load(name, path):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


class _Mod:
    def __init__(self, groups, layer_idx=0):
        self.num_key_value_groups = groups
        self.layer_idx = layer_idx
        self.training = False


def ragged_mask(B, M, H, lens):
    mask = torch.zeros(B, M, H, dtype=torch.bool)
    for b in range(B):
        for m in range(M):
            n = lens[b][m]
            if n:
                mask[b, m, H - n:] = True
    return mask


def attn_case(std, losses, name, seed, B, N, Nk, D, M, H, lens, dtype, num_last=16):
    g = torch.Generator().manual_seed(seed)
    S = M * H
    # memory layout [B,S,heads,D] viewed as (B,heads,S,D), as the HF model hands it over
    q = (torch.randn(B, S, N, D, generator=g) * 0.5).to(dtype).transpose(1, 2)
    k = (torch.randn(B, S, Nk, D, generator=g) * 0.5).to(dtype).transpose(1, 2)
    v = (torch.randn(B, S, Nk, D, generator=g) * 0.5).to(dtype).transpose(1, 2)
    mask = ragged_mask(B, M, H, lens)
    add = std.eager_blockrank_attention_mask(B, None, S, attention_mask=mask, dtype=dtype)
    scaling = D ** -0.5
    mod = _Mod(N // Nk)
    out, raw = std.eager_blockrank_attention_forward(mod, q, k, v, add, scaling,
                                                     return_last_block_attn_scores=True,
                                                     num_last_queries=num_last)
    out_sdpa, _ = std.sdpa_blockrank_attention_forward(mod, q, k, v, add, scaling)
    fx = dict(q=q.float().numpy(), k=k.float().numpy(), v=v.float().numpy(),
              mask=mask.numpy(), scaling=np.float64(scaling),
              out=out.float().numpy(), out_sdpa=out_sdpa.float().numpy(),
              add_mask=add.float().numpy() if S <= 256 else np.zeros(0, np.float32),
              dtype=str(dtype).replace("torch.", ""), num_last=num_last)
    if raw is not None:
        fx["raw"] = raw.float().numpy()
        if M >= 3:
            labels = torch.full((B, S), -100, dtype=torch.long)
            labels[:, -1] = 7
            logits = losses.compute_auxiliary_attention_loss(raw, labels, mask, None, return_logits=True)
            fx["labels"] = labels.numpy()
            fx["logits"] = logits.float().numpy()
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **fx)
    print(name, {k_: getattr(v_, "shape", v_) for k_, v_ in fx.items()})


def collate_case(ref_root):
    pkg = types.ModuleType("blockrank")
    pkg.__path__ = [os.path.join(ref_root, "src", "blockrank")]
    sys.modules["blockrank"] = pkg
    stub = types.ModuleType("blockrank.utils")
    for n in ("remap_documents", "create_prompt_completion_format", "create_conversation_format"):
        setattr(stub, n, None)
    sys.modules["blockrank.utils"] = stub
    ds = _load("blockrank.dataset", os.path.join(ref_root, "src", "blockrank", "dataset.py"))

    class Tok:
        pad_token_id = 0
        padding_side = "left"

    rng = np.random.default_rng(11)
    out = {}
    for ci, (B, M, lo, hi, cap) in enumerate([(2, 5, 3, 40, None), (3, 4, 1, 70, 48), (1, 3, 16, 17, None)]):
        batch, flat = [], []
        for b in range(B):
            lens = rng.integers(lo, hi, size=M).tolist()
            comp = 1
            ids = rng.integers(3, 1000, size=sum(lens) + comp)
            batch.append({"input_ids": torch.tensor(ids), "block_lengths": torch.tensor(lens + [comp]),
                          "answer_ids": torch.tensor([0])})
            flat.append((ids, lens, comp))
        res = ds.block_icr_collate_fn(batch, Tok(), pad_to_multiple_of=16, max_block_length=cap)
        out[f"c{ci}_cap"] = np.int64(cap or 0)
        out[f"c{ci}_n"] = np.int64(B)
        for b, (ids, lens, comp) in enumerate(flat):
            out[f"c{ci}_ids{b}"] = ids
            out[f"c{ci}_lens{b}"] = np.array(lens + [comp])
        for key in ("input_ids", "position_ids", "attention_mask", "labels"):
            out[f"c{ci}_{key}"] = res[key].numpy()
    np.savez_compressed(os.path.join(HERE, "collate.npz"), **out)
    print("collate", len(out))


def tiny_model_case(std, losses):
    """The tiny CPU-plumbing configuration: random-init Mistral, 32+10x64+32 tokens, score at layer 2, fp32 CPU."""
    from transformers import AttentionInterface, AttentionMaskInterface, MistralConfig, MistralForCausalLM

    def mask_shim(*a, **kw):
        kw.pop("q_length", None)
        kw.pop("q_offset", None)
        return std.eager_blockrank_attention_mask(kw.pop("batch_size"), kw.pop("cache_position", None),
                                                  kw.pop("kv_length"), **kw)

    AttentionInterface.register("eager_blockrank", std.eager_blockrank_attention_forward)
    AttentionMaskInterface.register("eager_blockrank", mask_shim)
    torch.manual_seed(0)
    cfg = MistralConfig(vocab_size=32768, hidden_size=256, intermediate_size=688, num_hidden_layers=4,
                        num_attention_heads=4, num_key_value_heads=2, head_dim=64, rope_theta=1e6,
                        rms_norm_eps=1e-5, sliding_window=None, attn_implementation="eager_blockrank")
    model = MistralForCausalLM(cfg).eval()
    M, H, L = 12, 64, 2
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(3, 32768, (1, M, H), generator=g)
    mask = torch.ones(1, M, H, dtype=torch.bool)
    mask[:, 0, :32] = False
    mask[:, -1, :32] = False
    pos = mask.long().cumsum(-1)
    pos[:, 1:-1] += pos[:, 0].max(-1).values[:, None, None]
    pos[:, -1] += 16384
    pos = (pos - 1).clamp_min(0)
    pos[~mask] = 0
    labels = torch.full((1, M * H), -100, dtype=torch.long)
    labels[:, -1] = ids.view(1, -1)[:, -1]
    layers = model.model.layers

    def ident(self, hidden_states, *a, **kw):
        return hidden_states

    for i in range(L + 1, len(layers)):
        layers[i].forward = ident.__get__(layers[i], type(layers[i]))
    model.lm_head.forward = ident.__get__(model.lm_head, type(model.lm_head))
    grabbed = {}

    def grab(mod, a, kw):
        grabbed["h"] = (a[0] if a else kw["hidden_states"]).detach().clone()

    hook = layers[L].register_forward_pre_hook(grab, with_kwargs=True)
    with torch.no_grad():
        out = model(input_ids=ids.view(1, -1), position_ids=pos.view(1, -1), attention_mask=mask,
                    output_attentions=True, layers_to_return_scores=[L])
    hook.remove()
    raw = out.attentions[0]
    logits = losses.compute_auxiliary_attention_loss(raw, labels, mask, None, return_logits=True)
    # a checksum of the seeded weights lets the test confirm it rebuilt the same model
    wsum = float(sum(p.double().abs().sum() for p in model.parameters()))
    np.savez_compressed(os.path.join(HERE, "tiny_mistral.npz"), input_ids=ids.view(1, -1).numpy(),
                        position_ids=pos.view(1, -1).numpy(), mask=mask.numpy(), labels=labels.numpy(),
                        raw=raw.numpy(), logits=logits.numpy(), hidden_in=grabbed["h"].numpy(),
                        score_layer=np.int64(L), weight_abs_sum=np.float64(wsum))
    print("tiny_mistral logits", logits)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    a = ap.parse_args()
    std = _load("ref_std", os.path.join(a.reference, "src", "blockrank", "blockrank_std_attention.py"))
    losses = _load("ref_losses", os.path.join(a.reference, "src", "blockrank", "losses.py"))
    with torch.no_grad():
        attn_case(std, losses, "attn_fp32_ragged", 21, B=2, N=4, Nk=2, D=64, M=5, H=32,
                  lens=[[20, 32, 1, 17, 9], [32, 5, 32, 30, 32]], dtype=torch.float32)
        attn_case(std, losses, "attn_bf16_ragged", 22, B=1, N=8, Nk=2, D=128, M=6, H=48,
                  lens=[[40, 48, 33, 7, 48, 21]], dtype=torch.bfloat16)
        attn_case(std, losses, "attn_fp32_m1", 23, B=1, N=2, Nk=1, D=64, M=1, H=16,
                  lens=[[11]], dtype=torch.float32)
        attn_case(std, losses, "attn_fp32_m2", 24, B=2, N=2, Nk=2, D=64, M=2, H=16,
                  lens=[[16, 9], [3, 16]], dtype=torch.float32)
        attn_case(std, losses, "attn_fp32_short_window", 25, B=1, N=2, Nk=1, D=64, M=4, H=16,
                  lens=[[5, 16, 2, 12]], dtype=torch.float32, num_last=4)
        # a grid narrower than the score window: the reference returns the last block's H rows (std:256-262)
        attn_case(std, losses, "attn_fp32_h8", 26, B=2, N=2, Nk=1, D=64, M=4, H=8,
                  lens=[[8, 3, 8, 6], [5, 8, 1, 8]], dtype=torch.float32)
        collate_case(a.reference)
        tiny_model_case(std, losses)


if __name__ == "__main__":
    main()
