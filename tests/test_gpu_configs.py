"""Parity of the CUDA path at the benchmarked geometries, and the device-side safety nets.

* op level, 100 documents x 160 tokens (the geometry bench.py times): tensor-core attention (16 key
  chunks of the query block, resident document blocks) and the score epilogue against the oracle;
* model level, one prompt of 64 + 20 x 160 + 48 tokens through the 7B-architecture runner (bf16,
  layers 0..20) against the fp32 oracle on the host, from the same weights;
* block shapes that take the other code paths of the tensor-core kernel (multi-slot prefix kept
  resident across documents, documents too long to be resident);
* status word: a bounded wait that runs out, malformed spans (nothing written: canaries), large
  finite values in padding slots of V.
"""
import ctypes as C

import pytest
import torch

from oracle import blockrank_oracle as orc
from tests import helpers as H_

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    from blockrank_b200 import BlockSpans, _lib, cuda_blockrank_attention_mask, ops
    from blockrank_b200.runner import MistralPrefillRanker, RankerConfig

SIMT, TC = 1, 2
N, NK, D = 32, 8, 128


def _packed_case(bl, seed, B=1):
    """Padding-free tensors for B copies of block lengths ``bl`` plus their padded-grid twin for the oracle."""
    start, ln, S, mbl = H_.packed_spans([bl] * B)
    g = torch.Generator().manual_seed(seed)
    qp = (torch.randn(B, S, N, D, generator=g) * 0.5).bfloat16()
    kp = (torch.randn(B, S, NK, D, generator=g) * 0.5).bfloat16()
    vp = (torch.randn(B, S, NK, D, generator=g) * 0.5).bfloat16()
    T, M = sum(bl), len(bl)
    Hp = -(-max(bl) // 16) * 16
    mask = H_.ragged_mask(B, M, Hp, [bl] * B)
    idx = H_.packed_to_padded(bl, Hp)
    pad = lambda t: torch.zeros(B, M * Hp, t.shape[2], D).index_copy_(1, idx, t[:, :T].float()).transpose(1, 2)
    return dict(start=start, ln=ln, S=S, mbl=mbl, T=T, M=M, Hp=Hp, mask=mask, idx=idx,
                qp=qp, kp=kp, vp=vp, qd=pad(qp), kd=pad(kp), vd=pad(vp))


def _check_against_oracle(c, B=1, canary=False):
    qc, kc, vc = (t.cuda().transpose(1, 2) for t in (c["qp"], c["kp"], c["vp"]))
    S, T, M, Hp, idx = c["S"], c["T"], c["M"], c["Hp"], c["idx"]
    scaling = D ** -0.5
    if canary:
        # output and log-sum-exp live inside larger buffers whose margins must come back untouched
        big = torch.full((B * S + 2 * S, N, D), 7.0, dtype=torch.bfloat16, device="cuda")
        out_buf = big[S:S + B * S].view(B, S, N, D)
        big_l = torch.full((B * N * S + 2048,), 7.0, dtype=torch.float32, device="cuda")
        lse_buf = big_l[1024:1024 + B * N * S].view(B, N, S)
        out, lse = ops.attention(qc, kc, vc, c["start"].cuda(), c["ln"].cuda(), scaling, c["mbl"], out=out_buf,
                                 lse=lse_buf, algo=TC, max_query_len=c["ln"][0, -1].item())
        ops.check_status()
        assert (big[:S] == 7.0).all() and (big[S + B * S:] == 7.0).all(), "attention wrote outside its output"
        assert (big_l[:1024] == 7.0).all() and (big_l[1024 + B * N * S:] == 7.0).all(), "lse written out of bounds"
    else:
        out = ops.attention(qc, kc, vc, c["start"].cuda(), c["ln"].cuda(), scaling, c["mbl"], algo=TC)
        ops.check_status()
    out = out.float().cpu()
    ref = orc.attention_blocked(c["qd"], c["kd"], c["vd"], c["mask"], scaling).float()  # fp32 math, bf16-rounded inputs
    err = (out[:, :T] - ref[:, idx]).abs().max().item()
    assert err < 2e-2, err
    assert out[:, T:].abs().sum().item() == 0
    rows = torch.tensor([[T - 2, T - 1]] * B, dtype=torch.int32)
    mass, logits = ops.doc_scores(qc, kc, c["start"].cuda(), c["ln"].cuda(), rows.cuda(), scaling)
    sig = torch.tensor([[M * Hp - 2, M * Hp - 1]] * B)
    exact = orc.doc_mass(c["qd"], c["kd"], c["mask"], scaling, sig)
    exact_logits = exact.mean(dim=(1, 2)) / 0.05
    assert torch.allclose(mass.cpu().double(), exact, rtol=1e-2, atol=1e-7)
    rel = ((logits.cpu().double() - exact_logits).abs() / exact_logits.abs()).max().item()
    assert rel < 1e-2, rel
    assert torch.equal(orc.topk_docs(logits.cpu()), orc.topk_docs(exact_logits.float()))
    return err, rel


def test_hundred_document_prompt_vs_oracle():
    """64 + 100 x 160 + 48 tokens, 32/8 heads, bf16, one prompt: the geometry the benchmark times.  The query
    block's context is cut into 16 key chunks; every document block runs with its K/V resident."""
    c = _packed_case([64] + [160] * 100 + [48], seed=12)
    err, rel = _check_against_oracle(c, canary=True)
    print(f"100-document prompt: attention max abs err {err:.3e}, logits max rel err {rel:.3e}")


@pytest.mark.parametrize("bl", [
    [130, 40, 200, 64, 129, 31, 190, 70],        # two-slot prefix kept resident across documents of 1..3 slots
    [64, 300, 33, 257, 160, 420, 48],            # documents too long to be resident take the streamed path
    [200, 250, 10, 96, 1, 128, 20],              # four-slot prefix: only one-slot documents fit beside it
    [64, 160, 160, 160, 160, 160, 160, 160, 160, 160, 5],   # more than one group of blocks per (prompt, KV head)
], ids=["kept-prefix", "streamed-docs", "wide-prefix", "groups"])
def test_block_shapes_vs_oracle(bl):
    c = _packed_case(bl, seed=sum(bl), B=2)
    _check_against_oracle(c, B=2, canary=True)


def test_many_blocks_grouped_with_resident_prefix():
    """Enough blocks (8 prompts x 8 KV heads x 111 blocks) for the kernel to hand them out in groups of
    consecutive blocks whose prefix K/V stays in shared memory from one block to the next: the tensor-core
    kernel against the CUDA-core kernel (itself checked against the oracle above)."""
    bl = [100] + [150, 64, 33, 160, 97] * 22 + [48]
    B = 8
    start, ln, S, mbl = H_.packed_spans([bl] * B)
    T = sum(bl)
    g = torch.Generator(device="cuda").manual_seed(8)
    mk = lambda h: (torch.randn(B, S, h, D, generator=g, device="cuda") * 0.5).bfloat16().transpose(1, 2)
    q, k, v = mk(N), mk(NK), mk(NK)
    o_tc = ops.attention(q, k, v, start.cuda(), ln.cuda(), D ** -0.5, mbl, algo=TC, max_query_len=48)
    o_si = ops.attention(q, k, v, start.cuda(), ln.cuda(), D ** -0.5, mbl, algo=SIMT)
    ops.check_status()
    assert (o_tc.float() - o_si.float())[:, :T].abs().max().item() < 2e-2


@pytest.mark.parametrize("algo", [SIMT, TC])
def test_long_gap_behind_the_last_block_is_zeroed(algo):
    """A batch padded to its longest prompt: the thousands of rows behind the short prompt's last block are zeroed in
    slices by many CTAs.  Every padding row must come back exactly zero (the output starts as NaN) and every valid
    row must agree with what the same prompt gives when it is run alone in a tight buffer."""
    bls = [[64] + [24] * 40 + [48], [64] + [160] * 40 + [48]]
    start, ln, S, mbl = H_.packed_spans(bls)
    g = torch.Generator(device="cuda").manual_seed(21)
    mk = lambda h: (torch.randn(2, S, h, D, generator=g, device="cuda") * 0.5).bfloat16().transpose(1, 2)
    q, k, v = mk(N), mk(NK), mk(NK)
    out = torch.full((2, S, N, D), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.attention(q, k, v, start.cuda(), ln.cuda(), D ** -0.5, mbl, out=out, algo=algo, max_query_len=48)
    ops.check_status()
    for b, bl in enumerate(bls):
        T = sum(bl)
        assert T < S or b == 1
        assert out[b, T:].float().abs().max().item() == 0 if T < S else True   # NaN would fail the comparison too
        st1, ln1, S1, mbl1 = H_.packed_spans([bl])
        solo = ops.attention(q[b:b + 1, :, :S1], k[b:b + 1, :, :S1], v[b:b + 1, :, :S1], st1.cuda(), ln1.cuda(), D ** -0.5,
                             mbl, algo=algo, max_query_len=48)
        ops.check_status()
        # (the query block's key chunks depend on the buffer length, so its rows may differ in the last bf16 bit)
        assert (out[b, :T].float() - solo[0, :T].float()).abs().max().item() < 1e-2


def test_large_finite_values_in_padding_slots_do_not_leak():
    """Keys outside a row's visible set get probability exactly zero, so finite garbage in the padding slots of
    K/V (here 1e30 behind every block of a padded grid) cannot reach a valid output row."""
    B, M, Hp = 1, 6, 96
    lens = [[70, 96, 33, 50, 96, 41]]
    mask = H_.ragged_mask(B, M, Hp, lens)
    q, k, v = H_.qkv(B, N, NK, M * Hp, D, 77, torch.bfloat16)
    scaling = D ** -0.5
    ref = orc.attention_blocked(q, k, v, mask, scaling).float()
    rows = mask.reshape(B, -1)
    k2, v2 = k.clone(), v.clone()
    k2.transpose(1, 2)[~rows] = 1e30
    v2.transpose(1, 2)[~rows] = 1e30
    start, ln = ops.spans_from_mask(mask.cuda())
    out = ops.attention(H_.to_cuda_view(q), H_.to_cuda_view(k2), H_.to_cuda_view(v2), start, ln, scaling, Hp, algo=TC)
    out = out.float().cpu()
    assert torch.isfinite(out).all()
    assert (out - ref)[rows].abs().max().item() < 2e-2


def _hf_weights(rk):
    """The ranker's fused device weights under their HF parameter names, converted to fp32 on the host on access."""
    c = rk.cfg
    qd, kd, inter = c.num_attention_heads * c.head_dim, c.num_key_value_heads * c.head_dim, c.intermediate_size

    class W:
        def __getitem__(self, name):
            if name == "model.embed_tokens.weight":
                return rk.embed.float().cpu()
            _, _, i, *rest = name.split(".")
            L, key = rk.layers[int(i)], ".".join(rest)
            pick = {
                "input_layernorm.weight": lambda: L["ln1"],
                "post_attention_layernorm.weight": lambda: L["ln2"],
                "self_attn.q_proj.weight": lambda: L["wqkv"][:qd] if "wqkv" in L else L["wq"],
                "self_attn.k_proj.weight": lambda: L["wqkv"][qd:qd + kd] if "wqkv" in L else L["wk"],
                "self_attn.v_proj.weight": lambda: L["wqkv"][qd + kd:],
                "self_attn.o_proj.weight": lambda: L["wo"],
                "mlp.gate_proj.weight": lambda: L["wgu"][:inter],
                "mlp.up_proj.weight": lambda: L["wgu"][inter:],
                "mlp.down_proj.weight": lambda: L["wd"],
            }[key]
            return pick().float().cpu()
    return W()


def test_7b_architecture_prompt_vs_fp32_oracle():
    """One prompt of 64 + 20 x 160 + 48 tokens through layers 0..20 of the Mistral-7B architecture (hidden 4096,
    32/8 heads, MLP 14336, random weights N(0, 0.02) rounded to bf16) against the fp32 oracle on the host reading
    the same weights (scripts/eval_attn.py:135-151 is the loop being reproduced).

    Random weights give nearly uniform document scores (logits 1.0 +- 0.05 with gaps down to 1e-4 between
    neighbours), so two statements are checked:
      * the runner in fp32 (the kernels' fp32 paths, same weights): logits within 1e-3 relative of the oracle, a tenth
        of the per-document tolerance.  Twenty random-weight layers amplify the summation-order differences between
        the host's CPU GEMMs and cuBLAS: 3.4e-6 on most hosts, 1.2e-4 seen on one (the bf16 figure against the same
        oracle moved in its fourth digit on that host too, while the one-layer check below did not), so the bound
        is not the 1e-4 of a single attention call;
      * the runner in bf16 (tensor-core attention, bf16 GEMMs): its scoring layer within 1e-2 relative of the oracle
        scoring the SAME hidden state (the per-document tolerance on identical inputs), and end to end within 3e-2 of
        the fp32 oracle (20 layers of bf16 rounding, which the reference's own bf16 run carries as well);
      * for both, the top-10 order: identical whenever the oracle's smallest gap among its top 11 exceeds four
        times the run's largest logit error; otherwise (printed as NEAR TIE) a differing position must hold two
        documents whose oracle scores are closer than twice that error -- the oracle's order up to ties the
        arithmetic cannot resolve."""
    cfg = RankerConfig.mistral_7b(20)
    rk = MistralPrefillRanker(cfg, "cuda", torch.bfloat16).init_random(seed=3)
    bl = [64] + [160] * 20 + [48]
    M, Hp, T = len(bl), 160, sum(bl)
    g = torch.Generator().manual_seed(4)
    ids_p = torch.randint(3, 32768, (1, T), generator=g)
    start, ln, S, mbl = H_.packed_spans([bl])
    ids = torch.zeros(1, S, dtype=torch.long)
    ids[:, :T] = ids_p
    pos = torch.zeros(1, S, dtype=torch.long)
    off = 0
    for m, n in enumerate(bl):
        base = 0 if m == 0 else (16384 if m == M - 1 else bl[0])
        pos[0, off:off + n] = base + torch.arange(n)
        off += n
    rows = torch.tensor([[T - 2, T - 1]], dtype=torch.int32)
    args = (ids.cuda(), pos.cuda(), start.cuda(), ln.cuda(), mbl, rows.cuda())
    h20 = rk.hidden_before_score_layer(*args[:5], bl[-1])                  # residual stream entering layer 20 (bf16)
    logits16, _ = rk.score_from_hidden(h20, args[1], args[2], args[3], args[5])
    ops.check_status()
    logits16 = logits16.float().cpu()
    # the same weights, upcast, through the fp32 paths of the same runner
    rk32 = MistralPrefillRanker(cfg, "cuda", torch.float32)
    rk32.embed = rk.embed.float()
    rk32.layers = [{k: v.float() for k, v in L.items()} for L in rk.layers]
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        logits32, _ = rk32.score(*args, max_query_len=bl[-1])
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    ops.check_status()
    logits32 = logits32.float().cpu()
    # the same prompt on the reference's left-padded (M, H) grid for the oracle
    idx = H_.packed_to_padded(bl, Hp)
    mask = H_.ragged_mask(1, M, Hp, [bl])
    ids_d = torch.zeros(1, M * Hp, dtype=torch.long).index_copy_(1, idx, ids_p)
    pos_d = torch.zeros(1, M * Hp, dtype=torch.long).index_copy_(1, idx, pos[:, :T])
    labels = torch.full((1, M * Hp), -100, dtype=torch.long)
    labels[:, -1] = 7
    ocfg = {"n_heads": 32, "n_kv_heads": 8, "head_dim": 128, "rope_theta": cfg.rope_theta, "rms_eps": cfg.rms_norm_eps}
    del rk32
    with torch.no_grad():
        ref, _, _ = orc.mistral_prefill_scores(_hf_weights(rk), ocfg, ids_d, pos_d, mask, labels, 20)
    ref = ref.float()
    srt = ref.sort(-1, descending=True).values
    gap = (srt[:, :10] - srt[:, 1:11]).min().item()
    rel32 = ((logits32 - ref).abs() / ref.abs()).max().item()
    rel16 = ((logits16 - ref).abs() / ref.abs()).max().item()
    err16 = (logits16 - ref).abs().max().item()
    err32 = (logits32 - ref).abs().max().item()
    top_ref, top32, top16 = orc.topk_docs(ref)[0], orc.topk_docs(logits32)[0], orc.topk_docs(logits16)[0]

    def same_order(top, err, what):
        """Identical top-10 where the oracle separates neighbours by more than the arithmetic's error; where it
        does not (a tie for that precision), a position may hold the other document of the tie."""
        swaps = [(int(a), int(b)) for a, b in zip(top, top_ref) if a != b]
        print(f"  {what}: logit error {err:.3e}; oracle's smallest gap in its top 11 {gap:.3e}; "
              f"{'well separated' if gap > 4 * err else 'NEAR TIE for this precision'}; differing positions {swaps}")
        if gap > 4 * err:
            assert not swaps, swaps
        for a, b in swaps:
            assert abs(ref[0, a].item() - ref[0, b].item()) < 2 * err, (what, a, b, ref[0, a].item(), ref[0, b].item(), err)

    # the scoring layer alone on identical input: the oracle's layer-20 scoring of the hidden state the bf16 run produced
    w = _hf_weights(rk)
    hd = torch.zeros(1, M * Hp, cfg.hidden_size).index_copy_(1, idx, h20.float().cpu()[None, :T])
    p20 = "model.layers.20."
    xq = orc.rms_norm(hd, w[p20 + "input_layernorm.weight"], cfg.rms_norm_eps)
    cos, sin = orc.rope_tables(pos_d, 128, cfg.rope_theta)
    q20 = orc.apply_rope((xq @ w[p20 + "self_attn.q_proj.weight"].T).view(1, M * Hp, 32, 128).transpose(1, 2), cos, sin)
    k20 = orc.apply_rope((xq @ w[p20 + "self_attn.k_proj.weight"].T).view(1, M * Hp, 8, 128).transpose(1, 2), cos, sin)
    sig = torch.tensor([[M * Hp - 2, M * Hp - 1]])
    ref20 = (orc.doc_mass(q20, k20, mask, 128 ** -0.5, sig).mean(dim=(1, 2)) / 0.05).float()
    rel20 = ((logits16 - ref20).abs() / ref20.abs()).max().item()
    err20 = (logits16 - ref20).abs().max().item()
    print(f"7B-architecture prompt: fp32 run vs oracle: logits max rel err {rel32:.3e}; bf16 run vs fp32 oracle end to end "
          f"{rel16:.3e}; bf16 scoring layer vs the oracle on the same hidden state {rel20:.3e}")
    assert rel32 < 1e-3, rel32
    same_order(top32, err32, "fp32 runner")
    assert rel20 < 1e-2, rel20          # the per-document score tolerance, on identical inputs
    top20 = orc.topk_docs(ref20)[0]
    for a_, b_ in [(int(a_), int(b_)) for a_, b_ in zip(top16, top20) if a_ != b_]:
        assert abs(ref20[0, a_].item() - ref20[0, b_].item()) < 2 * err20, (a_, b_, err20)
    # end to end the bf16 run carries the rounding of 20 decoder layers (about 1 % of the residual stream per layer,
    # as bench.py's parity line shows for one layer); 3e-2 bounds that accumulation, it is not an op tolerance
    assert rel16 < 3e-2, rel16
    same_order(top16, err16, "bf16 runner, end to end")


def test_bounded_wait_gives_up_and_is_reported():
    """A wait that runs out sets the status word and the kernel returns; the host sees BRK_E_TIMEOUT at its next
    poll, the word is cleared, and the next attention call is unaffected."""
    L = _lib.lib()
    ops.check_status()
    w = ops.status_word("cuda")
    rc = L.brk_selftest_bounded_wait(w.data_ptr(), 1024, torch.cuda.current_stream().cuda_stream)
    assert rc == 0, L.brk_last_error()
    with pytest.raises(_lib.BlockRankLibraryError, match="BRK_E_TIMEOUT"):
        ops.check_status()
    assert int(w.item()) == 0
    ops.check_status()
    c = _packed_case([64, 100, 48], seed=5)
    _check_against_oracle(c)


@pytest.mark.parametrize("algo", [SIMT, TC])
def test_malformed_spans_write_nothing_and_are_reported(algo):
    bl = [64, 100, 48]
    c = _packed_case(bl, seed=6)
    qc, kc, vc = (t.cuda().transpose(1, 2) for t in (c["qp"], c["kp"], c["vp"]))
    S = c["S"]
    for bad in ("past-the-end", "overlap", "too-long", "negative"):
        start, ln = c["start"].clone(), c["ln"].clone()
        if bad == "past-the-end":
            start[0, 2] = S - 10          # 48 tokens from S-10
        elif bad == "overlap":
            start[0, 1] = 10              # inside block 0
        elif bad == "too-long":
            ln[0, 1] = c["mbl"] + 1
        else:
            start[0, 0] = -4
        big = torch.full((3 * S, N, D), 7.0, dtype=torch.bfloat16, device="cuda")
        out = big[S:2 * S].view(1, S, N, D)
        ops.attention(qc, kc, vc, start.cuda(), ln.cuda(), D ** -0.5, c["mbl"], out=out, algo=algo)
        with pytest.raises(ValueError, match="malformed block spans"):
            ops.check_status()
        assert (big == 7.0).all(), bad
    ops.check_status()


def test_int32_block_mask_with_two_prompts_is_a_mask():
    """An int32 0/1 (B=2, M, H) block mask is a block mask, not a (2, B, M) pair of span arrays."""
    mask = H_.ragged_mask(2, 3, 16, [[16, 5, 9], [3, 16, 16]])
    spans = cuda_blockrank_attention_mask(attention_mask=mask.to(torch.int32).cuda())
    assert isinstance(spans, BlockSpans) and spans.shape == (2, 2, 3) and spans.grid_h == 16
    start, ln = orc.block_spans(mask)
    assert torch.equal(spans[0].cpu(), start) and torch.equal(spans[1].cpu(), ln)
