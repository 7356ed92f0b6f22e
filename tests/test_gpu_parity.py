"""GPU parity: the CUDA kernels, called through the C ABI, against the CPU oracle and the
fixtures generated from the reference.  Tolerances: fp32 1e-4 abs, bf16 2e-2 abs on attention
outputs (valid rows), 1e-2 relative on per-document scores, identical top-10 order."""
import os

import numpy as np
import pytest
import torch

from oracle import blockrank_oracle as orc
from tests import helpers as H_

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    from blockrank_b200 import _lib, ops

SIMT, TC = 1, 2


def _load(golden_dir, name):
    z = np.load(os.path.join(golden_dir, name + ".npz"))
    return {k: z[k] for k in z.files}


def _spans_cuda(mask):
    return ops.spans_from_mask(mask.cuda())


def _run_attn(q, k, v, mask, scaling, algo, lse=False):
    start, ln = _spans_cuda(mask)
    res = ops.attention(H_.to_cuda_view(q), H_.to_cuda_view(k), H_.to_cuda_view(v), start, ln, scaling,
                        mask.shape[-1], return_lse=lse, algo=algo)
    torch.cuda.synchronize()
    return res


def test_library_loads_on_device():
    L = _lib.lib()
    assert L.brk_version() >= 101
    assert L.brk_device_check() == 0, L.brk_last_error()


def test_spans_match_oracle():
    lens = H_.random_lens(3, 7, 48, seed=5)
    lens[1][2] = 0
    mask = H_.ragged_mask(3, 7, 48, lens)
    s, l = _spans_cuda(mask)
    es, el = orc.block_spans(mask)
    assert torch.equal(l.cpu(), el) and torch.equal(s.cpu()[el > 0], es[el > 0])


@pytest.mark.parametrize("name,algo", [("attn_fp32_ragged", SIMT), ("attn_fp32_m1", SIMT), ("attn_fp32_m2", SIMT),
                                       ("attn_fp32_short_window", SIMT), ("attn_bf16_ragged", SIMT),
                                       ("attn_bf16_ragged", TC)])
def test_attention_vs_reference_fixture(golden_dir, name, algo):
    fx = _load(golden_dir, name)
    bf16 = str(fx["dtype"]) == "bfloat16"
    dt = torch.bfloat16 if bf16 else torch.float32
    q, k, v = (torch.from_numpy(fx[n]).to(dt) for n in "qkv")
    mask = torch.from_numpy(fx["mask"])
    out = _run_attn(q, k, v, mask, float(fx["scaling"]), algo).float().cpu()
    rows = mask.reshape(mask.shape[0], -1)
    err = (out - torch.from_numpy(fx["out"]))[rows].abs().max().item()
    assert err < (2e-2 if bf16 else 1e-4), err
    assert out[~rows].abs().max().item() == 0 if (~rows).any() else True


CASES = [  # B, N, Nk, D, M, H, seed
    (2, 4, 2, 64, 5, 32, 1), (1, 8, 2, 128, 4, 80, 2), (2, 8, 8, 64, 3, 16, 3), (1, 4, 1, 128, 6, 48, 4),
    (1, 8, 1, 64, 3, 40, 5), (2, 4, 4, 128, 1, 64, 6), (2, 4, 2, 128, 2, 64, 7),
]


@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_attention_simt_vs_oracle(case, dt):
    B, N, Nk, D, M, H, seed = case
    lens = H_.random_lens(B, M, H, seed)
    mask = H_.ragged_mask(B, M, H, lens)
    q, k, v = H_.qkv(B, N, Nk, M * H, D, seed + 100, dt)
    out, lse = _run_attn(q, k, v, mask, D ** -0.5, SIMT, lse=True)
    ref, ref_lse = orc.attention_dense(q, k, v, mask, D ** -0.5)
    rows = mask.reshape(B, -1)
    err = (out.float().cpu() - ref.float())[rows].abs().max().item()
    assert err < (2e-2 if dt == torch.bfloat16 else 1e-4), err
    lrows = rows[:, None, :].expand(B, N, M * H)
    assert (lse.cpu() - ref_lse.float())[lrows].abs().max().item() < 1e-3
    assert out.float().cpu()[~rows].abs().sum().item() == 0


TC_CASES = [  # B, N, Nk, M, H, seed  (head_dim 128)
    (1, 4, 1, 3, 64, 11), (2, 8, 2, 5, 80, 12), (1, 8, 2, 4, 160, 13), (1, 4, 4, 4, 96, 14), (1, 8, 4, 3, 48, 15),
    (1, 8, 1, 3, 32, 16), (2, 4, 1, 1, 128, 17), (2, 4, 1, 2, 72, 18), (1, 32, 8, 12, 160, 19),
    (2, 8, 2, 40, 64, 20), (1, 4, 1, 3, 1024, 21),
]


@pytest.mark.parametrize("case", TC_CASES)
def test_attention_tc_vs_oracle(case):
    B, N, Nk, M, H, seed = case
    D = 128
    lens = H_.random_lens(B, M, H, seed)
    mask = H_.ragged_mask(B, M, H, lens)
    q, k, v = H_.qkv(B, N, Nk, M * H, D, seed + 100, torch.bfloat16)
    out, lse = _run_attn(q, k, v, mask, D ** -0.5, TC, lse=True)
    ref, ref_lse = orc.attention_dense(q, k, v, mask, D ** -0.5)
    rows = mask.reshape(B, -1)
    err = (out.float().cpu() - ref.float())[rows].abs().max().item()
    assert err < 2e-2, err
    lrows = rows[:, None, :].expand(B, N, M * H)
    assert (lse.cpu() - ref_lse.float())[lrows].abs().max().item() < 2e-3
    assert out.float().cpu()[~rows].abs().sum().item() == 0


@pytest.mark.parametrize("algo", [SIMT, TC])
def test_attention_large_logit_range(algo):
    """Logits spread over tens of units (queries scaled up): the running maximum jumps by more than the
    lazy-rescale threshold between key slots, so the paths that rescale O -- and, inside a 128-key tile,
    the P already written for its first slot -- are exercised; the softmax is nearly one-hot."""
    B, N, Nk, D, M, H = 1, 8, 2, 128, 5, 160
    lens = H_.random_lens(B, M, H, 31)
    lens[0][0], lens[0][-1] = 150, 130      # several key slots in the prefix and in the query block
    mask = H_.ragged_mask(B, M, H, lens)
    q, k, v = H_.qkv(B, N, Nk, M * H, D, 131, torch.bfloat16)
    q = (q.float() * 32).to(torch.bfloat16)
    out, lse = _run_attn(q, k, v, mask, D ** -0.5, algo, lse=True)
    ref, ref_lse = orc.attention_dense(q, k, v, mask, D ** -0.5)
    rows = mask.reshape(B, -1)
    assert torch.isfinite(out.float()).all()
    err = (out.float().cpu() - ref.float())[rows].abs().max().item()
    assert err < 3e-2, err
    lrows = rows[:, None, :].expand(B, N, M * H)
    assert (lse.cpu() - ref_lse.float())[lrows].abs().max().item() < 2e-2


def test_attention_tc_matches_simt_full_blocks():
    """Uniform full blocks at the standalone-op geometry (one prompt): both kernels, same inputs."""
    B, N, Nk, D = 1, 32, 8, 128
    M, H = 22, 160
    lens = [[64] + [160] * 20 + [48]]
    mask = H_.ragged_mask(B, M, H, lens)
    q, k, v = H_.qkv(B, N, Nk, M * H, D, 2, torch.bfloat16)
    a = _run_attn(q, k, v, mask, D ** -0.5, SIMT).float()
    b = _run_attn(q, k, v, mask, D ** -0.5, TC).float()
    assert (a - b).abs().max().item() < 2e-2


@pytest.mark.parametrize("algo", [SIMT, TC])
def test_attention_packed_layout_equals_padded(algo):
    """Padding-free spans give the same valid rows as the reference's left-padded grid."""
    B, N, Nk, D = 2, 8, 2, 128
    blens = [[20, 33, 7, 48, 15], [31, 48, 48, 1, 9]]
    Hp = 48
    start, ln, S, mbl = H_.packed_spans(blens)
    g = torch.Generator().manual_seed(77)
    qp = (torch.randn(B, S, N, D, generator=g) * 0.5).bfloat16()
    kp = (torch.randn(B, S, Nk, D, generator=g) * 0.5).bfloat16()
    vp = (torch.randn(B, S, Nk, D, generator=g) * 0.5).bfloat16()
    out = ops.attention(qp.cuda().transpose(1, 2), kp.cuda().transpose(1, 2), vp.cuda().transpose(1, 2),
                        start.cuda(), ln.cuda(), D ** -0.5, mbl, algo=algo).float().cpu()
    M = len(blens[0])
    mask = H_.ragged_mask(B, M, Hp, blens)
    qd = torch.zeros(B, M * Hp, N, D); kd = torch.zeros(B, M * Hp, Nk, D); vd = torch.zeros(B, M * Hp, Nk, D)
    for b in range(B):
        idx = H_.packed_to_padded(blens[b], Hp)
        n = idx.numel()
        qd[b, idx], kd[b, idx], vd[b, idx] = qp[b, :n].float(), kp[b, :n].float(), vp[b, :n].float()
    ref, _ = orc.attention_dense(qd.transpose(1, 2), kd.transpose(1, 2), vd.transpose(1, 2), mask, D ** -0.5)
    for b in range(B):
        idx = H_.packed_to_padded(blens[b], Hp)
        n = idx.numel()
        assert (out[b, :n] - ref[b, idx].float()).abs().max().item() < 2e-2
        assert out[b, n:].abs().sum().item() == 0


@pytest.mark.parametrize("name", ["attn_fp32_ragged", "attn_bf16_ragged", "attn_fp32_short_window", "attn_fp32_m2",
                                  "attn_fp32_h8"])
def test_raw_scores_vs_reference_fixture(golden_dir, name):
    fx = _load(golden_dir, name)
    bf16 = str(fx["dtype"]) == "bfloat16"
    dt = torch.bfloat16 if bf16 else torch.float32
    q, k = torch.from_numpy(fx["q"]).to(dt), torch.from_numpy(fx["k"]).to(dt)
    mask = torch.from_numpy(fx["mask"])
    start, ln = _spans_cuda(mask)
    raw = ops.raw_scores(H_.to_cuda_view(q), H_.to_cuda_view(k), start, ln, float(fx["scaling"]), int(fx["num_last"]),
                         grid_h=mask.shape[-1])   # the window never reaches past the last block's H grid slots
    raw = raw.float().cpu()
    ref = torch.from_numpy(fx["raw"])
    assert raw.shape == ref.shape
    live = ref > -1e30
    assert torch.equal(live, raw > -1e30)
    assert (raw - ref)[live].abs().max().item() < (6e-2 if bf16 else 1e-4)
    assert torch.allclose(raw[~live], ref[~live], rtol=1e-2)


@pytest.mark.parametrize("name", ["attn_fp32_ragged", "attn_bf16_ragged", "attn_fp32_short_window"])
def test_doc_scores_vs_reference_fixture(golden_dir, name):
    fx = _load(golden_dir, name)
    bf16 = str(fx["dtype"]) == "bfloat16"
    dt = torch.bfloat16 if bf16 else torch.float32
    q, k = torch.from_numpy(fx["q"]).to(dt), torch.from_numpy(fx["k"]).to(dt)
    mask = torch.from_numpy(fx["mask"])
    B, M, H = mask.shape
    S = M * H
    start, ln = _spans_cuda(mask)
    rows = torch.tensor([[S - 2, S - 1]] * B, dtype=torch.int32).cuda()
    mass, logits = ops.doc_scores(H_.to_cuda_view(q), H_.to_cuda_view(k), start, ln, rows, float(fx["scaling"]))
    ref = torch.from_numpy(fx["logits"])
    exact = orc.doc_mass(q, k, mask, float(fx["scaling"]), rows.cpu().long())
    assert torch.allclose(mass.cpu().double(), exact, rtol=1e-3, atol=1e-6)
    # Logits: the bar is 1e-2 relative.  The kernel is held to 1e-3 of the fp64 closed form; the reference's own
    # logits (made from raw scores rounded to the working dtype) are further from it in bf16, which is logged, and
    # the distance between the two must be explained by the reference's distance plus ours.
    exact_logits = exact.mean(dim=(1, 2)) / 0.05
    ours_rel = ((logits.cpu().double() - exact_logits).abs() / exact_logits.abs()).max().item()
    ref_rel = ((ref.double() - exact_logits).abs() / exact_logits.abs()).max().item()
    print(f"{name}: logits vs fp64 closed form: kernel {ours_rel:.2e}, reference fixture {ref_rel:.2e}")
    assert ours_rel < 1e-3
    assert ref_rel < (1e-2 if bf16 else 1e-4)
    assert ((logits.cpu().double() - ref.double()).abs() <= (ref_rel + 1e-3) * exact_logits.abs() + 1e-6).all()
    assert torch.allclose(mass.sum(-1).cpu(), torch.ones(B, q.shape[1], 2), atol=1e-5)


def test_doc_scores_many_rows_and_empty_doc():
    B, N, Nk, D, M, H = 2, 8, 2, 128, 9, 32
    lens = H_.random_lens(B, M, H, 31)
    lens[0][3] = 0
    lens[0][-1] = lens[1][-1] = H
    mask = H_.ragged_mask(B, M, H, lens)
    q, k, _ = H_.qkv(B, N, Nk, M * H, D, 131, torch.bfloat16)
    start, ln = _spans_cuda(mask)
    S = M * H
    rows = torch.arange(S - 5, S, dtype=torch.int32).expand(B, 5).contiguous()
    mass, logits = ops.doc_scores(H_.to_cuda_view(q), H_.to_cuda_view(k), start, ln, rows.cuda(), D ** -0.5, 0.05)
    exact = orc.doc_mass(q, k, mask, D ** -0.5, rows.long())
    assert torch.allclose(mass.cpu().double(), exact, rtol=1e-3, atol=1e-7)
    assert mass[0, :, :, 2].abs().sum().item() == 0
    assert torch.allclose(logits.cpu().double(), exact.mean(dim=(1, 2)) / 0.05, rtol=1e-3)


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float32])
def test_doc_scores_long_list(dt):
    """More documents than one warp keeps in registers (> 256): masses and logits of a 300-document list."""
    B, N, Nk, D, H = 2, 8, 2, 64, 8
    M = 302
    lens = H_.random_lens(B, M, H, 77)
    lens[1][40] = 0
    mask = H_.ragged_mask(B, M, H, lens)
    q, k, _ = H_.qkv(B, N, Nk, M * H, D, 78, dt)
    start, ln = _spans_cuda(mask)
    S = M * H
    rows = torch.tensor([[S - 2, S - 1]] * B, dtype=torch.int32)
    mass, logits = ops.doc_scores(H_.to_cuda_view(q), H_.to_cuda_view(k), start, ln, rows.cuda(), D ** -0.5, 0.05)
    exact = orc.doc_mass(q, k, mask, D ** -0.5, rows.long())
    assert torch.allclose(mass.cpu().double(), exact, rtol=1e-3, atol=1e-8)
    assert torch.allclose(logits.cpu().double(), exact.mean(dim=(1, 2)) / 0.05, rtol=1e-3, atol=1e-8)
    assert torch.allclose(mass.sum(-1).cpu(), torch.ones(B, N, 2), atol=1e-5)


def test_error_codes():
    q, k, v = H_.qkv(1, 4, 2, 32, 96, 1, torch.bfloat16)  # head_dim 96 unsupported
    mask = H_.ragged_mask(1, 2, 16, [[16, 16]])
    with pytest.raises(ValueError, match="head_dim"):
        _run_attn(q, k, v, mask, 0.1, SIMT)
    q, k, v = H_.qkv(1, 4, 2, 32, 64, 1, torch.float32)
    with pytest.raises(ValueError, match="bf16"):
        _run_attn(q, k, v, mask, 0.1, TC)
    with pytest.raises(RuntimeError, match="CUDA tensors"):
        ops.spans_from_mask(mask)


def test_tc_attention_needs_its_workspace():
    """The tensor-core path reports a workspace size and refuses to run without it (status, no launch)."""
    import ctypes as C
    B, N, Nk, D, M, H = 1, 4, 1, 128, 3, 64
    mask = H_.ragged_mask(B, M, H, [[64, 40, 30]])
    q, k, v = (H_.to_cuda_view(t) for t in H_.qkv(B, N, Nk, M * H, D, 3, torch.bfloat16))
    start, ln = _spans_cuda(mask)
    out = torch.empty(B, M * H, N, D, dtype=torch.bfloat16, device="cuda")
    p = _lib.AttnParams()
    p.dtype, p.algo = 0, TC
    p.B, p.N, p.Nk, p.D, p.S, p.M, p.max_block_len, p.scale = B, N, Nk, D, M * H, M, H, D ** -0.5
    p.q, p.k, p.v, p.o = ops._view(q), ops._view(k), ops._view(v), ops._view(out.permute(0, 2, 1, 3))
    p.lse, p.status = None, None
    p.blk_start, p.blk_len = start.data_ptr(), ln.data_ptr()
    L = _lib.lib()
    need = L.brk_attn_fwd_workspace_bytes(C.byref(p))
    assert need >= 256
    rc = L.brk_attn_fwd(C.byref(p), None, 0, None)
    assert rc == -3 and b"workspace" in L.brk_last_error()
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    assert L.brk_attn_fwd(C.byref(p), ws.data_ptr(), need - 1, None) == -3
    assert L.brk_attn_fwd(C.byref(p), ws.data_ptr(), need, None) == 0
    torch.cuda.synchronize()
    ref, _ = orc.attention_dense(q.cpu(), k.cpu(), v.cpu(), mask, D ** -0.5)
    rows = mask.reshape(B, -1)
    assert (out.float().cpu() - ref.float())[rows].abs().max().item() < 2e-2


def test_standalone_op_config_parity():
    """The standalone-op configuration: B4, 32/8 heads, D128, 64 + 20x160 + 48 tokens, bf16; O and [4,32,20] scores."""
    B, N, Nk, D = 4, 32, 8, 128
    blens = [[64] + [160] * 20 + [48]] * B
    M, Hp = 22, 160
    mask = H_.ragged_mask(B, M, Hp, blens)
    q, k, v = H_.qkv(B, N, Nk, M * Hp, D, 2, torch.bfloat16)
    scaling = D ** -0.5
    ref = orc.attention_blocked(q, k, v, mask, scaling).float()      # fp32 math on the bf16-rounded inputs
    rows = mask.reshape(B, -1)
    S = M * Hp
    sig = torch.tensor([[S - 2, S - 1]] * B)
    exact = orc.doc_mass(q, k, mask, scaling, sig)                   # (4,32,2,20)
    exact_logits = exact.mean(dim=(1, 2)) / 0.05
    start, ln = _spans_cuda(mask)
    qc, kc, vc = (H_.to_cuda_view(t) for t in (q, k, v))
    for algo in (SIMT, TC):
        out = ops.attention(qc, kc, vc, start, ln, scaling, Hp, algo=algo).float().cpu()
        assert (out - ref)[rows].abs().max().item() < 2e-2
    mass, logits = ops.doc_scores(qc, kc, start, ln, sig.int().cuda(), scaling)
    per_head = mass.mean(2).cpu().double()                           # [4,32,20]
    assert torch.allclose(per_head, exact.mean(2), rtol=1e-2)
    rel = ((logits.cpu().double() - exact_logits).abs() / exact_logits.abs()).max().item()
    assert rel < 1e-2, rel
    top_k, top_r = orc.topk_docs(logits.cpu()), orc.topk_docs(exact_logits.float())
    srt = exact_logits.sort(-1, descending=True).values
    gap = (srt[:, :10] - srt[:, 1:11]).min().item()
    err = (logits.cpu().double() - exact_logits).abs().max().item()
    print(f"standalone-op scores: max abs err {err:.3e}, min adjacent gap in top-11 {gap:.3e}")
    # identical top-10 where the oracle separates neighbours by more than twice the run's error; in any case the
    # document ranked p-th by the kernel must be worth the oracle's p-th value up to that error (ties only)
    if gap > 2 * err:
        assert torch.equal(top_k, top_r), (gap, err)
    got_vals = exact_logits.gather(1, top_k.long())
    assert bool((got_vals >= srt[:, :10] - 2 * err).all()), (gap, err)


def _ragged_prompt(n_docs, seed, lo=32, hi=256):
    g = torch.Generator().manual_seed(seed)
    return [64] + torch.randint(lo, hi + 1, (n_docs,), generator=g).tolist() + [48]


def test_ragged_long_list_packed_vs_oracle():
    """Reduced ragged long-list case (60 documents of 32..256 tokens, padding-free layout): the
    tcgen05 kernel against the oracle run on the reference's padded grid built from the same tokens."""
    N, Nk, D = 32, 8, 128
    bl = _ragged_prompt(60, seed=5)
    start, ln, S, mbl = H_.packed_spans([bl])
    g = torch.Generator().manual_seed(55)
    qp = (torch.randn(1, S, N, D, generator=g) * 0.5).bfloat16()
    kp = (torch.randn(1, S, Nk, D, generator=g) * 0.5).bfloat16()
    vp = (torch.randn(1, S, Nk, D, generator=g) * 0.5).bfloat16()
    qc, kc, vc = (t.cuda().transpose(1, 2) for t in (qp, kp, vp))
    out = ops.attention(qc, kc, vc, start.cuda(), ln.cuda(), D ** -0.5, mbl, algo=TC).float().cpu()
    T = sum(bl)
    rows = torch.tensor([[T - 2, T - 1]], dtype=torch.int32)
    mass, logits = ops.doc_scores(qc, kc, start.cuda(), ln.cuda(), rows.cuda(), D ** -0.5)
    M, Hp = len(bl), 256
    mask = H_.ragged_mask(1, M, Hp, [bl])
    idx = H_.packed_to_padded(bl, Hp)
    qd = torch.zeros(1, M * Hp, N, D); kd = torch.zeros(1, M * Hp, Nk, D); vd = torch.zeros(1, M * Hp, Nk, D)
    qd[0, idx], kd[0, idx], vd[0, idx] = qp[0, :T].float(), kp[0, :T].float(), vp[0, :T].float()
    ref = orc.attention_blocked(qd.transpose(1, 2), kd.transpose(1, 2), vd.transpose(1, 2), mask, D ** -0.5)
    assert (out[0, :T] - ref[0, idx].float()).abs().max().item() < 2e-2
    assert out[0, T:].abs().sum().item() == 0
    sig = torch.tensor([[M * Hp - 2, M * Hp - 1]])
    exact = orc.doc_mass(qd.transpose(1, 2), kd.transpose(1, 2), mask, D ** -0.5, sig)
    assert torch.allclose(mass.cpu().double(), exact, rtol=2e-3, atol=1e-7)


def test_full_size_ragged_long_list_properties():
    """The ragged long-list geometry at full size (500 documents of 32..256 tokens, ~72k tokens, one
    prompt): size-independent properties instead of an oracle run --
    (1) the tensor-core and CUDA-core kernels agree; (2) each row's document masses sum to one;
    (3) swapping two documents (moving their Q/K/V rows) moves their outputs and scores with them."""
    N, Nk, D = 32, 8, 128
    bl = _ragged_prompt(500, seed=5)
    start, ln, S, mbl = H_.packed_spans([bl])
    T = sum(bl)
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(5)
    mk = lambda h: (torch.randn(1, S, h, D, generator=g, device=dev) * 0.5).bfloat16()
    q, k, v = mk(N), mk(Nk), mk(Nk)
    sc, lc = start.cuda(), ln.cuda()
    run = lambda qq, kk, vv, s_, l_, algo: ops.attention(qq.transpose(1, 2), kk.transpose(1, 2), vv.transpose(1, 2),
                                                        s_, l_, D ** -0.5, mbl, algo=algo)
    o_tc = run(q, k, v, sc, lc, TC)
    o_si = run(q, k, v, sc, lc, SIMT)
    assert (o_tc.float() - o_si.float())[0, :T].abs().max().item() < 2e-2
    rows = torch.tensor([[T - 2, T - 1]], dtype=torch.int32, device=dev)
    mass, logits = ops.doc_scores(q.transpose(1, 2), k.transpose(1, 2), sc, lc, rows, D ** -0.5)
    assert torch.allclose(mass.sum(-1), torch.ones_like(mass.sum(-1)), atol=1e-4)
    # swap documents 7 and 311 (block indices 8 and 312)
    i, j = 8, 312
    order = list(range(len(bl)))
    order[i], order[j] = order[j], order[i]
    bl2 = [bl[m] for m in order]
    start2, ln2, S2, _ = H_.packed_spans([bl2])
    assert S2 == S
    perm = torch.cat([torch.arange(int(start[0, m]), int(start[0, m]) + bl[m]) for m in order]).to(dev)
    q2, k2, v2 = (torch.zeros_like(t) for t in (q, k, v))
    q2[0, :T], k2[0, :T], v2[0, :T] = q[0, perm], k[0, perm], v[0, perm]
    o2 = run(q2, k2, v2, start2.cuda(), ln2.cuda(), TC)
    assert (o2[0, :T].float() - o_tc[0, perm].float()).abs().max().item() < 1e-2
    mass2, _ = ops.doc_scores(q2.transpose(1, 2), k2.transpose(1, 2), start2.cuda(), ln2.cuda(), rows, D ** -0.5)
    docs = [m - 1 for m in order[1:-1]]
    assert torch.allclose(mass2, mass[..., docs], rtol=1e-3, atol=1e-7)
