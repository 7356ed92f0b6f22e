"""CPU tests of the host side: C-ABI exports, collators, score helpers, prompt partition and gather."""
import ctypes
import os
import re
import subprocess
import sys

import numpy as np
import pytest
import torch

from blockrank_b200 import (_lib, block_icr_collate_fn, notebook_scores, packed_block_collate_fn,
                            signal_rows_from_labels)
from blockrank_b200.parallel import gather_scores, partition_prompts
from oracle import blockrank_oracle as orc

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    """The shared object loads without a GPU and exports exactly what include/blockrank_b200.h declares."""
    header = open(os.path.join(ROOT, "include", "blockrank_b200.h")).read()
    declared = set(re.findall(r"BRK_API[^;(]*?\b(brk_\w+)\s*\(", header))
    assert declared, "no declarations found"
    assert os.path.exists(_lib.LIB_PATH), "run `python -m blockrank_b200.build` first"
    L = ctypes.CDLL(_lib.LIB_PATH)
    for name in declared:
        assert hasattr(L, name), name
    assert declared >= set(_lib.EXPORTS)
    L.brk_version.restype = ctypes.c_int
    version = int(re.search(r"#define BRK_VERSION (\d+)", header).group(1))
    assert L.brk_version() == version


def test_argument_checks_return_error_codes_without_a_gpu():
    """Bad arguments are refused by the host-side checks of the C ABI before anything touches a device."""
    L = _lib.lib()
    assert L.brk_attn_fwd(None, None, 0, None) == -1                       # BRK_E_ARG: params is null
    assert L.brk_attn_bwd(None, None, 0, None) == -1
    assert b"null" in L.brk_last_error()
    p = _lib.AttnBwdParams()
    p.dtype, p.B, p.N, p.Nk, p.D, p.S, p.M, p.max_block_len, p.scale = 0, 1, 6, 4, 128, 64, 2, 32, 0.1
    assert L.brk_attn_bwd(ctypes.byref(p), None, 0, None) == -1             # N is not a multiple of Nk
    assert b"multiple" in L.brk_last_error()
    p.N, p.D = 8, 96
    assert L.brk_attn_bwd(ctypes.byref(p), None, 0, None) == -2             # BRK_E_UNSUPPORTED: head_dim
    p.D, p.max_block_len = 128, 65
    assert L.brk_attn_bwd(ctypes.byref(p), None, 0, None) == -1             # max_block_len > S
    p.max_block_len = 32
    assert L.brk_attn_bwd(ctypes.byref(p), None, 0, None) == -1             # spans / lse are null
    assert L.brk_attn_bwd_workspace_bytes(None) == 0
    # delta [B,N,S] + two fp32 accumulators [B,Nk,S,D] + (bf16) the last block's dq [B,N,max_block_len,D]
    assert L.brk_attn_bwd_workspace_bytes(ctypes.byref(p)) == 8 * 64 * 4 + 2 * 4 * 64 * 128 * 4 + 8 * 32 * 128 * 4


def test_missing_library_fails_loudly(monkeypatch):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", "/nonexistent/libblockrank_b200.so")
    with pytest.raises(ImportError, match="no CPU or PyTorch fallback"):
        _lib.lib()


def test_ops_refuse_cpu_tensors():
    from blockrank_b200 import ops
    with pytest.raises(RuntimeError, match="CUDA tensors"):
        ops.rmsnorm(torch.zeros(2, 8), torch.ones(8), 1e-5)


class Tok:
    pad_token_id = 0
    padding_side = "left"


def _items(fx, ci):
    n = int(fx[f"c{ci}_n"])
    return [{"input_ids": torch.tensor(fx[f"c{ci}_ids{b}"]), "block_lengths": torch.tensor(fx[f"c{ci}_lens{b}"]),
             "answer_ids": torch.tensor([0])} for b in range(n)]


@pytest.mark.parametrize("ci", [0, 1, 2])
def test_block_collator_matches_reference(golden_dir, ci):
    fx = np.load(os.path.join(golden_dir, "collate.npz"))
    cap = int(fx[f"c{ci}_cap"]) or None
    got = block_icr_collate_fn(_items(fx, ci), Tok(), pad_to_multiple_of=16, max_block_length=cap)
    for key in ("input_ids", "position_ids", "attention_mask", "labels"):
        assert np.array_equal(got[key].numpy(), fx[f"c{ci}_{key}"]), key
    assert int(got["num_blocks"]) == got["attention_mask"].shape[1]


@pytest.mark.parametrize("ci", [0, 2])
def test_packed_collator_is_the_padded_one_without_pads(golden_dir, ci):
    fx = np.load(os.path.join(golden_dir, "collate.npz"))
    items = _items(fx, ci)
    pad = block_icr_collate_fn(items, Tok(), pad_to_multiple_of=16)
    pk = packed_block_collate_fn(_items(fx, ci), Tok())
    mask = pad["attention_mask"]
    B = mask.shape[0]
    for b in range(B):
        keep = mask[b].reshape(-1)
        n = int(keep.sum())
        assert torch.equal(pk["input_ids"][b, :n], pad["input_ids"][b][keep])
        assert torch.equal(pk["position_ids"][b, :n], pad["position_ids"][b][keep])
        assert torch.equal(pk["labels"][b, :n], pad["labels"][b][keep])
        assert int(pk["block_spans"][1, b].sum()) == n
    start, ln = orc.block_spans(mask)
    assert torch.equal(pk["block_spans"][1], ln)
    rows = signal_rows_from_labels(pad["labels"])
    # same two tokens, addressed in packed coordinates
    for b in range(B):
        keep = mask[b].reshape(-1).long().cumsum(0) - 1
        assert keep[rows[b, 1]].item() == pk["signal_rows"][b, 1].item()
        assert keep[rows[b, 0]].item() == pk["signal_rows"][b, 0].item()


def test_signal_rows_follow_reference_rule():
    labels = torch.full((2, 40), -100)
    labels[0, -1] = 5
    labels[1, -3:] = 7
    assert signal_rows_from_labels(labels).tolist() == [[38, 39], [36, 37]]
    bad = torch.full((1, 40), -100)
    with pytest.raises(ValueError):
        signal_rows_from_labels(bad)
    bad[0, -16:] = 3  # first labelled token sits at window index 0: the reference asserts here too
    with pytest.raises(ValueError):
        signal_rows_from_labels(bad)


def test_packed_collator_refuses_prompts_without_signal_rows():
    """A completion cut off by truncation, or an empty one, leaves no signal rows: the packed collator
    raises where the reference asserts 'Bracket token not found' (losses.py:43-48)."""
    ids = torch.arange(3, 3 + 30)
    ok = {"input_ids": ids, "block_lengths": torch.tensor([8, 8, 12, 2])}
    out = packed_block_collate_fn([ok])
    assert out["signal_rows"].tolist() == [[27, 28]]
    with pytest.raises(ValueError, match="no signal rows"):   # query block 14 tokens, kept 10: completion cut
        packed_block_collate_fn([ok], max_block_length=10)
    with pytest.raises(ValueError, match="no signal rows"):   # empty completion
        packed_block_collate_fn([{"input_ids": ids, "block_lengths": torch.tensor([8, 8, 14, 0])}])


def test_notebook_scores_is_last_row_head_mean():
    """quickstart.ipynb cell 9: softmax of the last query row over the document columns, summed per
    document, averaged over heads -- here restated from raw logits and compared with the helper."""
    g = torch.Generator().manual_seed(0)
    B, N, R, nd, H = 2, 4, 2, 5, 8
    logits = torch.randn(B, N, R, nd * H, generator=g, dtype=torch.float64)
    probs = torch.softmax(logits, dim=-1).view(B, N, R, nd, H).sum(-1)     # per-row, per-head document mass
    want = torch.softmax(logits[:, :, -1], dim=-1).view(B, N, nd, H).sum(-1).mean(1)
    got = notebook_scores(probs)
    assert got.shape == (B, nd)
    assert torch.allclose(got, want, atol=1e-12)
    assert torch.allclose(got.sum(-1), torch.ones(B, dtype=torch.float64))


def test_partition_covers_all_prompts():
    for n, w in [(64, 8), (16, 8), (7, 4), (3, 8), (0, 2)]:
        parts = [partition_prompts(n, w, r) for r in range(w)]
        flat = sorted(p for part in parts for p in part)
        assert flat == list(range(n))
        assert max(map(len, parts)) - min(map(len, parts)) <= 1
    costs = [100, 1, 1, 1, 50, 50, 2, 2]
    parts = [partition_prompts(8, 2, r, costs) for r in range(2)]
    assert sorted(parts[0] + parts[1]) == list(range(8))
    loads = [sum(costs[i] for i in p) for p in parts]
    assert abs(loads[0] - loads[1]) <= 10


def test_gather_single_process():
    s = torch.arange(6.).view(3, 2)
    out = gather_scores(s, [4, 0, 2], 5)
    assert out[4].tolist() == [0., 1.] and out[0].tolist() == [2., 3.] and out[1].tolist() == [0., 0.]


WORKER = r"""
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
from blockrank_b200.parallel import partition_prompts, gather_scores
mode = sys.argv[2]
dist.init_process_group("gloo", init_method="tcp://127.0.0.1:" + sys.argv[3], rank=int(os.environ["RANK"]),
                        world_size=int(os.environ["WORLD_SIZE"]), timeout=__import__("datetime").timedelta(seconds=20))
rank, world = dist.get_rank(), dist.get_world_size()
P, ND = 7, 5
costs = [9, 1, 1, 1, 5, 5, 2] if mode == "costs" else None
mine = partition_prompts(P, world, rank, costs)
local = torch.tensor([[p * 10.0 + d for d in range(ND)] for p in mine]).reshape(len(mine), ND)
if mode == "drop" and rank == 1:
    mine, local = mine[:-1], local[:-1]      # a rank that lost a prompt: the gather must notice
share = max(len(partition_prompts(P, world, r, costs)) for r in range(world))   # same on every rank, no communication
try:
    full = gather_scores(local, mine, P, max_share=share)
    ok = all(abs(full[p, d].item() - (p * 10.0 + d)) < 1e-6 for p in range(P) for d in range(ND))
    print("RESULT", rank, "ok" if ok else "bad")
except RuntimeError as e:
    print("RESULT", rank, "error", str(e)[:60])
dist.destroy_process_group()
"""


def _run_world(mode, port):
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE="2")
        procs.append(subprocess.Popen([sys.executable, "-c", WORKER, ROOT, mode, str(port)], env=env,
                                      stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=120)[0] for p in procs]
    return outs


@pytest.mark.parametrize("mode,port", [("plain", 29611), ("costs", 29612)])
def test_gather_two_gloo_ranks(mode, port):
    outs = _run_world(mode, port)
    for r, o in enumerate(outs):
        assert f"RESULT {r} ok" in o, o


def test_gather_detects_missing_prompt():
    outs = _run_world("drop", 29613)
    for r, o in enumerate(outs):
        assert f"RESULT {r} error" in o and "no rank delivered" in o, o
