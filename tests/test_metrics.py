"""Ranking metrics (CPU): hand-computed cases for the trec_eval definitions the reference relies on
(src/blockrank/utils.py:263-390 through pytrec_eval), qrels parsing in both formats, JSON output."""
import json
import math

import numpy as np
import pytest

from blockrank_b200 import metrics as M


def test_load_qrels_trec_and_beir(tmp_path):
    trec = tmp_path / "q.trec"
    trec.write_text("q1 0 d1 1\nq1 0 d2 0\nq2 0 d9 2\n\nbad line\n")
    beir = tmp_path / "q.tsv"
    beir.write_text("query-id\tcorpus-id\tscore\nq1\td1\t1\nq2\td9\t2\n")
    assert M.load_qrels(str(trec)) == {"q1": {"d1": 1, "d2": 0}, "q2": {"d9": 2}}
    assert M.load_qrels(str(beir)) == {"q1": {"d1": 1}, "q2": {"d9": 2}}


def test_ndcg_and_rr_hand_values():
    rels = {"a": 3, "b": 2, "c": 0, "d": 1}
    ranking = ["c", "a", "d", "b"]
    dcg3 = 0 / math.log2(2) + 3 / math.log2(3) + 1 / math.log2(4)
    idcg3 = 3 / math.log2(2) + 2 / math.log2(3) + 1 / math.log2(4)
    assert M.ndcg_at_k(ranking, rels, 3) == pytest.approx(dcg3 / idcg3)
    assert M.ndcg_at_k(ranking, rels, 1) == 0.0
    assert M.ndcg_at_k(["a", "b", "d", "c"], rels, 10) == pytest.approx(1.0)
    assert M.reciprocal_rank(ranking, rels) == 0.5
    assert M.reciprocal_rank(["c"], rels) == 0.0
    assert M.ndcg_at_k(ranking, {"x": 0}, 5) == 0.0  # nothing relevant: defined as 0


def test_ndcg_matches_sklearn_without_ties():
    sk = pytest.importorskip("sklearn.metrics")
    rng = np.random.default_rng(0)
    for _ in range(5):
        n = 12
        rel = rng.integers(0, 4, n)
        score = rng.permutation(n).astype(float)
        docs = [f"d{i:02d}" for i in range(n)]
        ranking = [docs[i] for i in np.argsort(-score)]
        rels = {d: int(r) for d, r in zip(docs, rel)}
        for k in (1, 3, 5, 10):
            assert M.ndcg_at_k(ranking, rels, k) == pytest.approx(sk.ndcg_score([rel], [score], k=k), abs=1e-12)


def test_ranking_metrics_accuracy_and_run_construction():
    preds = [[2, 0, 1], [1, 2, 0], 0]
    answers = [2, [0, 2], [1]]
    m = M.ranking_metrics(preds, answers)
    assert m["exact_match"] == 1 and m["total"] == 3 and m["accuracy"] == pytest.approx(100 / 3)
    qrels = {"q0": {"x2": 1}, "q1": {"y0": 1, "y2": 1}, "q2": {"z1": 1}, "q9": {"w": 1}}
    qids = ["q0", "q1", "q2"]
    remap = [["x0", "x1", "x2"], ["y0", "y1", "y2"], ["z0", "z1", "z2"]]
    run = M.build_run([[2, 0, 1], [1, 2, 0], [0]], qids, remap, qrels)
    assert run["q0"] == {"x2": 3.0, "x0": 2.0, "x1": 1.0}
    assert run["q2"] == {"z0": 1.0, "z1": 0.0, "z2": 0.0}
    m = M.ranking_metrics(preds, answers, qids, remap, qrels)
    # q0: relevant first -> RR 1, nDCG 1.  q1: ranking y1, y2, y0 -> RR 1/2.  q2: z0 first, then the
    # zero-score tie broken by id descending (z2 before z1) -> RR 1/3.
    assert m["mrr@10"] == pytest.approx(100 * (1 + 0.5 + 1 / 3) / 3)
    nd_q1 = (1 / math.log2(3) + 1 / math.log2(4)) / (1 + 1 / math.log2(3))
    nd_q2 = (1 / math.log2(4)) / 1.0
    assert m["ndcg@10"] == pytest.approx(100 * (1 + nd_q1 + nd_q2) / 3)
    assert m["ndcg@1"] == pytest.approx(100 / 3)
    with pytest.raises(ValueError):
        M.ranking_metrics(preds, answers, qrels=qrels)
    with pytest.raises(ValueError):
        M.ranking_metrics(preds, answers[:2])


def test_write_metrics(tmp_path):
    path = M.write_metrics(str(tmp_path / "out"), {"accuracy": 50.0}, attn_layer=20)
    assert path.endswith("attn_eval_metrics.json")
    assert json.load(open(path)) == {"accuracy": 50.0, "attn_layer": 20}
