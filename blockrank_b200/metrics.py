"""Ranking metrics for attention-based evaluation, without pytrec_eval.

Mirrors what scripts/eval_attn.py reports through ``calculate_accuracy``
(src/blockrank/utils.py:263-390): top-1 accuracy against ``answer_ids`` and, when
qrels are given, nDCG@{1,3,5,10} and MRR computed the way trec_eval does
(``ndcg_cut_k``: gain = relevance, discount log2(rank+1), ideal ranking from all
judged documents of the query; ``recip_rank``: first document with relevance > 0 in
the full ranking; ties in score broken by document id, larger id first).  The run
is built like the reference builds it: the k predicted documents get scores k..1,
every other candidate of the query gets 0.  Values are percentages, as in the
reference.  ``load_qrels`` follows src/blockrank/utils.py:232-261.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence, Union

Pred = Union[int, Sequence[int]]
NDCG_CUTS = (1, 3, 5, 10)


def load_qrels(path: str) -> Dict[str, Dict[str, int]]:
    """TREC (``qid iter docid rel``) or BEIR TSV (``qid docid rel`` with a ``query-id`` header) qrels."""
    qrels: Dict[str, Dict[str, int]] = {}
    with open(path, "r") as f:
        for i, line in enumerate(f):
            line = line.strip()
            if not line or (i == 0 and line.startswith("query-id")):
                continue
            parts = line.split("\t") if "\t" in line else line.split()
            if len(parts) == 4:
                qid, _, did, rel = parts
            elif len(parts) == 3:
                qid, did, rel = parts
            else:
                continue
            qrels.setdefault(qid, {})[str(did)] = int(rel)
    return qrels


def _trec_ranking(run_q: Dict[str, float]) -> List[str]:
    """Documents of one query in trec_eval order: score descending, then document id descending."""
    return [d for d, _ in sorted(run_q.items(), key=lambda kv: (kv[1], kv[0]), reverse=True)]


def ndcg_at_k(ranking: Sequence[str], rels: Dict[str, int], k: int) -> float:
    gains = [max(0, rels.get(d, 0)) for d in ranking[:k]]
    dcg = sum(g / math.log2(i + 2) for i, g in enumerate(gains))
    ideal = sorted((r for r in rels.values() if r > 0), reverse=True)[:k]
    idcg = sum(g / math.log2(i + 2) for i, g in enumerate(ideal))
    return dcg / idcg if idcg > 0 else 0.0


def reciprocal_rank(ranking: Sequence[str], rels: Dict[str, int]) -> float:
    for i, d in enumerate(ranking):
        if rels.get(d, 0) > 0:
            return 1.0 / (i + 1)
    return 0.0


def build_run(predictions: Sequence[Sequence[int]], query_ids: Sequence, remapped_doc_ids: Sequence[Sequence],
              qrels: Dict[str, Dict[str, int]]) -> Dict[str, Dict[str, float]]:
    """query id -> {doc id: score}: rank i of k predicted documents scores k - i, unranked candidates 0."""
    run: Dict[str, Dict[str, float]] = {}
    for pred, qid, doc_ids in zip(predictions, query_ids, remapped_doc_ids):
        qid = str(qid)
        if qid not in qrels:
            continue
        scores: Dict[str, float] = {}
        for rank, idx in enumerate(pred):
            if idx < len(doc_ids):
                scores[str(doc_ids[idx])] = float(len(pred) - rank)
        ranked = set(pred)
        for idx, did in enumerate(doc_ids):
            if idx not in ranked:
                scores[str(did)] = 0.0
        run[qid] = scores
    return run


def ranking_metrics(predictions: Sequence[Pred], answer_ids: Sequence, query_ids: Optional[Sequence] = None,
                    remapped_doc_ids: Optional[Sequence[Sequence]] = None,
                    qrels: Optional[Dict[str, Dict[str, int]]] = None) -> Dict[str, float]:
    """``predictions[i]``: top-k document indices of prompt i (or a single index); ``answer_ids[i]``: the relevant
    index or indices.  With ``qrels`` (and ``query_ids``, ``remapped_doc_ids``: candidate index -> corpus doc id)
    the trec_eval-style metrics are added."""
    preds = [[int(x) for x in p] if isinstance(p, (list, tuple)) else [int(p)] for p in predictions]
    truth = list(answer_ids)[:len(preds)]
    if len(truth) != len(preds):
        raise ValueError("predictions and answer_ids differ in length")
    correct = invalid = 0
    for p, g in zip(preds, truth):
        try:
            gt = {int(x) for x in g} if isinstance(g, (list, tuple)) else {int(g)}
            correct += bool(p) and p[0] in gt
        except (TypeError, ValueError):
            invalid += 1
    total = len(preds)
    out: Dict[str, float] = {
        "accuracy": 100.0 * correct / total if total else 0.0,
        "exact_match": correct,
        "total": total,
        "invalid_predictions": invalid,
        "invalid_rate": 100.0 * invalid / total if total else 0.0,
    }
    if qrels is not None:
        if query_ids is None or remapped_doc_ids is None:
            raise ValueError("qrels need query_ids and remapped_doc_ids")
        run = build_run(preds, query_ids, remapped_doc_ids, qrels)
        ndcg = {k: [] for k in NDCG_CUTS}
        rr = []
        for qid, scores in run.items():
            ranking = _trec_ranking(scores)
            for k in NDCG_CUTS:
                ndcg[k].append(ndcg_at_k(ranking, qrels[qid], k))
            rr.append(reciprocal_rank(ranking, qrels[qid]))
        for k in NDCG_CUTS:
            if ndcg[k]:
                out[f"ndcg@{k}"] = 100.0 * sum(ndcg[k]) / len(ndcg[k])
            if rr:
                out[f"mrr@{k}"] = 100.0 * sum(rr) / len(rr)  # the reference reports the same MRR under every k
    return out


def write_metrics(output_dir: str, metrics: Dict[str, float], attn_layer: int) -> str:
    """``attn_eval_metrics.json`` as scripts/eval_attn.py:176-186 writes it."""
    os.makedirs(output_dir, exist_ok=True)
    path = os.path.join(output_dir, "attn_eval_metrics.json")
    with open(path, "w") as f:
        json.dump({**metrics, "attn_layer": attn_layer}, f, indent=2)
    return path


def rank_items(ranker, items: Sequence[dict], tok=None, batch_size: int = 1, k: int = 10) -> List[List[int]]:
    """Top-k predictions for pre-tokenised prompts (``input_ids`` + ``block_lengths`` per item, the form the
    collators take): packs each batch without padding, runs the early-exit ranker, returns index lists in
    input order -- the ``all_attn_preds`` of scripts/eval_attn.py:133-160."""
    from .collate import packed_block_collate_fn

    preds: List[List[int]] = []
    for i in range(0, len(items), batch_size):
        batch = packed_block_collate_fn(items[i:i + batch_size], tok)
        _, top = ranker.rank_host(batch, k=k)
        preds.extend(top.tolist())
    return preds
