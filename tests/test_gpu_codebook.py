"""Offline cluster-pool codebook build on a B200 (`speedup_thingy_b200.codebook`) against the CPU oracle
(oracle/rte_oracle.py, pinned to the reference's builders by tests/golden/codebook.npz): selector features and pool
scores within the bf16 tolerance, k-means assignments bit-exact on well-separated data, centres and aggregated scores
at fp32 tolerance, candidate lists equal per cluster, and the built codebook drives the cluster-pool FFN."""
import numpy as np
import pytest
import torch

from oracle import rte_oracle as O
from tests.golden.cases import CODEBOOK, codebook_inputs

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def builder():
    from speedup_thingy_b200.codebook import CodebookBuilder
    from speedup_thingy_b200.ops import CudaOps
    return CodebookBuilder(CudaOps(DEV))


def _rel(a, b):
    a, b = a.detach().float().cpu(), b.detach().float().cpu()
    return ((a - b).abs().max() / b.abs().max().clamp_min(1e-6)).item()


@pytest.mark.parametrize("mode", ["sum", "upgate", "product"])
def test_features_and_scores_match_oracle(builder, mode):
    from speedup_thingy_b200.codebook import svd_factor_cache
    c, t = CODEBOOK, codebook_inputs()
    factors = svd_factor_cache(t["wug"], c["rank"], DEV)
    feats, scores = builder.features_and_scores(t["normed"].to(DEV), factors, t["wd"].to(DEV), rank=c["rank"], score_mode=mode)
    torch.cuda.synchronize()
    builder.ops.check_status()
    cpu = {k: v.cpu() for k, v in factors.items()}
    f_ref, s_ref = O.cluster_features_and_scores(t["normed"], cpu, t["wd"].norm(dim=0), c["rank"], mode)
    assert _rel(feats, f_ref) <= 1e-2 and _rel(scores, s_ref) <= 2e-2


@pytest.mark.parametrize("aggregation", ["mean", "max"])
def test_kmeans_aggregation_and_candidates_match_oracle(builder, aggregation):
    c = CODEBOOK
    gold = np.load(__import__("pathlib").Path(__file__).resolve().parent / "golden" / "codebook.npz")
    feats, scores = torch.from_numpy(gold["features"]), torch.from_numpy(gold["scores_sum"])
    book = builder.build(feats.to(DEV), scores.to(DEV), cluster_count=c["clusters"], candidate_m=c["candidate_m"],
                         aggregation=aggregation, iters=c["iters"])
    torch.cuda.synchronize()
    builder.ops.check_status()
    ref = O.build_cluster_pool_codebook(feats, scores, c["clusters"], c["candidate_m"], aggregation, c["iters"])
    assert torch.equal(book["assignments"].cpu().long(), ref["assignments"])                    # bit-exact indices
    assert np.array_equal(book["assignments"].cpu().numpy(), gold["assignments"])               # ... and the reference's
    assert _rel(book["centers"], ref["centers"]) <= 1e-5
    assert _rel(book["aggregate"], ref["aggregate"]) <= 1e-5
    # candidate order: (score desc, id asc) on the device's own aggregate
    want = O.topk_lowest(book["aggregate"].cpu(), c["candidate_m"])[1]
    assert torch.equal(book["candidate_ids"].cpu(), want)
    for mine, r in zip(book["candidate_ids"].cpu().tolist(), gold[f"candidate_ids_{aggregation}"].tolist()):
        assert set(mine) == set(r)
    assert book["nonempty_clusters"] == c["clusters"]


def test_kmeans_degenerate_cases(builder):
    g = torch.Generator().manual_seed(5)
    feats = torch.randn(40, 32, generator=g)
    a, cen = builder.fit_centers(feats.to(DEV), 1, 3)
    a_ref, cen_ref = O.fit_cluster_centers(feats, 1, 3)
    assert torch.equal(a.cpu().long(), a_ref) and _rel(cen, cen_ref) <= 1e-5
    # more clusters than distinct points: empty clusters keep their centre
    dup = feats[:3].repeat(10, 1)
    a, cen = builder.fit_centers(dup.to(DEV), 8, 4)
    a_ref, cen_ref = O.fit_cluster_centers(dup, 8, 4)
    assert torch.equal(a.cpu().long(), a_ref) and _rel(cen, cen_ref) <= 1e-5


def test_built_codebook_drives_the_cluster_pool_ffn(builder):
    """End of the offline step: factors + codebook built here go into StaticClusterPoolSwiGLU; with every neuron in
    every pool the sparse FFN reproduces the dense one (the reference's own "recover dense" property,
    tests/test_models_and_training.py:93-157)."""
    from speedup_thingy_b200.cluster_pool import StaticClusterPoolSwiGLU
    from speedup_thingy_b200.codebook import active_union_ids, svd_factor_cache
    c, t = CODEBOOK, codebook_inputs()
    factors = svd_factor_cache(t["wug"], c["rank"], DEV)
    feats, scores = builder.features_and_scores(t["normed"].to(DEV), factors, t["wd"].to(DEV), rank=c["rank"])
    book = builder.build(feats, scores, cluster_count=c["clusters"], candidate_m=c["f"], aggregation="mean", iters=c["iters"])
    assert sorted(book["candidate_ids"][0].tolist()) == list(range(c["f"]))
    mod = StaticClusterPoolSwiGLU(t["wug"].to(DEV), t["wd"].to(DEV), factors, book, rank=c["rank"], max_tokens=c["tokens"])
    x = t["normed"].to(DEV)
    out = mod.forward(x)
    dense = mod.dense_forward(x)
    torch.cuda.synchronize()
    assert _rel(out, dense) <= 2e-2
    small = builder.build(feats, scores, cluster_count=c["clusters"], candidate_m=c["candidate_m"], aggregation="mean", iters=c["iters"])
    union = active_union_ids(small["candidate_ids"], c["f"])
    assert torch.equal(union.cpu(), O.active_union_ids(small["candidate_ids"].cpu(), c["f"]))
    capped = active_union_ids(small["candidate_ids"], c["f"], cap=96)
    assert torch.equal(capped.cpu(), O.active_union_ids(small["candidate_ids"].cpu(), c["f"], cap=96))
