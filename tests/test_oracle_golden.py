"""The CPU oracle (oracle/dag_oracle.c) against golden vectors produced by the
reference's own torch-native functions (tests/golden/make_golden.py).  This is
what pins the oracle before any CUDA result is compared with it."""
import numpy as np
import pytest
import torch

from oracle import oracle
from da_transformer_b200 import workloads
from util import assert_rel, golden


@pytest.mark.parametrize("name", ["dag_small_full", "dag_small_band", "dag_small_even"])
def test_dag_loss_and_grads_match_reference_twin(name):
    g = golden(name)
    loss, gm, gl = oracle.dag_loss_fwd_bwd(g["match_all"], g["links"], g["output_length"],
                                           g["target_length"], dtype=np.float64)
    assert_rel(loss, g["loss"], 1e-12, "loss")
    # the twin's autograd leaves unreachable sentences at 0 like the CUDA formulas do
    assert_rel(gm, g["grad_match"], 1e-10, "grad_match")
    assert_rel(gl, g["grad_links"], 1e-10, "grad_links")


@pytest.mark.parametrize("name", ["dag_small_full", "dag_small_band", "dag_small_even"])
def test_dag_loss_fp32_oracle_within_tolerance(name):
    g = golden(name)
    loss, gm, gl = oracle.dag_loss_fwd_bwd(g["match_all"], g["links"], g["output_length"],
                                           g["target_length"], dtype=np.float32)
    assert_rel(loss, g["loss"], 1e-5, "loss")
    assert_rel(gm, g["grad_match"], 1e-4, "grad_match")
    assert_rel(gl, g["grad_links"], 1e-4, "grad_links")


@pytest.mark.parametrize("name", ["dag_small_full", "dag_small_band", "dag_small_even"])
@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_best_alignment_matches_reference_twin_on_tie_free_inputs(name, dtype):
    g = golden(name)
    path, alpha = oracle.dag_best_alignment(g["match_all"], g["links"], g["output_length"],
                                            g["target_length"], dtype=dtype)
    ok = np.isfinite(g["max_loss"])
    assert ok.any()
    # continuous random inputs have no ties, so the twin's argmax path is the path
    assert np.array_equal(path[ok], g["path"][ok])
    assert (path[~ok] == -1).all()
    b = np.arange(len(ok))[ok]
    score = alpha[b, g["target_length"][ok] - 1, g["output_length"][ok] - 1]
    assert_rel(score, g["max_loss"][ok], 1e-5 if dtype == np.float32 else 1e-12, "max score")


def test_tie_break_follows_the_shuffle_tree():
    """All-equal inputs: every path ties.  With 4 lanes the merge tree prefers
    lane 0, then lane 2, then lane 1, then lane 3 (lane = (d-1) mod 4), and the
    smallest d inside a lane (dag_best_alignment.cu:96-111)."""
    B, T, L = 1, 3, 9
    match = np.zeros((B, T, L))
    links = np.zeros((B, L, L - 1))
    path, _ = oracle.dag_best_alignment(match, links, [L], [T], dtype=np.float32)
    # last token sits on vertex 8; candidates d=1..8 tie; lane 0 holds d=1,5 -> d=1 -> vertex 7
    # vertex 7 at t=1: candidates d=1..7 -> d=1 -> vertex 6, which must be ... but t=0 is only
    # reachable at vertex 0, so alpha[0,6] = -inf and the only finite predecessor wins.
    assert path[0, 8] == 2 and path[0, 0] == 0
    assert (path[0] >= 0).sum() == T
    # a case where only lanes 1 and 2 hold the maximum: lane 2 (d=3) must win over lane 1 (d=2)
    T, L = 2, 5
    match = np.zeros((1, T, L))
    links = np.full((1, L, L - 1), -1.0)
    # predecessors of vertex 4 at t=1 is only vertex 0 (alpha[0,0]); make T=3 instead
    T = 3
    match = np.zeros((1, T, L))
    links = np.full((1, L, L - 1), -5.0)
    links[0, 0, :] = 0.0            # vertex 0 reaches every vertex at equal cost
    links[0, 2, 1] = 0.0            # 2 -> 4 (d=2, lane 1)
    links[0, 1, 2] = 0.0            # 1 -> 4 (d=3, lane 2)
    path, _ = oracle.dag_best_alignment(match, links, [L], [T], dtype=np.float32)
    assert path[0].tolist() == [0, 1, -1, -1, 2]


@pytest.mark.parametrize("name,tol_sel,tol_grad", [
    ("gather_small_f32", 1e-6, 1e-5),
    ("gather_small_f16", 1e-6, 2e-3),
    ("gather_small_bf16", 1e-6, 2e-3),
])
def test_gather_matches_reference_twin(name, tol_sel, tol_grad):
    g = golden(name)
    sel = oracle.logsoftmax_gather(g["logits"], g["select_idx"], dtype=np.float64)
    assert_rel(sel, g["sel_f64"], 1e-12, "sel vs fp64")
    assert_rel(sel, g["sel"], tol_sel, "sel vs twin")
    dx = oracle.logsoftmax_gather_backward(g["logits"], g["select_idx"], g["grad_sel"])
    assert_rel(dx, g["dlogits_f64"], 1e-12, "dlogits vs fp64")
    assert_rel(dx, g["dlogits"], tol_grad, "dlogits vs twin")
    sel32 = oracle.logsoftmax_gather(g["logits"], g["select_idx"], dtype=np.float32)
    assert_rel(sel32, g["sel_f64"], 1e-5, "fp32 oracle sel")


def test_gather_accepts_the_stride0_expand_of_the_criterion():
    batch = workloads.small_batch(seed=5)
    a = oracle.logsoftmax_gather(batch.logits.numpy(), batch.select_idx.numpy())
    b = oracle.logsoftmax_gather(batch.logits.numpy(), batch.select_idx.contiguous().numpy())
    assert np.array_equal(a, b)
    assert_rel(np.swapaxes(a, 1, 2), batch.match_all.numpy(), 1e-5, "match")


def test_config0_against_reference_twin():
    g = golden("config0")
    batch = workloads.config0()
    # the seeded generator must reproduce the inputs the fixture was made from
    assert np.array_equal(batch.targets.numpy(), g["targets"])
    assert abs(batch.logits.double().sum().item() - float(g["logits_sum"])) < 1e-6
    sel = oracle.logsoftmax_gather(batch.logits.numpy(), batch.select_idx.numpy())
    match = np.ascontiguousarray(np.swapaxes(sel, 1, 2))
    assert_rel(match[:, :, ::7], g["match_slice"], 1e-6, "match")
    loss, gm, gl = oracle.dag_loss_fwd_bwd(match, batch.links.numpy(), batch.output_length.numpy(),
                                           batch.target_length.numpy())
    assert_rel(loss, g["loss_f64"], 1e-6, "loss")  # match came through an fp32 twin in the fixture
    assert_rel(gm.sum(-1), g["grad_match_rowsum_f64"], 1e-5, "posterior row sums")
    assert_rel(gm[:, :, ::7], g["grad_match_slice_f64"], 1e-4, "grad_match")
    assert_rel(gl[:, ::5, ::3], g["grad_links_slice_f64"], 1e-4, "grad_links")
    path, _ = oracle.dag_best_alignment(match, batch.links.numpy(), batch.output_length.numpy(),
                                        batch.target_length.numpy(), dtype=np.float32)
    assert np.array_equal(path, g["path_f32"])
    tl = batch.target_length.numpy()
    for b in range(len(tl)):
        assert sorted(path[b][path[b] >= 0].tolist()) == list(range(tl[b]))


def test_band_square_round_trip():
    batch = workloads.small_batch(seed=7)
    sq = oracle.band_to_square(batch.links.numpy())
    assert np.array_equal(sq, workloads.band_to_square(batch.links.double()).numpy())
    assert np.array_equal(oracle.square_to_band(sq), batch.links.double().numpy())


def test_invalid_lengths_are_defined_not_trapped():
    batch = workloads.small_batch(seed=8, B=3)
    ol = batch.output_length.numpy().copy()
    tl = batch.target_length.numpy().copy()
    tl[1] = 1            # the reference would trap (dag_loss.cu:68)
    ol[2] = tl[2] - 1    # graph smaller than the target (dag_loss.cu:69)
    loss, gm, gl = oracle.dag_loss_fwd_bwd(batch.match_all.numpy(), batch.links.numpy(), ol, tl)
    assert np.isfinite(loss[0]) and np.isneginf(loss[1]) and np.isneginf(loss[2])
    assert (gm[1:] == 0).all() and (gl[1:] == 0).all()
    path, _ = oracle.dag_best_alignment(batch.match_all.numpy(), batch.links.numpy(), ol, tl)
    assert (path[1:] == -1).all()
