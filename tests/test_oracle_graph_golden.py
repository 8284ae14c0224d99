"""The oracle's restatements of the code on either side of the ops (oracle/graph_oracle_impl.inc)
against fixtures produced by running the reference's own method bodies
(tests/golden/make_golden_graph.py): forced alignment, extract_links tail with its autograd
gradients, node-passing probabilities, Viterbi decoding."""
import numpy as np
import pytest

from oracle import oracle
from util import assert_rel, golden


def _masks(g):
    nonpad = g["nonpad"] if g["nonpad"].size else None
    bound_end = g["bound_end"] if g["bound_end"].size else None
    return bound_end, nonpad


def test_force_alignment_matches_the_criterion():
    g = golden("force_alignment")
    out = oracle.force_alignment(g["match"], g["force_emit"])
    assert np.array_equal(out, g["forced"])
    # two vertices forced onto one step both keep 0
    assert out[1, 2, 5] == 0 and out[1, 2, 6] == 0 and np.isneginf(out[1, 2, 4])


@pytest.mark.parametrize("name", ["links_from_heads_nonpad", "links_from_heads_band", "links_from_heads_bound"])
@pytest.mark.parametrize("dtype,tv,tg", [(np.float64, 1e-6, 1e-5), (np.float32, 1e-5, 1e-4)])
def test_links_from_heads_matches_extract_links(name, dtype, tv, tg):
    """The reference ran in fp32 (training precision); the fp64 oracle is compared at fp32 accuracy."""
    g = golden(name)
    bound_end, nonpad = _masks(g)
    K = int(g["K"])
    links, _ = oracle.links_from_heads(g["content"], g["log_gates"], K, bound_end, nonpad, dtype=dtype)
    assert_rel(links, g["links"], tv, "links")
    gc, gg = oracle.links_from_heads_backward(g["grad_links"], g["content"], g["log_gates"], K, bound_end, nonpad,
                                              dtype=dtype)
    assert_rel(gc, g["grad_content"], tg, "grad_content")
    # the fixture holds the gradient with respect to the gate SCORES (before their log_softmax)
    lg = g["log_gates"].astype(np.float64)
    gs = gg - np.exp(lg) * gg.sum(-1, keepdims=True)
    assert_rel(gs, g["grad_gate_scores"], tg, "grad_gate_scores")


def test_node_passing_prob_matches_analyze_graph():
    g = golden("node_pass")
    out = oracle.node_passing_prob(g["links"])
    assert_rel(out, g["node_pass"], 1e-12, "node_pass")
    out32 = oracle.node_passing_prob(g["links"], dtype=np.float32)
    assert_rel(out32, g["node_pass"], 1e-5, "node_pass fp32")


@pytest.mark.parametrize("name", ["viterbi_plain", "viterbi_joint"])
def test_viterbi_decode_matches_inference_viterbi(name):
    g = golden(name)
    logp = g["logp"]
    unreduced_logits, unreduced_tokens = logp.max(-1), logp.argmax(-1)
    L = g["links"].shape[1]
    max_length = int(2 * L / int(g["scale"]))
    toks, lens, verts, score = oracle.viterbi_decode(g["links"], unreduced_logits, unreduced_tokens,
                                                     g["output_length"], max_length, joint=bool(g["joint"]),
                                                     beta=float(g["beta"]), pad=int(g["pad"]))
    ref = g["tokens"]                       # [B, longest result], padded with pad
    assert lens.max() == ref.shape[1]
    assert np.array_equal(toks[:, :ref.shape[1]], ref)
    assert (toks[:, ref.shape[1]:] == int(g["pad"])).all()
    for b in range(len(lens)):
        n = int((verts[b] >= 0).sum())
        assert n >= lens[b] and (np.diff(verts[b][:n]) > 0).all()
