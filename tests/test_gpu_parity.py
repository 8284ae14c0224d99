"""Parity of the CUDA path (through the C ABI, via the Python front end) with the CPU
oracle and with the golden vectors of the reference's torch-native functions.

Tolerances (max|d| / max|ref| per tensor):
  loss 1e-5, gradients 1e-4 (2e-3 with fp16 / bf16 logits), alignment paths bit-exact.
"""
import numpy as np
import pytest
import torch

from oracle import oracle
from da_transformer_b200 import (DagBestAlignmentFunc, DagLogsoftmaxGatherFunc, DagLossFunc, dag_best_alignment,
                                 dag_logsoftmax_gather_inplace, dag_loss, last_status, workloads)
from util import assert_rel, assert_rel_per_sentence, assert_rel_quantized, golden, plain_tol_16bit

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL_LOSS, TOL_GRAD, TOL_GRAD_HALF, TOL_SEL = 1e-5, 1e-4, 2e-3, 2e-6


@pytest.fixture(params=["fast", "exact"], autouse=True)
def dag_loss_path(request):
    """Every test runs with the fast (probability-domain, self-checking) forward and with the
    exact log-domain forward."""
    DagLossFunc.exact = request.param == "exact"
    yield request.param
    DagLossFunc.exact = False


def run_dag(match, links, ol, tl, grad_out=None):
    m = torch.as_tensor(match, dtype=torch.float32, device=DEV).requires_grad_()
    l = torch.as_tensor(links, dtype=torch.float32, device=DEV).requires_grad_()
    ol = torch.as_tensor(ol, dtype=torch.long, device=DEV)
    tl = torch.as_tensor(tl, dtype=torch.long, device=DEV)
    loss = dag_loss(m, l, ol, tl)
    g = torch.ones_like(loss) if grad_out is None else torch.as_tensor(grad_out, dtype=torch.float32, device=DEV)
    gm, gl = torch.autograd.grad(loss, [m, l], grad_outputs=g)
    with torch.no_grad():
        loss_nograd = dag_loss(m.detach(), l.detach(), ol, tl)
    return loss.detach().cpu().numpy(), gm.cpu().numpy(), gl.cpu().numpy(), loss_nograd.cpu().numpy()


def check_dag_against_oracle(batch, grad_out=None):
    match, links = batch.match_all.numpy(), batch.links.numpy()
    ol, tl = batch.output_length.numpy(), batch.target_length.numpy()
    loss, gm, gl, loss_ng = run_dag(match, links, ol, tl, grad_out)
    rl, rgm, rgl = oracle.dag_loss_fwd_bwd(match, links, ol, tl, grad_output=grad_out)
    assert_rel(loss, rl, TOL_LOSS, "loss (beta)")
    assert_rel(loss_ng, rl, TOL_LOSS, "loss (alpha, no grad)")
    assert_rel(gm, rgm, TOL_GRAD, "grad_match")
    assert_rel(gl, rgl, TOL_GRAD, "grad_links")
    assert_rel_per_sentence(gm, rgm, TOL_GRAD, "grad_match")
    assert_rel_per_sentence(gl, rgl, TOL_GRAD, "grad_links")


@pytest.mark.parametrize("seed,B,L,T,K", [
    (1, 5, 24, 6, None), (2, 4, 40, 9, 6), (3, 3, 33, 7, None), (4, 6, 97, 13, None),
    (5, 2, 130, 31, 40), (6, 3, 64, 2, None), (7, 2, 200, 50, None), (8, 4, 32, 32, None),
    # more than 64 target steps with all rows still in shared memory (strip sweep, two passes of its
    # matrix-product phase), full and banded links
    (9, 2, 190, 100, None), (10, 2, 190, 100, 40),
    # graphs longer than 1024 vertices (a thread of the exact alpha sweep then finalises more than two columns)
    (11, 2, 1300, 12, None), (12, 1, 2048, 6, 700),
    # rows that do not fit in one SM's shared memory: the sweep by a cluster of 8 / 16 CTAs (and, longer than
    # 1024 vertices with many steps, the tiled sweep or the exact kernels)
    (13, 2, 700, 120, None), (14, 2, 1000, 150, 300), (15, 1, 1024, 70, None), (16, 2, 1100, 140, None),
])
def test_dag_loss_matches_oracle(seed, B, L, T, K):
    batch = workloads.small_batch(seed=seed, B=B, L=L, T=T, V=50, translen=K)
    check_dag_against_oracle(batch)
    g = np.linspace(-1.0, 2.0, B).astype(np.float32)
    check_dag_against_oracle(batch, g)


@pytest.mark.parametrize("name", ["dag_small_full", "dag_small_band", "dag_small_even"])
def test_dag_loss_matches_reference_golden(name):
    g = golden(name)
    loss, gm, gl, loss_ng = run_dag(g["match_all"], g["links"], g["output_length"], g["target_length"])
    assert_rel(loss, g["loss"], TOL_LOSS, "loss")
    assert_rel(loss_ng, g["loss"], TOL_LOSS, "loss (no grad)")
    assert_rel(gm, g["grad_match"], TOL_GRAD, "grad_match")
    assert_rel(gl, g["grad_links"], TOL_GRAD, "grad_links")
    path = dag_best_alignment(torch.as_tensor(g["match_all"], device=DEV), torch.as_tensor(g["links"], device=DEV),
                              torch.as_tensor(g["output_length"], device=DEV),
                              torch.as_tensor(g["target_length"], device=DEV)).cpu().numpy()
    ok = np.isfinite(g["max_loss"])
    assert np.array_equal(path[ok], g["path"][ok])
    assert (path[~ok] == -1).all()
    last_status()


def test_forced_alignment_match_with_minus_inf_and_zero():
    """The criterion's forced alignment writes 0 and -inf into match
    (nat_dag_loss.py:111-120); both must flow through like in the reference."""
    batch = workloads.small_batch(seed=11, B=4, L=48, T=8, V=30, ragged=False)
    match = batch.match_all.clone()
    match[:, 3, :] = float("-inf")
    match[:, 3, 20] = 0.0
    match[1, 5, :] = float("-inf")   # sentence 1 becomes impossible
    batch.match_all = match
    check_dag_against_oracle(batch)


@pytest.mark.parametrize("config", [1, 2, 3, 4])
@pytest.mark.parametrize("seed,B,L,T,K,quant", [
    (1, 5, 24, 6, None, 0), (2, 4, 40, 9, 6, 0), (3, 4, 70, 12, None, 0.5), (4, 3, 97, 13, 20, 1.0),
    (5, 2, 160, 20, None, 0.25), (6, 2, 64, 5, None, 2.0), (7, 2, 190, 100, None, 0.5), (8, 2, 190, 100, 40, 0.5),
    (9, 1, 1300, 12, None, 0.5),
    # rows that do not fit one SM's shared memory: clusters of 16, 8 and 4 CTAs per sentence
    (10, 2, 1000, 150, None, 0.5), (11, 2, 700, 120, 300, 0.25), (12, 2, 400, 200, None, 1.0),
    (13, 1, 1024, 70, None, 0.0),
])
def test_best_alignment_bit_exact(config, seed, B, L, T, K, quant):
    batch = workloads.small_batch(seed=seed, B=B, L=L, T=T, V=50, translen=K)
    match, links = batch.match_all.clone(), batch.links.clone()
    if quant:  # coarse values make many candidates tie exactly
        match = torch.round(match / quant) * quant
        links = torch.round(links / quant) * quant
    DagBestAlignmentFunc.config = config
    try:
        path = dag_best_alignment(match.to(DEV), links.to(DEV), batch.output_length.to(DEV),
                                  batch.target_length.to(DEV)).cpu().numpy()
    finally:
        DagBestAlignmentFunc.config = 1
    ref, _ = oracle.dag_best_alignment(match.numpy(), links.numpy(), batch.output_length.numpy(),
                                       batch.target_length.numpy(), dtype=np.float32,
                                       trans_block=2 ** (config + 1))
    assert path.dtype == np.int64
    assert np.array_equal(path, ref)
    last_status()


@pytest.mark.parametrize("config", [1, 3])
@pytest.mark.parametrize("B,L,T,K,quant", [(330, 70, 12, None, 0.5), (200, 130, 40, 50, 0.0), (160, 200, 60, 30, 0.25)])
def test_best_alignment_more_sentences_than_sms(config, B, L, T, K, quant):
    """Batches larger than the SM count run on persistent CTAs (sentences taken from a counter, the backtrace of
    one sentence beside the sweep of the next): same paths, bit for bit, with invalid and path-less sentences among
    them."""
    batch = workloads.small_batch(seed=77, B=B, L=L, T=T, V=50, translen=K)
    match, links = batch.match_all.clone(), batch.links.clone()
    if quant:
        match = torch.round(match / quant) * quant
        links = torch.round(links / quant) * quant
    ol, tl = batch.output_length.clone(), batch.target_length.clone()
    bad = [3, 150, B - 1]
    tl[bad[0]] = 1                 # too short a target
    ol[bad[1]] = tl[bad[1]] - 1    # graph smaller than the target
    ol[bad[2]] = L + 1             # beyond the padded size
    nopath = 7
    links[nopath, : int(ol[nopath]), :] = float("-inf")   # no transition at all: no path
    good = [b for b in range(B) if b not in bad]
    last_status()
    DagBestAlignmentFunc.config = config
    try:
        path = dag_best_alignment(match.to(DEV), links.to(DEV), ol.to(DEV), tl.to(DEV)).cpu().numpy()
    finally:
        DagBestAlignmentFunc.config = 1
    st = last_status()
    assert st & 1 and st & 2
    assert (path[bad] == -1).all() and (path[nopath] == -1).all()
    good = [b for b in good if b != nopath]
    ref, _ = oracle.dag_best_alignment(match[good].numpy(), links[good].numpy(), ol[good].numpy(), tl[good].numpy(),
                                       dtype=np.float32, trans_block=2 ** (config + 1))
    assert np.array_equal(path[good], ref)


def test_all_equal_inputs_follow_the_reference_tie_break():
    B, T, L = 2, 7, 40
    match = torch.zeros(B, T, L)
    links = workloads.square_to_band(torch.zeros(B, L, L).masked_fill(
        ~(torch.arange(L).view(1, 1, L) > torch.arange(L).view(1, L, 1)), float("-inf")))
    ol = torch.tensor([L, L - 3])
    tl = torch.tensor([T, T - 2])
    for config in (1, 2, 3, 4):
        DagBestAlignmentFunc.config = config
        try:
            path = dag_best_alignment(match.to(DEV), links.to(DEV), ol.to(DEV), tl.to(DEV)).cpu().numpy()
        finally:
            DagBestAlignmentFunc.config = 1
        ref, _ = oracle.dag_best_alignment(match.numpy(), links.numpy(), ol.numpy(), tl.numpy(),
                                           dtype=np.float32, trans_block=2 ** (config + 1))
        assert np.array_equal(path, ref), config


def gather_case(logits, idx, gsel, transposed=False):
    x = logits.to(DEV).requires_grad_()
    DagLogsoftmaxGatherFunc.transposed_output = transposed
    try:
        work = x.clone()
        out, sel = dag_logsoftmax_gather_inplace(work, idx.to(DEV))
    finally:
        DagLogsoftmaxGatherFunc.transposed_output = False
    assert out is work
    (dx,) = torch.autograd.grad(sel, [x], grad_outputs=gsel.to(DEV))
    return sel.detach().cpu(), dx.cpu()


@pytest.mark.parametrize("dtype,tol", [(torch.float32, TOL_GRAD), (torch.float16, TOL_GRAD_HALF),
                                       (torch.bfloat16, TOL_GRAD_HALF)])
@pytest.mark.parametrize("B,L,V,S", [(2, 7, 37, 5), (3, 5, 1000, 20), (2, 3, 12345, 33), (1, 4, 4099, 64),
                                     (2, 2, 8, 3), (1, 3, 42000, 64), (1, 2, 5003, 300)])
@pytest.mark.parametrize("transposed", [False, True])
def test_gather_matches_oracle(dtype, tol, B, L, V, S, transposed):
    g = torch.Generator().manual_seed(V + S)
    logits = (torch.randn(B, L, V, generator=g) * 2.0).to(dtype)
    idx = torch.randint(0, V, (B, L, S), generator=g)
    idx[:, :, -1] = idx[:, :, 0]                       # duplicates accumulate
    gsel = torch.randn(B, L, S, generator=g)
    gsel[0, 0] = 0                                     # a row without gradient
    sel, dx = gather_case(logits, idx, gsel, transposed)
    ref_sel = oracle.logsoftmax_gather(logits.float().numpy(), idx.numpy())
    ref_dx = oracle.logsoftmax_gather_backward(logits.float().numpy(), idx.numpy(), gsel.numpy())
    assert sel.dtype == torch.float32 and dx.dtype == dtype
    assert_rel(sel.numpy(), ref_sel, TOL_SEL, "sel")
    if dtype == torch.float32:
        assert_rel(dx.numpy(), ref_dx, tol, "dlogits")
    else:
        assert_rel_quantized(dx.float().numpy(), ref_dx, tol, str(dtype).replace("torch.", ""), "dlogits")
        # the plain rule as well (2e-3 in fp16; in bf16 the format's own rounding bound, 2^-8)
        assert_rel(dx.float().numpy(), ref_dx, plain_tol_16bit(str(dtype).replace("torch.", ""), tol), "dlogits")


@pytest.mark.parametrize("name,tol", [("gather_small_f32", TOL_GRAD), ("gather_small_f16", TOL_GRAD_HALF),
                                      ("gather_small_bf16", TOL_GRAD_HALF)])
def test_gather_matches_reference_golden(name, tol):
    g = golden(name)
    dtype = getattr(torch, str(g["dtype"]))
    sel, dx = gather_case(torch.as_tensor(g["logits"]).to(dtype), torch.as_tensor(g["select_idx"]),
                          torch.as_tensor(g["grad_sel"]))
    assert_rel(sel.numpy(), g["sel"], TOL_SEL, "sel vs twin")
    if dtype == torch.float32:
        assert_rel(dx.numpy(), g["dlogits"], tol, "dlogits vs twin")
    else:
        name16 = str(dtype).replace("torch.", "")
        assert_rel_quantized(dx.float().numpy(), g["dlogits_f64"], tol, name16, "dlogits vs fp64")
        assert_rel(dx.float().numpy(), g["dlogits_f64"], plain_tol_16bit(name16, tol), "dlogits vs fp64, plain rule")
        # both round the same fp32 value once: they may differ by one unit in the last place
        ulp = 2.0 ** (np.floor(np.log2(np.maximum(np.abs(g["dlogits"]), 1e-30))) - (10 if dtype == torch.float16 else 7))
        assert (np.abs(dx.float().numpy() - g["dlogits"]) <= ulp + 1e-12).all()


def test_gather_autograd_contract():
    """What the reference wrapper guarantees (dag_loss.py:172-233)."""
    batch = workloads.small_batch(seed=21, B=2, L=10, T=4, V=33)
    x = batch.logits.to(DEV).requires_grad_()
    idx = batch.to(DEV).select_idx                     # stride-(T,0,1) expand, not contiguous
    assert not idx.is_contiguous()
    with pytest.raises(RuntimeError):                  # a leaf that requires grad cannot be modified in place
        dag_logsoftmax_gather_inplace(x, idx)
    work = x.clone()
    version = work._version
    out, sel = dag_logsoftmax_gather_inplace(work, idx)
    assert out is work and work._version > version
    ref = oracle.logsoftmax_gather(batch.logits.numpy(), batch.select_idx.numpy())
    assert_rel(sel.detach().cpu().numpy(), ref, TOL_SEL, "sel with expanded index")
    with pytest.raises(AssertionError):                # the returned logits must not be used
        (sel.sum() + out.sum()).backward()
    # without grad the input is left untouched
    keep = batch.logits.to(DEV)
    snapshot = keep.clone()
    with torch.no_grad():
        dag_logsoftmax_gather_inplace(keep, idx)
    assert torch.equal(keep, snapshot)
    # grad arrives in the logits dtype through a transposed consumer, as in the criterion
    work = x.clone()
    _, sel = dag_logsoftmax_gather_inplace(work, idx)
    match = sel.transpose(1, 2)
    w = torch.randn_like(match)
    (match * w).sum().backward()
    ref_dx = oracle.logsoftmax_gather_backward(batch.logits.numpy(), batch.select_idx.numpy(),
                                               w.transpose(1, 2).cpu().numpy())
    assert_rel(x.grad.cpu().numpy(), ref_dx, TOL_GRAD, "dlogits through transpose")


def test_config0_end_to_end_against_reference_golden():
    """C0: gather -> best alignment -> loss -> backward, chained as the criterion does."""
    g = golden("config0")
    batch = workloads.config0().to(DEV)
    logits = batch.logits.clone().requires_grad_()
    links = batch.links.clone().requires_grad_()
    _, sel = dag_logsoftmax_gather_inplace(logits.clone(), batch.select_idx)
    match = sel.transpose(1, 2)
    assert_rel(match[:, :, ::7].detach().cpu().numpy(), g["match_slice"], TOL_SEL, "match")
    path = dag_best_alignment(match.detach(), links.detach(), batch.output_length, batch.target_length)
    assert np.array_equal(path.cpu().numpy(), g["path_f32"])
    loss = dag_loss(match, links, batch.output_length, batch.target_length)
    assert_rel(loss.detach().cpu().numpy(), g["loss_f64"], TOL_LOSS, "loss")
    match.retain_grad()
    loss.sum().backward()
    gm = match.grad.cpu().numpy()
    assert_rel(gm.sum(-1), g["grad_match_rowsum_f64"], TOL_GRAD, "posterior row sums")
    assert_rel(gm[:, :, ::7], g["grad_match_slice_f64"], TOL_GRAD, "grad_match")
    assert_rel(links.grad.cpu().numpy()[:, ::5, ::3], g["grad_links_slice_f64"], TOL_GRAD, "grad_links")
    assert_rel(links.grad.sum((1, 2)).cpu().numpy(), g["grad_links_sum_f64"], TOL_GRAD, "grad_links sum")
    # gradient w.r.t. the logits, against the oracle chained the same way
    ref_dx = oracle.logsoftmax_gather_backward(batch.logits.cpu().numpy(), batch.select_idx.cpu().numpy(),
                                               np.swapaxes(gm, 1, 2))
    assert_rel(logits.grad.cpu().numpy(), ref_dx, TOL_GRAD, "dlogits")
    assert last_status() == 0


def _properties(batch, grads=True):
    """Size-independent properties of the DP: posterior marginals sum to one per target
    step, edge posteriors sum to tl-1, both recursions agree on the likelihood, the best
    path is monotone, complete and re-scores to the max-plus score."""
    b = batch.to(DEV)
    B, T, L = b.match_all.shape
    tl, ol = b.target_length, b.output_length
    m = b.match_all.clone().requires_grad_()
    l = b.links.clone().requires_grad_()
    loss = dag_loss(m, l, ol, tl)
    g = torch.linspace(0.5, 1.5, B, device=DEV)
    gm, gl = torch.autograd.grad(loss, [m, l], grad_outputs=g)
    with torch.no_grad():
        loss_a = dag_loss(m.detach(), l.detach(), ol, tl)
    assert_rel(loss_a.cpu().numpy(), loss.detach().cpu().numpy(), TOL_LOSS, "alpha vs beta likelihood")
    tmask = (torch.arange(T, device=DEV).view(1, T) < tl.view(B, 1)).float()
    rows = gm.sum(-1)
    assert torch.allclose(rows, g.view(B, 1) * tmask, rtol=0, atol=2e-4 * float(g.max()))
    assert torch.allclose(gl.sum((1, 2)), g * (tl - 1).float(), rtol=2e-4, atol=0)
    assert (gm >= 0).all() and (gl >= 0).all()
    # best path
    path = dag_best_alignment(m.detach(), l.detach(), ol, tl).cpu().numpy()
    mc, lc = batch.match_all.numpy(), batch.links.numpy()
    for s in range(B):
        pos = np.nonzero(path[s] >= 0)[0]
        assert path[s][pos].tolist() == list(range(int(tl[s])))
        assert pos[0] == 0 and pos[-1] == int(ol[s]) - 1
        score = mc[s, 0, 0] + sum(lc[s, pos[k - 1], pos[k] - pos[k - 1] - 1] + mc[s, k, pos[k]]
                                  for k in range(1, len(pos)))
        assert score <= float(loss[s].detach()) + 1e-3
    return loss.detach().cpu().numpy(), gm.cpu().numpy(), gl.cpu().numpy(), path


def test_properties_at_c4_size_and_oracle_on_a_slice(dag_loss_path):
    batch = workloads.config4(B=24)
    last_status()
    loss, gm, gl, path = _properties(batch)
    assert last_status() & 8 == 0     # no sentence needed the exact fallback
    sl = slice(0, 3)
    rl, rgm, rgl = oracle.dag_loss_fwd_bwd(batch.match_all[sl].numpy(), batch.links[sl].numpy(),
                                           batch.output_length[sl].numpy(), batch.target_length[sl].numpy(),
                                           grad_output=np.linspace(0.5, 1.5, 24)[sl])
    assert_rel(loss[sl], rl, TOL_LOSS, "loss")
    assert_rel(gm[sl], rgm, TOL_GRAD, "grad_match")
    assert_rel(gl[sl], rgl, TOL_GRAD, "grad_links")
    ref_path, _ = oracle.dag_best_alignment(batch.match_all[sl].numpy(), batch.links[sl].numpy(),
                                            batch.output_length[sl].numpy(), batch.target_length[sl].numpy())
    assert np.array_equal(path[sl], ref_path)


def test_properties_at_c1_shape():
    _properties(workloads.config1(B=16, with_logits=False))


def test_properties_at_c3_size_and_oracle_on_one_sentence():
    batch = workloads.config3(B=3)
    loss, gm, gl, path = _properties(batch)
    sl = slice(0, 1)
    rl, rgm, rgl = oracle.dag_loss_fwd_bwd(batch.match_all[sl].numpy(), batch.links[sl].numpy(),
                                           batch.output_length[sl].numpy(), batch.target_length[sl].numpy(),
                                           grad_output=np.array([0.5]))
    assert_rel(loss[sl], rl, TOL_LOSS, "loss")
    assert_rel(gm[sl], rgm, TOL_GRAD, "grad_match")
    assert_rel(gl[sl], rgl, TOL_GRAD, "grad_links")
    ref_path, _ = oracle.dag_best_alignment(batch.match_all[sl].numpy(), batch.links[sl].numpy(),
                                            batch.output_length[sl].numpy(), batch.target_length[sl].numpy())
    assert np.array_equal(path[sl], ref_path)


def test_invalid_lengths_do_not_trap():
    batch = workloads.small_batch(seed=31, B=4, L=30, T=6, V=20)
    ol, tl = batch.output_length.clone(), batch.target_length.clone()
    tl[1] = 1               # the reference asserts target_length >= 2
    ol[2] = tl[2] - 1       # graph smaller than the target
    ol[3] = 31              # beyond the padded size
    last_status()
    m = batch.match_all.to(DEV).requires_grad_()
    l = batch.links.to(DEV).requires_grad_()
    loss = dag_loss(m, l, ol.to(DEV), tl.to(DEV))
    gm, gl = torch.autograd.grad(loss, [m, l], grad_outputs=torch.ones_like(loss))
    assert torch.isfinite(loss[0]) and torch.isneginf(loss[1:]).all()
    assert (gm[1:] == 0).all() and (gl[1:] == 0).all() and torch.isfinite(gm).all() and torch.isfinite(gl).all()
    path = dag_best_alignment(m.detach(), l.detach(), ol.to(DEV), tl.to(DEV))
    assert (path[1:] == -1).all() and (path[0] >= 0).sum() == tl[0]
    assert last_status() & 1
    # band too narrow for the target: no path at all (the reference asserts, dag_best_alignment.cu:69)
    batch = workloads.small_batch(seed=32, B=2, L=40, T=4, V=20, translen=3, ragged=False)
    path = dag_best_alignment(batch.match_all.to(DEV), batch.links.to(DEV), batch.output_length.to(DEV),
                              batch.target_length.to(DEV))
    assert (path == -1).all()
    assert last_status() & 2
    with torch.no_grad():
        loss = dag_loss(batch.match_all.to(DEV), batch.links.to(DEV), batch.output_length.to(DEV),
                        batch.target_length.to(DEV))
    assert torch.isneginf(loss).all()


def test_host_side_argument_errors():
    batch = workloads.small_batch(seed=33, B=2, L=12, T=4, V=20).to(DEV)
    with pytest.raises(RuntimeError, match="batch size"):
        dag_loss(batch.match_all, batch.links[:1], batch.output_length, batch.target_length)
    with pytest.raises(RuntimeError, match="long"):
        dag_loss(batch.match_all, batch.links, batch.output_length.int(), batch.target_length)
    with pytest.raises(RuntimeError, match="float32"):
        dag_loss(batch.match_all.double(), batch.links.double(), batch.output_length, batch.target_length)
    with pytest.raises(RuntimeError, match="CUDA"):
        dag_loss(batch.match_all.cpu(), batch.links, batch.output_length, batch.target_length)
    with pytest.raises(RuntimeError, match="contiguous"):
        dag_logsoftmax_gather_inplace(batch.logits.transpose(0, 1).contiguous().transpose(0, 1), batch.select_idx)
    with pytest.raises(RuntimeError, match="long"):
        dag_logsoftmax_gather_inplace(batch.logits.clone(), batch.select_idx.int())
    with pytest.raises(RuntimeError, match="dtype"):
        dag_logsoftmax_gather_inplace(batch.logits.double(), batch.select_idx)


def test_empty_batch():
    m = torch.empty(0, 4, 8, device=DEV)
    l = torch.empty(0, 8, 7, device=DEV)
    z = torch.empty(0, dtype=torch.long, device=DEV)
    assert dag_loss(m, l, z, z).shape == (0,)
    assert dag_best_alignment(m, l, z, z).shape == (0, 8)
    _, sel = dag_logsoftmax_gather_inplace(torch.empty(0, 8, 5, device=DEV), torch.empty(0, 8, 3, dtype=torch.long, device=DEV))
    assert sel.shape == (0, 8, 3)


def test_fast_path_hands_extreme_dynamic_range_to_the_exact_kernels(dag_loss_path):
    """Inputs whose probabilities leave the fp32 range of the probability-domain recursion
    (links of -150 nats underflow exp(); match rows spanning hundreds of nats) must still
    meet the tolerances: the fast path detects them and recomputes those sentences exactly."""
    batch = workloads.small_batch(seed=61, B=6, L=40, T=7, V=30, ragged=False)
    links = batch.links.clone()
    links[0] = torch.where(torch.isfinite(links[0]), torch.full_like(links[0], -150.0), links[0])
    g = torch.Generator().manual_seed(5)
    match = batch.match_all.clone()
    match[1] = torch.randn(match[1].shape, generator=g) * 120.0
    match[2, 3, :] = -400.0
    match[2, 3, 17] = 0.0
    links[3] = torch.where(torch.isfinite(links[3]), links[3] * 12.0, links[3])
    batch.links, batch.match_all = links, match
    last_status()
    check_dag_against_oracle(batch)
    if dag_loss_path == "fast":
        assert last_status() & 8


def test_c1_shaped_chain_with_fp16_logits(dag_loss_path):
    """C1 shape (ragged lengths, L = 8 x source, V = 42000, fp16 logits), chained like the
    criterion: gather -> alignment -> loss -> backward down to the logits.  Checked through
    size-independent properties and, on a few rows, against the oracle."""
    batch = workloads.config1(B=6).to(DEV)
    B, L, V = batch.logits.shape
    tl, ol = batch.target_length, batch.output_length
    logits = batch.logits.clone().requires_grad_()
    links = batch.links.clone().requires_grad_()
    last_status()
    _, sel = dag_logsoftmax_gather_inplace(logits.clone(), batch.select_idx)
    match = sel.transpose(1, 2)
    path = dag_best_alignment(match.detach(), links.detach(), ol, tl)
    loss = dag_loss(match, links, ol, tl)
    assert torch.isfinite(loss).all()
    (-(loss / tl).mean()).backward()
    assert last_status() == 0
    # gather rows against the oracle
    rows = [(0, 0), (1, 7), (B - 1, int(ol[B - 1]) - 1)]
    for b, l in rows:
        ref = oracle.logsoftmax_gather(batch.logits[b:b + 1, l:l + 1].float().cpu().numpy(),
                                       batch.targets[b:b + 1].unsqueeze(1).cpu().numpy())
        assert_rel(sel[b, l].detach().cpu().numpy()[None, None], ref, TOL_SEL, "sel row")
    # the gradient of a log-softmax sums to zero over the vocabulary; padded rows get none
    dl = logits.grad.float()
    rowsum = dl.sum(-1).abs().max().item()
    assert rowsum <= 2e-3 * dl.abs().max().item() * 8
    for b in range(B):
        assert (dl[b, int(ol[b]):] == 0).all()
    # every aligned path is complete and monotone
    p = path.cpu().numpy()
    for b in range(B):
        pos = np.nonzero(p[b] >= 0)[0]
        assert p[b][pos].tolist() == list(range(int(tl[b]))) and pos[-1] == int(ol[b]) - 1
    assert torch.isfinite(links.grad).all() and (links.grad <= 0).all()   # d(-loss)/d links <= 0


@pytest.mark.gpu
def test_sentence_stats_kernel_matches_the_criterion_expression():
    """fs_plugins/criterions/nat_dag_loss.py:190-194: inf/nan likelihoods are zeroed and counted."""
    from da_transformer_b200 import dist as ddist
    gen = torch.Generator().manual_seed(5)
    for B in (1, 7, 512, 3000):
        loss = -torch.rand(B, generator=gen) * 900
        tl = torch.randint(2, 65, (B,), generator=gen)
        if B >= 7:
            loss[1] = float("-inf")
            loss[3] = float("nan")
            loss[B - 1] = float("inf")
        want = ddist.sentence_stats(loss, tl)                       # torch expression (CPU tensors)
        got = ddist.sentence_stats(loss.to(DEV), tl.to(DEV)).cpu()  # one launch of the library
        assert got.dtype == torch.float64
        assert torch.equal(got[1:], want[1:])
        assert abs(float(got[0] - want[0])) <= 1e-9 * max(1.0, abs(float(want[0])))
