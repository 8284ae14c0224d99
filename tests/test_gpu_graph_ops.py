"""GPU parity of the fused glue and of the producers / consumers of the transition matrix:
dag_match (gather + arg-max + forced alignment in one pass), dag_loss_mean, glat_alignment,
dag_links_from_heads (extract_links tail, forward + backward), dag_node_passing_prob and
dag_viterbi_decode, against the oracle and the fixtures made by the reference's own code."""
import numpy as np
import pytest
import torch

from oracle import oracle
from da_transformer_b200 import (dag_best_alignment, dag_links_from_heads, dag_logsoftmax_gather_inplace,
                                 dag_loss, dag_loss_mean, dag_match, dag_node_passing_prob, dag_viterbi_decode,
                                 glat_alignment, last_status, workloads)
from util import assert_rel, assert_rel_quantized, golden, plain_tol_16bit

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL_SEL, TOL_GRAD, TOL_GRAD_HALF = 2e-6, 1e-4, 2e-3


# ----------------------------------------------------------------------------- dag_match
def _force_emit(B, L, T, tl, gen):
    """A monotone forced alignment of some target steps (what the glancing sampler hands back)."""
    fe = torch.full((B, L), -1, dtype=torch.long)
    for b in range(B):
        steps = sorted(torch.randperm(int(tl[b]), generator=gen)[: max(1, int(tl[b]) // 3)].tolist())
        verts = sorted(torch.randperm(L, generator=gen)[: len(steps)].tolist())
        for s, v in zip(steps, verts):
            fe[b, v] = s
    return fe


@pytest.mark.parametrize("dtype,tol", [(torch.float32, TOL_GRAD), (torch.float16, TOL_GRAD_HALF),
                                       (torch.bfloat16, TOL_GRAD_HALF)])
@pytest.mark.parametrize("forced", [False, True])
@pytest.mark.parametrize("B,L,T,V", [(3, 17, 6, 41), (2, 9, 5, 4099), (2, 33, 12, 1000)])
def test_dag_match_values_argmax_and_gradient(dtype, tol, forced, B, L, T, V):
    gen = torch.Generator().manual_seed(V + L)
    batch = workloads.small_batch(seed=V + T, B=B, L=L, T=T, V=V, dtype=dtype)
    fe = _force_emit(B, L, T, batch.target_length, gen) if forced else None
    x = batch.logits.to(DEV).requires_grad_()
    tgt = batch.targets.to(DEV)
    work = x.clone()
    last_status()
    out, match, pred = dag_match(work, tgt, force_emit=None if fe is None else fe.to(DEV), return_argmax=True)
    assert out is work and match.shape == (B, T, L) and match.is_contiguous()
    assert torch.equal(pred, batch.logits.to(DEV).argmax(-1))
    x64 = batch.logits.float().numpy()
    ref = np.ascontiguousarray(np.swapaxes(oracle.logsoftmax_gather(x64, batch.select_idx.numpy()), 1, 2))
    if forced:
        ref = oracle.force_alignment(ref, fe.numpy())
    assert_rel(match.detach().cpu().numpy(), ref, TOL_SEL, "match")
    w = torch.randn(B, T, L, generator=gen)
    match.backward(w.to(DEV))
    gsel = w.numpy().copy()
    if forced:
        for b in range(B):
            gsel[b, np.unique(fe[b][fe[b] >= 0].numpy())] = 0     # no gradient into a forced step
    ref_dx = oracle.logsoftmax_gather_backward(x64, batch.select_idx.numpy(), np.swapaxes(gsel, 1, 2))
    if dtype == torch.float32:
        assert_rel(x.grad.cpu().numpy(), ref_dx, tol, "dlogits")
    else:
        name16 = str(dtype).replace("torch.", "")
        assert_rel_quantized(x.grad.float().cpu().numpy(), ref_dx, tol, name16, "dlogits")
        assert_rel(x.grad.float().cpu().numpy(), ref_dx, plain_tol_16bit(name16, tol), "dlogits, plain rule")
    assert last_status() == 0


def test_dag_match_equals_the_unfused_sequence():
    """Same numbers as gather -> transpose -> _force_aligment (nat_dag_loss.py:111-120, 166-179)."""
    g = golden("force_alignment")
    B, T, L = g["match"].shape
    V = 50
    gen = torch.Generator().manual_seed(7)
    logits = torch.randn(B, L, V, generator=gen).to(DEV)
    tgt = torch.randint(0, V, (B, T), generator=gen).to(DEV)
    fe = torch.as_tensor(g["force_emit"]).to(DEV)
    _, sel = dag_logsoftmax_gather_inplace(logits.clone(), tgt.unsqueeze(1).expand(-1, L, -1))
    match = sel.transpose(1, 2)
    matchmask = torch.zeros(B, T + 1, L, dtype=torch.bool, device=DEV).scatter_(1, fe.unsqueeze(1) + 1, 1)[:, 1:]
    target_mask = matchmask.sum(dim=-1, keepdim=True) > 0
    want = match.masked_fill(target_mask, 0) + torch.zeros_like(match).masked_fill_(
        ~matchmask, float("-inf")).masked_fill_(~target_mask, 0)
    _, got, _ = dag_match(logits.clone(), tgt, force_emit=fe)
    assert torch.equal(got, want)
    # the fixture itself (values produced by the reference's method) through the oracle's rule
    assert np.array_equal(oracle.force_alignment(g["match"], g["force_emit"]), g["forced"])


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_argmax_ties_nan_and_infinite_rows(dtype):
    V = 1031
    x = torch.zeros(8, 1, V, dtype=dtype)
    x[0, 0, 100] = 3; x[0, 0, 700] = 3; x[0, 0, 5] = 3          # ties: first index
    x[1, 0, :] = 1.5                                             # all equal
    x[2, 0, :] = float("-inf")                                   # nothing finite
    x[3, 0, 400] = float("nan"); x[3, 0, 900] = float("nan"); x[3, 0, 10] = 9   # NaN counts as the maximum
    x[4, 0, 1030] = float("inf"); x[4, 0, 6] = float("inf")
    x[5, 0, :] = torch.randn(V).to(dtype)
    x[6, 0, V - 1] = 2                                           # scalar tail of an unaligned row
    x[7, 0, 0] = 2
    tgt = torch.zeros(8, 2, dtype=torch.long)
    xd = x.to(DEV)
    _, _, pred = dag_match(xd.clone(), tgt.to(DEV), return_argmax=True)
    assert torch.equal(pred, xd.argmax(-1)), (pred.flatten().tolist(), xd.argmax(-1).flatten().tolist())
    last_status()


def test_argmax_at_vocabulary_size_with_many_ties():
    """bf16 logits of a 42000-word vocabulary repeat values often: many exact ties per row."""
    g = torch.Generator().manual_seed(3)
    x = (torch.randn(4, 37, 42000, generator=g) * 2).to(torch.bfloat16).to(DEV)
    tgt = torch.randint(0, 42000, (4, 5), generator=g).to(DEV)
    _, _, pred = dag_match(x.clone(), tgt, return_argmax=True)
    assert torch.equal(pred, x.argmax(-1))
    x = torch.round(x.float()).to(torch.float16)       # integers: ties everywhere
    _, _, pred = dag_match(x.clone(), tgt, return_argmax=True)
    assert torch.equal(pred, x.argmax(-1))


def test_dag_loss_mean_matches_the_criterion_expression():
    gen = torch.Generator().manual_seed(11)
    for B in (1, 6, 300):
        lr = (-torch.rand(B, generator=gen) * 500).to(DEV).requires_grad_()
        tl = torch.randint(2, 65, (B,), generator=gen).to(DEV)
        bad = torch.zeros(B, dtype=torch.bool)
        if B >= 6:
            bad[1] = bad[4] = True
        with torch.no_grad():
            lr[bad.to(DEV)] = float("-inf")
            if B >= 6:
                lr[4] = float("nan")
        loss, stats = dag_loss_mean(lr, tl)
        loss.backward()
        ref_in = lr.detach().clone().requires_grad_()
        work = ref_in * 1.0
        invalid = work.isinf().logical_or(work.isnan())
        work = work.masked_fill(invalid, 0)
        want = -(work / tl).mean()
        want.backward()
        assert abs(float(loss.detach()) - float(want.detach())) <= 1e-6 * max(1.0, abs(float(want.detach())))
        assert torch.allclose(lr.grad, ref_in.grad, rtol=1e-6, atol=0)
        assert int(stats[3]) == int(bad.sum()) and int(stats[2]) == B


def test_glat_alignment_equals_the_separate_calls():
    batch = workloads.small_batch(seed=77, B=4, L=40, T=8, V=120).to(DEV)
    keep = batch.logits.clone()
    pred, path, match = glat_alignment(batch.logits, batch.targets, batch.links, batch.output_length,
                                       batch.target_length)
    assert torch.equal(batch.logits, keep)
    with torch.no_grad():
        _, sel = dag_logsoftmax_gather_inplace(keep.clone(), batch.select_idx)
        want_path = dag_best_alignment(sel.transpose(1, 2), batch.links, batch.output_length, batch.target_length)
    assert torch.equal(match, sel.transpose(1, 2)) and torch.equal(path, want_path)
    assert torch.equal(pred, keep.argmax(-1))


# ----------------------------------------------------------------------------- links from heads
def _links_inputs(g):
    content = torch.as_tensor(g["content"]).to(DEV).requires_grad_()
    scores = torch.as_tensor(g["gate_scores"]).to(DEV).requires_grad_()
    nonpad = torch.as_tensor(g["nonpad"]).to(DEV) if g["nonpad"].size else None
    bound_end = torch.as_tensor(g["bound_end"]).to(DEV) if g["bound_end"].size else None
    return content, scores, nonpad, bound_end


@pytest.mark.parametrize("name", ["links_from_heads_nonpad", "links_from_heads_band", "links_from_heads_bound"])
def test_links_from_heads_matches_the_reference_fixture(name):
    g = golden(name)
    content, scores, nonpad, bound_end = _links_inputs(g)
    K = int(g["K"])
    links = dag_links_from_heads(content, torch.log_softmax(scores, -1), nonpad_mask=nonpad, bound_end=bound_end,
                                 max_transition_length=K)
    assert_rel(links.detach().cpu().numpy(), g["links"], 1e-5, "links")
    links.backward(torch.as_tensor(g["grad_links"]).to(DEV))
    assert_rel(content.grad.cpu().numpy(), g["grad_content"], TOL_GRAD, "grad_content")
    assert_rel(scores.grad.cpu().numpy(), g["grad_gate_scores"], TOL_GRAD, "grad_gate_scores")


@pytest.mark.parametrize("B,L,H,K,mask", [(3, 40, 8, 99999, "nonpad"), (2, 70, 16, 12, "nonpad"), (2, 33, 3, 99999, "bound"),
                                          (2, 130, 8, 99999, None), (1, 20, 1, 5, "nonpad"), (2, 48, 32, 20, "nonpad"),
                                          (2, 45, 4, 99999, "bound")])
def test_links_from_heads_matches_oracle(B, L, H, K, mask):
    gen = torch.Generator().manual_seed(L * H)
    content = torch.randn(B, L, L, H, generator=gen) * 2
    log_gates = torch.log_softmax(torch.randn(B, L, H, generator=gen), -1)
    out_len = [L] + torch.randint(2, L + 1, (B - 1,), generator=gen).tolist()
    nonpad = bound_end = None
    if mask == "nonpad":
        nonpad = torch.arange(L).view(1, L) < torch.tensor(out_len).view(B, 1)
    elif mask == "bound":
        bound_end = torch.stack([torch.where(torch.arange(L) < n, n - 1, 0) for n in out_len]).long()
    c = content.to(DEV).requires_grad_()
    lg = log_gates.to(DEV).requires_grad_()
    links = dag_links_from_heads(c, lg, nonpad_mask=None if nonpad is None else nonpad.to(DEV),
                                 bound_end=None if bound_end is None else bound_end.to(DEV), max_transition_length=K)
    Kk = min(K, L - 1)
    ref, _ = oracle.links_from_heads(content.numpy(), log_gates.numpy(), Kk,
                                     None if bound_end is None else bound_end.numpy(),
                                     None if nonpad is None else nonpad.numpy())
    assert links.shape == (B, L, Kk)
    assert_rel(links.detach().cpu().numpy(), ref, 1e-5, "links")
    w = torch.randn(B, L, Kk, generator=gen)
    w[~torch.isfinite(torch.as_tensor(ref))] = 0
    links.backward(w.to(DEV))
    rgc, rgg = oracle.links_from_heads_backward(w.numpy(), content.numpy(), log_gates.numpy(), Kk,
                                                None if bound_end is None else bound_end.numpy(),
                                                None if nonpad is None else nonpad.numpy())
    assert_rel(c.grad.cpu().numpy(), rgc, TOL_GRAD, "grad_content")
    assert_rel(lg.grad.cpu().numpy(), rgg, TOL_GRAD, "grad_log_gates")
    # every vertex with a successor distributes probability one
    tot = torch.logsumexp(links.detach(), -1)
    has = torch.isfinite(tot)
    assert torch.allclose(tot[has], torch.zeros_like(tot[has]), atol=2e-5)


def test_links_from_heads_at_c1_size_feeds_dag_loss():
    """B=8, L=512, H=8 (a slice of the C1 shape): rows normalise, and the result is a valid input of dag_loss."""
    batch = workloads.config1(B=8, with_logits=False).to(DEV)
    B, T, L = batch.match_all.shape
    gen = torch.Generator(device=DEV).manual_seed(5)
    content = (torch.randn(B, L, L, 8, device=DEV, generator=gen)).requires_grad_()
    lg = torch.log_softmax(torch.randn(B, L, 8, device=DEV, generator=gen), -1)
    nonpad = torch.arange(L, device=DEV).view(1, L) < batch.output_length.view(B, 1)
    links = dag_links_from_heads(content, lg, nonpad_mask=nonpad)
    tot = torch.logsumexp(links.detach(), -1)
    has = torch.isfinite(tot)
    assert has.sum() == (batch.output_length - 1).sum()
    assert torch.allclose(tot[has], torch.zeros_like(tot[has]), atol=5e-5)
    loss = dag_loss(batch.match_all, links, batch.output_length, batch.target_length)
    assert torch.isfinite(loss).all()
    loss.sum().backward()
    assert torch.isfinite(content.grad).all()
    # the gradient of a row's scores sums to zero per head (softmax), and is zero outside the valid successors
    assert float(content.grad.sum(2).abs().max()) <= 1e-3
    b0 = int(batch.output_length.argmin())
    n = int(batch.output_length[b0])
    assert (content.grad[b0, :, n:] == 0).all()
    ref, _ = oracle.links_from_heads(content.detach()[:1, :, :, :].cpu().numpy(), lg[:1].cpu().numpy(), L - 1,
                                     None, nonpad[:1].cpu().numpy())
    assert_rel(links[:1].detach().cpu().numpy(), ref, 1e-5, "links, one sentence vs oracle")


# ----------------------------------------------------------------------------- decode-side DPs
def test_node_passing_prob_matches_fixture_and_oracle():
    g = golden("node_pass")
    out = dag_node_passing_prob(torch.as_tensor(g["links"]).to(DEV))
    assert_rel(out.cpu().numpy(), g["node_pass"], 1e-5, "node_pass vs _analyze_graph")
    gen = torch.Generator().manual_seed(9)
    ol = torch.tensor([200, 150, 77])
    sq = workloads.band_to_square(workloads.make_links(3, 200, ol, gen))
    out = dag_node_passing_prob(sq.to(DEV))
    assert_rel(out.cpu().numpy(), oracle.node_passing_prob(sq.numpy()), 1e-5, "node_pass vs oracle")


@pytest.mark.parametrize("name", ["viterbi_plain", "viterbi_joint"])
def test_viterbi_decode_matches_the_reference_fixture(name):
    g = golden(name)
    links = torch.as_tensor(g["links"]).to(DEV)
    keep = links.clone()
    L = links.shape[1]
    max_length = int(2 * L / int(g["scale"]))
    toks, lens, verts, score = dag_viterbi_decode(links, torch.as_tensor(g["logp"]).to(DEV),
                                                  torch.as_tensor(g["output_length"]).to(DEV), max_length,
                                                  joint=bool(g["joint"]), viterbibeta=float(g["beta"]),
                                                  pad_index=int(g["pad"]))
    assert torch.equal(links, keep)
    ref = g["tokens"]
    assert int(lens.max()) == ref.shape[1]
    assert np.array_equal(toks[:, :ref.shape[1]].cpu().numpy(), ref)
    assert (toks[:, ref.shape[1]:] == int(g["pad"])).all()


@pytest.mark.parametrize("joint,beta", [(False, 1.0), (True, 1.0), (True, 0.5)])
def test_viterbi_decode_matches_oracle_at_decoding_size(joint, beta):
    gen = torch.Generator().manual_seed(17)
    B, L, V, scale = 5, 256, 31, 8
    ol = torch.tensor([256, 200, 255, 64, 17])
    sq = workloads.band_to_square(workloads.make_links(B, L, ol, gen))
    logp = torch.log_softmax(torch.randn(B, L, V, generator=gen) * 3, -1)
    ul, ut = logp.max(-1)
    ut[:, ::5] = 1                        # pad tokens inside the path are dropped
    ut[:, 2::5] = ut[:, 3::5][:, : ut[:, 2::5].shape[1]]   # and repeated tokens collapse
    max_length = int(2 * L / scale)
    toks, lens, verts, score = dag_viterbi_decode(sq.to(DEV), (ul.to(DEV), ut.to(DEV)), ol.to(DEV), max_length,
                                                  joint=joint, viterbibeta=beta, pad_index=1)
    rt, rl, rv, rs = oracle.viterbi_decode(sq.numpy(), ul.numpy(), ut.numpy(), ol.numpy(), max_length, joint=joint,
                                           beta=beta, pad=1)
    assert np.array_equal(verts.cpu().numpy(), rv)
    assert np.array_equal(toks.cpu().numpy(), rt) and np.array_equal(lens.cpu().numpy(), rl)
    assert_rel(score.cpu().numpy(), rs, 1e-5, "score")
    assert last_status() == 0


@pytest.mark.parametrize("joint", [False, True])
def test_viterbi_decode_ties_take_the_first_index(joint):
    """Coarsely quantised scores make many candidates tie exactly: the predecessor is torch.max's (the first index of
    the maximum), also where a step keeps only its row and the back-trace re-evaluates the candidates."""
    gen = torch.Generator().manual_seed(23)
    B, L, V, scale = 4, 192, 17, 8
    ol = torch.tensor([192, 100, 191, 33])
    sq = workloads.band_to_square(workloads.make_links(B, L, ol, gen))
    sq = torch.where(torch.isfinite(sq), torch.round(sq * 2) / 2, sq)
    logp = torch.log_softmax(torch.randn(B, L, V, generator=gen), -1)
    ul, ut = logp.max(-1)
    ul = torch.round(ul * 2) / 2
    max_length = int(2 * L / scale)
    toks, lens, verts, score = dag_viterbi_decode(sq.to(DEV), (ul.to(DEV), ut.to(DEV)), ol.to(DEV), max_length,
                                                  joint=joint, viterbibeta=1.0, pad_index=1)
    rt, rl, rv, rs = oracle.viterbi_decode(sq.numpy(), ul.numpy(), ut.numpy(), ol.numpy(), max_length, joint=joint,
                                           beta=1.0, pad=1)
    assert np.array_equal(verts.cpu().numpy(), rv)
    assert np.array_equal(toks.cpu().numpy(), rt) and np.array_equal(lens.cpu().numpy(), rl)
    assert_rel(score.cpu().numpy(), rs, 1e-5, "score")


@pytest.mark.parametrize("B,L,max_length", [(2, 1000, 40), (3, 520, 30), (2, 1300, 12)])
def test_viterbi_decode_long_graphs(B, L, max_length):
    """Graphs of 1000 and 520 vertices are decoded by clusters of 16 and 4 CTAs, 1300 vertices by the general kernel."""
    gen = torch.Generator().manual_seed(31 + L)
    ol = torch.randint(L // 2, L + 1, (B,), generator=gen)
    ol[0] = L
    sq = workloads.band_to_square(workloads.make_links(B, L, ol, gen))
    logp = torch.log_softmax(torch.randn(B, L, 11, generator=gen) * 2, -1)
    ul, ut = logp.max(-1)
    toks, lens, verts, score = dag_viterbi_decode(sq.to(DEV), (ul.to(DEV), ut.to(DEV)), ol.to(DEV), max_length,
                                                  joint=True, viterbibeta=1.0, pad_index=1)
    rt, rl, rv, rs = oracle.viterbi_decode(sq.numpy(), ul.numpy(), ut.numpy(), ol.numpy(), max_length, joint=True,
                                           beta=1.0, pad=1)
    assert np.array_equal(verts.cpu().numpy(), rv)
    assert np.array_equal(toks.cpu().numpy(), rt) and np.array_equal(lens.cpu().numpy(), rl)
    assert_rel(score.cpu().numpy(), rs, 1e-5, "score")
    assert last_status() == 0


def test_viterbi_decode_of_a_matrix_that_is_not_triangular():
    """Finite entries on and below the diagonal: the cluster kernel (which holds only the upper triangle) must leave
    such a sentence to the general kernel, which takes all L candidates; a triangular sentence in the same batch is
    unaffected."""
    gen = torch.Generator().manual_seed(29)
    B, L, V = 3, 96, 13
    ol = torch.tensor([96, 80, 96])
    sq = workloads.band_to_square(workloads.make_links(B, L, ol, gen))
    sq[1] = torch.randn(L, L, generator=gen) - 3.0          # dense
    sq[2, 40, 10] = -0.25                                    # one transition backwards
    logp = torch.log_softmax(torch.randn(B, L, V, generator=gen), -1)
    ul, ut = logp.max(-1)
    max_length = 24
    toks, lens, verts, score = dag_viterbi_decode(sq.to(DEV), (ul.to(DEV), ut.to(DEV)), ol.to(DEV), max_length,
                                                  joint=True, viterbibeta=1.0, pad_index=1)
    rt, rl, rv, rs = oracle.viterbi_decode(sq.numpy(), ul.numpy(), ut.numpy(), ol.numpy(), max_length, joint=True,
                                           beta=1.0, pad=1)
    assert np.array_equal(verts.cpu().numpy(), rv)
    assert np.array_equal(toks.cpu().numpy(), rt) and np.array_equal(lens.cpu().numpy(), rl)
    assert_rel(score.cpu().numpy(), rs, 1e-5, "score")


# ----------------------------------------------------------------------------- host upload
def test_upload_links_moves_the_real_entries_and_the_ops_never_read_the_rest():
    """The band's padding is not transferred; the device copy keeps NaN there, and loss, gradients and
    alignment are bit-identical to those on a whole copy (so no kernel reads a link past output_length)."""
    from da_transformer_b200 import host_io
    batch = workloads.small_batch(seed=93, B=5, L=150, T=20, V=30)
    host = batch.links.contiguous().pin_memory()
    n = int(batch.output_length.max())
    dev_links = torch.full(host.shape, float("nan"), device=DEV)
    host_io.upload_links(host, dev_links, n)
    torch.cuda.synchronize()
    B, L, K = host.shape
    real = (torch.arange(L).view(L, 1) + torch.arange(K).view(1, K) + 1) < n         # i + d + 1 < n
    got = dev_links.cpu()
    assert torch.equal(got[:, real], host[:, real])
    moved = int((~torch.isnan(got)).sum()) * 4
    # the first rows (at least three quarters real) go whole through the copy engine, the others as their real prefixes
    head = max(0, min(n - 1, n - 1 - (3 * K) // 4))
    exact = host_io.upload_links_bytes(B, L, K, n)
    assert exact == (head * K + int(real[head:].sum())) * 4 * B
    assert exact <= moved <= exact + 32 * B * (n - 1)              # plus the rounding to 16-byte units
    assert moved < 0.6 * host.numel() * 4                          # little more than half of the band
    # pageable source: the strided-copy path moves the covering staircase
    dev2 = torch.full(host.shape, float("nan"), device=DEV)
    host_io.upload_links(batch.links.contiguous(), dev2, n)
    torch.cuda.synchronize()
    got2 = dev2.cpu()
    assert torch.equal(got2[:, real], host[:, real])
    assert int((~torch.isnan(got2)).sum()) * 4 == host_io.upload_links_bytes(B, L, K, n, pinned=False)
    b = batch.to(DEV)
    res = []
    for lk in (b.links, dev_links):
        m = b.match_all.clone().requires_grad_()
        l = lk.clone().requires_grad_()
        loss = dag_loss(m, l, b.output_length, b.target_length)
        gm, gl = torch.autograd.grad(loss.sum(), [m, l])
        path = dag_best_alignment(m.detach(), l.detach(), b.output_length, b.target_length)
        res.append((loss.detach(), gm, gl, path))
    assert torch.equal(res[0][0], res[1][0]) and torch.equal(res[0][1], res[1][1]) and torch.equal(res[0][3], res[1][3])
    assert torch.equal(res[0][2][:, real], res[1][2][:, real])


@pytest.mark.gpu
@pytest.mark.parametrize("B,L,K,n", [(3, 96, 20, 96), (2, 130, 129, 77), (4, 64, 63, 2), (1, 40, 8, 33)])
def test_upload_links_shapes(B, L, K, n):
    """Narrow bands (most rows full: they go through the copy engine), graphs shorter than the padded length, the
    smallest graph: every real entry arrives, from page-locked and from pageable memory."""
    from da_transformer_b200 import host_io
    g = torch.Generator().manual_seed(1000 + L + K)
    host = torch.randn(B, L, K, generator=g).contiguous()
    real = ((torch.arange(L).view(L, 1) + torch.arange(K).view(1, K) + 1) < n)
    for src in (host.pin_memory(), host):
        dev_links = torch.full(host.shape, float("nan"), device=DEV)
        host_io.upload_links(src, dev_links, n)
        torch.cuda.synchronize()
        got = dev_links.cpu()
        assert torch.equal(got[:, real], host[:, real])
        moved = int((~torch.isnan(got)).sum()) * 4
        claimed = host_io.upload_links_bytes(B, L, K, n, pinned=src.is_pinned())
        assert claimed <= moved <= claimed + 32 * B * max(n - 1, 0)


@pytest.mark.gpu
def test_overlapped_stats_reducer_keeps_every_submission_apart():
    from da_transformer_b200 import dist as ddist

    dev = torch.device("cuda:0")
    red = ddist.OverlappedStatsReducer(dev, slots=3)
    src = torch.zeros(4, dtype=torch.float64, device=dev)
    got = []
    for k in range(3):
        src.fill_(float(k + 1))          # the producer overwrites its buffer every step
        got.append(red.submit(src))
    red.wait()
    torch.cuda.synchronize()
    assert [float(g[0]) for g in got] == [1.0, 2.0, 3.0]
