"""Parity at the full sizes of the benchmark configurations (the small-case suite is
test_gpu_parity.py): the gather on the real C2 tensors, the fast dag_loss path against the exact
kernels on all 512 C4 sentences, C4-sized sentences against the reference's own CUDA kernels, and
the criterion's call sequence (fs_plugins/criterions/nat_dag_loss.py:155-203, 239-271) executed
through the package and compared with the oracle chained the same way.
"""
import numpy as np
import pytest
import torch

from oracle import oracle, ref_cuda
from da_transformer_b200 import (DagLossFunc, dag_best_alignment, dag_logsoftmax_gather_inplace, dag_loss,
                                 last_status, workloads)
from util import assert_rel, assert_rel_per_sentence, assert_rel_quantized, plain_tol_16bit, rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL_LOSS, TOL_GRAD, TOL_GRAD_HALF, TOL_SEL = 1e-5, 1e-4, 2e-3, 2e-6


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_gather_on_the_full_c2_tensor(dtype):
    """C2 at V = 64000: logits [32, 1024, 64000] (4.19 GB, byte offsets beyond 2^31, every CTA walks
    many rows).  Sampled rows, among them the first, the last and rows past the 2 GiB mark, are checked
    against the oracle: gathered values and the dense gradient."""
    B, L, V, S = 32, 1024, 64000, 128
    g = torch.Generator(device=DEV).manual_seed(workloads.BASE_SEED + 2)
    x = torch.empty(B, L, V, dtype=dtype, device=DEV)
    for b in range(B):   # chunked: the fp32 staging tensor stays small
        x[b] = (torch.randn(L, V, device=DEV, generator=g) * 2.0).to(dtype)
    idx = torch.randint(0, V, (B, L, S), device=DEV, generator=g)
    idx[:, :, 5] = idx[:, :, 3]    # duplicates accumulate
    gsel = torch.randn(B, L, S, device=DEV, generator=g)
    rows = [(0, 0), (0, 1), (7, 511), (16, 400), (16, 401), (19, 544), (25, 1000), (31, 1022), (31, 1023)]
    first_past_2gib = (2 ** 31) // (V * x.element_size()) + 1
    rows.append((first_past_2gib // L, first_past_2gib % L))
    assert max(b * L + l for b, l in rows) * V * x.element_size() > 2 ** 31
    keep = {r: x[r[0], r[1]].float().cpu().numpy() for r in rows}
    xr = x.requires_grad_()
    work = xr.clone()
    del x
    last_status()
    out, sel = dag_logsoftmax_gather_inplace(work, idx)
    assert out is work
    sel.backward(gsel)
    dx = xr.grad
    assert last_status() == 0
    name16 = str(dtype).replace("torch.", "")
    for (b, l), row in keep.items():
        r_idx = idx[b, l].cpu().numpy()[None, None]
        r_g = gsel[b, l].cpu().numpy()[None, None]
        ref_sel = oracle.logsoftmax_gather(row[None, None], r_idx)
        ref_dx = oracle.logsoftmax_gather_backward(row[None, None], r_idx, r_g)
        assert_rel(sel[b, l].detach().cpu().numpy()[None, None], ref_sel, TOL_SEL, f"sel row {(b, l)}")
        got = dx[b, l].float().cpu().numpy()[None, None]
        assert_rel_quantized(got, ref_dx, TOL_GRAD_HALF, name16, f"dlogits row {(b, l)}")
        assert_rel(got, ref_dx, plain_tol_16bit(name16, TOL_GRAD_HALF), f"dlogits row {(b, l)}, plain rule")
    # a log-softmax gradient sums to zero over the vocabulary, on every row of the tensor
    rs = torch.zeros(B, L, device=DEV)
    for b in range(B):
        rs[b] = dx[b].float().sum(-1)
    scale = float(gsel.abs().sum(-1).max())
    assert float(rs.abs().max()) <= 2e-2 * scale


def test_fast_path_against_exact_kernels_on_all_512_c4_sentences():
    """The whole C4 batch through the fast (strip, probability-domain) forward and product-form
    backward, against the exact log-domain kernels on the same inputs."""
    batch = workloads.config4().to(DEV)
    B = batch.match_all.shape[0]
    g = torch.linspace(0.5, 1.5, B, device=DEV)
    res = {}
    for exact in (False, True):
        DagLossFunc.exact = exact
        try:
            m = batch.match_all.clone().requires_grad_()
            l = batch.links.clone().requires_grad_()
            last_status()
            loss = dag_loss(m, l, batch.output_length, batch.target_length)
            gm, gl = torch.autograd.grad(loss, [m, l], grad_outputs=g)
            flagged = last_status() & 8
        finally:
            DagLossFunc.exact = False
        res[exact] = (loss.detach(), gm, gl, flagged)
    assert res[False][3] == 0, "a C4 sentence was handed to the exact kernels"
    lf, gmf, glf, _ = res[False]
    le, gme, gle, _ = res[True]
    assert float(((lf - le).abs() / le.abs()).max()) <= TOL_LOSS
    for b0 in range(0, B, 64):     # per sentence, in slices that fit host memory comfortably
        sl = slice(b0, b0 + 64)
        assert_rel_per_sentence(gmf[sl].cpu().numpy(), gme[sl].cpu().numpy(), TOL_GRAD, "grad_match fast vs exact")
        assert_rel_per_sentence(glf[sl].cpu().numpy(), gle[sl].cpu().numpy(), TOL_GRAD, "grad_links fast vs exact")


@pytest.mark.skipif(not ref_cuda.available(), reason="reference CUDA extension not built")
def test_c4_sized_sentences_against_reference_cuda():
    """Four C4 sentences (L = 512, T = 64) against the reference's CUDA kernels: loss 1e-5, gradients
    2e-4 (two fp32 implementations; the reference's own rounding is ~6e-5 at |loss| ~ 700), alignment
    bit-exact; and each side against the fp64 oracle."""
    batch = workloads.config4(B=4)
    assert ref_cuda.lengths_are_valid(batch.output_length, batch.target_length, 512, 511)
    b = batch.to(DEV)
    g = torch.linspace(0.5, 1.5, 4, device=DEV)
    r_loss, r_gm, r_gl = ref_cuda.dag_loss_fwd_bwd(b.match_all, b.links, b.output_length, b.target_length, g)
    r_path, _ = ref_cuda.dag_best_alignment(b.match_all, b.links, b.output_length, b.target_length)
    o_loss, o_gm, o_gl = oracle.dag_loss_fwd_bwd(batch.match_all.numpy(), batch.links.numpy(),
                                                 batch.output_length.numpy(), batch.target_length.numpy(),
                                                 grad_output=g.cpu().numpy())
    for exact in (False, True):
        DagLossFunc.exact = exact
        try:
            m = b.match_all.clone().requires_grad_()
            l = b.links.clone().requires_grad_()
            loss = dag_loss(m, l, b.output_length, b.target_length)
            gm, gl = torch.autograd.grad(loss, [m, l], grad_outputs=g)
        finally:
            DagLossFunc.exact = False
        assert_rel(loss.detach().cpu().numpy(), r_loss.cpu().numpy(), 1e-5, "loss vs reference CUDA")
        assert_rel(gm.cpu().numpy(), r_gm.cpu().numpy(), 2e-4, "grad_match vs reference CUDA")
        assert_rel(gl.cpu().numpy(), r_gl.cpu().numpy(), 2e-4, "grad_links vs reference CUDA")
        assert_rel(loss.detach().cpu().numpy(), o_loss, TOL_LOSS, "loss vs oracle")
        assert_rel_per_sentence(gm.cpu().numpy(), o_gm, TOL_GRAD, "grad_match vs oracle")
        assert_rel_per_sentence(gl.cpu().numpy(), o_gl, TOL_GRAD, "grad_links vs oracle")
    path = dag_best_alignment(b.match_all, b.links, b.output_length, b.target_length)
    assert torch.equal(path, r_path)
    # how far the reference's own fp32 kernels are from the fp64 truth (reported, not asserted tightly)
    assert rel_err(r_gl.cpu().numpy(), o_gl) <= 5e-4


def _force_alignment_np(match, force_emit):
    """nat_dag_loss.py:111-120 restated: a target step that some vertex is forced to emit keeps
    only that vertex (0 there, -inf elsewhere); other steps are unchanged."""
    B, T, L = match.shape
    out = match.copy()
    for b in range(B):
        for j in range(L):
            t = int(force_emit[b, j])
            if t >= 0:
                out[b, t, :] = -np.inf
        for j in range(L):
            t = int(force_emit[b, j])
            if t >= 0:
                out[b, t, j] = 0.0
    return out


@pytest.mark.parametrize("forced", [False, True])
def test_criterion_call_sequence(forced):
    """What NATDAGLoss does around the ops (glat_function, nat_dag_loss.py:246-271, then
    _compute_dag_loss, :155-194), restated with plain torch glue around this package's ops, against
    the oracle chained the same way: argmax / gather (no grad) / best alignment, then gather /
    transpose / optional forced alignment / dag_loss / inf-nan masking / -(loss/tl).mean() and its
    gradient down to the logits and the links."""
    pad = workloads.PAD_TOKEN
    batch = workloads.small_batch(seed=91, B=5, L=56, T=9, V=97)
    ol_list = batch.output_length.tolist()
    prev = torch.full((5, 56), 7, dtype=torch.long)
    for b, n in enumerate(ol_list):
        prev[b, n:] = pad
    gpu = batch.to(DEV)
    prev = prev.to(DEV)
    tgt = gpu.targets
    B, L, V = gpu.logits.shape
    # ---- glancing pass (no grad)
    with torch.no_grad():
        word_ins_out = gpu.logits.clone()
        target_length = (~tgt.eq(pad)).sum(1)
        output_length = prev.ne(pad).sum(1)
        pred_tokens = word_ins_out.argmax(-1)
        word_ins_out, match = dag_logsoftmax_gather_inplace(word_ins_out, tgt.unsqueeze(1).expand(-1, L, -1))
        match = match.transpose(1, 2)
        path = dag_best_alignment(match, gpu.links, output_length, target_length)
    assert torch.equal(target_length, gpu.target_length) and torch.equal(output_length, gpu.output_length)
    x64 = batch.logits.numpy().astype(np.float64)
    o_sel = oracle.logsoftmax_gather(x64, batch.select_idx.numpy())
    o_match = np.ascontiguousarray(np.swapaxes(o_sel, 1, 2))
    ol, tl = batch.output_length.numpy(), batch.target_length.numpy()
    o_path, _ = oracle.dag_best_alignment(match.cpu().numpy(), batch.links.numpy(), ol, tl)
    assert np.array_equal(path.cpu().numpy(), o_path)
    assert np.array_equal(pred_tokens.cpu().numpy(), x64.argmax(-1))
    force_emit = None
    if forced:   # keep every third aligned vertex, as the sampler's next_force_emit does
        keep = torch.zeros(B, L, dtype=torch.bool, device=DEV)
        keep[:, ::3] = True
        force_emit = path.masked_fill(~keep, -1)
    # ---- loss pass
    outputs = gpu.logits.clone().requires_grad_()
    links = gpu.links.clone().requires_grad_()
    work = outputs.clone()
    work, match = dag_logsoftmax_gather_inplace(work, tgt.unsqueeze(1).expand(-1, L, -1))
    match = match.transpose(1, 2)
    if force_emit is not None:
        tarlen = match.shape[1]
        matchmask = torch.zeros(B, tarlen + 1, L, dtype=torch.bool, device=DEV).scatter_(
            1, force_emit.unsqueeze(1) + 1, 1)[:, 1:]
        target_mask = matchmask.sum(dim=-1, keepdim=True) > 0
        match = match.masked_fill(target_mask, 0) + torch.zeros_like(match).masked_fill_(
            ~matchmask, float("-inf")).masked_fill_(~target_mask, 0)
    loss_result = dag_loss(match, links, output_length, target_length)
    invalid = loss_result.isinf().logical_or(loss_result.isnan())
    loss_result.masked_fill_(invalid, 0)
    loss = -(loss_result / target_length).mean()
    loss.backward()
    # ---- the oracle, chained the same way
    fe = None if force_emit is None else force_emit.cpu().numpy()
    om = o_match if fe is None else _force_alignment_np(o_match, fe)
    g = -1.0 / (tl * B)
    o_loss, o_gm, o_gl = oracle.dag_loss_fwd_bwd(om, batch.links.numpy(), ol, tl, grad_output=g)
    bad = ~np.isfinite(o_loss)
    o_gm[bad] = 0
    o_gl[bad] = 0
    if fe is not None:   # masked_fill(target_mask, 0) cuts the gradient of the forced steps
        forced_t = np.zeros((B, om.shape[1]), dtype=bool)
        for b in range(B):
            forced_t[b, fe[b][fe[b] >= 0]] = True
        o_gm[forced_t] = 0
    o_total = -np.where(bad, 0.0, o_loss / tl).mean()
    o_dx = oracle.logsoftmax_gather_backward(x64, batch.select_idx.numpy(), np.swapaxes(o_gm, 1, 2))
    assert abs(float(loss.detach()) - o_total) <= TOL_LOSS * abs(o_total)
    assert_rel(links.grad.cpu().numpy(), o_gl, TOL_GRAD, "d loss / d links")
    assert_rel(outputs.grad.cpu().numpy(), o_dx, TOL_GRAD, "d loss / d logits")
    assert int(invalid.sum()) == int(bad.sum())


@pytest.mark.parametrize("forced", [False, True])
def test_peaky_trained_like_c4_sentences(forced):
    """C4 shapes with a trained graph's value distribution (transition scores x 8, one dominant vertex
    per target token), optionally with the criterion's forced alignment (0 / -inf rows in match): both
    dag_loss paths against the fp64 oracle, alignment bit-exact."""
    batch = workloads.config4_peaky(B=6)
    match = batch.match_all.numpy()
    links = batch.links.numpy()
    ol, tl = batch.output_length.numpy(), batch.target_length.numpy()
    b = batch.to(DEV)
    path = dag_best_alignment(b.match_all, b.links, b.output_length, b.target_length)
    o_path, _ = oracle.dag_best_alignment(match, links, ol, tl)
    assert np.array_equal(path.cpu().numpy(), o_path)
    if forced:
        fe = o_path.copy()
        fe[:, 1::3] = -1
        fe[:, 2::3] = -1
        match = oracle.force_alignment(match, fe).astype(np.float32)
    g = np.linspace(0.5, 1.5, 6)
    o_loss, o_gm, o_gl = oracle.dag_loss_fwd_bwd(match, links, ol, tl, grad_output=g)
    assert np.isfinite(o_loss).all()
    for exact in (False, True):
        DagLossFunc.exact = exact
        try:
            m = torch.as_tensor(match, device=DEV).requires_grad_()
            l = b.links.clone().requires_grad_()
            loss = dag_loss(m, l, b.output_length, b.target_length)
            gm, gl = torch.autograd.grad(loss, [m, l], grad_outputs=torch.as_tensor(g, dtype=torch.float32, device=DEV))
            with torch.no_grad():
                loss_ng = dag_loss(m.detach(), l.detach(), b.output_length, b.target_length)
        finally:
            DagLossFunc.exact = False
        assert_rel(loss.detach().cpu().numpy(), o_loss, TOL_LOSS, f"loss (exact={exact})")
        assert_rel(loss_ng.cpu().numpy(), o_loss, TOL_LOSS, f"loss without grad (exact={exact})")
        assert_rel_per_sentence(gm.cpu().numpy(), o_gm, TOL_GRAD, f"grad_match (exact={exact})")
        assert_rel_per_sentence(gl.cpu().numpy(), o_gl, TOL_GRAD, f"grad_links (exact={exact})")
    last_status()
