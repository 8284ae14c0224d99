"""Our CUDA path against the REFERENCE'S OWN CUDA kernels (compiled unmodified by
oracle/build_ref.py into oracle/_ref/, which travels to the GPU box but is never committed).
Skipped when that build is absent.  Only valid lengths are fed to the reference: its kernels
trap the context otherwise.

Both sides are fp32 implementations of the same formulas; the reference evaluates
exp(alpha + beta - Z) with |alpha| ~ |loss|, so its own rounding noise is ~1 ulp of |loss|
(6e-5 relative at |loss| ~ 700).  Gradients are therefore compared at 2e-4 against each
other; each side is held to 1e-4 against the fp64 oracle elsewhere.
"""
import numpy as np
import pytest
import torch

from oracle import oracle, ref_cuda
from da_transformer_b200 import (DagLossFunc, dag_best_alignment, dag_logsoftmax_gather_inplace, dag_loss,
                                 workloads)
from util import assert_rel, rel_err

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not ref_cuda.available(), reason="reference CUDA extension not built")]
DEV = "cuda:0"


def _valid_batch(seed, B, L, T):
    batch = workloads.small_batch(seed=seed, B=B, L=L, T=T, V=40, ragged=True)
    assert ref_cuda.lengths_are_valid(batch.output_length, batch.target_length, L, L - 1)
    return batch.to(DEV)


@pytest.mark.parametrize("exact", [False, True])
@pytest.mark.parametrize("seed,B,L,T", [(71, 4, 40, 7), (72, 6, 130, 20), (73, 3, 300, 40)])
def test_dag_loss_against_reference_cuda(seed, B, L, T, exact):
    b = _valid_batch(seed, B, L, T)
    g = torch.linspace(0.5, 1.5, B, device=DEV)
    r_loss, r_gm, r_gl = ref_cuda.dag_loss_fwd_bwd(b.match_all, b.links, b.output_length, b.target_length, g)
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
    # and who is closer to the fp64 truth
    o_loss, o_gm, o_gl = oracle.dag_loss_fwd_bwd(b.match_all.cpu().numpy(), b.links.cpu().numpy(),
                                                 b.output_length.cpu().numpy(), b.target_length.cpu().numpy(),
                                                 grad_output=g.cpu().numpy())
    ours = rel_err(gl.cpu().numpy(), o_gl)
    assert ours <= 1e-4


@pytest.mark.parametrize("config", [1, 2, 3, 4])
@pytest.mark.parametrize("quant", [0.0, 0.5])
def test_best_alignment_bit_exact_against_reference_cuda(config, quant):
    from da_transformer_b200 import DagBestAlignmentFunc

    b = _valid_batch(74, 5, 97, 13)
    match, links = b.match_all, b.links
    if quant:
        match = torch.round(match / quant) * quant
        links = torch.round(links / quant) * quant
    r_path, _ = ref_cuda.dag_best_alignment(match, links, b.output_length, b.target_length, config)
    DagBestAlignmentFunc.config = config
    try:
        path = dag_best_alignment(match, links, b.output_length, b.target_length)
    finally:
        DagBestAlignmentFunc.config = 1
    assert torch.equal(path, r_path)


def test_gather_against_reference_cuda_fp16():
    g = torch.Generator().manual_seed(75)
    x = (torch.randn(3, 9, 12347, generator=g) * 2).to(torch.float16).to(DEV)
    idx = torch.randint(0, 12347, (3, 9, 21), generator=g).to(DEV)
    gsel = torch.randn(3, 9, 21, generator=g).to(DEV)
    ref_in = x.clone()
    r_sel = ref_cuda.logsoftmax_gather(ref_in, idx, True)
    r_dx = ref_cuda.logsoftmax_gather_backward(ref_in, idx, gsel)
    xr = x.clone().requires_grad_()
    _, sel = dag_logsoftmax_gather_inplace(xr.clone(), idx)
    (dx,) = torch.autograd.grad(sel, [xr], grad_outputs=gsel)
    assert_rel(sel.detach().cpu().numpy(), r_sel.cpu().numpy(), 5e-6, "sel vs reference CUDA")
    # the reference rounds both factors to fp16 before multiplying (dag_loss.py:228-229)
    assert_rel(dx.float().cpu().numpy(), r_dx.float().cpu().numpy(), 2e-3, "dlogits vs reference CUDA")
