"""The package's torch-native twins against the golden vectors of the reference's twins."""
import numpy as np
import pytest
import torch

from da_transformer_b200 import (torch_dag_best_alignment, torch_dag_logsoftmax_gather_inplace, torch_dag_loss,
                                 workloads)
from util import assert_rel, golden


@pytest.mark.parametrize("name", ["dag_small_full", "dag_small_band", "dag_small_even"])
def test_twin_loss_gradients_and_path(name):
    g = golden(name)
    match = torch.tensor(g["match_all"], dtype=torch.float64, requires_grad=True)
    band = torch.tensor(g["links"], dtype=torch.float64, requires_grad=True)
    ol, tl = torch.tensor(g["output_length"]), torch.tensor(g["target_length"])
    loss = torch_dag_loss(match, workloads.band_to_square(band), ol, tl)
    assert_rel(loss.detach().numpy(), g["loss"], 1e-12, "loss")
    fin = torch.isfinite(loss)
    gm, gl = torch.autograd.grad(loss[fin].sum(), [match, band])
    assert torch.isfinite(gm).all() and torch.isfinite(gl).all()
    assert_rel(gm.numpy(), g["grad_match"], 1e-10, "grad_match")
    assert_rel(gl.numpy(), g["grad_links"], 1e-10, "grad_links")
    path = torch_dag_best_alignment(match.detach(), workloads.band_to_square(band.detach()), ol, tl).numpy()
    ok = np.isfinite(g["max_loss"])
    assert np.array_equal(path[ok], g["path"][ok])


def test_twin_gather():
    g = golden("gather_small_f16")
    x = torch.tensor(g["logits"]).half()
    out, sel = torch_dag_logsoftmax_gather_inplace(x, torch.tensor(g["select_idx"]))
    assert out is x and sel.dtype == torch.float32
    assert_rel(sel.numpy(), g["sel"], 1e-6, "sel")
