"""Generates the golden fixtures in this directory from the REFERENCE's own
torch-native implementation (fs_plugins/custom_ops/dag_loss.py: torch_dag_loss
:259-300, torch_dag_best_alignment :322-353, torch_dag_logsoftmax_gather_inplace
:355-359), imported in place from a checkout of thu-coai/DA-Transformer.

    python tests/golden/make_golden.py --reference /path/to/DA-Transformer

The checkout is only needed to (re)generate the fixtures; the tests read the
committed .npz files.  Inputs of the small cases are stored in the fixture; the
configuration-0 case stores outputs plus input checksums (its inputs are
regenerated from the seed by da_transformer_b200.workloads.config0).
"""
import argparse
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from da_transformer_b200 import workloads  # noqa: E402


def load_reference(root):
    path = os.path.join(root, "fs_plugins", "custom_ops", "dag_loss.py")
    spec = importlib.util.spec_from_file_location("ref_dag_loss", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def twin_dag(ref, match, band, ol, tl, dtype):
    """loss, grad_match, grad_links(band), path from the torch twins."""
    match = match.to(dtype).clone().requires_grad_()
    band = band.to(dtype).clone().requires_grad_()
    sq = workloads.band_to_square(band)
    loss = ref.torch_dag_loss(match, sq, ol, tl)
    finite = torch.isfinite(loss)
    gm, gl = torch.autograd.grad(loss[finite].sum(), [match, band], allow_unused=True)
    gm = torch.zeros_like(match) if gm is None else gm
    gl = torch.zeros_like(band) if gl is None else gl
    path = ref.torch_dag_best_alignment(match.detach().clone(), sq.detach(), ol, tl)
    max_loss = getattr(ref, "__torch_max_loss")(match.detach(), sq.detach(), ol, tl)
    return (loss.detach().numpy(), gm.numpy(), gl.numpy(), path.numpy(), max_loss.numpy())


def dag_case(ref, name, **kw):
    batch = workloads.small_batch(**kw)
    loss, gm, gl, path, max_loss = twin_dag(ref, batch.match_all, batch.links,
                                            batch.output_length, batch.target_length,
                                            torch.float64)
    # sentences without any path (loss = -inf) have no defined alignment in the twin
    np.savez_compressed(
        os.path.join(HERE, name + ".npz"),
        match_all=batch.match_all.numpy(), links=batch.links.numpy(),
        output_length=batch.output_length.numpy(), target_length=batch.target_length.numpy(),
        loss=loss, grad_match=gm, grad_links=gl, path=path, max_loss=max_loss)
    print(name, "loss", loss)


def gather_case(ref, name, B, L, V, S, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(B, L, V, generator=g) * 2.0).to(dtype)
    idx = torch.randint(0, V, (B, L, S), generator=g)
    idx[:, :, 1] = idx[:, :, 0]  # duplicate indices must accumulate in the backward
    gsel = torch.randn(B, L, S, generator=g)
    xr = x.clone().requires_grad_()
    _, sel = ref.torch_dag_logsoftmax_gather_inplace(xr, idx)
    (dx,) = torch.autograd.grad((sel * gsel).sum(), [xr])
    # fp64 truth on the same (already rounded) logits
    xd = x.double().requires_grad_()
    seld = torch.log_softmax(xd, -1).gather(-1, idx)
    (dxd,) = torch.autograd.grad((seld * gsel.double()).sum(), [xd])
    np.savez_compressed(
        os.path.join(HERE, name + ".npz"),
        logits=x.float().numpy(), select_idx=idx.numpy(), grad_sel=gsel.numpy(),
        sel=sel.detach().numpy(), dlogits=dx.float().numpy(),
        sel_f64=seld.detach().numpy(), dlogits_f64=dxd.numpy(),
        dtype=str(dtype).replace("torch.", ""))
    print(name, "sel[0,0]", sel[0, 0, :3].tolist())


def config0_case(ref):
    batch = workloads.config0()
    # the twin's gather, then the twin's loss / alignment, as the criterion chains them
    _, match = ref.torch_dag_logsoftmax_gather_inplace(batch.logits, batch.select_idx)
    match = match.transpose(1, 2).contiguous()
    out = {}
    for dtype, tag in ((torch.float64, "f64"), (torch.float32, "f32")):
        loss, gm, gl, path, max_loss = twin_dag(ref, match, batch.links, batch.output_length,
                                                batch.target_length, dtype)
        out["loss_" + tag] = loss
        out["path_" + tag] = path
        out["max_loss_" + tag] = max_loss
        out["grad_match_rowsum_" + tag] = gm.sum(-1)          # [B,T]: 1 for t < tl
        out["grad_match_slice_" + tag] = gm[:, :, ::7]
        out["grad_links_slice_" + tag] = gl[:, ::5, ::3]
        out["grad_links_sum_" + tag] = gl.sum((1, 2))
    np.savez_compressed(
        os.path.join(HERE, "config0.npz"),
        logits_sum=np.float64(batch.logits.double().sum().item()),
        links_finite_sum=np.float64(batch.links.double().masked_fill(
            ~torch.isfinite(batch.links), 0).sum().item()),
        targets=batch.targets.numpy(), target_length=batch.target_length.numpy(),
        match_slice=match[:, :, ::7].numpy(), **out)
    print("config0 loss", out["loss_f64"])


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get(
        "DAT_REFERENCE_DIR", os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(HERE))), "reference")))
    args = ap.parse_args()
    ref = load_reference(args.reference)
    torch.manual_seed(0)
    dag_case(ref, "dag_small_full", seed=1, B=5, L=24, T=6, V=50)
    dag_case(ref, "dag_small_band", seed=2, B=5, L=30, T=9, V=40, translen=6)
    dag_case(ref, "dag_small_even", seed=3, B=3, L=33, T=7, V=64, ragged=False)
    gather_case(ref, "gather_small_f32", 2, 7, 37, 5, torch.float32, 11)
    gather_case(ref, "gather_small_f16", 2, 5, 131, 6, torch.float16, 12)
    gather_case(ref, "gather_small_bf16", 2, 5, 131, 6, torch.bfloat16, 13)
    config0_case(ref)


if __name__ == "__main__":
    main()
