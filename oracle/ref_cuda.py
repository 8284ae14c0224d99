"""Loader of the reference's own CUDA extension built by oracle/build_ref.py, plus the few
lines of Python the reference wraps around it (fs_plugins/custom_ops/dag_loss.py:102-109,
160-163, 206-231), restated so that the outputs are comparable with ours.

TEST INFRASTRUCTURE ONLY (second checker and GPU baseline).  `available()` is False when the
extension was not built; nothing here is imported by the product.

The reference kernels trap the CUDA context on invalid lengths (device asserts,
dag_loss.cu:68-69, dag_best_alignment.cu:67-70,184): callers must pass VALID lengths only
(2 <= target_length <= output_length <= prelen, (target_length-1)*translen+1 >= output_length,
a finite best path).
"""
import importlib.util
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
SO_PATH = os.path.join(_HERE, "_ref", "dag_loss_fn.so")
_mod = None


def available():
    return os.path.exists(SO_PATH)


def module():
    global _mod
    if _mod is None:
        spec = importlib.util.spec_from_file_location("dag_loss_fn", SO_PATH)
        _mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(_mod)
    return _mod


def lengths_are_valid(output_length, target_length, prelen, translen):
    ol, tl = output_length.cpu(), target_length.cpu()
    return bool(((tl >= 2) & (ol >= tl) & (ol <= prelen) & ((tl - 1) * translen + 1 >= ol)).all())


def dag_loss_fwd_bwd(match_all, links, output_length, target_length, grad_output):
    """loss, grad_match_all, grad_links of the reference CUDA path (default configs 1, 2, 2)."""
    assert lengths_are_valid(output_length, target_length, match_all.shape[2], links.shape[2])
    m = module()
    match_all, links = match_all.contiguous(), links.contiguous()
    alpha, beta = m.dag_loss(match_all, links, output_length, target_length, True, 1)
    loss = beta[:, 0, 0].clone()
    gm, gl = m.dag_loss_backward(grad_output, alpha, beta, match_all, links, output_length,
                                 target_length, 2, 2)
    return loss, gm, gl


def dag_best_alignment(match_all, links, output_length, target_length, config=1):
    assert lengths_are_valid(output_length, target_length, match_all.shape[2], links.shape[2])
    alpha, path = module().dag_best_alignment(match_all.contiguous(), links.contiguous(),
                                              output_length, target_length, config)
    return path.to(torch.long), alpha


def logsoftmax_gather(word_ins_out, select_idx, require_gradient):
    """Returns the gathered values; `word_ins_out` is overwritten with probabilities when
    require_gradient (the reference's in-place contract)."""
    return module().logsoftmax_gather(word_ins_out, select_idx, require_gradient)


def logsoftmax_gather_backward(probs, select_idx, grad_output):
    """dag_loss.py:227-229, in the logits dtype, in place on `probs`."""
    probs.mul_(grad_output.sum(-1, keepdim=True).neg_().to(probs.dtype))
    probs.scatter_add_(-1, select_idx, grad_output.to(probs.dtype))
    return probs
