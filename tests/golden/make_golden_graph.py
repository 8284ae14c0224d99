"""Generates the golden fixtures of the code on either side of the three custom ops by RUNNING THE
REFERENCE'S OWN METHOD BODIES from a checkout of thu-coai/DA-Transformer:

  force_alignment.npz    NATDAGLoss._force_aligment           (fs_plugins/criterions/nat_dag_loss.py:111-120)
  links_from_heads_*.npz GlatDecomposedLink.extract_links     (fs_plugins/models/glat_decomposed_with_link.py:351-413)
                         with extract_valid_links / logsumexp  (:319-335, :61-66), values and autograd gradients
  node_pass.npz          the node-passing part of _analyze_graph (:559-569)
  viterbi_*.npz          GlatDecomposedLink.inference_viterbi  (:720-777)

    python tests/golden/make_golden_graph.py --reference /path/to/DA-Transformer

The two modules import fairseq at the top, which is not installed here, so they cannot be imported;
instead the wanted functions are lifted out of the parsed source (ast) and compiled on their own, with
a stand-in for `self`.  Nothing of the reference is copied into this repository: the checkout is read
when the fixtures are (re)generated, the tests read the committed .npz files.
"""
import argparse
import ast
import math
import os
import sys
import types

import numpy as np
import torch
import torch.nn.functional as F
from torch import Tensor

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from da_transformer_b200 import workloads  # noqa: E402


def lift(path, names, namespace, truncate_after=None):
    """Compile the named functions / methods of a source file into `namespace`.
    truncate_after = {function: variable}: keep the body up to the assignment of `variable` and
    return it (for a method of which only the first part is wanted)."""
    tree = ast.parse(open(path).read())
    found = {}
    for node in ast.walk(tree):
        if isinstance(node, ast.FunctionDef) and node.name in names:
            node.decorator_list = []
            found[node.name] = node
    for fn, var in (truncate_after or {}).items():
        body = found[fn].body
        for k, st in enumerate(body):
            if isinstance(st, ast.Assign) and any(isinstance(t, ast.Name) and t.id == var for t in st.targets):
                found[fn].body = body[:k + 1] + [ast.Return(value=ast.Name(id=var, ctx=ast.Load()))]
                break
        else:
            raise RuntimeError(f"{fn}: no assignment of {var}")
    mod = ast.Module(body=[found[n] for n in names], type_ignores=[])
    ast.fix_missing_locations(mod)
    exec(compile(mod, path, "exec"), namespace)
    return namespace


class TorchWithFixedEinsum:
    """`torch` for the lifted extract_links, except that einsum returns a given tensor: the scores
    q.k of the reference become an arbitrary leaf, so that values and gradients are obtained for
    any content (the method divides the einsum result by sqrt(chunk_size) afterwards)."""

    def __init__(self, result):
        self._result = result

    def einsum(self, *args, **kwargs):
        return self._result

    def __getattr__(self, name):
        return getattr(torch, name)


def links_case(model_py, name, B, L, H, K, seed, mask):
    g = torch.Generator().manual_seed(seed)
    chunk = 4                                   # sqrt(chunk) = 2: the scaling is exact
    content = (torch.randn(B, L, L, H, generator=g) * 1.5).requires_grad_()
    gate_scores = torch.randn(B, L, H, generator=g).requires_grad_()
    pad = 1
    prev = torch.full((B, L), 5, dtype=torch.long)
    net_input = None
    out_len = [L] + [int(x) for x in torch.randint(2, L + 1, (B - 1,), generator=g)]
    if mask == "nonpad":
        for b, n in enumerate(out_len):
            prev[b, n:] = pad
    else:
        be = torch.zeros(B, L, dtype=torch.long)
        for b, n in enumerate(out_len):
            be[b, :n] = n - 1
        net_input = {"bound_end": be}
    ns = {"torch": TorchWithFixedEinsum(content * 2.0), "F": F, "math": math, "Tensor": Tensor}
    lift(model_py, ["logsumexp", "extract_valid_links", "extract_links"], ns)
    me = types.SimpleNamespace(
        args=argparse.Namespace(links_feature="feature", decoder_attention_heads=H, decoder_embed_dim=H * chunk,
                                max_transition_length=K),
        pad=pad)
    me.extract_valid_links = types.MethodType(ns["extract_valid_links"], me)
    zeros = lambda x: torch.zeros(B, L, H * chunk)
    links = ns["extract_links"](me, torch.zeros(B, L, 3), prev, None, zeros, zeros, lambda x: gate_scores,
                                net_input=net_input, training=True)
    w = torch.randn(links.shape, generator=g)
    fin = torch.isfinite(links)
    gc, gs = torch.autograd.grad((links * w)[fin].sum(), [content, gate_scores])
    log_gates = torch.log_softmax(gate_scores.detach(), -1)
    np.savez_compressed(
        os.path.join(HERE, name + ".npz"),
        content=content.detach().numpy(), gate_scores=gate_scores.detach().numpy(), log_gates=log_gates.numpy(),
        nonpad=(prev != pad).numpy() if mask == "nonpad" else np.zeros(0),
        bound_end=net_input["bound_end"].numpy() if net_input else np.zeros(0),
        K=np.int64(links.shape[2]), links=links.detach().numpy(), grad_links=w.masked_fill(~fin, 0).numpy(),
        grad_content=gc.numpy(), grad_gate_scores=gs.numpy())
    print(name, "links", tuple(links.shape), "finite", int(fin.sum()), "nan grads", int(torch.isnan(gc).sum()))


def force_case(criterion_py):
    ns = lift(criterion_py, ["_force_aligment"], {"torch": torch})
    g = torch.Generator().manual_seed(41)
    B, T, L = 3, 7, 19
    match = torch.randn(B, T, L, generator=g, dtype=torch.float64)
    fe = torch.full((B, L), -1, dtype=torch.long)
    fe[0, 2], fe[0, 9], fe[0, 18] = 0, 3, 6
    fe[1, 0], fe[1, 5], fe[1, 6] = 0, 2, 2       # two vertices forced onto the same step
    out = ns["_force_aligment"](None, match, fe)
    np.savez_compressed(os.path.join(HERE, "force_alignment.npz"), match=match.numpy(), force_emit=fe.numpy(),
                        forced=out.numpy())
    print("force_alignment", int(torch.isinf(out).sum()), "entries at -inf")


def square_links(B, L, gen, out_len):
    band = workloads.make_links(B, L, torch.tensor(out_len), gen)
    return workloads.band_to_square(band)


def node_pass_case(model_py):
    ns = lift(model_py, ["_analyze_graph"], {"torch": torch}, truncate_after={"_analyze_graph": "node_pass_prob"})
    g = torch.Generator().manual_seed(43)
    B, L = 3, 37
    out_len = [37, 30, 12]
    links = square_links(B, L, g, out_len)
    toks = torch.full((B, L), 5, dtype=torch.long)
    me = types.SimpleNamespace(tgt_dict=types.SimpleNamespace(pad_index=1))
    res = ns["_analyze_graph"](me, toks[:, :4], toks, None, links.double())
    np.savez_compressed(os.path.join(HERE, "node_pass.npz"), links=links.numpy(), node_pass=np.array(res))
    print("node_pass", np.array(res)[0, :5])


def viterbi_case(model_py, name, joint, beta, seed):
    ns = lift(model_py, ["inference_viterbi"], {"torch": torch})
    g = torch.Generator().manual_seed(seed)
    B, L, V, scale = 4, 48, 13, 4
    out_len = [48, 40, 33, 9]
    links = square_links(B, L, g, out_len)
    logp = torch.log_softmax(torch.randn(B, L, V, generator=g) * 2, -1)
    pad = 1
    me = types.SimpleNamespace(args=argparse.Namespace(decode_strategy="jointviterbi" if joint else "viterbi",
                                                       decode_upsample_scale=scale, decode_viterbibeta=beta),
                               tgt_dict=types.SimpleNamespace(pad_index=pad))
    keep = torch.Tensor.cuda
    torch.Tensor.cuda = lambda self, *a, **k: self     # the method moves one tensor to "the" GPU; stay on the CPU
    try:
        toks, _ = ns["inference_viterbi"](me, links.clone(), logp, torch.tensor(out_len))
    finally:
        torch.Tensor.cuda = keep
    np.savez_compressed(os.path.join(HERE, name + ".npz"), links=links.numpy(), logp=logp.numpy(),
                        output_length=np.array(out_len), joint=np.int64(joint), beta=np.float64(beta),
                        scale=np.int64(scale), pad=np.int64(pad), tokens=toks.numpy())
    print(name, toks.tolist())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get(
        "DAT_REFERENCE_DIR", os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(HERE))), "reference")))
    root = ap.parse_args().reference
    criterion_py = os.path.join(root, "fs_plugins", "criterions", "nat_dag_loss.py")
    model_py = os.path.join(root, "fs_plugins", "models", "glat_decomposed_with_link.py")
    force_case(criterion_py)
    links_case(model_py, "links_from_heads_nonpad", B=3, L=21, H=4, K=99999, seed=51, mask="nonpad")
    links_case(model_py, "links_from_heads_band", B=2, L=26, H=8, K=7, seed=52, mask="nonpad")
    links_case(model_py, "links_from_heads_bound", B=3, L=18, H=2, K=99999, seed=53, mask="bound")
    node_pass_case(model_py)
    viterbi_case(model_py, "viterbi_plain", joint=False, beta=1.0, seed=61)
    viterbi_case(model_py, "viterbi_joint", joint=True, beta=1.0, seed=62)


if __name__ == "__main__":
    main()
