"""Producers and consumers of the transition matrix on either side of the three custom ops:

* ``dag_links_from_heads``: the tail of ``GlatDecomposedLink.extract_links``
  (fs_plugins/models/glat_decomposed_with_link.py:380-404), which turns per-head transition scores
  into the band ``links`` that ``dag_loss`` reads, forward and backward;
* ``dag_node_passing_prob`` and ``dag_viterbi_decode``: the decode-side dynamic programmes on the
  square transition matrix (``_analyze_graph`` :559-569, ``inference_viterbi`` :720-777).

All call the C ABI of ``libdat_b200.so``; there is no CPU or PyTorch fallback.
"""
import torch
from torch.autograd import Function

from ._native import check, lib, ptr, require_cuda, stream_ptr
from .dag_loss import _status_word

__all__ = ["DagLinksFromHeadsFunc", "dag_links_from_heads", "dag_node_passing_prob", "dag_viterbi_decode"]


def _mask_u8(mask):
    if mask is None:
        return None
    return (mask if mask.dtype == torch.uint8 else mask.to(torch.uint8)).contiguous()


class DagLinksFromHeadsFunc(Function):
    @staticmethod
    def forward(ctx, log_multi_content, log_gates, nonpad_mask, bound_end, max_transition_length):
        require_cuda(log_multi_content, log_gates, nonpad_mask, bound_end)
        if log_multi_content.dim() != 4 or log_multi_content.size(1) != log_multi_content.size(2):
            raise RuntimeError("log_multi_content should be [batch, prelen, prelen, heads]")
        bsz, prelen, _, heads = log_multi_content.shape
        if log_gates.shape != (bsz, prelen, heads):
            raise RuntimeError("log_gates should be [batch, prelen, heads]")
        if log_multi_content.dtype != torch.float32 or log_gates.dtype != torch.float32:
            raise RuntimeError("dag_links_from_heads is implemented for float32 (the reference computes the "
                               "training links in float32 too)")
        content = log_multi_content.contiguous()
        gates = log_gates.contiguous()
        translen = min(int(max_transition_length), prelen - 1)
        if translen < 1:
            raise RuntimeError("max_transition_length must be at least 1 and prelen at least 2")
        nonpad = _mask_u8(nonpad_mask)
        if nonpad is not None and nonpad.shape != (bsz, prelen):
            raise RuntimeError("nonpad_mask should be [batch, prelen]")
        if bound_end is not None:
            if bound_end.shape != (bsz, prelen) or bound_end.dtype != torch.long:
                raise RuntimeError("bound_end should be a long tensor of shape [batch, prelen]")
            bound_end = bound_end.contiguous()
        dev = content.device
        need_grad = ctx.needs_input_grad[0] or ctx.needs_input_grad[1]
        with torch.cuda.device(dev):
            links = torch.empty(bsz, prelen, translen, dtype=torch.float32, device=dev)
            head_lse = torch.empty(bsz, prelen, heads, dtype=torch.float32, device=dev) if need_grad else None
            check(lib().dat_links_from_heads(ptr(content), ptr(gates), ptr(bound_end), ptr(nonpad), ptr(links),
                                             ptr(head_lse), bsz, prelen, heads, translen, stream_ptr(dev)),
                  "links_from_heads")
        if need_grad:
            ctx.save_for_backward(content, gates, links, head_lse, nonpad, bound_end)
        return links

    @staticmethod
    def backward(ctx, grad_links):
        content, gates, links, head_lse, nonpad, bound_end = ctx.saved_tensors
        bsz, prelen, _, heads = content.shape
        translen = links.size(2)
        grad_links = grad_links.to(torch.float32).contiguous()
        dev = content.device
        with torch.cuda.device(dev):
            grad_content = torch.empty_like(content)
            grad_gates = torch.empty_like(gates)
            check(lib().dat_links_from_heads_backward(
                ptr(grad_links), ptr(content), ptr(gates), ptr(links), ptr(head_lse), ptr(bound_end),
                ptr(nonpad), ptr(grad_content), ptr(grad_gates), bsz, prelen, heads, translen,
                stream_ptr(dev)), "links_from_heads_backward")
        return grad_content, grad_gates, None, None, None


def dag_links_from_heads(log_multi_content, log_gates, nonpad_mask=None, bound_end=None,
                         max_transition_length=99999):
    r"""Band links from per-head transition scores (glat_decomposed_with_link.py:380-404, the
    finite ``max_transition_length`` branch)::

        extract, nouse = model.extract_valid_links(log_multi_content, valid_mask)     # [B,L,K,H]
        extract = F.log_softmax(extract.masked_fill(nouse, -inf), dim=2).masked_fill(nouse, -inf)
        links   = logsumexp(extract + log_gates.unsqueeze(2), dim=-1)                   # [B,L,K]

    log_multi_content [B,L,L,H] fp32, log_gates [B,L,H] fp32.  The valid successors of a vertex are
    the later vertices inside the band that ``nonpad_mask`` ([B,L] bool, ``prev_output_tokens != pad``)
    allows, or, while decoding, those up to ``bound_end`` ([B,L] int64).  Returns links [B,L,K] fp32
    with K = min(max_transition_length, L-1).  Differentiable in the first two arguments."""
    return DagLinksFromHeadsFunc.apply(log_multi_content, log_gates, nonpad_mask, bound_end,
                                       max_transition_length)


@torch.no_grad()
def dag_node_passing_prob(links):
    r"""Probability that a path from vertex 0 visits each vertex (``_analyze_graph``,
    glat_decomposed_with_link.py:559-569).  links [B,L,L] fp32 square, -inf on and below the diagonal.
    Returns [B,L] fp32."""
    require_cuda(links)
    if links.dim() != 3 or links.size(1) != links.size(2) or links.dtype != torch.float32:
        raise RuntimeError("links should be a float32 tensor of shape [batch, prelen, prelen]")
    links = links.contiguous()
    bsz, prelen, _ = links.shape
    dev = links.device
    with torch.cuda.device(dev):
        out = torch.empty(bsz, prelen, dtype=torch.float32, device=dev)
        check(lib().dat_node_passing_prob(ptr(links), ptr(out), bsz, prelen, stream_ptr(dev)), "node_passing_prob")
    return out


@torch.no_grad()
def dag_viterbi_decode(links, output_logits_normalized, output_length, max_length, joint=False,
                       viterbibeta=1.0, pad_index=1):
    r"""``inference_viterbi`` (glat_decomposed_with_link.py:720-777) on the device.

    links [B,L,L] fp32 square log-probabilities (left untouched), output_logits_normalized [B,L,V]
    (its maximum and arg-max over V are taken with torch), or a pair ``(unreduced_logits [B,L] fp32,
    unreduced_tokens [B,L] int64)``; output_length [B] int64; ``max_length`` is the reference's
    ``int(2 * L / decode_upsample_scale)``.  Returns ``(tokens [B,max_length] padded with pad_index,
    lengths [B], vertices [B,max_length] of the chosen path, -1 padded, scores [B])``."""
    if isinstance(output_logits_normalized, (tuple, list)):
        unreduced_logits, unreduced_tokens = output_logits_normalized
    else:
        unreduced_logits, unreduced_tokens = output_logits_normalized.max(dim=-1)
    require_cuda(links, unreduced_logits, unreduced_tokens, output_length)
    if links.dim() != 3 or links.size(1) != links.size(2) or links.dtype != torch.float32:
        raise RuntimeError("links should be a float32 tensor of shape [batch, prelen, prelen]")
    bsz, prelen, _ = links.shape
    if unreduced_logits.shape != (bsz, prelen) or unreduced_tokens.shape != (bsz, prelen):
        raise RuntimeError("token scores should be [batch, prelen]")
    if output_length.dtype != torch.long or unreduced_tokens.dtype != torch.long:
        raise RuntimeError("length should be long")
    links = links.contiguous()
    logit = unreduced_logits.to(torch.float32).contiguous()
    toks = unreduced_tokens.contiguous()
    ol = output_length.contiguous()
    max_length = int(max_length)
    dev = links.device
    L = lib()
    with torch.cuda.device(dev):
        ws = torch.empty(max(L.dat_viterbi_decode_workspace_bytes(bsz, prelen, max_length), 1),
                         dtype=torch.uint8, device=dev)
        tokens = torch.empty(bsz, max_length, dtype=torch.long, device=dev)
        verts = torch.empty(bsz, max_length, dtype=torch.long, device=dev)
        lengths = torch.empty(bsz, dtype=torch.long, device=dev)
        scores = torch.empty(bsz, dtype=torch.float32, device=dev)
        check(L.dat_viterbi_decode(ptr(links), ptr(logit), ptr(toks), ptr(ol), ptr(ws), ptr(tokens), ptr(lengths),
                                   ptr(verts), ptr(scores), ptr(_status_word(dev)), bsz, prelen, max_length,
                                   int(bool(joint)), float(viterbibeta), int(pad_index), stream_ptr(dev)),
              "viterbi_decode")
    return tokens, lengths, verts, scores
