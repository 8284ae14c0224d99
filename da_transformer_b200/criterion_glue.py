"""The criterion's glue around the three ops, fused into the ops' own passes.

``fs_plugins/criterions/nat_dag_loss.py`` surrounds the custom ops with plain torch code that
re-reads or re-writes their large tensors.  The functions here are what a maintainer calls
instead of those lines to get the same numbers from fewer passes:

===============================  ==========================================  ======================
reference lines                  what they do                                here
===============================  ==========================================  ======================
nat_dag_loss.py:246              ``word_ins_out.argmax(-1)``: a full extra   ``dag_match(...,
                                 read of the [B,L,V] logits                  return_argmax=True)``
nat_dag_loss.py:168-169          gather, ``transpose(1,2)``; dag_loss then   ``dag_match`` writes
(+ custom_ops/dag_loss.py:102)   ``.contiguous()``: a [B,T,L] copy           [B,T,L] directly
nat_dag_loss.py:111-120, 178     ``_force_aligment``: three [B,T,L]          ``dag_match(...,
                                 temporaries                                 force_emit=...)``
nat_dag_loss.py:190-194          inf/nan masking, ``-(loss/tl).mean()``      ``dag_loss_mean``
nat_dag_loss.py:246-271          glancing pass: argmax, gather, alignment    ``glat_alignment``
===============================  ==========================================  ======================

Like the ops themselves there is no CPU or PyTorch fallback: without the library or a GPU these raise.
"""
import torch
from torch.autograd import Function

from . import _native
from ._native import check, lib, ptr, require_cuda, stream_ptr
from .dag_loss import _status_word, dag_best_alignment

__all__ = ["DagMatchFunc", "dag_match", "SentenceMeanFunc", "dag_loss_mean", "glat_alignment"]


class DagMatchFunc(Function):
    @staticmethod
    def forward(ctx, word_ins_out, tgt_tokens, force_emit, return_argmax):
        require_gradient = ctx.needs_input_grad[0]
        require_cuda(word_ins_out, tgt_tokens, force_emit)
        if word_ins_out.dim() != 3:
            raise RuntimeError("word_ins_out dim != 3")
        if tgt_tokens.dim() != 2:
            raise RuntimeError("tgt_tokens dim != 2")
        bsz, prelen, vocab = word_ins_out.shape
        if tgt_tokens.size(0) != bsz:
            raise RuntimeError("batch size not match")
        if tgt_tokens.dtype != torch.long:
            raise RuntimeError("tgt_tokens should be long")
        if not word_ins_out.is_contiguous():
            raise RuntimeError("word_ins_out is not contiguous")
        tarlen = tgt_tokens.size(1)
        if force_emit is not None:
            if force_emit.shape != (bsz, prelen) or force_emit.dtype != torch.long:
                raise RuntimeError("force_emit should be a long tensor of shape [batch, prelen]")
            force_emit = force_emit.contiguous()
        dt = _native.dtype_code(word_ins_out.dtype)
        dev = word_ins_out.device
        with torch.cuda.device(dev):
            match = torch.empty(bsz, tarlen, prelen, dtype=torch.float32, device=dev)
            stats = torch.empty(bsz * prelen, 2, dtype=torch.float32, device=dev) if require_gradient else None
            pred = torch.empty(bsz, prelen, dtype=torch.long, device=dev) if return_argmax else None
            forced = torch.empty(bsz, tarlen, dtype=torch.int32, device=dev) if force_emit is not None else None
            check(lib().dat_logsoftmax_gather_fused(
                ptr(word_ins_out), dt,
                ptr(tgt_tokens), tgt_tokens.stride(0), 0, tgt_tokens.stride(1),      # index [b, l, s] = tgt[b, s]
                ptr(match), match.stride(0), match.stride(2), match.stride(1),       # value [b, l, s] -> match[b, s, l]
                ptr(stats), ptr(pred), ptr(force_emit), ptr(forced), ptr(_status_word(dev)),
                bsz, prelen, tarlen, vocab, stream_ptr(dev)), "logsoftmax_gather (fused)")
        ctx.mark_dirty(word_ins_out)
        ctx.set_materialize_grads(False)
        if pred is None:
            pred = torch.empty(0, dtype=torch.long, device=dev)
        ctx.mark_non_differentiable(pred)
        if require_gradient:
            ctx.save_for_backward(word_ins_out, tgt_tokens, stats, forced)
            ctx.has_backward = False
        return word_ins_out, match, pred

    @staticmethod
    def backward(ctx, grad_word_ins_out, grad_match, grad_pred):
        if not ctx.needs_input_grad[0]:
            return None, None, None, None
        assert grad_word_ins_out is None, "Cannot reuse word_ins_out after logsoftmax_gather"
        if grad_match is None:
            return None, None, None, None
        assert not ctx.has_backward, "Cannot backward twice in logsoftmax_gather"
        ctx.has_backward = True
        grad_input, tgt_tokens, stats, forced = ctx.saved_tensors
        bsz, prelen, vocab = grad_input.shape
        tarlen = tgt_tokens.size(1)
        if grad_match.dtype != torch.float32:
            grad_match = grad_match.float()
        dev = grad_input.device
        with torch.cuda.device(dev):
            check(lib().dat_logsoftmax_gather_backward_fused(
                ptr(grad_input), _native.dtype_code(grad_input.dtype),
                ptr(tgt_tokens), tgt_tokens.stride(0), 0, tgt_tokens.stride(1),
                ptr(grad_match), grad_match.stride(0), grad_match.stride(2), grad_match.stride(1),
                ptr(stats), ptr(forced), bsz, prelen, tarlen, vocab, stream_ptr(dev)),
                "logsoftmax_gather_backward (fused)")
        return grad_input.detach(), None, None, None


def dag_match(word_ins_out, tgt_tokens, force_emit=None, return_argmax=False):
    r"""``match_all`` for ``dag_loss`` / ``dag_best_alignment`` straight from the logits.

    Equivalent to (nat_dag_loss.py:166-179, 246-262)::

        pred = word_ins_out.argmax(-1)                                     # if return_argmax
        word_ins_out, match = dag_logsoftmax_gather_inplace(
            word_ins_out, tgt_tokens.unsqueeze(1).expand(-1, prelen, -1))
        match = match.transpose(1, 2)
        if force_emit is not None: match = criterion._force_aligment(match, force_emit)

    in one pass over the logits, with ``match`` [B,T,L] contiguous.  word_ins_out [B,L,V]
    fp32/fp16/bf16 contiguous is marked dirty exactly like in ``dag_logsoftmax_gather_inplace``
    (it receives its gradient in place in the backward); tgt_tokens [B,T] int64; force_emit [B,L]
    int64 (-1 = free).  Returns ``(word_ins_out, match, pred)``; ``pred`` is None unless asked for.
    """
    out, match, pred = DagMatchFunc.apply(word_ins_out, tgt_tokens, force_emit, bool(return_argmax))
    return out, match, (pred if return_argmax else None)


class SentenceMeanFunc(Function):
    @staticmethod
    def forward(ctx, loss_result, target_length):
        require_cuda(loss_result, target_length)
        if loss_result.dim() != 1 or target_length.shape != loss_result.shape:
            raise RuntimeError("loss_result and target_length must be [batch]")
        if target_length.dtype != torch.long:
            raise RuntimeError("length should be long")
        loss32 = loss_result.detach().to(torch.float32).contiguous()
        tl = target_length.contiguous()
        dev = loss_result.device
        bsz = loss32.numel()
        with torch.cuda.device(dev):
            stats = torch.empty(4, dtype=torch.float64, device=dev)
            mean = torch.empty((), dtype=torch.float32, device=dev)
            scale = torch.empty(bsz, dtype=torch.float32, device=dev)
            check(lib().dat_sentence_mean(ptr(loss32), ptr(tl), ptr(stats), ptr(mean), ptr(scale), bsz,
                                          stream_ptr(dev)), "dat_sentence_mean")
        ctx.save_for_backward(scale)
        ctx.mark_non_differentiable(stats)
        return mean, stats

    @staticmethod
    def backward(ctx, grad_mean, grad_stats):
        (scale,) = ctx.saved_tensors
        return scale * grad_mean, None


def dag_loss_mean(loss_result, target_length):
    r"""The criterion's reduction of the sentence log-likelihoods (nat_dag_loss.py:190-194)::

        invalid = loss_result.isinf() | loss_result.isnan()
        loss = -(loss_result.masked_fill(invalid, 0) / target_length).mean()

    in one launch.  Returns ``(loss, stats)``: the differentiable scalar, and the fp64 vector
    ``[sum clean/tl, sum tl, n_sentences, n_invalid]`` that ``dist.all_reduce_stats`` sums over ranks
    (``stats[3]`` is the criterion's ``invalid_nsentences``)."""
    return SentenceMeanFunc.apply(loss_result, target_length)


@torch.no_grad()
def glat_alignment(word_ins_out, tgt_tokens, links, output_length, target_length, force_emit=None):
    r"""The device part of the glancing sampler (``glat_function``, nat_dag_loss.py:239-271):
    the model's own predictions, the match matrix and the best alignment of the target, from one
    pass over the logits plus the alignment kernel.  Returns ``(pred_tokens [B,L], path [B,L],
    match [B,T,L])``; ``word_ins_out`` is left untouched (no gradient is recorded)."""
    _, match, pred = dag_match(word_ins_out, tgt_tokens, force_emit=force_emit, return_argmax=True)
    path = dag_best_alignment(match, links, output_length, target_length)
    return pred, path, match
