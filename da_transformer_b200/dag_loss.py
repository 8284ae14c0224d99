"""Drop-in for ``fs_plugins/custom_ops/dag_loss.py`` of thu-coai/DA-Transformer.

Same public names, argument order, dtypes and autograd behaviour:

    dag_loss(match_all, links, output_length, target_length)            -> [B] fp32
    dag_best_alignment(match_all, links, output_length, target_length)  -> [B,L] int64
    dag_logsoftmax_gather_inplace(word_ins_out, select_idx)             -> (word_ins_out, [B,L,S] fp32)

so ``fs_plugins/criterions/nat_dag_loss.py`` and
``fs_plugins/models/glat_decomposed_with_link.py`` can import this module in place of
the reference one.  The ``autograd.Function`` wrappers below call the C ABI of
``libdat_b200.so`` (hand-written sm_100a kernels) through ctypes; every buffer is
allocated here with PyTorch and handed to the library as a raw pointer, and every launch
goes to PyTorch's current stream.  There is no CPU or PyTorch fallback: without the
library or without a GPU the ops raise ``RuntimeError``.

Differences from the reference that a caller can observe:
  * bf16 logits are accepted by ``dag_logsoftmax_gather_inplace`` (the reference
    dispatches fp16/fp32/fp64 only, logsoftmax_gather.cu:46-58); fp64 is not supported
    by any op here and raises.
  * ``dag_logsoftmax_gather_inplace`` leaves ``word_ins_out`` untouched in the forward
    (the reference overwrites it with probabilities) and overwrites it with the gradient
    in the backward, as the reference does; it is still marked dirty and must not be
    used afterwards.
  * invalid lengths (the reference's device asserts, dag_loss.cu:68-69) give a ``-inf``
    loss, zero gradients and an all ``-1`` alignment instead of a trapped context;
    ``last_status()`` reports them.
"""
import torch
from torch.autograd import Function

from . import _native
from ._native import check, lib, ptr, require_cuda, stream_ptr

__all__ = [
    "DagLossFunc", "DagBestAlignmentFunc", "DagLogsoftmaxGatherFunc",
    "dag_loss", "dag_best_alignment", "dag_logsoftmax_gather_inplace", "logsoftmax_gather",
    "get_dag_kernel", "last_status",
]

_status = {}


def _status_word(device):
    """Per-device int32 word the kernels OR their DAT_STATUS_* bits into."""
    key = torch.device(device).index
    buf = _status.get(key)
    if buf is None:
        buf = torch.zeros(1, dtype=torch.int32, device=device)
        _status[key] = buf
    return buf


def last_status(device=None, reset=True):
    """Status bits accumulated on ``device`` since the last reset (synchronises):
    1 = a sentence had invalid lengths, 2 = a sentence had no finite alignment,
    4 = a gather index was outside the vocabulary, 8 = the fast dag_loss path handed at least
    one sentence to the exact kernels (informational)."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    buf = _status_word(device)
    value = int(buf.item())
    if reset:
        buf.zero_()
    return value


def get_dag_kernel():
    """The loaded native library (the reference JIT-compiles a pybind module here,
    dag_loss.py:36-63).  Raises ``RuntimeError`` without a GPU or without the library."""
    if not torch.cuda.is_available():
        raise RuntimeError("You need GPU to use the custom cuda operations")
    return lib()


def _check_dag_inputs(match_all, links, output_length, target_length):
    require_cuda(match_all, links, output_length, target_length)
    if match_all.dim() != 3:
        raise RuntimeError("match_all dim != 3")
    if links.dim() != 3:
        raise RuntimeError("links dim != 3")
    if output_length.dim() != 1:
        raise RuntimeError("output_length dim != 1")
    if target_length.dim() != 1:
        raise RuntimeError("target_length dim != 1")
    bsz, tarlen, prelen = match_all.shape
    if not (links.size(0) == bsz and output_length.size(0) == bsz and target_length.size(0) == bsz):
        raise RuntimeError("batch size not match")
    if links.size(1) != prelen:
        raise RuntimeError("prelen not match")
    if output_length.dtype != torch.long or target_length.dtype != torch.long:
        raise RuntimeError("length should be long")
    if match_all.dtype != torch.float32 or links.dtype != torch.float32:
        raise RuntimeError(
            f"dag ops are implemented for float32 (got {match_all.dtype}, {links.dtype})")
    return bsz, tarlen, prelen, links.size(2)


class DagLossFunc(Function):
    # launch-configuration knobs of the reference (dag_loss.py:66-68); accepted, ignored
    config = 1
    config1 = 2
    config2 = 2
    # False: the forward runs the fast probability-domain kernels, which fall back per sentence to
    # the exact log-domain kernels whenever their dynamic-range check does not pass.  Calls without
    # gradient (validation) take them too: the check needs both recursions, and both fast sweeps
    # together are still several times faster than the exact alpha recursion alone.
    # True: always the exact log-domain kernels.
    exact = False

    @staticmethod
    def forward(ctx, match_all, links, output_length, target_length):
        r"""Log-likelihood of the target under the DAG (dag_loss.py:71-111).

        match_all [B,T,L] fp32, links [B,L,K] fp32 band format (links[b,i,d] is the
        transition i -> i+d+1), output_length / target_length [B] int64.  Returns [B] fp32.
        """
        require_gradient = ctx.needs_input_grad[0] or ctx.needs_input_grad[1]
        match_all = match_all.contiguous()
        links = links.contiguous()
        bsz, tarlen, prelen, translen = _check_dag_inputs(match_all, links, output_length, target_length)
        output_length = output_length.contiguous()
        target_length = target_length.contiguous()
        dev = match_all.device
        L = lib()
        with torch.cuda.device(dev):
            fast = not DagLossFunc.exact and bsz > 0
            alpha = torch.empty(bsz, tarlen, prelen, dtype=torch.float32, device=dev)
            beta = (torch.empty(bsz, tarlen, prelen, dtype=torch.float32, device=dev)
                    if (require_gradient or fast) else None)
            offsets = torch.empty(bsz, 2 * tarlen + 2, dtype=torch.float64, device=dev)
            res = torch.empty(bsz, dtype=torch.float32, device=dev)
            scratch = None
            if fast:
                scratch = torch.empty(L.dat_dag_loss_fast_scratch_bytes(bsz, tarlen, prelen),
                                      dtype=torch.uint8, device=dev)
                check(L.dat_dag_loss_fast(ptr(match_all), ptr(links), ptr(output_length),
                                          ptr(target_length), ptr(alpha), ptr(beta), ptr(offsets),
                                          ptr(res), ptr(_status_word(dev)), ptr(scratch), bsz, tarlen,
                                          prelen, translen, stream_ptr(dev)), "dag_loss (fast)")
            else:
                check(L.dat_dag_loss(ptr(match_all), ptr(links), ptr(output_length), ptr(target_length),
                                     int(require_gradient), ptr(alpha), ptr(beta), ptr(offsets), ptr(res),
                                     ptr(_status_word(dev)), bsz, tarlen, prelen, translen,
                                     int(DagLossFunc.config), stream_ptr(dev)), "dag_loss")
        if require_gradient:
            ctx.save_for_backward(alpha, beta, offsets, match_all, links, output_length, target_length)
            ctx.fast_scratch = scratch   # exp(links) + per-sentence flags, reused by the backward
        return res

    @staticmethod
    def backward(ctx, grad_output):
        if not (ctx.needs_input_grad[0] or ctx.needs_input_grad[1]):
            return None, None, None, None
        alpha, beta, offsets, match_all, links, output_length, target_length = ctx.saved_tensors
        bsz, tarlen, prelen = match_all.shape
        translen = links.size(2)
        dev = match_all.device
        grad_output = grad_output.to(torch.float32).contiguous()
        with torch.cuda.device(dev):
            grad_match_all = torch.empty_like(match_all)
            grad_links = torch.empty_like(links)
            if ctx.fast_scratch is not None:
                check(lib().dat_dag_loss_backward_fast(
                    ptr(grad_output), ptr(alpha), ptr(beta), ptr(offsets), ptr(match_all), ptr(links),
                    ptr(output_length), ptr(target_length), ptr(grad_match_all), ptr(grad_links),
                    ptr(ctx.fast_scratch), bsz, tarlen, prelen, translen, stream_ptr(dev)),
                    "dag_loss_backward (fast)")
            else:
                check(lib().dat_dag_loss_backward(
                    ptr(grad_output), ptr(alpha), ptr(beta), ptr(offsets), ptr(match_all), ptr(links),
                    ptr(output_length), ptr(target_length), ptr(grad_match_all), ptr(grad_links),
                    bsz, tarlen, prelen, translen, int(DagLossFunc.config1), int(DagLossFunc.config2),
                    stream_ptr(dev)), "dag_loss_backward")
        return grad_match_all, grad_links, None, None


dag_loss = DagLossFunc.apply


class DagBestAlignmentFunc(Function):
    # 1..4 selects the reference's TRANS_BLOCK_SIZE 4/8/16/32 (dag_best_alignment.cu:253-256),
    # which only matters for which of several equally good paths is returned
    config = 1

    @staticmethod
    def forward(ctx, match_all, links, output_length, target_length):
        r"""Best alignment (dag_loss.py:128-164).  Returns [B,L] int64: the index of the
        target token vertex j emits on the most probable path, or -1."""
        match_all = match_all.contiguous()
        links = links.contiguous()
        bsz, tarlen, prelen, translen = _check_dag_inputs(match_all, links, output_length, target_length)
        output_length = output_length.contiguous()
        target_length = target_length.contiguous()
        dev = match_all.device
        L = lib()
        with torch.cuda.device(dev):
            path = torch.empty(bsz, prelen, dtype=torch.long, device=dev)
            # square copy of the links (+ room for the trace when it does not fit on chip)
            nbytes = L.dat_dag_best_alignment_workspace_bytes(bsz, tarlen, prelen)
            ws = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=dev)
            check(L.dat_dag_best_alignment(
                ptr(match_all), ptr(links), ptr(output_length), ptr(target_length), ptr(path),
                ptr(None), ptr(ws), ptr(_status_word(dev)), bsz, tarlen, prelen, translen,
                int(DagBestAlignmentFunc.config), stream_ptr(dev)), "dag_best_alignment")
        ctx.mark_non_differentiable(path)
        return path

    @staticmethod
    def backward(ctx, grad_output):
        assert False, "no backward function for best alignment"


dag_best_alignment = DagBestAlignmentFunc.apply


class DagLogsoftmaxGatherFunc(Function):
    # when True the gathered values are laid out [B,S,L]-contiguous (returned with the
    # usual [B,L,S] shape), which makes the criterion's transpose(1,2) + contiguous() free
    transposed_output = False

    @staticmethod
    def forward(ctx, word_ins_out, select_idx):
        r"""``word_ins_out.log_softmax(-1, dtype=float).gather(-1, select_idx)``
        (dag_loss.py:175-214).  word_ins_out [B,L,V] fp32/fp16/bf16 contiguous, select_idx
        [B,L,S] int64 with any strides.  Returns (word_ins_out, selected [B,L,S] fp32);
        word_ins_out is marked dirty and must not be used afterwards: its storage
        receives the gradient in the backward."""
        require_gradient = ctx.needs_input_grad[0]
        require_cuda(word_ins_out, select_idx)
        if word_ins_out.dim() != 3:
            raise RuntimeError("word_ins_out dim != 3")
        if select_idx.dim() != 3:
            raise RuntimeError("select_idx dim != 3")
        bsz, prelen, vocab = word_ins_out.shape
        slen = select_idx.size(2)
        if select_idx.size(0) != bsz:
            raise RuntimeError("batch size not match")
        if select_idx.size(1) != prelen:
            raise RuntimeError("prelen size not match")
        if select_idx.dtype != torch.long:
            raise RuntimeError("select_idx should be long")
        if not word_ins_out.is_contiguous():
            raise RuntimeError("word_ins_out is not contiguous")
        dt = _native.dtype_code(word_ins_out.dtype)
        dev = word_ins_out.device
        with torch.cuda.device(dev):
            if DagLogsoftmaxGatherFunc.transposed_output:
                selected = torch.empty(bsz, slen, prelen, dtype=torch.float32, device=dev).transpose(1, 2)
            else:
                selected = torch.empty(bsz, prelen, slen, dtype=torch.float32, device=dev)
            stats = torch.empty(bsz * prelen, 2, dtype=torch.float32, device=dev) if require_gradient else None
            check(lib().dat_logsoftmax_gather(
                ptr(word_ins_out), dt, ptr(select_idx), *select_idx.stride(),
                ptr(selected), *selected.stride(), ptr(stats), ptr(_status_word(dev)),
                bsz, prelen, slen, vocab, stream_ptr(dev)), "logsoftmax_gather")
        ctx.mark_dirty(word_ins_out)
        ctx.set_materialize_grads(False)
        if require_gradient:
            ctx.save_for_backward(word_ins_out, select_idx, stats)
            ctx.has_backward = False
        return word_ins_out, selected

    @staticmethod
    def backward(ctx, grad_word_ins_out, grad_output):
        if not ctx.needs_input_grad[0]:
            return None, None
        assert grad_word_ins_out is None, "Cannot reuse word_ins_out after logsoftmax_gather"
        if grad_output is None:
            return None, None
        assert not ctx.has_backward, "Cannot backward twice in logsoftmax_gather"
        ctx.has_backward = True

        grad_input, select_idx, stats = ctx.saved_tensors
        bsz, prelen, vocab = grad_input.shape
        slen = select_idx.size(2)
        if grad_output.dtype != torch.float32:
            grad_output = grad_output.float()
        dev = grad_input.device
        with torch.cuda.device(dev):
            check(lib().dat_logsoftmax_gather_backward(
                ptr(grad_input), _native.dtype_code(grad_input.dtype), ptr(select_idx),
                *select_idx.stride(), ptr(grad_output), *grad_output.stride(), ptr(stats),
                bsz, prelen, slen, vocab, stream_ptr(dev)), "logsoftmax_gather_backward")
        # the saved tensor is an output of this Function; hand autograd a plain view of its storage
        return grad_input.detach(), None


dag_logsoftmax_gather_inplace = DagLogsoftmaxGatherFunc.apply
# the name the native function carries in the reference (dag_loss.cpp:22)
logsoftmax_gather = dag_logsoftmax_gather_inplace
