"""Feeding the ops from host memory.

DA-Transformer produces ``links`` on the device, so the reference never moves them over PCIe; a
caller that does keep them in host memory (a data-loading or serving process in front of the ops)
should not pay for the half of the band that is padding.  ``upload_links`` moves only the entries a
graph can have (``dat_upload_links``: a kernel that reads page-locked host memory row by row, or
strided copies for pageable memory); the rest of the device tensor is left as it is, which is safe
because no op of this package reads a link whose destination is not below ``output_length``.
"""
import torch

from ._native import check, lib, ptr, stream_ptr

__all__ = ["upload_links", "upload_links_bytes"]


def upload_links_bytes(bsz, prelen, translen, max_output_length, pinned=True):
    """Bytes ``upload_links`` moves over the bus for these sizes.  Page-locked source: the first rows of every
    sentence whole (those at least three quarters real, copied by the copy engine) and the real entries of the
    others (the rows' prefixes, each rounded to 16-byte units by the copying kernel: at most 32 bytes more per
    row).  Otherwise the 32-row staircase that covers the real entries."""
    n = min(int(max_output_length), int(prelen))
    if not pinned:
        return int(lib().dat_upload_links_bytes(int(bsz), int(prelen), int(translen), n))
    head = int(lib().dat_upload_links_head_rows(int(prelen), int(translen), n))
    return int(bsz) * (head * int(translen) * 4
                       + sum(min(int(translen), n - 1 - i) * 4 for i in range(head, max(n - 1, 0))))


def upload_links(host_links, out, max_output_length=None):
    """Copies the real entries of the band ``host_links`` [B,L,K] (fp32, contiguous, ideally pinned)
    into the CUDA tensor ``out`` of the same shape, on the current stream, without blocking when the
    source is pinned.  ``max_output_length``: the largest ``output_length`` of the batch (default L).
    The padding of ``out`` keeps whatever it held; initialise it once (e.g. with -inf) if anything
    other than this package's ops will read it."""
    if host_links.is_cuda or not out.is_cuda:
        raise RuntimeError("upload_links copies from a host tensor to a CUDA tensor")
    if host_links.shape != out.shape or host_links.dim() != 3:
        raise RuntimeError("host_links and out must be [batch, prelen, translen] tensors of the same shape")
    if host_links.dtype != torch.float32 or out.dtype != torch.float32:
        raise RuntimeError("links are float32")
    if not host_links.is_contiguous() or not out.is_contiguous():
        raise RuntimeError("host_links and out must be contiguous")
    bsz, prelen, translen = host_links.shape
    n = prelen if max_output_length is None else int(max_output_length)
    with torch.cuda.device(out.device):
        check(lib().dat_upload_links(ptr(host_links), ptr(out), bsz, prelen, translen, n, stream_ptr(out.device)),
              "upload_links")
    return out
