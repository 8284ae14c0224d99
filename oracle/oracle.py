"""ctypes front end of the CPU oracle (oracle/dag_oracle.c).

TEST INFRASTRUCTURE ONLY.  The oracle is the checker for the CUDA path; only the
test suite, the smoke check and the benchmark's CPU-baseline leg may import this
module.  Nothing in the product package imports it.

All functions take and return NumPy arrays.  ``dtype`` selects the arithmetic the
oracle computes in (``np.float64`` = truth, ``np.float32`` = the reference CUDA
path's own arithmetic, needed for the bit-exact alignment tie-break).
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")
_lib = None


def build(force=False):
    """Compile oracle/dag_oracle.c -> oracle/liboracle.so (gcc, OpenMP)."""
    src = [os.path.join(_HERE, f) for f in ("dag_oracle.c", "dag_oracle_impl.inc", "graph_oracle_impl.inc")]
    if not force and os.path.exists(_LIB_PATH):
        if all(os.path.getmtime(_LIB_PATH) >= os.path.getmtime(s) for s in src):
            return _LIB_PATH
    subprocess.run(["make", "-C", _HERE, "-B", "liboracle.so"], check=True,
                   stdout=subprocess.DEVNULL)
    return _LIB_PATH


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB_PATH)
    return _lib


def set_threads(n=0):
    """Sets (n > 0) and returns the number of OpenMP threads the oracle's loops use."""
    return int(lib().oracle_set_threads(int(n)))


def _sfx(dtype):
    dtype = np.dtype(dtype)
    if dtype == np.float64:
        return "_f64", ctypes.c_double
    if dtype == np.float32:
        return "_f32", ctypes.c_float
    raise TypeError("oracle computes in float32 or float64 only")


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def _prep(dtype, *arrays):
    return [np.ascontiguousarray(np.asarray(a), dtype=dtype) for a in arrays]


def _lengths(output_length, target_length):
    ol = np.ascontiguousarray(np.asarray(output_length), dtype=np.int64)
    tl = np.ascontiguousarray(np.asarray(target_length), dtype=np.int64)
    return ol, tl


def dag_alpha_beta(match_all, links, output_length, target_length, dtype=np.float64):
    """alpha, beta of the reference CUDA path (dag_loss.cu:40-140, 178-274).

    match_all [B,T,L], links [B,L,K] in band format, lengths [B]."""
    sfx, _ = _sfx(dtype)
    match_all, links = _prep(dtype, match_all, links)
    ol, tl = _lengths(output_length, target_length)
    B, T, L = match_all.shape
    K = links.shape[2]
    assert links.shape[:2] == (B, L)
    alpha = np.empty((B, T, L), dtype=dtype)
    beta = np.empty((B, T, L), dtype=dtype)
    getattr(lib(), "oracle_dag_alpha" + sfx)(_p(match_all), _p(links), _p(ol), _p(tl),
                                               B, T, L, K, _p(alpha))
    getattr(lib(), "oracle_dag_beta" + sfx)(_p(match_all), _p(links), _p(ol), _p(tl),
                                              B, T, L, K, _p(beta))
    return alpha, beta


def dag_loss(match_all, links, output_length, target_length, dtype=np.float64):
    """Per-sentence log-likelihood, as DagLossFunc.forward returns it
    (dag_loss.py:106-109): beta[b,0,0] (== alpha[b,tl-1,ol-1])."""
    alpha, beta = dag_alpha_beta(match_all, links, output_length, target_length, dtype)
    return beta[:, 0, 0].copy(), alpha, beta


def dag_loss_backward(grad_output, alpha, beta, match_all, links, output_length,
                      target_length, dtype=np.float64):
    """grad_match_all, grad_links of the reference CUDA path (dag_loss.cu:378-485)."""
    sfx, _ = _sfx(dtype)
    grad_output, alpha, beta, match_all, links = _prep(dtype, grad_output, alpha, beta,
                                                       match_all, links)
    ol, tl = _lengths(output_length, target_length)
    B, T, L = match_all.shape
    K = links.shape[2]
    gm = np.empty((B, T, L), dtype=dtype)
    gl = np.empty((B, L, K), dtype=dtype)
    getattr(lib(), "oracle_dag_backward" + sfx)(_p(grad_output), _p(alpha), _p(beta),
                                                  _p(match_all), _p(links), _p(ol), _p(tl),
                                                  B, T, L, K, _p(gm), _p(gl))
    return gm, gl


def dag_loss_fwd_bwd(match_all, links, output_length, target_length, grad_output=None,
                     dtype=np.float64):
    loss, alpha, beta = dag_loss(match_all, links, output_length, target_length, dtype)
    if grad_output is None:
        grad_output = np.ones_like(loss)
    gm, gl = dag_loss_backward(grad_output, alpha, beta, match_all, links, output_length,
                               target_length, dtype)
    return loss, gm, gl


def dag_best_alignment(match_all, links, output_length, target_length, dtype=np.float32,
                       trans_block=4):
    """Best alignment with the CUDA tie-break (dag_best_alignment.cu:96-111) for
    TRANS_BLOCK_SIZE = trans_block (4 for the default config=1).  Returns
    (path int64 [B,L], max-alpha [B,T,L])."""
    sfx, _ = _sfx(dtype)
    match_all, links = _prep(dtype, match_all, links)
    ol, tl = _lengths(output_length, target_length)
    B, T, L = match_all.shape
    K = links.shape[2]
    alpha = np.empty((B, T, L), dtype=dtype)
    path = np.empty((B, L), dtype=np.int32)
    getattr(lib(), "oracle_dag_best_alignment" + sfx)(_p(match_all), _p(links), _p(ol),
                                                        _p(tl), B, T, L, K, int(trans_block),
                                                        _p(alpha), _p(path))
    return path.astype(np.int64), alpha


def logsoftmax_gather(logits, select_idx, dtype=np.float64):
    """sel[b,l,s] = log_softmax(logits[b,l,:])[select_idx[b,l,s]]
    (logsoftmax_gather.cu:256-310).  ``select_idx`` may be any strided view
    (the criterion passes a stride-0 expand)."""
    sfx, _ = _sfx(dtype)
    (x,) = _prep(dtype, logits)
    B, L, V = x.shape
    idx = np.ascontiguousarray(np.broadcast_to(np.asarray(select_idx), (B, L, select_idx.shape[2])),
                               dtype=np.int64)
    S = idx.shape[2]
    sel = np.empty((B, L, S), dtype=dtype)
    getattr(lib(), "oracle_logsoftmax_gather" + sfx)(
        _p(x), _p(idx), ctypes.c_int64(S), ctypes.c_int64(1), ctypes.c_int64(B * L), V, S,
        _p(sel), None, None)
    return sel


def logsoftmax_gather_backward(logits, select_idx, grad_sel, dtype=np.float64):
    """Dense gradient w.r.t. logits (dag_loss.py:217-231), computed in ``dtype``
    and NOT rounded to the logits dtype (the caller rounds once)."""
    sfx, _ = _sfx(dtype)
    x, g = _prep(dtype, logits, grad_sel)
    B, L, V = x.shape
    idx = np.ascontiguousarray(np.broadcast_to(np.asarray(select_idx), g.shape), dtype=np.int64)
    S = idx.shape[2]
    dx = np.empty((B, L, V), dtype=dtype)
    getattr(lib(), "oracle_logsoftmax_gather_backward" + sfx)(
        _p(x), _p(idx), ctypes.c_int64(S), ctypes.c_int64(1), _p(g), ctypes.c_int64(B * L),
        V, S, _p(dx))
    return dx


def band_to_square(band):
    """band[b,i,d] -> square[b,i,i+d+1] (restore_valid_links,
    glat_decomposed_with_link.py:337-349)."""
    (band,) = _prep(np.float64, band)
    B, L, K = band.shape
    sq = np.empty((B, L, L), dtype=np.float64)
    lib().oracle_band_to_square_f64(_p(band), B, L, K, _p(sq))
    return sq


def square_to_band(sq, K=None):
    """square[b,i,j] -> band[b,i,j-i-1] (extract_valid_links,
    glat_decomposed_with_link.py:319-335)."""
    (sq,) = _prep(np.float64, sq)
    B, L, _ = sq.shape
    K = L - 1 if K is None else K
    band = np.empty((B, L, K), dtype=np.float64)
    lib().oracle_square_to_band_f64(_p(sq), B, L, K, _p(band))
    return band


def force_alignment(match_all, force_emit, dtype=np.float64):
    """NATDAGLoss._force_aligment (nat_dag_loss.py:111-120) on match_all [B,T,L] with force_emit
    [B,L] (-1 = free).  Returns a new array."""
    sfx, _ = _sfx(dtype)
    m = np.array(match_all, dtype=dtype, order="C", copy=True)
    fe = np.ascontiguousarray(np.asarray(force_emit), dtype=np.int64)
    B, T, L = m.shape
    getattr(lib(), "oracle_force_alignment" + sfx)(_p(m), _p(fe), B, T, L)
    return m


def _masks(bound_end, nonpad, B, L):
    be = None if bound_end is None else np.ascontiguousarray(np.asarray(bound_end), dtype=np.int64)
    npd = None if nonpad is None else np.ascontiguousarray(np.asarray(nonpad), dtype=np.uint8)
    assert be is None or be.shape == (B, L)
    assert npd is None or npd.shape == (B, L)
    return be, npd


def links_from_heads(content, log_gates, K, bound_end=None, nonpad=None, dtype=np.float64):
    """Tail of extract_links (glat_decomposed_with_link.py:399-404): content [B,L,L,H], log_gates
    [B,L,H] -> band links [B,L,K] and the per-head normaliser [B,L,H]."""
    sfx, _ = _sfx(dtype)
    content, log_gates = _prep(dtype, content, log_gates)
    B, L, _, H = content.shape
    be, npd = _masks(bound_end, nonpad, B, L)
    links = np.empty((B, L, K), dtype=dtype)
    lse = np.empty((B, L, H), dtype=dtype)
    getattr(lib(), "oracle_links_from_heads" + sfx)(
        _p(content), _p(log_gates), None if be is None else _p(be), None if npd is None else _p(npd),
        B, L, H, int(K), _p(links), _p(lse))
    return links, lse


def links_from_heads_backward(grad_links, content, log_gates, K, bound_end=None, nonpad=None,
                              dtype=np.float64):
    """Gradient of links_from_heads with respect to (content, log_gates)."""
    sfx, _ = _sfx(dtype)
    grad_links, content, log_gates = _prep(dtype, grad_links, content, log_gates)
    B, L, _, H = content.shape
    be, npd = _masks(bound_end, nonpad, B, L)
    gc = np.empty_like(content)
    gg = np.empty_like(log_gates)
    getattr(lib(), "oracle_links_from_heads_backward" + sfx)(
        _p(grad_links), _p(content), _p(log_gates), None if be is None else _p(be),
        None if npd is None else _p(npd), B, L, H, int(K), _p(gc), _p(gg))
    return gc, gg


def node_passing_prob(links_square, dtype=np.float64):
    """_analyze_graph's node-passing probabilities (glat_decomposed_with_link.py:559-569), [B,L]."""
    sfx, _ = _sfx(dtype)
    (lk,) = _prep(dtype, links_square)
    B, L, _ = lk.shape
    out = np.empty((B, L), dtype=dtype)
    getattr(lib(), "oracle_node_passing_prob" + sfx)(_p(lk), B, L, _p(out))
    return out


def viterbi_decode(links_square, unreduced_logits, unreduced_tokens, output_length, max_length,
                   joint=False, beta=1.0, pad=1, dtype=np.float32):
    """inference_viterbi (glat_decomposed_with_link.py:720-777).  Returns (tokens [B,max_length],
    lengths [B], vertices [B,max_length], scores [B])."""
    sfx, ctype = _sfx(dtype)
    lk, lg = _prep(dtype, links_square, unreduced_logits)
    tk = np.ascontiguousarray(np.asarray(unreduced_tokens), dtype=np.int64)
    ol = np.ascontiguousarray(np.asarray(output_length), dtype=np.int64)
    B, L, _ = lk.shape
    toks = np.empty((B, max_length), dtype=np.int64)
    verts = np.empty((B, max_length), dtype=np.int64)
    lens = np.empty(B, dtype=np.int64)
    score = np.empty(B, dtype=dtype)
    getattr(lib(), "oracle_viterbi_decode" + sfx)(
        _p(lk), _p(lg), _p(tk), _p(ol), B, L, int(max_length), int(bool(joint)), ctype(beta),
        ctypes.c_int64(pad), _p(toks), _p(lens), _p(verts), _p(score))
    return toks, lens, verts, score
