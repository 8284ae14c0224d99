"""ctypes binding of ``libdat_b200.so`` (the C ABI declared in include/dat_b200.h).

The library is the only compute path: there is no CPU or PyTorch fallback.  If the
shared object is missing or a call fails, a ``RuntimeError`` is raised.
"""
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libdat_b200.so")

DAT_F32, DAT_F16, DAT_BF16 = 0, 1, 2
STATUS_BAD_LENGTH, STATUS_NO_PATH, STATUS_BAD_INDEX = 1, 2, 4

_DTYPES = {torch.float32: DAT_F32, torch.float16: DAT_F16, torch.bfloat16: DAT_BF16}

EXPORTS = (
    "dat_version", "dat_last_error", "dat_status_string", "dat_dag_loss_offsets_bytes",
    "dat_dag_best_alignment_workspace_bytes", "dat_logsoftmax_gather",
    "dat_logsoftmax_gather_backward", "dat_dag_loss", "dat_dag_loss_backward",
    "dat_dag_best_alignment", "dat_dag_loss_static", "dat_sentence_stats",
    "dat_dag_loss_fast", "dat_dag_loss_fast_scratch_bytes", "dat_dag_loss_backward_fast",
    "dat_logsoftmax_gather_fused", "dat_logsoftmax_gather_backward_fused", "dat_sentence_mean",
    "dat_links_from_heads", "dat_links_from_heads_backward", "dat_node_passing_prob",
    "dat_viterbi_decode", "dat_viterbi_decode_workspace_bytes", "dat_dag_loss_fast_flagged",
    "dat_upload_links", "dat_upload_links_bytes", "dat_upload_links_head_rows",
)

_lib = None
_vp, _i64, _i32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int


def _declare(lib):
    lib.dat_version.restype = _i32
    lib.dat_last_error.restype = ctypes.c_char_p
    lib.dat_status_string.restype = ctypes.c_char_p
    lib.dat_status_string.argtypes = [_i32]
    lib.dat_dag_loss_offsets_bytes.restype = ctypes.c_size_t
    lib.dat_dag_loss_offsets_bytes.argtypes = [_i32, _i32]
    lib.dat_dag_best_alignment_workspace_bytes.restype = ctypes.c_size_t
    lib.dat_dag_best_alignment_workspace_bytes.argtypes = [_i32, _i32, _i32]
    lib.dat_logsoftmax_gather.restype = _i32
    lib.dat_logsoftmax_gather.argtypes = [_vp, _i32, _vp, _i64, _i64, _i64, _vp, _i64, _i64, _i64,
                                          _vp, _vp, _i32, _i32, _i32, _i32, _vp]
    lib.dat_logsoftmax_gather_backward.restype = _i32
    lib.dat_logsoftmax_gather_backward.argtypes = [_vp, _i32, _vp, _i64, _i64, _i64, _vp, _i64,
                                                   _i64, _i64, _vp, _i32, _i32, _i32, _i32, _vp]
    lib.dat_dag_loss.restype = _i32
    lib.dat_dag_loss.argtypes = [_vp, _vp, _vp, _vp, _i32, _vp, _vp, _vp, _vp, _vp,
                                 _i32, _i32, _i32, _i32, _i32, _vp]
    lib.dat_dag_loss_backward.restype = _i32
    lib.dat_dag_loss_backward.argtypes = [_vp] * 10 + [_i32] * 6 + [_vp]
    lib.dat_dag_best_alignment.restype = _i32
    lib.dat_dag_best_alignment.argtypes = [_vp] * 8 + [_i32] * 5 + [_vp]
    lib.dat_dag_loss_static.restype = _i32
    lib.dat_dag_loss_static.argtypes = [_vp] * 6 + [_i32] * 4 + [_vp]
    lib.dat_dag_loss_fast_scratch_bytes.restype = ctypes.c_size_t
    lib.dat_dag_loss_fast_scratch_bytes.argtypes = [_i32, _i32, _i32]
    lib.dat_dag_loss_fast.restype = _i32
    lib.dat_dag_loss_fast.argtypes = [_vp] * 10 + [_i32] * 4 + [_vp]
    lib.dat_dag_loss_fast_flagged.restype = _i32
    lib.dat_dag_loss_fast_flagged.argtypes = [_vp, _vp, _i32, _i32, _i32, _vp]
    lib.dat_dag_loss_backward_fast.restype = _i32
    lib.dat_dag_loss_backward_fast.argtypes = [_vp] * 11 + [_i32] * 4 + [_vp]
    lib.dat_sentence_stats.restype = _i32
    lib.dat_sentence_stats.argtypes = [_vp, _vp, _vp, _i32, _vp]
    lib.dat_sentence_mean.restype = _i32
    lib.dat_sentence_mean.argtypes = [_vp, _vp, _vp, _vp, _vp, _i32, _vp]
    lib.dat_links_from_heads.restype = _i32
    lib.dat_links_from_heads.argtypes = [_vp] * 6 + [_i32] * 4 + [_vp]
    lib.dat_links_from_heads_backward.restype = _i32
    lib.dat_links_from_heads_backward.argtypes = [_vp] * 9 + [_i32] * 4 + [_vp]
    lib.dat_node_passing_prob.restype = _i32
    lib.dat_node_passing_prob.argtypes = [_vp, _vp, _i32, _i32, _vp]
    lib.dat_viterbi_decode_workspace_bytes.restype = ctypes.c_size_t
    lib.dat_viterbi_decode_workspace_bytes.argtypes = [_i32, _i32, _i32]
    lib.dat_viterbi_decode.restype = _i32
    lib.dat_viterbi_decode.argtypes = [_vp] * 10 + [_i32] * 4 + [ctypes.c_float, _i64, _vp]
    lib.dat_upload_links_bytes.restype = ctypes.c_size_t
    lib.dat_upload_links_bytes.argtypes = [_i32] * 4
    lib.dat_upload_links_head_rows.restype = _i32
    lib.dat_upload_links_head_rows.argtypes = [_i32] * 3
    lib.dat_upload_links.restype = _i32
    lib.dat_upload_links.argtypes = [_vp, _vp, _i32, _i32, _i32, _i32, _vp]
    lib.dat_logsoftmax_gather_fused.restype = _i32
    lib.dat_logsoftmax_gather_fused.argtypes = [_vp, _i32, _vp, _i64, _i64, _i64, _vp, _i64, _i64, _i64,
                                                _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp]
    lib.dat_logsoftmax_gather_backward_fused.restype = _i32
    lib.dat_logsoftmax_gather_backward_fused.argtypes = [_vp, _i32, _vp, _i64, _i64, _i64, _vp, _i64,
                                                         _i64, _i64, _vp, _vp, _i32, _i32, _i32, _i32, _vp]


def lib():
    """The loaded library.  Raises RuntimeError when it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m da_transformer_b200.build` "
                "(there is no fallback path)")
        handle = ctypes.CDLL(LIB_PATH)
        _declare(handle)
        _lib = handle
    return _lib


def check(rc, what):
    if rc != 0:
        msg = lib().dat_last_error().decode()
        kind = lib().dat_status_string(rc).decode()
        raise RuntimeError(f"{what}: {kind}: {msg}")


def dtype_code(dtype):
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise RuntimeError(f"unsupported dtype {dtype} (float32, float16, bfloat16 only)") from None


def require_cuda(*tensors):
    if not torch.cuda.is_available():
        raise RuntimeError("You need GPU to use the custom cuda operations")
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("all tensors of the custom cuda operations must be CUDA tensors")


def stream_ptr(device):
    return _vp(torch.cuda.current_stream(device).cuda_stream)


def ptr(t):
    return _vp(0 if t is None else t.data_ptr())
