"""The allocation-free likelihood entry point, `dat_dag_loss_static`.

Some hosts of this library cannot get device memory at call time: a serving process that
handed the whole GPU to its own pool at start-up has nothing left for cudaMalloc, and a
plugin slot may forbid allocation because cudaMalloc synchronises the device and stalls the
process's other streams.  For them the library carries its recursion workspace inside its
own image.  This test calls that entry point through the C ABI and checks it against the
regular entry point (`dat_dag_loss`, workspaces allocated by the caller) on two calls in a
row with different data, and checks that a batch beyond the built-in workspace is refused
with a clear message.  Collected last on purpose.
"""
import ctypes

import numpy as np
import pytest
import torch

from da_transformer_b200 import _native, workloads

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _regular(lib, b):
    B, T, L = b.match_all.shape
    K = b.links.shape[2]
    alpha = torch.empty(B, T, L, device=DEV)
    offsets = torch.empty(B, 2 * T + 2, dtype=torch.float64, device=DEV)
    loss = torch.empty(B, device=DEV)
    rc = lib.dat_dag_loss(_native.ptr(b.match_all), _native.ptr(b.links), _native.ptr(b.output_length),
                          _native.ptr(b.target_length), 0, _native.ptr(alpha), None, _native.ptr(offsets),
                          _native.ptr(loss), None, B, T, L, K, 1, _native.stream_ptr(torch.device(DEV)))
    _native.check(rc, "dat_dag_loss")
    return loss


def _static(lib, b):
    B, T, L = b.match_all.shape
    K = b.links.shape[2]
    loss = torch.full((B,), float("nan"), device=DEV)
    rc = lib.dat_dag_loss_static(_native.ptr(b.match_all), _native.ptr(b.links), _native.ptr(b.output_length),
                                 _native.ptr(b.target_length), _native.ptr(loss), None, B, T, L, K,
                                 _native.stream_ptr(torch.device(DEV)))
    _native.check(rc, "dat_dag_loss_static")
    return loss


def test_static_workspace_entry_point_matches_the_regular_one_twice():
    lib = _native.lib()
    torch.cuda.set_device(0)
    first = workloads.small_batch(seed=51, B=6, L=97, T=13, V=40).to(DEV)
    second = workloads.small_batch(seed=52, B=3, L=200, T=31, V=40, translen=60).to(DEV)
    for batch in (first, second):
        want = _regular(lib, batch)
        got = _static(lib, batch)
        torch.cuda.synchronize()
        w, g = want.cpu().numpy().astype(np.float64), got.cpu().numpy().astype(np.float64)
        fin = np.isfinite(w)
        assert np.array_equal(np.isfinite(g), fin) and fin.any()
        assert np.abs(g[fin] - w[fin]).max() <= 1e-5 * np.abs(w[fin]).max()
    # the same data again after the workspace was used for something else
    again = _static(lib, first)
    assert torch.equal(again, _static(lib, first))
    assert torch.allclose(again, _regular(lib, first), rtol=1e-5, atol=0, equal_nan=True)


def test_static_workspace_entry_point_refuses_oversized_batches():
    lib = _native.lib()
    dummy = torch.zeros(8, device=DEV)
    p = _native.ptr(dummy)
    # 64 * 128 * 512 = 2^22 floats > 2^21
    rc = lib.dat_dag_loss_static(p, p, p, p, p, None, 64, 128, 512, 511, _native.stream_ptr(torch.device(DEV)))
    assert rc == 2
    msg = lib.dat_last_error().decode()
    assert "exceeds the built-in workspace" in msg and "2097152" in msg
    torch.cuda.synchronize()
