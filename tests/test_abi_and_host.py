"""CPU-only checks: the shared library loads and exports every symbol the header declares,
the host-side front end validates arguments like the reference wrapper does, and the
synthetic workloads have the documented shapes.  No compute call is made."""
import os
import re

import pytest
import torch

import da_transformer_b200 as dat
from da_transformer_b200 import _native, build, workloads

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    text = open(os.path.join(ROOT, "include", "dat_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(dat_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    build.build()
    lib = _native.lib()
    names = header_symbols()
    assert len(names) >= 10
    for name in names:
        assert hasattr(lib, name), f"{name} declared in include/dat_b200.h but not exported"
    assert set(_native.EXPORTS) <= set(names)
    assert lib.dat_version() == 100
    assert lib.dat_status_string(0) == b"ok"
    assert lib.dat_dag_loss_offsets_bytes(3, 5) == 3 * 12 * 8
    assert lib.dat_dag_best_alignment_workspace_bytes(2, 4, 8) >= 2 * 4 * 8 * 2


def test_bad_arguments_are_rejected_before_any_cuda_call():
    lib = _native.lib()
    rc = lib.dat_dag_loss(None, None, None, None, 0, None, None, None, None, None, 2, 4, 8, 7, 1, None)
    assert rc == 1 and b"null" in lib.dat_last_error()
    rc = lib.dat_dag_loss(None, None, None, None, 0, None, None, None, None, None, 2, 0, 8, 7, 1, None)
    assert rc == 1 and b"bad sizes" in lib.dat_last_error()
    rc = lib.dat_dag_best_alignment(None, None, None, None, None, None, None, None, 2, 4, 8, 7, 9, None)
    assert rc == 1 and b"config" in lib.dat_last_error()
    rc = lib.dat_logsoftmax_gather(None, 7, None, 0, 0, 0, None, 0, 0, 0, None, None, 1, 1, 1, 0, None)
    assert rc == 1
    assert lib.dat_status_string(2) == b"unsupported dtype or size"


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU behaviour")
def test_ops_refuse_to_run_without_a_gpu():
    """There is no CPU fallback: like the reference (dag_loss.py:38-39) the ops raise."""
    b = workloads.small_batch(seed=0)
    with pytest.raises(RuntimeError, match="GPU"):
        dat.dag_loss(b.match_all, b.links, b.output_length, b.target_length)
    with pytest.raises(RuntimeError, match="GPU"):
        dat.dag_best_alignment(b.match_all, b.links, b.output_length, b.target_length)
    with pytest.raises(RuntimeError, match="GPU"):
        dat.dag_logsoftmax_gather_inplace(b.logits.clone(), b.select_idx)
    with pytest.raises(RuntimeError, match="GPU"):
        dat.get_dag_kernel()


def test_public_names_match_the_reference_module():
    for name in ("dag_loss", "dag_best_alignment", "dag_logsoftmax_gather_inplace",
                 "DagLossFunc", "DagBestAlignmentFunc", "DagLogsoftmaxGatherFunc", "get_dag_kernel"):
        assert hasattr(dat, name)
    assert (dat.DagLossFunc.config, dat.DagLossFunc.config1, dat.DagLossFunc.config2) == (1, 2, 2)
    assert dat.DagBestAlignmentFunc.config == 1


def test_workload_shapes():
    c0 = workloads.config0()
    assert c0.logits.shape == (8, 160, 1000) and c0.links.shape == (8, 160, 159)
    assert c0.select_idx.stride() == (c0.targets.shape[1], 0, 1)
    assert int(c0.target_length.min()) >= 10 and int(c0.target_length.max()) <= 20
    # links rows are log-distributions over the valid successors; the last vertex has none
    p = c0.links.exp().sum(-1)
    assert torch.allclose(p[:, :-1], torch.ones_like(p[:, :-1]), atol=1e-5) and (p[:, -1] == 0).all()
    c1 = workloads.config1(B=6, with_logits=False)
    assert (c1.output_length % 8 == 0).all() and c1.links.shape[1] == int(c1.output_length.max())
    assert (c1.target_length >= 2).all() and (c1.target_length <= 64).all()
    c4 = workloads.config4(B=4)
    assert c4.match_all.shape == (4, 64, 512) and c4.links.shape == (4, 512, 511)
    sq = workloads.band_to_square(c4.links[:1])
    assert torch.equal(workloads.square_to_band(sq), c4.links[:1])
    a, b = c4.shard(0, 2), c4.shard(1, 2)
    assert a.targets.shape[0] == 2 and torch.equal(torch.cat([a.links, b.links]), c4.links)
