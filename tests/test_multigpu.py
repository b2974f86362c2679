"""Several GPU ranks (2 and, where the box has them, 4 or 8): in-kernel NVLink collectives against
the NCCL strategy, for data parallelism, fused tensor parallelism and tensor-parallel serving."""
import os

import pytest
import torch

from test_distributed_cpu import _launch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]

_N = torch.cuda.device_count() if torch.cuda.is_available() else 0
RANKS = sorted({2, max([n for n in (2, 4, 8) if n <= _N] or [2])})


@pytest.mark.parametrize("nproc", RANKS)
def test_native_comm_matches_library_comm(tmp_path, nproc):
    out = str(tmp_path / "r")
    env_backup = dict(os.environ)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    try:
        lib = _launch("gpu_library", out, nproc=nproc, steps=3)
        nat = _launch("gpu_native", out, nproc=nproc, steps=3)
    finally:
        os.environ.clear(); os.environ.update(env_backup)
    assert all(r["ranks_match"] for r in lib) and all(r["ranks_match"] for r in nat)
    for a, b in zip(lib[0]["losses"], nat[0]["losses"]):
        assert abs(a - b) < 5e-2, (lib[0]["losses"], nat[0]["losses"])
    pl = torch.load(f"{out}.params.gpu_library.0.pt")
    pn = torch.load(f"{out}.params.gpu_native.0.pt")
    assert float((pl - pn).norm() / pl.norm()) < 2e-2


@pytest.mark.parametrize("nproc", RANKS)
def test_fused_tp_kernels_match_library_tp(tmp_path, nproc):
    """all-gather->GEMM and GEMM->reduce-scatter kernels against NCCL collectives around plain GEMMs."""
    out = str(tmp_path / "t")
    env_backup = dict(os.environ)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    try:
        lib = _launch("gpu_tp_library", out, nproc=nproc, steps=3)
        fused = _launch("gpu_tp_fused", out, nproc=nproc, steps=3)
    finally:
        os.environ.clear(); os.environ.update(env_backup)
    assert fused[0]["fused_calls"] > 0 and fused[0]["fallback_calls"] == 0, fused[0]
    for a, b in zip(lib[0]["losses"], fused[0]["losses"]):
        assert abs(a - b) < 5e-2, (lib[0]["losses"], fused[0]["losses"])
    pl = torch.load(f"{out}.params.gpu_tp_library.pt")
    pf = torch.load(f"{out}.params.gpu_tp_fused.pt")
    assert float((pl - pf).norm() / pl.norm()) < 2e-2


@pytest.mark.parametrize("nproc", RANKS)
def test_tensor_parallel_serving_native_allreduce(tmp_path, nproc):
    """Tensor-parallel serving over all ranks: decode steps run from CUDA graphs that contain the push all-reduce
    kernel; ranks stay in lock-step; the kernel matches an exact fp32 sum."""
    env_backup = dict(os.environ)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    try:
        res = _launch("gpu_tp_serve", str(tmp_path / "s"), nproc=nproc)
    finally:
        os.environ.clear(); os.environ.update(env_backup)
    for r in res:
        assert r["ranks_equal"]
        assert r["native_calls"] > 0
        assert r["allreduce_max_err"] == 0.0                     # push kernel: one rounding, exact
        assert r["multimem_rel_err"] <= 2.0 ** -7                # in-switch sum (if used): at most one bf16 ulp apart
        assert (r["multimem_calls"] == 5) == r["has_multicast"]  # used exactly when the buffers have a multicast mapping
        assert r["fused_gemm_calls"] == 4 and r["fused_gemm_rel_err"] < 1e-2     # product + all-reduce in one launch
        assert all(len(t) == 6 for t in r["tp"])
    # bf16: sharded sums round differently, so tokens may part at a near-tie; the logits may not
    assert res[0]["logit_rel_err_max"] < 4e-2 and res[0]["flips_ok"] and res[0]["logits_compared"] >= 10, res[0]


@pytest.mark.skipif(_N < 4, reason="needs four GPUs")
def test_tensor_parallel_groups_replicated_data_parallel_gpu(tmp_path):
    """Two tensor-parallel groups of two GPUs, each a data-parallel replica with its own batch (library
    collectives inside the groups and across them): replicas end identical and track one GPU that takes
    both batches as micro-batches."""
    env_backup = dict(os.environ)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    try:
        res = _launch("gpu_tp2_dp2", str(tmp_path / "h"), nproc=4, steps=3)
    finally:
        os.environ.clear(); os.environ.update(env_backup)
    assert all(r["replicas_match"] for r in res)
    r0 = res[0]
    assert r0["rel_param_diff"] < 2e-2, r0
    by_dp = {r["dp_rank"]: r["losses"] for r in res if r["tp_rank"] == 0}
    for i, ref in enumerate(r0["ref_losses"]):
        assert abs((by_dp[0][i] + by_dp[1][i]) / 2 - ref) < 5e-2, (by_dp, r0["ref_losses"])
