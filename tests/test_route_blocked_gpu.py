"""Blocked AttnRes routing kernels (phase 1 for all queries of a block, phase 2 merge per
sub-layer, both directions) against the plain-PyTorch fp32 statement of the same ops."""
import pytest
import torch

from kotodama_b200.ops.reference import TORCH_OPS

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from kotodama_b200.ops import get_ops
    o = get_ops("cuda")
    assert o.name == "sm100"
    return o


def rel_err(a, b):
    a, b = a.float(), b.float()
    return float((a - b).norm() / (b.norm() + 1e-12))


def bf(*shape, scale=1.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, device="cuda", generator=g) * scale).bfloat16()


@pytest.mark.parametrize("N,D,S,Q", [(777, 3072, 1, 3), (777, 3072, 2, 8), (512, 3072, 5, 8), (300, 3072, 7, 8),
                                     (300, 3072, 8, 11), (1000, 256, 3, 5), (260, 4096, 8, 8), (515, 1024, 4, 19),
                                     (129, 64, 2, 4)])
def test_route_phase1_forward_backward(ops, N, D, S, Q):
    assert ops.route_blocked_ok(S, D)
    srcs = [bf(N, D, seed=10 + s, scale=0.5 + 0.3 * s) for s in range(S)]
    qs, rns = bf(Q, D, seed=3, scale=0.05), (1 + 0.1 * bf(Q, D, seed=4).float()).bfloat16()
    o, lse, stats = ops.route_p1_fwd(srcs, qs, rns, 1e-5)
    ops.check_status()
    # the kernels fold the query in bf16 (as the reference model does: query * norm.weight in the parameter dtype)
    wq = (qs.float() * rns.float()).bfloat16()
    ones = torch.ones_like(wq)
    oref, lref, sref = TORCH_OPS.route_p1_fwd([s.float() for s in srcs], wq.float(), ones.float(), 1e-5)
    assert rel_err(o, oref) < 1e-2, rel_err(o, oref)
    assert float((lse - lref).abs().max()) < 2e-2
    assert rel_err(stats[0], sref[0]) < 1e-3 and float((stats[1] - sref[1]).abs().max()) < 2e-2
    # backward
    do = bf(Q, N, D, seed=7)
    dlse = torch.randn(Q, N, device="cuda", generator=torch.Generator(device="cuda").manual_seed(8)) * 0.1
    acc = [s % 2 == 1 for s in range(S)]
    init = [bf(N, D, seed=40 + s) for s in range(S)]
    dsrcs = [t.clone() for t in init]
    dws = ops.route_p1_bwd(srcs, qs, rns, do, dlse, lse, stats, dsrcs, acc)
    ops.check_status()
    dref = [t.float().clone() for t in init]
    dwr = TORCH_OPS.route_p1_bwd([s.float() for s in srcs], wq.float(), ones.float(), do.float(), dlse, lref, sref, dref, acc)
    for s in range(S):
        assert rel_err(dsrcs[s], dref[s]) < 1.5e-2, (s, rel_err(dsrcs[s], dref[s]))
    assert rel_err(dws, dwr) < 2e-2, rel_err(dws, dwr)


@pytest.mark.parametrize("N,D", [(777, 3072), (2048, 3072), (300, 4096), (1000, 256), (129, 64), (64, 8192)])
@pytest.mark.parametrize("with_partial,acc", [(True, False), (True, True), (False, False)])
def test_route_phase2_forward_backward(ops, N, D, with_partial, acc):
    o = bf(N, D, seed=1)
    part = bf(N, D, seed=2, scale=1.5) if with_partial else None
    lse = torch.randn(N, device="cuda", generator=torch.Generator(device="cuda").manual_seed(3))
    q, rn, nw = bf(D, seed=4, scale=0.05), (1 + 0.1 * bf(D, seed=5).float()).bfloat16(), (1 + 0.1 * bf(D, seed=6).float()).bfloat16()
    xn, st2 = ops.route_p2_fwd(o, lse, part, q, rn, nw, 1e-5)
    xr, sr = TORCH_OPS.route_p2_fwd(o.float(), lse, None if part is None else part.float(), q.float(), rn.float(), nw.float(), 1e-5)
    assert rel_err(xn, xr) < 1e-2, rel_err(xn, xr)
    assert float((st2[0] - sr).abs().max()) < 1e-2
    dxn = bf(N, D, seed=9)
    do, dlse = torch.empty_like(o), torch.empty(N, device="cuda")
    init = bf(N, D, seed=11)
    dpart = init.clone() if with_partial else None
    dw, dnw = ops.route_p2_bwd(dxn, o, lse, part, q, rn, nw, 1e-5, st2, do, dlse, dpart, acc)
    ops.check_status()
    dor, dlr = torch.empty(N, D, device="cuda"), torch.empty(N, device="cuda")
    dpr = init.float().clone() if with_partial else None
    dwr, dnwr = TORCH_OPS.route_p2_bwd(dxn.float(), o.float(), lse, None if part is None else part.float(), q.float(),
                                       rn.float(), nw.float(), 1e-5, sr, dor, dlr, dpr, acc)
    assert rel_err(do, dor) < 1e-2 and rel_err(dnw, dnwr) < 1e-2
    assert float((dlse - dlr).abs().max()) < 2e-2 * max(1.0, float(dlr.abs().max()))
    if with_partial:
        assert rel_err(dpart, dpr) < 1.5e-2, rel_err(dpart, dpr)
        assert rel_err(dw, dwr) < 2e-2, rel_err(dw, dwr)
    else:
        assert dw is None
