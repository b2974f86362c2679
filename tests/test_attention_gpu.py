"""The tcgen05 flash-attention kernels (forward, dQ, dK/dV) against plain PyTorch fp32 attention
with autograd, on the operand layout the executor uses (q|k and q|k|v side by side in fused rows,
gradients written into fused gradient rows)."""
import math

import pytest
import torch

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


def reference(q, k, v, do=None):
    """fp32 causal GQA attention of one batch element at a time: o, lse and (with ``do``) dq, dk, dv."""
    B, T, H, hd = q.shape
    KV = k.shape[2]
    outs = []
    for b in range(B):
        qf = q[b].float().permute(1, 0, 2).detach().requires_grad_(do is not None)        # [H,T,hd]
        kf = k[b].float().permute(1, 0, 2).detach().requires_grad_(do is not None)        # [KV,T,hd]
        vf = v[b].float().permute(1, 0, 2).detach().requires_grad_(do is not None)
        ke, ve = kf.repeat_interleave(H // KV, 0), vf.repeat_interleave(H // KV, 0)
        sc = (qf @ ke.transpose(-1, -2)) / math.sqrt(hd)
        sc = sc.masked_fill(~torch.ones(T, T, dtype=torch.bool, device=q.device).tril(), float("-inf"))
        lse = torch.logsumexp(sc, -1)
        o = torch.softmax(sc, -1) @ ve                                                    # [H,T,hd]
        res = [o.detach().permute(1, 0, 2), lse.detach()]
        if do is not None:
            dq, dk, dv = torch.autograd.grad(o, (qf, kf, vf), do[b].float().permute(1, 0, 2))
            res += [dq.permute(1, 0, 2), dk.permute(1, 0, 2), dv.permute(1, 0, 2)]
        outs.append(res)
        del sc, o
    return [torch.stack([r[i] for r in outs]) for i in range(len(outs[0]))]


def fused_operands(B, T, H, KV, hd, seed):
    qk = bf(B * T, (H + KV) * hd, seed=seed)                # q and k side by side, as the executor stores them
    qkv = bf(B * T, (H + 2 * KV) * hd, seed=seed + 1)
    q = qk[:, : H * hd].view(B, T, H, hd)
    k = qk[:, H * hd:].view(B, T, KV, hd)
    v = qkv[:, (H + KV) * hd:].view(B, T, KV, hd)
    return q, k, v


CASES = [(1, 128, 2, 1, 128), (2, 512, 6, 2, 128), (1, 1024, 3, 3, 128), (1, 200, 3, 1, 128), (2, 333, 4, 2, 128),
         (1, 77, 2, 2, 128), (1, 128, 24, 8, 128), (8, 333, 24, 8, 128), (1, 4096, 24, 8, 128), (2, 256, 4, 2, 64),
         (2, 333, 4, 2, 64), (1, 1000, 6, 2, 64)]


@pytest.mark.parametrize("B,T,H,KV,hd", CASES)
def test_flash_attention_forward_backward(ops, B, T, H, KV, hd):
    from kotodama_b200.ops.flash import flash_bwd, flash_fwd, supported
    q, k, v = fused_operands(B, T, H, KV, hd, seed=21)
    assert supported(q)
    o, lse = flash_fwd(ops, q, k, v)
    ops.check_status()
    do = bf(B, T, H, hd, seed=5)
    oref, lref, dqr, dkr, dvr = reference(q, k, v, do)
    assert rel_err(o, oref) < 2e-2, rel_err(o, oref)
    assert float((lse - lref).abs().max()) < 2e-2
    # gradients land inside fused buffers: dq|dk in one, dv at the tail of a q|k|v-wide one
    dqk = torch.full((B * T, (H + KV) * hd), float("nan"), device="cuda", dtype=torch.bfloat16)
    dqkv = torch.full((B * T, (H + 2 * KV) * hd), float("nan"), device="cuda", dtype=torch.bfloat16)
    dq = dqk[:, : H * hd].view(B, T, H, hd)
    dk = dqk[:, H * hd:].view(B, T, KV, hd)
    dv = dqkv[:, (H + KV) * hd:].view(B, T, KV, hd)
    flash_bwd(ops, do, q, k, v, o, lse, dq, dk, dv)
    ops.check_status()
    assert rel_err(dq, dqr) < 3e-2, rel_err(dq, dqr)
    assert rel_err(dk, dkr) < 3e-2, rel_err(dk, dkr)
    assert rel_err(dv, dvr) < 3e-2, rel_err(dv, dvr)
    assert torch.isnan(dqkv[:, : (H + KV) * hd]).all()       # nothing written outside the destination views


def test_flash_attention_large_batch_matches_small(ops):
    """B = 8, T = 4096, 24/8 heads (the training shape): every batch element equals the same element
    run alone (already checked against fp32 above), forward and backward."""
    from kotodama_b200.ops.flash import flash_bwd, flash_fwd
    B, T, H, KV, hd = 8, 4096, 24, 8, 128
    q, k, v = fused_operands(B, T, H, KV, hd, seed=31)
    do = bf(B, T, H, hd, seed=6)
    o, lse = flash_fwd(ops, q, k, v)
    dq, dk, dv = torch.empty_like(q.contiguous()), torch.empty_like(k.contiguous()), torch.empty_like(v.contiguous())
    flash_bwd(ops, do, q, k, v, o, lse, dq, dk, dv)
    ops.check_status()
    for b in (0, 5, 7):
        o1, l1 = flash_fwd(ops, q[b:b + 1], k[b:b + 1], v[b:b + 1])
        assert torch.equal(o1[0], o[b]) and torch.equal(l1[0], lse[b])
        dq1, dk1, dv1 = torch.empty_like(dq[:1]), torch.empty_like(dk[:1]), torch.empty_like(dv[:1])
        flash_bwd(ops, do[b:b + 1], q[b:b + 1], k[b:b + 1], v[b:b + 1], o1, l1, dq1, dk1, dv1)
        assert torch.equal(dq1[0], dq[b]) and torch.equal(dk1[0], dk[b]) and torch.equal(dv1[0], dv[b])
    ops.check_status()


@pytest.mark.parametrize("hd", [128, 64])
def test_flash_attention_packed_sequences(ops, hd):
    """cu_seqlens form (serving prefill): every packed sequence equals the same sequence run alone."""
    from kotodama_b200.ops.flash import flash_fwd
    H, KV = 6, 2
    lens = [130, 17, 512, 1, 300]
    total = sum(lens)
    q, k, v = fused_operands(1, total, H, KV, hd, seed=41)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), device="cuda", dtype=torch.int32)
    o, lse = flash_fwd(ops, q, k, v, cu_seqlens=cu, max_seqlen=max(lens))
    ops.check_status()
    at = 0
    for n in lens:
        oref, lref = reference(q[:, at:at + n], k[:, at:at + n], v[:, at:at + n])
        assert rel_err(o[:, at:at + n], oref) < 2e-2
        assert float((lse[:, at:at + n] - lref[0]).abs().max()) < 2e-2
        at += n
