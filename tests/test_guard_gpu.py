"""Guard regions on the device: the kernels of a training step, of the decode path and of the GEMM families keep
their writes inside the tensors they are given (canary bands around every output and workspace stay intact),
also for shapes that are not multiples of the tile sizes."""
import pytest
import torch

from kotodama_b200.config import MODEL_PRESETS, ModelConfig
from kotodama_b200.engine import TrainEngine
from kotodama_b200.models.llama import KotodamaModel
from kotodama_b200.utils.guard import GuardRegions

pytestmark = pytest.mark.gpu


def bf(*shape, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return torch.randn(*shape, device="cuda", generator=g).bfloat16()


@pytest.fixture(scope="module")
def ops():
    from kotodama_b200.ops import get_ops
    o = get_ops("cuda")
    assert o.name == "sm100"
    return o


def test_the_guard_sees_a_device_side_overrun():
    """The mechanism itself on the device: a copy that is one row too long is reported (it lands in the band,
    memory this process owns)."""
    with GuardRegions() as g:
        a = torch.empty(8, 64, device="cuda", dtype=torch.bfloat16)
        a.fill_(1.0)
        assert g.check() == []
        torch.as_strided(a, (9, 64), (64, 1)).fill_(2.0)
        v = g.check()
    assert len(v) == 1 and v[0].side == "after" and v[0].offset == 0 and v[0].damaged == 128


@pytest.mark.parametrize("M,N,K", [(200, 136, 72), (64, 5120, 3072), (37, 3072, 1024), (384, 768, 3072), (1000, 264, 520)])
def test_gemm_outputs_are_not_overrun(ops, M, N, K):
    a, b = bf(M, K, seed=1), bf(N, K, seed=2)
    with GuardRegions() as g:
        out = ops.gemm_nt(a, b)
        res = ops.gemm_nt(a, b, residual=out)
        g.assert_clean()
    ops.check_status()
    assert out.shape == (M, N) and res.shape == (M, N)


def test_decode_path_kernels_are_not_overrun(ops):
    nq, nkv, hd, P, B = 24, 8, 128, 96, 5
    qkv = bf(B, (nq + 2 * nkv) * hd, seed=3)
    qw, kw = bf(hd, seed=4) + 1, bf(hd, seed=5) + 1
    cos, sin = (torch.randn(2048, hd, device="cuda") for _ in range(2))
    pos = torch.tensor([3, 17, 300, 513, 1100], device="cuda", dtype=torch.int32)
    table = torch.arange(B * 80, device="cuda", dtype=torch.int32).reshape(B, 80) % P
    slots = (table[torch.arange(B), (pos // 16).long()].long() * 16 + (pos % 16).long())
    srcs = [bf(B, 3072, seed=10 + i) for i in range(3)]
    with GuardRegions() as g:
        kp = torch.zeros(P, nkv, 16, hd, device="cuda", dtype=torch.bfloat16)
        vp = torch.zeros_like(kp)
        qk, _ = ops.qknorm_rope_fwd(qkv, qw, kw, cos, sin, B, nq, nkv, hd, 1e-5, positions=pos, append=(kp, vp, slots))
        att = ops.paged_decode_attention(qk[:, : nq * hd], kp, vp, table, pos + 1, int(pos.max()) + 1, nq, nkv, hd)
        act = ops.swiglu_fwd(bf(B, 2 * 8192, seed=6))
        xn, _ = ops.route_norm_fwd(srcs, bf(3072, seed=7), bf(3072, seed=8) + 1, bf(3072, seed=9) + 1, 1e-5)
        tok = ops.argmax(bf(B, 49152, seed=11))
        g.assert_clean()
    ops.check_status()
    assert att.shape == (B, nq * hd) and act.shape == (B, 8192) and xn.shape == (B, 3072) and tok.shape == (B,)


def test_a_training_step_on_the_device_is_not_overrun():
    cfg = ModelConfig(**dict(MODEL_PRESETS["smoke"], attn_res=True, attn_res_n_blocks=2, z_loss_weight=1e-4))
    with torch.device("meta"):
        model = KotodamaModel(cfg)
    eng = TrainEngine.from_meta(model, cfg, device="cuda", dtype=torch.bfloat16, seed=1)
    ids = torch.randint(0, cfg.vocab_size, (3, 200), device="cuda")       # 600 tokens: no multiple of any tile
    eng.train_step([ids])
    with GuardRegions() as g:
        l0 = float(eng.train_step([ids])["loss"])
        l1 = float(eng.train_step([ids])["loss"])
        g.assert_clean()
        assert len(g.records) > 100
    eng.ops.check_status()
    assert l1 < l0
