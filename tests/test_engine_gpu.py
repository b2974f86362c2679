"""The executor on the sm_100a backend (bf16) against the same executor on the PyTorch backend (fp32)."""
import copy

import pytest
import torch

from kotodama_b200.config import MODEL_PRESETS, ModelConfig
from kotodama_b200.engine import TrainEngine
from kotodama_b200.models.llama import KotodamaModel

pytestmark = pytest.mark.gpu


def _cfg(**kw):
    base = dict(MODEL_PRESETS["smoke"])
    base.update(attn_res=True, attn_res_n_blocks=2, z_loss_weight=1e-4)
    base.update(kw)
    return ModelConfig(**base)


@pytest.mark.parametrize("attn_res", [True, False])
def test_gpu_step_matches_cpu_reference(attn_res):
    torch.manual_seed(0)
    cfg = _cfg(attn_res=attn_res)
    ref = KotodamaModel(cfg)
    with torch.no_grad():
        for n, p in ref.named_parameters():
            if "query" in n:
                p.normal_(0, 0.2)
    gpu_model = copy.deepcopy(ref)
    cpu = TrainEngine(ref, device="cpu", dtype=torch.float32)
    gpu = TrainEngine(gpu_model, device="cuda", dtype=torch.bfloat16)
    assert gpu.ops.name == "sm100"
    # same bf16-rounded weights on both sides
    cpu.arena.params.copy_(gpu.arena.params.float().cpu())
    ids = torch.randint(0, cfg.vocab_size, (2, 256))
    lc, _ = cpu.forward_backward(ids)
    lg, _ = gpu.forward_backward(ids.cuda())
    gpu.ops.check_status()
    assert abs(float(lc) - float(lg)) < 3e-2, (float(lc), float(lg))
    gc, gg = cpu.arena.grads, gpu.arena.grads.float().cpu()
    for s in cpu.arena.slots:
        a, b = gc[s.offset:s.offset + s.numel], gg[s.offset:s.offset + s.numel]
        err = float((a - b).norm() / (a.norm() + 1e-6))
        assert err < 8e-2 or float(a.norm()) < 1e-4, (s.name, err, float(a.norm()))


def test_gpu_training_reduces_loss():
    cfg = _cfg()
    with torch.device("meta"):
        model = KotodamaModel(cfg)
    eng = TrainEngine.from_meta(model, cfg, device="cuda", dtype=torch.bfloat16, seed=1)
    ids = torch.randint(0, cfg.vocab_size, (4, 256), device="cuda")
    losses = [float(eng.train_step([ids])["loss"]) for _ in range(8)]
    eng.ops.check_status()
    assert losses[-1] < losses[0] - 0.5, losses


def test_gpu_fp8_training_tracks_bf16():
    """--fp8 on the device: quantiser kernels + block-scaled tcgen05 GEMM in forward, data gradient and
    weight gradient of every projection; losses stay close to the bf16 run."""
    cfg = _cfg()
    ids = torch.randint(0, cfg.vocab_size, (4, 256), device="cuda", generator=torch.Generator(device="cuda").manual_seed(3))

    def run(fp8):
        with torch.device("meta"):
            model = KotodamaModel(cfg)
        eng = TrainEngine.from_meta(model, cfg, device="cuda", dtype=torch.bfloat16, seed=1, fp8=fp8)
        before = eng.ops.launches
        out = [float(eng.train_step([ids])["loss"]) for _ in range(6)]
        eng.ops.check_status()
        return out, eng.ops.launches - before

    (full, n_full), (q, n_q) = run(False), run(True)
    assert n_q > n_full                      # the quantisers ran
    assert q[-1] < q[0] - 0.5, q
    for a, b in zip(full, q):
        assert abs(a - b) < 0.15, (full, q)
