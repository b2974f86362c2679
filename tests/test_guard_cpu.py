"""Guard regions (kotodama_b200/utils/guard.py): the mechanism on CPU tensors, and a whole training step of the
CPU back end under guard (nothing writes outside its tensors, results are unchanged)."""
import torch

from kotodama_b200.config import MODEL_PRESETS, ModelConfig
from kotodama_b200.engine import TrainEngine
from kotodama_b200.models.llama import KotodamaModel
from kotodama_b200.utils.guard import CANARY, GuardRegions


def test_overruns_are_named_and_nothing_else_changes():
    plain = torch.empty
    with GuardRegions(band=256) as g:
        a = torch.empty(5, 7, dtype=torch.float32)
        b = torch.zeros(3, dtype=torch.bfloat16, device="cpu")
        c = torch.empty_like(a)
        d = torch.zeros_like(b)
        e = torch.empty((2, 2), dtype=torch.int64)
        pinned = torch.empty(4, pin_memory=False)
        assert a.shape == (5, 7) and a.is_contiguous() and a.data_ptr() % 64 == 0    # the host allocator aligns to 64 bytes, the device one to 512
        assert b.tolist() == [0, 0, 0] and d.tolist() == [0, 0, 0] and c.shape == a.shape and e.dtype == torch.int64
        a.fill_(1.0)
        c.copy_(a)
        assert g.check() == []
        # one element past the end of `a`, three elements before the start of `b`
        torch.as_strided(a, (1,), (1,), storage_offset=a.storage_offset() + a.numel()).fill_(9.0)
        torch.as_strided(b, (3,), (1,), storage_offset=b.storage_offset() - 3).fill_(1.0)
        v = g.check()
        assert len(v) == 2
        over, under = (v[0], v[1]) if v[0].side == "after" else (v[1], v[0])
        assert over.index == 0 and over.side == "after" and over.shape == (5, 7) and over.damaged >= 3
        assert under.index == 1 and under.side == "before" and under.offset == 0 and under.damaged >= 5
        assert "test_guard_cpu.py" in over.where and "written after the tensor" in str(over)
        try:
            g.assert_clean()
            raise RuntimeError("assert_clean did not raise")
        except AssertionError as err:
            assert "allocation #0" in str(err) and "allocation #1" in str(err)
        assert pinned.numel() == 4
    assert torch.empty is plain                                   # the allocators are restored
    assert int(torch.empty(1, dtype=torch.uint8).fill_(CANARY)) == 0xA5


def test_a_training_step_of_the_cpu_back_end_stays_inside_its_tensors():
    cfg = ModelConfig(**dict(MODEL_PRESETS["tiny"], vocab_size=512), attn_res=True, attn_res_n_blocks=2)
    ids = torch.randint(0, cfg.vocab_size, (2, 48), generator=torch.Generator().manual_seed(0))

    def step(guarded: bool):
        torch.manual_seed(0)
        eng = TrainEngine(KotodamaModel(cfg), device="cpu", dtype=torch.float32)
        if not guarded:
            return float(eng.train_step([ids])["loss"]), float(eng.train_step([ids])["loss"]), 0
        with GuardRegions(device_types=("cpu",)) as g:
            l0 = float(eng.train_step([ids])["loss"])
            l1 = float(eng.train_step([ids])["loss"])
            g.assert_clean()
            return l0, l1, len(g.records)
    a0, a1, _ = step(False)
    b0, b1, n = step(True)
    assert (a0, a1) == (b0, b1) and a1 < a0 and n > 10            # same numbers, and the guard saw the step's allocations
