"""Worker launched by the distributed tests (one process per rank)."""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from kotodama_b200.config import MODEL_PRESETS, ModelConfig  # noqa: E402
from kotodama_b200.engine import TrainEngine  # noqa: E402
from kotodama_b200.models.llama import KotodamaModel  # noqa: E402
from kotodama_b200.parallel.comm import LibraryComm  # noqa: E402


def build(cfg, device, dtype, comm, seed=0):
    torch.manual_seed(seed)
    model = KotodamaModel(cfg)
    return TrainEngine(model, device=device, dtype=dtype, comm=comm, muon_lr=0.02, adamw_lr=1e-3)


def tp_cfg(world: int) -> ModelConfig:
    """Model for the tensor-parallel modes: the smoke preset up to two ranks, a wider one (8 query and
    8 key/value heads, every projection a multiple of 64 columns per rank) for four and eight."""
    if world <= 2:
        return ModelConfig(**MODEL_PRESETS["smoke"], attn_res=True, attn_res_n_blocks=2)
    return ModelConfig(hidden_size=512, num_layers=4, num_attention_heads=8, num_kv_heads=8, head_dim=64,
                       intermediate_size=1024, vocab_size=1024, max_position_embeddings=2048, attn_res=True,
                       attn_res_n_blocks=2)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", required=True)
    ap.add_argument("--out", required=True)
    ap.add_argument("--steps", type=int, default=3)
    a = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    cuda = a.mode.startswith("gpu")
    if cuda:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    import datetime
    dist.init_process_group("nccl" if cuda else "gloo",
                            timeout=datetime.timedelta(seconds=20 if a.mode.startswith("cpu_rank_leaves") else 600))
    device = torch.device("cuda", torch.cuda.current_device()) if cuda else torch.device("cpu")
    dtype = torch.bfloat16 if cuda else torch.float32
    preset = "smoke" if cuda else "tiny"
    cfg = ModelConfig(**MODEL_PRESETS[preset], attn_res=True, attn_res_n_blocks=2)
    seq = 256
    g = torch.Generator().manual_seed(100 + rank)
    batch = torch.randint(0, cfg.vocab_size, (2, seq), generator=g)
    result = {"rank": rank}
    if a.mode in ("cpu_ddp", "gpu_library", "gpu_native"):
        if a.mode == "gpu_native":
            from kotodama_b200.parallel.native import NativeComm
            comm = NativeComm(distributed_muon=True)
        else:
            comm = LibraryComm(distributed_muon=True)
        eng = build(cfg, device, dtype, comm)
        losses = [float(eng.train_step([batch])["loss"]) for _ in range(a.steps)]
        eng.check()
        p = eng.arena.params.float()
        gathered = [torch.empty_like(p) for _ in range(world)]
        dist.all_gather(gathered, p)
        result.update(losses=losses, ranks_match=all(torch.equal(gathered[0], t) for t in gathered),
                      checksum=float(p.double().abs().sum()))
        if a.mode != "cpu_ddp":
            torch.save(p.cpu(), f"{a.out}.params.{a.mode}.{rank}.pt")
        sd = eng.muon_state_dict()
        result["momentum_entries"] = len(sd["state"])
    if a.mode in ("cpu_tp_sp", "cpu_tp"):
        from kotodama_b200.parallel.tp import TensorParallelComm, create_process_groups, gather_full_state_dict
        tp_group, _ = create_process_groups(world, world)
        comm = TensorParallelComm(tp_group, None, sequence_parallel=(a.mode == "cpu_tp_sp"))
        cfg = ModelConfig(**MODEL_PRESETS["smoke"], attn_res=True, attn_res_n_blocks=2)
        shared = torch.randint(0, cfg.vocab_size, (2, 64), generator=torch.Generator().manual_seed(7))
        eng = build(cfg, device, dtype, comm)
        losses = [float(eng.train_step([shared])["loss"]) for _ in range(a.steps)]
        full = gather_full_state_dict(eng.model, tp_group)
        result.update(losses=losses, checksum=float(sum(v.double().abs().sum() for v in full.values())),
                      q_shape=list(full["layers.0.attn.q_proj.weight"].shape),
                      local_q_shape=list(eng.model.layers[0].attn.q_proj.weight.shape),
                      momentum_shape=list(eng.muon_state_dict()["state"][0]["momentum_buffer"].shape))
    if a.mode in ("cpu_tp2_dp2", "gpu_tp2_dp2"):
        # tensor parallel groups of two ranks, replicated data-parallel: every replica gets its own batch
        from kotodama_b200.parallel.tp import TensorParallelComm, create_process_groups, gather_full_state_dict
        tp_group, dp_group = create_process_groups(world, 2)
        comm = TensorParallelComm(tp_group, dp_group, sequence_parallel=True)
        cfg = ModelConfig(**MODEL_PRESETS["smoke"], attn_res=True, attn_res_n_blocks=2)
        batches = [torch.randint(0, cfg.vocab_size, (2, 128 if cuda else 64), generator=torch.Generator().manual_seed(7 + d))
                   for d in range(world // 2)]
        eng = build(cfg, device, dtype, comm)
        losses = [float(eng.train_step([batches[comm.dp_rank]])["loss"]) for _ in range(a.steps)]
        if cuda:
            eng.check()
        full = gather_full_state_dict(eng.model, tp_group)
        flat = torch.cat([v.float().flatten() for _, v in sorted(full.items())])
        everyone = [torch.empty_like(flat) for _ in range(world)]
        dist.all_gather(everyone, flat)
        result.update(losses=losses, dp_rank=comm.dp_rank, tp_rank=comm.tp_rank,
                      replicas_match=all(torch.equal(everyone[0], t) for t in everyone),
                      checksum=float(flat.double().abs().sum()))
        if rank == 0:
            # the same job in one process: both replicas' batches as two micro-batches of one step
            ref = build(cfg, device, dtype, None)
            ref_losses = [float(ref.train_step(batches)["loss"]) for _ in range(a.steps)]
            ref_flat = torch.cat([v.float().flatten() for _, v in sorted(ref.model.state_dict().items())])
            result.update(ref_losses=ref_losses, ref_checksum=float(ref_flat.double().abs().sum()),
                          rel_param_diff=float((flat - ref_flat.to(flat.device)).norm() / ref_flat.norm()))
    if a.mode in ("gpu_tp_library", "gpu_tp_fused"):
        from kotodama_b200.parallel.tp import TensorParallelComm, create_process_groups, gather_full_state_dict
        tp_group, _ = create_process_groups(world, world)
        if a.mode == "gpu_tp_fused":
            from kotodama_b200.parallel.tp_native import FusedTensorParallelComm
            comm = FusedTensorParallelComm(tp_group, None)
        else:
            comm = TensorParallelComm(tp_group, None, sequence_parallel=True)
        cfg = tp_cfg(world)
        shared = torch.randint(0, cfg.vocab_size, (2, 128 * world), generator=torch.Generator().manual_seed(7))
        eng = build(cfg, device, dtype, comm)
        losses = [float(eng.train_step([shared])["loss"]) for _ in range(a.steps)]
        eng.check()
        full = gather_full_state_dict(eng.model, tp_group)
        flat = torch.cat([v.float().flatten() for _, v in sorted(full.items())])
        if rank == 0:
            torch.save(flat.cpu(), f"{a.out}.params.{a.mode}.pt")
        result.update(losses=losses, fused_calls=getattr(comm, "fused_calls", 0),
                      fallback_calls=getattr(comm, "fallback_calls", 0))
    if a.mode in ("cpu_tp_serve", "gpu_tp_serve"):
        import copy
        from kotodama_b200.serve.engine import SamplingParams, ServingEngine
        from kotodama_b200.serve.tp import ServeTP, TPLeader, run_follower
        cfg = tp_cfg(world) if cuda else ModelConfig(**MODEL_PRESETS["smoke"], attn_res=True, attn_res_n_blocks=2)
        torch.manual_seed(0)
        full = KotodamaModel(cfg)
        prompts = [[(7 * i + 3 * j) % cfg.vocab_size for j in range(5 + 3 * i)] for i in range(5)]
        params = SamplingParams(max_new_tokens=6, temperature=0.0)
        ref_eng = ServingEngine(copy.deepcopy(full), device=device, dtype=dtype, max_batch=8, max_ctx=256)
        ref_eng.logit_trace = []
        ref = ref_eng.generate(prompts, params)
        os.environ["KOTODAMA_SERVE_MULTIMEM"] = "1"     # exercise the in-switch all-reduce where the box offers it
        tp = ServeTP()
        eng = ServingEngine(full, device=device, dtype=dtype, max_batch=8, max_ctx=256, tp=tp)
        eng.logit_trace = []
        if rank == 0:
            lead = TPLeader(eng, tp)
            gen = lead.generate(prompts, params)
            # second phase: a request is cancelled while it decodes; every rank must drop it at the same step
            extra = [lead.add_request(p, SamplingParams(max_new_tokens=5, temperature=0.0)) for p in prompts[:3]]
            lead.step()
            lead.step()
            lead.cancel(extra[1].rid)
            while lead.has_work():
                lead.step()
            lead.shutdown()
            extra_out = [(list(r.generated), r.finish_reason) for r in extra]
            control = lead.control
        else:
            mirrored = run_follower(eng, tp)
            gen = [r.generated for r in mirrored[:len(prompts)]]
            extra_out = [(list(r.generated), r.finish_reason) for r in mirrored[len(prompts):]]
            control = None
        extras = [None] * world
        dist.all_gather_object(extras, extra_out)
        result.update(extra_equal=all(e == extras[0] for e in extras), extra=extras[0])
        if control is not None:
            result.update(control_steps=control.step_no, control_body_bytes=control.body_bytes)
        # every rank ran the same requests: compare what each rank generated
        gathered = [None] * world
        dist.all_gather_object(gathered, [list(g) for g in gen])
        result.update(ref=ref, tp=gathered[0], ranks_equal=all(g == gathered[0] for g in gathered),
                      native_calls=tp.native_calls, library_calls=tp.library_calls,
                      local_heads=eng.H, local_kv=eng.KV)
        # by logits: while a request's token history is shared, every pass must agree within rounding;
        # where the greedy tokens part, the unsharded margin between the two candidates must be within it

        def per_request(trace):
            out = {}
            for rids, lg in trace:
                for i, rid in enumerate(rids):
                    out.setdefault(rid, []).append(lg[i])
            return [out[k] for k in sorted(out)]
        worst, flips_ok, compared = 0.0, True, 0
        for rt, tt, rl, tl in zip(ref, gen, per_request(ref_eng.logit_trace), per_request(eng.logit_trace)):
            for i in range(min(len(rl), len(tl))):
                err = float((tl[i] - rl[i]).abs().max())
                worst = max(worst, float((tl[i] - rl[i]).norm() / (rl[i].norm() + 1e-12)))
                compared += 1
                if rt[i] != tt[i]:
                    margin = float(rl[i][rt[i]] - rl[i][tt[i]])
                    flips_ok = flips_ok and 0 <= margin <= 2 * err + 1e-6
                    break
        result.update(logit_rel_err_max=worst, flips_ok=flips_ok, logits_compared=compared)
        if cuda:
            eng.ops.check_status()
            # the all-reduce kernel alone, against an exact fp32 sum of the gathered partials
            g = torch.Generator(device="cuda").manual_seed(10 + rank)
            y = torch.randn(48, cfg.hidden_size, device="cuda", generator=g).to(torch.bfloat16)
            res = torch.randn(48, cfg.hidden_size, device="cuda", generator=torch.Generator(device="cuda").manual_seed(5)).to(torch.bfloat16)
            parts = [torch.empty_like(y) for _ in range(world)]
            dist.all_gather(parts, y)
            exact = (sum(p.float() for p in parts) + res.float()).to(torch.bfloat16)
            def worst():
                errs = []
                for _ in range(5):                  # repeated calls walk through both parities
                    got = tp.all_reduce(eng.ops, y, res)
                    errs.append(float((got.float() - exact.float()).abs().max()))
                eng.ops.check_status()
                return max(errs)
            # in-switch reduction (when the buffers have a multicast mapping): the switch rounds the sum to
            # bf16 before the residual is added, so it may differ from the once-rounded sum by one ulp
            mm_calls0 = tp.multimem_calls
            mm_err = worst()
            used_mm = tp.multimem_calls - mm_calls0
            saved, tp.mc_ptr = tp.mc_ptr, 0         # plain peer stores: exact
            push_err = worst()
            tp.mc_ptr = saved
            # the row-parallel projection in one launch (cluster split-K product with the all-reduce in its epilogue)
            saved_mc, tp.mc_ptr = tp.mc_ptr, 0
            f0 = tp.fused_calls
            errs_k = []
            for (Kk, Nk) in ((1024, 1536), (384, 3072)):          # the second: a shard as thin as 3072 / 8
                gk = torch.Generator(device="cuda").manual_seed(20 + rank)
                xk = (torch.randn(48, Kk, device="cuda", generator=gk) * 0.1).to(torch.bfloat16)
                wk = (torch.randn(Nk, Kk, device="cuda", generator=gk) * 0.1).to(torch.bfloat16)
                rk = torch.randn(48, Nk, device="cuda", generator=torch.Generator(device="cuda").manual_seed(6)).to(torch.bfloat16)
                part = (xk.float() @ wk.float().t()).to(torch.bfloat16)
                parts_k = [torch.empty_like(part) for _ in range(world)]
                dist.all_gather(parts_k, part)
                want = sum(t.float() for t in parts_k) + rk.float()
                for _ in range(2):                   # both parities, interleaved with the plain all-reduce
                    got = tp.row_linear(eng.ops, xk, wk, rk)
                    errs_k.append(float((got.float() - want).norm() / want.norm()))
                    tp.all_reduce(eng.ops, y, res)
            tp.mc_ptr = saved_mc
            eng.ops.check_status()
            result.update(fused_gemm_calls=tp.fused_calls - f0, fused_gemm_rel_err=max(errs_k))
            result.update(allreduce_max_err=push_err, multimem_calls=used_mm, has_multicast=bool(saved),
                          multimem_rel_err=mm_err / float(exact.float().abs().max()))
    if a.mode in ("cpu_rank_leaves", "cpu_rank_leaves_silent"):
        # the last rank leaves the job between steps: with a notice in the store (the others raise on
        # the host before their next step) or silently (their next collective ends with an error
        # within the process group's timeout)
        import time
        from kotodama_b200.parallel.health import PeerHealth, PeerLeft
        comm = LibraryComm(distributed_muon=True)
        eng = build(cfg, device, dtype, comm)
        health = PeerHealth()
        outcome, steps_done, t_detect = "completed", 0, None
        for step in range(4):
            try:
                if a.mode == "cpu_rank_leaves":
                    health.raise_if_peer_left()
                health.beat(step)
                if rank == world - 1 and step == 2:
                    if a.mode == "cpu_rank_leaves":
                        health.announce_leave("test: leaving between steps")
                    outcome = "left"
                    break
                if rank != world - 1 and step == 2:
                    time.sleep(1.0)                 # let the notice (or the exit) happen first
                    if a.mode == "cpu_rank_leaves":
                        health.raise_if_peer_left()
                t0 = time.time()
                eng.train_step([batch])
                steps_done += 1
            except PeerLeft as e:
                outcome, t_detect = "peer_left:" + str(e), 0.0
                break
            except Exception as e:                  # noqa: BLE001 - the collective failed
                outcome, t_detect = "collective_error:" + type(e).__name__, time.time() - t0
                break
        result.update(outcome=outcome, steps_done=steps_done, detect_s=t_detect)
        with open(f"{a.out}.{a.mode}.{rank}.json", "w") as fh:
            json.dump(result, fh)
        os._exit(0)                                 # no barrier: the group is incomplete by design
    if a.mode == "cpu_tp_autograd":
        from kotodama_b200.optim.muon import build_hybrid_optimizer
        from kotodama_b200.parallel.tp import (apply_tensor_parallelism, create_process_groups, gather_full_state_dict,
                                               sync_tp_replicated_grads, tp_clip_grad_norm)
        tp_group, _ = create_process_groups(world, world)
        cfg = ModelConfig(**MODEL_PRESETS["smoke"], attn_res=True, attn_res_n_blocks=2)
        torch.manual_seed(0)
        model = KotodamaModel(cfg)
        apply_tensor_parallelism(model, tp_group)
        muon, adamw = build_hybrid_optimizer(model, muon_lr=0.02, adamw_lr=1e-3)
        shared = torch.randint(0, cfg.vocab_size, (2, 64), generator=torch.Generator().manual_seed(7))
        losses = []
        for _ in range(a.steps):
            out = model(shared, labels=shared)
            out["loss"].backward()
            sync_tp_replicated_grads(model, tp_group)
            tp_clip_grad_norm(model, 1.0, tp_group)
            muon.step(); adamw.step(); muon.zero_grad(); adamw.zero_grad()
            losses.append(float(out["loss"]))
        full = gather_full_state_dict(model, tp_group)
        result.update(losses=losses, checksum=float(sum(v.double().abs().sum() for v in full.values())))
    if a.mode == "cpu_tp_reference_parity":
        # the reference's own tensor-parallel code (unmodified, from the baseline install) next to this package's
        # autograd API, same weights, same batch, same process group: shards, loss and local gradients
        import importlib
        import types
        ref_root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref")
        if not os.path.isdir(os.path.join(ref_root, "training")):
            result["skipped"] = "reference not installed"
        else:
            pkg = types.ModuleType("src")
            pkg.__path__ = [ref_root]
            sys.modules.setdefault("src", pkg)
            r_llama = importlib.import_module("src.model.llama")
            r_tp = importlib.import_module("src.training.tensor_parallel")
            from kotodama_b200.parallel import tp as o_tp
            kw = dict(hidden_size=64, num_layers=4, num_attention_heads=4, num_kv_heads=2, head_dim=16, intermediate_size=96,
                      vocab_size=211, max_position_embeddings=64, z_loss_weight=1e-3, attn_res=True, attn_res_n_blocks=2)
            torch.manual_seed(0)
            theirs = r_llama.LuxiaBaseModel(r_llama.LuxiaModelConfig(attn_impl="sdpa", **kw))
            gq = torch.Generator().manual_seed(3)
            with torch.no_grad():
                for n, p_ in theirs.named_parameters():
                    if "query" in n:
                        p_.copy_(torch.randn(p_.shape, generator=gq) * 0.3)
            ours = KotodamaModel(ModelConfig(**kw))
            ours.load_state_dict(theirs.state_dict())
            tp_group, _ = o_tp.create_process_groups(world, world)
            r_tp.apply_tensor_parallelism(theirs, tp_group)
            o_tp.apply_tensor_parallelism(ours, tp_group)
            shards_equal = all(torch.equal(p1, p2) for (_, p1), (_, p2) in zip(theirs.named_parameters(), ours.named_parameters()))
            shared = torch.randint(0, 211, (2, 24), generator=torch.Generator().manual_seed(7))
            la = theirs(shared, labels=shared)["loss"]
            lb = ours(shared, labels=shared)["loss"]
            la.backward()
            lb.backward()
            r_tp.sync_tp_replicated_grads(theirs, tp_group)
            o_tp.sync_tp_replicated_grads(ours, tp_group)
            worst = 0.0
            for (n, p1), (_, p2) in zip(theirs.named_parameters(), ours.named_parameters()):
                if p1.grad is None or p2.grad is None:
                    worst = max(worst, 0.0 if (p1.grad is None) == (p2.grad is None) else 1.0)
                    continue
                worst = max(worst, float((p1.grad - p2.grad).norm() / (p1.grad.norm() + 1e-12)))
            # the reference's tp_clip_grad_norm allocates on "cuda" unconditionally; on CPU ranks its rule is restated:
            # squared norms of the sharded gradients summed over the group, those of the replicated ones counted once
            sharded = sum(float(p_.grad.pow(2).sum()) for p_ in theirs.parameters() if p_.grad is not None and hasattr(p_, "_tp_shard_dim"))
            repl = sum(float(p_.grad.pow(2).sum()) for p_ in theirs.parameters() if p_.grad is not None and not hasattr(p_, "_tp_shard_dim"))
            t = torch.tensor([sharded], dtype=torch.float64)
            dist.all_reduce(t, group=tp_group)
            na = float((t[0] + repl) ** 0.5)
            nb = float(o_tp.tp_clip_grad_norm(ours, 1.0, tp_group))
            result.update(shards_equal=shards_equal, loss_theirs=float(la), loss_ours=float(lb), grad_rel_err_max=worst,
                          norm_theirs=na, norm_ours=nb, local_q_rows=int(ours.layers[0].attn.q_proj.weight.shape[0]))
    with open(f"{a.out}.{a.mode}.{rank}.json", "w") as fh:
        json.dump(result, fh)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
