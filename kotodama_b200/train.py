"""Training driver: ``torchrun -m kotodama_b200.train --config X.yaml [--flag ...]``.

Same flag surface and loop semantics as the reference driver (``src/training/train.py:195-850``):
micro-step loop with loss/GA scaling, one host read of the loss per step, global-norm clip
before Muon then AdamW, WSD schedule, batch-size ramp, the canonical log line, JSONL/wandb
metrics, periodic / SIGTERM / final checkpoints with automatic resume, profiler window and
geometric monitoring on rank 0.  What differs: it also runs on CPU with gloo, the step is
carried out by the hand-scheduled executor (``kotodama_b200.engine``), gradient reduction and
Muon are owner-computes, and throughput is additionally timed on the device (max over ranks).

Schedule order: by default the learning rates for step ``s`` are set *before* the step runs;
``--reference_lr_order`` reproduces the reference, which applies them after the step (so a fresh
run executes step 0 at full base LR and step 1 at LR zero).
"""
from __future__ import annotations

import argparse
import logging
import math
import os
import time
from typing import Any, Optional

import torch
import torch.distributed as dist

from .ckpt.manager import AsyncCheckpointManager, CheckpointManager, SIGTERMHandler, clean_state_dict
from .config import grad_accum_for_step, model_config_from_args, parse_args
from .data.dataset import BatchIterator, RandomTokenDataset, TokenizedDataset
from .engine import TrainEngine
from .models.llama import KotodamaModel
from .monitor.logger import WandbLogger, format_step_line, scheduler_hook
from .optim.muon import HybridScheduler

logger = logging.getLogger("kotodama_b200.train")


def setup_distributed(device_kind: str, backend: str) -> tuple[int, int, int]:
    """Returns ``(rank, world_size, local_rank)``; a single process needs no launcher."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if device_kind == "cuda":
        torch.cuda.set_device(local)
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        lib = "gloo" if device_kind == "cpu" or backend == "gloo" else "nccl"
        dist.init_process_group(lib)
    return rank, world, local


def cleanup_distributed() -> None:
    if dist.is_available() and dist.is_initialized():
        dist.destroy_process_group()


def setup_logging(rank: int) -> None:
    """INFO on rank 0, WARNING elsewhere (``train.py:180-187``)."""
    level = logging.INFO if rank == 0 else logging.WARNING
    logging.basicConfig(level=level, format=f"[rank {rank}] %(asctime)s %(levelname)s %(name)s: %(message)s",
                        datefmt="%H:%M:%S")
    logging.getLogger("kotodama_b200").setLevel(level)


def per_layer_grad_norms(model: torch.nn.Module) -> dict[str, float]:
    """Attention vs MLP gradient norms for every fourth layer and the last (``train.py:908-939``)."""
    out: dict[str, float] = {}
    layers = getattr(model, "layers", None)
    if layers is None:
        return out
    for i, layer in enumerate(layers):
        if i % 4 != 0 and i != len(layers) - 1:
            continue
        a = [p.grad.float().norm() for n, p in layer.named_parameters() if p.grad is not None and "attn" in n]
        m = [p.grad.float().norm() for n, p in layer.named_parameters() if p.grad is not None and "ffn" in n]
        at = float(torch.stack(a).square().sum().sqrt()) if a else 0.0
        mt = float(torch.stack(m).square().sum().sqrt()) if m else 0.0
        out[f"grad/layer_{i}/attn"], out[f"grad/layer_{i}/mlp"] = at, mt
        if mt > 1e-10:
            out[f"grad/layer_{i}/attn_mlp_ratio"] = at / (mt + 1e-10)
    return out


def load_nca_weights(model: KotodamaModel, path: str, reinit_mlps: bool) -> None:
    """NCA -> language transition (``train.py:248-288``): non-strict load, fresh embeddings of the
    language vocabulary, optionally fresh MLPs."""
    state = torch.load(path, map_location="cpu", weights_only=False)
    sd = clean_state_dict(state.get("model", state))
    vocab = model.config.vocab_size
    own = model.state_dict()
    sd = {k: v for k, v in sd.items() if k in own and own[k].shape == v.shape}
    missing, unexpected = model.load_state_dict(sd, strict=False)
    logger.info("NCA weights loaded (%d tensors, %d missing)", len(sd), len(missing))
    model.reinit_embeddings(new_vocab_size=vocab)
    if reinit_mlps:
        model.reinit_mlps()


def train(args: argparse.Namespace) -> dict[str, Any]:
    device_kind = args.device if (args.device == "cpu" or torch.cuda.is_available()) else "cpu"
    rank, world, local = setup_distributed(device_kind, args.backend)
    setup_logging(rank)
    is_main = rank == 0
    device = torch.device(f"cuda:{local}") if device_kind == "cuda" else torch.device("cpu")
    dtype = torch.bfloat16 if (args.dtype == "bf16" and device_kind == "cuda") else torch.float32
    tp_size = max(1, args.tp_size)
    dp_size = world // tp_size
    if is_main:
        logger.info("World size: %d, device: %s, dtype: %s, TP=%d DP=%d", world, device, dtype, tp_size, dp_size)

    # -- model ------------------------------------------------------------------
    cfg = model_config_from_args(args)
    torch.manual_seed(args.seed)
    small = cfg.param_count() < 500_000_000 or args.resume_nca
    if small:
        model = KotodamaModel(cfg)
        if args.resume_nca:
            load_nca_weights(model, args.resume_nca, args.reinit_mlps)
    else:
        with torch.device("meta"):
            model = KotodamaModel(cfg)
    if is_main:
        n = sum(p.numel() for p in model.parameters())
        logger.info("Model: %s (%.1fM params, config estimate: %.1fM)", args.model_size, n / 1e6, cfg.param_count() / 1e6)
    for flag in ("use_liger", "compile"):
        if getattr(args, flag, False) and is_main:
            logger.info("--%s accepted for config compatibility: the native kernel path is always on", flag)

    # -- parallelism + executor ---------------------------------------------------
    from .parallel import make_comm
    if tp_size > 1:
        from .parallel.tp import TensorParallelComm, create_process_groups
        tp_group, dp_group = create_process_groups(world, tp_size)
        comm = None
        # fused all-gather -> GEMM / GEMM -> reduce-scatter kernels over NVLink peer memory: the default on
        # CUDA with sequence parallelism when the TP group is the whole job (the measured configuration);
        # `--backend native` asks for them with data-parallel replicas too, `--backend nccl` never uses them
        want_fused = (device_kind == "cuda" and args.sequence_parallel
                      and (args.backend == "native" or (args.backend == "auto" and tp_size == world)))
        if want_fused:
            try:
                from .parallel.tp_native import FusedTensorParallelComm
                comm = FusedTensorParallelComm(tp_group, dp_group)
            except Exception as e:
                if args.backend == "native":
                    raise
                logger.warning("fused tensor-parallel kernels unavailable (%s): library collectives", e)
        if comm is None:
            comm = TensorParallelComm(tp_group, dp_group, sequence_parallel=args.sequence_parallel)
        if is_main:
            logger.info("Tensor parallelism: tp=%d, %s", tp_size, type(comm).__name__)
    else:
        backend = args.backend
        if device_kind == "cpu" or backend in ("gloo", "nccl"):
            backend = "library"
        comm = make_comm("nccl" if backend == "library" else backend, world,
                         distributed_muon=not args.no_distributed_muon)
        if is_main:
            logger.info("Data parallelism: %s", type(comm).__name__)
    kw = dict(device=device, dtype=dtype, comm=comm, muon_lr=args.muon_lr, muon_momentum=args.muon_momentum,
              muon_weight_decay=args.muon_weight_decay, muon_ns_iterations=args.muon_ns_iterations,
              muon_ns_coefficients=args.muon_ns_coefficients, adamw_lr=args.adamw_lr,
              adamw_betas=(args.adamw_beta1, args.adamw_beta2), adamw_weight_decay=args.adamw_weight_decay,
              gradient_clip=args.gradient_clip, adamw_only=args.adamw_only, fp8=args.fp8, fp8_recipe=args.fp8_recipe)
    engine = TrainEngine(model, **kw) if small else TrainEngine.from_meta(model, cfg, seed=args.seed, **kw)
    muon_opt, adamw_opt = engine.muon_opt, engine.adamw_opt

    # -- geometry --------------------------------------------------------------
    seq_len, mb = args.sequence_length, args.micro_batch_size
    tokens_per_global_micro = mb * seq_len * dp_size
    grad_accum = max(1, args.global_batch_tokens // tokens_per_global_micro)
    if args.total_steps is not None:
        total_steps = args.total_steps
        total_tokens = total_steps * grad_accum * tokens_per_global_micro
    else:
        total_tokens = args.total_tokens
        total_steps = total_tokens // (grad_accum * tokens_per_global_micro)
    if is_main:
        logger.info("Training: %d steps, %d grad_accum, %d tokens/step (%.2fM), %.1fB total tokens", total_steps,
                    grad_accum, grad_accum * tokens_per_global_micro, grad_accum * tokens_per_global_micro / 1e6,
                    total_tokens / 1e9)
    scheduler = HybridScheduler(muon_opt, adamw_opt, warmup_steps=args.warmup_steps, total_steps=total_steps,
                                decay_start_pct=args.decay_start_pct, decay_type=args.decay_type)

    # -- data ------------------------------------------------------------------
    dp_rank = comm.dp_rank if hasattr(comm, "dp_rank") else rank
    if args.random_data:
        dataset = RandomTokenDataset(cfg.vocab_size, seq_len, seed=args.seed, rank=dp_rank, fixed=args.fixed_batch)
    else:
        if not args.data_path:
            raise ValueError("--data_path required when not using --random_data")
        dataset = TokenizedDataset(args.data_path, seq_len, rank=dp_rank, world_size=dp_size, seed=args.seed)
    batches = BatchIterator(dataset, mb, pin=device_kind == "cuda")

    # -- checkpoints / resume ----------------------------------------------------
    if args.async_checkpoint:
        ckpt = AsyncCheckpointManager(args.checkpoint_dir, rank=rank, keep_last_n=args.keep_checkpoints,
                                      shm_dir=args.checkpoint_shm_dir, compress=args.checkpoint_compress)
    else:
        ckpt = CheckpointManager(args.checkpoint_dir, rank=rank, keep_last_n=args.keep_checkpoints)
    start_step, tokens_consumed = 0, 0
    state = ckpt.load_latest(model, muon_opt, adamw_opt, device)
    if state is not None:
        start_step = state["step"] + 1
        tokens_consumed = state.get("tokens_consumed", 0)
        if "data" in state and hasattr(dataset, "load_state_dict"):
            dataset.load_state_dict(state["data"])
            batches = BatchIterator(dataset, mb, pin=device_kind == "cuda")
        engine.after_load()
        if args.reference_lr_order:
            scheduler.step(start_step)
    sigterm = SIGTERMHandler()

    # -- monitoring ----------------------------------------------------------------
    monitor = None
    if is_main and args.geo_monitor:
        from .monitor.geometric import GeometricMonitor, MonitorConfig
        monitor = GeometricMonitor(model, MonitorConfig(tier1_every=args.geo_monitor_tier1_every,
                                                        tier2_every=args.geo_monitor_tier2_every))
        # a dataset instance of its own: drawing the probe batch must not advance the training stream
        probe_ds = (RandomTokenDataset(cfg.vocab_size, seq_len, seed=args.seed + 1, rank=0) if args.random_data
                    else TokenizedDataset(args.data_path, seq_len, rank=0, world_size=1, seed=args.seed + 1))
        it = iter(probe_ds)
        monitor.set_probe_batch(torch.stack([next(it) for _ in range(min(monitor.config.tier1_probe_size, 64))]))
    wb: Optional[WandbLogger] = None
    if is_main and args.wandb:
        wb = WandbLogger(project=args.wandb_project, run_name=args.wandb_run_name, log_dir=args.checkpoint_dir,
                         tags=["pretraining", args.model_size],
                         config={"model_size": args.model_size, "total_tokens": total_tokens,
                                 "total_steps": total_steps, "grad_accum": grad_accum,
                                 "tokens_per_step": grad_accum * tokens_per_global_micro, "micro_batch_size": mb,
                                 "sequence_length": seq_len, "world_size": world, "muon_lr": args.muon_lr,
                                 "muon_ns_coefficients": args.muon_ns_coefficients or "original",
                                 "adamw_lr": args.adamw_lr, "warmup_steps": args.warmup_steps,
                                 "precision": "bf16" if dtype == torch.bfloat16 else "fp32",
                                 "parallelism": f"tp{tp_size}" if tp_size > 1 else "ddp", "tp_size": tp_size,
                                 "dp_size": dp_size})
    from .monitor.profiler import StepProfiler
    from .monitor.watchdog import StepWatchdog
    profiler = StepProfiler(args, enabled=is_main and args.profile)
    watchdog = StepWatchdog(args.watchdog_s, rank=rank)
    health = None
    if world > 1:
        from .parallel.health import PeerHealth
        health = PeerHealth()

    # -- loop --------------------------------------------------------------------
    if is_main:
        logger.info("Starting training from step %d", start_step)
    t0 = time.time()
    log_loss = log_z = 0.0
    log_steps = 0
    dev_ms_acc = 0.0
    history: list[float] = []
    last_step = start_step - 1
    for step in range(start_step, total_steps):
        if health is not None:
            # a peer that left between steps is noticed here, on the host, before this rank enters
            # kernels and collectives that could no longer complete
            health.raise_if_peer_left()
            health.beat(step)
        profiler.step_begin(step)
        if not args.reference_lr_order:
            scheduler.step(step)
        ga = grad_accum_for_step(step, total_steps, grad_accum, args.batch_ramp_initial, args.batch_ramp_pct)
        watchdog.phase(step, "data")
        micro = [next(batches) for _ in range(ga)]
        if device_kind == "cuda":
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
        watchdog.phase(step, "train_step")
        res = engine.train_step(micro, keep_grads=wb is not None and step % 50 == 0)
        if device_kind == "cuda":
            ev1.record()
        watchdog.phase(step, "loss_readback")
        # the one device->host sync of the step: loss, z-loss and gradient norm in one read
        step_loss, step_z, grad_norm = torch.stack([res["loss"].reshape(()).float(), res["z_loss"].reshape(()).float(),
                                                    res["grad_norm"].reshape(()).float()]).tolist()
        if device_kind == "cuda":
            dev_ms_acc += ev0.elapsed_time(ev1)
        finite = math.isfinite(step_loss) and math.isfinite(grad_norm)
        if not finite:
            logger.error("Non-finite loss/grad-norm at step %d (loss=%s grad_norm=%s)", step, step_loss, grad_norm)
        watchdog.phase(step, "bookkeeping")
        if wb is not None and step % 50 == 0:
            wb.log_custom(step, per_layer_grad_norms(model))
        if args.reference_lr_order:
            scheduler.step(step)
        cur_tokens = ga * tokens_per_global_micro
        tokens_consumed += cur_tokens
        history.append(step_loss)
        log_loss += step_loss
        log_z += step_z
        log_steps += 1
        last_step = step
        if is_main and (step % args.log_every == 0 or step == total_steps - 1):
            elapsed = time.time() - t0
            lrs = scheduler.get_last_lr()
            tok_s = log_steps * cur_tokens / max(elapsed, 1e-6)
            it_s = log_steps / max(elapsed, 1e-6)
            mem = torch.cuda.max_memory_allocated(device) / 1e9 if device_kind == "cuda" else 0.0
            logger.info(format_step_line(step, total_steps, log_loss / log_steps, log_z / log_steps, grad_norm,
                                         lrs["muon_lr"], lrs["adamw_lr"], tok_s, it_s, tokens_consumed, mem))
            if device_kind == "cuda" and dev_ms_acc > 0:
                logger.info("  device-timed: %.1f ms/step, %.0f tok/s", dev_ms_acc / log_steps,
                            log_steps * cur_tokens / (dev_ms_acc / 1e3))
            if wb is not None:
                wb.log_step(step=step, loss=log_loss / log_steps, z_loss=log_z / log_steps, grad_norm=grad_norm,
                            muon_lr=lrs["muon_lr"], adamw_lr=lrs["adamw_lr"], tokens_per_sec=tok_s,
                            iters_per_sec=it_s, tokens_consumed=tokens_consumed, gpu_mem_gb=mem,
                            step_time_s=elapsed / log_steps)
            scheduler_hook(step, **{"train/loss": log_loss / log_steps, "train/grad_norm": grad_norm,
                                    "train/perplexity": math.exp(min(log_loss / log_steps, 20)),
                                    "perf/tokens_per_sec": tok_s})
            log_loss = log_z = 0.0
            log_steps = 0
            dev_ms_acc = 0.0
            t0 = time.time()
        if monitor is not None:
            for tier, every in ((monitor.tier1, args.geo_monitor_tier1_every), (monitor.tier2, args.geo_monitor_tier2_every)):
                if every > 0 and step % every == 0:
                    geo = tier(step)
                    if geo and wb is not None:
                        wb.log_geo(step, geo)
        if wb is not None:
            wb.commit(step)
        profiler.step_end(step)
        data_state = dataset.state_dict() if hasattr(dataset, "state_dict") else None
        want_save = step > 0 and args.save_every > 0 and step % args.save_every == 0
        # Health of the step, agreed by all ranks in the one host collective the loop has anyway.  The
        # bounded-wait status word (a kernel gave up on a peer flag or a copy and returned with partial
        # output) is read at every log interval and before anything is written to a checkpoint.
        fault = ""
        if want_save or sigterm.received or step % args.log_every == 0 or step == total_steps - 1:
            try:
                engine.check()
            except Exception as e:                                 # noqa: BLE001 - reported on every rank below
                fault = f"{type(e).__name__}: {e}"
        if args.halt_on_nonfinite and not finite:
            fault = fault or f"non-finite loss/grad-norm at step {step}"
        watchdog.phase(step, "health_allreduce")
        code = comm.all_reduce_max(2.0 if fault else (1.0 if sigterm.received else 0.0))
        if code > 1.5:
            ckpt.shutdown()
            watchdog.stop()
            raise RuntimeError(f"rank {rank}: training stopped at step {step}: " + (fault or "a peer rank reported a fault"))
        if want_save:
            watchdog.phase(step, "checkpoint")
            ckpt.save(step, model, muon_opt, adamw_opt, scheduler, tokens_consumed, data_state)
        if code > 0.5:
            if is_main:
                logger.info("SIGTERM exit: saving checkpoint at step %d", step)
            watchdog.phase(step, "checkpoint")
            ckpt.save_blocking(step, model, muon_opt, adamw_opt, scheduler, tokens_consumed, data_state)
            break
    else:
        if is_main:
            logger.info("Training complete: %d steps, %.2fB tokens", total_steps, tokens_consumed / 1e9)
        if total_steps > start_step:
            data_state = dataset.state_dict() if hasattr(dataset, "state_dict") else None
            ckpt.save(total_steps - 1, model, muon_opt, adamw_opt, scheduler, tokens_consumed, data_state)
    watchdog.stop()
    ckpt.shutdown()
    if wb is not None:
        wb.finish()
    sigterm.restore()
    engine.check()
    return {"losses": history, "last_step": last_step, "tokens_consumed": tokens_consumed, "engine": engine}


def main(argv: Optional[list[str]] = None) -> None:
    args = parse_args(argv)
    try:
        train(args)
    except Exception as e:
        logger.exception("Training failed")
        _announce_leave(f"{type(e).__name__}: {e}")
        raise
    finally:
        cleanup_distributed()


def _announce_leave(reason: str) -> None:
    """Tell the peers (through the rendezvous store) that this rank is on its way out."""
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        from .parallel.health import PeerHealth
        try:
            PeerHealth().announce_leave(reason)
        except Exception:                          # noqa: BLE001
            pass


if __name__ == "__main__":
    main()
