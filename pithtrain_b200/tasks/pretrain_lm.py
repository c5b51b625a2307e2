"""Pre-train a language model: ``launch(cfg)`` sets up the runtime and runs ``train_step`` until
``max_steps``.

One optimizer step = read this rank's slice of the global batch (pipeline rank 0 only), run all
micro-batches through ``DualPipeV.step``, normalise gradients by the token count, reduce them over
the shard groups, clip by the global L2 norm, step the owner-sharded optimizers, all-gather the
updated parameters, log one line. The line format, the token-weighted loss normalisation and the
batch layout across dp/ep/cp ranks follow pithtrain/tasks/pretrain_lm.py:56-122,327-493 of the
reference; step time is additionally measured on the device with CUDA events and an MFU is logged.
"""

from __future__ import annotations

import gc
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn
from torch.distributed.elastic.multiprocessing.errors import record

from ..config import SlottedDefault
from ..contexts import distributed, logging, training
from ..modules.distributed import DistributedCfg, setup_distributed
from ..modules.load_balance import MoELoadBalanceLossTracker
from ..modules.logging import LoggingCfg, activate_wandb, setup_logging
from ..modules.training import TrainingCfg, setup_training
from ..ops.cross_entropy import cross_entropy


@dataclass(init=False, slots=True)
class PretrainLMCfg(SlottedDefault):
    distributed: DistributedCfg = field(default_factory=DistributedCfg)
    training: TrainingCfg = field(default_factory=TrainingCfg)
    logging: LoggingCfg = field(default_factory=LoggingCfg)


# ------------------------------------------------------------------------------------------------
# data
# ------------------------------------------------------------------------------------------------
_PINNED: dict = {}


def _host_buffers(shape) -> Tuple[torch.Tensor, torch.Tensor]:
    key = tuple(shape)
    if key not in _PINNED:
        pin = torch.cuda.is_available()
        _PINNED[key] = (torch.empty(shape, dtype=torch.long, pin_memory=pin),
                        torch.empty(shape, dtype=torch.long, pin_memory=pin))
    return _PINNED[key]


def get_global_batch(cfg: PretrainLMCfg, device) -> Tuple[Optional[torch.Tensor], Optional[torch.Tensor]]:
    """This rank's rows of the global batch (tokens, next-token labels); ``None`` off pipeline rank 0.

    Rows are interleaved over (dp, ep) ranks per micro-batch. Under context parallelism each rank
    reads its two zigzag blocks ``r`` and ``2cp-1-r`` of every sequence.
    """
    if distributed.pp_rank != 0:
        return None, None
    t = cfg.training
    d = distributed
    mbs, gbs, S = t.micro_batch_size, t.global_batch_size, t.sequence_length
    eff = mbs * d.dp_size * d.ep_size
    local_bs = gbs // (d.dp_size * d.ep_size)
    start0 = training.step * gbs + (d.dp_rank * d.ep_size + d.ep_rank) * mbs
    block = S // (2 * d.cp_size)
    front, back = d.cp_rank * block, (2 * d.cp_size - d.cp_rank - 1) * block
    tokens, labels = _host_buffers((local_bs, 2 * block))
    ds = training.dataset
    for k in range(local_bs):
        acc, off = divmod(k, mbs)
        index = start0 + acc * eff + off
        if d.cp_size == 1:
            ta, la = ds.get_chunk(index, 0, S)
            tokens[k], labels[k] = ta, la
        else:
            ta, la = ds.get_chunk(index, front, block)
            tb, lb = ds.get_chunk(index, back, block)
            tokens[k, :block], tokens[k, block:] = ta, tb
            labels[k, :block], labels[k, block:] = la, lb
    return tokens.to(device, non_blocking=True), labels.to(device, non_blocking=True)


def criterion(output: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
    """Summed (not mean) cross-entropy of one micro-batch; the step divides by the token count."""
    return cross_entropy(output.view(-1, output.size(-1)), target.reshape(-1), ignore_index=-100, reduction="sum")


# ------------------------------------------------------------------------------------------------
# gradient post-processing
# ------------------------------------------------------------------------------------------------
@torch.no_grad()
def clip_grad_norm_(model: Optional[nn.Module] = None, max_norm: float = 1.0, norm_type: float = 2.0) -> torch.Tensor:
    """Clip by the global L2 norm over every distinct parameter of the job; returns the norm.

    With flat shard groups each parameter's reduced gradient lives on exactly one rank of its shard
    group, so the global sum of squares is the all-reduce of the owned regions' sums. The clip
    coefficient stays on the device (no host read-back).
    """
    assert norm_type == 2.0
    groups = training.shard_groups
    dev = distributed.device
    if groups:
        sq = torch.zeros((), dtype=torch.float32, device=dev)
        for g in groups:
            sq = sq + g.owned_grad_sumsq().to(dev)
    else:
        grads = [p.grad for p in model.parameters() if p.grad is not None]
        sq = torch.stack([g.float().pow(2).sum() for g in grads]).sum() if grads else torch.zeros((), device=dev)
    if dist.is_initialized() and distributed.world_size > 1:
        dist.all_reduce(sq)
    total = sq.sqrt().clamp(min=1e-6)
    coef = (max_norm / total).clamp(max=1.0)
    if groups:
        for g in groups:
            g.apply_clip(coef)
    else:
        for p in model.parameters():
            if p.grad is not None:
                p.grad.mul_(coef.to(p.grad.dtype))
    return total


# Dense bf16 tensor-core peak of one B200 (the vendor's 4.5 PFLOP/s figure is with 2:4 sparsity). The step line's
# utilisation is quoted against this nominal number; measured sustained cuBLAS throughput on a 1 kW part is ~0.6 of it.
NOMINAL_BF16_FLOPS = 2.25e15


def model_flops_per_token(config, seq_len: int) -> float:
    """Training FLOPs per token: 6 x active matmul parameters (lm_head included, embedding lookup
    excluded) + causal attention 3 x 2*S*Hq*D per layer."""
    from ..utils.model_stats import active_matmul_params, attention_dims

    p = active_matmul_params(config)
    hq, d_qk, d_v = attention_dims(config)
    attn = 3.0 * (seq_len * hq * (d_qk + d_v)) * config.num_hidden_layers
    return 6.0 * p + attn


# ------------------------------------------------------------------------------------------------
# step
# ------------------------------------------------------------------------------------------------
def forward_backward_update(cfg: PretrainLMCfg, tokens: Optional[torch.Tensor], labels: Optional[torch.Tensor]):
    """Device-side part of a step: all micro-batches through the pipeline, gradient normalisation,
    reduction, clipping, optimizer and scheduler steps, parameter all-gather. Nothing is read back to
    the host. Returns ``(loss, gradient_norm)`` as device tensors (``loss`` is ``None`` off pp rank 0).
    """
    t, d = cfg.training, distributed
    model, optimizers, schedulers = training.model, training.optimizers, training.schedulers
    model.train()
    for g in training.shard_groups:
        g.ensure_params()  # no-op unless DistributedCfg.reshard_params released them after the previous step
    assert t.global_batch_size % (t.micro_batch_size * d.dp_size * d.ep_size) == 0
    accumulate_steps = t.global_batch_size // (t.micro_batch_size * d.dp_size * d.ep_size)

    loss, _ = model.step(tokens, num_chunks=accumulate_steps, criterion=criterion, labels=labels, return_outputs=False)

    num_tokens = torch.ones((), device=d.device)
    if d.pp_rank == 0:
        num_tokens.fill_((labels != -100).sum().clamp_min(1))
    if d.pp_size > 1:
        dist.broadcast(num_tokens, src=dist.get_global_rank(d.pp_group, 0), group=d.pp_group)
    if loss is not None:
        loss = loss.sum() / num_tokens
        # mean over every rank that saw different tokens (the reference averages over cp only and logs
        # the first data-parallel shard's loss, pithtrain/tasks/pretrain_lm.py:390; the global mean makes
        # loss curves comparable across meshes)
        width = d.dp_size * d.cp_size * d.ep_size
        if width > 1:
            dist.all_reduce(loss, group=d.dp_cp_ep_group)
            loss /= width

    scale = 1.0 / num_tokens
    if training.shard_groups:
        for g in training.shard_groups:
            g.fold_autograd_grads()
            g.scale_grads(scale)
            g.reduce_grads()
            g.release_params()  # reshard_params: only the owned parameters stay through the optimizer step
    else:
        for p in model.parameters():
            if p.grad is not None:
                p.grad.mul_(scale)
    gradient_norm = clip_grad_norm_(model, max_norm=t.max_grad_norm)

    for optimizer, scheduler in zip(optimizers, schedulers):
        optimizer.step()
        optimizer.zero_grad(set_to_none=True)
        scheduler.step()
    for g in training.shard_groups:
        g.gather_params()
    for g in training.shard_groups:
        g.wait_params()
        g.zero_grad()
    MoELoadBalanceLossTracker.reset()
    return loss, gradient_norm


def read_kernel_status() -> int:
    """The device status word (4-byte device-to-host copy, cleared on read): non-zero when a bounded in-kernel wait ran
    out or a receive buffer overflowed during the step. 0 without the native library."""
    from .. import _native

    return _native.fetch_status() if _native.available() else 0


def raise_on_kernel_status(worst: int, own: int) -> None:
    """Raise on every rank when any rank's kernels reported a problem in this step: a transport whose wait timed out
    skipped its reduction or consumed stale rows, so the step's result must not be kept (nor checkpointed)."""
    if worst > 0:
        from .. import _native

        name = _native.STATUS_NAMES.get(worst, f"status {worst}")
        mine = _native.STATUS_NAMES.get(own, "none") if own else "none"
        raise _native.KernelStatusError(
            f"step {training.step}: a kernel reported '{name}' on at least one rank (this rank: {mine}); "
            "the step's gradients are not trustworthy")


def train_step(cfg: PretrainLMCfg) -> dict:
    """One optimizer step. Returns the step's metrics (populated on every rank)."""
    t = cfg.training
    d = distributed
    use_cuda = d.device.type == "cuda"
    if t.nsys_start is not None and training.step == t.nsys_start and use_cuda:
        torch.cuda.cudart().cudaProfilerStart()
        torch.cuda.nvtx.range_push(
            f"rank={d.rank}; pp={d.pp_rank}/{d.pp_size} dp={d.dp_rank}/{d.dp_size} cp={d.cp_rank}/{d.cp_size} "
            f"ep={d.ep_rank}/{d.ep_size}; mbs={t.micro_batch_size} seq={t.sequence_length}")
    if t.memory_profile_start is not None and training.step == t.memory_profile_start and use_cuda:
        torch.cuda.memory._record_memory_history(max_entries=65536, stacks="python")

    t0 = time.time()
    ev0 = ev1 = None
    if use_cuda:
        torch.cuda.reset_peak_memory_stats()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()

    tokens, labels = get_global_batch(cfg, d.device)
    loss, gradient_norm = forward_backward_update(cfg, tokens, labels)
    schedulers = training.schedulers

    device_ms = None
    status = 0
    if use_cuda:
        ev1.record()
        torch.cuda.synchronize()
        device_ms = ev0.elapsed_time(ev1)
        status = read_kernel_status()
    dt = torch.tensor([time.time() - t0, (device_ms or 0.0) / 1e3, float(status)], device=d.device)
    if dist.is_initialized() and d.world_size > 1:
        dist.all_reduce(dt, op=dist.ReduceOp.MAX)
    elapsed, device_s, worst = dt.tolist()
    raise_on_kernel_status(int(worst), status)

    peak = torch.tensor(torch.cuda.max_memory_allocated() / 1024 ** 3 if use_cuda else 0.0, device=d.device)
    if dist.is_initialized() and d.world_size > 1:
        dist.all_reduce(peak, op=dist.ReduceOp.MAX)

    coef = t.moe_load_balance_coef
    lb_total, lb_count = MoELoadBalanceLossTracker.get_total_count_and_clear()
    lb_loss = 0.0
    if coef > 0:
        st = torch.tensor([lb_total, float(lb_count)], device=d.device)
        if dist.is_initialized() and d.world_size > 1:
            dist.all_reduce(st)
        lb_loss = (st[0] / st[1].clamp(min=1)).item() / coef

    metrics = {"step": training.step, "step_time": elapsed, "device_step_time": device_s,
               "gradient_norm": float(gradient_norm), "peak_gpu_memory": float(peak), "load_balance_loss": lb_loss,
               "tokens_per_second": t.global_batch_size * t.sequence_length / max(elapsed, 1e-9)}
    mfu = None
    if use_cuda:
        try:
            per_gpu = metrics["tokens_per_second"] / d.world_size
            mfu = per_gpu * model_flops_per_token(training.model_config, t.sequence_length) / NOMINAL_BF16_FLOPS
            metrics["mfu"] = mfu
        except Exception:  # a model whose config lacks the fields of the FLOP count: no figure rather than no step
            mfu = None
    if d.rank == 0:
        lr = schedulers[0].get_last_lr()[0] if schedulers else t.lr
        loss_v = float(loss) if loss is not None else float("nan")
        metrics.update(loss=loss_v, lr=lr)
        parts = ["step %08d/%08d" % (training.step + 1, t.max_steps), "step-time %.3f sec" % elapsed,
                 "cross-entropy-loss %.4f" % loss_v]
        if coef > 0:
            parts.append("load-balance-loss %.6f" % lb_loss)
        parts += ["learning-rate %.6e" % lr, "gradient-norm %.4f" % metrics["gradient_norm"],
                  "tokens-per-second %s" % format(metrics["tokens_per_second"], ",.0f"),
                  "peak-gpu-memory %.2f GB" % metrics["peak_gpu_memory"]]
        if device_ms is not None:
            parts.append("device-step-time %.3f sec" % device_s)
        if mfu is not None:
            parts.append("model-flops-utilization %.3f" % mfu)
        logging.stdout.info(" | ".join(parts))
        activate_wandb(cfg)
        if logging.wandb is not None:
            logging.wandb.log({"train/step": training.step, "train/cross-entropy-loss": loss_v,
                               "train/load-balance-loss": lb_loss, "train/learning-rate": lr,
                               "train/gradient-norm": metrics["gradient_norm"],
                               "infra/tokens-per-second": metrics["tokens_per_second"],
                               "infra/peak-gpu-memory": metrics["peak_gpu_memory"], "infra/step-time": elapsed})
    training.step += 1

    if t.nsys_stop is not None and training.step == t.nsys_stop and use_cuda:
        torch.cuda.nvtx.range_pop()
        torch.cuda.cudart().cudaProfilerStop()
    if t.memory_profile_stop is not None and training.step == t.memory_profile_stop and use_cuda:
        out = Path(t.memory_profile_output)
        out.mkdir(parents=True, exist_ok=True)
        torch.cuda.memory._dump_snapshot(str(out / ("snapshot-rank%05d.pickle" % d.rank)))
        torch.cuda.memory._record_memory_history(enabled=None)

    if t.save_interval is not None and t.save_location is not None and training.step % t.save_interval == 0:
        save_checkpoint(cfg)
    _collect_garbage()
    return metrics


_STEPS_RUN = 0


def _collect_garbage() -> None:
    """Per-step collection (the automatic collector is off while training, so that no pause lands inside a step).

    A full collection walks every tracked object of the process — a few hundred thousand, almost all of them modules,
    the model, optimizer state and caches that live until the end — and takes ≈ 0.1 s with the GPU idle behind the
    step's synchronize. After the second step of a process everything alive is moved to the permanent generation
    (``gc.freeze``): later collections only look at what a step created and take about a millisecond."""
    global _STEPS_RUN
    gc.collect()
    _STEPS_RUN += 1
    if _STEPS_RUN == 2:
        gc.freeze()


# ------------------------------------------------------------------------------------------------
# checkpoints (thin wrappers; the format lives in modules.checkpoint)
# ------------------------------------------------------------------------------------------------
class AppState:
    """The ``app`` entry of a checkpoint as one object with ``state_dict`` / ``load_state_dict`` (the protocol of
    ``torch.distributed.checkpoint.stateful.Stateful``), for callers that drive ``dcp.save`` / ``dcp.load`` themselves.

    ``state_dict`` returns canonical (mesh-independent) keys: ``model`` without the ``module.N.`` prefix and with one
    entry per global expert, ``optimizer`` keyed the same way, ``scheduler`` as a list; with ``model_only`` just the
    model (what a checkpoint converted from Hugging Face holds). ``load_state_dict`` maps canonical keys back onto
    whatever this rank owns and skips optimizer and scheduler entries that are absent. Same role as the reference's
    class of this name (pithtrain/tasks/pretrain_lm.py:156-220); ``save_checkpoint`` / ``load_checkpoint`` below use
    the functions of ``modules.checkpoint`` directly.
    """

    def __init__(self, model: nn.Module, optimizers=(), schedulers=(), model_only: bool = False) -> None:
        self.model, self.optimizers, self.schedulers, self.model_only = model, tuple(optimizers), tuple(schedulers), model_only

    def state_dict(self) -> dict:
        from ..modules import checkpoint as ckpt

        model_state = ckpt.to_canonical_model(dict(self.model.state_dict()), self.model)
        if self.model_only:
            return {"model": model_state}
        return {"model": model_state, "optimizer": ckpt.to_canonical_optim(self.optimizers, self.model),
                "scheduler": [s.state_dict() for s in self.schedulers]}

    def load_state_dict(self, state_dict: dict) -> None:
        from ..modules import checkpoint as ckpt

        local = ckpt.to_localized_model(state_dict["model"], self.model)
        with torch.no_grad():
            own = self.model.state_dict()
            for k, v in local.items():
                own[k].copy_(v)  # in place: parameters are views into flat buffers
        optim = state_dict.get("optimizer")
        if optim and self.optimizers:
            if torch.is_tensor(optim.get("param_groups")):
                optim = dict(optim, param_groups=ckpt._from_blob(optim["param_groups"]))
            ckpt.to_localized_optim(optim, self.model, self.optimizers)
        sched = state_dict.get("scheduler")
        if torch.is_tensor(sched):
            sched = ckpt._from_blob(sched)
        if sched:
            if isinstance(sched, dict):  # a checkpoint written with a single scheduler
                sched = [sched]
            for s, st in zip(self.schedulers, sched):
                s.load_state_dict(st)


def save_checkpoint(cfg: PretrainLMCfg) -> None:
    from ..modules import checkpoint as ckpt

    ckpt.save_training_checkpoint(cfg)


def load_checkpoint(cfg: PretrainLMCfg) -> None:
    from ..modules import checkpoint as ckpt

    ckpt.load_training_checkpoint(cfg)


def raise_if_dataset_insufficient(cfg: PretrainLMCfg) -> None:
    t = cfg.training
    need = t.max_steps * t.global_batch_size
    have = len(training.dataset)
    if have < need:
        msg = f"dataset has {have} sequences of length {t.sequence_length}, but {need} are needed for {t.max_steps} steps"
        if distributed.rank == 0:
            raise ValueError(msg)
        raise SystemExit(1)


@record
def launch(cfg: PretrainLMCfg) -> None:
    """Entry point of the task: set up logging, distributed runtime and training state, resume from the
    newest checkpoint if there is one, and train. ``@record`` hands an uncaught exception to torchrun's error file,
    so the launcher's summary names the failing rank and its traceback (pithtrain/tasks/pretrain_lm.py:496)."""
    setup_logging(cfg)
    setup_distributed(cfg)
    setup_training(cfg)
    load_checkpoint(cfg)
    raise_if_dataset_insufficient(cfg)
    gc.disable()
    try:
        while training.step < cfg.training.max_steps:
            train_step(cfg)
    finally:
        gc.enable()
