"""Reshardable checkpoints: canonical (on-disk) <-> localized (runtime) state dictionaries.

Canonical format (what is written with ``torch.distributed.checkpoint``):

* keys carry no ``module.<N>.`` pipeline-chunk prefix; layer ids are global;
* expert tensors are stored one per *global* expert:
  ``layers.3.mlp.experts.17.gate_proj.weight`` (``...experts.17.gate_up_proj`` for raw GPT-OSS
  parameters), whatever the expert-parallel degree was;
* values are plain tensors, so any (pp, ep, dp) layout can load any checkpoint.

Runtime format: ``module.0.layers.3.mlp.experts.gate_proj.weight`` with experts stacked per EP rank
``[experts_per_rank, ...]``. The on-disk tree is ``app.model.*``, ``app.optimizer.state.<fqn>.<key>``,
``app.optimizer.param_groups``, ``app.scheduler`` plus ``rng-rank-%05d.pt`` — the layout described in
pithtrain/modules/checkpoint.py:1-10 and pithtrain/tasks/pretrain_lm.py:251-324 of the reference
(whose own expert unstacking is keyed on a module attribute no model sets; here it is keyed on the
parameter name and the expert-parallel rank of the distributed context).

Because parameters are owner-sharded (whole parameters, not slices), every rank can write the
tensors it holds: replicated tensors are de-duplicated by DCP's save planner, optimizer state exists
only on owners and therefore has unique keys.
"""

from __future__ import annotations

import re
import time
from pathlib import Path
from typing import Any, Dict, Iterable, List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from ..contexts import distributed, logging, training

__all__ = ["to_canonical_model", "to_canonical_optim", "to_localized_model", "to_localized_optim",
           "save_training_checkpoint", "load_training_checkpoint", "strip_prefix", "canonical_expert_keys"]

MODULE_PREFIX_RE = re.compile(r"^module\.\d+\.")
INDEXED_EXPERT_RE = re.compile(r"(.*)\.experts\.(\d+)\.(.*)")


def strip_prefix(key: str) -> str:
    """Drop the ``module.<N>.`` DualPipeV prefix."""
    return MODULE_PREFIX_RE.sub("", key)


def is_stacked_expert_key(key: str) -> bool:
    return ".experts." in key and INDEXED_EXPERT_RE.match(key) is None


def canonical_expert_keys(key: str, n_local: int, ep_rank: int) -> List[str]:
    """Canonical names of the ``n_local`` experts stacked under runtime key ``key`` on ``ep_rank``."""
    head, tail = key.split(".experts.", 1)
    first = ep_rank * n_local
    return [f"{strip_prefix(head)}.experts.{first + i}.{tail}" for i in range(n_local)]


def _ep_rank() -> int:
    return distributed.ep_rank


# ------------------------------------------------------------------------------------------------
# model
# ------------------------------------------------------------------------------------------------
def to_canonical_model(model_state: Dict[str, torch.Tensor], model: Optional[nn.Module] = None,
                       ep_rank: Optional[int] = None) -> Dict[str, torch.Tensor]:
    """Runtime state dict -> canonical: strip prefixes, unstack experts into per-expert views."""
    r = _ep_rank() if ep_rank is None else ep_rank
    out: Dict[str, torch.Tensor] = {}
    for k, v in model_state.items():
        if is_stacked_expert_key(k):
            for name, t in zip(canonical_expert_keys(k, v.shape[0], r), v.unbind(0)):
                out[name] = t
        else:
            out[strip_prefix(k)] = v
    return out


def to_localized_model(canonical: Dict[str, torch.Tensor], model: nn.Module, ep_rank: Optional[int] = None
                       ) -> Dict[str, torch.Tensor]:
    """Canonical state dict -> runtime keys of ``model`` (restacking this rank's experts).

    Keys the model does not own are ignored; keys missing from ``canonical`` are skipped.
    """
    r = _ep_rank() if ep_rank is None else ep_rank
    out: Dict[str, torch.Tensor] = {}
    for k, p in model.state_dict().items():
        if is_stacked_expert_key(k):
            names = canonical_expert_keys(k, p.shape[0], r)
            if all(n in canonical for n in names):
                out[k] = torch.stack([canonical[n] for n in names])
        else:
            ck = strip_prefix(k)
            if ck in canonical:
                out[k] = canonical[ck]
    return out


# ------------------------------------------------------------------------------------------------
# optimizer
# ------------------------------------------------------------------------------------------------
def _param_names(model: nn.Module) -> Dict[int, str]:
    return {id(p): n for n, p in model.named_parameters()}


def _unstack_state(entry: Dict[str, Any], n: int, i: int) -> Dict[str, Any]:
    """State of expert ``i`` out of a stacked parameter's state (tensors whose dim 0 is ``n``)."""
    return {k: (v[i] if torch.is_tensor(v) and v.dim() >= 1 and v.shape[0] == n else v) for k, v in entry.items()}


def to_canonical_optim(optimizers: Iterable[torch.optim.Optimizer], model: nn.Module,
                       ep_rank: Optional[int] = None) -> Dict[str, Any]:
    """``{"state": {fqn: {key: tensor}}, "param_groups": [...]}`` over the state this rank holds."""
    r = _ep_rank() if ep_rank is None else ep_rank
    names = _param_names(model)
    state: Dict[str, Any] = {}
    groups: List[Dict[str, Any]] = []
    for oi, opt in enumerate(optimizers):
        for gi, g in enumerate(opt.param_groups):
            hyper = {k: v for k, v in g.items() if k != "params"}
            fqns: List[str] = []
            for p in g["params"]:
                name = names.get(id(p))
                if name is None:
                    continue
                st = opt.state.get(p, {})
                if is_stacked_expert_key(name):
                    keys = canonical_expert_keys(name, p.shape[0], r)
                    fqns.extend(keys)
                    if st:
                        for i, ck in enumerate(keys):
                            state[ck] = _unstack_state(st, p.shape[0], i)
                else:
                    ck = strip_prefix(name)
                    fqns.append(ck)
                    if st:
                        state[ck] = dict(st)
            groups.append({"optimizer": oi, "group": gi, "type": type(opt).__name__, **hyper, "params": fqns})
    return {"state": state, "param_groups": groups}


def to_localized_optim(optim_state: Dict[str, Any], model: nn.Module, optimizers: Iterable[torch.optim.Optimizer],
                       ep_rank: Optional[int] = None) -> None:
    """Load a canonical optimizer state into the live optimizers (in place).

    Group membership comes from the live optimizers; hyper-parameters come from the checkpoint entry
    with the same (optimizer, group) position. Only parameters this rank owns receive state.
    """
    r = _ep_rank() if ep_rank is None else ep_rank
    names = _param_names(model)
    state = optim_state.get("state", {})
    saved_groups = {(g.get("optimizer"), g.get("group")): g for g in optim_state.get("param_groups", [])}
    for oi, opt in enumerate(optimizers):
        for gi, g in enumerate(opt.param_groups):
            sg = saved_groups.get((oi, gi))
            if sg is not None:
                for k, v in sg.items():
                    if k not in ("params", "optimizer", "group", "type") and k in g:
                        g[k] = v
            for p in g["params"]:
                name = names.get(id(p))
                grp = getattr(p, "_shard_group", None)
                if name is None or (grp is not None and not grp.is_owned(p)):
                    continue
                if is_stacked_expert_key(name):
                    keys = canonical_expert_keys(name, p.shape[0], r)
                    if not all(k in state for k in keys):
                        continue
                    merged: Dict[str, Any] = {}
                    for field in state[keys[0]]:
                        vals = [state[k][field] for k in keys]
                        if torch.is_tensor(vals[0]) and vals[0].dim() >= 1 and vals[0].shape == p.shape[1:]:
                            merged[field] = torch.stack(vals)
                        else:
                            merged[field] = vals[0]
                    _assign_state(opt, p, merged)
                else:
                    ck = strip_prefix(name)
                    if ck in state:
                        _assign_state(opt, p, state[ck])


def _assign_state(opt: torch.optim.Optimizer, p: torch.Tensor, entry: Dict[str, Any]) -> None:
    cur = opt.state[p]
    for k, v in entry.items():
        if torch.is_tensor(v):
            old = cur.get(k)
            if torch.is_tensor(old) and old.shape == v.shape:
                old.copy_(v)
            else:
                dev = p.device if v.dim() > 0 else v.device
                cur[k] = v.to(dev).clone()
        else:
            cur[k] = v
    if hasattr(opt, "_unit_state"):
        opt._unit_state.pop(id(p), None)


# ------------------------------------------------------------------------------------------------
# save / load of a training run
# ------------------------------------------------------------------------------------------------
def checkpoint_dir(save_location, step: int) -> Path:
    return Path(save_location, "torch-dcp", "step-%08d" % step)


def is_complete(path: Path) -> bool:
    """A DCP directory is complete once its ``.metadata`` exists: the coordinator writes it after every rank has
    finished its shard files, so a save that was interrupted (job killed, disk full) leaves a directory without it."""
    return Path(path, ".metadata").is_file()


def latest_checkpoint(save_location) -> Optional[Path]:
    """Newest complete ``step-*`` directory; incomplete ones are skipped (and reported) so that a job killed in the
    middle of a save resumes from the checkpoint before it."""
    root = Path(save_location, "torch-dcp")
    steps = sorted((p for p in root.glob("step-*") if p.is_dir() and p.name.removeprefix("step-").isdigit()),
                   key=lambda p: int(p.name.removeprefix("step-")))
    for p in reversed(steps):
        if is_complete(p):
            return p
        if logging.stdout is not None:
            logging.stdout.info("Skip incomplete checkpoint (no .metadata): %s" % p)
    return None


def _rng_state() -> torch.Tensor:
    if distributed.device.type == "cuda":
        return torch.cuda.get_rng_state()
    return torch.get_rng_state()


def _set_rng_state(state: torch.Tensor) -> None:
    if distributed.device.type == "cuda":
        torch.cuda.set_rng_state(state)
    else:
        torch.set_rng_state(state)


def _elapsed_min_max(t0: float) -> Tuple[float, float]:
    dt = torch.tensor([time.monotonic() - t0], device=distributed.device)
    lo, hi = dt.clone(), dt.clone()
    if dist.is_initialized() and distributed.world_size > 1:
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    return float(lo), float(hi)


def _to_blob(obj: Any) -> torch.Tensor:
    """Non-tensor metadata travels as one uint8 tensor so its key is a single checkpoint entry."""
    import io
    import pickle

    buf = io.BytesIO()
    pickle.dump(obj, buf)
    return torch.frombuffer(bytearray(buf.getvalue()), dtype=torch.uint8).clone()


def _from_blob(t: torch.Tensor) -> Any:
    import pickle

    return pickle.loads(t.cpu().numpy().tobytes())


def _skeleton_from_keys(md, prefix: str):
    """Nested lists / dicts with ``None`` leaves for every stored key under ``prefix`` (numeric path parts are list
    indices); None when nothing is stored there."""
    paths = [k[len(prefix):].split(".") for k in md if k.startswith(prefix)]
    if not paths:
        return None

    def build(items):
        if any(len(p) == 0 for p in items):
            return None
        heads = {}
        for p in items:
            heads.setdefault(p[0], []).append(p[1:])
        if all(h.isdigit() for h in heads):
            return [build(heads[str(i)]) for i in range(len(heads))]
        return {h: build(rest) for h, rest in heads.items()}

    return build(paths)


def _sched_state(s) -> Dict[str, Any]:
    # LambdaLR keeps its (unpicklable) lambdas out of the state; keep the slot so load_state_dict works
    d = dict(s.state_dict())
    if "lr_lambdas" in d:
        d["lr_lambdas"] = [None] * len(d["lr_lambdas"])
    return d


def build_save_state(model: nn.Module, optimizers, schedulers) -> Dict[str, Any]:
    """The ``{"app": ...}`` tree for this rank (tensors moved to the CPU).

    Every model tensor is staged by exactly one of the ranks that hold a replica of it: dense tensors are replicated over
    dp x cp x ep, expert tensors over dp x cp, and only the first rank of each replica set copies its tensors to the host
    and hands them to the writer. (Without this every rank of a data-parallel job would stage a full replica, tens of GB
    per rank, for the planner to discard all but one.) Optimizer state exists on its owner only and needs no filter.
    """
    for g in training.shard_groups:
        g.ensure_params()  # parameters released by DistributedCfg.reshard_params are gathered again (a collective)
    first_replica = distributed.dp_rank == 0 and distributed.cp_rank == 0
    model_state = {k: v.detach().cpu() for k, v in to_canonical_model(dict(model.state_dict()), model).items()
                   if first_replica and (".experts." in k or distributed.ep_rank == 0)}
    optim = to_canonical_optim(optimizers, model)
    optim["state"] = {fqn: {k: (v.detach().cpu() if torch.is_tensor(v) else v) for k, v in st.items()}
                      for fqn, st in optim["state"].items()}
    # param_groups (a list of dicts) and the scheduler states (a list of dicts) hold no tensors: DCP stores each as one
    # pickled object under ``app.optimizer.param_groups`` / ``app.scheduler`` -- the layout of the reference's AppState
    # (pithtrain/tasks/pretrain_lm.py:171-191), so either framework reads the other's optimizer section.
    return {"app": {"model": model_state, "optimizer": optim, "scheduler": [_sched_state(s) for s in schedulers]}}


def save_training_checkpoint(cfg) -> Path:
    """Write ``<save_location>/torch-dcp/step-XXXXXXXX`` (collective over all ranks)."""
    import torch.distributed.checkpoint as dcp

    assert cfg.training.save_location is not None
    path = checkpoint_dir(cfg.training.save_location, training.step)
    logging.stdout.info("Save checkpoint: %s" % path)
    if distributed.device.type == "cuda":
        from ..parallel.symm_mem import check_all_guards

        check_all_guards()  # never persist a state that a stray peer store may have corrupted
    t0 = time.monotonic()
    state = build_save_state(training.model, training.optimizers, training.schedulers)
    dcp.save(state, checkpoint_id=str(path))
    torch.save(_rng_state(), Path(path, "rng-rank-%05d.pt" % distributed.rank))
    lo, hi = _elapsed_min_max(t0)
    logging.stdout.info("Save checkpoint: Elapsed min=%.1fs, max=%.1fs" % (lo, hi))
    return path


def load_into(path: Path, model: nn.Module, optimizers=(), schedulers=(), strict: bool = True) -> bool:
    """Load checkpoint ``path`` into live objects; returns True when optimizer state was present.

    ``strict`` (default): every parameter and persistent buffer of the live model must be in the checkpoint, as with
    the reference's ``dcp.load`` through its ``AppState`` (pithtrain/tasks/pretrain_lm.py:308-313); a checkpoint of a
    different architecture, expert count or depth raises ``KeyError`` instead of leaving the missing tensors at their
    random initialisation. A full checkpoint that lacks optimizer state for a parameter this rank owns is reported
    with a warning. ``strict=False`` loads what is there."""
    import torch.distributed.checkpoint as dcp
    from torch.distributed.checkpoint import FileSystemReader

    md = FileSystemReader(str(path)).read_metadata().state_dict_metadata
    model_only = all(k.startswith("app.model.") for k in md)
    # model: load in place into (views of) the live parameters; tolerate missing keys
    targets = to_canonical_model(dict(model.state_dict()), model)
    want_model = {k: v for k, v in targets.items() if ("app.model." + k) in md}
    missing = sorted(k for k in targets if ("app.model." + k) not in md)
    if missing and strict:
        raise KeyError(f"checkpoint {path} lacks {len(missing)} of the model's {len(targets)} tensors "
                       f"(first: {missing[:5]}); pass strict=False to load the rest")
    request: Dict[str, Any] = {"app": {"model": want_model}}
    optim_req: Dict[str, Dict[str, Any]] = {}
    if not model_only and optimizers:
        names = _param_names(model)
        prefix = "app.optimizer.state."
        no_state: List[str] = []
        by_fqn: Dict[str, List[str]] = {}
        for k in md:
            if k.startswith(prefix):
                fqn, field = k[len(prefix):].rsplit(".", 1)
                by_fqn.setdefault(fqn, []).append(field)
        for opt in optimizers:
            for g in opt.param_groups:
                for p in g["params"]:
                    name = names.get(id(p))
                    grp = getattr(p, "_shard_group", None)
                    if name is None or (grp is not None and not grp.is_owned(p)):
                        continue
                    keys = (canonical_expert_keys(name, p.shape[0], _ep_rank()) if is_stacked_expert_key(name)
                            else [strip_prefix(name)])
                    for ck in keys:
                        if ck not in by_fqn:
                            no_state.append(ck)
                        for field in by_fqn.get(ck, []):
                            m = md[prefix + ck + "." + field]
                            if hasattr(m, "size"):
                                optim_req.setdefault(ck, {})[field] = torch.empty(tuple(m.size), dtype=m.properties.dtype)
                            else:
                                optim_req.setdefault(ck, {})[field] = None
        request["app"]["optimizer"] = {"state": optim_req}
        if no_state and by_fqn:
            logging.stdout.warning("Load checkpoint: no optimizer state for %d owned parameters (first: %s); "
                                   "they restart from empty state" % (len(no_state), no_state[:3]), rank=None)
        for key, holder, name in (("app.optimizer.param_groups", request["app"]["optimizer"], "param_groups"),
                                  ("app.scheduler", request["app"], "scheduler")):
            if key in md and hasattr(md[key], "size"):
                # written by an earlier version of this package: one uint8 tensor holding the pickled object
                holder[name] = torch.empty(tuple(md[key].size), dtype=torch.uint8)
            else:
                # DCP flattens lists of dicts field by field (``app.scheduler.0.last_epoch`` ...): rebuild the nesting
                # from the stored keys with placeholders that the load fills in
                skel = _skeleton_from_keys(md, key + ".")
                if skel is not None:
                    holder[name] = skel
    dcp.load(request, checkpoint_id=str(path))
    if not model_only and optimizers:
        opt_req = request["app"]["optimizer"]
        if torch.is_tensor(opt_req.get("param_groups")):
            opt_req["param_groups"] = _from_blob(opt_req["param_groups"])
        to_localized_optim(opt_req, model, optimizers)
        sched = request["app"].get("scheduler")
        if torch.is_tensor(sched):
            sched = _from_blob(sched)
        if sched:
            if isinstance(sched, dict):
                sched = [sched]
            for s, st in zip(schedulers, sched):
                s.load_state_dict(st)
    return not model_only


def load_training_checkpoint(cfg) -> Optional[Path]:
    """Resume from the newest ``step-*`` directory under ``save_location`` (no-op when there is none)."""
    out = logging.stdout
    if cfg.training.save_location is None:
        out.info("No save_location set; training from scratch.")
        return None
    path = latest_checkpoint(cfg.training.save_location)
    if path is None:
        out.info("No checkpoint found; training from scratch.")
        return None
    out.info("Load checkpoint: %s" % path)
    t0 = time.monotonic()
    try:
        load_into(path, training.model, training.optimizers, training.schedulers)
    except Exception as e:
        # a damaged shard file may already have overwritten part of the live state: never continue from here
        raise RuntimeError(f"checkpoint {path} could not be read ({type(e).__name__}: {e}); move it away to resume "
                           f"from an older one") from e
    rng = Path(path, "rng-rank-%05d.pt" % distributed.rank)
    if rng.exists():
        _set_rng_state(torch.load(rng, weights_only=True))
    training.step = int(path.name.removeprefix("step-"))
    lo, hi = _elapsed_min_max(t0)
    out.info("Load checkpoint: Elapsed min=%.1fs, max=%.1fs" % (lo, hi))
    return path
