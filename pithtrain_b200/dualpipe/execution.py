"""Five-stage layer executor with explicit autograd segments.

A decoder layer runs as five stages — (1) attention + router, (2) expert dispatch, (3) expert MLP,
(4) combine, (5) aggregate + residual — so the scheduler can interleave the forward of one
micro-batch with the backward of another and hide each exchange behind the other's compute
(stage layout of pithtrain/dualpipe/execution.py:75-406 in the reference).

Design: every stage is a :class:`Segment` — a small autograd graph whose inputs are detached leaf
tensors and whose outputs are kept until the stage's backward. Backward of a stage is
``torch.autograd.backward(outputs, grads)`` followed by reading ``.grad`` of its inputs; there is
no graph surgery and no private autograd-engine API. A layer's bookkeeping is a
:class:`LayerRecord` of five segments, a micro-batch's a :class:`ChunkRecord`.

Stages 2 and 4 are delegated to the expert-parallel exchange object
(:mod:`pithtrain_b200.parallel.ep`); with ``ep_size == 1`` they vanish and stage 3 consumes stage
1's outputs directly. NVTX range names follow ``layerNN.stageK_{f,b,w}`` so timeline tooling keyed
on those names keeps working.
"""

from __future__ import annotations

from contextlib import contextmanager
from dataclasses import dataclass, field
from typing import Any, List, Optional, Sequence, Tuple

import torch

from ..contexts import distributed
from .utils import WeightGradStore, run_backward


# ------------------------------------------------------------------------------------------------
# NVTX (no-op without CUDA)
# ------------------------------------------------------------------------------------------------
# Set by the step-profile capture tool: ranges then also become profiler annotations, so that a trace can attribute
# kernels to pipeline stages (NVTX ranges themselves are only visible to Nsight Systems).
RECORD_RANGES = False


@contextmanager
def nvtx_range(name: str):
    if RECORD_RANGES:
        with torch.profiler.record_function(name):
            yield
    elif torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        yield


# ------------------------------------------------------------------------------------------------
# Segments and records
# ------------------------------------------------------------------------------------------------
def _leaf(t: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    """Detach into a fresh leaf that records gradients (floating tensors only)."""
    if t is None:
        return None
    d = t.detach()
    if d.is_floating_point():
        d.requires_grad_(True)
    return d


class Segment:
    """One autograd sub-graph: leaf ``inputs`` -> ``outputs``."""

    __slots__ = ("inputs", "outputs")

    def __init__(self) -> None:
        self.inputs: Tuple[Optional[torch.Tensor], ...] = ()
        self.outputs: Tuple[Optional[torch.Tensor], ...] = ()

    def begin(self, *tensors: Optional[torch.Tensor]) -> Tuple[Optional[torch.Tensor], ...]:
        self.inputs = tuple(_leaf(t) for t in tensors)
        return self.inputs

    def end(self, *outputs: Optional[torch.Tensor]) -> Tuple[Optional[torch.Tensor], ...]:
        self.outputs = tuple(outputs)
        return self.outputs

    def backward(self, grads: Sequence[Optional[torch.Tensor]]) -> Tuple[Optional[torch.Tensor], ...]:
        outs, gs = [], []
        for o, g in zip(self.outputs, grads):
            if o is None or not o.requires_grad or g is None:
                continue
            outs.append(o)
            gs.append(g if g.dtype == o.dtype else g.to(o.dtype))
        run_backward(outs, gs)
        in_grads = tuple(None if i is None else i.grad for i in self.inputs)
        self.clear()
        return in_grads

    def clear(self) -> None:
        self.inputs = ()
        self.outputs = ()

    @property
    def live(self) -> bool:
        return bool(self.outputs)


class LayerRecord:
    __slots__ = ("s1", "s2", "s3", "s4", "s5", "routing", "is_moe", "merged_prev")

    def __init__(self) -> None:
        self.s1, self.s2, self.s3, self.s4, self.s5 = Segment(), Segment(), Segment(), Segment(), Segment()
        self.routing: Any = None
        self.is_moe = False
        self.merged_prev = False  # stage 1 of this layer shares a segment with stage 5 of the previous one

    def clear(self) -> None:
        for s in (self.s1, self.s2, self.s3, self.s4, self.s5):
            s.clear()
        self.routing = None


class ChunkRecord:
    """Bookkeeping of one micro-batch through one model chunk."""

    def __init__(self, num_layers: int) -> None:
        self.prolog = Segment()
        self.epilog = Segment()
        self.layers: List[LayerRecord] = [LayerRecord() for _ in range(num_layers)]
        self.rotary: Any = None
        self.cu_seqlens: Any = None

    def clear(self) -> None:
        self.prolog.clear()
        self.epilog.clear()
        for layer in self.layers:
            layer.clear()
        self.rotary = None
        self.cu_seqlens = None


@dataclass
class ExecutionCtx:
    """Streams and events shared by the stage functions of one overlapped region."""

    comp_stream: Any = None
    comm_stream: Any = None
    fwd_event: Any = None
    bwd_event: Any = None
    pending: List[Any] = field(default_factory=list)

    @staticmethod
    def make(comm_stream=None) -> "ExecutionCtx":
        ctx = ExecutionCtx()
        if torch.cuda.is_available() and distributed.device.type == "cuda":
            ctx.comp_stream = torch.cuda.current_stream()
            ctx.comm_stream = comm_stream
        return ctx

    def comm(self):
        """Context manager that runs the body on the communication stream, ordered after the
        compute stream's work so far. Returns an event the consumer must wait on."""
        return _CommRegion(self)


class _CommRegion:
    def __init__(self, ctx: ExecutionCtx) -> None:
        self.ctx = ctx
        self.event = None

    def __enter__(self):
        c = self.ctx
        if c.comm_stream is None:
            return self
        ev = torch.cuda.Event()
        ev.record(c.comp_stream)
        c.comm_stream.wait_event(ev)
        self._cm = torch.cuda.stream(c.comm_stream)
        self._cm.__enter__()
        return self

    def __exit__(self, *exc):
        c = self.ctx
        if c.comm_stream is None:
            return False
        self.event = torch.cuda.Event()
        self.event.record(c.comm_stream)
        self._cm.__exit__(*exc)
        return False

    def wait(self) -> None:
        if self.event is not None:
            self.ctx.comp_stream.wait_event(self.event)
            self.event = None

    def share(self, produced=(), consumed=()) -> None:
        """Tell the caching allocator about cross-stream use: ``produced`` tensors were allocated on the
        communication stream and will be read on the compute stream, ``consumed`` the other way."""
        c = self.ctx
        if c.comm_stream is None:
            return
        for t in produced:
            if t is not None and t.is_cuda:
                t.record_stream(c.comp_stream)
        for t in consumed:
            if t is not None and t.is_cuda:
                t.record_stream(c.comm_stream)


def _ep():
    from ..parallel import ep as _ep_mod

    return _ep_mod.current()


# ------------------------------------------------------------------------------------------------
# Stage functions
# ------------------------------------------------------------------------------------------------
def stage1_f(layer, rec: LayerRecord, hidden: torch.Tensor, rotary, cu_seqlens, extra_inputs: tuple = ()):
    """Attention + router. ``extra_inputs`` lets a merged stage-5 pass already-leafed tensors."""
    with nvtx_range("layer%02d.stage1_f" % layer.idx):
        if not rec.merged_prev:
            (hidden,) = rec.s1.begin(hidden)
        tokens, residual, routing = layer.forward_stage1(hidden, rotary, cu_seqlens)
        rec.routing = routing
        rec.is_moe = routing is not None
        w = routing.topk_weight if routing is not None else None
        rec.s1.end(tokens, residual, w)
    return tokens, residual, routing


def stage1_b(layer, rec: LayerRecord, grads: Tuple[Optional[torch.Tensor], ...]):
    with nvtx_range("layer%02d.stage1_b" % layer.idx):
        return rec.s1.backward(grads)


def stage2_f(ctx: ExecutionCtx, layer, rec: LayerRecord, tokens, routing):
    """Expert dispatch (no-op at ep_size == 1). Returns a region handle to wait on."""
    ep = _ep()
    if routing is None or ep is None:
        return None
    with nvtx_range("layer%02d.stage2_f" % layer.idx):
        x, w = rec.s2.begin(tokens, routing.topk_weight)
        region = ctx.comm()
        with region:
            recv_x, recv_w = ep.dispatch(x, w, routing.plan)
            rec.s2.end(recv_x, recv_w)
        region.share(produced=(recv_x, recv_w), consumed=(x, w))
    return region


def stage2_b(ctx: ExecutionCtx, layer, rec: LayerRecord, grads):
    with nvtx_range("layer%02d.stage2_b" % layer.idx):
        region = ctx.comm()
        with region:
            out = rec.s2.backward(grads)
        region.share(produced=out, consumed=grads)
    return out, region


def stage3_f(layer, rec: LayerRecord, routing, tokens, weights):
    with nvtx_range("layer%02d.stage3_f" % layer.idx):
        x, w = rec.s3.begin(tokens, weights)
        outs = layer.forward_stage3(x, w, routing)
        rec.s3.end(outs)
    return outs


def stage3_b(layer, rec: LayerRecord, grads, defer_wgrad: bool = False):
    with nvtx_range("layer%02d.stage3_b" % layer.idx):
        prev = WeightGradStore.enabled
        if defer_wgrad:
            WeightGradStore.enabled = True
        try:
            return rec.s3.backward(grads)
        finally:
            WeightGradStore.enabled = prev


def stage3_w(layer):
    """Run the expert weight-gradient GEMMs that ``stage3_b(defer_wgrad=True)`` queued."""
    with nvtx_range("layer%02d.stage3_w" % layer.idx):
        WeightGradStore.flush()
        WeightGradStore.pop()


def stage4_f(ctx: ExecutionCtx, layer, rec: LayerRecord, outs, routing):
    ep = _ep()
    if routing is None or ep is None:
        return None
    with nvtx_range("layer%02d.stage4_f" % layer.idx):
        (p,) = rec.s4.begin(outs)
        region = ctx.comm()
        with region:
            back = ep.combine(p, routing.plan)
            rec.s4.end(back)
        region.share(produced=(back,), consumed=(p,))
    return region


def stage4_b(ctx: ExecutionCtx, layer, rec: LayerRecord, grads):
    with nvtx_range("layer%02d.stage4_b" % layer.idx):
        region = ctx.comm()
        with region:
            out = rec.s4.backward(grads)
        region.share(produced=out, consumed=grads)
    return out, region


def stage5_f(layer, rec: LayerRecord, outs, residual, routing, begin: bool = True):
    with nvtx_range("layer%02d.stage5_f" % layer.idx):
        if begin:
            outs, residual = rec.s5.begin(outs, residual)
        hidden = layer.forward_stage5(outs, residual, routing)
        rec.s5.end(hidden)
    return hidden


def stage5_b(layer, rec: LayerRecord, grads):
    with nvtx_range("layer%02d.stage5_b" % layer.idx):
        return rec.s5.backward(grads)


# ------------------------------------------------------------------------------------------------
# Sequential layer / model execution (used outside the overlapped steady state)
# ------------------------------------------------------------------------------------------------
def layer_forward(ctx: ExecutionCtx, layer, rec: LayerRecord, hidden, rotary, cu_seqlens):
    tokens, residual, routing = stage1_f(layer, rec, hidden, rotary, cu_seqlens)
    weights = routing.topk_weight if routing is not None else None
    region = stage2_f(ctx, layer, rec, tokens, routing)
    if region is not None:
        region.wait()
        tokens, weights = rec.s2.outputs
    outs = stage3_f(layer, rec, routing, tokens, weights)
    region = stage4_f(ctx, layer, rec, outs, routing)
    if region is not None:
        region.wait()
        (outs,) = rec.s4.outputs
    return stage5_f(layer, rec, outs, residual, routing)


def layer_backward(ctx: ExecutionCtx, layer, rec: LayerRecord, d_hidden):
    d_outs, d_residual = stage5_b(layer, rec, (d_hidden,))
    if rec.s4.live:
        (d_outs,), region = stage4_b(ctx, layer, rec, (d_outs,))
        region.wait()
    d_tokens, d_weights = stage3_b(layer, rec, (d_outs,))
    if rec.s2.live:
        (d_tokens, d_weights), region = stage2_b(ctx, layer, rec, (d_tokens, d_weights))
        region.wait()
    (d_hidden,) = stage1_b(layer, rec, (d_tokens, d_residual, d_weights))
    rec.routing = None
    return d_hidden


def prolog_f(module, inputs, rec: ChunkRecord):
    with nvtx_range("prolog_f"):
        # token ids carry no gradient; the embedding op accumulates into its parameter directly
        hidden = module.forward_prolog(inputs)
        rec.prolog.inputs = ()
        rec.prolog.end(hidden)
    return hidden


def prolog_b(module, rec: ChunkRecord, d_hidden):
    with nvtx_range("prolog_b"):
        rec.prolog.backward((d_hidden,))


def epilog_f(module, hidden, rec: ChunkRecord):
    with nvtx_range("epilog_f"):
        (h,) = rec.epilog.begin(hidden)
        logits = module.forward_epilog(h)
    return logits


def model_forward(module, inputs, rec: ChunkRecord, cu_seqlens=None, ctx: Optional[ExecutionCtx] = None):
    """Forward of one micro-batch through one model chunk, filling ``rec``.

    Returns the chunk output: hidden states, or logits on the last stage.
    """
    ctx = ctx or ExecutionCtx.make()
    rec.cu_seqlens = cu_seqlens
    hidden = inputs
    if module.stage_index == 0:
        hidden = prolog_f(module, hidden, rec)
    rotary = module.forward_posemb(hidden.shape[1], cu_seqlens)
    rec.rotary = rotary
    for layer, lrec in zip(module.layers.values(), rec.layers):
        lrec.merged_prev = False
        hidden = layer_forward(ctx, layer, lrec, hidden, rotary, cu_seqlens)
    if module.stage_index == module.stage_count - 1:
        hidden = epilog_f(module, hidden, rec)
    return hidden


def model_backward(module, rec: ChunkRecord, output_grad: Optional[torch.Tensor], loss: Optional[torch.Tensor] = None,
                   ctx: Optional[ExecutionCtx] = None):
    """Backward of one micro-batch through one model chunk. Returns the gradient w.r.t. its input
    hidden states (``None`` on the first stage, whose input is token ids)."""
    ctx = ctx or ExecutionCtx.make()
    if module.stage_index == module.stage_count - 1:
        assert loss is not None
        with nvtx_range("loss.backward()"):
            loss.backward()
        (d_hidden,) = (rec.epilog.inputs[0].grad,)
        rec.epilog.clear()
    else:
        d_hidden = output_grad
    layers = list(module.layers.values())
    for layer, lrec in zip(reversed(layers), reversed(rec.layers)):
        d_hidden = layer_backward(ctx, layer, lrec, d_hidden)
    if module.stage_index == 0:
        prolog_b(module, rec, d_hidden)
        d_hidden = None
    rec.rotary = None
    return d_hidden
