"""Overlapped forward/backward of two micro-batches on one rank.

The forward of a micro-batch through one model chunk and the backward of another micro-batch
through the other chunk are written as two coroutines that yield at every stage boundary; the
driver alternates between them. Both sides are cut into four segments per layer so that every
expert exchange (stages 2 and 4, on the communication stream) is in flight under a compute segment
of the other side:

    backward: [B5, launch B4] [wait B4, B3 dgrad, launch B2] [B3 wgrad        ] [wait B2, B1 attention]
    forward :   [F1 attention, launch F2] [wait F2, F3 experts, launch F4] [ -- ] [wait F4, F5]

i.e. on the compute stream: B5, F1 (covers B4), B3 (covers F2), F3 (covers B2), W (covers F4), B1, F5. The reference hand-unrolls the same
idea for equal layer counts plus special cases (pithtrain/dualpipe/overlap.py:50-331); coroutines
cover unequal layer counts and dense layers without special cases.
"""

from __future__ import annotations

from typing import Callable, Generator, List

import torch

from .execution import (
    ChunkRecord,
    ExecutionCtx,
    epilog_f,
    nvtx_range,
    prolog_b,
    prolog_f,
    stage1_b,
    stage1_f,
    stage2_b,
    stage2_f,
    stage3_b,
    stage3_f,
    stage4_b,
    stage4_f,
    stage5_b,
    stage5_f,
)
from .utils import WeightGradStore


def forward_coroutine(ctx: ExecutionCtx, module, inputs, rec: ChunkRecord, cu_seqlens, result: list) -> Generator:
    """Yields at stage boundaries; appends the chunk output to ``result`` when done."""
    rec.cu_seqlens = cu_seqlens
    hidden = inputs
    if module.stage_index == 0:
        hidden = prolog_f(module, hidden, rec)
    rotary = module.forward_posemb(hidden.shape[1], cu_seqlens)
    rec.rotary = rotary
    for layer, lrec in zip(module.layers.values(), rec.layers):
        lrec.merged_prev = False
        # segment 1: attention + router, then the dispatch goes out on the communication stream
        tokens, residual, routing = stage1_f(layer, lrec, hidden, rotary, cu_seqlens)
        weights = routing.topk_weight if routing is not None else None
        region = stage2_f(ctx, layer, lrec, tokens, routing)
        yield
        # segment 2: experts, then the combine goes out
        if region is not None:
            region.wait()
            tokens, weights = lrec.s2.outputs
        outs = stage3_f(layer, lrec, routing, tokens, weights)
        region = stage4_f(ctx, layer, lrec, outs, routing)
        yield
        # segment 3: nothing to compute here; the other side's weight gradients cover the combine
        if region is not None:
            yield
            region.wait()
            (outs,) = lrec.s4.outputs
        # segment 4: residual add
        hidden = stage5_f(layer, lrec, outs, residual, routing)
        yield
    if module.stage_index == module.stage_count - 1:
        hidden = epilog_f(module, hidden, rec)
    result.append(hidden)


def backward_coroutine(ctx: ExecutionCtx, module, rec: ChunkRecord, output_grad, loss, result: list) -> Generator:
    """Backward twin of :func:`forward_coroutine`; appends the input gradient to ``result``."""
    if module.stage_index == module.stage_count - 1:
        with nvtx_range("loss.backward()"):
            loss.backward()
        d_hidden = rec.epilog.inputs[0].grad
        rec.epilog.clear()
    else:
        d_hidden = output_grad
    layers = list(module.layers.values())
    for layer, lrec in zip(reversed(layers), reversed(rec.layers)):
        # segment 1: residual split, then the combine-gradient exchange goes out
        d_outs, d_residual = stage5_b(layer, lrec, (d_hidden,))
        region = None
        if lrec.s4.live:
            (d_outs,), region = stage4_b(ctx, layer, lrec, (d_outs,))
        yield
        # segment 2: expert input gradients (weight gradients split off), then the dispatch-gradient exchange
        if region is not None:
            region.wait()
        local: List[Callable] = []
        defer = lrec.is_moe and not WeightGradStore.enabled
        if defer:
            saved, WeightGradStore.cache = WeightGradStore.cache, local
        d_tokens, d_weights = stage3_b(layer, lrec, (d_outs,), defer_wgrad=defer)
        if defer:
            WeightGradStore.cache = saved
        region = None
        if lrec.s2.live:
            (d_tokens, d_weights), region = stage2_b(ctx, layer, lrec, (d_tokens, d_weights))
        yield
        # segment 3: the expert weight gradients fill the time both exchanges are in flight
        if local:
            with nvtx_range("layer%02d.stage3_w" % layer.idx), torch.no_grad():
                for fn in local:
                    fn()
            local.clear()
        yield
        # segment 4: attention backward
        if region is not None:
            region.wait()
        (d_hidden,) = stage1_b(layer, lrec, (d_tokens, d_residual, d_weights))
        lrec.routing = None
        yield
    if module.stage_index == 0:
        prolog_b(module, rec, d_hidden)
        d_hidden = None
    rec.rotary = None
    result.append(d_hidden)


def overlapped_forward_backward(module0, inputs0, rec0: ChunkRecord, cu_seqlens0,
                                module1, rec1: ChunkRecord, output_grad1, loss1,
                                comm_stream=None):
    """Run forward(module0, inputs0) interleaved with backward(module1, rec1).

    Returns ``(outputs0, input_grad1)``.
    """
    ctx = ExecutionCtx.make(comm_stream)
    f_res: list = []
    b_res: list = []
    fwd = forward_coroutine(ctx, module0, inputs0, rec0, cu_seqlens0, f_res)
    bwd = backward_coroutine(ctx, module1, rec1, output_grad1, loss1, b_res)
    f_live = b_live = True
    while f_live or b_live:
        if b_live:
            try:
                next(bwd)
            except StopIteration:
                b_live = False
        if f_live:
            try:
                next(fwd)
            except StopIteration:
                f_live = False
    return f_res[0], b_res[0]
