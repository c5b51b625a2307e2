"""Protocols every model and decoder layer implements so the DualPipeV engine can drive them.

A layer is five stages: (1) attention + router, (2) expert dispatch, (3) expert MLP, (4) combine,
(5) aggregate + residual. Stages 2 and 4 belong to the engine / expert-parallel exchange; a layer
implements 1, 3 and 5 plus a plain-autograd ``reference_forward`` used as the numerical oracle.
The stage split and the model-level hooks mirror pithtrain/models/interface.py:26-116; the tensors
that travel differ because routing weights are applied on the expert rank here:

* stage 1 returns ``(tokens[m,H], residual[B,S,H], routing)``; ``routing`` is ``None`` for a dense layer;
* stage 3 takes the (dispatched) tokens and routing weights and returns weighted partial sums,
  one row per received token;
* stage 5 takes the (combined) partial rows, the residual and ``routing`` and returns hidden states.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, NamedTuple, Optional, Protocol, Tuple

import torch


class AllToAllSplits(NamedTuple):
    input_splits: List[int]
    output_splits: List[int]


@dataclass
class RoutingInfo:
    """Routing decision of one MoE layer for one micro-batch.

    ``topk_weight[m,k]`` (fp32, differentiable) and ``topk_idx[m,k]`` (global expert ids) come from the
    gate. ``plan`` is the expert-parallel dispatch plan (``None`` when ``ep_size == 1``); it carries
    what the reference calls ``moe_local_idxs`` / ``expand_idx`` / ``dispatch_splits`` /
    ``combine_splits``.
    """

    topk_weight: torch.Tensor
    topk_idx: torch.Tensor
    plan: Any = None
    lb_loss: Optional[torch.Tensor] = None

    @property
    def expert_idxs(self) -> torch.Tensor:
        return self.topk_idx


class MLPProtocol(Protocol):
    """MLP component of a decoder layer (dense or mixture of experts)."""


class LayerProtocol(Protocol):
    idx: int
    mlp: MLPProtocol

    def reference_forward(self, hidden_states: torch.Tensor, rotary_posemb, cu_seqlens=None) -> torch.Tensor: ...

    def forward_stage1(self, hidden_states: torch.Tensor, rotary_posemb, cu_seqlens: Optional[torch.Tensor] = None
                       ) -> Tuple[torch.Tensor, torch.Tensor, Optional[RoutingInfo]]: ...

    def forward_stage3(self, tokens: torch.Tensor, weights: Optional[torch.Tensor],
                       routing: Optional[RoutingInfo]) -> torch.Tensor: ...

    def forward_stage5(self, outs: torch.Tensor, residual: torch.Tensor,
                       routing: Optional[RoutingInfo]) -> torch.Tensor: ...


class ModelProtocol(Protocol):
    stage_index: int
    stage_count: int
    layers: Dict[str, LayerProtocol]

    def reference_forward(self, hidden_states: torch.Tensor, cu_seqlens=None) -> torch.Tensor: ...

    def forward_posemb(self, S: int, cu_seqlens: Optional[torch.Tensor] = None): ...

    def forward_prolog(self, hidden_states: torch.Tensor) -> torch.Tensor: ...

    def forward_epilog(self, hidden_states: torch.Tensor) -> torch.Tensor: ...
