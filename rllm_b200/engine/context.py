"""The description of one step's batch that every part sees."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

import torch


@dataclass
class GroupView:
    """Per cache group (layers with the same cache needs): where the step's new tokens go
    and where each sequence's pages are."""
    slots: torch.Tensor          # int32 [T]: page * page_size + offset
    block_table: torch.Tensor    # int32 [S, P]: page ids, -1 where given back / not yet held
    page_size: int


@dataclass
class StepContext:
    """One batch: T tokens of S sequences, rows of a sequence adjacent and in order.

    Device tensors (int32): `token_ids` [T], `positions` [T] (absolute position of each
    token in its sequence), `token_seq` [T] (which sequence), `cu_q` [S+1] (row range of
    each sequence), `kv_lens` [S] (keys visible to the sequence's last token, new ones
    included), `state_slots` [S]. Host mirrors (`q_lens`, `kv_lens_host`, ...) let a part
    choose a kernel without a device read."""
    backend: Any
    num_tokens: int
    num_seqs: int
    token_ids: torch.Tensor
    positions: torch.Tensor
    token_seq: torch.Tensor
    cu_q: torch.Tensor
    kv_lens: torch.Tensor
    state_slots: torch.Tensor | None
    q_lens_host: list[int]
    kv_lens_host: list[int]
    state_slots_host: list[int]
    groups: dict[int, GroupView] = field(default_factory=dict)
    max_q_len: int = 1
    max_kv_len: int = 1
    # decode-only steps captured in a CUDA graph read their sizes from device memory
    graph_safe: bool = False
    extras: dict[str, Any] = field(default_factory=dict)
    # what one forward pass shares between its layers (tables made at first use); the model
    # empties it when a pass begins, so nothing outlives the pass that made it
    per_forward: dict[str, Any] = field(default_factory=dict)

    @property
    def all_decode(self) -> bool:
        return self.max_q_len == 1
