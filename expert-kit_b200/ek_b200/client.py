"""In-process stand-in for `ExpertKitClient` (expertkit_torch/grpc_client.py:13-76): same
`forward_expert(expert_ids, hidden_state)` call and the same [T, k, H] reply, served by the
local CUDA backend instead of a gRPC round trip through controller and workers."""
from __future__ import annotations

from typing import List

import torch

from .backend import Backend, EKError


def parse_expert_id(expert_id: str):
    """"{model}/l{layer}-e{expert}" -> (model, layer, expert); the format produced at
    expertkit_torch/models/qwen3_moe.py:92-95 and deepseek_v3/model.py:72-76 and parsed by
    ExpertKey::from_expert_id (ek-db/src/safetensor/mod.rs:57-73)."""
    parts = expert_id.split("/l")
    if len(parts) != 2:
        raise EKError(3, f"invalid expert id: {expert_id}")
    inner = parts[1].split("-e")
    if len(inner) != 2:
        raise EKError(3, f"invalid expert id: {expert_id}")
    try:
        return parts[0], int(inner[0]), int(inner[1])
    except ValueError:
        raise EKError(3, f"invalid expert id: {expert_id}") from None


class LocalExpertKitClient:
    def __init__(self, backend: Backend, timeout_sec: float = 2.0):
        self.backend = backend
        self.timeout = timeout_sec   # kept for signature compatibility; local calls do not time out

    def forward_expert(self, expert_ids: List[List[str]], hidden_state: torch.Tensor) -> torch.Tensor:
        """expert_ids: [T][k] id strings; hidden_state: [T, H].  Returns [T, k, H] on the input's
        device.  Raises RuntimeError on failure, as the gRPC client does."""
        T = hidden_state.shape[0]
        if len(expert_ids) != T:
            raise RuntimeError("expert_ids and hidden_state disagree on the number of sequences")
        k = len(expert_ids[0]) if T else 0
        layer = None
        flat = []
        for row in expert_ids:
            if len(row) != k:
                raise RuntimeError("ragged expert id lists are not supported")
            for s in row:
                _, l, e = parse_expert_id(s)
                if layer is None:
                    layer = l
                elif l != layer:
                    raise RuntimeError("one request must address a single layer")
                flat.append(e)
        ids = torch.tensor(flat, dtype=torch.int32).view(T, k)
        try:
            return self.backend.moe_forward(layer, hidden_state, ids)
        except EKError as e:
            raise RuntimeError(f"expert forward failed: {e}") from e
