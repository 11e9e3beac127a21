"""torch modules that put the whole MoE block behind one library call.

The reference's interceptors keep the router and the combine in Python and send the expert work
through gRPC (`InterceptedMoE`, expertkit_torch/models/qwen3_moe.py:37-113;
`InterceptedDeepseekV3MoE`, expertkit_torch/models/deepseek_v3/model.py:24-106).  `B200MoEBlock`
has the same call shape -- `forward(hidden_states[..., H])` returning the block output (and the
router logits for the Qwen3 form) -- but router, bucketing, expert FFNs, weighted combine and the
shared expert run as the fused device-resident call, on torch's current stream, with no host
synchronisation: it can sit inside a decoder layer exactly where the intercepted block sits.
Because nothing synchronises, device-side errors surface only through `check()`: call it once per
model forward.
"""
from __future__ import annotations

from typing import Optional

import torch

from .backend import Backend


class B200MoEBlock(torch.nn.Module):
    def __init__(self, backend: Backend, layer_idx: int, return_router_logits: bool = False):
        """`backend` already holds the router, the experts and the shared expert of `layer_idx`
        (registered from the weight server's bundles).  `return_router_logits`: Qwen3's block
        returns `(hidden_states, router_logits)` (qwen3_moe.py:113); DeepSeek-V3's returns the
        hidden states alone (model.py:153)."""
        super().__init__()
        self.backend = backend
        self.layer_idx = layer_idx
        self.return_router_logits = return_router_logits

    def check(self):
        """Synchronises the backend's stream and raises `EKError` if any pass since the last check
        recorded a device-side error (an unregistered expert selected by routing, a failed index
        check, a bounded wait that ran out).  The DeepSeek-V3 form of `forward` is asynchronous and
        cannot report such an error itself; the device status word is sticky and every later pass
        on the backend skips its expert GEMMs until it has been read.  Call this once per model
        forward (after the last decoder layer), not per block."""
        self.backend.sync()

    def forward(self, hidden_states: torch.Tensor):
        if not hidden_states.is_cuda:
            raise RuntimeError("B200MoEBlock runs on CUDA tensors only")
        shape = hidden_states.shape
        x = hidden_states.reshape(-1, shape[-1]).to(torch.bfloat16).contiguous()
        self.backend.use_torch_stream()
        if self.return_router_logits:
            y, art = self.backend.moe_forward_fused(self.layer_idx, x, debug=True)
            return y.view(shape).to(hidden_states.dtype), art["logits"].to(x.device)
        y = torch.empty_like(x)
        self.backend.moe_forward_fused_async(self.layer_idx, x, y)
        return y.view(shape).to(hidden_states.dtype)
