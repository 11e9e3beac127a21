"""torch modules that put the whole MoE block behind one library call.

The reference's interceptors keep the router and the combine in Python and send the expert work
through gRPC (`InterceptedMoE`, expertkit_torch/models/qwen3_moe.py:37-113;
`InterceptedDeepseekV3MoE`, expertkit_torch/models/deepseek_v3/model.py:24-106).  `B200MoEBlock`
has the same call shape -- `forward(hidden_states[..., H])` returning the block output (and the
router logits for the Qwen3 form) -- but router, bucketing, expert FFNs, weighted combine and the
shared expert run as the fused device-resident call, on torch's current stream, with no host
synchronisation: it can sit inside a decoder layer exactly where the intercepted block sits.
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
        self._stream: Optional[int] = None

    def _use_current_stream(self):
        s = torch.cuda.current_stream().cuda_stream
        if s != self._stream:
            self.backend.set_stream(s)     # synchronises the old stream once, at the switch
            self._stream = s

    def forward(self, hidden_states: torch.Tensor):
        if not hidden_states.is_cuda:
            raise RuntimeError("B200MoEBlock runs on CUDA tensors only")
        shape = hidden_states.shape
        x = hidden_states.reshape(-1, shape[-1]).to(torch.bfloat16).contiguous()
        self._use_current_stream()
        if self.return_router_logits:
            y, art = self.backend.moe_forward_fused(self.layer_idx, x, debug=True)
            return y.view(shape).to(hidden_states.dtype), art["logits"].to(x.device)
        y = torch.empty_like(x)
        self.backend.moe_forward_fused_async(self.layer_idx, x, y)
        return y.view(shape).to(hidden_states.dtype)
