"""Host-side mirror of the worker's compute seam on top of the C ABI.

Names follow the reference: `ExpertDB` (ek-computation/src/worker/manager.rs:13-23) becomes the
registry methods of `Backend`; `ExpertBackend::forward` (ek-computation/src/ffn/mod.rs:39-52)
is `expert_forward`; `EKInstanceGate::forward` (ek-computation/src/worker/core.rs:47-74) is
`worker_forward_wire`; the controller's `NaiveExecutor` (controller/executor.rs) is
`moe_forward`.  torch is used only to own buffers and hand out pointers."""
from __future__ import annotations

import os

import ctypes as C
from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Tuple

import torch

from . import _lib as L


class EKError(RuntimeError):
    """An EKError of the reference (ek-base/src/error.rs:13-72) surfaced from the C ABI."""

    def __init__(self, status: int, message: str):
        self.status = status
        self.status_name = L.STATUS_NAMES.get(status, f"EK_{status}")
        super().__init__(f"{self.status_name}: {message}")


@dataclass
class BackendConfig:
    hidden: int
    intermediate: int
    n_experts: int
    top_k: int
    scoring: int = L.EK_SCORE_SOFTMAX
    n_group: int = 1
    topk_group: int = 1
    norm_topk_prob: bool = True
    routed_scaling: float = 1.0
    n_shared_experts: int = 0
    bf16_combine: bool = False
    quant: int = L.EK_QUANT_BF16
    max_tokens: int = 256
    max_layers: int = 1
    device: int = 0
    ep_rank: int = 0
    ep_size: int = 1
    model_name: str = "model"
    replica_slots: int = 0

    def to_c(self) -> L.Config:
        c = L.Config()
        for f in ("hidden", "intermediate", "n_experts", "top_k", "scoring", "n_group", "topk_group",
                  "n_shared_experts", "quant", "max_tokens", "max_layers", "device", "ep_rank", "ep_size",
                  "replica_slots"):
            setattr(c, f, int(getattr(self, f)))
        c.norm_topk_prob = int(bool(self.norm_topk_prob))
        c.bf16_combine = int(bool(self.bf16_combine))
        c.routed_scaling = float(self.routed_scaling)
        c.model_name = self.model_name.encode()
        return c


_TORCH_TO_EK = {
    torch.bfloat16: L.EK_BF16, torch.float32: L.EK_F32, torch.int8: L.EK_I8, torch.int32: L.EK_I32,
    torch.float16: L.EK_F16, torch.uint8: L.EK_U8, torch.int64: L.EK_I64,
}
if hasattr(torch, "float8_e4m3fn"):
    _TORCH_TO_EK[torch.float8_e4m3fn] = L.EK_F8_E4M3


def _tensors_ready(tensors):
    """Registration reads device tensors on the library's own stream, which does not wait for
    torch's: whatever produced them on torch's current stream must have finished first."""
    for dev in {t.device for t in tensors if t is not None and t.is_cuda}:
        torch.cuda.current_stream(dev).synchronize()


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else C.c_void_p(t.data_ptr())


class Backend:
    """One expert-worker compute backend bound to one GPU."""

    def __init__(self, cfg: BackendConfig):
        self._lib = L.load()
        self.cfg = cfg
        h = C.c_void_p()
        c = cfg.to_c()
        st = self._lib.ek_backend_create(C.byref(c), C.byref(h))
        if st != L.EK_OK:
            raise EKError(st, self._lib.ek_create_error().decode())
        self._h = h

    # ---- lifetime -------------------------------------------------------------------------
    def close(self):
        if getattr(self, "_h", None):
            self._lib.ek_backend_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def _check(self, st: int):
        if st != L.EK_OK:
            raise EKError(st, self._lib.ek_last_error(self._h).decode())

    def expert_id(self, layer: int, expert: int) -> str:
        """ExpertKey::as_object_key (ek-db/src/safetensor/mod.rs:88-90)."""
        return f"{self.cfg.model_name}/l{layer}-e{expert}"

    def shared_id(self, layer: int) -> str:
        return f"{self.cfg.model_name}/l{layer}-shared"

    # ---- registry (ExpertDB) ----------------------------------------------------------------
    def register_expert(self, expert_id: str, tensors: Dict[str, torch.Tensor]):
        """ExpertDB::insert(ExpertBackend::build(...)).  `tensors` maps the names the weight
        server uses to contiguous tensors (CPU or CUDA)."""
        keep = []
        _tensors_ready(tensors.values())
        views = (L.TensorView * len(tensors))()
        for i, (name, t) in enumerate(tensors.items()):
            t = t.contiguous()
            keep.append(t)
            if t.dtype not in _TORCH_TO_EK:
                raise EKError(3, f"unsupported dtype {t.dtype} for {name}")
            views[i].name = name.encode()
            views[i].dtype = _TORCH_TO_EK[t.dtype]
            views[i].ndim = t.dim()
            for j in range(4):
                views[i].shape[j] = t.shape[j] if j < t.dim() else 1
            views[i].data = t.data_ptr()
        self._check(self._lib.ek_expert_register(self._h, expert_id.encode(), views, len(tensors)))

    def register_bundle(self, expert_id: str, blob: bytes):
        """From the serialised per-expert bundle of the weight server."""
        buf = (C.c_char * len(blob)).from_buffer_copy(blob)
        self._check(self._lib.ek_expert_register_safetensors(self._h, expert_id.encode(), buf, len(blob)))

    def export_tiles(self, expert_id: str) -> bytes:
        """The registered expert in its device-ready form (tiles + scales as kept in HBM)."""
        need = C.c_size_t(0)
        self._lib.ek_expert_export_tiles(self._h, expert_id.encode(), None, 0, C.byref(need))
        if need.value == 0:
            raise EKError(3, self._lib.ek_last_error(self._h).decode())
        buf = (C.c_char * need.value)()
        self._check(self._lib.ek_expert_export_tiles(self._h, expert_id.encode(), buf, need.value, C.byref(need)))
        return bytes(buf)

    def register_tiles(self, expert_id: str, blob: bytes):
        """Registers a blob written by `export_tiles` with plain copies (no decoding, no re-tiling)."""
        buf = (C.c_char * len(blob)).from_buffer_copy(blob)
        self._check(self._lib.ek_expert_register_tiles(self._h, expert_id.encode(), buf, len(blob)))

    def mark_loading(self, expert_id: str) -> bool:
        fresh = C.c_int32(0)
        self._check(self._lib.ek_expert_mark_loading(self._h, expert_id.encode(), C.byref(fresh)))
        return bool(fresh.value)

    def evict(self, expert_id: str):
        self._check(self._lib.ek_expert_evict(self._h, expert_id.encode()))

    remove = evict

    def has(self, expert_id: str) -> bool:
        return bool(self._lib.ek_expert_has(self._h, expert_id.encode()))

    def loaded(self) -> int:
        return self._lib.ek_expert_loaded(self._h)

    def loading(self) -> int:
        return self._lib.ek_expert_loading(self._h)

    def keys(self) -> List[str]:
        need = C.c_size_t(0)
        self._lib.ek_expert_keys(self._h, None, 0, C.byref(need))
        buf = C.create_string_buffer(need.value)
        self._check(self._lib.ek_expert_keys(self._h, buf, need.value, C.byref(need)))
        s = buf.value.decode()
        return s.split("\n") if s else []

    def register_router(self, layer: int, weight: torch.Tensor, bias: Optional[torch.Tensor] = None):
        weight = weight.contiguous()
        if weight.dtype not in (torch.bfloat16, torch.float32):
            raise EKError(3, "router weight must be bf16 or fp32")
        if bias is not None:
            bias = bias.to(torch.float32).contiguous()
        _tensors_ready((weight, bias))
        self._check(self._lib.ek_router_register(self._h, layer, _ptr(weight), _TORCH_TO_EK[weight.dtype],
                                                 _ptr(bias)))

    # ---- forward ----------------------------------------------------------------------------
    def expert_forward(self, expert_id: str, x: torch.Tensor) -> torch.Tensor:
        """ExpertBackend::forward: one expert on an [n, H] bf16 batch."""
        if x.dim() != 2:
            raise EKError(3, "input must be 2-D")   # ffn/mod.rs:45 asserts this
        x = x.to(torch.bfloat16).contiguous()
        y = torch.empty_like(x)
        self._check(self._lib.ek_expert_forward(self._h, expert_id.encode(), _ptr(x), x.shape[0], _ptr(y)))
        return y

    def moe_forward(self, layer: int, x: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
        """NaiveExecutor: unweighted expert outputs [T, k, H] in the request's slot order."""
        x = x.to(torch.bfloat16).contiguous()
        ids = ids.to(torch.int32).contiguous()
        if ids.device != x.device:
            ids = ids.to(x.device)
        T, k = ids.shape
        out = torch.empty(T, k, x.shape[1], dtype=torch.bfloat16, device=x.device)
        self._check(self._lib.ek_moe_forward(self._h, layer, _ptr(x), T, _ptr(ids), k, _ptr(out)))
        return out

    def moe_forward_fused(self, layer: int, x: torch.Tensor, debug: bool = False):
        """Router + bucketing + experts + weighted combine + shared expert.  With `debug` the
        routing artefacts come back as a dict next to y."""
        x = x.to(torch.bfloat16).contiguous()
        T = x.shape[0]
        y = torch.empty_like(x)
        if not debug:
            self._check(self._lib.ek_moe_forward_fused(self._h, layer, _ptr(x), T, _ptr(y), None))
            return y
        E, k = self.cfg.n_experts, self.cfg.top_k
        art = dict(logits=torch.empty(T, E, dtype=torch.float32), ids=torch.empty(T, k, dtype=torch.int32),
                   weights=torch.empty(T, k, dtype=torch.float32), counts=torch.empty(E, dtype=torch.int32),
                   offsets=torch.empty(E + 1, dtype=torch.int32), perm=torch.empty(T * k, dtype=torch.int32))
        dbg = L.RouteDebug(*[art[n].data_ptr() for n in ("logits", "ids", "weights", "counts", "offsets", "perm")])
        self._check(self._lib.ek_moe_forward_fused(self._h, layer, _ptr(x), T, _ptr(y), C.byref(dbg)))
        return y, art

    def moe_forward_fused_async(self, layer: int, x: torch.Tensor, y: torch.Tensor):
        """Device-resident call, asynchronous on the backend stream; pair with `sync()`."""
        assert x.is_cuda and y.is_cuda and x.dtype == torch.bfloat16 and y.dtype == torch.bfloat16
        self._check(self._lib.ek_moe_forward_fused_async(self._h, layer, _ptr(x), x.shape[0], _ptr(y)))

    def sync(self):
        self._check(self._lib.ek_sync(self._h))

    def set_stream(self, cuda_stream: Optional[int]):
        """Run on the given CUDA stream handle (0 = the default stream); None = the backend's own."""
        h = C.c_void_p(-1) if cuda_stream is None else C.c_void_p(int(cuda_stream))
        self._check(self._lib.ek_set_stream(self._h, h))
        self._stream = cuda_stream

    def use_torch_stream(self):
        """Moves the backend to torch's current stream if it is not there already.  The backend has
        ONE stream, whoever calls: modules of different layers that share a backend all go through
        here, so none of them can keep running on a stream another one has left."""
        s = torch.cuda.current_stream(self.cfg.device).cuda_stream
        if getattr(self, "_stream", -2) != s:
            self.set_stream(s)     # synchronises the old stream once, at the switch

    # ---- expert-parallel stages (device tensors, asynchronous on the backend stream) -------------
    def ep_route(self, layer: int, x: torch.Tensor, send_rows: torch.Tensor, counts: torch.Tensor):
        assert x.is_cuda and send_rows.is_cuda and counts.is_cuda and counts.dtype == torch.int32
        assert x.dtype == torch.bfloat16 and x.is_contiguous() and send_rows.is_contiguous()
        self._check(self._lib.ek_ep_route(self._h, layer, _ptr(x), x.shape[0], _ptr(send_rows), _ptr(counts)))

    def ep_ffn(self, layer: int, rows: torch.Tensor, counts_src: torch.Tensor, x: torch.Tensor,
               out_rows: torch.Tensor):
        counts_src = counts_src.to(torch.int32).contiguous().cpu()
        assert rows.is_contiguous() and out_rows.is_contiguous() and x.is_contiguous()
        self._check(self._lib.ek_ep_ffn(self._h, layer, _ptr(rows) if rows.numel() else None, _ptr(counts_src), _ptr(x),
                                        x.shape[0], _ptr(out_rows) if out_rows.numel() else None))

    def ep_partial(self, layer: int, x_all: torch.Tensor, t0: int, T_local: int, partial: torch.Tensor):
        assert x_all.is_cuda and partial.is_cuda and partial.dtype == torch.float32
        assert x_all.dtype == torch.bfloat16 and x_all.is_contiguous() and partial.is_contiguous()
        self._check(self._lib.ek_ep_partial(self._h, layer, _ptr(x_all), x_all.shape[0], t0, T_local, _ptr(partial)))

    def set_owners(self, layer: int, owners: Optional[torch.Tensor]):
        """Names the rank that serves each expert in the following passes on `layer` (int32 [n_experts],
        the same table on every rank); None returns to the window rule."""
        if owners is None:
            self._check(self._lib.ek_ep_set_owners(self._h, layer, None))
            return
        o = owners.to(torch.int32).contiguous().cpu()
        self._check(self._lib.ek_ep_set_owners(self._h, layer, _ptr(o)))

    def ep_finish(self, layer: int, reduced: torch.Tensor, y: torch.Tensor):
        assert reduced.dtype == torch.float32 and reduced.is_contiguous() and y.is_contiguous()
        self._check(self._lib.ek_ep_finish(self._h, layer, _ptr(reduced), reduced.shape[0], _ptr(y)))

    def ep_combine(self, layer: int, returned: torch.Tensor, T: int, y: torch.Tensor):
        assert returned.is_contiguous() and y.is_contiguous()
        self._check(self._lib.ek_ep_combine(self._h, layer, _ptr(returned), T, _ptr(y)))

    def route_from_logits_device(self, logits: torch.Tensor, bias: Optional[torch.Tensor] = None):
        """`route_from_logits` with the results left on the logits' device."""
        return self.route_from_logits(logits, bias, out_device=logits.device)

    def route_from_logits(self, logits: torch.Tensor, bias: Optional[torch.Tensor] = None, out_device="cpu"):
        logits = logits.to(torch.float32).contiguous()
        T = logits.shape[0]
        E, k = self.cfg.n_experts, self.cfg.top_k
        if bias is not None:
            bias = bias.to(torch.float32).contiguous()
        d = out_device
        art = dict(ids=torch.empty(T, k, dtype=torch.int32, device=d), weights=torch.empty(T, k, dtype=torch.float32, device=d),
                   counts=torch.empty(E, dtype=torch.int32, device=d), offsets=torch.empty(E + 1, dtype=torch.int32, device=d),
                   perm=torch.empty(T * k, dtype=torch.int32, device=d))
        self._check(self._lib.ek_route_from_logits(self._h, _ptr(logits), T, _ptr(bias), _ptr(art["ids"]),
                                                   _ptr(art["weights"]), _ptr(art["counts"]),
                                                   _ptr(art["offsets"]), _ptr(art["perm"])))
        return art

    def combine(self, outputs: torch.Tensor, weights: torch.Tensor,
                shared: Optional[torch.Tensor] = None) -> torch.Tensor:
        outputs = outputs.to(torch.bfloat16).contiguous()
        weights = weights.to(torch.float32).contiguous()
        T, k, H = outputs.shape
        if shared is not None:
            shared = shared.to(torch.bfloat16).contiguous()
        y = torch.empty(T, H, dtype=torch.bfloat16, device=outputs.device)
        self._check(self._lib.ek_combine(self._h, _ptr(outputs), _ptr(weights), T, k, _ptr(shared), _ptr(y)))
        return y

    def w8a16_activate(self, w: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
        """w8a16_activate (ek-computation/src/ffn/expert_torch.rs:24-53)."""
        w = w.contiguous()
        scale = scale.to(torch.float32).contiguous()
        out = torch.empty(w.shape, dtype=torch.bfloat16, device=w.device)
        self._check(self._lib.ek_w8a16_activate(self._h, _ptr(w), _TORCH_TO_EK[w.dtype], _ptr(scale),
                                                w.shape[0], w.shape[1], _ptr(out)))
        return out

    def worker_forward_wire(self, expert_id: str, req_tensor: bytes) -> bytes:
        """EKInstanceGate::forward on the serialised tensor of a ForwardReq; returns the bytes
        of ForwardResp.output_tensor."""
        need = C.c_size_t(0)
        req = (C.c_char * len(req_tensor)).from_buffer_copy(req_tensor)
        cap = len(req_tensor) + 256
        resp = C.create_string_buffer(cap)
        self._check(self._lib.ek_worker_forward_wire(self._h, expert_id.encode(), req, len(req_tensor), resp, cap,
                                                     C.byref(need)))
        return resp.raw[:need.value]

    # ---- observability ----------------------------------------------------------------------
    def expert_counts(self, layer: int) -> torch.Tensor:
        out = torch.empty(self.cfg.n_experts, dtype=torch.int32)
        self._check(self._lib.ek_expert_counts(self._h, layer, _ptr(out)))
        return out

    def last_routing(self, T: int):
        """(ids [T,k] int32, weights [T,k] fp32) of the last routing pass, on the host."""
        k = self.cfg.top_k
        ids = torch.empty(T, k, dtype=torch.int32)
        w = torch.empty(T, k, dtype=torch.float32)
        self._check(self._lib.ek_last_routing(self._h, T, _ptr(ids), _ptr(w)))
        return ids, w

    def stage_timing(self, on: bool):
        self._check(self._lib.ek_stage_timing_enable(self._h, int(on)))

    def stage_times(self) -> Dict[str, float]:
        ms = (C.c_float * L.EK_STAGE_COUNT)()
        self._check(self._lib.ek_stage_times(self._h, ms))
        return {n: ms[i] for i, n in enumerate(L.STAGE_NAMES)}

    def kernel_launches(self) -> int:
        return int(self._lib.ek_kernel_launches(self._h))

    def worker_batch_stats(self):
        """(worker-level calls served, grouped passes that served them)."""
        calls, batches = C.c_int64(0), C.c_int64(0)
        self._check(self._lib.ek_worker_batch_stats(self._h, C.byref(calls), C.byref(batches)))
        return int(calls.value), int(batches.value)

    def set_precise_dequant(self, on: bool):
        """fp8: apply block scales in fp32 inside the GEMM (bit-exact reference dequantisation)."""
        self._check(self._lib.ek_set_precise_dequant(self._h, int(on)))

    def debug_set_ffn_impl(self, impl: int):
        self._check(self._lib.ek_debug_set_ffn_impl(self._h, impl))


def expert_tensors(layer: int, expert, up, gate, down, up_s=None, gate_s=None, down_s=None,
                   shared: bool = False) -> Dict[str, torch.Tensor]:
    """Names one expert's tensors the way the weight server does
    (ek-db/src/safetensor/transformer.rs:249-280)."""
    base = (f"model.layers.{layer}.mlp.shared_experts" if shared
            else f"model.layers.{layer}.mlp.experts.{expert}")
    t = {f"{base}.gate_proj.weight": gate, f"{base}.down_proj.weight": down, f"{base}.up_proj.weight": up}
    if up_s is not None:
        t[f"{base}.up_proj.weight_scale_inv"] = up_s
        t[f"{base}.down_proj.weight_scale_inv"] = down_s
        t[f"{base}.gate_proj.weight_scale_inv"] = gate_s
    return t


class TileCache:
    """File cache of device-ready experts, beside the raw bundles the weight server caches
    (ek-db/src/safetensor/mod.rs:144-171: `fs` cache keyed by ExpertKey::as_object_key).  A hit
    registers the expert with plain copies; a miss (or a blob written by another layout version or
    configuration) loads the bundle through `fetch_bundle`, registers it and writes the blob."""

    def __init__(self, backend: "Backend", root: str):
        self.be, self.root = backend, root
        os.makedirs(root, exist_ok=True)
        self.hits = self.misses = 0

    def path(self, expert_id: str) -> str:
        c = self.be.cfg
        name = f"{expert_id.replace('/', '__')}.v{L.EK_TILE_LAYOUT_VERSION}.q{c.quant}.h{c.hidden}.i{c.intermediate}.ektiles"
        return os.path.join(self.root, name)

    def load(self, expert_id: str, fetch_bundle) -> bool:
        """Registers `expert_id`; returns True when the cache served it."""
        p = self.path(expert_id)
        if os.path.exists(p):
            try:
                with open(p, "rb") as f:
                    self.be.register_tiles(expert_id, f.read())
                self.hits += 1
                return True
            except EKError:
                os.remove(p)          # stale or foreign blob: fall back to the bundle
        self.be.register_bundle(expert_id, fetch_bundle(expert_id))
        tmp = p + ".tmp"
        with open(tmp, "wb") as f:
            f.write(self.be.export_tiles(expert_id))
        os.replace(tmp, p)
        self.misses += 1
        return False
