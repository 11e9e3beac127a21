"""Expert-parallel MoE layer over the GPUs of one box.

The reference shards experts over worker processes and moves rows with one gRPC per distinct
expert (ek-computation/src/controller/executor.rs:141-226).  Here expert e lives on rank
e // (n_experts // world) and rows move with two all-to-all exchanges over NVLink
(`torch.distributed`, NCCL): dispatch of the routed rows to the expert owners and return of the
expert outputs.  Routing, bucketing, the grouped expert FFN and the weighted combine are the
library's kernels (`ek_ep_route`, `ek_ep_ffn`, `ek_ep_combine`).

One process per GPU.  In the all-to-all scheme the exchange plan is computed on the host from the
all-gathered per-expert row counts (one host synchronisation per layer); the gather scheme for
decode-sized batches (`ek_ep_partial`, `ek_ep_finish`) needs none.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import ctypes as C

import torch
import torch.distributed as dist


def plan_exchange(counts_all: torch.Tensor, rank: int, world: int):
    """counts_all[r, e] = rows rank r routes to global expert e (host tensor).

    Returns (send_splits, recv_splits, counts_src): rows this rank sends to / receives from each
    rank, and counts_src[s, le] = rows arriving from rank s for local expert le -- arrival order is
    source-major, expert-minor, because every source sends its rows sorted by expert."""
    E = counts_all.shape[1]
    if E % world:
        raise ValueError("the expert count must be divisible by the number of ranks")
    el = E // world
    per_dest = counts_all.view(world, world, el).sum(dim=2)          # [src, dst]
    send_splits = per_dest[rank].tolist()
    recv_splits = per_dest[:, rank].tolist()
    counts_src = counts_all[:, rank * el:(rank + 1) * el].contiguous().to(torch.int32)
    return send_splits, recv_splits, counts_src


def choose_owners(holders: List[List[int]], step: int, counts: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One serving rank per expert for a pass.  `holders[e]` lists the ranks that hold expert e (home
    rank first).  Deterministic in `step`, so every rank computes the same table without talking:
    an expert with several holders rotates over them from pass to pass -- the stand-in for the
    reference's uniform random pick.  With `counts` (rows per expert of the previous pass) only
    experts above the mean load leave their home rank."""
    owners = torch.empty(len(holders), dtype=torch.int32)
    mean = float(counts.float().mean()) if counts is not None else 0.0
    for e, h in enumerate(holders):
        if len(h) > 1 and (counts is None or float(counts[e]) > mean):
            owners[e] = h[(step + e) % len(h)]
        else:
            owners[e] = h[0]
    return owners


class BackendStages:
    """The three device stages of one rank, served by the CUDA backend."""

    def __init__(self, backend):
        self.be = backend
        cfg = backend.cfg
        self.n_experts, self.top_k, self.hidden = cfg.n_experts, cfg.top_k, cfg.hidden

    def route(self, layer: int, x: torch.Tensor, send_rows: torch.Tensor, counts: torch.Tensor):
        self.be.ep_route(layer, x, send_rows, counts)

    def ffn(self, layer: int, rows: torch.Tensor, counts_src: torch.Tensor, x: torch.Tensor, out_rows: torch.Tensor):
        self.be.ep_ffn(layer, rows, counts_src, x, out_rows)

    def combine(self, layer: int, returned: torch.Tensor, T: int, y: torch.Tensor):
        self.be.ep_combine(layer, returned, T, y)

    def partial(self, layer: int, x_all: torch.Tensor, t0: int, T_local: int, partial: torch.Tensor):
        self.be.ep_partial(layer, x_all, t0, T_local, partial)

    def finish(self, layer: int, reduced: torch.Tensor, y: torch.Tensor):
        self.be.ep_finish(layer, reduced, y)

    def set_owners(self, layer: int, owners: Optional[torch.Tensor]):
        self.be.set_owners(layer, owners)

    # --- the same scheme over peer memory (no collectives) ---
    def peer_setup(self, group, tokens_per_rank: int):
        return PeerWorkspace(self.be, group, tokens_per_rank)

    def peer_step(self, layer: int, x: torch.Tensor, y: torch.Tensor, step: int):
        lib, h, T = self.be._lib, self.be._h, x.shape[0]
        self.be._check(lib.ek_ep_peer_push(h, x.data_ptr(), T, step))
        self.be._check(lib.ek_ep_peer_partial(h, layer, T, step))
        self.be._check(lib.ek_ep_peer_finish(h, layer, T, step, y.data_ptr()))


class PeerWorkspace:
    """The backend's peer buffers (gathered tokens, fp32 partial sums, flag words): allocated by the
    library, their CUDA IPC handles exchanged over the process group, every peer's opened."""

    def __init__(self, backend, group, tokens_per_rank: int):
        from . import _lib as L
        self.be, self.group = backend, group
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        self.tokens_per_rank = tokens_per_rank
        self.open = False

        def agree(ok: bool, what: str):
            """Every rank learns whether all ranks got through the last phase; raises on all if not."""
            flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device="cuda")
            dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
            if not bool(flag.item()):
                backend._lib.ek_ep_peer_close(backend._h)
                raise RuntimeError(f"peer-memory workspace: {what} failed on at least one rank")

        mine = (C.c_uint8 * (3 * L.EK_IPC_HANDLE_BYTES))()
        err = None
        try:
            backend._check(backend._lib.ek_ep_peer_alloc(backend._h, tokens_per_rank, mine))
        except Exception as ex:   # noqa: BLE001
            err = ex
        agree(err is None, f"allocation ({err})")
        everyone = [None] * world
        dist.all_gather_object(everyone, bytes(mine), group=group)
        try:
            for r in range(world):
                if r != rank:
                    buf = (C.c_uint8 * (3 * L.EK_IPC_HANDLE_BYTES)).from_buffer_copy(everyone[r])
                    backend._check(backend._lib.ek_ep_peer_open(backend._h, r, buf))
        except Exception as ex:   # noqa: BLE001
            err = ex
        agree(err is None, f"mapping the peers' buffers ({err})")
        self.open = True
        dist.barrier(group=group)     # nobody steps before every rank has mapped everything

    def close(self):
        """Unmaps the peers' buffers, then synchronises the ranks: a rank may only destroy its
        backend (and free its own buffers) once nobody has them mapped."""
        if not self.open:
            return
        self.open = False
        self.be._check(self.be._lib.ek_ep_peer_close(self.be._h))
        dist.barrier(group=self.group)


class ExpertParallelMoE:
    """y = shared(x) + sum_k w_k expert_k(x) with the experts sharded over `group`.

    Two exchange schemes:

    "gather"  (default up to `gather_max_tokens` global tokens, equal batch per rank): all-gather
              the tokens, every rank runs its experts on the rows routed to them, reduce-scatter the
              fp32 partial sums.  Two collectives of fixed size, no host synchronisation.
    "a2a"     rows travel only to the ranks that own their experts (two all-to-alls whose split
              sizes come from the all-gathered per-expert counts: one host synchronisation).
    "peer"    the gather scheme without collectives: this library's kernels store the tokens into
              every rank's memory and load the partial sums from every rank's memory (CUDA IPC
              mappings), synchronised by flag words; GPU only."""

    def __init__(self, stages, group: Optional[dist.ProcessGroup] = None, max_recv_rows: Optional[int] = None,
                 mode: str = "auto", gather_max_tokens: int = 2048, peer_tokens: Optional[int] = None):
        self.mode = mode
        self.peer_tokens = peer_tokens      # per-rank capacity of the peer buffers (default: the first batch)
        self.gather_max_tokens = gather_max_tokens
        self.stages = stages
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.max_recv_rows = max_recv_rows
        self._bufs = {}
        self.last_counts_all = None
        self._peer_ok = None                # auto mode: None = not tried yet
        self.last_mode = None               # scheme the last forward used
        self._owners_set = {}               # layers that currently follow an owner table

    def _buf(self, name: str, rows: int, like: torch.Tensor) -> torch.Tensor:
        b = self._bufs.get(name)
        if b is None or b.shape[0] < rows or b.device != like.device:
            b = torch.empty(max(rows, 1), like.shape[1], dtype=like.dtype, device=like.device)
            self._bufs[name] = b
        return b

    def forward(self, layer: int, x: torch.Tensor, equal_batches: bool = True,
                owners: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x: this rank's tokens [T,H].  `equal_batches`: every rank passes the same T (required by
        the "gather" scheme; with "auto" unequal batches use the all-to-all scheme).
        `owners`: int32 [n_experts], the rank that serves each expert in THIS pass -- the same table on
        every rank, naming only ranks that hold the expert (its home rank or one with a replica).  The
        reference picks one holder per request at random (controller/registry.rs:49-72); here the
        caller decides, e.g. `choose_owners`.  Only the schemes in which every rank routes the
        gathered batch ("gather", "peer") can follow a table."""
        mode = self.mode
        if mode == "auto":
            small = equal_batches and (x.shape[0] * self.world <= self.gather_max_tokens or owners is not None)
            if small and x.is_cuda and hasattr(self.stages, "peer_setup") and self._peer_ok is not False:
                mode = "peer" if self._try_peer(x.shape[0]) else "gather"
            else:
                mode = "gather" if small else "a2a"
        self.last_mode = mode
        if owners is not None or self._owners_set.get(layer):
            if mode == "a2a":
                raise ValueError("an owner table needs the gather or peer scheme")
            self.stages.set_owners(layer, owners)
            self._owners_set[layer] = owners is not None
        if mode == "gather":
            return self._forward_gather(layer, x)
        if mode == "peer":
            return self._forward_peer(layer, x)
        return self._forward_a2a(layer, x)

    def _try_peer(self, T: int) -> bool:
        """Sets the peer buffers up once; every rank learns whether ALL ranks succeeded, so the
        group takes the same scheme."""
        if self._peer_ok is None:
            ok = 1
            try:
                self._bufs["peer_ws"] = self.stages.peer_setup(self.group, max(self.peer_tokens or 0, T))
                self._peer_step = 0
            except Exception as ex:   # noqa: BLE001
                import sys
                print(f"[ek_b200] peer-memory exchange unavailable on rank {self.rank}: {ex}; using the collective scheme",
                      file=sys.stderr)
                ok = 0
            flag = torch.tensor([ok], dtype=torch.int32, device="cuda")
            dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
            self._peer_ok = bool(flag.item())
            if not self._peer_ok:
                ws = self._bufs.pop("peer_ws", None)
                if ws is not None:
                    ws.close()
        ws = self._bufs.get("peer_ws")
        return self._peer_ok and ws is not None and T <= ws.tokens_per_rank

    def close(self):
        """Releases the peer-memory workspace (collective: every rank calls it)."""
        ws = self._bufs.pop("peer_ws", None)
        if ws is not None:
            ws.close()

    def _forward_peer(self, layer: int, x: torch.Tensor) -> torch.Tensor:
        """The gather scheme with the library's own kernels over NVLink: tokens are stored into every
        rank's buffer, the partial sums are loaded from every rank by the finishing kernel.  Equal
        batches, at most the size the workspace was made for; every rank must call in lockstep."""
        T = x.shape[0]
        ws = self._bufs.get("peer_ws")
        if ws is None:
            ws = self.stages.peer_setup(self.group, self.peer_tokens or T)
            self._bufs["peer_ws"] = ws
            self._peer_step = 0
        if T > ws.tokens_per_rank:
            raise ValueError(f"{T} tokens per rank, the peer buffers were made for {ws.tokens_per_rank}")
        y = torch.empty_like(x)
        self.stages.peer_step(layer, x, y, self._peer_step)
        self._peer_step += 1
        return y

    def _forward_gather(self, layer: int, x: torch.Tensor) -> torch.Tensor:
        st = self.stages
        T, H = x.shape
        Ta = T * self.world
        x_all = self._buf("x_all", Ta, x)[:Ta]
        dist.all_gather_into_tensor(x_all.view(-1), x.reshape(-1), group=self.group)
        part = self._bufs.get("partial")
        if part is None or part.shape[0] < Ta or part.device != x.device:
            part = torch.empty(Ta, H, dtype=torch.float32, device=x.device)
            self._bufs["partial"] = part
        part = part[:Ta]
        st.partial(layer, x_all, self.rank * T, T, part)
        red = self._bufs.get("reduced")
        if red is None or red.shape[0] < T or red.device != x.device:
            red = torch.empty(T, H, dtype=torch.float32, device=x.device)
            self._bufs["reduced"] = red
        red = red[:T]
        if dist.get_backend(self.group) == "gloo":      # no reduce-scatter there
            dist.all_reduce(part, group=self.group)
            red.copy_(part[self.rank * T:(self.rank + 1) * T])
        else:
            dist.reduce_scatter_tensor(red, part, group=self.group)
        y = torch.empty_like(x)
        st.finish(layer, red, y)
        return y

    def _forward_a2a(self, layer: int, x: torch.Tensor) -> torch.Tensor:
        st = self.stages
        T, H = x.shape
        Tk = T * st.top_k
        send = self._buf("send", Tk, x)
        counts = torch.empty(st.n_experts, dtype=torch.int32, device=x.device)
        st.route(layer, x, send, counts)
        # every rank learns every rank's per-expert row counts (one small collective + one D2H)
        gathered = torch.empty(self.world * st.n_experts, dtype=torch.int32, device=x.device)
        dist.all_gather_into_tensor(gathered, counts, group=self.group)
        counts_all = gathered.view(self.world, st.n_experts).cpu()
        self.last_counts_all = counts_all
        send_splits, recv_splits, counts_src = plan_exchange(counts_all, self.rank, self.world)
        n_recv = int(sum(recv_splits))
        if self.max_recv_rows is not None and n_recv > self.max_recv_rows:
            raise RuntimeError(f"{n_recv} rows arrive at rank {self.rank}, more than the {self.max_recv_rows} planned for")
        recv = self._buf("recv", n_recv, x)
        dist.all_to_all_single(recv[:n_recv], send[:Tk], recv_splits, send_splits, group=self.group)
        out_rows = self._buf("out", n_recv, x)
        st.ffn(layer, recv[:n_recv], counts_src, x, out_rows[:n_recv])
        returned = self._buf("ret", Tk, x)
        dist.all_to_all_single(returned[:Tk], out_rows[:n_recv], send_splits, recv_splits, group=self.group)
        y = torch.empty_like(x)
        st.combine(layer, returned[:Tk], T, y)
        return y
