"""One rank of the expert-parallel tests (launched by torch.distributed.run).

  python -m torch.distributed.run --nproc-per-node N tests/ep_worker.py {cpu|gpu}

cpu: gloo, CPU tensors, the three stages served by the CPU oracle (checks the exchange plan, the
     arrival-order bookkeeping and the collectives' split sizes without a GPU);
gpu: nccl, one GPU per rank, the stages served by the CUDA backend.
Each rank owns a slice of a global batch; the result must match the single-process oracle."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "expert-kit_b200"), os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)

from oracle import configs as OC          # noqa: E402
from oracle import ek_oracle as O         # noqa: E402
from ek_b200.ep import ExpertParallelMoE, plan_exchange  # noqa: E402


class OracleStages:
    """CPU stand-in with the interface of ek_b200.ep.BackendStages; holds only this rank's experts."""

    def __init__(self, cfg, layers, rank, world, replicas=()):
        self.cfg, self.layers = cfg, layers
        self.n_experts, self.top_k, self.hidden = cfg.n_experts, cfg.top_k, cfg.hidden
        self.el = cfg.n_experts // world
        self.lo = rank * self.el
        self.rank = rank
        self.held = list(range(self.lo, self.lo + self.el)) + list(replicas)   # replicas: experts of other ranks held too
        self.owners = None
        self._use(0)

    def _use(self, layer_idx):
        """Every layer of a stack has weights of its own."""
        self.layer = self.layers[layer_idx]
        self.local = {e: self.layer["experts"][e] for e in self.held}

    def set_owners(self, layer_idx, owners):
        if owners is not None:
            for e in range(self.n_experts):
                assert int(owners[e]) != self.rank or e in self.local, f"expert {e} assigned to a rank that does not hold it"
        self.owners = owners

    def route(self, layer_idx, x, send_rows, counts):
        self._use(layer_idx)
        _, ids, w = O.route(self.cfg, x, self.layer["wg"], self.layer["bias"])
        c, off, perm = O.bucket(ids, self.n_experts)
        self.w, self.perm = w, perm
        send_rows[:perm.numel()] = x[(perm // self.top_k).long()]
        counts.copy_(c)

    def ffn(self, layer_idx, rows, counts_src, x, out_rows):
        pos = 0
        for s in range(counts_src.shape[0]):
            for le in range(self.el):
                n = int(counts_src[s, le])
                if n:
                    up, gate, down = self.local[self.lo + le].bf16()
                    out_rows[pos:pos + n] = O.expert_ffn(rows[pos:pos + n], up, gate, down)
                    pos += n
        self.shared_out = None
        if self.layer["shared"] is not None:
            self.shared_out = O.expert_ffn(x, *self.layer["shared"].bf16())

    def partial(self, layer_idx, x_all, t0, T_local, partial):
        self._use(layer_idx)
        cfg = self.cfg
        _, ids, w = O.route(cfg, x_all, self.layer["wg"], self.layer["bias"])
        partial.zero_()
        mine = (range(self.lo, self.lo + self.el) if self.owners is None
                else [e for e in range(self.n_experts) if int(self.owners[e]) == self.rank])
        for e in mine:
            tok, slot = (ids == e).nonzero(as_tuple=True)
            if tok.numel():
                out = O.expert_ffn(x_all[tok], *self.local[e].bf16()).float()
                partial.index_add_(0, tok, out * w[tok, slot].float().unsqueeze(-1))
        self.shared_out = None
        if self.layer["shared"] is not None:
            self.shared_out = O.expert_ffn(x_all[t0:t0 + T_local], *self.layer["shared"].bf16())

    def finish(self, layer_idx, reduced, y):
        r = reduced.to(torch.bfloat16)
        if self.shared_out is not None:
            r = r + self.shared_out
        y.copy_(r)

    def combine(self, layer_idx, returned, T, y):
        k = self.top_k
        outs = torch.empty(T, k, self.hidden, dtype=torch.bfloat16)
        outs.view(T * k, self.hidden)[self.perm.long()] = returned
        r = O.combine(outs, self.w, self.cfg.bf16_combine)
        if self.shared_out is not None:
            r = r + self.shared_out
        y.copy_(r)


def main():
    mode = sys.argv[1]
    scheme = sys.argv[2] if len(sys.argv) > 2 else "a2a"
    import datetime
    dist.init_process_group("gloo" if mode == "cpu" else "nccl", timeout=datetime.timedelta(seconds=90))
    rank, world = dist.get_rank(), dist.get_world_size()
    if mode == "cpu":
        cfg = O.MoEConfig(hidden=64, intermediate=32, n_experts=8, top_k=3, scoring=O.SCORE_SIGMOID, n_group=4,
                          topk_group=3, routed_scaling=2.5, n_shared=1)
        T_global = 20 + world
    else:
        cfg = OC.config(1)
        cfg.quant = "fp8"
        T_global = 48 * world + 3
    layer = OC.make_layer(cfg, 777)
    x = OC.make_inputs(cfg, T_global, 778)
    ref = O.moe_layer(cfg, x, layer["wg"], layer["bias"], layer["experts"], layer["shared"])
    timeout_case = scheme == "peer_timeout"
    if timeout_case:
        scheme = "peer"
    # replicated experts: rank 1 also holds expert 0 and rank 0 the last expert; the serving rank of
    # each changes from pass to pass
    replica_case = scheme.endswith("_replica")
    if replica_case:
        scheme = scheme[:-len("_replica")]
    # a stack of layers, each with weights of its own, the output of one feeding the next (the shape
    # of the full-model configuration: 58 such layers over the GPUs of a box)
    stack_case = scheme.endswith("_stack")
    if stack_case:
        scheme = scheme[:-len("_stack")]
    layers = [layer] + ([OC.make_layer(cfg, 777 + 100 * l) for l in (1, 2)] if stack_case else [])
    replicas = ([cfg.n_experts - 1] if rank == 0 else [0] if rank == 1 else []) if replica_case else []
    if scheme in ("gather", "peer"):        # equal batches
        T_global -= T_global % world
        x = x[:T_global]
        ref = {"y": ref["y"][:T_global]}
        bounds = [T_global * r // world for r in range(world + 1)]
    else:                         # ragged split of the global batch
        bounds = [T_global * r // world + (1 if 0 < r < world else 0) for r in range(world + 1)]
    lo, hi = bounds[rank], bounds[rank + 1]
    if mode == "cpu":
        stages = OracleStages(cfg, layers, rank, world, replicas)
        xl = x[lo:hi].contiguous()
        be = None
    else:
        import ek_b200
        import helpers as Hh
        from ek_b200.backend import expert_tensors
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
        be = ek_b200.Backend(Hh.backend_config(cfg, max_tokens=T_global, device=torch.cuda.current_device(),
                                               ep_rank=rank, ep_size=world, replica_slots=len(replicas),
                                               max_layers=len(layers)))
        el = cfg.n_experts // world
        for li, lay in enumerate(layers):
            be.register_router(li, lay["wg"], lay["bias"])
            for e in list(range(rank * el, (rank + 1) * el)) + replicas:
                w = lay["experts"][e]
                be.register_expert(be.expert_id(li, e), expert_tensors(li, e, w.up, w.gate, w.down, w.up_s, w.gate_s, w.down_s))
            w = lay["shared"]
            be.register_expert(be.shared_id(li), expert_tensors(li, None, w.up, w.gate, w.down, w.up_s, w.gate_s, w.down_s,
                                                                shared=True))
        be.set_stream(torch.cuda.current_stream().cuda_stream)
        stages = ek_b200.BackendStages(be)
        xl = x[lo:hi].contiguous().cuda()
    moe = ExpertParallelMoE(stages, mode=scheme)
    if replica_case:
        from ek_b200.ep import choose_owners
        el = cfg.n_experts // world
        holders = [[e // el] for e in range(cfg.n_experts)]
        holders[0].append(1)
        holders[cfg.n_experts - 1].append(0)
        served = set()
        for step in range(4):               # the table differs from pass to pass; the result must not
            owners = choose_owners(holders, step)
            served.add((int(owners[0]), int(owners[cfg.n_experts - 1])))
            y = moe.forward(0, xl, owners=owners)
            if be is not None:
                be.sync()
            d = (y.cpu().float() - ref["y"][lo:hi].float()).abs()
            assert (d.max() / ref["y"][lo:hi].float().abs().max()).item() <= 2e-2, f"step {step}: wrong with owners {owners.tolist()}"
        assert len(served) > 1, "the replicated experts never changed hands"
        y = moe.forward(0, xl, owners=None)  # and back to the window rule
    if stack_case:
        # Each layer is checked on the input the stack really gave it: the ranks' slices are gathered
        # and the single-process oracle evaluates that layer on them (an error of layer l cannot hide
        # behind, or be blamed on, a routing flip it causes in layer l + 1).  Twice over the stack:
        # buffers and step parities are reused across layers and passes.
        ok = True
        for rnd in range(2):
            xin = xl
            for li, lay in enumerate(layers):
                y = moe.forward(li, xin)
                if be is not None:
                    be.sync()
                x_all = torch.empty(T_global, cfg.hidden, dtype=xin.dtype, device=xin.device)
                dist.all_gather_into_tensor(x_all, xin.contiguous())
                want = O.moe_layer(cfg, x_all.cpu(), lay["wg"], lay["bias"], lay["experts"], lay["shared"])["y"][lo:hi]
                d = (y.cpu().float() - want.float()).abs()
                max_rel = (d.max() / want.float().abs().max()).item()
                # the outputs grow from layer to layer (the gain below overshoots): the mean-abs bound of
                # unit-scale outputs, 1e-3 at mean|ref| <= 0.1, grows with them
                mean_ref = want.float().abs().mean().item()
                good = max_rel <= 2e-2 and d.mean().item() <= 1e-3 * max(1.0, mean_ref / 0.1)
                ok = ok and good
                print(f"rank {rank}/{world} round {rnd} layer {li} max-rel {max_rel:.3e} mean-abs {d.mean().item():.3e} "
                      f"mean|ref| {mean_ref:.3f} {'good' if good else 'BAD'}", flush=True)
                xin = (y * 16).to(xin.dtype)          # back to unit scale; a power of two, exact in bf16
        print(f"rank {rank}/{world} stack of {len(layers)} layers {'OK' if ok else 'FAIL'}", flush=True)
        if be is not None:
            moe.close()
            be.close()
        dist.barrier()
        dist.destroy_process_group()
        sys.exit(0 if ok else 1)
    for _ in range(0 if replica_case else 3):   # several times: buffers, staging areas and step parities are reused
        y = moe.forward(0, xl)
    if be is not None:
        be.sync()
    if timeout_case:
        # Failure detection without a fault: rank 1 sits the next pass out (it leaves between passes,
        # nothing of its own in flight); rank 0's device-side waits for rank 1's step number run out and
        # the host reads EK_TIMEOUT at the next synchronisation.  The context stays usable.
        import ek_b200
        seen = None
        if rank == 0:
            moe.forward(0, xl)
            try:
                be.sync()
            except ek_b200.EKError as ex:
                seen = ex.status
            y0 = be.expert_forward(be.expert_id(0, 0), xl[:4])          # a local call still works
            usable = bool(torch.isfinite(y0.float()).all())
            ok = seen == 17 and usable
        else:
            ok = True
        dist.barrier()
        print(f"rank {rank}/{world} timeout case: status {seen} {'OK' if ok else 'FAIL'}", flush=True)
        moe.close()
        be.close()
        dist.barrier()
        dist.destroy_process_group()
        sys.exit(0 if ok else 1)
    y = y.cpu()
    if scheme == "a2a":
        # plan consistency: what I send to d equals what d expects from me
        sp, rp, cs = plan_exchange(moe.last_counts_all, rank, world)
        assert sum(sp) == (hi - lo) * cfg.top_k
        assert int(cs.sum()) == sum(rp)
    want = ref["y"][lo:hi]
    d = (y.float() - want.float()).abs()
    max_rel = (d.max() / want.float().abs().max()).item()
    ok = max_rel <= 2e-2 and d.mean().item() <= 1e-3
    print(f"rank {rank}/{world} tokens {hi - lo} max-rel {max_rel:.3e} mean-abs {d.mean().item():.3e} {'OK' if ok else 'FAIL'}",
          flush=True)
    if be is not None:
        moe.close()
        be.close()
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
