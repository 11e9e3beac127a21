"""GPU tests of the worker-facing boundary: ExpertDB semantics, the wire blob of
ForwardReq/ForwardResp, weight-bundle loading by the reference's suffix rule, and the error
codes that stand in for the reference's EKError values and panics."""
import threading

import pytest
import torch
from safetensors.torch import load as st_load
from safetensors.torch import save as st_save

import helpers as Hh
from oracle import configs as OC
from oracle import ek_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture()
def small():
    import ek_b200
    cfg = O.MoEConfig(hidden=256, intermediate=128, n_experts=8, top_k=2, scoring=O.SCORE_SOFTMAX, quant="bf16")
    layer = OC.make_layer(cfg, 42)
    be = ek_b200.Backend(Hh.backend_config(cfg, max_tokens=64, max_layers=3))
    yield cfg, layer, be
    be.close()


def _tensors(layer_idx, e, w):
    from ek_b200.backend import expert_tensors
    return expert_tensors(layer_idx, e, w.up, w.gate, w.down, w.up_s, w.gate_s, w.down_s)


def test_expert_db_semantics(small):
    cfg, layer, be = small
    assert be.loaded() == 0 and be.keys() == []
    a, b = be.expert_id(2, 3), be.expert_id(2, 5)
    assert be.mark_loading(a) is True
    assert be.mark_loading(a) is False            # second claim is refused (manager.rs:60-70)
    assert be.has(a) and be.loading() == 1 and be.loaded() == 0
    be.register_expert(a, _tensors(2, 3, layer["experts"][3]))
    assert be.loading() == 0 and be.loaded() == 1
    be.register_expert(b, _tensors(2, 5, layer["experts"][5]))
    be.register_expert(be.expert_id(10, 0), _tensors(10, 0, layer["experts"][0]))
    assert be.keys() == sorted([a, b, be.expert_id(10, 0)])      # BTreeMap order
    be.evict(a)
    be.evict("model/l2-e7")                        # unknown id: not an error (manager.rs:71-74)
    assert not be.has(a) and be.loaded() == 2


def test_expert_forward_and_not_found(small):
    import ek_b200
    cfg, layer, be = small
    eid = be.expert_id(0, 4)
    x = OC.make_inputs(cfg, 19, 5)
    with pytest.raises(ek_b200.EKError) as e:
        be.expert_forward(eid, x)
    assert e.value.status_name == "EK_EXPERT_NOT_FOUND"
    be.register_expert(eid, _tensors(0, 4, layer["experts"][4]))
    y = be.expert_forward(eid, x)
    ref = O.expert_ffn(x, *layer["experts"][4].bf16())
    Hh.assert_outputs_close(y, ref, "expert_forward")
    # device-resident input and output
    yd = be.expert_forward(eid, x.cuda())
    assert yd.is_cuda
    assert torch.equal(yd.cpu(), y)
    be.evict(eid)
    with pytest.raises(ek_b200.EKError) as e:
        be.expert_forward(eid, x)
    assert e.value.status_name == "EK_EXPERT_NOT_FOUND"
    # re-registration into the freed slot with different weights is picked up
    be.register_expert(eid, _tensors(0, 4, layer["experts"][6]))
    y2 = be.expert_forward(eid, x)
    Hh.assert_outputs_close(y2, O.expert_ffn(x, *layer["experts"][6].bf16()), "after re-registration")


def test_bundle_suffix_rule_and_missing_weight(small):
    import ek_b200
    cfg, layer, be = small
    w = layer["experts"][1]
    # w1/w2/w3 naming (w1 = up, w3 = gate, w2 = down; meta.rs:58-63)
    blob = st_save({"experts.1.w1.weight": w.up, "experts.1.w2.weight": w.down, "experts.1.w3.weight": w.gate})
    be.register_bundle(be.expert_id(0, 1), blob)
    x = OC.make_inputs(cfg, 7, 1)
    Hh.assert_outputs_close(be.expert_forward(be.expert_id(0, 1), x), O.expert_ffn(x, *w.bf16()), "w1/w2/w3 bundle")
    with pytest.raises(ek_b200.EKError) as e:
        be.register_bundle(be.expert_id(0, 2), st_save({"a.up_proj.weight": w.up, "a.gate_proj.weight": w.gate}))
    assert e.value.status_name == "EK_EXPERT_WEIGHT_NOT_FOUND" and "w2/down_w" in str(e.value)
    with pytest.raises(ek_b200.EKError) as e:
        be.register_bundle(be.expert_id(0, 2), b"\x05\x00\x00\x00\x00\x00\x00\x00{bad")
    assert e.value.status_name == "EK_SAFETENSOR"
    with pytest.raises(ek_b200.EKError) as e:
        be.register_expert("model/l0-e2", {"up_proj.weight": w.up[:, :128], "gate_proj.weight": w.gate,
                                           "down_proj.weight": w.down})
    assert e.value.status_name == "EK_INVALID_INPUT"
    with pytest.raises(ek_b200.EKError) as e:
        be.register_expert("nonsense", _tensors(0, 2, w))
    assert e.value.status_name == "EK_INVALID_INPUT"


def test_wire_blob_round_trip(small):
    """The worker's handling of ForwardReq.tensor -> ForwardResp.output_tensor: a safetensors
    blob with the single key "data" each way (core.rs:52-63, grpc_client.py:53,68-72)."""
    import ek_b200
    cfg, layer, be = small
    eid = be.expert_id(1, 2)
    be.register_expert(eid, _tensors(1, 2, layer["experts"][2]))
    x = OC.make_inputs(cfg, 11, 3)
    resp = be.worker_forward_wire(eid, st_save({"data": x}))
    out = st_load(resp)["data"]
    assert out.shape == x.shape and out.dtype == torch.bfloat16
    Hh.assert_outputs_close(out, O.expert_ffn(x, *layer["experts"][2].bf16()), "wire reply")
    with pytest.raises(ek_b200.EKError) as e:
        be.worker_forward_wire(eid, st_save({"other": x}))
    assert e.value.status_name == "EK_SAFETENSOR"
    with pytest.raises(ek_b200.EKError) as e:
        be.worker_forward_wire(eid, st_save({"data": x.float()}))
    assert e.value.status_name == "EK_INVALID_INPUT"
    with pytest.raises(ek_b200.EKError) as e:
        be.worker_forward_wire(eid, st_save({"data": x.view(-1)}))       # must be 2-D (ffn/mod.rs:45)
    assert e.value.status_name == "EK_INVALID_INPUT"


def test_fused_call_reports_unregistered_expert_and_recovers(small):
    import ek_b200
    cfg, layer, be = small
    Hh.register_layer(be, 0, layer)
    x = OC.make_inputs(cfg, 32, 9)
    y_ok = be.moe_forward_fused(0, x)
    be.evict(be.expert_id(0, 0))
    # route a token to the missing expert through the controller-level call
    ids = torch.tensor([[0, 1]] * 4, dtype=torch.int32)
    with pytest.raises(ek_b200.EKError) as e:
        be.moe_forward(0, x[:4], ids)
    assert e.value.status_name == "EK_EXPERT_NOT_FOUND"
    with pytest.raises(ek_b200.EKError) as e:
        be.moe_forward(0, x[:4], torch.tensor([[99, 1]] * 4, dtype=torch.int32))
    assert e.value.status_name == "EK_BOUNDS"
    # the backend stays usable
    w = layer["experts"][0]
    be.register_expert(be.expert_id(0, 0), _tensors(0, 0, w))
    assert torch.equal(be.moe_forward_fused(0, x), y_ok)
    with pytest.raises(ek_b200.EKError):
        be.moe_forward_fused(0, OC.make_inputs(cfg, 65, 9))      # T beyond max_tokens
    with pytest.raises(ek_b200.EKError) as e:
        be.moe_forward_fused(2, x)                                 # layer without a router
    assert e.value.status_name == "EK_NOT_FOUND"


def test_concurrent_forwards_and_loads(small):
    """Many host threads, as the worker's tokio runtime has: forwards on some experts while
    others are being registered and evicted."""
    cfg, layer, be = small
    Hh.register_layer(be, 0, layer)
    x = OC.make_inputs(cfg, 16, 13)
    want = {e: O.expert_ffn(x, *layer["experts"][e].bf16()) for e in range(4)}
    errors = []

    def forwards(e):
        try:
            for _ in range(20):
                y = be.expert_forward(be.expert_id(0, e), x)
                Hh.assert_outputs_close(y, want[e], "threaded forward")
        except Exception as ex:   # noqa: BLE001
            errors.append(ex)

    def churn():
        try:
            for i in range(10):
                eid = be.expert_id(0, 4 + i % 4)
                be.evict(eid)
                be.register_expert(eid, _tensors(0, 4 + i % 4, layer["experts"][4 + i % 4]))
        except Exception as ex:   # noqa: BLE001
            errors.append(ex)

    ths = [threading.Thread(target=forwards, args=(e,)) for e in range(4)] + [threading.Thread(target=churn)]
    for t in ths:
        t.start()
    for t in ths:
        t.join()
    assert not errors, errors
    assert be.loaded() == 8


@pytest.mark.parametrize("quant", ["bf16", "fp8"])
def test_registrations_from_many_threads_at_once(quant):
    """The worker loads up to 64 experts concurrently (ek-computation/src/worker/state.rs:178-197):
    registrations from 16 threads run side by side on the loader lanes, two threads register the same
    id at once, and every expert then answers like the oracle."""
    import ek_b200
    cfg = O.MoEConfig(hidden=256, intermediate=128, n_experts=16, top_k=2, scoring=O.SCORE_SOFTMAX, quant=quant)
    layer = OC.make_layer(cfg, 77)
    be = ek_b200.Backend(Hh.backend_config(cfg, max_tokens=64))
    errors = []

    def load(e):
        try:
            for _ in range(3):     # host tensors (pageable): the path through the pinned bounce buffers
                be.register_expert(be.expert_id(0, e), _tensors(0, e, layer["experts"][e]))
        except Exception as ex:   # noqa: BLE001
            errors.append(ex)

    ths = [threading.Thread(target=load, args=(e % 16,)) for e in range(24)]   # experts 0..7 from two threads each
    for t in ths:
        t.start()
    for t in ths:
        t.join()
    assert not errors, errors
    assert be.loaded() == 16 and be.loading() == 0
    x = OC.make_inputs(cfg, 12, 3)
    for e in range(16):
        y = be.expert_forward(be.expert_id(0, e), x)
        Hh.assert_outputs_close(y, O.expert_ffn(x, *layer["experts"][e].bf16()), f"expert {e} after parallel registration")
    be.close()


def test_concurrent_worker_calls_share_grouped_launches(small):
    """Single-expert calls from many threads (one RPC per expert in the reference worker) are
    served in groups: same bits as the calls made one by one, fewer passes than calls."""
    cfg, layer, be = small
    Hh.register_layer(be, 0, layer)
    xs = {e: OC.make_inputs(cfg, 3 + 5 * e, 100 + e) for e in range(8)}   # ragged batch sizes 3..38
    alone = {e: be.expert_forward(be.expert_id(0, e), xs[e]) for e in range(8)}
    for e in range(8):
        Hh.assert_outputs_close(alone[e], O.expert_ffn(xs[e], *layer["experts"][e].bf16()), "single call")
    calls0, batches0 = be.worker_batch_stats()
    assert calls0 == batches0 == 8
    rounds, errors = 25, []
    start = threading.Barrier(8)

    def worker(e):
        try:
            for _ in range(rounds):
                start.wait()
                y = be.expert_forward(be.expert_id(0, e), xs[e])
                assert torch.equal(y, alone[e]), f"expert {e}: grouped result differs from the single call"
        except Exception as ex:   # noqa: BLE001
            errors.append(ex)
            start.abort()

    ths = [threading.Thread(target=worker, args=(e,)) for e in range(8)]
    for t in ths:
        t.start()
    for t in ths:
        t.join()
    assert not errors, errors
    calls, batches = be.worker_batch_stats()
    assert calls - calls0 == 8 * rounds
    assert batches - batches0 < 8 * rounds, "no two concurrent calls were ever served together"
    # an unknown expert in a group fails alone
    with pytest.raises(Exception):
        be.expert_forward("nope/l0-e0", xs[0])
    assert torch.equal(be.expert_forward(be.expert_id(0, 1), xs[1]), alone[1])


def test_cpp_worker_mirror_with_48_threads(tmp_path):
    """The C++ mirror of the worker (include/ek_b200.hpp) with the reference's 48 runtime threads:
    one EKInstanceGate::forward per expert; replies identical to the single-threaded ones,
    malformed requests rejected as errors, and concurrent requests share grouped launches."""
    import json
    import subprocess
    exe = Hh.build_host_shim(tmp_path)
    r = subprocess.run([exe, "1024", "512", "48", "4", "48", "5"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, (r.returncode, r.stdout, r.stderr)
    rep = json.loads(r.stdout.strip().splitlines()[-1])
    assert rep["mismatches"] == 0 and rep["errors"] == 0 and rep["rejected"] == 4
    assert rep["one_thread_passes"] == rep["one_thread_calls"] == 48 * 6   # warm-up round + 5 timed
    assert rep["threads_calls"] == 48 * 5
    assert rep["threads_passes"] < rep["threads_calls"], rep
    print(rep)


@pytest.mark.parametrize("quant", ["bf16", "fp8"])
def test_tile_blob_round_trip_and_file_cache(tmp_path, quant):
    """Device-ready blobs: export -> evict -> register the blob -> identical outputs; blobs of
    another layout version or configuration are refused; the file cache serves the second load."""
    import ek_b200
    cfg = O.MoEConfig(hidden=256, intermediate=128, n_experts=4, top_k=2, scoring=O.SCORE_SIGMOID, n_shared=1,
                      quant=quant)
    layer = OC.make_layer(cfg, 77)
    be = ek_b200.Backend(Hh.backend_config(cfg, max_tokens=32))
    try:
        Hh.register_layer(be, 0, layer)
        x = OC.make_inputs(cfg, 9, 5)
        ids = [be.expert_id(0, 1), be.shared_id(0)]
        before = {i: be.expert_forward(i, x) for i in ids}
        y_fused = be.moe_forward_fused(0, x)
        blobs = {i: be.export_tiles(i) for i in ids}
        for i in ids:
            be.evict(i)
            assert not be.has(i)
            be.register_tiles(i, blobs[i])
            assert be.has(i)
            assert torch.equal(be.expert_forward(i, x), before[i])
        assert torch.equal(be.moe_forward_fused(0, x), y_fused)
        # refused: other layout version, other configuration, truncated, not a blob
        bad = bytearray(blobs[ids[0]])
        bad[8] ^= 0xFF
        with pytest.raises(ek_b200.EKError) as e:
            be.register_tiles(ids[0], bytes(bad))
        assert e.value.status == 20
        with pytest.raises(ek_b200.EKError):
            be.register_tiles(ids[0], blobs[ids[0]][:-16])
        with pytest.raises(ek_b200.EKError):
            be.register_tiles(ids[0], b"x" * 4096)
        other = ek_b200.Backend(Hh.backend_config(O.MoEConfig(hidden=256, intermediate=256, n_experts=4, top_k=2,
                                                              quant=quant), max_tokens=32))
        try:
            with pytest.raises(ek_b200.EKError):
                other.register_tiles(ids[0], blobs[ids[0]])
        finally:
            other.close()
        assert torch.equal(be.expert_forward(ids[0], x), before[ids[0]])   # the failed loads left the slot alone
        # file cache: miss writes the blob, hit needs no bundle
        from safetensors.torch import save as st_save
        w = layer["experts"][2]
        tensors = {"w1.weight": w.up, "w2.weight": w.down, "w3.weight": w.gate}
        if quant != "bf16":
            tensors.update({"w1.weight_scale_inv": w.up_s, "w2.weight_scale_inv": w.down_s, "w3.weight_scale_inv": w.gate_s})
        bundle = st_save({k: v.contiguous() for k, v in tensors.items()})
        fetched = []

        def fetch(eid):
            fetched.append(eid)
            return bundle

        eid = be.expert_id(0, 2)
        want = be.expert_forward(eid, x)
        cache = ek_b200.TileCache(be, str(tmp_path / "tiles"))
        be.evict(eid)
        assert cache.load(eid, fetch) is False and fetched == [eid]
        assert torch.equal(be.expert_forward(eid, x), want)
        be.evict(eid)
        assert cache.load(eid, fetch) is True and fetched == [eid]
        assert torch.equal(be.expert_forward(eid, x), want)
        assert (cache.hits, cache.misses) == (1, 1)
    finally:
        be.close()


def test_layer_pass_can_be_captured_in_a_cuda_graph():
    """A decode loop may capture the device-resident call once and replay it: the pass issues no
    synchronisation, allocation or host read-back, and its programmatic launch edges survive capture."""
    import ek_b200
    cfg = O.MoEConfig(hidden=512, intermediate=256, n_experts=16, top_k=4, scoring=O.SCORE_SIGMOID, n_group=4,
                      topk_group=2, n_shared=1, routed_scaling=2.5, quant="fp8")
    layer = OC.make_layer(cfg, 5)
    be = ek_b200.Backend(Hh.backend_config(cfg, max_tokens=32))
    try:
        Hh.register_layer(be, 0, layer, device="cuda")
        s = torch.cuda.Stream()
        be.set_stream(s.cuda_stream)
        x = OC.make_inputs(cfg, 8, 1).cuda()
        y_eager, y_graph = torch.empty_like(x), torch.empty_like(x)
        with torch.cuda.stream(s):
            be.moe_forward_fused_async(0, x, y_eager)      # first call outside capture (one-time attribute set-up)
        be.sync()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=s):
            be.moe_forward_fused_async(0, x, y_graph)
        for seed in (2, 3):
            x.copy_(OC.make_inputs(cfg, 8, seed).cuda())
            graph.replay()
            with torch.cuda.stream(s):
                be.moe_forward_fused_async(0, x, y_eager)
            be.sync()
            torch.cuda.synchronize()
            assert torch.equal(y_graph, y_eager)
    finally:
        be.close()


def test_stage_times_and_launch_counter(small):
    cfg, layer, be = small
    Hh.register_layer(be, 0, layer)
    x = OC.make_inputs(cfg, 32, 2)
    before = be.kernel_launches()
    be.stage_timing(True)
    be.moe_forward_fused(0, x)
    t = be.stage_times()
    assert set(t) == {"route", "permute", "gateup", "down", "combine"}
    assert all(v > 0 for v in t.values())
    assert be.kernel_launches() - before == 7     # logits, select, permute + work list, gather, gate/up, down, combine


def test_many_layers_registered_back_to_back():
    """Layers created and filled in quick succession (device-resident weights, no host copies to
    slow the loader down): every layer's first expert must be usable right away."""
    import ek_b200
    cfg = O.MoEConfig(hidden=256, intermediate=128, n_experts=4, top_k=2, scoring=O.SCORE_SOFTMAX, quant="bf16")
    n_layers = 12
    be = ek_b200.Backend(Hh.backend_config(cfg, max_tokens=32, max_layers=n_layers))
    layers = [OC.make_layer(cfg, 500 + i) for i in range(n_layers)]
    for i, layer in enumerate(layers):
        Hh.register_layer(be, i, layer, device="cuda")
    x = OC.make_inputs(cfg, 24, 77)
    for i, layer in enumerate(layers):
        ref = O.moe_layer(cfg, x, layer["wg"], layer["bias"], layer["experts"], None)
        y = be.moe_forward_fused(i, x.cuda()).cpu()
        Hh.assert_outputs_close(y, ref["y"], f"layer {i}")
    be.close()


def test_replica_slots_and_owner_table_two_ranks_emulated_on_one_gpu():
    """Replicated experts without a second GPU: two backends (ep_rank 0 and 1 of 2) on one device,
    each holding its window plus one replica of the other's expert.  Every pass both route the whole
    batch and serve what the owner table gives them; the summed partials, finished per token slice,
    must equal the single-process oracle whichever holder serves the replicated experts."""
    import ek_b200
    from ek_b200.backend import expert_tensors
    from oracle import configs as OC
    from oracle import ek_oracle as O
    cfg = OC.config(1)
    cfg.quant = "fp8"
    layer = OC.make_layer(cfg, 515)
    T, E = 48, cfg.n_experts
    x = OC.make_inputs(cfg, T, 516)
    ref = O.moe_layer(cfg, x, layer["wg"], layer["bias"], layer["experts"], layer["shared"])
    el = E // 2
    replica = {0: E - 1, 1: 0}
    backs = []
    try:
        for rank in (0, 1):
            be = ek_b200.Backend(Hh.backend_config(cfg, max_tokens=T, ep_rank=rank, ep_size=2, replica_slots=1))
            be.register_router(0, layer["wg"], layer["bias"])
            for e in list(range(rank * el, (rank + 1) * el)) + [replica[rank]]:
                w = layer["experts"][e]
                be.register_expert(be.expert_id(0, e), expert_tensors(0, e, w.up, w.gate, w.down, w.up_s, w.gate_s, w.down_s))
            w = layer["shared"]
            be.register_expert(be.shared_id(0), expert_tensors(0, None, w.up, w.gate, w.down, w.up_s, w.gate_s, w.down_s,
                                                               shared=True))
            assert be.loaded() == el + 2
            backs.append(be)
        with pytest.raises(ek_b200.EKError) as err:     # the single replica slot is taken
            w = layer["experts"][3]
            backs[1].register_expert(backs[1].expert_id(0, 3), expert_tensors(0, 3, w.up, w.gate, w.down, w.up_s, w.gate_s, w.down_s))
        assert err.value.status_name == "EK_NO_MEMORY"
        xc = x.cuda()
        home = torch.tensor([e // el for e in range(E)], dtype=torch.int32)
        tables = [None, home.clone(), home.clone(), home.clone()]
        tables[2][0] = 1                                 # expert 0 served by its replica on rank 1
        tables[3][0], tables[3][E - 1] = 1, 0            # both replicated experts away from home
        for owners in tables:
            total = torch.zeros(T, cfg.hidden, dtype=torch.float32, device="cuda")
            for rank, be in enumerate(backs):
                be.set_owners(0, owners)
                part = torch.empty(T, cfg.hidden, dtype=torch.float32, device="cuda")
                be.ep_partial(0, xc, rank * (T // 2), T // 2, part)
                be.sync()
                total += part
            y = torch.empty(T, cfg.hidden, dtype=torch.bfloat16, device="cuda")
            for rank, be in enumerate(backs):
                sl = slice(rank * (T // 2), (rank + 1) * (T // 2))
                be.ep_finish(0, total[sl].contiguous(), y[sl])
                be.sync()
            mr, ma = Hh.output_errors(y, ref["y"])
            Hh.record(f"owner table {None if owners is None else owners.tolist()}", max_rel=mr, mean_abs=ma)
            assert mr <= Hh.MAX_REL and ma <= Hh.MEAN_ABS
        bad = home.clone()
        bad[1] = 1                                       # rank 1 holds no copy of expert 1
        with pytest.raises(ek_b200.EKError) as err:
            backs[1].set_owners(0, bad)
        assert err.value.status_name == "EK_EXPERT_NOT_FOUND"
        backs[1].evict(backs[1].expert_id(0, 0))        # the replica slot is free again
        w = layer["experts"][3]
        backs[1].register_expert(backs[1].expert_id(0, 3), expert_tensors(0, 3, w.up, w.gate, w.down, w.up_s, w.gate_s, w.down_s))
        assert backs[1].has(backs[1].expert_id(0, 3)) and not backs[1].has(backs[1].expert_id(0, 0))
    finally:
        for be in backs:
            be.close()
