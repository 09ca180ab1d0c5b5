"""Multi-process (gloo, CPU) equivalence tests: every parallel layout must reproduce the single-process
losses, global gradient norm and parameter updates of the same model, data and seed."""
import json
import os
import socket
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SCRIPT = os.path.join(ROOT, "tests", "dist", "run_parallel_equivalence.py")


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(tmp_path, nproc, tag, *extra, script=SCRIPT):
    out = tmp_path / f"{tag}.json"
    if nproc == 1:
        cmd = [sys.executable, script, "--out", str(out), *extra]
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
               "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), script, "--out", str(out), *extra]
    env = dict(os.environ, OMP_NUM_THREADS="1", MASTER_ADDR="127.0.0.1")
    for attempt in range(2):
        # a port found free can be taken before the rendezvous binds it: that one failure is retried on a new port
        if nproc > 1:
            cmd[cmd.index("--master-port") + 1] = str(_free_port())
        res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
        if res.returncode == 0 or attempt == 1 or not any(
                m in res.stderr for m in ("address already in use", "Address already in use", "EADDRINUSE")):
            break
    assert res.returncode == 0, res.stderr[-3000:]
    return json.loads(out.read_text())


def _close(a, b, tol):
    assert len(a["losses"]) == len(b["losses"])
    for x, y in zip(a["losses"], b["losses"]):
        assert abs(x - y) < tol, (a["losses"], b["losses"])
    assert abs(a["norm"] - b["norm"]) < tol * 10, (a["norm"], b["norm"])
    for k, v in a["digest"].items():
        assert abs(v - b["digest"][k]) < tol * 50, k


@pytest.fixture(scope="module")
def dense_ref(tmp_path_factory):
    return _run(tmp_path_factory.mktemp("ref"), 1, "ref")


def test_data_parallel_sharded_optimizer(tmp_path, dense_ref):
    _close(_run(tmp_path, 2, "dp2"), dense_ref, 2e-5)


def test_tensor_parallel(tmp_path, dense_ref):
    _close(_run(tmp_path, 2, "tp2", "--tp", "2"), dense_ref, 2e-5)


def test_tensor_parallel_above_kv_heads_replicates_kv(tmp_path):
    """tp = 4 with 2 KV heads (and tp = 2 with 1): every rank keeps one whole KV head; the forward pass matches tp = 1."""
    for groups, tp in ((2, 4), (1, 2)):
        ref = _run(tmp_path, 1, f"ref_g{groups}", "--forward-only", "1", "--kv-groups", str(groups))
        got = _run(tmp_path, tp, f"tp{tp}_g{groups}", "--tp", str(tp), "--forward-only", "1", "--kv-groups", str(groups))
        assert abs(ref["losses"][0] - got["losses"][0]) < 2e-5, (groups, tp, ref["losses"], got["losses"])


def test_tensor_parallel_sequence_parallel_with_dp(tmp_path, dense_ref):
    _close(_run(tmp_path, 4, "tp2sp_dp2", "--tp", "2", "--sp", "1"), dense_ref, 2e-5)


@pytest.mark.parametrize("kind", ["all_gather", "p2p", "a2a"])
def test_context_parallel(tmp_path, dense_ref, kind):
    _close(_run(tmp_path, 2, f"cp2_{kind}", "--cp", "2", "--cp-type", kind), dense_ref, 2e-5)


@pytest.mark.parametrize("name,extra", [
    ("ring4", ["--cp-type", "p2p"]),
    ("ring4_zigzag", ["--cp-type", "p2p", "--zigzag", "1"]),
    ("hybrid_u2_ring2", ["--cp-type", "a2a+p2p", "--ulysses", "2"]),
])
def test_ring_and_hybrid_context_parallel_over_four_ranks(tmp_path, dense_ref, name, extra):
    """cp = 4: the ring with contiguous chunks (K/V and their gradients travel the ring), the zig-zag balanced ring
    (half blocks per step) and Ulysses-in-pairs x ring-across-pairs all train like the unsharded model."""
    _close(_run(tmp_path, 4, name, "--cp", "4", *extra), dense_ref, 2e-5)


def test_expert_parallel(tmp_path):
    ref = _run(tmp_path, 1, "moe_ref", "--moe", "1")
    got = _run(tmp_path, 2, "moe_ep2", "--moe", "1", "--ep", "2")
    _close(got, ref, 5e-5)


PIPE = os.path.join(ROOT, "tests", "dist", "run_pipeline.py")


@pytest.fixture(scope="module")
def pipe_ref(tmp_path_factory):
    return _run(tmp_path_factory.mktemp("pref"), 1, "ref", script=PIPE)


def test_pipeline_parallel_1f1b(tmp_path, pipe_ref):
    _close(_run(tmp_path, 2, "pp2", "--pp", "2", script=PIPE), pipe_ref, 2e-5)


def test_pipeline_parallel_interleaved(tmp_path, pipe_ref):
    _close(_run(tmp_path, 2, "pp2v2", "--pp", "2", "--vpp", "2", script=PIPE), pipe_ref, 2e-5)


def test_pipeline_parallel_four_stages(tmp_path, pipe_ref):
    _close(_run(tmp_path, 4, "pp4", "--pp", "4", script=PIPE), pipe_ref, 2e-5)


def test_replicated_section_shard_and_merge_roundtrip():
    import torch
    from mindformers_b200.checkpoint.sharding import merge_shards
    from mindformers_b200.parallel.layers.tensor_parallel import section_local_sizes, shard_sections
    hd, nq, nkv, tp = 4, 8, 2, 4
    sections, groups = (nq * hd, nkv * hd, nkv * hd), (nq, nkv, nkv)
    full = torch.arange(sum(sections) * 3, dtype=torch.float32).view(sum(sections), 3)
    assert section_local_sizes(sections, tp, groups) == [8, 4, 4]
    shards = [shard_sections(full, sections, 0, r, tp, groups) for r in range(tp)]
    assert all(s.shape == (16, 3) for s in shards)
    k = full[nq * hd:nq * hd + nkv * hd]
    assert torch.equal(shards[0][8:12], k[:4]) and torch.equal(shards[1][8:12], k[:4]) and torch.equal(shards[2][8:12], k[4:])
    merged = merge_shards(shards, {"tp": tp, "dim": 0, "sections": list(sections), "groups": list(groups)})
    assert torch.equal(merged, full)


def test_dp_attention_with_ep_moe_generation_runs_in_lockstep(tmp_path):
    """Attention data-parallel (own prompts and lengths per rank), experts split over the ranks: a rank that is done
    keeps stepping until all are, and every rank's tokens equal those of the unsharded model."""
    out = tmp_path / "dpa.json"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), os.path.join(ROOT, "tests", "dist", "run_dp_attention_ep_moe.py"), str(out)]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300,
                         env=dict(os.environ, OMP_NUM_THREADS="1", MASTER_ADDR="127.0.0.1"))
    assert res.returncode == 0, res.stderr[-3000:]
    got = json.loads(out.read_text())
    assert got["ok"] and got["lens"] == [9, 9]


def test_legacy_dropless_moe_over_two_ranks_matches_one_rank():
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), os.path.join(ROOT, "tests", "dist", "run_moev3.py")]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300,
                         env=dict(os.environ, OMP_NUM_THREADS="1", MASTER_ADDR="127.0.0.1"))
    assert res.returncode == 0, res.stderr[-3000:]


def test_auto_trans_ckpt_loads_a_tp2_checkpoint_into_one_rank(tmp_path):
    """Per-rank checkpoint + strategy files of a tp = 2 run → merged and loaded by a single-rank model
    (``auto_trans_ckpt``); the loss of a fixed batch is the one the tp = 2 model had, and the resume context follows
    the scalars of the checkpoint with the step rescaled for the new global batch size."""
    import torch
    from tests.dist.run_save_tp_ckpt import CFG, batch
    from mindformers_b200.parallel.layers.gpt_model import GPTModel
    from mindformers_b200.parallel.transformer_config import TransformerConfig
    from mindformers_b200.trainer.utils import load_resume_context_from_checkpoint, transform_and_load_checkpoint
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), os.path.join(ROOT, "tests", "dist", "run_save_tp_ckpt.py"), str(tmp_path)]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300,
                         env=dict(os.environ, OMP_NUM_THREADS="1", MASTER_ADDR="127.0.0.1"))
    assert res.returncode == 0, res.stderr[-3000:]
    want = json.loads((tmp_path / "loss.json").read_text())["loss"]
    torch.manual_seed(5)                                            # other initial values than the saved model
    cfg = TransformerConfig(**CFG)
    cfg.device = "cpu"
    model = GPTModel(cfg).eval()
    inp, lab = batch()
    with torch.no_grad():
        before = float(model(inp, labels=lab))
    config = {"auto_trans_ckpt": True, "src_strategy_path_or_dir": str(tmp_path / "strategy"),
              "output_dir": str(tmp_path / "out"), "load_checkpoint": str(tmp_path / "checkpoint")}
    scalars = transform_and_load_checkpoint(config, model)
    with torch.no_grad():
        after = float(model(inp, labels=lab))
    assert abs(before - want) > 1e-3 and abs(after - want) < 1e-5
    assert os.path.exists(tmp_path / "out" / "transformed_checkpoint" / "model.safetensors")
    ctx = load_resume_context_from_checkpoint(scalars, str(tmp_path / "checkpoint"), True, global_batch_size=8,
                                              steps_per_epoch=100)
    assert ctx["initial_epoch"] == 0 and ctx["initial_step"] == 14            # 7 steps of 16 samples = 14 steps of 8


def _simulate_pipeline(pp, v, n, seq_split=1):
    """Blocking-rendezvous model of the pipeline schedule: a batch (at most one send and one receive on one ring) starts
    when its rank has computed what it sends and the rank's previous batch on that ring has finished; it finishes when
    both of its operations have met their counterparts, i.e. when the peers' matching batches have STARTED. A forward
    needs the previous activation batch finished, a backward the previous gradient batch. Returns True when every rank
    reaches the end of its schedule."""
    from mindformers_b200.parallel.pipeline import build_schedule
    sched = [build_schedule(pp, v, n, r, seq_split) for r in range(pp)]
    # batches per (rank, ring) in issue order: (step index, send k or None, recv k or None)
    rings = {}
    for r in range(pp):
        for ring, s_attr, r_attr in (("act", "send_act", "recv_act"), ("grad", "send_grad", "recv_grad")):
            rings[(r, ring)] = [(i, getattr(st, s_attr), getattr(st, r_attr)) for i, st in enumerate(sched[r])
                                if getattr(st, s_attr) is not None or getattr(st, r_attr) is not None]
    # message order between a pair must agree: the j-th send r -> peer meets the j-th receive at peer from r
    for r in range(pp):
        nxt, prv = (r + 1) % pp, (r - 1) % pp
        assert len([b for b in rings[(r, "act")] if b[1] is not None]) == \
            len([b for b in rings[(nxt, "act")] if b[2] is not None]), (pp, v, n, r, "act count")
        assert len([b for b in rings[(r, "grad")] if b[1] is not None]) == \
            len([b for b in rings[(prv, "grad")] if b[2] is not None]), (pp, v, n, r, "grad count")

    def counterpart_index(r, ring, bi, kind):
        """Index (in the peer's batch list) of the batch that holds the counterpart of the send / receive of batch bi."""
        peer = ((r + 1) if (ring == "act") == (kind == "send") else (r - 1)) % pp
        mine, theirs = rings[(r, ring)], rings[(peer, ring)]
        col, pcol = (1, 2) if kind == "send" else (2, 1)
        j = sum(1 for b in mine[:bi] if b[col] is not None)            # ordinal of this message on the pair
        seen = -1
        for pi, b in enumerate(theirs):
            if b[pcol] is not None:
                seen += 1
                if seen == j:
                    return peer, pi
        raise AssertionError("no counterpart")

    pos = [0] * pp                                     # next step to compute, per rank
    started = {key: 0 for key in rings}                # batches started per (rank, ring)
    finished = {key: 0 for key in rings}
    issued = {key: 0 for key in rings}                 # batches whose step has been computed (may start in order)
    progress = True
    while progress:
        progress = False
        for r in range(pp):
            # compute the next step if its inputs are there
            while pos[r] < len(sched[r]):
                st = sched[r][pos[r]]
                ok = True
                if st.fwd is not None:                 # all earlier activation batches finished
                    ok = ok and finished[(r, "act")] == issued[(r, "act")]
                if st.bwd is not None:
                    ok = ok and finished[(r, "grad")] == issued[(r, "grad")]
                # a step that issues a batch while one is still in flight on that ring waits for it too
                if st.send_act is not None or st.recv_act is not None:
                    ok = ok and finished[(r, "act")] == issued[(r, "act")]
                if st.send_grad is not None or st.recv_grad is not None:
                    ok = ok and (st.bwd is None or True) and finished[(r, "grad")] == issued[(r, "grad")]
                if not ok:
                    break
                if st.send_act is not None or st.recv_act is not None:
                    issued[(r, "act")] += 1
                if st.send_grad is not None or st.recv_grad is not None:
                    issued[(r, "grad")] += 1
                pos[r] += 1
                progress = True
            for ring in ("act", "grad"):
                key = (r, ring)
                if started[key] < issued[key] and started[key] == finished[key]:
                    started[key] += 1
                    progress = True
        for key, lst in rings.items():
            r, ring = key
            if started[key] > finished[key]:
                bi = finished[key]
                _, snd, rcv = lst[bi]
                ok = True
                for kind, present in (("send", snd), ("recv", rcv)):
                    if present is None:
                        continue
                    peer, pi = counterpart_index(r, ring, bi, kind)
                    ok = ok and started[(peer, ring)] > pi
                if ok:
                    finished[key] += 1
                    progress = True
    return all(pos[r] == len(sched[r]) for r in range(pp)) and all(finished[k] == len(rings[k]) for k in rings)


@pytest.mark.parametrize("pp", [2, 3, 4, 8])
@pytest.mark.parametrize("v", [1, 2, 3])
def test_pipeline_schedule_has_no_communication_cycle(pp, v):
    from mindformers_b200.parallel.pipeline import build_schedule, fwd_chunk, bwd_chunk
    for n in ([pp, 2 * pp, 4 * pp] if v > 1 else [1, 2, pp, pp + 1, 3 * pp]):
        assert _simulate_pipeline(pp, v, n), f"schedule deadlocks under blocking sends: pp={pp} v={v} n={n}"
        # every virtual micro-batch runs forward once and backward once on every rank, forward first
        for r in range(pp):
            steps = build_schedule(pp, v, n, r)
            f = [s.fwd for s in steps if s.fwd is not None]
            b = [s.bwd for s in steps if s.bwd is not None]
            assert f == list(range(n * v)) and b == list(range(n * v))
            done_f = set()
            for s in steps:
                if s.fwd is not None:
                    done_f.add((fwd_chunk(s.fwd, pp, v), s.fwd % pp + (s.fwd // (pp * v)) * pp))
                if s.bwd is not None:
                    assert (bwd_chunk(s.bwd, pp, v), s.bwd % pp + (s.bwd // (pp * v)) * pp) in done_f


def test_sequence_pipeline_schedule_orders_chunks_and_never_deadlocks():
    """``seq_split = C``: forward units (micro-batch, chunk) in order, backward with the chunks of a micro-batch reversed;
    a backward never comes before the forward of its unit, nor before the backward of a later chunk of its micro-batch;
    the rings meet without a cycle for every stage count."""
    from mindformers_b200.parallel.pipeline import build_schedule, seq_bwd_unit
    assert [seq_bwd_unit(b, 3) for b in range(6)] == [2, 1, 0, 5, 4, 3]
    for pp, n, C in [(2, 2, 2), (2, 3, 4), (3, 4, 2), (4, 4, 3), (4, 8, 2), (8, 8, 4), (2, 1, 8)]:
        assert _simulate_pipeline(pp, 1, n, C), f"sequence pipeline deadlocks: pp={pp} n={n} C={C}"
        for r in range(pp):
            steps = build_schedule(pp, 1, n, r, C)
            assert [s.fwd for s in steps if s.fwd is not None] == list(range(n * C))
            assert [s.bwd for s in steps if s.bwd is not None] == list(range(n * C))
            done_f, done_b = set(), set()
            for s in steps:
                if s.fwd is not None:
                    done_f.add(s.fwd)
                if s.bwd is not None:
                    u = seq_bwd_unit(s.bwd, C)
                    m, c = divmod(u, C)
                    assert u in done_f, (pp, n, C, r, "backward before its forward")
                    assert all(m * C + later in done_b for later in range(c + 1, C)), "a later chunk must go first"
                    done_b.add(u)
    with pytest.raises(ValueError):
        build_schedule(2, 2, 4, 0, 2)


def test_sequence_chunks_with_carried_keys_and_values_match_the_whole_sequence():
    """One stage: a micro-batch run as 4 sequence chunks (keys / values carried forward, chunks backward in reverse with
    the gradients of the carried tensors fed back) gives the loss and the gradients of the whole-sequence run."""
    import torch
    from mindformers_b200.parallel import parallel_state as ps
    from mindformers_b200.parallel.layers.gpt_model import GPTModel
    from mindformers_b200.parallel.pipeline import forward_backward_no_pipelining
    from mindformers_b200.parallel.transformer_config import TransformerConfig
    ps.initialize_model_parallel()
    torch.manual_seed(3)
    cfg = TransformerConfig(num_layers=2, hidden_size=64, num_attention_heads=4, num_query_groups=2, ffn_hidden_size=128,
                            vocab_size=128, seq_length=32, max_position_embeddings=32, params_dtype="float32",
                            compute_dtype="float32", pad_token_id=-1)
    cfg.device = "cpu"
    model = GPTModel(cfg)
    ids = torch.randint(0, 128, (3, 33))
    mbs = [{"input_ids": ids[i:i + 1, :-1].contiguous(), "labels": ids[i:i + 1, 1:].contiguous()} for i in range(3)]
    whole = forward_backward_no_pipelining(model, mbs)
    ref = {n: p.grad.clone() for n, p in model.named_parameters()}
    model.zero_grad()
    chunked = forward_backward_no_pipelining(model, mbs, seq_split=4)
    assert torch.allclose(torch.stack(whole), torch.stack(chunked), atol=1e-6)
    for n, p in model.named_parameters():
        assert torch.allclose(p.grad, ref[n], atol=2e-6), n


@pytest.mark.parametrize("mode", ["ep", "etp"])
def test_moe_dispatcher_variants_match_a_dense_loop_over_experts(mode):
    """4 gloo ranks. ``ep``: expert parallel 4 with the all-to-all, all-gather and two-level (2 ranks per node)
    dispatchers, each with and without safe tokens. ``etp``: tensor parallel 2 x expert parallel 2 with every expert's
    FFN split over the tensor-parallel pair. Output, input gradient, expert-weight and router gradients equal those
    of a dense loop over whole experts."""
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), os.path.join(ROOT, "tests", "dist", "run_moe_dispatchers.py"), "--mode", mode]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600,
                         env=dict(os.environ, OMP_NUM_THREADS="1", MASTER_ADDR="127.0.0.1"))
    assert res.returncode == 0, (res.stdout[-2000:], res.stderr[-3000:])


def test_layer_gradients_are_final_when_the_layer_hook_fires():
    """The hook that drives the bucketed data-parallel reduction fires once per layer, last layer first, and at that
    moment the layer's weight gradients already hold their value for the step (the last micro-batch included)."""
    import torch
    from mindformers_b200.trainer.engine import TrainingEngine
    cfg = dict(model_type="llama", num_hidden_layers=3, hidden_size=64, num_attention_heads=4, num_key_value_heads=2,
               intermediate_size=128, vocab_size=128, rms_norm_eps=1e-5, rope_theta=10000.0, max_position_embeddings=32)
    torch.manual_seed(0)
    eng = TrainingEngine.from_model_config(cfg, seq_length=32, device="cpu", dtype="float32", micro_batch_size=1)
    opt, block = eng.optimizer, eng.model.decoder
    ids = torch.randint(0, 128, (2, 33))
    batch = {"input_ids": ids[:, :-1].contiguous(), "labels": ids[:, 1:].contiguous()}
    seen = {}

    def record(gid):
        layer = block.layers._modules[str(gid)]
        seen[gid] = {n: p.main_grad.clone() if p.grad is None else p.main_grad + p.grad
                     for n, p in layer.named_parameters()}

    armed = []
    opt.begin_grad_overlap = lambda: (armed.append(1), setattr(block, "grads_final_hook", record))
    opt.max_grad_norm = 0.0
    final = {}
    orig = opt.reduce_and_norm

    def spy():
        block.grads_final_hook = None
        out = orig()
        for gid in block.layer_ids:
            final[gid] = {n: p.main_grad.clone() for n, p in block.layers._modules[str(gid)].named_parameters()}
        return out
    opt.reduce_and_norm = spy
    eng.train_step_device(batch)
    assert armed == [1]                                   # armed once, for the last of the two micro-batches
    assert list(seen) == [2, 1, 0]
    for gid, grads in seen.items():
        for n, g in grads.items():
            assert g.abs().sum() > 0
            torch.testing.assert_close(g, final[gid][n], rtol=0, atol=0)


def test_gradient_bucket_and_publication_plans_tile_the_flat_buffer(monkeypatch):
    """Host-side plans of the overlapped data-parallel paths, on a CPU model with the peer-memory state faked: the
    per-layer gradient ranges tile one interval of the flat buffer in layer order and hold only that layer's weight
    matrices; the publication rows (outside-the-layers below / above, then groups of layers) cover every element once;
    a model with more layers than flag rows groups its layers."""
    import torch
    from mindformers_b200.trainer.engine import TrainingEngine

    def plans(layers):
        cfg = dict(model_type="llama", num_hidden_layers=layers, hidden_size=32, num_attention_heads=4, num_key_value_heads=2,
                   intermediate_size=64, vocab_size=64, rms_norm_eps=1e-5, rope_theta=10000.0, max_position_embeddings=16)
        eng = TrainingEngine.from_model_config(cfg, seq_length=16, device="cpu", dtype="float32")
        opt = eng.optimizer
        for sh in opt.shards.values():
            sh.fused = True
        monkeypatch.setattr(torch.cuda, "Stream", lambda device=None: None)
        opt._setup_overlap("cpu")
        return opt

    opt = plans(3)
    info = opt._ov_layers["dense"]
    buf = opt.buffers["dense"]
    assert info["ids"] == [0, 1, 2] and info["group"] == 1
    for gid in info["ids"]:
        lo, hi = info["span"][gid]
        inside = [n for n, _, off, cnt in buf.entries if lo <= off < hi]
        assert inside and all(f"layers.{gid}." in n for n in inside) and all("norm" not in n for n in inside)
    assert all(info["span"][a][1] == info["span"][b][0] for a, b in zip(info["ids"], info["ids"][1:]))
    rows = opt._publish_rows("dense")
    assert [r for r, _, _ in rows] == list(range(len(rows))) and len(rows) == 2 + 3
    covered = sorted((lo, hi) for _, lo, hi in rows if hi > lo)
    assert covered[0][0] == 0 and covered[-1][1] == buf.ranges.numel
    assert all(a[1] == b[0] for a, b in zip(covered, covered[1:]))
    assert [opt._row_of_layer("dense", g) for g in info["ids"]] == [2, 3, 4]
    big = plans(130)
    info = big._ov_layers["dense"]
    assert info["group"] == 3                                   # 130 layers over 64 gradient-bucket rows
    rows = big._publish_rows("dense")
    assert len(rows) <= 62 and big._row_of_layer("dense", 129) == rows[-1][0]
    assert sorted({big._row_of_layer("dense", g) for g in info["ids"]}) == [r for r, _, _ in rows[2:]]


def test_offline_transform_between_layouts_round_trips(tmp_path):
    """``TransformCkpt`` / ``tools.transform_ckpt``: a tp = 2 checkpoint (per-rank files + strategy files) becomes (a) one
    complete checkpoint, (b) the rank file of a single-rank layout whose loss matches, and (c), transformed back with
    the tp = 2 strategy as destination, per-rank files whose tensors equal the original ones."""
    import glob
    import torch
    from safetensors.torch import load_file
    from tests.dist.run_save_tp_ckpt import CFG, batch
    from mindformers_b200.checkpoint.sharding import save_strategy
    from mindformers_b200.parallel.layers.gpt_model import GPTModel
    from mindformers_b200.parallel.transformer_config import TransformerConfig
    from mindformers_b200.tools import transform_ckpt
    from mindformers_b200.tools.resume_ckpt import get_resume_checkpoint
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), os.path.join(ROOT, "tests", "dist", "run_save_tp_ckpt.py"), str(tmp_path)]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300,
                         env=dict(os.environ, OMP_NUM_THREADS="1", MASTER_ADDR="127.0.0.1"))
    assert res.returncode == 0, res.stderr[-3000:]
    want = json.loads((tmp_path / "loss.json").read_text())["loss"]
    src, strat = str(tmp_path / "checkpoint"), str(tmp_path / "strategy")
    name = get_resume_checkpoint(src)
    assert name and name.endswith(".safetensors") and get_resume_checkpoint(src, "mine.safetensors") == "mine.safetensors"
    # (a) merge only
    merged = transform_ckpt.main(["--src_ckpt_dir", src, "--src_ckpt_strategy", strat, "--dst_ckpt_dir", str(tmp_path / "full")])
    full = load_file(os.path.join(merged, "model.safetensors"))
    # (b) single-rank destination
    torch.manual_seed(5)
    cfg = TransformerConfig(**CFG)
    cfg.device = "cpu"
    model = GPTModel(cfg).eval()
    save_strategy(model, str(tmp_path / "one" / "ckpt_strategy_rank_0.json"))
    out = transform_ckpt.main(["--src_ckpt_dir", src, "--src_ckpt_strategy", strat, "--dst_ckpt_strategy", str(tmp_path / "one"),
                               "--dst_ckpt_dir", str(tmp_path / "to_one"), "--prefix", "llama_"])
    one = load_file(os.path.join(out, "rank_0", "llama_rank_0.safetensors"))
    assert all(torch.equal(one[k], full[k]) for k in full)
    sd = {n: one[n] for n, _ in model.named_parameters()}
    model.load_state_dict(sd, strict=False)
    inp, lab = batch()
    with torch.no_grad():
        assert abs(float(model(inp, labels=lab)) - want) < 1e-5
    # (c) back to the source layout: the original shards come out again (weights and Adam moments)
    back = transform_ckpt.main(["--src_ckpt_dir", merged, "--dst_ckpt_strategy", strat, "--dst_ckpt_dir", str(tmp_path / "back")])
    for r in range(2):
        orig = load_file(sorted(glob.glob(os.path.join(src, f"rank_{r}", "*.safetensors")))[-1])
        again = load_file(os.path.join(back, f"rank_{r}", f"checkpoint_rank_{r}.safetensors"))
        params = json.load(open(os.path.join(strat, f"ckpt_strategy_rank_{r}.json")))["params"]
        for n in params:
            assert torch.equal(again[n], orig[n]), (r, n)
