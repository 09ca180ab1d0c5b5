"""The public training entry point (``Trainer`` / YAML-style configuration) under pipeline, tensor and data parallelism
on CPU (gloo): loss curves equal the single-process run, checkpoints written under one layout resume under another
with their optimizer state, ranks agree on the resume point, and asynchronous saves are snapshots."""
import copy
import json
import os
import socket
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
WORKER = os.path.join(ROOT, "tests", "dist", "run_trainer.py")

MODEL = dict(arch=dict(type="LlamaForCausalLM"),
             model_config=dict(model_type="llama", vocab_size=128, hidden_size=64, intermediate_size=128, num_hidden_layers=4,
                               num_attention_heads=4, num_key_value_heads=2, seq_length=32, max_position_embeddings=32,
                               params_dtype="float32", compute_dtype="float32", untie_embeddings_and_output_weights=True))


def _cfg(out, *, steps=4, parallel=None, use_parallel=False, batch_size=1, accum=1, callbacks=None, **over):
    cfg = dict(output_dir=str(out), run_mode="train", use_legacy=False, seed=3, model=copy.deepcopy(MODEL),
               use_parallel=use_parallel,
               runner_config=dict(epochs=1, batch_size=batch_size, gradient_accumulation_steps=accum, stop_step=steps),
               train_dataset=dict(data_loader=dict(type="MockDataLoader", num_samples=64, seq_length=32, vocab_size=128, seed=5)),
               train_dataset_task=dict(type="CausalLanguageModelDataset"),
               optimizer=dict(type="AdamW", learning_rate=2e-3, betas=[0.9, 0.95], weight_decay=0.01),
               lr_schedule=dict(type="ConstantWarmUpLR", learning_rate=2e-3, warmup_steps=0, total_steps=-1),
               context=dict(device_target="CPU"),
               parallel_config=parallel or {},
               callbacks=callbacks or [dict(type="MFLossMonitor")])
    cfg.update(over)
    return cfg


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _launch(tmp, tag, cfg, nproc):
    cfile, out = tmp / f"{tag}.json", tmp / f"{tag}.out.json"
    cfile.write_text(json.dumps(cfg))
    if nproc == 1:
        cmd = [sys.executable, WORKER, "--config", str(cfile), "--out", str(out)]
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
               "--master-port", str(_free_port()), WORKER, "--config", str(cfile), "--out", str(out)]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=900,
                         env=dict(os.environ, OMP_NUM_THREADS="1", MASTER_ADDR="127.0.0.1"))
    assert res.returncode == 0, res.stderr[-4000:]
    return json.loads(out.read_text())["losses"]


@pytest.fixture(scope="module")
def single_losses(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("single")
    return _launch(tmp, "one", _cfg(tmp / "o", batch_size=1, accum=4), 1)


def test_pipeline_two_stages_from_the_configuration_matches_one_process(tmp_path, single_losses):
    par = dict(data_parallel=1, model_parallel=1, pipeline_stage=2, micro_batch_num=4)
    got = _launch(tmp_path, "pp2", _cfg(tmp_path / "o", parallel=par, use_parallel=True), 2)
    assert len(got) == len(single_losses) == 4
    for a, b in zip(got, single_losses):
        assert abs(a - b) < 2e-4, (got, single_losses)


def test_sequence_pipeline_from_the_configuration_matches_one_process(tmp_path, single_losses):
    """``seq_split_num: 2`` over two stages: every micro-batch flows through the pipeline as two sequence chunks, each
    stage carries the keys and values of the first chunk to the second, chunks run backward in reverse; with data
    parallel 2 next to it. The losses are those of the unsharded run."""
    par = dict(data_parallel=1, model_parallel=1, pipeline_stage=2, micro_batch_num=4, seq_split_num=2)
    got = _launch(tmp_path, "pp2seq2", _cfg(tmp_path / "o", parallel=par, use_parallel=True), 2)
    assert len(got) == len(single_losses) == 4
    for a, b in zip(got, single_losses):
        assert abs(a - b) < 2e-4, (got, single_losses)
    par = dict(data_parallel=2, model_parallel=1, pipeline_stage=2, micro_batch_num=2, seq_split_num=4)
    got = _launch(tmp_path, "pp2dp2seq4", _cfg(tmp_path / "o2", parallel=par, use_parallel=True), 4)
    for a, b in zip(got, single_losses):
        assert abs(a - b) < 2e-4, (got, single_losses)


def test_pipeline_interleaved_with_data_parallel_matches_one_process(tmp_path, single_losses):
    par = dict(data_parallel=2, model_parallel=1, pipeline_stage=2, micro_batch_num=2, pp_interleave_num=2)
    got = _launch(tmp_path, "pp2dp2", _cfg(tmp_path / "o", parallel=par, use_parallel=True), 4)
    for a, b in zip(got, single_losses):
        assert abs(a - b) < 2e-4, (got, single_losses)


def test_checkpoint_of_tp2_dp2_pp2_resumes_on_other_layouts_with_adam_state(tmp_path):
    """Eight ranks (tensor 2 x data 2 x pipeline 2, sharded optimizer) train 3 steps and save; the run is continued
    (a) by one process and (b) under tensor 2 x data 4, both through ``auto_trans_ckpt``; the next 3 losses must equal
    those of an uninterrupted single-process run of 6 steps, which they only do if the Adam moments came along."""
    ref = _launch(tmp_path, "ref", _cfg(tmp_path / "ref", steps=6, batch_size=1, accum=4), 1)
    par8 = dict(data_parallel=2, model_parallel=2, pipeline_stage=2, micro_batch_num=2, use_seq_parallel=False)
    ck = [dict(type="MFLossMonitor"), dict(type="CheckpointMonitor", save_checkpoint_steps=3, prefix="t")]
    first = _launch(tmp_path, "first", _cfg(tmp_path / "first", steps=3, parallel=par8, use_parallel=True, callbacks=ck), 8)
    for a, b in zip(first, ref[:3]):
        assert abs(a - b) < 5e-4, (first, ref)
    src = tmp_path / "first" / "checkpoint"
    assert len([d for d in os.listdir(src) if d.startswith("rank_")]) == 8
    common = dict(load_checkpoint=str(src), resume_training=True, auto_trans_ckpt=True,
                  src_strategy_path_or_dir=str(tmp_path / "first" / "strategy"))
    one = _launch(tmp_path, "one", _cfg(tmp_path / "one", steps=6, batch_size=1, accum=4, **common), 1)
    assert len(one) == 3
    for a, b in zip(one, ref[3:]):
        assert abs(a - b) < 5e-3, (one, ref)
    par_b = dict(data_parallel=4, model_parallel=2, pipeline_stage=1)
    many = _launch(tmp_path, "many", _cfg(tmp_path / "many", steps=6, parallel=par_b, use_parallel=True, **common), 8)
    for a, b in zip(many, ref[3:]):
        assert abs(a - b) < 5e-3, (many, ref)


def test_ranks_resume_from_the_newest_checkpoint_they_all_have(tmp_path):
    """Data parallel 2, saves at steps 2 and 4; rank 1's file of step 4 is lost (a crash in the middle of a save):
    both ranks must continue from step 2 and reproduce the reference losses 3..6."""
    ref = _launch(tmp_path, "ref", _cfg(tmp_path / "ref", steps=6, batch_size=1, accum=2), 1)
    par = dict(data_parallel=2, model_parallel=1, pipeline_stage=1)
    ck = [dict(type="MFLossMonitor"), dict(type="CheckpointMonitor", save_checkpoint_steps=2, prefix="t")]
    _launch(tmp_path, "a", _cfg(tmp_path / "a", steps=4, parallel=par, use_parallel=True, callbacks=ck), 2)
    src = tmp_path / "a" / "checkpoint"
    os.remove(src / "rank_1" / "t_rank_1-1_4.safetensors")
    got = _launch(tmp_path, "b", _cfg(tmp_path / "b", steps=6, parallel=par, use_parallel=True, load_checkpoint=str(src),
                                      resume_training=True), 2)
    assert len(got) == 4, got
    for a, b in zip(got, ref[2:]):
        assert abs(a - b) < 5e-3, (got, ref)
    assert open(tmp_path / "b" / "resume_record" / "latest_checkpointed_iteration.txt").read().strip() == "1_2"


def test_remove_redundancy_checkpoint_round_trip_under_tensor_parallel(tmp_path):
    """Tensor parallel 2 with ``remove_redundancy``: rank 1's file holds no replicated tensors (norm weights), and a
    strict resume still restores them, from rank 0's file of the same save."""
    from safetensors import safe_open
    ref = _launch(tmp_path, "ref", _cfg(tmp_path / "ref", steps=4, batch_size=1, accum=2), 1)
    par = dict(data_parallel=1, model_parallel=2, pipeline_stage=1)
    ck = [dict(type="MFLossMonitor"), dict(type="CheckpointMonitor", save_checkpoint_steps=2, prefix="t", remove_redundancy=True)]
    _launch(tmp_path, "a", _cfg(tmp_path / "a", steps=2, batch_size=2, parallel=par, use_parallel=True, callbacks=ck), 2)
    src = tmp_path / "a" / "checkpoint"
    with safe_open(str(src / "rank_1" / "t_rank_1-1_2.safetensors"), framework="pt") as f:
        keys1 = set(f.keys())
    with safe_open(str(src / "rank_0" / "t_rank_0-1_2.safetensors"), framework="pt") as f:
        keys0 = set(f.keys())
    assert "decoder.final_layernorm.weight" in keys0 and "decoder.final_layernorm.weight" not in keys1
    got = _launch(tmp_path, "b", _cfg(tmp_path / "b", steps=4, batch_size=2, parallel=par, use_parallel=True,
                                      load_checkpoint=str(src), resume_training=True), 2)
    for a, b in zip(got, ref[2:]):
        assert abs(a - b) < 5e-3, (got, ref)


def test_async_save_writes_the_state_of_the_moment_save_was_called(tmp_path):
    from safetensors.torch import load_file
    from mindformers_b200.core.callback import CheckpointMonitor, RunContext
    from mindformers_b200.trainer.engine import TrainingEngine
    torch.manual_seed(0)
    eng = TrainingEngine.from_model_config(dict(MODEL["model_config"], num_hidden_layers=1), device="cpu", dtype="float32")
    ids = torch.randint(0, 128, (2, 33))
    eng.train_step({"input_ids": ids[:, :-1], "labels": ids[:, 1:]})
    want = {n: p.detach().clone() for n, p in eng.model.named_parameters()}
    want_m = {k: v.clone() for k, v in eng.optimizer.named_states().items()}
    mon = CheckpointMonitor(prefix="a", directory=str(tmp_path / "ck"), async_save=True, save_checkpoint_steps=1)
    ctx = RunContext(engine=eng, config={}, epochs=1, steps_per_epoch=10, total_steps=10, global_batch_size=2, seq_length=32)
    ctx.global_step, ctx.step_in_epoch = 1, 1
    mon.save(ctx)
    # the training loop goes on while the file is being written
    with torch.no_grad():
        for p in eng.model.parameters():
            p.add_(1.0)
    eng.train_step({"input_ids": ids[:, :-1], "labels": ids[:, 1:]})
    mon._wait_async()
    sd = load_file(mon.saved[0])
    for n, t in want.items():
        assert torch.equal(sd[n], t), n
    for n, t in want_m.items():
        assert torch.equal(sd[n], t), n


def test_trainer_honours_optimizer_type_and_rejects_unbuilt_modes(tmp_path):
    from mindformers_b200.core import context
    from mindformers_b200.core.optim import ReplicatedOptimizer
    from mindformers_b200.trainer import Trainer
    context._CONTEXT = None
    cfg = _cfg(tmp_path / "c", steps=3, batch_size=2, optimizer=dict(type="CAME", learning_rate=2e-3))
    t = Trainer(args=cfg)
    t.train()
    opt = t.trainer.engine.optimizer
    assert isinstance(opt, ReplicatedOptimizer) and type(opt.inner).__name__ == "CAME"
    hist = t.trainer.loss_history
    assert len(hist) == 3 and all(x == x and x < 10 for x in hist)
    assert opt.global_step == 3 and any("exp_avg" in k for k in opt.named_states())     # CAME's factored moments exist
    context._CONTEXT = None
    bad = _cfg(tmp_path / "d", steps=1, parallel=dict(seq_split_num=2))      # the sequence pipeline needs stages
    with pytest.raises(ValueError, match="pipeline_stage > 1"):
        Trainer(args=bad).train()
    context._CONTEXT = None
    cfg = _cfg(tmp_path / "e", steps=2, batch_size=2, micro_batch_interleave_num=2)
    t = Trainer(args=cfg)
    t.train()
    assert len(t.trainer.loss_history) == 2
